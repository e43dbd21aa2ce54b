// C-ABI layer of libfa_b200.so: argument validation, TMA descriptor construction, partition sizing and
// kernel launches.  Nothing in this file allocates device memory or synchronises the stream (except
// fa_b200_device_status, which is a diagnostic read).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {
namespace {

// Device-side status word (one per device that loads the library).
__device__ int g_device_status = 0;

// Per-stream scratch inside the library.  A (device, stream) pair owns one slot: a work counter for the persistent
// prefill kernels (zeroed on the stream before each launch) and a block of split-KV tickets for the decode kernel
// (zero whenever no decode launch of that stream is in flight: the kernel puts them back).  Launches of one stream
// are ordered by the stream and so may share a slot; different streams get different slots.
constexpr int kStreamSlots = 64;
constexpr int kTicketsPerSlot = 4096;   // (sequence, kv head) pairs of one decode launch that can merge in the kernel
__device__ int g_work_counters[kStreamSlots];
__device__ int g_tickets[kStreamSlots * kTicketsPerSlot];

std::atomic<uint64_t> g_launches{0};
#ifdef FA_B200_TEST_HOOKS
std::atomic<int> g_test_withhold{0};   // the next decode / two-tile prefill launch withholds one tile load
#endif
thread_local char g_last_error[256] = "";
thread_local char g_launch_info[320] = "";

void set_error(const char* what, const char* detail) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, detail ? detail : "");
}
int cuda_fail(const char* what, cudaError_t e) {
  set_error(what, cudaGetErrorString(e));
  return FA_B200_ERR_CUDA;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return static_cast<EncodeTiledFn>(nullptr);
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

int* status_ptr() {
  static std::atomic<int*> ptrs[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int* cached = ptrs[dev].load(std::memory_order_acquire);
  if (!cached) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
    cached = static_cast<int*>(ptr);
    ptrs[dev].store(cached, std::memory_order_release);
  }
  return cached;
}

// Slot of (current device, stream); the least recently used slot is taken over when all are in use, which is safe as
// long as no more than kStreamSlots streams have launches of this library in flight at once.
int stream_slot(int dev, cudaStream_t stream) {
  struct Entry { int dev; cudaStream_t stream; uint64_t stamp; };
  static std::mutex mu;
  static Entry entries[kStreamSlots];
  static int used = 0;
  static uint64_t clock = 0;
  std::lock_guard<std::mutex> lock(mu);
  ++clock;
  int lru = 0;
  for (int i = 0; i < used; ++i) {
    if (entries[i].dev == dev && entries[i].stream == stream) { entries[i].stamp = clock; return i; }
    if (entries[i].stamp < entries[lru].stamp) lru = i;
  }
  const int slot = used < kStreamSlots ? used++ : lru;
  entries[slot] = Entry{dev, stream, clock};
  return slot;
}

// Device addresses of the per-stream scratch arrays on the current device, looked up once per device.
struct SlotBases { std::atomic<int*> counters{nullptr}; std::atomic<int*> tickets{nullptr}; };
SlotBases* slot_bases(int* dev_out) {
  static SlotBases bases[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  SlotBases& b = bases[dev];
  if (!b.counters.load(std::memory_order_acquire)) {
    void *c = nullptr, *t = nullptr;
    if (cudaGetSymbolAddress(&c, g_work_counters) != cudaSuccess) return nullptr;
    if (cudaGetSymbolAddress(&t, g_tickets) != cudaSuccess) return nullptr;
    b.tickets.store(static_cast<int*>(t), std::memory_order_release);
    b.counters.store(static_cast<int*>(c), std::memory_order_release);
  }
  *dev_out = dev;
  return &b;
}

int* next_work_counter(cudaStream_t stream) {
  int dev = 0;
  SlotBases* b = slot_bases(&dev);
  if (!b) return nullptr;
  int* c = b->counters.load(std::memory_order_acquire) + stream_slot(dev, stream);
  if (cudaMemsetAsync(c, 0, sizeof(int), stream) != cudaSuccess) return nullptr;
  return c;
}

// Tickets for `count` (sequence, kv head) pairs of a decode launch on `stream`, or nullptr when the launch has to use
// the separate combine kernel: too many pairs, or the stream is being captured into a graph (a replay could overlap
// launches of the stream that owns the slot).
int* stream_tickets(cudaStream_t stream, int64_t count) {
  if (count > kTicketsPerSlot) return nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
  int dev = 0;
  SlotBases* b = slot_bases(&dev);
  if (!b) return nullptr;
  return b->tickets.load(std::memory_order_acquire) + static_cast<size_t>(stream_slot(dev, stream)) * kTicketsPerSlot;
}

int elem_size(int dtype) { return dtype == FA_B200_E4M3 ? 1 : 2; }

// 4-D tile descriptor over (d, heads, rows, batch) with a 128-byte-swizzled box of (128 bytes, 1, box_rows, 1).
// Strides are in elements.  Out-of-range rows read as zero.
int make_tmap(CUtensorMap* out, const void* base, int dtype, int64_t heads, int64_t rows, int64_t batch,
              int64_t head_stride, int64_t row_stride, int64_t batch_stride, int box_rows, int d = kHeadDim) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { set_error("cuTensorMapEncodeTiled", "driver entry point not found"); return FA_B200_ERR_CUDA; }
  const int es = elem_size(dtype);
  static const uint8_t dummy[64] __attribute__((aligned(64))) = {};
  void* addr = const_cast<void*>(base ? base : static_cast<const void*>(dummy));
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads > 0 ? heads : 1),
                        static_cast<cuuint64_t>(rows > 0 ? rows : 1), static_cast<cuuint64_t>(batch > 0 ? batch : 1)};
  auto fix = [&](int64_t s) { return static_cast<cuuint64_t>((s > 0 ? s : d) * es); };
  cuuint64_t strides[3] = {fix(head_stride), fix(row_stride), fix(batch_stride)};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / es), 1u, static_cast<cuuint32_t>(box_rows), 1u};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == FA_B200_E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype == FA_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 4, addr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_error("cuTensorMapEncodeTiled", buf);
    return FA_B200_ERR_CUDA;
  }
  return FA_B200_OK;
}

// 4-D tile descriptor over a transposed V pool (tokens of a page, d, heads, blocks): tokens contiguous, a
// 128-byte-swizzled box of (64 tokens, 128 d rows, 1, 1) of a 16-bit type.  Strides in elements.
int make_tmap_vt(CUtensorMap* out, const void* base, int dtype, int64_t page, int64_t heads, int64_t blocks,
                 int64_t d_stride, int64_t head_stride, int64_t block_stride) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { set_error("cuTensorMapEncodeTiled", "driver entry point not found"); return FA_B200_ERR_CUDA; }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(page), static_cast<cuuint64_t>(kHeadDim),
                        static_cast<cuuint64_t>(heads > 0 ? heads : 1), static_cast<cuuint64_t>(blocks > 0 ? blocks : 1)};
  auto fix = [&](int64_t s) { return static_cast<cuuint64_t>((s > 0 ? s : page) * 2); };
  cuuint64_t strides[3] = {fix(d_stride), fix(head_stride), fix(block_stride)};
  cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(kHeadDim), 1u, 1u};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dtype == FA_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_error("cuTensorMapEncodeTiled", buf);
    return FA_B200_ERR_CUDA;
  }
  return FA_B200_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
bool stride_ok(int64_t s, int es) { return s >= 0 && (s * es) % 16 == 0; }

// Environment switches, read once when the library is loaded (as the reference reads its own,
// csrc/flash_attn_cutlass/src/flash.h:20-25):
//   FA_B200_DECODE_PARTITION=<tokens>        partition size of the split-KV decode (0 / unset: heuristic)
//   FA_B200_PREFILL_KERNEL=single|pair|dense prefill kernel, where that kernel can take the call
//   FA_B200_DECODE_MERGE=combine|kernel      split decode calls merge their partitions with the separate combine launch /
//                                            in the decode kernel (unset: by grid size, see fa_b200_decode_paged)
//   FA_B200_DEPENDENT_LAUNCH=0               the decode, combine and exchange kernels are launched without programmatic stream
//                                            serialisation
//   FA_B200_PRINT_PARAM=1                    one line on stderr per attention call: kernel, grid, tiling
//                                            (the reference: FLASH_ATTENTION_PRINT_PARAM, flash_api.cpp:219-222;
//                                            PA_PRINT_PARAM, src/paged_attention.cu:40)
// Callers that want to switch per call use the struct fields partition_tokens / kernel_choice instead.
struct EnvConfig {
  int decode_partition = 0;
  int prefill_kernel = 0;   // 0 auto, 1 single, 2 pair, 3 dense
  int print_param = 0;
  int dependent_launch = 1;   // decode launches may start during the tail of the kernel before them
  int decode_merge = 0;   // 0 auto, 1 always the separate combine launch, 2 in the decode kernel wherever it can
  EnvConfig() {
    if (const char* v = getenv("FA_B200_DEPENDENT_LAUNCH")) dependent_launch = atoi(v) != 0;
    if (const char* v = getenv("FA_B200_DECODE_MERGE")) decode_merge = !strcmp(v, "combine") ? 1 : (!strcmp(v, "kernel") ? 2 : 0);
    if (const char* v = getenv("FA_B200_DECODE_PARTITION")) decode_partition = atoi(v);
    if (const char* v = getenv("FA_B200_PREFILL_KERNEL")) {
      if (!strcmp(v, "single")) prefill_kernel = 1;
      else if (!strcmp(v, "pair")) prefill_kernel = 2;
      else if (!strcmp(v, "dense")) prefill_kernel = 3;
    }
    if (const char* v = getenv("FA_B200_PRINT_PARAM")) print_param = atoi(v);
  }
};
const EnvConfig g_env;
std::atomic<int> g_print_param{-1};   // -1: follow the environment; 0 / 1: set by fa_b200_set_print_param
bool print_param() {
  const int v = g_print_param.load(std::memory_order_relaxed);
  return v < 0 ? g_env.print_param != 0 : v != 0;
}

// 128 everywhere; 64, 192 and 256 for 16-bit tensors in the plain layouts (`only128`: the call uses a variant that is
// built for 128 alone).
bool head_dim_ok(int d, bool only128) { return d == kHeadDim || (!only128 && (d == 64 || d == 192 || d == 256)); }

struct DecodePlan {
  int status;
  int group, tile, box_tok, partition_tokens, num_partitions, max_len;
  bool split;
};

DecodePlan plan_decode(const fa_b200_decode_params* p) {
  DecodePlan pl{};
  pl.status = FA_B200_OK;
  if (!p) { pl.status = FA_B200_ERR_NULL; return pl; }
  if (p->struct_size != sizeof(fa_b200_decode_params)) { pl.status = FA_B200_ERR_ABI; return pl; }
  if (!head_dim_ok(p->d, p->dtype == FA_B200_E4M3 || p->kv_e4m3 || p->v_transposed)) { pl.status = FA_B200_ERR_HEADDIM; return pl; }
  if (p->dtype != FA_B200_F16 && p->dtype != FA_B200_BF16 && p->dtype != FA_B200_E4M3) { pl.status = FA_B200_ERR_DTYPE; return pl; }
  if (p->b < 0 || p->h <= 0 || p->h_k <= 0 || p->max_blocks_per_seq < 0 || p->num_blocks < 0) { pl.status = FA_B200_ERR_SHAPE; return pl; }
  if (p->h % p->h_k != 0 || p->h / p->h_k > 16) { pl.status = FA_B200_ERR_HEADS; return pl; }
  pl.group = p->h / p->h_k;
  if (p->seqlen_q < 0 || (p->seqlen_q > 1 && p->seqlen_q * pl.group > 16)) { pl.status = FA_B200_ERR_HEADS; return pl; }
  if (p->kv_e4m3 && p->dtype == FA_B200_E4M3) { pl.status = FA_B200_ERR_DTYPE; return pl; }   // the flag is for 16-bit queries
  pl.tile = (p->dtype == FA_B200_E4M3 || p->kv_e4m3) ? 128 : 64;
  const int page = p->page_size;
  if (page >= 64) {
    if (page % 64 != 0) { pl.status = FA_B200_ERR_PAGE; return pl; }
    pl.box_tok = 64;
  } else {
    if (page != 16 && page != 32) { pl.status = FA_B200_ERR_PAGE; return pl; }
    pl.box_tok = page;
  }
  int64_t max_len = static_cast<int64_t>(p->max_blocks_per_seq) * page;
  if (p->max_seqlen_k > 0 && p->max_seqlen_k < max_len) max_len = p->max_seqlen_k;
  if (max_len > (1ll << 30)) { pl.status = FA_B200_ERR_TOO_LARGE; return pl; }
  pl.max_len = static_cast<int>(max_len);
  const int unit = pl.tile > page ? (pl.tile % page == 0 ? pl.tile : pl.tile * page) : (page % pl.tile == 0 ? page : pl.tile * page);
  int part = p->partition_tokens > 0 ? p->partition_tokens : g_env.decode_partition;
  if (part > 0) {
    if (part % pl.tile != 0 || (part % page != 0 && page % part != 0)) { pl.status = FA_B200_ERR_SHAPE; return pl; }
  } else {
    // Largest power-of-two partition (>= 8 tiles, so the pipeline fill is amortised) that still yields enough CTAs:
    // about four rounds of the 296 resident CTA slots (148 SMs x 2) for a batch, whose lengths may be ragged, and
    // about one round for a single sequence, whose partitions are all equal.  Measured on B200: per-CTA start-up
    // and drain cost more than a slightly ragged tail, so bigger partitions win until the grid gets this small.
    const int min_part = 8 * pl.tile;
    const int64_t rows = static_cast<int64_t>(p->b) * p->h_k;
    const int64_t enough = (p->b == 1) ? 237 : 1100;
    part = min_part;
    while (part < max_len) part *= 2;
    while (part > min_part && rows * ((max_len + part - 1) / part) < enough) part /= 2;
    // A small batch (a shard of a batch on one of several GPUs) would get short partitions from that rule, and every CTA
    // spends about 4 us on its way to the first tile (lengths, page ids and the first load are three dependent trips to
    // memory).  Partitions of 4096 tokens in one ragged round measured faster than 1024 tokens in three and a half
    // (8 sequences of 1k..32k tokens: 87 us against 98 us), so short partitions grow back to 4096 tokens as long as that
    // still leaves half a round of CTAs.
    if (p->b > 1 && part < 4096) {
      int grown = part;
      while (grown < 4096 && rows * ((max_len + 2 * grown - 1) / (2 * grown)) >= 148) grown *= 2;
      part = grown;
    }
    // e4m3 caches: a CTA streams at a fixed rate (its consumer warps are latency-bound, profile of the e4m3 decode), so
    // the launch takes (rounds of the 296 CTA slots) x (a CTA's tokens) and splitting a launch that would fit ONE round
    // into two rounds of half-sized CTAs only adds start-up and merge: 32 sequences x 8192 tokens measured 0.110 ms
    // unsplit (256 CTAs) against 0.127 ms in two partitions.  Halve the partition count while everything then fits one
    // round that is still at least three quarters full.
    if (pl.tile == 128 && p->b > 1) {
      while (part < max_len) {
        const int64_t ctas_half = rows * ((max_len + 2 * static_cast<int64_t>(part) - 1) / (2 * static_cast<int64_t>(part)));
        if (ctas_half > 296 || ctas_half * 4 < 296 * 3) break;
        part *= 2;
      }
    }
    while (static_cast<int64_t>(part) * 256 < max_len) part *= 2;   // at most 256 partitions per sequence
    if (part < unit) part = unit;
  }
  // keep the per-partition page list within the kernel's shared-memory table
  while (part / page > decode_max_pages_per_partition()) part /= 2;
  if (part <= 0 || part % pl.tile != 0) { pl.status = FA_B200_ERR_PAGE; return pl; }
  pl.partition_tokens = part;
  pl.num_partitions = max_len > 0 ? static_cast<int>((max_len + part - 1) / part) : 1;
  pl.split = pl.num_partitions > 1 || p->o_partial_out != nullptr;
  return pl;
}

size_t decode_ws_bytes(const fa_b200_decode_params* p, const DecodePlan& pl) {
  if (!pl.split) return 0;
  const size_t sq = p->seqlen_q > 1 ? p->seqlen_q : 1;
  return static_cast<size_t>(pl.num_partitions) * p->b * p->h * sq * (p->d + 1) * sizeof(float);
}

}  // namespace
}  // namespace fa

using namespace fa;

extern "C" {

#ifdef FA_B200_TEST_HOOKS
// Test library only (not declared in the public header): the next decode or two-tile prefill launch of this process
// announces one tile load and never issues it, so that a bounded device-side wait runs out.
__attribute__((visibility("default"))) void fa_b200_test_withhold_load(int on) { g_test_withhold.store(on ? 1 : 0); }
#endif

int fa_b200_abi_version(void) { return FA_B200_ABI_VERSION; }
void fa_b200_set_print_param(int on) { g_print_param.store(on < 0 ? -1 : (on ? 1 : 0)); }
const char* fa_b200_last_launch_info(void) { return g_launch_info; }
uint64_t fa_b200_launch_count(void) { return g_launches.load(); }
const char* fa_b200_last_cuda_error(void) { return g_last_error; }

const char* fa_b200_status_string(int s) {
  switch (s) {
    case FA_B200_OK: return "ok";
    case FA_B200_ERR_NULL: return "a required pointer is null";
    case FA_B200_ERR_DTYPE: return "unsupported element type";
    case FA_B200_ERR_HEADDIM: return "head dimension must be 128 (or 64, 192, 256 with fp16 / bf16 tensors in the plain layouts)";
    case FA_B200_ERR_HEADS: return "Number of heads in key/value must divide number of heads in query (group <= 16 for decode)";
    case FA_B200_ERR_STRIDE: return "Input tensor must have contiguous last dimension and 16-byte aligned strides";
    case FA_B200_ERR_SHAPE: return "inconsistent or negative sizes";
    case FA_B200_ERR_PAGE: return "Paged KV cache block size must be 16, 32 or a multiple of 64";
    case FA_B200_ERR_WORKSPACE: return "workspace missing or too small";
    case FA_B200_ERR_UNSUPPORTED: return "option not supported on this path";
    case FA_B200_ERR_CUDA: return "CUDA call failed";
    case FA_B200_ERR_ALIGN: return "pointer must be 16-byte aligned";
    case FA_B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case FA_B200_ERR_TOO_LARGE: return "size beyond a built-in limit";
    case FA_B200_ERR_DEVICE_RANGE: return "a kernel skipped an out-of-range cache position, page id or rotary row";
    case FA_B200_ERR_DEVICE_UNSUPPORTED: return "a kernel met device-resident input it does not take (vertical sparsity)";
    case FA_B200_ERR_ABI: return "struct_size does not match this library: caller and library were built from different headers";
  }
  return "unknown status";
}

int fa_b200_device_status(void) {
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return FA_B200_ERR_CUDA;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return FA_B200_ERR_CUDA;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    return (v & 0xffff) ? FA_B200_ERR_DEVICE_TIMEOUT : ((v & 0x10000) ? FA_B200_ERR_DEVICE_RANGE : FA_B200_ERR_DEVICE_UNSUPPORTED);
  }
  return FA_B200_OK;
}

size_t fa_b200_decode_workspace_bytes(const fa_b200_decode_params* p) {
  DecodePlan pl = plan_decode(p);
  if (pl.status != FA_B200_OK) return 0;
  return decode_ws_bytes(p, pl);
}

int32_t fa_b200_decode_partition_tokens(const fa_b200_decode_params* p) {
  DecodePlan pl = plan_decode(p);
  return pl.status == FA_B200_OK ? pl.partition_tokens : 0;
}

int fa_b200_kv_append(const fa_b200_kv_append_params* p, void* stream) {
  if (!p) return FA_B200_ERR_NULL;
  if (p->struct_size != sizeof(fa_b200_kv_append_params)) return FA_B200_ERR_ABI;
  if (p->d != kHeadDim) return FA_B200_ERR_HEADDIM;
  if (p->dtype != FA_B200_F16 && p->dtype != FA_B200_BF16 && p->dtype != FA_B200_E4M3) return FA_B200_ERR_DTYPE;
  if (p->b < 0 || p->seqlen_new < 0 || p->seqlen_q < 0 || p->h <= 0 || p->h_k <= 0 || p->page_size <= 0 ||
      p->num_blocks < 0 || p->max_blocks_per_seq < 0)
    return FA_B200_ERR_SHAPE;
  if (p->h % p->h_k != 0) return FA_B200_ERR_HEADS;
  const int rd = p->rotary_dim;
  if (rd < 0 || rd > kHeadDim || rd % 16 != 0) return FA_B200_ERR_SHAPE;
  if (rd > 0 && p->dtype == FA_B200_E4M3) return FA_B200_ERR_UNSUPPORTED;
  if (p->b == 0 || (p->seqlen_new == 0 && (rd == 0 || p->seqlen_q == 0) && !p->seqlens_out)) return FA_B200_OK;
  if (!p->seqlens_k) return FA_B200_ERR_NULL;
  if (p->seqlens_out == p->seqlens_k) return FA_B200_ERR_UNSUPPORTED;
  const int es = elem_size(p->dtype);
  // each lane moves four elements at once: 8-byte (4-byte for e4m3) alignment of every row start
  auto ok_ptr = [&](const void* q) { return (reinterpret_cast<uintptr_t>(q) % (4 * es)) == 0; };
  auto ok_str = [&](int64_t s) { return s >= 0 && s % 4 == 0; };
  if (p->seqlen_new > 0) {
    if (!p->k_new || !p->v_new || !p->k_cache || !p->v_cache || !p->block_table) return FA_B200_ERR_NULL;
    if (!ok_ptr(p->k_new) || !ok_ptr(p->v_new) || !ok_ptr(p->k_cache) || !ok_ptr(p->v_cache)) return FA_B200_ERR_ALIGN;
    if (!ok_str(p->k_new_batch_stride) || !ok_str(p->k_new_row_stride) || !ok_str(p->k_new_head_stride) ||
        !ok_str(p->v_new_batch_stride) || !ok_str(p->v_new_row_stride) || !ok_str(p->v_new_head_stride) ||
        !ok_str(p->k_block_stride) || !ok_str(p->k_row_stride) || !ok_str(p->k_head_stride) ||
        !ok_str(p->v_block_stride) || !ok_str(p->v_row_stride) || !ok_str(p->v_head_stride))
      return FA_B200_ERR_STRIDE;
  }
  if (rd > 0) {
    if (!p->rotary_cos || !p->rotary_sin || p->seqlen_ro <= 0) return FA_B200_ERR_NULL;
    if (!ok_ptr(p->rotary_cos) || !ok_ptr(p->rotary_sin)) return FA_B200_ERR_ALIGN;
    if (p->seqlen_q > 0) {
      if (!p->q || !p->q_out) return FA_B200_ERR_NULL;
      if (!ok_ptr(p->q) || !ok_ptr(p->q_out)) return FA_B200_ERR_ALIGN;
      if (!ok_str(p->q_batch_stride) || !ok_str(p->q_row_stride) || !ok_str(p->q_head_stride) ||
          !ok_str(p->q_out_batch_stride) || !ok_str(p->q_out_row_stride) || !ok_str(p->q_out_head_stride))
        return FA_B200_ERR_STRIDE;
    }
  }
  KvAppendKernelParams k{};
  k.status = status_ptr();
  if (!k.status) return cuda_fail("fa_b200_kv_append", cudaGetLastError());
  k.k_new = p->k_new; k.v_new = p->v_new; k.q = p->q; k.q_out = p->q_out;
  k.k_cache = p->k_cache; k.v_cache = p->v_cache;
  k.block_table = p->block_table; k.seqlens_k = p->seqlens_k; k.seqlens_out = p->seqlens_out;
  k.cos = p->rotary_cos; k.sin = p->rotary_sin;
  k.kn_b = p->k_new_batch_stride; k.kn_r = p->k_new_row_stride; k.kn_h = p->k_new_head_stride;
  k.vn_b = p->v_new_batch_stride; k.vn_r = p->v_new_row_stride; k.vn_h = p->v_new_head_stride;
  k.q_b = p->q_batch_stride; k.q_r = p->q_row_stride; k.q_h = p->q_head_stride;
  k.qo_b = p->q_out_batch_stride; k.qo_r = p->q_out_row_stride; k.qo_h = p->q_out_head_stride;
  k.kc_blk = p->k_block_stride; k.kc_row = p->k_row_stride; k.kc_h = p->k_head_stride;
  k.vc_blk = p->v_block_stride; k.vc_row = p->v_row_stride; k.vc_h = p->v_head_stride;
  k.bt_stride = p->block_table_batch_stride;
  k.b = p->b; k.seqlen_q = p->seqlen_q; k.seqlen_new = p->seqlen_new; k.h = p->h; k.h_k = p->h_k;
  k.page_size = p->page_size; k.num_blocks = p->num_blocks; k.max_blocks_per_seq = p->max_blocks_per_seq;
  k.rotary_dim = rd; k.seqlen_ro = p->seqlen_ro; k.interleaved = p->is_rotary_interleaved ? 1 : 0;
  k.q_per_token = p->rotate_q_per_token ? 1 : 0;
  cudaError_t e = launch_kv_append(p->dtype, k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("fa_b200_kv_append", e);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FA_B200_OK;
}

int fa_b200_read_stream(const void* src, int64_t bytes, uint32_t* sink, void* stream) {
  if (!src || !sink) return FA_B200_ERR_NULL;
  if (bytes < 0) return FA_B200_ERR_SHAPE;
  if (!aligned16(src)) return FA_B200_ERR_ALIGN;
  cudaError_t e = launch_read_stream(src, bytes, sink, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FA_B200_OK : cuda_fail("fa_b200_read_stream", e);
}

int fa_b200_unpad_plan(const void* mask, int32_t elem, int32_t b, int32_t s, int64_t row_stride, int32_t* seqlens,
                       int32_t* cu_seqlens, int64_t* indices, int32_t* stats, void* stream) {
  if (elem != 1 && elem != 4 && elem != 8) return FA_B200_ERR_DTYPE;
  if (b < 0 || s < 0 || row_stride < 0) return FA_B200_ERR_SHAPE;
  if (!cu_seqlens || !stats || (b > 0 && (!mask || !seqlens || (s > 0 && !indices)))) return FA_B200_ERR_NULL;
  if (b == 0) {
    cudaError_t e = cudaMemsetAsync(cu_seqlens, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(stats, 0, 2 * sizeof(int32_t), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_B200_OK : cuda_fail("fa_b200_unpad_plan", e);
  }
  cudaError_t e = launch_unpad_plan(mask, elem, b, s, row_stride, seqlens, cu_seqlens, indices, stats,
                                    static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("fa_b200_unpad_plan", e);
  g_launches += 3;
  return FA_B200_OK;
}

static int move_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                     int64_t limit_rows, bool scatter, void* stream) {
  if (n_rows < 0 || row_bytes < 0 || limit_rows < 0) return FA_B200_ERR_SHAPE;
  if (n_rows == 0 || row_bytes == 0) return FA_B200_OK;
  if (!src || !dst || !indices) return FA_B200_ERR_NULL;
  cudaError_t e = launch_move_rows(src, indices, dst, n_rows, row_bytes, limit_rows, scatter, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(scatter ? "fa_b200_scatter_rows" : "fa_b200_gather_rows", e);
  g_launches++;
  return FA_B200_OK;
}
int fa_b200_gather_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                        int64_t limit_rows, void* stream) {
  return move_rows(src, indices, dst, n_rows, row_bytes, limit_rows, false, stream);
}
int fa_b200_scatter_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                         int64_t limit_rows, void* stream) {
  return move_rows(src, indices, dst, n_rows, row_bytes, limit_rows, true, stream);
}

int fa_b200_block_map_to_offset(const uint8_t* block_map, int32_t* block_offset, int32_t* block_count, int64_t rows, int32_t k,
                                int32_t scale, int32_t fill, void* stream) {
  if (rows < 0 || k < 0) return FA_B200_ERR_SHAPE;
  if (rows == 0) return FA_B200_OK;
  if (!block_count || (k > 0 && (!block_map || !block_offset))) return FA_B200_ERR_NULL;
  cudaError_t e = launch_block_map(block_map, block_offset, block_count, rows, k, scale, fill, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("fa_b200_block_map_to_offset", e);
  g_launches++;
  return FA_B200_OK;
}

namespace {
bool sink_dtype_ok(const void* s_aux, int dtype) {
  return !s_aux || dtype == FA_B200_F16 || dtype == FA_B200_BF16 || dtype == FA_B200_F32;
}
}  // namespace

int fa_b200_combine(const fa_b200_combine_params* p, void* stream) {
  if (!p) return FA_B200_ERR_NULL;
  if (p->struct_size != sizeof(fa_b200_combine_params)) return FA_B200_ERR_ABI;
  if (!p->o_partial || !p->lse_partial) return FA_B200_ERR_NULL;
  if (!sink_dtype_ok(p->s_aux, p->s_aux_dtype)) return FA_B200_ERR_DTYPE;
  if (!head_dim_ok(p->d, false)) return FA_B200_ERR_HEADDIM;
  if (p->rows < 0 || p->num_parts < 0 || p->h <= 0 || p->rows % p->h != 0) return FA_B200_ERR_SHAPE;
  if (p->out_dtype != FA_B200_F16 && p->out_dtype != FA_B200_BF16 && p->out_dtype >= 0) return FA_B200_ERR_DTYPE;
  if (!aligned16(p->o_partial) || (p->out && !aligned16(p->out))) return FA_B200_ERR_ALIGN;
  if (p->out && p->out_row_stride % 8 != 0) return FA_B200_ERR_STRIDE;
  CombineKernelParams k{};
  k.dependent_launch = g_env.dependent_launch;
  k.o_partial = p->o_partial;
  k.lse_partial = p->lse_partial;
  k.out = p->out;
  k.lse = p->lse;
  k.seqlens = nullptr;
  k.parts_per_row = p->parts_per_row;
  k.out_row_stride = p->out_row_stride;
  k.out_batch_stride = p->out_row_stride * p->h;
  k.out_tok_stride = 0;
  k.sq = 1;
  k.num_parts = p->num_parts;
  k.rows = p->rows;
  k.h = p->h;
  k.partition_tokens = 1;
  k.out_dtype = p->out_dtype;
  k.lse_empty_is_neg = 0;
  k.out_scale = p->out_scale;
  k.s_aux = p->s_aux;
  k.s_aux_dtype = p->s_aux_dtype;
  k.d = p->d;
  k.o_part_stride = p->o_part_stride > 0 ? p->o_part_stride : static_cast<int64_t>(p->rows) * p->d;
  k.lse_part_stride = p->lse_part_stride > 0 ? p->lse_part_stride : p->rows;
  if (k.o_part_stride % 4 != 0) return FA_B200_ERR_STRIDE;
  cudaError_t e = launch_combine(k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("combine launch", e);
  if (p->rows > 0) g_launches++;
  return FA_B200_OK;
}

size_t fa_b200_exchange_bytes(int32_t world, int32_t rows, int32_t d) {
  if (world <= 0 || rows <= 0 || d <= 0) return 0;
  return 2 * exchange_region_bytes(world, rows, d);
}

int fa_b200_exchange_alloc(size_t bytes, void** buf, void* ipc_handle_out) {
  if (!buf || !ipc_handle_out) return FA_B200_ERR_NULL;
  if (bytes == 0) return FA_B200_ERR_SHAPE;
  static_assert(sizeof(cudaIpcMemHandle_t) == FA_B200_IPC_HANDLE_BYTES, "IPC handle size");
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  if (e != cudaSuccess) return cuda_fail("exchange alloc", e);
  e = cudaMemset(ptr, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    cudaFree(ptr);
    return cuda_fail("exchange alloc", e);
  }
  memcpy(ipc_handle_out, &h, sizeof(h));
  *buf = ptr;
  return FA_B200_OK;
}

int fa_b200_exchange_open(const void* ipc_handle, void** peer) {
  if (!ipc_handle || !peer) return FA_B200_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(peer, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? FA_B200_OK : cuda_fail("exchange open", e);
}

int fa_b200_exchange_close(void* peer) {
  if (!peer) return FA_B200_ERR_NULL;
  cudaError_t e = cudaIpcCloseMemHandle(peer);
  return e == cudaSuccess ? FA_B200_OK : cuda_fail("exchange close", e);
}

int fa_b200_exchange_free(void* buf) {
  if (!buf) return FA_B200_ERR_NULL;
  cudaError_t e = cudaFree(buf);
  return e == cudaSuccess ? FA_B200_OK : cuda_fail("exchange free", e);
}

int fa_b200_exchange_combine(const fa_b200_exchange_params* p, void* stream) {
  if (!p) return FA_B200_ERR_NULL;
  if (p->struct_size != sizeof(fa_b200_exchange_params)) return FA_B200_ERR_ABI;
  if (p->world <= 0 || p->world > FA_B200_MAX_EXCHANGE_RANKS || p->rank < 0 || p->rank >= p->world) return FA_B200_ERR_SHAPE;
  if (p->rows < 0 || p->h <= 0 || p->rows % p->h != 0 || p->d <= 0 || p->d % 4 != 0 || p->epoch == 0) return FA_B200_ERR_SHAPE;
  if (p->do_push && (!p->o_local || !p->lse_local)) return FA_B200_ERR_NULL;
  for (int i = 0; i < p->world; ++i)
    if (!p->peers[i]) return FA_B200_ERR_NULL;
  if (!sink_dtype_ok(p->s_aux, p->s_aux_dtype)) return FA_B200_ERR_DTYPE;
  if (p->out_dtype != FA_B200_F16 && p->out_dtype != FA_B200_BF16 && p->out_dtype >= 0) return FA_B200_ERR_DTYPE;
  if ((p->o_local && !aligned16(p->o_local)) || (p->out && !aligned16(p->out))) return FA_B200_ERR_ALIGN;
  if (p->out && (p->out_batch_stride % 4 != 0 || p->out_head_stride % 4 != 0 || p->out_tok_stride % 4 != 0)) return FA_B200_ERR_STRIDE;
  ExchangeKernelParams k{};
  k.status = status_ptr();
  if (!k.status) return FA_B200_ERR_CUDA;
  k.o_local = p->o_local;
  k.lse_local = p->lse_local;
  for (int i = 0; i < p->world; ++i) k.peers[i] = p->peers[i];
  k.region_bytes = exchange_region_bytes(p->world, p->rows, p->d);
  k.out = p->out;
  k.lse = p->lse;
  k.out_batch_stride = p->out_batch_stride;
  k.out_row_stride = p->out_head_stride;
  k.out_tok_stride = p->out_tok_stride;
  k.world = p->world;
  k.rank = p->rank;
  k.rows = p->rows;
  k.h = p->h;
  k.sq = p->seqlen_q > 0 ? p->seqlen_q : 1;
  k.d = p->d;
  k.epoch = p->epoch;
  k.out_dtype = p->out_dtype;
  k.s_aux = p->s_aux;
  k.s_aux_dtype = p->s_aux_dtype;
  k.do_push = p->do_push;
  k.do_wait = p->do_wait;
  k.dependent_launch = g_env.dependent_launch;
  cudaError_t e = launch_exchange_combine(k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("exchange launch", e);
  if (p->rows > 0) g_launches++;
  return FA_B200_OK;
}

int fa_b200_decode_paged(const fa_b200_decode_params* p, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  DecodePlan pl = plan_decode(p);
  if (pl.status != FA_B200_OK) return pl.status;
  if (!p->q || !p->k_cache || !p->v_cache || !p->block_table || !p->cache_seqlens) return FA_B200_ERR_NULL;
  if (!p->out && !p->o_partial_out) return FA_B200_ERR_NULL;
  if (p->o_partial_out && !p->lse_partial_out) return FA_B200_ERR_NULL;
  if (p->out_dtype != FA_B200_F16 && p->out_dtype != FA_B200_BF16) return FA_B200_ERR_DTYPE;
  if (!sink_dtype_ok(p->s_aux, p->s_aux_dtype)) return FA_B200_ERR_DTYPE;
  const int kv_dtype = p->kv_e4m3 ? FA_B200_E4M3 : p->dtype;   // element type of the caches
  const int es = elem_size(kv_dtype), qes = elem_size(p->dtype);
  if (!aligned16(p->q) || !aligned16(p->k_cache) || !aligned16(p->v_cache) || (p->out && !aligned16(p->out)))
    return FA_B200_ERR_ALIGN;
  // the kernel reads q in 4-byte pieces (8-byte pieces for 16-bit queries over an e4m3 cache)
  const int q_piece = p->kv_e4m3 ? 8 : 4;
  if (!stride_ok(p->k_block_stride, es) || !stride_ok(p->k_row_stride, es) || !stride_ok(p->k_head_stride, es) ||
      !stride_ok(p->v_block_stride, es) || !stride_ok(p->v_row_stride, es) || !stride_ok(p->v_head_stride, es) ||
      (p->q_batch_stride * qes) % q_piece != 0 || (p->q_head_stride * qes) % q_piece != 0 ||
      (p->q_row_stride * qes) % q_piece != 0 || p->o_batch_stride % 8 != 0 || p->o_head_stride % 8 != 0)
    return FA_B200_ERR_STRIDE;
  if (p->b == 0) return FA_B200_OK;
  const size_t need = decode_ws_bytes(p, pl);
  if (need > 0 && (!p->workspace || p->workspace_bytes < need || !aligned16(p->workspace))) return FA_B200_ERR_WORKSPACE;

  CUtensorMap tk, tv;
  int st = make_tmap(&tk, p->k_cache, kv_dtype, p->h_k, p->page_size, p->num_blocks, p->k_head_stride, p->k_row_stride,
                     p->k_block_stride, pl.box_tok, p->d);
  if (st != FA_B200_OK) return st;
  if (p->v_transposed) {
    if (kv_dtype == FA_B200_E4M3) return FA_B200_ERR_UNSUPPORTED;
    if (p->page_size % 64 != 0) return FA_B200_ERR_PAGE;
    st = make_tmap_vt(&tv, p->v_cache, p->dtype, p->page_size, p->h_k, p->num_blocks, p->v_row_stride,
                      p->v_head_stride, p->v_block_stride);
  } else {
    st = make_tmap(&tv, p->v_cache, kv_dtype, p->h_k, p->page_size, p->num_blocks, p->v_head_stride, p->v_row_stride,
                   p->v_block_stride, pl.box_tok, p->d);
  }
  if (st != FA_B200_OK) return st;

  DecodeKernelParams k{};
  k.status = status_ptr();
  if (!k.status) return cuda_fail("status word", cudaGetLastError());
  k.q = p->q;
  k.out = p->out;
  k.lse_out = p->softmax_lse;
  k.block_table = p->block_table;
  k.seqlens = p->cache_seqlens;
  k.q_descale = p->q_descale;
  k.k_descale = p->k_descale;
  k.v_descale = p->v_descale;
  k.qds_b = p->q_descale_batch_stride; k.qds_h = p->q_descale_head_stride;
  k.kds_b = p->k_descale_batch_stride; k.kds_h = p->k_descale_head_stride;
  k.vds_b = p->v_descale_batch_stride; k.vds_h = p->v_descale_head_stride;
  k.q_batch_stride = p->q_batch_stride;
  k.q_head_stride = p->q_head_stride;
  k.o_batch_stride = p->o_batch_stride;
  k.o_head_stride = p->o_head_stride;
  k.bt_stride = p->block_table_batch_stride;
  k.b = p->b; k.h = p->h; k.h_k = p->h_k; k.group = pl.group;
  k.page_size = p->page_size;
  k.box_tok = pl.box_tok;
  k.partition_tokens = pl.partition_tokens;
  k.num_partitions = pl.num_partitions;
  k.out_dtype = p->out_dtype;
  k.write_final = pl.split ? 0 : 1;
  k.scale_log2 = p->softmax_scale * kLog2e;
  k.s_aux = p->s_aux;
  k.s_aux_dtype = p->s_aux_dtype;
  k.window_left = (p->has_window && p->window_left >= 0) ? p->window_left : -1;
  k.v_transposed = p->v_transposed ? 1 : 0;
  k.sq = p->seqlen_q > 1 ? p->seqlen_q : 1;
  k.causal = p->is_causal ? 1 : 0;
  k.kv_e4m3 = p->kv_e4m3 ? 1 : 0;
  k.kv_e5m2 = (p->kv_e4m3 && p->kv_e5m2) ? 1 : 0;
  k.d = p->d;
  k.q_row_stride = p->q_row_stride;
  k.o_row_stride = p->o_row_stride;
  k.max_len = pl.max_len;
  k.dependent_launch = g_env.dependent_launch;
#ifdef FA_B200_TEST_HOOKS
  k.test_withhold = g_test_withhold.exchange(0);
#endif
  bool merge_in_kernel = false;
  auto final_rows_to_caller = [&] {
    // where the merged rows go: the caller's out / lse, or (o_partial_out) fp32 rows (b, h, tok) for a cross-GPU
    // combine, whose final combine adds the sink
    if (p->o_partial_out) {
      k.out = p->o_partial_out;
      k.lse_out = p->lse_partial_out;
      k.o_batch_stride = static_cast<int64_t>(p->h) * k.sq * p->d;
      k.o_head_stride = static_cast<int64_t>(k.sq) * p->d;
      k.o_row_stride = p->d;
      k.out_dtype = -1;
      k.merge_lse_empty_is_neg = 1;
    } else {
      k.merge_sink = 1;
    }
  };
  if (pl.split) {
    k.o_partial = static_cast<float*>(p->workspace);
    k.lse_partial = k.o_partial + static_cast<size_t>(pl.num_partitions) * p->b * p->h * k.sq * p->d;
    // The last CTA of each (sequence, kv head) merges the partials itself when there are tickets to count on and the
    // grid is at most two rounds of the 296 resident CTA slots.  The merge saves a launch (about 5 us per step, which
    // is what counts for a small batch), but every CTA pays for it at its end: a fence and a ticket, and for the last
    // one of a group the dependent reads of the merge, 2 to 5 us in which its half of the SM streams nothing.  In a grid
    // of many rounds that adds up: 128 sequences x 8192 tokens of e4m3 (7 rounds of 58 us CTAs) measured 0.424 ms
    // with the merge in the kernel against 0.389 ms with the combine launch; bf16 CTAs are longer and HBM-bound, and
    // measured the same both ways.
    const int64_t ctas = static_cast<int64_t>(pl.num_partitions) * p->h_k * p->b;
    const bool want = g_env.decode_merge == 2 || (g_env.decode_merge == 0 && ctas <= 2 * 296);
    if (pl.num_partitions <= 256 && want) k.tickets = p->tickets ? p->tickets : stream_tickets(stream, static_cast<int64_t>(p->b) * p->h_k);
    merge_in_kernel = k.tickets != nullptr;
    if (merge_in_kernel) final_rows_to_caller();
  }
  {
    const char* dt = p->dtype == FA_B200_E4M3 ? "e4m3" : (p->dtype == FA_B200_BF16 ? "bf16" : "f16");
    const char* cache = p->kv_e4m3 ? (p->kv_e5m2 ? "+e5m2 cache" : "+e4m3 cache") : "";
    snprintf(g_launch_info, sizeof(g_launch_info),
             "fa_b200 decode: kernel=decode_paged dtype=%s%s d=%d b=%d h=%d h_k=%d seqlen_q=%d page=%d partition_tokens=%d "
             "partitions=%d grid=(%d,%d,%d) threads=160 merge=%s",
             dt, cache, p->d, p->b, p->h, p->h_k, k.sq, p->page_size, pl.partition_tokens, pl.num_partitions,
             pl.num_partitions, p->h_k, p->b,
             !pl.split ? "none (one partition)" : (merge_in_kernel ? "in-kernel (last CTA per sequence and kv head)" : "combine kernel"));
    if (print_param()) fprintf(stderr, "%s\n", g_launch_info);
  }
  if (p->profile_start_event) cudaEventRecord(static_cast<cudaEvent_t>(p->profile_start_event), stream);
  cudaError_t e = launch_decode(p->dtype, tk, tv, k, stream);
  if (e != cudaSuccess) return cuda_fail("decode launch", e);
  if (p->profile_stop_event) cudaEventRecord(static_cast<cudaEvent_t>(p->profile_stop_event), stream);
  g_launches++;
  if (pl.split && !merge_in_kernel) {
    CombineKernelParams c{};
    c.dependent_launch = g_env.dependent_launch;
    c.o_partial = k.o_partial;
    c.lse_partial = k.lse_partial;
    c.seqlens = p->cache_seqlens;
    c.parts_per_row = nullptr;
    c.num_parts = pl.num_partitions;
    c.rows = p->b * p->h * k.sq;
    c.h = p->h;
    c.sq = k.sq;
    c.partition_tokens = pl.partition_tokens;
    c.out_scale = 1.f;
    c.d = p->d;
    c.o_part_stride = static_cast<int64_t>(c.rows) * p->d;
    c.lse_part_stride = c.rows;
    if (p->o_partial_out) {
      c.out = p->o_partial_out;
      c.lse = p->lse_partial_out;
      c.out_row_stride = static_cast<int64_t>(k.sq) * p->d;          // partial rows are (b, h, tok)
      c.out_batch_stride = static_cast<int64_t>(p->h) * k.sq * p->d;
      c.out_tok_stride = p->d;
      c.out_dtype = -1;
      c.lse_empty_is_neg = 1;
    } else {
      c.out = p->out;
      c.lse = p->softmax_lse;
      c.out_row_stride = p->o_head_stride;
      c.out_batch_stride = p->o_batch_stride;
      c.out_tok_stride = p->o_row_stride;
      c.out_dtype = p->out_dtype;
      c.lse_empty_is_neg = 0;
      c.s_aux = p->s_aux;   // partials handed to the caller stay without the sink: its final combine adds it
      c.s_aux_dtype = p->s_aux_dtype;
    }
    e = launch_combine(c, stream);
    if (e != cudaSuccess) return cuda_fail("combine launch", e);
    g_launches++;
  }
  return FA_B200_OK;
}

// ---- decode without caller-provided scratch ------------------------------------------------------
// Split-KV partials for fa_b200_decode_paged_static.  One copy per device that loads the library.
static __device__ __align__(256) unsigned char g_static_scratch[FA_B200_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use: the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static void* static_scratch_ptr(cudaError_t* err) {
  static std::atomic<void*> ptrs[64];
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  void* cached = ptrs[dev].load(std::memory_order_acquire);
  if (!cached) {
    *err = cudaGetSymbolAddress(&cached, g_static_scratch);
    if (*err != cudaSuccess) return nullptr;
    ptrs[dev].store(cached, std::memory_order_release);
  }
  return cached;
}

int fa_b200_decode_paged_static(const fa_b200_decode_params* p, void* stream) {
  if (!p) return FA_B200_ERR_NULL;
  DecodePlan pl = plan_decode(p);
  if (pl.status != FA_B200_OK) return pl.status;
  const size_t need = decode_ws_bytes(p, pl);
  if (need > FA_B200_STATIC_SCRATCH_BYTES) {
    char buf[96];
    snprintf(buf, sizeof(buf), "needs %zu bytes of scratch, the built-in array holds %u", need,
             static_cast<unsigned>(FA_B200_STATIC_SCRATCH_BYTES));
    set_error("fa_b200_decode_paged_static", buf);
    return FA_B200_ERR_TOO_LARGE;
  }
  cudaError_t err = cudaSuccess;
  void* scratch = static_scratch_ptr(&err);
  if (!scratch) return cuda_fail("cudaGetSymbolAddress(static scratch)", err);
  fa_b200_decode_params q = *p;
  q.workspace = scratch;
  q.workspace_bytes = FA_B200_STATIC_SCRATCH_BYTES;
  return fa_b200_decode_paged(&q, stream);
}

static int fwd_common(const fa_b200_fwd_params* p, void* stream_, bool sparse) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!p) return FA_B200_ERR_NULL;
  if (p->struct_size != sizeof(fa_b200_fwd_params)) return FA_B200_ERR_ABI;
  if (!head_dim_ok(p->d, p->dtype == FA_B200_E4M3)) return FA_B200_ERR_HEADDIM;
  const int dv = p->d_v > 0 ? p->d_v : p->d;
  if (dv != p->d && !(p->d == 192 && dv == 128)) return FA_B200_ERR_HEADDIM;
  if (p->dtype != FA_B200_F16 && p->dtype != FA_B200_BF16 && p->dtype != FA_B200_E4M3) return FA_B200_ERR_DTYPE;
  if (p->out_dtype != FA_B200_F16 && p->out_dtype != FA_B200_BF16) return FA_B200_ERR_DTYPE;
  if (!sink_dtype_ok(p->s_aux, p->s_aux_dtype)) return FA_B200_ERR_DTYPE;
  if (p->b < 0 || p->h <= 0 || p->h_k <= 0 || p->seqlen_q < 0 || p->seqlen_k < 0) return FA_B200_ERR_SHAPE;
  if (p->h % p->h_k != 0) return FA_B200_ERR_HEADS;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const bool paged = p->block_table != nullptr;
  if (!paged && varlen != (p->cu_seqlens_k != nullptr)) return FA_B200_ERR_NULL;
  int box_rows = 128;
  if (paged) {
    if (sparse) return FA_B200_ERR_UNSUPPORTED;
    if (!p->seqused_k) return FA_B200_ERR_NULL;
    if (p->num_blocks <= 0) return FA_B200_ERR_SHAPE;
    const int page = p->page_size;
    if (page >= 128 && page % 128 == 0) box_rows = 128;
    else if (page >= 64 && page % 64 == 0) box_rows = 64;
    else if (page == 16 || page == 32) box_rows = page;
    else return FA_B200_ERR_PAGE;
  }
  if (p->v_transposed) {
    if (!paged || p->dtype == FA_B200_E4M3) return FA_B200_ERR_UNSUPPORTED;
    if (p->d != kHeadDim || dv != kHeadDim) return FA_B200_ERR_HEADDIM;
    if (p->page_size % 64 != 0) return FA_B200_ERR_PAGE;
  }
  if (varlen && (p->total_q < 0 || p->total_k < 0)) return FA_B200_ERR_SHAPE;
  if (p->b == 0 || p->seqlen_q == 0 || (varlen && p->total_q == 0)) return FA_B200_OK;
  if (!p->q || !p->out) return FA_B200_ERR_NULL;
  const bool has_k = paged ? true : (varlen ? p->total_k > 0 : p->seqlen_k > 0);
  if (has_k && (!p->k || !p->v)) return FA_B200_ERR_NULL;
  const int es = elem_size(p->dtype);
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return FA_B200_ERR_ALIGN;
  if (!stride_ok(p->q_row_stride, es) || !stride_ok(p->q_head_stride, es) || !stride_ok(p->k_row_stride, es) ||
      !stride_ok(p->k_head_stride, es) || !stride_ok(p->v_row_stride, es) || !stride_ok(p->v_head_stride, es) ||
      (!varlen && !stride_ok(p->q_batch_stride, es)) ||
      ((!varlen || paged) && (!stride_ok(p->k_batch_stride, es) || !stride_ok(p->v_batch_stride, es))) ||
      p->o_row_stride % 8 != 0 || p->o_head_stride % 8 != 0 || (!varlen && p->o_batch_stride % 8 != 0))
    return FA_B200_ERR_STRIDE;
  if (sparse) {
    if (!p->block_count || !p->block_offset) return FA_B200_ERR_NULL;
    // packed sequences: the lists are (b, h, num_q_blocks, nnz_s) with num_q_blocks counted on the LONGEST sequence and
    // key row offsets relative to each sequence's first key (mha_varlen_fwd_sparse, flash_api_sparse.cpp:339-558)
    if ((p->block_m != 64 && p->block_m != 128) || p->nnz_s <= 0 || p->nnz_s > 512) return FA_B200_ERR_SHAPE;
    if (p->num_q_blocks != (p->seqlen_q + p->block_m - 1) / p->block_m) return FA_B200_ERR_SHAPE;
  }

  CUtensorMap tq, tk, tv;
  const int64_t q_rows = varlen ? p->total_q : p->seqlen_q, k_rows = varlen ? p->total_k : p->seqlen_k;
  const int64_t nb = varlen ? 1 : p->b;
  int st = make_tmap(&tq, p->q, p->dtype, p->h, q_rows, nb, p->q_head_stride, p->q_row_stride,
                     varlen ? p->q_row_stride * (q_rows > 0 ? q_rows : 1) : p->q_batch_stride, 128, p->d);
  if (st != FA_B200_OK) return st;
  if (paged) {
    st = make_tmap(&tk, p->k, p->dtype, p->h_k, p->page_size, p->num_blocks, p->k_head_stride, p->k_row_stride,
                   p->k_batch_stride, box_rows, p->d);
    if (st != FA_B200_OK) return st;
    if (p->v_transposed)
      st = make_tmap_vt(&tv, p->v, p->dtype, p->page_size, p->h_k, p->num_blocks, p->v_row_stride, p->v_head_stride,
                        p->v_batch_stride);
    else
      st = make_tmap(&tv, p->v, p->dtype, p->h_k, p->page_size, p->num_blocks, p->v_head_stride, p->v_row_stride,
                     p->v_batch_stride, box_rows, dv);
  } else {
    st = make_tmap(&tk, p->k, p->dtype, p->h_k, k_rows, nb, p->k_head_stride, p->k_row_stride,
                   varlen ? p->k_row_stride * (k_rows > 0 ? k_rows : 1) : p->k_batch_stride, 128, p->d);
    if (st != FA_B200_OK) return st;
    st = make_tmap(&tv, p->v, p->dtype, p->h_k, k_rows, nb, p->v_head_stride, p->v_row_stride,
                   varlen ? p->v_row_stride * (k_rows > 0 ? k_rows : 1) : p->v_batch_stride, 128, dv);
  }
  if (st != FA_B200_OK) return st;

  // output map for whole-tile stores (strides and base are 16-byte aligned by the checks above)
  CUtensorMap to;
  st = make_tmap(&to, p->out, p->out_dtype, p->h, q_rows, nb, p->o_head_stride, p->o_row_stride,
                 varlen ? p->o_row_stride * (q_rows > 0 ? q_rows : 1) : p->o_batch_stride, 128, dv);
  if (st != FA_B200_OK) return st;

  PrefillKernelParams k{};
  k.status = status_ptr();
  if (!k.status) return cuda_fail("status word", cudaGetLastError());
  k.o_tma = 1;
  k.d = p->d;
  k.d_v = dv;
  k.v_transposed = p->v_transposed ? 1 : 0;
  k.s_aux = p->s_aux;
  k.s_aux_dtype = p->s_aux_dtype;
  k.out = p->out;
  k.lse = p->softmax_lse;
  k.cu_seqlens_q = p->cu_seqlens_q;
  k.cu_seqlens_k = p->cu_seqlens_k;
  k.q_descale = p->q_descale; k.k_descale = p->k_descale; k.v_descale = p->v_descale;
  k.qds_b = p->q_descale_batch_stride; k.qds_h = p->q_descale_head_stride;
  k.kds_b = p->k_descale_batch_stride; k.kds_h = p->k_descale_head_stride;
  k.vds_b = p->v_descale_batch_stride; k.vds_h = p->v_descale_head_stride;
  k.o_batch_stride = varlen ? 0 : p->o_batch_stride;
  k.o_row_stride = p->o_row_stride;
  k.o_head_stride = p->o_head_stride;
  k.total_q = p->total_q;
  k.b = p->b; k.h = p->h; k.h_k = p->h_k;
  k.seqlen_q = p->seqlen_q; k.seqlen_k = p->seqlen_k;
  k.is_causal = p->is_causal ? 1 : 0;
  k.window_left = (p->has_window && p->window_left >= 0) ? p->window_left : -1;
  k.window_right = p->is_causal ? 0 : ((p->has_window && p->window_right >= 0) ? p->window_right : -1);
  if (sparse && (k.window_left >= 0 || (k.window_right >= 0 && !p->is_causal))) return FA_B200_ERR_UNSUPPORTED;
  k.out_dtype = p->out_dtype;
  k.scale_log2 = p->softmax_scale * kLog2e;
  k.sparse = sparse ? 1 : 0;
  k.paged = paged ? 1 : 0;
  if (paged) {
    k.block_table = p->block_table;
    k.bt_stride = p->block_table_batch_stride;
    k.seqused_k = p->seqused_k;
    k.page_size = p->page_size;
    k.box_rows = box_rows;
    k.max_keys = p->max_blocks_per_seq > 0 ? static_cast<int64_t>(p->max_blocks_per_seq) * p->page_size : 0;
  }
  if (sparse) {
    k.block_count = p->block_count;
    k.block_offset = p->block_offset;
    k.column_count = p->column_count;
    k.num_q_blocks = p->num_q_blocks;
    k.nnz_s = p->nnz_s;
    k.block_m = p->block_m;
    k.num_m_blocks = p->num_q_blocks;
  } else {
    k.num_m_blocks = (p->seqlen_q + 127) / 128;
  }
  // Kernel choice.  Dense / varlen prefill with an even GQA group: persistent CTAs that work on two heads of the
  // group at once and share every K/V tile ("pair").  Other head layouts (MHA, odd groups): one tile per CTA ("single"),
  // and for long sequences persistent CTAs with double-buffered scores ("dense").  Tile lists are per head: "single".
  // kernel_choice / FA_B200_PREFILL_KERNEL override the choice where the chosen kernel can take the call.
  const bool even_group = (p->h / p->h_k) % 2 == 0;
  // Tile lists and other head dimensions: the one-tile kernel.  Paged K/V: the two-tile kernel where the GQA group is
  // even (any pool layout), else the double-buffered kernel, which reads the block table too but no transposed V pool.
  const bool one_tile_only = sparse || p->d != kHeadDim || (paged && !even_group && p->v_transposed);
  // MHA and odd groups, measured (bf16, causal, 16 / 16 and 24 / 8 heads): the one-tile kernel with two CTAs per SM is
  // ahead of the double-buffered persistent kernel up to a few thousand tokens per sequence (8 x 4096: 884 against 728
  // TFLOP/s; 32 x 1024: 536 against 441; paged 8 x 4096: 850 against 705) and level or behind at 16384 (923 / 920 and
  // 865 / 901), so the persistent kernel takes over above 8192 query tokens.
  int which = one_tile_only ? 0 : (even_group ? 1 : (p->seqlen_q > 8192 ? 2 : 0));
  const int choice = p->kernel_choice > 0 ? p->kernel_choice : g_env.prefill_kernel;
  if (choice == 1) which = 0;
  else if (choice == 2 && !one_tile_only && even_group) which = 1;
  else if (choice == 3 && !one_tile_only && !(paged && p->v_transposed)) which = 2;
#ifdef FA_B200_TEST_HOOKS
  if (which == 1) k.test_withhold = g_test_withhold.exchange(0);
#endif
  if (which != 0) {   // the persistent kernels claim their work items from a counter
    if (p->work_counter) {   // the caller's own counter
      if (cudaMemsetAsync(p->work_counter, 0, sizeof(int), stream) != cudaSuccess) return cuda_fail("work counter", cudaGetLastError());
      k.work_counter = p->work_counter;
    } else {
      k.work_counter = next_work_counter(stream);
    }
    if (!k.work_counter) return cuda_fail("work counter", cudaGetLastError());
  }
  {
    static const char* const names[3] = {"prefill_single (one query tile per CTA, two CTAs per SM)",
                                         "prefill_pair (persistent, two heads of a GQA group per item)",
                                         "prefill_dense (persistent, double-buffered scores)"};
    const char* dt = p->dtype == FA_B200_E4M3 ? "e4m3" : (p->dtype == FA_B200_BF16 ? "bf16" : "f16");
    snprintf(g_launch_info, sizeof(g_launch_info),
             "fa_b200 prefill: kernel=%s dtype=%s d=%d d_v=%d b=%d h=%d h_k=%d seqlen_q=%d seqlen_k=%d varlen=%d paged=%d "
             "tile_lists=%d causal=%d window=(%d,%d) q_blocks=%d",
             names[which], dt, p->d, dv, p->b, p->h, p->h_k, p->seqlen_q, p->seqlen_k, varlen ? 1 : 0, paged ? 1 : 0,
             sparse ? 1 : 0, k.is_causal, k.window_left, k.window_right, k.num_m_blocks);
    if (print_param()) fprintf(stderr, "%s\n", g_launch_info);
  }
  if (p->profile_start_event) cudaEventRecord(static_cast<cudaEvent_t>(p->profile_start_event), stream);
  cudaError_t e = which == 2   ? launch_prefill_dense(p->dtype, tq, tk, tv, k, stream)
                  : which == 1 ? launch_prefill_pair(p->dtype, tq, tk, tv, to, k, stream)
                               : launch_prefill_single(p->dtype, tq, tk, tv, k, stream);
  if (e != cudaSuccess) return cuda_fail("prefill launch", e);
  if (p->profile_stop_event) cudaEventRecord(static_cast<cudaEvent_t>(p->profile_stop_event), stream);
  g_launches++;
  return FA_B200_OK;
}

int fa_b200_fwd(const fa_b200_fwd_params* p, void* stream) { return fwd_common(p, stream, false); }
int fa_b200_fwd_sparse(const fa_b200_fwd_params* p, void* stream) { return fwd_common(p, stream, true); }

int fa_b200_block_pool(const void* x, int32_t dtype, int64_t batch_stride, int64_t head_stride, int64_t row_stride,
                       int32_t b, int32_t h, int32_t n, int32_t d, int32_t block_rows, const float* sim_threshold,
                       void* pooled, uint8_t* sim, void* stream) {
  if (dtype != FA_B200_F16 && dtype != FA_B200_BF16) return FA_B200_ERR_DTYPE;
  if (d != 64 && d != 128 && d != 256) return FA_B200_ERR_HEADDIM;
  if (b < 0 || h <= 0 || n < 0 || block_rows <= 0 || block_rows > 128) return FA_B200_ERR_SHAPE;
  if (b == 0 || n == 0) return FA_B200_OK;
  if (!x || !sim_threshold || !pooled || !sim) return FA_B200_ERR_NULL;
  const int piece = d / 32 * 2;   // bytes one lane loads
  if (reinterpret_cast<uintptr_t>(x) % piece != 0 || (batch_stride * 2) % piece != 0 || (head_stride * 2) % piece != 0 ||
      (row_stride * 2) % piece != 0)
    return FA_B200_ERR_STRIDE;
  BlockPoolParams k{};
  k.x = x; k.batch_stride = batch_stride; k.head_stride = head_stride; k.row_stride = row_stride;
  k.b = b; k.h = h; k.n = n; k.d = d; k.dtype = dtype;
  k.block_rows = block_rows; k.num_blocks = (n + block_rows - 1) / block_rows;
  k.sim_threshold = sim_threshold; k.pooled = pooled; k.sim = sim;
  cudaError_t e = launch_block_pool(k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("block pool launch", e);
  g_launches++;
  return FA_B200_OK;
}

int fa_b200_block_select(const void* pooled_q, const void* pooled_k, const uint8_t* sim_q, const uint8_t* sim_k,
                         int32_t dtype, int32_t b, int32_t h, int32_t nq, int32_t nk, int32_t d, int32_t block_q,
                         int32_t block_k, float scale, const float* cdf_threshold, const float* topk, int32_t is_causal,
                         int32_t attention_sink, uint8_t* block_map, void* stream) {
  if (dtype != FA_B200_F16 && dtype != FA_B200_BF16) return FA_B200_ERR_DTYPE;
  if (d <= 0 || d > 256) return FA_B200_ERR_HEADDIM;
  if (b < 0 || h <= 0 || nq < 0 || nk < 0 || block_q <= 0 || block_k <= 0) return FA_B200_ERR_SHAPE;
  if (nk > block_select_max_key_blocks()) return FA_B200_ERR_TOO_LARGE;
  if ((cdf_threshold == nullptr) == (topk == nullptr)) return FA_B200_ERR_UNSUPPORTED;   // exactly one of the two
  if (b == 0 || nq == 0 || nk == 0) return FA_B200_OK;
  if (!pooled_q || !pooled_k || !sim_q || !sim_k || !block_map) return FA_B200_ERR_NULL;
  BlockSelectParams k{};
  k.pooled_q = pooled_q; k.pooled_k = pooled_k; k.sim_q = sim_q; k.sim_k = sim_k;
  k.dtype = dtype; k.b = b; k.h = h; k.nq = nq; k.nk = nk; k.d = d;
  k.nk_pow2 = 2;
  while (k.nk_pow2 < nk) k.nk_pow2 *= 2;
  k.block_q = block_q; k.block_k = block_k; k.scale = scale;
  k.cdf_threshold = cdf_threshold; k.topk = topk;
  k.is_causal = is_causal ? 1 : 0; k.attention_sink = attention_sink ? 1 : 0;
  k.block_map = block_map;
  cudaError_t e = launch_block_select(k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("block select launch", e);
  g_launches++;
  return FA_B200_OK;
}

namespace {
// The decode parameters of the raw-pointer entry (sizes only for the workspace query).
fa_b200_decode_params raw_decode_params(int32_t num_query, int32_t num_q_head, int32_t num_kv_head, int32_t num_dim,
                                        int32_t num_pages, int32_t page_size, int32_t max_seqlen_k, int32_t dtype) {
  fa_b200_decode_params d{};
  d.struct_size = sizeof(d);
  d.b = num_query; d.h = num_q_head; d.h_k = num_kv_head; d.d = num_dim;
  d.num_blocks = num_pages; d.page_size = page_size;
  d.max_blocks_per_seq = page_size > 0 ? (max_seqlen_k - 1) / page_size + 1 : 0;
  d.max_seqlen_k = max_seqlen_k;
  d.dtype = dtype; d.out_dtype = dtype;
  return d;
}
}  // namespace

size_t fa_b200_kv_cache_attention_workspace_bytes(int32_t num_query, int32_t num_q_head, int32_t num_kv_head,
                                                  int32_t num_dim, int32_t page_size, int32_t max_seqlen_k) {
  // the pool size and the 16-bit element type do not enter the partition plan
  fa_b200_decode_params d = raw_decode_params(num_query, num_q_head, num_kv_head, num_dim, 1, page_size, max_seqlen_k,
                                              FA_B200_BF16);
  return fa_b200_decode_workspace_bytes(&d);
}

int fa_b200_kv_cache_attention(const void* q, const int32_t* seq_offsets, int32_t max_seqlen_q, int32_t max_seqlen_k,
                               const void* k_caches, const void* v_caches, const int32_t* page_tables,
                               const int32_t* cache_lens, void* out, int32_t num_query, int32_t num_tokens,
                               int32_t num_q_head, int32_t num_kv_head, int32_t num_dim, int32_t num_pages,
                               int32_t page_size, int32_t dtype, int32_t layout, void* workspace, size_t workspace_bytes,
                               void* stream) {
  if (dtype != FA_B200_F16 && dtype != FA_B200_BF16) return FA_B200_ERR_DTYPE;
  if (layout < 0 || layout > 2) return FA_B200_ERR_UNSUPPORTED;
  if (num_query < 0 || num_tokens < num_query || num_q_head <= 0 || num_kv_head <= 0 || num_pages <= 0 || page_size <= 0 ||
      max_seqlen_k <= 0)
    return FA_B200_ERR_SHAPE;
  if (!head_dim_ok(num_dim, layout == 0)) return FA_B200_ERR_HEADDIM;
  if (num_query == 0) return FA_B200_OK;
  const int64_t d = num_dim, hk = num_kv_head, ps = page_size;
  const int64_t block_stride = hk * ps * d;
  const int64_t row_stride = layout == 2 ? hk * d : d, head_stride = layout == 2 ? d : ps * d;
  const int32_t max_pages = (max_seqlen_k - 1) / page_size + 1;
  const float scale = 1.0f / sqrtf(static_cast<float>(num_dim));
  if (num_query == num_tokens) {
    fa_b200_decode_params p = raw_decode_params(num_query, num_q_head, num_kv_head, num_dim, num_pages, page_size,
                                                max_seqlen_k, dtype);
    p.q = q; p.k_cache = k_caches; p.v_cache = v_caches; p.out = out;
    p.q_batch_stride = p.o_batch_stride = static_cast<int64_t>(num_q_head) * d;
    p.q_head_stride = p.o_head_stride = d;
    p.k_block_stride = p.v_block_stride = block_stride;
    p.k_row_stride = row_stride; p.k_head_stride = head_stride;
    if (layout == 0) {   // V (pages, kv heads, d, page): "row" = one d row of page_size tokens
      p.v_transposed = 1; p.v_row_stride = ps; p.v_head_stride = d * ps;
      p.k_row_stride = d; p.k_head_stride = ps * d;
    } else {
      p.v_row_stride = row_stride; p.v_head_stride = head_stride;
    }
    p.block_table = page_tables; p.block_table_batch_stride = max_pages;
    p.cache_seqlens = cache_lens;
    p.softmax_scale = scale;
    p.workspace = workspace; p.workspace_bytes = workspace_bytes;
    return fa_b200_decode_paged(&p, stream);
  }
  if (!seq_offsets) return FA_B200_ERR_NULL;
  fa_b200_fwd_params p{};
  p.struct_size = sizeof(p);
  p.q = q; p.k = k_caches; p.v = v_caches; p.out = out;
  p.q_row_stride = p.o_row_stride = static_cast<int64_t>(num_q_head) * d;
  p.q_head_stride = p.o_head_stride = d;
  p.k_batch_stride = p.v_batch_stride = block_stride;
  p.k_row_stride = p.v_row_stride = row_stride;
  p.k_head_stride = p.v_head_stride = head_stride;
  if (layout == 0) {   // V (pages, kv heads, d, page)
    p.v_transposed = 1; p.v_row_stride = ps; p.v_head_stride = d * ps;
  }
  p.b = num_query; p.seqlen_q = max_seqlen_q; p.seqlen_k = max_seqlen_k;
  p.h = num_q_head; p.h_k = num_kv_head; p.d = num_dim;
  p.total_q = num_tokens; p.total_k = 0;
  p.cu_seqlens_q = seq_offsets;
  p.softmax_scale = scale;
  p.is_causal = 1;
  p.dtype = dtype; p.out_dtype = dtype;
  p.block_table = page_tables; p.block_table_batch_stride = max_pages;
  p.seqused_k = cache_lens;
  p.page_size = page_size; p.num_blocks = num_pages;
  p.max_blocks_per_seq = max_pages;
  return fa_b200_fwd(&p, stream);
}

}  // extern "C"
