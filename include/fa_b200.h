/*
 * fa_b200.h — C ABI of libfa_b200.so: the forward attention hot path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers to DEVICE memory, sizes and strides (in elements), and a
 * CUDA stream passed as void* (a cudaStream_t).  Nothing here allocates, synchronises or throws:
 * a call validates its arguments, enqueues kernels on the given stream and returns a status code
 * (0 = ok).  Scratch memory is owned by the caller (see fa_b200_decode_workspace_bytes).
 *
 * The "replaces" notes name the interface of the reference project (HYGON-AI/flash-attention-das,
 * paths relative to its root) that each entry point stands in for.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Version 2: every parameter struct starts with struct_size (callers set it to sizeof of the struct they compiled
 * against; a call whose struct_size differs from the library's own is refused with FA_B200_ERR_ABI before any other
 * field is read), the decode struct gained `tickets`, the forward struct `kernel_choice` and `max_blocks_per_seq`. */
#define FA_B200_ABI_VERSION 2

#if defined(__GNUC__)
#define FA_B200_API __attribute__((visibility("default")))
#else
#define FA_B200_API
#endif

/* element types */
enum { FA_B200_F16 = 0, FA_B200_BF16 = 1, FA_B200_E4M3 = 2, FA_B200_F32 = 3 /* s_aux only */ };

/* status codes (host side).  fa_b200_status_string() gives the text. */
enum {
  FA_B200_OK = 0,
  FA_B200_ERR_NULL = 1,          /* a required pointer is null */
  FA_B200_ERR_DTYPE = 2,         /* unsupported element type combination */
  FA_B200_ERR_HEADDIM = 3,       /* head dimension not 128 (64, 192, 256: fp16 / bf16 in the plain layouts only) */
  FA_B200_ERR_HEADS = 4,         /* h not a multiple of h_k, or group too large for the decode tile */
  FA_B200_ERR_STRIDE = 5,        /* last dim not contiguous / stride not 16-byte aligned */
  FA_B200_ERR_SHAPE = 6,         /* negative or inconsistent sizes */
  FA_B200_ERR_PAGE = 7,          /* page size not a multiple of 16 (or of 64 above 64) */
  FA_B200_ERR_WORKSPACE = 8,     /* workspace missing or too small */
  FA_B200_ERR_UNSUPPORTED = 9,   /* option outside the hot path */
  FA_B200_ERR_CUDA = 10,         /* a CUDA runtime / driver call failed; see fa_b200_last_cuda_error */
  FA_B200_ERR_ALIGN = 11,        /* base pointer not 16-byte aligned */
  FA_B200_ERR_DEVICE_TIMEOUT = 12, /* a bounded device-side wait gave up (reported by fa_b200_device_status) */
  FA_B200_ERR_TOO_LARGE = 13,    /* size beyond a fixed built-in limit */
  FA_B200_ERR_DEVICE_RANGE = 14, /* a kernel skipped an out-of-range position or page id (fa_b200_device_status) */
  FA_B200_ERR_DEVICE_UNSUPPORTED = 15, /* a kernel met device-resident input it does not take (fa_b200_device_status) */
  FA_B200_ERR_ABI = 16           /* struct_size is not the size of this library's struct: header / library mismatch */
};

/*
 * Dense and varlen forward (also the block-sparse forward when block_count/block_offset are set).
 * Mirrors the fields of Flash_fwd_params that the forward path reads
 * (csrc/flash_attn_cutlass/src/flash.h:52-206): pointers, batch/row/head strides in ELEMENTS,
 * b, h, h_k, seqlen_q/k, d, total_q, cu_seqlens, scale, descale pointers and strides, is_causal.
 * d = 128 for every element type; 64, 192 and 256 for F16 / BF16 (see also d_v).
 *
 * Fixed length: cu_seqlens_q == cu_seqlens_k == NULL; q is (b, seqlen_q, h, d), k/v (b, seqlen_k, h_k, d);
 *               softmax_lse is (b, h, seqlen_q) fp32.
 * Varlen:       q is (total_q, h, d), k/v (total_k, h_k, d) packed; cu_seqlens_* are int32 (b + 1);
 *               seqlen_q/seqlen_k are the MAXIMUM lengths; softmax_lse is (h, total_q) fp32.
 * Fully masked rows give out = 0 and lse = +inf.  The causal mask is bottom-right aligned.
 */
typedef struct fa_b200_fwd_params {
  uint32_t struct_size;                /* sizeof(fa_b200_fwd_params) */
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* softmax_lse;
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int32_t b, seqlen_q, seqlen_k, h, h_k, d;
  int64_t total_q, total_k;            /* varlen only */
  const int32_t* cu_seqlens_q;         /* NULL for fixed length */
  const int32_t* cu_seqlens_k;
  float softmax_scale;
  int32_t is_causal;
  int32_t dtype;                       /* of q, k, v: FA_B200_F16 / BF16 / E4M3 */
  int32_t out_dtype;                   /* F16 or BF16 (BF16 for E4M3 inputs by default) */
  /* FP8 descale, fp32, indexed [batch * batch_stride + kv_head * head_stride]; NULL = 1.0 */
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  int64_t q_descale_batch_stride, q_descale_head_stride;
  int64_t k_descale_batch_stride, k_descale_head_stride;
  int64_t v_descale_batch_stride, v_descale_head_stride;
  /* block-sparse lists (fa_b200_fwd_sparse only), int32:
   *   block_count  (b, h, num_q_blocks), block_offset (b, h, num_q_blocks, nnz_s) = ascending K ROW
   *   offsets of 64-row K tiles (csrc/flash_attn_cutlass/flash_api_sparse.cpp:70-138). */
  const int32_t* block_count;
  const int32_t* block_offset;
  int32_t num_q_blocks, nnz_s, block_m;
  /* Optional cudaEvent_t handles recorded on the stream right before and right after the attention
   * kernel (timing of the dominant kernel alone); NULL = off. */
  void* profile_start_event;
  void* profile_stop_event;
  /* Paged K/V (fa_b200_fwd only): when block_table is set, k and v are pools (num_blocks, page_size, h_k, d) whose
   * block stride is k_batch_stride / v_batch_stride; int32 block_table (b, max_blocks) lists each sequence's pages and
   * int32 seqused_k (b) its number of keys (cu_seqlens_k is not read; seqlen_k is an upper bound).  Page sizes 16, 32
   * and multiples of 64.  Replaces the block_table branch of the reference's varlen entry
   * (flash_attn/flash_attn_interface.py:2223-2405: pagedkv_to_contiguous + varlen_fwd) without the gather copy. */
  const int32_t* block_table;
  int64_t block_table_batch_stride;
  const int32_t* seqused_k;
  int32_t page_size, num_blocks;
  /* Attention sinks (flash_attn_func(..., s_aux=), tests/test_flash_attn_saux.py:206-224): one extra logit per query
   * head that takes part in the softmax denominator and carries no value; (h) elements of type s_aux_dtype
   * (FA_B200_F16 / FA_B200_BF16, or FA_B200_F32), not multiplied by softmax_scale.  NULL = off. */
  const void* s_aux;
  int32_t s_aux_dtype;
  /* Sliding window (flash_attn_func(..., window_size=(left, right)), construct_local_mask in
   * tests/test_flash_attn.py:185-217): with has_window != 0, query i of a sequence with sq queries and sk keys sees key
   * j iff  i + sk - sq - window_left <= j <= i + sk - sq + window_right;  a negative value leaves that side open.
   * is_causal forces window_right = 0.  Not available with tile lists (fa_b200_fwd_sparse). */
  int32_t has_window, window_left, window_right;
  /* fa_b200_fwd_sparse only: the reference's vertical part of the sparsity pattern (column_count / column_index,
   * flash_attn_interface.py:2778-2855) is not built; pass column_count (b, h, num_q_blocks) here and a row whose count
   * is not zero is reported by fa_b200_device_status() as FA_B200_ERR_DEVICE_UNSUPPORTED (checked on the device: no host
   * synchronisation).  NULL = not checked. */
  const int32_t* column_count;
  /* Head dimension of v and out when it differs from d (q and k): the pair d = 192, d_v = 128 (fp16 / bf16), the
   * multi-head latent attention prefill shape the reference takes in its bshd paths (flash_attn_interface.py:2241-2242).
   * 0 = same as d. */
  int32_t d_v;
  /* Paged V stored transposed, (num_blocks, h_k, d, page_size) with the tokens of a page contiguous (the reference's
   * paged layout 0 / "custom", flash_attn/flash_attn_interface.py:2223-2227; K is then (num_blocks, h_k, page_size, d),
   * which the K strides express).  With v_transposed != 0, v_row_stride is the stride between consecutive d rows.
   * Needs block_table; F16 / BF16, d = 128, page_size a multiple of 64. */
  int32_t v_transposed;
  /* Optional int32 in device memory, owned by the caller for the duration of the kernel: the persistent prefill kernels
   * hand out their work items from it (the call zeroes it on the stream first).  NULL = a counter inside the library
   * that belongs to the (device, stream) pair of the call: launches of one stream follow each other and share it,
   * different streams use different ones (up to 64 streams with launches in flight).  A caller that replays a captured
   * launch on another stream than it was captured on, while launches run on the capture stream, should give each
   * captured call its own counter. */
  int32_t* work_counter;
  /* Kernel choice for this call: 0 = the library decides (or FA_B200_PREFILL_KERNEL, read when the library is loaded),
   * 1 = one query tile per CTA, 2 = persistent two-heads-per-item kernel, 3 = persistent double-buffered kernel.  A
   * choice the call cannot take (tile lists, other head dimensions, odd GQA groups for 2 ...) falls back to the
   * library's own. */
  int32_t kernel_choice;
  /* Paged K/V: columns of block_table that hold page ids.  A seqused_k entry beyond max_blocks_per_seq * page_size is
   * cut to that and reported by fa_b200_device_status() as FA_B200_ERR_DEVICE_RANGE.  0 = not given, not checked. */
  int32_t max_blocks_per_seq;
} fa_b200_fwd_params;

/* Replaces mha_fwd / mha_varlen_fwd -> run_mha_fwd -> flash_fwd_kernel_16x64_prefetch
 * (csrc/flash_attn_cutlass/flash_api.cpp:951-1215, 1216-1685; flash_c_api.cpp:96-144;
 *  src/flash_fwd_kernel.h:2818-3328, FP8: 3330-3778). */
FA_B200_API int fa_b200_fwd(const fa_b200_fwd_params* p, void* stream);

/* Replaces mha_fwd_sparse and mha_varlen_fwd_sparse -> run_mha_fwd_sparse -> sparse_attn_1rowblock
 * (csrc/flash_attn_cutlass/flash_api_sparse.cpp:170-338, 339-558, 140-149;
 *  src/flash_fwd_sparse_kernel.h:36-775), block-list path only.  With cu_seqlens (packed sequences) the lists are
 * (b, h, num_q_blocks, nnz_s) with num_q_blocks = ceil(seqlen_q / block_m) counted on the longest sequence, and the
 * key row offsets are relative to each sequence's first key. */
FA_B200_API int fa_b200_fwd_sparse(const fa_b200_fwd_params* p, void* stream);

/*
 * Paged-KV decode (one query token per sequence, or a few: seqlen_q; GQA group packed into one query tile), split-KV
 * over fixed-size token partitions plus an LSE-combine kernel.  d = 128; 64, 192 and 256 for F16 / BF16 caches in the
 * plain layout.
 * k_cache / v_cache: (num_blocks, page_size, h_k, d); block_table: int32 (b, max_blocks_per_seq);
 * cache_seqlens: int32 (b).  Physical page of token t of sequence s is
 * block_table[s * block_table_batch_stride + t / page_size], row t % page_size
 * (same addressing as src/paged_attention.cu:146,209 and paged_attention_decode_arch.h:3992-3998).
 * A cache_seqlens entry beyond what the call covers (max_blocks_per_seq * page_size, or max_seqlen_k if that is
 * smaller) is cut to it and reported by fa_b200_device_status() as FA_B200_ERR_DEVICE_RANGE: the kernel never reads
 * past a block_table row.
 */
typedef struct fa_b200_decode_params {
  uint32_t struct_size;                /* sizeof(fa_b200_decode_params) */
  const void* q;                       /* (b, 1, h, d) */
  const void* k_cache;
  const void* v_cache;
  void* out;                           /* (b, 1, h, d) */
  float* softmax_lse;                  /* (b, h) fp32 or NULL */
  int64_t q_batch_stride, q_head_stride;
  int64_t o_batch_stride, o_head_stride;
  int64_t k_block_stride, k_row_stride, k_head_stride;
  int64_t v_block_stride, v_row_stride, v_head_stride;
  const int32_t* block_table;
  int64_t block_table_batch_stride;
  const int32_t* cache_seqlens;
  int32_t b, h, h_k, d;
  int32_t num_blocks, page_size, max_blocks_per_seq;
  float softmax_scale;
  int32_t dtype;                       /* of q and the cache */
  int32_t out_dtype;
  const float* q_descale;              /* as in fa_b200_fwd_params */
  const float* k_descale;
  const float* v_descale;
  int64_t q_descale_batch_stride, q_descale_head_stride;
  int64_t k_descale_batch_stride, k_descale_head_stride;
  int64_t v_descale_batch_stride, v_descale_head_stride;
  int32_t partition_tokens;            /* 0 = heuristic; else a multiple of 64 (128 for E4M3) */
  int32_t max_seqlen_k;                /* upper bound on cache_seqlens; 0 = max_blocks_per_seq * page_size */
  void* workspace;                     /* fa_b200_decode_workspace_bytes() bytes, 16-byte aligned */
  size_t workspace_bytes;
  /* If set, the call stops before the final normalisation/cast and returns, per sequence and head,
   * the merged fp32 partial (o_partial_out (b, h, d), lse_partial_out (b, h)) for a cross-GPU
   * combine; out may then be NULL. */
  float* o_partial_out;
  float* lse_partial_out;
  /* Optional cudaEvent_t handles recorded right before and right after the partition kernel (a
   * separate combine kernel, when one is needed, runs after the stop event); NULL = off. */
  void* profile_start_event;
  void* profile_stop_event;
  /* Attention sinks: as in fa_b200_fwd_params (the reference's decode adds the sink in its first partition,
   * src/paged_attention.cu:333-335, 391-393; here it enters where the partitions are merged).  With
   * o_partial_out set the sink is left to the caller's final fa_b200_combine. */
  const void* s_aux;
  int32_t s_aux_dtype;
  /* Sliding window: with has_window != 0 and window_left >= 0 the query token sees only the last window_left + 1
   * keys of its sequence (the reference's decode takes window_size_left the same way,
   * src/paged_attention_window.h:47-109). */
  int32_t has_window, window_left;
  /* V stored transposed, (num_blocks, h_k, d, page_size) with the tokens of a page contiguous (the reference's paged
   * layout 0 / "custom", flash_attn_interface.py:2223-2227; K is then (num_blocks, h_k, page_size, d), which the
   * K strides already express).  With v_transposed != 0, v_row_stride is the stride between consecutive d rows.
   * F16 / BF16 only, page_size a multiple of 64. */
  int32_t v_transposed;
  /* Several query tokens per sequence (speculative decoding, multi-token prediction): q and out are
   * (b, seqlen_q, h, d) with q_row_stride / o_row_stride between tokens, softmax_lse (b, h, seqlen_q); the tokens are the
   * last seqlen_q positions of their sequence (cache_seqlens counts them) and with is_causal each sees the keys up to its
   * own position.  seqlen_q * (h / h_k) must fit the 16 rows of the kernel's tile (the reference sends this case to its
   * decode kernel under the same kind of bound, flash_attn_interface.py:2256).  0 or 1 = one token. */
  int32_t seqlen_q, is_causal;
  int64_t q_row_stride, o_row_stride;
  /* "fp8 KV cache": with kv_e4m3 != 0 the caches are E4M3 while q (and out) are of `dtype` F16 / BF16 (the reference's
   * paged_attention with kv_cache_dtype = "fp8" and k_scale / v_scale, flash_api.cpp:2496-2515).  k_descale / v_descale
   * carry the cache scales; q_descale is not used.  Not with v_transposed. */
  int32_t kv_e4m3;
  /* With kv_e4m3 != 0 and kv_e5m2 != 0 the cache bytes are E5M2 instead (kv_cache_dtype = "fp8_e5m2",
   * src/paged_attention.cu:747-1149 takes both fp8 formats): an e5m2 value is the high byte of an f16, so the
   * conversion on the way into the products is a byte move. */
  int32_t kv_e5m2;
  /* Split-KV merge inside the decode kernel.  When a call is split into partitions and its grid is small (at most two
   * rounds of the GPU's resident CTAs: that is where a saved launch counts; in larger grids the second launch is the
   * cheaper way and is used whatever this field holds), the CTA that finishes last for a (sequence, kv head) merges
   * that pair's partials itself, so the call is one launch.  The CTAs count themselves on one int32 per pair.  NULL = the library's own counters, one block per (device, stream) for up to 64 streams with
   * launches in flight and 4096 pairs per launch; beyond that (or with more than 256 partitions per sequence), and on a
   * stream that is being captured into a CUDA graph, the call falls back to a second launch (the LSE-combine kernel).
   * A caller that wants the single launch under capture, or more pairs, passes b * h_k int32 of its own here: zero
   * before the first use (the kernel leaves them zero), not shared by launches that can overlap on the GPU. */
  int32_t* tickets;
} fa_b200_decode_params;

/* Replaces mha_fwd_kvcache -> paged_attention(layout=2) -> paged_attention_kernel (+ combine)
 * (csrc/flash_attn_cutlass/flash_api.cpp:2530-2577; src/paged_attention.cu:747-1149, 61-558;
 *  src/paged_attention.h:356-445). */
FA_B200_API int fa_b200_decode_paged(const fa_b200_decode_params* p, void* stream);

/*
 * fa_b200_decode_paged for callers that have no way to hand over scratch memory: a plugin that runs inside
 * someone else's memory plan (an inference server that forbids allocation after start-up, a runtime whose
 * allocator is not reachable from the extension) cannot
 * call cudaMalloc and may not own a buffer to pass as `workspace`.  This variant takes the same parameters,
 * ignores `workspace` / `workspace_bytes`, and keeps the split-KV partials in a fixed array that lives inside
 * the library image: FA_B200_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the process
 * exits.  It has no counterpart in the reference, whose decode always allocates or caches a workspace.
 *
 *  - Sizes whose partials need more than FA_B200_STATIC_SCRATCH_BYTES
 *    (= fa_b200_decode_workspace_bytes(p)) are refused with FA_B200_ERR_TOO_LARGE; nothing is launched.
 *  - The first call on each device looks up the array's device address (one cudaGetSymbolAddress with that
 *    device current).  Make that first call outside any stream capture.
 *  - It calls no allocating routine: no cudaMalloc / cudaFree, nothing from an allocating library.
 *  - All calls on a device share the one array, and it keeps whatever the previous call left there (every
 *    slot a call reads is written by that call first, so nothing needs clearing).  Two calls whose kernels can
 *    overlap on the GPU (different streams, no ordering between them) race on it: serialise them.
 *  - If fa_b200_device_status() reports FA_B200_ERR_DEVICE_TIMEOUT after a call, throw that call's output away: a
 *    CTA that gave up on a wait wrote no partial, so the merge read what an earlier call had left in its slot, and
 *    the result can look plausible while being wrong.
 */
#define FA_B200_STATIC_SCRATCH_BYTES (32u << 20)
FA_B200_API int fa_b200_decode_paged_static(const fa_b200_decode_params* p, void* stream);

/* Bytes of scratch fa_b200_decode_paged needs for these sizes (0 when no split is used).
 * Replaces the per-(device, stream) workspace cache of src/paged_attention.cu:712-745. */
FA_B200_API size_t fa_b200_decode_workspace_bytes(const fa_b200_decode_params* p);

/* The partition size (tokens) the heuristic picks for these sizes. */
FA_B200_API int32_t fa_b200_decode_partition_tokens(const fa_b200_decode_params* p);

/*
 * LSE-combine of split-KV partials: o_partial (num_parts, rows, d) fp32 (each normalised by its own
 * partition), lse_partial (num_parts, rows) fp32 natural log (-inf / +inf = empty partition).
 * rows = b * h.  If parts_per_row is non-NULL (int32 (b)), row r uses only its first
 * parts_per_row[r / h] partitions.  Writes out (rows, d) in out_dtype (or fp32 when out_dtype < 0)
 * and lse (rows) fp32 (either may be NULL).
 * Replaces paged_attention_combine (src/paged_attention.h:356-445) and
 * flash_fwd_splitkv_reduce_varlen_kernel (csrc/flash_attn_hipc/src/flash_fwd_reduce.h:313-464).
 */
typedef struct fa_b200_combine_params {
  uint32_t struct_size;                /* sizeof(fa_b200_combine_params) */
  const float* o_partial;
  const float* lse_partial;
  void* out;
  float* lse;
  int64_t out_row_stride;              /* elements between consecutive rows of out */
  int32_t num_parts, rows, d, h;
  const int32_t* parts_per_row;
  int32_t out_dtype;
  float out_scale;                     /* multiplies out (v_descale); 1.0 normally */
  const void* s_aux;                   /* optional attention sinks, (h) elements of s_aux_dtype: one more term of the sum */
  int32_t s_aux_dtype;
  /* Floats between consecutive partitions of o_partial / lse_partial; 0 = packed (rows * d and rows).  Lets partials
   * that were gathered as one buffer per rank ([O | LSE] back to back) be combined in place; multiples of 4. */
  int64_t o_part_stride, lse_part_stride;
} fa_b200_combine_params;

FA_B200_API int fa_b200_combine(const fa_b200_combine_params* p, void* stream);

/*
 * Split-KV across GPUs without a collective library: exchange of the ranks' partial results over peer memory, fused
 * with their combine.  The reference has no multi-GPU path; this replaces the all-gather + fa_b200_combine pair a caller
 * would otherwise put after the per-rank decode (fa_b200_decode_params.o_partial_out).
 *
 * Set-up, once per process and problem shape (these calls allocate and synchronise; they are not for the hot path):
 *   fa_b200_exchange_bytes(world, rows, d)        size of a rank's exchange buffer (rows = b * h * seqlen_q)
 *   fa_b200_exchange_alloc(bytes, &buf, handle)   cudaMalloc + zero fill on the current device, and a 64-byte CUDA IPC
 *                                                 handle of the buffer to hand to the other ranks' processes
 *   fa_b200_exchange_open(handle, &peer)          maps another PROCESS's buffer on the current device (peer access is
 *                                                 enabled as needed); a rank uses its own `buf` for itself
 *   fa_b200_exchange_close(peer) / fa_b200_exchange_free(buf)
 * Per step, on every rank, after the decode that produced (o_local, lse_local):
 *   fa_b200_exchange_combine: one launch, one CTA per row.  It stores the row's partial into slot `rank` of every
 *   rank's buffer, publishes it with a system-scope release of the row's flag, waits until all slots of its own buffer
 *   carry the call's epoch, and writes the combined row (same arithmetic as fa_b200_combine, sinks included).
 *   `epoch` starts at 1 and grows by one per call, the same value on every rank; the buffer is double and calls
 *   alternate between its halves.  The wait is bounded: a rank whose peers never arrive returns, leaves `out` untouched
 *   and reports FA_B200_ERR_DEVICE_TIMEOUT through fa_b200_device_status().  world <= 16, d a multiple of 4.
 *   The kernels of the ranks wait for one another: run one rank per GPU, never two ranks' launches on one GPU.
 *   do_push / do_wait (both 1 in normal use) run the two halves of the kernel separately, for tests on one GPU.
 */
#define FA_B200_IPC_HANDLE_BYTES 64
#define FA_B200_MAX_EXCHANGE_RANKS 16
typedef struct fa_b200_exchange_params {
  uint32_t struct_size;                /* sizeof(fa_b200_exchange_params) */
  int32_t world, rank;
  int32_t rows, h, seqlen_q, d;        /* rows = b * h * seqlen_q, ordered (b, h, token) */
  const float* o_local;                /* (rows, d) fp32: this rank's partial */
  const float* lse_local;              /* (rows) fp32, natural log; +-inf = no keys on this rank */
  void* peers[FA_B200_MAX_EXCHANGE_RANKS];   /* exchange buffers of ranks 0 .. world-1 as mapped on this GPU */
  uint32_t epoch;
  int32_t do_push, do_wait;
  void* out;                           /* element offset of row (b, h, t): b*out_batch_stride + h*out_head_stride + t*out_tok_stride */
  float* lse;                          /* optional (rows) */
  int64_t out_batch_stride, out_head_stride, out_tok_stride;
  int32_t out_dtype;                   /* FA_B200_F16 / FA_B200_BF16, or -1 for fp32 */
  const void* s_aux;                   /* optional attention sinks (h) */
  int32_t s_aux_dtype;
} fa_b200_exchange_params;
FA_B200_API size_t fa_b200_exchange_bytes(int32_t world, int32_t rows, int32_t d);
FA_B200_API int fa_b200_exchange_alloc(size_t bytes, void** buf, void* ipc_handle_out);
FA_B200_API int fa_b200_exchange_open(const void* ipc_handle, void** peer);
FA_B200_API int fa_b200_exchange_close(void* peer);
FA_B200_API int fa_b200_exchange_free(void* buf);
FA_B200_API int fa_b200_exchange_combine(const fa_b200_exchange_params* p, void* stream);

/*
 * Raw-pointer paged attention over a whole batch of requests, with the argument list of the reference's
 * extern "C" kv_cache_attention(q, seq_offsets, max_seqlen_q, max_seqlen_k, k_caches, v_caches, page_tables, cache_lens,
 * out, num_query, num_tokens, num_q_head, num_kv_head, num_dim, num_pages, page_size, dtype, layout)
 * (csrc/flash_attn_cutlass/flash_api.cpp:2589-2624; cal_paged_attention, :2625-2631, is the same call with layout 1).
 * Differences forced by a C ABI that never allocates: the element type is an enum (the reference takes a std::string,
 * "fp16" or anything else for bf16), and the scratch memory and the stream are arguments.
 *
 *   q, out        (num_tokens, num_q_head, num_dim), packed
 *   seq_offsets   int32 (num_query + 1): first token of each request in q
 *   k_caches / v_caches   layout 1: (num_pages, num_kv_head, page_size, num_dim)
 *                         layout 2: (num_pages, page_size, num_kv_head, num_dim)
 *                         layout 0: K as layout 1, V (num_pages, num_kv_head, num_dim, page_size)
 *   page_tables   int32 (num_query, (max_seqlen_k - 1) / page_size + 1)
 *   cache_lens    int32 (num_query): keys of each request, the new tokens included
 *
 * num_query == num_tokens: one query token per request, every key visible (the reference's paged_attention branch).
 * Otherwise: each request's tokens are the last ones of its sequence and attend causally (bottom-right aligned) to its
 * pages (the reference's hg_prefix_prefill_varlen_fwd branch, which takes layouts 1 and 2).  softmax scale = 1 / sqrt(num_dim).
 * workspace: fa_b200_kv_cache_attention_workspace_bytes(num_query, num_q_head, num_kv_head, num_dim, page_size,
 * max_seqlen_k)
 * bytes, 16-byte aligned
 * (only the one-token branch uses it).
 */
FA_B200_API int fa_b200_kv_cache_attention(const void* q, const int32_t* seq_offsets, int32_t max_seqlen_q,
                                           int32_t max_seqlen_k, const void* k_caches, const void* v_caches,
                                           const int32_t* page_tables, const int32_t* cache_lens, void* out,
                                           int32_t num_query, int32_t num_tokens, int32_t num_q_head,
                                           int32_t num_kv_head, int32_t num_dim, int32_t num_pages, int32_t page_size,
                                           int32_t dtype, int32_t layout, void* workspace, size_t workspace_bytes,
                                           void* stream);
FA_B200_API size_t fa_b200_kv_cache_attention_workspace_bytes(int32_t num_query, int32_t num_q_head,
                                                              int32_t num_kv_head, int32_t num_dim, int32_t page_size,
                                                              int32_t max_seqlen_k);

/*
 * KV-cache append with optional rotary embedding, the first half of a decode call that is handed new keys and
 * values: flash_attn_with_kvcache(q, k_cache, v_cache, k=, v=, rotary_cos=, rotary_sin=, cache_seqlens=,
 * block_table=, rotary_interleaved=) (public signature flash_attn/flash_attn_interface.py:2478-2502, semantics
 * in its docstring :2503-2520 and in the test oracle tests/test_flash_attn.py:3073-3122; the reference's
 * mha_fwd_kvcache, csrc/flash_attn_cutlass/flash_api.cpp:2530-2577, accepts these arguments).
 *
 *   for each sequence b and new token s < seqlen_new:  pos = seqlens_k[b] + s
 *     k_cache[page(b, pos)][pos % page_size] = rotary(k_new[b, s], cos[pos], sin[pos])
 *     v_cache[page(b, pos)][pos % page_size] = v_new[b, s]
 *   q_out[b, s] = rotary(q[b, s], cos[p], sin[p]),  p = seqlens_k[b] + s if rotate_q_per_token (causal or
 *     local attention) else seqlens_k[b]
 *   seqlens_out[b] = seqlens_k[b] + seqlen_new          (the lengths the attention that follows must use)
 *
 * rotary(x): the first rotary_dim elements of a head are rotated pairwise, (x[2i], x[2i+1]) if
 * is_rotary_interleaved else (x[i], x[i + rotary_dim/2]):  o0 = x0 cos_i - x1 sin_i, o1 = x0 sin_i + x1 cos_i,
 * in fp32 from the 16-bit inputs with one rounding to the element type (as flash_attn/ops/triton/rotary.py:69-90);
 * the other elements are copied.  rotary_dim = 0 appends without rotation (q_out is then not written).
 * E4M3 caches take the append only (rotary_dim must be 0).
 * A position beyond max_blocks_per_seq * page_size, a page id outside [0, num_blocks) or a rotary row beyond
 * seqlen_ro is skipped and reported by fa_b200_device_status() as FA_B200_ERR_DEVICE_RANGE.
 * seqlens_out must not alias seqlens_k.  One kernel launch; nothing is allocated.
 */
typedef struct fa_b200_kv_append_params {
  uint32_t struct_size;                /* sizeof(fa_b200_kv_append_params) */
  const void* k_new;                   /* (b, seqlen_new, h_k, d) */
  const void* v_new;
  int64_t k_new_batch_stride, k_new_row_stride, k_new_head_stride;   /* elements */
  int64_t v_new_batch_stride, v_new_row_stride, v_new_head_stride;
  void* k_cache;                       /* (num_blocks, page_size, h_k, d), written in place */
  void* v_cache;
  int64_t k_block_stride, k_row_stride, k_head_stride;
  int64_t v_block_stride, v_row_stride, v_head_stride;
  const int32_t* block_table;          /* (b, max_blocks_per_seq) */
  int64_t block_table_batch_stride;
  const int32_t* seqlens_k;            /* (b) lengths before the append */
  int32_t* seqlens_out;                /* (b) lengths after the append; may be NULL */
  const void* q;                       /* (b, seqlen_q, h, d); read only when rotary_dim > 0 */
  void* q_out;                         /* (b, seqlen_q, h, d), same strides convention */
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t q_out_batch_stride, q_out_row_stride, q_out_head_stride;
  const void* rotary_cos;              /* (seqlen_ro, rotary_dim / 2), element type of q, rows contiguous */
  const void* rotary_sin;
  int32_t rotary_dim;                  /* 0 or a multiple of 16, <= d */
  int32_t seqlen_ro;
  int32_t is_rotary_interleaved;
  int32_t rotate_q_per_token;
  int32_t b, seqlen_q, seqlen_new, h, h_k, d;
  int32_t page_size, num_blocks, max_blocks_per_seq;
  int32_t dtype;                       /* FA_B200_F16 / BF16 / E4M3 (append only) */
} fa_b200_kv_append_params;

FA_B200_API int fa_b200_kv_append(const fa_b200_kv_append_params* p, void* stream);

/*
 * Callers' glue around the attention call (forward only).
 *
 * fa_b200_unpad_plan: from an attention mask (b, s) (element size 1, 4 or 8 bytes, nonzero = keep; mask_row_stride in
 * elements) the per-sequence lengths seqlens (b), cu_seqlens (b + 1), the flat indices row * s + column of the kept
 * tokens in order (indices, capacity b * s, int64) and stats = {max length, total kept}.  What unpad_input computes with
 * sum / nonzero / cumsum (flash_attn/bert_padding.py:98-122).  Three launches.
 * fa_b200_gather_rows: dst[r] = src[indices[r]] for r < n_rows (index_first_axis, bert_padding.py:8-37);
 * fa_b200_scatter_rows: dst[indices[r]] = src[r] (index_put_first_axis / pad_input, :40-67, :199-214; the caller zeroes
 * dst first).  Rows are row_bytes bytes, contiguous; indices outside [0, limit_rows) are skipped.
 * fa_b200_block_map_to_offset: a boolean tile map (rows, k) -> per row the ascending indices of its set entries times
 * `scale` (1 = block indices as flash_attn/utils/sparse_utils.py:526-566 returns them, 64 = the key-row offsets
 * fa_b200_fwd_sparse takes), padded with `fill` (the reference pads with 10000000), and their count.
 */
FA_B200_API int fa_b200_unpad_plan(const void* mask, int32_t mask_elem_size, int32_t b, int32_t s, int64_t mask_row_stride,
                                   int32_t* seqlens, int32_t* cu_seqlens, int64_t* indices, int32_t* stats, void* stream);
FA_B200_API int fa_b200_gather_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                                    int64_t limit_rows, void* stream);
FA_B200_API int fa_b200_scatter_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                                     int64_t limit_rows, void* stream);
FA_B200_API int fa_b200_block_map_to_offset(const uint8_t* block_map, int32_t* block_offset, int32_t* block_count,
                                            int64_t rows, int32_t k, int32_t scale, int32_t fill, void* stream);

/* Text for a status code. */
FA_B200_API const char* fa_b200_status_string(int status);
/* Last cudaError_t / CUresult text recorded by a failing call on this thread ("" if none). */
FA_B200_API const char* fa_b200_last_cuda_error(void);
/* Reads (with a device synchronise) and clears the device-side status word of the current device:
 * 0, FA_B200_ERR_DEVICE_TIMEOUT if a bounded wait inside a kernel gave up since the last call,
 * FA_B200_ERR_DEVICE_RANGE if fa_b200_kv_append skipped an out-of-range position, or
 * FA_B200_ERR_DEVICE_UNSUPPORTED if fa_b200_fwd_sparse met a non-zero column_count. */
FA_B200_API int fa_b200_device_status(void);
FA_B200_API int fa_b200_abi_version(void);
/* One line on stderr per attention call with the kernel, grid and tiling the library picked (what the reference prints
 * under FLASH_ATTENTION_PRINT_PARAM, csrc/flash_attn_cutlass/flash_api.cpp:219-222, and PA_PRINT_PARAM,
 * src/paged_attention.cu:40).  on = 1 / 0 switches it for the process; -1 goes back to the environment variable
 * FA_B200_PRINT_PARAM, which the library reads once when it is loaded.  fa_b200_last_launch_info() returns the line of
 * the calling thread's last attention call whether or not printing is on ("" before the first call). */
FA_B200_API void fa_b200_set_print_param(int on);
FA_B200_API const char* fa_b200_last_launch_info(void);
/* Measurement aid: one read-only pass over `bytes` bytes at `src` (16-byte aligned device memory) on `stream`, folded
 * into *sink (one uint32 in device memory).  Timed with events around it, it gives the bandwidth of a pure read
 * stream on this GPU, the yardstick for the decode kernels (a device-to-device copy, the usual figure, reads and
 * writes).  Not part of the attention path. */
FA_B200_API int fa_b200_read_stream(const void* src, int64_t bytes, uint32_t* sink, void* stream);
/* Number of kernels this library has launched in this process (for launch accounting). */
FA_B200_API uint64_t fa_b200_launch_count(void);

/*
 * Choice of the key tiles for fa_b200_fwd_sparse from the queries and keys themselves (the reference's
 * get_block_map_meansim, flash_attn/utils/sparse_utils.py:376-441), two launches:
 *
 * fa_b200_block_pool: x (b, h, n, d) F16 / BF16 (strides in elements, last dim contiguous, d = 64, 128 or 256) in blocks
 * of block_rows (<= 128) rows -> pooled (b, h, nb, d), the mean row of every block in the type of x, and sim (b, h, nb),
 * 1 where the mean cosine similarity over all pairs of rows of the block exceeds sim_threshold[head] (fp32 (h));
 * nb = ceil(n / block_rows); a block cut short by the end of the sequence is 0 (sparse_utils.py:281-299).
 *
 * fa_b200_block_select: block_map (b, h, nq, nk) uint8.  Per query block: softmax over the key blocks of
 * pooled_q . pooled_k * scale (key blocks with sim_k = 0 and, if is_causal, blocks that start at or after row
 * (qi + 1) * block_q: excluded), sorted descending; kept are the first #{cumulative sum <= cdf_threshold[head]} blocks
 * (or topk[head] * nk of them if topk is given; at least one), every key block with sim_k = 0, all of them where
 * sim_q = 0; then the causal mask again and, with attention_sink, key block 0.  fp32 arithmetic throughout.
 * nk <= 4096.  fa_b200_block_map_to_offset turns the map into the lists of fa_b200_fwd_sparse.
 */
FA_B200_API int fa_b200_block_pool(const void* x, int32_t dtype, int64_t batch_stride, int64_t head_stride,
                                   int64_t row_stride, int32_t b, int32_t h, int32_t n, int32_t d, int32_t block_rows,
                                   const float* sim_threshold, void* pooled, uint8_t* sim, void* stream);
FA_B200_API int fa_b200_block_select(const void* pooled_q, const void* pooled_k, const uint8_t* sim_q,
                                     const uint8_t* sim_k, int32_t dtype, int32_t b, int32_t h, int32_t nq, int32_t nk,
                                     int32_t d, int32_t block_q, int32_t block_k, float scale,
                                     const float* cdf_threshold, const float* topk, int32_t is_causal,
                                     int32_t attention_sink, uint8_t* block_map, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
