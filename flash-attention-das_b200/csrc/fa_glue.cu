// Callers' glue on either side of the attention call, as HBM-bound integer / byte kernels:
//   * padding removal: attention mask (batch, seqlen) -> per-sequence lengths, cu_seqlens, the flat indices of the kept
//     tokens, and row gather / scatter between the padded (batch * seqlen, ...) and packed (total, ...) layouts
//     (flash_attn/bert_padding.py:98-122 unpad_input, :199-214 pad_input, :8-67 index_first_axis / index_put_first_axis);
//   * block map -> block lists: boolean (rows, k) tile map -> ascending offsets of the selected tiles + their count
//     (flash_attn/utils/sparse_utils.py:526-566 block_map_to_block_offset, Triton version :78-105).
// Bytes per launch: the mask / map once, the index list once, and for the row moves 2 * rows * row_bytes.
#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {
namespace {

constexpr int kScanThreads = 256;

__device__ __forceinline__ bool mask_at(const void* mask, int elem, int64_t i) {
  if (elem == 1) return static_cast<const uint8_t*>(mask)[i] != 0;
  if (elem == 4) return static_cast<const int32_t*>(mask)[i] != 0;
  return static_cast<const int64_t*>(mask)[i] != 0;
}

// Block-wide exclusive prefix of one int per thread; returns the thread's prefix and the block total.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, s);
    if (lane >= s) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, s);
      if (lane >= s) w += t;
    }
    warp_sums[lane] = w;   // inclusive sums of the warps
  }
  __syncthreads();
  total = warp_sums[(blockDim.x >> 5) - 1];
  const int base = warp > 0 ? warp_sums[warp - 1] : 0;
  __syncthreads();
  return base + inc - v;
}

// One CTA per sequence: number of kept tokens.
__global__ void __launch_bounds__(kScanThreads) mask_count_kernel(const void* mask, int elem, int64_t row_stride, int s,
                                                                  int32_t* seqlens) {
  __shared__ int warp_sums[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * row_stride;
  int c = 0;
  for (int i = threadIdx.x; i < s; i += blockDim.x) c += mask_at(mask, elem, base + i) ? 1 : 0;
  int total;
  block_exclusive_scan(c, warp_sums, total);
  if (threadIdx.x == 0) seqlens[blockIdx.x] = total;
}

// One CTA: cu_seqlens = exclusive prefix of seqlens (b + 1 entries), stats = {max, total}.
__global__ void __launch_bounds__(kScanThreads) seqlens_scan_kernel(const int32_t* seqlens, int b, int32_t* cu_seqlens,
                                                                    int32_t* stats) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  int mx = 0;
  for (int base = 0; base < b; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int v = i < b ? seqlens[i] : 0;
    mx = max(mx, v);
    int total;
    const int ex = block_exclusive_scan(v, warp_sums, total);
    const int carry = carry_s;
    if (i < b) cu_seqlens[i] = carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + total;
    __syncthreads();
  }
  // block max
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    int m = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) m = max(m, warp_sums[w]);
    cu_seqlens[b] = carry_s;
    stats[0] = m;
    stats[1] = carry_s;
  }
}

// One CTA per sequence: flat indices (row * s + column) of its kept tokens, in order, at cu_seqlens[row].
__global__ void __launch_bounds__(kScanThreads) mask_compact_kernel(const void* mask, int elem, int64_t row_stride, int s,
                                                                    const int32_t* cu_seqlens, int64_t* indices) {
  __shared__ int warp_sums[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * row_stride;
  int64_t out = cu_seqlens[blockIdx.x];
  for (int c0 = 0; c0 < s; c0 += blockDim.x) {
    const int i = c0 + threadIdx.x;
    const int keep = (i < s && mask_at(mask, elem, base + i)) ? 1 : 0;
    int total;
    const int ex = block_exclusive_scan(keep, warp_sums, total);
    if (keep) indices[out + ex] = static_cast<int64_t>(blockIdx.x) * s + i;
    out += total;
  }
}

// Row moves: VEC-byte pieces, consecutive threads on consecutive pieces of a row.
template <typename V, bool kScatter>
__global__ void __launch_bounds__(256) move_rows_kernel(const uint8_t* src, const int64_t* indices, uint8_t* dst, int64_t n_rows,
                                                        int64_t row_bytes, int64_t limit_rows) {
  const int64_t per_row = row_bytes / static_cast<int64_t>(sizeof(V));
  const int64_t total = n_rows * per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / per_row, c = i - r * per_row;
    const int64_t other = indices[r];
    if (other < 0 || other >= limit_rows) continue;   // an index outside the other tensor is skipped
    const int64_t s_off = (kScatter ? r : other) * row_bytes, d_off = (kScatter ? other : r) * row_bytes;
    reinterpret_cast<V*>(dst + d_off)[c] = reinterpret_cast<const V*>(src + s_off)[c];
  }
}

// One warp per row of the tile map.
__global__ void __launch_bounds__(256) block_map_kernel(const uint8_t* map, int32_t* offset, int32_t* count, int64_t rows, int k,
                                                        int scale, int fill) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint8_t* m = map + row * k;
  int32_t* o = offset + row * k;
  int n = 0;
  for (int c0 = 0; c0 < k; c0 += 32) {
    const int i = c0 + lane;
    const bool on = i < k && m[i] != 0;
    const unsigned bal = __ballot_sync(0xffffffffu, on);
    if (on) o[n + __popc(bal & ((1u << lane) - 1u))] = i * scale;
    n += __popc(bal);
  }
  for (int i = n + lane; i < k; i += 32) o[i] = fill;
  if (lane == 0) count[row] = n;
}

int grid_for(int64_t work, int threads) {
  int64_t g = (work + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return static_cast<int>(g);
}

// Read-only stream over a buffer: every thread folds 16-byte loads into one word, one word per CTA leaves the SM.
// The yardstick for the decode kernels, which read their KV bytes once and write next to nothing (a device-to-device
// copy, the usual bandwidth figure, reads AND writes and turns the bus around).
__global__ void __launch_bounds__(256) read_stream_kernel(const uint4* __restrict__ src, int64_t n16, uint32_t* sink) {
  uint32_t acc = 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {   // four independent loads in flight per thread
    uint4 a, b, c, d;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src + i));
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + i + stride));
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(c.x), "=r"(c.y), "=r"(c.z), "=r"(c.w) : "l"(src + i + 2 * stride));
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w) : "l"(src + i + 3 * stride));
    acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
  }
  for (; i < n16; i += stride) {
    const uint4 a = src[i];
    acc ^= a.x ^ a.y ^ a.z ^ a.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc ^= __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0 && acc == 0x9e3779b9u) atomicXor(sink, acc);   // keeps the loads alive; almost never taken
}

}  // namespace

cudaError_t launch_read_stream(const void* src, int64_t bytes, uint32_t* sink, cudaStream_t stream) {
  const int64_t n16 = bytes / 16;
  if (n16 <= 0) return cudaSuccess;
  read_stream_kernel<<<148 * 8, 256, 0, stream>>>(static_cast<const uint4*>(src), n16, sink);
  return cudaGetLastError();
}

cudaError_t launch_unpad_plan(const void* mask, int elem, int b, int s, int64_t row_stride, int32_t* seqlens,
                              int32_t* cu_seqlens, int64_t* indices, int32_t* stats, cudaStream_t stream) {
  mask_count_kernel<<<b, kScanThreads, 0, stream>>>(mask, elem, row_stride, s, seqlens);
  seqlens_scan_kernel<<<1, kScanThreads, 0, stream>>>(seqlens, b, cu_seqlens, stats);
  mask_compact_kernel<<<b, kScanThreads, 0, stream>>>(mask, elem, row_stride, s, cu_seqlens, indices);
  return cudaGetLastError();
}

cudaError_t launch_move_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                             int64_t limit_rows, bool scatter, cudaStream_t stream) {
  if (n_rows <= 0 || row_bytes <= 0) return cudaSuccess;
  const uintptr_t align = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(row_bytes);
  const uint8_t* s8 = static_cast<const uint8_t*>(src);
  uint8_t* d8 = static_cast<uint8_t*>(dst);
#define FA_MOVE(V)                                                                                                     \
  do {                                                                                                                 \
    const int g = grid_for(n_rows * (row_bytes / static_cast<int64_t>(sizeof(V))), 256);                               \
    if (scatter) move_rows_kernel<V, true><<<g, 256, 0, stream>>>(s8, indices, d8, n_rows, row_bytes, limit_rows);      \
    else move_rows_kernel<V, false><<<g, 256, 0, stream>>>(s8, indices, d8, n_rows, row_bytes, limit_rows);             \
  } while (0)
  if ((align & 15) == 0) FA_MOVE(uint4);
  else if ((align & 7) == 0) FA_MOVE(uint2);
  else if ((align & 3) == 0) FA_MOVE(uint32_t);
  else if ((align & 1) == 0) FA_MOVE(uint16_t);
  else FA_MOVE(uint8_t);
#undef FA_MOVE
  return cudaGetLastError();
}

cudaError_t launch_block_map(const uint8_t* map, int32_t* offset, int32_t* count, int64_t rows, int k, int scale, int fill,
                             cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  const int64_t blocks = (rows + 7) / 8;
  block_map_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(map, offset, count, rows, k, scale, fill);
  return cudaGetLastError();
}

}  // namespace fa
