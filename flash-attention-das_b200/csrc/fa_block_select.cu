// Choice of the key tiles a block-sparse prefill keeps, from the queries and keys themselves ("mean similarity"
// selection): what the reference's get_block_map_meansim computes with two Triton kernels and a chain of torch ops
// (flash_attn/utils/sparse_utils.py:376-441; pooling and self-similarity :281-299; map fill :336-347).
//   1. pool_sim_kernel: per block of BS rows of x (b, h, n, d): the mean row (pooled) and whether the block is
//      self-similar: mean over all row pairs of the cosine similarity > simthreshd1[h].  The sum over pairs of
//      x^_i . x^_j (x^ = row / |row|, rounded to f16 as the reference does) equals |sum_i x^_i|^2, so one pass over
//      the rows suffices.  A block that is cut short by the end of the sequence, or holds a zero row, is "not similar"
//      (in the reference its padded rows divide 0 by 0 and the comparison with NaN is false).
//   2. block_select_kernel: per query block: scores of its pooled row against every pooled key block, masked (keys of
//      blocks that are not self-similar: -inf; causal), softmax, sort descending, cumulative sum; the first
//      num = #{cdf <= cdfthreshd[h]} (or topk[h] * nk) blocks of the sorted order are kept (at least one), plus every
//      key block that is not self-similar, plus everything if the query block is not self-similar; then the causal
//      mask again and, if asked, key block 0 (attention sink).
// All arithmetic of step 2 is fp32 (the reference's intermediate tensors are in the input's 16-bit type).
// HBM traffic: x once (step 1); step 2 reads nq * nk * d pooled values from L2.
#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {
namespace {

constexpr int kPoolThreads = 128;
constexpr int kSelectThreads = 256;
constexpr int kMaxKeyBlocks = 4096;   // sorted in shared memory: padded to a power of two

__device__ __forceinline__ float to_f32(uint16_t raw, int dt) {
  if (dt == FA_B200_BF16) return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  return __half2float(__ushort_as_half(raw));
}
__device__ __forceinline__ uint16_t from_f32(float v, int dt) {
  if (dt == FA_B200_BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  return __half_as_ushort(__float2half_rn(v));
}

// E elements of a row per lane (d = 32 * E).
template <int E>
__global__ void __launch_bounds__(kPoolThreads) pool_sim_kernel(const BlockPoolParams p) {
  __shared__ float sm_pool[kPoolThreads / 32][32 * E];
  __shared__ float sm_hat[kPoolThreads / 32][32 * E];
  __shared__ float sm_red[kPoolThreads / 32];
  __shared__ int sm_bad;
  const int nb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = nb * p.block_rows;
  const int rows = min(p.block_rows, p.n - row0);
  if (threadIdx.x == 0) sm_bad = 0;
  __syncthreads();
  const uint16_t* base = static_cast<const uint16_t*>(p.x) + static_cast<int64_t>(b) * p.batch_stride +
                         static_cast<int64_t>(h) * p.head_stride + lane * E;
  float pool[E], hat[E];
#pragma unroll
  for (int e = 0; e < E; ++e) pool[e] = hat[e] = 0.f;
  bool bad = false;
  for (int r = warp; r < rows; r += kPoolThreads / 32) {
    const uint16_t* src = base + static_cast<int64_t>(row0 + r) * p.row_stride;
    uint16_t raw[E];
    if constexpr (E == 8) *reinterpret_cast<uint4*>(raw) = __ldg(reinterpret_cast<const uint4*>(src));
    else if constexpr (E == 4) *reinterpret_cast<uint2*>(raw) = __ldg(reinterpret_cast<const uint2*>(src));
    else *reinterpret_cast<uint32_t*>(raw) = __ldg(reinterpret_cast<const uint32_t*>(src));
    float x[E], ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) { x[e] = to_f32(raw[e], p.dtype); ss += x[e] * x[e]; }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    const float norm = sqrtf(ss);
    bad |= !(norm > 0.f);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      pool[e] += x[e];
      hat[e] += __half2float(__float2half_rn(x[e] / norm));
    }
  }
  if (bad && lane == 0) sm_bad = 1;
#pragma unroll
  for (int e = 0; e < E; ++e) { sm_pool[warp][lane * E + e] = pool[e]; sm_hat[warp][lane * E + e] = hat[e]; }
  __syncthreads();
  const int d = 32 * E;
  float sq = 0.f;
  for (int c = threadIdx.x; c < d; c += kPoolThreads) {
    float ps = 0.f, hs = 0.f;
#pragma unroll
    for (int w = 0; w < kPoolThreads / 32; ++w) { ps += sm_pool[w][c]; hs += sm_hat[w][c]; }
    static_cast<uint16_t*>(p.pooled)[((static_cast<int64_t>(b) * p.h + h) * p.num_blocks + nb) * d + c] =
        from_f32(ps / static_cast<float>(rows), p.dtype);
    sq += hs * hs;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, s);
  if (lane == 0) sm_red[warp] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < kPoolThreads / 32; ++w) tot += sm_red[w];
    const float mean_sim = tot / (static_cast<float>(rows) * static_cast<float>(rows));
    const bool sim = rows == p.block_rows && !sm_bad && mean_sim > p.sim_threshold[h];
    p.sim[(static_cast<int64_t>(b) * p.h + h) * p.num_blocks + nb] = sim ? 1 : 0;
  }
}

// One CTA per query block.  Dynamic shared memory: float q[d], float key[np], int idx[np] (np = nk rounded up to a
// power of two).
__global__ void __launch_bounds__(kSelectThreads) block_select_kernel(const BlockSelectParams p) {
  extern __shared__ float sm_f[];
  __shared__ float sm_red[kSelectThreads / 32];
  __shared__ int sm_num;
  const int qi = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.d, nk = p.nk, np = p.nk_pow2;
  float* sm_q = sm_f;
  float* key = sm_f + d;
  int* idx = reinterpret_cast<int*>(key + np);
  const int64_t bh = static_cast<int64_t>(b) * p.h + h;
  const uint16_t* pq = static_cast<const uint16_t*>(p.pooled_q) + (bh * p.nq + qi) * d;
  const uint16_t* pk = static_cast<const uint16_t*>(p.pooled_k) + bh * nk * d;
  const uint8_t* simk = p.sim_k + bh * nk;
  for (int c = threadIdx.x; c < d; c += kSelectThreads) sm_q[c] = to_f32(pq[c], p.dtype);
  __syncthreads();
  // scores
  for (int j = warp; j < np; j += kSelectThreads / 32) {
    float s = -INFINITY;
    if (j < nk) {
      float acc = 0.f;
      for (int c = lane; c < d; c += 32) acc += sm_q[c] * to_f32(pk[static_cast<int64_t>(j) * d + c], p.dtype);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const bool causal_ok = !p.is_causal || static_cast<int64_t>(j) * p.block_k < static_cast<int64_t>(qi + 1) * p.block_q;
      s = (simk[j] && causal_ok) ? acc * p.scale : -INFINITY;
    }
    if (lane == 0) { key[j] = s; idx[j] = j; }
  }
  __syncthreads();
  // softmax over the nk scores
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < nk; j += kSelectThreads) mx = fmaxf(mx, key[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sm_red[warp] = mx;
  __syncthreads();
  mx = sm_red[0];
  for (int w = 1; w < kSelectThreads / 32; ++w) mx = fmaxf(mx, sm_red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < nk; j += kSelectThreads) {
    const float e = (mx == -INFINITY) ? 0.f : __expf(key[j] - mx);
    key[j] = e;
    sum += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) sm_red[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < kSelectThreads / 32; ++w) sum += sm_red[w];
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int j = threadIdx.x; j < np; j += kSelectThreads) key[j] = j < nk ? key[j] * inv : -1.f;   // padding sorts last
  __syncthreads();
  // bitonic sort, descending by probability, ties by ascending index
  for (int k2 = 2; k2 <= np; k2 <<= 1) {
    for (int j2 = k2 >> 1; j2 > 0; j2 >>= 1) {
      for (int i = threadIdx.x; i < np; i += kSelectThreads) {
        const int l = i ^ j2;
        if (l > i) {
          const float a = key[i], c = key[l];
          const int ia = idx[i], ic = idx[l];
          const bool a_first = a > c || (a == c && ia < ic);   // a belongs before c in the final order
          const bool up = (i & k2) == 0;
          if (up ? !a_first : a_first) { key[i] = c; key[l] = a; idx[i] = ic; idx[l] = ia; }
        }
      }
      __syncthreads();
    }
  }
  // number of blocks to keep
  if (warp == 0) {
    int num;
    if (p.topk) {
      num = static_cast<int>(p.topk[h] * static_cast<float>(nk));
    } else {
      // sequential fp32 prefix sums, lane by lane over contiguous chunks
      const float thr = p.cdf_threshold[h];
      const int chunk = (nk + 31) / 32;
      const int lo = min(lane * chunk, nk), hi = min(lo + chunk, nk);
      float part = 0.f;
      for (int i = lo; i < hi; ++i) part += key[i];
      float before = part;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, before, o);
        if (lane >= o) before += t;
      }
      before -= part;   // sum of the chunks before this lane's
      int cnt = 0;
      float run = before;
      for (int i = lo; i < hi; ++i) { run += key[i]; cnt += (run <= thr) ? 1 : 0; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
      num = cnt;
    }
    num = max(1, min(num, nk));
    if (lane == 0) sm_num = num;
  }
  __syncthreads();
  const int num = sm_num;
  // the map row: reuse key[] as flags
  const bool q_sim = p.sim_q[bh * p.nq + qi] != 0;
  for (int j = threadIdx.x; j < nk; j += kSelectThreads) key[j] = (!q_sim || !simk[j]) ? 1.f : 0.f;
  __syncthreads();
  for (int i = threadIdx.x; i < num; i += kSelectThreads) key[idx[i]] = 1.f;
  __syncthreads();
  uint8_t* out = p.block_map + (bh * p.nq + qi) * nk;
  for (int j = threadIdx.x; j < nk; j += kSelectThreads) {
    bool on = key[j] != 0.f;
    if (p.is_causal) on = on && static_cast<int64_t>(j) * p.block_k < static_cast<int64_t>(qi + 1) * p.block_q;
    if (p.attention_sink && j == 0) on = true;
    out[j] = on ? 1 : 0;
  }
}

}  // namespace

int block_select_max_key_blocks() { return kMaxKeyBlocks; }

cudaError_t launch_block_pool(const BlockPoolParams& p, cudaStream_t stream) {
  if (p.b <= 0 || p.h <= 0 || p.num_blocks <= 0) return cudaSuccess;
  dim3 grid(p.num_blocks, p.h, p.b);
  switch (p.d) {
    case 64: pool_sim_kernel<2><<<grid, kPoolThreads, 0, stream>>>(p); break;
    case 128: pool_sim_kernel<4><<<grid, kPoolThreads, 0, stream>>>(p); break;
    case 256: pool_sim_kernel<8><<<grid, kPoolThreads, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_block_select(const BlockSelectParams& p, cudaStream_t stream) {
  if (p.b <= 0 || p.h <= 0 || p.nq <= 0 || p.nk <= 0) return cudaSuccess;
  dim3 grid(p.nq, p.h, p.b);
  const size_t smem = sizeof(float) * p.d + (sizeof(float) + sizeof(int)) * p.nk_pow2;
  block_select_kernel<<<grid, kSelectThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fa
