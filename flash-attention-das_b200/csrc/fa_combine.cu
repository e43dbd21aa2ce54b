// LSE-combine of split-KV partials: one CTA of four warps per (sequence, head) row, each lane owns four of the
// 128 output columns.  Partials are fp32, normalised by their own partition's softmax sum, with a
// natural-log LSE (-inf or +inf marks a partition without keys).
//   M = max_i lse_i;  w_i = e^{lse_i - M};  O = sum_i w_i O_i / sum_i w_i;  LSE = M + ln sum_i w_i
// An attention sink (one logit per head) is one more term of the sum that carries no value.
// Same result as the reference's combine (csrc/flash_attn_cutlass/src/paged_attention.h:356-445) and
// its LSE-writing variant (csrc/flash_attn_hipc/src/flash_fwd_reduce.h:313-464).
#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {
namespace {

constexpr int kCombineWarps = 4;

// One CTA per (sequence, head) row.  The four warps share the partitions of the row (warp w takes partitions
// w, w + 4, ...), each lane owns four of the 128 output columns, and the warps' partial sums meet in shared memory,
// so a row with hundreds of partitions (one very long sequence) is not walked by a single warp.
__global__ void __launch_bounds__(kCombineWarps * 32) combine_kernel(const CombineKernelParams p) {
  __shared__ float red_max[kCombineWarps], red_sum[kCombineWarps];
  __shared__ float4 red_acc[kCombineWarps][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x;
  const int sq = p.sq > 0 ? p.sq : 1;
  const int bi = row / (p.h * sq), hi = (row / sq) % p.h, ti = row % sq;
  int nparts = p.num_parts;
  if (p.parts_per_row) nparts = min(nparts, p.parts_per_row[bi]);
  else if (p.seqlens) nparts = min(nparts, (p.seqlens[bi] + p.partition_tokens - 1) / p.partition_tokens);

  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nparts; i += kCombineWarps * 32) {
    float l = p.lse_partial[i * p.lse_part_stride + row];
    if (l == INFINITY) l = -INFINITY;
    mx = fmaxf(mx, l);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
  if (lane == 0) red_max[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red_max[0], red_max[1]), fmaxf(red_max[2], red_max[3]));
  float sum = 0.f;
  if (mx != -INFINITY) {
    for (int i = threadIdx.x; i < nparts; i += kCombineWarps * 32) {
      float l = p.lse_partial[i * p.lse_part_stride + row];
      if (l == INFINITY) l = -INFINITY;
      sum += expf(l - mx);
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  if (lane == 0) red_sum[warp] = sum;
  __syncthreads();
  sum = (red_sum[0] + red_sum[1]) + (red_sum[2] + red_sum[3]);
  if (p.s_aux) {   // the attention sink of this head: one more term e^sink of the row's sum
    const float sink = load_sink_log2(p.s_aux, p.s_aux_dtype, hi) * kLn2;
    const float m2 = fmaxf(mx, sink);
    sum = (mx == -INFINITY ? 0.f : sum * expf(mx - m2)) + expf(sink - m2);
    mx = m2;
  }
  const bool empty = !(sum > 0.f);
  const float lse_tot = empty ? 0.f : mx + logf(sum);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!empty) {
    const float4* op = reinterpret_cast<const float4*>(p.o_partial) + lane;
    int i = warp;
    for (; i + 3 * kCombineWarps < nparts; i += 4 * kCombineWarps) {
      float l[4];
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        l[j] = p.lse_partial[(i + j * kCombineWarps) * p.lse_part_stride + row];
        v[j] = op[((i + j * kCombineWarps) * p.o_part_stride + row * kHeadDim) / 4];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = (l[j] == INFINITY || l[j] == -INFINITY) ? 0.f : expf(l[j] - lse_tot);
        // a weight of exactly zero must not pick up NaN/Inf from an unused partial
        if (w != 0.f) { acc.x += w * v[j].x; acc.y += w * v[j].y; acc.z += w * v[j].z; acc.w += w * v[j].w; }
      }
    }
    for (; i < nparts; i += kCombineWarps) {
      const float l = p.lse_partial[i * p.lse_part_stride + row];
      const float4 v = op[(i * p.o_part_stride + row * kHeadDim) / 4];
      const float w = (l == INFINITY || l == -INFINITY) ? 0.f : expf(l - lse_tot);
      if (w != 0.f) { acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w; }
    }
  }
  red_acc[warp][lane] = acc;
  __syncthreads();
  if (warp != 0) return;
  // fixed summation order: the result does not depend on scheduling
  acc = red_acc[0][lane];
#pragma unroll
  for (int w = 1; w < kCombineWarps; ++w) {
    const float4 t = red_acc[w][lane];
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  acc.x *= p.out_scale; acc.y *= p.out_scale; acc.z *= p.out_scale; acc.w *= p.out_scale;
  if (p.out) {
    const int64_t off = static_cast<int64_t>(bi) * p.out_batch_stride + static_cast<int64_t>(hi) * p.out_row_stride +
                        static_cast<int64_t>(ti) * p.out_tok_stride + lane * 4;
    if (p.out_dtype == FA_B200_BF16) {
      __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), c = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = u;
    } else if (p.out_dtype == FA_B200_F16) {
      __half2 a = __floats2half2_rn(acc.x, acc.y), c = __floats2half2_rn(acc.z, acc.w);
      uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + off) = u;
    } else {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off) = acc;
    }
  }
  if (p.lse && lane == 0) p.lse[row] = empty ? (p.lse_empty_is_neg ? -INFINITY : INFINITY) : lse_tot;
}

}  // namespace

cudaError_t launch_combine(const CombineKernelParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return cudaSuccess;
  const int grid = p.rows;
  combine_kernel<<<grid, kCombineWarps * 32, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fa
