// LSE-combine of split-KV partials: one CTA of four warps per (sequence, head) row, each lane owns four of every
// 128 output columns (head dimension 128: one group of four; 256: two; 64: the first sixteen lanes).  Partials are fp32, normalised by their own partition's softmax sum, with a
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
// NV: groups of 128 columns (ceil(d / 128)).
template <int NV>
__global__ void __launch_bounds__(kCombineWarps * 32) combine_kernel(const CombineKernelParams p) {
  __shared__ float red_max[kCombineWarps], red_sum[kCombineWarps];
  __shared__ float4 red_acc[kCombineWarps][NV][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x;
  // launched with programmatic stream serialisation: the partials come from the kernel before this one
  griddep_wait();
  griddep_launch_dependents();
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

  // columns of this lane: 4 * lane + 128 * v, v < NV, those below d
  bool live[NV];
  float4 acc[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    live[v] = 4 * lane + 128 * v < p.d;
    acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (!empty) {
    const float4* op = reinterpret_cast<const float4*>(p.o_partial) + lane;
    const int64_t row_off = static_cast<int64_t>(row) * p.d;
    int i = warp;
    for (; i + 3 * kCombineWarps < nparts; i += 4 * kCombineWarps) {
      float l[4];
      float4 v[4][NV];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        l[j] = p.lse_partial[(i + j * kCombineWarps) * p.lse_part_stride + row];
#pragma unroll
        for (int g = 0; g < NV; ++g)
          if (live[g]) v[j][g] = op[((i + j * kCombineWarps) * p.o_part_stride + row_off) / 4 + 32 * g];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = (l[j] == INFINITY || l[j] == -INFINITY) ? 0.f : expf(l[j] - lse_tot);
        // a weight of exactly zero must not pick up NaN/Inf from an unused partial
        if (w != 0.f) {
#pragma unroll
          for (int g = 0; g < NV; ++g)
            if (live[g]) { acc[g].x += w * v[j][g].x; acc[g].y += w * v[j][g].y; acc[g].z += w * v[j][g].z; acc[g].w += w * v[j][g].w; }
        }
      }
    }
    for (; i < nparts; i += kCombineWarps) {
      const float l = p.lse_partial[i * p.lse_part_stride + row];
      const float w = (l == INFINITY || l == -INFINITY) ? 0.f : expf(l - lse_tot);
      if (w != 0.f) {
#pragma unroll
        for (int g = 0; g < NV; ++g)
          if (live[g]) {
            const float4 v = op[(i * p.o_part_stride + row_off) / 4 + 32 * g];
            acc[g].x += w * v.x; acc[g].y += w * v.y; acc[g].z += w * v.z; acc[g].w += w * v.w;
          }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < NV; ++g) red_acc[warp][g][lane] = acc[g];
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int g = 0; g < NV; ++g) {
    // fixed summation order: the result does not depend on scheduling
    float4 a = red_acc[0][g][lane];
#pragma unroll
    for (int w = 1; w < kCombineWarps; ++w) {
      const float4 t = red_acc[w][g][lane];
      a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
    }
    a.x *= p.out_scale; a.y *= p.out_scale; a.z *= p.out_scale; a.w *= p.out_scale;
    if (p.out && live[g]) {
      const int64_t off = static_cast<int64_t>(bi) * p.out_batch_stride + static_cast<int64_t>(hi) * p.out_row_stride +
                          static_cast<int64_t>(ti) * p.out_tok_stride + lane * 4 + 128 * g;
      if (p.out_dtype == FA_B200_BF16) {
        __nv_bfloat162 x = __floats2bfloat162_rn(a.x, a.y), c = __floats2bfloat162_rn(a.z, a.w);
        uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&c));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = u;
      } else if (p.out_dtype == FA_B200_F16) {
        __half2 x = __floats2half2_rn(a.x, a.y), c = __floats2half2_rn(a.z, a.w);
        uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&c));
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + off) = u;
      } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off) = a;
      }
    }
  }
  if (p.lse && lane == 0) p.lse[row] = empty ? (p.lse_empty_is_neg ? -INFINITY : INFINITY) : lse_tot;
}

}  // namespace

cudaError_t launch_combine(const CombineKernelParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return cudaSuccess;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.rows);
  cfg.blockDim = dim3(kCombineWarps * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.dependent_launch ? 1 : 0;
  return p.d > 128 ? cudaLaunchKernelEx(&cfg, combine_kernel<2>, p) : cudaLaunchKernelEx(&cfg, combine_kernel<1>, p);
}

}  // namespace fa
