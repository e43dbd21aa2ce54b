// KV-cache append with optional rotary embedding: writes the new keys (rotated) and values of a decode or
// chunked-prefill step into the paged cache at positions seqlens_k[b] .. seqlens_k[b] + seqlen_new - 1, writes
// the rotated queries to a separate buffer, and the updated lengths.  One warp per (token, head) row of 128
// elements; each lane owns four consecutive elements (8 bytes of a 16-bit type, 4 bytes of e4m3).
//
// Semantics: the public decode signature (flash_attn/flash_attn_interface.py:2478-2520) and its test oracle
// (tests/test_flash_attn.py:3073-3122).  Arithmetic: fp32 from the 16-bit inputs, one rounding, in the order
// o0 = x0 cos - x1 sin, o1 = x0 sin + x1 cos (flash_attn/ops/triton/rotary.py:69-90); the products are kept
// separate from the sum (no fused multiply-add) so the result is bit-identical to the same expression
// evaluated in fp32 on a CPU.
//
// Bytes per launch: reads b*(seqlen_new*h_k*2 + seqlen_q*h)*128*elem + cos/sin rows, writes the same amount:
// a few hundred KB for a decode step, so the launch is latency-bound, not bandwidth-bound.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {
namespace {

constexpr int kAppendWarps = 8;
constexpr int kStatusRange = 0x10000;  // bit of the device status word: an out-of-range position was skipped

template <int DT>
__device__ __forceinline__ float4 load4(const void* base, int64_t off) {
  const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + off);
  float4 r;
  if (DT == FA_B200_BF16) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    r = make_float4(a.x, a.y, c.x, c.y);
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    r = make_float4(a.x, a.y, c.x, c.y);
  }
  return r;
}

template <int DT>
__device__ __forceinline__ float2 load2(const void* base, int64_t off) {
  const uint32_t u = *reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(base) + off);
  if (DT == FA_B200_BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}

template <int DT>
__device__ __forceinline__ void store4(void* base, int64_t off, float4 v) {
  uint2 u;
  if (DT == FA_B200_BF16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), c = __floats2bfloat162_rn(v.z, v.w);
    u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
  } else {
    __half2 a = __floats2half2_rn(v.x, v.y), c = __floats2half2_rn(v.z, v.w);
    u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
  }
  *reinterpret_cast<uint2*>(static_cast<uint16_t*>(base) + off) = u;
}

// a*b - c*d and a*b + c*d with every operation rounded on its own
__device__ __forceinline__ float mul_sub(float a, float b, float c, float d) {
  return __fsub_rn(__fmul_rn(a, b), __fmul_rn(c, d));
}
__device__ __forceinline__ float mul_add(float a, float b, float c, float d) {
  return __fadd_rn(__fmul_rn(a, b), __fmul_rn(c, d));
}

// Rotates the lane's four elements of one head row.  The whole warp must call this (it shuffles).
template <int DT>
__device__ __forceinline__ float4 rotate_row(float4 x, int lane, int pos, const KvAppendKernelParams& p) {
  const int half = p.rotary_dim >> 1;
  if (p.interleaved) {
    if (4 * lane < p.rotary_dim) {
      const int64_t ci = static_cast<int64_t>(pos) * half + 2 * lane;
      const float2 c = load2<DT>(p.cos, ci), s = load2<DT>(p.sin, ci);
      x = make_float4(mul_sub(x.x, c.x, x.y, s.x), mul_add(x.x, s.x, x.y, c.x),
                      mul_sub(x.z, c.y, x.w, s.y), mul_add(x.z, s.y, x.w, c.y));
    }
    return x;
  }
  const int lanes_half = half >> 2;  // lanes holding the first element of each pair
  const int partner = lane < lanes_half ? lane + lanes_half : (lane < 2 * lanes_half ? lane - lanes_half : lane);
  float4 y;
  y.x = __shfl_sync(0xffffffffu, x.x, partner);
  y.y = __shfl_sync(0xffffffffu, x.y, partner);
  y.z = __shfl_sync(0xffffffffu, x.z, partner);
  y.w = __shfl_sync(0xffffffffu, x.w, partner);
  if (lane < 2 * lanes_half) {
    const bool first = lane < lanes_half;
    const int64_t ci = static_cast<int64_t>(pos) * half + 4 * (first ? lane : lane - lanes_half);
    const float4 c = load4<DT>(p.cos, ci), s = load4<DT>(p.sin, ci);
    if (first) {  // x = x0, y = x1
      x = make_float4(mul_sub(x.x, c.x, y.x, s.x), mul_sub(x.y, c.y, y.y, s.y), mul_sub(x.z, c.z, y.z, s.z),
                      mul_sub(x.w, c.w, y.w, s.w));
    } else {      // x = x1, y = x0
      x = make_float4(mul_add(y.x, s.x, x.x, c.x), mul_add(y.y, s.y, x.y, c.y), mul_add(y.z, s.z, x.z, c.z),
                      mul_add(y.w, s.w, x.w, c.w));
    }
  }
  return x;
}

template <int DT>
__global__ void __launch_bounds__(kAppendWarps * 32) kv_append_kernel(const KvAppendKernelParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (blockIdx.x == 0 && p.seqlens_out) {
    for (int i = threadIdx.x; i < p.b; i += kAppendWarps * 32) p.seqlens_out[i] = p.seqlens_k[i] + p.seqlen_new;
  }
  const int64_t kv_rows = static_cast<int64_t>(p.b) * p.seqlen_new * p.h_k;
  const int64_t q_rows = p.rotary_dim > 0 ? static_cast<int64_t>(p.b) * p.seqlen_q * p.h : 0;
  const int64_t total = 2 * kv_rows + q_rows;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kAppendWarps + warp; row < total;
       row += static_cast<int64_t>(gridDim.x) * kAppendWarps) {
    if (row < 2 * kv_rows) {
      const bool is_v = row >= kv_rows;
      const int64_t r = is_v ? row - kv_rows : row;
      const int hk = static_cast<int>(r % p.h_k);
      const int s = static_cast<int>((r / p.h_k) % p.seqlen_new);
      const int bi = static_cast<int>(r / (static_cast<int64_t>(p.h_k) * p.seqlen_new));
      const int pos = p.seqlens_k[bi] + s;
      const int slot = pos / p.page_size;
      bool ok = pos >= 0 && slot < p.max_blocks_per_seq;
      int page = 0;
      if (ok) {
        page = p.block_table[static_cast<int64_t>(bi) * p.bt_stride + slot];
        ok = page >= 0 && page < p.num_blocks;
      }
      const bool rot = !is_v && p.rotary_dim > 0;
      if (rot && pos >= p.seqlen_ro) ok = false;
      if (!ok) {
        if (lane == 0) atomicOr(p.status, kStatusRange);
        continue;
      }
      const int in_page = pos - slot * p.page_size;
      const int64_t src = is_v ? static_cast<int64_t>(bi) * p.vn_b + static_cast<int64_t>(s) * p.vn_r + static_cast<int64_t>(hk) * p.vn_h
                               : static_cast<int64_t>(bi) * p.kn_b + static_cast<int64_t>(s) * p.kn_r + static_cast<int64_t>(hk) * p.kn_h;
      const int64_t dst = is_v ? static_cast<int64_t>(page) * p.vc_blk + static_cast<int64_t>(in_page) * p.vc_row + static_cast<int64_t>(hk) * p.vc_h
                               : static_cast<int64_t>(page) * p.kc_blk + static_cast<int64_t>(in_page) * p.kc_row + static_cast<int64_t>(hk) * p.kc_h;
      if (DT == FA_B200_E4M3) {
        const uint32_t u = *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(is_v ? p.v_new : p.k_new) + src + 4 * lane);
        *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(is_v ? p.v_cache : p.k_cache) + dst + 4 * lane) = u;
      } else {
        constexpr int D16 = DT == FA_B200_E4M3 ? FA_B200_BF16 : DT;
        float4 x = load4<D16>(is_v ? p.v_new : p.k_new, src + 4 * lane);
        if (rot) x = rotate_row<D16>(x, lane, pos, p);
        store4<D16>(is_v ? p.v_cache : p.k_cache, dst + 4 * lane, x);
      }
    } else if (DT != FA_B200_E4M3) {
      constexpr int D16 = DT == FA_B200_E4M3 ? FA_B200_BF16 : DT;
      const int64_t r = row - 2 * kv_rows;
      const int hi = static_cast<int>(r % p.h);
      const int s = static_cast<int>((r / p.h) % p.seqlen_q);
      const int bi = static_cast<int>(r / (static_cast<int64_t>(p.h) * p.seqlen_q));
      const int pos = p.seqlens_k[bi] + (p.q_per_token ? s : 0);
      float4 x = load4<D16>(p.q, static_cast<int64_t>(bi) * p.q_b + static_cast<int64_t>(s) * p.q_r + static_cast<int64_t>(hi) * p.q_h + 4 * lane);
      if (pos >= 0 && pos < p.seqlen_ro) x = rotate_row<D16>(x, lane, pos, p);
      else if (lane == 0) atomicOr(p.status, kStatusRange);
      store4<D16>(p.q_out, static_cast<int64_t>(bi) * p.qo_b + static_cast<int64_t>(s) * p.qo_r + static_cast<int64_t>(hi) * p.qo_h + 4 * lane, x);
    }
  }
}

}  // namespace

cudaError_t launch_kv_append(int dtype, const KvAppendKernelParams& p, cudaStream_t stream) {
  const int64_t rows = 2ll * p.b * p.seqlen_new * p.h_k + (p.rotary_dim > 0 ? static_cast<int64_t>(p.b) * p.seqlen_q * p.h : 0);
  int64_t blocks = (rows + kAppendWarps - 1) / kAppendWarps;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int grid = static_cast<int>(blocks);
  if (dtype == FA_B200_BF16) kv_append_kernel<FA_B200_BF16><<<grid, kAppendWarps * 32, 0, stream>>>(p);
  else if (dtype == FA_B200_F16) kv_append_kernel<FA_B200_F16><<<grid, kAppendWarps * 32, 0, stream>>>(p);
  else kv_append_kernel<FA_B200_E4M3><<<grid, kAppendWarps * 32, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fa
