// Building blocks of the paged-decode kernel (fa_decode.cu): tile traits, the producer's tile loads, the query
// fragments, one K/V tile's worth of S = Q K^T, online softmax and O += P V for one consumer warp, and the merge of
// split-KV partials.
//
// Data flow as in the reference's partitioned paged attention (csrc/flash_attn_cutlass/src/paged_attention.cu:61-558),
// with exact softmax (no epsilon) and fp32 partials, as the reference's PyTorch oracle defines the result.
#pragma once

#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {

constexpr int kConsumerWarps = 4;
constexpr int kDecodeThreads = 32 * (1 + kConsumerWarps);
constexpr int kMaxPagesPerPartition = 512;

// HD: head dimension, 128 for every element type and 64 / 192 / 256 for the 16-bit ones.
template <int DT, int HD = 128>
struct DecodeTraits {
  static constexpr bool kFp8 = (DT == FA_B200_E4M3);
  static constexpr int kElem = kFp8 ? 1 : 2;
  static constexpr int kTile = kFp8 ? 128 : 64;            // tokens per stage
  static constexpr int kRowsPerWarp = kTile / kConsumerWarps;
  static constexpr int kSub = kRowsPerWarp / 16;            // 16-token sub-blocks per warp per tile
  static constexpr int kHalves = HD * kElem / 128;         // 128-byte column groups per K/V row
  static constexpr int kQSteps = HD * kElem / 32;          // MMA k-steps over d
  static constexpr int kNT = HD / 8;                        // 8-column accumulator tiles of O
  static constexpr int kStageBytes = 2 * kTile * HD * kElem;   // one K tile + one V tile
  static_assert(HD == 128 || (!kFp8 && (HD == 64 || HD == 192 || HD == 256)), "head dimension");
};

template <int DT>
__device__ __forceinline__ void mma_qk(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (DT == FA_B200_E4M3) mma_e4m3_16832(c, a, b0, b1);
  else if constexpr (DT == FA_B200_BF16) mma_bf16_16816(c, a, b0, b1);
  else mma_f16_16816(c, a, b0, b1);
}
template <int DT>
__device__ __forceinline__ void mma_pv(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (DT == FA_B200_BF16) mma_bf16_16816(c, a, b0, b1);
  else mma_f16_16816(c, a, b0, b1);
}
template <int DT>
__device__ __forceinline__ uint32_t pack_p(float lo, float hi) {
  if constexpr (DT == FA_B200_BF16) return pack_bf16(lo, hi);
  else return pack_f16(lo, hi);
}

// `n` consecutive block_table entries starting at `bt` -> shared memory, by one warp, 16-byte vector loads where the
// source is aligned.
__device__ __forceinline__ void load_page_ids(const int32_t* bt, int n, int* sm_pages, int lane) {
  if ((reinterpret_cast<uintptr_t>(bt) & 15) == 0) {
    const int nv = n >> 2;
    for (int i = lane; i < nv; i += 32) {
      int4 v = __ldg(reinterpret_cast<const int4*>(bt) + i);
      *reinterpret_cast<int4*>(sm_pages + 4 * i) = v;
    }
    for (int i = (nv << 2) + lane; i < n; i += 32) sm_pages[i] = __ldg(bt + i);
  } else {
    for (int i = lane; i < n; i += 32) sm_pages[i] = __ldg(bt + i);
  }
}

// Producer, one thread: the TMA loads of the K/V tile that starts at token tok0 of a sequence (kTile tokens, those below
// tok_end) into one ring stage; `pages[i]` is the physical page of the sequence's page first_page + i.  The stage's
// full barrier is armed with the bytes that will arrive.
// VT: the V pool is stored transposed, (num_blocks, h_k, d, page) with tokens contiguous (the reference's paged layout
// 0, flash_attn_interface.py:2223-2227): a V tile then lands in shared memory as 128 d rows of 64 tokens.
template <int DT, int HD, bool VT>
__device__ __forceinline__ void issue_tile_loads(const CUtensorMap* tmap_k, const CUtensorMap* tmap_v, const DecodeKernelParams& p,
                                                 uint32_t stage_smem, uint32_t full_bar, const int* pages, int first_page,
                                                 int tok0, int tok_end, int hk, bool withhold) {
  using T = DecodeTraits<DT, HD>;
  const int box_tok = p.box_tok;
  const uint32_t box_bytes = static_cast<uint32_t>(box_tok) * 128u;  // one 128-byte column group
  const int boxes_per_tile = T::kTile / box_tok;
  int nvalid = 0;
  for (int j = 0; j < boxes_per_tile; ++j) nvalid += (tok0 + j * box_tok < tok_end) ? 1 : 0;
  mbar_expect_tx(full_bar, 2u * T::kHalves * nvalid * box_bytes);
  if (withhold) return;   // failure-detection test build: the bytes announced above never arrive
  const uint32_t kdst = stage_smem;
  const uint32_t vdst = kdst + T::kStageBytes / 2;
  for (int j = 0; j < nvalid; ++j) {
    const int tok = tok0 + j * box_tok;
    const int page = pages[tok / p.page_size - first_page];
    const int row = tok % p.page_size;
    const uint32_t off = j * box_bytes;
#pragma unroll
    for (int hf = 0; hf < T::kHalves; ++hf) {
      tma_load_4d(kdst + hf * (T::kTile * 128) + off, tmap_k, full_bar, hf * 64, hk, row, page);
      if constexpr (!VT) tma_load_4d(vdst + hf * (T::kTile * 128) + off, tmap_v, full_bar, hf * 64, hk, row, page);
    }
    if constexpr (VT) tma_load_4d(vdst, tmap_v, full_bar, row, 0, hk, page);   // one box: 64 tokens x 128 d rows
  }
}

// Query fragments (A operand) of one (sequence, kv head).  Row r of the 16-row tile is query token r / group and head
// r % group of the kv head's group (one token per sequence: the rows are the heads); rows past sq * group are zero.
// QT: element type of the queries.  Normally QT == DT; QT = F16 / BF16 with DT = E4M3 is the "fp8 KV cache" mode: the
// cache is e4m3 (or e5m2), the queries (and the output) are 16-bit.  K is then converted to f16 in registers on its way
// into the Q K^T product (f16 MMA; bf16 queries are converted to f16 here), V as in the all-e4m3 mode.
template <int DT, int QT, int HD, int NQ>
__device__ __forceinline__ void load_q_frags(const DecodeKernelParams& p, int b, int hk, int lane, uint32_t (&qf)[NQ][4]) {
  using T = DecodeTraits<DT, HD>;
  constexpr bool kMixed = (QT != DT);
  constexpr int kQElem = kMixed ? 2 : T::kElem;
  const int g = lane >> 2, qd = lane & 3;
  const int group = p.group;
  const int rows = p.sq * group;
  const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q) +
                      (static_cast<int64_t>(b) * p.q_batch_stride + static_cast<int64_t>(hk * group) * p.q_head_stride) * kQElem;
  const int64_t off0 = ((g / group) * p.q_row_stride + (g % group) * p.q_head_stride) * kQElem;
  const int64_t off1 = (((g + 8) / group) * p.q_row_stride + ((g + 8) % group) * p.q_head_stride) * kQElem;
  if constexpr (kMixed) {
    // f16 product over an e4m3 K: per 16-wide k-step the thread holds the FOUR consecutive d values 4 * qd .. + 3
    // of its rows (first pair in registers 0/1, second in 2/3), the order in which the K bytes come out of
    // ldmatrix; the sum over k does not care about the order as long as both operands use the same one.
    auto to_f16x2 = [](uint32_t v) -> uint32_t {
      if (QT == FA_B200_F16) return v;
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
      return pack_f16(f.x, f.y);
    };
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = (16 * j + 4 * qd) * 2;
      const uint2 z = make_uint2(0u, 0u);
      const uint2 r0v = (g < rows) ? __ldg(reinterpret_cast<const uint2*>(qb + off0 + c)) : z;
      const uint2 r1v = (g + 8 < rows) ? __ldg(reinterpret_cast<const uint2*>(qb + off1 + c)) : z;
      qf[j][0] = to_f16x2(r0v.x);
      qf[j][1] = to_f16x2(r1v.x);
      qf[j][2] = to_f16x2(r0v.y);
      qf[j][3] = to_f16x2(r1v.y);
    }
  } else {
#pragma unroll
    for (int ks = 0; ks < T::kQSteps; ++ks) {
      // bytes of the two 4-byte groups this thread holds per row in k-step ks
      const int c0 = ks * 32 + 4 * qd;
      const int c1 = c0 + 16;
      qf[ks][0] = (g < rows) ? __ldg(reinterpret_cast<const uint32_t*>(qb + off0 + c0)) : 0u;
      qf[ks][1] = (g + 8 < rows) ? __ldg(reinterpret_cast<const uint32_t*>(qb + off1 + c0)) : 0u;
      qf[ks][2] = (g < rows) ? __ldg(reinterpret_cast<const uint32_t*>(qb + off0 + c1)) : 0u;
      qf[ks][3] = (g + 8 < rows) ? __ldg(reinterpret_cast<const uint32_t*>(qb + off1 + c1)) : 0u;
    }
  }
}

// Keys visible to a thread's two rows (g and g + 8 of the query tile) among the tokens below tok_end.
struct RowLimits { int hi0, hi1, lo0, lo1; };
__device__ __forceinline__ RowLimits row_limits(const DecodeKernelParams& p, int lane, int len, int tok_end, int tok_lo) {
  // query token s of sq sits at position len - sq + s, so it sees keys below len - (sq - 1 - s) when the mask is
  // causal, and not before its own window start
  RowLimits r{tok_end, tok_end, tok_lo, tok_lo};
  if (p.sq > 1) {
    const int g = lane >> 2;
    const int s0 = min(g / p.group, p.sq - 1), s1 = min((g + 8) / p.group, p.sq - 1);
    if (p.causal) {
      r.hi0 = min(tok_end, len - (p.sq - 1 - s0));
      r.hi1 = min(tok_end, len - (p.sq - 1 - s1));
    }
    if (p.window_left >= 0) {
      r.lo0 = max(0, len - (p.sq - 1 - s0) - 1 - p.window_left);
      r.lo1 = max(0, len - (p.sq - 1 - s1) - 1 - p.window_left);
    }
  }
  return r;
}

// One consumer warp's share of one landed K/V tile (tokens tok0 .. tok0 + kTile, those below tok_end are real): the
// warp owns kRowsPerWarp token rows of the tile and all 16 query rows; S = Q K^T with register-level MMAs, online
// softmax in the base-2 domain, O += P V.
template <int DT, bool VT, int QT, int HD, bool E5, int NQ>
__device__ __forceinline__ void consume_tile(uint32_t kbase, int tok0, int tok_end, int cw, int lane, const uint32_t (&qf)[NQ][4],
                                             const RowLimits& lim, float scale_log2, float (&m_run)[2], float (&l_run)[2],
                                             float (&o)[DecodeTraits<DT, HD>::kNT][4]) {
  using T = DecodeTraits<DT, HD>;
  constexpr bool kMixed = (QT != DT);
  const int g = lane >> 2, qd = lane & 3;
  (void)g;
  const uint32_t vbase = kbase + T::kStageBytes / 2;
  const int wrow0 = cw * T::kRowsPerWarp;
  // Rows at or past the end of the sequence were not loaded (or hold other tokens): their V must
  // be zero so that 0 * garbage cannot poison the PV product; their scores are masked by index.
  if (!VT && tok0 + wrow0 + T::kRowsPerWarp > tok_end) {
    const int first_bad = max(tok_end - tok0, wrow0);
    const int nchunk = T::kHalves * 8;
    for (int r = first_bad; r < wrow0 + T::kRowsPerWarp; ++r) {
      if (lane < nchunk) {
        const uint32_t a = vbase + (lane >> 3) * (T::kTile * 128) + r * 128 + ((lane & 7) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0u) : "memory");
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int sb = 0; sb < T::kSub; ++sb) {
    const int r0 = wrow0 + sb * 16;
    if (tok0 + r0 >= tok_end) continue;  // warp-uniform: nothing valid in this sub-block
    // ---- S = Q K^T for 16 tokens (two 8-token n-tiles)
    float sc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
    {
      const int row = r0 + ((lane >> 4) << 3) + (lane & 7);
      const uint32_t rbase = kbase + row * 128;
      const int rsw = row & 7;
#pragma unroll
      for (int ks = 0; ks < T::kQSteps; ++ks) {
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        const uint32_t addr = rbase + (chunk >> 3) * (T::kTile * 128) + (((chunk & 7) ^ rsw) << 4);
        uint32_t b00, b01, b10, b11;
        ldsm_x4(addr, b00, b01, b10, b11);
        if constexpr (kMixed) {
          // each register holds four consecutive e4m3 d values of one token: two f16 pairs, one 16-wide k-step
          mma_f16_16816(sc[0], qf[2 * ks], cvt_fp8x2_to_f16x2<E5>(b00), cvt_fp8x2_to_f16x2<E5>(b00 >> 16));
          mma_f16_16816(sc[0], qf[2 * ks + 1], cvt_fp8x2_to_f16x2<E5>(b01), cvt_fp8x2_to_f16x2<E5>(b01 >> 16));
          mma_f16_16816(sc[1], qf[2 * ks], cvt_fp8x2_to_f16x2<E5>(b10), cvt_fp8x2_to_f16x2<E5>(b10 >> 16));
          mma_f16_16816(sc[1], qf[2 * ks + 1], cvt_fp8x2_to_f16x2<E5>(b11), cvt_fp8x2_to_f16x2<E5>(b11 >> 16));
        } else {
          mma_qk<DT>(sc[0], qf[ks], b00, b01);
          mma_qk<DT>(sc[1], qf[ks], b10, b11);
        }
      }
    }
    // ---- online softmax (base-2 domain), rows g and g+8
    const int tokb = tok0 + r0 + 2 * qd;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tk = tokb + nt * 8 + e;
        sc[nt][e] = (tk < lim.hi0 && tk >= lim.lo0) ? sc[nt][e] * scale_log2 : -INFINITY;
        sc[nt][2 + e] = (tk < lim.hi1 && tk >= lim.lo1) ? sc[nt][2 + e] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, sc[nt][e]);
        mx1 = fmaxf(mx1, sc[nt][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
    const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float al0 = fast_exp2(m_run[0] - ms0), al1 = fast_exp2(m_run[1] - ms1);
    m_run[0] = mn0;
    m_run[1] = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sc[nt][e] = fast_exp2(sc[nt][e] - ms0);
        sc[nt][2 + e] = fast_exp2(sc[nt][2 + e] - ms1);
        ps0 += sc[nt][e];
        ps1 += sc[nt][2 + e];
      }
    }
    l_run[0] = l_run[0] * al0 + ps0;
    l_run[1] = l_run[1] * al1 + ps1;
    if (__any_sync(0xffffffffu, (al0 != 1.f) || (al1 != 1.f))) {
#pragma unroll
      for (int i = 0; i < T::kNT; ++i) {
        o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1;
      }
    }
    // ---- O += P V
    uint32_t pa[4];
    pa[0] = pack_p<DT>(sc[0][0], sc[0][1]);
    pa[1] = pack_p<DT>(sc[0][2], sc[0][3]);
    pa[2] = pack_p<DT>(sc[1][0], sc[1][1]);
    pa[3] = pack_p<DT>(sc[1][2], sc[1][3]);
    {
      const int mi = lane >> 3;
      if constexpr (VT) {
        // tokens at or past the end of the sequence were loaded with whatever the page holds there: their P is
        // zero, and the fragment halves that hold them are cleared so that 0 * NaN cannot reach O
        const int limv = tok_end - tok0 - r0;   // valid tokens of this 16-token sub-block
        const int t_lo = 2 * qd;
        const uint32_t keep_lo = (t_lo < limv ? 0x0000ffffu : 0u) | (t_lo + 1 < limv ? 0xffff0000u : 0u);
        const uint32_t keep_hi = (t_lo + 8 < limv ? 0x0000ffffu : 0u) | (t_lo + 9 < limv ? 0xffff0000u : 0u);
#pragma unroll
        for (int nd = 0; nd < 16; nd += 2) {
          const int drow = (nd + (mi >> 1)) * 8 + (lane & 7);
          const int chunk = (r0 >> 3) + (mi & 1);   // 16-byte piece (8 tokens) of the d row
          const uint32_t addr = vbase + drow * 128 + ((chunk ^ (drow & 7)) << 4);
          uint32_t v0, v1, v2, v3;
          ldsm_x4(addr, v0, v1, v2, v3);
          mma_pv<DT>(o[nd], pa, v0 & keep_lo, v1 & keep_hi);
          mma_pv<DT>(o[nd + 1], pa, v2 & keep_lo, v3 & keep_hi);
        }
      } else {
        const int row = r0 + ((mi & 1) << 3) + (lane & 7);
        const uint32_t rbase = vbase + row * 128;
        const int rsw = row & 7;
        if constexpr (!T::kFp8) {
#pragma unroll
          for (int nd = 0; nd < T::kNT; nd += 2) {
            const int chunk = nd + (mi >> 1);
            const uint32_t addr = rbase + (chunk >> 3) * (T::kTile * 128) + (((chunk & 7) ^ rsw) << 4);
            uint32_t v0, v1, v2, v3;
            ldsm_x4_trans(addr, v0, v1, v2, v3);
            mma_pv<DT>(o[nd], pa, v0, v1);
            mma_pv<DT>(o[nd + 1], pa, v2, v3);
          }
        } else {
          // e4m3 V: a transposed 16-bit ldmatrix yields, per thread, the bytes
          // {V[2q][2g], V[2q][2g+1], V[2q+1][2g], V[2q+1][2g+1]}; a byte permute separates the even
          // and odd d columns, each converted to an f16x2 B fragment.  Output n-tile 2c+par covers
          // d = 16c + 2n + par.
#pragma unroll
          for (int cc = 0; cc < 8; cc += 2) {
            const int chunk = cc + (mi >> 1);
            const uint32_t addr = rbase + ((chunk ^ rsw) << 4);
            uint32_t w0, w1, w2, w3;
            ldsm_x4_trans(addr, w0, w1, w2, w3);
            const uint32_t t0 = __byte_perm(w0, 0u, 0x3120), t1 = __byte_perm(w1, 0u, 0x3120);
            const uint32_t t2 = __byte_perm(w2, 0u, 0x3120), t3 = __byte_perm(w3, 0u, 0x3120);
            mma_pv<DT>(o[2 * cc], pa, cvt_fp8x2_to_f16x2<E5>(t0), cvt_fp8x2_to_f16x2<E5>(t1));
            mma_pv<DT>(o[2 * cc + 1], pa, cvt_fp8x2_to_f16x2<E5>(t0 >> 16), cvt_fp8x2_to_f16x2<E5>(t1 >> 16));
            mma_pv<DT>(o[2 * cc + 2], pa, cvt_fp8x2_to_f16x2<E5>(t2), cvt_fp8x2_to_f16x2<E5>(t3));
            mma_pv<DT>(o[2 * cc + 3], pa, cvt_fp8x2_to_f16x2<E5>(t2 >> 16), cvt_fp8x2_to_f16x2<E5>(t3 >> 16));
          }
        }
      }
    }
  }
}

// Column d of accumulator element e (0 / 1) of n-tile j held by quad lane qd.
template <int DT, int HD>
__device__ __forceinline__ int acc_column(int j, int qd, int e) {
  if constexpr (DecodeTraits<DT, HD>::kFp8) return (j >> 1) * 16 + 4 * qd + (j & 1) + 2 * e;
  else return j * 8 + 2 * qd + e;
}

// Four consecutive output columns of one row -> memory in the output type (-1: fp32).
__device__ __forceinline__ void store_out4(void* out, int out_dtype, int64_t off, float4 a) {
  if (out_dtype == FA_B200_BF16) {
    __nv_bfloat162 x = __floats2bfloat162_rn(a.x, a.y), c = __floats2bfloat162_rn(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + off) =
        make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&c));
  } else if (out_dtype == FA_B200_F16) {
    __half2 x = __floats2half2_rn(a.x, a.y), c = __floats2half2_rn(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + off) =
        make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&c));
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + off) = a;
  }
}

// Merge of one (sequence, kv head)'s split-KV partials by the CTA that finished last (DecodeKernelParams::tickets):
// the LSE-combine of fa_combine.cu for the rows of one GQA group, run by the four consumer warps inside the decode
// kernel so that a split decode is one launch.  Row r of the group is query token r / group, head r % group.
//   phase A  warp w, rows w, w + 4, ..: row maximum and sum over the partitions' LSEs (the sink as one more term) and
//            the merged LSE (kept in shared memory)
//   phase B  every warp walks its share of the partitions (w, w + 4, ..) for every row with the weights
//            e^{lse_i - LSE}, eight loads in flight
//   phase C  the four warps' sums are added in a fixed order and stored
// row_slot(i, r): index of partial i's row r in o_partial (x HD floats) and lse_partial; sync(): a barrier of every
// thread that calls this function.  smem: merge_smem_floats(rows, HD) floats.  Partials were written by other CTAs:
// read past L1.  cw < 0 (a producer warp that only takes part in the barriers): no work.
__host__ __device__ constexpr int merge_smem_floats(int rows, int hd) { return kConsumerWarps * rows * hd + 16; }
// What the merge reads of the kernel parameters.  The merge is a rarely executed tail: it is kept out of line (and
// handed this small copy) so that its registers do not weigh on the tile loop of the kernel that calls it.
struct MergeArgs {
  const float* o_partial;
  const float* lse_partial;
  void* out;
  float* lse_out;
  const void* s_aux;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int32_t h, group, sq, out_dtype, s_aux_dtype, merge_sink, merge_lse_empty_is_neg;
};
__device__ __forceinline__ MergeArgs merge_args(const DecodeKernelParams& p) {
  MergeArgs a;
  a.o_partial = p.o_partial; a.lse_partial = p.lse_partial; a.out = p.out; a.lse_out = p.lse_out; a.s_aux = p.s_aux;
  a.o_batch_stride = p.o_batch_stride; a.o_head_stride = p.o_head_stride; a.o_row_stride = p.o_row_stride;
  a.h = p.h; a.group = p.group; a.sq = p.sq; a.out_dtype = p.out_dtype; a.s_aux_dtype = p.s_aux_dtype;
  a.merge_sink = p.merge_sink; a.merge_lse_empty_is_neg = p.merge_lse_empty_is_neg;
  return a;
}
struct BlockSync {
  __device__ __forceinline__ bool operator()() { __syncthreads(); return true; }
};
template <int HD, class RowSlot, class Sync>
__device__ __noinline__ void merge_group_partials(const MergeArgs p, float* smem, int b, int hk, int nparts,
                                                  int cw, int lane, RowSlot row_slot, Sync sync) {
  constexpr int NV = (HD + 127) / 128;
  const int group = p.group, rows = p.sq * group;
  float* red = smem;                                        // [4][rows][HD]
  float* sm_tot = smem + kConsumerWarps * rows * HD;        // [rows] merged LSE; +inf: the row has no key at all
  if (cw >= 0) {
    for (int r = cw; r < rows; r += kConsumerWarps) {
      const int head = hk * group + r % group, tok = r / group;
      float mx = -INFINITY;
      for (int i = lane; i < nparts; i += 32) {
        float l = __ldcg(p.lse_partial + row_slot(i, r));
        if (l == INFINITY) l = -INFINITY;
        mx = fmaxf(mx, l);
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      float sum = 0.f;
      if (mx != -INFINITY) {
        for (int i = lane; i < nparts; i += 32) {
          float l = __ldcg(p.lse_partial + row_slot(i, r));
          if (l == INFINITY) l = -INFINITY;
          sum += expf(l - mx);
        }
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
      if (p.merge_sink && p.s_aux) {
        const float sink = load_sink_log2(p.s_aux, p.s_aux_dtype, head) * kLn2;
        const float m2 = fmaxf(mx, sink);
        sum = (mx == -INFINITY ? 0.f : sum * expf(mx - m2)) + expf(sink - m2);
        mx = m2;
      }
      const bool empty = !(sum > 0.f);
      const float lse_tot = empty ? 0.f : mx + logf(sum);
      if (lane == 0) sm_tot[r] = empty ? INFINITY : lse_tot;
      if (lane == 0 && p.lse_out)
        p.lse_out[(static_cast<int64_t>(b) * p.h + head) * p.sq + tok] =
            empty ? (p.merge_lse_empty_is_neg ? -INFINITY : INFINITY) : lse_tot;
    }
  }
  sync();
  if (cw >= 0) {
    for (int r = 0; r < rows; ++r) {
      const float lse_tot = sm_tot[r];
      float4 acc[NV];
#pragma unroll
      for (int g = 0; g < NV; ++g) acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
      constexpr int U = 8 / NV;
      for (int i0 = cw; i0 < nparts; i0 += U * kConsumerWarps) {
        float4 v[U][NV];
        float w[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const int i = i0 + j * kConsumerWarps;
          w[j] = 0.f;
          if (i < nparts && lse_tot != INFINITY) {
            const float l = __ldcg(p.lse_partial + row_slot(i, r));
            w[j] = (l == INFINITY || l == -INFINITY) ? 0.f : expf(l - lse_tot);
          }
          // a weight of exactly zero must not pick up NaN / Inf from a partial that was never written
          if (w[j] != 0.f) {
            const float4* src = reinterpret_cast<const float4*>(p.o_partial + row_slot(i, r) * HD) + lane;
#pragma unroll
            for (int g = 0; g < NV; ++g)
              if (4 * lane + 128 * g < HD) v[j][g] = __ldcg(src + 32 * g);
          }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
          if (w[j] != 0.f) {
#pragma unroll
            for (int g = 0; g < NV; ++g)
              if (4 * lane + 128 * g < HD) {
                acc[g].x += w[j] * v[j][g].x; acc[g].y += w[j] * v[j][g].y;
                acc[g].z += w[j] * v[j][g].z; acc[g].w += w[j] * v[j][g].w;
              }
          }
        }
      }
#pragma unroll
      for (int g = 0; g < NV; ++g)
        if (4 * lane + 128 * g < HD)
          *reinterpret_cast<float4*>(red + (static_cast<int64_t>(cw) * rows + r) * HD + 4 * lane + 128 * g) = acc[g];
    }
  }
  sync();
  if (cw >= 0) {
    for (int r = cw; r < rows; r += kConsumerWarps) {
      const int head = hk * group + r % group, tok = r / group;
#pragma unroll
      for (int g = 0; g < NV; ++g) {
        if (4 * lane + 128 * g >= HD) continue;
        float4 a = *reinterpret_cast<const float4*>(red + static_cast<int64_t>(r) * HD + 4 * lane + 128 * g);
#pragma unroll
        for (int w = 1; w < kConsumerWarps; ++w) {
          const float4 t = *reinterpret_cast<const float4*>(red + (static_cast<int64_t>(w) * rows + r) * HD + 4 * lane + 128 * g);
          a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
        }
        const int64_t off = static_cast<int64_t>(b) * p.o_batch_stride + static_cast<int64_t>(tok) * p.o_row_stride +
                            static_cast<int64_t>(head) * p.o_head_stride + 4 * lane + 128 * g;
        store_out4(p.out, p.out_dtype, off, a);
      }
    }
  }
}

}  // namespace fa
