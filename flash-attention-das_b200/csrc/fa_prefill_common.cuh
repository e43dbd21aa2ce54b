// Pieces shared by the two tcgen05 prefill kernels (one-tile CTAs in fa_prefill.cu, persistent two-tile CTAs
// in fa_prefill_pair.cu): tile traits, MMA issue sequences, the per-row softmax step and the epilogue.
#pragma once

#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {

// Optional phase trace (compile with -DFA_B200_PHASE_TRACE): CTA 0 records clock64 stamps of its softmax warps'
// and MMA thread's hand-offs into a device array read back by fa_b200_debug_trace().  Off in normal builds.
#ifdef FA_B200_PHASE_TRACE
static __device__ long long g_trace[3][2048];   // one copy per translation unit
#define FA_TRACE(role, idx, tag)                                                  \
  do {                                                                            \
    if (blockIdx.x == 0 && (idx) < 1023) {                                        \
      g_trace[role][2 * (idx)] = (tag);                                           \
      g_trace[role][2 * (idx) + 1] = clock64();                                   \
      ++(idx);                                                                    \
    }                                                                             \
  } while (0)
#define FA_TRACE_VAL(role, idx, tag, val)                                         \
  do {                                                                            \
    if (blockIdx.x == 0 && (idx) < 1023) {                                        \
      g_trace[role][2 * (idx)] = (tag);                                           \
      g_trace[role][2 * (idx) + 1] = (val);                                       \
      ++(idx);                                                                    \
    }                                                                             \
  } while (0)
// cycle counter read that is ordered after the value `dep` has been produced
__device__ __forceinline__ uint32_t clock_after(uint32_t dep) {
  uint32_t t;
  asm volatile("{\n\t.reg .b32 d;\n\tmov.b32 d, %1;\n\tmov.u32 %0, %%clock;\n\t}" : "=r"(t) : "r"(dep) : "memory");
  return t;
}
#define FA_PROF(slot, dep) do { if (prof) { const uint32_t now_ = clock_after(dep); prof[slot] += now_ - prof_t; prof_t = now_; } } while (0)
#else
#define FA_TRACE(role, idx, tag) do { } while (0)
#define FA_PROF(slot, dep) do { } while (0)
#endif

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: O in TMEM is rescaled only when the max grew by more

// HD: head dimension, 128 for every element type and 64 / 192 / 256 for the 16-bit ones (one-tile kernel only).
template <int DT, int HD = kHeadDim>
struct TileTraits {
  static constexpr bool kFp8 = (DT == FA_B200_E4M3);
  static constexpr int kElem = kFp8 ? 1 : 2;
  static constexpr int kTileBytes = kBlockN * HD * kElem;         // one Q, K or V tile
  static constexpr int kHalves = HD * kElem / 128;                // 128-byte column groups per row
  static constexpr int kHalfBytes = kTileBytes / kHalves;         // 128 rows x 128 bytes
  static constexpr int kUmmaK = kFp8 ? 32 : 16;
  static constexpr int kKSteps = HD / kUmmaK;                     // k-steps of Q K^T
  static constexpr int kPVSteps = kBlockN / kUmmaK;               // k-steps of P V
  static constexpr int kOChunks = HD / 32;                        // 32-column pieces of an O row
  static constexpr uint32_t kFormat = kFp8 ? 0u : (DT == FA_B200_BF16 ? 1u : 0u);
  static constexpr uint32_t kIdescQK = make_idesc(kFormat, false, kBlockM, kBlockN);
  static constexpr uint32_t kIdescPV = make_idesc(kFormat, true, kBlockM, HD);
  static_assert(HD == kHeadDim || (!kFp8 && (HD == 64 || HD == 192 || HD == 256)), "head dimension");
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int dt) {
  return dt == FA_B200_BF16 ? pack_bf16(lo, hi) : pack_f16(lo, hi);
}
// four floats -> four e4m3 bytes (byte i = value i): two conversions and one register pack
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

// ---- exponentials of the e4m3 softmax ----------------------------------------------------------------------------
// An e4m3 tile has half the tensor work of a 16-bit one (about 515 cycles per 128 x 128 tile) but the same 16,384
// exponentials (1,024 cycles of the MUFU unit per tile).  P is rounded to 3 mantissa bits right after, so a share of
// the exponentials can go to the FMA pipe in a cheap form: round-to-nearest range reduction with the magic-number add, a
// degree-2 polynomial of 2^f on [-0.5, 0.5] (relative error 1.7e-3), the integer part added to the exponent field; packed
// f32x2 arithmetic.  The row sum uses the same values, so P and its normaliser stay consistent.  Measured on 8 x 4096
// tokens (two-tile kernel): 0 / 1 / 2 / 3 / 4 / 6 of every 8 groups of four columns on the FMA pipe give 1312 / 1375 /
// 1415 / 1391 / 1246 / 1103 TFLOP/s — the softmax threads are bound by the instructions they issue as much as by the
// exponential unit, so the cheap form pays only for a quarter of the columns.  (Two exponentials per MUFU instruction
// in half precision, ex2.approx.f16x2 with the f16 pair converted straight to e4m3, measured 1112.)
constexpr int kFp8PolyGroups = 2;
// 2^x for two values on the FMA pipe; x = s * scale - m, clamped below (-inf for masked columns) so that the exponent
// arithmetic cannot wrap.
__device__ __forceinline__ void exp2_poly_x2(float s0, float s1, uint64_t sc2, uint64_t nm2, float& p0, float& p1) {
  float x0, x1;
  unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), sc2, nm2), x0, x1);
  x0 = fmaxf(x0, -120.f);
  x1 = fmaxf(x1, -120.f);
  const uint64_t x2 = pack_f32x2(x0, x1);
  const uint64_t magic = pack_f32x2(12582912.f, 12582912.f);              // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  const uint64_t t2 = add_f32x2(x2, magic);
  const uint64_t r2 = add_f32x2(t2, pack_f32x2(-12582912.f, -12582912.f));   // round(x)
  const uint64_t f2 = fma_f32x2(r2, pack_f32x2(-1.f, -1.f), x2);             // x - round(x) in [-0.5, 0.5]
  uint64_t q2 = fma_f32x2(f2, pack_f32x2(0.23842697f, 0.23842697f), pack_f32x2(0.7034453f, 0.7034453f));
  q2 = fma_f32x2(q2, f2, pack_f32x2(1.00044307f, 1.00044307f));
  float q0, q1, t0, t1;
  unpack_f32x2(q2, q0, q1);
  unpack_f32x2(t2, t0, t1);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}
// ---- MMA issue sequences ---------------------------------------------------------------------------------------
// One thread feeds the tensor pipe, and a 128x128x16 product takes only 64 cycles, so the issue path has to be a
// handful of instructions per MMA: each sequence below is ONE asm block that derives the k-step descriptors with a
// single 64-bit add (the start-address field is the low 14 bits, in 16-byte units; strides and swizzle mode stay
// in the high word) and issues the 8 (16-bit) or 4 (e4m3) MMAs back to back.
//   K-major operand (Q, K): k-step ks starts 32 bytes further along the row (+2 units); a 16-bit tile continues
//     in the second 128-byte column group after 4 steps (+kHalfBytes).
//   MN-major operand (V):   k-step ks starts kUmmaK key rows = kUmmaK * 128 bytes further.
//   TMEM operand (Q, P):    k-step ks starts 8 columns further.

// S[tmem] = Q[smem] K^T[smem]
template <int DT, int HD = kHeadDim>
__device__ __forceinline__ void issue_qk(uint32_t q_smem, uint32_t k_smem, uint32_t s_tmem) {
  using T = TileTraits<DT, HD>;
  const uint64_t a0 = make_smem_desc_sw128(q_smem, 16, 1024), b0 = make_smem_desc_sw128(k_smem, 16, 1024);
  if constexpr (HD != kHeadDim) {
    // other head dimensions (16-bit): one instruction per k-step, four steps per 128-byte column group
#pragma unroll
    for (int ks = 0; ks < T::kKSteps; ++ks) {
      const uint64_t off = static_cast<uint64_t>((ks >> 2) * (T::kHalfBytes >> 4) + (ks & 3) * 2);
      tc_mma_ss(s_tmem, a0 + off, b0 + off, T::kIdescQK, ks > 0 ? 1u : 0u, false);
    }
  } else if constexpr (T::kFp8) {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 a, b;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, pf;\n\t"
        "add.s64 a, %1, 2;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 4;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 6;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a, b, %3, pt;\n\t}"
        ::"r"(s_tmem), "l"(a0), "l"(b0), "r"(T::kIdescQK) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 a, b;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
        "add.s64 a, %1, 2;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 4;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 6;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1024;\n\tadd.s64 b, %2, 1024;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1026;\n\tadd.s64 b, %2, 1026;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1028;\n\tadd.s64 b, %2, 1028;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1030;\n\tadd.s64 b, %2, 1030;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t}"
        ::"r"(s_tmem), "l"(a0), "l"(b0), "r"(T::kIdescQK) : "memory");
  }
}
static_assert((TileTraits<FA_B200_BF16>::kHalfBytes >> 4) == 1024, "k-step offsets below assume 16 KB column groups");

// Q tile (shared memory, K-major, 128-byte swizzle) -> TMEM as the A operand of Q K^T: one 128x256b copy per
// k-step (32 bytes of every row), landing in 8 consecutive columns.
template <int DT>
__device__ __forceinline__ void issue_q_to_tmem(uint32_t q_smem, uint32_t q_tmem) {
  using T = TileTraits<DT>;
  const uint64_t d0 = make_smem_desc_sw128(q_smem, 16, 1024);
#pragma unroll
  for (int ks = 0; ks < T::kKSteps; ++ks) {
    const uint32_t off16 = T::kFp8 ? ks * 2u : ((ks >> 2) * (T::kHalfBytes >> 4) + (ks & 3) * 2u);
    tc_cp_128x256b(q_tmem + ks * 8, d0 + off16);
  }
}
// S[tmem] = Q[tmem] K^T[smem]: only K is read from shared memory.
template <int DT>
__device__ __forceinline__ void issue_qk_ts(uint32_t q_tmem, uint32_t k_smem, uint32_t s_tmem) {
  using T = TileTraits<DT>;
  const uint64_t b0 = make_smem_desc_sw128(k_smem, 16, 1024);
  if constexpr (T::kFp8) {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, pf;\n\t"
        "add.u32 a, %1, 8;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 16;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 24;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a], b, %3, pt;\n\t}"
        ::"r"(s_tmem), "r"(q_tmem), "l"(b0), "r"(T::kIdescQK) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
        "add.u32 a, %1, 8;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 16;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 24;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 32;\n\tadd.s64 b, %2, 1024;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 40;\n\tadd.s64 b, %2, 1026;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 48;\n\tadd.s64 b, %2, 1028;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 56;\n\tadd.s64 b, %2, 1030;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t}"
        ::"r"(s_tmem), "r"(q_tmem), "l"(b0), "r"(T::kIdescQK) : "memory");
  }
}
// O[tmem] (+)= P[tmem] V[smem]: V is MN-major (d contiguous); the two 64-column groups of a 16-bit tile are
// kHalfBytes apart (leading-dimension offset).  `overwrite`: the first k-step replaces O instead of accumulating.
template <int DT, int HD = kHeadDim>
__device__ __forceinline__ void issue_pv(uint32_t p_tmem, uint32_t v_smem, uint32_t o_tmem, bool overwrite) {
  using T = TileTraits<DT, HD>;
  const uint64_t b0 = make_smem_desc_sw128(v_smem, T::kHalfBytes, 1024);
  const uint32_t acc0 = overwrite ? 0u : 1u;
  if constexpr (HD != kHeadDim) {
    // other head dimensions (16-bit): N = HD columns per instruction, 16 key rows (2048 bytes) per k-step
#pragma unroll
    for (int ks = 0; ks < T::kPVSteps; ++ks)
      tc_mma_ts(o_tmem, p_tmem + ks * 8, b0 + static_cast<uint64_t>(ks * 128), T::kIdescPV, ks > 0 ? 1u : acc0, false);
  } else if constexpr (T::kFp8) {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "setp.ne.b32 pf, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, pf;\n\t"
        "add.u32 a, %1, 8;\n\tadd.s64 b, %2, 256;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 16;\n\tadd.s64 b, %2, 512;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 24;\n\tadd.s64 b, %2, 768;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a], b, %3, pt;\n\t}"
        ::"r"(o_tmem), "r"(p_tmem), "l"(b0), "r"(T::kIdescPV), "r"(acc0) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "setp.ne.b32 pf, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
        "add.u32 a, %1, 8;\n\tadd.s64 b, %2, 128;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 16;\n\tadd.s64 b, %2, 256;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 24;\n\tadd.s64 b, %2, 384;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 32;\n\tadd.s64 b, %2, 512;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 40;\n\tadd.s64 b, %2, 640;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 48;\n\tadd.s64 b, %2, 768;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
        "add.u32 a, %1, 56;\n\tadd.s64 b, %2, 896;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t}"
        ::"r"(o_tmem), "r"(p_tmem), "l"(b0), "r"(T::kIdescPV), "r"(acc0) : "memory");
  }
}

// O[tmem] (+)= P[tmem] V[smem] with V given transposed: the tile is 128 d rows of 128 keys (two 128-byte column groups
// of 64 keys, 16 KB apart), i.e. a K-major B operand laid out exactly like a K tile in Q K^T.  16-bit types.
template <int DT>
__device__ __forceinline__ void issue_pv_vt(uint32_t p_tmem, uint32_t vt_smem, uint32_t o_tmem, bool overwrite) {
  using T = TileTraits<DT>;
  static_assert(!T::kFp8, "transposed V: 16-bit types");
  // same operand walk as Q K^T with Q in TMEM (issue_qk_ts): the instruction descriptor is the K-major 128 x 128 one
  const uint64_t b0 = make_smem_desc_sw128(vt_smem, 16, 1024);
  const uint32_t acc0 = overwrite ? 0u : 1u;
  asm volatile(
      "{\n\t.reg .pred pf, pt;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
      "setp.ne.b32 pf, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
      "add.u32 a, %1, 8;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 16;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 24;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 32;\n\tadd.s64 b, %2, 1024;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 40;\n\tadd.s64 b, %2, 1026;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 48;\n\tadd.s64 b, %2, 1028;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 56;\n\tadd.s64 b, %2, 1030;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t}"
      ::"r"(o_tmem), "r"(p_tmem), "l"(b0), "r"(T::kIdescQK), "r"(acc0) : "memory");
}

// Visible key range of query row i (index inside its sequence): [row_lo, row_hi).
__device__ __forceinline__ int row_hi(const PrefillKernelParams& p, int i, int sk, int shift) {
  return p.window_right >= 0 ? min(sk, i + 1 + shift + p.window_right) : sk;
}
__device__ __forceinline__ int row_lo(const PrefillKernelParams& p, int i, int shift) {
  return p.window_left >= 0 ? max(0, i + shift - p.window_left) : 0;
}
// Key tiles a block of query rows [m0, m0 + rows) touches: tiles tile0 .. tile0 + n_tiles - 1.
__device__ __forceinline__ void key_tile_range(const PrefillKernelParams& p, int m0, int rows, int sk, int shift,
                                               int& tile0, int& n_tiles) {
  const int col_end = row_hi(p, m0 + rows - 1, sk, shift);
  const int col_begin = min(row_lo(p, m0, shift), max(col_end, 0));
  tile0 = col_begin / kBlockN;
  n_tiles = col_end > col_begin ? (col_end + kBlockN - 1) / kBlockN - tile0 : 0;
}

// Running softmax state of one query row (one thread).
struct RowState {
  float m_ref;   // reference max (scaled, log2 units) that the stored P and O are relative to
  float l_sum;   // sum of P relative to m_ref
};

// One key tile for one row: S (TMEM, 128 fp32 columns at t_s) -> masked, scaled, exponentiated P written back
// over the first columns of S in the input dtype; O (at t_o) rescaled when the row max grew past the threshold.
//   lo, lim    the row sees columns lo <= c < lim of this tile (lo <= 0 and lim >= 128: all)
//   need_mask  warp-uniform: some row of the warp has lim < 128 or lo > 0
//   first      first tile of this row's sweep (O holds nothing yet)
//   o_ready_bar  (kernels that issue Q K^T of the next key tile BEFORE P V of the current one) != 0: an mbarrier that
//                completes when the previous tile's P V has finished accumulating into O; waited for with
//                o_ready_parity before O is rescaled (elsewhere S is ready only after that product, nothing to wait for)
// Returns false when that wait gave up.
template <int DT, int HD = kHeadDim>
__device__ __forceinline__ bool softmax_tile(uint32_t t_s, uint32_t t_o, float scale_log2, int lo, int lim, bool need_mask,
                                             bool first, RowState& st, [[maybe_unused]] uint32_t* prof = nullptr,
                                             uint32_t o_ready_bar = 0, uint32_t o_ready_parity = 0,
                                             const WaitCtx* wctx = nullptr) {
  using T = TileTraits<DT, HD>;
#ifdef FA_B200_PHASE_TRACE
  uint32_t prof_t = prof ? clock_after(0) : 0u;
#endif
  uint32_t u[4][32];
#define FA_S_AT(idx) __uint_as_float(u[(idx) >> 5][(idx) & 31])
  tmem_ld_32x32(t_s + 0, u[0]);
  tmem_ld_32x32(t_s + 32, u[1]);
  tmem_ld_32x32(t_s + 64, u[2]);
  tmem_ld_32x32(t_s + 96, u[3]);
  tmem_wait_ld();
  FA_PROF(0, u[3][31]);
  if (need_mask) {
#pragma unroll
    for (int c = 0; c < 128; ++c) u[c >> 5][c & 31] = (c < lim && c >= lo) ? u[c >> 5][c & 31] : 0xff800000u;
  }
  float mx0 = fmaxf(FA_S_AT(0), FA_S_AT(1)), mx1 = fmaxf(FA_S_AT(2), FA_S_AT(3));
  float mx2 = fmaxf(FA_S_AT(4), FA_S_AT(5)), mx3 = fmaxf(FA_S_AT(6), FA_S_AT(7));
#pragma unroll
  for (int c = 8; c < 128; c += 8) {
    mx0 = max3(mx0, FA_S_AT(c), FA_S_AT(c + 1));
    mx1 = max3(mx1, FA_S_AT(c + 2), FA_S_AT(c + 3));
    mx2 = max3(mx2, FA_S_AT(c + 4), FA_S_AT(c + 5));
    mx3 = max3(mx3, FA_S_AT(c + 6), FA_S_AT(c + 7));
  }
  const float mx_scaled = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;   // scale > 0
  if (first) {
    st.m_ref = mx_scaled;
  } else {
    const bool grow = mx_scaled > st.m_ref + kRescaleThreshold;
    if (__any_sync(0xffffffffu, grow)) {
      if (o_ready_bar != 0) {
        if (!mbar_wait(o_ready_bar, o_ready_parity, *wctx)) return false;
        tc_fence_after();
      }
      const float m_new = grow ? mx_scaled : st.m_ref;
      const float alpha = grow ? fast_exp2(st.m_ref - m_new) : 1.f;   // m_ref = -inf -> 0
      st.l_sum *= alpha;
      st.m_ref = m_new;
#pragma unroll
      for (int c = 0; c < T::kOChunks; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32(t_o + c * 32, o);
      }
    }
  }
  const float m_safe = (st.m_ref == -INFINITY) ? 0.f : st.m_ref;
  float rs0 = 0.f, rs1 = 0.f;
  FA_PROF(1, __float_as_uint(m_safe));
  if constexpr (!T::kFp8) {
    {
      const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(-m_safe, -m_safe);
      uint64_t rs2 = pack_f32x2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(FA_S_AT(c * 32 + 2 * i), FA_S_AT(c * 32 + 2 * i + 1)), sc2, nm2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          rs2 = add_f32x2(rs2, pack_f32x2(p0, p1));
          pk[i] = pack2(p0, p1, DT);
        }
        tmem_st_32x16(t_s + c * 16, pk);
      }
      unpack_f32x2(rs2, rs0, rs1);
    }
  } else {
    // packed f32x2 arithmetic for the scaling and the row sum: the softmax threads are bound by the instructions they issue
    const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(-m_safe, -m_safe);
    uint64_t rs2 = pack_f32x2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float p0, p1, p2, p3;
        // kFp8PolyGroups of every 8 groups go to the FMA pipe, spread evenly so that both pipes always have work
        if (((i + 1) * kFp8PolyGroups) / 8 > (i * kFp8PolyGroups) / 8) {
          exp2_poly_x2(FA_S_AT(c * 32 + 4 * i), FA_S_AT(c * 32 + 4 * i + 1), sc2, nm2, p0, p1);
          exp2_poly_x2(FA_S_AT(c * 32 + 4 * i + 2), FA_S_AT(c * 32 + 4 * i + 3), sc2, nm2, p2, p3);
        } else {
          float x0, x1, x2, x3;
          unpack_f32x2(fma_f32x2(pack_f32x2(FA_S_AT(c * 32 + 4 * i), FA_S_AT(c * 32 + 4 * i + 1)), sc2, nm2), x0, x1);
          unpack_f32x2(fma_f32x2(pack_f32x2(FA_S_AT(c * 32 + 4 * i + 2), FA_S_AT(c * 32 + 4 * i + 3)), sc2, nm2), x2, x3);
          p0 = fast_exp2(x0);
          p1 = fast_exp2(x1);
          p2 = fast_exp2(x2);
          p3 = fast_exp2(x3);
        }
        rs2 = add_f32x2(rs2, add_f32x2(pack_f32x2(p0, p1), pack_f32x2(p2, p3)));
        pk[i] = pack4_e4m3(p0, p1, p2, p3);
      }
      tmem_st_32x8(t_s + c * 8, pk);
    }
    unpack_f32x2(rs2, rs0, rs1);
  }
#undef FA_S_AT
  st.l_sum += rs0 + rs1;
  FA_PROF(2, __float_as_uint(st.l_sum));
  tmem_wait_st();
  FA_PROF(3, 0);
  return true;
}

// Byte pointer of output row `grow`, head `head`.
__device__ __forceinline__ uint8_t* out_row_ptr(const PrefillKernelParams& p, int coord_b, int64_t grow, int head) {
  return reinterpret_cast<uint8_t*>(p.out) +
         2 * (static_cast<int64_t>(coord_b) * p.o_batch_stride + grow * p.o_row_stride + static_cast<int64_t>(head) * p.o_head_stride);
}
__device__ __forceinline__ int64_t lse_index(const PrefillKernelParams& p, int bidb, int head, int64_t grow, int row_in_seq) {
  return p.cu_seqlens_q ? (static_cast<int64_t>(head) * p.total_q + grow)
                        : ((static_cast<int64_t>(bidb) * p.h + head) * p.seqlen_q + row_in_seq);
}

// 32 accumulator columns [c*32, c*32+32) of one row -> 64 bytes of 16-bit output.
__device__ __forceinline__ void store_o_chunk(uint8_t* op, int c, const uint32_t (&o)[32], float inv, int out_dtype) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = pack2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv, out_dtype);
    v.y = pack2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv, out_dtype);
    v.z = pack2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv, out_dtype);
    v.w = pack2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv, out_dtype);
    reinterpret_cast<uint4*>(op)[c * 4 + i] = v;
  }
}

// A row that sees no key at all: out = 0, lse = +inf (or the sink, the only term of its sum).
template <int HD = kHeadDim>
__device__ __forceinline__ void store_empty_row(const PrefillKernelParams& p, int coord_b, int bidb, int head, int64_t grow,
                                                int row_in_seq) {
  uint8_t* op = out_row_ptr(p, coord_b, grow, head);
  const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) reinterpret_cast<uint4*>(op)[i] = z;
  if (p.lse) p.lse[lse_index(p, bidb, head, grow, row_in_seq)] = p.s_aux ? load_sink_log2(p.s_aux, p.s_aux_dtype, head) * kLn2 : INFINITY;
}

}  // namespace fa
