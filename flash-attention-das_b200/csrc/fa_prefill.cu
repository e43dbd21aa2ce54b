// Dense / varlen / block-sparse attention forward for sm_100a on tcgen05 tensor cores.
//
// A CTA owns kTiles query tiles of 128 rows (kTiles = 2: two query heads of one GQA group that share
// every K/V tile) and walks the key tiles (128 keys each) of its sequence:
//   warp 0          TMA producer: Q once, then K_j / V_j tiles into a shared-memory ring (128B swizzle)
//   warp 1          MMA issuer:   S_t = Q_t K_j^T and O_t += P_t V_j with tcgen05.mma, accumulators in TMEM
//   warps 2..       softmax:      one thread per query row; S from TMEM -> scale, mask, running max/sum,
//                                 P (input dtype) written back over S in TMEM as the A operand of P V;
//                                 rescales O in TMEM only when the row max grew by more than 2^8;
//                                 epilogue O / sum -> global, LSE
// Every mbarrier wait is bounded; a CTA that gives up raises the device status word and exits through
// the common teardown (TMEM is always released).
//
// Computes what the reference's dense forward computes
// (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:2818-3328; FP8 3330-3778; softmax.h:592-640,932-964)
// and, with tile lists, its block-sparse forward (src/flash_fwd_sparse_kernel.h:36-775).
#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kMaxSparseTiles = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

template <int DT, int kTiles>
struct PrefillTraits {
  static constexpr bool kFp8 = (DT == FA_B200_E4M3);
  static constexpr int kElem = kFp8 ? 1 : 2;
  static constexpr int kTileBytes = kBlockN * kHeadDim * kElem;   // one Q, K or V tile
  static constexpr int kHalves = kFp8 ? 1 : 2;                    // 128-byte column groups per row
  static constexpr int kHalfBytes = kTileBytes / kHalves;
  static constexpr int kSlots = (kTiles == 1) ? 2 : 4;            // K/V ring
  static constexpr int kThreads = 32 * (2 + 4 * kTiles);
  static constexpr int kTmemCols = 256 * kTiles;                  // per tile: S (128) + O (128)
  static constexpr int kUmmaK = kFp8 ? 32 : 16;
  static constexpr int kKSteps = kHeadDim / kUmmaK;               // k-steps of Q K^T
  static constexpr int kPVSteps = kBlockN / kUmmaK;               // k-steps of P V
  static constexpr uint32_t kFormat = kFp8 ? 0u : (DT == FA_B200_BF16 ? 1u : 0u);
  static constexpr uint32_t kIdescQK = make_idesc(kFormat, false, kBlockM, kBlockN);
  static constexpr uint32_t kIdescPV = make_idesc(kFormat, true, kBlockM, kHeadDim);
  static constexpr int kPCols = kFp8 ? 32 : 64;                   // TMEM columns holding P
};

struct SmemLayoutInfo {
  int q_off, ring_off, bar_off, tiles_off, misc_off, total;
};

template <int DT, int kTiles>
__host__ __device__ constexpr SmemLayoutInfo smem_layout() {
  using T = PrefillTraits<DT, kTiles>;
  SmemLayoutInfo s{};
  s.q_off = 0;
  s.ring_off = s.q_off + kTiles * T::kTileBytes;
  s.bar_off = s.ring_off + T::kSlots * T::kTileBytes;
  // barriers: q_full[kTiles], kv_full[kSlots], kv_empty[kSlots], s_full[kTiles], p_full[kTiles], o_full[kTiles]
  s.tiles_off = s.bar_off + 8 * (4 * kTiles + 2 * T::kSlots);
  s.misc_off = s.tiles_off + 4 * kMaxSparseTiles;
  s.total = s.misc_off + 32;
  return s;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int dt) {
  return dt == FA_B200_BF16 ? pack_bf16(lo, hi) : pack_f16(lo, hi);
}
// four floats -> four e4m3 bytes (byte i = value i)
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  uint32_t lo, hi;
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(lo) : "f"(a), "f"(b));
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(hi) : "f"(c), "f"(d));
  return lo | (hi << 16);
}

template <int DT, int kTiles>
__global__ void __launch_bounds__(PrefillTraits<DT, kTiles>::kThreads, (kTiles == 1) ? 2 : 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const PrefillKernelParams p) {
  using T = PrefillTraits<DT, kTiles>;
  constexpr SmemLayoutInfo L = smem_layout<DT, kTiles>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint64_t* q_full = bars;
  uint64_t* kv_full = q_full + kTiles;
  uint64_t* kv_empty = kv_full + T::kSlots;
  uint64_t* s_full = kv_empty + T::kSlots;
  uint64_t* p_full = s_full + kTiles;
  uint64_t* o_full = p_full + kTiles;
  int* sm_tiles = reinterpret_cast<int*>(smem + L.tiles_off);
  uint32_t* sm_tmem_base = reinterpret_cast<uint32_t*>(smem + L.misc_off);
  int* sm_ntiles = reinterpret_cast<int*>(smem + L.misc_off + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc_off + 8);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bidb = blockIdx.z;
  const int m_block = p.is_causal ? (p.num_m_blocks - 1 - static_cast<int>(blockIdx.y)) : static_cast<int>(blockIdx.y);
  const int head0 = blockIdx.x * kTiles;
  const int group = p.h / p.h_k;
  const int hk = head0 / group;

  // ---- sequence geometry
  int q_row0, k_row0, sq, sk, coord_b;
  if (p.cu_seqlens_q) {
    q_row0 = p.cu_seqlens_q[bidb];
    sq = p.cu_seqlens_q[bidb + 1] - q_row0;
    k_row0 = p.cu_seqlens_k[bidb];
    sk = p.cu_seqlens_k[bidb + 1] - k_row0;
    coord_b = 0;
  } else {
    q_row0 = 0; k_row0 = 0; sq = p.seqlen_q; sk = p.seqlen_k; coord_b = bidb;
  }
  const int block_rows = p.sparse ? p.block_m : kBlockM;   // query rows this CTA is responsible for
  const int m0 = m_block * block_rows;
  if (m0 >= sq) return;
  const int rows_valid = min(block_rows, sq - m0);
  const int causal_shift = sk - sq;                        // bottom-right alignment

  // ---- key tile list
  if (threadIdx.x == 0) {
    int n = 0;
    if (p.sparse) {
      // block_offset holds ascending K row offsets of 64-row tiles; two adjacent entries form one
      // 128-key tile, a lone entry is a half tile (upper 64 keys masked).  bit 31 marks a half tile.
      const int64_t lrow = (static_cast<int64_t>(bidb) * p.h + head0) * p.num_q_blocks + m_block;
      int cnt = p.block_count[lrow];
      cnt = max(0, min(cnt, p.nnz_s));
      const int32_t* offs = p.block_offset + lrow * p.nnz_s;
      const int col_end = p.is_causal ? min(sk, m0 + rows_valid + causal_shift) : sk;
      int e = 0;
      while (e < cnt && n < kMaxSparseTiles) {
        const int o0 = offs[e];
        if (o0 < 0 || o0 >= col_end) { ++e; continue; }     // nothing visible in this tile
        if (e + 1 < cnt && offs[e + 1] == o0 + 64) { sm_tiles[n++] = o0; e += 2; }
        else { sm_tiles[n++] = o0 | (1 << 31); e += 1; }
      }
    } else {
      const int col_end = p.is_causal ? min(sk, m0 + rows_valid + causal_shift) : sk;
      n = col_end > 0 ? (col_end + kBlockN - 1) / kBlockN : 0;
    }
    *sm_ntiles = n;
    *abort_flag = 0;
    for (int t = 0; t < kTiles; ++t) {
      mbar_init(smem_u32(&q_full[t]), 1);
      mbar_init(smem_u32(&s_full[t]), 1);
      mbar_init(smem_u32(&p_full[t]), 128);
      mbar_init(smem_u32(&o_full[t]), 1);
    }
    for (int s = 0; s < T::kSlots; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  __syncthreads();
  const int n_tiles = *sm_ntiles;

  if (n_tiles == 0) {
    // no visible key for any row of this tile: out = 0, lse = +inf
    if (warp >= 2) {
      const int t = (warp - 2) >> 2;
      const int row = (warp & 3) * 32 + lane;
      if (row < rows_valid) {
        const int head = head0 + t;
        const int64_t grow = static_cast<int64_t>(q_row0) + m0 + row;
        uint4 z = make_uint4(0, 0, 0, 0);
        uint8_t* op = reinterpret_cast<uint8_t*>(p.out) +
                      2 * (static_cast<int64_t>(coord_b) * p.o_batch_stride + grow * p.o_row_stride + static_cast<int64_t>(head) * p.o_head_stride);
#pragma unroll
        for (int i = 0; i < 16; ++i) reinterpret_cast<uint4*>(op)[i] = z;
        if (p.lse) {
          const int64_t li = p.cu_seqlens_q ? (static_cast<int64_t>(head) * p.total_q + grow)
                                            : ((static_cast<int64_t>(bidb) * p.h + head) * p.seqlen_q + m0 + row);
          p.lse[li] = INFINITY;
        }
      }
    }
    return;
  }

  // ---- TMEM allocation (warp 1 owns it)
  if (warp == 1) {
    tmem_alloc(smem_u32(sm_tmem_base), T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm_tmem_base;

  const uint32_t q_smem = smem_u32(smem + L.q_off);
  const uint32_t ring_smem = smem_u32(smem + L.ring_off);

  if (warp == 0) {
    // ================================================================== TMA producer
    if (lane == 0) {
      for (int t = 0; t < kTiles; ++t) {
        const uint32_t bar = smem_u32(&q_full[t]);
        mbar_expect_tx(bar, T::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < T::kHalves; ++hf)
          tma_load_4d(q_smem + t * T::kTileBytes + hf * T::kHalfBytes, &tmap_q, bar, hf * 64, head0 + t, q_row0 + m0, coord_b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int start = p.sparse ? (sm_tiles[j] & 0x7fffffff) : j * kBlockN;
        bool ok = true;
#pragma unroll
        for (int kv = 0; kv < 2; ++kv) {
          const int item = 2 * j + kv;
          const int slot = item % T::kSlots;
          const uint32_t ph = (item / T::kSlots) & 1;
          if (!mbar_wait(smem_u32(&kv_empty[slot]), ph ^ 1u, wctx)) { ok = false; break; }
          const uint32_t bar = smem_u32(&kv_full[slot]);
          mbar_expect_tx(bar, T::kTileBytes);
          const CUtensorMap* tm = kv ? &tmap_v : &tmap_k;
#pragma unroll
          for (int hf = 0; hf < T::kHalves; ++hf)
            tma_load_4d(ring_smem + slot * T::kTileBytes + hf * T::kHalfBytes, tm, bar, hf * 64, hk, k_row0 + start, coord_b);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ================================================================== MMA issuer
    if (lane == 0) {
      bool ok = true;
      auto issue_qk = [&](int t, int slot) {
        const uint32_t a0 = q_smem + t * T::kTileBytes;
        const uint32_t b0 = ring_smem + slot * T::kTileBytes;
        const uint32_t d = tmem_base + t * 256;
#pragma unroll
        for (int ks = 0; ks < T::kKSteps; ++ks) {
          // bytes along the row: ks * 32; 16-bit types cross into the second 128-byte column group at ks = 4
          const uint32_t off = T::kFp8 ? ks * 32u : ((ks >> 2) * T::kHalfBytes + (ks & 3) * 32u);
          tc_mma_ss(d, make_smem_desc_sw128(a0 + off, 16, 1024), make_smem_desc_sw128(b0 + off, 16, 1024),
                    T::kIdescQK, ks > 0 ? 1u : 0u, T::kFp8);
        }
      };
      auto issue_pv = [&](int t, int slot, bool first) {
        const uint32_t b0 = ring_smem + slot * T::kTileBytes;
        const uint32_t d = tmem_base + t * 256 + 128;
        const uint32_t a = tmem_base + t * 256;
#pragma unroll
        for (int ks = 0; ks < T::kPVSteps; ++ks) {
          // V tile rows are keys: a k-step spans kUmmaK rows of 128 bytes; the two 64-column groups of a
          // 16-bit tile are kHalfBytes apart (leading-dimension offset)
          tc_mma_ts(d, a + ks * 8, make_smem_desc_sw128(b0 + ks * (T::kUmmaK * 128), T::kHalfBytes, 1024),
                    T::kIdescPV, (first && ks == 0) ? 0u : 1u, T::kFp8);
        }
      };
      // S_t(0) = Q_t K_0^T
      if (!mbar_wait(smem_u32(&kv_full[0]), 0, wctx)) ok = false;
      for (int t = 0; ok && t < kTiles; ++t) {
        if (!mbar_wait(smem_u32(&q_full[t]), 0, wctx)) { ok = false; break; }
        tc_fence_after();
        issue_qk(t, 0);
        tc_commit(smem_u32(&s_full[t]));
      }
      if (ok) tc_commit(smem_u32(&kv_empty[0]));  // K_0 is free once every S_t(0) MMA has completed
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int v_item = 2 * j + 1, v_slot = v_item % T::kSlots;
        const int k_item = 2 * j + 2, k_slot = k_item % T::kSlots;
        if (!mbar_wait(smem_u32(&kv_full[v_slot]), (v_item / T::kSlots) & 1, wctx)) { ok = false; break; }
        const bool more = (j + 1 < n_tiles);
        for (int t = 0; t < kTiles; ++t) {
          if (!mbar_wait(smem_u32(&p_full[t]), j & 1, wctx)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, v_slot, j == 0);
          if (t == kTiles - 1) tc_commit(smem_u32(&kv_empty[v_slot]));
          if (more) {
            if (t == 0) {
              if (!mbar_wait(smem_u32(&kv_full[k_slot]), (k_item / T::kSlots) & 1, wctx)) { ok = false; break; }
              tc_fence_after();
            }
            issue_qk(t, k_slot);
            tc_commit(smem_u32(&s_full[t]));
            if (t == kTiles - 1) tc_commit(smem_u32(&kv_empty[k_slot]));
          } else {
            tc_commit(smem_u32(&o_full[t]));
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ================================================================== softmax / correction / epilogue
    const int t = (warp - 2) >> 2;
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    const uint32_t t_s = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + t * 256;
    const uint32_t t_o = t_s + 128;
    const int head = head0 + t;
    const int row_in_seq = m0 + row;
    const int row_limit = p.is_causal ? min(sk, row_in_seq + 1 + causal_shift) : sk;

    float scale_log2 = p.scale_log2;
    if (p.q_descale) scale_log2 *= p.q_descale[bidb * p.qds_b + hk * p.qds_h];
    if (p.k_descale) scale_log2 *= p.k_descale[bidb * p.kds_b + hk * p.kds_h];

    float m_ref = -INFINITY;   // reference max (scaled, log2 units) the stored P and O are relative to
    float l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(smem_u32(&s_full[t]), j & 1, wctx)) { ok = false; break; }
      tc_fence_after();
      int start = j * kBlockN;
      bool half_tile = false;
      if (p.sparse) { const int v = sm_tiles[j]; start = v & 0x7fffffff; half_tile = (v < 0); }

      uint32_t u[4][32];
      tmem_ld_32x32(t_s + 0, u[0]);
      tmem_ld_32x32(t_s + 32, u[1]);
      tmem_ld_32x32(t_s + 64, u[2]);
      tmem_ld_32x32(t_s + 96, u[3]);
      tmem_wait_ld();
#define S_AT(idx) __uint_as_float(u[(idx) >> 5][(idx) & 31])
      // mask by index where the tile crosses this row's limit (warp-uniform test on the tile)
      const int tile_limit_min = p.is_causal ? min(sk, m0 + lane_grp * 32 + 1 + causal_shift) : sk;
      if (half_tile || start + kBlockN > tile_limit_min) {
        int lim = row_limit - start;
        if (half_tile) lim = min(lim, 64);
#pragma unroll
        for (int c = 0; c < 128; ++c) u[c >> 5][c & 31] = (c < lim) ? u[c >> 5][c & 31] : 0xff800000u;
      }
      float mx = S_AT(0);
#pragma unroll
      for (int c = 1; c < 128; ++c) mx = fmaxf(mx, S_AT(c));
      const float mx_scaled = mx * scale_log2;   // scale > 0
      if (j == 0) {
        m_ref = mx_scaled;
      } else {
        const bool grow = mx_scaled > m_ref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? mx_scaled : m_ref;
          const float alpha = grow ? fast_exp2(m_ref - m_new) : 1.f;   // m_ref = -inf -> 0
          l_sum *= alpha;
          m_ref = m_new;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, o);
          }
        }
      }
      const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rs = 0.f;
      if constexpr (!T::kFp8) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = fast_exp2(fmaf(S_AT(c * 32 + 2 * i), scale_log2, -m_safe));
            const float p1 = fast_exp2(fmaf(S_AT(c * 32 + 2 * i + 1), scale_log2, -m_safe));
            rs += p0 + p1;
            pk[i] = pack2(p0, p1, DT);
          }
          tmem_st_32x16(t_s + c * 16, pk);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p0 = fast_exp2(fmaf(S_AT(c * 32 + 4 * i), scale_log2, -m_safe));
            const float p1 = fast_exp2(fmaf(S_AT(c * 32 + 4 * i + 1), scale_log2, -m_safe));
            const float p2 = fast_exp2(fmaf(S_AT(c * 32 + 4 * i + 2), scale_log2, -m_safe));
            const float p3 = fast_exp2(fmaf(S_AT(c * 32 + 4 * i + 3), scale_log2, -m_safe));
            rs += (p0 + p1) + (p2 + p3);
            pk[i] = pack4_e4m3(p0, p1, p2, p3);
          }
          tmem_st_32x8(t_s + c * 8, pk);
        }
      }
#undef S_AT
      l_sum += rs;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_full[t]));
    }
    // ---- epilogue
    if (ok && mbar_wait(smem_u32(&o_full[t]), 0, wctx)) {
      tc_fence_after();
      float vds = 1.f;
      if (p.v_descale) vds = p.v_descale[bidb * p.vds_b + hk * p.vds_h];
      const bool empty = !(l_sum > 0.f);
      const float inv = empty ? 0.f : vds / l_sum;
      const int64_t grow = static_cast<int64_t>(q_row0) + row_in_seq;
      uint8_t* op = reinterpret_cast<uint8_t*>(p.out) +
                    2 * (static_cast<int64_t>(coord_b) * p.o_batch_stride + grow * p.o_row_stride + static_cast<int64_t>(head) * p.o_head_stride);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
        tmem_wait_ld();
        if (row < rows_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv, p.out_dtype);
            v.y = pack2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv, p.out_dtype);
            v.z = pack2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv, p.out_dtype);
            v.w = pack2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv, p.out_dtype);
            reinterpret_cast<uint4*>(op)[c * 4 + i] = v;
          }
        }
      }
      if (p.lse && row < rows_valid) {
        const int64_t li = p.cu_seqlens_q ? (static_cast<int64_t>(head) * p.total_q + grow)
                                          : ((static_cast<int64_t>(bidb) * p.h + head) * p.seqlen_q + row_in_seq);
        p.lse[li] = empty ? INFINITY : (m_ref + log2f(l_sum)) * kLn2;
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace

size_t prefill_smem_bytes() { return 1024 + smem_layout<FA_B200_BF16, 1>().total; }

template <int DT, int kTiles>
static cudaError_t launch_prefill_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                    const PrefillKernelParams& p, cudaStream_t stream) {
  using T = PrefillTraits<DT, kTiles>;
  auto kern = prefill_kernel<DT, kTiles>;
  const size_t smem = 1024 + smem_layout<DT, kTiles>().total;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  dim3 grid(p.h / kTiles, p.num_m_blocks, p.b);
  kern<<<grid, T::kThreads, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

cudaError_t launch_prefill(int dtype, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const PrefillKernelParams& p, cudaStream_t stream) {
  switch (dtype) {
    case FA_B200_F16: return launch_prefill_t<FA_B200_F16, 1>(tq, tk, tv, p, stream);
    case FA_B200_BF16: return launch_prefill_t<FA_B200_BF16, 1>(tq, tk, tv, p, stream);
    case FA_B200_E4M3: return launch_prefill_t<FA_B200_E4M3, 1>(tq, tk, tv, p, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa
