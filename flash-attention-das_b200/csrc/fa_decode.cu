// Paged-KV decode for sm_100a: HBM-bound split-KV kernel.
//
// One CTA handles one (token partition, kv head, sequence).  A producer warp walks the sequence's
// block_table and streams the partition's K and V pages into a shared-memory ring with TMA tile loads
// (128-byte swizzle, one mbarrier pair per stage); four consumer warps each own 16 (or 32, e4m3) token
// rows of every tile and run S = Q K^T, an online softmax and O += P V with register-level MMAs on the
// GQA group's query heads packed into one 16-row query tile.  Each K/V byte is read from HBM once.
// The CTA writes either the final output (single partition) or an fp32 partial (O normalised by its
// own sum, natural-log LSE) that the combine kernel merges.
//
// Follows the data flow of the reference's partitioned paged attention
// (csrc/flash_attn_cutlass/src/paged_attention.cu:61-558) but with exact softmax (no epsilon) and fp32
// partials, as the reference's PyTorch oracle defines the result.
#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {

namespace {

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

// Merge of one (sequence, kv head)'s split-KV partials by the CTA that finished last (see DecodeKernelParams::tickets):
// the LSE-combine of fa_combine.cu for the rows of one GQA group, run by the four consumer warps inside the decode
// kernel so that a split decode is one launch.  Row r of the group is query token r / group, head r % group.
//   phase A  warp w, rows w, w + 4, ..: row maximum and sum over the partitions' LSEs (the sink as one more term),
//            the merged LSE, and every partition's weight e^{lse_i - LSE} into shared memory
//   phase B  every warp walks its share of the partitions (w, w + 4, ..) for every row, eight loads in flight
//   phase C  the four warps' sums are added in a fixed order and stored
// smem: at least (16 * 256 + 4 * 16 * HD) floats.  Partials were written by other CTAs: read past L1.
template <int HD>
__device__ __forceinline__ void merge_group_partials(const DecodeKernelParams& p, float* smem, int b, int hk, int nparts) {
  constexpr int NV = (HD + 127) / 128;
  constexpr int kMaxParts = 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cw = warp - 1;   // consumer warp index; the producer warp only takes part in the barriers
  const int group = p.group, rows = p.sq * group;
  float* sm_w = smem;                               // [rows][nparts]
  float* red = smem + 16 * kMaxParts;               // [4][rows][HD]
  const int64_t part_stride = static_cast<int64_t>(p.b) * p.h * p.sq;   // slots between consecutive partitions
  if (cw >= 0) {
    for (int r = cw; r < rows; r += kConsumerWarps) {
      const int head = hk * group + r % group, tok = r / group;
      const int64_t slot0 = (static_cast<int64_t>(b) * p.h + head) * p.sq + tok;
      float mx = -INFINITY;
      for (int i = lane; i < nparts; i += 32) {
        float l = __ldcg(p.lse_partial + i * part_stride + slot0);
        if (l == INFINITY) l = -INFINITY;
        mx = fmaxf(mx, l);
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      float sum = 0.f;
      if (mx != -INFINITY) {
        for (int i = lane; i < nparts; i += 32) {
          float l = __ldcg(p.lse_partial + i * part_stride + slot0);
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
      for (int i = lane; i < nparts; i += 32) {
        const float l = __ldcg(p.lse_partial + i * part_stride + slot0);
        sm_w[r * nparts + i] = (empty || l == INFINITY || l == -INFINITY) ? 0.f : expf(l - lse_tot);
      }
      if (lane == 0 && p.lse_out)
        p.lse_out[slot0] = empty ? (p.merge_lse_empty_is_neg ? -INFINITY : INFINITY) : lse_tot;
    }
  }
  __syncthreads();
  if (cw >= 0) {
    for (int r = 0; r < rows; ++r) {
      const int head = hk * group + r % group, tok = r / group;
      const int64_t slot0 = (static_cast<int64_t>(b) * p.h + head) * p.sq + tok;
      const float* wrow = sm_w + r * nparts;
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
          w[j] = (i < nparts) ? wrow[i] : 0.f;
          // a weight of exactly zero must not pick up NaN / Inf from a partial that was never written
          if (w[j] != 0.f) {
            const float4* src = reinterpret_cast<const float4*>(p.o_partial + (i * part_stride + slot0) * HD) + lane;
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
  __syncthreads();
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
        if (p.out_dtype == FA_B200_BF16) {
          __nv_bfloat162 x = __floats2bfloat162_rn(a.x, a.y), c = __floats2bfloat162_rn(a.z, a.w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) =
              make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&c));
        } else if (p.out_dtype == FA_B200_F16) {
          __half2 x = __floats2half2_rn(a.x, a.y), c = __floats2half2_rn(a.z, a.w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + off) =
              make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&c));
        } else {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off) = a;
        }
      }
    }
  }
}

// VT: the V pool is stored transposed, (num_blocks, h_k, d, page) with tokens contiguous (the reference's paged layout
// 0, flash_attn_interface.py:2223-2227): a V tile then lands in shared memory as 128 d rows of 64 tokens and feeds the
// P V product through plain (non-transposing) ldmatrix, exactly as K feeds Q K^T.  16-bit types, pages of 64 * n.
// QT: element type of the queries.  Normally QT == DT; QT = F16 / BF16 with DT = E4M3 is the "fp8 KV cache" mode: the
// cache is e4m3, the queries (and the output) are 16-bit.  K is then converted to f16 in registers on its way into the
// Q K^T product (f16 MMA; bf16 queries are converted to f16 once per CTA), V as in the all-e4m3 mode.
// E5 (mixed mode only): the cache bytes are e5m2.
template <int DT, int STAGES, bool VT, int QT = DT, int HD = 128, bool E5 = false>
__global__ void __launch_bounds__(kDecodeThreads, HD > 128 ? 1 : 2)
decode_paged_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const DecodeKernelParams p) {
  using T = DecodeTraits<DT, HD>;
  constexpr bool kMixed = (QT != DT);
  constexpr int kStageBytes = T::kStageBytes;
  static_assert(!kMixed || (DT == FA_B200_E4M3 && !VT), "mixed mode: 16-bit queries over an e4m3 cache");
  static_assert(HD == 128 || (!kMixed && !VT), "other head dimensions: plain 16-bit pools only");
  static_assert(!E5 || kMixed, "e5m2 bytes: cache under 16-bit queries only");
  constexpr int kQElem = kMixed ? 2 : T::kElem;
  constexpr int kQRegSteps = kMixed ? 8 : T::kQSteps;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits [4,10).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  float* sm_m = reinterpret_cast<float*>(empty_bar + STAGES);       // [4][16]
  float* sm_l = sm_m + kConsumerWarps * 16;                          // [4][16]
  int* sm_pages = reinterpret_cast<int*>(sm_l + kConsumerWarps * 16);  // [kMaxPagesPerPartition]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm_pages + kMaxPagesPerPartition);
  const WaitCtx wctx{abort_flag, p.status};

  const int part = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A length beyond what the block table covers would walk past the table row: cut it and report it.
  int len = p.seqlens[b];
  if (len > p.max_len) {
    len = p.max_len;
    if (threadIdx.x == 0 && part == 0) atomicOr(p.status, 0x10000);
  }
  // Partitions past the end of this sequence have nothing to do; partition 0 of an empty sequence
  // still runs to publish "no keys" (zero output, LSE marker).
  if (part * p.partition_tokens >= len && !(part == 0)) return;
  const int tok_end = min(len, (part + 1) * p.partition_tokens);
  // Sliding window: the query token (position len - 1) sees keys tok_lo .. len - 1.  A partition starts at the first
  // tile that holds a visible key; partitions wholly before the window publish "no keys" like an empty sequence.
  const int tok_lo = p.window_left >= 0 ? max(0, len - p.sq - p.window_left) : 0;   // of the first query token
  const int tok_begin = max(part * p.partition_tokens, (tok_lo / T::kTile) * T::kTile);
  const int n_tiles = (tok_end > tok_begin) ? (tok_end - tok_begin + T::kTile - 1) / T::kTile : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 0) {
    // This partition's slice of the block table -> shared memory, 16-byte vector loads where aligned.
    const int first_page = tok_begin / p.page_size;
    const int n_pages = (tok_end > tok_begin) ? (tok_end - 1) / p.page_size - first_page + 1 : 0;
    const int32_t* bt = p.block_table + static_cast<int64_t>(b) * p.bt_stride + first_page;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(bt) & 15) == 0);
    if (vec_ok) {
      const int nv = n_pages >> 2;
      for (int i = lane; i < nv; i += 32) {
        int4 v = __ldg(reinterpret_cast<const int4*>(bt) + i);
        *reinterpret_cast<int4*>(sm_pages + 4 * i) = v;
      }
      for (int i = (nv << 2) + lane; i < n_pages; i += 32) sm_pages[i] = __ldg(bt + i);
    } else {
      for (int i = lane; i < n_pages; i += 32) sm_pages[i] = __ldg(bt + i);
    }
  }
  __syncthreads();

  const int group = p.group;  // query heads per kv head (rows of the packed query tile), <= 16
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o[T::kNT][4];
#pragma unroll
  for (int i = 0; i < T::kNT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int box_tok = p.box_tok;
      const uint32_t box_bytes = static_cast<uint32_t>(box_tok) * 128u;  // one 128-byte column group
      const int boxes_per_tile = T::kTile / box_tok;
      const int first_page = tok_begin / p.page_size;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, wctx)) break;
        const int tok0 = tok_begin + t * T::kTile;
        int nvalid = 0;
        for (int j = 0; j < boxes_per_tile; ++j) nvalid += (tok0 + j * box_tok < tok_end) ? 1 : 0;
        const uint32_t fb = smem_u32(&full_bar[s]);
        mbar_expect_tx(fb, 2u * T::kHalves * nvalid * box_bytes);
#ifdef FA_B200_TEST_HOOKS
        // failure-detection test: the bytes announced above never arrive, the consumers' wait runs out
        if (p.test_withhold && t == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) continue;
#endif
        const uint32_t kdst = smem_u32(stages + s * kStageBytes);
        const uint32_t vdst = kdst + kStageBytes / 2;
        for (int j = 0; j < nvalid; ++j) {
          const int tok = tok0 + j * box_tok;
          const int page = sm_pages[tok / p.page_size - first_page];
          const int row = tok % p.page_size;
          const uint32_t off = j * box_bytes;
#pragma unroll
          for (int hf = 0; hf < T::kHalves; ++hf) {
            tma_load_4d(kdst + hf * (T::kTile * 128) + off, &tmap_k, fb, hf * 64, hk, row, page);
            if constexpr (!VT) tma_load_4d(vdst + hf * (T::kTile * 128) + off, &tmap_v, fb, hf * 64, hk, row, page);
          }
          if constexpr (VT) tma_load_4d(vdst, &tmap_v, fb, row, 0, hk, page);   // one box: 64 tokens x 128 d rows
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 1;
    const int g = lane >> 2, qd = lane & 3;
    const int head0 = hk * group;

    // Query fragments (A operand).  Row r of the 16-row tile is query token r / group and head r % group of the kv
    // head's group (one token per sequence: the rows are the heads); rows past sq * group are zero.
    const int rows = p.sq * group;
    uint32_t qf[kQRegSteps][4];
    {
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q) +
                          (static_cast<int64_t>(b) * p.q_batch_stride + static_cast<int64_t>(head0) * p.q_head_stride) * kQElem;
      const int64_t off0 = ((g / group) * p.q_row_stride + (g % group) * p.q_head_stride) * kQElem;
      const int64_t off1 = (((g + 8) / group) * p.q_row_stride + ((g + 8) % group) * p.q_head_stride) * kQElem;
      if constexpr (kMixed) {
        // f16 product over an e4m3 K: per 16-wide k-step the thread holds the FOUR consecutive d values 4 * qd .. + 3
        // of its rows (first pair in registers 0/1, second in 2/3), the order in which the K bytes come out of
        // ldmatrix below; the sum over k does not care about the order as long as both operands use the same one.
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
    // Keys visible to this thread's two rows: query token s of sq sits at position len - sq + s, so it sees keys below
    // len - (sq - 1 - s) when the mask is causal, and not before its own window start.
    int hi0 = tok_end, hi1 = tok_end, lo0 = tok_lo, lo1 = tok_lo;
    if (p.sq > 1) {
      const int s0 = min(g / group, p.sq - 1), s1 = min((g + 8) / group, p.sq - 1);
      if (p.causal) {
        hi0 = min(tok_end, len - (p.sq - 1 - s0));
        hi1 = min(tok_end, len - (p.sq - 1 - s1));
      }
      if (p.window_left >= 0) {
        lo0 = max(0, len - (p.sq - 1 - s0) - 1 - p.window_left);
        lo1 = max(0, len - (p.sq - 1 - s1) - 1 - p.window_left);
      }
    }
    float scale_log2 = p.scale_log2;
    if (p.q_descale) scale_log2 *= p.q_descale[b * p.qds_b + hk * p.qds_h];
    if (p.k_descale) scale_log2 *= p.k_descale[b * p.kds_b + hk * p.kds_h];

    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % STAGES;
      const uint32_t ph = (t / STAGES) & 1;
      if (!mbar_wait(smem_u32(&full_bar[s]), ph, wctx)) break;
      const uint32_t kbase = smem_u32(stages + s * kStageBytes);
      const uint32_t vbase = kbase + kStageBytes / 2;
      const int tok0 = tok_begin + t * T::kTile;
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
            sc[nt][e] = (tk < hi0 && tk >= lo0) ? sc[nt][e] * scale_log2 : -INFINITY;
            sc[nt][2 + e] = (tk < hi1 && tk >= lo1) ? sc[nt][2 + e] * scale_log2 : -INFINITY;
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
            const int lim = tok_end - tok0 - r0;   // valid tokens of this 16-token sub-block
            const int t_lo = 2 * qd;
            const uint32_t keep_lo = (t_lo < lim ? 0x0000ffffu : 0u) | (t_lo + 1 < lim ? 0xffff0000u : 0u);
            const uint32_t keep_hi = (t_lo + 8 < lim ? 0x0000ffffu : 0u) | (t_lo + 9 < lim ? 0xffff0000u : 0u);
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
          const int mi = lane >> 3;
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
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
    }
    // per-warp row sums: reduce over the quad
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    if (qd == 0) {
      sm_m[cw * 16 + g] = m_run[0];
      sm_m[cw * 16 + g + 8] = m_run[1];
      sm_l[cw * 16 + g] = l_run[0];
      sm_l[cw * 16 + g + 8] = l_run[1];
    }
  }
  __syncthreads();  // every tile consumed: the ring is free to be reused as the cross-warp reduce buffer
  const bool aborted = (*abort_flag != 0);
  float* red = reinterpret_cast<float*>(stages);  // [4 warps][16 rows][HD]
  static_assert(kConsumerWarps * 16 * HD * 4 <= STAGES * kStageBytes, "the reduce buffer reuses the ring");
  if (warp > 0 && !aborted) {
    const int cw = warp - 1;
    const int g = lane >> 2, qd = lane & 3;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int row = g + rr * 8;
      if (row < p.sq * group) {
        float mg = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) mg = fmaxf(mg, sm_m[w * 16 + row]);
        const float f = (mg == -INFINITY) ? 0.f : fast_exp2(m_run[rr] - mg);
        float* dst = red + (cw * 16 + row) * HD;
#pragma unroll
        for (int j = 0; j < T::kNT; ++j) {
          int d0, d1;
          if constexpr (T::kFp8) {
            d0 = (j >> 1) * 16 + 4 * qd + (j & 1);
            d1 = d0 + 2;
          } else {
            d0 = j * 8 + 2 * qd;
            d1 = d0 + 1;
          }
          dst[d0] = o[j][2 * rr] * f;
          dst[d1] = o[j][2 * rr + 1] * f;
        }
      }
    }
  }
  __syncthreads();
  if (warp > 0 && !aborted) {
    const int tid = threadIdx.x - 32;  // 0..127: column d = tid, tid + 128, ...
    float vds = 1.f;
    if (p.v_descale) vds = p.v_descale[b * p.vds_b + hk * p.vds_h];
    for (int row = 0; row < p.sq * group; ++row) {
      float mg = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) mg = fmaxf(mg, sm_m[w * 16 + row]);
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float mw = sm_m[w * 16 + row];
        L += (mw == -INFINITY) ? 0.f : sm_l[w * 16 + row] * fast_exp2(mw - mg);
      }
      const int tok = row / group;                 // query token of this row
      const int head = hk * group + row % group;
      bool empty = !(L > 0.f);
      float inv = empty ? 0.f : 1.f / L;
      float lse = empty ? -INFINITY : (mg + log2f(L)) * kLn2;
      const bool sink = p.write_final && p.s_aux;   // the sink is one more term of the row's sum
      if (sink) finish_row(mg, L, load_sink_log2(p.s_aux, p.s_aux_dtype, head), inv, lse, empty);
      const int64_t slot = ((static_cast<int64_t>(part) * p.b + b) * p.h + head) * p.sq + tok;
#pragma unroll
      for (int dd = tid; dd < HD; dd += 128) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) acc += red[(w * 16 + row) * HD + dd];
        const float outv = sink ? acc * inv * vds : (empty ? 0.f : acc / L * vds);
        if (p.write_final) {
          const int64_t oi = static_cast<int64_t>(b) * p.o_batch_stride + static_cast<int64_t>(tok) * p.o_row_stride +
                             static_cast<int64_t>(head) * p.o_head_stride + dd;
          if (p.out_dtype == FA_B200_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(outv);
          else reinterpret_cast<__half*>(p.out)[oi] = __float2half_rn(outv);
        } else {
          // partial rows are (sequence, head, token): the layout of the (b, h, sq) LSE
          p.o_partial[slot * HD + dd] = outv;
        }
      }
      if (tid == 0) {
        if (p.write_final) {
          if (p.lse_out) p.lse_out[(static_cast<int64_t>(b) * p.h + head) * p.sq + tok] = empty ? INFINITY : lse;
        } else {
          p.lse_partial[slot] = lse;
        }
      }
    }
  }
  if (p.tickets != nullptr) {
    // Split mode, merge in this kernel.  Every CTA that got here takes a ticket of its (sequence, kv head) once its
    // partial is visible device-wide (a CTA that gave up on a wait takes one too, so the count always comes back to
    // zero); the CTA that takes the last one merges.
    __threadfence();
    __syncthreads();
    int* s_last = const_cast<int*>(abort_flag) + 1;
    if (threadIdx.x == 0) {
      const int expected = max(1, min(p.num_partitions, (len + p.partition_tokens - 1) / p.partition_tokens));
      int* tk = p.tickets + b * p.h_k + hk;
      const int last = (atomicAdd(tk, 1) == expected - 1) ? 1 : 0;
      if (last) *tk = 0;   // nobody else of this launch touches it again: zero for the next launch
      *s_last = last ? expected : 0;
    }
    __syncthreads();
    const int nparts = *s_last;
    if (nparts == 0) return;
    __threadfence();
    static_assert((16 * 256 + kConsumerWarps * 16 * HD) * 4 <= STAGES * kStageBytes, "the merge buffers reuse the ring");
    merge_group_partials<HD>(p, reinterpret_cast<float*>(stages), b, hk, nparts);
  }
}

}  // namespace

static size_t decode_smem_bytes(int stages, int stage_bytes) {
  return 1024 + static_cast<size_t>(stages) * stage_bytes + 2 * stages * 8 + 2 * kConsumerWarps * 16 * 4 +
         kMaxPagesPerPartition * 4 + 16;
}
int decode_max_pages_per_partition() { return kMaxPagesPerPartition; }

template <int DT, bool VT, int QT = DT, int HD = 128, bool E5 = false>
static cudaError_t launch_decode_dt(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeKernelParams& p,
                                    cudaStream_t stream) {
  // about 96 KB of tiles in flight per CTA at two CTAs per SM; one CTA per SM above d = 128
  constexpr int STAGES = HD == 64 ? 6 : (HD == 192 ? 4 : 3);
  auto kern = decode_paged_kernel<DT, STAGES, VT, QT, HD, E5>;
  const size_t smem = decode_smem_bytes(STAGES, DecodeTraits<DT, HD>::kStageBytes);
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  dim3 grid(p.num_partitions, p.h_k, p.b);
  kern<<<grid, kDecodeThreads, smem, stream>>>(tk, tv, p);
  return cudaGetLastError();
}

cudaError_t launch_decode(int dtype, const CUtensorMap& tk, const CUtensorMap& tv, const DecodeKernelParams& p,
                          cudaStream_t stream) {
  if (p.d != 128) {   // other head dimensions: plain 16-bit pools
    if (p.kv_e4m3 || p.v_transposed || dtype == FA_B200_E4M3) return cudaErrorInvalidValue;
    const bool bf = dtype == FA_B200_BF16;
    switch (p.d) {
      case 64: return bf ? launch_decode_dt<FA_B200_BF16, false, FA_B200_BF16, 64>(tk, tv, p, stream)
                         : launch_decode_dt<FA_B200_F16, false, FA_B200_F16, 64>(tk, tv, p, stream);
      case 192: return bf ? launch_decode_dt<FA_B200_BF16, false, FA_B200_BF16, 192>(tk, tv, p, stream)
                          : launch_decode_dt<FA_B200_F16, false, FA_B200_F16, 192>(tk, tv, p, stream);
      case 256: return bf ? launch_decode_dt<FA_B200_BF16, false, FA_B200_BF16, 256>(tk, tv, p, stream)
                          : launch_decode_dt<FA_B200_F16, false, FA_B200_F16, 256>(tk, tv, p, stream);
    }
    return cudaErrorInvalidValue;
  }
  if (p.kv_e4m3) {   // 16-bit queries over an e4m3 cache
    if (p.v_transposed) return cudaErrorInvalidValue;
    if (p.kv_e5m2) {
      if (dtype == FA_B200_F16) return launch_decode_dt<FA_B200_E4M3, false, FA_B200_F16, 128, true>(tk, tv, p, stream);
      if (dtype == FA_B200_BF16) return launch_decode_dt<FA_B200_E4M3, false, FA_B200_BF16, 128, true>(tk, tv, p, stream);
      return cudaErrorInvalidValue;
    }
    if (dtype == FA_B200_F16) return launch_decode_dt<FA_B200_E4M3, false, FA_B200_F16>(tk, tv, p, stream);
    if (dtype == FA_B200_BF16) return launch_decode_dt<FA_B200_E4M3, false, FA_B200_BF16>(tk, tv, p, stream);
    return cudaErrorInvalidValue;
  }
  if (p.v_transposed) {
    if (dtype == FA_B200_F16) return launch_decode_dt<FA_B200_F16, true>(tk, tv, p, stream);
    if (dtype == FA_B200_BF16) return launch_decode_dt<FA_B200_BF16, true>(tk, tv, p, stream);
    return cudaErrorInvalidValue;
  }
  switch (dtype) {
    case FA_B200_F16: return launch_decode_dt<FA_B200_F16, false>(tk, tv, p, stream);
    case FA_B200_BF16: return launch_decode_dt<FA_B200_BF16, false>(tk, tv, p, stream);
    case FA_B200_E4M3: return launch_decode_dt<FA_B200_E4M3, false>(tk, tv, p, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa
