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
#include "fa_decode_common.cuh"

namespace fa {

namespace {

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
  // Up to here the CTA has touched its own shared memory and its parameters only.  With programmatic dependent launch
  // it may have started during the tail of the kernel before it in the stream; everything below reads what earlier
  // kernels wrote (lengths, page table, q, the cache, the scratch and ticket words of the previous decode call).
  griddep_wait();
  griddep_launch_dependents();
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

  if (warp == 0) {
    // This partition's slice of the block table -> shared memory
    const int first_page = tok_begin / p.page_size;
    const int n_pages = (tok_end > tok_begin) ? (tok_end - 1) / p.page_size - first_page + 1 : 0;
    load_page_ids(p.block_table + static_cast<int64_t>(b) * p.bt_stride + first_page, n_pages, sm_pages, lane);
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
      const int first_page = tok_begin / p.page_size;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, wctx)) break;
        bool withhold = false;
#ifdef FA_B200_TEST_HOOKS
        withhold = p.test_withhold && t == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#endif
        issue_tile_loads<DT, HD, VT>(&tmap_k, &tmap_v, p, smem_u32(stages + s * kStageBytes), smem_u32(&full_bar[s]), sm_pages,
                                     first_page, tok_begin + t * T::kTile, tok_end, hk, withhold);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 1;
    const int g = lane >> 2, qd = lane & 3;
    uint32_t qf[kQRegSteps][4];
    load_q_frags<DT, QT, HD>(p, b, hk, lane, qf);
    const RowLimits lim = row_limits(p, lane, len, tok_end, tok_lo);
    float scale_log2 = p.scale_log2;
    if (p.q_descale) scale_log2 *= p.q_descale[b * p.qds_b + hk * p.qds_h];
    if (p.k_descale) scale_log2 *= p.k_descale[b * p.kds_b + hk * p.kds_h];

    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % STAGES;
      const uint32_t ph = (t / STAGES) & 1;
      if (!mbar_wait(smem_u32(&full_bar[s]), ph, wctx)) break;
      consume_tile<DT, VT, QT, HD, E5>(smem_u32(stages + s * kStageBytes), tok_begin + t * T::kTile, tok_end, cw, lane, qf, lim,
                                       scale_log2, m_run, l_run, o);
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
          dst[acc_column<DT, HD>(j, qd, 0)] = o[j][2 * rr] * f;
          dst[acc_column<DT, HD>(j, qd, 1)] = o[j][2 * rr + 1] * f;
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
    static_assert(merge_smem_floats(16, HD) * 4 <= STAGES * kStageBytes, "the merge buffers reuse the ring");
    // partial i's row r: partitions are b * h * sq row slots apart, rows are (sequence, head, token)
    struct RowSlot {
      int64_t part_stride, base;
      int group, sq;
      __device__ __forceinline__ int64_t operator()(int i, int r) const { return i * part_stride + base + (r % group) * sq + r / group; }
    };
    const RowSlot slot{static_cast<int64_t>(p.b) * p.h * p.sq, (static_cast<int64_t>(b) * p.h + hk * p.group) * p.sq, p.group, p.sq};
    merge_group_partials<HD>(merge_args(p), reinterpret_cast<float*>(stages), b, hk, nparts, warp - 1, lane, slot, BlockSync{});
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
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.num_partitions, p.h_k, p.b);
  cfg.blockDim = dim3(kDecodeThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tk, tv, p);
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
