// Paged-KV decode for sm_100a with the work cut into EQUAL shares: the default decode kernel.
//
// The partition-grid kernel (fa_decode.cu) gives every CTA one fixed-size token partition of one (sequence, kv head);
// with ragged lengths the last round of CTAs runs half empty and every CTA pays its own start-up, which costs a
// quarter of the time once a batch is small (a shard of a batch on one of eight GPUs).  Here every kv head has the same
// flat list of K/V tiles — for each sequence b the tiles its query can see — and the persistent grid (two CTAs per SM)
// gives every head m = grid / h_k CTAs: CTA c works for head c / m on tiles [j * per, (j + 1) * per) of the list,
// j = c % m, per = ceil(list / m).  The m-th, 2m-th ... CTAs therefore stream the SAME token rows for different heads at
// the same time: a token's row holds all kv heads side by side, and reading it in pieces at unrelated times costs DRAM
// row locality (measured: a (sequence, head)-major list was 10 % slower at 16-bit and 27 % slower at 8-bit elements).
// A CTA's share is a run of SEGMENTS (pieces of consecutive sequences, for its head):
//   - a (sequence, head) pair that lies wholly inside one share is finished by that CTA and written as the final output;
//   - a pair that is cut by a share boundary leaves one fp32 partial per CTA that touches it (at most two partials per
//     CTA: the piece at the head of its share and the piece at the tail), and the CTA that finishes last — counted on a
//     ticket per pair — merges them (merge_group_partials).  One launch, no combine kernel.
// Every CTA works the list out for itself from cache_seqlens (a prefix sum over the batch in shared memory), so lengths
// stay device data and a captured launch serves other lengths.
//
// Roles per CTA as in fa_decode.cu: warp 0 streams tiles through the TMA ring (refilling its page-id window from the
// block table as it goes, across segment boundaries), warps 1-4 consume them (fa_decode_common.cuh).  At the end of a
// segment the consumers reduce across warps (and the last CTA of a pair merges) in a buffer of their own when the query
// tile has few rows (4 rows of 128 columns: the usual GQA group of one token), so the producer keeps streaming into
// the next segment; with more rows the buffer is the ring's memory and the producer waits for them (seg_done) before
// it loads the next segment's first tiles.  The consumers meet on an mbarrier, not on a named barrier: every wait in
// this kernel is bounded and a CTA that gives up raises the device status word.
#include "fa_decode_common.cuh"

namespace fa {

namespace {

constexpr int kMaxBalancedBatch = 1024;
#ifdef FA_B200_DECODE_TRACE
__device__ unsigned long long g_dtrace[320][8];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define DTRACE(slot) do { if (lane == 0 && (warp == 1 || (slot) < 2)) g_dtrace[blockIdx.x][slot] = gtime(); } while (0)
#define DTRACE_ADD(slot, v) do { if (lane == 0 && warp == 1) g_dtrace[blockIdx.x][slot] += (v); } while (0)
#else
#define DTRACE(slot) do { } while (0)
#define DTRACE_ADD(slot, v) do { } while (0)
#endif
constexpr int kOwnReduceFloats = 4 * kConsumerWarps * 128 + 16;   // the consumers' own reduce / merge buffer: 4 rows x 128 columns

// List indices are 32-bit: the host keeps b * (tiles of the longest sequence) below 2^31.
struct Segment {
  int b;
  int t0;          // first tile of the segment among the sequence's visible tiles
  int n;           // tiles of the list this CTA takes from the sequence (virtual tile of an empty one included)
  int nt;          // list tiles of the sequence (>= 1)
  int first;       // list index of the sequence's first tile
};

template <int DT, int STAGES, bool VT, int QT = DT, int HD = 128, bool E5 = false>
__global__ void __launch_bounds__(kDecodeThreads, HD > 128 ? 1 : 2)
decode_balanced_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       const DecodeKernelParams p) {
  using T = DecodeTraits<DT, HD>;
  constexpr bool kMixed = (QT != DT);
  constexpr int kStageBytes = T::kStageBytes;
  static_assert(!kMixed || (DT == FA_B200_E4M3 && !VT), "mixed mode: 16-bit queries over an e4m3 cache");
  static_assert(HD == 128 || (!kMixed && !VT), "other head dimensions: plain 16-bit pools only");
  constexpr int kQRegSteps = kMixed ? 8 : T::kQSteps;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits [4,10).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* seg_done = empty_bar + STAGES;   // the consumers are done with the ring's memory for this segment (4 arrivals)
  uint64_t* cons_bar = seg_done + 1;         // meeting point of the four consumer warps (4 arrivals)
  float* sm_m = reinterpret_cast<float*>(cons_bar + 1);              // [4][16]
  float* sm_l = sm_m + kConsumerWarps * 16;                          // [4][16]
  int* sm_pages = reinterpret_cast<int*>(sm_l + kConsumerWarps * 16);  // [kMaxPagesPerPartition]
  int* sm_pref = sm_pages + kMaxPagesPerPartition;                   // [b + 1] list tiles of the sequences before b (one kv head)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm_pref + kMaxBalancedBatch + 4);   // 16-byte aligned
  volatile int* s_last = abort_flag + 1;
  volatile int* sm_seg = abort_flag + 4;     // [4 warps][8]: the segment a consumer warp is working on
  volatile int* sm_cta = sm_seg + kConsumerWarps * 8;   // [8]: this CTA's share of the list (g0, g1, per, m, hk)
  float* sm_own = reinterpret_cast<float*>(const_cast<int*>(sm_cta) + 8);   // [kOwnReduceFloats]
  // few rows: the consumers reduce and merge in sm_own and the ring never waits for them
  const bool own_buffer = merge_smem_floats(p.sq * p.group, HD) <= kOwnReduceFloats;
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x;
#ifdef FA_B200_DECODE_TRACE
  if (threadIdx.x == 0) { for (int i = 0; i < 8; ++i) g_dtrace[c][i] = 0; g_dtrace[c][0] = gtime(); }
#endif

  // Sequence b: cache length (cut to what the block table covers), first visible tile, visible tiles.
  auto seq_geometry = [&](int b, int& len, int& first_tile, int& real_nt) {
    len = p.seqlens[b];
    if (len > p.max_len) len = p.max_len;
    if (len < 0) len = 0;
    // sliding window: the first query token (position len - sq) sees keys tok_lo .. ; tiles before tok_lo are skipped
    const int tok_lo = p.window_left >= 0 ? max(0, len - p.sq - p.window_left) : 0;
    first_tile = tok_lo / T::kTile;
    real_nt = len > first_tile * T::kTile ? (len + T::kTile - 1) / T::kTile - first_tile : 0;
  };

  // ---- the tile list: per-sequence tile counts, prefix sum (warp 0), this CTA's share
  for (int b = threadIdx.x; b < p.b; b += kDecodeThreads) {
    int len, first_tile, real_nt;
    seq_geometry(b, len, first_tile, real_nt);
    if (c == 0 && p.seqlens[b] > p.max_len) atomicOr(p.status, 0x10000);   // cut to the block table: reported once
    sm_pref[b + 1] = max(real_nt, 1);   // a pair without a visible key still gets one (virtual) tile: somebody must write its zeros
  }
  if (threadIdx.x == 0) {
    sm_pref[0] = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
    }
    mbar_init(smem_u32(seg_done), kConsumerWarps);
    mbar_init(smem_u32(cons_bar), kConsumerWarps);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  __syncthreads();
  if (warp == 0) {
    const int chunk = (p.b + 31) / 32;
    const int lo = min(p.b, lane * chunk), hi = min(p.b, lo + chunk);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += sm_pref[i + 1];
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    int run = incl - sum;
    for (int i = lo; i < hi; ++i) { run += sm_pref[i + 1]; sm_pref[i + 1] = run; }
  }
  __syncthreads();
  const int total = sm_pref[p.b];                                 // tiles of one head's list
  const int m = max(static_cast<int>(gridDim.x) / p.h_k, 1);      // CTAs per kv head
  const int per = max((total + m - 1) / m, p.min_tiles_per_cta);
  const int hk = c / m, share = c - hk * m;
  if (hk >= p.h_k) return;
  const int64_t g0_wide = static_cast<int64_t>(share) * per;
  if (g0_wide >= total) return;
  const int g0 = static_cast<int>(g0_wide), g1 = static_cast<int>(min(static_cast<int64_t>(total), g0_wide + per));

  // The consumers keep the share's bounds in shared memory, not in registers: their tile loop needs every register
  // for accumulators and fragments.
  if (threadIdx.x == 0) { sm_cta[0] = g0; sm_cta[1] = g1; sm_cta[2] = per; sm_cta[3] = m; sm_cta[4] = hk; }
  __syncthreads();

  if (threadIdx.x == 32) {
#ifdef FA_B200_DECODE_TRACE
    g_dtrace[c][1] = gtime();
#endif
  }
  // list index g -> the sequence it belongs to and what a share that ends at g1 takes of it
  auto locate = [&](int g, int g1) {
    int lo = 0, hi = p.b;   // largest b with pref[b] <= g
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (sm_pref[mid] <= g) lo = mid; else hi = mid;
    }
    Segment s;
    s.b = lo;
    s.first = sm_pref[lo];
    s.nt = sm_pref[lo + 1] - s.first;
    s.t0 = g - s.first;
    s.n = min(g1 - g, s.nt - s.t0);
    return s;
  };

  const int group = p.group;  // query heads per kv head (rows of the packed query tile), <= 16
  uint32_t t_glob = 0;        // tiles this CTA has moved through the ring so far (stage and parity of the next one)

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    uint32_t seg_cnt = 0;
    bool ok = true;
    for (int g = g0; ok && g < g1;) {
      const Segment s = locate(g, g1);
      int len, first_tile, real_nt;
      seq_geometry(s.b, len, first_tile, real_nt);
      const int n_real = real_nt == 0 ? 0 : s.n;
      const int tok_begin = (first_tile + s.t0) * T::kTile;
      const int tok_end = min(len, (first_tile + s.t0 + s.n) * T::kTile);
      const int32_t* bt = p.block_table + static_cast<int64_t>(s.b) * p.bt_stride;
      const int last_page = n_real > 0 ? (tok_end - 1) / p.page_size : -1;
      int win0 = 0, win1 = 0;   // page indices [win0, win1) of the sequence held in sm_pages
      for (int i = 0; ok && i < n_real; ++i) {
        const int tok0 = tok_begin + i * T::kTile;
        const int need_last = (min(tok0 + T::kTile, tok_end) - 1) / p.page_size;
        if (need_last >= win1) {   // refill the page-id window (whole warp); earlier loads already carry their coordinates
          __syncwarp();
          win0 = tok0 / p.page_size;
          win1 = min(last_page + 1, win0 + kMaxPagesPerPartition);
          load_page_ids(bt + win0, win1 - win0, sm_pages, lane);
          __syncwarp();
        }
        if (lane == 0) {
          const uint32_t st = t_glob % STAGES, ph = (t_glob / STAGES) & 1u;
          ok = mbar_wait(smem_u32(&empty_bar[st]), ph ^ 1u, wctx);
          if (ok) {
            bool withhold = false;
#ifdef FA_B200_TEST_HOOKS
            withhold = p.test_withhold && t_glob == 0 && c == 0;
#endif
            issue_tile_loads<DT, HD, VT>(&tmap_k, &tmap_v, p, smem_u32(stages + st * kStageBytes), smem_u32(&full_bar[st]),
                                         sm_pages, win0, tok0, tok_end, hk, withhold);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        ++t_glob;
      }
      g += s.n;
      // the consumers reduce this segment through the ring's memory: no load of the next segment before they are done
      if (ok && g < g1 && !own_buffer) {
        if (lane == 0) ok = mbar_wait(smem_u32(seg_done), seg_cnt & 1u, wctx);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      ++seg_cnt;
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 1;
    const int g_ = lane >> 2, qd = lane & 3;
    const int tid = threadIdx.x - 32;  // 0..127
    ConsumerSync cons_sync{smem_u32(cons_bar), 0u, wctx, lane};
    // [4 warps][16 rows][HD]: the consumers' own buffer, or the ring between segments
    float* red = own_buffer ? sm_own : reinterpret_cast<float*>(stages);
    static_assert(merge_smem_floats(16, HD) * 4 <= STAGES * kStageBytes, "the reduce and merge buffers reuse the ring");

    if (lane == 0) sm_seg[cw * 8 + 5] = g0;   // where this warp stands in the share
    __syncwarp();
    for (;;) {
      const int g = sm_seg[cw * 8 + 5];
      if (g >= sm_cta[1]) break;
      uint32_t qf[kQRegSteps][4];
      float m_run[2] = {-INFINITY, -INFINITY};
      float l_run[2] = {0.f, 0.f};
      float o[T::kNT][4];
#pragma unroll
      for (int i = 0; i < T::kNT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
      {
        // The tile loop below keeps a row of accumulators, the query fragments and little else in registers: what the
        // end of the segment needs is parked in shared memory (per warp) and read back after the loop.
        const int hk = sm_cta[4];
        const Segment s = locate(g, sm_cta[1]);
        int len, first_tile, real_nt;
        seq_geometry(s.b, len, first_tile, real_nt);
        const int n_real = real_nt == 0 ? 0 : s.n;
        int tok0 = (first_tile + s.t0) * T::kTile;
        const int tok_end = min(len, (first_tile + s.t0 + s.n) * T::kTile);
        const int tok_lo = p.window_left >= 0 ? max(0, len - p.sq - p.window_left) : 0;
        if (lane == 0) {
          volatile int* sg = sm_seg + cw * 8;
          sg[0] = s.b; sg[2] = s.first; sg[3] = s.nt; sg[4] = s.n;
        }
        load_q_frags<DT, QT, HD>(p, s.b, hk, lane, qf);
        const RowLimits lim = row_limits(p, lane, len, tok_end, tok_lo);
        float scale_log2 = p.scale_log2;
        if (p.q_descale) scale_log2 *= p.q_descale[s.b * p.qds_b + hk * p.qds_h];
        if (p.k_descale) scale_log2 *= p.k_descale[s.b * p.kds_b + hk * p.kds_h];
        for (int i = 0; i < n_real; ++i, tok0 += T::kTile) {
          const uint32_t st = t_glob % STAGES, ph = (t_glob / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&full_bar[st]), ph, wctx)) return;
#ifdef FA_B200_DECODE_TRACE
          if (t_glob == 0) DTRACE(2);
#endif
          consume_tile<DT, VT, QT, HD, E5>(smem_u32(stages + st * kStageBytes), tok0, tok_end, cw, lane, qf, lim, scale_log2,
                                           m_run, l_run, o);
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&empty_bar[st]));
          ++t_glob;
        }
      }
      __syncwarp();
      DTRACE(3);
      DTRACE_ADD(6, 1);
      const int b = sm_seg[cw * 8 + 0];
      const int seg_first = sm_seg[cw * 8 + 2], seg_nt = sm_seg[cw * 8 + 3], seg_n = sm_seg[cw * 8 + 4];
      const int per = sm_cta[2], m = sm_cta[3], hk = sm_cta[4];
      // this head's shares that hold a piece of the sequence: c_first .. c_last
      const int c_first = seg_first / per, c_last = (seg_first + seg_nt - 1) / per;
      const bool whole = (c_first == c_last);   // the pair lies inside this CTA's share: its result is final
      // ---- end of the segment: reduce over the four warps, then write the final rows or this CTA's partial
      // every warp is done with the ring's tiles and with the previous segment's statistics
      if (!cons_sync()) return;
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
      if (qd == 0) {
        sm_m[cw * 16 + g_] = m_run[0];
        sm_m[cw * 16 + g_ + 8] = m_run[1];
        sm_l[cw * 16 + g_] = l_run[0];
        sm_l[cw * 16 + g_ + 8] = l_run[1];
      }
      if (!cons_sync()) return;
      const int rows = p.sq * group;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int row = g_ + rr * 8;
        if (row < rows) {
          float mg = -INFINITY;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) mg = fmaxf(mg, sm_m[w * 16 + row]);
          const float f = (mg == -INFINITY) ? 0.f : fast_exp2(m_run[rr] - mg);
          float* dst = red + (cw * rows + row) * HD;
#pragma unroll
          for (int j = 0; j < T::kNT; ++j) {
            dst[acc_column<DT, HD>(j, qd, 0)] = o[j][2 * rr] * f;
            dst[acc_column<DT, HD>(j, qd, 1)] = o[j][2 * rr + 1] * f;
          }
        }
      }
      if (!cons_sync()) return;
      // this CTA's partial slot of the pair: the piece at the head of the share, or the one at its tail
      const int slot = 2 * c + (g == sm_cta[0] ? 0 : 1);
      float vds = 1.f;
      if (p.v_descale) vds = p.v_descale[b * p.vds_b + hk * p.vds_h];
      for (int row = 0; row < rows; ++row) {
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
        const bool sink = whole && p.merge_sink && p.s_aux;   // the sink is one more term of the row's sum
        if (sink) finish_row(mg, L, load_sink_log2(p.s_aux, p.s_aux_dtype, head), inv, lse, empty);
#pragma unroll
        for (int dd = tid; dd < HD; dd += 128) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) acc += red[(w * rows + row) * HD + dd];
          const float outv = sink ? acc * inv * vds : (empty ? 0.f : acc / L * vds);
          if (whole) {
            const int64_t oi = static_cast<int64_t>(b) * p.o_batch_stride + static_cast<int64_t>(tok) * p.o_row_stride +
                               static_cast<int64_t>(head) * p.o_head_stride + dd;
            if (p.out_dtype == FA_B200_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(outv);
            else if (p.out_dtype == FA_B200_F16) reinterpret_cast<__half*>(p.out)[oi] = __float2half_rn(outv);
            else reinterpret_cast<float*>(p.out)[oi] = outv;
          } else {
            p.o_partial[static_cast<int64_t>(slot * 16 + row) * HD + dd] = outv;
          }
        }
        if (tid == 0) {
          if (whole) {
            if (p.lse_out)
              p.lse_out[(static_cast<int64_t>(b) * p.h + head) * p.sq + tok] =
                  empty ? (p.merge_lse_empty_is_neg ? -INFINITY : INFINITY) : lse;
          } else {
            p.lse_partial[slot * 16 + row] = lse;
          }
        }
      }
      if (!whole) {
        // one ticket per CTA that holds a piece of the pair, once its partial is visible device-wide; the last one merges
        __threadfence();
        if (!cons_sync()) return;
        if (tid == 0) {
          const int expected = c_last - c_first + 1;
          int* tk = p.tickets + b * p.h_k + hk;
          const int last = (atomicAdd(tk, 1) == expected - 1) ? 1 : 0;
          if (last) *tk = 0;   // nobody else of this launch touches it again: zero for the next launch
          *s_last = last ? expected : 0;
        }
        if (!cons_sync()) return;
        const int nparts = *s_last;
        if (nparts > 0) {
          __threadfence();
          // partial i of the pair was written by share c_first + i of this head: its head slot if the pair began
          // before that share, else its tail slot
          struct RowSlot {
            int cta0, c_first, seg_first, per;
            __device__ __forceinline__ int64_t operator()(int i, int r) const {
              const int ci = c_first + i;
              return static_cast<int64_t>((2 * (cta0 + ci) + (seg_first <= ci * per ? 0 : 1)) * 16 + r);
            }
          };
          merge_group_partials<HD>(merge_args(p), red, b, hk, nparts, cw, lane, RowSlot{hk * m, c_first, seg_first, per}, cons_sync);
          cons_sync.phase += 2;   // the merge met twice on a copy of the counter
          DTRACE(5);
          if (*abort_flag) return;
        }
      }
      // this warp no longer reads the ring's memory: the producer may refill it once all four have said so
      __syncwarp();
      DTRACE(4);
      DTRACE_ADD(7, seg_n);
      if (lane == 0) {
        sm_seg[cw * 8 + 5] = g + seg_n;
        if (g + seg_n < sm_cta[1] && !own_buffer) mbar_arrive(smem_u32(seg_done));
      }
      __syncwarp();
    }
  }
}

}  // namespace

#ifdef FA_B200_DECODE_TRACE
extern "C" __attribute__((visibility("default"))) int fa_b200_debug_decode_trace(unsigned long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_dtrace, sizeof(g_dtrace)));
}
#endif

static size_t balanced_smem_bytes(int stages, int stage_bytes) {
  return 1024 + static_cast<size_t>(stages) * stage_bytes + (2 * stages + 2) * 8 + 2 * kConsumerWarps * 16 * 4 +
         kMaxPagesPerPartition * 4 + (kMaxBalancedBatch + 4) * 4 + 16 + kConsumerWarps * 8 * 4 + 32 + kOwnReduceFloats * 4;
}
int decode_balanced_max_batch() { return kMaxBalancedBatch; }

template <int DT, bool VT, int QT = DT, int HD = 128, bool E5 = false>
static cudaError_t launch_balanced_dt(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeKernelParams& p, int max_ctas,
                                      cudaStream_t stream) {
  constexpr int STAGES = HD == 64 ? 6 : (HD == 192 ? 4 : 3);
  auto kern = decode_balanced_kernel<DT, STAGES, VT, QT, HD, E5>;
  const size_t smem = balanced_smem_bytes(STAGES, DecodeTraits<DT, HD>::kStageBytes);
  static bool attr_done[64] = {};
  static int num_sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  // Every CTA resident at once: two per SM (one above d = 128).  With 16-bit caches the launch is purely
  // bandwidth-bound and measured fastest a little below full residency (272 of 296 CTAs on a B200: fewer concurrent
  // streams into DRAM); 8-bit caches need every consumer warp they can get.  A whole number of CTAs per kv head.
  int grid = HD > 128 ? num_sms[dev] : (DecodeTraits<DT, HD>::kFp8 ? num_sms[dev] * 2 : num_sms[dev] * 184 / 100);
  if (grid > max_ctas) grid = max_ctas;
  grid = grid >= p.h_k ? grid / p.h_k * p.h_k : p.h_k;
  kern<<<grid, kDecodeThreads, smem, stream>>>(tk, tv, p);
  return cudaGetLastError();
}

cudaError_t launch_decode_balanced(int dtype, const CUtensorMap& tk, const CUtensorMap& tv, const DecodeKernelParams& p,
                                   int max_ctas, cudaStream_t stream) {
  if (p.d != 128) {   // other head dimensions: plain 16-bit pools
    if (p.kv_e4m3 || p.v_transposed || dtype == FA_B200_E4M3) return cudaErrorInvalidValue;
    const bool bf = dtype == FA_B200_BF16;
    switch (p.d) {
      case 64: return bf ? launch_balanced_dt<FA_B200_BF16, false, FA_B200_BF16, 64>(tk, tv, p, max_ctas, stream)
                         : launch_balanced_dt<FA_B200_F16, false, FA_B200_F16, 64>(tk, tv, p, max_ctas, stream);
      case 192: return bf ? launch_balanced_dt<FA_B200_BF16, false, FA_B200_BF16, 192>(tk, tv, p, max_ctas, stream)
                          : launch_balanced_dt<FA_B200_F16, false, FA_B200_F16, 192>(tk, tv, p, max_ctas, stream);
      case 256: return bf ? launch_balanced_dt<FA_B200_BF16, false, FA_B200_BF16, 256>(tk, tv, p, max_ctas, stream)
                          : launch_balanced_dt<FA_B200_F16, false, FA_B200_F16, 256>(tk, tv, p, max_ctas, stream);
    }
    return cudaErrorInvalidValue;
  }
  if (p.kv_e4m3) {   // 16-bit queries over an e4m3 / e5m2 cache
    if (p.v_transposed) return cudaErrorInvalidValue;
    if (p.kv_e5m2) {
      if (dtype == FA_B200_F16) return launch_balanced_dt<FA_B200_E4M3, false, FA_B200_F16, 128, true>(tk, tv, p, max_ctas, stream);
      if (dtype == FA_B200_BF16) return launch_balanced_dt<FA_B200_E4M3, false, FA_B200_BF16, 128, true>(tk, tv, p, max_ctas, stream);
      return cudaErrorInvalidValue;
    }
    if (dtype == FA_B200_F16) return launch_balanced_dt<FA_B200_E4M3, false, FA_B200_F16>(tk, tv, p, max_ctas, stream);
    if (dtype == FA_B200_BF16) return launch_balanced_dt<FA_B200_E4M3, false, FA_B200_BF16>(tk, tv, p, max_ctas, stream);
    return cudaErrorInvalidValue;
  }
  if (p.v_transposed) {
    if (dtype == FA_B200_F16) return launch_balanced_dt<FA_B200_F16, true>(tk, tv, p, max_ctas, stream);
    if (dtype == FA_B200_BF16) return launch_balanced_dt<FA_B200_BF16, true>(tk, tv, p, max_ctas, stream);
    return cudaErrorInvalidValue;
  }
  switch (dtype) {
    case FA_B200_F16: return launch_balanced_dt<FA_B200_F16, false>(tk, tv, p, max_ctas, stream);
    case FA_B200_BF16: return launch_balanced_dt<FA_B200_BF16, false>(tk, tv, p, max_ctas, stream);
    case FA_B200_E4M3: return launch_balanced_dt<FA_B200_E4M3, false>(tk, tv, p, max_ctas, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa
