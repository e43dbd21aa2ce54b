// Dense / varlen / block-sparse attention forward for sm_100a on tcgen05 tensor cores — one query tile per CTA.
//
// A CTA owns one query tile of 128 rows of one head and walks the key tiles (128 keys each) of its sequence, or
// the tile list of a block-sparse row block.  Two CTAs share an SM (256 TMEM columns each):
//   warps 0-3   softmax:      one thread per query row (fa_prefill_common.cuh), then the epilogue
//   warp 4      TMA producer: Q once, then K_j / V_j tiles into a two-slot shared-memory ring (128B swizzle)
//   warp 5      MMA issuer:   S = Q K_j^T and O += P V_j with tcgen05.mma, accumulators in TMEM
//   warps 6-7   idle: they complete the second warpgroup, which hands its registers to the softmax warpgroup
//               (setmaxnreg: 40 / 216 per thread, 248 above d = 128; a row of 128 scores is live in registers at once)
// This kernel serves block-sparse lists (per-head tile lists cannot share K/V tiles between heads), K/V read through
// a block table (pages in the bshd / bhsd layouts, or with V stored transposed), and the head dimensions other than
// 128 (64, 192, 256, and 192 with 128 for v: fp16 / bf16; above 128 one CTA per SM, 512 TMEM columns); dense GQA
// prefill at d = 128 runs on the two-tile persistent kernel (fa_prefill_pair.cu), other head layouts on
// fa_prefill_dense.cu.  Every mbarrier wait is bounded; a CTA that gives up raises the device status word and
// leaves through the common teardown, so TMEM is always released.
//
// Computes what the reference's dense forward computes
// (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:2818-3328; FP8 3330-3778; softmax.h:592-640,932-964)
// and, with tile lists, its block-sparse forward (src/flash_fwd_sparse_kernel.h:36-775).
#include "fa_prefill_common.cuh"

namespace fa {
namespace {

constexpr int kMaxSparseTiles = 512;
constexpr int kMaxSlots = 3;        // K/V ring: barrier area laid out for this many
// Ring slots of a head dimension: two, and three at 192 (48 KB tiles: Q + 3 slots = 192 KB), where the third slot lets
// K_{j+1} arrive while K_j and V_j are still in use, so that the second S buffer is filled at once.
__host__ __device__ constexpr int ring_slots(int hd) { return hd == 192 ? 3 : 2; }
constexpr int kThreads = 32 * 8;
constexpr int kProducerWarp = 4, kMmaWarp = 5;
// TMEM columns: S (128) + O (head dimension of v), rounded up to a power of two.  Above 128 a CTA has its SM to itself
// and all 512 columns: two S buffers (256) + O (up to 256), see kTwoS in the kernel.
__host__ __device__ constexpr int tmem_cols(int hd) { return 128 + hd <= 256 ? 256 : 512; }

struct SmemLayoutInfo {
  int q_off, ring_off, bar_off, tiles_off, misc_off, total;
};

// Ring slots are sized for a K tile; a V tile of a smaller head dimension uses the head of its slot.
template <int DT, int HD>
__host__ __device__ constexpr SmemLayoutInfo smem_layout() {
  using T = TileTraits<DT, HD>;
  SmemLayoutInfo s{};
  s.q_off = 0;
  s.ring_off = s.q_off + T::kTileBytes;
  s.bar_off = s.ring_off + ring_slots(HD) * T::kTileBytes;
  // barriers: q_full, kv_full[kMaxSlots], kv_empty[kMaxSlots], s_full[2], p_full[2], o_full, pv_done
  s.tiles_off = s.bar_off + 8 * (7 + 2 * kMaxSlots);
  s.misc_off = s.tiles_off + 4 * kMaxSparseTiles;
  s.total = s.misc_off + 32;
  return s;
}

// kLeftWindow: the launch has a left sliding-window bound (kept out of the common build of the softmax loop).
// HD: head dimension of q and k (128; 64, 192, 256 for the 16-bit types — one CTA per SM above 128: shared memory and
// TMEM).  HDV: head dimension of v and out (= HD, or 128 with HD = 192).
// VT: the paged V pool is stored transposed (tokens contiguous): a V tile lands as 128 d rows x 128 keys.
template <int DT, bool kLeftWindow, int HD, int HDV = HD, bool VT = false>
__global__ void __launch_bounds__(kThreads, HD > 128 ? 1 : 2)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const PrefillKernelParams p) {
  using T = TileTraits<DT, HD>;
  using TV = TileTraits<DT, HDV>;
  static_assert(HDV <= HD, "a V tile must fit a ring slot");
  static_assert(!VT || (HD == kHeadDim && HDV == kHeadDim && !T::kFp8), "transposed V: 16-bit types, d = 128");
  constexpr SmemLayoutInfo L = smem_layout<DT, HD>();
  constexpr int kTmemCols = tmem_cols(HDV);
  constexpr int kSlots = ring_slots(HD);
  // Head dimensions above 128 (one CTA per SM, 512 TMEM columns): two S buffers.  Key tile j uses buffer j & 1, so
  // S(j+1) = Q K_{j+1}^T is issued BEFORE P(j) V_j and runs while the softmax of tile j is still at work; with one buffer
  // the products and the softmax of a CTA take turns and nothing else is resident on the SM to fill the gaps.
  constexpr bool kTwoS = HD > kHeadDim;
  constexpr uint32_t kColO = kTwoS ? 256 : 128;
  static_assert(!kTwoS || 256 + HDV <= 512, "two S buffers and O must fit tensor memory");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint64_t* q_full = bars;
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + kMaxSlots;
  uint64_t* s_full = kv_empty + kMaxSlots;   // [2]
  uint64_t* p_full = s_full + 2;          // [2]
  uint64_t* o_full = p_full + 2;
  uint64_t* pv_done = o_full + 1;         // (two S buffers) P V of a key tile has finished accumulating into O
  int* sm_tiles = reinterpret_cast<int*>(smem + L.tiles_off);
  uint32_t* sm_tmem_base = reinterpret_cast<uint32_t*>(smem + L.misc_off);
  int* sm_ntiles = reinterpret_cast<int*>(smem + L.misc_off + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc_off + 8);
  int* sm_tile0 = reinterpret_cast<int*>(smem + L.misc_off + 12);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bidb = blockIdx.z;
  // CTAs are dispatched in the order of their linear index (x fastest).  That order walks one kv head at a time, inside
  // it the query blocks (for causal masks: heaviest first) and for each block the query heads of the group: the CTAs
  // that are resident together then read the K/V of one or two kv heads, which stay in L2, instead of all of them
  // (32k tokens x 8 kv heads of K and V are 134 MB, more than L2: in head-fastest order every tile came back from
  // DRAM about five times).
  const int group = p.h / p.h_k;
  const int lin = static_cast<int>(blockIdx.y) * p.h + static_cast<int>(blockIdx.x);
  const int per_hk = group * p.num_m_blocks;
  const int hk = lin / per_hk;
  const int in_hk = lin - hk * per_hk;
  const int mrev = in_hk / group;
  const int head = hk * group + (in_hk - mrev * group);
  const int m_block = p.is_causal ? (p.num_m_blocks - 1 - mrev) : mrev;

  // ---- sequence geometry
  int q_row0, k_row0, sq, sk, coord_b;
  if (p.cu_seqlens_q) {
    q_row0 = p.cu_seqlens_q[bidb];
    sq = p.cu_seqlens_q[bidb + 1] - q_row0;
    k_row0 = p.paged ? 0 : p.cu_seqlens_k[bidb];
    sk = p.paged ? 0 : p.cu_seqlens_k[bidb + 1] - k_row0;
    coord_b = 0;
  } else {
    q_row0 = 0; k_row0 = 0; sq = p.seqlen_q; sk = p.seqlen_k; coord_b = bidb;
  }
  if (p.paged) {   // keys live in the paged cache: length from cache_seqlens
    sk = p.seqused_k[bidb];
    if (p.max_keys > 0 && sk > p.max_keys) {   // longer than the block table row: cut and report
      sk = static_cast<int>(p.max_keys);
      if (threadIdx.x == 0) atomicOr(p.status, 0x10000);
    }
  }
  const int block_rows = p.sparse ? p.block_m : kBlockM;   // query rows this CTA is responsible for
  const int m0 = m_block * block_rows;
  if (m0 >= sq) return;
  const int rows_valid = min(block_rows, sq - m0);
  const int causal_shift = sk - sq;                        // bottom-right alignment

  // ---- key tile list (warp 0) and barrier set-up (warp 1), side by side
  if (warp == 0) {
    int n = 0, tile0 = 0;
    const int col_end = row_hi(p, m0 + rows_valid - 1, sk, causal_shift);
    if (p.sparse) {
      // block_offset holds ascending K row offsets of 64-row tiles.  Walking the list in order, an entry that sees a key
      // (0 <= offset < col_end) starts a tile; if the entry after it lies exactly 64 rows further the two form one
      // 128-key tile, else it is a half tile (upper 64 keys masked; bit 31 marks it).  The walk is a recurrence
      // (an entry is swallowed iff its predecessor started a tile and links to it), so inside a run of linked entries
      // the starts alternate: the whole warp resolves 32 entries at a time from the distance to the run's first entry.
      const int64_t lrow = (static_cast<int64_t>(bidb) * p.h + head) * p.num_q_blocks + m_block;
      if (lane == 0 && p.column_count && p.column_count[lrow] != 0) atomicOr(p.status, 0x20000);   // vertical sparsity: not taken
      const int cnt = max(0, min(p.block_count[lrow], p.nnz_s));
      const int32_t* offs = p.block_offset + lrow * p.nnz_s;
      int carry_k = -1;   // distance of the previous chunk's last entry to its run's first entry
      for (int e0 = 0; e0 < cnt; e0 += 32) {
        const int e = e0 + lane;
        const bool in = e < cnt;
        const int o = in ? offs[e] : 0;
        const int o_prev = (in && e > 0) ? offs[e - 1] : 0;
        const int o_next = (in && e + 1 < cnt) ? offs[e + 1] : 0;
        const bool valid = in && o >= 0 && o < col_end;
        // this entry can be swallowed by its predecessor: the predecessor sees a key and links to it
        const bool chained = in && e > 0 && o_prev >= 0 && o_prev < col_end && o == o_prev + 64;
        const bool link = in && e + 1 < cnt && o_next == o + 64;
        const uint32_t heads = __ballot_sync(0xffffffffu, !chained);             // entries that begin a run
        const uint32_t upto = heads & (0xffffffffu >> (31 - lane));              // those at or before this lane
        const int k = upto ? lane - (31 - __clz(upto)) : carry_k + 1 + lane;     // distance to the run's first entry
        const bool start = valid && (k & 1) == 0;
        const uint32_t starts = __ballot_sync(0xffffffffu, start);
        const int idx = n + __popc(starts & ((1u << lane) - 1u));
        if (start && idx < kMaxSparseTiles) sm_tiles[idx] = link ? o : (o | (1 << 31));
        n = min(n + __popc(starts), kMaxSparseTiles);
        carry_k = __shfl_sync(0xffffffffu, k, 31);
      }
    } else {
      key_tile_range(p, m0, rows_valid, sk, causal_shift, tile0, n);
    }
    if (lane == 0) {
      *sm_ntiles = n;
      *sm_tile0 = tile0;
    }
  } else if (threadIdx.x == 32) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&p_full[i]), 128);
    }
    mbar_init(smem_u32(o_full), 1);
    mbar_init(smem_u32(pv_done), 1);
    for (int s = 0; s < kSlots; ++s) {
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
  const int tile0 = *sm_tile0;   // first key tile of a dense sweep (a sliding window skips the tiles before it)

  if (n_tiles == 0) {
    // no visible key for any row of this tile
    if (warp < 4) {
      const int row = (warp & 3) * 32 + lane;
      if (row < rows_valid) store_empty_row<HDV>(p, coord_b, bidb, head, static_cast<int64_t>(q_row0) + m0 + row, m0 + row);
    }
    return;
  }

  // ---- TMEM allocation (the MMA warp owns it)
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(sm_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm_tmem_base;
  const uint32_t q_smem = smem_u32(smem + L.q_off);
  const uint32_t ring_smem = smem_u32(smem + L.ring_off);

  if (warp >= 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(HD > kHeadDim ? 128 : 40));   // above d = 128 there is room
  if (warp == kProducerWarp) {
    // ================================================================== TMA producer
    if (lane == 0) {
      const uint32_t qbar = smem_u32(q_full);
      mbar_expect_tx(qbar, T::kTileBytes);
#pragma unroll
      for (int hf = 0; hf < T::kHalves; ++hf)
        tma_load_4d(q_smem + hf * T::kHalfBytes, &tmap_q, qbar, hf * 64, head, q_row0 + m0, coord_b);
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int start = p.sparse ? (sm_tiles[j] & 0x7fffffff) : (tile0 + j) * kBlockN;
#pragma unroll
        for (int kv = 0; kv < 2; ++kv) {
          const int item = 2 * j + kv;
          const int slot = item % kSlots;
          const uint32_t ph = (item / kSlots) & 1;
          if (!mbar_wait(smem_u32(&kv_empty[slot]), ph ^ 1u, wctx)) { ok = false; break; }
          const uint32_t bar = smem_u32(&kv_full[slot]);
          const CUtensorMap* tm = kv ? &tmap_v : &tmap_k;
          const int halves = kv ? TV::kHalves : T::kHalves;   // 128-byte column groups of this tile
          if (!p.paged) {
            mbar_expect_tx(bar, kv ? TV::kTileBytes : T::kTileBytes);
            for (int hf = 0; hf < halves; ++hf)
              tma_load_4d(ring_smem + slot * T::kTileBytes + hf * T::kHalfBytes, tm, bar, hf * 64, hk, k_row0 + start, coord_b);
          } else if (VT && kv) {
            // transposed V pool: one box of 64 keys x 128 d rows per column group; groups that start past the end of
            // the sequence are not fetched
            const int nbox = min(kBlockN / 64, (sk - start + 63) / 64);
            mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * T::kHalfBytes);
            const int32_t* bt = p.block_table + static_cast<int64_t>(bidb) * p.bt_stride;
            for (int i = 0; i < nbox; ++i) {
              const int tok = start + i * 64;
              tma_load_4d(ring_smem + slot * T::kTileBytes + i * T::kHalfBytes, tm, bar, tok % p.page_size, 0, hk,
                          bt[tok / p.page_size]);
            }
          } else {
            // the tile's 128 keys come from one or more pages: one box of box_rows rows per page piece; boxes that
            // start past the end of the sequence are not fetched (their block_table slots are not valid)
            const int nbox = min(kBlockN / p.box_rows, (sk - start + p.box_rows - 1) / p.box_rows);
            mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * p.box_rows * 128u * halves);
            const int32_t* bt = p.block_table + static_cast<int64_t>(bidb) * p.bt_stride;
            for (int i = 0; i < nbox; ++i) {
              const int tok = start + i * p.box_rows;
              const int page = bt[tok / p.page_size], row = tok % p.page_size;
              for (int hf = 0; hf < halves; ++hf)
                tma_load_4d(ring_smem + slot * T::kTileBytes + hf * T::kHalfBytes + i * p.box_rows * 128, tm, bar, hf * 64, hk,
                            row, page);
            }
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t t_o = tmem_base + kColO;
      // buffer, full barrier and phase of key tile j
      auto s_col = [&](int j) -> uint32_t { return tmem_base + (kTwoS ? static_cast<uint32_t>(j & 1) * 128u : 0u); };
      auto sp_idx = [&](int j) -> int { return kTwoS ? (j & 1) : 0; };
      auto sp_phase = [&](int j) -> uint32_t { return static_cast<uint32_t>(kTwoS ? (j >> 1) : j) & 1u; };
      bool ok = mbar_wait(smem_u32(&kv_full[0]), 0, wctx) && mbar_wait(smem_u32(q_full), 0, wctx);
      if (ok) {
        tc_fence_after();
        issue_qk<DT, HD>(q_smem, ring_smem, s_col(0));
        tc_commit(smem_u32(&s_full[0]));
        tc_commit(smem_u32(&kv_empty[0]));   // K_0 is free once S(0) has completed
      }
      auto next_qk = [&](int j) -> bool {    // S(j+1) = Q K_{j+1}^T
        const int k_item = 2 * j + 2, k_slot = k_item % kSlots;
        if (!mbar_wait(smem_u32(&kv_full[k_slot]), (k_item / kSlots) & 1, wctx)) return false;
        tc_fence_after();
        // the tensor pipe executes in issue order: this overwrite of a buffer follows the P V product that read it
        // (one buffer: P(j) V_j just above; two buffers: P(j-1) V_{j-1} of the iteration before)
        issue_qk<DT, HD>(q_smem, ring_smem + k_slot * T::kTileBytes, s_col(j + 1));
        tc_commit(smem_u32(&s_full[sp_idx(j + 1)]));
        tc_commit(smem_u32(&kv_empty[k_slot]));
        return true;
      };
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int v_item = 2 * j + 1, v_slot = v_item % kSlots;
        if (kTwoS && j + 1 < n_tiles && !next_qk(j)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&kv_full[v_slot]), (v_item / kSlots) & 1, wctx)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&p_full[sp_idx(j)]), sp_phase(j), wctx)) { ok = false; break; }
        tc_fence_after();
        if constexpr (VT) issue_pv_vt<DT>(s_col(j), ring_smem + v_slot * T::kTileBytes, t_o, j == 0);
        else issue_pv<DT, HDV>(s_col(j), ring_smem + v_slot * T::kTileBytes, t_o, j == 0);
        tc_commit(smem_u32(&kv_empty[v_slot]));
        if (kTwoS) tc_commit(smem_u32(pv_done));
        if (j + 1 < n_tiles) {
          if (!kTwoS && !next_qk(j)) { ok = false; break; }
        } else {
          tc_commit(smem_u32(o_full));
        }
      }
    }
    __syncwarp();
  }
  } else {
    // ================================================================== softmax / correction / epilogue
    // two CTAs per SM: 128 x (40 + 216) registers are exactly a CTA's half of the file; above d = 128 the CTA has the
    // file to itself (the kernel is then launched with 248 registers per thread, and this request is already met)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(HD > kHeadDim ? 248 : 216));
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    const uint32_t t_s0 = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16);
    const uint32_t t_o = t_s0 + kColO;
    const int row_in_seq = m0 + row;
    // visible keys of this row [row_first, row_limit); the smallest limit and the largest first key among this warp's
    // rows decide (warp-uniformly) whether a tile needs masking
    const int row_limit = row_hi(p, row_in_seq, sk, causal_shift);
    const int warp_limit = row_hi(p, m0 + lane_grp * 32, sk, causal_shift);
    const int row_first = kLeftWindow ? row_lo(p, row_in_seq, causal_shift) : 0;
    const int warp_first = kLeftWindow ? row_lo(p, m0 + lane_grp * 32 + 31, causal_shift) : 0;

    float scale_log2 = p.scale_log2;
    if (p.q_descale) scale_log2 *= p.q_descale[bidb * p.qds_b + hk * p.qds_h];
    if (p.k_descale) scale_log2 *= p.k_descale[bidb * p.kds_b + hk * p.kds_h];

    RowState st{-INFINITY, 0.f};
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sp = kTwoS ? (j & 1) : 0;                       // S / P buffer of this tile and its barriers' phase
      const uint32_t sp_ph = static_cast<uint32_t>(kTwoS ? (j >> 1) : j) & 1u;
      const uint32_t t_s = t_s0 + static_cast<uint32_t>(sp) * 128u;
      if (!mbar_wait(smem_u32(&s_full[sp]), sp_ph, wctx)) { ok = false; break; }
      tc_fence_after();
      int start = (tile0 + j) * kBlockN;
      bool half_tile = false;
      if (p.sparse) { const int v = sm_tiles[j]; start = v & 0x7fffffff; half_tile = (v < 0); }
      int lim = row_limit - start;
      if (half_tile) lim = min(lim, 64);
      // two S buffers: S(j) was computed before P(j-1) V_{j-1} was issued, so a rescale of O has to wait for that product
      if (!softmax_tile<DT, HDV>(t_s, t_o, scale_log2, kLeftWindow ? row_first - start : 0, lim,
                                 half_tile || start + kBlockN > warp_limit || (kLeftWindow && start < warp_first), j == 0, st,
                                 nullptr, (kTwoS && j > 0) ? smem_u32(pv_done) : 0u, static_cast<uint32_t>(j - 1) & 1u, &wctx)) {
        ok = false;
        break;
      }
      // Key rows of this tile that exist and are selected: the sequence may end inside the tile, and a half tile of a
      // tile list uses its first 64 keys only.  The other rows hold whatever lies there (the next sequence of a packed
      // batch, the rest of a page, keys the list left out, or nothing that was fetched).  Their P is zero, but
      // 0 * NaN would still poison O, so this thread clears V row `row` of the tile (after it has landed) before the
      // P V product may start, as the reference zero-fills out-of-range rows on load
      // (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:319).
      const int v_rows = min(sk - start, half_tile ? 64 : kBlockN);
      if (v_rows < kBlockN) {
        const int v_item = 2 * j + 1;
        if (!mbar_wait(smem_u32(&kv_full[v_item % kSlots]), (v_item / kSlots) & 1, wctx)) { ok = false; break; }
        if constexpr (VT) {
          // this thread owns d row `row` of the transposed tile: keys at or past the end are cleared, whole 16-byte
          // pieces (8 keys) where possible, element by element in the piece the end falls into
          const int lim_k = v_rows;
          const uint32_t vrow = ring_smem + (v_item % kSlots) * T::kTileBytes + row * 128;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const int k0 = c * 8;
            if (k0 + 8 <= lim_k) continue;
            const uint32_t addr = vrow + (c >> 3) * T::kHalfBytes + (((c & 7) ^ (row & 7)) << 4);
            uint32_t w[4] = {0u, 0u, 0u, 0u};
            if (k0 < lim_k) {
              asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int ka = k0 + 2 * e;
                w[e] = (ka < lim_k ? (w[e] & 0x0000ffffu) : 0u) | (ka + 1 < lim_k ? (w[e] & 0xffff0000u) : 0u);
              }
            }
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          }
        } else if (row >= v_rows) {
          const uint32_t vrow = ring_smem + (v_item % kSlots) * T::kTileBytes + row * 128;
#pragma unroll
          for (int hf = 0; hf < TV::kHalves; ++hf)
#pragma unroll
            for (int c16 = 0; c16 < 8; ++c16)
              asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(vrow + hf * T::kHalfBytes + c16 * 16), "r"(0u) : "memory");
        }
        fence_proxy_async_smem();
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&p_full[sp]));
    }
    if (ok && mbar_wait(smem_u32(o_full), 0, wctx)) {
      tc_fence_after();
      float vds = 1.f;
      if (p.v_descale) vds = p.v_descale[bidb * p.vds_b + hk * p.vds_h];
      float inv, lse_row;
      bool empty;
      finish_row(st.m_ref, st.l_sum, load_sink_log2(p.s_aux, p.s_aux_dtype, head), inv, lse_row, empty);
      inv *= vds;
      const int64_t grow = static_cast<int64_t>(q_row0) + row_in_seq;
      uint8_t* op = out_row_ptr(p, coord_b, grow, head);
#pragma unroll
      for (int c = 0; c < TV::kOChunks; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
        tmem_wait_ld();
        if (row < rows_valid) store_o_chunk(op, c, o, inv, p.out_dtype);
      }
      if (p.lse && row < rows_valid)
        p.lse[lse_index(p, bidb, head, grow, row_in_seq)] = lse_row;
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int DT, int HD = kHeadDim, int HDV = HD, bool VT = false>
cudaError_t launch_single_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const PrefillKernelParams& p, cudaStream_t stream) {
  const bool win = p.window_left >= 0;
  auto kern = win ? prefill_kernel<DT, true, HD, HDV, VT> : prefill_kernel<DT, false, HD, HDV, VT>;
  const size_t smem = 1024 + smem_layout<DT, HD>().total;
  static bool attr_done[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[win][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    attr_done[win][dev] = true;
  }
  dim3 grid(p.h, p.num_m_blocks, p.b);
  kern<<<grid, kThreads, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prefill_single(int dtype, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                  const PrefillKernelParams& p, cudaStream_t stream) {
  if (p.d != kHeadDim) {   // other head dimensions: 16-bit types
    const bool bf = dtype == FA_B200_BF16;
    if (dtype != FA_B200_BF16 && dtype != FA_B200_F16) return cudaErrorInvalidValue;
    switch (p.d) {
      case 64: return bf ? launch_single_t<FA_B200_BF16, 64>(tq, tk, tv, p, stream) : launch_single_t<FA_B200_F16, 64>(tq, tk, tv, p, stream);
      case 192:
        if (p.d_v == 128)
          return bf ? launch_single_t<FA_B200_BF16, 192, 128>(tq, tk, tv, p, stream) : launch_single_t<FA_B200_F16, 192, 128>(tq, tk, tv, p, stream);
        return bf ? launch_single_t<FA_B200_BF16, 192>(tq, tk, tv, p, stream) : launch_single_t<FA_B200_F16, 192>(tq, tk, tv, p, stream);
      case 256: return bf ? launch_single_t<FA_B200_BF16, 256>(tq, tk, tv, p, stream) : launch_single_t<FA_B200_F16, 256>(tq, tk, tv, p, stream);
    }
    return cudaErrorInvalidValue;
  }
  if (p.v_transposed) {
    if (dtype == FA_B200_BF16) return launch_single_t<FA_B200_BF16, kHeadDim, kHeadDim, true>(tq, tk, tv, p, stream);
    if (dtype == FA_B200_F16) return launch_single_t<FA_B200_F16, kHeadDim, kHeadDim, true>(tq, tk, tv, p, stream);
    return cudaErrorInvalidValue;
  }
  switch (dtype) {
    case FA_B200_F16: return launch_single_t<FA_B200_F16>(tq, tk, tv, p, stream);
    case FA_B200_BF16: return launch_single_t<FA_B200_BF16>(tq, tk, tv, p, stream);
    case FA_B200_E4M3: return launch_single_t<FA_B200_E4M3>(tq, tk, tv, p, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa
