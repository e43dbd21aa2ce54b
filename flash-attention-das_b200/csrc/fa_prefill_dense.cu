// Dense / varlen attention forward for sm_100a on tcgen05 tensor cores — persistent CTAs, score tile double-buffered.
//
// One CTA per SM walks work items (sequence, head, 128-row query block), heaviest query blocks first.  The score
// accumulator S is double-buffered in TMEM, so S(c+1) = Q K_{c+1}^T is issued BEFORE the softmax of tile c has
// finished: the tensor pipe computes the next scores (and the previous P V) while the softmax warps work, and the
// softmax warps find their next tile ready when they finish the current one.  Work crosses item boundaries the same
// way (the next item's Q tile follows in the same ring, its first S is issued before the current item's last
// P V).
//   warps 0-7   softmax: warpgroup g (warps 4g..4g+3) takes key columns 64g..64g+63 of every tile, thread = query
//               row; the threads of a row exchange their partial max through shared memory (one named barrier per
//               tile) and keep partial row sums.  (kSoftmaxWGs = 4, 32 columns per thread, measured slower.)
//   warp 8      TMA producer: one ring of 6 tiles carries Q, K_0, V_0, K_1, V_1, ... of item after item
//               (128B swizzle, no multicast)
//   warp 9      MMA issuer 1 (one thread): per item: Q tile shared memory -> TMEM (tcgen05.cp); per tile
//               S[c&1] = Q K_c^T, running up to two tiles ahead of the softmax
//   warp 10     MMA issuer 2 (one thread): O += P_c V_c.  Both products take their A operand (Q, P_c) from TMEM and
//               only K / V from shared memory.
//   warp 11     idle
// TMEM: S0 [0,128), S1 [128,256), O [256,384), Q of even items [384,448), Q of odd items [448,512).
// P (input dtype) overwrites the head of its S buffer.
// O in TMEM is rescaled only when a row max grew by more than 2^8 (and only after the previous P V has completed).
// Every mbarrier wait is bounded; a CTA that gives up raises the device status word and leaves through the common
// teardown (TMEM is always released).
//
// Same math as the reference's dense forward (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:2818-3328, FP8
// 3330-3778; softmax.h:592-640,932-964); the heaviest-first order plays the role of the reference's reversed
// m_block launch order (flash_fwd_kernel.h:8684).
#include <type_traits>

#include "fa_prefill_common.cuh"

namespace fa {
namespace {

constexpr int kSlots = 6;         // ring of 32 KB (16 KB e4m3) tiles: Q, K_0, V_0, K_1, V_1, ... of item after item
constexpr int kSoftmaxWGs = 2;                    // warpgroups sharing a tile's key columns
constexpr int kCols = kBlockN / kSoftmaxWGs;      // key (and output) columns per softmax thread
constexpr int kIdSlots = 4;       // claimed work item indices handed from the producer to the other roles
constexpr int kIdReaders = 2 + 4 * kSoftmaxWGs;   // the two MMA issuers and every softmax warp read each index
constexpr int kSoftmaxWarps = 4 * kSoftmaxWGs;
constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1;   // kMmaWarp + 1: second MMA issuer
constexpr int kThreads = 32 * (kSoftmaxWarps + 4);
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256, kColQ = 384;

struct DenseSmem {
  int ring_off, bar_off, xch_off, misc_off, total;
};
template <int DT>
__host__ __device__ constexpr DenseSmem dense_smem() {
  using T = TileTraits<DT>;
  DenseSmem s{};
  s.ring_off = 0;
  s.bar_off = s.ring_off + kSlots * T::kTileBytes;
  // s_full[2] p_full[2] o_full o_empty ring_full[kSlots] ring_empty[kSlots]
  s.xch_off = s.bar_off + 8 * (6 + 2 * kSlots + 2 * kIdSlots);
  s.misc_off = s.xch_off + 4 * 2 * kSoftmaxWGs * 128;
  s.total = s.misc_off + 32;
  return s;
}

// Position in the tile ring: slot and the parity of that slot's current use.
struct RingPos {
  uint32_t slot, phase;
  __device__ __forceinline__ void advance(uint32_t n) {   // n <= kSlots
    slot += n;
    if (slot >= kSlots) { slot -= kSlots; phase ^= 1u; }
  }
};

struct Item {
  int bidb, head, hk, m0, rows_valid, q_row0, k_row0, sk, coord_b, n_tiles, causal_shift, tile0;
};

// Virtual item L -> geometry.  false: the item does not exist (query block past the end of its sequence).
__device__ __forceinline__ bool get_item(const PrefillKernelParams& p, int L, Item& it) {
  it.head = L % p.h;
  const int r = L / p.h;
  it.bidb = r % p.b;
  const int mrev = r / p.b;
  const int m_block = p.is_causal ? (p.num_m_blocks - 1 - mrev) : mrev;
  it.hk = it.head / (p.h / p.h_k);
  int sq;
  if (p.cu_seqlens_q) {
    it.q_row0 = p.cu_seqlens_q[it.bidb];
    sq = p.cu_seqlens_q[it.bidb + 1] - it.q_row0;
    it.k_row0 = p.paged ? 0 : p.cu_seqlens_k[it.bidb];
    it.sk = p.paged ? 0 : p.cu_seqlens_k[it.bidb + 1] - it.k_row0;
    it.coord_b = 0;
  } else {
    it.q_row0 = 0; it.k_row0 = 0; sq = p.seqlen_q; it.sk = p.seqlen_k; it.coord_b = it.bidb;
  }
  if (p.paged) {   // keys in a paged pool: their number comes with the block table, rows are addressed page by page
    it.k_row0 = 0;
    it.sk = p.seqused_k[it.bidb];
    if (p.max_keys > 0 && it.sk > p.max_keys) {   // longer than the block table row: cut and report
      it.sk = static_cast<int>(p.max_keys);
      atomicOr(p.status, 0x10000);
    }
  }
  it.m0 = m_block * kBlockM;
  if (it.m0 >= sq) return false;
  it.rows_valid = min(kBlockM, sq - it.m0);
  it.causal_shift = it.sk - sq;
  key_tile_range(p, it.m0, it.rows_valid, it.sk, it.causal_shift, it.tile0, it.n_tiles);
  return true;
}


__device__ __forceinline__ void softmax_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kSoftmaxWarps) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1)
prefill_dense_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const PrefillKernelParams p) {
  using T = TileTraits<DT>;
  constexpr DenseSmem L = dense_smem<DT>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint64_t* s_full = bars;              // [2]  S buffer holds fresh scores          (tcgen05.commit)
  uint64_t* p_full = s_full + 2;        // [2]  P written, O rescaled if needed       (8 softmax warps)
  uint64_t* o_full = p_full + 2;        //      last P V of the item complete         (tcgen05.commit)
  uint64_t* o_empty = o_full + 1;       //      epilogue has read O                   (8 softmax warps)
  uint64_t* ring_full = o_empty + 1;    // [kSlots] tile landed                       (TMA transaction bytes)
  uint64_t* ring_empty = ring_full + kSlots;  // [kSlots] tile consumed: Q after its copy to TMEM and V after its P V
                                        //      (tcgen05.commit), K after its scores are complete (a softmax thread)
  uint64_t* id_full = ring_empty + kSlots;    // [kIdSlots] a claimed item index is published     (the producer)
  uint64_t* id_empty = id_full + kIdSlots;    // [kIdSlots] every reader has taken it
  int* id_ring = reinterpret_cast<int*>(smem + L.misc_off + 12);   // [kIdSlots]
  float* xch = reinterpret_cast<float*>(smem + L.xch_off);   // [2 parity][kSoftmaxWGs column groups][128 rows]
  uint32_t* sm_tmem_base = reinterpret_cast<uint32_t*>(smem + L.misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc_off + 8);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = p.h * p.b * p.num_m_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&s_full[t]), 1);
      mbar_init(smem_u32(&p_full[t]), kSoftmaxWarps);     // one elected lane per softmax warp
    }
    mbar_init(smem_u32(o_full), 1);
    mbar_init(smem_u32(o_empty), kSoftmaxWarps);
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(smem_u32(&ring_full[s]), 1);
      mbar_init(smem_u32(&ring_empty[s]), 1);
    }
    for (int s = 0; s < kIdSlots; ++s) {
      mbar_init(smem_u32(&id_full[s]), 1);
      mbar_init(smem_u32(&id_empty[s]), kIdReaders);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(sm_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm_tmem_base;
  const uint32_t ring_smem = smem_u32(smem + L.ring_off);

  // Work items are claimed in order from a global counter by the producer (a fixed stride over the item grid leaves the
  // CTAs of a varlen batch unevenly loaded) and their indices handed to the other roles through a small ring; -1 ends
  // the stream.  `take` returns the idx-th index of the stream (-2 if the wait gave up); one thread per reader releases.
  auto take = [&](uint32_t idx, bool release) -> int {
    const uint32_t slot = idx % kIdSlots;
    if (!mbar_wait(smem_u32(&id_full[slot]), (idx / kIdSlots) & 1u, wctx)) return -2;
    const int v = *reinterpret_cast<volatile int*>(&id_ring[slot]);
    if (release) mbar_arrive(smem_u32(&id_empty[slot]));
    return v;
  };

  if (warp == kProducerWarp) {
    // ================================================================== TMA producer
    if (lane == 0) {
      RingPos pos{0, 0};
      bool ok = true;
      // next ring tile: rows [row0, row0 + 128) of head `head` of tensor `tm`
      auto load_tile = [&](const CUtensorMap* tm, int head, int row0, int coord_b) -> bool {
        if (!mbar_wait(smem_u32(&ring_empty[pos.slot]), pos.phase ^ 1u, wctx)) return false;
        const uint32_t bar = smem_u32(&ring_full[pos.slot]);
        mbar_expect_tx(bar, T::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < T::kHalves; ++hf)
          tma_load_4d(ring_smem + pos.slot * T::kTileBytes + hf * T::kHalfBytes, tm, bar, hf * 64, head, row0, coord_b);
        pos.advance(1);
        return true;
      };
      // the same for a K or V tile whose 128 keys lie in a paged pool: one box of box_rows rows per page piece through
      // the block table; boxes that start past the end of the sequence are not fetched (their table slots are not
      // valid) and the softmax warps clear what the tile holds there
      auto load_paged_tile = [&](const CUtensorMap* tm, const Item& it, int start) -> bool {
        if (!mbar_wait(smem_u32(&ring_empty[pos.slot]), pos.phase ^ 1u, wctx)) return false;
        const uint32_t bar = smem_u32(&ring_full[pos.slot]);
        const int nbox = min(kBlockN / p.box_rows, (it.sk - start + p.box_rows - 1) / p.box_rows);
        mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * p.box_rows * 128u * T::kHalves);
        const int32_t* bt = p.block_table + static_cast<int64_t>(it.bidb) * p.bt_stride;
        for (int i = 0; i < nbox; ++i) {
          const int tok = start + i * p.box_rows;
          const int page = bt[tok / p.page_size], prow = tok % p.page_size;
#pragma unroll
          for (int hf = 0; hf < T::kHalves; ++hf)
            tma_load_4d(ring_smem + pos.slot * T::kTileBytes + hf * T::kHalfBytes + i * p.box_rows * 128, tm, bar, hf * 64, it.hk,
                        prow, page);
        }
        pos.advance(1);
        return true;
      };
      uint32_t pub = 0;
      auto publish = [&](int v) -> bool {
        const uint32_t slot = pub % kIdSlots;
        if (!mbar_wait(smem_u32(&id_empty[slot]), ((pub / kIdSlots) & 1u) ^ 1u, wctx)) return false;
        id_ring[slot] = v;
        mbar_arrive(smem_u32(&id_full[slot]));
        ++pub;
        return true;
      };
      Item it;
      int li = blockIdx.x;
      int li_next = static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);   // claimed one item ahead
      for (; ok && li < total_items; li = li_next, li_next = static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1)) {
        if (!get_item(p, li, it)) continue;
        if (!publish(li)) { ok = false; break; }
        if (it.n_tiles == 0) continue;
        ok = load_tile(&tmap_q, it.head, it.q_row0 + it.m0, it.coord_b);
        for (int j = 0; ok && j < it.n_tiles; ++j) {
          if (p.paged)
            ok = load_paged_tile(&tmap_k, it, (it.tile0 + j) * kBlockN) && load_paged_tile(&tmap_v, it, (it.tile0 + j) * kBlockN);
          else
            ok = load_tile(&tmap_k, it.hk, it.k_row0 + (it.tile0 + j) * kBlockN, it.coord_b) &&
                 load_tile(&tmap_v, it.hk, it.k_row0 + (it.tile0 + j) * kBlockN, it.coord_b);
        }
      }
      if (ok) publish(-1);
    }
  } else if (warp == kMmaWarp) {
    // ================================================================== MMA issuer 1: Q staging and S = Q K^T
    // The tensor pipe is fed by two threads in two warps (this one and the P V issuer below).  Issuing a product
    // holds its thread for about as long as the product runs, so with a single issuer every mbarrier wait and commit
    // between two products is a hole in the pipe; with two, one thread waits while the other one issues.
    if (lane == 0) {
      uint32_t c_next = 0, item_cnt = 0;
      RingPos qk_pos{0, 0};     // next tile this stream takes from the ring (a Q tile or a K tile)
      RingPos v_m2{0, 0}, v_m1{0, 0};   // V tiles of the two tiles before the one being issued
      [[maybe_unused]] int tr = 0;
      bool ok = true;
      Item it;
      for (uint32_t idx = 0; ok; ++idx) {
        const int li = take(idx, true);
        if (li < 0) { ok = (li == -1); break; }
        get_item(p, li, it);
        if (it.n_tiles == 0) continue;
        // item's Q: ring -> TMEM.  The copy runs in issue order with this thread's MMAs, so it cannot overtake the
        // Q K^T products of the item before last, which read the same TMEM columns.
        const uint32_t q_tmem = tmem_base + kColQ + (item_cnt & 1u) * 64;
        if (!mbar_wait(smem_u32(&ring_full[qk_pos.slot]), qk_pos.phase, wctx)) { ok = false; break; }
        tc_fence_after();
        issue_q_to_tmem<DT>(ring_smem + qk_pos.slot * T::kTileBytes, q_tmem);
        tc_commit(smem_u32(&ring_empty[qk_pos.slot]));
        qk_pos.advance(1);
        for (int j = 0; j < it.n_tiles; ++j) {
          FA_TRACE(2, tr, 1);
          // S[c_next & 1] still holds P of tile c_next - 2 until that tile's P V has completed (it then releases
          // its V tile)
          if (c_next >= 2 && !mbar_wait(smem_u32(&ring_empty[v_m2.slot]), v_m2.phase, wctx)) { ok = false; break; }
          v_m2 = v_m1;
          v_m1 = qk_pos;
          v_m1.advance(1);                             // V_j sits right behind K_j in the ring
          if (!mbar_wait(smem_u32(&ring_full[qk_pos.slot]), qk_pos.phase, wctx)) { ok = false; break; }
          tc_fence_after();
          FA_TRACE(2, tr, 3);
          issue_qk_ts<DT>(q_tmem, ring_smem + qk_pos.slot * T::kTileBytes, tmem_base + kColS + (c_next & 1u) * 128);
          FA_TRACE(2, tr, 4);
          tc_commit(smem_u32(&s_full[c_next & 1u]));   // the K slot itself is released by the softmax warps
          qk_pos.advance(2);                           // K_{j+1}, or the next item's Q after K_{n-1}
          ++c_next;
        }
        ++item_cnt;
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp + 1) {
    // ================================================================== MMA issuer 2: O (+)= P V
    if (lane == 0) {
      uint32_t c = 0, item_cnt = 0;
      RingPos v_pos{2, 0};      // ring: Q K_0 [V_0] K_1 V_1 ...
      [[maybe_unused]] int tr = 600;
      bool ok = true;
      Item it;
      for (uint32_t idx = 0; ok; ++idx) {
        const int li = take(idx, true);
        if (li < 0) { ok = (li == -1); break; }
        get_item(p, li, it);
        if (it.n_tiles == 0) continue;
        const int n = it.n_tiles;
        for (int j = 0; j < n; ++j) {
          FA_TRACE(2, tr, 10);
          if (!mbar_wait(smem_u32(&p_full[c & 1u]), (c >> 1) & 1u, wctx)) { ok = false; break; }
          // O still holds the previous item's result until its epilogue has read it
          if (j == 0 && !mbar_wait(smem_u32(o_empty), (item_cnt & 1u) ^ 1u, wctx)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&ring_full[v_pos.slot]), v_pos.phase, wctx)) { ok = false; break; }
          tc_fence_after();
          FA_TRACE(2, tr, 25);
          issue_pv<DT>(tmem_base + kColS + (c & 1u) * 128, ring_smem + v_pos.slot * T::kTileBytes, tmem_base + kColO, j == 0);
          FA_TRACE(2, tr, 28);
          tc_commit(smem_u32(&ring_empty[v_pos.slot]));
          if (j + 1 == n) tc_commit(smem_u32(o_full));
          v_pos.advance(j + 1 == n ? 3 : 2);    // next V: two tiles on, or three across an item boundary (Q, K_0)
          ++c;
        }
        ++item_cnt;
      }
    }
    __syncwarp();
  } else if (warp < kSoftmaxWarps) {
    // ================================================================== softmax / correction / epilogue
    const int wg = warp >> 2;             // which kCols key columns of every tile (and which output columns)
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(lane_grp * 32) << 16;
    const uint32_t t_o = tmem_base + lane_off + kColO + wg * kCols;    // this thread's accumulator columns
    uint32_t c = 0, item_cnt = 0, xpar = 0;
    RingPos k_pos{1, 0};      // K tile whose scores are awaited next (ring: Q K_0 V_0 K_1 V_1 ... Q K_0 ...)
    RingPos v_prev{0, 0};     // V tile of the previous P V (valid from the second tile of an item on)
    RingPos v_pos{2, 0};      // V tile of this tile's P V
    const bool releaser = (warp == 0 && lane == 0);
    [[maybe_unused]] int tr = 0;
    [[maybe_unused]] const bool tracer = (lane == 0 && warp == 0);
    bool ok = true;
    // A wait that gives up sets ok = false but the loops keep their shape (the named barriers below are not
    // bounded, so every softmax thread must reach each of them); results are discarded.
    for (uint32_t idx = 0;; ++idx) {
      const int li = take(idx, false);
      __syncwarp();
      if (lane == 0 && li != -2) mbar_arrive(smem_u32(&id_empty[idx % kIdSlots]));
      if (li < 0) break;
      Item it;
      get_item(p, li, it);
      const int row_in_seq = it.m0 + row;
      const int64_t grow = static_cast<int64_t>(it.q_row0) + row_in_seq;
      if (it.n_tiles == 0) {
        if (row < it.rows_valid) {
          uint8_t* op = out_row_ptr(p, it.coord_b, grow, it.head) + wg * (kCols * 2);
          const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < kCols / 8; ++i) reinterpret_cast<uint4*>(op)[i] = z;
          if (wg == 0 && p.lse)
            p.lse[lse_index(p, it.bidb, it.head, grow, row_in_seq)] =
                p.s_aux ? load_sink_log2(p.s_aux, p.s_aux_dtype, it.head) * kLn2 : INFINITY;   // only the sink, if any
        }
        continue;
      }
      // visible keys of this row [row_first, row_limit) and the warp-uniform bounds that decide whether a tile needs
      // masking at all
      const int row_limit = row_hi(p, row_in_seq, it.sk, it.causal_shift);
      const int warp_limit = row_hi(p, it.m0 + lane_grp * 32, it.sk, it.causal_shift);
      const int row_first = row_lo(p, row_in_seq, it.causal_shift);
      const int warp_first = row_lo(p, it.m0 + lane_grp * 32 + 31, it.causal_shift);
      float scale_log2 = p.scale_log2;
      if (p.q_descale) scale_log2 *= p.q_descale[it.bidb * p.qds_b + it.hk * p.qds_h];
      if (p.k_descale) scale_log2 *= p.k_descale[it.bidb * p.kds_b + it.hk * p.kds_h];
      float m_ref = -INFINITY, l_part = 0.f;
      for (int j = 0; j < it.n_tiles; ++j) {
        const uint32_t b = c & 1u;
        if (tracer) FA_TRACE(0, tr, 1);
        if (!mbar_wait(smem_u32(&s_full[b]), (c >> 1) & 1u, wctx)) ok = false;
        tc_fence_after();
        if (tracer) FA_TRACE(0, tr, 2);
        // the scores are complete, so the K tile they were computed from may be refilled
        if (releaser) mbar_arrive(smem_u32(&ring_empty[k_pos.slot]));
        k_pos.advance(j + 1 == it.n_tiles ? 3 : 2);
        const uint32_t t_s = tmem_base + lane_off + kColS + b * 128 + wg * kCols;
        uint32_t u[kCols / 32][32];
#pragma unroll
        for (int h2 = 0; h2 < kCols / 32; ++h2) tmem_ld_32x32(t_s + h2 * 32, u[h2]);
        tmem_wait_ld();
#define FA_S_AT(idx) __uint_as_float(u[(idx) >> 5][(idx) & 31])
        const int col0 = (it.tile0 + j) * kBlockN + wg * kCols;
        const bool masked_tile = col0 + kCols > warp_limit || col0 < warp_first;   // warp-uniform
        if (masked_tile) {
          const int lim = row_limit - col0, lo = row_first - col0;
#pragma unroll
          for (int i = 0; i < kCols; ++i) u[i >> 5][i & 31] = (i < lim && i >= lo) ? u[i >> 5][i & 31] : 0xff800000u;
        }
        float mx0 = fmaxf(FA_S_AT(0), FA_S_AT(1)), mx1 = fmaxf(FA_S_AT(2), FA_S_AT(3));
        float mx2 = fmaxf(FA_S_AT(4), FA_S_AT(5)), mx3 = fmaxf(FA_S_AT(6), FA_S_AT(7));
#pragma unroll
        for (int i = 8; i < kCols; i += 8) {
          mx0 = max3(mx0, FA_S_AT(i), FA_S_AT(i + 1));
          mx1 = max3(mx1, FA_S_AT(i + 2), FA_S_AT(i + 3));
          mx2 = max3(mx2, FA_S_AT(i + 4), FA_S_AT(i + 5));
          mx3 = max3(mx3, FA_S_AT(i + 6), FA_S_AT(i + 7));
        }
        float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // the other column groups of the row: exchange partial maxima.  After this barrier every thread of the row
        // has also finished READING its scores, so P may overwrite the head of the S buffer.
        float* xc = xch + (xpar * kSoftmaxWGs) * 128;
        xc[wg * 128 + row] = mx;
        if (tracer) FA_TRACE(0, tr, 7);
        softmax_bar_sync();
        if (tracer) FA_TRACE(0, tr, 8);
#pragma unroll
        for (int w = 0; w < kSoftmaxWGs; ++w) mx = fmaxf(mx, xc[w * 128 + row]);
        xpar ^= 1u;
        const float mx_scaled = mx * scale_log2;   // scale > 0
        if (j == 0) {
          m_ref = mx_scaled;
        } else {
          const bool grow_max = mx_scaled > m_ref + kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow_max)) {
            const float m_new = grow_max ? mx_scaled : m_ref;
            const float alpha = grow_max ? fast_exp2(m_ref - m_new) : 1.f;   // m_ref = -inf -> 0
            l_part *= alpha;
            m_ref = m_new;
            // O is being accumulated by the previous tile's P V until that product releases its V tile
            if (!mbar_wait(smem_u32(&ring_empty[v_prev.slot]), v_prev.phase, wctx)) ok = false;
            tc_fence_after();
#pragma unroll
            for (int h2 = 0; h2 < kCols / 32; ++h2) {
              uint32_t o[32];
              tmem_ld_32x32(t_o + h2 * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_32x32(t_o + h2 * 32, o);
            }
          }
        }
        const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
        float rs0 = 0.f, rs1 = 0.f;
        // P = 2^(S * scale - m) in the input dtype, written over the head of the S buffer.
        auto exp_store = [&]() {
          if constexpr (!T::kFp8) {
            const uint32_t t_p = tmem_base + lane_off + kColS + b * 128 + wg * (kCols / 2);
#pragma unroll
            for (int h2 = 0; h2 < kCols / 32; ++h2) {
              uint32_t pk[16];
              const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(-m_safe, -m_safe);
              uint64_t rs2 = pack_f32x2(0.f, 0.f);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                float x0, x1;
                unpack_f32x2(fma_f32x2(pack_f32x2(FA_S_AT(h2 * 32 + 2 * i), FA_S_AT(h2 * 32 + 2 * i + 1)), sc2, nm2), x0, x1);
                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                rs2 = add_f32x2(rs2, pack_f32x2(p0, p1));
                pk[i] = pack2(p0, p1, DT);
              }
              float r0, r1;
              unpack_f32x2(rs2, r0, r1);
              rs0 += r0;
              rs1 += r1;
              tmem_st_32x16(t_p + h2 * 16, pk);
            }
          } else {
            const uint32_t t_p = tmem_base + lane_off + kColS + b * 128 + wg * (kCols / 4);
            // as softmax_tile: packed arithmetic, a quarter of the exponentials on the FMA pipe
            const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(-m_safe, -m_safe);
            uint64_t rs2 = pack_f32x2(0.f, 0.f);
#pragma unroll
            for (int h2 = 0; h2 < kCols / 32; ++h2) {
              uint32_t pk[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float p0, p1, p2, p3;
                if (((i + 1) * kFp8PolyGroups) / 8 > (i * kFp8PolyGroups) / 8) {
                  exp2_poly_x2(FA_S_AT(h2 * 32 + 4 * i), FA_S_AT(h2 * 32 + 4 * i + 1), sc2, nm2, p0, p1);
                  exp2_poly_x2(FA_S_AT(h2 * 32 + 4 * i + 2), FA_S_AT(h2 * 32 + 4 * i + 3), sc2, nm2, p2, p3);
                } else {
                  float x0, x1, x2, x3;
                  unpack_f32x2(fma_f32x2(pack_f32x2(FA_S_AT(h2 * 32 + 4 * i), FA_S_AT(h2 * 32 + 4 * i + 1)), sc2, nm2), x0, x1);
                  unpack_f32x2(fma_f32x2(pack_f32x2(FA_S_AT(h2 * 32 + 4 * i + 2), FA_S_AT(h2 * 32 + 4 * i + 3)), sc2, nm2), x2, x3);
                  p0 = fast_exp2(x0);
                  p1 = fast_exp2(x1);
                  p2 = fast_exp2(x2);
                  p3 = fast_exp2(x3);
                }
                rs2 = add_f32x2(rs2, add_f32x2(pack_f32x2(p0, p1), pack_f32x2(p2, p3)));
                pk[i] = pack4_e4m3(p0, p1, p2, p3);
              }
              tmem_st_32x8(t_p + h2 * 8, pk);
            }
            float r0, r1;
            unpack_f32x2(rs2, r0, r1);
            rs0 += r0;
            rs1 += r1;
          }
        };
        exp_store();
#undef FA_S_AT
        l_part += rs0 + rs1;
        if (j + 1 == it.n_tiles) {
          // Last tile of the sweep: if the sequence ends inside it, the key rows past the end hold the next sequence of
          // a packed batch (or nothing).  Their P is zero, but 0 * NaN would still poison O: the first column group's
          // thread of each row clears V row `row` of the tile (after it has landed) before this tile's P V product may
          // start (every softmax warp arrives on p_full below), as the reference zero-fills out-of-range rows on load
          // (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:319).
          const int lim_k = it.sk - (it.tile0 + j) * kBlockN;
          if (lim_k < kBlockN && wg == 0) {
            if (!mbar_wait(smem_u32(&ring_full[v_pos.slot]), v_pos.phase, wctx)) ok = false;
            if (ok && row >= lim_k) {
              const uint32_t vrow = ring_smem + v_pos.slot * T::kTileBytes + row * 128;
#pragma unroll
              for (int hf = 0; hf < T::kHalves; ++hf)
#pragma unroll
                for (int c16 = 0; c16 < 8; ++c16)
                  asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(vrow + hf * T::kHalfBytes + c16 * 16), "r"(0u) : "memory");
            }
            fence_proxy_async_smem();
          }
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&p_full[b]));
        if (tracer) FA_TRACE(0, tr, 4);
        v_prev = v_pos;
        v_pos.advance(j + 1 == it.n_tiles ? 3 : 2);
        ++c;
      }
      // ---- epilogue of this item: this thread owns output columns [kCols wg, kCols wg + kCols) of its row
      if (!mbar_wait(smem_u32(o_full), item_cnt & 1u, wctx)) ok = false;
      tc_fence_after();
      uint32_t o[kCols / 32][32];
#pragma unroll
      for (int h2 = 0; h2 < kCols / 32; ++h2) tmem_ld_32x32(t_o + h2 * 32, o[h2]);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(o_empty));   // O may be overwritten by the next item from here on
      ++item_cnt;
      // total row sum = the column groups' partial sums (same reference max)
      float* xc = xch + (xpar * kSoftmaxWGs) * 128;
      xc[wg * 128 + row] = l_part;
      softmax_bar_sync();
      float l_sum = 0.f;
#pragma unroll
      for (int w = 0; w < kSoftmaxWGs; ++w) l_sum += xc[w * 128 + row];
      xpar ^= 1u;
      if (ok && row < it.rows_valid) {
        float vds = 1.f;
        if (p.v_descale) vds = p.v_descale[it.bidb * p.vds_b + it.hk * p.vds_h];
        float inv, lse_row;
        bool empty;
        finish_row(m_ref, l_sum, load_sink_log2(p.s_aux, p.s_aux_dtype, it.head), inv, lse_row, empty);
        inv *= vds;
        uint8_t* op = out_row_ptr(p, it.coord_b, grow, it.head) + wg * (kCols * 2);
#pragma unroll
        for (int h2 = 0; h2 < kCols / 32; ++h2) store_o_chunk(op, h2, o[h2], inv, p.out_dtype);
        if (wg == 0 && p.lse)
          p.lse[lse_index(p, it.bidb, it.head, grow, row_in_seq)] = lse_row;
      }
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

template <int DT>
cudaError_t launch_dense_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const PrefillKernelParams& p, cudaStream_t stream) {
  auto kern = prefill_dense_kernel<DT>;
  const size_t smem = 1024 + dense_smem<DT>().total;
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
  const long long total = static_cast<long long>(p.h) * p.b * p.num_m_blocks;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms[dev] ? total : num_sms[dev]);
  if (!p.work_counter) return cudaErrorInvalidValue;
  kern<<<grid, kThreads, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace

#ifdef FA_B200_PHASE_TRACE
extern "C" __attribute__((visibility("default"))) int fa_b200_debug_trace_dense(long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace)));
}
#endif

cudaError_t launch_prefill_dense(int dtype, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                 const PrefillKernelParams& p, cudaStream_t stream) {
  switch (dtype) {
    case FA_B200_F16: return launch_dense_t<FA_B200_F16>(tq, tk, tv, p, stream);
    case FA_B200_BF16: return launch_dense_t<FA_B200_BF16>(tq, tk, tv, p, stream);
    case FA_B200_E4M3: return launch_dense_t<FA_B200_E4M3>(tq, tk, tv, p, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa
