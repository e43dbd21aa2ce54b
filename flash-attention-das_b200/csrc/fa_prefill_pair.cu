// Dense / varlen GQA attention forward for sm_100a on tcgen05 tensor cores — persistent CTAs, two query tiles each.
//
// One CTA per SM.  A work item is (sequence, 128-row query block, PAIR of query heads of one GQA group): the two
// heads see the same keys under the same mask, so every K/V tile is loaded once and used by both
// (half the L2->SM traffic of one-tile CTAs), and while one tile's softmax runs the tensor pipe works on the other:
//   warps 0-3     softmax + epilogue of tile 0 (one thread per query row)
//   warps 4-7     softmax + epilogue of tile 1
//   warp 8        TMA producer: Q_0, Q_1 per item; K_j, V_j tiles into a four-slot ring, running ahead across items
//   warps 9, 10   MMA issuers of tile 0 and tile 1 (one thread each), per key tile j and under a common lock:
//                 O_t += P_t V_j,  S_t = Q_t K_{j+1}^T
//   warp 11       idle (completes the third warpgroup so that it can hand its registers to the softmax warps)
// TMEM (all 512 columns): S_0, S_1, O_0, O_1 of 128 fp32 columns each; P overwrites the head of S.
// CTAs claim their items from the virtual item list ordered by descending query block (for causal masks: heaviest
// first), so prologue, Q loads and epilogue of one item overlap the main loop of its neighbours.  K/V may live in a
// paged pool (kPaged build): the producer then fetches every key tile page piece by page piece through the block
// table.  In every build the softmax warpgroups clear the V rows past the end of the sequence in its last tile, so that
// what lies behind a sequence (the next one of a packed batch, the rest of a page) cannot reach the output.  All mbarrier phases simply
// keep counting across items.  Every wait is bounded; a CTA that gives up raises the device status word and leaves
// through the common teardown (TMEM is always released).
//
// Same math as the reference's dense forward (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:2818-3328, FP8
// 3330-3778; softmax.h:592-640,932-964); the heaviest-first order plays the role of the reference's reversed
// m_block launch order (flash_fwd_kernel.h:8684).
#include "fa_prefill_common.cuh"

namespace fa {
namespace {

constexpr int kSlots = 4;
constexpr int kThreads = 32 * 12;
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kTmemCols = 512;
constexpr int kSoftmaxRegs = 232, kOtherRegs = 40;
// setmaxnreg.inc waits (without a limit) until the CTA's pool holds enough registers, and the pool is what the CTA got
// at launch: 168 registers (the cap of a 384-thread CTA) for each of its threads.  A split that asks for more never
// gets it and the kernel hangs.
static_assert(128 * (2 * kSoftmaxRegs + kOtherRegs) <= 168 * kThreads, "register split exceeds the CTA's allocation");

constexpr int kStageBytes = 128 * 128;   // output staging per tile: 128 rows x 64 columns of a 16-bit type
constexpr int kItemSlots = 4;            // work items published by the producer for the other roles
constexpr int kItemReaders = 10;         // eight softmax warps and the two MMA issuers take a copy of every item
struct PairSmem {
  int q_off, ring_off, stage_off, bar_off, item_off, misc_off, total;
};
template <int DT>
__host__ __device__ constexpr PairSmem pair_smem() {
  using T = TileTraits<DT>;
  PairSmem s{};
  s.q_off = 0;
  s.ring_off = 2 * T::kTileBytes;
  s.stage_off = s.ring_off + kSlots * T::kTileBytes;
  s.bar_off = s.stage_off + 2 * kStageBytes;
  s.item_off = s.bar_off + 8 * (12 + 2 * kSlots + 2 * kItemSlots);
  s.misc_off = s.item_off + kItemSlots * 64;
  s.total = s.misc_off + 32;
  return s;
}

// n_tiles < 0 marks the end of the CTA's work in the published item stream.
struct Item {
  int bidb, head0, hk, m0, rows_valid, q_row0, k_row0, sk, coord_b, n_tiles, causal_shift, tile0;
};
static_assert(sizeof(Item) == 48, "Item is copied through shared memory as three 16-byte words");

// Virtual item L -> geometry.  false: the item does not exist (query block past the end of its sequence).
__device__ __forceinline__ bool get_item(const PrefillKernelParams& p, int L, Item& it) {
  const int hp = p.h >> 1;
  const int x = L % hp;
  const int r = L / hp;
  it.bidb = r % p.b;
  const int mrev = r / p.b;
  const int m_block = p.is_causal ? (p.num_m_blocks - 1 - mrev) : mrev;
  it.head0 = 2 * x;
  it.hk = it.head0 / (p.h / p.h_k);
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

// kLeftWindow: the launch has a left sliding-window bound (kept out of the common build of the hot loop: two more live
// values per softmax thread are enough to make it spill).
// kPaged: K/V are read through a block table (its own build, so that the common one carries none of its state).
// kVT (with kPaged, 16-bit types): the V pool is stored transposed, tokens contiguous: a V tile lands as 128 d rows of
// 128 keys and enters the P V product as a K-major operand (issue_pv_vt).
template <int DT, bool kLeftWindow, bool kPaged, bool kVT = false>
__global__ void __launch_bounds__(kThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                    const PrefillKernelParams p) {
  using T = TileTraits<DT>;
  static_assert(!kVT || (kPaged && !T::kFp8), "transposed V: paged pools of a 16-bit type");
  constexpr PairSmem L = pair_smem<DT>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  uint64_t* q_full = bars;            // [2]
  uint64_t* q_empty = q_full + 2;     // [2]
  uint64_t* s_full = q_empty + 2;     // [2]
  uint64_t* p_full = s_full + 2;      // [2]
  uint64_t* o_full = p_full + 2;      // [2]
  uint64_t* o_empty = o_full + 2;     // [2]
  uint64_t* kv_full = o_empty + 2;    // [kSlots]
  uint64_t* kv_empty = kv_full + kSlots;
  uint64_t* item_full = kv_empty + kSlots;      // [kItemSlots]
  uint64_t* item_empty = item_full + kItemSlots;
  uint32_t* sm_tmem_base = reinterpret_cast<uint32_t*>(smem + L.misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc_off + 8);
  int* issue_lock = reinterpret_cast<int*>(smem + L.misc_off + 12);   // held while one tile's MMA group is issued
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = (p.h >> 1) * p.b * p.num_m_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *issue_lock = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&q_full[t]), 1);
      mbar_init(smem_u32(&q_empty[t]), 1);
      mbar_init(smem_u32(&s_full[t]), 1);
      mbar_init(smem_u32(&p_full[t]), 128);
      mbar_init(smem_u32(&o_full[t]), 1);
      mbar_init(smem_u32(&o_empty[t]), 128);
    }
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 2);   // released by both tiles' MMA issuers
    }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(smem_u32(&item_full[s]), 1);
      mbar_init(smem_u32(&item_empty[s]), kItemReaders);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_o);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(sm_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm_tmem_base;
  // Register hand-over between warpgroups: the producer/MMA warpgroup keeps kOtherRegs registers per thread, each
  // softmax warpgroup (128 score registers per row live at once) grows to kSoftmaxRegs.
  const uint32_t q_smem = smem_u32(smem + L.q_off);
  const uint32_t ring_smem = smem_u32(smem + L.ring_off);
  const uint32_t stage_smem = smem_u32(smem + L.stage_off);

  // Work items: the producer works out each item's geometry once (integer divisions and cu_seqlens loads in rarely
  // executed code: thousands of cycles when every role repeats them at every item boundary) and publishes it in a small
  // shared-memory ring; the other roles take copies.
  auto item_slot = [&](uint32_t idx) { return reinterpret_cast<Item*>(smem + L.item_off + (idx % kItemSlots) * 64); };
  auto read_item = [&](uint32_t idx, Item& it) -> bool {
    if (!mbar_wait(smem_u32(&item_full[idx % kItemSlots]), (idx / kItemSlots) & 1u, wctx)) return false;
    const int4* src = reinterpret_cast<const int4*>(item_slot(idx));
    const int4 a = src[0], b = src[1], c = src[2];
    it.bidb = a.x; it.head0 = a.y; it.hk = a.z; it.m0 = a.w;
    it.rows_valid = b.x; it.q_row0 = b.y; it.k_row0 = b.z; it.sk = b.w;
    it.coord_b = c.x; it.n_tiles = c.y; it.causal_shift = c.z; it.tile0 = c.w;
    return true;
  };
  auto release_item = [&](uint32_t idx) { mbar_arrive(smem_u32(&item_empty[idx % kItemSlots])); };

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
  if (warp == kProducerWarp) {
    // ================================================================== TMA producer
    if (lane == 0) {
      uint32_t kv_cnt = 0, item_cnt = 0, pub = 0;
      bool ok = true;
      auto publish = [&](const Item& it) -> bool {
        const uint32_t slot = pub % kItemSlots;
        if (!mbar_wait(smem_u32(&item_empty[slot]), ((pub / kItemSlots) & 1u) ^ 1u, wctx)) return false;
        int4* dst = reinterpret_cast<int4*>(item_slot(pub));
        dst[0] = make_int4(it.bidb, it.head0, it.hk, it.m0);
        dst[1] = make_int4(it.rows_valid, it.q_row0, it.k_row0, it.sk);
        dst[2] = make_int4(it.coord_b, it.n_tiles, it.causal_shift, it.tile0);
        mbar_arrive(smem_u32(&item_full[slot]));
        ++pub;
        return true;
      };
      // Work items are claimed, not strided: the first one is the CTA's index, every further one comes from a global
      // counter (zeroed before the launch).  Items are ordered heaviest first and the sequences of a varlen batch leave
      // holes in the virtual item grid, so a fixed stride would leave some CTAs with 15 % more work than the average;
      // claiming in order keeps the CTAs within one light item of each other.  The next claim is issued one item
      // ahead, so that the atomic's round trip overlaps the loads of the current item.
      int li = blockIdx.x;
      int li_next = static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);
      for (; ok && li < total_items; li = li_next, li_next = static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1)) {
        Item it;
        if (!get_item(p, li, it)) continue;
        if (!publish(it)) { ok = false; break; }
        if (it.n_tiles == 0) continue;
        for (int t = 0; t < 2; ++t) {
          if (!mbar_wait(smem_u32(&q_empty[t]), (item_cnt & 1u) ^ 1u, wctx)) { ok = false; break; }
          const uint32_t bar = smem_u32(&q_full[t]);
          mbar_expect_tx(bar, T::kTileBytes);
#pragma unroll
          for (int hf = 0; hf < T::kHalves; ++hf)
            tma_load_4d(q_smem + t * T::kTileBytes + hf * T::kHalfBytes, &tmap_q, bar, hf * 64, it.head0 + t,
                        it.q_row0 + it.m0, it.coord_b);
        }
        for (int j = 0; ok && j < it.n_tiles; ++j) {
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const uint32_t slot = kv_cnt % kSlots, ph = (kv_cnt / kSlots) & 1u;
            if (!mbar_wait(smem_u32(&kv_empty[slot]), ph ^ 1u, wctx)) { ok = false; break; }
            const uint32_t bar = smem_u32(&kv_full[slot]);
            const CUtensorMap* tm = kv ? &tmap_v : &tmap_k;
            if constexpr (!kPaged) {
              mbar_expect_tx(bar, T::kTileBytes);
#ifdef FA_B200_TEST_HOOKS
              // failure-detection test: the bytes announced above never arrive, the MMA issuers' wait runs out
              if (p.test_withhold && kv_cnt == 0 && blockIdx.x == 0) { ++kv_cnt; continue; }
#endif
#pragma unroll
              for (int hf = 0; hf < T::kHalves; ++hf)
                tma_load_4d(ring_smem + slot * T::kTileBytes + hf * T::kHalfBytes, tm, bar, hf * 64, it.hk,
                            it.k_row0 + (it.tile0 + j) * kBlockN, it.coord_b);
            } else if (kVT && kv) {
              // transposed V pool: one box of 64 keys x 128 d rows per column group; groups that start past the end of
              // the sequence are not fetched
              const int start = (it.tile0 + j) * kBlockN;
              const int nbox = min(kBlockN / 64, (it.sk - start + 63) / 64);
              mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * T::kHalfBytes);
              const int32_t* bt = p.block_table + static_cast<int64_t>(it.bidb) * p.bt_stride;
              for (int i = 0; i < nbox; ++i) {
                const int tok = start + i * 64;
                tma_load_4d(ring_smem + slot * T::kTileBytes + i * T::kHalfBytes, tm, bar, tok % p.page_size, 0, it.hk,
                            bt[tok / p.page_size]);
              }
            } else {
              // the tile's 128 keys come from one or more pages: one box of box_rows rows per page piece; boxes that
              // start past the end of the sequence are not fetched (their block_table slots are not valid)
              const int start = (it.tile0 + j) * kBlockN;
              const int nbox = min(kBlockN / p.box_rows, (it.sk - start + p.box_rows - 1) / p.box_rows);
              mbar_expect_tx(bar, static_cast<uint32_t>(nbox) * p.box_rows * 128u * T::kHalves);
              const int32_t* bt = p.block_table + static_cast<int64_t>(it.bidb) * p.bt_stride;
              for (int i = 0; i < nbox; ++i) {
                const int tok = start + i * p.box_rows;
                const int page = bt[tok / p.page_size], prow = tok % p.page_size;
#pragma unroll
                for (int hf = 0; hf < T::kHalves; ++hf)
                  tma_load_4d(ring_smem + slot * T::kTileBytes + hf * T::kHalfBytes + i * p.box_rows * 128, tm, bar, hf * 64,
                              it.hk, prow, page);
              }
            }
            ++kv_cnt;
          }
        }
        ++item_cnt;
      }
      if (ok) {
        Item end{};
        end.n_tiles = -1;
        publish(end);
      }
    }
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ================================================================== MMA issuers: warp 9 feeds tile 0, warp 10 tile 1
    // One thread per tile.  Issuing a product holds its thread for about as long as the product runs, and every wait
    // or commit costs the issuing thread a few hundred cycles, so with a single issuer those are holes in the pipe.
    // With one issuer per tile, one thread waits and commits while the other one issues.  Each thread issues its
    // tile's group  O_t += P_t V_j ;  S_t = Q_t K_{j+1}^T  under a lock, so the groups of the two tiles never
    // interleave: S_0 and S_1 become ready a whole group apart, which keeps the two softmaxes out of phase (one runs
    // while the tensor pipe works for the other).  The pipe executes in issue order, so the overwrite of S_t / P_t
    // follows the P_t V read.  Each K/V slot is released by both issuers (empty barriers count two).
    if (lane == 0) {
      const int t = warp - kMmaWarp;
      const uint32_t t_s = tmem_base + t * 128, t_o = tmem_base + 256 + t * 128;
      const uint32_t q_t = q_smem + t * T::kTileBytes;
      uint32_t kv_cnt = 0, item_cnt = 0, sp_cnt = 0;
      [[maybe_unused]] int tr = t * 500;
      bool ok = true;
      auto lock = [&]() -> bool {
        uint32_t it = 0;
        while (atomicCAS(issue_lock, 0, 1) != 0) {
          if ((++it & 1023u) == 0u && *abort_flag) return false;
        }
        return true;
      };
      auto unlock = [&]() { __threadfence_block(); atomicExch(issue_lock, 0); };
      for (uint32_t idx = 0; ok; ++idx) {
        Item it;
        if (!read_item(idx, it)) { ok = false; break; }
        release_item(idx);
        if (it.n_tiles < 0) break;
        if (it.n_tiles == 0) continue;
        const int n = it.n_tiles;
        {  // S_t(0) = Q_t K_0^T
          const uint32_t slot = kv_cnt % kSlots;
          if (!mbar_wait(smem_u32(&kv_full[slot]), (kv_cnt / kSlots) & 1u, wctx)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&q_full[t]), item_cnt & 1u, wctx)) { ok = false; break; }
          tc_fence_after();
          if (!lock()) { ok = false; break; }
          issue_qk<DT>(q_t, ring_smem + slot * T::kTileBytes, t_s);
          tc_commit(smem_u32(&s_full[t]));
          unlock();
          tc_commit(smem_u32(&kv_empty[slot]));
          if (n == 1) tc_commit(smem_u32(&q_empty[t]));
          ++kv_cnt;
        }
        for (int j = 0; j < n; ++j) {
          const uint32_t vslot = kv_cnt % kSlots;
          const uint32_t kslot = (kv_cnt + 1) % kSlots;
          const bool more = (j + 1 < n);
          FA_TRACE(2, tr, 10 + t);
          // everything this group needs, before taking the lock
          if (!mbar_wait(smem_u32(&kv_full[vslot]), (kv_cnt / kSlots) & 1u, wctx)) { ok = false; break; }
          if (more && !mbar_wait(smem_u32(&kv_full[kslot]), ((kv_cnt + 1) / kSlots) & 1u, wctx)) { ok = false; break; }
          // O_t still holds the previous item's result until its epilogue has read it
          if (j == 0 && !mbar_wait(smem_u32(&o_empty[t]), (item_cnt & 1u) ^ 1u, wctx)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&p_full[t]), sp_cnt & 1u, wctx)) { ok = false; break; }
          tc_fence_after();
          FA_TRACE(2, tr, 20 + t);
          if (!lock()) { ok = false; break; }
          if constexpr (kVT) issue_pv_vt<DT>(t_s, ring_smem + vslot * T::kTileBytes, t_o, j == 0);
          else issue_pv<DT>(t_s, ring_smem + vslot * T::kTileBytes, t_o, j == 0);
          if (more) {
            issue_qk<DT>(q_t, ring_smem + kslot * T::kTileBytes, t_s);
            tc_commit(smem_u32(&s_full[t]));
          } else {
            tc_commit(smem_u32(&o_full[t]));
          }
          unlock();
          FA_TRACE(2, tr, 30 + t);
          tc_commit(smem_u32(&kv_empty[vslot]));
          if (more) {
            tc_commit(smem_u32(&kv_empty[kslot]));
            if (j + 2 == n) tc_commit(smem_u32(&q_empty[t]));
          }
          ++sp_cnt;
          kv_cnt += more ? 2u : 1u;
        }
        ++item_cnt;
      }
    }
    __syncwarp();
  }
  } else {
    // ================================================================== softmax / correction / epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int t = warp >> 2;
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    const uint32_t t_s = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + t * 128;
    const uint32_t t_o = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + 256 + t * 128;
    uint32_t sp_cnt = 0, item_cnt = 0;
    [[maybe_unused]] int tr = 0;
    [[maybe_unused]] const bool tracer = (lane == 0 && lane_grp == 0);
#ifdef FA_B200_PHASE_TRACE
    uint32_t prof[5] = {0, 0, 0, 0, 0};
#endif
    bool ok = true;
    for (uint32_t idx = 0; ok; ++idx) {
      // The item stays in its ring slot until the epilogue is done: the main loop keeps only what it needs in
      // registers (every register counts there) and the epilogue reads the rest again.
      if (!mbar_wait(smem_u32(&item_full[idx % kItemSlots]), (idx / kItemSlots) & 1u, wctx)) { ok = false; break; }
      const volatile Item* is = item_slot(idx);
      const int n_tiles = is->n_tiles;
      if (n_tiles < 0) break;
      if (n_tiles == 0) {
        Item it;
        read_item(idx, it);
        const int row_in_seq = it.m0 + row;
        if (row < it.rows_valid)
          store_empty_row(p, it.coord_b, it.bidb, it.head0 + t, static_cast<int64_t>(it.q_row0) + row_in_seq, row_in_seq);
        __syncwarp();
        if (lane == 0) release_item(idx);
        continue;
      }
      // this row's visible keys [row_first, row_limit) and, for the warp-uniform decision whether a tile needs masking
      // at all, the smallest limit and the largest first key among the warp's rows; all relative to the first tile
      int row_first, row_limit, warp_first, warp_limit;
      float scale_log2 = p.scale_log2;
      {
        const int sk = is->sk, m0 = is->m0, shift = is->causal_shift, base = is->tile0 * kBlockN;
        row_limit = row_hi(p, m0 + row, sk, shift) - base;
        warp_limit = row_hi(p, m0 + lane_grp * 32, sk, shift) - base;
        row_first = kLeftWindow ? row_lo(p, m0 + row, shift) - base : 0;
        warp_first = kLeftWindow ? row_lo(p, m0 + lane_grp * 32 + 31, shift) - base : 0;
        if (p.q_descale) scale_log2 *= p.q_descale[is->bidb * p.qds_b + is->hk * p.qds_h];
        if (p.k_descale) scale_log2 *= p.k_descale[is->bidb * p.kds_b + is->hk * p.kds_h];
      }
      RowState st{-INFINITY, 0.f};
      for (int j = 0; j < n_tiles; ++j) {
        if (tracer) FA_TRACE(t, tr, 1);
        if (!mbar_wait(smem_u32(&s_full[t]), sp_cnt & 1u, wctx)) { ok = false; break; }
        tc_fence_after();
        if (tracer) FA_TRACE(t, tr, 2);
        const int start = j * kBlockN;
#ifdef FA_B200_PHASE_TRACE
        softmax_tile<DT>(t_s, t_o, scale_log2, kLeftWindow ? row_first - start : 0, row_limit - start,
                         start + kBlockN > warp_limit || (kLeftWindow && start < warp_first), j == 0, st,
                         tracer ? prof : nullptr);
        if (tracer) ++prof[4];
#else
        softmax_tile<DT>(t_s, t_o, scale_log2, kLeftWindow ? row_first - start : 0, row_limit - start,
                         start + kBlockN > warp_limit || (kLeftWindow && start < warp_first), j == 0, st);
#endif
        if (tracer) FA_TRACE(t, tr, 3);
        if (j == n_tiles - 1) {
          // Last tile of the sweep: if the sequence ends inside it, the key rows past the end hold whatever lies there
          // (the next sequence of a packed batch, the rest of a page, or nothing that was fetched).  Their P is zero,
          // but 0 * NaN would still poison O, so this thread clears V row `row` of the tile (after it has landed)
          // before this tile's P V product may start, as the reference zero-fills out-of-range rows on load
          // (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:319).  Both softmax warpgroups do it (the two products read
          // the same V tile; writing zeros twice is harmless).  Key tile n of this CTA has its V in ring item 2 n + 1.
          const int lim_k = is->sk - (is->tile0 + j) * kBlockN;   // keys of this tile that exist
          if (lim_k < kBlockN) {
            const uint32_t v_item = 2 * sp_cnt + 1;
            if (!mbar_wait(smem_u32(&kv_full[v_item % kSlots]), (v_item / kSlots) & 1u, wctx)) { ok = false; break; }
            if constexpr (kVT) {
              // this thread owns d row `row` of the transposed tile: keys at or past the end are cleared, whole 16-byte
              // pieces (8 keys) where possible, element by element in the piece the end falls into
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
            } else if (row >= lim_k) {
              const uint32_t vrow = ring_smem + (v_item % kSlots) * T::kTileBytes + row * 128;
#pragma unroll
              for (int hf = 0; hf < T::kHalves; ++hf)
#pragma unroll
                for (int c16 = 0; c16 < 8; ++c16)
                  asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(vrow + hf * T::kHalfBytes + c16 * 16), "r"(0u) : "memory");
            }
            fence_proxy_async_smem();
          }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&p_full[t]));
        if (tracer) FA_TRACE(t, tr, 4);
        ++sp_cnt;
      }
      if (!ok) break;
      if (tracer) FA_TRACE(t, tr, 5);
      // while the last product runs: what does not need O
      Item it;
      read_item(idx, it);
      const int head = it.head0 + t;
      const int row_in_seq = it.m0 + row;
      const int64_t grow = static_cast<int64_t>(it.q_row0) + row_in_seq;
      float vds = 1.f;
      if (p.v_descale) vds = p.v_descale[it.bidb * p.vds_b + it.hk * p.vds_h];
      float inv, lse_row;
      bool empty;
      finish_row(st.m_ref, st.l_sum, load_sink_log2(p.s_aux, p.s_aux_dtype, head), inv, lse_row, empty);
      inv *= vds;
      if (row < it.rows_valid && p.lse) p.lse[lse_index(p, it.bidb, head, grow, row_in_seq)] = lse_row;
      if (!mbar_wait(smem_u32(&o_full[t]), item_cnt & 1u, wctx)) { ok = false; break; }
      tc_fence_after();
      if (tracer) FA_TRACE(t, tr, 6);
      if (p.o_tma && it.rows_valid == kBlockM) {
        // Whole tile: O goes out as two 64-column halves through a 16 KB staging buffer (128-byte rows, 16-byte
        // chunks XOR-swizzled by the row as the tensor map expects) and one tile store each: full 128-byte lines
        // instead of one 16-byte piece per row and instruction.
        const uint32_t stage = stage_smem + t * kStageBytes;
        const uint32_t my_row = stage + row * 128;
#pragma unroll 1
        for (int hd = 0; hd < 2; ++hd) {
          uint32_t o[2][32];
          tmem_ld_32x32(t_o + hd * 64, o[0]);
          tmem_ld_32x32(t_o + hd * 64 + 32, o[1]);
          if (lane_grp == 0 && lane == 0) tma_store_wait_read();   // the previous store has left the buffer
          tmem_wait_ld();
          if (hd == 1) {
            tc_fence_before();
            mbar_arrive(smem_u32(&o_empty[t]));   // O_t may be overwritten by the next item from here on
          }
          if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t* v = &o[c >> 2][(c & 3) * 8];
            const uint32_t w0 = pack2(__uint_as_float(v[0]) * inv, __uint_as_float(v[1]) * inv, p.out_dtype);
            const uint32_t w1 = pack2(__uint_as_float(v[2]) * inv, __uint_as_float(v[3]) * inv, p.out_dtype);
            const uint32_t w2 = pack2(__uint_as_float(v[4]) * inv, __uint_as_float(v[5]) * inv, p.out_dtype);
            const uint32_t w3 = pack2(__uint_as_float(v[6]) * inv, __uint_as_float(v[7]) * inv, p.out_dtype);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                         ::"r"(my_row + ((c ^ (row & 7)) << 4)), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
          }
          fence_proxy_async_smem();
          if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
          if (lane_grp == 0 && lane == 0) {
            tma_store_4d(&tmap_o, stage, hd * 64, head, it.q_row0 + it.m0, it.coord_b);
            tma_store_commit();
          }
        }
        ++item_cnt;
      } else {
        uint32_t o[4][32];
        tmem_ld_32x32(t_o + 0, o[0]);
        tmem_ld_32x32(t_o + 32, o[1]);
        tmem_ld_32x32(t_o + 64, o[2]);
        tmem_ld_32x32(t_o + 96, o[3]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(&o_empty[t]));   // O_t may be overwritten by the next item from here on
        ++item_cnt;
        if (row < it.rows_valid) {
          uint8_t* op = out_row_ptr(p, it.coord_b, grow, head);
#pragma unroll
          for (int c = 0; c < 4; ++c) store_o_chunk(op, c, o[c], inv, p.out_dtype);
        }
      }
      __syncwarp();
      if (lane == 0) release_item(idx);
    }
    if (lane_grp == 0 && lane == 0) tma_store_wait_all();   // shared memory must outlive the last store
#ifdef FA_B200_PHASE_TRACE
    if (tracer) {
      tr = 900;   // the tail of the role's trace array holds the summed softmax phases
      for (int i = 0; i < 5; ++i) FA_TRACE_VAL(t, tr, 100 + i, prof[i]);
    }
#endif
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
cudaError_t launch_pair_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                          const PrefillKernelParams& p, cudaStream_t stream) {
  const bool win = p.window_left >= 0;
  const bool paged = p.paged != 0;
  const bool vt = p.v_transposed != 0;
  auto kern = paged ? (win ? prefill_pair_kernel<DT, true, true> : prefill_pair_kernel<DT, false, true>)
                    : (win ? prefill_pair_kernel<DT, true, false> : prefill_pair_kernel<DT, false, false>);
  if (vt) {
    if constexpr (DT == FA_B200_E4M3) {
      return cudaErrorInvalidValue;
    } else {
      if (!paged) return cudaErrorInvalidValue;
      kern = win ? prefill_pair_kernel<DT, true, true, true> : prefill_pair_kernel<DT, false, true, true>;
    }
  }
  const size_t smem = 1024 + pair_smem<DT>().total;
  static bool attr_done[6][64] = {};
  static int num_sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_done[win + 2 * paged + 2 * vt][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    attr_done[win + 2 * paged + 2 * vt][dev] = true;
  }
  const long long total = static_cast<long long>(p.h / 2) * p.b * p.num_m_blocks;
  if (total <= 0) return cudaSuccess;
  const int grid = static_cast<int>(total < num_sms[dev] ? total : num_sms[dev]);
  if (!p.work_counter) return cudaErrorInvalidValue;
  kern<<<grid, kThreads, smem, stream>>>(tq, tk, tv, to, p);
  return cudaGetLastError();
}

}  // namespace

#ifdef FA_B200_PHASE_TRACE
extern "C" __attribute__((visibility("default"))) int fa_b200_debug_trace(long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace)));
}
#endif

cudaError_t launch_prefill_pair(int dtype, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                const CUtensorMap& to, const PrefillKernelParams& p, cudaStream_t stream) {
  switch (dtype) {
    case FA_B200_F16: return launch_pair_t<FA_B200_F16>(tq, tk, tv, to, p, stream);
    case FA_B200_BF16: return launch_pair_t<FA_B200_BF16>(tq, tk, tv, to, p, stream);
    case FA_B200_E4M3: return launch_pair_t<FA_B200_E4M3>(tq, tk, tv, to, p, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fa
