"""Multi-GPU helpers of the attention hot path (one process per GPU, torch.distributed).

The path shards without communication — decode batches by sequence, prefill by sequence (or (batch, kv head)) — so
the only collective is the one needed when a SINGLE very long sequence is split-KV across GPUs: every rank decodes
its own page range to an fp32 partial (O normalised by its own sum, natural-log LSE), the partials are all-gathered
(NCCL over NVLink; 16.5 KB per rank for 32 heads) into each rank's own memory and merged there by the LSE-combine
kernel.  No peer-memory loads are involved.

The reference has no counterpart (its long-context handling is single-device split-KV only,
csrc/flash_attn_cutlass/src/paged_attention.cu:792-826); the partial format is the one its combine kernels consume
(src/paged_attention.h:356-445), in LSE form.
"""
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_sequences_lpt(lengths: Sequence[int], world_size: int, power: float = 1.0) -> List[List[int]]:
    """Greedy longest-processing-time assignment of sequences to ranks.  Cost of a sequence = length ** power
    (1 for decode: KV bytes streamed; 2 for causal prefill: FLOPs).  Returns, per rank, the sorted indices it owns;
    every index appears exactly once and the result is deterministic."""
    order = sorted(range(len(lengths)), key=lambda i: (-float(lengths[i]) ** power, i))
    loads = [0.0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda x: (loads[x], x))
        owned[r].append(i)
        loads[r] += float(lengths[i]) ** power
    return [sorted(o) for o in owned]


def shard_prefill_grid(lengths: Sequence[int], h_k: int, world_size: int) -> Tuple[int, int, List[List[int]]]:
    """Two-axis split of a prefill batch: ``world_size = seq_groups * head_groups`` with ``head_groups`` dividing the kv
    heads.  Sequences go to the sequence groups by LPT on length squared (causal FLOPs); every rank of a sequence group
    takes the same sequences and one contiguous slice of the kv heads (and of the query heads that belong to them), so
    each rank still makes ONE varlen call and nothing is exchanged.  Of the admissible factorisations the one with the
    smallest largest load is taken (ties: fewer head groups, i.e. wider K/V sharing inside a rank) — a few long sequences
    go to the head axis, many sequences to the sequence axis.
    Returns (seq_groups, head_groups, owned) with owned[g] = sorted sequence indices of sequence group g; rank r works on
    sequence group r // head_groups and kv heads [hg * h_k / head_groups, (hg + 1) * h_k / head_groups), hg = r % head_groups."""
    best = None
    for hg in range(1, min(h_k, world_size) + 1):
        if h_k % hg or world_size % hg:
            continue
        sg = world_size // hg
        owned = shard_sequences_lpt(lengths, sg, power=2.0)
        load = max(sum(float(lengths[i]) ** 2 for i in o) for o in owned) / hg
        if best is None or load < best[0] * (1 - 1e-9):
            best = (load, sg, hg, owned)
    if best is None:
        raise ValueError("world_size must be a product of a sequence split and a divisor of the kv heads")
    return best[1], best[2], best[3]


def split_page_range(num_pages: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous page range [first, last) of one sequence owned by `rank` (earlier ranks take the remainder)."""
    base, rem = divmod(num_pages, world_size)
    first = rank * base + min(rank, rem)
    return first, first + base + (1 if rank < rem else 0)


def window_for_slice(seqlen_total: int, slice_first: int, slice_len: int, window_left: int) -> Tuple[int, int]:
    """Sliding window of a decode step seen from one rank's slice [slice_first, slice_first + slice_len) of the
    sequence's keys.  The query token (position seqlen_total - 1) sees keys lo .. seqlen_total - 1 with
    lo = max(0, seqlen_total - 1 - window_left) (window_left < 0: all).  Returns (local length, local window_left) to
    hand to the decode call on the slice: length 0 if the slice lies wholly before the window, window -1 if it lies
    wholly inside."""
    if window_left < 0:
        return slice_len, -1
    lo = max(0, seqlen_total - 1 - window_left)
    if lo >= slice_first + slice_len:
        return 0, -1
    if lo <= slice_first:
        return slice_len, -1
    return slice_len, slice_len - 1 - (lo - slice_first)


def gather_partials(o_partial: torch.Tensor, lse_partial: torch.Tensor,
                    group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather per-rank partials: o_partial (rows, d) fp32 and lse_partial (rows,) fp32 ->
    (world, rows, d) and (world, rows), rank-major, identical on every rank — the layout the combine kernel takes.
    Works on any backend (NCCL for CUDA tensors, gloo for CPU tensors)."""
    world = dist.get_world_size(group)
    o_all = torch.empty((world,) + tuple(o_partial.shape), dtype=o_partial.dtype, device=o_partial.device)
    l_all = torch.empty((world,) + tuple(lse_partial.shape), dtype=lse_partial.dtype, device=lse_partial.device)
    if o_partial.is_cuda:
        dist.all_gather_into_tensor(o_all.view(-1), o_partial.contiguous().view(-1), group=group)
        dist.all_gather_into_tensor(l_all.view(-1), lse_partial.contiguous().view(-1), group=group)
    else:  # gloo has no all_gather_into_tensor for every build: use the list form
        dist.all_gather(list(o_all.unbind(0)), o_partial.contiguous(), group=group)
        dist.all_gather(list(l_all.unbind(0)), lse_partial.contiguous(), group=group)
    return o_all, l_all


class PartialExchange:
    """Peer-memory exchange of the ranks' split-KV partials, fused with their combine (fa_b200_exchange_combine): one
    launch per step instead of an all-gather and a combine launch.

    Set-up (collective over ``group``; allocates and synchronises, so do it once, outside the step loop): every rank
    lets the library allocate its exchange buffer, the 64-byte CUDA IPC handles travel through ``all_gather_object``,
    and every rank maps the other ranks' buffers.  All ranks must be processes of one node with peer access between
    their GPUs.  ``combine`` must then be called the same number of times on every rank (the call counter is the epoch
    the kernels synchronise on).  ``close()`` unmaps and frees; call it on every rank after a barrier."""

    def __init__(self, rows: int, d: int, device, group: Optional[dist.ProcessGroup] = None):
        import flash_attn_2_cuda as cuda
        self._cuda = cuda
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 16:
            raise ValueError("PartialExchange takes at most 16 ranks")
        self.rows, self.d, self.device = rows, d, torch.device(device)
        self.epoch = 0
        self._own, self._opened, self.peers = 0, [], []
        failed = None
        # Every rank goes through the same collectives whatever fails locally, and raises only after the last one.
        try:
            self._own, handle, self.bytes = cuda.exchange_alloc(self.world, rows, d, self.device)
        except Exception as e:
            handle, failed = None, e
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        for r, hd in enumerate(handles):
            if r == self.rank:
                self.peers.append(self._own)
                continue
            try:
                if hd is None:
                    raise RuntimeError("rank %d could not allocate its exchange buffer" % r)
                ptr = cuda.exchange_open(hd, self.device)
                self._opened.append(ptr)
                self.peers.append(ptr)
            except Exception as e:
                failed = failed or e
                self.peers.append(0)
        dist.barrier(group=group)
        if failed is not None:
            self.close()
            raise RuntimeError("PartialExchange set-up failed on rank %d: %r" % (self.rank, failed))

    def combine(self, o_local: torch.Tensor, lse_local: torch.Tensor, h: int, out_dtype=torch.bfloat16, s_aux=None):
        """o_local (rows, d) fp32, lse_local (rows) fp32 of this rank -> (out (rows, d), lse (rows)), identical on every
        rank.  One launch on the current stream."""
        self.epoch += 1
        return self._cuda.exchange_combine(o_local, lse_local, self.peers, self.rank, self.epoch, h, out_dtype=out_dtype,
                                           s_aux=s_aux)

    def close(self):
        for ptr in self._opened:
            self._cuda.exchange_close(ptr)
        self._opened = []
        if self._own:
            self._cuda.exchange_free(self._own)
            self._own = 0


def decode_split_across_gpus(q, k_cache_local, v_cache_local, local_seqlens, local_block_table, softmax_scale=None,
                             group: Optional[dist.ProcessGroup] = None, out_dtype=torch.bfloat16, q_descale=None,
                             k_descale=None, v_descale=None, s_aux=None, local_window_left: int = -1,
                             phase_events: Optional[Sequence["torch.cuda.Event"]] = None,
                             exchange: Optional[PartialExchange] = None):
    """Decode where each rank holds a slice of every sequence's KV pages.  q: (b, 1, h, 128), identical on every
    rank; the caches, `local_seqlens` and `local_block_table` describe this rank's slice.  Attention sinks
    (``s_aux``, (h)) enter once, in the final combine; a sliding window is given per slice (``window_for_slice``).
    Returns (out (b, 1, h, 128) out_dtype, lse (b, h) fp32), identical on every rank.
    ``exchange``: a PartialExchange for (b * h rows, d) set up over the same group: the partials then cross NVLink as
    peer stores inside ONE kernel that also combines them, instead of an NCCL all-gather followed by a combine launch.
    ``phase_events``: four CUDA events recorded on the current stream before the local decode, after it (partition
    kernel with its in-kernel merge), after the all-gather and after the final combine (timing of the three phases)."""
    import flash_attn_2_cuda as cuda
    b, _, h, d = q.shape
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    if phase_events is not None:
        phase_events[0].record()
    o_part, l_part = cuda.decode_partial(q, k_cache_local, v_cache_local, local_seqlens, local_block_table,
                                         softmax_scale, q_descale, k_descale, v_descale, window_left=local_window_left)
    if phase_events is not None:
        phase_events[1].record()
    if exchange is not None:
        if phase_events is not None:
            phase_events[2].record()    # no separate gather phase: the exchange is part of the kernel that combines
        out, lse = exchange.combine(o_part.view(b * h, d), l_part.view(b * h), h, out_dtype=out_dtype, s_aux=s_aux)
        if phase_events is not None:
            phase_events[3].record()
        return out.view(b, 1, h, d), lse.view(b, h)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        rows = b * h
        if (o_part.is_cuda and (rows * (d + 1)) % 4 == 0 and
                o_part.untyped_storage().data_ptr() == l_part.untyped_storage().data_ptr()):
            # decode_partial returns [O | LSE] in one buffer: one all-gather moves both
            world = dist.get_world_size(group)
            packed = torch.empty((world, rows * (d + 1)), dtype=torch.float32, device=o_part.device)
            mine = torch.as_strided(o_part, (rows * (d + 1),), (1,), o_part.storage_offset())
            dist.all_gather_into_tensor(packed.view(-1), mine, group=group)
            o_all = packed[:, :rows * d].unflatten(1, (rows, d))
            l_all = packed[:, rows * d:]
        else:
            o_all, l_all = gather_partials(o_part.view(rows, d), l_part.view(rows), group)
    else:
        o_all, l_all = o_part.view(1, b * h, d), l_part.view(1, b * h)
    if phase_events is not None:
        phase_events[2].record()
    out, lse = cuda.combine(o_all, l_all, out_dtype=out_dtype, h=h, s_aux=s_aux)
    if phase_events is not None:
        phase_events[3].record()
    return out.view(b, 1, h, d), lse.view(b, h)
