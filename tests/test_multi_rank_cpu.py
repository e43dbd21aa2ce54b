"""CPU, world_size 2 over gloo: the host-side logic of the multi-GPU paths — sequence sharding, page-range split
of one long sequence, and the all-gather of (O, LSE) partials whose merge must equal the unsplit attention.  The
attention itself is evaluated by the CPU oracle here (no GPU in this test); the kernels' side of the same exchange
is covered by the GPU tests of the combine kernel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "flash-attention-das_b200", "flash_attn"))
    import split_kv_parallel as P            # the module itself needs no GPU; the package import would
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)        # same data on every rank
        page, h, hk, d, npages = 16, 4, 2, 128, 11
        L = npages * page - 5
        q = torch.randn(1, 1, h, d, generator=g)
        k = torch.randn(1, L, hk, d, generator=g)
        v = torch.randn(1, L, hk, d, generator=g)
        first, last = P.split_page_range(npages, world, rank)
        lo, hi = first * page, min(last * page, L)
        o, l = O.attention_ref(q, k[:, lo:hi], v[:, lo:hi], out_dtype=torch.float32)   # this rank's partial
        o_all, l_all = P.gather_partials(o.reshape(h, d).contiguous(), l.reshape(h).contiguous())
        assert o_all.shape == (world, h, d) and l_all.shape == (world, h)
        merged, lse = O.merge_partials_ref(o_all, l_all)
        full, lse_full = O.attention_ref(q, k, v, out_dtype=torch.float32)
        ok = torch.allclose(merged, full[0, 0], atol=1e-5) and torch.allclose(lse, lse_full[0, :, 0], atol=1e-5)
        # rank-major layout: slot r of the gathered buffer is rank r's partial
        mine_ok = torch.equal(o_all[rank], o.reshape(h, d))
        # the same exchange under a sliding window with attention sinks: each rank applies the window its slice sees
        # (window_for_slice), the sink enters once, after the merge
        win_ok = True
        s_aux = torch.randn(h, generator=g)
        for wl in (0, 3, 40, 90, 1000):
            n_loc, wl_loc = P.window_for_slice(L, lo, hi - lo, wl)
            if n_loc == 0:
                o_w, l_w = torch.zeros(h, d), torch.full((h,), float("-inf"))
            else:
                o_w, l_w = O.attention_ref(q, k[:, lo:lo + n_loc], v[:, lo:lo + n_loc], out_dtype=torch.float32,
                                           window_size=(wl_loc, -1))
                o_w, l_w = o_w.reshape(h, d), l_w.reshape(h)
            ow_all, lw_all = P.gather_partials(o_w.contiguous(), l_w.contiguous())
            merged_w, lse_w = O.merge_partials_ref(ow_all, lw_all)
            tot = torch.logaddexp(lse_w, s_aux)
            merged_w = merged_w * torch.exp(lse_w - tot).unsqueeze(-1)
            full_w, _ = O.attention_ref(q, k, v, out_dtype=torch.float32, window_size=(wl, -1), s_aux=s_aux)
            win_ok = win_ok and torch.allclose(merged_w, full_w[0, 0], atol=1e-5)
        ret[rank] = bool(ok and mine_ok and win_ok)
    finally:
        dist.destroy_process_group()


def test_gather_and_merge_two_ranks_gloo():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(ret) == {0: True, 1: True}


def test_lpt_sharding_properties():
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "split_kv_parallel", os.path.join(root, "flash-attention-das_b200", "flash_attn", "split_kv_parallel.py"))
    P = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(P)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(1024, 32769, (64,), generator=g).tolist()
    for world in (1, 2, 4, 8):
        shards = P.shard_sequences_lpt(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))          # a partition of the batch
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)                             # LPT bound
        assert shards == P.shard_sequences_lpt(lens, world)                     # deterministic
    sq = P.shard_sequences_lpt(lens, 4, power=2.0)
    loads2 = [sum(lens[i] ** 2 for i in s) for s in sq]
    assert max(loads2) - min(loads2) <= max(lens) ** 2
    # page ranges tile [0, n) exactly
    for n, w in ((4096, 8), (11, 2), (5, 8)):
        r = [P.split_page_range(n, w, k) for k in range(w)]
        assert r[0][0] == 0 and r[-1][1] == n and all(r[i][1] == r[i + 1][0] for i in range(w - 1))


def test_prefill_grid_sharding():
    """The (sequence group, kv-head group) grid of a prefill batch: a partition of the work, balanced, deterministic."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "split_kv_parallel", os.path.join(root, "flash-attention-das_b200", "flash_attn", "split_kv_parallel.py"))
    P = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(P)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(512, 4097, (16,), generator=g).tolist()
    total = sum(l * l for l in lens)
    for world in (1, 2, 4, 8):
        sg, hg, owned = P.shard_prefill_grid(lens, 8, world)
        assert sg * hg == world and 8 % hg == 0 and len(owned) == sg
        assert sorted(i for o in owned for i in o) == list(range(16))
        worst = max(sum(lens[i] ** 2 for i in o) for o in owned) / hg
        assert worst <= total / world * 1.0001          # few ragged sequences: the head axis balances exactly
        assert (sg, hg, owned) == P.shard_prefill_grid(lens, 8, world)
    # many equal sequences: the sequence axis is enough, K/V sharing inside a rank stays as wide as possible
    assert P.shard_prefill_grid([4096] * 8, 8, 8)[:2] == (8, 1)
    assert P.shard_prefill_grid([4096] * 8, 8, 4)[:2] == (4, 1)
    # sixteen ranks over eight kv heads and three sequences: both axes
    sg, hg, owned = P.shard_prefill_grid([1000, 3000, 2000], 8, 16)
    assert sg * hg == 16 and 8 % hg == 0
    with pytest.raises(ValueError):
        P.shard_prefill_grid([100], 2, 0)   # no rank, no factorisation
