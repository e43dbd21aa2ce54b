"""Failure detection without a GPU fault.

GPU: every device-side wait of the kernels is bounded.  The test library (the product's sources built with
-DFA_B200_TEST_HOOKS: waits give up after about a millisecond, one entry makes the next launch announce a tile load it
never issues) is loaded in a child process; a launch whose wait runs out must return, report
FA_B200_ERR_DEVICE_TIMEOUT through fa_b200_device_status(), leave the context usable and release its tensor memory (the
next launch of the same kernel allocates all 512 columns again and must pass its parity check).

CPU (gloo, world size 2): a rank that never joins the all-gather of the split-KV partials must not hang its peer: the
peer leaves gather_partials with an error inside the group's timeout.  The peer-memory exchange kernel is covered on
the GPU by the same kind of test: a launch whose peers never push gives up, reports, and the buffer stays usable."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-attention-das_b200")

_CHILD = textwrap.dedent('''
    import ctypes, os, sys
    sys.path[:0] = [%(pkg)r, %(root)r]
    import torch
    import flash_attn, flash_attn_2_cuda as cuda
    from oracle import attention_oracle as O
    lib = cuda.lib()
    assert hasattr(lib, "fa_b200_test_withhold_load"), "not the test-hook build"
    TIMEOUT = 12
    g = torch.Generator().manual_seed(5)
    dev = "cuda"

    # ---- decode: a partition CTA never gets its first tile
    lens, h, hk, page = [700, 64, 1300], 8, 2, 64
    nblk = [(L + page - 1) // page for L in lens]
    pool = sum(nblk)
    kc = torch.randn(pool, page, hk, 128, generator=g).to(torch.bfloat16)
    vc = torch.randn(pool, page, hk, 128, generator=g).to(torch.bfloat16)
    bt = torch.full((len(lens), max(nblk)), -1, dtype=torch.int32)
    p = 0
    for i, n in enumerate(nblk):
        bt[i, :n] = torch.arange(p, p + n, dtype=torch.int32)
        p += n
    sl = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(len(lens), 1, h, 128, generator=g).to(torch.bfloat16)
    args = (q.to(dev), kc.to(dev), vc.to(dev))
    kw = dict(cache_seqlens=sl.to(dev), block_table=bt.to(dev), causal=True)
    ref, _ = O.paged_decode_ref(q, kc, vc, sl, bt, out_dtype=torch.float32)
    os.environ["FA_B200_DECODE_PARTITION"] = "512"
    assert cuda.device_status() == 0
    lib.fa_b200_test_withhold_load(1)
    flash_attn.flash_attn_with_kvcache(*args, **kw)          # returns: the wait gives up after about a millisecond
    st = cuda.device_status()                                 # synchronises; the context must still answer
    assert st == TIMEOUT, ("decode", st)
    assert cuda.device_status() == 0                          # the status word was cleared by the read
    out = flash_attn.flash_attn_with_kvcache(*args, **kw)     # a normal launch right after
    assert cuda.device_status() == 0
    assert (out.cpu().float() - ref).abs().max().item() < 2e-2
    os.environ.pop("FA_B200_DECODE_PARTITION")

    # ---- two-tile prefill (tensor memory): CTA 0 never gets the first key tile of its first item
    lens = [300, 200]
    cu = torch.tensor([0, 300, 500], dtype=torch.int32)
    q = torch.randn(500, 8, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(500, 2, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(500, 2, 128, generator=g).to(torch.bfloat16)
    ref, _ = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, out_dtype=torch.float32)
    run = lambda: flash_attn.flash_attn_varlen_func(q.to(dev), k.to(dev), v.to(dev), cu.to(dev), cu.to(dev), 300, 300, causal=True)
    assert "prefill_pair" in (run(), cuda.last_launch_info())[1]
    assert cuda.device_status() == 0
    lib.fa_b200_test_withhold_load(1)
    run()
    st = cuda.device_status()
    assert st == TIMEOUT, ("prefill", st)
    for _ in range(3):                                        # every SM's tensor memory was released: these allocate it all again
        out = run()
    assert cuda.device_status() == 0
    assert (out.cpu().float() - ref).abs().max().item() < 2e-2

    # ---- exchange of split-KV partials between GPUs: the other ranks' partials never arrive
    buf, _, _ = cuda.exchange_alloc(2, 8, 128, torch.device(dev))
    o, l = torch.randn(8, 128, device=dev), torch.randn(8, device=dev)
    cuda.exchange_combine(o, l, [buf, buf], 0, 1, 8)          # "rank 0" pushes and waits for a rank 1 that does not exist
    st = cuda.device_status()                                  # the wait gave up after about a millisecond
    assert st == TIMEOUT, ("exchange", st)
    for r in (0, 1):                                           # the buffer is still usable: both ranks' pushes, then a wait
        cuda.exchange_combine(o, l, [buf, buf], r, 2, 8, push=True, wait=False)
    out, lse = cuda.exchange_combine(None, None, [buf, buf], 0, 2, 8, push=False, wait=True, rows=8, d=128, device=torch.device(dev),
                                     out_dtype=torch.float32)
    assert cuda.device_status() == 0
    assert (out - o).abs().max().item() < 1e-5                 # two equal partials merge to themselves
    cuda.exchange_free(buf)
    print("FAILURE-DETECTION-OK")
''')


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_the_gpu_stays_usable():
    hooks = os.path.join(PKG, "libfa_b200_testhooks.so")
    if not os.path.exists(hooks):
        import importlib.util
        spec = importlib.util.spec_from_file_location("_fa_build", os.path.join(PKG, "build.py"))
        b = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(b)
        b.build(test_hooks=True)
    env = dict(os.environ, FA_B200_LIB=hooks)
    env.pop("FA_B200_DECODE_PARTITION", None)
    r = subprocess.run([sys.executable, "-c", _CHILD % {"pkg": PKG, "root": ROOT}], env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0 and "FAILURE-DETECTION-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


# ------------------------------------------------------------------------------------------------------------------
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, ret):
    import datetime
    import time
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(PKG, "flash_attn"))
    import split_kv_parallel as P
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    short = dist.new_group(ranks=list(range(world)), timeout=datetime.timedelta(seconds=3))
    try:
        o, l = torch.zeros(4, 128), torch.zeros(4)
        # a first exchange that everybody joins: the group works
        o_all, _ = P.gather_partials(o + rank, l, group=short)
        ok_first = bool((o_all[:, 0, 0] == torch.arange(world, dtype=torch.float32)).all())
        if rank == 1:
            time.sleep(8.0)               # never joins the second exchange (alive, so no connection reset ends it early)
            ret[rank] = ("absent", ok_first)
            return
        t0 = time.monotonic()
        try:
            P.gather_partials(o, l, group=short)
            ret[rank] = ("returned", ok_first)
        except Exception as e:           # the wait ended with an error instead of hanging
            ret[rank] = ("error", ok_first, time.monotonic() - t0, type(e).__name__)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_never_joins_the_gather_does_not_hang_its_peer():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert not p.is_alive(), "a rank hung"
    got = dict(ret)
    assert got[1] == ("absent", True)
    assert got[0][0] == "error" and got[0][1] is True, got[0]
    assert got[0][2] < 8.0, got[0]            # inside the group's timeout, not when the peer went away
