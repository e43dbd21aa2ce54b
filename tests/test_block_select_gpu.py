"""GPU parity of the mean-similarity block selection (get_block_map_meansim: fa_b200_block_pool + fa_b200_block_select)
against the CPU oracle, which is pinned to the reference's own selection chain by the golden block_select cases.
Integer / boolean outputs are compared exactly, except where the oracle itself reports that the decision hangs on the
last bits of an fp32 sum (cut within 1e-5 of the threshold, or tied probabilities at the cut)."""
import pytest
import torch

from oracle import attention_oracle as O
from oracle import block_select_oracle as BS
from _util import assert_close_to_oracle, gen

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    from flash_attn.utils import sparse_utils
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda, sparse_utils


def _qk(g, b, h, n, d, noise, dtype):
    q = torch.randn(b, h, n, d, generator=g) * noise + torch.randn(b, h, 1, d, generator=g)
    k = torch.randn(b, h, n, d, generator=g) * noise + torch.randn(b, h, 1, d, generator=g)
    return q.to(dtype), k.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,d,block", [(900, 128, 128), (1024, 64, 64), (333, 256, 64), (128, 128, 128)])
def test_pooling_and_self_similarity(fa, n, d, block, dtype):
    _, cuda, _ = fa
    g = gen(n + d)
    x, _ = _qk(g, 2, 3, n, d, 0.8, dtype)
    x[0, 1, 5] = 0                                              # a zero row: its block is "not similar" (0 / 0 in the reference)
    th = torch.tensor([0.1, 0.55, 0.9])
    pooled, sim = cuda.block_pool(x.cuda(), block, th.cuda())
    torch.cuda.synchronize()
    ref_p, ref_s, val = BS.pool_sim_ref(x, block, th)
    assert (pooled.cpu().float() - ref_p.float()).abs().max() <= 2 ** -7 * ref_p.float().abs().max()   # one rounding of the mean
    decided = ~((val - th.view(1, 3, 1)).abs() < 1e-3)          # NaN (cut or zero-row blocks) compares as decided: False
    assert torch.equal(sim.cpu()[decided], ref_s[decided])
    assert not sim.cpu()[0, 1, 0]
    if n % block:
        assert not sim.cpu()[..., -1].any()
    # strided input: (B, N, H, D) storage viewed as (B, H, N, D)
    xs = x.permute(0, 2, 1, 3).contiguous().cuda().permute(0, 2, 1, 3)
    p2, s2 = cuda.block_pool(xs, block, th.cuda())
    assert torch.equal(p2, pooled) and torch.equal(s2, sim)


CASES = [
    dict(b=2, h=3, n=900, d=128, noise=0.3, causal=False, args=dict(cdfthreshd=0.9)),
    dict(b=1, h=4, n=1100, d=128, noise=0.3, causal=True, args=dict(cdfthreshd=0.5, attention_sink=True)),
    dict(b=1, h=2, n=1024, d=64, noise=0.5, causal=True, args=dict(cdfthreshd=None, topk=0.3)),
    dict(b=1, h=2, n=640, d=128, noise=3.0, causal=False, args=dict(cdfthreshd=0.7, simthreshd1=0.2)),
    dict(b=1, h=2, n=8192, d=128, noise=0.4, causal=True, args=dict(cdfthreshd=0.95)),
    dict(b=1, h=2, n=4000, d=128, noise=0.4, causal=True, args=dict(cdfthreshd=torch.tensor([0.3, 0.99]))),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"n{c['n']}d{c['d']}{'c' if c['causal'] else ''}")
def test_block_map_matches_oracle(fa, case, dtype):
    _, cuda, su = fa
    g = gen(case["n"] * 3 + case["d"])
    q, k = _qk(g, case["b"], case["h"], case["n"], case["d"], case["noise"], dtype)
    got = su.get_block_map_meansim(q.cuda(), k.cuda(), is_causal=case["causal"], **case["args"])
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref, margin = BS.block_map_meansim_ref(q, k, is_causal=case["causal"], **case["args"])
    assert got.shape == ref.shape and got.dtype == torch.bool
    # the self-similarity flags feed the map: leave out blocks whose flag is within 1e-3 of its threshold
    th1 = torch.full((case["h"],), float(case["args"].get("simthreshd1", 0.1)))
    _, _, vq = BS.pool_sim_ref(q, 128, th1)
    _, _, vk = BS.pool_sim_ref(k, 64, th1)
    assert not ((vq - th1.view(1, -1, 1)).abs() < 1e-3).any() and not ((vk - th1.view(1, -1, 1)).abs() < 1e-3).any()
    decided = margin > 1e-5
    assert decided.float().mean() > 0.8
    assert torch.equal(got.cpu()[decided], ref[decided])
    # undecided rows may differ by the blocks at the cut only
    assert (got.cpu() != ref).sum(dim=-1).max() <= 2
    off, cnt = su.get_block_map_meansim(q.cuda(), k.cuda(), is_causal=case["causal"], return_block_offset=True, **case["args"])
    off2, cnt2 = su.block_map_to_block_offset(got)
    assert torch.equal(off, off2) and torch.equal(cnt, cnt2) and torch.equal(cnt.cpu(), got.sum(-1).int().cpu())


def test_selected_blocks_drive_the_sparse_kernel(fa):
    """get_block_map_meansim -> block lists -> sparse_attn_func, against dense attention under the expanded mask."""
    flash_attn, cuda, su = fa
    g = gen(31337)
    b, h, n, d = 1, 4, 2304, 128          # > 2048 rows: 128-row query blocks in the sparse kernel, as in the selection
    q, k = _qk(g, b, h, n, d, 0.4, torch.bfloat16)
    v = torch.randn(b, h, n, d, generator=g).to(torch.bfloat16)
    bmap = su.get_block_map_meansim(q.cuda(), k.cuda(), is_causal=True, cdfthreshd=0.9)
    off, cnt = su.block_map_to_block_offset(bmap)
    offs = torch.where(off >= 10000000, off, off * 64)           # block indices -> K row offsets of 64-row tiles
    qs, ks, vs = [t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v)]       # (b, s, h, d)
    cc = torch.zeros(b, h, cnt.shape[2], dtype=torch.int32, device="cuda")
    ci = torch.zeros(b, h, cnt.shape[2], 1, dtype=torch.int32, device="cuda")
    out = flash_attn.sparse_attn_func(qs.cuda(), ks.cuda(), vs.cuda(), cnt, offs.int(), cc, ci, causal=True)
    out = out[0] if isinstance(out, (tuple, list)) else out
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    mask = O.block_lists_to_dense_mask(cnt.cpu(), offs.int().cpu(), n, n, 128)
    ref32, _ = O.attention_ref(qs, ks, vs, causal=True, out_dtype=torch.float32, extra_mask=mask)
    ref_pt, _ = O.attention_ref(qs, ks, vs, causal=True, upcast=False, reorder_ops=True, extra_mask=mask)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what="selected blocks")
    assert 0.05 < bmap.float().mean() < 0.6


@pytest.mark.parametrize("seed", range(12))
def test_random_selection_configurations(fa, seed):
    """Random lengths (cut blocks included), head dimensions, thresholds per head, top-k or cumulative selection,
    causal / sink flags: maps equal to the oracle's on every row the oracle calls decided."""
    import os
    import random
    _, cuda, su = fa
    off = int(os.environ.get("FA_TEST_SEED_OFFSET", "0"))
    rng = random.Random(7000 + seed + off)
    g = gen(7000 + seed + off)
    dtype = rng.choice([torch.bfloat16, torch.float16])
    b, h, d = rng.randint(1, 2), rng.randint(1, 4), rng.choice([64, 128, 256])
    n = rng.choice([64, 129, 500, 1024, 1500, 3000])
    noise = rng.choice([0.2, 0.4, 0.8])
    q, k = _qk(g, b, h, n, d, noise, dtype)
    causal, sink = rng.random() < 0.5, rng.random() < 0.3
    if rng.random() < 0.5:
        args = dict(cdfthreshd=torch.tensor([rng.choice([0.3, 0.6, 0.9, 0.98]) for _ in range(h)]))
    else:
        args = dict(cdfthreshd=None, topk=rng.choice([0.1, 0.25, 0.5]))
    got = su.get_block_map_meansim(q.cuda(), k.cuda(), is_causal=causal, attention_sink=sink, **args)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref, margin = BS.block_map_meansim_ref(q, k, is_causal=causal, attention_sink=sink, **args)
    th1 = torch.full((h,), 0.1)
    _, _, vq = BS.pool_sim_ref(q, 128, th1)
    _, _, vk = BS.pool_sim_ref(k, 64, th1)
    near = ((vq - 0.1).abs() < 1e-3).any() or ((vk - 0.1).abs() < 1e-3).any()
    if near:
        pytest.skip("a self-similarity value lies within 1e-3 of its threshold")
    decided = margin > 1e-5
    what = f"n{n} d{d} b{b} h{h} causal{causal} sink{sink} {args}"
    assert torch.equal(got.cpu()[decided], ref[decided]), what
    assert (got.cpu() != ref).sum(dim=-1).max() <= 2, what
