"""GPU parity: a sequence's output must not depend on what lies next to it in memory.

A key tile is always 128 rows, so the last tile of a packed sequence also holds the first rows of the next one, and a
tile-list entry of 64 rows brings the other half of its 128-row tile along.  Those rows are masked by index, but a
zero probability times a NaN / Inf value is NaN: the kernels have to clear the value rows they do not use, as the
reference zero-fills out-of-range rows on load (csrc/flash_attn_cutlass/src/flash_fwd_kernel.h:319,
src/utils.h:1194-1222).  Every case poisons the neighbours and checks the sequence in the middle against the oracle."""
import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, cos_diff, gen, max_err, randn

pytestmark = pytest.mark.gpu

KERNELS = ["pair", "dense", "single"]


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def _cu(lens):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)


@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("causal", [True, False])
def test_packed_sequences_do_not_see_poisoned_neighbours(fa, monkeypatch, kernel, causal, poison):
    """bf16 varlen batch; for each sequence in turn, the keys and values of every OTHER sequence are NaN / Inf."""
    flash_attn, cuda = fa
    monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kernel)
    g = gen(4100 + KERNELS.index(kernel))
    lens = [200, 77, 513, 128, 300]           # ends inside a tile, short, just past a tile, exactly a tile, ragged
    h, h_k = 8, 2
    cu = _cu(lens)
    q, k, v = randn(g, sum(lens), h, 128), randn(g, sum(lens), h_k, 128), randn(g, sum(lens), h_k, 128)
    ref32, ref_lse = O.attention_varlen_ref(q, k, v, cu, cu, causal=causal, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q, k, v, cu, cu, causal=causal, upcast=False, reorder_ops=True)
    for i in range(len(lens)):
        lo, hi = int(cu[i]), int(cu[i + 1])
        kp, vp = k.clone(), v.clone()
        kp[:lo] = poison; kp[hi:] = poison
        vp[:lo] = poison; vp[hi:] = poison
        out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), kp.cuda(), vp.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                     causal=causal, return_softmax_lse=True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        mine = out[lo:hi].cpu()
        assert torch.isfinite(mine.float()).all(), (kernel, i, "poison leaked into the output")
        assert_close_to_oracle(mine, ref32[lo:hi], ref_pt[lo:hi], mult=2.0, eps=2 ** -8, what=f"{kernel} seq {i}")
        assert max_err(lse[:, lo:hi].cpu(), ref_lse[:, lo:hi]) < 1e-3


@pytest.mark.parametrize("kernel", KERNELS)
def test_packed_e4m3_sequences_do_not_see_poisoned_neighbours(fa, monkeypatch, kernel):
    """The same with e4m3 tensors (e4m3 has no infinity: the neighbours are NaN bytes)."""
    flash_attn, cuda = fa
    monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kernel)
    g = gen(4200)
    lens = [130, 200, 65]
    h, h_k = 8, 2
    cu = _cu(lens)
    qb, kb, vb = randn(g, sum(lens), h, 128), randn(g, sum(lens), h_k, 128), randn(g, sum(lens), h_k, 128)
    (q8, qd), (k8, kd), (v8, vd) = [O.quantize_e4m3_per_tensor(t) for t in (qb, kb, vb)]
    desc = lambda s: s.reshape(1, 1).expand(len(lens), h_k).contiguous()
    ref32, _ = O.attention_varlen_ref(q8, k8, v8, cu, cu, causal=True, q_descale=desc(qd), k_descale=desc(kd),
                                      v_descale=desc(vd), out_dtype=torch.float32)
    ref_p8, _ = O.attention_varlen_ref(q8, k8, v8, cu, cu, causal=True, q_descale=desc(qd), k_descale=desc(kd),
                                       v_descale=desc(vd), intermediate_dtype=torch.float8_e4m3fn, out_dtype=torch.float32)
    nan8 = torch.tensor(float("nan")).to(torch.float8_e4m3fn)
    for i in range(len(lens)):
        lo, hi = int(cu[i]), int(cu[i + 1])
        kp, vp = k8.clone(), v8.clone()
        for t in (kp, vp):
            t.view(torch.uint8)[:lo] = nan8.view(torch.uint8)
            t.view(torch.uint8)[hi:] = nan8.view(torch.uint8)
        out = flash_attn.flash_attn_varlen_func(q8.cuda(), kp.cuda(), vp.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                causal=True, q_descale=qd.cuda(), k_descale=kd.cuda(), v_descale=vd.cuda())
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        mine = out[lo:hi].cpu().float()
        assert torch.isfinite(mine).all(), (kernel, i)
        # the FP8 tolerance of the other e4m3 tests: no worse than twice the error of the e4m3-P PyTorch evaluation
        assert max_err(mine, ref32[lo:hi]) <= 2 * max_err(ref_p8[lo:hi], ref32[lo:hi]) + 2 ** -6, (kernel, i)
        assert cos_diff(mine, ref32[lo:hi]) < 1e-3


@pytest.mark.parametrize("s", [512, 2304])       # 64-row and 128-row query blocks (flash_api_sparse.cpp:127-137)
@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
def test_tile_lists_do_not_see_the_unselected_half_of_a_tile(fa, s, poison):
    """Tile lists whose entries are lone 64-row key tiles: the 64 rows that follow each entry (the other half of the
    128-row tile the kernel fetches) are NaN / Inf in K and V and selected by nobody."""
    flash_attn, cuda = fa
    g = gen(4300 + s)
    h, h_k = 4, 2
    block_m = O.sparse_block_m(s)
    nq = (s + block_m - 1) // block_m
    n64 = s // 64
    q, k, v = randn(g, 1, s, h, 128), randn(g, 1, s, h_k, 128), randn(g, 1, s, h_k, 128)
    # every query block keeps the even 64-row key tiles 0, 2, 4, ... (per head a different subset of them)
    keep = torch.zeros(1, h, nq, n64, dtype=torch.bool)
    for hi in range(h):
        for m in range(nq):
            sel = torch.arange(0, n64, 2)
            sel = sel[torch.rand(sel.numel(), generator=g) < 0.6]
            keep[0, hi, m, sel] = True
            keep[0, hi, m, 0] = True
    cnt = keep.sum(-1).to(torch.int32)
    nnz = int(cnt.max())
    offs = torch.full((1, h, nq, nnz), 10_000_000, dtype=torch.int32)
    for hi in range(h):
        for m in range(nq):
            idx = torch.nonzero(keep[0, hi, m]).flatten() * 64
            offs[0, hi, m, :idx.numel()] = idx.to(torch.int32)
    kp, vp = k.clone(), v.clone()
    for t in range(1, n64, 2):                  # the odd 64-row tiles: selected by nobody
        kp[0, t * 64:(t + 1) * 64] = poison
        vp[0, t * 64:(t + 1) * 64] = poison
    cc = torch.zeros(1, h, nq, dtype=torch.int32)
    ci = torch.zeros(1, h, nq, 1, dtype=torch.int32)
    out, lse = flash_attn.sparse_attn_func(q.cuda(), kp.cuda(), vp.cuda(), cnt.cuda(), offs.cuda(), cc.cuda(), ci.cuda(),
                                           causal=False, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert torch.isfinite(out.float()).all()
    mask = O.block_lists_to_dense_mask(cnt, offs, s, s, block_m)
    ref32, ref_lse = O.attention_ref(q, k, v, out_dtype=torch.float32, extra_mask=mask)
    ref_pt, _ = O.attention_ref(q, k, v, upcast=False, reorder_ops=True, extra_mask=mask)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"tile lists s={s}")
    assert max_err(lse.cpu(), ref_lse) < 1e-3
