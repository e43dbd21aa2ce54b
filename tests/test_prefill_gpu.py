"""GPU parity: dense fixed-length, packed varlen, FP8 and block-sparse prefill (fa_b200_fwd /
fa_b200_fwd_sparse through the reference-shaped Python API) against the CPU oracle and the golden vectors."""
import importlib.util
import os

import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, cos_diff, gen, max_err, randn

pytestmark = pytest.mark.gpu

_spec = importlib.util.spec_from_file_location(
    "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
_mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mg)


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def _check_lse(lse, ref_lse):
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    if fin.any():
        assert max_err(lse[fin], ref_lse[fin]) < 1e-3
    assert torch.all(lse[~fin] == float("inf"))


def test_fixed_golden_cases(fa, golden):
    flash_attn, cuda = fa
    for c in [c for c in golden["cases"] if c["kind"] == "fixed"]:
        q, k, v = _mg.gen_inputs(c)
        out, lse, _ = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=c["causal"], return_attn_probs=True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        ref32, ref_lse = O.attention_ref(q, k, v, causal=c["causal"], out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(q, k, v, causal=c["causal"], upcast=False, reorder_ops=True)
        assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=c["name"])
        _check_lse(lse.cpu(), c["lse"])
        # against the reference-made fixture itself: the two differ by output rounding only
        assert max_err(out.cpu(), c["out"]) <= 2 * c["err_pt"] + 2 ** -8, c["name"]


def test_varlen_golden_cases(fa, golden):
    flash_attn, cuda = fa
    for c in [c for c in golden["cases"] if c["kind"] == "varlen"]:
        q, k, v, cq, ck = _mg.gen_inputs(c)
        out, lse = flash_attn.flash_attn_varlen_func(
            q.cuda(), k.cuda(), v.cuda(), cq.cuda(), ck.cuda(), max(c["lens_q"]), max(c["lens_k"]),
            causal=c["causal"], return_softmax_lse=True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        ref32, ref_lse = O.attention_varlen_ref(q, k, v, cq, ck, causal=c["causal"], out_dtype=torch.float32)
        ref_pt, _ = O.attention_varlen_ref(q, k, v, cq, ck, causal=c["causal"], upcast=False, reorder_ops=True)
        assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=c["name"])
        assert lse.shape == (c["h"], sum(c["lens_q"]))
        _check_lse(lse.cpu(), c["lse"])


SHAPES = [
    # dtype, b, sq, sk, h, h_k, causal
    (torch.bfloat16, 2, 128, 128, 4, 1, True),
    (torch.bfloat16, 1, 384, 384, 8, 2, True),
    (torch.float16, 2, 200, 333, 4, 4, False),
    (torch.bfloat16, 1, 1000, 1000, 4, 2, True),
    (torch.float16, 1, 64, 513, 2, 1, True),      # sq < sk, causal bottom-right
    (torch.bfloat16, 1, 300, 100, 2, 2, True),    # sq > sk: the first rows see nothing
    (torch.bfloat16, 3, 1, 257, 8, 2, True),      # single query row: causal is dropped
]


@pytest.mark.parametrize("dtype,b,sq,sk,h,h_k,causal", SHAPES)
def test_fixed_matches_oracle(fa, dtype, b, sq, sk, h, h_k, causal):
    flash_attn, cuda = fa
    g = gen(sq * 7 + sk * 3 + h)
    q, k, v = randn(g, b, sq, h, 128, dtype=dtype), randn(g, b, sk, h_k, 128, dtype=dtype), randn(g, b, sk, h_k, 128, dtype=dtype)
    out, lse, _ = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=causal, return_attn_probs=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    eff_causal = causal and sq > 1
    ref32, ref_lse = O.attention_ref(q, k, v, causal=eff_causal, out_dtype=torch.float32)
    ref_pt, _ = O.attention_ref(q, k, v, causal=eff_causal, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"fixed {sq}x{sk}")
    _check_lse(lse.cpu(), ref_lse)


def test_varlen_ragged_batch_and_noncontiguous_qkv(fa):
    flash_attn, cuda = fa
    g = gen(99)
    lens = [1, 127, 128, 129, 700, 33, 512]
    h, h_k = 8, 2
    total = sum(lens)
    # q, k, v as views of one packed (total, h + 2 h_k, d) buffer: row stride differs from h * d
    qkv = randn(g, total, h + 2 * h_k, 128)
    q, k, v = qkv[:, :h], qkv[:, h:h + h_k], qkv[:, h + h_k:]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    qkv_d = qkv.cuda()
    out, lse = flash_attn.flash_attn_varlen_func(
        qkv_d[:, :h], qkv_d[:, h:h + h_k], qkv_d[:, h + h_k:], cu.cuda(), cu.cuda(), max(lens), max(lens), causal=True,
        return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref32, ref_lse = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what="varlen ragged")
    _check_lse(lse.cpu(), ref_lse)
    # determinism: a second run is bit-identical (the reference's race-condition test)
    out2, lse2 = flash_attn.flash_attn_varlen_func(
        qkv_d[:, :h], qkv_d[:, h:h + h_k], qkv_d[:, h + h_k:], cu.cuda(), cu.cuda(), max(lens), max(lens), causal=True,
        return_softmax_lse=True)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)


def test_fp8_golden_and_varlen(fa, golden):
    flash_attn, cuda = fa
    for c in [c for c in golden["cases"] if c["kind"] == "fp8" and c["sq"] > 1]:
        q8, k8, v8, qd, kd, vd = _mg.gen_inputs(c)
        b, sq, sk = c["b"], c["sq"], c["sk"]
        cq = torch.arange(0, (b + 1) * sq, sq, dtype=torch.int32)
        ck = torch.arange(0, (b + 1) * sk, sk, dtype=torch.int32)
        out = flash_attn.flash_attn_varlen_func(
            q8.reshape(b * sq, c["h"], 128).cuda(), k8.reshape(b * sk, c["hk"], 128).cuda(),
            v8.reshape(b * sk, c["hk"], 128).cuda(), cq.cuda(), ck.cuda(), sq, sk, causal=c["causal"],
            q_descale=qd.cuda(), k_descale=kd.cuda(), v_descale=vd.cuda())
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert out.dtype == torch.bfloat16
        out = out.cpu().reshape(b, sq, c["h"], 128)
        # FP8 rule of the reference's tests: error <= 2x the error of the same math with P round-tripped
        # through e4m3 (tests/test_flash_attn_varlen_fp8.py:521-694), plus cosine-diff < 1e-3 (:477-484)
        e = max_err(out, c["out"])
        e_p8 = max_err(c["out_p8"], c["out"])
        assert e <= 2 * e_p8 + 2 ** -7, (e, e_p8)
        assert cos_diff(out, c["out"]) < 1e-3


def test_fp8_prefill_larger(fa):
    flash_attn, cuda = fa
    g = gen(4242)
    lens = [500, 129, 1024]
    h, h_k = 8, 2
    total = sum(lens)
    q16, k16, v16 = randn(g, total, h, 128), randn(g, total, h_k, 128), randn(g, total, h_k, 128)
    q8, qd = O.quantize_e4m3_per_tensor(q16)
    k8, kd = O.quantize_e4m3_per_tensor(k16)
    v8, vd = O.quantize_e4m3_per_tensor(v16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q8.cuda(), k8.cuda(), v8.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                 causal=True, q_descale=qd.cuda(), k_descale=kd.cuda(), v_descale=vd.cuda(),
                                                 return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    nb = len(lens)
    kw = dict(q_descale=qd.expand(nb, h_k), k_descale=kd.expand(nb, h_k), v_descale=vd.expand(nb, h_k))
    ref32, ref_lse = O.attention_varlen_ref(q8, k8, v8, cu, cu, causal=True, out_dtype=torch.float32, **kw)
    ref_p8, _ = O.attention_varlen_ref(q8, k8, v8, cu, cu, causal=True, out_dtype=torch.float32,
                                       intermediate_dtype=torch.float8_e4m3fn, **kw)
    e, e_p8 = max_err(out.cpu(), ref32), max_err(ref_p8, ref32)
    assert e <= 2 * e_p8 + 2 ** -7, (e, e_p8)
    assert cos_diff(out.cpu(), ref32) < 1e-3
    _check_lse(lse.cpu(), ref_lse)


def _sparse_inputs(g, b, s, h, h_k, density, causal):
    block_m = O.sparse_block_m(s)
    nq = (s + block_m - 1) // block_m
    nk = (s + 127) // 128
    tm = torch.rand(b, h, nq, nk, generator=g) < density
    if causal:
        qi = torch.arange(nq).view(-1, 1) * block_m
        ki = torch.arange(nk).view(1, -1) * 128
        tm &= (ki <= qi + block_m - 1)
        tm |= (ki <= qi) & (qi < ki + 128)        # always keep the diagonal tile
    cnt, offs = O.tile_mask_to_block_lists(tm, block_m=block_m, block_n=64, tile_n=128)
    q, k, v = randn(g, b, s, h, 128), randn(g, b, s, h_k, 128), randn(g, b, s, h_k, 128)
    return q, k, v, cnt, offs, block_m


@pytest.mark.parametrize("s,causal", [(256, False), (640, True), (2304, True)])
def test_sparse_matches_oracle(fa, s, causal):
    flash_attn, cuda = fa
    g = gen(s)
    b, h, h_k = 1, 4, 2
    q, k, v, cnt, offs, block_m = _sparse_inputs(g, b, s, h, h_k, 0.4, causal)
    nq = cnt.shape[2]
    cc = torch.zeros(b, h, nq, dtype=torch.int32)
    ci = torch.zeros(b, h, nq, 1, dtype=torch.int32)
    out, lse = flash_attn.sparse_attn_func(q.cuda(), k.cuda(), v.cuda(), cnt.cuda(), offs.cuda(), cc.cuda(), ci.cuda(),
                                           causal=causal, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref32, ref_lse = O.sparse_attention_ref(q, k, v, cnt, offs, causal, block_m)
    ref32f, _ = O.attention_ref(q, k, v, causal=causal, out_dtype=torch.float32,
                                extra_mask=O.block_lists_to_dense_mask(cnt, offs, s, s, block_m))
    ref_pt, _ = O.attention_ref(q, k, v, causal=causal, upcast=False, reorder_ops=True,
                                extra_mask=O.block_lists_to_dense_mask(cnt, offs, s, s, block_m))
    assert_close_to_oracle(out.cpu(), ref32f, ref_pt, mult=2.0, eps=2 ** -8, what=f"sparse {s}")
    _check_lse(lse.cpu(), ref_lse)
    cs = torch.nn.functional.cosine_similarity(out.cpu().float().flatten(), ref32f.flatten(), dim=0).item()
    assert cs > 0.9999                                     # tests/test_spas_fa2_attn.py:64-110 asks > 0.99


@pytest.mark.parametrize("max_len,causal", [(700, True), (700, False), (2300, True)])
def test_varlen_sparse_matches_oracle(fa, max_len, causal):
    """Tile lists over packed sequences (the reference binding's varlen_fwd_sparse, flash_api_sparse.cpp:339-558): lists
    of shape (batch, heads, NUM_ROWS of the longest sequence, NNZ_S), key offsets relative to each sequence."""
    _, cuda = fa
    g = gen(7000 + max_len)
    lens = [max_len, 130, 64, max_len // 2 + 3]
    b, h, h_k = len(lens), 4, 2
    block_m = O.sparse_block_m(max_len)
    nq, nk = (max_len + block_m - 1) // block_m, (max_len + 127) // 128
    tm = torch.rand(b, h, nq, nk, generator=g) < 0.5
    if causal:
        qi = torch.arange(nq).view(-1, 1) * block_m
        ki = torch.arange(nk).view(1, -1) * 128
        tm &= (ki <= qi + block_m - 1)
        tm |= (ki <= qi) & (qi < ki + 128)
    tm[..., 0] = True
    cnt, offs = O.tile_mask_to_block_lists(tm, block_m=block_m, block_n=64, tile_n=128)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    total = sum(lens)
    q, k, v = randn(g, total, h, 128), randn(g, total, h_k, 128), randn(g, total, h_k, 128)
    cc = torch.zeros(b, h, nq, dtype=torch.int32)
    ci = torch.zeros(b, h, nq, 1, dtype=torch.int32)
    out, lse = cuda.varlen_fwd_sparse(q.cuda(), k.cuda(), v.cuda(), cnt.cuda(), offs.cuda(), cc.cuda(), ci.cuda(), None,
                                      cu.cuda(), cu.cuda(), None, None, max_len, max_len, 0.0, 128 ** -0.5, False, causal,
                                      0.0, False, None)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert lse.shape == (h, total)
    for i, L in enumerate(lens):
        lo, hi = int(cu[i]), int(cu[i + 1])
        qi_, ki_, vi_ = q[lo:hi][None], k[lo:hi][None], v[lo:hi][None]
        mask = O.block_lists_to_dense_mask(cnt[i:i + 1], offs[i:i + 1], L, L, block_m)
        ref32, ref_lse = O.attention_ref(qi_, ki_, vi_, causal=causal, out_dtype=torch.float32, extra_mask=mask)
        ref_pt, _ = O.attention_ref(qi_, ki_, vi_, causal=causal, upcast=False, reorder_ops=True, extra_mask=mask)
        assert_close_to_oracle(out[lo:hi][None].cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"varlen sparse seq {i}")
        _check_lse(lse[:, lo:hi].cpu(), ref_lse[0])


def test_sparse_manual_two_block_selection(fa):
    """The reference's own sparse test case (tests/test_spas_fa2_attn.py:64-110): every q block attends K rows
    [0, 64) and [128, 192) only."""
    flash_attn, cuda = fa
    g = gen(42)
    b, s, h = 2, 256, 2
    q, k, v = randn(g, b, s, h, 128), randn(g, b, s, h, 128), randn(g, b, s, h, 128)
    nq = s // 64
    cnt = torch.full((b, h, nq), 2, dtype=torch.int32)
    offs = torch.full((b, h, nq, nq), 10_000_000, dtype=torch.int32)
    offs[..., 0] = 0
    offs[..., 1] = 128
    cc = torch.zeros(b, h, nq, dtype=torch.int32)
    ci = torch.zeros(b, h, nq, 1, dtype=torch.int32)
    out = flash_attn.sparse_attn_func(q.cuda(), k.cuda(), v.cuda(), cnt.cuda(), offs.cuda(), cc.cuda(), ci.cuda(), causal=False)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ks = torch.cat([k[:, 0:64], k[:, 128:192]], dim=1)
    vs = torch.cat([v[:, 0:64], v[:, 128:192]], dim=1)
    ref32, _ = O.attention_ref(q, ks, vs, out_dtype=torch.float32)
    ref_pt, _ = O.attention_ref(q, ks, vs, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what="sparse manual")
    # the vertical part of the pattern is not taken: a non-zero column_count is caught on the device (the call itself
    # does not synchronise) and reported by the status word
    cc[1, 0, 2] = 3
    flash_attn.sparse_attn_func(q.cuda(), k.cuda(), v.cuda(), cnt.cuda(), offs.cuda(), cc.cuda(), ci.cuda(), causal=False)
    torch.cuda.synchronize()
    assert cuda.device_status() == 15      # FA_B200_ERR_DEVICE_UNSUPPORTED, cleared by the read
    assert cuda.device_status() == 0


def test_prefill_rejects_what_the_path_does_not_do(fa):
    flash_attn, cuda = fa
    q = torch.zeros(1, 16, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError):
        flash_attn.flash_attn_func(q, q, q, dropout_p=0.1)
    with pytest.raises(NotImplementedError):
        flash_attn.flash_attn_func(q, q, q, softcap=30.0)
    with pytest.raises(RuntimeError):
        flash_attn.flash_attn_func(q[..., :96], q[..., :96], q[..., :96])
    with pytest.raises(RuntimeError):
        flash_attn.flash_attn_func(q, q[:, :, :1].expand(1, 16, 3, 128), q)


def test_all_prefill_kernels_agree_on_gqa(fa, monkeypatch):
    """Dense GQA prefill normally runs on the persistent kernel with double-buffered scores; the two-head
    persistent kernel and the one-tile kernel (block-sparse lists) must give the same answer when forced."""
    flash_attn, cuda = fa
    g = gen(2024)
    lens = [300, 1, 650, 128, 1500]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
    q, k, v = randn(g, sum(lens), 8, 128).cuda(), randn(g, sum(lens), 2, 128).cuda(), randn(g, sum(lens), 2, 128).cuda()
    ref32, ref_lse = O.attention_varlen_ref(q.cpu(), k.cpu(), v.cpu(), cu.cpu(), cu.cpu(), causal=True, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q.cpu(), k.cpu(), v.cpu(), cu.cpu(), cu.cpu(), causal=True, upcast=False, reorder_ops=True)
    outs = {}
    for kern in ("dense", "pair", "single"):
        monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kern)
        o, l = flash_attn.flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True, return_softmax_lse=True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert_close_to_oracle(o.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=kern)
        _check_lse(l.cpu(), ref_lse)
        outs[kern] = o.cpu()
    assert max_err(outs["dense"], outs["pair"]) <= 2 ** -6 and max_err(outs["dense"], outs["single"]) <= 2 ** -6


@pytest.mark.parametrize("page", [16, 64, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_prefill_reads_pages_directly(fa, page, dtype):
    """flash_attn_varlen_func(block_table=...): K/V in a paged pool (NaN-poisoned unused pages and tails), packed
    varlen q, causal mask bottom-right aligned to each sequence's key count (prefix-cache prefill)."""
    from _util import clean_nan, make_paged
    flash_attn, cuda = fa
    g = gen(500 + page)
    lens_k = [300, 130, 1000, 64, 257]
    lens_q = [300, 2, 129, 64, 200]           # full prefill, tiny chunk, chunk of a long prefix, exact tile, ragged
    h, h_k = 8, 2
    kc, vc, bt, sl = make_paged(g, lens_k, h_k, page, dtype)
    q = randn(g, sum(lens_q), h, 128, dtype=dtype)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cq.cuda(), None, max(lens_q), max(lens_k),
                                                 seqused_k=sl.cuda(), causal=True, block_table=bt.cuda(),
                                                 return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qi = q[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        ref32, ref_lse = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qi, ki, vi, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out[int(cq[i]):int(cq[i + 1])].cpu()[None], ref32, ref_pt, mult=2.0, eps=2 ** -8,
                               what=f"paged prefill seq {i} page {page}")
        _check_lse(lse[:, int(cq[i]):int(cq[i + 1])].cpu(), ref_lse[0])


@pytest.mark.parametrize("kernel,h,h_k", [("dense", 4, 4), ("dense", 6, 2), ("dense", 8, 2), ("single", 6, 2), ("pair", 8, 2)])
@pytest.mark.parametrize("page,dtype", [(16, torch.bfloat16), (64, torch.float8_e4m3fn), (256, torch.float16)])
def test_paged_prefill_on_each_kernel(fa, monkeypatch, kernel, h, h_k, page, dtype):
    """Every prefill kernel reads K/V through the block table: the persistent double-buffered kernel (MHA, odd and even
    groups), the one-tile kernel and the two-tile kernel over NaN-poisoned pools, against the oracle."""
    from _util import clean_nan, make_paged
    flash_attn, cuda = fa
    fp8 = dtype == torch.float8_e4m3fn
    g = gen(700 + page + h)
    lens_k = [300, 130, 1000, 64, 257]
    lens_q = [300, 2, 129, 64, 200]
    kc, vc, bt, sl = make_paged(g, lens_k, h_k, page, torch.bfloat16 if fp8 else dtype)
    q = randn(g, sum(lens_q), h, 128, dtype=torch.bfloat16 if fp8 else dtype)
    if fp8:   # NaN-poisoned e4m3 pools: every byte 0x7f outside the sequences
        nan_k, nan_v = torch.isnan(kc), torch.isnan(vc)
        kc, vc, q = [t.nan_to_num(0.0).to(dtype) for t in (kc, vc, q)]
        kc.view(torch.uint8)[nan_k] = 0x7f
        vc.view(torch.uint8)[nan_v] = 0x7f
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kernel)
    out = flash_attn.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cq.cuda(), None, max(lens_q), max(lens_k),
                                            seqused_k=sl.cuda(), causal=True, block_table=bt.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert ("prefill_" + kernel) in cuda.last_launch_info()
    kcc, vcc = (kc.float().nan_to_num(0.0), vc.float().nan_to_num(0.0)) if fp8 else (clean_nan(kc), clean_nan(vc))
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qi = q[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        got = out[int(cq[i]):int(cq[i + 1])].cpu()[None]
        if fp8:
            ref32, _ = O.attention_ref(qi.float(), ki, vi, causal=True, out_dtype=torch.float32)
            ref_p, _ = O.attention_ref(qi.float(), ki, vi, causal=True, out_dtype=torch.float32,
                                       intermediate_dtype=torch.float8_e4m3fn)
            assert max_err(got, ref32) <= 2 * max_err(ref_p, ref32) + 2 ** -6, (kernel, i)
        else:
            ref32, _ = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32)
            ref_pt, _ = O.attention_ref(qi, ki, vi, causal=True, upcast=False, reorder_ops=True)
            assert_close_to_oracle(got, ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"paged prefill {kernel} seq {i} page {page}")


def test_kvcache_call_with_several_query_tokens(fa):
    """flash_attn_with_kvcache with seqlen_q > 1 (speculative / chunked decoding) over the paged cache."""
    from _util import clean_nan, make_paged
    flash_attn, cuda = fa
    g = gen(77)
    lens = [9, 500, 128, 1031]
    h, h_k, sq = 16, 4, 7
    kc, vc, bt, sl = make_paged(g, lens, h_k, 64, torch.bfloat16)
    q = randn(g, len(lens), sq, h, 128)
    for causal in (True, False):
        out, lse = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(),
                                                      block_table=bt.cuda(), causal=causal, return_softmax_lse=True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        for i, L in enumerate(lens):
            ki, vi = O.gather_paged_kv(clean_nan(kc), bt[i], L)[None], O.gather_paged_kv(clean_nan(vc), bt[i], L)[None]
            ref32, ref_lse = O.attention_ref(q[i:i + 1], ki, vi, causal=causal, out_dtype=torch.float32)
            ref_pt, _ = O.attention_ref(q[i:i + 1], ki, vi, causal=causal, upcast=False, reorder_ops=True)
            assert_close_to_oracle(out[i:i + 1].cpu(), ref32, ref_pt, mult=3.0, eps=2 ** -8, what=f"kvcache sq=7 seq {i}")
            _check_lse(lse[i:i + 1].cpu(), ref_lse)


@pytest.mark.parametrize("page", [16, 128])
def test_paged_layout_bhsd_gives_identical_bits(fa, page):
    """layout "bhsd" pools (num_blocks, nheads_k, page, d) are read through strides: the same values as the bshd
    pools, so prefill and decode outputs must be bit-identical to the bshd calls (reference layouts:
    flash_attn_interface.py:2223-2237; vllm_flash_attn_with_kvcache layout 1 / 2, :2633-2775)."""
    from _util import clean_nan, make_paged
    flash_attn, cuda = fa
    g = gen(900 + page)
    lens_k, lens_q, h, h_k = [300, 130, 1000], [300, 2, 129], 8, 2
    kc, vc, bt, sl = make_paged(g, lens_k, h_k, page, torch.bfloat16, poison=False)
    q = randn(g, sum(lens_q), h, 128)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32).cuda()
    kc_d, vc_d = kc.cuda(), vc.cuda()
    kc_t, vc_t = kc_d.permute(0, 2, 1, 3).contiguous(), vc_d.permute(0, 2, 1, 3).contiguous()   # real bhsd storage
    args = dict(seqused_k=sl.cuda(), causal=True, block_table=bt.cuda())
    o1 = flash_attn.flash_attn_varlen_func(q.cuda(), kc_d, vc_d, cq, None, max(lens_q), max(lens_k), **args)
    o2 = flash_attn.flash_attn_varlen_func(q.cuda(), kc_t, vc_t, cq, None, max(lens_q), max(lens_k), layout="bhsd", **args)
    assert torch.equal(o1, o2)
    qd = randn(g, len(lens_k), 1, h, 128).cuda()
    d1 = flash_attn.flash_attn_with_kvcache(qd, kc_d, vc_d, cache_seqlens=sl.cuda(), block_table=bt.cuda(), causal=True)
    d2 = flash_attn.vllm_flash_attn_with_kvcache(qd, kc_t, vc_t, cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                 causal=True, layout=1, max_seqlen_k=max(lens_k))
    d3 = flash_attn.vllm_flash_attn_with_kvcache(qd, kc_d, vc_d, cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                 causal=True, layout=2)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert torch.equal(d1, d2) and torch.equal(d1, d3)
    ref32, _ = O.paged_decode_ref(qd.cpu(), kc, vc, sl, bt, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(qd.cpu(), kc, vc, sl, bt, upcast=False, reorder_ops=True)
    assert_close_to_oracle(d2.cpu(), ref32, ref_pt, mult=2.0, what="bhsd decode")
    if page % 64 == 0:
        # layout 0: K as bhsd, V stored transposed (num_blocks, nheads_k, d, page); the decode kernel reads it as it is
        vc_tt = vc_d.permute(0, 2, 3, 1).contiguous()
        d4 = flash_attn.vllm_flash_attn_with_kvcache(qd, kc_t, vc_tt, cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                     causal=True)          # layout 0 is the reference's default
        cq1 = torch.arange(len(lens_k) + 1, dtype=torch.int32, device="cuda")
        d5 = flash_attn.flash_attn_varlen_func(qd[:, 0], kc_t, vc_tt, cq1, None, 1, max(lens_k), seqused_k=sl.cuda(),
                                               causal=True, block_table=bt.cuda(), layout="custom")
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert torch.equal(d1, d4) and torch.equal(d1[:, 0], d5)
        # prefill over the transposed V pool: the same values reach the tensor cores through a K-major operand
        o3 = flash_attn.flash_attn_varlen_func(q.cuda(), kc_t, vc_tt, cq, None, max(lens_q), max(lens_k), layout="custom", **args)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert max_err(o3, o1) <= 2 ** -6
    else:
        with pytest.raises(RuntimeError):          # layout 0 needs pages of 64 * n
            flash_attn.vllm_flash_attn_with_kvcache(qd, kc_t, vc_d.permute(0, 2, 3, 1).contiguous(), cache_seqlens=sl.cuda(),
                                                    block_table=bt.cuda(), causal=True)


def test_torch_ops_reach_the_same_kernels(fa):
    """flash_attn::_flash_attn_forward and flash_attn2_c_op::varlen_fwd / fwd_kvcache (the names the reference registers)
    give the same bits as the Python API."""
    from _util import make_paged
    flash_attn, cuda = fa
    g = gen(321)
    q, k, v = randn(g, 2, 200, 8, 128).cuda(), randn(g, 2, 200, 2, 128).cuda(), randn(g, 2, 200, 2, 128).cuda()
    scale = 128 ** -0.5
    o1 = flash_attn.flash_attn_func(q, k, v, causal=True)
    o2, lse, _, _ = torch.ops.flash_attn._flash_attn_forward(q, k, v, 0.0, scale, True, -1, -1, 0.0, None, False)
    assert torch.equal(o1, o2) and lse.shape == (2, 8, 200)
    cu = torch.tensor([0, 150, 400], dtype=torch.int32, device="cuda")
    qv, kv, vv = q.reshape(400, 8, 128), k.reshape(400, 2, 128), v.reshape(400, 2, 128)
    o3 = flash_attn.flash_attn_varlen_func(qv, kv, vv, cu, cu, 250, 250, causal=True)
    o4, _, _, _ = torch.ops.flash_attn2_c_op.varlen_fwd(qv, kv, vv, None, cu, cu, None, None, None, None, 250, 250, 0.0,
                                                         scale, False, True, -1, -1, 0.0, False)
    assert torch.equal(o3, o4)
    kc, vc, bt, sl = make_paged(g, [70, 300], 2, 64, torch.bfloat16, poison=False)
    qd = randn(g, 2, 1, 8, 128).cuda()
    o5 = flash_attn.flash_attn_with_kvcache(qd, kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(), causal=True)
    o6, _ = torch.ops.flash_attn2_c_op.fwd_kvcache(qd, kc.cuda(), vc.cuda(), None, None, sl.cuda(), None, None, None, None,
                                                   bt.cuda(), None, None, scale, True, -1, -1, 0.0, True, 0)
    torch.cuda.synchronize()
    assert torch.equal(o5, o6)


@pytest.mark.parametrize("page", [64, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_prefill_over_transposed_v_pool(fa, page, dtype):
    """Layout "custom" (the reference's paged layout 0, flash_attn_interface.py:2223-2227): K (num_blocks, h_k, page, d),
    V (num_blocks, h_k, d, page).  Unused pages and the rows / columns past each sequence's end are NaN: nothing past
    the end may reach the output.  Also through flash_attn_with_kvcache with many query tokens."""
    from _util import clean_nan, make_paged
    flash_attn, cuda = fa
    g = gen(777 + page)
    lens_k = [300, 130, 1000, 64, 257, 960]
    lens_q = [300, 2, 129, 64, 200, 17]
    h, h_k = 8, 2
    kc, vc, bt, sl = make_paged(g, lens_k, h_k, page, dtype)
    q = randn(g, sum(lens_q), h, 128, dtype=dtype)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    kc_t = kc.cuda().permute(0, 2, 1, 3).contiguous()
    vc_tt = vc.cuda().permute(0, 2, 3, 1).contiguous()
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), kc_t, vc_tt, cq.cuda(), None, max(lens_q), max(lens_k),
                                                 seqused_k=sl.cuda(), causal=True, block_table=bt.cuda(), layout="custom",
                                                 return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qi = q[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        ref32, ref_lse = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qi, ki, vi, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out[int(cq[i]):int(cq[i + 1])].cpu()[None], ref32, ref_pt, mult=2.0, eps=2 ** -8,
                               what=f"transposed V pool seq {i} page {page}")
        _check_lse(lse[:, int(cq[i]):int(cq[i + 1])].cpu(), ref_lse[0])
    # the kvcache entry with 40 query tokens per sequence (40 x 4 rows: beyond the decode tile) takes the same kernel
    lens2 = [300, 130, 1000, 64]
    qd = randn(g, len(lens2), 40, h, 128, dtype=dtype)
    o2 = flash_attn.vllm_flash_attn_with_kvcache(qd.cuda(), kc_t, vc_tt, cache_seqlens=sl[:4].cuda(), block_table=bt[:4].cuda(),
                                                 causal=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    for i, lk in enumerate(lens2):
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        ref32, _ = O.attention_ref(qd[i][None], ki, vi, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qd[i][None], ki, vi, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(o2[i].cpu()[None], ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"kvcache transposed V seq {i}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kernel", ["pair", "dense", "single"])
def test_scores_that_outgrow_the_running_maximum(fa, monkeypatch, dtype, kernel):
    """Keys whose scores grow by hundreds of log2 units from one key tile to the next (and rows whose first tiles are
    fully masked by a window): every tile forces the rescale of O and of the row sum, down to a factor of zero."""
    flash_attn, cuda = fa
    monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kernel)
    g = gen(60)
    b, s, h, h_k = 1, 1024, 4, 2
    q = randn(g, b, s, h, 128, dtype=dtype)
    k = randn(g, b, s, h_k, 128, dtype=dtype)
    v = randn(g, b, s, h_k, 128, dtype=dtype)
    # key tile t is scaled by 4^t / 16: the largest scores of successive tiles are hundreds of log2 units apart
    ramp = (4.0 ** (torch.arange(s) // 128).float() / 16).view(1, s, 1, 1)
    k = (k.float() * ramp).to(dtype)
    for causal, window in ((False, (-1, -1)), (True, (-1, -1)), (False, (200, 300))):
        out, lse, _ = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=causal, window_size=window,
                                                 return_attn_probs=True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        ref32, ref_lse = O.attention_ref(q, k, v, causal=causal, window_size=window, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(q, k, v, causal=causal, window_size=window, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"{kernel} causal={causal} window={window}")
        fin = torch.isfinite(ref_lse)
        assert (lse.cpu()[fin] - ref_lse[fin]).abs().max() < 1e-3 * max(1.0, ref_lse[fin].abs().max().item())


@pytest.mark.parametrize("h,h_k", [(8, 2), (6, 2)])      # even group: two-tile kernel; odd group: one-tile kernel
@pytest.mark.parametrize("page", [16, 64, 256])
def test_fp8_paged_prefill(fa, page, h, h_k):
    """e4m3 queries over an e4m3 paged cache with several query tokens per sequence (chunked prefill in FP8), the
    unused pages and tails poisoned with the e4m3 NaN pattern.  Rule of the reference's FP8 tests: error <= 2 x the error
    of the same math with P round-tripped through e4m3, cosine difference < 1e-3."""
    from _util import make_paged
    flash_attn, cuda = fa
    g = gen(8800 + page + h)
    lens_k = [300, 130, 1000, 64, 257]
    lens_q = [300, 2, 129, 64, 200]
    n = len(lens_k)
    kc16, vc16, bt, sl = make_paged(g, lens_k, h_k, page, torch.bfloat16, poison=False)
    q16 = randn(g, sum(lens_q), h, 128)
    q8, qd = O.quantize_e4m3_per_tensor(q16)
    k8, kd = O.quantize_e4m3_per_tensor(kc16)
    v8, vd = O.quantize_e4m3_per_tensor(vc16)
    # poison what no sequence owns: spare pages and the rows past each sequence's end (0x7f = e4m3 NaN)
    k_dev, v_dev = k8.clone().view(torch.uint8), v8.clone().view(torch.uint8)
    used = torch.zeros(k8.shape[0], dtype=torch.bool)
    for i, L in enumerate(lens_k):
        nb = (L + page - 1) // page
        used[bt[i, :nb].long()] = True
        if L % page:
            last = int(bt[i, nb - 1])
            k_dev[last, L % page:] = 0x7f
            v_dev[last, L % page:] = 0x7f
    k_dev[~used] = 0x7f
    v_dev[~used] = 0x7f
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    out = flash_attn.flash_attn_varlen_func(q8.cuda(), k_dev.view(torch.float8_e4m3fn).cuda(), v_dev.view(torch.float8_e4m3fn).cuda(),
                                            cq.cuda(), None, max(lens_q), max(lens_k), seqused_k=sl.cuda(), causal=True,
                                            block_table=bt.cuda(), q_descale=qd.cuda(), k_descale=kd.cuda(), v_descale=vd.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert out.dtype == torch.bfloat16 and not torch.isnan(out.float()).any()
    kw = dict(q_descale=qd.expand(1, h_k), k_descale=kd.expand(1, h_k), v_descale=vd.expand(1, h_k))
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qi = q8[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(k8, bt[i], lk)[None], O.gather_paged_kv(v8, bt[i], lk)[None]
        ref32, _ = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32, **kw)
        ref_p8, _ = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32, intermediate_dtype=torch.float8_e4m3fn, **kw)
        got = out[int(cq[i]):int(cq[i + 1])].cpu()[None]
        assert max_err(got, ref32) <= 2 * max_err(ref_p8, ref32) + 2 ** -7, (i, page)
        assert cos_diff(got, ref32) < 1e-3, (i, page)


@pytest.mark.parametrize("h,h_k", [(8, 2), (3, 1)])      # two-tile and one-tile kernel
def test_paged_prefill_empty_and_short_caches(fa, h, h_k):
    """Paged prefill where a sequence has no keys at all, or fewer keys than queries (the first rows then see nothing:
    zero output, LSE = +inf), next to ordinary sequences."""
    from _util import clean_nan, make_paged
    flash_attn, cuda = fa
    g = gen(4711 + h)
    page = 64
    lens_k = [0, 40, 700, 1, 129]
    lens_q = [17, 100, 300, 64, 129]
    kc, vc, bt, sl = make_paged(g, [max(l, 1) for l in lens_k], h_k, page, torch.bfloat16)
    sl = torch.tensor(lens_k, dtype=torch.int32)
    q = randn(g, sum(lens_q), h, 128)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cq.cuda(), None, max(lens_q), max(lens_k),
                                                 seqused_k=sl.cuda(), causal=True, block_table=bt.cuda(), return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert not torch.isnan(out.float()).any()
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        o_i, l_i = out[int(cq[i]):int(cq[i + 1])].cpu(), lse[:, int(cq[i]):int(cq[i + 1])].cpu()
        if lk == 0:
            assert torch.all(o_i == 0) and torch.all(l_i == float("inf"))
            continue
        qi = q[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        ref32, ref_lse = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qi, ki, vi, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(o_i[None], ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"seq {i}")
        _check_lse(l_i, ref_lse[0])
        if lq > lk:
            assert torch.all(o_i[:lq - lk] == 0)
