"""GPU parity for head dimensions other than 128 (64, 192, 256; fp16 / bf16): the decode kernel, the LSE combine and
the one-tile prefill kernel (fixed length, packed varlen, paged K/V, tile lists) against the CPU oracle, with the
tolerance rule of the reference's tests (tests/test_flash_attn.py:989: err <= 2 x the same-dtype PyTorch error)."""
import os

import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, clean_nan, gen, make_paged, max_err, randn

pytestmark = pytest.mark.gpu

DIMS = [64, 192, 256]


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


@pytest.mark.parametrize("partition", [None, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", DIMS)
def test_decode_other_head_dims(fa, d, dtype, partition):
    flash_attn, cuda = fa
    lens, h, hk, page = [1, 200, 64, 513, 2000, 0], 8, 2, 64
    g = gen(d * 13 + (partition or 0))
    kc, vc, bt, sl = make_paged(g, lens, hk, page, dtype, d=d)
    q = randn(g, len(lens), 1, h, d, dtype=dtype)
    if partition is not None:
        os.environ["FA_B200_DECODE_PARTITION"] = str(partition)
    try:
        out, lse = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(),
                                                      block_table=bt.cuda(), causal=True, return_softmax_lse=True)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    ref32, ref_lse = O.paged_decode_ref(q, kcc, vcc, sl, bt, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q, kcc, vcc, sl, bt, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=3.0, eps=1e-5 + 2 ** -8, what=f"decode d={d}")
    fin = torch.isfinite(ref_lse)
    assert max_err(lse.cpu()[fin], ref_lse[fin]) < 1e-3
    assert torch.all(out[-1] == 0)        # the empty sequence


@pytest.mark.parametrize("d", DIMS)
def test_decode_few_tokens_sinks_and_window_other_head_dims(fa, d):
    """Two query tokens per sequence (causal among themselves), attention sinks and a sliding window at once."""
    flash_attn, cuda = fa
    lens, h, hk, page, sq, win = [300, 77, 1024], 8, 2, 64, 2, 150
    g = gen(d + 5)
    kc, vc, bt, sl = make_paged(g, lens, hk, page, torch.bfloat16, d=d)
    q = randn(g, len(lens), sq, h, d)
    s_aux = torch.randn(h, generator=g).to(torch.bfloat16)
    out = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                             causal=True, window_size=(win, 0), s_aux=s_aux.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    for i, L in enumerate(lens):
        ki, vi = O.gather_paged_kv(kcc, bt[i], L)[None], O.gather_paged_kv(vcc, bt[i], L)[None]
        ref32, _ = O.attention_ref(q[i][None], ki, vi, causal=True, out_dtype=torch.float32, s_aux=s_aux, window_size=(win, 0))
        ref_pt, _ = O.attention_ref(q[i][None], ki, vi, causal=True, upcast=False, reorder_ops=True, s_aux=s_aux,
                                    window_size=(win, 0))
        assert_close_to_oracle(out[i].cpu()[None], ref32, ref_pt, mult=3.0, eps=1e-5 + 2 ** -8, what=f"seq {i} d={d}")


@pytest.mark.parametrize("d", [64, 256])
def test_combine_other_head_dims(fa, d):
    _, cuda = fa
    g = gen(d)
    parts, rows = 7, 12
    o = torch.randn(parts, rows, d, generator=g)
    l = torch.randn(parts, rows, generator=g) * 3
    l[2, 5] = float("-inf")           # an empty partition: its O is never read on the device
    o_dev = o.clone()
    o_dev[2, 5] = float("nan")
    o[2, 5] = 0
    out, lse = cuda.combine(o_dev.cuda(), l.cuda(), out_dtype=torch.float32, h=4)
    ref_o, ref_l = O.merge_partials_ref(o, l)
    assert max_err(out.cpu(), ref_o) < 1e-5 and max_err(lse.cpu(), ref_l) < 1e-5


SHAPES = [
    # b, sq, sk, h, h_k, causal
    (2, 128, 128, 4, 1, True),
    (1, 384, 384, 8, 2, True),
    (2, 200, 333, 4, 4, False),
    (1, 64, 513, 2, 1, True),
    (1, 300, 100, 2, 2, True),
]


@pytest.mark.parametrize("b,sq,sk,h,h_k,causal", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", DIMS)
def test_fixed_other_head_dims(fa, d, dtype, b, sq, sk, h, h_k, causal):
    flash_attn, cuda = fa
    g = gen(sq * 7 + sk * 3 + h + d)
    q, k, v = randn(g, b, sq, h, d, dtype=dtype), randn(g, b, sk, h_k, d, dtype=dtype), randn(g, b, sk, h_k, d, dtype=dtype)
    out, lse, _ = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=causal, return_attn_probs=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref32, ref_lse = O.attention_ref(q, k, v, causal=causal, out_dtype=torch.float32)
    ref_pt, _ = O.attention_ref(q, k, v, causal=causal, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"fixed {sq}x{sk} d={d}")
    _check_lse(lse.cpu(), ref_lse)


@pytest.mark.parametrize("d", DIMS)
def test_varlen_sinks_window_other_head_dims(fa, d):
    flash_attn, cuda = fa
    g = gen(99 + d)
    lens, h, h_k = [1, 127, 128, 129, 700, 33], 8, 2
    total = sum(lens)
    q, k, v = randn(g, total, h, d), randn(g, total, h_k, d), randn(g, total, h_k, d)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                 causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref32, ref_lse = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"varlen d={d}")
    _check_lse(lse.cpu(), ref_lse)
    # fixed length with sinks and a two-sided window
    s_aux = torch.randn(h, generator=g).to(torch.bfloat16)
    qf, kf, vf = randn(g, 2, 300, h, d), randn(g, 2, 300, h_k, d), randn(g, 2, 300, h_k, d)
    out = flash_attn.flash_attn_func(qf.cuda(), kf.cuda(), vf.cuda(), window_size=(100, 20), s_aux=s_aux.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref32, _ = O.attention_ref(qf, kf, vf, out_dtype=torch.float32, s_aux=s_aux, window_size=(100, 20))
    ref_pt, _ = O.attention_ref(qf, kf, vf, upcast=False, reorder_ops=True, s_aux=s_aux, window_size=(100, 20))
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"window + sinks d={d}")


@pytest.mark.parametrize("page", [16, 128])
@pytest.mark.parametrize("d", DIMS)
def test_paged_prefill_other_head_dims(fa, d, page):
    flash_attn, cuda = fa
    g = gen(500 + page + d)
    lens_k, lens_q, h, h_k = [300, 130, 1000, 64], [300, 2, 129, 64], 8, 2
    kc, vc, bt, sl = make_paged(g, lens_k, h_k, page, torch.bfloat16, d=d)
    q = randn(g, sum(lens_q), h, d)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    out = flash_attn.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cq.cuda(), None, max(lens_q), max(lens_k),
                                            seqused_k=sl.cuda(), causal=True, block_table=bt.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qi = q[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        ref32, _ = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qi, ki, vi, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out[int(cq[i]):int(cq[i + 1])].cpu()[None], ref32, ref_pt, mult=2.0, eps=2 ** -8,
                               what=f"paged prefill seq {i} page {page} d={d}")


def test_other_head_dims_are_for_16bit_plain_layouts(fa):
    flash_attn, cuda = fa
    q = torch.zeros(1, 128, 2, 64, device="cuda").to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError):
        flash_attn.flash_attn_func(q, q, q)
    q = torch.zeros(1, 128, 2, 96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        flash_attn.flash_attn_func(q, q, q)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_qk_192_v_128(fa, dtype):
    """q / k with head dimension 192 and v / out with 128 (the multi-head latent attention prefill shape): fixed length,
    packed varlen and paged K/V."""
    flash_attn, cuda = fa
    g = gen(192128)
    h, h_k = 8, 2
    q, k, v = randn(g, 2, 300, h, 192, dtype=dtype), randn(g, 2, 450, h_k, 192, dtype=dtype), randn(g, 2, 450, h_k, 128, dtype=dtype)
    out, lse, _ = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=True, return_attn_probs=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0 and out.shape == (2, 300, h, 128)
    ref32, ref_lse = O.attention_ref(q, k, v, causal=True, out_dtype=torch.float32)
    ref_pt, _ = O.attention_ref(q, k, v, causal=True, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what="192/128 fixed")
    _check_lse(lse.cpu(), ref_lse)
    lens = [1, 127, 129, 700, 33]
    total = sum(lens)
    q, k, v = randn(g, total, h, 192, dtype=dtype), randn(g, total, h_k, 192, dtype=dtype), randn(g, total, h_k, 128, dtype=dtype)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                 causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0 and out.shape == (total, h, 128)
    ref32, ref_lse = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what="192/128 varlen")
    _check_lse(lse.cpu(), ref_lse)
    # paged K (d 192) and V (d 128) pools sharing one block table
    lens_k, lens_q, page = [300, 130, 1000], [300, 2, 129], 64
    kc, _, bt, sl = make_paged(g, lens_k, h_k, page, dtype, d=192)
    vc = randn(g, kc.shape[0], page, h_k, 128, dtype=dtype)
    q = randn(g, sum(lens_q), h, 192, dtype=dtype)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    out = flash_attn.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cq.cuda(), None, max(lens_q), max(lens_k),
                                            seqused_k=sl.cuda(), causal=True, block_table=bt.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    kcc = clean_nan(kc)
    for i, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qi = q[int(cq[i]):int(cq[i + 1])][None]
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vc, bt[i], lk)[None]
        ref32, _ = O.attention_ref(qi, ki, vi, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qi, ki, vi, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out[int(cq[i]):int(cq[i + 1])].cpu()[None], ref32, ref_pt, mult=2.0, eps=2 ** -8,
                               what=f"192/128 paged seq {i}")


@pytest.mark.parametrize("d", DIMS)
def test_tile_lists_other_head_dims(fa, d):
    """Block-sparse tile lists (sparse_attn_func) with another head dimension."""
    flash_attn, cuda = fa
    g = gen(7 + d)
    b, s, h, h_k = 1, 640, 4, 2
    block_m = O.sparse_block_m(s)
    nq, nk = (s + block_m - 1) // block_m, (s + 127) // 128
    tm = torch.rand(b, h, nq, nk, generator=g) < 0.4
    qi = torch.arange(nq).view(-1, 1) * block_m
    ki = torch.arange(nk).view(1, -1) * 128
    tm &= (ki <= qi + block_m - 1)
    tm |= (ki <= qi) & (qi < ki + 128)        # always keep the diagonal tile
    cnt, offs = O.tile_mask_to_block_lists(tm, block_m=block_m, block_n=64, tile_n=128)
    q, k, v = randn(g, b, s, h, d), randn(g, b, s, h_k, d), randn(g, b, s, h_k, d)
    cc = torch.zeros(b, h, nq, dtype=torch.int32)
    ci = torch.zeros(b, h, nq, 1, dtype=torch.int32)
    out, lse = flash_attn.sparse_attn_func(q.cuda(), k.cuda(), v.cuda(), cnt.cuda(), offs.cuda(), cc.cuda(), ci.cuda(),
                                           causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    mask = O.block_lists_to_dense_mask(cnt, offs, s, s, block_m)
    ref32, ref_lse = O.attention_ref(q, k, v, causal=True, out_dtype=torch.float32, extra_mask=mask)
    ref_pt, _ = O.attention_ref(q, k, v, causal=True, upcast=False, reorder_ops=True, extra_mask=mask)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"tile lists d={d}")
    _check_lse(lse.cpu(), ref_lse)


@pytest.mark.parametrize("d,dv", [(64, 64), (192, 192), (192, 128), (256, 256)])
def test_scores_that_outgrow_the_running_maximum_at_other_head_dims(fa, d, dv):
    """Keys whose scores grow by hundreds of log2 units from one key tile to the next: every tile rescales O.  Above
    d = 128 the kernel computes S of the next key tile before P V of the current one, so the rescale has to wait for the
    product that is still accumulating into O."""
    flash_attn, cuda = fa
    g = gen(61 + d)
    b, s, h, h_k = 1, 1024, 4, 2
    q = randn(g, b, s, h, d)
    k = randn(g, b, s, h_k, d)
    v = randn(g, b, s, h_k, dv)
    ramp = (4.0 ** (torch.arange(s) // 128).float() / 16).view(1, s, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    for causal, window in ((False, (-1, -1)), (True, (-1, -1)), (False, (200, 300)), (True, (17, 0))):
        out = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=causal, window_size=window)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        ref32, _ = O.attention_ref(q, k, v, causal=causal, window_size=window, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(q, k, v, causal=causal, window_size=window, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"d={d}/{dv} causal={causal} window={window}")
