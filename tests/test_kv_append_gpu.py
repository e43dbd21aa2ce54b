"""GPU parity: KV-cache append + rotary embedding inside the decode call (fa_b200_kv_append followed by the
attention over the updated cache).  The cache after the call and the rotated queries are compared bit for bit
with the CPU oracle; the attention output with the reference's error rule
(tests/test_flash_attn.py:3073-3210 is the test these cases follow)."""
import importlib.util
import math
import os

import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, gen, make_paged, randn

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


def _rotary_tables(g, seqlen_ro, rotary_dim, dtype):
    angle = torch.rand(seqlen_ro, rotary_dim // 2, generator=g) * 2 * math.pi
    return torch.cos(angle).to(dtype), torch.sin(angle).to(dtype)


def test_rotary_golden_cases_bit_exact(fa, golden):
    """The rotation of q inside fa_b200_kv_append reproduces the reference's formula (golden fp32 values) after
    one rounding to the element type."""
    _, cuda = fa
    for c in [c for c in golden["cases"] if c["kind"] == "rotary"]:
        x, cos, sin, off = _mg.gen_inputs(c)
        b, sq, h, d = x.shape
        page, hk = 64, 1
        nblk = (c["seqlen_ro"] + page - 1) // page + 1
        kc = torch.zeros(b * nblk, page, hk, d, dtype=x.dtype, device="cuda")
        vc = torch.zeros_like(kc)
        bt = torch.arange(b * nblk, dtype=torch.int32).view(b, nblk).cuda()
        kn = torch.zeros(b, sq, hk, d, dtype=x.dtype, device="cuda")
        q_ro, new_lens = cuda.kv_append(x.cuda(), kc, vc, kn, kn, off.cuda(), bt, cos.cuda(), sin.cuda(),
                                        c["interleaved"], True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert torch.equal(q_ro.cpu(), c["out"].to(x.dtype)), c["name"]
        assert torch.equal(new_lens.cpu(), off + sq)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page", [16, 64, 256])
@pytest.mark.parametrize("rotary_dim,interleaved", [(0, False), (128, False), (64, True), (32, False), (128, True)])
def test_decode_with_append_and_rotary(fa, dtype, page, rotary_dim, interleaved):
    flash_attn, cuda = fa
    g = gen(1000 + page + rotary_dim + (1 if interleaved else 0) + (7 if dtype == torch.float16 else 0))
    h, hk, d = 8, 2, 128
    lens = [0, 1, page - 1, page, 3 * page + 5, 700]
    b = len(lens)
    cap = [L + 1 for L in lens]          # room for the appended token
    kc, vc, bt, _ = make_paged(g, cap, hk, page, dtype, poison=False)
    cache_seqlens = torch.tensor(lens, dtype=torch.int32)
    q = randn(g, b, 1, h, d, dtype=dtype)
    kn = randn(g, b, 1, hk, d, dtype=dtype)
    vn = randn(g, b, 1, hk, d, dtype=dtype)
    cos = sin = None
    if rotary_dim:
        cos, sin = _rotary_tables(g, max(cap) + 4, rotary_dim, dtype)

    # oracle: append on a CPU copy, rotate q, attend over the updated cache
    kc_ref, vc_ref = kc.clone(), vc.clone()
    new_lens = O.kv_append_ref(kc_ref, vc_ref, bt, cache_seqlens, kn, vn, cos, sin, interleaved)
    q_ro = O.rotary_ref(q, cos, sin, cache_seqlens, interleaved) if rotary_dim else q
    ref32, _ = O.paged_decode_ref(q_ro, kc_ref, vc_ref, new_lens, bt, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q_ro, kc_ref, vc_ref, new_lens, bt, upcast=False, reorder_ops=True)

    kc_d, vc_d = kc.cuda(), vc.cuda()
    lens_d = cache_seqlens.cuda()
    out, lse = flash_attn.flash_attn_with_kvcache(
        q.cuda(), kc_d, vc_d, k=kn.cuda(), v=vn.cuda(), rotary_cos=None if cos is None else cos.cuda(),
        rotary_sin=None if sin is None else sin.cuda(), cache_seqlens=lens_d, block_table=bt.cuda(), causal=True,
        rotary_interleaved=interleaved, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    # the cache is updated in place, bit for bit, and only at the appended rows; cache_seqlens is not modified
    assert torch.equal(kc_d.cpu(), kc_ref)
    assert torch.equal(vc_d.cpu(), vc_ref)
    assert torch.equal(lens_d.cpu(), cache_seqlens)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, what="decode+append")


@pytest.mark.parametrize("causal", [True, False])
def test_chunk_append_several_tokens(fa, causal):
    """seqlen_q = seqlen_new = 5 over a paged cache: the keys are rotated at their own positions; the queries at
    their own positions when causal, all at cache_seqlens when not (flash_attn_interface.py:2512-2517)."""
    flash_attn, cuda = fa
    g = gen(77 + causal)
    dtype, page, h, hk, d, sq = torch.bfloat16, 64, 4, 2, 128, 5
    lens = [0, 60, 64, 200]
    b = len(lens)
    kc, vc, bt, _ = make_paged(g, [L + sq for L in lens], hk, page, dtype, poison=False)
    cache_seqlens = torch.tensor(lens, dtype=torch.int32)
    q = randn(g, b, sq, h, d, dtype=dtype)
    kn = randn(g, b, sq, hk, d, dtype=dtype)
    vn = randn(g, b, sq, hk, d, dtype=dtype)
    cos, sin = _rotary_tables(g, 300, 128, dtype)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    new_lens = O.kv_append_ref(kc_ref, vc_ref, bt, cache_seqlens, kn, vn, cos, sin, False)
    q_ro = O.rotary_ref(q, cos, sin, cache_seqlens, False, per_token=causal)
    refs32, refs_pt = [], []
    for i in range(b):
        L = int(new_lens[i])
        kk = O.gather_paged_kv(kc_ref, bt[i], L).unsqueeze(0)
        vv = O.gather_paged_kv(vc_ref, bt[i], L).unsqueeze(0)
        r32, _ = O.attention_ref(q_ro[i:i + 1], kk, vv, causal=causal, out_dtype=torch.float32)
        rpt, _ = O.attention_ref(q_ro[i:i + 1], kk, vv, causal=causal, upcast=False, reorder_ops=True)
        refs32.append(r32)
        refs_pt.append(rpt)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    out = flash_attn.flash_attn_with_kvcache(
        q.cuda(), kc_d, vc_d, k=kn.cuda(), v=vn.cuda(), rotary_cos=cos.cuda(), rotary_sin=sin.cuda(),
        cache_seqlens=cache_seqlens.cuda(), block_table=bt.cuda(), causal=causal, rotary_interleaved=False)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)
    assert_close_to_oracle(out.cpu(), torch.cat(refs32), torch.cat(refs_pt), mult=2.0, what="chunk append")


def test_append_e4m3_copies_bytes(fa):
    _, cuda = fa
    g = gen(5)
    page, hk, d = 64, 2, 128
    lens = torch.tensor([3, 64, 100], dtype=torch.int32)
    kc = torch.randint(0, 120, (8, page, hk, d), generator=g, dtype=torch.uint8)
    vc = torch.randint(0, 120, (8, page, hk, d), generator=g, dtype=torch.uint8)
    bt = torch.tensor([[5, 0], [1, 6], [2, 7]], dtype=torch.int32)
    kn = torch.randint(0, 120, (3, 2, hk, d), generator=g, dtype=torch.uint8)
    vn = torch.randint(0, 120, (3, 2, hk, d), generator=g, dtype=torch.uint8)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    O.kv_append_ref(kc_ref, vc_ref, bt, lens, kn, vn)
    f8 = torch.float8_e4m3fn
    kc_d, vc_d = kc.cuda().view(f8), vc.cuda().view(f8)
    q = torch.zeros(3, 1, 4, d, device="cuda").to(f8)
    _, new_lens = cuda.kv_append(q, kc_d, vc_d, kn.cuda().view(f8), vn.cuda().view(f8), lens.cuda(), bt.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert torch.equal(kc_d.view(torch.uint8).cpu(), kc_ref) and torch.equal(vc_d.view(torch.uint8).cpu(), vc_ref)
    assert new_lens.cpu().tolist() == [5, 66, 102]


def test_append_out_of_range_is_skipped_and_reported(fa):
    """A sequence whose cache is full: the append must not write anywhere and the status word says so."""
    _, cuda = fa
    page, hk, d = 16, 1, 128
    kc = torch.zeros(2, page, hk, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    bt = torch.tensor([[0], [1]], dtype=torch.int32).cuda()
    lens = torch.tensor([16, 3], dtype=torch.int32).cuda()      # sequence 0 has no room left
    kn = torch.ones(2, 1, hk, d, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(2, 1, 2, d, dtype=torch.bfloat16, device="cuda")
    cuda.kv_append(q, kc, vc, kn, kn, lens, bt)
    torch.cuda.synchronize()
    assert cuda.device_status() == 14      # FA_B200_ERR_DEVICE_RANGE, cleared by the read
    assert cuda.device_status() == 0
    assert kc[0].abs().sum().item() == 0 and kc[1, 3].float().sum().item() == d and kc[1].float().sum().item() == d


def test_rejects(fa):
    flash_attn, _ = fa
    q = torch.zeros(1, 1, 2, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16, device="cuda")
    bt = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    lens = torch.zeros(1, dtype=torch.int32, device="cuda")
    cos = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):   # rotary without new k/v
        flash_attn.flash_attn_with_kvcache(q, kc, kc, rotary_cos=cos, rotary_sin=cos, cache_seqlens=lens, block_table=bt)
    with pytest.raises(RuntimeError):   # k without v
        flash_attn.flash_attn_with_kvcache(q, kc, kc, k=q[:, :, :1], cache_seqlens=lens, block_table=bt)
    with pytest.raises(RuntimeError):   # rotary_dim not a multiple of 16
        flash_attn.flash_attn_with_kvcache(q, kc, kc, k=q[:, :, :1], v=q[:, :, :1], rotary_cos=cos[:, :4],
                                           rotary_sin=cos[:, :4], cache_seqlens=lens, block_table=bt)
