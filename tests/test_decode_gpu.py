"""GPU parity: paged-KV decode (fa_b200_decode_paged through the reference-shaped Python API) and the
LSE-combine kernel against the CPU oracle and the committed golden vectors."""
import importlib.util
import os

import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, clean_nan, gen, make_paged, max_err, randn

pytestmark = pytest.mark.gpu

_spec = importlib.util.spec_from_file_location(
    "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
_mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mg)


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    assert os.path.dirname(flash_attn.__file__).endswith(os.path.join("flash-attention-das_b200", "flash_attn"))
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def _run_decode(fa, q, kc, vc, lens, bt, monkeypatch=None, partition=None, **kw):
    flash_attn, cuda = fa
    if partition is not None:
        os.environ["FA_B200_DECODE_PARTITION"] = str(partition)
    else:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    try:
        out, lse = flash_attn.flash_attn_with_kvcache(
            q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens.cuda(), block_table=bt.cuda(), causal=True,
            return_softmax_lse=True, **kw)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    assert cuda.device_status() == 0
    return out.cpu(), lse.cpu()


def test_combine_matches_oracle_and_indexing_is_exact(fa):
    _, cuda = fa
    g = gen(0)
    parts, b, h, d = 9, 3, 8, 128
    o = torch.randn(parts, b * h, d, generator=g)
    lse = torch.randn(parts, b * h, generator=g) * 4
    lse[2] = float("-inf")            # an empty partition
    lse[5, 3] = float("inf")          # the other empty marker
    o[2] = float("nan")               # must never leak through a zero weight
    ref_o, ref_l = O.merge_partials_ref(torch.nan_to_num(o), lse)
    out, l = cuda.combine(o.cuda(), lse.cuda(), out_dtype=torch.float32, h=h)
    assert max_err(out.cpu(), ref_o) < 2e-6 * max(1.0, ref_o.abs().max().item())
    assert max_err(l.cpu(), ref_l) < 1e-5
    # bit-exact slot addressing: with one live partition per row the output must be that partial, bit for bit
    sel = torch.randint(0, parts, (b * h,), generator=g)
    lse1 = torch.full((parts, b * h), float("-inf"))
    lse1[sel, torch.arange(b * h)] = torch.randn(b * h, generator=g)
    o1 = torch.randn(parts, b * h, d, generator=g)
    out1, l1 = cuda.combine(o1.cuda(), lse1.cuda(), out_dtype=torch.float32, h=h)
    assert torch.equal(out1.cpu(), o1[sel, torch.arange(b * h)])
    assert torch.equal(l1.cpu(), lse1[sel, torch.arange(b * h)])
    # per-sequence partition counts: partials past the count are ignored even if they look valid
    ppr = torch.tensor([9, 4, 0], dtype=torch.int32)
    out2, l2 = cuda.combine(o1.cuda(), torch.zeros(parts, b * h).cuda(), out_dtype=torch.bfloat16, h=h,
                            parts_per_row=ppr.cuda())
    ref2, refl2 = O.merge_partials_ref(o1[:4, h:2 * h], torch.zeros(4, h))
    assert max_err(out2.cpu()[h:2 * h], ref2) < 1e-2
    assert torch.all(out2.cpu()[2 * h:] == 0) and torch.all(torch.isinf(l2.cpu()[2 * h:]))


def test_decode_golden_cases(fa, golden):
    for c in [c for c in golden["cases"] if c["kind"] == "paged"]:
        q, kc, vc, lens, bt = _mg.gen_inputs(c)
        out, _ = _run_decode(fa, q, kc, vc, lens, bt)
        ref32, _ = O.paged_decode_ref(q, kc, vc, lens, bt, out_dtype=torch.float32)
        pt, _ = O.paged_decode_ref(q, kc, vc, lens, bt, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out, ref32, pt, mult=3.0, eps=1e-5 + 2 ** -8, what=c["name"])
        # and against the reference-made golden output itself (same dtype, so one rounding apart at most)
        assert max_err(out, c["out"]) <= 2e-2, c["name"]


CASES = [
    # (dtype, batch lens, h, h_k, page, partition override)
    (torch.bfloat16, [1, 63, 64, 65, 300, 1000], 32, 8, 64, None),
    (torch.bfloat16, [517, 2048, 1, 130], 32, 8, 256, 512),
    (torch.float16, [777, 90, 4000], 8, 1, 128, 1024),       # group 8, MQA
    (torch.bfloat16, [40, 0, 257, 5], 16, 1, 16, None),       # group 16, tiny pages, an empty sequence
    (torch.float16, [100, 3000], 4, 4, 32, 512),              # group 1 (MHA)
    (torch.bfloat16, [9000], 32, 8, 256, 512),                # one sequence, 18 partitions
]


@pytest.mark.parametrize("dtype,lens,h,h_k,page,partition", CASES)
def test_decode_matches_oracle(fa, dtype, lens, h, h_k, page, partition):
    g = gen(sum(lens) * 31 + h * 7 + page)
    kc, vc, bt, sl = make_paged(g, lens, h_k, page, dtype)
    q = randn(g, len(lens), 1, h, 128, dtype=dtype)
    out, lse = _run_decode(fa, q, kc, vc, sl, bt, partition=partition)
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    ref32, ref_lse = O.paged_decode_ref(q, kcc, vcc, sl, bt, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q, kcc, vcc, sl, bt, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out, ref32, ref_pt, mult=3.0, eps=1e-5 + 2 ** -8, what=f"decode {lens}")
    assert torch.allclose(out.float(), ref32.float(), atol=1e-2, rtol=1e-2)        # tests/test_pa.py:108-117
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    assert max_err(lse[fin], ref_lse[fin]) < 1e-3
    assert torch.all(lse[~fin] == float("inf"))
    for i, L in enumerate(lens):
        if L == 0:
            assert torch.all(out[i] == 0)


def test_decode_split_invariance_and_determinism(fa):
    g = gen(77)
    lens = [5000, 123, 2500]
    kc, vc, bt, sl = make_paged(g, lens, 8, 64, torch.bfloat16)
    q = randn(g, 3, 1, 32, 128)
    a, la = _run_decode(fa, q, kc, vc, sl, bt, partition=512)
    b, lb = _run_decode(fa, q, kc, vc, sl, bt, partition=4096)
    c, lc = _run_decode(fa, q, kc, vc, sl, bt, partition=512)
    assert torch.equal(a, c) and torch.equal(la, lc)          # bit-identical across runs
    assert max_err(a, b) <= 2 ** -7 and max_err(la, lb) < 1e-4
    # doubling V doubles the output exactly (power-of-two scaling commutes with every rounding step)
    d2, _ = _run_decode(fa, q, kc, (vc.float() * 2).to(vc.dtype), sl, bt, partition=512)
    assert torch.equal(d2.float(), a.float() * 2)


def test_decode_noncontiguous_views_and_out_arg(fa):
    flash_attn, cuda = fa
    g = gen(5)
    lens = [200, 70]
    kc, vc, bt, sl = make_paged(g, lens, 2, 64, torch.float16, poison=False)
    # cache stored as one (pool, page, 2*h_k, d) buffer with K and V interleaved on the head axis
    kv = torch.stack([kc, vc], dim=3).reshape(kc.shape[0], 64, 4, 128).cuda()
    kview, vview = kv[:, :, 0::2], kv[:, :, 1::2]
    q = randn(g, 2, 1, 8, 128, dtype=torch.float16)
    out_buf = torch.zeros(2, 1, 8, 128, dtype=torch.float16, device="cuda")
    ret = flash_attn.flash_attn_with_kvcache(q.cuda(), kview, vview, cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                             out=out_buf)
    assert ret.data_ptr() == out_buf.data_ptr()
    ref32, _ = O.paged_decode_ref(q, kc, vc, sl, bt, out_dtype=torch.float32)
    assert torch.allclose(out_buf.cpu().float(), ref32, atol=1e-2, rtol=1e-2)


def test_decode_fp8_tolerance(fa):
    flash_attn, cuda = fa
    g = gen(31)
    lens = [8192, 100, 1500, 129]
    h, h_k, page = 32, 8, 256
    kc16, vc16, bt, sl = make_paged(g, lens, h_k, page, torch.bfloat16, poison=False)
    q16 = randn(g, len(lens), 1, h, 128)
    q8, qd = O.quantize_e4m3_per_tensor(q16)
    k8, kd = O.quantize_e4m3_per_tensor(kc16)
    v8, vd = O.quantize_e4m3_per_tensor(vc16)
    out, lse = _run_decode(fa, q8, k8, v8, sl, bt, q_descale=qd.cuda(), k_descale=kd.cuda(), v_descale=vd.cuda())
    assert out.dtype == torch.bfloat16
    b = len(lens)
    ref32, ref_lse = O.paged_decode_ref(q8, k8, v8, sl, bt, q_descale=qd.expand(b, h_k), k_descale=kd.expand(b, h_k),
                                        v_descale=vd.expand(b, h_k), out_dtype=torch.float32)
    # stated FP8 tolerance: atol 7e-2 / rtol 1e-2 against the fp32 oracle on the same quantised inputs
    # (tests/test_pa.py:108-117); the kernel keeps P in f16, so it is in practice far tighter
    assert torch.allclose(out.float(), ref32.float(), atol=7e-2, rtol=1e-2)
    assert max_err(out, ref32) < 2e-2
    assert max_err(lse, ref_lse) < 1e-3
    # per-(batch, kv head) descale tensors give the same result as the one-element form
    out2, _ = _run_decode(fa, q8, k8, v8, sl, bt, q_descale=qd.expand(b, h_k).contiguous().cuda(),
                          k_descale=kd.expand(b, h_k).contiguous().cuda(), v_descale=vd.expand(b, h_k).contiguous().cuda())
    assert torch.equal(out, out2)


def test_decode_rejects_what_the_path_does_not_do(fa):
    flash_attn, cuda = fa
    g = gen(1)
    kc, vc, bt, sl = make_paged(g, [64], 1, 64, torch.bfloat16, poison=False)
    q = randn(g, 1, 1, 4, 128).cuda()
    with pytest.raises(ValueError):
        flash_attn.flash_attn_with_kvcache(q, kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(), softcap=1.0)
    with pytest.raises(NotImplementedError):   # contiguous-cache options have no paged meaning
        flash_attn.flash_attn_with_kvcache(q, kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                           cache_batch_idx=torch.zeros(1, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError):          # new keys with the wrong number of kv heads
        flash_attn.flash_attn_with_kvcache(q, kc.cuda(), vc.cuda(), k=q, v=q, cache_seqlens=sl.cuda(), block_table=bt.cuda())
    with pytest.raises(RuntimeError):
        flash_attn.flash_attn_with_kvcache(q, kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=None)
    with pytest.raises(RuntimeError):
        flash_attn.flash_attn_with_kvcache(q[..., :96].contiguous(), kc.cuda()[..., :96].contiguous(),
                                           vc.cuda()[..., :96].contiguous(), cache_seqlens=sl.cuda(), block_table=bt.cuda())


def test_paged_attention_binding_layouts(fa):
    """flash_attn_2_cuda.paged_attention (the reference's second decode binding, flash_api.cpp:2496-2515) writes into the
    caller's out for the three pool layouts, bit-identical to flash_attn_with_kvcache."""
    flash_attn, cuda = fa
    g = gen(99)
    lens, h, hk = [1, 200, 64, 513], 8, 2
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, torch.bfloat16, poison=False)
    q = randn(g, len(lens), 1, h, 128).cuda()
    kc_d, vc_d = kc.cuda(), vc.cuda()
    want = flash_attn.flash_attn_with_kvcache(q, kc_d, vc_d, cache_seqlens=sl.cuda(), block_table=bt.cuda(), causal=True)
    pools = {2: (kc_d, vc_d),
             1: (kc_d.permute(0, 2, 1, 3).contiguous(), vc_d.permute(0, 2, 1, 3).contiguous()),
             0: (kc_d.permute(0, 2, 1, 3).contiguous(), vc_d.permute(0, 2, 3, 1).contiguous())}
    for layout, (kp, vp) in pools.items():
        out = torch.full_like(want, float("nan"))
        cuda.paged_attention(out, q, kp, vp, 128 ** -0.5, bt.cuda(), sl.cuda(), None, "auto", None, None, None, max(lens),
                             None, layout, -1, -1, True)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert torch.equal(out, want), layout


def test_combine_takes_strided_partitions(fa):
    """Partials laid out as one [O | LSE] buffer per partition (what a single all-gather of decode_partial's output
    produces) are combined in place, bit-identical to the packed layout."""
    _, cuda = fa
    g = gen(17)
    parts, rows, d = 6, 32, 128
    o = torch.randn(parts, rows, d, generator=g)
    lse = torch.randn(parts, rows, generator=g) * 3
    packed = torch.cat([o.reshape(parts, rows * d), lse], dim=1).cuda()          # (parts, rows * (d + 1))
    o_v = packed[:, :rows * d].unflatten(1, (rows, d))
    l_v = packed[:, rows * d:]
    out1, l1 = cuda.combine(o_v, l_v, out_dtype=torch.float32, h=8)
    out2, l2 = cuda.combine(o.cuda(), lse.cuda(), out_dtype=torch.float32, h=8)
    assert torch.equal(out1, out2) and torch.equal(l1, l2)
    # decode_partial hands back exactly that layout
    kc, vc, bt, sl = make_paged(g, [300, 77], 2, 64, torch.bfloat16, poison=False)
    q = randn(g, 2, 1, 8, 128).cuda()
    op, lp = cuda.decode_partial(q, kc.cuda(), vc.cuda(), sl.cuda(), bt.cuda(), 128 ** -0.5)
    assert op.untyped_storage().data_ptr() == lp.untyped_storage().data_ptr()
    ref, ref_l = O.paged_decode_ref(q.cpu(), kc, vc, sl, bt, out_dtype=torch.float32)
    assert max_err(op.cpu(), ref[:, 0]) < 2e-2 and max_err(lp.cpu(), ref_l[:, :, 0]) < 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float8_e4m3fn])
@pytest.mark.parametrize("sq,h,hk", [(2, 8, 2), (4, 8, 2), (3, 4, 4), (8, 4, 2), (2, 8, 1), (16, 2, 2)])
@pytest.mark.parametrize("causal", [True, False])
def test_few_query_tokens_stay_on_the_decode_kernel(fa, dtype, sq, h, hk, causal):
    """Speculative decoding / multi-token prediction: seqlen_q * group <= 16 query rows are packed into the decode
    kernel's tile (one pass over the cache for all of them), with and without a KV split, against the oracle."""
    flash_attn, cuda = fa
    g = gen(700 + sq * 31 + h)
    lens = [sq, sq + 1, 64, 65, 300, 1031]
    fp8 = dtype == torch.float8_e4m3fn
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, torch.bfloat16, poison=not fp8)
    q = randn(g, len(lens), sq, h, 128)
    kw, okw = {}, {}
    if fp8:
        q8, qd = O.quantize_e4m3_per_tensor(q)
        k8, kd = O.quantize_e4m3_per_tensor(kc)
        v8, vd = O.quantize_e4m3_per_tensor(vc)
        q, kc, vc = q8, k8, v8
        kw = dict(q_descale=qd.cuda(), k_descale=kd.cuda(), v_descale=vd.cuda())
    else:
        q, kc, vc = q.to(dtype), kc.to(dtype), vc.to(dtype)
    launches = cuda.launch_count()
    outs = {}
    for part in (None, 128 if fp8 else 64):      # without and with a KV split (the e4m3 tile is 128 tokens)
        if part is not None:
            os.environ["FA_B200_DECODE_PARTITION"] = str(part)
        try:
            out, lse = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(),
                                                          block_table=bt.cuda(), causal=causal, return_softmax_lse=True, **kw)
            torch.cuda.synchronize()
        finally:
            os.environ.pop("FA_B200_DECODE_PARTITION", None)
        assert cuda.device_status() == 0
        outs[part] = (out.cpu(), lse.cpu())
    assert cuda.launch_count() - launches <= 4          # decode (+ combine) per call: not the prefill kernel's path
    for i, L in enumerate(lens):
        ki = O.gather_paged_kv(clean_nan(kc) if not fp8 else kc, bt[i], L)[None]
        vi = O.gather_paged_kv(clean_nan(vc) if not fp8 else vc, bt[i], L)[None]
        if fp8:
            okw = dict(q_descale=qd.view(1, 1).expand(1, hk), k_descale=kd.view(1, 1).expand(1, hk), v_descale=vd.view(1, 1).expand(1, hk))
        ref32, ref_lse = O.attention_ref(q[i:i + 1], ki, vi, causal=causal, out_dtype=torch.float32, **okw)
        for part, (out, lse) in outs.items():
            if fp8:
                assert max_err(out[i:i + 1], ref32) < 7e-2, (i, part)
            else:
                ref_pt, _ = O.attention_ref(q[i:i + 1], ki, vi, causal=causal, upcast=False, reorder_ops=True)
                assert_close_to_oracle(out[i:i + 1], ref32, ref_pt, mult=3.0, eps=2 ** -8, what=f"few tokens seq {i} part {part}")
            ok = torch.isfinite(ref_lse[0])
            assert max_err(lse[i][ok], ref_lse[0][ok]) < 2e-3


def test_varlen_entry_with_few_tokens_uses_the_decode_kernel(fa):
    """flash_attn_varlen_func(block_table=...) with the same small number of query tokens for every sequence (the form
    vLLM-style callers use for speculative decoding) gives the bits of flash_attn_with_kvcache on the same inputs."""
    flash_attn, cuda = fa
    g = gen(55)
    lens, h, hk, sq = [40, 300, 64, 1000], 8, 2, 4
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, torch.bfloat16, poison=False)
    q = randn(g, len(lens), sq, h, 128).cuda()
    want, want_lse = flash_attn.flash_attn_with_kvcache(q, kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                        causal=True, return_softmax_lse=True)
    cu = torch.arange(0, (len(lens) + 1) * sq, sq, dtype=torch.int32, device="cuda")
    n0 = cuda.launch_count()
    got, got_lse = flash_attn.flash_attn_varlen_func(q.view(-1, h, 128), kc.cuda(), vc.cuda(), cu, None, sq, max(lens),
                                                     seqused_k=sl.cuda(), causal=True, block_table=bt.cuda(),
                                                     return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.launch_count() - n0 <= 2
    assert torch.equal(got.view(len(lens), sq, h, 128), want)
    assert torch.equal(got_lse.view(h, len(lens), sq).permute(1, 0, 2), want_lse)


@pytest.mark.parametrize("f8", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("sq", [1, 3])
def test_fp8_kv_cache_under_16bit_queries(fa, qdtype, sq, f8):
    """The reference's kv_cache_dtype = "fp8" / "fp8_e5m2" modes (flash_api.cpp:2496-2515): e4m3 or e5m2 K/V pools with
    per-tensor scales, 16-bit queries and output.  Checked against the oracle on the dequantised cache, through flash_attn_with_kvcache and the
    vLLM-named entry (raw uint8 pools, layout 1)."""
    flash_attn, cuda = fa
    g = gen(808 + sq)
    lens, h, hk = [sq, 100, 128, 129, 1000, 2049], 8, 2
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, torch.bfloat16, poison=False)
    if f8 == torch.float8_e4m3fn:
        k8, kd = O.quantize_e4m3_per_tensor(kc)
        v8, vd = O.quantize_e4m3_per_tensor(vc)
    else:   # e5m2: same per-tensor scheme, scaled into a range well inside the format's
        kd, vd = kc.float().abs().max() / 448.0, vc.float().abs().max() / 448.0
        k8, v8 = (kc.float() / kd).to(f8), (vc.float() / vd).to(f8)
        kd, vd = kd.reshape(1), vd.reshape(1)
    q = randn(g, len(lens), sq, h, 128, dtype=qdtype)
    k_deq, v_deq = k8.float() * kd, v8.float() * vd
    ref32, ref_lse = O.paged_decode_ref(q, k_deq, v_deq, sl, bt, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q, k_deq.to(qdtype), v_deq.to(qdtype), sl, bt, upcast=False, reorder_ops=True)
    for part in (None, 128):
        if part is not None:
            os.environ["FA_B200_DECODE_PARTITION"] = str(part)
        try:
            out, lse = flash_attn.flash_attn_with_kvcache(q.cuda(), k8.cuda(), v8.cuda(), cache_seqlens=sl.cuda(),
                                                          block_table=bt.cuda(), causal=True, return_softmax_lse=True,
                                                          k_descale=kd.cuda(), v_descale=vd.cuda())
            torch.cuda.synchronize()
        finally:
            os.environ.pop("FA_B200_DECODE_PARTITION", None)
        assert cuda.device_status() == 0
        assert out.dtype == qdtype
        assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=3.0, eps=2 ** -8, what=f"fp8 kv cache part {part}")
        assert max_err(lse.cpu(), ref_lse) < 2e-3
    if sq == 1:
        k_raw = k8.cuda().permute(0, 2, 1, 3).contiguous().view(torch.uint8)       # (blocks, h_k, page, d) bytes
        v_raw = v8.cuda().permute(0, 2, 1, 3).contiguous().view(torch.uint8)
        o2 = flash_attn.vllm_flash_attn_with_kvcache(q.cuda(), k_raw, v_raw, cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                     causal=True, k_scale=kd.cuda(), v_scale=vd.cuda(),
                                                     kv_cache_dtype="fp8" if f8 == torch.float8_e4m3fn else "fp8_e5m2",
                                                     layout=1)
        torch.cuda.synchronize()
        assert_close_to_oracle(o2.cpu(), ref32, ref_pt, mult=3.0, eps=2 ** -8, what="fp8 kv cache, vllm entry")


@pytest.mark.gpu
def test_raw_pointer_entry_matches_the_tensor_entries(fa):
    """kv_cache_attention / cal_paged_attention (the reference's extern "C" raw-pointer entry, flash_api.cpp:2589-2631):
    one token per request gives the bits of flash_attn_with_kvcache for the three layouts; several tokens per request give
    the bits of the paged varlen entry (causal, bottom-right aligned; layout 0 the same values through another operand
    layout) and agree with the oracle."""
    flash_attn, cuda = fa
    g = gen(123)
    lens, h, hk, page = [1, 200, 64, 513, 300], 8, 2, 64
    kc, vc, bt, sl = make_paged(g, lens, hk, page, torch.bfloat16)
    n, pool = len(lens), kc.shape[0]
    kc_d, vc_d, bt_d, sl_d = kc.cuda(), vc.cuda(), bt.cuda().contiguous(), sl.cuda()
    assert bt.shape[1] == (max(lens) - 1) // page + 1
    pools = {2: (kc_d, vc_d),
             1: (kc_d.permute(0, 2, 1, 3).contiguous(), vc_d.permute(0, 2, 1, 3).contiguous()),
             0: (kc_d.permute(0, 2, 1, 3).contiguous(), vc_d.permute(0, 2, 3, 1).contiguous())}
    # one token per request
    q = randn(g, n, h, 128).cuda()
    want = flash_attn.flash_attn_with_kvcache(q.unsqueeze(1), kc_d, vc_d, cache_seqlens=sl_d, block_table=bt_d).squeeze(1)
    for layout, (kp, vp) in pools.items():
        out = torch.full_like(q, float("nan"))
        cuda.kv_cache_attention(q, None, 1, max(lens), kp, vp, bt_d, sl_d, out, n, n, h, hk, 128, pool, page, "bf16", layout)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert torch.equal(out, want), layout
    out = torch.full_like(q, float("nan"))
    cuda.cal_paged_attention(q, None, 1, max(lens), pools[1][0], pools[1][1], bt_d, sl_d, out, n, n, h, hk, 128, pool, page)
    assert torch.equal(out, want)
    # several tokens per request: the last q_lens[i] positions of each sequence
    q_lens = [1, 37, 64, 130, 300]
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    total = int(cu[-1])
    qv = randn(g, total, h, 128)
    qv_d, cu_d = qv.cuda(), cu.cuda()
    want = flash_attn.flash_attn_varlen_func(qv_d, kc_d, vc_d, cu_d, None, max(q_lens), max(lens), causal=True,
                                             block_table=bt_d, seqused_k=sl_d)
    for layout in (0, 1, 2):
        out = torch.full_like(qv_d, float("nan"))
        cuda.kv_cache_attention(qv_d, cu_d, max(q_lens), max(lens), pools[layout][0], pools[layout][1], bt_d, sl_d, out, n,
                                total, h, hk, 128, pool, page, "bf16", layout)
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        assert torch.equal(out, want) if layout else max_err(out, want) <= 2 ** -6, layout
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    for i, (lq, lk) in enumerate(zip(q_lens, lens)):
        q_i = qv[int(cu[i]):int(cu[i + 1])][None]
        k_i, v_i = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        ref32, _ = O.attention_ref(q_i, k_i, v_i, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(q_i, k_i, v_i, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out[int(cu[i]):int(cu[i + 1])].cpu()[None], ref32, ref_pt, mult=2.0, eps=2 ** -8,
                               what=f"request {i}")


@pytest.mark.parametrize("partition", [None, 256])
def test_lengths_beyond_the_block_table_are_clamped_and_reported(fa, partition):
    """A cache_seqlens entry larger than what the sequence's row of the block table covers must not send the kernel past
    the row: the length is clamped to the covered tokens (the result is attention over exactly those) and the launch
    reports FA_B200_ERR_DEVICE_RANGE through fa_b200_device_status()."""
    flash_attn, cuda = fa
    g = gen(911)
    lens, h, hk, page = [300, 1024, 77], 8, 2, 64
    kc, vc, bt, sl = make_paged(g, lens, hk, page, torch.bfloat16, poison=False)
    covered = bt.shape[1] * page                                  # 1024 tokens per row of the table
    assert covered == 1024
    bt = bt.clone()
    bt[0, :] = bt[1, :]                                           # sequence 0 may read all 16 pages once it is clamped
    bad = sl.clone()
    bad[0] = covered + 1000                                       # 2024 tokens claimed, 1024 covered
    q = randn(g, len(lens), 1, h, 128)
    if partition is not None:
        os.environ["FA_B200_DECODE_PARTITION"] = str(partition)
    try:
        out = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=bad.cuda(),
                                                 block_table=bt.cuda(), causal=True)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    RANGE = 14
    assert cuda.device_status() == RANGE
    assert cuda.device_status() == 0                              # cleared by the read
    clamped = bad.clone()
    clamped[0] = covered
    ref32, _ = O.paged_decode_ref(q, kc, vc, clamped, bt, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q, kc, vc, clamped, bt, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=3.0, eps=1e-5 + 2 ** -8, what="clamped lengths")
