"""GPU parity: attention sinks (s_aux) and sliding windows on the prefill, paged-prefill and decode paths, against the
CPU oracle (pinned to the reference's sink oracle, tests/test_flash_attn_saux.py:107-232) with the reference's error
rule (tests/test_flash_attn_saux.py:312-316: err <= 2 * err of the same math in the input dtype + 1e-5)."""
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
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def test_sink_golden_cases(fa, golden):
    flash_attn, cuda = fa
    for c in [c for c in golden["cases"] if c["kind"] == "sink" and tuple(c["window"]) == (-1, -1)]:
        q, k, v, s_aux = _mg.gen_inputs(c)
        out = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=c["causal"], s_aux=s_aux.cuda())
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        e = max_err(out.cpu(), c["out"])
        assert e <= 2 * c["err_pt"] + 1e-5, (c["name"], e, c["err_pt"])


@pytest.mark.parametrize("kernel", ["pair", "dense", "single"])
@pytest.mark.parametrize("dtype,sink_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                              (torch.bfloat16, torch.float32)])
def test_prefill_sinks_all_kernels(fa, kernel, dtype, sink_dtype, monkeypatch):
    flash_attn, cuda = fa
    monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kernel)
    g = gen(31)
    lens_q, lens_k, h, hk = [200, 1, 77, 256], [200, 300, 77, 40], 8, 2     # last: more queries than keys (empty rows)
    q = randn(g, sum(lens_q), h, 128, dtype=dtype)
    k = randn(g, sum(lens_k), hk, 128, dtype=dtype)
    v = randn(g, sum(lens_k), hk, 128, dtype=dtype)
    s_aux = (torch.randn(h, generator=g) * 2.0).to(dtype)        # values representable in the input dtype
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    ck = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cq.cuda(), ck.cuda(), max(lens_q), max(lens_k),
                                                 causal=True, s_aux=s_aux.to(sink_dtype).cuda(), return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    ref32, ref_lse = O.attention_varlen_ref(q, k, v, cq, ck, causal=True, s_aux=s_aux, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q, k, v, cq, ck, causal=True, s_aux=s_aux, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"sinks {kernel}")
    assert max_err(lse.cpu(), ref_lse) < 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("partition", [None, 64, 256])
def test_decode_sinks(fa, dtype, partition):
    """One query token over a paged cache with sinks: without a split the kernel adds the sink itself, with a split the
    combine does; both must agree with the oracle and (to rounding) with each other."""
    flash_attn, cuda = fa
    g = gen(5 + (partition or 0))
    lens, h, hk = [1, 63, 64, 700, 0], 16, 4
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, dtype)
    q = randn(g, len(lens), 1, h, 128, dtype=dtype)
    s_aux = (torch.randn(h, generator=g) * 1.5).to(dtype)
    if partition is not None:
        os.environ["FA_B200_DECODE_PARTITION"] = str(partition)
    try:
        out, lse = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(),
                                                      block_table=bt.cuda(), causal=True, s_aux=s_aux.cuda(),
                                                      return_softmax_lse=True)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    ref32, ref_lse = O.paged_decode_ref(q, kcc, vcc, sl, bt, s_aux=s_aux, out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q, kcc, vcc, sl, bt, s_aux=s_aux, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=3.0, eps=2 ** -8, what="decode sinks")
    # the sequence without keys attends to the sink alone: out = 0, lse = the sink
    assert torch.all(out[-1] == 0)
    assert max_err(lse[-1, :, 0].cpu(), s_aux.float()) < 1e-3
    ok = torch.isfinite(ref_lse)
    assert max_err(lse.cpu()[ok], ref_lse[ok]) < 2e-3


def test_combine_with_sinks(fa):
    _, cuda = fa
    g = gen(3)
    parts, b, h, d = 5, 2, 4, 128
    o = torch.randn(parts, b * h, d, generator=g)
    lse = torch.randn(parts, b * h, generator=g) * 3
    s_aux = torch.randn(h, generator=g)
    ref_o, ref_l = O.merge_partials_ref(o, lse)
    sink = s_aux.repeat(b)
    tot = torch.logaddexp(ref_l, sink)
    want = ref_o * torch.exp(ref_l - tot).unsqueeze(-1)
    out, l = cuda.combine(o.cuda(), lse.cuda(), out_dtype=torch.float32, h=h, s_aux=s_aux.cuda())
    assert max_err(out.cpu(), want) < 3e-6 * max(1.0, want.abs().max().item())
    assert max_err(l.cpu(), tot) < 1e-5


def test_window_golden_cases(fa, golden):
    flash_attn, cuda = fa
    for c in [c for c in golden["cases"] if c["kind"] == "sink" and tuple(c["window"]) != (-1, -1)]:
        q, k, v, s_aux = _mg.gen_inputs(c)
        out = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=c["causal"], window_size=tuple(c["window"]),
                                         s_aux=None if s_aux is None else s_aux.cuda())
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        e = max_err(out.cpu(), c["out"])
        assert e <= 2 * c["err_pt"] + 1e-5, (c["name"], e, c["err_pt"])


@pytest.mark.parametrize("kernel", ["pair", "dense", "single"])
@pytest.mark.parametrize("causal,window", [(True, (0, -1)), (True, (100, -1)), (True, (127, 0)), (True, (300, 0)),
                                           (False, (64, 64)), (False, (5, 200)), (False, (-1, 17)), (False, (1000, 1000))])
def test_prefill_windows_all_kernels(fa, kernel, causal, window, monkeypatch):
    """Sliding windows on the three prefill kernels: windows smaller and larger than a tile, one-sided, wider than the
    sequences, sequences with more keys than queries and the other way round."""
    flash_attn, cuda = fa
    monkeypatch.setenv("FA_B200_PREFILL_KERNEL", kernel)
    g = gen(100 + window[0] * 7 + window[1])
    lens_q, lens_k, h, hk = [300, 64, 130, 257], [300, 500, 40, 257], 4, 2
    dtype = torch.bfloat16
    q = randn(g, sum(lens_q), h, 128, dtype=dtype)
    k = randn(g, sum(lens_k), hk, 128, dtype=dtype)
    v = randn(g, sum(lens_k), hk, 128, dtype=dtype)
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    ck = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cq.cuda(), ck.cuda(), max(lens_q), max(lens_k),
                                                 causal=causal, window_size=window, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    win = (window[0], 0) if causal else window
    ref32, ref_lse = O.attention_varlen_ref(q, k, v, cq, ck, causal=causal, window_size=win, out_dtype=torch.float32)
    ref_pt, _ = O.attention_varlen_ref(q, k, v, cq, ck, causal=causal, window_size=win, upcast=False, reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"window {window} {kernel}")
    ok = torch.isfinite(ref_lse)
    assert max_err(lse.cpu()[ok], ref_lse[ok]) < 1e-3
    assert torch.all(torch.isinf(lse.cpu()[~ok]))


@pytest.mark.parametrize("window_left", [0, 5, 63, 64, 200, 100000])
@pytest.mark.parametrize("partition", [None, 64, 256])
def test_decode_window(fa, window_left, partition):
    flash_attn, cuda = fa
    g = gen(900 + window_left % 977)
    dtype, lens, h, hk = torch.bfloat16, [1, 64, 65, 700, 1031], 8, 2
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, dtype)
    q = randn(g, len(lens), 1, h, 128, dtype=dtype)
    s_aux = (torch.randn(h, generator=g)).to(dtype)
    if partition is not None:
        os.environ["FA_B200_DECODE_PARTITION"] = str(partition)
    try:
        out = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                 causal=True, window_size=(window_left, 0), s_aux=s_aux.cuda())
        torch.cuda.synchronize()
    finally:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    assert cuda.device_status() == 0
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    ref32, _ = O.paged_decode_ref(q, kcc, vcc, sl, bt, s_aux=s_aux, window_size=(window_left, 0), out_dtype=torch.float32)
    ref_pt, _ = O.paged_decode_ref(q, kcc, vcc, sl, bt, s_aux=s_aux, window_size=(window_left, 0), upcast=False,
                                   reorder_ops=True)
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=3.0, eps=2 ** -8, what=f"decode window {window_left}")


@pytest.mark.parametrize("sq", [3, 7])
def test_paged_chunk_with_window_and_sinks(fa, sq):
    """Several query tokens over a paged cache with a window and sinks: 7 tokens x 4 heads per kv head go through the
    prefill kernel and the block table, 3 x 4 = 12 rows stay on the decode kernel."""
    flash_attn, cuda = fa
    g = gen(4242)
    dtype, lens, h, hk = torch.float16, [9, 500, 128, 1031], 8, 2
    kc, vc, bt, sl = make_paged(g, lens, hk, 64, dtype)
    q = randn(g, len(lens), sq, h, 128, dtype=dtype)
    s_aux = (torch.randn(h, generator=g)).to(dtype)
    out = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                             causal=True, window_size=(150, 0), s_aux=s_aux.cuda())
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    for i, L in enumerate(lens):
        ki, vi = O.gather_paged_kv(clean_nan(kc), bt[i], L)[None], O.gather_paged_kv(clean_nan(vc), bt[i], L)[None]
        ref32, _ = O.attention_ref(q[i:i + 1], ki, vi, causal=True, window_size=(150, 0), s_aux=s_aux, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(q[i:i + 1], ki, vi, causal=True, window_size=(150, 0), s_aux=s_aux, upcast=False,
                                    reorder_ops=True)
        assert_close_to_oracle(out[i:i + 1].cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"paged chunk window seq {i}")
