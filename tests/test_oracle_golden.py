"""CPU: the oracle restatement replays the committed golden vectors (made from the reference's own
PyTorch oracles by tests/golden/make_golden.py) without the reference tree."""
import importlib.util
import os

import pytest
import torch

from oracle import attention_oracle as O
from oracle import padding_oracle as PO

_spec = importlib.util.spec_from_file_location(
    "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
_mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mg)
gen_inputs = _mg.gen_inputs


def _cases(golden, kind):
    return [c for c in golden["cases"] if c["kind"] == kind]


def test_golden_has_all_cases(golden):
    assert [c["name"] for c in golden["cases"]] == [c["name"] for c in _mg.CASES]


def test_fixed_bit_exact(golden):
    for c in _cases(golden, "fixed"):
        q, k, v = gen_inputs(c)
        out, lse = O.attention_ref(q, k, v, causal=c["causal"])
        assert torch.equal(out, c["out"]), c["name"]
        assert torch.equal(lse, c["lse"]), c["name"]
        out_pt, _ = O.attention_ref(q, k, v, causal=c["causal"], upcast=False, reorder_ops=True)
        assert (out_pt.float() - out.float()).abs().max().item() == pytest.approx(c["err_pt"], abs=0)


def test_varlen_bit_exact(golden):
    for c in _cases(golden, "varlen"):
        q, k, v, cq, ck = gen_inputs(c)
        out, lse = O.attention_varlen_ref(q, k, v, cq, ck, causal=c["causal"])
        assert torch.equal(out, c["out"]), c["name"]
        assert torch.equal(lse, c["lse"]), c["name"]
        assert lse.shape == (c["h"], sum(c["lens_q"]))


def test_paged_bit_exact(golden):
    for c in _cases(golden, "paged"):
        q, kc, vc, lens, bt = gen_inputs(c)
        out, _ = O.paged_decode_ref(q, kc, vc, lens, bt, causal=True)
        assert torch.equal(out, c["out"]), c["name"]


def test_fp8_bit_exact(golden):
    for c in _cases(golden, "fp8"):
        q8, k8, v8, qd, kd, vd = gen_inputs(c)
        out, _ = O.attention_ref(q8, k8, v8, causal=c["causal"], q_descale=qd, k_descale=kd, v_descale=vd,
                                 out_dtype=torch.float32)
        assert torch.equal(out, c["out"]), c["name"]
        assert torch.equal(out.to(torch.float8_e4m3fn).view(torch.uint8), c["out_e4m3"]), c["name"]
        out8, _ = O.attention_ref(q8, k8, v8, causal=c["causal"], q_descale=qd, k_descale=kd, v_descale=vd,
                                  intermediate_dtype=torch.float8_e4m3fn, out_dtype=torch.float32)
        assert torch.equal(out8, c["out_p8"]), c["name"]


def test_sink_and_window_bit_exact(golden):
    for c in _cases(golden, "sink"):
        q, k, v, s_aux = gen_inputs(c)
        out, lse = O.attention_ref(q, k, v, causal=c["causal"], s_aux=s_aux, window_size=tuple(c["window"]))
        assert torch.equal(out, c["out"]), c["name"]
        # the sink only changes the normalisation: out * exp(lse_with - lse_without) is the sink-free result
        if s_aux is not None:
            out0, lse0 = O.attention_ref(q, k, v, causal=c["causal"], window_size=tuple(c["window"]), out_dtype=torch.float32)
            out1, lse1 = O.attention_ref(q, k, v, causal=c["causal"], s_aux=s_aux, window_size=tuple(c["window"]),
                                         out_dtype=torch.float32)
            scale = torch.exp(lse1 - lse0).permute(0, 2, 1).unsqueeze(-1)
            keep = torch.isfinite(lse0).permute(0, 2, 1).unsqueeze(-1)
            assert torch.allclose(torch.where(keep, out1 * scale, out0), out0, atol=2e-6, rtol=1e-5), c["name"]


def test_unpad_bit_exact(golden):
    for c in _cases(golden, "unpad"):
        x, mask = gen_inputs(c)
        xs, idx, cu, mx = PO.unpad_input_ref(x, mask)
        assert torch.equal(idx, c["indices"]) and torch.equal(cu, c["cu_seqlens"]) and mx == c["max_seqlen"], c["name"]
        assert torch.equal(xs, c["unpadded"]), c["name"]
        assert torch.equal(PO.pad_input_ref(xs, idx, c["b"], c["s"]), c["repadded"]), c["name"]


def test_block_selection_matches_the_reference_chain(golden):
    """oracle.block_map_meansim_ref against maps made by the reference's own get_block_map_meansim (its torch chain run
    on the CPU in fp32, its three Triton launches replaced by torch statements; tests/golden/make_golden.py)."""
    from oracle import block_select_oracle as BS
    cases = _cases(golden, "block_select")
    assert len(cases) >= 4
    for c in cases:
        q, k = gen_inputs(c)
        mine, margin = BS.block_map_meansim_ref(q, k, is_causal=c["causal"], **c["args"])
        assert torch.equal(mine, c["block_map"]), c["name"]
        assert 0.05 < mine.float().mean() < 0.98, c["name"]     # neither empty nor dense: the choice is exercised


def test_block_map_known_answer():
    """The worked example of the reference's docstring (flash_attn/utils/sparse_utils.py:537-541)."""
    bm = torch.tensor([[[[0, 0, 1, 0, 0, 1, 0, 1, 0, 1]]]], dtype=torch.bool)
    off, cnt = PO.block_map_to_block_offset_ref(bm)
    assert off[0, 0, 0, :4].tolist() == [2, 5, 7, 9] and torch.all(off[0, 0, 0, 4:] == 10000000)
    assert cnt.tolist() == [[[4]]]


def test_rotary_bit_exact(golden):
    for c in _cases(golden, "rotary"):
        x, cos, sin, off = gen_inputs(c)
        out = O.rotary_ref(x, cos, sin, off, c["interleaved"], out_dtype=torch.float32)
        assert torch.equal(out, c["out"]), c["name"]


def test_kv_append_ref_addresses_pages():
    """The append writes exactly the rows paged_element_offset() names and nothing else."""
    g = torch.Generator().manual_seed(5)
    page, hk, d = 16, 2, 128
    kc = torch.zeros(6, page, hk, d)
    vc = torch.zeros(6, page, hk, d)
    bt = torch.tensor([[4, 1, 0], [2, 5, 3]], dtype=torch.int32)
    lens = torch.tensor([15, 30], dtype=torch.int32)
    kn = torch.randn(2, 3, hk, d, generator=g)
    vn = torch.randn(2, 3, hk, d, generator=g)
    new_lens = O.kv_append_ref(kc, vc, bt, lens, kn, vn)
    assert new_lens.tolist() == [18, 33]
    flat_k, flat_v = kc.flatten(), vc.flatten()
    touched = torch.zeros_like(flat_k, dtype=torch.bool)
    for b in range(2):
        for s in range(3):
            for h in range(hk):
                off = O.paged_element_offset(bt[b].tolist(), int(lens[b]) + s, h, 0, page, page * hk * d, hk * d, d)
                assert torch.equal(flat_k[off:off + d], kn[b, s, h])
                assert torch.equal(flat_v[off:off + d], vn[b, s, h])
                touched[off:off + d] = True
    assert flat_k[~touched].abs().sum() == 0 and flat_v[~touched].abs().sum() == 0


def test_merge(golden):
    for c in _cases(golden, "merge"):
        es, mx, o = gen_inputs(c)
        lse_part = (torch.log(es) + mx * 0.6931471805599453).permute(2, 0, 1)
        out, lse = O.merge_partials_ref(o.permute(2, 0, 1, 3), lse_part)
        assert (out - c["out"]).abs().max().item() < 2e-6
        # merged LSE equals LSE over the union
        assert torch.allclose(lse, torch.logsumexp(lse_part, dim=0), atol=1e-5)


def test_merge_equals_unsplit_attention():
    g = torch.Generator().manual_seed(123)
    q = torch.randn(1, 1, 4, 128, generator=g)
    k = torch.randn(1, 300, 2, 128, generator=g)
    v = torch.randn(1, 300, 2, 128, generator=g)
    full, lse_full = O.attention_ref(q, k, v)
    parts_o, parts_l = [], []
    for a, b in [(0, 128), (128, 256), (256, 300)]:
        o, l = O.attention_ref(q, k[:, a:b], v[:, a:b])
        parts_o.append(o[0, 0])
        parts_l.append(l[0, :, 0])
    # an empty partition must not disturb the result
    parts_o.append(torch.zeros(4, 128))
    parts_l.append(torch.full((4,), float("inf")))
    out, lse = O.merge_partials_ref(torch.stack(parts_o), torch.stack(parts_l))
    assert torch.allclose(out, full[0, 0], atol=1e-5)
    assert torch.allclose(lse, lse_full[0, :, 0], atol=1e-5)


def test_empty_rows_and_empty_keys():
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 5, 2, 128, generator=g)
    k = torch.randn(1, 2, 2, 128, generator=g)
    out, lse = O.attention_ref(q, k, k, causal=True)
    assert torch.all(out[0, :3] == 0) and torch.all(torch.isinf(lse[0, :, :3]) & (lse[0, :, :3] > 0))
    assert torch.isfinite(lse[0, :, 3:]).all()


def test_paged_addressing_integer_model():
    page, hk, d = 64, 2, 128
    bt = [7, 2, 9]
    s0, s1, s2 = page * hk * d, hk * d, d
    assert O.paged_element_offset(bt, 0, 0, 0, page, s0, s1, s2) == 7 * s0
    assert O.paged_element_offset(bt, 64, 1, 5, page, s0, s1, s2) == 2 * s0 + d + 5
    assert O.paged_element_offset(bt, 191, 1, 127, page, s0, s1, s2) == 9 * s0 + 63 * s1 + s2 + 127
    assert O.partial_slot_index(2, 3, 5, batch=4, heads=8) == (2 * 4 + 3) * 8 + 5


def test_block_list_roundtrip():
    g = torch.Generator().manual_seed(11)
    nq = 4
    tm = torch.rand(1, 2, nq, nq, generator=g) < 0.4
    tm = (tm & torch.tril(torch.ones(nq, nq, dtype=torch.bool))) | torch.eye(nq, dtype=torch.bool)
    cnt, offs = O.tile_mask_to_block_lists(tm, block_m=128)
    assert cnt.dtype == torch.int32 and offs.dtype == torch.int32
    assert torch.equal(cnt, tm.sum(-1).to(torch.int32) * 2)
    dense = O.block_lists_to_dense_mask(cnt, offs, nq * 128, nq * 128, 128)
    expect = ~tm.repeat_interleave(128, 2).repeat_interleave(128, 3)
    assert torch.equal(dense, expect)
    assert O.sparse_block_m(2048) == 64 and O.sparse_block_m(2049) == 128


def test_quantize_e4m3():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 128, generator=g).to(torch.bfloat16)
    xq, ds = O.quantize_e4m3_per_tensor(x)
    assert xq.dtype == torch.float8_e4m3fn and ds.dtype == torch.float32 and ds.numel() == 1
    assert ds.item() == pytest.approx(x.float().abs().max().item() / 448.0)
    assert (xq.float() * ds - x.float()).abs().max().item() <= x.float().abs().max().item() / 16
