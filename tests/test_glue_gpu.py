"""GPU parity (bit-exact: integer and byte work): padding removal and block-map conversion against the CPU oracle and
the golden vectors made from the reference's own flash_attn/bert_padding.py."""
import importlib.util
import os

import pytest
import torch

from oracle import padding_oracle as PO
from _util import gen

pytestmark = pytest.mark.gpu

_spec = importlib.util.spec_from_file_location(
    "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
_mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mg)


@pytest.fixture(scope="module")
def mods():
    import flash_attn  # noqa: F401
    import flash_attn.bert_padding as bp
    import flash_attn.utils.sparse_utils as su
    return bp, su


def test_unpad_golden_cases(mods, golden):
    bp, _ = mods
    for c in [c for c in golden["cases"] if c["kind"] == "unpad"]:
        x, mask = _mg.gen_inputs(c)
        xs, idx, cu, mx = bp.unpad_input(x.cuda(), mask.cuda())
        assert torch.equal(idx.cpu(), c["indices"]) and torch.equal(cu.cpu(), c["cu_seqlens"]) and mx == c["max_seqlen"]
        assert torch.equal(xs.cpu(), c["unpadded"]), c["name"]
        back = bp.pad_input(xs, idx, c["b"], c["s"])
        assert torch.equal(back.cpu(), c["repadded"]), c["name"]


@pytest.mark.parametrize("mask_dtype", [torch.bool, torch.int32, torch.int64])
@pytest.mark.parametrize("feat,dtype", [((32, 128), torch.bfloat16), ((7,), torch.float32), ((3,), torch.uint8), ((5,), torch.float16)])
def test_unpad_pad_round_trip(mods, mask_dtype, feat, dtype):
    """Ragged, empty and full rows; row sizes that allow 16-, 4-, 2- and 1-byte moves; the round trip restores every
    kept token and zeroes the rest."""
    bp, _ = mods
    g = gen(11)
    b, s = 9, 1000
    mask = torch.rand(b, s, generator=g) < 0.5
    mask[2] = False
    mask[3] = True
    mask[4, :] = False
    mask[4, -1] = True
    x = (torch.randn(b, s, *feat, generator=g) * 20).to(dtype)
    xs, idx, cu, mx = bp.unpad_input(x.cuda(), mask.to(mask_dtype).cuda())
    r_xs, r_idx, r_cu, r_mx = PO.unpad_input_ref(x, mask)
    assert torch.equal(idx.cpu(), r_idx) and torch.equal(cu.cpu(), r_cu) and mx == r_mx
    assert torch.equal(xs.cpu(), r_xs)
    back = bp.pad_input(xs, idx, b, s)
    assert torch.equal(back.cpu(), PO.pad_input_ref(r_xs, r_idx, b, s))
    assert torch.equal(back.cpu()[mask], x[mask]) and torch.all(back.cpu()[~mask] == 0)


def test_unpad_feeds_varlen_attention(mods):
    """The helpers in their place: padded batch -> unpad -> flash_attn_varlen_func -> pad, against the oracle per
    sequence (the use the reference's models make of them, flash_attn/modules/mha.py)."""
    import flash_attn
    from oracle import attention_oracle as O
    from _util import assert_close_to_oracle, randn
    bp, _ = mods
    g = gen(12)
    b, s, h, hk = 3, 200, 4, 2
    lens = [200, 57, 130]
    mask = torch.zeros(b, s, dtype=torch.bool)
    for i, L in enumerate(lens):
        mask[i, :L] = True
    q, k, v = randn(g, b, s, h, 128), randn(g, b, s, hk, 128), randn(g, b, s, hk, 128)
    qs, idx, cu, mx = bp.unpad_input(q.cuda(), mask.cuda())
    ks, _, _, _ = bp.unpad_input(k.cuda(), mask.cuda())
    vs, _, _, _ = bp.unpad_input(v.cuda(), mask.cuda())
    out = bp.pad_input(flash_attn.flash_attn_varlen_func(qs, ks, vs, cu, cu, mx, mx, causal=True), idx, b, s).cpu()
    for i, L in enumerate(lens):
        ref32, _ = O.attention_ref(q[i:i + 1, :L], k[i:i + 1, :L], v[i:i + 1, :L], causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(q[i:i + 1, :L], k[i:i + 1, :L], v[i:i + 1, :L], causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out[i:i + 1, :L], ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"seq {i}")
        assert torch.all(out[i, L:] == 0)


def test_block_map_to_block_offset(mods):
    _, su = mods
    import flash_attn_2_cuda as cuda
    bm = torch.tensor([[[[0, 0, 1, 0, 0, 1, 0, 1, 0, 1]]]], dtype=torch.bool)
    off, cnt = su.block_map_to_block_offset(bm.cuda())
    assert off[0, 0, 0, :4].tolist() == [2, 5, 7, 9] and cnt.item() == 4     # the reference's worked example
    g = gen(13)
    for shape in [(2, 3, 17, 33), (1, 2, 256, 512), (1, 1, 5, 1)]:
        bm = torch.rand(*shape, generator=g) < 0.3
        bm[..., 0, :] = False
        bm[..., -1, :] = True
        off, cnt = su.block_map_to_block_offset(bm.cuda())
        r_off, r_cnt = PO.block_map_to_block_offset_ref(bm)
        assert torch.equal(off.cpu(), r_off) and torch.equal(cnt.cpu(), r_cnt)
        off64, _ = cuda.block_map_to_offset(bm.cuda(), 64, -1)                  # key-row offsets of 64-row tiles
        r64, _ = PO.block_map_to_block_offset_ref(bm, 64, -1)
        assert torch.equal(off64.cpu(), r64)
