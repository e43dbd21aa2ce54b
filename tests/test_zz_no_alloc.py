"""GPU: fa_b200_decode_paged_static, the decode entry point for callers that cannot allocate or pass scratch
(a plugin inside a server that forbids allocation after start-up, or code that does not own a buffer to hand
over): its split-KV partials live in a fixed array inside the library.  Called straight through the C ABI, it
must give what fa_b200_decode_paged gives with a caller workspace (and what the oracle gives), on two calls in a row
(the array is shared and keeps the previous call's contents), and must refuse sizes beyond the array.

Collected last on purpose, so that a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from oracle import attention_oracle as O
from _util import clean_nan, gen, make_paged, max_err, randn

pytestmark = pytest.mark.gpu

STATIC_BYTES = 32 << 20


def _params(cuda, q, kc, vc, sl, bt, out, lse, partition):
    p = cuda._decode_params(q, kc, vc, sl, bt, 128 ** -0.5, out, lse, partition_tokens=partition)
    return p


def _call(cuda, fn, p, q):
    st = fn(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    torch.cuda.synchronize()
    return st


@pytest.mark.parametrize("lens,partition", [([3000, 130, 1, 2049], 512), ([700, 5000, 0], 1024), ([3000, 130, 1, 2049, 0], 0)])
def test_static_scratch_matches_workspace_entry_point_twice(lens, partition):
    import flash_attn_2_cuda as cuda
    lib = cuda.lib()
    h, h_k = 32, 8
    for round_ in range(2):                       # second round reuses the array left by the first
        g = gen(1234 + round_)
        kc, vc, bt, sl = make_paged(g, lens, h_k, 64, torch.bfloat16)
        q = randn(g, len(lens), 1, h, 128).cuda()
        ref32, ref_lse = O.paged_decode_ref(q.cpu(), clean_nan(kc), clean_nan(vc), sl, bt, out_dtype=torch.float32)
        kc, vc, bt, sl = kc.cuda(), vc.cuda(), bt.cuda(), sl.cuda()
        out_a = torch.empty(len(lens), 1, h, 128, dtype=torch.bfloat16, device="cuda")
        lse_a = torch.empty(len(lens), h, 1, dtype=torch.float32, device="cuda")
        out_b, lse_b = torch.full_like(out_a, 7.0), torch.full_like(lse_a, 7.0)
        pa = _params(cuda, q, kc, vc, sl, bt, out_a, lse_a, partition)
        need = lib.fa_b200_decode_workspace_bytes(ctypes.byref(pa))
        assert 0 < need <= STATIC_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        pa.workspace, pa.workspace_bytes = ws.data_ptr(), need
        assert _call(cuda, lib.fa_b200_decode_paged, pa, q) == 0
        pb = _params(cuda, q, kc, vc, sl, bt, out_b, lse_b, partition)   # no workspace given
        assert _call(cuda, lib.fa_b200_decode_paged_static, pb, q) == 0
        assert cuda.device_status() == 0
        # same kernels, same partition plan: the tests' tolerance (atol 1e-2) is met with room to spare
        assert torch.allclose(out_b.float(), out_a.float(), atol=1e-2, rtol=1e-2)
        assert torch.equal(out_b, out_a) and torch.equal(lse_b, lse_a)
        # and against the oracle itself, not only against its sibling (the reference's decode tolerance)
        assert torch.allclose(out_b.cpu().float(), ref32, atol=1e-2, rtol=1e-2)
        fin = torch.isfinite(ref_lse)
        assert max_err(lse_b.cpu()[fin], ref_lse[fin]) < 1e-3


def test_static_scratch_refuses_sizes_beyond_the_array():
    import flash_attn_2_cuda as cuda
    lib = cuda.lib()
    # batch 64 x 32 heads x 128 partitions of 512 tokens: 135 MB of partials, more than the array holds
    b, h, h_k, page, maxb = 64, 32, 8, 256, 256
    q = torch.zeros(b, 1, h, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(4, page, h_k, 128, dtype=torch.bfloat16, device="cuda")
    bt = torch.zeros(b, maxb, dtype=torch.int32, device="cuda")
    sl = torch.ones(b, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    p = cuda._decode_params(q, kc, kc, sl, bt, 1.0, out, None, partition_tokens=512)
    assert lib.fa_b200_decode_workspace_bytes(ctypes.byref(p)) > STATIC_BYTES
    assert lib.fa_b200_decode_paged_static(ctypes.byref(p), None) == 13     # FA_B200_ERR_TOO_LARGE
    assert b"scratch" in lib.fa_b200_last_cuda_error()
