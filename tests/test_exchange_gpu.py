"""GPU (one device): the two halves of fa_b200_exchange_combine, the kernel that moves the ranks' split-KV partials
over peer memory and combines them.  The ranks' kernels wait for one another, so ranks are never emulated by
concurrent launches on one GPU: here every "rank" pushes its partial into ONE buffer with launches that do not wait
(do_wait = 0), and a last launch that pushes nothing finds every flag already set and combines.  The result must equal
the LSE-combine kernel's and the oracle's merge, for both halves of the double buffer, with sinks, and with ranks that
hold no keys.  The multi-process path (CUDA IPC mappings, real waiting) runs in bench.py at two or more GPUs, where the
step's output is checked against the oracle."""
import pytest
import torch

from oracle import attention_oracle as O
from _util import gen

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    import flash_attn  # noqa: F401
    import flash_attn_2_cuda
    assert torch.cuda.is_available()
    return flash_attn_2_cuda


@pytest.mark.parametrize("world,b,h,d,out_dtype", [(4, 1, 32, 128, torch.bfloat16), (8, 2, 8, 128, torch.float16),
                                                   (2, 3, 4, 64, torch.float32), (16, 1, 16, 256, torch.bfloat16)])
def test_push_then_wait_matches_combine_and_oracle(cuda, world, b, h, d, out_dtype):
    g = gen(1000 + world)
    rows = b * h
    dev = torch.device("cuda")
    buf, handle, nbytes = cuda.exchange_alloc(world, rows, d, dev)
    assert len(handle) == cuda.IPC_HANDLE_BYTES and nbytes >= 2 * world * rows * (d + 2) * 4
    try:
        peers = [buf] * world
        for epoch in (1, 2, 3):   # both halves of the buffer, and the first one again
            o = torch.randn(world, rows, d, generator=g)
            l = torch.randn(world, rows, generator=g) * 3
            l[world - 1, ::2] = float("-inf")          # a rank without keys for some rows
            o[world - 1, ::2] = float("nan")           # whose partial must not be looked at
            if epoch == 3:
                l[:, 1] = float("-inf")                # a row nobody has keys for
            sink = torch.randn(h, generator=g) if epoch == 2 else None
            o_d, l_d = o.to(dev), l.to(dev)
            for r in range(world):
                cuda.exchange_combine(o_d[r].contiguous(), l_d[r].contiguous(), peers, r, epoch, h, out_dtype=out_dtype,
                                      push=True, wait=False)
            out, lse = cuda.exchange_combine(None, None, peers, 0, epoch, h, out_dtype=out_dtype, push=False, wait=True,
                                             s_aux=None if sink is None else sink.to(dev), rows=rows, d=d, device=dev)
            torch.cuda.synchronize()
            assert cuda.device_status() == 0
            ref_out, ref_lse = cuda.combine(o_d, l_d, out_dtype=out_dtype, h=h, s_aux=None if sink is None else sink.to(dev))
            # the same arithmetic as the combine kernel (other summation order: a few ulp)
            both_inf = torch.isinf(lse.cpu()) & torch.isinf(ref_lse.cpu())
            assert torch.equal(torch.isinf(lse.cpu()), torch.isinf(ref_lse.cpu()))
            assert (lse.cpu()[~both_inf] - ref_lse.cpu()[~both_inf]).abs().max().item() < 1e-5
            tol = 1e-5 if out_dtype == torch.float32 else 2 ** -7
            assert (out.float().cpu() - ref_out.float().cpu()).abs().max().item() <= tol * max(1.0, ref_out.float().abs().max().item())
            if sink is None:
                o_ref, l_ref = O.merge_partials_ref(torch.nan_to_num(o), l)
                fin = torch.isfinite(l_ref)
                got = out.float().cpu()
                assert (got[fin] - o_ref[fin]).abs().max().item() < (1e-5 if out_dtype == torch.float32 else 3e-2)
                assert (lse.cpu()[fin] - l_ref[fin]).abs().max().item() < 1e-4
                assert (got[~fin] == 0).all()           # rows without any key: zero output
    finally:
        torch.cuda.synchronize()
        cuda.exchange_free(buf)


def test_arguments_are_checked(cuda):
    dev = torch.device("cuda")
    buf, _, _ = cuda.exchange_alloc(2, 8, 128, dev)
    try:
        o, l = torch.zeros(8, 128, device=dev), torch.zeros(8, device=dev)
        with pytest.raises(RuntimeError):
            cuda.exchange_combine(o, l, [buf, buf], 0, 0, 8, push=True, wait=False)        # epoch 0
        with pytest.raises(RuntimeError):
            cuda.exchange_combine(o, l, [buf, 0], 0, 1, 8, push=True, wait=False)          # a missing peer
        with pytest.raises(RuntimeError):
            cuda.exchange_combine(o, l, [buf, buf], 2, 1, 8, push=True, wait=False)        # rank outside the world
    finally:
        cuda.exchange_free(buf)
