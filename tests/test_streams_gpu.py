"""GPU: eager calls from two streams at once.  The persistent prefill kernels claim their work from a counter and the
split decode counts its partitions on tickets; both live in the library, one block per (device, stream), so launches
that overlap on the GPU never share them.  Many launches are queued on two streams without any synchronisation in
between (far more than the library has counter blocks) and every result must be bit-identical to the same call made
alone."""
import os

import pytest
import torch

from _util import gen, make_paged, randn

pytestmark = pytest.mark.gpu

ROUNDS = 48


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def test_prefill_launches_from_two_streams_do_not_share_work_counters(fa):
    flash_attn, cuda = fa
    g = gen(31337)
    h, hk = 8, 2
    cases = []
    for lens in ([700, 130, 1024, 3], [512, 512, 900]):
        total = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
        q, k, v = randn(g, total, h, 128).cuda(), randn(g, total, hk, 128).cuda(), randn(g, total, hk, 128).cuda()
        cases.append((q, k, v, cu, max(lens)))
    call = lambda c: flash_attn.flash_attn_varlen_func(c[0], c[1], c[2], c[3], c[3], c[4], c[4], causal=True)
    alone = [call(c) for c in cases]
    torch.cuda.synchronize()
    assert "prefill_pair" in cuda.last_launch_info()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[], []]
    for _ in range(ROUNDS):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                outs[i].append(call(cases[i]))
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    for i in range(2):
        for o in outs[i]:
            assert torch.equal(o, alone[i])


def test_split_decode_from_two_streams_does_not_share_tickets(fa):
    flash_attn, cuda = fa
    g = gen(4711)
    h, hk, page = 8, 2, 64
    cases = []
    for lens in ([1500, 64, 2047, 700], [1024, 1024, 33]):
        kc, vc, bt, sl = make_paged(g, lens, hk, page, torch.bfloat16, poison=False)
        q = randn(g, len(lens), 1, h, 128)
        cases.append((q.cuda(), kc.cuda(), vc.cuda(), sl.cuda(), bt.cuda()))
    os.environ["FA_B200_DECODE_PARTITION"] = "256"        # several partitions per sequence, merged in the kernel
    try:
        call = lambda c: flash_attn.flash_attn_with_kvcache(c[0], c[1], c[2], cache_seqlens=c[3], block_table=c[4], causal=True)
        alone = [call(c) for c in cases]
        torch.cuda.synchronize()
        assert "in-kernel" in cuda.last_launch_info()
        streams = [torch.cuda.Stream(), torch.cuda.Stream()]
        outs = [[], []]
        for _ in range(ROUNDS):
            for i, st in enumerate(streams):
                with torch.cuda.stream(st):
                    outs[i].append(call(cases[i]))
        torch.cuda.synchronize()
    finally:
        os.environ.pop("FA_B200_DECODE_PARTITION", None)
    assert cuda.device_status() == 0
    for i in range(2):
        for o in outs[i]:
            assert torch.equal(o, alone[i])
