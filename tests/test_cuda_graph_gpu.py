"""The calls are stream-capturable (no allocation or synchronisation inside the C layer; lengths, page tables and
cu_seqlens are read on the device): decode steps with KV append and a varlen prefill are captured into CUDA graphs and
replayed on changed inputs, each replay checked against the eager call and the CPU oracle.  The reference asks the same
of its paged attention (workspace taken fresh under capture, src/paged_attention.cu:712-745)."""
import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, gen, make_paged, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def test_decode_steps_with_append_replayed_from_a_graph(fa):
    flash_attn, cuda = fa
    g = gen(4242)
    lens0, h, hk, page, steps = [5, 700, 64, 2047], 8, 2, 64, 4
    kc, vc, bt, sl = make_paged(g, [L + steps for L in lens0], hk, page, torch.bfloat16, poison=False)
    sl = torch.tensor(lens0, dtype=torch.int32)
    b = len(lens0)
    kc_d, vc_d, bt_d, sl_d = kc.cuda(), vc.cuda(), bt.cuda(), sl.cuda()
    q_s = torch.zeros(b, 1, h, 128, dtype=torch.bfloat16, device="cuda")
    k_s = torch.zeros(b, 1, hk, 128, dtype=torch.bfloat16, device="cuda")
    v_s = torch.zeros_like(k_s)
    out_s = torch.zeros_like(q_s)

    def step():
        flash_attn.flash_attn_with_kvcache(q_s, kc_d, vc_d, k=k_s, v=v_s, cache_seqlens=sl_d, block_table=bt_d, causal=True,
                                           out=out_s)
        sl_d.add_(1)

    # warm-up outside capture on a side stream (first-call set-up: attributes, status word), then restore the state
    kc0, vc0 = kc_d.clone(), vc_d.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    kc_d.copy_(kc0); vc_d.copy_(vc0); sl_d.copy_(sl.cuda())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    kc_d.copy_(kc0); vc_d.copy_(vc0); sl_d.copy_(sl.cuda())     # capture does not run anything, but keep the state explicit
    kc_ref, vc_ref, lens = kc.clone(), vc.clone(), list(lens0)
    for t in range(steps):
        qn, kn, vn = randn(g, b, 1, h, 128), randn(g, b, 1, hk, 128), randn(g, b, 1, hk, 128)
        q_s.copy_(qn.cuda()); k_s.copy_(kn.cuda()); v_s.copy_(vn.cuda())
        graph.replay()
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        for i in range(b):                                      # the oracle's cache after the append
            pos = lens[i]
            pg, row = int(bt[i, pos // page]), pos % page
            kc_ref[pg, row], vc_ref[pg, row] = kn[i, 0], vn[i, 0]
            lens[i] += 1
        sl_now = torch.tensor(lens, dtype=torch.int32)
        assert torch.equal(sl_d.cpu(), sl_now)
        ref32, _ = O.paged_decode_ref(qn, kc_ref, vc_ref, sl_now, bt, out_dtype=torch.float32)
        ref_pt, _ = O.paged_decode_ref(qn, kc_ref, vc_ref, sl_now, bt, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out_s.cpu(), ref32, ref_pt, mult=3.0, eps=1e-5 + 2 ** -8, what=f"graph replay {t}")
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)


def test_varlen_prefill_replayed_with_other_lengths(fa):
    """One captured launch of the persistent prefill kernel serves other cu_seqlens of the same bounds: the work list is
    derived on the device, the work counter is the captured call's own."""
    flash_attn, cuda = fa
    g = gen(77)
    h, hk, total, max_len, b = 8, 2, 1500, 1024, 4
    q_s = torch.zeros(total, h, 128, dtype=torch.bfloat16, device="cuda")
    k_s = torch.zeros(total, hk, 128, dtype=torch.bfloat16, device="cuda")
    v_s = torch.zeros_like(k_s)
    cu_s = torch.zeros(b + 1, dtype=torch.int32, device="cuda")
    out_s = torch.zeros_like(q_s)

    def call():
        flash_attn.flash_attn_varlen_func(q_s, k_s, v_s, cu_s, cu_s, max_len, max_len, causal=True, out=out_s)

    cu_s.copy_(torch.tensor([0, 100, 200, 300, 400], dtype=torch.int32))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    for lens in ([1000, 1, 129, 370], [300, 300, 300, 300], [1024, 0, 0, 476]):
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
        q, k, v = randn(g, total, h, 128), randn(g, total, hk, 128), randn(g, total, hk, 128)
        q_s.copy_(q.cuda()); k_s.copy_(k.cuda()); v_s.copy_(v.cuda()); cu_s.copy_(cu.cuda())
        out_s.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        n = int(cu[-1])
        ref32, _ = O.attention_varlen_ref(q[:n], k[:n], v[:n], cu, cu, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_varlen_ref(q[:n], k[:n], v[:n], cu, cu, causal=True, upcast=False, reorder_ops=True)
        assert_close_to_oracle(out_s[:n].cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=f"graph prefill {lens}")


def test_chunks_of_new_tokens_over_the_paged_cache_replayed_concurrently(fa):
    """flash_attn_with_kvcache with a chunk of query tokens per sequence (more than the decode tile holds) runs the
    persistent paged prefill kernel.  Two such calls captured into two graphs get a work counter each, so their replays
    may overlap on two streams; each replay reads the lengths of the moment and is checked against the oracle."""
    from _util import make_paged
    flash_attn, cuda = fa
    g = gen(4343)
    h, hk, page, sq = 8, 2, 64, 48
    cap = [1500, 700, 2048]
    pools = [make_paged(g, cap, hk, page, torch.bfloat16, poison=False) for _ in range(2)]
    q_s = [torch.zeros(len(cap), sq, h, 128, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    out_s = [torch.zeros_like(x) for x in q_s]
    dev = [(kc.cuda(), vc.cuda(), bt.cuda(), sl.cuda()) for kc, vc, bt, sl in pools]

    def call(i):
        kc_d, vc_d, bt_d, sl_d = dev[i]
        flash_attn.flash_attn_with_kvcache(q_s[i], kc_d, vc_d, cache_seqlens=sl_d, block_table=bt_d, causal=True, out=out_s[i])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call(0)
        assert "prefill" in cuda.last_launch_info()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graphs = []
    for i in range(2):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            call(i)
        graphs.append(gr)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for lens in ([1500, 700, 2048], [48, 64, 1000], [777, 49, 130]):
        qs = [randn(g, len(cap), sq, h, 128) for _ in range(2)]
        for i in range(2):
            q_s[i].copy_(qs[i].cuda())
            dev[i][3].copy_(torch.tensor(lens, dtype=torch.int32).cuda())
            out_s[i].fill_(float("nan"))
        torch.cuda.synchronize()
        for rep in range(3):                                    # overlapping replays of the two graphs
            for i in range(2):
                with torch.cuda.stream(streams[i]):
                    graphs[i].replay()
        torch.cuda.synchronize()
        assert cuda.device_status() == 0
        for i in range(2):
            kc, vc, bt, _ = pools[i]
            for s, L in enumerate(lens):
                ki, vi = O.gather_paged_kv(kc, bt[s], L)[None], O.gather_paged_kv(vc, bt[s], L)[None]
                ref32, _ = O.attention_ref(qs[i][s:s + 1], ki, vi, causal=True, out_dtype=torch.float32)
                ref_pt, _ = O.attention_ref(qs[i][s:s + 1], ki, vi, causal=True, upcast=False, reorder_ops=True)
                assert_close_to_oracle(out_s[i][s:s + 1].cpu(), ref32, ref_pt, mult=3.0, eps=2 ** -8,
                                       what=f"graph chunk {i} lens {lens} seq {s}")
