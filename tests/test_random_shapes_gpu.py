"""Seeded random configurations over the public entries (fixed, varlen, paged prefill, decode, few-token decode):
ragged and empty sequences, every head grouping, page sizes, head dimensions, causal / window / sink options drawn at
random, each checked against the CPU oracle with the reference's tolerance rule.  The draws are reproducible (one
generator per case) and small enough for the oracle to finish in seconds."""
import os
import random

import pytest
import torch

from oracle import attention_oracle as O
from _util import assert_close_to_oracle, clean_nan, gen, make_paged, max_err, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    assert torch.cuda.is_available()
    return flash_attn, flash_attn_2_cuda


def _options(rng, allow_right=True):
    causal = rng.random() < 0.5
    window = (-1, -1)
    if rng.random() < 0.35:
        window = (rng.choice([0, 1, 17, 64, 200]), 0 if causal else (rng.choice([0, 3, 50]) if allow_right else -1))
    sink = rng.random() < 0.3
    return causal, window, sink


def _heads(rng, max_group=8):
    h_k = rng.choice([1, 2, 4])
    group = rng.choice([g for g in (1, 2, 3, 4, 8, 16) if g <= max_group])
    return h_k * group, h_k


def _dim(rng):
    return rng.choice([128, 128, 128, 64, 192, 256])


def _len(rng, hi):
    return rng.choice([0, 1, 2, 63, 64, 65, 127, 128, 129, rng.randint(1, hi), rng.randint(1, hi), rng.randint(1, hi)])


@pytest.mark.parametrize("seed", range(36))
def test_random_fixed_and_varlen(fa, seed):
    flash_attn, cuda = fa
    rng = random.Random(1000 + seed)
    g = gen(1000 + seed)
    dtype = rng.choice([torch.bfloat16, torch.float16])
    d, (h, h_k) = _dim(rng), _heads(rng)
    causal, window, sink = _options(rng)
    s_aux = (torch.randn(h, generator=g) * 2).to(dtype) if sink else None
    kw = dict(causal=causal, window_size=window, s_aux=None if s_aux is None else s_aux.cuda())
    okw = dict(causal=causal, window_size=window, s_aux=s_aux)
    if seed % 2 == 0:
        b, sq, sk = rng.randint(1, 3), max(1, _len(rng, 500)), max(1, _len(rng, 700))
        q, k, v = randn(g, b, sq, h, d, dtype=dtype), randn(g, b, sk, h_k, d, dtype=dtype), randn(g, b, sk, h_k, d, dtype=dtype)
        out, lse, _ = flash_attn.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True, **kw)
        torch.cuda.synchronize()
        if sq == 1:
            okw["causal"] = False                      # a single query row: the reference drops the causal flag
        ref32, ref_lse = O.attention_ref(q, k, v, out_dtype=torch.float32, **okw)
        ref_pt, _ = O.attention_ref(q, k, v, upcast=False, reorder_ops=True, **okw)
        what = f"fixed b{b} sq{sq} sk{sk} h{h}/{h_k} d{d} {kw}"
    else:
        n = rng.randint(1, 5)
        lens_q = [_len(rng, 400) for _ in range(n)]
        lens_k = lens_q if rng.random() < 0.5 else [_len(rng, 600) for _ in range(n)]
        if sum(lens_q) == 0:
            lens_q[0] = 5
            lens_k = list(lens_k)
            lens_k[0] = max(lens_k[0], 5)
        cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
        ck = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
        tk = max(int(ck[-1]), 1)
        q, k, v = randn(g, int(cq[-1]), h, d, dtype=dtype), randn(g, tk, h_k, d, dtype=dtype), randn(g, tk, h_k, d, dtype=dtype)
        k, v = k[:int(ck[-1])], v[:int(ck[-1])]
        out, lse = flash_attn.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cq.cuda(), ck.cuda(), max(max(lens_q), 1),
                                                     max(max(lens_k), 1), return_softmax_lse=True, **kw)
        torch.cuda.synchronize()
        ref32, ref_lse = O.attention_varlen_ref(q, k, v, cq, ck, out_dtype=torch.float32, **okw)
        ref_pt, _ = O.attention_varlen_ref(q, k, v, cq, ck, upcast=False, reorder_ops=True, **okw)
        what = f"varlen q{lens_q} k{lens_k} h{h}/{h_k} d{d} {kw}"
    assert cuda.device_status() == 0, what
    assert_close_to_oracle(out.cpu(), ref32, ref_pt, mult=2.0, eps=2 ** -8, what=what)
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse.cpu()), fin), what
    if fin.any():
        assert max_err(lse.cpu()[fin], ref_lse[fin]) < 1e-3, what


@pytest.mark.parametrize("seed", range(36))
def test_random_paged(fa, seed):
    flash_attn, cuda = fa
    rng = random.Random(2000 + seed)
    g = gen(2000 + seed)
    dtype = rng.choice([torch.bfloat16, torch.float16])
    d, (h, h_k) = _dim(rng), _heads(rng, max_group=16 if seed % 3 == 0 else 8)
    page = rng.choice([16, 32, 64, 128, 256])
    n = rng.randint(1, 5)
    lens_k = [max(1, _len(rng, 1500)) for _ in range(n)]
    kc, vc, bt, sl = make_paged(g, lens_k, h_k, page, dtype, d=d)
    kcc, vcc = clean_nan(kc), clean_nan(vc)
    causal, window, sink = _options(rng, allow_right=False)
    s_aux = (torch.randn(h, generator=g) * 2).to(dtype) if sink else None
    mode = seed % 3
    if mode == 0:      # decode: one token per sequence, with an empty sequence now and then
        if rng.random() < 0.5:
            sl[rng.randrange(n)] = 0
        q = randn(g, n, 1, h, d, dtype=dtype)
        part = rng.choice([None, 64, 256]) if dtype != torch.float8_e4m3fn else None
        if part:
            os.environ["FA_B200_DECODE_PARTITION"] = str(part)
        try:
            out = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                     causal=True, window_size=(window[0], -1),
                                                     s_aux=None if s_aux is None else s_aux.cuda())
            torch.cuda.synchronize()
        finally:
            os.environ.pop("FA_B200_DECODE_PARTITION", None)
        lens_q = [1] * n
        qs = [q[i] for i in range(n)]
        outs = [out[i].cpu() for i in range(n)]
        causal, window = True, (window[0], -1)
    elif mode == 1:    # a few query tokens per sequence on the decode kernel, or many on the prefill kernel
        sq = rng.choice([2, 3, 4, 40])
        sl = torch.maximum(sl, torch.tensor(sq, dtype=torch.int32))
        for i in range(n):
            if sl[i] > lens_k[i]:       # grown past the generated (and un-poisoned) keys: keep the sequence as generated
                sl[i] = lens_k[i]
        sq = min(sq, int(sl.min()))
        q = randn(g, n, sq, h, d, dtype=dtype)
        out = flash_attn.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=sl.cuda(), block_table=bt.cuda(),
                                                 causal=True, window_size=(window[0], -1),
                                                 s_aux=None if s_aux is None else s_aux.cuda())
        torch.cuda.synchronize()
        lens_q = [sq] * n
        qs = [q[i] for i in range(n)]
        outs = [out[i].cpu() for i in range(n)]
        causal, window = True, (window[0], -1)
    else:              # ragged chunks of queries against paged prefixes
        lens_q = [max(1, min(_len(rng, 300), lk)) for lk in lens_k]
        cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
        q = randn(g, int(cq[-1]), h, d, dtype=dtype)
        out = flash_attn.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cq.cuda(), None, max(lens_q), max(lens_k),
                                                seqused_k=sl.cuda(), causal=True, window_size=(window[0], -1 if window[0] < 0 else 0),
                                                block_table=bt.cuda(), s_aux=None if s_aux is None else s_aux.cuda())
        torch.cuda.synchronize()
        qs = [q[int(cq[i]):int(cq[i + 1])] for i in range(n)]
        outs = [out[int(cq[i]):int(cq[i + 1])].cpu() for i in range(n)]
        causal, window = True, (window[0], -1 if window[0] < 0 else 0)
    what0 = f"paged mode{mode} page{page} lens{[int(x) for x in sl]} q{lens_q} h{h}/{h_k} d{d} win{window} sink{sink}"
    assert cuda.device_status() == 0, what0
    for i in range(n):
        lk = int(sl[i])
        if lk == 0:
            assert torch.all(outs[i] == 0) or s_aux is not None, what0
            continue
        ki, vi = O.gather_paged_kv(kcc, bt[i], lk)[None], O.gather_paged_kv(vcc, bt[i], lk)[None]
        eff_causal = causal and lens_q[i] > 1
        win = window if lens_q[i] > 1 else (window[0], -1)
        ref32, _ = O.attention_ref(qs[i][None], ki, vi, causal=eff_causal, window_size=win, s_aux=s_aux, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qs[i][None], ki, vi, causal=eff_causal, window_size=win, s_aux=s_aux, upcast=False,
                                    reorder_ops=True)
        assert_close_to_oracle(outs[i][None], ref32, ref_pt, mult=3.0, eps=1e-5 + 2 ** -8, what=f"{what0} seq {i}")
