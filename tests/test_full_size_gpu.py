"""GPU parity at the full sizes of the baseline configurations, over the WHOLE output.

The CPU oracle cannot evaluate these configurations in seconds, so the same oracle statements (oracle/attention_oracle.py
follows its inputs' device) are evaluated in fp32 on the GPU, TF32 off, for every sequence and head of configurations 2,
3 and 4 and for a few hundred (head, query block) tiles of configuration 5.  Each test ties that device-side evaluation
back to the pinned CPU evaluation on one subset (the two must agree to 1e-5), and keeps the size-independent
properties: run-to-run bit equality, split-size invariance, exact linearity in V."""
import os

import pytest
import torch

from oracle import attention_oracle as O
from _util import max_err

pytestmark = pytest.mark.gpu
H, HK, D = 32, 8, 128


@pytest.fixture(scope="module")
def fa():
    import flash_attn
    import flash_attn_2_cuda
    return flash_attn, flash_attn_2_cuda


@pytest.fixture(autouse=True)
def _no_tf32():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old


def _anchor(dev_out, dev_lse, cpu_out, cpu_lse):
    """The device-side evaluation of the oracle against the pinned CPU evaluation of the same statements."""
    assert max_err(dev_out.cpu(), cpu_out) < 1e-5
    fin = torch.isfinite(cpu_lse)
    assert max_err(dev_lse.cpu()[fin], cpu_lse[fin]) < 1e-4


def _cuda_randn(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).to(dtype)


def test_config2_varlen_prefill_bf16_full(fa):
    flash_attn, cuda = fa
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 4097, (16,), generator=g)
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32)
    total = int(lens.sum())
    q, k, v = _cuda_randn((total, H, D), 20), _cuda_randn((total, HK, D), 21), _cuda_randn((total, HK, D), 22)
    out, lse = flash_attn.flash_attn_varlen_func(q, k, v, cu.cuda(), cu.cuda(), int(lens.max()), int(lens.max()),
                                                 causal=True, return_softmax_lse=True)
    out2, lse2 = flash_attn.flash_attn_varlen_func(q, k, v, cu.cuda(), cu.cuda(), int(lens.max()), int(lens.max()),
                                                   causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # every sequence, every head: the oracle in fp32 on the device; tolerance = the reference's rule against the same
    # math with P in bf16
    anchor = int(lens.argmin())
    for b in range(len(lens)):
        s0, s1 = int(cu[b]), int(cu[b + 1])
        qs, ks, vs = q[s0:s1][None], k[s0:s1][None], v[s0:s1][None]
        ref32, ref_lse = O.attention_ref(qs, ks, vs, causal=True, out_dtype=torch.float32)
        ref_pt, _ = O.attention_ref(qs, ks, vs, causal=True, upcast=False, reorder_ops=True)
        e, e_pt = max_err(out[s0:s1][None], ref32), max_err(ref_pt, ref32)
        assert e <= 2 * e_pt + 2 ** -8, (b, e, e_pt)
        assert max_err(lse[:, s0:s1], ref_lse[0]) < 1e-3, b
        if b == anchor:   # 8 heads of the shortest sequence on the CPU
            c32, c_lse = O.attention_ref(qs[:, :, :8].cpu(), ks[:, :, :2].cpu(), vs[:, :, :2].cpu(), causal=True,
                                         out_dtype=torch.float32)
            _anchor(ref32[:, :, :8], ref_lse[:, :8], c32, c_lse)
        del ref32, ref_pt, ref_lse
    # doubling V doubles the output exactly
    out3 = flash_attn.flash_attn_varlen_func(q, k, (v.float() * 2).to(v.dtype), cu.cuda(), cu.cuda(), int(lens.max()),
                                             int(lens.max()), causal=True)
    assert torch.equal(out3.float(), out.float() * 2)


def _paged_pool(lens, page, seed, dtype=torch.bfloat16):
    nblk = (lens + page - 1) // page
    pool = int(nblk.sum())
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pool, generator=g).to(torch.int32)
    bt = torch.full((len(lens), int(nblk.max())), -1, dtype=torch.int32)
    p = 0
    for i, n in enumerate(nblk.tolist()):
        bt[i, :n] = perm[p:p + n]
        p += n
    kc, vc = _cuda_randn((pool, page, HK, D), seed + 1, dtype), _cuda_randn((pool, page, HK, D), seed + 2, dtype)
    return kc, vc, bt


def test_config3_paged_decode_bf16_full(fa):
    flash_attn, cuda = fa
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(1024, 32769, (64,), generator=g)
    kc, vc, bt = _paged_pool(lens, 256, 30)
    q = _cuda_randn((64, 1, H, D), 33)
    sl = lens.to(torch.int32).cuda()

    def run(partition=None):
        if partition:
            os.environ["FA_B200_DECODE_PARTITION"] = str(partition)
        try:
            o, l = flash_attn.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=sl, block_table=bt.cuda(), causal=True,
                                                      return_softmax_lse=True)
            torch.cuda.synchronize()
        finally:
            os.environ.pop("FA_B200_DECODE_PARTITION", None)
        return o, l

    out, lse = run()
    out_b, lse_b = run()
    assert cuda.device_status() == 0
    assert torch.equal(out, out_b) and torch.equal(lse, lse_b)
    out_c, lse_c = run(partition=4096)            # another split of the same problem
    assert max_err(out, out_c) <= 2 ** -7 and max_err(lse, lse_c) < 1e-4
    # every sequence, every head: the oracle in fp32 on the device (the reference's decode tolerance, tests/test_pa.py:108-117)
    bt_d = bt.cuda()
    ref32, ref_lse = O.paged_decode_ref(q, kc, vc, sl, bt_d, out_dtype=torch.float32)
    assert torch.allclose(out.float(), ref32, atol=1e-2, rtol=1e-2)
    assert max_err(lse, ref_lse) < 1e-3
    b = int(lens.argmin())   # anchor: the shortest sequence on the CPU
    c32, c_lse = O.paged_decode_ref(q[b:b + 1].cpu(), kc.cpu(), vc.cpu(), lens[b:b + 1].to(torch.int32), bt[b:b + 1],
                                    out_dtype=torch.float32)
    _anchor(ref32[b:b + 1], ref_lse[b:b + 1], c32, c_lse)


def test_config4_fp8_decode_and_prefill_full(fa):
    flash_attn, cuda = fa
    # decode: batch 128 x 8192, page 256
    lens = torch.full((128,), 8192, dtype=torch.int64)
    kc16, vc16, bt = _paged_pool(lens, 256, 40)
    q16 = _cuda_randn((128, 1, H, D), 43)
    qd, kd, vd = [(t.abs().max().float() / 448.0).reshape(1) for t in (q16, kc16, vc16)]
    q8, k8, v8 = [(t.float() / s).to(torch.float8_e4m3fn) for t, s in ((q16, qd), (kc16, kd), (vc16, vd))]
    del kc16, vc16
    sl = lens.to(torch.int32).cuda()
    out, lse = flash_attn.flash_attn_with_kvcache(q8, k8, v8, cache_seqlens=sl, block_table=bt.cuda(), causal=True,
                                                  return_softmax_lse=True, q_descale=qd, k_descale=kd, v_descale=vd)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0 and out.dtype == torch.bfloat16
    dkw = dict(q_descale=qd.expand(1, HK), k_descale=kd.expand(1, HK), v_descale=vd.expand(1, HK))
    bt_d = bt.cuda()
    for b in range(128):   # every sequence, every head
        ref32, ref_lse = O.paged_decode_ref(q8[b:b + 1], k8, v8, sl[b:b + 1], bt_d[b:b + 1], out_dtype=torch.float32, **dkw)
        assert torch.allclose(out[b:b + 1].float(), ref32, atol=7e-2, rtol=1e-2), b
        assert max_err(lse[b:b + 1], ref_lse) < 1e-3, b
        if b == 77:   # anchor on the CPU
            ckw = {k: v.cpu() for k, v in dkw.items()}
            c32, c_lse = O.paged_decode_ref(q8[b:b + 1].cpu(), k8.cpu(), v8.cpu(), sl[b:b + 1].cpu(), bt[b:b + 1],
                                            out_dtype=torch.float32, **ckw)
            _anchor(ref32, ref_lse, c32, c_lse)
    del k8, v8
    # prefill: 8 x 4096
    S, nb = 4096, 8
    q16, k16, v16 = _cuda_randn((nb * S, H, D), 44), _cuda_randn((nb * S, HK, D), 45), _cuda_randn((nb * S, HK, D), 46)
    qd, kd, vd = [(t.abs().max().float() / 448.0).reshape(1) for t in (q16, k16, v16)]
    q8, k8, v8 = [(t.float() / s).to(torch.float8_e4m3fn) for t, s in ((q16, qd), (k16, kd), (v16, vd))]
    cu = torch.arange(0, (nb + 1) * S, S, dtype=torch.int32)
    out = flash_attn.flash_attn_varlen_func(q8, k8, v8, cu.cuda(), cu.cuda(), S, S, causal=True, q_descale=qd,
                                            k_descale=kd, v_descale=vd)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    # every sequence, every head: the oracle in fp32 on the device; FP8 tolerance: no worse than twice the error of the
    # same math with P rounded to e4m3, and cosine-diff < 1e-3
    from _util import cos_diff
    kw = dict(q_descale=qd.expand(1, HK), k_descale=kd.expand(1, HK), v_descale=vd.expand(1, HK))
    for b in range(nb):
        s0 = b * S
        qs, ks, vs = q8[s0:s0 + S][None], k8[s0:s0 + S][None], v8[s0:s0 + S][None]
        ref32, _ = O.attention_ref(qs, ks, vs, causal=True, out_dtype=torch.float32, **kw)
        ref_p8, _ = O.attention_ref(qs, ks, vs, causal=True, out_dtype=torch.float32, intermediate_dtype=torch.float8_e4m3fn, **kw)
        e, e_p8 = max_err(out[s0:s0 + S][None], ref32), max_err(ref_p8, ref32)
        assert e <= 2 * e_p8 + 2 ** -7, (b, e, e_p8)
        assert cos_diff(out[s0:s0 + S][None].float(), ref32) < 1e-3, b
        if b == 3:   # anchor: the first 512 query rows of kv head 1 (heads 4..7) on the CPU; they only see the first 512 keys
            ckw = dict(q_descale=qd.cpu().expand(1, 1), k_descale=kd.cpu().expand(1, 1), v_descale=vd.cpu().expand(1, 1))
            c32, c_lse = O.attention_ref(qs[:, :512, 4:8].cpu(), ks[:, :512, 1:2].cpu(), vs[:, :512, 1:2].cpu(), causal=True,
                                         out_dtype=torch.float32, **ckw)
            assert max_err(ref32[:, :512, 4:8].cpu(), c32) < 1e-5
        del ref32, ref_p8


def test_config5_sparse_32k_and_one_million_token_decode(fa):
    flash_attn, cuda = fa
    # ---- block-sparse causal prefill, 1 x 32768, 128x128 tiles at 25 % density per head, diagonal kept
    S = 32768
    n = S // 128
    g = torch.Generator().manual_seed(5)
    tm = torch.rand(1, H, n, n, generator=g) < 0.25
    tm = (tm & torch.tril(torch.ones(n, n, dtype=torch.bool))) | torch.eye(n, dtype=torch.bool)
    cnt, offs = O.tile_mask_to_block_lists(tm, block_m=128, block_n=64, tile_n=128)
    q, k, v = _cuda_randn((1, S, H, D), 50), _cuda_randn((1, S, HK, D), 51), _cuda_randn((1, S, HK, D), 52)
    cc = torch.zeros(1, H, n, dtype=torch.int32, device="cuda")
    ci = torch.zeros(1, H, n, 1, dtype=torch.int32, device="cuda")
    out, lse = flash_attn.sparse_attn_func(q, k, v, cnt.cuda(), offs.cuda(), cc, ci, causal=True, return_softmax_lse=True)
    out2 = flash_attn.sparse_attn_func(q, k, v, cnt.cuda(), offs.cuda(), cc, ci, causal=True)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert torch.equal(out, out2)
    # oracle on whole query tiles (head, q-block), in fp32 on the device: only the kept key tiles are gathered.  The four
    # corner cases plus 300 seeded pairs; the first four are also evaluated on the CPU (anchor).
    pairs = [(0, 0), (7, 100), (31, 255), (18, 37)]
    pg = torch.Generator().manual_seed(55)
    pairs += list(zip(torch.randint(0, H, (300,), generator=pg).tolist(), torch.randint(0, n, (300,), generator=pg).tolist()))
    for i, (head, m) in enumerate(pairs):
        kept = torch.nonzero(tm[0, head, m]).flatten().tolist()
        rows = slice(m * 128, m * 128 + 128)
        ks = torch.cat([k[0, j * 128:(j + 1) * 128, head // 4] for j in kept])[None, :, None]
        vs = torch.cat([v[0, j * 128:(j + 1) * 128, head // 4] for j in kept])[None, :, None]
        qs = q[0, rows, head][None, :, None]
        # causal mask inside the diagonal tile only (it is the last kept tile)
        mask = torch.zeros(128, len(kept) * 128, dtype=torch.bool, device="cuda")
        if kept[-1] == m:
            mask[:, -128:] = torch.triu(torch.ones(128, 128, dtype=torch.bool, device="cuda"), diagonal=1)
        ref32, ref_lse = O.attention_ref(qs, ks, vs, out_dtype=torch.float32, extra_mask=mask)
        ref_pt, _ = O.attention_ref(qs, ks, vs, upcast=False, reorder_ops=True, extra_mask=mask)
        e, e_pt = max_err(out[0, rows, head], ref32[0, :, 0]), max_err(ref_pt, ref32)
        assert e <= 2 * e_pt + 2 ** -8, (head, m, e, e_pt)
        assert max_err(lse[0, head, rows], ref_lse[0, 0]) < 1e-3
        if i < 4:
            c32, c_lse = O.attention_ref(qs.cpu(), ks.cpu(), vs.cpu(), out_dtype=torch.float32, extra_mask=mask.cpu())
            _anchor(ref32, ref_lse, c32, c_lse)
    del q, k, v, out, out2
    # ---- one sequence of 1,048,576 tokens, split-KV into fp32 partials and combined (the 8-GPU path on one GPU:
    # eight page ranges decoded separately, partials merged by the combine kernel)
    L, page, parts = 1 << 20, 256, 8
    npages = L // page
    kc, vc = _cuda_randn((npages, page, HK, D), 60), _cuda_randn((npages, page, HK, D), 61)
    qq = _cuda_randn((1, 1, H, D), 62)
    perm = torch.randperm(npages, generator=g).to(torch.int32)
    full = flash_attn.flash_attn_with_kvcache(qq, kc, vc, cache_seqlens=torch.tensor([L], dtype=torch.int32, device="cuda"),
                                              block_table=perm.view(1, -1).cuda(), causal=True)
    per = npages // parts
    o_parts, l_parts = [], []
    for r in range(parts):
        o, l = cuda.decode_partial(qq, kc, vc, torch.tensor([per * page], dtype=torch.int32, device="cuda"),
                                   perm[r * per:(r + 1) * per].view(1, -1).contiguous().cuda(), D ** -0.5)
        o_parts.append(o.view(H, D))
        l_parts.append(l.view(H))
    merged, lse_m = cuda.combine(torch.stack(o_parts), torch.stack(l_parts), out_dtype=torch.bfloat16, h=H)
    torch.cuda.synchronize()
    assert cuda.device_status() == 0
    assert max_err(merged.view(1, 1, H, D), full) <= 2 ** -7
    # oracle for every kv head in fp32 on the device, keys streamed in the block table's order; kv head 2 also on the CPU
    perm_d = perm.long().cuda()
    for hk in range(HK):
        kk = kc[perm_d, :, hk].reshape(L, D)[None, :, None]
        vv = vc[perm_d, :, hk].reshape(L, D)[None, :, None]
        ref32, ref_lse = O.attention_ref(qq[:, :, 4 * hk:4 * hk + 4], kk, vv, out_dtype=torch.float32)
        assert torch.allclose(full[:, :, 4 * hk:4 * hk + 4].float(), ref32, atol=1e-2, rtol=1e-2), hk
        assert max_err(lse_m.view(H)[4 * hk:4 * hk + 4], ref_lse[0, :, 0]) < 1e-3, hk
        if hk == 2:
            c32, c_lse = O.attention_ref(qq[:, :, 8:12].cpu(), kk.cpu(), vv.cpu(), out_dtype=torch.float32)
            _anchor(ref32, ref_lse, c32, c_lse)
