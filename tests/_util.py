"""Shared helpers for the GPU parity tests: seeded CPU inputs (identical for the oracle and the device),
tolerance rules taken from the reference's tests."""
import math

import torch

from oracle import attention_oracle as O


def gen(seed):
    return torch.Generator().manual_seed(seed)


def randn(g, *shape, dtype=torch.bfloat16):
    return torch.randn(*shape, generator=g).to(dtype)


def make_paged(g, lens, h_k, page, dtype, spare=3, poison=True, d=128):
    """Paged pool + block table built like the reference's _generate_block_kvcache: a seeded random
    permutation of the physical pages, spare pages, unused table slots = -1.  With ``poison`` the spare
    pages and the token rows past each sequence's end are NaN (fp8: 0x7f NaN pattern) so that any read past
    the end shows up in the output (the reference's prefix-cache tests do the same)."""
    nblk = [(L + page - 1) // page for L in lens]
    pool = sum(nblk) + spare
    kc = torch.randn(pool, page, h_k, d, generator=g)
    vc = torch.randn(pool, page, h_k, d, generator=g)
    perm = torch.randperm(pool, generator=g).to(torch.int32)
    bt = torch.full((len(lens), max(max(nblk), 1)), -1, dtype=torch.int32)
    used = torch.zeros(pool, dtype=torch.bool)
    p = 0
    for i, n in enumerate(nblk):
        bt[i, :n] = perm[p:p + n]
        used[perm[p:p + n].long()] = True
        p += n
    if poison:
        kc[~used] = float("nan")
        vc[~used] = float("nan")
        for i, L in enumerate(lens):
            if L % page:
                last = int(bt[i, nblk[i] - 1])
                kc[last, L % page:] = float("nan")
                vc[last, L % page:] = float("nan")
    return kc.to(dtype), vc.to(dtype), bt, torch.tensor(lens, dtype=torch.int32)


def clean_nan(t):
    """NaN-poisoned caches are for the device; the oracle never reads those rows, but keep it finite."""
    return torch.nan_to_num(t.float(), nan=0.0).to(t.dtype)


def max_err(a, b):
    return (a.float() - b.float()).abs().max().item()


def cos_diff(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return 1.0 - (2 * (a * b).sum() / ((a * a).sum() + (b * b).sum()).clamp_min(1e-30)).item()


def assert_close_to_oracle(out, ref32, ref_pt, mult=2.0, eps=1e-5, what=""):
    """The reference's rule: max|out - ref_fp32| <= mult * max|out_pt - ref_fp32| + eps where out_pt is the
    same math in the input dtype (tests/test_flash_attn.py:989, 2103, 3207-3210)."""
    e = max_err(out, ref32)
    e_pt = max_err(ref_pt, ref32)
    assert not torch.isnan(out.float()).any(), f"{what}: NaN in output"
    assert e <= mult * e_pt + eps, f"{what}: err {e:.3e} > {mult} * {e_pt:.3e} + {eps}"
    return e, e_pt
