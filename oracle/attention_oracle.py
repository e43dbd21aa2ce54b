"""CPU restatement of the reference's PyTorch attention oracles (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA hot path.  It is never imported by the product
package; only tests, the smoke entry and the benchmark's CPU-baseline leg use it.

Parity status: PINNED.  Every function below is checked bit-for-bit (same torch build) against the
reference's own test oracles imported from the reference tree by
``tests/golden/make_golden.py``; the resulting vectors are committed under ``tests/golden`` and
re-checked by ``tests/test_oracle_golden.py`` on CPU.

Each function cites the reference code it follows (paths relative to the reference project).
All math is fp32 on the CPU ("upcast=True" in the reference's vocabulary) unless stated.

The attention functions follow their inputs' device, so the GPU tests can also evaluate the same statements in
fp32 on the device over whole configurations (TF32 off); such a device-side evaluation is tied back to the pinned
CPU evaluation on a subset by the tests that use it.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

E4M3_MAX = 448.0


# ----------------------------------------------------------------------------------------------
# dense / fixed-length
# ----------------------------------------------------------------------------------------------
def causal_mask_bottom_right(seqlen_q: int, seqlen_k: int, device=None) -> torch.Tensor:
    """True where the score is masked OUT.  Follows construct_local_mask with window (-1, 0):
    ``col > row + seqlen_k - seqlen_q`` (tests/test_flash_attn.py:185-217)."""
    row = torch.arange(seqlen_q, dtype=torch.long, device=device).view(-1, 1)
    col = torch.arange(seqlen_k, dtype=torch.long, device=device)
    return col > row + seqlen_k - seqlen_q


def attention_ref(q, k, v, causal=False, upcast=True, reorder_ops=False, softmax_scale=None,
                  q_descale=None, k_descale=None, v_descale=None, intermediate_dtype=None,
                  extra_mask=None, out_dtype=None, s_aux=None, window_size=(-1, -1)):
    """Fixed-length GQA attention.  Follows attention_ref (tests/test_flash_attn.py:220-321) and its
    FP8 sibling with ``[b, h]`` descales and P round-tripped through ``intermediate_dtype``
    (tests/test_flash_attn_varlen_fp8.py:214-320).

    q: (b, sq, h, d); k, v: (b, sk, hk, d).  ``extra_mask`` (broadcastable to (b, h, sq, sk), True =
    masked out) carries tile masks for the block-sparse oracle.
    ``s_aux`` (h,): attention sinks, one extra logit per query head that joins the softmax as a last column
    and is dropped afterwards; ``window_size`` (left, right): key j is visible to query i only if
    i + sk - sq - left <= j <= i + sk - sq + right (-1 = unbounded).  Both follow the reference's sink oracle
    (tests/test_flash_attn_saux.py:178-224).
    Returns (out in q.dtype (or fp32/bf16 for fp8 inputs, see below), lse fp32 (b, h, sq)).
    Fully masked rows give out = 0 and lse = +inf (with sinks: lse = the sink).
    """
    dtype_og = q.dtype
    is_fp8 = dtype_og in (torch.float8_e4m3fn, torch.float8_e5m2)
    if upcast or is_fp8:
        q, k, v = q.float(), k.float(), v.float()
    g = q.shape[2] // k.shape[2]
    if q_descale is not None:
        q = q * q_descale.float().repeat_interleave(g, dim=1)[:, None, :, None]
    if k_descale is not None:
        k = k * k_descale.float()[:, None, :, None]
    if v_descale is not None:
        v = v * v_descale.float()[:, None, :, None]
    sq, sk = q.shape[1], k.shape[1]
    k = k.repeat_interleave(g, dim=2)
    v = v.repeat_interleave(g, dim=2)
    d = q.shape[-1]
    if softmax_scale is None:  # the reference divides by sqrt(d); keep that exact operation
        qs, ks = (q / math.sqrt(d), k) if not reorder_ops else (q, k / math.sqrt(d))
    else:
        qs, ks = (q * softmax_scale, k) if not reorder_ops else (q, k * softmax_scale)
    scores = torch.einsum("bthd,bshd->bhts", qs, ks)
    masked = None
    if causal:
        masked = causal_mask_bottom_right(sq, sk, q.device)
    if window_size[0] >= 0 or window_size[1] >= 0:
        row = torch.arange(sq, dtype=torch.long, device=q.device).view(-1, 1)
        col = torch.arange(sk, dtype=torch.long, device=q.device).view(1, -1)
        wmask = torch.zeros(sq, sk, dtype=torch.bool, device=q.device)
        if window_size[0] >= 0:
            wmask |= col < row + sk - sq - window_size[0]
        if window_size[1] >= 0:
            wmask |= col > row + sk - sq + window_size[1]
        masked = wmask if masked is None else (masked | wmask)
    if extra_mask is not None:
        masked = extra_mask if masked is None else (masked | extra_mask)
    if masked is not None:
        scores = scores.masked_fill(masked, float("-inf"))
    if s_aux is not None:
        sink = (s_aux.float() if (upcast or is_fp8) else s_aux).reshape(1, -1, 1, 1).expand(scores.shape[0], -1, sq, -1)
        scores = torch.cat([scores, sink.to(scores.dtype)], dim=-1)
    attention = torch.softmax(scores, dim=-1)
    if masked is not None and s_aux is None:
        all_masked = torch.all(masked.expand(scores.shape), dim=-1, keepdim=True)
        attention = attention.masked_fill(all_masked, 0.0)
    if s_aux is not None:
        attention = attention[..., :-1]
    attention = attention.to(v.dtype)
    if intermediate_dtype is not None:
        attention = attention.to(intermediate_dtype).to(attention.dtype)
    out = torch.einsum("bhts,bshd->bthd", attention.float(), v.float())
    lse = scores.logsumexp(dim=-1).float()
    lse = torch.where(lse == float("-inf"), torch.full_like(lse, float("inf")), lse)
    if out_dtype is None:
        out_dtype = torch.bfloat16 if is_fp8 else dtype_og
    return out.to(out_dtype), lse


def attention_varlen_ref(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=False, upcast=True,
                         softmax_scale=None, q_descale=None, k_descale=None, v_descale=None,
                         intermediate_dtype=None, reorder_ops=False, out_dtype=None, s_aux=None,
                         window_size=(-1, -1)):
    """Packed varlen attention, one sequence at a time.  Follows attention_varlen_ref
    (tests/test_flash_attn.py:432-494): LSE is (h, total_q) with -inf replaced by +inf and empty
    key ranges give zeros (LSE = the sink where sinks are given).  Descales are (batch, heads_k) fp32 or None."""
    nb = cu_seqlens_q.numel() - 1
    outs, lses = [], []
    cq = cu_seqlens_q.tolist()
    ck = cu_seqlens_k.tolist()
    for b in range(nb):
        qi = q[cq[b]:cq[b + 1]][None]
        ki = k[ck[b]:ck[b + 1]][None]
        vi = v[ck[b]:ck[b + 1]][None]
        if ki.shape[1] == 0:
            is_fp8 = q.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
            outs.append(torch.zeros(qi.shape[1], q.shape[1], v.shape[-1], device=q.device,
                                    dtype=out_dtype or (torch.bfloat16 if is_fp8 else q.dtype)))
            if s_aux is None:
                lses.append(torch.full((q.shape[1], qi.shape[1]), float("inf"), device=q.device))
            else:   # the sink is the only term of such a row's sum, as for fully masked rows in attention_ref
                lses.append(s_aux.float().reshape(-1, 1).expand(q.shape[1], qi.shape[1]).clone())
            continue
        o, l = attention_ref(
            qi, ki, vi, causal=causal, upcast=upcast, softmax_scale=softmax_scale,
            reorder_ops=reorder_ops, out_dtype=out_dtype,
            q_descale=None if q_descale is None else q_descale[b:b + 1],
            k_descale=None if k_descale is None else k_descale[b:b + 1],
            v_descale=None if v_descale is None else v_descale[b:b + 1],
            intermediate_dtype=intermediate_dtype, s_aux=s_aux, window_size=window_size)
        outs.append(o[0])
        lses.append(l[0])
    return torch.cat(outs, dim=0), torch.cat(lses, dim=-1).float()


# ----------------------------------------------------------------------------------------------
# paged KV
# ----------------------------------------------------------------------------------------------
def paged_element_offset(block_table_row: Sequence[int], token: int, kv_head: int, d: int,
                         page_size: int, stride_block: int, stride_token: int,
                         stride_head: int) -> int:
    """Integer address (in elements) of K/V[token, kv_head, d] of one sequence inside a paged
    BSHD pool.  Follows the reference's decode addressing: physical page =
    block_table[seq*max_blocks + token // page] (src/paged_attention.cu:146,209), row in page =
    token % page, offset = page*stride0 + row*(Hkv*D) + kv_head*D + d
    (src/paged_attention_decode_arch.h:3992-3998)."""
    page = int(block_table_row[token // page_size])
    return page * stride_block + (token % page_size) * stride_token + kv_head * stride_head + d


def gather_paged_kv(cache: torch.Tensor, block_table_row: torch.Tensor, seqlen: int) -> torch.Tensor:
    """(num_blocks, page, hk, d) pool + one block_table row -> contiguous (seqlen, hk, d).
    Follows _generate_block_kvcache's gather (tests/test_flash_attn.py:3221-3236)."""
    page = cache.shape[1]
    nblk = (seqlen + page - 1) // page
    idx = block_table_row[:nblk].to(torch.long)
    return cache[idx].reshape(nblk * page, *cache.shape[2:])[:seqlen]


def paged_decode_ref(q, k_cache, v_cache, cache_seqlens, block_table, softmax_scale=None,
                     causal=True, q_descale=None, k_descale=None, v_descale=None, upcast=True,
                     reorder_ops=False, out_dtype=None, s_aux=None, window_size=(-1, -1)):
    """Decode over a paged cache, one sequence at a time (a whole-batch call would need the GQA
    repeat of every sequence at once).  Follows the per-sequence loop of tests/test_pa.py:33-48,
    91-106 and the kvcache test (tests/test_flash_attn.py:3221-3236).
    q: (b, sq, h, d).  Returns (out (b, sq, h, d), lse (b, h, sq))."""
    b = q.shape[0]
    outs, lses = [], []
    for i in range(b):
        L = int(cache_seqlens[i])
        ki = gather_paged_kv(k_cache, block_table[i], L)[None]
        vi = gather_paged_kv(v_cache, block_table[i], L)[None]
        if L == 0:
            is_fp8 = q.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
            outs.append(torch.zeros(1, q.shape[1], q.shape[2], q.shape[3], device=q.device,
                                    dtype=out_dtype or (torch.bfloat16 if is_fp8 else q.dtype)))
            lses.append(torch.full((1, q.shape[2], q.shape[1]), float("inf"), device=q.device))
            continue
        o, l = attention_ref(
            q[i:i + 1], ki, vi, causal=causal, softmax_scale=softmax_scale, upcast=upcast,
            reorder_ops=reorder_ops, out_dtype=out_dtype, s_aux=s_aux, window_size=window_size,
            q_descale=None if q_descale is None else q_descale[i:i + 1],
            k_descale=None if k_descale is None else k_descale[i:i + 1],
            v_descale=None if v_descale is None else v_descale[i:i + 1])
        outs.append(o)
        lses.append(l)
    return torch.cat(outs, dim=0), torch.cat(lses, dim=0)


# ----------------------------------------------------------------------------------------------
# split-KV merge
# ----------------------------------------------------------------------------------------------
def merge_partials_ref(o_partial: torch.Tensor, lse_partial: torch.Tensor):
    """Combine per-partition results.  o_partial: (parts, ..., d) fp32, each already normalised by
    its own partition's softmax sum; lse_partial: (parts, ...) natural-log LSE (-inf or +inf marks
    an empty partition).  Same math as the reference's combine kernels
    (m = max_i; w_i = expsum_i * 2^(max_i - m); O = sum w_i O_i / sum w_i,
    src/paged_attention.h:356-445; merged LSE = ln sum e^{lse_i - M} + M,
    csrc/flash_attn_hipc/src/flash_fwd_reduce.h:313-464) and of merge() in
    tests/welm/test_welm_ops.py:22-32, restated in LSE form.
    Returns (out fp32 (..., d), lse fp32 (...)) with lse = +inf, out = 0 for rows with no keys."""
    lse = lse_partial.float().clone()
    lse[lse == float("inf")] = float("-inf")
    m = lse.max(dim=0, keepdim=True).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse - m_safe)
    wsum = w.sum(dim=0)
    out = (o_partial.float() * w[..., None]).sum(dim=0)
    out = torch.where(wsum[..., None] > 0, out / wsum[..., None].clamp_min(1e-38), torch.zeros_like(out))
    lse_out = torch.log(wsum) + m_safe[0]
    lse_out = torch.where(wsum > 0, lse_out, torch.full_like(lse_out, float("inf")))
    return out, lse_out


def partial_slot_index(split: int, seq: int, head: int, batch: int, heads: int) -> int:
    """Flat slot of a (split, seq, head) partial in the split-major workspace
    ``[split][seq][head]`` used by the CUDA decode and combine kernels."""
    return (split * batch + seq) * heads + head


# ----------------------------------------------------------------------------------------------
# FP8 e4m3 with descale
# ----------------------------------------------------------------------------------------------
def quantize_e4m3_per_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """descale = amax/448 (fp32), x_fp8 = (x/descale).to(e4m3).  Same recipe as the reference's FP8
    tests (tests/test_flash_attn_varlen_fp8.py:259-266 style per-tensor scaling)."""
    amax = x.float().abs().max().clamp_min(1e-12)
    descale = (amax / E4M3_MAX).to(torch.float32)
    xq = (x.float() / descale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return xq, descale.reshape(1)


# ----------------------------------------------------------------------------------------------
# block-sparse (tile lists)
# ----------------------------------------------------------------------------------------------
def tile_mask_to_block_lists(tile_mask: torch.Tensor, block_m: int, block_n: int = 64,
                             tile_n: Optional[int] = None):
    """tile_mask: (b, h, n_qblocks, n_ktiles) bool over (block_m x tile_n) tiles.  Produces the
    reference's metadata: block_count (b, h, n_qblocks) int32 and block_offset
    (b, h, n_qblocks, NNZ_S) int32 holding ascending K ROW offsets of block_n(=64)-row K tiles
    (csrc/flash_attn_cutlass/flash_api_sparse.cpp:127-137; offsets not block ids,
    src/flash_fwd_sparse_kernel.h:226-237).  Unused slots hold a large sentinel like
    block_map_to_block_offset does (flash_attn/utils/sparse_utils.py:526-563)."""
    if tile_n is None:
        tile_n = block_m
    b, h, nq, nk = tile_mask.shape
    sub = tile_n // block_n
    fine = tile_mask.repeat_interleave(sub, dim=-1)  # (b,h,nq,nk*sub) over 64-row K tiles
    count = fine.sum(dim=-1).to(torch.int32)
    nnz = max(int(count.max()), 1)
    idx = torch.arange(fine.shape[-1], dtype=torch.int64).expand_as(fine).clone()
    idx[~fine] = 10_000_000
    srt = torch.sort(idx, dim=-1).values[..., :nnz]
    offs = torch.where(srt >= 10_000_000, srt, srt * block_n)
    return count, offs.to(torch.int32)


def block_lists_to_dense_mask(block_count, block_offset, seqlen_q, seqlen_k, block_m, block_n=64):
    """Inverse of the above: (b, h, sq, sk) bool, True = masked OUT.  Expansion follows
    attention_blocksparse_ref's repeat of the block mask (tests/test_flash_attn.py:416-421)."""
    b, h, nq = block_count.shape
    keep = torch.zeros(b, h, seqlen_q, seqlen_k, dtype=torch.bool)
    bc = block_count.tolist()
    bo = block_offset.tolist()
    for bi in range(b):
        for hi in range(h):
            for m in range(nq):
                r0, r1 = m * block_m, min((m + 1) * block_m, seqlen_q)
                for j in range(bc[bi][hi][m]):
                    c0 = bo[bi][hi][m][j]
                    keep[bi, hi, r0:r1, c0:min(c0 + block_n, seqlen_k)] = True
    return ~keep


def sparse_attention_ref(q, k, v, block_count, block_offset, causal, block_m, softmax_scale=None,
                         upcast=True):
    """Block-list attention = dense attention with the expanded tile mask (and the causal mask on
    top).  Mirrors what the reference's sparse kernel computes for a block list
    (src/flash_fwd_sparse_kernel.h:226-371) and the manual check in
    tests/test_spas_fa2_attn.py:64-110."""
    mask = block_lists_to_dense_mask(block_count, block_offset, q.shape[1], k.shape[1], block_m)
    return attention_ref(q, k, v, causal=causal, upcast=upcast, softmax_scale=softmax_scale,
                         extra_mask=mask)


def sparse_block_m(seqlen_q: int) -> int:
    """Host rule NUM_ROWS == ceil(Sq / (Sq <= 2048 ? 64 : 128))
    (csrc/flash_attn_cutlass/flash_api_sparse.cpp:127-137)."""
    return 64 if seqlen_q <= 2048 else 128


# ----------------------------------------------------------------------------------------------
# KV-cache append + rotary embedding
# ----------------------------------------------------------------------------------------------
def rotary_ref(x, cos, sin, seqlen_offsets, interleaved=False, per_token=True, out_dtype=None):
    """Rotary embedding of x (batch, seqlen, nheads, d) at positions seqlen_offsets[b] + s (or
    seqlen_offsets[b] for every s when ``per_token`` is False).  cos, sin: (seqlen_ro, rotary_dim / 2).
    The pairing and the formula are those of rotate_half / apply_rotary_emb_torch
    (flash_attn/layers/rotary.py:11-33); the arithmetic is that of the reference's kernel: fp32 from the
    stored 16-bit values, ``o0 = x0*cos - x1*sin``, ``o1 = x0*sin + x1*cos``, one rounding to the element
    type (flash_attn/ops/triton/rotary.py:69-90).  Returns ``out_dtype`` (default x.dtype)."""
    b, s, h, d = x.shape
    half = cos.shape[-1]
    ro = 2 * half
    assert ro <= d
    pos = seqlen_offsets.to(torch.long).view(b, 1) + (torch.arange(s).view(1, s) if per_token else torch.zeros(1, s, dtype=torch.long))
    c = cos.float()[pos].unsqueeze(2)   # (b, s, 1, half)
    sn = sin.float()[pos].unsqueeze(2)
    xf = x.float()
    xr = xf[..., :ro]
    if interleaved:
        x0, x1 = xr[..., 0::2], xr[..., 1::2]
    else:
        x0, x1 = xr[..., :half], xr[..., half:]
    o0 = x0 * c - x1 * sn
    o1 = x0 * sn + x1 * c
    if interleaved:
        rot = torch.stack((o0, o1), dim=-1).reshape(b, s, h, ro)
    else:
        rot = torch.cat((o0, o1), dim=-1)
    out = torch.cat((rot, xf[..., ro:]), dim=-1)
    return out.to(out_dtype if out_dtype is not None else x.dtype)


def kv_append_ref(k_cache, v_cache, block_table, cache_seqlens, k_new, v_new, cos=None, sin=None,
                  interleaved=False):
    """In-place append of k_new / v_new (batch, seqlen_new, nheads_k, d) to a paged cache
    (num_blocks, page, nheads_k, d) at positions cache_seqlens[b] .. + seqlen_new - 1, keys rotated at
    those positions when cos/sin are given; returns cache_seqlens + seqlen_new.  Follows the update the
    reference's test applies to its cache copy (``update_mask`` / ``k_cache_ref[update_mask] = k_ro``,
    tests/test_flash_attn.py:3073-3122) with the page addressing of paged_element_offset()."""
    b, s_new = k_new.shape[0], k_new.shape[1]
    page = k_cache.shape[1]
    k_ro = rotary_ref(k_new, cos, sin, cache_seqlens, interleaved) if cos is not None else k_new
    for bi in range(b):
        for s in range(s_new):
            pos = int(cache_seqlens[bi]) + s
            blk = int(block_table[bi, pos // page])
            k_cache[blk, pos % page] = k_ro[bi, s]
            v_cache[blk, pos % page] = v_new[bi, s]
    return (cache_seqlens + s_new).to(torch.int32)
