"""Public Python API of the attention hot path, signature-compatible with the reference's
flash_attn/flash_attn_interface.py (flash_attn_func :1646, flash_attn_varlen_func :2111,
flash_attn_with_kvcache :2478, sparse_attn_func :2778).

Forward only.  Options outside the hot path (dropout, alibi, softcap, sliding window, attention sinks, rotary,
KV append, head dimensions other than 128, backward) raise NotImplementedError instead of silently taking
another code path: there is no Triton, eager or CPU fallback.
"""
from typing import List, Optional, Union

import torch

import flash_attn_2_cuda as flash_attn_cuda

DEFAULT_FA_VERSION = 2


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _no_backward(*tensors):
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise NotImplementedError("the B200 hot path is forward only: call under torch.no_grad() or detach inputs")


def flash_attn_func(
    q,
    k,
    v,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size=(-1, -1),  # -1 means infinite context window
    softcap=0.0,  # 0.0 means deactivated
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    bhsd=False,
    s_aux=None,
):
    """Fixed-length attention with MQA/GQA.  q: (batch, seqlen, nheads, 128); k, v: (batch, seqlen_k, nheads_k, 128).
    The causal mask is aligned to the bottom-right corner; fully masked rows return 0.
    Returns out, or (out, softmax_lse (batch, nheads, seqlen), None) when return_attn_probs=True."""
    _no_backward(q, k, v)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    res = flash_attn_cuda.fwd(
        q, k, v, None, alibi_slopes, dropout_p, softmax_scale, causal, window_size[0], window_size[1], softcap,
        False, None, bhsd, s_aux)
    out, softmax_lse = res[0], res[5]
    return out if not return_attn_probs else (out, softmax_lse, None)


def flash_attn_varlen_func(
    q,
    k,
    v,
    cu_seqlens_q=None,
    cu_seqlens_k=None,  # only used for non-paged prefill
    max_seqlen_q=0,
    max_seqlen_k=0,
    dropout_p=0.0,
    seqused_k=None,
    q_v=None,
    softmax_scale=None,
    causal=False,
    window_size: Optional[List[int]] = (-1, -1),
    softcap=0.0,  # 0.0 means deactivated
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    block_table=None,
    return_softmax_lse=False,
    out=None,
    layout="bshd",
    scheduler_metadata=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    num_splits: int = 0,
    fa_version: int = DEFAULT_FA_VERSION,
    s_aux=None,
    cp_world_size=1,
    cp_rank=0,
    cp_tot_seqused_k=None,
):
    """Packed variable-length attention.  q: (total_q, nheads, 128); k, v: (total_k, nheads_k, 128);
    cu_seqlens_*: int32 (batch + 1).  FP8 e4m3 inputs take fp32 q/k/v_descale of one element or shape
    (batch, nheads_k) and return bf16.  softmax_lse is (nheads, total_q).
    With `block_table` (int32 (batch, max_blocks)) k and v are paged pools (num_blocks, page_size, nheads_k, 128) and
    `seqused_k` (int32 (batch,)) gives each sequence's number of keys; cu_seqlens_k is not used.  The kernel reads
    the pages directly (the reference gathers them into a contiguous copy first, flash_attn_interface.py:2350-2373)."""
    _no_backward(q, k, v)
    if block_table is not None and layout != "bshd":
        raise NotImplementedError("paged K/V layouts other than bshd (num_blocks, page, nheads_k, d) are outside the B200 hot path")
    if q_v is not None:
        raise NotImplementedError("q_v is outside the B200 hot path of this build")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    res = flash_attn_cuda.varlen_fwd(
        q, k, v, out, cu_seqlens_q, cu_seqlens_k, seqused_k, None, block_table, alibi_slopes, max_seqlen_q,
        max_seqlen_k, dropout_p, softmax_scale, False, causal, window_size[0], window_size[1], softcap, False,
        q_descale, k_descale, v_descale, None, s_aux)
    o, softmax_lse = res[0], res[5]
    if return_attn_probs:
        return o, softmax_lse, None
    return (o, softmax_lse) if return_softmax_lse else o


def flash_attn_with_kvcache(
    q,
    k_cache,
    v_cache,
    k=None,
    v=None,
    rotary_cos=None,
    rotary_sin=None,
    cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
    cache_batch_idx: Optional[torch.Tensor] = None,
    cache_leftpad: Optional[torch.Tensor] = None,
    block_table: Optional[torch.Tensor] = None,
    softmax_scale=None,
    causal=False,
    window_size=(-1, -1),  # -1 means infinite context window
    softcap=0.0,  # 0.0 means deactivated
    rotary_interleaved=True,
    alibi_slopes=None,
    num_splits=0,
    s_aux=None,
    return_softmax_lse=False,
    *,
    out=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
):
    """Decode over a paged KV cache.  q: (batch, 1, nheads, 128); k_cache, v_cache:
    (num_blocks, page_block_size, nheads_k, 128) with page_block_size 16, 32 or a multiple of 64;
    block_table: int32 (batch, max_num_blocks_per_seq); cache_seqlens: int or int32 (batch,).
    FP8 e4m3 q/k/v take keyword-only fp32 q/k/v_descale (one element or (batch, nheads_k)) and return bf16.
    Returns out, or (out, softmax_lse (batch, nheads, 1)) when return_softmax_lse=True."""
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    s_aux = maybe_contiguous(s_aux)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if cache_seqlens is not None and isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((q.shape[0],), cache_seqlens, dtype=torch.int32, device=k_cache.device)
        cache_seqlens = maybe_contiguous(cache_seqlens)
    cache_batch_idx = maybe_contiguous(cache_batch_idx)
    block_table = maybe_contiguous(block_table)
    if block_table is not None and softcap is not None and softcap > 0.0:
        raise ValueError("softcap is not supported by paged attention (flash_attn_with_kvcache)")
    out, softmax_lse = flash_attn_cuda.fwd_kvcache(
        q, k_cache, v_cache, k, v, cache_seqlens, rotary_cos, rotary_sin, cache_batch_idx, cache_leftpad, block_table,
        alibi_slopes, out, softmax_scale, causal, window_size[0], window_size[1], softcap, rotary_interleaved,
        num_splits, s_aux, q_descale, k_descale, v_descale)
    return (out, softmax_lse) if return_softmax_lse else out


def sparse_attn_func(
    q,
    k,
    v,
    block_count,
    block_offset,
    column_count,
    column_index,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    softcap=0.0,  # 0.0 means deactivated
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    *,
    return_softmax_lse=False,
    out=None,
    pv_threshold=50.0,
    enable_dynamic_skip=False,
    is_sla=False,
):
    """Block-sparse attention from per-(batch, head, q-block) lists.  block_count: int32 (batch, nheads, NUM_ROWS);
    block_offset: int32 (batch, nheads, NUM_ROWS, NNZ_S) ascending K ROW offsets of 64-row K tiles, with
    NUM_ROWS = ceil(seqlen / (64 if seqlen <= 2048 else 128)).  column_count must be all zero (no vertical part)."""
    _no_backward(q, k, v)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    out, softmax_lse = flash_attn_cuda.fwd_sparse(
        q, k, v, block_count, block_offset, column_count, column_index, out, alibi_slopes, dropout_p, softmax_scale,
        causal, softcap, return_attn_probs and dropout_p > 0, None, is_sla, pv_threshold, enable_dynamic_skip)
    return (out, softmax_lse) if return_softmax_lse else out
