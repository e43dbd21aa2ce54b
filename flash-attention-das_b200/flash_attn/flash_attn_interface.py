"""Public Python API of the attention hot path, signature-compatible with the reference's
flash_attn/flash_attn_interface.py (flash_attn_func :1646, flash_attn_varlen_func :2111,
flash_attn_with_kvcache :2478, sparse_attn_func :2778).

Forward only, head dimension 128 (fp16 / bf16 also 64, 192, 256, and 192 with 128 for v).  Options outside the hot
path (dropout, alibi, softcap, backward) raise NotImplementedError instead of silently taking another code path: there
is no Triton, eager or CPU fallback.
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


def _paged_as_bshd(k, v, layout):
    """A (num_blocks, page, nheads_k, d) view of paged pools given in the reference's layouts
    (flash_attn_interface.py:2223-2237): "bshd" / 2 as is, "bhsd" / 1 = (num_blocks, nheads_k, page, d) permuted,
    "custom" / 0 = K as bhsd and V stored as (num_blocks, nheads_k, d, page).  No copies: the kernels take strides."""
    if layout in ("bshd", 2):
        return k, v
    if layout in ("bhsd", 1):
        return k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)
    if layout in ("custom", 0):
        # V is (num_blocks, nheads_k, d, page): the view keeps the tokens as its contiguous axis, which the binding
        # module recognises (one-token decode only; the prefill kernels do not take this layout)
        return k.permute(0, 2, 1, 3), v.permute(0, 3, 1, 2)
    raise ValueError(f"unknown paged layout {layout!r}")


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
    With `block_table` (int32 (batch, max_blocks)) k and v are paged pools, (num_blocks, page_size, nheads_k, 128)
    for layout "bshd" or (num_blocks, nheads_k, page_size, 128) for "bhsd", and `seqused_k` (int32 (batch,)) gives
    each sequence's number of keys; cu_seqlens_k is not used.  The kernel reads the pages directly, through strides,
    whatever the layout (the reference gathers them into a contiguous copy first,
    flash_attn_interface.py:2350-2373).  Layout "custom": K as "bhsd" and V stored transposed,
    (num_blocks, nheads_k, 128, page_size), fp16 / bf16 with pages of a multiple of 64 tokens; a V tile is then fed to
    the P V product as the K-major operand."""
    _no_backward(q, k, v)
    if window_size is None:
        window_size = (-1, -1)
    if block_table is not None:
        k, v = _paged_as_bshd(k, v, layout)
        # One or a few query tokens per sequence, the same number for all (decode, speculative decoding): the decode
        # kernel, as in the reference (its direct paged path, flash_attn_interface.py:2256, 2305-2348).  Rows of the
        # kernel's tile: tokens x heads per kv head <= 16.
        bs = block_table.shape[0]
        group = q.shape[1] // k.shape[2]
        few_tokens = max_seqlen_q >= 1 and max_seqlen_q * bs == q.shape[0] and max_seqlen_q * group <= 16
        if few_tokens and (max_seqlen_q > 1 or layout in ("custom", 0)) and q_v is None and dropout_p == 0.0:
            if softmax_scale is None:
                softmax_scale = q.shape[-1] ** (-0.5)
            q = maybe_contiguous(q)
            sq = max_seqlen_q
            o, lse = flash_attn_cuda.fwd_kvcache(
                q.view(bs, sq, q.shape[1], q.shape[2]), k, v, None, None, seqused_k, None, None, None, None, block_table,
                alibi_slopes, None if out is None else out.view(bs, sq, q.shape[1], q.shape[2]), softmax_scale, causal,
                window_size[0], window_size[1], softcap, True, num_splits, s_aux, q_descale, k_descale, v_descale,
                max_seqlen_k)
            o = o.view(bs * sq, q.shape[1], q.shape[2])
            lse = lse.permute(1, 0, 2).reshape(q.shape[1], bs * sq)      # (b, h, sq) -> (h, total_q)
            if return_attn_probs:
                return o, lse, None
            return (o, lse) if return_softmax_lse else o
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


def vllm_flash_attn_with_kvcache(
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
    window_size=(-1, -1),
    softcap=0.0,
    rotary_interleaved=True,
    alibi_slopes=None,
    num_splits=0,
    s_aux=None,
    return_softmax_lse=False,
    *,
    q_scale=None,
    k_scale=None,
    v_scale=None,
    kv_cache_dtype="auto",
    out=None,
    max_seqlen_k=0,
    layout=0,
):
    """The reference's second paged-decode entry (flash_attn_interface.py:2633-2775): like flash_attn_with_kvcache
    with fp32 q/k/v_scale (the e4m3 descales), an upper bound ``max_seqlen_k`` on cache_seqlens (0 = none) and the
    pool layout as an integer: 2 = (num_blocks, page, nheads_k, d), 1 = (num_blocks, nheads_k, page, d), 0 (the
    reference's default) = K as 1 and V as (num_blocks, nheads_k, d, page), which is taken for one query token per
    sequence in fp16 / bf16 with pages of 64 * n.  Like the reference it returns only ``out`` and does not append k / v."""
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    if k is not None or v is not None or rotary_cos is not None or rotary_sin is not None:
        raise NotImplementedError("vllm_flash_attn_with_kvcache does not append k/v (as in the reference); use "
                                  "flash_attn_with_kvcache")
    if str(kv_cache_dtype).startswith("fp8"):
        # an e4m3 cache under 16-bit (or e4m3) queries, or an e5m2 cache ("fp8_e5m2") under 16-bit queries; k_scale /
        # v_scale are its descales.  Raw-byte caches are viewed.
        if k_cache.dtype == torch.uint8:
            f8 = torch.float8_e5m2 if "e5m2" in str(kv_cache_dtype) else torch.float8_e4m3fn
            k_cache, v_cache = k_cache.view(f8), v_cache.view(f8)
    elif kv_cache_dtype not in ("auto", ""):
        raise NotImplementedError(f"kv_cache_dtype {kv_cache_dtype!r} is outside the B200 hot path")
    if softcap is not None and softcap > 0.0:
        raise ValueError("softcap is not supported by paged attention (vllm_flash_attn_with_kvcache)")
    q = maybe_contiguous(q)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if cache_seqlens is not None and isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((q.shape[0],), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    k_cache, v_cache = _paged_as_bshd(k_cache, v_cache, layout)
    out, _ = flash_attn_cuda.fwd_kvcache(
        q, k_cache, v_cache, None, None, cache_seqlens, None, None, maybe_contiguous(cache_batch_idx), cache_leftpad,
        maybe_contiguous(block_table), alibi_slopes, out, softmax_scale, causal, window_size[0], window_size[1], 0.0,
        rotary_interleaved, num_splits, s_aux, q_scale if q.dtype == torch.float8_e4m3fn else None, k_scale, v_scale,
        max_seqlen_k)
    return out


def vllm_flash_attn_varlen_func(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k=None, seqused_k=None,
                                q_v=None, dropout_p=0.0, softmax_scale=None, causal=False,
                                window_size: Optional[List[int]] = None, softcap=0.0, alibi_slopes=None,
                                deterministic=False, return_attn_probs=False, block_table=None,
                                return_softmax_lse=False, out=None, is_prefix_cache=True, scheduler_metadata=None,
                                q_descale=None, k_descale=None, v_descale=None, kv_cache_dtype="auto",
                                fa_version: int = DEFAULT_FA_VERSION, s_aux=None):
    """Argument order of the reference's vLLM entry (flash_attn_interface.py:2410-2475), which forwards to
    flash_attn_varlen_func with layout "custom" (K (num_blocks, nheads_k, page, d), V (num_blocks, nheads_k, d, page))."""
    return flash_attn_varlen_func(
        q, k, v, max_seqlen_q=max_seqlen_q, cu_seqlens_q=cu_seqlens_q, max_seqlen_k=max_seqlen_k,
        cu_seqlens_k=cu_seqlens_k, seqused_k=seqused_k, q_v=q_v, dropout_p=dropout_p, softmax_scale=softmax_scale,
        causal=causal, window_size=window_size, softcap=softcap, alibi_slopes=alibi_slopes,
        deterministic=deterministic, return_attn_probs=return_attn_probs, block_table=block_table,
        return_softmax_lse=return_softmax_lse, out=out, layout="custom", scheduler_metadata=scheduler_metadata,
        q_descale=q_descale, k_descale=k_descale, v_descale=v_descale, num_splits=0, fa_version=fa_version,
        s_aux=s_aux)


hg_flash_attn_varlen_func = flash_attn_varlen_func
varlen_fwd_unified = flash_attn_varlen_func


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
