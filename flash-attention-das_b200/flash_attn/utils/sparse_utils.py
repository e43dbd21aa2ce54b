"""Block-map helpers for sparse_attn_func with the reference's names (flash_attn/utils/sparse_utils.py)."""
import torch

import flash_attn_2_cuda as flash_attn_cuda


def block_map_to_block_offset(block_map):
    """block_map (B, H, x, y) bool -> (block_offset (B, H, x, y) int32: absolute indices of the selected blocks in
    ascending order, then 10000000; block_count (B, H, x) int32).  As flash_attn/utils/sparse_utils.py:526-566 and
    its Triton version :78-145."""
    assert block_map.dim() == 4
    return flash_attn_cuda.block_map_to_offset(block_map, 1, 10000000)


block_map_to_block_offset_triton = block_map_to_block_offset


def hyperparameter_check(hyper, H, device):
    """A float, or a tensor of 0 / 1 dimensions, -> fp32 (H) on ``device`` (sparse_utils.py:41-53)."""
    if isinstance(hyper, (float, int)):
        return torch.full((H,), float(hyper), device=device, dtype=torch.float32)
    if isinstance(hyper, torch.Tensor):
        assert hyper.dim() <= 1, "Hyperparameter tensor must be 1D"
        if hyper.dim() == 0:
            hyper = hyper.reshape(1).expand(H)
        assert hyper.numel() == H, f"Hyperparameter tensor must have {H} elements, but has {hyper.numel()}"
        return hyper.to(device=device, dtype=torch.float32).contiguous()
    raise ValueError("Hyperparameter must be a float or a tensor")


def get_pool_sim_triton_simmean(x, block_size, simthreshd1):
    """x (B, H, N, D) -> (pooled (B, H, nblock, D), sim_blocks (B, H, nblock) bool): sparse_utils.py:300-310."""
    return flash_attn_cuda.block_pool(x if x.stride(-1) == 1 else x.contiguous(), block_size, simthreshd1)


def get_block_map_meansim(q, k, is_causal=False, BLKQ=128, BLKK=64, simthreshd1=0.1, cdfthreshd=0.9, topk=None,
                          is_sparse=True, return_lut=False, return_block_offset=False, attention_sink=False):
    """The key blocks each query block attends to, chosen from mean-pooled q and k (sparse_utils.py:376-441): q, k
    (B, H, N, D) fp16 / bf16.  Returns the (B, H, nq, nk) bool map, or with ``return_block_offset`` the
    (block_offset, block_count) lists.  Two launches (three with the lists); the scores, softmax and cumulative sums
    are fp32, where the reference keeps them in the input's 16-bit type."""
    assert (cdfthreshd is None and topk is not None) or (cdfthreshd is not None and topk is None), \
        "Only one of cdfthreshd and topk can be set."
    assert not (return_lut and return_block_offset), "Only one of return_lut and return_block_offset can be True."
    if return_lut:
        raise NotImplementedError("the relative-offset LUT format belongs to another kernel family; use "
                                  "return_block_offset for sparse_attn_func")
    H = q.size(1)
    th1 = hyperparameter_check(simthreshd1, H, q.device)
    cdf = hyperparameter_check(cdfthreshd, H, q.device) if cdfthreshd is not None else None
    tk = hyperparameter_check(topk, H, q.device) if topk is not None else None
    pooled_q, sim_q = get_pool_sim_triton_simmean(q, BLKQ, th1)
    pooled_k, sim_k = get_pool_sim_triton_simmean(k, BLKK, th1)
    final_map = flash_attn_cuda.block_select(pooled_q, pooled_k, sim_q, sim_k, BLKQ, BLKK, q.shape[-1] ** -0.5, cdf, tk,
                                             is_causal, attention_sink)
    if return_block_offset:
        return block_map_to_block_offset(final_map)
    return final_map
