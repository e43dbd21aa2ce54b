"""Block-map helpers for sparse_attn_func with the reference's names (flash_attn/utils/sparse_utils.py)."""
import flash_attn_2_cuda as flash_attn_cuda


def block_map_to_block_offset(block_map):
    """block_map (B, H, x, y) bool -> (block_offset (B, H, x, y) int32: absolute indices of the selected blocks in
    ascending order, then 10000000; block_count (B, H, x) int32).  As flash_attn/utils/sparse_utils.py:526-566 and
    its Triton version :78-145."""
    assert block_map.dim() == 4
    return flash_attn_cuda.block_map_to_offset(block_map, 1, 10000000)


block_map_to_block_offset_triton = block_map_to_block_offset
