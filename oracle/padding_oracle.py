"""CPU restatement of the reference's padding-removal helpers and block-map conversion (TEST INFRASTRUCTURE ONLY).

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference's own flash_attn/bert_padding.py (plain
PyTorch) and checks ``unpad_input_ref`` / ``pad_input_ref`` against it bit for bit on seeded masks; the block-map
conversion is pinned by the worked example in the reference's docstring (flash_attn/utils/sparse_utils.py:537-541).
"""
import torch


def unpad_input_ref(hidden_states, attention_mask):
    """Follows unpad_input (flash_attn/bert_padding.py:98-122): lengths by row sum, flat indices by nonzero,
    cu_seqlens by cumsum with a leading zero, rows gathered from the flattened (batch * seqlen, ...) input."""
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    max_seqlen = int(seqlens.max().item()) if seqlens.numel() else 0
    cu_seqlens = torch.nn.functional.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape(hidden_states.shape[0] * hidden_states.shape[1], *hidden_states.shape[2:])
    return flat[indices], indices, cu_seqlens, max_seqlen


def pad_input_ref(hidden_states, indices, batch, seqlen):
    """Follows pad_input / IndexPutFirstAxis.forward (flash_attn/bert_padding.py:40-52, 199-214)."""
    out = torch.zeros(batch * seqlen, *hidden_states.shape[1:], dtype=hidden_states.dtype)
    out[indices] = hidden_states
    return out.reshape(batch, seqlen, *hidden_states.shape[1:])


def block_map_to_block_offset_ref(block_map, scale=1, fill=10000000):
    """Follows block_map_to_block_offset (flash_attn/utils/sparse_utils.py:526-566): per row the ascending positions of
    the set entries, then ``fill``; and the number of set entries."""
    k = block_map.shape[-1]
    flat = block_map.reshape(-1, k).bool()
    off = torch.full(flat.shape, fill, dtype=torch.int32)
    cnt = flat.sum(dim=-1).to(torch.int32)
    for r in range(flat.shape[0]):
        pos = torch.nonzero(flat[r]).flatten().to(torch.int32) * scale
        off[r, :pos.numel()] = pos
    return off.reshape(block_map.shape), cnt.reshape(block_map.shape[:-1])
