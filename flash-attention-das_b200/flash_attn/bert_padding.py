"""Padding removal around the varlen attention call, with the reference's names and return values
(flash_attn/bert_padding.py:8-67 index_first_axis / index_put_first_axis, :98-122 unpad_input, :199-214 pad_input).
Forward only; the work runs in the library's glue kernels (mask scan, row gather, row scatter)."""
import flash_attn_2_cuda as flash_attn_cuda


def index_first_axis(input, indices):
    """input (n, ...), indices int64 (z) -> input[indices]."""
    assert input.ndim >= 2
    return flash_attn_cuda.gather_rows(input, indices)


def index_put_first_axis(values, indices, first_axis_dim):
    """zeros (first_axis_dim, ...) with rows ``indices`` set to ``values``."""
    assert indices.ndim == 1
    assert values.ndim >= 2
    return flash_attn_cuda.scatter_rows(values, indices, first_axis_dim)


def unpad_input(hidden_states, attention_mask):
    """hidden_states (batch, seqlen, ...), attention_mask (batch, seqlen) bool / int (nonzero = valid) ->
    (hidden_states (total_nnz, ...), indices (total_nnz) int64, cu_seqlens (batch + 1) int32, max_seqlen_in_batch int)."""
    _, cu_seqlens, indices, max_seqlen_in_batch = flash_attn_cuda.unpad_plan(attention_mask)
    flat = hidden_states.reshape(hidden_states.shape[0] * hidden_states.shape[1], *hidden_states.shape[2:])
    return index_first_axis(flat, indices), indices, cu_seqlens, max_seqlen_in_batch


def pad_input(hidden_states, indices, batch, seqlen):
    """hidden_states (total_nnz, ...), indices (total_nnz) -> (batch, seqlen, ...) with zeros at the padded positions."""
    output = index_put_first_axis(hidden_states, indices, batch * seqlen)
    return output.reshape(batch, seqlen, *hidden_states.shape[1:])
