"""``flash_attn_2_cuda`` for B200: the binding module the reference's Python API imports
(``import flash_attn_2_cuda as flash_attn_cuda``, flash_attn/flash_attn_interface.py:10), re-implemented as a
thin ctypes layer over the C ABI of ``libfa_b200.so`` (include/fa_b200.h).

It keeps the reference binding's function names, positional argument order and return arity
(csrc/flash_attn_cutlass/flash_api.cpp:2993-3037):

    fwd          -> 9 tensors  (flash_api.cpp:951-1215)
    varlen_fwd   -> 8 tensors  (flash_api.cpp:1216-1685)
    fwd_kvcache  -> [out, softmax_lse]  (flash_api.cpp:2530-2577)
    fwd_sparse   -> [out, softmax_lse]  (flash_api_sparse.cpp:170-338)

PyTorch is used for what the reference binding used ATen for: output / scratch allocation on the input's
device and the current stream.  All compute happens in the library's sm_100a kernels; there is no CPU or
eager fallback — if the shared library is missing the import fails.
"""
import ctypes
import os
from typing import Optional, Sequence, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("FA_B200_LIB", os.path.join(_HERE, "libfa_b200.so"))
if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} not found: build it with `python {os.path.join(_HERE, 'build.py')}` "
        "(there is no fallback implementation)")
_lib = ctypes.CDLL(_LIB_PATH)

F16, BF16, E4M3 = 0, 1, 2
_DT = {torch.float16: F16, torch.bfloat16: BF16, torch.float8_e4m3fn: E4M3}

_c_i64, _c_i32, _c_f32, _c_vp = ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p


class _SizedStruct(ctypes.Structure):
    """Parameter structs start with ``struct_size``: the library refuses a struct whose size is not its own."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.struct_size = ctypes.sizeof(self)


class FwdParams(_SizedStruct):
    """struct fa_b200_fwd_params (include/fa_b200.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("q", _c_vp), ("k", _c_vp), ("v", _c_vp), ("out", _c_vp), ("softmax_lse", _c_vp),
        ("q_batch_stride", _c_i64), ("q_row_stride", _c_i64), ("q_head_stride", _c_i64),
        ("k_batch_stride", _c_i64), ("k_row_stride", _c_i64), ("k_head_stride", _c_i64),
        ("v_batch_stride", _c_i64), ("v_row_stride", _c_i64), ("v_head_stride", _c_i64),
        ("o_batch_stride", _c_i64), ("o_row_stride", _c_i64), ("o_head_stride", _c_i64),
        ("b", _c_i32), ("seqlen_q", _c_i32), ("seqlen_k", _c_i32), ("h", _c_i32), ("h_k", _c_i32), ("d", _c_i32),
        ("total_q", _c_i64), ("total_k", _c_i64),
        ("cu_seqlens_q", _c_vp), ("cu_seqlens_k", _c_vp),
        ("softmax_scale", _c_f32), ("is_causal", _c_i32), ("dtype", _c_i32), ("out_dtype", _c_i32),
        ("q_descale", _c_vp), ("k_descale", _c_vp), ("v_descale", _c_vp),
        ("q_descale_batch_stride", _c_i64), ("q_descale_head_stride", _c_i64),
        ("k_descale_batch_stride", _c_i64), ("k_descale_head_stride", _c_i64),
        ("v_descale_batch_stride", _c_i64), ("v_descale_head_stride", _c_i64),
        ("block_count", _c_vp), ("block_offset", _c_vp),
        ("num_q_blocks", _c_i32), ("nnz_s", _c_i32), ("block_m", _c_i32),
        ("profile_start_event", _c_vp), ("profile_stop_event", _c_vp),
        ("block_table", _c_vp), ("block_table_batch_stride", _c_i64), ("seqused_k", _c_vp),
        ("page_size", _c_i32), ("num_blocks", _c_i32),
        ("s_aux", _c_vp), ("s_aux_dtype", _c_i32),
        ("has_window", _c_i32), ("window_left", _c_i32), ("window_right", _c_i32),
        ("column_count", _c_vp), ("d_v", _c_i32), ("v_transposed", _c_i32), ("work_counter", _c_vp),
        ("kernel_choice", _c_i32), ("max_blocks_per_seq", _c_i32),
    ]


class DecodeParams(_SizedStruct):
    """struct fa_b200_decode_params (include/fa_b200.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("q", _c_vp), ("k_cache", _c_vp), ("v_cache", _c_vp), ("out", _c_vp), ("softmax_lse", _c_vp),
        ("q_batch_stride", _c_i64), ("q_head_stride", _c_i64),
        ("o_batch_stride", _c_i64), ("o_head_stride", _c_i64),
        ("k_block_stride", _c_i64), ("k_row_stride", _c_i64), ("k_head_stride", _c_i64),
        ("v_block_stride", _c_i64), ("v_row_stride", _c_i64), ("v_head_stride", _c_i64),
        ("block_table", _c_vp), ("block_table_batch_stride", _c_i64), ("cache_seqlens", _c_vp),
        ("b", _c_i32), ("h", _c_i32), ("h_k", _c_i32), ("d", _c_i32),
        ("num_blocks", _c_i32), ("page_size", _c_i32), ("max_blocks_per_seq", _c_i32),
        ("softmax_scale", _c_f32), ("dtype", _c_i32), ("out_dtype", _c_i32),
        ("q_descale", _c_vp), ("k_descale", _c_vp), ("v_descale", _c_vp),
        ("q_descale_batch_stride", _c_i64), ("q_descale_head_stride", _c_i64),
        ("k_descale_batch_stride", _c_i64), ("k_descale_head_stride", _c_i64),
        ("v_descale_batch_stride", _c_i64), ("v_descale_head_stride", _c_i64),
        ("partition_tokens", _c_i32), ("max_seqlen_k", _c_i32),
        ("workspace", _c_vp), ("workspace_bytes", ctypes.c_size_t),
        ("o_partial_out", _c_vp), ("lse_partial_out", _c_vp),
        ("profile_start_event", _c_vp), ("profile_stop_event", _c_vp),
        ("s_aux", _c_vp), ("s_aux_dtype", _c_i32),
        ("has_window", _c_i32), ("window_left", _c_i32),
        ("v_transposed", _c_i32),
        ("seqlen_q", _c_i32), ("is_causal", _c_i32),
        ("q_row_stride", _c_i64), ("o_row_stride", _c_i64),
        ("kv_e4m3", _c_i32), ("kv_e5m2", _c_i32),
        ("tickets", _c_vp),
    ]


class ExchangeParams(_SizedStruct):
    """struct fa_b200_exchange_params (include/fa_b200.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("world", _c_i32), ("rank", _c_i32),
        ("rows", _c_i32), ("h", _c_i32), ("seqlen_q", _c_i32), ("d", _c_i32),
        ("o_local", _c_vp), ("lse_local", _c_vp),
        ("peers", _c_vp * 16),
        ("epoch", ctypes.c_uint32), ("do_push", _c_i32), ("do_wait", _c_i32),
        ("out", _c_vp), ("lse", _c_vp),
        ("out_batch_stride", _c_i64), ("out_head_stride", _c_i64), ("out_tok_stride", _c_i64),
        ("out_dtype", _c_i32), ("s_aux", _c_vp), ("s_aux_dtype", _c_i32),
    ]


class CombineParams(_SizedStruct):
    """struct fa_b200_combine_params (include/fa_b200.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("o_partial", _c_vp), ("lse_partial", _c_vp), ("out", _c_vp), ("lse", _c_vp),
        ("out_row_stride", _c_i64),
        ("num_parts", _c_i32), ("rows", _c_i32), ("d", _c_i32), ("h", _c_i32),
        ("parts_per_row", _c_vp), ("out_dtype", _c_i32), ("out_scale", _c_f32),
        ("s_aux", _c_vp), ("s_aux_dtype", _c_i32),
        ("o_part_stride", _c_i64), ("lse_part_stride", _c_i64),
    ]


class KvAppendParams(_SizedStruct):
    """struct fa_b200_kv_append_params (include/fa_b200.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("k_new", _c_vp), ("v_new", _c_vp),
        ("k_new_batch_stride", _c_i64), ("k_new_row_stride", _c_i64), ("k_new_head_stride", _c_i64),
        ("v_new_batch_stride", _c_i64), ("v_new_row_stride", _c_i64), ("v_new_head_stride", _c_i64),
        ("k_cache", _c_vp), ("v_cache", _c_vp),
        ("k_block_stride", _c_i64), ("k_row_stride", _c_i64), ("k_head_stride", _c_i64),
        ("v_block_stride", _c_i64), ("v_row_stride", _c_i64), ("v_head_stride", _c_i64),
        ("block_table", _c_vp), ("block_table_batch_stride", _c_i64),
        ("seqlens_k", _c_vp), ("seqlens_out", _c_vp),
        ("q", _c_vp), ("q_out", _c_vp),
        ("q_batch_stride", _c_i64), ("q_row_stride", _c_i64), ("q_head_stride", _c_i64),
        ("q_out_batch_stride", _c_i64), ("q_out_row_stride", _c_i64), ("q_out_head_stride", _c_i64),
        ("rotary_cos", _c_vp), ("rotary_sin", _c_vp),
        ("rotary_dim", _c_i32), ("seqlen_ro", _c_i32), ("is_rotary_interleaved", _c_i32),
        ("rotate_q_per_token", _c_i32),
        ("b", _c_i32), ("seqlen_q", _c_i32), ("seqlen_new", _c_i32), ("h", _c_i32), ("h_k", _c_i32), ("d", _c_i32),
        ("page_size", _c_i32), ("num_blocks", _c_i32), ("max_blocks_per_seq", _c_i32),
        ("dtype", _c_i32),
    ]


_lib.fa_b200_fwd.argtypes = [ctypes.POINTER(FwdParams), _c_vp]
_lib.fa_b200_fwd.restype = ctypes.c_int
_lib.fa_b200_fwd_sparse.argtypes = [ctypes.POINTER(FwdParams), _c_vp]
_lib.fa_b200_fwd_sparse.restype = ctypes.c_int
_lib.fa_b200_decode_paged.argtypes = [ctypes.POINTER(DecodeParams), _c_vp]
_lib.fa_b200_decode_paged.restype = ctypes.c_int
_lib.fa_b200_decode_paged_static.argtypes = [ctypes.POINTER(DecodeParams), _c_vp]
_lib.fa_b200_decode_paged_static.restype = ctypes.c_int
_lib.fa_b200_decode_workspace_bytes.argtypes = [ctypes.POINTER(DecodeParams)]
_lib.fa_b200_decode_workspace_bytes.restype = ctypes.c_size_t
_lib.fa_b200_decode_partition_tokens.argtypes = [ctypes.POINTER(DecodeParams)]
_lib.fa_b200_decode_partition_tokens.restype = ctypes.c_int32
_lib.fa_b200_kv_append.argtypes = [ctypes.POINTER(KvAppendParams), _c_vp]
_lib.fa_b200_kv_append.restype = ctypes.c_int
_lib.fa_b200_combine.argtypes = [ctypes.POINTER(CombineParams), _c_vp]
_lib.fa_b200_combine.restype = ctypes.c_int
_lib.fa_b200_unpad_plan.argtypes = [_c_vp, _c_i32, _c_i32, _c_i32, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp]
_lib.fa_b200_unpad_plan.restype = ctypes.c_int
_lib.fa_b200_gather_rows.argtypes = [_c_vp, _c_vp, _c_vp, _c_i64, _c_i64, _c_i64, _c_vp]
_lib.fa_b200_gather_rows.restype = ctypes.c_int
_lib.fa_b200_scatter_rows.argtypes = [_c_vp, _c_vp, _c_vp, _c_i64, _c_i64, _c_i64, _c_vp]
_lib.fa_b200_scatter_rows.restype = ctypes.c_int
_lib.fa_b200_block_map_to_offset.argtypes = [_c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_vp]
_lib.fa_b200_block_map_to_offset.restype = ctypes.c_int
_lib.fa_b200_block_pool.argtypes = [_c_vp, _c_i32, _c_i64, _c_i64, _c_i64] + [_c_i32] * 5 + [_c_vp, _c_vp, _c_vp, _c_vp]
_lib.fa_b200_block_pool.restype = ctypes.c_int
_lib.fa_b200_block_select.argtypes = ([_c_vp] * 4 + [_c_i32] * 8 + [_c_f32, _c_vp, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp])
_lib.fa_b200_block_select.restype = ctypes.c_int
_lib.fa_b200_kv_cache_attention.argtypes = ([_c_vp, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp] + [_c_i32] * 9 +
                                            [_c_vp, ctypes.c_size_t, _c_vp])
_lib.fa_b200_kv_cache_attention.restype = ctypes.c_int
_lib.fa_b200_kv_cache_attention_workspace_bytes.argtypes = [_c_i32] * 6
_lib.fa_b200_kv_cache_attention_workspace_bytes.restype = ctypes.c_size_t
_lib.fa_b200_status_string.argtypes = [ctypes.c_int]
_lib.fa_b200_status_string.restype = ctypes.c_char_p
_lib.fa_b200_last_cuda_error.restype = ctypes.c_char_p
_lib.fa_b200_device_status.restype = ctypes.c_int
_lib.fa_b200_abi_version.restype = ctypes.c_int
_lib.fa_b200_launch_count.restype = ctypes.c_uint64
_lib.fa_b200_exchange_bytes.argtypes = [_c_i32, _c_i32, _c_i32]
_lib.fa_b200_exchange_bytes.restype = ctypes.c_size_t
_lib.fa_b200_exchange_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
_lib.fa_b200_exchange_alloc.restype = ctypes.c_int
_lib.fa_b200_exchange_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
_lib.fa_b200_exchange_open.restype = ctypes.c_int
_lib.fa_b200_exchange_close.argtypes = [_c_vp]
_lib.fa_b200_exchange_close.restype = ctypes.c_int
_lib.fa_b200_exchange_free.argtypes = [_c_vp]
_lib.fa_b200_exchange_free.restype = ctypes.c_int
_lib.fa_b200_exchange_combine.argtypes = [ctypes.POINTER(ExchangeParams), _c_vp]
_lib.fa_b200_exchange_combine.restype = ctypes.c_int
_lib.fa_b200_read_stream.argtypes = [_c_vp, _c_i64, _c_vp, _c_vp]
_lib.fa_b200_read_stream.restype = ctypes.c_int
_lib.fa_b200_set_print_param.argtypes = [ctypes.c_int]
_lib.fa_b200_set_print_param.restype = None
_lib.fa_b200_last_launch_info.restype = ctypes.c_char_p


def lib():
    """The loaded ctypes handle (tests call the C ABI through it)."""
    return _lib


_profile_events = None


def set_profile_events(start: Optional["torch.cuda.Event"], stop: Optional["torch.cuda.Event"]):
    """Benchmark hook: while set, every attention call records these two (already created) CUDA events
    right before and right after its main kernel, so the dominant kernel can be timed alone."""
    global _profile_events
    _profile_events = None if start is None else (start, stop)


def _own_work_counter(p, device):
    """Under stream capture every captured prefill call gets a work counter of its own (graph-private memory), so that a
    replay cannot meet another launch on the library's shared counters; kept alive by the returned tensor."""
    if torch.cuda.is_current_stream_capturing():
        c = torch.empty(1, dtype=torch.int32, device=device)
        p.work_counter = c.data_ptr()
        return c
    return None


def _own_tickets(p, device, pairs: int):
    """Under stream capture a split decode call gets ticket counters of its own (graph-private memory, zeroed by a
    memset node of the graph), so that the captured call is a single launch too and a replay cannot meet another launch
    on the library's per-stream counters; kept alive by the returned tensor."""
    if torch.cuda.is_current_stream_capturing():
        t = torch.zeros(pairs, dtype=torch.int32, device=device)
        p.tickets = t.data_ptr()
        return t
    return None


def _apply_profile_events(p):
    if _profile_events is not None:
        p.profile_start_event = _profile_events[0].cuda_event
        p.profile_stop_event = _profile_events[1].cuda_event


def launch_count() -> int:
    return int(_lib.fa_b200_launch_count())


def read_stream(buf: torch.Tensor, sink: torch.Tensor) -> None:
    """One read-only pass over ``buf`` on the current stream (fa_b200_read_stream): a measurement aid that gives, timed
    with events, the bandwidth of a pure read stream on this GPU.  ``sink``: one int32 / uint32 element on the device."""
    _require(buf.is_cuda and buf.is_contiguous() and sink.is_cuda and sink.numel() >= 1, "read_stream: contiguous CUDA tensors")
    with _on_device(buf.device):
        _check(_lib.fa_b200_read_stream(buf.data_ptr(), buf.numel() * buf.element_size(), sink.data_ptr(), _stream(buf)),
               "read_stream")


def set_print_param(on: Optional[bool]):
    """Print one line per attention call with the kernel, grid and tiling the library picked (None: back to the
    FA_B200_PRINT_PARAM environment variable, which the library reads once when it is loaded)."""
    _lib.fa_b200_set_print_param(-1 if on is None else int(bool(on)))


def last_launch_info() -> str:
    """The line describing this thread's last attention call (kernel, grid, tiling), whether or not printing is on."""
    return _lib.fa_b200_last_launch_info().decode()


# The library reads its environment switches once, when it is loaded.  This module looks at the same two variables on
# every call and passes them through the struct fields, so that a process may change them while it runs.
_KERNEL_CHOICE = {"single": 1, "pair": 2, "dense": 3}


def _env_partition() -> int:
    v = os.environ.get("FA_B200_DECODE_PARTITION")
    return int(v) if v else 0


def _env_kernel() -> int:
    return _KERNEL_CHOICE.get(os.environ.get("FA_B200_PREFILL_KERNEL", ""), 0)


def device_status() -> int:
    return int(_lib.fa_b200_device_status())


def _check(status: int, what: str):
    if status != 0:
        msg = _lib.fa_b200_status_string(status).decode()
        if status == 10:
            msg += " (" + _lib.fa_b200_last_cuda_error().decode() + ")"
        raise RuntimeError(f"{what}: {msg}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_handle(device) -> int:
    """The current stream of `device` as an integer handle (without building a torch.cuda.Stream object per call)."""
    if _raw_stream is not None:
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(_stream_handle(t.device))


class _on_device:
    """``with _on_device(dev):`` makes `dev` the current CUDA device for the call; costs nothing when it already is."""
    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index

    def __enter__(self):
        self.prev = -1
        if self.idx is not None:
            cur = torch.cuda.current_device()
            if cur != self.idx:
                self.prev = cur
                torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _require(cond: bool, msg: str):
    if not cond:
        raise RuntimeError(msg)


def _unsupported(cond: bool, what: str):
    if cond:
        raise NotImplementedError(f"{what} is outside the B200 hot path of this build")


def _is_fp8_kv(q, k) -> bool:
    """16-bit queries over an e4m3 or e5m2 cache (the reference's kv_cache_dtype = "fp8" / "fp8_e5m2" modes)."""
    return q.dtype in (torch.float16, torch.bfloat16) and k.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)


def _check_qkv(q, k, v, v_transposed=False, allow_fp8_kv=False, allow_dv=False):
    _require(q.dtype in _DT, "FlashAttention only support fp16, bf16 and fp8 e4m3 data type")
    if not (allow_fp8_kv and _is_fp8_kv(q, k)):
        _require(k.dtype == q.dtype, "query and key must have the same dtype")
    _require(v.dtype == k.dtype, "key and value must have the same dtype")
    _require(q.is_cuda and k.is_cuda and v.is_cuda, "Input tensor must be on CUDA device")
    for t in (q, k) if v_transposed else (q, k, v):
        _require(t.stride(-1) == 1, "Input tensor must have contiguous last dimension")
    _require(q.shape[-1] in (64, 128, 192, 256) and k.shape[-1] == q.shape[-1] and
             (v.shape[-1] == q.shape[-1] or (allow_dv and q.shape[-1] == 192 and v.shape[-1] == 128)),
             "head dimension must be 128 (or 64, 192, 256, or 192 with 128 for v, with fp16 / bf16 tensors in the plain "
             "layouts)")


def _descale(params, name, t: Optional[torch.Tensor], batch: int, h_k: int):
    """fp32 descale of numel 1 (per tensor) or shape (batch, h_k) -> pointer + strides."""
    if t is None:
        return
    _require(t.dtype == torch.float32 and t.is_cuda, f"{name} must be a float32 CUDA tensor")
    setattr(params, name, t.data_ptr())
    if t.numel() == 1:
        bs = hs = 0
    else:
        _require(t.dim() == 2 and t.shape[0] == batch and t.shape[1] == h_k,
                 f"{name} must have one element or shape (batch, nheads_k)")
        bs, hs = t.stride(0), t.stride(1)
    setattr(params, name + "_batch_stride", bs)
    setattr(params, name + "_head_stride", hs)


def _set_paged(p, kcache, vcache, block_table, seqused_k, batch):
    """K/V given as paged pools (num_blocks, page, h_k, d) + int32 block_table (batch, max_blocks) + int32
    seqused_k (batch)."""
    _require(block_table.dtype == torch.int32 and block_table.is_cuda, "block_table must have dtype torch.int32")
    _require(block_table.stride(-1) == 1, "block_table must have contiguous last dimension")
    _require(block_table.shape[0] == batch, "block_table batch mismatch")
    _require(seqused_k is not None, "seqused_k / cache_seqlens is required with block_table")
    _require(seqused_k.dtype == torch.int32 and seqused_k.is_contiguous() and seqused_k.numel() == batch,
             "seqused_k must be a contiguous int32 tensor of shape (batch,)")
    _require(kcache.dim() == 4 and kcache.shape[:3] == vcache.shape[:3], "paged k/v must be (num_blocks, page_size, nheads_k, d)")
    p.k, p.v = kcache.data_ptr(), vcache.data_ptr()
    p.k_batch_stride, p.k_row_stride, p.k_head_stride = kcache.stride(0), kcache.stride(1), kcache.stride(2)
    if _is_transposed_v(vcache):
        # (num_blocks, page, h_k, d) view of a pool stored as (num_blocks, h_k, d, page): the tokens are the contiguous axis
        p.v_transposed = 1
        p.v_batch_stride, p.v_head_stride, p.v_row_stride = vcache.stride(0), vcache.stride(2), vcache.stride(3)
    else:
        p.v_batch_stride, p.v_row_stride, p.v_head_stride = vcache.stride(0), vcache.stride(1), vcache.stride(2)
    p.block_table, p.block_table_batch_stride = block_table.data_ptr(), block_table.stride(0)
    p.seqused_k = seqused_k.data_ptr()
    p.page_size, p.num_blocks = kcache.shape[1], kcache.shape[0]
    p.max_blocks_per_seq = block_table.shape[1]


def _set_sinks(p, s_aux: Optional[torch.Tensor], h: int):
    """Attention sinks: one logit per query head, fp16 / bf16 (the reference asks for the dtype of q) or fp32."""
    if s_aux is None:
        return
    _require(s_aux.is_cuda and s_aux.dim() == 1 and s_aux.numel() == h, "s_aux must have shape (nheads,)")
    _require(s_aux.dtype in (torch.float16, torch.bfloat16, torch.float32), "s_aux must be fp16, bf16 or fp32")
    _require(s_aux.is_contiguous(), "s_aux must be contiguous")
    p.s_aux = s_aux.data_ptr()
    p.s_aux_dtype = 3 if s_aux.dtype == torch.float32 else _DT[s_aux.dtype]


def _set_window(p, left: int, right: int):
    """Sliding window (left, right), -1 = open side; the right side is dropped for the decode struct."""
    if left >= 0 or right >= 0:
        p.has_window = 1
        p.window_left = left
        if hasattr(p, "window_right"):
            p.window_right = right


def _out_dtype(q, out_):
    if out_ is not None:
        _require(out_.dtype in (torch.float16, torch.bfloat16), "Output must be fp16 or bf16")
        if q.dtype != torch.float8_e4m3fn:
            _require(out_.dtype == q.dtype, "Output must have the same dtype as inputs")
        return out_.dtype
    return torch.bfloat16 if q.dtype == torch.float8_e4m3fn else q.dtype


# ------------------------------------------------------------------------------------------------
# fwd  (fixed length)
# ------------------------------------------------------------------------------------------------
def fwd(q, k, v, out_, alibi_slopes_, p_dropout, softmax_scale, is_causal, window_size_left, window_size_right,
        softcap, return_softmax, gen_, is_bhsd=False, s_aux_=None, skip_softmax_threshold_scale_factor=0.0):
    _check_qkv(q, k, v, allow_dv=True)
    _unsupported(is_bhsd, "bhsd layout")
    _unsupported(alibi_slopes_ is not None, "alibi")
    _unsupported(p_dropout != 0.0, "dropout")
    _unsupported(softcap != 0.0, "softcap")
    _unsupported(return_softmax, "return_softmax")
    _unsupported(skip_softmax_threshold_scale_factor != 0.0, "skip-softmax")
    b, sq, h, d = q.shape
    sk, h_k, dv = k.shape[1], k.shape[2], v.shape[3]
    _require(b > 0, "batch size must be positive")
    _require(h % h_k == 0, "Number of heads in key/value must divide number of heads in query")
    _require(tuple(k.shape) == (b, sk, h_k, d) and tuple(v.shape) == (b, sk, h_k, dv), "k/v shape mismatch")
    # window normalisation as in mha_fwd (flash_api.cpp:1055-1060), except that a right bound is dropped only where it
    # cannot hide a key: with more queries than keys, bottom-right alignment puts the first rows' windows before key 0
    # (construct_local_mask, tests/test_flash_attn.py:185-217), however wide the bound
    if window_size_left >= sk:
        window_size_left = -1
    if window_size_right >= max(sk, sq):
        window_size_right = -1
    if sq == 1 and alibi_slopes_ is None:
        is_causal = False
    if is_causal:
        window_size_right = 0
    causal = window_size_right == 0   # a zero right window is the bottom-right causal mask (plus a left window, if any)
    if q.data_ptr() == k.data_ptr():
        q = q.clone()
    odt = _out_dtype(q, out_)
    if out_ is not None:
        _require(tuple(out_.shape) == (b, sq, h, dv), "out has wrong shape")
        _require(out_.stride(-1) == 1, "Output tensor must have contiguous last dimension")
        out = out_
    else:
        out = torch.empty((b, sq, h, dv), dtype=odt, device=q.device)
    lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    p = FwdParams()
    p.q, p.k, p.v, p.out, p.softmax_lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_batch_stride, p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
    p.k_batch_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
    p.v_batch_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
    p.o_batch_stride, p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d, p.d_v = b, sq, sk, h, h_k, d, dv
    p.softmax_scale = softmax_scale
    p.is_causal = 1 if causal else 0
    p.dtype, p.out_dtype = _DT[q.dtype], _DT[odt]
    _set_sinks(p, s_aux_, h)
    _set_window(p, window_size_left, window_size_right)
    _apply_profile_events(p)
    p.kernel_choice = _env_kernel()
    with _on_device(q.device):
        _counter = _own_work_counter(p, q.device)
        _check(_lib.fa_b200_fwd(ctypes.byref(p), _stream(q)), "fwd")
    rng_state = torch.empty((2,), dtype=torch.int64, device=q.device)
    s_dmask = torch.empty((0,), dtype=q.dtype, device=q.device)
    skip_blocks_info = torch.empty((0,), dtype=torch.int32, device=q.device)
    return [out, q, k, v, out, lse, s_dmask, rng_state, skip_blocks_info]


# ------------------------------------------------------------------------------------------------
# varlen_fwd  (packed sequences)
# ------------------------------------------------------------------------------------------------
def varlen_fwd(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k_, block_table_, alibi_slopes_,
               max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
               window_size_right, softcap, return_softmax, q_descale_=None, k_descale_=None, v_descale_=None,
               gen_=None, s_aux_=None):
    paged = block_table_ is not None
    _check_qkv(q, k, v, paged and _is_transposed_v(v), allow_dv=True)
    _unsupported(seqused_k is not None and not paged, "seqused_k without block_table")
    _unsupported(leftpad_k_ is not None, "leftpad_k")
    _unsupported(alibi_slopes_ is not None, "alibi")
    _unsupported(p_dropout != 0.0, "dropout")
    _unsupported(softcap != 0.0, "softcap")
    _unsupported(return_softmax, "return_softmax")
    for name, t in (("cu_seqlens_q", cu_seqlens_q),) + (() if paged else (("cu_seqlens_k", cu_seqlens_k),)):
        _require(t.dtype == torch.int32, f"{name} must have dtype int32")
        _require(t.is_cuda, f"{name} must be on CUDA device")
        _require(t.is_contiguous(), f"{name} must be contiguous")
    total_q, h, d = q.shape
    dv = v.shape[-1]
    total_k, h_k = (0, k.shape[2]) if paged else (k.shape[0], k.shape[1])
    b = cu_seqlens_q.numel() - 1
    _require(b > 0, "batch size must be positive")
    _require(paged or cu_seqlens_k.numel() == b + 1, "cu_seqlens_k must have shape (batch_size + 1)")
    _require(h % h_k == 0, "Number of heads in key/value must divide number of heads in query")
    if window_size_left >= max_seqlen_k:
        window_size_left = -1
    if window_size_right >= max(max_seqlen_k, max_seqlen_q):   # see fwd: a right bound can matter when sq > sk
        window_size_right = -1
    if max_seqlen_q == 1 and alibi_slopes_ is None:
        is_causal = False
    if is_causal:
        window_size_right = 0
    causal = window_size_right == 0
    if q.data_ptr() == k.data_ptr():
        q = q.clone()
    odt = _out_dtype(q, out_)
    if out_ is not None:
        _require(tuple(out_.shape) == (total_q, h, dv), "out has wrong shape")
        _require(out_.stride(-1) == 1, "Output tensor must have contiguous last dimension")
        out = out_
    else:
        out = torch.empty((total_q, h, dv), dtype=odt, device=q.device)
    lse = torch.empty((h, total_q), dtype=torch.float32, device=q.device)
    if zero_tensors:
        out.zero_()
        lse.fill_(float("-inf"))
    p = FwdParams()
    p.q, p.k, p.v, p.out, p.softmax_lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
    p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d, p.d_v = b, max_seqlen_q, max_seqlen_k, h, h_k, d, dv
    p.total_q, p.total_k = total_q, total_k
    p.cu_seqlens_q = cu_seqlens_q.data_ptr()
    if paged:
        _set_paged(p, k, v, block_table_, seqused_k, b)
    else:
        p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1)
        p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1)
        p.cu_seqlens_k = cu_seqlens_k.data_ptr()
    p.softmax_scale = softmax_scale
    p.is_causal = 1 if causal else 0
    p.dtype, p.out_dtype = _DT[q.dtype], _DT[odt]
    _descale(p, "q_descale", q_descale_, b, h_k)
    _descale(p, "k_descale", k_descale_, b, h_k)
    _descale(p, "v_descale", v_descale_, b, h_k)
    _set_sinks(p, s_aux_, h)
    _set_window(p, window_size_left, window_size_right)
    _apply_profile_events(p)
    p.kernel_choice = _env_kernel()
    with _on_device(q.device):
        _counter = _own_work_counter(p, q.device)
        _check(_lib.fa_b200_fwd(ctypes.byref(p), _stream(q)), "varlen_fwd")
    rng_state = torch.empty((2,), dtype=torch.int64, device=q.device)
    s_dmask = torch.empty((0,), dtype=q.dtype, device=q.device)
    return [out, q, k, v, out, lse, s_dmask, rng_state]


# ------------------------------------------------------------------------------------------------
# fwd_kvcache  (paged decode)
# ------------------------------------------------------------------------------------------------
_workspaces = {}


def _workspace(device, nbytes: int) -> Optional[torch.Tensor]:
    """Scratch for split-KV partials.  Cached per (device, stream) and grown on demand, like the
    reference's workspace cache (src/paged_attention.cu:712-745); under graph capture a fresh buffer is
    taken from the caching allocator instead."""
    if nbytes == 0:
        return None
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    key = (device.index, _stream_handle(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _is_transposed_v(vcache) -> bool:
    """A (num_blocks, page, h_k, d) view whose contiguous axis is the page's tokens (the reference's layout 0)."""
    return vcache.dim() == 4 and vcache.stride(-1) != 1 and vcache.stride(1) == 1


def _decode_params(q, kcache, vcache, seqlens_k, block_table, softmax_scale, out, lse, q_descale=None,
                   k_descale=None, v_descale=None, partition_tokens=0, max_seqlen_k=0):
    b, sq, h, d = q.shape
    num_blocks, page, h_k = kcache.shape[0], kcache.shape[1], kcache.shape[2]
    p = DecodeParams()
    p.q, p.k_cache, p.v_cache = q.data_ptr(), kcache.data_ptr(), vcache.data_ptr()
    p.out, p.softmax_lse = _ptr(out), _ptr(lse)
    # one stride() call per tensor: every Python -> torch call on this path is a good part of a microsecond
    qs, ks, vs = q.stride(), kcache.stride(), vcache.stride()
    p.q_batch_stride, p.q_row_stride, p.q_head_stride = qs[0], qs[1], qs[2]
    p.seqlen_q = sq
    if out is not None:
        os_ = out.stride()
        p.o_batch_stride, p.o_row_stride, p.o_head_stride = os_[0], os_[1], os_[2]
    p.k_block_stride, p.k_row_stride, p.k_head_stride = ks[0], ks[1], ks[2]
    if len(vs) == 4 and vs[3] != 1 and vs[1] == 1:
        # (num_blocks, page, h_k, d) view of a pool stored as (num_blocks, h_k, d, page): the tokens are the contiguous axis
        p.v_transposed = 1
        p.v_block_stride, p.v_head_stride, p.v_row_stride = vs[0], vs[2], vs[3]
    else:
        p.v_block_stride, p.v_row_stride, p.v_head_stride = vs[0], vs[1], vs[2]
    p.block_table, p.block_table_batch_stride = block_table.data_ptr(), block_table.stride(0)
    p.cache_seqlens = seqlens_k.data_ptr()
    p.b, p.h, p.h_k, p.d = b, h, h_k, d
    p.num_blocks, p.page_size, p.max_blocks_per_seq = num_blocks, page, block_table.shape[1]
    p.softmax_scale = softmax_scale
    p.dtype = _DT[q.dtype]
    p.kv_e4m3 = 1 if _is_fp8_kv(q, kcache) else 0
    p.kv_e5m2 = 1 if p.kv_e4m3 and kcache.dtype == torch.float8_e5m2 else 0
    p.out_dtype = _DT[out.dtype] if out is not None else BF16
    _descale(p, "q_descale", q_descale, b, h_k)
    _descale(p, "k_descale", k_descale, b, h_k)
    _descale(p, "v_descale", v_descale, b, h_k)
    p.partition_tokens = partition_tokens or _env_partition()
    p.max_seqlen_k = max_seqlen_k
    _apply_profile_events(p)
    return p


def fwd_kvcache(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_, leftpad_k_,
                block_table_, alibi_slopes_, out_, softmax_scale, is_causal, window_size_left, window_size_right,
                softcap, is_rotary_interleaved, num_splits, s_aux_=None, q_descale_=None, k_descale_=None,
                v_descale_=None, max_seqlen_k=0):
    """Attention over a paged KV cache: the decode kernel for one query token per sequence, the prefill kernel
    reading K/V through the block table for more.  Like the reference's mha_fwd_kvcache (flash_api.cpp:2530-2577) this path needs
    ``block_table`` and ``seqlens_k`` and ignores nothing silently.  New ``k_``/``v_`` are appended to the cache in
    place at positions seqlens_k.. (keys rotated by ``rotary_cos_``/``rotary_sin_``, queries rotated into a copy) and
    the attention then runs over seqlens_k + seqlen_new keys, the semantics the public signature documents
    (flash_attn_interface.py:2503-2520) and the reference's wrapper drops; cache_batch_idx and cache_leftpad
    (contiguous caches only) raise.  Unlike the reference, the returned softmax_lse is filled in."""
    v_t = _is_transposed_v(vcache)
    fp8_kv = _is_fp8_kv(q, kcache)
    _check_qkv(q, kcache, vcache, v_t, allow_fp8_kv=True)
    _unsupported(fp8_kv and (v_t or k_ is not None or q_descale_ is not None or
                             q.shape[1] * (q.shape[2] // max(kcache.shape[2], 1)) > 16),
                 "an e4m3 KV cache under 16-bit queries outside the decode of a few tokens (no append, no q_descale)")
    _unsupported(v_t and (k_ is not None or q.dtype == torch.float8_e4m3fn),
                 "a transposed V pool (layout 0) with e4m3 tensors or with new keys to append")
    _require((k_ is None) == (v_ is None), "k and v must be passed together")
    _require(rotary_cos_ is None or k_ is not None, "rotary_cos/rotary_sin are only applicable if k and v are passed in")
    _require((rotary_cos_ is None) == (rotary_sin_ is None), "rotary_cos and rotary_sin must be passed together")
    _unsupported(cache_batch_idx_ is not None, "cache_batch_idx")
    _unsupported(leftpad_k_ is not None, "cache_leftpad")
    _unsupported(alibi_slopes_ is not None, "alibi")
    _unsupported(softcap != 0.0, "softcap")
    _require(block_table_ is not None, "block_table is required (paged KV cache)")
    _require(seqlens_k_ is not None, "cache_seqlens is required")
    _require(block_table_.dtype == torch.int32, "block_table must have dtype torch.int32")
    _require(block_table_.stride(-1) == 1, "block_table must have contiguous last dimension")
    _require(seqlens_k_.dtype == torch.int32, "seqlens_k must have dtype int32")
    _require(seqlens_k_.is_contiguous(), "seqlens_k must be contiguous")
    b, sq, h, d = q.shape
    _require(seqlens_k_.numel() == b and block_table_.shape[0] == b, "cache_seqlens / block_table batch mismatch")
    _require(kcache.shape == vcache.shape, "k_cache and v_cache must have the same shape")
    h_k = kcache.shape[2]
    _require(h % h_k == 0, "Number of heads in key/value must divide number of heads in query")
    odt = _out_dtype(q, out_)
    if out_ is not None:
        _require(tuple(out_.shape) == (b, sq, h, d), "out has wrong shape")
        _require(out_.stride(-1) == 1, "Output tensor must have contiguous last dimension")
        out = out_
    else:
        out = torch.empty((b, sq, h, d), dtype=odt, device=q.device)
    lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    if k_ is not None:
        q, seqlens_k_ = kv_append(q, kcache, vcache, k_, v_, seqlens_k_, block_table_, rotary_cos_, rotary_sin_,
                                  is_rotary_interleaved, is_causal or window_size_left >= 0 or window_size_right >= 0)
    if sq > 1 and sq * (h // h_k) > 16:
        # several query tokens per sequence (chunked prefill) over the paged cache: the prefill kernel reads K/V through
        # the block table; the causal mask is bottom-right aligned to each cache length.  A few tokens (speculative
        # decoding: tokens x heads per kv head <= 16) stay on the decode kernel below, which packs them into the rows of
        # its tile and streams the cache once.
        fp = FwdParams()
        fp.q, fp.out, fp.softmax_lse = q.data_ptr(), out.data_ptr(), lse.data_ptr()
        fp.q_batch_stride, fp.q_row_stride, fp.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
        fp.o_batch_stride, fp.o_row_stride, fp.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
        fp.b, fp.seqlen_q, fp.h, fp.h_k, fp.d = b, sq, h, h_k, d
        fp.seqlen_k = kcache.shape[1] * block_table_.shape[1]
        if max_seqlen_k > 0:   # the caller's bound on the cache lengths
            fp.seqlen_k = min(fp.seqlen_k, max_seqlen_k)
        fp.softmax_scale = softmax_scale
        fp.is_causal = 1 if is_causal else 0
        fp.dtype, fp.out_dtype = _DT[q.dtype], _DT[odt]
        _descale(fp, "q_descale", q_descale_, b, h_k)
        _descale(fp, "k_descale", k_descale_, b, h_k)
        _descale(fp, "v_descale", v_descale_, b, h_k)
        _set_paged(fp, kcache, vcache, block_table_, seqlens_k_, b)
        _set_sinks(fp, s_aux_, h)
        _set_window(fp, window_size_left, 0 if is_causal else window_size_right)
        _apply_profile_events(fp)
        fp.kernel_choice = _env_kernel()
        with _on_device(q.device):
            _counter = _own_work_counter(fp, q.device)
            _check(_lib.fa_b200_fwd(ctypes.byref(fp), _stream(q)), "fwd_kvcache")
        return [out, lse]
    p = _decode_params(q, kcache, vcache, seqlens_k_, block_table_, softmax_scale, out, lse, q_descale_, k_descale_,
                       v_descale_, 0, max_seqlen_k)
    p.is_causal = 1 if is_causal else 0
    _unsupported(sq > 1 and not is_causal and window_size_right >= 0, "a right window bound with several decode tokens")
    _set_sinks(p, s_aux_, h)
    _set_window(p, window_size_left, -1)   # query tokens at the end of their sequence: only the left side matters
    with _on_device(q.device):
        ws = _workspace(q.device, int(_lib.fa_b200_decode_workspace_bytes(ctypes.byref(p))))
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
            _tickets = _own_tickets(p, q.device, b * h_k)
        _check(_lib.fa_b200_decode_paged(ctypes.byref(p), _stream(q)), "fwd_kvcache")
    return [out, lse]


def paged_attention(out, query, key_cache, value_cache, scale, block_tables, seq_lens, alibi_slopes=None, kv_cache_dtype="auto",
                    q_scale=None, k_scale=None, v_scale=None, max_seq_len=0, s_aux_=None, layout=0, window_size_left=-1,
                    window_size_right=-1, is_causal=False):
    """The reference's second decode binding (csrc/flash_attn_cutlass/flash_api.cpp:2496-2515): attention of
    query (num_seqs, seqlen_q, num_heads, 128) over paged pools into the caller's ``out``.  layout 0: key_cache
    (num_blocks, h_k, page, d) and value_cache (num_blocks, h_k, d, page); 1: both (num_blocks, h_k, page, d); 2: both
    (num_blocks, page, h_k, d).  q/k/v_scale are the e4m3 descales."""
    if str(kv_cache_dtype).startswith("fp8"):
        if key_cache.dtype == torch.uint8:      # caches kept as raw bytes
            f8 = torch.float8_e5m2 if "e5m2" in str(kv_cache_dtype) else torch.float8_e4m3fn
            key_cache, value_cache = key_cache.view(f8), value_cache.view(f8)
    else:
        _unsupported(kv_cache_dtype not in ("auto", ""), f"kv_cache_dtype {kv_cache_dtype!r}")
    if layout == 2:
        kc, vc = key_cache, value_cache
    elif layout == 1:
        kc, vc = key_cache.permute(0, 2, 1, 3), value_cache.permute(0, 2, 1, 3)
    elif layout == 0:
        kc, vc = key_cache.permute(0, 2, 1, 3), value_cache.permute(0, 3, 1, 2)
    else:
        raise RuntimeError(f"unknown paged layout {layout}")
    q4 = query if query.dim() == 4 else query.unsqueeze(1)
    o4 = out if out.dim() == 4 else out.unsqueeze(1)
    fwd_kvcache(q4, kc, vc, None, None, seq_lens, None, None, None, None, block_tables, alibi_slopes, o4, float(scale),
                is_causal, window_size_left, window_size_right, 0.0, True, 0, s_aux_, q_scale, k_scale, v_scale, max_seq_len)


def kv_cache_attention(q, seq_offsets, max_seqlen_q, max_seqlen_k, k_caches, v_caches, page_tables, cache_lens, out,
                       num_query, num_tokens, num_q_head, num_kv_head, num_dim, num_pages, page_size, dtype="bf16",
                       layout=1):
    """The reference's raw-pointer entry (extern "C" kv_cache_attention, csrc/flash_attn_cutlass/flash_api.cpp:2589-2624)
    with the same argument list; the tensors stand for its device pointers.  One token per request
    (num_query == num_tokens) decodes over all keys; otherwise the requests' tokens attend causally to their pages.
    layout 1: caches (num_pages, num_kv_head, page_size, num_dim); 2: (num_pages, page_size, num_kv_head, num_dim);
    0 (one token per request only): V (num_pages, num_kv_head, num_dim, page_size).  Writes ``out``."""
    for t in (q, k_caches, v_caches, page_tables, cache_lens, out):
        _require(t.is_cuda and t.is_contiguous(), "kv_cache_attention takes contiguous CUDA tensors")
    _require(page_tables.dtype == torch.int32 and cache_lens.dtype == torch.int32, "page_tables and cache_lens must be int32")
    offs = 0
    if num_query != num_tokens:
        _require(seq_offsets is not None and seq_offsets.dtype == torch.int32 and seq_offsets.is_cuda,
                 "seq_offsets must be an int32 CUDA tensor")
        offs = seq_offsets.data_ptr()
    code = F16 if dtype == "fp16" else BF16      # the reference: "fp16", anything else is bf16
    _require(q.dtype == (torch.float16 if code == F16 else torch.bfloat16), "q does not have the dtype named")
    with _on_device(q.device):
        nbytes = int(_lib.fa_b200_kv_cache_attention_workspace_bytes(num_query, num_q_head, num_kv_head, num_dim,
                                                                     page_size, max_seqlen_k)) if num_query == num_tokens else 0
        ws = _workspace(q.device, nbytes)
        _check(_lib.fa_b200_kv_cache_attention(
            q.data_ptr(), offs, max_seqlen_q, max_seqlen_k, k_caches.data_ptr(), v_caches.data_ptr(),
            page_tables.data_ptr(), cache_lens.data_ptr(), out.data_ptr(), num_query, num_tokens, num_q_head,
            num_kv_head, num_dim, num_pages, page_size, code, layout, ws.data_ptr() if ws is not None else None,
            nbytes, _stream(q)), "kv_cache_attention")


def cal_paged_attention(q, seq_offsets, max_seqlen_q, max_seqlen_k, k_caches, v_caches, page_tables, cache_lens, out,
                        num_query, num_tokens, num_q_head, num_kv_head, num_dim, num_pages, page_size, dtype="bf16"):
    """kv_cache_attention with layout 1 (flash_api.cpp:2625-2631)."""
    kv_cache_attention(q, seq_offsets, max_seqlen_q, max_seqlen_k, k_caches, v_caches, page_tables, cache_lens, out,
                       num_query, num_tokens, num_q_head, num_kv_head, num_dim, num_pages, page_size, dtype, 1)


def kv_append(q, kcache, vcache, k_new, v_new, seqlens_k, block_table, rotary_cos=None, rotary_sin=None,
              is_rotary_interleaved=True, rotate_q_per_token=True):
    """Writes k_new / v_new (batch, seqlen_new, nheads_k, d) into the paged cache at positions
    seqlens_k[b] .. seqlens_k[b] + seqlen_new - 1 (keys rotated when rotary_cos/sin (seqlen_ro, rotary_dim / 2) are
    given) and returns (q or its rotated copy, seqlens_k + seqlen_new).  q is rotated at positions
    seqlens_k[b] + s when ``rotate_q_per_token`` (causal or local attention), else at seqlens_k[b] for every s."""
    b, sq, h, d = q.shape
    _require(k_new.dim() == 4 and v_new.shape == k_new.shape, "k and v must be (batch, seqlen_new, nheads_k, d)")
    _require(k_new.shape[0] == b and k_new.shape[2] == kcache.shape[2] and k_new.shape[3] == d,
             "k and v must be (batch, seqlen_new, nheads_k, d)")
    _require(k_new.dtype == kcache.dtype and v_new.dtype == vcache.dtype and k_new.is_cuda and v_new.is_cuda,
             "Key and value must have the same dtype as the cache")
    _require(k_new.stride(-1) == 1 and v_new.stride(-1) == 1, "Key and value must have contiguous last dimension")
    p = KvAppendParams()
    p.k_new, p.v_new = k_new.data_ptr(), v_new.data_ptr()
    p.k_new_batch_stride, p.k_new_row_stride, p.k_new_head_stride = k_new.stride(0), k_new.stride(1), k_new.stride(2)
    p.v_new_batch_stride, p.v_new_row_stride, p.v_new_head_stride = v_new.stride(0), v_new.stride(1), v_new.stride(2)
    p.k_cache, p.v_cache = kcache.data_ptr(), vcache.data_ptr()
    p.k_block_stride, p.k_row_stride, p.k_head_stride = kcache.stride(0), kcache.stride(1), kcache.stride(2)
    p.v_block_stride, p.v_row_stride, p.v_head_stride = vcache.stride(0), vcache.stride(1), vcache.stride(2)
    p.block_table, p.block_table_batch_stride = block_table.data_ptr(), block_table.stride(0)
    seqlens_out = torch.empty_like(seqlens_k)
    p.seqlens_k, p.seqlens_out = seqlens_k.data_ptr(), seqlens_out.data_ptr()
    q_out = q
    if rotary_cos is not None:
        _require(q.dtype in (torch.float16, torch.bfloat16), "rotary embedding needs fp16 or bf16 inputs")
        _require(rotary_cos.dim() == 2 and rotary_sin.shape == rotary_cos.shape, "rotary_cos/sin must be (seqlen_ro, rotary_dim / 2)")
        _require(rotary_cos.dtype == q.dtype and rotary_sin.dtype == q.dtype, "rotary_cos/sin must have the same dtype as query")
        _require(rotary_cos.is_cuda and rotary_sin.is_cuda, "rotary_cos/sin must be on CUDA device")
        rotary_dim = rotary_cos.shape[1] * 2
        _require(rotary_dim <= d, "rotary_dim must be <= headdim")
        _require(rotary_dim % 16 == 0, "Only rotary dimensions divisible by 16 are currently supported")
        rotary_cos, rotary_sin = rotary_cos.contiguous(), rotary_sin.contiguous()
        q_out = torch.empty((b, sq, h, d), dtype=q.dtype, device=q.device)
        p.q, p.q_out = q.data_ptr(), q_out.data_ptr()
        p.q_batch_stride, p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
        p.q_out_batch_stride, p.q_out_row_stride, p.q_out_head_stride = q_out.stride(0), q_out.stride(1), q_out.stride(2)
        p.rotary_cos, p.rotary_sin = rotary_cos.data_ptr(), rotary_sin.data_ptr()
        p.rotary_dim, p.seqlen_ro = rotary_dim, rotary_cos.shape[0]
        p.is_rotary_interleaved = 1 if is_rotary_interleaved else 0
        p.rotate_q_per_token = 1 if rotate_q_per_token else 0
    p.b, p.seqlen_q, p.seqlen_new, p.h, p.h_k, p.d = b, sq, k_new.shape[1], h, kcache.shape[2], d
    p.page_size, p.num_blocks, p.max_blocks_per_seq = kcache.shape[1], kcache.shape[0], block_table.shape[1]
    p.dtype = _DT[kcache.dtype]
    with _on_device(q.device):
        _check(_lib.fa_b200_kv_append(ctypes.byref(p), _stream(q)), "kv_append")
    return q_out, seqlens_out


def decode_partial(q, kcache, vcache, seqlens_k, block_table, softmax_scale, q_descale=None, k_descale=None,
                   v_descale=None, max_seqlen_k=0, window_left=-1):
    """Decode over a LOCAL slice of each sequence's pages and return the unnormalised-merge inputs
    (o_partial fp32 (b, h, d), lse fp32 (b, h)) for a cross-GPU combine (one sequence split-KV across GPUs).
    ``window_left`` >= 0: only the last window_left + 1 keys of the slice are visible."""
    _check_qkv(q, kcache, vcache)
    b, sq, h, d = q.shape
    _require(sq == 1, "decode_partial takes one query token per sequence")
    # one buffer, [O | LSE] back to back: a cross-GPU exchange moves it with a single all-gather
    packed = torch.empty((b * h * (d + 1),), dtype=torch.float32, device=q.device)
    o_part, lse_part = packed[:b * h * d].view(b, h, d), packed[b * h * d:].view(b, h)
    p = _decode_params(q, kcache, vcache, seqlens_k, block_table, softmax_scale, None, None, q_descale, k_descale,
                       v_descale, 0, max_seqlen_k)
    p.o_partial_out, p.lse_partial_out = o_part.data_ptr(), lse_part.data_ptr()
    _set_window(p, window_left, -1)
    with _on_device(q.device):
        ws = _workspace(q.device, int(_lib.fa_b200_decode_workspace_bytes(ctypes.byref(p))))
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
            _tickets = _own_tickets(p, q.device, b * kcache.shape[2])
        _check(_lib.fa_b200_decode_paged(ctypes.byref(p), _stream(q)), "decode_partial")
    return o_part, lse_part


def combine(o_partial, lse_partial, out_dtype=torch.bfloat16, h: Optional[int] = None, parts_per_row=None, s_aux=None):
    """LSE-combine: o_partial (parts, rows, 128) fp32, lse_partial (parts, rows) fp32 ->
    (out (rows, 128) out_dtype, lse (rows) fp32).  rows = batch * h; ``s_aux`` (h) adds each head's attention sink."""
    _require(o_partial.dtype == torch.float32 and lse_partial.dtype == torch.float32, "partials must be fp32")
    # partitions may be strided (partials gathered as one [O | LSE] buffer per rank); rows and columns are packed
    _require(o_partial.dim() == 3 and o_partial.stride(2) == 1 and o_partial.stride(1) == o_partial.shape[2] and
             lse_partial.dim() == 2 and lse_partial.stride(1) == 1, "partials must be packed within a partition")
    parts, rows, d = o_partial.shape
    out = torch.empty((rows, d), dtype=out_dtype, device=o_partial.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=o_partial.device)
    p = CombineParams()
    p.o_partial, p.lse_partial, p.out, p.lse = o_partial.data_ptr(), lse_partial.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.out_row_stride = d
    p.num_parts, p.rows, p.d, p.h = parts, rows, d, (h or 1)
    p.parts_per_row = _ptr(parts_per_row)
    p.out_dtype = -1 if out_dtype == torch.float32 else _DT[out_dtype]
    p.out_scale = 1.0
    p.o_part_stride, p.lse_part_stride = o_partial.stride(0), lse_partial.stride(0)
    _set_sinks(p, s_aux, h or 1)
    with _on_device(o_partial.device):
        _check(_lib.fa_b200_combine(ctypes.byref(p), _stream(o_partial)), "combine")
    return out, lse


# ------------------------------------------------------------------------------------------------
# exchange of split-KV partials between GPUs over peer memory, fused with the combine
# ------------------------------------------------------------------------------------------------
IPC_HANDLE_BYTES = 64


def exchange_alloc(world: int, rows: int, d: int, device) -> Tuple[int, bytes, int]:
    """This rank's exchange buffer for ``rows`` partial rows of ``d`` columns among ``world`` ranks, allocated and
    zeroed by the library on ``device``: (device pointer, 64-byte CUDA IPC handle for the other ranks' processes, size).
    A set-up call: it allocates and synchronises."""
    n = int(_lib.fa_b200_exchange_bytes(world, rows, d))
    _require(n > 0, "exchange_alloc: world, rows and d must be positive")
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(IPC_HANDLE_BYTES)
    with _on_device(torch.device(device)):
        _check(_lib.fa_b200_exchange_alloc(n, ctypes.byref(ptr), handle), "exchange_alloc")
    return int(ptr.value), handle.raw, n


def exchange_open(handle: bytes, device) -> int:
    """Map another process's exchange buffer on ``device``; returns the device pointer."""
    _require(len(handle) == IPC_HANDLE_BYTES, "exchange_open: a 64-byte IPC handle")
    ptr = ctypes.c_void_p()
    with _on_device(torch.device(device)):
        _check(_lib.fa_b200_exchange_open(handle, ctypes.byref(ptr)), "exchange_open")
    return int(ptr.value)


def exchange_close(ptr: int) -> None:
    _check(_lib.fa_b200_exchange_close(ptr), "exchange_close")


def exchange_free(ptr: int) -> None:
    _check(_lib.fa_b200_exchange_free(ptr), "exchange_free")


def exchange_combine(o_local, lse_local, peers: Sequence[int], rank: int, epoch: int, h: int, out_dtype=torch.bfloat16,
                     s_aux=None, seqlen_q: int = 1, push: bool = True, wait: bool = True, rows: Optional[int] = None,
                     d: Optional[int] = None, device=None):
    """One launch of fa_b200_exchange_combine on the current stream: this rank's partial (o_local (rows, d) fp32,
    lse_local (rows) fp32) goes to slot ``rank`` of every buffer in ``peers`` (device pointers of ranks 0 .. world-1 as
    mapped on this GPU), the kernel waits for every rank's partial of this ``epoch`` in its own buffer and combines.
    Returns (out (rows, d) out_dtype, lse (rows) fp32).  ``push`` / ``wait`` run the two halves alone (tests)."""
    world = len(peers)
    if o_local is not None:
        _require(o_local.dtype == torch.float32 and lse_local.dtype == torch.float32 and o_local.is_contiguous() and
                 lse_local.is_contiguous() and o_local.dim() == 2, "exchange_combine: packed fp32 partials (rows, d) and (rows)")
        rows, d = o_local.shape
        device = o_local.device
    device = torch.device(device)
    out = torch.empty((rows, d), dtype=out_dtype, device=device)
    lse = torch.empty((rows,), dtype=torch.float32, device=device)
    p = ExchangeParams()
    p.world, p.rank, p.rows, p.h, p.seqlen_q, p.d = world, rank, rows, h, seqlen_q, d
    p.o_local, p.lse_local = _ptr(o_local), _ptr(lse_local)
    for i, ptr in enumerate(peers):
        p.peers[i] = ptr
    p.epoch, p.do_push, p.do_wait = epoch, int(push), int(wait)
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    # rows are (b, h, token), packed
    p.out_batch_stride, p.out_head_stride, p.out_tok_stride = h * seqlen_q * d, seqlen_q * d, d
    p.out_dtype = -1 if out_dtype == torch.float32 else _DT[out_dtype]
    _set_sinks(p, s_aux, h)
    with _on_device(device):
        _check(_lib.fa_b200_exchange_combine(ctypes.byref(p), ctypes.c_void_p(_stream_handle(device))), "exchange_combine")
    return out, lse


# ------------------------------------------------------------------------------------------------
# fwd_sparse  (block-list attention)
# ------------------------------------------------------------------------------------------------
def fwd_sparse(q, k, v, block_count, block_offset, column_count, column_index, out_, alibi_slopes_, p_dropout,
               softmax_scale, is_causal, softcap, return_softmax, gen_, is_sla=False, pv_threshold=50.0,
               enable_dynamic_skip=False):
    _check_qkv(q, k, v)
    _unsupported(alibi_slopes_ is not None, "alibi")
    _unsupported(p_dropout != 0.0, "dropout")
    _unsupported(softcap != 0.0, "softcap")
    _unsupported(return_softmax, "return_softmax")
    _unsupported(is_sla, "SLA sparse attention")
    _unsupported(enable_dynamic_skip, "dynamic PV skip")
    b, sq, h, d = q.shape
    sk, h_k = k.shape[1], k.shape[2]
    _require(h % h_k == 0, "Number of heads in key/value must divide number of heads in query")
    for name, t in (("block_count", block_count), ("block_offset", block_offset)):
        _require(t.dtype == torch.int32 and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous int32 CUDA tensor")
    if column_count is not None:
        # the vertical part of the pattern is not taken; the kernel checks the counts where it reads its lists (no host
        # synchronisation here) and a non-zero one shows up in device_status()
        _require(column_count.dtype == torch.int32 and column_count.is_cuda and column_count.is_contiguous(),
                 "column_count must be a contiguous int32 CUDA tensor")
    # host rule of the reference: NUM_ROWS == ceil(Sq / (Sq <= 2048 ? 64 : 128)) (flash_api_sparse.cpp:127-137)
    block_m = 64 if sq <= 2048 else 128
    num_rows = (sq + block_m - 1) // block_m
    _require(tuple(block_count.shape) == (b, h, num_rows), "block_count must have shape (batch, nheads, NUM_ROWS)")
    _require(block_offset.dim() == 4 and tuple(block_offset.shape[:3]) == (b, h, num_rows),
             "block_offset must have shape (batch, nheads, NUM_ROWS, NNZ_S)")
    if sq == 1:
        is_causal = False
    odt = _out_dtype(q, out_)
    out = out_ if out_ is not None else torch.empty((b, sq, h, d), dtype=odt, device=q.device)
    lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    p = FwdParams()
    p.q, p.k, p.v, p.out, p.softmax_lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_batch_stride, p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
    p.k_batch_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
    p.v_batch_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
    p.o_batch_stride, p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d = b, sq, sk, h, h_k, d
    p.softmax_scale = softmax_scale
    p.is_causal = 1 if is_causal else 0
    p.dtype, p.out_dtype = _DT[q.dtype], _DT[odt]
    p.block_count, p.block_offset = block_count.data_ptr(), block_offset.data_ptr()
    p.num_q_blocks, p.nnz_s, p.block_m = num_rows, block_offset.shape[3], block_m
    if column_count is not None:
        _require(tuple(column_count.shape) == (b, h, num_rows), "column_count must have shape (batch, nheads, NUM_ROWS)")
        p.column_count = column_count.data_ptr()
    _apply_profile_events(p)
    p.kernel_choice = _env_kernel()
    with _on_device(q.device):
        _check(_lib.fa_b200_fwd_sparse(ctypes.byref(p), _stream(q)), "fwd_sparse")
    return [out, lse]


def varlen_fwd_sparse(q, k, v, block_count, block_offset, column_count, column_index, out_, cu_seqlens_q, cu_seqlens_k,
                      seqused_k, alibi_slopes_, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors,
                      is_causal, softcap, return_softmax, gen_=None, pv_threshold=50.0, enable_dynamic_skip=False):
    """Block-list attention over packed sequences, the reference binding's ``varlen_fwd_sparse``
    (csrc/flash_attn_cutlass/flash_api_sparse.cpp:339-558, bound at flash_api.cpp:3018): q (total_q, h, 128), k / v
    (total_k, h_k, 128), int32 cu_seqlens; block_count (b, h, NUM_ROWS), block_offset (b, h, NUM_ROWS, NNZ_S) with
    NUM_ROWS = ceil(max_seqlen_q / (64 if max_seqlen_q <= 2048 else 128)) and key row offsets relative to each
    sequence's first key.  Returns [out, softmax_lse (h, total_q)]."""
    _check_qkv(q, k, v)
    _require(q.dtype in (torch.float16, torch.bfloat16), "FlashAttention only support fp16 and bf16 data type")
    _unsupported(seqused_k is not None, "seqused_k")
    _unsupported(alibi_slopes_ is not None, "alibi")
    _unsupported(p_dropout != 0.0, "dropout")
    _unsupported(softcap != 0.0, "softcap")
    _unsupported(return_softmax, "return_softmax")
    _unsupported(enable_dynamic_skip, "dynamic PV skip")
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k)):
        _require(t.dtype == torch.int32, f"{name} must have dtype int32")
        _require(t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous CUDA tensor")
    total_q, h, d = q.shape
    total_k, h_k = k.shape[0], k.shape[1]
    b = cu_seqlens_q.numel() - 1
    _require(b > 0, "batch size must be positive")
    _require(cu_seqlens_k.numel() == b + 1, "cu_seqlens_k must have shape (batch_size + 1)")
    _require(h % h_k == 0, "Number of heads in key/value must divide number of heads in query")
    for name, t in (("block_count", block_count), ("block_offset", block_offset)):
        _require(t.dtype == torch.int32 and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous int32 CUDA tensor")
    block_m = 64 if max_seqlen_q <= 2048 else 128
    num_rows = (max_seqlen_q + block_m - 1) // block_m
    _require(tuple(block_count.shape) == (b, h, num_rows), "block_count must have shape (batch, nheads, NUM_ROWS)")
    _require(block_offset.dim() == 4 and tuple(block_offset.shape[:3]) == (b, h, num_rows),
             "block_offset must have shape (batch, nheads, NUM_ROWS, NNZ_S)")
    if max_seqlen_q == 1:
        is_causal = False
    odt = _out_dtype(q, out_)
    out = out_ if out_ is not None else torch.empty((total_q, h, d), dtype=odt, device=q.device)
    lse = torch.empty((h, total_q), dtype=torch.float32, device=q.device)
    if zero_tensors:
        out.zero_()
        lse.fill_(float("-inf"))
    p = FwdParams()
    p.q, p.k, p.v, p.out, p.softmax_lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
    p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1)
    p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1)
    p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d = b, max_seqlen_q, max_seqlen_k, h, h_k, d
    p.total_q, p.total_k = total_q, total_k
    p.cu_seqlens_q, p.cu_seqlens_k = cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr()
    p.softmax_scale = softmax_scale
    p.is_causal = 1 if is_causal else 0
    p.dtype, p.out_dtype = _DT[q.dtype], _DT[odt]
    p.block_count, p.block_offset = block_count.data_ptr(), block_offset.data_ptr()
    p.num_q_blocks, p.nnz_s, p.block_m = num_rows, block_offset.shape[3], block_m
    if column_count is not None:
        _require(column_count.dtype == torch.int32 and column_count.is_cuda and column_count.is_contiguous() and
                 tuple(column_count.shape) == (b, h, num_rows), "column_count must be a contiguous int32 (batch, nheads, NUM_ROWS) CUDA tensor")
        p.column_count = column_count.data_ptr()
    _apply_profile_events(p)
    with _on_device(q.device):
        _check(_lib.fa_b200_fwd_sparse(ctypes.byref(p), _stream(q)), "varlen_fwd_sparse")
    return [out, lse]


# ------------------------------------------------------------------------------------------------
# callers' glue: padding removal and block-map conversion
# ------------------------------------------------------------------------------------------------
def unpad_plan(attention_mask):
    """attention_mask (batch, seqlen) bool / int -> (seqlens int32 (batch), cu_seqlens int32 (batch + 1), indices int64
    (total), max_seqlen int).  Reads the two totals back (one host synchronisation, as the reference's .item())."""
    _require(attention_mask.is_cuda and attention_mask.dim() == 2, "attention_mask must be a CUDA tensor of shape (batch, seqlen)")
    _require(attention_mask.element_size() in (1, 4, 8) and attention_mask.stride(1) == 1,
             "attention_mask must be bool / uint8 / int32 / int64 with contiguous rows")
    b, s = attention_mask.shape
    dev = attention_mask.device
    seqlens = torch.empty((b,), dtype=torch.int32, device=dev)
    cu = torch.empty((b + 1,), dtype=torch.int32, device=dev)
    indices = torch.empty((b * s,), dtype=torch.int64, device=dev)
    stats = torch.empty((2,), dtype=torch.int32, device=dev)
    with _on_device(dev):
        _check(_lib.fa_b200_unpad_plan(attention_mask.data_ptr(), attention_mask.element_size(), b, s, attention_mask.stride(0),
                                       seqlens.data_ptr(), cu.data_ptr(), indices.data_ptr(), stats.data_ptr(),
                                       _stream(attention_mask)), "unpad_plan")
    mx, total = stats.tolist()
    return seqlens, cu, indices[:total], mx


def _move_rows(fn, what, src2d, indices, dst2d):
    _require(src2d.is_cuda and dst2d.is_cuda and indices.is_cuda, "tensors must be on a CUDA device")
    _require(indices.dtype == torch.int64 and indices.is_contiguous(), "indices must be a contiguous int64 tensor")
    _require(src2d.is_contiguous() and dst2d.is_contiguous() and src2d.dtype == dst2d.dtype, "rows must be contiguous and of one dtype")
    row_bytes = src2d.shape[1] * src2d.element_size()
    limit = dst2d.shape[0] if fn is _lib.fa_b200_scatter_rows else src2d.shape[0]
    with _on_device(src2d.device):
        _check(fn(src2d.data_ptr(), indices.data_ptr(), dst2d.data_ptr(), indices.numel(), row_bytes, limit, _stream(src2d)), what)


def gather_rows(src, indices):
    """src (n, ...) -> src[indices] (index_first_axis of the reference's bert_padding.py)."""
    src2d = src.reshape(src.shape[0], -1)
    src2d = src2d if src2d.is_contiguous() else src2d.contiguous()
    out = torch.empty((indices.numel(), src2d.shape[1]), dtype=src.dtype, device=src.device)
    _move_rows(_lib.fa_b200_gather_rows, "gather_rows", src2d, indices, out)
    return out.reshape(indices.numel(), *src.shape[1:])


def scatter_rows(values, indices, first_axis_dim):
    """zeros (first_axis_dim, ...) with rows `indices` set to `values` (index_put_first_axis)."""
    v2d = values.reshape(values.shape[0], -1)
    v2d = v2d if v2d.is_contiguous() else v2d.contiguous()
    out = torch.zeros((first_axis_dim, v2d.shape[1]), dtype=values.dtype, device=values.device)
    _move_rows(_lib.fa_b200_scatter_rows, "scatter_rows", v2d, indices, out)
    return out.reshape(first_axis_dim, *values.shape[1:])


def block_map_to_offset(block_map, scale=1, fill=10000000):
    """block_map (..., k) bool -> (block_offset (..., k) int32: ascending set positions times ``scale`` then ``fill``,
    block_count (...) int32)."""
    _require(block_map.is_cuda and block_map.dtype in (torch.bool, torch.uint8), "block_map must be a CUDA bool / uint8 tensor")
    bm = block_map if block_map.is_contiguous() else block_map.contiguous()
    k = bm.shape[-1]
    rows = bm.numel() // k if k else 0
    off = torch.empty(bm.shape, dtype=torch.int32, device=bm.device)
    cnt = torch.empty(bm.shape[:-1], dtype=torch.int32, device=bm.device)
    with _on_device(bm.device):
        _check(_lib.fa_b200_block_map_to_offset(bm.data_ptr(), off.data_ptr(), cnt.data_ptr(), rows, k, scale, fill, _stream(bm)),
               "block_map_to_offset")
    return off, cnt


def block_pool(x, block_rows, sim_threshold):
    """x (B, H, N, D) fp16 / bf16 (last dim contiguous) -> (pooled (B, H, nb, D) of x's dtype: the mean row of every
    block of ``block_rows`` rows; sim (B, H, nb) bool: the block's rows are similar to one another, mean pairwise cosine
    similarity > sim_threshold[head]).  sim_threshold: fp32 (H) on the device."""
    _require(x.is_cuda and x.dim() == 4 and x.dtype in (torch.float16, torch.bfloat16) and x.stride(-1) == 1,
             "x must be a (B, H, N, D) fp16 / bf16 CUDA tensor with contiguous last dimension")
    _require(sim_threshold.is_cuda and sim_threshold.dtype == torch.float32 and sim_threshold.numel() == x.shape[1],
             "sim_threshold must be a float32 CUDA tensor with one element per head")
    B, H, N, D = x.shape
    nb = (N + block_rows - 1) // block_rows
    pooled = torch.empty((B, H, nb, D), dtype=x.dtype, device=x.device)
    sim = torch.empty((B, H, nb), dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        _check(_lib.fa_b200_block_pool(x.data_ptr(), _DT[x.dtype], x.stride(0), x.stride(1), x.stride(2), B, H, N, D,
                                       block_rows, sim_threshold.data_ptr(), pooled.data_ptr(), sim.data_ptr(), _stream(x)),
               "block_pool")
    return pooled, sim.view(torch.bool)


def block_select(pooled_q, pooled_k, sim_q, sim_k, block_q, block_k, scale, cdf_threshold=None, topk=None,
                 is_causal=False, attention_sink=False):
    """The key blocks every query block keeps: (B, H, nq, nk) bool.  cdf_threshold or topk: fp32 (H) on the device."""
    _require((cdf_threshold is None) != (topk is None), "Only one of cdfthreshd and topk can be set.")
    B, H, nq, D = pooled_q.shape
    nk = pooled_k.shape[2]
    for t in (pooled_q, pooled_k, sim_q, sim_k):
        _require(t.is_cuda and t.is_contiguous(), "block_select takes contiguous CUDA tensors")
    hyper = cdf_threshold if cdf_threshold is not None else topk
    _require(hyper.is_cuda and hyper.dtype == torch.float32 and hyper.numel() == H, "one float32 threshold per head")
    block_map = torch.empty((B, H, nq, nk), dtype=torch.uint8, device=pooled_q.device)
    with _on_device(pooled_q.device):
        _check(_lib.fa_b200_block_select(
            pooled_q.data_ptr(), pooled_k.data_ptr(), sim_q.data_ptr(), sim_k.data_ptr(), _DT[pooled_q.dtype], B, H, nq, nk,
            D, block_q, block_k, float(scale), _ptr(cdf_threshold), _ptr(topk), 1 if is_causal else 0,
            1 if attention_sink else 0, block_map.data_ptr(), _stream(pooled_q)), "block_select")
    return block_map.view(torch.bool)


# ------------------------------------------------------------------------------------------------
# torch.library ops the reference's compiled extension defines on import
# ------------------------------------------------------------------------------------------------
# flash_attn2_c_op::varlen_fwd and ::fwd_kvcache are C++ schemas in the reference (csrc/flash_attn_cutlass/
# flash_api.cpp:2796-2816, TORCH_LIBRARY + TORCH_LIBRARY_IMPL); its Python interface only adds fake implementations
# (flash_attn/flash_attn_interface.py:203-278) and calls them through torch.ops.  Defining them here, with the same
# schemas character for character, lets that interface run unchanged over this module.
VARLEN_FWD_SCHEMA = (
    "(Tensor q, Tensor k, Tensor v, Tensor? out, "
    "Tensor cu_seqlens_q, Tensor cu_seqlens_k, Tensor? seqused_k, "
    "Tensor? leftpad_k_, Tensor? block_table_, Tensor? alibi_slopes_, "
    "int max_seqlen_q, int max_seqlen_k, float p_dropout, "
    "float softmax_scale, bool zero_tensors, bool is_causal, "
    "int window_size_left, int window_size_right, float softcap, "
    "bool return_softmax) -> (Tensor, Tensor, Tensor, Tensor)")

FWD_KVCACHE_SCHEMA = (
    "(Tensor q, Tensor kcache, Tensor vcache, "
    "Tensor? k_, Tensor? v_, Tensor? seqlens_k_, "
    "Tensor? rotary_cos_, Tensor? rotary_sin_, "
    "Tensor? cache_batch_idx_, Tensor? leftpad_k_, "
    "Tensor? block_table_, Tensor? alibi_slopes_, Tensor? out_, "
    "float softmax_scale, bool is_causal, "
    "int window_size_left, int window_size_right, "
    "float softcap, bool is_rotary_interleaved, int num_splits) "
    "-> (Tensor, Tensor)")


def _varlen_fwd_op(q, k, v, out, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k_, block_table_, alibi_slopes_,
                   max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
                   window_size_right, softcap, return_softmax):
    res = varlen_fwd(q, k, v, out, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k_, block_table_, alibi_slopes_,
                     max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
                     window_size_right, softcap, return_softmax)
    return res[0], res[5], res[6], res[7]   # out, softmax_lse, S_dmask, rng_state (flash_api.cpp TORCH_LIBRARY_IMPL)


def _fwd_kvcache_op(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_, leftpad_k_,
                    block_table_, alibi_slopes_, out_, softmax_scale, is_causal, window_size_left, window_size_right,
                    softcap, is_rotary_interleaved, num_splits):
    out, lse = fwd_kvcache(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_, leftpad_k_,
                           block_table_, alibi_slopes_, out_, softmax_scale, is_causal, window_size_left,
                           window_size_right, softcap, is_rotary_interleaved, num_splits)
    return out, lse


def _define_c_ops():
    try:
        torch.library.define("flash_attn2_c_op::varlen_fwd", VARLEN_FWD_SCHEMA)
        torch.library.define("flash_attn2_c_op::fwd_kvcache", FWD_KVCACHE_SCHEMA)
    except RuntimeError:      # already defined in this process (the module was loaded under a second name)
        return
    torch.library.impl("flash_attn2_c_op::varlen_fwd", "CUDA")(_varlen_fwd_op)
    torch.library.impl("flash_attn2_c_op::fwd_kvcache", "CUDA")(_fwd_kvcache_op)


_define_c_ops()
