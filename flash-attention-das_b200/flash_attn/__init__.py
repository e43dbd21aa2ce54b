"""B200-native drop-in for the forward attention hot path of flash-attention-das.

Same public names as the reference package (flash_attn/__init__.py:5-39) for the entries on the hot path;
everything calls the sm_100a kernels of libfa_b200.so through ``flash_attn_2_cuda``.
"""
__version__ = "2.8.4+b200"

from .flash_attn_interface import (  # noqa: F401
    flash_attn_func,
    flash_attn_varlen_func,
    flash_attn_with_kvcache,
    hg_flash_attn_varlen_func,
    sparse_attn_func,
    varlen_fwd_unified,
    vllm_flash_attn_varlen_func,
    vllm_flash_attn_with_kvcache,
)
from . import torch_ops  # noqa: F401,E402  (registers flash_attn::_flash_attn_forward, flash_attn2_c_op::varlen_fwd / fwd_kvcache)
from . import split_kv_parallel  # noqa: F401,E402  (multi-GPU helpers: sharding, partial all-gather + combine)
