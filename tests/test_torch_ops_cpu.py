"""CPU: the torch.library ops the reference registers (flash_attn::_flash_attn_forward, a Python custom op at
flash_attn/flash_attn_interface.py:74; flash_attn2_c_op::varlen_fwd / fwd_kvcache, C++ schemas at
csrc/flash_attn_cutlass/flash_api.cpp:2796-2816) exist under the same names with the same schemas, and their fake
implementations produce the shapes the reference's fakes produce (no kernel runs here)."""
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import flash_attn  # noqa: F401  (registers the ops)


def _norm(s):
    return "".join(str(s).split())


def test_schemas_match_the_reference():
    v = torch.ops.flash_attn2_c_op.varlen_fwd.default._schema
    assert _norm(v) == _norm(
        "flash_attn2_c_op::varlen_fwd(Tensor q, Tensor k, Tensor v, Tensor? out, Tensor cu_seqlens_q, Tensor cu_seqlens_k, "
        "Tensor? seqused_k, Tensor? leftpad_k_, Tensor? block_table_, Tensor? alibi_slopes_, int max_seqlen_q, "
        "int max_seqlen_k, float p_dropout, float softmax_scale, bool zero_tensors, bool is_causal, int window_size_left, "
        "int window_size_right, float softcap, bool return_softmax) -> (Tensor, Tensor, Tensor, Tensor)")
    kv = torch.ops.flash_attn2_c_op.fwd_kvcache.default._schema
    assert _norm(kv) == _norm(
        "flash_attn2_c_op::fwd_kvcache(Tensor q, Tensor kcache, Tensor vcache, Tensor? k_, Tensor? v_, Tensor? seqlens_k_, "
        "Tensor? rotary_cos_, Tensor? rotary_sin_, Tensor? cache_batch_idx_, Tensor? leftpad_k_, Tensor? block_table_, "
        "Tensor? alibi_slopes_, Tensor? out_, float softmax_scale, bool is_causal, int window_size_left, "
        "int window_size_right, float softcap, bool is_rotary_interleaved, int num_splits) -> (Tensor, Tensor)")
    f = torch.ops.flash_attn._flash_attn_forward.default._schema
    names = [a.name for a in f.arguments]
    assert names == ["q", "k", "v", "dropout_p", "softmax_scale", "causal", "window_size_left", "window_size_right",
                     "softcap", "alibi_slopes", "return_softmax", "bhsd", "s_aux"]
    assert len(f.returns) == 4


def test_fake_shapes():
    with FakeTensorMode():
        q = torch.empty(2, 300, 8, 128, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 500, 2, 128, dtype=torch.bfloat16, device="cuda")
        out, lse, p, rng = torch.ops.flash_attn._flash_attn_forward(q, k, k, 0.0, 0.088, True, -1, -1, 0.0, None, False)
        assert out.shape == q.shape and out.dtype == q.dtype
        assert lse.shape == (2, 8, 300) and lse.dtype == torch.float32
        assert p.shape == (0,) and rng.shape == (2,)
        qv = torch.empty(700, 8, 128, dtype=torch.float16, device="cuda")
        kv = torch.empty(900, 2, 128, dtype=torch.float16, device="cuda")
        cu = torch.empty(4, dtype=torch.int32, device="cuda")
        o, l, p, rng = torch.ops.flash_attn2_c_op.varlen_fwd(qv, kv, kv, None, cu, cu, None, None, None, None, 300, 400,
                                                              0.0, 0.088, False, True, -1, -1, 0.0, False)
        assert o.shape == qv.shape and l.shape == (8, 700) and l.dtype == torch.float32
        qd = torch.empty(4, 1, 8, 128, dtype=torch.bfloat16, device="cuda")
        kc = torch.empty(64, 256, 2, 128, dtype=torch.bfloat16, device="cuda")
        sl = torch.empty(4, dtype=torch.int32, device="cuda")
        bt = torch.empty(4, 16, dtype=torch.int32, device="cuda")
        o, l = torch.ops.flash_attn2_c_op.fwd_kvcache(qd, kc, kc, None, None, sl, None, None, None, None, bt, None, None,
                                                      0.088, True, -1, -1, 0.0, True, 0)
        assert o.shape == qd.shape and l.shape == (4, 8, 1)
