"""GPU: the reference project's OWN Python interface (flash_attn/flash_attn_interface.py of the reference tree) running
unchanged over this repository's binding module ``flash_attn_2_cuda`` — the drop-in swap at the module boundary.

The reference tree is not part of this repository: the test runs where ``FA_REFERENCE_ROOT`` names a checkout of it
(or of just that one file at ``<root>/flash_attn/flash_attn_interface.py``) and is skipped elsewhere.  A child process
loads the reference file by path with this repository's ``flash_attn_2_cuda`` importable and the Triton-based helper
module it imports (``flash_attn.utils.sparse_utils``) replaced by an empty stand-in, calls its ``flash_attn_func``,
``flash_attn_varlen_func``, ``flash_attn_with_kvcache`` and ``sparse_attn_func`` and compares each with the oracle."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-attention-das_b200")
REF = os.environ.get("FA_REFERENCE_ROOT", "")
REF_FILE = os.path.join(REF, "flash_attn", "flash_attn_interface.py") if REF else ""

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF_FILE and os.path.exists(REF_FILE)),
                                 reason="FA_REFERENCE_ROOT does not name a checkout of the reference project")]

_CHILD = textwrap.dedent('''
    import importlib.util, sys, types
    # only the binding module of this repository is importable; the reference interface is loaded from its own tree
    sys.path.insert(0, %(pkg)r)
    sys.path.insert(0, %(root)r)
    import torch
    import flash_attn_2_cuda                      # this repository's binding: defines the flash_attn2_c_op ops
    fa_pkg = types.ModuleType("flash_attn"); fa_pkg.__path__ = []
    utils = types.ModuleType("flash_attn.utils"); utils.__path__ = []
    su = types.ModuleType("flash_attn.utils.sparse_utils")    # Triton helpers the four entry points do not use
    for n in ("get_block_map_meansim", "block_map_to_block_offset_triton", "get_block_map", "get_block_map_fast"):
        setattr(su, n, None)
    sys.modules.update({"flash_attn": fa_pkg, "flash_attn.utils": utils, "flash_attn.utils.sparse_utils": su})
    spec = importlib.util.spec_from_file_location("flash_attn.flash_attn_interface", %(ref_file)r)
    ref = importlib.util.module_from_spec(spec)
    sys.modules["flash_attn.flash_attn_interface"] = ref
    spec.loader.exec_module(ref)
    assert ref.flash_attn_cuda is flash_attn_2_cuda

    from oracle import attention_oracle as O
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
    err = lambda a, b: (a.float().cpu() - b.float()).abs().max().item()
    dev = "cuda"
    with torch.no_grad():
        # flash_attn_func (fixed length, causal GQA)
        q, k, v = rn(2, 256, 8, 128), rn(2, 256, 2, 128), rn(2, 256, 2, 128)
        out = ref.flash_attn_func(q.to(dev), k.to(dev), v.to(dev), causal=True)
        r, _ = O.attention_ref(q, k, v, causal=True, out_dtype=torch.float32)
        assert err(out, r) < 2e-2, ("flash_attn_func", err(out, r))
        # flash_attn_varlen_func (packed)
        lens = [200, 77, 384]
        cu = torch.tensor([0, 200, 277, 661], dtype=torch.int32)
        q, k, v = rn(661, 8, 128), rn(661, 2, 128), rn(661, 2, 128)
        out = ref.flash_attn_varlen_func(q.to(dev), k.to(dev), v.to(dev), cu.to(dev), cu.to(dev), 384, 384, causal=True)
        r, _ = O.attention_varlen_ref(q, k, v, cu, cu, causal=True, out_dtype=torch.float32)
        assert err(out, r) < 2e-2, ("flash_attn_varlen_func", err(out, r))
        # flash_attn_with_kvcache (paged decode)
        lens, page, hk = [700, 64, 1300], 64, 2
        nblk = [(L + page - 1) // page for L in lens]
        kc, vc = rn(sum(nblk), page, hk, 128), rn(sum(nblk), page, hk, 128)
        bt = torch.full((3, max(nblk)), 0, dtype=torch.int32)
        p = 0
        for i, n in enumerate(nblk):
            bt[i, :n] = torch.arange(p, p + n, dtype=torch.int32); p += n
        sl = torch.tensor(lens, dtype=torch.int32)
        q = rn(3, 1, 8, 128)
        out = ref.flash_attn_with_kvcache(q.to(dev), kc.to(dev), vc.to(dev), cache_seqlens=sl.to(dev), block_table=bt.to(dev),
                                          causal=True)
        r, _ = O.paged_decode_ref(q, kc, vc, sl, bt, out_dtype=torch.float32)
        assert err(out, r) < 2e-2, ("flash_attn_with_kvcache", err(out, r))
        # sparse_attn_func (tile lists)
        S, h = 512, 4
        tm = torch.rand(1, h, S // 64, S // 128, generator=g) < 0.5
        tm[..., 0] = True
        cnt, offs = O.tile_mask_to_block_lists(tm, block_m=64, block_n=64, tile_n=128)
        q, k, v = rn(1, S, h, 128), rn(1, S, 2, 128), rn(1, S, 2, 128)
        cc = torch.zeros(1, h, S // 64, dtype=torch.int32, device=dev)
        ci = torch.zeros(1, h, S // 64, 1, dtype=torch.int32, device=dev)
        out = ref.sparse_attn_func(q.to(dev), k.to(dev), v.to(dev), cnt.to(dev), offs.to(dev), cc, ci, causal=False)
        r, _ = O.sparse_attention_ref(q.float(), k.float(), v.float(), cnt, offs, False, 64)
        assert err(out, r) < 2e-2, ("sparse_attn_func", err(out, r))
    torch.cuda.synchronize()
    assert flash_attn_2_cuda.device_status() == 0
    print("REFERENCE-INTERFACE-OK", flash_attn_2_cuda.launch_count())
''')


def test_reference_python_interface_runs_over_this_binding():
    code = _CHILD % {"pkg": PKG, "root": ROOT, "ref_file": REF_FILE}
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "REFERENCE-INTERFACE-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
