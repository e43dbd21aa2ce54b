"""CPU: the C-ABI library loads and exports every symbol that include/fa_b200.h declares; host-side argument
validation returns status codes without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def binding():
    import importlib.util
    spec = importlib.util.spec_from_file_location("_fa_build", os.path.join(ROOT, "flash-attention-das_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build()
    import flash_attn_2_cuda
    return flash_attn_2_cuda


def test_every_declared_symbol_is_exported(binding):
    hdr = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    names = re.findall(r"FA_B200_API\s+[\w\s\*]+?\b(fa_b200_\w+)\s*\(", hdr)
    assert len(names) >= 11
    lib = binding.lib()
    for n in names:
        assert hasattr(lib, n), n
    assert lib.fa_b200_abi_version() == 2


def test_struct_sizes_match_header(binding):
    # field counts guard against the ctypes mirrors drifting from the header
    hdr = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    for struct, cls in (("fa_b200_fwd_params", binding.FwdParams), ("fa_b200_decode_params", binding.DecodeParams),
                        ("fa_b200_combine_params", binding.CombineParams),
                        ("fa_b200_kv_append_params", binding.KvAppendParams),
                        ("fa_b200_exchange_params", binding.ExchangeParams)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), hdr, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for stmt in body.split(";"):
            stmt = stmt.strip()
            if not stmt:
                continue
            stmt = re.sub(r"\[\w+\]", "", stmt)       # array fields: the name without its extent
            fields += [re.findall(r"(\w+)\s*$", x.strip())[0] for x in stmt.split(",")]
        assert fields == [f[0] for f in cls._fields_], struct


def test_a_struct_of_another_size_is_refused(binding):
    """Every parameter struct starts with its own size: a caller built against another header version (a shorter or a
    longer struct) is told so before any other field is read."""
    lib = binding.lib()
    calls = ((binding.FwdParams, lib.fa_b200_fwd), (binding.FwdParams, lib.fa_b200_fwd_sparse),
             (binding.DecodeParams, lib.fa_b200_decode_paged), (binding.DecodeParams, lib.fa_b200_decode_paged_static),
             (binding.CombineParams, lib.fa_b200_combine), (binding.KvAppendParams, lib.fa_b200_kv_append),
             (binding.ExchangeParams, lib.fa_b200_exchange_combine))
    for cls, fn in calls:
        p = cls()
        assert p.struct_size == ctypes.sizeof(cls)
        for wrong in (0, p.struct_size - 8, p.struct_size + 8):
            p.struct_size = wrong
            assert fn(ctypes.byref(p), None) == 16, (cls.__name__, wrong)
    d = binding.DecodeParams()
    d.struct_size = 8
    assert lib.fa_b200_decode_workspace_bytes(ctypes.byref(d)) == 0
    assert lib.fa_b200_decode_partition_tokens(ctypes.byref(d)) == 0
    assert b"struct_size" in lib.fa_b200_status_string(16)


def test_launch_description_is_empty_before_any_call(binding):
    assert binding.last_launch_info() == "" or binding.last_launch_info().startswith("fa_b200 ")
    binding.set_print_param(False)
    binding.set_print_param(None)


def test_status_strings(binding):
    lib = binding.lib()
    assert lib.fa_b200_status_string(0) == b"ok"
    assert b"128" in lib.fa_b200_status_string(3)
    assert lib.fa_b200_status_string(99) == b"unknown status"


def test_host_validation_needs_no_gpu(binding):
    lib = binding.lib()
    assert lib.fa_b200_fwd(None, None) == 1
    p = binding.FwdParams()
    p.d = 96
    assert lib.fa_b200_fwd(ctypes.byref(p), None) == 3          # head dim
    p.d, p.dtype = 64, 2
    assert lib.fa_b200_fwd(ctypes.byref(p), None) == 3          # 64 / 192 / 256 are for the 16-bit types
    p.d, p.dtype, p.out_dtype = 128, 7, 1
    assert lib.fa_b200_fwd(ctypes.byref(p), None) == 2          # dtype
    p.dtype, p.b, p.h, p.h_k, p.seqlen_q, p.seqlen_k = 1, 1, 6, 4, 8, 8
    assert lib.fa_b200_fwd(ctypes.byref(p), None) == 4          # heads
    d = binding.DecodeParams()
    d.d, d.dtype, d.out_dtype, d.b, d.h, d.h_k, d.page_size, d.max_blocks_per_seq = 128, 1, 1, 2, 8, 2, 48, 4
    assert lib.fa_b200_decode_paged(ctypes.byref(d), None) == 7  # page size
    d.page_size = 256
    d.h = 64
    assert lib.fa_b200_decode_paged(ctypes.byref(d), None) == 4  # group of 32 > 16
    d.h = 8
    assert lib.fa_b200_decode_paged(ctypes.byref(d), None) == 1  # null pointers
    a = binding.KvAppendParams()
    assert lib.fa_b200_kv_append(None, None) == 1
    a.d, a.dtype, a.b, a.seqlen_q, a.seqlen_new, a.h, a.h_k, a.page_size = 128, 1, 2, 1, 1, 8, 2, 64
    a.rotary_dim = 24
    assert lib.fa_b200_kv_append(ctypes.byref(a), None) == 6     # rotary_dim not a multiple of 16
    a.rotary_dim, a.dtype = 32, 2
    assert lib.fa_b200_kv_append(ctypes.byref(a), None) == 9     # no rotary on e4m3
    a.dtype = 1
    assert lib.fa_b200_kv_append(ctypes.byref(a), None) == 1     # null pointers
    assert b"out-of-range" in lib.fa_b200_status_string(14)


def test_partition_heuristic_and_workspace(binding):
    lib = binding.lib()
    d = binding.DecodeParams()
    d.d, d.dtype, d.out_dtype = 128, 1, 1
    d.b, d.h, d.h_k, d.page_size, d.max_blocks_per_seq = 64, 32, 8, 256, 128
    part = lib.fa_b200_decode_partition_tokens(ctypes.byref(d))
    assert part == 8192                     # 64 x 8 rows x 4 partitions = 2048 CTAs: about four rounds of the CTA slots
    nparts = (128 * 256 + part - 1) // part
    assert lib.fa_b200_decode_workspace_bytes(ctypes.byref(d)) == nparts * 64 * 32 * 129 * 4
    d.b, d.max_blocks_per_seq = 2, 1      # one page per sequence: no split, no scratch
    assert lib.fa_b200_decode_workspace_bytes(ctypes.byref(d)) == 0
    d.b, d.max_blocks_per_seq = 1, 4096   # one sequence of 1,048,576 tokens: equal partitions, one round of CTAs
    assert lib.fa_b200_decode_partition_tokens(ctypes.byref(d)) == 32768
    d.b, d.max_blocks_per_seq, d.dtype = 128, 32, 2   # e4m3, batch 128 x 8192
    assert lib.fa_b200_decode_partition_tokens(ctypes.byref(d)) == 4096
    d.dtype = 1
    d.partition_tokens = 100               # not a multiple of the tile
    assert lib.fa_b200_decode_partition_tokens(ctypes.byref(d)) == 0


def test_raw_pointer_entry_validates_before_touching_anything(binding):
    """fa_b200_kv_cache_attention (the reference's extern "C" kv_cache_attention argument list): argument errors come back
    as status codes without a GPU, and its workspace query agrees with the decode call's."""
    lib = binding.lib()

    def call(dtype=1, layout=1, num_query=4, num_tokens=4, hq=8, hk=2, d=128, pages=16, page=64, max_k=512):
        return lib.fa_b200_kv_cache_attention(None, None, 1, max_k, None, None, None, None, None, num_query, num_tokens, hq,
                                              hk, d, pages, page, dtype, layout, None, 0, None)
    assert call(dtype=2) == 2            # e4m3 is not taken by this entry
    assert call(layout=3) == 9
    assert call(d=96) == 3
    assert call(num_tokens=3) == 6       # fewer tokens than requests
    assert call(num_query=0, num_tokens=0) == 0
    assert call(hq=6, hk=4) == 4         # reaches the decode call's own checks
    assert call() == 1                   # null pointers
    assert call(num_tokens=9, layout=0, d=64) == 3   # a transposed V pool: head dimension 128 only
    assert call(num_tokens=9) == 1       # seq_offsets missing
    d = binding.DecodeParams()
    d.d, d.dtype, d.out_dtype = 128, 1, 1
    d.b, d.h, d.h_k, d.page_size, d.max_blocks_per_seq, d.max_seqlen_k = 64, 32, 8, 256, 128, 32768
    assert (lib.fa_b200_kv_cache_attention_workspace_bytes(64, 32, 8, 128, 256, 32768) ==
            lib.fa_b200_decode_workspace_bytes(ctypes.byref(d)) > 0)


def test_block_selection_entries_validate(binding):
    lib = binding.lib()
    assert lib.fa_b200_block_pool(None, 2, 0, 0, 0, 1, 1, 128, 128, 64, None, None, None, None) == 2      # e4m3
    assert lib.fa_b200_block_pool(None, 1, 0, 0, 0, 1, 1, 128, 96, 64, None, None, None, None) == 3       # head dim
    assert lib.fa_b200_block_pool(None, 1, 0, 0, 0, 1, 1, 128, 128, 256, None, None, None, None) == 6     # block too tall
    assert lib.fa_b200_block_pool(None, 1, 0, 0, 0, 0, 1, 128, 128, 64, None, None, None, None) == 0      # empty batch
    assert lib.fa_b200_block_pool(None, 1, 0, 0, 0, 1, 1, 128, 128, 64, None, None, None, None) == 1      # null pointers
    sel = lambda nk=8, cdf=None, topk=None: lib.fa_b200_block_select(None, None, None, None, 1, 1, 1, 4, nk, 128, 128, 64,
                                                                      ctypes.c_float(0.1), cdf, topk, 0, 0, None, None)
    assert sel() == 9                      # neither a cdf threshold nor a top-k fraction
    assert sel(nk=5000, cdf=1) == 13       # more key blocks than the in-kernel sort takes
    assert sel(cdf=1) == 1                 # null pointers


def test_exchange_entries_validate_before_touching_anything(binding):
    """The multi-GPU exchange: buffer sizes are host arithmetic, and a call with a bad shape, epoch 0, a rank outside
    the world or a missing peer pointer is refused with a status before any CUDA call."""
    lib = binding.lib()
    assert lib.fa_b200_exchange_bytes(0, 32, 128) == 0 and lib.fa_b200_exchange_bytes(8, 0, 128) == 0
    n = lib.fa_b200_exchange_bytes(8, 32, 128)
    assert n >= 2 * 8 * 32 * (128 + 2) * 4 and n % 512 == 0          # two halves, each a multiple of 256 bytes
    p = binding.ExchangeParams()
    p.world, p.rank, p.rows, p.h, p.seqlen_q, p.d, p.epoch = 2, 0, 32, 32, 1, 128, 1
    p.do_push = p.do_wait = 1
    NULL, SHAPE = 1, 6
    assert lib.fa_b200_exchange_combine(ctypes.byref(p), None) == NULL       # no partial, no peers
    p.o_local = p.lse_local = 4096
    assert lib.fa_b200_exchange_combine(ctypes.byref(p), None) == NULL       # peers missing
    p.peers[0] = p.peers[1] = 4096
    for field, bad in (("epoch", 0), ("rank", 2), ("world", 17), ("d", 126), ("rows", 33)):
        q = binding.ExchangeParams.from_buffer_copy(p)
        setattr(q, field, bad)
        assert lib.fa_b200_exchange_combine(ctypes.byref(q), None) == SHAPE, field
