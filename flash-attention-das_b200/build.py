"""Build libfa_b200.so (sm_100a only) in-tree with nvcc.  Usage: python build.py [--force] [--verbose] [--test-hooks]

--test-hooks builds libfa_b200_testhooks.so beside it: the same sources with -DFA_B200_TEST_HOOKS (device-side waits
give up after about a millisecond, and one entry lets a launch withhold a tile load).  Only the failure-detection
tests load that library; the product never does."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libfa_b200.so")
OUT_HOOKS = os.path.join(HERE, "libfa_b200_testhooks.so")
SOURCES = ["fa_api.cu", "fa_combine.cu", "fa_decode.cu", "fa_prefill.cu", "fa_prefill_pair.cu", "fa_prefill_dense.cu", "fa_kv_append.cu", "fa_glue.cu", "fa_block_select.cu", "fa_exchange.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(os.path.dirname(HERE), "include", "fa_b200.h"))
    return files


def needs_build(out=OUT):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(f) > t for f in _deps())


def build(force=False, verbose=False, test_hooks=False):
    out = OUT_HOOKS if test_hooks else OUT
    if not force and not needs_build(out):
        return out
    objdir = os.path.join(HERE, "build", "testhooks" if test_hooks else "")
    os.makedirs(objdir, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    if test_hooks:
        extra.append("-DFA_B200_TEST_HOOKS")

    def compile_one(src):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [NVCC, *FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=6) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [NVCC, "-shared", "-o", out, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, test_hooks="--test-hooks" in sys.argv))
