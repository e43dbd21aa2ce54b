#!/usr/bin/env python
"""Benchmark of the B200 attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The headline workload is the
paged-KV bf16 decode configuration (batch 64, context 1024..32768, page 256, 32/8 heads, d 128): `value` is whole-job
HBM GB/s of ALGORITHMIC bytes (KV bytes read once + q/out + block table) with the cache resident in HBM; `e2e` is the
same metric through the public Python API with the step's inputs (q, cache_seqlens, block_table) coming from pinned
host memory and the output read back to the host inside the timed region, every step; the decode and prefill
workloads run those steps as a serving loop would, on three streams with two sets of device buffers, so that one
step's copies overlap its neighbours' attention.  The other configurations are timed in the same run and reported under
`also`: varlen causal prefill bf16 (TFLOP/s, reference FLOP convention 4*S^2*H*D/2 per sequence), e4m3 decode and
prefill, block-sparse prefill and the single 1,048,576-token decode.  Every entry carries a `check`: the maximum
absolute error of the timed call's output against the fp32 oracle on a stated subset, computed outside the timed region.

Multi-GPU (torchrun, one rank per GPU): the SAME configurations, sharded over the ranks with no data-path collective
("strong" scaling: the total work is fixed, value = total algorithmic bytes or FLOPs / the slowest rank's step time
between two barriers): decode batches by sequence (longest-processing-time on the lengths), prefill over a
(sequence group, kv-head group) grid, block-sparse prefill by kv head; each rank builds only its own shard.  The one
case with an exchange step is the single 1,048,576-token sequence, split-KV across the ranks by page range: the partial
(O, LSE) are all-gathered with NCCL before the combine kernel (its three phases are also timed one by one).  The
whole-batch-per-rank figure ("weak" scaling) is kept under `also` as `decode_bf16_replica`.
`--shard-of W [--shard-rank R]` runs rank R's share of a W-way job on one GPU without any collective (sizing a shard
without the machine that would run it).

`--impl reference` times the CPU oracle (the reference's PyTorch attention restated in oracle/) on the host
cores over a bounded sample of the same workload; under torchrun only rank 0 runs it.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flash-attention-das_b200")
for _p in (PKG, ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

H, HK, D = 32, 8, 128
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, as a multiple of the
# algorithmic bytes, from the ncu captures summarised under profiles/ (None = not captured yet).
# decode: measured on a quarter of the batch (traffic grows in proportion to the tokens streamed).
TRAFFIC_RATIO = {"decode_bf16": 1.007, "decode_bf16_replica": 1.007, "decode_fp8": 1.013, "prefill_bf16": None,
                 "prefill_fp8": None, "sparse_bf16": None, "longseq": 1.007}
# prefill is tensor-bound, its algorithmic unit is FLOPs; DRAM traffic is reported in bytes per token of the
# captured case: bf16 526.2 MB for 19,679 tokens (1.31x the compulsory q+k+v+out bytes), e4m3 188.7 MB for
# 4 x 4096 tokens (0.80x: a third of the 134 MB bf16 output is still in L2 when the launch ends),
# block-sparse 0.406 GB read + 0.238 GB written for the full configuration's 32,768 tokens.
PREFILL_TRAFFIC_BYTES_PER_TOKEN = {"prefill_bf16": 526.2e6 / 19679, "prefill_fp8": 188.7e6 / 16384,
                                   "sparse_bf16": 0.6447e9 / 32768}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["source"] = "fallback"
    return d


# --------------------------------------------------------------------------------------------------
# clocks sampler
# --------------------------------------------------------------------------------------------------
_NVML_POLLER = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
uuid = sys.argv[1]
try:
    h = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
except Exception:
    h = nv.nvmlDeviceGetHandleByIndex(int(sys.argv[2]))
print("max", nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
while True:
    try:
        print(time.monotonic_ns(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
              nv.nvmlDeviceGetCurrentClocksEventReasons(h), flush=True)
    except Exception:
        pass
    time.sleep(0.001)
"""


class ClockSampler:
    """SM clock and throttle reasons sampled DURING the timed region.  A child process polls NVML every
    millisecond (a thread of this process would starve behind the launch loop, and one nvidia-smi call lasts longer
    than a whole timed region); the samples whose monotonic timestamp falls inside the region are summarised."""
    REASON_BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index, enabled=True):
        self.index = index
        self.proc = None
        self.t0 = self.t1 = 0
        if not enabled or os.environ.get("FA_B200_BENCH_NO_CLOCKS"):
            return
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
            self.proc = subprocess.Popen([sys.executable, "-c", _NVML_POLLER, uuid, str(index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.3)   # let the poller come up before the region starts
        except Exception:
            self.proc = None

    def __enter__(self):
        self.t0 = time.monotonic_ns()
        return self

    def __exit__(self, *a):
        self.t1 = time.monotonic_ns()

    def summary(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": "none"}
        time.sleep(0.01)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm_max, sm, bits = None, [], 0
        for line in out.splitlines():
            parts = line.split()
            if len(parts) == 2 and parts[0] == "max":
                sm_max = int(parts[1])
            elif len(parts) == 3:
                t, clk, r = int(parts[0]), int(parts[1]), int(parts[2])
                if self.t0 <= t <= self.t1:
                    sm.append(clk)
                    bits |= r
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": sm_max, "reasons": [], "samples": 0, "source": "nvml"}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": sm_max,
                "reasons": [n for n, b in self.REASON_BITS.items() if bits & b], "samples": len(sm), "source": "nvml"}


# --------------------------------------------------------------------------------------------------
# workloads (seeded synthetic data, shapes of the baseline configurations)
# --------------------------------------------------------------------------------------------------
def _cuda_gen(dev, seed):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return g


def _randn_into(t, g, chunk=1 << 26):
    flat = t.view(-1)
    for i in range(0, flat.numel(), chunk):
        n = min(chunk, flat.numel() - i)
        flat[i:i + n] = torch.randn(n, generator=g, device=t.device, dtype=torch.float32).to(t.dtype)


class E2EPipeline:
    """End-to-end steps as a serving loop would run them: three streams (host->device copies, the attention call,
    device->host copy of the result) and two sets of device buffers, so that the copies of one step overlap the
    attention of its neighbours.  Every step still moves its own inputs from pinned host memory and its own result
    back; ``begin`` / ``end`` tie the three streams to the stream the timing events are recorded on."""

    def __init__(self, dev):
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_run = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.i = 0

    def begin(self):
        cur = torch.cuda.current_stream()
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_stream(cur)

    def end(self):
        cur = torch.cuda.current_stream()
        for st in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(st)

    def step(self, copy_in, run, copy_out):
        """copy_in(buf), run(buf), copy_out(buf) are issued on their streams for buffer set buf = step parity."""
        buf = self.i & 1
        first_use = self.i < 2
        self.i += 1
        with torch.cuda.stream(self.s_in):
            if not first_use:
                self.s_in.wait_event(self.ev_run[buf])     # the attention that read these inputs two steps ago
            copy_in(buf)
            self.ev_in[buf].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[buf])
            if not first_use:
                self.s_run.wait_event(self.ev_out[buf])    # the result buffer has been read back
            run(buf)
            self.ev_run[buf].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[buf])
            copy_out(buf)
            self.ev_out[buf].record(self.s_out)


def _shard_helpers():
    from flash_attn import split_kv_parallel
    return split_kv_parallel


def _err(a, b):
    return float((a.float() - b.float()).abs().max().item())


def decode_config(cg, fp8, batch, page, shard):
    """Lengths of this rank's sequences and the `config` object of a decode workload (no device needed: the reference
    arm describes the same configuration)."""
    if fp8:
        batch = batch or 128
        all_lens = torch.full((batch,), 8192, dtype=torch.int64)
    else:
        batch = batch or 64
        all_lens = torch.randint(1024, 32769, (batch,), generator=cg)
    rank, world = shard
    owned = _shard_helpers().shard_sequences_lpt(all_lens.tolist(), world)[rank]
    lens = all_lens[owned]
    pool = int(((lens + page - 1) // page).sum())
    es = 1 if fp8 else 2
    # algorithmic bytes: every K and V byte once + q + out + the used block-table entries
    units = float(int(lens.sum()) * HK * D * 2 * es + len(lens) * H * D * (es + 2) + 4 * pool)
    desc = {"workload": ("paged-KV decode e4m3: batch %d x context 8192" % batch) if fp8 else
            "paged-KV decode bf16: batch %d, context uniform[1024,32768]" % batch,
            "page_block_size": page, "nheads": H, "nheads_kv": HK, "headdim": D,
            "sharding": "by sequence, longest-processing-time on the lengths: %d of %d sequences on rank %d of %d" %
                        (len(lens), batch, rank, world),
            "tokens": int(lens.sum()), "l2": "inputs larger than L2 (KV pool of this rank %.2f GB)" % (units / 1e9)}
    return lens, units, desc


class DecodeWorkload:
    """Paged-KV decode: batch of single-token queries over a paged pool; block_table is a seeded random
    permutation of the pool.  `shard` = (rank, world): this rank's sequences of the batch (LPT on the lengths)."""

    def __init__(self, dev, seed, fp8=False, batch=None, page=256, shard=(0, 1), data_rank=0, name=None):
        import flash_attn
        self.fa = flash_attn
        self.fp8 = fp8
        self.name = name or ("decode_fp8" if fp8 else "decode_bf16")
        cg = torch.Generator().manual_seed(seed)
        rank, world = shard
        lens, self.units, self.desc = decode_config(cg, fp8, batch, page, shard)
        self.lens = lens
        self.batch = len(lens)
        self.page = page
        nblk = (lens + page - 1) // page
        pool = int(nblk.sum())
        perm = torch.randperm(pool, generator=cg).to(torch.int32)
        bt = torch.full((self.batch, int(nblk.max())), -1, dtype=torch.int32)
        p = 0
        for i, n in enumerate(nblk.tolist()):
            bt[i, :n] = perm[p:p + n]
            p += n
        dg = _cuda_gen(dev, seed + 1 + 1000 * (rank + data_rank))
        dt = torch.bfloat16
        self.kc = torch.empty(pool, page, HK, D, dtype=dt, device=dev)
        self.vc = torch.empty(pool, page, HK, D, dtype=dt, device=dev)
        _randn_into(self.kc, dg)
        _randn_into(self.vc, dg)
        self.q_host = torch.randn(self.batch, 1, H, D, generator=cg).to(dt).pin_memory()
        self.kw = {}
        if fp8:
            amax_k, amax_v = self.kc.abs().max().float(), self.vc.abs().max().float()
            kd, vd = (amax_k / 448.0).reshape(1), (amax_v / 448.0).reshape(1)
            self.kc = (self.kc.float() / kd).to(torch.float8_e4m3fn)
            self.vc = (self.vc.float() / vd).to(torch.float8_e4m3fn)
            qd = (self.q_host.float().abs().max() / 448.0).reshape(1)
            self.q_host = (self.q_host.float() / qd).to(torch.float8_e4m3fn).pin_memory()
            self.kw = dict(q_descale=qd.to(dev), k_descale=kd, v_descale=vd)
        self.bt_host = bt.pin_memory()
        self.sl_host = lens.to(torch.int32).pin_memory()
        self.q = self.q_host.to(dev)
        self.bt = self.bt_host.to(dev)
        self.sl = self.sl_host.to(dev)
        self.out_host = torch.empty(self.batch, 1, H, D, dtype=torch.bfloat16).pin_memory()
        es = 1 if fp8 else 2
        self.unit_name = "bytes"
        self.h2d = self.q_host.numel() * es + self.bt_host.numel() * 4 + self.sl_host.numel() * 4
        self.d2h = self.out_host.numel() * 2

    def step(self):
        return self.fa.flash_attn_with_kvcache(self.q, self.kc, self.vc, cache_seqlens=self.sl, block_table=self.bt,
                                               causal=True, **self.kw)

    def check(self):
        """Timed call's output against the fp32 oracle evaluated on the device for the shortest, the longest and the
        middle sequence of this rank's shard."""
        from oracle import attention_oracle as O
        out = self.step()
        order = torch.argsort(self.lens)
        picks = sorted({int(order[0]), int(order[-1]), int(order[len(order) // 2])})
        worst = 0.0
        for b in picks:
            kw = {k: v.reshape(1, 1).expand(1, HK) for k, v in self.kw.items()}
            ref, _ = O.paged_decode_ref(self.q[b:b + 1], self.kc, self.vc, self.sl[b:b + 1], self.bt[b:b + 1],
                                        out_dtype=torch.float32, **kw)
            worst = max(worst, _err(out[b:b + 1], ref))
        tol = 7e-2 if self.fp8 else 1e-2
        return {"max_abs_err": worst, "tolerance": tol, "ok": worst <= tol,
                "subset": "%d of this rank's %d sequences (shortest, middle, longest), all heads; oracle in fp32 on the device" %
                          (len(picks), self.batch)}

    def e2e_setup(self):
        dev = self.q.device
        self.pipe = E2EPipeline(dev)
        self.d_q = [torch.empty_like(self.q) for _ in range(2)]
        self.d_bt = [torch.empty_like(self.bt) for _ in range(2)]
        self.d_sl = [torch.empty_like(self.sl) for _ in range(2)]
        self.d_out = [torch.empty(self.batch, 1, H, D, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.out_hosts = [self.out_host, torch.empty_like(self.out_host).pin_memory()]

    def step_e2e(self):
        def copy_in(b):
            self.d_q[b].copy_(self.q_host, non_blocking=True)
            self.d_bt[b].copy_(self.bt_host, non_blocking=True)
            self.d_sl[b].copy_(self.sl_host, non_blocking=True)

        def run(b):
            self.fa.flash_attn_with_kvcache(self.d_q[b], self.kc, self.vc, cache_seqlens=self.d_sl[b], block_table=self.d_bt[b],
                                            causal=True, out=self.d_out[b], **self.kw)

        def copy_out(b):
            self.out_hosts[b].copy_(self.d_out[b], non_blocking=True)

        self.pipe.step(copy_in, run, copy_out)


L2_MB = 126.0


def _rotating_copies(tensors, in_mb):
    """Inputs of a step that are not larger than L2 (a shard of a configuration on one of several GPUs) are kept in
    several identical copies used in turn, enough of them that the copies together are three times the size of L2: when a
    copy comes round again it has long been evicted, which is what an L2 flush between steps would achieve, without a
    flush inside the timed region."""
    n = 1 if in_mb > L2_MB else int(3 * L2_MB // in_mb) + 1
    return [tensors] + [tuple(t.clone() for t in tensors) for _ in range(n - 1)]


def _l2_note(in_mb, copies):
    if copies == 1:
        return "inputs larger than L2 (q+k+v of this rank %.0f MB)" % in_mb
    return ("q+k+v of this rank are %.0f MB, not larger than L2: %d identical copies are used in turn (%.0f MB together), "
            "so a step's inputs were last touched %d steps earlier" % (in_mb, copies, in_mb * copies, copies))


class PrefillWorkload:
    """Packed varlen causal GQA prefill.  `shard` = (rank, world): this rank's cell of the (sequence group, kv-head
    group) grid."""

    def __init__(self, dev, seed, fp8=False, nseq=None, shard=(0, 1)):
        import flash_attn
        self.fa = flash_attn
        self.fp8 = fp8
        self.name = "prefill_fp8" if fp8 else "prefill_bf16"
        cg = torch.Generator().manual_seed(seed)
        nseq = nseq or (8 if fp8 else 16)
        all_lens = torch.full((nseq,), 4096, dtype=torch.int64) if fp8 else torch.randint(512, 4097, (nseq,), generator=cg)
        rank, world = shard
        sg, hg, owned = _shard_helpers().shard_prefill_grid(all_lens.tolist(), HK, world)
        lens = all_lens[owned[rank // hg]]
        self.h, self.hk = H // hg, HK // hg
        self.lens = lens
        total = int(lens.sum())
        dg = _cuda_gen(dev, seed + 1 + 1000 * rank)
        mk = lambda h: torch.randn(total, h, D, generator=dg, device=dev, dtype=torch.float32).to(torch.bfloat16)
        q, k, v = mk(self.h), mk(self.hk), mk(self.hk)
        self.kw = {}
        if fp8:
            qd, kd, vd = [(t.abs().max().float() / 448.0).reshape(1) for t in (q, k, v)]
            q, k, v = [(t.float() / s).to(torch.float8_e4m3fn) for t, s in ((q, qd), (k, kd), (v, vd))]
            self.kw = dict(q_descale=qd, k_descale=kd, v_descale=vd)
        self.q, self.k, self.v = q, k, v
        self.cu_host = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32).pin_memory()
        self.cu = self.cu_host.to(dev)
        self.maxlen = int(lens.max())
        self.q_host, self.k_host, self.v_host = [t.cpu().pin_memory() for t in (q, k, v)]
        self.out_host = torch.empty(total, self.h, D, dtype=torch.bfloat16).pin_memory()
        # reference FLOP convention: 4 * S^2 * H * D / 2 per causal sequence (benchmarks/benchmark_attnmask.py:24-30)
        self.units = float((4 * lens.double() ** 2 * self.h * D / 2).sum())
        self.unit_name = "flops"
        es = 1 if fp8 else 2
        self.h2d = (q.numel() + k.numel() + v.numel()) * es + self.cu_host.numel() * 4
        self.d2h = self.out_host.numel() * 2
        self.desc = {"workload": ("varlen causal prefill e4m3: %d x 4096" % nseq if fp8 else
                                  "varlen causal GQA prefill bf16: %d sequences, length uniform[512,4096]" % nseq),
                     "nheads": H, "nheads_kv": HK, "headdim": D,
                     "sharding": "%d sequence group(s) (LPT on length^2) x %d kv-head group(s): rank %d of %d has %d sequences, "
                                 "%d query / %d kv heads" % (sg, hg, rank, world, len(lens), self.h, self.hk),
                     "tokens": total}
        in_mb = (q.numel() + 2 * k.numel()) * es / 1e6
        self.rot, self.rot_i = _rotating_copies((self.q, self.k, self.v), in_mb), 0
        self.desc["l2"] = _l2_note(in_mb, len(self.rot))

    def step(self):
        q, k, v = self.rot[self.rot_i % len(self.rot)]
        self.rot_i += 1
        return self.fa.flash_attn_varlen_func(q, k, v, self.cu, self.cu, self.maxlen, self.maxlen, causal=True, **self.kw)

    def check(self):
        """The shortest and the longest sequence of this rank, all of its heads, against the fp32 oracle on the device."""
        from oracle import attention_oracle as O
        out = self.step()
        picks = sorted({int(self.lens.argmin()), int(self.lens.argmax())})
        worst, worst_ref = 0.0, 0.0
        for i in picks:
            lo, hi = int(self.cu_host[i]), int(self.cu_host[i + 1])
            kw = {k: v.reshape(1, 1).expand(1, self.hk) for k, v in self.kw.items()}
            ref, _ = O.attention_ref(self.q[lo:hi][None], self.k[lo:hi][None], self.v[lo:hi][None], causal=True,
                                     out_dtype=torch.float32, **kw)
            worst = max(worst, _err(out[lo:hi][None], ref))
            # the tolerance is relative to what the same math gives with P rounded to the input type
            if self.fp8:
                ref_p, _ = O.attention_ref(self.q[lo:hi][None], self.k[lo:hi][None], self.v[lo:hi][None], causal=True,
                                           out_dtype=torch.float32, intermediate_dtype=torch.float8_e4m3fn, **kw)
            else:
                ref_p, _ = O.attention_ref(self.q[lo:hi][None], self.k[lo:hi][None], self.v[lo:hi][None], causal=True,
                                           upcast=False, reorder_ops=True)
            worst_ref = max(worst_ref, _err(ref_p, ref))
            del ref, ref_p
        tol = 2 * worst_ref + (2 ** -7 if self.fp8 else 2 ** -8)
        return {"max_abs_err": worst, "tolerance": tol, "ok": worst <= tol,
                "subset": "%d of this rank's %d sequences (shortest, longest), all of its heads; oracle in fp32 on the device; "
                          "tolerance = 2 x the error of the same math with P in the input type" % (len(picks), len(self.lens))}

    def e2e_setup(self):
        dev = self.q.device
        self.pipe = E2EPipeline(dev)
        self.d_qkv = [[torch.empty_like(t) for t in (self.q, self.k, self.v)] for _ in range(2)]
        self.d_cu = [torch.empty_like(self.cu) for _ in range(2)]
        self.d_out = [torch.empty(self.q.shape[0], self.h, D, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.out_hosts = [self.out_host, torch.empty_like(self.out_host).pin_memory()]

    def step_e2e(self):
        def copy_in(b):
            for dst, src in zip(self.d_qkv[b], (self.q_host, self.k_host, self.v_host)):
                dst.copy_(src, non_blocking=True)
            self.d_cu[b].copy_(self.cu_host, non_blocking=True)

        def run(b):
            q, k, v = self.d_qkv[b]
            self.fa.flash_attn_varlen_func(q, k, v, self.d_cu[b], self.d_cu[b], self.maxlen, self.maxlen, causal=True,
                                           out=self.d_out[b], **self.kw)

        def copy_out(b):
            self.out_hosts[b].copy_(self.d_out[b], non_blocking=True)

        self.pipe.step(copy_in, run, copy_out)


def tile_mask_to_block_lists(tile_mask):
    """(b, h, nq, nk) bool over 128x128 tiles -> block_count (b, h, nq) and block_offset (b, h, nq, NNZ_S) int32:
    ascending K row offsets, two 64-row entries per kept tile, unused slots = a large sentinel (the metadata
    format sparse_attn_func takes)."""
    fine = tile_mask.repeat_interleave(2, dim=-1)
    count = fine.sum(dim=-1).to(torch.int32)
    nnz = max(int(count.max()), 1)
    idx = torch.arange(fine.shape[-1], dtype=torch.int64).expand_as(fine).clone()
    idx[~fine] = 10_000_000
    srt = torch.sort(idx, dim=-1).values[..., :nnz]
    offs = torch.where(srt >= 10_000_000, srt, srt * 64)
    return count, offs.to(torch.int32).contiguous()


class SparseWorkload:
    """Block-sparse causal GQA prefill, one 32768-token sequence, 128x128 tile mask at 25 % density per head
    (diagonal tiles always kept).  `shard` = (rank, world): this rank's kv heads and their query heads."""

    def __init__(self, dev, seed, seqlen=32768, density=0.25, shard=(0, 1)):
        import flash_attn
        self.fa = flash_attn
        self.name = "sparse_bf16"
        rank, world = shard
        if HK % world:
            raise SystemExit("block-sparse prefill shards by kv head: the rank count must divide %d" % HK)
        self.h, self.hk = H // world, HK // world
        cg = torch.Generator().manual_seed(seed)
        n = seqlen // 128
        tm = torch.rand(1, H, n, n, generator=cg) < density
        tril = torch.tril(torch.ones(n, n, dtype=torch.bool))
        tm = (tm & tril) | torch.eye(n, dtype=torch.bool)
        tm = tm[:, rank * self.h:(rank + 1) * self.h].contiguous()
        self.tm = tm
        cnt, offs = tile_mask_to_block_lists(tm)
        self.kept = int(tm.sum())
        dg = _cuda_gen(dev, seed + 1 + 1000 * rank)
        mk = lambda h: torch.randn(1, seqlen, h, D, generator=dg, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.q, self.k, self.v = mk(self.h), mk(self.hk), mk(self.hk)
        self.cnt, self.offs = cnt.to(dev), offs.to(dev)
        self.cc = torch.zeros(1, self.h, n, dtype=torch.int32, device=dev)
        self.ci = torch.zeros(1, self.h, n, 1, dtype=torch.int32, device=dev)
        self.q_host, self.k_host, self.v_host = [t.cpu().pin_memory() for t in (self.q, self.k, self.v)]
        self.cnt_host, self.offs_host = cnt.pin_memory(), offs.pin_memory()
        self.out_host = torch.empty(1, seqlen, self.h, D, dtype=torch.bfloat16).pin_memory()
        # kept tiles x 4*128*128*128 FLOPs, diagonal tiles counted as full tiles
        self.units = float(self.kept) * 4 * 128 * 128 * 128
        self.unit_name = "flops"
        self.h2d = (self.q.numel() + 2 * self.k.numel()) * 2 + (cnt.numel() + offs.numel()) * 4
        self.d2h = self.out_host.numel() * 2
        self.desc = {"workload": "block-sparse causal GQA prefill bf16: 1 x %d, 128x128 tiles at %.0f%% density" %
                     (seqlen, density * 100), "kept_tiles": self.kept, "tokens": seqlen, "nheads": H, "nheads_kv": HK, "headdim": D,
                     "sharding": "by kv head: rank %d of %d has %d query / %d kv heads" % (rank, world, self.h, self.hk),
                     }
        in_mb = (self.q.numel() + 2 * self.k.numel()) * 2 / 1e6
        self.rot, self.rot_i = _rotating_copies((self.q, self.k, self.v), in_mb), 0
        self.desc["l2"] = _l2_note(in_mb, len(self.rot))

    def step(self):
        q, k, v = self.rot[self.rot_i % len(self.rot)]
        self.rot_i += 1
        return self.fa.sparse_attn_func(q, k, v, self.cnt, self.offs, self.cc, self.ci, causal=True)

    def check(self):
        """Whole query tiles (head, q-block) against the fp32 oracle on the device: only the kept key tiles are gathered,
        the causal mask acts inside the diagonal tile (the last kept one)."""
        from oracle import attention_oracle as O
        out = self.step()
        n = self.tm.shape[-1]
        cg = torch.Generator().manual_seed(11)
        pairs = {(0, 0), (self.h - 1, n - 1)}
        while len(pairs) < 12:
            pairs.add((int(torch.randint(0, self.h, (1,), generator=cg)), int(torch.randint(0, n, (1,), generator=cg))))
        worst, worst_ref = 0.0, 0.0
        for head, m in sorted(pairs):
            kept = torch.nonzero(self.tm[0, head, m]).flatten().tolist()
            rows = slice(m * 128, m * 128 + 128)
            hk = head // (self.h // self.hk)
            ks = torch.cat([self.k[0, j * 128:(j + 1) * 128, hk] for j in kept])[None, :, None]
            vs = torch.cat([self.v[0, j * 128:(j + 1) * 128, hk] for j in kept])[None, :, None]
            qs = self.q[0, rows, head][None, :, None]
            mask = torch.zeros(128, len(kept) * 128, dtype=torch.bool, device=qs.device)
            if kept[-1] == m:
                mask[:, -128:] = torch.triu(torch.ones(128, 128, dtype=torch.bool, device=qs.device), diagonal=1)
            ref, _ = O.attention_ref(qs, ks, vs, out_dtype=torch.float32, extra_mask=mask)
            ref_p, _ = O.attention_ref(qs, ks, vs, upcast=False, reorder_ops=True, extra_mask=mask)
            worst = max(worst, _err(out[0, rows, head], ref[0, :, 0]))
            worst_ref = max(worst_ref, _err(ref_p, ref))
        tol = 2 * worst_ref + 2 ** -8
        return {"max_abs_err": worst, "tolerance": tol, "ok": worst <= tol,
                "subset": "%d (head, query block) tiles of this rank, whole tiles; oracle in fp32 on the device" % len(pairs)}

    def step_e2e(self):
        dev = self.q.device
        q, k, v = [t.to(dev, non_blocking=True) for t in (self.q_host, self.k_host, self.v_host)]
        cnt, offs = self.cnt_host.to(dev, non_blocking=True), self.offs_host.to(dev, non_blocking=True)
        out = self.fa.sparse_attn_func(q, k, v, cnt, offs, self.cc, self.ci, causal=True)
        self.out_host.copy_(out, non_blocking=True)
        return out


class LongSeqWorkload:
    """One sequence of 1,048,576 tokens, split-KV across the ranks by page range; each rank decodes its slice to
    an fp32 partial (O, LSE); the partials are all-gathered (NCCL) and combined on every rank."""

    def __init__(self, dev, seed, shard, real_world, total_tokens=1 << 20, page=256):
        import flash_attn_2_cuda
        self.cuda = flash_attn_2_cuda
        self.name = "longseq"
        rank, world = shard
        self.world, self.real_world = world, real_world
        npages = total_tokens // page
        first, last = _shard_helpers().split_page_range(npages, world, rank)
        pool = last - first
        local = pool * page
        cg = torch.Generator().manual_seed(seed)  # same q on every rank
        dg = _cuda_gen(dev, seed + 1 + rank)
        self.kc = torch.empty(pool, page, HK, D, dtype=torch.bfloat16, device=dev)
        self.vc = torch.empty(pool, page, HK, D, dtype=torch.bfloat16, device=dev)
        _randn_into(self.kc, dg)
        _randn_into(self.vc, dg)
        self.q = torch.randn(1, 1, H, D, generator=cg).to(torch.bfloat16).to(dev)
        self.bt = torch.randperm(pool, generator=torch.Generator().manual_seed(seed + 7 + rank)).to(torch.int32).view(1, pool).to(dev)
        self.sl = torch.tensor([local], dtype=torch.int32, device=dev)
        self.units = float(local * HK * D * 2 * 2 + H * D * 4 + 4 * pool)   # this rank's bytes
        self.unit_name = "bytes"
        self.h2d, self.d2h = self.q.numel() * 2, H * D * 2
        self.q_host = self.q.cpu().pin_memory()
        self.out_host = torch.empty(H, D, dtype=torch.bfloat16).pin_memory()
        self.desc = {"workload": "single-sequence %d-token bf16 decode, split-KV across %d GPU(s), NCCL allgather of (O, LSE)" %
                     (total_tokens, world), "page_block_size": page, "nheads": H, "nheads_kv": HK, "headdim": D,
                     "sharding": "by page range: rank %d of %d holds pages [%d, %d)" % (rank, world, first, last),
                     "l2": "inputs larger than L2 (%.2f GB on this rank)" % (self.units / 1e9)}

    def _exchange(self):
        """At more than one rank the partials cross NVLink inside the library's exchange + combine kernel (peer stores
        over CUDA IPC mappings), set up once; FA_B200_BENCH_LONGSEQ=nccl keeps the all-gather + combine pair."""
        if not hasattr(self, "_ex"):
            self._ex = None
            import torch.distributed as dist
            if self.real_world > 1 and dist.is_initialized() and os.environ.get("FA_B200_BENCH_LONGSEQ", "") != "nccl":
                from flash_attn.split_kv_parallel import PartialExchange
                ex, err = None, ""
                try:
                    ex = PartialExchange(H, D, self.q.device)
                except Exception as e:   # e.g. CUDA IPC not permitted between the ranks' processes
                    err = repr(e)
                # every rank must take the same path: the NCCL form unless the set-up worked everywhere
                ok = torch.tensor([1.0 if ex is not None else 0.0], device=self.q.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if float(ok.item()) == 1.0:
                    self._ex = ex
                else:
                    if ex is not None:
                        ex.close()
                    self.exchange_note = "peer-memory exchange not available (%s): NCCL all-gather + combine" % (err or "on another rank")
        return self._ex

    def _run(self, q, events=None, nccl=False):
        from flash_attn.split_kv_parallel import decode_split_across_gpus
        out, _ = decode_split_across_gpus(q, self.kc, self.vc, self.sl, self.bt, D ** -0.5, phase_events=events,
                                          exchange=None if nccl else self._exchange())
        return out

    def step(self):
        return self._run(self.q)

    def check(self):
        """Every rank evaluates the fp32 oracle on kv head 2 (query heads 8..11) of its own slice on the device; the
        partials are all-gathered and merged by the oracle's merge; the kernel path's output (partition kernel, then the
        exchange + combine kernel over peer memory, or NCCL all-gather + combine kernel) is compared with that."""
        from oracle import attention_oracle as O
        from flash_attn.split_kv_parallel import gather_partials
        import torch.distributed as dist
        out = self.step()
        hk, g = 2, H // HK
        pages = self.bt[0].long()
        kk = self.kc[pages, :, hk].reshape(-1, D)[None, :, None]
        vv = self.vc[pages, :, hk].reshape(-1, D)[None, :, None]
        o, l = O.attention_ref(self.q[:, :, hk * g:(hk + 1) * g], kk, vv, out_dtype=torch.float32)
        o, l = o.reshape(g, D).contiguous(), l.reshape(g).contiguous()
        if self.real_world > 1 and dist.is_initialized():
            o_all, l_all = gather_partials(o, l)
        else:
            o_all, l_all = o[None], l[None]
        ref, _ = O.merge_partials_ref(o_all, l_all)
        e = _err(out.view(H, D)[hk * g:(hk + 1) * g], ref)
        return {"max_abs_err": e, "tolerance": 1e-2, "ok": e <= 1e-2,
                "subset": "kv head 2 (query heads 8..11) over the whole sequence: each rank's slice by the fp32 oracle on the "
                          "device, partials gathered and merged by the oracle's merge"}

    def phases(self, steps):
        """Average device time of the three phases of a step, from CUDA events on the launching stream."""
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        for _ in range(3):
            self._run(self.q)
        torch.cuda.synchronize()
        for e in ev:
            self._run(self.q, e)
        torch.cuda.synchronize()
        avg = lambda i: sum(e[i].elapsed_time(e[i + 1]) for e in ev) / steps * 1e3
        if self._exchange() is None:
            return {"partition_kernel_with_local_merge_us": round(avg(0), 2), "all_gather_us": round(avg(1), 2),
                    "final_combine_us": round(avg(2), 2), "note": "measured one step at a time with events between the "
                    "phases; the all-gather is an NCCL call on the same stream (no call at one rank)"}
        res = {"partition_kernel_with_local_merge_us": round(avg(0), 2), "exchange_and_combine_us": round(avg(2), 2),
               "note": "measured one step at a time with events between the phases; the partials cross NVLink as peer "
                       "stores inside the kernel that combines them (fa_b200_exchange_combine)"}
        # the same step with an NCCL all-gather and a combine launch instead, for comparison
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        for _ in range(3):
            self._run(self.q, nccl=True)
        torch.cuda.synchronize()
        for e in ev:
            self._run(self.q, e, nccl=True)
        torch.cuda.synchronize()
        res["nccl_path"] = {"all_gather_us": round(avg(1), 2), "final_combine_us": round(avg(2), 2)}
        return res

    def step_e2e(self):
        out = self._run(self.q_host.to(self.q.device, non_blocking=True))
        self.out_host.copy_(out.view(H, D), non_blocking=True)
        return out


def make_workload(name, dev, seed, shard, real_world, scale=1.0):
    if name == "decode_bf16":
        return DecodeWorkload(dev, seed, batch=max(1, int(64 * scale)), shard=shard)
    if name == "decode_bf16_replica":   # the whole batch on every rank, other values per rank ("weak" scaling)
        return DecodeWorkload(dev, seed, batch=max(1, int(64 * scale)), shard=(0, 1), data_rank=shard[0], name=name)
    if name == "decode_fp8":
        return DecodeWorkload(dev, seed, fp8=True, batch=max(1, int(128 * scale)), shard=shard)
    if name == "prefill_bf16":
        return PrefillWorkload(dev, seed, nseq=max(1, int(16 * scale)), shard=shard)
    if name == "prefill_fp8":
        return PrefillWorkload(dev, seed, fp8=True, nseq=max(1, int(8 * scale)), shard=shard)
    if name == "sparse_bf16":
        return SparseWorkload(dev, seed, shard=shard)
    if name == "longseq":
        return LongSeqWorkload(dev, seed, shard, real_world)
    raise ValueError(name)


METRIC = {"bytes": ("paged decode HBM GB/s", "GB/s", 1e9), "flops": ("varlen prefill TFLOPS", "TFLOP/s", 1e12)}


# --------------------------------------------------------------------------------------------------
# timing
# --------------------------------------------------------------------------------------------------
def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world, dev):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x, world, dev):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def time_steps(fn, steps, warmup, world, dev, pipe=None):
    """Average device time of `steps` calls after `warmup`, max over ranks.  With a pipeline (side streams), the side
    streams start behind the first event and the second event waits for all of them."""
    for _ in range(warmup):
        fn()
    if pipe is not None:
        pipe.end()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if pipe is not None:
        pipe.begin()
    for _ in range(steps):
        fn()
    if pipe is not None:
        pipe.end()
    e1.record()
    barrier(world)
    mine = e0.elapsed_time(e1)
    if world > 1:   # every rank's own time, for the record (the value is computed from the slowest)
        import torch.distributed as dist
        t = torch.tensor([mine], dtype=torch.float64, device=dev)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        time_steps.by_rank = [round(float(x.item()) / steps, 4) for x in allt]
    else:
        time_steps.by_rank = [round(mine / steps, 4)]
    return max_over_ranks(mine, world, dev) / steps


def time_kernel_alone(wl, steps, warmup):
    """Average duration of the dominant kernel alone: the library records a CUDA event right before and right
    after it on the launching stream (profile_start_event / profile_stop_event of the C ABI)."""
    import flash_attn_2_cuda
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in pairs:      # create the handles
        a.record()
        b.record()
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize()
    for a, b in pairs:
        flash_attn_2_cuda.set_profile_events(a, b)
        wl.step()
    flash_attn_2_cuda.set_profile_events(None, None)
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in pairs)
    return sum(ts) / len(ts), ts[len(ts) // 2]


_READ_PEAK = {}


def read_stream_gbs(dev):
    """Bandwidth of a read-only pass over 2 GiB of this GPU's memory (the library's fa_b200_read_stream kernel, median of
    10 timed passes after 3 warm-up ones).  The roofline's `peak` is the driver-measured COPY bandwidth (read + write);
    the decode kernels only read, so their fraction of that peak can exceed 1: this figure is reported beside it."""
    if dev.index in _READ_PEAK:
        return _READ_PEAK[dev.index]
    import flash_attn_2_cuda
    buf = torch.empty(2 << 30, dtype=torch.uint8, device=dev)
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
    for _ in range(3):
        flash_attn_2_cuda.read_stream(buf, sink)
    for a, b in ev:
        a.record()
        flash_attn_2_cuda.read_stream(buf, sink)
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in ev)
    _READ_PEAK[dev.index] = buf.numel() / (ts[len(ts) // 2] * 1e-3) / 1e9
    del buf
    return _READ_PEAK[dev.index]


def host_us_per_call(wl, calls=200):
    """Wall time the host spends inside one public API call when the stream is idle (median), in microseconds."""
    for _ in range(10):
        wl.step()
    ts = []
    for _ in range(calls):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        wl.step()
        ts.append(time.perf_counter() - t0)
    torch.cuda.synchronize()
    ts.sort()
    return round(ts[len(ts) // 2] * 1e6, 1)


def run_workload(name, args, dev, rank, world, shard, peaks, cpu_budget):
    import flash_attn_2_cuda
    wl = make_workload(name, dev, args.seed, shard, world, args.scale)
    metric, unit, div = METRIC[wl.unit_name]
    # rank 0's GPU is sampled (its line is the one printed); a poller per rank would only add eight busy processes
    sampler = ClockSampler(dev.index, enabled=(rank == 0))
    with sampler as cs:
        l0 = flash_attn_2_cuda.launch_count()
        ms = time_steps(wl.step, args.steps, args.warmup, world, dev)
        ms_by_rank = list(time_steps.by_rank)
        launches = (flash_attn_2_cuda.launch_count() - l0) // (args.steps + args.warmup) * args.steps
        if hasattr(wl, "e2e_setup"):
            wl.e2e_setup()
        ms_e2e = time_steps(wl.step_e2e, args.steps, args.warmup, world, dev, getattr(wl, "pipe", None))
    clocks = cs.summary()
    launch_info = flash_attn_2_cuda.last_launch_info()
    total_units = sum_over_ranks(wl.units, world, dev)
    value = total_units / (ms * 1e-3) / div
    e2e = total_units / (ms_e2e * 1e-3) / div
    k_avg, k_med = time_kernel_alone(wl, max(args.steps, 5), 2)
    achieved = wl.units / (k_avg * 1e-3) / div
    if wl.unit_name == "bytes":
        peak, bound, punit = peaks["hbm_gbs"], "hbm", "GB/s"
    else:
        # a kernel timed alone: burst figure; fp8 has no measured peak, 2x the bf16 figure is used and said so
        peak = peaks["bf16_tflops"] * (2.0 if "fp8" in name else 1.0)
        bound, punit = "tensor", "TFLOP/s"
    ratio = TRAFFIC_RATIO.get(name)
    # correctness of what was timed, outside the timed region; every rank checks its own shard, the worst is reported
    check = wl.check()
    check["max_abs_err"] = round(max_over_ranks(check["max_abs_err"], world, dev), 6)
    check["tolerance"] = round(max_over_ranks(check["tolerance"], world, dev), 6)
    check["ok"] = bool(max_over_ranks(0.0 if check["ok"] else 1.0, world, dev) == 0.0)
    check["device_status"] = int(max_over_ranks(float(flash_attn_2_cuda.device_status()), world, dev))
    replica = name.endswith("_replica")
    res = {
        "name": name, "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "ms_per_step_by_rank": ms_by_rank, "higher_is_better": True,
        "scaling": "weak" if replica else "strong",
        "vs_baseline": None, "dtype": "e4m3" if "fp8" in name else "bf16", "data": "synthetic (seeded)",
        "config": wl.desc,
        "e2e": {"value": round(e2e, 2), "unit": unit, "h2d_bytes_per_step": int(wl.h2d), "d2h_bytes_per_step": int(wl.d2h),
                "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": int(launches),
        "roofline": {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": punit,
                     "frac": round(achieved / peak, 4), "peak_source": peaks["source"] + (" (2x bf16 for fp8)" if "fp8" in name and bound == "tensor" else ""),
                     "traffic": (ratio * wl.units if ratio is not None else
                                 (PREFILL_TRAFFIC_BYTES_PER_TOKEN[name] * wl.desc["tokens"]
                                  if name in PREFILL_TRAFFIC_BYTES_PER_TOKEN else None)),
                     "traffic_source": "ncu capture of a smaller case (profiles/), scaled by the units processed",
                     "kernel_ms_avg": round(k_avg, 4), "kernel_ms_median": round(k_med, 4),
                     "algorithmic_per_launch": wl.units, "rank": rank},
        "check": check,
        "clocks": clocks,
        "kernel": launch_info,
    }
    if bound == "hbm":
        rp = read_stream_gbs(dev)
        res["roofline"]["read_stream_gbs"] = round(rp, 1)
        res["roofline"]["frac_of_read_stream"] = round(achieved / rp, 4)
        res["roofline"]["note"] = ("peak is the measured device-to-device COPY bandwidth (reads and writes); this kernel only "
                                   "reads, so frac can pass 1: read_stream_gbs is a read-only pass over 2 GiB measured in "
                                   "this run on this GPU")
    if shard[1] != world:
        res["config"]["emulated"] = "rank %d of a %d-way job on one GPU, no collective" % shard
    if "decode" in name:
        res["host_us_per_call"] = host_us_per_call(wl)
    if name == "longseq":
        res["phases"] = wl.phases(max(args.steps, 10))
        if getattr(wl, "exchange_note", None):
            res["phases"]["exchange"] = wl.exchange_note
        res["host_us_per_call"] = host_us_per_call(wl, 100)
    if cpu_budget > 0 and rank == 0:
        res["cpu_baseline"] = cpu_baseline(name, args.seed, budget_s=cpu_budget)
    if getattr(wl, "_ex", None) is not None:   # unmap the peers' exchange buffers once every rank is done with them
        barrier(world)
        wl._ex.close()
    del wl
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (port of the reference's PyTorch attention) on the host cores
# --------------------------------------------------------------------------------------------------
def cpu_baseline(name, seed, budget_s=15.0):
    from oracle import attention_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(seed)
    metric, unit, div = METRIC["bytes" if ("decode" in name or name == "longseq") else "flops"]
    done_units, t_used, n = 0.0, 0.0, 0
    if "decode" in name or name == "longseq":
        fp8 = "fp8" in name
        # sample: sequences of the workload's length distribution, one at a time, until the budget is spent
        while t_used < budget_s and n < 256:
            L = 8192 if fp8 else int(torch.randint(1024, 32769, (1,), generator=g))
            if name == "longseq":
                L = 32768
            page = 256
            nb = (L + page - 1) // page
            kc = torch.randn(nb, page, HK, D, generator=g).to(torch.bfloat16)
            vc = torch.randn(nb, page, HK, D, generator=g).to(torch.bfloat16)
            q = torch.randn(1, 1, H, D, generator=g).to(torch.bfloat16)
            bt = torch.randperm(nb, generator=g).to(torch.int32).view(1, nb)
            sl = torch.tensor([L], dtype=torch.int32)
            t0 = time.perf_counter()
            O.paged_decode_ref(q, kc, vc, sl, bt)
            t_used += time.perf_counter() - t0
            done_units += L * HK * D * 2 * (1 if fp8 else 2) + H * D * 4 + 4 * nb
            n += 1
        sample = "%d sequence(s) of the workload's length distribution, bf16 math in fp32 (fp8 inputs dequantised)" % n
    else:
        # sample: one causal sequence of 1024 tokens per call (cost grows with S^2; FLOP rate is what is compared)
        S = 1024
        while t_used < budget_s and n < 256:
            q = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
            k = torch.randn(S, HK, D, generator=g).to(torch.bfloat16)
            v = torch.randn(S, HK, D, generator=g).to(torch.bfloat16)
            cu = torch.tensor([0, S], dtype=torch.int32)
            t0 = time.perf_counter()
            O.attention_varlen_ref(q, k, v, cu, cu, causal=True)
            t_used += time.perf_counter() - t0
            done_units += 4.0 * S * S * H * D / 2
            n += 1
        sample = "%d causal sequence(s) of 1024 tokens (dense masked evaluation), FLOP rate compared" % n
    return {"value": round(done_units / max(t_used, 1e-9) / div, 4), "unit": unit, "cores": cores, "kind": "port",
            "sample": sample, "seconds": round(t_used, 2)}


def run_reference(args, rank, world):
    """--impl reference: the CPU restatement of the reference's PyTorch attention on the host cores, W warm-up and K
    timed steps, each step a bounded sample of the configuration our own arm is quoted on."""
    if rank != 0:
        return
    name = "decode_bf16" if args.workload in ("default", "all", "decode_bf16_replica") else args.workload
    metric, unit, _ = METRIC["bytes" if ("decode" in name or name == "longseq") else "flops"]
    n_all = args.steps + args.warmup
    per_step = max(0.5, min(args.cpu_budget / 2, 150.0 / n_all))   # the whole run ends within a few minutes
    for i in range(args.warmup):
        cpu_baseline(name, args.seed + 1000 + i, budget_s=per_step)
    vals = []
    t0 = time.perf_counter()
    for i in range(args.steps):
        vals.append(cpu_baseline(name, args.seed + i, budget_s=per_step))
    dt = time.perf_counter() - t0
    v = sum(x["value"] for x in vals) / len(vals)
    cb = dict(vals[-1])
    cb["value"] = round(v, 4)
    cb["sample"] = "each of the %d steps: %s" % (len(vals), cb["sample"])
    if name == "decode_bf16":   # the headline: the same `config` object as our own arm prints
        _, _, config = decode_config(torch.Generator().manual_seed(args.seed), False, max(1, int(64 * args.scale)), 256, (0, world))
    else:
        config = {"workload": name}
    line = {"impl": "reference", "metric": metric, "value": round(v, 4), "unit": unit, "n_gpus": world,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": round(dt / len(vals) * 1e3, 2), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
            "config": config,
            "cpu_baseline": cb,
            "e2e": {"value": round(v, 4), "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="default",
                    choices=["default", "all", "decode_bf16", "decode_bf16_replica", "prefill_bf16", "decode_fp8",
                             "prefill_fp8", "sparse_bf16", "longseq"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-budget", type=float, default=10.0, help="seconds of CPU work for each cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scale", type=float, default=1.0,
                    help="shrink the batch / sequence count (profiler captures on a small case); 1.0 = the baseline configuration")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="one GPU only: run one rank's share of a job sharded this many ways (no collective)")
    ap.add_argument("--shard-rank", type=int, default=0, help="with --shard-of: which rank's share")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        # The first collectives of a process set NCCL up (channels, proxy threads, buffers); the steps timed right after
        # the first barrier ran 6 us slower each than the same steps later on.  Get that over with before any workload.
        for _ in range(3):
            dist.barrier()
            t = torch.ones(1, device=dev)
            dist.all_reduce(t)
        torch.cuda.synchronize()
    shard = (rank, world)
    if args.shard_of > 0:
        if world != 1:
            raise SystemExit("--shard-of is for a single process")
        shard = (args.shard_rank, args.shard_of)
    peaks = load_peaks()
    if args.workload in ("default", "all"):
        names = ["decode_bf16"] + (["decode_bf16_replica"] if world > 1 else []) + \
                ["prefill_bf16", "decode_fp8", "prefill_fp8", "sparse_bf16", "longseq"]
    else:
        names = [args.workload]
    results = []
    for i, n in enumerate(names):
        # the CPU port is timed beside the two headline metrics (decode bytes, prefill FLOPs) on rank 0 of a one-GPU run
        cpu = args.cpu_budget if (world == 1 and not args.no_cpu_baseline and n in ("decode_bf16", "prefill_bf16")) else 0.0
        results.append(run_workload(n, args, dev, rank, world, shard, peaks, cpu))
    if rank == 0:
        line = results[0]
        if len(results) > 1:
            line["also"] = [{k: r[k] for k in ("name", "metric", "value", "unit", "ms_per_step", "ms_per_step_by_rank", "scaling", "dtype", "config",
                                                 "e2e", "gpu_launches", "roofline", "check", "clocks", "kernel", "phases",
                                                 "host_us_per_call", "cpu_baseline") if k in r}
                            for r in results[1:]]
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
