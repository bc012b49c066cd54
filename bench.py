#!/usr/bin/env python
"""Headline benchmark: bf16 GEMM 8192^3 (A row-major, B column-major, f32 accumulate, bf16
out), N-sharded over the GPUs of one box, with flash-attention forward reported beside it.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's CPU path, timed on host cores

A step is one pass of the hot path over one batch of synthetic input (one whole GEMM).  Rank 0
prints ONE JSON line.  `value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is the
same metric from HOST buffers (host<->device copies inside the timed region); `attention` holds
the same set of figures (rate, roofline, end to end, CPU baseline) for the attention forward of
batch 8 x 32 heads x 8192 causal, whole on one GPU at N = 1 and batch x head sharded at N > 1;
`parity` is the error of seeded tiles of what the timed steps produced -- tiles computed on other
GPUs included -- against the CPU oracle, outside every timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_OUT = sys.stdout  # where the one JSON line goes; main() replaces it with the process's original stdout
METRIC = "bf16 GEMM & flash-attn fwd TFLOPS per B200 (% of tensor peak), 1/2/4/8 GPU"
UNIT = "TFLOP/s"
GEMM_N = 8192
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture) per launch of the
# kernel named, on the workload named.  The figure is only reported while the library still picks
# that kernel for the workload (sile_cuda_last_kernel); if the choice changes the bench stops
# instead of attaching a stale number to another kernel.
NCU_DRAM_TRAFFIC = {
    ("gemm_bf16_8192", "gemm_tn_pair_wide_kernel<16-bit>"): 0.991e9,
    ("attn_fwd_b8_h32_s8192_d128_causal", "attn_fwd_kernel"): 2.170e9,
    ("attn_fwd_b4_h32_s4096_d128_noncausal", "attn_fwd_kernel"): 0.5348e9,
}


def ncu_traffic(workload, sb):
    """The ncu DRAM traffic recorded for (workload, the kernel the last launch chose)."""
    chosen = sb._lib.lib().sile_cuda_last_kernel().decode().split(" ")[0]
    known = {k for (w, k) in NCU_DRAM_TRAFFIC if w == workload}
    if chosen not in known:
        raise SystemExit(f"bench.py: {workload} now runs on {chosen!r}, for which no ncu traffic figure is recorded "
                         f"(recorded: {sorted(known)}); capture it and update NCU_DRAM_TRAFFIC")
    return chosen, NCU_DRAM_TRAFFIC[(workload, chosen)]
ORACLE_TILE = (64, 64, 32)  # logical tile of the reference's GEMM example configuration
# name -> (batch*heads, seq, causal) for attention; None for the f32 GEMM
SIDE_WORKLOADS = {
    "attn_fwd_b4_h32_s4096_d128_noncausal": (128, 4096, False),
    "attn_fwd_h32_s8192_d128_causal_one_gpu_shard": (32, 8192, True),
    "attn_fwd_b8_h32_s8192_d128_causal": (256, 8192, True),
    "gemm_f32_4096": None,
    # one rank's column block of the headline GEMM at 2 / 4 GPUs, on one GPU (no exchange)
    "gemm_bf16_8192_shard_of_2": ("shard", 4096),
    "gemm_bf16_8192_shard_of_4": ("shard", 2048),
    "tileops_hbm": "tileops",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML queries; never sets anything)
class ClockSampler:
    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _reason_names(self, mask):
        p = self._nvml
        table = {
            "sw_power_cap": getattr(p, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(p, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(p, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(p, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "hw_power_brake_slowdown": getattr(p, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        return {k for k, bit in table.items() if mask & bit}

    def _run(self):
        if self._nvml is None:
            self._run_smi()
            return
        p = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(p.nvmlDeviceGetClockInfo(self._h, p.NVML_CLOCK_SM))
                try:
                    mask = p.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = p.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.reasons |= self._reason_names(mask)
            except Exception:
                pass
            time.sleep(self.period)

    def _run_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                self.samples.append(int(parts[0]))
                self.max_mhz = int(parts[1])
                for n, v in zip(names, parts[2:]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.1)

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ---------------------------------------------------------------------------------------------
def bf16_round(x):
    """float32 array -> nearest-even bf16 value, kept as float32 (what the oracle runs on)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(np.float32)


def cpu_oracle_gemm_sample(num_tiles: int, seed: int = 0):
    """Times the CPU oracle (the plain-C port of the reference's generated matmul) on a seeded
    sample of logical 64x64 output tiles of the 8192^3 problem, all host cores."""
    import oracle
    o = oracle.load()
    o.use_all_cores()
    n = GEMM_N
    rng = np.random.default_rng(seed)
    a = bf16_round(rng.standard_normal((n, n), dtype=np.float32) / np.float32(np.sqrt(n)))
    b = bf16_round(rng.standard_normal((n, n), dtype=np.float32) / np.float32(np.sqrt(n)))
    bm, bn, bk = ORACLE_TILE
    ids = rng.choice((n // bm) * (n // bn), size=num_tiles, replace=False)
    return o, a, b, ids


def time_oracle(o, a, b, ids):
    bm, bn, bk = ORACLE_TILE
    t0 = time.perf_counter()
    o.matmul_tiles(a, b, bm, bn, bk, ids)
    dt = time.perf_counter() - t0
    flops = 2.0 * len(ids) * bm * bn * a.shape[1]
    return dt, flops


def attention_cpu_baseline(bh, s, causal, target_seconds=8.0, seed=3):
    """The oracle's composed attention (general mma, left-fold reductions, expf) timed on a seeded
    sample of (head, 128-row query tile) units of the configuration, all host cores; throughput in
    the metric's unit from the flops of the sampled units, full problem by linear extrapolation."""
    import oracle
    o = oracle.load()
    cores = o.use_all_cores()
    d, bm, bn = 128, 128, 64
    rng = np.random.default_rng(seed)
    heads = max(cores, 8)
    q = bf16_round(rng.standard_normal((heads * s, d), dtype=np.float32))
    kt = bf16_round(rng.standard_normal((heads * d, s), dtype=np.float32))
    v = bf16_round(rng.standard_normal((heads * s, d), dtype=np.float32))
    tiles = s // bm

    def flops_of(units):
        total = 0.0
        for u in units:
            t = int(u) % tiles
            keys = min((t + 1) * bm, s) if causal else s
            keys = -(-keys // bn) * bn if causal else s
            total += 4.0 * bm * keys * d
        return total

    def run(units):
        t0 = time.perf_counter()
        o.attention(q, kt, v, heads, s, d, bm, bn, 1.0 / np.sqrt(d), causal, units=np.asarray(units))
        return time.perf_counter() - t0

    probe = [h * tiles + int(rng.integers(tiles)) for h in range(cores)]
    dt = run(probe)
    rate = flops_of(probe) / dt
    count = int(max(cores, min(heads * tiles, target_seconds * rate / (flops_of(probe) / len(probe)))))
    units = [(i % heads) * tiles + int(rng.integers(tiles)) for i in range(count)]
    dt = run(units)
    fl = flops_of(units)
    full = 4.0 * bh * s * s * d * (0.5 if causal else 1.0)
    return {"value": fl / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{count} seeded (head, 128-row query tile) units of {bh} x {s} x {d}{' causal' if causal else ''} "
                      f"(tiles 128 x 64), {dt:.1f} s; full problem by linear extrapolation {full / (fl / dt):.0f} s"}


def cpu_baseline(target_seconds: float = 12.0):
    o, a, b, ids = cpu_oracle_gemm_sample(2048)
    dt, fl = time_oracle(o, a, b, ids[:16])  # probe
    rate = fl / dt
    per_tile = fl / 16
    count = int(max(16, min(len(ids), target_seconds * rate / per_tile)))
    dt, fl = time_oracle(o, a, b, ids[:count])
    return {
        "value": fl / dt / 1e12, "unit": UNIT, "cores": o.num_threads(), "kind": "port",
        "sample": f"{count} seeded logical 64x64 output tiles of the 8192^3 GEMM (k = 8192 each), "
                  f"{dt:.1f} s; full problem by linear extrapolation {2.0 * GEMM_N ** 3 / (fl / dt):.0f} s",
    }


def run_reference(args, rank, world):
    """The reference's own CPU implementation of the path (its generated C, restated in
    oracle/sile_oracle.c; the reference itself needs a Rust toolchain that is absent)."""
    if rank != 0:
        return
    tiles_per_step = 32
    o, a, b, ids = cpu_oracle_gemm_sample(tiles_per_step * 8)
    for w in range(args.warmup):
        time_oracle(o, a, b, ids[:tiles_per_step])
    total_t, total_f = 0.0, 0.0
    for s in range(args.steps):
        lo = (s % 8) * tiles_per_step
        dt, fl = time_oracle(o, a, b, ids[lo:lo + tiles_per_step])
        total_t += dt
        total_f += fl
    value = total_f / total_t / 1e12
    sample = f"{tiles_per_step} seeded logical 64x64 output tiles (k = 8192) of the 8192^3 GEMM per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_t / max(args.steps, 1) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemm_bf16_8192: M=N=K=8192, N(0,1)/sqrt(K) values rounded to bf16 and upcast to f32 "
                               "(the reference computes in f32)",
                   "tile": "64x64x32"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": o.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=_OUT, flush=True)


def run_side_workload(name, iters, warmup, peaks):
    """Times one side workload on the current device with CUDA events; returns its result dict."""
    import torch
    import sile_b200 as sb
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(2)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(iters):
            fn()
        s1.record()
        torch.cuda.synchronize()
        sb.synchronize()
        return s0.elapsed_time(s1) / iters

    spec = SIDE_WORKLOADS[name]
    if spec == "tileops":
        # HBM-bound tile ops on 2^28 f32 elements (1 GiB per array, far beyond L2); algorithmic
        # bytes per element: vec_add 12, relu in place 8, row softmax 8, sum-reduce 4, matvec 4.
        n = 1 << 28
        x = torch.rand(n, generator=g, device=dev) - 0.5
        y = torch.rand(n, generator=g, device=dev)
        z = torch.empty_like(x)
        out = torch.zeros(1, device=dev)
        rows, cols = n // 1024, 1024
        vec = torch.rand(cols, generator=g, device=dev)
        zr = torch.empty(rows, device=dev)
        res = {}
        for op, launcher, bytes_per_elt in [
            ("vec_add", sb.vec_add(x, y, z, 4), 12), ("relu", sb.relu(z), 8),
            ("softmax_rows_1024", sb.softmax(x.view(rows, cols), z.view(rows, cols), 1), 8),
            ("parallel_reduce", sb.parallel_reduce(x, out, 1024), 4),
            ("matvec_k1024", sb.matvec(x.view(rows, cols), vec, zr, 1, 1), 4),
        ]:
            ms = timed(launcher.apply)
            gbs = n * bytes_per_elt / (ms * 1e-3) / 1e9
            res[op] = {"ms": ms, "algorithmic_GBps": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
        return res
    if spec is None:
        af = torch.rand(4096, 4096, generator=g, device=dev) * 2 - 1
        bf = torch.rand(4096, 4096, generator=g, device=dev) * 2 - 1
        cf = torch.zeros(4096, 4096, device=dev)
        ms = timed(sb.matmul(af, bf, cf, 64, 64, 32).apply)
        return {"ms": ms, "tflops_f32_equivalent": 2.0 * 4096 ** 3 / (ms * 1e-3) / 1e12,
                "note": "3 bf16 tensor-core passes (hi*hi + hi*lo + lo*hi), f32 accumulate"}
    if spec[0] == "shard":
        n, ns = GEMM_N, spec[1]
        a = (torch.randn(n, n, generator=g, device=dev) / n ** 0.5).to(torch.bfloat16)
        b = (torch.randn(ns, n, generator=g, device=dev) / n ** 0.5).to(torch.bfloat16)   # [N/p, K]: column-major block
        c = torch.zeros(n, ns, device=dev, dtype=torch.bfloat16)
        ms = timed(sb.matmul(a, b, c, *ORACLE_TILE, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply)
        tf = 2.0 * n * ns * n / (ms * 1e-3) / 1e12
        return {"ms": ms, "tflops": tf, "frac_of_measured_gemm_peak": tf / peaks["bf16_tflops"],
                "launch": sb._lib.lib().sile_cuda_last_kernel().decode()}
    bh, s, causal = spec
    q, k, v = [torch.randn(bh, s, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
    o = torch.zeros_like(q)
    ms = timed(sb.attention(q, k, v, o, 1.0 / 128 ** 0.5, causal).apply)
    fl = 4.0 * bh * s * s * 128 * (0.5 if causal else 1.0)
    tf = fl / (ms * 1e-3) / 1e12
    return {"ms": ms, "tflops": tf, "frac_of_nominal_dense_bf16": tf / NOMINAL_BF16_TFLOPS,
            "frac_of_measured_gemm_peak": tf / peaks["bf16_tflops"]}


# ---------------------------------------------------------------------------------------------
def _claim_stdout():
    """Keeps stdout for the JSON line alone: file descriptor 1 is pointed at stderr for everything
    else in the process (libraries such as NCCL print a version banner on it), and the returned
    handle writes to the original stdout."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    global _OUT
    _OUT = _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunks", type=int, default=4, help="M chunks used to overlap the NCCL all-gather (N > 1)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: how C is assembled on every rank (fused = stores from the GEMM epilogue)")
    ap.add_argument("--no-extras", action="store_true", help="skip the attention / f32 side measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="gemm_bf16_8192", choices=["gemm_bf16_8192"] + sorted(SIDE_WORKLOADS),
                    help="gemm_bf16_8192 is the headline bench; the others time one side workload on one GPU "
                         "(used for profiling) and print a short JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import sile_b200 as sb
    import sile_b200.sharding  # noqa: F401

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    sb._lib.lib()  # fail loudly if the extension is missing
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=180))
    if args.workload != "gemm_bf16_8192":
        if rank == 0:
            peaks, _ = load_peaks()
            res = run_side_workload(args.workload, args.steps, args.warmup, peaks)
            res.update({"workload": args.workload, "steps": args.steps, "warmup": args.warmup})
            print(json.dumps(res), file=_OUT, flush=True)
        return
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)

    n = GEMM_N
    p = world
    nshard = n // p
    dev = torch.device("cuda", local_rank)
    g = torch.Generator(device=dev).manual_seed(0)
    a = (torch.randn(n, n, generator=g, device=dev) / n ** 0.5).to(torch.bfloat16)
    g.manual_seed(1)
    # column-major B: stored [N, K]; every rank draws the same B and keeps its column block
    b_full = (torch.randn(n, n, generator=g, device=dev) / n ** 0.5).to(torch.bfloat16)
    b_shard = b_full[rank * nshard:(rank + 1) * nshard].contiguous()
    if p > 1:
        del b_full
    c = torch.zeros(n, n, device=dev, dtype=torch.bfloat16) if p == 1 else None
    bm, bn, bk = ORACLE_TILE
    launches_per_step = 1

    exchange = "none"
    fused = None
    if p == 1:
        kl = sb.matmul(a, b_shard, c, bm, bn, bk, b_layout=sb._lib.LAYOUT_COL_MAJOR)

        def step():
            kl.apply()
    else:
        if args.exchange in ("auto", "fused"):
            try:
                # C lives in symmetric memory: every rank maps every rank's buffer, and the GEMM
                # epilogue stores its column block straight into all of them over NVLink.
                import torch.distributed._symmetric_memory as symm_mem
                c = symm_mem.empty((n, n), dtype=torch.bfloat16, device=dev)
                hdl = symm_mem.rendezvous(c, dist.group.WORLD)
                ptrs = [int(x) for x in hdl.buffer_ptrs]
                c.zero_()
                fused = (hdl, ptrs)
            except Exception as e:  # no peer mapping on this box: all-gather through NCCL instead
                if args.exchange == "fused":
                    raise
                if rank == 0:
                    print(f"symmetric memory unavailable ({e!r}); using the NCCL all-gather path", file=sys.stderr)
                c = torch.zeros(n, n, device=dev, dtype=torch.bfloat16)
        if fused is not None:
            exchange = ("fused epilogue: one TMA store per destination into every rank's C over NVLink (symmetric memory; "
                        "st.global for ragged or masked tiles), one device barrier per step")
            hdl, ptrs = fused
            launches_per_step = 1

            def step():
                sb.matmul_allgather(a, b_shard, ptrs, rank, n, torch.bfloat16, bm, bn, bk)
                hdl.barrier(channel=0, timeout_ms=20000)
        else:
            exchange = f"{args.chunks} M-chunks, NCCL all-gather of C overlapped with compute, unshard kernel"
            if c is None:
                c = torch.zeros(n, n, device=dev, dtype=torch.bfloat16)
            chunks = sb.sharding.row_chunks(n, max(1, args.chunks))
            nch = len(chunks)
            cs = torch.zeros(n, nshard, device=dev, dtype=torch.bfloat16)
            gathered = [torch.empty(p, rc, nshard, device=dev, dtype=torch.bfloat16) for _, rc in chunks]
            comm = torch.cuda.Stream(device=dev)
            events = [torch.cuda.Event() for _ in range(nch)]
            done = torch.cuda.Event()
            launches_per_step = 2 * nch

            def step():
                main_stream = torch.cuda.current_stream()
                comm.wait_stream(main_stream)
                for i, (r0, rc) in enumerate(chunks):
                    sb.matmul_shard(a[r0:r0 + rc], b_shard, cs[r0:r0 + rc], 0, nshard, bm, bn, bk)
                    events[i].record(main_stream)
                    with torch.cuda.stream(comm):
                        comm.wait_event(events[i])
                        dist.all_gather_into_tensor(gathered[i], cs[r0:r0 + rc])
                        sb.unshard_columns(c[r0:r0 + rc], gathered[i], stream=comm)
                done.record(comm)
                main_stream.wait_event(done)

    def barrier():
        if p > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if p == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing -------------------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    # A short timed region gives the 10 ms clock sampler too few readings under load: keep the
    # same work running for ~0.25 s more.  The count derives from the max-reduced time, so every
    # rank runs the same number of (collective) steps.
    if ms_total < 250.0:
        for _ in range(int(min(5000, 250.0 / max(ms_total / args.steps, 1e-3)))):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    barrier()
    sb.synchronize()
    ms_step = ms_total / args.steps
    flops = 2.0 * n ** 3
    value = flops / (ms_step * 1e-3) / 1e12

    gemm_launch = sb._lib.lib().sile_cuda_last_kernel().decode()  # kernel, slice plan if any, grid, block, shared memory
    gemm_kernel = gemm_launch.split(" ")[0]
    gemm_traffic = ncu_traffic("gemm_bf16_8192", sb)[1] if p == 1 else None

    # ---- how long the per-step device barrier alone takes (N > 1, fused exchange) -----------------
    barrier_ms = None
    if p > 1 and fused is not None:
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(20):
            fused[0].barrier(channel=0, timeout_ms=20000)
        b1.record()
        torch.cuda.synchronize()
        barrier_ms = max_over_ranks(b0.elapsed_time(b1) / 20)

    # ---- parity of what the timed steps produced, against the CPU oracle (rank 0, untimed) --------
    # Seeded logical 64 x 64 tiles of C, at least one inside every rank's column block: at N > 1
    # most of them were computed on ANOTHER GPU and reached this one through the fused all-gather.
    parity = {"tol": 2e-2}
    if rank == 0:
        import oracle as _oracle
        orc = _oracle.load()
        orc.use_all_cores()
        if p > 1:
            g.manual_seed(1)
            b_all = (torch.randn(n, n, generator=g, device=dev) / n ** 0.5).to(torch.bfloat16)
        else:
            b_all = b_full
        a_np = a.float().cpu().numpy()
        b_np = np.ascontiguousarray(b_all.float().cpu().numpy().T)  # [K, N] row-major, as the oracle reads it
        del b_all
        rng = np.random.default_rng(7)
        tiles_n = n // bn
        ids = []
        for i in range(max(8, p)):
            r = i % p  # rank whose column block the tile lies in
            col_tile = r * (nshard // bn) + int(rng.integers(nshard // bn))
            ids.append(int(rng.integers(n // bm)) * tiles_n + col_tile)
        want = orc.matmul_tiles(a_np, b_np, bm, bn, bk, ids)
        got = c.float().cpu().numpy()
        worst, scale = 0.0, float(np.abs(want).max())
        for t in ids:
            i, j = divmod(t, tiles_n)
            sl = (slice(i * bm, (i + 1) * bm), slice(j * bn, (j + 1) * bn))
            worst = max(worst, float(np.abs(got[sl] - want[sl]).max()))
        parity["gemm_rel_err"] = worst / scale
        parity["gemm_tiles"] = len(ids)
        parity["gemm_tiles_from_other_ranks"] = sum(1 for t in ids if (t % tiles_n) * bn // nshard != rank)
        del a_np, b_np, got, want

    # ---- end to end through the public API with host buffers ----------------------------------------
    a_h = a.cpu().pin_memory()
    b_h = b_shard.cpu().pin_memory()
    c_h = torch.zeros(n, nshard, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    if p == 1:
        class _KN:  # B travels as its logical [K, N_shard] shape
            shape = (n, nshard)

            @staticmethod
            def data_ptr():
                return b_h.data_ptr()

        desc = sb.make_desc(sb._lib.OP_MATMUL, sb._lib.DTYPE_BF16, sb._lib.DTYPE_BF16, sb._lib.LAYOUT_COL_MAJOR,
                            consts=(bm, bn, bk))
        host_launch = sb.KernelLauncher(desc, [a_h, _KN, c_h]).grid((n // bm, nshard // bn, 1))
        e2e_step = host_launch.apply_host
        h2d_per_rank = (a_h.numel() + b_h.numel()) * 2
        api = "sile_cuda_launch_host (pinned host buffers: A and B in, C out)"
    else:
        # every rank stages only its row slab of A and its column block of B over the host link;
        # the slabs of A are all-gathered device to device (NCCL over NVLink), then the rank's
        # column block is computed and copied back
        hm = sb.sharding.HostShardedMatmul(
            n, n, n, p, rank, torch.bfloat16,
            compute=lambda af, bs, cs: sb.matmul_shard(af, bs, cs, 0, nshard, bm, bn, bk),
            device_empty=lambda shape, dt: torch.empty(shape, dtype=dt, device=dev),
            all_gather=lambda full, part: dist.all_gather_into_tensor(full, part))

        def e2e_step():
            hm.step(a_h, b_h, c_h)
            torch.cuda.synchronize()

        h2d_per_rank = hm.h2d_bytes
        api = ("sile_b200.sharding.HostShardedMatmul (pinned host buffers: every rank stages its row slab of A and its "
               "column block of B, the slabs are all-gathered over NVLink, the rank returns its column block of C)")
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0) / e2e_steps
    e2e = {
        "value": flops / e2e_s / 1e12, "unit": UNIT,
        "h2d_bytes_per_step": p * h2d_per_rank,
        "d2h_bytes_per_step": p * c_h.numel() * 2,
        "ms_per_step": e2e_s * 1e3,
        "api": api,
    }
    e2e_check = float((c_h.float() - c[:, rank * nshard:(rank + 1) * nshard].float().cpu()).abs().max())
    # What the host link alone allows: plain copies of the same pinned buffers, timed with CUDA
    # events.  The inputs must all cross before the last rows of C can be computed, so the
    # host->device time of this rank's inputs is a floor for one end-to-end step on this box.
    in_elems = h2d_per_rank // 2
    scratch_in = torch.empty(in_elems, dtype=torch.bfloat16, device=dev)
    scratch_out = torch.empty(c_h.numel(), dtype=torch.bfloat16, device=dev)
    c_back = torch.empty_like(c_h).pin_memory()
    src_in = a_h.view(-1)[:in_elems] if in_elems <= a_h.numel() else None

    def timed_copy(fn):
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return best

    def copy_in():
        if src_in is not None:
            scratch_in.copy_(src_in, non_blocking=True)
        else:
            scratch_in[:a_h.numel()].copy_(a_h.view(-1), non_blocking=True)
            scratch_in[a_h.numel():].copy_(b_h.view(-1)[:in_elems - a_h.numel()], non_blocking=True)

    h2d_ms = timed_copy(copy_in)
    d2h_ms = timed_copy(lambda: c_back.view(-1).copy_(scratch_out, non_blocking=True))
    e2e["host_link"] = {
        "h2d_GBps": scratch_in.numel() * 2 / (h2d_ms * 1e-3) / 1e9, "d2h_GBps": scratch_out.numel() * 2 / (d2h_ms * 1e-3) / 1e9,
        "inputs_h2d_ms": h2d_ms, "frac_of_step": h2d_ms / (e2e_s * 1e3),
        "note": "plain pinned-memory copies of as many bytes as this rank stages in and returns; the step cannot be shorter than inputs_h2d_ms",
    }
    del scratch_in, scratch_out, c_back

    # ---- attention forward: the metric's second half ------------------------------------------------
    extras = {}
    attention = None
    peaks, peak_src = load_peaks()
    A5 = "attn_fwd_b8_h32_s8192_d128_causal"
    bh_total, s_len = 256, 8192
    afl = 4.0 * bh_total * s_len * s_len * 128 * 0.5
    scale_a = 1.0 / 128 ** 0.5

    def attention_parity(o_rows_of, inputs_of, units):
        """units: (global head, q tile); inputs_of(head) -> (q, k, v) [S, 128] bf16 tensors of that head;
        o_rows_of(head, tile) -> the [128, 128] rows this run produced.  Returns the worst error
        relative to the oracle's output scale."""
        worst = 0.0
        for head, tile in units:
            qh, kh, vh = inputs_of(head)
            kt = np.ascontiguousarray(kh.float().cpu().numpy().T)
            want = orc.attention(qh.float().cpu().numpy(), kt, vh.float().cpu().numpy(), 1, s_len, 128, 128, 64,
                                 scale_a, True, units=np.asarray([tile]))[tile * 128:(tile + 1) * 128]
            got = o_rows_of(head, tile).float().cpu().numpy()
            worst = max(worst, float(np.abs(got - want).max() / np.abs(want).max()))
        return worst

    if p == 1 and not args.no_extras:
        for name in SIDE_WORKLOADS:
            if "shard_of" in name:
                continue  # profiling helpers (one rank's block of the multi-GPU GEMM on one GPU)
            extras[name] = run_side_workload(name, 10 if "b8" in name else 20, 3, peaks)
        # the configuration the attention target is stated on, batch 8 x 32 heads x 8192 causal,
        # kept whole on this GPU: device-resident rate, roofline, parity, end to end, CPU baseline
        g.manual_seed(2)
        q, k, v = [torch.randn(bh_total, s_len, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
        o_dev = torch.zeros_like(q)
        akl = sb.attention(q, k, v, o_dev, scale_a, True)
        for _ in range(3):
            akl.apply()
        torch.cuda.synchronize()
        a_sampler = ClockSampler(local_rank).start()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(10):
            akl.apply()
        a1.record()
        torch.cuda.synchronize()
        a_ms = a0.elapsed_time(a1) / 10
        for _ in range(int(250.0 / a_ms)):  # enough load for the clock sampler
            akl.apply()
        torch.cuda.synchronize()
        a_clocks = a_sampler.stop()
        sb.synchronize()
        a_kernel, a_traffic = ncu_traffic(A5, sb)
        atf = afl / (a_ms * 1e-3) / 1e12
        attention = {
            "workload": f"{A5}: batch 8 x 32 heads x 8192 x 128, causal, bf16, f32 softmax statistics, whole on one GPU",
            "value": atf, "unit": UNIT, "ms_per_step": a_ms, "clocks": a_clocks,
            "roofline": {"bound": "tensor", "kernel": a_kernel, "achieved": atf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": atf / peaks["bf16_tflops"], "peak_source": f"{peak_src} bf16_tflops",
                         "frac_of_nominal_dense_bf16": atf / NOMINAL_BF16_TFLOPS, "traffic": a_traffic,
                         "algorithmic_flops_per_launch": afl, "algorithmic_bytes_per_launch": 4.0 * bh_total * s_len * 128 * 2},
        }
        if rank == 0:
            units = [(0, 63), (255, 63), (131, 0), (77, 31)]
            parity["attn_rel_err"] = attention_parity(lambda h, t: o_dev[h, t * 128:(t + 1) * 128],
                                                      lambda h: (q[h], k[h], v[h]), units)
            parity["attn_units"] = len(units)
        # end to end: host q, k, v in, host o out, through sile_cuda_launch_host
        qh_, kh_, vh_ = [x.cpu().pin_memory() for x in (q, k, v)]
        oh_ = torch.zeros(bh_total, s_len, 128, dtype=torch.bfloat16).pin_memory()
        host_attn = sb.attention(qh_, kh_, vh_, oh_, scale_a, True)
        host_attn.apply_host()
        t0 = time.perf_counter()
        for _ in range(3):
            host_attn.apply_host()
        ae2e_s = (time.perf_counter() - t0) / 3
        attention["e2e"] = {"value": afl / ae2e_s / 1e12, "unit": UNIT, "ms_per_step": ae2e_s * 1e3,
                            "h2d_bytes_per_step": 3 * q.numel() * 2, "d2h_bytes_per_step": q.numel() * 2,
                            "matches_device_result": bool(torch.equal(oh_, o_dev.cpu())),
                            "api": "sile_cuda_launch_host (pinned host q, k, v in, o out; heads streamed in chunks, copies and kernels overlapped)"}
        del q, k, v, o_dev, qh_, kh_, vh_, oh_
        if not args.no_cpu_baseline:
            attention["cpu_baseline"] = attention_cpu_baseline(bh_total, s_len, True)

    if p > 1 and not args.no_extras:
        # attention shards by batch x head: every rank runs its contiguous slab of the 256
        # (batch, head) pairs and the slabs are all-gathered straight into final layout
        h0, hc = sb.sharding.head_slab(bh_total, p, rank)

        def slab_inputs(r):
            g.manual_seed(100 + r)
            return [torch.randn(hc, s_len, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]

        q, k, v = slab_inputs(rank)
        o_slab = torch.zeros_like(q)
        o_full = torch.empty(bh_total, s_len, 128, device=dev, dtype=torch.bfloat16)
        akl = sb.attention(q, k, v, o_slab, scale_a, True)

        def attn_step_nccl():
            akl.apply()
            dist.all_gather_into_tensor(o_full, o_slab)

        def time_attn(fn):
            for _ in range(3):
                fn()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(10):
                fn()
            a1.record()
            barrier()
            return max_over_ranks(a0.elapsed_time(a1)) / 10

        nccl_ms = time_attn(attn_step_nccl)
        fused_ms, fused_matches = None, None
        o_gathered = o_full
        if args.exchange in ("auto", "fused"):
            try:
                # O lives in symmetric memory; every CTA's epilogue TMA-stores its rows into every
                # rank's buffer, so the exchange runs under the remaining CTAs' compute.
                import torch.distributed._symmetric_memory as symm_mem
                o_sym = symm_mem.empty((bh_total, s_len, 128), dtype=torch.bfloat16, device=dev)
                ohdl = symm_mem.rendezvous(o_sym, dist.group.WORLD)
                optrs = [int(x) for x in ohdl.buffer_ptrs]
                o_sym.zero_()

                def attn_step_fused():
                    sb.attention_allgather(q, k, v, optrs, rank, scale_a, True)
                    ohdl.barrier(channel=1, timeout_ms=20000)

                fused_ms = time_attn(attn_step_fused)
                torch.cuda.synchronize()
                barrier()
                fused_matches = bool(torch.equal(o_sym, o_full))
                o_gathered = o_sym
            except Exception as e:
                if args.exchange == "fused":
                    raise
                if rank == 0:
                    print(f"fused attention all-gather unavailable ({e!r})", file=sys.stderr)
        ams = fused_ms if fused_ms is not None else nccl_ms
        atf = afl / (ams * 1e-3) / 1e12
        if rank == 0:
            # units computed on other GPUs included: their inputs are redrawn here from the owning
            # rank's seed
            cache = {}

            def inputs_of(head):
                r = head // hc
                if r not in cache:
                    cache.clear()
                    cache[r] = slab_inputs(r)
                qq, kk, vv = cache[r]
                return qq[head - r * hc], kk[head - r * hc], vv[head - r * hc]

            units = [(0, 63), (hc - 1, 17), ((p - 1) * hc, 31), (bh_total - 1, 63)]
            parity["attn_rel_err"] = attention_parity(lambda h, t: o_gathered[h, t * 128:(t + 1) * 128], inputs_of, units)
            parity["attn_units"] = len(units)
            parity["attn_units_from_other_ranks"] = sum(1 for h, _ in units if h // hc != rank)
            cache.clear()
        exchange_a = ("all-gather folded into the kernel: every CTA TMA-stores its rows of O into every rank's buffer "
                      "(symmetric memory), one device barrier per step" if fused_ms is not None else
                      "NCCL all-gather of the output slabs (rank-major = final [B*H, S, D] layout)")
        attention = {
            "workload": f"{A5}: batch 8 x 32 heads x 8192 x 128, causal, bf16; batch x head sharded over {p} GPUs, "
                        "O all-gathered to every rank inside the timed step",
            "value": atf, "unit": UNIT, "ms_per_step": ams, "per_gpu_tflops": atf / p, "exchange": exchange_a,
            "nccl_all_gather_ms": nccl_ms, "nccl_all_gather_tflops_whole_job": afl / (nccl_ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor+nvlink", "kernel": sb._lib.lib().sile_cuda_last_kernel().decode().split(" ")[0],
                         "achieved": atf / p, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": atf / p / peaks["bf16_tflops"],
                         "frac_of_nominal_dense_bf16": atf / p / NOMINAL_BF16_TFLOPS, "traffic": None,
                         "nvlink_bytes_in_per_gpu_per_step": (p - 1) * hc * s_len * 128 * 2,
                         "note": "per-GPU share of the whole step: kernel, exchange of O and barrier"},
        }
        if fused_ms is not None:
            attention["fused_matches_nccl_result"] = fused_matches
        # end to end for this rank's slab: host q, k, v in, host o out
        qh_, kh_, vh_ = [x.cpu().pin_memory() for x in (q, k, v)]
        oh_ = torch.zeros(hc, s_len, 128, dtype=torch.bfloat16).pin_memory()
        host_attn = sb.attention(qh_, kh_, vh_, oh_, scale_a, True)
        host_attn.apply_host()
        barrier()
        t0 = time.perf_counter()
        for _ in range(3):
            host_attn.apply_host()
        barrier()
        ae2e_s = max_over_ranks(time.perf_counter() - t0) / 3
        attention["e2e"] = {"value": afl / ae2e_s / 1e12, "unit": UNIT, "ms_per_step": ae2e_s * 1e3,
                            "h2d_bytes_per_step": p * 3 * q.numel() * 2, "d2h_bytes_per_step": p * q.numel() * 2,
                            "matches_device_result": bool(torch.equal(oh_, o_slab.cpu())),
                            "api": "sile_cuda_launch_host per rank (pinned host slabs of q, k, v in, the rank's slab of o out)"}
        extras["attn_fwd_b8_h32_s8192_d128_causal_sharded"] = {"ms": ams, "tflops_whole_job": atf, "per_gpu_tflops": atf / p}
        sb.synchronize()
        del q, k, v, o_slab, o_full, o_gathered

    # ---- roofline of the dominant kernel ---------------------------------------------------------
    timed_region_s = ms_total * 1e-3
    peak_key = "bf16_tflops_sustained" if timed_region_s > 1.0 else "bf16_tflops"
    per_gpu_flops = flops / p
    gemm_ms = ms_step  # one step = one GEMM pass (N = 1: exactly one launch of the kernel named below)
    achieved = per_gpu_flops / (gemm_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peaks[peak_key], "unit": "TFLOP/s",
        "frac": achieved / peaks[peak_key], "traffic": gemm_traffic,
        "peak_source": f"{peak_src} {peak_key}", "frac_of_nominal_dense_bf16": achieved / NOMINAL_BF16_TFLOPS,
        "kernel": gemm_kernel, "launch": gemm_launch, "algorithmic_flops_per_launch": per_gpu_flops,
    }
    if p > 1:
        roofline["note"] = ("per-GPU share of the whole step (GEMM with the all-gather of C in its epilogue, then the barrier), "
                            "not the kernel alone; traffic = NVLink bytes that must enter each GPU per step")
        roofline["traffic"] = (p - 1) * n * nshard * 2
        roofline["nvlink_floor_ms"] = (p - 1) * n * nshard * 2 / 770e9 * 1e3
        roofline["barrier_ms"] = barrier_ms

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": p, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": "gemm_bf16_8192: M=N=K=8192, A row-major, B column-major, N(0,1)/sqrt(K) bf16, f32 accumulate, bf16 out",
            "parallelism": f"N-sharded x{p}" + ("" if p == 1 else f"; {exchange}"),
            "l2": "inputs (2 x 128 MiB) and output (128 MiB) exceed the 126 MB L2; no flush between steps",
            "per_gpu_tflops": value / p,
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
        "roofline": roofline, "e2e_matches_device_result": e2e_check == 0.0, "parity": parity,
    }
    if attention is not None:
        line["attention"] = attention
    if extras:
        line["extras"] = extras
    if rank == 0 and p == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    if rank == 0:
        print(json.dumps(line), file=_OUT, flush=True)
    if p > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
