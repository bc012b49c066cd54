#!/usr/bin/env python
"""Headline benchmark: bf16 GEMM 8192^3 (A row-major, B column-major, f32 accumulate, bf16
out), N-sharded over the GPUs of one box, with flash-attention forward reported beside it.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's CPU path, timed on host cores

A step is one pass of the hot path over one batch of synthetic input (one whole GEMM).  Rank 0
prints ONE JSON line.  `value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is the
same metric through the C ABI with HOST buffers (host<->device copies inside the timed region).
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
# DRAM bytes (read + write) of one 8192^3 GEMM launch; from the ncu capture summarised in
# profiles/gemm_tn_pair_wide_kernel_bf16_8192.md (dram__bytes_read.sum + dram__bytes_write.sum).
GEMM_DRAM_TRAFFIC_BYTES = 1.046e9
ORACLE_TILE = (64, 64, 32)  # logical tile of the reference's GEMM example configuration
# name -> (batch*heads, seq, causal) for attention; None for the f32 GEMM
SIDE_WORKLOADS = {
    "attn_fwd_b4_h32_s4096_d128_noncausal": (128, 4096, False),
    "attn_fwd_h32_s8192_d128_causal_one_gpu_shard": (32, 8192, True),
    "attn_fwd_b8_h32_s8192_d128_causal": (256, 8192, True),
    "gemm_f32_4096": None,
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
        "config": {"workload": "gemm_bf16_8192: M=N=K=8192 (oracle runs the bf16 values upcast to f32)",
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
    if p == 1:
        kl = sb.matmul(a, b_shard, c, bm, bn, bk, b_layout=sb._lib.LAYOUT_COL_MAJOR)

        def step():
            kl.apply()
    else:
        fused = None
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
            exchange = "fused epilogue: st.global into every rank's C over NVLink (symmetric memory), one device barrier per step"
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

    # ---- end to end through the C ABI with host buffers ----------------------------------------
    a_h = a.cpu().pin_memory()
    b_h = b_shard.cpu().pin_memory()
    c_h = torch.zeros(n, nshard, dtype=torch.bfloat16).pin_memory()

    class _KN:  # B travels as its logical [K, N_shard] shape
        shape = (n, nshard)

        @staticmethod
        def data_ptr():
            return b_h.data_ptr()

    desc = sb.make_desc(sb._lib.OP_MATMUL, sb._lib.DTYPE_BF16, sb._lib.DTYPE_BF16, sb._lib.LAYOUT_COL_MAJOR,
                        consts=(bm, bn, bk))
    host_launch = sb.KernelLauncher(desc, [a_h, _KN, c_h]).grid((n // bm, nshard // bn, 1))
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        host_launch.apply_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_launch.apply_host()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0) / e2e_steps
    e2e = {
        "value": flops / e2e_s / 1e12, "unit": UNIT,
        "h2d_bytes_per_step": p * (a_h.numel() + b_h.numel()) * 2,
        "d2h_bytes_per_step": p * c_h.numel() * 2,
        "ms_per_step": e2e_s * 1e3,
        "api": "sile_cuda_launch_host (pinned host buffers; every rank stages A and its column block of B, "
               "returns its column block of C)",
    }
    e2e_check = float((c_h[:64].float() - c[:64, rank * nshard:(rank + 1) * nshard].float().cpu()).abs().max())
    # What the host link alone allows: plain copies of the same pinned buffers, timed with CUDA
    # events.  The inputs must all cross before the last rows of C can be computed, so the
    # host->device time of A and B is a floor for one end-to-end step on this box.
    scratch_in = torch.empty(a_h.numel() + b_h.numel(), dtype=torch.bfloat16, device=dev)
    scratch_out = torch.empty(c_h.numel(), dtype=torch.bfloat16, device=dev)
    c_back = torch.empty_like(c_h).pin_memory()

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
        scratch_in[:a_h.numel()].copy_(a_h.view(-1), non_blocking=True)
        scratch_in[a_h.numel():].copy_(b_h.view(-1), non_blocking=True)

    h2d_ms = timed_copy(copy_in)
    d2h_ms = timed_copy(lambda: c_back.view(-1).copy_(scratch_out, non_blocking=True))
    e2e["host_link"] = {
        "h2d_GBps": scratch_in.numel() * 2 / (h2d_ms * 1e-3) / 1e9, "d2h_GBps": scratch_out.numel() * 2 / (d2h_ms * 1e-3) / 1e9,
        "inputs_h2d_ms": h2d_ms, "frac_of_step": h2d_ms / (e2e_s * 1e3),
        "note": "plain pinned-memory copies of this rank's A and B (in) and C (out); the step cannot be shorter than inputs_h2d_ms",
    }
    del scratch_in, scratch_out, c_back

    # ---- side measurements (N = 1): attention forward and the f32 GEMM ----------------------------
    extras = {}
    peaks, peak_src = load_peaks()
    if p == 1 and not args.no_extras:
        for name in SIDE_WORKLOADS:
            extras[name] = run_side_workload(name, 10 if "b8" in name else 20, 3, peaks)

    if p > 1 and not args.no_extras:
        # attention shards by batch x head: every rank runs its contiguous slab of the 256
        # (batch, head) pairs and the slabs are all-gathered (NCCL) straight into final layout
        bh_total, s_len = 256, 8192
        h0, hc = sb.sharding.head_slab(bh_total, p, rank)
        g.manual_seed(100 + rank)
        q, k, v = [torch.randn(hc, s_len, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
        o_slab = torch.zeros_like(q)
        o_full = torch.empty(bh_total, s_len, 128, device=dev, dtype=torch.bfloat16)
        akl = sb.attention(q, k, v, o_slab, 1.0 / 128 ** 0.5, True)

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

        afl = 4.0 * bh_total * s_len * s_len * 128 * 0.5
        nccl_ms = time_attn(attn_step_nccl)
        fused_ms = None
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
                    sb.attention_allgather(q, k, v, optrs, rank, 1.0 / 128 ** 0.5, True)
                    ohdl.barrier(channel=1, timeout_ms=20000)

                fused_ms = time_attn(attn_step_fused)
                torch.cuda.synchronize()
                barrier()
                fused_matches = bool(torch.equal(o_sym, o_full))
                del o_sym
            except Exception as e:
                if args.exchange == "fused":
                    raise
                if rank == 0:
                    print(f"fused attention all-gather unavailable ({e!r})", file=sys.stderr)
        ams = fused_ms if fused_ms is not None else nccl_ms
        atf = afl / (ams * 1e-3) / 1e12
        extras["attn_fwd_b8_h32_s8192_d128_causal_sharded"] = {
            "ms": ams, "tflops_whole_job": atf, "per_gpu_tflops": atf / p,
            "exchange": ("all-gather folded into the kernel: every CTA TMA-stores its rows of O into every rank's buffer "
                         "(symmetric memory), one device barrier per step" if fused_ms is not None else
                         "NCCL all-gather of the output slabs (rank-major = final [B*H, S, D] layout)"),
            "nccl_all_gather_ms": nccl_ms, "nccl_all_gather_tflops_whole_job": afl / (nccl_ms * 1e-3) / 1e12}
        if fused_ms is not None:
            extras["attn_fwd_b8_h32_s8192_d128_causal_sharded"]["fused_matches_nccl_result"] = fused_matches
        sb.synchronize()
        del q, k, v, o_slab, o_full

    # ---- roofline of the dominant kernel ---------------------------------------------------------
    timed_region_s = ms_total * 1e-3
    peak_key = "bf16_tflops_sustained" if timed_region_s > 1.0 else "bf16_tflops"
    per_gpu_flops = flops / p
    gemm_ms = ms_step  # one step = one GEMM pass (N = 1: exactly one launch of gemm_tn_kernel)
    achieved = per_gpu_flops / (gemm_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peaks[peak_key], "unit": "TFLOP/s",
        "frac": achieved / peaks[peak_key], "traffic": GEMM_DRAM_TRAFFIC_BYTES if p == 1 else None,
        "peak_source": f"{peak_src} {peak_key}", "frac_of_nominal_dense_bf16": achieved / NOMINAL_BF16_TFLOPS,
        "kernel": "gemm_tn_pair_wide_kernel<bf16>", "algorithmic_flops_per_launch": per_gpu_flops,
    }
    if p > 1:
        roofline["note"] = "per-GPU share of the whole step (GEMM chunks + all-gather + unshard), not the kernel alone"

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
        "roofline": roofline, "e2e_matches_device_result": e2e_check == 0.0,
    }
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
