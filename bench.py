#!/usr/bin/env python3
"""Benchmark of the prism_b200 hot path on one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemm_bf16|sgemm|scan] [--no-extras]

Prints ONE JSON line.  The headline workload is the bf16 GEMM D = A * B^T at
M = N = K = 8192 (rows of M sharded over the GPUs, B replicated; total work
fixed, so scaling is "strong"); `--workload` selects the FP32 SGEMM (4096^3,
alpha = 1.5, beta = 0.5) or the uint32 scan (2^28 on one GPU, 2^30 sharded)
instead.  With the default workload the line also carries the other two
families under "extras" (one GPU: kernel timings, roofline fractions, the
reference's own kernels recompiled for sm_100 timed beside ours).

A "step" is one launch of the path through the C ABI on inputs resident in HBM;
steps are timed with CUDA events on the launching stream, the job time is the
maximum over ranks.  "e2e" repeats the measurement through the host-buffer
operators (pinned host memory -> device -> kernel -> host inside the timed
region).  `--impl reference` times the CPU path (NumPy, all host threads) on a
bounded sample of the same workload; under torchrun only rank 0 does so.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GEMM_S = 8192
SGEMM_S = 4096
SCAN_N1 = 1 << 28
SCAN_NG = 1 << 30

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel,
# from the ncu captures whose summaries sit in the profiles/ folder (None = not captured).
NCU_TRAFFIC_BYTES = {
    "gemm_bf16": 1015.4e6,  # 8192^3: 888.5 MB read + 126.9 MB written
    "gemm_bf16_half": 501.6e6,  # 4096 x 8192 x 8192, one of two GPUs' share: 435.0 MB read + 66.6 MB written
    "sgemm": 631.5e6,       # 4096^3: 569.1 MB read + 62.3 MB written
    "scan": 1916.4e6,       # 2^28: 4 x the 479.1 MB captured at 2^26 (an undercount: the last writes are still in L2 when the kernel ends)
}


def use_all_host_threads() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core the
    process may run on.  Must be called before NumPy (and with it the BLAS library) is imported."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS", "GOTO_NUM_THREADS"):
        os.environ[var] = str(n)
    return n


def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "sm_max_mhz": 1965.0,
            "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs (NVML, every 5 ms;
    read-only queries).  Falls back to `nvidia-smi -lms` if NVML cannot be loaded."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples: list[tuple[float, float, int]] = []
        self.sm_max = None
        self.stop_flag = threading.Event()
        self.thread = None
        self.proc = None
        self.lines: list[str] = []
        self.nvml = None

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.nvml = (pynvml, h)
        except Exception:
            self.nvml = None
        if self.nvml is not None:
            def loop():
                nv, h = self.nvml
                get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
                while not self.stop_flag.is_set():
                    try:
                        self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                             nv.nvmlDeviceGetPowerUsage(h) / 1000.0, int(get_reasons(h))))
                    except Exception:
                        pass
                    time.sleep(0.005)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self, all_samples: bool = False) -> dict:
        """Median SM clock of the samples taken under load: the half with the highest power draw, or
        (all_samples) every sample, for a window that is load from end to end."""
        reasons: set[str] = set()
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            for _, _, mask in self.samples:
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        reasons.add(name)
            sm = sorted(c for c, _, _ in self.samples)
            power = [p for _, p, _ in self.samples]
            smax = self.sm_max
        elif self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            sm, smax, power = [], None, []
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for ln in self.lines:
                f = [t.strip() for t in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); smax = float(f[2]); power.append(float(f[3]))
                except ValueError:
                    continue
                for nm, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
            sm.sort()
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML and no nvidia-smi"]}
        # the samples with the highest power draw are the ones taken under load
        if self.nvml is not None and self.samples:
            by_power = sorted(self.samples, key=lambda t: t[1])
            load = sorted(c for c, _, _ in (by_power if all_samples else by_power[len(by_power) // 2:]))
        else:
            load = sm[: max(1, len(sm) // 2)] if sm else []
        return {"sm_mhz": (load[len(load) // 2] if load else None), "sm_max_mhz": smax,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- helpers
def dist_setup(n_gpus: int):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries the one JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(step, steps: int, warmup: int, world: int, reset=None, wait_for_result: bool = False):
    """Per-step CUDA-event timing on the current stream; returns (total_ms_max_over_ranks, per_step_ms list).
    wait_for_result: the host waits for each step to finish before it issues the next, as a caller does who
    reads the step's result from host memory (the end-to-end measurements)."""
    import torch
    for _ in range(warmup):
        if reset:
            reset()
        step()
    barrier(world)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        if reset:
            reset()          # outside the timed span of the step
        starts[i].record()
        step()
        ends[i].record()
        if wait_for_result:
            ends[i].synchronize()
    barrier(world)
    per = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    return max_over_ranks(sum(per), world), per


def measure_host_link(dev, mib: int = 256, world: int = 1) -> dict:
    """Pinned host <-> device copy rates of this GPU's link, best of 6 (GB/s).  One direction at a time; with
    several ranks all of them copy in that direction at once (a barrier keeps the directions apart), which is what
    a rank gets while its neighbours upload or download too."""
    import torch
    n = mib << 20
    h = torch.empty(n, dtype=torch.uint8).pin_memory()
    d = torch.empty(n, dtype=torch.uint8, device=dev)
    out = {}
    for name, (dst, src) in (("h2d_gbs", (d, h)), ("d2h_gbs", (h, d))):
        barrier(world)
        best = float("inf")
        dst.copy_(src, non_blocking=True)      # warm-up: first touch of the pages
        torch.cuda.synchronize()
        for _ in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            b.synchronize()
            best = min(best, a.elapsed_time(b))
        out[name] = n / (best * 1e-3) / 1e9
    barrier(world)
    out["sample_mib"] = mib
    out["how"] = "each direction alone" + (f", all {world} ranks copying at once" if world > 1 else "")
    return out


def host_link(args, dev) -> dict:
    """The link rates, measured once per run."""
    if getattr(args, "link", None) is None:
        args.link = measure_host_link(dev, world=int(os.environ.get("WORLD_SIZE", "1")))
    return args.link


def link_fraction(e2e_ms: float, h2d_bytes: float, d2h_bytes: float, link: dict) -> float:
    """Time the link needs for the step's copies at its measured rates (the two directions run at once)
    divided by the measured end-to-end time: 1.0 = the step costs nothing beyond its copies."""
    need_ms = max(h2d_bytes / link["h2d_gbs"], d2h_bytes / link["d2h_gbs"]) / 1e6
    return need_ms / e2e_ms


def sustained_run(step, flops_per_step: float, seconds: float, gpu_index: int, peak_sustained: float) -> dict:
    """The same launch back to back for `seconds`, with the clock sampler running over the whole window
    (hundreds of samples), so that what the kernel sustains under the power cap is visible."""
    import torch
    step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(); step(); b.record(); b.synchronize()
    reps = max(50, int(seconds * 1e3 / max(a.elapsed_time(b), 1e-3)))
    sampler = ClockSampler(gpu_index)
    sampler.start()
    a.record()
    for _ in range(reps):
        step()
    b.record()
    b.synchronize()
    clocks = sampler.stop(all_samples=True)
    ms = a.elapsed_time(b) / reps
    value = flops_per_step / (ms * 1e-3) / 1e12
    return {"value": value, "unit": "TFLOP/s", "launches": reps, "window_s": ms * reps * 1e-3, "ms_per_launch": ms,
            "sm_mhz_median": clocks.get("sm_mhz"), "power_w_max": clocks.get("power_w_max"), "reasons": clocks.get("reasons"),
            "samples": clocks.get("samples"), "frac": value / peak_sustained,
            "peak": peak_sustained, "peak_source": "measured cuBLAS bf16, back to back for seconds",
            "gflops_per_sm_mhz": (value * 1e3 / clocks["sm_mhz"]) if clocks.get("sm_mhz") else None}


def ref_gpu_lib():
    p = ROOT / "oracle" / "_ref" / "libprism_ref.so"
    if not p.exists():
        return None
    lib = ctypes.CDLL(str(p))
    lib.ref_sgemm.argtypes = [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                                   ctypes.c_void_p]
    lib.ref_scan_workspace_size.argtypes = [ctypes.c_size_t]
    lib.ref_scan_workspace_size.restype = ctypes.c_size_t
    lib.ref_scan.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def gemm_bf16_config(S: int, world: int) -> dict:
    """The `config` of the bf16 workload; both arms print this one dict."""
    rows = S // world
    return {"workload": "gemm_bf16 %dx%dx%d, A and B K-major, C column-major, values 0.1*normal bf16" % (S, S, S),
            "M": S, "N": S, "K": S, "sharding": f"rows of M over {world} GPU(s), B replicated, no collective",
            "rows_per_gpu": rows, "l2": "inputs larger than L2 (A+B = %d MiB per GPU)" % ((rows + S) * S * 2 >> 20)}


def sgemm_config(S: int, world: int) -> dict:
    return {"workload": "sgemm %dx%dx%d row-major, kernel 5, A/B/C uniform[-1,1)" % (S, S, S), "M": S, "N": S, "K": S,
            "alpha": 1.5, "beta": 0.5, "sharding": f"rows of M over {world} GPU(s), B replicated, no collective",
            "rows_per_gpu": S // world,
            "l2": "C restored from a pristine copy before every step (untimed), which also displaces L2"}


def scan_config(n_total: int, world: int, schedule: str) -> dict:
    return {"workload": f"scan n=2^{n_total.bit_length() - 1} int32 values in {{0,1}}, in place", "n": n_total,
            "sharding": f"contiguous chunks over {world} GPU(s); " +
            ("single pass" if world == 1 else
             f"{schedule}: " + ("one launch per GPU: chunk total stored into every peer's memory over NVLink, then the scan; "
                                "no collective" if schedule == "peer_words" else
                                "rank 0 owns the first half chunk and the last chunk of the array and scans them without adding "
                                "them up first (8 B/element), the other ranks one chunk each in one launch (total stored into every "
                                "peer's memory over NVLink, then the scan: 12 B/element); n = (world + 0.5) chunks; no collective"
                                if schedule == "head_tail" else "one all-gather of per-shard totals")),
            "elements_per_gpu": -(-n_total // world),
            "l2": "input restored from a pristine copy before every step (untimed); array larger than L2"}


# --------------------------------------------------------------------------- workloads (ours)
def run_gemm_bf16(args, world, rank, peaks):
    import torch
    import prism_b200 as pb
    from prism_b200 import host, sharded
    dev = torch.device("cuda", torch.cuda.current_device())
    S = args.size or GEMM_S
    plan = sharded.RowShardedGemmBF16(S, S, S)
    rows = plan.rows
    g = torch.Generator(device=dev).manual_seed(1234)           # B: same on every rank
    B = (torch.randn((S, S), device=dev, generator=g) * 0.1).to(torch.bfloat16)
    ga = torch.Generator(device=dev).manual_seed(5678 + rank)   # A: this rank's rows
    A = (torch.randn((rows, S), device=dev, generator=ga) * 0.1).to(torch.bfloat16)
    C = torch.empty((S, rows), dtype=torch.bfloat16, device=dev)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    l0 = pb.launch_count()
    total_ms, per = time_steps(lambda: plan(A, B, C), args.steps, args.warmup, world)
    launches = (pb.launch_count() - l0) - args.warmup
    clocks = sampler.stop()
    ms = total_ms / args.steps
    flops = 2.0 * S * S * S
    value = flops / (ms * 1e-3) / 1e12

    # spot check of this rank's result against fp64 on rows of C^T (= rows of B) that cover both CTAs of a pair and
    # both row blocks of a 512-row tile, the middle and the end (bf16-rounded inputs)
    n_idx = sorted({0, 127, 128, 255, 256, 383, 384, 511, S // 2 - 1, S // 2, S - 1})
    A64 = A.double()

    def rows_ok(c_rows):
        ref = (B[n_idx].double() @ A64.t()).cpu()
        got = c_rows.double().cpu()
        rms = float(ref.pow(2).mean().sqrt())
        return bool(((got - ref).abs() <= 1e-2 * ref.abs() + 1e-2 * rms).all())

    ok = rows_ok(C[n_idx])

    # what the kernel sustains: back to back for seconds, clocks sampled over the whole window
    sustained = None
    if args.sustained_seconds > 0:
        sustained = sustained_run(lambda: plan(A, B, C), 2.0 * rows * S * S, args.sustained_seconds,
                                  torch.cuda.current_device(), peaks["bf16_tflops_sustained"])

    # end to end through the host-buffer operator: pinned host arrays in, pinned host array out
    link = host_link(args, dev)
    op = sharded.ShardedHostGemmBF16(S, S, S, dev, wait_limit_s=10.0)    # ranks of a benchmark can be seconds apart at their first call
    Ah = host.pinned_near(dev, (rows, S), torch.bfloat16); Ah.copy_(A)
    Bh = host.pinned_near(dev, (S, S), torch.bfloat16); Bh.copy_(B)
    Ch = host.pinned_near(dev, (S, rows), torch.bfloat16)
    e2e_steps = max(3, min(args.steps, 5))
    e2e_total, _ = time_steps(lambda: op(Ah, Bh, Ch), e2e_steps, 2, world, wait_for_result=True)
    e2e_ms = e2e_total / e2e_steps
    torch.cuda.synchronize()
    e2e_ok = rows_ok(Ch[n_idx].to(dev))
    del A64
    e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": op.h2d_bytes, "d2h_bytes_per_step": op.d2h_bytes,
           "link_gbs": link, "frac_of_link": link_fraction(e2e_ms, op.h2d_bytes, op.d2h_bytes, link),
           "spot_check_ok": e2e_ok,
           "pipeline": ("%d blocks of B rows, upload / kernel / download on three streams" % op.steps) if world == 1 else
                       ("per rank: its rows of A and 1/%d of B over PCIe; B completed in %d blocks over NVLink into local HBM (%s), "
                        "each followed by the GEMM on that block of columns and its download"
                        % (world, op.steps, "one-sided pushes with flags, own kernels" if op.exchange == "peer"
                           else "in-place NCCL all-gathers"))}

    kernel_ms = sum(per) / len(per)     # this rank's kernel: rows x S x S
    achieved = 2.0 * rows * S * S / (kernel_ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    roofline = {"bound": "tensor", "kernel": ("cutlass_my_h100_match_no_tail_pair_wide[_fill]<16> (tcgen05, cta_group::2, 512 x 256 tiles, "
                                               "persistent over the CTA pairs; a last wave of at most half the pairs' tiles is cut into halves)"
                           if (rows % 256 == 0 and S % 512 == 0 and rows * S * S >= 2 ** 35)
                           else "cutlass_my_h100_match_no_tail family (tcgen05), form chosen by shape"), "achieved": achieved,
                "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{peaks['source']} cuBLAS bf16 burst (the timed region is a burst of %d launches)" % args.steps,
                "frac_of_nominal_2250": achieved / 2250.0,
                "traffic": (NCU_TRAFFIC_BYTES["gemm_bf16"] if (S == GEMM_S and world == 1) else
                            NCU_TRAFFIC_BYTES["gemm_bf16_half"] if (S == GEMM_S and world == 2) else None)}
    line = {"metric": "bf16 GEMM TFLOP/s (D = A*B^T, M=N=K=%d, fp32 accumulate, bf16 out)" % S, "value": value,
            "unit": "TFLOP/s", "ms_per_step": ms, "scaling": "strong", "dtype": "bf16",
            "config": gemm_bf16_config(S, world),
            "roofline": roofline, "sustained": sustained, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "spot_check_ok": ok and e2e_ok, "parity": "fp64 NumPy/torch on the bf16-rounded inputs; unpinned by the reference "
            "(its kernel is wgmma, sm_90a only)"}
    return line


def run_sgemm(args, world, rank, peaks, steps=None, warmup=None):
    import torch
    import prism_b200 as pb
    from prism_b200 import host, sharded
    steps = steps or args.steps
    warmup = warmup or args.warmup
    dev = torch.device("cuda", torch.cuda.current_device())
    S = (args.size if args.workload == "sgemm" else 0) or SGEMM_S
    plan = sharded.RowShardedSgemm(S, S, S, kernel=5)
    rows = plan.rows
    g = torch.Generator(device=dev).manual_seed(4321)
    B = torch.rand((S, S), device=dev, generator=g) * 2 - 1
    ga = torch.Generator(device=dev).manual_seed(8765 + rank)
    A = torch.rand((rows, S), device=dev, generator=ga) * 2 - 1
    C0 = torch.rand((rows, S), device=dev, generator=ga) * 2 - 1
    C = C0.clone()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    l0 = pb.launch_count()
    total_ms, per = time_steps(lambda: plan(1.5, A, B, 0.5, C), steps, warmup, world, reset=lambda: C.copy_(C0))
    launches = (pb.launch_count() - l0) - warmup
    clocks = sampler.stop()
    ms = total_ms / steps
    flops = 2.0 * S * S * S
    ridx = [0, 1, rows // 2, rows - 1]
    ref = 1.5 * (A[ridx].double() @ B.double()) + 0.5 * C0[ridx].double()
    err = float((C[ridx].double() - ref).abs().max() / ref.abs().max())

    op = sharded.ShardedHostSgemm(S, S, S, dev, wait_limit_s=10.0)
    Ah, Bh, Ch = A.cpu().pin_memory(), B.cpu().pin_memory(), C0.cpu().pin_memory()
    e2e_steps = 3
    e2e_total, _ = time_steps(lambda: op(1.5, Ah, Bh, 0.5, Ch), e2e_steps, 1, world, wait_for_result=True)
    e2e_ms = e2e_total / e2e_steps

    kernel_ms = sum(per) / len(per)
    achieved = 2.0 * rows * S * S / (kernel_ms * 1e-3) / 1e12
    sm_max = peaks.get("sm_max_mhz", 1965.0)
    peak_nominal = 148 * 128 * 2 * sm_max * 1e6 / 1e12
    sm_load = clocks.get("sm_mhz") or sm_max
    peak_at_clock = 148 * 128 * 2 * sm_load * 1e6 / 1e12
    return {"metric": "FP32 SGEMM TFLOP/s (C = 1.5*A*B + 0.5*C, M=N=K=%d, pure FFMA)" % S,
            "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "scaling": "strong", "dtype": "f32",
            "config": sgemm_config(S, world),
            "roofline": {"bound": "fp32_ffma", "kernel": "my_sgemm_kernel_5<packed>", "achieved": achieved,
                         "peak": peak_nominal, "unit": "TFLOP/s", "frac": achieved / peak_nominal,
                         "peak_source": "148 SMs x 128 FMA/clk x 2 x %.0f MHz (max SM clock)" % sm_max,
                         "frac_at_observed_clock": achieved / peak_at_clock, "observed_sm_mhz": sm_load,
                         "traffic": NCU_TRAFFIC_BYTES["sgemm"] if (S == SGEMM_S and world == 1) else None},
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": op.h2d_bytes, "d2h_bytes_per_step": op.d2h_bytes,
                    "link_gbs": host_link(args, dev),
                    "frac_of_link": link_fraction(e2e_ms, op.h2d_bytes, op.d2h_bytes, host_link(args, dev)),
                    "pipeline": ("%d blocks of rows of M, upload / kernel / download on three streams" % op.blocks) +
                                ("" if op.exchange == "none" else "; each rank uploads 1/%d of B and pushes it to the others over NVLink" % world)},
            "gpu_launches": launches, "clocks": clocks, "rel_error_sampled_rows": err, "spot_check_ok": err <= 1e-5}


def run_scan(args, world, rank, peaks, steps=None, warmup=None):
    import torch
    import prism_b200 as pb
    from prism_b200 import host, sharded
    steps = steps or args.steps
    warmup = warmup or args.warmup
    dev = torch.device("cuda", torch.cuda.current_device())
    n_total = (1 << args.scan_log2n) if args.scan_log2n else (SCAN_N1 if world == 1 else SCAN_NG)
    # Two to four GPUs: rank 0 owns a head and a tail of the array (8 B/element there, 12 elsewhere, 1.5 chunks on
    # rank 0) unless a schedule is asked for by name or the ranks have no peer-writable memory.  Measured at 2^30:
    # 2 GPUs 9.36 against 7.93 TB/s with equal chunks, 4 GPUs 16.4 against 15.6, 8 GPUs 28.9 against 29.8 (rank 0's
    # three launches and the others' wait for its word outweigh the 6 % that the layout saves there), hence the limit.
    scan, head = None, 0
    want_head_tail = args.scan_schedule == "head_tail" or (args.scan_schedule is None and 2 <= world <= 4)
    if world > 1 and want_head_tail and sharded.head_tail_bounds(n_total, world) is not None:
        pieces = sharded.head_tail_pieces(n_total, world, rank)
        n = sum(b - a for a, b in pieces)
        head = pieces[0][1] - pieces[0][0] if rank == 0 else 0
        try:
            scan = sharded.ShardedScan(n, dev, schedule="head_tail", head=head, wait_limit_s=10.0)
        except RuntimeError:
            scan, head = None, 0          # raised on every rank alike: fall through to equal chunks
    if scan is None:
        lo, hi = sharded.chunk_bounds(n_total, world, rank)
        n = hi - lo
        scan = sharded.ShardedScan(n, dev, schedule=None if args.scan_schedule == "head_tail" else args.scan_schedule,
                                   wait_limit_s=10.0)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    # The untimed restore before each step copies the same number of elements on every rank (the largest local
    # size), so that unequal pieces do not make the ranks enter the step apart.
    n_buf = n
    if scan.schedule == "head_tail":
        h_, c_, t_ = sharded.head_tail_bounds(n_total, world)
        n_buf = max(h_ + t_, c_)
    src_buf = torch.randint(0, 2, (n_buf,), dtype=torch.int32, device=dev, generator=g)
    x_buf = torch.empty_like(src_buf)
    src, x = src_buf[:n], x_buf[:n]
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    l0 = pb.launch_count()
    total_ms, per = time_steps(lambda: scan(x), steps, warmup, world, reset=lambda: x_buf.copy_(src_buf))
    head_tail = scan.schedule == "head_tail"
    per_step = (3 if rank == 0 else 1) if head_tail else (1 if (world == 1 or scan.schedule == "peer_words") else 2)
    sharded_kernel = scan.schedule in ("peer_words", "head_tail") and scan.slots is not None   # also on one GPU when asked for by name
    launches = (pb.launch_count() - l0) - warmup * per_step
    clocks = sampler.stop()
    ms = total_ms / steps
    nbytes = 8.0 * n_total
    # properties: differences reproduce the input; last element = carry + int64 total of the shard
    if head_tail and rank == 0:
        # the head starts from zero; the tail from the sum of every rank's word (rank 0's word is the head's total)
        words = scan.totals_int64()
        ok = (bool(torch.equal(x[1:head] - x[:head - 1], src[1:head])) and bool(torch.equal(x[head + 1:] - x[head:-1], src[head + 1:]))
              and (int(x[head - 1]) & 0xFFFFFFFF) == (int(src[:head].sum(dtype=torch.int64)) & 0xFFFFFFFF) == words[0]
              and (int(x[-1]) & 0xFFFFFFFF) == ((sum(words) + int(src[head:].sum(dtype=torch.int64))) & 0xFFFFFFFF))
    else:
        carry = sum(scan.totals_int64()[:rank]) if world > 1 else 0
        ok = bool(torch.equal(x[1:] - x[:-1], src[1:])) and (int(x[-1]) & 0xFFFFFFFF) == ((carry + int(src.sum(dtype=torch.int64))) & 0xFFFFFFFF)

    e2e = None
    if world == 1:
        op = host.HostScan(n, dev)
        xh = src.cpu().pin_memory()
        e2e_total, _ = time_steps(lambda: op(xh), 3, 1, world, wait_for_result=True)
        e2e_ms = e2e_total / 3
        e2e = {"value": nbytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": op.h2d_bytes, "d2h_bytes_per_step": op.d2h_bytes,
               "link_gbs": host_link(args, dev),
               "frac_of_link": link_fraction(e2e_ms, op.h2d_bytes, op.d2h_bytes, host_link(args, dev)),
               "pipeline": "%d blocks chained by their last element, upload / kernel / download on three streams" % op.blocks}
    kernel_ms = sum(per) / len(per)
    achieved = 8.0 * n / (kernel_ms * 1e-3) / 1e9
    peak = peaks["hbm_gbs"]
    return {"metric": "uint32 inclusive scan GB/s (8 bytes per element)", "value": nbytes / (ms * 1e-3) / 1e9,
            "unit": "GB/s", "ms_per_step": ms, "scaling": "strong" if world > 1 else "weak", "dtype": "u32",
            "config": scan_config(n_total, world, scan.schedule),
            "roofline": {"bound": "hbm", "kernel": ("scan_kernel_sharded (12 B/element moved: chunk total, then scan; rank 0 scans a head "
                                                   "and a tail of 1.5 chunks at 8 B/element with scan_kernel and scan_kernel_sharded)"
                                                   if head_tail else
                                                   "scan_kernel_sharded (12 B/element moved: chunk total, then scan)" if sharded_kernel
                                                   else "scan_kernel"), "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"{peaks['source']} copy bandwidth",
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "note": "8 B/element algorithmic; per-GPU rate of the whole step (all passes)",
                         "traffic": NCU_TRAFFIC_BYTES["scan"] if n == SCAN_N1 else None},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "spot_check_ok": ok}


def reference_kernels_beside(peaks):
    """The reference's own generated kernels, recompiled for sm_100, on the same inputs and GPU (one GPU)."""
    import torch
    lib = ref_gpu_lib()
    if lib is None:
        return {"unavailable": "oracle/_ref/libprism_ref.so not built"}
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    S = SGEMM_S
    A = torch.rand((S, S), device=dev) * 2 - 1
    B = torch.rand((S, S), device=dev) * 2 - 1
    C = torch.rand((S, S), device=dev) * 2 - 1
    ms, _ = time_steps(lambda: lib.ref_sgemm(5, S, S, S, 1.5, A.data_ptr(), B.data_ptr(), 0.5, C.data_ptr()), 5, 2, 1)
    out["sgemm_4096_my_sgemm_kernel_5_tflops"] = 2.0 * S ** 3 / (ms / 5 * 1e-3) / 1e12
    del A, B, C
    n = SCAN_N1
    src = torch.randint(0, 2, (n,), dtype=torch.int32, device=dev)
    x = torch.empty_like(src)
    ws = torch.empty(lib.ref_scan_workspace_size(n), dtype=torch.uint8, device=dev)
    ms, _ = time_steps(lambda: lib.ref_scan(n, x.data_ptr(), ws.data_ptr()), 5, 2, 1, reset=lambda: x.copy_(src))
    out["scan_2^28_scan_kernel_gbs"] = 8.0 * n / (ms / 5 * 1e-3) / 1e9
    out["bf16_gemm"] = "reference kernel is wgmma (sm_90a) only: does not assemble for sm_100"
    return out


# --------------------------------------------------------------------------- CPU arm
def cpu_gemm_bf16(sample_rows: int, reps: int):
    import numpy as np
    from oracle import cpu_oracle as O
    S = GEMM_S
    rng = np.random.default_rng(0)
    A = O.bf16_bits_to_f32(O.f32_to_bf16_bits((0.1 * rng.standard_normal((sample_rows, S))).astype(np.float32)))
    B = O.bf16_bits_to_f32(O.f32_to_bf16_bits((0.1 * rng.standard_normal((S, S))).astype(np.float32)))
    best = float("inf")
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        C = B @ A.T      # (N, rows): the reference's column-major C, fp32 accumulate (OpenBLAS sgemm)
        dt = time.perf_counter() - t0
        times.append(dt)
        best = min(best, dt)
    del C
    flops = 2.0 * sample_rows * S * S
    return flops, times


def cpu_sgemm(sample_rows: int, reps: int):
    import numpy as np
    S = SGEMM_S
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (sample_rows, S)).astype(np.float32)
    B = rng.uniform(-1, 1, (S, S)).astype(np.float32)
    C = rng.uniform(-1, 1, (sample_rows, S)).astype(np.float32)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        C = np.float32(1.5) * (A @ B) + np.float32(0.5) * C
        times.append(time.perf_counter() - t0)
    return 2.0 * sample_rows * S * S, times


def ref_cpu_lib():
    """The reference's own CPU scan loop (evals/4090_scan/scan_harness.cuh:30-36), compiled into oracle/_ref."""
    p = ROOT / "oracle" / "_ref" / "libref_cpu.so"
    if not p.exists():
        return None
    lib = ctypes.CDLL(str(p))
    lib.ref_scan_cpu.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    lib.ref_scan_cpu.restype = None
    return lib


def cpu_scan(n: int, reps: int):
    """Returns (bytes, times, kind): the reference's scan_cpu when it was built, else the NumPy port."""
    import numpy as np
    from oracle import cpu_oracle as O
    x = O.scan_inputs(n, seed=0, high=2)
    lib = ref_cpu_lib()
    out = np.empty_like(x)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        if lib is not None:
            lib.ref_scan_cpu(n, x.ctypes.data, out.ctypes.data)
        else:
            out = O.scan_cpu(x)
        times.append(time.perf_counter() - t0)
    if lib is not None:
        assert np.array_equal(out, O.scan_cpu(x))
    return 8.0 * n, times, ("reference" if lib is not None else "port")


def cpu_threads() -> int:
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 1) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    return os.cpu_count() or 1


def cpu_baseline(workload: str) -> dict:
    import numpy as np  # noqa: F401  (loads BLAS so that the thread count can be read)
    if workload == "gemm_bf16":
        rows = 2048
        work, times = cpu_gemm_bf16(rows, 3)
        return {"value": work / min(times) / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
                "sample": f"NumPy float32 matmul (BLAS, fp32 accumulate) on the bf16-rounded values, {rows} of the 8192 rows of M "
                          f"against all of B (N = K = 8192), best of 3; os.cpu_count() = {os.cpu_count()}"}
    if workload == "sgemm":
        rows = 2048
        work, times = cpu_sgemm(rows, 3)
        return {"value": work / min(times) / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
                "sample": f"NumPy float32 1.5*A@B+0.5*C, {rows} of the 4096 rows of M, best of 3; os.cpu_count() = {os.cpu_count()}"}
    n = 1 << 26
    work, times, kind = cpu_scan(n, 3)
    return {"value": work / min(times) / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
            "sample": ("the reference's own scan_cpu loop (oracle/_ref/libref_cpu.so)" if kind == "reference" else
                       "np.cumsum uint32 (the same loop as the reference's scan_cpu)") +
                      ", single thread, on 2^26 of the 2^28 elements, best of 3"}


def run_reference_arm(args):
    """CPU implementation of the path on the host cores; each step is a bounded sample of the workload.
    The line carries the same `config` as the GPU arm at this number of GPUs; what a step covers is in `sample`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    threads = use_all_host_threads()      # before NumPy loads its BLAS: torchrun exports OMP_NUM_THREADS=1
    world = max(1, args.gpus)
    steps, warmup = args.steps, args.warmup
    kind = "port"
    if args.workload == "gemm_bf16":
        rows = 1024
        work, times = cpu_gemm_bf16(rows, steps + warmup)
        unit, scale = "TFLOP/s", 1e12
        metric = "bf16 GEMM TFLOP/s (D = A*B^T, M=N=K=%d, fp32 accumulate, bf16 out)" % GEMM_S
        sample = f"NumPy float32 matmul on bf16-rounded values; each step = {rows} of the 8192 rows of M against all of B"
        cfg = gemm_bf16_config(GEMM_S, world)
        dtype, cores = "f32 on bf16-rounded inputs", cpu_threads()
    elif args.workload == "sgemm":
        rows = 1024
        work, times = cpu_sgemm(rows, steps + warmup)
        unit, scale = "TFLOP/s", 1e12
        metric = "FP32 SGEMM TFLOP/s (C = 1.5*A*B + 0.5*C, M=N=K=%d, pure FFMA)" % SGEMM_S
        sample = f"NumPy float32; each step = {rows} of the 4096 rows"
        cfg = sgemm_config(SGEMM_S, world)
        dtype, cores = "f32", cpu_threads()
    else:
        n = 1 << 25
        work, times, kind = cpu_scan(n, steps + warmup)
        unit, scale = "GB/s", 1e9
        metric = "uint32 inclusive scan GB/s (8 bytes per element)"
        sample = ("the reference's own scan_cpu loop" if kind == "reference" else "np.cumsum uint32") + \
            ", single thread; each step = 2^25 elements"
        cfg = scan_config(SCAN_N1 if world == 1 else SCAN_NG, world, args.scan_schedule or "peer_words")
        dtype, cores = "u32", 1
    timed = times[warmup:]
    ms = 1e3 * sum(timed) / len(timed)
    value = work / (ms * 1e-3) / scale
    return {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": dtype, "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind, "sample": sample +
                             f"; host threads offered to BLAS = {threads}, os.cpu_count() = {os.cpu_count()}; the reference has "
                             "no CPU GEMM and its bf16 kernel cannot run on sm_100, so the CPU path of the GEMMs is NumPy as "
                             "the benchmark definition prescribes"},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


# --------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["gemm_bf16", "sgemm", "scan"], default="gemm_bf16")
    ap.add_argument("--scan-schedule", choices=["head_tail", "peer_words", "reduce_then_scan", "scan_then_carry"], default=None,
                    help="sharded scan schedule (default: head_tail on 2 to 4 GPUs, peer_words on more, where the ranks can write each other's memory)")
    ap.add_argument("--size", type=int, default=0,
                    help="square GEMM size for --workload gemm_bf16/sgemm (default 8192 / 4096); smaller sizes are for profiling")
    ap.add_argument("--scan-log2n", type=int, default=0, help="scan length 2^k (default: 28 on one GPU, 30 sharded)")
    ap.add_argument("--sustained-seconds", type=float, default=2.5,
                    help="length of the back-to-back run that measures what the bf16 kernel sustains (0 = skip, e.g. under a profiler)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other two kernel families and the CPU baseline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        line = run_reference_arm(args)
        if line is not None:
            print(json.dumps(line), flush=True)
        return 0

    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: prism_b200 has no CPU path"}))
        return 1
    import prism_b200 as pb
    pb.load(build_if_missing=False)   # the CUDA library must be there; there is nothing to fall back to
    world, rank, local = dist_setup(args.gpus)
    peaks = load_peaks()
    runner = {"gemm_bf16": run_gemm_bf16, "sgemm": run_sgemm, "scan": run_scan}[args.workload]
    line = runner(args, world, rank, peaks)
    extras = {}
    if not args.no_extras and args.workload == "gemm_bf16":
        # the other two families at every N (sharded the same way), fewer steps
        extras["sgemm"] = run_sgemm(args, world, rank, peaks, steps=min(args.steps, 5), warmup=3)
        extras["scan"] = run_scan(args, world, rank, peaks, steps=min(args.steps, 10), warmup=3)
        if world == 1:
            extras["reference_kernels_sm100"] = reference_kernels_beside(peaks)
    code, msg = pb.last_error()
    if rank == 0:
        out = {"metric": line.pop("metric"), "value": line.pop("value"), "unit": line.pop("unit"), "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": line.pop("ms_per_step"), "higher_is_better": True,
               "scaling": line.pop("scaling"), "vs_baseline": None, "dtype": line.pop("dtype"), "data": "synthetic",
               "impl": "ours"}
        out.update(line)
        if world == 1 and not args.no_extras:
            out["cpu_baseline"] = cpu_baseline(args.workload)
            for k in ("sgemm", "scan"):
                if k in extras:
                    extras[k]["cpu_baseline"] = cpu_baseline(k)
        if extras:
            out["extras"] = extras
        out["library_status"] = {"code": code, "message": msg}
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return 0 if code == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
