#!/usr/bin/env python
"""Benchmark of the fp32-accurate GEMM hot path.

    python bench.py --gpus 1 --steps K --warmup W            this library, one B200
    torchrun ... bench.py --gpus N --steps K --warmup W      N-column-sharded over N GPUs
    python bench.py --impl reference ...                     the reference's own CPU matmul

A step is one product C = A x B of the large-square configuration: 16384^3 fp32, A and B
i.i.d. N(0, 1/K) (seeded, generated on the device: synthetic), B and C split by column blocks
over the ranks, every rank ending with all of C.  Total work is fixed as N grows (strong
scaling).  At N = 1 the 4096^3 product of the headline metric is measured too and reported
under "gemm_4096".

One JSON line is printed by rank 0.  `value` is useful TFLOP/s = 2*M*N*K / time (the three
TF32 products per term and the split are overhead, not counted).  `roofline.achieved` counts
the tensor-core math actually issued per GPU (3 x useful in the default 3xTF32 mode) against a fixed
peak: TF32 nominal = 1/2 of the pool's measured bf16 rate (MEASURED_PEAKS.json); the cuBLAS TF32
rate of the same run is carried beside it as context.

Timing: a warm-up of --warmup steps and at least --warm-seconds of back-to-back steps (so that
every N starts its timed region in the same power state), then windows of exactly --steps steps,
each between a barrier + synchronize on both sides and timed with CUDA events (max over ranks),
repeated until a second has been timed; the median window is reported.  Every rank samples its own
GPU's clocks; `timing.gpu_cycles_per_step_all_gpus` lets scaling be compared clock for clock.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fp32-accurate GEMM TFLOP/s at 4096^3 (1 GPU) and 16384^3 (1/2/4/8 B200), % roofline"
BIG = 16384
SMALL = 4096


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--size", type=int, default=BIG, help="square size of the main workload")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32"])
    ap.add_argument("--no-extras", action="store_true", help="skip 4096^3, e2e and the CPU baseline")
    ap.add_argument("--only", default="", help="with --suite engine: run only the shapes whose name contains this text")
    ap.add_argument("--with-cpu", action="store_true",
                    help="with --suite engine: also time the reference CPU matmul of each shape on the host cores")
    ap.add_argument("--no-peak", action="store_true", help="skip the cuBLAS TF32 context measurement (profiling runs)")
    ap.add_argument("--warm-seconds", type=float, default=2.0,
                    help="minimum duration of the untimed warm-up loop (same power state at every N)")
    ap.add_argument("--max-windows", type=int, default=50,
                    help="upper bound on the timed windows of --steps steps (1 for profiling runs)")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE",
                    help="library option (b200_gemm_set_option), e.g. --opt pdl=0; repeatable")
    ap.add_argument("--suite", default="", choices=["", "engine", "accuracy"],
                    help="'engine': time every GEMM of the char-LM, CNN and relu-sparse configurations "
                         "(one JSON line per shape) instead of the large-square benchmark")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        """`gpu`: what `nvidia-smi -i` takes — an index or, better, the GPU's UUID (an index means the
        physical GPU of that number, which is not the CUDA device of that number once
        CUDA_VISIBLE_DEVICES remaps them)."""
        self.gpu = gpu
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples taken while the GPU was actually loaded: the upper half by power draw
        if sm:
            cut = statistics.median(power) if power else 0
            loaded = [c for c, p in zip(sm, power) if p >= cut] or sm
            return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                    "samples": len(sm), "power_w_max": max(power) if power else None}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}


def gpu_identity(torch, local: int):
    """(`nvidia-smi -i` selector, PCI bus id) of CUDA device `local`."""
    props = torch.cuda.get_device_properties(local)
    uuid = getattr(props, "uuid", None)
    sel = f"GPU-{uuid}" if uuid is not None and not str(uuid).startswith("GPU-") else (str(uuid) if uuid else str(local))
    try:
        bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    except AttributeError:
        bus = None
    return sel, bus


def bind_host_thread_near_gpu(bus_id):
    """Runs this process on the CPU cores NVML lists as local to the GPU, so that the page-locked host
    buffers it allocates next sit in that socket's memory (first touch) and uploads do not cross the
    socket link.  Returns the previous affinity mask (to restore), or None when nothing was changed.
    Only this process's CPU affinity is touched; nothing of the GPU is."""
    if not bus_id or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {w * 64 + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        before = os.sched_getaffinity(0)
        cpus &= before
        if not cpus or cpus == before:
            return None
        os.sched_setaffinity(0, cpus)
        return before
    except Exception:
        return None


# ------------------------------------------------------------------------------------------
# shared by both arms
# ------------------------------------------------------------------------------------------
def make_config(n: int, world: int, exchange: str, precision: str) -> dict:
    """The `config` object of the line; the reference arm prints the same one (it times the CPU on
    the same workload), so that the two arms can be compared key by key."""
    return {"workload": f"fp32 GEMM {n}^3, A,B ~ N(0,1/K) seed 1, C N-column-sharded over {world} GPU(s), "
                        f"every rank ends with all of C",
            "M": n, "N": n, "K": n, "exchange": exchange if world > 1 else "none", "precision": precision,
            "l2": "operands (1 GiB each) far exceed L2; no flush needed" if n >= 8192
            else "operands and result together exceed L2; launches back to back"}


def measured_peaks() -> dict:
    """Denominators of the roofline: the pool's measured copy bandwidth and cuBLAS bf16 rates.  TF32
    is not measured there; the nominal ratio (TF32 dense = 1/2 bf16 dense on this part) is applied to
    the measured bf16 figures."""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": d.get("hbm_gbs", 6650.0), "tf32_burst": 0.5 * d["bf16_tflops"],
                "tf32_sustained": 0.5 * d["bf16_tflops_sustained"], "kind": "of measured",
                "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"]}
    return {"hbm_gbs": 6650.0, "tf32_burst": 0.5 * 1590.0, "tf32_sustained": 0.5 * 1400.0, "kind": "of fallback",
            "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# ------------------------------------------------------------------------------------------
# CPU reference arm
# ------------------------------------------------------------------------------------------
def cpu_rows(a_rows, b, repeats: int = 1):
    """The reference's CPU matmul (the unmodified engine when it was built here, else the C
    restatement) on the given rows of A: rows are independent in its loop, so this is an exact slice
    of the full product.  Returns (result rows, seconds, info)."""
    from oracle import oracle_py as orc

    if orc.have_ref():
        kind, cores = "reference", orc.ref_threads()
        secs = orc.ref_matmul_time(a_rows, b, repeats)
        out = orc.matmul(a_rows, b)  # the restatement is bit-identical to the engine (tests/test_oracle.py)
    else:
        kind, cores = "port", os.cpu_count() or 1
        best, out = float("inf"), None
        for _ in range(repeats):
            t0 = time.perf_counter()
            out = orc.matmul(a_rows, b)
            best = min(best, time.perf_counter() - t0)
        secs = best
    return out, secs, {"kind": kind, "cores": cores}


def synthetic_host_inputs(n: int, rows: int):
    import numpy as np

    rng = np.random.default_rng(1)
    scale = 1.0 / np.sqrt(n)
    a = (rng.standard_normal((rows, n), dtype=np.float32) * scale).astype(np.float32)
    b = (rng.standard_normal((n, n), dtype=np.float32) * scale).astype(np.float32)
    return a, b


def run_reference(args):
    """The reference's own CPU implementation of the path on the box's host cores, all threads: each
    step multiplies a bounded row slice of the workload (rows are independent in its loop) and the
    line reports whole-product figures extrapolated from it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = args.size
    rows = 64 if n >= 8192 else 256
    a, b = synthetic_host_inputs(n, rows)
    _, _, info = cpu_rows(a, b)  # warm-up
    for _ in range(max(0, args.warmup - 1)):
        cpu_rows(a, b)
    secs = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        secs.append(cpu_rows(a, b)[1])
        if time.perf_counter() - t0 > 150:
            break
    slice_s = statistics.mean(secs)
    value = 2.0 * rows * n * n / slice_s / 1e12
    step_ms = slice_s * (n / rows) * 1e3
    sample = (f"each step times {rows} of the {n} output rows of the {n}^3 product on all host threads; value and "
              f"ms_per_step are the whole product's at that rate ({slice_s * 1e3:.1f} ms per slice)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(secs), "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": make_config(n, args.gpus, args.exchange, args.precision),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def measure_cublas_tf32(torch, dev, seconds: float = 1.5):
    """cuBLAS TF32 8192^3 in this run, for context (not the roofline's denominator): best single
    launch (burst) and the rate of a back-to-back loop (sustained)."""
    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn((n, n), device=dev)
        b = torch.randn((n, n), device=dev)
        c = torch.empty((n, n), device=dev)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(10):
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        burst = 2.0 * n ** 3 / best / 1e9
        iters = max(10, int(seconds * 1e3 / best))
        e0.record()
        for _ in range(iters):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        sustained = 2.0 * n ** 3 * iters / e0.elapsed_time(e1) / 1e9
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    del a, b, c
    return burst, sustained


# sm__pipe_tensor_cycles_active of the 4096^3 main launch (ncu capture summarised under profiles/)
TENSOR_PIPE_ACTIVE_NCU = {"value": 0.669, "source": "profiles/gemm_tf32_kernel_pair_4096cubed.md"}
# dram__bytes_read.sum + dram__bytes_write.sum of the launches of one 16384^3 product on one GPU
DRAM_TRAFFIC_16384 = {"value": 34620849664, "source": "profiles/gemm_tf32_kernel_pair_16384cubed_dram.md"}


def run_b200(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.load()  # raises if the CUDA library is missing: there is no fallback
    for item in args.opt:
        name, _, val = item.partition("=")
        pkg.set_option(name, int(val))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    precision = pkg.PRECISION_3XTF32 if args.precision == "3xtf32" else pkg.PRECISION_TF32
    kfac = 3 if args.precision == "3xtf32" else 1
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather_objects(obj):
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    n = args.size
    gen = torch.Generator(device=dev).manual_seed(1)  # same bytes on every rank
    A = torch.randn((n, n), device=dev, generator=gen) / n ** 0.5
    B = torch.randn((n, n), device=dev, generator=gen) / n ** 0.5
    exchange = args.exchange if world > 1 else "none"
    op = None
    if world == 1:
        # one GPU holds every column: the plain entry point with its workspace, which lets the planner
        # split the tiles of a mostly empty last wave along K
        C = torch.empty((n, n), device=dev)
        ws_bytes = pkg.workspace_bytes(1, n, n, n)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

        def step():
            pkg.gemm(A, B, C, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n, precision=precision,
                     workspace=ws if ws_bytes else None, workspace_bytes=ws_bytes)
    else:
        try:
            op = pkg.shard.ColumnShardedMatmul(n, n, n, rank=rank, world=world, device=dev, mode=args.exchange,
                                               precision=precision)
        except Exception as exc:  # symmetric memory unavailable: the NCCL gather still works
            if args.exchange != "fused":
                raise
            if rank == 0:
                print(f"[bench] fused exchange unavailable ({exc!r}); using the NCCL all-gather", file=sys.stderr)
            exchange = "nccl"
            op = pkg.shard.ColumnShardedMatmul(n, n, n, rank=rank, world=world, device=dev, mode="nccl",
                                               precision=precision)
        C = op.C

        def step():
            op(A, B)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_window(fn, steps):
        """Exactly `steps` calls between a barrier + synchronize on both sides; CUDA events on the
        launching stream; max over ranks."""
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # Every rank samples its own GPU's clocks from here to the end of the timed windows.
    gpu_sel, gpu_bus = gpu_identity(torch, local)
    sampler = ClockSampler(gpu_sel)
    sampler.start()
    # Warm-up: the requested count (at least 3) AND at least two seconds of back-to-back steps, at
    # every N, so that every GPU is in the same power state (power-capped, clocks settled) when the
    # timed windows start — a 0.1 s window on a cold GPU runs at boost clocks a long step never sees.
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    t_warm = time.perf_counter()
    warm_steps = max(3, args.warmup)
    while args.warm_seconds > 0:
        for _ in range(4):
            step()
        warm_steps += 4
        torch.cuda.synchronize()
        go_on = 1.0 if time.perf_counter() - t_warm < args.warm_seconds else 0.0
        if max_over_ranks(go_on) == 0.0:  # every rank leaves the loop in the same round
            break
    pkg.status()
    # Timed: windows of exactly --steps steps, repeated until at least one second has been timed;
    # the line reports the median window.
    launches0 = pkg.launch_count()
    windows = [timed_window(step, args.steps)]
    while sum(windows) < 1000.0 and len(windows) < args.max_windows:
        windows.append(timed_window(step, args.steps))
    launches = (pkg.launch_count() - launches0) // len(windows)
    clocks_mine = sampler.stop()
    pkg.status()
    total_ms = statistics.median(windows)
    ms = total_ms / args.steps
    flops = 2.0 * n ** 3
    value = flops / ms / 1e9
    clocks_all = gather_objects(clocks_mine)
    mhz = [c.get("sm_mhz") for c in clocks_all if c.get("sm_mhz")]
    slowest_mhz = min(mhz) if mhz else None

    # ------------------------------------------------------------------ parity of the timed result
    # Every rank checks sampled rows of ITS copy of C, all columns (so the peers' stores are covered),
    # against fp64 on the device; two checksums of the whole of C are compared across ranks.
    rows = torch.arange(3, n, max(1, n // 16), device=dev)
    ref = A[rows].double() @ B.double()
    err = float(((C[rows].double() - ref).abs() / ref.abs().clamp(min=1.0)).max().item())
    del ref
    err_all = max_over_ranks(err)
    sums = (int(C.view(torch.int32).sum(dtype=torch.int64).item()),
            int(C.view(torch.int32)[:, ::3].sum(dtype=torch.int64).item()))
    same_everywhere = len(set(gather_objects(sums))) == 1

    # ------------------------------------------------------------------ what the exchange costs (N > 1)
    breakdown = None
    if world > 1 and exchange == "fused" and not args.no_extras:
        own, peer_c = op.C, [op._peer_views[0][(rank + i) % world] for i in range(world)]

        def local_only():
            pkg.gemm_colshard(A, B, [own], M=n, N=n, K=n, col0=op.col0, cols=op.cols, lda=n, ldb=n, ldc=n,
                              precision=precision)

        def with_stores():
            pkg.gemm_colshard(A, B, peer_c, M=n, N=n, K=n, col0=op.col0, cols=op.cols, lda=n, ldb=n, ldc=n,
                              precision=precision)

        k = max(4, args.steps)
        t_local = timed_window(local_only, k) / k
        t_stores = timed_window(with_stores, k) / k
        t_full = timed_window(step, k) / k
        breakdown = {"own_columns_only_ms": t_local, "with_peer_stores_ms": t_stores, "with_barriers_ms": t_full,
                     "peer_stores_cost_ms": t_stores - t_local, "barriers_cost_ms": t_full - t_stores,
                     "nvlink_bytes_stored_per_rank": int(n * op.cols * 4 * (world - 1)),
                     "note": "product kernel on this rank's columns with no peer destination / with the forwarder "
                             "warps storing every tile into the peers / the whole call with its two barriers; "
                             "each timed like the main windows (max over ranks)"}

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm_steps, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, fp32 accumulate)"
            if kfac == 3 else "tf32", "data": "synthetic",
            "config": make_config(n, world, exchange, args.precision),
            "gpu_launches": int(launches),
            "timing": {"windows_ms": [round(w, 3) for w in windows], "reported": "median window / steps",
                       "warmup_seconds": round(time.perf_counter() - t_warm, 2),
                       "cycles_per_step_slowest_gpu": ms * 1e3 * slowest_mhz if slowest_mhz else None,
                       "gpu_cycles_per_step_all_gpus": ms * 1e3 * slowest_mhz * world if slowest_mhz else None,
                       "note": "cycles = ms x median SM MHz under load of the slowest-clocked rank; "
                               "clock-normalised scaling efficiency = gpu_cycles_per_step_all_gpus at N=1 / at N"},
            "clocks": {"sm_mhz": slowest_mhz, "sm_max_mhz": clocks_all[0].get("sm_max_mhz"),
                       "reasons": sorted({r for c in clocks_all for r in c.get("reasons", [])}),
                       "sm_mhz_per_rank": [c.get("sm_mhz") for c in clocks_all],
                       "power_w_max_per_rank": [c.get("power_w_max") for c in clocks_all]},
            "check": {"scaled_max_error_vs_fp64_sampled_rows_max_over_ranks": err_all,
                      "all_ranks_hold_the_same_c": same_everywhere},
        }
        if breakdown:
            line["exchange_breakdown"] = breakdown
        achieved = kfac * value / world  # tensor-core TF32 math per GPU
        line["roofline"] = {
            "bound": "tensor", "achieved": achieved, "peak": peaks["tf32_sustained"], "unit": "TFLOP/s",
            "frac": achieved / peaks["tf32_sustained"],
            "traffic": DRAM_TRAFFIC_16384["value"] if (n == BIG and kfac == 3 and world == 1) else None,
            "traffic_source": DRAM_TRAFFIC_16384["source"] if (n == BIG and kfac == 3 and world == 1) else None,
            "algorithmic_bytes": int(3 * n * n * 4),
            "peak_kind": f"TF32 nominal = 1/2 measured bf16 (sustained, {peaks['bf16_tflops_sustained']} TFLOP/s; "
                         f"{peaks['kind']}): this step runs inside a long power-capped loop",
            "note": f"achieved = {kfac} x useful TFLOP/s per GPU: the TF32 tensor-core math issued per product "
                    f"(2*M*N*K*{kfac}) / mean time of one product by CUDA events; at one GPU a product is the main "
                    f"launch plus the K-split launch of the last wave's tiles and their reduction",
            "useful_tflops_per_gpu": value / world, "useful_frac": value / world / peaks["tf32_sustained"],
            "k_factor": kfac, "tensor_pipe_active_ncu": TENSOR_PIPE_ACTIVE_NCU,
        }

    extras = (world == 1 and not args.no_extras)
    if extras and not args.no_peak:
        time.sleep(2.0)  # let the power-capped clocks recover before the burst measurement
        burst, sustained = measure_cublas_tf32(torch, dev)
        line["roofline"]["cublas_tf32_same_run"] = {"burst": burst, "sustained": sustained,
                                                    "vs_cublas_tf32_sustained": kfac * value / sustained}

    # ------------------------------------------------------------------ 4096^3 (N = 1)
    if extras:
        m = SMALL
        a4 = torch.randn((m, m), device=dev, generator=gen) / m ** 0.5
        b4 = torch.randn((m, m), device=dev, generator=gen) / m ** 0.5
        c4 = torch.empty((m, m), device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        ws4_bytes = pkg.workspace_bytes(1, m, m, m)  # the tail-wave plan needs scratch for its partials
        ws4 = torch.empty(max(ws4_bytes, 16), dtype=torch.uint8, device=dev)

        def launch4():
            pkg.gemm(a4, b4, c4, batch=1, M=m, N=m, K=m, lda=m, ldb=m, ldc=m, precision=precision,
                     workspace=ws4, workspace_bytes=ws4_bytes)

        time.sleep(2.0)  # the state a burst peak is measured in: idle for two seconds
        for _ in range(3):
            launch4()
        torch.cuda.synchronize()
        iters = max(20, args.steps)
        e0.record()
        for _ in range(iters):
            launch4()
        e1.record()
        torch.cuda.synchronize()
        b2b_ms = e0.elapsed_time(e1) / iters
        times = []
        for _ in range(iters):
            flush.fill_(1)
            e0.record()
            launch4()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        pkg.status()
        cold_ms = statistics.mean(times)
        tf = 2.0 * m ** 3 / b2b_ms / 1e9
        line["gemm_4096"] = {
            "workload": "fp32 GEMM 4096^3, N(0,1/K); back-to-back launches (A+B+C = 201 MB exceed L2)",
            "ms_per_launch": b2b_ms, "useful_tflops": tf, "tensor_math_tflops": kfac * tf,
            "frac_of_tf32_peak": kfac * tf / peaks["tf32_burst"], "peak": peaks["tf32_burst"],
            "peak_kind": f"TF32 nominal = 1/2 measured bf16 (burst, {peaks['bf16_tflops']} TFLOP/s; {peaks['kind']}); "
                         f"this product is timed as a burst too: 20 launches after 2 s idle",
            "tensor_pipe_active_ncu": TENSOR_PIPE_ACTIVE_NCU,
            "l2_flushed": {"ms_mean": cold_ms, "ms_best": min(times),
                           "useful_tflops": 2.0 * m ** 3 / cold_ms / 1e9,
                           "note": "single launch after a 256 MB fill that evicts L2"},
        }
        del a4, b4, c4, flush

    # ------------------------------------------------------------------ engine-sized products (N = 1)
    if extras:
        line["engine"] = engine_block(pkg, torch, dev, peaks["hbm_gbs"])

    # ------------------------------------------------------------------ end to end, host buffers
    e2e = None
    if not args.no_extras:
        reps = max(2, min(args.steps, 4))
        old_affinity = bind_host_thread_near_gpu(gpu_bus)  # pinned buffers in the GPU's own socket
        if world == 1:
            h_a = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
            h_b = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
            h_c = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
            h_a.copy_(A)
            h_b.copy_(B)
            keep_rows = A[:64].cpu().numpy()  # for the CPU leg below
            b_host = h_b.numpy()
            del C
            torch.cuda.empty_cache()
            na, nb, nc = h_a.numpy(), h_b.numpy(), h_c.numpy()

            def e2e_step():
                pkg.matmul_host(na, nb, nc, batch=1, rows=n, inner=n, cols=n, a_batched=False, b_batched=False)

            path = "b200_matmul_f32_host: pinned host A, B -> device, kernels, C -> pinned host, synchronised"
            h2d, d2h = int(2 * n * n * 4), int(n * n * 4)
        else:
            hop = pkg.shard.ShardedHostMatmul(n, n, n, rank=rank, world=world, device=dev)
            per, cols, col0 = hop.rows_per_rank, hop.cols, hop.col0
            h_a = torch.empty((per, n), dtype=torch.float32, pin_memory=True)
            h_b = torch.empty((n, max(cols, 1)), dtype=torch.float32, pin_memory=True)[:, :cols]
            h_c = torch.empty((n, max(cols, 1)), dtype=torch.float32, pin_memory=True)[:, :cols]
            h_a.copy_(A[rank * per:(rank + 1) * per])
            h_b.copy_(B[:, col0:col0 + cols])
            na, nb, nc = h_a.numpy(), h_b.numpy(), h_c.numpy()

            def e2e_step():
                hop(na, nb, nc)

            path = ("b200_matmul_f32_host_sharded: every rank uploads 1/N of A's rows and its own columns of B "
                    "from pinned memory, the rows are all-gathered over NVLink chunk by chunk, strips are "
                    "multiplied as they arrive, the own columns of C return to pinned memory; bytes are the "
                    "whole job's (sum over ranks)")
            h2d, d2h = int(2 * n * n * 4), int(n * n * 4)
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            e2e_step()
        torch.cuda.synchronize()
        secs = max_over_ranks((time.perf_counter() - t0) / reps)
        barrier()
        pkg.status()
        # the result that came back, against fp64 of the same inputs (sampled rows, own columns)
        rr = torch.arange(5, n, max(1, n // 8), device=dev)
        if world == 1:
            got = torch.from_numpy(nc[rr.cpu().numpy()]).to(dev)
            ref = A[rr].double() @ B.double()
        else:
            got = torch.from_numpy(np.ascontiguousarray(nc[rr.cpu().numpy()])).to(dev)
            ref = A[rr].double() @ B[:, col0:col0 + cols].double()
        e2e_err = max_over_ranks(float(((got.double() - ref).abs() / ref.abs().clamp(min=1.0)).max().item())
                                 if got.numel() else 0.0)
        if old_affinity is not None:
            os.sched_setaffinity(0, old_affinity)  # the CPU leg below uses every host thread again
        e2e = {"value": flops / secs / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": secs * 1e3, "path": path,
               "host_buffers_bound_to_gpu_socket": old_affinity is not None,
               "scaled_max_error_vs_fp64_sampled_rows": e2e_err}
    if rank == 0:
        line["e2e"] = e2e

    # ------------------------------------------------------------------ CPU baseline + parity (rank 0, N = 1)
    if rank == 0 and world == 1 and not args.no_extras:
        # the reference's CPU matmul on the first 64 rows of the SAME A and B: timed (the baseline) and,
        # as the checker, compared with the rows the device path returned and with fp64
        cpu_out, cpu_s, info = cpu_rows(keep_rows, b_host)
        tf = 2.0 * 64 * n * n / cpu_s / 1e12
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
                                "sample": f"64 of {n} output rows of this {n}^3 product (rows are independent in "
                                          f"the reference loop), all host threads, {cpu_s * 1e3:.0f} ms"}
        ref64 = keep_rows.astype(np.float64) @ b_host.astype(np.float64)
        gpu_rows = nc[:64]

        def scaled(x, y):
            return float(np.max(np.abs(x - y) / np.maximum(1.0, np.abs(y))))

        line["parity"] = {"rows": 64, "gpu_vs_cpu_loop": scaled(gpu_rows, cpu_out), "gpu_vs_fp64": scaled(gpu_rows, ref64),
                          "cpu_loop_vs_fp64": scaled(cpu_out, ref64), "bar_vs_cpu_loop": 1e-5,
                          "note": "scaled max error |x - y| / max(1, |y|) on the first 64 rows of the product that "
                                  "the end-to-end call returned"}
    elif rank == 0:
        line["cpu_baseline"] = None

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# engine-sized shapes (configurations 1-4): HBM- or latency-bound, reported per launch
# ------------------------------------------------------------------------------------------
ENGINE_SHAPES = [
    # name, batch, M, N, K, transA, transB, a_batched, b_batched
    ("cfg1 bench 512^3", 1, 512, 512, 512, 0, 0, 0, 0),
    ("cfg2 proj fwd 2048x96x96", 1, 2048, 96, 96, 0, 0, 0, 0),
    ("cfg2 fused-QKV fwd 2048x96x288", 1, 2048, 288, 96, 0, 0, 0, 0),
    ("cfg2 FF1 fwd 2048x96x384", 1, 2048, 384, 96, 0, 0, 0, 0),
    ("cfg2 FF2 fwd 2048x384x96", 1, 2048, 96, 384, 0, 0, 0, 0),
    ("cfg2 LM head fwd 2048x96x121", 1, 2048, 121, 96, 0, 0, 0, 0),
    ("cfg2 dX=dY.W^T (FF1) NT", 1, 2048, 96, 384, 0, 1, 0, 0),
    ("cfg2 dW=X^T.dY (FF1) TN", 1, 96, 384, 2048, 1, 0, 0, 0),
    ("cfg2 scores Q.K^T NT b128", 128, 64, 64, 24, 0, 1, 1, 1),
    ("cfg2 context P.V b128", 128, 64, 24, 64, 0, 0, 1, 1),
    ("cfg2 dV=P^T.dO TN b128", 128, 64, 24, 64, 1, 0, 1, 1),
    ("cfg3 conv1 fwd cols.W^T NT", 1, 50176, 8, 9, 0, 1, 0, 0),
    ("cfg3 conv1 dW cols^T.dOut TN", 1, 9, 8, 50176, 1, 0, 0, 0),
    ("cfg3 conv2 fwd NT", 1, 12544, 16, 72, 0, 1, 0, 0),
    ("cfg3 conv2 dW TN", 1, 72, 16, 12544, 1, 0, 0, 0),
    ("cfg3 conv2 dCols", 1, 12544, 72, 16, 0, 0, 0, 0),
    ("cfg3 dense fwd 64x784x10", 1, 64, 10, 784, 0, 0, 0, 0),
    ("cfg4 relu-sparse 2048^3 NN", 1, 2048, 2048, 2048, 0, 0, 0, 0),
    ("cfg4 relu-sparse 2048^3 NT", 1, 2048, 2048, 2048, 0, 1, 0, 0),
    ("cfg4 relu-sparse 2048^3 TN", 1, 2048, 2048, 2048, 1, 0, 0, 0),
]


CONV_SHAPES = [
    # name, n, c, h, w, out_c, k, stride, pad
    ("cfg3 conv1 layer, implicit GEMM (64,1,28,28)->8", 64, 1, 28, 28, 8, 3, 1, 1),
    ("cfg3 conv2 layer, implicit GEMM (64,8,14,14)->16", 64, 8, 14, 14, 16, 3, 1, 1),
]


def cpu_matmul_time(batch, M, N, K, a_batched, b_batched, relu_a=False):
    """The reference's CPU matmul of one shape on all host threads (the compiled reference engine
    if it was built, else the C restatement): best of a few runs, bounded to about a second.
    The transposed forms are timed as the plain product of the same size — the reference
    materialises the transpose first, so this is a lower bound of what they cost it."""
    import numpy as np

    from oracle import oracle_py as orc

    rng = np.random.default_rng(0)
    a = rng.standard_normal(((batch,) if a_batched else ()) + (M, K), dtype=np.float32)
    if relu_a:  # half of A exactly zero: the reference's loop skips those terms
        a = np.maximum(a, np.float32(0))
    b = rng.standard_normal(((batch,) if b_batched else ()) + (K, N), dtype=np.float32)
    use_ref = orc.have_ref()
    best, spent, runs = float("inf"), 0.0, 0
    while runs < 3 or (spent < 0.3 and runs < 50):
        if use_ref:
            t = orc.ref_matmul_time(a, b, 1)
        else:
            t0 = time.perf_counter()
            orc.matmul(a, b)
            t = time.perf_counter() - t0
        best, spent, runs = min(best, t), spent + t, runs + 1
        if spent > 1.5:
            break
    return {"us": round(best * 1e6, 1), "kind": "reference" if use_ref else "port",
            "cores": orc.ref_threads() if use_ref else os.cpu_count(), "runs": runs}


# the engine-sized products the default line carries (configurations 1-3): name, batch, M, N, K, tA, tB, ab, bb
ENGINE_BLOCK_SHAPES = [
    ("cfg1 512^3", 1, 512, 512, 512, 0, 0, 0, 0),
    ("cfg2 FF1 fwd 2048x96x384", 1, 2048, 384, 96, 0, 0, 0, 0),
    ("cfg2 dW=X^T.dY 96x2048x384 TN (split-K)", 1, 96, 384, 2048, 1, 0, 0, 0),
    ("cfg2 scores Q.K^T 128x[64x24x64] NT", 128, 64, 64, 24, 0, 1, 1, 1),
    ("cfg3 conv1 im2col 50176x9x8 NT", 1, 50176, 8, 9, 0, 1, 0, 0),
]


def engine_block(pkg, torch, dev, hbm_gbs):
    """Per-launch figures of the engine-sized products and of the two convolution layers as single
    implicit-GEMM kernels: microseconds back to back and after an L2 flush, the fraction of the
    measured HBM bandwidth their algorithmic bytes reach, and the reference's CPU matmul of the same
    shape on the host cores beside it."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gen = torch.Generator(device=dev).manual_seed(2)
    out = []

    def time_call(launch):
        for _ in range(5):
            launch()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(50):
            launch()
        e1.record()
        torch.cuda.synchronize()
        hot = e0.elapsed_time(e1) / 50 * 1e3
        cold = []
        for _ in range(10):
            flush.fill_(1)
            e0.record()
            launch()
            e1.record()
            torch.cuda.synchronize()
            cold.append(e0.elapsed_time(e1) * 1e3)
        pkg.status()
        return hot, statistics.median(cold)

    for name, batch, M, N, K, tA, tB, ab, bb in ENGINE_BLOCK_SHAPES:
        a_shape = ((batch,) if ab else ()) + ((K, M) if tA else (M, K))
        b_shape = ((batch,) if bb else ()) + ((N, K) if tB else (K, N))
        A = torch.randn(a_shape, device=dev, generator=gen)
        B = torch.randn(b_shape, device=dev, generator=gen)
        C = torch.empty((batch, M, N), device=dev)
        ws_bytes = pkg.workspace_bytes(batch, M, N, K)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

        def launch():
            pkg.gemm(A, B, C, batch=batch, M=M, N=N, K=K, transA=bool(tA), transB=bool(tB),
                     lda=a_shape[-1], ldb=b_shape[-1], ldc=N, strideA=(K * M if ab else 0),
                     strideB=(K * N if bb else 0), strideC=M * N, workspace=ws, workspace_bytes=ws_bytes)

        hot, cold = time_call(launch)
        bytes_alg = 4.0 * ((batch if ab else 1) * M * K + (batch if bb else 1) * K * N + batch * M * N)
        cpu = cpu_matmul_time(batch, M, N, K, ab, bb)
        out.append({"shape": name, "us_back_to_back": round(hot, 2), "us_l2_flushed": round(cold, 2),
                    "algorithmic_bytes": int(bytes_alg),
                    "frac_of_measured_hbm": round(bytes_alg / cold / 1e3 / hbm_gbs, 4),
                    "kernels_per_call": pkg.plan(batch, M, N, K, ws_bytes)["kernels"],
                    "cpu_reference_us": cpu["us"], "cpu_kind": cpu["kind"], "cpu_cores": cpu["cores"]})
    for name, n, c, h, w, out_c, k, stride, pad in CONV_SHAPES:
        x = torch.rand((n, c, h, w), device=dev, generator=gen)
        wt = torch.randn((out_c, c, k, k), device=dev, generator=gen)
        b = torch.randn((out_c,), device=dev, generator=gen)
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = torch.empty((n, out_c, oh, ow), device=dev)

        def launch():
            pkg.lib.conv2d_forward(x, wt, b, y, n=n, c=c, h=h, w=w, out_c=out_c, kh=k, kw=k, stride=stride, pad=pad)

        hot, cold = time_call(launch)
        bytes_alg = 4.0 * (x.numel() + wt.numel() + b.numel() + y.numel())
        cpu = cpu_matmul_time(1, n * oh * ow, out_c, c * k * k, 0, 0)
        out.append({"shape": name, "us_back_to_back": round(hot, 2), "us_l2_flushed": round(cold, 2),
                    "algorithmic_bytes": int(bytes_alg),
                    "frac_of_measured_hbm": round(bytes_alg / cold / 1e3 / hbm_gbs, 4), "kernels_per_call": 1,
                    "cpu_reference_us": cpu["us"], "cpu_kind": cpu["kind"], "cpu_cores": cpu["cores"],
                    "cpu_note": "the reference's CPU matmul of the layer's im2col product alone (its im2col, bias "
                                "and permute passes are not counted)"})
    return out


def run_engine_suite(args):
    import torch

    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.load()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks_file.read_text()).get("hbm_gbs", 6650.0) if peaks_file.exists() else 6650.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gen = torch.Generator(device=dev).manual_seed(2)
    for name, batch, M, N, K, tA, tB, ab, bb in ENGINE_SHAPES:
        if args.only and args.only not in name:
            continue
        a_shape = ((batch,) if ab else ()) + ((K, M) if tA else (M, K))
        b_shape = ((batch,) if bb else ()) + ((N, K) if tB else (K, N))
        A = torch.randn(a_shape, device=dev, generator=gen)
        if "relu" in name or "FF2" in name:
            A = torch.relu(A)
        B = torch.randn(b_shape, device=dev, generator=gen)
        C = torch.empty((batch, M, N), device=dev)
        ws_bytes = pkg.workspace_bytes(batch, M, N, K)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

        def launch():
            pkg.gemm(A, B, C, batch=batch, M=M, N=N, K=K, transA=bool(tA), transB=bool(tB),
                     lda=a_shape[-1], ldb=b_shape[-1], ldc=N, strideA=(K * M if ab else 0),
                     strideB=(K * N if bb else 0), strideC=M * N, workspace=ws, workspace_bytes=ws_bytes)

        for _ in range(5):
            launch()
        torch.cuda.synchronize()
        iters = 50
        e0.record()
        for _ in range(iters):
            launch()
        e1.record()
        torch.cuda.synchronize()
        hot_us = e0.elapsed_time(e1) / iters * 1e3
        cold = []
        for _ in range(10):
            flush.fill_(1)
            e0.record()
            launch()
            e1.record()
            torch.cuda.synchronize()
            cold.append(e0.elapsed_time(e1) * 1e3)
        pkg.status()
        cold_us = statistics.median(cold)
        bytes_alg = 4.0 * ((batch if ab else 1) * M * K + (batch if bb else 1) * K * N + batch * M * N)
        flops = 2.0 * batch * M * N * K
        record = {
            "shape": name, "batch": batch, "M": M, "N": N, "K": K, "transA": tA, "transB": tB,
            "us_per_launch_back_to_back": round(hot_us, 2), "us_per_launch_l2_flushed": round(cold_us, 2),
            "algorithmic_bytes": int(bytes_alg), "useful_tflops_back_to_back": round(flops / hot_us / 1e6, 3),
            "hbm_gbs_l2_flushed": round(bytes_alg / cold_us / 1e3, 1),
            "frac_of_measured_hbm": round(bytes_alg / cold_us / 1e3 / hbm, 4),
            "kernels_per_call": pkg.plan(batch, M, N, K, ws_bytes)["kernels"]}
        if args.with_cpu:
            record["cpu"] = cpu_matmul_time(batch, M, N, K, ab, bb, relu_a=("relu" in name or "FF2" in name))
            record["gpu_over_cpu"] = round(record["cpu"]["us"] / hot_us, 1)
        print(json.dumps(record), flush=True)
    # the attention core of the char-LM block: 128 heads of 64 x 24, causal mask — one fused kernel
    # against the five separate steps (two products through this library, the rest through torch)
    q, k, v = (torch.randn((32, 4, 64, 24), device=dev, generator=gen) for _ in range(3))
    mask = torch.triu(torch.full((64, 64), -1e9, device=dev), 1)

    def separate():
        s_ = pkg.attention_scores(q, k, 24 ** -0.5, mask)
        w_ = torch.softmax(s_, dim=-1)
        return pkg.matmul(w_.reshape(128, 64, 64), v.reshape(128, 64, 24))

    def time_layer(label, fn, kernels, note="includes the output allocations by the Python wrapper"):
        if args.only and args.only not in label:
            return
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(50):
            fn()
        e1.record()
        torch.cuda.synchronize()
        pkg.status()
        print(json.dumps({"shape": label, "us_per_launch_back_to_back": round(e0.elapsed_time(e1) / 50 * 1e3, 2),
                          "kernels_per_call": kernels, "note": note}), flush=True)

    time_layer("cfg2 attention core fused (32,4,64,24)", lambda: pkg.scaled_dot_product_attention(q, k, v, mask), 1)
    time_layer("cfg2 attention core as 3 kernels (scores+mask, softmax, P.V)", separate, 3)
    # the same core on the (B, S, d_model) projections: heads split and merged by strides, against
    # the reference's three permute copies in, one out
    qp, kp, vp = (torch.randn((32, 64, 96), device=dev, generator=gen) for _ in range(3))

    def permuted():
        q4, k4, v4 = (t.reshape(32, 64, 4, 24).permute(0, 2, 1, 3).contiguous() for t in (qp, kp, vp))
        o4 = pkg.scaled_dot_product_attention(q4, k4, v4, mask)
        return o4.permute(0, 2, 1, 3).reshape(32, 64, 96).contiguous()

    time_layer("cfg2 attention, heads by strides (32,64,96)x3 -> (32,64,96)",
               lambda: pkg.multi_head_attention_core(qp, kp, vp, 4, mask), 1)
    time_layer("cfg2 attention, heads by permute copies + fused core", permuted, 5)
    # backward of the attention core: one kernel against the reference's sequence (product backward of
    # W x V, softmax backward, scale, product backward of Q x K^T, transpose) on the same GPU
    go = torch.randn((32, 4, 64, 24), device=dev, generator=gen)

    def composed_attention_backward():
        s_ = pkg.attention_scores(q, k, 24 ** -0.5, mask)
        w_ = torch.softmax(s_, dim=-1).reshape(128, 64, 64)
        dw, dv_ = pkg.matmul_backward(w_, v.reshape(128, 64, 24), go.reshape(128, 64, 24))
        ds_ = (w_ * (dw - (dw * w_).sum(-1, keepdim=True))) * (24 ** -0.5)
        kt = k.reshape(128, 64, 24).transpose(1, 2).contiguous()
        dq_, dkt = pkg.matmul_backward(q.reshape(128, 64, 24), kt, ds_)
        return dq_, dkt.transpose(1, 2).contiguous(), dv_

    time_layer("cfg2 attention backward fused (32,4,64,24)",
               lambda: pkg.scaled_dot_product_attention_backward(q, k, v, go, mask), 1)
    time_layer("cfg2 attention backward composed (scores, softmax, 4 products, softmax backward, transposes)",
               composed_attention_backward, 13)
    # The products of one char-LM Transformer block as five layer calls, eager and replayed from a CUDA
    # graph (no host cost per launch): fused Q|K|V projection, attention on its column slices, output
    # projection, FF1 + ReLU, FF2.
    if not args.only or "block" in args.only:
        xb = torch.randn((2048, 96), device=dev, generator=gen)
        wb = {k: torch.randn(s_, device=dev, generator=gen) * 0.1
              for k, s_ in (("qkv", (96, 288)), ("bqkv", (288,)), ("out", (96, 96)), ("bout", (96,)),
                            ("ff1", (96, 384)), ("b1", (384,)), ("ff2", (384, 96)), ("b2", (96,)))}

        def block():
            qkv = pkg.linear(xb, wb["qkv"], wb["bqkv"]).view(32, 64, 288)
            ctx = pkg.multi_head_attention_core(qkv[:, :, :96], qkv[:, :, 96:192], qkv[:, :, 192:], 4, mask)
            o = pkg.linear(ctx.view(2048, 96), wb["out"], wb["bout"])
            return pkg.linear(pkg.linear(o, wb["ff1"], wb["b1"], relu=True), wb["ff2"], wb["b2"])

        time_layer("cfg2 block products, 5 layer calls (6 kernels), eager", block, 6)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            block()
        time_layer("cfg2 block products, 5 layer calls (6 kernels), CUDA graph replay", graph.replay, 6,
                   note="one replay = all six kernels; no host work per launch")
    # whole Conv2d layers (im2col + product + bias + permute in the reference) as one kernel, and
    # their gradients (product backward over the columns + col2im in the reference)
    import torch.nn.functional as F

    for name, n, c, h, w, out_c, k, stride, pad in CONV_SHAPES:
        x = torch.rand((n, c, h, w), device=dev, generator=gen)
        wt = torch.randn((out_c, c, k, k), device=dev, generator=gen)
        b = torch.randn((out_c,), device=dev, generator=gen)
        time_layer(name, lambda: pkg.conv2d(x, wt, b, stride=stride, padding=pad), 1)
        y = pkg.conv2d(x, wt, b, stride=stride, padding=pad)
        dy = torch.randn(y.shape, device=dev, generator=gen)

        # The reference's sequence — im2col, product backward (two products), col2im, column sums —
        # with one index gather / one index scatter-add standing in for its im2col / col2im kernels.
        oh, ow = y.shape[2], y.shape[3]
        hp, wp = h + 2 * pad, w + 2 * pad
        ar = torch.arange
        row_base = ((ar(n, device=dev).view(n, 1, 1) * c * hp + ar(oh, device=dev).view(1, oh, 1) * stride) * wp
                    + ar(ow, device=dev).view(1, 1, ow) * stride).reshape(-1, 1)
        col_off = ((ar(c, device=dev).view(c, 1, 1) * hp + ar(k, device=dev).view(1, k, 1)) * wp
                   + ar(k, device=dev).view(1, 1, k)).reshape(1, -1)
        gather_idx = (row_base + col_off).reshape(-1)

        def composed_backward():
            xp = F.pad(x, (pad, pad, pad, pad))
            cols = xp.reshape(-1)[gather_idx].reshape(n * oh * ow, c * k * k)
            g = dy.reshape(n, out_c, -1).transpose(1, 2).reshape(-1, out_c).contiguous()
            wt_t = wt.reshape(out_c, -1).t().contiguous()   # the (K, outC) operand of the forward product
            dcols, dwt = pkg.matmul_backward(cols, wt_t, g)
            dxp = torch.zeros(n * c * hp * wp, device=dev)
            dxp.index_add_(0, gather_idx, dcols.reshape(-1))
            dx = dxp.reshape(n, c, hp, wp)[:, :, pad:pad + h, pad:pad + w].contiguous()
            return dx, dwt, g.sum(0)

        time_layer(name.replace("layer", "gradients (dx, dW, db)"),
                   lambda: pkg.conv2d_backward(x, wt, dy, stride=stride, padding=pad), 3)
        time_layer(name.replace("layer", "gradients composed: im2col gather, 2 products, col2im scatter, sums"),
                   composed_backward, 11)


def run_accuracy_suite(args):
    """Error of the device result and of the reference's CPU loop against an fp64 product of the same
    fp32 inputs (seeded with the reference's generator), for several promotion intervals and for
    the TF32 mode.  One JSON line per configuration."""
    import numpy as np
    import torch

    import __graft_entry__ as entry
    from oracle import oracle_py as orc

    pkg = entry.load_package()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)

    def case(name, a, b):
        A, B = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        M, K = a.shape
        N = b.shape[1]
        ref = A.double() @ B.double()
        cpu = torch.from_numpy(orc.matmul(a, b)).to(dev)

        def scaled(x, y=ref):
            return float(((x.double() - y.double()).abs() / y.double().abs().clamp(min=1)).max().item())

        def fro(x):
            return float(((x.double() - ref).norm() / ref.norm()).item())

        row = {"config": name, "M": M, "N": N, "K": K,
               "cpu_loop_vs_fp64": {"scaled_max": scaled(cpu), "frobenius_rel": fro(cpu)}}
        for pe in (1, 2, 4, 16):
            pkg.set_option("promote_every", pe)
            C = torch.empty((M, N), device=dev)
            pkg.gemm(A, B, C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N)
            pkg.status()
            row[f"3xtf32_promote_every_{pe}"] = {"scaled_max_vs_fp64": scaled(C), "frobenius_rel_vs_fp64": fro(C),
                                                 "scaled_max_vs_cpu_loop": scaled(C, cpu)}
        pkg.set_option("promote_every", 0)  # back to automatic
        C = torch.empty((M, N), device=dev)
        pkg.gemm(A, B, C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, precision=pkg.PRECISION_TF32)
        pkg.status()
        row["tf32"] = {"scaled_max_vs_fp64": scaled(C), "frobenius_rel_vs_fp64": fro(C)}
        print(json.dumps(row), flush=True)

    r = orc.Rng(0)
    case("cfg1 512^3 U[-1,1] seed 0", r.rand((512, 512), -1, 1), r.rand((512, 512), -1, 1))
    r = orc.Rng(2)
    case("cfg2 2048x96x384 N(0,1) x Xavier seed 2", r.randn((2048, 96)), r.rand((96, 384), -0.1118, 0.1118))
    r = orc.Rng(4)
    a = np.maximum(r.randn((2048, 2048)), 0).astype(np.float32)
    case("cfg4 2048^3 relu-sparse seed 4", a, r.randn((2048, 2048)))
    r = orc.Rng(1)
    case("cfg5 4096^3 N(0,1/K) seed 1", r.randn((4096, 4096), 0, 4096 ** -0.5), r.randn((4096, 4096), 0, 4096 ** -0.5))


def main():
    args = parse_args()
    if args.suite == "engine":
        run_engine_suite(args)
        return
    if args.suite == "accuracy":
        run_accuracy_suite(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
