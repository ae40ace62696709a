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
the tensor-core math actually issued (3 x useful in the default 3xTF32 mode) against the TF32
tensor-pipe rate measured in the same run with cuBLAS.
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
    ap.add_argument("--no-peak", action="store_true", help="skip the cuBLAS TF32 peak measurement (profiling runs)")
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

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
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


# ------------------------------------------------------------------------------------------
# CPU reference arm
# ------------------------------------------------------------------------------------------
def cpu_sample(n: int, rows: int, repeats: int = 1):
    """Times the reference's CPU matmul on `rows` rows of the n^3 product (rows are independent
    in its loop, so this is an exact slice of the full job).  Returns (TFLOP/s, info)."""
    import numpy as np

    from oracle import oracle_py as orc

    rng = np.random.default_rng(1)
    scale = 1.0 / np.sqrt(n)
    a = (rng.standard_normal((rows, n), dtype=np.float32) * scale).astype(np.float32)
    b = (rng.standard_normal((n, n), dtype=np.float32) * scale).astype(np.float32)
    if orc.have_ref():
        kind, cores = "reference", orc.ref_threads()
        secs = orc.ref_matmul_time(a, b, repeats)
    else:
        kind, cores = "port", os.cpu_count() or 1
        best = float("inf")
        for _ in range(repeats):
            t0 = time.perf_counter()
            orc.matmul(a, b)
            best = min(best, time.perf_counter() - t0)
        secs = best
    flops = 2.0 * rows * n * n
    return flops / secs / 1e12, {"kind": kind, "cores": cores, "seconds": secs,
                                 "sample": f"{rows} of {n} output rows of the {n}^3 product "
                                           f"(best of {repeats}), all host threads"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = args.size
    rows = 64 if n >= 8192 else 256
    tf, info = cpu_sample(n, rows, 1)  # warm-up, also sizes the job
    for _ in range(max(0, args.warmup - 1)):
        cpu_sample(n, rows, 1)
    vals = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, info = cpu_sample(n, rows, 1)
        vals.append(v)
        if time.perf_counter() - t0 > 150:
            break
    value = statistics.mean(vals)
    ms = 2.0 * rows * n * n / (value * 1e12) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(vals), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"fp32 GEMM {n}^3, N(0,1/K) inputs; CPU arm times a row slice per step",
                   "M": n, "N": n, "K": n},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
                         "sample": info["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def measure_tf32_peak(torch, dev, seconds: float = 1.5):
    """cuBLAS TF32 8192^3: best single launch (burst) and the rate of a back-to-back loop
    (sustained, what a kernel timed inside a long step should be held against)."""
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


def run_b200(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.load()  # raises if the CUDA library is missing: there is no fallback
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n = args.size
    gen = torch.Generator(device=dev).manual_seed(1)  # same bytes on every rank
    A = torch.randn((n, n), device=dev, generator=gen) / n ** 0.5
    B = torch.randn((n, n), device=dev, generator=gen) / n ** 0.5
    exchange = args.exchange if world > 1 else "none"
    try:
        op = pkg.shard.ColumnShardedMatmul(n, n, n, rank=rank, world=world, device=dev,
                                           mode=args.exchange if world > 1 else "nccl")
    except Exception as exc:  # symmetric memory unavailable: the NCCL gather still works
        if world > 1 and args.exchange == "fused":
            if rank == 0:
                print(f"[bench] fused exchange unavailable ({exc!r}); using the NCCL all-gather", file=sys.stderr)
            exchange = "nccl"
            op = pkg.shard.ColumnShardedMatmul(n, n, n, rank=rank, world=world, device=dev, mode="nccl")
        else:
            raise
    if precision != pkg.PRECISION_3XTF32:
        def block(A_, B_, dests, col0, cols, _op=op):
            pkg.gemm_colshard(A_, B_, dests, M=n, N=n, K=n, col0=col0, cols=cols, lda=n, ldb=n, ldc=n,
                              precision=precision)
        op._compute = block

    if world == 1:
        # one GPU holds every column: the plain entry point with its workspace, which lets the planner
        # split the tiles of a mostly empty last wave along K
        ws_bytes = pkg.workspace_bytes(1, n, n, n)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

        def whole(A_, B_, dests, col0, cols, _op=op):
            pkg.gemm(A_, B_, _op.C, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n, precision=precision,
                     workspace=ws if ws_bytes else None, workspace_bytes=ws_bytes)
        op._compute = whole

    def step():
        op(A, B)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    pkg.status()
    launches0 = pkg.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = pkg.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    pkg.status()
    ms = total_ms / args.steps
    flops = 2.0 * n ** 3
    value = flops / ms / 1e9

    # parity spot check of the timed result: sampled rows against fp64 on the device
    rows = torch.arange(3, n, max(1, n // 16), device=dev)
    ref = A[rows].double() @ B.double()
    err = float(((op.C[rows].double() - ref).abs() / ref.abs().clamp(min=1.0)).max().item())
    del ref

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, fp32 accumulate)"
            if kfac == 3 else "tf32", "data": "synthetic",
            "config": {"workload": f"fp32 GEMM {n}^3, A,B ~ N(0,1/K) seed 1, C N-column-sharded over "
                                   f"{world} GPU(s), every rank ends with all of C",
                       "M": n, "N": n, "K": n, "exchange": exchange, "precision": args.precision,
                       "l2": "operands (1 GiB each) far exceed L2; no flush needed"
                       if n >= 8192 else "L2 flushed between timed launches"},
            "gpu_launches": int(launches), "clocks": clocks,
            "check": {"scaled_max_error_vs_fp64_sampled_rows": err},
        }

    extras = (world == 1 and not args.no_extras)
    # ------------------------------------------------------------------ roofline (rank 0, N = 1)
    if rank == 0 and world == 1:
        if args.no_peak:
            burst = sustained = float("nan")
        else:
            time.sleep(2.0)  # let the power-capped clocks recover before the burst measurement
            burst, sustained = measure_tf32_peak(torch, dev)
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        bf16 = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
        achieved = kfac * value
        line["roofline"] = {
            "bound": "tensor", "achieved": achieved, "peak": sustained, "unit": "TFLOP/s",
            "frac": achieved / sustained,
            # dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of this workload
            # (profiles/gemm_tf32_kernel_pair_16384cubed_dram.md); algorithmic bytes are 3 * n^2 * 4
            "traffic": 30878857472 if (n == BIG and kfac == 3 and world == 1) else None,
            "algorithmic_bytes": int(3 * n * n * 4),
            "note": f"achieved = {kfac} x useful TFLOP/s: tensor-core TF32 math issued per product "
                    f"(2*M*N*K*{kfac}) / mean time of one product by CUDA events (at one GPU a product is the "
                    f"main launch plus the K-split launch of the last wave's tiles and their reduction; "
                    f"traffic is the ncu figure of the single-launch plan); peak = cuBLAS TF32 8192^3 "
                    f"sustained loop measured in this run (of measured); burst {burst:.1f}",
            "useful_tflops": value, "useful_frac": value / sustained, "k_factor": kfac,
            "peak_burst": burst,
            "bf16_measured_peaks": {k: bf16.get(k) for k in ("bf16_tflops", "bf16_tflops_sustained")},
        }
    if world > 1 and rank == 0:
        line["roofline"] = {"bound": "tensor", "achieved": kfac * value, "peak": None, "unit": "TFLOP/s",
                            "frac": None, "traffic": None,
                            "note": "whole-job tensor math over all ranks; see the N=1 line for the per-GPU peak"}

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

        time.sleep(2.0)  # same starting state as the burst peak it is compared with
        for _ in range(3):
            launch4()
        torch.cuda.synchronize()
        # (a) back to back: A, B and C together (201 MB) exceed the 126 MB L2
        iters = max(20, args.steps)
        e0.record()
        for _ in range(iters):
            launch4()
        e1.record()
        torch.cuda.synchronize()
        b2b_ms = e0.elapsed_time(e1) / iters
        # (b) one launch per timing with L2 evicted before each
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
        peak4 = line["roofline"]["peak_burst"]
        line["gemm_4096"] = {
            "workload": "fp32 GEMM 4096^3, N(0,1/K); back-to-back launches (A+B+C = 201 MB exceed L2)",
            "ms_per_launch": b2b_ms, "useful_tflops": tf, "tensor_math_tflops": kfac * tf,
            "frac_of_tf32_peak": kfac * tf / peak4, "peak": peak4,
            "peak_kind": "cuBLAS TF32 8192^3 burst (best single launch after 2 s idle) measured in this run; "
                         "this product is timed the same way: a 20-launch burst after 2 s idle",
            "l2_flushed": {"ms_mean": cold_ms, "ms_best": min(times),
                           "useful_tflops": 2.0 * m ** 3 / cold_ms / 1e9,
                           "note": "single launch after a 256 MB fill that evicts L2"},
        }
        del a4, b4, c4, flush

    # ------------------------------------------------------------------ end to end, host buffers
    if world == 1 and not args.no_extras:
        import numpy as np

        h_a = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
        h_b = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
        h_c = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
        h_a.copy_(A)
        h_b.copy_(B)
        del op
        torch.cuda.empty_cache()
        na, nb, nc = h_a.numpy(), h_b.numpy(), h_c.numpy()
        reps = max(2, min(args.steps, 4))
        pkg.matmul_host(na, nb, nc, batch=1, rows=n, inner=n, cols=n, a_batched=False, b_batched=False)
        t0 = time.perf_counter()
        for _ in range(reps):
            pkg.matmul_host(na, nb, nc, batch=1, rows=n, inner=n, cols=n, a_batched=False, b_batched=False)
        secs = (time.perf_counter() - t0) / reps
        line["e2e"] = {"value": flops / secs / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(2 * n * n * 4),
                       "d2h_bytes_per_step": int(n * n * 4), "ms_per_step": secs * 1e3,
                       "path": "b200_matmul_f32_host: pinned host A,B -> device, kernel, C -> pinned host, synchronised"}
        assert np.isfinite(nc[::997, ::991]).all()
    elif world > 1:
        # every rank uploads A and its B columns from pinned memory and downloads its C columns
        col0, cols = op.col0, op.cols
        h_a = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
        h_b = torch.empty((n, max(cols, 1)), dtype=torch.float32, pin_memory=True)
        h_c = torch.empty((n, max(cols, 1)), dtype=torch.float32, pin_memory=True)
        h_a.copy_(A)
        if cols:
            h_b.copy_(B[:, col0:col0 + cols])
        reps = max(2, min(args.steps, 4))

        def e2e_step():
            A.copy_(h_a, non_blocking=True)
            if cols:
                B[:, col0:col0 + cols].copy_(h_b, non_blocking=True)
            op(A, B)
            if cols:
                h_c.copy_(op.C[:, col0:col0 + cols], non_blocking=True)
            torch.cuda.synchronize()

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            e2e_step()
        barrier()
        secs = max_over_ranks((time.perf_counter() - t0) / reps * 1e3) / 1e3
        if rank == 0:
            line["e2e"] = {"value": flops / secs / 1e12, "unit": "TFLOP/s",
                           "h2d_bytes_per_step": int((n * n + n * cols) * 4), "d2h_bytes_per_step": int(n * cols * 4),
                           "ms_per_step": secs * 1e3,
                           "path": "per rank: pinned host A + B columns -> device, sharded kernel + exchange, "
                                   "own C columns -> pinned host; bytes are per rank"}
    elif rank == 0:
        line["e2e"] = None

    # ------------------------------------------------------------------ CPU baseline (rank 0, N = 1)
    if rank == 0 and world == 1 and not args.no_extras:
        tf, info = cpu_sample(n, 64, 1)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
                                "sample": info["sample"]}
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
            "kernels_per_call": 2 if ws_bytes else 1}
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
