#!/usr/bin/env python
"""Benchmark of the commitment hot path on B200: the PCS-commit microbench shape.

Workload (one "step"): `--cols` M31 trace columns of 2^`--log-size` values each are interpolated,
extended to the canonic domain of log size `--log-size + --log-blowup` (the low-degree extension) and
committed with the Blake2s-M31 Merkle tree (leaf layer over all columns, then every upper layer down to
the root). Inputs are seeded synthetic columns (SplitMix64, seed 0x5EED0001 + column index).

  python bench.py [--gpus N] [--steps K] [--warmup W]            the CUDA library through its C ABI
  python bench.py --impl reference ...                             the CPU restatement of the reference
                                                                   backend, on the host cores

One JSON line is printed by rank 0. `value` is device-resident throughput; `e2e` includes the host->device
copy of the trace from pinned memory and the device->host read of the root, every step.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

SEED0 = 0x5EED0001


def splitmix_column(seed, n):
    from util import m31_column

    return m31_column(seed, n)


def n_fft_passes(layers):
    return 1 + (max(0, layers - 12) + 9) // 10


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def cpu_leg(args, sample_cols):
    """Times the CPU oracle (a port of the reference's CpuBackend) on `sample_cols` columns of the workload."""
    import oracle

    log_n, log_out = args.log_size, args.log_size + args.log_blowup
    vals = np.stack([splitmix_column(SEED0 + c, 1 << log_n) for c in range(sample_cols)])
    oracle.twiddles(log_out - 1)  # the tower is built once, outside the timed region (as precompute_twiddles is)
    t0 = time.perf_counter()
    coeffs = oracle.interpolate_cols(vals, log_n)
    ev = oracle.evaluate_cols(coeffs, log_n, log_out)
    layer = oracle.commit_on_layer(log_out, None, list(ev), m31=True)
    for lg in range(log_out - 1, -1, -1):
        layer = oracle.commit_on_layer(lg, layer, [], m31=True)
    dt = time.perf_counter() - t0
    cells = sample_cols * (1 << log_n)
    return cells / dt, dt, oracle.num_threads(), layer


def run_reference(args, rank):
    if rank != 0:
        return
    sample_cols = min(args.cols, args.ref_cols)
    for _ in range(args.warmup if args.warmup < 1 else 1):
        cpu_leg(args, sample_cols)
    vals, times = [], []
    for _ in range(args.steps):
        v, dt, threads, _ = cpu_leg(args, sample_cols)
        vals.append(v)
        times.append(dt)
    value = float(np.mean(vals))
    sample = (f"{sample_cols} of {args.cols} columns at full height 2^{args.log_size}: interpolate + LDE to 2^"
              f"{args.log_size + args.log_blowup} + Blake2s-M31 Merkle tree, all host threads (OpenMP)")
    line = {
        "impl": "reference", "metric": "committed_m31_cells_per_s", "value": value, "unit": "cells/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times)) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u32 (M31)", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": "cells/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "cells/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is Rust and cannot be built with this image's toolchains; this arm times the C++ restatement "
                "of its CpuBackend (oracle/), not the reference's SIMD backend",
    }
    print(json.dumps(line))


def workload_config(args):
    return {"workload": f"pcs_commit_{args.cols}cols_log{args.log_size}_blowup{1 << args.log_blowup}",
            "columns": args.cols, "log_size": args.log_size, "log_blowup": args.log_blowup,
            "hasher": "blake2s_m31", "parallelism": f"replicas x{args.gpus}" if args.gpus > 1 else "single",
            "l2": "inputs (>= 1 GiB per step) are larger than L2"}


def run_ours(args, rank, world, local_rank):
    import zk_inference_prover_b200 as z

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    log_n, log_out, ncols = args.log_size, args.log_size + args.log_blowup, args.cols
    n, N = 1 << log_n, 1 << log_out
    ctx = z.Context(device=local_rank, max_log_size=max(log_out, 3))

    # host trace in pinned memory (the e2e leg copies it every step)
    h_trace, h_addr = ctx.alloc_pinned(ncols * n)
    for c in range(ncols):
        h_trace[c * n:(c + 1) * n] = splitmix_column(SEED0 + c, n)
    h_root, h_root_addr = ctx.alloc_pinned(8)

    d_src = ctx.alloc(ncols * n)    # resident copy of the trace
    d_work = ctx.alloc(ncols * n)   # interpolated in place
    d_eval = ctx.alloc(ncols * N)
    layers = [ctx.alloc(8 << lg) for lg in range(log_out + 1)]  # layers[lg]: 2^lg hashes
    ctx.h2d_async(d_src.ptr, h_addr, ncols * n * 4)
    ctx.sync()
    work_ptrs = [d_work.view(c * n) for c in range(ncols)]
    eval_ptrs = [d_eval.view(c * N) for c in range(ncols)]

    EV_START, EV_IN, EV_IFFT, EV_LDE, EV_LEAF, EV_TREE = 0, 1, 2, 3, 4, 5

    def step(e2e):
        ctx.event_record(EV_START)
        if e2e:
            ctx.h2d_async(d_work.ptr, h_addr, ncols * n * 4)
        else:
            ctx.d2d(d_work.ptr, d_src.ptr, ncols * n * 4)
        ctx.event_record(EV_IN)
        ctx.ifft_cols(work_ptrs, log_n)
        ctx.event_record(EV_IFFT)
        ctx.lde_cols(work_ptrs, log_n, eval_ptrs, log_out)
        ctx.event_record(EV_LDE)
        ctx.merkle_layer(log_out, 0, eval_ptrs, layers[log_out].ptr, m31_out=True)
        ctx.event_record(EV_LEAF)
        for lg in range(log_out - 1, -1, -1):
            ctx.merkle_layer(lg, layers[lg + 1].ptr, [], layers[lg].ptr, m31_out=True)
        ctx.d2h_async(h_root_addr, layers[0].ptr, 32)
        ctx.event_record(EV_TREE)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    phases = {"input_copy": 0.0, "ifft": 0.0, "lde": 0.0, "merkle_leaves": 0.0, "merkle_upper": 0.0}

    def timed(e2e, collect):
        for _ in range(args.warmup):
            step(e2e)
        barrier()
        t0 = time.perf_counter()
        total_ms = 0.0
        for _ in range(args.steps):
            step(e2e)
            # events of this step are read before the next step re-records them
            total_ms += ctx.event_elapsed_ms(EV_START, EV_TREE)
            if collect:
                for name, a, b in [("input_copy", EV_START, EV_IN), ("ifft", EV_IN, EV_IFFT), ("lde", EV_IFFT, EV_LDE),
                                   ("merkle_leaves", EV_LDE, EV_LEAF), ("merkle_upper", EV_LEAF, EV_TREE)]:
                    phases[name] += ctx.event_elapsed_ms(a, b)
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        return total_ms, wall_ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    dev_ms, dev_wall = timed(False, True)
    root_resident = h_root.copy()
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms, e2e_wall = timed(True, False)
    root_e2e = h_root.copy()
    assert (root_resident == root_e2e).all(), "resident and end-to-end legs disagree on the Merkle root"

    if dist is not None:
        import torch

        t = torch.tensor([dev_ms, e2e_ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])

    cells = ncols * n * world
    ms_per_step = dev_ms / args.steps
    value = cells / (ms_per_step * 1e-3)
    e2e_value = cells / (e2e_ms / args.steps * 1e-3)

    if rank == 0:
        per = {k: v / args.steps for k, v in phases.items()}
        # dominant kernel: the leaf-layer Blake2s kernel (one launch per step). Algorithmic bytes:
        # 4 * ncols * rows read + 32 * rows written.
        peak, peak_kind = measured_hbm_peak()
        leaf_bytes = 4.0 * ncols * N + 32.0 * N
        lde_bytes = (4.0 * n + 4.0 * N) * ncols
        ifft_bytes = 8.0 * n * ncols
        dom = max([("merkle_leaves", leaf_bytes), ("lde", lde_bytes), ("ifft", ifft_bytes)], key=lambda kv: per[kv[0]])
        achieved = dom[1] / (per[dom[0]] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": {"merkle_leaves": "merkle_layer_kernel", "lde": "fft_pass_kernel<false>",
                                                 "ifft": "fft_pass_kernel<true>"}[dom[0]],
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                    "peak_kind": peak_kind,
                    "per_phase_ms": per,
                    "per_phase_gbs": {"ifft": ifft_bytes / (per["ifft"] * 1e-3) / 1e9, "lde": lde_bytes / (per["lde"] * 1e-3) / 1e9,
                                      "merkle_leaves": leaf_bytes / (per["merkle_leaves"] * 1e-3) / 1e9}}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample_cols = min(ncols, args.ref_cols)
            v, dt, threads, _ = cpu_leg(args, sample_cols)
            cpu = {"value": v, "unit": "cells/s", "cores": threads, "kind": "port",
                   "sample": f"{sample_cols} of {ncols} columns at full height 2^{log_n} ({dt:.1f} s of CPU work): interpolate + LDE + Merkle tree"}
        launches = n_fft_passes(log_n) * 2 + (log_out + 1)
        line = {
            "metric": "committed_m31_cells_per_s", "value": value, "unit": "cells/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32 (M31)", "data": "synthetic", "config": workload_config(args),
            "e2e": {"value": e2e_value, "unit": "cells/s", "h2d_bytes_per_step": ncols * n * 4, "d2h_bytes_per_step": 32,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches * args.steps,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
            "root": "".join(f"{int(w):08x}" for w in root_resident),
        }
        print(json.dumps(line))
    ctx.free_pinned(h_addr)
    ctx.free_pinned(h_root_addr)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cols", type=int, default=256)
    ap.add_argument("--log-size", type=int, default=20)
    ap.add_argument("--log-blowup", type=int, default=2)
    ap.add_argument("--ref-cols", type=int, default=32, help="columns in the bounded CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
