#!/usr/bin/env python
"""Benchmark of the commitment hot path on B200: the PCS-commit microbench shape.

Workload (one "step"): `--cols` M31 trace columns of 2^`--log-size` values each are interpolated,
extended to the canonic domain of log size `--log-size + --log-blowup` (the low-degree extension),
committed with the Blake2s-M31 Merkle tree, opened at one channel-drawn point per column, and the
opening is proved: quotients, FRI commit to the last layer, proof of work, query decommitment
(PcsConfig: pow_bits 10, FriConfig(0, log_blowup, 3, 1), the library default with the blow-up
of the workload). Inputs are seeded synthetic columns (SplitMix64, seed 0x5EED0001 + column index).

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

SEED0 = 0x5EED0001


def splitmix_column(seed, n):
    from zk_inference_prover_b200.synth import m31_column

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


import contextlib


@contextlib.contextmanager
def stdout_to_stderr():
    """Routes file descriptor 1 to stderr for the duration (native libraries write to the fd directly)."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        yield
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def cpu_leg(args, sample_cols):
    """Times the CPU restatement of the reference's SIMD backend (oracle/simd.hpp: 16-lane packed M31 arithmetic for the FFTs,
    Blake2s over 16 rows, out-of-domain evaluation and quotient numerators; OpenMP over columns / row blocks; the rest of
    the protocol on the scalar restatement of CpuBackend) on `sample_cols` columns of the workload: the same commit + prove
    flow as the GPU step. Returns (cells/s, seconds, threads, lanes, proof words)."""
    import oracle

    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1 to its workers)
    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    lanes = oracle.set_simd(True)
    log_n, log_out = args.log_size, args.log_size + args.log_blowup
    cols = [splitmix_column(SEED0 + c, 1 << log_n) for c in range(sample_cols)]
    oracle.twiddles(log_out - 1)  # the tower is built once, outside the timed region (as precompute_twiddles is)
    t0 = time.perf_counter()
    words = oracle.pcs_prove([cols], pow_bits=args.pow_bits, log_blowup=args.log_blowup, log_last_layer=0,
                             n_queries=args.n_queries, cap=1 << 26)
    dt = time.perf_counter() - t0
    oracle.set_simd(False)
    cells = sample_cols * (1 << log_n)
    return cells / dt, dt, oracle.num_threads(), lanes, words


CPU_KIND_NOTE = ("the reference is Rust and cannot be built with this image's toolchains; this arm times the C++ restatement of its "
                 "SIMD backend's hot operators (packed 16-lane M31 FFTs, Blake2s over 16 rows, sampling, quotient numerators) inside "
                 "the restated protocol code (oracle/), not the reference's own binary")


def run_reference(args, rank):
    if rank != 0:
        return
    sample_cols = args.cols if args.ref_cols <= 0 else min(args.cols, args.ref_cols)
    # every column of the workload; when a step is slow on this host, fewer timed steps (never fewer columns), so that the
    # run ends within a few minutes
    budget_s = 150.0
    v, dt, threads, lanes, words = cpu_leg(args, sample_cols)  # warm-up (page faults, twiddles), also sizes the run
    steps = max(1, min(args.steps, int(budget_s / max(dt, 1e-3))))
    vals, times = [], []
    for _ in range(steps):
        v, dt, threads, lanes, _ = cpu_leg(args, sample_cols)
        vals.append(v)
        times.append(dt)
    value = float(np.mean(vals))
    sample = (f"{sample_cols} of {args.cols} columns at full height 2^{args.log_size}, {steps} timed step(s) of the {args.steps} asked for: "
              f"commit (interpolate, LDE, Merkle) + prove (sample, quotients, FRI, grind, decommit)")
    line = {
        "impl": "reference", "metric": "committed_m31_cells_per_s", "value": value, "unit": "cells/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times)) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u32 (M31)", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": "cells/s", "cores": threads, "kind": "port", "lanes": lanes, "sample": sample,
                         "timed_steps": steps},
        "e2e": {"value": value, "unit": "cells/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "accepts": verifier_accepts(words, sample_cols, args.log_size, args),
        "note": CPU_KIND_NOTE,
    }
    print(json.dumps(line))


def reference_gpu_leg(args):
    """Same-box GPU baseline: the reference's own CUDA kernels (compiled unmodified for sm_100a by
    oracle/Makefile.ref_cuda) on the commitment part of the workload: interpolate_columns, evaluate_polynomials
    (zero-extended copy + transform, as backend/cuda/poly.rs does) and the Merkle tree layer by layer. Timed with
    the host clock around device synchronisations (the library works on the default stream)."""
    from oracle import ref_cuda

    if not ref_cuda.available():
        return None
    ref = ref_cuda.RefCuda()
    log_n, log_out, ncols = args.log_size, args.log_size + args.log_blowup, args.cols
    n = 1 << log_n
    tree = ref.twiddle_tree(log_out - 1)
    src = [ref.upload(splitmix_column(SEED0 + c, n)) for c in range(ncols)]
    work = [ref.lib.cuda_malloc_uint32_t(n) for _ in range(ncols)]
    t = {"interpolate": [], "extend": [], "merkle": []}
    for it in range(3):
        for a, b in zip(src, work):
            ref.lib.copy_uint32_t_vec_from_device_to_device(a, b, n)
        ref.sync()
        t0 = time.perf_counter()
        ref.interpolate_columns(work, log_n, tree)
        ref.sync()
        t1 = time.perf_counter()
        ext = ref.extend_columns(work, log_n, log_out)
        ref.evaluate_extended(ext, log_out, tree)
        ref.sync()
        t2 = time.perf_counter()
        layers = [ref.commit_on_layer(log_out, None, ext)]
        for lg in range(log_out - 1, -1, -1):
            layers.append(ref.commit_on_layer(lg, layers[-1], []))
        ref.sync()
        t3 = time.perf_counter()
        for p in ext + layers:
            ref.free(p)
        if it:  # the first pass warms up
            t["interpolate"].append(t1 - t0)
            t["extend"].append(t2 - t1)
            t["merkle"].append(t3 - t2)
    for p in src + work + [tree["tw"], tree["itw"]]:
        ref.free(p)
    ms = {k: 1e3 * float(np.mean(v)) for k, v in t.items()}
    return {"kind": "the reference's CUDA kernels for this path, compiled unmodified for sm_100a, same GPU", "ms": ms,
            "commit_ms": sum(ms.values()), "cells_per_s_commit_only": ncols * n / (sum(ms.values()) * 1e-3)}


def golden_check(name, words):
    """Compares a proof with the committed digest of the CPU oracle's proof of the same seeded workload."""
    import hashlib

    path = os.path.join(ROOT, "tests", "golden", "proof_digests.json")
    try:
        want = json.load(open(path)).get(name)
    except OSError:
        want = None
    if want is None:
        return {"golden": None, "note": "no committed digest for this workload"}
    ok = int(len(words)) == want["words"] and hashlib.sha256(words.tobytes()).hexdigest() == want["sha256"]
    if not ok:
        raise SystemExit(f"proof differs from the committed oracle digest {name}")
    return {"golden": name, "match": True}


def verifier_accepts(words, ncols, log_n, args):
    """The proof of the timed run, checked by the CPU restatement of the reference's verifier (oracle/verify.hpp:
    CommitmentSchemeVerifier::verify_values with FriVerifier and MerkleVerifier). A checker, outside every timed region."""
    try:
        import oracle

        rc = oracle.pcs_verify(words, [[log_n] * ncols], pow_bits=args.pow_bits, log_blowup=args.log_blowup, log_last_layer=0,
                               n_queries=args.n_queries)
    except Exception as e:
        return {"unavailable": repr(e)}
    if rc[0] != 0:
        raise SystemExit(f"the reference's verifier rejects the proof: {rc}")
    return True


def workload_config(args):
    return {"workload": f"pcs_prove_{args.cols}cols_log{args.log_size}_blowup{1 << args.log_blowup}",
            "columns": args.cols, "log_size": args.log_size, "log_blowup": args.log_blowup, "pow_bits": args.pow_bits,
            "n_queries": args.n_queries, "log_last_layer_degree_bound": 0, "hasher": "blake2s_m31",
            "step": "interpolate + LDE + Merkle commit + out-of-domain sample + quotients + FRI commit + grind + decommit",
            "parallelism": f"replicas x{args.gpus}" if args.gpus > 1 else "single",
            "l2": "inputs (>= 1 GiB per step) are larger than L2"}


# Algorithmic bytes of the operators (per step), for the roofline figures.
def algorithmic_bytes(ncols, n, N):
    return {
        "interpolate": 8.0 * n * ncols,                 # read n + write n per column
        "extend": (4.0 * n + 4.0 * N) * ncols,          # read n coefficients, write N evaluations
        "merkle_leaves": 4.0 * ncols * N + 32.0 * N,    # read every evaluation, write one hash per row
        "quot_numerators": 4.0 * ncols * N + 16.0 * N,  # one sample batch
    }


def run_ours(args, rank, world, local_rank):
    import zk_inference_prover_b200 as z

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        with stdout_to_stderr():  # NCCL prints a version banner on stdout; the contract is ONE JSON line
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()

    log_n, log_out, ncols = args.log_size, args.log_size + args.log_blowup, args.cols
    n, N = 1 << log_n, 1 << log_out
    ctx = z.Context(device=local_rank, max_log_size=max(log_out, 3))

    # host trace in pinned memory (the e2e leg copies it every step)
    h_trace, h_addr = ctx.alloc_pinned(ncols * n)
    for c in range(ncols):
        h_trace[c * n:(c + 1) * n] = splitmix_column(SEED0 + c, n)
    host_cols = [h_trace[c * n:(c + 1) * n] for c in range(ncols)]

    d_src = ctx.alloc(ncols * n)    # resident copy of the trace
    d_work = ctx.alloc(ncols * n)   # consumed by each proof
    ctx.h2d_async(d_src.ptr, h_addr, ncols * n * 4)
    ctx.sync()
    work_ptrs = [d_work.view(c * n) for c in range(ncols)]
    kw = dict(pow_bits=args.pow_bits, log_blowup=args.log_blowup, log_last_layer=0, n_queries=args.n_queries, cap=1 << 26)

    EV_A, EV_B = 0, 1
    phases = {}

    def step(e2e, collect):
        ctx.event_record(EV_A)
        if e2e:
            words = ctx.pcs_prove_host([host_cols], **kw)
        else:
            ctx.d2d(d_work.ptr, d_src.ptr, ncols * n * 4)   # the trace "arrives" in device memory
            if collect:
                words, ph = ctx.pcs_prove_device([work_ptrs], [log_n] * ncols, phases=True, **kw)
                for k, v in ph.items():
                    phases[k] = phases.get(k, 0.0) + v
            else:
                words = ctx.pcs_prove_device([work_ptrs], [log_n] * ncols, **kw)
        ctx.event_record(EV_B)
        return words, ctx.event_elapsed_ms(EV_A, EV_B)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    def timed(e2e, collect):
        words = None
        for _ in range(args.warmup):
            words, _ = step(e2e, False)
        barrier()
        total_ms = 0.0
        for _ in range(args.steps):
            words, ms = step(e2e, collect)
            total_ms += ms
        barrier()
        return total_ms, words

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    dev_ms, words_dev = timed(False, True)
    clocks = sampler.stop() if rank == 0 else None
    # per-kernel timeline of one more (untimed) step
    ctx.d2d(d_work.ptr, d_src.ptr, ncols * n * 4)
    ctx.profile_begin()
    ctx.pcs_prove_device([work_ptrs], [log_n] * ncols, **kw)
    kernels = ctx.profile_end()
    # operators of the workload that the proof does not time on their own: bit reversal of extended columns,
    # the first circle fold and the first line fold (algorithmic bytes: 8n, 34n, 26n for n source elements)
    standalone, copy_ceiling = {}, {}
    if rank == 0:
        nb = min(ncols, 32)
        cols_b = [ctx.alloc(N) for _ in range(nb)]
        sec = [ctx.alloc(N) for _ in range(4)]
        half = [ctx.alloc(N // 2).zero() for _ in range(4)]
        quarter = [ctx.alloc(N // 4) for _ in range(4)]
        alpha = np.array([5, 6, 7, 8], np.uint32)
        for rep in range(2):
            ctx.event_record(2)
            for c in cols_b:
                ctx.bit_reverse_m31(c.ptr, log_out)
            ctx.event_record(3)
            ctx.fold_circle_into_line([h_.ptr for h_ in half], [s_.ptr for s_ in sec], log_out, alpha)
            ctx.event_record(4)
            ctx.fold_line([q.ptr for q in quarter], [h_.ptr for h_ in half], log_out - 1, alpha)
            ctx.event_record(5)
        standalone = {"bit_reverse": 8.0 * N * nb / (ctx.event_elapsed_ms(2, 3) * 1e-3) / 1e9,
                      "fold_circle_into_line": 34.0 * N / (ctx.event_elapsed_ms(3, 4) * 1e-3) / 1e9,
                      "fold_line": 26.0 * (N // 2) / (ctx.event_elapsed_ms(4, 5) * 1e-3) / 1e9}
        # The same numbers of bytes moved by the driver's own device-to-device copy, one launch each as above: at these sizes
        # (a launch of 14-40 us) a launch's fixed cost shows, and this is what a plain copy makes of it.
        copy_ceiling = {}
        for name, nbytes, launches in (("bit_reverse", 8 * N, nb), ("fold_circle_into_line", 34 * N, 1), ("fold_line", 13 * N, 1)):
            cw = nbytes // 8 // 4 * 4  # a copy of cw words moves 8 cw bytes
            src_c, dst_c = ctx.alloc(cw), ctx.alloc(cw)
            for rep in range(2):
                ctx.event_record(2)
                for _ in range(launches):
                    ctx.d2d(dst_c.ptr, src_c.ptr, cw * 4)
                ctx.event_record(3)
            ctx.sync()
            copy_ceiling[name] = 8.0 * cw * launches / (ctx.event_elapsed_ms(2, 3) * 1e-3) / 1e9
            del src_c, dst_c
        del cols_b, sec, half, quarter
    e2e_ms, words_e2e = timed(True, False)
    assert len(words_dev) == len(words_e2e) and (words_dev == words_e2e).all(), "resident and end-to-end legs disagree"
    commit_ms = sum(phases.get(k, 0.0) for k in ("interpolate", "extend", "merkle")) / args.steps
    extras = {} if args.no_extras else extra_legs(args, z, ctx, dist, rank, world, local_rank, words_dev, dev_ms / args.steps, h_addr, d_work, commit_ms)

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
        peak, peak_kind = measured_hbm_peak()
        ab = algorithmic_bytes(ncols, n, N)
        # dominant operator: the LDE (two launches: the strided radix-32 pass, then the contiguous one)
        fwd = [(k, v) for k, v in kernels.items() if "forward" in k]
        lde_ms = sum(v[0] for _, v in fwd)
        achieved = ab["extend"] / (lde_ms * 1e-3) / 1e9 if lde_ms else None
        kern = {k: {"ms": round(v[0], 4), "launches": v[1]} for k, v in sorted(kernels.items(), key=lambda kv: -kv[1][0])}
        # DRAM traffic of the two LDE launches: ncu's dram__bytes_read + dram__bytes_write on 32 columns of this shape
        # (137 + 482 MB for the wide pass, 569 + 479 MB for the twelve-layer contiguous pass), scaled by the column
        # count; a figure from a past capture, not measured in this run.
        traffic = 1666.6e6 / 32 * ncols if (log_n, args.log_blowup) == (20, 2) else None
        # The passes are bound by instruction issue: report them against the measured rate of the butterfly
        # arithmetic alone (the library's register-only butterfly kernel, timed in this run at this clock).
        butterflies = ncols * (N // 2) * log_n  # the layers above the coefficient count only copy
        ceiling = ctx.fft_arith_ceiling()
        issue = {"bound": "instruction issue", "achieved": butterflies / (lde_ms * 1e-3) if lde_ms else None, "peak": ceiling,
                 "unit": "butterflies/s", "frac": butterflies / (lde_ms * 1e-3) / ceiling if lde_ms else None,
                 "peak_kind": "measured in this run: the same radix-32 butterfly stages on registers only, no global traffic, 2 CTAs x 256 threads per SM",
                 "note": "about 10.5 machine instructions per butterfly at one instruction per cycle per scheduler saturate the "
                         "ALU and FMA-heavy pipes together"}
        roofline = {"bound": "hbm", "kernel": "+".join(k for k, _ in fwd) + " (the launches of one LDE)",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                    "traffic": traffic, "traffic_source": "ncu capture on 32 of the columns, scaled by the column count (an estimate for this run)",
                    "peak_kind": peak_kind, "issue": issue,
                    "note": "achieved = algorithmic bytes (read 2^log_size, write 2^(log_size+log_blowup) words per column) / the "
                            "CUDA-event time of the two launches; the kernels are instruction-issue bound (see `issue`), DRAM at "
                            "25-40% of peak; the 2.5x traffic is the array between the two passes",
                    "per_phase_ms": per, "kernels_one_step": kern,
                    "per_operator_gbs": {
                        "interpolate": ab["interpolate"] / (sum(v[0] for k, v in kernels.items() if "inverse" in k) * 1e-3) / 1e9,
                        "extend": achieved,
                        "merkle_leaves": ab["merkle_leaves"] / (kernels.get("merkle_layer_kernel(leaves)", (1e9, 1))[0] * 1e-3) / 1e9,
                        "quot_numerators": ab["quot_numerators"] / (kernels.get("quot_numerators_kernel", (1e9, 1))[0] * 1e-3) / 1e9,
                        **standalone}}
        roofline["per_operator_frac_of_hbm_peak"] = {k: v / peak for k, v in roofline["per_operator_gbs"].items()}
        roofline["same_bytes_by_device_copy_gbs"] = copy_ceiling  # one cudaMemcpyAsync D2D per launch, same byte counts
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample_cols = ncols if args.ref_cols <= 0 else min(ncols, args.ref_cols)
            v, dt, threads, lanes, cpu_words = cpu_leg(args, sample_cols)
            cpu = {"value": v, "unit": "cells/s", "cores": threads, "kind": "port", "lanes": lanes,
                   "sample": f"{sample_cols} of {ncols} columns at full height 2^{log_n}, one step ({dt:.1f} s of CPU work): the same commit + prove flow",
                   "same_proof_as_gpu": bool(sample_cols == ncols and len(cpu_words) == len(words_dev) and (cpu_words == words_dev).all()),
                   "note": CPU_KIND_NOTE}
        launches = sum(v[1] for v in kernels.values())
        gpu_ref = None
        if world == 1 and not args.no_gpu_baseline:
            try:
                gpu_ref = reference_gpu_leg(args)
                if gpu_ref:
                    gpu_ref["ours_commit_ms"] = per["interpolate"] + per["extend"] + per["merkle"]
            except Exception as e:  # the baseline must never cost the bench line
                gpu_ref = {"unavailable": repr(e)}
        import hashlib

        line = {
            "metric": "committed_m31_cells_per_s", "value": value, "unit": "cells/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32 (M31)", "data": "synthetic", "config": workload_config(args),
            "e2e": {"value": e2e_value, "unit": "cells/s", "h2d_bytes_per_step": ncols * n * 4, "d2h_bytes_per_step": int(len(words_dev)) * 4,
                    "ms_per_step": e2e_ms / args.steps, "host_memory": "pinned (zkb_host_alloc_pinned)"},
            "gpu_launches": launches * args.steps,
            "roofline": roofline, "cpu_baseline": cpu, "gpu_baseline": gpu_ref, "clocks": clocks,
            "proof_words": int(len(words_dev)), "proof_sha256": hashlib.sha256(words_dev.tobytes()).hexdigest(),
            **extras,
            "accepts": verifier_accepts(words_dev, ncols, log_n, args),
            "parity": golden_check(f"pcs_{ncols}x2e{log_n}_blowup{1 << args.log_blowup}" +
                                   ("" if (args.pow_bits, args.n_queries) == (10, 3) else f"_pow{args.pow_bits}_q{args.n_queries}"), words_dev),
        }
        print(json.dumps(line))
    ctx.free_pinned(h_addr)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


def extra_legs(args, z, ctx, dist, rank, world, local_rank, words_single, single_ms, h_addr, d_work, single_commit_ms=0.0):
    """Legs beside the headline, on the same GPUs in the same run, so that the driver's one line per N also carries: what the
    host can deliver to the ranks at once (reads the end-to-end scaling against), ONE proof sharded over all ranks (strong
    scaling of the proof itself; its words must equal the single-GPU proof), and the reference's first headline metric, the proof
    time of a composed decode segment (N = 1) or of a whole decode step dealt over the ranks (N > 1), as operator-trace
    replays. Every rank runs every leg; rank 0 keeps the results."""
    import torch

    out = {}
    dev = torch.device("cuda", local_rank)
    log_n, ncols = args.log_size, args.cols
    n = 1 << log_n

    def allmax(v):
        if dist is None:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    # ---- pinned host -> device, every rank at once
    nbytes = ncols * n * 4
    for _ in range(2):
        ctx.h2d_async(d_work.ptr, h_addr, nbytes)
    barrier()
    ctx.event_record(0)
    for _ in range(3):
        ctx.h2d_async(d_work.ptr, h_addr, nbytes)
    ctx.event_record(1)
    ms = allmax(ctx.event_elapsed_ms(0, 1) / 3)
    out["h2d_ceiling"] = {"gbs_per_rank": nbytes / (ms * 1e-3) / 1e9, "gbs_all_ranks": world * nbytes / (ms * 1e-3) / 1e9,
                          "bytes_per_copy": nbytes, "note": "one pinned-to-device copy of the trace per rank, all ranks at once, slowest rank"}

    # ---- one proof over all ranks
    if dist is not None and ncols % world == 0 and (world & (world - 1)) == 0:
        from zk_inference_prover_b200.sharded import ContextMem, Exchange, sharded_pcs_prove

        ncl = ncols // world
        mine = ctx.alloc(ncl * n)
        keep = ctx.alloc(ncl * n)
        for j in range(ncl):
            ctx.h2d_async(keep.view(j * n), h_addr + 4 * (rank * ncl + j) * n, n * 4)
        x = Exchange(ContextMem(ctx), dev)
        times, words, stages = [], None, {}
        for it in range(2 + 3):
            ctx.d2d(mine.ptr, keep.ptr, ncl * n * 4)
            barrier()
            t0 = time.perf_counter()
            sess = ctx.shard_pcs(rank, world, ncols, log_n, pow_bits=args.pow_bits, log_blowup=args.log_blowup, log_last_layer=0,
                                 n_queries=args.n_queries)
            words = sharded_pcs_prove(sess, x, [mine.view(j * n) for j in range(ncl)], stages if it >= 2 else None)
            ctx.sync()
            dt = (time.perf_counter() - t0) * 1e3
            sess.close()
            if it >= 2:
                times.append(dt)
        direct = x._peer is not None
        x.peer_close()
        ms = allmax(sum(times) / len(times))
        same = bool(len(words) == len(words_single) and (words == words_single).all())
        commit_ms = allmax((stages.get("interpolate_extend_exchange", 0.0) + stages.get("merkle_subtree_roots", 0.0)) / 3)
        # the commitment part on its own (columns -> exchange -> subtrees -> root), against the same phases of the one-GPU proof
        out["sharded_commit"] = {"ms": commit_ms, "single_gpu_ms": single_commit_ms, "strong_efficiency": single_commit_ms / commit_ms / world,
                                 "root_equals_single_gpu": same, "exchange": "direct copies between the GPUs (copy engines)" if direct else "all-to-all collective",
                                 "timer": "CUDA events on each rank's stream, slowest rank; the proof words (root included) are compared below"}
        out["sharded_proof"] = {"ms": ms, "cells_per_s": ncols * n / (ms * 1e-3), "single_gpu_ms": single_ms,
                                "strong_efficiency": single_ms / ms / world, "equals_single_gpu_proof": same,
                                "device_ms_per_stage_rank0": {k: v / 3 for k, v in stages.items()},
                                "commit_ms_rank0": (stages.get("interpolate_extend_exchange", 0.0) + stages.get("merkle_subtree_roots", 0.0)) / 3,
                                "timer": "host clock between barriers, slowest rank",
                                "what": "columns sharded for interpolate + LDE, one exchange to row shards, Merkle subtrees, sampling and "
                                        "quotients on the shards, FRI on the gathered quotient column, decommitment merged from the ranks"}
        if not same:
            raise SystemExit("the sharded proof differs from the single-GPU proof")
        del mine, keep

    # ---- the decode segment / decode step replays
    try:
        rctx = z.Context(device=local_rank, max_log_size=24)
        names = ["layer_8b_s32_c2048"] if world == 1 else (["layer_8b_s32_c2048"] * 32 + ["head_8b_s32_c2048"])[rank::world]
        shapes = {nm: SegmentReplay(z, rctx, nm, 0x5EED0006 + rank) for nm in sorted(set(names))}
        # the first steps grow the context's pools and the page-locked staging areas: two of them before the clock starts
        for nm in names[:1] * 2:
            shapes[nm].step()
        rctx.sync()
        if dist is not None:
            dist.barrier()
        reps = 3 if world == 1 else 1
        rctx.event_record(0)
        for _ in range(reps):
            for nm in names:
                shapes[nm].step()
        rctx.event_record(1)
        ms = allmax(rctx.event_elapsed_ms(0, 1)) / reps
        if world == 1:
            sr = shapes[names[0]]
            out["segment_replay"] = {"segment": names[0], "ms_per_segment": ms, "cells": sr.cells, "cells_per_s": sr.cells / (ms * 1e-3),
                                     "what": "the reference's first headline metric (proof ms per decode segment) as an operator-trace replay: the trees and GKR batches of one "
                                             "layer segment of the config-4 model on random data (timing only; the shape comes from the "
                                             "reference's cell-exact cost model)"}
        else:
            cells = 32 * 226711536 + 191812784
            out["decode_step_replay"] = {"ms": ms, "segments": 33, "segments_on_rank_0": len((["l"] * 33)[0::world]), "cells": cells,
                                         "cells_per_s": cells / (ms * 1e-3), "streams_per_gpu": 1,
                                         "what": "32 layer segments + the output head dealt round-robin to the ranks, no collective; slowest rank"}
        shapes.clear()
        rctx.close()
    except Exception as e:  # a replay must never cost the headline line
        out["segment_replay" if world == 1 else "decode_step_replay"] = {"unavailable": repr(e)}
    return out


def run_sharded_commit(args, rank, world, local_rank):
    """--mode sharded-commit: ONE commitment split over the ranks (columns -> all-to-all -> row subtrees).
    Strong scaling: the workload is fixed, every rank does 1/world of the LDE and of the leaf hashing."""
    import torch
    import torch.distributed as dist

    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200.sharded import ContextOps, ShardedCommitment

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 or not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        with stdout_to_stderr():
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
            dist.barrier()
    log_n, log_out, ncols = args.log_size, args.log_size + args.log_blowup, args.cols
    n = 1 << log_n
    ctx = z.Context(device=local_rank, max_log_size=log_out)
    sc = ShardedCommitment(ContextOps(ctx), dev)
    c0, c1 = sc.local_columns(ncols)
    src = torch.from_numpy(np.stack([splitmix_column(SEED0 + c, n) for c in range(c0, c1)]).view(np.int32).copy()).to(dev)
    times = []
    root = None
    for it in range(args.warmup + args.steps):
        trace = src.clone()
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        root, local, _ = sc.commit(trace, log_n, args.log_blowup)
        e1.record()
        torch.cuda.synchronize(dev)
        if it >= args.warmup:
            times.append(e0.elapsed_time(e1))
        del local, trace
    t = torch.tensor([sum(times)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t[0]) / args.steps
        cells = ncols * n
        print(json.dumps({
            "metric": "committed_m31_cells_per_s", "value": cells / (ms * 1e-3), "unit": "cells/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32 (M31)", "data": "synthetic",
            "config": {"workload": f"sharded_commit_{ncols}cols_log{log_n}_blowup{1 << args.log_blowup}", "columns": ncols,
                       "log_size": log_n, "log_blowup": args.log_blowup, "step": "interpolate + LDE (column-sharded) + all-to-all + Merkle tree (row-sharded)",
                       "parallelism": f"columns/rows x{world}"},
            "root": "".join(f"{int(w) & 0xffffffff:08x}" for w in root.cpu().tolist())}))
    ctx.close()
    dist.destroy_process_group()


def run_gkr(args, rank):
    """--mode gkr: the GKR logup microbench: one LogUpMultiplicities instance of 2^gkr_log fractions,
    M31 numerators, non-zero QM31 denominators, channel seeded with mix_u64(0x5EED0004)."""
    if rank != 0:
        return
    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200.synth import m31_column, qm31_array

    n = 1 << args.gkr_log
    ctx = z.Context(device=0, max_log_size=10)
    num = ctx.upload(m31_column(0x5EED0002, n))
    den = ctx.upload(qm31_array(0x5EED0003, n, nonzero=True))
    inst = [(z.GKR_LOGUP_MULTIPLICITIES, num.ptr, den.ptr, n)]
    words = None
    times = []
    for it in range(args.warmup + args.steps):
        ctx.sync()
        ctx.event_record(0)
        words = ctx.gkr_prove_device(inst, 0x5EED0004)
        ctx.event_record(1)
        if it >= args.warmup:
            times.append(ctx.event_elapsed_ms(0, 1))
    ctx.profile_begin()
    ctx.gkr_prove_device(inst, 0x5EED0004)
    kernels = ctx.profile_end()
    import hashlib

    ms = float(np.mean(times))
    line = {"metric": "gkr_fractions_per_s", "value": n / (ms * 1e-3), "unit": "fractions/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32 (M31/QM31)", "data": "synthetic",
            "config": {"workload": f"gkr_logup_multiplicities_2^{args.gkr_log}", "instances": 1},
            "rounds": sum(range(1, args.gkr_log)), "proof_words": int(len(words)),
            "proof_sha256": hashlib.sha256(words.tobytes()).hexdigest(),
            "parity": golden_check(f"gkr_logup_multiplicities_2e{args.gkr_log}", words),
            "gpu_launches": sum(v[1] for v in kernels.values()) * args.steps,
            "kernels_one_step": {k: {"ms": round(v[0], 4), "launches": v[1]} for k, v in kernels.items()}}
    if not args.no_cpu_baseline:
        import oracle

        small = min(args.gkr_log, 20)
        m = 1 << small
        t0 = time.perf_counter()
        oracle.gkr_prove([(2, m31_column(0x5EED0002, m), qm31_array(0x5EED0003, m, nonzero=True))], 0x5EED0004, verify=False)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": m / dt, "unit": "fractions/s", "cores": 1, "kind": "port",
                                "sample": f"one instance of 2^{small} fractions ({dt:.1f} s), scalar"}
    print(json.dumps(line))
    ctx.close()


def run_freivalds(args, rank):
    """--mode freivalds: the Freivalds component at the scaled-segment shape: n_in = n_out = 4096,
    32 tokens, 256 chunks (pk = 16, pq = 1, 2^20 rows), two matrices sharing the input."""
    if rank != 0:
        return
    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200.synth import qm31_array

    n_in, n_out, tokens, chunks, n_mats = 4096, 4096, 32, 256, 2
    pk, pq = n_out // chunks, -(-tokens // chunks)
    rows = n_in * chunks
    log_rows = (rows - 1).bit_length()
    grid = (log_rows, n_in, chunks, (1 << log_rows) - rows)
    rng = np.random.default_rng(0x5EED0005)
    qx = rng.integers(-128, 128, (tokens, n_in), dtype=np.int8)
    qws = [rng.integers(-128, 128, (n_in, n_out), dtype=np.int8) for _ in range(n_mats)]
    ctx = z.Context(device=0, max_log_size=10)
    d_qx, d_qw = ctx.upload_bytes(qx), [ctx.upload_bytes(w) for w in qws]
    R = 1 << log_rows
    base = [ctx.alloc(R) for _ in range(pq)]
    pre = [ctx.alloc(R) for _ in range(n_mats * pk + 4)]
    out = [ctx.alloc(R) for _ in range((1 + 2 * n_mats) * 4)]
    m_r8, off = ctx.alloc(256).zero(), ctx.alloc(2).zero()
    s, rv = qm31_array(1, 1)[0], qm31_array(2, 1)[0]
    t_sc, t_acc = [], []
    kernels = {}
    for it in range(args.warmup + args.steps + 1):
        if it == args.warmup + args.steps:
            ctx.profile_begin()  # one more, untimed pass with the library's own per-kernel events
        ctx.event_record(0)
        ctx.freivalds_scatter(d_qx.ptr, [w.ptr for w in d_qw], [n_out] * n_mats, grid, pq, pk, n_in, tokens, [b.ptr for b in base],
                              [p.ptr for p in pre], m_r8.ptr, 256, off.ptr)
        ctx.event_record(1)
        ctx.freivalds_acc([b.ptr for b in base], [p.ptr for p in pre[:n_mats * pk]], grid, pq, pk, n_mats, s, rv, [o.ptr for o in out])
        ctx.event_record(2)
        if it == args.warmup + args.steps:
            kernels = {k: round(v[0], 4) for k, v in ctx.profile_end().items()}
        elif it >= args.warmup:
            t_sc.append(ctx.event_elapsed_ms(0, 1))
            t_acc.append(ctx.event_elapsed_ms(1, 2))
    cells = (pq + n_mats * pk + 4) * R
    sc, ac = float(np.mean(t_sc)), float(np.mean(t_acc))
    gpu_ref = None
    if not args.no_gpu_baseline:
        try:  # the reference's own device chain on the same inputs (host clock around its blocking calls)
            import oracle
            from oracle import ref_cuda

            if ref_cuda.available():
                ref = ref_cuda.RefCudaFreivalds()
                s_pow, rv_pow = oracle.secure_powers(s, pq + 1), oracle.secure_powers(rv, pk + 1)
                rs, ra = [], []
                for it in range(3):
                    ref.sync()
                    t0 = time.perf_counter()
                    r_base, r_pre, r_m, r_c = ref.scatter(qx, qws, grid, pq, pk)
                    ref.sync()
                    t1 = time.perf_counter()
                    r_out, _ = ref.acc(r_base, r_pre, grid, pq, pk, n_mats, s, rv, s_pow[:pq], rv_pow[:pk], s_pow[pq], rv_pow[pk])
                    ref.sync()
                    t2 = time.perf_counter()
                    for p_ in r_base + r_pre + r_out + [r_m, r_c]:
                        ref.free(p_)
                    if it:
                        rs.append(t1 - t0)
                        ra.append(t2 - t1)
                gpu_ref = {"kind": "the reference's CUDA kernels, compiled unmodified for sm_100a, same GPU",
                           "scatter_ms_including_its_upload": 1e3 * float(np.mean(rs)), "acc_ms": 1e3 * float(np.mean(ra))}
        except Exception as e:
            gpu_ref = {"unavailable": repr(e)}
    print(json.dumps({"metric": "freivalds_cells_per_s", "value": cells / ((sc + ac) * 1e-3), "unit": "cells/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": sc + ac, "higher_is_better": True,
                      "config": {"workload": "freivalds_nin4096_nout4096_tokens32_chunks256_2mats", "rows": R, "pq": pq, "pk": pk},
                      "scatter_ms": sc, "scatter_gbs": (cells * 4 + n_mats * n_in * n_out) / (sc * 1e-3) / 1e9,
                      "acc_ms": ac, "acc_gbs": (4.0 * (pq + n_mats * pk) * R + 16.0 * (1 + 2 * n_mats) * R) / (ac * 1e-3) / 1e9,
                      "kernels_ms": kernels, "gpu_baseline": gpu_ref}))
    ctx.close()


def run_constraints(args, rank):
    """--mode constraints: evaluate_constraint_quotients_on_domain (zkb_constraint_quotients) for two AIRs of the reference at
    2^20 trace rows, evaluation domain 2^21: the wide Fibonacci example with --cols columns (base-field arithmetic, bandwidth
    heavy) and the Freivalds component at the scaled-segment shape pk = 16, pq = 1, two matrices, with its range check
    (secure-field arithmetic). Inputs are resident; columns are larger than L2."""
    if rank != 0:
        return
    from zk_inference_prover_b200 import air_cases
    import oracle
    import zk_inference_prover_b200 as z
    trace_log, eval_log = args.log_size, args.log_size + 1
    N = 1 << eval_log
    ctx = z.Context(device=0, max_log_size=10)
    results = {}

    def time_case(which):
        case = air_cases.bench_case(oracle, which, trace_log, args.cols)
        src = case["source"]
        prog = ctx.air_compile(src)
        st = prog.stats
        cols = [ctx.upload(c) for c in case["cols"]]
        case["cols"] = None
        acc = [ctx.alloc(N).zero() for _ in range(4)]
        ts = []
        for it in range(args.warmup + args.steps):
            ctx.event_record(0)
            ctx.constraint_quotients(prog, [c.ptr for c in cols], case["rcp"], trace_log, eval_log, [a.ptr for a in acc], accumulate=True,
                                     cumsum_shift=case["cumsum_shift"])
            ctx.event_record(1)
            ctx.sync()
            if it >= args.warmup:
                ts.append(ctx.event_elapsed_ms(0, 1))
        ms = float(np.mean(ts))
        # parity: one more pass that overwrites, against the committed digest of the oracle's output
        ctx.constraint_quotients(prog, [c.ptr for c in cols], case["rcp"], trace_log, eval_log, [a.ptr for a in acc], accumulate=False,
                                 cumsum_shift=case["cumsum_shift"])
        parity = golden_check(case["name"], np.stack([a.download() for a in acc]).reshape(-1))
        # the same program specialised into a kernel of its own (zkb_air_specialize)
        t0 = time.perf_counter()
        prog.specialize()
        jit_s = time.perf_counter() - t0
        tj = []
        for it in range(args.warmup + args.steps):
            ctx.event_record(0)
            ctx.constraint_quotients(prog, [c.ptr for c in cols], case["rcp"], trace_log, eval_log, [a.ptr for a in acc], accumulate=True,
                                     cumsum_shift=case["cumsum_shift"])
            ctx.event_record(1)
            ctx.sync()
            if it >= args.warmup:
                tj.append(ctx.event_elapsed_ms(0, 1))
        ctx.constraint_quotients(prog, [c.ptr for c in cols], case["rcp"], trace_log, eval_log, [a.ptr for a in acc], accumulate=False,
                                 cumsum_shift=case["cumsum_shift"])
        golden_check(case["name"], np.stack([a.download() for a in acc]).reshape(-1))
        ms_interp, ms = ms, float(np.mean(tj))
        st = prog.stats
        bytes_alg = (4.0 * st["n_columns_read"] + 32.0) * N  # every column read once, the accumulator read and written
        results[which] = {"workload": case["name"], "ms": ms, "ms_interpreter": ms_interp, "specialize_s": jit_s,
                          "rows_per_s": N / (ms * 1e-3), "columns": len(cols),
                          "constraints": int(src.n_constraints), "algorithmic_gbs": bytes_alg / (ms * 1e-3) / 1e9,
                          "m31_gmults_per_s": st["m31_mults"] * N / (ms * 1e-3) / 1e9, "program": st, "parity": parity}
        return cols, case["rcp"], ms, bytes_alg

    ncols = args.cols
    cols, rcp, wf_ms, wf_bytes = time_case("wide_fibonacci")
    gpu_ref = None
    if not args.no_gpu_baseline:
        try:  # the reference's hand-written kernel for the same AIR on the same columns (it overwrites; host clock around its blocking call)
            from oracle import ref_cuda

            if ref_cuda.available():
                ref = ref_cuda.RefCudaAir()
                denom = oracle.constraint_denom_inv(trace_log, eval_log)
                ptrs = [c.ptr for c in cols]
                rt = []
                for it in range(4):
                    ref.sync()
                    t0 = time.perf_counter()
                    r_out = ref.wide_fibonacci_quotients(ptrs, rcp, denom, trace_log, eval_log)
                    ref.sync()
                    dt = time.perf_counter() - t0
                    for p_ in r_out:
                        ref.free(p_)
                    if it:
                        rt.append(dt)
                gpu_ref = {"kind": "the reference's wide-Fibonacci CUDA kernel, compiled unmodified for sm_100a, same GPU, same columns",
                           "ms_including_its_allocations": 1e3 * float(np.mean(rt))}
        except Exception as e:
            gpu_ref = {"unavailable": repr(e)}
    del cols
    time_case("freivalds")
    cpu = None
    if not args.no_cpu_baseline:
        oracle.set_num_threads(len(os.sched_getaffinity(0)))
        small_eval = 15
        case = air_cases.wide_fibonacci_case(oracle, ncols, small_eval - 1, small_eval, 1)
        t0 = time.perf_counter()
        air_cases.by_air(oracle, case)
        dt = time.perf_counter() - t0
        cpu = {"value": ncols * (1 << (small_eval - 1)) / dt, "unit": "cells/s", "cores": oracle.num_threads(), "kind": "port",
               "sample": f"wide Fibonacci, {ncols} columns, evaluation domain 2^{small_eval} ({dt:.2f} s), the oracle's CpuDomainEvaluator restatement"}
    peak, peak_kind = measured_hbm_peak()
    line = {"metric": "constraint_cells_per_s", "value": ncols * (1 << trace_log) / (wf_ms * 1e-3), "unit": "cells/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wf_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32 (M31)", "data": "synthetic",
            "config": {"workload": f"constraint_quotients_wide_fibonacci_{ncols}cols_log{trace_log}_eval_log{eval_log}", "l2": "columns (2 GiB) are larger than L2"},
            "roofline": {"bound": "hbm", "kernel": "air_jit (the program's specialised kernel)", "achieved": wf_bytes / (wf_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": wf_bytes / (wf_ms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind, "traffic": None,
                         "note": "algorithmic bytes: every column read once, the accumulator read and written"},
            "gpu_launches": 2 * args.steps, "airs": results, "gpu_baseline": gpu_ref, "cpu_baseline": cpu}
    print(json.dumps(line))
    ctx.close()


def run_stark(args, rank):
    """--mode stark: a whole STARK proof of one component - prove() of the reference's generic prover - for the wide
    Fibonacci AIR over --cols columns of 2^--log-size rows: trace commitment, composition polynomial (constraint quotients
    with the program's specialised kernel), composition commitment, mask-point sampling, quotients, FRI, grind, decommit."""
    if rank != 0:
        return
    from zk_inference_prover_b200 import air_cases
    import oracle
    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200 import air

    n_cols, trace_log = args.cols, args.log_size
    kw = dict(pow_bits=args.pow_bits, log_blowup=args.log_blowup, n_queries=args.n_queries, cap=1 << 26)
    ctx = z.Context(device=0, max_log_size=trace_log + args.log_blowup)
    trace = air_cases.wide_fibonacci_trace(n_cols, trace_log)
    prog = ctx.air_compile(air.wide_fibonacci(air.ExprEvaluator(), n_cols).source())
    t0 = time.perf_counter()
    prog.specialize()
    jit_s = time.perf_counter() - t0
    n = 1 << trace_log
    src = [ctx.upload(c) for c in trace]
    work = [ctx.alloc(n) for _ in range(n_cols)]
    h_arr, pinned = ctx.alloc_pinned(n_cols * n)
    host = h_arr.reshape(n_cols, n)
    for c in range(n_cols):
        host[c] = trace[c]
    host_cols = [host[c] for c in range(n_cols)]
    phases = {}

    def step(e2e):
        if e2e:
            ctx.event_record(0)
            out = ctx.stark_prove(prog, [[], [], host_cols, []], trace_log, host=True, phases=phases, **kw)
        else:
            for w_, s_ in zip(work, src):
                ctx.d2d(w_.ptr, s_.ptr, n * 4)
            ctx.event_record(0)
            out = ctx.stark_prove(prog, [[], [], [w_.ptr for w_ in work], []], trace_log, phases=phases, **kw)
        ctx.event_record(1)
        ctx.sync()
        return out, ctx.event_elapsed_ms(0, 1)

    def timed(e2e):
        for _ in range(args.warmup):
            out, _ = step(e2e)
        ms = []
        for _ in range(args.steps):
            out, t = step(e2e)
            ms.append(t)
        return out, float(np.mean(ms))

    sampler = ClockSampler(0)
    sampler.start()
    out_dev, dev_ms = timed(False)
    clocks = sampler.stop()
    dev_phases = dict(phases)
    out_e2e, e2e_ms = timed(True)
    for out in (out_dev, out_e2e):
        assert (out[1] == out[2]).all(), "the proof fails the prover's own out-of-domain check"
    name = f"stark_wide_fibonacci_{n_cols}x2e{trace_log}_blowup{1 << args.log_blowup}"
    parity = golden_check(name, air_cases.stark_words(out_dev[0], out_dev[1], out_dev[2]))
    golden_check(name, air_cases.stark_words(out_e2e[0], out_e2e[1], out_e2e[2]))
    cells = n_cols * n
    cpu = None
    if not args.no_cpu_baseline:
        oracle.set_num_threads(len(os.sched_getaffinity(0)))
        sc, sl = min(n_cols, 32), min(trace_log, 16)
        tr = air_cases.wide_fibonacci_trace(sc, sl)
        t0 = time.perf_counter()
        oracle.stark_prove(0, [sc], np.zeros(4, np.uint32), [0, 0, sc, 0], tr, sl, sl + 1, pow_bits=args.pow_bits, log_blowup=args.log_blowup,
                           n_queries=args.n_queries)
        dt = time.perf_counter() - t0
        cpu = {"value": sc * (1 << sl) / dt, "unit": "cells/s", "cores": oracle.num_threads(), "kind": "port",
               "sample": f"the same proof of {sc} columns x 2^{sl} rows ({dt:.1f} s), the oracle's restatement of prove()"}
    line = {"metric": "committed_m31_cells_per_s", "value": cells / (dev_ms * 1e-3), "unit": "cells/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32 (M31)",
            "data": "synthetic (a valid wide Fibonacci trace)",
            "config": {"workload": f"stark_prove_wide_fibonacci_{n_cols}cols_log{trace_log}_blowup{1 << args.log_blowup}",
                       "step": "trace commit + composition polynomial + composition commit + mask-point samples + quotients + FRI + grind + decommit",
                       "pow_bits": args.pow_bits, "n_queries": args.n_queries, "l2": "inputs (1 GiB) are larger than L2"},
            "e2e": {"value": cells / (e2e_ms * 1e-3), "unit": "cells/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": cells * 4,
                    "d2h_bytes_per_step": int(out_e2e[0].size * 4)},
            "per_phase_ms": dev_phases, "specialize_s": jit_s, "clocks": clocks, "parity": parity, "proof_words": int(out_dev[0].size),
            "cpu_baseline": cpu}
    print(json.dumps(line))
    ctx.free_pinned(pinned)
    ctx.close()


def run_segment_replay(args, rank):
    """--mode segment-replay: the operator trace of one composed decode segment, replayed on seeded random columns.

    A segment of the reference prover is one STARK over hundreds of components of different heights (tens of thousands of
    columns of 2^4..2^23 rows) plus five batched LogUp-GKR reductions. tests/golden/segment_shapes.json holds those shapes,
    made from the reference's cell-exact cost model by tests/golden/make_segment_shapes.py. One step here: copy the trace in
    (device to device), commit the base, interaction and boundary trees and eight composition columns, prove one opening per column with the prover's own
    PcsConfig (blow-up 2, 100 queries, no proof of work), then one GKR batch proof per reduction family over LogUpSingles
    instances of the components' lookup counts (a component of L lookups per row is split along the binary decomposition of
    L, as the reference does). Timing only: the witness values, the gadgets' constraint programs and the digest of a real
    segment need the application code above the operators."""
    if rank != 0:
        return
    import zk_inference_prover_b200 as z

    P = (1 << 31) - 1
    seg = json.load(open(os.path.join(ROOT, "tests", "golden", "segment_shapes.json")))["segments"][args.segment]
    trees = [[], [], []]
    gkr = {}
    for c in seg["components"]:
        for _ in range(c["repeat"]):
            trees[0] += [c["log_rows"]] * c["base_cols"]
            trees[1] += [c["log_rows"]] * c["interaction_cols"]
            looks, b = c["lookups_per_row"], 0
            while looks:
                if looks & 1:
                    gkr.setdefault(c["family"], []).append(c["log_rows"] + b)
                looks >>= 1
                b += 1
    for b in seg["boundary_cols"]:
        trees[2] += [b["log_rows"]] * b["cols"]
    cells = sum(1 << l for t in trees for l in t)
    assert cells == seg["cells"]["fresh"]
    # the composition polynomial's eight half-coordinate columns at the height of the tallest trace: the last tree of a proof,
    # to whose height every column is lifted. Not counted in the committed trace cells.
    trees.append([max(l for t in trees for l in t)] * 8)
    logs = [l for t in trees for l in t]
    total_words = sum(1 << l for l in logs)
    log_blowup = 1
    ctx = z.Context(device=0, max_log_size=max(logs) + log_blowup)
    rng = np.random.default_rng(0x5EED0006)
    pristine = ctx.upload(rng.integers(0, P, total_words, dtype=np.uint32))
    work = ctx.alloc(total_words)
    ptrs, off = [], 0
    for t in trees:
        tp = []
        for l in t:
            tp.append(work.ptr + 4 * off)
            off += 1 << l
        ptrs.append(tp)
    gkr_entries = sum(1 << l for v in gkr.values() for l in v)
    dens = ctx.upload(rng.integers(1, P, 4 * gkr_entries, dtype=np.uint32))
    batches, off = [], 0
    for fam, ls in gkr.items():
        inst = []
        for l in sorted(ls, reverse=True):
            inst.append((z.GKR_LOGUP_SINGLES, 0, dens.ptr + 16 * off, 1 << l))
            off += 1 << l
        batches.append((fam, inst))
    prepared = ctx.pcs_prepare(ptrs, logs, cap=1 << 25)
    sampler = ClockSampler(0)
    t_pcs, t_gkr, phases, gkr_family_ms = [], [], None, {}
    for it in range(args.warmup + args.steps):
        if it == args.warmup:
            sampler.start()
        ctx.sync()
        ctx.event_record(0)
        ctx.d2d(work.ptr, pristine.ptr, total_words * 4)
        words, ph = ctx.pcs_prove_device(prepared, None, pow_bits=0, log_blowup=log_blowup, log_last_layer=0, n_queries=100, phases=True)
        ctx.event_record(1)
        gw = []
        for i, (_f, inst) in enumerate(batches):
            gw.append(ctx.gkr_prove_device(inst, 0x5EED0007 + i, cap=1 << 24))
            ctx.event_record(2 + i)
        ctx.sync()
        if it >= args.warmup:
            t_pcs.append(ctx.event_elapsed_ms(0, 1))
            t_gkr.append(ctx.event_elapsed_ms(1, 1 + len(batches)))
            for i, (f, _inst) in enumerate(batches):
                gkr_family_ms[f] = gkr_family_ms.get(f, 0.0) + ctx.event_elapsed_ms(1 + i, 2 + i) / args.steps
            phases = ph if phases is None else {k: phases[k] + ph[k] for k in ph}
    clocks = sampler.stop()
    ctx.profile_begin()
    ctx.d2d(work.ptr, pristine.ptr, total_words * 4)
    ctx.pcs_prove_device(prepared, None, pow_bits=0, log_blowup=log_blowup, log_last_layer=0, n_queries=100)
    for i, (_f, inst) in enumerate(batches):
        ctx.gkr_prove_device(inst, 0x5EED0007 + i, cap=1 << 24)
    kernels = ctx.profile_end(cap=128)
    pcs_ms, gkr_ms = float(np.mean(t_pcs)), float(np.mean(t_gkr))
    ms = pcs_ms + gkr_ms
    top = sorted(kernels.items(), key=lambda kv: -kv[1][0])[:12]
    print(json.dumps({
        "metric": "segment_proof_ms (operator-trace replay)", "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "u32 (M31/QM31)", "data": "synthetic",
        "config": {"workload": f"segment_replay_{args.segment}", "note": seg["note"], "columns": len(logs),
                   "tree_columns": [len(t) for t in trees], "log_rows": [min(logs), max(logs)], "log_blowup": log_blowup,
                   "n_queries": 100, "gkr_batches": {f: len(i) for f, i in batches}, "gkr_entries": gkr_entries,
                   "l2": "inputs larger than L2"},
        "cells": cells, "cells_per_s": cells / (ms * 1e-3), "pcs_ms": pcs_ms, "gkr_ms": gkr_ms, "gkr_ms_by_family": gkr_family_ms,
        "per_phase_ms": {k: v / args.steps for k, v in phases.items()}, "pcs_proof_words": int(words.size),
        "gkr_proof_words": int(sum(w.size for w in gw)), "clocks": clocks,
        "gpu_launches": int(sum(v[1] for v in kernels.values())) * args.steps,
        "launches_one_step": int(sum(v[1] for v in kernels.values())),
        "top_kernels_one_step": {k: {"ms": round(v[0], 3), "launches": v[1]} for k, v in top}}))
    ctx.close()


class SegmentReplay:
    """The device buffers and argument arrays of one segment shape of tests/golden/segment_shapes.json, and one step over
    them (see run_segment_replay for what a step is)."""

    def __init__(self, z, ctx, name, seed):
        P = (1 << 31) - 1
        seg = json.load(open(os.path.join(ROOT, "tests", "golden", "segment_shapes.json")))["segments"][name]
        trees, gkr = [[], [], []], {}
        for c in seg["components"]:
            for _ in range(c["repeat"]):
                trees[0] += [c["log_rows"]] * c["base_cols"]
                trees[1] += [c["log_rows"]] * c["interaction_cols"]
                looks, b = c["lookups_per_row"], 0
                while looks:
                    if looks & 1:
                        gkr.setdefault(c["family"], []).append(c["log_rows"] + b)
                    looks >>= 1
                    b += 1
        for b in seg["boundary_cols"]:
            trees[2] += [b["log_rows"]] * b["cols"]
        self.cells = sum(1 << l for t in trees for l in t)
        assert self.cells == seg["cells"]["fresh"]
        trees.append([max(l for t in trees for l in t)] * 8)  # the composition columns: the last and tallest tree
        logs = [l for t in trees for l in t]
        self.max_log = max(logs)
        self.ctx, self.total_words = ctx, sum(1 << l for l in logs)
        rng = np.random.default_rng(seed)
        self.pristine = ctx.upload(rng.integers(0, P, self.total_words, dtype=np.uint32))
        self.work = ctx.alloc(self.total_words)
        ptrs, off = [], 0
        for t in trees:
            tp = []
            for l in t:
                tp.append(self.work.ptr + 4 * off)
                off += 1 << l
            ptrs.append(tp)
        entries = sum(1 << l for v in gkr.values() for l in v)
        self.dens = ctx.upload(rng.integers(1, P, 4 * entries, dtype=np.uint32))
        self.batches, off = [], 0
        for _fam, ls in gkr.items():
            inst = []
            for l in sorted(ls, reverse=True):
                inst.append((z.GKR_LOGUP_SINGLES, 0, self.dens.ptr + 16 * off, 1 << l))
                off += 1 << l
            self.batches.append(inst)
        self.prepared = ctx.pcs_prepare(ptrs, logs, cap=1 << 25)

    def step(self):
        ctx = self.ctx
        ctx.d2d(self.work.ptr, self.pristine.ptr, self.total_words * 4)
        ctx.pcs_prove_device(self.prepared, None, pow_bits=0, log_blowup=1, log_last_layer=0, n_queries=100)
        for i, inst in enumerate(self.batches):
            ctx.gkr_prove_device(inst, 0x5EED0007 + i, cap=1 << 24)


def run_decode_step(args, rank, world, local_rank):
    """--mode decode-step: the proof of one decode step of the 32-layer model as operator-trace replays: 32 layer segments and
    the output head (the shapes of run_segment_replay), dealt round-robin to the ranks. Segments are independent proofs, so
    there is no collective on the data path; NCCL carries the barrier and the maximum over ranks of the device time."""
    import zk_inference_prover_b200 as z

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        with stdout_to_stderr():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
    names = ["layer_8b_s32_c2048"] * 32 + ["head_8b_s32_c2048"]
    mine = names[rank::world]
    # A segment's proof keeps the host busy for two thirds of its time, so a rank may run
    # several proofs side by side: --streams S gives it S host threads, each with a context (a stream) of its own, and deals
    # the rank's segments to them. The library allows one thread per context and any number of contexts.
    S = max(1, args.streams)
    ctxs = [z.Context(device=local_rank, max_log_size=24) for _ in range(S)]
    ctx = ctxs[0]
    work = [mine[k::S] for k in range(S)]
    shapes = [{n: SegmentReplay(z, ctxs[k], n, 0x5EED0006 + rank + 100 * k) for n in sorted(set(work[k]))} for k in range(S)]
    sampler = ClockSampler(local_rank)

    def barrier():
        for c in ctxs:
            c.sync()
        if dist is not None:
            dist.barrier()

    def one_pass():
        def run(k):
            for n in work[k]:
                shapes[k][n].step()
            ctxs[k].sync()

        if S == 1:
            run(0)
            return
        threads = [threading.Thread(target=run, args=(k,)) for k in range(S)]
        for th in threads:
            th.start()
        for th in threads:
            th.join()

    for _ in range(args.warmup):
        one_pass()
    barrier()
    if rank == 0:
        sampler.start()
    ctx.event_record(0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_pass()
    ctx.event_record(1)
    barrier()
    # one stream: CUDA events on it; several: the host clock between the two barriers (no single stream sees all the work)
    ms = ctx.event_elapsed_ms(0, 1) / args.steps if S == 1 else (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        import torch

        t = torch.tensor([ms], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    cells = 32 * 226711536 + 191812784
    if rank == 0:
        print(json.dumps({
            "metric": "decode_step_proof_ms (operator-trace replay)", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32 (M31/QM31)", "data": "synthetic",
            "config": {"workload": "decode_step_replay_32_layer_segments_plus_head", "segments": len(names),
                       "segments_on_rank_0": len(mine), "parallelism": f"segments round-robin over {world} GPU(s), no collective", "streams_per_gpu": S,
                       "timer": "cuda events" if S == 1 else "host clock between barriers",
                       "l2": "inputs larger than L2"},
            "cells": cells, "cells_per_s": cells / (ms * 1e-3), "ms_per_segment": ms / len(mine), "clocks": clocks}))
    for c in ctxs:
        c.close()
    if dist is not None:
        dist.destroy_process_group()


def run_witness(args, rank):
    """--mode witness: the device witness generators at the sizes of a layer segment, and a proof whose trace never leaves the
    device. Generators: the tables' own columns at 2^23 rows with four key-tile counters; a dequantize component of the
    bf16-chain variant for a 4096 x 4096 matmul over 512 tokens (16 slots per row, 2^17 rows, 242 committed and 37
    preprocessed columns); a residual-stream component (128 bf16 additions per row over 2^15 rows: 2,304 committed columns);
    the normalisation table's six preprocessed columns and its multiplicities. Byte work: reported against the HBM peak with
    the algorithmic bytes (every column written once, every input read once). The last leg generates the dequantize and
    residual-stream traces on the device and commits and opens them in one PCS proof (the reference's own device path: witness
    kernels, then commit, with no trace upload)."""
    if rank != 0:
        return
    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200.witness_cases import dequant_case, residual_stream_case, tables_case

    peak, peak_kind = measured_hbm_peak()
    ctx = z.Context(device=0, max_log_size=20)
    log_rows, n_counters = 23, 4
    expmap, counters, _, _ = tables_case(7, log_rows, n_counters)
    rows = 1 << log_rows
    d_map, d_cnt = ctx.upload(expmap), [ctx.upload(c) for c in counters]
    x, y, m = ctx.alloc(rows), ctx.alloc(rows), ctx.alloc(rows)
    case = dequant_case(8, 1, tokens=512, chunks=256, per_row=16, kmax=19, sticky=1, do_ref=0)
    cfg, drows = case["cfg"], case["rows"]
    up = lambda a: ctx.upload_bytes(np.ascontiguousarray(a))
    d_acc, d_norm, d_mul, d_sx, d_sw = up(case["acc"]), ctx.upload(case["norm3"]), ctx.upload(case["mul2"]), ctx.upload(case["sx"]), ctx.upload(case["sw"])
    base = [ctx.alloc(drows) for _ in range(case["n_base"])]
    pre = [ctx.alloc(drows) for _ in range(case["n_pre"])]
    m_norm, m_frac = ctx.alloc(cfg["n_norm"]).zero(), ctx.alloc(cfg["n_frac"]).zero()
    m_mul, m_r8, counts = ctx.alloc(cfg["n_mul"]).zero(), ctx.alloc(cfg["n_r8"]).zero(), ctx.alloc(3).zero()
    # residual stream: hd = 128 additions per row
    rs_log = 15
    rs = residual_stream_case(9, "pairs", 128, rs_log, 1 << rs_log, kind=0, sticky=True, kmax=13, spread=8)
    rrows, ml = 1 << rs_log, rs["m_len"]
    r_wit, r_norm = ctx.upload(rs["wit"]), ctx.upload(rs["norm3"])
    r_smul = up(np.ascontiguousarray(rs["smul3"], np.int32))
    r_cols = [ctx.alloc(rrows) for _ in range(rs["n_cols"])]
    r_out_pat, r_out_nat, r_in_nat = ctx.alloc(rrows * 128), ctx.alloc(rrows * 256), ctx.alloc(rrows * rs["n_leaves"] * 2)
    r_ms = {k: ctx.alloc(ml[k]).zero() for k in ("pow", "norm", "val", "frac", "smul")}
    r_counts = ctx.alloc(4).zero()
    # the normalisation table of that component: 256 + 14 * 512 rows in 2^13
    t_cols, t_m = [ctx.alloc(1 << 13) for _ in range(6)], ctx.alloc(1 << 13)

    def gen_residual():
        ctx.witness_residual_stream(rs["lowered_groups"], rs["lowered_slots"], rs["out_slot"], 0, True, 13, r_norm.ptr, len(rs["norm3"]) // 3,
                                    r_smul.ptr, len(rs["smul3"]) // 3, [], rs["n_val"], r_wit.ptr, rrows, rs_log, [c.ptr for c in r_cols],
                                    r_out_pat.ptr, r_out_nat.ptr, r_in_nat.ptr, {k: (v.ptr, ml[k]) for k, v in r_ms.items()}, [], r_counts.ptr)

    def gen_dequant():
        ctx.witness_dequant(cfg, d_acc.ptr, 0, 0, d_sx.ptr, d_sw.ptr, d_norm.ptr, d_mul.ptr, [b.ptr for b in base], [p.ptr for p in pre],
                            m_norm.ptr, m_frac.ptr, m_mul.ptr, m_r8.ptr, counts.ptr, 0)

    trace_ptrs = [b.ptr for b in base] + [c.ptr for c in r_cols]
    trace_logs = [drows.bit_length() - 1] * len(base) + [rs_log] * len(r_cols)
    t_tab, t_deq, t_rs, t_pre, t_gen, t_prove = [], [], [], [], [], []
    words = None
    for it in range(args.warmup + args.steps):
        ctx.sync()
        ctx.event_record(0)
        ctx.witness_tables(d_map.ptr, [c.ptr for c in d_cnt], log_rows, False, 2.0 ** 7, x.ptr, y.ptr, m.ptr)
        ctx.event_record(1)
        gen_dequant()
        ctx.event_record(2)
        gen_residual()
        ctx.event_record(3)
        ctx.witness_pre_table(0, 13, 13, 0, [r_ms["norm"].ptr], [c.ptr for c in t_cols], t_m.ptr)
        ctx.event_record(4)
        ctx.sync()
        # the trace generated on the device, committed and opened where it lies
        ctx.event_record(5)
        gen_dequant()
        gen_residual()
        ctx.event_record(6)
        words = ctx.pcs_prove_device([trace_ptrs], trace_logs, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=70, cap=1 << 26)
        ctx.event_record(7)
        ctx.sync()
        if it >= args.warmup:
            t_tab.append(ctx.event_elapsed_ms(0, 1))
            t_deq.append(ctx.event_elapsed_ms(1, 2))
            t_rs.append(ctx.event_elapsed_ms(2, 3))
            t_pre.append(ctx.event_elapsed_ms(3, 4))
            t_gen.append(ctx.event_elapsed_ms(5, 6))
            t_prove.append(ctx.event_elapsed_ms(6, 7))
    tab_ms, deq_ms, rs_ms, pre_ms = (float(np.mean(t)) for t in (t_tab, t_deq, t_rs, t_pre))
    gen_ms, prove_ms = float(np.mean(t_gen)), float(np.mean(t_prove))
    tab_bytes = rows * 4 * (3 + n_counters)
    deq_bytes = drows * 4 * (case["n_base"] + case["n_pre"] + cfg["per_row"])
    rs_bytes = rrows * 4 * (rs["n_cols"] + rs["n_leaves"] * 3 + 128 * 3)  # columns, patterns in, natural pairs in and out, patterns out
    cells = 3 * rows + drows * (case["n_base"] + case["n_pre"]) + rrows * rs["n_cols"]
    trace_cells = drows * len(base) + rrows * len(r_cols)
    gbs = lambda by, ms: by / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "witness_cells_per_s", "value": cells / ((tab_ms + deq_ms + rs_ms) * 1e-3), "unit": "cells/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": tab_ms + deq_ms + rs_ms, "higher_is_better": True, "dtype": "u32 / i32", "data": "synthetic",
        "config": {"workload": "witness_tables_2^23_4counters + witness_dequant_chain_512x4096_per_row16 + residual_stream_128adds_2^15"},
        "tables": {"ms": tab_ms, "algorithmic_bytes": tab_bytes, "gbs": gbs(tab_bytes, tab_ms), "frac_of_hbm_peak": gbs(tab_bytes, tab_ms) / peak},
        "dequant": {"ms": deq_ms, "columns": case["n_base"] + case["n_pre"], "rows": drows, "algorithmic_bytes": deq_bytes,
                    "gbs": gbs(deq_bytes, deq_ms), "frac_of_hbm_peak": gbs(deq_bytes, deq_ms) / peak, "counts": counts.download().tolist()},
        "residual_stream": {"ms": rs_ms, "columns": rs["n_cols"], "rows": rrows, "slots_per_row": 128, "algorithmic_bytes": rs_bytes,
                            "gbs": gbs(rs_bytes, rs_ms), "frac_of_hbm_peak": gbs(rs_bytes, rs_ms) / peak, "counts": r_counts.download()[:3].tolist()},
        "norm_table": {"ms": pre_ms, "rows": 1 << 13, "columns": 7, "note": "launch-latency sized: 229 KB written"},
        "device_trace_to_proof": {"ms": gen_ms + prove_ms, "witness_ms": gen_ms, "proof_ms": prove_ms, "cells": trace_cells,
                                  "cells_per_s": trace_cells / ((gen_ms + prove_ms) * 1e-3), "columns": len(trace_ptrs),
                                  "h2d_trace_bytes": 0, "proof_words": int(words.size),
                                  "what": "dequantize (2^17 rows) and residual-stream (2^15 rows) traces written by the witness kernels and "
                                          "committed and opened in one PCS proof (blow-up 2, 70 queries); nothing of the trace is uploaded"},
        "peak_gbs": peak, "peak_kind": peak_kind, "gpu_launches": 4 * args.steps}))
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cols", type=int, default=256)
    ap.add_argument("--log-size", type=int, default=20)
    ap.add_argument("--log-blowup", type=int, default=2)
    ap.add_argument("--pow-bits", type=int, default=10)
    ap.add_argument("--n-queries", type=int, default=3)
    ap.add_argument("--ref-cols", type=int, default=0, help="columns in the CPU legs (0: every column of the workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the legs beside the headline (h2d ceiling, sharded proof, segment replays)")
    ap.add_argument("--gkr-log", type=int, default=24)
    ap.add_argument("--streams", type=int, default=1, help="decode-step: proofs side by side on one GPU (host threads, one context each)")
    ap.add_argument("--segment", default="layer_8b_s32_c2048", help="segment-replay: a key of tests/golden/segment_shapes.json")
    ap.add_argument("--mode", default="proof", choices=["proof", "sharded-commit", "gkr", "freivalds", "constraints", "stark", "segment-replay", "decode-step", "witness"],
                    help="proof: one whole PCS proof per rank (ranks are independent); sharded-commit: one commitment over all ranks")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    elif args.mode == "sharded-commit":
        run_sharded_commit(args, rank, world, local_rank)
    elif args.mode == "gkr":
        run_gkr(args, rank)
    elif args.mode == "freivalds":
        run_freivalds(args, rank)
    elif args.mode == "constraints":
        run_constraints(args, rank)
    elif args.mode == "stark":
        run_stark(args, rank)
    elif args.mode == "segment-replay":
        run_segment_replay(args, rank)
    elif args.mode == "witness":
        run_witness(args, rank)
    elif args.mode == "decode-step":
        run_decode_step(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
