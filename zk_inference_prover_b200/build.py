"""Builds libzkb200.so (the CUDA library behind include/zkb200.h) for sm_100a with nvcc.

The library is plain CUDA runtime code: no torch headers, no third-party dependencies.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libzkb200.so")

SOURCES = ["ctx.cu", "fft.cu", "bitrev.cu", "blake2s.cu", "fri.cu", "quotients.cu", "gkr.cu", "gkr_fused.cu", "gkr_resident.cu", "gkr_batch.cu", "poly_eval.cu", "poly_bary.cu", "freivalds.cu", "witness_gen.cu", "witness_pre.cu", "constraints.cu", "host/prover.cpp", "host/air_compile.cpp", "host/air_jit.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(dp, f) for dp, _, fs in os.walk(CSRC) for f in fs] + [os.path.join(HERE, "..", "include", "zkb200.h"), os.path.join(HERE, "..", "include", "zkb200_prover.h"), os.path.join(HERE, "..", "include", "zkb200_air.h"), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every .cu of the package into lib/libzkb200.so. Returns the library path."""
    if not force and not _stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIB_DIR, os.path.basename(src).replace(".cu", ".o").replace(".cpp", ".o"))
        extra = os.environ.get("ZKB_NVCC_EXTRA", "").split()
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose or "warning" in out:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-ldl", "-lpthread"]  # cudart is linked statically (nvcc default)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
