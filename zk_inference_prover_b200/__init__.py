"""zkb200: B200 (sm_100a) CUDA kernels for the Circle-STARK backend operators, behind a C ABI.

The product is lib/libzkb200.so (built from csrc/ by build.py; interface in include/zkb200.h).
This package is the thin ctypes binding used by the tests and the benchmark. There is no CPU
fallback: loading fails loudly when the library has not been built.
"""
from .capi import (  # noqa: F401
    Context,
    DeviceBuffer,
    ZkbError,
    lib_path,
    load_library,
    gkr_sum_noalloc,
    GKR_GRAND_PRODUCT,
    GKR_LOGUP_GENERIC,
    GKR_LOGUP_MULTIPLICITIES,
    GKR_LOGUP_SINGLES,
    EXPORTED_SYMBOLS,
    PROVER_SYMBOLS,
    AIR_SYMBOLS,
    AirProgram,
    air_analyze,
    constraint_denom_inv,
    PCS_PHASES,
)
from . import air, capi  # noqa: F401,E402
