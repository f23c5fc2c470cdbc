"""The C-ABI library loads without a GPU and exports every symbol include/zkb200.h declares."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_are_exported(zkb):
    header = open(os.path.join(ROOT, "include", "zkb200.h")).read()
    declared = set(re.findall(r"\b(zkb_[a-z0-9_]+)\s*\(", header))
    declared.discard("zkb_ctx")
    lib = zkb.load_library()
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, missing
    assert declared == set(zkb.EXPORTED_SYMBOLS)
    header = open(os.path.join(ROOT, "include", "zkb200_prover.h")).read()
    declared = set(re.findall(r"\b(zkb_[a-z0-9_]+)\s*\(", header))
    assert declared == set(zkb.PROVER_SYMBOLS)
    assert all(hasattr(lib, s) for s in declared)
    header = open(os.path.join(ROOT, "include", "zkb200_air.h")).read()
    declared = set(re.findall(r"\b(zkb_[a-z0-9_]+)\s*\(", header))
    assert declared == set(zkb.AIR_SYMBOLS)
    assert all(hasattr(lib, s) for s in declared)


def test_no_oracle_in_product():
    """The product never reaches into oracle/ (the oracle is a checker, not a code path)."""
    pkg = os.path.join(ROOT, "zk_inference_prover_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                for needle in ("import oracle", "from oracle", "oracle/", "zko_", "zkoracle"):
                    assert needle not in text, (os.path.join(dirpath, f), needle)
