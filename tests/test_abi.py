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


def test_rust_binding_matches_the_headers():
    """shim/src/ffi.rs is what shim/gen_ffi.py writes from include/*.h today (the Rust binding cannot drift)."""
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "shim", "gen_ffi.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    ffi = open(os.path.join(ROOT, "shim", "src", "ffi.rs")).read()
    bound = set(re.findall(r"pub fn (zkb_[a-z0-9_]+)\(", ffi))
    assert bound == set(zkb_all_symbols())
    # every module lib.rs declares exists, and every zkb_* a module calls is declared in ffi.rs
    src = os.path.join(ROOT, "shim", "src")
    for mod in re.findall(r"^(?:pub )?mod ([a-z_]+);", open(os.path.join(src, "lib.rs")).read(), flags=re.M):
        text = open(os.path.join(src, mod + ".rs")).read()
        if mod != "ffi":
            called = set(re.findall(r"ffi::(zkb_[a-z0-9_]+)", text))
            assert called <= bound, (mod, sorted(called - bound))
            # no rustc here: at least the number of arguments at each call site equals the declaration's
            for m in re.finditer(r"ffi::(zkb_[a-z0-9_]+)\(", text):
                assert _call_args(text, m.end() - 1) == _declared_args(ffi, m.group(1)), (mod, m.group(1))


def _declared_args(ffi, name):
    m = re.search(r"pub fn " + name + r"\(([^;]*?)\)\s*(?:->[^;]*)?;", ffi, flags=re.S)
    return len([a for a in m.group(1).split(",") if a.strip()])


def _call_args(text, open_paren):
    depth, commas, j = 0, 0, open_paren
    while True:
        c = text[j]
        if c in "([{":
            depth += 1
        elif c in ")]}":
            depth -= 1
            if depth == 0:
                break
        elif c == "," and depth == 1:
            commas += 1
        j += 1
    inner = text[open_paren + 1:j].strip()
    if not inner:
        return 0
    return commas + (0 if inner.endswith(",") else 1)


def zkb_all_symbols():
    from zk_inference_prover_b200 import capi
    return list(capi.EXPORTED_SYMBOLS) + list(capi.PROVER_SYMBOLS) + list(capi.AIR_SYMBOLS)
