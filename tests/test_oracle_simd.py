"""The oracle's packed (16-lane) restatement of the reference's SIMD backend against the scalar oracle, word for word:
every packed operator (interpolate, evaluate, leaf hashing with ragged column counts, out-of-domain evaluation, quotient
numerators) and whole proofs, which also pass the restated verifier. The packed code exists to be timed as the CPU
baseline; this test is what lets that timing stand for the same computation."""
import numpy as np
import pytest

from util import edge_m31_column, m31_column, qm31_array


@pytest.fixture()
def simd(oracle):
    lanes = oracle.set_simd(True)
    if lanes == 0:
        oracle.set_simd(False)
        pytest.skip("this CPU has neither AVX-512 nor AVX2")
    yield oracle
    oracle.set_simd(False)


def _both(oracle, fn):
    oracle.set_simd(False)
    want = fn()
    assert oracle.set_simd(True) > 0
    got = fn()
    return got, want


@pytest.mark.parametrize("log_n", [5, 6, 9, 12, 16])
def test_packed_interpolate_and_evaluate(simd, log_n):
    vals = np.stack([edge_m31_column(300 + c, 1 << log_n) for c in range(3)])
    got, want = _both(simd, lambda: simd.interpolate_cols(vals, log_n))
    assert (got == want).all()
    for blow in (1, 2):
        g, w = _both(simd, lambda: simd.evaluate_cols(want, log_n, log_n + blow))
        assert (g == w).all()


@pytest.mark.parametrize("ncols", [1, 15, 16, 17, 33, 100])
@pytest.mark.parametrize("m31", [True, False])
def test_packed_leaf_hashes(simd, ncols, m31):
    log = 7
    cols = [edge_m31_column(400 + c, 1 << log) for c in range(ncols)]
    got, want = _both(simd, lambda: simd.commit_on_layer(log, None, cols, m31=m31))
    assert (got == want).all()


def test_packed_inner_merkle_layers(simd):
    log = 8
    cols = [edge_m31_column(450 + c, 1 << log) for c in range(5)]
    for m31 in (True, False):
        def tree():
            layer = simd.commit_on_layer(log, None, cols, m31=m31)
            out = [layer]
            for lg in range(log - 1, -1, -1):
                layer = simd.commit_on_layer(lg, layer, [], m31=m31)
                out.append(layer)
            return np.concatenate([o.reshape(-1) for o in out])
        got, want = _both(simd, tree)
        assert (got == want).all()


def test_packed_whole_proofs_equal_scalar_and_verify(simd):
    for shape, kw in [([[8] * 20], dict(pow_bits=5, log_blowup=2, n_queries=6)),
                      ([[6, 7, 7, 9], [10] * 3], dict(pow_bits=0, log_blowup=1, n_queries=30, two_sample_every=2))]:
        trees = [[m31_column(500 + 10 * t + c, 1 << l) for c, l in enumerate(logs)] for t, logs in enumerate(shape)]
        got, want = _both(simd, lambda: simd.pcs_prove(trees, **kw))
        assert len(got) == len(want) and (got == want).all()
        assert simd.pcs_verify(got, shape, **kw) == (0, 0, -1)
