"""Whole commitments, FRI proofs and GKR proofs from the CUDA path against the CPU oracle's
restatement of the reference's protocol code, word for word (roots, sampled values, every FRI layer
root, the last-layer polynomial, the proof-of-work nonce, queried values, decommitments, and the
channel digest after the proof). The oracle side also checks its own proof: FRI's last layer must
have the committed degree and the GKR proof must pass partially_verify_batch. Shapes follow
nitroo/crates/stwo/src/prover/pcs/quotient_ops.rs:324-399 (prove_and_verify_pcs with mixed column
sizes) and nitroo/crates/stwo/benches/{pcs,lookups}.rs."""
import numpy as np
import pytest

from util import m31_column, qm31_array

pytestmark = pytest.mark.gpu


def _trees(shape, seed):
    return [[m31_column(seed + 100 * t + c, 1 << lg) for c, lg in enumerate(logs)] for t, logs in enumerate(shape)]


@pytest.mark.parametrize(
    "shape,kw",
    [
        ([[6]], dict(pow_bits=0, log_blowup=1, n_queries=3)),
        ([[5, 5, 5]], dict(pow_bits=10, log_blowup=1, n_queries=3)),                      # library default PcsConfig
        ([[8] * 10], dict(pow_bits=10, log_blowup=2, n_queries=3)),
        ([[4, 6, 6, 5, 8, 8, 4]], dict(pow_bits=3, log_blowup=1, n_queries=20, two_sample_every=2)),
        ([[6, 6], [7, 5, 7, 3]], dict(pow_bits=0, log_blowup=1, n_queries=100)),           # the prover's own parameters
        ([[10] * 17 + [7] * 3], dict(pow_bits=5, log_blowup=2, n_queries=16, log_last_layer=2, two_sample_every=5)),
        ([[12] * 8, [12] * 3 + [9] * 2], dict(pow_bits=8, log_blowup=1, n_queries=30, log_last_layer=1, two_sample_every=3)),
    ],
)
def test_pcs_proof_matches_oracle(ctx, oracle, shape, kw):
    trees = _trees(shape, 4000)
    want = oracle.pcs_prove(trees, **kw)
    got = ctx.pcs_prove_host(trees, **kw)
    assert len(got) == len(want)
    assert (got == want).all()
    # and the reference's verifier (oracle/verify.hpp) accepts what the CUDA path wrote
    assert oracle.pcs_verify(got, shape, **kw) == (0, 0, -1)


def test_verifier_rejects_a_tampered_cuda_proof(ctx, oracle):
    """accepts=true has to mean something: the same verifier that accepts the CUDA path's proof rejects it after one word
    of a queried value, of a FRI witness or of the nonce has been changed on the host."""
    from proof_words import ProofWords

    shape, kw = [[9] * 6, [10] * 2], dict(pow_bits=6, log_blowup=1, n_queries=12)
    words = ctx.pcs_prove_host(_trees(shape, 4300), **kw)
    assert oracle.pcs_verify(words, shape, **kw) == (0, 0, -1)
    pw = ProofWords(words, [len(t) for t in shape])
    assert oracle.pcs_verify(pw.flip(pw.queried[0]["at"] + 1), shape, **kw) == (21, 5, 0)
    assert oracle.pcs_verify(pw.flip(pw.fri_layers[0]["witness_at"]), shape, **kw) == (12, 5, -1)
    assert oracle.pcs_verify(pw.flip(pw.pow_at, 4), shape, **kw)[0] == 20


def test_pcs_device_columns_and_phases(ctx, oracle):
    trees = _trees([[11] * 6], 4100)
    want = oracle.pcs_prove(trees, pow_bits=4, log_blowup=2, n_queries=10)
    bufs = [ctx.upload(c) for c in trees[0]]
    got, phases = ctx.pcs_prove_device([[b.ptr for b in bufs]], [11] * 6, pow_bits=4, log_blowup=2, n_queries=10, phases=True)
    assert (got == want).all()
    assert set(phases) == {"interpolate", "extend", "merkle", "sample", "quotients", "fri_commit", "grind", "decommit"}
    assert all(v >= 0 for v in phases.values()) and phases["merkle"] > 0


def test_pcs_rejects_a_last_tree_that_is_not_the_tallest(ctx, zkb):
    """Every column is lifted to the height of the last tree (nitroo/crates/stwo/src/prover/pcs/mod.rs:180, :232): a taller
    column in an earlier tree is refused (the reference's subtraction would overflow and panic)."""
    trees = _trees([[7, 5], [6]], 4200)
    with pytest.raises(zkb.ZkbError):
        ctx.pcs_prove_host(trees, pow_bits=0, log_blowup=1, n_queries=3)


def test_pcs_rejects_too_large_domain(ctx, zkb):
    with pytest.raises(zkb.ZkbError):
        ctx.pcs_prove_host([[np.zeros(1 << 10, np.uint32)]], log_blowup=16)


def _instance(kind, log_n, seed):
    n = 1 << log_n
    den = qm31_array(seed, n, nonzero=True)
    num = qm31_array(seed + 1, n) if kind == 1 else m31_column(seed + 1, n) if kind == 2 else None
    return kind, num, den


@pytest.mark.parametrize(
    "spec",
    [
        [(2, 6)],
        [(3, 1)],
        [(0, 5)],
        [(1, 4)],
        [(2, 10), (3, 7), (0, 8), (1, 3)],      # mixed kinds and sizes in one batch
        [(3, 12), (3, 12), (2, 12)],
        [(2, 16)],
        # more than 16 instances: the batch path, one launch per sum-check round for all instances (csrc/gkr_batch.cu)
        [(3, 9)] * 6 + [(3, 7)] * 5 + [(1, 8)] * 3 + [(2, 6), (0, 5), (3, 2), (2, 2), (1, 1), (3, 1), (0, 2), (0, 1)],
        [(3, 13)] * 20 + [(3, 11)] * 12 + [(2, 12), (1, 10)],
    ],
)
def test_gkr_proof_matches_oracle(ctx, oracle, spec):
    insts = [_instance(k, lg, 5000 + 10 * i) for i, (k, lg) in enumerate(spec)]
    want = oracle.gkr_prove(insts, 0x5EED0004, verify=True)
    keep, dev = [], []
    for kind, num, den in insts:
        nb = ctx.upload(num) if num is not None else None
        db = ctx.upload(den)
        keep += [nb, db]
        dev.append((kind, nb.ptr if nb else 0, db.ptr, den.shape[0]))
    got = ctx.gkr_prove_device(dev, 0x5EED0004)
    assert len(got) == len(want)
    assert (got == want).all()
    # inputs are not modified
    assert (keep[1].download(shape=(-1, 4)) == insts[0][2]).all()


_WIDE_BATCH = [(3, 13)] * 20 + [(3, 11)] * 12 + [(2, 12), (1, 10)]
_MIXED_BATCH = [(3, 9)] * 6 + [(3, 7)] * 5 + [(1, 8)] * 3 + [(2, 6), (0, 5), (3, 2), (2, 2), (1, 1), (3, 1), (0, 2), (0, 1)]


@pytest.mark.parametrize("driver,spec", [("resident", [(2, 10), (3, 7), (0, 8), (1, 3)]), ("resident", [(3, 12), (3, 12), (2, 12)]),
                                         ("batch", [(2, 11)]), ("batch", [(1, 6), (0, 6)]),
                                         # the batch driver's three ways through a layer's rounds: the transcript on the host and a
                                         # round trip per round; on the device with a launch per round; on the device with the small
                                         # rounds in one launch (the default, which the cases of the test above take)
                                         ("batch:host", _WIDE_BATCH), ("batch:host", _MIXED_BATCH),
                                         ("batch:launches", _WIDE_BATCH), ("batch:launches", _MIXED_BATCH), ("batch:launches", [(2, 11)]),
                                         ("batch", [(0, 15), (1, 14), (2, 15)])])
def test_gkr_drivers_give_the_same_proof(ctx, oracle, monkeypatch, driver, spec):
    """The library picks the device-resident transcript for one or two instances and the batched rounds otherwise;
    ZKB_GKR_DRIVER forces either, and both must reproduce the oracle's proof for any batch they accept."""
    driver, _, rounds = driver.partition(":")
    monkeypatch.setenv("ZKB_GKR_DRIVER", driver)
    if rounds:
        monkeypatch.setenv("ZKB_GKR_ROUNDS", rounds)
    insts = [_instance(k, lg, 5200 + 10 * i) for i, (k, lg) in enumerate(spec)]
    want = oracle.gkr_prove(insts, 0x5EED0004, verify=True)
    keep, dev = [], []
    for kind, num, den in insts:
        nb = ctx.upload(num) if num is not None else None
        db = ctx.upload(den)
        keep += [nb, db]
        dev.append((kind, nb.ptr if nb else 0, db.ptr, den.shape[0]))
    got = ctx.gkr_prove_device(dev, 0x5EED0004)
    assert len(got) == len(want) and (got == want).all()


@pytest.mark.parametrize("rounds", ["", "launches", "host"])
@pytest.mark.parametrize("spec", [[(1, 6)] * 3, [(1, 4), (0, 6), (1, 5), (0, 3)], [(1, 3)] * 20 + [(0, 7)], [(1, 12), (1, 12), (0, 12)]])
def test_gkr_batch_with_round_polynomials_of_low_degree(ctx, oracle, monkeypatch, rounds, spec):
    """Constant layers (numerators 0, denominators 1; a grand product of ones) give round polynomials whose leading coefficients
    vanish. The batch's combination then keeps the length of its longest trimmed term (lookups/utils.rs:165-170 under
    sumcheck.rs:139-149), which the proof shows as shorter polynomials: the three ways through a layer's rounds must all
    reproduce the oracle's words."""
    if rounds:
        monkeypatch.setenv("ZKB_GKR_ROUNDS", rounds)
    insts = []
    for kind, lg in spec:
        n = 1 << lg
        den = np.zeros((n, 4), np.uint32)
        den[:, 0] = 1
        insts.append((kind, np.zeros((n, 4), np.uint32) if kind == 1 else None, den))
    want = oracle.gkr_prove(insts, 0x5EED0014, verify=True)
    keep, dev = [], []
    for kind, num, den in insts:
        nb = ctx.upload(num) if num is not None else None
        db = ctx.upload(den)
        keep += [nb, db]
        dev.append((kind, nb.ptr if nb else 0, db.ptr, den.shape[0]))
    got = ctx.gkr_prove_device(dev, 0x5EED0014)
    assert len(got) == len(want) and (got == want).all()


def test_two_contexts_on_two_threads_prove_side_by_side(zkb, oracle):
    """Several contexts may be used from different host threads at once (one thread per context): two threads, each with
    its own context, prove a PCS opening over many short columns and a GKR batch of 20 instances three times over while the
    other does the same; every proof must equal the one a single thread produced. (The decommitment's gather buffer is
    per thread, the staging ring, scratch and stream per context.)"""
    import threading

    shape = [[6] * 40 + [4] * 70, [5] * 30, [8] * 8]
    trees = [_trees(shape, 4300), _trees(shape, 4400)]
    specs = [[(3, 8)] * 12 + [(1, 6)] * 5 + [(2, 7)] * 3, [(3, 9)] * 10 + [(0, 6)] * 6 + [(2, 5)] * 4]
    kw = dict(pow_bits=0, log_blowup=1, n_queries=20)
    want_pcs = [oracle.pcs_prove(t, **kw) for t in trees]
    want_gkr = []
    insts = []
    for k, spec in enumerate(specs):
        ins = [_instance(kd, lg, 5400 + 100 * k + 10 * i) for i, (kd, lg) in enumerate(spec)]
        insts.append(ins)
        want_gkr.append(oracle.gkr_prove(ins, 0x5EED0004 + k, verify=False))
    errors = []

    def worker(k):
        try:
            c = zkb.Context(device=0, max_log_size=12)
            keep, dev = [], []
            for kind, num, den in insts[k]:
                nb = c.upload(num) if num is not None else None
                db = c.upload(den)
                keep += [nb, db]
                dev.append((kind, nb.ptr if nb else 0, db.ptr, den.shape[0]))
            for _ in range(3):
                got = c.pcs_prove_host(trees[k], **kw)
                assert len(got) == len(want_pcs[k]) and (got == want_pcs[k]).all()
                gg = c.gkr_prove_device(dev, 0x5EED0004 + k)
                assert len(gg) == len(want_gkr[k]) and (gg == want_gkr[k]).all()
            c.close()
        except BaseException as e:  # reported by the main thread
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
