"""The CPU oracle against the known-answer vectors held by the reference's own tests, plus the
algebraic identities those tests check. Citations are paths inside the reference project
(STWO = nitroo/crates/stwo/src)."""
import numpy as np
import pytest

from util import P, m31_column, qm31_array


def test_blake2s_of_a(oracle):
    # STWO/core/vcs/blake2_hash.rs:134-140
    assert oracle.blake2s(b"a").hex() == "4a0d129873403037c2cd9b9048203687f6233fb6738956e0349bd4320fec3e90"


def test_blake2s_rfc7693_abc(oracle):
    # RFC 7693 appendix B
    assert oracle.blake2s(b"abc").hex() == "508c5e8c327c14e2e1a72ba34eeb452f37458b209ed63a294d999b4c86675982"


def test_blake2s_multiblock_matches_hashlib(oracle):
    import hashlib

    for n in [0, 1, 63, 64, 65, 127, 128, 129, 1024, 1025]:
        data = bytes((i * 7 + 3) & 0xFF for i in range(n))
        assert oracle.blake2s(data) == hashlib.blake2s(data).digest()


def test_channel_mix_u64(oracle):
    # STWO/core/channel/blake2s.rs:213-233
    ch = oracle.Channel(m31=False)
    ch.mix_u64(0x1111222233334444)
    d64 = ch.digest()
    ch2 = oracle.Channel(m31=False)
    ch2.mix_u32s([0x33334444, 0x11112222])
    assert d64 == ch2.digest()
    assert d64 == bytes([0xbc, 0x9e, 0x3f, 0xc1, 0xd2, 0x4e, 0x88, 0x97, 0x95, 0x6d, 0x33, 0x59, 0x32, 0x73, 0x97, 0x24,
                         0x9d, 0x6b, 0xca, 0xcd, 0x22, 0x4d, 0x92, 0x74, 0x4, 0xe7, 0xba, 0x4a, 0x77, 0xdc, 0x6e, 0xce])


def test_channel_mix_u32s(oracle):
    # STWO/core/channel/blake2s.rs:235-247
    ch = oracle.Channel(m31=False)
    ch.mix_u32s([1, 2, 3, 4, 5, 6, 7, 8, 9])
    assert ch.digest() == bytes([0x70, 0x91, 0x76, 0x83, 0x57, 0xbb, 0x1b, 0xb3, 0x34, 0x6f, 0xda, 0xb6, 0xb3, 0x57, 0xd7, 0xfa,
                                 0x46, 0xb8, 0xfb, 0xe3, 0x2c, 0x2e, 0x43, 0x24, 0xa0, 0xff, 0xc2, 0x94, 0xcb, 0xf9, 0xa1, 0xc7])


def test_channel_draw_counts(oracle):
    # STWO/core/channel/blake2s.rs:157-168: 9 secure felts take 5 hashes (2 per hash).
    ch = oracle.Channel(m31=False)
    a = ch.draw_u32s()
    b = ch.draw_u32s()
    assert (a != b).any()
    felts = oracle.Channel(m31=False).draw_secure_felts(9)
    assert len({tuple(f) for f in felts}) == 9
    assert (felts < P).all()


def test_m31_channel_digest_words_are_reduced(oracle):
    ch = oracle.Channel(m31=True)
    ch.mix_u32s(np.arange(20))
    words = np.frombuffer(ch.digest(), dtype="<u4")
    assert (words < P).all()


def test_bit_reverse_literal(oracle):
    # STWO/prover/backend/cpu/mod.rs:86-90
    assert list(oracle.bit_reverse(np.arange(8))) == [0, 4, 2, 6, 1, 5, 3, 7]


def test_domain_line_twiddles_slices(oracle):
    # STWO/core/poly/utils.rs:141-148
    s = oracle.line_twiddles_slices(4, np.arange(8))
    assert [list(x) for x in s] == [[0, 1, 2, 3], [4, 5], [6]]


def test_circle_generators(oracle):
    # STWO/core/circle.rs:202-214
    g = oracle.circle_point(1)
    assert list(g) == [2, 1268011823]
    assert (int(g[0]) ** 2 + int(g[1]) ** 2) % P == 1
    # order 2^31: 2^30 * G = (-1, 0)
    assert list(oracle.circle_point(1 << 30)) == [P - 1, 0]
    sg = oracle.secure_circle_mul(1)
    assert list(sg) == [1, 0, 478637715, 513582971, 992285211, 649143431, 740191619, 1186584352]
    # the secure generator has order p^4 - 1
    assert list(oracle.secure_circle_mul(P**4 - 1)) == [1, 0, 0, 0, 0, 0, 0, 0]


def test_field_literals(oracle):
    # STWO/core/fields/cm31.rs:99-114, qm31.rs:158-173
    assert list(oracle.cm31_mul([1, 2], [4, 5])) == [P - 6, 13]
    x = oracle.cm31_inv([1, 2])
    assert list(oracle.cm31_mul([1, 2], x)) == [1, 0]
    q0, q1 = [1, 2, 3, 4], [4, 5, 6, 7]
    assert list(oracle.qm31_mul(q0, q1)) == [P - 71, 93, P - 16, 50]
    qi = oracle.qm31_inv(q0)
    assert list(oracle.qm31_mul(q0, qi)) == [1, 0, 0, 0]
    assert oracle.m31_mul(oracle.m31_inv(19), 19) == 1
    assert oracle.m31_reduce64((P**2) - 19) == P - 19


def test_twiddle_tower_matches_points(oracle):
    tw, itw = oracle.twiddles(5)
    # first level: x of the first half of half_odds(5), bit-reversed
    init, step = 1 << (31 - 7), 1 << (31 - 5)
    xs = [int(oracle.circle_point((init + j * step) % (1 << 31))[0]) for j in range(16)]
    br = [xs[int(f"{i:04b}"[::-1], 2)] for i in range(16)]
    assert list(tw[:16]) == br
    assert tw[-1] == 1
    for a, b in zip(tw[:-1], itw[:-1]):
        assert oracle.m31_mul(int(a), int(b)) == 1


@pytest.mark.parametrize("log_n", [1, 2, 3, 4, 7, 10])
def test_interpolate_evaluate_roundtrip(oracle, log_n):
    # STWO/prover/backend/cpu/circle.rs:420-445 (interpolate then evaluate is the identity)
    vals = np.stack([m31_column(11 + c, 1 << log_n) for c in range(3)])
    coeffs = oracle.interpolate_cols(vals, log_n)
    back = oracle.evaluate_cols(coeffs, log_n, log_n)
    assert (back == vals).all()


@pytest.mark.parametrize("log_n,log_out", [(3, 4), (4, 6), (6, 7), (0, 3), (1, 5)])
def test_evaluate_agrees_with_eval_at_point(oracle, log_n, log_out):
    # STWO/prover/backend/cpu/circle.rs:365-418: an evaluation equals eval_at_point at the domain point
    coeffs = m31_column(5, 1 << log_n)
    ev = oracle.evaluate_cols([coeffs], log_n, log_out)[0]
    for i in [0, 1, 2, (1 << log_out) - 1]:
        br = int(f"{i:0{log_out}b}"[::-1], 2)
        p = oracle.domain_at(log_out, br)
        pt = [int(p[0]), 0, 0, 0, int(p[1]), 0, 0, 0]
        if log_n == 0:
            assert ev[i] == coeffs[0]
            continue
        val = oracle.eval_at_point(coeffs, pt)
        assert list(val) == [int(ev[i]), 0, 0, 0]


def test_lde_is_extension_of_small_domain(oracle):
    # the canonic domain of log 4 is contained in the one of log 6: a polynomial's values agree there
    coeffs = m31_column(77, 16)
    small = oracle.evaluate_cols([coeffs], 4, 4)[0]
    big = oracle.evaluate_cols([coeffs], 4, 6)[0]
    pts_small = {tuple(oracle.domain_at(4, int(f"{i:04b}"[::-1], 2))): int(small[i]) for i in range(16)}
    hits = 0
    for i in range(64):
        p = tuple(oracle.domain_at(6, int(f"{i:06b}"[::-1], 2)))
        if p in pts_small:
            assert pts_small[p] == int(big[i])
            hits += 1
    # CanonicCoset(4) is not a subset of CanonicCoset(6) (both are odd cosets of different
    # subgroups), so there may be no shared points; the check is only meaningful when there are.
    assert hits in (0, 16)


def test_fold_line_matches_definition(oracle):
    # STWO/core/fri.rs:702-724: f0 + alpha f1 with f(x) = f0(pi x) + x f1(pi x), on a degree-<n/2 line poly:
    # folding evaluations of a constant c gives 2c.
    n = 16
    cols = np.zeros((4, n), np.uint32)
    cols[0, :] = 5
    out = oracle.fold_line(cols, [3, 1, 4, 1])
    assert (out[0] == 10).all() and (out[1:] == 0).all()


def test_fold_circle_into_line_of_constant(oracle):
    n = 16
    src = np.zeros((4, n), np.uint32)
    src[1, :] = 7
    dst = np.zeros((4, n // 2), np.uint32)
    out = oracle.fold_circle_into_line(dst, src, [9, 8, 7, 6])
    assert (out[1] == 14).all() and (out[0] == 0).all()


def test_fri_fold_degree_halves(oracle):
    # Evaluate a polynomial of 2^3 coefficients on the domain of log 5, fold circle->line->line...;
    # after log2(8) folds the layer is constant on its domain (low-degree test identity).
    coeffs = m31_column(9, 8)
    ev = oracle.evaluate_cols([coeffs], 3, 5)[0]
    src = np.zeros((4, 32), np.uint32)
    src[0] = ev
    cur = oracle.fold_circle_into_line(np.zeros((4, 16), np.uint32), src, [2, 3, 4, 5])
    for a in ([7, 7, 7, 7], [1, 2, 3, 4]):
        cur = oracle.fold_line(cur, a)
    # 8 coefficients -> after circle fold 4, then 2, then 1: constant on 4 points
    assert (cur == cur[:, :1]).all()


def test_gkr_eq_evals_small(oracle):
    # STWO/prover/backend/cpu/lookups/gkr.rs:303-325: eq evals over the cube, bit-reversed
    y = qm31_array(3, 2)
    one = np.array([1, 0, 0, 0], np.uint32)
    ev = oracle.gkr_eq_evals(y, one)

    def sub(a, b):
        return (a.astype(np.int64) - b.astype(np.int64)) % P

    one_minus = [sub(one, y[0]), sub(one, y[1])]
    exp = [
        oracle.qm31_mul(one_minus[0], one_minus[1]),
        oracle.qm31_mul(one_minus[0], y[1]),
        oracle.qm31_mul(y[0], one_minus[1]),
        oracle.qm31_mul(y[0], y[1]),
    ]
    assert (ev == np.stack(exp)).all()


def test_grind_and_verify(oracle):
    ch = oracle.Channel(m31=True)
    ch.mix_u64(1234)
    nonce = ch.grind(10)
    assert ch.verify_pow_nonce(10, nonce)
    assert all(not ch.verify_pow_nonce(10, k) for k in range(nonce))


@pytest.mark.parametrize("spec", [[(1, 6)] * 3, [(1, 4), (0, 6), (1, 5), (0, 3)]])
def test_gkr_constant_layers_give_short_round_polynomials(oracle, spec):
    """Numerators 0 over denominators 1 and grand products of ones: every round polynomial loses its leading coefficients,
    and the batch's combination keeps the length of its longest trimmed term (lookups/utils.rs:165-170 under
    sumcheck.rs:139-149). The restated verifier (run inside gkr_prove) must accept the shorter proof, and the proof must be
    shorter than the one of random layers of the same shapes."""
    def instances(constant):
        out = []
        for i, (kind, lg) in enumerate(spec):
            n = 1 << lg
            if constant:
                den = np.zeros((n, 4), np.uint32)
                den[:, 0] = 1
                num = np.zeros((n, 4), np.uint32) if kind == 1 else None
            else:
                den = qm31_array(900 + i, n, nonzero=True)
                num = qm31_array(950 + i, n) if kind == 1 else None
            out.append((kind, num, den))
        return out
    short = oracle.gkr_prove(instances(True), 0x5EED0014, verify=True)
    full = oracle.gkr_prove(instances(False), 0x5EED0014, verify=True)
    assert 0 < len(short) < len(full)
