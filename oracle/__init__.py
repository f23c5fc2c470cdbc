"""TEST INFRASTRUCTURE ONLY: ctypes bindings over the CPU oracle (oracle/capi.cpp).

Only tests/, __graft_entry__.smoke() and bench.py's baseline legs may import this package.
The product package never does.

Pinning: the restatement is checked against the reference's own known-answer vectors (tests/test_oracle_kats.py)
and, operator by operator on a GPU, against the reference's own CUDA backend compiled out of tree
(oracle/Makefile.ref_cuda, oracle/ref_cuda.py, tests/test_gpu_reference_cuda.py). The protocol layer above the
operators has no reference output to compare with here (the reference's provers are Rust): parity of that layer
is unpinned, except where the protocol checks itself - a whole proof of a component (stark.hpp) must pass the
prover's own out-of-domain check, which ties the constraint evaluation, the composition polynomial, the mask points
and the sampled values together.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libzkoracle.so")

P = 2**31 - 1


def build(force=False):
    """Compile the oracle with the Makefile beside this file."""
    if force or not os.path.exists(_SO) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_SO)
        for f in os.listdir(_HERE) if f.endswith((".hpp", ".cpp"))
    ):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.zko_m31_mul.restype = C.c_uint32
        _lib.zko_m31_inv.restype = C.c_uint32
        _lib.zko_m31_reduce64.restype = C.c_uint32
        _lib.zko_m31_reduce64.argtypes = [C.c_uint64]
        _lib.zko_channel_new.restype = C.c_void_p
        _lib.zko_channel_grind.restype = C.c_uint64
        _lib.zko_channel_verify_pow.restype = C.c_int
        _lib.zko_num_threads.restype = C.c_int
    return _lib


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _pp(arrs):
    """Array of pointers to the rows of a list of contiguous uint32 arrays."""
    return (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


def num_threads():
    return lib().zko_num_threads()


def set_num_threads(n):
    """OpenMP threads of the heavy loops (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().zko_set_num_threads(C.c_int(n))


# ---------------------------------------------------------------- fields
def m31_mul(a, b):
    return lib().zko_m31_mul(C.c_uint32(a), C.c_uint32(b))


def m31_inv(a):
    return lib().zko_m31_inv(C.c_uint32(a))


def m31_reduce64(a):
    return lib().zko_m31_reduce64(a)


def cm31_mul(a, b):
    a, b, o = _u32(a), _u32(b), np.zeros(2, np.uint32)
    lib().zko_cm31_mul(_p(a), _p(b), _p(o))
    return o


def cm31_inv(a):
    a, o = _u32(a), np.zeros(2, np.uint32)
    lib().zko_cm31_inv(_p(a), _p(o))
    return o


def qm31_mul(a, b):
    a, b, o = _u32(a), _u32(b), np.zeros(4, np.uint32)
    lib().zko_qm31_mul(_p(a), _p(b), _p(o))
    return o


def qm31_inv(a):
    a, o = _u32(a), np.zeros(4, np.uint32)
    lib().zko_qm31_inv(_p(a), _p(o))
    return o


# ---------------------------------------------------------------- circle
def circle_point(index):
    o = np.zeros(2, np.uint32)
    lib().zko_circle_point(C.c_uint64(index), _p(o))
    return o


def secure_circle_mul(scalar):
    o = np.zeros(8, np.uint32)
    lib().zko_secure_circle_mul(C.c_uint64(scalar & (2**64 - 1)), C.c_uint64(scalar >> 64), _p(o))
    return o


def domain_at(log_size, i):
    o = np.zeros(2, np.uint32)
    lib().zko_domain_at(C.c_uint32(log_size), C.c_uint64(i), _p(o))
    return o


def twiddles(log_size):
    """(twiddles, itwiddles) of the tower rooted at Coset::half_odds(log_size)."""
    tw = np.zeros(1 << log_size, np.uint32)
    itw = np.zeros(1 << log_size, np.uint32)
    lib().zko_twiddles(C.c_uint32(log_size), _p(tw), _p(itw))
    return tw, itw


def line_twiddles_slices(domain_log_size, buf):
    buf = _u32(buf)
    k = domain_log_size - 1
    offs = np.zeros(k, np.uint64)
    lens = np.zeros(k, np.uint64)
    lib().zko_line_twiddles_slices(C.c_uint32(domain_log_size), _p(buf), C.c_size_t(len(buf)), _p(offs), _p(lens))
    return [buf[int(o):int(o) + int(n)] for o, n in zip(offs, lens)]


# ---------------------------------------------------------------- circle FFT
def interpolate_cols(cols, log_n):
    """cols: [ncols, 2^log_n] uint32, evaluations in bit-reversed order -> coefficients."""
    out = [np.array(c, dtype=np.uint32, copy=True) for c in cols]
    lib().zko_interpolate_cols(_pp(out), C.c_int(len(out)), C.c_uint32(log_n))
    return np.stack(out) if out else np.zeros((0, 1 << log_n), np.uint32)


def evaluate_cols(coeffs, log_n, log_out):
    ins = [_u32(c) for c in coeffs]
    outs = [np.zeros(1 << log_out, np.uint32) for _ in ins]
    lib().zko_evaluate_cols(_pp(ins), C.c_int(len(ins)), C.c_uint32(log_n), _pp(outs), C.c_uint32(log_out))
    return np.stack(outs) if outs else np.zeros((0, 1 << log_out), np.uint32)


def eval_at_point(coeffs, point8):
    coeffs, point8, o = _u32(coeffs), _u32(point8), np.zeros(4, np.uint32)
    log_n = int(len(coeffs)).bit_length() - 1
    lib().zko_eval_at_point(_p(coeffs), C.c_uint32(log_n), _p(point8), _p(o))
    return o


def barycentric_weights(log_n, point8):
    """cpu/circle.rs:101-132: [2^log_n][4] weights for the canonic domain and the point (x[4], y[4])."""
    o = np.zeros((1 << log_n, 4), np.uint32)
    lib().zko_barycentric_weights(C.c_uint32(log_n), _p(_u32(point8)), _p(o))
    return o


def barycentric_eval_at_point(evals, weights):
    e, w, o = _u32(evals), _u32(weights), np.zeros(4, np.uint32)
    lib().zko_barycentric_eval(_p(e), _p(w), C.c_uint32(int(len(e)).bit_length() - 1), _p(o))
    return o


def eval_at_point_by_folding(evals, point8):
    e, o = _u32(evals), np.zeros(4, np.uint32)
    lib().zko_eval_by_folding(_p(e), C.c_uint32(int(len(e)).bit_length() - 1), _p(_u32(point8)), _p(o))
    return o


def bit_reverse(v):
    v = np.array(v, dtype=np.uint32, copy=True)
    lib().zko_bit_reverse_u32(_p(v), C.c_uint32(int(len(v)).bit_length() - 1))
    return v


# ---------------------------------------------------------------- hashing
def blake2s(data: bytes, m31=False):
    o = np.zeros(32, np.uint8)
    lib().zko_blake2s(C.c_char_p(data), C.c_size_t(len(data)), C.c_int(int(m31)), _p(o))
    return o.tobytes()


def commit_on_layer(log_size, prev, cols, m31=True):
    """prev: [2^(log_size+1), 8] uint32 or None; cols: list of uint32 arrays of 2^log_size.
    Returns [2^log_size, 8] uint32 (the 32 digest bytes as little-endian words)."""
    cs = [_u32(c) for c in cols]
    out = np.zeros((1 << log_size, 8), np.uint32)
    pv = None if prev is None else _u32(prev)
    lib().zko_commit_on_layer(C.c_uint32(log_size), None if pv is None else _p(pv), _pp(cs), C.c_int(len(cs)),
                              C.c_int(int(m31)), _p(out))
    return out


class Channel:
    def __init__(self, m31=True):
        self._h = C.c_void_p(lib().zko_channel_new(C.c_int(int(m31))))

    def __del__(self):
        try:
            lib().zko_channel_free(self._h)
        except Exception:
            pass

    def digest(self):
        o = np.zeros(32, np.uint8)
        lib().zko_channel_digest(self._h, _p(o))
        return o.tobytes()

    def mix_u32s(self, data):
        d = _u32(data)
        lib().zko_channel_mix_u32s(self._h, _p(d), C.c_size_t(len(d)))

    def mix_u64(self, v):
        lib().zko_channel_mix_u64(self._h, C.c_uint64(v))

    def mix_felts(self, felts):
        f = _u32(felts).reshape(-1, 4)
        lib().zko_channel_mix_felts(self._h, _p(f), C.c_size_t(f.shape[0]))

    def mix_root(self, root_words):
        r = _u32(root_words)
        lib().zko_channel_mix_root(self._h, _p(r))

    def draw_u32s(self):
        o = np.zeros(8, np.uint32)
        lib().zko_channel_draw_u32s(self._h, _p(o))
        return o

    def draw_secure_felt(self):
        o = np.zeros(4, np.uint32)
        lib().zko_channel_draw_secure_felt(self._h, _p(o))
        return o

    def draw_secure_felts(self, n):
        o = np.zeros((n, 4), np.uint32)
        lib().zko_channel_draw_secure_felts(self._h, C.c_size_t(n), _p(o))
        return o

    def grind(self, pow_bits):
        return lib().zko_channel_grind(self._h, C.c_uint32(pow_bits))

    def verify_pow_nonce(self, pow_bits, nonce):
        return bool(lib().zko_channel_verify_pow(self._h, C.c_uint32(pow_bits), C.c_uint64(nonce)))

    def draw_queries(self, log_domain_size, n):
        o = np.zeros(n, np.uint64)
        lib().zko_draw_queries(self._h, C.c_uint32(log_domain_size), C.c_size_t(n), _p(o))
        return o


# ---------------------------------------------------------------- FRI
def fold_line(cols4, alpha):
    """cols4: [4, n] uint32 -> [4, n/2]."""
    ins = [_u32(c) for c in cols4]
    n = len(ins[0])
    outs = [np.zeros(n // 2, np.uint32) for _ in range(4)]
    a = _u32(alpha)
    lib().zko_fold_line(_pp(ins), C.c_uint32(n.bit_length() - 1), _p(a), _pp(outs))
    return np.stack(outs)


def fold_circle_into_line(dst4, src4, alpha):
    d = [np.array(c, dtype=np.uint32, copy=True) for c in dst4]
    s = [_u32(c) for c in src4]
    a = _u32(alpha)
    lib().zko_fold_circle_into_line(_pp(d), _pp(s), C.c_uint32(len(s[0]).bit_length() - 1), _p(a))
    return np.stack(d)


# ---------------------------------------------------------------- quotients
def quot_numerators(cols, point8, col_idx, values, rands):
    cs = [_u32(c) for c in cols]
    n = len(cs[0])
    outs = [np.zeros(n, np.uint32) for _ in range(4)]
    first = np.zeros(4, np.uint32)
    ci, va, ra, pt = _u32(col_idx), _u32(values).reshape(-1, 4), _u32(rands).reshape(-1, 4), _u32(point8)
    lib().zko_quot_numerators(_pp(cs), C.c_int(len(cs)), C.c_uint32(n.bit_length() - 1), _p(pt), C.c_int(len(ci)),
                              _p(ci), _p(va), _p(ra), _pp(outs), _p(first))
    return np.stack(outs), first


def line_coeffs(point8, value4, alpha4):
    o = np.zeros(12, np.uint32)
    a, b, c = _u32(point8), _u32(value4), _u32(alpha4)
    lib().zko_line_coeffs(_p(a), _p(b), _p(c), _p(o))
    return o.reshape(3, 4)


def quot_combine(accs, first_lin, points, lifting_log):
    """accs: list of [4, 2^k] arrays; first_lin: [n,4]; points: [n,8]."""
    flat = [_u32(a[c]) for a in accs for c in range(4)]
    logs = _u32([len(a[0]).bit_length() - 1 for a in accs])
    fl, pts = _u32(first_lin).reshape(-1, 4), _u32(points).reshape(-1, 8)
    outs = [np.zeros(1 << lifting_log, np.uint32) for _ in range(4)]
    lib().zko_quot_combine(C.c_int(len(accs)), _pp(flat), _p(logs), _p(fl), _p(pts), C.c_uint32(lifting_log), _pp(outs))
    return np.stack(outs)


def accumulate(col4, other4):
    a = [np.array(c, dtype=np.uint32, copy=True) for c in col4]
    b = [_u32(c) for c in other4]
    lib().zko_accumulate(_pp(a), _pp(b), C.c_size_t(len(a[0])))
    return np.stack(a)


def lift_and_accumulate(cols):
    flat = [_u32(a[c]) for a in cols for c in range(4)]
    logs = _u32([len(a[0]).bit_length() - 1 for a in cols])
    outs = [np.zeros(len(cols[-1][0]), np.uint32) for _ in range(4)]
    lib().zko_lift_and_accumulate(C.c_int(len(cols)), _pp(flat), _p(logs), _pp(outs))
    return np.stack(outs)


def secure_powers(felt4, n):
    o = np.zeros((n, 4), np.uint32)
    f = _u32(felt4)
    lib().zko_secure_powers(_p(f), C.c_size_t(n), _p(o))
    return o


# ---------------------------------------------------------------- GKR
GRAND_PRODUCT, LOGUP_GENERIC, LOGUP_MULTIPLICITIES, LOGUP_SINGLES = 0, 1, 2, 3


def gkr_eq_evals(y, v4):
    y = _u32(y).reshape(-1, 4)
    o = np.zeros((1 << y.shape[0], 4), np.uint32)
    v = _u32(v4)
    lib().zko_gkr_eq_evals(_p(y), C.c_size_t(y.shape[0]), _p(v), _p(o))
    return o


def gkr_next_layer(kind, num, den):
    den = _u32(den)
    n = den.shape[0]
    num = None if num is None else _u32(num)
    no, do = np.zeros((n // 2, 4), np.uint32), np.zeros((n // 2, 4), np.uint32)
    lib().zko_gkr_next_layer(C.c_int(kind), None if num is None else _p(num), _p(den), C.c_size_t(n), _p(no), _p(do))
    return (None if kind == GRAND_PRODUCT else no), do


def gkr_round_sums(kind, num, den, eq_evals, lam):
    den = _u32(den)
    n = den.shape[0]
    num = None if num is None else _u32(num)
    e, l, o = _u32(eq_evals), _u32(lam), np.zeros(8, np.uint32)
    lib().zko_gkr_round_sums(C.c_int(kind), None if num is None else _p(num), _p(den), C.c_size_t(n), _p(e), _p(l), _p(o))
    return o.reshape(2, 4)


def mle_fix_first(mle, r4):
    mle = _u32(mle)
    r = _u32(r4)
    n = mle.shape[0]
    o = np.zeros((n // 2, 4), np.uint32)
    if mle.ndim == 1:
        lib().zko_mle_fix_first_m31(_p(mle), C.c_size_t(n), _p(r), _p(o))
    else:
        lib().zko_mle_fix_first_qm31(_p(mle), C.c_size_t(n), _p(r), _p(o))
    return o


# ---------------------------------------------------------------- whole protocols
def pow_prefixed_digest(channel, pow_bits):
    o = np.zeros(8, np.uint32)
    lib().zko_channel_pow_prefixed_digest(channel._h, C.c_uint32(pow_bits), _p(o))
    return o


def pcs_prove(trees, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3, two_sample_every=0, cap=1 << 24):
    """trees: list of lists of uint32 columns (trace evaluations, bit-reversed). Returns the proof words."""
    flat = [_u32(c) for t in trees for c in t]
    ncols = np.array([len(t) for t in trees], np.int32)
    logs = _u32([len(c).bit_length() - 1 for c in flat])
    out = np.zeros(cap, np.uint32)
    lib().zko_pcs_prove.restype = C.c_long
    n = lib().zko_pcs_prove(C.c_int(len(trees)), _p(ncols), _pp(flat), _p(logs), C.c_uint32(pow_bits), C.c_uint32(log_blowup),
                            C.c_uint32(log_last_layer), C.c_uint32(n_queries), C.c_int(two_sample_every), _p(out), C.c_size_t(cap))
    if n < 0:
        raise RuntimeError(f"zko_pcs_prove failed: {n}")
    return out[:n].copy()


def set_simd(on=True):
    """Packed (16-lane) restatement of the reference's SIMD backend for the FFTs, leaf hashing, out-of-domain evaluation and
    quotient numerators, on or off for every later call. Returns the lanes in use (16: AVX-512, 8: AVX2, 0: scalar)."""
    lib().zko_set_simd.restype = C.c_int
    return int(lib().zko_set_simd(C.c_int(1 if on else 0)))


VERIFY_ERRORS = {0: "ok", 1: "merkle: witness too short", 2: "merkle: witness too long", 3: "merkle: too many queried values",
                 4: "merkle: too few queried values", 5: "merkle: root mismatch", 10: "fri: invalid number of layers",
                 11: "fri: first layer evaluations invalid", 12: "fri: first layer commitment invalid",
                 13: "fri: inner layer commitment invalid", 14: "fri: inner layer evaluations invalid",
                 15: "fri: last layer degree invalid", 16: "fri: last layer evaluations invalid", 20: "proof of work",
                 21: "trace decommitment invalid", 30: "malformed word stream", 31: "channel digest after the proof differs"}


def pcs_verify(words, tree_logs, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3, two_sample_every=0):
    """The reference's verifier (CommitmentSchemeVerifier::verify_values + FriVerifier + MerkleVerifier) on proof words as
    zko_pcs_prove / zkb_pcs_prove_* write them (the 8 channel-digest words at the end included). tree_logs: per tree, the
    TRACE log size of every column. Returns (code, nested merkle code, layer or tree index); code 0 = accepts."""
    w = _u32(words)
    ncols = np.array([len(t) for t in tree_logs], np.int32)
    logs = _u32([l for t in tree_logs for l in t])
    info = np.zeros(2, np.int32)
    lib().zko_pcs_verify.restype = C.c_int
    rc = lib().zko_pcs_verify(_p(w), C.c_size_t(len(w)), C.c_int(len(tree_logs)), _p(ncols), _p(logs), C.c_uint32(pow_bits),
                              C.c_uint32(log_blowup), C.c_uint32(log_last_layer), C.c_uint32(n_queries), C.c_int(two_sample_every), _p(info))
    return int(rc), int(info[0]), int(info[1])


def gkr_prove(instances, seed, verify=True, cap=1 << 22):
    """instances: list of (kind, num or None, den). Returns the proof words (rejects raise)."""
    kinds = np.array([k for k, _, _ in instances], np.int32)
    nums = [None if n is None else _u32(n) for _, n, _ in instances]
    dens = [_u32(d) for _, _, d in instances]
    ns = np.array([d.shape[0] for d in dens], np.uint64)
    nump = (C.c_void_p * len(nums))(*[None if n is None else n.ctypes.data for n in nums])
    out = np.zeros(cap, np.uint32)
    lib().zko_gkr_prove.restype = C.c_long
    n = lib().zko_gkr_prove(C.c_int(len(instances)), _p(kinds), nump, _pp(dens), _p(ns), C.c_uint64(seed), C.c_int(int(verify)),
                            _p(out), C.c_size_t(cap))
    if n == -2:
        raise AssertionError("GKR proof rejected by partially_verify_batch")
    if n < 0:
        raise RuntimeError(f"zko_gkr_prove failed: {n}")
    return out[:n].copy()


# ---------------------------------------------------------------- Freivalds component
def coset_perm(i, log_n):
    lib().zko_coset_perm.restype = C.c_uint64
    return lib().zko_coset_perm(C.c_uint64(i), C.c_uint32(log_n))


def freivalds_columns(qx, qws, grid, pq, pk, table_len=256):
    """qx: int8 [tokens, n_in]; qws: list of int8 [n_in, n_out_m]; grid = (log_rows, groups, chunks, lead).
    Returns (base [pq, rows], pre [n_mats*pk+4, rows], m_r8 [table_len], off_table)."""
    qx = np.ascontiguousarray(qx, np.int8)
    qws = [np.ascontiguousarray(w, np.int8) for w in qws]
    tokens, n_in = qx.shape
    n_out = _u32([w.shape[1] for w in qws])
    log_rows, groups, chunks, lead = grid
    rows = 1 << log_rows
    base = [np.zeros(rows, np.uint32) for _ in range(pq)]
    pre = [np.zeros(rows, np.uint32) for _ in range(len(qws) * pk + 4)]
    m_r8 = np.zeros(table_len, np.uint32)
    off = C.c_uint64()
    lib().zko_freivalds_columns(_p(qx), _pp(qws), _p(n_out), C.c_uint32(len(qws)), C.c_uint32(log_rows), C.c_uint32(groups),
                                C.c_uint32(chunks), C.c_uint32(lead), C.c_uint32(pq), C.c_uint32(pk), C.c_uint32(n_in),
                                C.c_uint32(tokens), _pp(base), _pp(pre), _p(m_r8), C.c_uint32(table_len), C.byref(off))
    return np.stack(base), np.stack(pre), m_r8, off.value


def freivalds_acc(base, pre, n_mats, grid, pq, pk, s4, rv4):
    """Returns (columns [(1+2 n_mats)*4, rows] in committed order, claims [n_mats, 4])."""
    b = [_u32(c) for c in base]
    p = [_u32(c) for c in pre[:n_mats * pk]]
    log_rows, groups, chunks, lead = grid
    rows = 1 << log_rows
    out = [np.zeros(rows, np.uint32) for _ in range((1 + 2 * n_mats) * 4)]
    claims = np.zeros((n_mats, 4), np.uint32)
    s, r = _u32(s4), _u32(rv4)
    lib().zko_freivalds_acc(_pp(b), _pp(p), C.c_uint32(n_mats), C.c_uint32(log_rows), C.c_uint32(groups), C.c_uint32(chunks),
                            C.c_uint32(lead), C.c_uint32(pq), C.c_uint32(pk), _p(s), _p(r), _pp(out), _p(claims))
    return np.stack(out), claims


# ---- witness generation: tables, dequantize (oracle/witness.hpp)
DEQUANT_CFG_FIELDS = ("variant", "sticky", "kmax", "do_ref", "tokens", "n_out", "per_row", "chunks", "log_rows", "slot0", "per_slot", "chan_w",
                      "f_acc", "f_sg", "f_m2", "f_ph", "f_st", "f_r", "f_m7", "f_ef", "f_nz", "f_eo", "f_mul0", "f_mul1", "f_mul2", "f_mul3",
                      "f_mul4", "f_mul5", "sh0", "sh1", "n_norm", "n_frac", "n_mul", "n_r8")


def witness_tables(expmap, counters, log_rows, bf16x, two_pow, patch_idx=(), patch_val=()):
    """Returns (x, y, m) columns of 2^log_rows words in committed order."""
    expmap = _u32(expmap)
    counters = [_u32(c) for c in counters]
    pi, pv = _u32(list(patch_idx)), _u32(list(patch_val))
    rows = 1 << log_rows
    x, y, m = (np.zeros(rows, np.uint32) for _ in range(3))
    lib().zko_witness_tables(_p(expmap), _pp(counters), C.c_uint32(len(counters)), _p(pi), _p(pv), C.c_uint32(len(pi)), C.c_uint32(log_rows),
                             C.c_int(int(bf16x)), C.c_double(two_pow), _p(x), _p(y), _p(m))
    return x, y, m


def witness_dequant(acc, jx, jw, sx, sw, norm3, mul2, n_base, n_pre, cfg):
    """cfg: dict over DEQUANT_CFG_FIELDS. Returns dict(base [n_base, rows], pre [n_pre, rows], m_norm, m_frac, m_mul, m_r8, counts [3],
    want [rows * per_row]); columns in committed order."""
    c34 = _u32([cfg[k] for k in DEQUANT_CFG_FIELDS])
    rows = 1 << cfg["log_rows"]
    acc = np.ascontiguousarray(acc, np.int32)
    jx, jw = np.ascontiguousarray(jx, np.int32), np.ascontiguousarray(jw, np.int32)
    sx, sw, norm3, mul2 = _u32(sx), _u32(sw), _u32(norm3), _u32(mul2)
    base = [np.zeros(rows, np.uint32) for _ in range(n_base)]
    pre = [np.zeros(rows, np.uint32) for _ in range(n_pre)]
    m_norm, m_frac = np.zeros(cfg["n_norm"], np.uint32), np.zeros(cfg["n_frac"], np.uint32)
    m_mul, m_r8 = np.zeros(max(1, cfg["n_mul"]), np.uint32), np.zeros(cfg["n_r8"], np.uint32)
    counts, want = np.zeros(3, np.uint32), np.zeros(rows * cfg["per_row"], np.uint32)
    lib().zko_witness_dequant(_p(acc), _p(jx), _p(jw), _p(sx), _p(sw), _p(norm3), _p(mul2), _pp(base), C.c_uint32(n_base), _pp(pre),
                              C.c_uint32(n_pre), _p(m_norm), _p(m_frac), _p(m_mul), _p(m_r8), _p(counts), _p(want), _p(c34))
    return {"base": np.stack(base), "pre": np.stack(pre), "m_norm": m_norm, "m_frac": m_frac, "m_mul": m_mul[:cfg["n_mul"]], "m_r8": m_r8,
            "counts": counts, "want": want}


# ---- witness generation: shared bf16 tables, key tile selectors, residual stream (oracle/witness_pre.hpp)
PRE_TABLE_COLS = {0: 6, 1: 3, 2: 4, 3: 2, 4: 1}


def witness_pre_table(kind, log_rows, kmax, round_mode, counters=(), patch_idx=(), patch_val=(), with_m=True):
    """Returns (cols [n_cols, rows], m or None) in committed order. patch_val: n_patch x n_cols."""
    rows, n_cols = 1 << log_rows, PRE_TABLE_COLS[kind]
    counters = [_u32(c) for c in counters]
    pi, pv = _u32(list(patch_idx)), _u32(np.asarray(patch_val, np.uint32).reshape(-1))
    cols = [np.zeros(rows, np.uint32) for _ in range(n_cols)]
    m = np.zeros(rows, np.uint32) if with_m else None
    lib().zko_witness_pre_table(C.c_uint32(kind), C.c_uint32(log_rows), C.c_uint32(kmax), C.c_uint32(round_mode), _pp(counters),
                                C.c_uint32(len(counters)), _p(pi), _p(pv), C.c_uint32(len(pi)), _pp(cols), _p(m) if with_m else None)
    return np.stack(cols), m


def key_tile_flags(shape, log_rows, groups, chunks, lead, descending, modulus, rw):
    flags = np.zeros(1 << log_rows, np.uint32)
    lib().zko_key_tile_flags(*(C.c_uint32(int(v)) for v in (shape, log_rows, groups, chunks, lead, descending, modulus, rw)), _p(flags))
    return flags


def witness_selectors(shape, log_rows, groups, chunks, lead, descending, flags, scale, ctx_len, with_scale, n_cols):
    flags, scale = _u32(flags), _u32(scale)
    cols = [np.zeros(1 << log_rows, np.uint32) for _ in range(n_cols)]
    lib().zko_witness_selectors(*(C.c_uint32(int(v)) for v in (shape, log_rows, groups, chunks, lead, descending)), _p(flags), _p(scale),
                                C.c_uint32(ctx_len), C.c_int(int(with_scale)), _pp(cols), C.c_uint32(n_cols))
    return np.stack(cols)


def rs_n_cols(groups, n_slots, kind, sticky):
    g = _u32(np.asarray(groups, np.uint32).reshape(-1))
    f = lib().zko_rs_n_cols
    f.restype = C.c_uint32
    return int(f(_p(g), C.c_uint32(len(groups)), C.c_uint32(n_slots), C.c_uint32(kind), C.c_uint32(int(sticky))))


def witness_residual_stream(case):
    """case: the dict zk_inference_prover_b200.witness_cases.residual_stream_case builds (the program in its host form under
    "groups", "src_slots", "out_slot"). Returns dict(cols [n_cols, rows], out_pat, out_nat, in_nat, m_pow, m_norm, m_val, m_frac,
    m_smul, m_un [n_un, n], counts [3])."""
    groups = _u32(np.asarray(case["groups"], np.uint32).reshape(-1))
    slots = _u32(np.asarray(case["src_slots"], np.uint32).reshape(-1))
    out_slot = _u32(case["out_slot"])
    n_groups, n_slots, out_w = len(case["groups"]), len(case["src_slots"]), len(case["out_slot"])
    rows, n_leaves = 1 << case["log_rows"], sum(g[0] for g in case["groups"])
    n_cols = rs_n_cols(case["groups"], n_slots, case["kind"], case["sticky"])
    norm3, smul3 = _u32(case["norm3"]), np.ascontiguousarray(case["smul3"], np.int32)
    un2 = [np.ascontiguousarray(u, np.int32) for u in case["un2"]]
    wit = _u32(case["wit"])
    m_len = np.asarray([case["m_len"][k] for k in ("pow", "norm", "val", "frac", "smul", "un")], np.uint64)
    cols = [np.zeros(rows, np.uint32) for _ in range(n_cols)]
    out_pat, out_nat = np.zeros(rows * out_w, np.uint32), np.zeros(rows * out_w * 2, np.int32)
    in_nat = np.zeros(rows * n_leaves * 2, np.int32)
    ms = [np.zeros(int(m_len[k]), np.uint32) for k in range(5)] + [np.zeros(int(m_len[5]), np.uint32) for _ in un2]
    counts = np.zeros(3, np.uint32)
    lib().zko_witness_residual_stream(_p(groups), C.c_uint32(n_groups), _p(slots), C.c_uint32(n_slots), _p(out_slot), C.c_uint32(out_w),
                                      C.c_uint32(case["kind"]), C.c_uint32(int(case["sticky"])), C.c_uint32(case["kmax"]), _p(norm3),
                                      C.c_uint32(len(norm3) // 3), _p(smul3), C.c_uint32(len(smul3) // 3), _pp(un2), C.c_uint32(len(un2)),
                                      C.c_uint32(case["n_val"]), _p(wit), C.c_uint32(case["live_rows"]), C.c_uint32(case["log_rows"]),
                                      _p(m_len), _pp(cols), _p(out_pat), _p(out_nat), _p(in_nat), _pp(ms), _p(counts))
    return {"cols": np.stack(cols), "out_pat": out_pat, "out_nat": out_nat, "in_nat": in_nat, "m_pow": ms[0], "m_norm": ms[1], "m_val": ms[2],
            "m_frac": ms[3], "m_smul": ms[4], "m_un": np.stack(ms[5:]) if un2 else np.zeros((0, int(m_len[5])), np.uint32), "counts": counts}


# ---- constraint quotients of an AIR (oracle/air.hpp)
def offset_bit_reversed_circle_domain_index(i, domain_log, eval_log, offset):
    f = lib().zko_offset_bit_reversed_circle_domain_index
    f.restype = C.c_uint64
    return int(f(C.c_uint64(i), C.c_uint32(domain_log), C.c_uint32(eval_log), C.c_int64(offset)))


def constraint_denom_inv(trace_log, eval_log):
    out = np.empty(1 << (eval_log - trace_log), np.uint32)
    lib().zko_constraint_denom_inv(C.c_uint32(trace_log), C.c_uint32(eval_log), _p(out))
    return out


def _col_ptrs(cols):
    cols = [None if c is None else _u32(c) for c in cols]
    return cols, (C.c_void_p * len(cols))(*[None if c is None else c.ctypes.data for c in cols])


def constraint_quotients_ssa(source, cols, rcp, trace_log, eval_log, accum=None, cumsum_shift=None, scalars=None):
    """The lowered program interpreted row by row. cols: flat list (trees concatenated) of 2^eval_log-word arrays.
    Returns the (4, 2^eval_log) accumulator; `accum` (same shape) is added to if given."""
    ops, cons, trees = _u32(source.ops), _u32(source.constraints), _u32(source.tree_cols)
    sc = _u32(source.scalars if scalars is None else scalars)
    keep, ptrs = _col_ptrs(cols)
    out = np.zeros((4, 1 << eval_log), np.uint32) if accum is None else _u32(accum).copy()
    acc_ptrs = (C.c_void_p * 4)(*[out[k].ctypes.data for k in range(4)])
    shift = _u32(cumsum_shift) if cumsum_shift is not None else None
    rcp = _u32(rcp)
    lib().zko_constraint_quotients_ssa(_p(ops), C.c_size_t(ops.shape[0]), _p(cons), C.c_size_t(cons.size), _p(trees), C.c_int(trees.size),
                                       ptrs, _p(sc), C.c_size_t(sc.size // 4), _p(shift) if shift is not None else None, _p(rcp),
                                       C.c_uint32(trace_log), C.c_uint32(eval_log), acc_ptrs, C.c_int(accum is not None))
    return out


def constraint_quotients_air(air, iparams, qparams, tree_cols, cols, rcp, trace_log, eval_log, accum=None, claimed_sum=None):
    """The AIR written against CpuDomainEvaluator: air 0 wide Fibonacci, 1 Plonk, 2 Freivalds (parameters as in capi.cpp)."""
    ip, qp, trees, rcp = _u32(iparams), _u32(qparams), _u32(tree_cols), _u32(rcp)
    keep, ptrs = _col_ptrs(cols)
    out = np.zeros((4, 1 << eval_log), np.uint32) if accum is None else _u32(accum).copy()
    acc_ptrs = (C.c_void_p * 4)(*[out[k].ctypes.data for k in range(4)])
    cs = _u32(claimed_sum) if claimed_sum is not None else None
    lib().zko_constraint_quotients_air(C.c_int(air), _p(ip), _p(qp), _p(trees), C.c_int(trees.size), ptrs,
                                       _p(cs) if cs is not None else None, _p(rcp), C.c_size_t(rcp.size // 4), C.c_uint32(trace_log),
                                       C.c_uint32(eval_log), acc_ptrs, C.c_int(accum is not None))
    return out


def stark_prove_multi(components, tree_cols, cols, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3, cap=1 << 24):
    """prove() for several components (oracle/stark.hpp). components: list of dicts with air, ip, qp ((n, 4) words), trace_log,
    claimed_sum (4 words or None). In every tree the columns of component k follow those of the components before it; cols is
    the flat list (trees concatenated) of the traces on their own trace domains.
    Returns (proof words incl. the channel digest, committed composition value [4], value from the constraints [4])."""
    airs = np.array([c["air"] for c in components], np.int32)
    logs = _u32([c["trace_log"] for c in components])
    ips = [_u32(c["ip"]).reshape(-1) for c in components]
    qps = [_u32(c["qp"]).reshape(-1, 4) for c in components]
    ip_off = _u32(np.cumsum([0] + [len(x) for x in ips[:-1]]))
    qp_off = _u32(np.cumsum([0] + [len(x) for x in qps[:-1]]))
    ip, qp = _u32(np.concatenate(ips)), _u32(np.concatenate(qps).reshape(-1))
    claimed = _u32(np.stack([np.zeros(4, np.uint32) if c.get("claimed_sum") is None else _u32(c["claimed_sum"]) for c in components]))
    trees = _u32(tree_cols)
    keep, ptrs = _col_ptrs(cols)
    col_logs = _u32([int(len(c)).bit_length() - 1 for c in keep])
    out = np.zeros(cap, np.uint32)
    f = lib().zko_stark_prove_multi
    f.restype = C.c_long
    n = f(C.c_int(len(components)), _p(airs), _p(logs), _p(ip), _p(ip_off), _p(qp), _p(qp_off), _p(claimed), _p(trees), C.c_int(trees.size),
          ptrs, _p(col_logs), C.c_uint32(pow_bits), C.c_uint32(log_blowup), C.c_uint32(log_last_layer), C.c_uint32(n_queries), _p(out),
          C.c_size_t(cap))
    if n < 0:
        raise RuntimeError("stark_prove: output buffer too small")
    return out[:n - 8].copy(), out[n - 8:n - 4].copy(), out[n - 4:n].copy()


def stark_prove(air, iparams, qparams, tree_cols, cols, trace_log, composition_log=None, claimed_sum=None, **kw):
    """One component (composition_log, if given, must be trace_log + 1: the only size the protocol has)."""
    assert composition_log is None or composition_log == trace_log + 1
    qp = _u32(qparams).reshape(-1, 4) if np.size(qparams) else np.zeros((1, 4), np.uint32)
    return stark_prove_multi([dict(air=air, ip=iparams, qp=qp, trace_log=trace_log, claimed_sum=claimed_sum)], tree_cols, cols, **kw)
