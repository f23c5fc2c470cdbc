"""TEST INFRASTRUCTURE ONLY: ctypes driver for the reference's own CUDA backend, compiled unmodified by
oracle/Makefile.ref_cuda into oracle/_ref/libstwo_cuda_ref.so (see that file). It is a second checker beside
the CPU oracle: the tests run the reference's kernels and this repository's kernels on the same inputs and
compare every word; bench.py times it as a same-box GPU baseline. The calls follow the reference's Rust call
sites (nitroo/crates/stwo/src/prover/backend/cuda/poly.rs:179-294, 422-576, blake2s.rs:61-118) over the
C functions declared in nitroo/crates/stwo/src/stwo_cuda/bindings.rs.

The library works on the legacy default stream and its own memory pool; every method here that returns host
data synchronises through the library's blocking copies."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libstwo_cuda_ref.so")
P = 2**31 - 1
GEN = (2, 1268011823)  # M31_CIRCLE_GEN, nitroo/crates/stwo/src/core/circle.rs:202-205


def available():
    return os.path.exists(LIB_PATH)


class _Point(C.Structure):  # stwo_cuda/cuda/point.cuh:7-10
    _fields_ = [("x", C.c_uint32), ("y", C.c_uint32)]


def _padd(a, b):
    return ((a[0] * b[0] - a[1] * b[1]) % P, (a[0] * b[1] + a[1] * b[0]) % P)


def _pmul(p, k):
    r = (1, 0)
    while k:
        if k & 1:
            r = _padd(r, p)
        p = _padd(p, p)
        k >>= 1
    return r


def _subgroup_gen(log_size):
    return _pmul(GEN, 1 << (31 - log_size))


class RefCuda:
    def __init__(self):
        if not available():
            raise RuntimeError("oracle/_ref/libstwo_cuda_ref.so is not built (make -f oracle/Makefile.ref_cuda)")
        L = self.lib = C.CDLL(LIB_PATH)
        vp, u32, i32 = C.c_void_p, C.c_uint32, C.c_int
        L.copy_uint32_t_vec_from_host_to_device.restype = vp
        L.copy_uint32_t_vec_from_host_to_device.argtypes = [vp, i32]
        L.copy_uint32_t_vec_from_device_to_host.restype = None
        L.copy_uint32_t_vec_from_device_to_host.argtypes = [vp, vp, i32]
        L.copy_uint32_t_vec_from_device_to_device.restype = None
        L.copy_uint32_t_vec_from_device_to_device.argtypes = [vp, vp, i32]
        L.cuda_malloc_uint32_t.restype = vp
        L.cuda_malloc_uint32_t.argtypes = [i32]
        L.cuda_alloc_zeroes_uint32_t.restype = vp
        L.cuda_alloc_zeroes_uint32_t.argtypes = [i32]
        L.cuda_malloc_blake_2s_hash.restype = vp
        L.cuda_malloc_blake_2s_hash.argtypes = [i32]
        L.copy_blake_2s_hash_vec_from_device_to_host.restype = None
        L.copy_blake_2s_hash_vec_from_device_to_host.argtypes = [vp, vp, u32]
        L.copy_device_pointer_vec_from_host_to_device.restype = vp
        L.copy_device_pointer_vec_from_host_to_device.argtypes = [vp, u32]
        L.cuda_free_memory.restype = None
        L.cuda_free_memory.argtypes = [vp]
        L.precompute_twiddles.restype = vp
        L.precompute_twiddles.argtypes = [_Point, _Point, i32]
        L.batch_inverse_base_field.restype = None
        L.batch_inverse_base_field.argtypes = [vp, vp, i32]
        for f in (L.ntt_b2n_column, L.ntt_n2b_columns):
            f.restype = None
            f.argtypes = [vp, u32, u32, vp, u32, u32]
        L.commit_on_first_layer_m31.restype = None
        L.commit_on_first_layer_m31.argtypes = [u32, u32, vp, vp]
        L.commit_on_layer_with_previous_m31.restype = None
        L.commit_on_layer_with_previous_m31.argtypes = [u32, u32, vp, vp, vp]
        L.gkr_device_synchronize.restype = None
        L.gkr_device_synchronize.argtypes = []

    # ---- memory
    def upload(self, arr):
        arr = np.ascontiguousarray(arr, dtype=np.uint32)
        return self.lib.copy_uint32_t_vec_from_host_to_device(arr.ctypes.data, arr.size)

    def download(self, ptr, n):
        out = np.empty(n, np.uint32)
        self.lib.copy_uint32_t_vec_from_device_to_host(ptr, out.ctypes.data, n)
        return out

    def download_hashes(self, ptr, n):
        out = np.empty((n, 8), np.uint32)
        self.lib.copy_blake_2s_hash_vec_from_device_to_host(ptr, out.ctypes.data, n)
        return out

    def free(self, ptr):
        self.lib.cuda_free_memory(ptr)

    def sync(self):
        self.lib.gkr_device_synchronize()

    # ---- PolyOps::precompute_twiddles (backend/cuda/poly.rs:554-576) for Coset::half_odds(log_half)
    def twiddle_tree(self, log_half):
        initial, step, size = _subgroup_gen(log_half + 2), _subgroup_gen(log_half), 1 << log_half
        tw = self.lib.precompute_twiddles(_Point(*initial), _Point(*step), size)
        itw = self.lib.cuda_malloc_uint32_t(size)
        self.lib.batch_inverse_base_field(tw, itw, size)
        return {"tw": tw, "itw": itw, "size": size}

    # ---- PolyOps::interpolate_columns (poly.rs:211-294): in place on columns of 2^log_n values
    def interpolate_columns(self, col_ptrs, log_n, tree):
        arr = (C.c_void_p * len(col_ptrs))(*col_ptrs)
        self.lib.ntt_b2n_column(arr, log_n, len(col_ptrs), tree["itw"], tree["size"], 1 << (log_n - 1))

    # ---- PolyOps::evaluate_polynomials (poly.rs:458-552): zero-extended copies, then one batched transform
    def extend_columns(self, coeff_ptrs, log_n, log_out):
        out = []
        for p in coeff_ptrs:
            q = self.lib.cuda_alloc_zeroes_uint32_t(1 << log_out)
            self.lib.copy_uint32_t_vec_from_device_to_device(p, q, 1 << log_n)
            out.append(q)
        return out

    def evaluate_extended(self, ext_ptrs, log_out, tree):
        arr = (C.c_void_p * len(ext_ptrs))(*ext_ptrs)
        self.lib.ntt_n2b_columns(arr, log_out, len(ext_ptrs), tree["tw"], tree["size"], 1 << (log_out - 1))

    # ---- MerkleOps<Blake2sM31MerkleHasher>::commit_on_layer (blake2s.rs:61-96)
    def commit_on_layer(self, log_size, prev_ptr, col_ptrs):
        n = 1 << log_size
        res = self.lib.cuda_malloc_blake_2s_hash(n)
        arr = (C.c_void_p * max(len(col_ptrs), 1))(*col_ptrs)
        dptrs = self.lib.copy_device_pointer_vec_from_host_to_device(arr, len(col_ptrs)) if col_ptrs else None
        if prev_ptr:
            self.lib.commit_on_layer_with_previous_m31(n, len(col_ptrs), dptrs, prev_ptr, res)
        else:
            self.lib.commit_on_first_layer_m31(n, len(col_ptrs), dptrs, res)
        if dptrs:
            self.sync()
            self.free(dptrs)
        return res


class _Q(C.Structure):  # qm31 by value (stwo_cuda/cuda/fields.cuh:10-18; bindings.rs CudaSecureField)
    _fields_ = [("a", C.c_uint32), ("b", C.c_uint32), ("c", C.c_uint32), ("d", C.c_uint32)]


def _q(v):
    v = [int(x) for x in np.asarray(v).reshape(4)]
    return _Q(*v)


def _ptrs(ps):
    return (C.c_void_p * len(ps))(*ps)


class RefCudaOps(RefCuda):
    """FriOps, QuotientOps, GkrOps, MleOps and ColumnOps of the reference's CUDA backend
    (prover/backend/cuda/{fri,quotient}.rs, prover/backend/cuda/lookups/gkr.rs)."""

    def __init__(self):
        super().__init__()
        L, vp, u32, i32 = self.lib, C.c_void_p, C.c_uint32, C.c_int
        for f in (L.fold_line, L.fold_circle_into_line):
            f.restype = None
            f.argtypes = [vp, u32, u32, vp, _Q, vp]
        L.accumulate_numerators_batch.restype = None
        L.accumulate_numerators_batch.argtypes = [i32, vp, vp, vp, vp, i32, vp, vp, vp, vp]
        L.compute_quotients_and_combine.restype = None
        L.compute_quotients_and_combine.argtypes = [i32, i32, u32, u32, i32, vp, vp, vp, vp, vp, vp, vp, vp]
        L.gen_eq_evals.restype = None
        L.gen_eq_evals.argtypes = [_Q, vp, u32, vp, u32]
        L.gkr_next_layer_grand_product.restype = None
        L.gkr_next_layer_grand_product.argtypes = [vp, vp, u32]
        L.gkr_next_layer_logup_generic.restype = None
        L.gkr_next_layer_logup_generic.argtypes = [vp, vp, vp, vp, u32]
        L.gkr_next_layer_logup_multiplicities.restype = None
        L.gkr_next_layer_logup_multiplicities.argtypes = [vp, vp, vp, vp, u32]
        L.gkr_next_layer_logup_singles.restype = None
        L.gkr_next_layer_logup_singles.argtypes = [vp, vp, vp, u32]
        L.gkr_sum_grand_product.restype = None
        L.gkr_sum_grand_product.argtypes = [vp, vp, u32, vp, u32]
        L.gkr_sum_logup_generic.restype = None
        L.gkr_sum_logup_generic.argtypes = [vp, vp, vp, _Q, u32, vp, u32]
        L.gkr_sum_logup_multiplicities.restype = None
        L.gkr_sum_logup_multiplicities.argtypes = [vp, vp, vp, _Q, u32, vp, u32]
        L.gkr_sum_logup_singles.restype = None
        L.gkr_sum_logup_singles.argtypes = [vp, vp, _Q, u32, vp, u32]
        L.fix_first_variable_base_field.restype = None
        L.fix_first_variable_base_field.argtypes = [vp, i32, _Q, vp]
        L.fix_first_variable_secure_field.restype = None
        L.fix_first_variable_secure_field.argtypes = [vp, i32, _Q, vp]
        L.bit_reverse_base_field.restype = None
        L.bit_reverse_base_field.argtypes = [vp, i32]

    def alloc(self, words):
        return self.lib.cuda_malloc_uint32_t(words)

    def alloc_zero(self, words):
        return self.lib.cuda_alloc_zeroes_uint32_t(words)

    # FriOps::fold_line (fri.rs:17-46): the line domain is LineDomain(Coset::half_odds(log_n)); the tree's root
    # coset is a half_odds coset at least that large.
    def fold_line(self, in_ptrs, log_n, alpha, tree):
        n = 1 << log_n
        out = [self.alloc(n // 2) for _ in range(4)]
        self.lib.fold_line(tree["itw"], tree["size"] - n, n, _ptrs(in_ptrs), _q(alpha), _ptrs(out))
        return out

    # FriOps::fold_circle_into_line (fri.rs:48-69): src on CanonicCoset(log_n).circle_domain()
    def fold_circle_into_line(self, dst_ptrs, src_ptrs, log_n, alpha, tree):
        n = 1 << log_n
        self.lib.fold_circle_into_line(tree["itw"], tree["size"] - n // 2, n, _ptrs(src_ptrs), _q(alpha), _ptrs(dst_ptrs))

    # QuotientOps::accumulate_numerators, one sample batch (quotient.rs:38-74)
    def quot_numerators(self, col_ptrs, log_n, col_idx, b, c):
        n, k = 1 << log_n, len(col_idx)
        dcols = self.lib.copy_device_pointer_vec_from_host_to_device(_ptrs(col_ptrs), len(col_ptrs))
        out = [self.alloc_zero(n) for _ in range(4)]
        b = np.ascontiguousarray(b, np.uint32)
        c = np.ascontiguousarray(c, np.uint32)
        idx = np.ascontiguousarray(col_idx, np.uint32)
        self.lib.accumulate_numerators_batch(n, dcols, b.ctypes.data, c.ctypes.data, idx.ctypes.data, k, *out)
        self.sync()
        self.free(dcols)
        return out

    # QuotientOps::compute_quotients_and_combine (quotient.rs:84-141)
    def quot_combine(self, acc_ptrs, acc_logs, first_lin, points, max_log):
        n = 1 << max_log
        out = [self.alloc_zero(n) for _ in range(4)]
        logs = np.ascontiguousarray(acc_logs, np.int32)
        fl = np.ascontiguousarray(first_lin, np.uint32)
        pts = np.ascontiguousarray(points, np.uint32)  # per accumulation: x (4 words), y (4 words)
        flat = [p for acc in acc_ptrs for p in acc]
        self.lib.compute_quotients_and_combine(n, max_log, 1 << (30 - max_log), (1 << (32 - max_log)) & 0xFFFFFFFF, len(acc_ptrs),
                                               _ptrs(flat), logs.ctypes.data, fl.ctypes.data, pts.ctypes.data, *out)
        self.sync()
        return out

    # GkrOps (lookups/gkr.rs)
    def gen_eq_evals(self, y, v):
        y = np.ascontiguousarray(y, np.uint32).reshape(-1, 4)
        m = y.shape[0]
        out = self.alloc(4 << m)
        self.lib.gen_eq_evals(_q(v), y.ctypes.data, m, out, 1 << m)
        return out

    def next_layer(self, kind, num, den, n):
        no, do = self.alloc(2 * n), self.alloc(2 * n)
        if kind == 0:
            self.lib.gkr_next_layer_grand_product(den, do, n // 2)
        elif kind == 1:
            self.lib.gkr_next_layer_logup_generic(num, den, no, do, n // 2)
        elif kind == 2:
            self.lib.gkr_next_layer_logup_multiplicities(num, den, no, do, n // 2)
        else:
            self.lib.gkr_next_layer_logup_singles(den, no, do, n // 2)
        return no, do

    def round_sums(self, kind, num, den, n, eq, lam):
        n_terms = n // 4
        blocks = max(1, min((n_terms + 255) // 256, 96))
        part = self.alloc(8 * blocks)
        if kind == 0:
            self.lib.gkr_sum_grand_product(den, eq, n_terms, part, blocks)
        elif kind == 1:
            self.lib.gkr_sum_logup_generic(num, den, eq, _q(lam), n_terms, part, blocks)
        elif kind == 2:
            self.lib.gkr_sum_logup_multiplicities(num, den, eq, _q(lam), n_terms, part, blocks)
        else:
            self.lib.gkr_sum_logup_singles(den, eq, _q(lam), n_terms, part, blocks)
        p = self.download(part, 8 * blocks).reshape(blocks, 2, 4).astype(np.uint64)
        self.free(part)
        return (p.sum(axis=0) % np.uint64(P)).astype(np.uint32)

    def fix_first_variable(self, ptr, n, r, base):
        out = self.alloc(2 * n)
        (self.lib.fix_first_variable_base_field if base else self.lib.fix_first_variable_secure_field)(ptr, n, _q(r), out)
        return out

    def bit_reverse(self, ptr, n):
        self.lib.bit_reverse_base_field(ptr, n)


class RefCudaMore(RefCudaOps):
    """AccumulationOps, batch_eval_at_point and GrindOps of the reference's CUDA backend
    (prover/backend/cuda/{accumulation,poly}.rs, stwo_cuda/cuda/grind_blake2s.cu)."""

    def __init__(self):
        super().__init__()
        L, vp, u32, i32 = self.lib, C.c_void_p, C.c_uint32, C.c_int
        L.accumulate.restype = None
        L.accumulate.argtypes = [i32, vp, vp]
        L.lift_and_accumulate.restype = None
        L.lift_and_accumulate.argtypes = [i32] + [vp] * 8 + [i32]
        L.batch_eval_at_points.restype = None
        L.batch_eval_at_points.argtypes = [vp, i32, i32, _Q, _Q, vp]
        L.grind_blake2s.restype = C.c_uint64
        L.grind_blake2s.argtypes = [vp, u32]

    def accumulate(self, left4, right4, n):
        self.lib.accumulate(n, _ptrs(left4), _ptrs(right4))

    def lift_and_accumulate(self, dst4, log_dst, src4, log_src):
        self.lib.lift_and_accumulate(1 << log_dst, *dst4, *src4, log_dst - log_src)

    def batch_eval_at_point(self, coeff_ptrs, log_n, point8):
        pt = np.ascontiguousarray(point8, np.uint32).reshape(8)
        d = self.lib.copy_device_pointer_vec_from_host_to_device(_ptrs(coeff_ptrs), len(coeff_ptrs))
        out = np.zeros((len(coeff_ptrs), 4), np.uint32)
        self.lib.batch_eval_at_points(d, 1 << log_n, len(coeff_ptrs), _q(pt[:4]), _q(pt[4:]), out.ctypes.data)
        self.free(d)
        return out

    def grind(self, prefixed_digest8, pow_bits):
        d = np.ascontiguousarray(prefixed_digest8, np.uint32)
        return int(self.lib.grind_blake2s(d.ctypes.data, pow_bits))


class _ZkGrid(C.Structure):  # stwo_cuda/cuda/zk_attention_freivalds_witness_gen.cuh:52-59 (= ZkAccGrid, zk_acc.cuh:88-95)
    _fields_ = [(n, C.c_uint32) for n in ("log_rows", "rows", "groups", "chunks", "lead", "descending")]


class _ZkMult(C.Structure):
    _fields_ = [("m", C.c_void_p), ("n", C.c_uint32)]


class _ZkFreivaldsCfg(C.Structure):
    _fields_ = [("g", _ZkGrid)] + [(n, C.c_uint32) for n in ("pq", "pk", "n_in", "tokens", "n_mats", "mutate")]


class _ZkAccFreivalds(C.Structure):
    _fields_ = [("g", _ZkGrid)] + [(n, C.c_uint32) for n in ("pq", "pk", "n_mats", "off_x", "mutate")]


class _ZkAccS2(C.Structure):  # zk_acc.cuh:194-202
    _fields_ = [(n, C.c_uint32) for n in ("dst", "src0", "src1", "sel_i")] + [("m_i", _Q), ("m_l", _Q), ("m_n", _Q)]


class RefCudaFreivalds(RefCudaMore):
    """The Freivalds attention-witness component of the reference's device path
    (prover/src/gadgets/freivalds/device.rs:56-133 and prover/src/devacc.rs:665-713)."""

    def __init__(self):
        super().__init__()
        L, vp, u32 = self.lib, C.c_void_p, C.c_uint32
        L.zk_witness_gen_freivalds.restype = None
        L.zk_witness_gen_freivalds.argtypes = [vp, vp, vp, vp, u32, vp, u32, _ZkMult, vp, _ZkFreivaldsCfg]
        L.zk_acc_freivalds.restype = None
        L.zk_acc_freivalds.argtypes = [vp, vp, vp, vp, _Q, _Q, vp, vp, vp, _ZkAccFreivalds]
        L.zk_acc_scan.restype = None
        L.zk_acc_scan.argtypes = [vp, vp, u32, u32, u32]
        L.zk_acc_stage2.restype = None
        L.zk_acc_stage2.argtypes = [vp, vp, vp, vp, u32, u32, u32]
        L.zk_acc_split.restype = None
        L.zk_acc_split.argtypes = [vp, vp, vp, u32, u32, u32, u32]
        L.zk_acc_last.restype = None
        L.zk_acc_last.argtypes = [vp, vp, u32, u32]

    @staticmethod
    def _grid(grid):
        log_rows, groups, chunks, lead = grid
        return _ZkGrid(log_rows, 1 << log_rows, groups, chunks, lead, 1)

    def upload_i8(self, arr):
        b = np.ascontiguousarray(arr, np.int8).reshape(-1)
        pad = (-b.size) % 4
        w = np.concatenate([b, np.zeros(pad, np.int8)]).view(np.uint32)
        return self.upload(w)

    def scatter(self, qx, qws, grid, pq, pk):
        tokens, n_in = qx.shape
        rows = 1 << grid[0]
        d_qx = self.upload_i8(qx)
        d_qw = [self.upload_i8(w) for w in qws]
        n_out = np.array([w.shape[1] for w in qws], np.uint32)
        base = [self.alloc(rows) for _ in range(pq)]
        pre = [self.alloc(rows) for _ in range(len(qws) * pk + 4)]
        m_r8, counts = self.alloc_zero(256), self.alloc_zero(3)
        cfg = _ZkFreivaldsCfg(self._grid(grid), pq, pk, n_in, tokens, len(qws), 0)
        self.lib.zk_witness_gen_freivalds(d_qx, _ptrs(d_qw), n_out.ctypes.data, _ptrs(base), len(base), _ptrs(pre), len(pre),
                                          _ZkMult(m_r8, 256), counts, cfg)
        for p in [d_qx] + d_qw:
            self.free(p)
        return base, pre, m_r8, counts

    def acc(self, base, pre, grid, pq, pk, n_mats, s, rv, s_pow, rv_pow, s_step, rv_step):
        rows = 1 << grid[0]
        lanes = 1 + 2 * n_mats
        a, b, flags = self.alloc(4 * lanes * rows), self.alloc(4 * lanes * rows), self.alloc_zero(rows)
        sp, rp = np.ascontiguousarray(s_pow, np.uint32), np.ascontiguousarray(rv_pow, np.uint32)
        cfg = _ZkAccFreivalds(self._grid(grid), pq, pk, n_mats, 128, 0)
        self.lib.zk_acc_freivalds(_ptrs(base), _ptrs(pre[:n_mats * pk]), sp.ctypes.data, rp.ctypes.data, _q(s_step), _q(rv_step), flags, a, b, cfg)
        self.lib.zk_acc_scan(a, b, rows, 1 + n_mats, 0)
        one = _Q(1, 0, 0, 0)
        s2 = (_ZkAccS2 * n_mats)(*[_ZkAccS2(1 + n_mats + m, 1 + m, 0, 0, one, one, one) for m in range(n_mats)])
        self.lib.zk_acc_stage2(flags, a, b, s2, n_mats, rows, 0)
        off = 16 * (1 + n_mats) * rows  # bytes: a QM31 is four words
        self.lib.zk_acc_scan(a + off, b + off, rows, n_mats, 0)
        last = np.zeros((lanes, 4), np.uint32)
        self.lib.zk_acc_last(b, last.ctypes.data, rows, lanes)
        order = [0]
        for m in range(n_mats):
            order += [1 + m, 1 + n_mats + m]
        order = np.array(order, np.uint32)
        out = [self.alloc(rows) for _ in range(4 * len(order))]
        self.lib.zk_acc_split(b, _ptrs(out), order.ctypes.data, len(order), rows, grid[0], 0)
        for p in (a, b, flags):
            self.free(p)
        return out, last[1 + n_mats:1 + 2 * n_mats]


class _ZkTabCfg(C.Structure):  # stwo_cuda/cuda/zk_table_witness_gen.cuh:57-68
    _fields_ = [("log_rows", C.c_uint32), ("rows", C.c_uint32), ("variant", C.c_uint32), ("n_counters", C.c_uint32), ("two_pow", C.c_double),
                ("mutate", C.c_uint32), ("mut_col", C.c_uint32)]


_DEQ_FIELDS = ("variant", "sticky", "kmax", "do_ref", "tokens", "n_out", "per_row", "chunks", "log_rows", "slot0", "per_slot", "chan_w",
               "f_acc", "f_sg", "f_m2", "f_ph", "f_st", "f_r", "f_m7", "f_ef", "f_nz", "f_eo", "f_mul0", "f_mul1", "f_mul2", "f_mul3",
               "f_mul4", "f_mul5", "sh0", "sh1", "n_norm", "n_frac", "n_mul", "n_r8")


class _ZkDequantCfg(C.Structure):  # stwo_cuda/cuda/zk_dequant_witness_gen.cuh:38-60 (f_mul[6] as six fields)
    _fields_ = [(n, C.c_uint32) for n in _DEQ_FIELDS + ("mutate",)]


class RefCudaWitness(RefCudaMore):
    """The reference's device witness generation for the tables' own columns (prover/src/devtab.rs:240-290) and for one
    dequantize component (prover/src/gadgets/dequant/device.rs:199-360), driven as those call sites do, with no defect
    selected (mutate = 0)."""

    def __init__(self):
        super().__init__()
        L, vp, u32 = self.lib, C.c_void_p, C.c_uint32
        L.zk_witness_gen_tables.restype = None
        L.zk_witness_gen_tables.argtypes = [vp, vp, vp, vp, u32, vp, vp, vp, _ZkTabCfg]
        L.zk_witness_gen_dequant.restype = None
        L.zk_witness_gen_dequant.argtypes = [vp] * 8 + [u32, vp, u32] + [vp] * 6 + [_ZkDequantCfg]

    def upload_any(self, arr):
        return self.upload(np.ascontiguousarray(arr).view(np.uint32).reshape(-1))

    def tables(self, expmap, counters, log_rows, bf16x, two_pow, patch_idx, patch_val):
        rows = 1 << log_rows
        d_map = self.upload(expmap)
        d_cnt = [self.upload(c) for c in counters]
        x, y, m = self.alloc(rows), self.alloc(rows), self.alloc_zero(rows)
        pi = self.upload(patch_idx) if len(patch_idx) else None
        pv = self.upload(patch_val) if len(patch_idx) else None
        cfg = _ZkTabCfg(log_rows, rows, 0 if bf16x else 1, len(counters), two_pow, 0, 0)
        self.lib.zk_witness_gen_tables(d_map, _ptrs(d_cnt) if d_cnt else None, pi, pv, len(patch_idx), x, y, m if counters else None, cfg)
        out = self.download(x, rows), self.download(y, rows), self.download(m, rows)
        for p in [d_map, x, y, m] + d_cnt + ([pi, pv] if pi else []):
            self.free(p)
        return out

    def dequant(self, case):
        cfg, rows = case["cfg"], case["rows"]
        chain = cfg["variant"] == 1
        d = {k: self.upload_any(case[k]) for k in ("acc", "jx", "jw", "sx", "sw", "norm3", "mul2")}
        base = [self.alloc_zero(rows) for _ in range(case["n_base"])]
        pre = [self.alloc_zero(rows) for _ in range(case["n_pre"])]
        m_norm, m_frac = self.alloc_zero(cfg["n_norm"]), self.alloc_zero(cfg["n_frac"])
        m_mul, m_r8, counts = self.alloc_zero(cfg["n_mul"]), self.alloc_zero(cfg["n_r8"]), self.alloc_zero(3)
        want = self.alloc_zero(rows * cfg["per_row"])
        c = _ZkDequantCfg(*([int(cfg[k]) for k in _DEQ_FIELDS] + [0]))
        self.lib.zk_witness_gen_dequant(d["acc"], None if chain else d["jx"], None if chain else d["jw"], d["sx"] if chain else None,
                                        d["sw"] if chain else None, d["norm3"], d["mul2"], _ptrs(base), len(base), _ptrs(pre), len(pre),
                                        m_norm, m_frac, m_mul, m_r8, counts, want, c)
        out = {"base": np.stack([self.download(b, rows) for b in base]), "pre": np.stack([self.download(p_, rows) for p_ in pre]),
               "m_norm": self.download(m_norm, cfg["n_norm"]), "m_frac": self.download(m_frac, cfg["n_frac"]),
               "m_mul": self.download(m_mul, cfg["n_mul"]), "m_r8": self.download(m_r8, cfg["n_r8"]), "counts": self.download(counts, 3),
               "want": self.download(want, rows * cfg["per_row"])}
        for p_ in list(d.values()) + base + pre + [m_norm, m_frac, m_mul, m_r8, counts, want]:
            self.free(p_)
        return out


class _ZkPreCfg(C.Structure):  # stwo_cuda/cuda/zk_pre_witness_gen.cuh:103-115
    _fields_ = [(n, C.c_uint32) for n in ("kind", "log_rows", "rows", "real_rows", "kmax", "round", "sticky", "n_cols", "n_counters", "mutate", "at")]


class _ZkAccGrid(C.Structure):  # stwo_cuda/cuda/zk_acc.cuh:88-95
    _fields_ = [(n, C.c_uint32) for n in ("log_rows", "rows", "groups", "chunks", "lead", "descending")]


class _ZkAccFlags(C.Structure):  # stwo_cuda/cuda/zk_acc.cuh:185-190
    _fields_ = [("shape", C.c_uint32), ("g", _ZkAccGrid), ("modulus", C.c_uint32), ("rw", C.c_uint32)]


class _ZkSelCfg(C.Structure):  # stwo_cuda/cuda/zk_pre_witness_gen.cuh:118-128
    _fields_ = [("shape", C.c_uint32), ("g", _ZkAccGrid)] + [(n, C.c_uint32) for n in ("ctx", "n_insts", "with_scale", "n_cols", "fam", "mutate", "at")]


class _ZkRsMult(C.Structure):  # stwo_cuda/cuda/zk_residual_stream_witness_gen.cuh (ZkResidualStreamMult)
    _fields_ = [("m", C.c_void_p), ("n", C.c_uint32)]


class _ZkRsCfg(C.Structure):  # ZkResidualStreamCfg
    _fields_ = [(n, C.c_uint32) for n in ("log_rows", "rows", "live", "n_groups", "n_leaves", "n_slots", "n_cols", "kind", "sticky", "kmax", "out_w",
                                          "mutate")]


class RefCudaWitnessPre(RefCudaWitness):
    """The reference's device witness generation for the shared tables (prover/src/devpre.rs:440-500), the key tile's flags and
    selectors (devpre.rs:590-640) and the residual-stream component (prover/src/gadgets/residual_stream/device.rs:300-440), with
    no defect selected (mutate = 0)."""

    def __init__(self):
        super().__init__()
        L, vp, u32 = self.lib, C.c_void_p, C.c_uint32
        L.zk_witness_gen_pre_table.restype = None
        L.zk_witness_gen_pre_table.argtypes = [vp, vp, vp, u32, vp, vp, _ZkPreCfg]
        L.zk_flags_key_tile.restype = None
        L.zk_flags_key_tile.argtypes = [vp, _ZkAccFlags]
        L.zk_witness_gen_sel.restype = None
        L.zk_witness_gen_sel.argtypes = [vp, vp, vp, _ZkSelCfg]
        L.zk_witness_gen_residual_stream.restype = None
        L.zk_witness_gen_residual_stream.argtypes = ([vp] * 4 + [u32, vp, u32, vp, u32, u32] + [vp] * 5 + [_ZkRsMult] * 5 + [vp, vp, _ZkRsCfg])

    def pre_table(self, kind, log_rows, kmax, round_mode, counters, patch_idx, patch_val):
        rows, n_cols = 1 << log_rows, {0: 6, 1: 3, 2: 4, 3: 2, 4: 1}[kind]
        sticky = 1 if round_mode == 0 else 0
        real = {0: 256 + (kmax + 1) * 256 * (1 + sticky), 1: 1 << (kmax + 1), 2: 1 << 14}.get(kind, rows)
        d_cnt = [self.upload(c) for c in counters]
        cols, m = [self.alloc_zero(rows) for _ in range(n_cols)], self.alloc_zero(rows)
        pi = self.upload(patch_idx) if len(patch_idx) else None
        pv = self.upload(np.ascontiguousarray(patch_val).reshape(-1)) if len(patch_idx) else None
        cfg = _ZkPreCfg(kind, log_rows, rows, real, kmax, round_mode, sticky, n_cols, len(counters), 0, 0)
        self.lib.zk_witness_gen_pre_table(_ptrs(d_cnt) if d_cnt else None, pi, pv, len(patch_idx), _ptrs(cols), m if counters else None, cfg)
        out = np.stack([self.download(c, rows) for c in cols]), self.download(m, rows)
        for p_ in cols + [m] + d_cnt + ([pi, pv] if pi else []):
            self.free(p_)
        return out

    def flags_and_selectors(self, shape, log_rows, groups, chunks, lead, descending, modulus, rw, scale, ctx_len, n_insts, with_scale, n_cols):
        rows = 1 << log_rows
        grid = _ZkAccGrid(log_rows, rows, groups, chunks, lead, descending)
        d_flags = self.alloc_zero(rows)
        self.lib.zk_flags_key_tile(d_flags, _ZkAccFlags(shape, grid, modulus, rw))
        flags = self.download(d_flags, rows)
        cols, d_scale = [self.alloc_zero(rows) for _ in range(n_cols)], self.upload(scale)
        fam = {0: 5, 1: 6, 2: 7}[shape]  # ZK_PRE_AT_CHAN / _KEY / _ROW
        self.lib.zk_witness_gen_sel(d_flags, _ptrs(cols), d_scale, _ZkSelCfg(shape, grid, ctx_len, n_insts, 1 if with_scale else 0, n_cols, fam, 0, 8))
        out = flags, np.stack([self.download(c, rows) for c in cols])
        for p_ in cols + [d_flags, d_scale]:
            self.free(p_)
        return out

    def residual_stream(self, case):
        rows, n_leaves, n_cols, out_w = 1 << case["log_rows"], case["n_leaves"], case["n_cols"], len(case["out_slot"])
        ml, n_un = case["m_len"], len(case["un2"])
        d = {k: self.upload_any(case[k]) for k in ("wit", "norm3", "smul3", "lowered_groups", "lowered_slots")}
        d_out_slot = self.upload(np.asarray(case["out_slot"], np.uint32))
        d_un = [self.upload_any(u) for u in case["un2"]]
        cols = [self.alloc_zero(rows) for _ in range(n_cols)]
        out_pat, out_nat, in_nat = self.alloc_zero(max(1, rows * out_w)), self.alloc_zero(max(1, rows * out_w * 2)), self.alloc_zero(rows * n_leaves * 2)
        ms = {k: self.alloc_zero(ml[k]) for k in ("pow", "norm", "val", "frac", "smul")}
        m_un = [self.alloc_zero(ml["un"]) for _ in range(n_un)]
        un_recs = np.zeros(max(1, n_un) * 4, np.uint32)  # ZkResidualStreamMult records: pointer (8 bytes), n, padding
        for u, p_ in enumerate(m_un):
            un_recs[4 * u:4 * u + 2] = np.array([int(p_)], np.uint64).view(np.uint32)
            un_recs[4 * u + 2] = ml["un"]
        d_un_recs, counts = self.upload(un_recs), self.alloc_zero(3)
        cfg = _ZkRsCfg(case["log_rows"], rows, case["live_rows"], len(case["groups"]), n_leaves, len(case["src_slots"]), n_cols, case["kind"],
                       1 if case["sticky"] else 0, case["kmax"], out_w, 0)
        mult = lambda k: _ZkRsMult(ms[k], ml[k])
        self.lib.zk_witness_gen_residual_stream(d["wit"], d["lowered_groups"], d["lowered_slots"], d["norm3"], len(case["norm3"]) // 3, d["smul3"],
                                                len(case["smul3"]) // 3, _ptrs(d_un) if d_un else None, n_un, case["n_val"], d_out_slot, _ptrs(cols),
                                                out_pat, out_nat, in_nat, mult("pow"), mult("norm"), mult("val"), mult("frac"), mult("smul"),
                                                d_un_recs, counts, cfg)
        out = {"cols": np.stack([self.download(c, rows) for c in cols]), "out_pat": self.download(out_pat, max(1, rows * out_w))[:rows * out_w],
               "out_nat": self.download(out_nat, max(1, rows * out_w * 2))[:rows * out_w * 2].view(np.int32),
               "in_nat": self.download(in_nat, rows * n_leaves * 2).view(np.int32), "m_pow": self.download(ms["pow"], ml["pow"]),
               "m_norm": self.download(ms["norm"], ml["norm"]), "m_val": self.download(ms["val"], ml["val"]),
               "m_frac": self.download(ms["frac"], ml["frac"]), "m_smul": self.download(ms["smul"], ml["smul"]),
               "m_un": np.stack([self.download(m_, ml["un"]) for m_ in m_un]) if m_un else np.zeros((0, ml["un"]), np.uint32),
               "counts": self.download(counts, 3)}
        for p_ in list(d.values()) + [d_out_slot, d_un_recs, counts, out_pat, out_nat, in_nat] + d_un + cols + list(ms.values()) + m_un:
            self.free(p_)
        return out


class RefCudaAir(RefCudaOps):
    """The reference's hand-written constraint kernel for the wide Fibonacci example AIR
    (stwo_cuda/cuda/evaluate_wide_fibonacci.cu:6-63, launcher :65-125; the AIR is
    nitroo/crates/examples/src/wide_fibonacci/mod.rs:47-57)."""

    def __init__(self):
        super().__init__()
        vp, u32 = C.c_void_p, C.c_uint32
        f = self.lib.evaluate_wide_fibonacci_constraint_quotients_on_domain
        f.restype = None
        f.argtypes = [vp, vp, vp, vp, vp, u32, vp, u32, vp, vp, u32, u32, u32, u32]

    def wide_fibonacci_quotients(self, col_ptrs, rcp, denom_inv, trace_log, eval_log):
        """col_ptrs: device pointers of the n columns on the evaluation domain. Returns 4 device pointers (the kernel
        overwrites its output: quotient = denom_inv * sum_i rcp[i] * constraint_i)."""
        n = 1 << eval_log
        out = [self.alloc_zero(n) for _ in range(4)]
        d_rcp, d_den = self.upload(np.ascontiguousarray(rcp, np.uint32).reshape(-1)), self.upload(denom_inv)
        table = (C.c_void_p * len(col_ptrs))(*col_ptrs)
        self.lib.evaluate_wide_fibonacci_constraint_quotients_on_domain(out[0], out[1], out[2], out[3], None, 0, table, len(col_ptrs),
                                                                        d_rcp, d_den, trace_log, eval_log, len(col_ptrs) - 2, 0)
        self.free(d_rcp)
        self.free(d_den)
        return out
