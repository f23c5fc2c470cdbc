"""ctypes bindings over include/zkb200.h. Every call goes through the C ABI of libzkb200.so."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "lib", "libzkb200.so")

GKR_GRAND_PRODUCT, GKR_LOGUP_GENERIC, GKR_LOGUP_MULTIPLICITIES, GKR_LOGUP_SINGLES = 0, 1, 2, 3

# Every symbol include/zkb200.h declares.
EXPORTED_SYMBOLS = [
    "zkb_init", "zkb_destroy", "zkb_last_error", "zkb_sync", "zkb_get_stream", "zkb_max_log_size",
    "zkb_event_record", "zkb_event_elapsed_ms", "zkb_profile_begin", "zkb_profile_end", "zkb_fft_arith_ceiling",
    "zkb_malloc", "zkb_free", "zkb_memset_zero", "zkb_h2d", "zkb_d2h", "zkb_h2d_async", "zkb_d2h_async", "zkb_h2d_overlapped", "zkb_wait_fence", "zkb_peer_buffer_alloc", "zkb_peer_buffer_free", "zkb_peer_buffer_open",
    "zkb_peer_buffer_close", "zkb_copy_to_peer", "zkb_peer_copies_wait", "zkb_d2d",
    "zkb_host_alloc_pinned", "zkb_host_free_pinned", "zkb_gather_multi", "zkb_gather_hashes", "zkb_gather_words", "zkb_twiddles_d2h",
    "zkb_ifft_cols", "zkb_lde_cols", "zkb_eval_at_point_cols", "zkb_barycentric_weights", "zkb_barycentric_eval_at_point", "zkb_eval_at_point_by_folding", "zkb_fri_decompose", "zkb_bit_reverse_m31", "zkb_bit_reverse_qm31",
    "zkb_merkle_layer", "zkb_merkle_leaves_partial", "zkb_merkle_levels", "zkb_merkle_top", "zkb_merkle_top_channel", "zkb_fold_line_dalpha", "zkb_fold_circle_into_line_dalpha", "zkb_channel_mix_root_draw", "zkb_fold_line_dalpha_leaves", "zkb_fold_circle_into_line_dalpha_leaves", "zkb_fold_circle_into_line", "zkb_fold_line", "zkb_quot_numerators", "zkb_quot_combine", "zkb_quot_combine_rows",
    "zkb_accumulate", "zkb_lift_accumulate", "zkb_secure_powers", "zkb_gkr_eq_evals", "zkb_gkr_next_layer",
    "zkb_gkr_sum", "zkb_gkr_fix_and_sum", "zkb_mle_fix_qm31", "zkb_mle_fix_m31", "zkb_grind", "zkb_gkr_sum_noalloc", "zkb_gkr_sum_noalloc_error",
    "zkb_freivalds_scatter", "zkb_freivalds_acc", "zkb_witness_tables", "zkb_witness_dequant", "zkb_witness_pre_table", "zkb_key_tile_flags",
    "zkb_witness_selectors", "zkb_witness_residual_stream",
]
# Every symbol include/zkb200_prover.h declares.
PROVER_SYMBOLS = ["zkb_pcs_prove_device", "zkb_pcs_prove_host", "zkb_stark_prove_device", "zkb_stark_prove_host", "zkb_stark_prove_multi_device", "zkb_stark_prove_multi_host", "zkb_gkr_prove_device",
                  "zkb_shard_pcs_begin", "zkb_shard_pcs_extend", "zkb_shard_pcs_set_rows", "zkb_shard_pcs_set_peer_rows", "zkb_shard_pcs_extend_begin", "zkb_shard_pcs_extend_chunk", "zkb_shard_pcs_subtree", "zkb_shard_pcs_sample", "zkb_shard_pcs_quotients",
                  "zkb_shard_pcs_fri_and_decommit", "zkb_shard_pcs_finish", "zkb_shard_pcs_end"]
# Every symbol include/zkb200_air.h declares.
AIR_SYMBOLS = ["zkb_air_compile", "zkb_air_analyze", "zkb_air_free", "zkb_air_specialize", "zkb_air_select", "zkb_air_get_stats", "zkb_constraint_quotients", "zkb_constraint_denom_inv"]
PCS_PHASES = ["interpolate", "extend", "merkle", "sample", "quotients", "fri_commit", "grind", "decommit"]


class Grid(C.Structure):
    _fields_ = [("log_rows", C.c_uint32), ("groups", C.c_uint32), ("chunks", C.c_uint32), ("lead", C.c_uint32)]


DEQUANT_CFG_FIELDS = ("variant", "sticky", "kmax", "do_ref", "tokens", "n_out", "per_row", "chunks", "log_rows", "slot0", "per_slot", "chan_w",
                      "f_acc", "f_sg", "f_m2", "f_ph", "f_st", "f_r", "f_m7", "f_ef", "f_nz", "f_eo", "f_mul0", "f_mul1", "f_mul2", "f_mul3",
                      "f_mul4", "f_mul5", "sh0", "sh1", "n_norm", "n_frac", "n_mul", "n_r8")


class DequantCfg(C.Structure):
    """zkb_dequant_cfg (f_mul[6] spelled as six fields)."""
    _fields_ = [(k, C.c_uint32) for k in DEQUANT_CFG_FIELDS]


class RsProgram(C.Structure):  # zkb_rs_program
    _fields_ = [("groups", C.c_void_p), ("n_groups", C.c_uint32), ("slots", C.c_void_p), ("n_slots", C.c_uint32), ("out_slot", C.c_void_p),
                ("out_w", C.c_uint32), ("kind", C.c_uint32), ("sticky", C.c_uint32), ("kmax", C.c_uint32)]


class RsTables(C.Structure):  # zkb_rs_tables
    _fields_ = [("norm3", C.c_void_p), ("n_norm", C.c_uint32), ("smul3", C.c_void_p), ("n_smul", C.c_uint32), ("un2", C.c_void_p),
                ("n_un", C.c_uint32), ("n_val", C.c_uint32)]


class RsMult(C.Structure):  # zkb_rs_mult
    _fields_ = [("m", C.c_void_p), ("n", C.c_uint32)]


class RsMults(C.Structure):  # zkb_rs_mults
    _fields_ = [("pow", RsMult), ("norm", RsMult), ("val", RsMult), ("frac", RsMult), ("smul", RsMult), ("un", C.c_void_p)]


class PcsConfig(C.Structure):
    _fields_ = [("pow_bits", C.c_uint32), ("log_blowup_factor", C.c_uint32), ("log_last_layer_degree_bound", C.c_uint32),
                ("n_queries", C.c_uint32)]



class AirStats(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_ops", "n_live_ops", "n_uniform", "n_instr", "n_loads", "n_columns_read", "reg_words",
                                          "uniform_words", "threads", "rows_per_thread", "smem_bytes", "m31_mults", "specialized", "specialized_regs")]


class StarkComponent(C.Structure):
    _fields_ = [("prog", C.c_void_p), ("trace_log", C.c_uint32), ("scalars", C.c_void_p), ("claimed_sum", C.c_void_p)]


class ZkbError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"zkb200 error {code}: {msg}")
        self.code = code


def lib_path():
    return _LIB


_lib = None


def load_library():
    """Loads libzkb200.so. Raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            raise ImportError(
                f"{_LIB} is missing: build it with `python -m zk_inference_prover_b200.build` "
                "(nvcc, sm_100a). zkb200 has no CPU fallback."
            )
        _lib = C.CDLL(_LIB)
        _lib.zkb_last_error.restype = C.c_char_p
        _lib.zkb_last_error.argtypes = [C.c_void_p]
        _lib.zkb_gkr_sum_noalloc_error.restype = C.c_char_p
        for name in EXPORTED_SYMBOLS + PROVER_SYMBOLS + AIR_SYMBOLS:
            if name not in ("zkb_last_error", "zkb_gkr_sum_noalloc_error"):
                getattr(_lib, name).restype = C.c_int
    return _lib


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def gkr_sum_noalloc(device, stream, kind, num_ptr, den_ptr, n, eq_ptr, lam, out_ptr):
    """zkb_gkr_sum_noalloc: needs no Context; the 8 result words land in device memory at out_ptr."""
    lib = load_library()
    l = _u32(lam)
    rc = lib.zkb_gkr_sum_noalloc(C.c_int(device), C.c_void_p(stream or None), C.c_int(kind), C.c_void_p(num_ptr or None), C.c_void_p(den_ptr),
                                 C.c_size_t(n), C.c_void_p(eq_ptr), l.ctypes.data_as(C.c_void_p), C.c_void_p(out_ptr))
    if rc != 0:
        raise ZkbError(rc, lib.zkb_gkr_sum_noalloc_error().decode())


class ShardPcsSession:
    """One rank's side of a PCS proof over several devices (include/zkb200_prover.h, zkb_shard_pcs_*). Every method is one
    stage; the caller performs the exchange the stage's docstring names before calling the next one."""

    def __init__(self, ctx, rank, world, ncols_total, log_n, cfg):
        self.ctx, self.rank, self.world, self.ncols, self.log_n = ctx, rank, world, ncols_total, log_n
        self.ncl = ncols_total // world
        self.log_out = log_n + cfg.log_blowup_factor
        self.N = 1 << self.log_out
        self.R = self.N // world
        self.h = C.c_void_p()
        self._cfg = cfg
        ctx._check(ctx.lib.zkb_shard_pcs_begin(ctx.h, C.c_int(rank), C.c_int(world), C.c_int(ncols_total), C.c_int(log_n), C.byref(cfg),
                                               C.byref(self.h)))

    def extend(self, col_ptrs):
        """-> (send address, rows address), both [world][ncl][R]. Then: one all-to-all, block d of `send` becomes block `rank`
        of rank d's `rows`."""
        e, r = C.c_void_p(), C.c_void_p()
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_extend(self.h, _ptr_array(col_ptrs), C.byref(e), C.byref(r)))
        return e.value, r.value

    def set_rows(self, rows_ptr):
        """The buffer the row shards are received into (ncols x R words); must outlive the session."""
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_set_rows(self.h, C.c_void_p(rows_ptr)))

    def set_peer_rows(self, peer_ptrs):
        """Every rank's receive buffer as this process sees it: the chunks' blocks are then copied there by extend_chunk."""
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_set_peer_rows(self.h, _ptr_array(peer_ptrs)))

    def extend_begin(self, col_ptrs, n_chunks):
        """The extend stage by chunks of columns (n_chunks must divide ncl): interpolates; then call extend_chunk(k) for every k."""
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_extend_begin(self.h, _ptr_array(col_ptrs), C.c_int(n_chunks)))

    def extend_chunk(self, k):
        """-> (send address, receive address, words per peer) of chunk k, both [world][ncl / n_chunks][R]. Then: one all-to-all
        of the chunk (it may run while the next chunk is extended; the subtree stage must come after all of them)."""
        e, r, w = C.c_void_p(), C.c_void_p(), C.c_size_t()
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_extend_chunk(self.h, C.c_int(k), C.byref(e), C.byref(r), C.byref(w)))
        return e.value, r.value, int(w.value)

    def subtree(self):
        """-> (root address (8 words), roots address [world][8]). Then: all-gather the roots."""
        a, b = C.c_void_p(), C.c_void_p()
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_subtree(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def sample(self):
        """-> this rank's sampled values [ncl][4] (host). Then: all-gather them in rank order."""
        out = np.empty((self.ncl, 4), np.uint32)
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_sample(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def quotients(self, all_samples):
        """-> (addresses of the 4 local coordinate columns (R words), of the 4 full ones (N words)). Then: all-gather each."""
        a = _u32(all_samples).reshape(-1)
        loc, full = (C.c_void_p * 4)(), (C.c_void_p * 4)()
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_quotients(self.h, a.ctypes.data_as(C.c_void_p), loc, full))
        return [loc[k] for k in range(4)], [full[k] for k in range(4)]

    def fri_and_decommit(self, cap=1 << 22):
        """-> this rank's part of the decommitment (host words). Then: gather the parts on the finishing rank."""
        out = np.empty(cap, np.uint32)
        n = C.c_size_t()
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_fri_and_decommit(self.h, out.ctypes.data_as(C.c_void_p), C.c_size_t(cap), C.byref(n)))
        return out[: n.value].copy()

    def finish(self, parts, cap=1 << 24):
        """parts: every rank's part, in rank order -> proof words (with the channel digest appended)."""
        keep = [_u32(p) for p in parts]
        ptrs = (C.c_void_p * len(keep))(*[k.ctypes.data for k in keep])
        sizes = (C.c_size_t * len(keep))(*[len(k) for k in keep])
        out = np.empty(cap, np.uint32)
        n = C.c_size_t()
        self.ctx._check(self.ctx.lib.zkb_shard_pcs_finish(self.h, ptrs, sizes, out.ctypes.data_as(C.c_void_p), C.c_size_t(cap), C.byref(n)))
        return out[: n.value].copy()

    def close(self):
        if self.h:
            self.ctx.lib.zkb_shard_pcs_end(self.h)
            self.h = C.c_void_p()


class DeviceBuffer:
    """A device allocation of `words` uint32, owned by this object."""

    def __init__(self, ctx, words):
        self.ctx = ctx
        self.words = int(words)
        p = C.c_void_p()
        ctx._check(ctx.lib.zkb_malloc(ctx.h, C.c_size_t(self.words * 4), C.byref(p)))
        self.ptr = p.value or 0

    def free(self):
        if self.ptr:
            self.ctx.lib.zkb_free(self.ctx.h, C.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def upload(self, arr):
        a = _u32(arr).reshape(-1)
        assert a.size <= self.words
        self.ctx._check(self.ctx.lib.zkb_h2d(self.ctx.h, C.c_void_p(self.ptr), a.ctypes.data_as(C.c_void_p), C.c_size_t(a.size * 4)))
        return self

    def download(self, words=None, shape=None):
        n = self.words if words is None else int(words)
        out = np.empty(n, np.uint32)
        self.ctx._check(self.ctx.lib.zkb_d2h(self.ctx.h, out.ctypes.data_as(C.c_void_p), C.c_void_p(self.ptr), C.c_size_t(n * 4)))
        return out if shape is None else out.reshape(shape)

    def zero(self):
        self.ctx._check(self.ctx.lib.zkb_memset_zero(self.ctx.h, C.c_void_p(self.ptr), C.c_size_t(self.words * 4)))
        return self

    def view(self, offset_words):
        """Raw device address `offset_words` into the buffer."""
        return self.ptr + 4 * int(offset_words)


def _ptr_array(ptrs):
    return (C.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def constraint_denom_inv(trace_log, eval_log):
    """zkb_constraint_denom_inv: host only."""
    out = np.empty(1 << (eval_log - trace_log), np.uint32)
    rc = load_library().zkb_constraint_denom_inv(C.c_int(trace_log), C.c_int(eval_log), out.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise ZkbError(rc, "zkb_constraint_denom_inv: invalid sizes")
    return out


def air_analyze(source, check_specialized=False):
    """zkb_air_analyze: the compiler's report on a program (host only, no GPU). Raises ZkbError with its reason if refused."""
    ops, cons, trees = _u32(source.ops), _u32(source.constraints), _u32(source.tree_cols)
    st = AirStats()
    err = C.create_string_buffer(1024)
    rc = load_library().zkb_air_analyze(ops.ctypes.data_as(C.c_void_p), C.c_size_t(ops.shape[0]), cons.ctypes.data_as(C.c_void_p),
                                        C.c_size_t(cons.size), trees.ctypes.data_as(C.c_void_p), C.c_int(trees.size),
                                        C.c_size_t(source.scalars.shape[0]), C.c_int(int(check_specialized)), C.byref(st), err,
                                        C.c_size_t(1024))
    if rc != 0:
        raise ZkbError(rc, err.value.decode())
    return {n: getattr(st, n) for n, _ in AirStats._fields_}


class AirProgram:
    """A compiled AIR (zkb_air_program), owned by this object."""

    def __init__(self, ctx, source):
        self.ctx, self.source = ctx, source
        ops, cons, trees = _u32(source.ops), _u32(source.constraints), _u32(source.tree_cols)
        h = C.c_void_p()
        ctx._check(ctx.lib.zkb_air_compile(ctx.h, ops.ctypes.data_as(C.c_void_p), C.c_size_t(ops.shape[0]), cons.ctypes.data_as(C.c_void_p),
                                           C.c_size_t(cons.size), trees.ctypes.data_as(C.c_void_p), C.c_int(trees.size),
                                           C.c_size_t(source.scalars.shape[0]), C.byref(h)))
        self.h = h

    @property
    def stats(self):
        st = AirStats()
        self.ctx._check(self.ctx.lib.zkb_air_get_stats(self.h, C.byref(st)))
        return {n: getattr(st, n) for n, _ in AirStats._fields_}

    def specialize(self):
        """zkb_air_specialize: compile a kernel for this program with NVRTC and use it from now on."""
        self.ctx._check(self.ctx.lib.zkb_air_specialize(self.ctx.h, self.h))
        return self

    def select(self, specialized):
        if self.ctx.lib.zkb_air_select(self.h, C.c_int(int(specialized))) != 0:
            raise ZkbError(-1, "zkb_air_select: the program has no specialised kernel")
        return self

    def free(self):
        if getattr(self, "h", None):
            self.ctx.lib.zkb_air_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Context:
    """A zkb_ctx: one device, one stream, the twiddle tower up to `max_log_size`."""

    def __init__(self, device=0, max_log_size=20):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.zkb_init(C.c_int(device), C.c_int(max_log_size), C.byref(h))
        if rc != 0:
            raise ZkbError(rc, "zkb_init failed (is a CUDA device visible?)")
        self.h = h
        self.max_log_size = max_log_size

    def close(self):
        if getattr(self, "h", None):
            self.lib.zkb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != 0:
            raise ZkbError(rc, self.lib.zkb_last_error(self.h).decode())

    # ---- memory
    def alloc(self, words):
        return DeviceBuffer(self, words)

    def upload(self, arr):
        a = _u32(arr)
        return DeviceBuffer(self, a.size).upload(a)

    def upload_bytes(self, arr):
        """Any contiguous host array, byte for byte, into a fresh device buffer (rounded up to words)."""
        a = np.ascontiguousarray(arr)
        buf = DeviceBuffer(self, (a.nbytes + 3) // 4)
        self._check(self.lib.zkb_h2d(self.h, C.c_void_p(buf.ptr), a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes)))
        return buf

    def sync(self):
        self._check(self.lib.zkb_sync(self.h))

    def event_record(self, slot):
        self._check(self.lib.zkb_event_record(self.h, C.c_int(slot)))

    def event_elapsed_ms(self, a, b):
        ms = C.c_float()
        self._check(self.lib.zkb_event_elapsed_ms(self.h, C.c_int(a), C.c_int(b), C.byref(ms)))
        return ms.value

    def profile_begin(self):
        self._check(self.lib.zkb_profile_begin(self.h))

    def profile_end(self, cap=64):
        """{kernel name: (total ms, launches)} since profile_begin."""
        names = (C.c_char_p * cap)()
        ms = (C.c_float * cap)()
        cnt = (C.c_int * cap)()
        n = C.c_int()
        self._check(self.lib.zkb_profile_end(self.h, names, ms, cnt, C.c_int(cap), C.byref(n)))
        return {names[i].decode(): (ms[i], cnt[i]) for i in range(n.value)}

    def barycentric_weights(self, log_size, point8):
        """-> DeviceBuffer of 2^log_size QM31 weights."""
        out = self.alloc(4 << log_size)
        self._check(self.lib.zkb_barycentric_weights(self.h, C.c_int(log_size), _u32(point8).ctypes.data_as(C.c_void_p), C.c_void_p(out.ptr)))
        return out

    def barycentric_eval_at_point(self, evals_ptr, weights_ptr, log_size):
        o = np.zeros(4, np.uint32)
        self._check(self.lib.zkb_barycentric_eval_at_point(self.h, C.c_void_p(evals_ptr), C.c_void_p(weights_ptr), C.c_int(log_size),
                                                           o.ctypes.data_as(C.c_void_p)))
        return o

    def eval_at_point_by_folding(self, evals_ptr, log_size, point8):
        o = np.zeros(4, np.uint32)
        self._check(self.lib.zkb_eval_at_point_by_folding(self.h, C.c_void_p(evals_ptr), C.c_int(log_size),
                                                          _u32(point8).ctypes.data_as(C.c_void_p), o.ctypes.data_as(C.c_void_p)))
        return o

    def fft_arith_ceiling(self):
        """Butterflies per second of the register-only butterfly kernel (the ceiling of the FFT passes)."""
        v = C.c_double()
        self._check(self.lib.zkb_fft_arith_ceiling(self.h, C.byref(v)))
        return v.value

    def alloc_pinned(self, words):
        """Pinned host memory as a numpy uint32 array (freed with free_pinned)."""
        p = C.c_void_p()
        self._check(self.lib.zkb_host_alloc_pinned(self.h, C.c_size_t(int(words) * 4), C.byref(p)))
        arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint32)), shape=(int(words),))
        return arr, p.value

    def free_pinned(self, addr):
        self._check(self.lib.zkb_host_free_pinned(self.h, C.c_void_p(addr)))

    def h2d_async(self, dptr, host_addr, nbytes):
        self._check(self.lib.zkb_h2d_async(self.h, C.c_void_p(dptr), C.c_void_p(host_addr), C.c_size_t(nbytes)))

    def d2h_async(self, host_addr, dptr, nbytes):
        self._check(self.lib.zkb_d2h_async(self.h, C.c_void_p(host_addr), C.c_void_p(dptr), C.c_size_t(nbytes)))

    def peer_buffer_alloc(self, nbytes):
        """-> (device address, 64-byte handle as uint8 array)."""
        p, h = C.c_void_p(), (C.c_ubyte * 64)()
        self._check(self.lib.zkb_peer_buffer_alloc(self.h, C.c_size_t(nbytes), C.byref(p), h))
        return p.value, np.frombuffer(bytes(h), np.uint8).copy()

    def peer_buffer_free(self, ptr):
        self._check(self.lib.zkb_peer_buffer_free(self.h, C.c_void_p(ptr)))

    def peer_buffer_open(self, handle):
        p = C.c_void_p()
        hb = (C.c_ubyte * 64)(*[int(b) for b in handle])
        self._check(self.lib.zkb_peer_buffer_open(self.h, hb, C.byref(p)))
        return p.value

    def peer_buffer_close(self, ptr):
        self._check(self.lib.zkb_peer_buffer_close(self.h, C.c_void_p(ptr)))

    def copy_to_peer(self, dst, src, nbytes, lane=0):
        self._check(self.lib.zkb_copy_to_peer(self.h, C.c_void_p(dst), C.c_void_p(src), C.c_size_t(nbytes), C.c_int(lane)))

    def peer_copies_wait(self):
        self._check(self.lib.zkb_peer_copies_wait(self.h))

    def d2d(self, dst, src, nbytes):
        self._check(self.lib.zkb_d2d(self.h, C.c_void_p(dst), C.c_void_p(src), C.c_size_t(nbytes)))

    def stream(self):
        s = C.c_void_p()
        self._check(self.lib.zkb_get_stream(self.h, C.byref(s)))
        return s.value or 0

    def gather_multi(self, col_ptrs, idx):
        idx = _u32(idx)
        out = np.empty((len(idx), len(col_ptrs)), np.uint32)
        self._check(self.lib.zkb_gather_multi(self.h, _ptr_array(col_ptrs), C.c_int(len(col_ptrs)), idx.ctypes.data_as(C.c_void_p),
                                              C.c_int(len(idx)), out.ctypes.data_as(C.c_void_p)))
        return out

    def gather_hashes(self, hashes_ptr, idx):
        idx = _u32(idx)
        out = np.empty((len(idx), 8), np.uint32)
        self._check(self.lib.zkb_gather_hashes(self.h, C.c_void_p(hashes_ptr), idx.ctypes.data_as(C.c_void_p), C.c_int(len(idx)),
                                               out.ctypes.data_as(C.c_void_p)))
        return out

    def gather_words(self, addrs):
        a = np.ascontiguousarray(addrs, dtype=np.uint64)
        out = np.empty(len(a), np.uint32)
        self._check(self.lib.zkb_gather_words(self.h, a.ctypes.data_as(C.c_void_p), C.c_size_t(len(a)), out.ctypes.data_as(C.c_void_p)))
        return out

    # ---- twiddles
    def twiddles(self, log_size):
        tw = np.empty(1 << log_size, np.uint32)
        itw = np.empty(1 << log_size, np.uint32)
        self._check(self.lib.zkb_twiddles_d2h(self.h, C.c_int(log_size), tw.ctypes.data_as(C.c_void_p), itw.ctypes.data_as(C.c_void_p)))
        return tw, itw

    # ---- PolyOps
    def ifft_cols(self, col_ptrs, log_n):
        self._check(self.lib.zkb_ifft_cols(self.h, _ptr_array(col_ptrs), C.c_int(len(col_ptrs)), C.c_int(log_n)))

    def lde_cols(self, coeff_ptrs, log_n, out_ptrs, log_out):
        self._check(self.lib.zkb_lde_cols(self.h, _ptr_array(coeff_ptrs), C.c_int(len(coeff_ptrs)), C.c_int(log_n),
                                          _ptr_array(out_ptrs), C.c_int(log_out)))

    def eval_at_point_cols(self, coeff_ptrs, log_n, point8):
        pt = _u32(point8)
        out = np.empty((len(coeff_ptrs), 4), np.uint32)
        self._check(self.lib.zkb_eval_at_point_cols(self.h, _ptr_array(coeff_ptrs), C.c_int(len(coeff_ptrs)), C.c_int(log_n),
                                                    pt.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)))
        return out

    def bit_reverse_m31(self, ptr, log_n):
        self._check(self.lib.zkb_bit_reverse_m31(self.h, C.c_void_p(ptr), C.c_int(log_n)))

    def bit_reverse_qm31(self, ptr, log_n):
        self._check(self.lib.zkb_bit_reverse_qm31(self.h, C.c_void_p(ptr), C.c_int(log_n)))

    # ---- MerkleOps
    def merkle_layer(self, log_size, prev_ptr, col_ptrs, out_ptr, m31_out=True):
        self._check(self.lib.zkb_merkle_layer(self.h, C.c_int(log_size), C.c_void_p(prev_ptr or None), _ptr_array(col_ptrs),
                                              C.c_int(len(col_ptrs)), C.c_int(int(m31_out)), C.c_void_p(out_ptr)))

    def merkle_leaves_partial(self, log_size, col_ptrs, cols_before, total_cols, out_ptr, m31_out=True):
        arr = (C.c_void_p * len(col_ptrs))(*col_ptrs)
        self._check(self.lib.zkb_merkle_leaves_partial(self.h, C.c_int(log_size), arr, C.c_int(len(col_ptrs)), C.c_int(cols_before),
                                                       C.c_int(total_cols), C.c_int(1 if m31_out else 0), C.c_void_p(out_ptr)))

    def merkle_levels(self, child_log, children_ptr, out_ptrs, m31_out=True):
        self._check(self.lib.zkb_merkle_levels(self.h, C.c_int(child_log), C.c_void_p(children_ptr), C.c_int(len(out_ptrs)), _ptr_array(out_ptrs),
                                               C.c_int(int(m31_out))))

    def merkle_top(self, top_log, top_ptr, lower_ptrs, m31_out=True):
        self._check(self.lib.zkb_merkle_top(self.h, C.c_int(top_log), C.c_void_p(top_ptr), _ptr_array(lower_ptrs), C.c_int(int(m31_out))))

    # ---- FriOps
    def fold_line(self, out4, in4, log_n, alpha):
        a = _u32(alpha)
        self._check(self.lib.zkb_fold_line(self.h, _ptr_array(out4), _ptr_array(in4), C.c_int(log_n), a.ctypes.data_as(C.c_void_p)))

    def fold_circle_into_line(self, dst4, src4, log_n_src, alpha):
        a = _u32(alpha)
        self._check(self.lib.zkb_fold_circle_into_line(self.h, _ptr_array(dst4), _ptr_array(src4), C.c_int(log_n_src),
                                                       a.ctypes.data_as(C.c_void_p)))

    def fold_line_dalpha(self, out4, in4, log_n, d_alpha):
        self._check(self.lib.zkb_fold_line_dalpha(self.h, _ptr_array(out4), _ptr_array(in4), C.c_int(log_n), C.c_void_p(d_alpha)))

    def fold_circle_into_line_dalpha(self, dst4, src4, log_n_src, d_alpha):
        self._check(self.lib.zkb_fold_circle_into_line_dalpha(self.h, _ptr_array(dst4), _ptr_array(src4), C.c_int(log_n_src),
                                                              C.c_void_p(d_alpha)))

    def fold_line_dalpha_leaves(self, out4, in4, log_n, d_alpha, leaves_ptr):
        self._check(self.lib.zkb_fold_line_dalpha_leaves(self.h, _ptr_array(out4), _ptr_array(in4), C.c_int(log_n), C.c_void_p(d_alpha),
                                                         C.c_void_p(leaves_ptr)))

    def fold_circle_into_line_dalpha_leaves(self, dst4, src4, log_n_src, d_alpha, leaves_ptr):
        self._check(self.lib.zkb_fold_circle_into_line_dalpha_leaves(self.h, _ptr_array(dst4), _ptr_array(src4), C.c_int(log_n_src),
                                                                     C.c_void_p(d_alpha), C.c_void_p(leaves_ptr)))

    def channel_mix_root_draw(self, d_chan, d_root, d_alpha, d_root_copy=0):
        self._check(self.lib.zkb_channel_mix_root_draw(self.h, C.c_void_p(d_chan), C.c_void_p(d_root), C.c_void_p(d_alpha),
                                                       C.c_void_p(d_root_copy or None)))

    # ---- QuotientOps / AccumulationOps
    def quot_numerators(self, col_ptrs, log_n, col_idx, b, c, out4):
        ci, bb, cc = _u32(col_idx), _u32(b), _u32(c)
        self._check(self.lib.zkb_quot_numerators(self.h, _ptr_array(col_ptrs), C.c_int(len(col_ptrs)), C.c_int(log_n),
                                                 ci.ctypes.data_as(C.c_void_p), bb.ctypes.data_as(C.c_void_p),
                                                 cc.ctypes.data_as(C.c_void_p), C.c_int(len(ci)), _ptr_array(out4)))

    def quot_combine(self, acc_ptrs, acc_logs, first_lin, points, lifting_log, out4):
        logs = np.ascontiguousarray(acc_logs, dtype=np.int32)
        fl, pts = _u32(first_lin), _u32(points)
        self._check(self.lib.zkb_quot_combine(self.h, C.c_int(len(logs)), _ptr_array(acc_ptrs), logs.ctypes.data_as(C.c_void_p),
                                              fl.ctypes.data_as(C.c_void_p), pts.ctypes.data_as(C.c_void_p), C.c_int(lifting_log),
                                              _ptr_array(out4)))

    def accumulate(self, col4, other4, n):
        self._check(self.lib.zkb_accumulate(self.h, _ptr_array(col4), _ptr_array(other4), C.c_size_t(n)))

    def lift_accumulate(self, dst4, log_dst, src4, log_src):
        self._check(self.lib.zkb_lift_accumulate(self.h, _ptr_array(dst4), C.c_int(log_dst), _ptr_array(src4), C.c_int(log_src)))

    def secure_powers(self, felt4, n):
        f = _u32(felt4)
        out = np.empty((n, 4), np.uint32)
        self._check(self.lib.zkb_secure_powers(self.h, f.ctypes.data_as(C.c_void_p), C.c_size_t(n), out.ctypes.data_as(C.c_void_p)))
        return out

    # ---- GkrOps / MleOps
    def gkr_eq_evals(self, y, v4, out_ptr):
        yy, v = _u32(y).reshape(-1, 4), _u32(v4)
        self._check(self.lib.zkb_gkr_eq_evals(self.h, yy.ctypes.data_as(C.c_void_p), C.c_int(yy.shape[0]), v.ctypes.data_as(C.c_void_p),
                                              C.c_void_p(out_ptr)))

    def gkr_next_layer(self, kind, num_ptr, den_ptr, n, num_out_ptr, den_out_ptr):
        self._check(self.lib.zkb_gkr_next_layer(self.h, C.c_int(kind), C.c_void_p(num_ptr or None), C.c_void_p(den_ptr), C.c_size_t(n),
                                                C.c_void_p(num_out_ptr or None), C.c_void_p(den_out_ptr)))

    def gkr_sum(self, kind, num_ptr, den_ptr, n, eq_ptr, lam):
        l = _u32(lam)
        out = np.empty(8, np.uint32)
        self._check(self.lib.zkb_gkr_sum(self.h, C.c_int(kind), C.c_void_p(num_ptr or None), C.c_void_p(den_ptr), C.c_size_t(n),
                                         C.c_void_p(eq_ptr), l.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)))
        return out.reshape(2, 4)

    def gkr_fix_and_sum(self, kind, num_ptr, den_ptr, n, r, eq_ptr, lam, num_out_ptr, den_out_ptr):
        rr, l = _u32(r), _u32(lam)
        out = np.empty(8, np.uint32)
        self._check(self.lib.zkb_gkr_fix_and_sum(self.h, C.c_int(kind), C.c_void_p(num_ptr or None), C.c_void_p(den_ptr), C.c_size_t(n),
                                                 rr.ctypes.data_as(C.c_void_p), C.c_void_p(eq_ptr), l.ctypes.data_as(C.c_void_p),
                                                 C.c_void_p(num_out_ptr or None), C.c_void_p(den_out_ptr), out.ctypes.data_as(C.c_void_p)))
        return out.reshape(2, 4)

    def mle_fix_qm31(self, in_ptr, n, r, out_ptr):
        rr = _u32(r)
        self._check(self.lib.zkb_mle_fix_qm31(self.h, C.c_void_p(in_ptr), C.c_size_t(n), rr.ctypes.data_as(C.c_void_p), C.c_void_p(out_ptr)))

    def mle_fix_m31(self, in_ptr, n, r, out_ptr):
        rr = _u32(r)
        self._check(self.lib.zkb_mle_fix_m31(self.h, C.c_void_p(in_ptr), C.c_size_t(n), rr.ctypes.data_as(C.c_void_p), C.c_void_p(out_ptr)))

    # ---- Freivalds component
    def freivalds_scatter(self, qx_ptr, qw_ptrs, n_out, grid, pq, pk, n_in, tokens, base_ptrs, pre_ptrs, m_r8_ptr, table_len, off_ptr):
        g = Grid(*grid)
        no = _u32(n_out)
        self._check(self.lib.zkb_freivalds_scatter(self.h, C.c_void_p(qx_ptr), _ptr_array(qw_ptrs), no.ctypes.data_as(C.c_void_p), C.byref(g),
                                                   C.c_uint32(pq), C.c_uint32(pk), C.c_uint32(n_in), C.c_uint32(tokens), C.c_uint32(len(qw_ptrs)),
                                                   _ptr_array(base_ptrs), _ptr_array(pre_ptrs), C.c_void_p(m_r8_ptr), C.c_uint32(table_len),
                                                   C.c_void_p(off_ptr)))

    def freivalds_acc(self, base_ptrs, pre_ptrs, grid, pq, pk, n_mats, s4, rv4, out_ptrs):
        g = Grid(*grid)
        s, r = _u32(s4), _u32(rv4)
        claims = np.empty((n_mats, 4), np.uint32)
        self._check(self.lib.zkb_freivalds_acc(self.h, _ptr_array(base_ptrs), _ptr_array(pre_ptrs), C.byref(g), C.c_uint32(pq), C.c_uint32(pk),
                                               C.c_uint32(n_mats), s.ctypes.data_as(C.c_void_p), r.ctypes.data_as(C.c_void_p),
                                               _ptr_array(out_ptrs), claims.ctypes.data_as(C.c_void_p)))
        return claims

    # ---- witness generation: the tables' own columns and the dequantize component
    def witness_tables(self, expmap_ptr, counter_ptrs, log_rows, bf16x, two_pow, x_ptr, y_ptr, m_ptr, patch_idx_ptr=0, patch_val_ptr=0, n_patch=0):
        self._check(self.lib.zkb_witness_tables(self.h, C.c_void_p(expmap_ptr), _ptr_array(counter_ptrs) if counter_ptrs else None,
                                                C.c_uint32(len(counter_ptrs)), C.c_void_p(patch_idx_ptr or None), C.c_void_p(patch_val_ptr or None),
                                                C.c_uint32(n_patch), C.c_uint32(log_rows), C.c_int(int(bf16x)), C.c_double(two_pow),
                                                C.c_void_p(x_ptr), C.c_void_p(y_ptr), C.c_void_p(m_ptr or None)))

    def witness_dequant(self, cfg, acc_ptr, jx_ptr, jw_ptr, sx_ptr, sw_ptr, norm3_ptr, mul2_ptr, base_ptrs, pre_ptrs, m_norm_ptr, m_frac_ptr,
                        m_mul_ptr, m_r8_ptr, counts_ptr, want_ptr=0):
        """cfg: dict over DEQUANT_CFG_FIELDS."""
        c = DequantCfg(*[int(cfg[k]) for k in DEQUANT_CFG_FIELDS])
        vp = lambda p: C.c_void_p(p or None)
        self._check(self.lib.zkb_witness_dequant(self.h, vp(acc_ptr), vp(jx_ptr), vp(jw_ptr), vp(sx_ptr), vp(sw_ptr), vp(norm3_ptr), vp(mul2_ptr),
                                                 _ptr_array(base_ptrs), C.c_uint32(len(base_ptrs)), _ptr_array(pre_ptrs),
                                                 C.c_uint32(len(pre_ptrs)), vp(m_norm_ptr), vp(m_frac_ptr), vp(m_mul_ptr), vp(m_r8_ptr),
                                                 vp(counts_ptr), vp(want_ptr), C.byref(c)))

    def witness_pre_table(self, kind, log_rows, kmax, round_mode, counter_ptrs, col_ptrs, m_ptr=0, patch_idx_ptr=0, patch_val_ptr=0, n_patch=0):
        self._check(self.lib.zkb_witness_pre_table(self.h, C.c_uint32(kind), C.c_uint32(log_rows), C.c_uint32(kmax), C.c_uint32(round_mode),
                                                   _ptr_array(counter_ptrs) if counter_ptrs else None, C.c_uint32(len(counter_ptrs)),
                                                   C.c_void_p(patch_idx_ptr or None), C.c_void_p(patch_val_ptr or None), C.c_uint32(n_patch),
                                                   _ptr_array(col_ptrs), C.c_uint32(len(col_ptrs)), C.c_void_p(m_ptr or None)))

    def key_tile_flags(self, shape, log_rows, groups, chunks, lead, descending, modulus, rw, flags_ptr):
        self._check(self.lib.zkb_key_tile_flags(self.h, *(C.c_uint32(int(v)) for v in (shape, log_rows, groups, chunks, lead, descending, modulus, rw)),
                                                C.c_void_p(flags_ptr)))

    def witness_selectors(self, shape, log_rows, groups, chunks, lead, descending, flags_ptr, scale_ptr, ctx_len, n_insts, with_scale, col_ptrs):
        self._check(self.lib.zkb_witness_selectors(self.h, *(C.c_uint32(int(v)) for v in (shape, log_rows, groups, chunks, lead, descending)),
                                                   C.c_void_p(flags_ptr), C.c_void_p(scale_ptr or None), C.c_uint32(ctx_len), C.c_uint32(n_insts),
                                                   C.c_int(int(with_scale)), _ptr_array(col_ptrs), C.c_uint32(len(col_ptrs))))

    def witness_residual_stream(self, groups, slots, out_slot, kind, sticky, kmax, norm3_ptr, n_norm, smul3_ptr, n_smul, un2_ptrs, n_val, wit_ptr,
                                live_rows, log_rows, col_ptrs, out_pat_ptr, out_nat_ptr, in_nat_ptr, mults, un_mults, counts_ptr):
        """groups [n, 5] / slots [n, 8] / out_slot: host uint32 arrays (zkb_rs_group, zkb_rs_slot records). mults: dict name -> (ptr, n)
        over pow, norm, val, frac, smul; un_mults: list of (ptr, n)."""
        groups = np.ascontiguousarray(groups, np.uint32).reshape(-1, 5)
        slots = np.ascontiguousarray(slots, np.uint32).reshape(-1, 8)
        out_slot = np.ascontiguousarray(out_slot, np.uint32)
        prog = RsProgram(groups.ctypes.data, len(groups), slots.ctypes.data if len(slots) else None, len(slots),
                         out_slot.ctypes.data if len(out_slot) else None, len(out_slot), int(kind), int(sticky), int(kmax))
        un2 = _ptr_array(un2_ptrs) if un2_ptrs else None
        tables = RsTables(norm3_ptr or None, n_norm, smul3_ptr or None, n_smul, C.cast(un2, C.c_void_p) if un2_ptrs else None, len(un2_ptrs), n_val)
        un_arr = (RsMult * max(1, len(un_mults)))(*[RsMult(p, n) for p, n in un_mults])
        m = RsMults(*[RsMult(mults[k][0] or None, mults[k][1]) for k in ("pow", "norm", "val", "frac", "smul")],
                    C.cast(un_arr, C.c_void_p) if un_mults else None)
        self._check(self.lib.zkb_witness_residual_stream(self.h, C.byref(prog), C.byref(tables), C.c_void_p(wit_ptr), C.c_uint32(live_rows),
                                                         C.c_uint32(log_rows), _ptr_array(col_ptrs), C.c_uint32(len(col_ptrs)),
                                                         C.c_void_p(out_pat_ptr), C.c_void_p(out_nat_ptr), C.c_void_p(in_nat_ptr), C.byref(m),
                                                         C.c_void_p(counts_ptr)))

    # ---- constraint quotients of a lowered AIR (include/zkb200_air.h)
    def air_compile(self, source):
        """source: an air.AirSource. Returns an AirProgram bound to this context's device."""
        return AirProgram(self, source)

    def constraint_quotients(self, prog, col_ptrs, random_coeff_powers, trace_log, eval_log, accum4, accumulate=True, scalars=None,
                             cumsum_shift=None, denom_inv=None):
        sc = _u32(prog.source.scalars if scalars is None else scalars)
        rcp = _u32(random_coeff_powers)
        assert rcp.size == 4 * prog.source.n_constraints and sc.size == prog.source.scalars.size
        di = _u32(constraint_denom_inv(trace_log, eval_log) if denom_inv is None else denom_inv)
        shift = _u32(cumsum_shift) if cumsum_shift is not None else None
        self._check(self.lib.zkb_constraint_quotients(self.h, prog.h, _ptr_array(col_ptrs), sc.ctypes.data_as(C.c_void_p),
                                                      shift.ctypes.data_as(C.c_void_p) if shift is not None else None,
                                                      rcp.ctypes.data_as(C.c_void_p), di.ctypes.data_as(C.c_void_p), C.c_int(trace_log),
                                                      C.c_int(eval_log), _ptr_array(accum4), C.c_int(int(accumulate))))

    # ---- GrindOps
    def grind(self, prefixed_digest8, pow_bits, m31_out=True):
        d = _u32(prefixed_digest8)
        nonce = C.c_uint64()
        self._check(self.lib.zkb_grind(self.h, d.ctypes.data_as(C.c_void_p), C.c_int(pow_bits), C.c_int(int(m31_out)), C.byref(nonce)))
        return nonce.value

    # ---- whole protocols (include/zkb200_prover.h)
    @staticmethod
    def pcs_prepare(trees_ptrs, logs, cap=1 << 24):
        """The argument arrays of a PCS proof, built once: a caller that proves the same tens of thousands of columns again and
        again passes the result as `trees_ptrs` (and None as `logs`) and does not pay for their conversion, nor for a fresh
        output buffer, in every call. The returned proof words are then a view of the prepared output buffer."""
        flat = [p for t in trees_ptrs for p in t]
        return {"n_trees": len(trees_ptrs), "ncols": np.array([len(t) for t in trees_ptrs], np.int32), "ptrs": _ptr_array(flat),
                "logs": _u32(logs), "out": np.empty(cap, np.uint32)}

    def _pcs(self, fn, trees_ptrs, logs, pow_bits, log_blowup, log_last_layer, n_queries, two_sample_every, cap, phases):
        prepared = trees_ptrs if isinstance(trees_ptrs, dict) else None
        a = prepared or self.pcs_prepare(trees_ptrs, logs, cap)
        cfg = PcsConfig(pow_bits, log_blowup, log_last_layer, n_queries)
        out = a["out"]
        n = C.c_size_t()
        ph = np.zeros(len(PCS_PHASES), np.float32)
        self._check(fn(self.h, C.c_int(a["n_trees"]), a["ncols"].ctypes.data_as(C.c_void_p), a["ptrs"], a["logs"].ctypes.data_as(C.c_void_p),
                       C.byref(cfg), C.c_int(two_sample_every), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.size), C.byref(n),
                       ph.ctypes.data_as(C.c_void_p) if phases else None))
        words = out[:n.value] if prepared else out[:n.value].copy()
        return (words, dict(zip(PCS_PHASES, ph.tolist()))) if phases else words

    def pcs_prove_device(self, trees_ptrs, logs, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3, two_sample_every=0,
                         cap=1 << 24, phases=False):
        """trees_ptrs: per tree, device addresses of the trace columns (consumed). logs: flat log sizes."""
        return self._pcs(self.lib.zkb_pcs_prove_device, trees_ptrs, logs, pow_bits, log_blowup, log_last_layer, n_queries,
                         two_sample_every, cap, phases)

    def shard_pcs(self, rank, world, ncols_total, log_n, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3):
        """A sharded-proof session of this rank (zkb_shard_pcs_*); see ShardPcsSession."""
        return ShardPcsSession(self, rank, world, ncols_total, log_n, PcsConfig(pow_bits, log_blowup, log_last_layer, n_queries))

    def pcs_prove_host(self, trees, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3, two_sample_every=0, cap=1 << 24,
                       phases=False):
        """trees: per tree, host uint32 arrays (trace evaluations, bit-reversed)."""
        arrs = [[_u32(c) for c in t] for t in trees]
        ptrs = [[c.ctypes.data for c in t] for t in arrs]
        logs = [len(c).bit_length() - 1 for t in arrs for c in t]
        return self._pcs(self.lib.zkb_pcs_prove_host, ptrs, logs, pow_bits, log_blowup, log_last_layer, n_queries,
                         two_sample_every, cap, phases)

    def stark_prove(self, prog, trees, trace_log, claimed_sum=None, scalars=None, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3,
                    cap=1 << 24, phases=None, host=False):
        """zkb_stark_prove_device / _host: trees is a list (one entry per tree) of lists of device pointers (or of host arrays
        when host=True). Returns (proof words incl. channel digest, committed composition value [4], value from the constraints
        [4], composition_ms)."""
        ncols = np.array([len(t) for t in trees], dtype=np.int32)
        cfg = PcsConfig(pow_bits, log_blowup, log_last_layer, n_queries)
        sc = _u32(prog.source.scalars if scalars is None else scalars)
        cs = _u32(claimed_sum) if claimed_sum is not None else None
        out = np.empty(cap, np.uint32)
        n = C.c_size_t()
        oods = np.zeros(8, np.uint32)
        ph = (C.c_float * len(PCS_PHASES))()
        comp_ms = C.c_float()
        if host:
            keep = [_u32(c) for t in trees for c in t]
            ptrs = (C.c_void_p * len(keep))(*[k.ctypes.data for k in keep])
            fn = self.lib.zkb_stark_prove_host
        else:
            ptrs = _ptr_array([p for t in trees for p in t])
            fn = self.lib.zkb_stark_prove_device
        self._check(fn(self.h, C.c_int(len(trees)), ncols.ctypes.data_as(C.c_void_p), ptrs, C.c_uint32(trace_log), prog.h,
                       sc.ctypes.data_as(C.c_void_p), cs.ctypes.data_as(C.c_void_p) if cs is not None else None, C.byref(cfg),
                       out.ctypes.data_as(C.c_void_p), C.c_size_t(cap), C.byref(n), oods.ctypes.data_as(C.c_void_p), ph, C.byref(comp_ms)))
        if phases is not None:
            phases.update({k: float(ph[i]) for i, k in enumerate(PCS_PHASES)})
            phases["composition"] = float(comp_ms.value)
        return out[:n.value].copy(), oods[:4].copy(), oods[4:].copy(), float(comp_ms.value)

    def stark_prove_multi(self, components, trees, pow_bits=10, log_blowup=1, log_last_layer=0, n_queries=3, cap=1 << 24, phases=None,
                          host=False):
        """zkb_stark_prove_multi_device / _host. components: list of (AirProgram, trace_log, claimed_sum or None[, scalars]); trees:
        per tree the list of device pointers (host arrays when host=True), the columns of component k after those of the components
        before it. Returns (proof words incl. channel digest, committed composition value [4], value from the constraints [4],
        composition_ms)."""
        keep = []
        arr = (StarkComponent * len(components))()
        for i, comp in enumerate(components):
            prog, trace_log, claimed = comp[0], comp[1], comp[2]
            sc = _u32(prog.source.scalars if len(comp) < 4 or comp[3] is None else comp[3])
            cs = _u32(claimed) if claimed is not None else None
            keep += [sc, cs]
            arr[i].prog = prog.h
            arr[i].trace_log = trace_log
            arr[i].scalars = sc.ctypes.data if sc.size else None
            arr[i].claimed_sum = cs.ctypes.data if cs is not None else None
        ncols = np.array([len(t) for t in trees], dtype=np.int32)
        cfg = PcsConfig(pow_bits, log_blowup, log_last_layer, n_queries)
        out = np.empty(cap, np.uint32)
        n = C.c_size_t()
        oods = np.zeros(8, np.uint32)
        ph = (C.c_float * len(PCS_PHASES))()
        comp_ms = C.c_float()
        if host:
            hk = [_u32(c) for t in trees for c in t]
            ptrs = (C.c_void_p * len(hk))(*[k.ctypes.data for k in hk])
            fn = self.lib.zkb_stark_prove_multi_host
        else:
            ptrs = _ptr_array([p for t in trees for p in t])
            fn = self.lib.zkb_stark_prove_multi_device
        self._check(fn(self.h, C.c_int(len(trees)), ncols.ctypes.data_as(C.c_void_p), ptrs, C.c_int(len(components)), arr, C.byref(cfg),
                       out.ctypes.data_as(C.c_void_p), C.c_size_t(cap), C.byref(n), oods.ctypes.data_as(C.c_void_p), ph, C.byref(comp_ms)))
        if phases is not None:
            phases.update({k: float(ph[i]) for i, k in enumerate(PCS_PHASES)})
            phases["composition"] = float(comp_ms.value)
        return out[:n.value].copy(), oods[:4].copy(), oods[4:].copy(), float(comp_ms.value)

    def gkr_prove_device(self, instances, seed, cap=1 << 22):
        """instances: list of (kind, num_ptr or 0, den_ptr, n_entries)."""
        kinds = np.array([k for k, _, _, _ in instances], np.int32)
        nums = (C.c_void_p * len(instances))(*[(n or None) for _, n, _, _ in instances])
        dens = (C.c_void_p * len(instances))(*[d for _, _, d, _ in instances])
        ns = np.array([n for _, _, _, n in instances], np.uint64)
        out = np.empty(cap, np.uint32)
        nw = C.c_size_t()
        self._check(self.lib.zkb_gkr_prove_device(self.h, C.c_int(len(instances)), kinds.ctypes.data_as(C.c_void_p), nums, dens,
                                                  ns.ctypes.data_as(C.c_void_p), C.c_uint64(seed), out.ctypes.data_as(C.c_void_p),
                                                  C.c_size_t(cap), C.byref(nw)))
        return out[:nw.value].copy()
