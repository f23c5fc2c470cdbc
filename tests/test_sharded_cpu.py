"""The multi-GPU commitment's host logic under `gloo` on CPU ranks: which columns and rows a rank owns,
the pack + all-to-all + unpack, the subtree hashing order and the assembly of the top layers. The
operators are supplied by a CPU stand-in over the oracle (the product's operators need a GPU); the
result must be the root of the single-process tree, bit for bit, and the row-sharded evaluations
must be the oracle's evaluations of every column restricted to the rank's row range."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _view(ptr, words):
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint32)), shape=(words,))


class OracleOps:
    """`ops` for CPU tensors: the same calls as zk_inference_prover_b200.sharded.ContextOps."""

    def __init__(self, oracle):
        self.o = oracle

    def ifft_cols(self, ptrs, log_n):
        for p in ptrs:
            v = _view(p, 1 << log_n)
            v[:] = self.o.interpolate_cols([v.copy()], log_n)[0]

    def lde_cols(self, src, log_n, dst, log_out):
        for s, d in zip(src, dst):
            _view(d, 1 << log_out)[:] = self.o.evaluate_cols([_view(s, 1 << log_n).copy()], log_n, log_out)[0]

    def merkle_layer(self, log_size, prev_ptr, col_ptrs, out_ptr):
        n = 1 << log_size
        prev = _view(prev_ptr, 16 * n).reshape(2 * n, 8).copy() if prev_ptr else None
        cols = [_view(p, n).copy() for p in col_ptrs]
        _view(out_ptr, 8 * n)[:] = self.o.commit_on_layer(log_size, prev, cols, m31=True).reshape(-1)

    def sync(self):
        pass


def _worker(rank, world, port, log_n, log_blowup, ncols, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from util import m31_column
    from zk_inference_prover_b200.sharded import ShardedCommitment

    sc = ShardedCommitment(OracleOps(oracle), torch.device("cpu"))
    c0, c1 = sc.local_columns(ncols)
    trace = torch.from_numpy(np.stack([m31_column(7000 + c, 1 << log_n) for c in range(c0, c1)]).view(np.int32).copy())
    root, local, coeffs = sc.commit(trace, log_n, log_blowup)
    np.save(os.path.join(out_dir, f"root{rank}.npy"), root.numpy().view(np.uint32))
    np.save(os.path.join(out_dir, f"local{rank}.npy"), local.numpy().view(np.uint32))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,log_n,log_blowup,ncols", [(2, 5, 1, 6), (4, 6, 2, 8)])
def test_sharded_commit_matches_single_tree(oracle, tmp_path, world, log_n, log_blowup, ncols):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from util import m31_column

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(world, port, log_n, log_blowup, ncols, str(tmp_path)), nprocs=world, join=True)
    cols = np.stack([m31_column(7000 + c, 1 << log_n) for c in range(ncols)])
    log_out = log_n + log_blowup
    evals = oracle.evaluate_cols(oracle.interpolate_cols(cols, log_n), log_n, log_out)
    layer = oracle.commit_on_layer(log_out, None, list(evals), m31=True)
    for lg in range(log_out - 1, -1, -1):
        layer = oracle.commit_on_layer(lg, layer, [], m31=True)
    rows = (1 << log_out) // world
    for r in range(world):
        assert (np.load(tmp_path / f"root{r}.npy") == layer[0]).all()
        assert (np.load(tmp_path / f"local{r}.npy") == evals[:, r * rows:(r + 1) * rows]).all()


# ------------------------------------------------------------------ the whole-proof driver's data movement
# The library's sharded session needs a GPU; what runs on CPU ranks here is everything around it: the order of the stages in
# sharded_pcs_prove and every movement of Exchange under gloo (all-to-all of row blocks, device and host all-gathers, the
# gather of parts of different lengths). The stand-in session keeps "device memory" in a numpy arena and computes, at every
# stage, values that depend on every word another rank must have delivered, so that a misplaced block changes the result.
class ArenaMem:
    def __init__(self, words):
        self.a = np.zeros(words, np.uint32)

    def stream(self):
        return 0

    def read(self, ptr, words):
        return self.a[ptr:ptr + int(words)].copy()

    def write(self, ptr, arr):
        arr = np.asarray(arr, np.uint32).reshape(-1)
        self.a[ptr:ptr + len(arr)] = arr


def _cell(c, i):
    return (np.uint64(2654435761) * np.uint64(c + 1) + np.uint64(40503) * np.asarray(i, np.uint64)) % np.uint64(2**31 - 1)


class StandInSession:
    def __init__(self, mem, rank, world, ncols, N):
        self.mem, self.rank, self.world, self.ncols, self.N = mem, rank, world, ncols, N
        self.ncl, self.R = ncols // world, N // world
        self.send, self.rows, self.root, self.roots = 0, ncols * N, 2 * ncols * N, 2 * ncols * N + 8
        self.ql = [self.roots + 8 * world + k * self.R for k in range(4)]
        self.qf = [self.ql[3] + self.R + k * N for k in range(4)]

    def extend(self, col_ptrs):
        ncl, R, G = self.ncl, self.R, self.world
        for d in range(G):
            for j in range(ncl):
                c = self.rank * ncl + j
                self.mem.write(self.send + (d * ncl + j) * R, _cell(c, np.arange(d * R, (d + 1) * R)).astype(np.uint32))
        return self.send, self.rows

    def _local(self):
        return self.mem.read(self.rows, self.ncols * self.R).reshape(self.ncols, self.R)

    def subtree(self):
        self.mem.write(self.root, (self._local().astype(np.uint64).sum(axis=0)[:8] % np.uint64(2**31 - 1)).astype(np.uint32))
        return self.root, self.roots

    def sample(self):
        self.all_roots = self.mem.read(self.roots, 8 * self.world)
        return np.stack([_cell(self.rank * self.ncl + j, np.arange(4)).astype(np.uint32) for j in range(self.ncl)])

    def quotients(self, everyone):
        self.samples = np.asarray(everyone).copy()
        loc = self._local().astype(np.uint64)
        for k in range(4):
            self.mem.write(self.ql[k], ((loc * np.uint64(k + 1)).sum(axis=0) % np.uint64(2**31 - 1)).astype(np.uint32))
        return self.ql, self.qf

    def fri_and_decommit(self):
        full = np.concatenate([self.mem.read(self.qf[k], self.N) for k in range(4)])
        self.full_sum = int(full.astype(np.uint64).sum() % (2**31 - 1))
        return np.arange(3 + 2 * self.rank, dtype=np.uint32) + np.uint32(1000 * self.rank)  # parts of different lengths

    def finish(self, parts):
        return np.concatenate([self.all_roots, self.samples.reshape(-1), np.array([self.full_sum], np.uint32)] + list(parts)).astype(np.uint32)


def _driver_worker(rank, world, port, ncols, N, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from zk_inference_prover_b200.sharded import Exchange, sharded_pcs_prove

    mem = ArenaMem(2 * ncols * N + 8 + 8 * world + 4 * (N // world) + 4 * N)
    sess = StandInSession(mem, rank, world, ncols, N)
    words = sharded_pcs_prove(sess, Exchange(mem, torch.device("cpu")), [])
    np.save(os.path.join(out_dir, f"words{rank}.npy"), words)
    np.save(os.path.join(out_dir, f"rows{rank}.npy"), sess._local())
    dist.destroy_process_group()


@pytest.mark.parametrize("world,ncols,N", [(2, 6, 64), (4, 8, 128)])
def test_sharded_proof_driver_moves_every_block_to_its_owner(tmp_path, world, ncols, N):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_driver_worker, args=(world, port, ncols, N, str(tmp_path)), nprocs=world, join=True)
    R, P = N // world, np.uint64(2**31 - 1)
    table = np.stack([_cell(c, np.arange(N)) for c in range(ncols)])  # [ncols][N], uint64
    roots = np.concatenate([(table[:, r * R:(r + 1) * R].sum(axis=0)[:8] % P).astype(np.uint32) for r in range(world)])
    samples = np.concatenate([_cell(c, np.arange(4)).astype(np.uint32) for c in range(ncols)])
    full = np.concatenate([((table * np.uint64(k + 1)).sum(axis=0) % P) for k in range(4)])
    full_sum = np.array([int(full.sum() % P)], np.uint32)
    parts = [np.arange(3 + 2 * r, dtype=np.uint32) + np.uint32(1000 * r) for r in range(world)]
    want = np.concatenate([roots, samples, full_sum] + parts)
    for r in range(world):
        assert (np.load(tmp_path / f"rows{r}.npy") == table[:, r * R:(r + 1) * R].astype(np.uint32)).all()  # the all-to-all
        assert (np.load(tmp_path / f"words{r}.npy") == want).all()


def _varlen_worker(rank, world, port, lengths, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from zk_inference_prover_b200.sharded import Exchange

    x = Exchange(None, torch.device("cpu"))
    mine = np.arange(lengths[rank], dtype=np.uint32) * np.uint32(3) + np.uint32(7 * rank)
    parts = x.all_gather_varlen(mine)
    np.save(os.path.join(out_dir, f"parts{rank}.npy"), np.concatenate([np.array([len(p) for p in parts], np.uint32)] + list(parts)))
    dist.destroy_process_group()


@pytest.mark.parametrize("lengths", [(5, 0), (3, 40000), (16383, 16383), (16384, 1)])
def test_all_gather_varlen_one_round_or_two(tmp_path, lengths):
    """Arrays that fit the first round (length and head in one block) arrive with one collective, longer ones with a second
    one sized by the longest: both ways must return every rank's array on every rank, empty ones included."""
    world = len(lengths)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_varlen_worker, args=(world, port, lengths, str(tmp_path)), nprocs=world, join=True)
    want = np.concatenate([np.array(lengths, np.uint32)] + [np.arange(n, dtype=np.uint32) * np.uint32(3) + np.uint32(7 * r) for r, n in enumerate(lengths)])
    for r in range(world):
        assert (np.load(tmp_path / f"parts{r}.npy") == want).all()
