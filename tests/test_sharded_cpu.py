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
