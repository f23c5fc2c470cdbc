"""The sharded commitment on real GPUs (NCCL, one process per GPU): the root equals the
single-GPU Merkle root of the same columns. Needs at least two GPUs; skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, log_n, log_blowup, ncols, out_dir):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import zk_inference_prover_b200 as z
    from util import m31_column
    from zk_inference_prover_b200.sharded import ContextOps, ShardedCommitment

    ctx = z.Context(device=rank, max_log_size=log_n + log_blowup)
    sc = ShardedCommitment(ContextOps(ctx), torch.device("cuda", rank))
    c0, c1 = sc.local_columns(ncols)
    host = np.stack([m31_column(7100 + c, 1 << log_n) for c in range(c0, c1)]).view(np.int32)
    trace = torch.from_numpy(host.copy()).cuda(rank)
    root, local, _ = sc.commit(trace, log_n, log_blowup)
    np.save(os.path.join(out_dir, f"root{rank}.npy"), root.cpu().numpy().view(np.uint32))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_root_equals_single_gpu_root(ctx, tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from util import m31_column

    log_n, log_blowup, ncols = 12, 2, 16
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(world, port, log_n, log_blowup, ncols, str(tmp_path)), nprocs=world, join=True)
    # single-GPU tree through the same C ABI
    log_out = log_n + log_blowup
    cols = [ctx.upload(m31_column(7100 + c, 1 << log_n)) for c in range(ncols)]
    ctx.ifft_cols([c.ptr for c in cols], log_n)
    evals = [ctx.alloc(1 << log_out) for _ in range(ncols)]
    ctx.lde_cols([c.ptr for c in cols], log_n, [e.ptr for e in evals], log_out)
    layer = ctx.alloc(8 << log_out)
    ctx.merkle_layer(log_out, 0, [e.ptr for e in evals], layer.ptr)
    for lg in range(log_out - 1, -1, -1):
        nxt = ctx.alloc(8 << lg)
        ctx.merkle_layer(lg, layer.ptr, [], nxt.ptr)
        layer = nxt
    want = layer.download()
    for r in range(world):
        assert (np.load(tmp_path / f"root{r}.npy") == want).all()


# ------------------------------------------------------------------ the whole proof, sharded
def _proof_worker(rank, world, port, backend, log_n, log_blowup, ncols, n_queries, out_dir):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = rank if backend == "nccl" else 0  # gloo: every rank on GPU 0, the exchanges go through the host
    torch.cuda.set_device(dev)
    if backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", dev))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200.sharded import ContextMem, Exchange, sharded_pcs_prove
    from zk_inference_prover_b200.synth import m31_column

    ctx = z.Context(device=dev, max_log_size=log_n + log_blowup)
    ncl = ncols // world
    cols = [ctx.upload(m31_column(7300 + c, 1 << log_n)) for c in range(rank * ncl, (rank + 1) * ncl)]
    sess = ctx.shard_pcs(rank, world, ncols, log_n, pow_bits=10, log_blowup=log_blowup, log_last_layer=0, n_queries=n_queries)
    words = sharded_pcs_prove(sess, Exchange(ContextMem(ctx), torch.device("cuda", dev)), [c.ptr for c in cols])
    sess.close()
    np.save(os.path.join(out_dir, f"proof{rank}.npy"), words)
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


def _single_gpu_proof(ctx, log_n, log_blowup, ncols, n_queries):
    from zk_inference_prover_b200.synth import m31_column

    cols = [ctx.upload(m31_column(7300 + c, 1 << log_n)) for c in range(ncols)]
    return ctx.pcs_prove_device([[c.ptr for c in cols]], [log_n] * ncols, pow_bits=10, log_blowup=log_blowup, log_last_layer=0,
                                n_queries=n_queries)


def _spawn(world, backend, *args):
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_proof_worker, args=(world, port, backend) + args, nprocs=world, join=True)


@pytest.mark.parametrize("world,log_n,log_blowup,ncols,n_queries", [(2, 10, 2, 8, 3), (4, 12, 1, 16, 20), (8, 11, 2, 8, 50), (1, 9, 1, 3, 5)])
def test_sharded_proof_equals_single_gpu_proof_ranks_on_one_gpu(ctx, tmp_path, world, log_n, log_blowup, ncols, n_queries):
    """All ranks share GPU 0 and exchange through the host (gloo): no kernel of a rank waits for another rank, so this is
    safe on one device, and it runs the library's sharded session and the merge exactly as a multi-GPU run does. The proof
    (every word, and the channel digest after it) equals the single-device proof of the same columns."""
    _spawn(world, "gloo", log_n, log_blowup, ncols, n_queries, str(tmp_path))
    want = _single_gpu_proof(ctx, log_n, log_blowup, ncols, n_queries)
    for r in range(world):
        got = np.load(tmp_path / f"proof{r}.npy")
        assert len(got) == len(want) and (got == want).all(), f"rank {r}"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_proof_equals_single_gpu_proof_nccl(ctx, tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    log_n, log_blowup, ncols, n_queries = 14, 2, 32, 30
    _spawn(world, "nccl", log_n, log_blowup, ncols, n_queries, str(tmp_path))
    want = _single_gpu_proof(ctx, log_n, log_blowup, ncols, n_queries)
    for r in range(world):
        got = np.load(tmp_path / f"proof{r}.npy")
        assert len(got) == len(want) and (got == want).all(), f"rank {r}"
