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
