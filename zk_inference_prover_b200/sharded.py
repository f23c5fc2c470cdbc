"""One commitment over G GPUs: column-sharded LDE, one all-to-all, row-sharded Merkle subtrees.

The reference has no multi-device code. The hot path shards naturally:

  1. rank r owns a contiguous block of `ncols / G` trace columns and runs interpolate + LDE on them
     (columns are independent);
  2. ONE exchange turns the column-sharded evaluations `[ncols/G][N]` into row-sharded ones
     `[ncols][N/G]`: rank d receives rows `[d N/G, (d+1) N/G)` of every column. Evaluations are in
     bit-reversed order, so that row range is a contiguous subtree of the Merkle tree and the sibling
     pairs (2i, 2i+1) the FRI folds use stay on one rank;
  3. every rank hashes its leaves and the `log2(N/G)` layers above them (MerkleOps::commit_on_layer,
     nitroo/crates/stwo/src/prover/vcs/ops.rs:24-29, in the layer order of
     nitroo/crates/stwo/src/prover/vcs/prover.rs:39-64);
  4. the G subtree roots (32 bytes each) are all-gathered and every rank hashes the top `log2 G`
     layers, so all ranks hold the root the single-GPU commitment produces, bit for bit.

`ops` supplies the operators on raw addresses (the zkb200 Context on GPUs; the tests pass a CPU
stand-in so that the sharding logic runs under `gloo`), `torch.distributed` supplies the exchange.
No kernel here reads another GPU's memory: the all-to-all lands in local HBM first.
"""
import math

import torch
import torch.distributed as dist


def _is_pow2(x):
    return x > 0 and (x & (x - 1)) == 0


class ShardedCommitment:
    def __init__(self, ops, device, group=None):
        self.ops = ops
        self.device = device
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if not _is_pow2(self.world):
            raise ValueError("the number of ranks must be a power of two")
        self.log_g = int(math.log2(self.world))

    # ---- plan
    def local_columns(self, ncols):
        """[start, end) of the global column indices this rank owns."""
        if ncols % self.world:
            raise ValueError("the column count must be a multiple of the number of ranks")
        per = ncols // self.world
        return self.rank * per, (self.rank + 1) * per

    def local_rows(self, log_out):
        n = (1 << log_out) // self.world
        return self.rank * n, (self.rank + 1) * n

    # ---- exchange
    def _all_to_all(self, recv, send):
        """recv[s] <- send[rank] of rank s, for tensors of shape [G, ...]."""
        if dist.get_backend(self.group) == "nccl":
            dist.all_to_all_single(recv.view(-1), send.view(-1), group=self.group)
            return
        # gloo has no all-to-all: pairwise exchange, lower rank sends first
        recv[self.rank].copy_(send[self.rank])
        for peer in range(self.world):
            if peer == self.rank:
                continue
            if self.rank < peer:
                dist.send(send[peer].contiguous(), peer, group=self.group)
                dist.recv(recv[peer], peer, group=self.group)
            else:
                dist.recv(recv[peer], peer, group=self.group)
                dist.send(send[peer].contiguous(), peer, group=self.group)

    # ---- the commitment
    def commit(self, trace, log_n, log_blowup):
        """trace: int32 tensor [ncols_local, 2^log_n] (this rank's columns, evaluations in bit-reversed
        order; consumed). Returns (root words as an int32 tensor of 8, row-sharded evaluations
        [ncols, N/G], coefficients [ncols_local, 2^log_n])."""
        ops, G = self.ops, self.world
        ncl = trace.shape[0]
        log_out = log_n + log_blowup
        N = 1 << log_out
        if log_out - self.log_g < 1:
            raise ValueError("each rank needs at least two rows")
        rows = N // G
        es = trace.element_size()
        # 1. interpolate + LDE on the local columns
        ops.ifft_cols([trace[c].data_ptr() for c in range(ncl)], log_n)
        evals = torch.empty((ncl, N), dtype=trace.dtype, device=self.device)
        ops.lde_cols([trace[c].data_ptr() for c in range(ncl)], log_n, [evals[c].data_ptr() for c in range(ncl)], log_out)
        ops.sync()
        # 2. pack per destination and exchange: send[d] = rows [d rows, (d+1) rows) of my columns
        send = evals.view(ncl, G, rows).permute(1, 0, 2).contiguous()
        del evals
        recv = torch.empty((G, ncl, rows), dtype=trace.dtype, device=self.device)
        self._all_to_all(recv, send)
        del send
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        local = recv.view(G * ncl, rows)  # global column order: source rank major
        # 3. the local subtree
        log_local = log_out - self.log_g
        col_ptrs = [local[c].data_ptr() for c in range(G * ncl)]
        layer = torch.empty((rows, 8), dtype=trace.dtype, device=self.device)
        ops.merkle_layer(log_local, 0, col_ptrs, layer.data_ptr())
        for lg in range(log_local - 1, -1, -1):
            nxt = torch.empty((1 << lg, 8), dtype=trace.dtype, device=self.device)
            ops.merkle_layer(lg, layer.data_ptr(), [], nxt.data_ptr())
            layer = nxt
        ops.sync()
        # 4. top of the tree from the G subtree roots
        roots = torch.empty((G, 8), dtype=trace.dtype, device=self.device)
        dist.all_gather_into_tensor(roots.view(-1), layer.view(-1), group=self.group) if dist.get_backend(self.group) == "nccl" \
            else self._all_gather(roots, layer)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        top = roots
        for lg in range(self.log_g - 1, -1, -1):
            nxt = torch.empty((1 << lg, 8), dtype=trace.dtype, device=self.device)
            ops.merkle_layer(lg, top.data_ptr(), [], nxt.data_ptr())
            top = nxt
        ops.sync()
        assert es == 4
        return top.view(-1), local, trace

    def _all_gather(self, out, mine):
        parts = [torch.empty_like(mine.view(-1)) for _ in range(self.world)]
        dist.all_gather(parts, mine.view(-1).contiguous(), group=self.group)
        for s in range(self.world):
            out[s].copy_(parts[s])


class ContextOps:
    """The zkb200 operators on raw device addresses (the GPU side of `ops`)."""

    def __init__(self, ctx):
        self.ctx = ctx

    def ifft_cols(self, ptrs, log_n):
        self.ctx.ifft_cols(ptrs, log_n)

    def lde_cols(self, src, log_n, dst, log_out):
        self.ctx.lde_cols(src, log_n, dst, log_out)

    def merkle_layer(self, log_size, prev_ptr, col_ptrs, out_ptr):
        self.ctx.merkle_layer(log_size, prev_ptr, col_ptrs, out_ptr, m31_out=True)

    def sync(self):
        self.ctx.sync()


# ---------------------------------------------------------------------------------------------------------------
# One whole PCS proof over G ranks (include/zkb200_prover.h, zkb_shard_pcs_*): the library computes, this class moves.

class _Alias:
    """A device range as something torch.as_tensor can alias (the CUDA array interface)."""

    def __init__(self, ptr, words):
        self.__cuda_array_interface__ = {"shape": (int(words),), "typestr": "<i4", "data": (int(ptr), False), "version": 2}


class Exchange:
    """The data movements a sharded proof needs, over torch.distributed.

    `nccl`: device tensors alias the library's buffers and the collectives are ordered on the context's own stream
    (torch.cuda.ExternalStream), so nothing synchronises with the host. `gloo`: the ranges are staged through host
    memory; this is what lets several ranks share one GPU in tests (no kernel of one rank waits on another rank:
    every wait is a host-side collective) and what the CPU tests of this logic run on."""

    def __init__(self, mem, device, group=None):
        self.mem, self.device, self.group = mem, device, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.nccl = dist.get_backend(group) == "nccl"
        self._pending = []
        self._peer = None

    def _dev(self, ptr, words):
        return torch.as_tensor(_Alias(ptr, words), device=self.device)

    def _stream(self):
        if not self.nccl:
            import contextlib

            return contextlib.nullcontext()
        return torch.cuda.stream(torch.cuda.ExternalStream(self.mem.stream(), device=self.device))

    # ---- direct copies between the ranks' GPUs (one host): the receive buffers are shared between the processes and a
    # rank writes its blocks into its peers' buffers with the copy engines, which need no SM and so run under kernels
    def peer_setup(self, ctx, words):
        """Collective: every rank allocates a receive buffer of `words` words its peers can write and opens the others'.
        Returns False (and sets nothing up) when the ranks are not GPUs of one host under nccl."""
        if self._peer is not None and self._peer["words"] >= words:
            return True
        if not self.nccl or not hasattr(ctx, "peer_buffer_alloc"):
            return False
        import socket

        import numpy as np

        self.peer_close()
        host = np.frombuffer(socket.gethostname().encode()[:32].ljust(32, b"\0"), np.uint32).copy()
        if len({bytes(h) for h in self.all_gather_host(host).reshape(self.world, -1)}) != 1:
            return False
        mine, handle = ctx.peer_buffer_alloc(words * 4)
        handles = self.all_gather_host(handle.view(np.uint32)).reshape(self.world, 16).view(np.uint8)
        ptrs = [mine if r == self.rank else ctx.peer_buffer_open(handles[r]) for r in range(self.world)]
        self._peer = {"ctx": ctx, "words": words, "mine": mine, "ptrs": ptrs}
        dist.barrier(group=self.group)
        return True

    def peer_close(self):
        """Collective: releases the shared receive buffers."""
        if self._peer is None:
            return
        p, self._peer = self._peer, None
        p["ctx"].sync()
        dist.barrier(group=self.group)  # nobody copies into a buffer that is about to go
        for r, ptr in enumerate(p["ptrs"]):
            if r != self.rank:
                p["ctx"].peer_buffer_close(ptr)
        dist.barrier(group=self.group)
        p["ctx"].peer_buffer_free(p["mine"])

    def peer_rows(self):
        return self._peer["mine"]

    def peer_ptrs(self):
        return list(self._peer["ptrs"])

    def peer_all_to_all(self, send_ptr, recv_ptr, words_per_peer):
        """Block d of `send` goes to the place of rank d's receive buffer that `recv_ptr` is in mine, block `rank`: enqueued on
        the copy stream after what the compute stream holds so far; peer_finish() makes the data visible."""
        p = self._peer
        off = recv_ptr - p["mine"] + 4 * self.rank * words_per_peer
        for k in range(self.world):
            d = (self.rank + k) % self.world  # start with the local block, then a different peer on every rank
            p["ctx"].copy_to_peer(p["ptrs"][d] + off, send_ptr + 4 * d * words_per_peer, 4 * words_per_peer, lane=k)

    def peer_finish(self):
        """Waits for this rank's copies, then for everybody's: after it every rank's receive buffer is complete."""
        self._peer["ctx"].peer_copies_wait()
        dist.barrier(group=self.group)

    def all_to_all(self, send_ptr, recv_ptr, words_per_peer, defer=False):
        """Block d of `send` ([world][words_per_peer]) becomes block `rank` of rank d's `recv`. With defer (nccl), the
        collective starts after what the context's stream holds so far and runs beside what is enqueued after it; the
        stream waits for it only at flush()."""
        G, me = self.world, self.rank
        if self.nccl:
            with self._stream():
                work = dist.all_to_all_single(self._dev(recv_ptr, G * words_per_peer), self._dev(send_ptr, G * words_per_peer),
                                              group=self.group, async_op=defer)
            if defer:
                self._pending.append(work)
            return
        sd = torch.from_numpy(self.mem.read(send_ptr, G * words_per_peer).view("int32")).view(G, words_per_peer)
        rv = torch.empty_like(sd)
        rv[me].copy_(sd[me])
        for peer in range(G):  # gloo has no all-to-all: pairwise, the lower rank sends first
            if peer == me:
                continue
            if me < peer:
                dist.send(sd[peer], peer, group=self.group)
                dist.recv(rv[peer], peer, group=self.group)
            else:
                dist.recv(rv[peer], peer, group=self.group)
                dist.send(sd[peer], peer, group=self.group)
        self.mem.write(recv_ptr, rv.numpy().view("uint32").reshape(-1))

    def flush(self):
        """Orders the context's stream after every deferred collective (a stream-side wait, the host does not block)."""
        if self._pending:
            with self._stream():
                for work in self._pending:
                    work.wait()
            self._pending = []

    def all_gather_device(self, src_ptr, dst_ptr, words):
        """dst[r * words ...] <- src of rank r."""
        if self.nccl:
            with self._stream():
                dist.all_gather_into_tensor(self._dev(dst_ptr, words * self.world), self._dev(src_ptr, words), group=self.group)
            return
        mine = torch.from_numpy(self.mem.read(src_ptr, words).view("int32"))
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        self.mem.write(dst_ptr, torch.cat(parts).numpy().view("uint32"))

    def _gather_buffers(self, words):
        """Page-locked host and device buffers for all_gather_host under nccl, kept between calls."""
        if getattr(self, "_gb", None) is None or self._gb[0] < words:
            cap = max(1024, 1 << (int(words) - 1).bit_length())
            self._gb = (cap, torch.empty(cap, dtype=torch.int32).pin_memory(), torch.empty(self.world * cap, dtype=torch.int32).pin_memory(),
                        torch.empty(cap, dtype=torch.int32, device=self.device), torch.empty(self.world * cap, dtype=torch.int32, device=self.device))
        return self._gb

    def all_gather_host(self, arr):
        """Equal-sized host arrays, concatenated in rank order."""
        import numpy as np

        mine = torch.from_numpy(np.ascontiguousarray(arr).view("int32").reshape(-1))
        if self.nccl:
            # one collective on one tensor, staged through page-locked memory on both sides
            n = mine.numel()
            _, send_h, recv_h, send_d, recv_d = self._gather_buffers(n)
            send_h[:n].copy_(mine)
            send_d[:n].copy_(send_h[:n], non_blocking=True)
            dist.all_gather_into_tensor(recv_d[: self.world * n], send_d[:n], group=self.group)
            recv_h[: self.world * n].copy_(recv_d[: self.world * n], non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            return recv_h[: self.world * n].numpy().view("uint32").copy()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        return torch.cat(parts).numpy().view("uint32")

    VARLEN_HEAD = 1 << 14  # words of the first round of all_gather_varlen: the length, then the array's head

    def all_gather_varlen(self, arr):
        """Host arrays of different lengths -> list in rank order (on every rank). One collective when every array fits
        the first round (its length travels in the same block), a second one sized by the longest array otherwise: every
        rank sees every length after the first round, so all take the same way."""
        import numpy as np

        cap = self.VARLEN_HEAD
        head = np.zeros(cap, np.uint32)
        head[0] = len(arr)
        k = min(len(arr), cap - 1)
        head[1 : 1 + k] = arr[:k]
        flat = self.all_gather_host(head).reshape(self.world, cap)
        lens = flat[:, 0]
        if int(lens.max()) <= cap - 1:
            return [flat[r, 1 : 1 + int(lens[r])].copy() for r in range(self.world)]
        cap = int(lens.max())
        pad = np.zeros(cap, np.uint32)
        pad[: len(arr)] = arr
        flat = self.all_gather_host(pad).reshape(self.world, cap)
        return [flat[r, : int(lens[r])].copy() for r in range(self.world)]


class ContextMem:
    """Raw device ranges of a zkb200 Context, for Exchange (`gloo` staging reads and writes them through the host)."""

    def __init__(self, ctx):
        self.ctx = ctx

    def stream(self):
        return self.ctx.stream()

    def read(self, ptr, words):
        import numpy as np

        import ctypes as C

        out = np.empty(int(words), np.uint32)
        self.ctx._check(self.ctx.lib.zkb_d2h(self.ctx.h, out.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), C.c_size_t(out.nbytes)))
        return out

    def write(self, ptr, arr):
        import ctypes as C
        import numpy as np

        a = np.ascontiguousarray(arr, dtype=np.uint32)
        self.ctx._check(self.ctx.lib.zkb_h2d(self.ctx.h, C.c_void_p(ptr), a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes)))


def sharded_pcs_prove(session, exchange, col_ptrs, timings=None):
    """Runs one sharded proof: `session` is this rank's ShardPcsSession (or an object with the same stages), `exchange`
    an Exchange over the same ranks, col_ptrs this rank's trace columns. Returns the proof words on every rank.
    timings, when a dict, receives per stage the device time between CUDA events on the context's stream (the collectives
    are ordered on that stream), summed over calls."""
    s, x = session, exchange
    ctx = getattr(s, "ctx", None) if timings is not None else None
    marks = []

    def lap(name):
        if ctx is not None:
            ctx.event_record(40 + len(marks))
            marks.append(name)

    lap("start")
    # By chunks of columns, so that a chunk travels while the next one is extended (sessions without the chunked stage, as
    # the stand-in of the CPU tests, take the whole shard at once).
    n_chunks = 1
    if hasattr(s, "extend_begin"):
        n_chunks = next((c for c in (4, 2) if s.ncl % c == 0), 1)
    peer = hasattr(s, "set_peer_rows") and hasattr(x, "peer_setup") and x.peer_setup(s.ctx, s.ncols * s.R)
    if peer:
        # the ranks write their blocks straight into each other's receive buffers with the copy engines, chunk by chunk
        # under the transform of the next chunk (a collective's copy kernels would wait for the SMs the transform holds)
        s.set_peer_rows(x.peer_ptrs())
        s.extend_begin(col_ptrs, n_chunks)
        for k in range(n_chunks):
            s.extend_chunk(k)  # transform, then the copies of the chunk's blocks into the peers' buffers
        x.peer_finish()
    elif n_chunks > 1:
        s.extend_begin(col_ptrs, n_chunks)
        for k in range(n_chunks):
            send, recv, words_per_peer = s.extend_chunk(k)
            x.all_to_all(send, recv, words_per_peer, defer=True)
        x.flush()
    else:
        send, rows = s.extend(col_ptrs)
        x.all_to_all(send, rows, s.ncl * s.R)
    lap("interpolate_extend_exchange")
    root, roots = s.subtree()
    x.all_gather_device(root, roots, 8)
    lap("merkle_subtree_roots")
    mine = s.sample()
    everyone = x.all_gather_host(mine)
    lap("top_layers_sample")
    local, full = s.quotients(everyone)
    for k in range(4):
        x.all_gather_device(local[k], full[k], s.R)
    lap("quotients_gather")
    part = s.fri_and_decommit()
    parts = x.all_gather_varlen(part)
    words = s.finish(parts)
    lap("fri_grind_decommit_merge")
    if ctx is not None:
        for i in range(1, len(marks)):
            timings[marks[i]] = timings.get(marks[i], 0.0) + ctx.event_elapsed_ms(40 + i - 1, 40 + i)
    return words
