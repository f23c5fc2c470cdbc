"""Locates the fields of a PCS proof's word stream (the order of PcsProof::write in csrc/host/prover.cpp and of
oracle/protocol.hpp's to_words), so that tests can tamper with single fields on the host and re-serialise."""
import numpy as np


class ProofWords:
    def __init__(self, words, tree_ncols):
        self.w = np.array(words, np.uint32)
        w, at = self.w, 0
        n = int(w[at]); at += 1
        assert n == len(tree_ncols)
        self.commitments = [(at + 8 * i, 8) for i in range(n)]
        at += 8 * n
        self.sampled = []  # per tree, per column: (offset, words)
        for nc in tree_ncols:
            assert int(w[at]) == nc
            at += 1
            cols = []
            for _ in range(nc):
                k = int(w[at]); at += 1
                cols.append((at, 4 * k))
                at += 4 * k
            self.sampled.append(cols)
        self.decommitments = [self._dec(at_) for at_ in [None] * 0]
        self.decommitments = []
        for _ in tree_ncols:
            d, at = self._dec(at)
            self.decommitments.append(d)
        self.queried = []
        for _ in tree_ncols:
            k = int(w[at])
            self.queried.append({"count_at": at, "at": at + 1, "n": k})
            at += 1 + k
        self.pow_at = at
        at += 2
        self.fri_layers = []
        l, at = self._layer(at)
        self.fri_layers.append(l)
        self.n_inner_at = at
        n_inner = int(w[at]); at += 1
        for _ in range(n_inner):
            l, at = self._layer(at)
            self.fri_layers.append(l)
        self.last_count_at = at
        k = int(w[at]); at += 1
        self.last_poly = (at, 4 * k)
        at += 4 * k
        self.proof_end = at
        self.digest_at = at if at + 8 <= len(w) else None

    def _dec(self, at):
        w = self.w
        h = int(w[at])
        d = {"hash_count_at": at, "hashes_at": at + 1, "n_hashes": h}
        at += 1 + 8 * h
        c = int(w[at])
        d.update({"col_count_at": at, "cols_at": at + 1, "n_cols": c})
        at += 1 + c
        d["end"] = at
        return d, at

    def _layer(self, at):
        w = self.w
        k = int(w[at])
        l = {"start": at, "witness_count_at": at, "witness_at": at + 1, "n_witness": k}
        at += 1 + 4 * k
        l["dec"], at = self._dec(at)
        l["commitment_at"] = at
        at += 8
        l["end"] = at
        return l, at

    # ---- edits (each returns a new word array)
    def flip(self, offset, mask=1):
        w = self.w.copy()
        w[offset] ^= np.uint32(mask)
        return w

    def remove(self, start, end, counter_at=None, dec=1):
        w = np.concatenate([self.w[:start], self.w[end:]])
        if counter_at is not None:
            w[counter_at] -= np.uint32(dec)
        return w

    def insert(self, at, words, counter_at=None, inc=1):
        w = np.concatenate([self.w[:at], np.array(words, np.uint32), self.w[at:]])
        if counter_at is not None:
            w[counter_at] += np.uint32(inc)
        return w
