"""zkb_gkr_sum_noalloc: the sum-check round sums for callers that may not allocate.

A prover that runs with its device allocator locked (the whole card carved into a fixed arena),
or a thread that must not cause the device-wide synchronisation an allocation can trigger, cannot
create a zkb context or let the library allocate scratch. This entry point keeps its scratch in an
array built into the library. The test calls it through the C ABI twice in a row on the same
inputs and on different ones, and requires the device-resident result to equal what zkb_gkr_sum
returns and what the CPU oracle computes from the same inputs, word for word (integer field
arithmetic: the tolerance is zero). This file sorts last so
that a run stopping at the first failure has already run every other test."""
import numpy as np
import pytest

import oracle
from util import m31_column, qm31_array

pytestmark = pytest.mark.gpu


def _layer(kind, n, seed):
    den = qm31_array(seed, n, nonzero=True)
    num = qm31_array(seed + 1, n) if kind == 1 else m31_column(seed + 1, n) if kind == 2 else None
    return num, den


@pytest.mark.parametrize("kind,log_n", [(2, 16), (1, 12), (3, 20), (0, 9), (2, 2)])
def test_noalloc_matches_context_entry_point_twice(zkb, ctx, kind, log_n):
    n = 1 << log_n
    out = ctx.alloc(8)
    for round_ in range(2):  # two calls in a row share the built-in scratch
        num, den = _layer(kind, n, 9000 + 17 * round_ + kind)
        eq = qm31_array(9100 + round_, n // 4)
        lam = qm31_array(9200 + round_, 1)[0]
        nb = ctx.upload(num) if num is not None else None
        db, eb = ctx.upload(den), ctx.upload(eq)
        want = ctx.gkr_sum(kind, nb.ptr if nb else 0, db.ptr, n, eb.ptr, lam)
        out.upload(np.full(8, 0xDEADBEEF, np.uint32))
        zkb.gkr_sum_noalloc(0, ctx.stream(), kind, nb.ptr if nb else 0, db.ptr, n, eb.ptr, lam, out.ptr)
        got = out.download(shape=(2, 4))  # ordered after the kernel on the same stream
        assert (got == want).all()
        assert (got == oracle.gkr_round_sums(kind, num, den, eq, lam)).all()  # not only the sibling entry point
        # and once more on identical inputs: the ticket and partials of the last call do not leak
        zkb.gkr_sum_noalloc(0, ctx.stream(), kind, nb.ptr if nb else 0, db.ptr, n, eb.ptr, lam, out.ptr)
        assert (out.download(shape=(2, 4)) == want).all()


def test_noalloc_rejects_oversize_and_bad_arguments(zkb, ctx):
    buf = ctx.alloc(64)
    lam = [1, 2, 3, 4]
    with pytest.raises(zkb.ZkbError) as e:
        zkb.gkr_sum_noalloc(0, ctx.stream(), 3, 0, buf.ptr, 1 << 29, buf.ptr, lam, buf.ptr)
    assert e.value.code == -1 and "2^28" in str(e.value)
    with pytest.raises(zkb.ZkbError):
        zkb.gkr_sum_noalloc(0, ctx.stream(), 1, 0, buf.ptr, 16, buf.ptr, lam, buf.ptr)  # generic layer without numerators
    with pytest.raises(zkb.ZkbError):
        zkb.gkr_sum_noalloc(0, ctx.stream(), 3, 0, buf.ptr, 24, buf.ptr, lam, buf.ptr)  # not a power of two
    # misaligned pointers are refused on the host; nothing is launched
    with pytest.raises(zkb.ZkbError) as e:
        zkb.gkr_sum_noalloc(0, ctx.stream(), 3, 0, buf.ptr + 4, 16, buf.ptr, lam, buf.ptr)
    assert "aligned" in str(e.value)
    with pytest.raises(zkb.ZkbError):
        zkb.gkr_sum_noalloc(0, ctx.stream(), 3, 0, buf.ptr, 16, buf.ptr + 8, lam, buf.ptr)
    with pytest.raises(zkb.ZkbError):
        zkb.gkr_sum_noalloc(0, ctx.stream(), 2, buf.ptr + 4, buf.ptr, 16, buf.ptr, lam, buf.ptr)
    with pytest.raises(zkb.ZkbError):
        zkb.gkr_sum_noalloc(0, ctx.stream(), 1, buf.ptr + 8, buf.ptr, 16, buf.ptr, lam, buf.ptr)
    with pytest.raises(zkb.ZkbError):
        ctx.gkr_sum(3, 0, buf.ptr + 4, 16, buf.ptr, lam)
