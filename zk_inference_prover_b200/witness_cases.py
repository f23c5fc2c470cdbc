"""Seeded inputs for the witness-generation tests: honest normalisation / mantissa-product tables and dequantize cases."""
import numpy as np


def norm_table(kmax, sticky):
    """The normalisation table in the row order the reference's O(1) index assumes (prover/src/layer.rs:2042-2062):
    row 0 is zero, rows 1..255 the exactly representable magnitudes, then per round-bit weight 2^k the 256 extended
    significands (times two when the rounding keeps a sticky bit). Each row: (m7, exponent field, non-zero flag) of the
    bf16 the magnitude rounds to, ties to even with the sticky bit, ties away from zero without."""
    rows = [(0, 0, 0)]
    for m2 in range(1, 256):
        bits = m2.bit_length()
        rows.append(((m2 << (8 - bits)) & 0x7F, 127 + bits - 1, 1))
    per = 2 if sticky else 1
    for k in range(kmax + 1):
        for m2 in range(256, 512):
            for st in range(per):
                keep, g = (m2 >> 1) & 0x7F, m2 & 1
                up = g and (st or (keep & 1)) if sticky else g
                m7, ef = keep + (1 if up else 0), 127 + 8 + k
                if m7 == 128:
                    m7, ef = 0, ef + 1
                rows.append((m7, ef, 1))
    return np.array(rows, np.uint32)


def mul_table():
    """(product mantissa, carry) of two 8-bit significands 1.m_in x 1.ms rounded to 8 bits, ties to even; row m_in * 128 + ms."""
    out = np.zeros((128 * 128, 2), np.uint32)
    for a in range(128):
        for b in range(128):
            p = (128 + a) * (128 + b)  # value p / 2^14 in [1, 4)
            c = 1 if p >= 1 << 15 else 0
            sh = 7 + c
            q, rem = divmod(p, 1 << sh)
            half = 1 << (sh - 1)
            q += 1 if (rem > half or (rem == half and (q & 1))) else 0
            if q == 256:
                q, c = 128, c + 1
            out[a * 128 + b] = (q - 128, c)
    return out


def dequant_case(seed, variant, tokens, chunks, per_row, kmax=16, sticky=1, do_ref=1, wide=False):
    """One dequantize component on seeded inputs. wide=True also draws accumulators beyond the kmax window and scales that
    leave the 8-bit range table, so that the three failure counters are exercised."""
    rng = np.random.default_rng(seed)
    n_out = chunks * per_row
    rows = tokens * chunks
    log_rows = rows.bit_length() - 1
    assert rows == 1 << log_rows
    lim = (1 << (kmax + 9)) - 1
    bits = rng.integers(0, kmax + 10, (tokens, n_out))
    acc = (rng.integers(0, 1 << 62, (tokens, n_out)) & ((1 << bits) - 1)).astype(np.int64)
    acc = np.minimum(acc, lim) * rng.choice([-1, 1], (tokens, n_out))
    acc[0, :4] = [0, 1, -1, 255][: min(4, n_out)]
    if wide:
        acc[rng.integers(0, tokens, 5), rng.integers(0, n_out, 5)] = (1 << 30) + 12345
        acc[0, -1] = -(1 << 31)
    acc = acc.astype(np.int32)
    norm3 = norm_table(kmax, sticky)
    mul2 = mul_table()
    chain = variant == 1
    n_fields = 8 + sticky + (6 if chain else 1)
    order = rng.permutation(n_fields)  # the column map is the caller's: any assignment of fields to columns must work
    names = ["f_acc", "f_sg", "f_m2", "f_ph", "f_r", "f_m7", "f_ef", "f_nz"] + (["f_st"] if sticky else []) + \
        ([f"f_mul{k}" for k in range(6)] if chain else ["f_eo"])
    cfg = {k: 0xFFFFFFFF for k in ("f_st", "f_eo", "f_mul0", "f_mul1", "f_mul2", "f_mul3", "f_mul4", "f_mul5")}
    cfg.update({n: int(o) for n, o in zip(names, order)})
    n_shared = 2 if chain else 1
    cfg.update(variant=variant, sticky=sticky, kmax=kmax, do_ref=do_ref, tokens=tokens, n_out=n_out, per_row=per_row, chunks=chunks,
               log_rows=log_rows, slot0=n_shared, per_slot=n_fields, chan_w=2 if chain else 1, sh0=0, sh1=1 if chain else 0,
               n_norm=len(norm3), n_frac=1 << (kmax + 1), n_mul=len(mul2), n_r8=256)
    lo, hi = (-150, 150) if wide else (-20, 20)
    jx = rng.integers(lo, hi, tokens).astype(np.int32)
    jw = rng.integers(lo, hi, n_out).astype(np.int32)
    e_lo, e_hi = (60, 200) if wide else (100, 140)
    sx = np.stack([rng.integers(0, 128, tokens), rng.integers(e_lo, e_hi, tokens)], 1).astype(np.uint32)
    sw = np.stack([rng.integers(0, 128, n_out), rng.integers(e_lo, e_hi, n_out)], 1).astype(np.uint32)
    return {"cfg": cfg, "acc": acc, "jx": jx, "jw": jw, "sx": sx, "sw": sw, "norm3": norm3, "mul2": mul2,
            "n_base": n_shared + per_row * n_fields, "n_pre": cfg["chan_w"] * per_row + 5, "rows": rows}


def tables_case(seed, log_rows, n_counters, n_patch=0):
    rng = np.random.default_rng(seed)
    rows = 1 << log_rows
    expmap = rng.integers(0, 512, 1 << 16).astype(np.uint32)
    counters = [rng.integers(0, 1000, rows).astype(np.uint32) for _ in range(n_counters)]
    patch_idx = rng.choice(rows, n_patch, replace=False).astype(np.uint32)
    patch_val = rng.integers(0, 512, n_patch).astype(np.uint32)
    return expmap, counters, patch_idx, patch_val
