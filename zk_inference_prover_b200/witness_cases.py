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


# ---- the residual-stream component ------------------------------------------------------------------------------------
RS_NONE = 0xFFFFFFFF
RS_DMAX, RS_UMIN = 12, 260


def signed_product_table(round_even=True):
    """The signed-significand product table in its row order: values 0, +128..+255, -128..-255 on both axes (257 x 257 rows);
    per row (rounded signed significand, binade carry, non-zero flag)."""
    vals = [0] + list(range(128, 256)) + [-m for m in range(128, 256)]
    out = np.zeros((257 * 257, 3), np.int32)
    for ia, a in enumerate(vals):
        for ib, b in enumerate(vals):
            if a == 0 or b == 0:
                continue
            p = abs(a) * abs(b)
            c = 1 if p >= 1 << 15 else 0
            sh = 7 + c
            q, rem = divmod(p, 1 << sh)
            half = 1 << (sh - 1)
            if round_even:
                q += 1 if (rem > half or (rem == half and (q & 1))) else 0
            else:
                q += 1 if rem >= half else 0
            if q == 256:
                q, c = 128, c + 1
            out[ia * 257 + ib] = (q if (a < 0) == (b < 0) else -q, c, 1)
    return out


def value_table_pairs():
    """(sm, ef) of every legal bf16 value in the value table's row order: zero, then (ef, m7, sign) ascending."""
    ef = np.repeat(np.arange(1, 255), 256)
    m7 = np.tile(np.repeat(np.arange(128), 2), 254)
    sign = np.tile(np.array([1, -1]), 254 * 128)
    sm = (128 + m7) * sign
    return np.concatenate([[0], sm]).astype(np.int64), np.concatenate([[0], ef]).astype(np.int64)


def unary_table(kind):
    """A unary image per value-table row as (sm, ef) pairs: bf16(f(x)) by float32 arithmetic and one round-to-nearest-even.
    The generators only read the table, so any function gives a valid test; `square` and `negate-halve` are used."""
    sm, ef = value_table_pairs()
    x = sm.astype(np.float64) * np.exp2(ef.astype(np.float64) - 134.0)
    with np.errstate(over="ignore"):
        y = (x * x if kind == "square" else -0.5 * x).astype(np.float32)
    u = y.view(np.uint32).astype(np.uint64)
    pat = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) & 0xFFFF
    e = (pat >> 7) & 0xFF
    finite = (e != 0) & (e != 0xFF)
    mag = 128 + (pat & 0x7F).astype(np.int64)
    osm = np.where(finite, np.where((pat >> 15) & 1 == 1, -mag, mag), 0)
    oef = np.where(finite, e, 0)
    return np.stack([osm, oef], axis=1).astype(np.int32)


def _rs_layout(groups, n_slots, kind, sticky):
    width = [2 if un == 0 else 4 for _, un in groups]
    base = np.concatenate([[0], np.cumsum([n * w for (n, _), w in zip(groups, width)])]).astype(int)
    slot_w = (13 + (1 if sticky else 0)) if kind == 0 else 4
    slot_at = lambda s: int(base[-1]) + s * slot_w
    if kind == 0:
        k = 11 + (1 if sticky else 0)
        out_cols = lambda s: (slot_at(s) + k, slot_at(s) + k + 1)
    else:
        out_cols = lambda s: (slot_at(s), slot_at(s) + 3)
    return width, base, slot_at, out_cols, int(base[-1]) + n_slots * slot_w


def rs_program(shape, n, pad=None, un=(0, 0), kind=0):
    """The reference's program shapes in their host form: `tree` (a pairwise reduction x[:h] + x[h:] over `pad` positions of
    which the first n are leaves and the rest the constant zero, zero positions pruned) and `pairs` (n independent binary
    operations on two groups). Sources are (kind, g, i): 0 zero, 1 leaf, 2 unary image of a leaf, 3 slot g."""
    if shape == "tree":
        groups = [(n, un[0])]
        leaf = (lambda i: (2, 0, i)) if un[0] else (lambda i: (1, 0, i))
        cur = [leaf(i) if i < n else (0, 0, 0) for i in range(pad)]
        slots = []
        while len(cur) > 1:
            h = len(cur) // 2
            nxt = []
            for i in range(h):
                x, y = cur[i], cur[i + h]
                if x[0] == 0:
                    nxt.append(y)
                elif y[0] == 0:
                    nxt.append(x)
                else:
                    slots.append((x, y))
                    nxt.append((3, len(slots) - 1, 0))
            cur = nxt
        return groups, slots, [cur[0][1]], 0
    groups = [(n, un[0]), (n, un[1])]
    src = lambda g, i: (2, g, i) if groups[g][1] else (1, g, i)
    return groups, [(src(0, i), src(1, i)) for i in range(n)], list(range(n)), kind


def residual_stream_case(seed, shape, n, log_rows, live_rows, pad=None, un=(0, 0), kind=0, sticky=True, kmax=13, spread=6):
    """One residual-stream component on seeded bf16 inputs: the program in host form (for the oracle) and lowered to column
    indices (for the kernels), honest tables, zeroed multiplicity lengths. `spread` bounds the exponents' range so that adds
    exercise both kept and dropped smaller operands; a few zeros, infinities and NaN patterns are planted."""
    rng = np.random.default_rng(seed)
    groups, src_slots, out_slot, kind = rs_program(shape, n, pad, un, kind)
    n_un = max([u for _, u in groups] + [0])
    n_leaves = sum(g[0] for g in groups)
    width, base, slot_at, out_cols, n_cols = _rs_layout(groups, len(src_slots), kind, sticky)
    ef = np.clip(rng.integers(127 - spread, 127 + spread + 1, (live_rows, n_leaves)), 0, 255)
    wit = ((rng.integers(0, 2, ef.shape) << 15) | (ef << 7) | rng.integers(0, 128, ef.shape)).astype(np.uint32)
    flat_idx = rng.integers(0, wit.size, max(4, wit.size // 50))
    wit.reshape(-1)[flat_idx] = rng.choice(np.array([0x0000, 0x8000, 0x7F80, 0xFF80, 0x7FC1, 0x0001, 0x3F80], np.uint32), flat_idx.size)
    lowered_groups, flat = [], 0
    for g, (gn, gu) in enumerate(groups):
        lowered_groups.append((gn, int(base[g]), width[g], gu, flat))
        flat += gn

    def cols_of(s):
        if s[0] == 0:
            return RS_NONE, RS_NONE
        if s[0] == 3:
            return out_cols(s[1])
        b = int(base[s[1]]) + s[2] * width[s[1]]
        return (b, b + 1) if s[0] == 1 else (b + 2, b + 3)

    slots = []
    for si, (a, b) in enumerate(src_slots):
        (a_sm, a_ef), (b_sm, b_ef), (o_sm, o_ef) = cols_of(a), cols_of(b), out_cols(si)
        slots.append((a_sm, a_ef, b_sm, b_ef, slot_at(si), o_sm, o_ef, (1 if a[0] == 3 else 0) | (2 if b[0] == 3 else 0)))
    n_val = 1 + 254 * 128 * 2
    norm = norm_table(kmax, sticky) if sticky else _norm_table_away(kmax)
    pow2 = lambda x: 1 << (x - 1).bit_length()
    m_len = {"pow": pow2(RS_DMAX + 1 + RS_UMIN), "norm": pow2(len(norm)), "val": pow2(n_val), "frac": pow2(1 << (kmax + 1)),
             "smul": pow2(257 * 257), "un": pow2(n_val)}
    return {"groups": groups, "src_slots": [tuple(a) + tuple(b) for a, b in src_slots], "out_slot": out_slot, "kind": kind, "sticky": sticky,
            "kmax": kmax, "norm3": norm.reshape(-1), "smul3": signed_product_table(sticky).reshape(-1),
            "un2": [unary_table(["square", "negate-halve"][u]).reshape(-1) for u in range(n_un)], "n_val": n_val, "wit": wit.reshape(-1),
            "live_rows": live_rows, "log_rows": log_rows, "m_len": m_len, "n_cols": n_cols, "n_leaves": n_leaves,
            "lowered_groups": np.array(lowered_groups, np.uint32), "lowered_slots": np.array(slots, np.uint32).reshape(-1, 8)}


def _norm_table_away(kmax):
    """norm_table for round-to-nearest, ties away from zero (no sticky rows)."""
    rows = [(0, 0, 0)]
    for m2 in range(1, 256):
        bits = m2.bit_length()
        rows.append(((m2 << (8 - bits)) & 0x7F, 127 + bits - 1, 1))
    for k in range(kmax + 1):
        for m2 in range(256, 512):
            m7, ef = ((m2 >> 1) & 0x7F) + (m2 & 1), 127 + 8 + k
            if m7 == 128:
                m7, ef = 0, ef + 1
            rows.append((m7, ef, 1))
    return np.array(rows, np.uint32)


def pre_table_case(seed, kind, log_rows, n_counters, n_patch):
    """Counter arrays and patch rows for one shared table of 2^log_rows committed rows."""
    rng = np.random.default_rng(seed)
    rows, n_cols = 1 << log_rows, {0: 6, 1: 3, 2: 4, 3: 2, 4: 1}[kind]
    counters = [rng.integers(0, 1 << 20, rows, dtype=np.uint32) for _ in range(n_counters)]
    patch_idx = rng.choice(rows, n_patch, replace=False).astype(np.uint32) if n_patch else np.zeros(0, np.uint32)
    patch_val = rng.integers(0, 1 << 30, (n_patch, n_cols), dtype=np.uint32)
    return counters, patch_idx, patch_val
