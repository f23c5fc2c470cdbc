#!/usr/bin/env python
"""Writes tests/golden/segment_shapes.json: the committed-column shapes of composed decode segments.

    python tests/golden/make_segment_shapes.py /path/to/reference/checkout

The reference prover proves one (layer, token block) segment as one STARK whose trees hold hundreds of
components of different heights. Its own cell-exact cost model (harness/costmodel/exact_cells.py in the
reference checkout) rebuilds every component's layout from a segment's `params` block and multiplies
columns by rows. This script imports that module, walks the same layout functions component by
component, and records what the totals alone do not carry: every component's (columns, log_rows) per
tree, its lookup count (the entries its LogUp-GKR instance holds per row) and the Freivalds layouts.
`bench.py --mode segment-replay` commits and proves trees of exactly these shapes on seeded random
columns (timing only: the witness and the gadgets' AIRs are application code outside the operators).

Every segment's recorded shapes are checked against exact_cells(): base, interaction and boundary
totals must agree to the cell, or the script stops.

Segments written:
  layer_8b_s32_c2048   a layer segment of the 32-layer model of the decode benchmark (hidden 4096,
                       32 query / 8 KV heads, head_dim 128, SwiGLU 14336), token block 32, context
                       2048, witness-calibrated fields at the modal values of the recorded runs
  head_8b_s32_c2048    the output head segment of the same model (vocabulary 32000)
  micro_s32_c128       the reference's recorded cell microbenchmark segment (s 32, ctx 128, hd 32,
                       intsplit6, kmax 16): the shape class of the built-in synthetic CI segment
"""
import json
import os
import sys


def components(ec, p):
    """[(family, base_cols, interaction_m31_cols, log_rows, lookups_per_row, repeat)] in exact_cells order."""
    out = []
    s, hd, nh = p["s"], p["hd"], p["nh"]
    sticky = p["round"] == "even"
    Q = ec.M31_PER_QM31
    gkr_kt = p.get("gkr_key_tiles", False) or p.get("gkr_bands", False)
    for n, lay, acc, look in ec.tile_components(p):
        qm = acc + (0 if gkr_kt else Q * -(-look // 2))
        out.append(("key_tiles", n, qm, lay["log_rows"], look if gkr_kt else 0, 1))
    for insts, _c, rows_comp, _d in ec._key_tile_shapes(p):
        if rows_comp:
            rw, lr = ec.row_layout(insts * s, p["rw"])
            out.append(("key_tiles", 4 * rw, 8 + (0 if gkr_kt else Q * 2 * rw), lr, 2 * rw if gkr_kt else 0, 1))
    mat_lays = {}
    for j, m in enumerate(p["mats"]):
        pr, _, lr = ec.mat_layout(m["n_out"], m["tokens"], p["deq_target"])
        mat_lays[j] = (pr, lr)
        qm = 2 + int(ec._has_output_claim(p, m["name"])) + int(ec._has_scale_claim(p, m))
        looks = ec.deq_looks(m["variant"], pr)
        if not p.get("gkr_dequant"):
            qm += -(-looks // 2)
        out.append(("dequant", ec.deq_columns(m["variant"], sticky, pr), Q * qm, lr, looks if p.get("gkr_dequant") else 0,
                    m.get("repeat", 1)))
    ao_pr, _, ao_lr = ec.ao_layout(nh, s, ec.hd_v(p), p["ao_target"])
    ao_cols = 2 + ao_pr * (9 + int(p.get("ao_acc_mag", False)))
    ao_qm = 5 if p.get("gkr_attnout") else 5 + -(-7 * ao_pr // 2)
    out.append(("attnout", ao_cols, Q * ao_qm, ao_lr, 7 * ao_pr if p.get("gkr_attnout") else 0, 1))
    fv_lays = []
    for name, mats in ec._freivalds_groups(p):
        pk, pq, lr = ec.freivalds_layout(mats[0]["n_in"], max(m["n_out"] for m in mats), mats[0]["tokens"], p["freivalds_p"])
        fv_lays.append((name, pk, pq, lr, len(mats)))
        qm = 2 * len(mats) + 2
        if not p.get("gkr_freivalds"):
            qm += -(-pq // 2)
        out.append(("freivalds", pq, Q * qm, lr, pq if p.get("gkr_freivalds") else 0, ec._repeat(mats)))
    rs_comps = ec.residual_stream_components(p) if p.get("residual_stream") else []
    for _tag, cols, lr, bindings, looks in rs_comps:
        qm = bindings + (0 if p.get("gkr_residual_stream") else -(-looks // 2))
        out.append(("residual_stream", cols, Q * qm, lr, looks if p.get("gkr_residual_stream") else 0, 1))
    for _name, n_out, toks, width, _bits in ec._quant_sides(p):
        pr, _, lr = ec.q_layout(n_out, width, toks, p["deq_target"])
        out.append(("quant", 7 * pr, Q * (-(-5 * pr // 2) + 2), lr, 0, 1))
    for name in ec._seam_names(p):
        pr, _, lr = ec.mat_layout(ec._seam_width(p, name), s, p["deq_target"])
        n_scale = 1 if ec._seam_variant(p, name) == "pow2" else 2
        out.append(("requant", 2 + n_scale + 7 * pr, Q * (-(-(5 * pr + 1) // 2) + 3), lr, 0, 1))
    if p.get("prove_argmax"):
        m = ec._mat(p, "lm_head")
        pr, _, lr = ec.mat_layout(m["n_out"], m["tokens"], p["deq_target"])
        out.append(("argmax", 2 * pr + 3, Q * (2 + -(-pr // 2)), lr, 0, 1))
    if p.get("embed_vocab"):
        pe, _k, log_use, log_tab = ec.embed_layout((p["residual_stream"] or {})["d"], s, p["embed_vocab"], p["embed_per_row"])
        out.append(("embed", 1 + 2 * pe, Q * (-(-(1 + pe) // 2) + 2), log_use, 0, 1))
        out.append(("embed", 1, Q, log_tab, 0, 1))
    for table in (ec.table_rows(p), ec.requant_table_rows(p)):
        for name, rows in table.items():
            lr = rows.bit_length() - 1
            if rows == 1 << lr:
                out.append(("tables", 1, Q, lr, 0, 1))
            else:  # a table whose row count is not a power of two is counted by its rows; none occurs in these segments
                raise SystemExit(f"table {name} has {rows} rows")
    heights = ec.link_heights(p, mat_lays, fv_lays, rs_comps, ao_lr)
    for h in heights:
        out.append(("gkrlink", 0, 16, h, 0, 1))
    return out, fv_lays


def boundary_columns(cells):
    """The boundary trees hand the residual stream and the key/value cache to the next segment; the cost model gives
    their cell count, not their column layout. Here: columns of 2^16 rows (the height class of the components that
    read them) and one shorter column set for the remainder."""
    cols = []
    lr = 16
    while cells and lr >= 4:
        n = cells >> lr
        if n:
            cols.append((n, lr))
            cells -= n << lr
        lr -= 1
    assert cells == 0, cells
    return cols


def describe(ec, name, note, p):
    comps, fv = components(ec, p)
    want = ec.exact_cells(p)
    base = sum(r * (b << lr) for _f, b, _i, lr, _l, r in comps)
    inter = sum(r * (i << lr) for _f, _b, i, lr, _l, r in comps)
    assert base == want["base"], (name, base, want["base"])
    assert inter == want["interaction"], (name, inter, want["interaction"])
    merged = {}
    for f, b, i, lr, l, r in comps:  # identical components become one row with a repeat count
        merged[(f, b, i, lr, l)] = merged.get((f, b, i, lr, l), 0) + r
    comps = [k + (r,) for k, r in merged.items()]
    bcols = boundary_columns(want["boundary"])
    assert sum(n << lr for n, lr in bcols) == want["boundary"]
    return {"note": note, "cells": {"base": base, "interaction": inter, "boundary": want["boundary"], "fresh": want["fresh"]},
            "components": [{"family": f, "base_cols": b, "interaction_cols": i, "log_rows": lr, "lookups_per_row": l, "repeat": r}
                           for f, b, i, lr, l, r in comps],
            "boundary_cols": [{"cols": n, "log_rows": lr} for n, lr in bcols],
            "freivalds": [{"group": n, "pk": pk, "pq": pq, "log_rows": lr, "n_mats": nm} for n, pk, pq, lr, nm in fv]}


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ZK_REFERENCE_DIR")
    if not ref:
        raise SystemExit(__doc__)
    sys.path.insert(0, ref)
    from harness.costmodel import exact_cells as ec

    out = {"_made_by": "tests/golden/make_segment_shapes.py from the reference's harness/costmodel/exact_cells.py",
           "segments": {}}
    w = ec.modal_assumption("layer")
    p = ec.segment_params("layer", 4096, 32, 8, 128, 14336, 32000, 32, 2048, w)
    out["segments"]["layer_8b_s32_c2048"] = describe(
        ec, "layer", "layer segment: hidden 4096, 32/8 heads, head_dim 128, SwiGLU 14336, token block 32, context 2048", p)
    wh = ec.modal_assumption("head")
    ph = ec.segment_params("head", 4096, 32, 8, 128, 14336, 32000, 32, 2048, wh)
    out["segments"]["head_8b_s32_c2048"] = describe(ec, "head", "output head segment of the same model, vocabulary 32000", ph)
    micro = next(c for c in ec.chunks() if "microbench" in c["run"])
    out["segments"]["micro_s32_c128"] = describe(
        ec, "micro", "the reference's recorded cell microbenchmark segment (s 32, ctx 128, hd 32, intsplit6, kmax 16)", micro["params"])
    assert out["segments"]["micro_s32_c128"]["cells"]["fresh"] == micro["fresh"]
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "segment_shapes.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=0, separators=(",", ":"))
        f.write("\n")
    for k, v in out["segments"].items():
        print(k, v["cells"], len(v["components"]), "components")


if __name__ == "__main__":
    main()
