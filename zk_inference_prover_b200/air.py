"""Host-side lowering of an AIR to the single-assignment program that zkb_air_compile takes.

`ExprEvaluator` has the calling surface of the reference's `EvalAtRow`
(nitroo/crates/constraint-framework/src/lib.rs:70-199): an AIR's `evaluate` is written against it once and, instead of
computing values, every call appends an instruction. It plays the part the reference's own symbolic evaluator plays
for its kernel generator (`ExprEvaluator`, constraint-framework/src/expr/evaluator.rs:62-78, lowered by
prover/src/cudagen.rs:942-1200): the LogUp identities are ordinary constraints of the program
(`finalize_logup_batched`, lib.rs:226-275), relation elements and claims are run-time scalars.

Three AIRs of the reference are written out below as examples and for the tests and the benchmark: wide Fibonacci,
Plonk and the Freivalds component.
"""
import numpy as np

P = (1 << 31) - 1

# interaction (tree) indices of the reference's fork: preprocessed, model, base trace, interaction (lib.rs:40-58)
PREPROCESSED_TRACE_IDX, MODEL_TRACE_IDX, ORIGINAL_TRACE_IDX, INTERACTION_TRACE_IDX = 0, 1, 2, 3

LOAD, CONST_M31, SCALAR, CUMSUM_SHIFT, ADD_B, SUB_B, MUL_B, NEG_B, ADD_E, SUB_E, MUL_E, NEG_E, PACK, INV_B = range(14)


class Expr:
    """A value of the program: the index of the instruction that produces it and whether it is a secure-field value."""
    __slots__ = ("ev", "idx", "ext")

    def __init__(self, ev, idx, ext):
        self.ev, self.idx, self.ext = ev, idx, ext

    def _bin(self, other, op_b, op_e, swap=False):
        other = self.ev.lift(other)
        a, b = (other, self) if swap else (self, other)
        if a.ext or b.ext:
            return self.ev.emit(op_e, a.idx, b.idx, ext=True)
        return self.ev.emit(op_b, a.idx, b.idx, ext=False)

    def __add__(self, o): return self._bin(o, ADD_B, ADD_E)
    def __radd__(self, o): return self._bin(o, ADD_B, ADD_E, swap=True)
    def __sub__(self, o): return self._bin(o, SUB_B, SUB_E)
    def __rsub__(self, o): return self._bin(o, SUB_B, SUB_E, swap=True)
    def __mul__(self, o): return self._bin(o, MUL_B, MUL_E)
    def __rmul__(self, o): return self._bin(o, MUL_B, MUL_E, swap=True)
    def __neg__(self): return self.ev.emit(NEG_E if self.ext else NEG_B, self.idx, ext=self.ext)
    def square(self): return self * self

    def inverse(self):
        assert not self.ext, "only base-field values have an inverse instruction"
        return self.ev.emit(INV_B, self.idx, ext=False)


class Relation:
    """A LogUp relation: combine(values) = sum_i alpha^i values[i] - z (constraint-framework/src/logup.rs:83-98). The
    elements are run-time scalars of the program."""

    def __init__(self, ev, z, alpha_powers):
        self.z = ev.scalar(z)
        self.alpha_powers = [ev.scalar(a) for a in alpha_powers]

    def combine(self, ev, values):
        assert len(self.alpha_powers) >= len(values), "Not enough alpha powers to combine values"
        acc = None
        for v, a in zip(values, self.alpha_powers):
            term = a * v
            acc = term if acc is None else acc + term
        return acc - self.z if acc is not None else -self.z


class ExprEvaluator:
    def __init__(self, n_interactions=4):
        self.ops = []
        self.constraints = []
        self.scalars = []
        self.column_index_per_interaction = [0] * n_interactions
        self.fracs = []
        self.logup_interaction = INTERACTION_TRACE_IDX
        self._consts = {}

    # ---- program construction
    def emit(self, op, a=0, b=0, c=0, d=0, ext=False):
        self.ops.append((op, a & 0xffffffff, b & 0xffffffff, c & 0xffffffff, d & 0xffffffff))
        return Expr(self, len(self.ops) - 1, ext)

    def const(self, v):
        v = int(v) % P
        if v not in self._consts:
            self._consts[v] = self.emit(CONST_M31, v)
        return self._consts[v]

    def scalar(self, value4):
        """A run-time secure-field scalar (relation element, claim, random power): a slot of the scalar array."""
        self.scalars.append([int(x) % P for x in value4])
        return self.emit(SCALAR, len(self.scalars) - 1, ext=True)

    def claim(self, value4):
        """EvalAtRow::claim (lib.rs:157-159): a value of the statement; always a scalar slot of its own."""
        return self.scalar(value4)

    def cumsum_shift(self):
        return self.emit(CUMSUM_SHIFT, ext=True)

    def lift(self, v):
        if isinstance(v, Expr):
            return v
        if isinstance(v, (int, np.integer)):
            return self.const(v)
        return self.scalar(v)  # a sequence of four words

    def ef(self, x):
        """E::EF::from(base): the secure value (x, 0, 0, 0), as the symbolic evaluator builds it (expr/mod.rs:105-114)."""
        z = self.const(0)
        return self.emit(PACK, x.idx, z.idx, z.idx, z.idx, ext=True)

    def combine_ef(self, values):
        a, b, c, d = values
        return self.emit(PACK, a.idx, b.idx, c.idx, d.idx, ext=True)

    # ---- EvalAtRow
    def next_interaction_mask(self, interaction, offsets):
        col = self.column_index_per_interaction[interaction]
        self.column_index_per_interaction[interaction] += 1
        return [self.emit(LOAD, interaction, col, int(off)) for off in offsets]

    def next_trace_mask(self):
        return self.next_interaction_mask(ORIGINAL_TRACE_IDX, [0])[0]

    def get_preprocessed_column(self, _column_id=None):
        return self.next_interaction_mask(PREPROCESSED_TRACE_IDX, [0])[0]

    def next_extension_interaction_mask(self, interaction, offsets):
        cols = [self.next_interaction_mask(interaction, offsets) for _ in range(4)]
        return [self.combine_ef([cols[k][j] for k in range(4)]) for j in range(len(offsets))]

    def add_constraint(self, c):
        self.constraints.append(self.lift(c).idx)

    def add_to_relation(self, relation, multiplicity, values):
        self.fracs.append((self.lift(multiplicity), relation.combine(self, values)))

    def _sum_fracs(self, fracs):
        num, den = fracs[0]
        for n2, d2 in fracs[1:]:
            num, den = d2 * num + den * n2, den * d2  # core/fraction.rs:27-33
        return num, den

    def finalize_logup_batched(self, batching):
        assert len(batching) == len(self.fracs), "Batching must be of the same length as the number of entries"
        last_batch = max(batching)
        by_batch = [[f for b, f in zip(batching, self.fracs) if b == k] for k in range(last_batch + 1)]
        assert all(by_batch), "Batching must contain all consecutive batches"
        prev_col_cumsum = None
        for k in range(last_batch):
            num, den = self._sum_fracs(by_batch[k])
            (cur,) = self.next_extension_interaction_mask(self.logup_interaction, [0])
            diff = cur if prev_col_cumsum is None else cur - prev_col_cumsum
            prev_col_cumsum = cur
            self.add_constraint(diff * den - num)
        num, den = self._sum_fracs(by_batch[last_batch])
        prev_row, cur = self.next_extension_interaction_mask(self.logup_interaction, [-1, 0])
        diff = cur - prev_row
        if prev_col_cumsum is not None:
            diff = diff - prev_col_cumsum
        self.add_constraint((diff + self.cumsum_shift()) * den - num)
        self.fracs = []

    def finalize_logup(self):
        self.finalize_logup_batched(list(range(len(self.fracs))))

    def finalize_logup_in_pairs(self):
        self.finalize_logup_batched([i // 2 for i in range(len(self.fracs))])

    # ---- result
    def source(self):
        assert not self.fracs, "LogupAtRow was not finalized"
        return AirSource(np.array(self.ops, dtype=np.uint32).reshape(-1, 5), np.array(self.constraints, dtype=np.uint32),
                         np.array(self.column_index_per_interaction, dtype=np.uint32),
                         np.array(self.scalars, dtype=np.uint32).reshape(-1, 4))


class AirSource:
    """ops (n, 5) uint32; constraints (k,) uint32; tree_cols (n_trees,) uint32; scalars (s, 4) uint32."""

    def __init__(self, ops, constraints, tree_cols, scalars):
        self.ops, self.constraints, self.tree_cols, self.scalars = ops, constraints, tree_cols, scalars

    @property
    def n_constraints(self):
        return len(self.constraints)


# ------------------------------------------------------------------------------------------------ AIRs of the reference

def wide_fibonacci(ev, n_cols):
    """nitroo/crates/examples/src/wide_fibonacci/mod.rs:47-57"""
    a, b = ev.next_trace_mask(), ev.next_trace_mask()
    for _ in range(2, n_cols):
        c = ev.next_trace_mask()
        ev.add_constraint(c - (a.square() + b.square()))
        a, b = b, c
    return ev


def plonk(ev, z, alpha_powers):
    """nitroo/crates/examples/src/plonk/mod.rs:51-88"""
    rel = Relation(ev, z, alpha_powers)
    a_wire, b_wire, c_wire, op = (ev.get_preprocessed_column() for _ in range(4))
    mult, a_val, b_val, c_val = (ev.next_trace_mask() for _ in range(4))
    ev.add_constraint(c_val - op * (a_val + b_val) + (1 - op) * a_val * b_val)
    one = ev.ef(ev.const(1))
    ev.add_to_relation(rel, one, [a_wire, a_val])
    ev.add_to_relation(rel, one, [b_wire, b_val])
    ev.add_to_relation(rel, ev.ef(-mult), [c_wire, c_val])
    ev.finalize_logup_in_pairs()
    return ev


def freivalds(ev, pk, pq, n_mats, rv_pow, rv_step, s_pow, s_step, claimed, act_off=128, range_rel=None):
    """prover/src/gadgets/freivalds/mod.rs:114-186 without the optional activation claim. `off_sum`, a value of the
    statement's scalars alone, is computed by the caller-side scalars exactly as the reference computes it on the host."""
    nofirst, last, notzero, end = (ev.get_preprocessed_column() for _ in range(4))
    ws = [[ev.get_preprocessed_column() for _ in range(pk)] for _ in range(n_mats)]
    acts = [ev.next_trace_mask() for _ in range(pq)]
    v_prev, v = ev.next_extension_interaction_mask(INTERACTION_TRACE_IDX, [-1, 0])
    s_pow_e = [ev.scalar(s) for s in s_pow]
    rv_pow_e = [ev.scalar(r) for r in rv_pow]
    s_step_e, rv_step_e = ev.scalar(s_step), ev.scalar(rv_step)
    vf = None
    for p, a in enumerate(acts):
        t = a * s_pow_e[p]
        vf = t if vf is None else vf + t
    off_sum = None
    for s in s_pow_e:
        off_sum = s if off_sum is None else off_sum + s
    off_sum = off_sum * ev.combine_ef([ev.const(act_off), ev.const(0), ev.const(0), ev.const(0)])
    vf = vf - off_sum
    ev.add_constraint(v - (v_prev * s_step_e) * nofirst - vf)
    for m in range(n_mats):
        u_prev, u = ev.next_extension_interaction_mask(INTERACTION_TRACE_IDX, [-1, 0])
        acc_prev, acc = ev.next_extension_interaction_mask(INTERACTION_TRACE_IDX, [-1, 0])
        uf = None
        for p, w in enumerate(ws[m]):
            t = w * rv_pow_e[p]
            uf = t if uf is None else uf + t
        ev.add_constraint(u - (u_prev * rv_step_e) * nofirst - uf)
        ev.add_constraint(acc - acc_prev * notzero - (u * v) * last)
        ev.add_constraint((acc - ev.claim(claimed[m])) * end)
    if range_rel is not None:
        rel = Relation(ev, range_rel[0], [range_rel[1]])
        one = ev.ef(ev.const(1))
        for a in acts:
            ev.add_to_relation(rel, one, [a])
        ev.finalize_logup_in_pairs()
    return ev
