// Lowers a single-assignment AIR program (include/zkb200_air.h) to the bytecode of csrc/constraints.cu.
//
// The input has the instruction set of the reference's own lowering of a FrameworkEval (`Op`,
// prover/src/cudagen.rs:270-300). What happens here:
//   1. kinds: every value is base-field or secure-field. A secure-field instruction whose operands are all base
//      values stays a base value (its upper three coordinates are zero), and PACK(x, 0, 0, 0) is x itself - the
//      reference's generator tracks the same thing as `width` (cudagen.rs:308-310). That turns most of an AIR's
//      "secure" arithmetic into 1- or 4-multiplication forms instead of 16.
//   2. row-independent instructions (literals, run-time scalars and everything computed from them alone) are taken
//      out of the per-row code; the host evaluates them once per call into a table every row reads.
//   3. dead instructions are dropped, repeated loads of one (column, offset) are merged.
//   4. a multiplication read only by one addition or subtraction is folded into it, and an instruction whose result
//      is a constraint also adds it to the row's sum (and skips the store when nothing else reads it).
//   5. loads are issued in batches of up to 8, each batch just before its first value is needed, so that a row has
//      several column reads in flight while its register footprint stays small.
//   6. registers (words of shared memory per row) are assigned by a linear scan over the final instruction order;
//      an operand that dies at an instruction gives its words to the result.
#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../air_program.hpp"

namespace zk {
namespace {

int arity(uint32_t op) {
    switch (op) {
        case ZKB_AIR_LOAD: case ZKB_AIR_CONST_M31: case ZKB_AIR_SCALAR: case ZKB_AIR_CUMSUM_SHIFT: return 0;
        case ZKB_AIR_NEG_B: case ZKB_AIR_NEG_E: case ZKB_AIR_INV_B: return 1;
        case ZKB_AIR_PACK: return 4;
        default: return 2;
    }
}

uint32_t operand(const zkb_air_op& o, int k) { return k == 0 ? o.a : k == 1 ? o.b : k == 2 ? o.c : o.d; }

struct WordPool {
    std::vector<uint8_t> used;
    uint32_t high = 0;
    uint32_t take(uint32_t n) {
        for (uint32_t s = 0;; s++) {
            if (used.size() < (size_t)s + n) used.resize((size_t)s + n, 0);
            uint32_t k = 0;
            while (k < n && !used[s + k]) k++;
            if (k == n) {
                for (k = 0; k < n; k++) used[s + k] = 1;
                high = std::max(high, s + n);
                return s;
            }
            s += k;  // skip past the occupied word
        }
    }
    void give(uint32_t s, uint32_t n) {
        for (uint32_t k = 0; k < n; k++) used[s + k] = 0;
    }
};

// An operand before the shared-memory layout is known: a register slot or a word of the uniform table.
struct Sym {
    bool reg = false;
    uint32_t idx = 0;
};
struct SymInstr {
    uint32_t op = BC_END, n = 0, dst = 0;
    bool has_dst = false;
    int64_t coef = -1;  // constraint whose coefficient multiplies the result (or the operand of an ACC instruction)
    Sym a, b, c;
    std::vector<std::pair<uint32_t, uint32_t>> loads;  // (column | offset << 20, dst slot)
};

}  // namespace

std::string air_compile(zkb_air_program& P, const zkb_air_op* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints,
                        const uint32_t* tree_cols, int n_trees, size_t n_scalars) {
    if (n_ops == 0 || n_ops > (1u << 24)) return "the program must have between 1 and 2^24 instructions";
    if (n_constraints == 0 || n_constraints > (1u << 20)) return "the program must have between 1 and 2^20 constraints";
    const uint32_t N = (uint32_t)n_ops;
    P.ops.assign(ops, ops + N);
    P.ext.assign(N, 0);
    P.uniform.assign(N, 0);
    P.live.assign(N, 0);
    P.alias.resize(N);
    P.uni_word.assign(N, -1);
    P.n_scalars = n_scalars;
    P.tree_base.clear();
    uint64_t total_cols = 0;
    for (int t = 0; t < n_trees; t++) {
        P.tree_base.push_back((uint32_t)total_cols);
        total_cols += tree_cols[t];
    }
    if (total_cols >= AIR_MAX_COLUMNS) return "too many columns";
    P.n_cols = (uint32_t)total_cols;

    // ---- 1. validate, resolve aliases, infer kinds and row dependence
    std::map<std::pair<uint32_t, int32_t>, uint32_t> load_of;
    auto err_at = [](uint32_t i, const char* what) { return "instruction " + std::to_string(i) + ": " + what; };
    for (uint32_t i = 0; i < N; i++) {
        zkb_air_op& o = P.ops[i];
        P.alias[i] = i;
        const int ar = arity(o.op);
        if (o.op > ZKB_AIR_INV_B) return err_at(i, "unknown opcode");
        uint32_t r[4] = {0, 0, 0, 0};
        for (int k = 0; k < ar; k++) {
            uint32_t v = operand(o, k);
            if (v >= i) return err_at(i, "an operand is not an earlier instruction");
            r[k] = P.alias[v];
        }
        if (ar >= 1) o.a = r[0];
        if (ar >= 2) o.b = r[1];
        if (ar == 4) { o.c = r[2]; o.d = r[3]; }
        bool any_ext = false, all_uni = true;
        for (int k = 0; k < ar; k++) {
            any_ext = any_ext || P.ext[r[k]];
            all_uni = all_uni && P.uniform[r[k]];
        }
        switch (o.op) {
            case ZKB_AIR_LOAD: {
                if (o.a >= (uint32_t)n_trees || o.b >= tree_cols[o.a]) return err_at(i, "LOAD names a column outside the trees given");
                const int32_t off = (int32_t)o.c;
                if (off > AIR_MAX_OFFSET || off < -AIR_MAX_OFFSET) return err_at(i, "mask offset out of range");
                auto key = std::make_pair(P.tree_base[o.a] + o.b, off);
                auto it = load_of.find(key);
                if (it != load_of.end()) P.alias[i] = it->second;
                else load_of[key] = i;
                break;
            }
            case ZKB_AIR_CONST_M31:
                if (o.a >= zk::P) return err_at(i, "literal is not a canonical M31 value");
                P.uniform[i] = 1;
                break;
            case ZKB_AIR_SCALAR:
                if (o.a >= n_scalars) return err_at(i, "scalar slot out of range");
                P.uniform[i] = 1;
                P.ext[i] = 1;
                break;
            case ZKB_AIR_CUMSUM_SHIFT:
                P.uniform[i] = 1;
                P.ext[i] = 1;
                break;
            case ZKB_AIR_ADD_B: case ZKB_AIR_SUB_B: case ZKB_AIR_MUL_B: case ZKB_AIR_NEG_B: case ZKB_AIR_INV_B:
                if (any_ext) return err_at(i, "secure-field operand where a base-field value is required");
                P.uniform[i] = all_uni;
                break;
            case ZKB_AIR_ADD_E: case ZKB_AIR_SUB_E: case ZKB_AIR_MUL_E: case ZKB_AIR_NEG_E:
                P.ext[i] = any_ext;
                P.uniform[i] = all_uni;
                break;
            case ZKB_AIR_PACK: {
                if (any_ext) return err_at(i, "PACK takes base-field values");
                auto zero = [&](uint32_t v) { return P.ops[v].op == ZKB_AIR_CONST_M31 && P.ops[v].a == 0; };
                if (zero(r[1]) && zero(r[2]) && zero(r[3])) P.alias[i] = r[0];
                else { P.ext[i] = 1; P.uniform[i] = all_uni; }
                break;
            }
        }
        if (P.alias[i] != i) { P.ext[i] = P.ext[P.alias[i]]; P.uniform[i] = P.uniform[P.alias[i]]; }
    }
    P.constraints.resize(n_constraints);
    for (size_t k = 0; k < n_constraints; k++) {
        if (constraints[k] >= N) return "constraint " + std::to_string(k) + " is not an instruction";
        P.constraints[k] = P.alias[constraints[k]];
    }

    // ---- 2. liveness
    {
        std::vector<uint32_t> stack(P.constraints.begin(), P.constraints.end());
        while (!stack.empty()) {
            uint32_t i = stack.back();
            stack.pop_back();
            if (P.live[i]) continue;
            P.live[i] = 1;
            for (int k = 0; k < arity(P.ops[i].op); k++) stack.push_back(operand(P.ops[i], k));
        }
    }

    // ---- 3. the bytecode form of every per-row instruction. A multiplication whose only reader is an addition or a
    //         subtraction is folded into it (a * b + c, a * b - c, c - a * b; for secure values the forms with one
    //         base factor), which saves its store and reload.
    std::vector<std::vector<uint32_t>> cons_of(N);
    for (uint32_t k = 0; k < n_constraints; k++) cons_of[P.constraints[k]].push_back(k);
    auto per_row_compute = [&](uint32_t i) { return P.live[i] && !P.uniform[i] && P.alias[i] == i && P.ops[i].op != ZKB_AIR_LOAD; };
    std::vector<uint32_t> uses(N, 0);
    for (uint32_t i = 0; i < N; i++)
        if (per_row_compute(i))
            for (int k = 0; k < arity(P.ops[i].op); k++) uses[operand(P.ops[i], k)]++;
    enum Cls { ADD, SUB, MUL, NEG, INV, PACKC };
    auto cls_of = [](uint32_t op) {
        switch (op) {
            case ZKB_AIR_ADD_B: case ZKB_AIR_ADD_E: return ADD;
            case ZKB_AIR_SUB_B: case ZKB_AIR_SUB_E: return SUB;
            case ZKB_AIR_MUL_B: case ZKB_AIR_MUL_E: return MUL;
            case ZKB_AIR_INV_B: return INV;
            case ZKB_AIR_PACK: return PACKC;
            default: return NEG;
        }
    };
    struct Form { uint32_t bc = BC_END; int n = 0; uint32_t src[4] = {0, 0, 0, 0}; };
    std::vector<Form> form(N);
    std::vector<uint8_t> folded(N, 0);
    auto foldable_mul = [&](uint32_t m, bool want_ext) {
        if (!per_row_compute(m) || cls_of(P.ops[m].op) != MUL || uses[m] != 1 || !cons_of[m].empty()) return false;
        if (!want_ext) return !P.ext[m];
        return P.ext[m] && P.ext[P.ops[m].a] != P.ext[P.ops[m].b];  // exactly one secure factor
    };
    uint64_t mults = 0;
    for (uint32_t i = 0; i < N; i++) {
        if (!per_row_compute(i)) continue;
        const zkb_air_op& o = P.ops[i];
        const Cls cls = cls_of(o.op);
        Form f;
        if (cls == PACKC) {
            f.bc = BC_MOV_B;
            f.n = 4;
            f.src[0] = o.a; f.src[1] = o.b; f.src[2] = o.c; f.src[3] = o.d;
            form[i] = f;
            continue;
        }
        if ((cls == ADD || cls == SUB) && o.a != o.b) {
            const bool we = P.ext[i];
            uint32_t m = N;
            bool m_is_b = false;
            if (foldable_mul(o.b, we) && (!we || P.ext[o.a])) { m = o.b; m_is_b = true; }
            else if (foldable_mul(o.a, we) && (!we || P.ext[o.b]) && (cls == ADD || !we)) m = o.a;
            if (m < N) {
                uint32_t fa = P.ops[m].a, fb = P.ops[m].b;
                if (we && !P.ext[fa]) std::swap(fa, fb);  // the secure factor first
                if (cls == ADD) f.bc = we ? BC_FMA_EB : BC_FMA_B;
                else if (m_is_b) f.bc = we ? BC_FNMS_EB : BC_FNMS_B;
                else f.bc = BC_FMS_B;
                f.n = 3;
                f.src[0] = fa; f.src[1] = fb; f.src[2] = m_is_b ? o.a : o.b;
                folded[m] = 1;
                mults += we ? 4 : 1;
                form[i] = f;
                continue;
            }
        }
        const int ar = arity(o.op);
        const bool ea = P.ext[o.a], eb = ar == 2 ? (bool)P.ext[o.b] : false;
        uint32_t s0 = o.a, s1 = ar == 2 ? o.b : 0;
        switch (cls) {
            case ADD:
                f.bc = ea && eb ? BC_ADD_EE : !ea && !eb ? BC_ADD_BB : BC_ADD_EB;
                if (!ea && eb) std::swap(s0, s1);
                break;
            case SUB: f.bc = ea && eb ? BC_SUB_EE : !ea && !eb ? BC_SUB_BB : ea ? BC_SUB_EB : BC_SUB_BE; break;
            case MUL:
                f.bc = ea && eb ? BC_MUL_EE : !ea && !eb ? BC_MUL_BB : BC_MUL_EB;
                if (!ea && eb) std::swap(s0, s1);
                break;
            case NEG: f.bc = ea ? BC_NEG_E : BC_NEG_B; break;
            case INV: f.bc = BC_INV_B; break;
            default: break;
        }
        f.n = ar;
        f.src[0] = s0; f.src[1] = s1;
        form[i] = f;
    }
    for (uint32_t i = 0; i < N; i++) {  // multiplications that stayed instructions of their own
        if (!per_row_compute(i) || folded[i]) continue;
        if (form[i].bc == BC_MUL_BB) mults += 1;
        else if (form[i].bc == BC_MUL_EB) mults += 4;
        else if (form[i].bc == BC_MUL_EE) mults += 16;
        else if (form[i].bc == BC_INV_B) mults += 37;
    }

    // ---- 4. order of the per-row work: instructions in program order; a constraint is accumulated by the
    //         instruction that computes it where that instruction has a free operand field, else right after it
    struct Item { int kind; uint32_t idx; };  // 0 compute, 1 accumulate constraint idx, 2 load batch [idx, n), 3 fold row_res
    std::vector<int64_t> acc_fused(N, -1);
    std::vector<uint8_t> nostore(N, 0);
    std::vector<Item> items;
    for (uint32_t i = 0; i < N; i++) {
        if (!per_row_compute(i) || folded[i]) continue;
        items.push_back({0, i});
        size_t first = 0;
        if (!cons_of[i].empty() && form[i].n <= 2) {
            acc_fused[i] = cons_of[i][0];
            nostore[i] = uses[i] == 0 && cons_of[i].size() == 1;
            first = 1;
        }
        for (size_t q = first; q < cons_of[i].size(); q++) items.push_back({1, cons_of[i][q]});
    }
    for (uint32_t k = 0; k < n_constraints; k++) {
        uint32_t v = P.constraints[k];
        if (P.uniform[v] || P.ops[v].op == ZKB_AIR_LOAD) items.push_back({1, k});
    }
    auto reads = [&](const Item& it, uint32_t out[4]) -> int {
        if (it.kind == 1) { out[0] = P.constraints[it.idx]; return 1; }
        if (it.kind != 0) return 0;
        for (int k = 0; k < form[it.idx].n; k++) out[k] = form[it.idx].src[k];
        return form[it.idx].n;
    };
    // loads by first use
    std::vector<int64_t> first_use(N, -1);
    for (size_t j = 0; j < items.size(); j++) {
        uint32_t rd[4];
        int n = reads(items[j], rd);
        for (int k = 0; k < n; k++)
            if (P.ops[rd[k]].op == ZKB_AIR_LOAD && first_use[rd[k]] < 0) first_use[rd[k]] = (int64_t)j;
    }
    std::vector<uint32_t> loads;
    for (uint32_t i = 0; i < N; i++)
        if (P.ops[i].op == ZKB_AIR_LOAD && P.alias[i] == i && P.live[i]) loads.push_back(i);
    std::stable_sort(loads.begin(), loads.end(), [&](uint32_t x, uint32_t y) { return first_use[x] < first_use[y]; });
    std::vector<Item> order;
    std::vector<uint32_t> batch_len;
    {
        size_t p = 0;
        int units = 0;  // base-field constraints added to row_res since it was last folded (each below 2^62)
        for (size_t j = 0; j < items.size(); j++) {
            while (p < loads.size() && first_use[loads[p]] <= (int64_t)j) {
                uint32_t n = (uint32_t)std::min<size_t>(AIR_LOAD_BATCH, loads.size() - p);
                order.push_back({2, (uint32_t)p});
                batch_len.resize(order.size(), 0);
                batch_len.back() = n;
                p += n;
            }
            const Item& it = items[j];
            const bool adds_base = (it.kind == 1 && !P.ext[P.constraints[it.idx]]) || (it.kind == 0 && acc_fused[it.idx] >= 0 && !P.ext[it.idx]);
            if (adds_base) {
                if (units == 3) { order.push_back({3, 0}); units = 0; }
                units++;
            }
            order.push_back(it);
            batch_len.resize(order.size(), 0);
        }
    }

    // ---- 5. last reads, then registers
    std::vector<int64_t> last_use(N, -1);
    for (size_t j = 0; j < order.size(); j++) {
        uint32_t rd[4];
        int n = reads(order[j], rd);
        for (int k = 0; k < n; k++) last_use[rd[k]] = (int64_t)j;
    }
    std::vector<int64_t> slot(N, -1);
    WordPool pool;
    uint32_t uni_words = 0;
    auto sym = [&](uint32_t v) {
        Sym s;
        if (P.uniform[v]) {
            if (P.uni_word[v] < 0) {
                P.uni_word[v] = (int32_t)uni_words;
                uni_words += P.ext[v] ? 4 : 1;
            }
            s.idx = (uint32_t)P.uni_word[v];
        } else {
            s.reg = true;
            s.idx = (uint32_t)slot[v];
        }
        return s;
    };
    auto release = [&](uint32_t v, int64_t j) {
        if (!P.uniform[v] && slot[v] >= 0 && last_use[v] == j) {
            pool.give((uint32_t)slot[v], P.ext[v] ? 4 : 1);
            slot[v] = -1;
        }
    };
    std::vector<SymInstr> sym_code;
    std::vector<uint8_t> col_read(P.n_cols, 0);
    for (size_t j = 0; j < order.size(); j++) {
        const Item& it = order[j];
        SymInstr si;
        if (it.kind == 3) {
            si.op = BC_ACC_RED;
            sym_code.push_back(si);
            continue;
        }
        if (it.kind == 2) {
            si.op = BC_LOAD;
            si.n = batch_len[j];
            for (uint32_t q = 0; q < si.n; q++) {
                uint32_t v = loads[it.idx + q];
                const zkb_air_op& o = P.ops[v];
                uint32_t col = P.tree_base[o.a] + o.b;
                int32_t off = (int32_t)o.c;
                col_read[col] = 1;
                slot[v] = pool.take(1);
                si.loads.push_back({col | ((uint32_t)off << 20), (uint32_t)slot[v]});
            }
            sym_code.push_back(si);
            continue;
        }
        if (it.kind == 1) {
            uint32_t v = P.constraints[it.idx];
            si.op = P.ext[v] ? BC_ACC_E : BC_ACC_B;
            si.a = sym(v);
            si.coef = (int64_t)it.idx;
            mults += P.ext[v] ? 16 : 4;
            sym_code.push_back(si);
            release(v, (int64_t)j);
            continue;
        }
        const uint32_t i = it.idx;
        const Form& f = form[i];
        if (f.bc == BC_MOV_B) {  // PACK: four moves into a fresh secure register
            slot[i] = pool.take(4);
            for (int k = 0; k < 4; k++) {
                SymInstr mv;
                mv.op = BC_MOV_B;
                mv.has_dst = true;
                mv.dst = (uint32_t)slot[i] + k;
                mv.a = sym(f.src[k]);
                sym_code.push_back(mv);
            }
            for (int k = 0; k < 4; k++) release(f.src[k], (int64_t)j);
            continue;
        }
        si.op = f.bc;
        si.a = sym(f.src[0]);
        if (f.n >= 2) si.b = sym(f.src[1]);
        if (f.n >= 3) si.c = sym(f.src[2]);
        for (int k = 0; k < f.n; k++) release(f.src[k], (int64_t)j);  // release() is a no-op the second time
        if (acc_fused[i] >= 0) {
            si.coef = acc_fused[i];
            mults += P.ext[i] ? 16 : 4;
        }
        if (!nostore[i]) {
            slot[i] = pool.take(P.ext[i] ? 4 : 1);
            si.has_dst = true;
            si.dst = (uint32_t)slot[i];
        }
        sym_code.push_back(si);
        if (last_use[i] < 0 && slot[i] >= 0) {  // stored for a later ACC only; cannot happen, but never leak a register
            pool.give((uint32_t)slot[i], P.ext[i] ? 4 : 1);
            slot[i] = -1;
        }
    }

    // ---- 6. shared-memory layout, CTA size, rows per thread
    P.reg_words = std::max<uint32_t>(pool.high, 1);
    P.coef_base = uni_words;
    uint32_t table = uni_words + 4 * (uint32_t)n_constraints;
    table += table & 1;
    P.ptr_base = table;
    P.reg_base = P.ptr_base + 2 * P.n_cols;
    const uint64_t budget = 227 * 1024;
    auto smem_of = [&](uint32_t t, uint32_t rpt) { return 4ull * (P.reg_base + (uint64_t)P.reg_words * t * rpt); };
    P.threads = 0;
    if (smem_of(256, 4) + 1024 <= budget / 2) {
        P.threads = 256; P.rows_per_thread = 4; P.ctas_per_sm = 2;
    } else if (smem_of(256, 2) + 1024 <= budget / 2) {
        P.threads = 256; P.rows_per_thread = 2;
        P.ctas_per_sm = (uint32_t)std::min<uint64_t>(3, budget / (smem_of(256, 2) + 1024));
    } else {
        uint32_t best_resident = 0;
        for (uint32_t t : {256u, 128u, 64u, 32u}) {
            uint64_t bytes = smem_of(t, 1);
            if (bytes + 1024 > budget) continue;
            uint32_t ctas = (uint32_t)std::min<uint64_t>({budget / (bytes + 1024), 1024 / t, 16});
            ctas = std::max(ctas, 1u);
            if (ctas * t > best_resident) { best_resident = ctas * t; P.threads = t; P.ctas_per_sm = ctas; }
        }
        P.rows_per_thread = 1;
    }
    if (!P.threads)
        return "the program keeps " + std::to_string(P.reg_words) + " words alive per row and reads " + std::to_string(P.n_cols) +
               " columns: more than one CTA's shared memory holds";
    const uint32_t RP = P.threads * P.rows_per_thread;
    P.smem_bytes = (uint32_t)smem_of(P.threads, P.rows_per_thread);

    // ---- 7. encode
    auto enc = [&](const Sym& s) { return s.reg ? ((P.reg_base + s.idx * RP) << 1) | 1u : (s.idx << 1); };
    P.code.clear();
    for (const SymInstr& si : sym_code) {
        if (si.op == BC_LOAD) {
            P.code.push_back({BC_LOAD | (si.n << 8), 0, 0, 0});
            for (uint32_t q = 0; q < si.n; q += 2) {
                AirInstr e{si.loads[q].first, P.reg_base + si.loads[q].second * RP, 0, 0};
                if (q + 1 < si.n) { e.z = si.loads[q + 1].first; e.w = P.reg_base + si.loads[q + 1].second * RP; }
                P.code.push_back(e);
            }
            continue;
        }
        AirInstr e{si.op, enc(si.a), enc(si.b), enc(si.c)};
        if (si.has_dst) e.x |= (P.reg_base + si.dst * RP) << 8;
        else if (si.op >= BC_ADD_BB) e.x |= BC_F_NOSTORE;
        if (si.coef >= 0) {
            e.w = (P.coef_base + 4 * (uint32_t)si.coef) << 1;
            if (si.op >= BC_ADD_BB) e.x |= BC_F_ACC;
        }
        P.code.push_back(e);
    }
    P.code.push_back({BC_END, 0, 0, 0});
    P.code.push_back({BC_END, 0, 0, 0});

    zkb_air_stats& st = P.stats;
    st.n_ops = N;
    st.n_live_ops = 0;
    st.n_uniform = 0;
    for (uint32_t i = 0; i < N; i++) {
        if (!P.live[i] || P.alias[i] != i) continue;
        st.n_live_ops++;
        if (P.uniform[i]) st.n_uniform++;
    }
    st.n_instr = (uint32_t)sym_code.size();
    st.n_loads = (uint32_t)loads.size();
    st.n_columns_read = (uint32_t)std::count(col_read.begin(), col_read.end(), 1);
    st.reg_words = P.reg_words;
    st.uniform_words = P.ptr_base;
    st.threads = P.threads;
    st.rows_per_thread = P.rows_per_thread;
    st.smem_bytes = P.smem_bytes;
    st.m31_mults = (uint32_t)std::min<uint64_t>(mults, 0xffffffffu);
    return "";
}

void air_fill_uniform(const zkb_air_program& P, const uint32_t* scalars, const uint32_t* cumsum_shift,
                      const uint32_t* random_coeff_powers, uint32_t* table) {
    const uint32_t N = (uint32_t)P.ops.size();
    std::vector<qm31> val(N, qm31_zero());
    for (uint32_t i = 0; i < N; i++) {
        if (!P.live[i] || !P.uniform[i] || P.alias[i] != i) continue;
        const zkb_air_op& o = P.ops[i];
        qm31 r = qm31_zero();
        switch (o.op) {
            case ZKB_AIR_CONST_M31: r = qm31_from_m31(o.a); break;
            case ZKB_AIR_SCALAR: for (int k = 0; k < 4; k++) r.c[k] = scalars[4 * (size_t)o.a + k]; break;
            case ZKB_AIR_CUMSUM_SHIFT: if (cumsum_shift) for (int k = 0; k < 4; k++) r.c[k] = cumsum_shift[k]; break;
            case ZKB_AIR_ADD_B: case ZKB_AIR_ADD_E: r = qm31_add(val[o.a], val[o.b]); break;
            case ZKB_AIR_SUB_B: case ZKB_AIR_SUB_E: r = qm31_sub(val[o.a], val[o.b]); break;
            case ZKB_AIR_MUL_B: case ZKB_AIR_MUL_E: r = qm31_mul(val[o.a], val[o.b]); break;
            case ZKB_AIR_NEG_B: case ZKB_AIR_NEG_E: r = qm31_neg(val[o.a]); break;
            case ZKB_AIR_INV_B: r = qm31_from_m31(m31_inv(val[o.a].c[0])); break;
            case ZKB_AIR_PACK: r = {{val[o.a].c[0], val[o.b].c[0], val[o.c].c[0], val[o.d].c[0]}}; break;
            default: break;
        }
        val[i] = r;
        if (P.uni_word[i] >= 0) {
            table[P.uni_word[i]] = r.c[0];
            if (P.ext[i]) for (int k = 1; k < 4; k++) table[P.uni_word[i] + k] = r.c[k];
        }
    }
    for (size_t k = 0; k < P.constraints.size(); k++)
        for (int q = 0; q < 4; q++) table[P.coef_base + 4 * k + q] = random_coeff_powers[4 * k + q];
    if ((P.coef_base + 4 * P.constraints.size()) & 1) table[P.ptr_base - 1] = 0;
}

}  // namespace zk
