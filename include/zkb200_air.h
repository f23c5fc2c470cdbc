/* zkb200_air.h - constraint-quotient evaluation of a lowered AIR on the evaluation domain.
 *
 * This is the ComponentProver<B>::evaluate_constraint_quotients_on_domain step of the reference
 * (nitroo/crates/constraint-framework/src/prover/component_prover.rs:296-600; the CPU statement is
 * accumulate_pointwise_cpu, :603-633, over CpuDomainEvaluator, prover/cpu_domain.rs:17-98). The reference's CUDA
 * backend answers it with one generated kernel per AIR shape, selected by a hash of the component name
 * (stwo_cuda/bindings.rs:557-578, generator prover/src/cudagen.rs). Here ONE kernel serves every AIR: the caller
 * hands over the AIR as straight-line code in single-assignment form - the same instruction set as the
 * reference's own lowering (`Op`, prover/src/cudagen.rs:270-300) - and the library compiles it once into a
 * register-allocated bytecode that a persistent kernel interprets, one evaluation-domain row per thread, with the
 * per-row values held in shared memory.
 *
 * Per row of the evaluation domain (bit-reversed circle-domain order, as every column of the library):
 *     row_res = sum_i random_coeff_powers[i] * constraint_i(mask values at this row)
 *     accum[row] = (accumulate ? accum[row] : 0) + row_res * denom_inv[row >> trace_log]
 * A mask value at offset `off` of a column is the column at
 * offset_bit_reversed_circle_domain_index(row, trace_log, eval_log, off) (core/utils.rs:97-113).
 *
 * All values are canonical M31 words; a secure-field (QM31) value is 4 words. Status codes as in zkb200.h.
 */
#ifndef ZKB200_AIR_H
#define ZKB200_AIR_H

#include "zkb200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* One instruction of the single-assignment program. Operands a..d are indices of EARLIER instructions, except where
 * stated. "B" values are base-field (M31), "E" values are secure-field (QM31); an E instruction accepts B operands
 * and promotes them (value, 0, 0, 0), as the reference's interpreter does (prover/src/cudagen.rs:1217-1262). */
enum zkb_air_opcode {
    ZKB_AIR_LOAD = 0,         /* a = tree, b = column within the tree, c = mask offset (int32 bit pattern) -> B */
    ZKB_AIR_CONST_M31 = 1,    /* a = literal in [0, p) -> B */
    ZKB_AIR_SCALAR = 2,       /* a = slot of the run-time scalar array -> E */
    ZKB_AIR_CUMSUM_SHIFT = 3, /* the LogUp shift claimed_sum / 2^log_size (logup.rs:33-41), a run-time argument -> E */
    ZKB_AIR_ADD_B = 4,
    ZKB_AIR_SUB_B = 5,
    ZKB_AIR_MUL_B = 6,
    ZKB_AIR_NEG_B = 7,
    ZKB_AIR_ADD_E = 8,
    ZKB_AIR_SUB_E = 9,
    ZKB_AIR_MUL_E = 10,
    ZKB_AIR_NEG_E = 11,
    ZKB_AIR_PACK = 12,        /* four B values -> E (EvalAtRow::combine_ef) */
    ZKB_AIR_INV_B = 13        /* 1/a in M31 (BaseExpr::Inv, expr/mod.rs:53); 0 maps to 0 */
};

typedef struct zkb_air_op {
    uint32_t op, a, b, c, d;
} zkb_air_op;

typedef struct zkb_air_program zkb_air_program;

/* What the compiler made of a program (for reports and roofline arithmetic). */
typedef struct zkb_air_stats {
    uint32_t n_ops;            /* instructions given */
    uint32_t n_live_ops;       /* of those, reachable from a constraint */
    uint32_t n_uniform;        /* live instructions that do not depend on the row: evaluated once per call on the host */
    uint32_t n_instr;          /* bytecode instructions one row executes (a batch of loads counts as one) */
    uint32_t n_loads;          /* distinct (column, offset) loads per row */
    uint32_t n_columns_read;   /* distinct columns read */
    uint32_t reg_words;        /* shared-memory words per row (register file) */
    uint32_t uniform_words;    /* shared-memory words per CTA shared by all rows */
    uint32_t threads;          /* threads per CTA */
    uint32_t rows_per_thread;  /* rows one thread evaluates side by side (1, 2 or 4) */
    uint32_t smem_bytes;       /* dynamic shared memory per CTA */
    uint32_t m31_mults;        /* M31 multiplications per row */
    uint32_t specialized;      /* 1 once zkb_air_specialize has succeeded */
    uint32_t specialized_regs; /* registers per thread of the specialised kernel, 0 if unknown */
} zkb_air_stats;

/* Compiles a program. `constraints[i]` is the instruction whose value is the i-th add_constraint call, in call
 * order (the order random_coeff_powers is indexed in). `tree_cols[t]` is the number of columns the caller will pass
 * for tree t; a LOAD outside that range, a B instruction with an E operand, an operand that is not an earlier
 * instruction, or a program whose live values do not fit the shared memory of one CTA are ZKB_EINVAL with a message
 * in zkb_last_error. The bytecode is uploaded to the context's device; the program can be used with any context of
 * that device, from one thread at a time. */
int zkb_air_compile(zkb_ctx* ctx, const zkb_air_op* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints,
                    const uint32_t* tree_cols, int n_trees, size_t n_scalars, zkb_air_program** out);
int zkb_air_free(zkb_air_program* prog);

/* Optional second step: turns the program into straight-line CUDA in which every per-row value is a register,
 * compiles it for sm_100a with NVRTC (found with dlopen at the first call; nothing links against it) and loads it.
 * This is the run-time counterpart of the reference's per-shape generated kernels (prover/src/cudagen.rs:1985-2290).
 * On success zkb_constraint_quotients uses the specialised kernel; zkb_air_select switches between it (1) and the
 * interpreter (0), whose results are identical. ZKB_ECUDA with a message if NVRTC is absent or the compilation fails:
 * the program stays usable through the interpreter. Takes about a second per thousand instructions. The environment
 * variable ZKB_NVRTC_LIB, read at the first use, names the NVRTC library to load instead of libnvrtc.so.12. */
int zkb_air_specialize(zkb_ctx* ctx, zkb_air_program* prog);
int zkb_air_select(zkb_air_program* prog, int specialized);
int zkb_air_get_stats(const zkb_air_program* prog, zkb_air_stats* out);

/* Host only, no context and no GPU: runs the compiler on a program and reports what it made of it (or why it refused
 * it, in err). With check_specialized non-zero it also generates the specialised kernel's source and compiles it for
 * sm_100a with NVRTC (which needs no device), filling specialized and specialized_regs; ZKB_ECUDA if that fails. */
int zkb_air_analyze(const zkb_air_op* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints, const uint32_t* tree_cols,
                    int n_trees, size_t n_scalars, int check_specialized, zkb_air_stats* out, char* err, size_t err_cap);

/* FrameworkComponent::evaluate_constraint_quotients_on_domain for one component.
 *   cols                 host array of device pointers: the component's columns on the evaluation domain, tree 0's
 *                        columns first, then tree 1's, ... (sum of tree_cols pointers; 2^eval_log words each). A column
 *                        the program never loads may be NULL.
 *   scalars              host, n_scalars x 4 words (the run-time blob of the lowering: relation elements, claims)
 *   cumsum_shift         host, 4 words (NULL = zero)
 *   random_coeff_powers  host, n_constraints x 4 words, entry i multiplies constraint i
 *   denom_inv            host, 2^(eval_log - trace_log) words: the inverses of the trace domain's vanishing polynomial
 *                        on the evaluation domain's cosets, bit-reversed (component_prover.rs:262-266);
 *                        zkb_constraint_denom_inv computes them
 *   accum                4 device columns of 2^eval_log words (secure column by coordinates)
 *   accumulate           non-zero: add to accum (the proving path); zero: overwrite
 * Requires 1 <= trace_log < eval_log <= 30 and eval_log - trace_log <= 16: on the trace domain itself the vanishing
 * polynomial is zero and has no inverse (the reference panics there). Asynchronous on the context's stream. */
int zkb_constraint_quotients(zkb_ctx* ctx, const zkb_air_program* prog, const uint32_t* const* cols, const uint32_t* scalars,
                             const uint32_t* cumsum_shift, const uint32_t* random_coeff_powers, const uint32_t* denom_inv,
                             int trace_log, int eval_log, uint32_t* const accum[4], int accumulate);

/* Requires trace_log < eval_log. denom_inv[j] for j < 2^(eval_log - trace_log): 1 / coset_vanishing(CanonicCoset(trace_log).coset,
 * CanonicCoset(eval_log).circle_domain().at(i)), i < 2^(eval_log - trace_log), then bit-reversed
 * (component_prover.rs:262-266, core/constraints.rs:12-35). Host only. */
int zkb_constraint_denom_inv(int trace_log, int eval_log, uint32_t* out);

#ifdef __cplusplus
}
#endif
#endif
