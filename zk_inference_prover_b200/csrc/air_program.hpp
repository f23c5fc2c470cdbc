// The compiled form of a lowered AIR (see include/zkb200_air.h): what the host evaluates once per call, and the
// bytecode one evaluation-domain row executes on the device.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/zkb200_air.h"
#include "m31.cuh"

namespace zk {

// Bytecode. An instruction is four words {opcode | flags | dst << 8, a, b, c}.
//   dst      word offset of the destination register in shared memory (a thread adds row_in_thread * threads + lane)
//   a, b, c  operands: (word offset << 1) | per_row. A per-row operand is a register (the thread adds its row's lane and
//            steps a secure-field value by the rows of the CTA); a uniform operand is a word of the table every row
//            shares (a secure-field value is 4 consecutive words).
//   flags    BC_F_ACC: the result is a constraint; row_res += coefficient(c) * result (instructions with at most two
//            sources); BC_F_NOSTORE: nothing else reads the result, so it is not written to its register.
// A LOAD instruction is followed by ceil(n / 2) words-quads {column | offset << 20, dst, column | offset << 20, dst}
// with the mask offset as a signed 12-bit field.
// row_res is kept per row as four unreduced 64-bit sums: a base-field constraint adds coefficient * value (< 2^62) to
// each, and BC_ACC_RED, which the compiler emits after every third such addition, folds them back below 2^31.
enum AirBytecode : uint32_t {
    BC_END = 0,
    BC_LOAD = 1,
    BC_ACC_B = 2,   // row_res += coefficient(c) * a (base)
    BC_ACC_E = 3,   // row_res += coefficient(c) * a (secure)
    BC_ACC_RED = 4,
    // base-field results
    BC_ADD_BB = 8,
    BC_SUB_BB = 9,
    BC_MUL_BB = 10,
    BC_NEG_B = 11,
    BC_INV_B = 12,
    BC_MOV_B = 13,
    BC_FMA_B = 14,   // a * b + c
    BC_FMS_B = 15,   // a * b - c
    BC_FNMS_B = 16,  // c - a * b
    // secure-field results
    BC_ADD_EE = 24,
    BC_SUB_EE = 25,
    BC_MUL_EE = 26,
    BC_NEG_E = 27,
    BC_ADD_EB = 28,   // a secure, b base
    BC_SUB_EB = 29,   // a secure - b base
    BC_SUB_BE = 30,   // a base - b secure
    BC_MUL_EB = 31,   // a secure * b base
    BC_FMA_EB = 32,   // c secure + a secure * b base
    BC_FNMS_EB = 33,  // c secure - a secure * b base
};
constexpr uint32_t BC_OP_MASK = 0x3f, BC_F_ACC = 0x40, BC_F_NOSTORE = 0x80;

constexpr int AIR_LOAD_BATCH = 8;
constexpr int AIR_MAX_OFFSET = 2047;      // mask offsets are a signed 12-bit field
constexpr uint32_t AIR_MAX_COLUMNS = 1u << 20;

struct AirInstr {
    uint32_t x, y, z, w;
};

}  // namespace zk

struct zkb_air_program {
    // ---- the single-assignment program, annotated
    std::vector<zkb_air_op> ops;
    std::vector<uint8_t> ext;      // value is a secure-field element (else base field)
    std::vector<uint8_t> uniform;  // value does not depend on the row
    std::vector<uint8_t> live;     // reachable from a constraint
    std::vector<uint32_t> alias;   // instruction whose value this one is (a PACK of (x, 0, 0, 0) is x; a repeated LOAD)
    std::vector<int32_t> uni_word; // word of the uniform table holding this (uniform) value, or -1
    std::vector<uint32_t> constraints;
    std::vector<uint32_t> tree_base;  // first flat column of each tree
    uint32_t n_cols = 0;
    size_t n_scalars = 0;
    // ---- shared-memory layout, in words: [uniform values | coefficients | column pointers | registers]
    uint32_t coef_base = 0;   // 4 words per constraint
    uint32_t ptr_base = 0;    // 2 words per column, 8-byte aligned
    uint32_t reg_base = 0;
    uint32_t reg_words = 0;   // per row
    uint32_t threads = 0;
    uint32_t rows_per_thread = 1;
    uint32_t smem_bytes = 0;
    uint32_t ctas_per_sm = 1;
    // ---- bytecode
    std::vector<zk::AirInstr> code;
    zk::AirInstr* d_code = nullptr;
    int device = -1;
    // ---- optional specialised kernel (csrc/host/air_jit.cpp): cudaLibrary_t / cudaKernel_t handles
    void* jit_library = nullptr;
    void* jit_kernel = nullptr;
    bool use_jit = false;
    zkb_air_stats stats{};
};

namespace zk {

// Fills prog from the caller's program; returns an empty string or the reason it was rejected.
std::string air_compile(zkb_air_program& prog, const zkb_air_op* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints,
                        const uint32_t* tree_cols, int n_trees, size_t n_scalars);

// Evaluates the row-independent instructions and writes the words [0, ptr_base) of the shared table:
// uniform values, then the constraint coefficients.
void air_fill_uniform(const zkb_air_program& prog, const uint32_t* scalars, const uint32_t* cumsum_shift,
                      const uint32_t* random_coeff_powers, uint32_t* table);

// csrc/host/air_jit.cpp: CUDA source of a kernel specialised to the program, and its compilation with NVRTC
// (loaded with dlopen). Both return an empty string on success or the reason.
std::string air_codegen(const zkb_air_program& prog);
std::string air_nvrtc_compile(const std::string& source, std::vector<char>& cubin, std::string* ptxas_info);

}  // namespace zk
