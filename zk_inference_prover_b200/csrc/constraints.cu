// Constraint-quotient evaluation on the evaluation domain: one kernel for every AIR.
//
// Replaces the reference's per-shape generated kernels (dispatch: nitroo/crates/stwo/src/stwo_cuda/bindings.rs:557-578;
// call site: nitroo/crates/constraint-framework/src/prover/component_prover.rs:296-600) and states the same function as
// accumulate_pointwise_cpu (component_prover.rs:603-633) over CpuDomainEvaluator (prover/cpu_domain.rs:52-98).
//
// A CTA owns tiles of threads x rows_per_thread consecutive rows. Each thread interprets the AIR's bytecode
// (csrc/air_program.hpp, produced by csrc/host/air_compile.cpp) for its 1, 2 or 4 rows. The values of a row live in
// shared memory, word w of row r of the tile at [reg_base + w * rows + r], so a warp's access to one register is one
// conflict-free row of banks, and the
// row-independent values (literals, relation elements, random-coefficient powers) sit once per CTA in front of them.
// All threads of a CTA execute the same instruction stream, so the interpreter's dispatch is uniform. Column reads
// are issued in batches of up to 8 independent loads; for a mask offset the 256 rows of a tile map to another run of
// consecutive rows except where the offset carries into the tile's own bits, so those reads coalesce as well.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <string>
#include <vector>

#include "air_program.hpp"
#include "common.cuh"

namespace zk {

struct AccumPtrs {
    uint32_t* c[4];
};

// Row of the column that a mask at `off` of `row` reads (core/utils.rs:97-113): step the natural-order index inside
// its half of the circle domain by off * 2^(eval_log - trace_log - 1), forwards in the first half, backwards in the second.
__device__ __forceinline__ uint32_t offset_row(uint32_t row, int off, int trace_log, int eval_log) {
    if (off == 0) return row;
    const uint32_t nat = __brev(row) >> (32 - eval_log);
    const uint32_t half = 1u << (eval_log - 1);
    const uint32_t step = (uint32_t)off << (eval_log - trace_log - 1);
    const uint32_t lo = (nat & half) ? nat - step : nat + step;
    const uint32_t moved = (lo & (half - 1u)) | (nat & half);
    return __brev(moved) >> (32 - eval_log);
}

// Order in which tiles are taken: consecutive tile numbers (CTAs running at the same time) get row ranges that differ
// in the top three bits of the row index. A mask at offset +-1 reads row +- N/2, N/4, N/8, ... in bit-reversed order, so
// with this order the neighbour rows of a tile are rows another CTA is reading as a mask-0 value at about the same
// time, and most of those reads hit L2 instead of going to DRAM a second time.
__device__ __forceinline__ uint32_t spread_tile(uint32_t t, uint32_t n_tiles) {
    if (n_tiles < 16u || (n_tiles & (n_tiles - 1u))) return t;
    const uint32_t bits = 31u - (uint32_t)__clz(n_tiles);
    return ((t & 7u) << (bits - 3u)) | (t >> 3);
}

extern __shared__ __align__(16) uint32_t air_smem[];

// RPT rows per thread: rows tile * T * RPT + j * T + lane, j < RPT. The instruction fetch, its decoding and the loads
// of uniform operands are paid once for the RPT rows, whose arithmetic is independent.
template <int RPT>
__global__ void __launch_bounds__(256, RPT == 4 ? 2 : RPT == 2 ? 3 : 4)
air_eval_kernel(const uint4* __restrict__ code, const uint32_t* __restrict__ table, uint32_t table_words, uint32_t ptr_base,
                const uint32_t* __restrict__ denom_inv, int trace_log, int eval_log, AccumPtrs accum, int accumulate,
                uint32_t n_tiles) {
    uint32_t* sm = air_smem;
    const uint32_t tid = threadIdx.x, T = blockDim.x, RP = T * RPT;
    for (uint32_t i = tid; i < table_words; i += T) sm[i] = table[i];
    __syncthreads();
    const unsigned long long* ptrs = reinterpret_cast<const unsigned long long*>(sm + ptr_base);
    const uint32_t n_rows = 1u << eval_log;

    // operand readers: word index of row j's copy, and the step between the coordinates of a secure value
    auto at = [&](uint32_t e, int j) -> uint32_t { return (e >> 1) + ((e & 1u) ? tid + j * T : 0u); };
    auto ldb = [&](uint32_t e, int j) -> uint32_t { return sm[at(e, j)]; };
    auto lde = [&](uint32_t e, int j) -> qm31 {
        const uint32_t base = at(e, j), stride = (e & 1u) ? RP : 1u;
        return {{sm[base], sm[base + stride], sm[base + 2 * stride], sm[base + 3 * stride]}};
    };

    for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const uint32_t tile = spread_tile(t, n_tiles);
        uint32_t row[RPT];
        bool active[RPT];
#pragma unroll
        for (int j = 0; j < RPT; j++) {
            const uint32_t r = tile * RP + j * T + tid;
            active[j] = r < n_rows;
            row[j] = active[j] ? r : n_rows - 1;
        }
        unsigned long long acc[RPT][4];
#pragma unroll
        for (int j = 0; j < RPT; j++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[j][k] = 0;

        // result handlers: accumulate as a constraint and / or store
        auto finish_b = [&](const uint4& ins, const uint32_t (&r)[RPT]) {
            if (ins.x & BC_F_ACC) {
                const qm31 coef = lde(ins.w, 0);
#pragma unroll
                for (int j = 0; j < RPT; j++)
#pragma unroll
                    for (int k = 0; k < 4; k++) acc[j][k] += (unsigned long long)coef.c[k] * r[j];
            }
            if (!(ins.x & BC_F_NOSTORE)) {
                const uint32_t d = (ins.x >> 8) + tid;
#pragma unroll
                for (int j = 0; j < RPT; j++) sm[d + j * T] = r[j];
            }
        };
        auto finish_e = [&](const uint4& ins, const qm31 (&r)[RPT]) {
            if (ins.x & BC_F_ACC) {
                const qm31 coef = lde(ins.w, 0);
#pragma unroll
                for (int j = 0; j < RPT; j++) {
                    const qm31 t = qm31_mul(coef, r[j]);
#pragma unroll
                    for (int k = 0; k < 4; k++) acc[j][k] += t.c[k];
                }
            }
            if (!(ins.x & BC_F_NOSTORE)) {
                const uint32_t d = (ins.x >> 8) + tid;
#pragma unroll
                for (int j = 0; j < RPT; j++)
#pragma unroll
                    for (int k = 0; k < 4; k++) sm[d + j * T + k * RP] = r[j].c[k];
            }
        };

        uint32_t pc = 0;
        uint4 ins = __ldg(code);
        for (;;) {
            const uint32_t op = ins.x & BC_OP_MASK;
            if (op == BC_END) break;
            if (op == BC_LOAD) {
                const uint32_t n = ins.x >> 8;
                uint32_t v[AIR_LOAD_BATCH][RPT], d[AIR_LOAD_BATCH];
#pragma unroll
                for (int q = 0; q < AIR_LOAD_BATCH / 2; q++) {
                    if (2 * q < (int)n) {
                        const uint4 e = __ldg(code + pc + 1 + q);
                        const uint32_t* c0 = reinterpret_cast<const uint32_t*>(ptrs[e.x & 0xfffffu]);
                        const int off0 = (int)e.x >> 20;
#pragma unroll
                        for (int j = 0; j < RPT; j++) v[2 * q][j] = __ldg(c0 + offset_row(row[j], off0, trace_log, eval_log));
                        d[2 * q] = e.y;
                        if (2 * q + 1 < (int)n) {
                            const uint32_t* c1 = reinterpret_cast<const uint32_t*>(ptrs[e.z & 0xfffffu]);
                            const int off1 = (int)e.z >> 20;
#pragma unroll
                            for (int j = 0; j < RPT; j++) v[2 * q + 1][j] = __ldg(c1 + offset_row(row[j], off1, trace_log, eval_log));
                            d[2 * q + 1] = e.w;
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < AIR_LOAD_BATCH; q++) {
                    if (q < (int)n) {
#pragma unroll
                        for (int j = 0; j < RPT; j++) sm[d[q] + tid + j * T] = v[q][j];
                    }
                }
                pc += 1 + (n + 1) / 2;
                ins = __ldg(code + pc);
                continue;
            }
            const uint4 nxt = __ldg(code + pc + 1);
            uint32_t rb[RPT];
            qm31 re[RPT];
            switch (op) {
                case BC_ACC_B: {
                    const qm31 coef = lde(ins.w, 0);
#pragma unroll
                    for (int j = 0; j < RPT; j++) {
                        const uint32_t a = ldb(ins.y, j);
#pragma unroll
                        for (int k = 0; k < 4; k++) acc[j][k] += (unsigned long long)coef.c[k] * a;
                    }
                    break;
                }
                case BC_ACC_E: {
                    const qm31 coef = lde(ins.w, 0);
#pragma unroll
                    for (int j = 0; j < RPT; j++) {
                        const qm31 t = qm31_mul(coef, lde(ins.y, j));
#pragma unroll
                        for (int k = 0; k < 4; k++) acc[j][k] += t.c[k];
                    }
                    break;
                }
                case BC_ACC_RED:
#pragma unroll
                    for (int j = 0; j < RPT; j++)
#pragma unroll
                        for (int k = 0; k < 4; k++) acc[j][k] = m31_reduce64(acc[j][k]);
                    break;
#define ZK_B_CASE(NAME, EXPR)                                    \
    case NAME:                                                   \
        _Pragma("unroll") for (int j = 0; j < RPT; j++) rb[j] = (EXPR); \
        finish_b(ins, rb);                                       \
        break;
#define ZK_E_CASE(NAME, EXPR)                                    \
    case NAME:                                                   \
        _Pragma("unroll") for (int j = 0; j < RPT; j++) re[j] = (EXPR); \
        finish_e(ins, re);                                       \
        break;
                ZK_B_CASE(BC_ADD_BB, m31_add(ldb(ins.y, j), ldb(ins.z, j)))
                ZK_B_CASE(BC_SUB_BB, m31_sub(ldb(ins.y, j), ldb(ins.z, j)))
                ZK_B_CASE(BC_MUL_BB, m31_mul(ldb(ins.y, j), ldb(ins.z, j)))
                ZK_B_CASE(BC_NEG_B, m31_neg(ldb(ins.y, j)))
                ZK_B_CASE(BC_INV_B, m31_inv(ldb(ins.y, j)))
                ZK_B_CASE(BC_MOV_B, ldb(ins.y, j))
                ZK_B_CASE(BC_FMA_B, m31_add(m31_mul(ldb(ins.y, j), ldb(ins.z, j)), ldb(ins.w, j)))
                ZK_B_CASE(BC_FMS_B, m31_sub(m31_mul(ldb(ins.y, j), ldb(ins.z, j)), ldb(ins.w, j)))
                ZK_B_CASE(BC_FNMS_B, m31_sub(ldb(ins.w, j), m31_mul(ldb(ins.y, j), ldb(ins.z, j))))
                ZK_E_CASE(BC_ADD_EE, qm31_add(lde(ins.y, j), lde(ins.z, j)))
                ZK_E_CASE(BC_SUB_EE, qm31_sub(lde(ins.y, j), lde(ins.z, j)))
                ZK_E_CASE(BC_MUL_EE, qm31_mul(lde(ins.y, j), lde(ins.z, j)))
                ZK_E_CASE(BC_NEG_E, qm31_neg(lde(ins.y, j)))
                ZK_E_CASE(BC_ADD_EB, qm31_add(lde(ins.y, j), qm31_from_m31(ldb(ins.z, j))))
                ZK_E_CASE(BC_SUB_EB, qm31_sub(lde(ins.y, j), qm31_from_m31(ldb(ins.z, j))))
                ZK_E_CASE(BC_SUB_BE, qm31_sub(qm31_from_m31(ldb(ins.y, j)), lde(ins.z, j)))
                ZK_E_CASE(BC_MUL_EB, qm31_mul_m31(lde(ins.y, j), ldb(ins.z, j)))
                ZK_E_CASE(BC_FMA_EB, qm31_add(lde(ins.w, j), qm31_mul_m31(lde(ins.y, j), ldb(ins.z, j))))
                ZK_E_CASE(BC_FNMS_EB, qm31_sub(lde(ins.w, j), qm31_mul_m31(lde(ins.y, j), ldb(ins.z, j))))
#undef ZK_B_CASE
#undef ZK_E_CASE
                default: break;
            }
            ins = nxt;
            pc++;
        }
#pragma unroll
        for (int j = 0; j < RPT; j++) {
            if (!active[j]) continue;
            const uint32_t di = __ldg(denom_inv + (row[j] >> trace_log));
#pragma unroll
            for (int k = 0; k < 4; k++) {
                uint32_t q = m31_mul(m31_reduce64(acc[j][k]), di);
                if (accumulate) q = m31_add(q, accum.c[k][row[j]]);
                accum.c[k][row[j]] = q;
            }
        }
    }
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_air_compile(zkb_ctx* ctx, const zkb_air_op* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints,
                    const uint32_t* tree_cols, int n_trees, size_t n_scalars, zkb_air_program** out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, ops != nullptr && constraints != nullptr && out != nullptr);
    ZKB_CHECK_ARG(ctx, n_trees >= 0 && n_trees <= 64 && (n_trees == 0 || tree_cols != nullptr));
    *out = nullptr;
    zkb_air_program* prog = new (std::nothrow) zkb_air_program();
    if (!prog) return set_error(ctx, ZKB_ENOMEM, "zkb_air_compile: out of host memory");
    std::string why;
    try {
        why = air_compile(*prog, ops, n_ops, constraints, n_constraints, tree_cols, n_trees, n_scalars);
    } catch (const std::bad_alloc&) {
        delete prog;
        return set_error(ctx, ZKB_ENOMEM, "zkb_air_compile: out of host memory");
    }
    if (!why.empty()) {
        delete prog;
        return set_error(ctx, ZKB_EINVAL, "zkb_air_compile: %s", why.c_str());
    }
    DeviceGuard g(ctx);
    prog->device = ctx->device;
    const size_t bytes = prog->code.size() * sizeof(AirInstr);
    cudaError_t e = cudaMalloc(&prog->d_code, bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(prog->d_code, prog->code.data(), bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(air_eval_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(air_eval_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(air_eval_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
        if (prog->d_code) cudaFree(prog->d_code);
        delete prog;
        return set_error(ctx, e == cudaErrorMemoryAllocation ? ZKB_ENOMEM : ZKB_ECUDA, "zkb_air_compile: %s", cudaGetErrorString(e));
    }
    *out = prog;
    return ZKB_OK;
}

int zkb_air_free(zkb_air_program* prog) {
    if (!prog) return ZKB_OK;
    if (prog->d_code) {
        int prev = -1;
        cudaGetDevice(&prev);
        if (prev != prog->device) cudaSetDevice(prog->device);
        if (prog->jit_library) cudaLibraryUnload((cudaLibrary_t)prog->jit_library);
        cudaFree(prog->d_code);
        if (prev >= 0 && prev != prog->device) cudaSetDevice(prev);
    }
    delete prog;
    return ZKB_OK;
}

int zkb_air_specialize(zkb_ctx* ctx, zkb_air_program* prog) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, prog != nullptr && prog->device == ctx->device);
    if (prog->jit_kernel) { prog->use_jit = true; return ZKB_OK; }
    const size_t table_bytes = 4 * ((size_t)prog->ptr_base + 2 * (size_t)prog->n_cols);
    if (table_bytes > 200 * 1024) return set_error(ctx, ZKB_EINVAL, "zkb_air_specialize: the program's table of %zu bytes does not fit shared memory", table_bytes);
    std::vector<char> cubin;
    std::string info, why;
    try {
        why = air_nvrtc_compile(air_codegen(*prog), cubin, &info);
    } catch (const std::bad_alloc&) {
        return set_error(ctx, ZKB_ENOMEM, "zkb_air_specialize: out of host memory");
    }
    if (!why.empty()) return set_error(ctx, ZKB_ECUDA, "zkb_air_specialize: %s", why.c_str());
    DeviceGuard g(ctx);
    cudaLibrary_t lib = nullptr;
    cudaKernel_t kernel = nullptr;
    cudaError_t e = cudaLibraryLoadData(&lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&kernel, lib, "air_jit");
    if (e == cudaSuccess && table_bytes > 48 * 1024)
        e = cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)table_bytes);
    if (e != cudaSuccess) {
        if (lib) cudaLibraryUnload(lib);
        return set_error(ctx, ZKB_ECUDA, "zkb_air_specialize: loading the compiled kernel: %s", cudaGetErrorString(e));
    }
    prog->jit_library = lib;
    prog->jit_kernel = kernel;
    prog->use_jit = true;
    prog->stats.specialized = 1;
    const size_t at = info.find("Used ");
    if (at != std::string::npos) prog->stats.specialized_regs = (uint32_t)atoi(info.c_str() + at + 5);
    return ZKB_OK;
}

int zkb_air_analyze(const zkb_air_op* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints, const uint32_t* tree_cols,
                    int n_trees, size_t n_scalars, int check_specialized, zkb_air_stats* out, char* err, size_t err_cap) {
    auto say = [&](const std::string& m) { if (err && err_cap) snprintf(err, err_cap, "%s", m.c_str()); };
    say("");
    if (!ops || !constraints || !out || n_trees < 0 || n_trees > 64 || (n_trees && !tree_cols)) { say("invalid argument"); return ZKB_EINVAL; }
    try {
        zkb_air_program prog;
        std::string why = air_compile(prog, ops, n_ops, constraints, n_constraints, tree_cols, n_trees, n_scalars);
        if (!why.empty()) { say(why); return ZKB_EINVAL; }
        if (check_specialized) {
            std::vector<char> cubin;
            std::string info;
            why = air_nvrtc_compile(air_codegen(prog), cubin, &info);
            if (!why.empty()) { say(why); return ZKB_ECUDA; }
            prog.stats.specialized = 1;
            const size_t at = info.find("Used ");
            if (at != std::string::npos) prog.stats.specialized_regs = (uint32_t)atoi(info.c_str() + at + 5);
        }
        *out = prog.stats;
        return ZKB_OK;
    } catch (const std::bad_alloc&) {
        say("out of host memory");
        return ZKB_ENOMEM;
    }
}

int zkb_air_select(zkb_air_program* prog, int specialized) {
    if (!prog || (specialized && !prog->jit_kernel)) return ZKB_EINVAL;
    prog->use_jit = specialized != 0;
    return ZKB_OK;
}

int zkb_air_get_stats(const zkb_air_program* prog, zkb_air_stats* out) {
    if (!prog || !out) return ZKB_EINVAL;
    *out = prog->stats;
    return ZKB_OK;
}

int zkb_constraint_quotients(zkb_ctx* ctx, const zkb_air_program* prog, const uint32_t* const* cols, const uint32_t* scalars,
                             const uint32_t* cumsum_shift, const uint32_t* random_coeff_powers, const uint32_t* denom_inv,
                             int trace_log, int eval_log, uint32_t* const accum[4], int accumulate) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, prog != nullptr && prog->d_code != nullptr && prog->device == ctx->device);
    ZKB_CHECK_ARG(ctx, random_coeff_powers != nullptr && denom_inv != nullptr && accum != nullptr);
    ZKB_CHECK_ARG(ctx, prog->n_cols == 0 || cols != nullptr);
    ZKB_CHECK_ARG(ctx, prog->n_scalars == 0 || scalars != nullptr);
    ZKB_CHECK_ARG(ctx, trace_log >= 1 && trace_log < eval_log && eval_log <= 30);
    ZKB_CHECK_ARG(ctx, eval_log - trace_log <= 16);
    for (int k = 0; k < 4; k++) ZKB_CHECK_ARG(ctx, accum[k] != nullptr);
    DeviceGuard g(ctx);
    // One staged blob: [uniform values | coefficients | column pointers | denominator inverses], in 8-byte units.
    const uint32_t n_denom = 1u << (eval_log - trace_log);
    const size_t table_words = (size_t)prog->ptr_base + 2 * (size_t)prog->n_cols;
    const size_t blob_words = table_words + n_denom + (n_denom & 1);
    std::vector<uint32_t> blob(blob_words, 0);
    air_fill_uniform(*prog, scalars, cumsum_shift, random_coeff_powers, blob.data());
    for (uint32_t c = 0; c < prog->n_cols; c++) {
        const unsigned long long p = (unsigned long long)(uintptr_t)cols[c];
        blob[prog->ptr_base + 2 * c] = (uint32_t)p;
        blob[prog->ptr_base + 2 * c + 1] = (uint32_t)(p >> 32);
    }
    for (uint32_t j = 0; j < n_denom; j++) blob[table_words + j] = denom_inv[j];
    void** d_blob = nullptr;
    int rc = stage_ptrs(ctx, reinterpret_cast<const void* const*>(blob.data()), (int)(blob_words / 2), &d_blob);
    if (rc != ZKB_OK) return rc;
    const uint32_t* d_table = reinterpret_cast<const uint32_t*>(d_blob);
    AccumPtrs ap{{accum[0], accum[1], accum[2], accum[3]}};
    const uint32_t T = prog->threads;
    const uint64_t n_rows = 1ull << eval_log;
    const uint32_t RP = T * prog->rows_per_thread;
    const uint32_t n_tiles = (uint32_t)((n_rows + RP - 1) / RP);
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx->device);
    const uint32_t grid = std::min<uint32_t>(n_tiles, (uint32_t)sms * prog->ctas_per_sm);
    if (prog->use_jit) {  // the specialised kernel: one row per thread, the same table and arguments
        uint32_t tw = (uint32_t)table_words, pb = prog->ptr_base, tiles = (uint32_t)((n_rows + 255) / 256);
        const uint32_t* d_den = d_table + table_words;
        uint32_t* q[4] = {accum[0], accum[1], accum[2], accum[3]};
        void* args[] = {(void*)&d_table, &tw, &pb, (void*)&d_den, &trace_log, &eval_log, &q[0], &q[1], &q[2], &q[3], &accumulate, &tiles};
        const uint32_t jgrid = std::min<uint32_t>(tiles, (uint32_t)sms * 8);
        ProfScope prof(ctx, "air_jit");
        ZKB_CUDA(ctx, cudaLaunchKernel((const void*)prog->jit_kernel, dim3(jgrid), dim3(256), args, table_words * 4, ctx->stream));
        return ZKB_OK;
    }
    ProfScope prof(ctx, "air_eval_kernel");
    auto kernel = prog->rows_per_thread == 4 ? air_eval_kernel<4> : prog->rows_per_thread == 2 ? air_eval_kernel<2> : air_eval_kernel<1>;
    kernel<<<grid, T, prog->smem_bytes, ctx->stream>>>(reinterpret_cast<const uint4*>(prog->d_code), d_table, (uint32_t)table_words,
                                                        prog->ptr_base, d_table + table_words, trace_log, eval_log, ap, accumulate, n_tiles);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_constraint_denom_inv(int trace_log, int eval_log, uint32_t* out) {
    if (!out || trace_log < 1 || trace_log >= eval_log || eval_log > 30 || eval_log - trace_log > 16) return ZKB_EINVAL;
    // Generator of the order-2^31 circle group (core/circle.rs:202-205); a point of index i is i * G.
    auto point = [](uint32_t idx) {
        cpoint r{1u, 0u}, g{2u, 1268011823u};
        for (int b = 0; b < 31; b++) {
            if ((idx >> b) & 1u) r = cpoint_add(r, g);
            g = cpoint_add(g, g);
        }
        return r;
    };
    auto subgroup_gen = [](int log_size) { return 1u << (31 - log_size); };
    const uint32_t mask = 0x7fffffffu;
    // trace coset: Coset::odds(trace_log) = (initial G_{trace_log+1}, step G_{trace_log}); the shift of coset_vanishing
    // is -initial + step/2 (core/constraints.rs:27), which is zero for a canonic coset's index arithmetic below.
    const uint32_t t_initial = subgroup_gen(trace_log + 1), t_step = subgroup_gen(trace_log);
    // evaluation domain: CircleDomain(half_odds(eval_log - 1)) = (initial G_{eval_log+1}, step G_{eval_log-1});
    // at(i) for i below the half size is initial + i * step.
    const uint32_t e_initial = subgroup_gen(eval_log + 1), e_step = subgroup_gen(eval_log - 1);
    const uint32_t n = 1u << (eval_log - trace_log), half = 1u << (eval_log - 1);
    const int bits = eval_log - trace_log;
    for (uint32_t i = 0; i < n; i++) {
        // CircleDomain::at: the second half of the domain is the conjugate coset
        uint32_t idx = i < half ? (e_initial + i * e_step) & mask : (0u - (e_initial + (i - half) * e_step)) & mask;
        uint32_t shifted = (idx - t_initial + (t_step >> 1)) & mask;
        uint32_t x = point(shifted).x;
        for (int k = 1; k < trace_log; k++) x = m31_double_x(x);
        uint32_t j = 0;
        for (int k = 0; k < bits; k++) j |= ((i >> k) & 1u) << (bits - 1 - k);
        out[j] = m31_inv(x);
    }
    return ZKB_OK;
}

}  // extern "C"
