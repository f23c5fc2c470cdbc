// Specialisation of a compiled AIR program into straight-line CUDA, compiled for sm_100a at run time with NVRTC.
//
// The interpreter of csrc/constraints.cu serves every AIR with one kernel but pays for it: each instruction of the
// program is fetched and decoded per tile, and every value of a row passes through shared memory. This file emits,
// from the same annotated program (kinds, row-independent values, merged loads, dead code removed), one kernel in
// which every per-row value is a local variable, so that the values live in registers and the compiler schedules the
// column loads and folds the arithmetic. It is what the reference's generator does ahead of time, per AIR shape, when
// the prover is built (prover/src/cudagen.rs:1985-2290 emits a .cu per family); here it happens when the caller asks
// for it (zkb_air_specialize), and the interpreter remains the path that needs nothing but the library itself.
//
// NVRTC is looked up with dlopen when first needed; nothing links against it. The kernel takes the interpreter's
// argument list (minus the bytecode) and reads the same staged table: row-independent values, constraint
// coefficients, column pointers.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

#include "../air_program.hpp"

namespace zk {
namespace {

const char* kPrelude = R"SRC(
typedef unsigned int u32;
typedef unsigned long long u64;
#define P 0x7fffffffu
#define P_SQ 0x3fffffff00000001ull
struct qm31 { u32 c[4]; };
__device__ __forceinline__ u32 umin32(u32 a, u32 b) { return a < b ? a : b; }
__device__ __forceinline__ u32 m31_add(u32 a, u32 b) { u32 s = a + b; return umin32(s, s - P); }
__device__ __forceinline__ u32 m31_sub(u32 a, u32 b) { u32 d = a - b; return umin32(d, d + P); }
__device__ __forceinline__ u32 m31_neg(u32 a) { return a ? P - a : 0u; }
__device__ __forceinline__ u32 m31_reduce64(u64 v) {
    u32 lo = (u32)v, hi = (u32)(v >> 32);
    u32 s = (lo & P) + (lo >> 31) + ((hi << 1) & P) + (hi >> 30);
    s = (s & P) + (s >> 31);
    return umin32(s, s - P);
}
__device__ __forceinline__ u32 m31_mul(u32 a, u32 b) {
    u64 p = (u64)a * b;
    u32 s = ((u32)p & P) + (u32)(p >> 31);
    return umin32(s, s - P);
}
__device__ __forceinline__ u32 m31_sqn(u32 v, int n) { for (int i = 0; i < n; i++) v = m31_mul(v, v); return v; }
__device__ __forceinline__ u32 m31_inv(u32 v) {
    u32 t0 = m31_mul(m31_sqn(v, 2), v);
    u32 t1 = m31_mul(m31_sqn(t0, 1), t0);
    u32 t2 = m31_mul(m31_sqn(t1, 3), t0);
    u32 t3 = m31_mul(m31_sqn(t2, 1), t0);
    u32 t4 = m31_mul(m31_sqn(t3, 8), t3);
    u32 t5 = m31_mul(m31_sqn(t4, 8), t3);
    return m31_mul(m31_sqn(t5, 7), t2);
}
__device__ __forceinline__ qm31 qm31_add(qm31 x, qm31 y) { return {{m31_add(x.c[0], y.c[0]), m31_add(x.c[1], y.c[1]), m31_add(x.c[2], y.c[2]), m31_add(x.c[3], y.c[3])}}; }
__device__ __forceinline__ qm31 qm31_sub(qm31 x, qm31 y) { return {{m31_sub(x.c[0], y.c[0]), m31_sub(x.c[1], y.c[1]), m31_sub(x.c[2], y.c[2]), m31_sub(x.c[3], y.c[3])}}; }
__device__ __forceinline__ qm31 qm31_neg(qm31 x) { return {{m31_neg(x.c[0]), m31_neg(x.c[1]), m31_neg(x.c[2]), m31_neg(x.c[3])}}; }
__device__ __forceinline__ qm31 qm31_add_m31(qm31 x, u32 y) { x.c[0] = m31_add(x.c[0], y); return x; }
__device__ __forceinline__ qm31 qm31_sub_m31(qm31 x, u32 y) { x.c[0] = m31_sub(x.c[0], y); return x; }
__device__ __forceinline__ qm31 m31_sub_qm31(u32 x, qm31 y) { qm31 r = qm31_neg(y); r.c[0] = m31_add(r.c[0], x); return r; }
__device__ __forceinline__ qm31 qm31_mul_m31(qm31 x, u32 y) { return {{m31_mul(x.c[0], y), m31_mul(x.c[1], y), m31_mul(x.c[2], y), m31_mul(x.c[3], y)}}; }
__device__ __forceinline__ qm31 qm31_mul(qm31 x, qm31 y) {
    const u32 x0 = x.c[0], x1 = x.c[1], x2 = x.c[2], x3 = x.c[3];
    const u32 y0 = y.c[0], y1 = y.c[1], y2 = y.c[2], y3 = y.c[3];
    u32 br = m31_reduce64((u64)x2 * y2 + (P_SQ - (u64)x3 * y3));
    u32 bi = m31_reduce64((u64)x2 * y3 + (u64)x3 * y2);
    u64 r0 = (u64)x0 * y0 + (P_SQ - (u64)x1 * y1) + 2ull * br + (u64)(P - bi);
    u64 r1 = (u64)x0 * y1 + (u64)x1 * y0 + (u64)br + 2ull * bi;
    u64 r2 = (u64)x0 * y2 + (u64)x2 * y0 + (2 * P_SQ - (u64)x1 * y3 - (u64)x3 * y1);
    u64 r3 = (u64)x0 * y3 + (u64)x1 * y2 + (u64)x2 * y1 + (u64)x3 * y0;
    return {{m31_reduce64(r0), m31_reduce64(r1), m31_reduce64(r2), m31_reduce64(r3)}};
}
// core/utils.rs:97-113 for a compile-time offset
template <int OFF>
__device__ __forceinline__ u32 offset_row(u32 row, int trace_log, int eval_log) {
    if (OFF == 0) return row;
    const u32 nat = __brev(row) >> (32 - eval_log);
    const u32 half = 1u << (eval_log - 1);
    const u32 step = (u32)OFF << (eval_log - trace_log - 1);
    const u32 lo = (nat & half) ? nat - step : nat + step;
    const u32 moved = (lo & (half - 1u)) | (nat & half);
    return __brev(moved) >> (32 - eval_log);
}
// consecutive tile numbers get row ranges that differ in the top three bits of the row index (see csrc/constraints.cu)
__device__ __forceinline__ u32 spread_tile(u32 t, u32 n_tiles) {
    if (n_tiles < 16u || (n_tiles & (n_tiles - 1u))) return t;
    const u32 bits = 31u - (u32)__clz(n_tiles);
    return ((t & 7u) << (bits - 3u)) | (t >> 3);
}
extern __shared__ __align__(16) u32 sm[];
#define U4(w) (qm31{{sm[(w)], sm[(w) + 1], sm[(w) + 2], sm[(w) + 3]}})
#define COL(c) (reinterpret_cast<const u32*>(ptrs[(c)]))
#define ACC_B(w, v) do { const u32 t_ = (v); a0 += (u64)sm[(w)] * t_; a1 += (u64)sm[(w) + 1] * t_; a2 += (u64)sm[(w) + 2] * t_; a3 += (u64)sm[(w) + 3] * t_; } while (0)
#define ACC_E(w, v) do { const qm31 t_ = qm31_mul(U4(w), (v)); a0 += t_.c[0]; a1 += t_.c[1]; a2 += t_.c[2]; a3 += t_.c[3]; } while (0)
#define RED() do { a0 = m31_reduce64(a0); a1 = m31_reduce64(a1); a2 = m31_reduce64(a2); a3 = m31_reduce64(a3); } while (0)
)SRC";

}  // namespace

// The kernel source for one program. Per-row instruction i is the local v<i>; row-independent operands are words of the
// staged table in shared memory.
std::string air_codegen(const zkb_air_program& G) {
    const uint32_t N = (uint32_t)G.ops.size();
    std::string s = kPrelude;
    s += "extern \"C\" __global__ void __launch_bounds__(256) air_jit(const u32* __restrict__ table, u32 table_words, u32 ptr_base,\n"
         "    const u32* __restrict__ denom_inv, int trace_log, int eval_log, u32* q0, u32* q1, u32* q2, u32* q3, int accumulate, u32 n_tiles) {\n"
         "  for (u32 i = threadIdx.x; i < table_words; i += blockDim.x) sm[i] = table[i];\n"
         "  __syncthreads();\n"
         "  const u64* ptrs = reinterpret_cast<const u64*>(sm + ptr_base);\n"
         "  const u32 n_rows = 1u << eval_log;\n"
         "  for (u32 t = blockIdx.x; t < n_tiles; t += gridDim.x) {\n"
         "    const u32 row = spread_tile(t, n_tiles) * blockDim.x + threadIdx.x;\n"
         "    if (row >= n_rows) continue;\n"
         "    u64 a0 = 0, a1 = 0, a2 = 0, a3 = 0;\n";
    auto per_row = [&](uint32_t i) { return G.live[i] && !G.uniform[i] && G.alias[i] == i; };
    auto val = [&](uint32_t v) -> std::string {
        if (!G.uniform[v]) return "v" + std::to_string(v);
        const std::string w = std::to_string(G.uni_word[v]);
        return G.ext[v] ? "U4(" + w + ")" : "sm[" + w + "]";
    };
    std::vector<std::vector<uint32_t>> cons_of(N);
    for (uint32_t k = 0; k < G.constraints.size(); k++) cons_of[G.constraints[k]].push_back(k);
    std::vector<uint8_t> emitted(N, 0);
    int units = 0;
    auto accumulate = [&](uint32_t v, uint32_t k) {
        const std::string w = std::to_string(G.coef_base + 4 * k);
        if (G.ext[v]) {
            s += "    ACC_E(" + w + ", " + val(v) + ");\n";
        } else {
            if (units == 3) { s += "    RED();\n"; units = 0; }
            units++;
            s += "    ACC_B(" + w + ", " + val(v) + ");\n";
        }
    };
    auto arity = [](uint32_t op) {
        switch (op) {
            case ZKB_AIR_LOAD: case ZKB_AIR_CONST_M31: case ZKB_AIR_SCALAR: case ZKB_AIR_CUMSUM_SHIFT: return 0;
            case ZKB_AIR_NEG_B: case ZKB_AIR_NEG_E: case ZKB_AIR_INV_B: return 1;
            case ZKB_AIR_PACK: return 4;
            default: return 2;
        }
    };
    // Column loads in the order of their first use. When a value is needed that has not been loaded yet, it and the
    // next JIT_LOAD_BATCH - 1 of that order are issued together, so that a thread has that many reads in flight
    // (the compiler keeps the order of the loads it is given; one load per use would leave one in flight).
    constexpr size_t JIT_LOAD_BATCH = 16;
    std::vector<uint32_t> load_order;
    {
        std::vector<uint8_t> seen(N, 0);
        auto note = [&](uint32_t v) {
            if (G.ops[v].op == ZKB_AIR_LOAD && !seen[v]) { seen[v] = 1; load_order.push_back(v); }
        };
        for (uint32_t i = 0; i < N; i++) {
            if (!per_row(i) || G.ops[i].op == ZKB_AIR_LOAD) continue;
            const zkb_air_op& o = G.ops[i];
            const uint32_t src[4] = {o.a, o.b, o.c, o.d};
            for (int k = 0; k < arity(o.op); k++) note(src[k]);
        }
        for (uint32_t v : G.constraints) note(v);
    }
    size_t next_load = 0;
    auto emit_load = [&](uint32_t v) {
        if (emitted[v]) return;
        while (!emitted[v]) {
            for (size_t q = 0; q < JIT_LOAD_BATCH && next_load < load_order.size(); q++, next_load++) {
                const uint32_t l = load_order[next_load];
                emitted[l] = 1;
                const zkb_air_op& o = G.ops[l];
                s += "    const u32 v" + std::to_string(l) + " = __ldg(COL(" + std::to_string(G.tree_base[o.a] + o.b) + ") + offset_row<" +
                     std::to_string((int32_t)o.c) + ">(row, trace_log, eval_log));\n";
            }
        }
    };
    for (uint32_t i = 0; i < N; i++) {
        if (!per_row(i) || G.ops[i].op == ZKB_AIR_LOAD) continue;
        const zkb_air_op& o = G.ops[i];
        const uint32_t src[4] = {o.a, o.b, o.c, o.d};
        const int ar = arity(o.op);
        for (int k = 0; k < ar; k++)
            if (G.ops[src[k]].op == ZKB_AIR_LOAD && !G.uniform[src[k]]) emit_load(src[k]);
        const bool ea = G.ext[o.a], eb = ar >= 2 ? (bool)G.ext[o.b] : false;
        const std::string a = val(o.a), b = ar >= 2 ? val(o.b) : "";
        std::string e;
        switch (o.op) {
            case ZKB_AIR_ADD_B: case ZKB_AIR_ADD_E:
                e = ea && eb ? "qm31_add(" + a + ", " + b + ")" : !ea && !eb ? "m31_add(" + a + ", " + b + ")"
                    : ea ? "qm31_add_m31(" + a + ", " + b + ")" : "qm31_add_m31(" + b + ", " + a + ")";
                break;
            case ZKB_AIR_SUB_B: case ZKB_AIR_SUB_E:
                e = ea && eb ? "qm31_sub(" + a + ", " + b + ")" : !ea && !eb ? "m31_sub(" + a + ", " + b + ")"
                    : ea ? "qm31_sub_m31(" + a + ", " + b + ")" : "m31_sub_qm31(" + a + ", " + b + ")";
                break;
            case ZKB_AIR_MUL_B: case ZKB_AIR_MUL_E:
                e = ea && eb ? "qm31_mul(" + a + ", " + b + ")" : !ea && !eb ? "m31_mul(" + a + ", " + b + ")"
                    : ea ? "qm31_mul_m31(" + a + ", " + b + ")" : "qm31_mul_m31(" + b + ", " + a + ")";
                break;
            case ZKB_AIR_NEG_B: case ZKB_AIR_NEG_E: e = (ea ? "qm31_neg(" : "m31_neg(") + a + ")"; break;
            case ZKB_AIR_INV_B: e = "m31_inv(" + a + ")"; break;
            case ZKB_AIR_PACK: e = "qm31{{" + val(o.a) + ", " + val(o.b) + ", " + val(o.c) + ", " + val(o.d) + "}}"; break;
            default: break;
        }
        s += std::string("    const ") + (G.ext[i] ? "qm31" : "u32") + " v" + std::to_string(i) + " = " + e + ";\n";
        for (uint32_t k : cons_of[i]) accumulate(i, k);
    }
    for (uint32_t k = 0; k < G.constraints.size(); k++) {
        const uint32_t v = G.constraints[k];
        if (G.uniform[v]) accumulate(v, k);
        else if (G.ops[v].op == ZKB_AIR_LOAD) { emit_load(v); accumulate(v, k); }
    }
    s += "    const u32 di = __ldg(denom_inv + (row >> trace_log));\n"
         "    u32 r0 = m31_mul(m31_reduce64(a0), di), r1 = m31_mul(m31_reduce64(a1), di), r2 = m31_mul(m31_reduce64(a2), di), r3 = m31_mul(m31_reduce64(a3), di);\n"
         "    if (accumulate) { r0 = m31_add(r0, q0[row]); r1 = m31_add(r1, q1[row]); r2 = m31_add(r2, q2[row]); r3 = m31_add(r3, q3[row]); }\n"
         "    q0[row] = r0; q1[row] = r1; q2[row] = r2; q3[row] = r3;\n"
         "  }\n"
         "}\n";
    return s;
}

// ---- NVRTC, looked up at run time
namespace {
struct Nvrtc {
    void* handle = nullptr;
    int (*create)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    int (*compile)(void*, int, const char* const*) = nullptr;
    int (*cubin_size)(void*, size_t*) = nullptr;
    int (*cubin)(void*, char*) = nullptr;
    int (*log_size)(void*, size_t*) = nullptr;
    int (*log)(void*, char*) = nullptr;
    int (*destroy)(void**) = nullptr;
    bool ok = false;
};
Nvrtc& nvrtc() {
    static Nvrtc n;
    static std::once_flag once;
    std::call_once(once, [] {
        if (const char* forced = getenv("ZKB_NVRTC_LIB")) {
            n.handle = dlopen(forced, RTLD_NOW | RTLD_LOCAL);
        } else {
            for (const char* name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"}) {
                n.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
                if (n.handle) break;
            }
        }
        if (!n.handle) return;
        auto sym = [&](const char* s) { return dlsym(n.handle, s); };
        n.create = reinterpret_cast<decltype(n.create)>(sym("nvrtcCreateProgram"));
        n.compile = reinterpret_cast<decltype(n.compile)>(sym("nvrtcCompileProgram"));
        n.cubin_size = reinterpret_cast<decltype(n.cubin_size)>(sym("nvrtcGetCUBINSize"));
        n.cubin = reinterpret_cast<decltype(n.cubin)>(sym("nvrtcGetCUBIN"));
        n.log_size = reinterpret_cast<decltype(n.log_size)>(sym("nvrtcGetProgramLogSize"));
        n.log = reinterpret_cast<decltype(n.log)>(sym("nvrtcGetProgramLog"));
        n.destroy = reinterpret_cast<decltype(n.destroy)>(sym("nvrtcDestroyProgram"));
        n.ok = n.create && n.compile && n.cubin_size && n.cubin && n.log_size && n.log && n.destroy;
    });
    return n;
}
}  // namespace

// Compiles `source` for sm_100a. Returns an empty string and the cubin, or the reason (with the compiler's log).
std::string air_nvrtc_compile(const std::string& source, std::vector<char>& cubin, std::string* ptxas_info) {
    Nvrtc& n = nvrtc();
    if (!n.ok) return "NVRTC (libnvrtc.so.12) could not be loaded";
    void* prog = nullptr;
    if (n.create(&prog, source.c_str(), "air_jit.cu", 0, nullptr, nullptr) != 0) return "nvrtcCreateProgram failed";
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo", "--ptxas-options=-v"};
    const int rc = n.compile(prog, 4, opts);
    size_t ls = 0;
    std::string log;
    if (n.log_size(prog, &ls) == 0 && ls > 1) {
        log.resize(ls);
        n.log(prog, &log[0]);
    }
    if (ptxas_info) *ptxas_info = log;
    if (rc != 0) {
        n.destroy(&prog);
        return "NVRTC compilation failed: " + log.substr(0, 400);
    }
    size_t cs = 0;
    if (n.cubin_size(prog, &cs) != 0 || cs == 0) {
        n.destroy(&prog);
        return "NVRTC produced no cubin";
    }
    cubin.resize(cs);
    n.cubin(prog, cubin.data());
    n.destroy(&prog);
    return "";
}

}  // namespace zk
