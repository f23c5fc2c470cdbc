// The Freivalds attention-witness component on the device: the committed / preprocessed columns
// (scatter of int8 activations and weights into M31 columns in committed order, with the 8-bit
// range multiplicities), and the Horner accumulators v, u_m, acc_m with their claims.
//
// Rows are laid out by a grid over input channels (prover/src/layout.rs:141-183): coset-order
// row j >= lead belongs to group (= input channel) groups-1-(j-lead)/chunks and chunk
// chunks-1-(j-lead)%chunks; a column stores row j at committed index coset_perm(j)
// (prover/src/common.rs:76-80; the permutation is an involution). Semantics follow
// prover/src/gadgets/freivalds/trace.rs:43-162 (columns) and claims.rs:37-109 (accumulators):
//   v[j]   = [chunk+1 < chunks] v[j-1] s^pq + sum_p s^p (act[p][j] - 128)
//   u_m[j] = [chunk+1 < chunks] u_m[j-1] rv^pk + sum_p rv^p w_m[p][j]
//   acc_m[j] = acc_m[j-1] + [chunk == 0] u_m[j] v[j]
// The Horner restarts at every group, so each group is scanned independently and acc_m is a prefix
// sum over the groups' totals. Kernels: per-row inner products (coalesced column reads, results in
// coset order), per-group scan, prefix over groups, split into coordinate columns.
#include <vector>

#include "common.cuh"

namespace zk {

struct FGrid { uint32_t log_rows, groups, chunks, lead; };

__device__ __forceinline__ uint32_t coset_perm(uint32_t i, uint32_t log_n) {
    uint32_t n = 1u << log_n;
    uint32_t c = (i & 1u) ? (2u * n - i - 1u) >> 1 : i >> 1;
    return __brev(c) >> (32 - log_n);
}
__device__ __forceinline__ uint32_t m31_of_i32(int v) { return v < 0 ? (uint32_t)(v + (int)P) : (uint32_t)v; }

// ---- F1: columns ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) freivalds_scatter_kernel(const int8_t* __restrict__ qx, const int8_t* const* __restrict__ qw,
                                                                const uint32_t* __restrict__ n_out, FGrid g, uint32_t pq, uint32_t pk,
                                                                uint32_t n_in, uint32_t tokens, uint32_t n_mats,
                                                                uint32_t* const* __restrict__ base_cols,
                                                                uint32_t* const* __restrict__ pre_cols, uint32_t* __restrict__ m_r8,
                                                                uint32_t table_len, unsigned long long* __restrict__ off_table) {
    extern __shared__ uint32_t hist[];  // table_len counters
    for (uint32_t t = threadIdx.x; t < table_len; t += blockDim.x) hist[t] = 0;
    __syncthreads();
    const uint32_t rows = 1u << g.log_rows;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) {
        const uint32_t j = coset_perm(i, g.log_rows);
        const bool some = j >= g.lead;
        uint32_t k = 0, chunk = 0;
        if (some) {
            uint32_t idx = j - g.lead;
            k = g.groups - 1 - idx / g.chunks;
            chunk = g.chunks - 1 - idx % g.chunks;
        }
        uint32_t off = 0;
        for (uint32_t p = 0; p < pq; p++) {
            int v = 128;
            uint32_t t = chunk * pq + p;
            if (some && t < tokens) v = (int)qx[(size_t)t * n_in + k] + 128;
            base_cols[p][i] = (uint32_t)v;
            if ((uint32_t)v < table_len) atomicAdd(&hist[v], 1u); else off++;
        }
        if (off) atomicAdd(off_table, (unsigned long long)off);
        for (uint32_t m = 0; m < n_mats; m++) {
            const uint32_t no = n_out[m];
            const int8_t* __restrict__ w = qw[m] + (size_t)k * no;
            for (uint32_t p = 0; p < pk; p++) {
                uint32_t c = chunk * pk + p;
                pre_cols[m * pk + p][i] = (some && c < no) ? m31_of_i32((int)w[c]) : 0u;
            }
        }
        uint32_t* const* sel = pre_cols + n_mats * pk;
        sel[0][i] = (some && chunk + 1 < g.chunks) ? 1u : 0u;
        sel[1][i] = (some && chunk == 0) ? 1u : 0u;
        sel[2][i] = j > 0 ? 1u : 0u;
        sel[3][i] = j + 1 == rows ? 1u : 0u;
    }
    __syncthreads();
    for (uint32_t t = threadIdx.x; t < table_len; t += blockDim.x)
        if (hist[t]) atomicAdd(&m_r8[t], hist[t]);
}

// ---- F2: inner products per row -----------------------------------------------------------------
__device__ __forceinline__ uint64_t fold64f(uint64_t v) { return (v & P) + (v >> 31); }

// lanes[l][j] (QM31, coset order): l = 0 is v_in, l = 1 + m is u_in of matrix m.
__global__ void __launch_bounds__(256) freivalds_inner_kernel(const uint32_t* const* __restrict__ base_cols,
                                                              const uint32_t* const* __restrict__ pre_cols,
                                                              const uint4* __restrict__ s_pow, const uint4* __restrict__ rv_pow, FGrid g,
                                                              uint32_t pq, uint32_t pk, uint32_t n_mats, uint4* __restrict__ lanes) {
    const uint32_t rows = 1u << g.log_rows;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows) return;
    const uint32_t j = coset_perm(i, g.log_rows);
    const bool some = j >= g.lead;
    {
        uint64_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (uint32_t p = 0; p < pq; p++) {
            uint32_t x = m31_sub(base_cols[p][i], 128u);
            uint4 c = s_pow[p];
            a0 += (uint64_t)c.x * x; a1 += (uint64_t)c.y * x; a2 += (uint64_t)c.z * x; a3 += (uint64_t)c.w * x;
            if ((p & 3) == 3) { a0 = fold64f(a0); a1 = fold64f(a1); a2 = fold64f(a2); a3 = fold64f(a3); }
        }
        lanes[j] = some ? make_uint4(m31_reduce64(a0), m31_reduce64(a1), m31_reduce64(a2), m31_reduce64(a3)) : make_uint4(0, 0, 0, 0);
    }
    for (uint32_t m = 0; m < n_mats; m++) {
        uint64_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (uint32_t p = 0; p < pk; p++) {
            uint32_t x = pre_cols[m * pk + p][i];
            uint4 c = rv_pow[p];
            a0 += (uint64_t)c.x * x; a1 += (uint64_t)c.y * x; a2 += (uint64_t)c.z * x; a3 += (uint64_t)c.w * x;
            if ((p & 3) == 3) { a0 = fold64f(a0); a1 = fold64f(a1); a2 = fold64f(a2); a3 = fold64f(a3); }
        }
        lanes[(size_t)(1 + m) * rows + j] =
            some ? make_uint4(m31_reduce64(a0), m31_reduce64(a1), m31_reduce64(a2), m31_reduce64(a3)) : make_uint4(0, 0, 0, 0);
    }
}

// ---- F3: per-group Horner, prefix over groups, split ------------------------------------------------
__device__ __forceinline__ qm31 q_of(uint4 v) { return {{v.x, v.y, v.z, v.w}}; }
__device__ __forceinline__ uint4 u_of(qm31 v) { return make_uint4(v.c[0], v.c[1], v.c[2], v.c[3]); }

// One thread per (group slot, lane): x_r = x_{r-1} step + in_r over the group's `chunks` rows.
__global__ void __launch_bounds__(128) freivalds_group_scan_kernel(uint4* __restrict__ lanes, FGrid g, uint32_t n_lanes, qm31 s_step,
                                                                   qm31 rv_step) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= g.groups * n_lanes) return;
    const uint32_t lane = t / g.groups, slot = t % g.groups;
    const qm31 step = lane == 0 ? s_step : rv_step;
    uint4* __restrict__ p = lanes + ((size_t)lane << g.log_rows) + g.lead + (size_t)slot * g.chunks;
    qm31 acc = q_of(p[0]);
    for (uint32_t r = 1; r < g.chunks; r++) {
        acc = qm31_add(qm31_mul(acc, step), q_of(p[r]));
        p[r] = u_of(acc);
    }
}

// The same recurrence with one WARP per group (groups of at most 256 rows): lane l takes rows 8l .. 8l+7, runs them from a
// zero carry into registers, the lanes' (multiplier, value) pairs are combined by a shuffle scan of affine maps
// ((A2, B2) o (A1, B1) = (A1 A2, B1 A2 + B2)), and each lane then adds its carry times the running power of the step. All
// lanes of the group go through the same warp one after the other, so that the product u_m v of the group's last row
// (what the prefix over groups sums) is at hand and is written to prod[m][slot]. One thread per (group, lane) walking 256
// rows in sequence kept 6% of the warp slots busy and took as long as the pass over all the input columns.
struct ScanSteps {
    qm31 pw[2][9];  // pw[kind][k] = step^k for k = 0..8; kind 0 is lane 0 (v, step s^pq), kind 1 the lanes u_m (step rv^pk)
};
__global__ void __launch_bounds__(256) freivalds_group_scan_warp_kernel(uint4* __restrict__ lanes, FGrid g, uint32_t n_mats, ScanSteps st,
                                                                        uint4* __restrict__ prod) {
    const uint32_t slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    if (slot >= g.groups) return;
    const uint32_t r0 = lane * 8u, n_here = r0 >= g.chunks ? 0u : (g.chunks - r0 < 8u ? g.chunks - r0 : 8u);
    qm31 v_last = qm31_zero();
    for (uint32_t l = 0; l <= n_mats; l++) {
        const qm31* pw = st.pw[l ? 1 : 0];
        const qm31 step = pw[1];
        uint4* __restrict__ p = lanes + ((size_t)l << g.log_rows) + g.lead + (size_t)slot * g.chunks + r0;
        qm31 y[8];
        qm31 acc = qm31_zero();
#pragma unroll
        for (uint32_t k = 0; k < 8; k++)
            if (k < n_here) {
                acc = qm31_add(qm31_mul(acc, step), q_of(p[k]));
                y[k] = acc;
            }
        const qm31 mult = pw[n_here];  // this lane's map: x -> mult x + acc
        // inclusive scan of the maps over the lanes
        qm31 A = mult, B = acc;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            qm31 a1, b1;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                a1.c[c] = __shfl_up_sync(0xffffffffu, A.c[c], off);
                b1.c[c] = __shfl_up_sync(0xffffffffu, B.c[c], off);
            }
            if ((int)lane >= off) {
                B = qm31_add(qm31_mul(b1, A), B);
                A = qm31_mul(a1, A);
            }
        }
        // carry into this lane = the value at the end of the previous lane
        qm31 carry;
#pragma unroll
        for (int c = 0; c < 4; c++) carry.c[c] = __shfl_up_sync(0xffffffffu, B.c[c], 1);
        if (lane == 0) carry = qm31_zero();
#pragma unroll
        for (uint32_t k = 0; k < 8; k++)
            if (k < n_here) p[k] = u_of(qm31_add(y[k], qm31_mul(carry, pw[k + 1])));
        // the group's last row is in the last lane that has rows; B of lane 31 is the value there either way
        qm31 end;
#pragma unroll
        for (int c = 0; c < 4; c++) end.c[c] = __shfl_sync(0xffffffffu, B.c[c], 31);
        if (l == 0) v_last = end;
        else if (lane == 0) prod[(size_t)(l - 1) * g.groups + slot] = u_of(qm31_mul(end, v_last));
    }
}

// prefix[m][slot] = sum over slots <= slot of prod[m][slot]; one CTA, coalesced reads.
__global__ void __launch_bounds__(1024) freivalds_prefix_prod_kernel(const uint4* __restrict__ prod, uint32_t groups, uint32_t n_mats,
                                                                     uint4* __restrict__ prefix) {
    __shared__ uint32_t warp_tot[32][4];
    __shared__ uint32_t carry_s[4];
    const int lane_id = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t m = 0; m < n_mats; m++) {
        if (threadIdx.x < 4) carry_s[threadIdx.x] = 0;
        __syncthreads();
        for (uint32_t base = 0; base < groups; base += blockDim.x) {
            const uint32_t slot = base + threadIdx.x;
            qm31 x = slot < groups ? q_of(prod[(size_t)m * groups + slot]) : qm31_zero();
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                qm31 o;
#pragma unroll
                for (int k = 0; k < 4; k++) o.c[k] = __shfl_up_sync(0xffffffffu, x.c[k], off);
                if (lane_id >= off) x = qm31_add(x, o);
            }
            if (lane_id == 31)
                for (int k = 0; k < 4; k++) warp_tot[warp][k] = x.c[k];
            __syncthreads();
            qm31 pre{{carry_s[0], carry_s[1], carry_s[2], carry_s[3]}};
            for (int w = 0; w < warp; w++) pre = qm31_add(pre, qm31{{warp_tot[w][0], warp_tot[w][1], warp_tot[w][2], warp_tot[w][3]}});
            x = qm31_add(x, pre);
            if (slot < groups) prefix[(size_t)m * groups + slot] = u_of(x);
            __syncthreads();
            if (threadIdx.x == blockDim.x - 1)
                for (int k = 0; k < 4; k++) carry_s[k] = x.c[k];
            __syncthreads();
        }
    }
}

// One CTA: prefix[m][slot] = sum over slots <= slot of u_m[last row] * v[last row].
__global__ void __launch_bounds__(1024) freivalds_prefix_kernel(const uint4* __restrict__ lanes, FGrid g, uint32_t n_mats,
                                                                uint4* __restrict__ prefix) {
    __shared__ uint32_t warp_tot[32][4];
    __shared__ uint32_t carry_s[4];
    const uint32_t rows = 1u << g.log_rows;
    const int lane_id = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t m = 0; m < n_mats; m++) {
        if (threadIdx.x < 4) carry_s[threadIdx.x] = 0;
        __syncthreads();
        for (uint32_t base = 0; base < g.groups; base += blockDim.x) {
            uint32_t slot = base + threadIdx.x;
            qm31 x = qm31_zero();
            if (slot < g.groups) {
                size_t last = (size_t)g.lead + (size_t)slot * g.chunks + g.chunks - 1;
                x = qm31_mul(q_of(lanes[(size_t)(1 + m) * rows + last]), q_of(lanes[last]));
            }
            // inclusive scan inside the warp
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                qm31 o;
#pragma unroll
                for (int k = 0; k < 4; k++) o.c[k] = __shfl_up_sync(0xffffffffu, x.c[k], off);
                if (lane_id >= off) x = qm31_add(x, o);
            }
            if (lane_id == 31)
                for (int k = 0; k < 4; k++) warp_tot[warp][k] = x.c[k];
            __syncthreads();
            qm31 pre{{carry_s[0], carry_s[1], carry_s[2], carry_s[3]}};
            for (int w = 0; w < warp; w++) pre = qm31_add(pre, qm31{{warp_tot[w][0], warp_tot[w][1], warp_tot[w][2], warp_tot[w][3]}});
            x = qm31_add(x, pre);
            if (slot < g.groups) prefix[(size_t)m * g.groups + slot] = u_of(x);
            __syncthreads();
            if (threadIdx.x == blockDim.x - 1)
                for (int k = 0; k < 4; k++) carry_s[k] = x.c[k];
            __syncthreads();
        }
    }
}

// out: (1 + 2 n_mats) secure columns of 4 coordinate columns each, committed order.
__global__ void __launch_bounds__(256) freivalds_split_kernel(const uint4* __restrict__ lanes, const uint4* __restrict__ prefix, FGrid g,
                                                              uint32_t n_mats, uint32_t* const* __restrict__ out) {
    const uint32_t rows = 1u << g.log_rows;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows) return;
    const uint32_t j = coset_perm(i, g.log_rows);
    const bool some = j >= g.lead;
    uint32_t slot = 0;
    bool last = false;
    if (some) {
        slot = (j - g.lead) / g.chunks;
        last = (j - g.lead) % g.chunks == g.chunks - 1;
    }
    uint4 v = lanes[j];
    out[0][i] = v.x; out[1][i] = v.y; out[2][i] = v.z; out[3][i] = v.w;
    for (uint32_t m = 0; m < n_mats; m++) {
        uint4 u = lanes[(size_t)(1 + m) * rows + j];
        uint32_t* const* ou = out + 4 + 8 * m;
        ou[0][i] = u.x; ou[1][i] = u.y; ou[2][i] = u.z; ou[3][i] = u.w;
        uint4 a = make_uint4(0, 0, 0, 0);
        if (some) {
            if (last) a = prefix[(size_t)m * g.groups + slot];
            else if (slot > 0) a = prefix[(size_t)m * g.groups + slot - 1];
        }
        uint32_t* const* oa = out + 8 + 8 * m;
        oa[0][i] = a.x; oa[1][i] = a.y; oa[2][i] = a.z; oa[3][i] = a.w;
    }
}

static bool grid_ok(const zkb_grid* g) {
    if (!g || g->log_rows < 1 || g->log_rows > 28 || g->groups == 0 || g->chunks == 0) return false;
    uint64_t rows = 1ull << g->log_rows;
    return (uint64_t)g->groups * g->chunks + g->lead == rows;
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_freivalds_scatter(zkb_ctx* ctx, const int8_t* qx, const int8_t* const* qw, const uint32_t* h_n_out, const zkb_grid* grid,
                          uint32_t pq, uint32_t pk, uint32_t n_in, uint32_t tokens, uint32_t n_mats, uint32_t* const* base_cols,
                          uint32_t* const* pre_cols, uint32_t* m_r8, uint32_t table_len, unsigned long long* off_table) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, grid_ok(grid) && grid->groups == n_in);
    ZKB_CHECK_ARG(ctx, qx && qw && h_n_out && base_cols && pre_cols && m_r8 && off_table && pq >= 1 && pk >= 1 && n_mats >= 1);
    ZKB_CHECK_ARG(ctx, table_len >= 1 && table_len <= 8192 && n_mats <= 64);
    ZKB_CHECK_ARG(ctx, (uint64_t)grid->chunks * pq >= tokens);
    for (uint32_t m = 0; m < n_mats; m++) ZKB_CHECK_ARG(ctx, qw[m] != nullptr && (uint64_t)grid->chunks * pk >= h_n_out[m]);
    DeviceGuard g(ctx);
    void **d_base, **d_pre, **d_qw;
    int rc = stage_ptrs(ctx, (const void* const*)base_cols, (int)pq, &d_base);
    if (rc) return rc;
    rc = stage_ptrs(ctx, (const void* const*)pre_cols, (int)(n_mats * pk + 4), &d_pre);
    if (rc) return rc;
    rc = stage_ptrs(ctx, (const void* const*)qw, (int)n_mats, &d_qw);
    if (rc) return rc;
    uint32_t* d_nout = ctx->scratch;
    ZKB_CUDA(ctx, cudaMemcpyAsync(d_nout, h_n_out, n_mats * 4, cudaMemcpyHostToDevice, ctx->stream));
    FGrid fg{grid->log_rows, grid->groups, grid->chunks, grid->lead};
    uint32_t rows = 1u << grid->log_rows;
    ProfScope prof(ctx, "freivalds_scatter_kernel");
    freivalds_scatter_kernel<<<(rows + 255) / 256, 256, table_len * 4, ctx->stream>>>(
        qx, (const int8_t* const*)d_qw, d_nout, fg, pq, pk, n_in, tokens, n_mats, (uint32_t* const*)d_base, (uint32_t* const*)d_pre,
        m_r8, table_len, off_table);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_freivalds_acc(zkb_ctx* ctx, const uint32_t* const* base_cols, const uint32_t* const* pre_cols, const zkb_grid* grid, uint32_t pq,
                      uint32_t pk, uint32_t n_mats, const uint32_t h_s[4], const uint32_t h_rv[4], uint32_t* const* out_cols,
                      uint32_t* h_claims) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, grid_ok(grid) && base_cols && pre_cols && h_s && h_rv && out_cols && h_claims);
    ZKB_CHECK_ARG(ctx, pq >= 1 && pk >= 1 && n_mats >= 1 && n_mats <= 64 && (size_t)(pq + pk) * 4 <= ctx->scratch_words);
    DeviceGuard g(ctx);
    const size_t rows = (size_t)1 << grid->log_rows;
    const uint32_t n_lanes = 1 + n_mats;
    // powers of the two challenges, and their steps s^pq, rv^pk (prover/src/relations.rs:85-93)
    std::vector<qm31> pows;
    qm31 s{{h_s[0], h_s[1], h_s[2], h_s[3]}}, rv{{h_rv[0], h_rv[1], h_rv[2], h_rv[3]}};
    qm31 cur = qm31_one();
    for (uint32_t p = 0; p < pq; p++) { pows.push_back(cur); cur = qm31_mul(cur, s); }
    qm31 s_step = cur;
    cur = qm31_one();
    for (uint32_t p = 0; p < pk; p++) { pows.push_back(cur); cur = qm31_mul(cur, rv); }
    qm31 rv_step = cur;
    // the powers go up through the pinned staging ring (two 8-byte slots each): no synchronisation with the work before
    void **d_base, **d_pre, **d_out, **d_pw;
    int rc = ZKB_OK;
    if (ctx->ring_pos & 1) {  // the ring hands out 8-byte slots; the kernels read the powers as 16-byte words
        const void* pad = nullptr;
        if ((rc = stage_ptrs(ctx, &pad, 1, &d_pw))) return rc;
    }
    if ((rc = stage_ptrs(ctx, reinterpret_cast<const void* const*>(pows.data()), (int)(pows.size() * 2), &d_pw))) return rc;
    if ((uintptr_t)d_pw & 15) return set_error(ctx, ZKB_ECUDA, "zkb_freivalds_acc: staging ring misaligned");
    uint4* d_pows = reinterpret_cast<uint4*>(d_pw);
    rc = stage_ptrs(ctx, (const void* const*)base_cols, (int)pq, &d_base);
    if (rc) return rc;
    rc = stage_ptrs(ctx, (const void* const*)pre_cols, (int)(n_mats * pk), &d_pre);
    if (rc) return rc;
    rc = stage_ptrs(ctx, (const void* const*)out_cols, (int)((1 + 2 * n_mats) * 4), &d_out);
    if (rc) return rc;
    // work buffers from the stream-ordered pool: lanes in coset order, prefix over groups
    uint4 *lanes = nullptr, *prefix = nullptr;
    ZKB_CUDA(ctx, cudaMallocAsync((void**)&lanes, (size_t)n_lanes * rows * 16, ctx->stream));
    cudaError_t e = cudaMallocAsync((void**)&prefix, (size_t)n_mats * grid->groups * 16, ctx->stream);
    if (e != cudaSuccess) { cudaFreeAsync(lanes, ctx->stream); return set_error(ctx, ZKB_ENOMEM, "zkb_freivalds_acc: %s", cudaGetErrorString(e)); }
    FGrid fg{grid->log_rows, grid->groups, grid->chunks, grid->lead};
    {
        ProfScope prof(ctx, "freivalds_inner_kernel");
        freivalds_inner_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(
            (const uint32_t* const*)d_base, (const uint32_t* const*)d_pre, d_pows, d_pows + pq, fg, pq, pk, n_mats, lanes);
    }
    if (grid->chunks <= 256) {
        ScanSteps scan_steps;
        for (int kind = 0; kind < 2; kind++) {
            scan_steps.pw[kind][0] = qm31_one();
            for (int k = 1; k <= 8; k++) scan_steps.pw[kind][k] = qm31_mul(scan_steps.pw[kind][k - 1], kind ? rv_step : s_step);
        }
        uint4* prod = nullptr;  // u_m v at each group's last row
        e = cudaMallocAsync((void**)&prod, (size_t)n_mats * grid->groups * 16, ctx->stream);
        if (e != cudaSuccess) {
            cudaFreeAsync(lanes, ctx->stream);
            cudaFreeAsync(prefix, ctx->stream);
            return set_error(ctx, ZKB_ENOMEM, "zkb_freivalds_acc: %s", cudaGetErrorString(e));
        }
        {
            ProfScope prof(ctx, "freivalds_group_scan_kernel");
            freivalds_group_scan_warp_kernel<<<(unsigned)(((size_t)grid->groups * 32 + 255) / 256), 256, 0, ctx->stream>>>(
                lanes, fg, n_mats, scan_steps, prod);
        }
        {
            ProfScope prof(ctx, "freivalds_prefix_kernel");
            freivalds_prefix_prod_kernel<<<1, 1024, 0, ctx->stream>>>(prod, grid->groups, n_mats, prefix);
        }
        cudaFreeAsync(prod, ctx->stream);
    } else {
        {
            ProfScope prof(ctx, "freivalds_group_scan_kernel");
            unsigned threads_total = grid->groups * n_lanes;
            freivalds_group_scan_kernel<<<(threads_total + 127) / 128, 128, 0, ctx->stream>>>(lanes, fg, n_lanes, s_step, rv_step);
        }
        {
            ProfScope prof(ctx, "freivalds_prefix_kernel");
            freivalds_prefix_kernel<<<1, 1024, 0, ctx->stream>>>(lanes, fg, n_mats, prefix);
        }
    }
    {
        ProfScope prof(ctx, "freivalds_split_kernel");
        freivalds_split_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(lanes, prefix, fg, n_mats, (uint32_t* const*)d_out);
    }
    e = cudaGetLastError();
    for (uint32_t m = 0; m < n_mats && e == cudaSuccess; m++)
        e = cudaMemcpyAsync(ctx->h_small + 4 * m, prefix + (size_t)m * grid->groups + grid->groups - 1, 16, cudaMemcpyDeviceToHost, ctx->stream);
    cudaFreeAsync(lanes, ctx->stream);
    cudaFreeAsync(prefix, ctx->stream);
    if (e != cudaSuccess) return set_error(ctx, ZKB_ECUDA, "zkb_freivalds_acc: %s", cudaGetErrorString(e));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(h_claims, ctx->h_small, (size_t)n_mats * 16);
    return ZKB_OK;
}

}  // extern "C"
