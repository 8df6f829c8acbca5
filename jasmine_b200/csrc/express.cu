// Expression evaluator: fused elementwise programs, row/column reductions,
// softmax, LayerNorm and RMSNorm in single kernels.
//
// The host lowers an expression tree (the reference's lazy nodes,
// mat_express_t.hpp:35-509) to a postfix program.  On the device the program
// runs on a value stack kept in registers (a shift-register stack: every index
// is static), one stack per 128-bit vector of four elements.  Row kernels keep
// the whole row in registers between the reduction and the write, so each
// operand is read once and the result written once.
#include "common.cuh"
#include "tc_utils.cuh"
#include <stdlib.h>
#include <math.h>
#include <string.h>

namespace jsm {

enum LeafKind { LK_FULL = 0, LK_ROWVEC = 1, LK_COLVEC = 2, LK_SCALAR = 3, LK_GENERIC = 4 };
enum ProKind { PRO_GENERIC = 0, PRO_LEAF = 1, PRO_AXPB = 2 /* l0*imm + l1 */, PRO_ADD = 3 /* l0 + l1 */ };

struct LeafDesc {
    const void* p;
    int rows, cols;
    long long rs, cs;
    int dtype;
    int kind;
};

struct EvalParams {
    int n_instr, n_leaves, pro;
    float pro_imm;
    signed char op[JSM_MAX_INSTR];
    signed char arg[JSM_MAX_INSTR];
    float imm[JSM_MAX_INSTR];
    LeafDesc leaf[JSM_MAX_LEAVES];
};

struct OutDesc {
    void* p;
    int rows, cols;
    long long rs, cs;
    int dtype;
    int vec;  // contiguous rows, 16-byte aligned: vector stores allowed
};

struct RowsArgs {
    int kind, R, C;
    const float* gain;
    const float* bias;
    float eps;
    OutDesc out;
};

// ---- leaf access ------------------------------------------------------------
__device__ __forceinline__ float load_elem(const void* p, long long idx, int dtype) {
    if (dtype == JSM_F32) return reinterpret_cast<const float*>(p)[idx];
    return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p)[idx]);
}

__device__ __forceinline__ float leaf_at(const LeafDesc& L, int r, int c) {
    int rr = (r < L.rows) ? r : r % L.rows;
    int cc = (c < L.cols) ? c : c % L.cols;
    return load_elem(L.p, rr * L.rs + cc * L.cs, L.dtype);
}

// four consecutive columns c..c+3 of row r (c % 4 == 0); only for kinds != GENERIC
__device__ __forceinline__ void leaf_vec4(const LeafDesc& L, int r, int c, float (&v)[4]) {
    if (L.kind == LK_FULL || L.kind == LK_ROWVEC) {
        long long base = (L.kind == LK_FULL ? r * L.rs : 0) + c;
        if (L.dtype == JSM_F32) {
            float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(L.p) + base);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
            uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(L.p) + base);
            v[0] = bf16lo(t.x); v[1] = bf16hi(t.x); v[2] = bf16lo(t.y); v[3] = bf16hi(t.y);
        }
    } else {
        float s = (L.kind == LK_COLVEC) ? load_elem(L.p, r * L.rs, L.dtype) : load_elem(L.p, 0, L.dtype);
        v[0] = v[1] = v[2] = v[3] = s;
    }
}

// ---- scalar ops ---------------------------------------------------------------
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }

__device__ __forceinline__ float apply_unary(int op, float x, float imm) {
    switch (op) {
        case JSM_OP_EXP: return expf(x);
        case JSM_OP_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case JSM_OP_POW: return imm == 2.0f ? x * x : powf(x, imm);
        case JSM_OP_SQRT: return sqrtf(x);
        case JSM_OP_NEG: return -x;
        case JSM_OP_RELU: return x > 0.0f ? x : 0.0f * x;  // (x > 0) * x keeps the sign of zero and NaN
        case JSM_OP_GELU: return gelu_erf(x);
        case JSM_OP_SILU: return x / (1.0f + expf(-x));
        case JSM_OP_TANH: return tanhf(x);
        default: return x;
    }
}
__device__ __forceinline__ float apply_binary(int op, float a, float b) {
    switch (op) {
        case JSM_OP_ADD: return a + b;
        case JSM_OP_SUB: return a - b;
        case JSM_OP_MUL: return a * b;
        case JSM_OP_DIV: return a / b;
        case JSM_OP_GT: return a > b ? 1.0f : 0.0f;
        case JSM_OP_LT: return a < b ? 1.0f : 0.0f;
        default: return a;
    }
}

// ---- the interpreter: V elements at a time, stack depth DEPTH ------------------
// VEC: the V(=4) elements are columns c..c+3 fetched with vector loads;
// otherwise V == 1 and leaves are fetched with modulo indexing.
template <int DEPTH, int V, bool VEC>
__device__ __forceinline__ void eval_program(const EvalParams& P, int r, int c, float (&out)[V]) {
    if (VEC) {
        if (P.pro == PRO_LEAF) {
            float a[4];
            leaf_vec4(P.leaf[0], r, c, a);
#pragma unroll
            for (int i = 0; i < V; ++i) out[i] = a[i];
            return;
        }
        if (P.pro == PRO_AXPB || P.pro == PRO_ADD) {
            float a[4], b[4];
            leaf_vec4(P.leaf[0], r, c, a);
            leaf_vec4(P.leaf[1], r, c, b);
#pragma unroll
            for (int i = 0; i < V; ++i)
                out[i] = (P.pro == PRO_AXPB) ? __fadd_rn(__fmul_rn(a[i], P.pro_imm), b[i]) : a[i] + b[i];
            return;
        }
    }
    float s[DEPTH][V];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d)
#pragma unroll
        for (int i = 0; i < V; ++i) s[d][i] = 0.0f;
    for (int ip = 0; ip < P.n_instr; ++ip) {
        int op = P.op[ip];
        if (op == JSM_OP_LEAF || op == JSM_OP_IMM) {
#pragma unroll
            for (int d = DEPTH - 1; d > 0; --d)
#pragma unroll
                for (int i = 0; i < V; ++i) s[d][i] = s[d - 1][i];
            if (op == JSM_OP_IMM) {
                float x = P.imm[ip];
#pragma unroll
                for (int i = 0; i < V; ++i) s[0][i] = x;
            } else {
                const LeafDesc& L = P.leaf[P.arg[ip]];
                if (VEC) {
                    float a[4];
                    leaf_vec4(L, r, c, a);
#pragma unroll
                    for (int i = 0; i < V; ++i) s[0][i] = a[i];
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) s[0][i] = leaf_at(L, r, c + i);
                }
            }
        } else if (op >= JSM_OP_ADD && op <= JSM_OP_LT) {
#pragma unroll
            for (int i = 0; i < V; ++i) s[0][i] = apply_binary(op, s[1][i], s[0][i]);
#pragma unroll
            for (int d = 1; d < DEPTH - 1; ++d)
#pragma unroll
                for (int i = 0; i < V; ++i) s[d][i] = s[d + 1][i];
        } else {
            float imm = P.imm[ip];
#pragma unroll
            for (int i = 0; i < V; ++i) s[0][i] = apply_unary(op, s[0][i], imm);
        }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = s[0][i];
}

__device__ __forceinline__ void store_elem(const OutDesc& O, int r, int c, float v) {
    long long idx = r * O.rs + c * O.cs;
    if (O.dtype == JSM_F32)
        reinterpret_cast<float*>(O.p)[idx] = v;
    else if (O.dtype == JSM_BF16)
        reinterpret_cast<uint16_t*>(O.p)[idx] = f32_to_bf16_bits(v);
    else
        reinterpret_cast<int32_t*>(O.p)[idx] = (int32_t)v;
}
__device__ __forceinline__ void store_vec4(const OutDesc& O, int r, int c, const float (&v)[4]) {
    long long idx = r * O.rs + c;
    if (O.dtype == JSM_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(O.p) + idx) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint2 t;
        t.x = pack_bf16x2(v[0], v[1]);
        t.y = pack_bf16x2(v[2], v[3]);
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(O.p) + idx) = t;
    }
}

// ---- K1: elementwise -----------------------------------------------------------
template <int DEPTH, bool VEC>
__global__ void __launch_bounds__(256) elementwise_kernel(EvalParams P, OutDesc O) {
    const int R = O.rows, C = O.cols;
    if (VEC) {
        const long long cv = C / 4;
        const long long total = (long long)R * cv;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
             i += (long long)gridDim.x * blockDim.x) {
            int r = (int)(i / cv);
            int c = (int)(i % cv) * 4;
            float v[4];
            eval_program<DEPTH, 4, true>(P, r, c, v);
            store_vec4(O, r, c, v);
        }
    } else {
        const long long total = (long long)R * C;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
             i += (long long)gridDim.x * blockDim.x) {
            int r = (int)(i / C);
            int c = (int)(i % C);
            float v[1];
            eval_program<DEPTH, 1, false>(P, r, c, v);
            store_elem(O, r, c, v[0]);
        }
    }
}

// ---- K1f: the programs x * imm + y and x + y over contiguous f32 matrices ---------------
// Four vectors per operand and thread are requested before the first use: 128 bytes in flight per thread.
template <int PRO>
__global__ void __launch_bounds__(256) elementwise_fast_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float imm,
                                                               float4* __restrict__ out, long long n_vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n_vec; i += 4 * stride) {
        float4 x[4], y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { x[u] = __ldcs(a + i + u * stride); y[u] = __ldcs(b + i + u * stride); }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float4 r;
            if (PRO == PRO_AXPB) {
                r.x = __fadd_rn(__fmul_rn(x[u].x, imm), y[u].x); r.y = __fadd_rn(__fmul_rn(x[u].y, imm), y[u].y);
                r.z = __fadd_rn(__fmul_rn(x[u].z, imm), y[u].z); r.w = __fadd_rn(__fmul_rn(x[u].w, imm), y[u].w);
            } else {
                r.x = x[u].x + y[u].x; r.y = x[u].y + y[u].y; r.z = x[u].z + y[u].z; r.w = x[u].w + y[u].w;
            }
            __stcs(out + i + u * stride, r);
        }
    }
    for (; i < n_vec; i += stride) {
        const float4 x = a[i], y = b[i];
        float4 r;
        if (PRO == PRO_AXPB) {
            r.x = __fadd_rn(__fmul_rn(x.x, imm), y.x); r.y = __fadd_rn(__fmul_rn(x.y, imm), y.y);
            r.z = __fadd_rn(__fmul_rn(x.z, imm), y.z); r.w = __fadd_rn(__fmul_rn(x.w, imm), y.w);
        } else {
            r.x = x.x + y.x; r.y = x.y + y.y; r.z = x.z + y.z; r.w = x.w + y.w;
        }
        out[i] = r;
    }
}

// ---- group reductions (GROUP = 32: one warp per row, 256: one CTA per row) -------
template <int GROUP>
__device__ __forceinline__ float group_sum(float v, float* smem) {
    v = warp_sum(v);
    if (GROUP > 32) {
        __syncthreads();
        if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
        __syncthreads();
        v = 0.0f;
        const int g0 = (threadIdx.x / GROUP) * (GROUP / 32);  // first warp of this row's group
#pragma unroll
        for (int w = 0; w < GROUP / 32; ++w) v += smem[g0 + w];
    }
    return v;
}
template <int GROUP>
__device__ __forceinline__ float group_max(float v, float* smem) {
    v = warp_max(v);
    if (GROUP > 32) {
        __syncthreads();
        if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
        __syncthreads();
        const int g0 = (threadIdx.x / GROUP) * (GROUP / 32);
        v = smem[g0];
#pragma unroll
        for (int w = 1; w < GROUP / 32; ++w) v = fmaxf(v, smem[g0 + w]);
    }
    return v;
}
// (value, index) maximum; ties go to the smaller index
template <int GROUP>
__device__ __forceinline__ void group_argmax(float& v, int& idx, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (GROUP > 32) {
        int* ismem = reinterpret_cast<int*>(smem + 8);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) { smem[threadIdx.x >> 5] = v; ismem[threadIdx.x >> 5] = idx; }
        __syncthreads();
        const int g0 = (threadIdx.x / GROUP) * (GROUP / 32);
        v = smem[g0]; idx = ismem[g0];
#pragma unroll
        for (int w = 1; w < GROUP / 32; ++w) {
            float ov = smem[g0 + w]; int oi = ismem[g0 + w];
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
    }
}

// ---- K2/K3/K4: one row per GROUP threads, row resident in registers ---------------
// VPT vectors of four elements per thread: C <= GROUP * VPT * 4.
template <int GROUP, int VPT, int DEPTH, bool VEC>
__device__ __forceinline__ void rows_block(const EvalParams& P, const RowsArgs& A, int block, float* smem) {
    constexpr int RPC = 256 / GROUP;
    const int row = block * RPC + threadIdx.x / GROUP;
    const int t = threadIdx.x % GROUP;
    const int C = A.C;
    const bool row_ok = row < A.R;  // GROUP == 256 -> always true
    float v[VPT][4];
    // column of element j of vector i
    auto col_of = [&](int i, int j) { return VEC ? (i * GROUP + t) * 4 + j : (i * 4 + j) * GROUP + t; };
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (VEC) {
            int c = (i * GROUP + t) * 4;
            if (row_ok && c < C) {
                eval_program<DEPTH, 4, true>(P, row, c, v[i]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[i][j] = 0.0f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c = col_of(i, j);
                float o[1] = {0.0f};
                if (row_ok && c < C) eval_program<DEPTH, 1, false>(P, row, c, o);
                v[i][j] = o[0];
            }
        }
    }
    const int kind = A.kind;
    const float NEG_INF = -INFINITY;

    if (kind == JSM_ROWS_SUM || kind == JSM_ROWS_MEAN) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s += (col_of(i, j) < C) ? v[i][j] : 0.0f;
        s = group_sum<GROUP>(s, smem);
        if (kind == JSM_ROWS_MEAN) s = s / (float)C;
        if (t == 0 && row_ok) store_elem(A.out, row, 0, s);
        return;
    }
    if (kind == JSM_ROWS_MAX || kind == JSM_ROWS_ARGMAX) {
        float m = NEG_INF;
        int mi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c = col_of(i, j);
                if (c < C && (v[i][j] > m || (v[i][j] == m && c < mi))) { m = v[i][j]; mi = c; }
            }
        if (kind == JSM_ROWS_MAX) {
            m = group_max<GROUP>(m, smem);
            if (t == 0 && row_ok) store_elem(A.out, row, 0, m);
        } else {
            group_argmax<GROUP>(m, mi, smem);
            if (t == 0 && row_ok) {
                long long idx = row * A.out.rs;
                if (A.out.dtype == JSM_I32)
                    reinterpret_cast<int32_t*>(A.out.p)[idx] = mi;
                else
                    store_elem(A.out, row, 0, (float)mi);
            }
        }
        return;
    }
    if (kind == JSM_ROWS_SOFTMAX) {
        float m = NEG_INF;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (col_of(i, j) < C) m = fmaxf(m, v[i][j]);
        m = group_max<GROUP>(m, smem);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // exp through ex2.approx of (x - m) * log2(e): relative error below 2e-6 for the arguments of a softmax row
                float e = (col_of(i, j) < C) ? exp2f((v[i][j] - m) * 1.4426950408889634f) : 0.0f;
                v[i][j] = e;
                s += e;
            }
        s = group_sum<GROUP>(s, smem);
        const float inv_s = 1.0f / s;  // one division per row; x * (1/s) is within one ulp of x / s
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) v[i][j] = v[i][j] * inv_s;
    } else {
        float mean = 0.0f;
        if (kind == JSM_ROWS_LAYERNORM) {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s += (col_of(i, j) < C) ? v[i][j] : 0.0f;
            mean = group_sum<GROUP>(s, smem) / (float)C;
        }
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float d = v[i][j] - mean;
                v[i][j] = d;
                if (col_of(i, j) < C) q = __fmaf_rn(d, d, q);  // pinned: the staged kernel forms the same sums
            }
        q = group_sum<GROUP>(q, smem) / (float)C;
        const float inv_sd = 1.0f / sqrtf(q + A.eps);  // one division per row
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c = col_of(i, j);
                if (c < C) {
                    float g = A.gain ? A.gain[c] : 1.0f;
                    float b = (A.bias && kind == JSM_ROWS_LAYERNORM) ? A.bias[c] : 0.0f;
                    v[i][j] = __fmaf_rn(g, __fmul_rn(v[i][j], inv_sd), b);
                }
            }
    }
    if (!row_ok) return;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (VEC && A.out.vec) {
            int c = (i * GROUP + t) * 4;
            if (c < C) store_vec4(A.out, row, c, v[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c = col_of(i, j);
                if (c < C) store_elem(A.out, row, c, v[i][j]);
            }
        }
    }
}

// The grid may be smaller than the number of row blocks: a CTA then walks several.
template <int GROUP, int VPT, int DEPTH, bool VEC>
__global__ void __launch_bounds__(256) rows_kernel(EvalParams P, RowsArgs A, int n_blocks) {
    __shared__ float smem[16];
    for (int block = blockIdx.x; block < n_blocks; block += gridDim.x) {
        rows_block<GROUP, VPT, DEPTH, VEC>(P, A, block, smem);
        __syncthreads();  // the reduction scratch is reused by the next row block
    }
}

// ---- K2s: rows staged through shared memory by bulk copies -----------------------------
// For f32 operands with contiguous rows of 1024, 2048 or 4096 columns and the programs x, x * imm + y and x + y.
// A fixed grid of two CTAs per SM walks the rows.  One producer thread copies each row of the operands into a ring of
// shared-memory stages with cp.async.bulk (completion on an mbarrier), so the bytes in flight per SM are set by the ring
// (96 KB per CTA) and not by how many rows sit in registers; the 256 consumer threads take a row into registers, release
// the stage at once and run the same arithmetic, in the same order, as rows_block<256, VPT>.  Every mbarrier wait is
// bounded; after a timeout the CTA keeps its barrier counts, stores nothing more and records an error code.
struct StagedArgs {
    const float* a;  // leaf 0
    const float* b;  // leaf 1 (programs with two operands)
    long long rsa, rsb;
    float imm;
    int R;
    const float* gain;
    const float* bias;
    float eps;
    float* out;      // full rows (softmax, norms) or one value per row (reductions)
    long long rso;
    int n_stages;
    int* err;
};
constexpr int RS_THREADS = 288;  // 8 consumer warps + 1 producer warp
constexpr int RS_ERR_FULL = 51, RS_ERR_EMPTY = 52;

__device__ __forceinline__ void rs_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(tc::smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(tc::smem_u32(bar))
                 : "memory");
}
// reductions over the 256 consumer threads, warps added in warp order like group_sum<256>; one named barrier each,
// the caller alternates the scratch rows
__device__ __forceinline__ float rs_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w];
    return s;
}
__device__ __forceinline__ float rs_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    return m;
}

template <int VPT, int KIND, int PRO>
__global__ void __launch_bounds__(RS_THREADS) rows_staged_kernel(StagedArgs A) {
    using namespace tc;
    constexpr int C = 1024 * VPT;
    constexpr int NL = PRO == PRO_LEAF ? 1 : 2;
    constexpr int STAGE_FLOATS = NL * C;
    // plain reductions: every consumer warp owns whole rows (row k of the CTA goes to warp k % 8), so no CTA barrier is
    // needed; a lane plays the threads l, 32 + l, .. 224 + l of the row-per-CTA layout to keep the order of the sums
    constexpr bool WARP_ROWS = KIND == JSM_ROWS_SUM || KIND == JSM_ROWS_MEAN || KIND == JSM_ROWS_MAX;
    extern __shared__ __align__(128) float rs_smem[];
    __shared__ uint64_t full_bar[8], empty_bar[8];
    __shared__ float red[2][8];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_stages = A.n_stages;
    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], WARP_ROWS ? 1 : 8);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 8) {
        if (lane == 0) {
            int it = 0;
            for (int row = blockIdx.x; row < A.R; row += gridDim.x, ++it) {
                const int s = it % n_stages;
                if (it >= n_stages && !mbar_wait(&empty_bar[s], ((it / n_stages) - 1) & 1, &abort_flag, A.err, RS_ERR_EMPTY)) break;
                float* dst = rs_smem + (size_t)s * STAGE_FLOATS;
                mbar_expect_tx(&full_bar[s], STAGE_FLOATS * 4);
                rs_bulk_load(dst, A.a + (long long)row * A.rsa, C * 4, &full_bar[s]);
                if (NL == 2) rs_bulk_load(dst + C, A.b + (long long)row * A.rsb, C * 4, &full_bar[s]);
            }
        }
        return;
    }
    if (WARP_ROWS) {
        for (int it = warp;; it += 8) {
            const long long row = (long long)blockIdx.x + (long long)it * gridDim.x;
            if (row >= A.R) break;
            const int s = it % n_stages;
            if (!mbar_wait(&full_bar[s], (it / n_stages) & 1, &abort_flag, A.err, RS_ERR_FULL)) break;
            const float4* sa = reinterpret_cast<const float4*>(rs_smem + (size_t)s * STAGE_FLOATS);
            float part[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                float acc = KIND == JSM_ROWS_MAX ? -INFINITY : 0.0f;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int q = i * 256 + w * 32 + lane;
                    const float4 x = sa[q];
                    float e[4] = {x.x, x.y, x.z, x.w};
                    if (PRO != PRO_LEAF) {
                        const float4 y = sa[C / 4 + q];
                        if (PRO == PRO_AXPB) {
                            e[0] = __fadd_rn(__fmul_rn(x.x, A.imm), y.x); e[1] = __fadd_rn(__fmul_rn(x.y, A.imm), y.y);
                            e[2] = __fadd_rn(__fmul_rn(x.z, A.imm), y.z); e[3] = __fadd_rn(__fmul_rn(x.w, A.imm), y.w);
                        } else {
                            e[0] = x.x + y.x; e[1] = x.y + y.y; e[2] = x.z + y.z; e[3] = x.w + y.w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc = KIND == JSM_ROWS_MAX ? fmaxf(acc, e[j]) : acc + e[j];
                }
                part[w] = acc;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
            float r;
            if (KIND == JSM_ROWS_MAX) {
                r = part[0];
#pragma unroll
                for (int w = 1; w < 8; ++w) r = fmaxf(r, part[w]);
                r = warp_max(r);
            } else {
#pragma unroll
                for (int w = 0; w < 8; ++w) part[w] = warp_sum(part[w]);
                r = 0.0f;
#pragma unroll
                for (int w = 0; w < 8; ++w) r += part[w];
                if (KIND == JSM_ROWS_MEAN) r = r / (float)C;
            }
            if (lane == 0) A.out[row * A.rso] = r;
        }
        return;
    }
    const int t = threadIdx.x;  // 0..255
    bool ok = true;
    int it = 0, par = 0;
    // the gain and the bias of a norm: the same columns for every row of this CTA
    float4 gain4[VPT], bias4[VPT];
    if (KIND == JSM_ROWS_LAYERNORM || KIND == JSM_ROWS_RMSNORM) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = (i * 256 + t) * 4;
            gain4[i] = A.gain ? *reinterpret_cast<const float4*>(A.gain + c) : make_float4(1.f, 1.f, 1.f, 1.f);
            bias4[i] = (A.bias && KIND == JSM_ROWS_LAYERNORM) ? *reinterpret_cast<const float4*>(A.bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    for (int row = blockIdx.x; row < A.R; row += gridDim.x, ++it) {
        const int s = it % n_stages;
        if (!ok || !mbar_wait(&full_bar[s], (it / n_stages) & 1, &abort_flag, A.err, RS_ERR_FULL)) ok = false;
        const float4* sa = reinterpret_cast<const float4*>(rs_smem + (size_t)s * STAGE_FLOATS);
        float v[VPT][4];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const float4 x = sa[i * 256 + t];
            if (PRO == PRO_LEAF) {
                v[i][0] = x.x; v[i][1] = x.y; v[i][2] = x.z; v[i][3] = x.w;
            } else {
                const float4 y = sa[C / 4 + i * 256 + t];
                if (PRO == PRO_AXPB) {
                    v[i][0] = __fadd_rn(__fmul_rn(x.x, A.imm), y.x); v[i][1] = __fadd_rn(__fmul_rn(x.y, A.imm), y.y);
                    v[i][2] = __fadd_rn(__fmul_rn(x.z, A.imm), y.z); v[i][3] = __fadd_rn(__fmul_rn(x.w, A.imm), y.w);
                } else {
                    v[i][0] = x.x + y.x; v[i][1] = x.y + y.y; v[i][2] = x.z + y.z; v[i][3] = x.w + y.w;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);  // the row is in registers: the stage can be refilled
        if (KIND == JSM_ROWS_SOFTMAX) {
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) m = fmaxf(m, v[i][j]);
            m = rs_max(m, red[0]);
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float e = exp2f((v[i][j] - m) * 1.4426950408889634f);
                    v[i][j] = e;
                    sum += e;
                }
            sum = rs_sum(sum, red[1]);
            const float inv_s = 1.0f / sum;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) v[i][j] = v[i][j] * inv_s;
        } else {  // LayerNorm, RMSNorm
            float mean = 0.0f;
            if (KIND == JSM_ROWS_LAYERNORM) {
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) sum += v[i][j];
                mean = rs_sum(sum, red[0]) / (float)C;
            }
            float q = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float d = v[i][j] - mean;
                    v[i][j] = d;
                    q = __fmaf_rn(d, d, q);
                }
            q = rs_sum(q, KIND == JSM_ROWS_LAYERNORM ? red[1] : red[par]) / (float)C;
            par ^= 1;
            const float inv_sd = 1.0f / sqrtf(q + A.eps);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const float4 g = gain4[i], b = bias4[i];
                v[i][0] = __fmaf_rn(g.x, __fmul_rn(v[i][0], inv_sd), b.x);
                v[i][1] = __fmaf_rn(g.y, __fmul_rn(v[i][1], inv_sd), b.y);
                v[i][2] = __fmaf_rn(g.z, __fmul_rn(v[i][2], inv_sd), b.z);
                v[i][3] = __fmaf_rn(g.w, __fmul_rn(v[i][3], inv_sd), b.w);
            }
        }
        if (ok) {
            float4* dst = reinterpret_cast<float4*>(A.out + (long long)row * A.rso);
#pragma unroll
            for (int i = 0; i < VPT; ++i) __stcs(dst + i * 256 + t, make_float4(v[i][0], v[i][1], v[i][2], v[i][3]));
        }
    }
}

// ---- long rows (C > 8192) and the column axis: re-evaluating multi-pass kernels ----
// One CTA of 256 threads per line.  `along_cols` = reduce over the columns of a row
// (axis 1) else over the rows of a column (axis 0).
template <int DEPTH>
__global__ void __launch_bounds__(256) lines_kernel(EvalParams P, RowsArgs A, int axis) {
    __shared__ float smem[16];
    const int line = blockIdx.x;
    const int L = axis == 1 ? A.C : A.R;  // elements per line
    auto at = [&](int k) {
        float o[1];
        if (axis == 1)
            eval_program<DEPTH, 1, false>(P, line, k, o);
        else
            eval_program<DEPTH, 1, false>(P, k, line, o);
        return o[0];
    };
    auto put = [&](int k, float x) {
        if (axis == 1) store_elem(A.out, line, k, x); else store_elem(A.out, k, line, x);
    };
    auto put0 = [&](float x) {
        if (axis == 1) store_elem(A.out, line, 0, x); else store_elem(A.out, 0, line, x);
    };
    const int kind = A.kind;
    if (kind == JSM_ROWS_SUM || kind == JSM_ROWS_MEAN) {
        float s = 0.0f;
        for (int k = threadIdx.x; k < L; k += 256) s += at(k);
        s = group_sum<256>(s, smem);
        if (kind == JSM_ROWS_MEAN) s = s / (float)L;
        if (threadIdx.x == 0) put0(s);
        return;
    }
    if (kind == JSM_ROWS_MAX || kind == JSM_ROWS_ARGMAX) {
        float m = -INFINITY;
        int mi = 0x7fffffff;
        for (int k = threadIdx.x; k < L; k += 256) {
            float x = at(k);
            if (x > m || (x == m && k < mi)) { m = x; mi = k; }
        }
        if (kind == JSM_ROWS_MAX) {
            m = group_max<256>(m, smem);
            if (threadIdx.x == 0) put0(m);
        } else {
            group_argmax<256>(m, mi, smem);
            if (threadIdx.x == 0) {
                long long idx = axis == 1 ? line * A.out.rs : line * A.out.cs;
                if (A.out.dtype == JSM_I32)
                    reinterpret_cast<int32_t*>(A.out.p)[idx] = mi;
                else
                    put0((float)mi);
            }
        }
        return;
    }
    if (kind == JSM_ROWS_SOFTMAX) {
        float m = -INFINITY;
        for (int k = threadIdx.x; k < L; k += 256) m = fmaxf(m, at(k));
        m = group_max<256>(m, smem);
        float s = 0.0f;
        for (int k = threadIdx.x; k < L; k += 256) s += expf(at(k) - m);
        s = group_sum<256>(s, smem);
        for (int k = threadIdx.x; k < L; k += 256) put(k, expf(at(k) - m) / s);
        return;
    }
    float mean = 0.0f;
    if (kind == JSM_ROWS_LAYERNORM) {
        float s = 0.0f;
        for (int k = threadIdx.x; k < L; k += 256) s += at(k);
        mean = group_sum<256>(s, smem) / (float)L;
    }
    float q = 0.0f;
    for (int k = threadIdx.x; k < L; k += 256) {
        float d = at(k) - mean;
        q += d * d;
    }
    q = group_sum<256>(q, smem) / (float)L;
    const float sd = sqrtf(q + A.eps);
    for (int k = threadIdx.x; k < L; k += 256) {
        float g = A.gain ? A.gain[k] : 1.0f;
        float b = (A.bias && kind == JSM_ROWS_LAYERNORM) ? A.bias[k] : 0.0f;
        put(k, g * ((at(k) - mean) / sd) + b);
    }
}

// ---- whole-matrix reductions: partial per CTA, then one CTA folds the partials -----
template <int DEPTH>
__global__ void __launch_bounds__(256) full_partial_kernel(EvalParams P, int R, int C, int mode /*0 sum 1 max 2 sumexp*/,
                                                           const float* shift, float* partial) {
    __shared__ float smem[16];
    const long long total = (long long)R * C;
    const long long per = (total + gridDim.x - 1) / gridDim.x;
    const long long beg = per * blockIdx.x;
    const long long end = beg + per < total ? beg + per : total;
    float acc = mode == 1 ? -INFINITY : 0.0f;
    const float sh = shift ? shift[0] : 0.0f;
    for (long long i = beg + threadIdx.x; i < end; i += 256) {
        float o[1];
        eval_program<DEPTH, 1, false>(P, (int)(i / C), (int)(i % C), o);
        if (mode == 0) acc += o[0];
        else if (mode == 1) acc = fmaxf(acc, o[0]);
        else acc += expf(o[0] - sh);
    }
    acc = mode == 1 ? group_max<256>(acc, smem) : group_sum<256>(acc, smem);
    if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(256) full_fold_kernel(const float* partial, int n, int mode, float divisor, float* out) {
    __shared__ float smem[16];
    float acc = mode == 1 ? -INFINITY : 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) acc = mode == 1 ? fmaxf(acc, partial[i]) : acc + partial[i];
    acc = mode == 1 ? group_max<256>(acc, smem) : group_sum<256>(acc, smem);
    if (threadIdx.x == 0) out[0] = divisor != 0.0f ? acc / divisor : acc;
}
template <int DEPTH>
__global__ void __launch_bounds__(256) full_softmax_write_kernel(EvalParams P, OutDesc O, const float* mx, const float* sum) {
    const long long total = (long long)O.rows * O.cols;
    const float m = mx[0], s = sum[0];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int r = (int)(i / O.cols), c = (int)(i % O.cols);
        float o[1];
        eval_program<DEPTH, 1, false>(P, r, c, o);
        store_elem(O, r, c, expf(o[0] - m) / s);
    }
}

// ---- host side: validation and lowering of the arguments ----------------------------
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct Lowered {
    EvalParams P;
    int R, C, depth;
    bool vec;
};

static jsm_status lower(const jsm_instr* prog, int n_instr, const jsm_mat* leaves, int n_leaves, Lowered& Lw,
                        const char* who) {
    if (n_instr <= 0 || n_instr > JSM_MAX_INSTR || !prog)
        JSM_FAIL(JSM_INVALID_ARG, "%s: program length %d outside 1..%d", who, n_instr, JSM_MAX_INSTR);
    if (n_leaves < 0 || n_leaves > JSM_MAX_LEAVES || (n_leaves > 0 && !leaves))
        JSM_FAIL(JSM_INVALID_ARG, "%s: %d leaves outside 0..%d", who, n_leaves, JSM_MAX_LEAVES);
    EvalParams& P = Lw.P;
    memset(&P, 0, sizeof(P));
    P.n_instr = n_instr;
    P.n_leaves = n_leaves;
    int R = 1, C = 1;
    for (int i = 0; i < n_leaves; ++i) {
        const jsm_mat& m = leaves[i];
        if (!m.data || m.rows <= 0 || m.cols <= 0)
            JSM_FAIL(JSM_INVALID_ARG, "%s: leaf %d is empty (%d x %d)", who, i, m.rows, m.cols);
        if (m.dtype != JSM_F32 && m.dtype != JSM_BF16) JSM_FAIL(JSM_UNSUPPORTED, "%s: leaf %d dtype %d", who, i, m.dtype);
        R = m.rows > R ? m.rows : R;
        C = m.cols > C ? m.cols : C;
    }
    int depth = 0, max_depth = 0;
    for (int i = 0; i < n_instr; ++i) {
        int op = prog[i].op;
        if (op < JSM_OP_LEAF || op > JSM_OP_TANH) JSM_FAIL(JSM_INVALID_ARG, "%s: unknown op %d at %d", who, op, i);
        if (op == JSM_OP_LEAF) {
            if (prog[i].arg < 0 || prog[i].arg >= n_leaves) JSM_FAIL(JSM_INVALID_ARG, "%s: leaf index %d at %d", who, prog[i].arg, i);
            ++depth;
        } else if (op == JSM_OP_IMM) {
            ++depth;
        } else if (op >= JSM_OP_ADD && op <= JSM_OP_LT) {
            if (depth < 2) JSM_FAIL(JSM_INVALID_ARG, "%s: stack underflow at %d", who, i);
            --depth;
        } else if (depth < 1) {
            JSM_FAIL(JSM_INVALID_ARG, "%s: stack underflow at %d", who, i);
        }
        max_depth = depth > max_depth ? depth : max_depth;
        P.op[i] = (signed char)op;
        P.arg[i] = (signed char)prog[i].arg;
        P.imm[i] = prog[i].imm;
    }
    if (depth != 1) JSM_FAIL(JSM_INVALID_ARG, "%s: program leaves %d values on the stack", who, depth);
    if (max_depth > JSM_MAX_STACK) JSM_FAIL(JSM_UNSUPPORTED, "%s: stack depth %d > %d", who, max_depth, JSM_MAX_STACK);
    bool vec = (C % 4 == 0);
    for (int i = 0; i < n_leaves; ++i) {
        const jsm_mat& m = leaves[i];
        LeafDesc& L = P.leaf[i];
        L.p = m.data; L.rows = m.rows; L.cols = m.cols; L.rs = m.row_stride; L.cs = m.col_stride; L.dtype = m.dtype;
        const int esz = m.dtype == JSM_F32 ? 4 : 2;
        const int per16 = 16 / esz;  // a vector of four elements needs 16 (f32) or 8 (bf16) byte alignment
        (void)per16;
        const uintptr_t addr = reinterpret_cast<uintptr_t>(m.data);
        const int valign = 4 * esz;
        if (m.rows == 1 && m.cols == 1) L.kind = LK_SCALAR;
        else if (m.cols == 1 && m.rows == R) L.kind = LK_COLVEC;
        else if (m.rows == 1 && m.cols == C && m.col_stride == 1 && addr % valign == 0) L.kind = LK_ROWVEC;
        else if (m.rows == R && m.cols == C && m.col_stride == 1 && addr % valign == 0 && (m.row_stride * esz) % valign == 0)
            L.kind = LK_FULL;
        else L.kind = LK_GENERIC;
        if (L.kind == LK_GENERIC) vec = false;
    }
    P.pro = PRO_GENERIC;
    if (n_instr == 1 && prog[0].op == JSM_OP_LEAF) P.pro = PRO_LEAF;
    if (n_instr == 3 && prog[0].op == JSM_OP_LEAF && prog[1].op == JSM_OP_LEAF && prog[2].op == JSM_OP_ADD &&
        prog[0].arg == 0 && prog[1].arg == 1)
        P.pro = PRO_ADD;
    if (n_instr == 5 && prog[0].op == JSM_OP_LEAF && prog[1].op == JSM_OP_IMM && prog[2].op == JSM_OP_MUL &&
        prog[3].op == JSM_OP_LEAF && prog[4].op == JSM_OP_ADD && prog[0].arg == 0 && prog[3].arg == 1) {
        P.pro = PRO_AXPB;
        P.pro_imm = prog[1].imm;
    }
    Lw.R = R; Lw.C = C; Lw.depth = max_depth; Lw.vec = vec;
    return JSM_OK;
}

static jsm_status make_out(const jsm_mat& out, int rows, int cols, OutDesc& O, const char* who) {
    if (!out.data) JSM_FAIL(JSM_INVALID_ARG, "%s: null output", who);
    if (out.rows != rows || out.cols != cols)
        JSM_FAIL(JSM_SHAPE, "%s: output is %d x %d, result is %d x %d", who, out.rows, out.cols, rows, cols);
    O.p = out.data; O.rows = rows; O.cols = cols; O.rs = out.row_stride; O.cs = out.col_stride; O.dtype = out.dtype;
    const int esz = out.dtype == JSM_BF16 ? 2 : 4;
    O.vec = (out.col_stride == 1 && cols % 4 == 0 && reinterpret_cast<uintptr_t>(out.data) % (4 * esz) == 0 &&
             (out.row_stride * esz) % (4 * esz) == 0 && out.dtype != JSM_I32);
    return JSM_OK;
}

template <int GROUP, int VPT>
static void launch_rows(const Lowered& Lw, const RowsArgs& A, cudaStream_t st) {
    constexpr int RPC = 256 / GROUP;
    const int n_blocks = (A.R + RPC - 1) / RPC;
    // one CTA per row block: a fixed grid walking the blocks measured 5-8 % slower for the plain reductions (a CTA cannot
    // request its next row before it has finished the current one); the kernel keeps the loop for grids that are capped
    const unsigned grid = (unsigned)n_blocks;
    if (Lw.vec) {
        if (Lw.depth <= 4) rows_kernel<GROUP, VPT, 4, true><<<grid, 256, 0, st>>>(Lw.P, A, n_blocks);
        else rows_kernel<GROUP, VPT, 8, true><<<grid, 256, 0, st>>>(Lw.P, A, n_blocks);
    } else {
        if (Lw.depth <= 4) rows_kernel<GROUP, VPT, 4, false><<<grid, 256, 0, st>>>(Lw.P, A, n_blocks);
        else rows_kernel<GROUP, VPT, 8, false><<<grid, 256, 0, st>>>(Lw.P, A, n_blocks);
    }
}

template <int VPT, int KIND>
static cudaError_t launch_staged_pro(int pro, const StagedArgs& S, unsigned grid, size_t smem, cudaStream_t st) {
#define JSM_RS(PRO_)                                                                                                      \
    {                                                                                                                     \
        static bool configured[64] = {false};                                                                             \
        int dev = 0;                                                                                                      \
        cudaGetDevice(&dev);                                                                                              \
        if (dev >= 0 && dev < 64 && !configured[dev]) {                                                                   \
            cudaError_t e = cudaFuncSetAttribute(rows_staged_kernel<VPT, KIND, PRO_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return e;                                                                               \
            configured[dev] = true;                                                                                       \
        }                                                                                                                 \
        rows_staged_kernel<VPT, KIND, PRO_><<<grid, RS_THREADS, smem, st>>>(S);                                           \
        return cudaGetLastError();                                                                                        \
    }
    if (pro == PRO_LEAF) JSM_RS(PRO_LEAF)
    if (pro == PRO_AXPB) JSM_RS(PRO_AXPB)
    JSM_RS(PRO_ADD)
#undef JSM_RS
}
template <int VPT>
static cudaError_t launch_staged_kind(int kind, int pro, const StagedArgs& S, unsigned grid, size_t smem, cudaStream_t st) {
    switch (kind) {
        case JSM_ROWS_SUM: return launch_staged_pro<VPT, JSM_ROWS_SUM>(pro, S, grid, smem, st);
        case JSM_ROWS_MEAN: return launch_staged_pro<VPT, JSM_ROWS_MEAN>(pro, S, grid, smem, st);
        case JSM_ROWS_MAX: return launch_staged_pro<VPT, JSM_ROWS_MAX>(pro, S, grid, smem, st);
        case JSM_ROWS_SOFTMAX: return launch_staged_pro<VPT, JSM_ROWS_SOFTMAX>(pro, S, grid, smem, st);
        case JSM_ROWS_LAYERNORM: return launch_staged_pro<VPT, JSM_ROWS_LAYERNORM>(pro, S, grid, smem, st);
        default: return launch_staged_pro<VPT, JSM_ROWS_RMSNORM>(pro, S, grid, smem, st);
    }
}

// Rows staged through shared memory: f32 operands with contiguous, 16-byte aligned rows of 1024, 2048 or 4096 columns,
// the programs x, x * imm + y and x + y, every kind but argmax.  Returns false when the call does not qualify.
static bool try_rows_staged(const Lowered& Lw, const RowsArgs& A, cudaStream_t st, cudaError_t* err) {
    const EvalParams& P = Lw.P;
    const int C = Lw.C;
    if (!Lw.vec || A.kind == JSM_ROWS_ARGMAX) return false;
    if (C != 1024 && C != 2048 && C != 4096) return false;
    if (P.pro != PRO_LEAF && P.pro != PRO_AXPB && P.pro != PRO_ADD) return false;
    const int nl = P.pro == PRO_LEAF ? 1 : 2;
    if (P.n_leaves < nl) return false;
    for (int i = 0; i < nl; ++i)
        if (P.leaf[i].kind != LK_FULL || P.leaf[i].dtype != JSM_F32) return false;
    if (A.out.dtype != JSM_F32) return false;
    const bool reduces = A.kind <= JSM_ROWS_ARGMAX;
    if (!reduces && !A.out.vec) return false;
    if ((A.gain && reinterpret_cast<uintptr_t>(A.gain) % 16) || (A.bias && reinterpret_cast<uintptr_t>(A.bias) % 16)) return false;
    StagedArgs S;
    S.a = reinterpret_cast<const float*>(P.leaf[0].p);
    S.rsa = P.leaf[0].rs;
    S.b = nl == 2 ? reinterpret_cast<const float*>(P.leaf[1].p) : nullptr;
    S.rsb = nl == 2 ? P.leaf[1].rs : 0;
    S.imm = P.pro_imm;
    S.R = A.R;
    S.gain = A.gain;
    S.bias = A.bias;
    S.eps = A.eps;
    S.out = reinterpret_cast<float*>(A.out.p);
    S.rso = A.out.rs;
    S.err = tc_error_word();
    const size_t stage_bytes = (size_t)nl * C * 4;
    int n_stages = (int)(96 * 1024 / stage_bytes);
    if (n_stages > 8) n_stages = 8;
    if (reduces) {
        // a warp per row: warp w must meet stage w in every phase (a parity wait tells consecutive phases apart only),
        // so the ring has exactly as many stages as consumer warps
        n_stages = 8;
        if (8 * stage_bytes > 200 * 1024) return false;
    }
    S.n_stages = n_stages;
    unsigned grid = (unsigned)((n_stages * stage_bytes > 100 * 1024 ? 1 : 2) * sm_count());
    if ((int)grid > A.R) grid = (unsigned)A.R;
    const size_t smem = (size_t)n_stages * stage_bytes;
    if (C == 1024) *err = launch_staged_kind<1>(A.kind, P.pro, S, grid, smem, st);
    else if (C == 2048) *err = launch_staged_kind<2>(A.kind, P.pro, S, grid, smem, st);
    else *err = launch_staged_kind<4>(A.kind, P.pro, S, grid, smem, st);
    return true;
}

}  // namespace jsm

using namespace jsm;

extern "C" {

jsm_status jsm_eval_elementwise(const jsm_instr* prog, int n_instr, const jsm_mat* leaves, int n_leaves, jsm_mat out,
                                void* stream) {
    Lowered Lw;
    jsm_status s = lower(prog, n_instr, leaves, n_leaves, Lw, "jsm_eval_elementwise");
    if (s != JSM_OK) return s;
    OutDesc O;
    s = make_out(out, Lw.R, Lw.C, O, "jsm_eval_elementwise");
    if (s != JSM_OK) return s;
    if (out.dtype == JSM_I32) JSM_FAIL(JSM_UNSUPPORTED, "jsm_eval_elementwise: integer output");
    const bool vec = Lw.vec && O.vec;
    const long long work = vec ? (long long)Lw.R * Lw.C / 4 : (long long)Lw.R * Lw.C;
    long long blocks = (work + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaStream_t st = as_stream(stream);
    // two contiguous f32 operands of the output's shape, x * imm + y or x + y: the batched-load kernel
    const EvalParams& P = Lw.P;
    if (vec && (P.pro == PRO_AXPB || P.pro == PRO_ADD) && P.n_leaves >= 2 && out.dtype == JSM_F32 && O.rs == Lw.C &&
        P.leaf[0].kind == LK_FULL && P.leaf[1].kind == LK_FULL && P.leaf[0].dtype == JSM_F32 && P.leaf[1].dtype == JSM_F32 &&
        P.leaf[0].rs == Lw.C && P.leaf[1].rs == Lw.C) {
        const long long n_vec = (long long)Lw.R * Lw.C / 4;
        long long fb = (n_vec + 1023) / 1024;
        if (fb > (long long)sm_count() * 8) fb = (long long)sm_count() * 8;
        if (fb < 1) fb = 1;
        const float4* pa = reinterpret_cast<const float4*>(P.leaf[0].p);
        const float4* pb = reinterpret_cast<const float4*>(P.leaf[1].p);
        if (P.pro == PRO_AXPB) elementwise_fast_kernel<PRO_AXPB><<<(unsigned)fb, 256, 0, st>>>(pa, pb, P.pro_imm, reinterpret_cast<float4*>(O.p), n_vec);
        else elementwise_fast_kernel<PRO_ADD><<<(unsigned)fb, 256, 0, st>>>(pa, pb, 0.0f, reinterpret_cast<float4*>(O.p), n_vec);
        JSM_LAUNCH_CHECK();
        return JSM_OK;
    }
    if (vec) {
        if (Lw.depth <= 4) elementwise_kernel<4, true><<<(unsigned)blocks, 256, 0, st>>>(Lw.P, O);
        else elementwise_kernel<8, true><<<(unsigned)blocks, 256, 0, st>>>(Lw.P, O);
    } else {
        if (Lw.depth <= 4) elementwise_kernel<4, false><<<(unsigned)blocks, 256, 0, st>>>(Lw.P, O);
        else elementwise_kernel<8, false><<<(unsigned)blocks, 256, 0, st>>>(Lw.P, O);
    }
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

jsm_status jsm_eval_rows(int kind, int axis, const jsm_instr* prog, int n_instr, const jsm_mat* leaves, int n_leaves,
                         const float* d_gain, const float* d_bias, float eps, jsm_mat out, void* stream) {
    if (kind < JSM_ROWS_SUM || kind > JSM_ROWS_RMSNORM) JSM_FAIL(JSM_INVALID_ARG, "jsm_eval_rows: kind %d", kind);
    if (axis != 0 && axis != 1) JSM_FAIL(JSM_INVALID_ARG, "jsm_eval_rows: axis %d", axis);
    Lowered Lw;
    jsm_status s = lower(prog, n_instr, leaves, n_leaves, Lw, "jsm_eval_rows");
    if (s != JSM_OK) return s;
    const bool reduces = kind <= JSM_ROWS_ARGMAX;
    OutDesc O;
    const int orow = reduces ? (axis == 1 ? Lw.R : 1) : Lw.R;
    const int ocol = reduces ? (axis == 1 ? 1 : Lw.C) : Lw.C;
    s = make_out(out, orow, ocol, O, "jsm_eval_rows");
    if (s != JSM_OK) return s;
    if ((out.dtype == JSM_I32) != (kind == JSM_ROWS_ARGMAX) && out.dtype == JSM_I32)
        JSM_FAIL(JSM_UNSUPPORTED, "jsm_eval_rows: integer output only for argmax");
    RowsArgs A;
    A.kind = kind; A.R = Lw.R; A.C = Lw.C; A.gain = d_gain; A.bias = d_bias; A.eps = eps; A.out = O;
    cudaStream_t st = as_stream(stream);
    const int C = Lw.C;
    cudaError_t staged_err = cudaSuccess;
    if (axis == 1 && try_rows_staged(Lw, A, st, &staged_err)) {
        if (staged_err != cudaSuccess) JSM_FAIL(JSM_CUDA, "jsm_eval_rows: launch failed: %s", cudaGetErrorString(staged_err));
        g_launches.fetch_add(1);
        return JSM_OK;
    }
    if (axis == 1 && C <= 8192) {
        if (C <= 128) launch_rows<32, 1>(Lw, A, st);
        else if (C <= 256) launch_rows<32, 2>(Lw, A, st);
        else if (C <= 512) launch_rows<32, 4>(Lw, A, st);
        else if (C <= 1024) launch_rows<256, 1>(Lw, A, st);
        else if (C <= 2048) launch_rows<256, 2>(Lw, A, st);
        else if (C <= 4096) launch_rows<256, 4>(Lw, A, st);  // fewer threads per row (128 x 8, 64 x 16 values) measured 25-60 % slower
        else launch_rows<256, 8>(Lw, A, st);
    } else {
        const unsigned lines = (unsigned)(axis == 1 ? Lw.R : Lw.C);
        if (Lw.depth <= 4) lines_kernel<4><<<lines, 256, 0, st>>>(Lw.P, A, axis);
        else lines_kernel<8><<<lines, 256, 0, st>>>(Lw.P, A, axis);
    }
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

jsm_status jsm_eval_full(int kind, const jsm_instr* prog, int n_instr, const jsm_mat* leaves, int n_leaves, jsm_mat out,
                         void* stream) {
    if (kind != JSM_ROWS_SUM && kind != JSM_ROWS_MAX && kind != JSM_ROWS_MEAN && kind != JSM_ROWS_SOFTMAX)
        JSM_FAIL(JSM_INVALID_ARG, "jsm_eval_full: kind %d", kind);
    Lowered Lw;
    jsm_status s = lower(prog, n_instr, leaves, n_leaves, Lw, "jsm_eval_full");
    if (s != JSM_OK) return s;
    OutDesc O;
    if (kind == JSM_ROWS_SOFTMAX) s = make_out(out, Lw.R, Lw.C, O, "jsm_eval_full");
    else s = make_out(out, 1, 1, O, "jsm_eval_full");
    if (s != JSM_OK) return s;
    if (out.dtype != JSM_F32 && kind != JSM_ROWS_SOFTMAX) JSM_FAIL(JSM_UNSUPPORTED, "jsm_eval_full: scalar result must be f32");
    cudaStream_t st = as_stream(stream);
    const long long total = (long long)Lw.R * Lw.C;
    int nblk = (int)((total + 4095) / 4096);
    const int cap = sm_count() * 4;
    if (nblk > cap) nblk = cap;
    if (nblk < 1) nblk = 1;
    float* scratch = nullptr;  // [nblk] partials + max + sum, stream-ordered allocation
    JSM_CUDA_CHECK(cudaMallocAsync(reinterpret_cast<void**>(&scratch), sizeof(float) * (nblk + 2), st));
    float* d_max = scratch + nblk;
    float* d_sum = scratch + nblk + 1;
    auto partial = [&](int mode, const float* shift) {
        if (Lw.depth <= 4) full_partial_kernel<4><<<nblk, 256, 0, st>>>(Lw.P, Lw.R, Lw.C, mode, shift, scratch);
        else full_partial_kernel<8><<<nblk, 256, 0, st>>>(Lw.P, Lw.R, Lw.C, mode, shift, scratch);
        g_launches.fetch_add(1);
    };
    if (kind == JSM_ROWS_SOFTMAX) {
        partial(1, nullptr);
        full_fold_kernel<<<1, 256, 0, st>>>(scratch, nblk, 1, 0.0f, d_max);
        partial(2, d_max);
        full_fold_kernel<<<1, 256, 0, st>>>(scratch, nblk, 0, 0.0f, d_sum);
        long long blocks = (total + 255) / 256;
        if (blocks > (long long)sm_count() * 8) blocks = (long long)sm_count() * 8;
        if (Lw.depth <= 4) full_softmax_write_kernel<4><<<(unsigned)blocks, 256, 0, st>>>(Lw.P, O, d_max, d_sum);
        else full_softmax_write_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(Lw.P, O, d_max, d_sum);
        g_launches.fetch_add(3);
    } else {
        const int mode = kind == JSM_ROWS_MAX ? 1 : 0;
        partial(mode, nullptr);
        full_fold_kernel<<<1, 256, 0, st>>>(scratch, nblk, mode, kind == JSM_ROWS_MEAN ? (float)total : 0.0f,
                                            reinterpret_cast<float*>(out.data));
        g_launches.fetch_add(1);
    }
    cudaError_t e = cudaGetLastError();
    cudaFreeAsync(scratch, st);
    if (e != cudaSuccess) JSM_FAIL(JSM_CUDA, "jsm_eval_full: launch failed: %s", cudaGetErrorString(e));
    return JSM_OK;
}

}  // extern "C"
