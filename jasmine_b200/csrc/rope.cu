// Table-driven rotary position embedding.
// The table holds, per (position m, pair i), (cos A, sin A, cos B, sin B) and the
// rotation is out0 = cosA*x0 - sinB*x1, out1 = sinA*x0 + cosB*x1: the 2x2 block
// product of RoPE_net_t::forward (mat_RoPE_t.hpp:166-188) with the table of
// mat_RoPE_t::init (:99-134).  In the reference's table the block of position m
// uses column 2m for its first column and 2m+1 for its second, i.e. A and B are
// two different angles; "standard" mode sets A = B = m / theta^(2i/d).
// The table is computed on the host with the reference's roundings (double pow,
// double quotient narrowed to float, float cos/sin) and uploaded.
#include "common.cuh"
#include "attn.cuh"
#include <cmath>
#include <vector>

namespace jsm {

template <typename T>
__global__ void rope_apply_kernel(const T* __restrict__ x, T* __restrict__ out, const float4* __restrict__ table, int d,
                                  int n_heads, const int32_t* __restrict__ positions, int T_tokens, long long row_stride) {
    const int half = d / 2;
    const long long total = (long long)T_tokens * n_heads * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int pair = (int)(i % half);
        const long long th = i / half;  // token * n_heads + head
        const int t = (int)(th / n_heads);
        const int m = positions ? positions[t] : t;
        const float4 e = table[(long long)m * half + pair];
        const long long base = (long long)t * row_stride + (long long)(th % n_heads) * d + 2 * pair;
        float x0, x1;
        if constexpr (sizeof(T) == 4) {
            float2 v = *reinterpret_cast<const float2*>(x + base);
            x0 = v.x; x1 = v.y;
        } else {
            uint32_t w = *reinterpret_cast<const uint32_t*>(x + base);
            x0 = bf16lo(w); x1 = bf16hi(w);
        }
        // (0 + cosA*x0) + (-sinB)*x1 and (0 + sinA*x0) + cosB*x1, each product rounded on its own
        const float o0 = __fadd_rn(__fmul_rn(e.x, x0), __fmul_rn(-e.w, x1));
        const float o1 = __fadd_rn(__fmul_rn(e.y, x0), __fmul_rn(e.z, x1));
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float2*>(out + base) = make_float2(o0, o1);
        } else {
            *reinterpret_cast<uint32_t*>(out + base) = pack_bf16x2(o0, o1);
        }
    }
}

// bf16, 128-bit path: a thread rotates four pairs (8 elements, 16 bytes) with four consecutive table entries; same
// arithmetic (each product rounded on its own) as the scalar kernel
__global__ void __launch_bounds__(256) rope_apply_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                  const float4* __restrict__ table, int d, int n_heads,
                                                                  const int32_t* __restrict__ positions, int T_tokens,
                                                                  long long row_stride) {
    const int quads = d / 8;  // groups of four pairs per head
    const long long total = (long long)T_tokens * n_heads * quads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int qd = (int)(i % quads);
        const long long th = i / quads;
        const int t = (int)(th / n_heads);
        const int m = positions ? positions[t] : t;
        const float4* e = table + (long long)m * (d / 2) + qd * 4;
        const long long base = (long long)t * row_stride + (long long)(th % n_heads) * d + 8 * qd;
        const uint4 w = *reinterpret_cast<const uint4*>(x + base);
        const uint32_t in[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float4 c = e[p];
            const float x0 = bf16lo(in[p]), x1 = bf16hi(in[p]);
            o[p] = pack_bf16x2(__fadd_rn(__fmul_rn(c.x, x0), __fmul_rn(-c.w, x1)), __fadd_rn(__fmul_rn(c.y, x0), __fmul_rn(c.z, x1)));
        }
        *reinterpret_cast<uint4*>(out + base) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// The same for many heads per token: a thread keeps the four table entries of its group of pairs and walks the heads,
// so the table (16 bytes per pair, four times the bytes of the bf16 data it rotates) is read once per token instead of
// once per head.  Block = 16 groups of pairs x 16 head lanes (d = 128); one token per loop step.
__global__ void __launch_bounds__(256) rope_apply_bf16_heads_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                    const float4* __restrict__ table, int n_heads,
                                                                    const int32_t* __restrict__ positions, int T_tokens,
                                                                    long long row_stride) {
    constexpr int D = 128;
    const int qd = threadIdx.x & 15, hl = threadIdx.x >> 4;
    for (int t = blockIdx.x; t < T_tokens; t += gridDim.x) {
        const int m = positions ? positions[t] : t;
        const float4* e = table + (long long)m * (D / 2) + qd * 4;
        const float4 c0 = e[0], c1 = e[1], c2 = e[2], c3 = e[3];
        const float4 c[4] = {c0, c1, c2, c3};
        for (int h0 = hl; h0 < n_heads; h0 += 64) {
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int h = h0 + 16 * u;
                if (h < n_heads) w[u] = __ldcs(reinterpret_cast<const uint4*>(x + (long long)t * row_stride + (long long)h * D + 8 * qd));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int h = h0 + 16 * u;
                if (h >= n_heads) break;
                const uint32_t in[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
                uint32_t o[4];
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float x0 = bf16lo(in[p]), x1 = bf16hi(in[p]);
                    o[p] = pack_bf16x2(__fadd_rn(__fmul_rn(c[p].x, x0), __fmul_rn(-c[p].w, x1)),
                                       __fadd_rn(__fmul_rn(c[p].y, x0), __fmul_rn(c[p].z, x1)));
                }
                *reinterpret_cast<uint4*>(out + (long long)t * row_stride + (long long)h * D + 8 * qd) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

// Queries and keys of a prefill in ONE launch (two tensors, the same positions): a thread issues the loads of all its
// heads of both tensors before the first rotation (four 16-byte loads in flight per thread at 32 + 32 heads instead of
// two), and the table entries of the next token are requested before the current token is rotated.
__global__ void __launch_bounds__(256) rope_apply_bf16_qk_kernel(const __nv_bfloat16* __restrict__ xq, __nv_bfloat16* __restrict__ oq, int Hq,
                                                                 const __nv_bfloat16* __restrict__ xk, __nv_bfloat16* __restrict__ ok, int Hk,
                                                                 const float4* __restrict__ table, const int32_t* __restrict__ positions,
                                                                 int T_tokens) {
    constexpr int D = 128, MAXU = 8;  // up to 64 + 64 heads
    const int qd = threadIdx.x & 15, hl = threadIdx.x >> 4;
    const int nq = (Hq - hl + 15) / 16, nk = (Hk - hl + 15) / 16;  // heads of this lane in q and in k
    int t = blockIdx.x;
    if (t >= T_tokens) return;
    float4 c[4];
    {
        const int m = positions ? positions[t] : t;
        const float4* e = table + (long long)m * (D / 2) + qd * 4;
#pragma unroll
        for (int p = 0; p < 4; ++p) c[p] = e[p];
    }
    while (t < T_tokens) {
        const int t_next = t + gridDim.x;
        uint4 w[MAXU];
#pragma unroll
        for (int u = 0; u < MAXU; ++u) {
            if (u < nq) w[u] = __ldcs(reinterpret_cast<const uint4*>(xq + ((long long)t * Hq + hl + 16 * u) * D + 8 * qd));
            else if (u - nq < nk) w[u] = __ldcs(reinterpret_cast<const uint4*>(xk + ((long long)t * Hk + hl + 16 * (u - nq)) * D + 8 * qd));
        }
        float4 cn[4];
        if (t_next < T_tokens) {
            const int m = positions ? positions[t_next] : t_next;
            const float4* e = table + (long long)m * (D / 2) + qd * 4;
#pragma unroll
            for (int p = 0; p < 4; ++p) cn[p] = e[p];
        }
#pragma unroll
        for (int u = 0; u < MAXU; ++u) {
            if (u >= nq + nk) break;
            const uint32_t in[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float x0 = bf16lo(in[p]), x1 = bf16hi(in[p]);
                o[p] = pack_bf16x2(__fadd_rn(__fmul_rn(c[p].x, x0), __fmul_rn(-c[p].w, x1)),
                                   __fadd_rn(__fmul_rn(c[p].y, x0), __fmul_rn(c[p].z, x1)));
            }
            __nv_bfloat16* dst = u < nq ? oq + ((long long)t * Hq + hl + 16 * u) * D + 8 * qd : ok + ((long long)t * Hk + hl + 16 * (u - nq)) * D + 8 * qd;
            __stcs(reinterpret_cast<uint4*>(dst), make_uint4(o[0], o[1], o[2], o[3]));
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) c[p] = cn[p];
        t = t_next;
    }
}

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_rope_apply_qk(const void* d_q, void* d_q_out, int Hq, const void* d_k, void* d_k_out, int Hkv, jsm_dtype dtype,
                                        const float* d_table, int d, const int32_t* d_positions, int T, void* stream) {
    if (T == 0) return JSM_OK;
    if (!d_q || !d_q_out || !d_k || !d_k_out || !d_table) JSM_FAIL(JSM_INVALID_ARG, "jsm_rope_apply_qk: null pointer");
    const bool aligned = !((reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_q_out) | reinterpret_cast<uintptr_t>(d_k) |
                            reinterpret_cast<uintptr_t>(d_k_out)) & 15);
    if (dtype == JSM_BF16 && d == 128 && aligned && Hq > 0 && Hkv > 0 && (Hq + 15) / 16 + (Hkv + 15) / 16 <= 8 && T >= 64) {
        const unsigned grid = (unsigned)(T < sm_count() * 8 ? T : sm_count() * 8);
        rope_apply_bf16_qk_kernel<<<grid, 256, 0, as_stream(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(d_q), reinterpret_cast<__nv_bfloat16*>(d_q_out), Hq,
                                                                       reinterpret_cast<const __nv_bfloat16*>(d_k), reinterpret_cast<__nv_bfloat16*>(d_k_out), Hkv,
                                                                       reinterpret_cast<const float4*>(d_table), d_positions, T);
        JSM_LAUNCH_CHECK();
        return JSM_OK;
    }
    jsm_status s = jsm_rope_apply(d_q, d_q_out, dtype, d_table, d, Hq, d_positions, T, stream);
    if (s != JSM_OK) return s;
    return jsm_rope_apply(d_k, d_k_out, dtype, d_table, d, Hkv, d_positions, T, stream);
}

extern "C" jsm_status jsm_rope_table(float* d_table, int mode, int d, float theta, int max_pos, void* stream) {
    if (!d_table) JSM_FAIL(JSM_INVALID_ARG, "jsm_rope_table: null table");
    if (d <= 0 || d % 2 || max_pos <= 0 || (mode != 0 && mode != 1))
        JSM_FAIL(JSM_INVALID_ARG, "jsm_rope_table: d %d, max_pos %d, mode %d", d, max_pos, mode);
    const int half = d / 2;
    std::vector<float> h((size_t)max_pos * half * 4);
    std::vector<double> p(half);
    for (int i = 0; i < half; ++i)
        p[i] = std::pow((double)theta, (double)((mode == 0 ? (float)i : (float)(2 * i)) / (float)d));
    for (int m = 0; m < max_pos; ++m)
        for (int i = 0; i < half; ++i) {
            float a, b;
            if (mode == 0) {
                a = (float)((2 * m) / p[i]);
                b = (float)((2 * m + 1) / p[i]);
            } else {
                a = b = (float)(m / p[i]);
            }
            float* e = &h[((size_t)m * half + i) * 4];
            e[0] = std::cos(a); e[1] = std::sin(a); e[2] = std::cos(b); e[3] = std::sin(b);
        }
    JSM_CUDA_CHECK(cudaMemcpyAsync(d_table, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice, as_stream(stream)));
    JSM_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream)));
    return JSM_OK;
}

extern "C" jsm_status jsm_rope_apply(const void* d_x, void* d_out, jsm_dtype dtype, const float* d_table, int d, int n_heads,
                                     const int32_t* d_positions, int T, void* stream) {
    return jsm::rope_apply_strided(d_x, d_out, dtype, d_table, d, n_heads, d_positions, T, (long long)n_heads * d, stream);
}

// rows of `row_stride` elements whose first n_heads * d entries are rotated (in place when d_out == d_x)
jsm_status jsm::rope_apply_strided(const void* d_x, void* d_out, jsm_dtype dtype, const float* d_table, int d, int n_heads,
                                   const int32_t* d_positions, int T, long long row_stride, void* stream) {
    if (T == 0) return JSM_OK;
    if (!d_x || !d_out || !d_table) JSM_FAIL(JSM_INVALID_ARG, "jsm_rope_apply: null pointer");
    if (d <= 0 || d % 2 || n_heads <= 0 || T < 0) JSM_FAIL(JSM_SHAPE, "Input dimension does not match RoPE dimension (d %d)", d);
    if (dtype != JSM_F32 && dtype != JSM_BF16) JSM_FAIL(JSM_UNSUPPORTED, "jsm_rope_apply: dtype %d", (int)dtype);
    const long long total = (long long)T * n_heads * (d / 2);
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 8) blocks = (long long)sm_count() * 8;
    const bool vec = dtype == JSM_BF16 && d % 8 == 0 && row_stride % 8 == 0 && !(reinterpret_cast<uintptr_t>(d_x) & 15) &&
                     !(reinterpret_cast<uintptr_t>(d_out) & 15);
    if (vec && d == 128 && n_heads >= 4 && T >= 64) {
        unsigned hb = (unsigned)(T < sm_count() * 16 ? T : sm_count() * 16);
        rope_apply_bf16_heads_kernel<<<hb, 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const __nv_bfloat16*>(d_x), reinterpret_cast<__nv_bfloat16*>(d_out),
            reinterpret_cast<const float4*>(d_table), n_heads, d_positions, T, row_stride);
    } else if (vec) {
        const long long work = (long long)T * n_heads * (d / 8);
        long long vb = (work + 255) / 256;
        if (vb > (long long)sm_count() * 16) vb = (long long)sm_count() * 16;
        rope_apply_bf16_vec_kernel<<<(unsigned)vb, 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const __nv_bfloat16*>(d_x), reinterpret_cast<__nv_bfloat16*>(d_out),
            reinterpret_cast<const float4*>(d_table), d, n_heads, d_positions, T, row_stride);
    } else if (dtype == JSM_F32)
        rope_apply_kernel<float><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const float*>(d_x), reinterpret_cast<float*>(d_out), reinterpret_cast<const float4*>(d_table), d,
            n_heads, d_positions, T, row_stride);
    else
        rope_apply_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const __nv_bfloat16*>(d_x), reinterpret_cast<__nv_bfloat16*>(d_out),
            reinterpret_cast<const float4*>(d_table), d, n_heads, d_positions, T, row_stride);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}
