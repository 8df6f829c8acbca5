// CUDA-core attention with fp32 arithmetic throughout: the reference-exact path
// of mat_head_gen_t::forward (mat_mha_t.hpp:45-74) for fp32 models, and the
// general fallback shape coverage (any head_dim <= 128, any lengths, GQA).
// One warp owns one query row; a CTA of 8 warps shares K/V tiles of 32 keys
// staged in shared memory.  Scores are the k-ascending dot product of the
// reference (separately rounded multiply and add), divided by sqrt(D) in double
// and narrowed to float as the reference does (:53 and mat_net_t.hpp:273-279);
// the softmax is computed online across tiles.
#include "common.cuh"
#include "attn.cuh"
#include <math.h>

namespace jsm {

constexpr int AQ = 8;    // queries (warps) per CTA
constexpr int AK = 32;   // keys per tile
constexpr int AD = 128;  // largest head_dim

template <typename T>
__device__ __forceinline__ float2 load_pair(const T* p) {
    if constexpr (sizeof(T) == 4) {
        return *reinterpret_cast<const float2*>(p);
    } else {
        uint32_t w = *reinterpret_cast<const uint32_t*>(p);
        return make_float2(bf16lo(w), bf16hi(w));
    }
}
__device__ __forceinline__ float2 rotate(float2 x, float4 e) {
    return make_float2(__fadd_rn(__fmul_rn(e.x, x.x), __fmul_rn(-e.w, x.y)), __fadd_rn(__fmul_rn(e.y, x.x), __fmul_rn(e.z, x.y)));
}

template <typename T>
__global__ void __launch_bounds__(AQ * 32) attn_simt_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                           const T* __restrict__ v, T* __restrict__ out, int Tq, int Tk,
                                                           int Hq, int Hkv, int D, int causal, float scale, int exact_div,
                                                           const float4* __restrict__ rope, long long q_rs, long long kv_rs,
                                                           long long o_rs, int pos0) {
    __shared__ float Ks[AK][AD + 1];
    __shared__ float Vs[AK][AD + 1];
    __shared__ float Qs[AQ][AD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (Hq / Hkv);
    const int q0 = blockIdx.x * AQ;
    const int shift = Tk - Tq;  // query i sits at position i + shift
    const int half = D / 2;

    // stage the CTA's queries (rotated when a rope table is given)
    for (int e = threadIdx.x; e < AQ * half; e += AQ * 32) {
        const int qi = e / half, pr = e % half;
        float2 x = make_float2(0.0f, 0.0f);
        if (q0 + qi < Tq) {
            x = load_pair(q + (long long)(b * Tq + q0 + qi) * q_rs + (long long)h * D + 2 * pr);
            if (rope) x = rotate(x, rope[(long long)(pos0 + q0 + qi + shift) * half + pr]);
        }
        Qs[qi][2 * pr] = x.x;
        Qs[qi][2 * pr + 1] = x.y;
    }
    const int qi = q0 + warp;
    const bool q_ok = qi < Tq;
    float m = -INFINITY, l = 0.0f, o[AD / 32];
#pragma unroll
    for (int r = 0; r < AD / 32; ++r) o[r] = 0.0f;
    const int last_q = min(q0 + AQ, Tq) - 1;
    const int k_end = causal ? min(Tk, last_q + shift + 1) : Tk;
    const double root = sqrt((double)D);

    for (int k0 = 0; k0 < k_end; k0 += AK) {
        __syncthreads();
        for (int e = threadIdx.x; e < AK * half; e += AQ * 32) {
            const int kj = e / half, pr = e % half;
            float2 kk = make_float2(0.0f, 0.0f), vv = make_float2(0.0f, 0.0f);
            if (k0 + kj < Tk) {
                const long long base = (long long)(b * Tk + k0 + kj) * kv_rs + (long long)hk * D + 2 * pr;
                kk = load_pair(k + base);
                vv = load_pair(v + base);
                if (rope) kk = rotate(kk, rope[(long long)(pos0 + k0 + kj) * half + pr]);
            }
            Ks[kj][2 * pr] = kk.x; Ks[kj][2 * pr + 1] = kk.y;
            Vs[kj][2 * pr] = vv.x; Vs[kj][2 * pr + 1] = vv.y;
        }
        __syncthreads();
        if (!q_ok) continue;
        const int j = k0 + lane;
        float s = 0.0f;
        for (int d = 0; d < D; ++d) s = __fadd_rn(s, __fmul_rn(Qs[warp][d], Ks[lane][d]));
        s = exact_div ? (float)((double)s / root) : s * scale;
        if (j >= Tk || (causal && j > qi + shift)) s = -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;  // nothing visible yet
        const float p = expf(s - m_new);
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < AD / 32; ++r) o[r] *= corr;
        for (int jj = 0; jj < AK; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
            for (int r = 0; r < AD / 32; ++r)
                if (lane + 32 * r < D) o[r] += pj * Vs[jj][lane + 32 * r];
        }
    }
    if (!q_ok) return;
    T* dst = out + (long long)(b * Tq + qi) * o_rs + (long long)h * D;
#pragma unroll
    for (int r = 0; r < AD / 32; ++r) {
        const int d = lane + 32 * r;
        if (d < D) {
            const float val = o[r] / l;
            if constexpr (sizeof(T) == 4) dst[d] = val; else dst[d] = __float2bfloat16_rn(val);
        }
    }
}

jsm_status attn_simt_launch(const void* q, const void* k, const void* v, void* out, jsm_dtype dtype, int batch, int Tq, int Tk,
                            int Hq, int Hkv, int D, int causal, float scale, const float* rope, cudaStream_t st, long long q_rs,
                            long long kv_rs, long long o_rs, int pos0) {
    if (q_rs <= 0) q_rs = (long long)Hq * D;
    if (kv_rs <= 0) kv_rs = (long long)Hkv * D;
    if (o_rs <= 0) o_rs = (long long)Hq * D;
    const float rs = 1.0f / sqrtf((float)D);
    const int exact_div = fabsf(scale - rs) <= 1e-7f * rs ? 1 : 0;
    dim3 grid((Tq + AQ - 1) / AQ, Hq, batch);
    if (dtype == JSM_F32)
        attn_simt_kernel<float><<<grid, AQ * 32, 0, st>>>((const float*)q, (const float*)k, (const float*)v, (float*)out, Tq, Tk,
                                                         Hq, Hkv, D, causal, scale, exact_div, (const float4*)rope, q_rs, kv_rs, o_rs, pos0);
    else
        attn_simt_kernel<__nv_bfloat16><<<grid, AQ * 32, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                                                 (const __nv_bfloat16*)v, (__nv_bfloat16*)out, Tq, Tk, Hq,
                                                                 Hkv, D, causal, scale, exact_div, (const float4*)rope, q_rs, kv_rs, o_rs, pos0);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

}  // namespace jsm
