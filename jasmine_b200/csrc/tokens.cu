// Token-level kernels of the decoder: embedding gather, fused residual-add + norm.
// None of these exist in the reference (its inputs are real-valued matrices); the
// norm follows the formula of layer_norm_net_t::forward (mat_net_t.hpp:209-225)
// with eps under the square root, RMSNorm drops the mean.
#include "common.cuh"
#include <math.h>

namespace jsm {

template <typename T>
struct VecIO;
template <>
struct VecIO<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[4]) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ static void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <>
struct VecIO<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 t = *reinterpret_cast<const uint4*>(p);
        v[0] = bf16lo(t.x); v[1] = bf16hi(t.x); v[2] = bf16lo(t.y); v[3] = bf16hi(t.y);
        v[4] = bf16lo(t.z); v[5] = bf16hi(t.z); v[6] = bf16lo(t.w); v[7] = bf16hi(t.w);
    }
    __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 t;
        t.x = pack_bf16x2(v[0], v[1]); t.y = pack_bf16x2(v[2], v[3]);
        t.z = pack_bf16x2(v[4], v[5]); t.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(p) = t;
    }
};

template <typename T>
__global__ void __launch_bounds__(256) embedding_kernel(const T* __restrict__ table, const T* __restrict__ pos_table,
                                                        const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                                                        T* __restrict__ out, int d) {
    constexpr int N = VecIO<T>::N;
    chain_trigger();
    chain_wait();
    const int t = blockIdx.x;
    const long long row = ids[t];
    const long long prow = pos_table ? (positions ? positions[t] : t) : 0;
    for (int c = threadIdx.x * N; c < d; c += 256 * N) {
        float a[N];
        VecIO<T>::load(table + row * d + c, a);
        if (pos_table) {
            float p[N];
            VecIO<T>::load(pos_table + prow * d + c, p);
#pragma unroll
            for (int i = 0; i < N; ++i) a[i] = a[i] + p[i];
        }
        VecIO<T>::store(out + (long long)t * d + c, a);
    }
}

__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += smem[w];
    return s;
}

// one CTA per token; the token's features stay in registers between the statistics and the write
template <typename T, int MAXV>
__global__ void __launch_bounds__(256) add_norm_kernel(int kind, const T* __restrict__ h, const T* __restrict__ delta,
                                                       T* __restrict__ h_out, T* __restrict__ y, const float* __restrict__ gain,
                                                       const float* __restrict__ bias, float eps, int d) {
    __shared__ float smem[8];
    constexpr int N = VecIO<T>::N;
    const long long base = (long long)blockIdx.x * d;
    float v[MAXV][N];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = (i * 256 + threadIdx.x) * N;
        if (c < d) {
            VecIO<T>::load(h + base + c, v[i]);
            if (delta) {
                float e[N];
                VecIO<T>::load(delta + base + c, e);
#pragma unroll
                for (int j = 0; j < N; ++j) v[i][j] = v[i][j] + e[j];
                if (sizeof(T) == 2) {  // the residual stream is stored in bf16: normalise what is stored
#pragma unroll
                    for (int j = 0; j < N; ++j) v[i][j] = bf16_bits_to_f32(f32_to_bf16_bits(v[i][j]));
                }
            }
            if (h_out) VecIO<T>::store(h_out + base + c, v[i]);
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j) v[i][j] = 0.0f;
        }
    }
    float mean = 0.0f;
    if (kind == JSM_ROWS_LAYERNORM) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i)
#pragma unroll
            for (int j = 0; j < N; ++j) s += v[i][j];
        mean = block_sum(s, smem) / (float)d;
    }
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = (i * 256 + threadIdx.x) * N;
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float dd = v[i][j] - mean;
            v[i][j] = dd;
            q += (c < d) ? dd * dd : 0.0f;
        }
    }
    q = block_sum(q, smem) / (float)d;
    const float sd = sqrtf(q + eps);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = (i * 256 + threadIdx.x) * N;
        if (c < d) {
            float o[N];
#pragma unroll
            for (int j = 0; j < N; ++j) {
                const float g = gain ? gain[c + j] : 1.0f;
                const float b = (bias && kind == JSM_ROWS_LAYERNORM) ? bias[c + j] : 0.0f;
                o[j] = g * (v[i][j] / sd) + b;
            }
            VecIO<T>::store(y + base + c, o);
        }
    }
}

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_embedding(const void* d_table, const void* d_pos_table, const int32_t* d_ids,
                                    const int32_t* d_positions, void* d_out, jsm_dtype dtype, int T, int d, void* stream) {
    if (T == 0) return JSM_OK;
    if (!d_table || !d_ids || !d_out) JSM_FAIL(JSM_INVALID_ARG, "jsm_embedding: null pointer");
    if (dtype == JSM_F32 && d % 4 == 0)
        JSM_CUDA_CHECK(launch_chained(embedding_kernel<float>, dim3(T), dim3(256), 0, as_stream(stream), (const float*)d_table,
                                      (const float*)d_pos_table, d_ids, d_positions, (float*)d_out, d));
    else if (dtype == JSM_BF16 && d % 8 == 0)
        JSM_CUDA_CHECK(launch_chained(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, as_stream(stream),
                                      (const __nv_bfloat16*)d_table, (const __nv_bfloat16*)d_pos_table, d_ids, d_positions,
                                      (__nv_bfloat16*)d_out, d));
    else
        JSM_FAIL(JSM_UNSUPPORTED, "jsm_embedding: dtype %d with d %d (d must be a multiple of 16 bytes)", (int)dtype, d);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

extern "C" jsm_status jsm_add_norm(int kind, const void* d_h, const void* d_delta, void* d_h_out, void* d_y, jsm_dtype dtype,
                                   const float* d_gain, const float* d_bias, float eps, int T, int d, void* stream) {
    if (T == 0) return JSM_OK;
    if (!d_h || !d_y) JSM_FAIL(JSM_INVALID_ARG, "jsm_add_norm: null pointer");
    if (kind != JSM_ROWS_LAYERNORM && kind != JSM_ROWS_RMSNORM) JSM_FAIL(JSM_INVALID_ARG, "jsm_add_norm: kind %d", kind);
    cudaStream_t st = as_stream(stream);
    if (dtype == JSM_F32) {
        if (d % 4 || d > 256 * 4 * 4) JSM_FAIL(JSM_UNSUPPORTED, "jsm_add_norm: f32 needs d %% 4 == 0 and d <= 4096 (d %d)", d);
        add_norm_kernel<float, 4><<<T, 256, 0, st>>>(kind, (const float*)d_h, (const float*)d_delta, (float*)d_h_out,
                                                     (float*)d_y, d_gain, d_bias, eps, d);
    } else if (dtype == JSM_BF16) {
        if (d % 8 || d > 256 * 8 * 4) JSM_FAIL(JSM_UNSUPPORTED, "jsm_add_norm: bf16 needs d %% 8 == 0 and d <= 8192 (d %d)", d);
        if (d <= 256 * 8 * 2)
            add_norm_kernel<__nv_bfloat16, 2><<<T, 256, 0, st>>>(kind, (const __nv_bfloat16*)d_h, (const __nv_bfloat16*)d_delta,
                                                                (__nv_bfloat16*)d_h_out, (__nv_bfloat16*)d_y, d_gain, d_bias, eps, d);
        else
            add_norm_kernel<__nv_bfloat16, 4><<<T, 256, 0, st>>>(kind, (const __nv_bfloat16*)d_h, (const __nv_bfloat16*)d_delta,
                                                                (__nv_bfloat16*)d_h_out, (__nv_bfloat16*)d_y, d_gain, d_bias, eps, d);
    } else {
        JSM_FAIL(JSM_UNSUPPORTED, "jsm_add_norm: dtype %d", (int)dtype);
    }
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}
