// C entry point of prefill attention: argument checks and the choice between the
// CUDA-core fp32 kernel and the tcgen05 flash kernel.
#include "common.cuh"
#include "attn.cuh"

using namespace jsm;

namespace {
__global__ void positions_kernel(int32_t* pos, int T, int offset, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pos[i] = i % T + offset;
}
jsm_status fill_positions(int32_t* pos, int batch, int T, int offset, cudaStream_t st) {
    const int n = batch * T;
    positions_kernel<<<(n + 255) / 256, 256, 0, st>>>(pos, T, offset, n);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}
}  // namespace

extern "C" jsm_status jsm_attn_prefill(const void* d_q, const void* d_k, const void* d_v, void* d_out, jsm_dtype dtype, int batch,
                                       int T_q, int T_k, int Hq, int Hkv, int D, int causal, float scale, const float* d_rope_table,
                                       int impl, void* stream) {
    if (batch <= 0 || T_q <= 0) return JSM_OK;
    if (!d_q || !d_k || !d_v || !d_out) JSM_FAIL(JSM_INVALID_ARG, "jsm_attn_prefill: null pointer");
    if (T_k <= 0) JSM_FAIL(JSM_SHAPE, "jsm_attn_prefill: no keys");
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) JSM_FAIL(JSM_SHAPE, "d_model must be divisible by num_heads (Hq %d, Hkv %d)", Hq, Hkv);
    if (D <= 0 || D % 2 || D > 128) JSM_FAIL(JSM_UNSUPPORTED, "jsm_attn_prefill: head_dim %d (even, <= 128)", D);
    if (dtype != JSM_F32 && dtype != JSM_BF16) JSM_FAIL(JSM_UNSUPPORTED, "jsm_attn_prefill: dtype %d", (int)dtype);
    if (causal && T_k < T_q) JSM_FAIL(JSM_SHAPE, "jsm_attn_prefill: causal attention needs T_k >= T_q");
    cudaStream_t st = as_stream(stream);
    const bool flash_ok = dtype == JSM_BF16 && D == 128;
    if (impl == 2 && !flash_ok) JSM_FAIL(JSM_UNSUPPORTED, "jsm_attn_prefill: the tcgen05 kernel needs bf16 and head_dim 128");
    if (impl == 2 || (impl == 0 && flash_ok && T_q >= 128)) {
        if (!d_rope_table) return flash_prefill_launch(d_q, d_k, d_v, d_out, batch, T_q, T_k, Hq, Hkv, causal, scale, nullptr, st);
        // the tensor-core kernel takes rotated q and k: rotate into stream-ordered temporaries first
        // (sequences start at position 0; queries sit at the end of the keys)
        // (stream-ordered allocations: no device synchronisation, legal inside a stream capture; released on every path)
        struct Temps {
            cudaStream_t st;
            void *qr = nullptr, *kr = nullptr;
            int32_t* pos = nullptr;
            ~Temps() {
                if (qr) cudaFreeAsync(qr, st);
                if (kr) cudaFreeAsync(kr, st);
                if (pos) cudaFreeAsync(pos, st);
            }
        } tmp{st};
        const size_t qn = (size_t)batch * T_q * Hq * D, kn = (size_t)batch * T_k * Hkv * D;
        JSM_CUDA_CHECK(cudaMallocAsync(&tmp.qr, qn * 2, st));
        JSM_CUDA_CHECK(cudaMallocAsync(&tmp.kr, kn * 2, st));
        JSM_CUDA_CHECK(cudaMallocAsync(reinterpret_cast<void**>(&tmp.pos), sizeof(int32_t) * (size_t)batch * (T_q + T_k), st));
        int32_t* pos = tmp.pos;
        jsm_status s = fill_positions(pos, batch, T_q, T_k - T_q, st);
        if (s == JSM_OK) s = fill_positions(pos + (size_t)batch * T_q, batch, T_k, 0, st);
        if (s == JSM_OK && T_q == T_k) {
            s = jsm_rope_apply_qk(d_q, tmp.qr, Hq, d_k, tmp.kr, Hkv, JSM_BF16, d_rope_table, D, pos, batch * T_q, st);  // one launch
        } else {
            if (s == JSM_OK) s = jsm_rope_apply(d_q, tmp.qr, JSM_BF16, d_rope_table, D, Hq, pos, batch * T_q, st);
            if (s == JSM_OK) s = jsm_rope_apply(d_k, tmp.kr, JSM_BF16, d_rope_table, D, Hkv, pos + (size_t)batch * T_q, batch * T_k, st);
        }
        if (s == JSM_OK) s = flash_prefill_launch(tmp.qr, tmp.kr, d_v, d_out, batch, T_q, T_k, Hq, Hkv, causal, scale, nullptr, st);
        return s;
    }
    return attn_simt_launch(d_q, d_k, d_v, d_out, dtype, batch, T_q, T_k, Hq, Hkv, D, causal, scale, d_rope_table, st);
}
