// Internal interface of the bf16 projection kernels (linear_bf16.cu).
#pragma once
#include "common.cuh"

namespace jsm {

enum LinearEpilogue { LIN_NONE = 0, LIN_RELU = 1, LIN_GELU = 2, LIN_SILU_MUL = 3, LIN_RESIDUAL = 4 };

struct LinearArgs {
    const void* X;      // [T, K] bf16
    const void* W;      // [N, K] bf16 ([2N, K] for LIN_SILU_MUL: N gate rows then N up rows)
    const float* bias;  // [N] or null
    int epilogue;
    const void* R;      // [T, N] bf16 residual or null
    void* Y;            // out_mode 0: bf16 [T,N]; 1: f32 [T,N]; 2: f32 partials [splits][T][N]
    int out_mode;
    int T, N, K;
    int splits;         // grid split along K: out_mode 2 writes the raw partials; with a workspace the kernel folds them itself
    int impl;           // 0 auto, 1 CUDA-core stream (T <= 4), 2 tcgen05
    float* ws = nullptr;      // workspace of splits * T * (N or 2N) floats for the in-kernel fix-up
    bool chained = false;     // launched as a link of a kernel chain whose weights are constant: W may be fetched before the
                              // predecessor kernel has finished (programmatic dependent launch)
    int* counters = nullptr;  // ceil(N/128) * ceil(T/BN) arrival counters, zero before the first launch
};

jsm_status linear_bf16_launch(const LinearArgs& a, cudaStream_t st);
// reads (and clears) the device error word of the tensor-core kernels; synchronises the stream
jsm_status tc_check_error(cudaStream_t st, const char* who);

}  // namespace jsm
