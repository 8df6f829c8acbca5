// Internal interface of the attention kernels.
#pragma once
#include "common.cuh"

namespace jsm {

jsm_status attn_simt_launch(const void* q, const void* k, const void* v, void* out, jsm_dtype dtype, int batch, int Tq, int Tk,
                            int Hq, int Hkv, int D, int causal, float scale, const float* rope, cudaStream_t st,
                            long long q_row_stride = 0, long long kv_row_stride = 0, long long out_row_stride = 0, int pos0 = 0);
bool flash_available();
jsm_status flash_prefill_launch(const void* q, const void* k, const void* v, void* out, int batch, int Tq, int Tk, int Hq, int Hkv,
                                int causal, float scale, const float* rope, cudaStream_t st, long long q_row_stride = 0,
                                long long kv_row_stride = 0, long long out_row_stride = 0);

jsm_status rope_apply_strided(const void* d_x, void* d_out, jsm_dtype dtype, const float* d_table, int d, int n_heads,
                              const int32_t* d_positions, int T, long long row_stride, void* stream);

}  // namespace jsm
