// Internal interface of the attention kernels.
#pragma once
#include "common.cuh"

namespace jsm {

jsm_status attn_simt_launch(const void* q, const void* k, const void* v, void* out, jsm_dtype dtype, int batch, int Tq, int Tk,
                            int Hq, int Hkv, int D, int causal, float scale, const float* rope, cudaStream_t st,
                            long long q_row_stride = 0, long long kv_row_stride = 0, long long out_row_stride = 0, int pos0 = 0);
jsm_status flash_prefill_launch(const void* q, const void* k, const void* v, void* out, int batch, int Tq, int Tk, int Hq, int Hkv,
                                int causal, float scale, const float* rope, cudaStream_t st, long long q_row_stride = 0,
                                long long kv_row_stride = 0, long long out_row_stride = 0);

jsm_status rope_apply_strided(const void* d_x, void* d_out, jsm_dtype dtype, const float* d_table, int d, int n_heads,
                              const int32_t* d_positions, int T, long long row_stride, void* stream);

// decode attention of grouped-query models on the tensor cores (attn_decode_mma.cu)
bool attn_decode_mma_usable(int G, int chunk, const void* pool);
struct DecodeMmaArgs {
    const void* q;
    long long q_stride;
    void* pool;
    const int32_t* block_table;
    int max_pages;
    const int32_t* context_lens;
    int n_seqs, Hq, Hkv;
    float scale_log2;
    const float* rope;
    int n_chunks, chunk;
    float* scratch;   // [n_seqs][Hq][n_chunks][130] floats of chunk partials
    bool fused;       // append k_new / v_new first and merge the partials into `out` (needs counters)
    const void* k_new;
    const void* v_new;
    long long kv_new_stride;
    int* counters;
    void* out;
};
jsm_status attn_decode_mma_launch(const DecodeMmaArgs& a, cudaStream_t st);

}  // namespace jsm
