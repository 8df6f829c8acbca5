// Decoder-only LLaMA-shape model on one GPU (one tensor-parallel rank): weights,
// paged KV cache, prefill and greedy decode step.  The block wiring is composed
// from the library's kernels the way the reference composes its stack from nets
// (encoder_t::forward loops the layers, mat_transformer_kernel_t.hpp:103-110;
// residual_net_t adds f(x) + x, mat_net_t.hpp:326-329), with the LLaMA parts the
// reference lacks (RMSNorm, SwiGLU, dense QKV, RoPE on q/k, GQA, token embedding,
// logits and argmax).
//
// Tensor parallelism: query/kv heads and FFN columns are split across tp_size
// ranks (one process per GPU).  The partial outputs of the attention output
// projection and of the FFN down projection are summed by one all-reduce each,
// issued through a callback so that the host owns the communicator.
#include "common.cuh"
#include "linear_bf16.cuh"
#include "attn.cuh"
#include <math.h>
#include <string.h>
#include <stdlib.h>
#include <string>
#include <vector>
#include <map>
#include <algorithm>

namespace jsm {

jsm_status attn_decode_append_checked(const void* d_q, int64_t q_row_stride, const void* d_k_new, const void* d_v_new,
                                      int64_t kv_new_stride, void* d_pool, const int32_t* d_block_table, int max_pages,
                                      const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D, float scale,
                                      const float* d_rope_table, int max_context, void* d_scratch, size_t scratch_bytes,
                                      int32_t* d_counters, void* d_out, void* stream);
int* tc_error_word();
constexpr int TC_CONTEXT_OVERFLOW = 32;  // error word code: a decode step met a sequence that already holds max_context tokens
jsm_status tp_argmax_exchange_launch(void* const* regions, int rank, int size, int max_tokens, int d, const int* pass, int site, int n_sites,
                                     const float* best_val, const int* best_idx, int32_t* out, int T, cudaStream_t st);
jsm_status tp_allreduce_add_norm_launch(void* const* regions, int rank, int size, size_t buf_offset, const int* pass, int site,
                                        int n_sites, void* h, void* xn, float eps, int T, int d, cudaStream_t st);

// The projection weights are kept packed (linear_packed.cu: contiguous 16 KB tiles in stream order); the logical
// matrices are the reference's [out, in] layout (mat_net_t.hpp:25-26).
struct LayerW {
    float* g1;
    uint8_t* wqkv;        // packed [(Hq_l + 2 Hkv_l) * D, d]: q rows, k rows, v rows
    uint8_t* wo;          // packed [d, Hq_l * D]
    float* g2;
    uint8_t* wgu;         // packed pairs of [2 * ffn_l, d]: gate rows, then up rows
    uint8_t* wdown;       // packed [d, ffn_l]
    __nv_bfloat16* pool;  // KV pages of this layer
};

}  // namespace jsm

struct jsm_model {
    jsm_model_config c;
    int Hq_l, Hkv_l, ffn_l, qkv_dim, pages_per_seq, max_tokens;
    std::vector<jsm::LayerW> layers;
    __nv_bfloat16* emb = nullptr;
    uint8_t* lm_head = nullptr;  // packed [vocab, d]
    __nv_bfloat16* unpack_buf = nullptr;  // row-major copy of the weight last asked for (jsm_llama_weight)
    size_t unpack_elems = 0;
    float* gf = nullptr;
    float* rope = nullptr;
    int32_t* block_table = nullptr;
    int32_t* ctx = nullptr;      // context length per sequence (device)
    int32_t* pos = nullptr;      // scratch: positions of the tokens of the current call
    int32_t* seq_ids = nullptr;  // scratch: sequence of each token of the current call
    __nv_bfloat16 *h = nullptr, *xn = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *red = nullptr;
    float* partial = nullptr;
    float* logits = nullptr;
    float* dec_scratch = nullptr;
    size_t dec_scratch_bytes = 0;
    float *ssq0 = nullptr, *ssq_a = nullptr, *ssq_b = nullptr;  // row statistics: after the embedding, after wo, after down
    size_t ws_floats = 0;        // capacity of `partial`: fp32 partials of the tiles that several CTAs share
    int* counters = nullptr;     // one arrival counter per tile (self-resetting)
    int n_counters = 0;
    int32_t* attn_counters = nullptr;  // one per (sequence, kv head) of the decode attention (self-resetting)
    std::vector<void*> allocs;
    // tensor-parallel exchange over peer memory (tp_comm.cu): own region, the peers' regions once connected, call state
    uint8_t* tp_region = nullptr;
    void* tp_regions[8] = {nullptr};
    int32_t* tp_state = nullptr;
    bool tp_connected = false;
    unsigned long long* argmax_key = nullptr;  // split arg-max: best (value, index) key per row (self-resetting)
    int32_t* argmax_ctr = nullptr;             // ... and the number of slices that have contributed
    float* best_val = nullptr;   // vocabulary-sharded lm_head: this rank's best logit per token
    int32_t* best_idx = nullptr;
    bool last_push = false;  // the last forward call exchanged by push (its final exchange is consumed by the logits projection)
    bool last_inband = false;  // ... as words that carry the exchange's epoch (at most TP_INBAND_MAX_T tokens)
    jsm_allreduce_fn allreduce = nullptr;
    void* allreduce_user = nullptr;
    uint64_t weight_bytes = 0;
    // host-buffer decode step (jsm_llama_decode_step_host): staging buffers and one instantiated graph per batch size
    int32_t *ids_dev = nullptr, *next_dev = nullptr;
    std::map<int, cudaGraphExec_t> step_graphs;
    // continuous batching (jsm_llama_create_paged): pages are handed out on demand from one pool; the active sequences
    // occupy the batch rows 0 .. n_active-1 and a retiring row is refilled with the last one (its block-table row moves,
    // its pages stay where they are)
    bool paged = false;
    int n_pool_pages = 0, n_active = 0;
    std::vector<int32_t> free_pages;
    std::vector<std::vector<int32_t>> row_pages;
    std::vector<int32_t> h_ctx;
    int32_t* prompt_dev = nullptr;
};

namespace jsm {

// Rows [start, start + rows) of a stacked logical matrix come from rows row0.. of the full tensor with generator key
// `key`; value (r, c) of a shard = element ((row0 + r) * full_cols + col0 + c) of the full tensor, so that all TP
// layouts agree.
struct RowSeg { long long start, rows, row0; uint64_t key; };
struct FillSpec { RowSeg seg[3]; int n_seg; long long full_cols, col0; float std; const float* gain; };  // gain[k] (or null) scales column k

// generates a weight matrix straight into its packed image (one thread per 16-byte chunk, see pack_weights_kernel)
__global__ void __launch_bounds__(256) fill_packed_kernel(uint8_t* __restrict__ dst, int N, int K, int n_tiles, int kbt, int paired,
                                                          FillSpec spec) {
    const long long total = (long long)n_tiles * kbt * 1024;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(idx % 1024);
        const long long unit = idx / 1024;
        const int kb = (int)(unit % kbt), j = (int)(unit / kbt);
        const int r = q >> 3, cs = q & 7, c = cs ^ (r & 7);
        const long long row = pk_source_row(paired, N, j, r);
        const int k = kb * 64 + c * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row >= 0 && k < K) {
            int sg = 0;
            while (sg + 1 < spec.n_seg && row >= spec.seg[sg].start + spec.seg[sg].rows) ++sg;
            const RowSeg& S = spec.seg[sg];
            const uint64_t base = (uint64_t)((S.row0 + (row - S.start)) * spec.full_cols + spec.col0 + k);
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // the tensor's own value is its bf16 rounding; the gain of the norm in front of the projection is folded in
                float lo = bf16_bits_to_f32(f32_to_bf16_bits(rng_value(S.key, base + 2 * e, 0, 0.0f, spec.std)));
                float hi = bf16_bits_to_f32(f32_to_bf16_bits(rng_value(S.key, base + 2 * e + 1, 0, 0.0f, spec.std)));
                if (spec.gain) { lo *= spec.gain[k + 2 * e]; hi *= spec.gain[k + 2 * e + 1]; }
                w[e] = (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
            }
            v = make_uint4(w[0], w[1], w[2], w[3]);
        }
        reinterpret_cast<uint4*>(dst)[idx] = v;
    }
}
// dst[r, k] = bf16(src[r, k] * gain[k]): the fold of a norm's gain into the projection behind it, rounded like the
// generated weights
__global__ void __launch_bounds__(256) scale_cols_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                         long long rows, int K, const float* __restrict__ gain) {
    const long long n = rows * K;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float g = gain ? gain[(int)(i % K)] : 1.0f;
        dst[i] = __float2bfloat16_rn(__bfloat162float(src[i]) * g);
    }
}
// row-major fill of a shard (the embedding table, which is gathered and not streamed)
__global__ void fill_shard_kernel(__nv_bfloat16* dst, long long rows, long long cols, long long full_cols, long long row0,
                                  long long col0, uint64_t key, float std) {
    const long long n = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i % cols;
        const float v = rng_value(key, (uint64_t)((row0 + r) * full_cols + col0 + c), 0, 0.0f, std);
        dst[i] = __float2bfloat16_rn(v);
    }
}
__global__ void fill_const_kernel(float* dst, long long n, float v) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] = v;
}
// pass: number of the forward pass (the epoch base of the tensor-parallel exchanges), bumped by the first kernel of a pass.
// That kernel lets its dependents start only after the new number has reached memory: the fused exchanges of the pass
// read it while their predecessors may still be running, so it must be in place before ANY later kernel of the chain can
// become resident (a kernel starts only after every CTA of its predecessor has passed its chain_trigger).
__global__ void iota_kernel(int32_t* pos, int32_t* seq_ids, int T, int seq, int pos0, int32_t* pass) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < T) { pos[i] = pos0 + i; seq_ids[i] = seq; }
    if (i == 0 && pass) {
        *pass = *pass + 1;
        __threadfence();
    }
    chain_trigger();
}
__global__ void set_ctx_kernel(int32_t* ctx, int seq, int value) { ctx[seq] = value; }
// decode bookkeeping on the device so that a captured step can be replayed: the new token of
// sequence b goes to position ctx[b], then the context grows by one
// A sequence that already holds max_context tokens does not grow: its new token overwrites the last position (every
// later access stays inside the sequence's pages and the rope table) and the error word records the overflow.
__global__ void advance_kernel(int32_t* ctx, int32_t* pos, int32_t* seq_ids, int batch, int32_t* pass, int max_context, int* err) {
    chain_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) {
        int c = ctx[b];
        if (c >= max_context) {
            c = max_context - 1;
            if (err) atomicCAS(err, 0, TC_CONTEXT_OVERFLOW);
        }
        pos[b] = c;
        seq_ids[b] = b;
        ctx[b] = c + 1;
    }
    if (b == 0 && pass) *pass = *pass + 1;
    __threadfence();
    chain_trigger();  // after the pass number and the context lengths are in memory (see iota_kernel): later kernels of the
                      // chain read both before they wait for their predecessors
}

__device__ __forceinline__ float block_sum_256(float v, float* smem) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += smem[w];
    return s;
}

// h[t,:] += sum_s partial[s][t][:] (+ delta[t,:]); h stored in bf16; y = RMSNorm(h) * gain.
// One CTA per token, d <= 256 * 8 * MAXV.
template <int MAXV>
__global__ void __launch_bounds__(256) fold_add_norm_kernel(__nv_bfloat16* __restrict__ h, const float* __restrict__ partial, int splits,
                                                            long long split_stride, const __nv_bfloat16* __restrict__ delta,
                                                            const float* __restrict__ gain, float eps, __nv_bfloat16* __restrict__ y, int d) {
    __shared__ float smem[8];
    chain_trigger();
    chain_wait();
    const long long base = (long long)blockIdx.x * d;
    float v[MAXV][8];
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = (i * 256 + threadIdx.x) * 8;
        if (c < d) {
            const uint4 w = *reinterpret_cast<const uint4*>(h + base + c);
            v[i][0] = bf16lo(w.x); v[i][1] = bf16hi(w.x); v[i][2] = bf16lo(w.y); v[i][3] = bf16hi(w.y);
            v[i][4] = bf16lo(w.z); v[i][5] = bf16hi(w.z); v[i][6] = bf16lo(w.w); v[i][7] = bf16hi(w.w);
#pragma unroll 4
            for (int s = 0; s < splits; ++s) {
                const float4 a = __ldcs(reinterpret_cast<const float4*>(partial + s * split_stride + base + c));
                const float4 b = __ldcs(reinterpret_cast<const float4*>(partial + s * split_stride + base + c + 4));
                v[i][0] += a.x; v[i][1] += a.y; v[i][2] += a.z; v[i][3] += a.w;
                v[i][4] += b.x; v[i][5] += b.y; v[i][6] += b.z; v[i][7] += b.w;
            }
            if (delta) {
                const uint4 e = *reinterpret_cast<const uint4*>(delta + base + c);
                v[i][0] += bf16lo(e.x); v[i][1] += bf16hi(e.x); v[i][2] += bf16lo(e.y); v[i][3] += bf16hi(e.y);
                v[i][4] += bf16lo(e.z); v[i][5] += bf16hi(e.z); v[i][6] += bf16lo(e.w); v[i][7] += bf16hi(e.w);
            }
            uint4 o;
            o.x = pack_bf16x2(v[i][0], v[i][1]); o.y = pack_bf16x2(v[i][2], v[i][3]);
            o.z = pack_bf16x2(v[i][4], v[i][5]); o.w = pack_bf16x2(v[i][6], v[i][7]);
            if (splits > 0 || delta) *reinterpret_cast<uint4*>(h + base + c) = o;
            // normalise what was stored
            v[i][0] = bf16lo(o.x); v[i][1] = bf16hi(o.x); v[i][2] = bf16lo(o.y); v[i][3] = bf16hi(o.y);
            v[i][4] = bf16lo(o.z); v[i][5] = bf16hi(o.z); v[i][6] = bf16lo(o.w); v[i][7] = bf16hi(o.w);
#pragma unroll
            for (int j = 0; j < 8; ++j) q += v[i][j] * v[i][j];
        }
    }
    if (!y) return;
    q = block_sum_256(q, smem) / (float)d;
    const float sd = sqrtf(q + eps);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = (i * 256 + threadIdx.x) * 8;
        if (c < d) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (gain ? gain[c + j] : 1.0f) * (v[i][j] / sd);
            uint4 w;
            w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]); w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(y + base + c) = w;
        }
    }
}

// ssq[t] = sum of squares of row t of x (bf16): the row statistics of the embedding output, in the form the packed
// projections exchange them (one "tile" per row)
__global__ void __launch_bounds__(256) row_ssq_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ ssq, int d) {
    __shared__ float smem[8];
    chain_trigger();
    chain_wait();
    const __nv_bfloat16* row = x + (long long)blockIdx.x * d;
    float q = 0.0f;
    for (int c = threadIdx.x * 8; c < d; c += 256 * 8) {
        const uint4 w = *reinterpret_cast<const uint4*>(row + c);
        const float f[8] = {bf16lo(w.x), bf16hi(w.x), bf16lo(w.y), bf16hi(w.y), bf16lo(w.z), bf16hi(w.z), bf16lo(w.w), bf16hi(w.w)};
#pragma unroll
        for (int j = 0; j < 8; ++j) q += f[j] * f[j];
    }
    q = block_sum_256(q, smem);
    if (threadIdx.x == 0) ssq[blockIdx.x] = q;
}

// The start of a decode step in one launch: the bookkeeping of advance_kernel for sequence b = blockIdx.x, the embedding
// row of its token and the row's sum of squares (what embedding_kernel and row_ssq_kernel do in two more launches; same
// order of the additions).  Like advance_kernel it lets its dependents start only after its stores are in memory.
__global__ void __launch_bounds__(256) decode_begin_kernel(int32_t* ctx, int32_t* pos, int32_t* seq_ids, int32_t* pass, int max_context,
                                                           int* err, const __nv_bfloat16* __restrict__ table,
                                                           const int32_t* __restrict__ ids, __nv_bfloat16* __restrict__ h,
                                                           float* __restrict__ ssq, int d) {
    __shared__ float smem[8];
    chain_wait();
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        int c = ctx[b];
        if (c >= max_context) {
            c = max_context - 1;
            if (err) atomicCAS(err, 0, TC_CONTEXT_OVERFLOW);
        }
        pos[b] = c;
        seq_ids[b] = b;
        ctx[b] = c + 1;
        if (b == 0 && pass) *pass = *pass + 1;
    }
    const __nv_bfloat16* src = table + (long long)ids[b] * d;
    __nv_bfloat16* dst = h + (long long)b * d;
    float q = 0.0f;
    for (int c = threadIdx.x * 8; c < d; c += 256 * 8) {
        const uint4 w = *reinterpret_cast<const uint4*>(src + c);
        *reinterpret_cast<uint4*>(dst + c) = w;
        const float f[8] = {bf16lo(w.x), bf16hi(w.x), bf16lo(w.y), bf16hi(w.y), bf16lo(w.z), bf16hi(w.z), bf16lo(w.w), bf16hi(w.w)};
#pragma unroll
        for (int j = 0; j < 8; ++j) q += f[j] * f[j];
    }
    q = block_sum_256(q, smem);
    if (threadIdx.x == 0) ssq[b] = q;
    __threadfence();
    chain_trigger();
}

__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ x, int32_t* __restrict__ out, int n) {
    __shared__ float sv[8];
    __shared__ int si[8];
    chain_trigger();
    chain_wait();
    const float* row = x + (long long)blockIdx.x * n;
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = row[i];
        if (v > m || (v == m && i < mi)) { m = v; mi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, m, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (ov > m || (ov == m && oi < mi)) { m = ov; mi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = m; si[threadIdx.x >> 5] = mi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > m || (sv[w] == m && si[w] < mi)) { m = sv[w]; mi = si[w]; }
        out[blockIdx.x] = mi == 0x7fffffff ? 0 : mi;
    }
}

// The same arg-max with every row split over gridDim.x CTAs (a row of 32000 logits is too long for one CTA on the path of
// a decode step): a slice's best (value, index) becomes one 64-bit key - the value's bits made monotone in the high word,
// the complemented index in the low word, so that the larger key is the larger value and, among equal values, the lower
// index - and goes into the row's key with atomicMax; the CTA that arrives last at the row's counter writes the token and
// resets both words for the next launch.  Same result as argmax_rows_kernel (NaNs never win, all -inf gives 0).
constexpr int ARGMAX_SPLIT = 16;
__global__ void __launch_bounds__(256) argmax_rows_split_kernel(const float* __restrict__ x, int32_t* __restrict__ out, int n,
                                                                unsigned long long* __restrict__ keys, int32_t* __restrict__ ctrs) {
    __shared__ float sv[8];
    __shared__ int si[8];
    chain_trigger();
    chain_wait();
    const int r = blockIdx.y;
    const float* row = x + (long long)r * n;
    const int lo = (int)((long long)blockIdx.x * n / gridDim.x), hi = (int)((long long)(blockIdx.x + 1) * n / gridDim.x);
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += 256) {
        const float v = row[i];
        if (v > m || (v == m && i < mi)) { m = v; mi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, m, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (ov > m || (ov == m && oi < mi)) { m = ov; mi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = m; si[threadIdx.x >> 5] = mi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > m || (sv[w] == m && si[w] < mi)) { m = sv[w]; mi = si[w]; }
        const uint32_t bits = __float_as_uint(m);
        const uint32_t mono = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
        const unsigned long long key = ((unsigned long long)mono << 32) | (uint32_t)(0xffffffffu - (uint32_t)mi);
        atomicMax(keys + r, key);
        __threadfence();
        if (atomicAdd(ctrs + r, 1) == (int)gridDim.x - 1) {
            __threadfence();
            const unsigned long long best = atomicExch(keys + r, 0ull);  // (read and reset in one)
            const uint32_t idx = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
            out[r] = idx == 0x7fffffffu ? 0 : (int32_t)idx;
            ctrs[r] = 0;
        }
    }
}

// best (value, index + col0) of every row: the local half of the arg-max over a vocabulary that is split across ranks
__global__ void __launch_bounds__(256) argmax_rows_pair_kernel(const float* __restrict__ x, float* __restrict__ best_val, int* __restrict__ best_idx,
                                                               int n, int col0) {
    __shared__ float sv[8];
    __shared__ int si[8];
    chain_trigger();
    chain_wait();
    const float* row = x + (long long)blockIdx.x * n;
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = row[i];
        if (v > m || (v == m && i < mi)) { m = v; mi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, m, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (ov > m || (ov == m && oi < mi)) { m = ov; mi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = m; si[threadIdx.x >> 5] = mi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (sv[w] > m || (sv[w] == m && si[w] < mi)) { m = sv[w]; mi = si[w]; }
        best_val[blockIdx.x] = m;
        best_idx[blockIdx.x] = mi == 0x7fffffff ? 0x7fffffff : mi + col0;
    }
}

template <typename T>
static jsm_status dev_alloc(jsm_model* m, T** p, size_t n) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, n * sizeof(T));
    if (e != cudaSuccess) {
        cudaGetLastError();
        JSM_FAIL(JSM_OOM, "jsm_llama_create: cudaMalloc of %zu bytes failed: %s", n * sizeof(T), cudaGetErrorString(e));
    }
    m->allocs.push_back(q);
    *p = reinterpret_cast<T*>(q);
    return JSM_OK;
}

static void fill_shard(__nv_bfloat16* dst, long long rows, long long cols, long long full_cols, long long row0, long long col0,
                       uint64_t seed, uint64_t tid, float std, cudaStream_t st) {
    const long long n = rows * cols;
    long long blocks = (n + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    fill_shard_kernel<<<(unsigned)blocks, 256, 0, st>>>(dst, rows, cols, full_cols, row0, col0, rng_key(seed, tid), std);
    g_launches.fetch_add(1);
}

// packed image of a stacked [N (or 2N when paired), K] matrix whose row blocks come from up to three tensors
static void fill_packed(uint8_t* dst, int N, int K, int paired, const FillSpec& spec, cudaStream_t st) {
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    const long long total = (long long)nt * kbt * 1024;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    fill_packed_kernel<<<(unsigned)blocks, 256, 0, st>>>(dst, N, K, nt, kbt, paired, spec);
    g_launches.fetch_add(1);
}

// Row statistics handed from the projection that writes the residual stream to the one that reads it (fused RMSNorm)
struct RowStats {
    const float* in = nullptr;  // [in_tiles][T] sums of squares of X's rows
    int in_tiles = 0;
    float* out = nullptr;       // [ceil(N/128)][T] sums of squares of the outputs
};

// One projection over packed weights for any number of tokens: chunks of 256 tokens, each streaming the weights once.
static jsm_status run_linear(jsm_model* m, const __nv_bfloat16* X, long long x_stride, const uint8_t* Wp, int N, int K, int epilogue,
                             const __nv_bfloat16* R, void* Y, bool out_f32, int T, cudaStream_t st, RowStats rs = RowStats(),
                             int stats_stride = 0, const TpFuse* tp = nullptr) {
    PackedArgs a;
    a.Wp = Wp; a.bias = nullptr; a.epilogue = epilogue; a.out_f32 = out_f32; a.N = N; a.K = K; a.x_row_stride = x_stride;
    a.ws = m->partial; a.ws_floats = m->ws_floats; a.counters = m->counters; a.n_counters = m->n_counters;
    a.chained = true;  // the model's weights are constant while its stream runs
    a.eps = m->c.norm_eps;
    a.ssq_in_tiles = rs.in_tiles;
    a.ssq_stride = stats_stride > 0 ? stats_stride : T;
    a.tp = tp;  // fused exchanges come with at most TP_PUSH_MAX_T tokens: one chunk
    for (int t0 = 0; t0 < T; t0 += 256) {
        a.T = T - t0 < 256 ? T - t0 : 256;
        a.X = X + (long long)t0 * x_stride;
        a.R = R ? R + (long long)t0 * N : nullptr;
        a.Y = out_f32 ? static_cast<void*>(reinterpret_cast<float*>(Y) + (long long)t0 * N)
                      : static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(Y) + (long long)t0 * N);
        a.ssq_in = rs.in ? rs.in + t0 : nullptr;
        a.ssq_out = rs.out ? rs.out + t0 : nullptr;
        jsm_status s = linear_packed_launch(a, st);
        if (s != JSM_OK) return s;
    }
    return JSM_OK;
}

// h += X . W^T (the residual stream).  One GPU: the projection adds into h in its epilogue and leaves the row
// statistics of the new h in `stats_out` for the projection that reads h next (which applies the RMSNorm itself).
// Tensor parallel: the rank-local product goes through the all-reduce, then h += sum and xn = RMSNorm(h) (the gain is
// folded into the next projection's weights) unless `normalise` is false.
static TpFuse exchange_base(jsm_model* m, int site) {
    TpFuse f;
    f.n_ranks = m->c.tp_size; f.rank = m->c.tp_rank;
    f.pass = m->tp_state; f.site = site; f.n_sites = 2 * m->c.n_layers + 1;  // two per layer and the arg-max exchange
    f.state = m->tp_state + 4;
    f.wait_limit = tp_wait_limit_cycles();
    f.inband = m->last_inband;
    return f;
}
// The consumer side of a pushed exchange: the projection that reads rows [first, first + rows) of the residual stream
// adds the ranks' slots of push buffer `which` to them first and writes their row statistics to `stats`.
static TpFuse consume_exchange(jsm_model* m, int which, int site, float* stats, int first) {
    TpFuse f = exchange_base(m, site);
    const int d = m->c.d_model;
    f.reduce = true;
    f.slots = f.inband ? m->tp_region + tp_inband_offset(which, m->max_tokens, d) + (size_t)first * d * 4  // (4 bytes per element)
                       : m->tp_region + tp_push_offset(which, m->max_tokens, d) + (size_t)first * d * sizeof(__nv_bfloat16);
    f.slot_stride = f.inband ? tp_inband_slot_bytes(d) : tp_slot_bytes(d);
    f.flags = reinterpret_cast<const int*>(m->tp_region) + tp_push_flag_word();
    f.h = m->h + (size_t)first * d;
    f.ssq = stats + first;
    return f;
}

static jsm_status project_into_residual(jsm_model* m, const __nv_bfloat16* X, const uint8_t* Wp, int T, int N, int K, float* stats_out,
                                        bool normalise, int which, int site, cudaStream_t st, bool push) {
    const int d = m->c.d_model;
    if (m->c.tp_size == 1) {
        RowStats rs;
        rs.out = stats_out;
        return run_linear(m, X, K, Wp, N, K, LIN_RESIDUAL, m->h, m->h, false, T, st, rs);
    }
    if (m->tp_connected && push) {
        // the projection stores its product straight into this rank's slot of every rank's push buffer and releases the
        // exchange's epoch; the projection that reads h next adds the slots to h in its prologue (consume_exchange)
        TpFuse f = exchange_base(m, site);
        f.push = true;
        const size_t off = f.inband ? tp_inband_offset(which, m->max_tokens, d) + (size_t)m->c.tp_rank * tp_inband_slot_bytes(d)
                                    : tp_push_offset(which, m->max_tokens, d) + (size_t)m->c.tp_rank * tp_slot_bytes(d);
        for (int r = 0; r < m->c.tp_size; ++r) {
            f.push_dst[r] = static_cast<uint8_t*>(m->tp_regions[r]) + off;
            f.push_flag[r] = static_cast<int*>(m->tp_regions[r]) + tp_push_flag_word() + m->c.tp_rank;
        }
        return run_linear(m, X, K, Wp, N, K, LIN_NONE, nullptr, nullptr, false, T, st, RowStats(), 0, &f);
    }
    if (m->tp_connected) {
        // the rank-local product goes into this call site's exchange buffer; one kernel then sums the ranks' buffers
        // over peer memory, adds the sum into h and normalises
        const size_t off = tp_buffer_offset(which, m->max_tokens, d);
        jsm_status s = run_linear(m, X, K, Wp, N, K, LIN_NONE, nullptr, m->tp_region + off, false, T, st);
        if (s != JSM_OK) return s;
        return tp_allreduce_add_norm_launch(m->tp_regions, m->c.tp_rank, m->c.tp_size, off, m->tp_state, site, 2 * m->c.n_layers + 1, m->h,
                                            normalise ? m->xn : nullptr, m->c.norm_eps, T, d, st);
    }
    jsm_status s = run_linear(m, X, K, Wp, N, K, LIN_NONE, nullptr, m->red, false, T, st);
    if (s != JSM_OK) return s;
    // no peer regions connected: the host's all-reduce (NCCL) sums the rank-local outputs, then add into the residual stream
    if (!m->allreduce) JSM_FAIL(JSM_NCCL, "tensor-parallel model without peer regions and without an all-reduce callback");
    if (m->allreduce(m->red, (size_t)T * N, JSM_BF16, st, m->allreduce_user) != 0) JSM_FAIL(JSM_NCCL, "all-reduce callback failed");
    JSM_CUDA_CHECK(launch_chained(fold_add_norm_kernel<2>, dim3(T), dim3(256), 0, st, m->h, nullptr, 0, 0, m->red, nullptr,
                                  m->c.norm_eps, normalise ? m->xn : nullptr, d));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

static jsm_status forward_tokens(jsm_model* m, const int32_t* d_ids, int T, bool decode, int batch, int prefill_seq, cudaStream_t st) {
    const jsm_model_config& c = m->c;
    const int d = c.d_model, D = c.head_dim;
    const bool tp = c.tp_size > 1;
    const int d_tiles = (d + 127) / 128;
    // few tokens (every decode step): the two exchanges of a layer are fused into the projections around them and the
    // step runs the one-GPU pipeline (un-normalised h + row statistics); otherwise the exchange kernel and a normalised copy
    const bool push = tp && m->tp_connected && T <= TP_PUSH_MAX_T && linear_packed_can_push(d, m->Hq_l * D, T) &&
                      linear_packed_can_push(d, m->ffn_l, T);
    m->last_push = push;
    m->last_inband = push && T <= TP_INBAND_MAX_T;
    const bool stats = !tp || push;  // h carries row statistics instead of a normalised copy
    jsm_status s = JSM_OK;
    if (decode && stats && d % 8 == 0) {
        // one launch: positions and context lengths of the step, the embedding rows and their statistics
        JSM_CUDA_CHECK(launch_chained(decode_begin_kernel, dim3(batch), dim3(256), 0, st, m->ctx, m->pos, m->seq_ids, m->tp_state,
                                      c.max_context, tc_error_word(), (const __nv_bfloat16*)m->emb, d_ids, m->h, m->ssq0, d));
    } else {
    if (decode) {
        JSM_CUDA_CHECK(launch_chained(advance_kernel, dim3((batch + 255) / 256), dim3(256), 0, st, m->ctx, m->pos, m->seq_ids, batch,
                                      m->tp_state, c.max_context, tc_error_word()));
        JSM_LAUNCH_CHECK();
    }
    s = jsm_embedding(m->emb, nullptr, d_ids, nullptr, m->h, JSM_BF16, T, d, st);
    if (s != JSM_OK) return s;
    if (!stats) {
        JSM_CUDA_CHECK(launch_chained(fold_add_norm_kernel<2>, dim3(T), dim3(256), 0, st, m->h, nullptr, 0, 0, nullptr, nullptr,
                                      c.norm_eps, m->xn, d));
    } else {
        JSM_CUDA_CHECK(launch_chained(row_ssq_kernel, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)m->h, m->ssq0, d));
    }
    }
    JSM_LAUNCH_CHECK();
    const __nv_bfloat16* x_in = stats ? m->h : m->xn;  // what the projections after a norm read
    const float scale = 1.0f / sqrtf((float)D);
    RowStats after_down;  // statistics of h as the previous layer (or the embedding) left it
    if (stats) { after_down.in = m->ssq0; after_down.in_tiles = 1; }
    for (int l = 0; l < c.n_layers; ++l) {
        LayerW& L = m->layers[l];
        if (push && l > 0) {
            const TpFuse f = consume_exchange(m, 1, 2 * (l - 1) + 1, m->ssq_b, 0);  // the previous layer's down projection
            s = run_linear(m, x_in, d, L.wqkv, m->qkv_dim, d, LIN_NONE, nullptr, m->qkv, false, T, st, after_down, 0, &f);
        } else
        s = run_linear(m, x_in, d, L.wqkv, m->qkv_dim, d, LIN_NONE, nullptr, m->qkv, false, T, st, after_down);
        if (s != JSM_OK) return s;
        const __nv_bfloat16* kk = m->qkv + (long long)m->Hq_l * D;
        const __nv_bfloat16* vv = kk + (long long)m->Hkv_l * D;
        if (decode) {
            // the new token: one launch rotates K into the cache, stores V, rotates q and attends over the context
            s = attn_decode_append_checked(m->qkv, m->qkv_dim, kk, vv, m->qkv_dim, L.pool, m->block_table, m->pages_per_seq, m->ctx, batch,
                                           m->Hq_l, m->Hkv_l, D, scale, m->rope, c.max_context, m->dec_scratch, m->dec_scratch_bytes,
                                           m->attn_counters, m->attn, st);
        } else {
            // prompt of one sequence starting at position 0: rotate q and k in place (the first Hq + Hkv heads of every
            // fused row), cache K and V, then causal attention over the fresh q, k, v
            s = rope_apply_strided(m->qkv, m->qkv, JSM_BF16, m->rope, D, m->Hq_l + m->Hkv_l, m->pos, T, m->qkv_dim, st);
            if (s != JSM_OK) return s;
            s = jsm_kv_append(L.pool, m->block_table, m->pages_per_seq, kk, vv, m->qkv_dim, m->seq_ids, m->pos, T, m->Hkv_l, D, nullptr, st);
            if (s != JSM_OK) return s;
            if (T >= 128)
                s = flash_prefill_launch(m->qkv, kk, vv, m->attn, 1, T, T, m->Hq_l, m->Hkv_l, 1, scale, nullptr, st, m->qkv_dim,
                                         m->qkv_dim, (long long)m->Hq_l * D);
            else
                s = attn_simt_launch(m->qkv, kk, vv, m->attn, JSM_BF16, 1, T, T, m->Hq_l, m->Hkv_l, D, 1, scale, nullptr, st,
                                     m->qkv_dim, m->qkv_dim, (long long)m->Hq_l * D, 0);
        }
        if (s != JSM_OK) return s;
        s = project_into_residual(m, m->attn, L.wo, T, d, m->Hq_l * D, m->ssq_a, true, 0, 2 * l, st, push);
        if (s != JSM_OK) return s;
        RowStats after_wo;
        if (stats) { after_wo.in = m->ssq_a; after_wo.in_tiles = d_tiles; }
        if (push) {
            const TpFuse f = consume_exchange(m, 0, 2 * l, m->ssq_a, 0);
            s = run_linear(m, x_in, d, L.wgu, m->ffn_l, d, LIN_SILU_MUL, nullptr, m->act, false, T, st, after_wo, 0, &f);
        } else
        s = run_linear(m, x_in, d, L.wgu, m->ffn_l, d, LIN_SILU_MUL, nullptr, m->act, false, T, st, after_wo);
        if (s != JSM_OK) return s;
        s = project_into_residual(m, m->act, L.wdown, T, d, m->ffn_l, m->ssq_b, true, 1, 2 * l + 1, st, push);
        if (s != JSM_OK) return s;
        if (stats) { after_down.in = m->ssq_b; after_down.in_tiles = d_tiles; }
    }
    (void)prefill_seq;
    return JSM_OK;
}

// logits of `rows` consecutive tokens starting at token `first` of the last forward call (which had T tokens)
static jsm_status logits_and_argmax(jsm_model* m, int first, int rows, int T, int32_t* d_next, float* d_logits, cudaStream_t st) {
    float* lg = d_logits ? d_logits : m->logits;
    const int d = m->c.d_model;
    const bool tp = m->c.tp_size > 1;
    const bool push = tp && m->last_push;  // the forward call that just ran pushed its exchanges: the last one is still to be consumed
    RowStats rs;
    if (!tp || push) { rs.in = m->ssq_b + first; rs.in_tiles = (d + 127) / 128; }
    const __nv_bfloat16* x = ((tp && !push) ? m->xn : m->h) + (long long)first * d;
    TpFuse f;
    if (push) f = consume_exchange(m, 1, 2 * (m->c.n_layers - 1) + 1, m->ssq_b, first);
    // Tokens only (no logits asked for) on a connected tensor-parallel group: every rank streams only its share of the
    // lm_head - a run of whole 128-row tiles of the same packed matrix - takes the best logit of its slice, and the ranks
    // exchange (value, index) pairs: 8 bytes per token and rank instead of (N-1)/N of the matrix on every rank.
    if (tp && m->tp_connected && d_next && !d_logits && rows <= m->c.max_batch) {
        int nt, kbt;
        pk_dims(m->c.vocab, d, 0, &nt, &kbt);
        const int t0 = (int)((long long)m->c.tp_rank * nt / m->c.tp_size), t1 = (int)((long long)(m->c.tp_rank + 1) * nt / m->c.tp_size);
        const int col0 = t0 * 128, n_local = std::min(t1 * 128, m->c.vocab) - col0;
        if (n_local > 0) {
            jsm_status s = run_linear(m, x, d, m->lm_head + (size_t)t0 * kbt * (128 * 64 * 2), n_local, d, LIN_NONE, nullptr, m->logits, true, rows, st,
                                      rs, T, push ? &f : nullptr);
            if (s != JSM_OK) return s;
            JSM_CUDA_CHECK(launch_chained(argmax_rows_pair_kernel, dim3(rows), dim3(256), 0, st, (const float*)m->logits, m->best_val, m->best_idx,
                                          n_local, col0));
            JSM_LAUNCH_CHECK();
            return tp_argmax_exchange_launch(m->tp_regions, m->c.tp_rank, m->c.tp_size, m->max_tokens, d, m->tp_state, 2 * m->c.n_layers,
                                             2 * m->c.n_layers + 1, m->best_val, m->best_idx, d_next, rows, st);
        }
    }
    jsm_status s = run_linear(m, x, d, m->lm_head, m->c.vocab, d, LIN_NONE, nullptr, lg, true, rows, st, rs, T, push ? &f : nullptr);
    if (s != JSM_OK) return s;
    if (d_next) {
        if (rows <= m->c.max_batch && m->c.vocab >= 4096)
            JSM_CUDA_CHECK(launch_chained(argmax_rows_split_kernel, dim3(ARGMAX_SPLIT, rows), dim3(256), 0, st, (const float*)lg, d_next,
                                          m->c.vocab, m->argmax_key, m->argmax_ctr));
        else
            JSM_CUDA_CHECK(launch_chained(argmax_rows_kernel, dim3(rows), dim3(256), 0, st, (const float*)lg, d_next, m->c.vocab));
        JSM_LAUNCH_CHECK();
    }
    return JSM_OK;
}

}  // namespace jsm

using namespace jsm;

extern "C" {

static jsm_status llama_create_impl(const jsm_model_config* cfg, uint64_t seed, int pool_pages, jsm_model** out) {
    if (!cfg || !out) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_create: null argument");
    *out = nullptr;
    const jsm_model_config& c = *cfg;
    if (c.n_layers <= 0 || c.d_model <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.d_ffn <= 0 || c.vocab <= 0 || c.max_batch <= 0 ||
        c.max_context <= 0)
        JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_create: non-positive dimension");
    if (c.head_dim != 128) JSM_FAIL(JSM_UNSUPPORTED, "jsm_llama_create: head_dim %d (128 only)", c.head_dim);
    if (c.n_heads % c.n_kv_heads) JSM_FAIL(JSM_SHAPE, "d_model must be divisible by num_heads (heads %d, kv heads %d)", c.n_heads, c.n_kv_heads);
    if (c.tp_size < 1 || c.tp_rank < 0 || c.tp_rank >= c.tp_size) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_create: tp rank %d of %d", c.tp_rank, c.tp_size);
    if (c.n_kv_heads % c.tp_size || c.d_ffn % c.tp_size || (c.d_ffn / c.tp_size) % 8)
        JSM_FAIL(JSM_SHAPE, "jsm_llama_create: kv heads %d / ffn %d not divisible across %d ranks", c.n_kv_heads, c.d_ffn, c.tp_size);
    if (c.d_model % 8 || c.d_model > 4096) JSM_FAIL(JSM_UNSUPPORTED, "jsm_llama_create: d_model %d (multiple of 8, <= 4096)", c.d_model);
    int ndev = 0;
    jsm_status s = jsm_device_count(&ndev);
    if (s != JSM_OK) return s;
    if (ndev == 0) JSM_FAIL(JSM_CUDA, "jsm_llama_create: no CUDA device");

    jsm_model* m = new jsm_model();
    m->c = c;
    m->Hq_l = c.n_heads / c.tp_size;
    m->Hkv_l = c.n_kv_heads / c.tp_size;
    m->ffn_l = c.d_ffn / c.tp_size;
    const int D = c.head_dim, d = c.d_model;
    m->qkv_dim = (m->Hq_l + 2 * m->Hkv_l) * D;
    m->pages_per_seq = (c.max_context + JSM_PAGE_SIZE - 1) / JSM_PAGE_SIZE;
    m->max_tokens = c.max_batch > 512 ? c.max_batch : 512;
    m->layers.resize(c.n_layers);
    cudaStream_t st = nullptr;
    const float std = 0.02f;
#define JSM_TRY(x)                  \
    do {                            \
        jsm_status s__ = (x);       \
        if (s__ != JSM_OK) {        \
            jsm_llama_destroy(m);   \
            return s__;             \
        }                           \
    } while (0)
    // static layout: every sequence owns its own run of pages; paged: a pool of pool_pages pages shared by all rows
    const long long table_entries = (long long)c.max_batch * m->pages_per_seq;
    const long long n_pages = pool_pages > 0 ? pool_pages : table_entries;
    m->paged = pool_pages > 0;
    m->n_pool_pages = (int)n_pages;
    const size_t page_elems = (size_t)2 * m->Hkv_l * JSM_PAGE_SIZE * D;
    uint64_t wbytes = 0;
    const int qdim = m->Hq_l * D;  // K of the attention output projection
    auto spec1 = [&](long long rows, long long row0, uint64_t tid, long long full_cols, long long col0) {
        FillSpec f{};
        f.n_seg = 1;
        f.seg[0] = RowSeg{0, rows, row0, rng_key(seed, tid)};
        f.full_cols = full_cols; f.col0 = col0; f.std = std; f.gain = nullptr;
        return f;
    };
    for (int l = 0; l < c.n_layers; ++l) {
        LayerW& L = m->layers[l];
        const uint64_t t0 = (uint64_t)l * 16;
        JSM_TRY(dev_alloc(m, &L.g1, (size_t)d));
        JSM_TRY(dev_alloc(m, &L.g2, (size_t)d));
        JSM_TRY(dev_alloc(m, &L.wqkv, linear_packed_bytes(m->qkv_dim, d, 0)));
        JSM_TRY(dev_alloc(m, &L.wo, linear_packed_bytes(d, qdim, 0)));
        JSM_TRY(dev_alloc(m, &L.wgu, linear_packed_bytes(m->ffn_l, d, 1)));
        JSM_TRY(dev_alloc(m, &L.wdown, linear_packed_bytes(d, m->ffn_l, 0)));
        JSM_TRY(dev_alloc(m, &L.pool, (size_t)n_pages * page_elems));
        fill_const_kernel<<<16, 256, 0, st>>>(L.g1, d, 1.0f);
        fill_const_kernel<<<16, 256, 0, st>>>(L.g2, d, 1.0f);
        // full tensors: wq [Hq*D, d] (id +0), wk [Hkv*D, d] (+1), wv (+2), wo [d, Hq*D] (+3), wgate [ffn, d] (+4), wup (+5), wdown [d, ffn] (+6)
        const long long qr = (long long)m->Hq_l * D, kr = (long long)m->Hkv_l * D;
        {
            FillSpec f{};
            f.n_seg = 3;
            f.seg[0] = RowSeg{0, qr, c.tp_rank * qr, rng_key(seed, t0 + 0)};
            f.seg[1] = RowSeg{qr, kr, c.tp_rank * kr, rng_key(seed, t0 + 1)};
            f.seg[2] = RowSeg{qr + kr, kr, c.tp_rank * kr, rng_key(seed, t0 + 2)};
            f.full_cols = d; f.col0 = 0; f.std = std; f.gain = L.g1;
            fill_packed(L.wqkv, m->qkv_dim, d, 0, f, st);
        }
        fill_packed(L.wo, d, qdim, 0, spec1(d, 0, t0 + 3, (long long)c.n_heads * D, c.tp_rank * qr), st);
        {
            FillSpec f{};
            f.n_seg = 2;
            f.seg[0] = RowSeg{0, m->ffn_l, (long long)c.tp_rank * m->ffn_l, rng_key(seed, t0 + 4)};
            f.seg[1] = RowSeg{m->ffn_l, m->ffn_l, (long long)c.tp_rank * m->ffn_l, rng_key(seed, t0 + 5)};
            f.full_cols = d; f.col0 = 0; f.std = std; f.gain = L.g2;
            fill_packed(L.wgu, m->ffn_l, d, 1, f, st);
        }
        fill_packed(L.wdown, d, m->ffn_l, 0, spec1(d, 0, t0 + 6, c.d_ffn, (long long)c.tp_rank * m->ffn_l), st);
        wbytes += 2ull * ((uint64_t)m->qkv_dim * d + (uint64_t)d * qdim + 2ull * m->ffn_l * d + (uint64_t)d * m->ffn_l) + 8ull * d;
    }
    JSM_TRY(dev_alloc(m, &m->emb, (size_t)c.vocab * d));
    JSM_TRY(dev_alloc(m, &m->lm_head, linear_packed_bytes(c.vocab, d, 0)));
    JSM_TRY(dev_alloc(m, &m->gf, (size_t)d));
    fill_shard(m->emb, c.vocab, d, d, 0, 0, seed, 1000000, std, st);
    fill_const_kernel<<<16, 256, 0, st>>>(m->gf, d, 1.0f);
    {
        FillSpec f = spec1(c.vocab, 0, 1000001, d, 0);
        f.gain = m->gf;
        fill_packed(m->lm_head, c.vocab, d, 0, f, st);
    }
    wbytes += 2ull * (uint64_t)c.vocab * d + 4ull * d;  // lm_head (streamed every step) and the final gain
    m->weight_bytes = wbytes;
    JSM_TRY(dev_alloc(m, &m->rope, (size_t)c.max_context * (D / 2) * 4));
    JSM_TRY(jsm_rope_table(m->rope, 1, D, c.rope_theta, c.max_context, st));
    JSM_TRY(dev_alloc(m, &m->block_table, (size_t)table_entries));
    {
        std::vector<int32_t> bt((size_t)table_entries, 0);
        if (!m->paged)
            for (long long i = 0; i < table_entries; ++i) bt[(size_t)i] = (int32_t)i;
        else {
            for (int p = (int)n_pages - 1; p >= 0; --p) m->free_pages.push_back(p);  // page 0 is handed out first
            m->row_pages.resize(c.max_batch);
            m->h_ctx.assign(c.max_batch, 0);
        }
        cudaError_t e = cudaMemcpy(m->block_table, bt.data(), bt.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { jsm_llama_destroy(m); JSM_FAIL(JSM_CUDA, "jsm_llama_create: block table upload: %s", cudaGetErrorString(e)); }
    }
    JSM_TRY(dev_alloc(m, &m->ctx, (size_t)c.max_batch));
    JSM_TRY(dev_alloc(m, &m->pos, (size_t)m->max_tokens));
    JSM_TRY(dev_alloc(m, &m->seq_ids, (size_t)m->max_tokens));
    const size_t Tm = (size_t)m->max_tokens;
    JSM_TRY(dev_alloc(m, &m->h, Tm * d));
    JSM_TRY(dev_alloc(m, &m->xn, Tm * d));
    JSM_TRY(dev_alloc(m, &m->red, Tm * d));
    JSM_TRY(dev_alloc(m, &m->qkv, Tm * m->qkv_dim));
    JSM_TRY(dev_alloc(m, &m->attn, Tm * m->Hq_l * D));
    JSM_TRY(dev_alloc(m, &m->act, Tm * m->ffn_l));
    {
        // fp32 partials of the tiles that several CTAs share: the largest need over the model's projections
        const int Tc = m->max_tokens < 256 ? m->max_tokens : 256;
        size_t need = linear_packed_ws_floats(Tc, m->qkv_dim, d, 0);
        need = std::max(need, linear_packed_ws_floats(Tc, d, qdim, 0));
        need = std::max(need, linear_packed_ws_floats(Tc, m->ffn_l, d, 1));
        need = std::max(need, linear_packed_ws_floats(Tc, d, m->ffn_l, 0));
        need = std::max(need, linear_packed_ws_floats(Tc, c.vocab, d, 0));
        m->ws_floats = need;
        JSM_TRY(dev_alloc(m, &m->partial, m->ws_floats));
        m->n_counters = std::max(1024, std::max((c.vocab + 127) / 128, (m->ffn_l + 63) / 64) + 1);
        JSM_TRY(dev_alloc(m, &m->counters, (size_t)m->n_counters));
        cudaError_t e0 = cudaMemset(m->counters, 0, m->n_counters * sizeof(int));
        if (e0 != cudaSuccess) { jsm_llama_destroy(m); JSM_FAIL(JSM_CUDA, "jsm_llama_create: %s", cudaGetErrorString(e0)); }
    }
    JSM_TRY(dev_alloc(m, &m->ssq0, Tm));
    JSM_TRY(dev_alloc(m, &m->ssq_a, Tm * ((d + 127) / 128)));
    JSM_TRY(dev_alloc(m, &m->ssq_b, Tm * ((d + 127) / 128)));
    if (c.tp_size > 1) {
        const size_t rb = tp_region_bytes(m->max_tokens, d);
        JSM_TRY(dev_alloc(m, &m->tp_region, rb));
        JSM_TRY(dev_alloc(m, &m->tp_state, (size_t)128));  // [0] forward passes; [4..] state of the fused exchanges (a counter, tile epochs)
        if (cudaMemset(m->tp_region, 0, rb) != cudaSuccess || cudaMemset(m->tp_state, 0, 128 * sizeof(int32_t)) != cudaSuccess) {
            jsm_llama_destroy(m);
            JSM_FAIL(JSM_CUDA, "jsm_llama_create: memset of the exchange region failed");
        }
    }
    JSM_TRY(dev_alloc(m, &m->attn_counters, (size_t)c.max_batch * m->Hkv_l));
    if (cudaMemset(m->attn_counters, 0, sizeof(int32_t) * c.max_batch * m->Hkv_l) != cudaSuccess) { jsm_llama_destroy(m); JSM_FAIL(JSM_CUDA, "jsm_llama_create: memset failed"); }
    JSM_TRY(dev_alloc(m, &m->logits, (size_t)c.max_batch * c.vocab));
    JSM_TRY(dev_alloc(m, &m->argmax_key, (size_t)c.max_batch));
    JSM_TRY(dev_alloc(m, &m->argmax_ctr, (size_t)c.max_batch));
    if (cudaMemset(m->argmax_key, 0, sizeof(unsigned long long) * c.max_batch) != cudaSuccess ||
        cudaMemset(m->argmax_ctr, 0, sizeof(int32_t) * c.max_batch) != cudaSuccess) { jsm_llama_destroy(m); JSM_FAIL(JSM_CUDA, "jsm_llama_create: memset failed"); }
    JSM_TRY(dev_alloc(m, &m->best_val, (size_t)c.max_batch));
    JSM_TRY(dev_alloc(m, &m->best_idx, (size_t)c.max_batch));
    JSM_TRY(dev_alloc(m, &m->ids_dev, (size_t)c.max_batch));
    JSM_TRY(dev_alloc(m, &m->prompt_dev, (size_t)m->max_tokens));
    JSM_TRY(dev_alloc(m, &m->next_dev, (size_t)c.max_batch));
    tc_error_word();  // first use allocates the device's error word: do it here, not inside a captured step
    // the chunk length of the decode attention depends on the batch of the step: room for the largest need over 1..max_batch
    m->dec_scratch_bytes = jsm_attn_decode_scratch_bytes_max(c.max_batch, m->Hq_l, D, c.max_context);
    JSM_TRY(dev_alloc(m, &m->dec_scratch, m->dec_scratch_bytes / sizeof(float) + 4));
    cudaError_t e = cudaMemset(m->ctx, 0, sizeof(int32_t) * c.max_batch);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { jsm_llama_destroy(m); JSM_FAIL(JSM_CUDA, "jsm_llama_create: initialisation failed: %s", cudaGetErrorString(e)); }
#undef JSM_TRY
    *out = m;
    return JSM_OK;
}

jsm_status jsm_llama_create(const jsm_model_config* cfg, uint64_t seed, jsm_model** out) { return llama_create_impl(cfg, seed, 0, out); }

jsm_status jsm_llama_create_paged(const jsm_model_config* cfg, uint64_t seed, int n_pages, jsm_model** out) {
    if (n_pages <= 0) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_create_paged: %d pages", n_pages);
    return llama_create_impl(cfg, seed, n_pages, out);
}

jsm_status jsm_llama_destroy(jsm_model* m) {
    if (!m) return JSM_OK;
    cudaDeviceSynchronize();
    for (auto& g : m->step_graphs) cudaGraphExecDestroy(g.second);
    for (void* p : m->allocs) cudaFree(p);
    if (m->unpack_buf) cudaFree(m->unpack_buf);
    delete m;
    return JSM_OK;
}

jsm_status jsm_llama_set_allreduce(jsm_model* m, jsm_allreduce_fn fn, void* user) {
    if (!m) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_set_allreduce: null model");
    m->allreduce = fn;
    m->allreduce_user = user;
    return JSM_OK;
}

jsm_status jsm_llama_tp_region(jsm_model* m, void** d_region, size_t* bytes) {
    if (!m || !d_region || !bytes) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_tp_region: null argument");
    if (!m->tp_region) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_tp_region: the model is not tensor parallel");
    *d_region = m->tp_region;
    *bytes = tp_region_bytes(m->max_tokens, m->c.d_model);
    return JSM_OK;
}

jsm_status jsm_llama_tp_connect(jsm_model* m, void* const* d_peer_regions) {
    if (!m || !d_peer_regions) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_tp_connect: null argument");
    if (!m->tp_region) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_tp_connect: the model is not tensor parallel");
    for (int r = 0; r < m->c.tp_size; ++r) {
        void* p = r == m->c.tp_rank ? static_cast<void*>(m->tp_region) : d_peer_regions[r];
        if (!p) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_tp_connect: no region for rank %d", r);
        m->tp_regions[r] = p;
    }
    m->tp_connected = true;
    return JSM_OK;
}

namespace {
// a named tensor of the rank's shard: either plain (ptr, bytes) or a packed projection (packed, N, K, paired, gain in front)
struct TensorRef {
    void* plain = nullptr;
    size_t plain_bytes = 0;
    bool f32 = false;
    uint8_t* packed = nullptr;
    int N = 0, K = 0, paired = 0;
    const float* gain = nullptr;
};
bool find_tensor(jsm_model* m, const char* name, TensorRef& t) {
    const int d = m->c.d_model, D = m->c.head_dim;
    std::string s(name);
    if (s == "emb") { t.plain = m->emb; t.plain_bytes = (size_t)m->c.vocab * d * 2; return true; }
    if (s == "gf") { t.plain = m->gf; t.plain_bytes = (size_t)d * 4; t.f32 = true; return true; }
    if (s == "lm_head") { t.packed = m->lm_head; t.N = m->c.vocab; t.K = d; t.gain = m->gf; return true; }
    int l = -1;
    char field[32] = "";
    if (sscanf(name, "layers.%d.%31s", &l, field) != 2 || l < 0 || l >= m->c.n_layers) return false;
    jsm::LayerW& L = m->layers[l];
    std::string f(field);
    if (f == "g1") { t.plain = L.g1; t.plain_bytes = (size_t)d * 4; t.f32 = true; return true; }
    if (f == "g2") { t.plain = L.g2; t.plain_bytes = (size_t)d * 4; t.f32 = true; return true; }
    if (f == "wqkv") { t.packed = L.wqkv; t.N = m->qkv_dim; t.K = d; t.gain = L.g1; return true; }
    if (f == "wo") { t.packed = L.wo; t.N = d; t.K = m->Hq_l * D; return true; }
    if (f == "wgu") { t.packed = L.wgu; t.N = m->ffn_l; t.K = d; t.paired = 1; t.gain = L.g2; return true; }
    if (f == "wdown") { t.packed = L.wdown; t.N = d; t.K = m->ffn_l; return true; }
    return false;
}
jsm_status grow_unpack(jsm_model* m, size_t elems) {
    if (elems <= m->unpack_elems) return JSM_OK;
    JSM_CUDA_CHECK(cudaDeviceSynchronize());
    if (m->unpack_buf) cudaFree(m->unpack_buf);
    m->unpack_buf = nullptr; m->unpack_elems = 0;
    JSM_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&m->unpack_buf), elems * sizeof(__nv_bfloat16)));
    m->unpack_elems = elems;
    return JSM_OK;
}
std::vector<std::string> tensor_names(const jsm_model* m) {
    std::vector<std::string> v = {"emb", "gf", "lm_head"};
    for (int l = 0; l < m->c.n_layers; ++l)
        for (const char* f : {"g1", "g2", "wqkv", "wo", "wgu", "wdown"}) v.push_back("layers." + std::to_string(l) + "." + f);
    return v;
}
constexpr char CKPT_MAGIC[8] = {'J', 'S', 'M', 'C', 'K', 'P', 'T', '1'};
}  // namespace

// Weight injection: the reference takes weights through init_t<tag>::cal (mat_init_t.hpp:10-118); here a tensor of the
// rank's shard is replaced from device memory.  Projections arrive row-major [out, in] in bf16 (wgu: gate rows then up
// rows), are multiplied column-wise by the gain of the RMSNorm in front of them (wqkv: g1, wgu: g2, lm_head: gf - the
// kernels apply that norm without a gain) and packed.  So: set a gain before the projection that follows it.
jsm_status jsm_llama_set_weight(jsm_model* m, const char* name, const void* d_src, size_t n_elems, void* stream) {
    if (!m || !name || !d_src) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_set_weight: null argument");
    TensorRef t;
    if (!find_tensor(m, name, t)) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_set_weight: unknown tensor '%s'", name);
    cudaStream_t st = as_stream(stream);
    if (t.plain) {
        const size_t want = t.plain_bytes / (t.f32 ? 4 : 2);
        if (n_elems != want) JSM_FAIL(JSM_SHAPE, "jsm_llama_set_weight: '%s' has %zu elements, got %zu", name, want, n_elems);
        JSM_CUDA_CHECK(cudaMemcpyAsync(t.plain, d_src, t.plain_bytes, cudaMemcpyDeviceToDevice, st));
        return JSM_OK;
    }
    const size_t rows = (size_t)(t.paired ? 2 * t.N : t.N), elems = rows * t.K;
    if (n_elems != elems) JSM_FAIL(JSM_SHAPE, "jsm_llama_set_weight: '%s' has %zu elements, got %zu", name, elems, n_elems);
    jsm_status s = grow_unpack(m, elems);
    if (s != JSM_OK) return s;
    scale_cols_kernel<<<(unsigned)std::min<size_t>((elems + 255) / 256, 148 * 16), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(d_src), m->unpack_buf, (long long)rows, t.K, t.gain);
    JSM_LAUNCH_CHECK();
    return linear_pack_launch(m->unpack_buf, t.N, t.K, t.paired, t.packed, false, st);
}

// Flat binary checkpoint of the rank's tensors in their stored form (packed projections with the gains folded in,
// gains, embedding): magic, the model configuration, then per tensor {u32 name length, name, u64 bytes, bytes}.
// The reference has no serialisation (mat_t.hpp:322-336 prints text only).  Loading checks the configuration.
jsm_status jsm_llama_save(jsm_model* m, const char* path) {
    if (!m || !path) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_save: null argument");
    FILE* f = fopen(path, "wb");
    if (!f) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_save: cannot open '%s'", path);
    JSM_CUDA_CHECK(cudaDeviceSynchronize());
    std::vector<uint8_t> host;
    bool ok = fwrite(CKPT_MAGIC, 1, 8, f) == 8 && fwrite(&m->c, sizeof(m->c), 1, f) == 1;
    for (const std::string& name : tensor_names(m)) {
        if (!ok) break;
        TensorRef t;
        find_tensor(m, name.c_str(), t);
        const void* src = t.plain ? t.plain : t.packed;
        const uint64_t bytes = t.plain ? t.plain_bytes : linear_packed_bytes(t.N, t.K, t.paired);
        host.resize(bytes);
        if (cudaMemcpy(host.data(), src, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) { ok = false; break; }
        const uint32_t nl = (uint32_t)name.size();
        ok = fwrite(&nl, 4, 1, f) == 1 && fwrite(name.data(), 1, nl, f) == nl && fwrite(&bytes, 8, 1, f) == 1 &&
             fwrite(host.data(), 1, bytes, f) == bytes;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) JSM_FAIL(JSM_CUDA, "jsm_llama_save: writing '%s' failed", path);
    return JSM_OK;
}

jsm_status jsm_llama_load(jsm_model* m, const char* path) {
    if (!m || !path) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: null argument");
    FILE* f = fopen(path, "rb");
    if (!f) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: cannot open '%s'", path);
    char magic[8];
    jsm_model_config c;
    if (fread(magic, 1, 8, f) != 8 || memcmp(magic, CKPT_MAGIC, 8) != 0 || fread(&c, sizeof(c), 1, f) != 1) {
        fclose(f);
        JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: '%s' is not a checkpoint of this library", path);
    }
    const jsm_model_config& o = m->c;
    if (c.n_layers != o.n_layers || c.d_model != o.d_model || c.n_heads != o.n_heads || c.n_kv_heads != o.n_kv_heads ||
        c.head_dim != o.head_dim || c.d_ffn != o.d_ffn || c.vocab != o.vocab || c.tp_rank != o.tp_rank || c.tp_size != o.tp_size) {
        fclose(f);
        JSM_FAIL(JSM_SHAPE, "jsm_llama_load: the checkpoint was written by a model of another shape or another tensor-parallel rank");
    }
    JSM_CUDA_CHECK(cudaDeviceSynchronize());
    std::vector<uint8_t> host;
    std::vector<char> nm;
    size_t seen = 0;
    const size_t expect = tensor_names(m).size();
    while (true) {
        uint32_t nl = 0;
        if (fread(&nl, 4, 1, f) != 1) break;  // end of file
        uint64_t bytes = 0;
        nm.assign(nl + 1, 0);
        if (nl > 256 || fread(nm.data(), 1, nl, f) != nl || fread(&bytes, 8, 1, f) != 1) { fclose(f); JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: truncated record"); }
        TensorRef t;
        if (!find_tensor(m, nm.data(), t)) { fclose(f); JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: unknown tensor '%s'", nm.data()); }
        const uint64_t want = t.plain ? t.plain_bytes : linear_packed_bytes(t.N, t.K, t.paired);
        if (bytes != want) { fclose(f); JSM_FAIL(JSM_SHAPE, "jsm_llama_load: '%s' holds %llu bytes, the model %llu", nm.data(), (unsigned long long)bytes, (unsigned long long)want); }
        host.resize(bytes);
        if (fread(host.data(), 1, bytes, f) != bytes) { fclose(f); JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: truncated tensor '%s'", nm.data()); }
        cudaError_t e = cudaMemcpy(t.plain ? t.plain : (void*)t.packed, host.data(), bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { fclose(f); JSM_FAIL(JSM_CUDA, "jsm_llama_load: upload of '%s': %s", nm.data(), cudaGetErrorString(e)); }
        ++seen;
    }
    fclose(f);
    if (seen != expect) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_load: %zu tensors in the file, the model has %zu", seen, expect);
    return JSM_OK;
}

jsm_status jsm_llama_weight(jsm_model* m, const char* name, void** d_ptr, size_t* n_elems) {
    if (!m || !name || !d_ptr || !n_elems) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_weight: null argument");
    const int d = m->c.d_model, D = m->c.head_dim;
    std::string s(name);
    if (s == "emb") { *d_ptr = m->emb; *n_elems = (size_t)m->c.vocab * d; return JSM_OK; }
    if (s == "gf") { *d_ptr = m->gf; *n_elems = d; return JSM_OK; }
    // projection weights live packed: the row-major [out, in] matrix is rebuilt into a buffer of the model that the
    // next call overwrites
    const uint8_t* packed = nullptr;
    int N = 0, K = 0, paired = 0;
    if (s == "lm_head") { packed = m->lm_head; N = m->c.vocab; K = d; }
    int l = -1;
    char field[32] = "";
    if (!packed && sscanf(name, "layers.%d.%31s", &l, field) == 2 && l >= 0 && l < m->c.n_layers) {
        LayerW& L = m->layers[l];
        std::string f(field);
        if (f == "g1") { *d_ptr = L.g1; *n_elems = d; return JSM_OK; }
        if (f == "g2") { *d_ptr = L.g2; *n_elems = d; return JSM_OK; }
        if (f == "wqkv") { packed = L.wqkv; N = m->qkv_dim; K = d; }
        else if (f == "wo") { packed = L.wo; N = d; K = m->Hq_l * D; }
        else if (f == "wgu") { packed = L.wgu; N = m->ffn_l; K = d; paired = 1; }
        else if (f == "wdown") { packed = L.wdown; N = d; K = m->ffn_l; }
    }
    if (!packed) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_weight: unknown tensor '%s'", name);
    const size_t elems = (size_t)(paired ? 2 * N : N) * K;
    if (elems > m->unpack_elems) {
        JSM_CUDA_CHECK(cudaDeviceSynchronize());
        if (m->unpack_buf) cudaFree(m->unpack_buf);
        m->unpack_buf = nullptr; m->unpack_elems = 0;
        JSM_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&m->unpack_buf), elems * sizeof(__nv_bfloat16)));
        m->unpack_elems = elems;
    }
    jsm_status st = linear_pack_launch(m->unpack_buf, N, K, paired, const_cast<uint8_t*>(packed), true, nullptr);
    if (st != JSM_OK) return st;
    JSM_CUDA_CHECK(cudaDeviceSynchronize());
    *d_ptr = m->unpack_buf;
    *n_elems = elems;
    return JSM_OK;
}

jsm_status jsm_llama_prefill(jsm_model* m, const int32_t* d_ids, int seq, int T, int32_t* d_next, float* d_logits_last, void* stream) {
    if (!m || !d_ids) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_prefill: null argument");
    if (seq < 0 || seq >= m->c.max_batch) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_prefill: sequence %d outside 0..%d", seq, m->c.max_batch - 1);
    if (T <= 0 || T > m->max_tokens || T > m->c.max_context) JSM_FAIL(JSM_SHAPE, "jsm_llama_prefill: %d tokens (1..%d)", T, m->max_tokens);
    cudaStream_t st = as_stream(stream);
    iota_kernel<<<(T + 255) / 256, 256, 0, st>>>(m->pos, m->seq_ids, T, seq, 0, m->tp_state);
    JSM_LAUNCH_CHECK();
    jsm_status s = forward_tokens(m, d_ids, T, false, 1, seq, st);
    if (s != JSM_OK) return s;
    set_ctx_kernel<<<1, 1, 0, st>>>(m->ctx, seq, T);
    JSM_LAUNCH_CHECK();
    return logits_and_argmax(m, T - 1, 1, T, d_next ? d_next + seq : nullptr, d_logits_last, st);
}

jsm_status jsm_llama_decode_step(jsm_model* m, const int32_t* d_ids, int batch, int32_t* d_next, float* d_logits, void* stream) {
    if (!m || !d_ids) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_decode_step: null argument");
    if (batch <= 0 || batch > m->c.max_batch) JSM_FAIL(JSM_SHAPE, "jsm_llama_decode_step: batch %d (1..%d)", batch, m->c.max_batch);
    cudaStream_t st = as_stream(stream);
    jsm_status s = forward_tokens(m, d_ids, batch, true, batch, -1, st);  // (positions and context lengths advance in its first launch)
    if (s != JSM_OK) return s;
    return logits_and_argmax(m, 0, batch, batch, d_next, d_logits, st);
}

// The decode step for callers that hold their tokens in HOST memory (the reference's generation loop keeps everything
// on the host, transformer_test.hpp:227-241): ids in, next tokens (and optionally logits) out.  The step itself is
// captured once per batch size into a CUDA graph that the model owns (positions and context lengths live on the device,
// so the same graph serves every step) and replayed: one graph launch instead of ~163 kernel launches per step.
jsm_status jsm_llama_decode_step_host(jsm_model* m, const int32_t* h_ids, int batch, int32_t* h_next, float* h_logits, void* stream) {
    if (!m || !h_ids || !h_next) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_decode_step_host: null argument");
    if (batch <= 0 || batch > m->c.max_batch) JSM_FAIL(JSM_SHAPE, "jsm_llama_decode_step_host: batch %d (1..%d)", batch, m->c.max_batch);
    cudaStream_t st = as_stream(stream);
    if (!st) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_decode_step_host: needs a stream of its own (the legacy default stream cannot be captured)");
    JSM_CUDA_CHECK(cudaMemcpyAsync(m->ids_dev, h_ids, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, st));
    const bool host_allreduce = m->c.tp_size > 1 && !m->tp_connected;  // the hook belongs to the host: run such a step eagerly
    float* lg = h_logits ? m->logits : nullptr;  // tokens only: a tensor-parallel group then shares the lm_head by vocabulary
    if (host_allreduce) {
        jsm_status s = jsm_llama_decode_step(m, m->ids_dev, batch, m->next_dev, lg, st);
        if (s != JSM_OK) return s;
    } else {
        const int key = 2 * batch + (lg ? 1 : 0);  // one graph per batch size and output form
        auto it = m->step_graphs.find(key);
        if (it == m->step_graphs.end()) {
            cudaGraph_t graph = nullptr;
            JSM_CUDA_CHECK(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
            jsm_status s = jsm_llama_decode_step(m, m->ids_dev, batch, m->next_dev, lg, st);
            cudaError_t e = cudaStreamEndCapture(st, &graph);
            if (s != JSM_OK) { if (graph) cudaGraphDestroy(graph); return s; }
            if (e != cudaSuccess) { cudaGetLastError(); JSM_FAIL(JSM_CUDA, "jsm_llama_decode_step_host: stream capture failed: %s", cudaGetErrorString(e)); }
            cudaGraphExec_t exec = nullptr;
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) { cudaGetLastError(); JSM_FAIL(JSM_CUDA, "jsm_llama_decode_step_host: graph instantiation failed: %s", cudaGetErrorString(e)); }
            it = m->step_graphs.emplace(key, exec).first;
        }
        JSM_CUDA_CHECK(cudaGraphLaunch(it->second, st));
    }
    JSM_CUDA_CHECK(cudaMemcpyAsync(h_next, m->next_dev, sizeof(int32_t) * batch, cudaMemcpyDeviceToHost, st));
    if (h_logits) JSM_CUDA_CHECK(cudaMemcpyAsync(h_logits, m->logits, sizeof(float) * (size_t)batch * m->c.vocab, cudaMemcpyDeviceToHost, st));
    JSM_CUDA_CHECK(cudaStreamSynchronize(st));
    return JSM_OK;
}

// ---- continuous batching over the paged cache ----------------------------------------------------------------------
// The reference's generation loop serves one sequence at a time and recomputes it from scratch (transformer_test.hpp:
// 231-239).  Here sequences of different lengths share one decode step; they are admitted and retired between steps.
namespace {
// pages for `positions` cached positions of batch row `row`; uploads the part of the row's block table that changed
jsm_status provision(jsm_model* m, int row, int positions, cudaStream_t st) {
    std::vector<int32_t>& pages = m->row_pages[row];
    const int have = (int)pages.size(), need = (positions + JSM_PAGE_SIZE - 1) / JSM_PAGE_SIZE;
    if (need <= have) return JSM_OK;
    if (need > m->pages_per_seq) JSM_FAIL(JSM_SHAPE, "context overflow: %d positions, the model was created for %d", positions, m->c.max_context);
    if (need - have > (int)m->free_pages.size())
        JSM_FAIL(JSM_OOM, "page pool exhausted: %d pages needed, %zu free of %d", need - have, m->free_pages.size(), m->n_pool_pages);
    for (int i = have; i < need; ++i) {
        pages.push_back(m->free_pages.back());
        m->free_pages.pop_back();
    }
    JSM_CUDA_CHECK(cudaMemcpyAsync(m->block_table + (size_t)row * m->pages_per_seq + have, pages.data() + have, sizeof(int32_t) * (need - have),
                                   cudaMemcpyHostToDevice, st));
    JSM_CUDA_CHECK(cudaStreamSynchronize(st));  // the host vector may be reallocated by the next call
    return JSM_OK;
}
}  // namespace

jsm_status jsm_llama_seq_admit(jsm_model* m, const int32_t* h_prompt, int T, int* row_out, int32_t* h_first_token, float* h_logits_last,
                               void* stream) {
    if (!m || !h_prompt || !row_out) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_seq_admit: null argument");
    if (!m->paged) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_seq_admit: the model was not created with jsm_llama_create_paged");
    if (T <= 0 || T > m->max_tokens || T >= m->c.max_context) JSM_FAIL(JSM_SHAPE, "jsm_llama_seq_admit: %d prompt tokens (1..%d)", T, std::min(m->max_tokens, m->c.max_context - 1));
    if (m->n_active >= m->c.max_batch) JSM_FAIL(JSM_OOM, "jsm_llama_seq_admit: all %d batch rows are in use", m->c.max_batch);
    cudaStream_t st = as_stream(stream);
    const int row = m->n_active;
    jsm_status s = provision(m, row, T, st);
    if (s != JSM_OK) return s;
    JSM_CUDA_CHECK(cudaMemcpyAsync(m->prompt_dev, h_prompt, sizeof(int32_t) * T, cudaMemcpyHostToDevice, st));
    float* lg = h_logits_last ? m->logits : nullptr;
    s = jsm_llama_prefill(m, m->prompt_dev, row, T, m->next_dev, lg, st);
    if (s != JSM_OK) return s;
    if (h_first_token) JSM_CUDA_CHECK(cudaMemcpyAsync(h_first_token, m->next_dev + row, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    if (h_logits_last) JSM_CUDA_CHECK(cudaMemcpyAsync(h_logits_last, m->logits, sizeof(float) * m->c.vocab, cudaMemcpyDeviceToHost, st));
    JSM_CUDA_CHECK(cudaStreamSynchronize(st));
    m->h_ctx[row] = T;
    m->n_active = row + 1;
    *row_out = row;
    return JSM_OK;
}

jsm_status jsm_llama_seq_retire(jsm_model* m, int row, int* moved_from, void* stream) {
    if (!m) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_seq_retire: null model");
    if (!m->paged) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_seq_retire: the model was not created with jsm_llama_create_paged");
    if (row < 0 || row >= m->n_active) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_seq_retire: row %d of %d active", row, m->n_active);
    cudaStream_t st = as_stream(stream);
    for (int32_t p : m->row_pages[row]) m->free_pages.push_back(p);
    m->row_pages[row].clear();
    const int last = m->n_active - 1;
    if (moved_from) *moved_from = -1;
    if (row != last) {
        // the last active row takes the freed place: its block-table row and context length move, its pages do not
        m->row_pages[row] = std::move(m->row_pages[last]);
        m->row_pages[last].clear();
        m->h_ctx[row] = m->h_ctx[last];
        JSM_CUDA_CHECK(cudaMemcpyAsync(m->block_table + (size_t)row * m->pages_per_seq, m->row_pages[row].data(),
                                       sizeof(int32_t) * m->row_pages[row].size(), cudaMemcpyHostToDevice, st));
        JSM_CUDA_CHECK(cudaMemcpyAsync(m->ctx + row, &m->h_ctx[row], sizeof(int32_t), cudaMemcpyHostToDevice, st));
        JSM_CUDA_CHECK(cudaStreamSynchronize(st));
        if (moved_from) *moved_from = last;
    }
    m->h_ctx[last] = 0;
    m->n_active = last;
    return JSM_OK;
}

jsm_status jsm_llama_step_active(jsm_model* m, const int32_t* h_ids, int32_t* h_next, float* h_logits, void* stream) {
    if (!m || !h_ids || !h_next) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_step_active: null argument");
    if (!m->paged) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_step_active: the model was not created with jsm_llama_create_paged");
    if (m->n_active == 0) return JSM_OK;
    cudaStream_t st = as_stream(stream);
    for (int row = 0; row < m->n_active; ++row) {
        if (m->h_ctx[row] >= m->c.max_context) JSM_FAIL(JSM_SHAPE, "context overflow: row %d already holds max_context = %d tokens", row, m->c.max_context);
        jsm_status s = provision(m, row, m->h_ctx[row] + 1, st);
        if (s != JSM_OK) return s;
    }
    jsm_status s = jsm_llama_decode_step_host(m, h_ids, m->n_active, h_next, h_logits, st);
    if (s != JSM_OK) return s;
    for (int row = 0; row < m->n_active; ++row) m->h_ctx[row] += 1;
    return JSM_OK;
}

jsm_status jsm_llama_pool_state(jsm_model* m, int* n_active, int* free_pages, int* total_pages) {
    if (!m) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_pool_state: null model");
    if (n_active) *n_active = m->n_active;
    if (free_pages) *free_pages = m->paged ? (int)m->free_pages.size() : 0;
    if (total_pages) *total_pages = m->n_pool_pages;
    return JSM_OK;
}

jsm_status jsm_llama_set_context(jsm_model* m, int seq, int context_len) {
    if (!m || seq < 0 || seq >= m->c.max_batch || context_len < 0 || context_len > m->c.max_context)
        JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_set_context: sequence %d, length %d", seq, context_len);
    JSM_CUDA_CHECK(cudaMemcpy(m->ctx + seq, &context_len, sizeof(int32_t), cudaMemcpyHostToDevice));
    return JSM_OK;
}

jsm_status jsm_llama_reset(jsm_model* m) {
    if (!m) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_reset: null model");
    JSM_CUDA_CHECK(cudaMemset(m->ctx, 0, sizeof(int32_t) * m->c.max_batch));
    return JSM_OK;
}

jsm_status jsm_llama_step_bytes(jsm_model* m, uint64_t* weight_bytes, uint64_t* kv_bytes_per_token) {
    if (!m) JSM_FAIL(JSM_INVALID_ARG, "jsm_llama_step_bytes: null model");
    // every projection including lm_head is streamed once per step; the embedding table is gathered (one row per token)
    // and is not part of the count
    // (a connected tensor-parallel rank that is asked for tokens only streams its 1/N share of lm_head)
    uint64_t w = m->weight_bytes;
    if (m->c.tp_size > 1 && m->tp_connected) {
        const uint64_t lm = 2ull * (uint64_t)m->c.vocab * m->c.d_model;
        w = w - lm + lm / m->c.tp_size;
    }
    if (weight_bytes) *weight_bytes = w;
    if (kv_bytes_per_token) *kv_bytes_per_token = (uint64_t)m->c.n_layers * 2ull * m->Hkv_l * m->c.head_dim * 2ull;
    return JSM_OK;
}

}  // extern "C"
