// Paged KV cache: append and split-K decode attention.
//
// The reference has no cache: generation recomputes the whole prefix for every
// token (transformer_test.hpp:227-241).  Here K (already rotated) and V of every
// position are kept in pages of 64 tokens, pool layout
// [page][K|V][kv_head][token in page][head_dim] bf16, and one decode step reads
// each cached byte once.  The arithmetic per (sequence, head) is the row of
// mat_head_gen_t::forward (mat_mha_t.hpp:53-71) for the newest query:
// scores = q.k * scale, softmax over the context, weighted sum of V.
//
// Decode kernel: grid (context chunk, kv head, sequence).  A CTA of 4 warps
// streams its chunk of K and V with 128-bit loads (16 lanes per key, two keys per
// warp load), all G = Hq/Hkv query heads of the group share every loaded byte,
// and the running (max, sum, weighted V) is kept per warp, merged through shared
// memory and written as one partial per chunk; a second kernel merges the
// partials of a sequence.
#include "attn.cuh"
#include <math.h>
#include <mutex>
#include <stdlib.h>

namespace jsm {

constexpr int DEC_CHUNK_MAX = 512;  // context positions per CTA at large batch
constexpr int DEC_WARPS = 4;
constexpr int DEC_UNROLL = 4;    // warp loads of K (and V) in flight per step: 8 keys
constexpr float LOG2E = 1.4426950408889634f;

// Context positions per CTA: small batches get short chunks so that the grid still fills the GPU
// (chunks x kv heads x sequences CTAs); always a multiple of the 32 positions a CTA covers per step.
inline int decode_chunk(int n_seqs, int Hq) {
    const int work = n_seqs * Hq;
    return work >= 512 ? DEC_CHUNK_MAX : work >= 128 ? 256 : work >= 32 ? 128 : 64;
}

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
    f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
    f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}

// ---- append ----------------------------------------------------------------------
__global__ void __launch_bounds__(128) kv_append_kernel(__nv_bfloat16* __restrict__ pool, const int32_t* __restrict__ block_table,
                                                        int max_pages, const __nv_bfloat16* __restrict__ k,
                                                        const __nv_bfloat16* __restrict__ v, long long row_stride,
                                                        const int32_t* __restrict__ seq_ids, const int32_t* __restrict__ positions,
                                                        int Hkv, int D, const float4* __restrict__ rope) {
    chain_trigger();
    chain_wait();
    const int t = blockIdx.x, hk = blockIdx.y;
    const int seq = seq_ids ? seq_ids[t] : 0;
    const int pos = positions[t];
    const int page = block_table[(long long)seq * max_pages + pos / JSM_PAGE_SIZE];
    const long long page_elems = 2ll * Hkv * JSM_PAGE_SIZE * D;
    __nv_bfloat16* kdst = pool + page * page_elems + ((long long)hk * JSM_PAGE_SIZE + pos % JSM_PAGE_SIZE) * D;
    __nv_bfloat16* vdst = kdst + (long long)Hkv * JSM_PAGE_SIZE * D;
    const __nv_bfloat16* ksrc = k + t * row_stride + (long long)hk * D;
    const __nv_bfloat16* vsrc = v + t * row_stride + (long long)hk * D;
    const int half = D / 2;
    for (int pr = threadIdx.x; pr < half; pr += blockDim.x) {
        uint32_t kw = *reinterpret_cast<const uint32_t*>(ksrc + 2 * pr);
        if (rope) {
            const float4 e = rope[(long long)pos * half + pr];
            const float x0 = bf16lo(kw), x1 = bf16hi(kw);
            kw = pack_bf16x2(__fadd_rn(__fmul_rn(e.x, x0), __fmul_rn(-e.w, x1)), __fadd_rn(__fmul_rn(e.y, x0), __fmul_rn(e.z, x1)));
        }
        *reinterpret_cast<uint32_t*>(kdst + 2 * pr) = kw;
        *reinterpret_cast<uint32_t*>(vdst + 2 * pr) = *reinterpret_cast<const uint32_t*>(vsrc + 2 * pr);
    }
}

// ---- decode: one partial per (sequence, kv head, chunk) -------------------------------
// scratch: [n_seqs][Hq][n_chunks][D + 2] floats: o[D] (unnormalised), m (log2 domain), l
// FUSED: the kernel also (a) appends the new token's K (rotated) and V of this (sequence, kv head) to the cache - the
// CTA whose chunk holds position ctx-1 writes them before it reads its chunk - and (b) merges the chunk partials
// itself: the CTA that arrives last at the (sequence, kv head) counter combines them and writes the output, so that a
// decode step needs one attention launch instead of three.
template <int G, bool FUSED>
__global__ void __launch_bounds__(DEC_WARPS * 32) attn_decode_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ pool,
    const int32_t* __restrict__ block_table, int max_pages, const int32_t* __restrict__ context_lens, int Hq, int Hkv,
    float scale_log2, const float4* __restrict__ rope, int n_chunks, int chunk_len, float* __restrict__ scratch,
    const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new, long long kv_new_stride,
    int* __restrict__ counters, __nv_bfloat16* __restrict__ out) {
    constexpr int D = 128;
    chain_trigger();
    chain_wait();
    const int chunk = blockIdx.x, hk = blockIdx.y, seq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c_begin = chunk * chunk_len;
    // The loads that do not depend on one another go out together: the context length, the page of the chunk's first
    // keys (read before the length is known: the entry exists whatever it holds, it is used only if the chunk has keys)
    // and the raw query heads.  One memory round trip instead of three on the way to the first K/V rows.
    const int32_t* bt = block_table + (long long)seq * max_pages;
    const int ks = lane >> 4;          // which of the two keys of a warp load
    const int dsub = (lane & 15) * 8;  // this lane's 8 dims
    const int first_base = c_begin + warp * (2 * DEC_UNROLL);
    const int page_first = first_base / JSM_PAGE_SIZE < max_pages ? bt[first_base / JSM_PAGE_SIZE] : 0;
    uint4 q_raw[G];
#pragma unroll
    for (int g = 0; g < G; ++g) q_raw[g] = *reinterpret_cast<const uint4*>(q + seq * q_stride + (long long)(hk * G + g) * D + dsub);
    const int ctx = context_lens[seq];
    if (c_begin >= ctx) return;
    const int c_end = min(ctx, c_begin + chunk_len);
    if (FUSED && k_new && ctx - 1 >= c_begin) {  // ctx - 1 < c_end always: this CTA owns the newest position
        const int pos = ctx - 1;
        if (threadIdx.x < D / 2) {
            const int pr = threadIdx.x;
            const int page = block_table[(long long)seq * max_pages + pos / JSM_PAGE_SIZE];
            __nv_bfloat16* kdst = pool + page * (2ll * Hkv * JSM_PAGE_SIZE * D) + ((long long)hk * JSM_PAGE_SIZE + pos % JSM_PAGE_SIZE) * D;
            __nv_bfloat16* vdst = kdst + (long long)Hkv * JSM_PAGE_SIZE * D;
            uint32_t kw = *reinterpret_cast<const uint32_t*>(k_new + seq * kv_new_stride + (long long)hk * D + 2 * pr);
            if (rope) {
                const float4 e = rope[(long long)pos * (D / 2) + pr];
                const float x0 = bf16lo(kw), x1 = bf16hi(kw);
                kw = pack_bf16x2(__fadd_rn(__fmul_rn(e.x, x0), __fmul_rn(-e.w, x1)), __fadd_rn(__fmul_rn(e.y, x0), __fmul_rn(e.z, x1)));
            }
            *reinterpret_cast<uint32_t*>(kdst + 2 * pr) = kw;
            *reinterpret_cast<uint32_t*>(vdst + 2 * pr) = *reinterpret_cast<const uint32_t*>(v_new + seq * kv_new_stride + (long long)hk * D + 2 * pr);
        }
        __syncthreads();  // the chunk loop below reads what was just written
    }
    const long long page_elems = 2ll * Hkv * JSM_PAGE_SIZE * D;
    const long long v_off = (long long)Hkv * JSM_PAGE_SIZE * D;
    constexpr int STEP = 2 * DEC_UNROLL;  // keys per warp step

    // the K and V rows of one warp step (8 keys); the next step's rows are requested before this step's arithmetic so that
    // the memory round trips of consecutive steps overlap
    auto fetch_page = [&](int base, int page, uint4 (&kw)[DEC_UNROLL], uint4 (&vw)[DEC_UNROLL]) {
        const __nv_bfloat16* kp = pool + page * page_elems + ((long long)hk * JSM_PAGE_SIZE + base % JSM_PAGE_SIZE) * D;
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            const int key = base + 2 * u + ks;
            if (key < c_end) {
                kw[u] = __ldcs(reinterpret_cast<const uint4*>(kp + (long long)(2 * u + ks) * D + dsub));
                vw[u] = __ldcs(reinterpret_cast<const uint4*>(kp + v_off + (long long)(2 * u + ks) * D + dsub));
            } else {
                kw[u] = make_uint4(0, 0, 0, 0);
                vw[u] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto fetch = [&](int base, uint4 (&kw)[DEC_UNROLL], uint4 (&vw)[DEC_UNROLL]) {
        if (base < c_end) fetch_page(base, bt[base / JSM_PAGE_SIZE], kw, vw);
    };
    uint4 kw[DEC_UNROLL], vw[DEC_UNROLL], kw_next[DEC_UNROLL], vw_next[DEC_UNROLL];
#pragma unroll
    for (int u = 0; u < DEC_UNROLL; ++u) kw_next[u] = vw_next[u] = make_uint4(0, 0, 0, 0);
    // the first rows are requested before the queries are rotated: the table entries of the rotation arrive meanwhile
    if (first_base < c_end) fetch_page(first_base, page_first, kw_next, vw_next);

    // query heads of the group, this lane's 8 dims, pre-scaled into the log2 domain
    float qf[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        unpack8(q_raw[g], qf[g]);
        if (rope) {
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float4 e = rope[(long long)(ctx - 1) * (D / 2) + dsub / 2 + p];
                const float x0 = qf[g][2 * p], x1 = qf[g][2 * p + 1];
                // rounded to bf16 like a stored, rotated q would be
                const uint32_t pk = pack_bf16x2(__fadd_rn(__fmul_rn(e.x, x0), __fmul_rn(-e.w, x1)),
                                                __fadd_rn(__fmul_rn(e.y, x0), __fmul_rn(e.z, x1)));
                qf[g][2 * p] = bf16lo(pk);
                qf[g][2 * p + 1] = bf16hi(pk);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[g][i] *= scale_log2;
    }

    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    }
    for (int base = c_begin + warp * STEP; base < c_end; base += DEC_WARPS * STEP) {
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) { kw[u] = kw_next[u]; vw[u] = vw_next[u]; }
        fetch(base + DEC_WARPS * STEP, kw_next, vw_next);
        float s[DEC_UNROLL][G];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float kf[8];
            unpack8(kw[u], kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float d = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(qf[g][i], kf[i], d);
                s[u][g] = d;
            }
        }
        // sum over the 16 lanes that share a key
#pragma unroll
        for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u)
#pragma unroll
                for (int g = 0; g < G; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], o);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                if (base + 2 * u + ks >= c_end) s[u][g] = -INFINITY;
                mx = fmaxf(mx, s[u][g]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m[g], mx);  // finite: key `base` is always valid
            const float corr = exp2f(m[g] - m_new);
            m[g] = m_new;
            l[g] *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] *= corr;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                const float p = exp2f(s[u][g] - m_new);
                s[u][g] = p;
                l[g] += p;
            }
        }
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float vf[8];
            unpack8(vw[u], vf);
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(s[u][g], vf[i], acc[g][i]);
        }
    }
    // the two key slots of the warp hold disjoint keys under the same running max: add them
#pragma unroll
    for (int g = 0; g < G; ++g) {
        l[g] += __shfl_xor_sync(0xffffffffu, l[g], 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] += __shfl_xor_sync(0xffffffffu, acc[g][i], 16);
    }
    // merge the warps of the CTA
    __shared__ float sm_m[DEC_WARPS][G], sm_l[DEC_WARPS][G];
    __shared__ float sm_o[DEC_WARPS][G][D];
    if (ks == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sm_o[warp][g][dsub + i] = acc[g][i];
            if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * D; e += DEC_WARPS * 32) {
        const int g = e / D, d = e % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][g]);
        float o = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = sm_m[w][g] == -INFINITY ? 0.0f : exp2f(sm_m[w][g] - M);
            o += f * sm_o[w][g][d];
            L += f * sm_l[w][g];
        }
        float* dst = scratch + (((long long)seq * Hq + hk * G + g) * n_chunks + chunk) * (D + 2);
        if (FUSED && ctx <= chunk_len) {
            // a single chunk: this is the result
            out[((long long)seq * Hq + hk * G + g) * D + d] = __float2bfloat16_rn(o / L);
        } else {
            dst[d] = o;
            if (d == 0) { dst[D] = M; dst[D + 1] = L; }
        }
    }
    if (!FUSED || ctx <= chunk_len) return;
    // ---- the last CTA of this (sequence, kv head) merges the chunk partials
    __shared__ int is_last;
    __syncthreads();  // all partial stores of the CTA precede the release below
    if (threadIdx.x == 0) {
        const int n_valid = (ctx + chunk_len - 1) / chunk_len;
        int old;
        int* ctr = counters + (long long)seq * Hkv + hk;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(ctr) : "memory");
        is_last = (old == n_valid - 1);
        if (is_last) *ctr = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    const int n = (ctx + chunk_len - 1) / chunk_len;
    for (int e = threadIdx.x; e < G * D; e += DEC_WARPS * 32) {
        const int g = e / D, d = e % D;
        const float* src = scratch + ((long long)seq * Hq + hk * G + g) * n_chunks * (D + 2);
        float M = -INFINITY;
        for (int c = 0; c < n; ++c) M = fmaxf(M, __ldcg(src + c * (D + 2) + D));
        float o = 0.0f, L = 0.0f;
        for (int c = 0; c < n; ++c) {
            const float f = exp2f(__ldcg(src + c * (D + 2) + D) - M);
            o += f * __ldcg(src + c * (D + 2) + d);
            L += f * __ldcg(src + c * (D + 2) + D + 1);
        }
        out[((long long)seq * Hq + hk * G + g) * D + d] = __float2bfloat16_rn(o / L);
    }
}

// merge the chunk partials of one (sequence, query head): 128 threads, one per dim
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const float* __restrict__ scratch,
                                                                const int32_t* __restrict__ context_lens, int Hq, int n_chunks,
                                                                int chunk_len, __nv_bfloat16* __restrict__ out) {
    constexpr int D = 128;
    chain_trigger();
    chain_wait();
    const int h = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
    const int n = (context_lens[seq] + chunk_len - 1) / chunk_len;
    const float* src = scratch + ((long long)seq * Hq + h) * n_chunks * (D + 2);
    float M = -INFINITY;
    for (int c = 0; c < n; ++c) M = fmaxf(M, src[c * (D + 2) + D]);
    float o = 0.0f, L = 0.0f;
    for (int c = 0; c < n; ++c) {
        const float f = exp2f(src[c * (D + 2) + D] - M);
        o += f * src[c * (D + 2) + d];
        L += f * src[c * (D + 2) + D + 1];
    }
    out[((long long)seq * Hq + h) * D + d] = __float2bfloat16_rn(n > 0 ? o / L : 0.0f);
}

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_kv_append(void* d_pool, const int32_t* d_block_table, int max_pages, const void* d_k, const void* d_v,
                                    int64_t kv_row_stride, const int32_t* d_seq_ids, const int32_t* d_positions, int T, int Hkv,
                                    int D, const float* d_rope_table, void* stream) {
    if (T == 0) return JSM_OK;
    if (!d_pool || !d_block_table || !d_k || !d_v || !d_positions) JSM_FAIL(JSM_INVALID_ARG, "jsm_kv_append: null pointer");
    if (D <= 0 || D % 2 || Hkv <= 0 || max_pages <= 0) JSM_FAIL(JSM_SHAPE, "jsm_kv_append: Hkv %d D %d max_pages %d", Hkv, D, max_pages);
    dim3 grid(T, Hkv);
    JSM_CUDA_CHECK(launch_chained(kv_append_kernel, grid, dim3(64), 0, as_stream(stream), (__nv_bfloat16*)d_pool, d_block_table, max_pages,
                                  (const __nv_bfloat16*)d_k, (const __nv_bfloat16*)d_v, (long long)kv_row_stride, d_seq_ids, d_positions,
                                  Hkv, D, (const float4*)d_rope_table));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

extern "C" size_t jsm_attn_decode_scratch_bytes(int n_seqs, int Hq, int D, int max_context) {
    if (n_seqs <= 0 || Hq <= 0 || D <= 0 || max_context <= 0) return 0;
    const int chunk = decode_chunk(n_seqs, Hq);
    const size_t n_chunks = (size_t)(max_context + chunk - 1) / chunk;
    return (size_t)n_seqs * Hq * n_chunks * (D + 2) * sizeof(float);
}

// The chunk length shrinks with the number of sequences of a call (short chunks keep the grid full), so the bytes a
// call needs are not monotone in n_seqs: a buffer that serves every call of 1..max_seqs sequences takes the maximum.
extern "C" size_t jsm_attn_decode_scratch_bytes_max(int max_seqs, int Hq, int D, int max_context) {
    size_t need = 0;
    for (int n = 1; n <= max_seqs; ++n) {
        const size_t b = jsm_attn_decode_scratch_bytes(n, Hq, D, max_context);
        if (b > need) need = b;
    }
    return need;
}

static jsm_status attn_decode_launch(const void* d_q, int64_t q_row_stride, void* d_pool, const int32_t* d_block_table, int max_pages,
                                     const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D, float scale,
                                     const float* d_rope_table, int max_context, void* d_scratch, void* d_out, const void* d_k_new,
                                     const void* d_v_new, int64_t kv_new_stride, int* d_counters, bool fused, void* stream,
                                     const char* who, size_t scratch_capacity) {
    if (n_seqs == 0) return JSM_OK;
    if (!d_q || !d_pool || !d_block_table || !d_context_lens || !d_scratch || !d_out) JSM_FAIL(JSM_INVALID_ARG, "%s: null pointer", who);
    if (D != 128) JSM_FAIL(JSM_UNSUPPORTED, "%s: head_dim %d (128 only)", who, D);
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) JSM_FAIL(JSM_SHAPE, "d_model must be divisible by num_heads (Hq %d, Hkv %d)", Hq, Hkv);
    if (max_context <= 0 || (q_row_stride % 8)) JSM_FAIL(JSM_INVALID_ARG, "%s: max_context %d, q stride %lld", who, max_context, (long long)q_row_stride);
    if (fused && !d_counters) JSM_FAIL(JSM_INVALID_ARG, "%s: null counters", who);
    if (fused && d_k_new && (!d_v_new || kv_new_stride % 2)) JSM_FAIL(JSM_INVALID_ARG, "%s: new K without V, or an odd row stride", who);
    const int G = Hq / Hkv;
    const int chunk = decode_chunk(n_seqs, Hq);
    const int n_chunks = (max_context + chunk - 1) / chunk;
    const size_t need = (size_t)n_seqs * Hq * n_chunks * (D + 2) * sizeof(float);
    if (need > scratch_capacity)
        JSM_FAIL(JSM_INVALID_ARG, "%s: %d sequences x %d heads x context %d write %zu bytes of partials, the scratch buffer holds %zu", who,
                 n_seqs, Hq, max_context, need, scratch_capacity);
    dim3 grid(n_chunks, Hkv, n_seqs);
    cudaStream_t st = as_stream(stream);
    const float sl2 = scale * LOG2E;
#define JSM_DEC(GG, FF)                                                                                                          \
    JSM_CUDA_CHECK(launch_chained(attn_decode_kernel<GG, FF>, grid, dim3(DEC_WARPS * 32), 0, st, (const __nv_bfloat16*)d_q,       \
                                  (long long)q_row_stride, (__nv_bfloat16*)d_pool, d_block_table, max_pages, d_context_lens, Hq,  \
                                  Hkv, sl2, (const float4*)d_rope_table, n_chunks, chunk, (float*)d_scratch,                      \
                                  (const __nv_bfloat16*)d_k_new, (const __nv_bfloat16*)d_v_new, (long long)kv_new_stride,         \
                                  d_counters, (__nv_bfloat16*)d_out))
    const DecodeMmaArgs mma_args = {d_q, (long long)q_row_stride, d_pool, d_block_table, max_pages, d_context_lens, n_seqs, Hq, Hkv, sl2,
                                    d_rope_table, n_chunks, chunk, (float*)d_scratch, fused, d_k_new, d_v_new,
                                    (long long)kv_new_stride, d_counters, d_out};
    if (fused && attn_decode_mma_usable(G, chunk, d_pool)) return attn_decode_mma_launch(mma_args, st);
    if (fused) {
        switch (G) {
            case 1: JSM_DEC(1, true); break;
            case 2: JSM_DEC(2, true); break;
            case 4: JSM_DEC(4, true); break;
            case 8: JSM_DEC(8, true); break;
            default: JSM_FAIL(JSM_UNSUPPORTED, "%s: %d query heads per kv head (1, 2, 4 or 8)", who, G);
        }
        JSM_LAUNCH_CHECK();
        return JSM_OK;
    }
    if (attn_decode_mma_usable(G, chunk, d_pool)) {
        jsm_status s = attn_decode_mma_launch(mma_args, st);
        if (s != JSM_OK) return s;
    } else
    switch (G) {
        case 1: JSM_DEC(1, false); break;
        case 2: JSM_DEC(2, false); break;
        case 4: JSM_DEC(4, false); break;
        case 8: JSM_DEC(8, false); break;
        default: JSM_FAIL(JSM_UNSUPPORTED, "%s: %d query heads per kv head (1, 2, 4 or 8)", who, G);
    }
#undef JSM_DEC
    JSM_LAUNCH_CHECK();
    JSM_CUDA_CHECK(launch_chained(attn_decode_merge_kernel, dim3(Hq, n_seqs), dim3(128), 0, st, (const float*)d_scratch, d_context_lens,
                                  Hq, n_chunks, chunk, (__nv_bfloat16*)d_out));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

extern "C" jsm_status jsm_attn_decode(const void* d_q, int64_t q_row_stride, const void* d_pool, const int32_t* d_block_table,
                                      int max_pages, const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D, float scale,
                                      const float* d_rope_table, int max_context, void* d_scratch, void* d_out, void* stream) {
    return attn_decode_launch(d_q, q_row_stride, const_cast<void*>(d_pool), d_block_table, max_pages, d_context_lens, n_seqs, Hq, Hkv, D,
                              scale, d_rope_table, max_context, d_scratch, d_out, nullptr, nullptr, 0, nullptr, false, stream,
                              "jsm_attn_decode", SIZE_MAX);
}

namespace jsm {
// the decoder runner's call: the capacity of its scratch buffer is checked against what this batch size writes
jsm_status attn_decode_append_checked(const void* d_q, int64_t q_row_stride, const void* d_k_new, const void* d_v_new,
                                      int64_t kv_new_stride, void* d_pool, const int32_t* d_block_table, int max_pages,
                                      const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D, float scale,
                                      const float* d_rope_table, int max_context, void* d_scratch, size_t scratch_bytes,
                                      int32_t* d_counters, void* d_out, void* stream) {
    return attn_decode_launch(d_q, q_row_stride, d_pool, d_block_table, max_pages, d_context_lens, n_seqs, Hq, Hkv, D, scale,
                              d_rope_table, max_context, d_scratch, d_out, d_k_new, d_v_new, kv_new_stride, d_counters, true, stream,
                              "jsm_llama_decode_step", scratch_bytes);
}
}  // namespace jsm

extern "C" jsm_status jsm_attn_decode_append(const void* d_q, int64_t q_row_stride, const void* d_k_new, const void* d_v_new,
                                             int64_t kv_new_stride, void* d_pool, const int32_t* d_block_table, int max_pages,
                                             const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D, float scale,
                                             const float* d_rope_table, int max_context, void* d_scratch, int32_t* d_counters,
                                             void* d_out, void* stream) {
    return attn_decode_launch(d_q, q_row_stride, d_pool, d_block_table, max_pages, d_context_lens, n_seqs, Hq, Hkv, D, scale,
                              d_rope_table, max_context, d_scratch, d_out, d_k_new, d_v_new, kv_new_stride, d_counters, true, stream,
                              "jsm_attn_decode_append", SIZE_MAX);
}

// ---- decode attention that allocates nothing ---------------------------------------------------------
// The chunk partials go to a fixed array in the library image.  In host code the array's name is only a
// stand-in for the symbol: the address a kernel can use is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached.
static __device__ __align__(256) float g_decode_static_scratch[JSM_ATTN_DECODE_STATIC_SCRATCH_BYTES / sizeof(float)];

extern "C" jsm_status jsm_attn_decode_static_scratch(const void* d_q, int64_t q_row_stride, const void* d_pool,
                                                     const int32_t* d_block_table, int max_pages, const int32_t* d_context_lens,
                                                     int n_seqs, int Hq, int Hkv, int D, float scale, const float* d_rope_table,
                                                     int max_context, void* d_out, void* stream) {
    if (n_seqs == 0) return JSM_OK;
    const size_t need = jsm_attn_decode_scratch_bytes(n_seqs, Hq, D, max_context);
    if (need == 0) JSM_FAIL(JSM_INVALID_ARG, "jsm_attn_decode_static_scratch: n_seqs %d, Hq %d, D %d, max_context %d", n_seqs, Hq, D, max_context);
    if (need > (size_t)JSM_ATTN_DECODE_STATIC_SCRATCH_BYTES)
        JSM_FAIL(JSM_UNSUPPORTED,
                 "jsm_attn_decode_static_scratch: %d sequences x %d heads x context %d need %zu bytes of partials, the built-in array "
                 "holds %u; use jsm_attn_decode with a caller-supplied buffer",
                 n_seqs, Hq, max_context, need, (unsigned)JSM_ATTN_DECODE_STATIC_SCRATCH_BYTES);
    static std::mutex mu;
    static float* addr[64] = {nullptr};
    int dev = -1;
    JSM_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) JSM_FAIL(JSM_UNSUPPORTED, "jsm_attn_decode_static_scratch: device index %d", dev);
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!addr[dev]) {
            void* p = nullptr;
            JSM_CUDA_CHECK(cudaGetSymbolAddress(&p, g_decode_static_scratch));
            addr[dev] = reinterpret_cast<float*>(p);
        }
        scratch = addr[dev];
    }
    return jsm_attn_decode(d_q, q_row_stride, d_pool, d_block_table, max_pages, d_context_lens, n_seqs, Hq, Hkv, D, scale,
                           d_rope_table, max_context, scratch, d_out, stream);
}
