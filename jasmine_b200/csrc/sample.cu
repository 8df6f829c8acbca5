// Sampling from the logits of a decode step: temperature, top-k, top-p (nucleus).
//
// The reference has no sampler (its generation loop takes the arg-max, transformer_test.hpp:231-239); this is the
// step after jsm_llama_decode_step for callers that want stochastic decoding.  One CTA of 1024 threads per row:
//   1. the K = top_k (at most 1024) largest logits are found exactly by a radix select over order-preserving 32-bit
//      keys (four passes of 8 bits, histogram in shared memory); ties at the threshold are taken in index order;
//   2. the candidates are sorted by (value descending, index ascending) with a bitonic sort in shared memory;
//   3. p_i = exp((x_i - x_0) / temperature); an inclusive scan gives the cumulative mass; top-p keeps the shortest
//      prefix whose mass reaches top_p of the candidates' total (at least one token);
//   4. u in [0, 1) from the counter-based generator (seed, step, row) selects the first token whose cumulative mass
//      exceeds u times the kept mass.
// temperature <= 0 or top_k == 1 is the arg-max (smallest index on ties).
#include "common.cuh"
#include <math.h>

namespace jsm {

constexpr int SM_THREADS = 1024;
constexpr int SM_MAXK = 1024;

__device__ __forceinline__ uint32_t sample_key(float x) {  // larger float -> larger key; NaN sorts lowest
    if (x != x) return 0u;
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive scan of one int per thread over the CTA (1024 threads); returns the thread's offset, *total = the sum
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();  // warp_sums may still be read from an earlier call
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += n;
        }
        warp_sums[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    *total = warp_sums[31];
    return inc - v + (warp > 0 ? warp_sums[warp - 1] : 0);
}

__global__ void __launch_bounds__(SM_THREADS) sample_rows_kernel(const float* __restrict__ logits, long long row_stride, int V,
                                                                 float inv_temperature, int top_k, float top_p, uint64_t key,
                                                                 int32_t* __restrict__ out) {
    __shared__ int hist[256];
    __shared__ int warp_sums[32];
    __shared__ uint32_t sel_prefix;
    __shared__ int sel_remaining;
    __shared__ float cand_v[SM_MAXK];
    __shared__ int cand_i[SM_MAXK];
    __shared__ float cum[SM_MAXK];
    __shared__ float fwarp[32];
    chain_trigger();
    chain_wait();
    const float* row = logits + (long long)blockIdx.x * row_stride;
    const int tid = threadIdx.x;
    const int K = min(min(top_k <= 0 ? SM_MAXK : top_k, SM_MAXK), V);
    // a thread owns a contiguous range of the row, so that "index order" is thread order
    const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    const int i0 = min(tid * chunk, V), i1 = min(i0 + chunk, V);

    // ---- 1. radix select: the key of the K-th largest element
    if (tid == 0) { sel_prefix = 0u; sel_remaining = K; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = sel_prefix;
        const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        for (int i = i0; i < i1; ++i) {
            const uint32_t k = sample_key(row[i]);
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int rem = sel_remaining, b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= rem) break;
                rem -= hist[b];
            }
            sel_prefix = prefix | ((uint32_t)b << shift);
            sel_remaining = rem;  // how many elements with exactly this prefix are still wanted
        }
        __syncthreads();
    }
    const uint32_t thr = sel_prefix;     // key of the K-th largest
    const int want_eq = sel_remaining;   // elements equal to the threshold that belong to the top K (index order)

    // ---- gather: keys above the threshold, then the first want_eq keys equal to it
    int n_gt = 0, n_eq = 0;
    for (int i = i0; i < i1; ++i) {
        const uint32_t k = sample_key(row[i]);
        n_gt += k > thr;
        n_eq += k == thr;
    }
    int tot_gt, tot_eq;
    int off_gt = block_exclusive_scan(n_gt, warp_sums, &tot_gt);
    int off_eq = block_exclusive_scan(n_eq, warp_sums, &tot_eq);
    for (int i = tid; i < SM_MAXK; i += SM_THREADS) { cand_v[i] = -INFINITY; cand_i[i] = 0x7fffffff; }
    __syncthreads();
    for (int i = i0; i < i1; ++i) {
        const float x = row[i];
        const uint32_t k = sample_key(x);
        if (k > thr) {
            cand_v[off_gt] = x; cand_i[off_gt] = i; ++off_gt;
        } else if (k == thr) {
            if (off_eq < want_eq) { cand_v[tot_gt + off_eq] = x; cand_i[tot_gt + off_eq] = i; }
            ++off_eq;
        }
    }
    __syncthreads();

    // ---- 2. bitonic sort of 1024 (value descending, index ascending); the padding sorts last
    for (int size = 2; size <= SM_MAXK; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int partner = tid ^ stride;
            if (partner > tid) {
                const bool descending = (tid & size) == 0;
                const float a = cand_v[tid], b = cand_v[partner];
                const int ia = cand_i[tid], ib = cand_i[partner];
                const bool a_first = a > b || (a == b && ia < ib);  // a belongs before b
                if (a_first != descending) {
                    cand_v[tid] = b; cand_v[partner] = a;
                    cand_i[tid] = ib; cand_i[partner] = ia;
                }
            }
            __syncthreads();
        }
    }

    // ---- 3. probabilities relative to the largest, inclusive scan
    const float top = cand_v[0];
    float p = tid < K ? expf((cand_v[tid] - top) * inv_temperature) : 0.0f;
    {
        const int lane = tid & 31, warp = tid >> 5;
        float inc = p;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) fwarp[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            float w = fwarp[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += n;
            }
            fwarp[lane] = w;
        }
        __syncthreads();
        cum[tid] = inc + (warp > 0 ? fwarp[warp - 1] : 0.0f);
    }
    __syncthreads();
    const float total = cum[K - 1];
    // ---- top-p: n_keep = 1 + number of positions whose cumulative mass stays below top_p * total
    const float cut = top_p * total;
    int below = (tid < K - 1 && cum[tid] < cut) ? 1 : 0;
    int n_below;
    block_exclusive_scan(below, warp_sums, &n_below);
    const int n_keep = (top_p >= 1.0f) ? K : min(K, n_below + 1);
    // ---- 4. the draw
    const float u = rng_uniform01(key, (uint64_t)blockIdx.x);
    const float target = u * cum[n_keep - 1];
    int before = (tid < n_keep - 1 && cum[tid] <= target) ? 1 : 0;
    int pos;
    block_exclusive_scan(before, warp_sums, &pos);
    if (tid == 0) out[blockIdx.x] = cand_i[min(pos, n_keep - 1)];
}

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_sample(const float* d_logits, int64_t row_stride, int n_rows, int vocab, float temperature, int top_k,
                                 float top_p, uint64_t seed, uint64_t step, int32_t* d_out, void* stream) {
    if (n_rows == 0) return JSM_OK;
    if (!d_logits || !d_out) JSM_FAIL(JSM_INVALID_ARG, "jsm_sample: null pointer");
    if (vocab <= 0 || n_rows < 0 || row_stride < vocab) JSM_FAIL(JSM_SHAPE, "jsm_sample: %d rows of %d logits, row stride %lld", n_rows, vocab, (long long)row_stride);
    if (!(top_p > 0.0f) || top_p > 1.0f) JSM_FAIL(JSM_INVALID_ARG, "jsm_sample: top_p %g outside (0, 1]", (double)top_p);
    if (top_k < 0) JSM_FAIL(JSM_INVALID_ARG, "jsm_sample: top_k %d", top_k);
    const bool greedy = !(temperature > 0.0f) || top_k == 1;
    JSM_CUDA_CHECK(launch_chained(sample_rows_kernel, dim3(n_rows), dim3(SM_THREADS), 0, as_stream(stream), d_logits, (long long)row_stride,
                                  vocab, greedy ? 1.0f : 1.0f / temperature, greedy ? 1 : top_k, greedy ? 1.0f : top_p,
                                  rng_key(seed, step), d_out));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}
