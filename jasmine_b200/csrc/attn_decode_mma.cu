// Decode attention over the paged KV cache for grouped-query models (2, 4 or 8 query heads per kv head).
//
// Same arithmetic and the same partial format as attn_decode_kernel (kv_cache.cu): per (sequence, kv head, context
// chunk) the scores q.k * scale of the newest query of every head of the group, an online softmax in the log2 domain
// and the weighted sum of V; one (o[128], max, sum) partial per chunk and query head.  With several query heads per
// cached byte the CUDA-core kernel is bound by instruction issue, not by memory, so here the two contractions run on
// the tensor cores and the cache is staged by TMA:
//   * a producer thread copies one page of the chunk per stage - the [64 keys x 128 dims] K block and V block of this
//     kv head, four 128-byte-swizzled [64 x 64] boxes, 32 KB - into a ring of three stages guarded by mbarriers;
//   * each of four warps owns 16 keys of the stage.  Scores, transposed: S^T[16 keys x 8 heads] = K[16 x 128] . Q^T
//     with the keys as the M dimension of mma.m16n8k16 (A from ldmatrix over the swizzled K block, B = the rotated
//     query heads, kept in registers), so that the 8 columns are the heads of the group and no row is padding;
//   * softmax over the keys (the rows) with three shuffles per head pair; P^T goes from accumulator to B-operand
//     layout through movmatrix;
//   * O^T[128 dims x 8 heads] += V^T[128 x 16 keys] . P^T, A from ldmatrix.trans over the V block.
// Keys past the context length are masked to -inf and their V rows are zeroed in shared memory first (a page past the
// context holds whatever was there before: 0 x NaN must not reach the sum).
// Every mbarrier wait is bounded (tc_utils.cuh); on a timeout the kernel records an error code and returns.
#include "attn.cuh"
#include "tc_utils.cuh"
#include <math.h>

namespace jsm {

using namespace tc;

constexpr int DM_D = 128;
constexpr int DM_PAGE = JSM_PAGE_SIZE;  // 64 keys per stage
constexpr int DM_STAGES = 3;
constexpr int DM_TILE_BYTES = 8192;                // [64 keys][64 dims] bf16, 128-byte swizzle
constexpr int DM_STAGE_BYTES = 4 * DM_TILE_BYTES;  // K dims 0-63 | K dims 64-127 | V dims 0-63 | V dims 64-127
constexpr int DM_CWARPS = 4;
constexpr int DM_THREADS = (DM_CWARPS + 1) * 32;
constexpr int DM_SMEM = DM_STAGES * DM_STAGE_BYTES + 1024;
constexpr int DM_ERR_FULL = 41, DM_ERR_EMPTY = 42;
static_assert(DM_PAGE == 64, "one stage is one page of 64 tokens");

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
// d += a[16x16] . b[16x8], bf16 operands, fp32 accumulators
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// the cache as a matrix of 128-wide rows: row of the first key of block (page, K or V, kv head)
__device__ __forceinline__ int dm_block_row(int page, int kv, int Hkv, int hk) { return ((page * 2 + kv) * Hkv + hk) * DM_PAGE; }

// FUSED: like attn_decode_kernel<G, true> the kernel first appends the new token's K (rotated) and V - the CTA whose
// chunk holds position ctx-1 writes them, then orders those writes before its bulk copies with a proxy fence - and the
// CTA that arrives last at the (sequence, kv head) counter merges the chunk partials and writes the output.
template <int G, bool FUSED>
__global__ void __launch_bounds__(DM_THREADS) attn_decode_mma_kernel(
    const __grid_constant__ CUtensorMap tmap, const __nv_bfloat16* __restrict__ q, long long q_stride,
    __nv_bfloat16* __restrict__ pool, const int32_t* __restrict__ block_table, int max_pages,
    const int32_t* __restrict__ context_lens, int Hq, int Hkv, float scale_log2, const float4* __restrict__ rope, int n_chunks,
    int chunk_len, float* __restrict__ scratch, const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
    long long kv_new_stride, int* __restrict__ counters, __nv_bfloat16* __restrict__ out, int* err) {
    extern __shared__ uint8_t dm_dyn[];
    uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dm_dyn) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[DM_STAGES], empty_bar[DM_STAGES];
    __shared__ int abort_flag;
    __shared__ float sm_m[DM_CWARPS][8], sm_l[DM_CWARPS][8];
    chain_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < DM_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], DM_CWARPS);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    chain_wait();
    const int chunk = blockIdx.x, hk = blockIdx.y, seq = blockIdx.z;
    const int ctx = context_lens[seq];
    const int c_begin = chunk * chunk_len;
    if (c_begin >= ctx) return;
    const int c_end = min(ctx, c_begin + chunk_len);
    const int n_it = (c_end - c_begin + DM_PAGE - 1) / DM_PAGE;
    const int32_t* bt = block_table + (long long)seq * max_pages + c_begin / DM_PAGE;
    if (FUSED && k_new && ctx - 1 >= c_begin) {  // ctx - 1 < c_end always: this CTA owns the newest position
        const int pos = ctx - 1;
        if (threadIdx.x < DM_D / 2) {
            const int pr = threadIdx.x;
            const int page = block_table[(long long)seq * max_pages + pos / DM_PAGE];
            __nv_bfloat16* kdst = pool + ((long long)dm_block_row(page, 0, Hkv, hk) + pos % DM_PAGE) * DM_D;
            __nv_bfloat16* vdst = pool + ((long long)dm_block_row(page, 1, Hkv, hk) + pos % DM_PAGE) * DM_D;
            uint32_t kw = *reinterpret_cast<const uint32_t*>(k_new + seq * kv_new_stride + (long long)hk * DM_D + 2 * pr);
            if (rope) {
                const float4 e = rope[(long long)pos * (DM_D / 2) + pr];
                const float x0 = bf16lo(kw), x1 = bf16hi(kw);
                kw = pack_bf16x2(__fadd_rn(__fmul_rn(e.x, x0), __fmul_rn(-e.w, x1)), __fadd_rn(__fmul_rn(e.y, x0), __fmul_rn(e.z, x1)));
            }
            *reinterpret_cast<uint32_t*>(kdst + 2 * pr) = kw;
            *reinterpret_cast<uint32_t*>(vdst + 2 * pr) = *reinterpret_cast<const uint32_t*>(v_new + seq * kv_new_stride + (long long)hk * DM_D + 2 * pr);
            asm volatile("fence.proxy.async.global;" ::: "memory");  // the bulk copies below read these rows
        }
        __syncthreads();
    }

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // heads (lane%4)*2 and +1
    float o[8][4];  // O^T: tile j = dims j*16 .. +15; [0],[1]: dim lane/4, the two heads; [2],[3]: dim lane/4 + 8
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    if (warp == DM_CWARPS) {
        // ---- producer: one page per stage
        if (lane == 0) {
            tma_prefetch_desc(&tmap);
            for (int it = 0; it < n_it; ++it) {
                const int s = it % DM_STAGES;
                if (it >= DM_STAGES && !mbar_wait(&empty_bar[s], ((it / DM_STAGES) - 1) & 1, &abort_flag, err, DM_ERR_EMPTY)) break;
                const int page = bt[it];
                uint8_t* dst = stages + s * DM_STAGE_BYTES;
                const int rk = dm_block_row(page, 0, Hkv, hk), rv = dm_block_row(page, 1, Hkv, hk);
                mbar_expect_tx(&full_bar[s], DM_STAGE_BYTES);
                tma_load_2d(dst, &tmap, 0, rk, &full_bar[s]);
                tma_load_2d(dst + DM_TILE_BYTES, &tmap, 64, rk, &full_bar[s]);
                tma_load_2d(dst + 2 * DM_TILE_BYTES, &tmap, 0, rv, &full_bar[s]);
                tma_load_2d(dst + 3 * DM_TILE_BYTES, &tmap, 64, rv, &full_bar[s]);
            }
        }
    } else {
        // ---- consumers.  B operand of the score product: the rotated query heads, head lane/4, dims (lane%4)*2 (+8)
        // of each 16-dim step, rounded to bf16 like a stored rotated q would be
        uint32_t qb[8][2];
        {
            const int head = lane >> 2;
            const __nv_bfloat16* qp = q + seq * q_stride + (long long)(hk * G + head) * DM_D;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int d0 = ks * 16 + h * 8 + (lane & 3) * 2;
                    uint32_t w = 0;
                    if (head < G) {
                        w = *reinterpret_cast<const uint32_t*>(qp + d0);
                        if (rope) {
                            const float4 e = rope[(long long)(ctx - 1) * (DM_D / 2) + d0 / 2];
                            const float x0 = bf16lo(w), x1 = bf16hi(w);
                            w = pack_bf16x2(__fadd_rn(__fmul_rn(e.x, x0), __fmul_rn(-e.w, x1)),
                                            __fadd_rn(__fmul_rn(e.y, x0), __fmul_rn(e.z, x1)));
                        }
                    }
                    qb[ks][h] = w;
                }
        }
        // ldmatrix row addresses of this lane inside a stage: matrix lane/8, row lane%8
        const int mi = lane >> 3, mr = lane & 7;
        const int krow = warp * 16 + (mi & 1) * 8 + mr;  // K (not transposed): matrices 0/1 = keys 0-7 / 8-15, 2/3 = dims +8
        const int kchunk = mi >> 1;                      // + 2 * step
        const int vrow = warp * 16 + (mi >> 1) * 8 + mr; // V (transposed): matrices 0/1 = dims 0-7 / 8-15, 2/3 = keys 8-15
        const int vchunk = mi & 1;                       // + 2 * tile
        const int r = lane >> 2;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % DM_STAGES;
            if (!mbar_wait(&full_bar[s], (it / DM_STAGES) & 1, &abort_flag, err, DM_ERR_FULL)) break;
            const uint32_t kbase = smem_u32(stages + s * DM_STAGE_BYTES), vbase = kbase + 2 * DM_TILE_BYTES;
            const int key0 = c_begin + it * DM_PAGE + warp * 16;
            if (key0 < c_end) {
                const int n_valid = min(16, c_end - key0);
                if (n_valid < 16) {
                    // zero the V rows past the context
                    uint8_t* vb = stages + s * DM_STAGE_BYTES + 2 * DM_TILE_BYTES;
                    for (int i = lane; i < (16 - n_valid) * 16; i += 32) {
                        const int row = warp * 16 + n_valid + (i >> 4), c = i & 15;
                        *reinterpret_cast<uint4*>(vb + (c >> 3) * DM_TILE_BYTES + row * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();  // the stage is overwritten by a bulk copy later
                    __syncwarp();
                }
                float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const int c = ks * 2 + kchunk;
                    uint32_t a[4];
                    ldsm_x4(kbase + (c >> 3) * DM_TILE_BYTES + krow * 128 + (((c & 7) ^ (krow & 7)) << 4), a);
                    mma_16816(sc, a, qb[ks][0], qb[ks][1]);
                }
                // sc[0], sc[1]: key r, heads h0, h0+1; sc[2], sc[3]: key r + 8
                float s0 = r < n_valid ? sc[0] * scale_log2 : -INFINITY, s1 = r < n_valid ? sc[1] * scale_log2 : -INFINITY;
                float s2 = r + 8 < n_valid ? sc[2] * scale_log2 : -INFINITY, s3 = r + 8 < n_valid ? sc[3] * scale_log2 : -INFINITY;
                float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
                for (int sh = 4; sh < 32; sh <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
                }
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: key 0 of the warp is valid
                const float corr0 = exp2f(m0 - mn0), corr1 = exp2f(m1 - mn1);
                m0 = mn0;
                m1 = mn1;
                const float p0 = exp2f(s0 - mn0), p1 = exp2f(s1 - mn1), p2 = exp2f(s2 - mn0), p3 = exp2f(s3 - mn1);
                l0 = fmaf(l0, corr0, p0 + p2);
                l1 = fmaf(l1, corr1, p1 + p3);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    o[j][0] *= corr0;
                    o[j][1] *= corr1;
                    o[j][2] *= corr0;
                    o[j][3] *= corr1;
                }
                const uint32_t pb0 = movmatrix_trans(pack_bf16x2(p0, p1)), pb1 = movmatrix_trans(pack_bf16x2(p2, p3));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = j * 2 + vchunk;
                    uint32_t a[4];
                    ldsm_x4_trans(vbase + (c >> 3) * DM_TILE_BYTES + vrow * 128 + (((c & 7) ^ (vrow & 7)) << 4), a);
                    mma_16816(o[j], a, pb0, pb1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
            l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
        }
    }
    __syncthreads();  // every stage has been consumed: the ring becomes the merge buffer [warp][head][dim]
    float* sm_o = reinterpret_cast<float*>(stages);
    if (warp < DM_CWARPS) {
        const int h0 = (lane & 3) * 2, dr = lane >> 2;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (h0 < G) {
                sm_o[(warp * 8 + h0) * DM_D + j * 16 + dr] = o[j][0];
                sm_o[(warp * 8 + h0) * DM_D + j * 16 + dr + 8] = o[j][2];
            }
            if (h0 + 1 < G) {
                sm_o[(warp * 8 + h0 + 1) * DM_D + j * 16 + dr] = o[j][1];
                sm_o[(warp * 8 + h0 + 1) * DM_D + j * 16 + dr + 8] = o[j][3];
            }
        }
        if (dr == 0) {
            sm_m[warp][h0] = m0;
            sm_l[warp][h0] = l0;
            sm_m[warp][h0 + 1] = m1;
            sm_l[warp][h0 + 1] = l1;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * DM_D; e += DM_THREADS) {
        const int g = e / DM_D, d = e % DM_D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DM_CWARPS; ++w) M = fmaxf(M, sm_m[w][g]);
        float acc = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < DM_CWARPS; ++w) {
            const float f = sm_m[w][g] == -INFINITY ? 0.0f : exp2f(sm_m[w][g] - M);
            acc += f * sm_o[(w * 8 + g) * DM_D + d];
            L += f * sm_l[w][g];
        }
        float* dst = scratch + (((long long)seq * Hq + hk * G + g) * n_chunks + chunk) * (DM_D + 2);
        if (FUSED && ctx <= chunk_len) {
            out[((long long)seq * Hq + hk * G + g) * DM_D + d] = __float2bfloat16_rn(acc / L);  // a single chunk: the result
        } else {
            dst[d] = acc;
            if (d == 0) {
                dst[DM_D] = M;
                dst[DM_D + 1] = L;
            }
        }
    }
    if (!FUSED || ctx <= chunk_len) return;
    // ---- the last CTA of this (sequence, kv head) merges the chunk partials
    __shared__ int is_last;
    __syncthreads();  // all partial stores of the CTA precede the release below
    const int n = (ctx + chunk_len - 1) / chunk_len;
    if (threadIdx.x == 0) {
        int old;
        int* ctr = counters + (long long)seq * Hkv + hk;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(ctr) : "memory");
        is_last = (old == n - 1);
        if (is_last) *ctr = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    for (int e = threadIdx.x; e < G * DM_D; e += DM_THREADS) {
        const int g = e / DM_D, d = e % DM_D;
        const float* src = scratch + ((long long)seq * Hq + hk * G + g) * n_chunks * (DM_D + 2);
        float M = -INFINITY;
        for (int c = 0; c < n; ++c) M = fmaxf(M, __ldcg(src + c * (DM_D + 2) + DM_D));
        float acc = 0.0f, L = 0.0f;
        for (int c = 0; c < n; ++c) {
            const float f = exp2f(__ldcg(src + c * (DM_D + 2) + DM_D) - M);
            acc += f * __ldcg(src + c * (DM_D + 2) + d);
            L += f * __ldcg(src + c * (DM_D + 2) + DM_D + 1);
        }
        out[((long long)seq * Hq + hk * G + g) * DM_D + d] = __float2bfloat16_rn(acc / L);
    }
}

template <int G, bool FUSED>
static jsm_status dm_launch(const CUtensorMap& map, dim3 grid, cudaStream_t st, const DecodeMmaArgs& a) {
    static bool configured[64] = {false};
    int dev = 0;
    JSM_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        JSM_CUDA_CHECK(cudaFuncSetAttribute(attn_decode_mma_kernel<G, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, DM_SMEM));
        configured[dev] = true;
    }
    JSM_CUDA_CHECK(launch_chained(attn_decode_mma_kernel<G, FUSED>, grid, dim3(DM_THREADS), (size_t)DM_SMEM, st, map,
                                  (const __nv_bfloat16*)a.q, a.q_stride, (__nv_bfloat16*)a.pool, a.block_table, a.max_pages,
                                  a.context_lens, a.Hq, a.Hkv, a.scale_log2, (const float4*)a.rope, a.n_chunks, a.chunk, a.scratch,
                                  (const __nv_bfloat16*)a.k_new, (const __nv_bfloat16*)a.v_new, a.kv_new_stride, a.counters,
                                  (__nv_bfloat16*)a.out, tc_error_word()));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

bool attn_decode_mma_usable(int G, int chunk, const void* pool) {
    return (G == 2 || G == 4 || G == 8) && chunk % DM_PAGE == 0 && (reinterpret_cast<uintptr_t>(pool) & 15) == 0;
}

jsm_status attn_decode_mma_launch(const DecodeMmaArgs& a, cudaStream_t st) {
    // The pool as rows of 128 bf16.  Its size is not known here: the row count only bounds the coordinates the copy
    // engine accepts, the block table decides which rows are read.
    CUtensorMap map;
    jsm_status s = make_tmap_bf16_2d(&map, a.pool, 1ull << 30, DM_D, DM_D, DM_PAGE, 64);
    if (s != JSM_OK) return s;
    dim3 grid(a.n_chunks, a.Hkv, a.n_seqs);
    const int G = a.Hq / a.Hkv;
    if (a.fused) {
        switch (G) {
            case 2: return dm_launch<2, true>(map, grid, st, a);
            case 4: return dm_launch<4, true>(map, grid, st, a);
            case 8: return dm_launch<8, true>(map, grid, st, a);
        }
    } else {
        switch (G) {
            case 2: return dm_launch<2, false>(map, grid, st, a);
            case 4: return dm_launch<4, false>(map, grid, st, a);
            case 8: return dm_launch<8, false>(map, grid, st, a);
        }
    }
    JSM_FAIL(JSM_UNSUPPORTED, "attn_decode_mma: %d query heads per kv head", G);
}

}  // namespace jsm
