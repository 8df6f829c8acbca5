// bf16 projections Y[t,n] = sum_k X[t,k] * W[n,k] with fp32 accumulation: the
// device form of weight_net_t::forward (mat_net_t.hpp:38-49, Y = W.X + b with W
// stored [out, in]).
//
// Two kernels:
//  * linear_tc_kernel  — tcgen05: W tiles (128 output features x 64 k) are the A
//    operand, X tiles (BN tokens x 64 k) the B operand, both staged by TMA with
//    the 128-byte swizzle through a ring of shared-memory stages; the 128 x BN fp32
//    accumulator lives in TMEM.  Roles: warp 0 issues TMA, warp 1 issues MMAs,
//    warps 2-5 read the accumulator back (one TMEM lane = one output feature per
//    thread) and apply the epilogue.  With few tokens the kernel is a weight
//    stream: every byte of W crosses HBM once and the grid is split along K so that
//    all SMs pull at once (fp32 partials, folded by the caller).
//  * gemv_kernel — CUDA cores, up to 4 tokens: each warp streams 4 weight rows with
//    128-bit loads that bypass L1 allocation and reduces with shuffles.
#include "tc_utils.cuh"
#include "linear_bf16.cuh"
#include <math.h>
#include <mutex>

namespace jsm {

using namespace tc;

// ---- driver entry point for tensor maps (no link-time dependency on libcuda) -------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_tiled_fn get_encode() {
    static encode_tiled_fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
    });
    return fn;
}

jsm_status make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                             uint32_t box_rows, uint32_t box_cols) {
    encode_tiled_fn enc = get_encode();
    if (!enc) JSM_FAIL(JSM_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver)");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_elems * 2) % 16)
        JSM_FAIL(JSM_INVALID_ARG, "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) JSM_FAIL(JSM_CUDA, "cuTensorMapEncodeTiled failed with %d (rows %llu cols %llu)", (int)r,
                                    (unsigned long long)rows, (unsigned long long)cols);
    return JSM_OK;
}

jsm_status make_tmap_bf16_3d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems,
                             uint64_t s2_elems, uint32_t b0, uint32_t b1, uint32_t b2) {
    encode_tiled_fn enc = get_encode();
    if (!enc) JSM_FAIL(JSM_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver)");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_elems * 2) % 16 || (s2_elems * 2) % 16)
        JSM_FAIL(JSM_INVALID_ARG, "TMA operand must be 16-byte aligned with 16-byte multiple pitches");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {s1_elems * 2, s2_elems * 2};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) JSM_FAIL(JSM_CUDA, "cuTensorMapEncodeTiled (3d) failed with %d", (int)r);
    return JSM_OK;
}

int* tc_error_word() {
    static int* words[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, sizeof(int));
        words[dev] = p;
    }
    return words[dev];
}

// ---- epilogue helpers -----------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// ---- tcgen05 kernel ----------------------------------------------------------------------------
constexpr int BM = 128;  // output features per tile (MMA M, TMEM lanes)
constexpr int BK = 64;   // k per stage: one 128-byte swizzled row
constexpr int TC_THREADS = 192;

struct TcParams {
    int T, N, K;          // tokens, output features, reduction length
    int kb_per_split;     // k-blocks (of 64) per grid.z slice
    int epilogue;         // LIN_*
    int out_mode;         // 0 bf16 Y, 1 f32 Y, 2 f32 partial [split][T][N]
    const float* bias;
    const __nv_bfloat16* R;
    void* Y;
    int* err;
    float* ws;            // split-K with in-kernel fix-up: partials [split][T][ldw]
    int* counters;        // one arrival counter per output tile, zero between launches
    int w_early;          // W is constant for the whole stream: its tiles may be fetched before the predecessor kernel ends
    int pf_kb;            // with w_early: k-blocks of W beyond the ring that are prefetched into L2 up front
};

template <int BN, bool GATEUP>
__global__ void __launch_bounds__(TC_THREADS, 1)
    linear_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, TcParams P, int stages) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int A_BYTES = BM * BK * 2 * (GATEUP ? 2 : 1);
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLS_NEEDED = GATEUP ? 2 * BN : BN;
    constexpr int TMEM_COLS = TMEM_COLS_NEEDED < 32 ? 32 : TMEM_COLS_NEEDED;
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns must be a power of two <= 512");
    constexpr int MAX_STAGES = 12;

    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t acc_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    chain_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM;   // first output feature of the tile
    const int t0 = blockIdx.y * BN;   // first token of the tile
    const int kb_total = (P.K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * P.kb_per_split;
    const int kb_end = min(kb_total, kb_begin + P.kb_per_split);
    const int n_kb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        mbar_fence_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ---- producer: one thread streams W and X tiles into the ring
        if (lane == 0) {
            int issued = 0;
            // weights never change while the stream runs: the first ring of W tiles is requested (and further tiles are
            // pulled into L2) before the predecessor kernel has finished; the tokens X are its output and wait for it
            const int pre = P.w_early ? min(n_kb, stages) : 0;
            for (int i = 0; i < pre; ++i) {
                uint8_t* st = tiles + (size_t)i * STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], STAGE_BYTES);
                const int kx = (kb_begin + i) * BK;
                tma_load_2d(st, &tmap_w, kx, n0, &full_bar[i]);
                if (GATEUP) tma_load_2d(st + BM * BK * 2, &tmap_w, kx, P.N + n0, &full_bar[i]);
            }
            if (P.w_early) {
                const int pf_end = min(n_kb, pre + P.pf_kb);
                for (int i = pre; i < pf_end; ++i) {
                    const int kx = (kb_begin + i) * BK;
                    tma_prefetch_2d(&tmap_w, kx, n0);
                    if (GATEUP) tma_prefetch_2d(&tmap_w, kx, P.N + n0);
                }
            }
            chain_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES + A_BYTES, &tmap_x, (kb_begin + i) * BK, t0, &full_bar[i]);
            issued = pre;
            for (int i = pre; i < n_kb; ++i) {
                const int s = i % stages;
                const uint32_t ph = (i / stages) & 1;
                if (i >= stages && !mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, P.err, TC_TIMEOUT_EMPTY)) break;
                uint8_t* st = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                const int kx = (kb_begin + i) * BK;
                tma_load_2d(st, &tmap_w, kx, n0, &full_bar[s]);
                if (GATEUP) tma_load_2d(st + BM * BK * 2, &tmap_w, kx, P.N + n0, &full_bar[s]);
                tma_load_2d(st + A_BYTES, &tmap_x, kx, t0, &full_bar[s]);
                issued = i + 1;
            }
            // on an abort, wait (bounded) for the copies still in flight before the CTA may exit
            if (abort_flag) {
                for (int i = max(0, issued - stages); i < issued; ++i) {
                    const long long t_start = clock64();
                    while (!mbar_try_wait(&full_bar[i % stages], (i / stages) & 1) && clock64() - t_start < WAIT_LIMIT_CYCLES) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % stages;
                const uint32_t ph = (i / stages) & 1;
                if (!mbar_wait(&full_bar[s], ph, &abort_flag, P.err, TC_TIMEOUT_FULL)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
                const uint64_t a_desc = smem_desc_sw128(a_addr);
                const uint64_t b_desc = smem_desc_sw128(b_addr);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    mma_ss(tmem_base, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, acc);
                    if (GATEUP) {
                        const uint64_t u_desc = smem_desc_sw128(a_addr + BM * BK * 2);
                        mma_ss(tmem_base + BN, u_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, acc);
                    }
                }
                mma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
            }
            if (ok) mma_commit(&acc_bar);    // accumulator complete
        }
    } else {
        // ---- epilogue: warps 2..5 -> TMEM lane quadrants (warp % 4)
        const int quad = warp & 3;
        const int feat = n0 + quad * 32 + lane;
        bool ok = n_kb > 0;
        if (ok) ok = mbar_wait(&acc_bar, 0, &abort_flag, P.err, TC_TIMEOUT_ACC);
        tc_fence_after();
        chain_wait();  // the residual input, the output and the workspace belong to the stream's other kernels
        if (ok && P.ws && gridDim.z > 1) {
            // ---- split-K with in-kernel fix-up: every CTA of a tile stores its raw partial; the one that arrives last
            // adds the partials in split order (so the result does not depend on who is last) and runs the epilogue
            __shared__ int is_last;
            const int ldw = GATEUP ? 2 * P.N : P.N;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= P.T) break;
                uint32_t r[16], u[16];
                tmem_ld16(lane_addr + c0, r);
                if (GATEUP) tmem_ld16(lane_addr + BN + c0, u);
                tmem_ld_wait();
                if (feat < P.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c0 + j;
                        if (t < P.T) {
                            float* w = P.ws + ((size_t)blockIdx.z * P.T + t) * ldw + feat;
                            __stcg(w, __uint_as_float(r[j]));
                            if (GATEUP) __stcg(w + P.N, __uint_as_float(u[j]));
                        }
                    }
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
            if (threadIdx.x == 64) {
                const int old = atomicAdd(&P.counters[tile_id], 1);
                is_last = (old == (int)gridDim.z - 1);
                if (is_last) P.counters[tile_id] = 0;  // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (is_last) {
                // 128 threads fold the tile: a thread owns 4 consecutive features of every fourth token, the partials of
                // four tokens are in flight at once and are added in split order (the result does not depend on who came last)
                __threadfence();
                const int tid = threadIdx.x - 64;
                const int n = n0 + (tid & 31) * 4, tsub = tid >> 5;
                const int t_end = min(P.T, t0 + BN);
                if (n < P.N) {
                    const float4 bias4 = P.bias ? *reinterpret_cast<const float4*>(P.bias + n) : make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int tb = t0 + tsub; tb < t_end; tb += 16) {
                        float4 g[4], u[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) { g[i] = make_float4(0.f, 0.f, 0.f, 0.f); u[i] = g[i]; }
#pragma unroll 2
                        for (int z = 0; z < (int)gridDim.z; ++z) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int t = tb + 4 * i;
                                if (t < t_end) {
                                    const float* w = P.ws + ((size_t)z * P.T + t) * ldw + n;
                                    const float4 a = __ldcg(reinterpret_cast<const float4*>(w));
                                    g[i].x += a.x; g[i].y += a.y; g[i].z += a.z; g[i].w += a.w;
                                    if (GATEUP) {
                                        const float4 c = __ldcg(reinterpret_cast<const float4*>(w + P.N));
                                        u[i].x += c.x; u[i].y += c.y; u[i].z += c.z; u[i].w += c.w;
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int t = tb + 4 * i;
                            if (t >= t_end) break;
                            float v[4] = {g[i].x + bias4.x, g[i].y + bias4.y, g[i].z + bias4.z, g[i].w + bias4.w};
                            const float uu[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
                            if (P.epilogue == LIN_RESIDUAL) {
                                const uint2 r = *reinterpret_cast<const uint2*>(P.R + (size_t)t * P.N + n);
                                v[0] += bf16lo(r.x); v[1] += bf16hi(r.x); v[2] += bf16lo(r.y); v[3] += bf16hi(r.y);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (GATEUP) v[j] = silu_f(v[j]) * uu[j];
                                else if (P.epilogue == LIN_RELU) v[j] = fmaxf(v[j], 0.0f);
                                else if (P.epilogue == LIN_GELU) v[j] = gelu_f(v[j]);
                            }
                            if (P.out_mode == 0) {
                                uint2 o;
                                o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
                                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(P.Y) + (size_t)t * P.N + n) = o;
                            } else {
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(P.Y) + (size_t)t * P.N + n) = make_float4(v[0], v[1], v[2], v[3]);
                            }
                        }
                    }
                }
            }
        } else if (ok) {
            const float bias = (P.bias && feat < P.N && (P.out_mode != 2 || blockIdx.z == 0)) ? P.bias[feat] : 0.0f;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= P.T) break;
                uint32_t r[16], u[16];
                tmem_ld16(lane_addr + c0, r);
                if (GATEUP) tmem_ld16(lane_addr + BN + c0, u);
                tmem_ld_wait();
                if (feat < P.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c0 + j;
                        if (t < P.T) {
                            float v = __uint_as_float(r[j]) + bias;
                            if (GATEUP) v = silu_f(v) * __uint_as_float(u[j]);
                            else if (P.epilogue == LIN_RELU) v = fmaxf(v, 0.0f);
                            else if (P.epilogue == LIN_GELU) v = gelu_f(v);
                            else if (P.epilogue == LIN_RESIDUAL) v += __bfloat162float(P.R[(size_t)t * P.N + feat]);
                            if (P.out_mode == 0)
                                reinterpret_cast<__nv_bfloat16*>(P.Y)[(size_t)t * P.N + feat] = __float2bfloat16_rn(v);
                            else if (P.out_mode == 1)
                                reinterpret_cast<float*>(P.Y)[(size_t)t * P.N + feat] = v;
                            else
                                reinterpret_cast<float*>(P.Y)[((size_t)blockIdx.z * P.T + t) * P.N + feat] = v;
                        }
                    }
                }
            }
        } else if (n_kb == 0 && P.out_mode == 2 && feat < P.N) {
            for (int t = t0; t < min(P.T, t0 + BN); ++t)
                reinterpret_cast<float*>(P.Y)[((size_t)blockIdx.z * P.T + t) * P.N + feat] = 0.0f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- CUDA-core weight stream for up to 4 tokens --------------------------------------------------
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x) {
    float s = bf16lo(w.x) * bf16lo(x.x);
    s = fmaf(bf16hi(w.x), bf16hi(x.x), s);
    s = fmaf(bf16lo(w.y), bf16lo(x.y), s);
    s = fmaf(bf16hi(w.y), bf16hi(x.y), s);
    s = fmaf(bf16lo(w.z), bf16lo(x.z), s);
    s = fmaf(bf16hi(w.z), bf16hi(x.z), s);
    s = fmaf(bf16lo(w.w), bf16lo(x.w), s);
    s = fmaf(bf16hi(w.w), bf16hi(x.w), s);
    return s;
}

// Each warp owns ROWS output rows (GATEUP: ROWS/2 gate rows and the matching up rows).
template <int TOK, bool GATEUP, int ROWS>
__global__ void __launch_bounds__(256) gemv_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                                                   const float* __restrict__ bias, int epilogue, const __nv_bfloat16* __restrict__ R,
                                                   void* __restrict__ Y, int out_f32, int N, int K, int w_early) {
    constexpr int OUTS = GATEUP ? ROWS / 2 : ROWS;
    chain_trigger();
    const int warp = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int o0 = warp * OUTS;  // first output of this warp
    if (o0 >= N) return;
    const uint4* wrow[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        int row;
        if (GATEUP) row = (r < OUTS) ? o0 + r : N + o0 + (r - OUTS);
        else row = o0 + r;
        const int lim = GATEUP ? 2 * N : N;
        if (row >= lim) row = lim - 1;
        wrow[r] = reinterpret_cast<const uint4*>(W + (size_t)row * K);
    }
    float acc[ROWS][TOK];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[r][t] = 0.0f;
    const int nvec = K / 8;
    chain_wait();
#pragma unroll 4
    for (int v = lane; v < nvec; v += 32) {
        uint4 w[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) w[r] = __ldcs(wrow[r] + v);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(X + (size_t)t * K) + v);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) acc[r][t] += dot8(w[r], x);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[r][t] = warp_sum(acc[r][t]);
    if (lane == 0) {
#pragma unroll
        for (int o = 0; o < OUTS; ++o) {
            const int n = o0 + o;
            if (n >= N) break;
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                float v = acc[o][t] + (bias ? bias[n] : 0.0f);
                if (GATEUP) v = silu_f(v) * acc[o + OUTS][t];
                else if (epilogue == LIN_RELU) v = fmaxf(v, 0.0f);
                else if (epilogue == LIN_GELU) v = gelu_f(v);
                else if (epilogue == LIN_RESIDUAL) v += __bfloat162float(R[(size_t)t * N + n]);
                if (out_f32) reinterpret_cast<float*>(Y)[(size_t)t * N + n] = v;
                else reinterpret_cast<__nv_bfloat16*>(Y)[(size_t)t * N + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int TOK>
static void launch_gemv(const void* X, const void* W, const float* bias, int epi, const void* R, void* Y, int out_f32, int N, int K,
                        bool chained, cudaStream_t st) {
    const bool gu = epi == LIN_SILU_MUL;
    // enough warps for two CTAs on every SM: narrow outputs use two rows per warp instead of four
    const bool narrow = !gu && (N / 4 + 7) / 8 < 2 * sm_count();
    const int outs_per_warp = gu ? 2 : (narrow ? 2 : 4);
    const int warps = (N + outs_per_warp - 1) / outs_per_warp;
    const int blocks = (warps + 7) / 8;
    const int early = chained ? 1 : 0;
    auto go = [&](auto kernel) {
        if (chained)
            launch_chained(kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, bias, epi,
                           (const __nv_bfloat16*)R, Y, out_f32, N, K, early);
        else
            kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)X, (const __nv_bfloat16*)W, bias, epi, (const __nv_bfloat16*)R, Y,
                                           out_f32, N, K, early);
    };
    if (gu) go(gemv_kernel<TOK, true, 4>);
    else if (narrow) go(gemv_kernel<TOK, false, 2>);
    else go(gemv_kernel<TOK, false, 4>);
}

template <int BN, bool GATEUP>
static jsm_status launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& P, int splits, cudaStream_t st) {
    constexpr int A_BYTES = BM * BK * 2 * (GATEUP ? 2 : 1);
    constexpr int STAGE_BYTES = A_BYTES + BN * BK * 2;
    // a weight stream split along K runs two CTAs per SM (about 100 KB of stages each) so that a grid of about twice
    // the SM count is resident at once; a single-wave grid takes the whole shared memory for one deep ring
    const int n_ctas = ((P.N + BM - 1) / BM) * ((P.T + BN - 1) / BN) * splits;
    const bool two_per_sm = n_ctas > sm_count() && 2 * (GATEUP ? 2 * BN : BN) <= 512;
    int stages = ((two_per_sm ? 104 : 200) * 1024) / STAGE_BYTES;
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    const size_t smem = (size_t)stages * STAGE_BYTES + 1024;
    static bool attr_done = false;  // per instantiation
    if (!attr_done) {
        JSM_CUDA_CHECK(cudaFuncSetAttribute(linear_tc_kernel<BN, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        attr_done = true;
    }
    dim3 grid((P.N + BM - 1) / BM, (P.T + BN - 1) / BN, splits);
    TcParams Q = P;
    if (Q.w_early) {
        // L2 prefetch beyond the ring: at most about 48 MB per launch over all CTAs
        const long long per_kb = (long long)A_BYTES * n_ctas;
        long long pf = per_kb > 0 ? (48ll << 20) / per_kb : 0;
        Q.pf_kb = (int)(pf > 64 ? 64 : pf);
        JSM_CUDA_CHECK(launch_chained(linear_tc_kernel<BN, GATEUP>, grid, dim3(TC_THREADS), smem, st, mw, mx, Q, stages));
        g_launches.fetch_add(1);
        return JSM_OK;
    }
    linear_tc_kernel<BN, GATEUP><<<grid, TC_THREADS, smem, st>>>(mw, mx, Q, stages);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

jsm_status linear_bf16_launch(const LinearArgs& a, cudaStream_t st) {
    if (a.T <= 0 || a.N <= 0) return JSM_OK;
    if (!a.X || !a.W || !a.Y) JSM_FAIL(JSM_INVALID_ARG, "linear_bf16: null pointer");
    if (a.K <= 0 || a.K % 8) JSM_FAIL(JSM_UNSUPPORTED, "linear_bf16: K (%d) must be a positive multiple of 8", a.K);
    if (a.epilogue < LIN_NONE || a.epilogue > LIN_RESIDUAL) JSM_FAIL(JSM_INVALID_ARG, "linear_bf16: epilogue %d", a.epilogue);
    if (a.epilogue == LIN_RESIDUAL && !a.R) JSM_FAIL(JSM_INVALID_ARG, "linear_bf16: residual epilogue without R");
    if (a.splits > 1 && !a.ws && (a.out_mode != 2 || a.epilogue != LIN_NONE))
        JSM_FAIL(JSM_INVALID_ARG, "linear_bf16: split-K without a workspace writes raw f32 partials only");
    if (a.splits > 1 && a.ws && (a.out_mode == 2 || !a.counters || a.N % 4))
        JSM_FAIL(JSM_INVALID_ARG, "linear_bf16: split-K with in-kernel fix-up needs arrival counters, a final output and N %% 4 == 0");
    const bool use_gemv = a.impl == 1 || (a.impl == 0 && a.T <= 4 && a.out_mode != 2);
    if (use_gemv) {
        if (a.T > 4) JSM_FAIL(JSM_UNSUPPORTED, "linear_bf16: the CUDA-core kernel takes at most 4 tokens");
        const int f32 = a.out_mode == 1;
        switch (a.T) {
            case 1: launch_gemv<1>(a.X, a.W, a.bias, a.epilogue, a.R, a.Y, f32, a.N, a.K, a.chained, st); break;
            case 2: launch_gemv<2>(a.X, a.W, a.bias, a.epilogue, a.R, a.Y, f32, a.N, a.K, a.chained, st); break;
            case 3: launch_gemv<3>(a.X, a.W, a.bias, a.epilogue, a.R, a.Y, f32, a.N, a.K, a.chained, st); break;
            default: launch_gemv<4>(a.X, a.W, a.bias, a.epilogue, a.R, a.Y, f32, a.N, a.K, a.chained, st); break;
        }
        JSM_LAUNCH_CHECK();
        return JSM_OK;
    }
    const bool gu = a.epilogue == LIN_SILU_MUL;
    CUtensorMap mw, mx;
    const int bn = a.T <= 16 ? 16 : a.T <= 32 ? 32 : a.T <= 64 ? 64 : 128;
    jsm_status s = make_tmap_bf16_2d(&mw, a.W, (uint64_t)(gu ? 2 * a.N : a.N), (uint64_t)a.K, (uint64_t)a.K, BM, BK);
    if (s != JSM_OK) return s;
    s = make_tmap_bf16_2d(&mx, a.X, (uint64_t)a.T, (uint64_t)a.K, (uint64_t)a.K, bn, BK);
    if (s != JSM_OK) return s;
    TcParams P;
    P.T = a.T; P.N = a.N; P.K = a.K;
    const int kb_total = (a.K + BK - 1) / BK;
    int splits = a.splits < 1 ? 1 : (a.splits > kb_total ? kb_total : a.splits);
    P.kb_per_split = (kb_total + splits - 1) / splits;
    splits = (kb_total + P.kb_per_split - 1) / P.kb_per_split;  // no empty slice: every CTA of a tile must arrive
    P.epilogue = a.epilogue; P.out_mode = a.out_mode; P.bias = a.bias; P.R = (const __nv_bfloat16*)a.R; P.Y = a.Y;
    P.err = tc_error_word();
    P.ws = a.ws; P.counters = a.counters;
    P.w_early = a.chained ? 1 : 0; P.pf_kb = 0;
    const int grid_z = a.out_mode == 2 ? (a.splits < 1 ? 1 : a.splits) : (a.ws ? splits : 1);
    if (gu) {
        switch (bn) {
            case 16: return launch_tc<16, true>(mw, mx, P, grid_z, st);
            case 32: return launch_tc<32, true>(mw, mx, P, grid_z, st);
            case 64: return launch_tc<64, true>(mw, mx, P, grid_z, st);
            default: return launch_tc<128, true>(mw, mx, P, grid_z, st);
        }
    }
    switch (bn) {
        case 16: return launch_tc<16, false>(mw, mx, P, grid_z, st);
        case 32: return launch_tc<32, false>(mw, mx, P, grid_z, st);
        case 64: return launch_tc<64, false>(mw, mx, P, grid_z, st);
        default: return launch_tc<128, false>(mw, mx, P, grid_z, st);
    }
}

jsm_status tc_check_error(cudaStream_t st, const char* who) {
    int* w = tc_error_word();
    if (!w) return JSM_OK;
    int h = 0;
    JSM_CUDA_CHECK(cudaMemcpyAsync(&h, w, sizeof(int), cudaMemcpyDeviceToHost, st));
    JSM_CUDA_CHECK(cudaStreamSynchronize(st));
    if (h != 0) {
        cudaMemsetAsync(w, 0, sizeof(int), st);
        if (h == 32) JSM_FAIL(JSM_SHAPE, "%s: context overflow: a decode step met a sequence that already holds max_context tokens", who);
        JSM_FAIL(JSM_TIMEOUT, "%s: a bounded device-side wait ran out (code %d)", who, h);
    }
    return JSM_OK;
}

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_check_device_errors(void* stream) { return tc_check_error(as_stream(stream), "jsm_check_device_errors"); }

extern "C" jsm_status jsm_linear_bf16(const void* d_X, const void* d_W, const float* d_bias, int epilogue, const void* d_R,
                                      void* d_Y, int out_dtype, int T, int N, int K, void* stream) {
    if (out_dtype != JSM_BF16 && out_dtype != JSM_F32) JSM_FAIL(JSM_UNSUPPORTED, "jsm_linear_bf16: out dtype %d", out_dtype);
    LinearArgs a;
    a.X = d_X; a.W = d_W; a.bias = d_bias; a.epilogue = epilogue; a.R = d_R; a.Y = d_Y;
    a.out_mode = out_dtype == JSM_F32 ? 1 : 0;
    a.T = T; a.N = N; a.K = K; a.splits = 1; a.impl = 0; a.ws = nullptr; a.counters = nullptr;
    return linear_bf16_launch(a, as_stream(stream));
}
