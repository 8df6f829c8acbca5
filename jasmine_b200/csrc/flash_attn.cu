// Flash-attention prefill on the 5th-generation tensor cores (tcgen05 + TMEM), bf16, head_dim 128:
// the device form of mat_head_gen_t::forward (mat_mha_t.hpp:53-71: scores = Q^T K / sqrt(d), causal
// -inf above the diagonal, row softmax, out = V P^T) without ever materialising the S x S score matrix.
//
// One CTA owns 256 consecutive queries of one (sequence, head) as two 128-row tiles and walks the keys in
// tiles of 128.  Roles (320 threads):
//   warp 0      TMA producer: Q once, then K and V tiles through two-stage rings (128-byte swizzle)
//   warp 1      MMA issuer:   S_t = Q_t . K^T  (operands in shared memory) and O_t += P_t . V
//                             (P_t read from TMEM, V from shared memory, N-contiguous)
//   warps 2-5   softmax of query tile 0, one thread per query row (= TMEM lane): no shuffles
//   warps 6-9   softmax of query tile 1
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each; P_t (bf16, 64 columns) overwrites the
// first half of S_t in place.  While one tile's softmax runs on the CUDA cores, the tensor cores work on the
// other tile.  The running maximum is only raised (and O rescaled) when it grew by more than 2^8, so the
// rescale of the accumulator is rare; the final division by the row sum happens in the epilogue.
// Every wait is bounded; on a timeout the CTA unwinds, frees its TMEM and records a code for the host.
#include "attn.cuh"
#include "tc_utils.cuh"
#include <stdlib.h>
#include <math.h>

namespace jsm {

using namespace tc;

constexpr int FA_D = 128;          // head_dim
constexpr int FA_BM = 128;         // queries per tile (TMEM lanes)
constexpr int FA_BN = 128;         // keys per tile
constexpr int FA_THREADS = 320;
constexpr int FA_KV_STAGES = 2;
constexpr uint32_t FA_TILE_BYTES = FA_BM * FA_D * 2;  // 32 KB: two 16 KB halves of 64 columns
constexpr float FA_RESCALE_THRESHOLD = 8.0f;          // log2 domain

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Blackwell's packed fp32 pairs and three-input maximum: half the FMA / ADD / MAX instructions of the softmax rows
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

struct FlashParams {
    int Tq, Tk, Hq, Hkv, causal;
    float scale_log2;
    __nv_bfloat16* out;
    long long out_rs;
    int* err;
};

// 2^x for a pair of scores without the special-function unit: x = n + f with n = round(x) taken from the mantissa of
// x + 1.5 * 2^23, 2^f on [-0.5, 0.5] by a cubic (relative error 7.5e-5, far below the bf16 rounding of P), n added to
// the exponent field.  The MUFU pipe (16 results per clock and SM) is what the softmax of a tile waits for once the
// tensor pipe runs tcgen05 rates, so a share of the exponentials goes to the FMA pipe instead.
__device__ __forceinline__ void ex2_poly2(uint64_t x2, float& p0, float& p1) {
    float x0, x1;
    unpack2(x2, x0, x1);
    x2 = pack2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const uint64_t magic2 = pack2(12582912.0f, 12582912.0f), neg_magic2 = pack2(-12582912.0f, -12582912.0f);
    const uint64_t r2 = fadd2(x2, magic2);
    const uint64_t n2 = fadd2(r2, neg_magic2);
    const uint64_t f2 = ffma2(n2, pack2(-1.0f, -1.0f), x2);
    uint64_t q2 = ffma2(pack2(0.0551716685f, 0.0551716685f), f2, pack2(0.2426111251f, 0.2426111251f));
    q2 = ffma2(q2, f2, pack2(0.6932609677f, 0.6932609677f));
    q2 = ffma2(q2, f2, pack2(0.9999280572f, 0.9999280572f));
    float q0, q1, r0, r1;
    unpack2(q2, q0, q1);
    unpack2(r2, r0, r1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

// POLY: of every four pairs of scores, this many take ex2_poly2 instead of ex2.approx
template <int POLY>
__global__ void __launch_bounds__(FA_THREADS, 1)
    flash_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, FlashParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = tiles;                                   // 2 x 32 KB
    uint8_t* k_smem = tiles + 2 * FA_TILE_BYTES;               // FA_KV_STAGES x 32 KB
    uint8_t* v_smem = k_smem + FA_KV_STAGES * FA_TILE_BYTES;   // FA_KV_STAGES x 32 KB
    __shared__ __align__(8) uint64_t q_full, o_done;
    __shared__ __align__(8) uint64_t k_full[FA_KV_STAGES], k_empty[FA_KV_STAGES], v_full[FA_KV_STAGES], v_empty[FA_KV_STAGES];
    __shared__ __align__(8) uint64_t s_full[2], p_ready[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // longest tiles first: with a causal mask the last query block has the most keys
    const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / (P.Hq / P.Hkv);
    const int q0 = qblk * 2 * FA_BM;
    const int shift = P.Tk - P.Tq;  // query i sits at position i + shift
    // number of key tiles each query tile needs
    int n_tiles[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int last_row = min(q0 + (t + 1) * FA_BM, P.Tq) - 1;  // may be < first row when the tile is empty
        int kv_end = P.causal ? min(P.Tk, last_row + shift + 1) : P.Tk;
        if (q0 + t * FA_BM >= P.Tq) kv_end = 0;
        n_tiles[t] = (kv_end + FA_BN - 1) / FA_BN;
    }
    const int n_max = max(n_tiles[0], n_tiles[1]);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&q_full, 1);
        mbar_init(&o_done, 1);
        for (int s = 0; s < FA_KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_ready[t], 128); }
        mbar_fence_init();
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_smem;
    const uint32_t S_COL[2] = {0, 128}, O_COL[2] = {256, 384};

    if (warp == 0) {
        if (lane == 0) {
            // Q: both tiles, two 64-column halves each
            mbar_expect_tx(&q_full, 2 * FA_TILE_BYTES);
            for (int t = 0; t < 2; ++t)
                for (int half = 0; half < 2; ++half)
                    tma_load_2d(q_smem + t * FA_TILE_BYTES + half * (FA_TILE_BYTES / 2), &tmap_q, h * FA_D + half * 64,
                                b * P.Tq + q0 + t * FA_BM, &q_full);
            int issued = 0;
            for (int j = 0; j < n_max; ++j) {
                const int s = j % FA_KV_STAGES;
                const uint32_t ph = (j / FA_KV_STAGES) & 1;
                if (j >= FA_KV_STAGES && !mbar_wait(&k_empty[s], ph ^ 1, &abort_flag, P.err, TC_TIMEOUT_EMPTY)) break;
                mbar_expect_tx(&k_full[s], FA_TILE_BYTES);
                for (int half = 0; half < 2; ++half)
                    tma_load_2d(k_smem + s * FA_TILE_BYTES + half * (FA_TILE_BYTES / 2), &tmap_k, hk * FA_D + half * 64,
                                b * P.Tk + j * FA_BN, &k_full[s]);
                if (j >= FA_KV_STAGES && !mbar_wait(&v_empty[s], ph ^ 1, &abort_flag, P.err, TC_TIMEOUT_EMPTY)) { issued = j + 1; break; }
                mbar_expect_tx(&v_full[s], FA_TILE_BYTES);
                for (int half = 0; half < 2; ++half)
                    tma_load_2d(v_smem + s * FA_TILE_BYTES + half * (FA_TILE_BYTES / 2), &tmap_v, hk * FA_D + half * 64,
                                b * P.Tk + j * FA_BN, &v_full[s]);
                issued = j + 1;
            }
            if (abort_flag) {  // let the copies in flight land before the CTA exits (bounded)
                const long long t_start = clock64();
                for (int j = max(0, issued - FA_KV_STAGES); j < issued; ++j) {
                    while (!mbar_try_wait(&k_full[j % FA_KV_STAGES], (j / FA_KV_STAGES) & 1) && clock64() - t_start < WAIT_LIMIT_CYCLES) {}
                    while (!mbar_try_wait(&v_full[j % FA_KV_STAGES], (j / FA_KV_STAGES) & 1) && clock64() - t_start < WAIT_LIMIT_CYCLES) {}
                }
                while (!mbar_try_wait(&q_full, 0) && clock64() - t_start < WAIT_LIMIT_CYCLES) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc_bf16(FA_BM, FA_BN, 0, 0);  // both operands K-major (head_dim contiguous)
            constexpr uint32_t idesc_pv = instr_desc_bf16(FA_BM, FA_D, 0, 1);   // V is N-contiguous: MN-major B
            bool ok = mbar_wait(&q_full, 0, &abort_flag, P.err, TC_TIMEOUT_FULL);
            // S_t(j) = Q_t . K(j)^T into the S columns of tile t (overwrites P_t(j-1): the tensor pipe runs the MMAs of
            // this thread in issue order, so the P.V product issued before it has read P by then)
            auto issue_s = [&](int t, uint32_t k_addr) {
                const uint32_t q_addr = smem_u32(q_smem + t * FA_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < FA_D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * (FA_TILE_BYTES / 2);
                    mma_ss(tmem_base + S_COL[t], smem_desc_sw128(q_addr + off) + (uint64_t)((kk % 4) * 2),
                           smem_desc_sw128(k_addr + off) + (uint64_t)((kk % 4) * 2), idesc_qk, kk > 0 ? 1u : 0u);
                }
                mma_commit(&s_full[t]);
            };
            // The scores run one key tile ahead of the P.V products: S_t(j+1) is issued right after O_t += P_t(j).V(j),
            // so the softmax of one query tile overlaps the softmax of the other instead of alternating with it.
            if (ok && n_max > 0) {
                ok = mbar_wait(&k_full[0], 0, &abort_flag, P.err, TC_TIMEOUT_FULL);
                tc_fence_after();
                if (ok) {
                    const uint32_t k_addr = smem_u32(k_smem);
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                        if (n_tiles[t] > 0) issue_s(t, k_addr);
                    mma_commit(&k_empty[0]);
                }
            }
            for (int j = 0; j < n_max && ok; ++j) {
                const int s = j % FA_KV_STAGES, s1 = (j + 1) % FA_KV_STAGES;
                const uint32_t ph = (j / FA_KV_STAGES) & 1, ph1 = ((j + 1) / FA_KV_STAGES) & 1;
                const bool more = j + 1 < n_max;
                if (!mbar_wait(&v_full[s], ph, &abort_flag, P.err, TC_TIMEOUT_FULL)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(v_smem + s * FA_TILE_BYTES);
                const uint32_t k_addr = smem_u32(k_smem + s1 * FA_TILE_BYTES);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j < n_tiles[t]) {
                        if (!mbar_wait(&p_ready[t], j & 1, &abort_flag, P.err, TC_TIMEOUT_MISC)) { ok = false; break; }
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < FA_BN / 16; ++kk) {
                            // 16 keys = two 8-row groups of 1024 bytes; the two 64-column halves of V are 16 KB apart
                            const uint64_t v_desc = smem_desc_sw128_mn(v_addr + kk * 2048, FA_TILE_BYTES / 2);
                            mma_ts(tmem_base + O_COL[t], tmem_base + S_COL[t] + kk * 8, v_desc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    if (t == 0 && more) {
                        if (!mbar_wait(&k_full[s1], ph1, &abort_flag, P.err, TC_TIMEOUT_FULL)) { ok = false; break; }
                        tc_fence_after();
                    }
                    if (j + 1 < n_tiles[t]) issue_s(t, k_addr);
                }
                if (!ok) break;
                mma_commit(&v_empty[s]);
                if (more) mma_commit(&k_empty[s1]);
            }
            if (ok) mma_commit(&o_done);
        }
    } else {
        // ---- softmax / correction / epilogue: one thread per query row
        const int t = (warp - 2) / 4;       // query tile
        const int quad = warp & 3;          // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;   // row in the tile = TMEM lane
        const int qi = q0 + t * FA_BM + row;
        const int qpos = qi + shift;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t s_addr = lane_addr + S_COL[t], o_addr = lane_addr + O_COL[t];
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles[t] && ok; ++j) {
            if (!mbar_wait(&s_full[t], j & 1, &abort_flag, P.err, TC_TIMEOUT_ACC)) { ok = false; break; }
            tc_fence_after();
            // the whole score row of this thread: four TMEM loads in flight, one wait
            uint32_t sr[FA_BN];
#pragma unroll
            for (int c = 0; c < FA_BN; c += 32) tmem_ld32(s_addr + c, reinterpret_cast<uint32_t(&)[32]>(sr[c]));
            tmem_ld_wait();
            float sv[FA_BN];
#pragma unroll
            for (int i = 0; i < FA_BN; ++i) sv[i] = __uint_as_float(sr[i]);
            const int key0 = j * FA_BN;
            const bool needs_mask = (P.causal && key0 + FA_BN - 1 > q0 + t * FA_BM + shift) || key0 + FA_BN > P.Tk;
            if (needs_mask) {
#pragma unroll
                for (int i = 0; i < FA_BN; ++i)
                    if ((P.causal && key0 + i > qpos) || key0 + i >= P.Tk) sv[i] = -INFINITY;
            }
            // scores stay unscaled in registers; the scale (> 0, log2 domain) is applied inside the exponent's FMA
            // eight independent chains instead of one 127-deep dependency chain (two warps per scheduler: the row needs ILP)
            float mxs[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) mxs[k] = sv[k];
#pragma unroll
            for (int i = 8; i + 16 <= FA_BN; i += 16)
#pragma unroll
                for (int k = 0; k < 8; ++k) mxs[k] = fmax3(mxs[k], sv[i + k], sv[i + 8 + k]);
#pragma unroll
            for (int k = 0; k < 8; ++k) mxs[k] = fmaxf(mxs[k], sv[FA_BN - 8 + k]);
            float mx = fmaxf(fmax3(mxs[0], mxs[1], mxs[2]), fmaxf(fmax3(mxs[3], mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
            mx *= P.scale_log2;
            // tcgen05.ld / st are warp-collective: the decision to touch the accumulator is taken per warp,
            // each lane then applies its own factor (1 for the rows whose maximum did not move)
            const bool grow = mx > m_ref + FA_RESCALE_THRESHOLD;
            if (__any_sync(0xffffffffu, grow)) {
                // raise the reference maximum; the accumulated O and l shrink by 2^(old - new)
                const float alpha = grow ? ex2_approx(m_ref - mx) : 1.0f;
                if (j > 0) {
#pragma unroll
                    for (int c = 0; c < FA_D; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(o_addr + c, r);
                        tmem_ld_wait();
                        uint32_t w[16];
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(__uint_as_float(r[half * 16 + i]) * alpha);
                            tmem_st16(o_addr + c + half * 16, w);
                        }
                    }
                }
                if (grow) {
                    l *= alpha;
                    m_ref = mx;
                }
            }
            // p = 2^(s - m_ref), packed to bf16 pairs, written over the first 64 columns of S
            uint64_t ls2[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) ls2[k] = pack2(0.0f, 0.0f);
            const uint64_t neg_m2 = pack2(-m_ref, -m_ref), sc2 = pack2(P.scale_log2, P.scale_log2);
#pragma unroll
            for (int c = 0; c < FA_BN / 2; c += 16) {
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint64_t x2 = ffma2(pack2(sv[2 * (c + i)], sv[2 * (c + i) + 1]), sc2, neg_m2);
                    float p0, p1;
                    if ((i & 3) < POLY) {
                        ex2_poly2(x2, p0, p1);
                    } else {
                        float x0, x1;
                        unpack2(x2, x0, x1);
                        p0 = ex2_approx(x0);
                        p1 = ex2_approx(x1);
                    }
                    ls2[i & 3] = fadd2(ls2[i & 3], pack2(p0, p1));
                    w[i] = pack_bf16x2(p0, p1);
                }
                tmem_st16(s_addr + c, w);
            }
            float la, lb;
            unpack2(fadd2(fadd2(ls2[0], ls2[1]), fadd2(ls2[2], ls2[3])), la, lb);
            const float lsum = la + lb;
            l += lsum;
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_ready[t]);
        }
        // epilogue: O / l -> bf16 -> global
        if (ok && n_tiles[t] > 0) ok = mbar_wait(&o_done, 0, &abort_flag, P.err, TC_TIMEOUT_ACC);
        tc_fence_after();
        if (ok && n_tiles[t] > 0) {  // warp-uniform: the TMEM loads are collective, only the stores are per row
            const float inv = 1.0f / l;
            const bool store = qi < P.Tq;
            __nv_bfloat16* dst = P.out + (long long)(b * P.Tq + (store ? qi : 0)) * P.out_rs + (long long)h * FA_D;
#pragma unroll
            for (int c = 0; c < FA_D; c += 32) {
                uint32_t r[32];
                tmem_ld32(o_addr + c, r);
                tmem_ld_wait();
                if (store) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        o.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        o.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        o.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + i) = o;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

jsm_status flash_prefill_launch(const void* q, const void* k, const void* v, void* out, int batch, int Tq, int Tk, int Hq, int Hkv,
                                int causal, float scale, const float* rope, cudaStream_t st, long long q_rs, long long kv_rs,
                                long long o_rs) {
    if (rope) JSM_FAIL(JSM_UNSUPPORTED, "flash_prefill: q and k must already be rotated");
    if (!(scale > 0.0f)) JSM_FAIL(JSM_UNSUPPORTED, "flash_prefill: the softmax scale (%g) must be positive", (double)scale);
    if (q_rs <= 0) q_rs = (long long)Hq * FA_D;
    if (kv_rs <= 0) kv_rs = (long long)Hkv * FA_D;
    if (o_rs <= 0) o_rs = (long long)Hq * FA_D;
    if (o_rs % 8 || (reinterpret_cast<uintptr_t>(out) & 15)) JSM_FAIL(JSM_INVALID_ARG, "flash_prefill: output must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    jsm_status s = make_tmap_bf16_2d(&mq, q, (uint64_t)batch * Tq, (uint64_t)Hq * FA_D, (uint64_t)q_rs, FA_BM, 64);
    if (s != JSM_OK) return s;
    s = make_tmap_bf16_2d(&mk, k, (uint64_t)batch * Tk, (uint64_t)Hkv * FA_D, (uint64_t)kv_rs, FA_BN, 64);
    if (s != JSM_OK) return s;
    s = make_tmap_bf16_2d(&mv, v, (uint64_t)batch * Tk, (uint64_t)Hkv * FA_D, (uint64_t)kv_rs, FA_BN, 64);
    if (s != JSM_OK) return s;
    FlashParams P;
    P.Tq = Tq; P.Tk = Tk; P.Hq = Hq; P.Hkv = Hkv; P.causal = causal;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.out = reinterpret_cast<__nv_bfloat16*>(out);
    P.out_rs = o_rs;
    P.err = tc_error_word();
    const size_t smem = (size_t)(2 + 2 * FA_KV_STAGES) * FA_TILE_BYTES + 1024;
    static bool attr_done = false;
    if (!attr_done) {
        JSM_CUDA_CHECK(cudaFuncSetAttribute(flash_prefill_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_done = true;
    }
    dim3 grid((Tq + 2 * FA_BM - 1) / (2 * FA_BM), Hq, batch);
    // a quarter of the exponentials on the FMA pipe: the measured optimum (none: MUFU-bound, half: issue-bound)
    flash_prefill_kernel<1><<<grid, FA_THREADS, smem, st>>>(mq, mk, mv, P);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

}  // namespace jsm
