// bf16 projections over PACKED weights: Y[t,n] = sum_k X[t,k] * W[n,k] with fp32 accumulation, the device form of
// weight_net_t::forward (mat_net_t.hpp:38-49, Y = W.X + b with W stored [out, in]) for weights that stay constant
// between calls (inference).
//
// Why a packed layout.  A [out, in] row-major weight matrix read in 128 x 64 tiles touches 128 different rows per
// tile, 128 bytes each, 2*K bytes apart: every DRAM page is opened for 128 bytes.  Packed once at load time, a tile
// (128 output features x 64 k, 16 KB) is ONE contiguous block that already has the shared-memory image the tensor
// core wants (128-byte swizzle), the k-blocks of a tile follow each other, and the tiles follow each other.  The whole
// matrix is then a single linear stream and a CTA's share of it is one contiguous byte range fetched with plain bulk
// copies (cp.async.bulk), 16 KB per request.
//
// Work split ("stream-K").  The matrix is n_tiles * kbt units (tile, k-block) in stream order; CTA c of G owns units
// [c*U/G, (c+1)*U/G).  A CTA therefore finishes the tail of one tile, possibly some whole tiles, and the head of
// another.  Whole tiles are written straight from the accumulator; a tile shared by several CTAs is reduced through
// fp32 partials in a workspace: every contributor stores its partial in its own slot, the one that arrives last
// (a counter per tile) adds the slots in slot order, so the sum does not depend on the arrival order, and runs the
// epilogue.  All SMs stream the same number of bytes whatever the shape.
//
// Kernel roles (224 threads): warp 0 streams W (bulk copies), warp 6 the tiles of X (TMA): two issuing threads, because a
// thread's rate of copy requests, not the bytes in flight, bounds the stream; warp 1 MMA issuer
// (tcgen05.mma 128 x BN x 16, accumulators in TMEM, two accumulator buffers so that the epilogue of one segment
// overlaps the MMAs of the next), warps 2-5 epilogue (tcgen05.ld, one TMEM lane = one packed row per thread).
// Chained launches: the W stream does not depend on the predecessor kernel, so the first ring of W tiles is
// requested (and more is prefetched into L2) before griddepcontrol.wait; X, R, Y and the workspace come after it.
#include "tc_utils.cuh"
#include "linear_bf16.cuh"
#include <math.h>
#include <mutex>
#include <algorithm>
#include <stdlib.h>

namespace jsm {

using namespace tc;

constexpr int PK_TILE_BYTES = 128 * 64 * 2;  // one packed unit: 128 rows x 64 k, bf16
constexpr int PK_THREADS = 224;
constexpr int PK_MAX_STAGES = 12;

__device__ __noinline__ float pk_gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float pk_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }  // 2 ulp division: short code

// 1-D bulk copy global -> shared (this CTA), completion counted in bytes on `bar`; both addresses 16-byte aligned
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes) : "memory");
}

struct PkParams {
    int T, N, K;          // tokens (<= BN), output features (paired: gate features), reduction length
    int n_tiles, kbt;     // tiles of 128 packed rows, k-blocks of 64 per tile
    int local_epi;        // whole tiles that end a CTA's range use the vectorised epilogue through shared memory
    int paired;           // epilogue silu(gate) * up over a paired tile
    int epilogue;         // LIN_* (LIN_SILU_MUL exactly when paired)
    int out_f32;
    const float* bias;
    const __nv_bfloat16* R;
    void* Y;
    const uint8_t* Wp;
    float* ws;            // [n_tiles][max_slots][T][128] fp32 partials
    int* counters;        // [n_tiles], zero between launches
    int max_slots;
    int* err;
    int pf_units;         // units beyond the ring that are prefetched into L2 up front
    int stages;
    int cluster_s;        // > 1: aligned split, the cluster_s CTAs of a tile form a cluster and fold through shared memory
    int pair_ok;          // K is a multiple of 64: two k-blocks of X can be fetched as one 3-D tile
    const float* ssq_in;  // [ssq_in_tiles][ssq_stride] per-tile sums of squares of X's rows (null: X is used as it is)
    int ssq_in_tiles;
    int ssq_stride;       // row pitch of ssq_in and ssq_out (tokens of the whole call)
    float inv_d, eps;     // 1 / (features of X), epsilon under the square root
    float* ssq_out;       // [n_tiles][ssq_stride]: sums of squares of this launch's outputs per tile and token, or null
    unsigned long long* trace;  // optional timeline: 8 time stamps (globaltimer, ns) per CTA of this launch
    // tensor-parallel exchange fused into the launch (TpFuse in linear_bf16.cuh; protocol in tp_comm.cu)
    int tp_mode;                // 0 none, 1 push the outputs to every rank's slot, 2 reduce the slots into h before X is read
    int tp_n, tp_rank;
    int tp_site, tp_n_sites;
    const int* tp_pass;
    int* tp_state;              // local: [0] folding CTAs done, [1] tiles of h reduced (self-resetting); [2] epoch up to which h is reduced
    int tp_expect;              // push: folding CTAs of this launch
    int tp_inband;              // the pushed words carry the exchange's epoch ({two bf16, epoch} per 8 bytes): no flags
    uint8_t* tp_dst[8];
    int* tp_flag[8];
    const uint8_t* tp_slots;
    size_t tp_slot_stride;
    const int* tp_flags;
    __nv_bfloat16* tp_h;
    float* tp_ssq;
    long long tp_wait;
};

constexpr int TP_TIMEOUT_CODE = 16;  // error word code of an exchange whose peers did not arrive in time (as in tp_comm.cu)
__device__ __forceinline__ void pk_st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int pk_ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int pk_ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 pk_ld_cg_v4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
// the words of an in-band exchange carry their own epoch: they are read and written with volatile (relaxed, system scope)
// 16-byte accesses, each 8-byte half of which is one word
__device__ __forceinline__ uint4 pk_ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int pk_ld_volatile(const void* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pk_st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// generic-proxy writes to global memory (other CTAs' stores of h) before the copy engine's reads of the same bytes
__device__ __forceinline__ void pk_fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// One thread waits (bounded) until the word *p has reached epoch E; epochs only grow, the comparison is wrap-safe.  The
// polls are spaced out: thousands of spinning threads would slow down the very kernels they wait for.  A wait that runs out
// records the error and returns.
__device__ __forceinline__ void pk_wait_epoch(const int* p, int E, long long limit, int* err) {
    const long long t0 = clock64();
    while ((int)(pk_ld_acquire_gpu(p) - E) < 0) {
        __nanosleep(64);
        if (clock64() - t0 > limit) {
            if (err) atomicCAS(err, 0, TP_TIMEOUT_CODE);
            break;
        }
    }
}
// local state words of the fused exchange: [0] folding CTAs of a pushing launch done, [1] tiles of h reduced (both
// self-resetting), [2] epoch up to which h is completely reduced

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define PK_TRACE(slot)                                                              \
    do {                                                                            \
        if (P.trace) P.trace[(size_t)blockIdx.x * 8 + (slot)] = global_ns();        \
    } while (0)

// unit range of CTA c: [c*U/G, (c+1)*U/G)
__host__ __device__ inline long long pk_begin(long long c, long long U, long long G) { return c * U / G; }
// CTA that owns unit u: the largest c with c*U/G <= u
__host__ __device__ inline int pk_owner(long long u, long long U, long long G) { return (int)(((u + 1) * G + U - 1) / U - 1); }
// The kernel's own copies in 32-bit arithmetic (a 64-bit division is a routine of about a hundred instructions, and the
// kernel's code is fetched cold by every launch).  The host checks (U + 1) * (G + 1) < 2^31 before it launches.
__device__ __forceinline__ int pk_begin32(unsigned c, unsigned U, unsigned G) { return (int)(c * U / G); }
__device__ __forceinline__ int pk_owner32(unsigned u, unsigned U, unsigned G) { return (int)(((u + 1u) * G + U - 1u) / U) - 1; }

// ---- thread-block cluster helpers: the CTAs that share a tile exchange their partials through distributed shared memory
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// Units of the stream a stage holds: two consecutive k-blocks of one tile when the segment has two left (one 32 KB
// request instead of two of 16 KB: the copy engine's rate of requests, not the bytes in flight, bounds a CTA's stream),
// else one.  Producer and MMA issuer walk the same sequence.
__device__ __forceinline__ int pk_chunk(int pair_ok, int left) { return (pair_ok && left >= 2) ? 2 : 1; }

// CL: the instantiation contains the cluster path (launches of 32 tokens and more); the few-token kernel carries none of it.
// TPM: what the instantiation contains of the fused tensor-parallel exchange (nothing / push / reduce / both).  Code that a
// launch never runs still costs it - the step time follows the size of the image of every launch, 0.1 - 0.2 % per KB - so
// launches without an exchange run an image without it, and the common launches have images of their own (PRM below).
template <int BN, bool CL, int TPM, int PRM>
__global__ void __launch_bounds__(PK_THREADS, 1)
    linear_packed_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_x2, PkParams P) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int B_BYTES = BN * 128;  // BN tokens x 64 k, bf16
    constexpr int STAGE_BYTES = 2 * (PK_TILE_BYTES + B_BYTES);  // [W unit 0][W unit 1][X block 0][X block 1]
    constexpr int X_OFF = 2 * PK_TILE_BYTES;
    constexpr int TMEM_NEED = 2 * BN;  // two accumulator buffers
    constexpr int TMEM_COLS = TMEM_NEED < 32 ? 32 : TMEM_NEED;
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns: power of two, at most 512");

    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[PK_MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[PK_MAX_STAGES];
    __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;
    __shared__ int is_last_smem[2];
    // ROWS: whole tiles that do not end the CTA's range take the row-per-thread epilogue straight from the accumulator (the
    // stage ring is busy).  The images of up to 64 tokens have a staging tile of their own instead and send every whole
    // tile through the vectorised epilogue: one epilogue, a third less code to fetch in the tail that runs once per launch.
    constexpr bool ROWS = BN >= 128;
    __shared__ float pair_smem[ROWS ? 64 * 17 : 1];   // paired epilogue: up values of 16 token columns, padded rows
    __shared__ float row_scale[256];                  // 1 / rms of every token when the RMSNorm is fused into this projection
    __shared__ float ssq_part[ROWS ? 4 * 256 : 1];    // per-warp sums of squares of a whole tile's outputs
    __shared__ __align__(16) float stage_small[ROWS ? 4 : BN * 128];  // up to 64 tokens: a whole tile's accumulator
    __shared__ int tp_ok_smem;            // reduce: every peer's flag arrived in time

    // PRM: what the image can do.  -1: everything; 0 / 1: plain tiles only / gate-up pairs only (what the other kind needs is
    // not in it); 2, 3, 4: exactly one projection of a LLaMA-style decoder step each - 2: plain tiles, fused RMSNorm row
    // scale, no bias, no activation, bf16 out (qkv); 3: plain tiles, residual added, per-tile sums of squares written, bf16
    // out (wo, down); 4: gate-up pairs with the row scale, bf16 out.  The host picks the image from the arguments; a launch
    // pays for the size of its image, so the common launches get the smallest ones.
    // TPM: 0 = no tensor-parallel exchange in the image, 3 = push or reduce, with flags or in-band epochs, as the launch says,
    // 1 / 2 = it pushes its outputs / reduces the ranks' slots into its token operand first, with flags, 4 / 5 = the same
    // with in-band epochs.
    // PRM 5: the pushing projection (plain tiles, bf16, nothing else).
    const bool tp_push = TPM == 1 || TPM == 4 || (TPM == 3 && P.tp_mode == 1);
    const bool tp_reduce = TPM == 2 || TPM == 5 || (TPM == 3 && P.tp_mode == 2);
    const bool tp_inband = BN == 16 && (TPM == 4 || TPM == 5 || (TPM == 3 && P.tp_inband != 0));  // (at most 16 tokens)
    constexpr bool FIX = PRM >= 2;
    const bool paired = PRM < 0 ? P.paired != 0 : (PRM == 1 || PRM == 4);
    const bool has_ssq_in = FIX ? (PRM == 2 || PRM == 4) : P.ssq_in != nullptr;
    const bool f32o = FIX ? false : P.out_f32 != 0;
    const float* const biasp = FIX ? nullptr : P.bias;
    const int epi = FIX ? (PRM == 3 ? LIN_RESIDUAL : PRM == 4 ? LIN_SILU_MUL : LIN_NONE) : P.epilogue;
    chain_trigger();
    if (threadIdx.x == 0) PK_TRACE(0);  // CTA resident
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = P.stages;
    const unsigned U = (unsigned)(P.n_tiles * P.kbt), G = gridDim.x;
    const int u_begin = pk_begin32(blockIdx.x, U, G), u_end = pk_begin32(blockIdx.x + 1, U, G);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 2);  // the W producer and the X producer each arrive with their bytes
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_x2);
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
        // ---- producer ------------------------------------------------------------------------------------
        if (lane == 0) {
            const uint8_t* wsrc = P.Wp + (size_t)u_begin * PK_TILE_BYTES;
            // weights first: the ring is filled with W before the predecessor kernel has finished (constant weights);
            // the X blocks of the same stages follow once it has
            // loop state kept incrementally (k-block within the tile, stage, phase): no division per request
            int rem = u_end - u_begin, kb = u_begin % P.kbt;
            int i = 0, s = 0;
            uint32_t ph = 0;
            const uint8_t* src = wsrc;
            auto issue = [&]() {
                const int n = pk_chunk(P.pair_ok, min(P.kbt - kb, rem));
                mbar_expect_tx(&full_bar[s], (uint32_t)n * PK_TILE_BYTES);
                bulk_load(tiles + (size_t)s * STAGE_BYTES, src, (uint32_t)n * PK_TILE_BYTES, &full_bar[s]);
                src += (size_t)n * PK_TILE_BYTES;
                rem -= n;
                kb += n;
                if (kb == P.kbt) kb = 0;
                ++i;
                if (++s == stages) { s = 0; ph ^= 1; }
            };
            while (rem > 0) {  // the first ring goes out at once: before the predecessor kernel has finished
                if (i >= stages && !mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, P.err, TC_TIMEOUT_EMPTY)) break;
                issue();
                if (i == stages) PK_TRACE(1);  // first ring of W requested
            }
            const int issued = i;
            if (abort_flag) {  // let the copies in flight land before the CTA exits (bounded)
                const long long t_start = clock64();
                for (int j = max(0, issued - stages); j < issued; ++j)
                    while (!mbar_try_wait(&full_bar[j % stages], (j / stages) & 1) && clock64() - t_start < WAIT_LIMIT_CYCLES) {}
            }
        }
        if (CL && P.cluster_s > 1) {  // every thread of the cluster takes part in its two barriers (see the epilogue)
            __syncwarp();
            cluster_sync_all();
            cluster_sync_all();
        }
    } else if (warp == 6) {
        // ---- X producer: the token blocks of every stage, once the predecessor kernel has written them --------------
        if (lane == 0) {
            if (tp_reduce) {
                // X is the residual stream that the first CTAs of this launch are completing (h += the ranks' slots).  Its
                // readiness is announced through an epoch word, not by the end of the predecessor kernel; then the generic
                // writes of the reducing CTAs are ordered before the copy engine's reads.  Nothing else the X producer
                // touches belongs to another kernel, so it does not wait for the predecessor.
                const int E = *reinterpret_cast<const volatile int*>(P.tp_pass) * P.tp_n_sites + P.tp_site + 1;
                pk_wait_epoch(P.tp_state + 2, E, P.tp_wait, P.err);
                pk_fence_proxy_async();
            } else chain_wait();
            PK_TRACE(2);  // predecessor complete (fused exchange: h complete)
            int rem = u_end - u_begin, kb = u_begin % P.kbt;
            int i = 0, s = 0;
            uint32_t ph = 0;
            while (rem > 0) {
                if (i >= stages && !mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, P.err, TC_TIMEOUT_EMPTY)) break;
                const int n = pk_chunk(P.pair_ok, min(P.kbt - kb, rem));
                uint8_t* xs = tiles + (size_t)s * STAGE_BYTES + X_OFF;
                mbar_expect_tx(&full_bar[s], (uint32_t)n * B_BYTES);
                if (n == 2) tma_load_3d(xs, &tmap_x2, 0, 0, kb, &full_bar[s]);
                else tma_load_2d(xs, &tmap_x, kb * 64, 0, &full_bar[s]);
                rem -= n;
                kb += n;
                if (kb == P.kbt) kb = 0;
                ++i;
                if (++s == stages) { s = 0; ph ^= 1; }
            }
        }
        if (CL && P.cluster_s > 1) {
            __syncwarp();
            cluster_sync_all();
            cluster_sync_all();
        }
    } else if (warp == 1) {
        // ---- MMA issuer ------------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(128, BN);
            bool ok = true;
            int it = 0, seg = 0, s = 0;
            uint32_t ph = 0;
            int rem = u_end - u_begin, kb0 = u_begin % P.kbt;
            while (rem > 0 && ok) {
                const int len = min(P.kbt - kb0, rem);
                const int buf = seg & 1;
                if (seg >= 2) {
                    // the epilogue must have drained this buffer's previous segment
                    if (!mbar_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1, &abort_flag, P.err, TC_TIMEOUT_MISC)) { ok = false; break; }
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int j = 0; j < len; ++it) {
                    const int n = pk_chunk(P.pair_ok, len - j);
                    if (!mbar_wait(&full_bar[s], ph, &abort_flag, P.err, TC_TIMEOUT_FULL)) { ok = false; break; }
                    if (it == 0) PK_TRACE(3);  // first stage landed
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                    for (int q = 0; q < n; ++q) {
                        const uint64_t a_desc = smem_desc_sw128(a_addr + q * PK_TILE_BYTES);
                        const uint64_t b_desc = smem_desc_sw128(a_addr + X_OFF + q * B_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma_ss(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (j > 0 || q > 0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit(&empty_bar[s]);
                    j += n;
                    if (++s == stages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                mma_commit(&acc_full[buf]);
                rem -= len;
                kb0 = 0;  // every segment after the first starts a tile
                ++seg;
            }
            PK_TRACE(4);  // last MMA issued
        }
        if (CL && P.cluster_s > 1) {
            __syncwarp();
            cluster_sync_all();
            cluster_sync_all();
        }
    } else {
        // ---- epilogue: warps 2..5 own the TMEM lane quadrants warp % 4 ------------------------------------------
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // packed row of the tile = TMEM lane
        const int etid = threadIdx.x - 64; // 0..127 within the epilogue warps
        const bool want_ssq = FIX ? PRM == 3 : (!paired && P.ssq_out != nullptr);  // plain tiles only (checked on the host)
        bool ok = true;
        int seg = 0, cl_syncs = 0;
        // R, Y, the row statistics, the workspace and the counters belong to the stream's other kernels: wait for the
        // predecessor now (the MMA warp is busy with the weight stream meanwhile) and prepare what does not need the accumulator.
        if (tp_reduce) {
            // ---- tensor-parallel exchange, consumer side.  Every rank (this one included) has pushed its block of the
            // previous projection's output into its slot of this rank's buffer and released the exchange's epoch to this
            // rank's flag word for it.  The first CTAs of the launch (one per 128-column tile of h, while all CTAs stream
            // their weights) wait for the flags - not for the end of the predecessor kernel: its own flag says that its
            // block is complete - add the slots in rank order to h (local loads only), store h and the tile's sums of
            // squares and publish the tile's epoch; every CTA waits for all tiles before it reads the statistics.
            const int red_tiles = (P.K + 127) / 128;
            const int E = *reinterpret_cast<const volatile int*>(P.tp_pass) * P.tp_n_sites + P.tp_site + 1;
            if ((int)blockIdx.x < red_tiles) {
                if (etid == 0) tp_ok_smem = 1;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid < P.tp_n) {
                    // flags: the rank's flag word.  In-band: the epoch of the first word of this CTA's tile in the rank's slot
                    // (a cheap probe that keeps the polling traffic small; the loads below check every word they take)
                    const int* flag = tp_inband ? reinterpret_cast<const int*>(P.tp_slots + (size_t)etid * P.tp_slot_stride +
                                                                               (size_t)blockIdx.x * 128 * 4) + 1
                                                : P.tp_flags + etid;
                    const long long t0 = clock64();
                    while ((int)((tp_inband ? pk_ld_volatile(flag) : pk_ld_acquire_sys(flag)) - E) < 0) {
                        __nanosleep(64);
                        if (clock64() - t0 > P.tp_wait) {
                            tp_ok_smem = 0;
                            if (P.err) atomicCAS(P.err, 0, TP_TIMEOUT_CODE);
                            break;
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool tp_ok = tp_ok_smem != 0;  // a rank that never arrived: h stays as it is, the error word says so
                const int n_vec = P.T * 16;  // 16-byte vectors of one tile: 16 per token
                int handled = 0;
                for (int j = blockIdx.x; j < red_tiles; j += gridDim.x, ++handled) {
                    for (int v0 = 0; v0 < n_vec; v0 += 128) {  // warp-uniform trip count: the shuffles below need every lane
                        const int v = v0 + etid;
                        const int t = v >> 4, c = j * 128 + (v & 15) * 8;
                        const bool in_range = v < n_vec && c < P.K;
                        float sq = 0.0f;
                        if (in_range) {
                            const size_t off = ((size_t)t * P.K + c) * 2;
                            uint4 o = pk_ld_cg_v4(reinterpret_cast<const uint8_t*>(P.tp_h) + off);
                            bool ready = tp_ok;
                            uint4 w[8];
                            if (tp_ok && tp_inband) {
                                // 8 bf16 of a slot = four words {two bf16, epoch} = 32 bytes; all ranks' loads go out together,
                                // and again until every word is of this exchange (or later: the peers never run ahead by a
                                // whole buffer cycle); the load that polls is the load that fetches
                                const uint8_t* src = P.tp_slots + ((size_t)t * P.K + c) * 4;
                                const long long t0 = clock64();
                                while (true) {
                                    int oldest = 0;
#pragma unroll
                                    for (int r = 0; r < 8; ++r) {
                                        if (r < P.tp_n) {
                                            const uint4 a = pk_ld_volatile_v4(src + (size_t)r * P.tp_slot_stride);
                                            const uint4 b = pk_ld_volatile_v4(src + (size_t)r * P.tp_slot_stride + 16);
                                            w[r] = make_uint4(a.x, a.z, b.x, b.z);
                                            oldest = min(oldest, min(min((int)a.y - E, (int)a.w - E), min((int)b.y - E, (int)b.w - E)));
                                        }
                                    }
                                    if (oldest >= 0) break;
                                    if (clock64() - t0 > P.tp_wait) {  // (a rank that stopped in the middle of its pushes)
                                        ready = false;
                                        if (P.err) atomicCAS(P.err, 0, TP_TIMEOUT_CODE);
                                        break;
                                    }
                                    __nanosleep(32);
                                }
                            } else if (tp_ok) {
#pragma unroll
                                for (int r = 0; r < 8; ++r)
                                    if (r < P.tp_n) w[r] = pk_ld_cg_v4(P.tp_slots + (size_t)r * P.tp_slot_stride + off);
                            }
                            if (ready) {
                                float sm[8];
#pragma unroll
                                for (int q = 0; q < 8; ++q) sm[q] = 0.0f;
                                // rank order; one copy of the adds: the slots take turns in w[0] (short code, see the kernel's
                                // template parameters)
#pragma unroll 1
                                for (int r = 0; r < P.tp_n; ++r) {
                                    sm[0] += bf16lo(w[0].x); sm[1] += bf16hi(w[0].x); sm[2] += bf16lo(w[0].y); sm[3] += bf16hi(w[0].y);
                                    sm[4] += bf16lo(w[0].z); sm[5] += bf16hi(w[0].z); sm[6] += bf16lo(w[0].w); sm[7] += bf16hi(w[0].w);
#pragma unroll
                                    for (int q = 0; q < 7; ++q) w[q] = w[q + 1];
                                }
                                // the rank-local products were rounded to bf16 when they were pushed; their sum is rounded once
                                // more (the all-reduce of a bf16 buffer) and then added to the residual stream
                                uint32_t sb[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) sb[q] = pack_bf16x2(sm[2 * q], sm[2 * q + 1]);
                                const uint4 hw = o;
                                o.x = pack_bf16x2(bf16lo(hw.x) + bf16lo(sb[0]), bf16hi(hw.x) + bf16hi(sb[0]));
                                o.y = pack_bf16x2(bf16lo(hw.y) + bf16lo(sb[1]), bf16hi(hw.y) + bf16hi(sb[1]));
                                o.z = pack_bf16x2(bf16lo(hw.z) + bf16lo(sb[2]), bf16hi(hw.z) + bf16hi(sb[2]));
                                o.w = pack_bf16x2(bf16lo(hw.w) + bf16lo(sb[3]), bf16hi(hw.w) + bf16hi(sb[3]));
                                __stcg(reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(P.tp_h) + off), o);
                            }
                            const float f[8] = {bf16lo(o.x), bf16hi(o.x), bf16lo(o.y), bf16hi(o.y), bf16lo(o.z), bf16hi(o.z), bf16lo(o.w), bf16hi(o.w)};
#pragma unroll
                            for (int q = 0; q < 8; ++q) sq += f[q] * f[q];
                        }
#pragma unroll
                        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);  // the 16 lanes of a token
                        if (v < n_vec && (lane & 15) == 0) __stcg(P.tp_ssq + (size_t)j * P.ssq_stride + t, sq);
                    }
                }
                // the barrier orders every thread's stores before thread 0, whose fences (cumulative) order them before its
                // count; the CTA that completes h publishes the epoch: for the other CTAs' loads and, through the proxy
                // fences, for their copy engines' reads of h
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0) {
                    asm volatile("fence.acq_rel.gpu;" ::: "memory");
                    pk_fence_proxy_async();
                    int old;
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(P.tp_state + 1), "r"(handled) : "memory");
                    if (old + handled == red_tiles) {
                        P.tp_state[1] = 0;  // ready for the next exchange
                        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(P.tp_state + 2), "r"(E) : "memory");
                    }
                }
            }
            if (etid == 0) pk_wait_epoch(P.tp_state + 2, E, P.tp_wait, P.err);
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        chain_wait();
        // the epoch an in-band push writes into its words (the pass number is in memory before any kernel of the pass starts)
        const int tp_epoch = (tp_push && tp_inband) ? *reinterpret_cast<const volatile int*>(P.tp_pass) * P.tp_n_sites + P.tp_site + 1 : 0;
        // Row scale of a fused RMSNorm: X is the un-normalised residual stream and the norm's gain is folded into the packed
        // weights, so y[t, :] = (W' . x[t]) / sqrt(mean(x[t]^2) + eps); the mean comes from the per-tile sums of squares that
        // the kernel which wrote x left behind (added in tile order).
        if (has_ssq_in) {
#pragma unroll 1
            for (int t = etid; t < P.T; t += 128) {
                float q = 0.0f;
                int j = 0;
#pragma unroll 1
                for (; j + 8 <= P.ssq_in_tiles; j += 8) {  // eight loads in flight, added in tile order
                    float v8[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) v8[k] = __ldcg(P.ssq_in + (size_t)(j + k) * P.ssq_stride + t);
#pragma unroll
                    for (int k = 0; k < 8; ++k) q += v8[k];
                }
#pragma unroll 1
                for (; j < P.ssq_in_tiles; ++j) q += __ldcg(P.ssq_in + (size_t)j * P.ssq_stride + t);
                row_scale[t] = rsqrtf(q * P.inv_d + P.eps);  // 2 ulp; the exact 1 / sqrt costs 1.7 KB of code in every launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }  // cluster barriers this thread has taken part in (two per CTA, whatever happens)
        int u = u_begin;
        while (u < u_end && ok) {
            const int tile = u / P.kbt;
            const int kb0 = u - tile * P.kbt;
            const int len = min(P.kbt - kb0, u_end - u);
            const int buf = seg & 1;
            // A shared tile that ends this CTA's range: if every other contributor has already arrived at the tile counter
            // (the usual case: they hold the tile's later k-blocks as their FIRST segment), this CTA is the one that folds,
            // and its own partial need not travel through the workspace - it stays in shared memory.  The counter is read
            // while the accumulator is still being produced.
            // Everything about the segment that does not need the accumulator is worked out before the wait for it: who
            // shares the tile (two divisions) and this thread's place in the vectorised epilogue.  The tail after
            // the last MMA runs once per launch on four warps, so every instruction moved out of it shortens the launch.
            const bool whole = (len == P.kbt);
            const int uf = tile * P.kbt;
            const int c_first = whole ? (int)blockIdx.x : pk_owner32((unsigned)uf, U, G);
            const int c_last = whole ? (int)blockIdx.x : pk_owner32((unsigned)(uf + P.kbt - 1), U, G);
            const int n_contrib = c_last - c_first + 1;
            const int slot = (int)blockIdx.x - c_first;
            const int gshift = paired ? 4 : 5;  // 16 or 32 groups of 4 features per tile
            const int f4 = (etid & ((1 << gshift) - 1)) * 4, tsub = etid >> gshift, TS = 128 >> gshift;
            const int n_f = (paired ? tile * 64 : tile * 128) + f4;
            const bool valid_f = n_f < P.N;
            const float4 bias4 = (biasp && !paired && valid_f) ? *reinterpret_cast<const float4*>(biasp + n_f) : make_float4(0.f, 0.f, 0.f, 0.f);
            const size_t slot_stride = (size_t)P.T * 128;
            const float* tbase = P.ws + (size_t)tile * P.max_slots * slot_stride;
            float* wbase = P.ws + ((size_t)tile * P.max_slots + slot) * slot_stride;
            bool solo = false;
            if (!whole && u + len == u_end && !(CL && P.cluster_s > 1) && P.local_epi) {
                if (etid == 0) {
                    const int nc = n_contrib;
                    int c;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(c) : "l"(P.counters + tile) : "memory");
                    is_last_smem[seg & 1] = (c == nc - 1);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");  // also carries thread 0's acquire to the other threads' loads
                solo = is_last_smem[seg & 1] != 0;
            }
            if (!mbar_wait(&acc_full[buf], (seg >> 1) & 1, &abort_flag, P.err, TC_TIMEOUT_ACC)) { ok = false; break; }
            tc_fence_after();
            const bool scaled = has_ssq_in;
            const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
            // A whole tile that is this CTA's last segment goes through shared memory (the stage ring is free: every MMA
            // of the CTA has completed) and the vectorised epilogue below, whose stores are 8 or 16 bytes per thread and
            // contiguous per token; earlier segments overlap the main loop and keep the row-per-thread epilogue.
            const bool local = whole && (!ROWS || ((u + len == u_end) && P.local_epi));
            bool rows_done = false;
            if constexpr (ROWS) {
            if (whole && !local) {
                rows_done = true;
                // ---- the tile is complete in this CTA: epilogue straight from the accumulator
                if (!paired) {
                    const int n = tile * 128 + row;
                    const bool valid = n < P.N;
                    const float bias = (biasp && valid) ? biasp[n] : 0.0f;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        if (c0 >= P.T) break;
                        uint32_t r[16];
                        tmem_ld16(acc_addr + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = c0 + j;  // warp-uniform
                            if (t < P.T) {
                                float v = __uint_as_float(r[j]);
                                if (scaled) v *= row_scale[t];
                                v += bias;
                                if (epi == LIN_RELU) v = fmaxf(v, 0.0f);
                                else if (epi == LIN_GELU) v = pk_gelu(v);
                                else if ((!paired && epi == LIN_RESIDUAL) && valid) v += __bfloat162float(P.R[(size_t)t * P.N + n]);
                                float stored = v;
                                if (!f32o) {
                                    const __nv_bfloat16 hb = __float2bfloat16_rn(v);
                                    stored = __bfloat162float(hb);
                                    if (valid) reinterpret_cast<__nv_bfloat16*>(P.Y)[(size_t)t * P.N + n] = hb;
                                } else if (valid) {
                                    reinterpret_cast<float*>(P.Y)[(size_t)t * P.N + n] = v;
                                }
                                if (want_ssq) {  // sum of squares of what was stored, over the 128 features of the tile
                                    const float sq = warp_sum(valid ? stored * stored : 0.0f);
                                    if (lane == 0) ssq_part[quad * 256 + t] = sq;
                                }
                            }
                        }
                    }
                    if (want_ssq) {
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        for (int t = etid; t < P.T; t += 128)
                            P.ssq_out[(size_t)tile * P.ssq_stride + t] = (ssq_part[t] + ssq_part[256 + t]) + (ssq_part[512 + t] + ssq_part[768 + t]);
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                } else {
                    // lanes 0..63 hold gate, lanes 64..127 the matching up rows: hand the up values over through shared memory
                    const int f = row & 63;
                    const int n = tile * 64 + f;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        if (c0 >= P.T) break;
                        uint32_t r[16];
                        tmem_ld16(acc_addr + c0, r);
                        tmem_ld_wait();
                        if (row >= 64) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) pair_smem[f * 17 + j] = __uint_as_float(r[j]);
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (row < 64 && n < P.N) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int t = c0 + j;
                                if (t < P.T) {
                                    const float sc = scaled ? row_scale[t] : 1.0f;
                                    const float v = pk_silu(__uint_as_float(r[j]) * sc) * (pair_smem[f * 17 + j] * sc);
                                    if (f32o) reinterpret_cast<float*>(P.Y)[(size_t)t * P.N + n] = v;
                                    else reinterpret_cast<__nv_bfloat16*>(P.Y)[(size_t)t * P.N + n] = __float2bfloat16_rn(v);
                                }
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
            }
            if (!rows_done) {
                // ---- shared tile: store the raw partial in this CTA's slot, the last contributor folds
                // aligned split: the contributors are the CTAs of this cluster and the partial goes to this CTA's own shared
                // memory (the stage ring is free: every MMA of the CTA has completed); otherwise to its workspace slot
                const bool cl = CL && P.cluster_s > 1 && !local;
                float* part_smem = (!ROWS && local) ? stage_small : reinterpret_cast<float*>(tiles);
                if (!ROWS && local) asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous tile's fold has read the staging tile
                const bool to_smem = cl || local || solo;
                if (BN >= 32 && to_smem) {
                    // 32 columns per round trip to tensor memory
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        if (c0 >= P.T) break;
                        uint32_t r[32];
                        tmem_ld32(acc_addr + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c0 + j < P.T) part_smem[(c0 + j) * 128 + row] = __uint_as_float(r[j]);
                    }
                } else {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        if (c0 >= P.T) break;
                        uint32_t r[16];
                        tmem_ld16(acc_addr + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (c0 + j < P.T) {
                                if (to_smem) part_smem[(c0 + j) * 128 + row] = __uint_as_float(r[j]);
                                else __stcg(wbase + (size_t)(c0 + j) * 128 + row, __uint_as_float(r[j]));
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the MMA warp may reuse the buffer while the fold runs
                int t_lo = 0, t_hi = P.T;
                bool do_fold;
                if (local) {
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // the tile is in shared memory
                    do_fold = true;
                } else if (solo) {
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // own partial in shared memory, the others' in the workspace
                    if (etid == 0) P.counters[tile] = 0;            // ready for the next launch
                    do_fold = true;
                } else if (cl) {
                    // first cluster barrier: every CTA's partial is in place.  CTA `slot` then folds its share of the tokens
                    // reading all partials in slot order; the second barrier keeps the shared memory alive until all have read.
                    cluster_sync_all();
                    ++cl_syncs;
                    t_lo = slot * P.T / n_contrib;
                    t_hi = (slot + 1) * P.T / n_contrib;
                    do_fold = true;
                } else {
                    // release / acquire through the tile counter: the barrier orders every thread's partial stores before the
                    // release of thread 0, and its acquire before every thread's loads of the other CTAs' slots
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (etid == 0) {
                        int old;
                        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(P.counters + tile) : "memory");
                        const int last = (old == n_contrib - 1);
                        if (last) P.counters[tile] = 0;  // ready for the next launch
                        is_last_smem[seg & 1] = last;
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    do_fold = is_last_smem[seg & 1] != 0;
                }
                if (do_fold) {
                    // A thread owns 4 consecutive output features of every TS-th token; the partials of NT tokens (four; two in the
                    // few-token image, which keeps its code short) are in flight at once and the slots are added in slot order.  Plain tiles: a warp shares its tokens (32 groups
                    // of 4 features), so the per-token sum of squares is one warp reduction.
                    const int n = n_f;
                    const bool valid = valid_f;
                    const uint32_t part_addr = smem_u32(part_smem);
                    constexpr int NT = BN >= 32 ? 4 : 2;
                    for (int tb = t_lo + tsub; tb < t_hi; tb += NT * TS) {  // warp-uniform trip count for plain tiles
                        float4 g[NT], up[NT];
                        uint2 rr[NT];
#pragma unroll
                        for (int i = 0; i < NT; ++i) {
                            g[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                            up[i] = g[i];
                            rr[i] = make_uint2(0u, 0u);
                            const int t = tb + TS * i;
                            if ((!paired && epi == LIN_RESIDUAL) && valid && t < t_hi) rr[i] = *reinterpret_cast<const uint2*>(P.R + (size_t)t * P.N + n);
                        }
                        if (valid && local) {
#pragma unroll
                            for (int i = 0; i < NT; ++i) {
                                const int t = tb + TS * i;
                                if (t < t_hi) {
                                    g[i] = *reinterpret_cast<const float4*>(part_smem + t * 128 + f4);
                                    if (paired) up[i] = *reinterpret_cast<const float4*>(part_smem + t * 128 + f4 + 64);
                                }
                            }
                        }
                        if (valid && cl) {
                            // shared-memory partials of the cluster: short latency, NT tokens in flight, adds in slot order
#pragma unroll 4
                            for (int z = 0; z < n_contrib; ++z) {
                                const uint32_t zbase = dsmem_addr(part_addr, (uint32_t)z);
#pragma unroll
                                for (int i = 0; i < NT; ++i) {
                                    const int t = tb + TS * i;
                                    if (t < t_hi) {
                                        const uint32_t ra = zbase + (uint32_t)(t * 128 + f4) * 4u;
                                        const float4 av = ld_dsmem_f4(ra);
                                        g[i].x += av.x; g[i].y += av.y; g[i].z += av.z; g[i].w += av.w;
                                        if (paired) {
                                            const float4 cv = ld_dsmem_f4(ra + 256u);
                                            up[i].x += cv.x; up[i].y += cv.y; up[i].z += cv.z; up[i].w += cv.w;
                                        }
                                    }
                                }
                            }
                        }
                        if (valid && !cl && !local) {
                            // workspace partials (L2 round trips): slots in batches of four for all NT tokens; all loads of a batch
                            // are issued before the first add, so a batch costs one round trip; the adds run in slot order
                            constexpr int TOKB = NT, ip = 0;
                            {
#pragma unroll 1
                                for (int zb = 0; zb < n_contrib; zb += 4) {
                                    float4 a[4][TOKB], c[4][TOKB];
#pragma unroll
                                    for (int zz = 0; zz < 4; ++zz) {
#pragma unroll
                                        for (int ii = 0; ii < TOKB; ++ii) {
                                            const int t = tb + TS * (ip + ii);
                                            const int z = zb + zz;
                                            a[zz][ii] = make_float4(0.f, 0.f, 0.f, 0.f);
                                            c[zz][ii] = a[zz][ii];
                                            if (t < t_hi && z < n_contrib) {
                                                if (solo && z == slot) {
                                                    a[zz][ii] = *reinterpret_cast<const float4*>(part_smem + t * 128 + f4);
                                                    if (paired) c[zz][ii] = *reinterpret_cast<const float4*>(part_smem + t * 128 + f4 + 64);
                                                } else {
                                                    const float* w = tbase + z * slot_stride + (size_t)t * 128 + f4;
                                                    a[zz][ii] = __ldcg(reinterpret_cast<const float4*>(w));
                                                    if (paired) c[zz][ii] = __ldcg(reinterpret_cast<const float4*>(w + 64));
                                                }
                                            }
                                        }
                                    }
#pragma unroll
                                    for (int zz = 0; zz < 4; ++zz) {
#pragma unroll
                                        for (int ii = 0; ii < TOKB; ++ii) {
                                            const int i = ip + ii;
                                            g[i].x += a[zz][ii].x; g[i].y += a[zz][ii].y; g[i].z += a[zz][ii].z; g[i].w += a[zz][ii].w;
                                            up[i].x += c[zz][ii].x; up[i].y += c[zz][ii].y; up[i].z += c[zz][ii].z; up[i].w += c[zz][ii].w;
                                        }
                                    }
                                }
                            }
                        }
                        float sc4[NT];
#pragma unroll
                        for (int i = 0; i < NT; ++i) sc4[i] = (scaled && tb + TS * i < t_hi) ? row_scale[tb + TS * i] : 1.0f;
                        // one copy of the epilogue's code for the NT tokens: the loop stays rolled and the tokens' registers
                        // move up by one after each (a dozen moves; the code is fetched once per launch, cold)
#pragma unroll 1
                        for (int i = 0; i < NT; ++i) {
                            const int t = tb + TS * i;
                            if (t >= t_hi) break;
                            const float sc = sc4[0];
                            float v[4] = {g[0].x * sc + bias4.x, g[0].y * sc + bias4.y, g[0].z * sc + bias4.z, g[0].w * sc + bias4.w};
                            float uu[4] = {up[0].x * sc, up[0].y * sc, up[0].z * sc, up[0].w * sc};
                            if ((!paired && epi == LIN_RESIDUAL)) {
                                v[0] += bf16lo(rr[0].x); v[1] += bf16hi(rr[0].x); v[2] += bf16lo(rr[0].y); v[3] += bf16hi(rr[0].y);
                            }
#pragma unroll
                            for (int q = 0; q < NT - 1; ++q) { g[q] = g[q + 1]; up[q] = up[q + 1]; rr[q] = rr[q + 1]; sc4[q] = sc4[q + 1]; }
                            if (paired) {
#pragma unroll 1
                                for (int j = 0; j < 4; ++j) {  // one copy of the division: the values take turns in v[0]
                                    const float y = pk_silu(v[0]) * uu[0];
                                    v[0] = v[1]; v[1] = v[2]; v[2] = v[3]; v[3] = y;
                                    uu[0] = uu[1]; uu[1] = uu[2]; uu[2] = uu[3];
                                }
                            } else if (epi == LIN_RELU) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) v[j] = fmaxf(v[j], 0.0f);
                            } else if (epi == LIN_GELU) {
#pragma unroll 1
                                for (int j = 0; j < 4; ++j) {  // one call site: the values take turns in v[0]
                                    const float y = pk_gelu(v[0]);
                                    v[0] = v[1]; v[1] = v[2]; v[2] = v[3]; v[3] = y;
                                }
                            }
                            float sq = 0.0f;
                            if (f32o) {
                                if (valid) *reinterpret_cast<float4*>(reinterpret_cast<float*>(P.Y) + (size_t)t * P.N + n) = make_float4(v[0], v[1], v[2], v[3]);
                                sq = (v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3]);
                            } else {
                                uint2 o;
                                o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
                                if (tp_push) {
                                    // this rank's block of every rank's exchange buffer (peers over NVLink): plain stores, or two
                                    // words {two bf16, epoch} per thread and token - the epoch in a word tells the reader that
                                    // the word is there
                                    if (valid && tp_inband) {
                                        const size_t off = ((size_t)t * P.N + n) * 4;
#pragma unroll
                                        for (int r = 0; r < 8; ++r)
                                            if (r < P.tp_n) pk_st_volatile_v4(P.tp_dst[r] + off, o.x, (uint32_t)tp_epoch, o.y, (uint32_t)tp_epoch);
                                    } else if (valid) {
                                        const size_t off = ((size_t)t * P.N + n) * 2;
#pragma unroll
                                        for (int r = 0; r < 8; ++r)
                                            if (r < P.tp_n) *reinterpret_cast<uint2*>(P.tp_dst[r] + off) = o;
                                    }
                                } else if (valid) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(P.Y) + (size_t)t * P.N + n) = o;
                                const float s0 = bf16lo(o.x), s1 = bf16hi(o.x), s2 = bf16lo(o.y), s3 = bf16hi(o.y);
                                sq = (s0 * s0 + s1 * s1) + (s2 * s2 + s3 * s3);
                            }
                            if (want_ssq) {  // plain tiles: all 32 lanes of the warp hold token t
                                sq = warp_sum(valid ? sq : 0.0f);
                                if (lane == 0) P.ssq_out[(size_t)tile * P.ssq_stride + t] = sq;
                            }
                        }
                    }
                }
                if (do_fold && tp_push && !tp_inband) {
                    // The barrier orders every thread's slot stores before thread 0, which releases them (device scope) through
                    // the launch's counter.  The CTA that completes the launch has thereby acquired every other CTA's stores;
                    // ONE system-scope fence then orders all of them before the epoch it stores (relaxed) into every rank's
                    // flag word for this rank - its own included: the consumer on this GPU waits for flags, not for the end of
                    // this kernel.  (A system-scope fence costs microseconds: one per launch, not one per CTA or per flag.)
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (etid == 0) {
                        int old;
                        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(P.tp_state) : "memory");
                        if (old == P.tp_expect - 1) {
                            P.tp_state[0] = 0;  // ready for the next launch
                            const int E = *reinterpret_cast<const volatile int*>(P.tp_pass) * P.tp_n_sites + P.tp_site + 1;
                            asm volatile("fence.acq_rel.sys;" ::: "memory");
#pragma unroll
                            for (int r = 0; r < 8; ++r)
                                if (r < P.tp_n) asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(P.tp_flag[r]), "r"(E) : "memory");
                        }
                    }
                }
                if (cl) { cluster_sync_all(); ++cl_syncs; }
            }
            if (etid == 0) PK_TRACE(5 + (seg > 1 ? 1 : seg));  // end of the first / of the last segment's epilogue
            u += len;
            ++seg;
        }
        if (CL && P.cluster_s > 1)
            for (; cl_syncs < 2; ++cl_syncs) cluster_sync_all();  // a CTA that gave up on a wait must not leave its peers waiting
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0) PK_TRACE(7);  // CTA done
}

// ---- packing ---------------------------------------------------------------------------------------------
// One thread per 16-byte chunk of the packed image.  Chunk q of a unit sits at row r = q / 8, position cs = q % 8 of
// the 128-byte row and holds the logical chunk cs ^ (r % 8): the 128-byte swizzle of the shared-memory tile.
__global__ void __launch_bounds__(256) pack_weights_kernel(const __nv_bfloat16* __restrict__ src, uint8_t* __restrict__ dst, int N, int K,
                                                           int n_tiles, int kbt, int paired, int unpack) {
    const long long total = (long long)n_tiles * kbt * 1024;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(idx % 1024);
        const long long unit = idx / 1024;
        const int kb = (int)(unit % kbt), j = (int)(unit / kbt);
        const int r = q >> 3, cs = q & 7, c = cs ^ (r & 7);
        const long long row = pk_source_row(paired, N, j, r);
        const int k = kb * 64 + c * 8;
        uint4* packed = reinterpret_cast<uint4*>(dst) + idx;
        if (unpack) {  // dst is the packed image here, src the row-major matrix to rebuild
            if (row >= 0 && k < K) *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(src) + row * K + k) = *packed;
        } else {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row >= 0 && k < K) v = *reinterpret_cast<const uint4*>(src + row * K + k);
            *packed = v;
        }
    }
}

void pk_dims(int N, int K, int paired, int* n_tiles, int* kbt) {
    *n_tiles = paired ? (N + 63) / 64 : (N + 127) / 128;
    *kbt = (K + 63) / 64;
}

size_t linear_packed_bytes(int N, int K, int paired) {
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    return (size_t)nt * kbt * PK_TILE_BYTES;
}

jsm_status linear_pack_launch(const void* W, int N, int K, int paired, void* packed, bool unpack, cudaStream_t st) {
    if (!W || !packed) JSM_FAIL(JSM_INVALID_ARG, "linear_pack: null pointer");
    if (N <= 0 || K <= 0 || K % 8) JSM_FAIL(JSM_UNSUPPORTED, "linear_pack: N %d, K %d (K must be a positive multiple of 8)", N, K);
    if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(packed) & 15))
        JSM_FAIL(JSM_INVALID_ARG, "linear_pack: pointers must be 16-byte aligned");
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    const long long total = (long long)nt * kbt * 1024;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 32) blocks = (long long)sm_count() * 32;
    pack_weights_kernel<<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)W, (uint8_t*)packed, N, K, nt, kbt, paired, unpack ? 1 : 0);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

// Work split of a launch with T tokens.  Few tokens (T < 32): the fold of a shared tile is a short chain of round trips,
// so SM coverage decides: the even split of the whole stream, or, with few tiles, every tile over the same number of
// CTAs when that still occupies four fifths of the SMs.  Many tokens: the fold's volume grows with T, so whole tiles
// (no fold at all) or an aligned split whose CTAs fold through distributed shared memory win as soon as they occupy
// three fifths of the SMs.
int linear_packed_grid(int N, int K, int paired, int T) {
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    const long long U = (long long)nt * kbt;
    long long G = sm_count();
    if (nt < G) {
        long long S = G / nt;  // CTAs per tile of the aligned split
        bool use;
        if (T >= 32) {
            // a power of two up to 8 (the cluster that folds through shared memory), from half of the SMs on
            S = S >= 8 ? 8 : S >= 4 ? 4 : S >= 2 ? 2 : 1;
            use = nt * S * 2 >= G;
        } else {
            // at most 8 contributors per tile (the fold reads every slot); from four fifths of the SMs on, or whenever the
            // even split of the stream would put more than 8 CTAs on a tile
            const bool capped = S > 8;
            if (capped) S = 8;
            use = capped || nt * S * 5 >= G * 4;
        }
        if (S > kbt) S = kbt;
        if (use && S >= 1) G = nt * S;
    }
    if (U < 4 * G && T < 32) G = U / 4;  // at least four units per CTA
    if (G > U) G = U;
    if (G < 1) G = 1;
    return (int)G;
}

// > 1 when the grid is the aligned split (every tile shared by the same power-of-two number of consecutive CTAs) and
// the launch has enough tokens for the exchange to matter: those CTAs are launched as one thread-block cluster and fold
// their partials through distributed shared memory
int linear_packed_cluster(int N, int K, int paired, int T) {
    if (T < 32) return 0;
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    const int G = linear_packed_grid(N, K, paired, T);
    if (G % nt) return 0;
    const int S = G / nt;
    if (S != 2 && S != 4 && S != 8) return 0;
    if ((long long)nt * kbt / G < 1) return 0;
    return S;
}

// The outputs of a launch can be pushed to the ranks' exchange buffers when every finished tile leaves through the
// vectorised (folding) epilogue: the aligned split, where a CTA holds exactly one segment of exactly one tile.
bool linear_packed_can_push(int N, int K, int T) {
    int nt, kbt;
    pk_dims(N, K, 0, &nt, &kbt);
    const int G = linear_packed_grid(N, K, 0, T);
    return T <= TP_PUSH_MAX_T && G % nt == 0 && N % 4 == 0;
}

static int slots_for_grid(int nt, int kbt, long long G) {
    const long long U = (long long)nt * kbt;
    // a tile of kbt units is covered by at most ceil(kbt / floor(U/G)) + 1 consecutive CTA ranges
    const long long per = U / G > 0 ? U / G : 1;
    return (int)((kbt + per - 1) / per + 1);
}

int linear_packed_slots(int N, int K, int paired, int T) {
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    return slots_for_grid(nt, kbt, linear_packed_grid(N, K, paired, T));
}

// enough for every launch of at most T tokens (the split depends on the token count)
size_t linear_packed_ws_floats(int T, int N, int K, int paired) {
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    const int slots = std::max(linear_packed_slots(N, K, paired, 1), linear_packed_slots(N, K, paired, 64));
    return (size_t)nt * slots * (size_t)T * 128;
}

// ---- optional timeline of the packed projections (a profiling aid; off unless jsm_trace_begin was called) ----------
static unsigned long long* g_trace_buf = nullptr;  // [launch][CTA][8]
static int g_trace_cap = 0, g_trace_n = 0, g_trace_ctas = 0;

template <int BN, bool CL, int TPM, int PRM = -1>
static jsm_status launch_packed(const CUtensorMap& mx, const CUtensorMap& mx2, PkParams& P, int grid, int cluster, bool chained, cudaStream_t st) {
    constexpr int STAGE_BYTES = 2 * (PK_TILE_BYTES + BN * 128);
    // up to 64 tokens two CTAs share an SM (the successor kernel of a chain prefetches next to the running one)
    const int budget = (BN <= 64 ? 150 : 200) * 1024;
    int stages = budget / STAGE_BYTES;
    if (stages > PK_MAX_STAGES) stages = PK_MAX_STAGES;
    if (stages < 2) stages = 2;
    P.stages = stages;
    P.trace = nullptr;
    if (g_trace_buf && g_trace_n < g_trace_cap && grid <= g_trace_ctas) {
        P.trace = g_trace_buf + (size_t)g_trace_n * g_trace_ctas * 8;
        ++g_trace_n;
    }
    const size_t smem = (size_t)stages * STAGE_BYTES + 1024;
    static bool attr_done = false;  // per instantiation
    if (!attr_done) {
        cudaFuncAttributes fa;
        JSM_CUDA_CHECK(cudaFuncGetAttributes(&fa, linear_packed_kernel<BN, CL, TPM, PRM>));
        // 227 KB per CTA in all: what the kernel's static arrays leave is open to the stage ring
        JSM_CUDA_CHECK(cudaFuncSetAttribute(linear_packed_kernel<BN, CL, TPM, PRM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            227 * 1024 - (int)fa.sharedSizeBytes));
        attr_done = true;
    }
    P.pf_units = 0;
    P.cluster_s = cluster > 1 ? cluster : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(PK_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (chained && chained_launch_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (cluster > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = (unsigned)cluster;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    JSM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, linear_packed_kernel<BN, CL, TPM, PRM>, mx, mx2, P));
    g_launches.fetch_add(1);
    return JSM_OK;
}

jsm_status linear_packed_launch(const PackedArgs& a, cudaStream_t st) {
    if (a.T <= 0 || a.N <= 0) return JSM_OK;
    const bool tp_push = a.tp && a.tp->push, tp_reduce = a.tp && a.tp->reduce;
    if (!a.X || !a.Wp || (!a.Y && !tp_push)) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: null pointer");
    if (a.K <= 0 || a.K % 8) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: K (%d) must be a positive multiple of 8", a.K);
    if (a.N % 4) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: N (%d) must be a multiple of 4", a.N);
    if (a.T > 256) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: at most 256 tokens per launch (%d)", a.T);
    if (a.epilogue < LIN_NONE || a.epilogue > LIN_RESIDUAL) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: epilogue %d", a.epilogue);
    const int paired = a.epilogue == LIN_SILU_MUL ? 1 : 0;
    if (paired && a.bias) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: the gate/up projection takes no bias");
    if (a.epilogue == LIN_RESIDUAL && !a.R) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: residual epilogue without R");
    if (a.bias && (reinterpret_cast<uintptr_t>(a.bias) & 15)) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: bias must be 16-byte aligned");
    PkParams P;
    P.T = a.T; P.N = a.N; P.K = a.K;
    pk_dims(a.N, a.K, paired, &P.n_tiles, &P.kbt);
    P.local_epi = 1;
    P.paired = paired; P.epilogue = a.epilogue; P.out_f32 = a.out_f32 ? 1 : 0;
    P.bias = a.bias; P.R = (const __nv_bfloat16*)a.R; P.Y = a.Y; P.Wp = (const uint8_t*)a.Wp;
    const int grid = linear_packed_grid(a.N, a.K, paired, a.T);
    P.max_slots = linear_packed_slots(a.N, a.K, paired, a.T);
    const long long U = (long long)P.n_tiles * P.kbt;
    if ((U + 1) * ((long long)grid + 1) >= (1ll << 31))  // the kernel partitions the units in 32-bit arithmetic
        JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: %lld units of work on %d CTAs exceed one launch (a packed matrix of tens of gigabytes)", U, grid);
    const bool shared_tiles = (U % grid) != 0 || ((U / grid) % P.kbt) != 0;
    if (shared_tiles) {
        if (!a.ws || !a.counters)
            JSM_FAIL(JSM_INVALID_ARG, "linear_packed: no workspace on this device (jsm_linear_pack / jsm_linear_packed_reserve size it at set-up time)");
        if ((size_t)P.n_tiles * P.max_slots * (size_t)a.T * 128 > a.ws_floats)
            JSM_FAIL(JSM_INVALID_ARG, "linear_packed: workspace of %zu floats, %zu needed", a.ws_floats,
                     linear_packed_ws_floats(a.T, a.N, a.K, paired));
        if (P.n_tiles > a.n_counters) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: %d tile counters, %d needed", a.n_counters, P.n_tiles);
    }
    P.ws = a.ws; P.counters = a.counters;
    P.err = tc_error_word();
    if (a.ssq_out && (paired || a.out_f32)) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: row statistics are written for plain bf16 outputs only");
    if (a.ssq_in && (a.ssq_in_tiles <= 0 || a.K <= 0)) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: row statistics without their tile count");
    P.ssq_in = a.ssq_in; P.ssq_in_tiles = a.ssq_in_tiles; P.ssq_stride = a.ssq_stride > 0 ? a.ssq_stride : a.T;
    P.inv_d = 1.0f / (float)a.K; P.eps = a.eps; P.ssq_out = a.ssq_out;
    const int bn = a.T <= 16 ? 16 : a.T <= 32 ? 32 : a.T <= 64 ? 64 : a.T <= 128 ? 128 : 256;
    CUtensorMap mx;
    jsm_status s = make_tmap_bf16_2d(&mx, a.X, (uint64_t)a.T, (uint64_t)a.K, (uint64_t)(a.x_row_stride > 0 ? a.x_row_stride : a.K), bn, 64);
    if (s != JSM_OK) return s;
    // the same matrix as [k-block][row][64]: a box two k-blocks deep lands as two consecutive swizzled X blocks
    const long long xs = a.x_row_stride > 0 ? a.x_row_stride : a.K;
    P.pair_ok = (a.K % 64 == 0) ? 1 : 0;
    CUtensorMap mx2 = mx;
    if (P.pair_ok) {
        s = make_tmap_bf16_3d(&mx2, a.X, 64, (uint64_t)a.T, (uint64_t)(a.K / 64), (uint64_t)xs, 64, 64, bn, 2);
        if (s != JSM_OK) return s;
        if (a.K / 64 < 2) P.pair_ok = 0;
    }
    const int cluster = linear_packed_cluster(a.N, a.K, paired, a.T);
    P.tp_mode = 0;
    P.tp_inband = 0;
    if (tp_push || tp_reduce) {
        const TpFuse& f = *a.tp;
        if (tp_push && tp_reduce) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: a launch either pushes or reduces");
        if (f.n_ranks < 2 || f.n_ranks > 8 || f.rank < 0 || f.rank >= f.n_ranks || !f.pass || !f.state || f.wait_limit <= 0)
            JSM_FAIL(JSM_INVALID_ARG, "linear_packed: tensor-parallel exchange of rank %d of %d", f.rank, f.n_ranks);
        if (a.T > TP_PUSH_MAX_T) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: the fused exchange takes at most %d tokens (%d)", TP_PUSH_MAX_T, a.T);
        P.tp_n = f.n_ranks; P.tp_rank = f.rank; P.tp_site = f.site; P.tp_n_sites = f.n_sites; P.tp_pass = f.pass; P.tp_state = f.state;
        P.tp_wait = f.wait_limit;
        if (f.inband && a.T > TP_INBAND_MAX_T)
            JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: in-band exchange words for at most %d tokens (%d)", TP_INBAND_MAX_T, a.T);
        P.tp_inband = f.inband ? 1 : 0;
        for (int r = 0; r < 8; ++r) { P.tp_dst[r] = nullptr; P.tp_flag[r] = nullptr; }
        P.tp_slots = nullptr; P.tp_slot_stride = 0; P.tp_flags = nullptr; P.tp_h = nullptr; P.tp_ssq = nullptr; P.tp_expect = 0;
        if (tp_push) {
            if (!linear_packed_can_push(a.N, a.K, a.T) || paired || a.out_f32 || a.bias || a.epilogue != LIN_NONE || a.ssq_out)
                JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: this launch cannot push its outputs (plain bf16 projection on an aligned split only)");
            for (int r = 0; r < f.n_ranks; ++r) {
                if (!f.push_dst[r] || !f.push_flag[r]) JSM_FAIL(JSM_INVALID_ARG, "linear_packed: no exchange buffer for rank %d", r);
                P.tp_dst[r] = reinterpret_cast<uint8_t*>(f.push_dst[r]);
                P.tp_flag[r] = f.push_flag[r];
            }
            P.tp_expect = cluster > 1 ? grid : P.n_tiles;
            P.tp_mode = 1;
        } else {
            if (!f.slots || !f.flags || !f.h || !f.ssq || a.ssq_in != f.ssq || a.ssq_in_tiles != (a.K + 127) / 128 ||
                (a.x_row_stride > 0 && a.x_row_stride != a.K) || a.X != f.h)
                JSM_FAIL(JSM_INVALID_ARG, "linear_packed: the reducing launch reads X = h with the statistics the reduction writes");
            P.tp_slots = reinterpret_cast<const uint8_t*>(f.slots); P.tp_slot_stride = f.slot_stride; P.tp_flags = f.flags;
            P.tp_h = reinterpret_cast<__nv_bfloat16*>(f.h); P.tp_ssq = f.ssq;
            P.tp_mode = 2;
        }
    }
    // A launch pays for the size of the image it runs.  The common launches of a decoder step (up to 64 tokens) have
    // lean images of their own, chosen below; what remains runs the general images: with the cluster path from 32 tokens
    // on (cluster size 1 where no cluster forms), with the exchange code when the launch pushes or reduces.
    const bool with_cl = cluster > 1 || a.T >= 32;
    const bool with_tp = P.tp_mode != 0;  // (at most 64 tokens: checked above)
#define PK_GO(BN_)                                                                                  \
    return with_cl ? launch_packed<BN_, true, 0>(mx, mx2, P, grid, cluster, a.chained, st)     \
                   : launch_packed<BN_, false, 0>(mx, mx2, P, grid, cluster, a.chained, st)
#define PK_GO_TP(BN_)                                                                                        \
    if (with_tp)                                                                                             \
        return with_cl ? launch_packed<BN_, true, 3>(mx, mx2, P, grid, cluster, a.chained, st)           \
                       : launch_packed<BN_, false, 3>(mx, mx2, P, grid, cluster, a.chained, st);        \
    PK_GO(BN_)
    // the few-token launches without an exchange (the decode step of one GPU): an image per kind of tile
    if (bn == 16 && !with_cl && !with_tp) {
        const bool lean = !a.bias && !a.out_f32;  // the projections of a LLaMA-style decoder step have images of their own
        if (lean && paired && a.ssq_in) return launch_packed<16, false, 0, 4>(mx, mx2, P, grid, cluster, a.chained, st);
        if (lean && !paired && a.epilogue == LIN_NONE && a.ssq_in && !a.ssq_out)
            return launch_packed<16, false, 0, 2>(mx, mx2, P, grid, cluster, a.chained, st);
        if (lean && !paired && a.epilogue == LIN_RESIDUAL && !a.ssq_in && a.ssq_out)
            return launch_packed<16, false, 0, 3>(mx, mx2, P, grid, cluster, a.chained, st);
        return paired ? launch_packed<16, false, 0, 1>(mx, mx2, P, grid, cluster, a.chained, st)
                      : launch_packed<16, false, 0, 0>(mx, mx2, P, grid, cluster, a.chained, st);
    }
    // 17 to 64 tokens without an exchange: the same three images per token block, with and without the cluster path
    if ((bn == 32 || bn == 64) && !with_tp && !a.bias && !a.out_f32) {
#define PK_LEAN(BN_, CL_)                                                                                                    \
    do {                                                                                                                     \
        if (paired && a.ssq_in) return launch_packed<BN_, CL_, 0, 4>(mx, mx2, P, grid, cluster, a.chained, st);              \
        if (!paired && a.epilogue == LIN_NONE && a.ssq_in && !a.ssq_out)                                                     \
            return launch_packed<BN_, CL_, 0, 2>(mx, mx2, P, grid, cluster, a.chained, st);                                  \
        if (!paired && a.epilogue == LIN_RESIDUAL && !a.ssq_in && a.ssq_out)                                                 \
            return launch_packed<BN_, CL_, 0, 3>(mx, mx2, P, grid, cluster, a.chained, st);                                  \
    } while (0)
        if (bn == 32) {
            if (cluster > 1) PK_LEAN(32, true); else PK_LEAN(32, false);
        } else {
            if (cluster > 1) PK_LEAN(64, true); else PK_LEAN(64, false);
        }
#undef PK_LEAN
    }
    // 17 to 64 tokens of a tensor-parallel rank (flags): the pushing projection and the two reducing ones
    if ((bn == 32 || bn == 64) && with_tp && !P.tp_inband && !a.bias && !a.out_f32) {
#define PK_LEAN_TP(BN_, CL_)                                                                                                 \
    do {                                                                                                                     \
        if (P.tp_mode == 1 && !a.ssq_in) return launch_packed<BN_, CL_, 1, 5>(mx, mx2, P, grid, cluster, a.chained, st);     \
        if (P.tp_mode == 2 && paired) return launch_packed<BN_, CL_, 2, 4>(mx, mx2, P, grid, cluster, a.chained, st);        \
        if (P.tp_mode == 2 && a.epilogue == LIN_NONE && !a.ssq_out)                                                          \
            return launch_packed<BN_, CL_, 2, 2>(mx, mx2, P, grid, cluster, a.chained, st);                                  \
    } while (0)
        if (bn == 32) {
            if (cluster > 1) PK_LEAN_TP(32, true); else PK_LEAN_TP(32, false);
        } else {
            if (cluster > 1) PK_LEAN_TP(64, true); else PK_LEAN_TP(64, false);
        }
#undef PK_LEAN_TP
    }
    if (bn == 16 && !with_cl && with_tp && P.tp_inband && !a.bias && !a.out_f32) {  // the decode step of a tensor-parallel rank
        if (P.tp_mode == 1 && !a.ssq_in) return launch_packed<16, false, 4, 5>(mx, mx2, P, grid, cluster, a.chained, st);  // (plain, nothing else: checked above)
        if (P.tp_mode == 2 && paired) return launch_packed<16, false, 5, 4>(mx, mx2, P, grid, cluster, a.chained, st);
        if (P.tp_mode == 2 && a.epilogue == LIN_NONE && !a.ssq_out) return launch_packed<16, false, 5, 2>(mx, mx2, P, grid, cluster, a.chained, st);
    }
    switch (bn) {
        case 16: PK_GO_TP(16);
        case 32: PK_GO_TP(32);
        case 64: PK_GO_TP(64);
        case 128: PK_GO(128);
        default: PK_GO(256);
    }
#undef PK_GO_TP
#undef PK_GO
}

// ---- per-device workspace of the public entry point -------------------------------------------------------------
struct PkWorkspace {
    float* ws = nullptr;
    size_t ws_floats = 0;
    int* counters = nullptr;
    int n_counters = 0;
};
static PkWorkspace g_pk_ws[64];
static std::mutex g_pk_mu;

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_trace_begin(int max_launches) {
    if (max_launches <= 0 || max_launches > 100000) JSM_FAIL(JSM_INVALID_ARG, "jsm_trace_begin: %d launches", max_launches);
    if (g_trace_buf) cudaFree(g_trace_buf);
    g_trace_buf = nullptr;
    g_trace_ctas = sm_count();
    const size_t bytes = (size_t)max_launches * g_trace_ctas * 8 * sizeof(unsigned long long);
    JSM_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&g_trace_buf), bytes));
    JSM_CUDA_CHECK(cudaMemset(g_trace_buf, 0, bytes));
    g_trace_cap = max_launches;
    g_trace_n = 0;
    return JSM_OK;
}

extern "C" jsm_status jsm_trace_end(uint64_t* h_stamps, int max_launches, int* n_launches, int* ctas_per_launch) {
    if (!n_launches || !ctas_per_launch) JSM_FAIL(JSM_INVALID_ARG, "jsm_trace_end: null argument");
    JSM_CUDA_CHECK(cudaDeviceSynchronize());
    const int n = g_trace_n < max_launches ? g_trace_n : max_launches;
    *n_launches = n;
    *ctas_per_launch = g_trace_ctas;
    if (g_trace_buf && h_stamps && n > 0)
        JSM_CUDA_CHECK(cudaMemcpy(h_stamps, g_trace_buf, (size_t)n * g_trace_ctas * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    if (g_trace_buf) cudaFree(g_trace_buf);
    g_trace_buf = nullptr;
    g_trace_cap = g_trace_n = 0;
    return JSM_OK;
}

extern "C" jsm_status jsm_linear_packed_plan(int N, int K, int paired, int* n_tiles, int* kbt, int* grid, int* max_slots) {
    if (N <= 0 || K <= 0 || !n_tiles || !kbt || !grid || !max_slots) JSM_FAIL(JSM_INVALID_ARG, "jsm_linear_packed_plan: bad argument");
    pk_dims(N, K, paired ? 1 : 0, n_tiles, kbt);
    *grid = linear_packed_grid(N, K, paired ? 1 : 0, 1);
    *max_slots = linear_packed_slots(N, K, paired ? 1 : 0, 1);
    return JSM_OK;
}

extern "C" size_t jsm_linear_packed_bytes(int N, int K, int paired) {
    if (N <= 0 || K <= 0) return 0;
    return linear_packed_bytes(N, K, paired ? 1 : 0);
}

// Grows the workspace of the current device so that any launch of this shape (up to 256 tokens per launch) finds room.
// Set-up time only: synchronises the device when it has to reallocate.
extern "C" jsm_status jsm_linear_packed_reserve(int N, int K, int paired) {
    if (N <= 0 || K <= 0) JSM_FAIL(JSM_INVALID_ARG, "jsm_linear_packed_reserve: N %d, K %d", N, K);
    int dev = -1;
    JSM_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) JSM_FAIL(JSM_UNSUPPORTED, "jsm_linear_packed_reserve: device index %d", dev);
    paired = paired ? 1 : 0;
    std::lock_guard<std::mutex> lock(g_pk_mu);
    PkWorkspace& w = g_pk_ws[dev];
    size_t need = 0;
    for (int T : {16, 32, 64, 128, 256}) need = std::max(need, linear_packed_ws_floats(T, N, K, paired));
    int nt, kbt;
    pk_dims(N, K, paired, &nt, &kbt);
    if (need > w.ws_floats) {
        JSM_CUDA_CHECK(cudaDeviceSynchronize());
        if (w.ws) cudaFree(w.ws);
        w.ws = nullptr; w.ws_floats = 0;
        JSM_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&w.ws), need * sizeof(float)));
        w.ws_floats = need;
    }
    if (nt > w.n_counters) {
        JSM_CUDA_CHECK(cudaDeviceSynchronize());
        if (w.counters) cudaFree(w.counters);
        w.counters = nullptr; w.n_counters = 0;
        const int n = nt < 1024 ? 1024 : nt;
        JSM_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&w.counters), n * sizeof(int)));
        JSM_CUDA_CHECK(cudaMemset(w.counters, 0, n * sizeof(int)));
        w.n_counters = n;
    }
    return JSM_OK;
}

extern "C" jsm_status jsm_linear_pack(const void* d_W, int N, int K, int paired, void* d_packed, void* stream) {
    jsm_status s = linear_pack_launch(d_W, N, K, paired ? 1 : 0, d_packed, false, as_stream(stream));
    if (s != JSM_OK) return s;
    return jsm_linear_packed_reserve(N, K, paired);
}

extern "C" jsm_status jsm_linear_unpack(const void* d_packed, int N, int K, int paired, void* d_W, void* stream) {
    return linear_pack_launch(d_W, N, K, paired ? 1 : 0, const_cast<void*>(d_packed), true, as_stream(stream));
}

static jsm_status linear_bf16_packed_entry(const void* d_X, const void* d_packed, const float* d_bias, int epilogue, const void* d_R,
                                           void* d_Y, int out_dtype, int T, int N, int K, void* stream, bool chained) {
    if (out_dtype != JSM_BF16 && out_dtype != JSM_F32) JSM_FAIL(JSM_UNSUPPORTED, "jsm_linear_bf16_packed: out dtype %d", out_dtype);
    if (T <= 0 || N <= 0) return JSM_OK;
    int dev = -1;
    JSM_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) JSM_FAIL(JSM_UNSUPPORTED, "jsm_linear_bf16_packed: device index %d", dev);
    cudaStream_t st = as_stream(stream);
    PackedArgs a;
    a.X = d_X; a.Wp = d_packed; a.bias = d_bias; a.epilogue = epilogue; a.R = d_R; a.out_f32 = out_dtype == JSM_F32;
    a.N = N; a.K = K; a.x_row_stride = 0; a.chained = chained;
    {
        // the workspace of this device, sized at set-up time (jsm_linear_pack / jsm_linear_packed_reserve); the launch
        // checks its capacity and fails rather than allocate
        std::lock_guard<std::mutex> lock(g_pk_mu);
        const PkWorkspace& w = g_pk_ws[dev];
        a.ws = w.ws; a.ws_floats = w.ws_floats; a.counters = w.counters; a.n_counters = w.n_counters;
    }
    // more than 256 tokens: token chunks, each streaming the weights once
    for (int t0 = 0; t0 < T; t0 += 256) {
        const int tc = T - t0 < 256 ? T - t0 : 256;
        a.T = tc;
        a.X = reinterpret_cast<const __nv_bfloat16*>(d_X) + (size_t)t0 * K;
        a.R = d_R ? reinterpret_cast<const __nv_bfloat16*>(d_R) + (size_t)t0 * N : nullptr;
        a.Y = a.out_f32 ? static_cast<void*>(reinterpret_cast<float*>(d_Y) + (size_t)t0 * N)
                        : static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(d_Y) + (size_t)t0 * N);
        jsm_status s = linear_packed_launch(a, st);
        if (s != JSM_OK) return s;
    }
    return JSM_OK;
}

extern "C" jsm_status jsm_linear_bf16_packed(const void* d_X, const void* d_packed, const float* d_bias, int epilogue, const void* d_R,
                                             void* d_Y, int out_dtype, int T, int N, int K, void* stream) {
    return linear_bf16_packed_entry(d_X, d_packed, d_bias, epilogue, d_R, d_Y, out_dtype, T, N, K, stream, false);
}

extern "C" jsm_status jsm_linear_bf16_packed_chained(const void* d_X, const void* d_packed, const float* d_bias, int epilogue,
                                                     const void* d_R, void* d_Y, int out_dtype, int T, int N, int K, void* stream) {
    return linear_bf16_packed_entry(d_X, d_packed, d_bias, epilogue, d_R, d_Y, out_dtype, T, N, K, stream, true);
}

// ---- the fused exchange on its own (what the decoder runner composes; also how the protocol is tested on one GPU) ----
static jsm_status device_workspace(PackedArgs& a) {
    int dev = -1;
    JSM_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) JSM_FAIL(JSM_UNSUPPORTED, "linear_packed: device index %d", dev);
    std::lock_guard<std::mutex> lock(g_pk_mu);
    const PkWorkspace& w = g_pk_ws[dev];
    a.ws = w.ws; a.ws_floats = w.ws_floats; a.counters = w.counters; a.n_counters = w.n_counters;
    return JSM_OK;
}

extern "C" jsm_status jsm_tp_linear_push(void* const* d_regions, int rank, int size, int which_buffer, int max_tokens, int32_t* d_state,
                                         int site, int n_sites, const void* d_X, const void* d_packed, int T, int N, int K, void* stream) {
    if (!d_regions || !d_state || !d_X || !d_packed) JSM_FAIL(JSM_INVALID_ARG, "jsm_tp_linear_push: null argument");
    if (size < 2 || size > 8 || rank < 0 || rank >= size) JSM_FAIL(JSM_INVALID_ARG, "jsm_tp_linear_push: rank %d of %d", rank, size);
    if (T <= 0 || T > TP_PUSH_MAX_T || T > max_tokens) JSM_FAIL(JSM_SHAPE, "jsm_tp_linear_push: %d tokens (1..%d)", T, TP_PUSH_MAX_T);
    if (!linear_packed_can_push(N, K, T)) JSM_FAIL(JSM_UNSUPPORTED, "jsm_tp_linear_push: a [%d x %d] projection over %d tokens has no aligned split", N, K, T);
    TpFuse f;
    f.n_ranks = size; f.rank = rank; f.pass = d_state; f.state = d_state + 1; f.site = site; f.n_sites = n_sites;
    f.wait_limit = tp_wait_limit_cycles();
    f.push = true;
    f.inband = T <= TP_INBAND_MAX_T;
    const size_t off = f.inband ? tp_inband_offset(which_buffer, max_tokens, N) + (size_t)rank * tp_inband_slot_bytes(N)
                                : tp_push_offset(which_buffer, max_tokens, N) + (size_t)rank * tp_slot_bytes(N);
    for (int r = 0; r < size; ++r) {
        if (!d_regions[r]) JSM_FAIL(JSM_INVALID_ARG, "jsm_tp_linear_push: no region for rank %d", r);
        f.push_dst[r] = static_cast<uint8_t*>(d_regions[r]) + off;
        f.push_flag[r] = static_cast<int*>(d_regions[r]) + tp_push_flag_word() + rank;
    }
    PackedArgs a;
    a.X = d_X; a.Wp = d_packed; a.bias = nullptr; a.epilogue = LIN_NONE; a.R = nullptr; a.Y = nullptr; a.out_f32 = false;
    a.T = T; a.N = N; a.K = K; a.x_row_stride = 0; a.chained = false; a.tp = &f;
    jsm_status s = device_workspace(a);
    if (s != JSM_OK) return s;
    return linear_packed_launch(a, as_stream(stream));
}

extern "C" jsm_status jsm_tp_linear_reduce(void* d_region, int rank, int size, int which_buffer, int max_tokens, int32_t* d_state, int site,
                                           int n_sites, void* d_h, float* d_ssq, const void* d_packed, int epilogue, void* d_Y,
                                           int out_dtype, int T, int N, int d, float eps, void* stream) {
    if (!d_region || !d_state || !d_h || !d_ssq || !d_packed || !d_Y) JSM_FAIL(JSM_INVALID_ARG, "jsm_tp_linear_reduce: null argument");
    if (size < 2 || size > 8 || rank < 0 || rank >= size) JSM_FAIL(JSM_INVALID_ARG, "jsm_tp_linear_reduce: rank %d of %d", rank, size);
    if (T <= 0 || T > TP_PUSH_MAX_T || T > max_tokens) JSM_FAIL(JSM_SHAPE, "jsm_tp_linear_reduce: %d tokens (1..%d)", T, TP_PUSH_MAX_T);
    if (out_dtype != JSM_BF16 && out_dtype != JSM_F32) JSM_FAIL(JSM_UNSUPPORTED, "jsm_tp_linear_reduce: out dtype %d", out_dtype);
    TpFuse f;
    f.n_ranks = size; f.rank = rank; f.pass = d_state; f.state = d_state + 1; f.site = site; f.n_sites = n_sites;
    f.wait_limit = tp_wait_limit_cycles();
    f.reduce = true;
    f.inband = T <= TP_INBAND_MAX_T;
    f.slots = static_cast<const uint8_t*>(d_region) + (f.inband ? tp_inband_offset(which_buffer, max_tokens, d) : tp_push_offset(which_buffer, max_tokens, d));
    f.slot_stride = f.inband ? tp_inband_slot_bytes(d) : tp_slot_bytes(d);
    f.flags = static_cast<const int*>(d_region) + tp_push_flag_word();
    f.h = d_h; f.ssq = d_ssq;
    PackedArgs a;
    a.X = d_h; a.Wp = d_packed; a.bias = nullptr; a.epilogue = epilogue; a.R = nullptr; a.Y = d_Y; a.out_f32 = out_dtype == JSM_F32;
    a.T = T; a.N = N; a.K = d; a.x_row_stride = 0; a.chained = false;
    a.ssq_in = d_ssq; a.ssq_in_tiles = (d + 127) / 128; a.ssq_stride = T; a.eps = eps; a.tp = &f;
    jsm_status s = device_workspace(a);
    if (s != JSM_OK) return s;
    return linear_packed_launch(a, as_stream(stream));
}
