// Tensor-parallel exchange of the decoder: the all-reduce after the attention output projection and after the FFN
// down projection, fused with what consumes it (residual add + RMSNorm), over peer memory.
//
// The reference has no parallelism at all (one thread, no collectives); its heads are independent
// (mat_mha_t.hpp:278-282) and its FFN columns are, so the split needs exactly one sum per block.
//
// One process per GPU.  Every rank owns a REGION in its own HBM: [flags | buffer A | buffer B].  The projection
// writes the rank-local product [T, d] (bf16) into one of its buffers; then ONE kernel per rank
//   1. tells every peer "my buffer is complete" by storing the call's epoch into the peer's flag word for this rank
//      (release, system scope) and waits (acquire, bounded) until all peers have said the same,
//   2. reads every rank's buffer - its own from HBM, the peers' over NVLink with plain peer loads - and adds them in
//      rank order in fp32, so that all ranks compute bit-identical sums,
//   3. adds the sum into the residual stream h (bf16) and writes xn = RMSNorm(h) for the next projection.
// The epoch of a call is (number of the forward pass) * (exchanges per pass) + (index of the exchange) + 1: every rank
// runs the same sequence, the pass number lives in device memory (graph replays see it change) and is bumped by the
// first kernel of the pass, so the exchange kernel neither counts nor publishes anything itself.
// There is no second barrier: the two call sites of a layer alternate between buffer A and buffer B, and a rank can
// only write buffer A again after it has passed the barrier of the B exchange, which every peer enters only after it
// has finished reading A.
// A wait that runs out (a peer that never arrives) records an error code and the kernel returns without touching h;
// the host sees it through jsm_check_device_errors.  No in-switch reduction and no multicast objects are involved:
// a rank that leaves cannot fault its peers' GPUs.
//
// Launches of at most TP_PUSH_MAX_T tokens (every decode step) do not run this kernel at all: the exchange is fused
// into the projections on either side of it (linear_packed.cu, TpFuse).
//   push    The projection whose output is to be summed (attention output, FFN down) stores its finished bf16 tiles
//           straight into its rank's SLOT of every rank's push buffer - plain peer stores from the epilogue, no local copy
//           first - and the CTA that completes the launch releases the exchange's epoch to every peer's push flag.
//   reduce  The projection that reads the residual stream next (gate/up, the next layer's qkv, lm_head) becomes
//           resident while its predecessor still runs and streams its weights; one CTA per 128-column tile of h waits
//           for the peers' flags, adds the slots in rank order to h - LOCAL loads only: the data crossed NVLink once, as
//           stores, off the critical path of the consumer - and leaves h and the tile's sums of squares behind; all CTAs
//           then read h as their token operand with the RMSNorm applied as a row scale.
// One NVLink traversal (store + flag) lies between the two projections instead of signal -> wait -> remote load, and no
// kernel launch.  Exchanges of at most TP_INBAND_MAX_T tokens (the decode step at small batches) drop the flag as well:
// the slot holds 8-byte words {two bf16, epoch}, a word is written by one store, so its epoch says that it has arrived;
// the producer then needs no counter of finished CTAs, no system-scope fence and no flag stores (its tail is that of a
// plain projection), and the consumer's load that polls is the load that fetches (linear_bf16.cuh, TpFuse::inband).  The
// in-band words have buffers of their own: whatever a reader finds there is zero or a word of an earlier in-band exchange
// (an older epoch), never plain data that could pass for an epoch.
// Region layout: [flags | buffer A | buffer B | push buffer 0: 8 slots | push buffer 1: 8 slots | in-band buffer 0: 8 slots
// | in-band buffer 1: 8 slots | arg-max slots]; the push flags are the words TP_PUSH_FLAG_WORD.. of the flag block.  The
// same two-buffer argument holds: a rank pushes into buffer 0 again only after it has consumed the exchange over buffer
// 1, which every peer pushed only after it had finished reading buffer 0.
#include "tc_utils.cuh"
#include "linear_bf16.cuh"
#include <math.h>

namespace jsm {

constexpr int TP_MAX_RANKS = 8;
constexpr size_t TP_FLAG_BYTES = 1024;
constexpr int TP_TIMEOUT_CODE = 16;  // error word code of an exchange whose peers did not arrive in time

static long long g_tp_wait_limit_cycles = 2000000000ll;  // about one second

struct TpArgs {
    uint8_t* regions[TP_MAX_RANKS];  // regions[rank] is the local one
    int rank, size;
    size_t buf_offset;  // of the buffer of this call inside a region
    const int* pass;    // local: number of the forward pass (bumped by the pass's first kernel, long before this one runs)
    int site, n_sites;  // exchange `site` of `n_sites` per forward pass: the call's epoch is pass * n_sites + site + 1
    __nv_bfloat16* h;   // [T, d] residual stream (updated in place)
    __nv_bfloat16* xn;  // [T, d] normalised copy, or null
    float eps;
    int d;
    int* err;
    long long wait_limit;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// one CTA per token, d <= 256 * 8 * MAXV
template <int MAXV>
__global__ void __launch_bounds__(256) tp_allreduce_add_norm_kernel(TpArgs a) {
    __shared__ float red[8];
    __shared__ int ok_s;
    chain_trigger();
    chain_wait();  // this rank's projection has written its buffer (and, before it, the pass counter was bumped)
    // the epoch needs no hand-shake inside the kernel: every rank runs the same sequence of passes and sites
    const int E = *reinterpret_cast<const volatile int*>(a.pass) * a.n_sites + a.site + 1;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < a.size) {
        const int r = threadIdx.x;
        if (blockIdx.x == 0 && r != a.rank) st_release_sys(reinterpret_cast<int*>(a.regions[r]) + a.rank, E);
        if (r != a.rank) {
            const int* flag = reinterpret_cast<const int*>(a.regions[a.rank]) + r;
            const long long t0 = clock64();
            while ((int)(ld_acquire_sys(flag) - E) < 0) {  // wrap-safe: epochs only ever grow
                if (clock64() - t0 > a.wait_limit) {
                    ok_s = 0;
                    if (a.err) atomicCAS(a.err, 0, TP_TIMEOUT_CODE);
                    break;
                }
            }
        }
    }
    __syncthreads();
    const bool ok = ok_s != 0;
    const long long base = (long long)blockIdx.x * a.d;
    if (ok) {
        float v[MAXV][8];
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int c = (i * 256 + threadIdx.x) * 8;
            if (c < a.d) {
                // all ranks' loads are issued before the first add (one NVLink round trip, not one per rank); the adds run in
                // rank order: every rank forms the same sum
                uint4 w[TP_MAX_RANKS];
#pragma unroll
                for (int r = 0; r < TP_MAX_RANKS; ++r) {
                    if (r < a.size) {
                        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.regions[r] + a.buf_offset) + base + c;
                        w[r] = (r == a.rank) ? *reinterpret_cast<const uint4*>(src) : ld_relaxed_sys_v4(src);
                    }
                }
                float s[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) s[j] = 0.0f;
#pragma unroll
                for (int r = 0; r < TP_MAX_RANKS; ++r) {
                    if (r < a.size) {
                        s[0] += bf16lo(w[r].x); s[1] += bf16hi(w[r].x); s[2] += bf16lo(w[r].y); s[3] += bf16hi(w[r].y);
                        s[4] += bf16lo(w[r].z); s[5] += bf16hi(w[r].z); s[6] += bf16lo(w[r].w); s[7] += bf16hi(w[r].w);
                    }
                }
                const uint4 hw = *reinterpret_cast<const uint4*>(a.h + base + c);
                const float hv[8] = {bf16lo(hw.x), bf16hi(hw.x), bf16lo(hw.y), bf16hi(hw.y), bf16lo(hw.z), bf16hi(hw.z), bf16lo(hw.w), bf16hi(hw.w)};
                uint4 o;
                // the rank-local products were rounded to bf16 when they were stored; the sum is rounded once more, like
                // the all-reduce of a bf16 buffer followed by the residual add
                uint32_t sb[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) sb[j] = pack_bf16x2(s[2 * j], s[2 * j + 1]);
                o.x = pack_bf16x2(hv[0] + bf16lo(sb[0]), hv[1] + bf16hi(sb[0]));
                o.y = pack_bf16x2(hv[2] + bf16lo(sb[1]), hv[3] + bf16hi(sb[1]));
                o.z = pack_bf16x2(hv[4] + bf16lo(sb[2]), hv[5] + bf16hi(sb[2]));
                o.w = pack_bf16x2(hv[6] + bf16lo(sb[3]), hv[7] + bf16hi(sb[3]));
                *reinterpret_cast<uint4*>(a.h + base + c) = o;
                v[i][0] = bf16lo(o.x); v[i][1] = bf16hi(o.x); v[i][2] = bf16lo(o.y); v[i][3] = bf16hi(o.y);
                v[i][4] = bf16lo(o.z); v[i][5] = bf16hi(o.z); v[i][6] = bf16lo(o.w); v[i][7] = bf16hi(o.w);
#pragma unroll
                for (int j = 0; j < 8; ++j) q += v[i][j] * v[i][j];
            }
        }
        if (a.xn) {
            q = warp_sum(q);
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) tot += red[w];
            const float sd = sqrtf(tot / (float)a.d + a.eps);
#pragma unroll
            for (int i = 0; i < MAXV; ++i) {
                const int c = (i * 256 + threadIdx.x) * 8;
                if (c < a.d) {
                    uint4 w;
                    w.x = pack_bf16x2(v[i][0] / sd, v[i][1] / sd); w.y = pack_bf16x2(v[i][2] / sd, v[i][3] / sd);
                    w.z = pack_bf16x2(v[i][4] / sd, v[i][5] / sd); w.w = pack_bf16x2(v[i][6] / sd, v[i][7] / sd);
                    *reinterpret_cast<uint4*>(a.xn + base + c) = w;
                }
            }
        }
    }
}

constexpr int TP_PUSH_FLAG_WORD = 16;  // first push flag inside the flag block (one word per source rank)
size_t tp_slot_bytes(int d) { return (size_t)TP_PUSH_MAX_T * d * sizeof(__nv_bfloat16); }
size_t tp_argmax_offset(int max_tokens, int d);
size_t tp_region_bytes(int max_tokens, int d) { return tp_argmax_offset(max_tokens, d) + (size_t)TP_MAX_RANKS * max_tokens * 8; }
size_t tp_buffer_offset(int which, int max_tokens, int d) { return TP_FLAG_BYTES + (size_t)(which & 1) * max_tokens * d * sizeof(__nv_bfloat16); }
// slot 0 of push buffer `which`; rank r's slot follows at r * tp_slot_bytes(d)
size_t tp_push_offset(int which, int max_tokens, int d) {
    return TP_FLAG_BYTES + 2 * (size_t)max_tokens * d * sizeof(__nv_bfloat16) + (size_t)(which & 1) * TP_MAX_RANKS * tp_slot_bytes(d);
}
// The arg-max exchange of a vocabulary-sharded lm_head: every rank's (best logit, its index) per token, 8 slots of
// max_tokens pairs behind the push buffers; flag words TP_ARGMAX_FLAG_WORD.. (one per source rank)
constexpr int TP_ARGMAX_FLAG_WORD = 32;
// in-band exchanges (at most TP_INBAND_MAX_T tokens): 4 bytes per element; slot 0 of in-band buffer `which`
size_t tp_inband_slot_bytes(int d) { return (size_t)TP_INBAND_MAX_T * d * 4; }
size_t tp_inband_offset(int which, int max_tokens, int d) {
    return tp_push_offset(0, max_tokens, d) + 2 * (size_t)TP_MAX_RANKS * tp_slot_bytes(d) + (size_t)(which & 1) * TP_MAX_RANKS * tp_inband_slot_bytes(d);
}
size_t tp_argmax_offset(int max_tokens, int d) {
    const size_t off = tp_inband_offset(0, max_tokens, d) + 2 * (size_t)TP_MAX_RANKS * tp_inband_slot_bytes(d);
    return (off + 255) & ~(size_t)255;
}
int tp_push_flag_word() { return TP_PUSH_FLAG_WORD; }
long long tp_wait_limit_cycles() { return g_tp_wait_limit_cycles; }

jsm_status tp_allreduce_add_norm_launch(void* const* regions, int rank, int size, size_t buf_offset, const int* pass, int site,
                                        int n_sites, void* h, void* xn, float eps, int T, int d, cudaStream_t st) {
    if (T <= 0) return JSM_OK;
    if (!regions || !pass || !h) JSM_FAIL(JSM_INVALID_ARG, "tp_allreduce: null pointer");
    if (n_sites < 1 || site < 0 || site >= n_sites) JSM_FAIL(JSM_INVALID_ARG, "tp_allreduce: site %d of %d", site, n_sites);
    if (size < 1 || size > TP_MAX_RANKS || rank < 0 || rank >= size) JSM_FAIL(JSM_INVALID_ARG, "tp_allreduce: rank %d of %d", rank, size);
    if (d % 8 || d > 256 * 8 * 2) JSM_FAIL(JSM_UNSUPPORTED, "tp_allreduce: d %d (multiple of 8, at most 4096)", d);
    TpArgs a;
    for (int r = 0; r < TP_MAX_RANKS; ++r) a.regions[r] = r < size ? reinterpret_cast<uint8_t*>(regions[r]) : nullptr;
    for (int r = 0; r < size; ++r)
        if (!a.regions[r]) JSM_FAIL(JSM_INVALID_ARG, "tp_allreduce: region of rank %d is not connected", r);
    a.rank = rank; a.size = size; a.buf_offset = buf_offset; a.pass = pass; a.site = site; a.n_sites = n_sites;
    a.h = reinterpret_cast<__nv_bfloat16*>(h); a.xn = reinterpret_cast<__nv_bfloat16*>(xn);
    a.eps = eps; a.d = d; a.err = tc_error_word(); a.wait_limit = g_tp_wait_limit_cycles;
    JSM_CUDA_CHECK(launch_chained(tp_allreduce_add_norm_kernel<2>, dim3(T), dim3(256), 0, st, a));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

// ---- arg-max over a vocabulary that is split across the ranks --------------------------------------------------------
// Every rank has the best logit of its vocabulary slice per token (value, global index).  One CTA per rank: stores its
// pairs into its slot of every rank's region (plain peer stores), one system-scope fence, the epoch into every peer's flag
// word; waits (bounded) for the peers; takes, per token, the largest value over the ranks in rank order (the lowest index
// wins a tie, as in the one-GPU arg-max).  8 bytes per token and rank cross NVLink instead of every rank streaming the
// whole lm_head.
struct TpArgmaxArgs {
    uint8_t* regions[TP_MAX_RANKS];
    int rank, size;
    size_t slot_offset;     // of slot 0 inside a region; slot r follows at r * max_tokens * 8
    int max_tokens;
    const int* pass;
    int site, n_sites;
    const float* best_val;  // local [T]
    const int* best_idx;    // local [T], global vocabulary indices
    int32_t* out;           // [T]
    int T;
    int* err;
    long long wait_limit;
};
__global__ void __launch_bounds__(256) tp_argmax_exchange_kernel(TpArgmaxArgs a) {
    __shared__ int ok_s;
    chain_trigger();
    chain_wait();
    const int E = *reinterpret_cast<const volatile int*>(a.pass) * a.n_sites + a.site + 1;
    if (threadIdx.x == 0) ok_s = 1;
    for (int i = threadIdx.x; i < a.size * a.T; i += blockDim.x) {
        const int r = i / a.T, t = i % a.T;
        uint2 pair = make_uint2(__float_as_uint(a.best_val[t]), (uint32_t)a.best_idx[t]);
        *reinterpret_cast<uint2*>(a.regions[r] + a.slot_offset + ((size_t)a.rank * a.max_tokens + t) * 8) = pair;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        for (int r = 0; r < a.size; ++r)
            if (r != a.rank)
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(reinterpret_cast<int*>(a.regions[r]) + TP_ARGMAX_FLAG_WORD + a.rank), "r"(E) : "memory");
    }
    if (threadIdx.x < a.size && threadIdx.x != a.rank) {
        const int* flag = reinterpret_cast<const int*>(a.regions[a.rank]) + TP_ARGMAX_FLAG_WORD + threadIdx.x;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(flag) - E) < 0) {
            __nanosleep(64);
            if (clock64() - t0 > a.wait_limit) {
                ok_s = 0;
                if (a.err) atomicCAS(a.err, 0, TP_TIMEOUT_CODE);
                break;
            }
        }
    }
    __syncthreads();
    if (!ok_s) return;  // the tokens stay as they were; the error word says why
    for (int t = threadIdx.x; t < a.T; t += blockDim.x) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int r = 0; r < a.size; ++r) {
            const uint2 pair = __ldcg(reinterpret_cast<const uint2*>(a.regions[a.rank] + a.slot_offset + ((size_t)r * a.max_tokens + t) * 8));
            const float v = __uint_as_float(pair.x);
            const int idx = (int)pair.y;
            if (v > bv || (v == bv && idx < bi)) { bv = v; bi = idx; }
        }
        a.out[t] = bi == 0x7fffffff ? 0 : bi;
    }
}

jsm_status tp_argmax_exchange_launch(void* const* regions, int rank, int size, int max_tokens, int d, const int* pass, int site, int n_sites,
                                     const float* best_val, const int* best_idx, int32_t* out, int T, cudaStream_t st) {
    if (T <= 0) return JSM_OK;
    if (!regions || !pass || !best_val || !best_idx || !out) JSM_FAIL(JSM_INVALID_ARG, "tp_argmax: null pointer");
    if (size < 1 || size > TP_MAX_RANKS || rank < 0 || rank >= size || T > max_tokens) JSM_FAIL(JSM_INVALID_ARG, "tp_argmax: rank %d of %d, %d tokens", rank, size, T);
    TpArgmaxArgs a;
    for (int r = 0; r < TP_MAX_RANKS; ++r) a.regions[r] = r < size ? reinterpret_cast<uint8_t*>(regions[r]) : nullptr;
    for (int r = 0; r < size; ++r)
        if (!a.regions[r]) JSM_FAIL(JSM_INVALID_ARG, "tp_argmax: region of rank %d is not connected", r);
    a.rank = rank; a.size = size; a.slot_offset = tp_argmax_offset(max_tokens, d); a.max_tokens = max_tokens;
    a.pass = pass; a.site = site; a.n_sites = n_sites; a.best_val = best_val; a.best_idx = best_idx; a.out = out; a.T = T;
    a.err = tc_error_word(); a.wait_limit = g_tp_wait_limit_cycles;
    JSM_CUDA_CHECK(launch_chained(tp_argmax_exchange_kernel, dim3(1), dim3(256), 0, st, a));
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

}  // namespace jsm

using namespace jsm;

extern "C" size_t jsm_tp_inband_slot_offset(int which_buffer, int rank, int max_tokens, int d) {
    if (max_tokens <= 0 || d <= 0 || rank < 0 || rank >= TP_MAX_RANKS) return 0;
    return tp_inband_offset(which_buffer, max_tokens, d) + (size_t)rank * tp_inband_slot_bytes(d);
}

extern "C" size_t jsm_tp_region_bytes(int max_tokens, int d) {
    if (max_tokens <= 0 || d <= 0) return 0;
    return tp_region_bytes(max_tokens, d);
}

extern "C" jsm_status jsm_tp_set_wait_limit_ms(int ms) {
    if (ms <= 0 || ms > 60000) JSM_FAIL(JSM_INVALID_ARG, "jsm_tp_set_wait_limit_ms: %d", ms);
    g_tp_wait_limit_cycles = (long long)ms * 2000000ll;  // about 2 GHz
    return JSM_OK;
}

extern "C" jsm_status jsm_tp_allreduce_add_norm(void* const* d_regions, int rank, int size, int which_buffer, int max_tokens,
                                                const int32_t* d_pass, int site, int n_sites, void* d_h, void* d_xn, float eps, int T,
                                                int d, void* stream) {
    if (T > max_tokens) JSM_FAIL(JSM_SHAPE, "jsm_tp_allreduce_add_norm: %d tokens, the region holds %d", T, max_tokens);
    return tp_allreduce_add_norm_launch(d_regions, rank, size, tp_buffer_offset(which_buffer, max_tokens, d), d_pass, site, n_sites, d_h,
                                        d_xn, eps, T, d, as_stream(stream));
}

extern "C" jsm_status jsm_tp_argmax_exchange(void* const* d_regions, int rank, int size, int max_tokens, int d, const int32_t* d_pass, int site,
                                             int n_sites, const float* d_best_val, const int32_t* d_best_idx, int32_t* d_out, int T, void* stream) {
    return tp_argmax_exchange_launch(d_regions, rank, size, max_tokens, d, d_pass, site, n_sites, d_best_val, d_best_idx, d_out, T, as_stream(stream));
}

extern "C" jsm_status jsm_ipc_export(const void* d_ptr, unsigned char* handle64) {
    if (!d_ptr || !handle64) JSM_FAIL(JSM_INVALID_ARG, "jsm_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    JSM_CUDA_CHECK(cudaIpcGetMemHandle(&h, const_cast<void*>(d_ptr)));
    memcpy(handle64, &h, 64);
    return JSM_OK;
}

extern "C" jsm_status jsm_ipc_import(const unsigned char* handle64, void** d_ptr) {
    if (!handle64 || !d_ptr) JSM_FAIL(JSM_INVALID_ARG, "jsm_ipc_import: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    JSM_CUDA_CHECK(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return JSM_OK;
}

extern "C" jsm_status jsm_ipc_close(void* d_ptr) {
    if (!d_ptr) return JSM_OK;
    JSM_CUDA_CHECK(cudaIpcCloseMemHandle(d_ptr));
    return JSM_OK;
}
