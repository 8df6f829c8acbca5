// Shared host/device helpers of the jasmine_b200 C-ABI library: status handling,
// launch accounting, the counter-based generator, small vector types.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>
#include "../../include/jasmine_b200.h"

namespace jsm {

// ---- status / errors ------------------------------------------------------
void set_error(const char* fmt, ...);
extern std::atomic<uint64_t> g_launches;

#define JSM_FAIL(code, ...)            \
    do {                               \
        ::jsm::set_error(__VA_ARGS__); \
        return (code);                 \
    } while (0)

#define JSM_CUDA_CHECK(expr)                                                                  \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            ::jsm::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                             __LINE__);                                                       \
            return e__ == cudaErrorMemoryAllocation ? JSM_OOM : JSM_CUDA;                     \
        }                                                                                     \
    } while (0)

// Called after every kernel launch: counts it and turns a launch error into a status.
#define JSM_LAUNCH_CHECK()                          \
    do {                                            \
        ::jsm::g_launches.fetch_add(1);             \
        JSM_CUDA_CHECK(cudaGetLastError());         \
    } while (0)

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
int sm_count();

// ---- programmatic dependent launch ------------------------------------------------
// The kernels of a decode step are chained with programmatic stream serialisation: a kernel may become
// resident while its predecessor still runs, do the work that does not depend on it (barrier set-up, TMEM
// allocation, streaming or prefetching its WEIGHTS, which no kernel writes) and only then wait for the
// predecessor's results.  Rules every kernel launched through launch_chained keeps:
//   * chain_trigger() first, so that its own successor can be made resident early;
//   * chain_wait() before the first access (read or write) to anything another kernel of the stream
//     produces or consumes; it returns once the predecessor grid has completed and its writes are visible.
// Both are no-ops for a kernel launched without the attribute.
bool chained_launch_enabled();  // JSM_PDL=0 in the environment turns the attribute off (plain stream order)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- counter-based generator (bit-identical on host and device) ------------
__host__ __device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline uint64_t rng_key(uint64_t seed, uint64_t tensor_id) {
    return splitmix64(splitmix64(seed) ^ (tensor_id * 0xD1342543DE82EF95ull));
}
// Standard normal from the sum of twelve 16-bit uniforms (Irwin-Hall): integer
// arithmetic, then one exact int->float conversion, one subtraction and one
// multiplication, so that host and device agree to the bit.
__host__ __device__ inline float rng_normal(uint64_t key, uint64_t idx) {
    uint32_t acc = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        uint64_t h = splitmix64(key + 3ull * idx + (uint64_t)j);
        acc += (uint32_t)(h & 0xFFFF) + (uint32_t)((h >> 16) & 0xFFFF) + (uint32_t)((h >> 32) & 0xFFFF) +
               (uint32_t)((h >> 48) & 0xFFFF);
    }
    float f = (float)acc;  // < 2^20: exact
#ifdef __CUDA_ARCH__
    return __fmul_rn(__fsub_rn(f, 393210.0f), 1.0f / 65536.0f);
#else
    volatile float d = f - 393210.0f;
    return d * (1.0f / 65536.0f);
#endif
}
__host__ __device__ inline float rng_uniform01(uint64_t key, uint64_t idx) {
    uint64_t h = splitmix64(key + idx);
    return (float)(uint32_t)(h >> 40) * (1.0f / 16777216.0f);  // 24 bits: exact
}
__host__ __device__ inline float rng_value(uint64_t key, uint64_t idx, int dist, float a, float b) {
    if (dist == 0) {
        float n = rng_normal(key, idx);
#ifdef __CUDA_ARCH__
        return __fadd_rn(a, __fmul_rn(b, n));
#else
        volatile float p = b * n;
        return a + p;
#endif
    }
    float u = rng_uniform01(key, idx);
#ifdef __CUDA_ARCH__
    return __fadd_rn(a, __fmul_rn(__fsub_rn(b, a), u));
#else
    volatile float w = b - a;
    volatile float p = w * u;
    return a + p;
#endif
}
__host__ __device__ inline int32_t rng_int(uint64_t key, uint64_t idx, int32_t lo, int32_t hi) {
    uint64_t h = splitmix64(key + idx);
    uint64_t span = (uint64_t)(uint32_t)(hi - lo);
    return lo + (int32_t)(((h >> 32) * span) >> 32);
}

// ---- bf16 helpers -----------------------------------------------------------
__host__ __device__ inline uint16_t f32_to_bf16_bits(float f) {
    union { float f; uint32_t u; } v;
    v.f = f;
    uint32_t u = v.u;
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x40);  // NaN
    uint32_t r = 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)((u + r) >> 16);
}
__host__ __device__ inline float bf16_bits_to_f32(uint16_t b) {
    union { float f; uint32_t u; } v;
    v.u = (uint32_t)b << 16;
    return v.f;
}

#ifdef __CUDACC__
__device__ __forceinline__ void chain_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
#endif

}  // namespace jsm
