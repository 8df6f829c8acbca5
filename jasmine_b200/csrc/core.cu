// Library plumbing of the C ABI: error strings, device memory, seeded fills, dtype conversion.
#include "common.cuh"
#include <string.h>
#include <stdlib.h>

namespace jsm {

static thread_local char t_error[512] = "";
std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

bool chained_launch_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("JSM_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

__global__ void fill_kernel(void* dst, int dtype, size_t n, uint64_t key, int dist, float a, float b) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        if (dtype == JSM_I32) {
            reinterpret_cast<int32_t*>(dst)[i] = rng_int(key, i, (int32_t)a, (int32_t)b);
        } else {
            float v = rng_value(key, i, dist, a, b);
            if (dtype == JSM_F32)
                reinterpret_cast<float*>(dst)[i] = v;
            else
                reinterpret_cast<uint16_t*>(dst)[i] = f32_to_bf16_bits(v);
        }
    }
}

__global__ void convert_kernel(void* dst, int dd, const void* src, int sd, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = sd == JSM_F32 ? reinterpret_cast<const float*>(src)[i]
                                : bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(src)[i]);
        if (dd == JSM_F32)
            reinterpret_cast<float*>(dst)[i] = v;
        else
            reinterpret_cast<uint16_t*>(dst)[i] = f32_to_bf16_bits(v);
    }
}

}  // namespace jsm

using namespace jsm;

extern "C" {

const char* jsm_last_error(void) { return t_error; }
int jsm_version(void) { return 100; }
uint64_t jsm_launch_count(void) { return g_launches.load(); }

jsm_status jsm_device_count(int* count) {
    if (!count) JSM_FAIL(JSM_INVALID_ARG, "jsm_device_count: null argument");
    *count = 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        JSM_FAIL(JSM_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
    }
    *count = n;
    return JSM_OK;
}

jsm_status jsm_malloc(void** d_ptr, size_t bytes) {
    if (!d_ptr) JSM_FAIL(JSM_INVALID_ARG, "jsm_malloc: null argument");
    *d_ptr = nullptr;
    if (bytes == 0) return JSM_OK;
    JSM_CUDA_CHECK(cudaMalloc(d_ptr, bytes));
    JSM_CUDA_CHECK(cudaMemset(*d_ptr, 0, bytes));
    return JSM_OK;
}

jsm_status jsm_free(void* d_ptr) {
    if (d_ptr) JSM_CUDA_CHECK(cudaFree(d_ptr));
    return JSM_OK;
}

jsm_status jsm_upload(void* d_dst, const void* h_src, size_t bytes, void* stream) {
    if (bytes == 0) return JSM_OK;
    if (!d_dst || !h_src) JSM_FAIL(JSM_INVALID_ARG, "jsm_upload: null pointer");
    JSM_CUDA_CHECK(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return JSM_OK;
}

jsm_status jsm_download(void* h_dst, const void* d_src, size_t bytes, void* stream) {
    if (bytes == 0) return JSM_OK;
    if (!h_dst || !d_src) JSM_FAIL(JSM_INVALID_ARG, "jsm_download: null pointer");
    JSM_CUDA_CHECK(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    JSM_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream)));
    return JSM_OK;
}

jsm_status jsm_memset(void* d_dst, int byte, size_t bytes, void* stream) {
    if (bytes == 0) return JSM_OK;
    if (!d_dst) JSM_FAIL(JSM_INVALID_ARG, "jsm_memset: null pointer");
    JSM_CUDA_CHECK(cudaMemsetAsync(d_dst, byte, bytes, as_stream(stream)));
    return JSM_OK;
}

jsm_status jsm_stream_sync(void* stream) {
    JSM_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream)));
    return JSM_OK;
}

jsm_status jsm_fill(void* d_dst, jsm_dtype dtype, size_t n, uint64_t seed, uint64_t tensor_id, int dist, float a,
                    float b, void* stream) {
    if (n == 0) return JSM_OK;
    if (!d_dst) JSM_FAIL(JSM_INVALID_ARG, "jsm_fill: null pointer");
    if (dist < 0 || dist > 2 || (dtype == JSM_I32) != (dist == 2))
        JSM_FAIL(JSM_INVALID_ARG, "jsm_fill: dist %d does not fit dtype %d", dist, (int)dtype);
    size_t blocks = (n + 255) / 256;
    size_t cap = (size_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    fill_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(d_dst, (int)dtype, n, rng_key(seed, tensor_id),
                                                                   dist, a, b);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

jsm_status jsm_fill_host(void* h_dst, jsm_dtype dtype, size_t n, uint64_t seed, uint64_t tensor_id, int dist,
                         float a, float b) {
    if (n == 0) return JSM_OK;
    if (!h_dst) JSM_FAIL(JSM_INVALID_ARG, "jsm_fill_host: null pointer");
    if (dist < 0 || dist > 2 || (dtype == JSM_I32) != (dist == 2))
        JSM_FAIL(JSM_INVALID_ARG, "jsm_fill_host: dist %d does not fit dtype %d", dist, (int)dtype);
    uint64_t key = rng_key(seed, tensor_id);
    for (size_t i = 0; i < n; ++i) {
        if (dtype == JSM_I32) {
            reinterpret_cast<int32_t*>(h_dst)[i] = rng_int(key, i, (int32_t)a, (int32_t)b);
        } else {
            float v = rng_value(key, i, dist, a, b);
            if (dtype == JSM_F32)
                reinterpret_cast<float*>(h_dst)[i] = v;
            else
                reinterpret_cast<uint16_t*>(h_dst)[i] = f32_to_bf16_bits(v);
        }
    }
    return JSM_OK;
}

jsm_status jsm_convert(void* d_dst, jsm_dtype dd, const void* d_src, jsm_dtype sd, size_t n, void* stream) {
    if (n == 0) return JSM_OK;
    if (!d_dst || !d_src) JSM_FAIL(JSM_INVALID_ARG, "jsm_convert: null pointer");
    if (dd == JSM_I32 || sd == JSM_I32) JSM_FAIL(JSM_UNSUPPORTED, "jsm_convert: only f32 <-> bf16");
    size_t blocks = (n + 255) / 256;
    size_t cap = (size_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    convert_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(d_dst, (int)dd, d_src, (int)sd, n);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}

}  // extern "C"
