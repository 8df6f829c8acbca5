// tcgen05 flash-attention prefill (placeholder until the kernel lands: reports itself unavailable,
// callers then use the CUDA-core kernel).
#include "attn.cuh"

namespace jsm {

bool flash_available() { return false; }

jsm_status flash_prefill_launch(const void*, const void*, const void*, void*, int, int, int, int, int, int, float, const float*,
                                cudaStream_t, long long, long long, long long) {
    JSM_FAIL(JSM_UNSUPPORTED, "flash_prefill: not built");
}

}  // namespace jsm
