// Internal interface of the bf16 projection kernels (linear_bf16.cu).
#pragma once
#include "common.cuh"

namespace jsm {

enum LinearEpilogue { LIN_NONE = 0, LIN_RELU = 1, LIN_GELU = 2, LIN_SILU_MUL = 3, LIN_RESIDUAL = 4 };

struct LinearArgs {
    const void* X;      // [T, K] bf16
    const void* W;      // [N, K] bf16 ([2N, K] for LIN_SILU_MUL: N gate rows then N up rows)
    const float* bias;  // [N] or null
    int epilogue;
    const void* R;      // [T, N] bf16 residual or null
    void* Y;            // out_mode 0: bf16 [T,N]; 1: f32 [T,N]; 2: f32 partials [splits][T][N]
    int out_mode;
    int T, N, K;
    int splits;         // grid split along K: out_mode 2 writes the raw partials; with a workspace the kernel folds them itself
    int impl;           // 0 auto, 1 CUDA-core stream (T <= 4), 2 tcgen05
    float* ws = nullptr;      // workspace of splits * T * (N or 2N) floats for the in-kernel fix-up
    bool chained = false;     // launched as a link of a kernel chain whose weights are constant: W may be fetched before the
                              // predecessor kernel has finished (programmatic dependent launch)
    int* counters = nullptr;  // ceil(N/128) * ceil(T/BN) arrival counters, zero before the first launch
};

jsm_status linear_bf16_launch(const LinearArgs& a, cudaStream_t st);

// ---- projections over packed weights (linear_packed.cu) ----
struct PackedArgs {
    const void* X;            // [T, K] bf16, row pitch x_row_stride elements (0 = K)
    const void* Wp;           // packed weights (linear_pack_launch)
    const float* bias;        // [N] or null (16-byte aligned)
    int epilogue;             // LIN_*; LIN_SILU_MUL = weights packed as gate/up pairs, N = gate features
    const void* R;            // [T, N] bf16 residual or null
    void* Y;                  // [T, N] bf16 or f32
    bool out_f32 = false;
    int T = 0, N = 0, K = 0;  // T <= 256 per launch
    long long x_row_stride = 0;
    float* ws = nullptr;      // fp32 partials of the tiles shared between CTAs (linear_packed_ws_floats)
    size_t ws_floats = 0;
    int* counters = nullptr;  // one per tile, zero before the first launch (the kernel leaves them zero)
    int n_counters = 0;
    bool chained = false;     // link of a kernel chain: W may be fetched before the predecessor kernel ends
    // Fused RMSNorm.  ssq_in: [ssq_in_tiles][ssq_stride] per-tile sums of squares of the rows of X, as a previous launch
    // wrote them through ssq_out; then Y = (X . W'^T) / sqrt(mean(x^2) + eps) with the norm's gain already folded into
    // the packed weights.  ssq_out: [ceil(N/128)][ssq_stride], sums of squares of the bf16 outputs of this launch.
    const float* ssq_in = nullptr;
    int ssq_in_tiles = 0;
    int ssq_stride = 0;       // 0 = T
    float eps = 0.0f;
    float* ssq_out = nullptr;
    // Tensor-parallel exchange fused into the projection (tp_comm.cu describes the protocol).
    // push: the bf16 outputs are stored into this rank's slot of EVERY rank's exchange buffer (peer stores) instead of
    // Y, and the CTA that finishes last releases the call's epoch to every peer's flag word.
    // reduce: before the token operand X (= the residual stream h) is read, the launch waits for the peers' flags, forms
    // h += sum over the ranks' slots (rank order, local loads only), leaves the per-tile sums of squares of the new h in
    // ssq_in's place and only then streams X; Y = (h . W'^T) / rms(h) as with ssq_in.
    const struct TpFuse* tp = nullptr;
};

constexpr int TP_PUSH_MAX_T = 64;  // launches of at most this many tokens exchange by push; longer ones by the exchange kernel
// Exchanges of at most this many tokens travel as 8-byte words {two bf16, epoch of the exchange} (4 bytes per element in
// the slot): a word is written by one store, so its epoch says that the word has arrived - no flag, no fence, no counter of
// finished CTAs on the producer's side, and the consumer's load that polls is the load that fetches.  Larger exchanges keep
// plain bf16 slots and a flag per source rank (twice the bytes would cost them more than the flag does).  Producer and
// consumer of an exchange must agree: both decide by the token count of the forward pass.
constexpr int TP_INBAND_MAX_T = 16;
struct TpFuse {
    int n_ranks = 0, rank = 0;
    const int* pass = nullptr;     // device: number of the forward pass
    int site = 0, n_sites = 1;     // the exchange's place in the pass: epoch = pass * n_sites + site + 1
    int* state = nullptr;          // device, local, 4 words, zero at first: [0] folding CTAs of a pushing launch done, [1] tiles of h
                                   // reduced (both self-resetting), [2] epoch up to which h is completely reduced
    // push
    bool inband = false;           // {two bf16, epoch} words instead of bf16 slots and flags (TP_INBAND_MAX_T)
    bool push = false;
    void* push_dst[8] = {nullptr};   // per rank: where this rank's [T, N] block goes in that rank's memory
    int* push_flag[8] = {nullptr};   // per rank: that rank's flag word for this rank
    // reduce
    bool reduce = false;
    const void* slots = nullptr;     // local: rank r's block at slots + r * slot_stride bytes
    size_t slot_stride = 0;
    const int* flags = nullptr;      // local: flag word per source rank
    void* h = nullptr;               // [T, d] bf16 rows to update (d = K of the launch)
    float* ssq = nullptr;            // [ceil(d/128)][ssq_stride] sums of squares of the new h (becomes ssq_in)
    long long wait_limit = 0;        // cycles
};
// Row of the logical (stacked) weight matrix that packed row r of tile j holds; -1 = padding.
// plain : rows j*128 .. j*128+127 of an [N, K] matrix.
// paired: the matrix is [2*N, K] = N gate rows then N up rows; tile j holds gate rows j*64..+63 in its first 64
//         packed rows and the matching up rows in its last 64, so that silu(gate)*up needs one tile only.
__host__ __device__ inline long long pk_source_row(int paired, int N, int j, int r) {
    if (!paired) {
        const long long row = (long long)j * 128 + r;
        return row < N ? row : -1;
    }
    const long long f = (long long)j * 64 + (r & 63);
    if (f >= N) return -1;
    return r < 64 ? f : (long long)N + f;
}

size_t linear_packed_bytes(int N, int K, int paired);
size_t linear_packed_ws_floats(int T, int N, int K, int paired);
// packs (or, with unpack, rebuilds) a row-major [N, K] matrix ([2N, K] gate rows then up rows when paired)
jsm_status linear_pack_launch(const void* W, int N, int K, int paired, void* packed, bool unpack, cudaStream_t st);
jsm_status linear_packed_launch(const PackedArgs& a, cudaStream_t st);
// exchange regions (tp_comm.cu): [flags | buffer A | buffer B | push buffer 0 | push buffer 1]
size_t tp_region_bytes(int max_tokens, int d);
size_t tp_buffer_offset(int which, int max_tokens, int d);
size_t tp_push_offset(int which, int max_tokens, int d);
size_t tp_slot_bytes(int d);
size_t tp_inband_offset(int which, int max_tokens, int d);
size_t tp_inband_slot_bytes(int d);
int tp_push_flag_word();
long long tp_wait_limit_cycles();
// whether a plain bf16 projection of this shape and token count can push its outputs (TpFuse::push)
bool linear_packed_can_push(int N, int K, int T);
// dimensions of the packed image
void pk_dims(int N, int K, int paired, int* n_tiles, int* kbt);
// reads (and clears) the device error word of the tensor-core kernels; synchronises the stream
jsm_status tc_check_error(cudaStream_t st, const char* who);

}  // namespace jsm
