/*
 * jasmine_b200 — C ABI of the B200 (sm_100a) implementation of jasmine's
 * transformer-inference hot path.
 *
 * jasmine (the reference) is a header-only C++20 library with no FFI of its
 * own: its "plugin surface" is the template/concept surface of its headers.
 * The C++20 headers under include/jasmine/ keep those spellings and lower every
 * materialisation point (`.clone()`, conversion to mat_t, `forward`) to one of
 * the calls declared here.  Each entry point cites the reference code whose
 * arithmetic it replaces (paths are relative to the reference project root).
 *
 * Conventions
 *  - Every call returns a jsm_status; on failure a thread-local message is
 *    available through jsm_last_error().
 *  - All pointers named d_* / jsm_mat::data are DEVICE pointers; h_* are host.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *    Calls are asynchronous on that stream unless stated otherwise.
 *  - No call falls back to the CPU.  Without a usable device every compute call
 *    returns JSM_CUDA.
 *  - The library reads one environment variable: JSM_PDL=0 launches the chained
 *    kernels of a decode step in plain stream order instead of with programmatic
 *    dependent launch (same results; for debugging launch-order problems).
 */
#ifndef JASMINE_B200_H_
#define JASMINE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef enum jsm_status {
    JSM_OK = 0,
    JSM_INVALID_ARG = 1, /* maps to std::invalid_argument (mat_express_t.hpp:709-712) */
    JSM_SHAPE = 2,       /* maps to std::runtime_error   (mat_mha_t.hpp:268-269)      */
    JSM_OOM = 3,
    JSM_CUDA = 4,
    JSM_NCCL = 5,
    JSM_TIMEOUT = 6, /* a bounded device-side wait ran out */
    JSM_UNSUPPORTED = 7
} jsm_status;

typedef enum jsm_dtype { JSM_F32 = 0, JSM_BF16 = 1, JSM_I32 = 2 } jsm_dtype;

/* ---- library ---------------------------------------------------------- */
const char* jsm_last_error(void);
int jsm_version(void);
/* Number of CUDA devices visible; 0 (and JSM_CUDA) when there is none. */
jsm_status jsm_device_count(int* count);
/* Count of kernels launched by this library in this process (all threads). */
uint64_t jsm_launch_count(void);

/* Synchronises `stream` and reports (then clears) the error word of the tensor-core kernels: JSM_TIMEOUT when a
 * bounded device-side wait ran out since the last check (the kernel unwound and its result is invalid). */
jsm_status jsm_check_device_errors(void* stream);

/* ---- device memory (mat_t storage: mat_t.hpp:30-69 new[]/memset/delete[]) */
jsm_status jsm_malloc(void** d_ptr, size_t bytes); /* zero-filled like init_matrix */
jsm_status jsm_free(void* d_ptr);
jsm_status jsm_upload(void* d_dst, const void* h_src, size_t bytes, void* stream);
jsm_status jsm_download(void* h_dst, const void* d_src, size_t bytes, void* stream); /* synchronises */
jsm_status jsm_memset(void* d_dst, int byte, size_t bytes, void* stream);
jsm_status jsm_stream_sync(void* stream);

/* ---- seeded synthetic data -------------------------------------------- */
/* Counter-based generator, bit-identical on host and device: element i of
 * tensor (seed, tensor_id).  dist 0: normal(mean=a, std=b) (12-uniform sum),
 * dist 1: uniform [a, b), dist 2: integer uniform [a, b) (I32 only).
 * jsm_fill_host writes the same values to host memory (f32 / bf16 bits / i32). */
jsm_status jsm_fill(void* d_dst, jsm_dtype dtype, size_t n, uint64_t seed, uint64_t tensor_id, int dist,
                    float a, float b, void* stream);
jsm_status jsm_fill_host(void* h_dst, jsm_dtype dtype, size_t n, uint64_t seed, uint64_t tensor_id, int dist,
                         float a, float b);
jsm_status jsm_convert(void* d_dst, jsm_dtype dst_dtype, const void* d_src, jsm_dtype src_dtype, size_t n,
                       void* stream);

/* ---- matrix operand ----------------------------------------------------
 * A strided 2-D window.  Element (r, c) lives at data[(r % rows) * row_stride +
 * (c % cols) * col_stride]: the modulo broadcast of mat_t::operator()
 * (mat_t.hpp:302-320).  A mat_view_t (mat_view_t.hpp:7-135) is the same struct
 * with an offset pointer; a transposed view swaps the strides. */
typedef struct jsm_mat {
    void* data;
    int32_t rows, cols;
    int64_t row_stride, col_stride; /* in elements */
    int32_t dtype;                  /* jsm_dtype */
} jsm_mat;

/* ---- expression programs (mat_express_t.hpp:35-509) --------------------
 * An expression tree is lowered by the header layer to a postfix program over
 * a value stack (depth <= 8).  Result shape = max of the leaf shapes
 * (mat_express_t.hpp:51-59). */
typedef enum jsm_op {
    JSM_OP_LEAF = 0, /* push leaves[arg](r, c)                            */
    JSM_OP_IMM = 1,  /* push imm (scalar operand, storage_selector :18-33) */
    JSM_OP_ADD = 2,  /* mat_add_t :189-223  */
    JSM_OP_SUB = 3,  /* mat_sub_t :253-286  */
    JSM_OP_MUL = 4,  /* mat_mul_t :288-321  */
    JSM_OP_DIV = 5,  /* mat_div_t :323-358  */
    JSM_OP_GT = 6,   /* mat_greater_t :119-152 -> 1.0 / 0.0 */
    JSM_OP_LT = 7,   /* mat_less_t :154-187 */
    JSM_OP_EXP = 8,  /* mat_exp_t :439-468  */
    JSM_OP_SIGMOID = 9, /* mat_sigmoid_t :479-509 */
    JSM_OP_POW = 10,    /* pow(x, imm) :587-596 */
    JSM_OP_SQRT = 11,   /* sqrt :804-813 */
    JSM_OP_NEG = 12,
    JSM_OP_RELU = 13, /* (x > 0) * x, relu_net_t::forward mat_net_t.hpp:146-153 */
    JSM_OP_GELU = 14, /* erf form; not in the reference */
    JSM_OP_SILU = 15, /* x * sigmoid(x); not in the reference */
    JSM_OP_TANH = 16
} jsm_op;

typedef struct jsm_instr {
    int32_t op;
    int32_t arg;
    float imm;
} jsm_instr;

#define JSM_MAX_INSTR 32
#define JSM_MAX_LEAVES 8
#define JSM_MAX_STACK 8

/* out(r,c) = program(leaves)(r,c) for the whole result shape.
 * Replaces mat_express_*_stable_t::clone / operator mat_t (mat_express_t.hpp:96-112, 416-432)
 * and operator+= (:225-251, out aliased with leaf 0). */
jsm_status jsm_eval_elementwise(const jsm_instr* prog, int n_instr, const jsm_mat* leaves, int n_leaves,
                                jsm_mat out, void* stream);

/* Reductions / normalisations along one axis of the value of a program.
 * axis 1: along each row  (h* functions: hsum hmax hmean hsoftmax, mat_express_t.hpp:548-628, 681-694)
 * axis 0: along each column (v* functions vsum vmean :531-546, 566-571;
 *         layer_norm_net_t::forward normalises columns, mat_net_t.hpp:209-225) */
typedef enum jsm_rows_kind {
    JSM_ROWS_SUM = 0,
    JSM_ROWS_MAX = 1,
    JSM_ROWS_MEAN = 2,
    JSM_ROWS_ARGMAX = 3,   /* out is I32; first maximum wins */
    JSM_ROWS_SOFTMAX = 4,  /* exp(x - max) / sum(exp(x - max)) */
    JSM_ROWS_LAYERNORM = 5, /* gain * (x - mean) / sqrt(mean((x-mean)^2) + eps) + bias; eps = 0 is reference-exact */
    JSM_ROWS_RMSNORM = 6    /* gain * x / sqrt(mean(x^2) + eps); not in the reference */
} jsm_rows_kind;

/* gain / bias: F32 vectors indexed along the normalised axis, or NULL (1 / 0).
 * out: reductions -> [R,1] (axis 1) or [1,C] (axis 0); others -> [R,C]. */
jsm_status jsm_eval_rows(int kind, int axis, const jsm_instr* prog, int n_instr, const jsm_mat* leaves,
                         int n_leaves, const float* d_gain, const float* d_bias, float eps, jsm_mat out,
                         void* stream);

/* Whole-matrix reductions: sum / mean / max (mat_express_t.hpp:518-529, 573-585, 598-609) into d_out[0]
 * (F32), and the whole-matrix softmax of mat_softmax_t (:630-679, global max and sum). */
jsm_status jsm_eval_full(int kind /* SUM, MAX, MEAN, SOFTMAX */, const jsm_instr* prog, int n_instr,
                         const jsm_mat* leaves, int n_leaves, jsm_mat out, void* stream);

/* ---- dense contraction, fp32 (mat_dot_t, mat_express_t.hpp:696-777) -----
 * C = A . B (+ bias broadcast by modulo, + epilogue), all F32, any strides.
 * Every output element is accumulated in ascending k with separately rounded
 * multiply and add, i.e. the order of mat_dot_t::operator() (:730-736).
 * JSM_INVALID_ARG when A.cols != B.rows (:709-712).
 * epilogue: 0 none, 1 relu, 2 gelu(erf), 3 add residual R (same shape as C). */
jsm_status jsm_dot_f32(jsm_mat A, jsm_mat B, const jsm_mat* bias, int epilogue, const jsm_mat* R, jsm_mat C,
                       void* stream);

/* ---- projections in bf16 (weight_net_t::forward, mat_net_t.hpp:38-49) ---
 * Y[t, n] = sum_k X[t, k] * W[n, k] (+ bias[n]); X:[T,K] bf16 token-major,
 * W:[N,K] bf16 (the reference's [out,in] layout), fp32 accumulation.
 * T <= 4 runs a CUDA-core weight-streaming kernel, larger T the tcgen05 kernel.
 * out_dtype: JSM_BF16 or JSM_F32.
 * epilogue: 0 none, 1 relu, 2 gelu, 3 silu(gate)*up where W holds N gate rows followed by N up rows
 * (Y is [T,N]), 4 add residual R[t,n] (bf16). */
jsm_status jsm_linear_bf16(const void* d_X, const void* d_W, const float* d_bias, int epilogue, const void* d_R,
                           void* d_Y, int out_dtype, int T, int N, int K, void* stream);

/* The same projection over weights that were packed once (inference: weight_net_t's W does not change between
 * forwards).  The packed image stores every 128-feature x 64-k tile as one contiguous 16 KB block in the
 * shared-memory layout of the tensor cores, tiles in stream order, so that the kernel reads the matrix as one linear
 * stream split evenly over all SMs.  paired != 0 packs a [2N, K] matrix of N gate rows followed by N up rows for
 * epilogue 3 (silu(gate)*up), N being the number of gate rows.
 * jsm_linear_packed_bytes: size of the packed image.  jsm_linear_pack / jsm_linear_unpack convert between the
 * reference's [out, in] layout and the packed image.  jsm_linear_bf16_packed: any T (chunks of 256 tokens);
 * N % 4 == 0, K % 8 == 0.  The tiles that several CTAs share are reduced through a per-device workspace that the calls
 * on a device share (calls that overlap on different streams would race on it).  The compute call never allocates:
 * jsm_linear_pack (or jsm_linear_packed_reserve, for a packed image that was loaded rather than packed here) sizes the
 * workspace of the current device for that shape - both synchronise the device and may allocate, so call them at
 * set-up time, outside any stream capture; jsm_linear_bf16_packed returns JSM_INVALID_ARG when the workspace of the
 * current device was never reserved for a shape this large. */
size_t jsm_linear_packed_bytes(int N, int K, int paired);
jsm_status jsm_linear_packed_reserve(int N, int K, int paired);
/* The work split of a packed projection: tiles of 128 packed rows, k-blocks of 64 per tile, CTAs in the grid
 * (CTA c streams units [c*U/G, (c+1)*U/G) of the U = n_tiles*kbt units) and the most CTAs that share one tile. */
jsm_status jsm_linear_packed_plan(int N, int K, int paired, int* n_tiles, int* kbt, int* grid, int* max_slots);
jsm_status jsm_linear_pack(const void* d_W, int N, int K, int paired, void* d_packed, void* stream);
jsm_status jsm_linear_unpack(const void* d_packed, int N, int K, int paired, void* d_W, void* stream);
jsm_status jsm_linear_bf16_packed(const void* d_X, const void* d_packed, const float* d_bias, int epilogue,
                                  const void* d_R, void* d_Y, int out_dtype, int T, int N, int K, void* stream);
/* The same call launched as a link of a kernel chain (programmatic dependent launch), which is how the decoder runner
 * launches its projections: the kernel may become resident and fetch its first weights while the kernel before it in
 * the stream is still finishing, and waits for that kernel only before it touches X, R, Y or the workspace.  The caller
 * promises that no work earlier in the stream that may still be running writes d_packed (weights that are packed once
 * and then only read: inference).  Same results, bit for bit; back-to-back projections overlap their set-up and first
 * weight requests with the predecessor's tail.  JSM_PDL=0 makes it the plain call. */
jsm_status jsm_linear_bf16_packed_chained(const void* d_X, const void* d_packed, const float* d_bias, int epilogue,
                                          const void* d_R, void* d_Y, int out_dtype, int T, int N, int K, void* stream);

/* Timeline of the packed projections (profiling aid, off by default; the reference has no tracing).  Between
 * jsm_trace_begin and jsm_trace_end every launch of the packed projection kernel (up to max_launches, eager launches
 * only: not inside a replayed graph) records 8 device time stamps in ns per CTA: resident, first weights requested,
 * predecessor complete, first stage landed, last MMA issued, first / last epilogue done, CTA done.
 * h_stamps: [n_launches][ctas_per_launch][8] uint64, zero where a CTA did not exist. */
jsm_status jsm_trace_begin(int max_launches);
jsm_status jsm_trace_end(uint64_t* h_stamps, int max_launches, int* n_launches, int* ctas_per_launch);

/* ---- RoPE (mat_RoPE_t::init mat_RoPE_t.hpp:99-134, RoPE_net_t::forward :166-188)
 * Table entry for (pair i, position m): (cos A, sin A, cos B, sin B);
 *   out0 = cosA*x0 - sinB*x1 ; out1 = sinA*x0 + cosB*x1.
 * mode 0 "reference": A = 2m / theta^(i/d), B = (2m+1) / theta^(i/d)  (the reference's table indexing)
 * mode 1 "standard" : A = B = m / theta^(2i/d).
 * d_table: F32 [max_pos, d/2, 4]. Built on the host with the reference's
 * sequence of roundings and uploaded (synchronous). */
jsm_status jsm_rope_table(float* d_table, int mode, int d, float theta, int max_pos, void* stream);
/* x, out: token-major [T, n_heads*d] (F32 or BF16); positions: I32 [T] or NULL (= t). */
jsm_status jsm_rope_apply(const void* d_x, void* d_out, jsm_dtype dtype, const float* d_table, int d, int n_heads,
                          const int32_t* d_positions, int T, void* stream);

/* Queries and keys of one prefill rotated by ONE launch (both share the positions): q [T, Hq*d], k [T, Hkv*d]; the same
 * arithmetic as two jsm_rope_apply calls (bit-identical results). */
jsm_status jsm_rope_apply_qk(const void* d_q, void* d_q_out, int Hq, const void* d_k, void* d_k_out, int Hkv, jsm_dtype dtype,
                             const float* d_table, int d, const int32_t* d_positions, int T, void* stream);

/* ---- attention (mat_head_gen_t::forward, mat_mha_t.hpp:45-74) -----------
 * q:[T_q, Hq*D], k,v:[T_k, Hkv*D] token-major, per sequence b of `batch`
 * equally long sequences; out:[T_q, Hq*D].  scores = q.k / sqrt(D) (scale passed
 * explicitly), causal mask j > i + (T_k - T_q) -> -inf (:58-67), row softmax
 * (:69), out = P.V (:71).  GQA: query head h reads kv head h / (Hq/Hkv).
 * F32: CUDA-core kernel, fp32 throughout.  BF16: tcgen05/TMEM flash kernel when
 * D == 128, fp32 accumulation; rope tables (or NULL) are applied to q and k on load. */
jsm_status jsm_attn_prefill(const void* d_q, const void* d_k, const void* d_v, void* d_out, jsm_dtype dtype,
                            int batch, int T_q, int T_k, int Hq, int Hkv, int D, int causal, float scale,
                            const float* d_rope_table, int impl /* 0 auto, 1 cuda-core, 2 tcgen05 */,
                            void* stream);

/* ---- paged KV cache (new: the reference recomputes the whole prefix per
 *      token, transformer_test.hpp:227-241) --------------------------------
 * Pool layout: [n_pages][2 (K,V)][Hkv][page_size][D] bf16, page_size = 64.
 * block_table: I32 [n_seqs, max_pages]; context_lens: I32 [n_seqs]. */
#define JSM_PAGE_SIZE 64
/* Append T new tokens (token t belongs to sequence seq_ids[t] at position positions[t]);
 * k is rotated with the rope table row of its position when d_rope_table != NULL. */
jsm_status jsm_kv_append(void* d_pool, const int32_t* d_block_table, int max_pages, const void* d_k,
                         const void* d_v, int64_t kv_row_stride, const int32_t* d_seq_ids,
                         const int32_t* d_positions, int T, int Hkv, int D, const float* d_rope_table,
                         void* stream);
/* One query token per sequence against its cached context (split-K over the
 * context, then a combine pass).  q:[n_seqs, Hq*D] bf16 (rotated here when a
 * rope table is given, at position context_len-1), out:[n_seqs, Hq*D] bf16.
 * d_scratch: F32, jsm_attn_decode_scratch_bytes() bytes for exactly this n_seqs.  The split of the context into chunks
 * depends on n_seqs (few sequences get short chunks), so the bytes are NOT monotone in n_seqs: a buffer that is reused
 * for every call of 1..max_seqs sequences must hold jsm_attn_decode_scratch_bytes_max(max_seqs, ...) bytes. */
size_t jsm_attn_decode_scratch_bytes(int n_seqs, int Hq, int D, int max_context);
size_t jsm_attn_decode_scratch_bytes_max(int max_seqs, int Hq, int D, int max_context);
jsm_status jsm_attn_decode(const void* d_q, int64_t q_row_stride, const void* d_pool,
                           const int32_t* d_block_table, int max_pages, const int32_t* d_context_lens,
                           int n_seqs, int Hq, int Hkv, int D, float scale, const float* d_rope_table,
                           int max_context, void* d_scratch, void* d_out, void* stream);

/* The decode step of one layer in a single launch: appends the new token of every sequence (d_k_new, d_v_new:
 * [n_seqs, ...] rows with pitch kv_new_stride, head h at column h*D; K is rotated with the rope row of its position
 * context_len-1 when a table is given) to the cache and attends over the context including it; the chunk partials are
 * merged by the last CTA of each (sequence, kv head), in chunk order.  d_context_lens already counts the new token.
 * d_counters: I32 [n_seqs * Hkv], zero before the first call; the kernel leaves them zero.  d_k_new may be NULL
 * (nothing to append).  Replaces jsm_kv_append + jsm_attn_decode; same arithmetic. */
jsm_status jsm_attn_decode_append(const void* d_q, int64_t q_row_stride, const void* d_k_new, const void* d_v_new,
                                  int64_t kv_new_stride, void* d_pool, const int32_t* d_block_table, int max_pages,
                                  const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D, float scale,
                                  const float* d_rope_table, int max_context, void* d_scratch, int32_t* d_counters,
                                  void* d_out, void* stream);

/* Decode attention for hosts that must not allocate.
 * No counterpart in the reference (it has neither a KV cache nor device memory).
 * Same arithmetic and arguments as jsm_attn_decode, but the per-chunk partial results live in a
 * fixed array that is part of the library image instead of a caller-supplied buffer, and the call
 * performs no cudaMalloc / cudaFree or any other allocating routine.  Meant for embedders whose
 * device-memory budget is fixed before the first request - a serving process that has handed all
 * remaining HBM to its KV page pool, or a plugin that is only given input and output buffers by
 * its host - where an allocation would fail, fragment the pool or stall the device.
 *  - Limit: jsm_attn_decode_scratch_bytes(n_seqs, Hq, D, max_context) must not exceed
 *    JSM_ATTN_DECODE_STATIC_SCRATCH_BYTES (8 MiB, held by every GPU that loads the library until
 *    the process exits); larger problems are rejected with JSM_UNSUPPORTED.
 *  - The first call on each device looks up the device address of the array; make that first call
 *    outside any stream capture.  The address is cached per device ordinal for the life of the
 *    process: after the device's primary context has been reset (cudaDeviceReset) in the same
 *    process the cached address is stale and this entry point must not be used any more.
 *  - All calls on a device share the array and it keeps the contents of the last call.  Nothing in
 *    it has to start at zero (every slot that is read is written first by the same call), but two
 *    calls that overlap on the GPU (different streams) race on it: serialise them. */
#define JSM_ATTN_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
jsm_status jsm_attn_decode_static_scratch(const void* d_q, int64_t q_row_stride, const void* d_pool,
                                          const int32_t* d_block_table, int max_pages,
                                          const int32_t* d_context_lens, int n_seqs, int Hq, int Hkv, int D,
                                          float scale, const float* d_rope_table, int max_context, void* d_out,
                                          void* stream);

/* ---- token-level helpers (not in the reference) ------------------------- */
/* Sampling from F32 logits [n_rows, vocab] (row pitch row_stride elements): temperature, top-k (0 = 1024, the most the
 * sampler considers) and top-p in (0, 1]; temperature <= 0 or top_k == 1 gives the arg-max (the reference's generation
 * loop, transformer_test.hpp:231-239, always takes it).  The draw of row r is the uniform number of the counter-based
 * generator for (seed, step, r): the same arguments give the same tokens. */
jsm_status jsm_sample(const float* d_logits, int64_t row_stride, int n_rows, int vocab, float temperature, int top_k,
                      float top_p, uint64_t seed, uint64_t step, int32_t* d_out, void* stream);
/* out[t, :] = table[ids[t], :] (+ pos_table[positions[t], :]) */
jsm_status jsm_embedding(const void* d_table, const void* d_pos_table, const int32_t* d_ids,
                         const int32_t* d_positions, void* d_out, jsm_dtype dtype, int T, int d, void* stream);
/* bf16/f32 RMSNorm / LayerNorm of token-major activations with optional fused residual add:
 * h_out = h (+ delta) ; y = norm(h_out) * gain (+ bias).  kind: JSM_ROWS_LAYERNORM / JSM_ROWS_RMSNORM. */
jsm_status jsm_add_norm(int kind, const void* d_h, const void* d_delta, void* d_h_out, void* d_y,
                        jsm_dtype dtype, const float* d_gain, const float* d_bias, float eps, int T, int d,
                        void* stream);

/* ---- decoder-only model (new; block wiring composed from the parts above;
 *      stack loop: encoder_t::forward mat_transformer_kernel_t.hpp:103-110) -- */
typedef struct jsm_model_config {
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ffn, vocab;
    int32_t max_batch, max_context; /* cache capacity */
    float norm_eps, rope_theta;
    int32_t tp_rank, tp_size; /* heads and FFN columns are split across tp_size ranks */
} jsm_model_config;

typedef struct jsm_model jsm_model;
/* all-reduce hook: sum `count` bf16 (dtype 1) / f32 (dtype 0) elements in place across the TP group, on `stream`. */
typedef int (*jsm_allreduce_fn)(void* d_buf, size_t count, int dtype, void* stream, void* user);

/* LLaMA-shape model (RMSNorm, SwiGLU, RoPE, bf16).  Weights are generated from
 * (seed, tensor id, index) ~ N(0, 0.02), norm gains 1; each TP rank generates its own shard. */
jsm_status jsm_llama_create(const jsm_model_config* cfg, uint64_t seed, jsm_model** out);
jsm_status jsm_llama_destroy(jsm_model* m);
jsm_status jsm_llama_set_allreduce(jsm_model* m, jsm_allreduce_fn fn, void* user);
/* Tensor-parallel exchange over peer memory (no counterpart in the reference, which has no parallelism).
 * Every rank owns a region [flags | buffer A | buffer B | two push buffers of 8 slots | arg-max slots] in its own memory
 * (jsm_llama_tp_region); the host makes the
 * peers' regions addressable (jsm_ipc_export / jsm_ipc_import between processes of one node) and hands them to
 * jsm_llama_tp_connect ([tp_size] device pointers, the entry of the own rank is ignored).  From then on the model sums
 * the rank-local outputs of the attention output projection and of the FFN down projection itself: one kernel per
 * exchange that signals the peers, waits (bounded) for them, adds all ranks' buffers in rank order, adds the sum into
 * the residual stream and normalises; calls of at most 64 tokens (every decode step) fuse the exchange into the
 * projections instead (jsm_tp_linear_push / jsm_tp_linear_reduce below).  Without a connection the all-reduce hook
 * (jsm_llama_set_allreduce) is used. */
jsm_status jsm_llama_tp_region(jsm_model* m, void** d_region, size_t* bytes);
jsm_status jsm_llama_tp_connect(jsm_model* m, void* const* d_peer_regions);
/* The exchange kernel on its own.  d_regions: [size] regions of jsm_tp_region_bytes(max_tokens, d) bytes, zero before
 * the first call; which_buffer 0 / 1 must alternate from call to call; the call's epoch is
 * (*d_pass) * n_sites + site + 1 and must grow from call to call, identically on every rank (d_pass: I32 in device
 * memory, written before the launch); h (bf16 [T, d]) += sum over ranks of their buffer; xn (or NULL) = RMSNorm(h)
 * without gain.
 * A peer that does not arrive within the wait limit (jsm_tp_set_wait_limit_ms, default about 1 s) raises JSM_TIMEOUT at
 * the next jsm_check_device_errors; the CTAs (one per token) time their waits separately, so the tokens whose CTA gave up
 * keep their old h while a token whose CTA still saw the flag is updated: after JSM_TIMEOUT the step's result is invalid
 * as a whole.  The self-resetting counters of the projections stay consistent (no kernel leaves one half-counted). */
size_t jsm_tp_region_bytes(int max_tokens, int d);
/* Byte offset, inside a region, of the slot into which `rank` pushes the in-band words ({two bf16, epoch} per 8 bytes,
 * 16 x d x 4 bytes per slot) of an exchange of at most 16 tokens over in-band buffer `which_buffer` (see
 * jsm_tp_linear_push).  For tests and tools that stand in for a peer; 0 on invalid arguments. */
size_t jsm_tp_inband_slot_offset(int which_buffer, int rank, int max_tokens, int d);
jsm_status jsm_tp_set_wait_limit_ms(int ms);
jsm_status jsm_tp_allreduce_add_norm(void* const* d_regions, int rank, int size, int which_buffer, int max_tokens,
                                     const int32_t* d_pass, int site, int n_sites, void* d_h, void* d_xn, float eps,
                                     int T, int d, void* stream);
/* The exchange fused into the projections around it, which is what a decode step (at most 64 tokens) runs instead of the
 * kernel above - no launch of its own, one NVLink traversal between producer and consumer:
 * jsm_tp_linear_push   Y = X . W^T (packed W [N, K], N = d_model) is not stored locally: every finished tile goes,
 *                      as bf16, straight into slot `rank` of push buffer `which_buffer` of EVERY region (peer stores
 *                      from the epilogue), and the CTA that completes the launch releases the epoch
 *                      d_state[0] * n_sites + site + 1 to every peer's push flag for this rank.
 * jsm_tp_linear_reduce the projection that reads the residual stream next: while all CTAs stream their weights, one CTA
 *                      per 128-column tile of h waits (bounded) for the peers' flags of that epoch, forms
 *                      h += sum of the size slots in rank order (local loads only), stores h and its per-tile sums
 *                      of squares (d_ssq: F32 [ceil(d/128)][T]); then Y = (h . W'^T) / sqrt(mean(h^2) + eps) with the
 *                      epilogue of jsm_linear_bf16_packed (the RMSNorm gain folded into W').
 * d_state: I32 [8] of the calling rank, zero before the first call: word 0 is the number of the forward pass (the
 * caller bumps it between passes, before any kernel of the pass can run), the rest belongs to the kernels (counters
 * of finished CTAs and reduced tiles, the epoch up to which h is reduced).  The ranks must run the same
 * sequence of (which_buffer alternating, site), epochs growing from call to call.  Workspace: as for
 * jsm_linear_bf16_packed (jsm_linear_pack / jsm_linear_packed_reserve).  A peer that does not arrive within the wait
 * limit leaves h as it is and raises JSM_TIMEOUT at the next jsm_check_device_errors.
 * Exchanges of at most 16 tokens (T of the push and of the reduce, which must be the same) do not use the flags: the
 * slot then holds 8-byte words {two bf16, epoch} - the epoch in a word says that the word has arrived, so the producer
 * needs no counter of finished CTAs, no system-scope fence and no flag stores, and the consumer's load that polls is the
 * load that fetches.  There a peer that stops in the middle of its pushes can leave the tiles that did arrive added to h
 * (JSM_TIMEOUT is raised either way); a peer that never pushes leaves h as it is. */
jsm_status jsm_tp_linear_push(void* const* d_regions, int rank, int size, int which_buffer, int max_tokens,
                              int32_t* d_state, int site, int n_sites, const void* d_X, const void* d_packed, int T,
                              int N, int K, void* stream);
jsm_status jsm_tp_linear_reduce(void* d_region, int rank, int size, int which_buffer, int max_tokens, int32_t* d_state,
                                int site, int n_sites, void* d_h, float* d_ssq, const void* d_packed, int epilogue,
                                void* d_Y, int out_dtype, int T, int N, int d, float eps, void* stream);
/* Arg-max over a vocabulary that is split across the ranks (a tensor-parallel group that is asked for tokens only lets
 * every rank stream just its share of the lm_head): d_best_val / d_best_idx hold this rank's best logit per token and its
 * index in the full vocabulary; one CTA stores the pairs into its slot of every region, releases the epoch
 * (*d_pass) * n_sites + site + 1, waits (bounded) for the peers and writes the index of the largest value over the ranks
 * (lowest index on a tie) to d_out[T].  The slots lie behind the push buffers of a region (d = d_model of the region). */
jsm_status jsm_tp_argmax_exchange(void* const* d_regions, int rank, int size, int max_tokens, int d, const int32_t* d_pass,
                                  int site, int n_sites, const float* d_best_val, const int32_t* d_best_idx, int32_t* d_out,
                                  int T, void* stream);
/* CUDA IPC plumbing for regions that live in another process of the same node (64-byte handles). */
jsm_status jsm_ipc_export(const void* d_ptr, unsigned char* handle64);
jsm_status jsm_ipc_import(const unsigned char* handle64, void** d_ptr);
jsm_status jsm_ipc_close(void* d_ptr);

/* Device pointer / element count of a named weight of this rank's shard ("layers.3.wqkv", "lm_head", ...).
 * Projections come back row-major [out, in] bf16 (wgu: gate rows, then up rows) in their stored form, i.e. with the
 * gain of the RMSNorm in front of them (wqkv: g1, wgu: g2, lm_head: gf) multiplied into their columns; gains are f32 [d]. */
jsm_status jsm_llama_weight(jsm_model* m, const char* name, void** d_ptr, size_t* n_elems);
/* Weight injection (the reference's init_t<tag>::cal, mat_init_t.hpp:10-118): replaces a named tensor of this rank's
 * shard from device memory - "emb" bf16 [vocab, d]; "gf", "layers.L.g1|g2" f32 [d]; "lm_head", "layers.L.wqkv|wo|wgu|
 * wdown" bf16 row-major [out, in] WITHOUT the gain folded in: the call multiplies the current gain of the norm in front
 * of the projection into its columns, so set a gain before the projection that follows it. */
jsm_status jsm_llama_set_weight(jsm_model* m, const char* name, const void* d_src, size_t n_elems, void* stream);
/* Flat binary checkpoint of this rank's tensors in their stored form (the reference has no serialisation:
 * mat_t.hpp:322-336 prints text only).  jsm_llama_load checks that shape and tensor-parallel rank match. */
jsm_status jsm_llama_save(jsm_model* m, const char* path);
jsm_status jsm_llama_load(jsm_model* m, const char* path);
/* Prefill `T` prompt tokens of sequence `seq` (positions 0..T-1); writes the argmax of the last position to d_next[seq]. */
jsm_status jsm_llama_prefill(jsm_model* m, const int32_t* d_ids, int seq, int T, int32_t* d_next, float* d_logits_last,
                             void* stream);
/* One greedy decode step for sequences 0..batch-1: d_ids[b] is appended at the
 * sequence's current length; d_next[b] = argmax of the logits; d_logits (or NULL): F32 [batch, vocab].
 * A sequence whose context already holds max_context tokens cannot grow: its context length stays where it is, the new
 * token overwrites the last cached position (no access outside the sequence's pages or the rope table), its outputs of
 * this step are meaningless and the next jsm_check_device_errors returns JSM_SHAPE ("context overflow"). */
jsm_status jsm_llama_decode_step(jsm_model* m, const int32_t* d_ids, int batch, int32_t* d_next, float* d_logits,
                                 void* stream);
/* The same step for callers whose tokens live in HOST memory (the reference's generation loop is host code,
 * transformer_test.hpp:227-241): h_ids[batch] in, h_next[batch] out, h_logits (or NULL) F32 [batch, vocab] out; the
 * copies run on `stream` (a non-default stream), pinned host buffers make them asynchronous up to the final
 * synchronisation, after which the outputs are valid.  The model captures the step once per batch size into a CUDA
 * graph of its own and replays it (the first call of a batch size captures: slower, and it must not itself run inside
 * a stream capture).  A tensor-parallel model that still uses the host all-reduce hook runs the step eagerly. */
jsm_status jsm_llama_decode_step_host(jsm_model* m, const int32_t* h_ids, int batch, int32_t* h_next, float* h_logits,
                                      void* stream);
/* ---- continuous batching over the paged cache (the step after decode_step; the reference's loop serves one sequence
 *      at a time by full recompute, transformer_test.hpp:231-239) -------------------------------------------------
 * jsm_llama_create_paged: like jsm_llama_create, but the KV pages form ONE pool of n_pages pages (64 positions each, all
 * layers) that is handed out on demand, instead of max_batch fixed runs of pages; n_pages may be smaller than
 * max_batch * ceil(max_context / 64) (over-subscription: admission then fails with JSM_OOM when the pool is empty).
 * The active sequences occupy the batch rows 0 .. n_active-1.
 * jsm_llama_seq_admit   takes the next free row, allocates pages for the prompt, prefills it (T <= 512 tokens) and
 *                       returns the row and the first generated token (h_logits_last or NULL: F32 [vocab]).
 * jsm_llama_step_active one greedy decode step for all active rows: h_ids[r] is appended to row r (a row that crosses a
 *                       page boundary gets a new page first), h_next[r] / h_logits (or NULL, F32 [n_active, vocab]) out.
 * jsm_llama_seq_retire  returns the row's pages to the pool; the LAST active row then takes the freed row (its block-table
 *                       row moves, its pages stay): *moved_from is that row's old index, or -1 if nothing moved.
 * Admission and retirement happen between steps; all three calls synchronise `stream` (a non-default stream).
 * A model created this way serves only these calls; one created with jsm_llama_create only the calls above. */
jsm_status jsm_llama_create_paged(const jsm_model_config* cfg, uint64_t seed, int n_pages, jsm_model** out);
jsm_status jsm_llama_seq_admit(jsm_model* m, const int32_t* h_prompt, int T, int* row, int32_t* h_first_token,
                               float* h_logits_last, void* stream);
jsm_status jsm_llama_step_active(jsm_model* m, const int32_t* h_ids, int32_t* h_next, float* h_logits, void* stream);
jsm_status jsm_llama_seq_retire(jsm_model* m, int row, int* moved_from, void* stream);
jsm_status jsm_llama_pool_state(jsm_model* m, int* n_active, int* free_pages, int* total_pages);
/* Host-side bookkeeping of context lengths (advance after a captured step is replayed). */
jsm_status jsm_llama_set_context(jsm_model* m, int seq, int context_len);
jsm_status jsm_llama_reset(jsm_model* m);
/* bytes of weights read by one decode step on this rank, and KV bytes per cached token */
jsm_status jsm_llama_step_bytes(jsm_model* m, uint64_t* weight_bytes, uint64_t* kv_bytes_per_token);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* JASMINE_B200_H_ */
