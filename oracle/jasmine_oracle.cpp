// TEST INFRASTRUCTURE, not product code.
//
// CPU restatement ("port") of the arithmetic of jasmine's inference hot path, in
// plain C++ over dense float arrays.  Every function cites the reference code it
// follows (paths relative to the reference project root) and keeps its order of
// floating-point operations: sequential left-to-right sums, k-ascending dot
// products with separately rounded multiply and add, libm expf/cosf/sinf.
// The port is pinned against the reference itself (oracle/_ref, built from the
// reference headers) by tests/test_oracle.py and by the vectors under
// tests/golden/, which were produced by running the reference's own code.
// Parts that the reference lacks (RMSNorm, GELU, SiLU, GQA, standard RoPE,
// embeddings, argmax, the LLaMA-shape block) are restated from the formulas given
// in the comments.
//
// Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load
// this library; the product never does.
//
// Layout: "token-major" [T, d] means the reference's [d, T] matrix transposed, so
// a token's features are contiguous.  OpenMP only parallelises across independent
// output elements; it never changes the order of a sum.
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

static inline float bf16_round(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return f;
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    memcpy(&f, &u, 4);
    return f;
}

// modulo broadcast of mat_t::operator() (mat_t.hpp:302-320)
static inline float at(const float* p, int R, int C, int r, int c) { return p[(long)(r % R) * C + (c % C)]; }

// ---- a3/a4: elementwise nodes (mat_express_t.hpp:119-509); result shape = max (:51-59)
// op numbering as in ref_harness.cpp: 0 + 1 - 2 * 3 / 4 > 5 < 6 exp 7 sigmoid 8 A*s+B 9 (A>0)*A
// 10 pow(A,s) 11 sqrt 12 A+=B 13 ((A+B-A)*B/A) 14 A*s 15 A+s
API int orc_expr(int op, const float* A, int R, int C, const float* B, int Br, int Bc, float s, float* out) {
    if (op < 0 || op > 15) return 1;
    const int OR = (B && Br > R && op != 12) ? Br : R, OC = (B && Bc > C && op != 12) ? Bc : C;
#pragma omp parallel for
    for (int i = 0; i < OR; ++i)
        for (int j = 0; j < OC; ++j) {
            const float a = at(A, R, C, i, j);
            const float b = B ? at(B, Br, Bc, i, j) : 0.0f;
            float y;
            switch (op) {
                case 0: y = a + b; break;
                case 1: y = a - b; break;
                case 2: y = a * b; break;
                case 3: y = a / b; break;
                case 4: y = a > b ? 1.0f : 0.0f; break;
                case 5: y = a < b ? 1.0f : 0.0f; break;
                case 6: y = expf(a); break;                                           // mat_exp_t :453-456
                case 7: y = (float)(1.0 / (1.0 + (double)expf(-a))); break;           // mat_sigmoid_t :493-496 (double 1.0)
                case 8: { float t = a * s; y = t + b; } break;
                case 9: y = (a > 0 ? 1.0f : 0.0f) * a; break;                         // relu_net_t mat_net_t.hpp:146-153
                case 10: y = (float)std::pow((double)a, (double)s); break;            // pow :587-596
                case 11: y = std::sqrt(a); break;                                      // sqrt :804-813
                case 12: y = a + b; break;                                             // operator+= :225-238
                case 13: { float t = a + b; float u = t - a; float w = u * b; y = w / a; } break;
                case 14: y = a * s; break;
                case 15: y = a + s; break;
                default: y = NAN; break;
            }
            out[(long)i * OC + j] = y;
        }
    return 0;
}

// ---- a6: eager reductions (mat_express_t.hpp:511-628); sequential left-to-right in float
// kind: 0 hsum 1 hmax 2 hmean 3 vsum 4 vmean 5 sum 6 mean 7 max
API int orc_reduce(int kind, const float* A, int R, int C, float* out) {
    const float lowest = std::numeric_limits<float>::lowest();
    switch (kind) {
        case 0: case 1: case 2:
#pragma omp parallel for
            for (int i = 0; i < R; ++i) {
                float s = kind == 1 ? lowest : 0.0f;
                for (int j = 0; j < C; ++j) {
                    float v = A[(long)i * C + j];
                    if (kind == 1) { if (v > s) s = v; } else s += v;
                }
                out[i] = kind == 2 ? s / C : s;  // hmean = hsum / col_num (:573-578)
            }
            return 0;
        case 3: case 4:
#pragma omp parallel for
            for (int j = 0; j < C; ++j) {
                float s = 0.0f;
                for (int i = 0; i < R; ++i) s += A[(long)i * C + j];
                out[j] = kind == 4 ? s / R : s;
            }
            return 0;
        case 5: case 6: {
            float s = 0.0f;
            for (long i = 0; i < (long)R * C; ++i) s += A[i];
            out[0] = kind == 6 ? s / (R * C) : s;
            return 0;
        }
        case 7: {
            float s = lowest;
            for (long i = 0; i < (long)R * C; ++i) if (A[i] > s) s = A[i];
            out[0] = s;
            return 0;
        }
    }
    return 1;
}

// ---- a7: hsoftmax (mat_express_t.hpp:681-694): row max, exp(x - max), row sum, divide
static void hsoftmax_row(const float* x, int C, float* y) {
    float m = std::numeric_limits<float>::lowest();
    for (int j = 0; j < C; ++j) if (x[j] > m) m = x[j];
    float s = 0.0f;
    for (int j = 0; j < C; ++j) { y[j] = expf(x[j] - m); s += y[j]; }
    for (int j = 0; j < C; ++j) y[j] = y[j] / s;
}
API int orc_hsoftmax(const float* A, const float* B, float s, int R, int C, float* out) {
#pragma omp parallel for
    for (int i = 0; i < R; ++i) {
        std::vector<float> x(C);
        for (int j = 0; j < C; ++j) {
            float a = A[(long)i * C + j];
            if (B) { float t = a * s; a = t + B[(long)i * C + j]; }
            x[j] = a;
        }
        hsoftmax_row(x.data(), C, out + (long)i * C);
    }
    return 0;
}
// a5: whole-matrix softmax of mat_softmax_t (:630-665): global max, global sum of exp(x - max)
API int orc_softmax_full(const float* A, int R, int C, float* out) {
    const long n = (long)R * C;
    float m = std::numeric_limits<float>::lowest();
    for (long i = 0; i < n; ++i) if (A[i] > m) m = A[i];
    float s = 0.0f;
    for (long i = 0; i < n; ++i) s += expf(A[i] - m);
    for (long i = 0; i < n; ++i) out[i] = expf(A[i] - m) / s;
    return 0;
}

// ---- a11: layer_norm_net_t::forward (mat_net_t.hpp:209-225) on token-major rows:
// mean = sum/d; delta = x - mean; std = sqrt(mean(delta^2) + eps); y = gain * (delta/std) + bias.
// eps = 0 and gain/bias NULL reproduce the reference exactly.  x2 (optional) is added to x first.
API int orc_layer_norm_rows(const float* x, const float* x2, int T, int d, const float* gain, const float* bias, float eps,
                            float* out) {
#pragma omp parallel for
    for (int t = 0; t < T; ++t) {
        std::vector<float> v(d);
        for (int i = 0; i < d; ++i) v[i] = x2 ? x[(long)t * d + i] + x2[(long)t * d + i] : x[(long)t * d + i];
        float s = 0.0f;
        for (int i = 0; i < d; ++i) s += v[i];
        const float mean = s / d;
        float q = 0.0f;
        for (int i = 0; i < d; ++i) { v[i] = v[i] - mean; q += (float)std::pow((double)v[i], 2.0); }
        float var = q / d;
        const float sd = std::sqrt(var + eps);
        for (int i = 0; i < d; ++i) {
            float hx = v[i] / sd;
            float gx = (gain ? gain[i] : 1.0f) * hx;
            out[(long)t * d + i] = gx + (bias ? bias[i] : 0.0f);
        }
    }
    return 0;
}
// RMSNorm (not in the reference): y = gain * (x / sqrt(mean(x^2) + eps)), same primitive order as above
API int orc_rms_norm_rows(const float* x, int T, int d, const float* gain, float eps, float* out) {
#pragma omp parallel for
    for (int t = 0; t < T; ++t) {
        float q = 0.0f;
        for (int i = 0; i < d; ++i) { float v = x[(long)t * d + i]; q += v * v; }
        float ms = q / d;
        const float r = std::sqrt(ms + eps);
        for (int i = 0; i < d; ++i) {
            float hx = x[(long)t * d + i] / r;
            out[(long)t * d + i] = (gain ? gain[i] : 1.0f) * hx;
        }
    }
    return 0;
}

// ---- a8: mat_dot_t::operator() (mat_express_t.hpp:730-736): s = 0; s += l(i,k) * r(k,j), k ascending
API int orc_dot(const float* A, int M, int K, const float* B, int K2, int N, float* out) {
    if (K != K2) return 1;  // std::invalid_argument (:709-712)
#pragma omp parallel for
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float s = 0.0f;
            for (int k = 0; k < K; ++k) { float p = A[(long)i * K + k] * B[(long)k * N + j]; s += p; }
            out[(long)i * N + j] = s;
        }
    return 0;
}
// a9: weight_net_t::forward (mat_net_t.hpp:38-43), token-major: Y[t,n] = (sum_k W[n,k]*X[t,k]) + b[n]
// With several tokens the same sums are formed for a block of tokens at a time: X is transposed once so that the tokens
// of one k are contiguous, and every accumulator still receives its products in ascending k with separately rounded
// multiply and add (no contraction: -ffp-contract=off), so the results are bit-identical to the scalar loop - the
// compiler may merely keep several tokens in one vector register.
__attribute__((target_clones("avx2", "default")))
static void linear_rows_block(const float* XT, const float* W, const float* b, int T, int Tp, int N, int K, float* Y, int n0, int n1) {
    std::vector<float> acc(Tp);
    for (int n = n0; n < n1; ++n) {
        const float* w = W + (long)n * K;
        float* a = acc.data();
        for (int t = 0; t < Tp; ++t) a[t] = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float wk = w[k];
            const float* x = XT + (long)k * Tp;
#pragma omp simd
            for (int t = 0; t < Tp; ++t) { float p = wk * x[t]; a[t] += p; }
        }
        for (int t = 0; t < T; ++t) Y[(long)t * N + n] = b ? a[t] + b[n] : a[t];
    }
}
static void linear(const float* X, const float* W, const float* b, int T, int N, int K, float* Y) {
    if (T >= 4) {
        const int Tp = (T + 7) / 8 * 8;
        std::vector<float> XT((long)K * Tp, 0.0f);
        for (int t = 0; t < T; ++t)
            for (int k = 0; k < K; ++k) XT[(long)k * Tp + t] = X[(long)t * K + k];
        const int NB = 16;
#pragma omp parallel for schedule(dynamic)
        for (int n0 = 0; n0 < N; n0 += NB) linear_rows_block(XT.data(), W, b, T, Tp, N, K, Y, n0, n0 + NB < N ? n0 + NB : N);
        return;
    }
#pragma omp parallel for
    for (int t = 0; t < T; ++t)
        for (int n = 0; n < N; ++n) {
            float s = 0.0f;
            const float* w = W + (long)n * K;
            const float* x = X + (long)t * K;
            for (int k = 0; k < K; ++k) { float p = w[k] * x[k]; s += p; }
            Y[(long)t * N + n] = b ? s + b[n] : s;
        }
}
API int orc_linear(const float* X, const float* W, const float* b, int T, int N, int K, float* Y) {
    linear(X, W, b, T, N, K, Y);
    return 0;
}

static inline float gelu_erf(float v) { return 0.5f * v * (1.0f + std::erf(v * 0.70710678118654752440f)); }
static inline float sigmoid_ref(float v) { return (float)(1.0 / (1.0 + (double)expf(-v))); }  // mat_express_t.hpp:493-496
// kind: 0 relu (mat_net_t.hpp:146-153) 1 sigmoid (:101-106) 2 gelu(erf) 3 silu = x*sigmoid(x)
API int orc_activation(int kind, const float* X, long n, float* Y) {
#pragma omp parallel for
    for (long i = 0; i < n; ++i) {
        float v = X[i];
        Y[i] = kind == 0 ? (v > 0 ? 1.0f : 0.0f) * v : kind == 1 ? sigmoid_ref(v) : kind == 2 ? gelu_erf(v) : v * sigmoid_ref(v);
    }
    return 0;
}

// ---- a18: RoPE table (mat_RoPE_t::init, mat_RoPE_t.hpp:99-134) ----------------------
// table[pos][pair] = (cos A, sin A, cos B, sin B).
// mode 0 (reference): the 2x2 block of (pair i, position m) is T[2i..2i+1, 2m..2m+1] with
//   T(r,c): angle = c / pow(10000.0, (r/2)/float(d)) rounded to float (:113), so A uses c = 2m, B uses c = 2m+1.
// mode 1 (standard): A = B = m / theta^(2i/d).
API int orc_rope_table(int mode, int d, float theta, int max_pos, float* table) {
    for (int m = 0; m < max_pos; ++m)
        for (int i = 0; i < d / 2; ++i) {
            float a, b;
            if (mode == 0) {
                const double p = std::pow((double)theta, (double)((float)i / (float)d));
                a = (float)((2 * m) / p);
                b = (float)((2 * m + 1) / p);
            } else {
                const double p = std::pow((double)theta, (double)((float)(2 * i) / (float)d));
                a = b = (float)(m / p);
            }
            float* e = table + ((long)m * (d / 2) + i) * 4;
            e[0] = std::cos(a); e[1] = std::sin(a); e[2] = std::cos(b); e[3] = std::sin(b);
        }
    return 0;
}
// RoPE_net_t::forward (:166-188): out[2i..2i+1] = block . x[2i..2i+1], the dot accumulating from 0
// x, out: [T, n_heads*d]; positions NULL -> t
API int orc_rope_apply(const float* x, float* out, const float* table, int d, int n_heads, const int* positions, int T) {
#pragma omp parallel for
    for (int t = 0; t < T; ++t) {
        const int m = positions ? positions[t] : t;
        for (int h = 0; h < n_heads; ++h)
            for (int i = 0; i < d / 2; ++i) {
                const float* e = table + ((long)m * (d / 2) + i) * 4;
                const float x0 = x[((long)t * n_heads + h) * d + 2 * i], x1 = x[((long)t * n_heads + h) * d + 2 * i + 1];
                float p0 = e[0] * x0, p1 = (-e[3]) * x1, p2 = e[1] * x0, p3 = e[2] * x1;
                float s0 = 0.0f + p0, s1 = 0.0f + p2;
                out[((long)t * n_heads + h) * d + 2 * i] = s0 + p1;
                out[((long)t * n_heads + h) * d + 2 * i + 1] = s1 + p3;
            }
    }
    return 0;
}

// ---- a15: attention of mat_head_gen_t::forward (mat_mha_t.hpp:53-71) on given q,k,v -----
// q:[batch*Tq, Hq*D], k,v:[batch*Tk, Hkv*D] token-major, out like q.
// scores(i,j) = float( double(sum_d q_i[d]*k_j[d]) / sqrt(double(D)) )   (:53, the quotient is double, then
//   narrowed when hsoftmax_net_t<mat_t<float>> takes it, mat_net_t.hpp:273-279); when exact_div == 0 the
//   score is the float product dot*scale instead.
// causal: j > i + (Tk - Tq) -> -inf (:58-67); weights = hsoftmax(scores) (:69); out_i[d] = sum_j v_j[d]*w(i,j) (:71)
API int orc_attention(const float* q, const float* k, const float* v, float* out, int batch, int Tq, int Tk, int Hq,
                      int Hkv, int D, int causal, float scale, int exact_div) {
    const int group = Hq / Hkv;
    const double root = std::sqrt((double)D);
#pragma omp parallel for collapse(2)
    for (int b = 0; b < batch; ++b)
        for (int h = 0; h < Hq; ++h) {
            const int hk = h / group;
            std::vector<float> sc(Tk), w(Tk);
            for (int i = 0; i < Tq; ++i) {
                const float* qi = q + ((long)(b * Tq + i) * Hq + h) * D;
                for (int j = 0; j < Tk; ++j) {
                    const float* kj = k + ((long)(b * Tk + j) * Hkv + hk) * D;
                    float s = 0.0f;
                    for (int d = 0; d < D; ++d) { float p = qi[d] * kj[d]; s += p; }
                    sc[j] = exact_div ? (float)((double)s / root) : s * scale;
                    if (causal && j > i + (Tk - Tq)) sc[j] = -std::numeric_limits<float>::infinity();
                }
                hsoftmax_row(sc.data(), Tk, w.data());
                float* oi = out + ((long)(b * Tq + i) * Hq + h) * D;
                for (int d = 0; d < D; ++d) {
                    float s = 0.0f;
                    for (int j = 0; j < Tk; ++j) { float p = v[((long)(b * Tk + j) * Hkv + hk) * D + d] * w[j]; s += p; }
                    oi[d] = s;
                }
            }
        }
    return 0;
}

// ---- a15-a17: mat_mha_t::forward (mat_mha_t.hpp:265-291), token-major -----------------
// weights in the reference's init order: per head q(W[dh,dh], b[dh]) k(..) v(..), then out proj W[d,d], b[d].
// Each head projects only its own slice of the input (vsplit :199-215; block-diagonal projections).
static long mha_weight_count(int H, int d) { long dh = d / H; return (long)H * 3 * (dh * dh + dh) + ((long)d * d + d); }
static void mha_forward(const float* w, const float* x, int T, int H, int d, int causal, float* out) {
    const int dh = d / H;
    std::vector<float> q((long)T * d), k((long)T * d), v((long)T * d), cat((long)T * d);
    for (int h = 0; h < H; ++h) {
        const float* wh = w + (long)h * 3 * (dh * dh + dh);
        float* dst[3] = {q.data(), k.data(), v.data()};
        for (int p = 0; p < 3; ++p) {
            const float* W = wh + (long)p * (dh * dh + dh);
            const float* b = W + (long)dh * dh;
#pragma omp parallel for
            for (int t = 0; t < T; ++t)
                for (int n = 0; n < dh; ++n) {
                    float s = 0.0f;
                    for (int kk = 0; kk < dh; ++kk) { float pr = W[(long)n * dh + kk] * x[(long)t * d + h * dh + kk]; s += pr; }
                    dst[p][(long)t * d + h * dh + n] = s + b[n];
                }
        }
    }
    orc_attention(q.data(), k.data(), v.data(), cat.data(), 1, T, T, H, H, dh, causal, 0.0f, 1);
    const float* Wo = w + (long)H * 3 * (dh * dh + dh);
    linear(cat.data(), Wo, Wo + (long)d * d, T, d, d, out);
}
API long orc_mha_weight_count(int H, int d) { return mha_weight_count(H, d); }
API int orc_mha(const float* weights, const float* x, int T, int H, int d, int causal, float* out) {
    if (d % H) return 2;
    mha_forward(weights, x, T, H, d, causal, out);
    return 0;
}

// ---- a19/a20: encoder_t::forward (mat_transformer_kernel_t.hpp:103-110), post-LN blocks --
// layer = LN(x + MHA(x)) then LN(x + ReLU(W x + b)) (:14-39), LN without eps, gain 1, bias 0;
// rope != 0 applies the reference-mode RoPE to the input first (transformer_base_t::forward, mat_transformer_t.hpp:41-44)
API long orc_encoder_weight_count(int L, int H, int d) { return (long)L * (mha_weight_count(H, d) + (long)d * d + d); }
API int orc_encoder(const float* weights, const float* x, int L, int H, int d, int T, int causal, int rope, float* out) {
    std::vector<float> cur(x, x + (long)T * d), a((long)T * d), tmp((long)T * d);
    if (rope) {
        std::vector<float> table((long)T * (d / 2) * 4);
        orc_rope_table(0, d, 10000.0f, T, table.data());
        orc_rope_apply(cur.data(), tmp.data(), table.data(), d, 1, nullptr, T);
        cur = tmp;
    }
    const long per_layer = mha_weight_count(H, d) + (long)d * d + d;
    for (int l = 0; l < L; ++l) {
        const float* w = weights + l * per_layer;
        mha_forward(w, cur.data(), T, H, d, causal, a.data());
        for (long i = 0; i < (long)T * d; ++i) a[i] = a[i] + cur[i];  // residual_net_t::forward mat_net_t.hpp:326-329: f(x) + x
        orc_layer_norm_rows(a.data(), nullptr, T, d, nullptr, nullptr, 0.0f, cur.data());
        const float* Wf = w + mha_weight_count(H, d);
        linear(cur.data(), Wf, Wf + (long)d * d, T, d, d, a.data());
        for (long i = 0; i < (long)T * d; ++i) a[i] = ((a[i] > 0 ? 1.0f : 0.0f) * a[i]) + cur[i];
        orc_layer_norm_rows(a.data(), nullptr, T, d, nullptr, nullptr, 0.0f, cur.data());
    }
    memcpy(out, cur.data(), sizeof(float) * (long)T * d);
    return 0;
}

// ---- configuration 1: tiny GPT-2-style decoder (pre-LN, GELU FFN, learned positions) -----
// weight order as in ref_harness.cpp: tok_emb[vocab,d], pos_emb[max_pos,d], per layer
// { ln1 g,b; mha; ln2 g,b; W1[ffn,d],b1; W2[d,ffn],b2 }, lnf g,b, W_out[vocab,d], b_out.
API long orc_gpt_weight_count(int L, int d, int H, int ffn, int vocab, int max_pos) {
    long per_layer = 2L * d + mha_weight_count(H, d) + 2L * d + ((long)ffn * d + ffn) + ((long)d * ffn + d);
    return (long)vocab * d + (long)max_pos * d + L * per_layer + 2L * d + ((long)vocab * d + vocab);
}
static void gpt_forward(const float* w, int L, int d, int H, int ffn, int vocab, int max_pos, float eps, const int* ids, int T,
                        float* logits /*[T,vocab]*/) {
    const float* tok = w;
    const float* pos = tok + (long)vocab * d;
    const float* lw = pos + (long)max_pos * d;
    std::vector<float> x((long)T * d), n((long)T * d), a((long)T * d), h((long)T * ffn);
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < d; ++i) x[(long)t * d + i] = tok[(long)ids[t] * d + i] + pos[(long)t * d + i];
    for (int l = 0; l < L; ++l) {
        const float* g1 = lw; const float* b1 = g1 + d; const float* mha = b1 + d;
        const float* g2 = mha + mha_weight_count(H, d); const float* b2 = g2 + d;
        const float* W1 = b2 + d; const float* c1 = W1 + (long)ffn * d;
        const float* W2 = c1 + ffn; const float* c2 = W2 + (long)d * ffn;
        lw = c2 + d;
        orc_layer_norm_rows(x.data(), nullptr, T, d, g1, b1, eps, n.data());
        mha_forward(mha, n.data(), T, H, d, 1, a.data());
        for (long i = 0; i < (long)T * d; ++i) x[i] = a[i] + x[i];
        orc_layer_norm_rows(x.data(), nullptr, T, d, g2, b2, eps, n.data());
        linear(n.data(), W1, c1, T, ffn, d, h.data());
        for (long i = 0; i < (long)T * ffn; ++i) h[i] = gelu_erf(h[i]);
        linear(h.data(), W2, c2, T, d, ffn, a.data());
        for (long i = 0; i < (long)T * d; ++i) x[i] = a[i] + x[i];
    }
    const float* gf = lw; const float* bf = gf + d; const float* Wout = bf + d; const float* bout = Wout + (long)vocab * d;
    orc_layer_norm_rows(x.data(), nullptr, T, d, gf, bf, eps, n.data());
    linear(n.data(), Wout, bout, T, vocab, d, logits);
}
// greedy generation by full-prefix recompute (transformer_test.hpp:227-241): the behaviour a KV cache must reproduce
API int orc_gpt(const float* weights, int L, int d, int H, int ffn, int vocab, int max_pos, float eps, const int* ids, int S,
                float* logits_out, int n_gen, int* gen_out, float* gen_logits_out) {
    std::vector<int> seq(ids, ids + S);
    std::vector<float> logits((long)(S + n_gen) * vocab);
    gpt_forward(weights, L, d, H, ffn, vocab, max_pos, eps, seq.data(), S, logits.data());
    if (logits_out) memcpy(logits_out, logits.data(), sizeof(float) * (long)S * vocab);
    for (int g = 0; g < n_gen; ++g) {
        const float* last = logits.data() + (long)(seq.size() - 1) * vocab;
        int best = 0;
        for (int v = 1; v < vocab; ++v) if (last[v] > last[best]) best = v;
        gen_out[g] = best;
        seq.push_back(best);
        if (g + 1 < n_gen || gen_logits_out) {
            gpt_forward(weights, L, d, H, ffn, vocab, max_pos, eps, seq.data(), (int)seq.size(), logits.data());
            if (gen_logits_out) memcpy(gen_logits_out + (long)g * vocab, logits.data() + (long)(seq.size() - 1) * vocab, sizeof(float) * vocab);
        }
    }
    return 0;
}

// ---- configuration 5 shape: LLaMA-style decoder (not in the reference) -------------------
// h = emb[ids]; per layer: a = RMSNorm(h)*g1; q,k,v = Wq a, Wk a, Wv a (dense, no bias); standard RoPE on q,k per
// head; attention (GQA, causal, scale 1/sqrt(D)); h += Wo attn; m = RMSNorm(h)*g2; h += Wdown (silu(Wgate m) * (Wup m));
// logits = Wlm RMSNorm(h)*gf.  Weights are bf16 values promoted to float; when round_act != 0 the activations are
// rounded to bf16 where the device stores bf16 (after every projection, norm and activation product).
struct llama_cfg { int L, d, Hq, Hkv, D, ffn, vocab; float eps, theta; };
API int orc_llama_forward(const llama_cfg* c, const float* emb, const float* const* layer_w /* per layer: g1,wq,wk,wv,wo,g2,wgate,wup,wdown */,
                          const float* gf, const float* wlm, const int* ids, int T, int round_act, float* logits /*[T,vocab]*/,
                          int last_rows /* > 0: only the logits of the last `last_rows` tokens are computed (rows T-last_rows..T-1 of `logits`) */) {
    const int d = c->d, D = c->D, Hq = c->Hq, Hkv = c->Hkv, ffn = c->ffn;
    auto R = [&](std::vector<float>& v) { if (round_act) for (auto& x : v) x = bf16_round(x); };
    std::vector<float> h((long)T * d), a((long)T * d), q((long)T * Hq * D), k((long)T * Hkv * D), v((long)T * Hkv * D),
        qr((long)T * Hq * D), kr((long)T * Hkv * D), att((long)T * Hq * D), o((long)T * d), g((long)T * ffn), u((long)T * ffn);
    std::vector<float> table((long)T * (D / 2) * 4);
    orc_rope_table(1, D, c->theta, T, table.data());
    for (int t = 0; t < T; ++t) memcpy(&h[(long)t * d], emb + (long)ids[t] * d, sizeof(float) * d);
    for (int l = 0; l < c->L; ++l) {
        const float* const* w = layer_w + (long)l * 9;
        orc_rms_norm_rows(h.data(), T, d, w[0], c->eps, a.data()); R(a);
        linear(a.data(), w[1], nullptr, T, Hq * D, d, q.data()); R(q);
        linear(a.data(), w[2], nullptr, T, Hkv * D, d, k.data()); R(k);
        linear(a.data(), w[3], nullptr, T, Hkv * D, d, v.data()); R(v);
        orc_rope_apply(q.data(), qr.data(), table.data(), D, Hq, nullptr, T); R(qr);
        orc_rope_apply(k.data(), kr.data(), table.data(), D, Hkv, nullptr, T); R(kr);
        orc_attention(qr.data(), kr.data(), v.data(), att.data(), 1, T, T, Hq, Hkv, D, 1, 1.0f / std::sqrt((float)D), 0); R(att);
        linear(att.data(), w[4], nullptr, T, d, Hq * D, o.data());
        for (long i = 0; i < (long)T * d; ++i) h[i] += o[i];
        R(h);
        orc_rms_norm_rows(h.data(), T, d, w[5], c->eps, a.data()); R(a);
        linear(a.data(), w[6], nullptr, T, ffn, d, g.data());
        linear(a.data(), w[7], nullptr, T, ffn, d, u.data());
        for (long i = 0; i < (long)T * ffn; ++i) g[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
        R(g);
        linear(g.data(), w[8], nullptr, T, d, ffn, o.data());
        for (long i = 0; i < (long)T * d; ++i) h[i] += o[i];
        R(h);
    }
    orc_rms_norm_rows(h.data(), T, d, gf, c->eps, a.data()); R(a);
    const int r0 = (last_rows > 0 && last_rows < T) ? T - last_rows : 0;
    linear(a.data() + (long)r0 * d, wlm, nullptr, T - r0, c->vocab, d, logits + (long)r0 * c->vocab);
    return 0;
}

// ---- seeded data: the generator of the product (csrc/common.cuh), restated ----------------
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// dist 0 normal(a, b) from twelve 16-bit uniforms, 1 uniform [a,b), 2 integers [a,b) (written as float)
API int orc_fill(float* dst, long n, uint64_t seed, uint64_t tensor_id, int dist, float a, float b, int to_bf16) {
    const uint64_t key = splitmix64(splitmix64(seed) ^ (tensor_id * 0xD1342543DE82EF95ull));
#pragma omp parallel for
    for (long i = 0; i < n; ++i) {
        float v;
        if (dist == 0) {
            uint32_t acc = 0;
            for (int j = 0; j < 3; ++j) {
                uint64_t hh = splitmix64(key + 3ull * (uint64_t)i + (uint64_t)j);
                acc += (uint32_t)(hh & 0xFFFF) + (uint32_t)((hh >> 16) & 0xFFFF) + (uint32_t)((hh >> 32) & 0xFFFF) + (uint32_t)((hh >> 48) & 0xFFFF);
            }
            float dd = (float)acc - 393210.0f;
            float nn = dd * (1.0f / 65536.0f);
            float p = b * nn;
            v = a + p;
        } else if (dist == 1) {
            uint64_t hh = splitmix64(key + (uint64_t)i);
            float uu = (float)(uint32_t)(hh >> 40) * (1.0f / 16777216.0f);
            float w = b - a;
            float p = w * uu;
            v = a + p;
        } else {
            uint64_t hh = splitmix64(key + (uint64_t)i);
            uint64_t span = (uint64_t)(uint32_t)((int32_t)b - (int32_t)a);
            v = (float)((int32_t)a + (int32_t)(((hh >> 32) * span) >> 32));
        }
        dst[i] = to_bf16 ? bf16_round(v) : v;
    }
    return 0;
}
