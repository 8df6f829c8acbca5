// TEST INFRASTRUCTURE, not product code.
//
// C entry points over the UNMODIFIED jasmine headers (included by path with
// -I<reference root>; nothing of the reference is copied here).  Built by
// oracle/Makefile into oracle/_ref/libjasmine_ref.so and used only to check the
// restatement in jasmine_oracle.cpp, to generate tests/golden/ and as the
// "reference" CPU baseline.  Matrices cross this boundary as dense row-major
// float arrays.
//
// Seeded weights enter the reference's nets through a user specialisation of
// init_t<tag> (mat_init_t.hpp:10-118): init_weight<inject_t>() walks every
// weight in a fixed order and copies the next values of a flat array into it.
// Nets are built with their direct constructors and d_head >= 2 only (the
// default-constructed wrappers read out of bounds, mat_mha_t.hpp:36-38).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <vector>

// include order of the reference's main.cpp:1-9 (the headers depend on it)
#include "mat_t.hpp"
#include "mat_express_t.hpp"
#include "mat_view_t.hpp"
#include "mat_net_t.hpp"
#include "mat_init_t.hpp"
#include "mat_mha_t.hpp"
#include "mat_transformer_kernel_t.hpp"
#include "mat_RoPE_t.hpp"
#include "mat_transformer_t.hpp"

using F = float;
using M = mat_t<F>;

// ---- weight injection ---------------------------------------------------------
static thread_local const float* g_cursor = nullptr;
static thread_local long g_taken = 0;
struct inject_t;
template <>
struct init_t<inject_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) {
        for (int i = 0; i < m.row_num(); ++i)
            for (int j = 0; j < m.col_num(); ++j) {
                m(i, j) = *g_cursor++;
                ++g_taken;
            }
    }
};

static M load(const float* p, int R, int C) {
    M m(R, C);
    for (int i = 0; i < R; ++i)
        for (int j = 0; j < C; ++j) m(i, j) = p[(long)i * C + j];
    return m;
}
template <typename mat_type>
static void store(const mat_type& m, float* out) {
    const int R = m.row_num(), C = m.col_num();
    for (int i = 0; i < R; ++i)
        for (int j = 0; j < C; ++j) out[(long)i * C + j] = static_cast<float>(m(i, j));
}

#define GUARD(...)                     \
    try {                              \
        __VA_ARGS__;                   \
        return 0;                      \
    } catch (const std::invalid_argument&) { \
        return 1;                      \
    } catch (const std::runtime_error&) {    \
        return 2;                      \
    } catch (...) {                    \
        return 9;                      \
    }

// GELU / LayerNorm-with-eps / RMSNorm do not exist in the reference: they are
// composed here from its primitives so that the arithmetic runs through its code.
template <typename input_type>
struct gelu_net_t {
    using val_type = typename input_type::ele_type;
    mat_t<val_type> forward(const input_type& x) {
        mat_t<val_type> y(x.row_num(), x.col_num());
        for (int i = 0; i < x.row_num(); ++i)
            for (int j = 0; j < x.col_num(); ++j) {
                val_type v = x(i, j);
                y(i, j) = val_type(0.5) * v * (val_type(1) + std::erf(v * val_type(0.70710678118654752440)));
            }
        return y;
    }
    template <typename> void init_weight() {}
    void step() {}
    std::string net_type(int const& = 0) const { return "gelu_net_t"; }
};

// formula of layer_norm_net_t::forward (mat_net_t.hpp:209-225) with eps under the
// square root and explicit gain/bias [d,1]; normalises each column.
template <typename input_type, template <typename> class updator_type>
struct layer_norm_eps_net_t {
    using val_type = typename input_type::ele_type;
    mat_t<val_type> m_gama, m_beta;
    val_type m_eps = 0;
    mat_t<val_type> forward(const input_type& input) {
        mat_t<val_type> mean = vmean(input);
        auto delta = input - mean;
        mat_t<val_type> var = vmean(pow(delta.clone(), 2.0));
        mat_t<val_type> stdv = sqrt((var + m_eps).clone());
        mat_t<val_type> hx = delta / stdv;
        return (m_gama * hx + m_beta).clone();
    }
    template <typename init_type>
    void init_weight() {
        init_matrix<init_type>(m_gama);
        init_matrix<init_type>(m_beta);
    }
    void step() {}
    std::string net_type(int const& = 0) const { return "layer_norm_eps_net_t"; }
};

extern "C" {

// ---- a3/a4: lazy elementwise nodes, materialised by clone() ----------------------
// B is [Br,Bc] and broadcasts by modulo.  op: 0 + 1 - 2 * 3 / 4 > 5 < 6 exp(A) 7 sigmoid(A)
// 8 A*s+B 9 (A>0)*A 10 pow(A,s) 11 sqrt(A) 12 A+=B 13 ((A+B-A)*B/A) 14 A*s 15 A+s
int ref_expr(int op, const float* A, int R, int C, const float* B, int Br, int Bc, float s, float* out) {
    GUARD({
        M a = load(A, R, C);
        M b = B ? load(B, Br, Bc) : M(1, 1);
        M y;
        switch (op) {
            case 0: y = (a + b).clone(); break;
            case 1: y = (a - b).clone(); break;
            case 2: y = (a * b).clone(); break;
            case 3: y = (a / b).clone(); break;
            case 4: y = (a > b).clone(); break;
            case 5: y = (a < b).clone(); break;
            case 6: y = exp(a).clone(); break;
            case 7: y = sigmoid(a).clone(); break;
            case 8: y = (a * s + b).clone(); break;
            case 9: y = ((a > 0) * a).clone(); break;
            case 10: y = pow(a, (double)s); break;
            case 11: y = sqrt(a); break;
            case 12: a += b; y = a; break;
            case 13: y = ((a + b - a) * b / a).clone(); break;
            case 14: y = (a * s).clone(); break;
            case 15: y = (a + s).clone(); break;
            default: throw std::invalid_argument("op");
        }
        store(y, out);
    })
}

// ---- a6: eager reductions.  kind: 0 hsum 1 hmax 2 hmean 3 vsum 4 vmean 5 sum 6 mean 7 max
int ref_reduce(int kind, const float* A, int R, int C, float* out) {
    GUARD({
        M a = load(A, R, C);
        switch (kind) {
            case 0: store(hsum(a), out); break;
            case 1: store(hmax(a), out); break;
            case 2: store(hmean(a), out); break;
            case 3: store(vsum(a), out); break;
            case 4: store(vmean(a), out); break;
            case 5: out[0] = sum(a); break;
            case 6: out[0] = mean(a); break;
            case 7: out[0] = max(a); break;
            default: throw std::invalid_argument("kind");
        }
    })
}

// ---- a7 / a5: hsoftmax(A*s + B) (B may be null: hsoftmax(A)); whole-matrix softmax(A)
int ref_hsoftmax(const float* A, const float* B, float s, int R, int C, float* out) {
    GUARD({
        M a = load(A, R, C);
        if (B) {
            M b = load(B, R, C);
            store(hsoftmax(a * s + b), out);
        } else {
            store(hsoftmax(a), out);
        }
    })
}
int ref_softmax_full(const float* A, int R, int C, float* out) {
    GUARD({
        M a = load(A, R, C);
        store(softmax(a).clone(), out);
    })
}

// ---- a11: layer_norm_net_t::forward on x:[d,S] (each column normalised, no eps, gain 1, bias 0)
int ref_layer_norm(const float* x, int d, int S, float* out) {
    GUARD({
        layer_norm_net_t<M, sgd_t> ln;
        store(ln.forward(load(x, d, S)), out);
    })
}
// same formula with eps, gain[d], bias[d] composed from the reference's primitives; x may be the sum x + x2
int ref_layer_norm_eps(const float* x, const float* x2, int d, int S, const float* gain, const float* bias, float eps,
                       float* out) {
    GUARD({
        layer_norm_eps_net_t<M, sgd_t> ln;
        ln.m_gama = load(gain, d, 1);
        ln.m_beta = load(bias, d, 1);
        ln.m_eps = eps;
        M in = load(x, d, S);
        if (x2) in = (in + load(x2, d, S)).clone();
        store(ln.forward(in), out);
    })
}
// RMSNorm of each column from the reference's primitives: gain * x / sqrt(vmean(pow(x,2)) + eps)
int ref_rms_norm(const float* x, int d, int S, const float* gain, float eps, float* out) {
    GUARD({
        M in = load(x, d, S);
        M g = load(gain, d, 1);
        M ms = vmean(pow(in, 2.0));
        M r = sqrt((ms + eps).clone());
        M hx = in / r;
        store((g * hx).clone(), out);
    })
}

// ---- a8 / a9: dot and weight_net_t::forward (Y = W.X + b) -------------------------
int ref_dot(const float* A, int Mr, int K, const float* B, int K2, int N, float* out) {
    GUARD({
        M a = load(A, Mr, K);
        M b = load(B, K2, N);
        store(a.dot(b).clone(), out);
    })
}
// weights: W[out,in] then b[out]
int ref_weight_net(const float* weights, int in, int out_dim, const float* X, int S, float* Y) {
    GUARD({
        weight_net_t<M, sgd_t> net(in, out_dim);
        g_cursor = weights;
        net.init_weight<inject_t>();
        store(net.forward(load(X, in, S)), Y);
    })
}
// a10: relu_net_t / sigmoid_net_t forward
int ref_activation(int kind, const float* X, int R, int C, float* Y) {
    GUARD({
        M x = load(X, R, C);
        if (kind == 0) {
            relu_net_t<M> net;
            store(net.forward(x), Y);
        } else {
            sigmoid_net_t<M> net;
            store(net.forward(x), Y);
        }
    })
}

// ---- a15-a17: mat_mha_t::forward.  weights in init_weight order: per head q(W,b) k(W,b) v(W,b), then out proj (W,b)
long ref_mha_weight_count(int H, int d_model) {
    long dh = d_model / H;
    return (long)H * 3 * (dh * dh + dh) + ((long)d_model * d_model + d_model);
}
int ref_mha(const float* weights, const float* x, int H, int d_model, int S, int mask, float* out) {
    GUARD({
        mat_mha_t<M, sgd_t> mha(H, d_model, mask != 0, S);
        g_cursor = weights;
        mha.init_weight<inject_t>();
        store(mha.forward(load(x, d_model, S)), out);
    })
}

// ---- a18: RoPE_net_t::forward on x:[d,S] -------------------------------------------
int ref_rope(const float* x, int d, int S, float* out) {
    GUARD({
        RoPE_net_t<M> rope(d);
        store(rope.forward(load(x, d, S)), out);
    })
}

// ---- a19/a20: encoder_t stack (post-LN blocks), optionally causal and with RoPE on the input
// weights per layer in init_weight order: mha (as above), [mha norm: nothing before the first forward],
// ffn W[d,d], b[d].
long ref_encoder_weight_count(int L, int H, int d) { return (long)L * (ref_mha_weight_count(H, d) + (long)d * d + d); }
int ref_encoder(const float* weights, const float* x, int L, int H, int d, int S, int causal, int rope, float* out) {
    GUARD({
        encoder_t<F, sgd_t> enc(L, H, d, S);
        if (causal)
            for (int i = 0; i < L; ++i) enc.get_mha(i).set_param(H, d, true, S);
        g_cursor = weights;
        enc.init_weight<inject_t>();
        M in = load(x, d, S);
        if (rope) {
            RoPE_net_t<M> r(d);
            in = r.forward(in);
        }
        store(enc.forward(in), out);
    })
}

// ---- configuration 1: tiny GPT-2-style decoder composed from the reference's nets ---
// pre-LN blocks: x + MHA(LN(x)), x + W2.GELU(W1.LN(x)); learned positional embedding; final LN; logits.
// weight order: tok_emb[vocab,d], pos_emb[max_pos,d], per layer { ln1 g,b; mha; ln2 g,b; W1,b1; W2,b2 }, lnf g,b, W_out[vocab,d], b_out
using ln_t = layer_norm_eps_net_t<M, sgd_t>;
using attn_block_t = residual_net_t<complex_net_t<ln_t, mat_mha_t<M, sgd_t>>>;
using ffn_block_t = residual_net_t<complex_net_t<ln_t, weight_net_t<M, sgd_t>, gelu_net_t<M>, weight_net_t<M, sgd_t>>>;

long ref_gpt_weight_count(int L, int d, int H, int ffn, int vocab, int max_pos) {
    long per_layer = 2L * d + ref_mha_weight_count(H, d) + 2L * d + ((long)ffn * d + ffn) + ((long)d * ffn + d);
    return (long)vocab * d + (long)max_pos * d + L * per_layer + 2L * d + ((long)vocab * d + vocab);
}

struct gpt_t {
    int L, d, H, ffn, vocab, max_pos;
    M tok, pos;
    std::vector<attn_block_t> attn;
    std::vector<ffn_block_t> mlp;
    ln_t lnf;
    weight_net_t<M, sgd_t> head;
    gpt_t(int L_, int d_, int H_, int ffn_, int vocab_, int max_pos_, float eps, const float* w)
        : L(L_), d(d_), H(H_), ffn(ffn_), vocab(vocab_), max_pos(max_pos_), attn(L_), mlp(L_), head(d_, vocab_) {
        g_cursor = w;
        tok = M(vocab, d);
        pos = M(max_pos, d);
        init_matrix<inject_t>(tok);
        init_matrix<inject_t>(pos);
        for (int l = 0; l < L; ++l) {
            auto& ln1 = attn[l].base_net().template get<0>();
            ln1.m_gama = M(d, 1); ln1.m_beta = M(d, 1); ln1.m_eps = eps;
            attn[l].base_net().template get<1>().set_param(H, d, true, 1);
            attn[l].template init_weight<inject_t>();
            auto& ln2 = mlp[l].base_net().template get<0>();
            ln2.m_gama = M(d, 1); ln2.m_beta = M(d, 1); ln2.m_eps = eps;
            mlp[l].base_net().reinit(std::vector<int>{d, ffn, d});
            mlp[l].template init_weight<inject_t>();
        }
        lnf.m_gama = M(d, 1); lnf.m_beta = M(d, 1); lnf.m_eps = eps;
        lnf.init_weight<inject_t>();
        head.init_weight<inject_t>();
    }
    // ids[S] -> logits [vocab, S] (reference orientation: features x tokens)
    M forward(const int* ids, int S) {
        M x(d, S);
        for (int t = 0; t < S; ++t)
            for (int i = 0; i < d; ++i) x(i, t) = tok(ids[t], i) + pos(t, i);
        for (int l = 0; l < L; ++l) {
            x = attn[l].forward(x);
            x = mlp[l].forward(x);
        }
        return head.forward(lnf.forward(x));
    }
};

// logits_out: [S, vocab] (token-major); gen_out: n_gen greedy tokens by full-prefix recompute
// (the generation loop of transformer_test.hpp:227-241 applied to token ids).
int ref_gpt(const float* weights, int L, int d, int H, int ffn, int vocab, int max_pos, float eps, const int* ids,
            int S, float* logits_out, int n_gen, int* gen_out, float* gen_logits_out) {
    GUARD({
        gpt_t net(L, d, H, ffn, vocab, max_pos, eps, weights);
        std::vector<int> seq(ids, ids + S);
        M logits = net.forward(seq.data(), S);
        if (logits_out)
            for (int t = 0; t < S; ++t)
                for (int v = 0; v < vocab; ++v) logits_out[(long)t * vocab + v] = logits(v, t);
        for (int g = 0; g < n_gen; ++g) {
            auto last = logits.back_col();
            int best = 0;
            for (int v = 1; v < vocab; ++v)
                if (last(v, 0) > last(best, 0)) best = v;
            gen_out[g] = best;
            seq.push_back(best);
            if (g + 1 < n_gen || gen_logits_out) {
                logits = net.forward(seq.data(), (int)seq.size());
                if (gen_logits_out)
                    for (int v = 0; v < vocab; ++v) gen_logits_out[(long)g * vocab + v] = logits(v, (int)seq.size() - 1);
            }
        }
    })
}

// ---- a21: causal-prefix property of test_sequence_mha (transformer_test.hpp:246-282):
// returns the largest |difference| between column 0..S1-1 of a causal mha forward on the
// first S1 columns and on all S2 columns.
int ref_prefix_property(const float* weights, const float* x, int H, int d_model, int S1, int S2, float* max_diff) {
    GUARD({
        mat_mha_t<M, sgd_t> mha(H, d_model, true, S2);
        g_cursor = weights;
        mha.init_weight<inject_t>();
        M full = load(x, d_model, S2);
        M part(d_model, S1);
        for (int i = 0; i < d_model; ++i)
            for (int j = 0; j < S1; ++j) part(i, j) = full(i, j);
        M y1 = mha.forward(part);
        M y2 = mha.forward(full);
        float md = 0;
        for (int i = 0; i < d_model; ++i)
            for (int j = 0; j < S1; ++j) md = std::max(md, std::fabs(y1(i, j) - y2(i, j)));
        *max_diff = md;
    })
}

}  // extern "C"
