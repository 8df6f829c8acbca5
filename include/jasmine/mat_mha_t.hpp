// Attention of the jasmine API, forward halves (reference: mat_mha_t.hpp): mat_head_gen_t (one head),
// vconcat / vsplit, mat_mha_t (multi-head self and cross attention) and mat_mhca_t.
//
// Inputs and outputs are [d_model, seq_len] like in the reference.  Internally q, k and v are produced
// token-major ([seq_len, d_model], a head = a column slice) straight from the per-head projections, which are
// d_head x d_head on the head's own row slice of the input (the reference's block-diagonal projections,
// mat_mha_t.hpp:199-215, 278-282); one attention kernel then covers all heads and the output projection
// reads the result through a transposed window.  No split / concat copies are made.
#ifndef JASMINE_B200_MAT_MHA_T_HPP_
#define JASMINE_B200_MAT_MHA_T_HPP_
#include <cmath>
#include <limits>
#include <stdexcept>
#include <vector>

#include "mat_express_t.hpp"
#include "mat_net_t.hpp"
#include "mat_t.hpp"
#include "mat_view_t.hpp"

namespace jsm_attn {

// rows [r0, r0+n) of a [features, tokens] window, seen token-major: [tokens, n]
inline jsm_mat token_major_rows(const jsm_mat& x, int r0, int n) {
    jsm_mat t = x;
    t.data = static_cast<char*>(x.data) + (int64_t)r0 * x.row_stride * (int64_t)sizeof(float);
    t.rows = x.cols; t.cols = n;
    t.row_stride = x.col_stride; t.col_stride = x.row_stride;
    return t;
}
inline jsm_mat columns(const jsm_mat& x, int c0, int n) {
    jsm_mat t = x;
    t.data = static_cast<char*>(x.data) + (int64_t)c0 * x.col_stride * (int64_t)sizeof(float);
    t.cols = n;
    return t;
}
// rows [r0, r0+n) of a matrix window
inline jsm_mat rows(const jsm_mat& x, int r0, int n) {
    jsm_mat t = x;
    t.data = static_cast<char*>(x.data) + (int64_t)r0 * x.row_stride * (int64_t)sizeof(float);
    t.rows = n;
    return t;
}
inline jsm_mat transposed(const jsm_mat& x) {
    jsm_mat t = x;
    t.rows = x.cols; t.cols = x.rows; t.row_stride = x.col_stride; t.col_stride = x.row_stride;
    return t;
}
// softmax(mask(Q K^T * scale)) V over token-major fp32 q [Sq, H*dh], k and v (the first Sk rows of their buffers), all
// contiguous rows of H*dh floats.  fp32 kernel with the reference's arithmetic (mat_mha_t.hpp:53-71), or - when the
// caller opted in (jsm_rt::attention_bf16) and the heads are 128 wide - the tensor-core flash kernel on bf16 copies.
inline void attention(const float* q, const float* k, const float* v, float* out, int Sq, int Sk, int H, int dh, bool mask) {
    const float scale = 1.0f / std::sqrt((float)dh);
    if (!(jsm_rt::attention_bf16() && dh == 128)) {
        jsm_rt::check(jsm_attn_prefill(q, k, v, out, JSM_F32, 1, Sq, Sk, H, H, dh, mask ? 1 : 0, scale, nullptr, 1, jsm_rt::stream()));
        return;
    }
    const size_t nq = (size_t)Sq * H * dh, nk = (size_t)Sk * H * dh;
    jsm_rt::device_buffer qb(nq * 2), kb(nk * 2), vb(nk * 2), ob(nq * 2);
    jsm_rt::check(jsm_convert(qb.p, JSM_BF16, q, JSM_F32, nq, jsm_rt::stream()));
    jsm_rt::check(jsm_convert(kb.p, JSM_BF16, k, JSM_F32, nk, jsm_rt::stream()));
    jsm_rt::check(jsm_convert(vb.p, JSM_BF16, v, JSM_F32, nk, jsm_rt::stream()));
    jsm_rt::check(jsm_attn_prefill(qb.p, kb.p, vb.p, ob.p, JSM_BF16, 1, Sq, Sk, H, H, dh, mask ? 1 : 0, scale, nullptr, 2, jsm_rt::stream()));
    jsm_rt::check(jsm_convert(out, JSM_F32, ob.p, JSM_BF16, nq, jsm_rt::stream()));
    jsm_rt::check(jsm_stream_sync(jsm_rt::stream()));  // the temporaries are released on return
}

// Y[tokens, out] = X_tm . W^T + b^T for a weight_net_t: the same k-ascending sums as W . X + b
template <typename net>
void project(const net& w, const jsm_mat& x_tm, const jsm_mat& out) {
    jsm_mat W = transposed(w.jsm_weight().jsm_device());
    jsm_mat B = transposed(w.jsm_bias().jsm_device());
    jsm_rt::check(jsm_dot_f32(x_tm, W, &B, 0, nullptr, out, jsm_rt::stream()));
}

}  // namespace jsm_attn

template <typename input_type, template <typename> class updator_type>
class mat_head_gen_t {
public:
    using val_type = typename input_type::ele_type;
    using ele_type = typename input_type::ele_type;

private:
    using ffn_type = weight_net_t<input_type, updator_type>;
    ffn_type m_q_net, m_k_net, m_v_net;
    bool m_mask;
    int m_d;

public:
    mat_head_gen_t(int const& d_model = 1, bool const& mask = false, int const& = 1)
        : m_q_net(d_model, d_model), m_k_net(d_model, d_model), m_v_net(d_model, d_model), m_mask(mask), m_d(d_model) {}

    void set_param(int const& d_model, bool const& mask = false, int const& = 1) {
        m_q_net.reinit(std::vector<int>{d_model, d_model});
        m_k_net.reinit(std::vector<int>{d_model, d_model});
        m_v_net.reinit(std::vector<int>{d_model, d_model});
        m_mask = mask;
        m_d = d_model;
    }
    bool mask() const { return m_mask; }
    const ffn_type& q_net() const { return m_q_net; }
    const ffn_type& k_net() const { return m_k_net; }
    const ffn_type& v_net() const { return m_v_net; }
    ffn_type& q_net() { return m_q_net; }
    ffn_type& k_net() { return m_k_net; }
    ffn_type& v_net() { return m_v_net; }

    // softmax(mask(Q^T K / sqrt(d))) applied to V (reference: mat_mha_t.hpp:45-74); input: [d, S]
    template <typename any_input>
    mat_t<val_type> forward(const any_input& input) { return forward(input, input, m_mask); }
    // cross attention: queries from the first argument, keys and values from the second (:76-90), no mask
    template <typename any_q, typename any_kv>
    mat_t<val_type> forward(const any_q& decoder_input, const any_kv& encoder_input) { return forward(decoder_input, encoder_input, false); }

    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        m_q_net.set_updator(args...); m_k_net.set_updator(args...); m_v_net.set_updator(args...);
    }
    template <typename init_type>
    void init_weight() {
        m_q_net.template init_weight<init_type>();
        m_k_net.template init_weight<init_type>();
        m_v_net.template init_weight<init_type>();
    }
    std::string net_type(int const& indent = 0) const { return print_indent(indent) + "mat_head_gen_t"; }
    void step() { m_q_net.step(); m_k_net.step(); m_v_net.step(); }
    void save(std::ostream& os) const { m_q_net.save(os); m_k_net.save(os); m_v_net.save(os); }
    void load(std::istream& is) { m_q_net.load(is); m_k_net.load(is); m_v_net.load(is); }

private:
    template <typename any_q, typename any_kv>
    mat_t<val_type> forward(const any_q& xq, const any_kv& xkv, bool mask) {
        std::vector<std::shared_ptr<void>> keep;
        const jsm_mat Xq = jsm_expr::operand(xq, keep), Xkv = jsm_expr::operand(xkv, keep);
        const int Sq = Xq.cols, Sk = Xkv.cols, d = m_d;
        if (Xq.rows != d || Xkv.rows != d) throw std::invalid_argument("mat_dot_t: inner dimensions do not match for dot product");
        mat_t<val_type> q(Sq, d), k(Sk, d), v(Sk, d), o(Sq, d);
        jsm_attn::project(m_q_net, jsm_attn::token_major_rows(Xq, 0, d), q.jsm_device_out());
        jsm_attn::project(m_k_net, jsm_attn::token_major_rows(Xkv, 0, d), k.jsm_device_out());
        jsm_attn::project(m_v_net, jsm_attn::token_major_rows(Xkv, 0, d), v.jsm_device_out());
        jsm_rt::check(jsm_attn_prefill(q.jsm_device().data, k.jsm_device().data, v.jsm_device().data, o.jsm_device_out().data, JSM_F32,
                                       1, Sq, Sk, 1, 1, d, mask ? 1 : 0, 1.0f / std::sqrt((float)d), nullptr, 1, jsm_rt::stream()));
        return o.t().clone();  // back to [d, S]
    }
};

// row-wise concatenation (reference: mat_mha_t.hpp:164-196)
template <typename val_type>
mat_t<val_type> vconcat(const std::vector<mat_t<val_type>>& mats) {
    if (mats.empty()) throw std::runtime_error("Cannot concatenate empty vector");
    const int cols = mats[0].col_num();
    int total_rows = 0;
    for (const auto& m : mats) {
        if (m.col_num() != cols) throw std::runtime_error("All matrices must have the same number of columns");
        total_rows += m.row_num();
    }
    mat_t<val_type> result(total_rows, cols);
    int row_offset = 0;
    for (const auto& m : mats) {
        if (m.row_num() > 0) result.view(row_offset, 0, m.row_num(), cols).assign(m);
        row_offset += m.row_num();
    }
    return result;
}

// equal row slices as views (reference: mat_mha_t.hpp:199-215)
template <typename mat_type>
std::vector<mat_view_t<mat_type>> vsplit(mat_type& mat, int num_splits) {
    if (num_splits <= 0 || mat.row_num() % num_splits != 0) throw std::runtime_error("Invalid number of splits or row count mismatch");
    const int rows = mat.row_num() / num_splits;
    std::vector<mat_view_t<mat_type>> views;
    for (int i = 0; i < num_splits; ++i) views.emplace_back(mat, i * rows, 0, rows, mat.col_num());
    return views;
}

template <typename input_type, template <typename> class updator_type>
class mat_mha_t {
public:
    using val_type = typename input_type::ele_type;

private:
    std::vector<mat_head_gen_t<input_type, updator_type>> m_heads;
    weight_net_t<mat_t<val_type>, updator_type> m_output_proj;
    int m_num_heads, m_d_model, m_d_head;
    bool m_mask;
    // Keys and values of the positions seen so far, token-major [capacity, d_model], resident on the device.
    // Self attention: grown by forward_cached.  Cross attention: computed once from the encoder output (set_memory).
    mat_t<val_type> m_k_cache, m_v_cache;
    int m_cached = 0;
    mat_t<val_type> m_train_input;  // the last self-attention forward's input, for backward

    void reserve_cache(int positions) {
        if (positions <= m_k_cache.row_num() && m_k_cache.col_num() == m_d_model) return;
        const int cap = std::max(positions, std::max(64, 2 * m_k_cache.row_num()));
        mat_t<val_type> k(cap, m_d_model), v(cap, m_d_model);
        if (m_cached > 0) {
            k.view(0, 0, m_cached, m_d_model).assign(m_k_cache.view(0, 0, m_cached, m_d_model));
            v.view(0, 0, m_cached, m_d_model).assign(m_v_cache.view(0, 0, m_cached, m_d_model));
        }
        m_k_cache = std::move(k);
        m_v_cache = std::move(v);
    }
    // keys and values of the columns of x (token-major rows) into rows [at, at + columns) of the cache
    void project_kv(const jsm_mat& X, int at) {
        const jsm_mat K = jsm_attn::rows(m_k_cache.jsm_device_inout(), at, X.cols), V = jsm_attn::rows(m_v_cache.jsm_device_inout(), at, X.cols);
        for (int h = 0; h < m_num_heads; ++h) {
            jsm_attn::project(m_heads[h].k_net(), jsm_attn::token_major_rows(X, h * m_d_head, m_d_head), jsm_attn::columns(K, h * m_d_head, m_d_head));
            jsm_attn::project(m_heads[h].v_net(), jsm_attn::token_major_rows(X, h * m_d_head, m_d_head), jsm_attn::columns(V, h * m_d_head, m_d_head));
        }
    }
    // queries of the columns of x against the first n_keys cached positions, then the output projection
    mat_t<val_type> attend_cached(const jsm_mat& Xq, int n_keys, bool mask) {
        const int Sq = Xq.cols, d = m_d_model, dh = m_d_head;
        mat_t<val_type> q(Sq, d), att(Sq, d);
        const jsm_mat Q = q.jsm_device_out();
        for (int h = 0; h < m_num_heads; ++h)
            jsm_attn::project(m_heads[h].q_net(), jsm_attn::token_major_rows(Xq, h * dh, dh), jsm_attn::columns(Q, h * dh, dh));
        jsm_attn::attention(static_cast<const float*>(Q.data), static_cast<const float*>(m_k_cache.jsm_device().data),
                            static_cast<const float*>(m_v_cache.jsm_device().data), static_cast<float*>(att.jsm_device_out().data), Sq, n_keys,
                            m_num_heads, dh, mask);
        mat_t<val_type> out(d, Sq);
        jsm_mat Wo = m_output_proj.jsm_weight().jsm_device(), Bo = m_output_proj.jsm_bias().jsm_device();
        jsm_rt::check(jsm_dot_f32(Wo, jsm_attn::transposed(att.jsm_device()), &Bo, 0, nullptr, out.jsm_device_out(), jsm_rt::stream()));
        return out;
    }

public:
    mat_mha_t(int num_heads = 1, int d_model = 1, bool mask = false, int seq_len = 1)
        : m_output_proj(d_model, d_model), m_num_heads(num_heads), m_d_model(d_model), m_d_head(d_model / num_heads), m_mask(mask) {
        if (d_model % num_heads != 0) throw std::runtime_error("d_model must be divisible by num_heads");
        for (int i = 0; i < num_heads; ++i) m_heads.emplace_back(m_d_head, mask, seq_len);
    }

    void set_param(int num_heads, int d_model, bool mask = false, int seq_len = 1) {
        if (d_model % num_heads != 0) throw std::runtime_error("d_model must be divisible by num_heads");
        m_num_heads = num_heads; m_d_model = d_model; m_d_head = d_model / num_heads; m_mask = mask;
        m_heads.resize(num_heads);
        for (auto& h : m_heads) h.set_param(m_d_head, mask, seq_len);
        m_output_proj.reinit(std::vector<int>{d_model, d_model});
    }

    // self attention (reference: mat_mha_t.hpp:265-291)
    mat_t<val_type> forward(const input_type& input) {
        if (input.row_num() != m_d_model) throw std::runtime_error("Input row dimension must match d_model");
        m_train_input = input;
        return attend(input, input, m_mask, /*remember=*/true);
    }
    // Training step of self attention (reference: mat_mha_t.hpp:92-117 per head, :324-346 for the layer).  The forward
    // kernel keeps no probabilities, so each head's q, k, v and softmax are rebuilt here from the stored input with the
    // matrix operations of the API (the head's weight nets thereby remember their inputs for their own backward):
    //   dV = delta . P, dP = delta^T . V, dS = P * (dP - rowsum(P * dP)) with the masked entries zeroed,
    //   dQ = K . dS^T / sqrt(d_head), dK = Q . dS / sqrt(d_head), input gradient = sum of the three nets' backward.
    mat_t<val_type> backward(const input_type& delta) {
        if (!m_train_input.valid()) throw std::runtime_error("backward without a preceding forward");
        mat_t<val_type> delta_concat = m_output_proj.backward(delta);
        const int S = m_train_input.col_num(), dh = m_d_head;
        const val_type root = static_cast<val_type>(std::sqrt((double)dh));
        mat_t<val_type> keep(S, S), drop(S, S);  // causal mask as factors: 1 where key <= query; additive: -inf elsewhere
        if (m_mask) {
            for (int i = 0; i < S; ++i)
                for (int j = 0; j < S; ++j) {
                    keep(i, j) = j <= i ? val_type(1) : val_type(0);
                    drop(i, j) = j <= i ? val_type(0) : -std::numeric_limits<val_type>::infinity();
                }
        }
        mat_t<val_type> total(delta.row_num(), delta.col_num());
        for (int h = 0; h < m_num_heads; ++h) {
            mat_t<val_type> x_h = m_train_input.view(h * dh, 0, dh, S).clone();
            mat_t<val_type> d_h = delta_concat.view(h * dh, 0, dh, S).clone();
            mat_t<val_type> q = m_heads[h].q_net().forward(x_h), k = m_heads[h].k_net().forward(x_h), v = m_heads[h].v_net().forward(x_h);
            mat_t<val_type> scores = (q.t().dot(k) / root).clone();
            if (m_mask) scores = (scores + drop).clone();
            mat_t<val_type> P = hsoftmax(scores);
            mat_t<val_type> d_v = d_h.dot(P).clone();
            mat_t<val_type> d_P = d_h.t().dot(v).clone();
            mat_t<val_type> row_dot = hsum(P * d_P);
            mat_t<val_type> d_S = (P * (d_P - row_dot)).clone();
            if (m_mask) d_S = (d_S * keep).clone();
            mat_t<val_type> d_q = (k.dot(d_S.t()) / root).clone();
            mat_t<val_type> d_k = (q.dot(d_S) / root).clone();
            mat_t<val_type> gq = m_heads[h].q_net().backward(d_q), gk = m_heads[h].k_net().backward(d_k), gv = m_heads[h].v_net().backward(d_v);
            total.view(h * dh, 0, dh, S).assign((gq + gk + gv).clone());
        }
        return total;
    }
    // cross attention (reference: :293-322)
    mat_t<val_type> forward(const input_type& input, const input_type& encoder_input) {
        if (input.row_num() != m_d_model) throw std::runtime_error("Input row dimension must match d_model");
        if (encoder_input.row_num() != m_d_model) throw std::runtime_error("Encoder input row dimension must match d_model");
        return attend(input, encoder_input, false);
    }

    // ---- generation against cached keys and values --------------------------------------------------------------
    // The reference generates by recomputing the whole prefix for every new position (transformer_test.hpp:227-241).
    // forward_cached(x_new) returns what forward(prefix + x_new) returns in its LAST x_new.col_num() columns (the causal
    // prefix property the reference demonstrates, transformer_test.hpp:246-282), but projects only the new columns and
    // attends over the cached keys and values of the earlier ones.  Needs a masked (causal) attention layer.
    void reset_cache() { m_cached = 0; }
    int cached_positions() const { return m_cached; }
    mat_t<val_type> forward_cached(const input_type& x_new) {
        if (x_new.row_num() != m_d_model) throw std::runtime_error("Input row dimension must match d_model");
        if (!m_mask) throw std::runtime_error("forward_cached needs a masked (causal) attention layer");
        const jsm_mat X = x_new.jsm_device();
        reserve_cache(m_cached + X.cols);
        project_kv(X, m_cached);
        m_cached += X.cols;
        return attend_cached(X, m_cached, true);  // query i of the new block sees keys 0 .. m_cached - X.cols + i
    }
    // Cross attention against a fixed memory (the encoder output): its keys and values are projected ONCE here instead
    // of at every decoding step (reference: :293-322 projects them in every forward).
    void set_memory(const input_type& encoder_input) {
        if (encoder_input.row_num() != m_d_model) throw std::runtime_error("Encoder input row dimension must match d_model");
        m_cached = 0;
        const jsm_mat X = encoder_input.jsm_device();
        reserve_cache(X.cols);
        project_kv(X, 0);
        m_cached = X.cols;
    }
    mat_t<val_type> forward_memory(const input_type& input) {
        if (input.row_num() != m_d_model) throw std::runtime_error("Input row dimension must match d_model");
        if (m_cached == 0) throw std::runtime_error("Encoder output not set for cross attention");
        return attend_cached(input.jsm_device(), m_cached, false);
    }

    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        for (auto& h : m_heads) h.set_updator(args...);
        m_output_proj.set_updator(args...);
    }
    void save(std::ostream& os) const {
        for (auto const& h : m_heads) h.save(os);
        m_output_proj.save(os);
    }
    void load(std::istream& is) {
        for (auto& h : m_heads) h.load(is);
        m_output_proj.load(is);
    }
    // order: every head q(W,b) k(W,b) v(W,b), then the output projection (reference: :384-392)
    template <typename init_type>
    void init_weight() {
        for (auto& h : m_heads) h.template init_weight<init_type>();
        m_output_proj.template init_weight<init_type>();
    }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "mat_mha_t:(heads:" << m_num_heads << ", d_model:" << m_d_model << ")";
        return ss.str();
    }
    void step() {
        for (auto& h : m_heads) h.step();
        m_output_proj.step();
    }

private:
    mat_t<val_type> attend(const input_type& xq, const input_type& xkv, bool mask, bool remember = false) {
        const jsm_mat Xq = xq.jsm_device(), Xkv = xkv.jsm_device();
        const int Sq = Xq.cols, Sk = Xkv.cols, d = m_d_model, dh = m_d_head;
        mat_t<val_type> q(Sq, d), k(Sk, d), v(Sk, d), att(Sq, d);
        const jsm_mat Q = q.jsm_device_out(), K = k.jsm_device_out(), V = v.jsm_device_out();
        for (int h = 0; h < m_num_heads; ++h) {
            jsm_attn::project(m_heads[h].q_net(), jsm_attn::token_major_rows(Xq, h * dh, dh), jsm_attn::columns(Q, h * dh, dh));
            jsm_attn::project(m_heads[h].k_net(), jsm_attn::token_major_rows(Xkv, h * dh, dh), jsm_attn::columns(K, h * dh, dh));
            jsm_attn::project(m_heads[h].v_net(), jsm_attn::token_major_rows(Xkv, h * dh, dh), jsm_attn::columns(V, h * dh, dh));
        }
        jsm_attn::attention(static_cast<const float*>(Q.data), static_cast<const float*>(K.data), static_cast<const float*>(V.data),
                            static_cast<float*>(att.jsm_device_out().data), Sq, Sk, m_num_heads, dh, mask);
        // out[d, S] = Wo . concat + bo, the concatenated heads being att^T
        if (remember) m_output_proj.jsm_remember_input(att.t().clone());  // the output projection's input, for its backward
        mat_t<val_type> out(d, Sq);
        jsm_mat Wo = m_output_proj.jsm_weight().jsm_device(), Bo = m_output_proj.jsm_bias().jsm_device();
        jsm_rt::check(jsm_dot_f32(Wo, jsm_attn::transposed(att.jsm_device()), &Bo, 0, nullptr, out.jsm_device_out(), jsm_rt::stream()));
        return out;
    }
};

// cross-attention holder: keys and values come from a stored encoder output (reference: mat_mha_t.hpp:410-453)
template <typename input_type, template <typename> class updator_type>
class mat_mhca_t : public mat_mha_t<input_type, updator_type> {
public:
    using base_type = mat_mha_t<input_type, updator_type>;
    using val_type = typename input_type::ele_type;

private:
    mat_t<val_type>* m_encoder_output = nullptr;
    mat_t<val_type>* m_encoder_delta = nullptr;

public:
    mat_mhca_t(int num_heads = 1, int d_model = 1, bool mask = false, int seq_len = 1) : base_type(num_heads, d_model, mask, seq_len) {}
    void set_encoder_param(mat_t<val_type>& encoder_output, mat_t<val_type>& encoder_delta) {
        m_encoder_output = &encoder_output;
        m_encoder_delta = &encoder_delta;
    }
    mat_t<val_type> forward(const input_type& input) {
        if (m_encoder_output == nullptr) throw std::runtime_error("Encoder output not set for cross attention");
        return base_type::forward(input, *m_encoder_output);
    }
    // the static cross cache: keys and values of the stored encoder output, projected once per encoder pass
    void refresh_memory() {
        if (m_encoder_output == nullptr) throw std::runtime_error("Encoder output not set for cross attention");
        base_type::set_memory(*m_encoder_output);
    }
    mat_t<val_type> forward_cached(const input_type& input) { return base_type::forward_memory(input); }
    void step() {}
};

#endif
