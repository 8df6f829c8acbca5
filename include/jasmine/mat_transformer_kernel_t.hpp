// Encoder / decoder stacks of the jasmine API, forward halves (reference: mat_transformer_kernel_t.hpp).
// Layers are post-LN blocks built from the nets of mat_net_t.hpp and mat_mha_t.hpp:
//   encoder layer = LN(x + MHA(x)), LN(x + ReLU(W x + b))                      (:14-45)
//   decoder layer = LN(x + MHA_causal(x)), LN(x + MHCA(x, encoder out)), LN(x + ReLU(W x + b))   (:47-52)
// A decoder-only causal stack is an encoder_t whose attention layers are set to masked:
//   enc.get_mha(i).set_param(heads, d_model, /*mask=*/true, seq_len).
#ifndef JASMINE_B200_MAT_TRANSFORMER_KERNEL_T_HPP_
#define JASMINE_B200_MAT_TRANSFORMER_KERNEL_T_HPP_
#include <sstream>
#include <vector>

#include "mat_mha_t.hpp"
#include "mat_net_t.hpp"

template <typename val_type, template <typename> class updator_type>
using res_mha_t = residual_net_t<mat_mha_t<mat_t<val_type>, updator_type>>;
template <typename val_type, template <typename> class updator_type>
using res_mhca_t = residual_net_t<mat_mhca_t<mat_t<val_type>, updator_type>>;
template <typename val_type, template <typename> class updator_type>
using res_mha_norm_t = typename complex_net_builder_t<val_type>::template push_back_impl<res_mha_t<val_type, updator_type>>::
    template push_back_updatable<layer_norm_net_t, updator_type>::type;
template <typename val_type, template <typename> class updator_type>
using res_mhca_norm_t = typename complex_net_builder_t<val_type>::template push_back_impl<res_mhca_t<val_type, updator_type>>::
    template push_back_updatable<layer_norm_net_t, updator_type>::type;
template <typename val_type, template <typename> class updator_type>
using base_ffn_t = typename complex_net_builder_t<val_type>::template push_back_updatable<weight_net_t, updator_type>::
    template push_back_staticnet<relu_net_t>::type;
template <typename val_type, template <typename> class updator_type>
using res_ffn_t = residual_net_t<base_ffn_t<val_type, updator_type>>;
template <typename val_type, template <typename> class updator_type>
using res_ffn_norm_t = typename complex_net_builder_t<val_type>::template push_back_impl<res_ffn_t<val_type, updator_type>>::
    template push_back_updatable<layer_norm_net_t, updator_type>::type;
template <typename val_type, template <typename> class updator_type>
using encoder_layer_t = typename complex_net_builder_t<val_type>::template push_back_impl<res_mha_norm_t<val_type, updator_type>>::
    template push_back_impl<res_ffn_norm_t<val_type, updator_type>>::type;
template <typename val_type, template <typename> class updator_type>
using decoder_layer_t = typename complex_net_builder_t<val_type>::template push_back_impl<res_mha_norm_t<val_type, updator_type>>::
    template push_back_impl<res_mhca_norm_t<val_type, updator_type>>::template push_back_impl<res_ffn_norm_t<val_type, updator_type>>::type;

template <typename val_type_, template <typename> class updator_type>
class encoder_t {
public:
    using val_type = val_type_;

private:
    std::vector<encoder_layer_t<val_type, updator_type>> m_layers;

public:
    encoder_t(int const& n_layers = 1, int const& head_num = 1, int const& d_model = 1, int const& seq_len = 1) {
        set_param(n_layers, head_num, d_model, seq_len);
    }
    void set_param(int const& n_layers, int const& head_num, int const& d_model, int const& seq_len) {
        m_layers.resize(n_layers);
        for (int i = 0; i < n_layers; ++i) {
            get_mha(i).set_param(head_num, d_model, false, seq_len);
            get_ffn(i).reinit(std::vector<int>{d_model, d_model});
        }
    }
    mat_t<val_type> forward(mat_t<val_type> input) {
        for (auto& layer : m_layers) input = layer.forward(input);
        return input;
    }
    // Training step of the stack: the layers' backward steps in reverse order (reference: :112-119)
    mat_t<val_type> backward(mat_t<val_type> delta) {
        for (int i = (int)m_layers.size() - 1; i >= 0; --i) delta = m_layers[i].backward(delta);
        return delta;
    }
    // Generation with cached keys and values for a causal (decoder-only) stack: the output columns of the new input
    // columns, equal to the last columns of forward(whole prefix) - which is how the reference generates
    // (transformer_test.hpp:227-241) - at the cost of the new columns only.  Norms and feed-forward act per column.
    void reset_cache() {
        for (size_t i = 0; i < size(); ++i) get_mha(i).reset_cache();
    }
    mat_t<val_type> forward_cached(mat_t<val_type> x) {
        for (size_t i = 0; i < size(); ++i) {
            mat_t<val_type> a = get_mha(i).forward_cached(x);
            x = get_mha_norm(i).forward((a + x).clone());
            mat_t<val_type> f = get_ffn(i).forward(x);
            x = get_ffn_norm(i).forward((((f > 0) * f) + x).clone());
        }
        return x;
    }
    void save(std::ostream& os) const { for (auto const& l : m_layers) l.save(os); }
    void load(std::istream& is) { for (auto& l : m_layers) l.load(is); }
    auto& get_mha(int const& i) { return m_layers[i].template get<0, 0>().base_net(); }
    auto& get_mha_norm(int const& i) { return m_layers[i].template get<0, 1>(); }
    auto& get_ffn(int const& i) { return m_layers[i].template get<1, 0, 0>(); }
    auto& get_ffn_norm(int const& i) { return m_layers[i].template get<1, 1>(); }
    auto& get_mha(int const& i) const { return m_layers[i].template get<0, 0>().base_net(); }
    auto& get_ffn(int const& i) const { return m_layers[i].template get<1, 0, 0>(); }
    size_t size() const { return m_layers.size(); }

    // order per layer: attention, its norm, feed-forward, its norm (reference: :166-176)
    template <typename init_type>
    void init_weight() {
        for (size_t i = 0; i < size(); ++i) {
            get_mha(i).template init_weight<init_type>();
            get_mha_norm(i).template init_weight<init_type>();
            get_ffn(i).template init_weight<init_type>();
            get_ffn_norm(i).template init_weight<init_type>();
        }
    }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "encoder = [";
        for (size_t i = 0; i < size(); ++i)
            ss << "\n" << print_indent(indent + 2) << "Layer " << i << " mha: " << get_mha(i).net_type() << "-->" << "ffn: " << get_ffn(i).net_type();
        ss << std::endl << print_indent(indent) << "]";
        return ss.str();
    }
    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        for (size_t i = 0; i < size(); ++i) {
            get_mha(i).set_updator(args...);
            get_mha_norm(i).set_updator(args...);
            get_ffn(i).set_updator(args...);
            get_ffn_norm(i).set_updator(args...);
        }
    }
    void step() {
        for (size_t i = 0; i < size(); ++i) {
            get_mha(i).step(); get_mha_norm(i).step(); get_ffn(i).step(); get_ffn_norm(i).step();
        }
    }
};

template <typename val_type_, template <typename> class updator_type>
class decoder_t {
public:
    using val_type = val_type_;

private:
    mat_t<val_type> m_encoder_output, m_encoder_delta;
    bool m_memory_fresh = false;  // the cross-attention layers hold the keys and values of m_encoder_output
    encoder_t<val_type, updator_type>* m_encoder = nullptr;
    std::vector<decoder_layer_t<val_type, updator_type>> m_layers;

public:
    decoder_t(int const& n_layers = 1, int const& head_num = 1, int const& d_model = 1, int const& seq_len = 1) {
        set_param(n_layers, head_num, d_model, seq_len);
    }
    decoder_t(const decoder_t&) = delete;  // the cross-attention layers point at this object's encoder output
    decoder_t& operator=(const decoder_t&) = delete;

    void set_param(int const& n_layers, int const& head_num, int const& d_model, int const& seq_len = 1) {
        m_layers.resize(n_layers);
        for (size_t i = 0; i < size(); ++i) {
            get_mha(i).set_param(head_num, d_model, true, seq_len);
            get_mhca(i).set_param(head_num, d_model, false, seq_len);
            get_mhca(i).set_encoder_param(m_encoder_output, m_encoder_delta);
            get_ffn(i).reinit(std::vector<int>{d_model, d_model});
        }
    }
    mat_t<val_type> forward(const mat_t<val_type>& input) {
        mat_t<val_type> output = input;
        for (auto& layer : m_layers) output = layer.forward(output);
        return output;
    }
    void set_encoder(encoder_t<val_type, updator_type>& encoder) {
        m_encoder = &encoder;
        for (size_t i = 0; i < size(); ++i) get_mhca(i).set_encoder_param(m_encoder_output, m_encoder_delta);
    }
    // a new encoder output: the self-attention caches start over and the cross-attention layers project their keys and
    // values once, lazily at the first cached step
    void set_encoder_output(const mat_t<val_type>& encoder_output) {
        m_encoder_output = encoder_output;
        m_memory_fresh = false;
        reset_cache();
    }
    void reset_cache() {
        for (size_t i = 0; i < size(); ++i) get_mha(i).reset_cache();
    }
    // the decoder outputs of the new input columns, equal to the last columns of forward(whole prefix) (the reference's
    // predict loop, transformer_test.hpp:227-241, recomputes that prefix at every step)
    mat_t<val_type> forward_cached(mat_t<val_type> x) {
        if (!m_memory_fresh) {
            for (size_t i = 0; i < size(); ++i) get_mhca(i).refresh_memory();
            m_memory_fresh = true;
        }
        for (size_t i = 0; i < size(); ++i) {
            mat_t<val_type> a = get_mha(i).forward_cached(x);
            x = get_mha_norm(i).forward((a + x).clone());
            mat_t<val_type> c = get_mhca(i).forward_cached(x);
            x = get_mhca_norm(i).forward((c + x).clone());
            mat_t<val_type> f = get_ffn(i).forward(x);
            x = get_ffn_norm(i).forward((((f > 0) * f) + x).clone());
        }
        return x;
    }
    void save(std::ostream& os) const { for (auto const& l : m_layers) l.save(os); }
    void load(std::istream& is) { for (auto& l : m_layers) l.load(is); }
    mat_t<val_type> get_encoder_output() const { return m_encoder_output; }
    size_t size() const { return m_layers.size(); }

    // order per layer: self attention, norm, cross attention, norm, feed-forward, norm (reference: :340-352)
    template <typename init_type>
    void init_weight() {
        for (size_t i = 0; i < size(); ++i) {
            get_mha(i).template init_weight<init_type>();
            get_mha_norm(i).template init_weight<init_type>();
            get_mhca(i).template init_weight<init_type>();
            get_mhca_norm(i).template init_weight<init_type>();
            get_ffn(i).template init_weight<init_type>();
            get_ffn_norm(i).template init_weight<init_type>();
        }
    }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "decoder = [";
        for (size_t i = 0; i < size(); ++i)
            ss << "\n" << print_indent(indent + 2) << "Layer " << i << " mha: " << get_mha(i).net_type() << "-->" << "mhca: " << get_mhca(i).net_type()
               << "-->" << "ffn: " << get_ffn(i).net_type();
        ss << std::endl << print_indent(indent) << "]";
        return ss.str();
    }
    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        for (size_t i = 0; i < size(); ++i) {
            get_mha(i).set_updator(args...); get_mha_norm(i).set_updator(args...);
            get_mhca(i).set_updator(args...); get_mhca_norm(i).set_updator(args...);
            get_ffn(i).set_updator(args...); get_ffn_norm(i).set_updator(args...);
        }
    }
    void step() {}
    auto& get_mha(int const& i) { return m_layers[i].template get<0, 0>().base_net(); }
    auto& get_mha_norm(int const& i) { return m_layers[i].template get<0, 1>(); }
    auto& get_mhca(int const& i) { return m_layers[i].template get<1, 0>().base_net(); }
    auto& get_mhca_norm(int const& i) { return m_layers[i].template get<1, 1>(); }
    auto& get_ffn(int const& i) { return m_layers[i].template get<2, 0, 0>(); }
    auto& get_ffn_norm(int const& i) { return m_layers[i].template get<2, 1>(); }
    auto& get_mha(int const& i) const { return m_layers[i].template get<0, 0>().base_net(); }
    auto& get_mhca(int const& i) const { return m_layers[i].template get<1, 0>().base_net(); }
    auto& get_ffn(int const& i) const { return m_layers[i].template get<2, 0, 0>(); }
};

template <typename val_type_, template <typename> class updator_type>
class transformer_kernel_t {
public:
    using val_type = val_type_;
    using encoder_type = encoder_t<val_type, updator_type>;
    using decoder_type = decoder_t<val_type, updator_type>;

private:
    encoder_type m_encoder;
    decoder_type m_decoder;

public:
    transformer_kernel_t(int const& en_layers = 1, int const& de_layers = 1, int const& head_num = 1, int const& d_model = 1, int const& seq_len = 1)
        : m_encoder(en_layers, head_num, d_model, seq_len), m_decoder(de_layers, head_num, d_model, seq_len) {
        m_decoder.set_encoder(m_encoder);
    }
    void encoder_forward(const mat_t<val_type>& input) { m_decoder.set_encoder_output(m_encoder.forward(input)); }
    // after encoder_forward; may be called many times to generate a sequence (reference: :475-478)
    mat_t<val_type> forward(const mat_t<val_type>& input) { return m_decoder.forward(input); }
    // the same for the new columns only, against cached self-attention keys / values and the static cross cache
    mat_t<val_type> forward_cached(const mat_t<val_type>& new_columns) { return m_decoder.forward_cached(new_columns); }
    void reset_cache() { m_decoder.reset_cache(); }
    void save(std::ostream& os) const { m_encoder.save(os); m_decoder.save(os); }
    void load(std::istream& is) { m_encoder.load(is); m_decoder.load(is); }
    template <typename... upr_param_types>
    void set_updator(upr_param_types&&... params) { m_encoder.set_updator(params...); m_decoder.set_updator(params...); }
    template <typename init_type>
    void init_weight() {
        m_encoder.template init_weight<init_type>();
        m_decoder.template init_weight<init_type>();
    }
    void set_param(int const& en_layers, int const& de_layers, int const& head_num, int const& d_model) {
        m_encoder.set_param(en_layers, head_num, d_model, 1);
        m_decoder.set_param(de_layers, head_num, d_model, 1);
    }
    encoder_type& encoder() { return m_encoder; }
    decoder_type& decoder() { return m_decoder; }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "transformer_kernel = [\n" << m_encoder.net_type(indent + 2) << " \n" << m_decoder.net_type(indent + 2) << std::endl
           << print_indent(indent) << "]";
        return ss.str();
    }
    void step() {}
};

#endif
