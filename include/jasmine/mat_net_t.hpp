// Layer library of the jasmine API, forward halves (reference: mat_net_t.hpp): weight_net_t (linear),
// sigmoid_net_t, relu_net_t, layer_norm_net_t, hsoftmax_net_t, residual_net_t, the tuple composition
// complex_net_t and its builder.  Matrices are [features, tokens] like in the reference; every forward is
// one or two kernels of libjasmine_b200.  backward() belongs to training and is not provided.
#ifndef JASMINE_B200_MAT_NET_T_HPP_
#define JASMINE_B200_MAT_NET_T_HPP_
#include <sstream>
#include <string>
#include <tuple>
#include <vector>

#include "mat_express_t.hpp"
#include "mat_init_t.hpp"
#include "mat_t.hpp"
#include "mat_updator_t.hpp"

// Y = W . X + b, W:[out, in], b:[out, 1] broadcast over the columns (reference: mat_net_t.hpp:12-89)
template <typename input_type, template <typename> class updator_type>
class weight_net_t {
public:
    using val_type = typename input_type::ele_type;

private:
    mat_t<val_type> m_weight, m_bias;
    updator_type<val_type> m_weight_updator, m_bias_updator;
    mat_t<val_type> m_input;  // the last forward's input, for backward (reference: mat_net_t.hpp:23, 40)

public:
    weight_net_t(int const& input_size = 1, int const& output_size = 1) : m_weight(output_size, input_size), m_bias(output_size, 1) {}

    // {input size, output size}; storage is replaced only when the element count changes (mat_t::reshape)
    void reinit(std::vector<int> const& container) {
        m_weight.reshape(container[1], container[0]);
        m_bias.reshape(container[1], 1);
    }

    // one kernel: k-ascending fp32 dot products with the bias added in the epilogue
    template <typename any_input>
    mat_t<val_type> forward(const any_input& input) {
        if (m_weight.col_num() != input.row_num()) throw std::invalid_argument("mat_dot_t: inner dimensions do not match for dot product");
        std::vector<std::shared_ptr<void>> keep;
        jsm_mat X = jsm_expr::operand(input, keep);
        jsm_mat W = m_weight.jsm_device(), B = m_bias.jsm_device();
        mat_t<val_type> out(m_weight.row_num(), input.col_num());
        jsm_rt::check(jsm_dot_f32(W, X, &B, 0, nullptr, out.jsm_device_out(), jsm_rt::stream()));
        if constexpr (std::is_same_v<any_input, mat_t<val_type>>) m_input = input;  // a device-to-device copy: kept for backward
        else m_input = mat_t<val_type>();
        return out;
    }

    // Training step of the layer (reference: mat_net_t.hpp:65-75): dW = delta . X^T, db = row sums of delta, the
    // gradient handed down is W^T . delta (with the weights BEFORE the update), then both updaters run.
    template <typename other_type>
    mat_t<val_type> backward(const other_type& delta) {
        if (!m_input.valid()) throw std::runtime_error("backward without a preceding forward on a matrix input");
        mat_t<val_type> d = delta;
        mat_t<val_type> delta_weight = d.dot(m_input.t()).clone();
        mat_t<val_type> delta_bias = hsum(d);
        mat_t<val_type> ret = m_weight.t().dot(d).clone();
        m_weight_updator.update(delta_weight, m_weight);
        m_bias_updator.update(delta_bias, m_bias);
        return ret;
    }

    template <typename init_type>
    void init_weight() {
        init_matrix<init_type>(m_weight);
        init_matrix<init_type>(m_bias);
    }
    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        m_weight_updator.set(std::forward<upr_arg_types>(args)...);
        m_bias_updator.set(std::forward<upr_arg_types>(args)...);
    }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "weight_net_t:(in:" << m_weight.col_num() << ", out:" << m_weight.row_num() << ")";
        return ss.str();
    }
    void step() { m_weight_updator.step(); m_bias_updator.step(); }

    // device windows for fused callers (attention packs the per-head projections itself)
    const mat_t<val_type>& jsm_weight() const { return m_weight; }
    const mat_t<val_type>& jsm_bias() const { return m_bias; }
    // a fused caller ran the projection itself: it hands over the input that backward needs
    void jsm_remember_input(const mat_t<val_type>& input) { m_input = input; }
    // flat binary checkpoint (not in the reference, which cannot store a net): W then b
    void save(std::ostream& os) const { jsm_rt::save_tensor(os, m_weight); jsm_rt::save_tensor(os, m_bias); }
    void load(std::istream& is) { jsm_rt::load_tensor(is, m_weight); jsm_rt::load_tensor(is, m_bias); }
};

namespace jsm_net {
template <typename val_type, typename any_input>
mat_t<val_type> unary(const any_input& input, int opcode) {
    jsm_rt::builder b;
    jsm_expr::lower(b, input);
    b.op(opcode);
    mat_t<val_type> out(input.row_num(), input.col_num());
    jsm_rt::check(jsm_eval_elementwise(b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), out.jsm_device_out(), jsm_rt::stream()));
    return out;
}
}  // namespace jsm_net

template <typename input_type>
class sigmoid_net_t {
public:
    using val_type = typename input_type::ele_type;
    sigmoid_net_t() = default;
    void save(std::ostream&) const {}
    void load(std::istream&) {}
    mat_t<val_type> m_output;  // reference: mat_net_t.hpp:97
    mat_t<val_type> forward(const input_type& input) {
        m_output = jsm_net::unary<val_type>(input, JSM_OP_SIGMOID);
        return m_output;
    }
    // delta * (1 - y) * y (reference: :108-116)
    mat_t<val_type> backward(const mat_t<val_type>& delta) {
        if (delta.row_num() != m_output.row_num() || delta.col_num() != m_output.col_num()) throw std::runtime_error("delta size does not match input size");
        return (delta * (1 - m_output) * m_output).clone();
    }
    std::string net_type(int const& indent = 0) const { return print_indent(indent) + "sigmoid_net_t"; }
    template <typename init_type>
    void init_weight() {}
    void step() {}
};

// (x > 0) * x (reference: mat_net_t.hpp:146-153)
template <typename input_type>
class relu_net_t {
public:
    using val_type = typename input_type::ele_type;
    relu_net_t() = default;
    void save(std::ostream&) const {}
    void load(std::istream&) {}
    mat_t<val_type> m_input;  // reference: mat_net_t.hpp:142
    mat_t<val_type> forward(const input_type& input) {
        m_input = input;
        return jsm_net::unary<val_type>(input, JSM_OP_RELU);
    }
    // delta * (x > 0) (reference: :155-165)
    template <typename other_type>
    mat_t<val_type> backward(const other_type& delta) {
        if (delta.row_num() != m_input.row_num() || delta.col_num() != m_input.col_num()) throw std::runtime_error("delta size does not match input size");
        return (delta * (m_input > 0)).clone();
    }
    std::string net_type(int const& indent = 0) const { return print_indent(indent) + "relu_net_t"; }
    template <typename init_type>
    void init_weight() {}
    void step() {}
};

// Normalises every column (= token) of the input: population standard deviation, no epsilon, gain and bias
// [features, 1] created as 1 / 0 on the first forward (reference: mat_net_t.hpp:186-264).
template <typename input_type, template <typename> class updator_type>
class layer_norm_net_t {
    using val_type = typename input_type::ele_type;
    mat_t<val_type> m_gama, m_beta;
    updator_type<val_type> m_gama_updator, m_beta_updator;
    val_type m_eps = 0;
    mat_t<val_type> m_input;  // the last forward's input: backward rebuilds the normalised values and deviations from it

public:
    layer_norm_net_t() = default;
    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        m_gama_updator.set(std::forward<upr_arg_types>(args)...);
        m_beta_updator.set(std::forward<upr_arg_types>(args)...);
    }
    // not in the reference: an epsilon under the square root (0 keeps the reference's arithmetic)
    void set_eps(val_type eps) { m_eps = eps; }
    mat_t<val_type>& gain() { return m_gama; }
    mat_t<val_type>& bias() { return m_beta; }

    mat_t<val_type> forward(const input_type& input) {
        if (!m_gama.valid()) {
            m_gama = mat_t<val_type>(input.row_num(), 1);
            m_beta = mat_t<val_type>(input.row_num(), 1);
            m_gama = val_type(1);
            m_beta = val_type(0);
        }
        const float* g = static_cast<const float*>(m_gama.jsm_device().data);
        const float* b = static_cast<const float*>(m_beta.jsm_device().data);
        m_input = input;
        return jsm_expr::along_axis(JSM_ROWS_LAYERNORM, 0, input, g, b, (float)m_eps);
    }
    // Training step (reference: mat_net_t.hpp:227-243, eps = 0).  With x_hat the normalised input, sigma the per-column
    // deviation and m the number of rows: d_gain = row sums of delta * x_hat, d_bias = row sums of delta, and the gradient
    // handed down is (g * m - rowsum(g) - x_hat * rowsum(g * x_hat)) / m / sigma with g = delta * gain - the reference's
    // own formula, row sums included.
    template <typename other_type>
    mat_t<val_type> backward(const other_type& delta_in) {
        if (!m_input.valid()) throw std::runtime_error("backward without a preceding forward");
        mat_t<val_type> delta = delta_in;
        mat_t<val_type> mean_row = vmean(m_input);
        mat_t<val_type> centred = (m_input - mean_row).clone();
        mat_t<val_type> sigma = sqrt(vmean(pow(centred, 2.0)));
        mat_t<val_type> hx = (centred / sigma).clone();
        mat_t<val_type> d_gain = hsum(delta * hx);
        mat_t<val_type> d_bias = hsum(delta);
        const val_type m = static_cast<val_type>(delta.row_num());
        mat_t<val_type> g = (delta * m_gama).clone();
        mat_t<val_type> sum_g = hsum(g);
        mat_t<val_type> sum_g_hx = hsum(g * hx);
        mat_t<val_type> down = ((g * m - sum_g - hx * sum_g_hx) / m / sigma).clone();
        m_gama_updator.update(d_gain, m_gama);
        m_beta_updator.update(d_bias, m_beta);
        return down;
    }
    std::string net_type(int const& indent = 0) const { return print_indent(indent) + "layer_norm_net_t"; }
    template <typename init_type>
    void init_weight() {
        init_matrix<init_type>(m_gama);
        init_matrix<init_type>(m_beta);
    }
    void step() { m_gama_updator.step(); m_beta_updator.step(); }
    // gain and bias exist from the first forward on: a flag says whether the record holds them
    void save(std::ostream& os) const {
        const int32_t present = m_gama.valid() ? 1 : 0;
        os.write(reinterpret_cast<const char*>(&present), 4);
        if (present) { jsm_rt::save_tensor(os, m_gama); jsm_rt::save_tensor(os, m_beta); }
    }
    void load(std::istream& is) {
        int32_t present = 0;
        is.read(reinterpret_cast<char*>(&present), 4);
        if (!is) throw std::runtime_error("load: truncated layer norm record");
        if (present) { jsm_rt::load_tensor(is, m_gama, true); jsm_rt::load_tensor(is, m_beta, true); }
    }
};

template <typename input_type>
class hsoftmax_net_t {
public:
    using val_type = typename input_type::ele_type;
    mat_t<val_type> m_output;
    template <typename any_input>
    mat_t<val_type> forward(const any_input& input) {
        m_output = jsm_expr::along_axis(JSM_ROWS_SOFTMAX, 1, input);
        return m_output;
    }
    // y * (delta - rowsum(y * delta)) (reference: mat_net_t.hpp:281-285)
    mat_t<val_type> backward(const mat_t<val_type>& delta) {
        mat_t<val_type> dot_rows = hsum(m_output * delta);
        return (m_output * (delta - dot_rows)).clone();
    }
    std::string net_type(int const& indent = 0) const { return print_indent(indent) + "hsoftmax_net_t"; }
    template <typename init_type>
    void init_weight() {}
    void step() {}
    void save(std::ostream&) const {}
    void load(std::istream&) {}
};

// f(x) + x (reference: mat_net_t.hpp:304-364)
template <typename base_net_type>
class residual_net_t {
public:
    using val_type = typename base_net_type::val_type;
    base_net_type m_net;
    residual_net_t() : m_net() {}
    base_net_type& base_net() { return m_net; }
    base_net_type const& base_net() const { return m_net; }
    mat_t<val_type> forward(const mat_t<val_type>& input) {
        mat_t<val_type> y = m_net.forward(input);
        return (y + input).clone();
    }
    // reference: mat_net_t.hpp:330-334
    template <typename other_type>
    mat_t<val_type> backward(const other_type& delta) {
        mat_t<val_type> d = delta;
        mat_t<val_type> inner = m_net.backward(d);
        return (inner + d).clone();
    }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "residual_net_t:\n" << m_net.net_type(indent + 2);
        return ss.str();
    }
    template <typename init_type>
    void init_weight() { m_net.template init_weight<init_type>(); }
    template <size_t... nums>
    decltype(auto) get() { return m_net.template get<nums...>(); }
    template <size_t... nums>
    decltype(auto) get() const { return m_net.template get<nums...>(); }
    void step() { m_net.step(); }
    void save(std::ostream& os) const { m_net.save(os); }
    void load(std::istream& is) { m_net.load(is); }
};

// a tuple of nets applied left to right (reference: mat_net_t.hpp:366-488)
template <typename... net_types>
class complex_net_t {
    std::tuple<net_types...> m_nets;

public:
    using val_type = typename std::tuple_element_t<0, std::tuple<net_types...>>::val_type;

    template <typename input_type>
    auto forward(const input_type& input) {
        return std::apply([&input](auto&... nets) { return net_forward(input, nets...); }, m_nets);
    }
    // the members' backward steps from the last net to the first (reference: mat_net_t.hpp:381-385)
    template <typename input_type>
    auto backward(const input_type& delta) {
        return std::apply([&delta](auto&... nets) { return net_backward(delta, nets...); }, m_nets);
    }
    constexpr size_t size() { return sizeof...(net_types); }

    // container = layer widths; every net with reinit() consumes one {in, out} pair
    template <typename container_type, size_t N = 0, size_t I = 0>
    void reinit(container_type const& container) {
        using member = std::tuple_element_t<N, std::tuple<net_types...>>;
        if constexpr (is_reinitable_net<member>) {
            if (I + 1 >= container.size()) throw std::runtime_error("container size does not match net size");
            std::get<N>(m_nets).reinit({container[I], container[I + 1]});
            if constexpr (N + 1 < sizeof...(net_types)) reinit<container_type, N + 1, I + 1>(container);
        } else {
            if constexpr (N + 1 < sizeof...(net_types)) reinit<container_type, N + 1, I>(container);
        }
    }
    template <typename... upr_arg_types>
    void set_updator(upr_arg_types&&... args) {
        std::apply([&](auto&... nets) { (set_one(nets, args...), ...); }, m_nets);
    }
    template <typename init_type>
    void init_weight() {
        std::apply([](auto&... nets) { ((nets.template init_weight<init_type>()), ...); }, m_nets);
    }
    void step() {
        std::apply([](auto&... nets) { ((nets.step()), ...); }, m_nets);
    }
    // the members' records in tuple order
    void save(std::ostream& os) const {
        std::apply([&os](auto const&... nets) { ((nets.save(os)), ...); }, m_nets);
    }
    void load(std::istream& is) {
        std::apply([&is](auto&... nets) { ((nets.load(is)), ...); }, m_nets);
    }
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "complex_net_t = [";
        std::apply([&ss, indent](auto const&... nets) { ((ss << std::endl << nets.net_type(indent + 2)), ...); }, m_nets);
        ss << std::endl << print_indent(indent) << "]";
        return ss.str();
    }
    auto back() { return std::get<sizeof...(net_types) - 1>(m_nets); }

    template <size_t N, size_t... nums>
    decltype(auto) get() {
        if constexpr (sizeof...(nums) == 0) return (std::get<N>(m_nets));
        else return std::get<N>(m_nets).template get<nums...>();
    }
    template <size_t N, size_t... nums>
    decltype(auto) get() const {
        if constexpr (sizeof...(nums) == 0) return (std::get<N>(m_nets));
        else return std::get<N>(m_nets).template get<nums...>();
    }

private:
    template <typename net, typename... upr_arg_types>
    static void set_one(net& n, upr_arg_types&... args) {
        if constexpr (is_updatable_net<net>) n.set_updator(args...);
    }
};

template <typename val_type, typename... net_types>
struct complex_net_builder_t {
    template <template <typename, template <typename> class> class cur_net_tpl, template <typename> class updator_tpl>
    using push_back_updatable = complex_net_builder_t<val_type, net_types..., cur_net_tpl<mat_t<val_type>, updator_tpl>>;
    template <template <typename> class cur_net_tpl>
    using push_back_staticnet = complex_net_builder_t<val_type, net_types..., cur_net_tpl<mat_t<val_type>>>;
    template <typename new_net_type>
    using push_back_impl = complex_net_builder_t<val_type, net_types..., new_net_type>;
    using type = complex_net_t<net_types...>;
};

#endif
