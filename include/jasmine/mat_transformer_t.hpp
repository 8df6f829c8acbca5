// transformer_base_t of the jasmine API, forward (reference: mat_transformer_t.hpp:18-85):
// RoPE applied once to the [d_model, seq_len] input, then the encoder / decoder stacks.
#ifndef JASMINE_B200_MAT_TRANSFORMER_T_HPP_
#define JASMINE_B200_MAT_TRANSFORMER_T_HPP_
#include "mat_RoPE_t.hpp"
#include "mat_net_t.hpp"
#include "mat_transformer_kernel_t.hpp"

template <typename input_type, template <typename> class updator_type>
class transformer_base_t {
public:
    using val_type = typename input_type::ele_type;
    using RoPE_type = RoPE_net_t<input_type>;
    using kernel_type = transformer_kernel_t<val_type, updator_type>;

private:
    kernel_type m_kernel;
    RoPE_type m_rope;
    int m_generated = 0;  // decoder positions consumed by forward_cached since the last encoder pass

public:
    transformer_base_t(size_t en_layers = 1, size_t de_layers = 1, size_t head_num = 1, int d_model = 1)
        : m_kernel((int)en_layers, (int)de_layers, (int)head_num, d_model), m_rope(d_model) {}

    void encoder_forward(const mat_t<val_type>& input) {
        m_kernel.encoder_forward(m_rope.forward(input));
        m_generated = 0;
    }
    mat_t<val_type> forward(const mat_t<val_type>& input) { return m_kernel.forward(m_rope.forward(input)); }
    // Generation step with caches: `new_columns` continue the decoder input at position generated(); they are rotated at
    // their own positions and run against the cached keys / values.  The result equals the last columns of
    // forward(all decoder input columns so far), which is what the reference's predict loop recomputes at every step
    // (transformer_test.hpp:227-241).  encoder_forward (or reset_cache) starts a new sequence.
    mat_t<val_type> forward_cached(const mat_t<val_type>& new_columns) {
        mat_t<val_type> rotated = m_rope.forward(new_columns, m_generated);
        m_generated += new_columns.col_num();
        return m_kernel.forward_cached(rotated);
    }
    void reset_cache() { m_kernel.reset_cache(); m_generated = 0; }
    int generated() const { return m_generated; }
    void save(std::ostream& os) const { m_kernel.save(os); }
    void load(std::istream& is) { m_kernel.load(is); }

    template <typename... upr_param_types>
    void set_updator(upr_param_types&&... params) { m_kernel.set_updator(std::forward<upr_param_types>(params)...); }
    template <typename init_type>
    void init_weight() { m_kernel.template init_weight<init_type>(); }
    void set_param(size_t en_layers, size_t de_layers, size_t head_num, int d_model) {
        m_kernel.set_param((int)en_layers, (int)de_layers, (int)head_num, d_model);
        m_rope.set_param(d_model);
    }
    kernel_type& kernel() { return m_kernel; }
    void step() {}
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "transformer_base_t = [\n" << m_kernel.net_type(indent + 2) << " \n" << m_rope.net_type(indent + 2) << std::endl
           << print_indent(indent) << "]";
        return ss.str();
    }
};

#endif
