// Loss layers of the jasmine API (reference: mat_loss_t.hpp): a loss is a net whose forward passes its input through and
// remembers it; backward(target) is the gradient that starts the backward chain.
#ifndef JASMINE_B200_MAT_LOSS_T_HPP_
#define JASMINE_B200_MAT_LOSS_T_HPP_
#include <sstream>
#include <string>

#include "mat_concepts.hpp"
#include "mat_express_t.hpp"

template <typename input_type>
class mat_loss_t {
public:
    using val_type = typename input_type::ele_type;
    mat_loss_t() = default;
    mat_t<val_type> m_input;
    mat_t<val_type> forward(const input_type& input) {
        m_input = input;
        return input;
    }
};

// mean squared error (reference: mat_loss_t.hpp:27-58): gradient = prediction - target, loss = mean((prediction - target)^2)
template <typename input_type>
class mse_loss_t : public mat_loss_t<input_type> {
public:
    using base_type = mat_loss_t<input_type>;
    using val_type = typename base_type::val_type;
    mse_loss_t() = default;
    mat_t<val_type> backward(const mat_t<val_type>& target) const { return (base_type::m_input - target).clone(); }
    val_type loss(const mat_t<val_type>& target) const { return mean(pow((base_type::m_input - target).clone(), 2.0)); }
    std::string net_type(int const& indent = 0) const { return print_indent(indent) + "mse_loss_t"; }
    template <typename init_type>
    void init_weight() {}
    void step() {}
    void save(std::ostream&) const {}
    void load(std::istream&) {}
};

#endif
