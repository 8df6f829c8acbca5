// Stream output and the net-folding operators of the jasmine API (reference: mat_utility.hpp:7-39, 94-100).
// The learning-rate schedule of the reference (mat_utility.hpp:102-239) belongs to training and is not provided.
#ifndef JASMINE_B200_MAT_UTILITY_HPP_
#define JASMINE_B200_MAT_UTILITY_HPP_
#include <cmath>
#include <ostream>
#include <string>

#include "mat_concepts.hpp"

template <typename M>
requires is_serializable<M>
std::ostream& operator<<(std::ostream& os, const M& m) {
    return os << m.to_string();
}

// input >> net  ==  net.forward(input); a chain folds left to right (complex_net_t::forward)
template <typename Net, typename In>
requires is_forwardable<Net, In>
auto operator>>(In const& input, Net& net) {
    return net.forward(input);
}
template <typename In, typename... Nets>
auto net_forward(In const& input, Nets&&... nets) {
    return (input >> ... >> nets);
}

// net << delta  ==  net.backward(delta); a chain folds right to left (complex_net_t::backward; reference: mat_utility.hpp:28-39)
template <typename Net, typename In>
requires is_backwardable<Net, In>
auto operator<<(Net& net, In const& input) {
    return net.backward(input);
}
template <typename In, typename... Nets>
auto net_backward(In const& input, Nets&&... nets) {
    return (nets << ... << input);
}

inline std::string print_indent(int n) { return std::string(n > 0 ? (size_t)n : 0, ' '); }

#endif
