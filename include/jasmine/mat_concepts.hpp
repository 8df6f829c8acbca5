// Concepts of the jasmine API surface (reference: mat_concepts.hpp:6-57): what counts as a matrix,
// as a net, as serialisable.  Code written against the reference's concepts compiles against these.
#ifndef JASMINE_B200_MAT_CONCEPTS_HPP_
#define JASMINE_B200_MAT_CONCEPTS_HPP_
#include <concepts>
#include <string>
#include <type_traits>
#include <vector>

// anything with row_num(), col_num() and element access (i, j)
template <typename M>
concept is_matrix = requires(M m, int i, int j) {
    { m.row_num() } -> std::convertible_to<int>;
    { m.col_num() } -> std::convertible_to<int>;
    { m(i, j) };
};

template <typename... Ts>
concept is_caculable = ((std::is_arithmetic_v<Ts> || is_matrix<Ts>) && ...);

template <typename M>
concept is_serializable = requires(M m) {
    { m.to_string() } -> std::convertible_to<std::string>;
};

template <typename Net, typename In>
concept is_forwardable = requires(Net net, In x) {
    { net.forward(x) };
};

template <typename Net, typename In>
concept is_backwardable = requires(Net net, In x) {
    { net.backward(x) };
};

template <typename Net>
concept is_reinitable_net = requires(Net net) { net.reinit(std::vector<int>()); };
template <typename Net>
concept is_unreinitable_net = !is_reinitable_net<Net>;

template <typename Net>
concept is_updatable_net = requires(Net net) { net.set_updator(0.01); };
template <typename Net>
concept is_unupdatable_net = !is_updatable_net<Net>;

#endif
