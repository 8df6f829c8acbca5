// Weight initialisation hook of the jasmine API (reference: mat_init_t.hpp:10-118).
// init_t<tag>::cal(m) receives every weight matrix of a net in a fixed order; user code specialises it for
// its own tag to inject (or read back) weights, which is the only access to them the API offers.  Writes go
// to the host mirror of the matrix and reach the GPU with the next forward.
// The policies below are provided for completeness of the surface; training itself is not part of this library.
#ifndef JASMINE_B200_MAT_INIT_T_HPP_
#define JASMINE_B200_MAT_INIT_T_HPP_
#include <cmath>
#include <random>

#include "mat_concepts.hpp"
#include "mat_t.hpp"

static std::default_random_engine g_random_engine;

template <typename init_type>
struct init_t {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type&) {}
};

namespace jsm_init {
template <typename mat_type, typename dist_type>
void draw(mat_type& m, dist_type dist) {
    for (int i = 0; i < m.row_num(); ++i)
        for (int j = 0; j < m.col_num(); ++j) m(i, j) = dist(g_random_engine);
}
}  // namespace jsm_init

template <>
struct init_t<class zeros_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) {
        for (int i = 0; i < m.row_num(); ++i)
            for (int j = 0; j < m.col_num(); ++j) m(i, j) = 0;
    }
};
template <>
struct init_t<class xavier_gaussian_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) { jsm_init::draw(m, std::normal_distribution<double>(0.0, std::sqrt(2.0 / (m.row_num() + m.col_num())))); }
};
template <>
struct init_t<class xavier_uniform_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) {
        const double a = std::sqrt(6.0 / (m.row_num() + m.col_num()));
        jsm_init::draw(m, std::uniform_real_distribution<double>(-a, a));
    }
};
template <>
struct init_t<class he_gaussian_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) { jsm_init::draw(m, std::normal_distribution<double>(0.0, std::sqrt(2.0 / m.col_num()))); }
};
template <>
struct init_t<class he_uniform_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) {
        const double a = std::sqrt(6.0 / m.col_num());
        jsm_init::draw(m, std::uniform_real_distribution<double>(-a, a));
    }
};

template <typename init_type, typename mat_type, typename... args_types>
requires is_matrix<mat_type>
void init_matrix(mat_type& m, args_types&&... args) {
    init_t<init_type>::cal(m, std::forward<args_types>(args)...);
}

#endif
