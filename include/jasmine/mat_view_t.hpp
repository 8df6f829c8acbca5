// mat_view_t: a non-owning window (offset, size, transpose flag) over a mat_t
// (reference: mat_view_t.hpp:7-135) and the view factories of mat_t (:137-243).
// On the device a view is the parent's buffer with an offset pointer and (possibly swapped)
// strides: no copy is made until the view is materialised.
//
// A transposed view indexes the parent at (column + row_offset, row + col_offset), i.e. the
// window is transposed as a whole; the reference swaps the two offsets instead
// (mat_view_t.hpp:30-33), which only shows with unequal offsets and is used by its training code alone.
#ifndef JASMINE_B200_MAT_VIEW_T_HPP_
#define JASMINE_B200_MAT_VIEW_T_HPP_
#include <sstream>

#include "mat_concepts.hpp"
#include "mat_t.hpp"
#include "mat_utility.hpp"

template <typename agent_type>
class mat_view_t {
public:
    using val_type = typename agent_type::ele_type;
    using ele_type = val_type;

private:
    agent_type* m_mat;
    int m_row_offset, m_col_offset, m_row_size, m_col_size;
    bool m_transposed = false;

public:
    mat_view_t(agent_type& m, int row_offset = 0, int col_offset = 0, int row_size = -1, int col_size = -1) noexcept
        : m_mat(&m), m_row_offset(row_offset), m_col_offset(col_offset),
          m_row_size(row_size == -1 ? m.row_num() - row_offset : row_size),
          m_col_size(col_size == -1 ? m.col_num() - col_offset : col_size) {}

    int row_num() const noexcept { return m_transposed ? m_col_size : m_row_size; }
    int col_num() const noexcept { return m_transposed ? m_row_size : m_col_size; }

    decltype(auto) operator()(int row, int col) const {
        return m_transposed ? (*m_mat)(col + m_row_offset, row + m_col_offset) : (*m_mat)(row + m_row_offset, col + m_col_offset);
    }
    decltype(auto) operator()(int row, int col) {
        return m_transposed ? (*m_mat)(col + m_row_offset, row + m_col_offset) : (*m_mat)(row + m_row_offset, col + m_col_offset);
    }

    mat_view_t t() const noexcept {
        mat_view_t v(*this);
        v.m_transposed = !m_transposed;
        return v;
    }

    std::string to_string() const {
        std::stringstream ss;
        ss << "matrix_view(" << row_num() << ", " << col_num() << ")";
        for (int i = 0; i < row_num(); ++i) {
            ss << "\n[ ";
            for (int j = 0; j < col_num(); ++j) ss << (*this)(i, j) << " ";
            ss << "]";
        }
        return ss.str();
    }

    // device window of the parent (float parents only)
    jsm_mat jsm_device() const {
        jsm_mat p = m_mat->jsm_device();
        return window(p);
    }
    jsm_mat jsm_device_inout() {
        jsm_mat p = m_mat->jsm_device_inout();
        return window(p);
    }
    void jsm_lower(jsm_rt::builder& b) const {
        b.leaf(jsm_device());
        b.keep.push_back(m_mat->jsm_keepalive());
    }

    // element-wise copy of `other` (matrix, view or expression) into the window (reference: :53-63)
    template <typename other_type>
    void assign(const other_type& other);

    template <typename other_type>
    requires is_matrix<other_type>
    auto dot(const other_type& m) const;

    mat_t<val_type> clone() const;
    operator std::remove_const_t<agent_type>() const { return clone(); }

private:
    jsm_mat window(jsm_mat p) const {
        jsm_mat w = p;
        w.data = static_cast<char*>(p.data) + ((int64_t)m_row_offset * p.row_stride + (int64_t)m_col_offset * p.col_stride) * (int64_t)sizeof(val_type);
        if (m_transposed) {
            w.rows = m_col_size; w.cols = m_row_size;
            w.row_stride = p.col_stride; w.col_stride = p.row_stride;
        } else {
            w.rows = m_row_size; w.cols = m_col_size;
        }
        return w;
    }
};

// ---- view factories of mat_t ----------------------------------------------------------------
#define JSM_VIEW_FACTORY(NAME, ARGS, ...)                                                             \
    template <typename val_type>                                                                      \
    requires std::is_arithmetic_v<val_type>                                                           \
    mat_view_t<mat_t<val_type>> mat_t<val_type>::NAME ARGS noexcept {                                 \
        return mat_view_t<mat_t<val_type>>(*this, __VA_ARGS__);                                       \
    }                                                                                                 \
    template <typename val_type>                                                                      \
    requires std::is_arithmetic_v<val_type>                                                           \
    mat_view_t<const mat_t<val_type>> mat_t<val_type>::NAME ARGS const noexcept {                     \
        return mat_view_t<const mat_t<val_type>>(*this, __VA_ARGS__);                                 \
    }
JSM_VIEW_FACTORY(view, (int const& row_offset, int const& col_offset, int const& row_size, int const& col_size), row_offset, col_offset, row_size, col_size)
JSM_VIEW_FACTORY(col, (int const& idx), 0, idx, row_num(), 1)
JSM_VIEW_FACTORY(row, (int const& idx), idx, 0, 1, col_num())
JSM_VIEW_FACTORY(back_col, (), 0, col_num() - 1, row_num(), 1)
JSM_VIEW_FACTORY(back_row, (), row_num() - 1, 0, 1, col_num())
JSM_VIEW_FACTORY(front_col, (), 0, 0, row_num(), 1)
JSM_VIEW_FACTORY(front_row, (), 0, 0, 1, col_num())
#undef JSM_VIEW_FACTORY

template <typename val_type>
requires std::is_arithmetic_v<val_type>
mat_view_t<mat_t<val_type>> mat_t<val_type>::t() noexcept {
    return mat_view_t<mat_t<val_type>>(*this).t();
}

#endif
