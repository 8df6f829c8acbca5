// Rotary position embedding of the jasmine API (reference: mat_RoPE_t.hpp): the growable table holder
// mat_cache_t, the memoised table mat_RoPE_t and the layer RoPE_net_t (forward).
//
// The reference's table T(r, c) holds cos / -sin / sin / cos of angle = c / 10000^((r/2)/d) by the parity of
// (r, c), and the block of (pair i, position m) is T[2i..2i+1, 2m..2m+1] (mat_RoPE_t.hpp:99-148): the two
// columns of a block use the angles of columns 2m and 2m+1.  RoPE_net_t::forward keeps exactly that
// arithmetic but runs it as one table-driven kernel over the whole [d_model, seq_len] input.
#ifndef JASMINE_B200_MAT_ROPE_T_HPP_
#define JASMINE_B200_MAT_ROPE_T_HPP_
#include <algorithm>
#include <cmath>
#include <stdexcept>

#include "mat_express_t.hpp"
#include "mat_view_t.hpp"

template <typename val_type>
class mat_cache_t {
    mat_t<val_type> m_cache;
    int m_cache_rows = 0, m_cache_cols = 0;
    static constexpr int EXPAND_SIZE = 1024;

    void expand_cache(int rows, int cols) {
        if (rows <= m_cache.row_num() && cols <= m_cache.col_num()) return;
        const int new_rows = rows > m_cache.row_num() ? std::max(rows, m_cache.row_num() + EXPAND_SIZE) : m_cache.row_num();
        const int new_cols = cols > m_cache.col_num() ? std::max(cols, m_cache.col_num() + EXPAND_SIZE) : m_cache.col_num();
        mat_t<val_type> grown(new_rows, new_cols);
        for (int i = 0; i < m_cache_rows; ++i)
            for (int j = 0; j < m_cache_cols; ++j) grown(i, j) = m_cache(i, j);
        m_cache = std::move(grown);
    }

public:
    mat_cache_t() : m_cache(EXPAND_SIZE, EXPAND_SIZE) {}
    val_type& operator()(int row, int col) {
        if (row >= m_cache_rows || col >= m_cache_cols) {
            expand_cache(row + 1, col + 1);
            m_cache_rows = std::max(m_cache_rows, row + 1);
            m_cache_cols = std::max(m_cache_cols, col + 1);
        }
        return m_cache(row, col);
    }
    const val_type& operator()(int row, int col) const {
        if (row >= m_cache_rows || col >= m_cache_cols) throw std::out_of_range("Cache access out of range");
        return m_cache(row, col);
    }
    mat_view_t<mat_t<val_type>> range(int row, int col, int rows, int cols) {
        if (row + rows > m_cache_rows || col + cols > m_cache_cols) {
            expand_cache(row + rows, col + cols);
            m_cache_rows = std::max(m_cache_rows, row + rows);
            m_cache_cols = std::max(m_cache_cols, col + cols);
        }
        return m_cache.view(row, col, rows, cols);
    }
};

template <typename val_type>
class mat_RoPE_t {
    mat_cache_t<val_type> m_cache;
    int m_enable_rows = 0, m_enable_cols = 0, m_d;

public:
    mat_RoPE_t(int const& d) : m_d(d) {}
    void set_d(int const& d) { m_d = d; m_enable_rows = 0; m_enable_cols = 0; }
    val_type get_d() const { return m_d; }

    // fills the not yet initialised part of rows [0, row_beg+rows) x columns [0, col_beg+cols)
    void init(int const& row_beg, int const& rows, int const& col_beg, int const& cols) {
        const int R = row_beg + rows, Cn = col_beg + cols;
        for (int i = 0; i < R; ++i)
            for (int j = 0; j < Cn; ++j) {
                if (i < m_enable_rows && j < m_enable_cols) continue;
                const val_type angle = static_cast<val_type>(j / std::pow(10000.0, (i / 2) / static_cast<val_type>(m_d)));
                const bool even_r = (i % 2 == 0), even_c = (j % 2 == 0);
                m_cache(i, j) = (even_r == even_c) ? std::cos(angle) : (even_r ? -std::sin(angle) : std::sin(angle));
            }
        m_enable_rows = std::max(m_enable_rows, R);
        m_enable_cols = std::max(m_enable_cols, Cn);
    }
    mat_view_t<mat_t<val_type>> range(int row_beg, int row_num, int col_beg, int col_num) {
        if (row_beg + row_num >= m_enable_rows || col_beg + col_num >= m_enable_cols) init(row_beg, row_num, col_beg, col_num);
        return m_cache.range(row_beg, col_beg, row_num, col_num);
    }
    // the 2x2 rotation block of (pair i, position m)
    mat_view_t<mat_t<val_type>> forward_unite(int const& i, int const& m) { return range(i * 2, 2, m * 2, 2); }
};

template <typename input_type>
class RoPE_net_t {
    using val_type = typename input_type::ele_type;
    int m_d;
    std::shared_ptr<jsm_rt::device_buffer> m_table;  // [positions][d/2][cosA, sinA, cosB, sinB]
    int m_table_pos = 0;

    void need_table(int positions) {
        if (m_table && positions <= m_table_pos) return;
        const int cap = std::max(positions, m_table_pos + 1024);  // grows like the reference's cache (+1024)
        m_table = std::make_shared<jsm_rt::device_buffer>((size_t)cap * (m_d / 2) * 4 * sizeof(float));
        jsm_rt::check(jsm_rope_table(static_cast<float*>(m_table->p), 0, m_d, 10000.0f, cap, jsm_rt::stream()));
        m_table_pos = cap;
    }

public:
    RoPE_net_t(int const& d_model) : m_d(d_model) {}
    void set_param(int const& d_model) { m_d = d_model; m_table.reset(); m_table_pos = 0; }

    // x: [d_model, seq_len]; every pair of rows (2i, 2i+1) of column m is rotated by the block of (i, m)
    mat_t<val_type> forward(input_type const& x) { return forward(x, 0); }
    // the same for columns that sit at positions first_position, first_position + 1, ... of a longer sequence (generation
    // with cached keys and values feeds the new columns only); not in the reference, whose columns always start at 0
    mat_t<val_type> forward(input_type const& x, int first_position) {
        const int seq_len = x.col_num(), d_model = x.row_num();
        if (d_model != m_d) throw std::runtime_error("Input dimension does not match RoPE dimension");
        need_table(first_position + seq_len);
        mat_t<val_type> xt = x.view().t().clone();  // token-major: the pair of a token is adjacent in memory
        mat_t<val_type> yt(seq_len, d_model);
        std::shared_ptr<jsm_rt::device_buffer> pos;
        if (first_position != 0) {
            std::vector<int32_t> h(seq_len);
            for (int i = 0; i < seq_len; ++i) h[i] = first_position + i;
            pos = std::make_shared<jsm_rt::device_buffer>(sizeof(int32_t) * (size_t)seq_len);
            jsm_rt::check(jsm_upload(pos->p, h.data(), sizeof(int32_t) * (size_t)seq_len, jsm_rt::stream()));
            jsm_rt::check(jsm_stream_sync(jsm_rt::stream()));  // h leaves scope
        }
        jsm_rt::check(jsm_rope_apply(xt.jsm_device().data, yt.jsm_device_out().data, JSM_F32, static_cast<const float*>(m_table->p), d_model, 1,
                                     pos ? static_cast<const int32_t*>(pos->p) : nullptr, seq_len, jsm_rt::stream()));
        if (pos) jsm_rt::check(jsm_stream_sync(jsm_rt::stream()));  // the position buffer is released on return
        return yt.t().clone();
    }
    template <typename>
    void init_weight() {}
    void step() {}
    std::string net_type(int const& indent = 0) const {
        std::stringstream ss;
        ss << print_indent(indent) << "RoPE_net_t:(d_model:" << m_d << ")";
        return ss.str();
    }
};

#endif
