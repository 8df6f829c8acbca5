// mat_t: the owning dense matrix of the jasmine API (reference: mat_t.hpp:15-381) with a device mirror.
//
// Same public members as the reference (constructors, shape, modulo-broadcast element access, views,
// transpose, clone, dot).  Storage differs: a host mirror for element access and, for float matrices,
// a buffer in GPU memory that the kernels of libjasmine_b200 read and write.  The two copies are
// synchronised lazily: an element write marks the device copy stale, a kernel result marks the host
// copy stale, and whichever side is needed next is refreshed with one transfer.
#ifndef JASMINE_B200_MAT_T_HPP_
#define JASMINE_B200_MAT_T_HPP_
#include <algorithm>
#include <initializer_list>
#include <sstream>
#include <string>
#include <tuple>
#include <type_traits>
#include <vector>

#include "jsm_runtime.hpp"
#include "mat_utility.hpp"

template <typename agent_type>
class mat_view_t;

template <typename val_type>
requires std::is_arithmetic_v<val_type>
class mat_t {
    template <typename U>
    requires std::is_arithmetic_v<U>
    friend class mat_t;

public:
    using ele_type = val_type;
    static constexpr bool on_device = std::is_same_v<val_type, float>;

private:
    int m_rows = 0, m_cols = 0;
    bool m_row_first = true;
    bool m_scalar = false;
    mutable std::vector<val_type> m_host;
    mutable std::shared_ptr<jsm_rt::device_buffer> m_dev;
    mutable bool m_host_valid = true, m_dev_valid = false;

    size_t count() const noexcept { return (size_t)m_rows * (size_t)m_cols; }
    size_t index(int r, int c) const noexcept {
        const int i = r % m_rows, j = c % m_cols;  // modulo broadcast (reference: mat_t.hpp:302-320)
        return m_row_first ? (size_t)i * m_cols + j : (size_t)j * m_rows + i;
    }
    void init(int rows, int cols, bool row_first) {
        m_rows = rows; m_cols = cols; m_row_first = row_first;
        m_scalar = (rows == 1 && cols == 1);
        m_host.assign(count(), val_type{});  // zero-filled like the reference (mat_t.hpp:53-69)
        m_dev.reset();
        m_host_valid = true; m_dev_valid = false;
    }
    void need_host() const {
        if (m_host_valid) return;
        if constexpr (on_device) {
            m_host.resize(count());
            if (count()) jsm_rt::check(jsm_download(m_host.data(), m_dev->p, count() * sizeof(val_type), jsm_rt::stream()));
        }
        m_host_valid = true;
    }

public:
    mat_t() noexcept {}
    mat_t(const ele_type& val) { init(1, 1, true); m_host[0] = val; }
    mat_t(int rows, int cols, bool row_first = true) { init(rows, cols, row_first); }
    mat_t(const int& rows, const int& cols, std::initializer_list<val_type> l) {
        init(rows, cols, true);
        std::copy_n(l.begin(), std::min(l.size(), m_host.size()), m_host.begin());
    }
    mat_t(const mat_t& m) { *this = m; }
    mat_t(mat_t&& m) noexcept { *this = std::move(m); }
    template <typename other>
    requires std::is_convertible_v<other, val_type>
    mat_t(const mat_t<other>& m) { *this = m; }

    mat_t& operator=(const mat_t& m) {
        if (this == &m) return *this;
        m_rows = m.m_rows; m_cols = m.m_cols; m_row_first = m.m_row_first; m_scalar = m.m_scalar;
        bool copied = false;
        if constexpr (on_device) {
            if (!m.m_host_valid) {  // deep copy on the device: the source's newest data lives there
                copy_on_device(m);
                copied = true;
            }
        }
        if (!copied) {
            m_host = m.m_host;
            m_host_valid = true; m_dev_valid = false; m_dev.reset();
        }
        return *this;
    }

private:
    void copy_on_device(const mat_t& m) requires on_device {
        {
            jsm_mat src = m.jsm_device();
            m_host.clear();
            m_dev = std::make_shared<jsm_rt::device_buffer>(count() * sizeof(val_type));
            jsm_instr ins{JSM_OP_LEAF, 0, 0.0f};
            jsm_mat dst = src;
            dst.data = m_dev->p;
            jsm_rt::check(jsm_eval_elementwise(&ins, 1, &src, 1, dst, jsm_rt::stream()));
            m_host_valid = false; m_dev_valid = true;
        }
    }

public:
    mat_t& operator=(mat_t&& m) noexcept {
        if (this == &m) return *this;
        m_rows = m.m_rows; m_cols = m.m_cols; m_row_first = m.m_row_first; m_scalar = m.m_scalar;
        m_host = std::move(m.m_host); m_dev = std::move(m.m_dev);
        m_host_valid = m.m_host_valid; m_dev_valid = m.m_dev_valid;
        m.m_rows = m.m_cols = 0; m.m_host.clear(); m.m_dev.reset(); m.m_host_valid = true; m.m_dev_valid = false;
        return *this;
    }
    template <typename other>
    requires std::is_convertible_v<other, val_type> && (!std::is_same_v<other, val_type>)
    mat_t& operator=(const mat_t<other>& m) {
        m.need_host();
        init(m.m_rows, m.m_cols, m.m_row_first);
        for (size_t i = 0; i < m_host.size(); ++i) m_host[i] = static_cast<val_type>(m.m_host[i]);
        return *this;
    }
    // fill with a scalar (reference: mat_t.hpp:162-174)
    template <typename scalar_type>
    requires std::is_arithmetic_v<scalar_type>
    mat_t& operator=(scalar_type s) {
        m_host.assign(count(), static_cast<val_type>(s));
        m_host_valid = true; m_dev_valid = false;
        return *this;
    }

    bool is_scalar() const noexcept { return m_scalar; }
    int row_num() const noexcept { return m_rows; }
    int col_num() const noexcept { return m_cols; }
    std::tuple<int, int> shape() const noexcept { return std::make_tuple(m_rows, m_cols); }
    bool valid() const noexcept { return count() > 0; }

    // like the reference (mat_t.hpp:280-300): storage is replaced only when the element count changes
    void reshape(int rows, int cols) {
        if (rows == 1 && cols == 1) {
            if (!m_scalar) {
                val_type v = count() ? (*this)(0, 0) : val_type{};
                init(1, 1, true);
                m_host[0] = v;
            }
        } else if ((size_t)rows * (size_t)cols != count()) {
            init(rows, cols, true);
        }
    }

    val_type& operator()(int r, int c) {
        need_host();
        m_dev_valid = false;
        return m_host[index(r, c)];
    }
    const val_type& operator()(int r, int c) const {
        need_host();
        return m_host[index(r, c)];
    }

    std::string to_string() const {
        std::stringstream ss;
        ss << "matrix(" << m_rows << ", " << m_cols << ")";
        for (int i = 0; i < m_rows; ++i) {
            ss << "\n[ ";
            for (int j = 0; j < m_cols; ++j) ss << (*this)(i, j) << " ";
            ss << "]";
        }
        return ss.str();
    }

    mat_view_t<mat_t<val_type>> t() noexcept;
    mat_view_t<mat_t<val_type>> view(int const& row_offset = 0, int const& col_offset = 0, int const& row_size = -1, int const& col_size = -1) noexcept;
    mat_view_t<const mat_t<val_type>> view(int const& row_offset = 0, int const& col_offset = 0, int const& row_size = -1, int const& col_size = -1) const noexcept;
    mat_view_t<mat_t<val_type>> col(int const& idx) noexcept;
    mat_view_t<const mat_t<val_type>> col(int const& idx) const noexcept;
    mat_view_t<mat_t<val_type>> row(int const& idx) noexcept;
    mat_view_t<const mat_t<val_type>> row(int const& idx) const noexcept;
    mat_view_t<mat_t<val_type>> back_col() noexcept;
    mat_view_t<const mat_t<val_type>> back_col() const noexcept;
    mat_view_t<mat_t<val_type>> back_row() noexcept;
    mat_view_t<const mat_t<val_type>> back_row() const noexcept;
    mat_view_t<mat_t<val_type>> front_col() noexcept;
    mat_view_t<const mat_t<val_type>> front_col() const noexcept;
    mat_view_t<mat_t<val_type>> front_row() noexcept;
    mat_view_t<const mat_t<val_type>> front_row() const noexcept;

    // in-place transpose (reference: mat_t.hpp:359-371); the logical shape flips, the layout becomes row-major
    mat_t& t_() {
        mat_t out(m_cols, m_rows);
        for (int i = 0; i < m_rows; ++i)
            for (int j = 0; j < m_cols; ++j) out(j, i) = (*this)(i, j);
        *this = std::move(out);
        return *this;
    }
    mat_t clone() const { return mat_t(*this); }

    template <typename other_type>
    requires is_matrix<other_type>
    auto dot(const other_type& m) const;

    // ---- device side (not in the reference) -------------------------------------------------
    // Descriptor of the up-to-date device copy (uploads the host mirror when it is newer).
    jsm_mat jsm_device() const requires on_device {
        if (!m_dev) m_dev = std::make_shared<jsm_rt::device_buffer>(std::max<size_t>(count(), 1) * sizeof(val_type));
        if (!m_dev_valid) {
            if (count()) jsm_rt::check(jsm_upload(m_dev->p, m_host.data(), count() * sizeof(val_type), jsm_rt::stream()));
            m_dev_valid = true;
        }
        return jsm_mat{m_dev->p, m_rows, m_cols, m_row_first ? (int64_t)m_cols : 1, m_row_first ? 1 : (int64_t)m_rows, JSM_F32};
    }
    // Descriptor for a kernel that overwrites the whole matrix: the host mirror becomes stale.
    jsm_mat jsm_device_out() requires on_device {
        if (!m_dev) m_dev = std::make_shared<jsm_rt::device_buffer>(std::max<size_t>(count(), 1) * sizeof(val_type));
        m_dev_valid = true; m_host_valid = false;
        return jsm_mat{m_dev->p, m_rows, m_cols, m_row_first ? (int64_t)m_cols : 1, m_row_first ? 1 : (int64_t)m_rows, JSM_F32};
    }
    // Descriptor for a kernel that overwrites a part: current contents are kept (uploaded first if needed).
    jsm_mat jsm_device_inout() requires on_device {
        jsm_mat m = jsm_device();
        m_host_valid = false;
        return m;
    }
    std::shared_ptr<jsm_rt::device_buffer> jsm_keepalive() const { return m_dev; }
    void jsm_lower(jsm_rt::builder& b) const requires on_device {
        b.leaf(jsm_device());
        b.keep.push_back(m_dev);
    }
};

#endif
