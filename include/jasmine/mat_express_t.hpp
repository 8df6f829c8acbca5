// Expression layer of the jasmine API (reference: mat_express_t.hpp): lazy element-wise nodes built by
// the operators + - * / > < and exp / sigmoid, eager reductions (sum vsum hsum vmean hmean mean max hmax),
// pow, sqrt, softmax, hsoftmax, the lazy dot product and the in-place +=.
//
// The reference evaluates a node by pulling one element at a time through the tree on the CPU
// (mat_express_t.hpp:66-71, 96-107).  Here a node lowers itself to a postfix program; materialising it
// (clone(), conversion to mat_t, or the first element access) runs ONE fused kernel of libjasmine_b200 over
// the whole result.  Result shape = max of the operand shapes with modulo broadcast (:51-59), element type =
// common type of the operands (:44), exactly as in the reference; the device arithmetic is fp32, so a
// double-typed expression is computed in fp32 and widened.
#ifndef JASMINE_B200_MAT_EXPRESS_T_HPP_
#define JASMINE_B200_MAT_EXPRESS_T_HPP_
#include <algorithm>
#include <cmath>
#include <limits>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>

#include "mat_concepts.hpp"
#include "mat_view_t.hpp"

namespace jsm_expr {

template <typename T, bool = std::is_arithmetic_v<T>>
struct ele_of { using type = T; };
template <typename T>
struct ele_of<T, false> { using type = typename std::decay_t<T>::ele_type; };
template <typename T>
using ele_of_t = typename ele_of<std::decay_t<T>>::type;

// operands are held like in the reference (storage_selector, mat_express_t.hpp:18-33):
// scalars by value, matrices and nodes by reference (valid within the enclosing full-expression)
template <typename T>
using held_t = std::conditional_t<std::is_arithmetic_v<T>, T, T const&>;

template <typename T>
int rows_of(const T& x) { if constexpr (std::is_arithmetic_v<T>) return 1; else return x.row_num(); }
template <typename T>
int cols_of(const T& x) { if constexpr (std::is_arithmetic_v<T>) return 1; else return x.col_num(); }

template <typename T>
concept lowers_itself = requires(const T& x, jsm_rt::builder& b) { x.jsm_lower(b); };

// any matrix-like value as a float matrix on the device (element-wise conversion for non-float storage)
template <typename T>
std::shared_ptr<mat_t<float>> to_float_matrix(const T& x) {
    auto m = std::make_shared<mat_t<float>>(x.row_num(), x.col_num());
    for (int i = 0; i < x.row_num(); ++i)
        for (int j = 0; j < x.col_num(); ++j) (*m)(i, j) = static_cast<float>(x(i, j));
    return m;
}

template <typename T>
void lower(jsm_rt::builder& b, const T& x) {
    if constexpr (std::is_arithmetic_v<T>) {
        b.imm(static_cast<float>(x));
    } else if constexpr (lowers_itself<T>) {
        x.jsm_lower(b);
    } else {
        auto tmp = to_float_matrix(x);
        b.keep.push_back(tmp);
        tmp->jsm_lower(b);
    }
}

template <typename out_ele>
mat_t<out_ele> finish(mat_t<float>&& r) {
    if constexpr (std::is_same_v<out_ele, float>) return std::move(r);
    else return mat_t<out_ele>(r);
}

// one fused kernel over the whole result
template <typename E>
mat_t<float> evaluate(const E& e) {
    jsm_rt::builder b;
    lower(b, e);
    mat_t<float> out(rows_of(e), cols_of(e));
    if (out.row_num() > 0 && out.col_num() > 0)
        jsm_rt::check(jsm_eval_elementwise(b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), out.jsm_device_out(), jsm_rt::stream()));
    return out;
}

// reduction / normalisation of the value of an expression along one axis
template <typename E>
mat_t<float> along_axis(int kind, int axis, const E& e, const float* gain = nullptr, const float* bias = nullptr, float eps = 0.0f) {
    jsm_rt::builder b;
    lower(b, e);
    const int R = rows_of(e), C = cols_of(e);
    const bool reduces = kind <= JSM_ROWS_ARGMAX;
    mat_t<float> out(reduces ? (axis == 1 ? R : 1) : R, reduces ? (axis == 1 ? 1 : C) : C);
    if (R > 0 && C > 0)
        jsm_rt::check(jsm_eval_rows(kind, axis, b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), gain, bias, eps, out.jsm_device_out(), jsm_rt::stream()));
    return out;
}

template <typename E>
float whole(int kind, const E& e) {
    jsm_rt::builder b;
    lower(b, e);
    mat_t<float> out(1, 1);
    jsm_rt::check(jsm_eval_full(kind, b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), out.jsm_device_out(), jsm_rt::stream()));
    return out(0, 0);
}

// matrix operand of a contraction: a strided device window (no copy for mat_t / views of float)
template <typename T>
jsm_mat operand(const T& x, std::vector<std::shared_ptr<void>>& keep) {
    if constexpr (requires { x.jsm_device(); }) {
        return x.jsm_device();
    } else if constexpr (lowers_itself<T>) {
        auto tmp = std::make_shared<mat_t<float>>(evaluate(x));
        keep.push_back(tmp);
        return tmp->jsm_device();
    } else {
        auto tmp = to_float_matrix(x);
        keep.push_back(tmp);
        return tmp->jsm_device();
    }
}

}  // namespace jsm_expr

template <typename lval_type, typename rval_type>
requires is_matrix<lval_type> && is_matrix<rval_type>
auto dot(lval_type const& lval, rval_type const& rval);

// ---- binary nodes -------------------------------------------------------------------------------
template <typename lval_type, typename rval_type, template <typename, typename> class tpl>
class mat_express_2_param_stable_t {
public:
    using lval_base_type = jsm_expr::ele_of_t<lval_type>;
    using rval_base_type = jsm_expr::ele_of_t<rval_type>;
    using derived_type = tpl<lval_type, rval_type>;
    using ele_type = std::common_type_t<lval_base_type, rval_base_type>;

    mat_express_2_param_stable_t(lval_type const& left, rval_type const& right) : m_left(left), m_right(right) {}

    int row_num() const { return std::max(jsm_expr::rows_of(m_left), jsm_expr::rows_of(m_right)); }
    int col_num() const { return std::max(jsm_expr::cols_of(m_left), jsm_expr::cols_of(m_right)); }
    std::tuple<int, int> shape() const { return std::make_tuple(row_num(), col_num()); }

    // element access materialises the node once (one kernel) and reads from the result
    ele_type operator()(int i, int j) const {
        if (!m_value) m_value = std::make_shared<mat_t<float>>(jsm_expr::evaluate(*this));
        return static_cast<ele_type>((*m_value)(i, j));
    }
    std::string to_string() const {
        std::stringstream ss;
        ss << derived_type::type_name() << "(" << row_num() << ", " << col_num() << ")";
        for (int i = 0; i < row_num(); ++i) {
            ss << "\n[ ";
            for (int j = 0; j < col_num(); ++j) ss << (*this)(i, j) << " ";
            ss << " ]";
        }
        return ss.str();
    }
    template <typename other_type>
    auto dot(const other_type& m) const { return ::dot(*static_cast<derived_type const*>(this), m); }

    mat_t<ele_type> clone() const { return jsm_expr::finish<ele_type>(jsm_expr::evaluate(*this)); }
    operator mat_t<ele_type>() const { return clone(); }

    void jsm_lower(jsm_rt::builder& b) const {
        jsm_expr::lower(b, m_left);
        jsm_expr::lower(b, m_right);
        b.op(derived_type::opcode);
    }

protected:
    jsm_expr::held_t<lval_type> m_left;
    jsm_expr::held_t<rval_type> m_right;
    mutable std::shared_ptr<mat_t<float>> m_value;
};

#define JSM_BINARY_NODE(NAME, OPCODE, SYMBOL)                                                             \
    template <typename lval_type, typename rval_type>                                                     \
    class NAME : public mat_express_2_param_stable_t<lval_type, rval_type, NAME> {                        \
    public:                                                                                               \
        using base_type = mat_express_2_param_stable_t<lval_type, rval_type, NAME>;                       \
        using ele_type = typename base_type::ele_type;                                                    \
        static constexpr int opcode = OPCODE;                                                             \
        NAME(lval_type const& left, rval_type const& right) : base_type(left, right) {}                   \
        static std::string type_name() { return #NAME; }                                                  \
    };                                                                                                    \
    template <typename lval_type, typename rval_type>                                                     \
    requires is_caculable<lval_type, rval_type> && (is_matrix<lval_type> || is_matrix<rval_type>)         \
    auto operator SYMBOL(lval_type const& left, rval_type const& right) {                                 \
        return NAME<lval_type, rval_type>(left, right);                                                   \
    }
JSM_BINARY_NODE(mat_greater_t, JSM_OP_GT, >)
JSM_BINARY_NODE(mat_less_t, JSM_OP_LT, <)
JSM_BINARY_NODE(mat_add_t, JSM_OP_ADD, +)
JSM_BINARY_NODE(mat_sub_t, JSM_OP_SUB, -)
JSM_BINARY_NODE(mat_mul_t, JSM_OP_MUL, *)
JSM_BINARY_NODE(mat_div_t, JSM_OP_DIV, /)
#undef JSM_BINARY_NODE

// in-place accumulation (reference: mat_express_t.hpp:225-251): one kernel writing into `left`
template <typename lval_type, typename rval_type>
requires is_matrix<lval_type> && (is_matrix<rval_type> || std::is_arithmetic_v<rval_type>)
decltype(auto) operator+=(lval_type& left, rval_type const& right) {
    jsm_rt::builder b;
    jsm_expr::lower(b, left);
    jsm_expr::lower(b, right);
    b.op(JSM_OP_ADD);
    // the program reads the operands at the result's own indices: shape of the left side
    jsm_mat out = left.jsm_device_inout();
    jsm_rt::check(jsm_eval_elementwise(b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), out, jsm_rt::stream()));
    return left;
}

// ---- unary nodes -----------------------------------------------------------------------------------
template <typename val_type, template <typename> class tpl>
class mat_express_1_param_stable_t {
public:
    using derived_type = tpl<val_type>;
    using val_base_type = jsm_expr::ele_of_t<val_type>;
    using ele_type = val_base_type;

    mat_express_1_param_stable_t(val_type const& val) : m_val(val) {}
    int row_num() const { return m_val.row_num(); }
    int col_num() const { return m_val.col_num(); }
    std::tuple<int, int> shape() const { return std::make_tuple(row_num(), col_num()); }
    ele_type operator()(int i, int j) const {
        if (!m_value) m_value = std::make_shared<mat_t<float>>(jsm_expr::evaluate(*static_cast<derived_type const*>(this)));
        return static_cast<ele_type>((*m_value)(i, j));
    }
    std::string to_string() const {
        std::stringstream ss;
        ss << derived_type::type_name() << "(" << row_num() << ", " << col_num() << ")";
        for (int i = 0; i < row_num(); ++i) {
            ss << "\n[ ";
            for (int j = 0; j < col_num(); ++j) ss << (*this)(i, j) << " ";
            ss << " ]";
        }
        return ss.str();
    }
    template <typename other_type>
    auto dot(const other_type& m) const { return ::dot(*static_cast<derived_type const*>(this), m); }
    mat_t<ele_type> clone() const { return jsm_expr::finish<ele_type>(jsm_expr::evaluate(*static_cast<derived_type const*>(this))); }
    operator mat_t<ele_type>() const { return clone(); }

protected:
    val_type const& m_val;
    mutable std::shared_ptr<mat_t<float>> m_value;
};

template <typename val_type>
class mat_exp_t : public mat_express_1_param_stable_t<val_type, mat_exp_t> {
public:
    using base_type = mat_express_1_param_stable_t<val_type, mat_exp_t>;
    using ele_type = typename base_type::ele_type;
    mat_exp_t(val_type const& val) : base_type(val) {}
    static std::string type_name() { return "mat_exp_t"; }
    void jsm_lower(jsm_rt::builder& b) const { jsm_expr::lower(b, this->m_val); b.op(JSM_OP_EXP); }
};
template <typename val_type>
requires is_matrix<val_type>
auto exp(val_type const& val) { return mat_exp_t<val_type>(val); }

template <typename val_type>
requires std::is_arithmetic_v<val_type>
val_type sigmoid(val_type const& val) { return static_cast<val_type>(1.0 / (1.0 + std::exp(-val))); }

template <typename val_type>
requires is_matrix<val_type>
class mat_sigmoid_t : public mat_express_1_param_stable_t<val_type, mat_sigmoid_t> {
public:
    using base_type = mat_express_1_param_stable_t<val_type, mat_sigmoid_t>;
    using ele_type = typename base_type::ele_type;
    mat_sigmoid_t(val_type const& val) : base_type(val) {}
    static std::string type_name() { return "mat_sigmoid_t"; }
    void jsm_lower(jsm_rt::builder& b) const { jsm_expr::lower(b, this->m_val); b.op(JSM_OP_SIGMOID); }
};
template <typename val_type>
requires is_matrix<val_type>
auto sigmoid(val_type const& val) { return mat_sigmoid_t<val_type>(val); }

// ---- eager reductions (reference: mat_express_t.hpp:511-628): one kernel each --------------------------
template <typename val_type>
requires std::is_arithmetic_v<val_type>
auto sum(val_type const& val) { return val; }

template <typename val_type>
requires is_matrix<val_type>
auto sum(val_type const& val) { return static_cast<typename val_type::ele_type>(jsm_expr::whole(JSM_ROWS_SUM, val)); }

template <typename val_type>
requires is_matrix<val_type>
auto vsum(val_type const& val) { return jsm_expr::finish<typename val_type::ele_type>(jsm_expr::along_axis(JSM_ROWS_SUM, 0, val)); }

template <typename val_type>
requires is_matrix<val_type>
auto hsum(val_type const& val) { return jsm_expr::finish<typename val_type::ele_type>(jsm_expr::along_axis(JSM_ROWS_SUM, 1, val)); }

template <typename val_type>
requires is_matrix<val_type>
auto vmean(val_type const& val) { return jsm_expr::finish<typename val_type::ele_type>(jsm_expr::along_axis(JSM_ROWS_MEAN, 0, val)); }

template <typename val_type>
requires is_matrix<val_type>
auto hmean(val_type const& val) { return jsm_expr::finish<typename val_type::ele_type>(jsm_expr::along_axis(JSM_ROWS_MEAN, 1, val)); }

template <typename val_type>
requires is_matrix<val_type>
auto mean(val_type const& val) { return static_cast<typename val_type::ele_type>(jsm_expr::whole(JSM_ROWS_MEAN, val)); }

template <typename input_type>
requires is_matrix<input_type>
auto pow(input_type const& val, double const p = 2.) {
    jsm_rt::builder b;
    jsm_expr::lower(b, val);
    b.op(JSM_OP_POW, (float)p);
    mat_t<float> out(val.row_num(), val.col_num());
    jsm_rt::check(jsm_eval_elementwise(b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), out.jsm_device_out(), jsm_rt::stream()));
    return jsm_expr::finish<typename std::decay_t<input_type>::ele_type>(std::move(out));
}

template <typename input_type>
requires is_matrix<input_type>
auto max(input_type const& val) { return static_cast<typename input_type::ele_type>(jsm_expr::whole(JSM_ROWS_MAX, val)); }

template <typename input_type>
requires is_matrix<input_type>
auto hmax(input_type const& val) { return jsm_expr::finish<typename input_type::ele_type>(jsm_expr::along_axis(JSM_ROWS_MAX, 1, val)); }

template <typename val_type>
requires is_matrix<val_type>
auto sqrt(val_type const& val) {
    jsm_rt::builder b;
    jsm_expr::lower(b, val);
    b.op(JSM_OP_SQRT);
    mat_t<float> out(val.row_num(), val.col_num());
    jsm_rt::check(jsm_eval_elementwise(b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), out.jsm_device_out(), jsm_rt::stream()));
    return jsm_expr::finish<typename val_type::ele_type>(std::move(out));
}

// ---- whole-matrix softmax (reference: mat_softmax_t, mat_express_t.hpp:630-679) ---------------------------
// global maximum and global sum of exp(x - max), computed when the node is built
template <typename val_type>
class mat_softmax_t {
public:
    using ele_type = typename val_type::ele_type;
    mat_softmax_t(val_type const& val) : m_val(val) { reset(); }
    void reset() {
        jsm_rt::builder b;
        jsm_expr::lower(b, m_val);
        m_value = std::make_shared<mat_t<float>>(m_val.row_num(), m_val.col_num());
        jsm_rt::check(jsm_eval_full(JSM_ROWS_SOFTMAX, b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), m_value->jsm_device_out(), jsm_rt::stream()));
    }
    int row_num() const { return m_val.row_num(); }
    int col_num() const { return m_val.col_num(); }
    std::tuple<int, int> shape() const { return std::make_tuple(row_num(), col_num()); }
    ele_type operator()(int i, int j) const { return static_cast<ele_type>((*m_value)(i, j)); }
    mat_t<ele_type> clone() const { return jsm_expr::finish<ele_type>(mat_t<float>(*m_value)); }
    operator mat_t<ele_type>() const { return clone(); }
    static std::string type_name() { return "mat_softmax_t"; }
    void jsm_lower(jsm_rt::builder& b) const { b.keep.push_back(m_value); m_value->jsm_lower(b); }

private:
    val_type const& m_val;
    std::shared_ptr<mat_t<float>> m_value;
};
template <typename val_type>
requires std::is_arithmetic_v<val_type>
auto softmax(val_type const&) { return static_cast<val_type>(1.); }
template <typename val_type>
requires is_matrix<val_type>
auto softmax(val_type const& val) { return mat_softmax_t<val_type>(val); }

// per-row softmax (reference: hsoftmax, mat_express_t.hpp:681-694): the argument expression is fused in
template <typename input_type>
auto hsoftmax(const input_type& input) {
    return jsm_expr::finish<typename std::decay_t<input_type>::ele_type>(jsm_expr::along_axis(JSM_ROWS_SOFTMAX, 1, input));
}

// ---- dot (reference: mat_dot_t, mat_express_t.hpp:696-802) ---------------------------------------------------
template <typename lval_type, typename rval_type>
requires is_matrix<lval_type> && is_matrix<rval_type>
class mat_dot_t {
public:
    using ele_type = std::common_type_t<typename lval_type::ele_type, typename rval_type::ele_type>;
    mat_dot_t(lval_type const& lval, rval_type const& rval) : m_lval(lval), m_rval(rval) {
        if (lval.col_num() != rval.row_num()) throw std::invalid_argument("mat_dot_t: inner dimensions do not match for dot product");
    }
    int row_num() const { return m_lval.row_num(); }
    int col_num() const { return m_rval.col_num(); }
    std::tuple<int, int> shape() const { return std::make_tuple(row_num(), col_num()); }
    ele_type operator()(int i, int j) const { return static_cast<ele_type>(value()(i, j)); }
    template <typename other_type>
    auto dot(const other_type& m) const { return ::dot(*this, m); }
    std::string to_string() const {
        std::stringstream ss;
        ss << "mat_dot_t(" << row_num() << ", " << col_num() << ")";
        for (int i = 0; i < row_num(); ++i) {
            ss << "\n[ ";
            for (int j = 0; j < col_num(); ++j) ss << (*this)(i, j) << " ";
            ss << " ]";
        }
        return ss.str();
    }
    mat_t<ele_type> clone() const { return jsm_expr::finish<ele_type>(mat_t<float>(value())); }
    operator mat_t<ele_type>() const { return clone(); }
    // inside a larger expression the product is computed once and enters as an operand
    void jsm_lower(jsm_rt::builder& b) const { b.keep.push_back(m_value_ptr()); m_value_ptr()->jsm_lower(b); }

private:
    const mat_t<float>& value() const { return *m_value_ptr(); }
    std::shared_ptr<mat_t<float>> m_value_ptr() const {
        if (!m_value) {
            std::vector<std::shared_ptr<void>> keep;
            jsm_mat A = jsm_expr::operand(m_lval, keep), B = jsm_expr::operand(m_rval, keep);
            m_value = std::make_shared<mat_t<float>>(row_num(), col_num());
            if (row_num() > 0 && col_num() > 0)
                jsm_rt::check(jsm_dot_f32(A, B, nullptr, 0, nullptr, m_value->jsm_device_out(), jsm_rt::stream()));
        }
        return m_value;
    }
    lval_type const& m_lval;
    rval_type const& m_rval;
    mutable std::shared_ptr<mat_t<float>> m_value;
};

template <typename lval_type, typename rval_type>
requires is_matrix<lval_type> && is_matrix<rval_type>
auto dot(lval_type const& lval, rval_type const& rval) {
    return mat_dot_t<lval_type, rval_type>(lval, rval);
}

template <typename val_type>
requires std::is_arithmetic_v<val_type>
template <typename other_type>
requires is_matrix<other_type>
auto mat_t<val_type>::dot(const other_type& m) const { return ::dot(*this, m); }

template <typename agent_type>
template <typename other_type>
requires is_matrix<other_type>
auto mat_view_t<agent_type>::dot(const other_type& m) const { return ::dot(*this, m); }

// ---- view members that need the evaluator ---------------------------------------------------------------------
template <typename agent_type>
mat_t<typename mat_view_t<agent_type>::val_type> mat_view_t<agent_type>::clone() const {
    if constexpr (std::is_same_v<val_type, float>) {
        return jsm_expr::evaluate(*this);
    } else {
        mat_t<val_type> m(row_num(), col_num());
        for (int i = 0; i < row_num(); ++i)
            for (int j = 0; j < col_num(); ++j) m(i, j) = (*this)(i, j);
        return m;
    }
}

template <typename agent_type>
template <typename other_type>
void mat_view_t<agent_type>::assign(const other_type& other) {
    if constexpr (std::is_same_v<val_type, float>) {
        jsm_rt::builder b;
        jsm_expr::lower(b, other);
        // the window is written at its own indices; `other` must have the window's shape
        jsm_mat self = jsm_device_inout();
        jsm_rt::check(jsm_eval_elementwise(b.prog.data(), (int)b.prog.size(), b.leaves.data(), (int)b.leaves.size(), self, jsm_rt::stream()));
    } else {
        for (int i = 0; i < row_num(); ++i)
            for (int j = 0; j < col_num(); ++j) (*this)(i, j) = other(i, j);
    }
}

#endif
