// Optimisers of the jasmine API (reference: mat_updator_t.hpp:9-170): plain gradient descent, Adam and Nesterov-Adam.
// update(grad, mat) changes `mat` in place; the arithmetic is the reference's formula written with the same matrix
// expressions, which here run as fused element-wise kernels on the device copy of the weights (float throughout: the
// reference promotes the beta2 / epsilon terms to double, the results agree to float rounding).
#ifndef JASMINE_B200_MAT_UPDATOR_T_HPP_
#define JASMINE_B200_MAT_UPDATOR_T_HPP_
#include "mat_express_t.hpp"
#include "mat_t.hpp"

template <typename val_type>
class sgd_t {
    val_type m_learning_rate;

public:
    sgd_t(val_type learning_rate = val_type(0.001)) : m_learning_rate(learning_rate) {}
    void set(val_type learning_rate = val_type(0.001)) { m_learning_rate = learning_rate; }
    void set_lr(val_type lr) { m_learning_rate = lr; }
    val_type lr() const { return m_learning_rate; }
    // mat = mat - lr * grad (reference: :31-34)
    void update(const mat_t<val_type>& grad, mat_t<val_type>& mat) { mat = (mat - m_learning_rate * grad).clone(); }
    void step() {}
};

namespace jsm_opt {
// first and second moment estimates shared by adam_t and nadam_t (reference: :78-92, :150-164)
template <typename val_type>
struct moments {
    mat_t<val_type> m, v;
    val_type beta1, beta1_t, beta2, beta2_t, lr, eps;
    int t = 0;
    void set(val_type learning_rate, val_type b1, double b2, double epsilon, bool reset_powers) {
        beta1 = b1; beta2 = (val_type)b2; lr = learning_rate; eps = (val_type)epsilon; t = 0;
        if (reset_powers) { beta1_t = 1; beta2_t = 1; }
    }
    void accumulate(const mat_t<val_type>& grad) {
        ++t;
        if (!m.valid()) {
            m = mat_t<val_type>(grad.row_num(), grad.col_num());
            v = mat_t<val_type>(grad.row_num(), grad.col_num());
        }
        m = (beta1 * m + (1 - beta1) * grad).clone();
        v = (beta2 * v + (1 - beta2) * grad * grad).clone();
        beta1_t *= beta1;
        beta2_t *= beta2;
    }
};
}  // namespace jsm_opt

template <typename val_type>
class adam_t {
    jsm_opt::moments<val_type> s;

public:
    adam_t(val_type learning_rate = val_type(0.001), val_type beta1 = val_type(0.9), double beta2 = 0.999, double epsilon = 1e-8) {
        s.beta1_t = 1; s.beta2_t = 1;
        s.set(learning_rate, beta1, beta2, epsilon, true);
    }
    void set(val_type learning_rate = val_type(0.001), val_type beta1 = val_type(0.9), double beta2 = 0.999, double epsilon = 1e-8) {
        s.set(learning_rate, beta1, beta2, epsilon, true);
    }
    void set_lr(val_type lr) { s.lr = lr; }
    // reference: :76-95
    void update(const mat_t<val_type>& grad, mat_t<val_type>& mat) {
        s.accumulate(grad);
        mat_t<val_type> m_hat = (s.m / (1 - s.beta1_t)).clone();
        mat_t<val_type> v_hat = (s.v / (1 - s.beta2_t)).clone();
        mat = (mat - s.lr * m_hat / (sqrt(v_hat) + s.eps)).clone();
    }
    void step() {}
};

template <typename val_type>
class nadam_t {
    jsm_opt::moments<val_type> s;

public:
    nadam_t(val_type learning_rate = val_type(0.002), val_type beta1 = val_type(0.9), double beta2 = 0.999, double epsilon = 1e-8) {
        s.beta1_t = 1; s.beta2_t = 1;
        s.set(learning_rate, beta1, beta2, epsilon, true);
    }
    // the reference's set() keeps the running powers of beta (:129-137)
    void set(val_type learning_rate = val_type(0.002), val_type beta1 = val_type(0.9), double beta2 = 0.999, double epsilon = 1e-8) {
        s.set(learning_rate, beta1, beta2, epsilon, false);
    }
    void set_lr(val_type lr) { s.lr = lr; }
    // reference: :144-164
    void update(const mat_t<val_type>& grad, mat_t<val_type>& mat) {
        s.accumulate(grad);
        mat_t<val_type> m_hat = (s.m / (1 - s.beta1_t)).clone();
        mat_t<val_type> v_hat = (s.v / (1 - s.beta2_t)).clone();
        mat_t<val_type> step = (s.lr * (s.beta1 * m_hat / (1 - s.beta1_t * s.beta1) + (1 - s.beta1) / (1 - s.beta1_t) * grad)).clone();
        mat = (mat - step / (sqrt(v_hat) + s.eps)).clone();
    }
    void step() {}
};

// Averages the gradients of several backward passes and applies them with the wrapped updater at step()
// (reference: mat_updator_t.hpp:172-218): a running mean, cache = cache * (1 - 1/(n+1)) + grad / (n+1).
template <typename val_type, template <typename> class updator_type>
class cache_updator_t {
    updator_type<val_type> m_updator;
    mat_t<val_type> m_cache;
    mat_t<val_type>* m_mat = nullptr;
    val_type m_count = 0;

public:
    cache_updator_t(val_type learning_rate = val_type(0.001)) : m_updator(learning_rate) {}
    void update(const mat_t<val_type>& grad, mat_t<val_type>& mat) {
        if (m_mat == nullptr) {
            m_cache = mat_t<val_type>(grad.row_num(), grad.col_num());
            m_mat = &mat;
        }
        m_cache = (m_cache * (val_type(1.0) - val_type(1.0) / val_type(m_count + 1)) + grad / val_type(m_count + 1)).clone();
        m_count += 1;
    }
    void step() {
        if (m_mat == nullptr) return;
        m_updator.update(m_cache, *m_mat);
        m_cache = val_type(0);
        m_count = 0;
    }
    void set_lr(val_type lr) { m_updator.set_lr(lr); }
    template <typename... upr_arg_types>
    void set(val_type learning_rate, upr_arg_types&&... args) { m_updator.set(learning_rate, std::forward<upr_arg_types>(args)...); }
};

#endif
