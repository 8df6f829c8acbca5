// Updater slot of the jasmine net templates (reference: mat_updator_t.hpp).  Every net template takes an
// updater as a template-template parameter, so the type has to exist; optimisation is a training concern and
// outside this inference library, hence the updaters only keep their settings and never change a weight.
#ifndef JASMINE_B200_MAT_UPDATOR_T_HPP_
#define JASMINE_B200_MAT_UPDATOR_T_HPP_
#include "mat_t.hpp"

template <typename val_type>
class sgd_t {
    val_type m_learning_rate;

public:
    sgd_t(val_type learning_rate = val_type(0.001)) : m_learning_rate(learning_rate) {}
    void set(val_type learning_rate = val_type(0.001)) { m_learning_rate = learning_rate; }
    void set_lr(val_type lr) { m_learning_rate = lr; }
    val_type lr() const { return m_learning_rate; }
    void step() {}
};

template <typename val_type>
using adam_t = sgd_t<val_type>;
template <typename val_type>
using nadam_t = sgd_t<val_type>;

#endif
