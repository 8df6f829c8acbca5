// Stream output and the net-folding operators of the jasmine API (reference: mat_utility.hpp:7-39, 94-100).
// and the learning-rate schedule cosine_annealing_decay (reference: mat_utility.hpp:102-239).
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

// Cosine annealing with linear warm-up and warm restarts (reference: mat_utility.hpp:102-239).  A cycle of
// decay_total_epoches steps: the first warmup_steps ramp linearly from 0 to max_lr, the rest follow
// min_lr + (max_lr - min_lr) * (1 + cos(pi * progress)) / 2.  When a cycle ends the next one is T_multiplier times longer
// and both rates shrink by lr_decay_rate.  step() returns false once total_epochs steps have been taken.
struct cosine_annealing_decay {
    double max_lr, min_lr;
    int init_decay_epoch, decay_total_epoches, decay_curr_epoch = 0;
    double warmup_rate, warmup_steps;
    double T_multiplier, lr_decay_rate;
    int total_epochs, current_epoch = 0;
    int total_cycle = 0, cur_cycle = 0;

    cosine_annealing_decay(int epoch_max = 1000, int init_decay_steps = 100, double max_lr_ = 1e-4, double min_lr_ = 1e-6,
                           double warmup_rate_ = 0.2, double T_multiplier_ = 2.0, double lr_decay_rate_ = 0.8) {
        reset_config(epoch_max, init_decay_steps, max_lr_, min_lr_, warmup_rate_, T_multiplier_, lr_decay_rate_);
    }
    void reset_config(int epoch_max, int init_decay_steps = 100, double max_lr_ = 1e-4, double min_lr_ = 1e-6, double warmup_rate_ = 0.2,
                      double T_multiplier_ = 2.0, double lr_decay_rate_ = 0.8) {
        max_lr = max_lr_; min_lr = min_lr_;
        warmup_rate = warmup_rate_; T_multiplier = T_multiplier_; lr_decay_rate = lr_decay_rate_;
        total_epochs = epoch_max;
        current_epoch = 0; decay_curr_epoch = 0; cur_cycle = 0;
        begin_cycles(init_decay_steps);
    }
    int get_total_cycle() const { return total_cycle; }
    int get_current_cycle() const { return cur_cycle; }
    // (the reference recomputes the cycle count from the new length over itself here: one cycle)
    void set_init_decay_epoch(int init_epoch) {
        init_decay_epoch = decay_total_epoches = init_epoch;
        warmup_steps = static_cast<int>(decay_total_epoches * warmup_rate);
        total_cycle = cycles_for(decay_total_epoches);
    }
    double get_lr() {
        if (decay_curr_epoch < warmup_steps) return max_lr * (decay_curr_epoch / static_cast<double>(warmup_steps));
        const double progress = static_cast<double>(decay_curr_epoch - warmup_steps) / (decay_total_epoches - warmup_steps);
        return min_lr + 0.5 * (max_lr - min_lr) * (1 + std::cos(3.14159265358979323846 * progress));
    }
    bool step() {
        ++decay_curr_epoch;
        ++current_epoch;
        if (current_epoch >= total_epochs) return false;
        if (decay_curr_epoch > decay_total_epoches) warm_restart();
        return true;
    }
    void warm_restart() {
        decay_curr_epoch = 0;
        decay_total_epoches = static_cast<int>(decay_total_epoches * T_multiplier);
        max_lr *= lr_decay_rate;
        min_lr *= lr_decay_rate;
        ++cur_cycle;
    }
    // back to the first cycle with the default rates (the reference resets the rates to 1e-4 / 1e-6 and keeps the warm-up
    // length of the last cycle's setting)
    void reset() {
        decay_curr_epoch = 0; current_epoch = 0; cur_cycle = 0;
        decay_total_epoches = init_decay_epoch;
        max_lr = 1e-4; min_lr = 1e-6;
        warmup_steps = static_cast<int>(decay_total_epoches * warmup_rate);
        total_cycle = cycles_for(decay_total_epoches);
    }

private:
    int cycles_for(int length) const {
        return static_cast<int>(std::log2(static_cast<double>(length) / init_decay_epoch) / std::log2(T_multiplier)) + 1;
    }
    void begin_cycles(int first_length) {
        init_decay_epoch = decay_total_epoches = first_length;
        warmup_steps = static_cast<int>(decay_total_epoches * warmup_rate);
        total_cycle = cycles_for(total_epochs);
    }
};

inline std::string print_indent(int n) { return std::string(n > 0 ? (size_t)n : 0, ' '); }

#endif
