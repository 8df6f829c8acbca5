// Encoder-decoder generation of the jasmine API with the attention layers on the tensor cores (bf16 operands, the tcgen05
// flash kernel) against the same model on the fp32 kernels: self attention with cached keys / values, cross attention
// against keys / values of the encoder output that were projected once.  Heads are 128 wide (the flash kernel's shape).
// Prints the largest difference relative to the largest fp32 value for (1) a full decoder pass over 160 columns
// (non-causal cross attention with Tq != Tk through the flash kernel) and (2) six cached generation steps.
#include <algorithm>
#include <cmath>
#include <cstdio>

#include "mat_t.hpp"
#include "mat_express_t.hpp"
#include "mat_view_t.hpp"
#include "mat_net_t.hpp"
#include "mat_init_t.hpp"
#include "mat_mha_t.hpp"
#include "mat_transformer_kernel_t.hpp"
#include "mat_RoPE_t.hpp"
#include "mat_transformer_t.hpp"

using F = float;
using M = mat_t<F>;
static unsigned g_state = 4242u;
static F next_value() {
    g_state = g_state * 1664525u + 1013904223u;
    return (F)((g_state >> 8) & 0xFFFF) / 32768.0f - 1.0f;
}
struct seeded_t;
template <>
struct init_t<seeded_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) {
        const F s = 1.0f / std::sqrt((F)std::max(1, (int)m.col_num()));
        for (int i = 0; i < m.row_num(); ++i)
            for (int j = 0; j < m.col_num(); ++j) m(i, j) = s * next_value();
    }
};
static M make(int r, int c) {
    M m(r, c);
    for (int i = 0; i < r; ++i)
        for (int j = 0; j < c; ++j) m(i, j) = next_value();
    return m;
}
static double rel_diff(const M& a, const M& b) {
    double worst = 0, scale = 1e-30;
    for (int i = 0; i < a.row_num(); ++i)
        for (int j = 0; j < a.col_num(); ++j) {
            worst = std::max(worst, (double)std::abs(a(i, j) - b(i, j)));
            scale = std::max(scale, (double)std::abs(b(i, j)));
        }
    return worst / scale;
}

int main() {
    const int d = 256, heads = 2, src_len = 200, dec_len = 160, steps = 6;
    transformer_base_t<M, sgd_t> tf(1, 2, heads, d);
    tf.init_weight<seeded_t>();
    M src = make(d, src_len), dec = make(d, dec_len), first = make(d, 1);

    jsm_rt::attention_bf16() = false;
    tf.encoder_forward(src);
    M full_f32 = tf.forward(dec);
    M gen_f32(d, steps);
    M col = first;
    for (int s = 0; s < steps; ++s) {
        col = tf.forward_cached(col);
        gen_f32.view(0, s, d, 1).assign(col);
    }

    jsm_rt::attention_bf16() = true;
    tf.encoder_forward(src);
    M full_bf16 = tf.forward(dec);
    M gen_bf16(d, steps);
    col = first;
    for (int s = 0; s < steps; ++s) {
        col = tf.forward_cached(col);
        gen_bf16.view(0, s, d, 1).assign(col);
    }
    std::printf("full_pass %.6g\n", rel_diff(full_bf16, full_f32));
    std::printf("cached_generation %.6g\n", rel_diff(gen_bf16, gen_f32));
    return 0;
}
