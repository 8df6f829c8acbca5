// A program written against the jasmine API only (inference side).  The SAME source is compiled twice:
//   g++ -std=c++20 -I<jasmine reference>               -> CPU, the reference's own headers (expected output)
//   g++ -std=c++20 -Iinclude/jasmine -Iinclude -ljasmine_b200   -> this library, every operation on the GPU
// and the two outputs are compared value by value (tests/test_gpu_dropin.py).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <sstream>
#include <stdexcept>
#include <vector>

#include "mat_t.hpp"
#include "mat_express_t.hpp"
#include "mat_view_t.hpp"
#include "mat_net_t.hpp"
#include "mat_init_t.hpp"
#include "mat_mha_t.hpp"
#include "mat_transformer_kernel_t.hpp"
#include "mat_RoPE_t.hpp"
#include "mat_transformer_t.hpp"
#include "mat_loss_t.hpp"
#include "mat_updator_t.hpp"

using F = float;
using M = mat_t<F>;

// deterministic values in [-1, 1)
static unsigned g_state = 12345u;
static F next_value() {
    g_state = g_state * 1664525u + 1013904223u;
    return (F)((g_state >> 8) & 0xFFFF) / 32768.0f - 1.0f;
}
template <typename T>
using averaged_sgd_t = cache_updator_t<T, sgd_t>;
// every weight of a net, in the API's fixed order, through the init_t customisation point
struct seeded_t;
template <>
struct init_t<seeded_t> {
    template <typename mat_type>
    requires is_matrix<mat_type>
    static void cal(mat_type& m) {
        for (int i = 0; i < m.row_num(); ++i)
            for (int j = 0; j < m.col_num(); ++j) m(i, j) = 0.4f * next_value();
    }
};
static M make(int r, int c, F scale = 1.0f, F shift = 0.0f) {
    M m(r, c);
    for (int i = 0; i < r; ++i)
        for (int j = 0; j < c; ++j) m(i, j) = scale * next_value() + shift;
    return m;
}
template <typename T>
static void dump(const char* name, const T& m) {
    std::printf("%s %d %d", name, (int)m.row_num(), (int)m.col_num());
    for (int i = 0; i < m.row_num(); ++i)
        for (int j = 0; j < m.col_num(); ++j) std::printf(" %.9g", (double)m(i, j));
    std::printf("\n");
}
static void dump_scalar(const char* name, double v) { std::printf("%s 1 1 %.9g\n", name, v); }

int main() {
    // ---- expression operators, broadcast, materialisation ----
    M a = make(4, 6), b = make(4, 6), colv = make(4, 1), rowv = make(1, 6), pos = make(4, 6, 0.5f, 1.0f);
    dump("add", (a + b).clone());
    dump("chain", ((a + b - a) * b / pos).clone());
    dump("axpb", (a * 0.125f + b).clone());
    dump("bcast_col", (a - colv).clone());
    dump("bcast_row", (a * rowv).clone());
    dump("scalar_left", (2.0f - a).clone());
    dump("greater", (a > b).clone());
    dump("less", (a < 0.25f).clone());
    dump("relu_expr", ((a > 0) * a).clone());
    dump("exp", exp(a).clone());
    dump("sigmoid", sigmoid(a).clone());
    M acc = a;
    acc += b;
    acc += 1.5f;
    dump("plus_assign", acc);
    M conv = a + b;  // conversion operator
    dump("convert", conv);
    dump_scalar("elem_of_expr", (a + b)(2, 3));
    // ---- reductions ----
    dump("hsum", hsum(a)); dump("vsum", vsum(a)); dump("hmean", hmean(a)); dump("vmean", vmean(a)); dump("hmax", hmax(a));
    dump_scalar("sum", sum(a)); dump_scalar("mean", mean(a)); dump_scalar("max", max(a));
    dump("pow2", pow(a, 2.0)); dump("sqrt", sqrt(pos));
    dump("hsoftmax", hsoftmax(a * 0.125f + b));
    dump("softmax", softmax(a).clone());
    dump("hsum_of_expr", hsum(a * b));
    // ---- views ----
    dump("view", a.view(1, 2, 2, 3).clone());
    dump("transpose", a.t().clone());
    dump("back_col", a.back_col().clone());
    dump("row", a.row(2).clone());
    dump("view_expr", (a.view(0, 0, 2, 2) + b.view(2, 4, 2, 2)).clone());
    M target(4, 6);
    target.view(1, 1, 2, 3).assign(a.view(0, 0, 2, 3));
    dump("assign", target);
    // ---- dot ----
    M c = make(6, 3);
    dump("dot", a.dot(c).clone());
    dump("dot_t", a.t().dot(b).clone());
    dump("dot_chain", a.dot(c).dot(c.t()).clone());
    dump("dot_plus", (a.dot(c) + colv).clone());
    try {
        auto bad = a.dot(b).clone();
        std::printf("dot_error 1 1 0\n");
    } catch (const std::invalid_argument&) {
        std::printf("dot_error 1 1 1\n");
    }
    // ---- nets ----
    weight_net_t<M, sgd_t> lin(6, 5);
    lin.init_weight<seeded_t>();
    M x = make(6, 7);
    dump("weight_net", lin.forward(x));
    relu_net_t<M> relu;
    dump("relu_net", relu.forward(x));
    sigmoid_net_t<M> sig;
    dump("sigmoid_net", sig.forward(x));
    layer_norm_net_t<M, sgd_t> ln;
    dump("layer_norm", ln.forward(x));
    hsoftmax_net_t<M> hs;
    dump("hsoftmax_net", hs.forward(x));
    using mlp_t = complex_net_builder_t<F>::push_back_updatable<weight_net_t, sgd_t>::push_back_staticnet<relu_net_t>::
        push_back_updatable<weight_net_t, sgd_t>::type;
    mlp_t mlp;
    mlp.reinit(std::vector<int>{6, 9, 4});
    mlp.init_weight<seeded_t>();
    dump("mlp", mlp.forward(x));
    dump("mlp_fold", x >> mlp);
    residual_net_t<complex_net_t<weight_net_t<M, sgd_t>, relu_net_t<M>>> res;
    res.base_net().reinit(std::vector<int>{6, 6});
    res.init_weight<seeded_t>();
    dump("residual", res.forward(x));
    // ---- attention ----
    mat_mha_t<M, sgd_t> mha(4, 16, true, 9);
    mha.init_weight<seeded_t>();
    M seq = make(16, 9);
    M att = mha.forward(seq);
    dump("mha_causal", att);
    M prefix(16, 4);
    for (int i = 0; i < 16; ++i)
        for (int j = 0; j < 4; ++j) prefix(i, j) = seq(i, j);
    dump("mha_prefix", mha.forward(prefix));  // equals the first 4 columns of mha_causal
    mat_mha_t<M, sgd_t> mha_full(2, 16, false, 9);
    mha_full.init_weight<seeded_t>();
    dump("mha_full", mha_full.forward(seq));
    M enc_in = make(16, 5);
    dump("mha_cross", mha_full.forward(seq, enc_in));
    try {
        mha.forward(make(8, 3));
        std::printf("mha_error 1 1 0\n");
    } catch (const std::runtime_error&) {
        std::printf("mha_error 1 1 1\n");
    }
    mat_head_gen_t<M, sgd_t> head(8, true, 6);
    head.init_weight<seeded_t>();
    M hx = make(8, 6);
    dump("head", head.forward(hx.view(0, 0, 8, 6)));
    // ---- RoPE ----
    RoPE_net_t<M> rope(16);
    dump("rope", rope.forward(seq));
    // ---- stacks ----
    encoder_t<F, sgd_t> enc(2, 2, 8, 5);
    for (int i = 0; i < 2; ++i) enc.get_mha(i).set_param(2, 8, true, 5);  // decoder-only causal stack
    enc.init_weight<seeded_t>();
    M ex = make(8, 5);
    dump("encoder_causal", enc.forward(ex));
    transformer_base_t<M, sgd_t> tf(1, 1, 2, 8);
    tf.init_weight<seeded_t>();
    tf.encoder_forward(ex);
    M dx = make(8, 3);
    dump("transformer", tf.forward(dx));

    // ---- vsplit / vconcat (mat_mha_t.hpp:164-215) and their errors ----
    {
        M big = make(6, 4);
        auto parts = vsplit(big, 3);
        dump("vsplit_mid", parts[1].clone());
        std::vector<M> pieces;
        for (auto& p : parts) pieces.push_back(p.clone());
        std::swap(pieces[0], pieces[2]);
        dump("vconcat", vconcat(pieces));
        int caught = 0;
        try { vsplit(big, 4); } catch (const std::runtime_error&) { ++caught; }       // 6 rows do not split in 4
        try { vsplit(big, 0); } catch (const std::runtime_error&) { ++caught; }
        try { vconcat(std::vector<M>{}); } catch (const std::runtime_error&) { ++caught; }
        try { vconcat(std::vector<M>{make(2, 3), make(2, 4)}); } catch (const std::runtime_error&) { ++caught; }
        dump_scalar("split_concat_errors", caught);
    }

    // ---- generation: the reference's predict loop (transformer_test.hpp:227-241) feeds the growing decoder input through
    // the whole stack at every step and takes the last output column as the next input column.  With JASMINE_B200 the same
    // columns come from forward_cached: one new column per step against cached keys / values (self attention) and the
    // keys / values of the encoder output projected once (cross attention). ----
    {
        const int d = 8, steps = 6;
        transformer_base_t<M, sgd_t> gen(2, 2, 2, d);
        gen.init_weight<seeded_t>();
        M src = make(d, 4);
        gen.encoder_forward(src);
        M dec(d, steps + 1);
        M first = make(d, 1);
        dec.view(0, 0, d, 1).assign(first);
        for (int len = 1; len <= steps; ++len) {
#ifdef JASMINE_B200
            M out_col = gen.forward_cached(dec.view(0, len - 1, d, 1).clone());
            dec.view(0, len, d, 1).assign(out_col);
#else
            M out = gen.forward(dec.view(0, 0, d, len).clone());
            dec.view(0, len, d, 1).assign(out.back_col());
#endif
        }
        dump("predict", dec);
        // a second sequence on the same object: the caches start over with the new encoder pass
        M src2 = make(d, 3);
        gen.encoder_forward(src2);
        M dec2(d, 4);
        dec2.view(0, 0, d, 1).assign(first);
        for (int len = 1; len <= 3; ++len) {
#ifdef JASMINE_B200
            dec2.view(0, len, d, 1).assign(gen.forward_cached(dec2.view(0, len - 1, d, 1).clone()));
#else
            dec2.view(0, len, d, 1).assign(gen.forward(dec2.view(0, 0, d, len).clone()).back_col());
#endif
        }
        dump("predict_again", dec2);

        // decoder-only causal stack: a prompt of 3 columns at once, then column by column
        encoder_t<F, sgd_t> lm(2, 2, d, 16);
        for (int i = 0; i < 2; ++i) lm.get_mha(i).set_param(2, d, true, 16);
        lm.init_weight<seeded_t>();
        M seqm(d, 7);
        seqm.view(0, 0, d, 3).assign(make(d, 3));
#ifdef JASMINE_B200
        M o3 = lm.forward_cached(seqm.view(0, 0, d, 3).clone());
        seqm.view(0, 3, d, 1).assign(o3.back_col());
        for (int len = 4; len < 7; ++len) seqm.view(0, len, d, 1).assign(lm.forward_cached(seqm.view(0, len - 1, d, 1).clone()));
#else
        for (int len = 3; len < 7; ++len) seqm.view(0, len, d, 1).assign(lm.forward(seqm.view(0, 0, d, len).clone()).back_col());
#endif
        dump("causal_stack_generate", seqm);

        // checkpoint: a net that was initialised differently computes the saved net's outputs after loading its record
#ifdef JASMINE_B200
        std::stringstream file;
        gen.save(file);
        transformer_base_t<M, sgd_t> other(2, 2, 2, d);
        other.init_weight<seeded_t>();        // other values: the generator has moved on
        other.encoder_forward(src2);
        M before = other.forward(dec2);
        other.load(file);
        other.encoder_forward(src2);
        M after = other.forward(dec2);
        M want = gen.forward(dec2);
        double diff_before = 0, diff_after = 0;
        for (int i = 0; i < d; ++i)
            for (int j = 0; j < 4; ++j) {
                diff_before = std::max(diff_before, (double)std::abs(before(i, j) - want(i, j)));
                diff_after = std::max(diff_after, (double)std::abs(after(i, j) - want(i, j)));
            }
        dump_scalar("save_load", (diff_before > 1e-3 && diff_after == 0.0) ? 1 : 0);
#else
        dump_scalar("save_load", 1);
#endif
    }

    // ---- training of the basic nets: forward, mse gradient, backward through the chain, updater (mat_net_t.hpp:65-75,
    // 108-116, 155-165, 330-334, 381-385; mat_updator_t.hpp; mat_loss_t.hpp) ----
    {
        g_state = 777u;  // the checkpoint block above draws a different number of values under the two sets of headers
        M tx = make(6, 5), ty = make(4, 5);
        {
            using net_t = complex_net_builder_t<F>::push_back_updatable<weight_net_t, sgd_t>::push_back_staticnet<relu_net_t>::
                push_back_updatable<weight_net_t, sgd_t>::type;
            net_t net;
            net.reinit(std::vector<int>{6, 7, 4});
            net.init_weight<seeded_t>();
            net.set_updator(0.05f);
            mse_loss_t<M> loss;
            M losses(1, 6);
            for (int it = 0; it < 6; ++it) {
                loss.forward(net.forward(tx));
                losses(0, it) = loss.loss(ty);
                net.backward(loss.backward(ty));
                net.step();
            }
            dump("train_sgd_loss", losses);
            dump("train_sgd_out", net.forward(tx));
        }
        {
            residual_net_t<complex_net_t<weight_net_t<M, nadam_t>, relu_net_t<M>>> net;
            net.base_net().reinit(std::vector<int>{6, 6});
            net.init_weight<seeded_t>();
            mse_loss_t<M> loss;
            M target = make(6, 5);
            for (int it = 0; it < 4; ++it) {
                loss.forward(net.forward(tx));
                net.backward(loss.backward(target));
            }
            dump("train_nadam_residual_out", net.forward(tx));
        }
        {
            weight_net_t<M, adam_t> net(6, 4);
            net.init_weight<seeded_t>();
            mse_loss_t<M> loss;
            M down;
            for (int it = 0; it < 4; ++it) {
                loss.forward(net.forward(tx));
                down = net.backward(loss.backward(ty));
            }
            dump("train_adam_out", net.forward(tx));
            dump("train_adam_grad_in", down);
        }
        {
            // a layer norm inside the chain: its gain and bias train too (mat_net_t.hpp:227-243)
            using net_t = complex_net_builder_t<F>::push_back_updatable<weight_net_t, sgd_t>::push_back_updatable<layer_norm_net_t, sgd_t>::
                push_back_updatable<weight_net_t, sgd_t>::type;
            net_t net;
            net.reinit(std::vector<int>{6, 7, 4});
            net.init_weight<seeded_t>();
            net.set_updator(0.02f);
            mse_loss_t<M> loss;
            M down;
            for (int it = 0; it < 4; ++it) {
                loss.forward(net.forward(tx));
                down = net.backward(loss.backward(ty));
            }
            dump("train_layer_norm_out", net.forward(tx));
            dump("train_layer_norm_grad_in", down);
        }
        {
            hsoftmax_net_t<M> hs;
            M sx = make(5, 6);
            hs.forward(sx);
            dump("hsoftmax_backward", hs.backward(make(5, 6)));
        }
        {
            // gradients of two backward passes averaged, applied at step() (mat_updator_t.hpp:172-218)
            weight_net_t<M, averaged_sgd_t> net(6, 4);
            net.init_weight<seeded_t>();
            net.set_updator(0.1f);
            mse_loss_t<M> loss;
            M tx2 = make(6, 5);
            for (int round = 0; round < 2; ++round) {
                loss.forward(net.forward(tx));
                net.backward(loss.backward(ty));
                loss.forward(net.forward(tx2));
                net.backward(loss.backward(ty));
                net.step();
            }
            dump("train_averaged_out", net.forward(tx));
        }
        {
            cosine_annealing_decay sched(40, 8, 1e-3, 1e-5, 0.25, 2.0, 0.5);
            M lrs(1, 40);
            int n = 0;
            do {
                lrs(0, n++) = (F)(sched.get_lr() * 1000.0);
            } while (sched.step() && n < 40);
            dump("cosine_schedule", lrs);
            dump_scalar("cosine_cycles", sched.get_total_cycle() * 100 + sched.get_current_cycle());
        }
        {
            // self attention and a causal two-layer stack: backward through softmax, the per-head projections, the layer
            // norms and the residual connections (mat_mha_t.hpp:92-117, 324-346; mat_transformer_kernel_t.hpp:112-119).
            // One head: the reference's backward of every further head goes through a transposed view with a row offset,
            // whose element access adds the row offset to the column and the column offset to the row
            // (mat_view_t.hpp:29-39), so it reads another head's gradient rows.
            M ax = make(8, 5), target = make(8, 5);
            mse_loss_t<M> loss;
            M down;
            mat_mha_t<M, sgd_t> att(1, 8, true, 5);
            att.init_weight<seeded_t>();
            att.set_updator(0.05f);
            for (int it = 0; it < 3; ++it) {
                loss.forward(att.forward(ax));
                down = att.backward(loss.backward(target));
                att.step();
            }
            dump("train_mha_out", att.forward(ax));
            dump("train_mha_grad_in", down);
            encoder_t<F, sgd_t> stack(2, 1, 8, 5);
            for (int i = 0; i < 2; ++i) stack.get_mha(i).set_param(1, 8, true, 5);
            stack.init_weight<seeded_t>();
            stack.set_updator(0.02f);
            for (int it = 0; it < 3; ++it) {
                loss.forward(stack.forward(ax));
                down = stack.backward(loss.backward(target));
                stack.step();
            }
            dump("train_stack_out", stack.forward(ax));
            dump("train_stack_grad_in", down);
        }
        // (sigmoid_net_t::backward is left out: the reference's version, mat_net_t.hpp:108-116, keeps an expression that
        // refers to a temporary of the previous statement and reads freed memory when optimised.)
    }
    return 0;
}
