"""Pins the CPU restatement (oracle/jasmine_oracle.cpp) against the reference's own outputs:
the committed vectors under tests/golden/ (made by tests/golden/make_golden.py from the reference's
headers) and, where oracle/_ref was built, the reference library itself on fresh inputs.
Because the port keeps the reference's order of floating-point operations, most cases are bit-exact."""
from pathlib import Path

import numpy as np
import pytest

import cases
import oracle_lib as ol

GOLD = Path(__file__).resolve().parent / "golden"
OPS = np.load(GOLD / "ops.npz")
port = ol.port_oracle()


def same(a, b, tol=0.0):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    if tol == 0.0:
        assert np.array_equal(a, b, equal_nan=True), f"max |diff| {np.nanmax(np.abs(a - b))}"
    else:
        scale = max(float(np.max(np.abs(b))), 1e-30)
        assert float(np.max(np.abs(a - b))) <= tol * scale


@pytest.mark.parametrize("case", cases.EXPR_CASES, ids=[c[0] for c in cases.EXPR_CASES])
def test_expr_matches_golden(case):
    name, op, sa, sb, s = case
    A, B = cases.expr_inputs(*case)
    same(port.expr(op, A, B, s), OPS[f"expr_{name}"])


@pytest.mark.parametrize("kind", range(8), ids=cases.REDUCE_KINDS)
def test_reduce_matches_golden(kind):
    same(port.reduce(kind, cases.reduce_input()), OPS[f"reduce_{cases.REDUCE_KINDS[kind]}"].ravel())


def test_softmax_matches_golden():
    A, B = cases.softmax_inputs()
    same(port.hsoftmax(A, B, 0.125), OPS["hsoftmax_axpb"])
    same(port.hsoftmax(A), OPS["hsoftmax_plain"])
    same(port.softmax_full(A[:6, :10]), OPS["softmax_full"])


def test_norms_match_golden():
    x, x2, g, b = cases.norm_inputs()
    same(port.layer_norm(x), OPS["layer_norm_ref"])
    same(port.layer_norm(x, x2, g, b, 1e-5), OPS["layer_norm_eps"])
    same(port.rms_norm(x, g, 1e-5), OPS["rms_norm"])


def test_dot_linear_activation_match_golden():
    A, B = cases.dot_inputs()
    rc, y = port.dot(A, B)
    assert rc == 0
    same(y, OPS["dot"])
    X, W, b = cases.linear_inputs()
    same(port.linear(X, W, b), OPS["linear"])
    same(port.activation(0, X), OPS["relu_net"])
    same(port.activation(1, X), OPS["sigmoid_net"])


def test_dot_shape_error_like_reference():
    # mat_dot_t throws std::invalid_argument on an inner-dimension mismatch (mat_express_t.hpp:709-712)
    rc, _ = port.dot(np.zeros((3, 4), np.float32), np.zeros((5, 2), np.float32))
    assert rc == 1
    r = ol.ref_oracle()
    if r is not None:
        assert r.dot(np.zeros((3, 4), np.float32), np.zeros((5, 2), np.float32))[0] == 1


def test_mha_matches_golden():
    w, x = cases.mha_inputs()
    same(port.mha(w, x, cases.MHA["H"], True), OPS["mha_causal"])
    same(port.mha(w, x, cases.MHA["H"], False), OPS["mha_full"])


def test_rope_matches_golden():
    same(port.rope(cases.rope_input()), OPS["rope"])


def test_encoder_matches_golden():
    w, x = cases.encoder_inputs()
    e = cases.ENC
    same(port.encoder(w, x, e["L"], e["H"], True, True), OPS["encoder_causal_rope"])
    same(port.encoder(w, x, e["L"], e["H"], False, False), OPS["encoder_plain"])


def test_gpt_tiny_matches_golden():
    """Configuration 1: logits [64, 256] and 16 greedy tokens by full-prefix recompute."""
    gold = np.load(GOLD / "gpt_tiny.npz")
    g = cases.GPT
    logits, gen, gl = port.gpt(cases.gpt_weights(), g["L"], g["d"], g["H"], g["ffn"], g["vocab"], g["max_pos"], g["eps"],
                               cases.gpt_ids(), g["n_gen"])
    same(logits, gold["logits"])
    assert np.array_equal(gen, gold["tokens"])
    same(gl, gold["gen_logits"])


def test_causal_prefix_property():
    """test_sequence_mha (transformer_test.hpp:246-282): with a causal mask the outputs of a prefix do not
    depend on later columns.  Holds bit-exactly in the port, like in the reference."""
    w, x = cases.mha_inputs()
    H = cases.MHA["H"]
    full = port.mha(w, x, H, True)
    for s1 in (1, 5):
        assert np.array_equal(port.mha(w, x[:s1], H, True), full[:s1])


def test_standard_rope_is_a_rotation():
    t = ol.rope_table(1, 8, 10000.0, 6)
    x = cases.normal((6, 16), 601, 0)
    y = ol.rope_apply(x, t, 8, 2)
    assert np.allclose(np.linalg.norm(y.reshape(6, 2, 8), axis=-1), np.linalg.norm(x.reshape(6, 2, 8), axis=-1), rtol=1e-5)
    assert np.array_equal(y[0], x[0])  # position 0: identity


def test_attention_gqa_equals_repeated_kv():
    q = cases.normal((2 * 5, 4 * 8), 610, 0)
    k = cases.normal((2 * 5, 2 * 8), 610, 1)
    v = cases.normal((2 * 5, 2 * 8), 610, 2)
    a = ol.attention(q, k, v, 2, 4, 2, 8, True)
    kr = np.repeat(k.reshape(10, 2, 8), 2, axis=1).reshape(10, 32)
    vr = np.repeat(v.reshape(10, 2, 8), 2, axis=1).reshape(10, 32)
    assert np.array_equal(a, ol.attention(q, kr, vr, 2, 4, 4, 8, True))


@pytest.mark.skipif(ol.ref() is None, reason="oracle/_ref not built (reference sources absent)")
def test_port_equals_reference_on_fresh_inputs():
    r = ol.ref_oracle()
    A, B = cases.normal((33, 40), 900, 0), cases.normal((33, 40), 900, 1)
    same(port.hsoftmax(A, B, 0.125), r.hsoftmax(A, B, 0.125))
    for kind in range(8):
        same(port.reduce(kind, A), r.reduce(kind, A))
    x = cases.normal((11, 48), 901, 0)
    g, b = cases.uniform((48,), 901, 1, 0.5, 1.5), cases.normal((48,), 901, 2, 0.1)
    same(port.layer_norm(x, None, g, b, 1e-5), r.layer_norm(x, None, g, b, 1e-5))
    same(port.rms_norm(x, g, 1e-5), r.rms_norm(x, g, 1e-5))
    n = port.mha_weight_count(2, 24)
    w = cases.normal((n,), 902, 0, 0.3)
    xx = cases.normal((20, 24), 902, 1)
    same(port.mha(w, xx, 2, True), r.mha(w, xx, 2, True))
    same(port.rope(xx), r.rope(xx))


def test_generator_statistics():
    x = ol.fill(200000, 7, 3, 0, 0.0, 1.0)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01
    u = ol.fill(100000, 7, 4, 1, 0.5, 1.5)
    assert u.min() >= 0.5 and u.max() < 1.5
    i = ol.fill(1000, 7, 5, 2, 0, 256)
    assert i.min() >= 0 and i.max() <= 255 and np.all(i == np.floor(i))
