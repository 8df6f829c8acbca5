"""Seeded inputs of the parity cases, shared by the golden-vector generator and the tests.

Every array comes from the counter-based generator (seed, tensor id), so a case is
fully described by its name; tests/golden/*.npz hold only the reference's outputs.
"""
from __future__ import annotations

import numpy as np

import oracle_lib as ol


def normal(shape, seed, tid, std=1.0, mean=0.0):
    n = int(np.prod(shape))
    return ol.fill(n, seed, tid, 0, mean, std).reshape(shape)


def uniform(shape, seed, tid, lo, hi):
    n = int(np.prod(shape))
    return ol.fill(n, seed, tid, 1, lo, hi).reshape(shape)


def ints(n, seed, tid, lo, hi):
    return ol.fill(n, seed, tid, 2, lo, hi).astype(np.int32)


# ---- expression cases: (name, op, A shape, B shape or None, scalar) ---------------------------
EXPR_CASES = [
    ("add", 0, (5, 12), (5, 12), 0.0),
    ("sub_colvec", 1, (5, 12), (5, 1), 0.0),
    ("mul_rowvec", 2, (5, 12), (1, 12), 0.0),
    ("div", 3, (5, 12), (5, 12), 0.0),
    ("greater", 4, (5, 12), (5, 12), 0.0),
    ("less_scalar", 5, (5, 12), (1, 1), 0.0),
    ("exp", 6, (5, 12), None, 0.0),
    ("sigmoid", 7, (5, 12), None, 0.0),
    ("axpb", 8, (16, 64), (16, 64), 0.125),
    ("relu", 9, (7, 9), None, 0.0),
    ("pow2", 10, (7, 9), None, 2.0),
    ("pow3", 10, (7, 9), None, 3.0),
    ("sqrt", 11, (7, 9), None, 0.0),
    ("iadd", 12, (5, 12), (5, 12), 0.0),
    ("chain", 13, (6, 8), (6, 8), 0.0),
    ("scale", 14, (5, 12), None, -1.5),
    ("shift", 15, (5, 12), None, 2.25),
    ("tile_modulo", 0, (6, 8), (3, 4), 0.0),  # B repeats by modulo (mat_t.hpp:302-320)
]


def expr_inputs(name, op, sa, sb, s):
    seed = 100 + [c[0] for c in EXPR_CASES].index(name)
    A = normal(sa, seed, 0)
    if op == 11:
        A = np.abs(A) + np.float32(0.01)
    if op in (3, 13):
        A = A + np.sign(A) * np.float32(0.5)
    B = normal(sb, seed, 1) if sb is not None else None
    if op == 3 and B is not None:
        B = B + np.sign(B) * np.float32(0.5)
    return A, B


REDUCE_KINDS = ["hsum", "hmax", "hmean", "vsum", "vmean", "sum", "mean", "max"]


def reduce_input():
    return normal((7, 33), 200, 0)


def softmax_inputs():
    return normal((16, 64), 1, 0), normal((16, 64), 1, 1)


def norm_inputs():
    x = normal((9, 32), 300, 0)  # token-major [T, d]
    x2 = normal((9, 32), 300, 1)
    g = uniform((32,), 300, 2, 0.5, 1.5)
    b = normal((32,), 300, 3, 0.1)
    return x, x2, g, b


def dot_inputs():
    return normal((9, 17), 400, 0), normal((17, 5), 400, 1)


def linear_inputs():
    return normal((7, 24), 401, 0), normal((12, 24), 401, 1, 0.2), normal((12,), 401, 2, 0.1)


MHA = dict(H=4, d=32, T=12)


def mha_inputs():
    n = ol.port_oracle().mha_weight_count(MHA["H"], MHA["d"])
    return normal((n,), 500, 0, 0.3), normal((MHA["T"], MHA["d"]), 500, 1)


def rope_input():
    return normal((10, 16), 600, 0)


ENC = dict(L=2, H=2, d=16, T=8)


def encoder_inputs():
    n = ol.port_oracle().encoder_weight_count(ENC["L"], ENC["H"], ENC["d"])
    return normal((n,), 700, 0, 0.3), normal((ENC["T"], ENC["d"]), 700, 1)


# configuration 1 of the baseline: tiny GPT-2-style decoder, seed 0
GPT = dict(L=2, d=128, H=4, ffn=512, vocab=256, max_pos=80, eps=1e-5, S=64, n_gen=16)


def gpt_weights():
    """Flat weights in the order of ref_gpt: N(0, 0.02) matrices, LayerNorm gains 1, all biases 0."""
    g = GPT
    d, H, ffn, vocab = g["d"], g["H"], g["ffn"], g["vocab"]
    dh = d // H
    parts = []
    tid = [0]

    def mat(*shape):
        tid[0] += 1
        parts.append(normal(shape, 0, tid[0], 0.02).ravel())

    def const(n, v):
        parts.append(np.full(n, v, np.float32))

    mat(vocab, d)
    mat(g["max_pos"], d)
    for _ in range(g["L"]):
        const(d, 1.0); const(d, 0.0)
        for _h in range(H):
            for _p in range(3):
                mat(dh, dh); const(dh, 0.0)
        mat(d, d); const(d, 0.0)
        const(d, 1.0); const(d, 0.0)
        mat(ffn, d); const(ffn, 0.0)
        mat(d, ffn); const(d, 0.0)
    const(d, 1.0); const(d, 0.0)
    mat(vocab, d); const(vocab, 0.0)
    w = np.concatenate(parts).astype(np.float32)
    assert w.size == ol.port_oracle().gpt_weight_count(g["L"], d, H, ffn, vocab, g["max_pos"])
    return w


def gpt_ids():
    return ints(GPT["S"], 0, 1000, 0, GPT["vocab"])


def gpt_unpack(w):
    """Split the flat cfg-1 weights into named arrays (same order as gpt_weights)."""
    g = GPT
    d, H, ffn, vocab = g["d"], g["H"], g["ffn"], g["vocab"]
    dh = d // H
    o = [0]

    def take(*shape):
        n = int(np.prod(shape))
        a = w[o[0]:o[0] + n].reshape(shape)
        o[0] += n
        return a

    out = {"tok": take(vocab, d), "pos": take(g["max_pos"], d), "layers": []}
    for _ in range(g["L"]):
        lw = {"ln1_g": take(d), "ln1_b": take(d), "heads": []}
        for _h in range(H):
            lw["heads"].append([(take(dh, dh), take(dh)) for _p in range(3)])
        lw["wo"], lw["bo"] = take(d, d), take(d)
        lw["ln2_g"], lw["ln2_b"] = take(d), take(d)
        lw["w1"], lw["b1"] = take(ffn, d), take(ffn)
        lw["w2"], lw["b2"] = take(d, ffn), take(d)
        out["layers"].append(lw)
    out["lnf_g"], out["lnf_b"] = take(d), take(d)
    out["w_out"], out["b_out"] = take(vocab, d), take(vocab)
    assert o[0] == w.size
    return out
