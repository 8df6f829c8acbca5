"""GPU parity of the expression evaluator (elementwise nodes, reductions, softmax, norms) against
the golden vectors of the reference and the CPU oracle; everything goes through the C ABI."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
import oracle_lib as ol
from gpu_util import FP32_RTOL, assert_close, dev, host

pytestmark = pytest.mark.gpu
OPS = np.load(Path(__file__).resolve().parent / "golden" / "ops.npz")
port = ol.port_oracle()

L0, L1 = (jb.OP_LEAF, 0), (jb.OP_LEAF, 1)
PROGRAMS = {  # op number of tests/cases.py -> postfix program
    0: [L0, L1, (jb.OP_ADD,)], 1: [L0, L1, (jb.OP_SUB,)], 2: [L0, L1, (jb.OP_MUL,)], 3: [L0, L1, (jb.OP_DIV,)],
    4: [L0, L1, (jb.OP_GT,)], 5: [L0, L1, (jb.OP_LT,)], 6: [L0, (jb.OP_EXP,)], 7: [L0, (jb.OP_SIGMOID,)],
    9: [L0, (jb.OP_IMM, 0.0), (jb.OP_GT,), L0, (jb.OP_MUL,)], 11: [L0, (jb.OP_SQRT,)], 12: [L0, L1, (jb.OP_ADD,)],
    13: [L0, L1, (jb.OP_ADD,), L0, (jb.OP_SUB,), L1, (jb.OP_MUL,), L0, (jb.OP_DIV,)],
}


def program_for(op, s):
    if op == 8:
        return [L0, (jb.OP_IMM, s), (jb.OP_MUL,), L1, (jb.OP_ADD,)]
    if op == 10:
        return [L0, (jb.OP_POW, s)]
    if op == 14:
        return [L0, (jb.OP_IMM, s), (jb.OP_MUL,)]
    if op == 15:
        return [L0, (jb.OP_IMM, s), (jb.OP_ADD,)]
    return PROGRAMS[op]


@pytest.mark.parametrize("case", cases.EXPR_CASES, ids=[c[0] for c in cases.EXPR_CASES])
def test_elementwise_matches_reference(case):
    name, op, sa, sb, s = case
    A, B = cases.expr_inputs(*case)
    want = OPS[f"expr_{name}"]
    a = dev(A)
    leaves = [a] if B is None else [a, dev(B)]
    out = a if op == 12 else torch.empty(want.shape, device="cuda")  # += writes into its left operand
    jb.eval_elementwise(program_for(op, s), leaves, out)
    exact = op in (0, 1, 2, 3, 4, 5, 9, 11, 12, 14, 15) or (op == 10 and s == 2.0)
    if exact:  # IEEE add/sub/mul/div/sqrt/compare: bit-identical to the reference
        assert np.array_equal(host(out), want)
    else:
        assert_close(host(out), want, FP32_RTOL, name)


def test_elementwise_views_and_transposes():
    """Leaves may be windows and transposed views (mat_view_t.hpp:7-135): strided operands."""
    A = cases.normal((9, 14), 120, 0)
    B = cases.normal((14, 9), 120, 1)
    a, b = dev(A), dev(B)
    out = torch.empty(5, 6, device="cuda")
    # A.view(2,3,5,6) + B.t().view(2,3,5,6)
    jb.eval_elementwise([L0, L1, (jb.OP_ADD,)], [a[2:7, 3:9], b.t()[2:7, 3:9]], out)
    assert np.array_equal(host(out), A[2:7, 3:9] + B.T[2:7, 3:9])
    # transposed output
    out_t = torch.empty(6, 5, device="cuda")
    jb.eval_elementwise([L0, (jb.OP_IMM, 2.0), (jb.OP_MUL,)], [a[2:7, 3:9]], out_t.t())
    assert np.array_equal(host(out_t), (A[2:7, 3:9] * np.float32(2)).T)


def test_elementwise_bf16_and_large_vector_path():
    A = cases.normal((300, 1024), 121, 0)
    Bv = cases.normal((1, 1024), 121, 1)
    a, b = dev(A, torch.bfloat16), dev(Bv)
    out = torch.empty(300, 1024, device="cuda", dtype=torch.bfloat16)
    jb.eval_elementwise([L0, L1, (jb.OP_MUL,), (jb.OP_SILU,)], [a, b], out)
    x = a.float().cpu().numpy() * Bv
    want = torch.from_numpy(x / (1 + np.exp(-x))).to(torch.bfloat16).float().numpy()
    assert_close(host(out), want, 8e-3, "bf16 silu")


@pytest.mark.parametrize("kind", range(8), ids=cases.REDUCE_KINDS)
def test_reductions_match_reference(kind):
    R = cases.reduce_input()
    want = OPS[f"reduce_{cases.REDUCE_KINDS[kind]}"].ravel()
    a = dev(R)
    rows, cols = R.shape
    k = {0: jb.ROWS_SUM, 1: jb.ROWS_MAX, 2: jb.ROWS_MEAN, 3: jb.ROWS_SUM, 4: jb.ROWS_MEAN, 5: jb.ROWS_SUM, 6: jb.ROWS_MEAN,
         7: jb.ROWS_MAX}[kind]
    if kind < 3:
        out = torch.empty(rows, 1, device="cuda")
        jb.eval_rows(k, 1, [L0], [a], out)
    elif kind < 5:
        out = torch.empty(1, cols, device="cuda")
        jb.eval_rows(k, 0, [L0], [a], out)
    else:
        out = torch.empty(1, 1, device="cuda")
        jb.eval_full(k, [L0], [a], out)
    got = host(out).ravel()
    if kind in (1, 7):
        assert np.array_equal(got, want)
    else:  # a tree sum against the reference's left-to-right sum
        assert float(np.max(np.abs(got - want))) <= FP32_RTOL * float(np.max(np.abs(R))) * (cols if kind < 5 else rows * cols) ** 0.5


def test_hsoftmax_matches_reference():
    A, B = cases.softmax_inputs()
    a, b = dev(A), dev(B)
    out = torch.empty_like(a)
    jb.eval_rows(jb.ROWS_SOFTMAX, 1, program_for(8, 0.125), [a, b], out)
    assert_close(host(out), OPS["hsoftmax_axpb"], FP32_RTOL, "hsoftmax(A*0.125+B)")
    jb.eval_rows(jb.ROWS_SOFTMAX, 1, [L0], [a], out)
    assert_close(host(out), OPS["hsoftmax_plain"], FP32_RTOL, "hsoftmax(A)")
    sub = a[:6, :10].contiguous()
    o2 = torch.empty_like(sub)
    jb.eval_full(jb.ROWS_SOFTMAX, [L0], [sub], o2)
    assert_close(host(o2), OPS["softmax_full"], FP32_RTOL, "softmax (whole matrix)")


def test_softmax_masked_row_like_reference():
    """-inf entries (the causal mask, mat_mha_t.hpp:58-67) give exact zeros."""
    A = cases.normal((4, 40), 130, 0)
    A[:, 25:] = -np.inf
    out = torch.empty(4, 40, device="cuda")
    jb.eval_rows(jb.ROWS_SOFTMAX, 1, [L0], [dev(A)], out)
    got = host(out)
    assert np.all(got[:, 25:] == 0.0)
    assert_close(got, port.hsoftmax(A), FP32_RTOL, "masked softmax")


def test_norms_match_reference():
    x, x2, g, b = cases.norm_inputs()
    xd, x2d, gd, bd = dev(x), dev(x2), dev(g), dev(b)
    out = torch.empty_like(xd)
    jb.eval_rows(jb.ROWS_LAYERNORM, 1, [L0], [xd], out, eps=0.0)
    assert_close(host(out), OPS["layer_norm_ref"], FP32_RTOL, "layer_norm_net_t (no eps)")
    jb.eval_rows(jb.ROWS_LAYERNORM, 1, [L0, L1, (jb.OP_ADD,)], [xd, x2d], out, gain=gd, bias=bd, eps=1e-5)
    assert_close(host(out), OPS["layer_norm_eps"], FP32_RTOL, "LayerNorm(A+B)*g+b")
    jb.eval_rows(jb.ROWS_RMSNORM, 1, [L0], [xd], out, gain=gd, eps=1e-5)
    assert_close(host(out), OPS["rms_norm"], FP32_RTOL, "RMSNorm")
    # the reference's own orientation: features are rows, every column is normalised (axis 0)
    xt = xd.t().contiguous()
    out_t = torch.empty_like(xt)
    jb.eval_rows(jb.ROWS_LAYERNORM, 0, [L0], [xt], out_t, eps=0.0)
    assert_close(host(out_t).T, OPS["layer_norm_ref"], FP32_RTOL, "layer_norm_net_t on [d,S]")
    # the fused residual-add + norm of the decoder
    y = jb.add_norm(jb.ROWS_LAYERNORM, xd, x2d, gd, bd, 1e-5)
    assert_close(host(y), OPS["layer_norm_eps"], FP32_RTOL, "jsm_add_norm")


@pytest.mark.parametrize("shape", [(3, 5), (33, 130), (17, 1000), (9, 3000), (5, 8192), (3, 10000), (257, 64)])
def test_row_kernels_ragged_shapes(shape):
    """Row lengths that are not multiples of the vector width, shorter and longer than a CTA's registers."""
    A = cases.normal(shape, 140, shape[1])
    a = dev(A)
    out = torch.empty_like(a)
    jb.eval_rows(jb.ROWS_SOFTMAX, 1, [L0], [a], out)
    assert_close(host(out), port.hsoftmax(A), FP32_RTOL, f"softmax {shape}")
    g = cases.uniform((shape[1],), 141, 0, 0.5, 1.5)
    jb.eval_rows(jb.ROWS_RMSNORM, 1, [L0], [a], out, gain=dev(g), eps=1e-5)
    assert_close(host(out), port.rms_norm(A, g, 1e-5), FP32_RTOL, f"rmsnorm {shape}")
    s = torch.empty(shape[0], 1, device="cuda")
    jb.eval_rows(jb.ROWS_MAX, 1, [L0], [a], s)
    assert np.array_equal(host(s).ravel(), A.max(axis=1))
    am = torch.empty(shape[0], 1, device="cuda", dtype=torch.int32)
    jb.eval_rows(jb.ROWS_ARGMAX, 1, [L0], [a], am)
    assert np.array_equal(am.cpu().numpy().ravel(), A.argmax(axis=1))


@pytest.mark.parametrize("cols", [1024, 2048, 4096])
@pytest.mark.parametrize("rows", [1, 7, 300, 613])
def test_staged_row_kernels_match_oracle_and_register_kernel(rows, cols):
    """Contiguous f32 rows of 1024 / 2048 / 4096 columns with the programs x, x*imm+y and x+y run through the kernels
    that stage rows in shared memory (a fixed grid: one row, fewer rows than CTAs, more rows than CTAs with a
    remainder).  Checked against the oracle and, bit for bit, against the register kernel: the same program with
    `+ 0.0` appended is not one of the staged forms, takes the register kernel and has the same values."""
    A = cases.normal((rows, cols), 170, cols)
    B = cases.normal((rows, cols), 171, cols)
    g = cases.uniform((cols,), 172, 0, 0.5, 1.5)
    bb = cases.normal((cols,), 173, 1) * np.float32(0.1)
    a, b = dev(A), dev(B)
    plus0 = [(jb.OP_IMM, 0.0), (jb.OP_ADD,)]
    y, y2 = torch.empty_like(a), torch.empty_like(a)
    axpb = program_for(8, 0.125)
    add = [L0, L1, (jb.OP_ADD,)]
    for name, kind, prog, leaves, kw, want in [
        ("softmax", jb.ROWS_SOFTMAX, axpb, [a, b], {}, lambda: port.hsoftmax(A, B, 0.125)),
        ("layernorm", jb.ROWS_LAYERNORM, add, [a, b], dict(gain=dev(g), bias=dev(bb), eps=1e-5), lambda: port.layer_norm(A, B, g, bb, 1e-5)),
        ("rmsnorm", jb.ROWS_RMSNORM, [L0], [a], dict(gain=dev(g), eps=1e-5), lambda: port.rms_norm(A, g, 1e-5)),
    ]:
        jb.eval_rows(kind, 1, prog, leaves, y, **kw)
        jb.eval_rows(kind, 1, prog + plus0, leaves, y2, **kw)
        assert_close(host(y), want(), FP32_RTOL, f"staged {name} {rows}x{cols}")
        assert torch.equal(y, y2), f"staged {name} differs from the register kernel ({rows}x{cols})"
    s, s2 = torch.empty(rows, 1, device="cuda"), torch.empty(rows, 1, device="cuda")
    for name, kind, prog, leaves in [("sum", jb.ROWS_SUM, [L0], [a]), ("mean", jb.ROWS_MEAN, [L0], [a]), ("max", jb.ROWS_MAX, [L0], [b]),
                                     ("sum(a+b)", jb.ROWS_SUM, add, [a, b]), ("max(a*0.125+b)", jb.ROWS_MAX, axpb, [a, b])]:
        jb.eval_rows(kind, 1, prog, leaves, s)
        jb.eval_rows(kind, 1, prog + plus0, leaves, s2)
        assert torch.equal(s, s2), f"staged row {name} differs from the register kernel ({rows}x{cols})"
    jb.eval_rows(jb.ROWS_SUM, 1, [L0], [a], s)
    assert float((s.ravel() - a.double().sum(dim=1).float()).abs().max()) < 1e-3
    jb.check(jb.lib().jsm_check_device_errors(jb.stream_ptr()))


def test_config2_full_size_properties():
    """Configuration 2 at 4096 x 4096: rows of the softmax sum to one, normalised rows have zero mean and
    unit variance, and 64 sampled rows equal the oracle."""
    n = 4096
    a = torch.empty(n, n, device="cuda"); b = torch.empty(n, n, device="cuda")
    jb.fill(a, 1, 0, 0, 0.0, 1.0); jb.fill(b, 1, 1, 0, 0.0, 1.0)
    g = torch.empty(n, device="cuda"); bb = torch.empty(n, device="cuda")
    jb.fill(g, 1, 2, 1, 0.5, 1.5); jb.fill(bb, 1, 3, 0, 0.0, 0.1)
    y = torch.empty_like(a)
    jb.eval_rows(jb.ROWS_SOFTMAX, 1, program_for(8, 0.125), [a, b], y)
    assert float((y.sum(dim=1) - 1).abs().max()) < 1e-5
    rows = np.arange(0, n, 64)
    A, B = host(a[rows]), host(b[rows])
    assert_close(host(y[rows]), port.hsoftmax(A, B, 0.125), FP32_RTOL, "cfg2 softmax")
    jb.eval_rows(jb.ROWS_LAYERNORM, 1, [L0, L1, (jb.OP_ADD,)], [a, b], y, gain=g, bias=bb, eps=1e-5)
    assert_close(host(y[rows]), port.layer_norm(A, B, host(g), host(bb), 1e-5), FP32_RTOL, "cfg2 layernorm")
    z = (y - bb) / g
    assert float(z.mean(dim=1).abs().max()) < 1e-4 and float((z.var(dim=1, unbiased=False) - 1).abs().max()) < 1e-3
    jb.eval_rows(jb.ROWS_RMSNORM, 1, [L0], [a], y, gain=g, eps=1e-5)
    assert_close(host(y[rows]), port.rms_norm(A, host(g), 1e-5), FP32_RTOL, "cfg2 rmsnorm")
    s = torch.empty(n, 1, device="cuda")
    jb.eval_rows(jb.ROWS_SUM, 1, [L0], [a], s)
    assert float((s.ravel() - a.double().sum(dim=1).float()).abs().max()) < 1e-3
    jb.eval_rows(jb.ROWS_MAX, 1, [L0], [a], s)
    assert torch.equal(s.ravel(), a.max(dim=1).values)
