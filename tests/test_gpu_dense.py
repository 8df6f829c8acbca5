"""GPU parity of the contractions: the fp32 dot (bit-exact against the reference's k-ascending sum) and
the bf16 projections (CUDA-core weight stream and tcgen05 kernel) with their epilogues."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
import oracle_lib as ol
from gpu_util import BF16_RTOL, FP32_RTOL, assert_close, dev, host

pytestmark = pytest.mark.gpu
OPS = np.load(Path(__file__).resolve().parent / "golden" / "ops.npz")
port = ol.port_oracle()


def test_dot_f32_bit_exact_with_reference():
    A, B = cases.dot_inputs()
    out = torch.empty(9, 5, device="cuda")
    jb.dot_f32(dev(A), dev(B), out)
    assert np.array_equal(host(out), OPS["dot"])


def test_weight_net_forward_bit_exact():
    """weight_net_t::forward (mat_net_t.hpp:38-43): Y = W.X + b in the reference's [features, tokens] orientation,
    here with X given token-major and read through a transposed view."""
    X, W, b = cases.linear_inputs()
    xd, wd, bd = dev(X), dev(W), dev(b.reshape(-1, 1))
    out = torch.empty(12, 7, device="cuda")
    jb.dot_f32(wd, xd.t(), out, bias=bd)
    assert np.array_equal(host(out).T, OPS["linear"])
    # relu epilogue = relu_net_t::forward applied to the same product
    jb.dot_f32(wd, xd.t(), out, bias=bd, epilogue=1)
    want = OPS["linear"].T
    assert np.array_equal(host(out), np.where(want > 0, want, 0 * want))


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (65, 130, 67), (128, 512, 256), (300, 77, 5)])
def test_dot_f32_shapes(M, K, N):
    A, B = cases.normal((M, K), 410, M), cases.normal((K, N), 411, N)
    out = torch.empty(M, N, device="cuda")
    jb.dot_f32(dev(A), dev(B), out)
    rc, want = port.dot(A, B)
    assert rc == 0 and np.array_equal(host(out), want)


def test_dot_shape_error():
    with pytest.raises(jb.JsmError) as e:
        jb.dot_f32(torch.zeros(3, 4, device="cuda"), torch.zeros(5, 2, device="cuda"), torch.zeros(3, 2, device="cuda"))
    assert e.value.status == jb.INVALID_ARG


def ref_linear(X, W, bias=None):
    y = X.float() @ W.float().t()
    return y + bias if bias is not None else y


def make_xw(T, N, K, seed, rows=None):
    X = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
    W = torch.empty(rows or N, K, device="cuda", dtype=torch.bfloat16)
    jb.fill(X, seed, 0, 0, 0.0, 1.0)
    jb.fill(W, seed, 1, 0, 0.0, 0.05)
    return X, W


@pytest.mark.parametrize("T", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(512, 1024), (1000, 4096), (64, 11008)])
def test_linear_bf16_weight_stream(T, N, K):
    X, W = make_xw(T, N, K, 20 + T)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    jb.linear_bf16(X, W, Y)
    assert_close(host(Y), host(ref_linear(X, W)), 2e-3, f"gemv T={T} N={N} K={K}")


@pytest.mark.parametrize("T,N,K", [(8, 256, 512), (16, 128, 64), (5, 384, 4096), (64, 4096, 4096), (64, 256, 11008),
                                   (100, 1000, 1000), (128, 256, 256), (200, 512, 1024), (512, 384, 512)])
def test_linear_bf16_tcgen05(T, N, K):
    X, W = make_xw(T, N, K, 40 + T)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    jb.linear_bf16(X, W, Y)
    torch.cuda.synchronize()
    assert_close(host(Y), host(ref_linear(X, W)), 2e-3, f"tcgen05 T={T} N={N} K={K}")
    Yb = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    jb.linear_bf16(X, W, Yb)
    assert_close(host(Yb), host(ref_linear(X, W)), BF16_RTOL, "bf16 output")


@pytest.mark.parametrize("T", [2, 32])
def test_linear_bf16_epilogues(T):
    N, K = 256, 512
    X, W = make_xw(T, N, K, 60 + T, rows=2 * N)
    bias = torch.empty(N, device="cuda"); jb.fill(bias, 61, 2, 0, 0.0, 0.5)
    R = torch.empty(T, N, device="cuda", dtype=torch.bfloat16); jb.fill(R, 61, 3, 0, 0.0, 1.0)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    base = ref_linear(X, W[:N], bias)
    jb.linear_bf16(X, W, Y, bias=bias, epilogue=1)
    assert_close(host(Y), host(torch.relu(base)), 2e-3, "relu")
    jb.linear_bf16(X, W, Y, bias=bias, epilogue=2)
    assert_close(host(Y), host(torch.nn.functional.gelu(base)), 2e-3, "gelu")
    jb.linear_bf16(X, W, Y, bias=bias, epilogue=4, residual=R)
    assert_close(host(Y), host(base + R.float()), 2e-3, "residual")
    jb.linear_bf16(X, W, Y, epilogue=3)
    gate, up = ref_linear(X, W[:N]), ref_linear(X, W[N:])
    assert_close(host(Y), host(torch.nn.functional.silu(gate) * up), 3e-3, "silu(gate)*up")


# ---- packed weights: one linear stream split evenly over the SMs (stream-K), shared tiles folded in slot order ----
PACKED_SHAPES = [(1, 256, 512), (8, 4096, 4096), (8, 12288, 4096), (5, 1000, 1000), (16, 384, 64), (17, 512, 1024),
                 (64, 4096, 11008), (64, 1376, 4096), (100, 1024, 1376), (128, 256, 256), (200, 640, 1024), (256, 4096, 512),
                 (300, 384, 512), (512, 256, 2048), (2, 32000, 512)]


@pytest.mark.parametrize("T,N,K", PACKED_SHAPES)
def test_linear_packed(T, N, K):
    X, W = make_xw(T, N, K, 140 + T)
    Wp = jb.linear_pack(W, N)
    assert torch.equal(jb.linear_unpack(Wp, N, K), W), "pack / unpack round trip"
    want = host(ref_linear(X, W))
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    jb.linear_bf16_packed(X, Wp, Y)
    jb.check_device_errors()
    assert_close(host(Y), want, 2e-3, f"packed T={T} N={N} K={K}")
    # the fold of shared tiles is ordered: a second run gives the same bits
    Y2 = torch.empty_like(Y)
    jb.linear_bf16_packed(X, Wp, Y2)
    assert torch.equal(Y, Y2)
    Yb = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    jb.linear_bf16_packed(X, Wp, Yb)
    assert_close(host(Yb), want, BF16_RTOL, "bf16 output")


@pytest.mark.parametrize("T,N,K", [(8, 11008, 4096), (64, 4096, 11008), (8, 12288, 4096)])
def test_linear_packed_against_the_oracle(T, N, K):
    """The projection shapes of the 7B decoder against the CPU oracle's weight_net_t::forward restatement (k-ascending
    fp32 sums of the same bf16 inputs), not only against torch."""
    X, W = make_xw(T, N, K, 170 + T)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    jb.linear_bf16_packed(X, jb.linear_pack(W, N), Y)
    jb.check_device_errors()
    want = port.linear(host(X), host(W), np.zeros(N, np.float32))
    assert_close(host(Y), want, 2e-3, f"packed vs oracle T={T} N={N} K={K}")


def test_linear_packed_chained_launches_give_the_same_bits():
    """jsm_linear_bf16_packed_chained (each launch a link of a kernel chain: resident and fetching weights while its
    predecessor finishes) against the plain call: a chain of projections that feed one another, results bit-equal."""
    T, d, ffn = 8, 1024, 2816
    X, Wgu = make_xw(T, 2 * ffn, d, 190)
    _, Wd = make_xw(T, d, ffn, 191)
    jb.fill(Wgu, 190, 1, 0, 0.0, 0.01)           # small weights: the update is quadratic in h and must stay bounded
    jb.fill(Wd, 191, 1, 0, 0.0, 0.01)
    Pgu, Pd = jb.linear_pack(Wgu, ffn, paired=True), jb.linear_pack(Wd, d)

    def run(chained):
        h = X.clone()
        act = torch.empty(T, ffn, device="cuda", dtype=torch.bfloat16)
        for _ in range(6):                       # h += down(silu(gate(h)) * up(h)), six times back to back
            jb.linear_bf16_packed(h, Pgu, act, epilogue=3, chained=chained)
            jb.linear_bf16_packed(act, Pd, h, epilogue=4, residual=h, chained=chained)
        jb.check_device_errors()
        return h

    with torch.cuda.stream(torch.cuda.Stream()):
        plain, chained = run(False), run(True)
        torch.cuda.current_stream().synchronize()
    assert torch.isfinite(plain.float()).all()
    assert torch.equal(plain, chained)


def test_linear_packed_needs_a_reserved_workspace():
    """The compute call never allocates: a packed image that did not come from jsm_linear_pack on this device (loaded
    from a file, say) needs jsm_linear_packed_reserve once, at set-up time; without it the call is refused."""
    T, N, K = 8, 1100 * 128, 64                  # more tiles (arrival counters) than any shape another test packs
    Wp = torch.zeros(jb.lib().jsm_linear_packed_bytes(N, K, 0), dtype=torch.uint8, device="cuda")
    X = torch.zeros(T, K, device="cuda", dtype=torch.bfloat16)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    with pytest.raises(jb.JsmError) as e:
        jb.linear_bf16_packed(X, Wp, Y)
    assert e.value.status == jb.INVALID_ARG
    jb.check(jb.lib().jsm_linear_packed_reserve(N, K, 0))
    jb.linear_bf16_packed(X, Wp, Y)
    jb.check_device_errors()
    assert float(Y.abs().max()) == 0.0


@pytest.mark.parametrize("T,N,K", [(1, 256, 512), (8, 11008, 4096), (32, 1376, 512), (64, 704, 1024), (130, 320, 256)])
def test_linear_packed_epilogues(T, N, K):
    X, W = make_xw(T, N, K, 160 + T, rows=2 * N)
    bias = torch.empty(N, device="cuda"); jb.fill(bias, 161, 2, 0, 0.0, 0.5)
    R = torch.empty(T, N, device="cuda", dtype=torch.bfloat16); jb.fill(R, 161, 3, 0, 0.0, 1.0)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    Wp = jb.linear_pack(W[:N].contiguous(), N)
    base = ref_linear(X, W[:N], bias)
    jb.linear_bf16_packed(X, Wp, Y, bias=bias, epilogue=1)
    assert_close(host(Y), host(torch.relu(base)), 2e-3, "relu")
    jb.linear_bf16_packed(X, Wp, Y, bias=bias, epilogue=2)
    assert_close(host(Y), host(torch.nn.functional.gelu(base)), 2e-3, "gelu")
    jb.linear_bf16_packed(X, Wp, Y, bias=bias, epilogue=4, residual=R)
    assert_close(host(Y), host(base + R.float()), 2e-3, "residual")
    # in place on the residual stream, as the decoder uses it
    H = R.clone()
    jb.linear_bf16_packed(X, Wp, H, epilogue=4, residual=H)
    assert_close(host(H), host(ref_linear(X, W[:N]) + R.float()), BF16_RTOL, "residual in place")
    Wpair = jb.linear_pack(W, N, paired=True)
    assert torch.equal(jb.linear_unpack(Wpair, N, K, paired=True), W), "paired pack / unpack round trip"
    jb.linear_bf16_packed(X, Wpair, Y, epilogue=3)
    gate, up = ref_linear(X, W[:N]), ref_linear(X, W[N:])
    assert_close(host(Y), host(torch.nn.functional.silu(gate) * up), 3e-3, "silu(gate)*up")
    jb.check_device_errors()


def test_linear_matches_oracle_on_small_case():
    """The bf16 projection against the CPU oracle's weight_net_t restatement on bf16-rounded inputs."""
    T, N, K = 6, 128, 256
    X, W = make_xw(T, N, K, 70)
    Y = torch.empty(T, N, device="cuda", dtype=torch.float32)
    jb.linear_bf16(X, W, Y)
    want = port.linear(host(X), host(W), np.zeros(N, np.float32))
    assert_close(host(Y), want, 1e-4, "oracle linear")
