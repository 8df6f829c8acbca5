"""GPU parity of RoPE and attention against the reference's golden vectors and the CPU oracle."""
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


def test_rope_reference_mode_matches_reference():
    """RoPE_net_t::forward over the whole feature vector, the reference's own table (two angles per block)."""
    x = cases.rope_input()
    T, d = x.shape
    table = jb.rope_table(0, d, 10000.0, T)
    assert np.array_equal(host(table), ol.rope_table(0, d, 10000.0, T))
    y = jb.rope_apply(dev(x), table, d, 1)
    assert np.array_equal(host(y), OPS["rope"])


def test_rope_standard_mode_matches_oracle():
    T, H, D = 37, 3, 128
    x = cases.normal((T, H * D), 620, 0)
    pos = np.arange(T, dtype=np.int32)[::-1].copy() * 3
    table = jb.rope_table(1, D, 10000.0, 128)
    tab_h = ol.rope_table(1, D, 10000.0, 128)
    assert np.array_equal(host(table), tab_h)
    y = jb.rope_apply(dev(x), table, D, H, positions=torch.from_numpy(pos).cuda())
    assert np.array_equal(host(y), ol.rope_apply(x, tab_h, D, H, pos))
    yb = jb.rope_apply(dev(x, torch.bfloat16), table, D, H, positions=torch.from_numpy(pos).cuda())
    xb = dev(x, torch.bfloat16).float().cpu().numpy()
    want_b = ol.rope_apply(xb, tab_h, D, H, pos)
    assert_close(host(yb), want_b, 8e-3, "bf16 rope")
    # the 128-bit bf16 kernel rounds every product on its own like the oracle: equal to the oracle rounded to bf16
    assert np.array_equal(host(yb), torch.from_numpy(want_b).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("T,Hq,Hkv", [(200, 32, 32), (96, 12, 4), (130, 5, 64)])
def test_rope_of_queries_and_keys_in_one_launch(T, Hq, Hkv):
    """jsm_rope_apply_qk rotates q and k of a prefill with one launch: bit-identical to two jsm_rope_apply calls."""
    D = 128
    q = dev(cases.normal((T, Hq * D), 625, 0), torch.bfloat16)
    k = dev(cases.normal((T, Hkv * D), 625, 1), torch.bfloat16)
    pos = torch.from_numpy((np.arange(T, dtype=np.int32) * 7) % 256).cuda()
    table = jb.rope_table(1, D, 10000.0, 256)
    qr, kr = jb.rope_apply_qk(q, k, table, D, Hq, Hkv, positions=pos)
    assert torch.equal(qr, jb.rope_apply(q, table, D, Hq, positions=pos))
    assert torch.equal(kr, jb.rope_apply(k, table, D, Hkv, positions=pos))
    qr2, kr2 = jb.rope_apply_qk(q, k, table, D, Hq, Hkv)           # positions 0..T-1
    assert torch.equal(qr2, jb.rope_apply(q, table, D, Hq)) and torch.equal(kr2, jb.rope_apply(k, table, D, Hkv))


def mha_device(w, x, H, causal):
    """mat_mha_t::forward (mat_mha_t.hpp:265-291) from C-ABI calls: block-diagonal per-head projections
    (each head sees its own slice, :199-215), attention, concatenation, output projection."""
    T, d = x.shape
    dh = d // H
    xd = dev(x)
    q = torch.empty(T, d, device="cuda"); k = torch.empty_like(q); v = torch.empty_like(q)
    o = 0
    for h in range(H):
        for dst in (q, k, v):
            W = dev(w[o:o + dh * dh].reshape(dh, dh)); o += dh * dh
            b = dev(w[o:o + dh].reshape(1, dh)); o += dh
            # token-major: Y[T,dh] = X_h[T,dh] . W^T + b, same k-ascending sums as W . X
            jb.dot_f32(xd[:, h * dh:(h + 1) * dh], W.t(), dst[:, h * dh:(h + 1) * dh], bias=b)
    att = jb.attn_prefill(q, k, v, 1, H, H, dh, causal=causal, impl=1)
    Wo = dev(w[o:o + d * d].reshape(d, d)); o += d * d
    bo = dev(w[o:o + d].reshape(1, d))
    out = torch.empty(T, d, device="cuda")
    jb.dot_f32(att, Wo.t(), out, bias=bo)
    return out


@pytest.mark.parametrize("causal", [True, False])
def test_mha_forward_matches_reference(causal):
    w, x = cases.mha_inputs()
    out = mha_device(w, x, cases.MHA["H"], causal)
    assert_close(host(out), OPS["mha_causal" if causal else "mha_full"], FP32_RTOL, "mat_mha_t::forward")


def test_causal_prefix_property_on_device():
    """test_sequence_mha (transformer_test.hpp:246-282): the outputs of a prefix do not change when
    later tokens are appended."""
    w, x = cases.mha_inputs()
    H = cases.MHA["H"]
    full = host(mha_device(w, x, H, True))
    for s1 in (1, 5):
        part = host(mha_device(w, x[:s1], H, True))
        assert_close(part, full[:s1], 1e-6, f"prefix {s1}")


@pytest.mark.parametrize("batch,Tq,Tk,Hq,Hkv,D", [(1, 1, 1, 1, 1, 2), (2, 9, 9, 4, 2, 32), (1, 70, 70, 2, 2, 128), (3, 5, 33, 8, 2, 64),
                                                  (1, 1, 100, 4, 4, 128), (2, 40, 40, 3, 1, 30)])
def test_attention_fp32_shapes(batch, Tq, Tk, Hq, Hkv, D):
    q = cases.normal((batch * Tq, Hq * D), 630, 0)
    k = cases.normal((batch * Tk, Hkv * D), 630, 1)
    v = cases.normal((batch * Tk, Hkv * D), 630, 2)
    for causal in (True, False):
        got = jb.attn_prefill(dev(q), dev(k), dev(v), batch, Hq, Hkv, D, causal=causal, impl=1)
        want = ol.attention(q, k, v, batch, Hq, Hkv, D, causal)
        assert_close(host(got), want, FP32_RTOL, f"attention causal={causal}")


def test_attention_with_fused_rope_fp32():
    batch, T, Hq, Hkv, D = 2, 19, 4, 2, 64
    q = cases.normal((batch * T, Hq * D), 640, 0)
    k = cases.normal((batch * T, Hkv * D), 640, 1)
    v = cases.normal((batch * T, Hkv * D), 640, 2)
    table = jb.rope_table(1, D, 10000.0, T)
    tab_h = ol.rope_table(1, D, 10000.0, T)
    pos = np.tile(np.arange(T, dtype=np.int32), batch)
    want = ol.attention(ol.rope_apply(q, tab_h, D, Hq, pos), ol.rope_apply(k, tab_h, D, Hkv, pos), v, batch, Hq, Hkv, D, True)
    got = jb.attn_prefill(dev(q), dev(k), dev(v), batch, Hq, Hkv, D, causal=True, rope=table, impl=1)
    assert_close(host(got), want, FP32_RTOL, "attention with RoPE on load")


def test_attention_bf16_cuda_core_matches_oracle():
    batch, T, Hq, Hkv, D = 1, 150, 4, 2, 128
    q = dev(cases.normal((batch * T, Hq * D), 650, 0), torch.bfloat16)
    k = dev(cases.normal((batch * T, Hkv * D), 650, 1), torch.bfloat16)
    v = dev(cases.normal((batch * T, Hkv * D), 650, 2), torch.bfloat16)
    got = jb.attn_prefill(q, k, v, batch, Hq, Hkv, D, causal=True, impl=1)
    want = ol.attention(host(q), host(k), host(v), batch, Hq, Hkv, D, True)
    assert_close(host(got), want, BF16_RTOL / 2, "bf16 attention")


def test_attention_argument_errors():
    z = torch.zeros(4, 6, device="cuda")
    with pytest.raises(jb.JsmError) as e:
        jb.attn_prefill(z, z, z, 1, 3, 2, 2)  # 3 query heads over 2 kv heads
    assert e.value.status == jb.SHAPE


# ---- tcgen05 flash-attention prefill (bf16, head_dim 128) ------------------------------------------
@pytest.mark.parametrize("batch,Tq,Tk,Hq,Hkv,causal", [(1, 128, 128, 1, 1, True), (1, 256, 256, 2, 2, True), (2, 300, 300, 4, 2, True),
                                                      (1, 1000, 1000, 2, 1, True), (1, 384, 384, 2, 2, False), (2, 200, 456, 2, 2, True),
                                                      (1, 130, 515, 4, 4, False)])
def test_flash_prefill_matches_oracle(batch, Tq, Tk, Hq, Hkv, causal):
    D = 128
    q = dev(cases.normal((batch * Tq, Hq * D), 660, 0), torch.bfloat16)
    k = dev(cases.normal((batch * Tk, Hkv * D), 660, 1), torch.bfloat16)
    v = dev(cases.normal((batch * Tk, Hkv * D), 660, 2), torch.bfloat16)
    got = jb.attn_prefill(q, k, v, batch, Hq, Hkv, D, causal=causal, impl=2)
    jb.check_device_errors()
    want = ol.attention(host(q), host(k), host(v), batch, Hq, Hkv, D, causal, exact_div=False)
    assert_close(host(got), want, 1e-2, f"flash B{batch} Tq{Tq} Tk{Tk} Hq{Hq} Hkv{Hkv} causal={causal}")


def test_flash_prefill_with_rope_matches_cuda_core_kernel():
    batch, T, Hq, Hkv, D = 2, 640, 4, 2, 128
    q = dev(cases.normal((batch * T, Hq * D), 670, 0), torch.bfloat16)
    k = dev(cases.normal((batch * T, Hkv * D), 670, 1), torch.bfloat16)
    v = dev(cases.normal((batch * T, Hkv * D), 670, 2), torch.bfloat16)
    table = jb.rope_table(1, D, 10000.0, T)
    a = jb.attn_prefill(q, k, v, batch, Hq, Hkv, D, causal=True, rope=table, impl=2)
    b = jb.attn_prefill(q, k, v, batch, Hq, Hkv, D, causal=True, rope=table, impl=1)
    assert_close(host(a), host(b), 1e-2, "flash vs CUDA-core kernel with RoPE")


def test_config3_full_size():
    """Configuration 3: batch 4, 32 heads, head_dim 128, seq 4096, causal, RoPE theta 10000, bf16 ~N(0,1) (seed 2):
    the tcgen05 kernel against the fp32 CUDA-core kernel on every row, and against the CPU oracle on two heads."""
    batch, T, H, D = 4, 4096, 32, 128
    q = torch.empty(batch * T, H * D, device="cuda", dtype=torch.bfloat16)
    k = torch.empty_like(q); v = torch.empty_like(q)
    jb.fill(q, 2, 0, 0, 0.0, 1.0); jb.fill(k, 2, 1, 0, 0.0, 1.0); jb.fill(v, 2, 2, 0, 0.0, 1.0)
    table = jb.rope_table(1, D, 10000.0, T)
    pos = torch.arange(T, dtype=torch.int32, device="cuda").repeat(batch)
    qr, kr = jb.rope_apply(q, table, D, H, positions=pos), jb.rope_apply(k, table, D, H, positions=pos)
    a = jb.attn_prefill(qr, kr, v, batch, H, H, D, causal=True, impl=2)
    jb.check_device_errors()
    b = jb.attn_prefill(qr, kr, v, batch, H, H, D, causal=True, impl=1)
    torch.cuda.synchronize()
    assert float((a.float() - b.float()).abs().max()) <= 1e-2 * float(b.float().abs().max())
    # causal row 0 attends only to key 0: the output is v[0]
    assert torch.equal(a[0], v[0])
    for (bb, hh) in ((0, 0), (3, 31)):
        rows = slice(bb * T, bb * T + 512)  # the first 512 queries only need the first 512 keys
        cols = slice(hh * D, (hh + 1) * D)
        want = ol.attention(host(qr[rows, cols]), host(kr[rows, cols]), host(v[rows, cols]), 1, 1, 1, D, True, exact_div=False)
        assert_close(host(a[rows, cols]), want, 1e-2, f"cfg3 oracle (batch {bb}, head {hh})")
