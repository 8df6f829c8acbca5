"""GPU parity of the paged KV cache: append, split-K decode attention (ragged context lengths, GQA,
shuffled pages) against the CPU oracle's attention on the same bf16 values."""
import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
import oracle_lib as ol
from gpu_util import assert_close, dev, host

pytestmark = pytest.mark.gpu
D = 128


def build_cache(lens, Hkv, seed, rope_table=None, shuffle=True):
    n = len(lens)
    max_pages = (max(lens) + jb.PAGE_SIZE - 1) // jb.PAGE_SIZE
    n_pages = n * max_pages
    rng = np.random.default_rng(seed)
    perm = rng.permutation(n_pages).astype(np.int32) if shuffle else np.arange(n_pages, dtype=np.int32)
    block_table = torch.from_numpy(perm.reshape(n, max_pages)).cuda()
    pool = torch.zeros(n_pages, 2, Hkv, jb.PAGE_SIZE, D, device="cuda", dtype=torch.bfloat16)
    total = int(sum(lens))
    k = dev(cases.normal((total, Hkv * D), seed, 1), torch.bfloat16)
    v = dev(cases.normal((total, Hkv * D), seed, 2), torch.bfloat16)
    seq_ids = np.concatenate([np.full(L, i, np.int32) for i, L in enumerate(lens)])
    positions = np.concatenate([np.arange(L, dtype=np.int32) for L in lens])
    jb.kv_append(pool, block_table, k, v, torch.from_numpy(seq_ids).cuda(), torch.from_numpy(positions).cuda(), Hkv, D,
                 rope=rope_table)
    return pool, block_table, host(k), host(v), seq_ids, positions


@pytest.mark.parametrize("Hq,Hkv", [(4, 4), (8, 2), (8, 1), (4, 2)])
def test_decode_attention_ragged_contexts(Hq, Hkv):
    lens = [1, 7, 63, 64, 65, 511, 512, 513, 1300]
    pool, bt, k, v, seq_ids, _ = build_cache(lens, Hkv, 800 + Hq)
    q = dev(cases.normal((len(lens), Hq * D), 801, 0), torch.bfloat16)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, max(lens))
    qh = host(q)
    o = 0
    for i, L in enumerate(lens):
        want = ol.attention(qh[i:i + 1], k[o:o + L], v[o:o + L], 1, Hq, Hkv, D, False, exact_div=False)
        assert_close(host(out[i:i + 1]), want, 1e-2, f"sequence {i} (context {L})")
        o += L


def test_append_and_decode_with_rope():
    Hq, Hkv = 4, 2
    lens = [5, 130, 600]
    table = jb.rope_table(1, D, 10000.0, 1024)
    tab_h = ol.rope_table(1, D, 10000.0, 1024)
    pool, bt, k, v, seq_ids, positions = build_cache(lens, Hkv, 810, rope_table=table)
    # what the cache must hold: rotated keys rounded to bf16, values unchanged
    k_rot = dev(ol.rope_apply(k, tab_h, D, Hkv, positions), torch.bfloat16)
    kp = host(k_rot)
    o = 0
    for i, L in enumerate(lens):
        for pos in (0, L - 1):
            page = int(bt[i, pos // jb.PAGE_SIZE])
            got_k = host(pool[page, 0, :, pos % jb.PAGE_SIZE, :]).reshape(-1)
            got_v = host(pool[page, 1, :, pos % jb.PAGE_SIZE, :]).reshape(-1)
            assert np.array_equal(got_k, kp[o + pos]) and np.array_equal(got_v, v[o + pos])
        o += L
    q = dev(cases.normal((len(lens), Hq * D), 811, 0), torch.bfloat16)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, 1024, rope=table)
    qh = host(q)
    o = 0
    for i, L in enumerate(lens):
        q_rot = host(dev(ol.rope_apply(qh[i:i + 1], tab_h, D, Hq, np.array([L - 1], np.int32)), torch.bfloat16))
        want = ol.attention(q_rot, kp[o:o + L], v[o:o + L], 1, Hq, Hkv, D, False, exact_div=False)
        assert_close(host(out[i:i + 1]), want, 1e-2, f"rope sequence {i}")
        o += L


@pytest.mark.parametrize("Hq,Hkv,use_rope", [(4, 4, True), (8, 2, True), (4, 1, False)])
def test_fused_append_decode_equals_append_then_decode(Hq, Hkv, use_rope):
    """jsm_attn_decode_append (one launch: append + attention + merge) against jsm_kv_append followed by
    jsm_attn_decode on a copy of the same cache: same cache contents bit for bit, same outputs; repeated for three
    steps so that the self-resetting counters and the growing contexts are exercised (context 64 -> 65 crosses a page)."""
    lens = [1, 63, 64, 129, 700, 1299]
    n = len(lens)
    table = jb.rope_table(1, D, 10000.0, 2048) if use_rope else None
    pool, bt, *_ = build_cache(lens, Hkv, 830 + Hq, rope_table=table)
    pool_ref = pool.clone()
    counters = torch.zeros(n * Hkv, dtype=torch.int32, device="cuda")
    ctx_len = list(lens)
    for step in range(3):
        qkv = dev(cases.normal((n, (Hq + 2 * Hkv) * D), 840 + step, 0), torch.bfloat16)
        q, k_new, v_new = qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]
        pos = torch.tensor(ctx_len, dtype=torch.int32, device="cuda")
        ctx_len = [c + 1 for c in ctx_len]
        ctx = torch.tensor(ctx_len, dtype=torch.int32, device="cuda")
        jb.kv_append(pool_ref, bt, k_new, v_new, torch.arange(n, dtype=torch.int32, device="cuda"), pos, Hkv, D, rope=table)
        want = jb.attn_decode(q, pool_ref, bt, ctx, Hq, Hkv, D, 2048, rope=table)
        got = jb.attn_decode_append(q, k_new, v_new, pool, bt, ctx, Hq, Hkv, D, 2048, counters, rope=table)
        torch.cuda.synchronize()
        assert torch.equal(pool, pool_ref), f"cache contents differ at step {step}"
        assert_close(host(got), host(want), 1e-6, f"fused decode step {step}")
        assert int(counters.abs().sum()) == 0, "counters must be left at zero"


@pytest.mark.parametrize("Hq,Hkv", [(4, 4), (8, 2), (8, 1), (4, 2)])
def test_decode_ignores_cache_past_context(Hq, Hkv):
    """Whatever the last page holds past the context length (NaN here) must not reach the result."""
    lens = [1, 17, 63, 64, 65, 200, 1000]
    pool, bt, *_ = build_cache(lens, Hkv, 860 + Hq)
    q = dev(cases.normal((len(lens), Hq * D), 861, 0), torch.bfloat16)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    want = jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, max(lens))
    for i, L in enumerate(lens):
        if L % jb.PAGE_SIZE:
            pool[int(bt[i, (L - 1) // jb.PAGE_SIZE]), :, :, L % jb.PAGE_SIZE:, :] = float("nan")
    got = jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, max(lens))
    assert torch.isfinite(got.float()).all()
    assert torch.equal(got, want)


def test_decode_equals_prefill_last_row():
    """KV-cache decode == attention of the last query over the whole prefix (the recompute the reference does)."""
    Hq, Hkv, L = 4, 4, 200
    pool, bt, k, v, _, _ = build_cache([L], Hkv, 820, shuffle=False)
    q = dev(cases.normal((L, Hq * D), 821, 0), torch.bfloat16)
    full = jb.attn_prefill(q, dev(k, torch.bfloat16), dev(v, torch.bfloat16), 1, Hq, Hkv, D, causal=True, impl=1)
    ctx = torch.tensor([L], dtype=torch.int32, device="cuda")
    last = jb.attn_decode(q[L - 1:L].contiguous(), pool, bt, ctx, Hq, Hkv, D, L)
    assert_close(host(last), host(full[L - 1:L]), 1e-2, "decode vs prefill")


def test_config4_shape_properties():
    """Configuration 4: 64 sequences, 32 query / 8 kv heads, contexts uniform in [512, 8192] (seed 3):
    every output row is a convex combination of the cached values, and sampled sequences equal the oracle."""
    Hq, Hkv, n = 32, 8, 64
    lens = cases.ints(n, 3, 0, 512, 8193).tolist()
    max_ctx = 8192
    max_pages = max_ctx // jb.PAGE_SIZE
    pool = torch.empty(n * max_pages, 2, Hkv, jb.PAGE_SIZE, D, device="cuda", dtype=torch.bfloat16)
    jb.fill(pool, 3, 1, 0, 0.0, 1.0)
    bt = torch.arange(n * max_pages, dtype=torch.int32, device="cuda").reshape(n, max_pages)
    q = torch.empty(n, Hq * D, device="cuda", dtype=torch.bfloat16)
    jb.fill(q, 3, 2, 0, 0.0, 1.0)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, max_ctx)
    assert torch.isfinite(out.float()).all()
    for i in (0, 17, 63):
        L = lens[i]
        pages = pool[bt[i, :(L + 63) // 64].long()]               # [p, 2, Hkv, 64, D]
        kk = pages[:, 0].permute(0, 2, 1, 3).reshape(-1, Hkv * D)[:L]
        vv = pages[:, 1].permute(0, 2, 1, 3).reshape(-1, Hkv * D)[:L]
        want = ol.attention(host(q[i:i + 1]), host(kk), host(vv), 1, Hq, Hkv, D, False, exact_div=False)
        assert_close(host(out[i:i + 1]), want, 1e-2, f"cfg4 sequence {i}")
        vmax = vv.float().reshape(L, Hkv, D).amax(dim=0).repeat_interleave(Hq // Hkv, dim=0).reshape(-1)
        assert bool((out[i].float() <= vmax + 1e-2).all())
