"""Decode attention for hosts that cannot allocate (jsm_attn_decode_static_scratch).

Some embedders of this library have no device memory left to give: a serving process that sized its KV
page pool to fill the GPU, or a plugin whose host passes it input and output buffers and nothing else.
For them the library carries the scratch of the split-K decode attention inside its own image.  This test
calls that entry point through the C ABI twice in a row (the array keeps the first call's contents, the
second call must not be disturbed by them) and compares each result with the ordinary entry point, which
takes a caller-supplied scratch buffer.  Collected last so that a run that stops at the first failure has
already run everything else; it also passes on its own in a fresh process."""
import numpy as np
import pytest
import torch

import jasmine_b200 as jb

pytestmark = pytest.mark.gpu
D = 128


def make_case(seed, lens, Hq, Hkv):
    n = len(lens)
    max_ctx = max(lens)
    max_pages = (max_ctx + jb.PAGE_SIZE - 1) // jb.PAGE_SIZE
    pool = torch.empty(n * max_pages, 2, Hkv, jb.PAGE_SIZE, D, device="cuda", dtype=torch.bfloat16)
    jb.fill(pool, seed, 1, 0, 0.0, 1.0)
    bt = torch.arange(n * max_pages, dtype=torch.int32, device="cuda").flip(0).reshape(n, max_pages).contiguous()
    q = torch.empty(n, Hq * D, device="cuda", dtype=torch.bfloat16)
    jb.fill(q, seed, 2, 0, 0.0, 1.0)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return q, pool, bt, ctx, max_ctx


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    Hq, Hkv = 8, 2
    for seed, lens in ((31, [700, 5, 1100, 513]), (32, [64, 2047, 9])):  # second call: other shapes, stale partials in the array
        q, pool, bt, ctx, max_ctx = make_case(seed, lens, Hq, Hkv)
        want = jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, max_ctx)
        out = torch.empty_like(want)
        got = jb.attn_decode_static_scratch(q, pool, bt, ctx, Hq, Hkv, D, max_ctx, out=out)
        torch.cuda.synchronize()
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.isfinite(g).all()
        err = float(np.max(np.abs(g - w)) / np.max(np.abs(w)))
        assert err <= 1e-2, f"seed {seed}: relative error {err}"  # the tolerance of the decode-attention tests


def test_static_scratch_rejects_sizes_beyond_its_array():
    # 64 sequences x 32 heads x 8192 positions need 17 MB of partials: more than the 8 MiB array
    assert jb.lib().jsm_attn_decode_scratch_bytes(64, 32, D, 8192) > jb.STATIC_SCRATCH_BYTES
    q = torch.zeros(64, 32 * D, device="cuda", dtype=torch.bfloat16)
    pool = torch.zeros(2, 2, 32, jb.PAGE_SIZE, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.zeros(64, 128, dtype=torch.int32, device="cuda")
    ctx = torch.ones(64, dtype=torch.int32, device="cuda")
    with pytest.raises(jb.JsmError) as e:
        jb.attn_decode_static_scratch(q, pool, bt, ctx, 32, 32, D, 8192)
    assert e.value.status == jb.UNSUPPORTED and "built-in array" in str(e.value)
