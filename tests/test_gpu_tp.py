"""GPU check of the tensor-parallel exchange kernel (sum of the ranks' buffers + residual add + RMSNorm) on ONE GPU:
the "ranks" are regions of the same device and every flag a kernel waits for has been set by the host before the
launch, so no kernel ever waits for another kernel.  The multi-GPU path itself runs in bench.py --gpus N."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
from gpu_util import assert_close, dev, host

pytestmark = pytest.mark.gpu


def make_regions(n, max_tokens, d):
    nbytes = jb.lib().jsm_tp_region_bytes(max_tokens, d)
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
    ptrs = (C.c_void_p * n)(*[r.data_ptr() for r in regions])
    return regions, ptrs


def buffer_view(region, which, max_tokens, d):
    off = 1024 + which * max_tokens * d * 2
    return region[off:off + max_tokens * d * 2].view(torch.bfloat16).view(max_tokens, d)


def set_flags(regions, epoch):
    for r in regions:
        r[:64].view(torch.int32).fill_(epoch)


@pytest.mark.parametrize("n,T,d", [(2, 8, 4096), (4, 5, 512), (8, 64, 1024), (3, 1, 256)])
def test_exchange_sums_in_rank_order_adds_and_normalises(n, T, d):
    max_tokens = 64
    regions, ptrs = make_regions(n, max_tokens, d)
    passes = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(n)]
    h0 = dev(cases.normal((T, d), 900, 0), torch.bfloat16)
    eps = 1e-5
    for call in range(3):                      # buffers A, B, A: epochs 1, 2, 3
        which = call % 2
        parts = [dev(cases.normal((T, d), 901 + call, r), torch.bfloat16) for r in range(n)]
        for r in range(n):
            buffer_view(regions[r], which, max_tokens, d)[:T] = parts[r]
        set_flags(regions, call + 1)           # every peer has "arrived" before any kernel starts
        s = torch.zeros(T, d, device="cuda")
        for r in range(n):
            s = s + parts[r].float()
        want_h = (h0.float() + s.to(torch.bfloat16).float()).to(torch.bfloat16)
        want_xn = want_h.float() / torch.sqrt((want_h.float() ** 2).mean(dim=1, keepdim=True) + eps)
        outs = []
        for r in range(n):
            h = h0.clone()
            xn = torch.empty_like(h)
            passes[r].fill_(call // 2)     # two exchanges per "pass": epochs 1, 2, 3
            jb.check(jb.lib().jsm_tp_allreduce_add_norm(ptrs, r, n, which, max_tokens, passes[r].data_ptr(), call % 2, 2,
                                                         h.data_ptr(), xn.data_ptr(), eps, T, d, jb.stream_ptr()))
            outs.append((h, xn))
        jb.check_device_errors()
        for r, (h, xn) in enumerate(outs):
            assert torch.equal(h, outs[0][0]), f"rank {r} differs from rank 0"
            assert_close(host(h), host(want_h), 1e-2, f"h of rank {r}, call {call}")   # one bf16 ulp of the sum order
            assert_close(host(xn), host(want_xn), 1e-2, f"xn of rank {r}, call {call}")
        h0 = outs[0][0]


def test_exchange_gives_up_when_a_peer_never_arrives():
    """A flag that nothing sets: the wait runs out after the (shortened) limit, h stays untouched and the host reads the
    error; the context stays usable."""
    n, T, d, max_tokens = 2, 4, 512, 16
    regions, ptrs = make_regions(n, max_tokens, d)
    state = torch.zeros(1, dtype=torch.int32, device="cuda")
    h = dev(cases.normal((T, d), 910, 0), torch.bfloat16)
    before = h.clone()
    jb.check(jb.lib().jsm_tp_set_wait_limit_ms(20))
    try:
        jb.check(jb.lib().jsm_tp_allreduce_add_norm(ptrs, 0, n, 0, max_tokens, state.data_ptr(), 0, 1, h.data_ptr(), None, 1e-5,
                                                     T, d, jb.stream_ptr()))
        with pytest.raises(jb.JsmError) as e:
            jb.check_device_errors()
        assert e.value.status == jb.TIMEOUT
        assert torch.equal(h, before)
        jb.check_device_errors()                # the error word was cleared; the device still answers
        assert int(torch.ones(4, device="cuda").sum()) == 4
    finally:
        jb.check(jb.lib().jsm_tp_set_wait_limit_ms(1000))


# ---- the exchange fused into the projections (push from the producer's epilogue, reduce in the consumer's prologue) ----
def _rms_rows(h, eps):
    return h.float() / torch.sqrt((h.float() ** 2).mean(dim=1, keepdim=True) + eps)


@pytest.mark.parametrize("n,T,d,K,N2", [(2, 8, 4096, 512, 1536), (8, 8, 4096, 1376, 2752), (4, 33, 1024, 256, 512),
                                        (3, 1, 256, 512, 256), (2, 64, 512, 1024, 384)])
def test_fused_exchange_push_then_reduce(n, T, d, K, N2):
    """All "ranks" are regions of one device.  First every rank's producer projection runs (it stores its tiles into its
    slot of every region and releases its flag - or, at up to 16 tokens, tags every stored word with the exchange's
    epoch), then every rank's consumer projection (it finds all flags set / all words of the epoch, adds the slots to h
    and projects the normalised h): no kernel ever waits for another.  Three exchanges: buffers 0, 1, 0."""
    max_tokens = 64
    regions, ptrs = make_regions(n, max_tokens, d)
    states = [torch.zeros(80, dtype=torch.int32, device="cuda") for _ in range(n)]
    eps = 1e-5
    W2 = dev(cases.normal((N2, d), 930, 0, 0.05), torch.bfloat16)
    W2p = jb.linear_pack(W2, N2)
    h = dev(cases.normal((T, d), 931, 0), torch.bfloat16)
    d_tiles = (d + 127) // 128
    for call in range(3):
        which, site = call % 2, call % 2
        Xs = [dev(cases.normal((T, K), 932 + call, r), torch.bfloat16) for r in range(n)]
        Ws = [dev(cases.normal((d, K), 940 + call, r, 0.05), torch.bfloat16) for r in range(n)]
        packed = [jb.linear_pack(w, d) for w in Ws]
        for r in range(n):
            states[r][0] = call // 2          # the forward pass: epochs 1, 2, 3
            jb.check(jb.lib().jsm_tp_linear_push(ptrs, r, n, which, max_tokens, states[r].data_ptr(), site, 2, Xs[r].data_ptr(),
                                                 packed[r].data_ptr(), T, d, K, jb.stream_ptr()))
        jb.check_device_errors()
        total = torch.zeros(T, d, device="cuda")
        for r in range(n):                    # rank order, each product rounded to bf16 as it was pushed
            total = total + (Xs[r].float() @ Ws[r].float().t()).to(torch.bfloat16).float()
        want_h = (h.float() + total.to(torch.bfloat16).float()).to(torch.bfloat16)
        want_y = _rms_rows(want_h, eps) @ W2.float().t()
        outs = []
        for r in range(n):
            hr = h.clone()
            ssq = torch.zeros(d_tiles, T, device="cuda")
            y = torch.empty(T, N2, device="cuda")
            jb.check(jb.lib().jsm_tp_linear_reduce(regions[r].data_ptr(), r, n, which, max_tokens, states[r].data_ptr(), site, 2,
                                                   hr.data_ptr(), ssq.data_ptr(), W2p.data_ptr(), 0, y.data_ptr(), jb.F32, T, N2, d,
                                                   eps, jb.stream_ptr()))
            outs.append((hr, ssq, y))
        jb.check_device_errors()
        for r, (hr, ssq, y) in enumerate(outs):
            assert torch.equal(hr, outs[0][0]), f"rank {r}: h differs from rank 0"
            assert torch.equal(y, outs[0][2]), f"rank {r}: projection differs from rank 0"
            assert_close(host(hr), host(want_h), 1e-2, f"h of rank {r}, exchange {call}")
            assert_close(host(ssq.sum(dim=0)), host((hr.float() ** 2).sum(dim=1)), 1e-5, f"row statistics of rank {r}")
            assert_close(host(y), host(want_y), 2e-2, f"projection of the normalised h, rank {r}, exchange {call}")
        h = outs[0][0]


def test_fused_exchange_gives_up_when_a_peer_never_pushes():
    """The consumer of an exchange whose peer never released its flag: the wait runs out after the (shortened) limit,
    h stays as it was, the host reads JSM_TIMEOUT and the device still answers."""
    n, T, d, N2, max_tokens = 2, 4, 512, 256, 64
    regions, ptrs = make_regions(n, max_tokens, d)
    # 4 tokens: the exchange would arrive as words that carry their epoch.  Those words have buffers of their own, so what
    # larger (plain bf16) exchanges left in the push buffers - here: bytes that would read as a far-future epoch - can never
    # pass for an arrived word
    inband0 = jb.lib().jsm_tp_inband_slot_offset(0, 0, max_tokens, d)
    assert 1024 < inband0 < regions[0].numel()
    regions[0][1024:inband0] = 0x3f
    state = torch.zeros(80, dtype=torch.int32, device="cuda")   # epoch 1 is expected; nothing was ever pushed
    W2p = jb.linear_pack(dev(cases.normal((N2, d), 950, 0, 0.05), torch.bfloat16), N2)
    h = dev(cases.normal((T, d), 951, 0), torch.bfloat16)
    before = h.clone()
    ssq = torch.zeros(4, T, device="cuda")
    y = torch.empty(T, N2, device="cuda")
    jb.check(jb.lib().jsm_tp_set_wait_limit_ms(20))
    try:
        jb.check(jb.lib().jsm_tp_linear_reduce(regions[0].data_ptr(), 0, n, 0, max_tokens, state.data_ptr(), 0, 1, h.data_ptr(),
                                               ssq.data_ptr(), W2p.data_ptr(), 0, y.data_ptr(), jb.F32, T, N2, d, 1e-5, jb.stream_ptr()))
        with pytest.raises(jb.JsmError) as e:
            jb.check_device_errors()
        assert e.value.status == jb.TIMEOUT
        assert torch.equal(h, before)
        jb.check_device_errors()
        assert int(torch.ones(4, device="cuda").sum()) == 4
    finally:
        jb.check(jb.lib().jsm_tp_set_wait_limit_ms(1000))


def test_argmax_exchange_over_vocabulary_shards():
    """The arg-max of a vocabulary-sharded lm_head: every rank contributes (best logit, global index) per token.  The
    peers' pairs are written into this rank's region by the host and their flags are set before the launch, so the one
    kernel of rank 1 never waits: it must publish its own pairs into every region and pick, per token, the largest value
    over the ranks (lowest index on a tie)."""
    n, T, d, max_tokens, rank = 4, 7, 512, 16, 1
    regions, ptrs = make_regions(n, max_tokens, d)
    nbytes = jb.lib().jsm_tp_region_bytes(max_tokens, d)
    slot0 = nbytes - 8 * max_tokens * 8                      # the arg-max slots are the last part of a region
    vals = cases.normal((n, T), 960, 0).astype(np.float32)
    idx = np.stack([cases.ints(T, 4, 961 + r, r * 1000, (r + 1) * 1000) for r in range(n)]).astype(np.int32)
    vals[2, 3] = vals[0, 3] = 9.0                            # a tie between ranks 0 and 2: the lower index (rank 0's) wins
    vals[3, 5] = 8.0
    for r in range(n):
        if r == rank:
            continue
        pairs = np.zeros((max_tokens, 2), np.uint32)
        pairs[:T, 0] = vals[r].view(np.uint32)
        pairs[:T, 1] = idx[r].view(np.uint32)
        off = slot0 + r * max_tokens * 8
        regions[rank][off:off + max_tokens * 8] = torch.from_numpy(pairs.view(np.uint8).reshape(-1)).cuda()
    regions[rank][128:128 + 32].view(torch.int32).fill_(1 << 30)   # flag words 32..39: every peer has "arrived"
    state = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((T,), -1, dtype=torch.int32, device="cuda")
    bv, bi = dev(vals[rank]), torch.from_numpy(idx[rank]).cuda()
    jb.check(jb.lib().jsm_tp_argmax_exchange(ptrs, rank, n, max_tokens, d, state.data_ptr(), 0, 1, bv.data_ptr(), bi.data_ptr(),
                                             out.data_ptr(), T, jb.stream_ptr()))
    jb.check_device_errors()
    want = []
    for t in range(T):
        best = max(range(n), key=lambda r: (vals[r, t], -idx[r, t]))
        want.append(int(idx[best, t]))
    assert out.cpu().tolist() == want
    # rank 1's own pairs reached its slot in every region, and its flag word in every peer's region holds epoch 1
    for r in range(n):
        off = slot0 + rank * max_tokens * 8
        got = regions[r][off:off + T * 8].cpu().numpy().view(np.uint32).reshape(T, 2)
        assert np.array_equal(got[:, 0], vals[rank].view(np.uint32)) and np.array_equal(got[:, 1], idx[rank].view(np.uint32))
        if r != rank:
            assert int(regions[r][128:128 + 32].view(torch.int32)[rank]) == 1
