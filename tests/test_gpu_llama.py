"""GPU parity of the LLaMA-shape decoder (prefill, paged-cache greedy decode) against the CPU oracle's
full-prefix recompute on the same bf16 weights."""
import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
import oracle_lib as ol
from gpu_util import BF16_RTOL, assert_close, host
from jasmine_b200.model import Llama

pytestmark = pytest.mark.gpu


def oracle_weights(m, cfg, tp_rank=0, tp_size=1):
    Hq, Hkv, D, ffn = cfg["Hq"] // tp_size, cfg["Hkv"] // tp_size, cfg["D"], cfg["ffn"] // tp_size
    d = cfg["d"]
    layers = []
    for l in range(cfg["L"]):
        wqkv = m.weight(f"layers.{l}.wqkv").reshape(-1, d)
        wq, wk, wv = wqkv[:Hq * D], wqkv[Hq * D:(Hq + Hkv) * D], wqkv[(Hq + Hkv) * D:]
        wgu = m.weight(f"layers.{l}.wgu").reshape(-1, d)
        layers.append((m.weight(f"layers.{l}.g1"), wq, wk, wv, m.weight(f"layers.{l}.wo").reshape(d, Hq * D),
                       m.weight(f"layers.{l}.g2"), wgu[:ffn], wgu[ffn:], m.weight(f"layers.{l}.wdown").reshape(d, ffn)))
    return m.weight("emb").reshape(-1, d), layers, m.weight("gf"), m.weight("lm_head").reshape(-1, d)


@pytest.mark.parametrize("Hq,Hkv,batch", [(2, 2, 2), (4, 1, 3), (4, 2, 8)])
def test_prefill_and_greedy_decode_match_oracle(Hq, Hkv, batch):
    cfg = dict(L=2, d=256, Hq=Hq, Hkv=Hkv, D=128, ffn=512, vocab=1024, eps=1e-5, theta=10000.0)
    T, n_gen = 40, 6
    m = Llama(cfg["L"], cfg["d"], Hq, Hkv, cfg["ffn"], cfg["vocab"], max_batch=batch, max_context=128, seed=4)
    emb, layers, gf, wlm = oracle_weights(m, cfg)
    prompts = [cases.ints(T, 4, 100 + b, 0, cfg["vocab"]) for b in range(batch)]
    nxt = torch.zeros(batch, dtype=torch.int32, device="cuda")
    last_logits = torch.empty(cfg["vocab"], device="cuda")
    seqs = [list(p) for p in prompts]
    for b in range(batch):
        m.prefill(torch.from_numpy(prompts[b]).cuda(), b, nxt, last_logits)
        want = ol.llama_forward(cfg, emb, layers, gf, wlm, prompts[b])[-1]
        assert_close(host(last_logits), want, BF16_RTOL, f"prefill logits of sequence {b}")
    logits = torch.empty(batch, cfg["vocab"], device="cuda")
    for step in range(n_gen):
        tokens = nxt.clone()
        for b in range(batch):
            seqs[b].append(int(tokens[b]))
        m.decode_step(tokens, nxt, logits)
        got = host(logits)
        for b in range(batch):
            want = ol.llama_forward(cfg, emb, layers, gf, wlm, np.array(seqs[b], np.int32))[-1]
            assert_close(got[b], want, BF16_RTOL, f"decode step {step} sequence {b}")
            top = np.sort(want)[-2:]
            if top[1] - top[0] > 2 * BF16_RTOL * float(np.abs(want).max()):  # a clear winner must be reproduced
                assert int(nxt[b]) == int(np.argmax(want)), f"greedy token differs at step {step}, sequence {b}"
    m.close()


def test_decode_step_is_replayable_in_a_cuda_graph():
    """The step keeps its positions on the device, so a captured step can be replayed: graph replay == eager."""
    cfg = dict(L=2, d=256, Hq=2, Hkv=2, D=128, ffn=512, vocab=1024)
    outs = []
    for use_graph in (False, True):
        m = Llama(cfg["L"], cfg["d"], 2, 2, cfg["ffn"], cfg["vocab"], max_batch=2, max_context=128, seed=4)
        nxt = torch.zeros(2, dtype=torch.int32, device="cuda")
        for b in range(2):
            m.prefill(torch.from_numpy(cases.ints(20, 4, 200 + b, 0, 1024)).cuda(), b, nxt)
        ids = nxt.clone()
        toks = []
        if use_graph:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                m.decode_step(ids, nxt)  # warm-up outside capture (first-use set-up)
                m.set_context(0, 20); m.set_context(1, 20)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    m.decode_step(ids, nxt)
            torch.cuda.current_stream().wait_stream(s)
            for _ in range(5):
                g.replay()
                torch.cuda.synchronize()
                toks.append(nxt.cpu().tolist())
                ids.copy_(nxt)
        else:
            for _ in range(5):
                m.decode_step(ids, nxt)
                toks.append(nxt.cpu().tolist())
                ids.copy_(nxt)
        outs.append(toks)
        m.close()
    assert outs[0] == outs[1]


def _greedy(m, prompts, n_gen, vocab):
    batch = len(prompts)
    nxt = torch.zeros(batch, dtype=torch.int32, device="cuda")
    for b in range(batch):
        m.prefill(torch.from_numpy(prompts[b]).cuda(), b, nxt)
    logits = torch.empty(batch, vocab, device="cuda")
    toks = []
    for _ in range(n_gen):
        ids = nxt.clone()
        toks.append(ids.cpu().numpy().copy())
        m.decode_step(ids, nxt, logits)
    return np.stack(toks), host(logits)


def test_checkpoint_round_trip_and_weight_injection(tmp_path):
    """(1) save / load: a model created from another seed generates the saved model's tokens and logits, bit for bit,
    after loading its checkpoint; a checkpoint of another shape is refused.  (2) weight injection with gains that are
    not one: the model with injected (g1, g2, gf, un-folded projections) matches the oracle run on the same tensors."""
    cfg = dict(L=2, d=256, Hq=4, Hkv=2, D=128, ffn=512, vocab=1024, eps=1e-5, theta=10000.0)
    mk = lambda seed, L=2: Llama(L, cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["ffn"], cfg["vocab"], max_batch=2, max_context=128, seed=seed)
    prompts = [cases.ints(24, 4, 300 + b, 0, cfg["vocab"]) for b in range(2)]
    a, b = mk(11), mk(12)
    ta, la = _greedy(a, prompts, 4, cfg["vocab"])
    tb, _ = _greedy(b, prompts, 4, cfg["vocab"])
    assert not np.array_equal(ta, tb)
    path = tmp_path / "model.jsmckpt"
    a.save(path)
    b.reset()
    b.load(path)
    tb, lb = _greedy(b, prompts, 4, cfg["vocab"])
    assert np.array_equal(ta, tb) and np.array_equal(la, lb)
    other = mk(13, L=1)
    with pytest.raises(jb.JsmError):
        other.load(path)
    other.close()
    # ---- injection: tensors made here, gains in [0.5, 1.5]
    d, D, ffn, V = cfg["d"], cfg["D"], cfg["ffn"], cfg["vocab"]
    bf = lambda x: torch.from_numpy(x).cuda().to(torch.bfloat16)
    wide = lambda t: t.float().cpu().numpy()
    b.reset()
    layers = []
    emb = bf(cases.normal((V, d), 21, 0, 0.02)); b.set_weight("emb", emb)
    gf = torch.from_numpy(cases.uniform((d,), 21, 1, 0.5, 1.5)).cuda(); b.set_weight("gf", gf)
    wlm = bf(cases.normal((V, d), 21, 2, 0.02)); b.set_weight("lm_head", wlm)
    for l in range(cfg["L"]):
        g1 = torch.from_numpy(cases.uniform((d,), 22 + l, 0, 0.5, 1.5)).cuda()
        g2 = torch.from_numpy(cases.uniform((d,), 22 + l, 1, 0.5, 1.5)).cuda()
        wqkv = bf(cases.normal(((cfg["Hq"] + 2 * cfg["Hkv"]) * D, d), 22 + l, 2, 0.02))
        wo = bf(cases.normal((d, cfg["Hq"] * D), 22 + l, 3, 0.02))
        wgu = bf(cases.normal((2 * ffn, d), 22 + l, 4, 0.02))
        wdown = bf(cases.normal((d, ffn), 22 + l, 5, 0.02))
        b.set_weight(f"layers.{l}.g1", g1); b.set_weight(f"layers.{l}.g2", g2)   # gains first
        b.set_weight(f"layers.{l}.wqkv", wqkv); b.set_weight(f"layers.{l}.wo", wo)
        b.set_weight(f"layers.{l}.wgu", wgu); b.set_weight(f"layers.{l}.wdown", wdown)
        q = wide(wqkv)
        layers.append((g1.cpu().numpy(), q[:cfg["Hq"] * D], q[cfg["Hq"] * D:(cfg["Hq"] + cfg["Hkv"]) * D], q[(cfg["Hq"] + cfg["Hkv"]) * D:],
                       wide(wo), g2.cpu().numpy(), wide(wgu)[:ffn], wide(wgu)[ffn:], wide(wdown)))
    nxt = torch.zeros(2, dtype=torch.int32, device="cuda")
    last = torch.empty(V, device="cuda")
    for s in range(2):
        b.prefill(torch.from_numpy(prompts[s]).cuda(), s, nxt, last)
        want = ol.llama_forward(cfg, wide(emb), layers, gf.cpu().numpy(), wide(wlm), prompts[s])[-1]
        assert_close(host(last), want, BF16_RTOL, f"injected weights, prefill logits of sequence {s}")
    a.close(); b.close()


def test_full_width_layers_match_oracle():
    """Configuration 5 at full width: two decoder layers of the 7B shape (d 4096, 32 x 128 heads, SwiGLU 11008, vocabulary
    32000), batch 8, prompts of 136 tokens (the prefill takes the tensor-core flash kernel), then three decode steps
    against the paged cache.  Logits against the oracle's full-prefix recompute within the bf16 bar; the greedy token
    must be the oracle's wherever its top-2 margin is clear."""
    cfg = dict(L=2, d=4096, Hq=32, Hkv=32, D=128, ffn=11008, vocab=32000, eps=1e-5, theta=10000.0)
    batch, T, n_gen = 8, 136, 3
    m = Llama(cfg["L"], cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["ffn"], cfg["vocab"], max_batch=batch, max_context=192, seed=4)
    emb, layers, gf, wlm = oracle_weights(m, cfg)
    prompts = [cases.ints(T, 4, 700 + b, 0, cfg["vocab"]) for b in range(batch)]
    nxt = torch.zeros(batch, dtype=torch.int32, device="cuda")
    last_logits = torch.empty(cfg["vocab"], device="cuda")
    seqs = [list(p) for p in prompts]

    def check(got, seq_tokens, what, token=None):
        want = ol.llama_forward(cfg, emb, layers, gf, wlm, np.array(seq_tokens, np.int32), last_rows=1)[-1]
        assert_close(got, want, BF16_RTOL, what)
        top = np.sort(want)[-2:]
        if token is not None and top[1] - top[0] > 2 * BF16_RTOL * float(np.abs(want).max()):
            assert token == int(np.argmax(want)), f"{what}: greedy token differs"

    for b in range(batch):
        m.prefill(torch.from_numpy(prompts[b]).cuda(), b, nxt, last_logits)
        if b in (0, 3, 7):
            check(host(last_logits), seqs[b], f"prefill logits of sequence {b}", int(nxt[b]))
    jb.check_device_errors()
    logits = torch.empty(batch, cfg["vocab"], device="cuda")
    for step in range(n_gen):
        tokens = nxt.clone()
        for b in range(batch):
            seqs[b].append(int(tokens[b]))
        m.decode_step(tokens, nxt, logits)
        got = host(logits)
        for b in (range(batch) if step == n_gen - 1 else (0,)):
            check(got[b], seqs[b], f"decode step {step} sequence {b}", int(nxt[b]))
    jb.check_device_errors()
    m.close()


def test_decode_with_fewer_sequences_than_max_batch():
    """The split of the context into chunks depends on the batch of the step (fewer sequences: shorter chunks, more
    partials per head), so a step with fewer sequences than max_batch can need MORE scratch than a full one: 32 heads,
    max_batch 4, a step of 3 sequences over a context beyond 128 positions.  Checked against the oracle."""
    cfg = dict(L=1, d=256, Hq=32, Hkv=32, D=128, ffn=512, vocab=1024, eps=1e-5, theta=10000.0)
    assert jb.lib().jsm_attn_decode_scratch_bytes(3, 32, 128, 320) > jb.lib().jsm_attn_decode_scratch_bytes(4, 32, 128, 320)
    assert jb.lib().jsm_attn_decode_scratch_bytes_max(4, 32, 128, 320) >= jb.lib().jsm_attn_decode_scratch_bytes(3, 32, 128, 320)
    m = Llama(cfg["L"], cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["ffn"], cfg["vocab"], max_batch=4, max_context=320, seed=4)
    emb, layers, gf, wlm = oracle_weights(m, cfg)
    batch, T = 3, 200
    prompts = [cases.ints(T, 4, 800 + b, 0, cfg["vocab"]) for b in range(batch)]
    nxt = torch.zeros(4, dtype=torch.int32, device="cuda")
    seqs = [list(p) for p in prompts]
    for b in range(batch):
        m.prefill(torch.from_numpy(prompts[b]).cuda(), b, nxt)
    logits = torch.empty(batch, cfg["vocab"], device="cuda")
    for step in range(2):
        tokens = nxt[:batch].clone()
        for b in range(batch):
            seqs[b].append(int(tokens[b]))
        m.decode_step(tokens, nxt, logits)
        got = host(logits)
        for b in range(batch):
            want = ol.llama_forward(cfg, emb, layers, gf, wlm, np.array(seqs[b], np.int32), last_rows=1)[-1]
            assert_close(got[b], want, BF16_RTOL, f"step {step}, sequence {b} of 3 (max_batch 4)")
    jb.check_device_errors()
    m.close()


def test_decode_past_max_context_is_reported_not_faulted():
    """A sequence that already fills max_context cannot grow: the step stays inside the sequence's pages and the rope
    table, and the host reads JSM_SHAPE at the next error check; the neighbouring sequence's cache is left alone."""
    cfg = dict(L=1, d=256, Hq=2, Hkv=2, D=128, ffn=512, vocab=1024, eps=1e-5, theta=10000.0)
    m = Llama(cfg["L"], cfg["d"], 2, 2, cfg["ffn"], cfg["vocab"], max_batch=2, max_context=64, seed=4)
    emb, layers, gf, wlm = oracle_weights(m, cfg)
    p0, p1 = cases.ints(62, 4, 810, 0, 1024), cases.ints(20, 4, 811, 0, 1024)
    nxt = torch.zeros(2, dtype=torch.int32, device="cuda")
    m.prefill(torch.from_numpy(p0).cuda(), 0, nxt)
    m.prefill(torch.from_numpy(p1).cuda(), 1, nxt)
    logits = torch.empty(2, 1024, device="cuda")
    s1 = list(p1)
    for step in range(4):   # sequence 0 reaches 64 cached tokens after two steps; steps 2 and 3 overflow it
        tokens = nxt.clone()
        s1.append(int(tokens[1]))
        m.decode_step(tokens, nxt, logits)
        if step < 2:
            jb.check_device_errors()
        else:
            with pytest.raises(jb.JsmError) as e:
                jb.check_device_errors()
            assert e.value.status == jb.SHAPE
        # the sequence that still has room is unaffected by its neighbour's overflow
        want = ol.llama_forward(cfg, emb, layers, gf, wlm, np.array(s1, np.int32), last_rows=1)[-1]
        assert_close(host(logits)[1], want, BF16_RTOL, f"sequence 1 at step {step}")
    jb.check_device_errors()
    assert int(torch.ones(4, device="cuda").sum()) == 4
    m.close()


def test_host_buffer_step_equals_device_step():
    """jsm_llama_decode_step_host (ids from host memory, the library's own CUDA graph of the step, tokens and logits back
    to host memory) generates what the device-pointer step generates, for two batch sizes on one model."""
    cfg = dict(L=2, d=256, Hq=4, Hkv=2, D=128, ffn=512, vocab=1024)
    mk = lambda: Llama(cfg["L"], cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["ffn"], cfg["vocab"], max_batch=3, max_context=128, seed=4)
    prompts = [cases.ints(30, 4, 820 + b, 0, 1024) for b in range(3)]
    a, b = mk(), mk()
    nxt_a = torch.zeros(3, dtype=torch.int32, device="cuda")
    nxt_b = torch.zeros(3, dtype=torch.int32, device="cuda")
    for s in range(3):
        a.prefill(torch.from_numpy(prompts[s]).cuda(), s, nxt_a)
        b.prefill(torch.from_numpy(prompts[s]).cuda(), s, nxt_b)
    assert torch.equal(nxt_a, nxt_b)
    h_ids = nxt_b.cpu().pin_memory()
    h_next = torch.empty(3, dtype=torch.int32).pin_memory()
    h_logits = torch.empty(3, 1024).pin_memory()
    logits = torch.empty(3, 1024, device="cuda")
    with torch.cuda.stream(torch.cuda.Stream()):
        for step in range(5):
            n = 3 if step < 3 else 2          # the last steps run a smaller batch: a second graph of the same model
            ids = nxt_a[:n].clone()
            a.decode_step(ids, nxt_a[:n], logits[:n])
            b.decode_step_host(h_ids[:n], h_next[:n], h_logits[:n])
            torch.cuda.current_stream().synchronize()
            assert torch.equal(nxt_a[:n].cpu(), h_next[:n]), f"step {step}"
            assert torch.equal(logits[:n].cpu(), h_logits[:n]), f"logits of step {step}"
            h_ids[:n].copy_(h_next[:n])
    jb.check_device_errors()
    a.close(); b.close()
