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
