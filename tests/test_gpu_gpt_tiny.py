"""Configuration 1 on the GPU: the tiny GPT-2-style decoder (2 layers, d 128, 4 heads x 32, pre-LayerNorm,
GELU FFN 512, learned positions, vocab 256, seed 0) composed from C-ABI calls, fp32 throughout.
Checked against the reference's own output (tests/golden/gpt_tiny.npz): full logits [64, 256] within
1e-5 and the same 16 greedy tokens, generated here with a KV cache where the reference recomputes the
whole prefix for every token (transformer_test.hpp:227-241)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
from gpu_util import FP32_RTOL, assert_close, dev, host

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).resolve().parent / "golden" / "gpt_tiny.npz")
L0 = (jb.OP_LEAF, 0)


class TinyGpt:
    def __init__(self):
        g = cases.GPT
        w = cases.gpt_unpack(cases.gpt_weights())
        self.g, d, H = g, g["d"], g["H"]
        dh = d // H
        self.tok, self.pos = dev(w["tok"]), dev(w["pos"])
        self.layers = []
        for lw in w["layers"]:
            # the reference's heads project their own slice of the input (block-diagonal weights)
            Wq, Wk, Wv = (np.zeros((d, d), np.float32) for _ in range(3))
            bq, bk, bv = (np.zeros(d, np.float32) for _ in range(3))
            for h, head in enumerate(lw["heads"]):
                sl = slice(h * dh, (h + 1) * dh)
                for (W, b), (Wd, bd) in zip(head, ((Wq, bq), (Wk, bk), (Wv, bv))):
                    Wd[sl, sl] = W
                    bd[sl] = b
            self.layers.append(dict(
                ln1=(dev(lw["ln1_g"]), dev(lw["ln1_b"])), ln2=(dev(lw["ln2_g"]), dev(lw["ln2_b"])),
                qkv=[(dev(W), dev(b.reshape(1, d))) for W, b in ((Wq, bq), (Wk, bk), (Wv, bv))],
                wo=(dev(lw["wo"]), dev(lw["bo"].reshape(1, d))),
                w1=(dev(lw["w1"]), dev(lw["b1"].reshape(1, -1))), w2=(dev(lw["w2"]), dev(lw["b2"].reshape(1, d))),
                k=torch.zeros(g["max_pos"], d, device="cuda"), v=torch.zeros(g["max_pos"], d, device="cuda")))
        self.lnf = (dev(w["lnf_g"]), dev(w["lnf_b"]))
        self.head = (dev(w["w_out"]), dev(w["b_out"].reshape(1, -1)))
        self.ctx = 0

    def norm(self, x, gb):
        out = torch.empty_like(x)
        return jb.eval_rows(jb.ROWS_LAYERNORM, 1, [L0], [x], out, gain=gb[0], bias=gb[1], eps=self.g["eps"])

    def linear(self, x, wb, epilogue=0, residual=None):
        out = torch.empty(x.shape[0], wb[0].shape[0], device="cuda")
        return jb.dot_f32(x, wb[0].t(), out, bias=wb[1], epilogue=epilogue, residual=residual)

    def forward(self, ids):
        """Appends `ids` at positions ctx.. and returns their logits [T, vocab]; K/V of every position stay cached."""
        g = self.g
        T, H, dh = len(ids), g["H"], g["d"] // g["H"]
        idt = torch.tensor(ids, dtype=torch.int32, device="cuda")
        post = torch.arange(self.ctx, self.ctx + T, dtype=torch.int32, device="cuda")
        x = jb.embedding(self.tok, idt, self.pos, post)
        end = self.ctx + T
        for lw in self.layers:
            n = self.norm(x, lw["ln1"])
            q = self.linear(n, lw["qkv"][0])
            lw["k"][self.ctx:end] = self.linear(n, lw["qkv"][1])
            lw["v"][self.ctx:end] = self.linear(n, lw["qkv"][2])
            att = jb.attn_prefill(q, lw["k"][:end], lw["v"][:end], 1, H, H, dh, causal=True, impl=1)
            x = self.linear(att, lw["wo"], epilogue=3, residual=x)
            h = self.linear(self.norm(x, lw["ln2"]), lw["w1"], epilogue=2)
            x = self.linear(h, lw["w2"], epilogue=3, residual=x)
        self.ctx = end
        return self.linear(self.norm(x, self.lnf), self.head)


def test_tiny_gpt_logits_and_greedy_tokens_match_reference():
    g = cases.GPT
    net = TinyGpt()
    ids = cases.gpt_ids().tolist()
    logits = net.forward(ids)
    assert_close(host(logits), GOLD["logits"], FP32_RTOL, "prefill logits [64, 256]")
    tokens = []
    last = logits[-1:]
    for step in range(g["n_gen"]):
        am = torch.empty(1, 1, device="cuda", dtype=torch.int32)
        jb.eval_rows(jb.ROWS_ARGMAX, 1, [L0], [last.contiguous()], am)
        tok = int(am.item())
        tokens.append(tok)
        last = net.forward([tok])  # one new token against the cache
        assert_close(host(last), GOLD["gen_logits"][step:step + 1], FP32_RTOL, f"logits after generated token {step}")
    assert tokens == GOLD["tokens"].tolist()
