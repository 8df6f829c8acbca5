"""Continuous batching over the paged KV cache (jsm_llama_create_paged / seq_admit / step_active / seq_retire).

Sequences of different prompt lengths join and leave a running batch between decode steps; pages come from one shared
pool.  Every sequence must compute what it computes alone: its per-step logits are compared (bf16 bar) with those of a
solo run of the same prompt on a model with the fixed one-run-of-pages-per-sequence layout, and the greedy token must
agree wherever the solo run's top-2 margin is clear.  The batched run is fed the solo run's tokens (teacher forcing), so a
near-tie cannot make the two runs decode different prefixes.  The behaviour this replaces is the reference's one-sequence
full-recompute loop (transformer_test.hpp:231-239)."""
import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
from gpu_util import BF16_RTOL, assert_close
from jasmine_b200.model import Llama

pytestmark = pytest.mark.gpu

CFG = dict(L=2, d=256, Hq=4, Hkv=2, ffn=512, vocab=1024)
MAX_CTX = 256


def solo_run(prompt, n_steps):
    """Greedy generation of one sequence alone: the first token, then per step (input token, logits)."""
    m = Llama(CFG["L"], CFG["d"], CFG["Hq"], CFG["Hkv"], CFG["ffn"], CFG["vocab"], max_batch=1, max_context=MAX_CTX, seed=4)
    nxt = torch.zeros(1, dtype=torch.int32, device="cuda")
    m.prefill(torch.from_numpy(prompt).cuda(), 0, nxt)
    logits = torch.empty(1, CFG["vocab"], device="cuda")
    tokens, step_logits = [int(nxt[0])], []
    for _ in range(n_steps):
        ids = nxt.clone()
        m.decode_step(ids, nxt, logits)
        step_logits.append(logits[0].cpu().numpy().copy())
        tokens.append(int(nxt[0]))
    m.close()
    return tokens, step_logits


def test_sequences_join_and_leave_a_running_batch():
    lengths = [20, 70, 130, 40, 64, 100]           # 130 tokens: the prefill takes the flash kernel; 64: a full page
    prompts = [cases.ints(n, 4, 880 + i, 0, CFG["vocab"]) for i, n in enumerate(lengths)]
    n_steps = 12
    solo = [solo_run(p, n_steps) for p in prompts]

    pool = 9                                        # fewer pages than 4 rows x 4 pages: over-subscribed on purpose
    m = Llama(CFG["L"], CFG["d"], CFG["Hq"], CFG["Hkv"], CFG["ffn"], CFG["vocab"], max_batch=4, max_context=MAX_CTX, seed=4,
              pool_pages=pool)
    rows = []                                       # rows[r] = [sequence index, steps done]
    with torch.cuda.stream(torch.cuda.Stream()):
        def admit(i):
            row, tok = m.admit(torch.from_numpy(prompts[i]))
            assert row == len(rows)
            assert tok == solo[i][0][0], f"first token of sequence {i}"
            rows.append([i, 0])

        def retire(r):
            moved = m.retire(r)
            last = rows.pop()
            if moved >= 0:                          # the last row took the freed place
                assert moved == len(rows) and r < len(rows)
                rows[r] = last
            return moved

        def step():
            n = len(rows)
            h_ids = torch.tensor([solo[i][0][k] for i, k in rows], dtype=torch.int32).pin_memory()
            h_next = torch.empty(n, dtype=torch.int32).pin_memory()
            h_logits = torch.empty(n, CFG["vocab"]).pin_memory()
            m.step_active(h_ids, h_next, h_logits)
            for r, (i, k) in enumerate(rows):
                want = solo[i][1][k]
                assert_close(h_logits[r].numpy(), want, BF16_RTOL, f"sequence {i} step {k} in row {r} of {n}")
                top = np.sort(want)[-2:]
                if top[1] - top[0] > 2 * BF16_RTOL * float(np.abs(want).max()):
                    assert int(h_next[r]) == int(np.argmax(want)), f"greedy token of sequence {i} step {k}"
                rows[r][1] += 1

        admit(0); admit(1)
        for _ in range(3):
            step()
        admit(2)                                    # 130 tokens: 3 pages
        for _ in range(2):
            step()
        assert retire(0) == 2                       # sequence 2 (the last row) moves into row 0
        assert [r[0] for r in rows] == [2, 1]
        admit(3); admit(4)
        for _ in range(4):
            step()
        # the pool: 3 (seq 2) + 2 (seq 1) + 1 (seq 3) + 2 (seq 4: 64 + steps crossed into a second page) = 8 of 9 pages
        active, free, total = m.pool_state()
        assert (active, total) == (4, pool) and free == pool - 8
        with pytest.raises(jb.JsmError) as e:       # no batch row left
            m.admit(torch.from_numpy(prompts[5]))
        assert e.value.status == jb.OOM
        retire(1)                                   # row 1 <- the last row (sequence 4)
        with pytest.raises(jb.JsmError) as e:       # a row is free now and 3 pages are, but a 250-token prompt needs 4
            m.admit(torch.from_numpy(cases.ints(250, 4, 899, 0, CFG["vocab"])))
        assert e.value.status == jb.OOM
        assert m.pool_state() == (3, 3, pool)       # the refused admission took nothing
        admit(5)
        for _ in range(3):
            step()
        while rows:
            retire(len(rows) - 1)
        active, free, total = m.pool_state()
        assert (active, free, total) == (0, pool, pool)
    jb.check_device_errors()
    m.close()
