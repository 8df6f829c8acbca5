"""TP-N == TP-1 for the decoder runner on ONE GPU.

The ranks of a tensor-parallel group are separate model objects of this process, each driven by its own host thread
on its own stream.  Their all-reduce is the host hook (jsm_llama_set_allreduce): inside the hook every thread
synchronises its stream, the threads meet at a barrier, one of them adds the ranks' buffers on the device and all of
them continue.  Host threads wait for each other; no kernel ever waits for another kernel.

What is checked is the sharding of the runner itself (csrc/llama.cu: heads and FFN columns by rank, shards generated
from indices of the full tensors) - the independence of heads the split rests on is the reference's head loop,
mat_mha_t.hpp:278-288 (heads computed separately, concatenated, then one output projection)."""
import threading

import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb
import oracle_lib as ol
from gpu_util import BF16_RTOL, assert_close, host
from jasmine_b200.model import Llama
from test_gpu_llama import oracle_weights

pytestmark = pytest.mark.gpu


def as_tensor(ptr, count, dtype):
    iface = {"shape": (count,), "typestr": "<u2" if dtype == jb.BF16 else "<f4", "data": (ptr, False), "version": 2}
    t = torch.as_tensor(type("DevBuf", (), {"__cuda_array_interface__": iface})(), device="cuda")
    return t.view(torch.bfloat16) if dtype == jb.BF16 else t


class HostAllReduce:
    """Sum across the rank threads of one process (see the module docstring)."""

    def __init__(self, n):
        self.n, self.bufs = n, [None] * n
        self.barrier = threading.Barrier(n, timeout=60.0)

    def hook(self, rank):
        def fn(ptr, count, dtype, stream):
            torch.cuda.current_stream().synchronize()
            self.bufs[rank] = as_tensor(ptr, count, dtype)
            self.barrier.wait()
            if rank == 0:
                total = self.bufs[0].float()
                for r in range(1, self.n):          # rank order, like the exchange kernel
                    total = total + self.bufs[r].float()
                total = total.to(self.bufs[0].dtype)
                for r in range(self.n):
                    self.bufs[r].copy_(total)
                torch.cuda.current_stream().synchronize()
            self.barrier.wait()
        return fn


def run_tp_group(cfg, n, prompts, n_gen, max_context):
    """Greedy generation by an n-way tensor-parallel group of rank threads; returns rank 0's (prefill logits, per-step
    logits, tokens) and checks that all ranks produced the same tokens."""
    batch = len(prompts)
    ar = HostAllReduce(n)
    results, errors = [None] * n, []

    def worker(rank):
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                m = Llama(cfg["L"], cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["ffn"], cfg["vocab"], max_batch=batch,
                          max_context=max_context, seed=4, tp_rank=rank, tp_size=n)
                m.set_allreduce(ar.hook(rank))
                nxt = torch.zeros(batch, dtype=torch.int32, device="cuda")
                pre = torch.empty(batch, cfg["vocab"], device="cuda")
                for b in range(batch):
                    m.prefill(torch.from_numpy(prompts[b]).cuda(), b, nxt, pre[b])
                logits = torch.empty(batch, cfg["vocab"], device="cuda")
                steps, toks = [], []
                for _ in range(n_gen):
                    ids = nxt.clone()
                    toks.append(ids.cpu().numpy().copy())
                    m.decode_step(ids, nxt, logits)
                    steps.append(host(logits))
                jb.check_device_errors()
                results[rank] = (host(pre), steps, np.stack(toks))
                m.close()
        except Exception as e:  # a failed rank must not leave the others at the barrier
            errors.append(e)
            ar.barrier.abort()

    threads = [threading.Thread(target=worker, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    for r in range(1, n):
        assert np.array_equal(results[0][2], results[r][2]), f"rank {r} generated other tokens than rank 0"
    return results[0]


@pytest.mark.parametrize("n,cfg", [
    (2, dict(L=2, d=256, Hq=4, Hkv=2, D=128, ffn=512, vocab=1024, eps=1e-5, theta=10000.0)),
    (4, dict(L=2, d=512, Hq=8, Hkv=4, D=128, ffn=1024, vocab=1024, eps=1e-5, theta=10000.0)),
    (2, dict(L=1, d=4096, Hq=32, Hkv=32, D=128, ffn=11008, vocab=2048, eps=1e-5, theta=10000.0)),
])
def test_tensor_parallel_group_equals_one_rank(n, cfg):
    batch, T, n_gen = 3, 40, 3
    prompts = [cases.ints(T, 4, 600 + b, 0, cfg["vocab"]) for b in range(batch)]
    pre_n, steps_n, toks_n = run_tp_group(cfg, n, prompts, n_gen, 128)
    pre_1, steps_1, toks_1 = run_tp_group(cfg, 1, prompts, n_gen, 128)
    # TP-N against TP-1: same model, another summation order (rank-local bf16 products, then the sum)
    for b in range(batch):
        assert_close(pre_n[b], pre_1[b], BF16_RTOL, f"TP-{n} vs TP-1 prefill logits, sequence {b}")
    seqs = [list(p) for p in prompts]
    same_tokens = True
    for s in range(n_gen):
        for b in range(batch):
            seqs[b].append(int(toks_n[s][b]))
        if not np.array_equal(toks_n[s], toks_1[s]):
            same_tokens = False  # from here on the two runs decode different prefixes: compare with the oracle instead
        if same_tokens:
            for b in range(batch):
                assert_close(steps_n[s][b], steps_1[s][b], BF16_RTOL, f"TP-{n} vs TP-1 decode step {s}, sequence {b}")
    # and against the oracle's full-prefix recompute on the unsharded weights (taken from a one-rank model)
    m = Llama(cfg["L"], cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["ffn"], cfg["vocab"], max_batch=1, max_context=64, seed=4)
    emb, layers, gf, wlm = oracle_weights(m, cfg)
    m.close()
    for b in range(batch):
        want = ol.llama_forward(cfg, emb, layers, gf, wlm, np.array(seqs[b], np.int32), last_rows=1)[-1]
        assert_close(steps_n[-1][b], want, BF16_RTOL, f"TP-{n} last decode step vs oracle, sequence {b}")
