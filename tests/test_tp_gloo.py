"""Tensor-parallel partition of a decoder layer, checked on CPU with two gloo ranks.

Each rank holds the shard the GPU runner gives it (query/kv heads and the matching output-projection columns;
FFN gate/up rows and the matching down-projection columns), computes its partial outputs with the CPU oracle
and the two partial sums meet in ONE all-reduce per block, exactly where the GPU model issues them.  The result
must equal the unsharded layer (TP-N == TP-1)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

CFG = dict(d=64, Hq=4, Hkv=2, D=16, ffn=96, T=7)


def layer_inputs():
    import cases
    c = CFG
    d, Hq, Hkv, D, ffn, T = c["d"], c["Hq"], c["Hkv"], c["D"], c["ffn"], c["T"]
    w = dict(wq=cases.normal((Hq * D, d), 950, 0, 0.2), wk=cases.normal((Hkv * D, d), 950, 1, 0.2), wv=cases.normal((Hkv * D, d), 950, 2, 0.2),
             wo=cases.normal((d, Hq * D), 950, 3, 0.2), wg=cases.normal((ffn, d), 950, 4, 0.2), wu=cases.normal((ffn, d), 950, 5, 0.2),
             wd=cases.normal((d, ffn), 950, 6, 0.2))
    x = cases.normal((T, d), 951, 0)
    return w, x


def shard(w, rank, world):
    c = CFG
    qh, kh, f, D = c["Hq"] // world, c["Hkv"] // world, c["ffn"] // world, c["D"]
    return dict(wq=w["wq"][rank * qh * D:(rank + 1) * qh * D], wk=w["wk"][rank * kh * D:(rank + 1) * kh * D],
                wv=w["wv"][rank * kh * D:(rank + 1) * kh * D], wo=w["wo"][:, rank * qh * D:(rank + 1) * qh * D],
                wg=w["wg"][rank * f:(rank + 1) * f], wu=w["wu"][rank * f:(rank + 1) * f], wd=w["wd"][:, rank * f:(rank + 1) * f])


def layer_partial(w, x, Hq, Hkv, allreduce):
    """One decoder layer on (a shard of) the weights; `allreduce` sums the two block outputs across ranks."""
    import oracle_lib as ol
    po = ol.port_oracle()
    D = CFG["D"]
    zero = lambda n: np.zeros(n, np.float32)
    q, k, v = po.linear(x, w["wq"], zero(Hq * D)), po.linear(x, w["wk"], zero(Hkv * D)), po.linear(x, w["wv"], zero(Hkv * D))
    att = ol.attention(q, k, v, 1, Hq, Hkv, D, True)
    h = x + allreduce(po.linear(att, w["wo"], zero(CFG["d"])))
    g, u = po.linear(h, w["wg"], zero(w["wg"].shape[0])), po.linear(h, w["wu"], zero(w["wu"].shape[0]))
    act = po.activation(3, g) * u
    return h + allreduce(po.linear(act, w["wd"], zero(CFG["d"])))


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_calls = [0]

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        dist.all_reduce(t)
        n_calls[0] += 1
        return t.numpy()

    w, x = layer_inputs()
    y = layer_partial(shard(w, rank, world), x, CFG["Hq"] // world, CFG["Hkv"] // world, allreduce)
    np.save(Path(out_dir) / f"rank{rank}.npy", y)
    assert n_calls[0] == 2  # one all-reduce per attention block and one per FFN block
    dist.destroy_process_group()


def test_tp2_layer_equals_tp1(tmp_path):
    w, x = layer_inputs()
    want = layer_partial(w, x, CFG["Hq"], CFG["Hkv"], lambda a: a)
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        got = np.load(tmp_path / f"rank{r}.npy")
        err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
        assert err <= 1e-5, f"rank {r}: {err}"
