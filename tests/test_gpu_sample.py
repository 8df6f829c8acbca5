"""GPU sampler (temperature, top-k, top-p) against a numpy restatement with the same uniform draws."""
import numpy as np
import pytest
import torch

import cases
import jasmine_b200 as jb

pytestmark = pytest.mark.gpu


def reference(logits, temperature, top_k, top_p, u):
    """Per row: the K largest logits by (value desc, index asc), p = exp((x - x0) / T), the shortest prefix whose mass
    reaches top_p of the candidates' total, then the first token whose cumulative mass exceeds u * kept mass.
    Returns the token and the distance of the draw from the nearest boundary, relative to the kept mass."""
    toks, margins = [], []
    for r in range(logits.shape[0]):
        x = logits[r]
        K = min(1024 if top_k <= 0 else min(top_k, 1024), x.size)
        order = np.lexsort((np.arange(x.size), -x.astype(np.float64)))[:K]
        p = np.exp((x[order].astype(np.float64) - float(x[order[0]])) / temperature)
        cum = np.cumsum(p)
        n_keep = K if top_p >= 1.0 else min(K, int(np.sum(cum[:K - 1] < top_p * cum[-1])) + 1)
        target = float(u[r]) * cum[n_keep - 1]
        pos = min(int(np.sum(cum[:n_keep - 1] <= target)), n_keep - 1)
        toks.append(int(order[pos]))
        margins.append(float(np.min(np.abs(cum[:n_keep] - target)) / cum[n_keep - 1]))
    return np.array(toks), np.array(margins)


@pytest.mark.parametrize("vocab", [50, 1000, 32000])
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 40, 1.0), (1.3, 0, 0.9), (0.8, 200, 0.5), (1.0, 1024, 0.95)])
def test_sampler_matches_numpy(vocab, temperature, top_k, top_p):
    rows, seed, step = 16, 9, 3
    L = cases.normal((rows, vocab), 50, vocab, 3.0)
    L[0, :5] = L[0].max() + 1.0                      # ties at the top
    u = cases.uniform((rows,), seed, step, 0.0, 1.0)  # the sampler's draws: same generator, same (seed, step, row)
    got = jb.sample(torch.from_numpy(L).cuda(), temperature, top_k, top_p, seed, step).cpu().numpy()
    want, margin = reference(L, temperature, top_k, top_p, u)
    # float32 sums on the device against float64 here: a draw within 1e-5 of a boundary may fall on either side
    bad = (got != want) & (margin > 1e-5)
    assert not bad.any(), f"rows {np.nonzero(bad)[0]}: got {got[bad]}, want {want[bad]}"
    assert (got >= 0).all() and (got < vocab).all()


def test_greedy_and_determinism():
    L = cases.normal((8, 4096), 51, 0, 2.0)
    L[3, 100] = L[3, 7] = L[3].max() + 2.0  # tie: the smaller index wins
    d = torch.from_numpy(L).cuda()
    want = np.array([int(np.flatnonzero(r == r.max())[0]) for r in L])
    assert np.array_equal(jb.sample(d, 0.0).cpu().numpy(), want)
    assert np.array_equal(jb.sample(d, 1.0, top_k=1).cpu().numpy(), want)
    a = jb.sample(d, 1.0, 50, 0.9, seed=1, step=5).cpu().numpy()
    b = jb.sample(d, 1.0, 50, 0.9, seed=1, step=5).cpu().numpy()
    c = jb.sample(d, 1.0, 50, 0.9, seed=1, step=6).cpu().numpy()
    assert np.array_equal(a, b) and not np.array_equal(a, c)


def test_sample_frequencies_follow_the_distribution():
    """2000 draws (steps) of one row with 6 candidates: empirical frequencies within 4 sigma of softmax(x / T)."""
    x = np.array([2.0, 1.0, 0.5, 0.0, -1.0, -3.0] + [-30.0] * 58, np.float32)
    d = torch.from_numpy(np.tile(x, (2000, 1))).cuda()
    toks = jb.sample(d, 1.5, 6, 1.0, seed=4, step=0).cpu().numpy()   # rows = independent draws
    p = np.exp(x[:6].astype(np.float64) / 1.5); p /= p.sum()
    freq = np.bincount(toks, minlength=6)[:6] / 2000.0
    assert toks.max() < 6
    assert np.all(np.abs(freq - p) < 4 * np.sqrt(p * (1 - p) / 2000) + 1e-3)
