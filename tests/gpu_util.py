"""Helpers of the GPU parity tests: tolerances and array transport."""
import numpy as np
import torch

FP32_RTOL = 1e-5     # relative to the largest reference magnitude: the bar for fp32 paths
BF16_RTOL = 2e-2     # bar for bf16 results


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dtype)


def host(t):
    return t.detach().float().cpu().numpy()


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    scale = max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(got - want))) / scale


def assert_close(got, want, tol, what=""):
    e = rel_err(got, want)
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"
    return e
