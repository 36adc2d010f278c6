"""Shared helpers of the test-suite: bf16 <-> NumPy conversion, seeded inputs in the reference's recipes."""
import hashlib

import numpy as np
import torch


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def to_bf16_cuda(x_f32):
    """float32 NumPy array holding bf16-representable values -> CUDA bfloat16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(x_f32, np.float32)).cuda().to(torch.bfloat16)


def bf16_np(t):
    """bfloat16 tensor -> float32 NumPy array."""
    return t.detach().float().cpu().numpy()


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def llm_weights(rng, n, k, sigma=0.3):
    """w = N(0,1) * 0.02 * lognormal(0, sigma) per column (sim/make_testcase.py:48-50)."""
    return (rng.standard_normal((n, k)) * 0.02 * rng.lognormal(0, sigma, (1, k))).astype(np.float32)


def llm_acts(rng, m, k, oracle, outliers=8):
    """x = N(0,1) * lognormal(0, 0.5) per column with a few x20 outlier channels, rounded to bf16
    (sim/make_testcase.py:51-53)."""
    x = rng.standard_normal((m, k)) * rng.lognormal(0, 0.5, (1, k))
    x[:, rng.choice(k, outliers, replace=False)] *= 20
    return oracle.bf16_round(x.astype(np.float32))


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-300)))
