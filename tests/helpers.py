"""Shared helpers: golden-fixture loading and the statistical closeness check.

The closeness rule follows the reference test-suite's budget semantics
(tests/helpers.py:28-110, tests/ops/tolerances.py:6-11 of the reference): an element is bad when
|a-b| > atol + rtol*|b|; a comparison passes when it is allclose, or when the bad fraction, the
95th and the 99th percentile of the normalised error stay inside the budget.
"""
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

FP32_TOL = dict(atol=5e-4, rtol=5e-4, max_err_rate=0.01, max_q99=1.5)
BEHAVIOR_TOL = dict(atol=1e-4, rtol=1e-4, max_err_rate=0.01, max_q99=1.5)
BF16_TOL = dict(atol=7.5e-2, rtol=7.5e-2, max_err_rate=0.02, max_q99=2.0)
FP16_TOL = dict(atol=1e-2, rtol=1e-2, max_err_rate=0.01, max_q99=1.5)


def load(name):
    z = np.load(GOLDEN / name, allow_pickle=False)
    return {k: z[k] for k in z.files}


def t(a, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a))
    return x if dtype is None else x.to(dtype)


def in_dtype(z):
    return {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}[str(z["in_dtype"])]


def assert_close_stats(name, val, ref, *, atol, rtol, max_err_rate=0.002, max_q99=1.0):
    val = torch.as_tensor(val).detach().double().cpu().flatten()
    ref = torch.as_tensor(ref).detach().double().cpu().flatten()
    assert val.shape == ref.shape, f"{name}: shape {tuple(val.shape)} != {tuple(ref.shape)}"
    if val.numel() == 0:
        return
    assert torch.isfinite(val).all() and torch.isfinite(ref).all(), f"{name}: non-finite values"
    if torch.allclose(val, ref, atol=atol, rtol=rtol):
        return
    err = (val - ref).abs() / (atol + rtol * ref.abs())
    if err.numel() > 4_000_000:
        err = err[torch.randperm(err.numel())[:4_000_000]]
    bad = int((err > 1).sum())
    q95, q99 = err.quantile(0.95).item(), err.quantile(0.99).item()
    ok = bad <= int(max_err_rate * err.numel()) and q95 <= 1 and (max_q99 is None or q99 <= max_q99)
    assert ok, (f"{name}: bad={bad}/{err.numel()} q95={q95:.3f} q99={q99:.3f} max={err.max().item():.3f} "
                f"(atol={atol}, rtol={rtol})")
