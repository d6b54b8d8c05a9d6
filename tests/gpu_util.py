"""Helpers shared by the GPU parity tests.

Inputs are drawn in float64 from a seeded NumPy generator, rounded to the storage dtype on the
way to the device, and the oracle sees the *rounded* values upcast to float64 — so the
tolerances measure the kernels, not input quantisation.

Tolerances (from the build contract):
  fp32 storage : normalised max error  max|got - ref| <= 1e-5 * max|ref| + 1e-6
                 (the 1e-6 floor covers references that are exactly zero, e.g. a causal
                 query that sees one key has dQ = 0)
  bf16 storage : max-abs <= 2e-2 and mean-abs <= 2e-3 (fp16 is held to the same bound)
  gradients in 16-bit storage (`scale_hint` given): the same two numbers times
                 max(1, P / 4), P = the power of two at or above the hint (callers pass max|ref|): a bf16
                 result in [P/2, P) is spaced P * 2^-8 apart, so its rounding alone reaches P * 2^-9 — 0.016
                 for values between 4 and 8, before any arithmetic error — and no kernel can meet a fixed
                 2e-2 on results of that size.  Outputs of magnitude below 4 keep the plain bound.
"""
from __future__ import annotations

import numpy as np
import torch

DEV = "cuda"
TORCH_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def to_dev(x64: np.ndarray, dt: str) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x64)).to(TORCH_DT[dt]).to(DEV)


def back(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float64).cpu().numpy()


def draw(rng, shape, dt, scale=1.0, shift=0.0):
    """Returns (device tensor in dtype dt, float64 array of the rounded values)."""
    t = to_dev(rng.standard_normal(shape) * scale + shift, dt)
    return t, back(t)


def grad_scale(max_ref) -> float:
    """Factor on the 16-bit bounds for a result whose largest reference magnitude is `max_ref`:
    max(1, P / 4) with P the power of two at or above it (1 when no hint is given)."""
    if max_ref is None or not max_ref > 0:
        return 1.0
    return max(1.0, 2.0 ** float(np.ceil(np.log2(max_ref))) / 4.0)


def check(got: torch.Tensor, ref: np.ndarray, dt: str, what: str = "", scale_hint: float | None = None):
    g = back(got)
    assert g.shape == ref.shape, f"{what}: shape {g.shape} vs {ref.shape}"
    assert np.isfinite(g).all(), f"{what}: non-finite values in the result"
    err = np.abs(g - ref)
    if dt == "f32":
        bound = 1e-5 * float(np.abs(ref).max()) + 1e-6
        assert err.max() <= bound, f"{what}: max error {err.max():.3e} > {bound:.3e} (1e-5 relative)"
    else:
        s = grad_scale(scale_hint)
        assert err.max() <= 2e-2 * s, f"{what}: max-abs error {err.max():.3e} > {2e-2 * s:.1e}"
        assert err.mean() <= 2e-3 * s, f"{what}: mean-abs error {err.mean():.3e} > {2e-3 * s:.1e}"
