"""Helpers shared by the GPU parity tests.

Inputs are drawn in float64 from a seeded NumPy generator, rounded to the storage dtype on the
way to the device, and the oracle sees the *rounded* values upcast to float64 — so the
tolerances measure the kernels, not input quantisation.

Tolerances (from the build contract):
  fp32 storage : normalised max error  max|got - ref| <= 1e-5 * max|ref| + 1e-6
                 (the 1e-6 floor covers references that are exactly zero, e.g. a causal
                 query that sees one key has dQ = 0)
  bf16 storage : max-abs <= 2e-2 and mean-abs <= 2e-3 (fp16 is held to the same bound)
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


def check(got: torch.Tensor, ref: np.ndarray, dt: str, what: str = "", scale_hint: float | None = None):
    g = back(got)
    assert g.shape == ref.shape, f"{what}: shape {g.shape} vs {ref.shape}"
    assert np.isfinite(g).all(), f"{what}: non-finite values in the result"
    err = np.abs(g - ref)
    if dt == "f32":
        bound = 1e-5 * float(np.abs(ref).max()) + 1e-6
        assert err.max() <= bound, f"{what}: max error {err.max():.3e} > {bound:.3e} (1e-5 relative)"
    else:
        # gradients that sum many terms are compared relative to their own magnitude
        s = 1.0 if scale_hint is None else max(1.0, scale_hint)
        assert err.max() <= 2e-2 * s, f"{what}: max-abs error {err.max():.3e} > {2e-2 * s:.1e}"
        assert err.mean() <= 2e-3 * s, f"{what}: mean-abs error {err.mean():.3e} > {2e-3 * s:.1e}"
