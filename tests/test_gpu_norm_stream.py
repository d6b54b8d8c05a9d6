"""GPU parity: the streaming backward of RMSNorm / LayerNorm (rows of exactly one 16-byte packet per
thread: 512 or 1024 packets) with more rows than walking CTAs, uneven row counts, and saved statistics
from the library's own forward; formulas of test/norm.jl:78-102."""
import numpy as np
import pytest

from gpu_util import check, draw

pytestmark = pytest.mark.gpu

CASES = [("bf16", 8192, 700), ("bf16", 4096, 1000), ("f32", 4096, 333), ("f32", 2048, 901), ("f16", 8192, 150)]


@pytest.mark.parametrize("dt,M,N", CASES)
def test_stream_backward(tylo, oracle, dt, M, N):
    rng = np.random.default_rng(M + N)
    eps = 1e-5
    X, X64 = draw(rng, (N, M), dt, shift=0.3)
    W, W64 = draw(rng, (M,), dt, scale=0.1, shift=1.0)
    B, B64 = draw(rng, (M,), dt, scale=0.1)
    dY, dY64 = draw(rng, (N, M), dt)
    cp = tylo.allocate_checkpoints_rms_norm(X, W)
    tylo.rms_norm(X, W, eps=eps, offset=0.25, checkpoints=cp)
    dX, dW = tylo.grad_rms_norm(dY, X, W, checkpoints=cp, offset=0.25)
    dXr, dWr, _ = oracle.rms_norm_bwd_ref(dY64, X64, W64, eps=eps, offset=0.25)
    check(dX, dXr, dt, "rms dX"); check(dW, dWr, dt, "rms dW", scale_hint=4 * float(np.abs(dWr).max()))
    cpl = tylo.allocate_checkpoints_layer_norm(X, W, B)
    tylo.layer_norm(X, W, B, eps=eps, checkpoints=cpl)
    dX, dW, dB = tylo.grad_layer_norm(dY, X, W, B, checkpoints=cpl)
    dXr, dWr, dBr, _, _ = oracle.layer_norm_bwd_ref(dY64, X64, W64, eps=eps)
    check(dX, dXr, dt, "ln dX")
    check(dW, dWr, dt, "ln dW", scale_hint=4 * float(np.abs(dWr).max()))
    check(dB, dBr, dt, "ln dB", scale_hint=4 * float(np.abs(dBr).max()))
