"""GPU parity: softmax, RMSNorm, LayerNorm (forward + backward) against the oracle.
Shape matrix follows test/softmax.jl:37-45 and test/norm.jl:44-69,119-145 of the reference,
plus the long-row / clustered shapes of the benchmark configs."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw, to_dev

pytestmark = pytest.mark.gpu

SOFTMAX_SHAPES = [(1, 8), (17, 64), (256, 128), (4096, 16), (4097, 16), (5000, 8), (16384, 4),
                  (8192, 32), (32768, 24), (65536, 6), (40000, 5)]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("M,N", SOFTMAX_SHAPES)
def test_softmax_fwd_bwd(tylo, oracle, M, N, dt):
    rng = np.random.default_rng(2 + M + N)
    X, X64 = draw(rng, (N, M), dt, scale=2.0)
    Y = tylo.softmax(X)
    ref = oracle.softmax_ref(X64)
    check(Y, ref, dt, "softmax")
    assert np.allclose(back(Y).sum(-1), 1.0, atol=2e-2 if dt != "f32" else 1e-5)  # test/softmax.jl:54
    dY, dY64 = draw(rng, (N, M), dt)
    Yr, Yr64 = Y, back(Y)
    dX = tylo.grad_softmax(dY, Yr)
    check(dX, oracle.softmax_bwd_ref(dY64, Yr64), dt, "softmax bwd")


def test_softmax_inf_entries(tylo, oracle):
    X = torch.randn(4, 1024, device="cuda")
    X[:, ::3] = float("-inf")
    check(tylo.softmax(X), oracle.softmax_ref(back(X)), "f32", "softmax with -inf entries")


NORM_SHAPES = [(256, 32), (512, 16), (768, 8), (130, 16), (300, 8), (8192, 48), (4096, 33), (16384, 5), (33000, 3)]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("offset", [0.0, 1.0])
@pytest.mark.parametrize("M,N", NORM_SHAPES)
def test_rms_norm(tylo, oracle, M, N, offset, dt):
    rng = np.random.default_rng(3 + M)
    eps = 1e-5
    X, X64 = draw(rng, (N, M), dt)
    W, W64 = draw(rng, (M,), dt, scale=0.1, shift=1.0 - offset)
    cp = tylo.allocate_checkpoints_rms_norm(X, W)
    Y = tylo.rms_norm(X, W, eps=eps, offset=offset, checkpoints=cp)
    check(Y, oracle.rms_norm_ref(X64, W64, eps=eps, offset=offset), dt, "rms_norm")
    dY, dY64 = draw(rng, (N, M), dt)
    dXr, dWr, rstd = oracle.rms_norm_bwd_ref(dY64, X64, W64, eps=eps, offset=offset)
    np.testing.assert_allclose(back(cp.Rstd), rstd, rtol=2e-6)
    # backward in isolation: reference statistics as checkpoints (test/norm.jl:104-114)
    cp_ref = tylo.RmsCheckpoints(torch.from_numpy(rstd).float().cuda())
    for groups in (7, 64, 296):
        sc = tylo.allocate_scratchspace_grad_rms_norm(X, W, N_GROUPS=groups)
        dX, dW = tylo.grad_rms_norm(dY, X, W, checkpoints=cp_ref, offset=offset, scratch=sc)
        check(dX, dXr, dt, "rms_norm dX")
        check(dW, dWr, dt, "rms_norm dW", scale_hint=4 * float(np.abs(dWr).max()))


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("M,N", NORM_SHAPES)
def test_layer_norm(tylo, oracle, M, N, dt):
    rng = np.random.default_rng(5 + M)
    eps = 1e-5
    X, X64 = draw(rng, (N, M), dt, shift=0.5)
    W, W64 = draw(rng, (M,), dt, scale=0.1, shift=1.0)
    B, B64 = draw(rng, (M,), dt, scale=0.1)
    cp = tylo.allocate_checkpoints_layer_norm(X, W, B)
    Y = tylo.layer_norm(X, W, B, eps=eps, checkpoints=cp)
    check(Y, oracle.layer_norm_ref(X64, W64, B64, eps=eps), dt, "layer_norm")
    dY, dY64 = draw(rng, (N, M), dt)
    dXr, dWr, dBr, mean, rstd = oracle.layer_norm_bwd_ref(dY64, X64, W64, eps=eps)
    np.testing.assert_allclose(back(cp.Mean), mean, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(back(cp.Rstd), rstd, rtol=1e-5)
    cp_ref = tylo.LnCheckpoints(torch.from_numpy(mean).float().cuda(), torch.from_numpy(rstd).float().cuda())
    dX, dW, dB = tylo.grad_layer_norm(dY, X, W, B, checkpoints=cp_ref)
    check(dX, dXr, dt, "layer_norm dX")
    check(dW, dWr, dt, "layer_norm dW", scale_hint=4 * float(np.abs(dWr).max()))
    check(dB, dBr, dt, "layer_norm dB", scale_hint=4 * float(np.abs(dBr).max()))


def test_norm_bwd_is_deterministic(tylo):
    g = torch.Generator(device="cuda").manual_seed(0)
    X = torch.randn(512, 2048, device="cuda", generator=g, dtype=torch.bfloat16)
    W = torch.randn(2048, device="cuda", generator=g, dtype=torch.bfloat16)
    dY = torch.randn_like(X)
    cp = tylo.allocate_checkpoints_rms_norm(X, W)
    tylo.rms_norm(X, W, eps=1e-6, checkpoints=cp)
    a = tylo.grad_rms_norm(dY, X, W, checkpoints=cp)
    b = tylo.grad_rms_norm(dY, X, W, checkpoints=cp)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])   # lock-free two-stage reduction: bit-repeatable


def test_benchmark_shapes_rowwise(tylo, oracle):
    """Config 2 at full size: bf16, hidden 8192 x 16384 tokens (norms), 32768 x 4096 (softmax).
    Whole-array properties plus the oracle on a sample of rows."""
    g = torch.Generator(device="cuda").manual_seed(1)
    X = torch.randn(16384, 8192, device="cuda", generator=g).to(torch.bfloat16)
    W = (1 + 0.02 * torch.randn(8192, device="cuda", generator=g)).to(torch.bfloat16)
    Bv = (0.02 * torch.randn(8192, device="cuda", generator=g)).to(torch.bfloat16)
    rows = [0, 1, 777, 8191, 16383]
    Y = tylo.rms_norm(X, W, eps=1e-6)
    check(Y[rows], oracle.rms_norm_ref(back(X[rows]), back(W), eps=1e-6), "bf16", "rms_norm C2")
    Y = tylo.layer_norm(X, W, Bv, eps=1e-6)
    check(Y[rows], oracle.layer_norm_ref(back(X[rows]), back(W), back(Bv), eps=1e-6), "bf16", "layer_norm C2")
    del X, Y
    Z = (2 * torch.randn(4096, 32768, device="cuda", generator=g)).to(torch.bfloat16)
    P = tylo.softmax(Z)
    sums = P.float().sum(-1)
    assert float((sums - 1).abs().max()) < 2e-2
    rows = [0, 5, 2048, 4095]
    check(P[rows], oracle.softmax_ref(back(Z[rows])), "bf16", "softmax C2")
