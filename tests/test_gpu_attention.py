"""GPU parity: attention! / ∇attention! against the oracle.  Shapes follow
test/attention.jl:57-114 of the reference plus the benchmark configs."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw

pytestmark = pytest.mark.gpu


def _run(tylo, oracle, dt, *, B, H, Hkv, Sq, Sk, Dk, Dv, causal, seed, bwd=True):
    rng = np.random.default_rng(seed)
    Q, Q64 = draw(rng, (B, H, Sq, Dk), dt)
    K, K64 = draw(rng, (B, Hkv, Sk, Dk), dt)
    V, V64 = draw(rng, (B, Hkv, Sk, Dv), dt)
    cp = tylo.allocate_checkpoints_attention(Q, K, V)
    O = tylo.attention(Q, K, V, causal=causal, checkpoints=cp)
    mask = oracle.MaskSpec(causal=True) if causal else None
    Oref, Mref, Lref = oracle.flex_ref(Q64, K64, V64, mask=mask, return_stats=True)
    check(O, Oref, dt, "attention O")
    # checkpoints: M = row max in log2 units, L = sum exp2 (attention.jl:52-56,83-85)
    lse = back(cp.M) * np.log(2.0) + np.log(back(cp.L))
    np.testing.assert_allclose(lse, Mref + np.log(Lref), rtol=0, atol=2e-2 if dt != "f32" else 2e-5)
    if not bwd:
        return
    dO, dO64 = draw(rng, (B, H, Sq, Dv), dt)
    dQ, dK, dV = tylo.grad_attention(dO, Q, K, V, O, checkpoints=cp, causal=causal)
    rQ, rK, rV = oracle.attn_bwd_ref(dO64, Q64, K64, V64, causal=causal)
    # backward consumes the storage-rounded O; its effect is inside the bf16 tolerance
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"attention {name}", scale_hint=float(np.abs(ref).max()))


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("causal", [False, True])
def test_reference_shape_mha(tylo, oracle, causal, dt):
    _run(tylo, oracle, dt, B=2, H=4, Hkv=4, Sq=96, Sk=128, Dk=64, Dv=64, causal=causal, seed=8)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_reference_shape_gqa(tylo, oracle, dt):
    _run(tylo, oracle, dt, B=2, H=4, Hkv=2, Sq=96, Sk=128, Dk=64, Dv=64, causal=True, seed=9)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [
    dict(B=1, H=2, Hkv=1, Sq=33, Sk=47, Dk=40, Dv=24),      # ragged everything, odd head dims
    dict(B=2, H=8, Hkv=2, Sq=256, Sk=256, Dk=128, Dv=128),   # benchmark geometry, small
    dict(B=1, H=2, Hkv=2, Sq=1, Sk=300, Dk=64, Dv=64),       # single query row
    dict(B=1, H=1, Hkv=1, Sq=130, Sk=70, Dk=256, Dv=256),    # largest supported head dim, Sq > Sk
])
@pytest.mark.parametrize("causal", [False, True])
def test_shapes(tylo, oracle, shape, causal, dt):
    _run(tylo, oracle, dt, causal=causal, seed=21, **shape)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [
    dict(B=2, H=4, Hkv=2, Sq=300, Sk=300, Dk=96, Dv=96),     # padded to the 128-wide tile of the tensor-core kernels
    dict(B=1, H=3, Hkv=3, Sq=130, Sk=257, Dk=80, Dv=80),
    dict(B=2, H=2, Hkv=1, Sq=200, Sk=200, Dk=32, Dv=32),     # padded to the 64-wide tile
    dict(B=1, H=2, Hkv=2, Sq=96, Sk=160, Dk=40, Dv=40),
    dict(B=1, H=1, Hkv=1, Sq=64, Sk=64, Dk=8, Dv=8),         # one 16-byte packet per row
])
@pytest.mark.parametrize("causal", [False, True])
def test_zero_padded_head_dims(tylo, oracle, shape, causal, dt):
    """Head dims that are multiples of 8 below 64 / 128 run on the tensor-core kernels with the missing columns
    read as zeros (the reference pads the same way, attention.jl:241-242); forward, statistics and gradients."""
    _run(tylo, oracle, dt, causal=causal, seed=33, **shape)


def test_config1_fp32(tylo, oracle):
    """Benchmark config 1: fp32, non-causal, D 64, S 512, H 8, B 2, seed 0; <= 1e-5."""
    _run(tylo, oracle, "f32", B=2, H=8, Hkv=8, Sq=512, Sk=512, Dk=64, Dv=64, causal=False, seed=0, bwd=False)


def test_lengths_and_input_pos(tylo, oracle):
    """k_lengths masks keys beyond the per-batch length (attention.jl:60); input_pos shifts the
    causal diagonal (attention.jl:61); q_lengths skips whole 64-row blocks (attention.jl:25-26)."""
    rng = np.random.default_rng(3)
    B, H, Sq, Sk, D = 2, 2, 128, 160, 64
    Q, Q64 = draw(rng, (B, H, Sq, D), "f32"); K, K64 = draw(rng, (B, H, Sk, D), "f32"); V, V64 = draw(rng, (B, H, Sk, D), "f32")
    kl = torch.tensor([160, 75], dtype=torch.int32, device="cuda")
    O = tylo.attention(Q, K, V, causal=True, input_pos=32, k_lengths=kl)
    for b, n in enumerate((160, 75)):
        ref = oracle.flex_ref(Q64[b:b + 1], K64[b:b + 1, :, :n], V64[b:b + 1, :, :n], mask=oracle.MaskSpec(causal=True), input_pos=32)
        check(O[b:b + 1], ref, "f32", "k_lengths")
    ql = torch.tensor([128, 40], dtype=torch.int32, device="cuda")
    O2 = torch.full_like(Q, 7.0)
    tylo.attention_(O2, Q, K, V, q_lengths=ql)
    ref = oracle.flex_ref(Q64, K64, V64)
    check(O2[0], ref[0], "f32", "q_lengths full batch entry")
    check(O2[1, :, :64], ref[1, :, :64], "f32", "q_lengths live block")
    assert bool((O2[1, :, 64:] == 7.0).all())          # skipped blocks are left untouched


def test_config3_geometry_sampled(tylo, oracle):
    """Benchmark config 3 geometry (causal GQA, Hq 32 / Hkv 8, D 128, bf16) at S 1024, B 1:
    oracle on every head, forward and backward."""
    _run(tylo, oracle, "bf16", B=1, H=32, Hkv=8, Sq=1024, Sk=1024, Dk=128, Dv=128, causal=True, seed=2)
