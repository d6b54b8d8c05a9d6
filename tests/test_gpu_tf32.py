"""GPU parity of the opt-in TF32 forward: Float32 storage, both matrix products on the tensor cores with the
operands read as TF32 (`tensorcore=TFloat32`; the reference's default for Float32, utils.jl:43-44).

The oracle is the float64 one, fed the fp32 inputs.  Tolerance: a TF32 operand keeps 10 mantissa bits, so each
product carries a relative error of up to 2^-9; over head dim 64 and 1/8 scaling that is about 1e-3 absolute on
a score and 1e-3 relative on a probability.  The test holds the output to max-abs 4e-3 * max(1, max|ref|) and
mean-abs 4e-4, a fifth of the bf16 contract; the true-fp32 default stays at 1e-5 relative (test_gpu_attention.py).
Measured errors are printed (run with -s).
"""
import numpy as np
import pytest
import torch

from gpu_util import back, draw

pytestmark = pytest.mark.gpu


def _check_tf32(got, ref, what):
    g = back(got)
    assert g.shape == ref.shape and np.isfinite(g).all(), what
    err = np.abs(g - ref)
    s = max(1.0, float(np.abs(ref).max()))
    print(f"PARITY tf32 {what}: max_abs {err.max():.3e} mean_abs {err.mean():.3e} max_ref {np.abs(ref).max():.3e}")
    assert err.max() <= 4e-3 * s, f"{what}: max-abs error {err.max():.3e}"
    assert err.mean() <= 4e-4 * s, f"{what}: mean-abs error {err.mean():.3e}"
    return err.max()


def _run(tylo, oracle, *, B, H, Hkv, Sq, Sk, D, causal, seed, k_lengths=None, input_pos=0):
    rng = np.random.default_rng(seed)
    Q, Q64 = draw(rng, (B, H, Sq, D), "f32")
    K, K64 = draw(rng, (B, Hkv, Sk, D), "f32")
    V, V64 = draw(rng, (B, Hkv, Sk, D), "f32")
    cp = tylo.allocate_checkpoints_attention(Q, K, V)
    kl = None if k_lengths is None else torch.tensor(k_lengths, dtype=torch.int32, device="cuda")
    O = tylo.attention(Q, K, V, causal=causal, checkpoints=cp, tensorcore=tylo.TFloat32, k_lengths=kl,
                       input_pos=input_pos)
    assert tylo.device_status() == 0
    mask = oracle.MaskSpec(causal=True) if causal else None
    Oref = np.zeros((B, H, Sq, D)); lse_ref = np.zeros((B, H, Sq))
    for b in range(B):                      # keys at or beyond k_lengths[b] do not exist for the oracle
        n = Sk if k_lengths is None else k_lengths[b]
        o, m, l = oracle.flex_ref(Q64[b:b + 1], K64[b:b + 1, :, :n], V64[b:b + 1, :, :n], mask=mask, return_stats=True,
                                  input_pos=input_pos)
        Oref[b], lse_ref[b] = o[0], (m + np.log(l))[0]
    worst = _check_tf32(O, Oref, f"O B{B} H{H}/{Hkv} S{Sq}x{Sk} D{D} causal={causal}")
    lse = back(cp.M) * np.log(2.0) + np.log(back(cp.L))
    ok = np.isfinite(lse_ref)
    np.testing.assert_allclose(lse[ok], lse_ref[ok], rtol=0, atol=4e-3)
    # the true-fp32 default on the same inputs is three orders of magnitude closer: the flag is what changed
    O32 = tylo.attention(Q, K, V, causal=causal, k_lengths=kl, input_pos=input_pos)
    e32 = float(np.abs(back(O32) - Oref).max())
    assert e32 <= 1e-5 * float(np.abs(Oref).max()) + 1e-6
    assert worst > 10 * e32, "the TF32 call did not run on TF32 operands"


@pytest.mark.parametrize("causal", [False, True])
def test_config1_shape(tylo, oracle, causal):
    """Benchmark config 1 (B 2, H 8, S 512, D 64, seed 0) with TF32 operands."""
    _run(tylo, oracle, B=2, H=8, Hkv=8, Sq=512, Sk=512, D=64, causal=causal, seed=0)


@pytest.mark.parametrize("shape", [
    dict(B=2, H=4, Hkv=2, Sq=96, Sk=128, D=64),       # reference test shape, GQA
    dict(B=1, H=6, Hkv=2, Sq=300, Sk=517, D=64),      # odd group size, ragged tile edges, Sq != Sk
    dict(B=2, H=8, Hkv=2, Sq=1024, Sk=1024, D=32),    # head dim 32; more items than one pass of small launches
    dict(B=1, H=2, Hkv=2, Sq=1, Sk=300, D=64),        # single query row
    dict(B=1, H=4, Hkv=2, Sq=200, Sk=333, D=48),      # zero-padded to the 64-wide tile
    dict(B=1, H=2, Hkv=2, Sq=96, Sk=96, D=20),        # rows of 80 bytes, padded to the 32-wide tile
])
@pytest.mark.parametrize("causal", [False, True])
def test_shapes(tylo, oracle, shape, causal):
    _run(tylo, oracle, causal=causal, seed=5, **shape)


def test_many_items_per_cta(tylo, oracle):
    """Enough work items for the persistent form (more items than SMs)."""
    _run(tylo, oracle, B=2, H=16, Hkv=4, Sq=2048, Sk=2048, D=64, causal=True, seed=6)


def test_key_lengths_and_input_pos(tylo, oracle):
    _run(tylo, oracle, B=3, H=4, Hkv=2, Sq=128, Sk=384, D=64, causal=True, seed=7, k_lengths=[384, 200, 129],
         input_pos=256)


def test_flex_mods(tylo, oracle):
    """Window + document mask and a soft cap through the run-time-flag variant, natural-base statistics."""
    rng = np.random.default_rng(11)
    B, H, S, D, W, cap = 2, 4, 640, 64, 200, 20.0
    Q, Q64 = draw(rng, (B, H, S, D), "f32", scale=1.5)
    K, K64 = draw(rng, (B, H, S, D), "f32", scale=1.5)
    V, V64 = draw(rng, (B, H, S, D), "f32")
    tab = np.sort(rng.integers(0, 4, size=(B, S)), axis=1).astype(np.int32)
    docs = torch.from_numpy(tab).cuda()
    mask = tylo.CausalMask() & tylo.SlidingWindowMask(W) & tylo.DocumentMask(docs)
    cp = tylo.allocate_checkpoints_flex_attention(Q, K, V)
    O = tylo.flex_attention(Q, K, V, score_mod=tylo.SoftCapScore(cap), mask_mod=mask, checkpoints=cp,
                            tensorcore=tylo.TFloat32)
    assert tylo.device_status() == 0
    for b in range(B):
        m = oracle.MaskSpec(causal=True, window=W, doc_q=tab[b], doc_kv=tab[b])
        Oref, Mref, Lref = oracle.flex_ref(Q64[b:b + 1], K64[b:b + 1], V64[b:b + 1], score=oracle.ScoreSpec([("softcap", cap)]),
                                           mask=m, return_stats=True)
        _check_tf32(O[b:b + 1], Oref, f"flex O batch {b}")
        np.testing.assert_allclose(back(cp.M[b:b + 1]) + np.log(back(cp.L[b:b + 1])), Mref + np.log(Lref), rtol=0, atol=1e-2)


def test_head_dim_without_a_tensor_core_form_runs_in_fp32(tylo, oracle):
    """Head dim 128 has no TF32 kernel (the tiles would not fit shared memory): the call computes in true fp32."""
    rng = np.random.default_rng(12)
    Q, Q64 = draw(rng, (1, 2, 96, 128), "f32"); K, K64 = draw(rng, (1, 2, 160, 128), "f32"); V, V64 = draw(rng, (1, 2, 160, 128), "f32")
    O = tylo.attention(Q, K, V, tensorcore=tylo.TFloat32)
    Oref = oracle.flex_ref(Q64, K64, V64)
    assert float(np.abs(back(O) - Oref).max()) <= 1e-5 * float(np.abs(Oref).max()) + 1e-6


def test_backward_rejects_the_tf32_code(tylo):
    import ctypes
    lib = ctypes.CDLL(str(tylo._LIB_PATH))
    rc = lib.tylo_b200_attention_bwd_workspace_bytes(64, 64, 128, 128, 2, 2, 1, tylo.F32_TF32)
    assert rc == 0      # no tensor-core backward workspace for it: the backward entry points take TYLO_F32
