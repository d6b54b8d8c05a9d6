"""CPU: the NumPy oracle against the committed known-answer vectors (scalar-loop restatement,
tests/golden/make_golden.py), closed-form cases, and an independent torch float64 formulation."""
from pathlib import Path

import numpy as np
import pytest
import torch

GOLD = np.load(Path(__file__).parent / "golden" / "oracle_kat.npz")
TOL = dict(rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("name,causal", [("full", False), ("causal", True)])
def test_attention_kat(oracle, name, causal):
    Q, K, V, dO = (GOLD[k] for k in ("attn_Q", "attn_K", "attn_V", "attn_dO"))
    np.testing.assert_allclose(oracle.attn_ref(Q, K, V, causal=causal), GOLD[f"attn_{name}_O"], **TOL)
    dQ, dK, dV = oracle.attn_bwd_ref(dO, Q, K, V, causal=causal)
    np.testing.assert_allclose(dQ, GOLD[f"attn_{name}_dQ"], **TOL)
    np.testing.assert_allclose(dK, GOLD[f"attn_{name}_dK"], **TOL)
    np.testing.assert_allclose(dV, GOLD[f"attn_{name}_dV"], **TOL)


def test_flex_kat(oracle):
    Q, K, V, dO = (GOLD[k] for k in ("attn_Q", "attn_K", "attn_V", "attn_dO"))
    mask = oracle.MaskSpec(causal=True, window=int(GOLD["flex_window"]), doc_q=GOLD["flex_docs"])
    score = oracle.ScoreSpec([("alibi", GOLD["flex_slopes"]), ("softcap", float(GOLD["flex_cap"]))])
    ip = int(GOLD["flex_input_pos"])
    np.testing.assert_allclose(oracle.flex_ref(Q, K, V, score=score, mask=mask, input_pos=ip), GOLD["flex_O"], **TOL)
    dQ, dK, dV, _ = oracle.flex_bwd_ref(dO, Q, K, V, score=score, mask=mask, input_pos=ip)
    np.testing.assert_allclose(dQ, GOLD["flex_dQ"], **TOL)
    np.testing.assert_allclose(dK, GOLD["flex_dK"], **TOL)
    np.testing.assert_allclose(dV, GOLD["flex_dV"], **TOL)


def test_decode_kat(oracle):
    O = oracle.decode_reference(GOLD["dec_Q"], GOLD["dec_K"], GOLD["dec_V"], GOLD["dec_lengths"])
    np.testing.assert_allclose(O, GOLD["dec_O"], **TOL)
    assert np.all(O[2] == 0)          # empty cache gives zeros (test/decode.jl:23)


def test_rowwise_kat(oracle):
    X, dY, W, B = (GOLD[k] for k in ("row_X", "row_dY", "row_W", "row_B"))
    eps, off = float(GOLD["row_eps"]), float(GOLD["row_offset"])
    np.testing.assert_allclose(oracle.softmax_ref(X), GOLD["softmax_Y"], **TOL)
    np.testing.assert_allclose(oracle.softmax_bwd_ref(dY, GOLD["softmax_Y"]), GOLD["softmax_dX"], **TOL)
    np.testing.assert_allclose(oracle.rms_norm_ref(X, W, eps=eps, offset=off), GOLD["rms_Y"], **TOL)
    dX, dW, _ = oracle.rms_norm_bwd_ref(dY, X, W, eps=eps, offset=off)
    np.testing.assert_allclose(dX, GOLD["rms_dX"], **TOL)
    np.testing.assert_allclose(dW, GOLD["rms_dW"], **TOL)
    np.testing.assert_allclose(oracle.layer_norm_ref(X, W, B, eps=eps), GOLD["ln_Y"], **TOL)
    dX, dW, dB, _, _ = oracle.layer_norm_bwd_ref(dY, X, W, eps=eps)
    np.testing.assert_allclose(dX, GOLD["ln_dX"], **TOL)
    np.testing.assert_allclose(dW, GOLD["ln_dW"], **TOL)
    np.testing.assert_allclose(dB, GOLD["ln_dB"], **TOL)


def test_closed_forms(oracle):
    rng = np.random.default_rng(0)
    # identical keys => uniform probabilities => O is the mean of V
    Q = rng.standard_normal((1, 2, 3, 8)); K = np.tile(rng.standard_normal((1, 1, 1, 8)), (1, 2, 5, 1))
    V = rng.standard_normal((1, 2, 5, 4))
    np.testing.assert_allclose(oracle.attn_ref(Q, K, V), np.broadcast_to(V.mean(2, keepdims=True), (1, 2, 3, 4)), **TOL)
    # causal: query 0 sees only key 0
    O = oracle.attn_ref(rng.standard_normal((1, 1, 4, 8)), rng.standard_normal((1, 1, 4, 8)), V[:, :1, :4], causal=True)
    np.testing.assert_allclose(O[0, 0, 0], V[0, 0, 0], **TOL)
    # fully masked rows give zeros (test/flex.jl:168-173)
    O = oracle.flex_ref(Q, K, V, mask=oracle.MaskSpec(prefix=0))
    assert np.all(O == 0)
    # softmax rows sum to one; norms have unit rms / zero mean
    X = rng.standard_normal((4, 33))
    np.testing.assert_allclose(oracle.softmax_ref(X).sum(-1), 1.0, rtol=1e-12)
    Y = oracle.rms_norm_ref(X, np.ones(33), eps=0.0)
    np.testing.assert_allclose((Y * Y).mean(-1), 1.0, rtol=1e-12)
    Y = oracle.layer_norm_ref(X, np.ones(33), np.zeros(33), eps=0.0)
    np.testing.assert_allclose(Y.mean(-1), 0.0, atol=1e-12)


def test_against_torch_autograd(oracle):
    """Independent formulation: torch float64 SDPA-style math with autograd for the gradients."""
    g = torch.Generator().manual_seed(5)
    B, H, Hkv, Sq, Sk, D = 2, 4, 2, 9, 11, 8
    Q = torch.randn(B, H, Sq, D, dtype=torch.float64, generator=g, requires_grad=True)
    K = torch.randn(B, Hkv, Sk, D, dtype=torch.float64, generator=g, requires_grad=True)
    V = torch.randn(B, Hkv, Sk, D, dtype=torch.float64, generator=g, requires_grad=True)
    dO = torch.randn(B, H, Sq, D, dtype=torch.float64, generator=g)
    Ke, Ve = K.repeat_interleave(H // Hkv, 1), V.repeat_interleave(H // Hkv, 1)
    S = Q @ Ke.transpose(-1, -2) / D ** 0.5
    cap, ip = 3.0, 2
    slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625], dtype=torch.float64, requires_grad=True)
    q = torch.arange(Sq)[:, None] + ip; kv = torch.arange(Sk)[None, :]
    S = cap * torch.tanh((S + slopes[None, :, None, None] * (q - kv)) / cap)
    S = S.masked_fill(~((q >= kv) & (q <= kv + 4)), float("-inf"))
    O = torch.softmax(S, -1) @ Ve
    O.backward(dO)
    mask = oracle.MaskSpec(causal=True, window=4)
    score = oracle.ScoreSpec([("alibi", slopes.detach().numpy()), ("softcap", cap)])
    args = [t.detach().numpy() for t in (Q, K, V)]
    np.testing.assert_allclose(oracle.flex_ref(*args, score=score, mask=mask, input_pos=ip), O.detach().numpy(), rtol=1e-9, atol=1e-11)
    dQ, dK, dV, sg = oracle.flex_bwd_ref(dO.numpy(), *args, score=score, mask=mask, input_pos=ip)
    np.testing.assert_allclose(dQ, Q.grad.numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dK, K.grad.numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dV, V.grad.numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(sg[0], slopes.grad.numpy(), rtol=1e-9, atol=1e-11)


def test_decode_split_merge_is_exact(oracle):
    """Split partials merged with the reference's combine algebra reproduce the unsplit result
    for any split layout, including empty splits (test/decode.jl:114-124, decode.jl:119-140)."""
    rng = np.random.default_rng(1)
    B, H, Hkv, Sk, D = 3, 8, 2, 50, 16
    Q = rng.standard_normal((B, H, D)); K = rng.standard_normal((B, Hkv, Sk, D)); V = rng.standard_normal((B, Hkv, Sk, D))
    lengths = np.array([50, 17, 0])
    ref = oracle.decode_reference(Q, K, V, lengths)
    for n_splits in (1, 2, 5, 16):
        size = -(-Sk // n_splits)
        parts = [oracle.decode_partials(Q, K, V, lengths, s * size, (s + 1) * size) for s in range(n_splits)]
        O = oracle.decode_combine(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]),
                                  np.stack([p[2] for p in parts]))
        np.testing.assert_allclose(O, ref, rtol=1e-12, atol=1e-14)
