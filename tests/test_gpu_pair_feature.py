"""GPU parity: PairFeatureScore (pair.jl:49-157) through its bias-table lowering, against the oracle fed
with the bias computed by explicit scalar-style math (as test/flex.jl:212-232,403-452 does): forward,
dQ/dK/dV, projection gradient and feature gradients."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw
from test_host import _RbfOp

pytestmark = pytest.mark.gpu


def _check_reduced(got, ref, dt, what):
    """Gradients that sum a bias-table gradient over every (q, kv) pair (projection, features): each term
    carries the 16-bit error of the attention backward, so the sum is held to a bound relative to its own
    largest entry: 1e-2 for 16-bit storage, 1e-4 for fp32 (summation order)."""
    err = np.abs(back(got) - ref)
    bound = (1e-4 if dt == "f32" else 1e-2) * float(np.abs(ref).max()) + 1e-6
    assert err.max() <= bound, f"{what}: max error {err.max():.3e} > {bound:.3e}"


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("compose", [None, "softcap"])
def test_pair_feature_score(tylo, oracle, dt, compose):
    t, o = tylo, oracle
    B, H, Hkv, Sq, Sk, D, F, PD, c = 2, 4, 2, 96, 128, 64, 3, 2, 0.3
    rng = np.random.default_rng(11)
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    qf, qf64 = draw(rng, (B, Sq, F), "f32"); kf, kf64 = draw(rng, (B, Sk, F), "f32"); pr, pr64 = draw(rng, (PD, H), "f32", 0.5)
    mod = t.PairFeatureScore(_RbfOp(c), qf, kf, pr)
    # the reference bias, written out directly (not through pair_feature)
    d2 = ((qf64[:, :, None, :] - kf64[:, None, :, :]) ** 2).sum(-1)             # (B, Sq, Sk)
    phi = np.stack([np.exp(-c * d2), d2 * np.exp(-c * d2)])                     # (PD, B, Sq, Sk)
    bias64 = np.einsum("ph,pbqk->bhqk", pr64, phi)
    ops = [("bias", bias64)]
    smod = mod
    if compose == "softcap":
        smod, ops = t.SoftCapScore(6.0) @ mod, ops + [("softcap", 6.0)]
    kw = dict(score_mod=smod, mask_mod=t.CausalMask()); okw = dict(score=o.ScoreSpec(ops), mask=o.MaskSpec(causal=True))
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    check(O, o.flex_ref(Q64, K64, V64, **okw), dt, "pair fwd")

    dO, dO64 = draw(rng, tuple(O.shape), dt)
    d_mod = t.grad_shadow(smod) if compose else t.grad_shadow(mod, feature_grads=True)
    dQ, dK, dV = t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, d_score_mod=d_mod, **kw)
    rQ, rK, rV, pg = o.flex_bwd_ref(dO64, Q64, K64, V64, **okw)
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"pair {name}", scale_hint=float(np.abs(ref).max()))
    dbias = pg[0]                                                                # (B, H, Sq, Sk) gradient of the table
    leaf = d_mod.a if compose else d_mod
    proj_ref = np.einsum("bhqk,pbqk->ph", dbias, phi)
    _check_reduced(leaf.pair_proj, proj_ref, dt, "pair projection gradient")
    if not compose:
        # d bias / d d2 = sum_p proj[p, h] * dphi_p/dd2, then d d2 / d qf = 2 (qf - kf)
        e = np.exp(-c * d2)
        dphi_dd2 = np.stack([-c * e, e - c * d2 * e])                            # (PD, B, Sq, Sk)
        g = np.einsum("bhqk,ph,pbqk->bqk", dbias, pr64, dphi_dd2)
        diff = qf64[:, :, None, :] - kf64[:, None, :, :]
        qref = (2 * g[..., None] * diff).sum(2); kref = (-2 * g[..., None] * diff).sum(1)
        _check_reduced(leaf.q_features, qref, dt, "pair q-feature gradient")
        _check_reduced(leaf.k_features, kref, dt, "pair k-feature gradient")
    assert tylo.device_status() == 0
