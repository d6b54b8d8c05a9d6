"""GPU parity: BiasScore (mods.jl:212-237) forward, backward and bias gradient (mods.jl:305-313) against
the oracle; cases follow test/flex.jl's bias cases in spirit: full table, broadcast over heads and
batch, composed with a soft cap on either side, under a causal mask, GQA, uneven lengths."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw

pytestmark = pytest.mark.gpu

CASES = [  # name, B, H, Hkv, Sq, Sk, D, bias (nb, nh), compose, causal
    ("full table", 2, 2, 2, 96, 160, 64, (2, 2), None, False),
    ("broadcast heads+batch", 2, 4, 2, 128, 128, 64, (1, 1), None, True),
    ("broadcast heads", 2, 4, 4, 100, 150, 32, (2, 1), None, True),
    ("bias then softcap", 1, 2, 1, 128, 192, 128, (1, 2), "cap_outer", False),
    ("softcap then bias", 1, 2, 1, 128, 192, 128, (1, 2), "cap_inner", True),
]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_bias_score(tylo, oracle, case, dt):
    t, o = tylo, oracle
    _, B, H, Hkv, Sq, Sk, D, (nb, nh), compose, causal = case
    rng = np.random.default_rng(Sq + Sk + nh)
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    bias, bias64 = draw(rng, (nb, nh, Sq, Sk), "f32")
    mod, ops = t.BiasScore(bias), [("bias", bias64)]
    if compose == "cap_outer":
        mod, ops = t.SoftCapScore(4.0) @ mod, ops + [("softcap", 4.0)]
    elif compose == "cap_inner":
        mod, ops = mod @ t.SoftCapScore(4.0), [("softcap", 4.0)] + ops
    kw = dict(score_mod=mod); okw = dict(score=o.ScoreSpec(ops))
    if causal:
        kw["mask_mod"] = t.CausalMask(); okw["mask"] = o.MaskSpec(causal=True)
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    check(O, o.flex_ref(Q64, K64, V64, **okw), dt, "bias fwd")

    dO, dO64 = draw(rng, tuple(O.shape), dt)
    d_mod = t.grad_shadow(mod)
    dQ, dK, dV = t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, d_score_mod=d_mod, **kw)
    rQ, rK, rV, pg = o.flex_bwd_ref(dO64, Q64, K64, V64, **okw)
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"bias {name}", scale_hint=float(np.abs(ref).max()))
    def find(m):
        if isinstance(m, t.BiasScore):
            return m
        if isinstance(m, t.ComposeScore):
            return find(m.a) or find(m.b)
        return None

    leaf = find(d_mod)
    ref = [v for i, v in pg.items() if ops[i][0] == "bias"][0]
    # The bias gradient is dS itself, P (dP - Delta) per pair.  The kernel's Delta comes from O as stored
    # (rounded to 16 bits by the forward), the oracle's from the exact O, so for 16-bit storage each row
    # carries an offset of about |Delta| * 2^-9 on its largest probabilities: compare at half the
    # gradient's own magnitude there; fp32 storage pins the formula at 1e-5.
    check(leaf.bias, ref, dt, "bias gradient", scale_hint=2 * float(np.abs(ref).max()))
    assert tylo.device_status() == 0


def test_bias_rejections(tylo):
    Q = torch.randn(1, 2, 64, 64, device="cuda"); K = torch.randn(1, 2, 64, 64, device="cuda"); V = torch.randn_like(K)
    with pytest.raises(ValueError):
        tylo.flex_attention(Q, K, V, score_mod=tylo.BiasScore(torch.zeros(1, 1, 64, 32, device="cuda")))
    with pytest.raises(TypeError):
        tylo.flex_attention(Q, K, V, score_mod=tylo.BiasScore(torch.zeros(1, 1, 64, 64, device="cuda", dtype=torch.bfloat16)))
    slopes = torch.ones(2, device="cuda")
    both_sides = tylo.BiasScore(torch.zeros(1, 1, 64, 64, device="cuda")) @ (tylo.SoftCapScore(5.0) @ tylo.AliBiScore(slopes))
    with pytest.raises(tylo.TyloError):
        tylo.flex_attention(Q, K, V, score_mod=both_sides)


def test_score_chain_mapping(tylo):
    """Composed score mods -> descriptor flags: additive mods on either side of the soft cap."""
    bias = torch.zeros(1, 1, 4, 4, device="cuda")
    slopes = torch.ones(2, device="cuda")
    keep = []
    d = tylo._score_desc(tylo.SoftCapScore(5.0) @ (tylo.BiasScore(bias) @ tylo.AliBiScore(slopes)), None, keep)
    assert d.flags == tylo.SCORE_SOFTCAP | tylo.SCORE_BIAS | tylo.SCORE_ALIBI and (d.bias_batch, d.bias_heads) == (1, 1)
    d = tylo._score_desc(tylo.BiasScore(bias) @ tylo.SoftCapScore(5.0), None, keep)
    assert d.flags == tylo.SCORE_SOFTCAP | tylo.SCORE_BIAS | tylo.SCORE_SOFTCAP_FIRST
