"""GPU parity: ALiBi slope gradient (mods.jl:296-303) from the tensor-core backward (16-bit storage),
alone and under a soft cap on either side, against the oracle.  fp16 storage keeps the rounding of O
(which enters through Delta) small enough for a few-percent bound on this ill-conditioned sum."""
import numpy as np
import pytest
import torch

from gpu_util import back, draw

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chain", ["alibi", "softcap o alibi", "alibi o softcap"])
def test_slope_gradient_tensor_core(tylo, oracle, chain):
    t, o = tylo, oracle
    rng = np.random.default_rng(len(chain))
    B, H, Hkv, S, D = 2, 4, 2, 256, 64
    Q, Q64 = draw(rng, (B, H, S, D), "f16"); K, K64 = draw(rng, (B, Hkv, S, D), "f16"); V, V64 = draw(rng, (B, Hkv, S, D), "f16")
    slopes = torch.tensor([0.02, -0.01, 0.005, 0.03], device="cuda")
    s64 = back(slopes)
    if chain == "alibi":
        mod, ops = t.AliBiScore(slopes), [("alibi", s64)]
    elif chain == "softcap o alibi":
        mod, ops = t.SoftCapScore(8.0) @ t.AliBiScore(slopes), [("alibi", s64), ("softcap", 8.0)]
    else:
        mod, ops = t.AliBiScore(slopes) @ t.SoftCapScore(8.0), [("softcap", 8.0), ("alibi", s64)]
    kw = dict(score_mod=mod, mask_mod=t.CausalMask()); okw = dict(score=o.ScoreSpec(ops), mask=o.MaskSpec(causal=True))
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    dO, dO64 = draw(rng, tuple(O.shape), "f16")
    d_mod = t.grad_shadow(mod)
    t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, d_score_mod=d_mod, **kw)
    _, _, _, pg = o.flex_bwd_ref(dO64, Q64, K64, V64, **okw)
    ref = [v for i, v in pg.items() if ops[i][0] == "alibi"][0]

    def find(m):
        if isinstance(m, t.AliBiScore):
            return m
        if isinstance(m, t.ComposeScore):
            return find(m.a) or find(m.b)
        return None

    got = back(find(d_mod).slopes)
    assert np.all(np.abs(got - ref) <= 0.03 * np.abs(ref).max() + 0.05 * S / 256), (got, ref)
    assert t.device_status() == 0
