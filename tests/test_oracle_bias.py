"""CPU: the oracle's BiasScore forward/backward (mods.jl:212-237, 305-313) is consistent with itself —
its analytic gradients equal central finite differences of its own forward — and the host evaluator of
the Python mirror agrees with the oracle's table indexing (local rows, mod1 broadcast)."""
import numpy as np

from conftest import load_oracle


def _loss(o, Q, K, V, W, ops, mask):
    return float(np.sum(o.flex_ref(Q, K, V, score=o.ScoreSpec(ops), mask=mask) * W))


def test_bias_gradients_match_finite_differences():
    o = load_oracle()
    rng = np.random.default_rng(0)
    B, H, Hkv, Sq, Sk, D = 2, 4, 2, 5, 7, 4
    Q = rng.standard_normal((B, H, Sq, D)); K = rng.standard_normal((B, Hkv, Sk, D)); V = rng.standard_normal((B, Hkv, Sk, D))
    W = rng.standard_normal((B, H, Sq, D))
    bias = rng.standard_normal((1, 2, Sq, Sk))               # broadcast over batch, two head slices for four heads
    mask = o.MaskSpec(causal=True)
    for ops in ([("bias", bias)], [("bias", bias), ("softcap", 3.0)], [("softcap", 3.0), ("bias", bias)]):
        dQ, dK, dV, pg = o.flex_bwd_ref(W, Q, K, V, score=o.ScoreSpec(ops), mask=mask)
        i_bias = [i for i, (k, _) in enumerate(ops) if k == "bias"][0]
        g = pg[i_bias]
        assert g.shape == bias.shape
        eps = 1e-6
        for idx in [(0, 0, 0, 0), (0, 1, 3, 2), (0, 0, 4, 4), (0, 1, 2, 6)]:
            bp, bm = bias.copy(), bias.copy()
            bp[idx] += eps; bm[idx] -= eps
            opp = [(k, bp if k == "bias" else p) for k, p in ops]
            opm = [(k, bm if k == "bias" else p) for k, p in ops]
            fd = (_loss(o, Q, K, V, W, opp, mask) - _loss(o, Q, K, V, W, opm, mask)) / (2 * eps)
            assert abs(fd - g[idx]) <= 1e-6 * max(1.0, abs(fd)), (ops[0][0], idx, fd, g[idx])
        # one entry of dQ as well: the bias op must not disturb the chain rule to the inputs
        Qp, Qm = Q.copy(), Q.copy()
        Qp[1, 2, 3, 1] += eps; Qm[1, 2, 3, 1] -= eps
        fd = (_loss(o, Qp, K, V, W, ops, mask) - _loss(o, Qm, K, V, W, ops, mask)) / (2 * eps)
        assert abs(fd - dQ[1, 2, 3, 1]) <= 1e-6 * max(1.0, abs(fd))


def test_masked_pairs_get_no_bias_gradient():
    o = load_oracle()
    rng = np.random.default_rng(1)
    Q = rng.standard_normal((1, 1, 4, 4)); K = rng.standard_normal((1, 1, 4, 4)); V = rng.standard_normal((1, 1, 4, 4))
    bias = rng.standard_normal((1, 1, 4, 4))
    _, _, _, pg = o.flex_bwd_ref(np.ones((1, 1, 4, 4)), Q, K, V, score=o.ScoreSpec([("bias", bias)]), mask=o.MaskSpec(causal=True))
    assert np.all(pg[0][0, 0][np.triu_indices(4, 1)] == 0.0)
