"""GPU parity: document masks whose documents span whole 128-position tiles — tiles of a foreign
document (skipped by the kernels), tiles of the rows' own document (no element-wise comparison) and
tiles with a boundary inside — forward and backward, alone and combined with causal / sliding window /
soft cap, batch-shared and per-batch id tables (DocumentMask, mods.jl:141-147)."""
import numpy as np
import pytest
import torch

from gpu_util import check, draw

pytestmark = pytest.mark.gpu

S = 1024
CUTS = {
    "tile aligned": [256, 640],                  # boundaries on tile edges: every tile is one document
    "inside tiles": [100, 333, 700],             # boundaries inside tiles
    "mixed": [128, 200, 768, 1000],
}


def _table(cuts):
    return np.searchsorted(np.asarray(cuts), np.arange(S), side="right").astype(np.int32)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("extra", ["docs only", "causal", "causal+window+softcap"])
@pytest.mark.parametrize("cuts", list(CUTS), ids=list(CUTS))
def test_document_tiles(tylo, oracle, cuts, extra, dt):
    t, o = tylo, oracle
    rng = np.random.default_rng(len(cuts) + len(extra))
    B, H, Hkv, D = 2, 2, 1, 128 if dt == "bf16" else 64
    Q, Q64 = draw(rng, (B, H, S, D), dt); K, K64 = draw(rng, (B, Hkv, S, D), dt); V, V64 = draw(rng, (B, Hkv, S, D), dt)
    tab = np.stack([_table(CUTS[cuts]), _table([c + 17 for c in CUTS[cuts]])])      # one table per batch entry
    mask = t.DocumentMask(torch.from_numpy(tab).cuda())
    kw, okw = {}, dict(doc_per_batch=tab)
    if extra == "docs only":
        okw["mask"] = o.MaskSpec()
    elif extra == "causal":
        mask = t.CausalMask() & mask; okw["mask"] = o.MaskSpec(causal=True)
    else:
        mask = t.CausalMask() & t.SlidingWindowMask(300) & mask
        okw["mask"] = o.MaskSpec(causal=True, window=300)
        kw["score_mod"] = t.SoftCapScore(20.0); okw["score"] = o.ScoreSpec([("softcap", 20.0)])
    kw["mask_mod"] = mask
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    check(O, o.flex_ref(Q64, K64, V64, **okw), dt, "docs fwd")
    dO, dO64 = draw(rng, tuple(O.shape), dt)
    dQ, dK, dV = t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, **kw)
    rQ, rK, rV, _ = o.flex_bwd_ref(dO64, Q64, K64, V64, **okw)
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"docs {name}", scale_hint=float(np.abs(ref).max()))
    assert t.device_status() == 0
