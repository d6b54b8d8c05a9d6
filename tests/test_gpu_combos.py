"""GPU parity of feature combinations on the tensor-core kernels: zero-padded head dims with score / mask mods,
bias tables with ALiBi and padded head dims, OR-ed clauses over more than one tile with GQA, block lists with TF32
operands, many items per CTA with mods.  Each against the float64 oracle, forward and (where one exists) backward."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw

pytestmark = pytest.mark.gpu


def _fwd_bwd(t, o, dt, Q, K, V, Q64, K64, V64, kw, okw, rng, what, d_score_mod=None):
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    check(O, o.flex_ref(Q64, K64, V64, **okw), dt, f"{what} fwd")
    dO, dO64 = draw(rng, tuple(O.shape), dt)
    extra = {} if d_score_mod is None else dict(d_score_mod=d_score_mod)
    dQ, dK, dV = t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, **kw, **extra)
    rQ, rK, rV, pg = o.flex_bwd_ref(dO64, Q64, K64, V64, **okw)
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"{what} {name}", scale_hint=float(np.abs(ref).max()))
    assert t.device_status() == 0
    return pg


@pytest.mark.parametrize("D", [96, 40])
def test_padded_head_dim_with_window_documents_softcap(tylo, oracle, D):
    t, o = tylo, oracle
    rng = np.random.default_rng(D)
    B, H, Hkv, S, W = 2, 4, 2, 700, 150
    dt = "bf16"
    Q, Q64 = draw(rng, (B, H, S, D), dt); K, K64 = draw(rng, (B, Hkv, S, D), dt); V, V64 = draw(rng, (B, Hkv, S, D), dt)
    docs = np.sort(rng.integers(0, 5, size=S)).astype(np.int32)
    mask = t.CausalMask() & t.SlidingWindowMask(W) & t.DocumentMask(torch.from_numpy(docs).cuda())
    kw = dict(mask_mod=mask, score_mod=t.SoftCapScore(15.0))
    okw = dict(mask=o.MaskSpec(causal=True, window=W, doc_q=docs), score=o.ScoreSpec([("softcap", 15.0)]))
    _fwd_bwd(t, o, dt, Q, K, V, Q64, K64, V64, kw, okw, rng, f"D{D} window+doc+softcap")


def test_bias_with_alibi_and_padded_head_dim(tylo, oracle):
    """Both additive mods at once (the straight-line path), head dim 80, Sq != Sk, slope and table gradients."""
    t, o = tylo, oracle
    rng = np.random.default_rng(4)
    B, H, Hkv, Sq, Sk, D = 2, 4, 2, 200, 333, 80
    dt = "bf16"
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    bias, bias64 = draw(rng, (1, H, Sq, Sk), "f32")
    slopes, slopes64 = draw(rng, (H,), "f32", scale=0.02)
    mod = t.BiasScore(bias) @ t.AliBiScore(slopes)                 # ALiBi first, then the table
    ops = [("alibi", slopes64), ("bias", bias64)]
    kw = dict(score_mod=mod, mask_mod=t.CausalMask())
    okw = dict(score=o.ScoreSpec(ops), mask=o.MaskSpec(causal=True))
    d_mod = t.grad_shadow(mod)
    pg = _fwd_bwd(t, o, dt, Q, K, V, Q64, K64, V64, kw, okw, rng, "alibi+bias D80", d_score_mod=d_mod)
    leaves = {}
    def walk(m):
        if isinstance(m, t.ComposeScore):
            walk(m.a); walk(m.b)
        elif isinstance(m, t.BiasScore):
            leaves["bias"] = m.bias
        elif isinstance(m, t.AliBiScore):
            leaves["alibi"] = m.slopes
    walk(d_mod)
    for i, (name, _) in enumerate(ops):
        ref = pg[i]
        check(leaves[name], ref, dt, f"{name} gradient", scale_hint=2 * float(np.abs(ref).max()))


def test_or_clauses_over_many_tiles_gqa(tylo, oracle):
    """Affine OR clauses on the tensor-core forward and backward over several 128-wide tiles."""
    t, o = tylo, oracle
    rng = np.random.default_rng(8)
    B, H, Hkv, S, D = 1, 8, 2, 900, 128
    dt = "bf16"
    Q, Q64 = draw(rng, (B, H, S, D), dt); K, K64 = draw(rng, (B, Hkv, S, D), dt); V, V64 = draw(rng, (B, Hkv, S, D), dt)
    mask = (t.CausalMask() & t.SlidingWindowMask(100)) | t.PrefixMask(200) | (t.CausalMask() & t.SlidingWindowMask(400) & t.PrefixMask(700))
    omask = o.MaskAny(o.MaskSpec(causal=True, window=100), o.MaskSpec(prefix=200), o.MaskSpec(causal=True, window=400, prefix=700))
    _fwd_bwd(t, o, dt, Q, K, V, Q64, K64, V64, dict(mask_mod=mask), dict(mask=omask), rng, "three clauses")


def test_block_list_with_tf32(tylo, oracle):
    t, o = tylo, oracle
    rng = np.random.default_rng(9)
    B, H, Hkv, S, D, TM, TN = 1, 4, 2, 384, 64, 64, 32
    Q, Q64 = draw(rng, (B, H, S, D), "f32"); K, K64 = draw(rng, (B, Hkv, S, D), "f32"); V, V64 = draw(rng, (B, Hkv, S, D), "f32")
    keep = lambda q, kv: q >= kv and q - kv <= 120
    cnt, idx, full = o.build_block_mask_ref(keep, S, S, TILE_M=TM, TILE_N=TN)
    bm = t.BlockMask(torch.from_numpy(cnt).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(full).cuda(), TM, TN)
    mask = t.CausalMask() & t.SlidingWindowMask(120)
    O = t.flex_attention(Q, K, V, mask_mod=mask, block_mask=bm, tensorcore=t.TFloat32)
    ref = o.flex_block_mask_ref(Q64, K64, V64, cnt, idx, full, TILE_M=TM, TILE_N=TN, mask=o.MaskSpec(causal=True, window=120))
    err = np.abs(back(O) - ref)
    assert err.max() <= 4e-3 * max(1.0, float(np.abs(ref).max())) and err.mean() <= 4e-4       # the TF32 bound
    O32 = t.flex_attention(Q, K, V, mask_mod=mask, block_mask=bm)
    check(O32, ref, "f32", "block list, true fp32")
    assert err.max() > 10 * float(np.abs(back(O32) - ref).max())                                 # TF32 really ran
    assert t.device_status() == 0


def test_many_items_per_cta_with_alibi(tylo, oracle):
    """More work items than SMs under a causal mask with a score mod (persistent CTAs, chunked tile loop)."""
    t, o = tylo, oracle
    rng = np.random.default_rng(10)
    B, H, Hkv, S, D = 2, 16, 4, 1536, 64
    dt = "bf16"
    Q, Q64 = draw(rng, (B, H, S, D), dt); K, K64 = draw(rng, (B, Hkv, S, D), dt); V, V64 = draw(rng, (B, Hkv, S, D), dt)
    slopes, slopes64 = draw(rng, (H,), "f32", scale=0.01)
    kw = dict(score_mod=t.AliBiScore(slopes), mask_mod=t.CausalMask())
    okw = dict(score=o.ScoreSpec([("alibi", slopes64)]), mask=o.MaskSpec(causal=True))
    # the oracle on a sample of (batch, kv-head) groups keeps the test short
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    G = H // Hkv
    for b, hk in ((0, 0), (1, 3)):
        hs = slice(hk * G, (hk + 1) * G)
        sk = dict(score=o.ScoreSpec([("alibi", slopes64[hs])]), mask=o.MaskSpec(causal=True))
        check(O[b:b + 1, hs], o.flex_ref(Q64[b:b + 1, hs], K64[b:b + 1, hk:hk + 1], V64[b:b + 1, hk:hk + 1], **sk), dt, "alibi many items")
    assert t.device_status() == 0
