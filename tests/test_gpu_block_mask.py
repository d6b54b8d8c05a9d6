"""GPU parity: flex_attention! with a host-built BlockMask (flex.jl:107-182,347-360; mods.jl:436-476)
against the oracle's restatement of the block walk.  The first two cases are the reference's own
(test/flex.jl:258-280: three documents over 192 positions; causal with Sq 100, Sk 150); the others
check what the walk does when the list and the mask mod disagree (unlisted blocks contribute nothing,
blocks marked full skip the mask mod), other block edges, GQA with a score mod, and the statistics."""
import numpy as np
import pytest
import torch

from gpu_util import check, draw

pytestmark = pytest.mark.gpu


def _bm_from_oracle(t, o, keep, n_q, n_kv, **kw):
    cnt, idx, full = o.build_block_mask_ref(keep, n_q, n_kv, **kw)
    return (cnt, idx, full), t.BlockMask(torch.from_numpy(cnt).cuda(), torch.from_numpy(idx).cuda(),
                                         torch.from_numpy(full).cuda(), kw.get("TILE_M", 64), kw.get("TILE_N", 64))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_reference_document_case(tylo, oracle, dt):
    t, o = tylo, oracle
    rng = np.random.default_rng(5)
    S, D = 192, 64
    docs = np.concatenate([np.full(70, 1), np.full(80, 2), np.full(42, 3)]).astype(np.int32)
    Q, Q64 = draw(rng, (1, 2, S, D), dt); K, K64 = draw(rng, (1, 2, S, D), dt); V, V64 = draw(rng, (1, 2, S, D), dt)
    bm = t.build_block_mask(lambda q, kv: docs[q] == docs[kv], S, S)
    ref_arrays = o.build_block_mask_ref(lambda q, kv: docs[q] == docs[kv], S, S)
    for got, ref in zip((bm.count, bm.idx, bm.full), ref_arrays):
        assert np.array_equal(got.cpu().numpy(), ref)
    dm = t.DocumentMask(torch.from_numpy(docs).cuda())
    O = t.flex_attention(Q, K, V, mask_mod=dm, block_mask=bm)
    ref = o.flex_ref(Q64, K64, V64, mask=o.MaskSpec(doc_q=docs))
    check(O, ref, dt, "block mask, documents")
    check(O, o.flex_block_mask_ref(Q64, K64, V64, *ref_arrays, mask=o.MaskSpec(doc_q=docs)), dt, "block walk, documents")
    assert t.device_status() == 0


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_reference_causal_case(tylo, oracle, dt):
    t, o = tylo, oracle
    rng = np.random.default_rng(6)
    Sq, Sk, D = 100, 150, 64
    Q, Q64 = draw(rng, (1, 2, Sq, D), dt); K, K64 = draw(rng, (1, 2, Sk, D), dt); V, V64 = draw(rng, (1, 2, Sk, D), dt)
    bm = t.build_block_mask(lambda q, kv: q >= kv, Sq, Sk)
    O = t.flex_attention(Q, K, V, mask_mod=t.CausalMask(), block_mask=bm)
    check(O, o.flex_ref(Q64, K64, V64, mask=o.MaskSpec(causal=True)), dt, "block mask, causal")
    assert t.device_status() == 0


@pytest.mark.parametrize("tiles", [(64, 64), (128, 32), (32, 96)])
def test_walk_semantics_when_list_and_mask_disagree(tylo, oracle, tiles):
    t, o = tylo, oracle
    TM, TN = tiles
    rng = np.random.default_rng(TM + TN)
    B, H, Hkv, Sq, Sk, D = 2, 4, 2, 300, 420, 128
    dt = "bf16"
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    (cnt, idx, full), _ = _bm_from_oracle(t, o, lambda q, kv: q + 40 >= kv, Sq, Sk, TILE_M=TM, TILE_N=TN, input_pos=7)
    # drop the last listed block of every second query block, mark a partial block full, list blocks out of order
    cnt = cnt.copy(); full = full.copy(); idx = idx.copy()
    for i in range(0, len(cnt), 2):
        if cnt[i] > 1:
            cnt[i] -= 1
    full[1, 0] = 1 - full[1, 0]
    idx[0, :cnt[0]] = idx[0, :cnt[0]][::-1].copy(); full[0, :cnt[0]] = full[0, :cnt[0]][::-1].copy()
    bm = t.BlockMask(torch.from_numpy(cnt).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(full).cuda(), TM, TN)
    mask = t.CausalMask() & t.SlidingWindowMask(200)
    omask = o.MaskSpec(causal=True, window=200)
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, mask_mod=mask, score_mod=t.SoftCapScore(30.0), block_mask=bm, input_pos=7, checkpoints=cp)
    ref, Mr, Lr = o.flex_block_mask_ref(Q64, K64, V64, cnt, idx, full, TILE_M=TM, TILE_N=TN, mask=omask,
                                        score=o.ScoreSpec([("softcap", 30.0)]), input_pos=7, return_stats=True)
    check(O, ref, dt, f"block walk {tiles}")
    M = cp.M.cpu().numpy().astype(np.float64); L = cp.L.cpu().numpy().astype(np.float64)
    live = Lr > 0
    assert np.array_equal(L > 0, live)
    assert np.all(np.isneginf(M[~live]))
    lse, lse_ref = M[live] + np.log(L[live]), Mr[live] + np.log(Lr[live])
    assert np.max(np.abs(lse - lse_ref)) < 2e-2
    assert t.device_status() == 0


def test_block_edges_must_be_multiples_of_32(tylo):
    t = tylo
    Q = torch.randn(1, 1, 96, 64, device="cuda").bfloat16()
    bm = t.build_block_mask(lambda q, kv: q >= kv, 96, 96, TILE_M=48, TILE_N=48)
    with pytest.raises(t.TyloError):
        t.flex_attention(Q, Q, Q, mask_mod=t.CausalMask(), block_mask=bm)
    bm64 = t.build_block_mask(lambda q, kv: q >= kv, 200, 96)
    with pytest.raises(ValueError):
        t.flex_attention(Q, Q, Q, mask_mod=t.CausalMask(), block_mask=bm64)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("agree", [True, False], ids=["list agrees with mask", "list edited"])
def test_backward_over_the_listed_blocks(tylo, oracle, dt, agree):
    """Gradients of the block-list forward (no counterpart in the reference, flex.jl:193-194): the pairs
    the forward used, and only those, carry gradient."""
    t, o = tylo, oracle
    rng = np.random.default_rng(11 + agree)
    B, H, Hkv, Sq, Sk, D = 2, 4, 2, 200, 260, 64
    TM, TN = 64, 32
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    docs = np.repeat(np.arange(8), 40)[:Sk + 5].astype(np.int32)
    keep = lambda q, kv: bool(q >= kv and docs[q] == docs[kv])
    (cnt, idx, full), bm = _bm_from_oracle(t, o, keep, Sq, Sk, TILE_M=TM, TILE_N=TN, input_pos=5)
    if not agree:
        cnt = cnt.copy(); full = full.copy()
        cnt[1] = max(cnt[1] - 1, 0)                 # a listed block dropped: its pairs get no gradient
        full[2, 0] = 1                              # a partial block marked full: the mask mod is skipped there
        bm = t.BlockMask(torch.from_numpy(cnt).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(full).cuda(), TM, TN)
    mask = t.CausalMask() & t.DocumentMask(torch.from_numpy(docs).cuda())
    omask = o.MaskSpec(causal=True, doc_q=docs)
    kw = dict(mask_mod=mask, score_mod=t.SoftCapScore(25.0), block_mask=bm, input_pos=5)
    okw = dict(TILE_M=TM, TILE_N=TN, mask=omask, score=o.ScoreSpec([("softcap", 25.0)]), input_pos=5)
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    check(O, o.flex_block_mask_ref(Q64, K64, V64, cnt, idx, full, **okw), dt, "block walk fwd")
    dO, dO64 = draw(rng, tuple(O.shape), dt)
    dQ, dK, dV = t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, **kw)
    rQ, rK, rV, _ = o.flex_block_mask_bwd_ref(dO64, Q64, K64, V64, cnt, idx, full, **okw)
    if agree:
        aQ, aK, aV, _ = o.flex_bwd_ref(dO64, Q64, K64, V64, score=okw["score"], mask=omask, input_pos=5)
        assert np.allclose(rQ, aQ) and np.allclose(rK, aK) and np.allclose(rV, aV)
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"block walk {name}", scale_hint=float(np.abs(ref).max()))
    assert t.device_status() == 0
