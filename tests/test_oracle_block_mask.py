"""CPU: the oracle's block-mask builder and block walk (mods.jl:448-476, flex.jl:107-182) and the host
builder of the package against them — the reference's own two cases (test/flex.jl:258-280) included."""
import numpy as np
import pytest


def _inputs(rng, Sq, Sk, H=2, D=16):
    return rng.standard_normal((1, H, Sq, D)), rng.standard_normal((1, H, Sk, D)), rng.standard_normal((1, H, Sk, D))


def test_builder_marks_any_and_all(oracle):
    o = oracle
    cnt, idx, full = o.build_block_mask_ref(lambda q, kv: q >= kv, 256, 256)
    assert cnt.tolist() == [1, 2, 3, 4]
    for i in range(4):
        assert idx[i, :cnt[i]].tolist() == list(range(i + 1))
        assert full[i, :cnt[i]].tolist() == [1] * i + [0]        # diagonal blocks are partial
    # blocks touching the end of Q or K are never full (mods.jl:468-470)
    cnt, idx, full = o.build_block_mask_ref(lambda q, kv: True, 100, 150)
    assert cnt.tolist() == [3, 3]
    assert full[0, :3].tolist() == [1, 1, 0] and full[1, :3].tolist() == [0, 0, 0]
    # input_pos shifts the query positions the predicate sees
    cnt, _, _ = o.build_block_mask_ref(lambda q, kv: q >= kv, 64, 256, input_pos=128)
    assert cnt.tolist() == [3]


def test_reference_cases_agree_with_flex_ref(oracle):
    o = oracle
    rng = np.random.default_rng(1)
    docs = np.concatenate([np.full(70, 1), np.full(80, 2), np.full(42, 3)]).astype(np.int32)
    Q, K, V = _inputs(rng, 192, 192)
    bm = o.build_block_mask_ref(lambda q, kv: docs[q] == docs[kv], 192, 192)
    got = o.flex_block_mask_ref(Q, K, V, *bm, mask=o.MaskSpec(doc_q=docs))
    assert np.allclose(got, o.flex_ref(Q, K, V, mask=o.MaskSpec(doc_q=docs)), atol=1e-12)
    Q, K, V = _inputs(rng, 100, 150)
    bm = o.build_block_mask_ref(lambda q, kv: q >= kv, 100, 150)
    got = o.flex_block_mask_ref(Q, K, V, *bm, mask=o.MaskSpec(causal=True))
    assert np.allclose(got, o.flex_ref(Q, K, V, mask=o.MaskSpec(causal=True)), atol=1e-12)


def test_unlisted_blocks_contribute_nothing_and_full_skips_the_mask(oracle):
    o = oracle
    rng = np.random.default_rng(2)
    Q, K, V = _inputs(rng, 128, 128)
    cnt = np.array([1, 1], np.int32); idx = np.array([[1, 0], [0, 0]], np.int32); full = np.array([[1, 0], [0, 0]], np.int32)
    got = o.flex_block_mask_ref(Q, K, V, cnt, idx, full, mask=o.MaskSpec(causal=True))
    keep = np.zeros((128, 128), bool)
    keep[:64, 64:] = True                                   # full: the causal mask is not applied
    keep[64:, :64] = True                                   # partial, and causal keeps all of it
    assert np.allclose(got, o.flex_ref(Q, K, V, keep_dense=keep), atol=1e-12)


@pytest.mark.parametrize("tiles", [(64, 64), (32, 96)])
def test_package_builder_matches_the_oracle(tylo, oracle, tiles):
    TM, TN = tiles
    docs = np.repeat(np.arange(7), 37)[:230].astype(np.int32)
    preds = [lambda q, kv: q >= kv, lambda q, kv: (q >= kv) & (q <= kv + 50),
             lambda q, kv: bool(docs[min(q, 229)] == docs[kv])]          # the last one only works pair by pair
    for keep in preds:
        ref = oracle.build_block_mask_ref(keep, 200, 230, TILE_M=TM, TILE_N=TN, input_pos=3)
        bm = tylo.build_block_mask(keep, 200, 230, TILE_M=TM, TILE_N=TN, input_pos=3, device="cpu")
        assert (bm.TILE_M, bm.TILE_N) == (TM, TN)
        for got, want in zip((bm.count, bm.idx, bm.full), ref):
            assert np.array_equal(got.numpy(), want)
