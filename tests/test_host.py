"""CPU: host-side mirror of the Tylo API — mods, host evaluators, descriptors, buffers."""
import numpy as np
import pytest
import torch


def test_hmask_hscore_match_reference_semantics(tylo):
    t = tylo
    docs = torch.tensor([1] * 5 + [2] * 7, dtype=torch.int32)
    dm = t.DocumentMask(docs)
    assert all(t.hmask(dm, q, kv) == (docs[q] == docs[kv]) for q in range(12) for kv in range(12))  # test/flex.jl:240-242
    slopes = torch.tensor([2.0 ** -(i + 1) for i in range(4)])
    assert t.hscore(t.AliBiScore(slopes), 0.5, 7, 3, h=2) == pytest.approx(0.5 + float(slopes[1]) * 4)  # :244-246
    cm = t.CausalMask() & dm
    assert t.hmask(cm, 6, 5) == bool(docs[6] == docs[5]) and not t.hmask(cm, 5, 6)  # :253-255
    sw = t.SlidingWindowMask(37)
    assert t.hmask(sw, 40, 3) and not t.hmask(sw, 41, 3) and not t.hmask(sw, 2, 3)
    assert t.hmask(t.prefix_lm(50), 3, 40) and not t.hmask(t.prefix_lm(50), 3, 60)
    comp = t.SoftCapScore(5.0) @ t.AliBiScore(slopes)      # softcap ∘ alibi: alibi first
    import math
    assert t.hscore(comp, 0.25, 5, 3, h=1) == pytest.approx(5 * math.tanh((0.25 + 0.5 * 2) / 5))


def test_mask_descriptor_mapping(tylo):
    t = tylo
    keep = []
    d = t._mask_desc(t.CausalMask() & t.SlidingWindowMask(1024), keep)
    assert d.flags == t.MASK_CAUSAL | t.MASK_SLIDING and d.window == 1024
    d = t._mask_desc(t.prefix_lm(50), keep)
    assert d.flags == t.MASK_PREFIX_LM and d.prefix_len == 50
    d = t._mask_desc(t.CausalMask() & t.PrefixMask(100), keep)
    assert d.flags == t.MASK_CAUSAL | t.MASK_PREFIX and d.prefix_len == 100
    d = t._mask_desc(None, keep)
    assert d.flags == 0
    # an OrMask beyond prefix_lm becomes a chain of conjunctions (mods.jl:164-167)
    d = t._mask_desc(t.PrefixMask(3) | (t.CausalMask() & t.PrefixMask(4)), keep)
    assert d.flags == t.MASK_PREFIX and d.prefix_len == 3 and d.or_next
    nxt = t._MaskDesc.from_address(d.or_next)
    assert nxt.flags == t.MASK_CAUSAL | t.MASK_PREFIX and nxt.prefix_len == 4 and not nxt.or_next
    with pytest.raises(t.TyloError):
        t._mask_desc(t.PrefixMask(1) | t.PrefixMask(2) | t.PrefixMask(3) | t.PrefixMask(4) | t.PrefixMask(5), keep)


def test_score_descriptor_order(tylo, monkeypatch):
    t = tylo
    monkeypatch.setattr(t, "_dense", lambda *a: None)   # descriptors normally demand device arrays
    slopes = torch.zeros(4)
    keep = []
    d = t._score_desc(t.SoftCapScore(5.0) @ t.AliBiScore(slopes), None, keep)
    assert d.flags == t.SCORE_ALIBI | t.SCORE_SOFTCAP
    d = t._score_desc(t.AliBiScore(slopes) @ t.SoftCapScore(5.0), None, keep)
    assert d.flags == t.SCORE_ALIBI | t.SCORE_SOFTCAP | t.SCORE_SOFTCAP_FIRST
    d = t._score_desc(t.NoOpScore(), None, keep)
    assert d.flags == 0
    sh = t.grad_shadow(t.SoftCapScore(5.0) @ t.AliBiScore(torch.ones(4)))
    assert isinstance(sh, t.ComposeScore) and float(sh.a.slopes.sum()) == 0.0


def test_duplicated_and_cpu_rejection(tylo):
    x = torch.ones(4, 8)
    d = tylo.Duplicated(x)
    assert tylo.primal(d) is x and tylo.shadow(d).shape == x.shape and tylo.primal(x) is x
    with pytest.raises(ValueError):          # device arrays only: there is no CPU path
        tylo.softmax(x)


def test_host_tensors_are_refused_before_any_launch(tylo):
    """A host array must never reach a kernel as an address (the Julia wrapper's `devptr` refuses it the
    same way): the pointer helper itself raises, as do the block-list and mod descriptors."""
    t = tylo
    with pytest.raises(ValueError):
        t._p(torch.zeros(4))
    assert t._p(None) is None
    bm = t.build_block_mask(lambda q, kv: q >= kv, 128, 128, device="cpu")
    with pytest.raises(ValueError):
        t._check_block_mask(bm, 128)
    with pytest.raises(ValueError):
        t._mask_desc(t.DocumentMask(torch.zeros(8, dtype=torch.int32)), [])


class _RbfOp:
    """Pair op of the kind test/flex.jl:46-60 uses: two radial basis features of a squared distance."""

    def __init__(self, c):
        self.c = c

    def pair_feature(self, qv, kv):
        d2 = sum((a - b) ** 2 for a, b in zip(qv, kv))
        e = torch.exp(-self.c * d2) if isinstance(d2, torch.Tensor) else __import__("math").exp(-self.c * d2)
        return (e, d2 * e)

    def grad_pair_feature(self, qv, kv, dphi):
        d2 = sum((a - b) ** 2 for a, b in zip(qv, kv))
        e = torch.exp(-self.c * d2)
        g = dphi[0] * (-self.c) * e + dphi[1] * (e - self.c * d2 * e)     # d/d(d2)
        dq = tuple(g * 2 * (a - b) for a, b in zip(qv, kv))
        dk = tuple(-x for x in dq)
        return dq, dk


def _pair_mod(t, B=2, Sq=5, Sk=7, F=3, PD=2, H=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    return t.PairFeatureScore(_RbfOp(0.7), torch.randn(B, Sq, F, generator=g), torch.randn(B, Sk, F, generator=g),
                              torch.randn(PD, H, generator=g))


def test_pair_feature_table_matches_host_evaluation(tylo):
    """The bias table a PairFeatureScore is lowered to equals its scalar host evaluation (pair.jl:90-96)
    pair by pair."""
    t = tylo
    m = _pair_mod(t)
    tab = m.bias_table()
    assert tab.shape == (2, 3, 5, 7)
    for b in range(2):
        for h in range(3):
            for q in range(5):
                for kv in range(7):
                    assert float(tab[b, h, q, kv]) == pytest.approx(t.hscore(m, 0.0, q, kv, b=b + 1, h=h + 1), abs=1e-5)
    low = t._lower_pairs(t.SoftCapScore(5.0) @ m)
    assert isinstance(low, t.ComposeScore) and isinstance(low.a, t.BiasScore) and isinstance(low.b, t.SoftCapScore)


def test_pair_feature_gradients_fold_back(tylo):
    """Projection and feature gradients recovered from a bias-table gradient equal autograd through the
    table (pair.jl:127-157 semantics)."""
    t = tylo
    m = _pair_mod(t, seed=1)
    qf, kf, pr = (x.clone().requires_grad_(True) for x in (m.q_features, m.k_features, m.pair_proj))
    tab = t.PairFeatureScore(m.op, qf, kf, pr).bias_table()
    d_bias = torch.randn(tab.shape, generator=torch.Generator().manual_seed(2))
    (tab * d_bias).sum().backward()
    sh = t.grad_shadow(m, feature_grads=True)
    m.fold_grads_(sh, d_bias)
    assert torch.allclose(sh.pair_proj, pr.grad, atol=1e-4)
    assert torch.allclose(sh.q_features, qf.grad, atol=1e-4) and torch.allclose(sh.k_features, kf.grad, atol=1e-4)
    sh2 = t.grad_shadow(m)
    assert sh2.q_features is None and sh2.k_features is None
    m.fold_grads_(sh2, d_bias)
    assert torch.allclose(sh2.pair_proj, pr.grad, atol=1e-4)


def test_score_tangent_is_generic_over_fields(tylo):
    """Every array field of a shadow is its own tangent, nested mods recurse, plain fields have none
    (ext/ChainRulesCoreExt.jl:110-113): a bias table inside a composition keeps its gradient."""
    t = tylo
    sh = t.grad_shadow(t.SoftCapScore(5.0) @ t.BiasScore(torch.ones(1, 1, 4, 4)))
    tan = t.score_tangent(sh)
    assert set(tan) == {"a", "b"} and tan["a"]["bias"] is sh.a.bias and tan["b"]["cap"] is None
    tan = t.score_tangent(t.grad_shadow(t.AliBiScore(torch.ones(3))))
    assert float(tan["slopes"].sum()) == 0.0
    assert t.score_tangent(t.grad_shadow(_pair_mod(t)))["pair_proj"].shape == (2, 3)


def test_adapt_rebuilds_mods(tylo):
    """adapt(to, mod) maps every array field and keeps the rest (mods.jl:41-44)."""
    t = tylo
    docs = torch.arange(6, dtype=torch.int32)
    m = t.adapt(lambda x: x.to(torch.int64), t.CausalMask() & t.DocumentMask(docs))
    assert isinstance(m, t.AndMask) and m.b.doc_q.dtype == torch.int64 and t.hmask(m, 3, 3) and not t.hmask(m, 3, 2)
    s = t.adapt(lambda x: x * 2, t.SoftCapScore(5.0) @ t.AliBiScore(torch.ones(2)))
    assert s.b.cap == 5.0 and float(s.a.slopes[0]) == 2.0


def test_tensorcore_keyword_maps_to_the_dtype_code(tylo):
    """`tensorcore = TFloat32` asks for TF32 operands on Float32 storage only (utils.jl:43-44: the reference's default);
    16-bit storage keeps its own code, None keeps true fp32, anything else is refused."""
    t = tylo
    f32, bf = torch.empty(1, dtype=torch.float32), torch.empty(1, dtype=torch.bfloat16)
    assert t._fwd_dtype(f32, None) == t.F32
    assert t._fwd_dtype(f32, t.TFloat32) == t.F32_TF32 == 3
    assert t._fwd_dtype(f32, "tf32") == t.F32_TF32
    assert t._fwd_dtype(bf, t.TFloat32) == t.BF16
    assert t._fwd_dtype(f32, "Float32") == t.F32

    class TFloat32:          # a type of that name from another package
        pass
    assert t._fwd_dtype(f32, TFloat32) == t.F32_TF32
    with pytest.raises(ValueError):
        t._fwd_dtype(f32, "fp8")


def test_bench_block_list_matches_the_oracle_builder(oracle):
    """The closed-form block list the bench builds for `causal & window & document` equals the oracle's pairwise
    builder (mods.jl:436-476) on seeded document tables, and the union / intersection over batch entries."""
    import importlib.util
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("tylo_bench", Path(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)
    rng = np.random.default_rng(1)
    S, W, T = 384, 150, 64
    tabs = []
    for _ in range(2):
        cuts = np.sort(rng.choice(np.arange(1, S), size=3, replace=False))
        tabs.append(np.searchsorted(cuts, np.arange(S), side="right").astype(np.int32))
    keep = lambda tab: (lambda q, kv: bool(q >= kv and q - kv <= W and tab[q] == tab[kv]))
    for tab in tabs:
        cnt, idx, full = bench.band_block_list(tab[None], S, W, T)
        rc, ri, rf = oracle.build_block_mask_ref(keep(tab), S, S, TILE_M=T, TILE_N=T)
        assert np.array_equal(cnt, rc)
        for i in range(S // T):
            assert np.array_equal(idx[i, :cnt[i]], ri[i, :rc[i]]) and np.array_equal(full[i, :cnt[i]], rf[i, :rc[i]])
    # two batch entries: listed = in either, full = in both
    cnt, idx, full = bench.band_block_list(np.stack(tabs), S, W, T)
    any_keep = lambda q, kv: keep(tabs[0])(q, kv) or keep(tabs[1])(q, kv)
    rc, ri, _ = oracle.build_block_mask_ref(any_keep, S, S, TILE_M=T, TILE_N=T)
    assert np.array_equal(cnt, rc) and all(np.array_equal(idx[i, :cnt[i]], ri[i, :rc[i]]) for i in range(S // T))
    singles = [bench.band_block_list(tab[None], S, W, T) for tab in tabs]
    for i in range(S // T):
        for n in range(cnt[i]):
            j = idx[i, n]
            both = all(any(sj == j and sf for sj, sf in zip(si[i, :sc[i]], sfl[i, :sc[i]])) for sc, si, sfl in singles)
            assert bool(full[i, n]) == both
