"""CPU: host-side mirror of the Tylo API — mods, host evaluators, descriptors, buffers."""
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
