"""GPU parity: OrMask trees (mods.jl:164-167) beyond prefix_lm — passed to the library in disjunctive
normal form (up to four conjunctions), forward and backward, against the oracle's OR of dense masks."""
import numpy as np
import pytest
import torch

from gpu_util import check, draw

pytestmark = pytest.mark.gpu

S = 300
DOCS = np.repeat(np.arange(6), 55)[:S + 9].astype(np.int32)


def _cases(t, o):
    dm = t.DocumentMask(torch.from_numpy(DOCS).cuda())
    return {
        "window | global prefix": ((t.CausalMask() & t.SlidingWindowMask(40)) | t.PrefixMask(24),
                                   o.MaskAny(o.MaskSpec(causal=True, window=40), o.MaskSpec(prefix=24))),
        "document | prefix": (dm | t.PrefixMask(16), o.MaskAny(o.MaskSpec(doc_q=DOCS), o.MaskSpec(prefix=16))),
        "(window | prefix) & document": ((t.SlidingWindowMask(30) | t.PrefixMask(70)) & dm,
                                         o.MaskAny(o.MaskSpec(window=30, doc_q=DOCS), o.MaskSpec(prefix=70, doc_q=DOCS))),
        "four conjunctions": ((t.SlidingWindowMask(10) | t.PrefixMask(8)) & (t.CausalMask() | dm),
                              o.MaskAny(o.MaskSpec(window=10, causal=True), o.MaskSpec(window=10, doc_q=DOCS),
                                        o.MaskSpec(prefix=8, causal=True), o.MaskSpec(prefix=8, doc_q=DOCS))),
        "prefix_lm | window-less document": (t.prefix_lm(50) | dm,
                                             o.MaskAny(o.MaskSpec(prefix_or_causal=50), o.MaskSpec(doc_q=DOCS))),
    }


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("case", ["window | global prefix", "document | prefix", "(window | prefix) & document",
                                  "four conjunctions", "prefix_lm | window-less document"])
def test_or_mask_fwd_bwd(tylo, oracle, case, dt):
    t, o = tylo, oracle
    mask, omask = _cases(t, o)[case]
    rng = np.random.default_rng(len(case))
    B, H, Hkv, D = 2, 4, 2, 64
    Q, Q64 = draw(rng, (B, H, S, D), dt); K, K64 = draw(rng, (B, Hkv, S, D), dt); V, V64 = draw(rng, (B, Hkv, S, D), dt)
    kw = dict(mask_mod=mask, score_mod=t.SoftCapScore(20.0), input_pos=9)
    okw = dict(mask=omask, score=o.ScoreSpec([("softcap", 20.0)]), input_pos=9)
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    O = t.flex_attention(Q, K, V, checkpoints=cp, **kw)
    check(O, o.flex_ref(Q64, K64, V64, **okw), dt, f"{case} fwd")
    dO, dO64 = draw(rng, tuple(O.shape), dt)
    dQ, dK, dV = t.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, **kw)
    rQ, rK, rV, _ = o.flex_bwd_ref(dO64, Q64, K64, V64, **okw)
    for got, ref, name in ((dQ, rQ, "dQ"), (dK, rK, "dK"), (dV, rV, "dV")):
        check(got, ref, dt, f"{case} {name}", scale_hint=float(np.abs(ref).max()))
    assert t.device_status() == 0


def test_too_many_conjunctions_are_refused(tylo):
    t = tylo
    Q = torch.randn(1, 1, 64, 64, device="cuda").bfloat16()
    m = t.PrefixMask(1) | t.PrefixMask(2) | t.PrefixMask(3) | t.PrefixMask(4) | t.SlidingWindowMask(5)
    with pytest.raises(t.TyloError):
        t.flex_attention(Q, Q, Q, mask_mod=m)
