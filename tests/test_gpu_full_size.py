"""GPU parity at the benchmark configurations' own sizes.

The kernels run the whole problem; the float64 oracle checks a sample of it that is complete in itself
(every output compared is computed by the oracle from all the inputs it depends on):

  config 3  causal GQA prefill, B 4, S 4096, Hq 32 / Hkv 8, D 128: four (batch, kv-head) groups, forward,
            statistics and all three gradients (a group's dK/dV sum its four query heads).
  config 4  flex, B 2, S 8192, H 16, D 128, causal & window 1024 & 7 seeded document cuts, soft cap 50:
            four (batch, head) slices, three query bands each (start, a band with a document cut in it, end);
            a band's queries with every key they can see give O and dQ, the band's middle keys get dK/dV.
  config 5a decode, all 64 sequences with lengths in [1024, 32768].
  config 5b decode, one sequence of 1,048,576 keys (the wide-merge path), every head.

Inputs come from the counter-based generator of the package (`synth.py`), rounded to bf16; the oracle
sees the rounded values.  Tolerances are the contract's: max-abs 2e-2, mean-abs 2e-3 for outputs; a
gradient is held to the same numbers times max(1, P / 4), P the power of two at or above max|ref| (bf16
results in [P/2, P) are spaced P * 2^-8 apart, so rounding alone reaches P * 2^-9; see gpu_util.py).
Measured errors are printed (run with -s to see them).
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import back, check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _synth():
    if "tylo_b200_synth" not in sys.modules:
        p = Path(__file__).resolve().parent.parent / "tylo.jl_b200" / "synth.py"
        spec = importlib.util.spec_from_file_location("tylo_b200_synth", p)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["tylo_b200_synth"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["tylo_b200_synth"]


def _report(what, got, ref):
    err = np.abs(back(got) - ref)
    print(f"PARITY {what}: max_abs {err.max():.3e} mean_abs {err.mean():.3e} max_ref {np.abs(ref).max():.3e}")


def _grad_check(got, ref, what):
    _report(what, got, ref)
    check(got, ref, "bf16", what, scale_hint=float(np.abs(ref).max()))


def test_generator_is_identical_on_cpu_and_gpu():
    s = _synth()
    g = s.normal_cuda(2, 1, (3, 5000), BF, start=12345)
    c = s.rounded_numpy(2, 1, 12345, 12345 + 15000, BF).reshape(3, 5000)
    assert np.array_equal(back(g), c)
    gi = s.integers_cuda(4, 9, 64, 1024, 32768).cpu().numpy()
    assert np.array_equal(gi, s.integers_numpy(4, 9, 0, 64, 1024, 32768))


def test_config3_full_size(tylo, oracle):
    s = _synth()
    B, H, Hkv, S, D, seed = 4, 32, 8, 4096, 128, 2
    G = H // Hkv
    Q = s.normal_cuda(seed, 0, (B, H, S, D), BF); K = s.normal_cuda(seed, 1, (B, Hkv, S, D), BF)
    V = s.normal_cuda(seed, 2, (B, Hkv, S, D), BF); dO = s.normal_cuda(seed, 3, (B, H, S, D), BF)
    cp = tylo.allocate_checkpoints_attention(Q, K, V)
    O = tylo.attention(Q, K, V, causal=True, checkpoints=cp)
    dQ, dK, dV = tylo.grad_attention(dO, Q, K, V, O, checkpoints=cp, causal=True)
    assert tylo.device_status() == 0
    for b, hk in ((0, 0), (1, 3), (2, 5), (3, 7)):
        q0 = ((b * H + hk * G) * S) * D
        k0 = ((b * Hkv + hk) * S) * D
        Q64 = s.rounded_numpy(seed, 0, q0, q0 + G * S * D, BF).reshape(1, G, S, D)
        K64 = s.rounded_numpy(seed, 1, k0, k0 + S * D, BF).reshape(1, 1, S, D)
        V64 = s.rounded_numpy(seed, 2, k0, k0 + S * D, BF).reshape(1, 1, S, D)
        dO64 = s.rounded_numpy(seed, 3, q0, q0 + G * S * D, BF).reshape(1, G, S, D)
        hs = slice(hk * G, (hk + 1) * G)
        Oref, Mref, Lref = oracle.flex_ref(Q64, K64, V64, mask=oracle.MaskSpec(causal=True), return_stats=True)
        _report(f"C3 O (b{b},kv{hk})", O[b:b + 1, hs], Oref)
        check(O[b:b + 1, hs], Oref, "bf16", "config 3 O")
        lse = back(cp.M[b:b + 1, hs]) * np.log(2.0) + np.log(back(cp.L[b:b + 1, hs]))
        np.testing.assert_allclose(lse, Mref + np.log(Lref), rtol=0, atol=2e-2)
        rQ, rK, rV = oracle.attn_bwd_ref(dO64, Q64, K64, V64, causal=True)
        _grad_check(dQ[b:b + 1, hs], rQ, f"C3 dQ (b{b},kv{hk})")
        _grad_check(dK[b:b + 1, hk:hk + 1], rK, f"C3 dK (b{b},kv{hk})")
        _grad_check(dV[b:b + 1, hk:hk + 1], rV, f"C3 dV (b{b},kv{hk})")


def _documents(B, S, ndocs, seed):
    rng = np.random.default_rng(seed)
    tab = np.zeros((B, S), dtype=np.int32)
    cuts = []
    for b in range(B):
        c = np.sort(rng.choice(np.arange(1, S), size=ndocs - 1, replace=False))
        tab[b] = np.searchsorted(c, np.arange(S), side="right")
        cuts.append(c)
    return tab, cuts


def test_config4_full_size(tylo, oracle):
    s = _synth()
    B, H, S, D, W, cap, seed = 2, 16, 8192, 128, 1024, 50.0, 3
    Q = s.normal_cuda(seed, 0, (B, H, S, D), BF); K = s.normal_cuda(seed, 1, (B, H, S, D), BF)
    V = s.normal_cuda(seed, 2, (B, H, S, D), BF); dO = s.normal_cuda(seed, 3, (B, H, S, D), BF)
    tab, cuts = _documents(B, S, 8, seed)
    docs = torch.from_numpy(tab).cuda()
    mask = tylo.CausalMask() & tylo.SlidingWindowMask(W) & tylo.DocumentMask(docs)
    score = tylo.SoftCapScore(cap)
    cp = tylo.allocate_checkpoints_flex_attention(Q, K, V)
    O = tylo.flex_attention(Q, K, V, score_mod=score, mask_mod=mask, checkpoints=cp)
    dQ, dK, dV = tylo.grad_flex_attention(dO, Q, K, V, O, checkpoints=cp, score_mod=score, mask_mod=mask)
    assert tylo.device_status() == 0
    ospec = oracle.ScoreSpec([("softcap", cap)])
    for b, h in ((0, 0), (0, 9), (1, 5), (1, 15)):
        mid = int(cuts[b][3]) // 128 * 128                       # a band with a document boundary inside
        for k0 in (0, min(mid, S - 1536), S - 1536):
            klo, hi = max(0, k0 - W), min(S, k0 + 1536)
            base = ((b * H + h) * S) * D
            sl = lambda tid, lo, n: s.rounded_numpy(seed, tid, base + lo * D, base + (lo + n) * D, BF).reshape(1, 1, n, D)
            nq, nk = hi - k0, hi - klo
            Q64, dO64 = sl(0, k0, nq), sl(3, k0, nq)
            K64, V64 = sl(1, klo, nk), sl(2, klo, nk)
            m = oracle.MaskSpec(causal=True, window=W, doc_q=tab[b][klo:], doc_kv=tab[b][klo:])
            kw = dict(score=ospec, mask=m, input_pos=k0 - klo)
            Oref = oracle.flex_ref(Q64, K64, V64, **kw)
            got = O[b:b + 1, h:h + 1, k0:hi]
            _report(f"C4 O (b{b},h{h},q{k0})", got, Oref)
            check(got, Oref, "bf16", "config 4 O")
            rQ, rK, rV, _ = oracle.flex_bwd_ref(dO64, Q64, K64, V64, **kw)
            _grad_check(dQ[b:b + 1, h:h + 1, k0:hi], rQ, f"C4 dQ (b{b},h{h},q{k0})")
            # keys [k0, k0 + 512): every query that can see them (q <= kv + W < k0 + 1536) is in the band
            ks = slice(k0 - klo, k0 - klo + 512)
            _grad_check(dK[b:b + 1, h:h + 1, k0:k0 + 512], rK[:, :, ks], f"C4 dK (b{b},h{h},k{k0})")
            _grad_check(dV[b:b + 1, h:h + 1, k0:k0 + 512], rV[:, :, ks], f"C4 dV (b{b},h{h},k{k0})")


def test_config5a_full_size(tylo, oracle):
    s = _synth()
    B, H, Hkv, D, Smax, seed = 64, 64, 8, 128, 32768, 4
    Q = s.normal_cuda(seed, 0, (B, H, D), BF)
    K = s.normal_cuda(seed, 1, (B, Hkv, Smax, D), BF); V = s.normal_cuda(seed, 2, (B, Hkv, Smax, D), BF)
    lengths = s.integers_numpy(seed, 3, 0, B, 1024, Smax)
    ln = torch.from_numpy(lengths.astype(np.int32)).cuda()
    O = tylo.decode_attention_(torch.empty_like(Q), Q, K, V, lengths=ln, n_splits=None)
    worst = 0.0
    for b in range(B):
        n = int(lengths[b])
        ref = oracle.decode_reference(back(Q[b:b + 1]), back(K[b:b + 1, :, :n]), back(V[b:b + 1, :, :n]), [n])
        check(O[b:b + 1], ref, "bf16", f"config 5a sequence {b} (length {n})")
        worst = max(worst, float(np.abs(back(O[b:b + 1]) - ref).max()))
    print(f"PARITY C5a decode, 64 sequences: worst max_abs {worst:.3e}")
    # the generator gives the CPU the same keys without a copy back
    b, hk, n = 7, 3, int(lengths[7])
    a0 = ((b * Hkv + hk) * Smax) * D
    assert np.array_equal(back(K[b, hk, :n]), s.rounded_numpy(seed, 1, a0, a0 + n * D, BF).reshape(n, D))


def test_config5b_full_size(tylo, oracle):
    s = _synth()
    H, Hkv, D, S, seed = 64, 8, 128, 1 << 20, 4
    G = H // Hkv
    Q = s.normal_cuda(seed, 10, (1, H, D), BF)
    K = s.normal_cuda(seed, 11, (1, Hkv, S, D), BF); V = s.normal_cuda(seed, 12, (1, Hkv, S, D), BF)
    ln = torch.tensor([S], dtype=torch.int32, device="cuda")
    n_splits = tylo.decode_suggest_splits(S, Hkv, 1)
    assert n_splits >= 64                                   # the many-split path with the wide merge
    O = tylo.decode_attention_(torch.empty_like(Q), Q, K, V, lengths=ln, n_splits=n_splits)
    worst = 0.0
    for hk in range(Hkv):
        hs = slice(hk * G, (hk + 1) * G)
        ref = oracle.decode_reference(back(Q[:, hs]), back(K[:, hk:hk + 1]), back(V[:, hk:hk + 1]), [S])
        check(O[:, hs], ref, "bf16", f"config 5b kv head {hk}")
        worst = max(worst, float(np.abs(back(O[:, hs]) - ref).max()))
    print(f"PARITY C5b decode, 1,048,576 keys, {n_splits} splits: worst max_abs {worst:.3e}")
    # fewer, longer splits must give the same answer (test/decode.jl:114-124)
    O8 = tylo.decode_attention_(torch.empty_like(Q), Q, K, V, lengths=ln, n_splits=8)
    assert torch.allclose(O8.float(), O.float(), atol=8e-3, rtol=1e-3)
