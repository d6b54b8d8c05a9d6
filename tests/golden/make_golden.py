"""Generates tests/golden/*.npz: small known-answer vectors for the CPU oracle.

The reference (Tylo.jl) ships no golden vectors and cannot be executed next to this
repository (it needs Julia, cuTile.jl and a GPU), so these vectors come from a second,
independent restatement: scalar pure-Python loops written straight from the formulas in
the reference's test files (test/attention.jl:9-55, test/flex.jl:8-35,75-114,
test/decode.jl:15-36, test/softmax.jl:10-13, test/norm.jl:8-20,78-102) using `math` only —
no NumPy linear algebra, no broadcasting — so that an indexing or axis mistake in the
vectorised oracle cannot hide.  Run:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import math
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def rnd(rng, *shape):
    return rng.standard_normal(shape)


def attn_loops(Q, K, V, *, mask=None, score=None, input_pos=0):
    """Q[b][h][m][d] ... scalar loops; returns O and (M, L) natural-base stats."""
    B, H, Sq, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    g = H // Hkv
    scale = 1.0 / math.sqrt(Dk)
    O = np.zeros((B, H, Sq, Dv))
    P = np.zeros((B, H, Sq, Sk))
    S0 = np.zeros((B, H, Sq, Sk))
    for b in range(B):
        for h in range(H):
            hk = h // g
            for m in range(Sq):
                row = []
                for n in range(Sk):
                    s = 0.0
                    for d in range(Dk):
                        s += K[b, hk, n, d] * Q[b, h, m, d]
                    s *= scale
                    S0[b, h, m, n] = s
                    qpos, kvpos = m + input_pos, n
                    if score is not None:
                        s = score(s, b + 1, h + 1, qpos, kvpos)
                    if mask is not None and not mask(b + 1, h + 1, qpos, kvpos):
                        s = -math.inf
                    row.append(s)
                mx = max(row)
                if not math.isfinite(mx):
                    continue
                e = [math.exp(x - mx) if math.isfinite(x) else 0.0 for x in row]
                tot = sum(e)
                for n in range(Sk):
                    P[b, h, m, n] = e[n] / tot
                for d in range(Dv):
                    acc = 0.0
                    for n in range(Sk):
                        acc += V[b, hk, n, d] * P[b, h, m, n]
                    O[b, h, m, d] = acc
    return O, P, S0


def attn_bwd_loops(dO, Q, K, V, *, mask=None, score=None, dscore=None, input_pos=0):
    B, H, Sq, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    g = H // Hkv
    scale = 1.0 / math.sqrt(Dk)
    _, P, S0 = attn_loops(Q, K, V, mask=mask, score=score, input_pos=input_pos)
    dQ = np.zeros_like(Q); dK = np.zeros_like(K); dV = np.zeros_like(V)
    for b in range(B):
        for h in range(H):
            hk = h // g
            for m in range(Sq):
                dP = [sum(V[b, hk, n, d] * dO[b, h, m, d] for d in range(Dv)) for n in range(Sk)]
                dot = sum(P[b, h, m, n] * dP[n] for n in range(Sk))
                for n in range(Sk):
                    ds = P[b, h, m, n] * (dP[n] - dot)
                    if dscore is not None:
                        ds = dscore(S0[b, h, m, n], b + 1, h + 1, m + input_pos, n, ds)
                    for d in range(Dk):
                        dQ[b, h, m, d] += K[b, hk, n, d] * ds * scale
                        dK[b, hk, n, d] += Q[b, h, m, d] * ds * scale
                    for d in range(Dv):
                        dV[b, hk, n, d] += dO[b, h, m, d] * P[b, h, m, n]
    return dQ, dK, dV


def decode_loops(Q, K, V, lengths):
    B, H, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    G = H // Hkv
    scale = 1.0 / math.sqrt(Dk)
    O = np.zeros((B, H, Dv))
    for b in range(B):
        L = int(lengths[b])
        if L == 0:
            continue
        for h in range(H):
            hk = h // G
            sc = [scale * sum(Q[b, h, d] * K[b, hk, n, d] for d in range(Dk)) for n in range(L)]
            mx = max(sc)
            w = [math.exp(s - mx) for s in sc]
            tot = sum(w)
            for d in range(Dv):
                O[b, h, d] = sum(w[n] / tot * V[b, hk, n, d] for n in range(L))
    return O


def main():
    rng = np.random.default_rng(20240611)
    out = {}

    # --- attention / flex ---------------------------------------------------------------------
    Q = rnd(rng, 2, 4, 5, 4); K = rnd(rng, 2, 2, 7, 4); V = rnd(rng, 2, 2, 7, 3); dO = rnd(rng, 2, 4, 5, 3)
    out.update(attn_Q=Q, attn_K=K, attn_V=V, attn_dO=dO)
    for name, mask in (("full", None), ("causal", lambda b, h, q, kv: q >= kv)):
        O, _, _ = attn_loops(Q, K, V, mask=mask)
        dQ, dK, dV = attn_bwd_loops(dO, Q, K, V, mask=mask)
        out.update({f"attn_{name}_O": O, f"attn_{name}_dQ": dQ, f"attn_{name}_dK": dK, f"attn_{name}_dV": dV})

    docs = np.array([0, 0, 0, 1, 1, 2, 2], dtype=np.int32)
    slopes = np.array([0.5, 0.25, 0.125, 0.0625])
    cap = 1.5
    mask = lambda b, h, q, kv: q >= kv and q <= kv + 2 and docs[q] == docs[kv]
    score = lambda s, b, h, q, kv: cap * math.tanh((s + slopes[h - 1] * (q - kv)) / cap)

    def dscore(s0, b, h, q, kv, ds):
        th = math.tanh((s0 + slopes[h - 1] * (q - kv)) / cap)
        return ds * (1 - th * th)

    O, _, _ = attn_loops(Q, K, V, mask=mask, score=score, input_pos=2)
    dQ, dK, dV = attn_bwd_loops(dO, Q, K, V, mask=mask, score=score, dscore=dscore, input_pos=2)
    out.update(flex_docs=docs, flex_slopes=slopes, flex_cap=np.array(cap), flex_window=np.array(2),
               flex_input_pos=np.array(2), flex_O=O, flex_dQ=dQ, flex_dK=dK, flex_dV=dV)

    # --- decode ---------------------------------------------------------------------------------
    Qd = rnd(rng, 3, 4, 4); Kd = rnd(rng, 3, 2, 9, 4); Vd = rnd(rng, 3, 2, 9, 3)
    lengths = np.array([9, 4, 0], dtype=np.int32)
    out.update(dec_Q=Qd, dec_K=Kd, dec_V=Vd, dec_lengths=lengths, dec_O=decode_loops(Qd, Kd, Vd, lengths))

    # --- softmax / norms ------------------------------------------------------------------------
    X = rnd(rng, 3, 6); dY = rnd(rng, 3, 6); W = 1 + 0.1 * rnd(rng, 6); Bv = 0.1 * rnd(rng, 6)
    eps, offset = 1e-5, 1.0
    Y = np.zeros_like(X); dXs = np.zeros_like(X)
    for n in range(3):
        mx = max(X[n]); e = [math.exp(v - mx) for v in X[n]]; tot = sum(e)
        for i in range(6):
            Y[n, i] = e[i] / tot
        dot = sum(Y[n, i] * dY[n, i] for i in range(6))
        for i in range(6):
            dXs[n, i] = Y[n, i] * (dY[n, i] - dot)
    rms = np.zeros_like(X); ln = np.zeros_like(X)
    rms_dX = np.zeros_like(X); rms_dW = np.zeros(6); ln_dX = np.zeros_like(X); ln_dW = np.zeros(6); ln_dB = np.zeros(6)
    for n in range(3):
        M = 6
        rstd = 1 / math.sqrt(sum(v * v for v in X[n]) / M + eps)
        dd = sum(dY[n, i] * (W[i] + offset) * X[n, i] for i in range(M)) / M
        mu = sum(X[n]) / M
        var = sum((v - mu) ** 2 for v in X[n]) / M
        rs2 = 1 / math.sqrt(var + eps)
        c1 = sum((X[n, i] - mu) * rs2 * W[i] * dY[n, i] for i in range(M)) / M
        c2 = sum(W[i] * dY[n, i] for i in range(M)) / M
        for i in range(M):
            rms[n, i] = X[n, i] * rstd * (W[i] + offset)
            rms_dX[n, i] = rstd * (dY[n, i] * (W[i] + offset) - rstd * rstd * dd * X[n, i])
            rms_dW[i] += dY[n, i] * X[n, i] * rstd
            xhat = (X[n, i] - mu) * rs2
            ln[n, i] = xhat * W[i] + Bv[i]
            ln_dX[n, i] = (W[i] * dY[n, i] - (xhat * c1 + c2)) * rs2
            ln_dW[i] += dY[n, i] * xhat
            ln_dB[i] += dY[n, i]
    out.update(row_X=X, row_dY=dY, row_W=W, row_B=Bv, row_eps=np.array(eps), row_offset=np.array(offset),
               softmax_Y=Y, softmax_dX=dXs, rms_Y=rms, rms_dX=rms_dX, rms_dW=rms_dW,
               ln_Y=ln, ln_dX=ln_dX, ln_dW=ln_dW, ln_dB=ln_dB)

    np.savez(HERE / "oracle_kat.npz", **out)
    print("wrote", HERE / "oracle_kat.npz", len(out), "arrays")


if __name__ == "__main__":
    main()
