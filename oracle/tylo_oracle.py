"""CPU oracle: a NumPy float64 restatement of Tylo's own plain-Julia array references.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path may import this module; only
the tests, the smoke check and the CPU-baseline leg of the benchmark use it, and only
as the checker (or as the timed CPU baseline), never as the thing shipped.

Every function follows one function of the reference's test suite (file:line given in
each docstring; paths are relative to the Tylo.jl project root).  The reference is a
Julia package and Julia cannot be run next to this code, so this is a *port*.

PARITY UNPINNED: the reference holds no golden vectors, known-answer tests or fixtures
for this path, and its own code cannot be executed here to produce any.  What checks
this port instead are the known-answer vectors under tests/golden/ (an independent
scalar-loop restatement of the same formulas, tests/golden/make_golden.py), closed-form
cases and a torch float64 autograd formulation (tests/test_oracle.py).

Array convention: Julia arrays are column-major.  A Julia array of size (D, S, H, B)
has the same bytes as a C-contiguous NumPy array of shape (B, H, S, D).  All
functions here take and return the NumPy (reversed-axes) view:

    Q  (B, H,   Sq, Dk)      K (B, Hkv, Sk, Dk)      V (B, Hkv, Sk, Dv)
    decode: Q (B, H, Dk)     lengths (B,)
    softmax / norms: X (N, M) with the reduction along the last axis (Julia dim 1).
"""
from __future__ import annotations

import math
import numpy as np

F64 = np.float64


# --------------------------------------------------------------------------------------
# mods: host evaluators (src/attention/mods.jl:53,62 hmask/hscore; bodies :101-249)
# --------------------------------------------------------------------------------------
class MaskSpec:
    """Pointwise mask over 0-based absolute positions; mirrors the mask mods.

    causal   : q >= kv                                   (mods.jl:110)
    window w : q >= kv and q <= kv + w                   (mods.jl:120)
    prefix n : kv < n                                    (mods.jl:131)
    document : doc_q[q] == doc_kv[kv]                    (mods.jl:146-147)
    The fields are AND-ed (mods.jl:157); `prefix_or_causal` gives prefix_lm's
    `causal | prefix` (mods.jl:167,178).
    """

    def __init__(self, causal=False, window=None, prefix=None, doc_q=None, doc_kv=None,
                 prefix_or_causal=None):
        self.causal = causal
        self.window = window
        self.prefix = prefix
        self.doc_q = None if doc_q is None else np.asarray(doc_q)
        self.doc_kv = self.doc_q if doc_kv is None else np.asarray(doc_kv)
        self.prefix_or_causal = prefix_or_causal

    def dense(self, q_pos: np.ndarray, kv_pos: np.ndarray) -> np.ndarray:
        """Boolean (len(q_pos), len(kv_pos)) matrix; True = attend."""
        q = q_pos[:, None].astype(np.int64)
        kv = kv_pos[None, :].astype(np.int64)
        keep = np.ones((q_pos.size, kv_pos.size), dtype=bool)
        if self.causal:
            keep &= q >= kv
        if self.window is not None:
            keep &= (q >= kv) & (q <= kv + int(self.window))
        if self.prefix is not None:
            keep &= kv < int(self.prefix)
        if self.prefix_or_causal is not None:
            keep &= (q >= kv) | (kv < int(self.prefix_or_causal))
        if self.doc_q is not None:
            dq = self.doc_q if self.doc_q.ndim == 1 else None
            if dq is None:
                raise ValueError("per-batch document ids are resolved by the caller")
            keep &= self.doc_q[q_pos][:, None] == self.doc_kv[kv_pos][None, :]
        return keep


class MaskAny:
    """OrMask (mods.jl:164-167): attend where any of the given MaskSpec conjunctions does."""

    def __init__(self, *specs):
        self.specs = specs

    def dense(self, q_pos: np.ndarray, kv_pos: np.ndarray) -> np.ndarray:
        keep = np.zeros((q_pos.size, kv_pos.size), dtype=bool)
        for sp in self.specs:
            keep |= sp.dense(q_pos, kv_pos)
        return keep


class ScoreSpec:
    """Score mod chain applied to the scaled score s0; mirrors the score mods.

    ops is a sequence of ("softcap", cap) / ("alibi", slopes) applied left to right,
    i.e. ComposeScore(a, b) = b(a(s)) (mods.jl:244-249) is ops=[a, b].
    softcap: cap * tanh(s / cap) (mods.jl:198); alibi: s + slopes[h] * (q - kv)
    (mods.jl:209, one slope per QUERY head, plus sign).
    """

    def __init__(self, ops=()):
        self.ops = list(ops)

    @staticmethod
    def _bias_slice(par, b, h):
        """bias[kv+1, q+1, mod1(h, nh), mod1(b, nb)] on LOCAL rows (mods.jl:236-237); the table is
        held as (nb, nh, Sq, Sk)."""
        t = np.asarray(par, dtype=F64)
        return t[b % t.shape[0], h % t.shape[1]]

    def _step(self, kind, par, s, b, h, rel):
        if kind == "softcap":
            return float(par) * np.tanh(s / float(par))
        if kind == "alibi":
            return s + float(np.asarray(par, dtype=F64)[h]) * rel
        if kind == "bias":
            return s + self._bias_slice(par, b, h)
        raise ValueError(kind)

    def apply(self, s0, h, q_pos, kv_pos, b=0):
        s = s0
        rel = (q_pos[:, None] - kv_pos[None, :]).astype(F64)
        for kind, par in self.ops:
            s = self._step(kind, par, s, b, h, rel)
        return s

    def vjp(self, s0, h, q_pos, kv_pos, sbar, b=0):
        """VJP at the PRE-mod score (mods.jl:288-319): returns (s0bar, {op index: parameter grad}):
        a scalar slope gradient for an ALiBi op (mods.jl:296-303), the (Sq, Sk) gradient of this
        (b, h) slice for a bias op (mods.jl:305-313)."""
        rel = (q_pos[:, None] - kv_pos[None, :]).astype(F64)
        inter = [s0]
        s = s0
        for kind, par in self.ops:
            s = self._step(kind, par, s, b, h, rel)
            inter.append(s)
        g = sbar
        pgrads = {}
        for i in reversed(range(len(self.ops))):
            kind, par = self.ops[i]
            if kind == "softcap":
                th = np.tanh(inter[i] / float(par))
                g = g * (1.0 - th * th)
            elif kind == "alibi":
                pgrads[i] = float(np.sum(g * rel))
            else:
                pgrads[i] = g.copy()
        return g, pgrads


# --------------------------------------------------------------------------------------
# attention forward / backward
# --------------------------------------------------------------------------------------
def _softmax_cols(S):
    """Row-wise (over kv) softmax with the fully-masked guard of test/flex.jl:25-32."""
    mx = np.max(S, axis=-1, keepdims=True)
    finite = np.isfinite(mx)
    P = np.exp(S - np.where(finite, mx, 0.0))
    P = np.where(finite, P, 0.0)
    den = np.sum(P, axis=-1, keepdims=True)
    P = np.divide(P, den, out=np.zeros_like(P), where=den > 0)
    return P, mx, den


def flex_ref(Q, K, V, *, score: ScoreSpec | None = None, mask: MaskSpec | None = None,
             input_pos: int = 0, qk_scale: float | None = None, doc_per_batch=None,
             return_stats: bool = False, keep_dense=None):
    """test/flex.jl:8-35 (flex_ref); with score=None, mask=causal-or-None it is also
    test/attention.jl:9-28 (attn_ref: `n > m` masked == causal with input_pos = 0).

    doc_per_batch: optional (B, S) int array — a per-sequence document-id table, the
    extension used for the causal ∧ window ∧ document benchmark config; it overrides
    the mask's 1-D document vector for batch b.
    keep_dense: optional boolean (Sq, Sk) matrix used instead of `mask` (block-mask path below).
    Returns O (B, H, Sq, Dv) [and natural-base row max M and row sum L, (B, H, Sq)].
    """
    Q = np.asarray(Q, F64); K = np.asarray(K, F64); V = np.asarray(V, F64)
    B, H, Sq, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    g = H // Hkv
    scale = 1.0 / math.sqrt(Dk) if qk_scale is None else float(qk_scale)
    q_pos = np.arange(Sq) + int(input_pos)
    kv_pos = np.arange(Sk)
    O = np.zeros((B, H, Sq, Dv), F64)
    Ms = np.zeros((B, H, Sq), F64); Ls = np.zeros((B, H, Sq), F64)
    keep_shared = None
    if mask is not None and doc_per_batch is None:
        keep_shared = mask.dense(q_pos, kv_pos)
    if keep_dense is not None:
        keep_shared = np.asarray(keep_dense, dtype=bool)
        mask = None
    for b in range(B):
        keep = keep_shared
        if mask is not None and doc_per_batch is not None:
            m2 = MaskSpec(mask.causal, mask.window, mask.prefix,
                          doc_per_batch[b], doc_per_batch[b], mask.prefix_or_causal)
            keep = m2.dense(q_pos, kv_pos)
        for h in range(H):
            hk = h // g                          # cld(h, g) on 1-based h (attention.jl:23)
            S = (Q[b, h] @ K[b, hk].T) * scale   # (Sq, Sk)
            if score is not None:
                S = score.apply(S, h, q_pos, kv_pos, b)
            if keep is not None:
                S = np.where(keep, S, -np.inf)
            P, mx, den = _softmax_cols(S)
            O[b, h] = P @ V[b, hk]
            Ms[b, h] = mx[:, 0]; Ls[b, h] = den[:, 0]
    if return_stats:
        return O, Ms, Ls
    return O


def build_block_mask_ref(keep, n_q, n_kv, *, TILE_M=64, TILE_N=64, input_pos=0):
    """src/attention/mods.jl:448-476 (build_block_mask), element by element as the reference does.
    keep(q, kv) -> bool on 0-based absolute positions.  Returns (count (n_qb,), idx (n_qb, n_kb),
    full (n_qb, n_kb)) int32 — the reference's [n_kb, n_qb] column-major arrays, same bytes."""
    nqb, nkb = -(-n_q // TILE_M), -(-n_kv // TILE_N)
    idx = np.zeros((nqb, nkb), np.int32); full = np.zeros((nqb, nkb), np.int32)
    cnt = np.zeros(nqb, np.int32)
    for i in range(nqb):
        qlo, qhi = i * TILE_M, min((i + 1) * TILE_M, n_q) - 1
        slot = 0
        for j in range(nkb):
            klo, khi = j * TILE_N, min((j + 1) * TILE_N, n_kv) - 1
            anyk, allk = False, True
            for q in range(qlo, qhi + 1):
                for kv in range(klo, khi + 1):
                    k = bool(keep(q + input_pos, kv))
                    anyk |= k; allk &= k
            if anyk:
                idx[i, slot] = j
                # boundary blocks are never "full" (mods.jl:468-470)
                full[i, slot] = 1 if (allk and (i + 1) * TILE_M <= n_q and (j + 1) * TILE_N <= n_kv) else 0
                slot += 1
        cnt[i] = slot
    return cnt, idx, full


def flex_block_mask_ref(Q, K, V, count, idx, full, *, TILE_M=64, TILE_N=64, score: ScoreSpec | None = None,
                        mask: MaskSpec | None = None, input_pos: int = 0, qk_scale: float | None = None,
                        return_stats: bool = False):
    """src/attention/flex.jl:107-182 (flex_fwd_bm) on plain arrays: query block i visits only the key
    blocks idx[i, :count[i]]; in a block marked full the mask mod is skipped (only kv < Sk applies),
    elsewhere it is evaluated per pair; pairs of unlisted blocks contribute nothing.  The reference has
    no plain-array version of this walk; its tests compare it with flex_ref under an agreeing mask
    (test/flex.jl:258-280), which tests/test_oracle_block_mask.py repeats."""
    Sq, Sk = np.asarray(Q).shape[2], np.asarray(K).shape[2]
    eff = block_mask_dense(count, idx, full, Sq, Sk, TILE_M=TILE_M, TILE_N=TILE_N, mask=mask, input_pos=input_pos)
    return flex_ref(Q, K, V, score=score, input_pos=input_pos, qk_scale=qk_scale, return_stats=return_stats,
                    keep_dense=eff)


def block_mask_dense(count, idx, full, Sq, Sk, *, TILE_M=64, TILE_N=64, mask: MaskSpec | None = None,
                     input_pos: int = 0):
    """The pairs the block walk of flex.jl:107-182 lets through, as a boolean (Sq, Sk) matrix."""
    q_pos = np.arange(Sq) + int(input_pos); kv_pos = np.arange(Sk)
    dense = mask.dense(q_pos, kv_pos) if mask is not None else np.ones((Sq, Sk), bool)
    eff = np.zeros((Sq, Sk), bool)
    for i in range(-(-Sq // TILE_M)):
        rows = slice(i * TILE_M, min((i + 1) * TILE_M, Sq))
        for t in range(int(count[i])):
            j = int(idx[i, t])
            cols = slice(j * TILE_N, min((j + 1) * TILE_N, Sk))
            eff[rows, cols] = True if full[i, t] else dense[rows, cols]
    return eff


def flex_block_mask_bwd_ref(dO, Q, K, V, count, idx, full, *, TILE_M=64, TILE_N=64, score: ScoreSpec | None = None,
                            mask: MaskSpec | None = None, input_pos: int = 0, qk_scale: float | None = None):
    """Gradients of flex_block_mask_ref: test/flex.jl:75-114 (flex_bwd_ref) over the pairs the block walk
    lets through.  The reference has no backward for this path (flex.jl:193-194)."""
    Sq, Sk = np.asarray(Q).shape[2], np.asarray(K).shape[2]
    eff = block_mask_dense(count, idx, full, Sq, Sk, TILE_M=TILE_M, TILE_N=TILE_N, mask=mask, input_pos=input_pos)
    return flex_bwd_ref(dO, Q, K, V, score=score, input_pos=input_pos, qk_scale=qk_scale, keep_dense=eff)


def attn_ref(Q, K, V, *, causal=False):
    """test/attention.jl:9-28."""
    return flex_ref(Q, K, V, mask=MaskSpec(causal=True) if causal else None)


def flex_bwd_ref(dO, Q, K, V, *, score: ScoreSpec | None = None, mask: MaskSpec | None = None,
                 input_pos: int = 0, qk_scale: float | None = None, doc_per_batch=None, keep_dense=None):
    """test/flex.jl:75-114 (flex_bwd_ref) == test/attention.jl:30-55 (attn_bwd_ref) when
    there is no score mod.  Returns (dQ, dK, dV, slope_grads) where slope_grads maps the
    index of each ALiBi op in the chain to its (H,) slope gradient (mods.jl:296-303)."""
    dO = np.asarray(dO, F64); Q = np.asarray(Q, F64); K = np.asarray(K, F64); V = np.asarray(V, F64)
    B, H, Sq, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    g = H // Hkv
    scale = 1.0 / math.sqrt(Dk) if qk_scale is None else float(qk_scale)
    q_pos = np.arange(Sq) + int(input_pos)
    kv_pos = np.arange(Sk)
    dQ = np.zeros_like(Q); dK = np.zeros_like(K); dV = np.zeros_like(V)
    slope_grads = {}
    if score is not None:
        for i, (kind, par) in enumerate(score.ops):
            if kind == "alibi":
                slope_grads[i] = np.zeros(H, F64)
            elif kind == "bias":
                slope_grads[i] = np.zeros(np.asarray(par).shape, F64)
    keep_shared = None
    if mask is not None and doc_per_batch is None:
        keep_shared = mask.dense(q_pos, kv_pos)
    if keep_dense is not None:                  # boolean (Sq, Sk) used instead of `mask` (block-mask path)
        keep_shared = np.asarray(keep_dense, dtype=bool)
        mask = None
    for b in range(B):
        keep = keep_shared
        if mask is not None and doc_per_batch is not None:
            m2 = MaskSpec(mask.causal, mask.window, mask.prefix,
                          doc_per_batch[b], doc_per_batch[b], mask.prefix_or_causal)
            keep = m2.dense(q_pos, kv_pos)
        for h in range(H):
            hk = h // g
            S0 = (Q[b, h] @ K[b, hk].T) * scale
            S = S0 if score is None else score.apply(S0, h, q_pos, kv_pos, b)
            if keep is not None:
                S = np.where(keep, S, -np.inf)
            P, _, _ = _softmax_cols(S)
            do = dO[b, h]                                   # (Sq, Dv)
            dP = do @ V[b, hk].T                            # (Sq, Sk)
            dS = P * (dP - np.sum(P * dP, axis=-1, keepdims=True))
            if score is not None:
                dS0, pg = score.vjp(S0, h, q_pos, kv_pos, dS, b)
                for i, val in pg.items():
                    if score.ops[i][0] == "alibi":
                        slope_grads[i][h] += val
                    else:                       # heads / batch entries that share a table slice add up
                        t = slope_grads[i]
                        t[b % t.shape[0], h % t.shape[1]] += val
            else:
                dS0 = dS
            dQ[b, h] = (dS0 @ K[b, hk]) * scale
            dK[b, hk] += (dS0.T @ Q[b, h]) * scale
            dV[b, hk] += P.T @ do
    return dQ, dK, dV, slope_grads


def attn_bwd_ref(dO, Q, K, V, *, causal=False):
    """test/attention.jl:30-55."""
    return flex_bwd_ref(dO, Q, K, V, mask=MaskSpec(causal=True) if causal else None)[:3]


# --------------------------------------------------------------------------------------
# decode (test/decode.jl:15-36) and the split merge algebra (src/attention/decode.jl:119-140)
# --------------------------------------------------------------------------------------
def decode_reference(Q, K, V, lengths):
    """test/decode.jl:15-36. Q (B,H,Dk), K (B,Hkv,Sk,Dk), V (B,Hkv,Sk,Dv) → O (B,H,Dv)."""
    Q = np.asarray(Q, F64); K = np.asarray(K, F64); V = np.asarray(V, F64)
    B, H, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    G = H // Hkv
    scale = 1.0 / math.sqrt(Dk)
    O = np.zeros((B, H, Dv), F64)
    for b in range(B):
        L = int(lengths[b])
        if L == 0:
            continue
        for hk in range(Hkv):
            q = Q[b, hk * G:(hk + 1) * G]                   # (G, Dk)
            s = scale * (q @ K[b, hk, :L].T)                # (G, L)
            w = np.exp(s - s.max(axis=-1, keepdims=True))
            w /= w.sum(axis=-1, keepdims=True)
            O[b, hk * G:(hk + 1) * G] = w @ V[b, hk, :L]
    return O


def decode_partials(Q, K, V, lengths, kv_begin, kv_end):
    """Partial (normalised O, M in log2 units, L) of one KV slice [kv_begin, kv_end) —
    what one split / one GPU owns (src/attention/decode.jl:50-53,92-98)."""
    Q = np.asarray(Q, F64); K = np.asarray(K, F64); V = np.asarray(V, F64)
    B, H, Dk = Q.shape
    _, Hkv, Sk, Dv = V.shape
    G = H // Hkv
    scale = 1.0 / math.sqrt(Dk) * math.log2(math.e)
    O = np.zeros((B, H, Dv), F64); M = np.full((B, H), -np.inf); Ls = np.zeros((B, H))
    for b in range(B):
        hi = min(int(lengths[b]), kv_end)
        if hi <= kv_begin:
            continue
        for h in range(H):
            hk = h // G
            s = scale * (K[b, hk, kv_begin:hi] @ Q[b, h])
            m = s.max(); p = np.exp2(s - m); l = p.sum()
            O[b, h] = (p @ V[b, hk, kv_begin:hi]) / l
            M[b, h] = m; Ls[b, h] = l
    return O, M, Ls


def decode_combine(O_parts, M_parts, L_parts):
    """src/attention/decode.jl:119-140: LSE merge over the leading `split` axis with the
    -Inf guards; O_parts (S,B,H,Dv), M_parts/L_parts (S,B,H)."""
    S = O_parts.shape[0]
    m = np.full(M_parts.shape[1:], -np.inf); l = np.zeros(M_parts.shape[1:])
    acc = np.zeros(O_parts.shape[1:])
    for s in range(S):
        m_new = np.maximum(m, M_parts[s])
        fin = np.isfinite(m_new)
        with np.errstate(invalid="ignore"):
            alpha = np.where(fin, np.exp2(m - m_new), 1.0)
            gamma = np.where(fin, np.exp2(M_parts[s] - m_new), 0.0)
        ls = L_parts[s] * gamma
        l = l * alpha + ls
        acc = acc * alpha[..., None] + ls[..., None] * O_parts[s]
        m = m_new
    return np.divide(acc, l[..., None], out=np.zeros_like(acc), where=l[..., None] > 0)


# --------------------------------------------------------------------------------------
# softmax (test/softmax.jl:10,13) and norms (test/norm.jl:8-20,78-102)
# --------------------------------------------------------------------------------------
def softmax_ref(X):
    """test/softmax.jl:10 — softmax along the contiguous axis."""
    X = np.asarray(X, F64)
    e = np.exp(X - X.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def softmax_bwd_ref(dY, Y):
    """test/softmax.jl:13."""
    dY = np.asarray(dY, F64); Y = np.asarray(Y, F64)
    return Y * (dY - np.sum(Y * dY, axis=-1, keepdims=True))


def rms_norm_ref(X, W, *, eps, offset=0.0):
    """test/norm.jl:8-12."""
    X = np.asarray(X, F64); W = np.asarray(W, F64)
    rstd = 1.0 / np.sqrt(np.mean(X * X, axis=-1, keepdims=True) + eps)
    return (X * rstd) * (W + offset)


def layer_norm_ref(X, W, Bv, *, eps):
    """test/norm.jl:15-20."""
    X = np.asarray(X, F64); W = np.asarray(W, F64); Bv = np.asarray(Bv, F64)
    xc = X - X.mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(np.mean(xc * xc, axis=-1, keepdims=True) + eps)
    return (xc * rstd) * W + Bv


def rms_norm_bwd_ref(dY, X, W, *, eps, offset=0.0):
    """test/norm.jl:78-87 → (dX, dW, rstd)."""
    dY = np.asarray(dY, F64); X = np.asarray(X, F64); W = np.asarray(W, F64)
    M = X.shape[-1]
    g = W + offset
    rstd = 1.0 / np.sqrt(np.mean(X * X, axis=-1, keepdims=True) + eps)
    dd = np.sum(dY * (g * X), axis=-1, keepdims=True) / M
    dX = rstd * (dY * g - (rstd ** 2 * dd) * X)
    dW = np.sum(dY * X * rstd, axis=0)
    return dX, dW, rstd[..., 0]


def layer_norm_bwd_ref(dY, X, W, *, eps):
    """test/norm.jl:90-102 → (dX, dW, dB, mean, rstd)."""
    dY = np.asarray(dY, F64); X = np.asarray(X, F64); W = np.asarray(W, F64)
    mean = X.mean(axis=-1, keepdims=True)
    xc = X - mean
    rstd = 1.0 / np.sqrt(np.mean(xc * xc, axis=-1, keepdims=True) + eps)
    xhat = xc * rstd
    wdy = W * dY
    c1 = np.mean(xhat * wdy, axis=-1, keepdims=True)
    c2 = np.mean(wdy, axis=-1, keepdims=True)
    dX = (wdy - (xhat * c1 + c2)) * rstd
    dW = np.sum(dY * xhat, axis=0)
    dB = np.sum(dY, axis=0)
    return dX, dW, dB, mean[..., 0], rstd[..., 0]
