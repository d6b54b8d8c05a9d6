"""Python host binding of libtylo_b200 — a mirror of Tylo.jl's exported API.

The production host layer is the Julia package under ``julia/Tylo`` (same directory), whose
wrappers ``ccall`` the C ABI declared in ``include/tylo_b200.h``.  Julia is not available where
this library is tested, so this module binds the *same* C ABI through ctypes and mirrors the
Julia API one to one; the tests and the benchmark drive the kernels through it.

Naming: Julia's ``f!`` is ``f_`` here, ``∇f`` is ``grad_f`` and ``∇f!`` is ``grad_f_``.

Layout: a Julia array of size (D, S, H, B) is column-major; the same bytes are a contiguous
torch tensor of shape (B, H, S, D).  Every tensor below is given in that reversed-axes form:

    Q (B, H, Sq, Dk)   K (B, Hkv, Sk, Dk)   V (B, Hkv, Sk, Dv)   O (B, H, Sq, Dv)
    decode: Q (B, H, Dk), O (B, H, Dv), lengths (B,) int32
    softmax / norms: X (N, M), reduction over the last axis; W, B (M,)

torch is used only for device memory and streams.  There is no CPU implementation and no
fallback: if the shared library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import math
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_uint32, c_void_p
from pathlib import Path
from typing import NamedTuple, Optional

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = Path(os.environ.get("TYLO_B200_LIB", _HERE / "libtylo_b200.so"))
if not _LIB_PATH.exists():
    raise ImportError(
        f"{_LIB_PATH} not found: build it with `python {_HERE / 'build.py'}` "
        "(libtylo_b200 has no CPU or pure-PyTorch fallback)")
_lib = ctypes.CDLL(str(_LIB_PATH))

F32, BF16, F16, F32_TF32 = 0, 1, 2, 3
_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
TFloat32 = "TFloat32"      # value of the `tensorcore` keyword that asks for TF32 products on Float32 storage

MASK_CAUSAL, MASK_SLIDING, MASK_DOCUMENT, MASK_PREFIX, MASK_PREFIX_LM = 1, 2, 4, 8, 16
SCORE_ALIBI, SCORE_SOFTCAP, SCORE_SOFTCAP_FIRST, SCORE_BIAS = 1, 2, 4, 8


class _MaskDesc(Structure):
    _fields_ = [("flags", c_uint32), ("window", c_int32), ("prefix_len", c_int32), ("reserved", c_int32),
                ("doc_q", c_void_p), ("doc_kv", c_void_p), ("doc_batch_stride", c_int64),
                ("doc_q_len", c_int64), ("doc_kv_len", c_int64), ("or_next", c_void_p)]


class _ScoreDesc(Structure):
    _fields_ = [("flags", c_uint32), ("cap", c_float), ("slopes", c_void_p), ("d_slopes", c_void_p),
                ("bias", c_void_p), ("d_bias", c_void_p), ("bias_heads", c_int32), ("bias_batch", c_int32)]


class TyloError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libtylo_b200 status {status} ({_status_string(status)}): {message}")
        self.status = status


_lib.tylo_b200_version.restype = c_int32
_lib.tylo_b200_status_string.restype = c_char_p
_lib.tylo_b200_status_string.argtypes = [c_int32]
_lib.tylo_b200_last_error.restype = c_char_p
_lib.tylo_b200_attention_bwd_workspace_bytes.restype = c_int64
_lib.tylo_b200_attention_bwd_workspace_bytes.argtypes = [c_int32] * 8
_lib.tylo_b200_device_status.restype = c_int32
_lib.tylo_b200_device_status.argtypes = [POINTER(c_int32)]
_lib.tylo_b200_decode_suggest_splits.restype = c_int32
_lib.tylo_b200_decode_suggest_splits.argtypes = [c_int32] * 3
_lib.tylo_b200_decode_ticket_count.restype = c_int64
_lib.tylo_b200_decode_ticket_count.argtypes = [c_int32] * 3
_lib.tylo_b200_decode_exchange_bytes.restype = c_int64
_lib.tylo_b200_decode_exchange_bytes.argtypes = [c_int32] * 4
_lib.tylo_b200_peer_handle_bytes.restype = c_int32
_lib.tylo_b200_peer_handle_bytes.argtypes = []

_i32, _i64, _f32, _ptr = c_int32, c_int64, c_float, c_void_p
_SIGS = {
    "tylo_b200_attention_fwd": [_ptr] * 8 + [_i32] * 10 + [_ptr],
    "tylo_b200_attention_bwd": [_ptr] * 13 + [_i64] + [_ptr] * 2 + [_i32] * 10 + [_ptr],
    "tylo_b200_flex_attention_fwd": [_ptr] * 6 + [POINTER(_MaskDesc), POINTER(_ScoreDesc)] + [_i32] * 8 + [_f32, _i32, _i32, _ptr],
    "tylo_b200_flex_attention_fwd_block_mask": [_ptr] * 6 + [POINTER(_MaskDesc), POINTER(_ScoreDesc)] + [_ptr] * 3
                                               + [_i32] * 3 + [_i32] * 8 + [_f32, _i32, _ptr],
    "tylo_b200_flex_attention_bwd_block_mask": [_ptr] * 12 + [c_int64, POINTER(_MaskDesc), POINTER(_ScoreDesc)]
                                               + [_ptr] * 3 + [_i32] * 3 + [_i32] * 8 + [_f32, _i32, _ptr],
    "tylo_b200_flex_attention_bwd": [_ptr] * 13 + [_i64, POINTER(_MaskDesc), POINTER(_ScoreDesc)] + [_i32] * 8 + [_f32, _i32, _i32, _ptr],
    "tylo_b200_decode_attention": [_ptr] * 8 + [_i32] * 8 + [_ptr],
    "tylo_b200_decode_split": [_ptr] * 7 + [_i32] * 8 + [_ptr],
    "tylo_b200_decode_attention_fused": [_ptr] * 9 + [_i32] * 8 + [_ptr],
    "tylo_b200_decode_attention_paged": [_ptr] * 10 + [_i32] * 9 + [_ptr],
    "tylo_b200_decode_attention_sharded": [_ptr] * 9 + [_i32, POINTER(c_void_p)] + [_i32] * 9 + [_i64, _ptr],
    "tylo_b200_decode_combine": [_ptr] * 7 + [_i32, _i64, _i64] + [_i32] * 4 + [_ptr],
    "tylo_b200_decode_exchange": [_ptr] * 4 + [_i32, _i64, _i64, POINTER(c_void_p)] + [_i32] * 6 + [_i64, _ptr],
    "tylo_b200_decode_exchange_status": [_ptr, POINTER(c_int32)],
    "tylo_b200_peer_alloc": [POINTER(c_void_p), _i64],
    "tylo_b200_peer_free": [_ptr],
    "tylo_b200_peer_export": [_ptr, _ptr],
    "tylo_b200_peer_open": [POINTER(c_void_p), _ptr],
    "tylo_b200_peer_close": [_ptr],
    "tylo_b200_softmax_fwd": [_ptr, _ptr, _i64, _i64, _i32, _ptr],
    "tylo_b200_softmax_bwd": [_ptr, _ptr, _ptr, _i64, _i64, _i32, _ptr],
    "tylo_b200_rms_norm_fwd": [_ptr] * 4 + [_i64, _i64, _f32, _f32, _i32, _ptr],
    "tylo_b200_rms_norm_bwd": [_ptr] * 7 + [_i32, _i64, _i64, _f32, _i32, _ptr],
    "tylo_b200_layer_norm_fwd": [_ptr] * 6 + [_i64, _i64, _f32, _i32, _ptr],
    "tylo_b200_layer_norm_bwd": [_ptr] * 10 + [_i32, _i64, _i64, _i32, _ptr],
}
for _name, _sig in _SIGS.items():
    _fn = getattr(_lib, _name)
    _fn.restype = c_int32
    _fn.argtypes = _sig


def _status_string(status: int) -> str:
    return _lib.tylo_b200_status_string(status).decode()


def _check(status: int) -> None:
    if status != 0:
        raise TyloError(status, _lib.tylo_b200_last_error().decode())


def version() -> int:
    return int(_lib.tylo_b200_version())


def lib_path() -> str:
    return str(_LIB_PATH)


def device_status() -> int:
    """Synchronises and returns the device-side health word (0 = healthy); raises TyloError with
    status 6 if a bounded wait inside a tensor-core kernel gave up."""
    code = c_int32(0)
    _check(_lib.tylo_b200_device_status(ctypes.byref(code)))
    return int(code.value)


def _p(t: Optional[torch.Tensor]):
    """Raw device address of a tensor (None stays a null pointer).  A host tensor is refused here, before
    any launch: the kernels would read its address on the GPU (the Julia wrapper's `devptr` does the same)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("libtylo_b200 reads device memory only: got a host tensor; move it to the GPU first")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported element type {t.dtype}") from None


def _fwd_dtype(t: torch.Tensor, tensorcore) -> int:
    """Element-type code of a forward attention call.  `tensorcore` mirrors the reference's keyword
    (utils.jl:43-44: Float32 storage defaults to TFloat32 operands there): None computes Float32 in true fp32;
    TFloat32 / "tf32" reads the operands of both matrix products as TF32 on the tensor cores (Float32 storage
    only; 16-bit storage always runs in its own type, as in the reference)."""
    code = _dtype(t)
    if tensorcore is None:
        return code
    name = tensorcore if isinstance(tensorcore, str) else getattr(tensorcore, "__name__", str(tensorcore))
    if name.lower() in ("tfloat32", "tf32"):
        return F32_TF32 if code == F32 else code
    if name.lower() in ("float32", "fp32", "f32", "bfloat16", "bf16", "float16", "f16", "fp16"):
        return code
    raise ValueError(f"tensorcore={tensorcore!r}: expected None or TFloat32")


def _dense(*ts):
    for t in ts:
        if t is not None:
            if not t.is_cuda:
                raise ValueError("libtylo_b200 takes device arrays (there is no CPU path)")
            if not t.is_contiguous():
                raise ValueError("arrays must be dense")


# ---------------------------------------------------------------------------------------------
# buffer vocabulary (src/buffers.jl)
# ---------------------------------------------------------------------------------------------
class Duplicated:
    """A primal array paired with its gradient buffer (buffers.jl:26-31).  ``Duplicated(x)``
    allocates an uninitialised shadow (the backward entry points overwrite it)."""

    __slots__ = ("primal", "shadow")

    def __init__(self, primal_, shadow_=None):
        self.primal = primal_
        self.shadow = torch.empty_like(primal_) if shadow_ is None else shadow_


def primal(x):
    return x.primal if isinstance(x, Duplicated) else x


def shadow(x):
    return x.shadow


# ---------------------------------------------------------------------------------------------
# mods (src/attention/mods.jl)
# ---------------------------------------------------------------------------------------------
class MaskMod:
    def __and__(self, other):
        return AndMask(self, other)

    def __or__(self, other):
        return OrMask(self, other)


class FullMask(MaskMod):
    def __call__(self, b, h, q, kv):
        return True


class CausalMask(MaskMod):
    def __call__(self, b, h, q, kv):
        return q >= kv


class SlidingWindowMask(MaskMod):
    def __init__(self, w: int):
        self.w = int(w)

    def __call__(self, b, h, q, kv):
        return q >= kv and q <= kv + self.w


class PrefixMask(MaskMod):
    def __init__(self, length: int):
        self.len = int(length)

    def __call__(self, b, h, q, kv):
        return kv < self.len


class DocumentMask(MaskMod):
    """Same-document attention.  ``doc`` is an int32 vector indexed by absolute position
    (mods.jl:141-147).  Extension: a 2-D ``(B, S)`` table gives every batch entry its own ids."""

    def __init__(self, doc_q, doc_kv=None):
        self.doc_q = doc_q
        self.doc_kv = doc_q if doc_kv is None else doc_kv

    def __call__(self, b, h, q, kv):
        dq, dk = self.doc_q, self.doc_kv
        if dq.dim() == 2:
            return bool(dq[b - 1, q] == dk[b - 1, kv])
        return bool(dq[q] == dk[kv])


class AndMask(MaskMod):
    def __init__(self, a, b):
        self.a, self.b = a, b

    def __call__(self, b, h, q, kv):
        return self.a(b, h, q, kv) and self.b(b, h, q, kv)


class OrMask(MaskMod):
    def __init__(self, a, b):
        self.a, self.b = a, b

    def __call__(self, b, h, q, kv):
        return self.a(b, h, q, kv) or self.b(b, h, q, kv)


def prefix_lm(length: int) -> MaskMod:
    return CausalMask() | PrefixMask(length)


class BlockMask(NamedTuple):
    """Precomputed coarse block sparsity (mods.jl:436-440): per query block the key blocks holding any
    unmasked pair and which of those are fully unmasked.  ``count`` (n_qb,), ``idx`` and ``full``
    (n_qb, n_kb) are int32 device tensors (the reference's [n_kb, n_qb] column-major arrays); the block
    edges the mask was built for travel with it.  Forward only (flex.jl:193-194)."""
    count: torch.Tensor
    idx: torch.Tensor
    full: torch.Tensor
    TILE_M: int = 64
    TILE_N: int = 64


def build_block_mask(keep, n_q: int, n_kv: int, *, TILE_M: int = 64, TILE_N: int = 64, input_pos: int = 0,
                     device="cuda") -> BlockMask:
    """build_block_mask(keep, n_q, n_kv; TILE_M, TILE_N, input_pos) (mods.jl:448-476): built on the host
    from ``keep(q, kv) -> bool`` over 0-based absolute positions, e.g. ``lambda q, kv: hmask(mod, q, kv)``.
    ``keep`` is first tried on whole index arrays (a predicate written with comparisons works as is)
    and evaluated pair by pair otherwise.  A block that touches the end of Q or K is never marked full."""
    import numpy as np
    nqb, nkb = -(-n_q // TILE_M), -(-n_kv // TILE_N)
    dense = None
    try:
        got = keep(np.arange(n_q, dtype=np.int64)[:, None] + int(input_pos), np.arange(n_kv, dtype=np.int64)[None, :])
        got = np.asarray(got)
        if got.shape == (n_q, n_kv) and got.dtype == np.bool_:
            dense = got
    except Exception:
        dense = None
    if dense is None:
        dense = np.zeros((n_q, n_kv), dtype=bool)
        for q in range(n_q):
            for kv in range(n_kv):
                dense[q, kv] = bool(keep(q + int(input_pos), kv))
    idx = np.zeros((nqb, nkb), np.int32); full = np.zeros((nqb, nkb), np.int32); cnt = np.zeros(nqb, np.int32)
    for i in range(nqb):
        slot = 0
        for j in range(nkb):
            blk = dense[i * TILE_M:(i + 1) * TILE_M, j * TILE_N:(j + 1) * TILE_N]
            if blk.any():
                idx[i, slot] = j
                full[i, slot] = int(blk.all() and (i + 1) * TILE_M <= n_q and (j + 1) * TILE_N <= n_kv)
                slot += 1
        cnt[i] = slot
    dev = torch.device(device)
    return BlockMask(torch.from_numpy(cnt).to(dev), torch.from_numpy(idx).to(dev), torch.from_numpy(full).to(dev),
                     int(TILE_M), int(TILE_N))


class ScoreMod:
    def __matmul__(self, inner):  # Julia's `outer ∘ inner`
        return ComposeScore(inner, self)


class NoOpScore(ScoreMod):
    def __call__(self, s, b, h, q, kv):
        return s


class SoftCapScore(ScoreMod):
    def __init__(self, cap: float):
        self.cap = float(cap)

    def __call__(self, s, b, h, q, kv):
        return self.cap * math.tanh(s / self.cap)


class AliBiScore(ScoreMod):
    def __init__(self, slopes: torch.Tensor):
        self.slopes = slopes

    def __call__(self, s, b, h, q, kv):
        return s + float(self.slopes[h - 1]) * (q - kv)


class BiasScore(ScoreMod):
    """``s + bias[kv, q, mod1(h, nh), mod1(b, nb)]`` (mods.jl:212-237).  ``bias`` is a float32 tensor
    (nb, nh, Sq, Sk) — Julia's (Sk, Sq, nh, nb) — indexed by local rows: q and kv are not shifted by
    ``input_pos``.  Runs on the fp32-arithmetic kernels."""

    def __init__(self, bias: torch.Tensor):
        if bias.dim() != 4:
            raise ValueError("BiasScore expects (bias_batch, bias_heads, Sq, Sk)")
        self.bias = bias

    def __call__(self, s, b, h, q, kv):
        nb, nh = self.bias.shape[:2]
        return s + float(self.bias[(b - 1) % nb, (h - 1) % nh, q, kv])


class ComposeScore(ScoreMod):
    """Apply ``a`` then ``b`` (mods.jl:244-249)."""

    def __init__(self, a, b):
        self.a, self.b = a, b

    def __call__(self, s, b, h, q, kv):
        return self.b(self.a(s, b, h, q, kv), b, h, q, kv)


def pair_feature(op, qvals, kvals):
    """pair_feature(op, qvals, kvals) -> tuple of PD pair features (pair.jl:37).  User code: ``op`` provides
    ``pair_feature(qvals, kvals)`` written with broadcasting arithmetic, so that the one definition serves
    scalars (host evaluation) and (Sq, 1) / (1, Sk) device rows (bias-table construction)."""
    return op.pair_feature(qvals, kvals)


def grad_pair_feature(op, qvals, kvals, dphi):
    """∇pair_feature(op, qvals, kvals, dphi) -> (dq, dk) (pair.jl:112): the VJP of ``pair_feature``; needed
    only for feature gradients."""
    return op.grad_pair_feature(qvals, kvals, dphi)


class PairFeatureScore(ScoreMod):
    """PairFeatureScore(op, q_features, k_features, pair_proj) (pair.jl:49-70):
    ``s + sum_p pair_proj[h, p] * pair_feature(op, qvals, kvals)[p]`` with ``qvals = q_features[b, q, :]``,
    ``kvals = k_features[b, kv, :]`` (local positions).  Tensors: q_features (batch, Sq, F), k_features
    (batch, Sk, F), pair_proj (PD, heads) — Julia's (F, Sq, batch), (F, Sk, batch), (heads, PD).

    The op is user code and cannot be compiled into the library's kernels: the wrappers evaluate it on
    whole feature rows with device broadcasts into the (batch, heads, Sq, Sk) table of a BiasScore and the
    kernels run that; gradients of the table are folded back into the projection (and the features)."""

    def __init__(self, op, q_features, k_features, pair_proj):
        if q_features is not None and k_features is not None and q_features.shape[-1] != k_features.shape[-1]:
            raise ValueError(f"q_features has {q_features.shape[-1]} feature rows, k_features has {k_features.shape[-1]}")
        self.op, self.q_features, self.k_features, self.pair_proj = op, q_features, k_features, pair_proj

    def __call__(self, s, b, h, q, kv):
        F = self.q_features.shape[-1]
        qv = tuple(float(self.q_features[b - 1, q, f]) for f in range(F))
        kvv = tuple(float(self.k_features[b - 1, kv, f]) for f in range(F))
        phi = pair_feature(self.op, qv, kvv)
        return s + sum(float(self.pair_proj[p, h - 1]) * float(phi[p]) for p in range(self.pair_proj.shape[0]))

    def _rows(self, b):
        F = self.q_features.shape[-1]
        return (tuple(self.q_features[b, :, f].float()[:, None] for f in range(F)),
                tuple(self.k_features[b, :, f].float()[None, :] for f in range(F)))

    def bias_table(self) -> torch.Tensor:
        """The (batch, heads, Sq, Sk) float32 table this mod stands for."""
        B, Sq, Sk = self.q_features.shape[0], self.q_features.shape[1], self.k_features.shape[1]
        PD, H = self.pair_proj.shape
        out = torch.empty(B, H, Sq, Sk, dtype=torch.float32, device=self.q_features.device)
        proj = self.pair_proj.float()
        for b in range(B):
            phi = pair_feature(self.op, *self._rows(b))
            stack = torch.stack([torch.broadcast_to(x, (Sq, Sk)) for x in phi])          # (PD, Sq, Sk)
            out[b] = torch.einsum("ph,pqk->hqk", proj, stack)
        return out

    def fold_grads_(self, shadow_: "PairFeatureScore", d_bias: torch.Tensor) -> None:
        """Adds the gradients carried by a bias-table gradient (batch, heads, Sq, Sk) to ``shadow_``."""
        proj = self.pair_proj.float()
        for b in range(d_bias.shape[0]):
            qv, kv = self._rows(b)
            phi = pair_feature(self.op, qv, kv)
            Sq, Sk = d_bias.shape[2:]
            stack = torch.stack([torch.broadcast_to(x, (Sq, Sk)) for x in phi])
            shadow_.pair_proj += torch.einsum("hqk,pqk->ph", d_bias[b], stack).to(shadow_.pair_proj.dtype)
            if shadow_.q_features is not None:
                for h in range(d_bias.shape[1]):
                    dphi = tuple(proj[p, h] * d_bias[b, h] for p in range(proj.shape[0]))
                    dq, dk = grad_pair_feature(self.op, qv, kv, dphi)
                    for f in range(len(qv)):
                        shadow_.q_features[b, :, f] += torch.broadcast_to(dq[f], (Sq, Sk)).sum(1).to(shadow_.q_features.dtype)
                        shadow_.k_features[b, :, f] += torch.broadcast_to(dk[f], (Sq, Sk)).sum(0).to(shadow_.k_features.dtype)


def _has_pairs(m) -> bool:
    return isinstance(m, PairFeatureScore) or (isinstance(m, ComposeScore) and (_has_pairs(m.a) or _has_pairs(m.b)))


def _lower_pairs(m):
    """The score chain with every PairFeatureScore replaced by the BiasScore of its table."""
    if isinstance(m, PairFeatureScore):
        return BiasScore(m.bias_table())
    if isinstance(m, ComposeScore):
        return ComposeScore(_lower_pairs(m.a), _lower_pairs(m.b))
    return m


def _lower_pair_shadows(low, dm):
    if dm is None:
        return None
    if isinstance(dm, PairFeatureScore):
        return BiasScore(torch.zeros_like(low.bias))
    if isinstance(dm, ComposeScore):
        return ComposeScore(_lower_pair_shadows(low.a, dm.a), _lower_pair_shadows(low.b, dm.b))
    return dm


def _raise_pair_grads(dm, m, dlow) -> None:
    if isinstance(dm, PairFeatureScore):
        m.fold_grads_(dm, dlow.bias)
    elif isinstance(dm, ComposeScore):
        _raise_pair_grads(dm.a, m.a, dlow.a); _raise_pair_grads(dm.b, m.b, dlow.b)


def adapt(to, m):
    """adapt(to, mod): the mod rebuilt with every tensor field passed through ``to`` (mods.jl:41-44), e.g.
    ``adapt(torch.Tensor.cpu, mod)`` for a host-indexable copy to evaluate with hmask / hscore."""
    if isinstance(m, torch.Tensor):
        return to(m)
    if isinstance(m, (MaskMod, ScoreMod)):
        out = object.__new__(type(m))
        for k, v in vars(m).items():
            setattr(out, k, adapt(to, v))
        return out
    return m


def score_tangent(dm):
    """A gradient shadow of a score mod as a plain tangent (ext/ChainRulesCoreExt.jl:110-113): tensors are
    their own tangent, nested mods become {field: tangent}, anything else has none (None)."""
    if isinstance(dm, torch.Tensor):
        return dm
    if isinstance(dm, ScoreMod):
        return {k: score_tangent(v) for k, v in vars(dm).items()}
    return None


def hmask(m: MaskMod, q: int, kv: int, *, b: int = 1, h: int = 1) -> bool:
    """Evaluate a mask mod on the host at 0-based positions (mods.jl:53); b, h are 1-based."""
    return bool(m(b, h, q, kv))


def hscore(m: ScoreMod, s: float, q: int, kv: int, *, b: int = 1, h: int = 1) -> float:
    """Evaluate a score mod on the host (mods.jl:62)."""
    return float(m(s, b, h, q, kv))


def grad_shadow(x, *, feature_grads: bool = False):
    """Zeroed gradient accumulator for an array or a score mod (mods.jl:281-286; pair.jl:121-125 for the
    opt-in feature gradients of a PairFeatureScore)."""
    if isinstance(x, torch.Tensor):
        return torch.zeros_like(x)
    if isinstance(x, AliBiScore):
        return AliBiScore(torch.zeros_like(x.slopes))
    if isinstance(x, BiasScore):
        return BiasScore(torch.zeros_like(x.bias))
    if isinstance(x, ComposeScore):
        return ComposeScore(grad_shadow(x.a), grad_shadow(x.b))
    if isinstance(x, PairFeatureScore):
        fg = bool(feature_grads)
        return PairFeatureScore(x.op, torch.zeros_like(x.q_features) if fg else None,
                                torch.zeros_like(x.k_features) if fg else None, torch.zeros_like(x.pair_proj))
    return x


def _unsupported(what):
    raise TyloError(2, f"{what} is not supported by libtylo_b200 (there is no fallback)")


class _PrefixLM(MaskMod):
    """prefix_lm(len) = CausalMask() | PrefixMask(len) (mods.jl:178) kept as ONE term of a conjunction."""

    def __init__(self, length: int):
        self.len = int(length)

    def __call__(self, b, h, q, kv):
        return q >= kv or kv < self.len


_MAX_MASK_CLAUSES = 4


def _mask_clauses(x) -> list:
    """Disjunctive normal form of a mask tree: a list of conjunctions, each a list of atomic masks."""
    if x is None or isinstance(x, FullMask):
        return [[]]
    if isinstance(x, AndMask):
        return [a + b for a in _mask_clauses(x.a) for b in _mask_clauses(x.b)]
    if isinstance(x, OrMask):
        if {type(x.a), type(x.b)} == {CausalMask, PrefixMask}:
            return [[_PrefixLM(x.a.len if isinstance(x.a, PrefixMask) else x.b.len)]]
        return _mask_clauses(x.a) + _mask_clauses(x.b)
    return [[x]]


def _clause_desc(terms: list, keep: list) -> _MaskDesc:
    d = _MaskDesc()
    for x in terms:
        if isinstance(x, CausalMask):
            d.flags |= MASK_CAUSAL
        elif isinstance(x, SlidingWindowMask):
            if d.flags & MASK_SLIDING:
                d.window = min(d.window, x.w)
            else:
                d.flags |= MASK_SLIDING; d.window = x.w
        elif isinstance(x, PrefixMask):
            if d.flags & MASK_PREFIX:
                d.prefix_len = min(d.prefix_len, x.len)
            elif d.flags & MASK_PREFIX_LM:
                _unsupported("PrefixMask combined with prefix_lm in one conjunction")
            else:
                d.flags |= MASK_PREFIX; d.prefix_len = x.len
        elif isinstance(x, _PrefixLM):
            if d.flags & (MASK_PREFIX | MASK_PREFIX_LM):
                _unsupported("prefix_lm combined with another prefix term in one conjunction")
            d.flags |= MASK_PREFIX_LM; d.prefix_len = x.len
        elif isinstance(x, DocumentMask):
            if d.flags & MASK_DOCUMENT:
                _unsupported("more than one DocumentMask in one conjunction")
            dq, dk = x.doc_q, x.doc_kv
            if dq.dtype != torch.int32 or dk.dtype != torch.int32:
                raise TypeError("DocumentMask ids must be int32")
            _dense(dq, dk)
            if dq.dim() != dk.dim() or dq.dim() not in (1, 2):
                raise ValueError("DocumentMask ids must both be vectors or both be (B, S) tables")
            d.flags |= MASK_DOCUMENT
            d.doc_q, d.doc_kv = dq.data_ptr(), dk.data_ptr()
            d.doc_q_len, d.doc_kv_len = dq.shape[-1], dk.shape[-1]
            if dq.dim() == 2:
                if dq.shape != dk.shape:
                    raise ValueError("per-batch DocumentMask tables must have one shape")
                d.doc_batch_stride = dq.shape[-1]
            keep.extend([dq, dk])
        else:
            _unsupported(f"mask mod {type(x).__name__}")
    return d


def _mask_desc(m: Optional[MaskMod], keep: list) -> Optional[_MaskDesc]:
    """Mask tree -> chain of conjunction descriptors linked through ``or_next`` (AndMask / OrMask,
    mods.jl:151-167).  One conjunction (the common case) runs on every kernel; several run on the
    fp32-arithmetic kernels."""
    clauses = _mask_clauses(m)
    if len(clauses) > _MAX_MASK_CLAUSES:
        _unsupported(f"a mask with {len(clauses)} OR-ed conjunctions (at most {_MAX_MASK_CLAUSES})")
    descs = [_clause_desc(c, keep) for c in clauses]
    for a, b in zip(descs, descs[1:]):
        a.or_next = ctypes.addressof(b)
    keep.extend(descs)
    return descs[0]


def _score_desc(m: Optional[ScoreMod], dm, keep: list) -> _ScoreDesc:
    d = _ScoreDesc()
    chain = []

    def walk(x, dx):
        if x is None or isinstance(x, NoOpScore):
            return
        if isinstance(x, ComposeScore):
            walk(x.a, None if dx is None else dx.a); walk(x.b, None if dx is None else dx.b); return
        chain.append((x, dx))

    walk(m, dm)
    # The additive mods (ALiBi, bias) share one place in the chain: all before or all after the soft cap.
    caps = [i for i, (x, _) in enumerate(chain) if isinstance(x, SoftCapScore)]
    adds = [i for i, (x, _) in enumerate(chain) if isinstance(x, (AliBiScore, BiasScore))]
    if caps and adds and not (max(adds) < caps[0] or min(adds) > caps[0]):
        _unsupported("additive score mods on both sides of a SoftCapScore")
    for i, (x, dx) in enumerate(chain):
        if isinstance(x, SoftCapScore):
            if d.flags & SCORE_SOFTCAP:
                _unsupported("more than one SoftCapScore")
            d.flags |= SCORE_SOFTCAP; d.cap = x.cap
            if adds and min(adds) > i:
                d.flags |= SCORE_SOFTCAP_FIRST
        elif isinstance(x, BiasScore):
            if d.flags & SCORE_BIAS:
                _unsupported("more than one BiasScore")
            if x.bias.dtype != torch.float32:
                raise TypeError("BiasScore bias must be float32")
            _dense(x.bias)
            d.flags |= SCORE_BIAS; d.bias = x.bias.data_ptr(); keep.append(x.bias)
            d.bias_batch, d.bias_heads = int(x.bias.shape[0]), int(x.bias.shape[1])
            d._bias_shape = tuple(x.bias.shape[2:])
            if dx is not None:
                _dense(dx.bias)
                d.d_bias = dx.bias.data_ptr(); keep.append(dx.bias)
        elif isinstance(x, AliBiScore):
            if d.flags & SCORE_ALIBI:
                _unsupported("more than one AliBiScore")
            if x.slopes.dtype != torch.float32:
                raise TypeError("AliBiScore slopes must be float32")
            _dense(x.slopes)
            d.flags |= SCORE_ALIBI; d.slopes = x.slopes.data_ptr(); keep.append(x.slopes)
            if dx is not None:
                d.d_slopes = dx.slopes.data_ptr(); keep.append(dx.slopes)
        else:
            _unsupported(f"score mod {type(x).__name__}")
    return d


# ---------------------------------------------------------------------------------------------
# attention (src/attention/attention.jl)
# ---------------------------------------------------------------------------------------------
class AttnCheckpoints(NamedTuple):
    M: torch.Tensor
    L: torch.Tensor


class AttnScratch(NamedTuple):
    dO_scaled: Optional[torch.Tensor]   # the reference's Ō′ (kept for API shape; unused)
    Delta: torch.Tensor
    workspace: Optional[torch.Tensor]


def _attn_dims(Q, K, V, O=None):
    if Q.dim() != 4 or K.dim() != 4 or V.dim() != 4:
        raise ValueError("Q, K, V must be 4-D: (B, H, S, D)")
    B, H, Sq, Dq = Q.shape
    Bk, Hkv, Sk, Dk = K.shape
    Bv, Hv, Sv, Dv = V.shape
    assert Dq == Dk, "Q and K head dims differ"
    assert Sk == Sv, "K and V lengths differ"
    assert Hkv == Hv, "K and V head counts differ"
    assert B == Bk == Bv, "batch sizes differ"
    assert H % Hkv == 0, "Heads must be a multiple of Heads_KV"
    if O is not None:
        assert tuple(O.shape) == (B, H, Sq, Dv), "O has the wrong shape"
    if not (Q.dtype == K.dtype == V.dtype):
        raise TypeError("Q, K, V must share one element type")
    return B, H, Hkv, Sq, Sk, Dk, Dv


def allocate_checkpoints_attention(Q, K, V) -> AttnCheckpoints:
    """allocate_checkpoints(attention!, Q, K, V) (attention.jl:271-273): fp32 (B, H, Sq)."""
    B, H, Sq, _ = Q.shape
    return AttnCheckpoints(torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device),
                           torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device))


def allocate_scratchspace_grad_attention(Q, K, V, O) -> AttnScratch:
    """allocate_scratchspace(∇attention!, Q, K, V, O) (attention.jl:367-370) plus the
    library's own workspace."""
    B, H, Hkv, Sq, Sk, Dk, Dv = _attn_dims(Q, K, V, O)
    nbytes = int(_lib.tylo_b200_attention_bwd_workspace_bytes(Dk, Dv, Sq, Sk, H, Hkv, B, _dtype(Q)))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=Q.device) if nbytes > 0 else None
    return AttnScratch(None, torch.empty(B, H, Sq, dtype=torch.float32, device=Q.device), ws)


def attention_(O, Q, K, V, *, causal=False, input_pos=0, k_lengths=None, q_lengths=None, checkpoints=None,
               tensorcore=None):
    """attention!(O, Q, K, V; ...) (attention.jl:219-262).  Returns None.  `tensorcore=TFloat32` on Float32
    arrays: products on the tensor cores with TF32 operands (head dims up to 64); default true fp32."""
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    B, H, Hkv, Sq, Sk, Dk, Dv = _attn_dims(pQ, pK, pV, pO)
    _dense(pO, pQ, pK, pV, k_lengths, q_lengths)
    M = None if checkpoints is None else checkpoints.M
    L = None if checkpoints is None else checkpoints.L
    _check(_lib.tylo_b200_attention_fwd(_p(pO), _p(pQ), _p(pK), _p(pV), _p(M), _p(L), _p(k_lengths), _p(q_lengths),
                                        Dk, Dv, Sq, Sk, H, Hkv, B, int(input_pos), int(bool(causal)),
                                        _fwd_dtype(pQ, tensorcore), _stream()))


def attention(Q, K, V, **kw):
    """attention(Q, K, V; ...) -> O (attention.jl:281-285)."""
    O = torch.empty(Q.shape[0], Q.shape[1], Q.shape[2], V.shape[3], dtype=Q.dtype, device=Q.device)
    attention_(O, Q, K, V, **kw)
    return O


def grad_attention_(O: Duplicated, Q: Duplicated, K: Duplicated, V: Duplicated, *, causal, checkpoints,
                    input_pos=0, k_lengths=None, q_lengths=None, scratch=None):
    """∇attention!(O, Q, K, V; causal, checkpoints, scratch) (attention.jl:297-357)."""
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    B, H, Hkv, Sq, Sk, Dk, Dv = _attn_dims(pQ, pK, pV, pO)
    if scratch is None:
        scratch = allocate_scratchspace_grad_attention(pQ, pK, pV, pO)
    dO = shadow(O)
    _dense(pO, pQ, pK, pV, dO, Q.shadow, K.shadow, V.shadow)
    ws = scratch.workspace
    _check(_lib.tylo_b200_attention_bwd(_p(Q.shadow), _p(K.shadow), _p(V.shadow), _p(pQ), _p(pK), _p(pV), _p(pO),
                                        _p(dO), _p(checkpoints.M), _p(checkpoints.L), _p(scratch.dO_scaled),
                                        _p(scratch.Delta), _p(ws), 0 if ws is None else ws.numel(),
                                        _p(k_lengths), _p(q_lengths), Dk, Dv, Sq, Sk, H, Hkv, B, int(input_pos),
                                        int(bool(causal)), _dtype(pQ), _stream()))


def grad_attention(dO, Q, K, V, O, *, checkpoints, causal, **kw):
    """∇attention(Ō, Q, K, V, O; checkpoints, causal) -> (Q̄, K̄, V̄) (attention.jl:379-388)."""
    Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
    grad_attention_(Duplicated(O, dO), Qd, Kd, Vd, checkpoints=checkpoints, causal=causal, **kw)
    return Qd.shadow, Kd.shadow, Vd.shadow


# ---------------------------------------------------------------------------------------------
# flex attention (src/attention/flex.jl)
# ---------------------------------------------------------------------------------------------
allocate_checkpoints_flex_attention = allocate_checkpoints_attention       # flex.jl:391-393
allocate_scratchspace_grad_flex_attention = allocate_scratchspace_grad_attention  # flex.jl:519-522


def _check_bias_shape(sd: _ScoreDesc, Sq: int, Sk: int) -> None:
    shape = getattr(sd, "_bias_shape", None)
    if shape is not None and shape != (Sq, Sk):
        raise ValueError(f"BiasScore bias covers {shape} (Sq, Sk) pairs but the call has ({Sq}, {Sk})")


def _check_block_mask(bm: BlockMask, Sq: int) -> None:
    for t in (bm.count, bm.idx, bm.full):
        if t.dtype != torch.int32:
            raise TypeError("BlockMask arrays must be int32")
    _dense(bm.count, bm.idx, bm.full)
    nqb = -(-Sq // bm.TILE_M)
    if bm.count.numel() != nqb or bm.idx.dim() != 2 or bm.idx.shape != bm.full.shape or bm.idx.shape[0] != nqb:
        raise ValueError(f"BlockMask was built for another shape: {nqb} query blocks of {bm.TILE_M} rows expected")


def flex_attention_(O, Q, K, V, *, score_mod=None, mask_mod=None, block_mask=None, block_sparse=True,
                    input_pos=0, qk_scale=None, checkpoints=None, tensorcore=None):
    """flex_attention!(O, Q, K, V; score_mod, mask_mod, ...) (flex.jl:312-383)."""
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    B, H, Hkv, Sq, Sk, Dk, Dv = _attn_dims(pQ, pK, pV, pO)
    _dense(pO, pQ, pK, pV)
    keep: list = []
    md = _mask_desc(mask_mod, keep)
    if _has_pairs(score_mod):
        score_mod = _lower_pairs(score_mod)           # pair features run as bias tables
    sd = _score_desc(score_mod, None, keep)
    _check_bias_shape(sd, Sq, Sk)
    M = None if checkpoints is None else checkpoints.M
    L = None if checkpoints is None else checkpoints.L
    if block_mask is not None:
        # flex.jl:347-360: walk the host-built block list instead of the analytic range
        bm = block_mask
        _check_block_mask(bm, Sq)
        _check(_lib.tylo_b200_flex_attention_fwd_block_mask(
            _p(pO), _p(pQ), _p(pK), _p(pV), _p(M), _p(L), ctypes.byref(md), ctypes.byref(sd), _p(bm.count), _p(bm.idx),
            _p(bm.full), int(bm.idx.shape[1]), int(bm.TILE_M), int(bm.TILE_N), Dk, Dv, Sq, Sk, H, Hkv, B,
            int(input_pos), 0.0 if qk_scale is None else float(qk_scale), _fwd_dtype(pQ, tensorcore), _stream()))
        return
    _check(_lib.tylo_b200_flex_attention_fwd(_p(pO), _p(pQ), _p(pK), _p(pV), _p(M), _p(L), ctypes.byref(md),
                                             ctypes.byref(sd), Dk, Dv, Sq, Sk, H, Hkv, B, int(input_pos),
                                             0.0 if qk_scale is None else float(qk_scale), int(bool(block_sparse)),
                                             _fwd_dtype(pQ, tensorcore), _stream()))


def flex_attention(Q, K, V, **kw):
    """flex_attention(Q, K, V; score_mod, mask_mod, ...) -> O (flex.jl:430-431)."""
    O = torch.empty(Q.shape[0], Q.shape[1], Q.shape[2], V.shape[3], dtype=Q.dtype, device=Q.device)
    flex_attention_(O, Q, K, V, **kw)
    return O


def grad_flex_attention_(O: Duplicated, Q: Duplicated, K: Duplicated, V: Duplicated, *, checkpoints,
                         score_mod=None, mask_mod=None, d_score_mod=None, block_mask=None, block_sparse=True,
                         input_pos=0, qk_scale=None, scratch=None):
    """∇flex_attention!(...; score_mod, mask_mod, ∂score_mod, checkpoints, scratch) (flex.jl:445-511).
    Extension: ``block_mask`` differentiates the block-list forward (the reference has no backward for it,
    flex.jl:193-194)."""
    pO, pQ, pK, pV = primal(O), primal(Q), primal(K), primal(V)
    B, H, Hkv, Sq, Sk, Dk, Dv = _attn_dims(pQ, pK, pV, pO)
    if scratch is None:
        scratch = allocate_scratchspace_grad_attention(pQ, pK, pV, pO)
    dO = shadow(O)
    _dense(pO, pQ, pK, pV, dO, Q.shadow, K.shadow, V.shadow)
    keep: list = []
    md = _mask_desc(mask_mod, keep)
    pair_mod, d_pair_mod = score_mod, d_score_mod
    if _has_pairs(score_mod):                         # pair features run as bias tables; gradients folded back below
        score_mod = _lower_pairs(pair_mod)
        d_score_mod = _lower_pair_shadows(score_mod, d_pair_mod)
    sd = _score_desc(score_mod, d_score_mod, keep)
    _check_bias_shape(sd, Sq, Sk)
    ws = scratch.workspace
    if block_mask is not None:
        bm = block_mask
        _check_block_mask(bm, Sq)
        _check(_lib.tylo_b200_flex_attention_bwd_block_mask(
            _p(Q.shadow), _p(K.shadow), _p(V.shadow), _p(pQ), _p(pK), _p(pV), _p(pO), _p(dO), _p(checkpoints.M),
            _p(checkpoints.L), _p(scratch.Delta), _p(ws), 0 if ws is None else ws.numel(), ctypes.byref(md),
            ctypes.byref(sd), _p(bm.count), _p(bm.idx), _p(bm.full), int(bm.idx.shape[1]), int(bm.TILE_M),
            int(bm.TILE_N), Dk, Dv, Sq, Sk, H, Hkv, B, int(input_pos), 0.0 if qk_scale is None else float(qk_scale),
            _dtype(pQ), _stream()))
        _raise_pair_grads(d_pair_mod, pair_mod, d_score_mod)
        return
    _check(_lib.tylo_b200_flex_attention_bwd(_p(Q.shadow), _p(K.shadow), _p(V.shadow), _p(pQ), _p(pK), _p(pV),
                                             _p(pO), _p(dO), _p(checkpoints.M), _p(checkpoints.L),
                                             _p(scratch.dO_scaled), _p(scratch.Delta), _p(ws),
                                             0 if ws is None else ws.numel(), ctypes.byref(md), ctypes.byref(sd),
                                             Dk, Dv, Sq, Sk, H, Hkv, B, int(input_pos),
                                             0.0 if qk_scale is None else float(qk_scale), int(bool(block_sparse)),
                                             _dtype(pQ), _stream()))
    _raise_pair_grads(d_pair_mod, pair_mod, d_score_mod)


def grad_flex_attention(dO, Q, K, V, O, *, checkpoints, **kw):
    """∇flex_attention(Ō, Q, K, V, O; checkpoints, ...) -> (Q̄, K̄, V̄) (flex.jl:530-539)."""
    Qd, Kd, Vd = Duplicated(Q), Duplicated(K), Duplicated(V)
    grad_flex_attention_(Duplicated(O, dO), Qd, Kd, Vd, checkpoints=checkpoints, **kw)
    return Qd.shadow, Kd.shadow, Vd.shadow


# ---------------------------------------------------------------------------------------------
# decode (src/attention/decode.jl)
# ---------------------------------------------------------------------------------------------
class DecodeScratch(NamedTuple):
    O_partial: torch.Tensor   # (n_splits, B, H, Dv) fp32
    M_partial: torch.Tensor   # (n_splits, B, H) fp32
    L_partial: torch.Tensor
    tickets: Optional[torch.Tensor] = None   # int32 counters of the one-launch form, zeroed once (the kernels put them back)


def decode_suggest_splits(Sk: int, Hkv: int, B: int) -> int:
    return int(_lib.tylo_b200_decode_suggest_splits(Sk, Hkv, B))


def allocate_scratchspace_decode_attention(O, Q, *, n_splits=8) -> DecodeScratch:
    """allocate_scratchspace(decode_attention!, O, Q; n_splits) (decode.jl:223-231)."""
    B, H, Dv = O.shape
    f = dict(dtype=torch.float32, device=O.device)
    # ticket words for any kv-head count up to H (the library indexes them by (kv head, batch))
    nt = int(_lib.tylo_b200_decode_ticket_count(int(n_splits), H, B))
    return DecodeScratch(torch.empty(n_splits, B, H, Dv, **f), torch.empty(n_splits, B, H, **f),
                         torch.empty(n_splits, B, H, **f), torch.zeros(max(nt, 1), dtype=torch.int32, device=O.device))


def _decode_dims(O, Q, K, V):
    B, H, Dq = Q.shape
    Bk, Hkv, Sk, Dk = K.shape
    Bv, Hv, Sv, Dv = V.shape
    assert Dq == Dk and Sk == Sv and Hkv == Hv and B == Bk == Bv and H % Hkv == 0
    if O is not None:
        assert tuple(O.shape) == (B, H, Dv)
    return B, H, Hkv, Sk, Dk, Dv


def decode_attention_(O, Q, K, V, *, lengths, n_splits=8, scratch=None, one_launch=True):
    """decode_attention!(O, Q, K, V; lengths, n_splits, scratch) -> O (decode.jl:158-212).
    ``n_splits=None`` asks the library for a count that fills the GPU.  With ``one_launch`` (and a scratch
    that carries ticket words) the split kernel also merges; otherwise split and merge are two launches as
    in the reference."""
    B, H, Hkv, Sk, Dk, Dv = _decode_dims(O, Q, K, V)
    if scratch is not None:
        n_splits = scratch.O_partial.shape[0]
    elif n_splits is None:
        n_splits = decode_suggest_splits(Sk, Hkv, B)
    if scratch is None:
        scratch = allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
    if lengths.dtype != torch.int32:
        raise TypeError("lengths must be int32")
    _dense(O, Q, K, V, lengths, *scratch)
    if one_launch and len(scratch) > 3 and scratch.tickets is not None:
        _check(_lib.tylo_b200_decode_attention_fused(_p(O), _p(Q), _p(K), _p(V), _p(lengths), _p(scratch.O_partial),
                                                     _p(scratch.M_partial), _p(scratch.L_partial), _p(scratch.tickets),
                                                     n_splits, Dk, Dv, Sk, H, Hkv, B, _dtype(Q), _stream()))
        return O
    _check(_lib.tylo_b200_decode_attention(_p(O), _p(Q), _p(K), _p(V), _p(lengths), _p(scratch.O_partial),
                                           _p(scratch.M_partial), _p(scratch.L_partial), n_splits, Dk, Dv, Sk, H,
                                           Hkv, B, _dtype(Q), _stream()))
    return O


def paged_decode_attention_(O, Q, K_pages, V_pages, *, block_table, lengths, n_splits=None, scratch=None):
    """decode_attention! over a paged KV cache: ``K_pages`` / ``V_pages`` are (n_pages, Hkv, page_size, D) pools
    (Julia's (D, page_size, Hkv, n_pages)), ``block_table`` an int32 (B, max_pages) tensor of page ids,
    ``lengths`` the live keys per sequence.  One launch."""
    B, H, Dk = Q.shape
    n_pages, Hkv, page_size, Dkp = K_pages.shape
    Dv = V_pages.shape[3]
    assert Dkp == Dk and tuple(V_pages.shape[:3]) == (n_pages, Hkv, page_size) and tuple(O.shape) == (B, H, Dv)
    assert block_table.dim() == 2 and block_table.shape[0] == B and H % Hkv == 0
    if block_table.dtype != torch.int32 or lengths.dtype != torch.int32:
        raise TypeError("block_table and lengths must be int32")
    max_pages = int(block_table.shape[1])
    if scratch is None:
        if n_splits is None:
            n_splits = decode_suggest_splits(page_size * max_pages, Hkv, B)
        scratch = allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
    _dense(O, Q, K_pages, V_pages, block_table, lengths, *scratch)
    _check(_lib.tylo_b200_decode_attention_paged(
        _p(O), _p(Q), _p(K_pages), _p(V_pages), _p(block_table), _p(lengths), _p(scratch.O_partial), _p(scratch.M_partial),
        _p(scratch.L_partial), _p(scratch.tickets), scratch.O_partial.shape[0], page_size, max_pages, Dk, Dv, H, Hkv, B,
        _dtype(Q), _stream()))
    return O


def decode_split_(Q, K, V, *, lengths, scratch: DecodeScratch):
    """First half of decode_attention! (mha_decode_split_fwd, decode.jl:187-199)."""
    B, H, Hkv, Sk, Dk, Dv = _decode_dims(None, Q, K, V)
    _dense(Q, K, V, lengths, *scratch)
    _check(_lib.tylo_b200_decode_split(_p(Q), _p(K), _p(V), _p(lengths), _p(scratch.O_partial),
                                       _p(scratch.M_partial), _p(scratch.L_partial), scratch.O_partial.shape[0],
                                       Dk, Dv, Sk, H, Hkv, B, _dtype(Q), _stream()))


def decode_combine_(O, O_partial, M_partial, L_partial, *, n_splits, o_stride, ml_stride, Dv, H, B,
                    merged: Optional[DecodeScratch] = None, dtype=None):
    """Second half (mha_decode_combine, decode.jl:201-209); also merges per-GPU partials."""
    dt = _dtype(O) if O is not None else (F32 if dtype is None else dtype)
    mo = mm = ml = None
    if merged is not None:
        mo, mm, ml = merged[:3]
    _check(_lib.tylo_b200_decode_combine(_p(O), _p(mo), _p(mm), _p(ml), _p(O_partial), _p(M_partial), _p(L_partial),
                                         int(n_splits), int(o_stride), int(ml_stride), Dv, H, B, dt, _stream()))


class DecodeExchange:
    """Receive buffers for decode with one sequence's KV cache sharded over the GPUs of a node.

    Each rank allocates one buffer through the library (cudaMalloc, zeroed), the CUDA IPC handles
    travel over ``group`` (any torch.distributed backend), and every rank maps all of them.
    ``exchange_`` then merges this rank's split partials with every peer's in one launch over
    NVLink.  With ``group=None`` the object is a single-rank exchange (world 1).  The merge algebra
    is the reference's (mha_decode_combine, decode.jl:119-140); the reference itself is single-GPU.
    """

    def __init__(self, B: int, H: int, Dv: int, *, group=None, rank: int = 0, world: int = 1, timeout_us: int = 0):
        self.B, self.H, self.Dv, self.rank, self.world = B, H, Dv, rank, world
        self.timeout_us = int(timeout_us)
        self.nbytes = int(_lib.tylo_b200_decode_exchange_bytes(world, Dv, H, B))
        if self.nbytes <= 0:
            raise TyloError(1, f"decode exchange: unsupported extents (world={world}, Dv={Dv}, H={H}, B={B})")
        own = c_void_p()
        _check(_lib.tylo_b200_peer_alloc(ctypes.byref(own), self.nbytes))
        self._own = own
        self._opened = []
        ptrs = [None] * world
        ptrs[rank] = own.value
        if world > 1:
            import torch.distributed as dist
            hb = int(_lib.tylo_b200_peer_handle_bytes())
            handle = ctypes.create_string_buffer(hb)
            _check(_lib.tylo_b200_peer_export(own, handle))
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r in range(world):
                if r == rank:
                    continue
                p = c_void_p()
                _check(_lib.tylo_b200_peer_open(ctypes.byref(p), ctypes.create_string_buffer(handles[r], hb)))
                self._opened.append(p)
                ptrs[r] = p.value
            dist.barrier(group=group)       # every buffer is zeroed and mapped before the first launch
        self._peers = (c_void_p * world)(*ptrs)

    @classmethod
    def local_group(cls, B: int, H: int, Dv: int, *, world: int, timeout_us: int = 0):
        """``world`` exchange objects inside ONE process on the current GPU, wired to each other's buffers:
        one process driving several shards in turn.  A rank whose peers have not pushed yet gives up
        after ``timeout_us``; a rank called after all its peers finds their records and completes."""
        nbytes = int(_lib.tylo_b200_decode_exchange_bytes(world, Dv, H, B))
        if nbytes <= 0:
            raise TyloError(1, f"decode exchange: unsupported extents (world={world}, Dv={Dv}, H={H}, B={B})")
        bufs = []
        for _ in range(world):
            p = c_void_p()
            _check(_lib.tylo_b200_peer_alloc(ctypes.byref(p), nbytes))
            bufs.append(p)
        out = []
        for r in range(world):
            x = object.__new__(cls)
            x.B, x.H, x.Dv, x.rank, x.world, x.timeout_us, x.nbytes = B, H, Dv, r, world, int(timeout_us), nbytes
            x._own, x._opened = bufs[r], []
            x._peers = (c_void_p * world)(*[b.value for b in bufs])
            out.append(x)
        return out

    def exchange_(self, O, scratch: "DecodeScratch"):
        """Merges ``scratch`` (this rank's split partials) across all ranks into O (B, H, Dv)."""
        n_splits = scratch.O_partial.shape[0]
        B, H, Dv = self.B, self.H, self.Dv
        assert tuple(O.shape) == (B, H, Dv) and tuple(scratch.O_partial.shape[1:]) == (B, H, Dv)
        _dense(O, *scratch)
        _check(_lib.tylo_b200_decode_exchange(_p(O), _p(scratch.O_partial), _p(scratch.M_partial),
                                              _p(scratch.L_partial), n_splits, B * H * Dv, B * H, self._peers,
                                              self.rank, self.world, Dv, H, B, _dtype(O), self.timeout_us,
                                              _stream()))
        return O

    def status(self) -> int:
        """Synchronises; 0 if every wait of the calls so far was served, else raises TyloError (status 6)."""
        code = c_int32(0)
        _check(_lib.tylo_b200_decode_exchange_status(self._own, ctypes.byref(code)))
        return int(code.value)

    def close(self):
        for p in self._opened:
            _lib.tylo_b200_peer_close(p)
        self._opened = []
        if self._own is not None:
            _lib.tylo_b200_peer_free(self._own)
            self._own = None


SHARDED_DECODE_LAUNCHES = 2      # kernels per sharded decode step (split, exchange)


def sharded_decode_attention_(O, Q, K_local, V_local, *, lengths_local, exchange: DecodeExchange, scratch,
                              one_launch=False):
    """decode_attention! with the keys of every sequence sharded over ranks (``lengths_local`` = live keys
    inside this rank's range).  Default: the split kernel, then the exchange kernel, which is placed while the
    splits still run (programmatic dependent launch) and merges every head in a CTA of its own — measured
    faster than the one-launch form at 2 and 8 GPUs (108 us against 123 us per step at 8).
    ``one_launch=True``: the split kernel's last CTA per (kv head, batch) merges the local splits, pushes the
    records to every peer and merges theirs."""
    if not (one_launch and len(scratch) > 3 and scratch.tickets is not None):
        decode_split_(Q, K_local, V_local, lengths=lengths_local, scratch=scratch)
        return exchange.exchange_(O, scratch)
    B, H, Hkv, Sk, Dk, Dv = _decode_dims(O, Q, K_local, V_local)
    _dense(O, Q, K_local, V_local, lengths_local, *scratch)
    _check(_lib.tylo_b200_decode_attention_sharded(
        _p(O), _p(Q), _p(K_local), _p(V_local), _p(lengths_local), _p(scratch.O_partial), _p(scratch.M_partial),
        _p(scratch.L_partial), _p(scratch.tickets), scratch.O_partial.shape[0], exchange._peers, exchange.rank,
        exchange.world, Dk, Dv, Sk, H, Hkv, B, _dtype(Q), exchange.timeout_us, _stream()))
    return O


# ---------------------------------------------------------------------------------------------
# softmax (src/softmax/softmax.jl)
# ---------------------------------------------------------------------------------------------
def _mn(X):
    if X.dim() != 2:
        raise ValueError("expected a matrix (N, M)")
    return X.shape[1], X.shape[0]


def softmax_(Y, X):
    """softmax!(Y, X) (softmax.jl:96-105)."""
    pY, pX = primal(Y), primal(X)
    M, N = _mn(pX)
    assert pY.shape == pX.shape and pY.dtype == pX.dtype
    _dense(pY, pX)
    _check(_lib.tylo_b200_softmax_fwd(_p(pY), _p(pX), M, N, _dtype(pX), _stream()))


def softmax(X):
    Y = torch.empty_like(X)
    softmax_(Y, X)
    return Y


def grad_softmax_(Y: Duplicated, X: Duplicated):
    """∇softmax!(Y, X) (softmax.jl:127-136): X.shadow = y ∘ (ȳ − Σ y∘ȳ)."""
    M, N = _mn(Y.primal)
    _dense(Y.primal, Y.shadow, X.shadow)
    _check(_lib.tylo_b200_softmax_bwd(_p(X.shadow), _p(Y.shadow), _p(Y.primal), M, N, _dtype(Y.primal), _stream()))


def grad_softmax(dY, Y):
    """∇softmax(Ȳ, Y) -> X̄ (softmax.jl:144-148)."""
    Xd = Duplicated(Y, torch.empty_like(Y))
    grad_softmax_(Duplicated(Y, dY), Xd)
    return Xd.shadow


# ---------------------------------------------------------------------------------------------
# RMSNorm / LayerNorm (src/norm/*.jl)
# ---------------------------------------------------------------------------------------------
class RmsCheckpoints(NamedTuple):
    Rstd: torch.Tensor


class LnCheckpoints(NamedTuple):
    Mean: torch.Tensor
    Rstd: torch.Tensor


class RmsScratch(NamedTuple):
    dW_partial: torch.Tensor   # (n_groups, M) fp32


class LnScratch(NamedTuple):
    dW_partial: torch.Tensor
    dB_partial: torch.Tensor


DEFAULT_N_GROUPS = 296   # two CTAs per SM; the reference's default of 64 leaves most SMs idle


def allocate_checkpoints_rms_norm(X, W) -> RmsCheckpoints:
    return RmsCheckpoints(torch.empty(X.shape[0], dtype=torch.float32, device=X.device))


def allocate_checkpoints_layer_norm(X, W, B) -> LnCheckpoints:
    f = dict(dtype=torch.float32, device=X.device)
    return LnCheckpoints(torch.empty(X.shape[0], **f), torch.empty(X.shape[0], **f))


def allocate_scratchspace_grad_rms_norm(X, W, *, N_GROUPS=DEFAULT_N_GROUPS) -> RmsScratch:
    return RmsScratch(torch.empty(N_GROUPS, X.shape[1], dtype=torch.float32, device=X.device))


def allocate_scratchspace_grad_layer_norm(X, W, B, *, N_GROUPS=DEFAULT_N_GROUPS) -> LnScratch:
    f = dict(dtype=torch.float32, device=X.device)
    return LnScratch(torch.empty(N_GROUPS, X.shape[1], **f), torch.empty(N_GROUPS, X.shape[1], **f))


def rms_norm_(Y, X, W, *, eps, offset=0.0, checkpoints=None):
    """rms_norm!(Y, X, W; eps, offset, checkpoints) (rms_norm.jl:115-128)."""
    pY, pX, pW = primal(Y), primal(X), primal(W)
    M, N = _mn(pX)
    assert pY.shape == pX.shape and pW.shape == (M,)
    _dense(pY, pX, pW)
    R = None if checkpoints is None else checkpoints.Rstd
    _check(_lib.tylo_b200_rms_norm_fwd(_p(pY), _p(pX), _p(pW), _p(R), M, N, float(eps), float(offset), _dtype(pX),
                                       _stream()))


def rms_norm(X, W, *, eps, offset=0.0, **kw):
    Y = torch.empty_like(X)
    rms_norm_(Y, X, W, eps=eps, offset=offset, **kw)
    return Y


def grad_rms_norm_(Y: Duplicated, X: Duplicated, W: Duplicated, *, checkpoints, offset=0.0, scratch=None):
    """∇rms_norm!(Y, X, W; checkpoints, scratch, offset) (rms_norm.jl:162-185)."""
    pX, pW = primal(X), primal(W)
    M, N = _mn(pX)
    if scratch is None:
        scratch = allocate_scratchspace_grad_rms_norm(pX, pW)
    _dense(pX, pW, Y.shadow, X.shadow, W.shadow, scratch.dW_partial)
    _check(_lib.tylo_b200_rms_norm_bwd(_p(X.shadow), _p(W.shadow), _p(Y.shadow), _p(pX), _p(pW),
                                       _p(checkpoints.Rstd), _p(scratch.dW_partial), scratch.dW_partial.shape[0],
                                       M, N, float(offset), _dtype(pX), _stream()))


def grad_rms_norm(dY, X, W, *, checkpoints, offset=0.0, **kw):
    """∇rms_norm(Ȳ, X, W; checkpoints, offset) -> (X̄, W̄) (rms_norm.jl:206-220)."""
    Xd, Wd = Duplicated(X), Duplicated(W)
    grad_rms_norm_(Duplicated(dY, dY), Xd, Wd, checkpoints=checkpoints, offset=offset, **kw)
    return Xd.shadow, Wd.shadow


def layer_norm_(Y, X, W, B, *, eps, checkpoints=None):
    """layer_norm!(Y, X, W, B; eps, checkpoints) (layer_norm.jl:157-173)."""
    pY, pX, pW, pB = primal(Y), primal(X), primal(W), primal(B)
    M, N = _mn(pX)
    assert pY.shape == pX.shape and pW.shape == (M,) and pB.shape == (M,)
    _dense(pY, pX, pW, pB)
    Mean = None if checkpoints is None else checkpoints.Mean
    R = None if checkpoints is None else checkpoints.Rstd
    _check(_lib.tylo_b200_layer_norm_fwd(_p(pY), _p(pX), _p(pW), _p(pB), _p(Mean), _p(R), M, N, float(eps),
                                         _dtype(pX), _stream()))


def layer_norm(X, W, B, *, eps, **kw):
    Y = torch.empty_like(X)
    layer_norm_(Y, X, W, B, eps=eps, **kw)
    return Y


def grad_layer_norm_(Y: Duplicated, X: Duplicated, W: Duplicated, B: Duplicated, *, checkpoints, scratch=None):
    """∇layer_norm!(Y, X, W, B; checkpoints, scratch) (layer_norm.jl:207-230)."""
    pX, pW = primal(X), primal(W)
    M, N = _mn(pX)
    if scratch is None:
        scratch = allocate_scratchspace_grad_layer_norm(pX, pW, primal(B))
    _dense(pX, pW, Y.shadow, X.shadow, W.shadow, B.shadow, *scratch)
    _check(_lib.tylo_b200_layer_norm_bwd(_p(X.shadow), _p(W.shadow), _p(B.shadow), _p(Y.shadow), _p(pX), _p(pW),
                                         _p(checkpoints.Mean), _p(checkpoints.Rstd), _p(scratch.dW_partial),
                                         _p(scratch.dB_partial), scratch.dW_partial.shape[0], M, N, _dtype(pX),
                                         _stream()))


def grad_layer_norm(dY, X, W, B, *, checkpoints, **kw):
    """∇layer_norm(Ȳ, X, W, B; checkpoints) -> (X̄, W̄, B̄) (layer_norm.jl:253-268)."""
    Xd, Wd, Bd = Duplicated(X), Duplicated(W), Duplicated(B)
    grad_layer_norm_(Duplicated(dY, dY), Xd, Wd, Bd, checkpoints=checkpoints, **kw)
    return Xd.shadow, Wd.shadow, Bd.shadow
