"""Counter-based synthetic inputs: element `i` of tensor `t` under seed `s` is a pure function of
(s, t, i), bit-identical on the CPU (NumPy) and on the GPU (torch), independent of how the tensor is
sharded or in which order it is filled.

A 64-bit mix of (seed, tensor id, linear index) picks one of 65,536 equally likely standard-normal
quantiles (a table built once on the CPU in float64 and rounded to float32); only integer arithmetic
and a table look-up are involved, so both sides agree to the bit.  The linear index is the
column-major index of the Julia array = the C-order index of the reversed-axes tensor used here.

    x = normal_cuda(seed, tensor_id, shape, dtype)          # whole tensor, on the current device
    x = normal_numpy(seed, tensor_id, start, stop)          # float32 values of elements [start, stop)
    idx = integers_numpy / integers_cuda (...)              # uniform integers in [lo, hi]
"""
from __future__ import annotations

import numpy as np

_TABLE_BITS = 16
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB
_GOLD = 0x9E3779B97F4A7C15
_MASK64 = (1 << 64) - 1
_table_np = None
_table_cuda = {}


def quantile_table() -> np.ndarray:
    """65,536 standard-normal quantiles at the mid-points (k + 1/2) / 65,536, float32."""
    global _table_np
    if _table_np is None:
        import torch
        p = (torch.arange(1 << _TABLE_BITS, dtype=torch.float64) + 0.5) / float(1 << _TABLE_BITS)
        _table_np = torch.special.ndtri(p).to(torch.float32).numpy()       # always on the CPU: one source of truth
    return _table_np


def _key(seed: int, tensor_id: int) -> int:
    return ((int(seed) + 1) * _GOLD + (int(tensor_id) + 1) * _M2) & _MASK64


def _mix_numpy(key: int, idx: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = idx.astype(np.uint64) * np.uint64(_GOLD) + np.uint64(key)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
        return z ^ (z >> np.uint64(31))


def _signed(c: int) -> int:
    return c - (1 << 64) if c >= (1 << 63) else c


def _lsr(z, s: int):
    """Logical right shift of int64 torch values (torch's >> is arithmetic)."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix_cuda(key: int, idx):
    z = idx * _signed(_GOLD) + _signed(key)           # int64 arithmetic wraps like uint64
    z = (z ^ _lsr(z, 30)) * _signed(_M1)
    z = (z ^ _lsr(z, 27)) * _signed(_M2)
    return z ^ _lsr(z, 31)


def normal_numpy(seed: int, tensor_id: int, start: int, stop: int) -> np.ndarray:
    """float32 N(0,1) values of elements [start, stop) of tensor `tensor_id` under `seed`."""
    h = _mix_numpy(_key(seed, tensor_id), np.arange(start, stop, dtype=np.uint64))
    return quantile_table()[(h >> np.uint64(64 - _TABLE_BITS)).astype(np.int64)]


def integers_numpy(seed: int, tensor_id: int, start: int, stop: int, lo: int, hi: int) -> np.ndarray:
    """Uniform integers in [lo, hi] (int64) for elements [start, stop)."""
    h = _mix_numpy(_key(seed, tensor_id), np.arange(start, stop, dtype=np.uint64))
    return (lo + ((h >> np.uint64(33)) % np.uint64(hi - lo + 1)).astype(np.int64))


def normal_cuda(seed: int, tensor_id: int, shape, dtype, *, scale: float = 1.0, shift: float = 0.0, start: int = 0,
                device="cuda", chunk: int = 1 << 25):
    """Tensor of `shape` whose flat element j is element `start + j` of the stream, as
    `(value * scale + shift)` rounded to `dtype`; filled in chunks to bound temporary memory."""
    import torch
    dev = torch.device(device)
    tab = _table_cuda.get(dev)
    if tab is None:
        tab = _table_cuda[dev] = torch.from_numpy(quantile_table()).to(dev)
    n = int(np.prod(shape))
    out = torch.empty(n, dtype=dtype, device=dev)
    key = _key(seed, tensor_id)
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        idx = torch.arange(start + a, start + b, dtype=torch.int64, device=dev)
        v = tab[_lsr(_mix_cuda(key, idx), 64 - _TABLE_BITS)]
        if scale != 1.0 or shift != 0.0:
            v = v * scale + shift
        out[a:b] = v.to(dtype)
    return out.view(*shape)


def integers_cuda(seed: int, tensor_id: int, n: int, lo: int, hi: int, *, device="cuda"):
    import torch
    idx = torch.arange(n, dtype=torch.int64, device=torch.device(device))
    return lo + _lsr(_mix_cuda(_key(seed, tensor_id), idx), 33) % (hi - lo + 1)


def rounded_numpy(seed: int, tensor_id: int, start: int, stop: int, dtype, *, scale: float = 1.0, shift: float = 0.0) -> np.ndarray:
    """What `normal_cuda(..., dtype)` holds in elements [start, stop), upcast to float64 (the oracle's
    input): the same float32 arithmetic and the same rounding to the storage type."""
    import torch
    v = torch.from_numpy(normal_numpy(seed, tensor_id, start, stop))
    if scale != 1.0 or shift != 0.0:
        v = v * scale + shift
    return v.to(dtype).to(torch.float64).numpy()
