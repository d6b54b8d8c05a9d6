"""Host-side partitioning for one 8-GPU box: what each rank owns, and the packed partial that
crosses NVLink in the sharded decode.  Pure Python/torch: no device work happens here, so the same
code runs under gloo on CPU ranks in the tests and under NCCL on GPUs in the benchmark.

The shardings (the reference itself is single-GPU):
  * prefill forward/backward: (kv-head, batch) units are independent -> contiguous ranges, no exchange;
  * long-context decode: contiguous key ranges -> one all-gather of (O, max, sum) partials, then the
    same log-sum-exp merge the split kernel's combine uses (src/attention/decode.jl:119-140);
  * long-context decode the other way: KV heads divided over the ranks, every rank keeps all keys of its heads
    and writes the output of their query heads -> nothing crosses NVLink."""
from __future__ import annotations

from typing import NamedTuple, Tuple


def unit_range(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced [begin, end) of `n_units` independent units for `rank`."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(n_units, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def prefill_shard(Hkv: int, B: int, rank: int, world: int):
    """(kv-head, batch) units of the prefill owned by `rank`, as a list of (b, hk_begin, hk_end)
    slabs; the G query heads of a kv head travel with it.  Units are ordered batch-major like the
    arrays ([b][h][s][d]), so each slab is contiguous in memory."""
    lo, hi = unit_range(Hkv * B, rank, world)
    slabs = []
    u = lo
    while u < hi:
        b, hk = divmod(u, Hkv)
        take = min(hi - u, Hkv - hk)
        slabs.append((b, hk, hk + take))
        u += take
    return slabs


def kv_shard(Sk: int, rank: int, world: int, align: int = 128) -> Tuple[int, int]:
    """Key range of the decode cache owned by `rank`: contiguous, aligned to `align` keys except at
    the end of the cache."""
    per = -(-Sk // world)
    per = -(-per // align) * align
    begin = min(rank * per, Sk)
    return begin, min(begin + per, Sk)


def head_shard(Hkv: int, G: int, rank: int, world: int):
    """Decode with the KV heads divided over the ranks (no exchange: the ranks' outputs are disjoint query heads):
    returns (kv_head_begin, kv_head_end, query_head_begin, query_head_end) of `rank`.  The G query heads of a KV head
    stay with it; `Hkv` must divide evenly, so that every rank streams the same number of bytes."""
    if Hkv % world != 0:
        raise ValueError(f"{Hkv} KV heads do not divide over {world} ranks")
    lo, hi = unit_range(Hkv, rank, world)
    return lo, hi, lo * G, hi * G


def local_lengths(lengths, begin: int, end: int):
    """Valid keys of each sequence inside [begin, end) (works on torch tensors and numpy arrays)."""
    return (lengths - begin).clip(0, end - begin)


class PackedPartial(NamedTuple):
    """Offsets (in fp32 elements) inside the per-rank buffer that is all-gathered."""
    o: int
    m: int
    l: int
    size: int


def packed_layout(B: int, H: int, Dv: int) -> PackedPartial:
    n = B * H * Dv
    return PackedPartial(0, n, n + B * H, n + 2 * B * H)
