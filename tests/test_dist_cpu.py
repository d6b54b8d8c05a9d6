"""CPU, world size 2 over gloo: the multi-GPU host logic — partitioning, the packed partial that is
all-gathered in the sharded decode, and the merge algebra (checked with the oracle)."""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


sharding = _load("tylo_b200_sharding", ROOT / "tylo.jl_b200" / "sharding.py")


def test_partitions_tile_the_work():
    for n, w in ((32, 1), (32, 8), (7, 4), (3, 8)):
        cover = []
        for r in range(w):
            lo, hi = sharding.unit_range(n, r, w)
            cover += list(range(lo, hi))
        assert cover == list(range(n))
    # config 3: 8 kv heads x 4 batches over 8 GPUs -> 4 kv heads of one batch each
    assert sharding.prefill_shard(8, 4, 3, 8) == [(1, 4, 8)]
    assert sharding.prefill_shard(8, 4, 0, 1) == [(0, 0, 8), (1, 0, 8), (2, 0, 8), (3, 0, 8)]
    # config 5b: 1,048,576 keys over 8 GPUs
    assert [sharding.kv_shard(1 << 20, r, 8) for r in (0, 7)] == [(0, 131072), (917504, 1048576)]
    assert [sharding.head_shard(8, 8, r, 4) for r in (0, 3)] == [(0, 2, 0, 16), (6, 8, 48, 64)]
    with pytest.raises(ValueError):
        sharding.head_shard(8, 8, 0, 3)
    spans = [sharding.kv_shard(1000, r, 3) for r in range(3)]
    assert spans[0][0] == 0 and spans[-1][1] == 1000 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        sharding.unit_range(4, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle = _load("tylo_oracle", ROOT / "oracle" / "tylo_oracle.py")
    rng = np.random.default_rng(4)                       # same inputs on every rank (q is replicated)
    B, H, Hkv, Sk, D = 2, 8, 2, 700, 16
    Q = rng.standard_normal((B, H, D)); K = rng.standard_normal((B, Hkv, Sk, D)); V = rng.standard_normal((B, Hkv, Sk, D))
    lengths = np.array([700, 150])
    begin, end = sharding.kv_shard(Sk, rank, world)
    O, M, L = oracle.decode_partials(Q, K, V, lengths, begin, end)       # what the rank's GPU would produce
    lay = sharding.packed_layout(B, H, D)
    pack = torch.zeros(lay.size, dtype=torch.float64)
    pack[lay.o:lay.m] = torch.from_numpy(O.reshape(-1)); pack[lay.m:lay.l] = torch.from_numpy(M.reshape(-1))
    pack[lay.l:] = torch.from_numpy(L.reshape(-1))
    gathered = torch.zeros(world * lay.size, dtype=torch.float64)
    dist.all_gather_into_tensor(gathered, pack)
    g = gathered.view(world, lay.size).numpy()
    merged = oracle.decode_combine(g[:, lay.o:lay.m].reshape(world, B, H, D), g[:, lay.m:lay.l].reshape(world, B, H),
                                   g[:, lay.l:].reshape(world, B, H))
    ref = oracle.decode_reference(Q, K, V, lengths)
    ll = sharding.local_lengths(lengths, begin, end)
    ok = np.allclose(merged, ref, rtol=1e-12, atol=1e-14) and int(ll.sum()) == int(np.clip(lengths - begin, 0, end - begin).sum())
    out[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_decode_merge_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = 29500 + os.getpid() % 2000
        procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(out) == {0: True, 1: True}
