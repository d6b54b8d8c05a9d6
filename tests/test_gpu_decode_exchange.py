"""GPU parity: decode with one sequence's keys sharded over ranks, merged by the one-launch peer
exchange.  The oracle is the plain-array decode reference over the whole key range
(test/decode.jl:15-36): sharding must not change the result.

On one GPU the ranks of a group are driven in turn from this process.  A rank that runs before its
peers have pushed meets the bounded wait: it must give up within its time limit, report status 6
and leave the context usable.  A rank that runs after its peers must complete with the full merge.
With two or more GPUs a second test runs real ranks as child processes over CUDA IPC buffers."""
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import check, draw

pytestmark = pytest.mark.gpu


def _shard(t, K, V, lengths, r, world):
    Sk = K.shape[2]
    per = Sk // world
    b, e = r * per, (Sk if r == world - 1 else (r + 1) * per)
    ll = torch.tensor([min(max(n - b, 0), e - b) for n in lengths], dtype=torch.int32, device="cuda")
    return K[:, :, b:e].contiguous(), V[:, :, b:e].contiguous(), ll


@pytest.mark.parametrize("one_launch", [True, False], ids=["one-launch", "two-launch"])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_single_rank_exchange_equals_decode(tylo, oracle, dt, one_launch):
    rng = np.random.default_rng(3)
    B, H, Hkv, Sk, D = 2, 16, 4, 1024, 128
    Q, Q64 = draw(rng, (B, H, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    lengths = [1024, 700]
    ln = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    ex = tylo.DecodeExchange(B, H, D)
    try:
        O = torch.empty_like(Q)
        sc = tylo.allocate_scratchspace_decode_attention(O, Q, n_splits=6)
        for _ in range(3):                      # the call counter in the buffer advances per call
            O.fill_(float("nan"))
            tylo.sharded_decode_attention_(O, Q, K, V, lengths_local=ln, exchange=ex, scratch=sc, one_launch=one_launch)
            assert ex.status() == 0
            check(O, ref, dt, "single-rank exchange")
            assert int(sc.tickets.abs().sum()) == 0        # every counter is back at zero for the next call
    finally:
        ex.close()


@pytest.mark.parametrize("one_launch", [True, False], ids=["one-launch", "two-launch"])
@pytest.mark.parametrize("world", [2, 4])
def test_ranks_in_turn_merge_and_bounded_wait(tylo, oracle, world, one_launch):
    rng = np.random.default_rng(world)
    B, H, Hkv, Sk, D = 2, 8, 2, 2048, 64
    dt = "bf16"
    Q, Q64 = draw(rng, (B, H, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    lengths = [2048, 900]                       # the second sequence leaves the last shards empty
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    group = tylo.DecodeExchange.local_group(B, H, D, world=world, timeout_us=20_000)
    shards = [_shard(tylo, K, V, lengths, r, world) for r in range(world)]
    # 11 splits per shard: two ticket groups (8 + 3) in the one-launch form
    scs = [tylo.allocate_scratchspace_decode_attention(torch.empty_like(Q), Q, n_splits=11) for _ in range(world)]
    try:
        for order in (list(range(world)), list(reversed(range(world)))):   # two calls: both record parities
            for i, r in enumerate(order):
                Kr, Vr, lr = shards[r]
                O = torch.full_like(Q, 7.0)
                t0 = time.time()
                tylo.sharded_decode_attention_(O, Q, Kr, Vr, lengths_local=lr, exchange=group[r], scratch=scs[r],
                                               one_launch=one_launch)
                if i < world - 1:
                    # peers have not pushed: the wait must run out, be reported, and O stay untouched
                    with pytest.raises(tylo.TyloError) as e:
                        group[r].status()
                    assert e.value.status == 6
                    assert time.time() - t0 < 5.0
                    assert bool((O == 7.0).all())
                    assert group[r].status() == 0          # reading the status cleared it
                else:
                    assert group[r].status() == 0
                    check(O, ref, dt, f"sharded decode, world {world}")
        assert tylo.device_status() == 0
    finally:
        for g in group:
            g.close()


def test_exchange_rejects_bad_arguments(tylo):
    with pytest.raises(tylo.TyloError):
        tylo.DecodeExchange(1, 8, 64, world=17)
    ex = tylo.DecodeExchange(1, 8, 64)
    try:
        O = torch.empty(1, 8, 64, device="cuda")
        sc = tylo.allocate_scratchspace_decode_attention(O, O, n_splits=2)
        ex.rank = 3
        with pytest.raises(tylo.TyloError) as e:
            ex.exchange_(O, sc)
        assert e.value.status == 1
    finally:
        ex.rank = 0
        ex.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_process_exchange_over_ipc():
    worker = Path(__file__).with_name("dist_decode_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29600 + os.getpid() % 200
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(worker)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "EXCHANGE-OK" in r.stdout
