"""GPU parity: split-KV decode against the oracle; cases follow test/decode.jl:69-124."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw

pytestmark = pytest.mark.gpu

CASES = [  # name, Dk, Dv, H, Hkv, Sk, lengths, n_splits
    ("mha full", 64, 64, 8, 8, 128, [128, 128], 4),
    ("mha ragged", 64, 64, 4, 4, 200, [200, 137, 65], 4),
    ("gqa G=4", 64, 64, 8, 2, 512, [512, 301], 8),
    ("gqa G=8", 128, 128, 8, 1, 384, [384, 200], 6),
    ("short + empty", 64, 64, 4, 2, 512, [30, 1, 0], 8),
    ("single split", 64, 64, 4, 4, 256, [256, 173], 1),
    ("oversplit", 64, 64, 4, 2, 96, [96, 50], 16),
    ("gqa G=16", 128, 128, 32, 2, 700, [700, 33], 5),
    ("odd head dim", 80, 48, 6, 3, 150, [150, 77], 3),
]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_decode_vs_reference(tylo, oracle, case, dt):
    _, Dk, Dv, H, Hkv, Sk, lengths, n_splits = case
    B = len(lengths)
    rng = np.random.default_rng(Sk + H)
    Q, Q64 = draw(rng, (B, H, Dk), dt)
    K, K64 = draw(rng, (B, Hkv, Sk, Dk), dt)
    V, V64 = draw(rng, (B, Hkv, Sk, Dv), dt)
    ln = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    for one_launch in (True, False):                       # the split kernel finishing the merge itself, or two launches
        O = torch.full((B, H, Dv), float("nan"), dtype=Q.dtype, device="cuda")
        tylo.decode_attention_(O, Q, K, V, lengths=ln, n_splits=n_splits, one_launch=one_launch)
        check(O, ref, dt, f"decode (one_launch={one_launch})")


@pytest.mark.parametrize("n_splits", [1, 7, 8, 9, 37, 148])
def test_one_launch_ticket_groups(tylo, oracle, n_splits):
    """The one-launch form over split counts around its group size of eight (one group, a partial group,
    many groups), repeated on one scratch: the ticket words must be left at zero by every call."""
    rng = np.random.default_rng(n_splits)
    B, H, Hkv, Sk, D = 2, 16, 2, 5000, 128
    Q, Q64 = draw(rng, (B, H, D), "bf16"); K, K64 = draw(rng, (B, Hkv, Sk, D), "bf16"); V, V64 = draw(rng, (B, Hkv, Sk, D), "bf16")
    lengths = [5000, 3]
    ln = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    O = torch.empty_like(Q)
    sc = tylo.allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
    for _ in range(3):
        O.fill_(float("nan"))
        tylo.decode_attention_(O, Q, K, V, lengths=ln, scratch=sc)
        check(O, ref, "bf16", f"one-launch decode, {n_splits} splits")
        assert int(sc.tickets.abs().sum()) == 0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_split_invariance(tylo, dt):
    rng = np.random.default_rng(1)
    Q, _ = draw(rng, (3, 8, 64), dt); K, _ = draw(rng, (3, 2, 500, 64), dt); V, _ = draw(rng, (3, 2, 500, 64), dt)
    ln = torch.tensor([500, 333, 64], dtype=torch.int32, device="cuda")
    base = tylo.decode_attention_(torch.empty_like(Q), Q, K, V, lengths=ln, n_splits=1)
    for n in (2, 4, 8, 16):
        got = tylo.decode_attention_(torch.empty_like(Q), Q, K, V, lengths=ln, n_splits=n)
        assert torch.allclose(got.float(), base.float(), atol=1e-3 if dt == "f32" else 8e-3, rtol=1e-3)  # test/decode.jl:122


def test_partials_and_two_level_merge(tylo, oracle):
    """Partials follow decode.jl:92-98 (normalised O, log2-unit max, sum); merging shard-level
    merged partials (the multi-GPU path) equals the single-level merge."""
    rng = np.random.default_rng(7)
    B, H, Hkv, Sk, D = 2, 16, 2, 2048, 128
    Q, Q64 = draw(rng, (B, H, D), "bf16"); K, K64 = draw(rng, (B, Hkv, Sk, D), "bf16"); V, V64 = draw(rng, (B, Hkv, Sk, D), "bf16")
    lengths = [2048, 1500]
    ln = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    sc = tylo.allocate_scratchspace_decode_attention(torch.empty(B, H, D, device="cuda"), Q, n_splits=8)
    tylo.decode_split_(Q, K, V, lengths=ln, scratch=sc)
    size = 256
    for s in (0, 5, 7):
        Or, Mr, Lr = oracle.decode_partials(Q64, K64, V64, lengths, s * size, (s + 1) * size)
        np.testing.assert_allclose(back(sc.M_partial[s]), Mr, rtol=1e-5, atol=1e-4)
        live = np.isfinite(Mr)
        np.testing.assert_allclose(back(sc.L_partial[s])[live], Lr[live], rtol=2e-2)
        np.testing.assert_allclose(back(sc.O_partial[s]), Or, atol=2e-2)
    # two shards of the KV axis, as two GPUs would hold them
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    packs = []
    for r in range(2):
        Kr, Vr = K[:, :, r * 1024:(r + 1) * 1024].contiguous(), V[:, :, r * 1024:(r + 1) * 1024].contiguous()
        lr = (ln - r * 1024).clamp(0, 1024).to(torch.int32)
        scr = tylo.allocate_scratchspace_decode_attention(torch.empty(B, H, D, device="cuda"), Q, n_splits=4)
        tylo.decode_split_(Q, Kr, Vr, lengths=lr, scratch=scr)
        merged = tylo.allocate_scratchspace_decode_attention(torch.empty(B, H, D, device="cuda"), Q, n_splits=1)
        tylo.decode_combine_(None, scr.O_partial, scr.M_partial, scr.L_partial, n_splits=4, o_stride=B * H * D,
                             ml_stride=B * H, Dv=D, H=H, B=B, merged=merged)
        packs.append(torch.cat([merged.O_partial.flatten(), merged.M_partial.flatten(), merged.L_partial.flatten()]))
    gathered = torch.stack(packs)                          # what an all-gather leaves on every rank
    n = B * H * D
    O = torch.empty(B, H, D, dtype=torch.bfloat16, device="cuda")
    flat = gathered.flatten()
    stride = gathered.shape[1]
    tylo.decode_combine_(O, flat, flat[n:], flat[n + B * H:], n_splits=2, o_stride=stride, ml_stride=stride,
                         Dv=D, H=H, B=B)
    check(O, ref, "bf16", "two-level merge")


def test_decode_benchmark_shape_sample(tylo, oracle):
    """Config 5a geometry (Hq 64, Hkv 8, D 128, ragged lengths) at batch 4, oracle on every head."""
    g = torch.Generator(device="cuda").manual_seed(4)
    B, H, Hkv, Sk, D = 4, 64, 8, 32768, 128
    Q = torch.randn(B, H, D, device="cuda", generator=g).to(torch.bfloat16)
    K = torch.randn(B, Hkv, Sk, D, device="cuda", generator=g).to(torch.bfloat16)
    V = torch.randn(B, Hkv, Sk, D, device="cuda", generator=g).to(torch.bfloat16)
    lengths = [32768, 1024, 20011, 7]
    ln = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    O = tylo.decode_attention_(torch.empty_like(Q), Q, K, V, lengths=ln, n_splits=None)
    check(O, oracle.decode_reference(back(Q), back(K), back(V), lengths), "bf16", "decode C5a sample")
