"""GPU parity: ragged batches on the tensor-core forward (16-bit storage, head dim 64 / 128):
`k_lengths` masks keys at or beyond the per-batch length (attention.jl:60), `q_lengths` skips 64-row
query blocks that start at or beyond the per-batch length and leaves their output rows untouched
(attention.jl:25-26), `input_pos` shifts the causal diagonal (attention.jl:61).  A chunked-prefill
caller uses exactly this combination."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt,D", [("bf16", 128), ("f16", 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_forward(tylo, oracle, dt, D, causal):
    rng = np.random.default_rng(D + causal)
    B, H, Hkv, Sq, Sk = 4, 4, 2, 384, 640
    input_pos = 256 if causal else 0
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    k_lens, q_lens = [640, 300, 129, 0], [384, 200, 64, 1]
    kl = torch.tensor(k_lens, dtype=torch.int32, device="cuda")
    ql = torch.tensor(q_lens, dtype=torch.int32, device="cuda")
    O = torch.full_like(Q, 7.0)
    cp = tylo.allocate_checkpoints_attention(Q, K, V)
    cp.M.fill_(7.0); cp.L.fill_(7.0)
    tylo.attention_(O, Q, K, V, causal=causal, input_pos=input_pos, k_lengths=kl, q_lengths=ql, checkpoints=cp)
    assert tylo.device_status() == 0
    mask = oracle.MaskSpec(causal=True) if causal else None
    for b in range(B):
        n, live = k_lens[b], min(Sq, -(-q_lens[b] // 64) * 64)
        if n > 0:
            ref, Mr, Lr = oracle.flex_ref(Q64[b:b + 1], K64[b:b + 1, :, :n], V64[b:b + 1, :, :n], mask=mask,
                                          input_pos=input_pos, return_stats=True)
            check(O[b:b + 1, :, :live], ref[:, :, :live], dt, f"ragged O, batch {b}")
            # checkpoints of attention!: M in log2 units, L = sum exp2(. - M); compare the log-sum-exp
            lse = back(cp.M[b, :, :live]) * np.log(2.0) + np.log(back(cp.L[b, :, :live]))
            lse_ref = Mr[0, :, :live] + np.log(Lr[0, :, :live])
            fin = np.isfinite(lse_ref)
            np.testing.assert_allclose(lse[fin], lse_ref[fin], atol=2e-2)
        else:                                          # no keys at all: zeros, M = -inf, L = 0
            assert bool((O[b, :, :live] == 0).all()) and bool((cp.L[b, :, :live] == 0).all())
        assert bool((O[b, :, live:] == 7.0).all()), "rows of skipped query blocks must stay untouched"
        assert bool((cp.M[b, :, live:] == 7.0).all())


@pytest.mark.parametrize("dt,D", [("bf16", 128), ("f16", 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_backward(tylo, oracle, dt, D, causal):
    """∇attention! with k_lengths / q_lengths on the tensor-core kernels: gradients of the live part equal
    the oracle's on the sliced problem, everything beyond the lengths is overwritten with zeros
    (overwrite semantics, buffers.jl:17-18)."""
    rng = np.random.default_rng(7 + D + causal)
    B, H, Hkv, Sq, Sk = 3, 4, 2, 320, 448
    input_pos = 128 if causal else 0
    Q, Q64 = draw(rng, (B, H, Sq, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    dO, dO64 = draw(rng, (B, H, Sq, D), dt)
    k_lens, q_lens = [448, 200, 129], [320, 150, 64]
    kl = torch.tensor(k_lens, dtype=torch.int32, device="cuda")
    ql = torch.tensor(q_lens, dtype=torch.int32, device="cuda")
    O = torch.zeros_like(Q)                       # skipped rows stay finite (they meet zero probabilities)
    cp = tylo.allocate_checkpoints_attention(Q, K, V)
    cp.M.zero_(); cp.L.zero_()
    tylo.attention_(O, Q, K, V, causal=causal, input_pos=input_pos, k_lengths=kl, q_lengths=ql, checkpoints=cp)
    Qd, Kd, Vd = tylo.Duplicated(Q), tylo.Duplicated(K), tylo.Duplicated(V)
    for d in (Qd, Kd, Vd):
        d.shadow.fill_(5.0)
    tylo.grad_attention_(tylo.Duplicated(O, dO), Qd, Kd, Vd, causal=causal, checkpoints=cp, input_pos=input_pos,
                         k_lengths=kl, q_lengths=ql)
    assert tylo.device_status() == 0
    mask = oracle.MaskSpec(causal=True) if causal else None
    for b in range(B):
        n, live = k_lens[b], min(Sq, -(-q_lens[b] // 64) * 64)
        rQ, rK, rV, _ = oracle.flex_bwd_ref(dO64[b:b + 1, :, :live], Q64[b:b + 1, :, :live], K64[b:b + 1, :, :n],
                                            V64[b:b + 1, :, :n], mask=mask, input_pos=input_pos)
        for got, ref, name in ((Qd.shadow[b:b + 1, :, :live], rQ, "dQ"), (Kd.shadow[b:b + 1, :, :n], rK, "dK"),
                               (Vd.shadow[b:b + 1, :, :n], rV, "dV")):
            check(got, ref, dt, f"ragged {name}, batch {b}", scale_hint=float(np.abs(ref).max()))
        assert bool((Qd.shadow[b, :, live:] == 0).all()) and bool((Kd.shadow[b, :, n:] == 0).all())
        assert bool((Vd.shadow[b, :, n:] == 0).all())
