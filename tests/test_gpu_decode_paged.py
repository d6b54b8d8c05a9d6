"""GPU parity: split-KV decode over a paged KV cache against the oracle on the dense cache the pages were cut
from (test/decode.jl:15-36): the pages are scattered through the pools in a random order, sequences have ragged
lengths (one empty, one ending inside a page), and a multi-step decode loop grows the lengths on the device
inside one CUDA graph."""
import numpy as np
import pytest
import torch

from gpu_util import back, check, draw

pytestmark = pytest.mark.gpu


def _paginate(K, V, page_size, rng):
    """Dense (B, Hkv, Sk, D) caches -> pools (n_pages, Hkv, page_size, D) in shuffled order + block table."""
    B, Hkv, Sk, D = K.shape
    per_seq = -(-Sk // page_size)
    n_pages = B * per_seq + 3                               # a few pages nobody owns
    perm = rng.permutation(n_pages)[:B * per_seq].reshape(B, per_seq)
    Kp = torch.zeros(n_pages, Hkv, page_size, D, dtype=K.dtype, device=K.device); Vp = torch.zeros_like(Kp)
    Vp = torch.zeros(n_pages, Hkv, page_size, V.shape[3], dtype=V.dtype, device=V.device)
    for b in range(B):
        for i in range(per_seq):
            n = min(page_size, Sk - i * page_size)
            Kp[perm[b, i], :, :n] = K[b, :, i * page_size:i * page_size + n]
            Vp[perm[b, i], :, :n] = V[b, :, i * page_size:i * page_size + n]
    return Kp, Vp, torch.from_numpy(perm.astype(np.int32)).cuda()


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("D,page_size,G", [(128, 16, 8), (128, 256, 4), (64, 32, 1), (64, 128, 16)])
def test_paged_decode_vs_reference(tylo, oracle, dt, D, page_size, G):
    rng = np.random.default_rng(D + page_size)
    B, Hkv, Sk = 4, 2, 1500
    H = Hkv * G
    Q, Q64 = draw(rng, (B, H, D), dt); K, K64 = draw(rng, (B, Hkv, Sk, D), dt); V, V64 = draw(rng, (B, Hkv, Sk, D), dt)
    lengths = [1500, 777, 0, page_size * 3]
    ln = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    Kp, Vp, table = _paginate(K, V, page_size, rng)
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    for n_splits in (None, 1, 5):
        O = torch.full_like(Q, float("nan"))
        tylo.paged_decode_attention_(O, Q, Kp, Vp, block_table=table, lengths=ln, n_splits=n_splits)
        check(O, ref, dt, f"paged decode ({n_splits} splits)")
    assert tylo.device_status() == 0


def test_paged_decode_multi_step_graph(tylo, oracle):
    """A decode loop as a serving engine runs it: the lengths live on the device and grow by one per step; all
    steps are captured in one CUDA graph and replayed."""
    rng = np.random.default_rng(5)
    B, H, Hkv, D, Sk, page_size, steps = 3, 16, 2, 128, 640, 64, 4
    Q, Q64 = draw(rng, (B, H, D), "bf16"); K, K64 = draw(rng, (B, Hkv, Sk, D), "bf16"); V, V64 = draw(rng, (B, Hkv, Sk, D), "bf16")
    Kp, Vp, table = _paginate(K, V, page_size, rng)
    start = [600, 129, 63]
    ln = torch.tensor(start, dtype=torch.int32, device="cuda")
    outs = [torch.empty_like(Q) for _ in range(steps)]
    sc = tylo.allocate_scratchspace_decode_attention(outs[0], Q, n_splits=4)
    tylo.paged_decode_attention_(outs[0], Q, Kp, Vp, block_table=table, lengths=ln, scratch=sc)   # warm-up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for s in range(steps):
                tylo.paged_decode_attention_(outs[s], Q, Kp, Vp, block_table=table, lengths=ln, scratch=sc)
                ln.add_(1)
    for rep in range(2):
        ln.copy_(torch.tensor(start, dtype=torch.int32))
        g.replay()
        torch.cuda.synchronize()
        for s in range(steps):
            ref = oracle.decode_reference(Q64, K64, V64, [n + s for n in start])
            check(outs[s], ref, "bf16", f"graph replay {rep}, step {s}")


def test_paged_decode_rejections(tylo):
    Q = torch.zeros(1, 4, 128, device="cuda", dtype=torch.bfloat16)
    Kp = torch.zeros(4, 1, 24, 128, device="cuda", dtype=torch.bfloat16)          # page size not a multiple of 16
    table = torch.zeros(1, 2, dtype=torch.int32, device="cuda"); ln = torch.ones(1, dtype=torch.int32, device="cuda")
    with pytest.raises(tylo.TyloError) as e:
        tylo.paged_decode_attention_(torch.empty_like(Q), Q, Kp, Kp, block_table=table, lengths=ln, n_splits=2)
    assert e.value.status == 2
    Qf = Q.float(); Kf = torch.zeros(4, 1, 32, 128, device="cuda")
    with pytest.raises(tylo.TyloError):
        tylo.paged_decode_attention_(torch.empty_like(Qf), Qf, Kf, Kf, block_table=table, lengths=ln, n_splits=2)
