"""Child process of the two-GPU decode test: one rank per GPU, keys of every sequence sharded over
ranks, merged by the peer exchange; every rank checks its result against the oracle over the whole
key range.  Launched by torch.distributed.run; the process group (gloo) only carries the IPC handles."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).parent))
from conftest import load_oracle, load_package  # noqa: E402
from gpu_util import check, draw  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    tylo, oracle = load_package(), load_oracle()
    rng = np.random.default_rng(11)                     # same draw on every rank
    B, H, Hkv, Sk, D = 2, 16, 2, 4096, 128
    Q, Q64 = draw(rng, (B, H, D), "bf16"); K, K64 = draw(rng, (B, Hkv, Sk, D), "bf16"); V, V64 = draw(rng, (B, Hkv, Sk, D), "bf16")
    lengths = [4096, 2500]
    per = Sk // world
    b, e = rank * per, (rank + 1) * per
    Kr, Vr = K[:, :, b:e].contiguous(), V[:, :, b:e].contiguous()
    lr = torch.tensor([min(max(n - b, 0), e - b) for n in lengths], dtype=torch.int32, device="cuda")
    ex = tylo.DecodeExchange(B, H, D, rank=rank, world=world)
    O = torch.empty_like(Q)
    sc = tylo.allocate_scratchspace_decode_attention(O, Q, n_splits=8)
    ref = oracle.decode_reference(Q64, K64, V64, lengths)
    for it in range(6):                                 # one-launch and two-launch forms share the buffers
        O.fill_(float("nan"))
        tylo.sharded_decode_attention_(O, Q, Kr, Vr, lengths_local=lr, exchange=ex, scratch=sc, one_launch=it % 3 != 2)
        assert ex.status() == 0
        check(O, ref, "bf16", "two-process sharded decode")
    # replayed from a CUDA graph, as a serving loop would
    torch.cuda.synchronize(); dist.barrier()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            tylo.sharded_decode_attention_(O, Q, Kr, Vr, lengths_local=lr, exchange=ex, scratch=sc)
    for _ in range(3):
        O.fill_(float("nan"))
        g.replay()
        assert ex.status() == 0
        check(O, ref, "bf16", "graph replay")
    dist.barrier()
    ex.close()
    dist.destroy_process_group()
    if rank == 0:
        print("EXCHANGE-OK")


if __name__ == "__main__":
    main()
