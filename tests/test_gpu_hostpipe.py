"""GPU: the host-tensor pipeline (copies and kernels of different batch entries overlapped on three
streams) returns what the device-tensor entry point returns, call after call without synchronising."""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _hostpipe():
    name = "tylo_b200_hostpipe"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, ROOT / "tylo.jl_b200" / "hostpipe.py")
    mod = importlib.util.module_from_spec(spec); sys.modules[name] = mod; spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("causal", [False, True])
def test_pipeline_matches_device_call(tylo, causal):
    B, H, Hkv, S, D = 3, 4, 2, 384, 128
    pipe = _hostpipe().HostAttentionPipeline(tylo, B, H, Hkv, S, S, D, causal=causal)
    g = torch.Generator().manual_seed(5)
    outs, refs = [], []
    for _ in range(3):                                   # three calls back to back, no synchronise between them
        hQ = torch.randn(B, H, S, D, generator=g).bfloat16().pin_memory()
        hK = torch.randn(B, Hkv, S, D, generator=g).bfloat16().pin_memory()
        hV = torch.randn(B, Hkv, S, D, generator=g).bfloat16().pin_memory()
        hO = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16).pin_memory()
        pipe.run(hO, hQ, hK, hV)
        outs.append(hO)
        refs.append((hQ, hK, hV))
    torch.cuda.synchronize()
    for hO, (hQ, hK, hV) in zip(outs, refs):
        ref = tylo.attention(hQ.cuda(), hK.cuda(), hV.cuda(), causal=causal)
        torch.cuda.synchronize()
        assert torch.equal(hO, ref.cpu())                # same kernel on the same inputs: bit-identical
    assert tylo.device_status() == 0
