"""GPU: the scratch-free decode entry point against the ordinary one, through the C ABI.

`tylo_b200_decode_attention_static` serves callers that must not allocate device memory when they
call (a frozen serving pool, a plugin under a runtime that owns the memory): its split partials live
in a fixed array inside the library.  Because that array is shared by every call and keeps old
contents, the check runs twice in a row with different inputs and a different split count, and each
result must equal what `tylo_b200_decode_attention` produces with caller-owned scratch.  The file is
named so that pytest collects it last."""
import ctypes
from ctypes import c_int32, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind(lib):
    fn = lib.tylo_b200_decode_attention_static
    fn.restype = c_int32
    fn.argtypes = [c_void_p] * 5 + [c_int32] * 8 + [c_void_p]
    cap = lib.tylo_b200_decode_static_scratch_floats
    cap.restype = c_int64
    ref = lib.tylo_b200_decode_attention
    return fn, cap, ref


def _p(t):
    return c_void_p(t.data_ptr())


def test_static_scratch_decode_matches_twice(tylo):
    lib = tylo._lib
    fn, cap, ref = _bind(lib)
    assert cap() == 2 << 20
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(123)
    # (B, H, Hkv, Sk, D, n_splits, lengths): the second call uses fewer, larger slots over stale contents
    for B, H, Hkv, Sk, D, n_splits, lens in ((3, 16, 2, 3000, 128, 12, [3000, 1234, 0]),
                                             (2, 8, 8, 900, 64, 5, [17, 900])):
        Q = torch.randn(B, H, D, device="cuda", generator=g).to(torch.bfloat16)
        K = torch.randn(B, Hkv, Sk, D, device="cuda", generator=g).to(torch.bfloat16)
        V = torch.randn(B, Hkv, Sk, D, device="cuda", generator=g).to(torch.bfloat16)
        ln = torch.tensor(lens, dtype=torch.int32, device="cuda")
        want = torch.empty_like(Q)
        sc = tylo.allocate_scratchspace_decode_attention(want, Q, n_splits=n_splits)
        rc = ref(_p(want), _p(Q), _p(K), _p(V), _p(ln), _p(sc.O_partial), _p(sc.M_partial), _p(sc.L_partial),
                 n_splits, D, D, Sk, H, Hkv, B, tylo.BF16, stream)
        assert rc == 0, lib.tylo_b200_last_error()
        got = torch.full_like(Q, float("nan"))
        rc = fn(_p(got), _p(Q), _p(K), _p(V), _p(ln), n_splits, D, D, Sk, H, Hkv, B, tylo.BF16, stream)
        assert rc == 0, lib.tylo_b200_last_error()
        torch.cuda.synchronize()
        # same kernels, same split layout: the outputs agree to the decode tests' tolerance (in fact bit for bit)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=0)
        assert torch.equal(got, want)


def test_static_scratch_rejects_oversize(tylo):
    lib = tylo._lib
    fn, cap, _ = _bind(lib)
    fake = c_void_p(0x10000)           # never dereferenced: the size check comes first
    n_splits, B, H, D = 4096, 8, 64, 128
    assert n_splits * B * H * (D + 2) > cap()
    rc = fn(fake, fake, fake, fake, fake, n_splits, D, D, 1 << 20, H, 8, B, tylo.BF16, None)
    assert rc == 7 and b"exceeds the built-in scratch" in lib.tylo_b200_last_error()
