"""CPU: the sharded-decode exchange and the bias score mod validate their arguments before touching a
device (no launch, no allocation is made here)."""
import ctypes


def _fake(i=1):
    return ctypes.c_void_p(0x1000 * i)


def test_exchange_bytes_and_argument_validation(tylo):
    lib = tylo._lib
    # layout: 16 header words, call counters, flags, then 2 x world x heads records of Dv + 4 floats
    assert lib.tylo_b200_decode_exchange_bytes(1, 128, 64, 1) == 4 * (16 + 64 + 64 + 2 * 1 * 64 * 132)
    assert lib.tylo_b200_decode_exchange_bytes(8, 128, 64, 1) == 4 * (16 + 64 + 512 + 2 * 8 * 64 * 132)
    assert lib.tylo_b200_decode_exchange_bytes(17, 128, 64, 1) == 0      # more ranks than the kernel supports
    assert lib.tylo_b200_decode_exchange_bytes(2, 130, 64, 1) == 0       # Dv must be a multiple of 4
    assert lib.tylo_b200_decode_exchange_bytes(2, 1024, 64, 1) == 0
    f = _fake
    peers = (ctypes.c_void_p * 2)(0x10000, 0x20000)
    call = lambda *a: lib.tylo_b200_decode_exchange(*a)
    assert call(f(1), f(2), f(3), f(4), 4, 64 * 128, 64, None, 0, 2, 128, 64, 1, 1, 0, None) == 1           # no peer table
    assert call(f(1), f(2), f(3), f(4), 4, 64 * 128, 64, peers, 2, 2, 128, 64, 1, 1, 0, None) == 1          # rank out of range
    assert b"rank" in lib.tylo_b200_last_error()
    assert call(f(1), f(2), f(3), f(4), 4, 64 * 128, 64, peers, 0, 17, 128, 64, 1, 1, 0, None) == 2         # world too large
    assert call(f(1), f(2), f(3), f(4), 4, 64 * 128, 64, peers, 0, 2, 130, 64, 1, 1, 0, None) == 2          # Dv % 4
    assert call(f(1), f(2), f(3), f(4), 4, 100, 64, peers, 0, 2, 128, 64, 1, 1, 0, None) == 1               # stride too small
    assert call(f(1), ctypes.c_void_p(0x2004), f(3), f(4), 4, 64 * 128, 64, peers, 0, 2, 128, 64, 1, 1, 0, None) == 3
    bad = (ctypes.c_void_p * 2)(0x10000, None)
    assert call(f(1), f(2), f(3), f(4), 4, 64 * 128, 64, bad, 0, 2, 128, 64, 1, 1, 0, None) == 1            # unmapped peer
    code = ctypes.c_int32(0)
    assert lib.tylo_b200_decode_exchange_status(None, ctypes.byref(code)) == 1
    assert lib.tylo_b200_peer_alloc(None, 16) == 1
    assert lib.tylo_b200_peer_export(None, None) == 1
    assert lib.tylo_b200_peer_handle_bytes() == 64


def test_bias_descriptor_validation(tylo):
    lib = tylo._lib
    f = _fake
    md = tylo._MaskDesc()
    sd = tylo._ScoreDesc(); sd.flags = tylo.SCORE_BIAS                  # bias flag without a table
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 1 and b"BiasScore" in lib.tylo_b200_last_error()
    sd = tylo._ScoreDesc(); sd.flags = tylo.SCORE_BIAS; sd.bias = 0x4000; sd.bias_heads = 0; sd.bias_batch = 1
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 1
    sd = tylo._ScoreDesc(); sd.flags = 1 << 7                           # unknown score flag
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 2


def test_score_chain_mapping_on_host(tylo):
    """Host-side checks of composed score mods that need no device: additive mods must share one place in
    the chain, and host tensors are refused (the library has no CPU path)."""
    import pytest
    import torch
    bias = torch.zeros(1, 1, 4, 4)
    slopes = torch.ones(2)
    with pytest.raises(tylo.TyloError):
        tylo._score_desc(tylo.BiasScore(bias) @ (tylo.SoftCapScore(5.0) @ tylo.AliBiScore(slopes)), None, [])
    with pytest.raises(ValueError, match="no CPU path"):
        tylo._score_desc(tylo.BiasScore(bias), None, [])
    assert tylo.hscore(tylo.BiasScore(bias + 2.0), 1.0, 3, 1, b=5, h=7) == 3.0      # mod1 broadcast of b and h
