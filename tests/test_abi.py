"""CPU: the shared library loads, exports every symbol the header declares, and validates its
arguments before touching a device (no compute call is made here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "tylo_b200.h").read_text()
DECLARED = sorted(set(re.findall(r"\b(tylo_b200_\w+)\s*\(", HEADER)))


def test_header_declares_entry_points():
    assert len(DECLARED) >= 18
    for must in ("tylo_b200_attention_fwd", "tylo_b200_attention_bwd", "tylo_b200_flex_attention_fwd",
                 "tylo_b200_flex_attention_bwd", "tylo_b200_decode_attention", "tylo_b200_softmax_fwd",
                 "tylo_b200_rms_norm_fwd", "tylo_b200_layer_norm_fwd"):
        assert must in DECLARED


@pytest.mark.parametrize("sym", DECLARED)
def test_symbol_exported(tylo, sym):
    lib = ctypes.CDLL(tylo.lib_path())
    assert hasattr(lib, sym), f"{sym} declared in include/tylo_b200.h but not exported"


def test_version_and_status_strings(tylo):
    assert tylo.version() == 100
    assert tylo._status_string(0) == "ok"
    assert "unsupported" in tylo._status_string(2)


def _fake(n=1):
    return ctypes.c_void_p(0x1000 * n)  # aligned, never dereferenced: validation fails first


def test_argument_validation_without_device(tylo):
    lib = tylo._lib
    # null pointer
    assert lib.tylo_b200_softmax_fwd(None, _fake(), 8, 8, 0, None) == 1
    # non-positive extent
    assert lib.tylo_b200_softmax_fwd(_fake(), _fake(2), 0, 8, 0, None) == 1
    assert b"positive" in lib.tylo_b200_last_error()
    # misaligned
    assert lib.tylo_b200_rms_norm_fwd(ctypes.c_void_p(0x1004), _fake(), _fake(2), None, 8, 8, 1e-5, 0.0, 0, None) == 3
    # heads not a multiple of kv heads (attention.jl:237)
    f = _fake
    rc = lib.tylo_b200_attention_fwd(f(1), f(2), f(3), f(4), None, None, None, None, 64, 64, 16, 16, 3, 2, 1, 0, 0, 0, None)
    assert rc == 1 and b"multiple" in lib.tylo_b200_last_error()
    # backward without checkpoints (attention.jl:306: `checkpoints` is required)
    rc = lib.tylo_b200_attention_bwd(f(1), f(2), f(3), f(4), f(5), f(6), f(7), f(8), None, None, None, f(9), None, 0,
                                     None, None, 64, 64, 16, 16, 2, 2, 1, 0, 0, 0, None)
    assert rc == 1 and b"checkpoints" in lib.tylo_b200_last_error()
    # decode: n_splits must be positive
    rc = lib.tylo_b200_decode_attention(f(1), f(2), f(3), f(4), f(5), f(6), f(7), f(8), 0, 64, 64, 128, 4, 4, 1, 0, None)
    assert rc == 1
    # one-launch decode: same checks, and a rank outside the world is refused
    rc = lib.tylo_b200_decode_attention_fused(f(1), f(2), f(3), f(4), f(5), f(6), f(7), f(8), f(9), 0, 64, 64, 128, 4, 4, 1, 1, None)
    assert rc == 1
    peers = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    rc = lib.tylo_b200_decode_attention_sharded(f(1), f(2), f(3), f(4), f(5), f(6), f(7), f(8), f(9), 4, peers, 2, 2,
                                                64, 64, 128, 4, 4, 1, 1, 0, None)
    assert rc == 1 and b"rank" in lib.tylo_b200_last_error()
    assert lib.tylo_b200_decode_ticket_count(148, 8, 1) == 8 * (19 + 1)
    # unknown dtype is rejected before any launch
    assert lib.tylo_b200_softmax_fwd(_fake(), _fake(2), 8, 8, 7, None) == 1


def test_flex_descriptor_validation(tylo):
    lib = tylo._lib
    f = _fake
    md = tylo._MaskDesc(); md.flags = tylo.MASK_DOCUMENT       # document mask without id tables
    sd = tylo._ScoreDesc()
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 1 and b"DocumentMask" in lib.tylo_b200_last_error()
    md = tylo._MaskDesc(); md.flags = 1 << 9
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 2
    md = tylo._MaskDesc(); sd = tylo._ScoreDesc(); sd.flags = tylo.SCORE_SOFTCAP; sd.cap = 0.0
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 1
    # a bias table that is not 16-byte aligned is refused before any launch (the kernels read it with 16-byte loads)
    md = tylo._MaskDesc(); sd = tylo._ScoreDesc(); sd.flags = tylo.SCORE_BIAS; sd.bias = 0x2004; sd.bias_heads = 1; sd.bias_batch = 1
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 1, None)
    assert rc == 3 and b"16-byte aligned" in lib.tylo_b200_last_error()


def test_decode_suggest_splits(tylo):
    n = tylo.decode_suggest_splits(1 << 20, 8, 1)
    assert n >= 64                      # enough CTAs for a 148-SM part with 8 KV heads
    assert tylo.decode_suggest_splits(512, 8, 64) >= 1
    assert tylo.decode_suggest_splits(100, 1, 1) == 1


def test_block_mask_and_or_chain_validation(tylo):
    """Argument checks of the block-list entry points and of OR-ed mask clauses; nothing is launched."""
    lib = tylo._lib
    f = _fake
    md, sd = tylo._MaskDesc(), tylo._ScoreDesc()
    args_tail = (64, 64, 128, 128, 2, 2, 1, 0, 0.0, 0, None)
    # block edges that are not multiples of 32 are unsupported
    rc = lib.tylo_b200_flex_attention_fwd_block_mask(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                                     f(5), f(6), f(7), 2, 48, 64, *args_tail)
    assert rc == 2 and b"multiples of 32" in lib.tylo_b200_last_error()
    # the three list arrays are required
    rc = lib.tylo_b200_flex_attention_fwd_block_mask(f(1), f(2), f(3), f(4), None, None, ctypes.byref(md), ctypes.byref(sd),
                                                     None, f(6), f(7), 2, 64, 64, *args_tail)
    assert rc == 1 and b"count" in lib.tylo_b200_last_error()
    # the backward needs the forward's statistics
    rc = lib.tylo_b200_flex_attention_bwd_block_mask(f(1), f(2), f(3), f(4), f(5), f(6), f(7), f(8), None, None, f(9), None, 0,
                                                     ctypes.byref(md), ctypes.byref(sd), f(10), f(11), f(12), 2, 64, 64,
                                                     *args_tail)
    assert rc == 1 and b"checkpoints" in lib.tylo_b200_last_error()
    # five OR-ed conjunctions: one more than the library takes
    chain = [tylo._MaskDesc() for _ in range(5)]
    for a, b in zip(chain, chain[1:]):
        a.or_next = ctypes.addressof(b)
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(chain[0]), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 2 and b"OR-ed" in lib.tylo_b200_last_error()
    # a clause further down the chain is validated like the first one
    chain = [tylo._MaskDesc() for _ in range(2)]
    chain[0].or_next = ctypes.addressof(chain[1]); chain[1].flags = tylo.MASK_DOCUMENT
    rc = lib.tylo_b200_flex_attention_fwd(f(1), f(2), f(3), f(4), None, None, ctypes.byref(chain[0]), ctypes.byref(sd),
                                          64, 64, 16, 16, 2, 2, 1, 0, 0.0, 1, 0, None)
    assert rc == 1 and b"DocumentMask" in lib.tylo_b200_last_error()


def test_decode_split_suggestion_follows_the_cache_size():
    """`tylo_b200_decode_suggest_splits` needs no GPU: without one it assumes 148 SMs.  One CTA per SM below ~0.8 GB
    of cache (keys x KV heads x batch < 1.5 Mi), four up to ~3 GB, eight above; never fewer than 256 keys per split."""
    import ctypes
    from pathlib import Path
    lib = ctypes.CDLL(str(Path(__file__).resolve().parent.parent / "tylo.jl_b200" / "libtylo_b200.so"))
    f = lib.tylo_b200_decode_suggest_splits
    assert f(131072, 8, 1) == 19          # 537 MB as 8 heads x 131,072 keys: 148 CTAs
    assert f(1 << 20, 1, 1) == 148        # 537 MB as one head x 1,048,576 keys
    assert f(262144, 8, 1) == 74          # 1.07 GB: four per SM
    assert f(1 << 20, 8, 1) == 148        # 4.3 GB: eight per SM
    assert f(32768, 8, 64) == 3           # the ragged batch: eight per SM over 512 groups
    assert f(100, 1, 1) == 1 and f(0, 1, 1) == 1
    assert f(300, 1, 1) == 2              # at least 256 keys per split


def test_julia_wrappers_call_only_exported_symbols_with_matching_arity():
    """Every `ccall((:tylo_b200_x, libtylo), ...)` of the Julia package names a symbol that `include/tylo_b200.h`
    declares, and passes as many arguments as the declaration has parameters (the Julia sources cannot be executed
    here, so the binding is checked as text against the header)."""
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    header = (root / "include" / "tylo_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    decl = {}
    for m in re.finditer(r"\b(tylo_b200_\w+)\s*\(([^;{]*?)\)\s*;", header, flags=re.S):
        params = m.group(2).strip()
        decl[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    assert len(decl) > 30
    seen = 0
    for jl in (root / "tylo.jl_b200" / "julia" / "Tylo").rglob("*.jl"):
        text = jl.read_text()
        for m in re.finditer(r"ccall\(\(:(tylo_b200_\w+), libtylo\),\s*\w+,\s*\(", text):
            name = m.group(1)
            assert name in decl, f"{jl.name}: {name} is not declared in the header"
            # the argument-type tuple follows: count its entries up to the matching parenthesis
            i, depth, n, nonempty = m.end(), 1, 0, False
            while depth:
                c = text[i]
                if c in "({[":
                    depth += 1
                elif c in ")}]":
                    depth -= 1
                elif c == "," and depth == 1:
                    n += 1
                elif not c.isspace():
                    nonempty = True
                i += 1
            tail = text[m.end():i - 1].rstrip()
            n_types = 0 if not nonempty else n + (0 if tail.endswith(",") else 1)
            assert n_types == decl[name], f"{jl.name}: {name} passes {n_types} argument types, the header declares {decl[name]}"
            seen += 1
    assert seen >= 20
