#!/usr/bin/env python
"""Benchmark of the Tylo hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Headline (default workload `prefill_fwd`): causal GQA prefill forward, bf16, batch 4 per GPU,
seq 4096, Hq 32 / Hkv 8, head dim 128 — throughput in TFLOP/s counted on unmasked pairs
(4 * D * pairs).  One JSON line is printed by rank 0.  The other configs of the build contract
are measured briefly and reported under "extras" (decode in GB/s of live KV bytes, norms and
softmax in GB/s, backward and flex in TFLOP/s), each with its own roofline fraction.

Multi-GPU (`--gpus N`, launched under torchrun): prefill shards over batch x heads with no
communication (every rank runs the per-GPU problem: weak scaling); the 1M-token decode extra
shards the KV sequence across ranks and merges the per-rank (O, max, sum) partials with the
library's own exchange kernel (peer stores over NVLink into IPC-shared buffers, one launch);
`decode_1m_heads` cuts the same cache by KV heads instead, which needs no exchange at all.  At N > 1 both decode
workloads replay eight decode steps per CUDA graph and report the time per decode step beside the replay's.

Strong-scaling prefill (`prefill_fwd_sharded`, `prefill_bwd_sharded`): ONE batch-4 problem whose 32
(kv-head, batch) units are cut into contiguous ranges, one per rank, no exchange.

Variants outside the contract's configs, each on the tensor-core kernels and each checked against the oracle:
`mha_tf32` (config 1 with TF32 operands), `flex_bias_fwd_bwd` (bias table with its gradient), `flex_block_list_fwd`
and `flex_fwd_block_list` (host-built block lists: a causal window, and config 4's own mask).

Inputs come from the package's counter-based generator (`synth.py`: element i of tensor t under seed s
is the same number on the CPU and on the GPU, however the tensor is sharded).  After a workload has been
timed, a sample of its output is checked against the float64 CPU oracle, outside the timed region, and
the measured error is reported under `parity` (`--no-verify` skips it, e.g. under a profiler).

`--impl reference` times the CPU restatement of the reference's plain-array code (the oracle;
the reference itself is Julia and cannot run here) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

PEAK_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_by_path(name, path, search=None):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=search)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {k: float(d[k]) for k in PEAK_FALLBACK if k in d} | {"source": "measured"}
    return dict(PEAK_FALLBACK, source="fallback")


def synth():
    return load_by_path("tylo_b200_synth", ROOT / "tylo.jl_b200" / "synth.py")


def oracle():
    """The CPU checker (float64 restatement of the reference's plain-array code): used after a timed
    region to verify a sample of its output, and as the timed CPU baseline; never on the product path."""
    return load_by_path("tylo_oracle", ROOT / "oracle" / "tylo_oracle.py")


def f64(x):
    import torch
    return x.detach().to(torch.float64).cpu().numpy()


def parity(got, ref, sample, tol=(2e-2, 2e-3), grad=False):
    """Error of a bf16 result against the oracle: max-abs and mean-abs, with the contract's bounds
    (2e-2, 2e-3; for a gradient times max(1, P / 4), P the power of two at or above max|ref|: bf16 results
    in [P/2, P) are spaced P * 2^-8 apart, so rounding alone reaches P * 2^-9)."""
    import numpy as np
    err = np.abs(f64(got) - ref)
    top = float(np.abs(ref).max())
    s = max(1.0, 2.0 ** math.ceil(math.log2(top)) / 4) if grad and top > 0 else 1.0
    out = {"max_abs": float(err.max()), "mean_abs": float(err.mean()), "bound_max": tol[0] * s, "bound_mean": tol[1] * s,
           "sample": sample}
    out["ok"] = bool(out["max_abs"] <= out["bound_max"] and out["mean_abs"] <= out["bound_mean"] and np.isfinite(err).all())
    return out


def worst(parts):
    """Folds several parity records into one (largest error relative to its bound)."""
    key = lambda p: max(p["max_abs"] / p["bound_max"], p["mean_abs"] / p["bound_mean"])
    w = dict(max(parts, key=key))
    w["ok"] = all(p["ok"] for p in parts)
    w["checks"] = len(parts)
    return w


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[1])); mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# workloads.  Each returns a dict with: step() (one pass, device-resident inputs), work (algorithmic
# FLOPs or bytes per step on this rank), unit, bound, launches per step, and for the headline an
# e2e_step() that stages host buffers in and the result out.
# ------------------------------------------------------------------------------------------------
C3 = dict(B=4, S=4096, H=32, Hkv=8, D=128)
C4 = dict(B=2, S=8192, H=16, D=128, window=1024, ndocs=8, cap=50.0)
C5A = dict(B=64, H=64, Hkv=8, D=128, Smax=32768, lo=1024)
C5B = dict(B=1, H=64, Hkv=8, D=128, S=1 << 20)
ROWS = dict(softmax=(4096, 32768), norm=(16384, 8192))
GRAPH_STEPS = 8     # decode steps captured in one CUDA graph by the multi-GPU decode workloads


def shrink():
    """--small: same kernels and tile shapes on a few hundred MB, for profiler captures (a capture
    replays each launch dozens of times; the full-size workloads would take minutes per kernel)."""
    C3.update(B=1); C4.update(B=1, H=16); C5A.update(B=8); C5B.update(S=1 << 17)
    ROWS.update(softmax=(1024, 32768), norm=(4096, 8192))


def causal_pairs(S):
    return S * (S + 1) // 2


def make_prefill(t, torch, seed, bwd=False, rank=0, world=1, sharded=False):
    """Config 3.  Replicated (default): every rank runs the whole batch-4 problem.  `sharded`: one batch-4
    problem whose (kv-head, batch) units are cut into contiguous slabs, one range per rank; a slab is a
    contiguous piece of the (B, H, S, D) arrays, so each rank generates and holds only its own part."""
    import numpy as np
    sy = synth()
    c = C3
    B, H, Hkv, S, D = c["B"], c["H"], c["Hkv"], c["S"], c["D"]
    G = H // Hkv
    BF = torch.bfloat16
    if sharded:
        sharding = load_by_path("tylo_b200_sharding", ROOT / "tylo.jl_b200" / "sharding.py")
        slabs = sharding.prefill_shard(Hkv, B, rank, world)
    else:
        slabs = [(b, 0, Hkv) for b in range(B)]
    parts = []
    for (b, h0, h1) in slabs:
        n = h1 - h0
        qs, ks = ((b * H + h0 * G) * S) * D, ((b * Hkv + h0) * S) * D
        Q = sy.normal_cuda(seed, 0, (1, n * G, S, D), BF, start=qs)
        K = sy.normal_cuda(seed, 1, (1, n, S, D), BF, start=ks)
        V = sy.normal_cuda(seed, 2, (1, n, S, D), BF, start=ks)
        parts.append(dict(b=b, h0=h0, n=n, qs=qs, ks=ks, Q=Q, K=K, V=V))
    if not sharded:   # one launch over the whole batch: the slabs of a batch-major array are adjacent
        Q, K, V = (torch.cat([x[k] for x in parts]) for k in "QKV")
        parts = [dict(b=0, h0=0, n=Hkv, qs=0, ks=0, Q=Q, K=K, V=V)]
    for x in parts:
        x["O"] = torch.empty_like(x["Q"])
        x["cp"] = t.allocate_checkpoints_attention(x["Q"], x["K"], x["V"])
    units = sum(x["Q"].shape[0] * x["n"] for x in parts)
    pairs_unit = causal_pairs(S) * G
    name = ("prefill_bwd" if bwd else "prefill_fwd") + ("_sharded" if sharded else "")
    w = dict(name=name, unit="TFLOP/s", bound="tensor", scale=1e-12)
    if not bwd and not sharded and B == 4:
        # DRAM bytes of one launch of the forward kernel on this very workload (batch 4, one launch per step):
        # dram__bytes_read.sum 201,710,080 + dram__bytes_write.sum 104,483,584 from a one-launch, three-metric
        # ncu capture; the algorithmic bytes are 339.7 MB (Q, O 134.2 MB each, K + V 67.1 MB, statistics 4.2 MB),
        # the difference being output still in L2 when the kernel ends.
        w["traffic"] = 306193664
        w["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum, one full-size launch (see profiles/)"

    def fwd():
        for x in parts:
            t.attention_(x["O"], x["Q"], x["K"], x["V"], causal=True, checkpoints=x["cp"])

    def sample_inputs(x, hk):
        """float64 inputs of kv head `hk` (of the part's first batch entry) from the generator, on the CPU."""
        q0, k0 = x["qs"] + hk * G * S * D, x["ks"] + hk * S * D
        return (sy.rounded_numpy(seed, 0, q0, q0 + G * S * D, BF).reshape(1, G, S, D),
                sy.rounded_numpy(seed, 1, k0, k0 + S * D, BF).reshape(1, 1, S, D),
                sy.rounded_numpy(seed, 2, k0, k0 + S * D, BF).reshape(1, 1, S, D),
                sy.rounded_numpy(seed, 3, q0, q0 + G * S * D, BF).reshape(1, G, S, D))

    if not bwd:
        flops = 4 * D * pairs_unit
        w.update(step=fwd, work=flops * units, launches=len(parts))

        def verify():
            o = oracle()
            x = parts[-1]; hk = x["n"] - 1; hs = slice(hk * G, (hk + 1) * G)
            Q64, K64, V64, _ = sample_inputs(x, hk)
            Oref, Mref, Lref = o.flex_ref(Q64, K64, V64, mask=o.MaskSpec(causal=True), return_stats=True)
            what = f"all {G} query heads of (batch {x['b']}, kv head {x['h0'] + hk}), every row"
            p = parity(x["O"][:1, hs], Oref, what)
            lse = f64(x["cp"].M[:1, hs]) * np.log(2.0) + np.log(f64(x["cp"].L[:1, hs]))
            p["lse_max_abs"] = float(np.abs(lse - (Mref + np.log(Lref))).max())
            p["ok"] = p["ok"] and p["lse_max_abs"] <= 2e-2
            return p
        w["verify"] = verify
        if not sharded:
            x = parts[0]
            hQ, hK, hV = (x[k].cpu().pin_memory() for k in "QKV")
            hO = torch.empty_like(x["O"], device="cpu").pin_memory()
            # End to end from pinned host tensors: every step copies Q, K, V in and O out.  The package's
            # host pipeline streams the batch entries through three streams so that inbound copies, kernels
            # and outbound copies overlap (within a step and across consecutive steps).
            hostpipe = load_by_path("tylo_b200_hostpipe", ROOT / "tylo.jl_b200" / "hostpipe.py")
            pipe = hostpipe.HostAttentionPipeline(t, B, H, Hkv, S, S, D, causal=True)
            w.update(e2e_step=lambda: pipe.run(hO, hQ, hK, hV), h2d=sum(x[k].numel() * 2 for k in "QKV"),
                     d2h=x["O"].numel() * 2, e2e_note="host pipeline: per-batch-entry copies and kernels overlapped on 3 streams")
    else:
        fwd()
        for x in parts:
            x["dO"] = sy.normal_cuda(seed, 3, tuple(x["O"].shape), BF, start=x["qs"])
            x["d"] = (t.Duplicated(x["O"], x["dO"]), t.Duplicated(x["Q"]), t.Duplicated(x["K"]), t.Duplicated(x["V"]))
            x["sc"] = t.allocate_scratchspace_grad_attention(x["Q"], x["K"], x["V"], x["O"])

        def bwd_step():
            for x in parts:
                t.grad_attention_(*x["d"], causal=True, checkpoints=x["cp"], scratch=x["sc"])

        w.update(step=bwd_step, work=10 * D * pairs_unit * units, launches=3 * len(parts))

        def verify():
            o = oracle()
            x = parts[-1]; hk = x["n"] - 1; hs = slice(hk * G, (hk + 1) * G)
            Q64, K64, V64, dO64 = sample_inputs(x, hk)
            rQ, rK, rV = o.attn_bwd_ref(dO64, Q64, K64, V64, causal=True)
            what = f"(batch {x['b']}, kv head {x['h0'] + hk}): dQ of its {G} query heads, dK, dV"
            _, Qd, Kd, Vd = x["d"]
            return worst([parity(Qd.shadow[:1, hs], rQ, what + " [dQ]", grad=True),
                          parity(Kd.shadow[:1, hk:hk + 1], rK, what + " [dK]", grad=True),
                          parity(Vd.shadow[:1, hk:hk + 1], rV, what + " [dV]", grad=True)])
        w["verify"] = verify
    if sharded:
        w["global_work"] = (10 if bwd else 4) * D * pairs_unit * Hkv * B
        # CTAs of the forward on this rank against its 148 SMs (each CTA owns 256 query rows of one head)
        w["waves"] = units * G * ((S + 255) // 256) / 148.0
    w["config"] = dict(workload="causal GQA prefill %s, bf16%s" % ("backward" if bwd else "forward",
                                                                    ", one batch-4 problem sharded over (kv-head, batch) units" if sharded else ""),
                       batch_per_gpu=(None if sharded else B), batch=B, seq_len=S, heads_q=H, heads_kv=Hkv, head_dim=D,
                       units_per_gpu=units if sharded else Hkv * B)
    return w


def documents(B, S, ndocs, seed):
    """Per sequence `ndocs - 1` distinct cut positions drawn uniformly from 1..S-1 (seeded, on the host);
    returns the (B, S) table of document ids and the cuts."""
    import numpy as np
    rng = np.random.default_rng(seed)
    tab = np.zeros((B, S), dtype=np.int32)
    cuts = []
    for b in range(B):
        c = np.sort(rng.choice(np.arange(1, S), size=ndocs - 1, replace=False))
        tab[b] = np.searchsorted(c, np.arange(S), side="right")
        cuts.append(c)
    return tab, cuts


def band_block_list(tab, S, W, T):
    """Host-built block list (mods.jl:436-476) of `causal & window W & document` for the document tables `tab` (B, S):
    T x T blocks, listed if any pair of the block survives in any batch entry, full if every pair survives in every
    batch entry.  Returns (count [nb], idx [nb, nb], full [nb, nb]) int32, key blocks in ascending order.  A query
    keeps the keys [lo(q), q] with lo non-decreasing in q, so both tests are two comparisons per block and entry."""
    import numpy as np
    nb = S // T
    los = []
    for b in range(tab.shape[0]):
        start = np.zeros(S, dtype=np.int64)
        first = np.r_[0, np.flatnonzero(np.diff(tab[b])) + 1]
        start[first] = first
        los.append(np.maximum(np.arange(S) - W, np.maximum.accumulate(start)))
    cnt = np.zeros(nb, np.int32); idx = np.zeros((nb, nb), np.int32); full = np.zeros((nb, nb), np.int32)
    for i in range(nb):
        r0, r1 = i * T, i * T + T - 1
        for j in range(i + 1):
            c0, c1 = j * T, j * T + T - 1
            qs = max(r0, c0)                                   # the first query of the block that may see the block's keys
            if any(lo[qs] <= c1 for lo in los):
                idx[i, cnt[i]] = j
                full[i, cnt[i]] = int(r0 >= c1 and all(lo[r1] <= c0 for lo in los))
                cnt[i] += 1
    return cnt, idx, full


def make_flex(t, torch, seed, bwd=False, block_list=False):
    import numpy as np
    sy = synth()
    c = C4
    B, H, S, D, W = c["B"], c["H"], c["S"], c["D"], c["window"]
    BF = torch.bfloat16
    Q, K, V = (sy.normal_cuda(seed, i, (B, H, S, D), BF) for i in range(3))
    tab, cuts = documents(B, S, c["ndocs"], seed)
    docs = torch.from_numpy(tab).cuda()
    mask = t.CausalMask() & t.SlidingWindowMask(W) & t.DocumentMask(docs)
    score = t.SoftCapScore(c["cap"])
    # exact count of unmasked pairs: per query, keys in [max(q - w, doc start), q]
    pairs = 0
    for b in range(B):
        start = np.zeros(S, dtype=np.int64)
        first = np.r_[0, np.flatnonzero(np.diff(tab[b])) + 1]
        start[first] = first
        start = np.maximum.accumulate(start)
        q = np.arange(S)
        pairs += int((q - np.maximum(q - W, start) + 1).sum())
    pairs *= H
    O = torch.empty_like(Q)
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    w = dict(name="flex_bwd" if bwd else ("flex_fwd_block_list" if block_list else "flex_fwd"), unit="TFLOP/s", bound="tensor",
             scale=1e-12)
    bm = None
    if block_list:
        # The same mask as a host-built BlockMask (mods.jl:436-476) of 64 x 64 blocks: a block is listed if any pair in
        # it survives in any batch entry, full if every pair survives in every batch entry (the list has no batch
        # axis; the mask mod still runs per pair in listed blocks that are not full).  A query keeps the keys
        # [lo(q), q] with lo non-decreasing in q, which makes both tests two comparisons per block and batch entry.
        T = 64
        cnt, idx, full = band_block_list(tab, S, W, T)
        bm = t.BlockMask(torch.from_numpy(cnt).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(full).cuda(), T, T)
        w["listed_blocks"] = int(cnt.sum()); w["full_blocks"] = int(full.sum())

    def band(b, h, k0):
        """Oracle inputs of the queries [k0, k0 + 1536) of (b, h) with every key they can see."""
        o = oracle()
        klo, hi = max(0, k0 - W), min(S, k0 + 1536)
        base = ((b * H + h) * S) * D
        sl = lambda tid, lo, n: sy.rounded_numpy(seed, tid, base + lo * D, base + (lo + n) * D, BF).reshape(1, 1, n, D)
        kw = dict(score=o.ScoreSpec([("softcap", c["cap"])]), input_pos=k0 - klo,
                  mask=o.MaskSpec(causal=True, window=W, doc_q=tab[b][klo:], doc_kv=tab[b][klo:]))
        return klo, hi, sl, kw

    b0, h0 = B - 1, H - 1
    k0 = min(int(cuts[b0][3]) // 128 * 128, S - 1536)            # a band with a document cut inside
    if not bwd:
        w.update(step=lambda: t.flex_attention_(O, Q, K, V, score_mod=score, mask_mod=mask, checkpoints=cp, block_mask=bm),
                 work=4 * D * pairs, launches=1)

        def verify():
            klo, hi, sl, kw = band(b0, h0, k0)
            ref = oracle().flex_ref(sl(0, k0, hi - k0), sl(1, klo, hi - klo), sl(2, klo, hi - klo), **kw)
            return parity(O[b0:b0 + 1, h0:h0 + 1, k0:hi], ref, f"queries {k0}..{hi - 1} of (batch {b0}, head {h0})")
        w["verify"] = verify
    else:
        t.flex_attention_(O, Q, K, V, score_mod=score, mask_mod=mask, checkpoints=cp)
        dO = sy.normal_cuda(seed, 3, tuple(O.shape), BF)
        Od, Qd, Kd, Vd = t.Duplicated(O, dO), t.Duplicated(Q), t.Duplicated(K), t.Duplicated(V)
        sc = t.allocate_scratchspace_grad_flex_attention(Q, K, V, O)
        w.update(step=lambda: t.grad_flex_attention_(Od, Qd, Kd, Vd, score_mod=score, mask_mod=mask, checkpoints=cp, scratch=sc),
                 work=10 * D * pairs, launches=3)

        def verify():
            klo, hi, sl, kw = band(b0, h0, k0)
            rQ, rK, rV, _ = oracle().flex_bwd_ref(sl(3, k0, hi - k0), sl(0, k0, hi - k0), sl(1, klo, hi - klo), sl(2, klo, hi - klo), **kw)
            what = f"(batch {b0}, head {h0}): dQ of queries {k0}..{hi - 1}, dK and dV of keys {k0}..{k0 + 511}"
            ks = slice(k0 - klo, k0 - klo + 512)
            return worst([parity(Qd.shadow[b0:b0 + 1, h0:h0 + 1, k0:hi], rQ, what + " [dQ]", grad=True),
                          parity(Kd.shadow[b0:b0 + 1, h0:h0 + 1, k0:k0 + 512], rK[:, :, ks], what + " [dK]", grad=True),
                          parity(Vd.shadow[b0:b0 + 1, h0:h0 + 1, k0:k0 + 512], rV[:, :, ks], what + " [dV]", grad=True)])
        w["verify"] = verify
    w["config"] = dict(workload="flex attention %s, bf16: causal & window 1024 & document, softcap 50" % ("backward" if bwd else "forward")
                       + (", walked over a host-built list of 64 x 64 blocks" if block_list else ""),
                       batch=B, seq_len=S, heads=H, head_dim=D, unmasked_pairs=pairs)
    if block_list:
        w["config"].update(listed_blocks=w.pop("listed_blocks"), full_blocks=w.pop("full_blocks"))
    return w


def make_variants(t, torch, seed, which):
    """Two score / mask variants of the flex path that run on the tensor-core kernels, at sizes of their own
    (not BASELINE.json configs; recorded so that these paths have a measured number and a parity check):
      flex_bias_fwd_bwd    BiasScore with a learnable (Sk, Sq, heads) table under a causal mask: forward, backward and
                           the table's gradient (B 2, H 8, S 2048, D 128; 134 MB table, read by both backward kernels);
      flex_block_list_fwd  host-built BlockMask (64 x 64 blocks of a causal 512-key window): the forward walks the
                           list (B 2, H 16, S 4096, D 128)."""
    import numpy as np
    sy = synth()
    BF = torch.bfloat16
    o = oracle
    if which == "bias":
        B, H, S, D = 2, 8, 2048, 128
        Q, K, V, dO = (sy.normal_cuda(seed, i, (B, H, S, D), BF) for i in range(4))
        bias = sy.normal_cuda(seed, 4, (1, H, S, S), torch.float32)
        mod, mask = t.BiasScore(bias), t.CausalMask()
        O = torch.empty_like(Q)
        cp = t.allocate_checkpoints_flex_attention(Q, K, V)
        d_mod = t.grad_shadow(mod)
        Od, Qd, Kd, Vd = t.Duplicated(O, dO), t.Duplicated(Q), t.Duplicated(K), t.Duplicated(V)
        sc = t.allocate_scratchspace_grad_flex_attention(Q, K, V, O)

        def step():
            t.flex_attention_(O, Q, K, V, score_mod=mod, mask_mod=mask, checkpoints=cp)
            t.grad_flex_attention_(Od, Qd, Kd, Vd, score_mod=mod, mask_mod=mask, d_score_mod=d_mod, checkpoints=cp, scratch=sc)

        def verify():
            b0, h0 = B - 1, H - 1
            d_mod.bias.zero_()
            step()
            sl = lambda x: f64(x[b0:b0 + 1, h0:h0 + 1])
            bias64 = f64(bias[:, h0:h0 + 1])
            kw = dict(score=o().ScoreSpec([("bias", bias64)]), mask=o().MaskSpec(causal=True))
            ref = o().flex_ref(sl(Q), sl(K), sl(V), **kw)
            rQ, rK, rV, pg = o().flex_bwd_ref(sl(dO), sl(Q), sl(K), sl(V), **kw)
            what = f"(batch {b0}, head {h0})"
            # the table gradient of head h0 sums both batch entries; the oracle slice has one: check dQ, dK, dV and O
            return worst([parity(O[b0:b0 + 1, h0:h0 + 1], ref, what + " [O]"),
                          parity(Qd.shadow[b0:b0 + 1, h0:h0 + 1], rQ, what + " [dQ]", grad=True),
                          parity(Kd.shadow[b0:b0 + 1, h0:h0 + 1], rK, what + " [dK]", grad=True),
                          parity(Vd.shadow[b0:b0 + 1, h0:h0 + 1], rV, what + " [dV]", grad=True)])
        pairs = causal_pairs(S) * H * B
        return dict(name="flex_bias_fwd_bwd", unit="TFLOP/s", bound="tensor", scale=1e-12, launches=4, step=step, verify=verify,
                    work=14 * D * pairs,
                    config=dict(workload="flex attention forward + backward with a BiasScore table and its gradient, bf16, causal",
                                batch=B, seq_len=S, heads=H, head_dim=D, bias_table_bytes=int(bias.numel() * 4)))
    B, H, S, D, W, T = 2, 16, 4096, 128, 512, 64
    Q, K, V = (sy.normal_cuda(seed, i, (B, H, S, D), BF) for i in range(3))
    nqb = S // T
    cnt = np.zeros(nqb, np.int32); idx = np.zeros((nqb, nqb), np.int32); full = np.zeros((nqb, nqb), np.int32)
    for i in range(nqb):
        q_lo, q_hi = i * T, i * T + T - 1
        js = [j for j in range(nqb) if j * T <= q_hi and j * T + T - 1 >= q_lo - W]
        cnt[i] = len(js); idx[i, :len(js)] = js
        full[i, :len(js)] = [int(j * T + T - 1 <= q_lo and j * T >= q_hi - W) for j in js]
    bm = t.BlockMask(torch.from_numpy(cnt).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(full).cuda(), T, T)
    mask = t.CausalMask() & t.SlidingWindowMask(W)
    O = torch.empty_like(Q)
    q = np.arange(S)
    pairs = int((q - np.maximum(q - W, 0) + 1).sum()) * H * B

    def verify():
        b0, h0 = B - 1, H - 1
        sl = lambda x: f64(x[b0:b0 + 1, h0:h0 + 1])
        ref = o().flex_block_mask_ref(sl(Q), sl(K), sl(V), cnt, idx, full, TILE_M=T, TILE_N=T,
                                      mask=o().MaskSpec(causal=True, window=W))
        return parity(O[b0:b0 + 1, h0:h0 + 1], ref, f"(batch {b0}, head {h0}), every row, against the oracle's block walk")
    return dict(name="flex_block_list_fwd", unit="TFLOP/s", bound="tensor", scale=1e-12, launches=1, verify=verify,
                step=lambda: t.flex_attention_(O, Q, K, V, mask_mod=mask, block_mask=bm), work=4 * D * pairs,
                config=dict(workload="flex attention forward over a host-built block list (64 x 64 blocks, causal 512-key window), bf16",
                            batch=B, seq_len=S, heads=H, head_dim=D, unmasked_pairs=pairs))


def make_decode(t, torch, seed, long_ctx, rank=0, world=1, dist=None):
    import numpy as np
    sy = synth()
    c = C5B if long_ctx else C5A
    BF = torch.bfloat16
    B, H, Hkv, D = c["B"], c["H"], c["Hkv"], c["D"]
    G = H // Hkv
    Q = sy.normal_cuda(seed, 10 if long_ctx else 0, (B, H, D), BF)     # the same on every rank: q is replicated
    if long_ctx:
        S_all = c["S"]
        S_local = S_all // world                                  # contiguous KV range per rank
        k_begin = rank * S_local
        lengths_host = np.full(B, S_local, dtype=np.int64)
        total_len = S_all * B
        # this rank's keys of head hk are elements [(hk * S_all + k_begin) * D, ...) of the full (1, Hkv, S, D) array
        K = torch.empty(B, Hkv, S_local, D, device="cuda", dtype=BF); V = torch.empty_like(K)
        for hk in range(Hkv):
            a = (hk * S_all + k_begin) * D
            K[0, hk] = sy.normal_cuda(seed, 11, (S_local, D), BF, start=a)
            V[0, hk] = sy.normal_cuda(seed, 12, (S_local, D), BF, start=a)
    else:
        S_local = c["Smax"]
        lengths_host = sy.integers_numpy(seed, 3, 0, B, c["lo"], c["Smax"])
        total_len = int(lengths_host.sum())
        K = torch.empty(B, Hkv, S_local, D, device="cuda", dtype=BF); V = torch.empty_like(K)
        for b in range(B):                                           # filled per batch entry: keeps temporaries small
            a = b * Hkv * S_local * D
            K[b] = sy.normal_cuda(seed, 1, (Hkv, S_local, D), BF, start=a)
            V[b] = sy.normal_cuda(seed, 2, (Hkv, S_local, D), BF, start=a)
    lengths = torch.from_numpy(lengths_host.astype(np.int32)).cuda()
    O = torch.empty_like(Q)
    n_splits = t.decode_suggest_splits(S_local, Hkv, B)
    if long_ctx and world > 1:
        # the two-launch sharded step (split kernel, then the exchange kernel placed under its tail) measured best
        # with two CTAs per SM: 107 us per step at 8 GPUs against 115 us with the one per SM suggested for a
        # stand-alone 537 MB cache
        n_splits = max(n_splits, -(-2 * torch.cuda.get_device_properties(0).multi_processor_count // (Hkv * B)))
    sc = t.allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
    kv_bytes = total_len * Hkv * 2 * D * 2                       # live K+V bytes over all ranks
    w = dict(name="decode_1m" if long_ctx else "decode_ragged", unit="GB/s", bound="hbm", scale=1e-9, launches=2)
    if long_ctx and world > 1:
        # Receive buffers shared over CUDA IPC; the merge across GPUs happens inside the library's own
        # kernels (peer stores over NVLink + flags), no collective-library call on the data path.
        ex = t.DecodeExchange(B, H, D, rank=rank, world=world)
        w["exchange"] = ex

        def step():
            t.sharded_decode_attention_(O, Q, K, V, lengths_local=lengths, exchange=ex, scratch=sc)

        # The sharded step is short (~80 us of work per GPU at 8 GPUs): replay it as one CUDA graph so that
        # launch gaps do not dominate.  Falls back to eager launches if capture fails.
        eager = step
        eager(); torch.cuda.synchronize(); dist.barrier()
        per_graph = 1
        try:
            # a decode loop replays as a graph of several steps (the host launches one graph per GRAPH_STEPS tokens);
            # one timed "step" of this workload is one replay, its work GRAPH_STEPS decode steps
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(GRAPH_STEPS):
                    eager()
            step = graph.replay
            w["graphed"] = True
            per_graph = GRAPH_STEPS
        except Exception:
            step = eager
            w["graphed"] = False
        w.update(step=step, work=per_graph * (kv_bytes // world), launches=per_graph * t.SHARDED_DECODE_LAUNCHES,
                 global_work=per_graph * kv_bytes, decode_steps_per_step=per_graph)

        def verify():
            # (1) this rank's merged record of two heads against the oracle's partial over the rank's own keys;
            # (2) every rank's record gathered and merged on the host with the oracle's merge algebra, against
            #     the output the exchange left on this rank.
            o = oracle()
            # (the one-launch step folds groups of partials in place, so the record is rebuilt here from a
            # plain split pass over the same keys)
            vs = t.allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
            t.decode_split_(Q, K, V, lengths=lengths, scratch=vs)
            merged = t.allocate_scratchspace_decode_attention(O, Q, n_splits=1)
            t.decode_combine_(None, vs.O_partial, vs.M_partial, vs.L_partial, n_splits=n_splits, o_stride=B * H * D,
                              ml_stride=B * H, Dv=D, H=H, B=B, merged=merged)
            checks = []
            for h in (0, H - 1):
                hk = h // G
                Or, Mr, Lr = o.decode_partials(f64(Q[:, h:h + 1]), f64(K[:, hk:hk + 1]), f64(V[:, hk:hk + 1]), [S_local], 0, S_local)
                checks.append(parity(merged.O_partial[0, :, h:h + 1], Or, f"rank {rank}: merged local record of head {h} (keys {k_begin}..{k_begin + S_local - 1})"))
                lse_err = abs(float(merged.M_partial[0, 0, h]) + math.log2(float(merged.L_partial[0, 0, h])) - float(Mr[0, 0] + np.log2(Lr[0, 0])))
                checks[-1]["ok"] = checks[-1]["ok"] and lse_err < 1e-2
            rec = torch.cat([merged.O_partial.flatten(), merged.M_partial.flatten(), merged.L_partial.flatten()])
            allrec = [torch.empty_like(rec) for _ in range(world)]
            dist.all_gather(allrec, rec)
            n = B * H * D
            Os = np.stack([f64(r[:n]).reshape(B, H, D) for r in allrec]); Ms = np.stack([f64(r[n:n + B * H]).reshape(B, H) for r in allrec])
            Ls = np.stack([f64(r[n + B * H:]).reshape(B, H) for r in allrec])
            checks.append(parity(O, o.decode_combine(Os, Ms, Ls), f"rank {rank}: exchanged output of all {H} heads against the host merge of the {world} ranks' records"))
            return worst(checks)
        w["verify"] = verify
        w["verify_all_ranks"] = True
    else:
        w.update(step=lambda: t.decode_attention_(O, Q, K, V, lengths=lengths, scratch=sc), work=kv_bytes)   # replicas at N > 1

        def verify():
            o = oracle()
            if long_ctx:
                hk = Hkv - 1; hs = slice(hk * G, (hk + 1) * G)
                ref = o.decode_reference(f64(Q[:, hs]), f64(K[:, hk:hk + 1]), f64(V[:, hk:hk + 1]), [S_local])
                return parity(O[:, hs], ref, f"the {G} query heads of kv head {hk}, all {S_local} keys")
            checks = []
            for b in (int(np.argmax(lengths_host)), int(np.argmin(lengths_host))):
                n = int(lengths_host[b])
                ref = o.decode_reference(f64(Q[b:b + 1]), f64(K[b:b + 1, :, :n]), f64(V[b:b + 1, :, :n]), [n])
                checks.append(parity(O[b:b + 1], ref, f"sequence {b} (length {n}), all {H} heads"))
            return worst(checks)
        w["verify"] = verify
    w["config"] = dict(workload=("split-KV decode, bf16, 1 sequence x 1,048,576 keys" + (f", KV sharded over {world} GPUs, merged by the library's exchange kernel (peer stores over NVLink, placed under the split kernel's tail)" if world > 1 else ""))
                       if long_ctx else "split-KV decode, bf16, 64 sequences, lengths U[1024,32768]",
                       heads_q=H, heads_kv=Hkv, head_dim=D, n_splits=n_splits, live_kv_bytes=kv_bytes,
                       cuda_graph=w.get("graphed", False), decode_steps_per_graph=w.get("decode_steps_per_step", 1))
    return w


def make_decode_heads(t, torch, seed, rank, world):
    """Config 5b cut the other way: the 8 KV heads (with their query heads) are divided over the GPUs, every GPU
    keeps ALL 1,048,576 keys of its heads.  The same bytes per GPU as the key-range sharding of `decode_1m`, but
    the GPUs' outputs are disjoint (query heads), so there is nothing to exchange — the layout a tensor-parallel
    decoder has anyway (heads sharded, the output projection row-parallel).  Only divides as far as the KV heads
    go (8).  Strong scaling: value = the whole cache's bytes / the slowest rank's step."""
    import numpy as np
    sy = synth()
    c = C5B
    BF = torch.bfloat16
    B, H, Hkv, D, S = c["B"], c["H"], c["Hkv"], c["D"], c["S"]
    G = H // Hkv
    sharding = load_by_path("tylo_b200_sharding", ROOT / "tylo.jl_b200" / "sharding.py")
    hk0, hk1, _, _ = sharding.head_shard(Hkv, G, rank, world)
    hk_n = hk1 - hk0
    Qall = sy.normal_cuda(seed, 10, (B, H, D), BF)
    Q = Qall[:, hk0 * G:(hk0 + hk_n) * G].contiguous()
    K = torch.empty(B, hk_n, S, D, device="cuda", dtype=BF); V = torch.empty_like(K)
    for i in range(hk_n):
        a = ((hk0 + i) * S) * D
        K[0, i] = sy.normal_cuda(seed, 11, (S, D), BF, start=a)
        V[0, i] = sy.normal_cuda(seed, 12, (S, D), BF, start=a)
    lengths = torch.full((B,), S, dtype=torch.int32, device="cuda")
    O = torch.empty_like(Q)
    n_splits = t.decode_suggest_splits(S, hk_n, B)
    sc = t.allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
    kv_bytes = S * B * Hkv * 2 * D * 2
    eager = lambda: t.decode_attention_(O, Q, K, V, lengths=lengths, scratch=sc)
    step, graphed, per_graph = eager, False, 1
    if world > 1:
        eager(); torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(GRAPH_STEPS):
                    eager()
            step, graphed, per_graph = graph.replay, True, GRAPH_STEPS
        except Exception:
            step = eager

    def verify():
        i = hk_n - 1
        hs = slice(i * G, (i + 1) * G)
        ref = oracle().decode_reference(f64(Q[:, hs]), f64(K[:, i:i + 1]), f64(V[:, i:i + 1]), [S])
        return parity(O[:, hs], ref, f"rank {rank}: the {G} query heads of kv head {hk0 + i}, all {S} keys")
    w = dict(name="decode_1m_heads", unit="GB/s", bound="hbm", scale=1e-9, launches=1, step=step, verify=verify,
             work=per_graph * (kv_bytes // world), global_work=per_graph * kv_bytes, verify_all_ranks=True,
             decode_steps_per_step=per_graph,
             config=dict(workload="split-KV decode, bf16, 1 sequence x 1,048,576 keys, KV heads divided over the GPUs (no exchange)",
                         heads_q=H, heads_kv=Hkv, head_dim=D, kv_heads_per_gpu=hk_n, n_splits=n_splits, live_kv_bytes=kv_bytes,
                         cuda_graph=graphed, decode_steps_per_graph=per_graph))
    return w


def make_rowwise(t, torch, seed, kind):
    """Row kernels, forward (`softmax`, `rms_norm`, `layer_norm`) and backward (`*_bwd`).  Algorithmic bytes:
    forward one read + one write of the matrix; backward two reads (the saved tensor and the incoming
    gradient) + one write, 2 bytes each; parameter vectors and per-group partials are not counted."""
    sy = synth()
    BF = torch.bfloat16
    bwd = kind.endswith("_bwd")
    base = kind[:-4] if bwd else kind
    launches = 1
    rows = slice(0, 48)
    if base == "softmax":
        N, M = ROWS["softmax"]
        X = sy.normal_cuda(seed, 4, (N, M), BF, scale=2.0)
        Y = torch.empty_like(X)
        step = lambda: t.softmax_(Y, X)
        verify = lambda: parity(Y[rows], oracle().softmax_ref(f64(X[rows])), "first 48 rows")
        if bwd:
            step()
            dY = sy.normal_cuda(seed, 5, (N, M), BF)
            Yd, Xd = t.Duplicated(Y, dY), t.Duplicated(X)
            step = lambda: t.grad_softmax_(Yd, Xd)
            verify = lambda: parity(Xd.shadow[rows], oracle().softmax_bwd_ref(f64(dY[rows]), f64(Y[rows])), "first 48 rows", grad=True)
    else:
        N, M = ROWS["norm"]
        X = sy.normal_cuda(seed, 0, (N, M), BF)
        W = sy.normal_cuda(seed, 1, (M,), BF, scale=0.02, shift=1.0)
        Bv = sy.normal_cuda(seed, 2, (M,), BF, scale=0.02)
        Y = torch.empty_like(X)
        o = oracle
        if base == "rms_norm":
            cp = t.allocate_checkpoints_rms_norm(X, W)
            step = lambda: t.rms_norm_(Y, X, W, eps=1e-6, checkpoints=cp if bwd else None)
            verify = lambda: parity(Y[rows], o().rms_norm_ref(f64(X[rows]), f64(W), eps=1e-6), "first 48 rows", tol=(4e-2, 2e-3))
        else:
            cp = t.allocate_checkpoints_layer_norm(X, W, Bv)
            step = lambda: t.layer_norm_(Y, X, W, Bv, eps=1e-6, checkpoints=cp if bwd else None)
            verify = lambda: parity(Y[rows], o().layer_norm_ref(f64(X[rows]), f64(W), f64(Bv), eps=1e-6), "first 48 rows", tol=(4e-2, 2e-3))
        if bwd:
            step()
            dY = sy.normal_cuda(seed, 3, (N, M), BF)
            Yd, Xd, Wd = t.Duplicated(Y, dY), t.Duplicated(X), t.Duplicated(W)
            launches = 2
            if base == "rms_norm":
                sc = t.allocate_scratchspace_grad_rms_norm(X, W)
                step = lambda: t.grad_rms_norm_(Yd, Xd, Wd, checkpoints=cp, scratch=sc)
                verify = lambda: parity(Xd.shadow[rows], o().rms_norm_bwd_ref(f64(dY[rows]), f64(X[rows]), f64(W), eps=1e-6)[0],
                                        "dX of the first 48 rows", tol=(4e-2, 2e-3), grad=True)
            else:
                Bd = t.Duplicated(Bv)
                sc = t.allocate_scratchspace_grad_layer_norm(X, W, Bv)
                step = lambda: t.grad_layer_norm_(Yd, Xd, Wd, Bd, checkpoints=cp, scratch=sc)
                verify = lambda: parity(Xd.shadow[rows], o().layer_norm_bwd_ref(f64(dY[rows]), f64(X[rows]), f64(W), eps=1e-6)[0],
                                        "dX of the first 48 rows", tol=(4e-2, 2e-3), grad=True)
    return dict(name=kind, unit="GB/s", bound="hbm", scale=1e-9, launches=launches, step=step, verify=verify,
                work=N * M * (6 if bwd else 4),
                config=dict(workload=f"{base} {'backward' if bwd else 'forward'}, bf16", rows=N, row_len=M))


def make_fp32(t, torch, seed, tf32=False):
    """Config 1 (Float32, non-causal, B 2, H 8, S 512, D 64).  Default: true fp32 arithmetic, held to 1e-5 relative.
    `tf32`: the opt-in tensor-core form (`tensorcore=TFloat32`, the reference's default for Float32), held to
    max-abs 4e-3 / mean-abs 4e-4 (10-bit operand mantissas)."""
    sy = synth()
    Q, K, V = (sy.normal_cuda(seed, i, (2, 8, 512, 64), torch.float32) for i in range(3))
    O = torch.empty_like(Q)
    kw = dict(tensorcore=t.TFloat32) if tf32 else {}

    def verify():
        import numpy as np
        ref = oracle().attn_ref(f64(Q), f64(K), f64(V))
        err = np.abs(f64(O) - ref)
        if tf32:
            bmax, bmean = 4e-3 * max(1.0, float(np.abs(ref).max())), 4e-4
        else:
            bmax = bmean = 1e-5 * float(np.abs(ref).max()) + 1e-6
        return {"max_abs": float(err.max()), "mean_abs": float(err.mean()), "bound_max": bmax, "bound_mean": bmean,
                "sample": "every element", "ok": bool(err.max() <= bmax and err.mean() <= bmean)}
    what = "TF32 operands on the tensor cores, fp32 accumulation and softmax" if tf32 else "true fp32 arithmetic"
    return dict(name="mha_tf32" if tf32 else "mha_fp32", unit="TFLOP/s", bound="tensor", scale=1e-12, launches=1, verify=verify,
                step=lambda: t.attention_(O, Q, K, V, **kw), work=4 * 64 * 512 * 512 * 16,
                config=dict(workload=f"fused MHA forward, fp32 storage ({what}), non-causal", batch=2, seq_len=512, heads=8,
                            head_dim=64))


def time_steps(torch, step, steps, warmup, sync_all=None):
    for _ in range(warmup):
        step()
    if sync_all:
        sync_all()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if sync_all:
        sync_all()
    return e0.elapsed_time(e1) / steps  # ms per step


# ------------------------------------------------------------------------------------------------
# CPU baseline (the oracle timed on the host cores)
# ------------------------------------------------------------------------------------------------
def cpu_prefill_sample(n_heads=4, S=C3["S"], D=C3["D"]):
    """Causal attention forward of `n_heads` (batch, head) slices of the config-3 problem with the
    oracle.  Returns (seconds, FLOPs counted on unmasked pairs)."""
    import numpy as np
    oracle = load_by_path("tylo_oracle", ROOT / "oracle" / "tylo_oracle.py")
    rng = np.random.default_rng(2)
    Q = rng.standard_normal((1, n_heads, S, D)); K = rng.standard_normal((1, max(1, n_heads // 4), S, D))
    V = rng.standard_normal(K.shape)
    t0 = time.perf_counter()
    oracle.attn_ref(Q, K, V, causal=True)
    return time.perf_counter() - t0, 4 * D * causal_pairs(S) * n_heads


def cpu_baseline(budget_s=20.0):
    n, dt, fl = 1, *cpu_prefill_sample(1)
    while dt < budget_s / 4 and n < 64:
        n *= 4
        dt, fl = cpu_prefill_sample(n)
    return {"value": fl / dt * 1e-12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n} of {C3['B'] * C3['H']} (batch, head) slices of the config-3 forward, NumPy float64 oracle"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = 4
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_prefill_sample(1)
    t0 = time.perf_counter(); fl = 0
    for _ in range(args.steps):
        _, f = cpu_prefill_sample(n); fl += f
    dt = time.perf_counter() - t0
    v = fl / dt * 1e-12
    c = C3
    sample = f"each step = {n} of the {c['B'] * c['H']} (batch, head) slices of the config-3 forward"
    line = {"impl": "reference", "metric": "prefill_attn_fwd_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "causal GQA prefill forward, bf16", "batch_per_gpu": c["B"], "batch": c["B"],
                       "seq_len": c["S"], "heads_q": c["H"], "heads_kv": c["Hkv"], "head_dim": c["D"],
                       "units_per_gpu": c["Hkv"] * c["B"], "l2": "inputs exceed the 126 MB L2; no flush between steps",
                       "sample": sample},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="prefill_fwd")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--extras", default="", help="comma-separated subset of extras")
    ap.add_argument("--small", action="store_true", help="reduced sizes for profiler captures (not a bench result)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check of each workload's output (profiler runs)")
    ap.add_argument("--sustained-seconds", type=float, default=2.0, help="length of the sustained-clock loop of the headline")
    args = ap.parse_args()
    if args.small:
        shrink()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device (libtylo_b200 has no CPU path); use --impl reference for the CPU baseline")
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    t = load_by_path("tylo_b200", ROOT / "tylo.jl_b200" / "__init__.py", [str(ROOT / "tylo.jl_b200")])
    pk = peaks()

    def sync_all():
        if dist is not None:
            dist.barrier()

    def all_ranks_ok(ok):
        if world == 1:
            return ok
        v = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(v, op=dist.ReduceOp.MIN)
        return bool(v.item() > 0.5)

    def max_over_ranks(ms):
        if dist is None:
            return ms
        x = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x.item())

    makers = {
        "prefill_fwd": lambda: make_prefill(t, torch, 2),
        "prefill_bwd": lambda: make_prefill(t, torch, 2, bwd=True),
        "prefill_fwd_sharded": lambda: make_prefill(t, torch, 2, rank=rank, world=world, sharded=True),
        "prefill_bwd_sharded": lambda: make_prefill(t, torch, 2, bwd=True, rank=rank, world=world, sharded=True),
        "flex_fwd": lambda: make_flex(t, torch, 3),
        "flex_bwd": lambda: make_flex(t, torch, 3, bwd=True),
        "decode_ragged": lambda: make_decode(t, torch, 4, False),
        "decode_1m": lambda: make_decode(t, torch, 4, True, rank, world, dist),
        "decode_1m_heads": lambda: make_decode_heads(t, torch, 4, rank, world),
        "rms_norm": lambda: make_rowwise(t, torch, 1, "rms_norm"),
        "layer_norm": lambda: make_rowwise(t, torch, 1, "layer_norm"),
        "softmax": lambda: make_rowwise(t, torch, 1, "softmax"),
        "rms_norm_bwd": lambda: make_rowwise(t, torch, 1, "rms_norm_bwd"),
        "layer_norm_bwd": lambda: make_rowwise(t, torch, 1, "layer_norm_bwd"),
        "softmax_bwd": lambda: make_rowwise(t, torch, 1, "softmax_bwd"),
        "mha_fp32": lambda: make_fp32(t, torch, 0),
        "mha_tf32": lambda: make_fp32(t, torch, 0, tf32=True),
        "flex_fwd_block_list": lambda: make_flex(t, torch, 3, block_list=True),
        "flex_bias_fwd_bwd": lambda: make_variants(t, torch, 5, "bias"),
        "flex_block_list_fwd": lambda: make_variants(t, torch, 6, "block_list"),
    }

    def roofline(w, ms):
        ach = w["work"] * w["scale"] / (ms * 1e-3)
        if w["bound"] == "hbm":
            peak, unit = pk["hbm_gbs"], "GB/s"
        else:
            peak, unit = pk["bf16_tflops"], "TFLOP/s"
        return {"bound": w["bound"], "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                "traffic": w.get("traffic"), "traffic_source": w.get("traffic_source"), "peak_source": pk["source"]}

    def replicated(w):   # whole-job work for this workload
        return w.get("global_work", w["work"] * world)

    def verified(w):
        """Oracle check of a sample of the workload's output, after its timed region.  Replicated workloads
        are checked on rank 0; sharded ones on every rank (each checks its own shard), worst case reported."""
        if args.no_verify or "verify" not in w:
            return None
        every = w.get("verify_all_ranks", False) or ("global_work" in w and world > 1)
        rec = None
        if rank == 0 or every:
            try:
                rec = w["verify"]()
            except Exception as e:
                rec = {"ok": False, "error": f"{type(e).__name__}: {e}"}
        if every and world > 1:
            recs = [None] * world
            dist.all_gather_object(recs, rec)
            bad = [r for r in recs if not r.get("ok", False)]
            rec = bad[0] if bad else max(recs, key=lambda r: r["max_abs"] / r["bound_max"])
            rec["ranks_checked"] = world
        return rec

    with ClockSampler(local) as clk:
        w = makers[args.workload]()
        ms = max_over_ranks(time_steps(torch, w["step"], args.steps, args.warmup, sync_all))
    clocks = clk.summary()
    headline_parity = verified(w)
    value = replicated(w) * w["scale"] / (ms * 1e-3)
    line = {"metric": {"prefill_fwd": "prefill_attn_fwd_tflops"}.get(w["name"], w["name"]), "value": value, "unit": w["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if "global_work" in w and world > 1 else "weak", "vs_baseline": None,
            "dtype": {"mha_fp32": "f32", "mha_tf32": "tf32"}.get(w["name"], "bf16"), "data": "synthetic",
            "config": dict(w["config"], l2="inputs exceed the 126 MB L2; no flush between steps"),
            "roofline": roofline(w, ms), "gpu_launches": w["launches"] * args.steps, "clocks": clocks}
    if headline_parity is not None:
        line["parity"] = headline_parity
    if "waves" in w:
        line["config"]["forward_ctas_per_sm"] = round(w["waves"], 2)
    if args.workload == "prefill_fwd" and args.sustained_seconds > 0 and not args.small:
        # The same launch back to back for seconds, with the clocks sampled meanwhile: what the kernel holds
        # once the part has settled under its power limit (the headline's timed region is a 12 ms burst).
        n = max(args.steps, int(args.sustained_seconds * 1e3 / ms) + 1)
        with ClockSampler(local) as sclk:
            sms = max_over_ranks(time_steps(torch, w["step"], n, 1, sync_all))
        sus = replicated(w) * w["scale"] / (sms * 1e-3)
        line["sustained"] = {"value": sus, "unit": w["unit"], "steps": n, "ms_per_step": sms, "seconds": sms * n * 1e-3,
                             "peak": pk.get("bf16_tflops_sustained"), "frac": sus / world / pk["bf16_tflops_sustained"]
                             if pk.get("bf16_tflops_sustained") else None, "clocks": sclk.summary()}
    if "e2e_step" in w:
        ems = max_over_ranks(time_steps(torch, w["e2e_step"], max(3, args.steps // 4), 2, sync_all))
        line["e2e"] = {"value": replicated(w) * w["scale"] / (ems * 1e-3), "unit": w["unit"], "ms_per_step": ems,
                       "h2d_bytes_per_step": w["h2d"], "d2h_bytes_per_step": w["d2h"], "how": w.get("e2e_note", "")}
    del w
    torch.cuda.empty_cache()

    if not args.no_extras:
        names = [n for n in makers if n != args.workload]
        if args.extras:
            names = [n for n in names if n in args.extras.split(",")]
        extras = {}
        for n in names:
            w, err = None, None
            try:
                w = makers[n]()
            except Exception as e:  # an extra must never take the headline down
                err = f"{type(e).__name__}: {e}"
            if not all_ranks_ok(err is None):      # every rank times the extra, or none does
                extras[n] = {"error": err or "setup failed on another rank"}
                w = None
                torch.cuda.empty_cache()
                continue
            try:
                k = max(3, min(args.steps, 10))
                ems = max_over_ranks(time_steps(torch, w["step"], k, 3, sync_all))
                if "exchange" in w:
                    w["exchange"].status()          # raises if a bounded wait for a peer's record gave up
                r = roofline(w, ems)
                extras[n] = {"value": replicated(w) * w["scale"] / (ems * 1e-3), "unit": w["unit"], "ms_per_step": ems,
                             "steps": k, "roofline_frac": r["frac"], "per_gpu": r["achieved"], "config": w["config"],
                             "scaling": "strong" if "global_work" in w and world > 1 else "weak"}
                if "waves" in w:
                    extras[n]["forward_ctas_per_sm"] = round(w["waves"], 2)
                if w.get("decode_steps_per_step", 1) > 1:
                    # one timed step of this workload is one graph replay of several decode steps
                    extras[n]["decode_steps_per_step"] = w["decode_steps_per_step"]
                    extras[n]["ms_per_decode_step"] = ems / w["decode_steps_per_step"]
                pr = verified(w)
                if pr is not None:
                    extras[n]["parity"] = pr
                    if not pr.get("ok", False):
                        extras[n]["error"] = "output outside tolerance of the CPU oracle: the number above is not a result"
            except Exception as e:
                extras[n] = {"error": f"{type(e).__name__}: {e}"}
            if w is not None and "exchange" in w:
                sync_all()
                w["exchange"].close()
            w = None
            torch.cuda.empty_cache()
        line["extras"] = extras

    if args.small:
        line["config"]["small"] = True
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
