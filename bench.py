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
library's own exchange kernel (peer stores over NVLink into IPC-shared buffers, one launch).

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


def shrink():
    """--small: same kernels and tile shapes on a few hundred MB, for profiler captures (a capture
    replays each launch dozens of times; the full-size workloads would take minutes per kernel)."""
    C3.update(B=1); C4.update(B=1, H=4); C5A.update(B=8); C5B.update(S=1 << 17)
    ROWS.update(softmax=(1024, 32768), norm=(4096, 8192))


def causal_pairs(S):
    return S * (S + 1) // 2


def make_prefill(t, torch, seed, bwd=False):
    c = C3
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    Q, K, V = mk(c["B"], c["H"], c["S"], c["D"]), mk(c["B"], c["Hkv"], c["S"], c["D"]), mk(c["B"], c["Hkv"], c["S"], c["D"])
    O = torch.empty_like(Q)
    cp = t.allocate_checkpoints_attention(Q, K, V)
    pairs = causal_pairs(c["S"]) * c["H"] * c["B"]
    w = dict(name="prefill_bwd" if bwd else "prefill_fwd", unit="TFLOP/s", bound="tensor", scale=1e-12)
    if not bwd:
        w.update(step=lambda: t.attention_(O, Q, K, V, causal=True, checkpoints=cp), work=4 * c["D"] * pairs, launches=1)
        # DRAM bytes per launch: read + written by the kernel in one profiler capture at batch 1
        # (50.5 MB + 2.5 MB; K/V re-reads hit L2), times the batch — traffic is per (batch, head).
        w.update(traffic=53.0e6 * c["B"], traffic_source="ncu dram__bytes_read+write at batch 1, scaled by batch")
        hQ, hK, hV = (x.cpu().pin_memory() for x in (Q, K, V))
        hO = torch.empty_like(O, device="cpu").pin_memory()
        # End to end from pinned host tensors: every step copies Q, K, V in and O out.  The package's
        # host pipeline streams the batch entries through three streams so that inbound copies, kernels
        # and outbound copies overlap (within a step and across consecutive steps).
        hostpipe = load_by_path("tylo_b200_hostpipe", ROOT / "tylo.jl_b200" / "hostpipe.py")
        pipe = hostpipe.HostAttentionPipeline(t, c["B"], c["H"], c["Hkv"], c["S"], c["S"], c["D"], causal=True)

        w.update(e2e_step=lambda: pipe.run(hO, hQ, hK, hV), h2d=sum(x.numel() * 2 for x in (Q, K, V)),
                 d2h=O.numel() * 2, e2e_note="host pipeline: per-batch-entry copies and kernels overlapped on 3 streams")
    else:
        t.attention_(O, Q, K, V, causal=True, checkpoints=cp)
        dO = mk(*O.shape)
        Od, Qd, Kd, Vd = t.Duplicated(O, dO), t.Duplicated(Q), t.Duplicated(K), t.Duplicated(V)
        sc = t.allocate_scratchspace_grad_attention(Q, K, V, O)
        w.update(step=lambda: t.grad_attention_(Od, Qd, Kd, Vd, causal=True, checkpoints=cp, scratch=sc),
                 work=10 * c["D"] * pairs, launches=3)
    w["config"] = dict(workload="causal GQA prefill %s, bf16" % ("backward" if bwd else "forward"), batch_per_gpu=c["B"],
                       seq_len=c["S"], heads_q=c["H"], heads_kv=c["Hkv"], head_dim=c["D"])
    return w


def make_flex(t, torch, seed, bwd=False):
    import numpy as np
    c = C4
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    Q, K, V = (mk(c["B"], c["H"], c["S"], c["D"]) for _ in range(3))
    rng = np.random.default_rng(seed)
    tab = np.zeros((c["B"], c["S"]), dtype=np.int32)
    for b in range(c["B"]):
        cuts = np.sort(rng.choice(np.arange(1, c["S"]), size=c["ndocs"] - 1, replace=False))
        tab[b] = np.searchsorted(cuts, np.arange(c["S"]), side="right")
    docs = torch.from_numpy(tab).cuda()
    mask = t.CausalMask() & t.SlidingWindowMask(c["window"]) & t.DocumentMask(docs)
    score = t.SoftCapScore(c["cap"])
    # exact count of unmasked pairs: per query, keys in [max(q - w, doc start), q]
    pairs = 0
    for b in range(c["B"]):
        start = np.zeros(c["S"], dtype=np.int64)
        first = np.r_[0, np.flatnonzero(np.diff(tab[b])) + 1]
        start[first] = first
        start = np.maximum.accumulate(start)
        q = np.arange(c["S"])
        pairs += int((q - np.maximum(q - c["window"], start) + 1).sum())
    pairs *= c["H"]
    O = torch.empty_like(Q)
    cp = t.allocate_checkpoints_flex_attention(Q, K, V)
    w = dict(name="flex_bwd" if bwd else "flex_fwd", unit="TFLOP/s", bound="tensor", scale=1e-12)
    if not bwd:
        w.update(step=lambda: t.flex_attention_(O, Q, K, V, score_mod=score, mask_mod=mask, checkpoints=cp),
                 work=4 * c["D"] * pairs, launches=1)
    else:
        t.flex_attention_(O, Q, K, V, score_mod=score, mask_mod=mask, checkpoints=cp)
        dO = mk(*O.shape)
        Od, Qd, Kd, Vd = t.Duplicated(O, dO), t.Duplicated(Q), t.Duplicated(K), t.Duplicated(V)
        sc = t.allocate_scratchspace_grad_flex_attention(Q, K, V, O)
        w.update(step=lambda: t.grad_flex_attention_(Od, Qd, Kd, Vd, score_mod=score, mask_mod=mask, checkpoints=cp, scratch=sc),
                 work=10 * c["D"] * pairs, launches=3)
    w["config"] = dict(workload="flex attention %s, bf16: causal & window 1024 & document, softcap 50" % ("backward" if bwd else "forward"),
                       batch=c["B"], seq_len=c["S"], heads=c["H"], head_dim=c["D"], unmasked_pairs=pairs)
    return w


def make_decode(t, torch, seed, long_ctx, rank=0, world=1, dist=None):
    c = C5B if long_ctx else C5A
    g = torch.Generator(device="cuda").manual_seed(seed)      # same seed on every rank: q is replicated
    B, H, Hkv, D = c["B"], c["H"], c["Hkv"], c["D"]
    Q = torch.randn(B, H, D, device="cuda", generator=g).to(torch.bfloat16)
    if long_ctx:
        S_local = c["S"] // world                                # contiguous KV range per rank
        lengths = torch.full((B,), S_local, dtype=torch.int32, device="cuda")
        total_len = c["S"] * B
    else:
        S_local = c["Smax"]
        lengths = torch.randint(c["lo"], c["Smax"] + 1, (B,), device="cuda", generator=g).to(torch.int32)
        total_len = int(lengths.sum().item())
    gk = torch.Generator(device="cuda").manual_seed(seed * 1000 + rank)
    K = torch.empty(B, Hkv, S_local, D, device="cuda", dtype=torch.bfloat16)
    V = torch.empty_like(K)
    for b in range(B):                                           # chunked fill keeps peak memory low
        K[b].copy_(torch.randn(Hkv, S_local, D, device="cuda", generator=gk)); V[b].copy_(torch.randn(Hkv, S_local, D, device="cuda", generator=gk))
    O = torch.empty_like(Q)
    n_splits = t.decode_suggest_splits(S_local, Hkv, B)
    sc = t.allocate_scratchspace_decode_attention(O, Q, n_splits=n_splits)
    kv_bytes = total_len * Hkv * 2 * D * 2                       # live K+V bytes over all ranks
    w = dict(name="decode_1m" if long_ctx else "decode_ragged", unit="GB/s", bound="hbm", scale=1e-9, launches=2)
    if long_ctx and world > 1:
        # Receive buffers shared over CUDA IPC; the merge across GPUs is one launch of the library's own
        # exchange kernel (peer stores over NVLink + flags), no collective-library call on the data path.
        ex = t.DecodeExchange(B, H, D, rank=rank, world=world)
        w["exchange"] = ex

        def step():
            t.sharded_decode_attention_(O, Q, K, V, lengths_local=lengths, exchange=ex, scratch=sc)

        # The sharded step is two short launches (~80 us of work per GPU at 8 GPUs): replay it as one
        # CUDA graph so that launch gaps do not dominate.  Falls back to eager launches if capture fails.
        eager = step
        eager(); torch.cuda.synchronize(); dist.barrier()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                eager()
            step = graph.replay
            w["graphed"] = True
        except Exception:
            step = eager
            w["graphed"] = False
        w.update(step=step, work=kv_bytes // world, launches=2, global_work=kv_bytes)
    else:
        w.update(step=lambda: t.decode_attention_(O, Q, K, V, lengths=lengths, scratch=sc), work=kv_bytes)   # replicas at N > 1
    w["config"] = dict(workload=("split-KV decode, bf16, 1 sequence x 1,048,576 keys" + (f", KV sharded over {world} GPUs, merged by one peer-store exchange launch over NVLink" if world > 1 else ""))
                       if long_ctx else "split-KV decode, bf16, 64 sequences, lengths U[1024,32768]",
                       heads_q=H, heads_kv=Hkv, head_dim=D, n_splits=n_splits, live_kv_bytes=kv_bytes,
                       cuda_graph=w.get("graphed", False))
    return w


def make_rowwise(t, torch, seed, kind):
    """Row kernels, forward (`softmax`, `rms_norm`, `layer_norm`) and backward (`*_bwd`).  Algorithmic bytes:
    forward one read + one write of the matrix; backward two reads (the saved tensor and the incoming
    gradient) + one write, 2 bytes each; parameter vectors and per-group partials are not counted."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    bwd = kind.endswith("_bwd")
    base = kind[:-4] if bwd else kind
    launches = 1
    if base == "softmax":
        N, M = ROWS["softmax"]
        X = (2 * torch.randn(N, M, device="cuda", generator=g)).to(torch.bfloat16)
        Y = torch.empty_like(X)
        step = lambda: t.softmax_(Y, X)
        if bwd:
            step()
            dY = torch.randn(N, M, device="cuda", generator=g).to(torch.bfloat16)
            Yd, Xd = t.Duplicated(Y, dY), t.Duplicated(X)
            step = lambda: t.grad_softmax_(Yd, Xd)
    else:
        N, M = ROWS["norm"]
        X = torch.randn(N, M, device="cuda", generator=g).to(torch.bfloat16)
        W = (1 + 0.02 * torch.randn(M, device="cuda", generator=g)).to(torch.bfloat16)
        Bv = (0.02 * torch.randn(M, device="cuda", generator=g)).to(torch.bfloat16)
        Y = torch.empty_like(X)
        if base == "rms_norm":
            cp = t.allocate_checkpoints_rms_norm(X, W)
            step = lambda: t.rms_norm_(Y, X, W, eps=1e-6, checkpoints=cp if bwd else None)
        else:
            cp = t.allocate_checkpoints_layer_norm(X, W, Bv)
            step = lambda: t.layer_norm_(Y, X, W, Bv, eps=1e-6, checkpoints=cp if bwd else None)
        if bwd:
            step()
            dY = torch.randn(N, M, device="cuda", generator=g).to(torch.bfloat16)
            Yd, Xd, Wd = t.Duplicated(Y, dY), t.Duplicated(X), t.Duplicated(W)
            launches = 2
            if base == "rms_norm":
                sc = t.allocate_scratchspace_grad_rms_norm(X, W)
                step = lambda: t.grad_rms_norm_(Yd, Xd, Wd, checkpoints=cp, scratch=sc)
            else:
                Bd = t.Duplicated(Bv)
                sc = t.allocate_scratchspace_grad_layer_norm(X, W, Bv)
                step = lambda: t.grad_layer_norm_(Yd, Xd, Wd, Bd, checkpoints=cp, scratch=sc)
    return dict(name=kind, unit="GB/s", bound="hbm", scale=1e-9, launches=launches, step=step,
                work=N * M * (6 if bwd else 4),
                config=dict(workload=f"{base} {'backward' if bwd else 'forward'}, bf16", rows=N, row_len=M))


def make_fp32(t, torch, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    Q, K, V = (torch.randn(2, 8, 512, 64, device="cuda", generator=g) for _ in range(3))
    O = torch.empty_like(Q)
    return dict(name="mha_fp32", unit="TFLOP/s", bound="tensor", scale=1e-12, launches=1,
                step=lambda: t.attention_(O, Q, K, V), work=4 * 64 * 512 * 512 * 16,
                config=dict(workload="fused MHA forward, fp32 (true fp32 arithmetic), non-causal", batch=2, seq_len=512, heads=8, head_dim=64))


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
    line = {"impl": "reference", "metric": "prefill_attn_fwd_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "causal GQA prefill forward (CPU restatement of the reference's plain-array code)",
                       "seq_len": C3["S"], "head_dim": C3["D"]},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                             "sample": f"each step = {n} (batch, head) slices of the config-3 forward"},
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
        "flex_fwd": lambda: make_flex(t, torch, 3),
        "flex_bwd": lambda: make_flex(t, torch, 3, bwd=True),
        "decode_ragged": lambda: make_decode(t, torch, 4, False),
        "decode_1m": lambda: make_decode(t, torch, 4, True, rank, world, dist),
        "rms_norm": lambda: make_rowwise(t, torch, 1, "rms_norm"),
        "layer_norm": lambda: make_rowwise(t, torch, 1, "layer_norm"),
        "softmax": lambda: make_rowwise(t, torch, 1, "softmax"),
        "rms_norm_bwd": lambda: make_rowwise(t, torch, 1, "rms_norm_bwd"),
        "layer_norm_bwd": lambda: make_rowwise(t, torch, 1, "layer_norm_bwd"),
        "softmax_bwd": lambda: make_rowwise(t, torch, 1, "softmax_bwd"),
        "mha_fp32": lambda: make_fp32(t, torch, 0),
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

    with ClockSampler(local) as clk:
        w = makers[args.workload]()
        ms = max_over_ranks(time_steps(torch, w["step"], args.steps, args.warmup, sync_all))
    clocks = clk.summary()
    value = replicated(w) * w["scale"] / (ms * 1e-3)
    line = {"metric": {"prefill_fwd": "prefill_attn_fwd_tflops"}.get(w["name"], w["name"]), "value": value, "unit": w["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if "global_work" in w and world > 1 else "weak", "vs_baseline": None,
            "dtype": "f32" if w["name"] == "mha_fp32" else "bf16", "data": "synthetic",
            "config": dict(w["config"], l2="inputs exceed the 126 MB L2; no flush between steps"),
            "roofline": roofline(w, ms), "gpu_launches": w["launches"] * args.steps, "clocks": clocks}
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
                             "steps": k, "roofline_frac": r["frac"], "per_gpu": r["achieved"], "config": w["config"]}
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
