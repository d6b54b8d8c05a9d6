"""Attention forward for HOST-resident tensors: batch entries stream through the GPU with the
host-to-device copy of entry b+1, the kernel of entry b and the device-to-host copy of entry b-1
running at the same time on three streams (PCIe is full duplex, so inbound and outbound copies overlap
too).  Calls may follow each other without a synchronise: entry b of the next call starts its inbound
copy as soon as the previous call's kernel on that entry's device buffers has finished.

The reference has no host-tensor entry point (its wrappers take device arrays,
src/attention/attention.jl:204-262); this is the thin host-side driver a caller with pinned host
buffers would write around `attention!`.
"""
from __future__ import annotations

import torch


class HostAttentionPipeline:
    def __init__(self, api, B: int, H: int, Hkv: int, Sq: int, Sk: int, D: int, *, dtype=torch.bfloat16,
                 causal: bool = False, device="cuda"):
        self.api, self.B, self.causal = api, B, causal
        mk = lambda h, s: torch.empty(B, h, s, D, dtype=dtype, device=device)
        self.Q, self.K, self.V, self.O = mk(H, Sq), mk(Hkv, Sk), mk(Hkv, Sk), mk(H, Sq)
        self.cp = [api.allocate_checkpoints_attention(self.Q[b:b + 1], self.K[b:b + 1], self.V[b:b + 1]) for b in range(B)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        ev = lambda: [torch.cuda.Event() for _ in range(B)]
        self.e_in, self.e_run, self.e_out = ev(), ev(), ev()
        self.first = True

    def run(self, hO, hQ, hK, hV):
        """hQ/hK/hV/hO: pinned host tensors (B, H, S, D).  Returns after enqueueing; the calling stream
        is made to wait for the last outbound copy, so an event recorded on it afterwards (or a
        synchronise) covers the whole call."""
        cur = torch.cuda.current_stream()
        if self.first:
            for s in (self.s_in, self.s_run, self.s_out):
                s.wait_stream(cur)
        for b in range(self.B):
            with torch.cuda.stream(self.s_in):
                if not self.first:
                    self.s_in.wait_event(self.e_run[b])          # the previous call's kernel has read these buffers
                self.Q[b].copy_(hQ[b], non_blocking=True)
                self.K[b].copy_(hK[b], non_blocking=True)
                self.V[b].copy_(hV[b], non_blocking=True)
                self.e_in[b].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.e_in[b])
                if not self.first:
                    self.s_run.wait_event(self.e_out[b])         # the previous call's O[b] has left the device
                self.api.attention_(self.O[b:b + 1], self.Q[b:b + 1], self.K[b:b + 1], self.V[b:b + 1],
                                    causal=self.causal, checkpoints=self.cp[b])
                self.e_run[b].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.e_run[b])
                hO[b].copy_(self.O[b], non_blocking=True)
                self.e_out[b].record(self.s_out)
        cur.wait_event(self.e_out[self.B - 1])
        self.first = False
        return hO
