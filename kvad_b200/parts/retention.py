"""Retention as a mixer: linear attention with a fixed decay per head, no softmax and no denominator.

    q = W_q h, k = W_k h (heads x key_dim), v = W_v h (heads x value_dim), turned by position (`position`,
    a rotary encoding over the heads' first entries), k scaled by `key_scale` afterwards;
    S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t           per sequence and head;
    each head's o over its root mean square (`unit_norm`), the heads side by side times silu(W_g h) (`gate`),
    then the output projection.

What a sequence keeps is one 32-bit state `[heads, key_dim, value_dim]` in its cache slot, zero at the
start and carried from row to row and from step to step.  The four projections run as one product; the
turning, the recurrence, the norm and the gate are one kernel (`csrc/retention.cu`), everything in it 32-bit.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..cache.layout import StateNeed
from .base import Mixer, PartSpec, build_part, register_part
from .linear import FusedLinear, Linear


class Retention(Mixer):
    graph_safe = True
    kernel_families = ("retention", "norm_rotary")

    def __init__(self, prefix: str, width: int, n_heads: int, key_dim: int, decay: Sequence[float],
                 value_dim: Optional[int] = None, key_scale: Optional[float] = None, position: Optional[PartSpec] = None,
                 unit_norm_eps: Optional[float] = None, gate: bool = True, q_name: str = "q", k_name: str = "k",
                 v_name: str = "v", gate_name: str = "g", out_name: str = "o"):
        super().__init__(prefix)
        self.width, self.n_heads, self.key_dim = int(width), int(n_heads), int(key_dim)
        self.value_dim = int(value_dim) if value_dim else self.key_dim
        if len(decay) != self.n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.n_heads} heads")
        self.decay_values = [float(d) for d in decay]
        self.key_scale = float(key_scale) if key_scale is not None else 1.0
        self.unit_norm_eps = None if unit_norm_eps is None else float(unit_norm_eps)
        self.gated = bool(gate)
        self.qk_width, self.v_width = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        maps = [(q_name, self.qk_width), (k_name, self.qk_width), (v_name, self.v_width)]
        if self.gated:
            maps.append((gate_name, self.v_width))
        self.proj = FusedLinear(prefix, self.width, maps)
        self.out = Linear(prefix + out_name, self.v_width, self.width, bias=False, weight_name="")
        self.position = build_part("position", position, prefix) if position is not None else None
        if self.position is not None and getattr(self.position, "dims", 0) > self.key_dim:
            raise ValueError("retention: more rotated entries than a head has")
        self.decay = None

    def children(self):
        return [self.proj, self.out] + ([self.position] if self.position is not None else [])

    def load_own(self, fetch):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=getattr(fetch, "device", "cuda"))

    def cache_need(self):
        return StateNeed((self.n_heads, self.key_dim, self.value_dim), torch.float32)

    def forward(self, ctx, h, residual, call):
        n = h.shape[0]
        buf = ctx.buffer((n, self.proj.out_features))
        self.proj.forward(ctx, h, buf)
        q, k, v = (buf[:, self.proj.columns(i)] for i in range(3))
        gate = buf[:, self.proj.columns(3)] if self.gated else None
        mixed = ctx.buffer((n, self.v_width))
        pos = self.position
        raw = ctx.buffer((n, self.v_width), torch.float32) if ctx.ops.retention_needs_raw(self.key_dim, self.value_dim) else None
        ctx.ops.retention(q, k, v, mixed, ctx.state(call.cache), ctx.seq_starts, ctx.kv_lens, ctx.seq_slots, ctx.n_seqs,
                          self.decay, self.n_heads, inv_freq=pos.inv_freq if pos is not None else None,
                          rot_dims=pos.dims if pos is not None else 0, interleaved=pos.interleaved if pos is not None else False,
                          k_scale=self.key_scale, gate=gate, unit_norm_eps=self.unit_norm_eps, raw=raw)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "retention", Retention)
