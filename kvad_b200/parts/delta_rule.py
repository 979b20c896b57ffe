"""The gated delta rule with a decay per key channel as a mixer.

    q = W_q h, k = W_k h (kv_heads x key_dim), v = W_v h (heads x value_dim); head a reads the q/k head a // (heads / kv_heads)
    each of q, k, v: a short causal convolution over time per channel (`conv_taps`, zeros before the start), then silu
    q, k: unit vectors per head, x / sqrt(sum(x^2) + unit_eps); q also times key_dim^(-1/2)
    beta = sigmoid(W_b h) per head;  g = exp(-exp(A_log_a) softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel
    per head: S <- g * S (rows of S are key channels); u = beta (v - S^T k); S <- S + k u^T; o = S^T q
    each head's o over its root mean square, times a weight as long as one head, times sigmoid(W_g2 (W_g1 h)), then W_o

A sequence keeps in its cache slot, in 32-bit: S per head, and the last `conv_taps` - 1 inputs of the
convolutions.  All projections of h run as one product; the convolutions, silu, unit vectors and beta are one
kernel, the recurrence another, the per-head norm with weight and gate a third (`csrc/gated_recurrence.cu`);
everything after the convolutions is 32-bit.
"""
from __future__ import annotations

import torch

from ..cache.layout import StateNeed
from ..weights.source import TensorRequest
from .base import Mixer, register_part
from .linear import FusedLinear, Linear


class GatedDeltaRule(Mixer):
    graph_safe = True
    kernel_families = ("gated_recurrence",)

    def __init__(self, prefix: str, width: int, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, conv_taps: int,
                 decay_rank: int, gate_rank: int, norm_eps: float, unit_eps: float = 1e-6, q_name: str = "q", k_name: str = "k",
                 v_name: str = "v", beta_name: str = "b", decay_down_name: str = "a1", decay_up_name: str = "a2",
                 gate_down_name: str = "g1", gate_up_name: str = "g2", out_name: str = "o", conv_suffix: str = ".conv",
                 a_log_name: str = "A_log", dt_bias_name: str = "dt_bias", norm_name: str = "norm"):
        super().__init__(prefix)
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"delta rule: {n_heads} heads do not divide into {n_kv_heads} query/key heads")
        self.key_dim, self.value_dim, self.conv_taps = int(key_dim), int(value_dim), int(conv_taps)
        if not (1 <= self.conv_taps <= 16):
            raise ValueError("delta rule: 1 to 16 taps")
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.qk_width, self.v_width = self.n_kv_heads * self.key_dim, self.n_heads * self.value_dim
        self.channels = 2 * self.qk_width + self.v_width
        # q | k | v | beta side by side (what the convolution kernel walks), the two low-rank inputs on 16-byte boundaries
        self.proj = FusedLinear(prefix, self.width, [(q_name, self.qk_width), (k_name, self.qk_width), (v_name, self.v_width),
                                                     (beta_name, self.n_heads), (decay_down_name, int(decay_rank), 8),
                                                     (gate_down_name, int(gate_rank), 8)], pad_to=8)
        self.decay_up = Linear(prefix + decay_up_name, int(decay_rank), self.n_heads * self.key_dim, bias=False, weight_name="")
        self.gate_up = Linear(prefix + gate_up_name, int(gate_rank), self.v_width, bias=False, weight_name="")
        self.out = Linear(prefix + out_name, self.v_width, self.width, bias=False, weight_name="")
        self.names = dict(conv=[n + conv_suffix for n in (q_name, k_name, v_name)], a_log=a_log_name, dt_bias=dt_bias_name, norm=norm_name)
        self.taps = self.a_log = self.dt_bias = self.norm_weight = None
        self.state_floats = self.v_width * self.key_dim

    def children(self):
        return [self.proj, self.decay_up, self.gate_up, self.out]

    def own_requests(self):
        p, n = self.prefix, self.names
        sizes = (self.qk_width, self.qk_width, self.v_width)
        return [TensorRequest(p + c, (s, self.conv_taps)) for c, s in zip(n["conv"], sizes)] + [
            TensorRequest(p + n["a_log"], (self.n_heads,)), TensorRequest(p + n["dt_bias"], (self.n_heads * self.key_dim,)),
            TensorRequest(p + n["norm"], (self.value_dim,))]

    def load_own(self, fetch):
        p, n = self.prefix, self.names
        self.taps = torch.cat([fetch(p + c) for c in n["conv"]], dim=0).contiguous()
        self.a_log = fetch(p + n["a_log"], keep_f32=True).float()
        self.dt_bias = fetch(p + n["dt_bias"], keep_f32=True).float()
        self.norm_weight = fetch(p + n["norm"], keep_f32=True)

    def own_tensors(self):
        return [t for t in (self.taps, self.a_log, self.dt_bias, self.norm_weight) if t is not None]

    def cache_need(self):
        return StateNeed((self.state_floats + (self.conv_taps - 1) * self.channels,), torch.float32)

    def forward(self, ctx, h, residual, call):
        n, ops, H, G, dk = h.shape[0], ctx.ops, self.n_heads, self.n_kv_heads, self.key_dim
        C, state = self.channels, ctx.state(call.cache)
        buf = ctx.buffer((n, self.proj.out_features))
        self.proj.forward(ctx, h, buf)
        y = ctx.buffer((n, (C + H + 3) // 4 * 4), torch.float32)
        ops.short_conv(buf, self.taps, y, state, self.state_floats, ctx.row_seq, ctx.row_pos, ctx.seq_starts, ctx.seq_slots,
                       n_sigmoid=H, unit_heads=2 * G, unit_dim=dk, scaled_heads=G, head_scale=dk ** -0.5, unit_eps=self.unit_eps)
        ops.conv_state(buf, C, self.conv_taps, state, self.state_floats, ctx.seq_starts, ctx.seq_slots, ctx.n_seqs)
        decay = ctx.buffer((n, H * dk), torch.float32)
        self.decay_up.forward(ctx, buf[:, self.proj.columns(4)], decay, "store_f32")
        gate = ctx.buffer((n, self.v_width))
        self.gate_up.forward(ctx, buf[:, self.proj.columns(5)], gate)
        raw = ctx.buffer((n, self.v_width), torch.float32)
        # prompts: the decays once per row in a pass of their own (every block of a head's columns would work them out again);
        # single-token rows: inside the recurrence, one launch fewer
        ready = not ctx.batch.is_decode
        if ready:
            ops.decay_gate(decay, self.a_log, self.dt_bias, H, dk)
        ops.gated_recurrence("delta_rule", y[:, :G * dk], y[:, G * dk:2 * G * dk], y[:, 2 * G * dk:C], decay, raw, state, ctx.seq_starts,
                             ctx.seq_slots, ctx.n_seqs, H, G, dk, self.value_dim, beta=y[:, C:C + H], a_log=self.a_log, dt_bias=self.dt_bias,
                             gates_ready=ready)
        mixed = ctx.buffer((n, self.v_width))
        ops.head_norm_gate(raw, gate, self.norm_weight, mixed, H, self.norm_eps, weight_per_head=False)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
