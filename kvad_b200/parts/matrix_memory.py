"""A matrix memory with exponential gates as a mixer (the mLSTM cell of xLSTM).

    q = W_q h * dk^(-1/2), k = W_k h (heads x key_dim), v = W_v h (heads x value_dim)
    i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))          per head
    m_t = max(f + m_(t-1), i);  S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;  n_t likewise with k alone
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    each head's o over its root mean square, the heads side by side times a weight, times sigmoid(W_g h), then W_o

m starts at 0 like S and n.  A sequence keeps S, n and m in 32-bit in its cache slot.  q, k, v and the output gate
run as one product, the two gate projections with their biases as a second one that leaves 32-bit sums; the
caps, the running maximum, the recurrence and the read-out are one kernel, the per-head norm with weight and gate
another (`csrc/gated_recurrence.cu`); everything after the projections is 32-bit.
"""
from __future__ import annotations

import torch

from ..cache.layout import StateNeed
from ..weights.source import TensorRequest
from .base import Mixer, register_part
from .linear import FusedLinear, Linear


class MatrixMemory(Mixer):
    graph_safe = True
    kernel_families = ("gated_recurrence",)

    def __init__(self, prefix: str, width: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 q_name: str = "q", k_name: str = "k", v_name: str = "v", gate_name: str = "g", out_name: str = "o",
                 input_gate_name: str = "i", forget_gate_name: str = "f", bias_suffix: str = ".b", norm_name: str = "norm"):
        super().__init__(prefix)
        self.width, self.n_heads, self.key_dim, self.value_dim = int(width), int(n_heads), int(key_dim), int(value_dim)
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        if self.gate_cap <= 0:
            raise ValueError("matrix memory: the gate cap must be positive")
        self.qk_width, self.v_width = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        self.proj = FusedLinear(prefix, self.width, [(q_name, self.qk_width, 8), (k_name, self.qk_width, 8), (v_name, self.v_width, 8),
                                                     (gate_name, self.v_width, 8)], pad_to=8)
        self.gates = FusedLinear(prefix, self.width, [(input_gate_name, self.n_heads), (forget_gate_name, self.n_heads)], pad_to=16,
                                 bias_suffix=bias_suffix)
        self.out = Linear(prefix + out_name, self.v_width, self.width, bias=False, weight_name="")
        self.norm_name = norm_name
        self.norm_weight = None
        self._state_size = None

    def children(self):
        return [self.proj, self.gates, self.out]

    def own_requests(self):
        return [TensorRequest(self.prefix + self.norm_name, (self.v_width,))]

    def load_own(self, fetch):
        self.norm_weight = fetch(self.prefix + self.norm_name, keep_f32=True)

    def own_tensors(self):
        return [self.norm_weight] if self.norm_weight is not None else []

    def cache_need(self):
        tiles = -(-self.value_dim // 16)          # (the kernel keeps n and m once per block of 16 value columns)
        return StateNeed((self.n_heads * (self.value_dim * self.key_dim + tiles * (self.key_dim + 1)),), torch.float32)

    def forward(self, ctx, h, residual, call):
        n, ops, H = h.shape[0], ctx.ops, self.n_heads
        buf = ctx.buffer((n, self.proj.out_features))
        self.proj.forward(ctx, h, buf)
        gates = ctx.buffer((n, self.gates.out_features), torch.float32)
        self.gates.forward(ctx, h, gates, "store_f32")
        q, k, v, g = (buf[:, self.proj.columns(i)] for i in range(4))
        raw = ctx.buffer((n, self.v_width), torch.float32)
        ops.gated_recurrence("matrix_memory", q, k, v, gates[:, :2 * H], raw, ctx.state(call.cache), ctx.seq_starts, ctx.seq_slots,
                             ctx.n_seqs, H, H, self.key_dim, self.value_dim, q_scale=self.key_dim ** -0.5, cap=self.gate_cap)
        mixed = ctx.buffer((n, self.v_width))
        ops.head_norm_gate(raw, g, self.norm_weight, mixed, H, self.norm_eps, weight_per_head=True)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "matrix_memory", MatrixMemory)
