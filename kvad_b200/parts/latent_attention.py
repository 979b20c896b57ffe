"""Latent attention as a mixer: queries and keys/values go through low-rank latents, and only the
key/value latent and one rotated key part are cached.

    c_q = norm(W_dq h);  q = W_uq c_q, head by head [nope_dim unrotated | rot_dim rotated]      (no `q_rank`: q = W_q h)
    W_dkv h = [kv_rank | rot_dim]:  c = norm(first kv_rank),  k_r = rotate(last rot_dim)   (one for all heads)
    per head: k_n = W_uk c, v = W_uv c;  s_ij = (q_n . k_n + q_r . k_r) * score_scale;  window;  softmax;  W_o

The cache holds [c | k_r] per position: one "head" of kv_rank + rot_dim entries and no values.  The
keys and values of the heads are never rebuilt: q_n . (W_uk c) = (W_uk^T q_n) . c, so each head's query is
carried into the latent's space (a head-wise map: one launch for a few rows, one product a head for many),
attention runs with ONE shared key [c | k_r] and the latent c itself as the value, and W_uv is applied to
the attended latent (head-wise again) before the output projection.  Prompts and single-token rows take the same road.

A layer may read the cache entry of another latent layer instead of keeping one (`own_kv=False`, and a run order
whose call has `writes_cache=False`): it has no W_dkv and attends over that layer's [c | k_r] as they are cached,
with its own queries, W_uk and W_uv.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.layout import KVNeed
from .base import Mixer, PartSpec, build_part, register_part
from .linear import FusedLinear, Linear
from ..weights.source import TensorRequest


class LatentAttention(Mixer):
    graph_safe = True
    kernel_families = ("scored_attention", "norm_rotary")

    def __init__(self, prefix: str, width: int, n_heads: int, nope_dim: int, rot_dim: int, value_dim: int, q_rank: Optional[int],
                 kv_rank: int, score_scale: float, norm_eps: float, position: PartSpec, window: Optional[int] = None,
                 own_kv: bool = True, q_name: str = "q",
                 dq_name: str = "dq", dq_norm_name: str = "dq.norm", uq_name: str = "uq", dkv_name: str = "dkv",
                 dkv_norm_name: str = "dkv.norm", uk_name: str = "uk", uv_name: str = "uv", out_name: str = "o"):
        super().__init__(prefix)
        self.width, self.n_heads = int(width), int(n_heads)
        self.nope_dim, self.rot_dim, self.value_dim = int(nope_dim), int(rot_dim), int(value_dim)
        self.q_rank, self.kv_rank, self.own_kv = (int(q_rank) if q_rank else 0), int(kv_rank), bool(own_kv)
        self.score_scale, self.norm_eps = float(score_scale), float(norm_eps)
        self.window = int(window) if window else None
        self.q_dim = self.nope_dim + self.rot_dim              # a head of the query as the checkpoint has it
        self.key_dim = self.kv_rank + self.rot_dim             # a cached row, and a head of the carried query
        # everything that reads h runs as one product: the query (its latent, or the heads' queries themselves) and,
        # in a layer that keeps a cache entry of its own, the key/value latent with the shared key part
        maps = [(dq_name, self.q_rank, 8) if self.q_rank else (q_name, self.n_heads * self.q_dim, 8)]
        if self.own_kv:
            maps.append((dkv_name, self.key_dim, 8))
        self.down = FusedLinear(prefix, self.width, maps, pad_to=8)
        self.up_q = Linear(prefix + uq_name, self.q_rank, self.n_heads * self.q_dim, bias=False, weight_name="") if self.q_rank else None
        self.out = Linear(prefix + out_name, self.n_heads * self.value_dim, self.width, bias=False, weight_name="")
        self.position = build_part("position", position, prefix)
        if self.position.dims != self.rot_dim:
            raise ValueError("latent attention: the rotary encoding turns exactly the rotated part")
        self.names = dict(dq_norm=dq_norm_name, dkv_norm=dkv_norm_name, uk=uk_name, uv=uv_name)
        self.q_norm = self.kv_norm = None
        self._uk = None          # [heads, kv_rank, nope_dim]: head h's W_uk_h^T, the map of its query into the latent's space
        self._uv = None          # [heads, value_dim, kv_rank]: head h's W_uv_h

    def children(self):
        return [self.down, self.out, self.position] + ([self.up_q] if self.up_q is not None else [])

    def own_requests(self):
        p, n = self.prefix, self.names
        return ([TensorRequest(p + n["dq_norm"], (self.q_rank,))] if self.q_rank else []) + \
               ([TensorRequest(p + n["dkv_norm"], (self.kv_rank,))] if self.own_kv else []) + \
               [TensorRequest(p + n["uk"], (self.n_heads * self.nope_dim, self.kv_rank)),
                TensorRequest(p + n["uv"], (self.n_heads * self.value_dim, self.kv_rank))]

    def load_own(self, fetch):
        p, n = self.prefix, self.names
        self.q_norm = fetch(p + n["dq_norm"], keep_f32=True) if self.q_rank else None
        self.kv_norm = fetch(p + n["dkv_norm"], keep_f32=True) if self.own_kv else None
        uk = fetch(p + n["uk"]).view(self.n_heads, self.nope_dim, self.kv_rank)
        self._uk = uk.transpose(1, 2).contiguous()             # [heads, kv_rank, nope_dim]: head h's map into the latent's space
        self._uv = fetch(p + n["uv"]).view(self.n_heads, self.value_dim, self.kv_rank).contiguous()

    def own_tensors(self):
        return [t for t in (self.q_norm, self.kv_norm, self._uk, self._uv) if t is not None]

    def cache_need(self):
        return KVNeed(1, self.key_dim, self.window, value_dim=0)

    def forward(self, ctx, h, residual, call):
        n, ops, b, H = h.shape[0], ctx.ops, ctx.batch, self.n_heads
        down = ctx.buffer((n, self.down.out_features))
        self.down.forward(ctx, h, down)
        view = ctx.kv(call.cache)
        if call.writes_cache != self.own_kv:
            raise ValueError("latent attention: a layer with a key/value latent of its own writes its cache entry, one without reads another's")
        if call.writes_cache:
            ops.latent_store(down[:, self.down.columns(1)], self.kv_norm, self.norm_eps, self.position.inv_freq, ctx.row_seq,
                             ctx.row_pos, view.page_table, view.k_pages, self.kv_rank, self.rot_dim,
                             interleaved=self.position.interleaved)
        if self.q_rank:
            cq = ctx.buffer((n, self.q_rank))
            ops.rmsnorm(down[:, self.down.columns(0)], self.q_norm, self.norm_eps, cq)
            q = ctx.buffer((n, H * self.q_dim))
            self.up_q.forward(ctx, cq, q)
        else:
            q = down[:, self.down.columns(0)]
        # each head's query in the latent's space: [W_uk_h^T q_n | rotate(q_r)]
        ql = ctx.buffer((n, H * self.key_dim))
        ops.linear_heads(q, self._uk, ql, head_stride_a=self.q_dim, head_stride_out=self.key_dim)
        self.position.rotate_heads(ctx, q, ql, H, self.q_dim, self.nope_dim, self.key_dim, self.kv_rank)
        attended = ctx.buffer((n, H * self.kv_rank))
        splits, scratch = 1, None
        if b.is_decode:
            splits = ops.scored_splits(n, 1, H, self.window or view.page_table.shape[1] * view.page_size)
            scratch = ctx.buffer((n * H * splits * (self.kv_rank + 2),), torch.float32) if splits > 1 else None
        ops.attention_scored(ql, attended, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table, view.k_pages,
                             None, H, self.score_scale, value_dim=self.kv_rank, window=self.window or 0,
                             heads_per_block=min(H, 32) if b.is_decode else max(d for d in (1, 2, 4) if H % d == 0),
                             n_splits=splits, scratch=scratch)
        mixed = ctx.buffer((n, H * self.value_dim))
        ops.linear_heads(attended, self._uv, mixed, head_stride_a=self.kv_rank, head_stride_out=self.value_dim)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "latent_attention", LatentAttention)
