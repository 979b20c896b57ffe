"""Nifulix: a decoder of `parallel` blocks whose mixer is chosen layer by layer.

    x = embed[token]
    per layer:  h = norm(x);  x = x + residual_mult * (mixer(h) + mlp(h))       (mlp may be absent)
    logits = head . norm(x)

Norms are RMS norms whose weight is stored around zero (1 + w).  The mixer of a layer is one of
`attention` (grouped heads, capped scores, a linear distance penalty per head, a sliding window that keeps
the first tokens, values blended with the first such layer's, a sigmoid gate on the output),
`retention` (linear attention with a fixed decay per head; queries and keys turned by position, pairs half a
head apart; each head's output over its root mean square, times silu of a gate) and `latent_attention`
(queries and keys/values through low-rank latents, one rotated key part shared by the heads, pairs
interleaved; a sliding window).  The feed-forward is down(silu(gate h) * (up h)).  No biases anywhere.

config.json: `architecture`, `vocab`, `width`, `residual_mult`, `norm.eps`, and `layers`, a list of
{`type`, `mixer`: the mixer's sizes and constants, `mlp`: {`kind`: "dense", `ff`} or null}.  Tensors:
`embed`, `l<i>.norm1`, `l<i>.mix.<name>`, `l<i>.mlp.{gate,up,down}`, `final.norm`, `head`; matrices are
`[out, in]`.  This module only describes: the configuration, the plan (which parts, with which sizes and
tensor names) and the random-weights recipe; all computing is in the parts.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass

from ..config.json_view import ConfigError, JsonView
from ..config.registry import Architecture, register
from ..parts.base import PartSpec
from .plan import ModelPlan

MIXER_TYPES = ("attention", "retention", "latent_attention")
#: the distance penalty of head h of H is 2^(-SLOPE_SPAN (h + 1) / H) per position
SLOPE_SPAN = 8.0


@dataclass(frozen=True)
class NifulixConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple            # of dicts {"type", "mixer", "mlp"} as config.json has them
    arch_id: str = "nifulix"


def _need(d: dict, key: str, where: str, kinds=(int, float)):
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"config: {where} has no `{key}`")
    return v


def _pos_int(d: dict, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise ConfigError(f"config: {where}: `{key}` must be positive")
    return int(v)


def read_config(view: JsonView) -> NifulixConfig:
    tree = view.tree
    vocab, width = _pos_int(tree, "vocab", "the model"), _pos_int(tree, "width", "the model")
    eps = float(_need(tree.get("norm"), "eps", "`norm`"))
    mult = float(_need(tree, "residual_mult", "the model"))
    layers = tree.get("layers")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("config: `layers` must be a non-empty list")
    blend_shape = None
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"config: {where}: `type` must be one of {MIXER_TYPES}")
        m = layer.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"config: {where} has no `mixer`")
        heads, dim, vdim = _pos_int(m, "heads", where), _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
        if layer["type"] == "attention":
            kv = _pos_int(m, "kv_heads", where)
            if heads % kv:
                raise ConfigError(f"config: {where}: {heads} heads do not divide into {kv} key/value heads")
            _need(m, "scale", where)
            if m.get("v_mix"):
                if blend_shape is not None and blend_shape != (kv, vdim):
                    raise ConfigError(f"config: {where}: layers that blend values must have values of one shape")
                blend_shape = (kv, vdim)
        elif layer["type"] == "retention":
            decay = m.get("decay")
            if not isinstance(decay, list) or len(decay) != heads:
                raise ConfigError(f"config: {where}: `decay` must list one number per head")
            rot = m.get("rot")
            if rot is not None:
                dims = _pos_int(rot, "dims", where + " rot")
                _need(rot, "base", where + " rot")
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config: {where}: {dims} rotated entries of a head of {dim}")
        else:
            rot_dim = _pos_int(m, "rot_dim", where)
            _pos_int(m, "kv_rank", where), _pos_int(m, "q_rank", where), _need(m, "scale", where)
            _need(m.get("rot"), "base", where + " rot")
            if rot_dim % 2:
                raise ConfigError(f"config: {where}: rot_dim must be even")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"config: {where}: `mlp` is null or of kind `dense`")
            _pos_int(mlp, "ff", where + " mlp")
    return NifulixConfig(vocab=vocab, width=width, norm_eps=eps, residual_mult=mult, layers=tuple(copy.deepcopy(layers)))


def write_config(c: NifulixConfig) -> dict:
    return {"architecture": "Nifulix", "vocab": c.vocab, "width": c.width, "residual_mult": c.residual_mult,
            "norm": {"eps": c.norm_eps}, "layers": copy.deepcopy(list(c.layers))}


def _mixer_spec(c: NifulixConfig, layer: dict, first_blend: bool) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    mask = m.get("mask") or {}
    if kind == "attention":
        return PartSpec("shaped_score_attention", {
            "width": c.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
            "score_scale": m["scale"], "softcap": m.get("softcap"), "slope_span": SLOPE_SPAN,
            "window": mask.get("size"), "keep_first": mask.get("keep_first", 0),
            "value_blend": (("source" if first_blend else "blend") if m.get("v_mix") else None), "gate": True})
    if kind == "retention":
        rot = m.get("rot")
        return PartSpec("retention", {
            "width": c.width, "n_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"], "decay": tuple(m["decay"]),
            "key_scale": float(m["dim"]) ** -0.5, "unit_norm_eps": c.norm_eps, "gate": True,
            "position": PartSpec("rotary", {"dims": rot["dims"], "base": rot["base"], "layout": "half"}) if rot else None})
    return PartSpec("latent_attention", {
        "width": c.width, "n_heads": m["heads"], "nope_dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"],
        "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "score_scale": m["scale"], "norm_eps": c.norm_eps,
        "window": mask.get("size"),
        "position": PartSpec("rotary", {"dims": m["rot_dim"], "base": m["rot"]["base"], "layout": "interleaved"})})


def plan(c: NifulixConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "unit_offset": True, "name": ""})
    blocks, prefixes, seen_blend, kinds = [], [], False, []
    for i, layer in enumerate(c.layers):
        is_blend = layer["type"] == "attention" and bool(layer["mixer"].get("v_mix"))
        mixer = _mixer_spec(c, layer, first_blend=is_blend and not seen_blend)
        seen_blend = seen_blend or is_blend
        mlp = layer.get("mlp")
        ff = PartSpec("gated_mlp", {"width": c.width, "hidden": mlp["ff"], "activation": "silu"}) if mlp is not None else None
        blocks.append(PartSpec("parallel", {"norm": norm, "mixer": mixer, "feed_forward": ff, "residual_mult": c.residual_mult}))
        prefixes.append(f"l{i}.")
        kinds.append(layer["type"][0])
    return ModelPlan(
        arch_id="nifulix", vocab_size=c.vocab, width=c.width,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "width": c.width, "name": "embed"}),
        blocks=tuple(blocks), block_prefixes=tuple(prefixes),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "width": c.width, "norm": norm, "tied": False, "bias": False,
                                  "norm_name": "final.norm", "name": "head", "weight_name": ""}),
        order=ModelPlan.straight_order(len(c.layers)), max_positions=None,
        summary=f"nifulix · {len(c.layers)} layers ({''.join(kinds)}) · {c.width} wide · {c.vocab} vocab",
    )


def random_tensors(c: NifulixConfig, rng) -> dict:
    """Matrices ~N(0, 1/in), the embedding ~N(0, 1), norm weights ~N(0, 0.1) around their stored zero, blend
    weights away from 0 and 1 so that a dropped blend shows."""
    def mat(out, inp, gain=1.0):
        return rng.normal((out, inp), gain / math.sqrt(inp))

    w = c.width
    t = {"embed": rng.normal((c.vocab, w), 1.0)}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer["mixer"]
        t[p + "norm1"] = rng.normal((w,), 0.1)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * dk, w, 2.0), mat(G * dk, w, 2.0), mat(G * dv, w)
            t[p + "mix.g"], t[p + "mix.o"] = mat(H * dv, w), mat(w, H * dv)
            if m.get("v_mix"):
                t[p + "mix.vmix"] = rng.normal((), 0.1, 0.35)
        elif layer["type"] == "retention":
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * dk, w), mat(H * dk, w), mat(H * dv, w)
            t[p + "mix.g"], t[p + "mix.o"] = mat(H * dv, w), mat(w, H * dv)
        else:
            rq, rk, dr = m["q_rank"], m["kv_rank"], m["rot_dim"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = mat(rq, w), rng.normal((rq,), 0.1, 1.0)
            t[p + "mix.uq"] = mat(H * (dk + dr), rq, 2.0)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(rk + dr, w), rng.normal((rk,), 0.1, 1.0)
            t[p + "mix.uk"], t[p + "mix.uv"], t[p + "mix.o"] = mat(H * dk, rk, 2.0), mat(H * dv, rk), mat(w, H * dv)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(ff, w), mat(ff, w), mat(w, ff)
    t["final.norm"] = rng.normal((w,), 0.1)
    t["head"] = mat(c.vocab, w)
    return t


ARCH = register(Architecture(
    id="nifulix", model_types=("nifulix",),
    about="Nifulix: parallel blocks; shaped-score attention, retention or latent attention, layer by layer",
    read_config=read_config, plan=plan, write_config=write_config, random_tensors=random_tensors,
), replace=True)
