"""Vepinex: a decoder of `parallel` blocks over a normalised embedding, with a tied output head.

    x = norm(embed[token])
    per layer:  h = norm(x);  x = x + mixer(h) + mlp(h)                        (mlp may be absent)
    logits = embed . norm(x)

Norms are RMS norms with a plain weight.  The mixer of a layer is one of `mlstm` (a matrix memory with capped
exponential gates and a running maximum), `latent_attention` (keys and values through one low-rank latent, one
rotated key part shared by the heads, pairs interleaved; queries straight from h; with `kv_from`: j the layer
keeps nothing and reads layer j's cached latent) and `channel_delta` (the delta rule with a decay per key
channel, short causal convolutions on q, k and v).  The feed-forward is `dense` (down(silu(gate h) * (up h)))
or `moe` (clamped experts chosen by a router with a bias, an optional shared expert).

config.json: `architecture`, `vocab`, `width`, `norm.eps`, and `layers`, a list of {`type`, `mixer`: the mixer's
sizes and constants, `mlp`: {`kind`: "dense", `ff`} or {`kind`: "moe", `router`: {`experts`, `top`}, `expert`:
{`ff`, `limit`}, `shared`: {`ff`, `limit`} or absent} or null}.  Tensors: `embed`, `embed.norm`, `l<i>.norm1`,
`l<i>.mix.<name>`, `l<i>.mlp.<name>`, `final.norm`; matrices are `[out, in]`.  The ranks of the delta rule's two
low-rank maps are not in config.json; they are read from the shapes of `a1` and `g1` when a model folder is
loaded and stand in the typed configuration as `mixer.decay_rank` / `mixer.gate_rank`.  This module only
describes: the configuration, the plan (which parts, with which sizes and tensor names) and the random-weights
recipe; all computing is in the parts.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass

from ..config.json_view import ConfigError, JsonView
from ..config.registry import Architecture, register
from ..parts.base import PartSpec
from .plan import LayerCall, ModelPlan

MIXER_TYPES = ("mlstm", "latent_attention", "channel_delta")
#: constants the design fixes
EXPERT_ALPHA = 1.702        # the experts' gate is g * sigmoid(EXPERT_ALPHA * g)
UNIT_EPS = 1e-6             # under the root that makes the delta rule's q and k unit vectors
DEFAULT_RANK = 24           # random-weights mode: rank of the delta rule's low-rank maps where a configuration names none


@dataclass(frozen=True)
class VepinexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple            # of dicts {"type", "mixer", "mlp"} as config.json has them
    arch_id: str = "vepinex"


def _need(d, key: str, where: str, kinds=(int, float)):
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"config: {where} has no `{key}`")
    return v


def _pos_int(d, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise ConfigError(f"config: {where}: `{key}` must be positive")
    return int(v)


def _check_glu(d, where: str) -> None:
    _pos_int(d, "ff", where)
    if float(_need(d, "limit", where)) <= 0:
        raise ConfigError(f"config: {where}: `limit` must be positive")


def read_config(view: JsonView) -> VepinexConfig:
    tree = view.tree
    vocab, width = _pos_int(tree, "vocab", "the model"), _pos_int(tree, "width", "the model")
    eps = float(_need(tree.get("norm"), "eps", "`norm`"))
    layers = tree.get("layers")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("config: `layers` must be a non-empty list")
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"config: {where}: `type` must be one of {MIXER_TYPES}")
        m = layer.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"config: {where} has no `mixer`")
        heads = _pos_int(m, "heads", where)
        _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
        if layer["type"] == "mlstm":
            if float(_need(m, "gate_cap", where)) <= 0:
                raise ConfigError(f"config: {where}: `gate_cap` must be positive")
        elif layer["type"] == "channel_delta":
            kv = _pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads      # (absent: a query/key head per head)
            if heads % kv:
                raise ConfigError(f"config: {where}: {heads} heads do not divide into {kv} query/key heads")
            _pos_int(m, "conv", where)
        else:
            rot_dim = _pos_int(m, "rot_dim", where)
            _pos_int(m, "kv_rank", where), _need(m, "scale", where)
            rot = m.get("rot")
            _need(rot, "base", where + " rot")
            if rot_dim % 2 or _pos_int(rot, "dims", where + " rot") != rot_dim:
                raise ConfigError(f"config: {where}: the rotation turns the whole rotated part, an even number of entries")
            src = m.get("kv_from")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
                    raise ConfigError(f"config: {where}: `kv_from` must name an earlier layer")
                o = layers[src]
                if o.get("type") != "latent_attention" or o["mixer"].get("kv_from") is not None:
                    raise ConfigError(f"config: {where}: `kv_from` must name a latent-attention layer with a latent of its own")
                if any(o["mixer"].get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                    raise ConfigError(f"config: {where}: the layer it reads from must have its latent size and rotation")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config: {where}: `mlp` is null or of kind `dense` or `moe`")
            if mlp["kind"] == "dense":
                _pos_int(mlp, "ff", where + " mlp")
            else:
                r = mlp.get("router")
                if _pos_int(r, "top", where + " router") > _pos_int(r, "experts", where + " router"):
                    raise ConfigError(f"config: {where}: more experts a token than experts")
                _check_glu(mlp.get("expert"), where + " expert")
                if mlp.get("shared") is not None:
                    _check_glu(mlp["shared"], where + " shared expert")
    return VepinexConfig(vocab=vocab, width=width, norm_eps=eps, layers=tuple(copy.deepcopy(layers)))


def with_checkpoint_shapes(c: VepinexConfig, shape_of) -> VepinexConfig:
    """Sizes that only the tensors' shapes give: the ranks of the delta rule's low-rank maps."""
    layers = copy.deepcopy(list(c.layers))
    for i, layer in enumerate(layers):
        if layer["type"] == "channel_delta":
            for key, name in (("decay_rank", "a1"), ("gate_rank", "g1")):
                shape = shape_of(f"l{i}.mix.{name}")
                if shape is not None and len(shape) == 2:
                    layer["mixer"][key] = int(shape[0])
    return VepinexConfig(vocab=c.vocab, width=c.width, norm_eps=c.norm_eps, layers=tuple(layers))


def write_config(c: VepinexConfig) -> dict:
    layers = copy.deepcopy(list(c.layers))
    for layer in layers:                      # (the ranks live in the tensors' shapes, not in config.json)
        layer["mixer"].pop("decay_rank", None), layer["mixer"].pop("gate_rank", None)
    return {"architecture": "Vepinex", "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps}, "layers": layers}


def _mixer_spec(c: VepinexConfig, layer: dict) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "mlstm":
        return PartSpec("matrix_memory", {"width": c.width, "n_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                                          "gate_cap": m["gate_cap"], "norm_eps": c.norm_eps})
    if kind == "channel_delta":
        return PartSpec("gated_delta_rule", {
            "width": c.width, "n_heads": m["heads"], "n_kv_heads": m.get("kv_heads") or m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
            "conv_taps": m["conv"], "decay_rank": m.get("decay_rank", DEFAULT_RANK), "gate_rank": m.get("gate_rank", DEFAULT_RANK),
            "norm_eps": c.norm_eps, "unit_eps": UNIT_EPS})
    return PartSpec("latent_attention", {
        "width": c.width, "n_heads": m["heads"], "nope_dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"], "q_rank": None,
        "kv_rank": m["kv_rank"], "score_scale": m["scale"], "norm_eps": c.norm_eps, "own_kv": m.get("kv_from") is None,
        "position": PartSpec("rotary", {"dims": m["rot"]["dims"], "base": m["rot"]["base"], "layout": "interleaved"})})


def _mlp_spec(c: VepinexConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"width": c.width, "hidden": mlp["ff"], "activation": "silu"})
    shared = mlp.get("shared")
    return PartSpec("routed_mlp", {
        "width": c.width, "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "hidden": mlp["expert"]["ff"],
        "limit": mlp["expert"]["limit"], "alpha": EXPERT_ALPHA,
        "shared": {"hidden": shared["ff"], "limit": shared["limit"], "alpha": EXPERT_ALPHA} if shared else None})


def plan(c: VepinexConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "unit_offset": False, "name": ""})
    blocks, prefixes, order, kinds = [], [], [], []
    for i, layer in enumerate(c.layers):
        blocks.append(PartSpec("parallel", {"norm": norm, "mixer": _mixer_spec(c, layer), "feed_forward": _mlp_spec(c, layer.get("mlp")),
                                            "residual_mult": 1.0}))
        prefixes.append(f"l{i}.")
        src = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
        order.append(LayerCall(i, i) if src is None else LayerCall(i, int(src), writes_cache=False))
        kinds.append({"mlstm": "m", "latent_attention": "l", "channel_delta": "d"}[layer["type"]])
    return ModelPlan(
        arch_id="vepinex", vocab_size=c.vocab, width=c.width,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "width": c.width, "name": "embed", "norm": norm,
                                               "norm_name": "embed.norm"}),
        blocks=tuple(blocks), block_prefixes=tuple(prefixes),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "width": c.width, "norm": norm, "tied": True, "bias": False,
                                  "norm_name": "final.norm", "name": "head", "weight_name": ""}),
        order=tuple(order), max_positions=None,
        summary=f"vepinex · {len(c.layers)} layers ({''.join(kinds)}) · {c.width} wide · {c.vocab} vocab",
    )


def random_tensors(c: VepinexConfig, rng) -> dict:
    """Matrices ~N(0, 1/in), the embedding ~N(0, 1), norm weights near 1, gate biases and decays spread so that every
    branch of the gates is met, router biases small so that the router's matrix decides."""
    def mat(out, inp, gain=1.0):
        return rng.normal((out, inp), gain / math.sqrt(inp))

    def glu(t, p, ff, w):
        t[p + "gate"], t[p + "up"], t[p + "down"] = mat(ff, w, 2.0), mat(ff, w, 2.0), mat(w, ff)

    w = c.width
    t = {"embed": rng.normal((c.vocab, w), 1.0), "embed.norm": rng.normal((w,), 0.1, 1.0), "final.norm": rng.normal((w,), 0.1, 1.0)}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer["mixer"]
        t[p + "norm1"] = rng.normal((w,), 0.1, 1.0)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "mlstm":
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * dk, w), mat(H * dk, w), mat(H * dv, w)
            t[p + "mix.g"], t[p + "mix.o"], t[p + "mix.norm"] = mat(H * dv, w), mat(w, H * dv), rng.normal((H * dv,), 0.1, 1.0)
            t[p + "mix.i"], t[p + "mix.i.b"] = mat(H, w, 2.0), rng.normal((H,), 1.0)
            t[p + "mix.f"], t[p + "mix.f.b"] = mat(H, w, 2.0), rng.normal((H,), 1.0, 3.0)
        elif layer["type"] == "channel_delta":
            G, taps = m.get("kv_heads") or H, m["conv"]
            ra, rg = m.get("decay_rank", DEFAULT_RANK), m.get("gate_rank", DEFAULT_RANK)
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(G * dk, w, 2.0), mat(G * dk, w, 2.0), mat(H * dv, w, 2.0)
            for name, ch in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                t[p + f"mix.{name}.conv"] = rng.normal((ch, taps), 0.5)
            t[p + "mix.b"], t[p + "mix.A_log"] = mat(H, w, 2.0), rng.normal((H,), 0.5, -1.0)
            t[p + "mix.a1"], t[p + "mix.a2"], t[p + "mix.dt_bias"] = mat(ra, w), mat(H * dk, ra, 2.0), rng.normal((H * dk,), 1.0, -1.0)
            t[p + "mix.g1"], t[p + "mix.g2"] = mat(rg, w), mat(H * dv, rg, 2.0)
            t[p + "mix.norm"], t[p + "mix.o"] = rng.normal((dv,), 0.1, 1.0), mat(w, H * dv)
        else:
            rk, dr = m["kv_rank"], m["rot_dim"]
            t[p + "mix.q"] = mat(H * (dk + dr), w, 2.0)
            if m.get("kv_from") is None:
                t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(rk + dr, w), rng.normal((rk,), 0.1, 1.0)
            t[p + "mix.uk"], t[p + "mix.uv"], t[p + "mix.o"] = mat(H * dk, rk, 2.0), mat(H * dv, rk), mat(w, H * dv)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(mlp["ff"], w), mat(mlp["ff"], w), mat(w, mlp["ff"])
            continue
        E = mlp["router"]["experts"]
        for e in range(E):
            glu(t, p + f"mlp.e{e}.", mlp["expert"]["ff"], w)
        t[p + "mlp.router"], t[p + "mlp.router.b"] = mat(E, w, 4.0), rng.normal((E,), 0.1)
        if mlp.get("shared"):
            glu(t, p + "mlp.shared.", mlp["shared"]["ff"], w)
    return t


ARCH = register(Architecture(
    id="vepinex", model_types=("vepinex",),
    about="Vepinex: parallel blocks; matrix memory, latent attention or delta rule, layer by layer; dense or routed feed-forward",
    read_config=read_config, plan=plan, write_config=write_config, random_tensors=random_tensors,
    with_checkpoint_shapes=with_checkpoint_shapes,
), replace=True)
