"""A plain, slow Vepinex: whole sequences, no cache, one function per mechanism.

Vepinex is a decoder of `parallel` blocks - one RMS norm, a mixer and a feed-forward that both read it,
their sum added to the residual stream - over a normalised embedding, with a tied output head.  The mixer
of a layer is one of `mlstm` (a matrix memory with exponential gates and a running maximum),
`latent_attention` (keys and values through one low-rank latent, one rotated key part shared by the heads;
a layer may read another layer's latent) and `channel_delta` (the delta rule with a decay per key channel,
short causal convolutions on q, k and v).  The feed-forward is dense (gated, silu) or a mixture of
clamped experts with a shared expert.

This file shares no code with `kvad_b200`: it reads safetensors with its own few lines and computes with
NumPy in float64, token by token where the design has a recurrence and with full score matrices where it
has attention.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_tensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, dt = blob[lo:hi], info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif dt in ("I32", "I64"):
            a = np.frombuffer(raw, dtype="<i4" if dt == "I32" else "<i8").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = a.reshape(info["shape"])
    return out


# ----------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def logsigmoid(z):
    return -np.logaddexp(0.0, -z)


def softmax_rows(s):
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def rotate_pairs(x, positions, base, dims):
    """Turns neighbouring pairs (2i, 2i+1) of the first `dims` entries of x [tokens, heads, size]."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers
def gate_caps(a, b, cap):
    """Log input gate and log forget gate from the two gate projections."""
    return cap * np.tanh(a / cap), logsigmoid(cap * np.tanh(b / cap))


def matrix_memory_cell(q, k, v, gi, gf, state=None):
    """One head, token by token: q, k [T, dk], v [T, dv], log gates gi, gf [T].  Returns (read-outs [T, dv], state);
    the state is (S [dk, dv], n [dk], m) and starts at zero, the running maximum too."""
    S, n, mx = state if state is not None else (np.zeros((q.shape[1], v.shape[1])), np.zeros(q.shape[1]), 0.0)
    out = np.zeros(v.shape)
    for t in range(q.shape[0]):
        new = max(gf[t] + mx, gi[t])
        keep, take = math.exp(gf[t] + mx - new), math.exp(gi[t] - new)
        S = keep * S + take * np.outer(k[t], v[t])
        n = keep * n + take * k[t]
        mx = new
        out[t] = (S.T @ q[t]) / (max(abs(n @ q[t]), math.exp(-mx)) + 1e-6)
    return out, (S, n, mx)


def mlstm(h, w, p, m, eps):
    """Matrix memory.  h [T, width]; returns [T, width]."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi, gf = gate_caps(h @ w[p + "i"].T + w[p + "i.b"], h @ w[p + "f"].T + w[p + "f.b"], cap)
    out = np.stack([matrix_memory_cell(q[:, a], k[:, a], v[:, a], gi[:, a], gf[:, a])[0] for a in range(H)], axis=1)
    o = rms_unit(out, eps).reshape(T, H * dv) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def latent_kv(h, w, p, m, eps, positions):
    """What a latent layer keeps per position: the normalised latent and the rotated shared key part."""
    r, dr = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = rms_unit(d[:, :r], eps) * w[p + "dkv.norm"]
    kr = rotate_pairs(d[:, None, r:], positions, m["rot"]["base"], m["rot"]["dims"])[:, 0]
    return c, kr


def latent_attention(h, w, p, m, kept, positions):
    """Softmax attention with keys and values rebuilt from the kept latent `kept` = (c, k_r) head by head."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kept
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    qn, qr = q[..., :dn], rotate_pairs(q[..., dn:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    mask = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, dv))
    for a in range(H):
        s = (qn[:, a] @ kn[:, a].T + qr[:, a] @ kr.T) * m["scale"]
        out[:, a] = softmax_rows(np.where(mask, s, -np.inf)) @ v[:, a]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def short_conv(x, taps):
    """Causal convolution over time per channel: x [T, C], taps [C, n], the last column meets the current row."""
    T, n = x.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, x.shape[1])), x], axis=0)
    return sum(padded[j:j + T] * taps[:, j][None, :] for j in range(n))


def unit_vectors(x, eps=1e-6):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + eps)


def channel_decay(a, a_log, dt_bias):
    """a [T, H, dk] raw, A_log [H], dt_bias [H, dk] -> the decay of every key channel."""
    return np.exp(-np.exp(a_log)[None, :, None] * softplus(a + dt_bias[None]))


def delta_cell(q, k, v, beta, g, S=None):
    """One head, token by token: q, k, g [T, dk], v [T, dv], beta [T].  Returns (read-outs [T, dv], S [dk, dv])."""
    S = np.zeros((q.shape[1], v.shape[1])) if S is None else S
    out = np.zeros(v.shape)
    for t in range(q.shape[0]):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out, S


def channel_delta(h, w, p, m, eps):
    """The delta rule with a decay per key channel."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q, k = unit_vectors(q) * dk ** -0.5, unit_vectors(k)
    beta = sigmoid(h @ w[p + "b"].T)
    g = channel_decay(((h @ w[p + "a1"].T) @ w[p + "a2"].T).reshape(T, H, dk), w[p + "A_log"], w[p + "dt_bias"].reshape(H, dk))
    out = np.stack([delta_cell(q[:, a // (H // G)], k[:, a // (H // G)], v[:, a], beta[:, a], g[:, a])[0] for a in range(H)], axis=1)
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    o = rms_unit(out, eps) * w[p + "norm"][None, None, :] * gate
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_glu(gate, up, limit):
    g, u = np.minimum(gate, limit), np.clip(up, -limit, limit)
    return g * sigmoid(1.702 * g) * (u + 1.0)


def clamped_expert(h, w, p, limit):
    return clamped_glu(h @ w[p + "gate"].T, h @ w[p + "up"].T, limit) @ w[p + "down"].T


def choose(z, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits (ties: the lower index), softmax over the chosen only."""
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    return chosen, softmax_rows(np.take_along_axis(z, chosen, -1))


def route(h, w, p, top):
    return choose(h @ w[p + "router"].T + w[p + "router.b"], top)


def routing_margin(h, w, p, top):
    """Per row, how far the last chosen logit is above the first one left out (infinite where all are chosen)."""
    z = np.sort(h @ w[p + "router"].T + w[p + "router.b"], axis=-1)[:, ::-1]
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else np.full(h.shape[0], np.inf)


def moe_ff(h, w, p, mlp, margins=None, forced=None, own=None):
    """`forced` [T, top]: these experts instead of the router's own choice (their weights still from its logits);
    `own`: a list that receives the router's own choice."""
    chosen, weight = route(h, w, p, mlp["router"]["top"])
    if own is not None:
        own.append(chosen)
    if forced is not None:
        chosen = np.asarray(forced)
        weight = softmax_rows(np.take_along_axis(h @ w[p + "router"].T + w[p + "router.b"], chosen, -1))
    if margins is not None:
        margins.append(routing_margin(h, w, p, mlp["router"]["top"]))
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weight[t]):
            out[t] += g * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# ----------------------------------------------------------------------------- the model
def forward(config, w, tokens, return_layers=False, margins=None, forced=None, own=None):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer, if asked).  `margins`: a list that
    receives, per routed layer, every row's routing margin.  `forced`: per routed layer, the experts [T, top] to use;
    `own`: a list that receives, per routed layer, what its router chose by itself given the layers before it."""
    forced = list(forced) if forced is not None else None
    eps = config["norm"]["eps"]
    positions = np.arange(len(tokens))
    x = rms_unit(w["embed"][np.asarray(tokens)], eps) * w["embed.norm"]
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms_unit(x, eps) * w[p + "norm1"]
        if layer["type"] == "mlstm":
            y = mlstm(h, w, p + "mix.", m, eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, w, p + "mix.", m, eps, positions)
                src = i
            y = latent_attention(h, w, p + "mix.", m, kept[src], positions)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, margins, forced.pop(0) if forced else None, own))
        x = x + y
        after.append(x.copy())
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, np.stack(after)) if return_layers else logits


def greedy(config, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(config, w, toks)[-1].argmax()))
    return toks[len(prompt):]


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    return config, read_tensors(os.path.join(model_dir, "model.safetensors"))
