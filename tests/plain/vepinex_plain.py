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
def mlstm(h, w, p, m, eps):
    """Matrix memory, token by token.  h [T, width]; returns [T, width]."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = logsigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = np.zeros((T, H, dv))
    for a in range(H):
        S, n, mx = np.zeros((dk, dv)), np.zeros(dk), 0.0
        for t in range(T):
            new = max(gf[t, a] + mx, gi[t, a])
            keep, take = math.exp(gf[t, a] + mx - new), math.exp(gi[t, a] - new)
            S = keep * S + take * np.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            mx = new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(n @ q[t, a]), math.exp(-mx)) + 1e-6)
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


def channel_delta(h, w, p, m, eps):
    """The delta rule with a decay per key channel, token by token."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)
    a = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, dk)
    g = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * softplus(a))
    out = np.zeros((T, H, dv))
    for a_ in range(H):
        kv = a_ // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = g[t, a_][:, None] * S
            u = beta[t, a_] * (v[t, a_] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            out[t, a_] = S.T @ q[t, kv]
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    o = rms_unit(out, eps) * w[p + "norm"][None, None, :] * gate
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen only."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    return chosen, softmax_rows(np.take_along_axis(z, chosen, -1))


def moe_ff(h, w, p, mlp):
    chosen, weight = route(h, w, p, mlp["router"]["top"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weight[t]):
            out[t] += g * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# ----------------------------------------------------------------------------- the model
def forward(config, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer, if asked)."""
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
            y = y + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp))
        x = x + y
        after.append(x.copy())
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, np.stack(after)) if return_layers else logits


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    return config, read_tensors(os.path.join(model_dir, "model.safetensors"))
