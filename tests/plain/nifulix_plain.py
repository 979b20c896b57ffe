"""A plain, slow Nifulix: whole sequences, no cache, one function per mechanism.

Nifulix is a decoder whose layers are `parallel` blocks - one norm, a mixer and a gated
feed-forward that both read it, their sum scaled into the residual stream - with three kinds
of mixer chosen layer by layer: `attention` (grouped heads, capped scores, a linear distance
penalty, a sliding window that keeps the first tokens, values blended with the first such
layer's, a sigmoid gate on the output), `retention` (linear attention with a fixed decay per
head and a rotation of queries and keys) and `latent_attention` (queries and keys/values
through low-rank latents, one rotated key part shared by the heads, a sliding window).

This file shares no code with `kvad_b200`: it reads safetensors with its own few lines and
computes with NumPy in float64 on whole sequences, every mechanism in its textbook form
(full score matrices, a token-by-token recurrence).
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
        elif dt == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        elif dt == "I64":
            a = np.frombuffer(raw, dtype="<i8").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = a.reshape(info["shape"])
    return out


# ----------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_offset(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softmax_rows(s):
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(-1, keepdims=True)


def rotate(x, positions, base, dims, layout):
    """Rotates the first `dims` entries of the last axis of x [tokens, heads, size] by the
    tokens' positions.  layout "half": entry i pairs with i + dims/2; "interleaved": 2i with 2i+1."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None, None] * freq[None, None, :]
    c, s = np.cos(ang), np.sin(ang)
    y = x.copy()
    if layout == "half":
        u, v = x[..., :half], x[..., half:dims]
        y[..., :half], y[..., half:dims] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        y[..., 0:dims:2], y[..., 1:dims:2] = u * c - v * s, v * c + u * s
    return y


def visible(n, window=None, keep_first=0):
    """[n, n] bool: query i sees key j."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j < window) | (j < keep_first)
    return ok


# ----------------------------------------------------------------------------- mixers
def mix_attention(h, t, p, m, eps, shared):
    """Grouped-head softmax attention with capped scores, distance penalty, window + kept first tokens,
    value blending across layers and an output gate."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T).reshape(n, H, dk)
    k = (h @ t[p + "k"].T).reshape(n, G, dk)
    v = (h @ t[p + "v"].T).reshape(n, G, dv)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = float(t[p + "vmix"])
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    mask = m.get("mask") or {}
    ok = visible(n, mask.get("size"), mask.get("keep_first", 0))
    dist = (np.arange(n)[:, None] - np.arange(n)[None, :]).astype(np.float64)
    out = np.zeros((n, H, dv))
    cap = m.get("softcap")
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        s = s - 2.0 ** (-8.0 * (hd + 1) / H) * dist
        s = np.where(ok, s, -np.inf)
        out[:, hd] = softmax_rows(s) @ v[:, g]
    gate = sigmoid(h @ t[p + "g"].T)
    return (out.reshape(n, H * dv) * gate) @ t[p + "o"].T


def mix_retention(h, t, p, m, eps, shared):
    """Linear attention with a fixed decay per head; the state is walked token by token."""
    n = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q, k = (h @ t[p + "q"].T).reshape(n, H, dk), (h @ t[p + "k"].T).reshape(n, H, dk)
    if m.get("rot"):
        q = rotate(q, pos, m["rot"]["base"], m["rot"]["dims"], "half")
        k = rotate(k, pos, m["rot"]["base"], m["rot"]["dims"], "half")
    k = k * dk ** -0.5
    v = (h @ t[p + "v"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv))
    for hd in range(H):
        S = np.zeros((dk, dv))
        for i in range(n):
            S = m["decay"][hd] * S + np.outer(k[i, hd], v[i, hd])
            out[i, hd] = S.T @ q[i, hd]
    out = rms_unit(out, eps).reshape(n, H * dv)
    return (out * silu(h @ t[p + "g"].T)) @ t[p + "o"].T


def mix_latent_attention(h, t, p, m, eps, shared):
    """Queries and keys/values through latents; keys and values are rebuilt from the latent for every
    head, the rotated key part is one vector shared by all heads."""
    n = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n)
    cq = norm_plain(h @ t[p + "dq"].T, t[p + "dq.norm"], eps)
    q = (cq @ t[p + "uq"].T).reshape(n, H, dn + dr)
    q_n, q_r = q[..., :dn], rotate(q[..., dn:], pos, m["rot"]["base"], dr, "interleaved")
    kv = h @ t[p + "dkv"].T
    c = norm_plain(kv[:, :rk], t[p + "dkv.norm"], eps)
    k_r = rotate(kv[:, None, rk:], pos, m["rot"]["base"], dr, "interleaved")[:, 0]
    k_n = (c @ t[p + "uk"].T).reshape(n, H, dn)
    v = (c @ t[p + "uv"].T).reshape(n, H, dv)
    ok = visible(n, (m.get("mask") or {}).get("size"))
    out = np.zeros((n, H, dv))
    for hd in range(H):
        s = (q_n[:, hd] @ k_n[:, hd].T + q_r[:, hd] @ k_r.T) * m["scale"]
        out[:, hd] = softmax_rows(np.where(ok, s, -np.inf)) @ v[:, hd]
    return out.reshape(n, H * dv) @ t[p + "o"].T


MIXERS = {"attention": mix_attention, "retention": mix_retention, "latent_attention": mix_latent_attention}


def feed_forward(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


# ----------------------------------------------------------------------------- the model
class PlainNifulix:
    def __init__(self, model_dir=None, config=None, tensors=None):
        if model_dir is not None:
            with open(os.path.join(model_dir, "config.json")) as f:
                config = json.load(f)
            tensors = read_tensors(os.path.join(model_dir, "model.safetensors"))
        self.cfg, self.t = config, {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}

    def forward(self, tokens, return_layers=False):
        """Logits [tokens, vocab] of one whole sequence (and the residual stream after every layer)."""
        cfg, t = self.cfg, self.t
        eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
        x = t["embed"][np.asarray(tokens)]
        shared, layers = {}, []
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = norm_offset(x, t[p + "norm1"], eps)
            y = MIXERS[layer["type"]](h, t, p + "mix.", layer["mixer"], eps, shared)
            if layer.get("mlp") is not None:
                y = y + feed_forward(h, t, p + "mlp.")
            x = x + mult * y
            layers.append(x.copy())
        logits = norm_offset(x, t["final.norm"], eps) @ t["head"].T
        return (logits, np.stack(layers)) if return_layers else logits

    def greedy(self, prompt, n):
        ids = list(prompt)
        for _ in range(n):
            ids.append(int(np.argmax(self.forward(ids)[-1])))
        return ids[len(prompt):]
