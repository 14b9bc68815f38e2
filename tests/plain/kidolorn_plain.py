"""Plain, slow, whole-sequence statement of the Kidolorn design, one function per mechanism.

A decoder-only model whose layers wrap each sublayer in two norms, x <- x + post(mixer(conv(pre(x)))) and then the same
around the feed-forward; every norm has ONE number as its gain.  What a sublayer reads first passes a short causal
convolution per channel that is added to its own input.  A layer's mixer is a linear attention with one fixed decay per
head (``lightning``), an element-wise gated recurrence (``mingru``), or softmax attention over a small latent per token
with one rotated key part shared by the heads and a sink in the denominator (``latent_attention``; such a layer may read
another layer's latents).  The feed-forward is a clamped gated unit, dense with biases or a mixture of experts behind a
softmax-over-the-chosen router.

Everything is numpy in one floating type (float64 by default), no cache, no batching, token by token where a recurrence
is stated token by token.  Shares no code with the package.
"""

from __future__ import annotations

import json
import math
import struct

import numpy as np


# ---- model folder ---------------------------------------------------------------------------

def read_safetensors(path: str, dtype=np.float64) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(dtype)
        elif meta["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(dtype)
        elif meta["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = arr.reshape(meta["shape"]).copy()
    return out


def load_model(model_dir: str, dtype=np.float64):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{model_dir}/model.safetensors", dtype)


# ---- small pieces ---------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_scalar(x, g, eps):
    """A norm whose gain is one number for all channels."""
    return unit_rms(x, eps) * float(np.asarray(g).reshape(()))


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def input_convolution(h, taps_w):
    """h [T, C] -> h + conv(h): per channel, out_t = h_t + sum_j w[:, j] h_(t - (taps-1) + j), zeros before the start."""
    T, C = h.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), h.dtype), h], axis=0)
    out = h.copy()
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j][None, :]
    return out


def rotary_frequencies(rot: dict):
    dims = int(rot["dims"])
    i = np.arange(dims // 2, dtype=np.float64)
    return float(rot["base"]) ** (-2.0 * i / dims)


def rotate(x, positions, rot: dict):
    """x [T, heads, d]: the first ``dims`` channels of each head in the rotate-half layout (channel i with i + dims/2)."""
    dims = int(rot["dims"])
    half = dims // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---- mixers -----------------------------------------------------------------------------------

def lightning(h, w, p, m, eps):
    """Linear attention with a fixed decay per head: S <- decay_h S + k v^T, o = S^T q; q, k, v through silu; the heads'
    outputs normed TOGETHER, gated by a sigmoid, projected."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    decay = np.asarray(m["decay"], dtype=h.dtype)
    S = np.zeros((H, dk, dv), h.dtype)
    o = np.zeros((T, H, dv), h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    y = norm_plain(o.reshape(T, H * dv), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def mingru_candidate(u):
    return np.where(u >= 0, u + 0.5, sigmoid(u))


def mingru(h, w, p, m):
    """An element-wise recurrence: S <- (1 - z) S + z cand, gates from the current token only."""
    T = h.shape[0]
    z = sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    cand = mingru_candidate(h @ w[p + "x"].T + w[p + "x.b"])
    gate = silu(h @ w[p + "g"].T)
    S = np.zeros(m["width"], h.dtype)
    y = np.zeros((T, m["width"]), h.dtype)
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        y[t] = S * gate[t]
    return y @ w[p + "o"].T


def latent_parts(h, w, p, m, eps, positions):
    """(c [T, rank], rotated shared key part [T, rot_dim]) of a layer that owns a down-projection."""
    r = m["kv_rank"]
    d = h @ w[p + "dkv"].T
    c = norm_plain(d[:, :r], w[p + "dkv.norm"], eps)
    kr = rotate(d[:, None, r:], positions, m["rot"])[:, 0]
    return c, kr


def latent_attention(h, w, p, m, eps, positions, latents):
    """Softmax attention whose keys and values are up-projections of ``latents = (c, kr)``; a query head has ``dim``
    unrotated channels and ``rot_dim`` rotated ones; the denominator also holds exp(sink_h)."""
    T = h.shape[0]
    H, dk, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = latents
    q = (h @ w[p + "q"].T).reshape(T, H, dk + dr)
    qn, qr = q[..., :dk], rotate(q[..., dk:], positions, m["rot"])
    kn = (c @ w[p + "uk"].T).reshape(T, H, dk)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    sink = w[p + "sink"]
    out = np.zeros((T, H, dv), h.dtype)
    for t in range(T):
        for hh in range(H):
            s = (kn[:t + 1, hh] @ qn[t, hh] + kr[:t + 1] @ qr[t, hh]) * m["scale"]
            mx = max(s.max(), sink[hh])
            e = np.exp(s - mx)
            out[t, hh] = (e / (e.sum() + math.exp(sink[hh] - mx))) @ v[:t + 1, hh]
    y = out.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------

def clamped_unit(g, u, limit):
    g = np.minimum(g, limit)
    u = np.clip(u, -limit, limit)
    return g * sigmoid(1.702 * g) * (u + 1.0)


def dense(h, w, p, mlp):
    y = clamped_unit(h @ w[p + "gate"].T + w[p + "gate.b"], h @ w[p + "up"].T + w[p + "up.b"], mlp["limit"])
    return y @ w[p + "down"].T + w[p + "down.b"]


def route(h, w, p, r, margins=None):
    """(indices [T, top] by falling logit, weights [T, top]): the largest logits win, softmax over the winners only.
    ``margins``: a list that receives one array per call: per token, the gap between the last winner and the first loser
    relative to the largest logit's size (infinite where every expert is chosen)."""
    z = h @ w[p + "router"].T
    order = np.argsort(-z, axis=-1, kind="stable")
    idx = order[:, :r["top"]]
    chosen = np.take_along_axis(z, idx, axis=-1)
    if margins is not None:
        if r["top"] < r["experts"]:
            gap = chosen[:, -1] - np.take_along_axis(z, order[:, r["top"]:r["top"] + 1], axis=-1)[:, 0]
            margins.append(gap / (np.abs(z).max(-1) + 1e-30))
        else:
            margins.append(np.full(z.shape[0], np.inf))
    e = np.exp(chosen - chosen.max(-1, keepdims=True))
    return idx, e / e.sum(-1, keepdims=True)


def mixture(h, w, p, mlp, margins=None):
    idx, wt = route(h, w, p, mlp["router"], margins)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]), h.dtype)
    lim = mlp["expert"]["limit"]
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wt[t]):
            q = f"{p}e{int(e)}."
            y = clamped_unit(w[q + "gate"] @ h[t], w[q + "up"] @ h[t], lim)
            out[t] += a * (w[q + "down"] @ y)
    return out


# ---- the model ----------------------------------------------------------------------------------------

def forward(ids, cfg, w, dtype=np.float64, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the stream after each layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(ids)].astype(dtype)
    positions = np.arange(len(ids))
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        m = layer["mixer"]
        h = input_convolution(norm_scalar(x, w[L + "norm1"], eps), w[L + "canon1"])
        if layer["type"] == "lightning":
            y = lightning(h, w, L + "mix.", m, eps)
        elif layer["type"] == "mingru":
            y = mingru(h, w, L + "mix.", m)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                latents[i] = latent_parts(h, w, L + "mix.", m, eps, positions)
            y = latent_attention(h, w, L + "mix.", m, eps, positions, latents[i if m.get("kv_from") is None else m["kv_from"]])
        else:
            raise ValueError(layer["type"])
        x = x + norm_scalar(y, w[L + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = input_convolution(norm_scalar(x, w[L + "norm2"], eps), w[L + "canon2"])
            y = dense(h, w, L + "mlp.", mlp) if mlp["kind"] == "dense" else mixture(h, w, L + "mlp.", mlp, margins)
            x = x + norm_scalar(y, w[L + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    x = norm_scalar(x, w["final.norm"], eps)
    return x @ w["head"].T
