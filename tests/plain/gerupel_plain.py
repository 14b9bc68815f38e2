"""Plain, slow, whole-sequence statement of the Gerupel design, one function per mechanism.

A decoder-only model whose embedding is normed before it enters the stream, whose layers add the mixer's and the
feed-forward's terms in parallel, x <- x + m (mixer(norm1 x) + ff(norm2 x)), and of which a range of layers may run
several times in a row with the same weights (each pass with a cache of its own, the embedding output and a vector per
pass added in front).  The mixer is two mixers side by side on one input, summed with a factor each: softmax attention
(grouped heads, part of each head rotated by position with a three-regime frequency scaling, a factor per head on the
scores, a window of recent tokens plus one mean key and value per block of older tokens, one added to the softmax's
denominator) and a linear attention whose forget gate also writes (HGRN2).  The feed-forward is a mixture of gated
experts behind a softmax router.  The output head is the embedding table.

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


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


# ---- rotation -------------------------------------------------------------------------------

def rotary_frequencies(base: float, dims: int, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` (factor, low, high, original) a frequency whose wavelength is
    longer than original/low is divided by factor, one whose wavelength is shorter than original/high stays, and between
    the two the divided and the plain frequency are blended by s = (original/wavelength - low) / (high - low)."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out[i] = fi
        elif wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, freqs):
    """x [T, heads, dim]: the first 2 len(freqs) channels of each head in pairs (i, i + len(freqs))."""
    half = len(freqs)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


# ---- the attention side -----------------------------------------------------------------------

def pooled_window_attention(q, k, v, scale, temp, window: int, pool: int):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] of one sequence (positions 0..T-1), ``temp`` [H].

    Query i sees the keys j with 0 <= i - j < window, and one key and value per block b of ``pool`` positions that ends
    at or before i - window: the means of the block's keys and of its values.  One softmax over both kinds, with one
    added to its denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=q.dtype)
    nblocks = T // pool if pool else 0
    pk = np.stack([k[b * pool:(b + 1) * pool].mean(0) for b in range(nblocks)]) if nblocks else np.zeros((0,) + k.shape[1:], q.dtype)
    pv = np.stack([v[b * pool:(b + 1) * pool].mean(0) for b in range(nblocks)]) if nblocks else np.zeros((0,) + v.shape[1:], q.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)
        seen = [b for b in range(nblocks) if b * pool + pool - 1 <= i - window]
        for h in range(H):
            g = h // (H // G)
            keys = np.concatenate([pk[seen, g], k[lo:i + 1, g]], axis=0)
            vals = np.concatenate([pv[seen, g], v[lo:i + 1, g]], axis=0)
            s = keys @ q[i, h] * scale * temp[h]
            m = max(float(s.max()), 0.0)
            e = np.exp(s - m)
            out[i, h] = (e[:, None] * vals).sum(0) / (math.exp(-m) + e.sum())
    return out


def attention_side(h, w, p, cfg, positions=None):
    """The left mixer: projections, rotation, the pooled-window softmax, the output projection.  ``w``: tensors by their
    names under the side's prefix; ``p``: the side's section of the configuration."""
    T = h.shape[0]
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = (h @ w["q"].T).reshape(T, H, dim)
    k = (h @ w["k"].T).reshape(T, G, dim)
    v = (h @ w["v"].T).reshape(T, G, vdim)
    rot = p.get("rot")
    if rot:
        f = rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        pos = np.arange(T) if positions is None else positions
        q, k = rotate(q, pos, f), rotate(k, pos, f)
    mask = p.get("mask")
    window = mask["size"] if mask else T + 1                      # no mask: every earlier token, no blocks
    pool = mask.get("pool") if mask else None
    o = pooled_window_attention(q, k, v, p["scale"], w["temp"], window, pool)
    return o.reshape(T, H * vdim) @ w["o"].T


# ---- the recurrent side -------------------------------------------------------------------------

def hgrn2(q, f, v):
    """q, f [T, H, dim], v [T, H, vdim]: S <- diag(f) S + (1 - f) v^T, o = S^T q per head, from a zero state."""
    T, H, dim = q.shape
    S = np.zeros((H, dim, v.shape[2]), dtype=q.dtype)
    out = np.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out


def recurrent_side(h, w, p, eps):
    T = h.shape[0]
    H, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, dim)
    v = (h @ w["v"].T).reshape(T, H, vdim)
    lower = w["lower"]
    f = (lower + (1.0 - lower) * sigmoid(h @ w["f"].T + w["f.b"])).reshape(T, H, dim)
    o = hgrn2(q, f, v)
    o = rms_norm(o, w["norm"], eps)
    return o.reshape(T, H * vdim) @ w["o"].T


# ---- the feed-forward -----------------------------------------------------------------------------

def route(z, top: int, scale: float):
    """Router logits z [T, E] -> (indices [T, top], weights [T, top]): softmax over all experts, the ``top`` largest, their
    scores over their sum, times ``scale``."""
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(s, idx, axis=-1)
    return idx, chosen / (chosen.sum(-1, keepdims=True) + 1e-20) * scale


def experts(h, w, p, margins=None):
    """The mixture: w by names under the feed-forward's prefix (``router``, ``e<i>.gate``, ``.up``, ``.down``).  ``margins``
    (a list) receives, per token, the gap between the last chosen logit and the best one left out, relative to the
    logits' size (infinite where every expert is chosen)."""
    r = p["router"]
    z = h @ w["router"].T
    idx, wts = route(z, r["top"], r["scale"])
    if margins is not None:
        zs = -np.sort(-z, axis=-1)
        top = r["top"]
        margins.append((zs[:, top - 1] - zs[:, top]) / (np.abs(z).max(-1) + 1e-30) if top < z.shape[1] else np.full(len(z), np.inf))
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]), dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wts[t]):
            act = silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])
            out[t] += a * (w[f"e{e}.down"] @ act)
    return out


# ---- the model --------------------------------------------------------------------------------------

def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix) + 1:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def run_order(cfg):
    """[(layer, pass number or None)]: the layers before the loop, the looped range ``times`` times, the rest."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t) for i in range(loop["start"], loop["stop"])]
    order += [(i, None) for i in range(loop["stop"], L)]
    return order


def layer(x, i, cfg, weights, margins=None):
    lc = cfg["layers"][i]
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    mix = lc["mixer"]
    h1 = rms_norm(x, weights[f"l{i}.norm1"], eps)
    term = mix["left_scale"] * attention_side(h1, sub(weights, f"l{i}.mix.left"), mix["left"], cfg) \
        + mix["right_scale"] * recurrent_side(h1, sub(weights, f"l{i}.mix.right"), mix["right"], eps)
    if lc.get("mlp") is not None:
        h2 = rms_norm(x, weights[f"l{i}.norm2"], eps)
        term = term + experts(h2, sub(weights, f"l{i}.mlp"), lc["mlp"], margins)
    return x + m * term


def forward(cfg, weights, tokens, collect=None, margins=None):
    """Logits [T, vocab] of one sequence.  ``collect``: a list that receives the stream after every layer run; ``margins``:
    one that receives every router's margins (see `experts`)."""
    eps = cfg["norm"]["eps"]
    emb = rms_norm(weights["embed"][np.asarray(tokens)], weights["embed.norm"], eps)
    x = emb.copy()
    loop = cfg.get("loop")
    for i, t in run_order(cfg):
        if t is not None and i == loop["start"]:
            if t > 0:
                x = x + emb
            x = x + weights["loop.step"][t]
        x = layer(x, i, cfg, weights, margins)
        if collect is not None:
            collect.append(x.copy())
    return rms_norm(x, weights["final.norm"], eps) @ weights["embed"].T
