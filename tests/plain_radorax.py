"""A plain, slow restatement of Radorax in NumPy float64, one function per mechanism, written
from the design's equations and sharing nothing with the engine.  Keys and values of every
head are formed here (k_h = U_h c, v_h = V_h c), which the engine never does.

Notation: n tokens, W width, H heads; per head d unrotated and e rotated query/key elements,
m value elements; r the latent's width.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch

from crane_b200.weights.safetensors_io import TensorSource, model_files


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    src = TensorSource(model_files(folder))
    w = {}
    for name in src.names():
        t = src.tensor(name)
        w[name] = t.to(torch.float64).numpy() if t.dtype.is_floating_point else t.numpy()
    return cfg, w


def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int, before: Optional[int] = None):
    """Row of the bigram table for every token; ``before``: the token ahead of tokens[0]
    (None: tokens[0] opens the sequence and takes the table's last row)."""
    rows, prev = [], before
    for t in tokens:
        rows.append(buckets if prev is None else (prev * mul_prev + t * mul_cur) % buckets)
        prev = t
    return rows


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdims=True)
    var = ((x - mean) ** 2).mean(-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def softplus(v):
    return np.log1p(np.exp(v))


def xielu(z, p, q):
    above = softplus(p) * z * z + z / 2
    below = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - np.minimum(z, 0.0)) + z / 2
    return np.where(z > 0, above, below)


def yarn_tables(rot: dict, positions: np.ndarray):
    """cos, sin [len(positions), dims / 2] with the scaling's factor on both."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        def dim_of(t):
            return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(dim_of(sc["fast"])), 0)
        hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(sc["factor"]) + 1.0
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    return np.cos(a) * mult, np.sin(a) * mult


def rotate_pairs(x, cos, sin, dims: int):
    """x [..., n, width]: elements (2i, 2i + 1), i < dims / 2, are turned by the angle of row n."""
    out = np.array(x, dtype=np.float64, copy=True)
    if dims == 0:
        return out
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_cache_rows(h, w, prefix, m, eps, positions):
    """What a layer with a cache of its own keeps per position: latent c [n, r], rotated part kr [n, e]."""
    r = m["kv_rank"]
    cos, sin = yarn_tables(m["rot"], positions)
    down = h @ w[prefix + "dkv"].T
    c = rms_norm(down[:, :r], w[prefix + "dkv.norm"], eps)
    kr = rotate_pairs(down[:, r:], cos, sin, m["rot"]["dims"])
    return c, kr


def latent_attention(h, w, prefix, m, c, kr, positions, key_positions):
    """h [n, W]: the mixer's input at ``positions``; c, kr: cache rows at ``key_positions``
    (a superset).  Causal: a query at position p sees keys at positions <= p."""
    n = h.shape[0]
    H, d, e, mv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cos, sin = yarn_tables(m["rot"], positions)
    q = (h @ w[prefix + "q"].T).reshape(n, H, d + e)
    q_plain = q[..., :d]
    q_rot = rotate_pairs(q[..., d:].transpose(1, 0, 2), cos, sin, m["rot"]["dims"]).transpose(1, 0, 2)
    keys = (c @ w[prefix + "uk"].T).reshape(len(c), H, d)
    vals = (c @ w[prefix + "uv"].T).reshape(len(c), H, mv)
    s = (np.einsum("ihd,jhd->hij", q_plain, keys) + np.einsum("ihe,je->hij", q_rot, kr)) * m["scale"]
    seen = np.asarray(key_positions)[None, :] <= np.asarray(positions)[:, None]
    s = np.where(seen[None], s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    o = np.einsum("hij,jhm->ihm", p, vals).reshape(n, H * mv)
    o = o / (1.0 + np.exp(-(h @ w[prefix + "g"].T)))
    return o @ w[prefix + "o"].T


def feed_forward(h, w, prefix):
    p, q = w[prefix + "act"]
    return xielu(h @ w[prefix + "up"].T, p, q) @ w[prefix + "down"].T


def depth_average(results: List[np.ndarray], weights: np.ndarray):
    return sum(weights[j] * results[j] for j in range(len(results)))


def embed(cfg, w, tokens):
    x = w["embed"][tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + w["bigram"][bigram_rows(list(tokens), bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


def logits_all(cfg, w, tokens, streams: Optional[list] = None) -> np.ndarray:
    """Logits [n, vocab] at every position of one sequence.  ``streams``: gets the stream
    after every layer (after its depth-weighted average)."""
    n, eps = len(tokens), cfg["norm"]["eps"]
    pos = np.arange(n)
    x = embed(cfg, w, tokens)
    results = [x]
    caches: Dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if m.get("kv_from") is None:
            caches[i] = latent_cache_rows(h, w, p + "mix.", m, eps, pos)
        c, kr = caches[i if m.get("kv_from") is None else m["kv_from"]]
        y = latent_attention(h, w, p + "mix.", m, c, kr, pos, pos)
        if layer.get("mlp"):
            y = y + feed_forward(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.")
        results.append(x + y)
        x = depth_average(results, w[p + "dwa"])
        if streams is not None:
            streams.append(x)
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T


def greedy_generate(cfg, w, prompt: List[int], n_new: int) -> List[int]:
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(logits_all(cfg, w, tokens)[-1])))
    return tokens
