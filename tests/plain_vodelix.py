"""A plain, slow restatement of Vodelix in NumPy float64, one function per mechanism, written
from the design's equations and sharing nothing with the engine.

Notation: n tokens, W width, H heads, G key/value heads, d key size, m value size, E experts.
Weights are dictionaries name -> float64 array (integer tables stay integer).  Every matrix
is stored [out, in] and applied as ``x @ M.T`` to rows x.
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


# ------------------------------------------------------------------ small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def relu_squared(z):
    return np.maximum(z, 0.0) ** 2


def unit_rms(x, eps):
    """x over the root of its mean square, eps under the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps, offset=0.0):
    return unit_rms(x, eps) * (offset + w)


def sinusoid(positions, width):
    """[n, W]: column 2i is sin(p f_i), column 2i + 1 is cos(p f_i), f_i = 10000^(-2i / W)."""
    out = np.zeros((len(positions), width))
    p = np.asarray(positions, dtype=np.float64)[:, None]
    i = np.arange((width + 1) // 2, dtype=np.float64)[None, :]
    ang = p * 10000.0 ** (-2.0 * i / width)
    out[:, 0::2] = np.sin(ang)[:, :out[:, 0::2].shape[1]]
    out[:, 1::2] = np.cos(ang)[:, :out[:, 1::2].shape[1]]
    return out


def embedding(w, tokens, positions, width):
    return w["embed"][np.asarray(tokens)] + sinusoid(positions, width)


# ------------------------------------------------------------------ mixers
def sink_attention(h, w, p, mixer, eps):
    """Causal attention without positions whose softmax has one more, silent, candidate of
    score 0 and no value; q and k are RMS-normed over their whole projections."""
    H, d = mixer["heads"], mixer["dim"]
    G = mixer.get("kv_heads", H)
    m = mixer.get("vdim", d)
    n = h.shape[0]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(n, H, d)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(n, G, d)
    v = (h @ w[p + "v"].T).reshape(n, G, m)
    out = np.zeros((n, H, m))
    for hd in range(H):
        g = hd // (H // G)
        for i in range(n):
            s = (k[:i + 1, g] @ q[i, hd]) * mixer["scale"]
            e = np.exp(s)
            out[i, hd] = (e / (1.0 + e.sum())) @ v[:i + 1, g]
    return out.reshape(n, H * m) @ w[p + "o"].T


def delta_rule_inputs(h, w, p, H, d):
    """Per token and head: receptance, key, value, decay, removal rate, unit key, output gate."""
    n = h.shape[0]
    r = (h @ w[p + "r"].T).reshape(n, H, d)
    k = (h @ w[p + "k"].T).reshape(n, H, d)
    v = (h @ w[p + "v"].T).reshape(n, H, d)
    low = np.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    decay = np.exp(-math.exp(-0.5) * sigmoid(low)).reshape(n, H, d)
    rate = sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(n, H, d)
    unit = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    gate = sigmoid(h @ w[p + "g"].T)
    return r, k, v, decay, rate, unit, gate


def delta_rule_step(S, r, k, v, decay, rate, unit):
    """One token of one head.  S [d, d] (key channel x value channel):
    S' = decay[:, None] * S - (rate * unit)[:, None] * (unit @ S)[None, :] + k[:, None] * v[None, :];
    the read-out is S'^T r."""
    S = decay[:, None] * S - np.outer(rate * unit, unit @ S) + np.outer(k, v)
    return S, S.T @ r


def general_delta(h, w, p, mixer, eps, state=None):
    """``state``: [H, d, d] carried in from earlier tokens (None: zeros).  Returns the mixer's
    output and the state after the last token."""
    H, d = mixer["heads"], mixer["dim"]
    n = h.shape[0]
    r, k, v, decay, rate, unit, gate = delta_rule_inputs(h, w, p, H, d)
    S = np.zeros((H, d, d)) if state is None else state.copy()
    o = np.zeros((n, H, d))
    for t in range(n):
        for hd in range(H):
            S[hd], o[t, hd] = delta_rule_step(S[hd], r[t, hd], k[t, hd], v[t, hd], decay[t, hd],
                                              rate[t, hd], unit[t, hd])
    o = unit_rms(o, eps).reshape(n, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T, S


# ------------------------------------------------------------------ feed-forward
def dense_ffn(h, w, p):
    return relu_squared(h @ w[p + "up"].T) @ w[p + "down"].T


def expert(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def route(h, w, p, top):
    """Per token the chosen experts (largest logits first) and their weights: a softmax over
    the chosen logits only."""
    z = h @ w[p + "router"].T
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, -1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return idx, e / e.sum(-1, keepdims=True)


def moe_ffn(h, w, p, mlp):
    idx, wt = route(h, w, p, mlp["router"]["top"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(idx[t]):
            out[t] += wt[t, j] * expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out += expert(h, w, p + "shared.")
    return out


def feed_forward(h, w, p, mlp):
    return dense_ffn(h, w, p) if mlp["kind"] == "dense" else moe_ffn(h, w, p, mlp)


# ------------------------------------------------------------------ the layer and the model
def token_side(x, tokens, w, i, side_dim, eps):
    """The per-layer token input: layer i's slice of the side table gates a small projection
    of the stream; the result is normed (plain weight) and added."""
    e = w["side.embed"][np.asarray(tokens)][:, i * side_dim:(i + 1) * side_dim]
    g = gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e
    y = g @ w[f"l{i}.side.proj"].T
    return x + unit_rms(y, eps) * w[f"l{i}.side.norm"]


def layer(x, tokens, cfg, w, i, state=None):
    """One run of layer i over a whole sequence (or its continuation, for the recurrent
    mixer, from ``state``).  Returns the stream and the mixer's state (None for attention)."""
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps, 1.0)
    if L["type"] == "attention":
        m, state = sink_attention(h, w, p + "mix.", L["mixer"], eps), None
    else:
        m, state = general_delta(h, w, p + "mix.", L["mixer"], eps, state)
    x = x + rms_norm(m, w[p + "norm1b"], eps, 1.0)
    if L.get("mlp"):
        f = feed_forward(rms_norm(x, w[p + "norm2"], eps, 1.0), w, p + "mlp.", L["mlp"])
        x = x + rms_norm(f, w[p + "norm2b"], eps, 1.0)
    if cfg.get("token_side"):
        x = token_side(x, tokens, w, i, cfg["token_side"]["dim"], eps)
    return x, state


def layer_runs(cfg):
    """The order in which layers run: (layer, pass number or None, first of its pass)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, keep_layers=False):
    """Logits [n, vocab] of one whole sequence; with ``keep_layers`` also the stream after
    every layer run [runs, n, W]."""
    x0 = embedding(w, tokens, range(len(tokens)), cfg["width"])
    x = x0.copy()
    kept = []
    for i, t, first in layer_runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x, _ = layer(x, tokens, cfg, w, i)
        kept.append(x.copy())
    logits = rms_norm(x, w["final.norm"], cfg["norm"]["eps"], 1.0) @ w["embed"].T
    return (logits, np.stack(kept)) if keep_layers else logits


def logits_all(cfg, w, tokens):
    return forward(cfg, w, tokens)


def greedy_generate(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, w, toks)[-1])))
    return toks
