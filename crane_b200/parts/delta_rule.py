"""The generalized delta rule: a mixer whose memory is one matrix per head and request.

Per token and head, with receptance r, key k and value v (each ``dim`` wide, all products of
the block's input), decay w and removal rate a per key channel and the unit key
u = k / sqrt(sum(k^2) + key_eps):

    S <- diag(w) S - (a * u) (u^T S) + k v^T          (both corrections read the old S)
    o  = S^T r

    w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0)),   a = sigmoid(W_a x + b_a)

Each head's o is divided by its root mean square, multiplied by a weight over all heads and by
sigmoid(W_g x), and goes through the output projection.  S [dim, dim] starts at zero and is
kept in 32-bit in the request's state slot; everything between the projections and the output
projection is computed in 32-bit.
"""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, register_part

_NAMES = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2", "w0": "w0",
          "norm": "norm", "o": "o"}


@register_part("mixer", "general_delta")
class GeneralDelta(Part):
    """params: ``hidden_size``, ``heads``, ``dim``, ``norm_eps`` (of the head norm), ``decay_scale``
    (default exp(-1/2)), ``key_eps`` (default 1e-6), ``decay_rank`` (the inner size of the decay's
    two products; None: read from the stored tensor), ``names`` (tensor names behind the prefix).
    Tensors: r, k, v, g, a, o [H dim, hidden] ([hidden, H dim] for o), w1 [rank, hidden],
    w2 [H dim, rank], and in 32-bit a_bias, w0, norm [H dim]."""
    kind = "mixer"
    state_graph_safe = True      # the kernels read the step's metadata on the device, skip rows of no
                                 # entry and touch no slot for an entry without rows

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, hd = int(a["hidden_size"]), int(a["heads"]) * int(a["dim"])
        nm = dict(_NAMES, **(a.get("names") or {}))
        rank = a.get("decay_rank")
        rank, free = (-1, 16) if rank is None else (int(rank), 0)
        m = {p + nm[n]: TensorSpec((hd, w)) for n in ("r", "k", "v", "g", "a")}
        m[p + nm["o"]] = TensorSpec((w, hd))
        m[p + nm["w1"]] = TensorSpec((rank, w), free=free)
        m[p + nm["w2"]] = TensorSpec((hd, rank), free=free)
        m[p + nm["a_bias"]] = TensorSpec((hd,), "float32", "offset")
        m[p + nm["w0"]] = TensorSpec((hd,), "float32", "offset")
        m[p + nm["norm"]] = TensorSpec((hd,), "float32", "scale")
        return m

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.H, self.d = int(a["heads"]), int(a["dim"])
        nm = dict(_NAMES, **(a.get("names") or {}))
        self.eps = float(a.get("norm_eps") or 0.0)
        self.decay_scale = float(a["decay_scale"]) if a.get("decay_scale") is not None else math.exp(-0.5)
        self.key_eps = float(a["key_eps"]) if a.get("key_eps") is not None else 1e-6
        if self.d > rt.kernels.delta_rule_max_dim():
            raise ValueError(f"{p}: a head of {self.d} elements is wider than the recurrence kernel takes "
                             f"({rt.kernels.delta_rule_max_dim()})")
        # one product for everything that reads the block's input: [r | k | v | g | a | w1]
        self.w_in = torch.cat([weights.pop(p + nm[n]) for n in ("r", "k", "v", "g", "a", "w1")], dim=0).contiguous()
        self.cols = self.w_in.shape[0]
        self.w2t = weights.pop(p + nm["w2"]).t().contiguous()         # [rank, H dim]: channels side by side
        self.w0, self.a_bias, self.norm_w = weights[p + nm["w0"]], weights[p + nm["a_bias"]], weights[p + nm["norm"]]
        self.o_w = weights[p + nm["o"]]
        if self.w2t.shape[0] != self.cols - 5 * self.H * self.d:
            raise ValueError(f"{p}: the decay's two matrices do not share their inner size")

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(self.H, self.d, self.d), state_dtype=torch.float32)

    def forward(self, h, ctx, cache, rt):
        n = h.shape[0]
        k = rt.kernels
        hd = self.H * self.d
        proj = rt.linear(h, self.w_in, None, "delta_proj")
        aux = rt.ws.get("delta_aux", n, 3 * hd, torch.float32)
        k.delta_rule_prep(proj, self.cols, ctx.tok_entry, self.w2t, self.w0, self.a_bias, aux, self.H, self.d,
                          self.decay_scale, self.key_eps, rt.dtype)
        o = rt.ws.get("delta_o", n, hd, rt.dtype)
        # Few and long entries (a prompt alone): a head's columns go over four CTAs, or the one CTA per
        # (entry, head) leaves most of the device idle while it walks the tokens.  (Rows and entries are
        # part of a padded step's shape, so a recorded graph holds the choice.)
        blocks = 4 if n >= 64 * ctx.n_entries and 4 * ctx.n_entries * self.H <= 3 * rt.num_sms else 1
        o_raw = rt.ws.get("delta_o_raw", n, hd, torch.float32) if blocks > 1 else None
        k.delta_rule_scan(proj, self.cols, aux, ctx.cu_q, ctx.kv_len, ctx.slots, cache.state, self.norm_w,
                          self.eps, o, self.H, self.d, rt.err, col_blocks=blocks, o_raw=o_raw, tok_entry=ctx.tok_entry)
        rt.launches += 2 if blocks == 1 else 3
        return rt.linear(o, self.o_w, None, "delta_out")
