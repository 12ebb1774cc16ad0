"""Arrangements of parts in a layer.

``prenorm_residual``: h = norm1(x); x += mixer(h); h = norm2(x); x += ffn(h)
(crane-core/src/models/hunyuan_dense/modeling.rs:792-810).  Each addition is
fused into the norm that follows it, so a block hands its last output on
unadded ("pending") and receives the one of the block before it.

``parallel_depth_average``: both branches read norms of the same x, their sum
is added once, and what the next layer reads is a weighted sum of all layer
results so far.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, build_part, register_block, register_part
from .norm import BranchSum, combine_and_norm


@register_block("prenorm_residual")
class PreNormResidualBlock:
    """parts: ``norm1``, ``mixer``, ``norm2``, ``ffn``."""

    def __init__(self, layer_spec):
        self.norm1 = build_part(layer_spec.parts["norm1"])
        self.mixer = build_part(layer_spec.parts["mixer"])
        self.norm2 = build_part(layer_spec.parts["norm2"])
        self.ffn = build_part(layer_spec.parts["ffn"])

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, x, pending, ctx, cache, rt):
        h = self.norm1.forward(x, pending, rt)
        a = self.mixer.forward(h, ctx, cache, rt)
        h = self.norm2.forward(x, a, rt)
        return self.ffn.forward(h, ctx, rt)


@register_part("combine", "depth_average")
class DepthAverage(Part):
    """After layer ``index`` the stream is sum_j w[j] X_j over j = 0 .. index + 1, X_0 the
    embedding output and X_(j+1) the result of layer j (its input stream plus its branches).
    params: ``index``, ``slots`` (layers + 1), ``size``, ``weight`` (tensor name behind the
    prefix).  Tensor [index + 2], kept float.  The X_j of a step live in one float buffer
    [slots, rows, size] that all layers' parts share; the kernel that adds a block's
    branches writes X_(index+1) there and reads the others."""
    kind = "combine"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + spec.params.get("weight", "weight"):
                TensorSpec((spec.params["index"] + 2,), "float32", "mix")}

    def load(self, weights, rt):
        self.weights = weights[self.prefix + self.params.get("weight", "weight")]
        self.index, self.slots, self.size = (int(self.params[k]) for k in ("index", "slots", "size"))

    def history(self, rt, rows: int):
        buf = rt.ws.get("layer_history", self.slots * rows, self.size, torch.float32,
                        cap=self.slots * rt.ws.max_rows)
        return buf.view(self.slots, rows, self.size)


@register_block("parallel_depth_average")
class ParallelDepthAverageBlock:
    """x <- x + (mixer(norm1(x)) + ffn(norm2(x))), both branches of the same x, then the
    depth-weighted average of ``combine``.  parts: ``norm1``, ``mixer``, ``combine`` and,
    unless the layer has no feed-forward, ``norm2`` and ``ffn``.  The additions, the
    average and the next reader's norms are one kernel (``norm.combine_and_norm``), so
    the block hands its branches on as a ``BranchSum``."""

    def __init__(self, layer_spec):
        p = layer_spec.parts
        self.norm1 = build_part(p["norm1"])
        self.mixer = build_part(p["mixer"])
        self.combine = build_part(p["combine"]) if "combine" in p else None
        self.ffn = build_part(p["ffn"]) if "ffn" in p else None
        self.norm2 = build_part(p["norm2"]) if self.ffn is not None else None
        self.norm1.history_of = self.combine

    def parts(self):
        return [q for q in (self.norm1, self.mixer, self.norm2, self.ffn, self.combine) if q is not None]

    def forward(self, x, pending, ctx, cache, rt):
        h1, h2 = combine_and_norm(x, pending, self.norm1, self.norm2, rt)
        a = self.mixer.forward(h1, ctx, cache, rt)
        f = self.ffn.forward(h2, ctx, rt) if self.ffn is not None else None
        return BranchSum(a, f, self.combine)
