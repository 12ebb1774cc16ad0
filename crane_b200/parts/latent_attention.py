"""Latent attention over the paged cache.

Per position the cache holds one latent vector c [rank] (the leading rows of the down
projection, RMS-normed with a weight) and one rotated key part kr [rot] that all heads share.
Head h has the unrotated key U_h c and the value V_h c; its query is [q_h (dim), qr_h (rot,
rotated)] and its score (q_h . U_h c + qr_h . kr) * scale, causal, softmax.  The concatenated
heads are multiplied by sigmoid(W_g x) and go through the output projection.

The keys and values of a head are never formed.  Since q_h . U_h c = (U_h^T q_h) . c and
sum_j p_j V_h c_j = V_h sum_j p_j c_j, attention runs on the cache rows themselves: one shared
key/value head of width rank + rot whose values are the leading rank columns of the key rows,
queried by H heads [U_h^T q_h, qr_h], between two small per-head products (``head_linear``).
A layer with ``own_kv`` False has no down projection and reads the cache it is given, with U,
V, queries and everything else of its own.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, build_part, register_part

_NAMES = {"q": "q_proj.weight", "dkv": "kv_down_proj.weight", "dkv_norm": "kv_norm.weight",
          "uk": "k_up_proj.weight", "uv": "v_up_proj.weight", "gate": "gate_proj.weight",
          "out": "o_proj.weight"}


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: ``hidden_size``, ``heads``, ``dim`` / ``rot_dim`` (unrotated / rotated elements of a
    query or key head), ``vdim``, ``kv_rank``, ``scale`` (of the scores; as given, nothing is
    folded in), ``norm_eps`` (of the latent's RMS norm), ``own_kv``, ``gate`` (the sigmoid
    output gate; default off), ``position`` (a PartSpec whose tables rotate the leading
    ``width()`` elements of the rotated part, interleaved pairs), ``names`` (tensor names
    behind the prefix for q, dkv, dkv_norm, uk, uv, gate, out).
    Tensors: q [H (dim + rot), hidden], dkv [rank + rot, hidden], dkv_norm [rank] (float),
    uk [H dim, rank], uv [H vdim, rank], gate [H vdim, hidden], out [hidden, H vdim]."""
    kind = "mixer"

    @classmethod
    def _sizes(cls, a):
        return (int(a["hidden_size"]), int(a["heads"]), int(a["dim"]), int(a["rot_dim"]), int(a["vdim"]),
                int(a["kv_rank"]))

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, H, dim, rot, vd, r = cls._sizes(a)
        nm = dict(_NAMES, **(a.get("names") or {}))
        m = {p + nm["q"]: TensorSpec((H * (dim + rot), w)), p + nm["uk"]: TensorSpec((H * dim, r)),
             p + nm["uv"]: TensorSpec((H * vd, r)), p + nm["out"]: TensorSpec((w, H * vd))}
        if a.get("gate"):
            m[p + nm["gate"]] = TensorSpec((H * vd, w))
        if a.get("own_kv", True):
            m[p + nm["dkv"]] = TensorSpec((r + rot, w))
            m[p + nm["dkv_norm"]] = TensorSpec((r,), "float32", "scale")
        return m

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.w, self.H, self.dim, self.rot, self.vd, self.r = self._sizes(a)
        nm = dict(_NAMES, **(a.get("names") or {}))
        self.own_kv = bool(a.get("own_kv", True))
        self.gated = bool(a.get("gate"))
        self.scale = float(a["scale"])
        self.eps = float(a.get("norm_eps") or 0.0)
        H, dim, rot, vd, r = self.H, self.dim, self.rot, self.vd, self.r
        # one product for everything that reads the block's input: [q | gate | down projection]
        mats = [weights.pop(p + nm["q"])]
        self.g_off = mats[0].shape[0]
        if self.gated:
            mats.append(weights.pop(p + nm["gate"]))
        self.dkv_off = -1
        if self.own_kv:
            self.dkv_off = sum(m.shape[0] for m in mats)
            mats.append(weights.pop(p + nm["dkv"]))
        self.w_in = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.cols = self.w_in.shape[0]
        self.norm_w = weights.get(p + nm["dkv_norm"]) if self.own_kv else None
        # per head [inputs, outputs]: U_h as stored maps the latent to the key, so it is U_h^T's
        # [dim, rank] already; V_h [vdim, rank] is turned over
        self.uk = weights.pop(p + nm["uk"]).view(H, dim, r).contiguous()
        self.uv_t = weights.pop(p + nm["uv"]).view(H, vd, r).transpose(1, 2).contiguous()
        self.o_w = weights[p + nm["out"]]
        self.position = build_part(a["position"]) if a.get("position") is not None else None
        self.rot_dims = 0
        if self.position is not None:
            self.position.load(weights, rt)
            self.rot_dims = int(self.position.width())
        if rot % 2 or self.rot_dims % 2 or self.rot_dims > rot:
            raise ValueError(f"{p}: the rotated part ({rot}) and the rotated width ({self.rot_dims}) must be "
                             "even, the width at most the part")
        if r + rot > 1024 or r > 512:
            raise ValueError(f"{p}: cache rows of {r} + {rot} elements are wider than the attention "
                             "kernels take (1024, of which 512 latent)")

    def cache_need(self) -> CacheNeed:
        if not self.own_kv:
            return CacheNeed("none")
        return CacheNeed("kv", kv_heads=1, head_dim=self.r + self.rot, v_head_dim=self.r, values_in_keys=True)

    def forward(self, h, ctx, cache, rt):
        n = h.shape[0]
        k = rt.kernels
        H, dim, rot, vd, r = self.H, self.dim, self.rot, self.vd, self.r
        width = r + rot
        proj = rt.linear(h, self.w_in, None, "latent_proj")
        if self.position is not None:
            cos, sin = self.position.tables(rt, ctx.max_positions)
        else:
            cos, sin = _no_rotation(rt, ctx.max_positions)
        table = ctx.block_tables[cache.group]
        q_abs = rt.ws.get("latent_q", n, H * width, rt.dtype)
        k.latent_prep(proj, self.cols, 0, self.dkv_off, H, dim, rot, r, self.rot_dims, cos, sin,
                      ctx.positions, ctx.tok_entry, table, cache.k, cache.page_size, self.norm_w, self.eps,
                      q_abs, rt.err)
        k.head_linear(proj, self.cols, 0, dim + rot, self.uk, dim, r, q_abs, H * width, width, H,
                      tok_entry=ctx.tok_entry)
        o_lat = rt.ws.get("latent_o", n, H * r, rt.dtype)
        shape_only = ctx.graph_key is not None or ctx.graph_bucket > 0
        rt.launches += latent_attention_kernel(
            k, q_abs, o_lat, cache.k, ctx.positions, ctx.tok_entry, ctx.cu_q, ctx.kv_len, ctx.h_cu_q,
            ctx.h_kv_len, table, cache.page_size, H, r, rot, self.scale, rt.err, rt.exact,
            padded=ctx.n_tokens if shape_only else None, num_sms=rt.num_sms,
            all_single=bool(getattr(ctx, "all_single", False)) or ctx.graph_bucket > 0,
            scratch=lambda name, rows, cols, cap: rt.ws.get(name, rows, cols, torch.float32, cap=cap))
        o = rt.ws.get("attn_o", n, H * vd, rt.dtype)
        k.head_linear(o_lat, H * r, 0, r, self.uv_t, r, vd, o, H * vd, vd, H, tok_entry=ctx.tok_entry,
                      gate=proj if self.gated else None, g_cols=self.cols, g_off=self.g_off)
        rt.launches += 3
        # (hold: a parallel block adds this only after its feed-forward's products have run)
        return rt.linear(o, self.o_w, None, "attn_out", hold=True)


def latent_attention_kernel(k, q, out, pool, positions, tok_entry, cu_q, kv_len, h_cu_q, h_kv_len, table,
                            page_size, heads, rank, rot, scale, err, exact, padded=None, num_sms=148,
                            scratch=None, all_single=False) -> int:
    """out [N, heads * rank] = attention of q [N, heads * (rank + rot)] over the cache rows of
    ``pool`` [pages, 1, page_size, rank + rot], whose values are their leading ``rank`` columns.
    True 32-bit, or widths that the tensor-core kernel does not take: the FP32-core kernel.
    Else the tensor-core kernel, once for the entries of one token or at most 16 rows (16-row
    tiles) and once for the others, each with its keys in as many slices as fill the device.
    ``padded``: the step's shape is fixed by a captured graph (this many rows): tile counts
    and slices are then bounds that depend on the shape alone (``all_single``: the shape says
    that every entry has one token).  Returns the launches."""
    width = rank + rot
    if exact or not k.latent_attention_mma_supports(width, rank):
        k.paged_attention_simt(q, out, pool, pool, positions, tok_entry, table, page_size, heads, 1, width, 0,
                               scale, err, dv=rank, v_stride=width)
        return 1
    n_entries = kv_len.shape[0]
    if padded is not None:
        small_tiles = n_entries * (-(-heads // 16))
        # (a step of nothing but single tokens, which is part of a padded step's shape, has no 64-row tiles)
        big_tiles = 0 if all_single else n_entries + (int(padded) * heads) // 64
        most_keys = 1 << 30
    else:
        q_lens = h_cu_q[1:n_entries + 1] - h_cu_q[:n_entries]
        rows = q_lens * heads
        small = (rows > 0) & ((q_lens == 1) | (rows <= 16))
        small_tiles = int(((rows[small] + 15) // 16).sum())
        big_tiles = int(((rows[(rows > 0) & ~small] + 63) // 64).sum())
        most_keys = int(h_kv_len[:n_entries].max())
    if scratch is None:
        scratch = lambda name, n, cols, cap: torch.empty((n, cols), dtype=torch.float32, device=q.device)
    launches = 0
    for small, tiles in ((True, small_tiles), (False, big_tiles)):
        if tiles == 0:
            continue
        bm = 16 if small else 64
        # slices: enough CTAs to fill the device (four times over for the 16-row tiles, whose CTAs are
        # short chains of dependent steps), none of fewer than 128 keys
        splits = max(1, min(64 if small else 8, ((4 if small else 1) * num_sms) // tiles, -(-most_keys // 128)))
        part_o = part_ml = None
        if splits > 1:
            # (with two slices or more, tiles x slices is at most the CTAs aimed at)
            cap = 4 * num_sms * 16 if small else (num_sms + 1) * 64
            part_o = scratch("latent_part_o" + ("_s" if small else ""), tiles * splits * bm, rank, max(cap, tiles * splits * bm))
            part_ml = scratch("latent_part_ml" + ("_s" if small else ""), tiles * splits * bm, 2, max(cap, tiles * splits * bm))
        k.latent_attention_mma(q, out, pool, cu_q, kv_len, table, page_size, tiles, splits, small, heads, width,
                               rank, scale, part_o, part_ml, err)
        launches += 1 if splits == 1 else 2
    return launches


_IDENTITY = {}


def _no_rotation(rt, n):
    key = (str(rt.device), int(n))
    if key not in _IDENTITY:
        _IDENTITY[key] = (torch.ones((n, 1), dtype=torch.float32, device=rt.device),
                          torch.zeros((n, 1), dtype=torch.float32, device=rt.device))
    return _IDENTITY[key]
