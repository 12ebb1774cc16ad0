"""Tiny Radorax configurations for tests.  They differ from one another in every size, and
each sets apart what a model may happen to make equal: value and key widths, feed-forward and
model width, the rotated width and the rotated part, the layers' head counts."""


def _mixer(heads, dim, rot_dim, vdim, kv_rank, dims, base, scaling, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": dims, "base": base}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


_YA = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
_YB = {"factor": 1.5, "original": 64, "fast": 16.0, "slow": 2.0}

# three layers: own cache; a reader of it with other head count and sizes; own cache without
# feed-forward, partly rotated (rot.dims < rot_dim), no scaling
RA = {
    "architecture": "Radorax", "vocab": 203, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 37, "mul_prev": 31, "mul_cur": 5}},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(4, 16, 8, 24, 32, 8, 1000.0, _YA, 0.21),
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "latent_attention", "mixer": _mixer(2, 32, 8, 16, 32, 8, 1000.0, _YA, 0.17, kv_from=0),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "latent_attention", "mixer": _mixer(3, 8, 16, 8, 48, 8, 300.0, None, 0.3), "mlp": None},
    ],
}

# odd head count, widths off the powers of two, two readers of one cache, large multipliers
RB = {
    "architecture": "Radorax", "vocab": 333, "width": 160, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 101, "mul_prev": 1000003, "mul_cur": 7919}},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(5, 24, 4, 40, 72, 4, 50.0, _YB, 0.15),
         "mlp": {"kind": "dense", "ff": 200}},
        {"type": "latent_attention", "mixer": _mixer(5, 24, 4, 40, 72, 4, 50.0, _YB, 0.2, kv_from=0),
         "mlp": {"kind": "dense", "ff": 200}},
        {"type": "latent_attention", "mixer": _mixer(1, 48, 4, 56, 72, 4, 50.0, _YB, 0.1, kv_from=0),
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "latent_attention", "mixer": _mixer(2, 64, 32, 64, 96, 32, 20000.0, _YB, 0.12),
         "mlp": {"kind": "dense", "ff": 160}},
    ],
}

# one layer, one head, no bigram table, nothing rotated
RC = {
    "architecture": "Radorax", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "layers": [{"type": "latent_attention", "mixer": _mixer(1, 16, 0, 16, 16, 0, 10.0, None, 0.25),
                "mlp": {"kind": "dense", "ff": 48}}],
}

# layer sizes at which the tensor-core kernels are taken (key rows of 128 + 32 elements)
RL = {
    "architecture": "Radorax", "vocab": 512, "width": 512, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 509, "mul_prev": 3, "mul_cur": 11}},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(8, 64, 32, 64, 128, 32, 10000.0, _YB, 0.1),
         "mlp": {"kind": "dense", "ff": 1024}},
        {"type": "latent_attention", "mixer": _mixer(8, 64, 32, 64, 128, 32, 10000.0, _YB, 0.1, kv_from=0),
         "mlp": {"kind": "dense", "ff": 1024}},
    ],
}

# more heads than a 16-row tile holds: decoded tokens take the 64-row tiles; the second layer without
# feed-forward reads the first one's cache
RH = {
    "architecture": "Radorax", "vocab": 150, "width": 96, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 53, "mul_prev": 17, "mul_cur": 3}},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(20, 16, 16, 8, 32, 16, 5000.0, _YA, 0.18),
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "latent_attention", "mixer": _mixer(18, 8, 16, 16, 32, 16, 5000.0, _YA, 0.2, kv_from=0), "mlp": None},
    ],
}

TINY = {
    "RA": {"config": RA, "seed": 11, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "RB": {"config": RB, "seed": 12, "std": 0.06, "norm_std": 0.05, "page_size": 8},
    "RC": {"config": RC, "seed": 13, "std": 0.1, "norm_std": 0.05, "page_size": 64},
    "RL": {"config": RL, "seed": 14, "std": 0.03, "norm_std": 0.05, "page_size": 64},
    "RH": {"config": RH, "seed": 15, "std": 0.08, "norm_std": 0.05, "page_size": 32},
}
