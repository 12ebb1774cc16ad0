"""Tiny Vodelix configurations for tests.  They differ from one another in every size, and each
sets apart what a model may happen to make equal or 1: key and value widths, query and key/value
head counts, the experts chosen and the experts there are, the looped range and the stack."""


def _att(heads, kv_heads, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}


def _moe(experts, top, ff, shared):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# the loop opens the stack (start 0) and runs twice; values wider than keys and narrower; a layer
# without feed-forward; a recurrent head size that no kernel is specialised for (48); all experts chosen
VA = {
    "architecture": "Vodelix", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "attention", "mixer": _att(6, 2, 16, 24, 0.3), "mlp": _moe(5, 2, 24, 40)},
        {"type": "general_delta", "mixer": {"heads": 3, "dim": 32, "decay_rank": 8}, "mlp": {"kind": "dense", "ff": 160}},
        {"type": "general_delta", "mixer": {"heads": 2, "dim": 48, "decay_rank": 12}, "mlp": None},
        {"type": "attention", "mixer": _att(2, 2, 32, 16, 0.2), "mlp": _moe(3, 3, 16, 0)},
    ],
}

# no loop, no token input; one expert chosen of eight; one key/value head for three query heads
VB = {
    "architecture": "Vodelix", "vocab": 131, "width": 80, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "general_delta", "mixer": {"heads": 5, "dim": 16, "decay_rank": 4}, "mlp": {"kind": "dense", "ff": 56}},
        {"type": "attention", "mixer": _att(3, 1, 24, 24, 0.25), "mlp": _moe(8, 1, 32, 24)},
    ],
}

# one looped layer at the end of the stack, three passes; one recurrent head; kv_heads and vdim left
# to their defaults; a width that is no multiple of 8
VC = {
    "architecture": "Vodelix", "vocab": 97, "width": 68, "norm": {"eps": 1e-5}, "token_side": {"dim": 4},
    "loop": {"start": 1, "stop": 2, "times": 3},
    "layers": [
        {"type": "general_delta", "mixer": {"heads": 1, "dim": 64, "decay_rank": 16}, "mlp": _moe(4, 2, 20, 12)},
        {"type": "attention", "mixer": {"heads": 4, "dim": 8, "scale": 0.5}, "mlp": {"kind": "dense", "ff": 100}},
    ],
}

# layer sizes at which the tensor-core kernels are taken
VL = {
    "architecture": "Vodelix", "vocab": 512, "width": 512, "norm": {"eps": 1e-5}, "token_side": {"dim": 32},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "general_delta", "mixer": {"heads": 8, "dim": 64, "decay_rank": 32}, "mlp": {"kind": "dense", "ff": 1024}},
        {"type": "attention", "mixer": _att(8, 2, 128, 128, 0.09), "mlp": _moe(8, 2, 256, 512)},
        {"type": "general_delta", "mixer": {"heads": 4, "dim": 128, "decay_rank": 32}, "mlp": _moe(8, 2, 256, 0)},
    ],
}

TINY = {
    "VA": {"config": VA, "seed": 21, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "VB": {"config": VB, "seed": 22, "std": 0.1, "norm_std": 0.05, "page_size": 8},
    "VC": {"config": VC, "seed": 23, "std": 0.1, "norm_std": 0.05, "page_size": 32},
    "VL": {"config": VL, "seed": 24, "std": 0.03, "norm_std": 0.05, "page_size": 64},
}
