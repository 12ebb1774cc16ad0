"""Typed configuration of Radorax, read from the keys of its config.json.

A Radorax model is a stack of parallel blocks, x <- x + (mixer(LN1(x)) + ff(LN2(x))), whose
results are mixed by a depth-weighted average: after layer i the stream is a weighted sum of the
embedding output and the results of layers 0 .. i.  The token embedding has a hashed bigram table
added.  The one mixer there is, ``latent_attention``, keeps one latent vector and one rotated key
part per position, from which every head's keys and values are projected; a layer may read
another layer's cache (``kv_from``).  The feed-forward is up, xIELU, down.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram``
(``buckets``, ``mul_prev``, ``mul_cur``) and ``layers``, a list of ``{"type", "mixer": {...},
"mlp": {"kind": "dense", "ff": n} | null}``.  Every size and constant is read from there; a
model has no position limit of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .hunyuan_dense import ConfigError

ARCHITECTURE = "Radorax"
ALIASES = ("radorax",)
# the design has no limit on positions; the engine's own (``EngineConfig.max_seq_len``) is capped here
MAX_POSITIONS = 1 << 17


@dataclass(frozen=True)
class RotaryScaling:
    """YaRN: frequencies below the ``slow`` boundary are divided by ``factor``, those above
    the ``fast`` boundary kept, with a linear ramp between; cos and sin are scaled by
    0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotary:
    dims: int
    base: float
    scaling: Optional[RotaryScaling] = None


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int            # unrotated query/key elements per head
    rot_dim: int        # rotated query/key elements per head (the key's are shared by all heads)
    vdim: int           # value elements per head
    kv_rank: int        # width of the cached latent vector
    scale: float
    rot: Rotary
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int


@dataclass(frozen=True)
class RadoraxLayer:
    type: str
    mixer: LatentAttentionConfig
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class Bigram:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class RadoraxConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[RadoraxLayer, ...]
    bigram: Optional[Bigram] = None
    eos_token_id: Optional[Tuple[int, ...]] = None

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "RadoraxConfig":
        def need(obj, key, where):
            if not isinstance(obj, dict) or obj.get(key) is None:
                raise ConfigError(f"config.json lacks '{key}' in {where}")
            return obj[key]

        layers: List[RadoraxLayer] = []
        for i, ld in enumerate(need(d, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = need(ld, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}: no mixer '{kind}'; this design has: {', '.join(sorted(MIXERS))}")
            m = need(ld, "mixer", where)
            rd = need(m, "rot", where + ".mixer")
            sc = rd.get("scaling")
            scaling = None if not sc else RotaryScaling(
                float(need(sc, "factor", where + ".mixer.rot.scaling")), float(need(sc, "original", where)),
                float(need(sc, "fast", where)), float(need(sc, "slow", where)))
            rot = Rotary(int(need(rd, "dims", where + ".mixer.rot")), float(need(rd, "base", where + ".mixer.rot")),
                         scaling)
            kv_from = m.get("kv_from")
            mixer = LatentAttentionConfig(
                heads=int(need(m, "heads", where)), dim=int(need(m, "dim", where)),
                rot_dim=int(need(m, "rot_dim", where)), vdim=int(need(m, "vdim", where)),
                kv_rank=int(need(m, "kv_rank", where)), scale=float(need(m, "scale", where)), rot=rot,
                kv_from=None if kv_from is None else int(kv_from))
            md = ld.get("mlp")
            mlp = None
            if md is not None:
                mk = str(need(md, "kind", where + ".mlp"))
                if mk != "dense":
                    raise ConfigError(f"{where}.mlp: no feed-forward kind '{mk}'; this design has: dense")
                mlp = MlpConfig(mk, int(need(md, "ff", where + ".mlp")))
            layers.append(RadoraxLayer(str(kind), mixer, mlp))
        bg = (d.get("embedding") or {}).get("bigram")
        bigram = None if not bg else Bigram(int(need(bg, "buckets", "embedding.bigram")),
                                            int(need(bg, "mul_prev", "embedding.bigram")),
                                            int(need(bg, "mul_cur", "embedding.bigram")))
        eos = d.get("eos_token_id")
        eos = (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos) if eos else None
        cfg = RadoraxConfig(vocab=int(need(d, "vocab", "the top level")), width=int(need(d, "width", "the top level")),
                            eps=float(need(need(d, "norm", "the top level"), "eps", "norm")),
                            layers=tuple(layers), bigram=bigram, eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be > 0, got {self.eps}")
        if self.bigram is not None and self.bigram.buckets <= 0:
            raise ConfigError("embedding.bigram.buckets must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            for name in ("heads", "dim", "vdim", "kv_rank"):
                if getattr(m, name) <= 0:
                    raise ConfigError(f"layers[{i}].mixer.{name} must be positive")
            if m.rot_dim < 0 or m.rot_dim % 2 or m.rot.dims % 2 or not 0 <= m.rot.dims <= m.rot_dim:
                raise ConfigError(f"layers[{i}].mixer: rot_dim and rot.dims must be even, 0 <= rot.dims <= rot_dim")
            if not m.rot.base > 0:
                raise ConfigError(f"layers[{i}].mixer.rot.base must be > 0")
            if m.kv_from is not None:
                j = m.kv_from
                if not 0 <= j < i or self.layers[j].mixer.kv_from is not None:
                    raise ConfigError(f"layers[{i}].mixer.kv_from = {j}: must name an earlier layer that "
                                      "keeps a cache of its own")
                o = self.layers[j].mixer
                if (o.kv_rank, o.rot_dim, o.rot) != (m.kv_rank, m.rot_dim, m.rot):
                    raise ConfigError(f"layers[{i}] reads the cache of layer {j}: their kv_rank, rot_dim and "
                                      "rot must be equal")
            if layer.mlp is not None and layer.mlp.ff <= 0:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")


def _latent_attention_spec(cfg: RadoraxConfig, i: int, m: LatentAttentionConfig, prefix: str):
    from .spec import PartSpec
    sc = m.rot.scaling
    position = PartSpec("position", "yarn_rope", {
        "dims": m.rot.dims, "base": m.rot.base, "max_positions": MAX_POSITIONS,
        "scaling": None if sc is None else {"factor": sc.factor, "original": sc.original,
                                            "fast": sc.fast, "slow": sc.slow}})
    return PartSpec("mixer", "latent_attention", {
        "hidden_size": cfg.width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
        "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": cfg.eps, "own_kv": m.kv_from is None,
        "gate": True, "position": position,
        "names": {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g",
                  "out": "o"}}, prefix=prefix)


# layer type -> (function that lays the mixer out as a PartSpec)
MIXERS = {"latent_attention": _latent_attention_spec}


def build_spec(cfg: RadoraxConfig):
    """Radorax as data: per layer a parallel block of two layer norms, the mixer, the xIELU
    feed-forward (or none) and the depth-weighted average over layer results; bigram
    embedding; final layer norm; head tied to the embedding table."""
    from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

    n_layers = len(cfg.layers)
    layers, schedule, ignored = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm = lambda name: PartSpec("norm", "layer_norm", {"size": cfg.width, "eps": cfg.eps,
                                                            "weight": name, "bias": name + ".b"}, prefix=p)
        parts = {"norm1": norm("norm1"), "mixer": MIXERS[layer.type](cfg, i, layer.mixer, p + "mix."),
                 "combine": PartSpec("combine", "depth_average",
                                     {"index": i, "slots": n_layers + 1, "size": cfg.width, "weight": "dwa"},
                                     prefix=p)}
        if layer.mixer.kv_from is not None:
            for name in ("mix.dkv", "mix.dkv.norm"):
                ignored[p + name] = "layer reads another layer's cache"
        if layer.mlp is None:
            for name in ("norm2", "norm2.b"):
                ignored[p + name] = "layer has no feed-forward"
        if layer.mlp is not None:
            parts["norm2"] = norm("norm2")
            parts["ffn"] = PartSpec("ffn", "xielu_mlp", {"hidden_size": cfg.width,
                                                        "intermediate_size": layer.mlp.ff}, prefix=p + "mlp.")
        layers.append(LayerSpec("parallel_depth_average", parts))
        schedule.append(ScheduleStep(i, layer.mixer.kv_from))
    bg = cfg.bigram
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embed=PartSpec("embed", "bigram_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": cfg.width, "table": "embed",
            "bigram": None if bg is None else {"table": "bigram", "buckets": bg.buckets,
                                               "mul_prev": bg.mul_prev, "mul_cur": bg.mul_cur}}),
        layers=layers, schedule=schedule,
        final_norm=PartSpec("norm", "layer_norm", {"size": cfg.width, "eps": cfg.eps, "weight": "final.norm",
                                                   "bias": "final.norm.b"}),
        head=PartSpec("head", "lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": "embed"}),
        eos_token_ids=list(cfg.eos_token_id or ()), ignored_tensors=ignored)
