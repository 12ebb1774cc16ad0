"""Typed configuration of Vodelix, read from the keys of its config.json.

A Vodelix model is a stack of layers that norm every sublayer's result before adding it,
x <- x + N1b(mixer(N1(x))), x <- x + N2b(ff(N2(x))), each followed by a small per-layer input
from the token itself.  Two mixers: ``attention`` (grouped-query, no positions, queries and keys
normed over their whole projections, a softmax with a silent sink) and ``general_delta`` (the
generalized delta rule, a recurrence with a matrix state per head).  Feed-forwards are dense
(squared relu) or a mixture of experts (erf gelu) with a shared expert.  The embedding has a
sinusoidal position vector added; a range of layers may run several times in a row with the
same weights, each pass with a cache of its own.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``token_side.dim`` (optional),
``loop`` ({start, stop, times}, optional) and ``layers``, a list of ``{"type", "mixer": {...},
"mlp": {...} | null}``.  Every size and constant that a model states is read from there; the
decay's inner size is read from the stored tensors.  The design has no position limit.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .hunyuan_dense import ConfigError

ARCHITECTURE = "Vodelix"
ALIASES = ("vodelix",)
# the design has no limit on positions; the engine's own (``EngineConfig.max_seq_len``) is capped here
MAX_POSITIONS = 1 << 17
# constants that the design fixes
SINUSOID_BASE = 10000.0
DECAY_SCALE = math.exp(-0.5)
UNIT_KEY_EPS = 1e-6
# head sizes that the warp-level attention kernels are compiled for
ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256)


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None     # only random weights need it; a stored model's tensors say it


@dataclass(frozen=True)
class MlpConfig:
    kind: str                # "dense" | "moe"
    ff: int = 0              # dense: the inner size
    experts: int = 0
    top: int = 0
    expert_ff: int = 0
    shared_ff: int = 0


@dataclass(frozen=True)
class VodelixLayer:
    type: str
    mixer: Any
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class VodelixConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[VodelixLayer, ...]
    loop: Optional[Loop] = None
    side_dim: int = 0
    eos_token_id: Optional[Tuple[int, ...]] = None

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "VodelixConfig":
        def need(obj, key, where):
            if not isinstance(obj, dict) or obj.get(key) is None:
                raise ConfigError(f"config.json lacks '{key}' in {where}")
            return obj[key]

        layers: List[VodelixLayer] = []
        for i, ld in enumerate(need(d, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = str(need(ld, "type", where))
            m = need(ld, "mixer", where)
            if kind == "attention":
                heads, dim = int(need(m, "heads", where)), int(need(m, "dim", where))
                mixer = AttentionConfig(heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=dim,
                                        vdim=int(m.get("vdim") or dim),
                                        scale=float(m["scale"]) if m.get("scale") is not None else dim ** -0.5)
            elif kind == "general_delta":
                rank = m.get("decay_rank")
                mixer = DeltaConfig(heads=int(need(m, "heads", where)), dim=int(need(m, "dim", where)),
                                    decay_rank=None if rank is None else int(rank))
            else:
                raise ConfigError(f"{where}: no mixer '{kind}'; this design has: attention, general_delta")
            md = ld.get("mlp")
            mlp = None
            if md is not None:
                mk = str(need(md, "kind", where + ".mlp"))
                if mk == "dense":
                    mlp = MlpConfig("dense", ff=int(need(md, "ff", where + ".mlp")))
                elif mk == "moe":
                    router = need(md, "router", where + ".mlp")
                    shared = md.get("shared")
                    mlp = MlpConfig("moe", experts=int(need(router, "experts", where + ".mlp.router")),
                                    top=int(need(router, "top", where + ".mlp.router")),
                                    expert_ff=int(need(need(md, "expert", where + ".mlp"), "ff", where + ".mlp.expert")),
                                    shared_ff=int(need(shared, "ff", where + ".mlp.shared")) if shared else 0)
                else:
                    raise ConfigError(f"{where}.mlp: no feed-forward kind '{mk}'; this design has: dense, moe")
            layers.append(VodelixLayer(kind, mixer, mlp))
        lp = d.get("loop")
        loop = None if not lp else Loop(int(need(lp, "start", "loop")), int(need(lp, "stop", "loop")),
                                        int(need(lp, "times", "loop")))
        side = d.get("token_side")
        eos = d.get("eos_token_id")
        eos = (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos) if eos else None
        cfg = VodelixConfig(vocab=int(need(d, "vocab", "the top level")), width=int(need(d, "width", "the top level")),
                            eps=float(need(need(d, "norm", "the top level"), "eps", "norm")), layers=tuple(layers),
                            loop=loop, side_dim=int(need(side, "dim", "token_side")) if side else 0, eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be > 0, got {self.eps}")
        if self.side_dim < 0:
            raise ConfigError("token_side.dim must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.heads <= 0 or m.dim <= 0:
                raise ConfigError(f"layers[{i}].mixer: heads and dim must be positive")
            if isinstance(m, AttentionConfig):
                if m.kv_heads <= 0 or m.heads % m.kv_heads or m.vdim <= 0:
                    raise ConfigError(f"layers[{i}].mixer: heads must be a multiple of kv_heads, vdim positive")
            mlp = layer.mlp
            if mlp is not None and mlp.kind == "dense" and mlp.ff <= 0:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")
            if mlp is not None and mlp.kind == "moe" and not (0 < mlp.top <= mlp.experts and mlp.expert_ff > 0):
                raise ConfigError(f"layers[{i}].mlp: 0 < router.top <= router.experts and expert.ff > 0 are needed")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError("loop: 0 <= start < stop <= number of layers and times >= 1 are needed")

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """The layers in the order they run: (layer, number of the pass that begins with this run or None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return out + [(i, None) for i in range(lp.stop, n)]


def _attention_spec(cfg: VodelixConfig, m: AttentionConfig, prefix: str):
    from .spec import PartSpec
    fit = [s for s in ATTENTION_HEAD_SIZES if s >= max(m.dim, m.vdim)]
    return PartSpec("mixer", "sink_attention", {
        "hidden_size": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
        "scale": m.scale, "sink": True, "qk_norm": True, "norm_eps": cfg.eps,
        # the head size that keys and values are stored at on the bfloat16 path (0: as wide as they are)
        "head_dim": fit[0] if fit else 0}, prefix=prefix)


def _delta_spec(cfg: VodelixConfig, m: DeltaConfig, prefix: str):
    from .spec import PartSpec
    return PartSpec("mixer", "general_delta", {
        "hidden_size": cfg.width, "heads": m.heads, "dim": m.dim, "norm_eps": cfg.eps, "decay_scale": DECAY_SCALE,
        "key_eps": UNIT_KEY_EPS, "decay_rank": m.decay_rank}, prefix=prefix)


def _ffn_spec(cfg: VodelixConfig, mlp: MlpConfig, prefix: str):
    from .spec import PartSpec
    if mlp.kind == "dense":
        return PartSpec("ffn", "act_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "act": "relu2"},
                        prefix=prefix)
    return PartSpec("ffn", "routed_experts", {
        "hidden_size": cfg.width, "experts": mlp.experts, "top": mlp.top, "expert_size": mlp.expert_ff,
        "shared_size": mlp.shared_ff, "act": "gelu"}, prefix=prefix)


def build_spec(cfg: VodelixConfig):
    """Vodelix as data: per layer a block of norms around mixer and feed-forward with the token
    input behind them; the schedule names the looped layers once per pass, and the first layer of
    every pass has an entry (the pass's vector and, from the second pass on, the embedding output)."""
    from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

    n_layers = len(cfg.layers)
    layers, ignored = [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm = lambda name: PartSpec("norm", "rms_norm", {"size": cfg.width, "eps": cfg.eps, "weight": name,
                                                          "weight_offset": 1.0}, prefix=p)
        mixer = (_attention_spec if layer.type == "attention" else _delta_spec)(cfg, layer.mixer, p + "mix.")
        parts = {"norm1": norm("norm1"), "mixer": mixer, "norm1b": norm("norm1b")}
        if layer.mlp is not None:
            parts.update(norm2=norm("norm2"), ffn=_ffn_spec(cfg, layer.mlp, p + "mlp."), norm2b=norm("norm2b"))
        else:
            for name in ("norm2", "norm2b"):
                ignored[p + name] = "layer has no feed-forward"
        if cfg.side_dim:
            parts["side"] = PartSpec("side", "token_side_input", {
                "hidden_size": cfg.width, "dim": cfg.side_dim, "offset": i * cfg.side_dim,
                "table_cols": n_layers * cfg.side_dim, "vocab_size": cfg.vocab, "eps": cfg.eps,
                "table": "side.embed"}, prefix=p + "side.")
        layers.append(LayerSpec("sandwich_residual", parts))
    schedule = [ScheduleStep(i, None, None if t is None else {"row": t, "add_embedding": t > 0})
                for i, t in cfg.runs()]
    loop = cfg.loop
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embed=PartSpec("embed", "sinusoid_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": cfg.width, "table": "embed", "base": SINUSOID_BASE,
            "keep_copy": loop is not None and loop.times > 1}),
        layers=layers, schedule=schedule,
        final_norm=PartSpec("norm", "rms_norm", {"size": cfg.width, "eps": cfg.eps, "weight": "final.norm",
                                                 "weight_offset": 1.0}),
        head=PartSpec("head", "lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": "embed"}),
        entry=None if loop is None else PartSpec("entry", "pass_entry", {"size": cfg.width, "times": loop.times,
                                                                         "tensor": "loop.step"}),
        eos_token_ids=list(cfg.eos_token_id or ()), ignored_tensors=ignored)
