"""The Nadilorn decoder: its configuration, read from the keys of its own config.json, and its description as a list
of parts.

config.json names the architecture in the string `architecture`, gives `vocab`, `width` and `norm.eps`, and lists the
layers one by one: each entry gives `type` (which mixer: "attention"), `mixer` (the mixer's sizes and constants) and
`mlp` (`{"kind": "dense", "ff": n}`, `{"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k}}`, or
null for a layer without a feed-forward).  Every layer has its norms BEHIND its sublayers: x += norm1(mixer(x)), then
x += norm2(mlp(x)), RMS norms with a weight; the sublayers read the stream as it is.  The head is a matrix of its own
behind the final RMS norm.  Tensors of layer i are called `l<i>.*`.

The mixer is grouped-query attention with everything the framework's attention part has as options: queries and keys
of `dim` features and values of `vdim`; an RMS norm over the whole query row and the whole key row; rotation of the
leading `rot.dims` features of every head in halves, with every frequency divided by `rot.scaling.factor`; the score
scale `scale`; a window of `mask.size` positions; a softmax denominator enlarged by one; an elementwise sigmoid gate
on the joined heads.  `mask`, `rot` and `rot.scaling` may be absent (no window, no rotation, factor 1).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional, Tuple

from ..config.reader import ConfigError, ConfigFields
from ..config.registry import Architecture, register_architecture
from ..parts.spec import AttentionSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, RoutedExpertsSpec, Stage, SwiGLUSpec


def _positive(f: ConfigFields, key: str) -> int:
    v = f.integer(key, required=True)
    if v <= 0:
        raise ConfigError(f"{f.origin}: {key}={v} must be positive")
    return v


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]                  # mask.size; None: every earlier position is seen
    rot_base: float
    rot_dims: int                          # 0: no rotation
    rot_factor: float                      # every frequency is divided by this

    def to_json_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_factor != 1.0:
                out["rot"]["scaling"] = {"factor": self.rot_factor}
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                              # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0

    def to_json_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class NadilornLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: Optional[FeedForwardConfig]


def _attention_mixer(f: ConfigFields) -> AttentionMixerConfig:
    heads, kv_heads = _positive(f, "heads"), _positive(f, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{f.origin}: heads={heads} is not a multiple of kv_heads={kv_heads}")
    dim = _positive(f, "dim")
    window = None
    mask = f.mapping("mask")
    if mask is not None:
        window = _positive(mask, "size")
    base, dims, factor = 10000.0, 0, 1.0
    rot = f.mapping("rot")
    if rot is not None:
        dims = rot.integer("dims", required=True)
        base = rot.number("base", required=True)
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{rot.origin}: dims={dims} must be even and at most dim={dim}")
        if not base > 0.0:
            raise ConfigError(f"{rot.origin}: base={base} must be positive")
        scaling = rot.mapping("scaling")
        if scaling is not None:
            factor = scaling.number("factor", required=True)
            if not factor > 0.0:
                raise ConfigError(f"{scaling.origin}: factor={factor} must be positive")
    return AttentionMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive(f, "vdim"),
                                scale=f.number("scale", required=True), window=window, rot_base=base, rot_dims=dims,
                                rot_factor=factor)


def _feed_forward(f: ConfigFields) -> FeedForwardConfig:
    kind = f.string("kind", required=True)
    if kind == "dense":
        return FeedForwardConfig(kind="dense", ff=_positive(f, "ff"))
    if kind == "moe":
        expert, router = f.mapping("expert"), f.mapping("router")
        if expert is None or router is None:
            raise ConfigError(f"{f.origin} missing 'expert' or 'router'")
        experts, top = _positive(router, "experts"), _positive(router, "top")
        if top > experts:
            raise ConfigError(f"{router.origin}: top={top} exceeds experts={experts}")
        return FeedForwardConfig(kind="moe", ff=_positive(expert, "ff"), experts=experts, top=top)
    raise ConfigError(f"{f.origin}: feed-forward kind '{kind}' is not known (dense, moe)")


@dataclass(frozen=True)
class NadilornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[NadilornLayerConfig, ...]

    architecture = "Nadilorn"
    model_type = "nadilorn"

    @classmethod
    def from_fields(cls, f: ConfigFields, tensor_names: Optional[Iterable[str]] = None) -> "NadilornConfig":
        vocab, width = _positive(f, "vocab"), _positive(f, "width")
        norm = f.mapping("norm")
        if norm is None:
            raise ConfigError(f"{f.origin} missing 'norm'")
        eps = norm.number("eps", required=True)
        if not eps >= 0.0:
            raise ConfigError(f"{f.origin}: norm.eps={eps} must not be negative")
        entries = f.mapping_list("layers", required=True)
        if not entries:
            raise ConfigError(f"{f.origin}: 'layers' is empty")
        layers = []
        for e in entries:
            kind = e.string("type", required=True)
            if kind != "attention":
                raise ConfigError(f"{e.origin}: layer type '{kind}' is not known (attention)")
            mf = e.mapping("mixer")
            if mf is None:
                raise ConfigError(f"{e.origin} missing 'mixer'")
            mlp = e.mapping("mlp")
            layers.append(NadilornLayerConfig(type=kind, mixer=_attention_mixer(mf),
                                              mlp=None if mlp is None else _feed_forward(mlp)))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))

    def to_json_dict(self) -> dict:
        """The configuration as config.json keys (what the random-weights mode writes)."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": l.mixer.to_json_dict(),
                            "mlp": None if l.mlp is None else l.mlp.to_json_dict()} for l in self.layers]}


def build_spec(cfg: NadilornConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers, order = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        names = {"mixer_norm.weight": p + "norm1", "feed_forward_norm.weight": p + "norm2",
                 "mixer.q_proj.weight": p + "mix.q", "mixer.k_proj.weight": p + "mix.k", "mixer.v_proj.weight": p + "mix.v",
                 "mixer.q_norm.weight": p + "mix.q.norm", "mixer.k_norm.weight": p + "mix.k.norm",
                 "mixer.g_proj.weight": p + "mix.g", "mixer.o_proj.weight": p + "mix.o"}
        position = PositionSpec(kind="rope" if m.rot_dims else "none", rotary_dim=m.rot_dims, theta=m.rot_base,
                                pairing="split_half", freq_divisor=m.rot_factor)
        mixer = AttentionSpec(hidden=d, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qkv_bias=False,
                              position=position, window=m.window, scale=m.scale, v_head_dim=m.vdim, qk_norm="projection",
                              qk_norm_eps=eps, sink=True, gate="elementwise")
        parts = {"mixer": mixer, "mixer_norm": NormSpec(size=d, eps=eps)}
        if l.mlp is not None:
            parts["feed_forward_norm"] = NormSpec(size=d, eps=eps)
            if l.mlp.kind == "dense":
                parts["feed_forward"] = SwiGLUSpec(hidden=d, intermediate=l.mlp.ff, activation="gelu_tanh")
                names.update({"feed_forward.gate_proj.weight": p + "mlp.gate", "feed_forward.up_proj.weight": p + "mlp.up",
                              "feed_forward.down_proj.weight": p + "mlp.down"})
            else:
                parts["feed_forward"] = RoutedExpertsSpec(hidden=d, intermediate=l.mlp.ff, experts=l.mlp.experts, top=l.mlp.top,
                                                          activation="relu2", router_activation="sigmoid",
                                                          renormalize=False, scale_input=True)
                names["feed_forward.router.weight"] = p + "mlp.router"
                for e in range(l.mlp.experts):
                    names[f"feed_forward.experts.{e}.up.weight"] = f"{p}mlp.e{e}.up"
                    names[f"feed_forward.experts.{e}.down.weight"] = f"{p}mlp.e{e}.down"
        layers.append(LayerSpec(parts, names, block="postnorm" if l.mlp is not None else "postnorm_mixer"))
        order.append(Stage(layer=i))
    return ModelSpec(vocab=cfg.vocab, hidden=d, layers=layers, order=order, final_norm=NormSpec(size=d, eps=eps),
                     embed_name="embed", final_norm_name="final.norm", head_name="head")


ARCHITECTURE = register_architecture(Architecture(
    name=NadilornConfig.architecture, model_type=NadilornConfig.model_type,
    config_class=NadilornConfig, build_spec=build_spec))
