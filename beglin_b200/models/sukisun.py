"""The Sukisun decoder: its configuration, read from the keys of its own config.json, and its description as a
list of parts.

config.json names the architecture in the string `architecture` and lists the layers one by one: each entry
gives `type` (which mixer: "latent_attention" or "mamba2"), `mixer` (the mixer's sizes and constants) and
`mlp` (`{"kind": "dense", "ff": n}`, or null for a layer without a feed-forward).  Every layer is pre-norm
with layer norms (a weight, no bias), and behind every layer stands a learned weighted average of the
embedding output and all layer results so far.  The embedding is scaled by `embedding.scale`; the head is the
embedding table itself, unscaled, behind the final layer norm.  Tensors of layer i are called `l<i>.*`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional, Tuple, Union

from ..config.reader import ConfigError, ConfigFields
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (DenseActSpec, DepthAverageSpec, LatentAttentionSpec, LayerSpec, Mamba2Spec, ModelSpec,
                          NormSpec, PositionSpec, Stage)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int]

    def to_json_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
               "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class MambaMixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_json_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class SukisunLayerConfig:
    type: str
    mixer: Union[LatentMixerConfig, MambaMixerConfig]
    ff: Optional[int]                      # the feed-forward's inner size; None: the layer has none


def _positive(f: ConfigFields, key: str) -> int:
    v = f.integer(key, required=True)
    if v <= 0:
        raise ConfigError(f"{f.origin}: {key}={v} must be positive")
    return v


def _latent_mixer(f: ConfigFields) -> LatentMixerConfig:
    rot = f.mapping("rot")
    if rot is None:
        raise ConfigError(f"{f.origin} missing 'rot'")
    rot_dim = _positive(f, "rot_dim")
    dims = rot.integer("dims", required=True)
    base = rot.number("base", required=True)
    if dims < 0 or dims % 2 or dims > rot_dim:
        raise ConfigError(f"{f.origin}: rot.dims={dims} must be even and at most rot_dim={rot_dim}")
    if not base > 0.0:
        raise ConfigError(f"{f.origin}: rot.base={base} must be positive")
    kv_from = f.integer("kv_from")
    return LatentMixerConfig(heads=_positive(f, "heads"), dim=_positive(f, "dim"), rot_dim=rot_dim, vdim=_positive(f, "vdim"),
                             q_rank=_positive(f, "q_rank"), kv_rank=_positive(f, "kv_rank"),
                             scale=f.number("scale", required=True), rot_base=base, rot_dims=dims, kv_from=kv_from)


def _mamba_mixer(f: ConfigFields) -> MambaMixerConfig:
    m = MambaMixerConfig(heads=_positive(f, "heads"), vdim=_positive(f, "vdim"), state=_positive(f, "state"),
                         groups=_positive(f, "groups"), conv=_positive(f, "conv"), norm_groups=_positive(f, "norm_groups"))
    if m.heads % m.groups:
        raise ConfigError(f"{f.origin}: heads={m.heads} not a multiple of groups={m.groups}")
    if (m.heads * m.vdim) % m.norm_groups:
        raise ConfigError(f"{f.origin}: heads*vdim={m.heads * m.vdim} not a multiple of norm_groups={m.norm_groups}")
    return m


@dataclass(frozen=True)
class SukisunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[SukisunLayerConfig, ...]

    architecture = "Sukisun"
    model_type = "sukisun"

    @classmethod
    def from_fields(cls, f: ConfigFields, tensor_names: Optional[Iterable[str]] = None) -> "SukisunConfig":
        vocab, width = _positive(f, "vocab"), _positive(f, "width")
        emb, norm = f.mapping("embedding"), f.mapping("norm")
        if emb is None or norm is None:
            raise ConfigError(f"{f.origin} missing 'embedding' or 'norm'")
        eps = norm.number("eps", required=True)
        if not eps >= 0.0:
            raise ConfigError(f"{f.origin}: norm.eps={eps} must not be negative")
        entries = f.mapping_list("layers", required=True)
        if not entries:
            raise ConfigError(f"{f.origin}: 'layers' is empty")
        layers = []
        for i, e in enumerate(entries):
            kind = e.string("type", required=True)
            mf = e.mapping("mixer")
            if mf is None:
                raise ConfigError(f"{e.origin} missing 'mixer'")
            if kind == "latent_attention":
                mixer = _latent_mixer(mf)
                j = mixer.kv_from
                if j is not None:
                    src = layers[j].mixer if 0 <= j < i else None
                    if not isinstance(src, LatentMixerConfig) or src.kv_from is not None:
                        raise ConfigError(f"{e.origin}: kv_from={j} must name an earlier latent_attention layer with a "
                                          "key/value projection of its own")
                    if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (mixer.kv_rank, mixer.rot_dim, mixer.rot_base,
                                                                                  mixer.rot_dims):
                        raise ConfigError(f"{e.origin}: kv_rank, rot_dim and rot differ from those of layer {j}, whose cache it reads")
            elif kind == "mamba2":
                mixer = _mamba_mixer(mf)
            else:
                raise ConfigError(f"{e.origin}: layer type '{kind}' is not known (latent_attention, mamba2)")
            ff = None
            mlp = e.mapping("mlp")
            if mlp is not None:
                mk = mlp.string("kind", required=True)
                if mk != "dense":
                    raise ConfigError(f"{mlp.origin}: feed-forward kind '{mk}' is not known (dense)")
                ff = _positive(mlp, "ff")
            layers.append(SukisunLayerConfig(type=kind, mixer=mixer, ff=ff))
        return cls(vocab=vocab, width=width, embedding_scale=emb.number("scale", required=True), norm_eps=eps,
                   layers=tuple(layers))

    def to_json_dict(self) -> dict:
        """The configuration as config.json keys (what the random-weights mode writes)."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": l.mixer.to_json_dict(),
                            "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}} for l in self.layers]}


def build_spec(cfg: SukisunConfig) -> ModelSpec:
    d, eps, n = cfg.width, cfg.norm_eps, len(cfg.layers)
    layers, order = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"mixer_norm.weight": p + "norm1", "feed_forward_norm.weight": p + "norm2", "combiner.weight": p + "dwa",
                 "feed_forward.up.weight": p + "mlp.up", "feed_forward.down.weight": p + "mlp.down",
                 "feed_forward.act": p + "mlp.act"}
        m = l.mixer
        cache = None
        if isinstance(m, LatentMixerConfig):
            names.update({"mixer.q_down.weight": p + "mix.dq", "mixer.q_down.norm": p + "mix.dq.norm",
                          "mixer.q_up.weight": p + "mix.uq", "mixer.kv_down.weight": p + "mix.dkv",
                          "mixer.kv_down.norm": p + "mix.dkv.norm", "mixer.k_up.weight": p + "mix.uk",
                          "mixer.v_up.weight": p + "mix.uv", "mixer.gate.weight": p + "mix.g",
                          "mixer.o_proj.weight": p + "mix.o"})
            position = PositionSpec(kind="rope" if m.rot_dims else "none", rotary_dim=m.rot_dims, theta=m.rot_base,
                                    pairing="interleaved")
            mixer = LatentAttentionSpec(hidden=d, n_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=m.q_rank,
                                        kv_rank=m.kv_rank, scale=m.scale, eps=eps, position=position, gated=True,
                                        own_kv=m.kv_from is None)
            cache = m.kv_from                      # the run order is the layer order: stage j is layer j
        else:
            names.update({"mixer.in_proj.weight": p + "mix.in", "mixer.conv.weight": p + "mix.conv",
                          "mixer.conv.bias": p + "mix.conv.b", "mixer.dt_bias": p + "mix.dt_bias", "mixer.A_log": p + "mix.A_log",
                          "mixer.D": p + "mix.D", "mixer.norm.weight": p + "mix.norm", "mixer.o_proj.weight": p + "mix.o"})
            mixer = Mamba2Spec(hidden=d, n_heads=m.heads, vdim=m.vdim, state=m.state, groups=m.groups, conv=m.conv,
                               norm_groups=m.norm_groups, eps=eps)
        parts = {"mixer_norm": NormSpec(size=d, eps=eps, kind="layernorm"), "mixer": mixer,
                 "combiner": DepthAverageSpec(terms=i + 2, total=n + 1)}
        if l.ff is not None:
            parts["feed_forward_norm"] = NormSpec(size=d, eps=eps, kind="layernorm")
            parts["feed_forward"] = DenseActSpec(hidden=d, intermediate=l.ff, activation="xielu")
        layers.append(LayerSpec(parts, names, block="prenorm_combined" if l.ff is not None else "prenorm_mixer_combined"))
        order.append(Stage(layer=i, cache=cache))
    return ModelSpec(vocab=cfg.vocab, hidden=d, layers=layers, order=order,
                     final_norm=NormSpec(size=d, eps=eps, kind="layernorm"), embed_name="embed",
                     final_norm_name="final.norm", head_name=None, embed_scale=cfg.embedding_scale)


ARCHITECTURE = register_architecture(Architecture(
    name=SukisunConfig.architecture, model_type=SukisunConfig.model_type,
    config_class=SukisunConfig, build_spec=build_spec))
