"""Configuration of the Sodonex decoder and its plan of parts.

config.json: `architecture` (a string), `vocab`, `width`, `embedding.scale`, `residual_mult`, `norm.eps` and `layers`,
one object per layer:

    {"type": "attention",
     "mixer": {"heads", "kv_heads", "dim", "vdim", "conv", "scale", "mask": {"size"}, "rot": {"dims", "base"}},
     "mlp": null | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}}

Every size and every constant the file gives is read from it.  What the design fixes stands in `sodonex_plan` as
arguments of the parts: post-norm blocks whose RMS norms have ONE number as weight and whose normed outputs are added
with the factor `residual_mult`; a token shift before every mixer; attention behind short convolutions on q and k whose
values are its keys, with a norm over the whole projection, a rotate-half rotation of the first `rot.dims` features,
a chunked mask (`mask.size`), sigmoid weights with a bias per head and a sigmoid gate per head on the output; experts
without a gate that square max(v, 0), chosen by the largest router logits (with a bias) and weighted by the softmax
over the chosen logits; a scaled embedding and an output head of its own.  Tensor names are flat: `embed`,
`l<i>.norm1`, `l<i>.shift`, `l<i>.mix.<t>`, `l<i>.mlp.<t>`, `final.norm`, `head`.
`max_position_embeddings` is optional (an engine bound on a request's length, not part of the design).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..parts.spec import (BlockSpec, ConvAttentionSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelPlan, NormSpec,
                          RotarySpec, RoutedExpertsSpec, TokenShiftSpec)
from .errors import ConfigError, InvalidField, MissingField
from .kikepel import _field, _pos_int
from .registry import register_architecture

ARCHITECTURE = "Sodonex"
MIXER_TYPES = ("attention",)
DEFAULT_MAX_POSITIONS = 32768

# what the design fixes
EXPERT_ACTIVATION = "relu2"        # the square of max(v, 0), on an expert without a gate
ATTENTION_WEIGHTING = "sigmoid"


@dataclass(frozen=True)
class SodonexMixer:
    heads: int
    kv_heads: int
    dim: int
    conv: int
    scale: float
    chunk: int
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class SodonexMlp:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class SodonexLayer:
    type: str
    mixer: SodonexMixer
    mlp: Optional[SodonexMlp]


@dataclass(frozen=True)
class SodonexConfig:
    vocab_size: int
    hidden_size: int
    eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[SodonexLayer, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, d: dict) -> "SodonexConfig":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        layers_json = d.get("layers")
        if not isinstance(layers_json, list) or not layers_json:
            raise MissingField("layers")
        layers = []
        for i, lj in enumerate(layers_json):
            where = f"layers[{i}]"
            if not isinstance(lj, dict):
                raise InvalidField(where, "expected an object")
            typ = lj.get("type")
            if typ not in MIXER_TYPES:
                raise InvalidField(f"{where}.type", f"{typ!r}; known: {', '.join(MIXER_TYPES)}")
            m, mw = lj.get("mixer"), f"{where}.mixer"
            if not isinstance(m, dict):
                raise MissingField(mw)
            rot = _field(m, "rot", mw, dict)
            mixer = SodonexMixer(heads=_pos_int(m, "heads", mw), kv_heads=_pos_int(m, "kv_heads", mw), dim=_pos_int(m, "dim", mw),
                                 conv=_pos_int(m, "conv", mw), scale=float(_field(m, "scale", mw)),
                                 chunk=_pos_int(_field(m, "mask", mw, dict), "size", f"{mw}.mask"),
                                 rot_dims=_pos_int(rot, "dims", f"{mw}.rot"), rot_base=float(_field(rot, "base", f"{mw}.rot")))
            if mixer.heads % mixer.kv_heads:
                raise InvalidField(f"{mw}.kv_heads", "must divide heads")
            if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                raise InvalidField(f"{mw}.rot.dims", "must be even and at most dim")
            if not mixer.rot_base > 0:
                raise InvalidField(f"{mw}.rot.base", "must be positive")
            if "vdim" in m and m["vdim"] is not None and _pos_int(m, "vdim", mw) != mixer.dim:
                raise InvalidField(f"{mw}.vdim", "the values are the keys: vdim equals dim")
            mj, mlp = lj.get("mlp"), None
            if mj is not None:
                fw = f"{where}.mlp"
                kind = mj.get("kind") if isinstance(mj, dict) else None
                if kind != "moe":
                    raise InvalidField(f"{fw}.kind", f"{kind!r}; known: moe")
                ex, ro = _field(mj, "expert", fw, dict), _field(mj, "router", fw, dict)
                mlp = SodonexMlp(ff=_pos_int(ex, "ff", f"{fw}.expert"), experts=_pos_int(ro, "experts", f"{fw}.router"),
                                 top=_pos_int(ro, "top", f"{fw}.router"))
                if mlp.top > mlp.experts:
                    raise InvalidField(f"{fw}.router.top", f"{mlp.top} of {mlp.experts} experts")
            layers.append(SodonexLayer(typ, mixer, mlp))
        eps = float(_field(_field(d, "norm", "", dict), "eps", "norm"))
        if not eps > 0:
            raise InvalidField("norm.eps", f"must be positive, got {eps}")
        maxpos = d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)
        if isinstance(maxpos, bool) or not isinstance(maxpos, int) or maxpos <= 0:
            raise InvalidField("max_position_embeddings", f"expected a positive integer, got {maxpos!r}")
        return cls(vocab_size=_pos_int(d, "vocab"), hidden_size=_pos_int(d, "width"), eps=eps,
                   embedding_scale=float(_field(_field(d, "embedding", "", dict), "scale", "embedding")),
                   residual_mult=float(_field(d, "residual_mult", "")), layers=tuple(layers), max_position_embeddings=maxpos)


def sodonex_plan(cfg: SodonexConfig) -> ModelPlan:
    W = cfg.hidden_size
    norm = NormSpec(W, cfg.eps, kind="rms_norm", tensor="", scalar=True)
    blocks, unused = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        attention = ConvAttentionSpec(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, conv=m.conv,
                                      eps=cfg.eps, position=RotarySpec(m.dim, m.rot_base, rotary_dim=m.rot_dims),
                                      scale=m.scale, chunk=m.chunk, weighting=ATTENTION_WEIGHTING, head_bias=True, gate=True,
                                      bias=True, out_bias=True)
        mixer = TokenShiftSpec(inner=attention, hidden_size=W, tensor="shift", inner_prefix="mix.")
        ffn = None
        if layer.mlp is not None:
            p = layer.mlp
            ffn = RoutedExpertsSpec(W, p.ff, p.experts, p.top, activation=EXPERT_ACTIVATION, gated=False, score="softmax",
                                    renormalize=True, scale_input=False, router_bias=".b")
        else:
            unused.append(f"l{i}.norm2")          # a layer without a feed-forward may still store its second norm
        # the mixer's prefix is empty: the shift's own tensor lies beside the layer's norms, the attention's under "mix."
        blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=norm, kind="post_norm",
                                residual_mult=cfg.residual_mult, names=("norm1", "", "norm2", "mlp.")))
    return ModelPlan(architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=W, layers=tuple(blocks),
                     order=tuple(LayerCall(i) for i in range(len(blocks))), final_norm=norm, tie_word_embeddings=False,
                     max_position_embeddings=cfg.max_position_embeddings, layer_prefix="l{}.", embed_prefix="",
                     final_norm_prefix="final.norm", head_prefix="",
                     embedding=EmbeddingSpec(cfg.vocab_size, W, tensor="embed", scale=cfg.embedding_scale),
                     head=HeadSpec(cfg.vocab_size, W, tied=False, tensor="head"), unused_tensors=tuple(unused))


register_architecture(ARCHITECTURE, SodonexConfig, sodonex_plan, model_types=("sodonex",), replace=True)
