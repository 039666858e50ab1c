"""Configuration of the Puturax decoder and its plan of parts.

config.json: `architecture` (a string), `vocab`, `width`, `embedding.scale`, `norm.eps` and `layers`, one object per layer:

    {"type": "latent_attention",
     "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot": {"dims", "base"}},
     "mlp": ...}
    {"type": "parallel",
     "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "q_temp": {"coef", "every"}},
               "right": {"heads", "dim"}, "left_scale", "right_scale"},
     "mlp": ...}
    "mlp": null | {"kind": "dense", "ff"}
               | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}}, "shared": {"ff"}}

Every size and every constant the file gives is read from it; the rank of the time mixing's decay is the first size of
the tensor `l<i>.mix.right.w1` (`shapes`, from the weight file's header; a config.json may carry `decay_rank` in the
right mixer's object, which the random-weights writer needs).  What the design fixes stands in `puturax_plan` as
arguments of the parts: blocks with an RMS norm before AND after every sub-layer, the norms' weights stored around zero
(factor 1 + w); latent attention with a rotated part of its own (rotate-half, shared key part), plain weights on the two
latent norms, a sigmoid output gate; beside each other an attention without rotation (weightless RMS norms on q, k and v,
a query factor that grows with the position, capped scores less a bias that grows with the logarithm of the distance, a
sink of score 0, a sigmoid output gate) and a time mixing (five token shifts, a decay per key channel, a bonus for the
current token, a norm per head, a silu gate); a dense feed-forward that squares max(v, 0), or experts with silu gates
chosen by sigmoid score plus a correction within the best groups (a group counts by its two best), weights renormalised
over the chosen, and a shared expert; a scaled embedding whose table is also the output head.  Tensor names are flat:
`embed`, `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.<t>`, `l<i>.mlp.<t>`, `final.norm`.
`max_position_embeddings` is optional (an engine bound on a request's length, not part of the design).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..parts.spec import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LatentAttentionSpec, LayerCall,
                          ModelPlan, NormSpec, ParallelMixerSpec, RotarySpec, RoutedExpertsSpec, TimeMixSpec)
from .errors import ConfigError, InvalidField, MissingField
from .kikepel import _field, _pos_int
from .registry import register_architecture

ARCHITECTURE = "Puturax"
MIXER_TYPES = ("latent_attention", "parallel")
DEFAULT_MAX_POSITIONS = 32768

# what the design fixes
NORM_OFFSET = 1.0                  # a norm's factor is 1 + its stored weight
DENSE_ACTIVATION = "relu2"         # the square of max(v, 0)
EXPERT_ACTIVATION = "silu"
GROUP_TOP = 2                      # a group of experts counts by the sum of its two largest choice scores
RENORM_EPS = 1e-20


def _number(d, key, where):
    return float(_field(d, key, where))


@dataclass(frozen=True)
class PuturaxLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class PuturaxConfig:
    vocab_size: int
    hidden_size: int
    eps: float
    embedding_scale: float
    layers: Tuple[PuturaxLayer, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    architecture: str = ARCHITECTURE

    needs_shapes = True            # `from_dict(d, shapes=...)`: the decay's rank is a tensor's first size

    @classmethod
    def from_dict(cls, d: dict, shapes: Optional[dict] = None) -> "PuturaxConfig":
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
            if typ == "latent_attention":
                rot = _field(m, "rot", mw, dict)
                mixer = {k: _pos_int(m, k, mw) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank")}
                mixer.update(scale=_number(m, "scale", mw), rot_dims=_pos_int(rot, "dims", f"{mw}.rot"),
                             rot_base=_number(rot, "base", f"{mw}.rot"))
                if mixer["rot_dims"] % 2 or mixer["rot_dims"] > mixer["rot_dim"]:
                    raise InvalidField(f"{mw}.rot.dims", "must be even and at most rot_dim")
                if not mixer["rot_base"] > 0:
                    raise InvalidField(f"{mw}.rot.base", "must be positive")
            else:
                left, right = _field(m, "left", mw, dict), _field(m, "right", mw, dict)
                lw, rw = f"{mw}.left", f"{mw}.right"
                lm = {k: _pos_int(left, k, lw) for k in ("heads", "kv_heads", "dim", "vdim")}
                lm["scale"] = _number(left, "scale", lw)
                lm["softcap"] = _number(left, "softcap", lw) if left.get("softcap") is not None else None
                if lm["softcap"] is not None and not lm["softcap"] > 0:
                    raise InvalidField(f"{lw}.softcap", "must be positive")
                lm["q_temp"] = None
                if left.get("q_temp") is not None:
                    qt = _field(left, "q_temp", lw, dict)
                    lm["q_temp"] = (_number(qt, "coef", f"{lw}.q_temp"), _pos_int(qt, "every", f"{lw}.q_temp"))
                if lm["heads"] % lm["kv_heads"]:
                    raise InvalidField(f"{lw}.kv_heads", "must divide heads")
                rm = {k: _pos_int(right, k, rw) for k in ("heads", "dim")}
                tensor = f"l{i}.mix.right.w1"
                if "decay_rank" in right:
                    rm["decay_rank"] = _pos_int(right, "decay_rank", rw)
                elif shapes is not None and tensor in shapes:
                    rm["decay_rank"] = int(shapes[tensor][0])
                else:
                    raise MissingField(f"{rw}.decay_rank (neither in config.json nor given by the shape of {tensor})")
                mixer = {"left": lm, "right": rm, "left_scale": _number(m, "left_scale", mw),
                         "right_scale": _number(m, "right_scale", mw)}
            mj, mlp = lj.get("mlp"), None
            if mj is not None:
                fw = f"{where}.mlp"
                kind = mj.get("kind") if isinstance(mj, dict) else None
                if kind == "dense":
                    mlp = {"kind": "dense", "ff": _pos_int(mj, "ff", fw)}
                elif kind == "moe":
                    ex, ro = _field(mj, "expert", fw, dict), _field(mj, "router", fw, dict)
                    mlp = {"kind": "moe", "ff": _pos_int(ex, "ff", f"{fw}.expert"), "experts": _pos_int(ro, "experts", f"{fw}.router"),
                           "top": _pos_int(ro, "top", f"{fw}.router"), "groups": 1, "keep": 1, "shared_ff": None}
                    if ro.get("groups") is not None:
                        gr = _field(ro, "groups", f"{fw}.router", dict)
                        mlp["groups"] = _pos_int(gr, "count", f"{fw}.router.groups")
                        mlp["keep"] = _pos_int(gr, "keep", f"{fw}.router.groups")
                    if mlp["experts"] % mlp["groups"] or mlp["keep"] > mlp["groups"] \
                            or mlp["keep"] * (mlp["experts"] // mlp["groups"]) < mlp["top"] or mlp["top"] > mlp["experts"]:
                        raise InvalidField(f"{fw}.router", f"{mlp['experts']} experts in {mlp['groups']} groups of which "
                                                           f"{mlp['keep']} are kept cannot offer {mlp['top']} choices")
                    if mj.get("shared") is not None:
                        mlp["shared_ff"] = _pos_int(_field(mj, "shared", fw, dict), "ff", f"{fw}.shared")
                else:
                    raise InvalidField(f"{fw}.kind", f"{kind!r}; known: dense, moe")
            layers.append(PuturaxLayer(typ, mixer, mlp))
        eps = _number(_field(d, "norm", "", dict), "eps", "norm")
        if not eps > 0:
            raise InvalidField("norm.eps", f"must be positive, got {eps}")
        maxpos = d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)
        if isinstance(maxpos, bool) or not isinstance(maxpos, int) or maxpos <= 0:
            raise InvalidField("max_position_embeddings", f"expected a positive integer, got {maxpos!r}")
        return cls(vocab_size=_pos_int(d, "vocab"), hidden_size=_pos_int(d, "width"), eps=eps,
                   embedding_scale=_number(_field(d, "embedding", "", dict), "scale", "embedding"),
                   layers=tuple(layers), max_position_embeddings=maxpos)


def puturax_plan(cfg: PuturaxConfig) -> ModelPlan:
    W, eps = cfg.hidden_size, cfg.eps
    norm = NormSpec(W, eps, kind="rms_norm", tensor="", offset=NORM_OFFSET)
    blocks, unused = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "latent_attention":
            mixer = LatentAttentionSpec(hidden_size=W, num_heads=m["heads"], dim=m["dim"], vdim=m["vdim"], q_rank=m["q_rank"],
                                        kv_rank=m["kv_rank"], eps=eps, scale=m["scale"], rot_dim=m["rot_dim"],
                                        position=RotarySpec(m["rot_dim"], m["rot_base"], rotary_dim=m["rot_dims"]), gate="g")
        else:
            lm, rm = m["left"], m["right"]
            left = AttentionSpec(hidden_size=W, num_heads=lm["heads"], num_kv_heads=lm["kv_heads"], head_dim=lm["dim"],
                                 v_head_dim=lm["vdim"], qk_norm=NormSpec(lm["dim"], eps, has_weight=False), position=None,
                                 scale=lm["scale"], names=("q", "k", "v", "o"), q_temp=lm["q_temp"], v_norm=eps,
                                 softcap=lm["softcap"], distance_bias=("r1", "r2"), unit_sink=True, gate="g")
            right = TimeMixSpec(hidden_size=W, num_heads=rm["heads"], dim=rm["dim"], decay_rank=rm["decay_rank"], eps=eps)
            mixer = ParallelMixerSpec(left=left, right=right, left_scale=m["left_scale"], right_scale=m["right_scale"])
        ffn = None
        p = layer.mlp
        if p is None:
            unused += [f"l{i}.norm2", f"l{i}.norm2b"]      # a layer without a feed-forward may still store its norms
        elif p["kind"] == "dense":
            ffn = GatedMlpSpec(W, p["ff"], activation=DENSE_ACTIVATION, gated=False, names=("gate", "up", "down"))
        else:
            shared = None
            if p["shared_ff"] is not None:
                shared = GatedMlpSpec(W, p["shared_ff"], activation=EXPERT_ACTIVATION, names=("gate", "up", "down"))
            ffn = RoutedExpertsSpec(W, p["ff"], p["experts"], p["top"], activation=EXPERT_ACTIVATION, score="sigmoid",
                                    renormalize=True, scale_input=False, groups=p["groups"], keep_groups=p["keep"],
                                    choice_bias="correction", group_top=GROUP_TOP, renorm_eps=RENORM_EPS, shared=shared)
        blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=norm, kind="sandwich", post_norms=(norm, norm),
                                names=("norm1", "mix.", "norm2", "mlp."), post_names=("norm1b", "norm2b")))
    return ModelPlan(architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=W, layers=tuple(blocks),
                     order=tuple(LayerCall(i) for i in range(len(blocks))), final_norm=norm, tie_word_embeddings=True,
                     max_position_embeddings=cfg.max_position_embeddings, layer_prefix="l{}.", embed_prefix="",
                     final_norm_prefix="final.norm", head_prefix="",
                     embedding=EmbeddingSpec(cfg.vocab_size, W, tensor="embed", scale=cfg.embedding_scale),
                     head=HeadSpec(cfg.vocab_size, W, tied=True), unused_tensors=tuple(unused))


register_architecture(ARCHITECTURE, PuturaxConfig, puturax_plan, model_types=("puturax",), replace=True)
