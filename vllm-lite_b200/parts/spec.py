"""Descriptions of model parts as plain data.

A model is a `ModelPlan`: an embedding, a list of layer descriptions, the order
in which layers run, a final norm and an output head (each of them a part).  Every description is a
frozen dataclass whose `kind` names the implementation in the part registries
(`parts.registry`); sizes and constants are fields, never code.  Layers may
differ from one another, and `order` may name a layer twice or let a layer read
the cache that an earlier call wrote.

Descriptions hold no tensors and import nothing from the GPU side, so the
configuration, the weight loader, the random-weights writer and the CPU tests
can all work from them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One tensor that a part binds by name.

    `init` names the distribution of the random-weights mode: "linear"
    (N(0, std)), "norm" (1 + N(0, norm_std)), "identity" (a square matrix: I + N(0, norm_std)), "conv" / "unit" (N(0, 0.5): taps of a short convolution, biases and
    logarithms of gates and decays), "rate" (0.05 + |N(0, 0.5)|: a positive factor).  `store` is the dtype the tensor
    has in a written folder and the least precision it is kept in:
    "model" (the model dtype, bfloat16 on disk) or "float32".
    """
    shape: Tuple[int, ...]
    init: str = "linear"
    store: str = "model"


@dataclass(frozen=True)
class NormSpec:
    """`kind`: "rms_norm" (x / sqrt(mean x^2 + eps) * w), "layer_norm" ((x - mean) / sqrt(var + eps) * w,
    no bias) or "dyn_tanh" (tanh(alpha x) * w + b, alpha a learned scalar: no mean, no variance, eps unused).
    `tensor`: the weight's name relative to the norm's prefix ("" when the prefix is the whole name); a norm with
    a bias vector or a scalar stores them as `tensor + bias_suffix` / `tensor + alpha_suffix`.
    `scalar`: the weight is ONE stored number for all `size` coordinates (an "rms_norm" only).
    `offset`: the stored weight lies around zero and the factor is offset + w (an "rms_norm" only; 0: the weight as stored).
    `has_weight` False: no tensor at all, the factor is 1 (an "rms_norm" only)."""
    size: int
    eps: float
    kind: str = "rms_norm"
    tensor: str = "weight"
    bias_suffix: str = ".b"
    alpha_suffix: str = ".alpha"
    scalar: bool = False
    offset: float = 0.0
    has_weight: bool = True


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding of the first `rotary_dim` features of each head; inv_freq[i] =
    theta^(-2i / rotary_dim).  Feature i turns with feature i + rotary_dim/2 (rotate-half), or, when
    `interleaved`, feature 2i with feature 2i+1."""
    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None
    kind: str = "rotary"
    interleaved: bool = False

    @property
    def dim(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache.

    `window`: None reads every earlier key; w reads the last w keys (the
    query's own position included).  `qk_norm`: norm over head_dim applied to
    every q and k head before the position encoding.  `scale` defaults to
    head_dim ** -0.5.

    Options on the scores and around them, each on its own (all off by default):
    `q_temp` (coef, every): the normed query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1);
    `v_norm`: every value head is divided by its root mean square over its own size (an RMS norm without a weight,
    with this eps) before it is cached;
    `softcap` c: score <- c tanh(score / c) after the scale;
    `distance_bias` (name a, name b): tensors [num_heads] each; a[h] ln(1 + b[h] (i - j)) is taken off the capped score
    of the key j that query i reads;
    `unit_sink`: the softmax denominator holds one more term exp(0) = 1, with no key and no value;
    `gate` (a tensor name): the concatenated heads are multiplied element by element by sigmoid(W_g h),
    W_g [num_heads * value size, hidden], before the output projection.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: Optional[NormSpec] = None
    position: Optional[RotarySpec] = None
    window: Optional[int] = None
    scale: Optional[float] = None
    bias: bool = False              # q/k/v projections with a bias vector each
    kind: str = "gqa_attention"
    out_bias: bool = False          # the output projection has a bias vector too
    v_head_dim: Optional[int] = None    # size of a value head when it differs from head_dim
    # tensor names relative to the mixer's prefix: q, k, v, o weights; the suffix of a projection's bias; the
    # prefixes of the two head norms
    names: Tuple[str, str, str, str] = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight")
    bias_names: Tuple[str, str, str, str] = ("q_proj.bias", "k_proj.bias", "v_proj.bias", "o_proj.bias")
    norm_prefixes: Tuple[str, str] = ("q_norm.", "k_norm.")
    q_temp: Optional[Tuple[float, int]] = None
    v_norm: Optional[float] = None
    softcap: Optional[float] = None
    distance_bias: Optional[Tuple[str, str]] = None
    unit_sink: bool = False
    gate: Optional[str] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token ids to rows of the residual stream: x[t] = table[id[t]] * scale (float32)."""
    vocab_size: int
    hidden_size: int
    kind: str = "token_embedding"
    tensor: str = "weight"          # the table's name relative to the embedding's prefix
    scale: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """The output head: logits = h W^T in float32, no bias.  `tied`: W is the embedding's table
    (the head then declares no tensor of its own)."""
    vocab_size: int
    hidden_size: int
    tied: bool = False
    kind: str = "linear_head"
    tensor: str = "weight"          # the matrix's name relative to the head's prefix (untied)


@dataclass(frozen=True)
class CappedHeadSpec:
    """logits = cap * tanh((h W^T) * scale / cap) in float32, W a matrix of the head's own; `softcap` None: only
    the scale."""
    vocab_size: int
    hidden_size: int
    scale: float = 1.0
    softcap: Optional[float] = None
    tensor: str = "weight"
    kind: str = "capped_head"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are both expanded from one cached latent row per token.

    c_q = rmsnorm(W_dq h), q = W_uq c_q (heads x dim); c = rmsnorm(W_dkv h) (kv_rank, the cached row);
    k_h = W_uk[h] c (dim), v_h = W_uv[h] c (vdim); scores scale * q.k over the last `window` positions
    (None: all earlier ones); `sink`: a learned number per head joins every softmax denominator;
    out = W_o concat_h(sum p v).  `names`: the tensors' names relative to the mixer's
    prefix, in the order (dq, dq norm, uq, dkv, dkv norm, uk, uv, o, sink).
    No position encoding unless `rot_dim` > 0: every query head then has rot_dim more features behind its `dim`
    (W_uq has heads * (dim + rot_dim) rows), W_dkv has rot_dim more rows behind the latent's, which are NOT normed and
    are ONE more key part shared by all heads; `position` turns the first `position.dim` features of both parts, and the
    score is scale * (q . k + q_rot . k_rot).  The cached row is then [c | rotated key part].
    `gate` (a tensor name): the concatenated heads times sigmoid(W_g h), W_g [heads * vdim, hidden], before W_o."""
    hidden_size: int
    num_heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    eps: float
    scale: Optional[float] = None
    window: Optional[int] = None
    sink: bool = False
    names: Tuple[str, ...] = ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o", "sink")
    kind: str = "latent_attention"
    rot_dim: int = 0
    position: Optional[RotarySpec] = None
    gate: Optional[str] = None


@dataclass(frozen=True)
class GatedMlpSpec:
    """down(act(gate(h)) * up(h)) with a choice of activation ("silu", "relu", or "capped_swish": g' = min(g, limit),
    u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + up_shift)) and optional bias vectors on all
    three projections.  `names`: (gate, up, down) relative to the part's prefix; a bias is `<name><bias_suffix>`.
    `gated` False: down(f(up(h))) with f a function of one argument ("relu2": the square of max(v, 0)); there is no gate
    matrix and no bias."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    bias: bool = False
    alpha: float = 1.0
    limit: float = 0.0
    up_shift: float = 0.0
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    bias_suffix: str = ".b"
    kind: str = "gated_mlp"
    gated: bool = True


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of small gated feed-forwards of which every token uses `top`.

    Router: z = W_r h in float32, score = sigmoid(z) ("sigmoid") or softmax(z) ("softmax"); the `top`
    largest scores choose; weights are the chosen scores, divided by their sum when `renormalize`.
    `scale_input`: the weight multiplies the expert's input (out = sum_e E_e(w_e h)), else its output.
    Expert: g = gate y, u = up y, no biases; activation "capped_swish": g' = min(g, limit),
    u' = clamp(u, -limit, limit), down(g' sigmoid(alpha g') (u' + up_shift)); "silu" / "relu": down(act(g) u).
    `gated` False: an expert is down(f(up y)) with f a function of one argument ("relu2": the square of max(v, 0)),
    and has no gate matrix.  `router_bias`: a vector `router + router_bias` added to the logits.  Score "softmax"
    with `renormalize` is the softmax over the chosen logits alone.
    `choice_bias` (a tensor name, [num_experts]): experts, and groups, are chosen by score + choice_bias; the weights are
    the scores without it.  `group_top`: a group's score is the sum of that many of its largest choice values (1: its
    largest).  `renorm_eps` is added to the sum that `renormalize` divides by.
    `shared`: the description of one more feed-forward (any registered kind) that runs for every token and is added; its
    tensors lie under `shared_prefix`.
    Tensors: `router`, and per expert i `expert_prefix.format(i)` + gate / up / down of `names`."""
    hidden_size: int
    intermediate_size: int
    num_experts: int
    top: int
    activation: str = "capped_swish"
    alpha: float = 1.702
    limit: float = 0.0
    up_shift: float = 1.0
    score: str = "sigmoid"
    renormalize: bool = False
    scale_input: bool = True
    # experts in `groups` equal groups of neighbours; a group's score is its largest score and only experts of
    # the `keep_groups` best groups can be chosen (1, 1: no grouping)
    groups: int = 1
    keep_groups: int = 1
    router: str = "router"
    expert_prefix: str = "e{}."
    names: Tuple[str, str, str] = ("gate", "up", "down")
    kind: str = "routed_experts"
    gated: bool = True
    router_bias: Optional[str] = None
    choice_bias: Optional[str] = None
    group_top: int = 1
    renorm_eps: float = 0.0
    shared: Optional[object] = None
    shared_prefix: str = "shared."


@dataclass(frozen=True)
class StateSpaceSpec:
    """Selective state space with one scalar decay per head (state-space duality form).

    W_in h = [z: inner | x: inner | B: groups*state | C: groups*state | dt: heads], inner = heads * vdim; x, B, C pass a
    causal convolution of `conv` taps per channel (with bias) and silu; dt = softplus(dt + dt_bias);
    S <- exp(-exp(A_log) dt) S + dt B x^T (state x vdim per head, heads share B, C in groups), y = S^T C + D x;
    out = W_o (rms_parts(y * silu(z)) * norm), the RMS norm over `norm_groups` equal parts.
    `names`: (in, conv, conv bias, dt_bias, A_log, D, norm, o)."""
    hidden_size: int
    num_heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int
    eps: float
    names: Tuple[str, ...] = ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")
    kind: str = "state_space"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """Matrix memory with an exponential input gate, stabilised by a running maximum m (starting at 0).

    q = W_q h dim^-1/2, k = W_k h (heads x dim), v = W_v h (heads x vdim); per head i = cap tanh((W_i h + b_i) / cap),
    f = logsigmoid(cap tanh((W_f h + b_f) / cap)); m' = max(f + m, i); S <- e^(f+m-m') S + e^(i-m') k v^T; n likewise
    with k; o = S^T q / (max(|n.q|, e^-m') + denom_eps); out = W_o (rms_head(o) * norm * sigmoid(W_g h)).
    `names`: (q, k, v, g, o, norm, i, i bias, f, f bias)."""
    hidden_size: int
    num_heads: int
    dim: int
    vdim: int
    gate_cap: float
    eps: float
    denom_eps: float = 1e-6
    names: Tuple[str, ...] = ("q", "k", "v", "g", "o", "norm", "i", "i.b", "f", "f.b")
    kind: str = "matrix_memory"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule with one decay per head and key channel.

    q = W_q h, k = W_k h (kv_heads x dim), v = W_v h (heads x vdim), each through a causal convolution of `conv` taps
    (no bias) and silu; q, k -> x / sqrt(sum x^2 + unit_eps), q also times dim^-1/2; beta = sigmoid(W_b h);
    g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias)) (heads x dim); S <- diag(g) S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q; out = W_o (rms_head(o) * norm * sigmoid(W_g2 W_g1 h)), norm of vdim entries shared by heads.
    `rank`: the width of both low-rank pairs.  `names`: (q, k, v, conv suffix, b, A_log, norm, a1, a2, dt_bias, g1, g2, o)."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int
    eps: float
    unit_eps: float = 1e-6
    names: Tuple[str, ...] = ("q", "k", "v", ".conv", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")
    kind: str = "delta_rule"


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Attention whose queries and keys pass a short convolution over time and whose values are its keys.

    q = W_q h (+ b), k = W_k h (+ b) (heads x head_dim, kv_heads x head_dim), each channel through a causal convolution of
    `conv` taps (no bias, no activation; 1 tap with weight 1 is no convolution); v = k as the convolution leaves it;
    q and k are then divided by the root mean square of their WHOLE row (all heads at once, eps inside the root) and
    multiplied by a weight of that size, and `position` turns the first features of every head.
    score = scale q.k over the keys that `chunk` (positions in blocks of that many from the sequence's start, no key of
    an earlier block) and `window` (the last that many keys) leave; `weighting` "sigmoid": a key weighs
    sigmoid(score + pb[head]) by itself (`head_bias`: the tensor pb), nothing is summed to one; "softmax": as usual.
    `gate`: head h's output is multiplied by sigmoid((W_g h)_h), W_g [heads, hidden].  out = W_o concat (+ b).
    `names`: (q, k, g, o, pb); a bias is `<name><bias_suffix>`, the taps `<name><conv_suffix>` [channels, conv], the norm
    weights `<name><norm_suffix>`."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    conv: int
    eps: float
    position: Optional[RotarySpec] = None
    scale: Optional[float] = None
    chunk: Optional[int] = None
    window: Optional[int] = None
    weighting: str = "sigmoid"
    head_bias: bool = True
    gate: bool = True
    bias: bool = True
    out_bias: bool = True
    names: Tuple[str, ...] = ("q", "k", "g", "o", "pb")
    bias_suffix: str = ".b"
    conv_suffix: str = ".conv"
    norm_suffix: str = ".norm"
    kind: str = "conv_attention"


@dataclass(frozen=True)
class TokenShiftSpec:
    """A mixer whose input is first mixed with the token before: h_t <- h_t + (h_(t-1) - h_t) * mu, element by element,
    h_(t-1) the input row of the sequence's token before as it was BEFORE this replacement (zeros before the first
    token); the last row of a request is part of its state.  `inner`: the mixer's description; its tensors lie under
    `inner_prefix`, mu [hidden] is `tensor`."""
    inner: object
    hidden_size: int
    tensor: str = "shift"
    inner_prefix: str = "mix."
    kind: str = "token_shift"


@dataclass(frozen=True)
class TimeMixSpec:
    """A memory per head with a decay per key channel, read through token shifts (time mixing in the manner of RWKV).

    With h' the row of the token before (zeros before a sequence's first token; the last row is part of the state), each of
    r, k, v, g, w reads its own mix h + (h' - h) * mu_s.  r, k, v = W_r, W_k, W_v of their mixes (heads x dim each),
    gate = silu(W_g mix_g), decay = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)) per head and key channel (`decay_rank`: rows of
    W_w1).  Per head, S [dim x dim] from zero: o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(decay_t) S + k_t v_t^T.
    out = W_o (rms_head(o) * norm * gate), the RMS norm over every head's dim values with `eps`, no weight but `norm`
    [heads * dim].  `names`: (mu prefix, r, k, v, g, w1, w2, w0, u, norm, o); the five mu are `<mu prefix><s>`."""
    hidden_size: int
    num_heads: int
    dim: int
    decay_rank: int
    eps: float
    names: Tuple[str, ...] = ("mu.", "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")
    kind: str = "time_mix"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side on the same input: left_scale * left(h) + right_scale * right(h).  Each keeps its own
    cache or state; their tensors lie under `prefixes`."""
    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    prefixes: Tuple[str, str] = ("left.", "right.")
    kind: str = "parallel_mixer"


@dataclass(frozen=True)
class HyperConnectionSpec:
    """The learned numbers of one sub-layer of a block with several streams: `in` [streams], `out` [streams],
    `mix` [streams, streams] (indexed [from, to]), named `<prefix><name>`."""
    streams: int
    names: Tuple[str, str, str] = ("in", "out", "mix")


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """kind "pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x)).
    kind "post_norm": x += m norm1(mixer(x)); x += m norm2(ffn(x)), m = `residual_mult`: the sub-layers read the stream
    itself and their OUTPUTS are normed; `ffn` may be None (the block is then its mixer alone, and norm2 is unused).
    kind "hyper_connection": `streams` copies x_1..x_S of the stream (all equal to the single stream when the first
    such block meets it); sub-layer q reads u = sum_s in_q[s] x_s through its norm and writes
    x_t <- sum_s mix_q[s, t] x_s + out_q[t] y; the single stream is the sum of the copies.  `hyper`: the two
    sub-layers' `HyperConnectionSpec`; `hyper_prefixes`: where their tensors lie.  `ffn` may be None.
    kind "sandwich": x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x))): a norm before and a norm after every
    sub-layer (`post_norms`, their tensors under `post_names`); `ffn` may be None."""
    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: NormSpec
    kind: str = "pre_norm"
    streams: int = 1
    hyper: Optional[Tuple[object, object]] = None
    hyper_prefixes: Tuple[str, str] = ("hc1.", "hc2.")
    residual_mult: float = 1.0      # post_norm: the factor on every normed sub-layer output
    # tensor-name prefixes of the four parts inside a layer (norm1, mixer, norm2, feed-forward)
    names: Tuple[str, str, str, str] = ("input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp.")
    post_norms: Optional[Tuple[NormSpec, NormSpec]] = None     # sandwich: the norms on the two sub-layers' outputs
    post_names: Tuple[str, str] = ("post_mixer_norm.", "post_mlp_norm.")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the running order.

    `layer` indexes `ModelPlan.layers` (the weights).  `cache_of`, when set, is
    the index of an EARLIER entry of the order whose cache this call reads
    instead of writing one of its own.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_prefix: str = "model.layers.{}."
    embed_prefix: str = "model.embed_tokens."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    init_std: float = 0.02
    norm_init_std: float = 0.1
    extra: dict = field(default_factory=dict, compare=False, hash=False)
    # The two ends of the model are parts like the layers' (registries EMBEDDINGS and HEADS).  Left None
    # they are the plain ones, described by vocab_size, hidden_size and tie_word_embeddings.
    embedding: Optional[object] = None
    head: Optional[object] = None
    # names of stored tensors that the model does not bind and that the loader passes over
    unused_tensors: Tuple[str, ...] = ()

    @property
    def embedding_spec(self):
        return self.embedding if self.embedding is not None else EmbeddingSpec(self.vocab_size, self.hidden_size)

    @property
    def head_spec(self):
        return self.head if self.head is not None else HeadSpec(self.vocab_size, self.hidden_size,
                                                                tied=self.tie_word_embeddings)

    def validate(self) -> "ModelPlan":
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {call.layer}, the plan has {len(self.layers)}")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < i:
                    raise ValueError(f"order[{i}].cache_of={call.cache_of} must name an earlier entry")
                if self.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}].cache_of={call.cache_of} names an entry that owns no cache")
        return self
