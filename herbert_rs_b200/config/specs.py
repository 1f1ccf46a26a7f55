"""Size-and-constant records ("specs") from which parts are built.

A spec is plain data: it says which kind of part stands at a place and with which
sizes and constants.  An architecture's configuration produces a `ModelSpec`; the
part registry (`herbert_rs_b200.registry`) turns every spec into a part by its
`kind`.  No spec and no part knows which model it belongs to.

The reference keeps the same facts as fields of its generic parts
(crates/backends/backend_common/src/generic_attention/mod.rs:27-59 for the mixer,
generic_mlp.rs:20-28 for the feed-forward, generic_layer.rs:705-719 for the block);
here they are separated from the parts so that a layer list is data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis.  kind "rmsnorm": y = x / sqrt(mean(x^2) + eps) * w;
    kind "layernorm": y = (x - mean(x)) / sqrt(var(x) + eps) * w (no bias).  `weight_offset` c: the
    stored tensor is w - c (a weight kept around zero with c = 1), so the factor is c + stored."""

    dim: int
    eps: float
    kind: str = "rmsnorm"
    weight_name: str = "weight"     # the weight's tensor name under the part's prefix
    weight_offset: float = 0.0
    # rmsnorm only: the axis is cut into this many equal consecutive parts and each part is divided by
    # its own root mean square; the weight still spans the whole axis
    groups: int = 1


@dataclass(frozen=True)
class PositionSpec:
    """A position encoding applied inside a mixer.  kind "rope": half-split rotary pairs."""

    head_dim: int
    rotary_dim: int
    theta: float
    max_position: int
    kind: str = "rope"


@dataclass(frozen=True)
class ScaledRotarySpec:
    """Half-split rotary pairs whose angles are computed from the position (no table, no longest
    position), optionally with frequencies stretched band by band.  f_i = theta^(-2i/rotary_dim);
    with `factor` set: d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1),
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- f_i / factor * r_i + f_i * (1 - r_i),
    and cos and sin are both multiplied by 0.1 ln(factor) + 1."""

    rotary_dim: int
    theta: float
    factor: Optional[float] = None
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    kind: str = "scaled_rope"


@dataclass(frozen=True)
class RotaryPairsSpec:
    """Rotary pairs whose angles are computed from the position (no table): pair m of `rotary_dim`
    channels turns by p * theta^(-2m/rotary_dim) / linear_factor.  layout "interleaved": pair m is
    channels (2m, 2m + 1); "halves": (m, m + rotary_dim/2).  Channels beyond rotary_dim pass unchanged.
    `band_scaling` (factor, low, high, original) changes the frequencies band by band: with the wavelength
    l = 2 pi / f, f stays where l < original / high, becomes f / factor where l > original / low, and in between
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""

    rotary_dim: int
    theta: float
    linear_factor: float = 1.0
    layout: str = "interleaved"
    kind: str = "rope_pairs"
    band_scaling: Optional[tuple] = None


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are products of one cached latent per token.
    Per head: `nope_dim` unrotated and `rope_dim` rotated query/key channels, values of `v_dim`;
    queries through a latent of `q_rank` (None: straight from the input), keys and values from one
    of `kv_rank`, plus one rotated key part shared by all heads.  `sink`: a learned number per head
    joins the softmax's denominator.  `gate`: the heads' outputs are multiplied by sigmoid(G h)."""

    hidden_size: int
    num_heads: int
    nope_dim: int
    rope_dim: int
    v_dim: int
    kv_rank: int
    scale: float
    norm_eps: float
    q_rank: Optional[int] = None
    position: Optional[ScaledRotarySpec] = None
    window: Optional[int] = None
    sink: bool = False
    gate: bool = False
    kind: str = "latent_attention"


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a state matrix per head and a decay per key channel:
    S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, a = sigmoid(W2 W1 h + b)^(1/tau);
    per-head RMSNorm of o, gate silu(G h), output product."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay_rank: int
    decay_tau: float
    norm_eps: float
    kind: str = "gla"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over cached keys and values.

    Options beyond the plain form (each off by default):
    `bias`: q, k (and v) = W h + b, the bias tensors named as the matrices with `bias_suffix` added;
    `values_are_keys`: no value product: a head's values are its keys as projected, and the cache
        keeps one plane;
    `q_temperature` (coef, every): the query at position p is multiplied by
        1 + coef * ln(floor((p + 1) / every) + 1);
    `softcap` c: score <- c * tanh(score / c) after the scale;
    `sink`: a learned number per query head (tensor `names[4]`) whose exponential joins the softmax's
        denominator; it has no key and no value.
    `names`: the tensors of q, k, v, o and the sink under the mixer's prefix."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    window: Optional[int] = None  # None: every earlier key; n: the last n keys (itself included)
    kind: str = "attention"
    bias: bool = False
    bias_suffix: str = ".b"
    values_are_keys: bool = False
    q_temperature: Optional[tuple] = None
    softcap: Optional[float] = None
    sink: bool = False
    names: tuple = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "sink")
    # A third form, taken when `position` is a RotaryPairsSpec or any of the following is set:
    # `value_dim`: the values' size per head where it differs from `head_dim` (the queries' and keys');
    # `whole_qk_norm`: one RMS norm over the whole q projection and one over the whole k projection
    #     (all heads at once, weights named by `norm_names`, eps of `qk_norm`), before the rotation;
    # `value_rotation`: the value at position j is stored turned by j (over all of its channels), and
    #     a head's result at position i is turned back by -i: the result then depends on i - j only.
    value_dim: Optional[int] = None
    whole_qk_norm: bool = False
    value_rotation: Optional[RotaryPairsSpec] = None
    norm_names: tuple = ("q_norm.weight", "k_norm.weight")
    # Further options of that form (each takes it):
    # `key_weights` "sigmoid": no softmax; a visible key weighs sigmoid(score + b) with a learned b per query head
    #     (tensor `key_bias_name`), and the weights are not normalised over the keys;
    # `conv_taps`: q, k and v each pass a short causal convolution over time, channel by channel, right after the
    #     projection (tensors named as the matrices with `conv_suffix`, [channels, taps], the last column weighs the
    #     token itself); a sequence's last taps - 1 projected rows are state;
    # `head_gate`: a head's result is multiplied by sigmoid(G h), one number per token and head (tensor `head_gate_name`);
    # `reads_kv`: the mixer has no key and value tensors: its schedule step reads what another step stored;
    # `cache_window`: how many of the last keys the cache must keep, where that differs from the mixer's own window
    #     (another step with a longer window reads this one's keys); -1: the mixer's window, None: every key.
    key_weights: str = "softmax"
    key_bias_name: str = "pb"
    conv_taps: Optional[int] = None
    conv_suffix: str = ".conv"
    head_gate: bool = False
    head_gate_name: str = "g"
    reads_kv: bool = False
    cache_window: Optional[int] = -1


@dataclass(frozen=True)
class LightningAttentionSpec:
    """Linear attention with a matrix of state per head and one constant decay per head:
    q, k, v = silu(W h);  S_t = decay_h S_{t-1} + k_t v_t^T;  o_t = S_t^T q_t;  the heads' results,
    side by side, pass one RMS norm (weight over all of them), are multiplied by sigmoid(G h) and
    projected."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: tuple
    norm_eps: float
    kind: str = "lightning"
    names: tuple = ("q", "k", "v", "g", "o", "norm")


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule: per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with
    q, k of `qk_heads` heads (value head h uses q/k head h / (num_heads / qk_heads)), each of q, k, v
    through a short causal convolution of `conv_taps` taps and silu, q and k made unit vectors per
    head (q also times key_dim^-1/2), beta = sigmoid(B h), g = exp(-exp(A_log) softplus(A h + dt_bias));
    per-head RMS norm of o (weight of value_dim, shared), gate silu(G h), output product."""

    hidden_size: int
    num_heads: int
    qk_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    kind: str = "gated_delta"
    unit_eps: float = 1e-6      # inside the root of the unit vectors' length


@dataclass(frozen=True)
class GeneralDeltaSpec:
    """The generalised delta rule: per head S <- diag(w) S - (a * u) (u^T S) + k v^T (both terms read the old S),
    o = S^T r, with u = k / sqrt(sum k^2 + unit_eps) per head, a decay per head and key channel
    w = exp(-decay_constant * sigmoid(W2 tanh(W1 h) + w0)) and a removal rate a = sigmoid(A h + a0) likewise;
    r, k, v = R h, K h, V h.  Each head's o is divided by its root mean square, the heads side by side are
    multiplied by a weight (one number per head and channel) and by sigmoid(G h), then projected.  The decay's
    inner width is the stored tensor's."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    norm_eps: float
    decay_constant: float
    unit_eps: float = 1e-6
    kind: str = "general_delta"
    names: tuple = ()          # pairs (role, tensor name) that replace the mixer's defaults


@dataclass(frozen=True)
class TokenSideSpec:
    """A second input chosen by the token, added at the end of a layer: e = table[token][column0 : column0 + dim];
    y = P (gelu_tanh(G x) * e); x <- x + y / sqrt(mean(y^2) + eps) * w.  `names`: G, P and w under the block's prefix.
    The table belongs to the model (`ModelSpec.token_side_table`); a layer reads its own columns of it."""

    dim: int
    column0: int
    eps: float
    names: tuple = ("side.gate", "side.proj", "side.norm")


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; the result is left_scale * left + right_scale * right.
    Their tensors lie under the sub-prefixes of `names`."""

    left: object
    right: object
    left_scale: float
    right_scale: float
    kind: str = "side_by_side"
    names: tuple = ("left", "right")


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """A second embedding table chosen by a token and its predecessor: row
    (previous * mul_prev + token * mul_cur) mod buckets of a table of buckets + 1 rows, whose last
    row serves a sequence's first token; it is added to the token's own embedding."""

    buckets: int
    mul_prev: int
    mul_cur: int
    table_name: str = "bigram"


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)); act "silu", "gelu_tanh", "gelu" or "relu".
    `names`: the tensors of gate, up and down; with `bias` every projection adds a vector named as
    its matrix with `bias_suffix`."""

    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"
    activation: str = "silu"
    names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    bias: bool = False
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class RoutedFFSpec:
    """A mixture of small feed-forwards down(act(up(x))) without biases: a token uses the `top_k`
    experts with the largest softmax(router x) (taken over all experts), weighted by those values,
    divided by their sum only with `renormalize`.  Tensor names: `router_name`, and
    `expert_names` formatted with the expert's index for up and down.

    Options: `gated`: an expert is down(act(gate(x)) * up(x)) and `expert_names` holds gate, up, down;
    `score` "sigmoid": the scores are sigmoid(router x) instead of the softmax; `groups`, `keep_groups`,
    `group_top`: the experts form `groups` equal groups of neighbours, a group's score is the sum of its
    `group_top` largest scores, and only experts of the `keep_groups` best groups can be chosen;
    `weight_scale`: a factor on every chosen weight; `shared`: a dense gated feed-forward (its own
    spec, which also names its tensors) that runs for every token and is added.  activation "swish_clamp" (gated
    experts only) takes `act_limit` L: g = min(gate, L), u = clamp(up, -L, L), hidden = g sigmoid(1.702 g) (u + 1)."""

    hidden_size: int
    num_experts: int
    top_k: int
    expert_size: int
    activation: str = "gelu"
    renormalize: bool = False
    router_name: str = "router"
    expert_names: tuple = ("e{e}.up", "e{e}.down")
    kind: str = "moe"
    gated: bool = False
    score: str = "softmax"
    groups: int = 1
    keep_groups: int = 1
    group_top: int = 2
    weight_scale: float = 1.0
    shared: Optional[SwiGLUSpec] = None
    act_limit: float = 0.0


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how a mixer, a feed-forward and their norms are arranged.

    kind "prenorm": h = x + mixer(norm1(x)); out = h + ffn(norm2(h)).
    kind "sublayer_norm": h = x + s1 * norm1(mixer(x)); out = h + s2 * norm2(ffn(h)): the sublayers
    read the stream itself and their results are normed; s1, s2 are per-channel scales named by
    `layer_scale` (None: no scales); `ffn` may be None (then the layer ends after the mixer).  With
    `input_conv_taps` the mixer reads x + conv(x) instead, a causal convolution over time on each
    channel (tensor `input_conv_name`, [width, taps], the last column weighs the token itself).
    kind "parallel": h = norm1(x); out = x + residual_mult * (mixer(h) + ffn(h)): one norm, both
    sublayers read its result; `ffn` may be None; norm2 is unused (None).
    kind "sandwich": a norm before and after each sublayer, h = norm1(x); x <- x + post1(mixer(h) * gate1);
    h = norm2(x); x <- x + post2(ffn(h) * gate2): `post_norms` are the two norms of the results, `residual_gates`
    (None: no gates) names two matrices R with biases (R's name + `residual_gate_bias`): gate = sigmoid(R h + b), a
    number per channel, from the same h the sublayer reads; `ffn` may be None; `token_side` adds a token's own second
    input at the layer's end.
    `names` maps the block's local part names to the sub-prefixes used in tensor names.
    """

    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: Optional[NormSpec]
    kind: str = "prenorm"
    layer_scale: Optional[tuple] = None
    residual_mult: float = 1.0
    input_conv_taps: Optional[int] = None
    input_conv_name: str = "canon1"
    post_norms: Optional[tuple] = None
    residual_gates: Optional[tuple] = None
    residual_gate_bias: str = ".b"
    token_side: Optional[TokenSideSpec] = None
    names: tuple = (
        ("norm1", "input_layernorm"),
        ("mixer", "self_attn"),
        ("norm2", "post_attention_layernorm"),
        ("ffn", "mlp"),
    )


@dataclass(frozen=True)
class ScheduleStep:
    """One entry of the execution order.

    `layer` indexes `ModelSpec.blocks`; a layer may be named by several steps (its weights
    are then used several times, each step with a cache entry of its own).  A step with
    `reads_cache_of = k` stores nothing: its mixer reads what step k (an earlier step) stored.
    """

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs: table sizes, layers, order, output head."""

    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: Sequence[BlockSpec]
    schedule: Sequence[ScheduleStep]
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_position: int
    stop_token_ids: tuple = ()
    layer_prefix: str = "model.layers.{i}."
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    # How many numbers place a token: 1 for a position in a sequence.  An encoding that needs
    # more (rows and columns of an image, say) raises this; the step then carries that many position
    # rows per token, which the caller may give per sequence (Engine.step(..., positions=...)) and
    # which default to the token's index in its sequence in every component.
    position_components: int = 1
    embedding_scale: float = 1.0                  # the embedding rows are multiplied by this
    # A learned vector per position, [max_position, hidden], added (unscaled) to the embedding row;
    # None: the model has none.  A sequence cannot grow beyond the table.
    position_table_name: Optional[str] = None
    # A table chosen by (previous token, token), added to the embedding; the previous token is state.
    pair_embedding: Optional[PairEmbeddingSpec] = None
    # c: logits <- c * tanh(logits / c)
    logit_softcap: Optional[float] = None
    # (tensor name, columns): a second table [vocab, columns] of which blocks with a `token_side` read their columns
    token_side_table: Optional[tuple] = None
    extra: dict = field(default_factory=dict)     # free for an architecture's own model class


def identity_schedule(n: int) -> tuple:
    """Every layer once, in order, each with its own cache entry."""
    return tuple(ScheduleStep(i) for i in range(n))
