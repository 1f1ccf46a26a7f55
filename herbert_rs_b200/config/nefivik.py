"""The Nefivik decoder's configuration: a list of layers, each with one of two mixers and a routed feed-forward
or none.

config.json of this design is nested:

    architecture: "Nefivik"      vocab, width      norm.eps      token_side.dim (optional)
    layers: [{type, mixer: {...}, mlp: {kind: "moe", expert: {ff, limit}, router: {experts, top, groups: {count, keep}}} or null}, ...]
      type "attention":      mixer has heads, kv_heads, dim, vdim, scale, conv (taps, optional), mask.size (window, optional),
                             rot.{base, dims, scaling.{factor, low, high, original}} (optional), kv_from (optional: the
                             layer whose keys and values this one reads; it then has no key and value tensors)
      type "general_delta":  mixer has heads, dim

Every layer is a block with an RMS norm before and after each sublayer, a sigmoid gate (a full matrix with a bias,
reading the sublayer's input) on each sublayer's result, and at its end a second input chosen by the token: the
layer's own `token_side.dim` columns of one table of the model's.  The model ends with the same norm and a separate
head.  Tensor names: embed, side.embed, head, final.norm, and per layer
l<i>.{norm1, norm1b, norm2, norm2b, rg1, rg1.b, rg2, rg2.b, side.gate, side.proj, side.norm, mix.*, mlp.*}.

What the design fixes stands here as constants: the rotation pairs channel i with i + dims/2, the decay constant
exp(-1/2) and the unit keys' 1e-6 of the delta rule, the experts' activation, a group's score (its best expert).
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass

from ..errors import ConfigError
from .base import Reader
from .kebisun import NO_POSITION_LIMIT, _sub
from .specs import (AttentionSpec, BlockSpec, GeneralDeltaSpec, ModelSpec, NormSpec, RotaryPairsSpec, RoutedFFSpec,
                    ScheduleStep, TokenSideSpec)

PAIR_LAYOUT = "halves"
DECAY_CONSTANT = math.exp(-0.5)        # w = exp(-DECAY_CONSTANT * sigmoid(.))
UNIT_EPS = 1e-6
EXPERT_ACTIVATION = "swish_clamp"
GROUP_TOP = 1                          # a group of experts scores as its best member
SIDE_TABLE = "side.embed"


@dataclass
class NefivikConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: object         # int or None
    layers: tuple            # of (mixer spec, feed-forward spec or None, index of the layer whose cache is read or None)
    source: dict             # the config.json it was read from

    @classmethod
    def from_dict(cls, c: dict) -> "NefivikConfig":
        r = Reader(c)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps")
        if not eps > 0.0:
            raise ConfigError("norm.eps must be > 0")
        side = _sub(r, "token_side", required=False)
        side_dim = side.integer("dim", minimum=1) if side is not None else None
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = Reader(entry, f"layers[{i}]")
            kind = lr.string("type")
            m = _sub(lr, "mixer")
            src = None
            if kind == "attention":
                mixer, src = cls._attention(m, width, i, layers)
            elif kind == "general_delta":
                heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
                mixer = GeneralDeltaSpec(width, heads, dim, dim, float(eps), DECAY_CONSTANT, UNIT_EPS)
            else:
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (attention, general_delta)")
            f = _sub(lr, "mlp", required=False)
            layers.append((mixer, cls._ff(f, width) if f is not None else None, src))
        # a layer whose keys other layers read keeps them as long as the longest of their windows asks
        for i, (mixer, ff, src) in enumerate(layers):
            if src is None:
                continue
            owner = layers[src][0]
            keep = owner.window if owner.cache_window == -1 else owner.cache_window
            if keep is not None and (mixer.window is None or mixer.window > keep):
                layers[src] = (_with(owner, cache_window=mixer.window), layers[src][1], None)
        return cls(vocab, width, float(eps), side_dim, tuple(layers), copy.deepcopy(c))

    @staticmethod
    def _attention(m: Reader, width: int, index: int, before: list):
        heads, kv = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv:
            raise ConfigError(f"{m.where}: heads ({heads}) must be a multiple of kv_heads ({kv})")
        dim, vdim = m.integer("dim", minimum=1), m.integer("vdim", minimum=1)
        position = None
        rot = _sub(m, "rot", required=False)
        if rot is not None:
            dims = rot.integer("dims", minimum=0)
            if dims % 2 or dims > dim:
                raise ConfigError(f"{m.where}: rot.dims ({dims}) must be even and at most dim ({dim})")
            sc = _sub(rot, "scaling", required=False)
            bands = None
            if sc is not None:
                bands = (sc.number("factor"), sc.number("low"), sc.number("high"), sc.number("original"))
                if not (bands[0] > 0.0 and bands[3] > 0.0 and bands[2] > bands[1] >= 0.0):
                    raise ConfigError(f"{m.where}: rot.scaling needs factor > 0, original > 0 and high > low >= 0")
            if dims:
                position = RotaryPairsSpec(dims, rot.number("base"), 1.0, PAIR_LAYOUT, band_scaling=bands)
        mask = _sub(m, "mask", required=False)
        window = mask.integer("size", minimum=1) if mask is not None else None
        taps = m.integer("conv", None, minimum=1)
        src = m.integer("kv_from", None, minimum=0)
        if src is not None:
            if src >= index:
                raise ConfigError(f"{m.where}: kv_from ({src}) must name an earlier layer")
            owner = before[src][0]
            if not isinstance(owner, AttentionSpec) or owner.reads_kv:
                raise ConfigError(f"{m.where}: kv_from ({src}) must name an attention layer with keys and values of its own")
            if (owner.num_kv_heads, owner.head_dim, owner.value_dim) != (kv, dim, vdim):
                raise ConfigError(f"{m.where}: kv_from ({src}) names a layer with other key/value heads or sizes")
        spec = AttentionSpec(
            hidden_size=width, num_heads=heads, num_kv_heads=kv, head_dim=dim, scale=m.number("scale"), position=position,
            window=window, names=("q", "k", "v", "o", "sink"), value_dim=vdim, key_weights="sigmoid", key_bias_name="pb",
            conv_taps=taps, conv_suffix=".conv", head_gate=True, head_gate_name="g", reads_kv=src is not None)
        return spec, src

    @staticmethod
    def _ff(f: Reader, width: int):
        kind = f.string("kind")
        if kind != "moe":
            raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (moe)")
        ex, rt = _sub(f, "expert"), _sub(f, "router")
        experts, top = rt.integer("experts", minimum=1), rt.integer("top", minimum=1)
        gr = _sub(rt, "groups", required=False)
        count, keep = (gr.integer("count", minimum=1), gr.integer("keep", minimum=1)) if gr is not None else (1, 1)
        if experts % count or keep > count or top > keep * (experts // count):
            raise ConfigError(f"{f.where}: {experts} experts in {count} groups of which {keep} stay cannot give {top} per token")
        limit = ex.number("limit")
        if not limit > 0.0:
            raise ConfigError(f"{f.where}: expert.limit must be > 0")
        return RoutedFFSpec(width, experts, top, ex.integer("ff", minimum=1), activation=EXPERT_ACTIVATION, renormalize=False,
                            router_name="router", expert_names=("e{e}.gate", "e{e}.up", "e{e}.down"), gated=True,
                            score="softmax", groups=count, keep_groups=keep, group_top=GROUP_TOP, act_limit=float(limit))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.source)

    def model_spec(self) -> ModelSpec:
        def norm(name):
            return NormSpec(self.width, self.norm_eps, weight_name=name)
        blocks, schedule = [], []
        for i, (mixer, ff, src) in enumerate(self.layers):
            side = TokenSideSpec(self.side_dim, i * self.side_dim, self.norm_eps) if self.side_dim is not None else None
            blocks.append(BlockSpec(
                mixer=mixer, ffn=ff, norm1=norm("norm1"), norm2=norm("norm2"), kind="sandwich",
                post_norms=(norm("norm1b"), norm("norm2b")), residual_gates=("rg1", "rg2"), residual_gate_bias=".b",
                token_side=side,
                names=(("norm1", ""), ("post1", ""), ("mixer", "mix"), ("norm2", ""), ("post2", ""), ("ffn", "mlp"))))
            schedule.append(ScheduleStep(i, reads_cache_of=src))
        table = (SIDE_TABLE, len(self.layers) * self.side_dim) if self.side_dim is not None else None
        return ModelSpec(
            architecture="Nefivik", vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=tuple(schedule), final_norm=norm("norm"), tie_word_embeddings=False, max_position=NO_POSITION_LIMIT,
            stop_token_ids=(), layer_prefix="l{i}.", embed_name="embed", final_norm_name="final.norm", head_name="head",
            token_side_table=table)


def _with(spec, **changes):
    import dataclasses
    return dataclasses.replace(spec, **changes)
