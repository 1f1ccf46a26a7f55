"""The Begupel decoder's configuration: a list of layers, each with one of two mixers and a dense
feed-forward or none.

config.json of this design is nested:

    architecture: "Begupel"      vocab, width      norm.{eps, groups}      canon.taps      logit_softcap
    embedding.bigram.{buckets, mul_prev, mul_cur}
    layers: [{type, mixer: {...}, mlp: {kind: "dense", ff} or null}, ...]
      type "lightning": mixer has heads, dim, vdim, decay (one number per head)
      type "parallel":  mixer has left_scale, right_scale and
            left  = {heads, kv_heads, dim, vdim, scale, mask.size (window), rot.{base, dims, scaling.factor}}
            right = {heads, kv_heads, dim, vdim, conv (taps)}

Every layer is a block whose sublayers read the residual stream itself (the mixer through a short causal
convolution added to it) and whose results pass an RMS norm in groups before they join the stream.  The
embedding adds a row chosen by (previous token, token); the model ends with the same norm, a separate
head and a tanh cap on the logits.  Tensor names: embed, bigram, head, final.norm, and per layer
l<i>.{norm1, norm2, canon1, mix.*, mlp.*}.

What the design fixes stands here as constants: the pairs of a rotation are neighbouring channels, the
values turn at the keys' base without its linear factor, the feed-forward's activation is relu and its
projections have biases.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import ConfigError
from .base import Reader
from .kebisun import NO_POSITION_LIMIT, _sub
from .specs import (AttentionSpec, BlockSpec, GatedDeltaSpec, LightningAttentionSpec, ModelSpec, NormSpec, PairEmbeddingSpec,
                    RotaryPairsSpec, SideBySideSpec, SwiGLUSpec, identity_schedule)

PAIR_LAYOUT = "interleaved"
FF_ACTIVATION = "relu"


@dataclass
class BegupelConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    canon_taps: int
    pair_embedding: PairEmbeddingSpec
    logit_softcap: object    # float or None
    layers: tuple            # of (mixer spec, feed-forward spec or None)
    source: dict             # the config.json it was read from

    @classmethod
    def from_dict(cls, c: dict) -> "BegupelConfig":
        r = Reader(c)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        norm = _sub(r, "norm")
        eps = norm.number("eps")
        if not eps > 0.0:
            raise ConfigError("norm.eps must be > 0")
        groups = norm.integer("groups", 1, minimum=1)
        if width % groups:
            raise ConfigError(f"norm.groups ({groups}) must divide width ({width})")
        taps = _sub(r, "canon").integer("taps", minimum=1)
        big = _sub(_sub(r, "embedding"), "bigram")
        pair = PairEmbeddingSpec(big.integer("buckets", minimum=1), big.integer("mul_prev"), big.integer("mul_cur"))
        cap = r.number("logit_softcap", None)
        if cap is not None and not cap > 0.0:
            raise ConfigError("logit_softcap must be > 0")
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = Reader(entry, f"layers[{i}]")
            kind = lr.string("type")
            m = _sub(lr, "mixer")
            if kind == "lightning":
                mixer = cls._lightning(m, width, eps)
            elif kind == "parallel":
                mixer = SideBySideSpec(cls._left(_sub(m, "left"), width, eps), cls._right(_sub(m, "right"), width, eps),
                                       m.number("left_scale"), m.number("right_scale"))
            else:
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (lightning, parallel)")
            f = _sub(lr, "mlp", required=False)
            layers.append((mixer, cls._ff(f, width) if f is not None else None))
        return cls(vocab, width, float(eps), groups, taps, pair, None if cap is None else float(cap), tuple(layers),
                   copy.deepcopy(c))

    @staticmethod
    def _lightning(m: Reader, width: int, eps: float) -> LightningAttentionSpec:
        heads = m.integer("heads", minimum=1)
        decay = m.raw("decay")
        if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"{m.where}: 'decay' must list one number per head ({heads})")
        return LightningAttentionSpec(width, heads, m.integer("dim", minimum=1), m.integer("vdim", minimum=1),
                                      tuple(float(d) for d in decay), eps)

    @staticmethod
    def _left(m: Reader, width: int, eps: float) -> AttentionSpec:
        heads, kv = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv:
            raise ConfigError(f"{m.where}: heads ({heads}) must be a multiple of kv_heads ({kv})")
        dim, vdim = m.integer("dim", minimum=1), m.integer("vdim", minimum=2)
        if vdim % 2:
            raise ConfigError(f"{m.where}: vdim ({vdim}) must be even: the values are turned in pairs")
        rot = _sub(m, "rot")
        dims = rot.integer("dims", minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{m.where}: rot.dims ({dims}) must be even and at most dim ({dim})")
        base = rot.number("base")
        sc = _sub(rot, "scaling", required=False)
        factor = sc.number("factor", 1.0) if sc is not None else 1.0
        if not factor > 0.0:
            raise ConfigError(f"{m.where}: rot.scaling.factor must be > 0")
        mask = _sub(m, "mask", required=False)
        return AttentionSpec(
            hidden_size=width, num_heads=heads, num_kv_heads=kv, head_dim=dim, scale=m.number("scale"),
            qk_norm=NormSpec(dim, eps), position=RotaryPairsSpec(dims, base, factor, PAIR_LAYOUT),
            window=mask.integer("size", minimum=1) if mask is not None else None,
            names=("q", "k", "v", "o", "sink"), value_dim=vdim, whole_qk_norm=True,
            value_rotation=RotaryPairsSpec(vdim, base, 1.0, PAIR_LAYOUT), norm_names=("q.norm", "k.norm"))

    @staticmethod
    def _right(m: Reader, width: int, eps: float) -> GatedDeltaSpec:
        heads, kv = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv:
            raise ConfigError(f"{m.where}: heads ({heads}) must be a multiple of kv_heads ({kv})")
        return GatedDeltaSpec(width, heads, kv, m.integer("dim", minimum=1), m.integer("vdim", minimum=1),
                              m.integer("conv", minimum=1), eps)

    @staticmethod
    def _ff(f: Reader, width: int):
        kind = f.string("kind")
        if kind == "dense":
            return SwiGLUSpec(width, f.integer("ff", minimum=1), activation=FF_ACTIVATION, names=("gate", "up", "down"),
                              bias=True, bias_suffix=".b")
        raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (dense)")

    def to_dict(self) -> dict:
        return copy.deepcopy(self.source)

    def model_spec(self) -> ModelSpec:
        def norm(name):
            return NormSpec(self.width, self.norm_eps, weight_name=name, groups=self.norm_groups)
        blocks = []
        for mixer, ff in self.layers:
            blocks.append(BlockSpec(
                mixer=mixer, ffn=ff, norm1=norm("norm1"), norm2=norm("norm2"), kind="sublayer_norm",
                input_conv_taps=self.canon_taps, input_conv_name="canon1",
                names=(("norm1", ""), ("mixer", "mix"), ("norm2", ""), ("ffn", "mlp"))))
        return ModelSpec(
            architecture="Begupel", vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=identity_schedule(len(blocks)), final_norm=norm("norm"),
            tie_word_embeddings=False, max_position=NO_POSITION_LIMIT, stop_token_ids=(),
            layer_prefix="l{i}.", embed_name="embed", final_norm_name="final.norm", head_name="head",
            pair_embedding=self.pair_embedding, logit_softcap=self.logit_softcap)
