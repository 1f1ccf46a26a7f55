"""Models: the generic decoder, and the architectures registered for it."""

from ..config.begupel import BegupelConfig
from ..config.kebisun import KebisunConfig
from ..config.nefivik import NefivikConfig
from ..config.qwen3 import Qwen3Config
from ..config.votapel import VotapelConfig
from ..registry import register_architecture
from .decoder import DecoderModel

# "qwen3" is the reference's family key (crates/core/src/config.rs:93-103).
register_architecture("Qwen3ForCausalLM", Qwen3Config, model_types=("qwen3",), default=True)
# Layers of two mixer kinds (latent attention, gated linear attention) with dense or routed
# feed-forwards; config.json names it under "architecture".
register_architecture("Kebisun", KebisunConfig)
# Parallel blocks (one norm, attention and a routed feed-forward side by side) of attention whose values
# are its keys, with biases, a query temperature, capped scores and a sink; learned position vectors.
register_architecture("Votapel", VotapelConfig)
# Layers of lightning attention (a decaying matrix state per head) and of windowed attention with rotated
# values beside a gated delta rule; an input convolution per layer, RMS norms in groups on the sublayers'
# results, a pair embedding, capped logits.
register_architecture("Begupel", BegupelConfig)
# Layers of sigmoid-weighted windowed attention (convolved projections, a gate per head, keys and values that a
# later layer may read) and of a generalised delta rule, each sublayer between two norms and behind a gate; routed
# experts in groups with a clamped activation; a second input by token id at every layer's end.
register_architecture("Nefivik", NefivikConfig)

__all__ = ["DecoderModel"]
