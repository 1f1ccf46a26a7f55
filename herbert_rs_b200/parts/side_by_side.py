"""Two mixers side by side: both read the same input, and the result is a * left(h) + b * right(h) with two
constants.  Each keeps what it needs in the cache: the step's keys and values belong to the one that asks for
them (at most one may), and the fixed-size states of the right one live under a prefix of their own."""

from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from ..registry import build_part, register_part
from .base import Mixer

_RIGHT = "right."


class SideBySideMixer(Mixer):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.left = build_part("mixer", spec.left, rt=rt)
        self.right = build_part("mixer", spec.right, rt=rt)
        self.a, self.b = float(spec.left_scale), float(spec.right_scale)
        self.prefixes = tuple(spec.names)
        for part in (self.left, self.right):
            if not part.can_store:
                raise ConfigError(f"{type(part).__name__} cannot store its result apart from the residual stream, "
                                  "which a mixer beside another needs")

    @property
    def graph_safe(self):
        return self.left.graph_safe and self.right.graph_safe

    def children(self):
        return ((self.prefixes[0], self.left), (self.prefixes[1], self.right))

    def param_specs(self):
        return {f"{pre}.{name}": ps for pre, part in self.children() for name, ps in part.param_specs().items()}

    def load(self, tensors):
        for pre, part in self.children():
            part.load({name: tensors[f"{pre}.{name}"] for name in part.param_specs()})

    def weight_bytes(self):
        return self.left.weight_bytes() + self.right.weight_bytes()

    def cache_need(self):
        return self.left.cache_need().merged(self.right.cache_need(), _RIGHT)

    def forward_parts(self, h, y, batch, cache):
        """Both results apart: the left one into y, the right one into a float array z that is returned with the two
        constants, for a caller whose next kernel can take a * y + b * z as its input (a block that norms the sum)."""
        self.left.forward(h, y, batch, cache, accumulate=False)
        z = self.rt.workspace.take(y.shape, torch.float32)
        self.right.forward(h, z, batch, cache.sub(_RIGHT), accumulate=False)
        return z, self.a, self.b

    def forward(self, h, residual, batch, cache, accumulate=True):
        ws = self.rt.workspace
        y = residual if not accumulate else ws.take(residual.shape, torch.float32)
        self.left.forward(h, y, batch, cache, accumulate=False)
        z = ws.take(residual.shape, torch.float32)
        self.right.forward(h, z, batch, cache.sub(_RIGHT), accumulate=False)
        ops.axpby(y, self.a, z, self.b)
        if accumulate:
            ops.add_residual(residual, y)


register_part("mixer", "side_by_side", SideBySideMixer)
