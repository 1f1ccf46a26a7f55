"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, in float
(crates/backends/backend_common/src/kernels.rs:54-64), and the layer norm with a weight and no bias.
A spec with `weight_offset` c stores w - c (weights around zero with c = 1); the offset is added once,
in float, when the tensor is loaded, so every kernel and the norm shared between two products see w."""

from __future__ import annotations

from .. import ops
from ..errors import ConfigError
from ..registry import register_part
from .base import Norm, ParamSpec


class RMSNorm(Norm):
    kind = "rmsnorm"

    def __init__(self, spec, rt):
        self.dim, self.eps, self.rt = spec.dim, spec.eps, rt
        self.name = getattr(spec, "weight_name", "weight")
        self.offset = float(getattr(spec, "weight_offset", 0.0))
        self.groups = int(getattr(spec, "groups", 1))
        if self.groups < 1 or self.dim % self.groups:
            raise ConfigError(f"a norm over {self.dim} channels cannot be cut into {self.groups} equal parts")
        self.weight = None

    def param_specs(self):
        # random weights lie around 1 - offset: the factor the kernels see is around 1 either way
        return {self.name: ParamSpec((self.dim,), role="vector", init="ones_noise" if self.offset == 0.0 else "zeros_noise")}

    def load(self, tensors):
        w = tensors[self.name]
        self.weight = (w + self.offset if self.offset != 0.0 else w).contiguous()

    def weight_bytes(self):
        return self.dim * 4

    def forward(self, x, out, rows=None):
        if self.groups > 1:
            ops.group_rmsnorm(x, self.weight, out, self.eps, self.groups, rows)
        else:
            ops.rmsnorm(x, self.weight, out, self.eps, rows)

    def shareable(self):
        return (self.weight, self.eps) if self.groups == 1 else None


class LayerNorm(RMSNorm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w, no bias, in float (var: mean of squared deviations)."""

    kind = "layernorm"

    def forward(self, x, out, rows=None):
        ops.layernorm(x, self.weight, out, self.eps, rows)

    def shareable(self):
        return None         # the products' shared norm is the RMS form only


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
