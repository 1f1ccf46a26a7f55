"""The dense gated feed-forward: down( act(gate(h)) * up(h) ), added to the residual stream
(crates/backends/backend_common/src/generic_mlp.rs:83-96; silu(x) = x / (1 + exp(-x)),
kernels.rs:677-687).  act is silu unless the spec names another (gelu in its tanh or erf form, relu); the
product's fused epilogue serves silu, the others take the product and then the activation kernel.
With `bias` every projection adds a stored vector: gate and up leave float sums, one kernel adds their
biases, applies the activation and rounds once; the down projection's bias is added to the float result,
or handed to a block that norms that result (`take_output_bias`), which adds it while it reads.

gate_proj and up_proj are one matrix here.  When the intermediate size is a multiple of 8
their rows alternate in groups of 8 (8 gate rows, the 8 up rows of the same channels, ...), so
that a kernel holding 16 consecutive output columns has both halves of 8 channels; otherwise
the up rows follow all gate rows.
"""

from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from ..registry import register_part
from .base import FeedForward, ParamSpec

INTERLEAVE = 8


def join_gate_up(gate: torch.Tensor, up: torch.Tensor):
    inter, hidden = gate.shape
    if inter % INTERLEAVE == 0:
        g = gate.view(inter // INTERLEAVE, INTERLEAVE, hidden)
        u = up.view(inter // INTERLEAVE, INTERLEAVE, hidden)
        return torch.cat([g, u], dim=1).reshape(2 * inter, hidden).contiguous(), INTERLEAVE
    return torch.cat([gate, up], dim=0).contiguous(), 0


class SwiGLU(FeedForward):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.wgu = self.wd = None
        self.interleave = 0
        self.names = tuple(getattr(spec, "names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        act = getattr(spec, "activation", "silu")
        if act not in ops.ACTIVATIONS:
            raise ConfigError(f"unknown activation {act!r}: {', '.join(ops.ACTIVATIONS)}")
        self.act = ops.ACTIVATIONS[act]
        self.bias = bool(getattr(spec, "bias", False))
        self.bias_suffix = getattr(spec, "bias_suffix", ".b")
        self.bgu = self.bd = None
        # the fused kernels and the shared norm serve the form without biases
        self.shares_norms = not self.bias

    def param_specs(self):
        s, (gate, up, down) = self.spec, self.names
        p = {
            gate: ParamSpec((s.intermediate_size, s.hidden_size)),
            up: ParamSpec((s.intermediate_size, s.hidden_size)),
            down: ParamSpec((s.hidden_size, s.intermediate_size)),
        }
        if self.bias:
            for n in (gate, up, down):
                p[n + self.bias_suffix] = ParamSpec((p[n].shape[0],), role="vector", init="normal")
        return p

    def load(self, tensors):
        gate, up, down = self.names
        self.wgu, self.interleave = join_gate_up(tensors[gate], tensors[up])
        self.wd = tensors[down].contiguous()
        if self.bias:
            sfx = self.bias_suffix
            self.bgu, _ = join_gate_up(tensors[gate + sfx].view(-1, 1), tensors[up + sfx].view(-1, 1))
            self.bgu = self.bgu.view(-1).contiguous()
            self.bd = tensors[down + sfx].contiguous()

    def take_output_bias(self):
        """The down projection's bias, for a caller that adds it itself right after forward(accumulate=False,
        with_output_bias=False); None if there is none."""
        return self.bd

    def weight_bytes(self):
        return (self.wgu.numel() + self.wd.numel()) * self.wgu.element_size()

    shares_norms = True
    can_store = True

    def _forward_bias(self, h, residual, accumulate, with_output_bias):
        ws, T, inter = self.rt.workspace, h.shape[0], self.spec.intermediate_size
        gu = ws.take((T, 2 * inter), torch.float32)
        ops.gemm(h, self.wgu, gu, ops.EPI_STORE_F32, scratch=ws.take)
        act = ws.take((T, inter), self.rt.dtype)
        ops.bias_glu(gu, self.bgu, act, self.interleave, self.act)
        if accumulate:
            ops.gemm(act, self.wd, residual, ops.EPI_RESIDUAL, scratch=ws.take)
        else:
            ops.gemm(act, self.wd, residual, ops.EPI_STORE_F32, scratch=ws.take)
        if with_output_bias:
            ops.add_row_bias(residual, self.bd)
        return None

    def forward(self, h, residual, batch, next_norm=None, accumulate=True, with_output_bias=True):
        if self.bias:
            return self._forward_bias(h, residual, accumulate, with_output_bias)
        ws, T, inter = self.rt.workspace, h.shape[0], self.spec.intermediate_size
        act = ws.take((T, inter), self.rt.dtype)
        if self.act == ops.ACT_SILU:
            ops.gemm_swiglu(h, self.wgu, act, self.interleave, ws.take)
        else:
            gu = ws.take((T, 2 * inter), self.rt.dtype)
            ops.gemm(h, self.wgu, gu, scratch=ws.take)
            ops.swiglu(gu, act, self.interleave, self.act)
        if not accumulate:
            return ops.gemm(act, self.wd, residual, ops.EPI_STORE_F32, scratch=ws.take)
        return ops.gemm(act, self.wd, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)


register_part("ffn", "swiglu", SwiGLU)
