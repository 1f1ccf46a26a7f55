"""The gated-delta-rule mixer: a float matrix of state per head that is decayed, corrected toward the
token's value along its key, and read with the query.

    q, k = silu(conv(Wq h)), silu(conv(Wk h))   ([G, dk], G query/key heads);   v = silu(conv(Wv h))   ([H, dv])
    q <- q / sqrt(sum q^2 + 1e-6) * dk^-1/2,  k <- k / sqrt(sum k^2 + 1e-6)      per head
    beta = sigmoid(Wb h),  g = exp(-exp(A_log) * softplus(Wa h + dt_bias))       one of each per head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                 head h reads q/k head h / (H / G)
    out = Wo ( RMSNorm_head(o) * w * silu(Wg h) )                                w: dv numbers for all heads

conv is a short causal convolution over time on each channel whose last taps - 1 inputs are kept per
sequence, beside the state matrix, in the cache's fixed-size region of the sequence's slot.  The six
products that read h are one matrix (rows q, k, v, g, b, a) that leaves float sums.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, StateNeed
from ..errors import ConfigError
from ..registry import register_part
from .base import Mixer, ParamSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "beta": "b", "step": "a", "out": "o", "norm": "norm",
          "A_log": "A_log", "dt_bias": "dt_bias", "conv_suffix": ".conv"}


class GatedDeltaMixer(Mixer):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.H, self.G, self.dk, self.dv, self.taps = spec.num_heads, spec.qk_heads, spec.key_dim, spec.value_dim, spec.conv_taps
        if self.H % self.G:
            raise ConfigError(f"{self.H} heads are no multiple of {self.G} query/key heads")
        if self.taps < 1:
            raise ConfigError("a convolution has at least one tap")
        self.n = dict(_NAMES)
        self.n.update(dict(getattr(spec, "names", ()) or ()))
        self.conv_channels = 2 * self.G * self.dk + self.H * self.dv

    def param_specs(self):
        s, n, H, G, dk, dv = self.spec, self.n, self.H, self.G, self.dk, self.dv
        c = n["conv_suffix"]
        return {
            n["q"]: ParamSpec((G * dk, s.hidden_size)),
            n["k"]: ParamSpec((G * dk, s.hidden_size)),
            n["v"]: ParamSpec((H * dv, s.hidden_size)),
            n["q"] + c: ParamSpec((G * dk, self.taps), role="vector", init="wide"),
            n["k"] + c: ParamSpec((G * dk, self.taps), role="vector", init="wide"),
            n["v"] + c: ParamSpec((H * dv, self.taps), role="vector", init="wide"),
            n["gate"]: ParamSpec((H * dv, s.hidden_size)),
            n["beta"]: ParamSpec((H, s.hidden_size)),
            n["step"]: ParamSpec((H, s.hidden_size)),
            n["A_log"]: ParamSpec((H,), role="vector", init="zeros_noise"),
            n["dt_bias"]: ParamSpec((H,), role="vector", init="wide"),
            n["norm"]: ParamSpec((dv,), role="vector", init="ones_noise"),
            n["out"]: ParamSpec((s.hidden_size, H * dv)),
        }

    def load(self, t):
        n = self.n
        c = n["conv_suffix"]
        self.w_in = torch.cat([t[n["q"]], t[n["k"]], t[n["v"]], t[n["gate"]], t[n["beta"]], t[n["step"]]], dim=0).contiguous()
        self.w_conv = torch.cat([t[n["q"] + c], t[n["k"] + c], t[n["v"] + c]], dim=0).contiguous()
        self.a_log, self.dt_bias = t[n["A_log"]].contiguous(), t[n["dt_bias"]].contiguous()
        self.norm = t[n["norm"]].contiguous()
        self.w_out = t[n["out"]].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_conv, self.w_out))

    def cache_need(self):
        states = ()
        if self.taps > 1:
            states = (("conv", StateNeed((self.taps - 1, self.conv_channels), torch.float32)),)
        return CacheNeed(state=StateNeed((self.H, self.dk, self.dv), torch.float32), states=states)

    def forward(self, h, residual, batch, cache, accumulate=True):
        s, ws, T, H, G, dk, dv = self.spec, self.rt.workspace, h.shape[0], self.H, self.G, self.dk, self.dv
        f32 = torch.float32
        proj = ws.take((T, self.w_in.shape[0]), f32)
        ops.gemm(h, self.w_in, proj, ops.EPI_STORE_F32, scratch=ws.take)
        C = self.conv_channels
        k_off, v_off, g_off, b_off, a_off = G * dk, 2 * G * dk, C, C + H * dv, C + H * dv + H
        qkv = ws.take((T, C), f32)
        ops.short_conv(proj[:, :C], self.w_conv, cache.states.get("conv"), batch, qkv, add_input=False, silu=True)
        gates = ws.take((T, 2 * H), f32)
        ops.delta_prepare(qkv, 0, k_off, G, dk, dk ** -0.5, proj, b_off, a_off, self.a_log, self.dt_bias, gates, H)
        o = ws.take((T, H * dv), f32)
        ops.linear_scan(qkv[:, :k_off], qkv[:, k_off:v_off], qkv[:, v_off:], cache.state, batch, o, H, G, dk, dv, gates=gates)
        y = ws.take((T, H * dv), h.dtype)
        ops.gated_rmsnorm(o, self.norm, s.norm_eps, proj[:, g_off:b_off], y, H, dv, sigmoid_gate=False)
        ops.gemm(y, self.w_out, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)


register_part("mixer", "gated_delta", GatedDeltaMixer)
