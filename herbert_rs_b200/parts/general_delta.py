"""The generalised-delta-rule mixer: a float matrix of state per head with a decay per key channel, from which the
part along the token's unit key is removed, channel by channel at a learned rate, before k v^T is added.

    r, k, v = R h, K h, V h                                        ([H, n], [H, n], [H, nv])
    w = exp(-c * sigmoid(W2 tanh(W1 h) + w0)),  a = sigmoid(A h + a0)   one of each per head and key channel
    u = k / sqrt(sum k^2 + 1e-6)                                   per head
    S <- diag(w) S - (a * u) (u^T S) + k v^T                       both terms read the old S;   o = S^T r
    out = O ( o / rms_head(o) * nw * sigmoid(G h) )                nw: one number per head and value channel

The six products that read h are one matrix (rows r, k, v, g, a, W1) that leaves float sums; decays, rates, unit
keys, the state and the norm are float on both paths.  The state lives in the cache's fixed-size region of the
sequence's slot.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, StateNeed
from ..errors import WeightError
from ..registry import register_part
from .base import Mixer, ParamSpec

_NAMES = {"r": "r", "k": "k", "v": "v", "gate": "g", "rate": "a", "rate_bias": "a.b", "decay_down": "w1", "decay_up": "w2",
          "decay_bias": "w0", "norm": "norm", "out": "o"}


class GeneralDeltaMixer(Mixer):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dk, self.dv = spec.num_heads, spec.key_dim, spec.value_dim
        self.n = dict(_NAMES)
        self.n.update(dict(getattr(spec, "names", ()) or ()))

    def param_specs(self):
        s, n, H, dk, dv = self.spec, self.n, self.H, self.dk, self.dv
        return {
            n["r"]: ParamSpec((H * dk, s.hidden_size)),
            n["k"]: ParamSpec((H * dk, s.hidden_size)),
            n["v"]: ParamSpec((H * dv, s.hidden_size)),
            n["gate"]: ParamSpec((H * dv, s.hidden_size)),
            n["rate"]: ParamSpec((H * dk, s.hidden_size)),
            n["rate_bias"]: ParamSpec((H * dk,), role="vector", init="wide"),
            n["decay_down"]: ParamSpec((-1, s.hidden_size)),                  # the inner width is the stored tensor's
            n["decay_up"]: ParamSpec((H * dk, -1), init="wide"),
            n["decay_bias"]: ParamSpec((H * dk,), role="vector", init="wide"),
            n["norm"]: ParamSpec((H * dv,), role="vector", init="ones_noise"),
            n["out"]: ParamSpec((s.hidden_size, H * dv)),
        }

    def load(self, t):
        n = self.n
        if t[n["decay_down"]].shape[0] != t[n["decay_up"]].shape[1]:
            raise WeightError(f"{n['decay_down']} has {t[n['decay_down']].shape[0]} rows but {n['decay_up']} "
                              f"has {t[n['decay_up']].shape[1]} columns")
        self.w_in = torch.cat([t[n["r"]], t[n["k"]], t[n["v"]], t[n["gate"]], t[n["rate"]], t[n["decay_down"]]], dim=0).contiguous()
        self.w_decay = t[n["decay_up"]].contiguous()
        self.decay_bias, self.rate_bias = t[n["decay_bias"]].contiguous(), t[n["rate_bias"]].contiguous()
        self.norm = t[n["norm"]].contiguous()
        self.w_out = t[n["out"]].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_decay, self.w_out))

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.H, self.dk, self.dv), torch.float32))

    def forward(self, h, residual, batch, cache, accumulate=True):
        s, ws, T, H, dk, dv = self.spec, self.rt.workspace, h.shape[0], self.H, self.dk, self.dv
        f32 = torch.float32
        proj = ws.take((T, self.w_in.shape[0]), f32)
        ops.gemm(h, self.w_in, proj, ops.EPI_STORE_F32, scratch=ws.take)
        k_off, v_off, g_off = H * dk, 2 * H * dk, 2 * H * dk + H * dv
        a_off = g_off + H * dv
        low_off = a_off + H * dk
        prep = ws.take((T, H, 5, dk), f32)
        ops.general_delta_prepare(proj, 0, k_off, a_off, low_off, self.w_decay, self.decay_bias, self.rate_bias,
                                  s.decay_constant, s.unit_eps, prep, H, dk)
        o = ws.take((T, H * dv), f32)
        ops.general_delta_scan(prep, proj[:, v_off:g_off], cache.state, batch, o, H, dk, dv)
        y = ws.take((T, H * dv), h.dtype)
        ops.gated_rmsnorm(o, self.norm, s.norm_eps, proj[:, g_off:a_off], y, H, dv, sigmoid_gate=True)
        ops.gemm(y, self.w_out, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)


register_part("mixer", "general_delta", GeneralDeltaMixer)
