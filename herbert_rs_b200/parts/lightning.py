"""The lightning-attention mixer: linear attention with a float matrix of state per head and one constant
decay per head.

    q = silu(Wq h), k = silu(Wk h)  ([H, dk]);   v = silu(Wv h)  ([H, dv])
    S_t = d_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t           per head, S starts at zero, no other scale
    out = Wo ( RMSNorm(concat_h o_h) * w * sigmoid(Wg h) )     one norm over all heads, w of H dv numbers

The state is the cache's fixed-size region of the sequence's slot ([H, dk, dv] floats, zeroed when the slot is
handed out); every step continues from it, whatever the prompt was cut into.  The four products that read h
are one matrix (rows q, k, v, g) whose float sums feed the activations, the recurrence and the gate.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, StateNeed
from ..errors import ConfigError
from ..registry import register_part
from .base import Mixer, ParamSpec


class LightningMixer(Mixer):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dk, self.dv = spec.num_heads, spec.key_dim, spec.value_dim
        if len(spec.decay) != self.H:
            raise ConfigError(f"{len(spec.decay)} decays for {self.H} heads")
        self.n_q, self.n_k, self.n_v, self.n_g, self.n_o, self.n_norm = spec.names
        self.decay = torch.tensor([float(d) for d in spec.decay], dtype=torch.float32).to(rt.device)

    def param_specs(self):
        s, H = self.spec, self.H
        return {
            self.n_q: ParamSpec((H * self.dk, s.hidden_size)),
            self.n_k: ParamSpec((H * self.dk, s.hidden_size)),
            self.n_v: ParamSpec((H * self.dv, s.hidden_size)),
            self.n_g: ParamSpec((H * self.dv, s.hidden_size)),
            self.n_o: ParamSpec((s.hidden_size, H * self.dv)),
            self.n_norm: ParamSpec((H * self.dv,), role="vector", init="ones_noise"),
        }

    def load(self, t):
        self.w_in = torch.cat([t[self.n_q], t[self.n_k], t[self.n_v], t[self.n_g]], dim=0).contiguous()
        self.norm = t[self.n_norm].contiguous()
        self.w_out = t[self.n_o].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_out))

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.H, self.dk, self.dv), torch.float32))

    def forward(self, h, residual, batch, cache, accumulate=True):
        ws, T, H, dk, dv = self.rt.workspace, h.shape[0], self.H, self.dk, self.dv
        proj = ws.take((T, self.w_in.shape[0]), torch.float32)
        ops.gemm(h, self.w_in, proj, ops.EPI_STORE_F32, scratch=ws.take)
        k_off, v_off, g_off = H * dk, 2 * H * dk, 2 * H * dk + H * dv
        ops.silu_columns(proj, 0, g_off)
        o = ws.take((T, H * dv), torch.float32)
        ops.linear_scan(proj[:, :k_off], proj[:, k_off:v_off], proj[:, v_off:g_off], cache.state, batch, o, H, H, dk, dv,
                        decay=self.decay)
        y = ws.take((T, H * dv), h.dtype)
        ops.gated_rmsnorm(o, self.norm, self.spec.norm_eps, proj[:, g_off:], y, 1, H * dv, sigmoid_gate=True)
        ops.gemm(y, self.w_out, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)


register_part("mixer", "lightning", LightningMixer)
