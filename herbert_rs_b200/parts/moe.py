"""The routed feed-forward: a router picks `top_k` of the experts for every token.

    s = softmax(R h) over all experts (float);  chosen: the top_k largest s
    out = sum over chosen e of w_e * Down_e act(Up_e h),   w_e = s_e (or s_e / sum of the chosen s)

The experts' matrices are stacked at load time ([E, F, D] and [E, D, F]) so that a kernel finds an
expert by its index; which experts a token uses never reaches the host, so a recorded step replays.

Options of the spec: sigmoid scores; groups of experts of which only the best stay open to the choice;
a factor on the weights; gated experts, out_e = Down_e (act(Gate_e h) * (Up_e h)), whose gate and up
rows are stored in one [E, 2F, D] stack, in turn in groups of 8 (the dense gated feed-forward's layout,
which the tensor-core products' epilogues read) or, where F is no multiple of 8, all gate rows first; a
shared dense feed-forward that every token passes and that is added to the experts' sum; a clamped gated
activation with a limit L, min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1).
"""

from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from ..registry import build_part, register_part
from .base import FeedForward, ParamSpec
from .swiglu import join_gate_up

SCORES = {"softmax": 0, "sigmoid": 1}


class RoutedFeedForward(FeedForward):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        if spec.activation not in ops.ACTIVATIONS:
            raise ConfigError(f"unknown activation {spec.activation!r}: {', '.join(ops.ACTIVATIONS)}")
        self.act = ops.ACTIVATIONS[spec.activation]
        self.act_limit = float(getattr(spec, "act_limit", 0.0))
        if self.act == ops.ACT_SWISH_CLAMP and not (spec.gated and self.act_limit > 0.0):
            raise ConfigError("the clamped activation is a gated expert's and needs its limit (> 0)")
        if spec.score not in SCORES:
            raise ConfigError(f"unknown router score {spec.score!r}: {', '.join(SCORES)}")
        if len(spec.expert_names) != (3 if spec.gated else 2):
            raise ConfigError("a gated expert has three tensors (gate, up, down), a plain one two (up, down)")
        if spec.groups < 1 or spec.num_experts % spec.groups or not (1 <= spec.keep_groups <= spec.groups):
            raise ConfigError(f"{spec.num_experts} experts cannot form {spec.groups} equal groups of which {spec.keep_groups} stay")
        if spec.top_k > spec.keep_groups * (spec.num_experts // spec.groups):
            raise ConfigError(f"top_k ({spec.top_k}) exceeds the experts of the {spec.keep_groups} kept groups")
        self.shared = build_part("ffn", spec.shared, rt=rt) if spec.shared is not None else None
        if self.shared is not None and not self.shared.can_store:
            raise ConfigError("the shared feed-forward must be able to add into a given array")

    def _names(self, e):
        return tuple(n.format(e=e) for n in self.spec.expert_names)

    def param_specs(self):
        s = self.spec
        # random sigmoid routers stay small: wide logits would all score exactly 1 and tie
        p = {s.router_name: ParamSpec((s.num_experts, s.hidden_size), init="wide" if s.score == "softmax" else "normal")}
        for e in range(s.num_experts):
            names = self._names(e)
            for n in names[:-1]:
                p[n] = ParamSpec((s.expert_size, s.hidden_size))
            p[names[-1]] = ParamSpec((s.hidden_size, s.expert_size))
        if self.shared is not None:
            p.update(self.shared.param_specs())
        return p

    def load(self, t):
        s = self.spec
        self.router = t[s.router_name].contiguous()
        self.gated = 0
        if s.gated:
            joined = [join_gate_up(t[self._names(e)[0]], t[self._names(e)[1]]) for e in range(s.num_experts)]
            self.up = torch.stack([j[0] for j in joined]).contiguous()
            self.gated = ops.GATED_GROUPS_OF_8 if joined[0][1] else ops.GATED_HALVES
        else:
            self.up = torch.stack([t[self._names(e)[0]] for e in range(s.num_experts)]).contiguous()
        self.down = torch.stack([t[self._names(e)[-1]] for e in range(s.num_experts)]).contiguous()
        if self.shared is not None:
            self.shared.load({n: t[n] for n in self.shared.param_specs()})

    def weight_bytes(self):
        """What a step of one token reads: the router, top_k experts and the shared feed-forward."""
        s = self.spec
        per = (3 if s.gated else 2) * s.expert_size * s.hidden_size * self.up.element_size()
        shared = self.shared.weight_bytes() if self.shared is not None else 0
        return self.router.numel() * self.router.element_size() + s.top_k * per + shared

    def forward(self, h, residual, batch, accumulate=True):
        s, ws, T = self.spec, self.rt.workspace, h.shape[0]
        ids = ws.take((T, s.top_k), torch.int32)
        weights = ws.take((T, s.top_k), torch.float32)
        ops.moe_route(h, self.router, ids, weights, s.top_k, s.renormalize, SCORES[s.score], s.groups, s.keep_groups,
                      s.group_top, s.weight_scale)
        if ops.moe_tc_ok(h, self.up, s.top_k, self.gated, self.act):
            ops.moe_experts_tc(h, self.up, self.down, ids, weights, residual, accumulate, ws.take,
                               act_limit=self.act_limit if self.act == ops.ACT_SWISH_CLAMP else 0.0)
        elif ops.moe_grouped_ok(h, self.up, self.gated):
            ops.moe_experts_grouped(h, self.up, self.down, ids, weights, residual, self.act, accumulate, ws.take, gated=self.gated,
                                    act_limit=self.act_limit)
        else:
            mid = ws.take((T * s.top_k, s.expert_size), h.dtype)
            ops.moe_experts(h, self.up, self.down, ids, weights, mid, residual, self.act, accumulate, gated=self.gated,
                            act_limit=self.act_limit)
        if self.shared is not None:
            self.shared.forward(h, residual, batch, accumulate=True)


register_part("ffn", "moe", RoutedFeedForward)
