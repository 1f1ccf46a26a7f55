"""The pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(crates/backends/backend_common/src/generic_layer.rs:1131-1328)."""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, StateNeed
from ..errors import ConfigError
from ..registry import build_part, register_part
from .base import Block, ParamSpec


class PreNormBlock(Block):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.norm1 = build_part("norm", spec.norm1, rt=rt)
        self.mixer = build_part("mixer", spec.mixer, rt=rt)
        self.norm2 = build_part("norm", spec.norm2, rt=rt)
        self.ffn = build_part("ffn", spec.ffn, rt=rt)
        self._names = dict(spec.names)

    @property
    def graph_safe(self):
        return all(p.graph_safe for _, p in self.children())

    def children(self):
        return (("norm1", self.norm1), ("mixer", self.mixer), ("norm2", self.norm2), ("ffn", self.ffn))

    def param_specs(self):
        out = {}
        for local, part in self.children():
            for name, ps in part.param_specs().items():
                out[f"{self._names[local]}.{name}"] = ps
        return out

    def load(self, tensors):
        for local, part in self.children():
            prefix = self._names[local] + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def weight_bytes(self):
        return sum(p.weight_bytes() for _, p in self.children())

    def cache_need(self):
        return self.mixer.cache_need()

    chains_norms = True

    def first_norm(self):
        return self.norm1

    def _input(self, pending, norm, part, x):
        """What `part` reads: the pending norm itself if it can finish it, else the plain result."""
        if isinstance(pending, torch.Tensor):
            return pending              # the block before has already run this norm to its end
        if pending is not None and part.shares_norms:
            return pending
        h = self.rt.workspace.take(x.shape, self.rt.dtype)
        if pending is not None:
            ops.finish_norm(pending, h)
        else:
            norm.forward(x, h)
        return h

    def forward(self, x, batch, cache, normed=None, next_norm=None):
        share = ops.shared_norm_ok(x.shape[0], self.rt.dtype, x.shape[1])
        h = self._input(normed, self.norm1, self.mixer, x)
        mid = self.norm2.shareable() if share and self.mixer.shares_norms else None
        if self.mixer.shares_norms:
            pending = self.mixer.forward(h, x, batch, cache, next_norm=mid)
        else:
            pending = self.mixer.forward(h, x, batch, cache)
        h2 = self._input(pending, self.norm2, self.ffn, x)
        if self.ffn.shares_norms:
            return self.ffn.forward(h2, x, batch, next_norm=next_norm if share else None)
        self.ffn.forward(h2, x, batch)
        return None


class SublayerNormBlock(Block):
    """x += s1 * norm1(mixer(x)); x += s2 * norm2(ffn(x)): the sublayers read the residual stream
    itself (its rounding to the activation dtype on the bfloat16 path), their results are normed (a
    layer norm, or an RMS norm in groups) and multiplied channel by channel by a stored scale before
    they join the stream.  The spec may leave out the scales (`layer_scale` None) and the feed-forward
    (`ffn` None).  Norm, scale and sum are one kernel, which also hands the next sublayer its input.
    With `input_conv_taps` the mixer reads x + conv(x), a causal convolution over time on each channel
    of the stream; the stream's rows of the last taps - 1 positions are kept per sequence in the cache's
    fixed-size region (named "input_conv"), so a step continues where the one before ended."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.norm1 = build_part("norm", spec.norm1, rt=rt)
        self.mixer = build_part("mixer", spec.mixer, rt=rt)
        self.ffn = build_part("ffn", spec.ffn, rt=rt) if spec.ffn is not None else None
        self.norm2 = build_part("norm", spec.norm2, rt=rt) if self.ffn is not None else None
        self._names = dict(spec.names)
        self.scale_names = tuple(spec.layer_scale) if spec.layer_scale else None
        self.scale1 = self.scale2 = None
        for part in (self.mixer, self.ffn):
            if part is not None and not part.can_store:
                raise ConfigError(f"{type(part).__name__} cannot store its result apart from the residual stream, "
                                  "which a block that norms a sublayer's result needs")
        for norm in (spec.norm1, spec.norm2) if self.ffn is not None else (spec.norm1,):
            if norm.kind not in ("layernorm", "rmsnorm"):
                raise ConfigError("the block that norms a sublayer's result applies a layer norm or an RMS norm")
            if norm.kind == "rmsnorm" and (self.scale_names or norm.weight_offset):
                raise ConfigError("the RMS norm of a sublayer's result has no channel scales and no weight offset")
        self.taps = int(spec.input_conv_taps) if spec.input_conv_taps else 0
        self.conv_name = spec.input_conv_name
        self.conv_w = None

    @property
    def graph_safe(self):
        return all(p.graph_safe for _, p in self.children())

    def children(self):
        parts = [("norm1", self.norm1), ("mixer", self.mixer)]
        if self.ffn is not None:
            parts += [("norm2", self.norm2), ("ffn", self.ffn)]
        return tuple(parts)

    def _key(self, local, name):
        prefix = self._names[local]
        return f"{prefix}.{name}" if prefix else name

    def param_specs(self):
        out = {}
        for local, part in self.children():
            for name, ps in part.param_specs().items():
                out[self._key(local, name)] = ps
        if self.scale_names:
            dim = self.spec.norm1.dim
            out[self.scale_names[0]] = ParamSpec((dim,), role="vector", init="ones_noise")
            if self.ffn is not None:
                out[self.scale_names[1]] = ParamSpec((dim,), role="vector", init="ones_noise")
        if self.taps:
            out[self.conv_name] = ParamSpec((self.spec.norm1.dim, self.taps), role="vector", init="normal")
        return out

    def load(self, tensors):
        for local, part in self.children():
            part.load({name: tensors[self._key(local, name)] for name in part.param_specs()})
        if self.scale_names:
            self.scale1 = tensors[self.scale_names[0]].contiguous()
            if self.ffn is not None:
                self.scale2 = tensors[self.scale_names[1]].contiguous()
        if self.taps:
            self.conv_w = tensors[self.conv_name].contiguous()

    def weight_bytes(self):
        return sum(p.weight_bytes() for _, p in self.children()) + (8 * self.spec.norm1.dim if self.scale_names else 0)

    def cache_need(self):
        need = self.mixer.cache_need()
        if self.taps > 1:
            conv = StateNeed((self.taps - 1, self.spec.norm1.dim), torch.float32)
            need = CacheNeed(need.kv, need.state, need.states + (("input_conv", conv),))
        return need

    def _join(self, y, norm, scale, x, h, bias=None, second=None):
        """x += norm(y + bias) (* scale); h, if given, receives the new x in the activation dtype.  `second` = (z, a, b):
        the normed vector is a * y + b * z (an RMS norm takes the sum of two mixers side by side in the same pass)."""
        if norm.kind == "rmsnorm":
            ops.group_rmsnorm_residual(y, norm.weight, x, h, norm.eps, norm.groups, self.rt.dtype, bias=bias, second=second)
            return
        if second is not None:
            ops.axpby(y, second[1], second[0], second[2])
        if bias is not None:
            ops.add_row_bias(y, bias)
        ops.layernorm_residual(y, norm.weight, scale, x, h, norm.eps, self.rt.dtype)

    def forward(self, x, batch, cache, normed=None, next_norm=None):
        ws, dtype = self.rt.workspace, self.rt.dtype
        wide = dtype == torch.float32
        if self.taps:
            h = ws.take(x.shape, dtype)
            ops.short_conv(x, self.conv_w, cache.states.get("input_conv"), batch, h, add_input=True)
        elif wide:
            h = x
        else:
            h = ws.take(x.shape, dtype)
            ops.to_activation(x, h)
        y = ws.take(x.shape, torch.float32)
        second = None
        if getattr(self.mixer, "forward_parts", None) is not None:
            second = self.mixer.forward_parts(h, y, batch, cache)
        else:
            self.mixer.forward(h, y, batch, cache, accumulate=False)
        h2 = None if (wide or self.ffn is None) else ws.take(x.shape, dtype)
        self._join(y, self.norm1, self.scale1, x, h2, second=second)
        if self.ffn is not None:
            bias = None
            if getattr(self.ffn, "take_output_bias", None) is not None and self.ffn.take_output_bias() is not None:
                bias = self.ffn.take_output_bias()
                self.ffn.forward(x if wide else h2, y, batch, accumulate=False, with_output_bias=False)
            else:
                self.ffn.forward(x if wide else h2, y, batch, accumulate=False)
            self._join(y, self.norm2, self.scale2, x, None, bias=bias)
        return None


class ParallelBlock(Block):
    """h = norm1(x); x += m * (mixer(h) + ffn(h)): one norm whose result both sublayers read, one
    factor m on their sum.  The sublayers write into one float array (the mixer stores, the
    feed-forward adds), and one kernel adds it, times m, to the stream and runs the RMS norm the next
    block begins with, so that between two layers the stream is read and written once.  The spec may
    leave out the feed-forward."""

    chains_norms = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.norm1 = build_part("norm", spec.norm1, rt=rt)
        self.mixer = build_part("mixer", spec.mixer, rt=rt)
        self.ffn = build_part("ffn", spec.ffn, rt=rt) if spec.ffn is not None else None
        self.mult = float(spec.residual_mult)
        self._names = dict(spec.names)
        for part in (self.mixer, self.ffn):
            if part is not None and not part.can_store:
                raise ConfigError(f"{type(part).__name__} cannot store its result apart from the residual stream, "
                                  "which a block that adds both sublayers at once needs")

    @property
    def graph_safe(self):
        return all(p.graph_safe for _, p in self.children())

    def children(self):
        parts = [("norm1", self.norm1), ("mixer", self.mixer)]
        if self.ffn is not None:
            parts.append(("ffn", self.ffn))
        return tuple(parts)

    def _key(self, local, name):
        prefix = self._names[local]
        return f"{prefix}.{name}" if prefix else name

    def param_specs(self):
        return {self._key(local, name): ps for local, part in self.children() for name, ps in part.param_specs().items()}

    def load(self, tensors):
        for local, part in self.children():
            part.load({name: tensors[self._key(local, name)] for name in part.param_specs()})

    def weight_bytes(self):
        return sum(p.weight_bytes() for _, p in self.children())

    def cache_need(self):
        return self.mixer.cache_need()

    def first_norm(self):
        return self.norm1

    def forward(self, x, batch, cache, normed=None, next_norm=None):
        ws, dtype = self.rt.workspace, self.rt.dtype
        if isinstance(normed, torch.Tensor):
            h = normed
        else:
            h = ws.take(x.shape, dtype)
            if normed is not None:
                ops.finish_norm(normed, h)
            else:
                self.norm1.forward(x, h)
        y = ws.take(x.shape, torch.float32)
        self.mixer.forward(h, y, batch, cache, accumulate=False)
        if self.ffn is not None:
            self.ffn.forward(h, y, batch, accumulate=True)
        if next_norm is None:
            ops.scaled_residual_norm(y, self.mult, x)
            return None
        h_next = ws.take(x.shape, dtype)
        ops.scaled_residual_norm(y, self.mult, x, next_norm[0], h_next, next_norm[1])
        return h_next


class SandwichBlock(Block):
    """A norm before and after each sublayer, and a gate on each result:

        h = norm1(x);  x += post1( mixer(h) * sigmoid(R1 h + b1) )
        h = norm2(x);  x += post2( ffn(h)   * sigmoid(R2 h + b2) )
        e = table[token][column0 : column0 + m];  y = P (gelu_tanh(G x) * e);  x += y / sqrt(mean(y^2) + eps) * w

    The gates are optional (`BlockSpec.residual_gates`), so are the feed-forward and the last line (`token_side`: a
    second input that the token's id chooses from a table of the model's, this layer its own columns of it).
    A sublayer stores its result as floats; gate, norm of the result, the sum and the norm that the next sublayer (or
    the next block) begins with are one kernel, so that between two sublayers the stream is read and written once."""

    chains_norms = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.norm1 = build_part("norm", spec.norm1, rt=rt)
        self.mixer = build_part("mixer", spec.mixer, rt=rt)
        self.ffn = build_part("ffn", spec.ffn, rt=rt) if spec.ffn is not None else None
        self.norm2 = build_part("norm", spec.norm2, rt=rt) if self.ffn is not None else None
        if not spec.post_norms or len(spec.post_norms) != 2:
            raise ConfigError("a block with a norm before and after each sublayer needs the two norms of the results")
        self.post1 = build_part("norm", spec.post_norms[0], rt=rt)
        self.post2 = build_part("norm", spec.post_norms[1], rt=rt) if self.ffn is not None else None
        for norm in (self.norm1, self.norm2, self.post1, self.post2):
            if norm is not None and norm.shareable() is None:
                raise ConfigError("the block with a norm before and after each sublayer applies plain RMS norms")
        for part in (self.mixer, self.ffn):
            if part is not None and not part.can_store:
                raise ConfigError(f"{type(part).__name__} cannot store its result apart from the residual stream, "
                                  "which a block that norms a sublayer's result needs")
        self._names = dict(spec.names)
        self.gate_names = tuple(spec.residual_gates) if spec.residual_gates else None
        self.gate_bias_suffix = spec.residual_gate_bias
        self.side = spec.token_side
        self.gate1 = self.gate2 = self.gate1_b = self.gate2_b = None
        self.side_gate = self.side_proj = self.side_norm = self.side_table = None

    @property
    def graph_safe(self):
        return all(p.graph_safe for _, p in self.children())

    def children(self):
        parts = [("norm1", self.norm1), ("mixer", self.mixer), ("post1", self.post1)]
        if self.ffn is not None:
            parts += [("norm2", self.norm2), ("ffn", self.ffn), ("post2", self.post2)]
        return tuple(parts)

    def _key(self, local, name):
        prefix = self._names[local]
        return f"{prefix}.{name}" if prefix else name

    def param_specs(self):
        out = {}
        for local, part in self.children():
            for name, ps in part.param_specs().items():
                out[self._key(local, name)] = ps
        D = self.spec.norm1.dim
        if self.gate_names:
            for n in self.gate_names[:2 if self.ffn is not None else 1]:
                out[n] = ParamSpec((D, D))
                out[n + self.gate_bias_suffix] = ParamSpec((D,), role="vector", init="wide")
        if self.side is not None:
            g, p, w = self.side.names
            out[g] = ParamSpec((self.side.dim, D))
            out[p] = ParamSpec((D, self.side.dim), init="wide")
            out[w] = ParamSpec((D,), role="vector", init="ones_noise")
        return out

    def load(self, tensors):
        for local, part in self.children():
            part.load({name: tensors[self._key(local, name)] for name in part.param_specs()})
        if self.gate_names:
            self.gate1 = tensors[self.gate_names[0]].contiguous()
            self.gate1_b = tensors[self.gate_names[0] + self.gate_bias_suffix].contiguous()
            if self.ffn is not None:
                self.gate2 = tensors[self.gate_names[1]].contiguous()
                self.gate2_b = tensors[self.gate_names[1] + self.gate_bias_suffix].contiguous()
        if self.side is not None:
            g, p, w = self.side.names
            self.side_gate, self.side_proj, self.side_norm = tensors[g].contiguous(), tensors[p].contiguous(), tensors[w].contiguous()

    def load_token_table(self, table):
        """The model's second table [vocab, columns]; this block reads `token_side.dim` columns from `column0`."""
        self.side_table = table

    def weight_bytes(self):
        n = sum(p.weight_bytes() for _, p in self.children())
        for w in (self.gate1, self.gate2, self.side_gate, self.side_proj):
            if w is not None:
                n += w.numel() * w.element_size()
        return n

    def cache_need(self):
        return self.mixer.cache_need()

    def first_norm(self):
        return self.norm1

    def _join(self, y, h_in, gate_w, gate_b, post, x, next_norm, want_h):
        """x += post(y * sigmoid(gate_w h_in + gate_b)); returns what the next sublayer reads (its norm of x, or x
        itself in the activation dtype where `next_norm` is None), or None if nothing is wanted."""
        ws, dtype = self.rt.workspace, self.rt.dtype
        z = None
        if gate_w is not None:
            z = ws.take(x.shape, torch.float32)
            ops.gemm(h_in, gate_w, z, ops.EPI_STORE_F32, scratch=ws.take)
        h = ws.take(x.shape, dtype) if want_h else None
        ops.gated_norm_residual(y, post.weight, post.eps, x, dtype, gate=z, gate_bias=gate_b, next_norm=next_norm, h=h)
        return h

    def forward(self, x, batch, cache, normed=None, next_norm=None):
        ws, dtype = self.rt.workspace, self.rt.dtype
        if isinstance(normed, torch.Tensor):
            h = normed
        else:
            h = ws.take(x.shape, dtype)
            if normed is not None:
                ops.finish_norm(normed, h)
            else:
                self.norm1.forward(x, h)
        side = self.side is not None
        y = ws.take(x.shape, torch.float32)
        self.mixer.forward(h, y, batch, cache, accumulate=False)
        last = self.ffn is None
        # after the last sublayer: the token's second input reads x itself; without one, the next block's norm
        after = (None if side else next_norm) if last else self.norm2.shareable()
        h = self._join(y, h, self.gate1, self.gate1_b, self.post1, x, after, want_h=not last or side or next_norm is not None)
        if not last:
            y = ws.take(x.shape, torch.float32)
            self.ffn.forward(h, y, batch, accumulate=False)
            h = self._join(y, h, self.gate2, self.gate2_b, self.post2, x, None if side else next_norm,
                           want_h=side or next_norm is not None)
        if side:
            if self.side_table is None:
                raise ConfigError("the block's second token input needs the model's table")
            m = self.side.dim
            s = ws.take((x.shape[0], m), torch.float32)
            ops.gemm(h, self.side_gate, s, ops.EPI_STORE_F32, scratch=ws.take)
            g = ws.take((x.shape[0], m), dtype)
            ops.token_gate(s, self.side_table, self.side.column0, batch.token_ids, g)
            y = ws.take(x.shape, torch.float32)
            ops.gemm(g, self.side_proj, y, ops.EPI_STORE_F32, scratch=ws.take)
            h = ws.take(x.shape, dtype) if next_norm is not None else None
            ops.gated_norm_residual(y, self.side_norm, self.side.eps, x, dtype, next_norm=next_norm, h=h)
        return h if next_norm is not None else None


register_part("block", "sandwich", SandwichBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "sublayer_norm", SublayerNormBlock)
