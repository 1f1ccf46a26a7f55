"""The attention mixer: q/k/v projections, per-head q/k norm, rotation, cache, GQA softmax
attention, output projection with the residual sum.

Order of operations (crates/backends/backend_common/src/generic_attention/prefill/mod.rs:73-293,
decode.rs:49-508): q,k,v = h W^T; RMSNorm over each head of q and of k with one weight vector
per projection (mod.rs:62-76), before the rotation; rotate q and k at the token's position;
store k (normed, rotated) and v; each query head attends the keys of kv head h / (nh/nkv) up to
its own position; result times o_proj, added to the residual stream.

The three projections are one matrix here (rows of q, then k, then v), joined at load time, so
one product yields the row layout the fused norm/rotation/cache kernel reads.

Options of the spec that other designs use (`AttentionSpec`): biases on the projections, values
that are the keys themselves (no value product, a cache of one plane), a query temperature that
grows with the position, a cap on the scores, a sink in the softmax's denominator.  A mixer with
any of these takes the second path below: the product leaves float rows, one kernel adds the
biases, applies the temperature and writes q and the cache (each number rounded once), and the
attention kernels take the cap and the sink as parameters.

A third form (`AttentionSpec.whole_qk_norm`, `value_dim`, `value_rotation`, or a position part that turns
pairs by angles taken from the position): q and k are normed over the whole projection, the first channels of
every q and k head are turned at the token's position, and the values are stored turned by their own
position over all their channels; a head's result is turned back by the query's position, so that it depends
on the distance only.  Values may be narrower or wider than keys: the cache's heads have max(dk, dv)
channels, the unused ones are zeros, and the attention kernels run unchanged over heads of that size.
The same form takes four more options: a short causal convolution over time on every channel of q, k and v right
after the projection (its last inputs are state of the sequence); sigmoid weights, sigmoid(score + b_head) for
every visible key with nothing normalised over the keys; one output gate per token and head, sigmoid(G h), whose
rows are part of the one projection; and a mixer without keys and values of its own, whose schedule step reads
another step's cache with its own queries, window and gates.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, KVNeed, StateNeed
from ..errors import ConfigError
from ..registry import build_part, register_part
from .base import Mixer, ParamSpec


class AttentionMixer(Mixer):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.nh, self.nkv, self.hd = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd
        self.qkv_dim = self.q_dim + 2 * self.kv_dim
        self.position = build_part("position", spec.position, rt=rt) if spec.position is not None else None
        self.wqkv = self.wo = self.q_norm = self.k_norm = self.bias = self.sink = None
        self.n_q, self.n_k, self.n_v, self.n_o, self.n_sink = spec.names
        self.shared_values = bool(spec.values_are_keys)
        # the plain form (no option set) keeps the path with the fused kernels of the dense decoder
        self.plain = not (spec.bias or spec.values_are_keys or spec.q_temperature or spec.softcap or spec.sink)
        self.pairs = bool(spec.whole_qk_norm or spec.value_dim is not None or spec.value_rotation is not None
                          or getattr(spec.position, "kind", None) == "rope_pairs" or spec.key_weights != "softmax"
                          or spec.conv_taps is not None or spec.head_gate or spec.reads_kv)
        if self.pairs:
            self._init_pairs()
            return
        if not self.plain and (spec.qk_norm is not None or spec.position is not None):
            raise ConfigError("attention with biases, shared values, a query temperature, a cap or a sink has no "
                              "head norm and no rotation here")
        self.shares_norms = self.plain
        self.can_store = not self.plain
        if not self.shared_values:
            self.qkv_dim = self.q_dim + 2 * self.kv_dim
        else:
            self.qkv_dim = self.q_dim + self.kv_dim

    def _matrices(self):
        return [self.n_q, self.n_k] + ([] if self.shared_values else [self.n_v])

    # -- the third form ------------------------------------------------------------------------
    def _init_pairs(self):
        s = self.spec
        if not self.plain or s.qk_norm is not None and not s.whole_qk_norm:
            raise ConfigError("attention with rotated pairs, a norm over the whole projection or rotated values has "
                              "none of the other options (biases, shared values, temperature, cap, sink, head norm)")
        if s.whole_qk_norm and s.qk_norm is None:
            raise ConfigError("a norm over the whole q and k projections needs its eps (qk_norm)")
        self.plain = False
        self.dk = s.head_dim
        self.dv = s.value_dim if s.value_dim is not None else s.head_dim
        self.hd = max(self.dk, self.dv)              # the cache's and the attention kernels' head size
        self.q_dim, self.kv_dim = self.nh * self.dk, self.nkv * self.dk
        if s.key_weights not in ("softmax", "sigmoid"):
            raise ConfigError(f"unknown key weights {s.key_weights!r}: softmax, sigmoid")
        self.sigmoid_keys = s.key_weights == "sigmoid"
        self.reads_kv = bool(s.reads_kv)
        self.taps = int(s.conv_taps) if s.conv_taps is not None else 0
        if s.conv_taps is not None and self.taps < 1:
            raise ConfigError("a convolution has at least one tap")
        # what the projection's rows hold: q, then (unless another step's are read) k and v, then one gate per head
        self.qkv_dim = self.q_dim + (0 if self.reads_kv else self.kv_dim + self.nkv * self.dv)
        self.proj_dim = self.qkv_dim + (self.nh if s.head_gate else 0)
        self.key_bias = self.w_conv = None
        self.value_position = build_part("position", s.value_rotation, rt=self.rt) if s.value_rotation is not None else None
        if self.value_position is not None and self.value_position.rotary_dim != self.dv:
            raise ConfigError(f"values of {self.dv} channels are turned over all of them, not {self.value_position.rotary_dim}")
        if self.position is not None and self.value_position is not None and self.position.halves != self.value_position.halves:
            raise ConfigError("keys and values are turned in one layout of pairs")
        self.shares_norms = False
        self.can_store = True
        self.shared_values = False

    def _projections(self):
        """(tensor name, rows) of the projections that pass the convolution, in the order of the rows."""
        out = [(self.n_q, self.q_dim)]
        if not self.reads_kv:
            out += [(self.n_k, self.kv_dim), (self.n_v, self.nkv * self.dv)]
        return out

    def _param_specs_pairs(self):
        s = self.spec
        p = {n: ParamSpec((rows, s.hidden_size)) for n, rows in self._projections()}
        p[self.n_o] = ParamSpec((s.hidden_size, self.nh * self.dv))
        if self.taps:
            for n, rows in self._projections():
                p[n + s.conv_suffix] = ParamSpec((rows, self.taps), role="vector", init="wide")
        if self.sigmoid_keys:
            p[s.key_bias_name] = ParamSpec((self.nh,), role="vector", init="wide")
        if s.head_gate:
            p[s.head_gate_name] = ParamSpec((self.nh, s.hidden_size))
        if s.whole_qk_norm:
            p[s.norm_names[0]] = ParamSpec((self.q_dim,), role="vector", init="ones_noise")
            p[s.norm_names[1]] = ParamSpec((self.kv_dim,), role="vector", init="ones_noise")
        return p

    def _load_pairs(self, tensors):
        s = self.spec
        mats = [tensors[n] for n, _ in self._projections()] + ([tensors[s.head_gate_name]] if s.head_gate else [])
        self.wqkv = torch.cat(mats, dim=0).contiguous()
        self.wo = tensors[self.n_o].contiguous()
        if self.taps:
            self.w_conv = torch.cat([tensors[n + s.conv_suffix] for n, _ in self._projections()], dim=0).contiguous()
        if self.sigmoid_keys:
            self.key_bias = tensors[s.key_bias_name].contiguous()
        if s.whole_qk_norm:
            self.q_norm = tensors[s.norm_names[0]].contiguous()
            self.k_norm = tensors[s.norm_names[1]].contiguous()

    def _forward_pairs(self, h, residual, batch, cache, accumulate):
        s, ws, T = self.spec, self.rt.workspace, h.shape[0]
        proj = ws.take((T, self.proj_dim), torch.float32)
        ops.gemm(h, self.wqkv, proj, ops.EPI_STORE_F32, scratch=ws.take)
        rows = proj
        if self.taps:
            rows = ws.take((T, self.qkv_dim), torch.float32)
            ops.short_conv(proj[:, :self.qkv_dim], self.w_conv, cache.states.get("conv"), batch, rows)
        q = ws.take((T, self.nh * self.hd), h.dtype)
        pages = batch.pages[cache.kv_group]
        pos, vpos = self.position, self.value_position
        halves = pos.halves if pos is not None else (vpos.halves if vpos is not None else False)
        fv = vpos.freq if vpos is not None else None
        ops.qkv_rotary_cache(rows, self.q_norm, self.k_norm, s.qk_norm.eps if s.qk_norm is not None else 0.0,
                             pos.freq if pos is not None else None, pos.rotary_dim if pos is not None else 0, halves, fv,
                             batch, pages, q, cache.k, cache.v, self.nh, self.nkv, self.dk, self.dv, self.hd,
                             cache.page_size, write_cache=cache.writes_kv and not self.reads_kv)
        att = ws.take((T, self.nh * self.hd), h.dtype)
        # the gate per token and head multiplies a head's float result inside the attention kernel, before it is rounded
        ops.attention(q, q.stride(0), att, cache.k, cache.v, batch, self.nh, self.nkv, self.hd, cache.page_size, s.scale,
                      s.window, pages, scratch=ws.take, gate_bias=self.key_bias,
                      out_gate=proj[:, self.qkv_dim:] if s.head_gate else None)
        y = att
        if fv is not None:
            y = ws.take((T, self.nh * self.dv), h.dtype)
            ops.rotate_heads_back(att, self.hd, fv, halves, batch.tok_pos, y, self.nh, self.dv)
        elif self.hd != self.dv:          # heads of the cache's width -> heads of the values' width
            y = ws.take((T, self.nh * self.dv), h.dtype)
            ops.head_gate(att, self.hd, None, y, self.nh, self.dv)
        ops.gemm(y, self.wo, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)

    def param_specs(self):
        s = self.spec
        if self.pairs:
            return self._param_specs_pairs()
        p = {
            self.n_q: ParamSpec((self.q_dim, s.hidden_size)),
            self.n_k: ParamSpec((self.kv_dim, s.hidden_size)),
            self.n_o: ParamSpec((s.hidden_size, self.q_dim)),
        }
        if not self.shared_values:
            p[self.n_v] = ParamSpec((self.kv_dim, s.hidden_size))
        if s.bias:
            for n in self._matrices():
                p[n + s.bias_suffix] = ParamSpec((p[n].shape[0],), role="vector", init="normal")
        if s.sink:
            p[self.n_sink] = ParamSpec((self.nh,), role="vector", init="wide")
        if s.qk_norm is not None:
            p["q_norm.weight"] = ParamSpec((self.hd,), role="vector", init="ones_noise")
            p["k_norm.weight"] = ParamSpec((self.hd,), role="vector", init="ones_noise")
        return p

    def load(self, tensors):
        s = self.spec
        if self.pairs:
            return self._load_pairs(tensors)
        self.wqkv = torch.cat([tensors[n] for n in self._matrices()], dim=0).contiguous()
        self.wo = tensors[self.n_o].contiguous()
        if s.bias:
            self.bias = torch.cat([tensors[n + s.bias_suffix] for n in self._matrices()], dim=0).contiguous()
        if s.sink:
            self.sink = tensors[self.n_sink].contiguous()
        if s.qk_norm is not None:
            self.q_norm = tensors["q_norm.weight"].contiguous()
            self.k_norm = tensors["k_norm.weight"].contiguous()

    def weight_bytes(self):
        return (self.wqkv.numel() + self.wo.numel()) * self.wqkv.element_size()

    def cache_need(self):
        s = self.spec
        keep = s.window if s.cache_window == -1 else s.cache_window
        states = ()
        if self.pairs and self.taps > 1:
            states = (("conv", StateNeed((self.taps - 1, self.qkv_dim), torch.float32)),)
        return CacheNeed(kv=KVNeed(self.nkv, self.hd, keep, planes=1 if self.shared_values else 2), states=states)

    def _forward_options(self, h, residual, batch, cache, accumulate):
        """The path of a mixer with any of the spec's options (see the module's notes)."""
        s, ws, T = self.spec, self.rt.workspace, h.shape[0]
        rows = ws.take((T, self.qkv_dim), torch.float32)
        ops.gemm(h, self.wqkv, rows, ops.EPI_STORE_F32, scratch=ws.take)
        q = ws.take((T, self.q_dim), h.dtype)
        pages = batch.pages[cache.kv_group]
        coef, every = s.q_temperature if s.q_temperature else (0.0, 0)
        ops.qk_prepare_cache(rows, self.bias, q, coef, every, batch.tok_seq, batch.tok_pos, pages, cache.k,
                             None if self.shared_values else cache.v, self.nh, self.nkv, self.hd, cache.page_size,
                             write_cache=cache.writes_kv)
        att = ws.take((T, self.q_dim), h.dtype)
        ops.attention(q, q.stride(0), att, cache.k, cache.k if self.shared_values else cache.v, batch, self.nh, self.nkv,
                      self.hd, cache.page_size, s.scale, s.window, pages, scratch=ws.take, softcap=s.softcap, sink=self.sink)
        ops.gemm(att, self.wo, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)

    def forward(self, h, residual, batch, cache, next_norm=None, accumulate=True):
        if self.pairs:
            return self._forward_pairs(h, residual, batch, cache, accumulate)
        if not self.plain:
            return self._forward_options(h, residual, batch, cache, accumulate)
        ws, T = self.rt.workspace, h.shape[0]
        qkv = ws.take((T, self.qkv_dim), h.dtype)
        pages = batch.pages[cache.kv_group]
        pos = self.position
        att = ws.take((T, self.q_dim), h.dtype)
        norm_eps = self.spec.qk_norm.eps if self.spec.qk_norm is not None else 0.0
        if not batch.is_decode and pos is not None and cache.k is not None and \
                ops.gemm_qkv_fused_ok(h, self.wqkv, qkv, self.hd, pos.rotary_dim, pos):
            # long prompts: head norm, rotation and cache write happen in the product's epilogue
            ops.gemm_qkv_fused(h, self.wqkv, qkv, self.q_norm, self.k_norm, norm_eps, pos.cos, pos.sin, batch.tok_seq,
                               batch.tok_pos, pages, cache.k, cache.v, self.nh, self.nkv, cache.page_size, cache.writes_kv,
                               ws.take)
            ops.attention(qkv, qkv.stride(0), att, cache.k, cache.v, batch, self.nh, self.nkv, self.hd,
                          cache.page_size, self.spec.scale, self.spec.window, pages, scratch=ws.take)
            return ops.gemm(att, self.wo, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)
        ops.gemm(h, self.wqkv, qkv, scratch=ws.take)
        if batch.is_decode and pos is not None and ops.attention_decode_fused_ok(
                qkv, att, self.nh, self.nkv, self.hd, cache.page_size, pos.rotary_dim, batch.n_seqs):
            nsplit = ops.decode_splits(batch.n_seqs, self.nkv, pages.shape[1] * (cache.page_size // 64))
            buf = ws.take((ops.attention_decode_scratch_floats(batch.n_seqs, self.nh, self.hd, nsplit),), torch.float32)
            ops.attention_decode_fused(qkv, att, cache.k, cache.v, self.q_norm, self.k_norm, norm_eps, pos.cos, pos.sin,
                                       cache.writes_kv, batch.seq_len, pages, buf, self.nh, self.nkv, cache.page_size,
                                       nsplit, self.spec.scale, self.spec.window)
        else:
            ops.qk_norm_rope_cache(
                qkv, self.q_norm, self.k_norm, norm_eps,
                pos.cos if pos is not None else None, pos.sin if pos is not None else None,
                pos.rotary_dim if pos is not None else 0, batch.tok_seq, batch.tok_pos, pages,
                cache.k, cache.v, self.nh, self.nkv, self.hd, cache.page_size, write_cache=cache.writes_kv)
            ops.attention(qkv, qkv.stride(0), att, cache.k, cache.v, batch, self.nh, self.nkv, self.hd,
                          cache.page_size, self.spec.scale, self.spec.window, pages, scratch=ws.take)
        return ops.gemm(att, self.wo, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)


register_part("mixer", "attention", AttentionMixer)
