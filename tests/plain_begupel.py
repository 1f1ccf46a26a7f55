"""A plain, slow implementation of the Begupel decoder: whole sequences, no cache, no batching,
one function per mechanism, written from the design's equations.  It shares no code with the
library: it parses config.json and the safetensors file itself and computes with torch on the CPU.

The design in this file's notation (T tokens, D = width; positions count from 0 in a sequence):

  x_0[t] = E[tok_t] + B[(tok_{t-1} * m_prev + tok_t * m_cur) mod n]      (B's last row, index n, for t = 0)
  a layer:  h = x + canon(x);  x <- x + GN1(mixer(h));  x <- x + GN2(ff(x))    (a layer may lack ff)
            canon(x)_t = sum_j c[:, j] * x_{t - taps + 1 + j}                   (zeros before the sequence)
            GN(y): y cut into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times w
  logits = cap * tanh((head GN_final(x)) / cap)

Mixers: "lightning" (a decaying matrix state per head) and "parallel" (windowed softmax attention with
rotated queries, keys and values beside a gated delta rule, summed with two constants).

`dtype` is the dtype of all arithmetic (float64 for a ground truth).  Weights are used as stored
(bfloat16 values widened exactly).  `store`, where given, is applied to every activation that an
engine would keep in its activation dtype between two kernels (`bf16_storage` rounds those to
bfloat16): what the number format alone does to the logits follows from it.
"""

from __future__ import annotations

import json
import math
import struct
from typing import Dict, Sequence

import numpy as np
import torch


# ---- reading a model folder ---------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if info["dtype"] == "BF16":
            u = np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<f4").copy())
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<i4").copy())
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        out[name] = t.reshape(info["shape"])
    return out


def bf16_storage(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


def _keep(t):
    return t


# ---- small functions --------------------------------------------------------------------------
def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.clamp(z, min=0.0) + torch.log1p(torch.exp(-z.abs()))


def rms_norm(y, w, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w


def group_norm(y, w, groups, eps):
    """Each of `groups` equal consecutive parts of the last axis divided by its own root mean square."""
    T, D = y.shape
    parts = y.reshape(T, groups, D // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, D) * w


def causal_conv(x, w):
    """y_t = sum_j w[:, j] * x_{t - taps + 1 + j}; x [T, C], w [C, taps]; the last column weighs x_t itself."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


# ---- embedding --------------------------------------------------------------------------------
def embedding(tokens: Sequence[int], W, cfg, dtype):
    E, B = W["embed"].to(dtype), W["bigram"].to(dtype)
    big = cfg["embedding"]["bigram"]
    n, mp, mc = int(big["buckets"]), int(big["mul_prev"]), int(big["mul_cur"])
    rows = []
    for t, tok in enumerate(tokens):
        r = n if t == 0 else (int(tokens[t - 1]) * mp + int(tok) * mc) % n
        rows.append(E[int(tok)] + B[r])
    return torch.stack(rows)


# ---- rotations --------------------------------------------------------------------------------
def turn_pairs(u, angles, layout="interleaved"):
    """u [..., n] with n = 2 * angles.shape[-1]: every pair (a, b) becomes (a cos - b sin, b cos + a sin).
    interleaved: pair m is (2m, 2m + 1); halves: pair m is (m, m + n/2)."""
    c, s = torch.cos(angles), torch.sin(angles)
    out = torch.empty_like(u)
    if layout == "interleaved":
        a, b = u[..., 0::2], u[..., 1::2]
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = b * c + a * s
    else:
        half = u.shape[-1] // 2
        a, b = u[..., :half], u[..., half:]
        out[..., :half] = a * c - b * s
        out[..., half:] = b * c + a * s
    return out


def pair_frequencies(base, n, dtype):
    """base^(-2m/n) for m < n/2."""
    m = torch.arange(n // 2, dtype=dtype)
    return torch.pow(torch.tensor(float(base), dtype=dtype), -2.0 * m / n)


# ---- the windowed attention with rotated values ("left") ----------------------------------------
def rotated_value_attention(h, W, p, m, eps, store=_keep):
    """h [T, D]; W: tensors under prefix p; m: the mixer's sizes and constants."""
    T = h.shape[0]
    dt = h.dtype
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W[p + "q"].to(dt).T
    k = h @ W[p + "k"].to(dt).T
    v = h @ W[p + "v"].to(dt).T
    q = rms_norm(q, W[p + "q.norm"].to(dt), eps).reshape(T, H, dk)
    k = rms_norm(k, W[p + "k.norm"].to(dt), eps).reshape(T, G, dk)
    v = v.reshape(T, G, dv)
    pos = torch.arange(T, dtype=dt)
    rot = m["rot"]
    rd = int(rot["dims"])
    factor = float(rot.get("scaling", {}).get("factor", 1.0)) if rot.get("scaling") else 1.0
    f = pair_frequencies(rot["base"], rd, dt) / factor
    ang = pos[:, None, None] * f[None, None, :]
    q = torch.cat([turn_pairs(q[..., :rd], ang), q[..., rd:]], dim=-1)
    k = torch.cat([turn_pairs(k[..., :rd], ang), k[..., rd:]], dim=-1)
    fv = pair_frequencies(rot["base"], dv, dt)
    angv = pos[:, None, None] * fv[None, None, :]
    v = turn_pairs(v, angv)
    q, k, v = store(q), store(k), store(v)
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=dt)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - int(window) + 1)
            s = (k[lo:i + 1, g] @ q[i, hd]) * float(m["scale"])
            w = torch.softmax(s, dim=0)
            out[i, hd] = w @ v[lo:i + 1, g]
    out = turn_pairs(out, -angv)
    return store(out.reshape(T, H * dv)) @ W[p + "o"].to(dt).T


# ---- the gated delta rule ("right") -------------------------------------------------------------
def delta_recurrence(q, k, v, decay, beta, state=None):
    """q, k [T, G, dk]; v [T, H, dv]; decay, beta [T, H].  Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  `state`, a list, receives the final matrices [H, dk, dv]."""
    T, H, dv = v.shape
    G, dk = q.shape[1], q.shape[2]
    o = torch.zeros(T, H, dv, dtype=v.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=v.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
        if state is not None:
            state.append(S)
    return o


def decay_recurrence(q, k, v, decay, state=None):
    """q, k [T, H, dk]; v [T, H, dv]; decay [H].  Per head: S <- d S + k v^T; o = S^T q."""
    T, H, dv = v.shape
    dk = q.shape[2]
    o = torch.zeros(T, H, dv, dtype=v.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=v.dtype)
        for t in range(T):
            S = float(decay[hd]) * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
        if state is not None:
            state.append(S)
    return o


def gated_delta_rule(h, W, p, m, eps, store=_keep):
    T = h.shape[0]
    dt = h.dtype
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].to(dt).T, W[p + "q.conv"].to(dt))).reshape(T, G, dk)
    k = silu(causal_conv(h @ W[p + "k"].to(dt).T, W[p + "k.conv"].to(dt))).reshape(T, G, dk)
    v = silu(causal_conv(h @ W[p + "v"].to(dt).T, W[p + "v.conv"].to(dt))).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].to(dt).T)                                        # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"].to(dt)) * softplus(h @ W[p + "a"].to(dt).T + W[p + "dt_bias"].to(dt)))
    gate = h @ W[p + "g"].to(dt).T
    o = delta_recurrence(q, k, v, decay, beta)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[p + "norm"].to(dt)
    y = o.reshape(T, H * dv) * silu(gate)
    return store(y) @ W[p + "o"].to(dt).T


def parallel_mixer(h, W, p, m, eps, store=_keep):
    left = rotated_value_attention(h, W, p + "left.", m["left"], eps, store)
    right = gated_delta_rule(h, W, p + "right.", m["right"], eps, store)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- lightning attention ------------------------------------------------------------------------
def lightning(h, W, p, m, eps, store=_keep):
    T = h.shape[0]
    dt = h.dtype
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].to(dt).T).reshape(T, H, dk)
    k = silu(h @ W[p + "k"].to(dt).T).reshape(T, H, dk)
    v = silu(h @ W[p + "v"].to(dt).T).reshape(T, H, dv)
    gate = sigmoid(h @ W[p + "g"].to(dt).T)
    o = decay_recurrence(q, k, v, m["decay"])
    y = rms_norm(o.reshape(T, H * dv), W[p + "norm"].to(dt), eps) * gate
    return store(y) @ W[p + "o"].to(dt).T


# ---- feed-forward -------------------------------------------------------------------------------
def dense_ff(h, W, p, store=_keep):
    dt = h.dtype
    g = h @ W[p + "gate"].to(dt).T + W[p + "gate.b"].to(dt)
    u = h @ W[p + "up"].to(dt).T + W[p + "up.b"].to(dt)
    return store(torch.relu(g) * u) @ W[p + "down"].to(dt).T + W[p + "down.b"].to(dt)


# ---- the model ----------------------------------------------------------------------------------
def forward(tokens: Sequence[int], W, cfg, dtype=torch.float64, store=_keep, layers_out=None):
    """Logits [T, vocab] of one sequence from its start.  `layers_out`, a list, receives the stream after every layer."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    x = embedding(tokens, W, cfg, dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = store(x + causal_conv(x, W[p + "canon1"].to(dtype)))
        if layer["type"] == "lightning":
            y = lightning(h, W, p + "mix.", layer["mixer"], eps, store)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, W, p + "mix.", layer["mixer"], eps, store)
        else:
            raise ValueError(layer["type"])
        x = x + group_norm(y, W[p + "norm1"].to(dtype), groups, eps)
        if layer.get("mlp") is not None:
            y = dense_ff(store(x), W, p + "mlp.", store)
            x = x + group_norm(y, W[p + "norm2"].to(dtype), groups, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    z = store(group_norm(x, W["final.norm"].to(dtype), groups, eps)) @ W["head"].to(dtype).T
    cap = cfg.get("logit_softcap")
    return z if cap is None else float(cap) * torch.tanh(z / float(cap))


def load(folder: str):
    with open(f"{folder}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{folder}/model.safetensors")


class PlainBegupel:
    """The plain model of a folder, or of a configuration and tensors given directly."""

    def __init__(self, folder: str = None, config: dict = None, tensors: Dict[str, torch.Tensor] = None):
        if folder is not None:
            config, tensors = load(folder)
        self.cfg = config
        self.w = {k: (v.float() if v.is_floating_point() else v) for k, v in tensors.items()}

    def logits(self, ids, dtype=torch.float64, store=_keep) -> torch.Tensor:
        return forward(list(ids), self.w, self.cfg, dtype, store)

    def layers(self, ids, dtype=torch.float64):
        out = []
        forward(list(ids), self.w, self.cfg, dtype, _keep, layers_out=out)
        return out
