"""A plain, slow implementation of the Nefivik decoder: whole sequences, no cache, no batching,
one function per mechanism, written from the design's equations.  It shares no code with the
library: it parses config.json and the safetensors file itself and computes with torch on the CPU.

The design in this file's notation (T tokens, D = width; positions count from 0 in a sequence):

  x_0[t] = E[tok_t]
  a layer:  h1 = N1(x);   x <- x + N1b( mixer(h1) * sigmoid(R1 h1 + r1) )
            h2 = N2(x);   x <- x + N2b( ff(h2)    * sigmoid(R2 h2 + r2) )          (a layer may lack ff)
            e  = P[tok_t][i*m : (i+1)*m]   (m numbers of a second table, for layer i)
            y  = Sp ( gelu_tanh(Sg x) * e );   x <- x + y / sqrt(mean(y^2) + eps) * sn
  N(y) = y / sqrt(mean(y^2) + eps) * w
  logits = head N_final(x)

Mixers: "attention" (grouped query heads over a sliding window, every projection through a short causal
convolution, rotated first channels, weights sigmoid(score + b_head) that are not normalised over the keys,
one output gate per head; a layer may read another layer's keys and values) and "general_delta" (a matrix
of state per head with a decay per key channel, from which a part along the unit key is removed before
k v^T is added).  Feed-forward: experts chosen by a softmax router within the best groups.

`dtype` is the dtype of all arithmetic (float64 for a ground truth).  Weights are used as stored
(bfloat16 values widened exactly).  `store`, where given, is applied to every activation that an
engine would keep in its activation dtype between two kernels (`bf16_storage` rounds those to
bfloat16): what the number format alone does to the logits follows from it.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, Sequence

import numpy as np
import torch

DECAY_CONSTANT = math.exp(-0.5)     # w = exp(-DECAY_CONSTANT * sigmoid(.))
UNIT_EPS = 1e-6
GLU_SLOPE = 1.702


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
def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(y, w, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w


def causal_conv(u, w):
    """y_t = sum_j w[:, j] * u_{t - taps + 1 + j}; u [T, C], w [C, taps]; the last column weighs u_t itself."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


# ---- rotation ---------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2, as python floats; with `scaling` (factor, low, high, original) a
    frequency whose wavelength l = 2 pi / f is shorter than original/high stays, one longer than original/low
    is divided by factor, and between the two the result moves linearly in original/l from one to the other."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            l = 2.0 * math.pi / f
            if l < orig / high:
                pass
            elif l > orig / low:
                f = f / factor
            else:
                s = (orig / l - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_heads(x, positions, freqs, dims):
    """x [T, heads, dim]: channel i < dims/2 of every head is paired with channel i + dims/2; the pair (u, v) at
    position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i.  Channels from dims on pass."""
    if dims == 0:
        return x
    half = dims // 2
    ang = torch.tensor(positions, dtype=x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]     # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---- attention --------------------------------------------------------------------------------
def sigmoid_attention(q, k, v, scale, window, head_bias):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv].  Query i sees key j with 0 <= i - j < window
    (window None: every j <= i); the weight of a visible key is sigmoid(q.k * scale + b_head), used as it is."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale + head_bias[h]
            out[i, h] = sigmoid(s) @ v[lo:i + 1, g]
    return out


def attention_keys_values(h, W, p, m, positions, dtype, store):
    """What an attention layer caches: keys after convolution and rotation, values after convolution."""
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = h @ W[p + "k"].to(dtype).T
    v = h @ W[p + "v"].to(dtype).T
    if "conv" in m:
        k = causal_conv(k, W[p + "k.conv"].to(dtype))
        v = causal_conv(v, W[p + "v.conv"].to(dtype))
    rot = m.get("rot")
    k = k.reshape(T, G, dk)
    if rot:
        k = rotate_heads(k, positions, rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")), rot["dims"])
    return store(k), store(v.reshape(T, G, dv))


def attention_mixer(h, W, p, m, positions, dtype, store, kv):
    """kv: (keys, values) of the layer this one reads, or None (then its own)."""
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    if kv is None:
        kv = attention_keys_values(h, W, p, m, positions, dtype, store)
    q = h @ W[p + "q"].to(dtype).T
    if "conv" in m:
        q = causal_conv(q, W[p + "q.conv"].to(dtype))
    q = q.reshape(T, H, dk)
    rot = m.get("rot")
    if rot:
        q = rotate_heads(q, positions, rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")), rot["dims"])
    q = store(q)
    window = m["mask"]["size"] if m.get("mask") else None
    o = sigmoid_attention(q, kv[0], kv[1], float(m["scale"]), window, W[p + "pb"].to(dtype))
    gate = sigmoid(h @ W[p + "g"].to(dtype).T)                        # [T, H]
    o = store((o * gate[:, :, None]).reshape(T, H * dv))
    return o @ W[p + "o"].to(dtype).T, kv


# ---- the generalised delta rule -----------------------------------------------------------------
def general_delta_scan(r, k, v, w, a, state=None):
    """r, k, w, a [T, H, n], v [T, H, n_v].  Per head, with u = k / sqrt(sum k^2 + 1e-6):
    S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T;  o_t = S_t^T r_t.  Returns o [T, H, n_v], S."""
    T, H, n = k.shape
    nv = v.shape[2]
    S = torch.zeros(H, n, nv, dtype=k.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, nv, dtype=k.dtype)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(-1, keepdim=True) + UNIT_EPS)                 # [H, n]
        seen = torch.einsum("hn,hnv->hv", u, S)                                               # u^T S_{t-1}
        S = w[t][:, :, None] * S - (a[t] * u)[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hnv,hn->hv", S, r[t])
    return o, S


def general_delta_mixer(h, W, p, m, eps, dtype, store):
    H, n = m["heads"], m["dim"]
    T = h.shape[0]
    r = (h @ W[p + "r"].to(dtype).T).reshape(T, H, n)
    k = (h @ W[p + "k"].to(dtype).T).reshape(T, H, n)
    v = (h @ W[p + "v"].to(dtype).T).reshape(T, H, n)
    inner = torch.tanh(h @ W[p + "w1"].to(dtype).T)
    w = torch.exp(-DECAY_CONSTANT * sigmoid(inner @ W[p + "w2"].to(dtype).T + W[p + "w0"].to(dtype))).reshape(T, H, n)
    a = sigmoid(h @ W[p + "a"].to(dtype).T + W[p + "a.b"].to(dtype)).reshape(T, H, n)
    o, _ = general_delta_scan(r, k, v, w, a)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
    y = o.reshape(T, H * n) * W[p + "norm"].to(dtype) * sigmoid(h @ W[p + "g"].to(dtype).T)
    return store(y) @ W[p + "o"].to(dtype).T


# ---- the routed feed-forward ------------------------------------------------------------------
def route(z, top, groups, keep):
    """z [E] router logits -> (chosen experts, their weights).  Scores are softmax(z) over all experts; the experts
    form `groups` equal groups of neighbours, a group scores as its best expert, only the `keep` best groups stay
    open, and of their experts the `top` best are chosen; the weights are the scores themselves."""
    s = torch.softmax(z, dim=-1)
    E = s.shape[0]
    per = E // groups
    gs = s.reshape(groups, per).max(dim=1).values
    order = sorted(range(groups), key=lambda g: (-float(gs[g]), g))[:keep]
    open_ = [e for e in range(E) if e // per in order]
    chosen = sorted(open_, key=lambda e: (-float(s[e]), e))[:top]
    return chosen, [s[e] for e in chosen]


def expert(h, Wg, Wu, Wd, limit, store):
    g = torch.clamp(h @ Wg.T, max=limit)
    u = torch.clamp(h @ Wu.T, min=-limit, max=limit)
    y = g * sigmoid(GLU_SLOPE * g) * (u + 1.0)
    return store(y) @ Wd.T


def routed_ff(h, W, p, f, dtype, store, router_input=None):
    rt, limit = f["router"], float(f["expert"]["limit"])
    E, top = rt["experts"], rt["top"]
    gr = rt.get("groups") or {"count": 1, "keep": 1}
    hz = h if router_input is None else router_input
    z = hz @ W[p + "router"].to(dtype).T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], top, gr["count"], gr["keep"])
        for e, wt in zip(chosen, weights):
            q = f"{p}e{e}."
            out[t] += wt * expert(h[t], W[q + "gate"].to(dtype), W[q + "up"].to(dtype), W[q + "down"].to(dtype), limit, store)
    return out


# ---- the per-layer token input ------------------------------------------------------------------
def token_side(x, tokens, layer, W, p, m, eps, dtype, store):
    e = W["side.embed"].to(dtype)[torch.tensor(list(tokens))][:, layer * m:(layer + 1) * m]
    g = gelu_tanh(store(x) @ W[p + "gate"].to(dtype).T) * e
    y = store(g) @ W[p + "proj"].to(dtype).T
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * W[p + "norm"].to(dtype)


# ---- the model ----------------------------------------------------------------------------------
class PlainNefivik:
    def __init__(self, folder: str = None, config: dict = None, tensors: dict = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                config = json.load(f)
            tensors = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.cfg = config
        self.W = {k: v.float() if v.is_floating_point() else v for k, v in tensors.items()}

    def layer(self, i, x, tokens, positions, dtype, store, kvs, drop=()):
        c, W = self.cfg, self.W
        eps = float(c["norm"]["eps"])
        L = c["layers"][i]
        p, m = f"l{i}.", L["mixer"]
        h = store(rms_norm(x, W[p + "norm1"].to(dtype), eps))
        if L["type"] == "attention":
            src = m.get("kv_from")
            y, kvs[i] = attention_mixer(h, W, p + "mix.", m, positions, dtype, store, None if src is None else kvs[src])
        elif L["type"] == "general_delta":
            y = general_delta_mixer(h, W, p + "mix.", m, eps, dtype, store)
        else:
            raise ValueError(L["type"])
        if "gate" not in drop:
            y = y * sigmoid(h @ W[p + "rg1"].to(dtype).T + W[p + "rg1.b"].to(dtype))
        x = x + rms_norm(y, W[p + "norm1b"].to(dtype), eps)
        f = L.get("mlp")
        if f:
            h = store(rms_norm(x, W[p + "norm2"].to(dtype), eps))
            y = routed_ff(h, W, p + "mlp.", f, dtype, store)
            if "gate" not in drop:
                y = y * sigmoid(h @ W[p + "rg2"].to(dtype).T + W[p + "rg2.b"].to(dtype))
            x = x + rms_norm(y, W[p + "norm2b"].to(dtype), eps)
        side = c.get("token_side")
        if side and "side" not in drop:
            x = x + token_side(x, tokens, i, W, p + "side.", int(side["dim"]), eps, dtype, store)
        return x

    def hidden(self, tokens: Sequence[int], dtype=torch.float64, store=None, drop=()):
        """The residual stream after every layer, [layers, T, D], and the last one."""
        store = store or _keep
        tokens = [int(t) for t in tokens]
        positions = list(range(len(tokens)))
        x = self.W["embed"].to(dtype)[torch.tensor(tokens)]
        kvs, per_layer = {}, []
        for i in range(len(self.cfg["layers"])):
            x = self.layer(i, x, tokens, positions, dtype, store, kvs, drop)
            per_layer.append(x)
        return torch.stack(per_layer), x

    def layers(self, tokens: Sequence[int], dtype=torch.float64):
        return list(self.hidden(tokens, dtype)[0])

    def logits(self, tokens: Sequence[int], dtype=torch.float64, store=None, drop=()):
        store = store or _keep
        _, x = self.hidden(tokens, dtype, store, drop)
        h = store(rms_norm(x, self.W["final.norm"].to(dtype), float(self.cfg["norm"]["eps"])))
        return h @ self.W["head"].to(dtype).T
