"""Small Begupel configurations and weights for tests.  Nothing here is shared with the library's compute
path: tensors are drawn with torch's generator and written with the container writer.

Weights: matrices N(0, gain^2 / in), norm weights around 1, biases 0.3 N, convolution taps 0.5 N,
A_log and dt_bias N(0, 1) around values that give decays between about 0.3 and 0.99.
"""
from __future__ import annotations

import copy
import json
import math
import os

import torch

from herbert_rs_b200.weights.safetensors_io import save_file


def lightning(heads=2, dim=16, vdim=8, decay=None):
    if decay is None:
        decay = [math.exp(-1.0 / (2.0 ** (3 * h))) for h in range(heads)]        # fast to slow
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def parallel(heads=4, kv_heads=2, dim=16, vdim=16, window=12, rot_dims=None, base=10000.0, factor=2.0, scale=None, sharp=1.0,
             rheads=4, rkv=2, rdim=16, rvdim=8, conv=4, left_scale=1.3, right_scale=0.8):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": sharp / math.sqrt(dim) if scale is None else scale,
            "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}
    if factor is not None:
        left["rot"]["scaling"] = {"factor": factor}
    if window is not None:
        left["mask"] = {"size": window}
    right = {"heads": rheads, "kv_heads": rkv, "dim": rdim, "vdim": rvdim, "conv": conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def config(layers, vocab=131, width=64, eps=1e-5, groups=2, taps=3, buckets=97, mul_prev=37, mul_cur=11, softcap=20.0):
    """layers: list of (mixer entry, mlp entry or None)."""
    c = {"architecture": "Begupel", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
         "canon": {"taps": taps}, "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
         "layers": [copy.deepcopy(dict(m, mlp=f)) for m, f in layers]}
    if softcap is not None:
        c["logit_softcap"] = softcap
    return c


def weights(cfg, seed=0, embed_gain=1.0):
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, mean=0.0, std=0.2):
        return mean + std * torch.randn(n, generator=g)

    n = cfg["embedding"]["bigram"]["buckets"]
    w = {"embed": torch.randn(V, D, generator=g) * embed_gain, "bigram": torch.randn(n + 1, D, generator=g) * 0.7,
         "head": mat(V, D, 2.0), "final.norm": vec(D, 1.0)}
    taps = cfg["canon"]["taps"]
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        w[p + "norm1"] = vec(D, 1.0)
        w[p + "canon1"] = torch.randn(D, taps, generator=g) * 0.4
        if l["type"] == "lightning":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": mat(H * dk, D, 1.5), p + "mix.k": mat(H * dk, D, 1.5), p + "mix.v": mat(H * dv, D, 1.5),
                      p + "mix.g": mat(H * dv, D, 1.5), p + "mix.o": mat(D, H * dv), p + "mix.norm": vec(H * dv, 1.0)})
        else:
            a, b = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            w.update({q + "q": mat(H * dk, D, 1.5), q + "k": mat(G * dk, D, 1.5), q + "v": mat(G * dv, D), q + "o": mat(D, H * dv),
                      q + "q.norm": vec(H * dk, 1.0), q + "k.norm": vec(G * dk, 1.0)})
            H, G, dk, dv, c = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            q = p + "mix.right."
            w.update({q + "q": mat(G * dk, D, 1.5), q + "k": mat(G * dk, D, 1.5), q + "v": mat(H * dv, D, 1.5),
                      q + "q.conv": torch.randn(G * dk, c, generator=g) * 0.5, q + "k.conv": torch.randn(G * dk, c, generator=g) * 0.5,
                      q + "v.conv": torch.randn(H * dv, c, generator=g) * 0.5,
                      q + "b": mat(H, D, 1.5), q + "a": mat(H, D, 1.5), q + "A_log": vec(H, -0.5, 1.0), q + "dt_bias": vec(H, -1.0, 1.0),
                      q + "norm": vec(dv, 1.0), q + "g": mat(H * dv, D, 1.5), q + "o": mat(D, H * dv)})
        f = l.get("mlp")
        if f:
            ff = f["ff"]
            w[p + "norm2"] = vec(D, 1.0)
            w.update({p + "mlp.gate": mat(ff, D, 1.5), p + "mlp.gate.b": vec(ff, 0.0, 0.3), p + "mlp.up": mat(ff, D),
                      p + "mlp.up.b": vec(ff, 0.0, 0.3), p + "mlp.down": mat(D, ff), p + "mlp.down.b": vec(D, 0.0, 0.3)})
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write(cfg, tensors, folder):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(dict(tensors), os.path.join(folder, "model.safetensors"))
    return str(folder)


def make(folder, layers, seed=0, embed_gain=1.0, **kw):
    """Write a model folder; returns (folder, plain model)."""
    import plain_begupel as P
    cfg = config(layers, **kw)
    write(cfg, weights(cfg, seed, embed_gain), folder)
    return str(folder), P.PlainBegupel(str(folder))
