"""Small Nefivik configurations and weights for tests.  Nothing here is shared with the library's compute
path: tensors are drawn with torch's generator and written with the container writer.

Weights: matrices N(0, gain^2 / in), norm weights around 1, biases 0.3-1 N, convolution taps 0.5 N.
Routers are made decisive unless asked otherwise, so that no comparison in bfloat16 rests on a close call
between two experts or two groups: the first E channels of the stream carry, for every token id, a ranking of
the experts (in steps of `step`), no sublayer writes to those channels (the norms of the results and of the
second token input have weight zero there), and router row e reads channel e with a large weight beside small
random weights elsewhere.  The norm before the router divides all of them by one number, which keeps the order.
"""
from __future__ import annotations

import copy
import json
import math
import os

import torch

from herbert_rs_b200.weights.safetensors_io import save_file


def attention(heads=4, kv_heads=2, dim=16, vdim=8, window=12, rot_dims=None, base=10000.0, scaling="default", scale=None,
              sharp=1.0, conv=3, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": sharp / math.sqrt(dim) if scale is None else scale}
    dims = dim if rot_dims is None else rot_dims
    if dims:
        m["rot"] = {"base": base, "dims": dims}
        if scaling == "default":
            scaling = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    if window is not None:
        m["mask"] = {"size": window}
    if conv is not None:
        m["conv"] = conv
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def delta(heads=2, dim=16):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def moe(experts=6, top=2, ff=24, limit=1.5, groups=3, keep=2):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def config(layers, vocab=131, width=64, eps=1e-5, side=5):
    """layers: list of (mixer entry, mlp entry or None)."""
    c = {"architecture": "Nefivik", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [copy.deepcopy(dict(m, mlp=f)) for m, f in layers]}
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


def weights(cfg, seed=0, decay_rank=6, decisive_router=True, step=1.0, embed_gain=1.0):
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, mean=0.0, std=0.2):
        return mean + std * torch.randn(n, generator=g)

    L = len(cfg["layers"])
    w = {"embed": torch.randn(V, D, generator=g) * embed_gain, "head": mat(V, D, 2.0), "final.norm": vec(D, 1.0)}
    side = cfg.get("token_side")
    if side:
        w["side.embed"] = torch.randn(V, L * side["dim"], generator=g)
    E = max((l["mlp"]["router"]["experts"] for l in cfg["layers"] if l.get("mlp")), default=0)
    if E and decisive_router:
        assert E < D
        for tok in range(V):
            w["embed"][tok, :E] = torch.randperm(E, generator=g).double() * step
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = vec(D, 1.0), vec(D, 1.0)
        w[p + "rg1"], w[p + "rg1.b"] = mat(D, D, 1.5), vec(D, 0.5, 0.7)
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            q = p + "mix."
            w.update({q + "q": mat(H * dk, D, 1.5), q + "pb": vec(H, -1.0, 1.0), q + "g": mat(H, D, 1.5), q + "o": mat(D, H * dv)})
            if "kv_from" not in m:
                w.update({q + "k": mat(G * dk, D, 1.5), q + "v": mat(G * dv, D)})
            if "conv" in m:
                w[q + "q.conv"] = torch.randn(H * dk, m["conv"], generator=g) * 0.5
                if "kv_from" not in m:
                    w[q + "k.conv"] = torch.randn(G * dk, m["conv"], generator=g) * 0.5
                    w[q + "v.conv"] = torch.randn(G * dv, m["conv"], generator=g) * 0.5
        else:
            H, n = m["heads"], m["dim"]
            q = p + "mix."
            w.update({q + "r": mat(H * n, D, 1.5), q + "k": mat(H * n, D, 1.5), q + "v": mat(H * n, D, 1.5), q + "g": mat(H * n, D, 1.5),
                      q + "a": mat(H * n, D, 1.5), q + "a.b": vec(H * n, 0.0, 1.0), q + "w1": mat(decay_rank, D, 1.5),
                      q + "w2": mat(H * n, decay_rank, 3.0), q + "w0": vec(H * n, -1.0, 2.0), q + "norm": vec(H * n, 1.0),
                      q + "o": mat(D, H * n)})
        f = l.get("mlp")
        if f:
            n, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "norm2"], w[p + "norm2b"] = vec(D, 1.0), vec(D, 1.0)
            w[p + "rg2"], w[p + "rg2.b"] = mat(D, D, 1.5), vec(D, 0.5, 0.7)
            for e in range(n):
                # gains that reach both clamps for some channels
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = mat(ff, D, 2.5), mat(ff, D, 2.5)
                w[p + f"mlp.e{e}.down"] = mat(D, ff)
            r = mat(n, D, 3.0)
            if decisive_router:
                r = r * 0.1
                r[:, :E] = 0.0
                r[:, :n] = torch.eye(n) * 6.0
            w[p + "mlp.router"] = r
        if side:
            w.update({p + "side.gate": mat(side["dim"], D, 1.5), p + "side.proj": mat(D, side["dim"]), p + "side.norm": vec(D, 0.7)})
        if E and decisive_router:
            for k in ("norm1b", "norm2b", "side.norm"):
                if p + k in w:
                    w[p + k][:E] = 0.0
            for k in ("norm1", "norm2"):
                if p + k in w:
                    w[p + k][:E] = 1.0
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write(cfg, tensors, folder):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(dict(tensors), os.path.join(folder, "model.safetensors"))
    return str(folder)


def make(folder, layers, seed=0, **kw):
    """Write a model folder; returns (folder, plain model)."""
    import plain_nefivik as P
    wkw = {k: kw.pop(k) for k in ("decay_rank", "decisive_router", "step", "embed_gain") if k in kw}
    cfg = config(layers, **kw)
    write(cfg, weights(cfg, seed, **wkw), folder)
    return str(folder), P.PlainNefivik(str(folder))


def router_margins(plain, ids):
    """The smallest gap, over all layers and tokens of `ids`, between the router logits of a chosen and the best
    unchosen open expert, and between a kept and the best dropped group (exact arithmetic; the softmax keeps the order
    of the logits, and a gap between logits is what a rounding of the router's input moves)."""
    import plain_nefivik as P
    c, W = plain.cfg, plain.W
    dtype = torch.float64
    eps = float(c["norm"]["eps"])
    tokens = [int(t) for t in ids]
    x = W["embed"].to(dtype)[torch.tensor(tokens)]
    kvs, worst = {}, math.inf
    for i, L in enumerate(c["layers"]):
        f = L.get("mlp")
        if f:
            # the stream after the mixer's part of this layer
            only_mixer = copy.deepcopy(plain)
            only_mixer.cfg = copy.deepcopy(c)
            only_mixer.cfg["layers"][i]["mlp"] = None
            only_mixer.cfg.pop("token_side", None)
            xm = only_mixer.layer(i, x, tokens, list(range(len(tokens))), dtype, P._keep, dict(kvs))
            h = P.rms_norm(xm, W[f"l{i}.norm2"].to(dtype), eps)
            z = h @ W[f"l{i}.mlp.router"].to(dtype).T
            rt = f["router"]
            gr = rt.get("groups") or {"count": 1, "keep": 1}
            per = rt["experts"] // gr["count"]
            for t in range(len(tokens)):
                s = z[t]
                gs = s.reshape(gr["count"], per).max(1).values.sort(descending=True).values
                if gr["keep"] < gr["count"]:
                    worst = min(worst, float(gs[gr["keep"] - 1] - gs[gr["keep"]]))
                chosen, _ = P.route(z[t], rt["top"], gr["count"], gr["keep"])
                kept = sorted(range(gr["count"]), key=lambda q: (-float(s.reshape(gr["count"], per).max(1).values[q]), q))[:gr["keep"]]
                open_ = [e for e in range(rt["experts"]) if e // per in kept and e not in chosen]
                if open_:
                    worst = min(worst, float(min(s[e] for e in chosen) - max(s[e] for e in open_)))
        x = plain.layer(i, x, tokens, list(range(len(tokens))), dtype, P._keep, kvs)
    return worst
