"""The Nefivik design without a GPU: configuration reading and its error messages, the tensor
declaration, cache needs, and the plain implementation against second forms of its own mechanisms."""
import copy
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import plain_nefivik as P
import nefivik_util as U
from herbert_rs_b200.cache import SequenceCache
from herbert_rs_b200.config.nefivik import DECAY_CONSTANT, NefivikConfig
from herbert_rs_b200.errors import ConfigError
from herbert_rs_b200.parts.rope import pair_frequencies
from herbert_rs_b200.weights.loader import build_model

F64 = torch.float64


def test_configuration_is_read_from_the_nested_keys():
    cfg = U.config([(U.attention(heads=6, kv_heads=3, dim=24, vdim=40, window=9, rot_dims=10, base=777.0, scale=0.3, conv=5,
                                 scaling={"factor": 3.0, "low": 0.5, "high": 2.0, "original": 100}), U.moe(experts=8, top=3, ff=56, limit=2.5, groups=4, keep=2)),
                    (U.delta(heads=3, dim=20), None),
                    (U.attention(heads=6, kv_heads=3, dim=24, vdim=40, window=30, rot_dims=10, base=777.0, conv=None, kv_from=0), U.moe(groups=None))],
                   vocab=99, width=72, eps=3e-6, side=7)
    spec = NefivikConfig.from_dict(cfg).model_spec()
    assert (spec.vocab_size, spec.hidden_size, spec.token_side_table) == (99, 72, ("side.embed", 21))
    b0, b1, b2 = spec.blocks
    assert b0.kind == "sandwich" and (b0.norm1.eps, b0.post_norms[0].weight_name, b0.post_norms[1].weight_name) == (3e-6, "norm1b", "norm2b")
    assert b0.residual_gates == ("rg1", "rg2") and (b1.token_side.dim, b1.token_side.column0, b2.token_side.column0) == (7, 7, 14)
    a = b0.mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.window, a.scale, a.conv_taps) == (6, 3, 24, 40, 9, 0.3, 5)
    assert a.key_weights == "sigmoid" and a.head_gate and not a.reads_kv
    assert (a.position.rotary_dim, a.position.theta, a.position.layout, a.position.band_scaling) == (10, 777.0, "halves", (3.0, 0.5, 2.0, 100.0))
    assert a.cache_window == 30                      # the layer that reads these keys looks further back than their owner
    f = b0.ffn
    assert (f.num_experts, f.top_k, f.expert_size, f.act_limit, f.groups, f.keep_groups, f.group_top) == (8, 3, 56, 2.5, 4, 2, 1)
    assert f.gated and f.activation == "swish_clamp" and f.score == "softmax" and not f.renormalize
    assert b1.ffn is None and (b1.mixer.num_heads, b1.mixer.key_dim, b1.mixer.value_dim) == (3, 20, 20)
    assert b1.mixer.decay_constant == math.exp(-0.5) == DECAY_CONSTANT and b1.mixer.unit_eps == 1e-6
    assert b2.mixer.reads_kv and b2.mixer.conv_taps is None and b2.mixer.window == 30 and (b2.ffn.groups, b2.ffn.keep_groups) == (1, 1)
    assert [(s.layer, s.reads_cache_of) for s in spec.schedule] == [(0, None), (1, None), (2, 0)]
    assert hb.registry.architecture_for(cfg) == "Nefivik"
    del cfg["token_side"], cfg["layers"][0]["mixer"]["mask"], cfg["layers"][0]["mixer"]["rot"], cfg["layers"][0]["mixer"]["conv"]
    spec = NefivikConfig.from_dict(cfg).model_spec()
    a = spec.blocks[0].mixer
    assert spec.token_side_table is None and spec.blocks[0].token_side is None
    assert a.window is None and a.position is None and a.conv_taps is None and a.cache_window == -1


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), "scaling"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.5), "scaling"),
    (lambda c: c["layers"][0]["mixer"].update(conv=0), "conv"),
    (lambda c: c["layers"][0]["mixer"].update(kv_from=0), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=12), "other key/value heads or sizes"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "cannot give"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "cannot give"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c["token_side"].update(dim=0), "dim"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(edit, message):
    cfg = U.config([(U.attention(), U.moe()), (U.delta(), None), (U.attention(kv_from=0), None)])
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        NefivikConfig.from_dict(cfg)


def test_declared_tensors_and_cache_need(tmp_path):
    cfg = U.config([(U.attention(heads=4, kv_heads=2, dim=16, vdim=32, window=12, conv=4), U.moe()),
                    (U.delta(heads=3, dim=8), None),
                    (U.attention(heads=4, kv_heads=2, dim=16, vdim=32, window=12, conv=1, kv_from=0), U.moe(groups=None))])
    model = build_model(cfg, hb.Runtime("cpu", torch.bfloat16))
    specs = model.param_specs()
    t = U.weights(cfg)
    assert set(specs) == set(t)
    for name, w in t.items():
        assert all(s in (-1, d) for s, d in zip(specs[name].shape, w.shape)) and len(specs[name].shape) == w.dim(), name
    assert "l1.norm2" not in specs and "l1.rg2" not in specs and "l2.mix.k" not in specs and "l2.mix.v.conv" not in specs
    assert specs["side.embed"].shape == (131, 15) and specs["l1.mix.w1"].shape == (-1, 64)
    n0, n1, n2 = model.cache_needs()
    assert (n0.kv.num_kv_heads, n0.kv.head_dim, n0.kv.window) == (2, 32, 12)          # heads as wide as the wider of key and value
    assert dict(n0.states)["conv"].shape == (3, 4 * 16 + 2 * 16 + 2 * 32) and n0.state is None
    assert n1.kv is None and tuple(n1.state.shape) == (3, 8, 8) and n1.state.dtype == torch.float32
    assert n2.states == () and (n2.kv.num_kv_heads, n2.kv.head_dim) == (2, 32)        # a convolution of one tap keeps nothing
    cache = SequenceCache(model.cache_needs(), model.reads_cache_of(), num_pages=8, num_slots=2, page_size=16)
    assert len(cache.kv_needs) == 1 and cache.step_kv[2] == (0, 0, False)             # one group, one entry, read by two steps
    U.write(cfg, t, tmp_path)
    assert P.PlainNefivik(str(tmp_path)).logits([1, 2, 3]).shape == (3, 131)


def test_pages_stay_as_long_as_the_longest_window_that_reads_them():
    cfg = U.config([(U.attention(window=5), None), (U.attention(window=40, kv_from=0), None), (U.attention(window=None), None),
                    (U.attention(window=3, kv_from=2), None)])
    model = build_model(cfg, hb.Runtime("cpu", torch.bfloat16))
    needs = model.cache_needs()
    assert needs[0].kv.window == 40 and needs[2].kv.window is None
    cache = SequenceCache(needs, model.reads_cache_of(), num_pages=16, num_slots=1, page_size=16)
    s = cache.alloc_slot()
    cache.reserve([(s, 100)])
    cache.advance(s, 100)
    g_windowed = cache.step_kv[0][0]
    held = [p for p in cache.pages_of(s, g_windowed) if p >= 0]
    assert len(held) == 4                            # positions 61.. are still in reach of the reader: pages 3 to 6
    assert all(p >= 0 for p in cache.pages_of(s, cache.step_kv[2][0]))


def test_a_missing_or_misshapen_tensor_is_reported(tmp_path):
    from herbert_rs_b200.errors import WeightError
    from herbert_rs_b200.weights.loader import check_tensors
    from herbert_rs_b200.weights.safetensors_io import ModelFiles
    cfg = U.config([(U.attention(), U.moe()), (U.delta(), None)])
    t = U.weights(cfg)
    del t["l1.mix.w0"]
    t["l0.mix.q.conv"] = t["l0.mix.q.conv"][:, :-1].contiguous()
    t["side.embed"] = t["side.embed"][:, :-1].contiguous()
    U.write(cfg, t, tmp_path)
    files = ModelFiles(str(tmp_path))
    with pytest.raises(WeightError) as e:
        check_tensors(build_model(cfg, hb.Runtime("cpu", torch.bfloat16)), files)
    files.close()
    assert "l1.mix.w0" in str(e.value) and "l0.mix.q.conv" in str(e.value) and "side.embed" in str(e.value)


# ---- the plain implementation against second forms of its mechanisms --------------------------------
def test_small_functions_against_torch():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(5, 24, generator=g, dtype=F64) * 3, 1 + 0.1 * torch.randn(24, generator=g, dtype=F64)
    F = torch.nn.functional
    assert (P.rms_norm(x, w, 1e-5) - F.rms_norm(x, (24,), w, 1e-5)).abs().max() < 1e-12
    assert (P.gelu_tanh(x) - F.gelu(x, approximate="tanh")).abs().max() < 1e-12
    assert (P.sigmoid(x) - torch.sigmoid(x)).abs().max() < 1e-12
    cw = torch.randn(24, 4, generator=g, dtype=F64)
    ref = F.conv1d(F.pad(x.T[None], (3, 0)), cw[:, None, :], groups=24)[0].T
    assert (P.causal_conv(x, cw) - ref).abs().max() < 1e-12


def test_frequencies_band_by_band_and_the_library_s_own():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    f = P.rotary_frequencies(32, 10000.0, sc)
    plain = P.rotary_frequencies(32, 10000.0)
    kinds = set()
    for a, b in zip(f, plain):
        l = 2 * math.pi / b
        if l < 16:
            assert a == b; kinds.add("short")
        elif l > 64:
            assert a == b / 8.0; kinds.add("long")
        else:
            assert b / 8.0 < a < b; kinds.add("between")
    assert kinds == {"short", "long", "between"}
    lib = pair_frequencies(32, 10000.0, 1.0, (8.0, 1.0, 4.0, 64))
    assert np.abs(lib.double().numpy() - np.array(f)).max() < 1e-7 * max(f)
    assert np.abs(pair_frequencies(32, 10000.0).double().numpy() - np.array(plain)).max() < 1e-7


def test_rotation_makes_scores_depend_on_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 16, generator=g, dtype=F64), torch.randn(1, 1, 16, generator=g, dtype=F64)
    f = P.rotary_frequencies(8, 100.0)
    def score(i, j):
        return float((P.rotate_heads(q, [i], f, 8)[0, 0] * P.rotate_heads(k, [j], f, 8)[0, 0]).sum())
    assert abs(score(10, 3) - score(107, 100)) < 1e-9 and abs(score(10, 3) - score(10, 4)) > 1e-3
    r = P.rotate_heads(q, [5], f, 8)[0, 0]
    assert torch.equal(r[8:], q[0, 0, 8:]) and abs(float(r[:8].norm() - q[0, 0, :8].norm())) < 1e-12
    # the pair of channel 1 is channel 1 + dims / 2
    a = 5 * f[1]
    assert abs(float(r[1]) - float(q[0, 0, 1] * math.cos(a) - q[0, 0, 5] * math.sin(a))) < 1e-12


def test_sigmoid_attention_as_a_masked_matrix():
    g = torch.Generator().manual_seed(2)
    T, H, G, dk, dv, window = 20, 4, 2, 8, 6, 5
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=F64) for n, d in ((H, dk), (G, dk), (G, dv)))
    bias = torch.randn(H, generator=g, dtype=F64)
    out = P.sigmoid_attention(q, k, v, 0.4, window, bias)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = ((i - j >= 0) & (i - j < window)).to(F64)
    for h in range(H):
        w = torch.sigmoid(q[:, h] @ k[:, h // 2].T * 0.4 + bias[h]) * mask
        assert (out[:, h] - w @ v[:, h // 2]).abs().max() < 1e-12
        assert float(w.sum(-1).max()) > 1.2 and float(w.sum(-1).min()) < 0.9          # nothing is normalised over the keys
    everything = P.sigmoid_attention(q, k, v, 0.4, None, bias)
    assert (everything[:window] - out[:window]).abs().max() < 1e-12 and (everything[window:] - out[window:]).abs().max() > 1e-2


def test_delta_rule_state_as_a_product_of_matrices():
    """S_t = (diag(w_t) - (a_t u_t) u_t^T) S_(t-1) + k_t v_t^T, written with explicit matrices."""
    g = torch.Generator().manual_seed(3)
    T, H, n, nv = 9, 2, 6, 4
    r, k, v = (torch.randn(T, H, d, generator=g, dtype=F64) for d in (n, n, nv))
    w, a = torch.rand(T, H, n, generator=g, dtype=F64), torch.rand(T, H, n, generator=g, dtype=F64)
    o, S = P.general_delta_scan(r, k, v, w, a)
    for h in range(H):
        M = torch.zeros(n, nv, dtype=F64)
        for t in range(T):
            u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + 1e-6)
            M = (torch.diag(w[t, h]) - torch.outer(a[t, h] * u, u)) @ M + torch.outer(k[t, h], v[t, h])
            assert (o[t, h] - M.T @ r[t, h]).abs().max() < 1e-12
        assert (S[h] - M).abs().max() < 1e-12
    o2, S2 = P.general_delta_scan(r[5:], k[5:], v[5:], w[5:], a[5:], state=P.general_delta_scan(r[:5], k[:5], v[:5], w[:5], a[:5])[1])
    assert (o2 - o[5:]).abs().max() < 1e-12 and (S2 - S).abs().max() < 1e-12


def test_routing_against_a_sort_and_the_experts_clamps():
    g = torch.Generator().manual_seed(4)
    changed = 0
    for _ in range(200):
        z = torch.randn(8, generator=g, dtype=F64)
        chosen, weights = P.route(z, 3, 4, 2)
        s = torch.softmax(z, -1)
        groups = s.view(4, 2).max(1).values
        kept = set(torch.argsort(groups, descending=True)[:2].tolist())
        order = [e for e in torch.argsort(s, descending=True).tolist() if e // 2 in kept][:3]
        assert chosen == order and all(abs(float(w) - float(s[e])) < 1e-15 for w, e in zip(weights, chosen))
        assert abs(sum(float(w) for w in weights) - 1.0) > 1e-3                      # not renormalised
        changed += chosen != torch.argsort(s, descending=True)[:3].tolist()
    assert 5 < changed < 150
    h = torch.tensor([1.0, -1.0], dtype=F64)
    Wg, Wu, Wd = torch.tensor([[5.0, 0.0], [0.0, 5.0], [0.3, 0.0]], dtype=F64), torch.tensor([[0.0, 7.0], [9.0, 0.0], [0.0, 0.5]], dtype=F64), torch.eye(3, dtype=F64)
    y = P.expert(h, Wg, Wu, Wd, 2.0, P._keep)
    sw = lambda x: x / (1 + math.exp(-1.702 * x))
    assert abs(float(y[0]) - sw(2.0) * (-2.0 + 1)) < 1e-12             # gate capped from above, up clamped from below
    assert abs(float(y[1]) - sw(-5.0) * (2.0 + 1)) < 1e-12            # the gate has no lower limit, up clamped from above
    assert abs(float(y[2]) - sw(0.3) * (-0.5 + 1)) < 1e-12


def test_leaving_out_a_mechanism_moves_the_logits(tmp_path):
    layers = [(U.attention(window=6), U.moe(top=3)), (U.delta(), U.moe(experts=4, top=1, groups=2, keep=1)), (U.attention(window=9, kv_from=0), None)]
    d, pm = U.make(tmp_path / "m", layers, seed=5)
    ids = np.random.default_rng(5).integers(0, 131, 40).tolist()
    ref = pm.logits(ids)
    low = float((pm.logits(ids, F64, P.bf16_storage) - ref).abs().max())

    def moved(cfg=None, W=None, drop=()):
        other = P.PlainNefivik(config=cfg or pm.cfg, tensors=W or pm.W).logits(ids, drop=drop)
        return float((other - ref).abs().max())
    assert moved(drop=("gate",)) > 4 * low and moved(drop=("side",)) > 4 * low
    for path, value in ((("mask", "size"), 7), (("mask", "size"), 5), (("conv",), None), (("rot", "dims"), 0), (("rot", "scaling"), None),
                        (("scale",), 0.3)):
        cfg = copy.deepcopy(pm.cfg)
        m = cfg["layers"][0]["mixer"]
        for key in path[:-1]:
            m = m[key]
        if value is None:
            del m[path[-1]]
        else:
            m[path[-1]] = value
        W = dict(pm.W)
        if path == ("conv",):                      # without a convolution: its last tap alone would be a scaling, so take taps of 1
            for n in ("q", "k", "v"):
                W[f"l0.mix.{n}.conv"] = torch.ones_like(W[f"l0.mix.{n}.conv"][:, :1])
            cfg["layers"][0]["mixer"]["conv"] = 1
        assert moved(cfg, W) > 4 * low, path
    cfg = copy.deepcopy(pm.cfg)
    cfg["layers"][2]["mixer"]["mask"]["size"] = 6          # the reader's own window, not its owner's
    assert moved(cfg) > 4 * low
    W = dict(pm.W)
    W["l0.mix.pb"] = W["l0.mix.pb"] * 0
    assert moved(W=W) > 4 * low
    W = dict(pm.W)
    W["l0.mix.g"] = W["l0.mix.g"] * 0
    assert moved(W=W) > 4 * low
    cfg = copy.deepcopy(pm.cfg)
    cfg["layers"][0]["mlp"]["expert"]["limit"] = 100.0
    assert moved(cfg) > 4 * low
    cfg = copy.deepcopy(pm.cfg)
    cfg["layers"][0]["mlp"]["router"]["groups"] = {"count": 1, "keep": 1}
    W = dict(pm.W)                                           # with a router that is not made to agree with the groups
    W["l0.mlp.router"] = (torch.randn(6, 64, generator=torch.Generator().manual_seed(1)) * 0.1).to(torch.bfloat16).float()
    assert float((P.PlainNefivik(config=cfg, tensors=W).logits(ids) - P.PlainNefivik(config=pm.cfg, tensors=W).logits(ids)).abs().max()) > 4 * low
