"""The Begupel design without a GPU: configuration reading and its error messages, the tensor
declaration, cache needs, and the plain implementation against second forms of its own mechanisms."""
import copy
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import plain_begupel as P
import begupel_util as U
from herbert_rs_b200.config.begupel import BegupelConfig
from herbert_rs_b200.errors import ConfigError
from herbert_rs_b200.weights.loader import build_model

F64 = torch.float64


def test_configuration_is_read_from_the_nested_keys():
    cfg = U.config([(U.parallel(heads=6, kv_heads=3, dim=24, vdim=40, window=9, rot_dims=10, base=777.0, factor=4.0, scale=0.3,
                                rheads=4, rkv=1, rdim=12, rvdim=20, conv=5, left_scale=0.7, right_scale=1.9), U.dense(56)),
                    (U.lightning(heads=3, dim=8, vdim=24, decay=[0.5, 0.75, 1.0]), None)],
                   vocab=99, width=72, eps=3e-6, groups=3, taps=2, buckets=11, mul_prev=5, mul_cur=9, softcap=12.5)
    spec = BegupelConfig.from_dict(cfg).model_spec()
    assert (spec.vocab_size, spec.hidden_size, spec.logit_softcap) == (99, 72, 12.5)
    pe = spec.pair_embedding
    assert (pe.buckets, pe.mul_prev, pe.mul_cur) == (11, 5, 9)
    b0, b1 = spec.blocks
    assert b0.kind == "sublayer_norm" and b0.input_conv_taps == 2 and (b0.norm1.groups, b0.norm1.eps) == (3, 3e-6)
    assert (b0.mixer.left_scale, b0.mixer.right_scale) == (0.7, 1.9)
    a, r = b0.mixer.left, b0.mixer.right
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.window, a.scale) == (6, 3, 24, 40, 9, 0.3)
    assert a.whole_qk_norm and (a.position.rotary_dim, a.position.theta, a.position.linear_factor, a.position.layout) == (10, 777.0, 4.0, "interleaved")
    assert (a.value_rotation.rotary_dim, a.value_rotation.theta, a.value_rotation.linear_factor) == (40, 777.0, 1.0)
    assert (r.num_heads, r.qk_heads, r.key_dim, r.value_dim, r.conv_taps) == (4, 1, 12, 20, 5)
    assert b0.ffn.intermediate_size == 56 and b0.ffn.activation == "relu" and b0.ffn.bias
    assert b1.ffn is None and b1.mixer.decay == (0.5, 0.75, 1.0) and (b1.mixer.key_dim, b1.mixer.value_dim) == (8, 24)
    assert hb.registry.architecture_for(cfg) == "Begupel"
    del cfg["logit_softcap"], cfg["layers"][0]["mixer"]["left"]["mask"], cfg["layers"][0]["mixer"]["left"]["rot"]["scaling"]
    spec = BegupelConfig.from_dict(cfg).model_spec()
    assert spec.logit_softcap is None and spec.blocks[0].mixer.left.window is None and spec.blocks[0].mixer.left.position.linear_factor == 1.0


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=7), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=0.0), "factor"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "unknown feed-forward kind"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["canon"].update(taps=0), "taps"),
    (lambda c: c.update(logit_softcap=0.0), "logit_softcap"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(edit, message):
    cfg = U.config([(U.parallel(), U.dense()), (U.lightning(), None)])
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        BegupelConfig.from_dict(cfg)


def test_declared_tensors_and_cache_need(tmp_path):
    cfg = U.config([(U.parallel(heads=4, kv_heads=2, dim=16, vdim=32, window=12, rheads=4, rkv=2, rdim=16, rvdim=8, conv=4), U.dense(48)),
                    (U.lightning(heads=3, dim=8, vdim=24), None),
                    (U.parallel(conv=1), None)], taps=3)
    model = build_model(cfg, hb.Runtime("cpu", torch.bfloat16))
    specs = model.param_specs()
    t = U.weights(cfg)
    assert set(specs) == set(t)
    for name, w in t.items():
        assert tuple(specs[name].shape) == tuple(w.shape), name
    assert "l1.norm2" not in specs and specs["bigram"].shape == (98, 64)
    n0, n1, n2 = model.cache_needs()
    assert (n0.kv.num_kv_heads, n0.kv.head_dim, n0.kv.window) == (2, 32, 12)          # heads as wide as the wider of key and value
    assert n0.state is None and n1.kv is None and tuple(n1.state.shape) == (3, 8, 24) and n1.state.dtype == torch.float32
    named = dict(n0.states)
    assert tuple(named["right.state"].shape) == (4, 16, 8) and tuple(named["right.conv"].shape) == (3, 2 * 2 * 16 + 4 * 8)
    assert tuple(named["input_conv"].shape) == (2, 64) and tuple(named["embedding.last_id"].shape) == (1,)
    assert set(dict(n2.states)) == {"right.state", "input_conv"}                          # a convolution of one tap keeps nothing
    assert set(dict(n1.states)) == {"input_conv"}
    U.write(cfg, t, tmp_path)
    assert P.PlainBegupel(str(tmp_path)).logits([1, 2, 3]).shape == (3, 131)


def test_a_missing_or_misshapen_tensor_is_reported(tmp_path):
    from herbert_rs_b200.errors import WeightError
    from herbert_rs_b200.weights.loader import check_tensors
    from herbert_rs_b200.weights.safetensors_io import ModelFiles
    cfg = U.config([(U.parallel(), U.dense())])
    t = U.weights(cfg)
    del t["l0.mix.right.A_log"]
    t["l0.canon1"] = t["l0.canon1"][:, :-1].contiguous()
    U.write(cfg, t, tmp_path)
    files = ModelFiles(str(tmp_path))
    with pytest.raises(WeightError) as e:
        check_tensors(build_model(cfg, hb.Runtime("cpu", torch.bfloat16)), files)
    files.close()
    assert "l0.mix.right.A_log" in str(e.value) and "l0.canon1" in str(e.value)


# ---- the plain implementation against second forms of its mechanisms --------------------------------
def test_small_functions_against_torch():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(5, 24, generator=g, dtype=F64) * 3, 1 + 0.1 * torch.randn(24, generator=g, dtype=F64)
    F = torch.nn.functional
    assert (P.rms_norm(x, w, 1e-5) - F.rms_norm(x, (24,), w, 1e-5)).abs().max() < 1e-12
    assert (P.silu(x) - F.silu(x)).abs().max() < 1e-12 and (P.softplus(x * 10) - F.softplus(x * 10, threshold=1000.0)).abs().max() < 1e-12
    parts = torch.cat([F.rms_norm(x[:, i:i + 8], (8,), None, 1e-5) for i in (0, 8, 16)], -1) * w
    assert (P.group_norm(x, w, 3, 1e-5) - parts).abs().max() < 1e-12
    cw = torch.randn(24, 4, generator=g, dtype=F64)
    ref = F.conv1d(F.pad(x.T[None], (3, 0)), cw[:, None, :], groups=24)[0].T
    assert (P.causal_conv(x, cw) - ref).abs().max() < 1e-12


def test_decaying_memory_is_a_weighted_sum_over_earlier_tokens():
    g = torch.Generator().manual_seed(1)
    T, H, dk, dv = 9, 2, 4, 3
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=F64) for d in (dk, dk, dv))
    decay = [0.8, 1.0]
    o = P.decay_recurrence(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            ref = sum(decay[h] ** (t - j) * float(q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert (o[t, h] - ref).abs().max() < 1e-12


def test_delta_rule_stores_and_overwrites_along_a_key():
    """With beta = 1 and no decay a write makes the memory return exactly the token's value for its key; a second write
    along the same key replaces the first; orthogonal keys do not disturb one another."""
    e = torch.eye(4, dtype=F64)
    k = torch.stack([e[0], e[1], e[0]])[:, None, :]
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=F64)[:, None, :]
    q = torch.stack([e[0], e[0] + e[1], e[0] + e[1]])[:, None, :]
    ones = torch.ones(3, 1, dtype=F64)
    o = P.delta_recurrence(q, k, v, ones, ones)
    assert o[:, 0].tolist() == [[1.0, 2.0], [4.0, 6.0], [8.0, 10.0]]
    o = P.delta_recurrence(q, k, v, ones * 0.5, ones * 0.5)        # decay first, then half of the correction
    S1 = 0.5 * torch.outer(e[0], v[0, 0])
    S2 = 0.5 * S1 + torch.outer(e[1], 0.5 * v[1, 0])
    assert (o[1, 0] - S2.T @ q[1, 0]).abs().max() < 1e-15


def test_rotated_values_make_the_result_depend_on_distance_only():
    """Attention over values turned by their positions and turned back by the query's equals attention over values
    turned by minus the distance: shifting all positions changes nothing."""
    g = torch.Generator().manual_seed(2)
    T, dv = 7, 6
    v = torch.randn(T, dv, generator=g, dtype=F64)
    w = torch.softmax(torch.randn(T, T, generator=g, dtype=F64), -1)
    f = P.pair_frequencies(100.0, dv, F64)
    for layout in ("interleaved", "halves"):
        outs = []
        for shift in (0, 1000):
            pos = torch.arange(T, dtype=F64) + shift
            turned = P.turn_pairs(v, pos[:, None] * f[None], layout)
            outs.append(P.turn_pairs(w @ turned, -pos[:, None] * f[None], layout))
        assert (outs[0] - outs[1]).abs().max() < 1e-9
        i = 4
        ref = sum(w[i, j] * P.turn_pairs(v[j:j + 1], torch.tensor(float(j - i), dtype=F64) * f[None], layout)[0] for j in range(T))
        assert (outs[0][i] - ref).abs().max() < 1e-12
    assert float(f[0]) == 1.0 and abs(float(f[1]) - 100.0 ** (-2 / 6)) < 1e-15
    a = P.turn_pairs(torch.tensor([[1.0, 0.0, 0.0, 0.0]], dtype=F64), torch.tensor([[math.pi / 2, 0.0]], dtype=F64), "interleaved")
    assert (a - torch.tensor([[0.0, 1.0, 0.0, 0.0]], dtype=F64)).abs().max() < 1e-15        # (u, v) -> (u cos - v sin, v cos + u sin)


def test_the_pair_row_and_the_first_token():
    cfg = {"embedding": {"bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}}}
    W = {"embed": torch.zeros(10, 8), "bigram": torch.arange(8.0)[:, None].repeat(1, 8)}
    x = P.embedding([4, 9, 2], W, cfg, F64)
    assert x[:, 0].tolist() == [7.0, float((4 * 3 + 9 * 5) % 7), float((9 * 3 + 2 * 5) % 7)]


def test_leaving_out_one_mechanism_changes_the_logits(tmp_path):
    """The small models are sensitive to every mechanism: the plain logits move by far more than any bound."""
    layers = [(U.parallel(sharp=2.0, rot_dims=8), U.dense()), (U.lightning(), None), (U.parallel(window=20), U.dense())]
    d, pm = U.make(tmp_path, layers, seed=3)
    ids = np.random.default_rng(1).integers(0, 131, 40).tolist()
    ref = pm.logits(ids)

    def variant(edit_cfg=None, edit_w=None):
        cfg, w = copy.deepcopy(pm.cfg), dict(pm.w)
        if edit_cfg:
            edit_cfg(cfg)
        if edit_w:
            edit_w(w)
        return float((P.PlainBegupel(config=cfg, tensors=w).logits(ids) - ref).abs().max())

    zero = lambda name: (lambda w: w.update({name: torch.zeros_like(w[name])}))      # noqa: E731
    assert variant(lambda c: c.pop("logit_softcap")) > 0.01
    assert variant(lambda c: c["norm"].update(groups=1)) > 0.05
    assert variant(lambda c: c["embedding"]["bigram"].update(mul_prev=38)) > 0.05
    assert variant(edit_w=zero("bigram")) > 0.05
    assert variant(edit_w=zero("l1.canon1")) > 0.05
    assert variant(lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=11)) > 0.01
    assert variant(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=16)) > 0.05
    assert variant(lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=1.0)) > 0.05
    assert variant(lambda c: c["layers"][0]["mixer"].update(right_scale=0.0)) > 0.05
    assert variant(lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.5])) > 0.05
    assert variant(edit_w=zero("l0.mix.right.dt_bias")) > 0.01
    assert variant(edit_w=zero("l0.mlp.up.b")) > 0.05
    assert variant(edit_w=lambda w: w.update({"l0.mix.right.q.conv": w["l0.mix.right.q.conv"].flip(1)})) > 0.05
