"""The Nefivik design in the engine against the plain implementation (`plain_nefivik.py`): every
mechanism alone, prompts against decoding, prompts in pieces, unequal batches, slots and pages that
are used again, keys at the window's edge and far away, the first tokens, long decoding, other sizes,
greedy generation through the library's entry points."""
import copy
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import plain_nefivik as P
import nefivik_util as U
from gpu_util import (DTYPES, assert_close, bound_for, engine_for, replay_batches, replay_tail_one_by_one, replay_whole, to_np)
from herbert_rs_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
VOCAB = 131


def ids_for(rng, vocab, n):
    return rng.integers(0, vocab, n).tolist()


_model_own: dict = {}
_plain_assert_close = assert_close


def assert_close(got, ref, dtype, what="", bound=None, plain=None, ids=None, rows=None, arith=torch.float64):
    """gpu_util's comparison, with a steadier bfloat16 bound for whole models.  A norm behind every sublayer brings a
    small result to full size, so at a position where a result happens to be small any rounding is amplified, by how
    much depends on its direction: what bfloat16 storage between kernels does to the plain implementation varies
    twentyfold from position to position.  The bound is therefore three times the largest such figure, over all rows of
    the request and over one fixed 64-token request of the model; at most one row in fifty (or one row) may lie above
    it, and none above one and a half times it."""
    if not (dtype == "bfloat16" and bound is None and plain is not None):
        return _plain_assert_close(got, ref, dtype, what, bound=bound, plain=plain, ids=ids, rows=rows, arith=arith)
    key = id(plain)
    if key not in _model_own:
        fixed = ids_for(np.random.default_rng(77), VOCAB, 64)
        _model_own[key] = float((plain.logits(fixed, arith, P.bf16_storage) - plain.logits(fixed, arith)).abs().max())
    own = float((plain.logits(ids, arith, P.bf16_storage) - plain.logits(ids, arith)).abs().max())
    bound = 3.0 * max(own, _model_own[key])
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    err = np.abs(got - ref).max(axis=-1)
    over = int((err > bound).sum())
    assert err.max() <= 1.5 * bound and over <= max(1, len(err) // 50), \
        f"{what} [bfloat16]: {over} of {len(err)} rows over {bound:.3e}, the largest error {err.max():.3e} at row {int(err.argmax())}"
    return float(err.max())


def td_of(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def step_of(lens, slots, pos0=None, ids=None):
    """The device arrays of a step that the kernels of this file read: sequences of `lens` new tokens in `slots`."""
    pos0 = pos0 or [0] * len(lens)
    starts = np.concatenate([[0], np.cumsum(lens)])
    tok_seq = [b for b, n in enumerate(lens) for _ in range(n)]
    tok_pos = [pos0[b] + i for b, n in enumerate(lens) for i in range(n)]
    return SimpleNamespace(seq_slot=i32(slots), seq_start=i32(starts.tolist()), seq_pos0=i32(pos0), tok_seq=i32(tok_seq),
                           tok_pos=i32(tok_pos), token_ids=i32(ids) if ids is not None else None, n_seqs=len(lens),
                           n_tokens=int(sum(lens)), max_q_len=max(lens), seq_len=i32([p + n for p, n in zip(pos0, lens)]),
                           is_decode=all(n == 1 for n in lens))


@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    """Both mixers; a layer that reads the first layer's keys and values with a longer window than that layer's own; key and
    value sizes that differ; a window shorter than a page; partly rotated keys; a layer without a feed-forward."""
    layers = [(U.attention(heads=4, kv_heads=2, dim=16, vdim=8, window=12, rot_dims=8, conv=3), U.moe()),
              (U.delta(heads=2, dim=16), U.moe(experts=4, top=1, groups=2, keep=1)),
              (U.attention(heads=4, kv_heads=2, dim=16, vdim=8, window=20, rot_dims=8, conv=2, kv_from=0), None),
              (U.delta(heads=3, dim=8), U.moe(experts=6, top=3, ff=16, groups=None))]
    return U.make(tmp_path_factory.mktemp("nefivik_mixed"), layers, seed=3)


# ---- each mechanism alone -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [48, 336, 1000, 4608])
def test_gate_norm_and_sum_into_the_stream(dtype, dim):
    g = torch.Generator().manual_seed(dim)
    T = 6
    y = torch.randn(T, dim + 8, generator=g) * torch.linspace(0.1, 5.0, dim + 8)
    z, zb = torch.randn(T, dim + 4, generator=g) * 2.0, torch.randn(dim, generator=g)
    x, w, w2 = torch.randn(T, dim, generator=g), 1.0 + 0.2 * torch.randn(dim, generator=g), 1.0 + 0.2 * torch.randn(dim, generator=g)
    for gate, bias, nxt in ((True, True, True), (True, True, False), (True, False, True), (False, False, True), (False, False, False)):
        x1, h = x.clone().to(DEV), torch.empty(T, dim, dtype=td_of(dtype), device=DEV)
        ops.gated_norm_residual(y.to(DEV)[:, :dim], w.to(DEV), 1e-5, x1, td_of(dtype), gate=z.to(DEV)[:, :dim] if gate else None,
                                gate_bias=zb.to(DEV) if bias else None, next_norm=(w2.to(DEV), 3e-5) if nxt else None, h=h)
        v = y.double()[:, :dim]
        if gate:
            v = v * P.sigmoid(z.double()[:, :dim] + (zb.double() if bias else 0.0))
        ref = x.double() + P.rms_norm(v, w.double(), 1e-5)
        assert_close(to_np(x1), ref.numpy(), "float32", "stream")
        assert_close(to_np(h), (P.rms_norm(ref, w2.double(), 3e-5) if nxt else ref).numpy(), dtype, "what the next sublayer reads")
    x1 = x.clone().to(DEV)
    ops.gated_norm_residual(y.to(DEV)[:, :dim], w.to(DEV), 1e-5, x1, td_of(dtype))          # nothing handed on
    assert_close(to_np(x1), (x.double() + P.rms_norm(y.double()[:, :dim], w.double(), 1e-5)).numpy(), "float32", "stream alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_gate_and_head_gate(dtype):
    g = torch.Generator().manual_seed(5)
    T, m, V, L = 9, 7, 23, 3
    s = torch.randn(T, m + 3, generator=g) * 2.0
    table = torch.randn(V, L * m, generator=g).to(torch.bfloat16).float()
    ids = torch.randint(0, V, (T,), generator=g)
    for layer in range(L):
        out = torch.empty(T, m, dtype=td_of(dtype), device=DEV)
        ops.token_gate(s.to(DEV)[:, :m], table.to(DEV).to(td_of(dtype)), layer * m, i32(ids.tolist()), out)
        ref = P.gelu_tanh(s.double()[:, :m]) * table.double()[ids][:, layer * m:(layer + 1) * m]
        assert_close(to_np(out), ref.numpy(), dtype, f"columns of layer {layer}")
    H, hd, dv = 3, 16, 10
    att = torch.randn(T, H * hd, generator=g).to(td_of(dtype))
    gate = torch.randn(T, H + 2, generator=g) * 2.0
    out = torch.empty(T, H * dv, dtype=td_of(dtype), device=DEV)
    ops.head_gate(att.to(DEV), hd, gate.to(DEV)[:, 1:1 + H], out, H, dv)
    ref = att.double().view(T, H, hd)[:, :, :dv] * P.sigmoid(gate.double()[:, 1:1 + H])[:, :, None]
    assert_close(to_np(out), ref.reshape(T, H * dv).numpy(), dtype, "head gate")
    ops.head_gate(att.to(DEV), hd, None, out, H, dv)
    assert np.array_equal(to_np(out), att.double().view(T, H, hd)[:, :, :dv].reshape(T, H * dv).numpy())


def _delta_inputs(g, T, H, n, nv, rank, extreme=False):
    cols = 3 * H * n + 2 * H * nv + rank          # r, k, v, g, a, low
    rows = torch.randn(T, cols + 3, generator=g)
    w2 = (torch.randn(H * n, rank, generator=g) * 1.5).to(torch.bfloat16).float()
    w0, a0 = torch.randn(H * n, generator=g) * 2.0 - 1.0, torch.randn(H * n, generator=g)
    if extreme:                                    # decays at both ends, rates of exactly 0 and 1, a key of zeros
        w0[::3], w0[1::3] = 40.0, -40.0
        a0[::4], a0[2::4] = 60.0, -60.0
        rows[T // 2, H * n:2 * H * n] = 0.0
    return rows, w2, w0, a0


def _delta_plain(rows, w2, w0, a0, T, H, n, nv, rank):
    d = rows.double()
    k_off, v_off, g_off = H * n, 2 * H * n, 2 * H * n + H * nv
    a_off = g_off + H * nv
    low_off = a_off + H * n
    r, k = d[:, :k_off].view(T, H, n), d[:, k_off:v_off].view(T, H, n)
    v = d[:, v_off:g_off].view(T, H, nv)
    w = torch.exp(-P.DECAY_CONSTANT * P.sigmoid(torch.tanh(d[:, low_off:low_off + rank]) @ w2.double().T + w0.double())).view(T, H, n)
    a = P.sigmoid(d[:, a_off:low_off] + a0.double()).view(T, H, n)
    return r, k, v, w, a


@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("H,n,nv,rank", [(2, 32, 32, 12), (2, 64, 64, 6), (3, 24, 40, 5), (1, 130, 6, 3), (2, 256, 128, 8), (6, 7, 5, 1), (1, 520, 24, 4)])
def test_generalised_delta_rule_in_steps_of_any_size(H, n, nv, rank, wdtype):
    """Three sequences in slots out of order, fed in steps of 1, 2, 17 and 33 tokens and more: every step continues the
    recurrence from the slot's state; decays near 0 and 1, removal rates of 0 and 1, a key of zeros."""
    g = torch.Generator().manual_seed(H * n + nv)
    slots, lens = [4, 1, 2], [70, 1, 36]
    cuts = [[1, 2, 17, 33, 17], [1], [2, 34]]
    data = [_delta_inputs(g, L, H, n, nv, rank, extreme=True) for L in lens]
    w2, w0, a0 = data[0][1:]
    state = torch.zeros(6, H, n, nv, device=DEV)
    state[3] = 7.0                                                              # a slot nobody uses stays as it is
    done, got = [0, 0, 0], [[] for _ in lens]
    for r in range(5):
        live = [b for b in range(3) if r < len(cuts[b])]
        cnt = [cuts[b][r] for b in live]
        rows = torch.cat([data[b][0][done[b]:done[b] + c] for b, c in zip(live, cnt)]).to(DEV)
        T = rows.shape[0]
        prep = torch.empty(T, H, 5, n, device=DEV)
        k_off, v_off, g_off = H * n, 2 * H * n, 2 * H * n + H * nv
        a_off = g_off + H * nv
        ops.general_delta_prepare(rows, 0, k_off, a_off, a_off + H * n, w2.to(DEV).to(td_of(wdtype)), w0.to(DEV), a0.to(DEV),
                                  P.DECAY_CONSTANT, P.UNIT_EPS, prep, H, n)
        out = torch.empty(T, H * nv, device=DEV)
        ops.general_delta_scan(prep, rows[:, v_off:g_off], state, step_of(cnt, [slots[b] for b in live]), out, H, n, nv)
        o = 0
        for b, c in zip(live, cnt):
            got[b].append(out[o:o + c].cpu()); o += c; done[b] += c
    for b, L in enumerate(lens):
        r, k, v, w, a = _delta_plain(data[b][0], w2, w0, a0, L, H, n, nv, rank)
        ref, S = P.general_delta_scan(r, k, v, w, a)
        scale = max(1.0, float(ref.abs().max()))
        assert np.abs(torch.cat(got[b]).double().view(L, H, nv).numpy() - ref.numpy()).max() < 2e-5 * scale, b
        assert np.abs(to_np(state[slots[b]]) - S.numpy()).max() < 2e-5 * max(1.0, float(S.abs().max())), b
    assert float((state[3] - 7.0).abs().max()) == 0.0 and float(state[[0, 5]].abs().max()) == 0.0


def test_the_delta_rule_forgets_along_the_key_and_keeps_the_rest():
    """With w = 1 and a = 1 a token takes out of the state exactly what lies along its unit key: a value stored under a
    key is gone after the same key comes again with a zero value... and what was stored under a key at right angles stays."""
    n = 8
    e0, e1 = torch.zeros(n, dtype=torch.float64), torch.zeros(n, dtype=torch.float64)
    e0[0], e1[1] = 1.0, 1.0
    ones = torch.ones(3, 1, n, dtype=torch.float64)
    k = torch.stack([e0, e1, e0]).view(3, 1, n)
    v = torch.tensor([[2.0, 3.0], [5.0, 7.0], [0.0, 0.0]], dtype=torch.float64).view(3, 1, 2)
    r = torch.stack([e0, e0, e0 + e1]).view(3, 1, n)
    o, S = P.general_delta_scan(r, k, v, ones, ones)
    assert torch.allclose(o[:, 0], torch.tensor([[2.0, 3.0], [2.0, 3.0], [5.0, 7.0]], dtype=torch.float64), atol=1e-5)
    prep = torch.stack([r, k, ones, k, k], dim=2).float().to(DEV).contiguous()           # r, k, w, u, a * u
    out, state = torch.empty(3, 2, device=DEV), torch.zeros(1, 1, n, 2, device=DEV)
    ops.general_delta_scan(prep, v.view(3, 2).float().to(DEV), state, step_of([3], [0]), out, 1, n, 2)
    assert np.abs(to_np(out) - o[:, 0].numpy()).max() < 1e-5          # the plain unit key carries its 1e-6


def _paged(keys, values, hd, page, order, dtype):
    """keys [G, T, dk], values [G, T, dv] into a paged cache whose pages lie in `order`; heads of hd channels."""
    G, T, dk = keys.shape
    dv = values.shape[2]
    n_pages = -(-T // page)
    kc = torch.zeros(max(order) + 1, G, page, hd)
    vc = torch.zeros(max(order) + 1, G, page, hd)
    for j in range(T):
        kc[order[j // page], :, j % page, :dk] = keys[:, j]
        vc[order[j // page], :, j % page, :dv] = values[:, j]
    return kc.to(td_of(dtype)).to(DEV), vc.to(td_of(dtype)).to(DEV), i32([order[:n_pages]])


@pytest.mark.parametrize("window", [None, 1, 5, 64, 65, 200])
@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 64, 32), (2, 1, 16, 16), (8, 1, 128, 128), (3, 3, 24, 40)])
def test_sigmoid_weights_in_every_attention_kernel(H, G, dk, dv, window):
    """One sequence of 300 cached keys in pages that are not in order; the queries of the last 70 positions as a prompt's
    portion (any-shape kernel in both precisions, the tensor-core prefill kernel) and the last one alone (the split-key
    decode kernel).  One query and key are scaled so that a single far key, a key just inside and one just outside the
    window each carry a weight near 1 against small ones elsewhere."""
    g = torch.Generator().manual_seed(dk + dv + (window or 0))
    T, page, hd = 300, 64, max(dk, dv)
    order = [3, 0, 4, 1, 2]
    q = (torch.randn(T, H, dk, generator=g)).to(torch.bfloat16).float()
    k = (torch.randn(G, T, dk, generator=g)).to(torch.bfloat16).float()
    v = (torch.randn(G, T, dv, generator=g)).to(torch.bfloat16).float()
    bias = torch.tensor([-6.0, -2.0, 0.5, -4.0, -3.0, -5.0, 1.0, -1.0])[:H]
    scale = 1.0 / math.sqrt(dk)
    last = T - 1
    edges = [3, 63, 64] + ([last - window + 1, last - window] if window and 1 < window < T else [])
    for j in edges:                                 # keys that the last query's first head matches strongly
        if 0 <= j < T:
            k[0, j] = q[last, 0] * 3.0
    ref = P.sigmoid_attention(q.double(), k.double().transpose(0, 1), v.double().transpose(0, 1), scale, window, bias.double())
    gate = torch.randn(T, H + 3, generator=g) * 2.0          # a gate per token and head, in rows with a stride of their own
    ref_plain, ref = ref, ref * P.sigmoid(gate.double()[:, 1:1 + H])[:, :, None]
    gd = gate.to(DEV)
    rows = list(range(T - 70, T))
    for dtype in DTYPES:
        kc, vc, pages = _paged(k, v, hd, page, order, dtype)
        qq = torch.zeros(T, H, hd)
        qq[:, :, :dk] = q
        qd = qq.view(T, H * hd).to(td_of(dtype)).to(DEV)
        kernels = ["simt"] + (["auto", "mma"] if dtype == "bfloat16" else [])      # "auto": tcgen05 for prompts of heads of 64 / 128
        for kern in kernels:
            ops.options.attention = "simt" if kern == "simt" else "auto"
            ops.options.prefill_attention = "mma" if kern == "mma" else "tcgen05"
            try:
                batch = step_of([70], [0], [T - 70])
                out = torch.empty(70, H * hd, dtype=td_of(dtype), device=DEV)
                ops.attention(qd[T - 70:], H * hd, out, kc, vc, batch, H, G, hd, page, scale, window, pages,
                              scratch=lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV), gate_bias=bias.to(DEV),
                              out_gate=gd[T - 70:, 1:1 + H])
                got = to_np(out).reshape(70, H, hd)[:, :, :dv]
                bound = 2e-5 * max(1.0, float(ref.abs().max())) if dtype == "float32" else 1.5e-2 * float(ref[rows].abs().amax())
                assert np.abs(got - ref[rows].numpy()).max() < bound, (dtype, kern, "portion")
                batch = step_of([1], [0], [T - 1])
                out = torch.empty(1, H * hd, dtype=td_of(dtype), device=DEV)
                ops.attention(qd[T - 1:], H * hd, out, kc, vc, batch, H, G, hd, page, scale, window, pages,
                              scratch=lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV), gate_bias=bias.to(DEV),
                              out_gate=gd[T - 1:, 1:1 + H])
                got = to_np(out).reshape(1, H, hd)[:, :, :dv]
                assert np.abs(got - ref[[last]].numpy()).max() < bound, (dtype, kern, "alone")
                ops.attention(qd[T - 1:], H * hd, out, kc, vc, batch, H, G, hd, page, scale, window, pages,
                              scratch=lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV), gate_bias=bias.to(DEV))
                got = to_np(out).reshape(1, H, hd)[:, :, :dv]
                assert np.abs(got - ref_plain[[last]].numpy()).max() < bound, (dtype, kern, "alone, no gate")
                ops.check_kernel_errors()
            finally:
                ops.options.attention, ops.options.prefill_attention = "auto", "tcgen05"
    if window and 1 < window < T:
        # the window shows: one key more moves the last row far beyond any bound
        a = P.sigmoid_attention(q.double(), k.double().transpose(0, 1), v.double().transpose(0, 1), scale, window + 1, bias.double())
        assert (a[last, 0] - ref_plain[last, 0]).abs().max() > 0.3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,E,top,F,D", [(5, 6, 2, 24, 64), (70, 10, 3, 48, 256), (40, 4, 4, 8, 48), (300, 10, 2, 96, 256)])
def test_clamped_experts_few_tokens_and_grouped(dtype, T, E, top, F, D):
    g = torch.Generator().manual_seed(T + E)
    limit = 1.25
    h = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    Wg = (torch.randn(E, F, D, generator=g) * (2.5 / math.sqrt(D))).to(torch.bfloat16).float()
    Wu = (torch.randn(E, F, D, generator=g) * (2.5 / math.sqrt(D))).to(torch.bfloat16).float()
    Wd = (torch.randn(E, D, F, generator=g) / math.sqrt(F)).to(torch.bfloat16).float()
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)])
    wts = torch.rand(T, top, generator=g)
    ref = torch.zeros(T, D, dtype=torch.float64)
    hidden_all = []
    for t in range(T):
        for r in range(top):
            e = int(ids[t, r])
            ref[t] += wts[t, r].double() * P.expert(h[t].double(), Wg[e].double(), Wu[e].double(), Wd[e].double(), limit, P._keep)
            hidden_all.append((h[t].double() @ Wg[e].double().T))
    assert max(float(x.max()) for x in hidden_all) > limit            # the clamp is reached
    from herbert_rs_b200.parts.swiglu import join_gate_up
    joined = [join_gate_up(Wg[e].to(td_of(dtype)).to(DEV), Wu[e].to(td_of(dtype)).to(DEV)) for e in range(E)]
    up = torch.stack([j[0] for j in joined]).contiguous()
    layout = ops.GATED_GROUPS_OF_8 if joined[0][1] else ops.GATED_HALVES
    down = Wd.to(td_of(dtype)).to(DEV)
    hd_, idd, wd = h.to(td_of(dtype)).to(DEV), ids.to(torch.int32).to(DEV), wts.to(DEV)
    y = torch.zeros(T, D, device=DEV)
    mid = torch.empty(T * top, F, dtype=td_of(dtype), device=DEV)
    ops.moe_experts(hd_, up, down, idd, wd, mid, y, ops.ACT_SWISH_CLAMP, accumulate=False, gated=layout, act_limit=limit)
    assert_close(to_np(y), ref.numpy(), dtype, "few-token experts")
    if dtype == "bfloat16" and ops.moe_grouped_ok(hd_, up, layout):
        y2 = torch.ones(T, D, device=DEV)
        ops.moe_experts_grouped(hd_, up, down, idd, wd, y2, ops.ACT_SWISH_CLAMP, True, lambda s, dt: torch.empty(s, dtype=dt, device=DEV),
                                gated=layout, act_limit=limit)
        assert_close(to_np(y2) - 1.0, ref.numpy(), dtype, "grouped experts")
    if dtype == "bfloat16" and ops.moe_tc_ok(hd_, up, top, layout, ops.ACT_SWISH_CLAMP):
        y3 = torch.ones(T, D, device=DEV)
        ops.moe_experts_tc(hd_, up, down, idd, wd, y3, True, lambda s, dt: torch.empty(s, dtype=dt, device=DEV), act_limit=limit)
        ops.check_kernel_errors()
        assert_close(to_np(y3) - 1.0, ref.numpy(), dtype, "experts on tcgen05")
        assert T * top >= 512


@pytest.mark.parametrize("E,groups,keep,top", [(12, 4, 2, 3), (6, 3, 2, 2), (8, 1, 1, 8), (8, 8, 3, 3), (4, 2, 1, 2), (5, 1, 1, 1)])
def test_router_with_groups_that_score_as_their_best_expert(E, groups, keep, top):
    g = torch.Generator().manual_seed(E * groups + top)
    T, D = 50, 40
    h = torch.randn(T, D, generator=g)
    R = torch.randn(E, D, generator=g) * 0.5
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    ops.moe_route(h.to(DEV), R.to(DEV), ids, wts, top, False, 0, groups, keep, 1, 1.0)
    z = h.double() @ R.double().T
    differs = 0
    for t in range(T):
        chosen, weights = P.route(z[t], top, groups, keep)
        assert ids[t].tolist() == chosen, t
        assert np.abs(to_np(wts[t]) - np.array([float(x) for x in weights])).max() < 1e-6
        differs += chosen != P.route(z[t], top, 1, 1)[0]
    if keep < groups and top > keep:
        assert differs > 0            # the groups change the choice for some tokens (never while top <= keep: the best
                                      # experts' groups are the best groups)


# ---- whole models ---------------------------------------------------------------------------------
ALONE = {
    "attention": [(U.attention(), None)],
    "attention_ff": [(U.attention(heads=2, kv_heads=2, dim=8, vdim=24, conv=4, window=7), U.moe())],
    "attention_no_window_no_scaling_no_conv": [(U.attention(window=None, scaling=None, conv=None, heads=2, kv_heads=1), None)],
    "attention_no_rotation_conv_of_one": [(U.attention(rot_dims=0, conv=1, window=1, heads=1, kv_heads=1, dim=16, vdim=16), None)],
    "attention_sharp_heads_of_64": [(U.attention(heads=4, kv_heads=1, dim=64, vdim=64, window=33, sharp=3.0, rot_dims=32), None)],
    "delta": [(U.delta(), None)],
    "delta_ff_one_head": [(U.delta(heads=1, dim=24), U.moe(experts=4, top=4, groups=2, keep=2))],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_one_layer_of_each_kind(tmp_path, which, dtype):
    d, pm = U.make(tmp_path / which, ALONE[which], seed=len(which))
    ids = ids_for(np.random.default_rng(1), VOCAB, 70)
    eng = engine_for(d, dtype, max_tokens=512)
    ref = pm.logits(ids).numpy()
    assert_close(replay_whole(eng, ids), ref, dtype, which, plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 69), ref, dtype, which + " token by token", plain=pm, ids=ids)


def test_the_residual_stream_after_every_layer(mixed):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(4), VOCAB, 33)
    want = pm.layers(ids)
    eng = engine_for(d, "float32", max_tokens=256)
    got = []
    for b in eng.model.blocks:
        def run(x, batch, cache, inner=b.forward, **kw):
            out = inner(x, batch, cache, **kw)
            got.append(to_np(x))
            return out
        b.forward = run
    replay_whole(eng, ids)
    assert len(got) == len(want) == 4
    for i, (a, b) in enumerate(zip(got, want)):
        assert np.abs(a - b.numpy()).max() < 3e-5 * float(b.abs().max()), i


def test_the_test_models_routers_are_decisive(mixed):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(2), VOCAB, 150)
    assert U.router_margins(pm, ids) > 0.5


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_token_by_token_and_pieces(mixed, dtype):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(2), VOCAB, 150)
    ref = pm.logits(ids).numpy()
    eng = engine_for(d, dtype, max_tokens=1024)
    assert_close(replay_whole(eng, ids), ref, dtype, "whole", plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 149), ref, dtype, "one by one", plain=pm, ids=ids)
    for piece in (2, 3, 16, 21, 64, 71):
        s, rows = eng.alloc_slot(), []
        for at in range(0, len(ids), piece):
            rows.append(to_np(eng.step([(s, ids[at:at + piece])], "all")))
        eng.free_slot(s)
        assert_close(np.concatenate(rows), ref, dtype, f"pieces of {piece}", plain=pm, ids=ids)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_in_slots_and_pages_that_were_used_before(mixed, dtype):
    """Three slots serve eight requests: the recurrent states, the convolutions' inputs and the pages of a slot's former
    user must not reach its next one (a request of one token reads nothing but zeros)."""
    d, pm = mixed
    rng = np.random.default_rng(3)
    reqs = [ids_for(rng, VOCAB, n) for n in (1, 37, 80, 5, 64, 23, 2, 70)]
    refs = [pm.logits(r).numpy() for r in reqs]
    eng = engine_for(d, dtype, max_tokens=64 * 5, max_slots=3)
    got = replay_batches(eng, reqs, [1, 30, 64, 2, 40, 23, 1, 65], [[0, 1, 2], [3, 4], [5, 6, 7]])
    for i, (g, ref) in enumerate(zip(got, refs)):
        assert_close(g, ref, dtype, f"request {i}", plain=pm, ids=reqs[i])
    assert eng.cache.slots.free_count == 3


def _with_windows(pm, sizes):
    cfg = copy.deepcopy(pm.cfg)
    att = [l for l in cfg["layers"] if l["type"] == "attention"]
    for layer, size in zip(att, sizes):
        layer["mixer"]["mask"] = {"size": size}
    return P.PlainNefivik(config=cfg, tensors=pm.W)


@pytest.mark.parametrize("window,reader", [(1, 3), (12, 12), (16, 40), (17, 5), (64, 65), (65, 64), (70, 100)])
def test_a_window_one_key_off_shows_in_prompts_and_in_decoding(tmp_path, window, reader):
    """Sharp attention (large scores against negative biases: a few keys carry each sum), pages of 16 keys, a second
    layer that reads the first one's keys through a window of its own, shorter or longer: the key that has just left a
    window and the one just inside it are told apart at every position past the window, in a prompt, in a prompt's second
    portion and token by token.  A longer reader's window also shows that the first layer's pages stay long enough."""
    layers = [(U.attention(heads=2, kv_heads=1, dim=16, vdim=16, window=window, sharp=5.0, conv=2), None),
              (U.attention(heads=2, kv_heads=1, dim=16, vdim=16, window=reader, sharp=5.0, conv=2, kv_from=0), None)]
    d, pm = U.make(tmp_path / "w", layers, seed=window, side=None)
    ids = ids_for(np.random.default_rng(window), VOCAB, 150)
    ref = pm.logits(ids).numpy()
    eng = engine_for(d, "float32", max_tokens=16 * 40, page_size=16)
    runs = {"whole": replay_whole(eng, ids), "decoded": replay_tail_one_by_one(eng, ids, 130)}
    s = eng.alloc_slot()
    cut = min(window, reader) + 3
    runs["portions"] = np.concatenate([to_np(eng.step([(s, ids[:cut])], "all")), to_np(eng.step([(s, ids[cut:])], "all"))])
    eng.free_slot(s)
    wrong = [_with_windows(pm, (window + 1, reader)), _with_windows(pm, (window, reader + 1))]
    if window > 1:
        wrong.append(_with_windows(pm, (window - 1, reader)))
    if reader > 1:
        wrong.append(_with_windows(pm, (window, reader - 1)))
    wrong = [w.logits(ids).numpy() for w in wrong]
    for what, got in runs.items():
        assert np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), what
        for other in wrong:
            far_off = np.abs(got - other).max(axis=-1) > 1e-2
            assert far_off.sum() > (len(ids) - max(window, reader)) // 10, what
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_tokens_far_back_stay_in_the_states(tmp_path, dtype):
    """Decays near 1 and small removal rates: the first tokens of 400 still move the last logits, and the engine has
    them whether the prompt came at once, in portions, or mostly token by token."""
    layers = [(U.delta(heads=2, dim=16), None), (U.attention(window=8), None)]
    d, pm = U.make(tmp_path / "far", layers, seed=21)
    W = dict(pm.W)
    W["l0.mix.w0"] = W["l0.mix.w0"] * 0 - 9.0             # decays near 1
    W["l0.mix.w2"] = W["l0.mix.w2"] * 0.1
    W["l0.mix.a.b"] = W["l0.mix.a.b"] * 0 - 7.0           # hardly anything is removed
    W["l0.mix.a"] = W["l0.mix.a"] * 0.1
    U.write(pm.cfg, {k: v.to(torch.bfloat16) for k, v in W.items()}, d)
    pm = P.PlainNefivik(d)
    ids = ids_for(np.random.default_rng(6), VOCAB, 400)
    rows = list(range(380, 400))
    ref = pm.logits(ids).numpy()[rows]
    other = pm.logits([(t + 1) % VOCAB for t in ids[:4]] + ids[4:]).numpy()[rows]
    assert np.abs(other - ref).max(axis=-1).min() > 1e-3
    eng = engine_for(d, dtype, max_tokens=2048)
    for cuts in ([400], [7, 200, 193], [300] + [1] * 100):
        s, got, at = eng.alloc_slot(), [], 0
        for n in cuts:
            want = [r - at for r in rows if at <= r < at + n]
            out = eng.step([(s, ids[at:at + n])], [want])
            if want:
                got.append(to_np(out))
            at += n
        eng.free_slot(s)
        assert_close(np.concatenate(got), ref, dtype, f"cuts {cuts[:3]}", plain=pm, ids=ids, rows=rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(mixed, dtype):
    """Prompts of 1 to 5 tokens (shorter than the convolutions, the windows and a page), alone and as a batch."""
    d, pm = mixed
    rng = np.random.default_rng(8)
    reqs = [ids_for(rng, VOCAB, n) for n in (1, 2, 3, 4, 5)]
    eng = engine_for(d, dtype, max_tokens=512)
    for r in reqs:
        assert_close(replay_whole(eng, r), pm.logits(r).numpy(), dtype, f"{len(r)} tokens", plain=pm, ids=r)
        assert_close(replay_tail_one_by_one(eng, r, len(r) - 1), pm.logits(r).numpy(), dtype, f"{len(r)} tokens one by one", plain=pm, ids=r)
    got = replay_batches(eng, reqs, [1, 1, 2, 4, 3], [[0, 1, 2, 3, 4]])
    for g, r in zip(got, reqs):
        assert_close(g, pm.logits(r).numpy(), dtype, "batch of short prompts", plain=pm, ids=r)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_small_pages(tmp_path, dtype):
    layers = [(U.attention(window=40, sharp=2.0), U.moe()), (U.delta(), None), (U.attention(window=17, kv_from=0, sharp=2.0), None)]
    d, pm = U.make(tmp_path / "long", layers, seed=9)
    ids = ids_for(np.random.default_rng(9), VOCAB, 190)
    ref = pm.logits(ids).numpy()
    page = 16 if dtype == "float32" else 64       # the tensor-core kernels read pages in tiles of 64 keys
    eng = engine_for(d, dtype, max_tokens=page * 20, page_size=page)
    assert_close(replay_tail_one_by_one(eng, ids, 170), ref, dtype, "170 decoded tokens", plain=pm, ids=ids)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_and_its_continuation(tmp_path, dtype):
    """600 tokens at once and in two portions (several tiles of queries, of keys and of expert pairs), then 24 more."""
    layers = [(U.attention(heads=4, kv_heads=2, dim=64, vdim=32, window=80, rot_dims=16, conv=3), U.moe(experts=8, top=3, ff=48, groups=4, keep=2)),
              (U.delta(heads=2, dim=64), U.moe(experts=8, top=3, ff=48, groups=4, keep=2))]
    d, pm = U.make(tmp_path / "p600", layers, seed=12, width=128)
    ids = ids_for(np.random.default_rng(12), VOCAB, 624)
    rows = [0, 1, 63, 64, 79, 80, 81, 299, 300, 511, 512, 599] + list(range(600, 624))
    ref = pm.logits(ids, torch.float32).double().numpy()[rows]
    eng = engine_for(d, dtype, max_tokens=2048)
    for cuts in ([600], [300, 300]):
        s, got, at = eng.alloc_slot(), [], 0
        for n in cuts + [1] * 24:
            want = [r - at for r in rows if at <= r < at + n]
            out = eng.step([(s, ids[at:at + n])], [want])
            if want:
                got.append(to_np(out))
            at += n
        eng.free_slot(s)
        bound = None if dtype == "bfloat16" else 1e-3 * max(1.0, float(np.abs(ref).max()))
        assert_close(np.concatenate(got), ref, dtype, f"cuts {cuts}", plain=pm, ids=ids, rows=rows, arith=torch.float32, bound=bound)


OTHER = {
    "one_head_top_one_of_two": [(U.attention(heads=1, kv_heads=1, dim=16, vdim=16), U.moe(experts=2, top=1, groups=1, keep=1)),
                                (U.delta(heads=1, dim=8), U.moe(experts=2, top=1, groups=2, keep=1))],
    "sizes_no_tile_divides": [(U.attention(heads=6, kv_heads=3, dim=10, vdim=20, rot_dims=6, conv=7, window=33), U.moe(experts=9, top=4, ff=20, groups=3, keep=2)),
                              (U.delta(heads=5, dim=7), None)],
    "values_wider_than_keys_heads_equal": [(U.attention(heads=3, kv_heads=3, dim=16, vdim=96, window=None), None),
                                           (U.attention(heads=3, kv_heads=3, dim=16, vdim=96, window=5, kv_from=0), U.moe())],
    "two_readers_of_one_layer": [(U.attention(window=6), None), (U.attention(window=30, kv_from=0, conv=None), None), (U.delta(), None),
                                 (U.attention(window=None, kv_from=0, rot_dims=16), U.moe(top=4, groups=3, keep=3))],
    "delta_first_heads_of_160": [(U.delta(heads=1, dim=160), U.moe()), (U.attention(heads=2, kv_heads=2, dim=160, vdim=32, rot_dims=64), None)],
    "all_experts_chosen": [(U.delta(heads=2, dim=32), U.moe(experts=4, top=4, groups=1, keep=1, limit=0.5))],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(OTHER))
def test_other_sizes_and_orders(tmp_path, which, dtype):
    kw = {"width": 96, "side": 9} if which == "sizes_no_tile_divides" else ({"side": None} if which == "two_readers_of_one_layer" else {})
    d, pm = U.make(tmp_path / which, OTHER[which], seed=len(which), **kw)
    ids = ids_for(np.random.default_rng(5), VOCAB, 90)
    ref = pm.logits(ids).numpy()
    eng = engine_for(d, dtype, max_tokens=1024)
    assert_close(replay_whole(eng, ids), ref, dtype, which, plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 50), ref, dtype, which + " decoded", plain=pm, ids=ids)
    s = eng.alloc_slot()
    rows = [to_np(eng.step([(s, ids[:37])], "all")), to_np(eng.step([(s, ids[37:39])], "all")), to_np(eng.step([(s, ids[39:])], "all"))]
    eng.free_slot(s)
    assert_close(np.concatenate(rows), ref, dtype, which + " in portions", plain=pm, ids=ids)
    eng.cache.check()


def test_random_routers_in_32_bit(tmp_path):
    layers = [(U.attention(), U.moe(experts=9, top=3, groups=3, keep=2)), (U.delta(), U.moe(experts=8, top=2, groups=4, keep=2))]
    d, pm = U.make(tmp_path / "rr", layers, seed=31, decisive_router=False)
    ids = ids_for(np.random.default_rng(31), VOCAB, 120)
    eng = engine_for(d, "float32", max_tokens=512)
    ref = pm.logits(ids).numpy()
    got = replay_whole(eng, ids)
    close = np.abs(got - ref).max(axis=-1) < 1e-4 * max(1.0, np.abs(ref).max())
    assert close.mean() > 0.97            # a close call between two experts may move a token, hardly ever does


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_steps_equal_eager_ones(mixed, dtype):
    d, pm = mixed
    rng = np.random.default_rng(11)
    reqs = [ids_for(rng, VOCAB, n) for n in (40, 70)]
    out = []
    for graphs in (True, False):
        eng = engine_for(d, dtype, max_tokens=1024, use_graphs=graphs)
        out.append(replay_batches(eng, reqs, [10, 33], [[0, 1]]))
        if graphs:
            assert eng.graph_replays > 20
    for a, b in zip(*out):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_any_shape_attention_kernel_agrees_with_the_tensor_core_ones(mixed, dtype):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(12), VOCAB, 100)
    ref = pm.logits(ids).numpy()
    ops.options.attention = "simt"
    try:
        eng = engine_for(d, dtype, max_tokens=512)
        assert_close(replay_tail_one_by_one(eng, ids, 20), ref, dtype, "simt", plain=pm, ids=ids)
    finally:
        ops.options.attention = "auto"


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(mixed, dtype):
    d, pm = mixed
    eng = engine_for(d, dtype, max_tokens=2048)
    rng = np.random.default_rng(15)
    prompts = [ids_for(rng, VOCAB, n) for n in (9, 1, 30, 4, 17)]
    res = hb.generate(eng, prompts, hb.GenerationOptions(max_tokens=10, ignore_eos=True, max_batch=3),
                      hb.SamplingParams(temperature=0.0))
    assert res.stats.batches == 2 and all(len(t) == 10 for t in res.tokens)
    for p, got in zip(prompts, res.tokens):
        ids = list(p)
        for tok in got:
            ref = pm.logits(ids)[-1].numpy()
            margin = 1e-4 if dtype == "float32" else 2 * bound_for(pm, ids, dtype, ref, rows=[len(ids) - 1])
            assert ref.max() - ref[tok] <= margin
            ids.append(tok)
    eng.cache.check()
    assert eng.cache.slots.free_count == eng.cache.num_slots


def test_random_weights_from_the_configuration(tmp_path):
    cfg = U.config([(U.attention(), U.moe()), (U.delta(), None), (U.attention(kv_from=0), None)])
    hb.write_random_model(cfg, str(tmp_path), seed=1)
    pm = P.PlainNefivik(str(tmp_path))
    assert {k: tuple(v.shape) for k, v in pm.W.items() if ".w1" not in k and ".w2" not in k} == \
           {k: tuple(v.shape) for k, v in U.weights(cfg).items() if ".w1" not in k and ".w2" not in k}
    assert pm.W["side.embed"].shape == (VOCAB, 15)
    ids = ids_for(np.random.default_rng(1), VOCAB, 50)
    eng = engine_for(str(tmp_path), "float32", max_tokens=256)
    got, ref = replay_whole(eng, ids), pm.logits(ids).numpy()
    assert (np.abs(got - ref).max(axis=-1) < 1e-4 * max(1.0, np.abs(ref).max())).mean() > 0.9      # random routers


def test_command_line_trace_replay_and_prompts_in_pieces(mixed, tmp_path, capsys):
    """The design through the library's other entry points: the command line, `bin/trace_run`, and the
    generation loop with prompts fed in pieces and sampling on the device."""
    import json
    import os
    import subprocess
    import sys
    from herbert_rs_b200 import cli
    d, pm = mixed
    rng = np.random.default_rng(21)
    a, b = ids_for(rng, VOCAB, 40), ids_for(rng, VOCAB, 7)
    assert cli.main(["--model", d, "--prompt-ids", ",".join(map(str, a)), "--prompt-ids", ",".join(map(str, b)),
                     "--max-tokens", "5", "--temperature", "0", "--ignore-eos", "--backend", "cuda-fp32"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2
    ids = list(a)
    for tok in map(int, lines[0].split(",")):
        ref = pm.logits(ids)[-1].numpy()
        assert ref.max() - ref[tok] <= 1e-4
        ids.append(tok)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[6:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:32], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in DTYPES:
        out = tmp_path / ("trace_" + dtype)
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
        assert r.returncode == 0 and [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
        ra, rb = pm.logits(a).numpy(), pm.logits(b).numpy()
        read = lambda n, rows: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(rows, VOCAB).astype(np.float64)      # noqa: E731
        assert_close(read(0, 2), ra[[0, 29]], dtype, "trace step 0", plain=pm, ids=a, rows=[0, 29])
        assert_close(read(1, 2)[:1], ra[[30]], dtype, "trace step 1 a", plain=pm, ids=a, rows=[30])
        assert_close(read(1, 2)[1:], rb[[6]], dtype, "trace step 1 b", plain=pm, ids=b, rows=[6])
        assert_close(read(2, 1), ra[[31]], dtype, "trace step 2", plain=pm, ids=a, rows=[31])
    outs = []
    for piece in (None, 16):
        eng = engine_for(d, "float32", max_tokens=1024)
        res = hb.generate(eng, [a, b], hb.GenerationOptions(max_tokens=8, ignore_eos=True, prefill_chunk_size=piece),
                          hb.SamplingParams(temperature=0.8, top_k=20, top_p=0.95, seed=5))
        outs.append(res.tokens)
    assert outs[0] == outs[1]
