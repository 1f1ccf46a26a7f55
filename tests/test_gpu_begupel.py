"""The Begupel design in the engine against the plain implementation (`plain_begupel.py`): every
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
import plain_begupel as P
import begupel_util as U
from gpu_util import (DTYPES, assert_close, bound_for, engine_for, replay_batches, replay_tail_one_by_one, replay_whole, to_np)
from herbert_rs_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
VOCAB = 131


def ids_for(rng, vocab, n):
    return rng.integers(0, vocab, n).tolist()


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
                           n_tokens=int(sum(lens)), max_q_len=max(lens))


@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    """Both layer kinds, each with and without a feed-forward; key and value sizes that differ; a window shorter than a
    page; partly rotated keys."""
    layers = [(U.parallel(heads=4, kv_heads=2, dim=16, vdim=32, window=12, rot_dims=8), U.dense(48)),
              (U.lightning(heads=2, dim=16, vdim=8), None),
              (U.parallel(heads=2, kv_heads=2, dim=64, vdim=16, window=70, rheads=2, rkv=1, rdim=32, rvdim=16, conv=3), None),
              (U.lightning(heads=3, dim=8, vdim=24, decay=[0.5, 0.97, 1.0]), U.dense(40))]
    return U.make(tmp_path_factory.mktemp("begupel_mixed"), layers, seed=3)


# ---- each mechanism alone -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,groups", [(48, 1), (48, 2), (60, 5), (1024, 4), (4608, 2), (64, 64)])
def test_rms_norm_in_groups_alone_and_on_the_way_into_the_stream(dtype, dim, groups):
    g = torch.Generator().manual_seed(dim + groups)
    y = torch.randn(7, dim + 8, generator=g) * torch.linspace(0.1, 5.0, dim + 8)      # parts of very different size
    x, w, bias = torch.randn(7, dim, generator=g), 1.0 + 0.2 * torch.randn(dim, generator=g), torch.randn(dim, generator=g)
    rows = [5, 0, 6]
    out = torch.empty(3, dim, dtype=td_of(dtype), device=DEV)
    ops.group_rmsnorm(x.to(DEV), w.to(DEV), out, 1e-5, groups, i32(rows))
    assert_close(to_np(out), P.group_norm(x.double()[rows], w.double(), groups, 1e-5).numpy(), dtype, "norm of rows")
    for b in (None, bias):
        x1, h = x.clone().to(DEV), torch.empty(7, dim, dtype=td_of(dtype), device=DEV)
        ops.group_rmsnorm_residual(y.to(DEV)[:, :dim], w.to(DEV), x1, h, 1e-5, groups, td_of(dtype), bias=None if b is None else b.to(DEV))
        yy = y.double()[:, :dim] + (0.0 if b is None else b.double())
        ref = x.double() + P.group_norm(yy, w.double(), groups, 1e-5)
        assert_close(to_np(x1), ref.numpy(), "float32", "stream")
        assert_close(to_np(h), ref.numpy(), dtype, "next input")
    # the sum of two arrays with two constants, normed in the same pass
    z = torch.randn(7, dim + 3, generator=g) * 2.0
    x1, h = x.clone().to(DEV), torch.empty(7, dim, dtype=td_of(dtype), device=DEV)
    ops.group_rmsnorm_residual(y.to(DEV)[:, :dim], w.to(DEV), x1, h, 1e-5, groups, td_of(dtype), bias=bias.to(DEV),
                               second=(z.to(DEV)[:, :dim], 1.25, -0.6))
    ref = x.double() + P.group_norm(1.25 * y.double()[:, :dim] - 0.6 * z.double()[:, :dim] + bias.double(), w.double(), groups, 1e-5)
    assert_close(to_np(x1), ref.numpy(), "float32", "stream, two arrays")
    assert_close(to_np(h), ref.numpy(), dtype, "next input, two arrays")
    if groups > 1:       # one norm over the whole row is something else
        assert (P.group_norm(x.double(), w.double(), groups, 1e-5) - P.group_norm(x.double(), w.double(), 1, 1e-5)).abs().max() > 1e-2


@pytest.mark.parametrize("taps,add,silu", [(4, True, False), (4, False, True), (2, False, True), (1, True, False), (7, False, False)])
def test_short_convolution_continues_from_its_state(taps, add, silu):
    """Three sequences in slots that are not in order, fed in steps of unequal sizes (some shorter than the state):
    every step continues the convolution of the whole sequence; a slot handed out again starts from zeros."""
    g = torch.Generator().manual_seed(taps)
    C, slots = 70, [4, 1, 2]
    lens = [23, 1, 9]
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, C, generator=g) for n in lens]
    state = torch.zeros(6, max(taps - 1, 0), C, device=DEV) if taps > 1 else None
    cuts = [[1, 1, 2, 5, 14], [1], [2, 7]]
    done, got = [0, 0, 0], [[] for _ in lens]
    for r in range(5):
        live = [b for b in range(3) if r < len(cuts[b])]
        n = [cuts[b][r] for b in live]
        inp = torch.cat([seqs[b][done[b]:done[b] + k] for b, k in zip(live, n)])
        wide = torch.zeros(inp.shape[0], C + 5)
        wide[:, :C] = inp                                                    # rows with a stride of their own
        batch = step_of(n, [slots[b] for b in live], [done[b] for b in live])
        out = torch.empty(inp.shape[0], C, device=DEV)
        ops.short_conv(wide.to(DEV)[:, :C], w.to(DEV), state, batch, out, add_input=add, silu=silu)
        o = 0
        for b, k in zip(live, n):
            got[b].append(out[o:o + k].cpu()); o += k; done[b] += k
    for b in range(3):
        ref = P.causal_conv(seqs[b].double(), w.double())
        ref = ref + seqs[b].double() if add else ref
        ref = P.silu(ref) if silu else ref
        assert np.abs(torch.cat(got[b]).double().numpy() - ref.numpy()).max() < 2e-5, b
    if taps > 1:
        assert float(state[[0, 3, 5]].abs().max()) == 0.0                    # no other slot was touched
        assert np.abs(to_np(state[4]) - seqs[0][-(taps - 1):].double().numpy()).max() == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_with_the_row_of_the_token_pair(dtype):
    """The first token of a sequence takes the table's last row; a step's first token takes its predecessor from the
    slot's state; multipliers whose products pass 32 bits."""
    td = td_of(dtype)
    g = torch.Generator().manual_seed(4)
    V, D, n, mp, mc = 50000, 24, 97, 1000003, 77777
    E, B = torch.randn(V, D, generator=g).to(td), torch.randn(n + 1, D, generator=g).to(td)
    cfg = {"embedding": {"bigram": {"buckets": n, "mul_prev": mp, "mul_cur": mc}}}
    W = {"embed": E.float(), "bigram": B.float()}
    a, b = [49999, 49998, 3, 3, 0, 17, 41234], [7, 7]
    last = torch.full((5, 1), 12345, dtype=torch.int32, device=DEV)          # stale ids of the slots' former users
    out1 = torch.zeros(5, D, device=DEV)
    ops.pair_embed(E.to(DEV), B.to(DEV), step_of([4, 1], [3, 0], ids=a[:4] + b[:1]), last, out1, n, mp, mc)
    out2 = torch.zeros(4, D, device=DEV)
    ops.pair_embed(E.to(DEV), B.to(DEV), step_of([3, 1], [3, 0], [4, 1], ids=a[4:] + b[1:]), last, out2, n, mp, mc)
    ra, rb = P.embedding(a, W, cfg, torch.float64), P.embedding(b, W, cfg, torch.float64)
    got_a, got_b = torch.cat([out1[:4], out2[:3]]), torch.cat([out1[4:], out2[3:]])
    assert np.abs(to_np(got_a) - ra.numpy()).max() < 1e-6 and np.abs(to_np(got_b) - rb.numpy()).max() < 1e-6
    assert last.view(-1).tolist() == [7, 12345, 12345, 41234, 12345]
    assert float((ra[0] - E[a[0]].double() - B[n].double()).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("halves", [False, True])
@pytest.mark.parametrize("H,G,dk,dv,rot", [(4, 2, 16, 16, 16), (3, 1, 24, 8, 10), (2, 2, 8, 40, 0), (1, 1, 64, 64, 32)])
def test_whole_projection_norm_rotation_of_pairs_cache_and_the_turn_back(dtype, halves, H, G, dk, dv, rot):
    """q and k normed over all heads at once, pairs turned at positions up to a few thousand, values turned over all their
    channels and stored in pages that are not in order; then the turn back brings a rotated value to where it was."""
    td = td_of(dtype)
    g = torch.Generator().manual_seed(H * dk + dv)
    page, hd = 16, max(dk, dv)
    pos = [0, 1, 15, 16, 17, 2047, 5000, 31, 32]
    seq = [0] * 7 + [1] * 2
    pages = torch.full((2, 320), 0, dtype=torch.int32)
    pages[0, [0, 1, 127, 312]] = torch.tensor([5, 2, 7, 0], dtype=torch.int32)
    pages[1, [1, 2]] = torch.tensor([3, 1], dtype=torch.int32)
    T = len(pos)
    rows = torch.randn(T, H * dk + G * (dk + dv), generator=g)
    wq, wk = 1 + 0.2 * torch.randn(H * dk, generator=g), 1 + 0.2 * torch.randn(G * dk, generator=g)
    layout = "halves" if halves else "interleaved"
    fqk = (P.pair_frequencies(10000.0, rot, torch.float64) / 2.0) if rot else None
    fv = P.pair_frequencies(10000.0, dv, torch.float64)
    cache = torch.zeros(2, 8, G, page, hd, dtype=td, device=DEV)
    q = torch.zeros(T, H * hd, dtype=td, device=DEV)
    batch = SimpleNamespace(tok_seq=i32(seq), tok_pos=i32(pos))
    ops.qkv_rotary_cache(rows.to(DEV), wq.to(DEV), wk.to(DEV), 1e-5, fqk.float().to(DEV) if rot else None, rot, halves,
                         fv.float().to(DEV), batch, pages.to(DEV), q, cache[0], cache[1], H, G, dk, dv, hd, page)
    p64 = torch.tensor(pos, dtype=torch.float64)
    rq = P.rms_norm(rows[:, :H * dk].double(), wq.double(), 1e-5).view(T, H, dk)
    rk = P.rms_norm(rows[:, H * dk:(H + G) * dk].double(), wk.double(), 1e-5).view(T, G, dk)
    rv = rows[:, (H + G) * dk:].double().view(T, G, dv)
    if rot:
        ang = p64[:, None, None] * fqk[None, None, :]
        rq = torch.cat([P.turn_pairs(rq[..., :rot], ang, layout), rq[..., rot:]], -1)
        rk = torch.cat([P.turn_pairs(rk[..., :rot], ang, layout), rk[..., rot:]], -1)
    angv = p64[:, None, None] * fv[None, None, :]
    rvt = P.turn_pairs(rv, angv, layout)
    # the float product position * frequency itself is off by up to 2^-24 of the angle
    slack = 5000 * 2.0 ** -23 * 4 if dtype == "float32" else None
    qg = to_np(q).reshape(T, H, hd)
    assert_close(qg[..., :dk], rq.numpy(), dtype, "q", bound=slack)
    assert np.abs(qg[..., dk:]).max(initial=0.0) == 0.0
    for t in range(T):
        pg = int(pages[seq[t], pos[t] // page])
        kk, vv = to_np(cache[0, pg, :, pos[t] % page]), to_np(cache[1, pg, :, pos[t] % page])
        assert_close(kk[:, :dk], rk[t].numpy(), dtype, f"k of token {t}", bound=slack)
        assert_close(vv[:, :dv], rvt[t].numpy(), dtype, f"v of token {t}", bound=slack)
        assert np.abs(kk[:, dk:]).max(initial=0.0) == 0.0 and np.abs(vv[:, dv:]).max(initial=0.0) == 0.0
    assert int((cache != 0).sum()) <= T * G * (dk + dv)
    # the turn back: a head's "result" that is one rotated value comes back as the value itself
    att = torch.zeros(T, H * hd, dtype=td, device=DEV)
    att.view(T, H, hd)[..., :dv] = rvt[:, [h // (H // G) for h in range(H)]].to(td).to(DEV)
    y = torch.empty(T, H * dv, dtype=td, device=DEV)
    ops.rotate_heads_back(att, hd, fv.float().to(DEV), halves, i32(pos), y, H, dv)
    want = rv[:, [h // (H // G) for h in range(H)]].reshape(T, H * dv)
    assert_close(to_np(y), want.numpy(), dtype, "turned back", bound=slack)


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 16, 8), (2, 2, 64, 64), (3, 1, 24, 40), (1, 1, 130, 6), (2, 1, 256, 128), (6, 3, 7, 5)])
def test_recurrences_in_steps_of_any_size(delta, H, G, dk, dv):
    """Two sequences in slots 2 and 0, the first fed in steps of 1, 2, 17 and 33 tokens (more than one staged chunk), the
    second at once: outputs and final states are the whole sequence's."""
    if not delta:
        G = H
    g = torch.Generator().manual_seed(dk * dv + H)
    lens = [53, 20]
    mk = lambda n, h, d, s=1.0: torch.randn(n, h, d, generator=g) * s       # noqa: E731
    seqs = []
    for n in lens:
        q, k, v = mk(n, G, dk), mk(n, G, dk), mk(n, H, dv)
        if delta:
            q, k = q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True)
        else:
            k = k / math.sqrt(dk)
        seqs.append((q, k, v, torch.rand(n, H, generator=g) * 0.7 + 0.3, torch.rand(n, H, generator=g)))
    decay = torch.tensor([0.9 + 0.1 * h / max(H - 1, 1) for h in range(H)])          # the last head never forgets
    state = torch.zeros(3, H, dk, dv, device=DEV)
    state[1] = 7.0                                                           # a slot no sequence of this test holds
    cuts, slots = [[1, 2, 17, 33], [20]], [2, 0]
    done, got = [0, 0], [[], []]
    for r in range(4):
        live = [b for b in range(2) if r < len(cuts[b])]
        n = [cuts[b][r] for b in live]
        cat = lambda i: torch.cat([seqs[b][i][done[b]:done[b] + k].reshape(k, -1) for b, k in zip(live, n)]).to(DEV)   # noqa: E731
        q, k, v = cat(0), cat(1), cat(2)
        gates = torch.cat([cat(3), cat(4)], dim=1).contiguous() if delta else None
        out = torch.zeros(sum(n), H * dv, device=DEV)
        ops.linear_scan(q, k, v, state, step_of(n, [slots[b] for b in live]), out, H, G, dk, dv, gates=gates,
                        decay=None if delta else decay.to(DEV))
        o = 0
        for b, kk in zip(live, n):
            got[b].append(out[o:o + kk].cpu()); o += kk; done[b] += kk
    for b in range(2):
        q, k, v, gd, beta = (t.double() for t in seqs[b])
        fin = []
        ref = P.delta_recurrence(q, k, v, gd, beta, fin) if delta else P.decay_recurrence(q, k, v, decay.double(), fin)
        scale = float(ref.abs().max())
        assert np.abs(torch.cat(got[b]).double().numpy() - ref.reshape(lens[b], -1).numpy()).max() < 2e-5 * max(scale, 1.0), b
        assert np.abs(to_np(state[slots[b]]) - torch.stack(fin).numpy()).max() < 2e-5 * max(float(torch.stack(fin).abs().max()), 1.0)
    assert float((state[1] - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("H,G,dk,dv", [(2, 1, 32, 16), (1, 1, 128, 128), (3, 3, 20, 9)])
@pytest.mark.parametrize("lens", [[16], [32], [8], [15, 17], [47, 1, 9]])
def test_delta_rule_over_many_tokens_with_gates_at_their_ends(lens, H, G, dk, dv):
    """Steps long enough for the kernel that takes sixteen tokens at a time (whole groups, one token short, one over,
    a single token beside long sequences), continued once from the state they left.  Some decays are exactly 0 (the
    state is wiped there and nothing else is) or 1, some step sizes exactly 0 (the token writes nothing) or 1."""
    g = torch.Generator().manual_seed(sum(lens) * dk + dv)
    total = [2 * n for n in lens]
    seqs = []
    for n in total:
        q, k, v = (torch.randn(n, G, dk, generator=g), torch.randn(n, G, dk, generator=g), torch.randn(n, H, dv, generator=g))
        q, k = q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True)
        gd, beta = torch.rand(n, H, generator=g) * 0.6 + 0.4, torch.rand(n, H, generator=g)
        for t in range(n):
            gd[t, t % H] = (0.0, 1.0, 1e-30)[t % 3] if t % 5 == 2 else gd[t, t % H]
            beta[t, (t + 1) % H] = (0.0, 1.0)[t % 2] if t % 7 == 3 else beta[t, (t + 1) % H]
        seqs.append((q, k, v, gd, beta))
    state = torch.zeros(len(lens) + 1, H, dk, dv, device=DEV)
    slots = list(range(len(lens), 0, -1))
    got = [[] for _ in lens]
    for r in range(2):
        cat = lambda i: torch.cat([seqs[b][i][r * n:(r + 1) * n].reshape(n, -1) for b, n in enumerate(lens)]).to(DEV)   # noqa: E731
        out = torch.zeros(sum(lens), H * dv, device=DEV)
        ops.linear_scan(cat(0), cat(1), cat(2), state, step_of(lens, slots), out, H, G, dk, dv,
                        gates=torch.cat([cat(3), cat(4)], dim=1).contiguous())
        o = 0
        for b, n in enumerate(lens):
            got[b].append(out[o:o + n].cpu()); o += n
    for b, n in enumerate(total):
        q, k, v, gd, beta = (t.double() for t in seqs[b])
        fin = []
        ref = P.delta_recurrence(q, k, v, gd, beta, fin)
        assert np.abs(torch.cat(got[b]).double().numpy() - ref.reshape(n, -1).numpy()).max() < 2e-5 * max(float(ref.abs().max()), 1.0), b
        assert np.abs(to_np(state[slots[b]]) - torch.stack(fin).numpy()).max() < 2e-5 * max(float(torch.stack(fin).abs().max()), 1.0)
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_unit_vectors_gates_output_norms_and_the_small_kernels(dtype):
    td = td_of(dtype)
    g = torch.Generator().manual_seed(8)
    T, H, G, dk, dv = 9, 4, 2, 24, 10
    qk = torch.randn(T, 3 + 2 * G * dk, generator=g) * 3
    qk[0, 3:3 + dk] = 0.0                                                    # a zero vector stays finite
    ab = torch.randn(T, 2 * H + 5, generator=g) * 4
    a_log, dt_bias = torch.randn(H, generator=g), torch.randn(H, generator=g)
    gates = torch.zeros(T, 2 * H, device=DEV)
    qk_d = qk.clone().to(DEV)
    ops.delta_prepare(qk_d, 3, 3 + G * dk, G, dk, dk ** -0.5, ab.to(DEV), 5, 5 + H, a_log.to(DEV), dt_bias.to(DEV), gates, H)
    q = qk[:, 3:3 + G * dk].double().view(T, G, dk)
    k = qk[:, 3 + G * dk:].double().view(T, G, dk)
    rq = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    rk = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    assert np.abs(to_np(qk_d[:, 3:3 + G * dk]) - rq.reshape(T, -1).numpy()).max() < 1e-6
    assert np.abs(to_np(qk_d[:, 3 + G * dk:]) - rk.reshape(T, -1).numpy()).max() < 1e-6
    beta = P.sigmoid(ab[:, 5:5 + H].double())
    gd = torch.exp(-torch.exp(a_log.double()) * P.softplus(ab[:, 5 + H:5 + 2 * H].double() + dt_bias.double()))
    assert np.abs(to_np(gates[:, :H]) - gd.numpy()).max() < 1e-6 and np.abs(to_np(gates[:, H:]) - beta.numpy()).max() < 1e-6
    # output norms: per head with a shared weight and a silu gate; over all heads with a sigmoid gate
    o, gate = torch.randn(T, H * dv + 3, generator=g) * 5, torch.randn(T, H * dv + 1, generator=g) * 2
    w1, wall = 1 + 0.2 * torch.randn(dv, generator=g), 1 + 0.2 * torch.randn(H * dv, generator=g)
    y = torch.empty(T, H * dv, dtype=td, device=DEV)
    ops.gated_rmsnorm(o.to(DEV)[:, :H * dv], w1.to(DEV), 1e-5, gate.to(DEV)[:, :H * dv], y, H, dv, sigmoid_gate=False)
    od, gd2 = o[:, :H * dv].double(), gate[:, :H * dv].double()
    ref = (P.rms_norm(od.view(T, H, dv), w1.double(), 1e-5)).reshape(T, -1) * P.silu(gd2)
    assert_close(to_np(y), ref.numpy(), dtype, "per head")
    ops.gated_rmsnorm(o.to(DEV)[:, :H * dv], wall.to(DEV), 1e-5, gate.to(DEV)[:, :H * dv], y, 1, H * dv, sigmoid_gate=True)
    assert_close(to_np(y), (P.rms_norm(od, wall.double(), 1e-5) * P.sigmoid(gd2)).numpy(), dtype, "all heads")
    # silu on a range of columns, a x + b y, the gated activation with biases, the cap
    x = torch.randn(T, 40, generator=g).to(DEV)
    x0 = x.clone()
    ops.silu_columns(x, 4, 30)
    assert np.abs(to_np(x[:, 4:34]) - P.silu(x0[:, 4:34].double().cpu()).numpy()).max() < 1e-6
    assert torch.equal(x[:, :4], x0[:, :4]) and torch.equal(x[:, 34:], x0[:, 34:])
    z, x1 = torch.randn(T, 40, generator=g).to(DEV), x.clone()
    ops.axpby(x, 1.2, z, -0.7)
    assert np.abs(to_np(x) - (1.2 * x1.double() - 0.7 * z.double()).cpu().numpy()).max() < 1e-5
    x2 = x1.clone()
    ops.add_row_bias(x2, z[0])
    assert np.abs(to_np(x2) - (x1.double() + z[0].double()).cpu().numpy()).max() < 1e-6
    for inter, il in ((24, 8), (21, 0)):
        gu, b = torch.randn(T, 2 * inter, generator=g) * 2, torch.randn(2 * inter, generator=g)
        out = torch.empty(T, inter, dtype=td, device=DEV)
        ops.bias_glu(gu.to(DEV), b.to(DEV), out, il, ops.ACT_RELU)
        s = (gu + b).double()
        if il:
            s = s.view(T, inter // il, 2, il)
            gt, up = s[:, :, 0].reshape(T, inter), s[:, :, 1].reshape(T, inter)
        else:
            gt, up = s[:, :inter], s[:, inter:]
        assert_close(to_np(out), (torch.relu(gt) * up).numpy(), dtype, f"relu glu {inter}")
    lg = (torch.randn(3, 50, generator=g) * 40).to(DEV)
    l0 = lg.clone()
    ops.tanh_cap(lg, 30.0)
    assert np.abs(to_np(lg) - (30.0 * torch.tanh(l0.double().cpu() / 30.0)).numpy()).max() < 1e-5 and float(lg.abs().max()) <= 30.0


# ---- whole models ---------------------------------------------------------------------------------
ALONE = {
    "lightning": [(U.lightning(heads=2, dim=16, vdim=8), None)],
    "lightning_ff_one_head": [(U.lightning(heads=1, dim=24, vdim=40, decay=[0.93]), U.dense(40))],
    "parallel": [(U.parallel(), None)],
    "parallel_no_window_no_factor": [(U.parallel(window=None, factor=None, heads=2, kv_heads=2, conv=1), U.dense(24))],
    "parallel_window_of_one": [(U.parallel(window=1, rot_dims=0, heads=2, kv_heads=1, vdim=8, rheads=1, rkv=1, conv=2), None)],
    "parallel_sharp_heads_of_64": [(U.parallel(heads=4, kv_heads=1, dim=64, vdim=64, window=33, sharp=3.0, rot_dims=32,
                                               rheads=2, rkv=2, rdim=64, rvdim=64), None)],
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
    """Three slots serve eight requests: the recurrent states, the convolutions' inputs, the previous token and the pages of
    a slot's former user must not reach its next one (a request of one token reads nothing but zeros and the last row)."""
    d, pm = mixed
    rng = np.random.default_rng(3)
    reqs = [ids_for(rng, VOCAB, n) for n in (1, 37, 80, 5, 64, 23, 2, 70)]
    refs = [pm.logits(r).numpy() for r in reqs]
    eng = engine_for(d, dtype, max_tokens=64 * 5, max_slots=3)
    got = replay_batches(eng, reqs, [1, 30, 64, 2, 40, 23, 1, 65], [[0, 1, 2], [3, 4], [5, 6, 7]])
    for i, (g, ref) in enumerate(zip(got, refs)):
        assert_close(g, ref, dtype, f"request {i}", plain=pm, ids=reqs[i])
    assert eng.cache.slots.free_count == 3


def _with_window(pm, size):
    cfg = copy.deepcopy(pm.cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["mask"] = {"size": size}
    return P.PlainBegupel(config=cfg, tensors=pm.w)


@pytest.mark.parametrize("window", [1, 12, 16, 17, 64, 65, 70])
def test_a_window_one_key_off_shows_in_prompts_and_in_decoding(tmp_path, window):
    """Sharp attention (a few keys carry each softmax), pages of 16 keys: the key that has just left the window and the
    one that is just inside it are told apart at every position past the window, in a prompt, in a prompt's second
    portion and token by token."""
    layers = [(U.parallel(heads=2, kv_heads=1, dim=16, vdim=16, window=window, sharp=4.0, left_scale=2.0, right_scale=0.3), None)]
    d, pm = U.make(tmp_path / "w", layers, seed=window)
    ids = ids_for(np.random.default_rng(window), VOCAB, 150)
    ref = pm.logits(ids).numpy()
    eng = engine_for(d, "float32", max_tokens=16 * 40, page_size=16)
    runs = {"whole": replay_whole(eng, ids), "decoded": replay_tail_one_by_one(eng, ids, 130)}
    s = eng.alloc_slot()
    runs["portions"] = np.concatenate([to_np(eng.step([(s, ids[:window + 3])], "all")), to_np(eng.step([(s, ids[window + 3:])], "all"))])
    eng.free_slot(s)
    wrong = [_with_window(pm, w).logits(ids).numpy() for w in (window + 1, max(window - 1, 1))][:2 if window > 1 else 1]
    for what, got in runs.items():
        assert np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), what
        for other in wrong:
            far_off = np.abs(got - other).max(axis=-1) > 1e-2
            assert not far_off[:max(window - 1, 1)].any() and far_off[window:].sum() > (len(ids) - window) // 10, what


@pytest.mark.parametrize("dtype", DTYPES)
def test_tokens_far_back_stay_in_the_states(tmp_path, dtype):
    """A head that never forgets and slow delta-rule decays: the first tokens of 400 still move the last logits, and
    the engine has them whether the prompt came at once, in portions, or mostly token by token."""
    layers = [(U.lightning(heads=2, dim=16, vdim=16, decay=[1.0, 0.999]), None),
              (U.parallel(window=8, rheads=2, rkv=1, rdim=32, rvdim=16, left_scale=0.2, right_scale=1.5), None)]
    d, pm = U.make(tmp_path / "far", layers, seed=21)
    pm.w["l1.mix.right.A_log"] = pm.w["l1.mix.right.A_log"] * 0 - 6.0           # decays near 1
    U.write(pm.cfg, {k: v.to(torch.bfloat16) for k, v in pm.w.items()}, d)
    pm = P.PlainBegupel(d)
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
        assert_close(np.concatenate(got), ref, dtype, f"prompt cut in {len(cuts)}", plain=pm, ids=ids, rows=rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(mixed, dtype):
    """Sequences of one, two and three tokens (shorter than every convolution) after a long one in the same slot."""
    d, pm = mixed
    eng = engine_for(d, dtype, max_tokens=512, max_slots=1)
    rng = np.random.default_rng(17)
    replay_whole(eng, ids_for(rng, VOCAB, 90))
    for n in (1, 2, 3, 5):
        ids = ids_for(rng, VOCAB, n)
        ref = pm.logits(ids).numpy()
        assert_close(replay_whole(eng, ids), ref, dtype, f"{n} at once", plain=pm, ids=ids)
        assert_close(replay_tail_one_by_one(eng, ids, n - 1), ref, dtype, f"{n} one by one", plain=pm, ids=ids)
    changed = pm.logits([5, 9]).numpy()[0] - pm.logits([6, 9]).numpy()[0]
    assert np.abs(changed).max() > 1e-2                                       # the first token's own rows matter


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_small_pages(tmp_path, dtype):
    layers = [(U.parallel(heads=2, kv_heads=1, dim=16, vdim=32, window=40, sharp=3.0), U.dense(32)),
              (U.lightning(heads=2, dim=32, vdim=16), None),
              (U.parallel(heads=2, kv_heads=2, dim=64, vdim=64, window=100, sharp=3.0, rheads=2, rkv=2, conv=2), None)]
    d, pm = U.make(tmp_path / "s", layers, seed=11)
    ids = ids_for(np.random.default_rng(11), VOCAB, 260)
    ref = pm.logits(ids).numpy()
    page = 16 if dtype == "float32" else 64       # the tensor-core kernels read pages in tiles of 64 keys
    eng = engine_for(d, dtype, max_tokens=page * 20, page_size=page)
    assert_close(replay_whole(eng, ids), ref, dtype, "whole", plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 210), ref, dtype, "decoded", plain=pm, ids=ids)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_and_its_continuation(tmp_path, dtype):
    """600 tokens at once (many staged chunks of the recurrences, ten pages of keys, several windows), then the same
    prompt in two portions, each followed by 24 tokens one by one."""
    layers = [(U.parallel(heads=4, kv_heads=2, dim=32, vdim=64, window=130, rot_dims=16, rheads=4, rkv=2, rdim=32, rvdim=32), U.dense(96)),
              (U.lightning(heads=4, dim=32, vdim=16, decay=[0.6, 0.9, 0.99, 0.9995]), None),
              (U.parallel(heads=2, kv_heads=1, dim=64, vdim=32, window=300, rheads=2, rkv=1, rdim=64, rvdim=64, conv=3), U.dense(72))]
    d, pm = U.make(tmp_path / "long", layers, seed=13, width=128, vocab=500, groups=4, taps=5)
    ids = ids_for(np.random.default_rng(13), 500, 624)
    rows = [0, 1, 63, 64, 129, 130, 299, 300, 511, 512, 598, 599] + list(range(600, 624))
    arith = torch.float32 if dtype == "bfloat16" else torch.float64
    ref = pm.logits(ids).numpy()[rows]
    eng = engine_for(d, dtype, max_tokens=2048)
    for cuts in ([600], [333, 267]):
        s, got, at = eng.alloc_slot(), [], 0
        for n in cuts + [1] * 24:
            want = [r - at for r in rows if at <= r < at + n]
            out = eng.step([(s, ids[at:at + n])], [want])
            if want:
                got.append(to_np(out))
            at += n
        eng.free_slot(s)
        assert_close(np.concatenate(got), ref, dtype, f"prompt in {len(cuts)}", plain=pm, ids=ids, rows=rows, arith=arith)
    eng.check_kernels()


OTHER = {
    "ones": ([(U.parallel(heads=1, kv_heads=1, dim=8, vdim=2, window=3, rot_dims=2, factor=1.0, rheads=1, rkv=1, rdim=8, rvdim=8, conv=1), U.dense(8)),
              (U.lightning(heads=1, dim=8, vdim=8, decay=[0.9]), U.dense(16))],
             dict(vocab=77, width=40, groups=1, taps=1, buckets=1, mul_prev=1, mul_cur=1, softcap=None, eps=1e-6)),
    "wide_heads": ([(U.parallel(heads=6, kv_heads=2, dim=96, vdim=128, window=90, rot_dims=64, base=500.0, factor=8.0,
                                rheads=6, rkv=3, rdim=128, rvdim=96, conv=2, left_scale=0.5, right_scale=2.0), U.dense(200)),
                    (U.lightning(heads=5, dim=96, vdim=48), U.dense(72)),
                    (U.lightning(heads=2, dim=160, vdim=128), None)],
                   dict(vocab=300, width=136, groups=8, taps=6, buckets=1021, mul_prev=999983, mul_cur=65537, softcap=7.5)),
    "odd_sizes": ([(U.lightning(heads=3, dim=10, vdim=6), None),
                   (U.parallel(heads=6, kv_heads=3, dim=10, vdim=6, window=5, rot_dims=6, rheads=3, rkv=3, rdim=7, rvdim=5, conv=7), U.dense(13)),
                   (U.parallel(heads=3, kv_heads=1, dim=20, vdim=26, window=64, rot_dims=20, rheads=5, rkv=1, rdim=12, rvdim=18, conv=3), None)],
                  dict(vocab=61, width=50, groups=5, taps=2, buckets=13, mul_prev=5, mul_cur=3, softcap=50.0)),
    "keys_wider_than_values": ([(U.parallel(heads=8, kv_heads=8, dim=128, vdim=32, window=32, rheads=2, rkv=2, rdim=128, rvdim=32), None),
                                (U.lightning(heads=2, dim=128, vdim=32), U.dense(128))],
                               dict(vocab=200, width=128, groups=2, taps=4)),
    # no layer keeps keys and values: the cache has states only
    "recurrences_only": ([(U.lightning(heads=4, dim=32, vdim=64, decay=[0.0, 0.5, 0.99, 1.0]), U.dense(96)),
                          (U.lightning(heads=2, dim=64, vdim=32), None),
                          (U.lightning(heads=8, dim=16, vdim=16), U.dense(64))],
                         dict(vocab=150, width=96, groups=3, taps=5, buckets=31, mul_prev=17, mul_cur=29)),
    # every layer keeps keys and values, each with its own window, head count and head sizes; a window of one key
    "attention_in_every_layer": ([(U.parallel(heads=4, kv_heads=1, dim=32, vdim=64, window=1, rot_dims=16, rheads=2, rkv=1, rdim=32, rvdim=64, conv=4), U.dense(80)),
                                  (U.parallel(heads=2, kv_heads=2, dim=64, vdim=32, window=17, rot_dims=64, factor=None, rheads=4, rkv=4, rdim=16, rvdim=16, conv=2), None),
                                  (U.parallel(heads=8, kv_heads=4, dim=16, vdim=16, window=None, rot_dims=0, rheads=8, rkv=2, rdim=64, rvdim=32, conv=5,
                                              left_scale=-1.0, right_scale=0.25), U.dense(40))],
                                 dict(vocab=90, width=80, groups=4, taps=3, buckets=7, mul_prev=-3, mul_cur=2)),
    # nearer a real model's sizes: the tensor-core products and attention kernels, state matrices of 128 x 128
    "larger": ([(U.lightning(heads=4, dim=128, vdim=128), U.dense(512)),
                (U.parallel(heads=4, kv_heads=2, dim=128, vdim=128, window=100, rot_dims=64, rheads=4, rkv=2, rdim=128, rvdim=128), U.dense(512)),
                (U.parallel(heads=8, kv_heads=8, dim=64, vdim=64, window=48, rheads=8, rkv=8, rdim=64, rvdim=64), None),
                (U.lightning(heads=8, dim=64, vdim=32), None)],
               dict(vocab=1000, width=512, groups=2, taps=4, buckets=4093, mul_prev=31, mul_cur=7, softcap=30.0)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(OTHER))
def test_other_sizes_and_orders(tmp_path, which, dtype):
    layers, kw = OTHER[which]
    d, pm = U.make(tmp_path / which, layers, seed=7, **kw)
    rng = np.random.default_rng(5)
    reqs = [ids_for(rng, kw["vocab"], n) for n in (130, 2, 66)]
    refs = [pm.logits(r).numpy() for r in reqs]
    eng = engine_for(d, dtype, max_tokens=64 * 8, max_slots=3)
    assert_close(replay_whole(eng, reqs[0]), refs[0], dtype, "whole", plain=pm, ids=reqs[0])
    assert_close(replay_tail_one_by_one(eng, reqs[0], 40), refs[0], dtype, "tail", plain=pm, ids=reqs[0])
    got = replay_batches(eng, reqs, [100, 1, 30], [[0, 1, 2]])
    for g, ref, r in zip(got, refs, reqs):
        assert_close(g, ref, dtype, "batched", plain=pm, ids=r)


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_steps_equal_eager_ones(mixed, dtype):
    d, pm = mixed
    rng = np.random.default_rng(8)
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
    cfg = U.config([(U.parallel(), U.dense(40)), (U.lightning(), None)])
    hb.write_random_model(cfg, str(tmp_path), seed=1)
    pm = P.PlainBegupel(str(tmp_path))
    assert set(pm.w) == set(U.weights(cfg)) and pm.w["bigram"].shape == (98, 64)
    ids = ids_for(np.random.default_rng(1), VOCAB, 50)
    eng = engine_for(str(tmp_path), "float32", max_tokens=256)
    assert_close(replay_whole(eng, ids), pm.logits(ids).numpy(), "float32", "random model")


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
