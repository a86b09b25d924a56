"""The kernels of the Vadelix parts one by one, each against the oracle's function of the same mechanism on the same
(bfloat16-rounded) inputs: a request's tokens cut into steps of several sizes (down to one and two tokens) against the
whole sequence, states carried in slots that are not the requests' indices, keys far away, at page borders and on both
sides of a window's edge with planted scores that stand out, sinks that take most of the weight."""

from __future__ import annotations

import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vadelix as pv

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CUTS = ([1] * 9, [2, 2, 2, 2, 1], [9], [3, 1, 5], [1, 8], [7, 2], [4, 5])


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(device=DEV, dtype=dtype).contiguous()


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def bf(a):
    """float64 numpy values that bfloat16 holds exactly."""
    return torch.as_tensor(np.asarray(a, dtype=np.float64)).to(torch.bfloat16).to(torch.float64).numpy()


def close(got, want, tol, what=""):
    got, want = np.asarray(got.detach().float().cpu() if torch.is_tensor(got) else got, dtype=np.float64), np.asarray(want)
    scale = max(float(np.abs(want).max()), 1e-30)
    err = float(np.abs(got - want).max()) / scale
    assert err < tol, f"{what}: largest difference {err:.3e} of the largest value"


def batches(lengths, cuts_of):
    """Steps over several requests: each step is [(request, first token, count)], requests advancing side by side."""
    at = [0] * len(lengths)
    turn = [0] * len(lengths)
    steps = []
    while any(a < n for a, n in zip(at, lengths)):
        step = []
        for r, n in enumerate(lengths):
            if at[r] < n:
                c = min(cuts_of[r][turn[r] % len(cuts_of[r])], n - at[r])
                step.append((r, at[r], c))
                at[r] += c
                turn[r] += 1
        steps.append(step)
    return steps


def step_arrays(step):
    cu = [0]
    seq_of = []
    for i, (_, _, c) in enumerate(step):
        cu.append(cu[-1] + c)
        seq_of += [i] * c
    return i32(cu), i32(seq_of)


def segments(q_lens, seg_len):
    from acvram_b200.kernels import ops
    if not seg_len:
        return None
    arrays, values = ops.segment_work(q_lens, seg_len)
    return {**{k: i32(v) for k, v in arrays.items()}, **values}


# --------------------------------------------------------------------------- grouped norm and the input convolution
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,groups,taps", [(32, 1, 1), (96, 3, 3), (100, 5, 5), (1024, 4, 4), (2048, 16, 2), (256, 64, 6)])
def test_grouped_norm_and_convolution_over_steps(H, groups, taps, dtype):
    """Three requests side by side, cut differently, their kept rows in slots 5, 0 and 2; steps in which every request
    brings one token take the fused launch.  The stream after the sums and the mixer's input must be the oracle's."""
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(H + taps)
    lengths = (9, 9, 9)
    slots_of = (5, 0, 2)
    x0 = [rng.standard_normal((n, H)) for n in lengths]
    delta = [bf(rng.standard_normal((n, H))) for n in lengths]
    w, tp = bf(1.0 + 0.2 * rng.standard_normal(H)), bf(0.5 * rng.standard_normal((H, taps)))
    eps, mult = 1e-5, 0.7
    state = torch.zeros((6, max(taps - 1, 1), H), device=DEV)
    got_h = [np.zeros((n, H)) for n in lengths]
    got_x = [np.zeros((n, H)) for n in lengths]
    for step in batches(lengths, (CUTS[0], CUTS[3], CUTS[6])):
        cu, seq_of = step_arrays(step)
        x = dev(np.concatenate([x0[r][a:a + c] for r, a, c in step]))
        d = dev(np.concatenate([delta[r][a:a + c] for r, a, c in step]), DT[dtype])
        slots = i32([slots_of[r] for r, _, _ in step])
        out = torch.empty(x.shape, device=DEV, dtype=DT[dtype])
        if all(c == 1 for _, _, c in step):
            ops.add_group_rmsnorm_conv(x, d, dev(w), eps, groups, dev(tp), state, slots, out, mult)
        else:
            normed = torch.empty(x.shape, device=DEV)
            ops.add_group_rmsnorm(x, d, dev(w), eps, groups, normed, None, mult)
            ops.input_conv(normed, dev(tp), state, slots, cu, seq_of, out, dev(tp.T.copy()) if H % 8 == 0 else None)
        o = 0
        for r, a, c in step:
            got_h[r][a:a + c] = out[o:o + c].float().cpu().numpy()
            got_x[r][a:a + c] = x[o:o + c].cpu().numpy()
            o += c
    for r, n in enumerate(lengths):
        xs = np.float32(x0[r]).astype(np.float64) + mult * delta[r]
        h = pv.grouped_norm(xs, w, eps, groups)
        close(got_x[r], xs, 1e-6, "the stream")
        close(got_h[r], h + pv.short_conv(h, tp), 2e-5 if dtype == "float32" else 1.2e-2, f"request {r}")


def test_grouped_norm_of_chosen_rows_leaves_the_stream():
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(1)
    x0 = rng.standard_normal((7, 48))
    d = bf(rng.standard_normal((7, 48)))
    x = dev(x0)
    out = torch.empty((2, 48), device=DEV, dtype=torch.bfloat16)
    ops.add_group_rmsnorm(x, dev(d, torch.bfloat16), dev(np.ones(48)), 1e-6, 4, out, i32([5, 1]), 0.5)
    assert torch.equal(x.cpu(), torch.as_tensor(np.float32(x0)))
    close(out, pv.grouped_norm((np.float32(x0) + 0.5 * d)[[5, 1]], np.ones(48), 1e-6, 4), 1e-2)


# --------------------------------------------------------------------------- projections to pages, attention with sinks and slopes
class Paged:
    """One request's keys and values in pages handed out in a shuffled order, on a row of the block table that is not
    the request's index."""

    def __init__(self, n, NKV, D, DV, page, dtype, seed):
        pages = -(-n // page) + 2
        order = list(range(pages))
        random.Random(seed).shuffle(order)
        self.table = torch.full((3, pages), -1, dtype=torch.int32)
        self.table[2, :-(-n // page)] = torch.tensor(order[:-(-n // page)], dtype=torch.int32)
        self.table = self.table.to(DEV)
        self.k = torch.zeros((pages, NKV, page, D), device=DEV, dtype=dtype)
        self.v = torch.zeros((pages, NKV, page, DV), device=DEV, dtype=dtype)
        self.rows = i32([2])


def run_attention(x, cuts, NH, NKV, D, DV, page, dtype, seed, prepare, attend):
    """The stacked projection ``x`` of one request through ``ops.qkv_prepare`` and ``ops.attention``, cut into steps."""
    from acvram_b200.kernels import ops
    n = x.shape[0]
    pc = Paged(n, NKV, D, DV, page, DT[dtype], seed)
    got = np.zeros((n, NH * DV))
    kept = {}
    at = 0
    for c in cuts:
        rows = dev(x[at:at + c], DT[dtype])
        pos, seq_of = i32(range(at, at + c)), i32([0] * c)
        shared = prepare.get("shared_values")
        step_prepare = dict(prepare)
        if shared is not None:
            step_prepare["shared_values"] = dev(shared[at:at + c]) if prepare["share"] == "mix" else torch.empty((c, NKV * DV), device=DEV)
        ops.qkv_prepare(rows, NH, NKV, D, DV, positions=pos, seq_of_token=seq_of, block_table=pc.table, k_pages=pc.k, v_pages=pc.v,
                        table_rows=pc.rows, **step_prepare)
        if prepare.get("share") == "source":
            kept[at] = step_prepare["shared_values"].cpu().numpy()
        out = torch.empty((c, NH * DV), device=DEV, dtype=DT[dtype])
        ctx = SimpleNamespace(positions=pos, seq_of_token=seq_of, table_rows=pc.rows, cu_q=i32([0, c]), kv_len=i32([at + c]), work={})
        work = ops.attention_work([c], [at + c], [0, c])
        work = {**{k_: dev(v_, torch.int32) for k_, v_ in work[0].items()}, **work[1]}
        ops.attention(rows, out, pc.k, pc.v, ctx, pc.table, NH, NKV, D, work=work, value_dim=DV, **attend)
        got[at:at + c] = out.float().cpu().numpy()
        at += c
    return got, kept


SHAPES = [(4, 2, 16, 24, 8, 20, 16, 200), (2, 2, 32, 32, 32, 24, 16, 200), (3, 3, 24, 40, 10, 7, 8, 200),
          (6, 2, 64, 80, 48, 120, 16, 200), (2, 1, 64, 64, 64, 48, 16, 200), (4, 2, 128, 128, 64, 100, 64, 700),
          (8, 1, 64, 64, 32, 130, 32, 450), (2, 1, 128, 128, 64, 900, 64, 1300)]    # (the last: several splits in the decode kernel)


def cuts_for(n):
    return ([n], [n - 1, 1], [37, 2, n - 50, 1, 1, 9], [n - 140, 130, 1] + [1] * 9) if n <= 1000 else ([n - 3, 1, 1, 1],)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("NH,NKV,D,DV,rot,window,page,n", SHAPES)
def test_rotated_attention_with_a_sink_and_planted_keys(NH, NKV, D, DV, rot, window, page, n, dtype):
    """Norm over the whole of q and of k, partial rotation, value heads of unit RMS, every key seen, a learned sink.  A
    key planted far back (at the first position, at a page's last and first row) wins the softmax of the last query
    unless the sink does: two sink levels, one far below the scores and one beside the planted score."""
    rng = np.random.default_rng(NH * 100 + D)
    rs = {"base": 3000.0, "dims": rot, "scaling": {"factor": 2.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mag = pv.rotary_frequencies(rs)
    ang = np.arange(n + 8)[:, None] * f[None, :]
    table = dev(np.concatenate([np.cos(ang), np.sin(ang)], axis=1) * mag)
    scale, eps = 0.4, 1e-5
    wq, wk = bf(1.0 + 0.2 * rng.standard_normal(NH * D)), bf(1.0 + 0.2 * rng.standard_normal(NKV * D))
    places = [0, page - 1, page, n - page - 3] if n <= 200 else [page - 1]
    for place, sink_level in [(pl, s) for pl in places for s in (-20.0, 4.0)][:(8 if n <= 200 else 2)]:
        x = bf(rng.standard_normal((n, NH * D + NKV * D + NKV * DV)))
        q = x[:, :NH * D].reshape(n, NH, D)
        k = x[:, NH * D:NH * D + NKV * D].reshape(n, NKV, D)
        if rot < D:     # along the last query of head 0 on the elements that do not turn
            k[place, 0, rot:] = bf(4.0 * q[n - 1, 0, rot:])
        else:
            k[place, 0] = bf(5.0 * k[place, 0])
        sinks = bf(sink_level + rng.standard_normal(NH))
        qn = (pv.unit_rms(x[:, :NH * D], eps) * wq).reshape(n, NH, D)
        kn = (pv.unit_rms(x[:, NH * D:NH * D + NKV * D], eps) * wk).reshape(n, NKV, D)
        qr, kr = pv.rotate(qn, rs, np.arange(n)), pv.rotate(kn, rs, np.arange(n))
        v = pv.unit_rms(x[:, NH * D + NKV * D:].reshape(n, NKV, DV), eps)
        want = np.zeros((n, NH, DV))
        for a in range(NH):
            g = a // (NH // NKV)
            s = (qr[:, a] @ kr[:, g].T) * scale
            for i in range(n):
                want[i, a] = pv.sink_softmax_sum(s[i], list(range(i + 1)), sinks[a], v[:, g])
        want = want.reshape(n, NH * DV)
        prepare = {"q_weight": dev(wq), "k_weight": dev(wk), "eps": eps, "cos_sin": table, "value_norm_eps": eps}
        attend = {"scale": scale, "window": 0, "sinks": dev(sinks)}
        for cuts in cuts_for(n):
            got, _ = run_attention(x, cuts, NH, NKV, D, DV, page, dtype, place, prepare, attend)
            close(got, want, 3e-5 if dtype == "float32" else 4e-2, f"planted at {place}, sinks near {sink_level}, cuts {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("NH,NKV,D,DV,rot,window,page,n", SHAPES)
def test_windowed_attention_with_slopes_and_planted_keys(NH, NKV, D, DV, rot, window, page, n, dtype):
    """No rotation, a query temperature, a distance bias with a slope per head, a sliding window, a sink of score 0, and
    values blended with a given tensor.  The planted key stands just outside and just inside the last query's window, at
    a page's border and right behind the query; whether it is seen shows."""
    rng = np.random.default_rng(NH * 100 + D + 1)
    scale, lam, temp = 0.3, 0.35, (0.4, 16)
    slopes = np.array([2.0 ** (-8.0 * (a + 1) / NH) for a in range(NH)])
    places = sorted({n - window - 1, n - window, n - window + 1, n - 2, (n - window) // page * page,
                     min(n - 2, (n - window) // page * page + page)})
    if n > 200:
        places = [n - window - 1, n - window]
    if n > 1000:
        places = [n - window]
    for place in places:
        x = bf(rng.standard_normal((n, NH * D + NKV * D + NKV * DV)))
        q = x[:, :NH * D].reshape(n, NH, D)
        k = x[:, NH * D:NH * D + NKV * D].reshape(n, NKV, D)
        k[place, 0] = bf(3.0 * q[n - 1, 0])          # along the last query of head 0: far above every other score
        first = bf(rng.standard_normal((n, NKV * DV)))
        pos = np.arange(n)
        t = 1.0 + temp[0] * np.log(np.floor((pos + 1) / temp[1]) + 1.0)
        qt = bf(q * t[:, None, None]) if dtype == "bfloat16" else q * t[:, None, None]     # (queries are rounded as they are written back)
        v = ((1.0 - lam) * x[:, NH * D + NKV * D:] + lam * first).reshape(n, NKV, DV)
        want = np.zeros((n, NH, DV))
        for a in range(NH):
            g = a // (NH // NKV)
            s = (qt[:, a] @ k[:, g].T) * scale - slopes[a] * (pos[:, None] - pos[None, :])
            for i in range(n):
                want[i, a] = pv.sink_softmax_sum(s[i], list(range(max(0, i - window + 1), i + 1)), 0.0, v[:, g])
        want = want.reshape(n, NH * DV)
        prepare = {"q_weight": None, "k_weight": None, "eps": 0.0, "cos_sin": None, "temp": temp, "shared_values": first,
                   "share": "mix", "share_weight": lam}
        attend = {"scale": scale, "window": window, "sinks": dev(np.zeros(NH)), "slopes": dev(slopes)}
        for cuts in cuts_for(n):
            got, _ = run_attention(x, cuts, NH, NKV, D, DV, page, dtype, place, prepare, attend)
            close(got, want, 3e-5 if dtype == "float32" else 4e-2, f"planted at {place}, cuts {cuts}")


def test_the_source_layer_leaves_its_values():
    rng = np.random.default_rng(5)
    n, NH, NKV, D, DV = 40, 2, 2, 16, 24
    x = bf(rng.standard_normal((n, NH * D + NKV * D + NKV * DV)))
    prepare = {"q_weight": None, "k_weight": None, "eps": 0.0, "cos_sin": None, "value_norm_eps": 1e-5,
               "shared_values": np.zeros((n, NKV * DV)), "share": "source"}
    _, kept = run_attention(x, [25, 15], NH, NKV, D, DV, 16, "bfloat16", 0, prepare, {"scale": 0.25, "window": 0})
    want = pv.unit_rms(x[:, NH * D + NKV * D:].reshape(n, NKV, DV), 1e-5).reshape(n, -1)
    close(np.concatenate([kept[0], kept[25]]), want, 2e-6, "the values a later layer blends with")


# --------------------------------------------------------------------------- time mixing
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,rank,seg", [(3, 16, 8, 0), (1, 32, 4, 4), (5, 12, 6, 3), (2, 64, 16, 4), (2, 128, 32, 0), (4, 48, 8, 5),
                                          (2, 10, 3, 2), (1, 256, 8, 4)])
def test_time_mixing_over_steps(H, D, rank, seg, dtype):
    """Token shift with five mixes, the decays and the recurrence for three requests side by side, cut differently
    (portions longer than a segment run the three launches), their states in slots 4, 1 and 3 (zero at first, as the
    manager leaves a slot at admission)."""
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(H * 10 + D)
    C = 40
    lengths = (9, 9, 9)
    slots_of = (4, 1, 3)
    hs = [bf(rng.standard_normal((n, C))) for n in lengths]
    W = {"x.mu." + s: bf(rng.random(C)) for s in "rkvgw"}
    for nme in "rkvg":
        W["x." + nme] = bf(rng.standard_normal((H * D, C)) / math.sqrt(C))
    W["x.w1"], W["x.w2"] = bf(rng.standard_normal((rank, C)) / math.sqrt(C)), bf(rng.standard_normal((H * D, rank)) / math.sqrt(rank))
    W["x.w0"], W["x.u"] = bf(-1.0 + rng.standard_normal(H * D)), bf(0.5 * rng.standard_normal((H, D)))
    W["x.norm"], W["x.o"] = bf(1.0 + 0.2 * rng.standard_normal(H * D)), np.eye(H * D)
    mu = dev(np.stack([W["x.mu." + s] for s in "rkvgw"]))
    prev = torch.zeros((5, C), device=DEV)
    state = torch.zeros((5, H, D, D), device=DEV)
    t = DT[dtype]
    got = [np.zeros((n, H * D)) for n in lengths]
    for step in batches(lengths, (CUTS[1], CUTS[2], CUTS[5])):
        cu, seq_of = step_arrays(step)
        h = dev(np.concatenate([hs[r][a:a + c] for r, a, c in step]), t)
        T = h.shape[0]
        x = torch.empty((5, T, C), device=DEV, dtype=t)
        ops.token_shift_multi(h, mu, prev, i32([slots_of[r] for r, _, _ in step]), cu, seq_of, x)
        # the products in float64 on the kernel's own (rounded) mixes: what is judged is the kernels around them
        xs = x.double().cpu().numpy()
        r_, k_, v_, g_ = (xs[i] @ W["x." + nme].T for i, nme in enumerate("rkvg"))
        a = dev(xs[4] @ W["x.w1"].T)
        decay = torch.empty((T, H * D), device=DEV)
        ops.wkv_decay(a, dev(W["x.w2"].T.copy()), dev(W["x.w0"]), decay)
        o = torch.empty((T, H * D), device=DEV)
        ops.wkv(dev(r_), dev(k_), dev(v_), decay, dev(W["x.u"].reshape(-1)), state, i32([slots_of[r] for r, _, _ in step]), cu,
                len(step), o, H, D, D, work=segments([c for _, _, c in step], seg))
        out = torch.empty((T, H * D), device=DEV, dtype=t)
        ops.retention_gate(o, dev(g_, t), out, H, D, 1e-5, weight=dev(W["x.norm"]))
        at = 0
        for r, a0, c in step:
            got[r][a0:a0 + c] = out[at:at + c].float().cpu().numpy()
            at += c
    for r, n in enumerate(lengths):
        want = pv.wkv(hs[r], W, "x.", {"heads": H, "dim": D}, 1e-5)
        close(got[r], want, 1e-4 if dtype == "float32" else 3e-2, f"request {r}")


def test_a_long_portion_in_segments_equals_token_by_token():
    """300 tokens of one request as one portion (segments of 64: the three launches with a fold over four summaries) and
    one by one; decays close to 1, so that what the first segment leaves still weighs at the end."""
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(3)
    n, H, D = 300, 2, 16
    r_, k_, v_ = (dev(rng.standard_normal((n, H * D))) for _ in range(3))
    decay = dev(0.97 + 0.03 * rng.random((n, H * D)))
    u = dev(rng.standard_normal(H * D))
    outs = []
    for cuts in ([n], [1] * n, [130, 1, 169]):
        state = torch.zeros((2, H, D, D), device=DEV)
        o = torch.empty((n, H * D), device=DEV)
        at = 0
        for c in cuts:
            work = segments([c], 64)
            ops.wkv(r_[at:at + c], k_[at:at + c], v_[at:at + c], decay[at:at + c].contiguous(), u, state, i32([1]), i32([0, c]), 1,
                    o[at:at + c], H, D, D, work=work)
            at += c
        outs.append((o.cpu().numpy(), state[1].cpu().numpy()))
    for o, s in outs[1:]:
        close(o, outs[0][0], 2e-5, "outputs")
        close(s, outs[0][1], 2e-5, "the state left behind")


# --------------------------------------------------------------------------- experts without gates, chosen by groups
@pytest.mark.parametrize("E,top,count,keep", [(6, 2, 3, 2), (4, 1, 1, 1), (5, 2, 5, 2), (8, 3, 4, 2), (64, 6, 8, 3), (32, 4, 32, 4),
                                              (128, 5, 64, 7), (96, 3, 48, 47)])
def test_routing_by_groups(E, top, count, keep):
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(E + top)
    T, H = 50, 24
    h = dev(rng.standard_normal((T, H)))
    z = 2.0 * rng.standard_normal((T, E))
    z[0, :] = 0.0                                                   # all equal: the lowest indices of the lowest groups
    ids = torch.empty((T, top), device=DEV, dtype=torch.int32)
    weights = torch.empty((T, top), device=DEV)
    ops.moe_route(h, None, None, top, True, True, ids.view(-1), weights.view(-1), None, logits=dev(z), experts=E,
                  groups=(count, keep), renorm_eps=1e-20)
    chosen, w = pv.route(np.float32(z).astype(np.float64), top, count, keep)
    assert ids.cpu().numpy().tolist() == chosen.tolist()
    close(weights, w, 1e-5, "weights")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,F,E,top", [(1, 64, 48, 4, 1), (9, 96, 40, 6, 2), (70, 100, 36, 5, 2), (300, 128, 64, 8, 3),
                                         (700, 128, 64, 8, 3), (1500, 256, 192, 4, 1)])      # (the last two: grouped tcgen05 products)
def test_plain_experts(T, H, F, E, top, dtype):
    """The part as a whole against the oracle's mixture (softmax scores, groups, weights on the outputs, a shared expert
    without a gate), on weights and inputs that bfloat16 holds."""
    from acvram_b200.parts.base import Runtime
    from acvram_b200.parts.feed_forward import RoutedExperts
    rng = np.random.default_rng(T + H)
    count = 2 if E % 2 == 0 else E
    keep = max(-(-top // (E // count)), count - 1) if count > 1 else 1
    W = {"m.router": bf(3.0 * rng.standard_normal((E, H)) / math.sqrt(H)), "m.shared.up": bf(rng.standard_normal((56, H)) / math.sqrt(H)),
         "m.shared.down": bf(rng.standard_normal((H, 56)) / math.sqrt(56))}
    for e in range(E):
        W[f"m.e{e}.up"] = bf(rng.standard_normal((F, H)) / math.sqrt(H))
        W[f"m.e{e}.down"] = bf(rng.standard_normal((H, F)) / math.sqrt(F))
    part = RoutedExperts(H, E, top, F, 0.0, shared_ff=56, scoring="softmax", renormalize=True, weight_on="output", prefix="m.",
                         expert_form="plain", activation="gelu", groups=(count, keep), renorm_eps=1e-20, shared_gate=False)
    part.load({n: torch.as_tensor(v) for n, v in W.items()}, Runtime(torch.device(DEV), DT[dtype]))
    h = bf(rng.standard_normal((T, H)))
    got = part.forward(dev(h, DT[dtype]), None)
    spec = {"router": {"experts": E, "top": top, "groups": {"count": count, "keep": keep}}, "shared": {"ff": 56}}
    want = pv.moe_ff(h, W, "m.", spec)
    if dtype == "float32":
        close(got, want, 3e-5, "mixture")
    else:       # a close call of the router moves a whole row: judge the typical row
        err = np.abs(got.float().cpu().numpy() - want).max(-1) / np.abs(want).max()
        assert float(np.median(err)) < 2e-2 and float((err > 6e-2).mean()) <= 0.05, f"median {np.median(err)}, worst {err.max()}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,F", [(1, 64, 80), (33, 96, 200), (300, 128, 384)])
def test_gated_unit_with_a_gelu_gate(T, H, F, dtype):
    from acvram_b200.parts.base import Runtime
    from acvram_b200.parts.feed_forward import SwiGLU
    rng = np.random.default_rng(T + F)
    W = {"m.gate": bf(1.5 * rng.standard_normal((F, H)) / math.sqrt(H)), "m.up": bf(rng.standard_normal((F, H)) / math.sqrt(H)),
         "m.down": bf(rng.standard_normal((H, F)) / math.sqrt(F))}
    part = SwiGLU(H, F, prefix="m.", bias=False, names={"gate": "gate", "up": "up", "down": "down"}, activation="gelu_tanh")
    part.load({n: torch.as_tensor(v) for n, v in W.items()}, Runtime(torch.device(DEV), DT[dtype]))
    h = bf(rng.standard_normal((T, H)))
    close(part.forward(dev(h, DT[dtype]), None), pv.dense_ff(h, W, "m."), 3e-5 if dtype == "float32" else 3e-2, "gated unit")
