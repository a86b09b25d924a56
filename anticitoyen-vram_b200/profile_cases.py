"""The hot kernels one by one: ``acvram bench --what kernels`` (the reference's name for its per-kernel
measurements, acvram/cli.py:1476), and the small cases that are profiled under ncu.

    acvram bench --what kernels [--case NAME] [--json]
    python -m acvram_b200.profile_cases gemm_decode|gemm_prefill|attention_decode|attention_prefill [--reps N]

Each case runs a few launches of one kernel at the layer sizes of Qwen3-8B on inputs larger than
the L2 cache (weights and pages rotate), holding a few GB at most, and ends by itself in seconds;
it reports the mean CUDA-event time of a launch with the bytes or operations per second that this
makes.  The summaries under profiles/ name the command.
"""

from __future__ import annotations

import argparse

import torch

from .kernels.ops import QUERY_TILE
from .kernels import ops


def _time(fn, reps: int) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(reps):
        fn(3 + i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps * 1e3


def gemm_case(M: int, N: int, K: int, reps: int, plan: tuple | None = None) -> dict:
    copies = max(2, int(400e6 // (N * K * 2)) + 1)
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: ops.gemm_tc(x, ws[i % copies], out, plan), reps)
    plan = plan or ops.gemm_tc_plan(M, N, K)
    print(f"gemm_tc M={M} N={N} K={K} plan(swap, bn, splits)={plan}: {us:.1f} us, "
          f"{N * K * 2 / us / 1e3:.0f} GB/s of weights, {2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    return {"kernel": "gemm_tc", "M": M, "N": N, "K": K, "us": us, "weights_gbs": N * K * 2 / us / 1e3,
            "tflops": 2 * M * N * K / us / 1e6}


def attention_case(batch: int, q_len: int, context: int, reps: int, legacy: bool = False, page: int = 64) -> dict:
    NH, NKV, D = 32, 8, 128
    pages_per = (context + page - 1) // page
    n_pages = batch * pages_per
    # rotate over so many pools that a launch finds nothing of its pages in L2 (126 MB): 600 MB in all, three at least
    sets = max(3, -(-600_000_000 // (2 * n_pages * NKV * page * D * 2)))
    pools = [(torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16),
              torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16)) for _ in range(sets)]
    table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(batch, pages_per)
    T = batch * q_len
    qkv = torch.randn(T, (NH + 2 * NKV) * D, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, NH * D, device="cuda", dtype=torch.bfloat16)
    kv_len = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    cu_q = (torch.arange(batch + 1, dtype=torch.int32, device="cuda") * q_len)
    if q_len == 1:
        rows = torch.arange(batch, dtype=torch.int32, device="cuda")
        splits, in_clusters = ops.decode_plan(batch, NH, NKV, D, page, context)
        fn = lambda i: ops.attention_decode(qkv, out, *pools[i % sets], rows, rows, batch, kv_len, table, NH, NKV, D,
                                            D ** -0.5, 0, splits, context, cluster_merge=in_clusters)
        us = _time(fn, reps)
        gb = batch * context * NKV * D * 2 * 2 / 1e9
        print(f"attention_decode batch={batch} context={context} page={page} splits={splits}{' in clusters' if in_clusters else ''}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s of pages")
        return {"kernel": "attention_decode", "batch": batch, "context": context, "us": us, "pages_gbs": gb / us * 1e6}
    else:
        tiles = [(b, s) for b in range(batch) for s in range(0, q_len, QUERY_TILE)][::-1]
        tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
        tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
        kernel = ops.attention_chunk if legacy else ops.attention_tc
        fn = lambda i: kernel(qkv, out, *pools[i % sets], tile_seq, tile_q0, len(tiles), cu_q, kv_len, table, NH, NKV,
                              D, D ** -0.5, 0)
        us = _time(fn, reps)
        flops = batch * 4.0 * NH * D * (q_len * (context - q_len) + q_len * (q_len + 1) / 2)
        print(f"{kernel.__name__} batch={batch} q_len={q_len} context={context} page={page}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")
        return {"kernel": kernel.__name__, "batch": batch, "q_len": q_len, "context": context, "us": us, "tflops": flops / us / 1e6}


def decode_split_case(reps: int) -> dict:
    """The split-KV kernel with every way of cutting the context that ``ops.decode_plan`` chooses from, for a few
    batches and context lengths (Qwen3-8B head sizes, pages of 64, rotating pools larger than L2): microseconds a
    launch, with the time the plan reckons and the way it takes."""
    NH, NKV, D, page = 32, 8, 128, 64
    out = {}
    for batch, context in ((1, 8192), (2, 8192), (4, 8192), (4, 16384), (8, 2048), (8, 8192), (12, 8192), (32, 8192), (1, 65536)):
        pages_per = context // page
        n_pages = batch * pages_per
        sets = max(3, -(-600_000_000 // (2 * n_pages * NKV * page * D * 2)))       # 600 MB in all: nothing is found in L2
        pools = [(torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16),
                  torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16)) for _ in range(sets)]
        table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(batch, pages_per)
        qkv = torch.randn(batch, (NH + 2 * NKV) * D, device="cuda", dtype=torch.bfloat16)
        o = torch.empty(batch, NH * D, device="cuda", dtype=torch.bfloat16)
        kv_len = torch.full((batch,), context, dtype=torch.int32, device="cuda")
        rows = torch.arange(batch, dtype=torch.int32, device="cuda")
        chosen = ops.decode_plan(batch, NH, NKV, D, page, context)
        cells = []
        for reckoned, n_splits, cluster, _ in ops.decode_ways(batch, NH, NKV, D, page, context):
            fn = lambda i: ops.attention_decode(qkv, o, *pools[i % sets], rows, rows, batch, kv_len, table, NH, NKV, D,
                                                D ** -0.5, 0, n_splits, context, cluster_merge=cluster)
            us = min(_time(fn, max(reps, sets)), _time(fn, max(reps, sets)))
            name = f"{n_splits}{'c' if cluster else 's' if n_splits > 1 else ''}"
            out[f"b{batch} c{context} {name}"] = us
            cells.append(f"{name}{'*' if (n_splits, cluster) == chosen else ''} {us:.0f}/{reckoned:.0f}")
        print(f"batch {batch:2d} context {context:6d}: " + "  ".join(cells))
        del pools
        torch.cuda.empty_cache()
    print("   (splits, c = merged inside a cluster, s = through scratch memory, * = the plan's choice: measured / reckoned us)")
    return out


def tile_width_case(reps: int) -> dict:
    """The tokens-on-rows product at every tile width, for the shapes of a 2048-token prefill (8B sizes) and of a
    1024-token portion beside 32 decoding requests (14B sizes): what ``ops.GEMM_TILE_OVERHEAD`` was read from."""
    out = {}
    for M, N, K in ((2048, 4096, 4096), (2048, 4096, 12288), (2048, 24576, 4096), (1056, 5120, 5120), (1056, 5120, 17408),
                    (1056, 34816, 5120)):
        for bn in ops.GEMM_TILE_WIDTHS:
            out[f"{M}x{N}x{K} bn={bn}"] = gemm_case(M, N, K, reps, plan=(0, bn, 1, 8))["us"]
        print(f"   chosen for {M}x{N}x{K}: {ops.gemm_tc_plan(M, N, K)[1]} columns")
    return out


def pair_case(reps: int) -> dict:
    """The tokens-on-rows product with a CTA to a tile of 128 x 256 and with a pair of CTAs to a tile of 256 x 256
    (tcgen05 ``cta_group::2``), launch by launch in turn so that both see the same clocks: the shapes of a prompt of
    2048 and of 8192 tokens (8B sizes) and of a 1024-token portion beside 32 decoding requests (14B sizes)."""
    out = {}
    single, pair = (0, 256, 1, 8), (0, 256, 1, 6, ops.GEMM_PAIR)
    for M, N, K, swiglu in ((2048, 6144, 4096, False), (2048, 4096, 4096, False), (2048, 24576, 4096, True), (2048, 4096, 12288, False),
                            (8192, 6144, 4096, False), (8192, 24576, 4096, True), (8192, 4096, 12288, False),
                            (1056, 5120, 5120, False), (1056, 34816, 5120, True), (512, 4096, 12288, False)):
        copies = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        res = torch.empty(M, N // 2 if swiglu else N, device="cuda", dtype=torch.bfloat16)
        times = {single: [], pair: []}
        n = 0
        for it in range(3 + 2 * reps):
            for plan in (single, pair):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ops.gemm_tc(x, ws[n % copies], res, plan, swiglu_pairs=swiglu, static_weights=True)
                b.record()
                n += 1
                if it >= 3:
                    times[plan].append((a, b))
        torch.cuda.synchronize()
        med = {plan: sorted(a.elapsed_time(b) for a, b in ev)[len(ev) // 2] * 1e3 for plan, ev in times.items()}
        chosen = ops.gemm_tc_plan(M, N, K)
        print(f"gemm_tc M={M} N={N} K={K}{' SiLU(gate)*up' if swiglu else ''}: a CTA to a tile {med[single]:.1f} us "
              f"({2 * M * N * K / med[single] / 1e6:.0f} TFLOP/s), a pair {med[pair]:.1f} us ({2 * M * N * K / med[pair] / 1e6:.0f} TFLOP/s); "
              f"the plan takes {'the pair' if len(chosen) > 4 and chosen[4] == ops.GEMM_PAIR else f'tiles of {chosen[1]} columns'}")
        out[f"{M}x{N}x{K}"] = {"single_us": med[single], "pair_us": med[pair]}
    return out


def sample_case(rows: int, vocab: int, reps: int) -> dict:
    """Temperature 0.7 and top-p 0.9 over rows of a real vocabulary (a cluster of CTAs shares a row)."""
    logits = [torch.randn(rows, vocab, device="cuda") * 3.0 for _ in range(4)]
    f = lambda v: torch.full((rows,), v, device="cuda", dtype=torch.float32)
    temp, top_p, min_p = f(0.7), f(0.9), f(0.0)
    top_k = torch.zeros(rows, device="cuda", dtype=torch.int32)
    seed = torch.arange(rows, device="cuda", dtype=torch.int64)
    out = torch.empty(rows, device="cuda", dtype=torch.int32)
    counter = torch.zeros(rows, device="cuda", dtype=torch.int64)
    us = _time(lambda i: ops.sample(logits[i % 4], temp, top_k, top_p, min_p, seed, counter, out), reps)
    print(f"sample rows={rows} vocab={vocab} temperature 0.7 top-p 0.9: {us:.1f} us")
    return {"kernel": "sample", "rows": rows, "vocab": vocab, "us": us}


def decode_layer_case(batch: int, context: int, reps: int, fused: bool) -> dict:
    """One layer of the Qwen3-8B sizes in a decode step of ``batch`` requests: the persistent kernel, or the seven
    separate launches, on the same inputs (weights rotate over three layers so that none is found in L2)."""
    from .config import Qwen3Config
    from .engine.batch import StepEntry
    from .engine.runner import ModelRunner
    from .models import build_random
    cfg = Qwen3Config(vocab_size=2048, hidden_size=4096, intermediate_size=12288, num_hidden_layers=3, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=16384, tie_word_embeddings=False)
    model = build_random(cfg, 0, torch.bfloat16, "cuda:0")
    for b in model.blocks:
        b.fuse_decode = fused
    page = 16
    runner = ModelRunner(model, page, batch * (context + 256) // page + 8, batch, max_len=context + 256)
    runner.enable_graphs()          # as serving runs decode steps: replayed from a captured graph
    names = [f"r{i}" for i in range(batch)]
    ids = [(7 * i + 3) % 2000 + 5 for i in range(context)]
    for n in names:
        for pos in range(0, context, 2048):
            runner.step([StepEntry(n, ids[pos:pos + 2048], ())])
    entries = [StepEntry(n, [11], (0,)) for n in names]
    us = _time(lambda i: runner.step(entries), reps) / 3.0
    runner.check_status()
    if fused:       # when each CTA finished each phase of the last layer that ran (device-wide nanosecond timer)
        ops.DECODE_LAYER_TRACE = torch.zeros(ops.sm_count(), 8, dtype=torch.int64, device="cuda")
        runner.graphs = None        # a captured graph holds the arguments it was captured with: this one step runs eagerly
        runner.step(entries)
        torch.cuda.synchronize()
        t = ops.DECODE_LAYER_TRACE.cpu().numpy()
        ops.DECODE_LAYER_TRACE = None
        rel = (t - t[:, 0].min()) / 1e3
        names_ph = ["begin", "norm", "q/k/v", "attention", "output", "norm", "gate/up", "down"]
        print("phase ends, us after the first CTA began (earliest..latest CTA): " +
              "  ".join(f"{n} {rel[:, i].min():.1f}..{rel[:, i].max():.1f}" for i, n in enumerate(names_ph)))
    print(f"decode layer ({'one persistent kernel' if fused else 'separate launches'}) batch={batch} context={context}: "
          f"{us:.1f} us a layer (the step's embedding, final norm and head included, divided by 3 layers)")
    return {"kernel": "decode_layer" if fused else "separate", "batch": batch, "context": context, "us_per_layer": us}


def moe_case(tokens: int, reps: int, H: int = 4096, E: int = 64, top: int = 6, F: int = 768) -> dict:
    """The experts' two grouped products of a mixture (64 experts of 768 at width 4096, six a token) for a step of
    ``tokens`` tokens with choices drawn evenly: the tcgen05 form from 1024 rows on, the mma.sync form below.  The
    weights (1.2 GB) are larger than the L2; what is reported is the useful work, 6 * rows * F * H operations, and the
    weights of the experts that were chosen."""
    dev = "cuda"
    gate_up = torch.randn(E, 2 * F, H, device=dev, dtype=torch.bfloat16) * 0.02
    down = torch.randn(E, H, F, device=dev, dtype=torch.bfloat16) * 0.02
    h = torch.randn(tokens, H, device=dev, dtype=torch.bfloat16)
    rows = tokens * top
    ids = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(tokens)]).to(torch.int32).reshape(-1)
    weights = torch.rand(rows, device=dev)
    place = torch.empty(rows, device=dev, dtype=torch.int32)
    big = rows >= ops.MOE_TC_ROWS and rows >= ops.MOE_TC_ROWS_PER_EXPERT * E
    tile = ops.MOE_TC_TILE if big else ops.MOE_TILE
    tiles = ops.moe_max_tiles(rows, E, tile)
    grouped = torch.empty(tiles * tile, device=dev, dtype=torch.int32)
    tile_expert = torch.empty(tiles, device=dev, dtype=torch.int32)
    used = torch.empty(1, device=dev, dtype=torch.int32)
    ops.moe_group(ids, E, grouped, place, tile_expert, tile, used)
    act = torch.empty(tiles * tile, F, device=dev, dtype=torch.bfloat16)
    if big:
        hg = torch.empty(tiles * tile, H, device=dev, dtype=torch.bfloat16)
        scale = torch.empty(tiles * tile, device=dev)
        ops.moe_gather(h, grouped, weights, top, hg, scale, used, tile)
        parts = torch.empty(tiles * tile, H, device=dev, dtype=torch.bfloat16)
        up = lambda i: ops.gemm_tc_grouped(hg, gate_up, act, tile_expert, used, True, scale, 7.0, 1.702)
        dn = lambda i: ops.gemm_tc_grouped(act, down, parts, tile_expert, used)
    else:
        parts = torch.empty(tiles * tile, H, device=dev, dtype=torch.float32)
        up = lambda i: ops.moe_gemm_mma(h, gate_up, act, grouped, tile_expert, weights, top, True, 7.0, 1.702, True)
        dn = lambda i: ops.moe_gemm_mma(act, down, parts, grouped, tile_expert, None, top, False)
    us_up, us_dn = _time(up, reps), _time(dn, reps)
    chosen = int(torch.unique(ids).numel())
    form = "tcgen05" if big else "mma.sync"
    print(f"moe experts ({form}) tokens={tokens} rows={rows} experts chosen={chosen}/{E}: gate/up {us_up:.1f} us "
          f"({4.0 * rows * F * H / us_up / 1e6:.0f} TFLOP/s, {chosen * 2 * F * H * 2 / us_up / 1e3:.0f} GB/s of weights), "
          f"down {us_dn:.1f} us ({2.0 * rows * F * H / us_dn / 1e6:.0f} TFLOP/s, {chosen * F * H * 2 / us_dn / 1e3:.0f} GB/s)")
    return {"kernel": f"moe_{form}", "tokens": tokens, "rows": rows, "experts_chosen": chosen, "us_gate_up": us_up,
            "us_down": us_dn, "tflops_gate_up": 4.0 * rows * F * H / us_up / 1e6, "tflops_down": 2.0 * rows * F * H / us_dn / 1e6,
            "weights_gbs_gate_up": chosen * 2 * F * H * 2 / us_up / 1e3, "weights_gbs_down": chosen * F * H * 2 / us_dn / 1e3}


# ----------------------------------------------------------------------------- the kernels of the state-keeping mixers
def _steps(q_len: int, batch: int):
    """cu_q, seq_of_token, positions, slots and the segment items of ``batch`` requests that bring ``q_len`` tokens each."""
    dev = "cuda"
    cu = torch.arange(batch + 1, device=dev, dtype=torch.int32) * q_len
    seq_of = torch.arange(batch, device=dev, dtype=torch.int32).repeat_interleave(q_len)
    pos = torch.arange(q_len, device=dev, dtype=torch.int32).repeat(batch)
    slots = torch.arange(batch, device=dev, dtype=torch.int32)
    arrays, values = ops.segment_work([q_len] * batch)
    work = {**{k: torch.from_numpy(v).to(dev) for k, v in arrays.items()}, **values}
    return cu, seq_of, pos, slots, work


def retention_case(q_len: int, batch: int, reps: int, H: int = 16, D: int = 64, DV: int = 128) -> dict:
    """Retention of ``batch`` requests that bring ``q_len`` tokens each: 16 heads of 64 x 128, rotary over the whole key."""
    dev = "cuda"
    T = q_len * batch
    cu, _, pos, slots, work = _steps(q_len, batch)
    proj = torch.randn(T, H * (2 * D + 2 * DV), device=dev, dtype=torch.bfloat16)
    table = torch.rand(max(q_len, 2), D, device=dev)
    decay = torch.full((H,), 0.97, device=dev)
    state = torch.zeros(batch, H, D, DV, device=dev)
    o = torch.empty(T, H * DV, device=dev)
    out = torch.empty(T, H * DV, device=dev, dtype=torch.bfloat16)
    a, b = H * D, 2 * H * D
    fn = lambda i: ops.retention(proj[:, :a], proj[:, a:b], proj[:, b:b + H * DV], table, pos, decay, D ** -0.5, state, slots,
                                 cu, batch, o, H, D, DV, work=work)
    us = _time(fn, reps)
    us_gate = _time(lambda i: ops.retention_gate(o, proj[:, b + H * DV:], out, H, DV, 1e-6, 0.5), reps)
    flops = 4.0 * T * H * D * DV * (1.5 if work["summaries"] else 1.0)
    nbytes = 2 * state.numel() * 4 + T * H * (2 * D + DV) * 2 + o.numel() * 4
    print(f"retention q_len={q_len} batch={batch} heads={H} of {D}x{DV}: {us:.1f} us ({flops / us / 1e6:.2f} TFLOP/s float, "
          f"{nbytes / us / 1e3:.0f} GB/s), gate {us_gate:.1f} us")
    return {"kernel": "retention", "q_len": q_len, "batch": batch, "us": us, "us_gate": us_gate, "tflops": flops / us / 1e6,
            "gbs": nbytes / us / 1e3}


def wkv_case(q_len: int, batch: int, reps: int, H: int = 32, D: int = 64, C: int = 2048, rank: int = 32) -> dict:
    """Time mixing's own kernels for ``batch`` requests that bring ``q_len`` tokens each: the five mixes of the token
    shift, the decays, and the recurrence of 32 heads of 64 x 64 with decays of the token's own."""
    dev = "cuda"
    T = q_len * batch
    cu, seq_of, _, slots, work = _steps(q_len, batch)
    h = torch.randn(T, C, device=dev).to(torch.bfloat16)
    mu = torch.rand(5, C, device=dev)
    prev = torch.zeros(batch, C, device=dev)
    x = torch.empty(5, T, C, device=dev, dtype=torch.bfloat16)
    r, k, v = (torch.randn(T, H * D, device=dev) for _ in range(3))
    a = torch.randn(T, rank, device=dev)
    w2_t, w0 = torch.randn(rank, H * D, device=dev) / rank ** 0.5, torch.full((H * D,), -2.0, device=dev)
    decay = torch.empty(T, H * D, device=dev)
    u = torch.randn(H * D, device=dev)
    state = torch.zeros(batch, H, D, D, device=dev)
    o = torch.empty(T, H * D, device=dev)
    us_shift = _time(lambda i: ops.token_shift_multi(h, mu, prev, slots, cu, seq_of, x), reps)
    us_decay = _time(lambda i: ops.wkv_decay(a, w2_t, w0, decay), reps)
    us = _time(lambda i: ops.wkv(r, k, v, decay, u, state, slots, cu, batch, o, H, D, D, work=work), reps)
    flops = 7.0 * T * H * D * D * (1.5 if work["summaries"] else 1.0)
    nbytes = 2 * state.numel() * 4 + T * H * D * 4 * 5
    print(f"wkv q_len={q_len} batch={batch} heads={H} of {D}x{D}: {us:.1f} us ({flops / us / 1e6:.2f} TFLOP/s float, "
          f"{nbytes / us / 1e3:.0f} GB/s), token shift {us_shift:.1f} us ({T * C * 12 / us_shift / 1e3:.0f} GB/s), "
          f"decays {us_decay:.1f} us")
    return {"kernel": "wkv", "q_len": q_len, "batch": batch, "us": us, "us_shift": us_shift, "us_decay": us_decay,
            "tflops": flops / us / 1e6, "gbs": nbytes / us / 1e3}


def recurrence_case(q_len: int, batch: int, reps: int, C: int = 4096, blocks: int = 16, taps: int = 4) -> dict:
    """The gated linear recurrence's kernels for ``batch`` requests of ``q_len`` tokens: 4096 channels in 16 blocks."""
    dev = "cuda"
    T = q_len * batch
    bw = C // blocks
    cu, seq_of, _, slots, work = _steps(q_len, batch)
    xy = torch.randn(T, 2 * C, device=dev)
    bias = torch.zeros(C, device=dev)
    taps_w = torch.randn(C, taps, device=dev)
    conv_state = torch.zeros(batch, taps - 1, C, device=dev)
    u, a, b = (torch.empty(T, C, device=dev) for _ in range(3))
    wa = (torch.randn(blocks, bw, bw, device=dev) / bw ** 0.5).to(torch.bfloat16)
    wb = (torch.randn(blocks, bw, bw, device=dev) / bw ** 0.5).to(torch.bfloat16)
    wa_t, wb_t = wa.float().transpose(1, 2).contiguous(), wb.float().transpose(1, 2).contiguous()
    sp = torch.rand(C, device=dev)
    state = torch.zeros(batch, C, device=dev)
    out = torch.empty(T, C, device=dev, dtype=torch.bfloat16)
    taps_t = taps_w.t().contiguous()
    us_conv = _time(lambda i: ops.causal_conv(xy[:, :C], bias, taps_w, bias, conv_state, slots, cu, seq_of, u, taps_t=taps_t), reps)
    us_mma = _time(lambda i: ops.block_gates(u, wa_t, bias, wb_t, bias, sp, -8.0, a, b, bf16_weights=(wa, wb)), reps)
    us_ffma = _time(lambda i: ops.block_gates(u, wa_t, bias, wb_t, bias, sp, -8.0, a, b), reps)
    us_scan = _time(lambda i: ops.gated_scan(a, b, xy[:, C:], bias, state, slots, cu, batch, out, work=work), reps)
    gflop = 4.0 * T * C * bw / 1e9
    print(f"recurrence q_len={q_len} batch={batch} channels={C} in {blocks} blocks: conv {us_conv:.1f} us "
          f"({T * C * 12 / us_conv / 1e3:.0f} GB/s), gates mma.sync {us_mma:.1f} us ({gflop / us_mma * 1e3:.1f} TFLOP/s) / FFMA "
          f"{us_ffma:.1f} us ({gflop / us_ffma * 1e3:.1f} TFLOP/s), scan {us_scan:.1f} us ({T * C * 14 / us_scan / 1e3:.0f} GB/s)")
    return {"kernel": "recurrence", "q_len": q_len, "batch": batch, "us_conv": us_conv, "us_gates_mma": us_mma,
            "us_gates_ffma": us_ffma, "us_scan": us_scan}


def norm_shift_case(q_len: int, batch: int, reps: int, H: int = 4096) -> dict:
    """Residual sum + layer norm + token shift over a float stream of width 4096."""
    dev = "cuda"
    T = q_len * batch
    cu, seq_of, _, slots, _ = _steps(q_len, batch)
    x = torch.randn(T, H, device=dev)
    delta = torch.randn(T, H, device=dev, dtype=torch.bfloat16) * 0.01
    w, b, mu = torch.ones(H, device=dev), torch.zeros(H, device=dev), torch.rand(H, device=dev)
    state = torch.zeros(batch, H, device=dev)
    n, out = torch.empty(T, H, device=dev), torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def two(i):
        ops.add_layernorm(x, delta, w, b, 1e-6, n, None, 0.5)
        ops.token_shift(n, mu, state, slots, cu, seq_of, out)

    us = _time(two, reps)
    nbytes = T * H * (4 + 4 + 2 + 2) + T * H * 8 * 2
    line = f"layer norm + token shift T={T} width={H}: two launches {us:.1f} us ({nbytes / us / 1e3:.0f} GB/s)"
    res = {"kernel": "layernorm_shift", "T": T, "us_two": us}
    if q_len == 1:
        us1 = _time(lambda i: ops.add_layernorm_shift(x, delta, w, b, 1e-6, mu, state, slots, out, 0.5), reps)
        line += f", one launch {us1:.1f} us ({T * H * 12 / us1 / 1e3:.0f} GB/s)"
        res["us_one"] = us1
    print(line)
    return res

# ----------------------------------------------------------------------------- attention with score steps; over kept latent rows
class _Step:
    pass


def _paged_step(q_len: int, batch: int, context: int, page: int):
    """The step's context, work lists and block table for ``batch`` requests that hold ``context`` tokens, the last
    ``q_len`` of them new; pages in order."""
    dev = "cuda"
    per = (context + page - 1) // page
    table = torch.arange(batch * per, device=dev, dtype=torch.int32).view(batch, per)
    ctx = _Step()
    ctx.positions = torch.arange(context - q_len, context, device=dev, dtype=torch.int32).repeat(batch)
    ctx.seq_of_token = torch.arange(batch, device=dev, dtype=torch.int32).repeat_interleave(q_len)
    cu = [i * q_len for i in range(batch + 1)]
    ctx.cu_q = torch.tensor(cu, device=dev, dtype=torch.int32)
    ctx.kv_len = torch.full((batch,), context, device=dev, dtype=torch.int32)
    ctx.table_rows = None
    arrays, values = ops.attention_work([q_len] * batch, [context] * batch, cu)
    work = {**{k: torch.from_numpy(v).to(dev) for k, v in arrays.items()}, **values}
    return ctx, work, table, batch * per


def mixed_attention_case(q_len: int, batch: int, context: int, reps: int, NH: int = 16, NKV: int = 4, D: int = 128,
                         page: int = 64, rel_rows: int = 32) -> dict:
    """Head-mixing attention (a number per head, soft cap, distance bias, mix across heads) on the tensor cores."""
    dev = "cuda"
    ctx, work, table, n_pages = _paged_step(q_len, batch, context, page)
    T = q_len * batch
    q = torch.randn(T, NH * D, device=dev).to(torch.bfloat16)
    k = torch.randn(n_pages, NKV, page, D, device=dev).to(torch.bfloat16)
    v = torch.randn(n_pages, NKV, page, D, device=dev).to(torch.bfloat16)
    temp = torch.rand(NH, device=dev) + 0.5
    talk = (torch.eye(NH, device=dev) + 0.1 * torch.randn(NH, NH, device=dev)).contiguous()
    rel = torch.randn(rel_rows, NH, device=dev)
    bucket, last = ops.distance_buckets(rel_rows, 4096.0)
    bucket = bucket.to(dev)
    out = torch.empty(T, NH * D, device=dev, dtype=torch.bfloat16)
    fn = lambda i: ops.attention_mixed(q, out, k, v, ctx.positions, ctx.seq_of_token, table, NH, NKV, D, D ** -0.5, 0,
                                       temp=temp, softcap=50.0, rel=rel, bucket_of=bucket, last_row=last, talk=talk,
                                       ctx=ctx, work=work)
    us = _time(fn, reps)
    seen = batch * (q_len * (context - q_len) + q_len * (q_len + 1) / 2)
    flops = 4.0 * NH * D * seen
    nbytes = batch * context * 2 * NKV * D * 2 + 2 * T * NH * D * 2
    print(f"mixed attention q_len={q_len} batch={batch} context={context} heads={NH}/{NKV} of {D}: {us:.1f} us "
          f"({flops / us / 1e6:.2f} TFLOP/s, {nbytes / us / 1e3:.0f} GB/s)")
    return {"kernel": "attention_mixed_tc", "q_len": q_len, "batch": batch, "context": context, "us": us,
            "tflops": flops / us / 1e6, "gbs": nbytes / us / 1e3}


def latent_attention_case(q_len: int, batch: int, context: int, reps: int, NH: int = 16, ROW: int = 576, KR: int = 512,
                          window: int = 1024, page: int = 64) -> dict:
    """Attention over kept latent rows (one key/value head; values are the front of the keys) on the tensor cores."""
    dev = "cuda"
    ctx, work, table, n_pages = _paged_step(q_len, batch, context, page)
    T = q_len * batch
    q = torch.randn(T, NH * ROW, device=dev).to(torch.bfloat16)
    pages = torch.randn(n_pages, 1, page, ROW, device=dev).to(torch.bfloat16)
    out = torch.empty(T, NH * KR, device=dev, dtype=torch.bfloat16)
    fn = lambda i: ops.attention_latent(q, out, pages, ctx, table, NH, ROW, KR, ROW ** -0.5, window, work=work)
    us = _time(fn, reps)
    seen = batch * sum(min(window, p + 1) if window > 0 else p + 1 for p in range(context - q_len, context))
    flops = 2.0 * NH * (ROW + KR) * seen
    keys = batch * (min(context, window + q_len - 1) if window > 0 else context)
    nbytes = keys * ROW * 2 + T * NH * (ROW + KR) * 2
    print(f"latent attention q_len={q_len} batch={batch} context={context} window={window} heads={NH} rows of {ROW} "
          f"(values {KR}): {us:.1f} us ({flops / us / 1e6:.2f} TFLOP/s, {nbytes / us / 1e3:.0f} GB/s)")
    return {"kernel": "attention_latent_tc", "q_len": q_len, "batch": batch, "context": context, "us": us,
            "tflops": flops / us / 1e6, "gbs": nbytes / us / 1e3}


CASES = {
    "mixed_attention_prefill": lambda r: mixed_attention_case(2048, 1, 2048, r),
    "mixed_attention_prefill_small": lambda r: mixed_attention_case(512, 1, 512, r),
    "mixed_attention_decode_b64": lambda r: mixed_attention_case(1, 64, 2048, r),
    "latent_attention_prefill": lambda r: latent_attention_case(2048, 1, 2048, r),
    "latent_attention_prefill_small": lambda r: latent_attention_case(512, 1, 512, r, window=256),
    "latent_attention_decode_b64": lambda r: latent_attention_case(1, 64, 2048, r),
    "retention_prefill": lambda r: retention_case(2048, 1, r),
    "retention_decode_b64": lambda r: retention_case(1, 64, r),
    "wkv_prefill": lambda r: wkv_case(2048, 1, r),
    "wkv_prefill_small": lambda r: wkv_case(512, 1, r),
    "wkv_decode_b64": lambda r: wkv_case(1, 64, r),
    "recurrence_prefill": lambda r: recurrence_case(2048, 1, r),
    "recurrence_decode_b64": lambda r: recurrence_case(1, 64, r),
    "norm_shift_prefill": lambda r: norm_shift_case(2048, 1, r),
    "norm_shift_decode_b64": lambda r: norm_shift_case(1, 64, r),
    "moe_decode_b64": lambda r: moe_case(64, r),
    "moe_decode_b8": lambda r: moe_case(8, r),
    "moe_prefill": lambda r: moe_case(2048, r),
    "moe_prefill_8k": lambda r: moe_case(8192, r),
    "gemm_decode": lambda r: gemm_case(8, 6144, 4096, r),
    "gemm_decode_mlp": lambda r: gemm_case(8, 24576, 4096, r),
    "gemm_decode_b64": lambda r: gemm_case(64, 24576, 4096, r),
    "gemm_prefill": lambda r: gemm_case(2048, 24576, 4096, r),
    "attention_decode": lambda r: attention_case(8, 1, 2048, r),
    "attention_decode_b64": lambda r: attention_case(64, 1, 2048, r),
    "attention_decode_32k": lambda r: attention_case(8, 1, 32768, r),
    "attention_decode_b1_128k": lambda r: attention_case(1, 1, 131072, r),
    "attention_prefill": lambda r: attention_case(1, 2048, 2048, r),
    "attention_prefill_8k": lambda r: attention_case(1, 2048, 8192, r),
    "attention_prefill_mma_sync": lambda r: attention_case(1, 2048, 2048, r, legacy=True),
    "gemm_prefill_down": lambda r: gemm_case(2048, 4096, 12288, r),
    "attention_decode_splits": decode_split_case,
    "gemm_tile_widths": tile_width_case,
    "gemm_pairs": pair_case,
    "sample": lambda r: sample_case(8, 151936, r),
    "decode_layer_fused": lambda r: decode_layer_case(8, 2048, r, True),
    "decode_layer_separate": lambda r: decode_layer_case(8, 2048, r, False),
}


def bench_kernels(cases=None, reps: int = 6) -> dict:
    """{case: its figures} for the named cases (default: all)."""
    ops.library()
    return {name: CASES[name](reps) for name in (cases or sorted(CASES))}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--reps", type=int, default=6)
    args = ap.parse_args(argv)
    ops.library()
    CASES[args.case](args.reps)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
