"""The attention kernels of the Nizedra parts alone, on pages filled by hand, against dense float64 sums written out
here: the head-mixing attention in both of its kernels (one block a token; tiles of 16 tokens with all heads on the
tensor cores, a cluster of CTAs where the heads are many), portions beside one-token requests in one call, pages in
any order, windows, bias tables whose last row is reached, keys at page borders; and the attention over kept latent
rows (one key/value head whose values are the front of its keys) in its generic and its tensor-core kernel."""

from __future__ import annotations

import math

import pytest
import torch

from acvram_b200.kernels import ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


class Step:
    pass


def paged_case(NKV, D, DV, page, lens, q_lens, seed, dtype):
    """Pages in a shuffled order for requests of ``lens`` tokens whose last ``q_lens`` are this step's; unit-RMS keys."""
    g = torch.Generator().manual_seed(seed)
    per = [(n + page - 1) // page for n in lens]
    n_pages = sum(per) + 3
    order = torch.randperm(n_pages, generator=g)
    table = torch.full((len(lens), max(per)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(per):
        table[b, :n] = order[at:at + n]
        at += n
    k = torch.randn(n_pages, NKV, page, D, generator=g)
    k = (k / k.pow(2).mean(-1, keepdim=True).sqrt()).to(dtype)
    v = torch.randn(n_pages, NKV, page, DV, generator=g).to(dtype)
    ctx = Step()
    ctx.positions = torch.cat([torch.arange(n - q, n) for n, q in zip(lens, q_lens)]).to(torch.int32).to(DEV)
    ctx.seq_of_token = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32).to(DEV)
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    ctx.cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
    ctx.kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    ctx.table_rows = None
    arrays, values = ops.attention_work(q_lens, lens, cu)
    work = {n: torch.as_tensor(a).to(DEV) for n, a in arrays.items()}
    work.update(values)
    return ctx, work, table.to(DEV), k.to(DEV), v.to(DEV), cu[-1]


def dense_mixed(q, k_pages, v_pages, table, lens, q_lens, NH, NKV, D, DV, scale, window, temp, cap, rel, far, talk):
    """float64, request by request: score, times temp, soft cap, plus the bias of the distance's row, mixed over the
    heads, softmax over the visible keys, weighted sum of values."""
    page = k_pages.shape[2]
    out = []
    t0 = 0
    rows = rel.shape[0] if rel is not None else 0

    def row_of(n):
        half = rows // 2
        return n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))

    for b, (n, ql) in enumerate(zip(lens, q_lens)):
        pages = table[b].long().cpu()
        js = torch.arange(n)
        kk = k_pages.cpu().double()[pages[js // page], :, js % page]          # [n, NKV, D]
        vv = v_pages.cpu().double()[pages[js // page], :, js % page]
        qq = q[t0:t0 + ql, :NH * D].cpu().double().view(ql, NH, D)
        s = torch.einsum("ihd,jhd->hij", qq, kk.repeat_interleave(NH // NKV, dim=1)) * scale
        if temp is not None:
            s = s * temp.cpu().double()[:, None, None]
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        pos = torch.arange(n - ql, n)
        dist = pos[:, None] - js[None, :]
        if rel is not None:
            idx = torch.tensor([[row_of(int(d)) if d >= 0 else 0 for d in r] for r in dist])
            s = s + rel.cpu().double()[idx].permute(2, 0, 1)
        if talk is not None:
            s = torch.einsum("hg,gij->hij", talk.cpu().double(), s)
        seen = (dist >= 0) & ((dist < window) if window > 0 else torch.ones_like(dist, dtype=torch.bool))
        p = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1)
        out.append(torch.einsum("hij,jhd->ihd", p, vv.repeat_interleave(NH // NKV, dim=1)).reshape(ql, NH * DV))
        t0 += ql
    return torch.cat(out)


CASES = [
    # NH NKV  D   DV page  lens             q_lens          window rel far   cap
    (4, 2, 16, 24, 16, [37, 5, 70], [37, 1, 20], 0, 12, 100.0, 30.0),
    (4, 2, 48, 48, 16, [150, 129, 64, 17], [150, 1, 2, 17], 0, 16, 120.0, 50.0),      # the last row is reached
    (3, 3, 40, 8, 16, [100, 33], [50, 1], 20, 6, 17.0, 0.0),                          # a window, no cap, odd head count
    (8, 1, 64, 64, 64, [200, 150], [130, 1], 48, 0, 0.0, 0.0),                        # no bias table
    (32, 8, 32, 32, 16, [90, 60], [40, 1], 0, 8, 50.0, 20.0),                         # a cluster of two CTAs
    (40, 40, 16, 16, 16, [50, 33], [18, 1], 0, 10, 40.0, 10.0),                       # a cluster of four
    # one-token requests whose keys several CTAs share (partial results merged by a second launch): alone, beside a
    # portion, with a short request whose last shares are empty, under a window, in clusters
    (4, 2, 32, 32, 16, [700, 520, 40], [1, 1, 1], 0, 12, 300.0, 30.0),
    (8, 2, 64, 64, 64, [600, 900], [40, 1], 0, 16, 500.0, 50.0),
    (4, 4, 16, 24, 16, [1500, 70], [1, 1], 600, 8, 90.0, 0.0),
    (32, 8, 32, 32, 16, [800, 300], [1, 1], 0, 8, 50.0, 20.0),
    # one-token requests with a warp a key/value head: groups of 3, of 12 (the tile's upper half in part) and of 16
    (6, 2, 40, 24, 16, [300, 77, 5], [1, 1, 1], 0, 10, 50.0, 20.0),
    (12, 1, 32, 32, 16, [400, 33], [1, 1], 0, 8, 60.0, 0.0),
    (16, 1, 64, 64, 64, [700, 130], [1, 1], 90, 0, 0.0, 30.0),
    (16, 16, 16, 16, 16, [90, 600], [7, 1], 0, 6, 30.0, 10.0),                        # sixteen key/value heads of one head each
    # shapes whose one-token requests stay in the tile kernel (more than 16 key/value heads; more than 16 heads to one),
    # with their keys shared among clusters
    (40, 40, 16, 16, 16, [700, 300], [1, 1], 0, 10, 40.0, 10.0),
    (32, 1, 32, 32, 16, [600, 45], [1, 1], 0, 8, 50.0, 20.0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"h{c[0]}k{c[1]}d{c[2]}v{c[3]}")
def test_head_mixing_attention_kernels(case):
    NH, NKV, D, DV, page, lens, q_lens, window, rel_rows, far, cap = case
    ctx, work, table, k, v, T = paged_case(NKV, D, DV, page, lens, q_lens, 5 + NH, torch.bfloat16)
    g = torch.Generator().manual_seed(NH * 7 + D)
    q = torch.randn(T, NH * D + 64, generator=g)                 # queries are the first columns of wider rows
    q = (q / q.pow(2).mean(-1, keepdim=True).sqrt()).to(torch.bfloat16).to(DEV)
    temp = (torch.rand(NH, generator=g) + 0.5).to(DEV)
    talk = (torch.eye(NH) + 0.2 * torch.randn(NH, NH, generator=g)).contiguous().to(DEV)
    rel = torch.randn(rel_rows, NH, generator=g).to(DEV) if rel_rows else None
    bucket, last = ops.distance_buckets(rel_rows, far) if rel_rows else (None, 0)
    bucket = bucket.to(DEV) if bucket is not None else None
    scale = D ** -0.5 * 6.0
    want = dense_mixed(q, k, v, table, lens, q_lens, NH, NKV, D, DV, scale, window, temp, cap, rel, far, talk)
    kw = dict(value_dim=DV, temp=temp, softcap=cap, rel=rel, bucket_of=bucket, last_row=last, talk=talk)
    ref = float(want.abs().max())
    # one block a token, in float32 on the same (bfloat16-exact) numbers
    out = torch.zeros((T, NH * DV), device=DEV, dtype=torch.float32)
    ops.attention_mixed(q.float(), out, k.float(), v.float(), ctx.positions, ctx.seq_of_token, table, NH, NKV, D, scale,
                        window, **kw)
    assert float((out.cpu().double() - want).abs().max()) < 2e-4 * ref
    # tensor cores: bfloat16 weights of the softmax and a bfloat16 result
    assert ops.attention_mixed_tc_takes(torch.bfloat16, NH, NKV, D, DV, rel_rows)
    out = torch.full((T, NH * DV), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.attention_mixed(q, out, k, v, ctx.positions, ctx.seq_of_token, table, NH, NKV, D, scale, window, ctx=ctx,
                        work=work, **kw)
    assert float((out.cpu().double() - want).abs().max()) < 2e-2 * ref


def test_head_mixing_tensor_core_kernel_refuses_what_it_cannot_hold():
    assert not ops.attention_mixed_tc_takes(torch.float32, 4, 2, 16, 16, 8)
    assert not ops.attention_mixed_tc_takes(torch.bfloat16, 4, 2, 12, 16, 8)        # rows that are no 16-byte pieces
    assert not ops.attention_mixed_tc_takes(torch.bfloat16, 4, 2, 16, 256, 8)       # values too wide for the registers
    assert not ops.attention_mixed_tc_takes(torch.bfloat16, 6, 4, 16, 16, 8)


LATENT_CASES = [
    # NH  ROW  KR  page  lens              q_lens        window
    (8, 144, 128, 64, [200, 150, 97], [130, 1, 2], 96),          # one warp a row group; a portion, a decoded token, two tokens
    (4, 40, 32, 16, [70, 33], [70, 1], 0),                       # narrow values, no window, rows that are no multiple of 16
    (16, 320, 256, 16, [300, 140], [45, 1], 64),                 # two warps share a row group
    (16, 576, 512, 64, [400, 300, 64], [150, 1, 1], 128),        # four warps share a row group; key tiles of 32
    (3, 72, 48, 16, [90, 21], [17, 1], 10),                      # odd head count: a row group holds heads of several tokens
    (80, 576, 512, 16, [60, 40], [9, 1], 0),                     # more heads than one CTA takes: head blocks
    (16, 144, 128, 16, [900, 40, 1300], [1, 1, 1], 0),           # one-token requests whose rows several CTAs share
    (8, 320, 256, 64, [1500, 700], [1, 1], 600),                 # the same under a window
]


@pytest.mark.parametrize("case", LATENT_CASES, ids=lambda c: f"h{c[0]}row{c[1]}kr{c[2]}")
def test_latent_rows_attention_kernels(case):
    NH, ROW, KR, page, lens, q_lens, window = case
    ctx, work, table, k, _, T = paged_case(1, ROW, 8, page, lens, q_lens, 11 + NH, torch.bfloat16)
    v = k[..., :KR].contiguous()                                   # the values: the first KR elements of the kept rows
    g = torch.Generator().manual_seed(NH * 5 + ROW)
    q = torch.randn(T, NH * ROW, generator=g)
    q = (q / q.pow(2).mean(-1, keepdim=True).sqrt()).to(torch.bfloat16).to(DEV)
    scale = ROW ** -0.5 * 5.0
    want = dense_mixed(q, k, v, table, lens, q_lens, NH, 1, ROW, KR, scale, window, None, 0.0, None, 0.0, None)
    ref = float(want.abs().max())
    # the generic paged kernel in float32 on the same (bfloat16-exact) numbers
    out = torch.zeros((T, NH * KR), device=DEV, dtype=torch.float32)
    ops.attention_latent(q.float(), out, k.float(), ctx, table, NH, ROW, KR, scale, window)
    assert float((out.cpu().double() - want).abs().max()) < 2e-4 * ref
    # tensor cores: bfloat16 weights of the softmax and a bfloat16 result
    assert ops.attention_latent_tc_takes(torch.bfloat16, NH, ROW, KR)
    before = ops.LAUNCHES
    out = torch.full((T, NH * KR), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.attention_latent(q, out, k, ctx, table, NH, ROW, KR, scale, window, work=work)
    assert ops.LAUNCHES == before + 1
    assert float((out.cpu().double() - want).abs().max()) < 2e-2 * ref
    # one-token requests alone take units of one token
    dec = [i for i, n in enumerate(q_lens) if n == 1]
    arrays, values = ops.attention_work([1] * len(dec), [lens[i] for i in dec], list(range(len(dec) + 1)))
    work1 = {n: torch.as_tensor(a).to(DEV) for n, a in arrays.items()}
    work1.update(values)
    step = Step()
    step.cu_q = torch.arange(len(dec) + 1, dtype=torch.int32, device=DEV)
    step.kv_len = torch.tensor([lens[i] for i in dec], dtype=torch.int32, device=DEV)
    step.table_rows = None
    rows = torch.tensor([sum(q_lens[:i]) for i in dec], device=DEV)
    out1 = torch.full((len(dec), NH * KR), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.attention_latent(q[rows].contiguous(), out1, k, step, table[torch.tensor(dec, device=DEV)].contiguous(), NH, ROW, KR,
                         scale, window, work=work1)
    assert float((out1.cpu().double() - want[rows.cpu()]).abs().max()) < 2e-2 * ref


def test_latent_rows_tensor_core_kernel_refuses_what_it_cannot_hold():
    assert not ops.attention_latent_tc_takes(torch.float32, 8, 144, 128)
    assert not ops.attention_latent_tc_takes(torch.bfloat16, 8, 140, 128)           # rows that are no 16-byte pieces
    assert not ops.attention_latent_tc_takes(torch.bfloat16, 8, 1088, 1024)         # latents too wide for the registers


@pytest.mark.parametrize("T,B,K,N,pad_a,pad_c", [(70, 3, 64, 96, 16, 8), (1, 16, 64, 512, 64, 64), (200, 4, 136, 50, 0, 0),
                                                 (33, 2, 12, 20, 4, 3), (130, 5, 512, 128, 0, 0)])
def test_per_head_products_over_strided_views(T, B, K, N, pad_a, pad_c):
    """out[:, b, :] = a[:, b, :] @ w[b]^T on views into wider rows: on the tensor cores where rows are 16-byte pieces,
    on the CUDA cores otherwise, and in float32; rows past a tile's end and K that is no multiple of the tile."""
    g = torch.Generator().manual_seed(T + K)
    a_full = torch.randn(T, B, K + pad_a, generator=g)
    w = (torch.randn(B, N, K, generator=g) * K ** -0.5)
    want = torch.einsum("tbk,bnk->tbn", a_full[:, :, :K].to(torch.bfloat16).double(), w.to(torch.bfloat16).double())
    ref = float(want.abs().max())
    for dtype, tol in ((torch.bfloat16, 1e-2), (torch.float32, 1e-5)):
        a = a_full.to(torch.bfloat16).to(dtype).to(DEV)
        wd = w.to(torch.bfloat16).to(dtype).to(DEV).contiguous()
        out_full = torch.full((T, B, N + pad_c), 7.0, device=DEV, dtype=dtype)
        ops.gemm_batched(a[:, :, :K], wd, out_full[:, :, :N])
        assert float((out_full[:, :, :N].cpu().double() - want).abs().max()) < tol * ref
        assert bool((out_full[:, :, N:] == 7.0).all())                  # nothing beside the view is written
