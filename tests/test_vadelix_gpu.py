"""Vadelix on the GPU: the engine against the plain implementation of tests/plain_vadelix.py.

Small configurations with random weights (tests/vadelix_util.py), logits asked at every position.  float32 runs must
agree with the float64 oracle to rounding, whatever the cut into steps, the batch, the pages or the state slots;
bfloat16 runs within what rounding does: judged by the median position, and seven positions in eight must stay under
a loose bound (a router's close call sends a token to another expert than the oracle's, which moves that position's
logits as a whole and, through keys, values and states, the positions behind it a little; single positions are judged
sharply in float32 here and at the kernels in bfloat16).
"""

from __future__ import annotations

import functools
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vadelix as pv
import vadelix_util as vu
from conftest import ROOT

pytestmark = pytest.mark.gpu

F32_BOUND = 2e-4        # float32 engine against the float64 oracle, per position (relative, see vu.row_errors)
BF16_MEDIAN, BF16_WORST = 0.04, 0.25     # bfloat16: the median position, and seven in eight


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("vadelix")
    return {w: vu.write_model(str(root / w), vu.config(w), seed=51 + i) for i, w in enumerate("ABCD")}


@functools.lru_cache(maxsize=None)
def _read(folder):
    return vu.read_folder(folder)


@functools.lru_cache(maxsize=None)
def oracle(folder: str, ids: tuple) -> np.ndarray:
    cfg, tensors = _read(folder)
    return pv.forward(cfg, tensors, list(ids))


def ids_of(folder, n, seed):
    rng = random.Random(seed)
    vocab = _read(folder)[0]["vocab"]
    return tuple(rng.randrange(vocab) for _ in range(n))


def make_runner(folder, dtype, pages=64, page_size=16, max_requests=4, graphs=False):
    from acvram_b200.engine.runner import ModelRunner
    from acvram_b200.models import build_from_folder
    _, model = build_from_folder(folder, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], "cuda:0")
    runner = ModelRunner(model, page_size, pages, max_requests)
    if graphs:
        runner.enable_graphs()
    return runner


def play(runner, requests: dict, steps) -> dict:
    """steps: list of {request: number of its next tokens}; a request is released with its last token.  Returns
    {request: logits [len, vocab]} with logits asked at every position."""
    from acvram_b200.engine.batch import StepEntry
    at = {r: 0 for r in requests}
    rows = {r: [] for r in requests}
    for step in steps:
        entries = [StepEntry(r, list(requests[r][at[r]:at[r] + n]), list(range(n))) for r, n in step.items()]
        logits = runner.step(entries).cpu()
        runner.check_status()
        o = 0
        for r, n in step.items():
            rows[r].append(logits[o:o + n])
            o += n
            at[r] += n
            if at[r] == len(requests[r]):
                runner.release(r)
    runner.manager.check()
    assert all(at[r] == len(requests[r]) for r in requests), "the schedule does not cover the requests"
    return {r: torch.cat(v).numpy() for r, v in rows.items()}


def agree(folder, requests, got, dtype, what=""):
    for r, ids in requests.items():
        err = vu.row_errors(got[r], oracle(folder, tuple(ids)))
        assert np.isfinite(err).all(), f"{what} {r}: not finite"
        if dtype == "float32":
            bad = np.nonzero(err > F32_BOUND)[0].tolist()
            assert not bad, f"{what} {r}: positions {bad[:8]} differ by {err[bad[:8]].tolist()}"
        else:
            over = int((err > BF16_WORST).sum())
            # (a request of a few tokens has no typical position: one close call is its median)
            assert (len(err) < 8 or float(np.median(err)) < BF16_MEDIAN) and over <= max(1, len(err) // 8), \
                f"{what} {r}: median {float(np.median(err)):.4f}, {over} of {len(err)} over {BF16_WORST}, largest at {int(err.argmax())}"


# --------------------------------------------------------------------------- whole prompts, layer by layer
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_whole_prompts(folders, which, dtype):
    f = folders[which]
    runner = make_runner(f, dtype)
    requests = {f"w{n}": ids_of(f, n, n) for n in (1, 2, 23, 150, 333)}     # the first tokens alone; page and window borders
    got = play(runner, requests, [{r: len(ids)} for r, ids in requests.items()])
    agree(f, requests, got, dtype, "whole")


@pytest.mark.parametrize("which", ["A", "C"])
def test_stream_after_every_layer(folders, which):
    f = folders[which]
    runner = make_runner(f, "float32")
    ids = ids_of(f, 61, 5)
    streams = []
    for blk in runner.model.blocks:
        def wrapped(x, delta, ctx, cache, orig=blk.forward, mult=blk.residual_mult):
            x, d = orig(x, delta, ctx, cache)
            streams.append((x.double() + mult * d.double()).cpu().numpy())     # the part's output joins in the next norm
            return x, d
        blk.forward = wrapped
    play(runner, {"s": ids}, [{"s": len(ids)}])
    cfg, tensors = _read(f)
    want = []
    pv.forward(cfg, tensors, list(ids), streams=want)
    assert len(streams) == len(want) == len(cfg["layers"])
    for run, (g, w) in enumerate(zip(streams, want)):
        assert float(np.abs(g - w).max()) < 1e-4 * float(np.abs(w).max()), f"the stream leaves the oracle's after layer {run}"


# --------------------------------------------------------------------------- prefill against decoding, portions
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_decoding_token_by_token(folders, which, dtype):
    """A prompt, then 120 tokens one by one: over page borders (16), past every window (7 to 80), through the query
    temperature's steps; in bfloat16 through captured graphs.  A second request decodes from its second token on (its
    convolution and token shift begin from zeros)."""
    f = folders[which]
    runner = make_runner(f, dtype, graphs=dtype == "bfloat16")
    requests = {"d": ids_of(f, 37 + 120, 21), "e": ids_of(f, 1 + 30, 22)}
    steps = [{"d": 37}] + [{"d": 1}] * 120 + [{"e": 1}] * 31
    got = play(runner, requests, steps)
    agree(f, requests, got, dtype, "decode")
    if dtype == "bfloat16":
        assert runner.graph_launches > 0, "the decode steps did not replay a captured graph"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_portions_of_any_size(folders, which, dtype):
    """Portions shorter than the convolution's reach (2 and 3 tokens under 3 and 5 taps), longer than a segment of the
    recurrence (70 tokens), and single tokens between them."""
    f = folders[which]
    runner = make_runner(f, dtype)
    ids = ids_of(f, 260, 31)
    sizes = [2, 3, 2, 17, 5, 31, 2, 70, 1, 7, 64, 2, 16, 1, 1, 1]
    sizes.append(len(ids) - sum(sizes))
    got = play(runner, {"p": ids}, [{"p": n} for n in sizes])
    agree(f, {"p": ids}, got, dtype, "portions")


def test_long_decoding_in_few_pages(folders):
    """C in pages of 8: the windows of 7 and 33 keep a page or a few, the rotated layer every page.  A request of 500
    tokens, 400 of them decoded one by one: the windows' pages are written again and again and the recurrence's state
    runs on for hundreds of steps."""
    f = folders["C"]
    runner = make_runner(f, "float32", pages=80, page_size=8, max_requests=2)
    ids = ids_of(f, 500, 77)
    got = play(runner, {"long": ids}, [{"long": 30}, {"long": 11}, {"long": 2}, {"long": 30}, {"long": 27}] + [{"long": 1}] * 400)
    agree(f, {"long": ids}, got, "float32", "long")


# --------------------------------------------------------------------------- batches, pages and slots used again
def mixed_schedule(requests: dict, seed: int, max_live: int):
    rng = random.Random(seed)
    waiting = list(requests)
    live, at, steps = [], {}, []
    while waiting or live:
        while waiting and len(live) < max_live:
            r = waiting.pop(0)
            live.append(r)
            at[r] = 0
        step = {}
        for r in list(live):
            if step and rng.random() < 0.2:
                continue                                   # left out of this step
            left = len(requests[r]) - at[r]
            n = 1 if left <= 12 else min(left - 12, rng.choice([2, 3, 9, 16, 29, 50, 75]))
            step[r] = n
            at[r] += n
            if at[r] == len(requests[r]):
                live.remove(r)
        steps.append(step)
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_mixed_batches_in_a_small_pool(folders, which, dtype):
    """Seven unequal requests, three live at a time, portions beside single tokens, with rows of the block tables, pages
    and state slots for three requests: all are used again (the convolution's rows, the previous token and the
    recurrence's state of a slot's former request must be gone), and every request must come out as it does alone."""
    f = folders[which]
    lengths = (90, 14, 131, 1, 57, 160, 33)
    requests = {f"m{i}": ids_of(f, n, 40 + i) for i, n in enumerate(lengths)}
    pages = 3 * (-(-160 // 16))
    runner = make_runner(f, dtype, pages=pages, max_requests=3, graphs=dtype == "bfloat16")
    got = play(runner, requests, mixed_schedule(requests, 7, 3))
    agree(f, requests, got, dtype, "mixed")
    assert all(g.pool.num_free == pages for g in runner.manager.paged_groups)
    assert all(g.num_free == 3 for g in runner.manager.state_groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_decides(folders, dtype):
    """B's rotated attention has a sharp softmax and no window: position 600 must find the keys of the first tokens.
    The oracle's logits without those tokens differ from the true ones by more than the bounds, so a kernel that lost
    them fails."""
    f = folders["B"]
    ids = ids_of(f, 640, 99)
    runner = make_runner(f, dtype, pages=48)
    got = play(runner, {"far": ids}, [{"far": 590}] + [{"far": 1}] * 50)
    agree(f, {"far": ids}, got, dtype, "far")
    cut = oracle(f, tuple(ids[48:]))                   # the same tokens without the first three pages
    err = vu.row_errors(cut[-40:], oracle(f, ids)[-40:])
    assert float(np.median(err)) > 2 * BF16_MEDIAN, "the far keys do not matter in this test: it shows nothing"


def _shouting(cfg, seed):
    """Weights in which token 63 shouts: its embedding is the stream's element 0 alone, which no other token has, and
    the convolution leaves that element to its own token."""
    w = vu.random_weights(cfg, seed)
    w["embed"][:, 0] = 0.0
    w["embed"][63] = 0.0
    w["embed"][63, 0] = 1.0
    w["l0.norm1"][0] = 1.0
    w["l0.canon1"][0, :] = 0.0
    return w


def _edges(f, places, n, steps_list):
    """``places``: (position of the shouting token, whether the last position sees it)."""
    c, tensors = vu.read_folder(f)
    base = [t % 60 for t in ids_of(f, n, 4)]
    quiet = pv.forward(c, tensors, base)[-1]
    for place, seen in places:
        ids = list(base)
        ids[place] = 63
        want = pv.forward(c, tensors, ids)
        moved = float(vu.row_errors(want[-1:], quiet[None])[0])
        assert (moved > 0.3) if seen else (moved < 1e-5), f"the oracle itself: place {place} moves the last logits by {moved}"
        for steps in steps_list:
            runner = make_runner(f, "float32", pages=8)
            got = play(runner, {"r": ids}, steps)["r"]
            assert float(vu.row_errors(got, want).max()) < F32_BOUND, f"place {place}, steps {steps[:2]}"


def test_the_windows_edge_decides(tmp_path):
    """One windowed layer alone, window 12.  The shouting token's value row stands out and its key is like any other's.
    It is placed just inside the window of the last position and just outside it (two places further back, since the
    convolution of 3 taps carries a token's other channels two positions on), for a prompt, for a decoded token and for
    portions."""
    cfg = vu.model(64, 32, [vu.layer(vu.window_attention(2, 1, 8, 8, 12, (0.3, 4), scale=0.05), None)], 1e-5, 2, 0.9, 3)
    w = _shouting(cfg, 3)
    w["l0.mix.v"][:, 0] = 4.0
    w["l0.mix.q"][:, 0] = 0.0
    w["l0.mix.k"][:, 0] = 0.0
    f = vu.write_model(str(tmp_path / "edge"), cfg, 0, w)
    n = 40
    _edges(f, ((n - 15, False), (n - 12, True), (0, False)), n,
           ([{"r": n}], [{"r": n - 1}, {"r": 1}], [{"r": 3}, {"r": n - 8}] + [{"r": 1}] * 5))


def test_the_convolutions_reach_decides(tmp_path):
    """One recurrence layer alone whose decays are tiny (the state forgets at once) and whose mixes look at the current
    token only, under a convolution of 4 taps: the last position sees the shouting token through the convolution up to
    3 positions back, through the state one position more (a token's own k v^T enters the state undecayed), and no
    further, whatever the cut (the kept rows of a request cross steps of 1, 2 and 3 tokens)."""
    cfg = vu.model(64, 32, [vu.layer(vu.wkv(2, 8, rank=2), None)], 1e-5, 1, 1.0, 4)
    w = vu.random_weights(cfg, 9)
    w["embed"][:, 0] = 0.0
    w["embed"][63] = 0.0
    w["embed"][63, 0] = 1.0
    w["l0.norm1"][0] = 1.0
    w["l0.canon1"][0, :] = 1.0
    for s in "rkvgw":
        w["l0.mix.mu." + s][:] = 0.0
    w["l0.mix.w0"][:] = 3.0            # decay exp(-exp(3)): nothing survives a step
    w["l0.mix.w2"][:] = 0.0
    w["l0.mix.v"][:, 0] = 4.0
    f = vu.write_model(str(tmp_path / "reach"), cfg, 0, w)
    n = 30
    _edges(f, ((n - 6, False), (n - 5, True), (n - 2, True)), n,
           ([{"r": n}], [{"r": n - 1}, {"r": 1}], [{"r": n - 6}, {"r": 1}, {"r": 2}, {"r": 3}], [{"r": n - 7}] + [{"r": 1}] * 7))


def test_the_sink_takes_its_share(tmp_path):
    """One rotated attention layer alone.  With sinks of +6 (far above every score) the layer's output all but vanishes;
    with sinks of -30 it is a plain softmax.  The engine must follow the oracle in both, and the two oracles differ."""
    cfg = vu.model(64, 32, [vu.layer(vu.attention(2, 1, 8, 8, vu.rot(100.0, 4)), None)], 1e-5, 2, 1.0, 2)
    ids = [t % 64 for t in range(7, 47)]
    outs = []
    for sink in (6.0, -30.0):
        w = vu.random_weights(cfg, 11)
        w["l0.mix.sink"][:] = sink
        f = vu.write_model(str(tmp_path / f"sink{int(sink)}"), cfg, 0, w)
        c, tensors = vu.read_folder(f)
        want = pv.forward(c, tensors, ids)
        outs.append(want)
        for dtype in ("float32", "bfloat16"):
            runner = make_runner(f, dtype, pages=8)
            got = play(runner, {"r": ids}, [{"r": 30}] + [{"r": 1}] * 10)["r"]
            err = vu.row_errors(got, want)
            assert float(err.max()) < (F32_BOUND if dtype == "float32" else BF16_WORST), f"sink {sink}, {dtype}: {float(err.max())}"
    assert float(np.median(vu.row_errors(outs[0], outs[1]))) > 0.2, "the sink does not matter in this test: it shows nothing"


# --------------------------------------------------------------------------- the entry points
@pytest.mark.parametrize("which", ["A", "D"])
def test_greedy_generation_through_the_engine(folders, which):
    from acvram_b200 import Engine, SamplingParams
    f = folders[which]
    cfg, tensors = _read(f)
    prompts = [list(ids_of(f, 19, 1)), list(ids_of(f, 70, 2)), list(ids_of(f, 3, 3))]
    want = [pv.greedy(cfg, tensors, p, 12) for p in prompts]
    for dtype in ("float32", "bfloat16"):
        engine = Engine(f, dtype, max_batch_size=3, max_model_len=128, page_size=16, num_pages=24, token_budget=48,
                        device="cuda:0")
        got = engine.generate_batch(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
        assert not engine.stats.failed_steps, engine.last_error
        if dtype == "float32":
            assert got == want
        else:
            assert [g[:2] for g in got] == [w[:2] for w in want]


def test_trace_run_program(folders, tmp_path):
    f = folders["C"]
    ids = ids_of(f, 45, 8)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": list(ids[:30]), "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": list(ids[30:44]), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": [ids[44]], "want": [0]},
                                     {"id": "y", "tokens": list(ids[:7]), "want": [6]}], "end": ["x", "y"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", f, "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    full = oracle(f, tuple(ids))
    vocab = full.shape[1]
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, vocab)
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, vocab)
    assert float(vu.row_errors(a, full[[0, 29]]).max()) < F32_BOUND
    assert float(vu.row_errors(b, np.stack([full[44], full[6]])).max()) < F32_BOUND


@pytest.mark.parametrize("ahead", [False, True])
def test_preemption_starts_the_states_anew(folders, ahead):
    """B's rotated layer keeps all keys, so a pool of 7 pages cannot hold three requests of 55 tokens: requests are
    preempted and computed again from their first token, in state slots that others have used meanwhile.  Their states
    must start at zero again: the greedy tokens stay the oracle's."""
    from acvram_b200 import Engine, SamplingParams
    f = folders["B"]
    cfg, tensors = _read(f)
    prompts = [list(ids_of(f, n, 500 + n)) for n in (20, 25, 18)]
    want = [pv.greedy(cfg, tensors, p, 30) for p in prompts]
    engine = Engine(f, "float32", max_batch_size=3, max_model_len=128, page_size=16, num_pages=7, token_budget=16,
                    device="cuda:0", run_ahead=ahead)
    got = engine.generate_batch(prompts, SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True))
    assert not engine.stats.failed_steps, engine.last_error
    assert engine.stats.preempted > 0, "the pool was meant to be too small"
    assert got == want
    engine.runner.manager.check()
    assert all(g.num_free == g.max_requests for g in engine.runner.manager.state_groups)
