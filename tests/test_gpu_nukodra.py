"""Nukodra on the GPU against the plain implementation: the step function under every way of cutting
requests into steps, batches, pages and slots used again, then generation through the entry point.  (The new
mechanisms alone are in ``test_gpu_nukodra_parts.py``.)"""

from __future__ import annotations

import io
import itertools
import json

import numpy as np
import pytest
import torch

from nukodra_cases import (PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits, random_weights,
                           relative_error, tokens_for)

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, NukodraConfig, SamplingParams
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

# Largest |engine - plain| on a row of logits, over the row's own spread.  32-bit: rounding of sums.
# bfloat16: both sides use the same weights; activations are rounded to 8 bits between kernels.  A
# lost key, state, sink, stream or gate shows as 0.3 and more.
TOL = {"float32": 3e-4, "bfloat16": 1e-1}
CASES = [(w, d) for w in "ABCDEF" for d in ("float32", "bfloat16")]
IDS = [f"{w}-{d}" for w, d in CASES]


def setup(which, dtype, num_pages=64, seed=3, max_requests=4, raw=None):
    from mini_gpt_inference_b200.kernels.ops import default_ops

    raw = raw or config(which)
    # (sharp softmaxes in 32-bit, where nothing but the order of sums differs; in bfloat16 they would magnify
    # the rounding of queries and keys)
    tensors = random_weights(raw, seed, sharp=3.0 if dtype == "float32" else 1.0, as_bfloat16=dtype == "bfloat16")
    loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    runner = make_runner(loaded, default_ops("cuda:0"), PAGE_TOKENS[which], num_pages, max_requests)
    return raw, tensors, runner, (TOL[dtype], 0.03 if dtype == "bfloat16" else 0.0)


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_whole_prompts(which, dtype):
    raw, tensors, runner, tol = setup(which, dtype, num_pages=100)
    pt = PAGE_TOKENS[which]
    for length, seed in [(150, 1), (37, 2), (1, 3), (2, 4), (pt + 1, 5), (pt, 6), (190, 7)]:
        tokens = tokens_for(raw, length, seed)
        got = runner.step([StepEntry("r", tokens, list(range(length)))])
        runner.finish("r")
        assert got.shape == (length, raw["vocab"]) and got.dtype == torch.float32
        assert_rows_close(got, plain_logits(raw, tensors, tokens), tol[0], f"whole prompt of {length}", outliers=tol[1])
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_prefill_then_single_tokens(which, dtype):
    """A short prompt, then a long run of single tokens (replayed from a CUDA graph) that carries every window
    over decoded tokens alone, and the same sequence token by token from the very first token."""
    raw, tensors, runner, tol = setup(which, dtype)
    tokens = tokens_for(raw, 150, 7)
    want = plain_logits(raw, tensors, tokens)
    outs = [runner.step([StepEntry("r", tokens[:9], list(range(9)))])]
    outs += [runner.step([StepEntry("r", tokens[t: t + 1], [0])]) for t in range(9, 150)]
    assert_rows_close(torch.cat(outs), want, tol[0], "prefill then single tokens", outliers=tol[1])
    assert runner.graph_replays > 100
    one_by_one = torch.cat([runner.step([StepEntry("s", tokens[t: t + 1], [0])]) for t in range(40)])
    assert_rows_close(one_by_one, want[:40], tol[0], "single tokens from the first", outliers=tol[1])
    if dtype == "float32":
        # in 32-bit the cut into steps changes no bit
        assert torch.equal(one_by_one, torch.cat(outs)[:40])


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_portions_of_changing_size(which, dtype):
    raw, tensors, runner, tol = setup(which, dtype)
    tokens = tokens_for(raw, 131, 8)
    want = plain_logits(raw, tensors, tokens)
    sizes = itertools.cycle([13, 7, 2, 5, 2, 1, 3, 16, 2, 9, 33])
    outs, pos = [], 0
    while pos < len(tokens):
        n = min(next(sizes), len(tokens) - pos)
        outs.append(runner.step([StepEntry("r", tokens[pos: pos + n], list(range(n)))]))
        pos += n
    assert_rows_close(torch.cat(outs), want, tol[0], "portions of changing size", outliers=tol[1])


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_mixed_batches_reuse_pages_and_slots(which, dtype):
    """Up to four live requests, portions of some beside single tokens of others, requests left out of
    steps; pages and state slots are handed out again.  Every cache row and state slot starts as NaN and
    turns NaN again when its request ends."""
    pt = PAGE_TOKENS[which]
    lengths = [90, 29, 71, 3, 41, 2 * pt, 17, 55, 1]
    pool = sum(sorted(-(-n // pt) for n in lengths)[-4:])
    raw, tensors, runner, tol = setup(which, dtype, num_pages=pool)
    for pages in runner.storage.k + runner.storage.v:
        if pages is not None:
            pages.fill_(float("nan"))
    for state in runner.storage.state.values():
        state.fill_(float("nan") if state.is_floating_point() else -1)
    reqs = {f"q{i}": tokens_for(raw, n, 20 + i) for i, n in enumerate(lengths)}
    want = {rid: plain_logits(raw, tensors, toks) for rid, toks in reqs.items()}
    got = {rid: [] for rid in reqs}
    waiting, live = list(reqs), {}
    sizes = itertools.cycle([5, 1, 2, 11, 1, 1, 7, 3, 1, 2, 1, 1, 19])
    gen = torch.Generator().manual_seed(99)
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, order = [], []
        for rid in list(live):
            if len(live) > 1 and torch.rand((), generator=gen).item() < 0.25:
                continue
            pos = live[rid]
            n = min(next(sizes), len(reqs[rid]) - pos)
            entries.append(StepEntry(rid, reqs[rid][pos: pos + n], list(range(n))))
            order.append((rid, n))
            live[rid] = pos + n
        if not entries:
            continue
        logits = runner.step(entries)
        row = 0
        for rid, n in order:
            got[rid].append(logits[row: row + n].clone())
            row += n
            if live[rid] == len(reqs[rid]):
                held = runner.manager.get(rid)
                tables, slot = [list(t) for t in held.tables], held.state_slot
                runner.finish(rid)
                del live[rid]
                for g, table in enumerate(tables):
                    for page in table:
                        if page >= 0:
                            for pages in (runner.storage.k[g], runner.storage.v[g]):
                                if pages is not None:
                                    pages[:, page] = float("nan")
                for state in runner.storage.state.values():
                    state[slot] = float("nan") if state.is_floating_point() else -1
    for rid in reqs:
        assert_rows_close(torch.cat(got[rid]), want[rid], tol[0], f"request {rid} in mixed batches", outliers=tol[1])
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_unequal_requests_equals_each_alone(dtype):
    raw, tensors, runner, tol = setup("A", dtype, num_pages=64, max_requests=8)
    prompts = [tokens_for(raw, n, 70 + n) for n in (1, 2, 33, 64, 7)]
    alone = []
    for i, p in enumerate(prompts):
        alone.append(runner.step([StepEntry(f"a{i}", p, list(range(len(p))))]))
        runner.finish(f"a{i}")
    together = runner.step([StepEntry(f"b{i}", p, list(range(len(p)))) for i, p in enumerate(prompts)])
    if dtype == "float32":
        assert torch.equal(together, torch.cat(alone))
    else:
        assert float(relative_error(together, torch.cat(alone).cpu()).max()) < tol[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windows_pass_over_long_prompts_and_long_decoding(dtype):
    """Sequences several windows long: the prompt's later tokens and every decoded token see only their
    window's keys, while the latent layers and the state-space layer still carry the first tokens."""
    raw, tensors, runner, tol = setup("B", dtype, num_pages=40)
    tokens = tokens_for(raw, 400, 17)
    want = plain_logits(raw, tensors, tokens)
    outs = [runner.step([StepEntry("r", tokens[:300], list(range(300)))])]
    outs += [runner.step([StepEntry("r", tokens[t: t + 1], [0])]) for t in range(300, 400)]
    assert_rows_close(torch.cat(outs), want, tol[0], "long prompt, long decoding", outliers=tol[1])


# ---- generation through the entry point, its scheduler and sampler ---------------------------------
@pytest.mark.parametrize("which", "ABC")
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(which, dtype):
    raw = config(which)
    tensors = random_weights(raw, 11, as_bfloat16=dtype == "bfloat16")
    loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype=dtype, block_size=PAGE_TOKENS[which], num_blocks=48,
                                            max_batch_size=3, max_num_batched_tokens=16, max_prefill_chunk=7))
    prompts = [tokens_for(raw, n, 40 + i) for i, n in enumerate([5, 1, 23, 12, 2, 17])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 12 and out["finish_reason"] == "length"
        seq = prompt + out["token_ids"]
        want = plain_logits(raw, tensors, seq[:-1])
        for i, token in enumerate(out["token_ids"]):
            row = want[len(prompt) - 1 + i]
            assert row.max() - row[token] <= 2 * TOL[dtype] * row.std(), (i, token, int(row.argmax()))
        if dtype == "float32":
            assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 12)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


def test_preemption_and_recompute_through_the_engine():
    """A pool too small for the three running requests (no window, so that no page comes back early): requests
    are preempted, give back their pages and state slot, and are computed again from their first token in a
    slot that another request used meanwhile."""
    raw = config("C")
    tensors = random_weights(raw, 14)
    loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=10, max_batch_size=3,
                                            max_num_batched_tokens=16, max_prefill_chunk=7))
    prompts = [tokens_for(raw, n, 60 + i) for i, n in enumerate([20, 25, 18, 9])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=16, temperature=0.0))
    assert engine.scheduler.num_preemptions > 0
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 16)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


def test_long_decoding_through_the_engine():
    raw = config("A")
    tensors = random_weights(raw, 12)
    loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=40, max_batch_size=2))
    prompt = tokens_for(raw, 3, 9)
    out = engine.generate([prompt], SamplingParams(max_tokens=160, temperature=0.0))[0]
    assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 160)


def test_trace_replay(tmp_path):
    """The replay program on a model folder: two requests, portions beside single tokens, a slot and pages
    used again by a third request."""
    from mini_gpt_inference_b200.engine.trace import main
    from mini_gpt_inference_b200.weights.safetensors_io import save_file

    raw = config("A")
    tensors = random_weights(raw, 13, as_bfloat16=True)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    save_file({k: v.to(torch.bfloat16) for k, v in tensors.items()}, folder / "model.safetensors")
    a, b, c = tokens_for(raw, 50, 1), tokens_for(raw, 20, 2), tokens_for(raw, 64, 3)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[:7], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [12]}, {"id": "a", "tokens": a[31:], "want": [18]}], "end": ["a", "b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": c[:62], "want": [61]}], "end": []},
        {"step": 4, "entries": [{"id": "c", "tokens": c[62:], "want": [0, 1]}], "end": ["c"]},
    ]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        stdout = io.StringIO()
        code = main(["--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "128",
                     "--live-requests", "2"], stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"),
                    stdout=stdout)
        assert code == 0 and stdout.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "4"]
        la, lb, lc = (plain_logits(raw, tensors, t) for t in (a, b, c))
        want = {0: la[[0, 29]], 1: la[[30]], 2: torch.stack([lb[19], la[49]]), 3: lc[[61]], 4: lc[[62, 63]]}
        for step, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), raw["vocab"]))
            assert_rows_close(got, rows, 2 * TOL[dtype], f"{dtype} step {step}")


def test_command_line_writes_and_generates(tmp_path):
    """bin/generate: a random-weights folder from a config.json, then greedy tokens from it that equal the
    plain implementation's on the folder's own tensors."""
    import subprocess
    import sys
    from pathlib import Path

    from mini_gpt_inference_b200.weights import load_file

    root = Path(__file__).resolve().parent.parent
    raw = config("D")
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(raw))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--random-weights", "3", "--config", str(cfg_path),
                           "--write-model", str(folder), "--weights-dtype", "bfloat16"], capture_output=True, text=True)
    assert made.returncode == 0, made.stderr[-2000:]
    prompt = tokens_for(raw, 9, 5)
    run = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--model", str(folder), "--dtype", "float32",
                          "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "8", "--temperature", "0"],
                         capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
    out = json.loads(run.stdout.strip().splitlines()[-1])
    assert out["token_ids"] == plain_greedy(raw, load_file(folder / "model.safetensors"), prompt, 8)


class _AttentionContext:
    """The few fields of a step's context that the attention kernels read."""

    def __init__(self, tables, token_request, positions, q_len, decode_only):
        to = lambda rows: torch.tensor(rows, dtype=torch.int32, device="cuda:0")
        self.block_tables = [to(tables)]
        self.token_request, self.positions = to(token_request), to(positions)
        self.req_q_start = to([sum(q_len[:i]) for i in range(len(q_len))])
        self.req_q_len = to(q_len)
        self.host_q_len = list(q_len)
        self.decode_only = decode_only
        self.max_ctx_after = max(positions) + 1


@pytest.mark.parametrize("path", ["tiles", "ranges"])
@pytest.mark.parametrize("heads,d,dv,pt", [(5, 160, 128, 16), (16, 576, 512, 64), (40, 80, 48, 8), (3, 520, 264, 32)])
def test_attention_over_wide_rows_that_hold_their_values(path, heads, d, dv, pt):
    """One key row per token, shared by all heads, whose first features are the values, wider than the warp-tile
    kernel's registers take: portions of two requests, and single tokens over ranges of keys.  Every query is made
    to favour one key far back (the first, one at a page's last row, one in the middle), among hundreds."""
    import math

    from mini_gpt_inference_b200.cache.storage import PagedKVView
    from mini_gpt_inference_b200.kernels.ops import default_ops

    ops = default_ops("cuda:0")
    gen = torch.Generator().manual_seed(heads * d + dv)
    lengths = [333, 70]
    n_pages = [-(-n // pt) for n in lengths]
    order = torch.randperm(sum(n_pages) + 3, generator=gen).tolist()
    tables = [order[:n_pages[0]] + [0] * (max(n_pages) - n_pages[0]), order[n_pages[0]: sum(n_pages)] + [0] * (max(n_pages) - n_pages[1])]
    rows_all = [torch.randn(n, d, generator=gen).bfloat16().float() for n in lengths]
    if path == "tiles":
        rows = [(0, p) for p in range(300, 333)] + [(1, p) for p in range(0, 70)]
        q_len = [33, 70]
    else:
        rows = [(0, 332), (1, 69)]
        q_len = [1, 1]
    targets = [[0, pt * max(1, p // pt) - 1 if p >= pt else 0, p // 2][i % 3] for i, (_, p) in enumerate(rows)]
    for (r, _), j in zip(rows, targets):
        rows_all[r][j, dv:] = 3.0 * torch.sign(rows_all[r][j, dv:])       # a long key part outside the values
    pages = torch.full((len(order), 1, pt, d), float("nan"))
    for r, n in enumerate(lengths):
        for j in range(n):
            pages[tables[r][j // pt], 0, j % pt] = rows_all[r][j]
    n = len(rows)
    q = 0.3 * torch.randn(n, heads, d, generator=gen)
    for i, ((r, _), j) in enumerate(zip(rows, targets)):
        q[i] += 0.3 * rows_all[r][j]
    q_rows = torch.cat([q.reshape(n, -1), torch.randn(n, 16, generator=gen)], dim=1).bfloat16()
    gate = torch.randn(n, heads * dv, generator=gen).bfloat16()
    sinks = torch.randn(heads, generator=gen) + 2.0
    scale = 1.0 / math.sqrt(d)
    k_dev = pages.to(device="cuda:0", dtype=torch.bfloat16)
    cache = PagedKVView(k_dev, k_dev, 0, pt, None, False, values_in_keys=True)
    ctx = _AttentionContext(tables, [r for r, _ in rows], [p for _, p in rows], q_len, path == "ranges")
    launches = ops.launches
    got = ops.paged_attention_general(q_rows.cuda(), heads, 1, d, dv, scale, cache, ctx, gate=gate.cuda(), sinks=sinks.cuda())
    assert ops.launches - launches == (1 if path == "tiles" else 2)       # tensor-core kernels, not the general one
    ops.use_mma_attention = False
    try:
        general = ops.paged_attention_general(q_rows.cuda(), heads, 1, d, dv, scale, cache, ctx, gate=gate.cuda(), sinks=sinks.cuda())
    finally:
        ops.use_mma_attention = True
    want = torch.empty(n, heads, dv, dtype=torch.float64)
    peak = []
    for i, (r, p) in enumerate(rows):
        keys = rows_all[r][: p + 1].double()
        for h in range(heads):
            s = (keys @ q_rows[i, h * d: (h + 1) * d].double()) * scale
            top = max(float(s.max()), float(sinks[h]))
            w = torch.exp(s - top)
            w = w / (w.sum() + math.exp(float(sinks[h]) - top))
            peak.append(float(w[targets[i]]))
            want[i, h] = w @ keys[:, :dv]
    assert min(peak) > 0.4                                   # the chosen key does carry the weight
    want = want.view(n, -1) * torch.sigmoid(gate.double())
    assert torch.allclose(general.double().cpu(), want, atol=3e-2, rtol=3e-2)
    assert torch.allclose(got.double().cpu(), want, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens", [1, 5, 16, 150])
@pytest.mark.parametrize("heads,n_in,n_out", [(3, 24, 40), (5, 72, 136), (2, 200, 16), (4, 20, 12)])
def test_one_small_matrix_per_head(dtype, tokens, heads, n_in, n_out):
    """Both layouts of the heads' matrices (a head's rows as its outputs, or as its inputs), inputs at an offset
    inside wider rows, outputs into a wider buffer, with and without the gate; few tokens and many (bfloat16 steps
    of 16 tokens and more run on the tensor cores)."""
    from mini_gpt_inference_b200.kernels.ops import default_ops

    ops = default_ops("cuda:0")
    t = torch.float32 if dtype == "float32" else torch.bfloat16
    gen = torch.Generator().manual_seed(tokens * heads + n_in)
    x_head = n_in + 8
    x = torch.randn(tokens, 16 + heads * x_head, generator=gen).to(t)
    gate = torch.randn(tokens, heads * n_out, generator=gen).to(t)
    xs = torch.stack([x[:, 16 + h * x_head: 16 + h * x_head + n_in] for h in range(heads)], 1).double()     # [n, h, i]
    tol = 1e-5 if dtype == "float32" else 2e-2
    for rows_are_inputs in (False, True):
        w = (torch.randn(heads * (n_in if rows_are_inputs else n_out), n_out if rows_are_inputs else n_in, generator=gen)
             / n_in ** 0.5).to(t)
        per_head = w.double().view(heads, n_in, n_out) if rows_are_inputs else w.double().view(heads, n_out, n_in).transpose(1, 2)
        want = torch.einsum("nhi,hij->nhj", xs, per_head)
        got = ops.head_linear(x.cuda(), 16, x_head, w.cuda(), rows_are_inputs, heads, n_in, n_out)
        assert torch.allclose(got.double().cpu().view(tokens, heads, n_out), want, atol=tol, rtol=tol)
        got = ops.head_linear(x.cuda(), 16, x_head, w.cuda(), rows_are_inputs, heads, n_in, n_out, gate=gate.cuda())
        gated = want * torch.sigmoid(gate.double()).view(tokens, heads, n_out)
        assert torch.allclose(got.double().cpu().view(tokens, heads, n_out), gated, atol=tol, rtol=tol)
        wide = torch.full((tokens, 8 + heads * (n_out + 4)), 7.0, dtype=t, device="cuda:0")
        ops.head_linear(x.cuda(), 16, x_head, w.cuda(), rows_are_inputs, heads, n_in, n_out, out=wide, out_off=8, out_head=n_out + 4)
        back = wide.double().cpu()
        for h in range(heads):
            lo = 8 + h * (n_out + 4)
            assert torch.allclose(back[:, lo: lo + n_out], want[:, h], atol=tol, rtol=tol)
            assert bool((back[:, lo + n_out: lo + n_out + 4] == 7.0).all())       # nothing written between the heads


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed):
    """Other sizes, head counts, layer orders, windows and constants than the fixed cases: whole prompts, and the
    same prompt in portions of changing size with its last 40 tokens one by one, in both dtypes."""
    import random

    from nukodra_cases import random_config

    rng = random.Random(seed)
    raw = random_config(rng)
    pt = rng.choice([16, 64])
    n = rng.choice([150, 333, 420])
    tokens = tokens_for(raw, n, seed)
    for dtype in ("float32", "bfloat16"):
        from mini_gpt_inference_b200.kernels.ops import default_ops

        tensors = random_weights(raw, seed, sharp=2.0 if dtype == "float32" else 1.0, as_bfloat16=dtype == "bfloat16")
        loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
        runner = make_runner(loaded, default_ops("cuda:0"), pt, 64, 4)
        want = plain_logits(raw, tensors, tokens)
        whole = runner.step([StepEntry("w", tokens, list(range(n)))])
        runner.finish("w")
        cuts, at = [], 0
        while at < n - 40:
            cuts.append(min(rng.choice([2, 3, 17, 64, 65, 130]), n - 40 - at))
            at += cuts[-1]
        cuts += [1] * (n - at)
        rows, at = [], 0
        for c in cuts:
            rows.append(runner.step([StepEntry("c", tokens[at: at + c], list(range(c)))]))
            at += c
        runner.finish("c")
        for what, got in (("whole", whole), ("in portions", torch.cat(rows))):
            assert_rows_close(got, want, TOL[dtype], f"seed {seed} {dtype} {what}", outliers=0.03 if dtype == "bfloat16" else 0.0)
        runner.manager.check()
        assert runner.manager.stats()["allocated_blocks"] == 0
