"""Lunelorn on the GPU against the plain implementation: the new kernels alone, the step function under every way of
cutting requests into steps, batches, pages and slots used again, then generation through the entry point."""

from __future__ import annotations

import io
import itertools
import json
import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_lunelorn as plain
from lunelorn_cases import (PAGE_TOKENS, all_experts, assert_rows_close, config, plain_greedy, plain_logits, random_config,
                            random_weights, relative_error, rounding_spread, tokens_for)

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, LunelornConfig, SamplingParams
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

# Largest |engine - plain| on a row of logits, over the row's own spread.  32-bit: rounding of sums.
# bfloat16: both sides use the same weights; activations are rounded to 8 bits between kernels.  A
# lost key, state, decay, bonus or norm shows as 0.3 and more.
TOL = {"float32": 3e-4, "bfloat16": 1e-1}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CASES = [(w, d) for w in "ABCDE" for d in ("float32", "bfloat16")]
IDS = [f"{w}-{d}" for w, d in CASES]


@pytest.fixture(scope="module")
def ops():
    from mini_gpt_inference_b200.kernels.ops import default_ops

    return default_ops("cuda:0")


def dev(t, dtype=None):
    return t.to(device="cuda:0", dtype=dtype or t.dtype).contiguous()


def ints(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda:0")


def batch(q_len, ctx_before, slots, tokens=None):
    """The few fields of a step's context that the recurrent kernels read."""
    starts = [sum(q_len[:i]) for i in range(len(q_len))]
    n = sum(q_len)
    request = [r for r, m in enumerate(q_len) for _ in range(m)]
    positions = [ctx_before[r] + i for r, m in enumerate(q_len) for i in range(m)]
    return SimpleNamespace(req_q_start=ints(starts), req_q_len=ints(q_len), req_ctx_before=ints(ctx_before),
                           req_state_slot=ints(slots), token_request=ints(request), positions=ints(positions),
                           token_ids=ints(tokens if tokens is not None else [0] * n), num_requests=len(q_len),
                           token_source=None, fed_ids=None, extra={}, max_q_len=max(q_len))


# ---- the new kernels alone ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,width", [(1, 40), (5, 192), (37, 100), (130, 1024)])
def test_norm_behind_a_sublayer_and_the_sums_into_the_stream(ops, rows, width):
    gen = torch.Generator().manual_seed(rows + width)
    x, a, b = (torch.randn(rows, width, generator=gen) for _ in range(3))
    w = 1 + 0.3 * torch.randn(width, generator=gen)
    got = ops.rmsnorm_add(dev(x), dev(a * 50.0), dev(w), 1e-3)                     # the norm takes the size away
    assert torch.allclose(got.double().cpu(), x.double() + plain.rms_norm(a.double() * 50.0, w.double(), 1e-3), atol=1e-5)
    got = ops.rmsnorm_add(dev(x), dev(a), dev(w), 1e-6, other32=dev(b), scale=1.2, other_scale=-0.5)
    assert torch.allclose(got.double().cpu(), x.double() + plain.rms_norm(1.2 * a.double() - 0.5 * b.double(), w.double(), 1e-6), atol=1e-5)
    assert torch.allclose(ops.scaled_sum_(dev(x), dev(a), 0.7, dev(b), 2.0).cpu(), x + 0.7 * a + 2.0 * b, atol=1e-5)
    # with `clear` the inputs come back as zeros, the results are the same
    xa, ya, yb = dev(x), dev(a), dev(b)
    assert torch.equal(ops.rmsnorm_add(xa, ya, dev(w), 1e-6, other32=yb, scale=1.2, other_scale=-0.5, clear=True), got)
    assert not bool(ya.any()) and not bool(yb.any())
    ya, yb = dev(a), dev(b)
    assert torch.allclose(ops.scaled_sum_(dev(x), ya, 0.7, yb, 2.0, clear=True).cpu(), x + 0.7 * a + 2.0 * b, atol=1e-5)
    assert not bool(ya.any()) and not bool(yb.any())
    assert torch.allclose(ops.add_rows(dev(x), dev(a), dev(w)).cpu(), x + a + w, atol=1e-6)
    assert torch.allclose(ops.add_rows(dev(x), None, dev(w)).cpu(), x + w, atol=1e-6)
    assert torch.allclose(ops.softcap_(dev(10 * x), 7.0).cpu(), 7.0 * torch.tanh(10 * x / 7.0), atol=1e-5)
    assert bool((ops.zeros32(rows, width) == 0).all())
    assert torch.equal(ops.cast(dev(x), torch.bfloat16).cpu(), x.to(torch.bfloat16))
    assert torch.allclose(ops.tanh_cast(dev(x), torch.float32).cpu(), torch.tanh(x), atol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,parts", [(24, 4), (5, 1), (130, 3)])
def test_gated_slice_of_the_token_table(ops, dtype, dim, parts):
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(dim)
    vocab, n = 50, 9
    table = torch.randn(vocab, parts * dim, generator=gen).to(t)
    gate = 2 * torch.randn(n, dim, generator=gen)
    tokens = torch.randint(0, vocab, (n,), generator=gen).tolist()
    ctx = batch([n - 1, 1], [0, 3], [0, 1], tokens)
    ctx.positions[3] = -1                                                            # a padding row gives zeros
    for index in range(parts):
        got = ops.token_gate(ctx, dev(gate), dev(table), index * dim, t).float().cpu()
        want = plain.gelu_tanh(gate.double()) * table.double()[tokens][:, index * dim: (index + 1) * dim]
        want[3] = 0
        assert torch.allclose(got.double(), want, atol=1e-5 if dtype == "float32" else 3e-2, rtol=1e-2)
    # tokens that the step before sampled, still on the device
    ctx.token_source, ctx.fed_ids = ints([-1, 0, -1, -1, 2, -1, -1, -1, 1]), ints([7, 8, 9])
    fed = list(tokens)
    fed[1], fed[4], fed[8] = 7, 9, 8
    got = ops.token_gate(ctx, dev(gate), dev(table), 0, t).float().cpu()
    want = plain.gelu_tanh(gate.double()) * table.double()[fed][:, :dim]
    want[3] = 0
    assert torch.allclose(got.double(), want, atol=1e-5 if dtype == "float32" else 3e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,dim,index,tokens", [(64, 12, 1, 5), (160, 40, 3, 16), (1024, 128, 0, 8), (96, 8, 2, 40)])
def test_token_input_of_a_layer(ops, dtype, width, dim, index, tokens):
    """The gate's projection of the stream itself, the token's slice, the projection back and the norm, against the
    plain function; a padding row stays as it is."""
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width + dim)
    vocab = 40
    w = {"side.embed": torch.randn(vocab, 4 * dim, generator=gen), "gate": torch.randn(dim, width, generator=gen) / math.sqrt(width),
         "proj": torch.randn(width, dim, generator=gen) / math.sqrt(dim), "norm": 1 + 0.3 * torch.randn(width, generator=gen)}
    w = {k: v.to(t).float() for k, v in w.items()}
    x = 3 * torch.randn(tokens, width, generator=gen)
    ids = torch.randint(0, vocab, (tokens,), generator=gen)
    ctx = batch([tokens], [0], [0], ids.tolist())
    ctx.positions[2] = -1
    want = x.double() + plain.token_side_input(x.to(t).double(), ids, {k: v.double() for k, v in w.items()}, "", index, dim, 1e-5)
    got = ops.token_side_residual(ctx, dev(x), dev(w["gate"], t), dev(w["proj"], t), dev(w["norm"]), dev(w["side.embed"], t),
                                  index * dim, 1e-5, t)
    live = [i for i in range(tokens) if i != 2]
    assert torch.allclose(got.double().cpu()[live], want[live], atol=2e-5 if dtype == "float32" else 4e-2, rtol=1e-2)
    assert torch.equal(got.cpu()[2], x[2])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [72, 70, 1024])
def test_blend_with_the_token_before_across_steps(ops, dtype, width):
    """Two requests in unequal portions: the row before a portion's first row comes from the state slot, zeros for a
    sequence's first token; slots start as NaN.  (Widths that the 16-byte form takes, and one that it does not.)"""
    t = DTYPES[dtype]
    mixes = 5
    gen = torch.Generator().manual_seed(1)
    mu = torch.rand(mixes, width, generator=gen)
    seqs = [torch.randn(13, width, generator=gen).to(t), torch.randn(6, width, generator=gen).to(t)]
    state = dev(torch.full((3, width + 10), float("nan")))
    pos, got = [0, 0], [[], []]
    for portions in ([5, 1], [1, 2], [7, 3]):
        live = [r for r in (0, 1) if portions[r]]
        rows = torch.cat([seqs[r][pos[r]: pos[r] + portions[r]] for r in live])
        ctx = batch([portions[r] for r in live], [pos[r] for r in live], [2 - r for r in live])
        out = ops.token_shift_mix(ctx, dev(rows), dev(mu), state)
        ops.conv_state_update(ctx, dev(rows), 0, width, 2, state)
        at = 0
        for r in live:
            got[r].append(out[:, at: at + portions[r]].float().cpu())
            at += portions[r]
            pos[r] += portions[r]
    for r in (0, 1):
        x = seqs[r].double()
        before = torch.cat([torch.zeros(1, width, dtype=torch.float64), x[:-1]])
        want = x[None] + (before - x)[None] * mu.double()[:, None, :]
        assert torch.allclose(torch.cat(got[r], dim=1).double(), want, atol=1e-6 if dtype == "float32" else 4e-2)
    assert torch.equal(state[2, :width].cpu(), seqs[0][-1].float()) and torch.equal(state[1, :width].cpu(), seqs[1][-1].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [33, 256, 700])
def test_gated_recurrence_in_portions(ops, dtype, width):
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width)
    lengths = [300, 9]      # (bfloat16: the portion of 200 runs with the warps sharing its tokens, the others token by token)
    pre = [torch.randn(n, 3 * width + 4, generator=gen) * 3.0 for n in lengths]        # gates that open and shut
    offset = 6
    state = dev(torch.full((2, width + offset), float("nan")))
    pos, got = [0, 0], [[], []]
    for portions in ([200, 2], [1, 1], [2, 6], [97, 0]):
        live = [r for r in (0, 1) if portions[r]]
        rows = torch.cat([pre[r][pos[r]: pos[r] + portions[r]] for r in live])
        ctx = batch([portions[r] for r in live], [pos[r] for r in live], [r for r in live])
        out = ops.gated_recurrence(ctx, dev(rows), 4, 4 + width, 4 + 2 * width, width, state, offset, t)
        at = 0
        for r in live:
            got[r].append(out[at: at + portions[r]].float().cpu())
            at += portions[r]
            pos[r] += portions[r]
    for r in (0, 1):
        p = pre[r].double()
        z, u, g = torch.sigmoid(p[:, 4: 4 + width]), p[:, 4 + width: 4 + 2 * width], p[:, 4 + 2 * width: 4 + 3 * width]
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        s, rows = torch.zeros(width, dtype=torch.float64), []
        for i in range(lengths[r]):
            s = (1 - z[i]) * s + z[i] * cand[i]
            rows.append(s * g[i] * torch.sigmoid(g[i]))
        assert torch.allclose(torch.cat(got[r]).double(), torch.stack(rows), atol=2e-5 if dtype == "float32" else 5e-2, rtol=1e-2)
        assert torch.allclose(state[r, offset:].double().cpu(), s, atol=2e-5)


def _memory_reference(mode, q, k, v, gates, consts):
    """o [T, H, dv] in float64 from q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=torch.float64)
    out = []
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        if mode == "retention":
            S = consts[:, None, None] * S + kv * d ** -0.5
            out.append(torch.einsum("hde,hd->he", S, q[t]))
        else:
            out.append(torch.einsum("hde,hd->he", S + consts.view(H, d, 1) * kv, q[t]))
            S = torch.exp(-torch.exp(gates[t].view(H, d)))[:, :, None] * S + kv
    return torch.stack(out)


@pytest.mark.parametrize("mode", ["retention", "wkv"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,d,dv", [(3, 16, 24), (2, 64, 64), (1, 72, 72), (2, 128, 40)])
def test_fixed_decays_and_reads_before_the_update_through_both_scans(ops, mode, dtype, heads, d, dv):
    """Three unequal requests: whole, in portions down to two tokens, and token by token, through the token-by-token
    scan and (bfloat16, long portions) the chunked kernels, from NaN-filled slots.  A token far back owns the read-out:
    its key and the last query are made large and aligned, its decays are (nearly) one."""
    if mode == "wkv":
        dv = d
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(heads * d + dv)
    lengths = [210, 70, 3]
    planes = mode == "wkv"
    seqs = []
    for n in lengths:
        q, k = torch.randn(n, heads, d, generator=gen), torch.randn(n, heads, d, generator=gen)
        v = torch.randn(n, heads, dv, generator=gen)
        gates = torch.randn(n, heads * d, generator=gen) - 2.0
        if n > 100:                                                                   # the far token
            k[5] *= 4.0
            q[-1] = k[5] * 0.5
            gates[6:] -= 4.0
        seqs.append(tuple(x.to(t).float() for x in (q, k, v)) + (gates,))
    consts = (1 - 2.0 ** -torch.arange(8, 8 + heads, dtype=torch.float64)) if mode == "retention" else \
        0.5 * torch.randn(heads * d, generator=gen).double()
    consts_dev = dev(consts.float())
    width = heads * (2 * d + dv)

    def run(portion_lists, chunked):
        state = dev(torch.full((4, heads * dv * d + 7), float("nan")))
        pos, got = [0] * 3, [[] for _ in lengths]
        ops.use_chunked_memory = chunked
        for portions in portion_lists:
            live = [r for r in range(3) if portions[r]]
            sl = [slice(pos[r], pos[r] + portions[r]) for r in live]
            n = sum(portions)
            cat = lambda i: torch.cat([seqs[r][i][s] for r, s in zip(live, sl)])
            q, k, v, gates = cat(0).reshape(n, -1), cat(1).reshape(n, -1), cat(2).reshape(n, -1), cat(3)
            if planes:
                proj = dev(torch.stack([q, k, v]), t)
                offs = (0, n * heads * d, 2 * n * heads * d)
            else:
                proj = dev(torch.cat([q, k, v], dim=1), t)
                offs = (0, heads * d, 2 * heads * d)
            ctx = batch([portions[r] for r in live], [pos[r] for r in live], [3 - r for r in live])
            if chunked:
                plan = SimpleNamespace(arrays={}, signature=[])
                ops.plan_memory_chunks(SimpleNamespace(q_len=[portions[r] for r in live], act_dtype=t), plan, d, dv, False)
                ctx.extra = {name: ints(a.tolist()).reshape(a.shape) for name, a in plan.arrays.items()}
            out, _ = ops.matrix_memory_scan(ctx, mode, proj, *offs, heads, d, dv, None if mode == "retention" else dev(gates),
                                            0.0, state, state_offset=7, head_consts=consts_dev)
            at = 0
            for r in live:
                got[r].append(out[at: at + portions[r]].cpu())
                at += portions[r]
                pos[r] += portions[r]
        ops.use_chunked_memory = True
        return [torch.cat(g) for g in got]

    want = [_memory_reference(mode, s[0].double(), s[1].double(), s[2].double(), s[3].double(), consts).reshape(len(s[0]), -1)
            for s in seqs]
    # the far token is most of what the last query reads
    k_without = seqs[0][1].double().clone()
    k_without[5] = 0
    without = _memory_reference(mode, seqs[0][0].double(), k_without, seqs[0][2].double(), seqs[0][3].double(), consts)
    assert float((without[-1].reshape(-1) - want[0][-1]).abs().max()) > 0.3 * float(want[0][-1].abs().max())
    whole = [lengths]
    cut = [[100, 33, 1], [2, 2, 2], [64, 35, 0], [44, 0, 0]]
    single = [[1 if i < n else 0 for n in lengths] for i in range(40)]
    for name, lists, chunked in (("whole", whole, False), ("portions", cut, False), ("whole in chunks", whole, True),
                                 ("portions in chunks", cut, True)):
        got = run(lists, chunked and dtype == "bfloat16")
        for r in range(3):
            scale = want[r].abs().max()
            assert float((got[r].double() - want[r]).abs().max() / scale) < 2e-5, (name, r)
    got = run(single, False)
    for r in range(3):
        m = min(40, lengths[r])
        assert float((got[r].double() - want[r][:m]).abs().max() / want[r].abs().max()) < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,d,dv,rot", [(4, 2, 16, 8, 8), (3, 3, 24, 24, 24), (2, 1, 40, 64, 0), (4, 1, 64, 64, 16)])
def test_unit_values_turned_with_their_position_and_turned_back(ops, dtype, heads, kv_heads, d, dv, rot):
    from mini_gpt_inference_b200.cache.storage import PagedKVView

    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(heads * d + rot)
    positions = torch.tensor([0, 1, 2, 77, 5000, 70001, -1], dtype=torch.int32)
    n = positions.numel()
    q_off, k_off, v_off = 8, 8 + heads * d, 8 + (heads + kv_heads) * d
    proj = torch.randn(n, v_off + kv_heads * dv, generator=gen).to(t)
    base, eps = 500.0, 1e-3
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float() if rot else None
    v_freq = torch.tensor([base ** (-2.0 * m / dv) for m in range(dv // 2)], dtype=torch.float64).float()
    pt = 4
    cache = PagedKVView(dev(torch.full((5, kv_heads, pt, d), float("nan")), t), dev(torch.full((5, kv_heads, pt, dv), float("nan")), t),
                        0, pt, None, True)
    slots = torch.tensor([3, 4, 17, 0, 9, 12, -1], dtype=torch.int32)
    rows = dev(proj.clone())
    ops.qk_norm_rotary(rows, heads, kv_heads, d, dv, q_off, k_off, v_off, False, eps, rot, dev(freq) if rot else None, cache,
                       dev(slots), dev(positions), v_unit_norm=True, v_freq=dev(v_freq))
    p64 = proj.double()
    live = positions >= 0
    pos = positions[live].long()
    q = plain.rotate(p64[live, q_off: k_off].view(-1, heads, d), pos, rot, base)
    k = plain.rotate(p64[live, k_off: v_off].view(-1, kv_heads, d), pos, rot, base)
    v = plain.rotate(plain.rms_norm(p64[live, v_off:].view(-1, kv_heads, dv), None, eps), pos, dv, base)
    # (a 32-bit angle at position p is off by up to p * 2^-24 of a turn's argument; bfloat16 rounds the results)
    tol = (2e-5 + 2e-7 * pos.double() if dtype == "float32" else torch.full((len(pos),), 6e-2, dtype=torch.float64))

    def close(got, want):
        got, want = got.double().cpu().reshape(len(pos), -1), want.reshape(len(pos), -1)
        return bool(((got - want).abs().amax(-1) <= tol * (1 + want.abs().amax(-1))).all())
    assert close(rows[live, q_off: k_off], q)
    assert torch.equal(rows[~live].cpu(), proj[~live])
    s = slots[live].long()
    assert close(cache.k_pages[s // pt, :, s % pt], k)
    assert close(cache.v_pages[s // pt, :, s % pt], v)
    # turned back by the same positions, the unit values come out again
    out = dev(v.reshape(len(pos), -1).float(), t)
    ops.rotate_heads(out, kv_heads, dv, dev(v_freq), dev(positions[live]), -1.0)
    assert close(out, plain.rms_norm(p64[live, v_off:].view(-1, kv_heads, dv), None, eps))


# ---- the step function ---------------------------------------------------------------------------------------------
def setup(which, dtype, num_pages=64, seed=3, max_requests=4, raw=None, page_tokens=None, sharp=None):
    from mini_gpt_inference_b200.kernels.ops import default_ops

    raw = raw or config(which, every_expert=dtype == "bfloat16")      # (see lunelorn_cases.all_experts)
    # (sharp softmaxes in 32-bit, where nothing but the order of sums differs; in bfloat16 they would magnify
    # the rounding of queries and keys)
    sharp = sharp if sharp is not None else (3.0 if dtype == "float32" else 1.0)
    tensors = random_weights(raw, seed, sharp=sharp, as_bfloat16=dtype == "bfloat16", steady=dtype == "bfloat16")
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    runner = make_runner(loaded, default_ops("cuda:0"), page_tokens or PAGE_TOKENS[which], num_pages, max_requests)
    return raw, tensors, runner, (TOL[dtype], 0.03 if dtype == "bfloat16" else 0.0, dtype)


def expect(raw, tensors, tokens, tol):
    """The plain logits of a sequence and the keywords of the comparison with them (see ``rounding_spread``)."""
    kw = {"outliers": tol[1]}
    if tol[2] == "bfloat16":
        kw["slack"] = rounding_spread(raw, tensors, tokens)
    return plain_logits(raw, tensors, tokens), kw


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_whole_prompts(which, dtype):
    raw, tensors, runner, tol = setup(which, dtype, num_pages=100)
    pt = PAGE_TOKENS[which]
    for length, seed in [(150, 1), (37, 2), (1, 3), (2, 4), (pt + 1, 5), (pt, 6), (190, 7)]:
        tokens = tokens_for(raw, length, seed)
        got = runner.step([StepEntry("r", tokens, list(range(length)))])
        runner.finish("r")
        assert got.shape == (length, raw["vocab"]) and got.dtype == torch.float32
        want, kw = expect(raw, tensors, tokens, tol)
        assert_rows_close(got, want, tol[0], f"whole prompt of {length}", **kw)
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_prefill_then_single_tokens(which, dtype):
    """A short prompt, then a long run of single tokens (replayed from a CUDA graph), and the same sequence token by
    token from the very first token."""
    raw, tensors, runner, tol = setup(which, dtype)
    tokens = tokens_for(raw, 150, 7)
    want, kw = expect(raw, tensors, tokens, tol)
    outs = [runner.step([StepEntry("r", tokens[:9], list(range(9)))])]
    outs += [runner.step([StepEntry("r", tokens[t: t + 1], [0])]) for t in range(9, 150)]
    assert_rows_close(torch.cat(outs), want, tol[0], "prefill then single tokens", **kw)
    assert runner.graph_replays > 100
    one_by_one = torch.cat([runner.step([StepEntry("s", tokens[t: t + 1], [0])]) for t in range(40)])
    assert_rows_close(one_by_one, want[:40], tol[0], "single tokens from the first",
                      **{k: (v[:40] if k == "slack" else v) for k, v in kw.items()})
    if dtype == "float32":
        # in 32-bit the cut into steps changes no bit
        assert torch.equal(one_by_one, torch.cat(outs)[:40])


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_portions_of_changing_size(which, dtype):
    raw, tensors, runner, tol = setup(which, dtype)
    tokens = tokens_for(raw, 171, 8)
    want, kw = expect(raw, tensors, tokens, tol)
    sizes = itertools.cycle([13, 7, 2, 5, 2, 1, 3, 16, 2, 9, 70])
    outs, pos = [], 0
    while pos < len(tokens):
        n = min(next(sizes), len(tokens) - pos)
        outs.append(runner.step([StepEntry("r", tokens[pos: pos + n], list(range(n)))]))
        pos += n
    assert_rows_close(torch.cat(outs), want, tol[0], "portions of changing size", **kw)
    if dtype == "float32":
        runner.finish("r")
        assert torch.equal(torch.cat(outs), runner.step([StepEntry("r", tokens, list(range(len(tokens))))]))


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
    want = {rid: expect(raw, tensors, toks, tol) for rid, toks in reqs.items()}
    got = {rid: [] for rid in reqs}
    waiting, live = list(reqs), {}
    sizes = itertools.cycle([5, 1, 2, 11, 1, 1, 7, 3, 1, 2, 1, 1, 40])
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
        assert_rows_close(torch.cat(got[rid]), want[rid][0], tol[0], f"request {rid} in mixed batches", **want[rid][1])
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
@pytest.mark.parametrize("far", [0, 15, 16, 31, 32])
def test_a_key_far_back_at_a_pages_border(dtype, far):
    """One attention layer alone; the last query is made to lean on the key at position `far` (the first token, a
    page's last row, a page's first row) among hundreds: the key matrix is the first query head's, and that position
    holds the last token's own id, so the two of them outweigh all others.  Whole, and with the last tokens decoded one by one."""
    raw = {"architecture": "Lunelorn", "vocab": 50, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        {"type": "parallel", "mlp": None, "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 1.0,
                                                                "rot": {"dims": 0, "base": 100.0}},
                                                    "right": {"width": 64}, "left_scale": 1.0, "right_scale": 0.01}}]}
    tensors = random_weights(raw, 5, as_bfloat16=True)
    tensors["l0.mix.left.k"] = tensors["l0.mix.left.q"][:32].clone()                  # q . k = |W h|^2 for a token with itself
    tokens = tokens_for(raw, 300, 3)
    tokens = [t if t != 7 else 8 for t in tokens]
    tokens[far] = tokens[-1] = 7                                                       # the same token twice: aligned
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    from mini_gpt_inference_b200.kernels.ops import default_ops

    runner = make_runner(loaded, default_ops("cuda:0"), 16, 40, 2)
    want = plain_logits(raw, tensors, tokens)
    gone = plain_logits(raw, tensors, tokens[:far] + [9] + tokens[far + 1:])
    assert float(relative_error(gone[-1:], want[-1:])) > 0.3                           # the far key matters
    got = runner.step([StepEntry("w", tokens, [299])])
    assert_rows_close(got, want[-1:], TOL[dtype], "whole")
    outs = [runner.step([StepEntry("d", tokens[:290], [289])])]
    outs += [runner.step([StepEntry("d", tokens[t: t + 1], [0])]) for t in range(290, 300)]
    assert_rows_close(torch.cat(outs), want[289:], TOL[dtype], "decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_and_long_decoding(dtype):
    raw, tensors, runner, tol = setup("B", dtype, num_pages=40)
    tokens = tokens_for(raw, 400, 17)
    want, kw = expect(raw, tensors, tokens, tol)
    outs = [runner.step([StepEntry("r", tokens[:300], list(range(300)))])]
    outs += [runner.step([StepEntry("r", tokens[t: t + 1], [0])]) for t in range(300, 400)]
    assert_rows_close(torch.cat(outs), want, tol[0], "long prompt, long decoding", **kw)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed):
    rng = random.Random(seed)
    raw = random_config(rng)
    pt = rng.choice([16, 64])
    for dtype in ("float32", "bfloat16"):
        if dtype == "bfloat16":
            raw = all_experts(raw)
        _, tensors, runner, tol = setup(None, dtype, num_pages=600 // pt + 8, seed=seed, raw=raw, page_tokens=pt, sharp=1.0)
        tokens = tokens_for(raw, 200, seed)
        want, kw = expect(raw, tensors, tokens, tol)
        whole = runner.step([StepEntry("w", tokens, list(range(200)))])
        assert_rows_close(whole, want, tol[0], f"seed {seed} {dtype} whole", **kw)
        sizes = itertools.cycle([70, 3, 2, 33, 1, 64])
        outs, pos = [], 0
        while pos < 170:
            n = min(next(sizes), 170 - pos)
            outs.append(runner.step([StepEntry("p", tokens[pos: pos + n], list(range(n)))]))
            pos += n
        outs += [runner.step([StepEntry("p", tokens[t: t + 1], [0])]) for t in range(170, 200)]
        assert_rows_close(torch.cat(outs), want, tol[0], f"seed {seed} {dtype} portions", **kw)
        if dtype == "float32":
            assert torch.equal(torch.cat(outs), whole)


# ---- generation through the entry point, its scheduler and sampler ---------------------------------
@pytest.mark.parametrize("which", "ABC")
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(which, dtype):
    raw = config(which, every_expert=dtype == "bfloat16")
    tensors = random_weights(raw, 11, as_bfloat16=dtype == "bfloat16", steady=dtype == "bfloat16")
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype=dtype, block_size=PAGE_TOKENS[which], num_blocks=48,
                                            max_batch_size=3, max_num_batched_tokens=16, max_prefill_chunk=7))
    prompts = [tokens_for(raw, n, 40 + i) for i, n in enumerate([5, 1, 23, 12, 2, 17])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 12 and out["finish_reason"] == "length"
        seq = prompt + out["token_ids"]
        want = plain_logits(raw, tensors, seq[:-1])
        slack = rounding_spread(raw, tensors, seq[:-1]) if dtype == "bfloat16" else torch.zeros(len(seq))
        for i, token in enumerate(out["token_ids"]):
            row, at = want[len(prompt) - 1 + i], len(prompt) - 1 + i
            assert row.max() - row[token] <= 2 * (TOL[dtype] + 3 * float(slack[at])) * row.std(), (i, token, int(row.argmax()))
        if dtype == "float32":
            assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 12)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


def test_preemption_and_recompute_through_the_engine():
    raw = config("C")
    tensors = random_weights(raw, 14)
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
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
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=40, max_batch_size=2))
    prompt = tokens_for(raw, 3, 9)
    out = engine.generate([prompt], SamplingParams(max_tokens=160, temperature=0.0))[0]
    assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 160)


def test_trace_replay(tmp_path):
    """The replay program on a model folder: two requests, portions beside single tokens, a slot and pages
    used again by a third request."""
    from mini_gpt_inference_b200.engine.trace import main
    from mini_gpt_inference_b200.weights.safetensors_io import save_file

    raw = config("A", every_expert=True)
    tensors = random_weights(raw, 13, as_bfloat16=True, steady=True)
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
        sa, sb, sc = (rounding_spread(raw, tensors, t) if dtype == "bfloat16" else torch.zeros(len(t)) for t in (a, b, c))
        want = {0: (la[[0, 29]], sa[[0, 29]]), 1: (la[[30]], sa[[30]]), 2: (torch.stack([lb[19], la[49]]), torch.stack([sb[19], sa[49]])),
                3: (lc[[61]], sc[[61]]), 4: (lc[[62, 63]], sc[[62, 63]])}
        for step, (rows, slack) in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), raw["vocab"]))
            assert_rows_close(got, rows, 2 * TOL[dtype], f"{dtype} step {step}", slack=slack)


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
