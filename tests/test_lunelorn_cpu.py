"""Lunelorn without a GPU: the plain implementation's mechanisms against restatements by hand, the configuration
and the loader, and the model through the step function, the cache manager, the scheduler and the entry point with
the torch test double in place of the CUDA kernel set."""

from __future__ import annotations

import itertools
import json
import math

import pytest
import torch

import plain_lunelorn as pl
from lunelorn_cases import PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits, random_weights, tokens_for
from torch_ops import TorchOps

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, LunelornConfig, SamplingParams
from mini_gpt_inference_b200.cache.spec import FixedStateSpec, PagedKVWithStateSpec
from mini_gpt_inference_b200.config import ConfigError, lookup
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import WeightsError, check_and_bind, load_file, write_random_model

F64 = torch.float64


def _rand(shapes, seed):
    gen = torch.Generator().manual_seed(seed)
    return {k: torch.randn(*s, generator=gen, dtype=F64) for k, s in shapes.items()}


def _unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---- the plain mechanisms against restatements by hand ---------------------------------------------------
def test_retention_is_a_sum_over_the_past_weighed_by_powers_of_the_decay():
    T, c, H, d, dv = 7, 10, 2, 4, 3
    m = {"heads": H, "dim": d, "vdim": dv, "decay": [0.5, 0.9]}
    w = _rand({"q": (H * d, c), "k": (H * d, c), "v": (H * dv, c), "g": (H * dv, c), "o": (c, H * dv)}, 0)
    h = _rand({"h": (T, c)}, 1)["h"]
    got = pl.retention_mixer(h, w, "", m, 1e-5)
    q, k, v = (h @ w["q"].T).view(T, H, d), (h @ w["k"].T).view(T, H, d) / 2.0, (h @ w["v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for a in range(H):
            for j in range(t + 1):
                o[t, a] += m["decay"][a] ** (t - j) * (q[t, a] @ k[j, a]) * v[j, a]
    g = h @ w["g"].T
    want = (_unit(o, 1e-5).reshape(T, -1) * g * torch.sigmoid(g)) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_wkv_reads_before_it_updates_and_the_bonus_weighs_the_token_itself():
    T, c, H, d, r = 6, 9, 2, 3, 2
    m = {"heads": H, "dim": d}
    shapes = {"mu." + s: (c,) for s in "rkvgw"}
    shapes.update({s: (H * d, c) for s in "rkvg"})
    shapes.update({"w1": (r, c), "w2": (H * d, r), "w0": (H * d,), "u": (H, d), "norm": (H * d,), "o": (c, H * d)})
    w = _rand(shapes, 2)
    h = _rand({"h": (T, c)}, 3)["h"]
    got = pl.wkv_mixer(h, w, "", m, 1e-5)
    prev = torch.cat([torch.zeros(1, c, dtype=F64), h[:-1]])
    mix = {s: h + (prev - h) * w["mu." + s] for s in "rkvgw"}
    assert torch.allclose(mix["r"][0], h[0] * (1 - w["mu.r"]), atol=1e-14)                  # nothing before the first token
    rr, kk, vv = ((mix[s] @ w[s].T).view(T, H, d) for s in "rkv")
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).view(T, H, d)
    assert bool(((decay > 0) & (decay < 1)).all())
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        for a in range(H):
            o[t, a] = (rr[t, a] * w["u"][a] * kk[t, a]).sum() * vv[t, a]       # the token itself: the bonus, no decay
            for j in range(t):
                through = torch.ones(d, dtype=F64)
                for s in range(j + 1, t):                                      # decays of the tokens in between only
                    through = through * decay[s, a]
                o[t, a] += (rr[t, a] * through * kk[j, a]).sum() * vv[j, a]
    g = mix["g"] @ w["g"].T
    want = (_unit(o, 1e-5).reshape(T, -1) * w["norm"] * g * torch.sigmoid(g)) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_gated_recurrence_candidate_and_state_by_hand():
    c, n = 5, 4
    w = _rand({"z": (n, c), "z.b": (n,), "x": (n, c), "x.b": (n,), "g": (n, c), "o": (c, n)}, 4)
    h = _rand({"h": (5, c)}, 5)["h"]
    got = pl.gated_recurrence(h, w, "", {"width": n})
    s = torch.zeros(n, dtype=F64)
    rows = []
    for t in range(5):
        z = 1 / (1 + torch.exp(-(h[t] @ w["z"].T + w["z.b"])))
        u = h[t] @ w["x"].T + w["x.b"]
        cand = torch.stack([ui + 0.5 if ui >= 0 else 1 / (1 + torch.exp(-ui)) for ui in u])
        s = (1 - z) * s + z * cand
        g = h[t] @ w["g"].T
        rows.append((s * g / (1 + torch.exp(-g))) @ w["o"].T)
    assert torch.allclose(got, torch.stack(rows), atol=1e-12)
    # the candidate is continuous and positive: 1/2 at zero from both sides
    tiny = torch.tensor([-1e-9, 0.0, 1e-9], dtype=F64)
    cand = torch.where(tiny >= 0, tiny + 0.5, torch.sigmoid(tiny))
    assert torch.allclose(cand, torch.full((3,), 0.5, dtype=F64), atol=1e-8)


def test_rotated_values_enter_the_sum_turned_by_their_distance_to_the_query():
    T, c = 8, 12
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 4, "scale": 0.4, "rot": {"dims": 4, "base": 30.0}}
    w = _rand({"q": (24, c), "k": (12, c), "v": (8, c), "o": (c, 16)}, 6)
    h = _rand({"h": (T, c)}, 7)["h"]
    got = pl.rotated_value_attention(h, w, "", m, 1e-5)
    pos = torch.arange(T)
    q = pl.rotate((h @ w["q"].T).view(T, 4, 6), pos, 4, 30.0)
    k = pl.rotate((h @ w["k"].T).view(T, 2, 6), pos, 4, 30.0)
    assert torch.equal(q[..., 4:], (h @ w["q"].T).view(T, 4, 6)[..., 4:])      # the features beyond rot.dims pass
    v = _unit((h @ w["v"].T).view(T, 2, 4), 1e-5)
    assert torch.allclose((v * v).mean(-1), torch.ones(T, 2, dtype=F64), atol=1e-4)
    rows = []
    for i in range(T):
        heads = []
        for a in range(4):
            s = torch.stack([0.4 * (q[i, a] @ k[j, a // 2]) for j in range(i + 1)])
            p = torch.softmax(s, 0)
            acc = torch.zeros(4, dtype=F64)
            for j in range(i + 1):
                # the value of position j, turned by j - i over all four features (pairs (0, 2) and (1, 3))
                acc += p[j] * pl.rotate(v[j: j + 1, a // 2: a // 2 + 1], torch.tensor([j - i]), 4, 30.0)[0, 0]
            heads.append(acc)
        rows.append(torch.cat(heads) @ w["o"].T)
    assert torch.allclose(got, torch.stack(rows), atol=1e-10)


def test_experts_softmax_over_the_chosen_logits_only():
    c, n, ff = 6, 5, 4
    shapes = {"router": (n, c)}
    for e in range(n):
        shapes.update({f"e{e}.gate": (ff, c), f"e{e}.up": (ff, c), f"e{e}.down": (c, ff)})
    w = _rand(shapes, 8)
    h = _rand({"h": (3, c)}, 9)["h"]
    got = pl.routed_experts(h, w, "", {"router": {"experts": n, "top": 2}, "expert": {"ff": ff}})
    for t in range(3):
        z = h[t] @ w["router"].T
        first, second = sorted(range(n), key=lambda e: -float(z[e]))[:2]
        a = 1 / (1 + math.exp(float(z[second] - z[first])))

        def expert(e):
            gate = h[t] @ w[f"e{e}.gate"].T
            return (gate * torch.sigmoid(gate) * (h[t] @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
        assert torch.allclose(got[t], a * expert(first) + (1 - a) * expert(second), atol=1e-12)


def test_run_order_loop_vector_and_the_layers_own_token_input():
    raw = config("B")
    assert pl.run_order(raw) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert pl.run_order(config("C")) == [(0, None), (1, None), (2, None)]
    # one layer by hand: norms on both sides of the mixer, no feed-forward, then the token's slice, gated
    raw = {"architecture": "Lunelorn", "vocab": 11, "width": 8, "norm": {"eps": 1e-3}, "token_side": {"dim": 2},
           "loop": {"start": 0, "stop": 1, "times": 2},
           "layers": [{"type": "retention", "mixer": {"heads": 1, "dim": 2, "vdim": 2, "decay": [0.5]}, "mlp": None}]}
    w = random_weights(raw, 0, dtype=F64)
    toks = [3, 7, 3]
    logits, after = pl.forward(raw, w, toks, return_layers=True)
    ids = torch.tensor(toks)
    x0 = _unit(w["embed"][ids], 1e-3) * w["embed.norm"]
    x = x0
    for p in range(2):
        x = x + (x0 if p else 0) + w["loop.step"][p]
        y = pl.retention_mixer(_unit(x, 1e-3) * w["l0.norm1"], w, "l0.mix.", raw["layers"][0]["mixer"], 1e-3)
        x = x + _unit(y, 1e-3) * w["l0.norm1b"]
        z = x @ w["l0.side.gate"].T
        gelu = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
        y = (gelu * w["side.embed"][ids][:, 0:2]) @ w["l0.side.proj"].T
        x = x + _unit(y, 1e-3) * w["l0.side.norm"]
        assert torch.allclose(after[p], x, atol=1e-12)
    assert torch.allclose(logits, (_unit(x, 1e-3) * w["final.norm"]) @ w["head"].T, atol=1e-12)      # no cap in this file
    capped = pl.forward({**raw, "logit_softcap": 2.0}, w, toks)
    assert torch.allclose(capped, 2.0 * torch.tanh(logits / 2.0), atol=1e-12) and float(capped.abs().max()) < 2.0


# ---- configuration, registry, names, loader ------------------------------------------------------------------
@pytest.mark.parametrize("which", "ABCDE")
def test_config_round_trip_and_names(which, tmp_path):
    raw = config(which)
    cfg = LunelornConfig.from_dict(raw)
    assert LunelornConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert cfg.to_dict() == {k: v for k, v in raw.items()}
    assert lookup("Lunelorn").config_class is LunelornConfig
    model = DecoderModel(lookup(cfg.architecture).describe(cfg))
    tensors = random_weights(raw, 1)
    specs = model.tensor_specs()
    assert {k for k, v in specs.items() if not v.optional} == set(tensors)
    bound = check_and_bind(tensors, specs)
    assert all(specs[k].fits(v.shape) for k, v in bound.items())
    # every run of a layer keeps a cache or state of its own; a parallel layer keeps pages and a state tensor
    order = pl.run_order(raw)
    kept = model.cache_specs()
    assert len(kept) == len(order)
    for (i, _), spec in zip(order, kept):
        kind = raw["layers"][i]["type"]
        assert isinstance(spec, PagedKVWithStateSpec if kind == "parallel" else FixedStateSpec)
    folder = write_random_model(tmp_path / which, cfg, 3, "bfloat16")
    assert {k for k in load_file(folder / "model.safetensors")} >= set(tensors)
    assert LunelornConfig.from_json(folder) == cfg


def test_config_errors_and_loader_errors():
    raw = config("A")
    for breaker in (lambda r: r.pop("width"), lambda r: r["layers"][0].update(type="conv"),
                    lambda r: r["layers"][2]["mixer"]["left"].update(kv_heads=4),
                    lambda r: r["layers"][2]["mixer"]["left"]["rot"].update(dims=34),
                    lambda r: r["layers"][2]["mixer"]["left"]["rot"].update(dims=7),
                    lambda r: r["layers"][2]["mixer"]["left"].update(vdim=15),
                    lambda r: r["layers"][2]["mixer"].pop("left_scale"),
                    lambda r: r["layers"][1]["mixer"].update(decay=[0.5, 0.5]),
                    lambda r: r["layers"][1]["mixer"].update(decay=[0.5, 0.5, 0.5, 1.5]),
                    lambda r: r["layers"][0]["mlp"]["router"].update(top=7),
                    lambda r: r["layers"][0]["mlp"].update(kind="dense"),
                    lambda r: r["loop"].update(stop=5), lambda r: r["loop"].update(times=0),
                    lambda r: r.update(logit_softcap=0.0), lambda r: r["token_side"].update(dim=0),
                    lambda r: r["norm"].update(eps=0)):
        broken = json.loads(json.dumps(raw))
        breaker(broken)
        with pytest.raises(ConfigError):
            LunelornConfig.from_dict(broken)
    cfg = LunelornConfig.from_dict(raw)
    tensors = random_weights(raw, 2)
    del tensors["l0.mix.u"]
    tensors["loop.step"] = tensors["loop.step"][:1]
    tensors["l2.mix.right.z.b"] = tensors["l2.mix.right.z.b"][:5]
    tensors["l0.mix.w1"] = tensors["l0.mix.w1"][:4]                         # its inner size no longer meets w2's
    with pytest.raises((WeightsError, ValueError)) as err:
        load_model(config=cfg, tensors=tensors, dtype="float32", device="cpu")
    assert all(name in str(err.value) for name in ("l0.mix.u", "loop.step", "l2.mix.right.z.b"))


# ---- the model through the step function on the test double ----------------------------------------------------
def cpu_runner(raw, tensors, page_tokens, num_pages, max_requests=4):
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    return make_runner(loaded, TorchOps(), page_tokens, num_pages, max_requests)


@pytest.mark.parametrize("which", "ABCE")
def test_cuttings_agree_with_plain(which):
    raw = config(which)
    tensors = random_weights(raw, 3, sharp=3.0)
    pt = PAGE_TOKENS[which]
    lengths = {"a": 41, "b": 36, "c": 9, "d": 2 * pt + 1}
    runner = cpu_runner(raw, tensors, pt, sum(-(-n // pt) for n in lengths.values()))
    reqs = {k: tokens_for(raw, n, i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: plain_logits(raw, tensors, v) for k, v in reqs.items()}
    got = {k: [] for k in reqs}
    pos = dict.fromkeys(reqs, 0)
    sizes = itertools.cycle([13, 1, 2, 7, 1, 1, 5, 2])
    while any(pos[k] < len(reqs[k]) for k in reqs):
        entries, order = [], []
        for k in reqs:
            if pos[k] == len(reqs[k]):
                continue
            m = min(next(sizes), len(reqs[k]) - pos[k])
            entries.append(StepEntry(k, reqs[k][pos[k]: pos[k] + m], list(range(m))))
            order.append((k, m))
            pos[k] += m
        out = runner.step(entries)
        row = 0
        for k, m in order:
            got[k].append(out[row: row + m])
            row += m
        runner.manager.check()
    for k in reqs:
        assert_rows_close(torch.cat(got[k]), want[k], 2e-4, f"request {k}")
        runner.finish(k)
    assert runner.manager.stats()["allocated_blocks"] == 0


def test_slots_and_pages_used_again():
    raw = config("A")
    tensors = random_weights(raw, 5)
    runner = cpu_runner(raw, tensors, 8, 6, max_requests=2)
    for n, name in enumerate(["p", "q", "r", "s", "t"]):                # five requests through two slots
        toks = tokens_for(raw, 17 + n, 40 + n)
        want = plain_logits(raw, tensors, toks)
        first = runner.step([StepEntry(name, toks[:9], list(range(9)))])
        rest = [runner.step([StepEntry(name, [t], [0])]) for t in toks[9:]]
        assert_rows_close(torch.cat([first] + rest), want, 2e-4, name)
        if n % 2 == 0:
            runner.finish(name)
        else:                                                           # two live at once, the older one ends later
            other = tokens_for(raw, 5, 90 + n)
            got = runner.step([StepEntry(name + "x", other, [4])])
            assert_rows_close(got, plain_logits(raw, tensors, other, [4]), 2e-4, name + "x")
            runner.finish(name)
            runner.finish(name + "x")
        runner.manager.check()


def test_generation_through_the_engine_on_the_double():
    raw = config("A")
    tensors = random_weights(raw, 4)
    loaded = load_model(config=LunelornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", device="cpu", block_size=8, num_blocks=12, max_batch_size=2,
                                            max_num_batched_tokens=12, max_prefill_chunk=5), ops=TorchOps())
    prompts = [tokens_for(raw, n, 30 + n) for n in (7, 1, 18)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 6)
    assert engine.stats()["allocated_blocks"] == 0
