"""Nukodra without a GPU: the plain implementation's mechanisms against restatements by hand, the
configuration and the loader, and the model through the step function, the cache manager, the scheduler
and the entry point with the torch test double in place of the CUDA kernel set."""

from __future__ import annotations

import itertools
import json
import math

import pytest
import torch

import plain_nukodra as pn
from nukodra_cases import PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits, random_weights, tokens_for
from torch_ops import TorchOps

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, NukodraConfig, SamplingParams
from mini_gpt_inference_b200.config import ConfigError, lookup
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import WeightsError, check_and_bind, load_file, write_random_model


def _rand(shapes, seed):
    gen = torch.Generator().manual_seed(seed)
    return {k: torch.randn(*s, generator=gen, dtype=torch.float64) for k, s in shapes.items()}


# ---- the plain mechanisms against restatements by hand ---------------------------------------------------
def test_rotation_pairs_a_feature_with_the_one_half_the_span_further():
    x = torch.arange(1.0, 9.0, dtype=torch.float64).view(1, 1, 8).repeat(3, 1, 1)
    got = pn.rotate(x, torch.tensor([0, 1, 5]), 4, 100.0)
    assert torch.equal(got[0], x[0]) and torch.equal(got[..., 4:], x[..., 4:])      # position 0 and the features beyond
    for t, p in ((1, 1), (2, 5)):
        for i, f in enumerate((1.0, 100.0 ** -0.5)):
            a = p * f
            u, v = x[t, 0, i], x[t, 0, i + 2]
            assert math.isclose(got[t, 0, i], u * math.cos(a) - v * math.sin(a), abs_tol=1e-12)
            assert math.isclose(got[t, 0, i + 2], v * math.cos(a) + u * math.sin(a), abs_tol=1e-12)


def test_stream_connections_by_hand():
    X = torch.tensor([[[1.0, 2.0]], [[10.0, 20.0]]], dtype=torch.float64)              # two streams, one token
    assert torch.equal(pn.streams_read(X, torch.tensor([0.5, 2.0], dtype=torch.float64)), torch.tensor([[20.5, 41.0]], dtype=torch.float64))
    M = torch.tensor([[1.0, 3.0], [0.0, -1.0]], dtype=torch.float64)                  # [from, to]
    y = torch.tensor([[100.0, 200.0]], dtype=torch.float64)
    new = pn.streams_write(X, M, torch.tensor([1.0, 0.1], dtype=torch.float64), y)
    assert torch.allclose(new[0], torch.tensor([[101.0, 202.0]], dtype=torch.float64))     # 1 * x0 + 0 * x1 + y
    assert torch.allclose(new[1], torch.tensor([[3.0, 6.0]]) - torch.tensor([[10.0, 20.0]]) + 0.1 * y)


def test_attention_window_sink_cap_and_groups_by_hand():
    T, c = 9, 10
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.4, "softcap": 1.5, "mask": {"size": 3},
         "rot": {"dims": 4, "base": 30.0}}
    w = _rand({"q": (24, c), "q.b": (24,), "k": (12, c), "k.b": (12,), "v": (6, c), "v.b": (6,), "q.norm": (24,),
               "k.norm": (12,), "sink": (4,), "g": (12, c), "o": (c, 12)}, 0)
    h = torch.randn(T, c, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    got = pn.attention_mixer(h, w, "", m, 1e-5)
    # a key that has left the window does not matter, however large it is
    h2 = h.clone()
    h2[2] *= 40.0
    again = pn.attention_mixer(h2, w, "", m, 1e-5)
    assert torch.allclose(got[5:], again[5:], atol=1e-12) and not torch.allclose(got[4], again[4])
    # one position and head by hand: the norm over the whole projection, the rotation, the cap, the sink
    qa = h @ w["q"].T + w["q.b"]
    ka = h @ w["k"].T + w["k.b"]
    qn = (qa / torch.sqrt((qa * qa).mean(-1, keepdim=True) + 1e-5) * w["q.norm"]).view(T, 4, 6)
    kn = (ka / torch.sqrt((ka * ka).mean(-1, keepdim=True) + 1e-5) * w["k.norm"]).view(T, 2, 6)
    v = (h @ w["v"].T + w["v.b"]).view(T, 2, 3)
    pos = torch.arange(T)
    qn, kn = pn.rotate(qn, pos, 4, 30.0), pn.rotate(kn, pos, 4, 30.0)
    t, heads = 6, []
    for a in range(4):
        s = torch.stack([1.5 * torch.tanh(0.4 * (qn[t, a] @ kn[j, a // 2]) / 1.5) for j in (4, 5, 6)])
        e = torch.exp(s)
        heads.append((e / (e.sum() + torch.exp(w["sink"][a]))) @ v[4:7, a // 2])
    want = (torch.cat(heads) * torch.sigmoid(h[t] @ w["g"].T)) @ w["o"].T
    assert torch.allclose(got[t], want, atol=1e-10)
    # the weights of a row sum to less than one: the sink takes its share and gives nothing
    m1 = dict(m, heads=1, kv_heads=1)
    w1 = {k: v for k, v in _rand({"q": (6, c), "q.b": (6,), "k": (6, c), "k.b": (6,), "v": (3, c), "v.b": (3,), "q.norm": (6,),
                                   "k.norm": (6,), "sink": (1,), "g": (3, c), "o": (c, 3)}, 2).items()}
    big = dict(w1, sink=torch.tensor([50.0], dtype=torch.float64))
    assert pn.attention_mixer(h, big, "", m1, 1e-5).abs().max() < 1e-12 < pn.attention_mixer(h, w1, "", m1, 1e-5).abs().max()


def test_latent_attention_equals_attention_over_full_keys_and_values():
    T, c = 7, 12
    m = {"heads": 3, "dim": 4, "rot_dim": 2, "vdim": 5, "kv_rank": 6, "scale": 0.3, "rot": {"dims": 2, "base": 10.0}}
    w = _rand({"q": (18, c), "dkv": (8, c), "dkv.norm": (6,), "uk": (12, 6), "uv": (15, 6), "g": (15, c), "o": (c, 15)}, 3)
    h = torch.randn(T, c, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    latent = pn.latent_of(h, w, "", m, 1e-5)
    got = pn.latent_attention_mixer(h, w, "", m, 1e-5, latent)
    low = h @ w["dkv"].T
    cc = low[:, :6] / torch.sqrt((low[:, :6] ** 2).mean(-1, keepdim=True) + 1e-5) * w["dkv.norm"]
    assert torch.allclose(latent[0], cc, atol=1e-12)
    t = 5
    a_t = [t * 1.0]                                                                  # one pair, frequency 1
    heads = []
    for a in range(3):
        q = (h[t] @ w["q"].T).view(3, 6)[a]
        qr = torch.stack([q[4] * math.cos(a_t[0]) - q[5] * math.sin(a_t[0]), q[5] * math.cos(a_t[0]) + q[4] * math.sin(a_t[0])])
        s = []
        for j in range(t + 1):
            kr = torch.stack([low[j, 6] * math.cos(j) - low[j, 7] * math.sin(j), low[j, 7] * math.cos(j) + low[j, 6] * math.sin(j)])
            s.append(0.3 * (q[:4] @ (w["uk"][4 * a: 4 * a + 4] @ cc[j]) + qr @ kr))
        p = torch.softmax(torch.stack(s), 0)
        heads.append(p @ (cc[: t + 1] @ w["uv"][5 * a: 5 * a + 5].T))
    want = (torch.cat(heads) * torch.sigmoid(h[t] @ w["g"].T)) @ w["o"].T
    assert torch.allclose(got[t], want, atol=1e-10)


def test_mamba2_is_a_decayed_sum_over_the_past():
    T, c = 8, 9
    m = {"heads": 4, "vdim": 3, "state": 5, "groups": 2, "conv": 3, "norm_groups": 3}
    inner, ch = 12, 12 + 20
    w = _rand({"in": (2 * inner + 20 + 4, c), "conv": (ch, 3), "conv.b": (ch,), "dt_bias": (4,), "A_log": (4,), "D": (4,),
               "norm": (inner,), "o": (c, inner)}, 5)
    h = torch.randn(T, c, dtype=torch.float64, generator=torch.Generator().manual_seed(6))
    got = pn.mamba2_mixer(h, w, "", m, 1e-5)
    proj = h @ w["in"].T
    z, raw, dt = proj[:, :inner], proj[:, inner: inner + ch], proj[:, inner + ch:]
    conv = torch.zeros(T, ch, dtype=torch.float64)
    for t in range(T):
        conv[t] = w["conv.b"] + sum(w["conv"][:, 2 - k] * raw[t - k] for k in range(3) if t - k >= 0)
    conv = conv * torch.sigmoid(conv)
    x, B, C = conv[:, :inner].view(T, 4, 3), conv[:, inner: inner + 10].view(T, 2, 5), conv[:, inner + 10:].view(T, 2, 5)
    dt = torch.log1p(torch.exp(dt + w["dt_bias"]))
    la = -torch.exp(w["A_log"]) * dt                                                # [T, heads]: logarithm of the decay
    y = torch.zeros(T, 4, 3, dtype=torch.float64)
    for t in range(T):
        for a in range(4):
            for j in range(t + 1):
                kept = torch.exp(la[j + 1: t + 1, a].sum())
                y[t, a] += kept * dt[j, a] * (C[t, a // 2] @ B[j, a // 2]) * x[j, a]
            y[t, a] += w["D"][a] * x[t, a]
    y = (y.reshape(T, inner) * z * torch.sigmoid(z)).view(T, 3, 4)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-5)).reshape(T, inner) * w["norm"]
    assert torch.allclose(got, y @ w["o"].T, atol=1e-10)


# ---- configuration, registry, names, loader ------------------------------------------------------------------
@pytest.mark.parametrize("which", "ABCDEF")
def test_config_round_trip_and_names(which, tmp_path):
    raw = config(which)
    cfg = NukodraConfig.from_dict(raw)
    assert NukodraConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert lookup("Nukodra").config_class is NukodraConfig
    model = DecoderModel(lookup(cfg.architecture).describe(cfg))
    tensors = random_weights(raw, 1)
    specs = model.tensor_specs()
    assert {k for k, v in specs.items() if not v.optional} == set(tensors)
    bound = check_and_bind(tensors, specs)
    assert all(specs[k].fits(v.shape) for k, v in bound.items())
    assert cfg.num_parameters() == sum(v.numel() for v in tensors.values())
    # a layer that reads another layer's latents keeps nothing of its own
    own = sum(1 for layer in raw["layers"] if layer["mixer"].get("kv_from") is None)
    assert sum(1 for s in model.cache_specs() if s is not None) == own
    folder = write_random_model(tmp_path / which, cfg, 3, "bfloat16")
    assert set(load_file(folder / "model.safetensors")) == set(tensors)
    assert NukodraConfig.from_json(folder) == cfg


def test_config_errors_and_loader_errors():
    raw = config("A")
    for breaker in (lambda r: r.pop("width"), lambda r: r["layers"][0].update(type="conv"),
                    lambda r: r["layers"][0]["mixer"].update(kv_heads=4), lambda r: r["layers"][0]["mixer"]["rot"].update(dims=34),
                    lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), lambda r: r["layers"][1]["mixer"].update(groups=3),
                    lambda r: r["layers"][1]["mixer"].update(norm_groups=5), lambda r: r["layers"][2]["mixer"].pop("kv_rank"),
                    lambda r: r["layers"][3]["mixer"].update(kv_from=1), lambda r: r["layers"][3]["mixer"].update(kv_from=3),
                    lambda r: r["layers"][3]["mixer"].update(kv_rank=32), lambda r: r["layers"][2]["mixer"]["rot"].update(dims=8),
                    lambda r: r["layers"][2]["mlp"].update(kind="moe"), lambda r: r.update(streams=0),
                    lambda r: r["norm"].update(eps=0)):
        broken = json.loads(json.dumps(raw))
        breaker(broken)
        with pytest.raises(ConfigError):
            NukodraConfig.from_dict(broken)
    cfg = NukodraConfig.from_dict(raw)
    tensors = random_weights(raw, 2)
    del tensors["l0.mix.sink"]
    tensors["l1.mix.conv"] = tensors["l1.mix.conv"][:, :3].contiguous()
    tensors["l3.hc1.mix"] = tensors["l3.hc1.mix"][:2]
    with pytest.raises(WeightsError) as err:
        load_model(config=cfg, tensors=tensors, dtype="float32", device="cpu")
    assert all(name in str(err.value) for name in ("l0.mix.sink", "l1.mix.conv", "l3.hc1.mix"))


# ---- the model through the step function on the test double ----------------------------------------------------
def cpu_runner(raw, tensors, page_tokens, num_pages, max_requests=4):
    loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    return make_runner(loaded, TorchOps(), page_tokens, num_pages, max_requests)


@pytest.mark.parametrize("which", "ABCEF")
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
    loaded = load_model(config=NukodraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", device="cpu", block_size=8, num_blocks=12, max_batch_size=2,
                                            max_num_batched_tokens=12, max_prefill_chunk=5), ops=TorchOps())
    prompts = [tokens_for(raw, n, 30 + n) for n in (7, 1, 18)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 6)
    assert engine.stats()["allocated_blocks"] == 0
