"""Small Nukodra configurations and random weights for the tests, made here (names and shapes written
out from the design, not taken from the engine's own list), and the plain logits."""

from __future__ import annotations

import math

import torch

import plain_nukodra


def _attn(heads, kv_heads, dim, vdim, scale, window=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def config(which: str) -> dict:
    """A: every mixer, three streams, a layer that reads an earlier layer's latents, a window shorter than the
    tests' sequences, part of a head rotated, grouped key heads, a state-space layer without a feed-forward.
    B: one stream (through the connections all the same), the state-space layer first, one group and one norm
    part, two taps, as many key heads as query heads, a window of one page, whole heads rotated, no cap.
    C: no streams at all (plain residual sums), attention without window, rotation or cap, odd head sizes, five
    taps, a latent layer without a feed-forward.  D: heads of 128 and 64 features, a latent of 256, a state of
    128.  E: state-space layers alone (nothing is kept in pages), a single tap.  F: latent attention alone, two
    layers reading the first one's latents, four streams."""
    if which == "A":
        layers = [
            {**_attn(6, 2, 32, 16, 0.3, window=40, rot=(16, 5000.0), softcap=4.0), "mlp": _dense(96)},
            {**_mamba(4, 16, 24, 2, 4, 4), "mlp": None},
            {**_latent(4, 24, 16, 40, 48, 0.2, 300.0), "mlp": _dense(80)},
            {**_latent(2, 16, 16, 24, 48, 0.25, 300.0, kv_from=2), "mlp": _dense(80)},
        ]
        return {"architecture": "Nukodra", "vocab": 211, "width": 64, "streams": 3, "layers": layers, "norm": {"eps": 1e-4}}
    if which == "B":
        layers = [
            {**_mamba(3, 40, 16, 1, 2, 1), "mlp": _dense(128)},
            {**_attn(3, 3, 24, 24, 0.2, window=16, rot=(24, 10000.0)), "mlp": _dense(200)},
            {**_latent(1, 32, 8, 32, 24, 0.15, 10000.0), "mlp": None},
            {**_attn(4, 1, 16, 40, 0.25, window=33, rot=(8, 100.0), softcap=30.0), "mlp": None},
        ]
        return {"architecture": "Nukodra", "vocab": 300, "width": 96, "streams": 1, "layers": layers, "norm": {"eps": 1e-6}}
    if which == "C":
        layers = [
            {**_latent(5, 10, 6, 33, 20, 0.3, 50.0), "mlp": None},
            {**_attn(5, 1, 24, 33, 0.25), "mlp": _dense(72)},
            {**_mamba(6, 12, 10, 3, 5, 2), "mlp": _dense(40)},
            {**_attn(2, 2, 80, 8, 0.1, softcap=2.0), "mlp": _dense(72)},
        ]
        return {"architecture": "Nukodra", "vocab": 97, "width": 72, "layers": layers, "norm": {"eps": 1e-5}}
    if which == "D":
        layers = [
            {**_attn(4, 2, 128, 128, 0.09, window=100, rot=(64, 1e6), softcap=50.0), "mlp": _dense(256)},
            {**_mamba(4, 64, 128, 1, 4, 1), "mlp": None},
            {**_latent(4, 128, 64, 128, 256, 0.07, 10000.0), "mlp": _dense(256)},
            {**_attn(2, 1, 64, 128, 0.125, window=64, rot=(64, 10000.0)), "mlp": None},
            {**_latent(2, 64, 64, 64, 256, 0.1, 10000.0, kv_from=2), "mlp": None},
        ]
        return {"architecture": "Nukodra", "vocab": 384, "width": 128, "streams": 2, "layers": layers, "norm": {"eps": 1e-5}}
    if which == "E":
        layers = [
            {**_mamba(2, 8, 16, 2, 1, 2), "mlp": _dense(64)},
            {**_mamba(4, 24, 8, 4, 3, 3), "mlp": None},
        ]
        return {"architecture": "Nukodra", "vocab": 64, "width": 40, "streams": 2, "layers": layers, "norm": {"eps": 1e-5}}
    if which == "F":
        layers = [
            {**_latent(2, 16, 4, 16, 32, 0.2, 20.0), "mlp": _dense(48)},
            {**_latent(3, 8, 4, 8, 32, 0.3, 20.0, kv_from=0), "mlp": None},
            {**_latent(1, 40, 4, 24, 32, 0.1, 20.0, kv_from=0), "mlp": _dense(48)},
        ]
        return {"architecture": "Nukodra", "vocab": 80, "width": 48, "streams": 4, "layers": layers, "norm": {"eps": 1e-5}}
    raise KeyError(which)


def random_config(rng) -> dict:
    """A configuration drawn at random: 3 to 8 layers of the three mixer kinds in any order, some without a
    feed-forward, latent layers that read an earlier one's rows, none to four streams, sizes that are not the
    fixed cases' (1 to 20 heads, heads of 32 to 128, windows of 17 to 257, latents of 48 to 256, states of 16 to 128)."""
    width = rng.choice([96, 128, 160, 192, 256, 320])
    n_layers = rng.randint(3, 8)
    layers, latent_sources = [], []
    for i in range(n_layers):
        kind = rng.choice(["attention", "latent_attention", "mamba2"])
        mlp = None if rng.random() < 0.3 else _dense(rng.choice([128, 192, 256, 384]))
        if kind == "attention":
            kv = rng.choice([1, 2, 3, 4]); heads = kv * rng.choice([1, 2, 3, 4])
            dim = rng.choice([32, 48, 64, 96, 128]); vdim = rng.choice([32, 64, 128])
            rot = rng.choice([dim, dim // 2, 16]); rot -= rot % 2
            layer = _attn(heads, kv, dim, vdim, 1 / math.sqrt(dim), window=rng.choice([17, 64, 100, 140, 200, 257]),
                             rot=(rot, rng.choice([1e4, 3e5, 1e6])), softcap=rng.choice([15.0, 25.0, 50.0]))
        elif kind == "latent_attention":
            heads = rng.choice([2, 4, 6, 8, 12, 16, 20]); dim = rng.choice([32, 64, 128]); vdim = rng.choice([32, 64, 128])
            if latent_sources and rng.random() < 0.5:
                src = rng.choice(latent_sources)
                m = layers[src]["mixer"]
                layer = _latent(heads, dim, m["rot_dim"], vdim, m["kv_rank"], 1 / math.sqrt(dim + m["rot_dim"]), m["rot"]["base"], kv_from=src)
            else:
                rot_dim = rng.choice([16, 32, 64]); rank = rng.choice([48, 64, 96, 128, 192, 256])
                layer = _latent(heads, dim, rot_dim, vdim, rank, 1 / math.sqrt(dim + rot_dim), rng.choice([1e4, 5e4]))
                latent_sources.append(i)
        else:
            groups = rng.choice([1, 2, 4]); heads = groups * rng.choice([1, 2, 3, 4]); vdim = rng.choice([16, 32, 64])
            parts = rng.choice([p for p in (1, 2, 4, heads) if (heads * vdim) % p == 0])
            layer = _mamba(heads, vdim, rng.choice([16, 32, 64, 128]), groups, rng.choice([2, 3, 4]), parts)
        layers.append({**layer, "mlp": mlp})
    raw = {"architecture": "Nukodra", "vocab": rng.choice([300, 480, 512, 1000]), "width": width, "layers": layers,
           "norm": {"eps": rng.choice([1e-5, 1e-6])}}
    s = rng.choice([None, 1, 2, 3, 4])
    if s: raw["streams"] = s
    return raw


PAGE_TOKENS = {"A": 8, "B": 16, "C": 4, "D": 16, "E": 8, "F": 4}


def random_weights(raw: dict, seed: int, dtype=torch.float32, sharp: float = 1.0, as_bfloat16: bool = False) -> dict:
    """Weights with unit-variance activations: matrices ``N(0, 1 / inputs)``, output projections smaller by the
    depth, norm weights (stored around zero) and biases ``N(0, 0.3)``, embeddings ``N(0, 1)``, stream connections
    near the identity.  ``sharp`` scales what makes a softmax lean on few keys: the gains of the attention's
    query norm, the query projection of the latent layers.  ``as_bfloat16``: every number is one that bfloat16
    holds (an engine that computes in bfloat16 and the plain side then use the same weights)."""
    gen = torch.Generator().manual_seed(seed)
    c = raw["width"]
    depth = len(raw["layers"])
    streams = raw.get("streams")

    def mat(rows, cols, scale=1.0):
        return torch.randn(rows, cols, generator=gen) * (scale / math.sqrt(cols))

    def vec(n, scale=0.3):
        return torch.randn(n, generator=gen) * scale

    def connection(name):
        if streams is None:
            return
        w[name + ".in"] = 1.0 / streams + vec(streams, 0.2)
        w[name + ".out"] = 1.0 + vec(streams, 0.3)
        w[name + ".mix"] = torch.eye(streams) + vec(streams * streams, 0.15).view(streams, streams)

    w = {"embed": torch.randn(raw["vocab"], c, generator=gen), "final.norm": vec(c)}
    out_scale = 1.0 / math.sqrt(2 * depth)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = vec(c)
        connection(p + "hc1")
        x = p + "mix."
        if layer["type"] == "attention":
            h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[x + "q"], w[x + "q.b"] = mat(h * d, c), vec(h * d)
            w[x + "k"], w[x + "k.b"] = mat(g * d, c), vec(g * d)
            w[x + "v"], w[x + "v.b"] = mat(g * dv, c), vec(g * dv)
            w[x + "q.norm"], w[x + "k.norm"] = sharp * (1.0 + vec(h * d)), 1.0 + vec(g * d)
            w[x + "sink"] = 1.0 + vec(h, 1.0)
            w[x + "g"], w[x + "o"] = mat(h * dv, c), mat(c, h * dv, out_scale)
        elif layer["type"] == "latent_attention":
            h, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[x + "q"] = mat(h * (d + dr), c, sharp)
            if m.get("kv_from") is None:
                w[x + "dkv"], w[x + "dkv.norm"] = mat(r + dr, c), 1.0 + vec(r)
            w[x + "uk"], w[x + "uv"] = mat(h * d, r), mat(h * dv, r)
            w[x + "g"], w[x + "o"] = mat(h * dv, c), mat(c, h * dv, out_scale)
        else:
            h, dv, n, g, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = h * dv, h * dv + 2 * g * n
            w[x + "in"] = mat(2 * inner + 2 * g * n + h, c)
            w[x + "conv"], w[x + "conv.b"] = mat(ch, taps, 1.5), vec(ch)
            w[x + "dt_bias"], w[x + "A_log"], w[x + "D"] = vec(h, 1.0) - 1.0, vec(h, 0.7) - 0.5, 1.0 + vec(h)
            w[x + "norm"], w[x + "o"] = 1.0 + vec(inner), mat(c, inner, out_scale)
        f = layer.get("mlp")
        if f is None:
            continue
        w[p + "norm2"] = vec(c)
        connection(p + "hc2")
        y = p + "mlp."
        w[y + "gate"], w[y + "up"] = mat(f["ff"], c), mat(f["ff"], c)
        w[y + "down"] = mat(c, f["ff"], out_scale)
    if as_bfloat16:
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def tokens_for(raw: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, raw["vocab"], (length,), generator=gen).tolist()


def plain_logits(raw: dict, tensors: dict, tokens, rows=None, dtype=torch.float64) -> torch.Tensor:
    out = plain_nukodra.forward(raw, tensors, tokens, dtype)
    return out if rows is None else out[list(rows)]


def plain_greedy(raw: dict, tensors: dict, prompt, new_tokens: int) -> list[int]:
    return plain_nukodra.greedy(raw, tensors, prompt, new_tokens)


def relative_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: the largest difference of the logits over the row's own spread."""
    want = want.double()
    return (got.double().cpu() - want).abs().amax(-1) / want.std(-1)


def assert_rows_close(got, want, tol, what: str, places=None, outliers: float = 0.0) -> None:
    """``outliers``: the share of rows (at least one, if not zero) that may miss ``tol``, though not five times
    ``tol`` (bfloat16 runs: a norm after a read-out that nearly cancels magnifies one token's rounding)."""
    err = relative_error(got, want)
    bad = (~(err <= tol)).nonzero()
    if outliers and 0 < bad.numel() <= max(1, int(outliers * err.numel())):
        bad = (~(err <= 5 * tol)).nonzero()
    if bad.numel():
        i = int(bad[0])
        raise AssertionError(f"{what}: first wrong logits at {places[i] if places is not None else i}: "
                             f"error {float(err[i]):.3e} of the row's spread > {tol:.1e}")
