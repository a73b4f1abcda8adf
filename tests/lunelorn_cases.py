"""Small Lunelorn configurations and random weights for the tests, made here (names and shapes written out from the
design, not taken from the engine's own list), and the plain logits."""

from __future__ import annotations

import math

import torch

import plain_lunelorn


def _retention(heads, dim, vdim, decay):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _wkv(heads, dim):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def _parallel(heads, kv_heads, dim, vdim, scale, rot, gru, left_scale, right_scale):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"dims": rot[0], "base": rot[1]}}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": gru}, "left_scale": left_scale,
                                          "right_scale": right_scale}}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def all_experts(raw: dict) -> dict:
    """The same configuration with every router choosing all its experts (the weights stay a softmax).  A choice
    among experts is discrete: where two router logits are close, the rounding of bfloat16 activations can turn it,
    and the two sides then compute different functions.  Whole models are therefore compared with real choices in
    32-bit and with all experts in bfloat16; the router alone is compared in both formats."""
    for layer in raw["layers"]:
        if layer.get("mlp") is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def config(which: str, every_expert: bool = False) -> dict:
    if every_expert:
        return all_experts(config(which))
    return _config(which)


def _config(which: str) -> dict:
    """A: every mixer, a loop of two passes over the first three of four layers, a token input per layer, grouped key
    heads, part of a head rotated, a layer without a feed-forward.  B: the loop in the middle (a layer before it and
    one after it), three passes, as many key heads as query heads, whole heads rotated, one chosen expert, value heads
    larger than key heads, no cap on the logits.  C: no loop and no token input, all experts chosen, nothing of the
    query and key heads rotated, a decay of exactly 1 and one of 0, odd head sizes.  D: a loop of one pass over all
    layers (its vector is added once), heads of 128, a recurrence wider than the model.  E: recurrent layers alone
    (nothing is kept in pages)."""
    if which == "A":
        layers = [
            {**_wkv(3, 16), "mlp": _moe(6, 2, 40)},
            {**_retention(4, 24, 16, (0.9, 0.97, 0.99, 0.999)), "mlp": None},
            {**_parallel(6, 2, 32, 16, 0.2, (8, 5000.0), 80, 1.3, 0.6), "mlp": _moe(4, 3, 24)},
            {**_parallel(2, 1, 16, 24, 0.3, (16, 300.0), 48, 0.7, 1.1), "mlp": _moe(6, 2, 40)},
        ]
        return {"architecture": "Lunelorn", "vocab": 211, "width": 64, "layers": layers, "norm": {"eps": 1e-5},
                "logit_softcap": 8.0, "loop": {"start": 0, "stop": 3, "times": 2}, "token_side": {"dim": 12}}
    if which == "B":
        layers = [
            {**_parallel(3, 3, 24, 40, 0.25, (24, 10000.0), 96, 1.0, 1.0), "mlp": _moe(5, 1, 64)},
            {**_retention(2, 40, 40, (0.95, 0.5)), "mlp": _moe(3, 2, 32)},
            {**_wkv(2, 40), "mlp": None},
            {**_wkv(4, 8), "mlp": _moe(2, 1, 16)},
        ]
        return {"architecture": "Lunelorn", "vocab": 300, "width": 96, "layers": layers, "norm": {"eps": 1e-6},
                "loop": {"start": 1, "stop": 3, "times": 3}, "token_side": {"dim": 8}}
    if which == "C":
        layers = [
            {**_retention(3, 10, 34, (1.0, 0.0, 0.875)), "mlp": _moe(3, 3, 24)},
            {**_parallel(5, 1, 24, 10, 0.25, (0, 100.0), 33, 2.0, 0.25), "mlp": None},
            {**_wkv(1, 72), "mlp": _moe(8, 2, 16)},
        ]
        return {"architecture": "Lunelorn", "vocab": 97, "width": 72, "layers": layers, "norm": {"eps": 1e-4},
                "logit_softcap": 30.0}
    if which == "D":
        layers = [
            {**_parallel(4, 2, 128, 128, 0.09, (64, 1e6), 192, 1.2, 0.5), "mlp": _moe(4, 2, 128)},
            {**_retention(2, 128, 64, (0.99, 0.9990234375)), "mlp": None},
            {**_wkv(2, 64), "mlp": _moe(4, 2, 64)},
        ]
        return {"architecture": "Lunelorn", "vocab": 384, "width": 128, "layers": layers, "norm": {"eps": 1e-5},
                "logit_softcap": 15.0, "loop": {"start": 0, "stop": 3, "times": 1}, "token_side": {"dim": 32}}
    if which == "E":
        layers = [
            {**_wkv(2, 24), "mlp": _moe(4, 2, 32)},
            {**_retention(2, 16, 24, (0.8, 0.96)), "mlp": _moe(4, 1, 32)},
        ]
        return {"architecture": "Lunelorn", "vocab": 64, "width": 40, "layers": layers, "norm": {"eps": 1e-5},
                "loop": {"start": 1, "stop": 2, "times": 2}, "token_side": {"dim": 4}}
    raise KeyError(which)


def random_config(rng) -> dict:
    """A configuration drawn at random: 2 to 6 layers of the three mixer kinds in any order, some without a
    feed-forward, with or without a loop, a token input and a cap, sizes that are not the fixed cases'."""
    width = rng.choice([96, 128, 160, 192, 256, 320])
    n_layers = rng.randint(2, 6)
    layers = []
    for _ in range(n_layers):
        kind = rng.choice(["retention", "parallel", "wkv"])
        mlp = None
        if rng.random() > 0.25:
            experts = rng.choice([2, 4, 8, 12, 16])
            mlp = _moe(experts, rng.randint(1, min(experts, 4)), rng.choice([32, 64, 96, 128]))
        if kind == "retention":
            heads = rng.randint(1, 8)
            layer = _retention(heads, rng.choice([16, 32, 48, 64, 128]), rng.choice([16, 32, 64, 128]),
                               [1.0 - 2.0 ** -rng.randint(3, 11) for _ in range(heads)])
        elif kind == "wkv":
            layer = _wkv(rng.randint(1, 8), rng.choice([16, 32, 64]))
        else:
            kv = rng.choice([1, 2, 3, 4]); heads = kv * rng.choice([1, 2, 3, 4])
            dim = rng.choice([32, 48, 64, 96, 128]); vdim = rng.choice([32, 64, 128])
            rot = rng.choice([dim, dim // 2, 16, 0]); rot -= rot % 2
            layer = _parallel(heads, kv, dim, vdim, 1 / math.sqrt(dim), (rot, rng.choice([1e4, 3e5, 1e6])),
                              rng.choice([64, 160, 256, 384]), rng.choice([0.5, 1.0, 1.2]), rng.choice([0.5, 1.0, 1.5]))
        layers.append({**layer, "mlp": mlp})
    raw = {"architecture": "Lunelorn", "vocab": rng.choice([300, 480, 512, 1000]), "width": width, "layers": layers,
           "norm": {"eps": rng.choice([1e-5, 1e-6])}}
    if rng.random() < 0.7:
        start = rng.randint(0, n_layers - 1)
        raw["loop"] = {"start": start, "stop": rng.randint(start + 1, n_layers), "times": rng.randint(1, 3)}
    if rng.random() < 0.7:
        raw["token_side"] = {"dim": rng.choice([8, 16, 24, 40])}
    if rng.random() < 0.7:
        raw["logit_softcap"] = rng.choice([10.0, 15.0, 30.0])
    return raw


PAGE_TOKENS = {"A": 8, "B": 16, "C": 4, "D": 16, "E": 8}
DECAY_RANK = 6          # inner size of the two thin decay matrices of the tests' wkv layers


def random_weights(raw: dict, seed: int, dtype=torch.float32, sharp: float = 1.0, as_bfloat16: bool = False,
                   steady: bool = False) -> dict:
    """Weights with unit-variance activations: matrices ``N(0, 1 / inputs)``, norm weights ``1 + N(0, 0.3)``, biases
    ``N(0, 0.3)``, embeddings ``N(0, 1)``, blend weights in 0..1.  ``sharp`` scales the attention's query projection
    (a softmax that leans on few keys).  ``as_bfloat16``: every number is one that bfloat16 holds.  ``steady``: the
    matrix memories' query matrices lean towards their key matrices and the wkv bonus is positive, so that a token's
    read-out of its own key is well away from zero.  (Every head's read-out is divided by its root mean square:
    where it is one term, as for a sequence's first tokens, and that term nearly cancels, the norm magnifies the
    rounding of bfloat16 queries and keys without bound.  Runs in bfloat16 use steady weights; 32-bit runs do not.)"""
    gen = torch.Generator().manual_seed(seed)
    c = raw["width"]

    def mat(rows, cols, scale=1.0):
        return torch.randn(rows, cols, generator=gen) * (scale / math.sqrt(cols))

    def vec(n, scale=0.3):
        return torch.randn(n, generator=gen) * scale

    w = {"embed": torch.randn(raw["vocab"], c, generator=gen), "embed.norm": 1.0 + vec(c), "final.norm": 1.0 + vec(c),
         "head": mat(raw["vocab"], c, 2.0)}
    side = raw.get("token_side")
    if side is not None:
        w["side.embed"] = torch.randn(raw["vocab"], side["dim"] * len(raw["layers"]), generator=gen)
    if raw.get("loop"):
        w["loop.step"] = vec(raw["loop"]["times"] * c, 0.5).view(raw["loop"]["times"], c)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = 1.0 + vec(c), 1.0 + vec(c)
        x = p + "mix."
        if layer["type"] == "retention":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            w[x + "q"], w[x + "k"], w[x + "v"], w[x + "g"] = mat(h * d, c), mat(h * d, c), mat(h * dv, c), mat(h * dv, c)
            w[x + "o"] = mat(c, h * dv)
            if steady:
                w[x + "q"] = w[x + "k"] + 0.5 * w[x + "q"]
        elif layer["type"] == "wkv":
            h, d = m["heads"], m["dim"]
            for s in "rkvgw":
                w[x + "mu." + s] = torch.rand(c, generator=gen)
            for s in "rkvg":
                w[x + s] = mat(h * d, c)
            w[x + "w1"], w[x + "w2"], w[x + "w0"] = mat(DECAY_RANK, c), mat(h * d, DECAY_RANK, 2.0), vec(h * d, 1.0) - 1.0
            w[x + "u"], w[x + "norm"], w[x + "o"] = vec(h * d, 0.5).view(h, d), 1.0 + vec(h * d), mat(c, h * d)
            if steady:
                w[x + "r"], w[x + "mu.r"], w[x + "u"] = w[x + "k"] + 0.5 * w[x + "r"], w[x + "mu.k"].clone(), w[x + "u"].abs() + 0.5
        else:
            a, n = m["left"], m["right"]["width"]
            w[x + "left.q"] = mat(a["heads"] * a["dim"], c, sharp)
            w[x + "left.k"], w[x + "left.v"] = mat(a["kv_heads"] * a["dim"], c), mat(a["kv_heads"] * a["vdim"], c)
            w[x + "left.o"] = mat(c, a["heads"] * a["vdim"])
            w[x + "right.z"], w[x + "right.z.b"] = mat(n, c), vec(n, 1.0)
            w[x + "right.x"], w[x + "right.x.b"] = mat(n, c), vec(n)
            w[x + "right.g"], w[x + "right.o"] = mat(n, c), mat(c, n)
        f = layer.get("mlp")
        if f is not None:
            w[p + "norm2"], w[p + "norm2b"] = 1.0 + vec(c), 1.0 + vec(c)
            y = p + "mlp."
            w[y + "router"] = mat(f["router"]["experts"], c, 2.0)
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                w[f"{y}e{e}.gate"], w[f"{y}e{e}.up"], w[f"{y}e{e}.down"] = mat(ff, c), mat(ff, c), mat(c, ff)
        if side is not None:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(side["dim"], c), mat(c, side["dim"]), 1.0 + vec(c)
    if as_bfloat16:
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def tokens_for(raw: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, raw["vocab"], (length,), generator=gen).tolist()


def plain_logits(raw: dict, tensors: dict, tokens, rows=None, dtype=torch.float64) -> torch.Tensor:
    out = plain_lunelorn.forward(raw, tensors, tokens, dtype)
    return out if rows is None else out[list(rows)]


def rounding_spread(raw: dict, tensors: dict, tokens, rows=None) -> torch.Tensor:
    """Per row: how far the logits move (over the row's spread) when the activations between matrix products are
    rounded to bfloat16 in the plain implementation and nothing else changes.  The design divides sublayer outputs and heads by their root mean square,
    so a row where a sum nearly cancels magnifies rounding many times over; a bfloat16 run is held to its tolerance
    plus three times this."""
    exact = plain_lunelorn.forward(raw, tensors, tokens)
    moved = plain_lunelorn.forward(raw, tensors, tokens, round_inputs=torch.bfloat16)
    err = relative_error(moved, exact)
    return err if rows is None else err[list(rows)]


def plain_greedy(raw: dict, tensors: dict, prompt, new_tokens: int) -> list[int]:
    return plain_lunelorn.greedy(raw, tensors, prompt, new_tokens)


def relative_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: the largest difference of the logits over the row's own spread."""
    want = want.double()
    return (got.double().cpu() - want).abs().amax(-1) / want.std(-1)


def assert_rows_close(got, want, tol, what: str, places=None, outliers: float = 0.0, slack=None) -> None:
    """``outliers``: the share of rows (at least one, if not zero) that may miss ``tol``, though not five times
    ``tol`` (bfloat16 runs: a unit norm after a read-out that nearly cancels magnifies one token's rounding).
    ``slack``: per row, what rounding alone does (``rounding_spread``); three times it is added to ``tol``."""
    err = relative_error(got, want)
    limit = tol if slack is None else tol + 3.0 * slack
    bad = (~(err <= limit)).nonzero()
    if outliers and 0 < bad.numel() <= max(1, int(outliers * err.numel())):
        bad = (~(err <= 5 * limit)).nonzero()
    if bad.numel():
        i = int(bad[0])
        raise AssertionError(f"{what}: first wrong logits at {places[i] if places is not None else i}: "
                             f"error {float(err[i]):.3e} of the row's spread > {float(limit[i]) if slack is not None else tol:.1e}")
