"""A plain, slow Lunelorn: one function per mechanism, whole sequences, float64 by default.

It takes the model as a config dict (the keys of ``config.json``) and a dict of tensors by their
checkpoint names, and shares no code with the engine.  Notation: ``x`` is the residual stream
``[T, width]`` of one sequence, ``h`` the input of a mixer or feed-forward, ``t`` a position.

* embedding:   ``n(E[tok_t])`` with the model's norm and the gain ``embed.norm``; this is ``x0``
* rms norm:    ``n(x) = x / sqrt(mean(x^2) + eps) * w`` (``w`` left out for a unit norm)
* run order:   layers before ``loop.start`` once; then ``times`` passes over ``start .. stop-1`` with the same
  weights, in front of pass ``p``: ``x += x0`` (not for ``p = 0``), then ``x += step[p]``; then the rest
* a layer:     ``x += n1b(mixer(n1(x)))``, ``x += n2b(ff(n2(x)))`` (if it has a feed-forward), then the token's
  own input: ``e`` = the layer's part of ``side.embed[tok]``, ``y = P (gelu(G x) * e)``, ``x += n_side(y)``
* retention:   ``S_t = a_h S_(t-1) + (k_t / sqrt(d)) v_t^T``, ``o_t = S_t^T q_t``, unit norm per head, times
  ``silu(W_g h)``
* parallel:    ``ls * attention + rs * gru``.  Attention: grouped key heads, the first ``n`` features of query and
  key heads rotated, values divided by their root mean square and rotated over all their features, causal
  softmax of ``scale * q . k``, the head's output rotated back by the query's position.  Gated recurrence:
  ``s_t = (1 - z_t) s_(t-1) + z_t c_t``, ``z = sigmoid(.)``, ``c = u + 1/2`` for ``u >= 0``, ``sigmoid(u)`` below
* wkv:         every projection reads its own blend of ``h_t`` and ``h_(t-1)``; ``w_t = exp(-exp(.))`` per key
  channel; ``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t``; ``S_t = diag(w_t) S_(t-1) + k_t v_t^T``
* experts:     the ``top`` largest router logits choose, softmax over the chosen logits weighs,
  an expert is ``W_down (silu(W_gate h) * W_up h)``
* output:      ``cap * tanh(W n(x) / cap)``
"""

from __future__ import annotations

import math

import torch


# ---- pieces --------------------------------------------------------------------------------------
ROUND = None      # a dtype through which activations between two products are rounded (see ``forward``), or None


def _r(x):
    return x if ROUND is None else x.to(ROUND).to(x.dtype)


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x, positions, n, base, sign=1.0):
    """x: [T, heads, features]; the first n features of every head turn with the position (feature ``i`` with
    ``i + n/2``, angle ``sign * t * base^(-2i/n)``)."""
    if n == 0:
        return x
    half = n // 2
    freq = torch.tensor([base ** (-2.0 * i / n) for i in range(half)], dtype=x.dtype)
    angle = sign * positions.to(x.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:n]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., n:]], dim=-1)


# ---- mixers --------------------------------------------------------------------------------------
def retention_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    dv = m.get("vdim", d)
    q = _r(h @ w[p + "q"].T).view(T, H, d)
    k = _r(h @ w[p + "k"].T).view(T, H, d) * d ** -0.5
    v = _r(h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    o = rms_norm(torch.stack(out), None, eps).reshape(T, H * dv)
    return _r(o * silu(_r(h @ w[p + "g"].T))) @ w[p + "o"].T


def rotated_value_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    pos = torch.arange(T)
    q = _r(rotate(_r(h @ w[p + "q"].T).view(T, H, d), pos, rot["dims"], rot["base"]))
    k = _r(rotate(_r(h @ w[p + "k"].T).view(T, G, d), pos, rot["dims"], rot["base"]))
    v = rms_norm(_r(h @ w[p + "v"].T).view(T, G, dv), None, eps)
    v = _r(rotate(v, pos, dv, rot["base"]))
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    s = s.masked_fill(pos[None, :, None] < pos[None, None, :], float("-inf"))
    o = torch.einsum("hij,jhe->ihe", torch.softmax(s, dim=-1), v)
    o = _r(rotate(_r(o), pos, dv, rot["base"], sign=-1.0))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gated_recurrence(h, w, p, m):
    T = h.shape[0]
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros(m["width"], dtype=h.dtype)
    out = []
    for t in range(T):
        s = (1 - z[t]) * s + z[t] * cand[t]
        out.append(s)
    return _r(torch.stack(out) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = rotated_value_attention(h, w, p + "left.", m["left"], eps)
    right = gated_recurrence(h, w, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def wkv_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def blend(name):
        return _r(h + (before - h) * w[p + "mu." + name])
    r = _r(blend("r") @ w[p + "r"].T).view(T, H, d)
    k = _r(blend("k") @ w[p + "k"].T).view(T, H, d)
    v = _r(blend("v") @ w[p + "v"].T).view(T, H, d)
    gate = silu(_r(blend("g") @ w[p + "g"].T))
    decay = torch.exp(-torch.exp(_r(torch.tanh(blend("w") @ w[p + "w1"].T)) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    bonus = w[p + "u"].view(H, d)
    S = torch.zeros(H, d, d, dtype=h.dtype)
    out = []
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", S + bonus[:, :, None] * kv, r[t]))
        S = decay[t][:, :, None] * S + kv
    o = rms_norm(torch.stack(out), None, eps).reshape(T, H * d) * w[p + "norm"]
    return _r(o * gate) @ w[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------
def routed_experts(h, w, p, f):
    n, top = f["router"]["experts"], f["router"]["top"]
    logits = h @ w[p + "router"].T
    best, ids = torch.topk(logits, top, dim=-1)
    weights = torch.softmax(best, dim=-1)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = f"{p}e{int(ids[t, j])}."
            out[t] += weights[t, j] * (_r(silu(h[t] @ w[e + "gate"].T) * (h[t] @ w[e + "up"].T)) @ w[e + "down"].T)
    return out


def token_side_input(x, ids, w, p, index, dim, eps):
    e = w["side.embed"][ids][:, index * dim: (index + 1) * dim]
    y = _r(gelu_tanh(_r(x) @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_norm(y, w[p + "norm"], eps)


# ---- the model -----------------------------------------------------------------------------------
def run_order(cfg):
    """``(layer, pass that begins in front of it or None)`` in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for p in range(loop["times"]):
        order += [(i, p if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, dtype=torch.float64, return_layers=False, round_inputs=None):
    """Logits ``[T, vocab]`` of one sequence (and the stream after every run of a layer).  ``round_inputs``: a dtype
    through which every activation that passes from one matrix product to the next is rounded on its way (the
    sublayers' inputs, projected queries, keys, values and gates, gated heads, hidden features), as a run that keeps
    such activations in that dtype does: a measure of how far rounding alone moves a row.  Sums, norms, states and
    scores stay as they are."""
    global ROUND
    if round_inputs is not None and ROUND is None:
        ROUND = round_inputs
        try:
            return forward(cfg, w, tokens, dtype, return_layers, round_inputs)
        finally:
            ROUND = None
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x0 = rms_norm(w["embed"][ids], w["embed.norm"], eps)
    x = x0.clone()
    side = cfg.get("token_side")
    after = []

    def rounded(h):
        return h if round_inputs is None else h.to(round_inputs).to(dtype)
    for i, begins in run_order(cfg):
        if begins is not None:
            if begins > 0:
                x = x + x0
            x = x + w["loop.step"][begins]
        layer = cfg["layers"][i]
        p, m = f"l{i}.", layer["mixer"]
        h = rounded(rms_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "retention":
            y = retention_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "wkv":
            y = wkv_mixer(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = routed_experts(rounded(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.", layer["mlp"])
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if side is not None:
            x = x + token_side_input(x, ids, w, p + "side.", i, side["dim"], eps)
        after.append(x)
    logits = rounded(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, after) if return_layers else logits


def greedy(cfg, w, prompt, new_tokens, dtype=torch.float64):
    """The prompt's greedy continuation, every token from a whole pass over the sequence so far."""
    seq, out = list(prompt), []
    for _ in range(new_tokens):
        out.append(int(forward(cfg, w, seq, dtype)[-1].argmax()))
        seq.append(out[-1])
    return out
