"""A plain, slow Nukodra: one function per mechanism, whole sequences, float64 by default.

It takes the model as a config dict (the keys of ``config.json``) and a dict of tensors by their
checkpoint names, and shares no code with the engine.  Notation: ``X`` holds the residual streams
``[streams, T, width]`` of one sequence, ``h`` the input of a mixer or feed-forward, ``t`` a position.

* embedding:  ``E[tok_t]``, copied into every stream
* rms norm:   ``x / sqrt(mean(x^2) + eps) * (offset + w)``; offset 1 for the layers' norms and the
  final one, 0 for norms inside mixers
* streams:    ``u = sum_s a[s] X_s``; ``y = sublayer(norm(u))``; ``X'_t = sum_s M[s, t] X_s + b[t] y``
* rotation:   of the first ``n`` features of a head, feature ``i`` with ``i + n/2``, by ``t * base^(-2i/n)``
* attention:  grouped key heads, biases, one RMS norm over all query (key) features of a token, rotation,
  ``cap * tanh(scale * q.k / cap)``, a window, a sink in the softmax's denominator, a sigmoid gate
* latent attention: keys and values of every head made from one small latent per token plus one rotated
  key part that all heads share; a layer may read the latents of an earlier layer
* mamba2:     causal convolution and silu on ``[x | B | C]``, ``S_t = exp(-exp(A) dt) S_(t-1) + dt B x^T``,
  ``y = S^T C + D x``, times ``silu(z)``, RMS norm in equal parts
* dense ff:   ``W_down (silu(W_gate h) * W_up h)``
"""

from __future__ import annotations

import math

import torch


# ---- pieces --------------------------------------------------------------------------------------
def rms_norm(x, w, eps, offset=0.0):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * (offset + w)


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, n, base):
    """x: [T, heads, features]; the first n features of every head turn with the position."""
    if n == 0:
        return x
    half = n // 2
    freq = torch.tensor([base ** (-2.0 * i / n) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]             # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:n]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., n:]], dim=-1)


def streams_read(X, a):
    return torch.einsum("s,stc->tc", a, X)


def streams_write(X, M, b, y):
    return torch.einsum("sr,stc->rtc", M, X) + b[:, None, None] * y[None]


# ---- mixers --------------------------------------------------------------------------------------
def attention_mixer(h, w, p, m, eps):
    heads, groups, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = rms_norm(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.norm"], eps).view(T, heads, d)
    k = rms_norm(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.norm"], eps).view(T, groups, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, groups, dv)
    if m.get("rot") is not None:
        q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"])
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    if m.get("mask") is not None:
        seen = seen & (dist < m["mask"]["size"])
    cap = m.get("softcap")
    per = heads // groups
    out = torch.empty(T, heads, dv, dtype=h.dtype)
    for a in range(heads):
        s = (q[:, a] @ k[:, a // per].T) * m["scale"]
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, -math.inf)
        sink = w[p + "sink"][a]
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        out[:, a] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))) @ v[:, a // per]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, heads * dv) * gate) @ w[p + "o"].T


def latent_of(h, w, p, m, eps):
    """What a latent-attention layer keeps per token: the normed latent and the rotated key part."""
    T = h.shape[0]
    r = m["kv_rank"]
    low = h @ w[p + "dkv"].T
    c = rms_norm(low[:, :r], w[p + "dkv.norm"], eps)
    shared = rotate(low[:, None, r:], torch.arange(T), m["rot_dim"], m["rot"]["base"])[:, 0]
    return c, shared


def latent_attention_mixer(h, w, p, m, eps, latent):
    """``latent``: (c, rotated key part) of this layer or of the layer it reads."""
    heads, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    c, shared = latent
    q = (h @ w[p + "q"].T).view(T, heads, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, dr, m["rot"]["base"])
    k_plain = (c @ w[p + "uk"].T).view(T, heads, d)
    v = (c @ w[p + "uv"].T).view(T, heads, dv)
    seen = pos[None, :] <= pos[:, None]
    out = torch.empty(T, heads, dv, dtype=h.dtype)
    for a in range(heads):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ shared.T) * m["scale"]
        s = s.masked_fill(~seen, -math.inf)
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, heads * dv) * gate) @ w[p + "o"].T


def causal_conv(x, taps, bias):
    """x: [T, channels]; taps: [channels, n], the last column weighs the current token."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    out = bias[None, :].expand(T, -1).clone()
    for j in range(n):
        out = out + padded[j: j + T] * taps[:, j][None, :]
    return out


def mamba2_mixer(h, w, p, m, eps):
    heads, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * dv
    T = h.shape[0]
    zxbcdt = h @ w[p + "in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner: 2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, heads, dv)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :] * dt)          # [T, heads]
    per = heads // G
    S = torch.zeros(heads, N, dv, dtype=h.dtype)
    y = torch.empty(T, heads, dv, dtype=h.dtype)
    for t in range(T):
        for a in range(heads):
            g = a // per
            S[a] = decay[t, a] * S[a] + dt[t, a] * B[t, g][:, None] * x[t, a][None, :]
            y[t, a] = S[a].T @ C[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---- the model -----------------------------------------------------------------------------------
def forward(cfg, w, tokens, dtype=torch.float64, return_layers=False):
    """Logits ``[T, vocab]`` of one sequence (and the summed streams after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["embed"][ids]
    many = cfg.get("streams") is not None
    X = x[None].repeat(cfg["streams"] if many else 1, 1, 1)
    one = torch.ones(1, dtype=dtype)

    def connection(name):
        # without streams: u = x, x <- x + y
        return (w[name + ".in"], w[name + ".mix"], w[name + ".out"]) if many else (one, one[None], one)
    latents = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        a, M, b = connection(p + "hc1")
        h = rms_norm(streams_read(X, a), w[p + "norm1"], eps, 1.0)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(h, w, p + "mix.", m, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, p + "mix.", m, eps)
                src = i
            y = latent_attention_mixer(h, w, p + "mix.", m, eps, latents[src])
        X = streams_write(X, M, b, y)
        if layer.get("mlp") is not None:
            a, M, b = connection(p + "hc2")
            h = rms_norm(streams_read(X, a), w[p + "norm2"], eps, 1.0)
            X = streams_write(X, M, b, dense_ff(h, w, p + "mlp."))
        after.append(X.sum(0))
    logits = rms_norm(X.sum(0), w["final.norm"], eps, 1.0) @ w["embed"].T
    return (logits, after) if return_layers else logits


def greedy(cfg, w, prompt, new_tokens, dtype=torch.float64):
    """The prompt's greedy continuation, every token from a whole pass over the sequence so far."""
    seq, out = list(prompt), []
    for _ in range(new_tokens):
        out.append(int(forward(cfg, w, seq, dtype)[-1].argmax()))
        seq.append(out[-1])
    return out
