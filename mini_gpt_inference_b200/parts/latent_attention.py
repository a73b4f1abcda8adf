"""Causal attention whose keys and values are made from one small latent per token.

``q = W_q h`` gives every head ``head_dim`` features that do not turn and ``rot_dim`` that turn with the
position (rotary; feature ``i`` pairs with ``i + rot_dim / 2``, angle ``position * rot_base ** (-2 i / rot_dim)``).
``W_dkv h`` has ``kv_rank + rot_dim`` numbers: the first ``kv_rank``, RMS-normed with a gain, are the latent
``c``; the last ``rot_dim``, turned, are one key part that all heads share.  Head ``a``'s key is
``[W_uk,a c | shared part]``, its value ``W_uv,a c``, its score ``scale * (q_plain . k_plain + q_rot . k_rot)``;
softmax over positions up to the query's own; the concatenated heads times ``sigmoid(W_g h)``, then ``W_o``.

Only ``[c | shared part]`` is cached, one row per token whatever the number of heads.  Scores are taken
against those rows themselves: a query's plain part is first carried into the latent's space with its head's
key matrix, ``q_abs = W_uk,a^T q_plain`` (so ``q_abs . c = q_plain . (W_uk,a c)``), attention then runs with one
shared key head of ``kv_rank + rot_dim`` features whose first ``kv_rank`` are also the values, and the heads'
weighted latents are carried to value space with ``W_uv,a`` afterwards.  A layer with ``kv_source`` has no
``W_dkv``: it reads the rows that an earlier layer cached (the run order hands it that layer's cache, read-only),
with matrices, queries and everything else of its own.
"""

from __future__ import annotations

import torch

from ..cache.spec import PagedKVSpec
from .base import Mixer, register_mixer
from .spec import TensorSpec

_DEFAULT_NAMES = {"q": "q", "down": "dkv", "norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "out": "o"}


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step
    accepts_deferred_norm = True

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int,
                 scale: float, eps: float, rot_base: float = 10000.0, gate: bool = True, own_latents: bool = True,
                 cache_page_tokens: int | None = None, cache_pages: int | None = None, names: dict | None = None,
                 init: str = "normal", position=None) -> None:
        super().__init__(prefix)
        if rot_dim < 0 or rot_dim % 2:
            raise ValueError(f"rot_dim {rot_dim}: an even number of features")
        self.width, self.n_head, self.head_dim, self.rot_dim = width, n_head, head_dim, rot_dim
        self.v_head_dim, self.kv_rank = v_head_dim, kv_rank
        self.scale, self.eps, self.rot_base = float(scale), float(eps), float(rot_base)
        self.has_gate, self.own_latents = bool(gate), bool(own_latents)
        self.cache_page_tokens, self.cache_pages = cache_page_tokens, cache_pages
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self._init = init
        self.q_width = n_head * (head_dim + rot_dim)
        self.low_width = kv_rank + rot_dim if self.own_latents else 0
        self.o_width = n_head * v_head_dim
        self.low_off, self.g_off = self.q_width, self.q_width + self.low_width
        self.row_dim = kv_rank + rot_dim                 # a cache row, and a query head as the attention sees it
        self.fused_weight = self.out_weight = self.up_k = self.up_v = self.latent_gain = self.freq = None

    def _name(self, which: str) -> str:
        return self.prefix + self.names[which]

    def tensor_specs(self):
        init, init_out = self._init, ("residual_proj" if self._init == "normal" else self._init + "_residual")
        specs = {
            self._name("q"): TensorSpec((self.q_width, self.width), "matrix", init),
            self._name("up_k"): TensorSpec((self.n_head * self.head_dim, self.kv_rank), "matrix", "fan_in"),
            self._name("up_v"): TensorSpec((self.o_width, self.kv_rank), "matrix", "fan_in"),
            self._name("out"): TensorSpec((self.width, self.o_width), "matrix", init_out),
        }
        if self.own_latents:
            specs[self._name("down")] = TensorSpec((self.low_width, self.width), "matrix", init)
            specs[self._name("norm")] = TensorSpec((self.kv_rank,), "vector", "norm_gain")
        if self.has_gate:
            specs[self._name("gate")] = TensorSpec((self.o_width, self.width), "matrix", init)
        return specs

    def bind(self, tensors) -> None:
        rows = [tensors.get(self._name("q"))]
        if self.own_latents:
            rows.append(tensors.get(self._name("down")))
        if self.has_gate:
            rows.append(tensors.get(self._name("gate")))
        # one matrix for the step's one projection [q | low | g]: a layout made once, when the weights arrive
        self.fused_weight = torch.cat(rows, dim=0).contiguous() if all(r is not None for r in rows) else None
        self.out_weight = tensors.get(self._name("out"))
        self.up_k, self.up_v = tensors.get(self._name("up_k")), tensors.get(self._name("up_v"))
        self.latent_gain = tensors.get(self._name("norm")) if self.own_latents else None
        if self.rot_dim and self.out_weight is not None:
            freq = [self.rot_base ** (-2.0 * i / self.rot_dim) for i in range(self.rot_dim // 2)]
            self.freq = torch.tensor(freq, dtype=torch.float64).to(dtype=torch.float32, device=self.out_weight.device)

    def cache_spec(self):
        """One key head of ``kv_rank + rot_dim`` features per token; its first ``kv_rank`` are the values.  (A layer
        that reads another layer's rows is never asked: the run order names that layer's cache entry.)"""
        if not self.own_latents:
            return None
        return PagedKVSpec(1, self.row_dim, None, self.cache_page_tokens, self.cache_pages, self.kv_rank,
                           values_in_keys=True)

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if cache is None:
            raise RuntimeError(f"{self.prefix}: no cache entry holds the latents this layer reads")
        proj = ops.linear(y, self.fused_weight, None, "none", ctx.act_dtype)
        # queries as the attention sees them: per head [W_uk^T q_plain | turned q_rot]
        q = ops.latent_prepare(proj, self.n_head, 0, self.head_dim, self.rot_dim, self.low_off, self.kv_rank,
                               self.latent_gain, self.eps, self.freq, cache if self.own_latents else None,
                               ctx.slot_mapping[cache.group], ctx.positions)
        ops.head_linear(proj, 0, self.head_dim + self.rot_dim, self.up_k, True, self.n_head, self.head_dim, self.kv_rank,
                        out=q, out_off=0, out_head=self.row_dim)
        mixed = ops.paged_attention_general(q, self.n_head, 1, self.row_dim, self.kv_rank, self.scale, cache, ctx)
        gate = proj[:, self.g_off: self.g_off + self.o_width] if self.has_gate else None
        heads = ops.head_linear(mixed, 0, self.kv_rank, self.up_v, False, self.n_head, self.kv_rank, self.v_head_dim,
                                gate=gate)
        ops.linear_residual(heads, self.out_weight, None, residual32)
