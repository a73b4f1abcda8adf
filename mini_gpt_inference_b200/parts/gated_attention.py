"""Causal attention with unit-RMS queries and keys, an output gate and blended values.

One fused projection gives ``[q | k | v | g]`` of a token: ``n_head`` query heads and
``n_kv_head`` key heads of ``head_dim`` features, ``n_kv_head`` value heads of
``v_head_dim`` features (keys and values may differ in size) and, with ``gate``, one gate
value per output feature.  Then, per token:

* ``unit_norm``: every query and key head is divided by its root mean square,
  ``u / sqrt(mean(u^2) + eps)``, in 32-bit, without a gain;
* ``value_blend``: ``"source"`` publishes this layer's values for the layers after it,
  ``"blend"`` replaces ``v`` by ``(1 - t) v + t v_source`` with the published values of the
  same token and this layer's own scalar ``t``; the blended values are what the cache holds;
* keys and values go to their pages, and every query attends to the keys of its own request
  at positions up to its own, ``softmax(scale * q . k)`` in 32-bit, read from the pages
  whichever step brought them;
* ``gate``: the concatenated heads are multiplied by ``sigmoid(g)`` before the output
  projection, which adds into the residual stream.

Further variants, all parameters: ``bias`` (the q, k and output projections have biases, named after
their matrices with ``.b``); ``norm_weights`` (the unit-RMS query and key heads are multiplied by a
stored gain of ``head_dim`` numbers each, shared by the heads, named ``q.norm`` and ``k.norm``);
``values="keys"`` (there is no value projection: a token's values are its keys as projected, before
their norm); ``slope_rate`` (a distance bias: ``slope_h * (i - j)`` is taken off the score of query
``i`` and key ``j``, ``slope_h = 2 ** (-slope_rate * (h + 1) / n_head)``); ``block_mask`` (a query sees
only the keys of its own block of that many positions, blocks counted from position 0: the cache
gives back the pages of blocks that are over).

More variants, again parameters: ``bias`` may also name which of the projections have biases (a tuple out of
``"q"``, ``"k"``, ``"v"``, ``"out"``); ``norm_scope="projection"`` (one RMS norm over all query features of a
token at once and one over all key features, before they are split into heads, with gains of those whole sizes
named ``q.norm`` and ``k.norm``); ``rot_dims`` and ``rot_base`` (rotary positions: the first ``rot_dims`` features
of every query and key head turn with the token's position, feature ``i`` paired with ``i + rot_dims / 2``, by the
angle ``position * rot_base ** (-2 i / rot_dims)``, after the norm; the rest pass unchanged); ``softcap`` (a
score ``s``, scale included, becomes ``softcap * tanh(s / softcap)``); ``sink`` (a learned number per head, named
``sink``, whose exponential is added to the softmax's denominator: it has no key and no value and is neither
scaled nor capped); ``value_unit_norm`` (every value head is divided by its root mean square over its features,
without a gain, and cached so); ``value_rot`` (the value of position ``j``, after that norm, turns by ``j`` over all
its features, feature ``m`` paired with ``m + v_head_dim / 2``, angle ``j * rot_base ** (-2 m / v_head_dim)``, and is
cached so; every head's output at position ``i`` is turned back by ``-i`` before the gate and the output projection,
so that a value enters the sum turned by its distance to the query).

Positions do not enter otherwise unless the model's position encoding rotates q and k.  The four
matrices are stored apart in the checkpoint (``q``, ``k``, ``v``, ``g``, then ``o`` and the
scalar ``vmix``, under names given by ``names``) and joined once when they are bound.
"""

from __future__ import annotations

import math

import torch

from ..cache.spec import PagedKVSpec
from .base import Mixer, register_mixer
from .spec import TensorSpec

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "blend": "vmix"}
VALUE_SOURCE = "attention_value_source"     # key in ctx.shared


@register_mixer("gated_unit_attention")
class GatedUnitAttention(Mixer):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step
    accepts_deferred_norm = True

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, n_kv_head: int | None = None,
                 v_head_dim: int | None = None, scale: float | None = None, eps: float = 1e-6,
                 unit_norm: bool = True, gate: bool = True, value_blend: str | None = None,
                 blend_tensor: bool = False, window: int | None = None,
                 cache_page_tokens: int | None = None, cache_pages: int | None = None,
                 names: dict | None = None, position=None, bias: bool = False, norm_weights: bool = False,
                 values: str = "projected", slope_rate: float | None = None, block_mask: int | None = None,
                 init: str = "normal", norm_scope: str = "head", rot_dims: int = 0, rot_base: float = 10000.0,
                 softcap: float | None = None, sink: bool = False, value_unit_norm: bool = False,
                 value_rot: bool = False) -> None:
        super().__init__(prefix)
        self.width, self.n_head, self.head_dim = width, n_head, head_dim
        self.n_kv_head = n_head if n_kv_head is None else n_kv_head
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        if self.n_head % self.n_kv_head != 0:
            raise ValueError(f"n_head {n_head} is not a multiple of n_kv_head {self.n_kv_head}")
        if value_blend not in (None, "source", "blend"):
            raise ValueError(f"value_blend {value_blend!r}: None, 'source' or 'blend'")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.eps, self.unit_norm, self.has_gate = float(eps), bool(unit_norm), bool(gate)
        self.value_blend = value_blend
        # whether a layer that does not blend may still carry the scalar in its checkpoint
        self.has_blend_tensor = bool(blend_tensor)
        self.window = window
        if values not in ("projected", "keys"):
            raise ValueError(f"values {values!r}: 'projected' or 'keys'")
        if values == "keys" and (self.v_head_dim != head_dim or value_blend is not None):
            raise ValueError("values that are the keys have the keys' size and are not blended")
        if norm_weights and not unit_norm:
            raise ValueError("norm_weights without unit_norm")
        # which projections have biases: True means the queries', the keys' and the output's
        self.biased = ("q", "k", "out") if bias is True else tuple(bias or ())
        if any(b not in ("q", "k", "v", "out") for b in self.biased):
            raise ValueError(f"bias {bias!r}: True, or some of 'q', 'k', 'v', 'out'")
        if norm_scope not in ("head", "projection"):
            raise ValueError(f"norm_scope {norm_scope!r}: 'head' or 'projection'")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > head_dim:
            raise ValueError(f"rot_dims {rot_dims}: an even number of at most head_dim ({head_dim}) features")
        self.norm_scope, self.rot_dims, self.rot_base = norm_scope, int(rot_dims), float(rot_base)
        # queries and keys that turn with the position, or are normed across heads, go through another kernel
        self.value_unit_norm, self.value_rot = bool(value_unit_norm), bool(value_rot)
        if self.value_rot and self.v_head_dim % 2:
            raise ValueError(f"value_rot: value heads of {self.v_head_dim} features do not turn in pairs")
        if self.value_rot and gate:
            raise ValueError("value_rot: the heads are turned back before any gate; a gated output is not built")
        self.turns = self.rot_dims > 0 or norm_scope == "projection" or self.value_unit_norm or self.value_rot
        if self.turns and (value_blend is not None or values == "keys" or (unit_norm and not norm_weights
                                                                           and norm_scope == "projection")):
            raise ValueError("rotary positions and the projection-wide norm go with projected, unblended values "
                             "and with gains on the norm")
        if self.turns and unit_norm and norm_scope == "head":
            raise ValueError("rotary positions go with the projection-wide norm or with none")
        self.softcap = None if softcap is None else float(softcap)
        self.has_sink = bool(sink)
        self.has_bias, self.has_norm_weights, self.values_are_keys = bool(self.biased), bool(norm_weights), values == "keys"
        self.slope_rate = None if slope_rate is None else float(slope_rate)
        self.block_mask = block_mask
        self._init = init
        self.cache_page_tokens, self.cache_pages = cache_page_tokens, cache_pages
        self.position = position
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.q_width = n_head * head_dim
        self.k_width = self.n_kv_head * head_dim
        self.v_width = self.n_kv_head * self.v_head_dim
        self.o_width = n_head * self.v_head_dim
        self.k_off, self.v_off = self.q_width, self.q_width + self.k_width
        if self.values_are_keys:
            self.v_off, self.g_off = self.k_off, self.k_off + self.k_width
        else:
            self.g_off = self.v_off + self.v_width
        self.fused_weight = self.out_weight = self.blend = None
        self.fused_bias = self.out_bias = self.q_gain = self.k_gain = self.slopes = self.sinks = self.freq = None
        self.v_freq = None

    def _name(self, which: str) -> str:
        return self.prefix + self.names[which]

    def tensor_specs(self):
        init, init_out = self._init, ("residual_proj" if self._init == "normal" else self._init + "_residual")
        specs = {
            self._name("q"): TensorSpec((self.q_width, self.width), "matrix", init),
            self._name("k"): TensorSpec((self.k_width, self.width), "matrix", init),
            self._name("out"): TensorSpec((self.width, self.o_width), "matrix", init_out),
        }
        if not self.values_are_keys:
            specs[self._name("v")] = TensorSpec((self.v_width, self.width), "matrix", init)
        for which, size in (("q", self.q_width), ("k", self.k_width), ("v", self.v_width)):
            if which in self.biased:
                specs[self._name(which) + ".b"] = TensorSpec((size,), "vector", "norm_shift")
        if "out" in self.biased:
            specs[self._name("out") + ".b"] = TensorSpec((self.width,), "vector", "bias")
        if self.has_norm_weights:
            whole = self.norm_scope == "projection"
            specs[self._name("q") + ".norm"] = TensorSpec((self.q_width if whole else self.head_dim,), "vector", "norm_gain")
            specs[self._name("k") + ".norm"] = TensorSpec((self.k_width if whole else self.head_dim,), "vector", "norm_gain")
        if self.has_sink:
            specs[self.prefix + self.names.get("sink", "sink")] = TensorSpec((self.n_head,), "vector", "unit_normal")
        if self.has_gate:
            specs[self._name("gate")] = TensorSpec((self.o_width, self.width), "matrix")
        if self.value_blend is not None or self.has_blend_tensor:
            # a layer that does not blend may still find the scalar in its checkpoint, unused
            specs[self._name("blend")] = TensorSpec((), "vector", "unit_interval",
                                                    optional=self.value_blend is None)
        return specs

    def bind(self, tensors) -> None:
        rows = [tensors.get(self._name(w)) for w in (("q", "k") if self.values_are_keys else ("q", "k", "v"))]
        if self.has_gate:
            rows.append(tensors.get(self._name("gate")))
        # one matrix for the step's one projection: a layout made once, when the weights arrive
        self.fused_weight = torch.cat(rows, dim=0).contiguous() if all(r is not None for r in rows) else None
        self.out_weight = tensors.get(self._name("out"))
        if self.has_bias and self.fused_weight is not None:
            if any(b in self.biased for b in ("q", "k", "v")):
                self.fused_bias = torch.zeros(self.fused_weight.shape[0], dtype=torch.float32, device=self.fused_weight.device)
                for which, off, size in (("q", 0, self.q_width), ("k", self.k_off, self.k_width), ("v", self.v_off, self.v_width)):
                    if which in self.biased:
                        self.fused_bias[off: off + size] = tensors.get(self._name(which) + ".b")
            if "out" in self.biased:
                self.out_bias = tensors.get(self._name("out") + ".b")
        if self.has_sink:
            self.sinks = tensors.get(self.prefix + self.names.get("sink", "sink"))
        if self.rot_dims and self.out_weight is not None:
            # f_i = base^(-2 i / n), worked out in 64-bit and handed to the kernel as 32-bit numbers
            freq = [self.rot_base ** (-2.0 * i / self.rot_dims) for i in range(self.rot_dims // 2)]
            self.freq = torch.tensor(freq, dtype=torch.float64).to(dtype=torch.float32, device=self.out_weight.device)
        if self.value_rot and self.out_weight is not None:
            freq = [self.rot_base ** (-2.0 * m / self.v_head_dim) for m in range(self.v_head_dim // 2)]
            self.v_freq = torch.tensor(freq, dtype=torch.float64).to(dtype=torch.float32, device=self.out_weight.device)
        if self.has_norm_weights:
            self.q_gain, self.k_gain = tensors.get(self._name("q") + ".norm"), tensors.get(self._name("k") + ".norm")
        if self.slope_rate is not None and self.out_weight is not None:
            slopes = [2.0 ** (-self.slope_rate * (h + 1) / self.n_head) for h in range(self.n_head)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(dtype=torch.float32, device=self.out_weight.device)
        blend = tensors.get(self._name("blend")) if self.value_blend == "blend" else None
        self.blend = blend.reshape(1).contiguous() if blend is not None else None

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_head, self.head_dim, self.window, self.cache_page_tokens,
                           self.cache_pages,
                           None if self.v_head_dim == self.head_dim else self.v_head_dim, self.block_mask)

    def plan_step(self, batch, plan, ops) -> None:
        # where keys and values have one size, the kernel set may cut prompt portions into the tiles of
        # its tiled attention kernel (the same work list as the plain causal attention's)
        planner = getattr(ops, "plan_prompt_attention", None)
        if (planner is not None and self.head_dim == self.v_head_dim and self.slopes is None and self.block_mask is None
                and self.softcap is None and not self.has_sink):
            planner(batch, plan, self.n_head, self.n_kv_head, self.head_dim)

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        proj = ops.linear(y, self.fused_weight, self.fused_bias, "none", ctx.act_dtype)
        if self.position is not None:
            self.position.rotate(ctx, proj, self.n_head, self.n_kv_head, self.head_dim)
        other = blend = None
        if self.value_blend == "blend":
            other = ctx.shared.get(VALUE_SOURCE)
            if other is None:
                raise RuntimeError(f"{self.prefix}: no layer before this one published its values")
            if other.shape[1] != self.v_width:
                raise RuntimeError(f"{self.prefix}: the published values have another size")
            blend = self.blend
        elif self.value_blend == "source":
            ctx.shared[VALUE_SOURCE] = proj[:, self.v_off: self.v_off + self.v_width]
        extra = {"q_gain": self.q_gain, "k_gain": self.k_gain} if self.has_norm_weights else {}
        if self.value_unit_norm or self.value_rot:
            extra.update(v_unit_norm=self.value_unit_norm, v_freq=self.v_freq)
        if self.turns:
            ops.qk_norm_rotary(proj, self.n_head, self.n_kv_head, self.head_dim, self.v_head_dim, 0, self.k_off,
                               self.v_off, self.unit_norm, self.eps, self.rot_dims, self.freq, cache,
                               ctx.slot_mapping[cache.group], ctx.positions, **extra)
        else:
            ops.head_prepare(proj, self.n_head, self.n_kv_head, self.head_dim, self.v_head_dim, 0, self.k_off,
                             self.v_off, self.unit_norm, self.eps, cache, ctx.slot_mapping[cache.group],
                             ctx.positions, v_other=other, blend=blend, **extra)
        gate = proj[:, self.g_off: self.g_off + self.o_width] if self.has_gate else None
        extra = {}
        if self.slopes is not None:
            extra["slopes"] = self.slopes
        if self.block_mask is not None:
            extra["block"] = self.block_mask
        if self.softcap is not None:
            extra["softcap"] = self.softcap
        if self.sinks is not None:
            extra["sinks"] = self.sinks
        out = ops.paged_attention_general(proj, self.n_head, self.n_kv_head, self.head_dim, self.v_head_dim,
                                          self.scale, cache, ctx, gate=gate, **extra)
        if self.value_rot:
            ops.rotate_heads(out, self.n_head, self.v_head_dim, self.v_freq, ctx.positions, -1.0)
        ops.linear_residual(out, self.out_weight, self.out_bias, residual32)
