"""A gated recurrence whose gates read only the current token (minGRU), and two mixers side by side.

``min_gru``: ``z = sigmoid(W_z h + b_z)`` and ``u = W_x h + b_x`` of ``inner`` features each; the candidate is
``u + 1/2`` where ``u >= 0`` and ``sigmoid(u)`` below; feature by feature ``s_t = (1 - z_t) s_(t-1) + z_t * candidate_t``
from ``s = 0``; the output is ``W_o (s_t * silu(W_g h))``.  Tensors ``z``, ``z.b``, ``x``, ``x.b``, ``g``, ``o``.  The
three projections are one product that writes 32-bit (gates, candidate and state never pass through the compute
dtype); ``s`` lives in the request's state slot in 32-bit.

``parallel_mixers``: two mixers read the same input; the result is ``left_scale * left + right_scale * right``.  Each
child is any registered mixer, named with its parameters; their tensors sit under ``left.`` and ``right.``.  One child
may keep pages and the other a state tensor: the layer then keeps both (``PagedKVWithStateSpec``).
"""

from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec, PagedKVSpec, PagedKVWithStateSpec
from .base import MIXERS, Mixer, register_mixer
from .spec import PartSpec, TensorSpec


@register_mixer("min_gru")
class MinGRU(Mixer):
    graph_safe = True      # launches kernels only; the state slot and the token counts are read on the device
    accepts_deferred_norm = True

    def __init__(self, prefix: str, width: int, inner: int, position=None) -> None:
        super().__init__(prefix)
        self.width, self.inner = width, inner
        self.fused_weight = self.fused_bias = self.out_weight = None

    def tensor_specs(self):
        p, c, n = self.prefix, self.width, self.inner
        return {p + "z": TensorSpec((n, c), "matrix", "fan_in"), p + "z.b": TensorSpec((n,), "vector", "unit_normal"),
                p + "x": TensorSpec((n, c), "matrix", "fan_in"), p + "x.b": TensorSpec((n,), "vector", "norm_shift"),
                p + "g": TensorSpec((n, c), "matrix", "fan_in"),
                p + "o": TensorSpec((c, n), "matrix", "fan_in_residual")}

    def bind(self, tensors) -> None:
        p = self.prefix
        rows = [tensors.get(p + n) for n in ("z", "x", "g")]
        if any(r is None for r in rows):
            return
        self.fused_weight = torch.cat(rows, dim=0).contiguous()
        self.fused_bias = torch.cat([tensors[p + "z.b"], tensors[p + "x.b"],
                                     torch.zeros_like(tensors[p + "z.b"])]).contiguous()
        self.out_weight = tensors[p + "o"]

    def cache_spec(self):
        return FixedStateSpec((self.inner,), "float32")

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        pre = ops.linear(y, self.fused_weight, self.fused_bias, "none", torch.float32)          # [z | u | g]
        out = ops.gated_recurrence(ctx, pre, 0, self.inner, 2 * self.inner, self.inner, cache.state, 0, ctx.act_dtype)
        ops.linear_residual(out, self.out_weight, None, residual32)


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):

    def __init__(self, prefix: str, left: dict, right: dict, left_scale: float = 1.0, right_scale: float = 1.0,
                 position=None) -> None:
        super().__init__(prefix)
        self.scales = (float(left_scale), float(right_scale))
        self.children = [MIXERS.build(PartSpec(c["kind"], c["params"], name), prefix, position=position)
                         for name, c in (("left", left), ("right", right))]
        self.graph_safe = all(getattr(c, "graph_safe", False) for c in self.children)
        # a norm that both sides can take into their first projection is handed on as it is: in steps of few tokens it
        # rides in both projections' prologues, in longer ones it runs once (a deferred norm keeps its rows)
        self.accepts_deferred_norm = all(getattr(c, "accepts_deferred_norm", False) for c in self.children)

    def tensor_specs(self):
        specs = {}
        for child in self.children:
            specs.update(child.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        for child in self.children:
            child.bind(tensors)

    def plan_step(self, batch, plan, ops) -> None:
        for child in self.children:
            child.plan_step(batch, plan, ops)

    def cache_spec(self):
        specs = [s for s in (c.cache_spec() for c in self.children) if s is not None]
        if len(specs) <= 1:
            return specs[0] if specs else None
        pages = [s for s in specs if isinstance(s, PagedKVSpec)]
        states = [s for s in specs if isinstance(s, FixedStateSpec)]
        if len(pages) != 1 or len(states) != 1:
            raise ValueError(f"{self.prefix}: of two mixers side by side one may keep pages and one a state tensor")
        return PagedKVWithStateSpec(pages[0], states[0])

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        rows, width = residual32.shape
        outs, own = [], True
        for index, child in enumerate(self.children):
            zeros = ops.zeros32(rows, width, ctx, 1 + index)           # (buffer 0 is the layer arrangement's)
            held = child.forward(ctx, cache, y, zeros)
            own = own and held is None
            outs.append(zeros if held is None else held)
        ops.scaled_sum_(residual32, outs[0], self.scales[0], outs[1], self.scales[1], clear=own)
