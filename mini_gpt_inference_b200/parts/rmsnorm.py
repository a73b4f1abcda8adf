"""RMS norm over the width, statistics in 32-bit: ``y = x / sqrt(mean(x^2) + eps) * (offset + w)``.

``offset`` is 1 for a weight that is stored around zero, 0 for a plain gain.  ``weight_name``
names the tensor in the checkpoint where it is not ``<prefix>weight``.
"""

from __future__ import annotations

from .base import Norm, register_norm
from .spec import TensorSpec


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, eps: float, offset: float = 0.0,
                 weight_name: str | None = None, optional: bool = False) -> None:
        super().__init__(prefix)
        self.width, self.eps, self.offset = width, float(eps), float(offset)
        self.optional = bool(optional)     # a norm that a layer carries but never runs
        self.weight_name = weight_name if weight_name is not None else self.prefix + "weight"
        self.weight = None

    def tensor_specs(self):
        init = "norm_shift" if self.offset == 1.0 else "norm_gain"
        return {self.weight_name: TensorSpec((self.width,), "vector", init, optional=self.optional)}

    def bind(self, tensors) -> None:
        self.weight = tensors.get(self.weight_name)

    def forward(self, ctx, x32):
        return ctx.ops.rmsnorm(x32, self.weight, self.eps, self.offset, ctx.act_dtype)

    def add_normed(self, ctx, y32, residual32, clear=False):
        """``residual32 += norm(y32)`` in 32-bit, in place: the norm behind a sublayer.  ``clear``: ``y32`` is left
        as zeros (a buffer that the next sublayer adds into)."""
        return ctx.ops.rmsnorm_add(residual32, y32, self.weight, self.eps, self.offset, clear=clear)

    def defer(self, ctx, x32, rows=None):
        if not hasattr(ctx.ops, "defer_rmsnorm"):
            return super().defer(ctx, x32, rows)
        return ctx.ops.defer_rmsnorm(x32, self.weight, self.eps, self.offset, ctx.act_dtype, rows)
