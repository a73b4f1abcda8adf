"""Re-entry of a loop over layers: in front of pass ``p`` the residual stream becomes
``W [x ; x_emb] + step[p]``, ``x_emb`` being the embedding's output of the same token, ``W`` a
``[width, 2 width]`` matrix (the stream's columns first) and ``step`` a ``[passes, width]`` table.
The sum is 32-bit; the product runs in the compute dtype like any projection.

``additive_reentry`` has no matrix: in front of pass ``p`` the stream becomes ``x + x_emb + step[p]``, without
``x_emb`` for the first pass (``p = 0``), all 32-bit.
"""

from __future__ import annotations

from .base import StreamEntry, register_stream_entry
from .spec import TensorSpec


@register_stream_entry("embedding_reentry")
class EmbeddingReentry(StreamEntry):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, passes: int, matrix_name: str = "in",
                 step_name: str = "step") -> None:
        super().__init__(prefix)
        self.width, self.passes = width, passes
        self.matrix_name, self.step_name = self.prefix + matrix_name, self.prefix + step_name
        self.matrix = self.steps = None

    def tensor_specs(self):
        return {self.matrix_name: TensorSpec((self.width, 2 * self.width), "matrix", "fan_in"),
                self.step_name: TensorSpec((self.passes, self.width), "vector", "norm_shift")}

    def bind(self, tensors) -> None:
        self.matrix, self.steps = tensors.get(self.matrix_name), tensors.get(self.step_name)

    def forward(self, ctx, x32, embedded32, index: int):
        if not 0 <= index < self.passes:
            raise ValueError(f"{self.prefix}: pass {index} is outside 0..{self.passes - 1}")
        both = ctx.ops.concat_cast(x32, embedded32, ctx.act_dtype)
        return ctx.ops.linear(both, self.matrix, self.steps[index], "none", x32.dtype)


@register_stream_entry("additive_reentry")
class AdditiveReentry(StreamEntry):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, passes: int, step_name: str = "step") -> None:
        super().__init__(prefix)
        self.width, self.passes = width, passes
        self.step_name = self.prefix + step_name
        self.steps = None

    def tensor_specs(self):
        return {self.step_name: TensorSpec((self.passes, self.width), "vector", "norm_shift")}

    def bind(self, tensors) -> None:
        self.steps = tensors.get(self.step_name)

    def forward(self, ctx, x32, embedded32, index: int):
        if not 0 <= index < self.passes:
            raise ValueError(f"{self.prefix}: pass {index} is outside 0..{self.passes - 1}")
        return ctx.ops.add_rows(x32, embedded32 if index > 0 else None, self.steps[index])
