"""A layer's own token input: a slice of a second embedding table, gated by the residual stream.

The model has one table ``[vocab, layers * dim]`` (named by ``table_name``, shared by the layers: only the first part
built for it names it in the checkpoint); layer ``index`` owns columns ``index * dim .. (index + 1) * dim - 1``.
After the layer's sublayers, with ``x`` the stream and ``e`` the token's slice,

    g = gelu_tanh(W_gate x) * e;   y = W_proj g;   x += y / sqrt(mean(y^2) + eps) * norm

(``gate`` ``[dim, width]``, ``proj`` ``[width, dim]``, ``norm`` ``[width]``, a plain gain).  The gate's product reads the
stream in the compute dtype and writes 32-bit; the norm and the sum are 32-bit.
"""

from __future__ import annotations

from .base import SideInput, register_side_input
from .spec import TensorSpec


@register_side_input("token_side_input")
class TokenSideInput(SideInput):
    graph_safe = True      # launches kernels only; tokens fed back on the device are read there

    def __init__(self, prefix: str, width: int, vocab_size: int, dim: int, index: int, parts: int, eps: float,
                 table_name: str = "side.embed", owns_table: bool = False) -> None:
        super().__init__(prefix)
        self.width, self.vocab_size, self.dim, self.index, self.n_parts = width, vocab_size, dim, index, parts
        self.eps = float(eps)
        self.table_name, self.owns_table = table_name, bool(owns_table)
        self.table = self.gate = self.proj = self.norm = None

    def tensor_specs(self):
        p = self.prefix
        specs = {p + "gate": TensorSpec((self.dim, self.width), "matrix", "fan_in"),
                 p + "proj": TensorSpec((self.width, self.dim), "matrix", "fan_in"),
                 p + "norm": TensorSpec((self.width,), "vector", "norm_gain")}
        if self.owns_table:
            specs[self.table_name] = TensorSpec((self.vocab_size, self.n_parts * self.dim), "matrix", "unit_normal")
        return specs

    def bind(self, tensors) -> None:
        p = self.prefix
        self.table = tensors.get(self.table_name)
        self.gate, self.proj, self.norm = tensors.get(p + "gate"), tensors.get(p + "proj"), tensors.get(p + "norm")

    def forward(self, ctx, residual32) -> None:
        ctx.ops.token_side_residual(ctx, residual32, self.gate, self.proj, self.norm, self.table, self.index * self.dim,
                                    self.eps, ctx.act_dtype)
