"""Token embedding (plus the position table's rows, if the position encoding has one) and
the output head that shares its matrix.

``x = tok_emb[id] + pos_emb[pos]`` into the 32-bit residual stream
(src/minigpt_infer/model.py:183); ``logits = y @ tok_emb^T`` without bias, 32-bit out
(src/minigpt_infer/model.py:128-130, 187).  Both take a scale (1 unless given):
``x = scale * tok_emb[id] + ...`` and ``logits = scale * (y @ tok_emb^T)``; the head uses the
table as stored, without the embedding's scale.  ``tensor_name`` names the table in the
checkpoint where it is not ``<prefix>weight``.

``hashed_pair_embedding`` adds a row of a second table chosen by the token and the token before
it: row ``(previous * mul_prev + token * mul_cur) mod buckets``, and the table's last row
(number ``buckets``) for a sequence's first token.  The token before a step's first token is part
of the request's state: the embedding keeps it in a slot of the state pool.  ``linear_head`` is
an output projection with a matrix of its own.
"""

from __future__ import annotations

from ..cache.spec import FixedStateSpec
from .base import Part, register_embedding, register_head
from .spec import TensorSpec


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step
    # forward() honours ctx.token_source / ctx.fed_ids (tokens taken from the ids that the step
    # before sampled); an embedding without this flag gets its tokens gathered by a kernel in front.
    takes_token_source = True

    def __init__(self, prefix: str, vocab_size: int, width: int, scale: float = 1.0,
                 tensor_name: str | None = None, norm_name: str | None = None, norm_eps: float = 1e-6,
                 norm_offset: float = 0.0, init: str = "normal") -> None:
        super().__init__(prefix)
        self.vocab_size, self.width, self.scale = vocab_size, width, float(scale)
        self.tensor_name = tensor_name if tensor_name is not None else self.prefix + "weight"
        # an RMS norm over the embedded rows (32-bit in and out), its gain under ``norm_name``
        self.norm_name, self.norm_eps, self.norm_offset = norm_name, float(norm_eps), float(norm_offset)
        self._init = init
        self.weight = self.norm_weight = None

    def tensor_specs(self):
        specs = {self.tensor_name: TensorSpec((self.vocab_size, self.width), "matrix", self._init)}
        if self.norm_name is not None:
            specs[self.norm_name] = TensorSpec((self.width,), "vector", "norm_shift" if self.norm_offset == 1.0 else "norm_gain")
        return specs

    def bind(self, tensors) -> None:
        self.weight = tensors.get(self.tensor_name)
        if self.norm_name is not None:
            self.norm_weight = tensors.get(self.norm_name)

    def forward(self, ctx, position):
        table = position.table() if position is not None else None
        if getattr(ctx, "token_source", None) is not None:
            # some tokens are still on the device where the step before sampled them
            x = ctx.ops.embed(ctx.token_ids, ctx.positions, self.weight, table,
                              source=ctx.token_source, previous=ctx.fed_ids, **self._scale_arg())
        else:
            x = ctx.ops.embed(ctx.token_ids, ctx.positions, self.weight, table, **self._scale_arg())
        if self.norm_name is not None:
            x = ctx.ops.rmsnorm(x, self.norm_weight, self.norm_eps, self.norm_offset, x.dtype)
        return x

    def _scale_arg(self) -> dict:
        return {} if self.scale == 1.0 else {"scale": self.scale}


@register_head("tied_head")
class TiedHead(Part):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    """Output projection with the embedding's matrix.  A checkpoint may store it again
    under the head's own name; then it must equal the embedding."""

    def __init__(self, prefix: str, vocab_size: int, width: int, tied_to: str,
                 embedding=None, scale: float = 1.0, stored_again: bool = True) -> None:
        super().__init__(prefix)
        self.vocab_size, self.width, self.tied_to = vocab_size, width, tied_to
        self.embedding = embedding
        self.scale = float(scale)
        self.stored_again = stored_again      # whether a checkpoint may repeat the table under the head's name

    def tensor_specs(self):
        if not self.stored_again:
            return {}
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.width), "matrix",
                                                   optional_alias_of=self.tied_to)}

    accepts_deferred_norm = True

    def bind(self, tensors) -> None:
        return None

    def forward(self, ctx, y):
        greedy_out = getattr(ctx, "greedy_out", None)
        if greedy_out is not None:
            # the step also wants each row's greedy choice: the projection may take it on its way
            logits, ctx.greedy_taken = ctx.ops.logits(y, self.embedding.weight, greedy_out,
                                                      getattr(ctx, "greedy_vocab_limit", None), **self._scale_arg())
            return logits
        return ctx.ops.logits(y, self.embedding.weight, **self._scale_arg())

    def _scale_arg(self) -> dict:
        return {} if self.scale == 1.0 else {"scale": self.scale}


@register_embedding("hashed_pair_embedding")
class HashedPairEmbedding(Part):
    """``x = tok[id] + pair[row(previous id, id)] + pos[p]``; see the module's description."""

    graph_safe = True      # launches kernels only; the token before a step's first one is read on the device
    takes_token_source = True

    def __init__(self, prefix: str, vocab_size: int, width: int, buckets: int, mul_prev: int, mul_cur: int,
                 tensor_name: str | None = None, pair_name: str | None = None) -> None:
        super().__init__(prefix)
        self.vocab_size, self.width = vocab_size, width
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.tensor_name = tensor_name if tensor_name is not None else self.prefix + "weight"
        self.pair_name = pair_name if pair_name is not None else self.prefix + "pair.weight"
        self.weight = self.pair = None

    def tensor_specs(self):
        return {self.tensor_name: TensorSpec((self.vocab_size, self.width), "matrix", "unit_normal"),
                self.pair_name: TensorSpec((self.buckets + 1, self.width), "matrix", "unit_normal")}

    def bind(self, tensors) -> None:
        self.weight, self.pair = tensors.get(self.tensor_name), tensors.get(self.pair_name)

    def cache_spec(self):
        return FixedStateSpec((1,), "int32")        # the last token the request brought

    def forward(self, ctx, position, cache):
        table = position.table() if position is not None else None
        return ctx.ops.embed_pairs(ctx, self.weight, self.pair, table, self.buckets, self.mul_prev, self.mul_cur,
                                   cache.state, source=getattr(ctx, "token_source", None),
                                   previous=getattr(ctx, "fed_ids", None))


@register_head("linear_head")
class LinearHead(Part):
    """``logits = W y`` with a matrix of the head's own (no bias), 32-bit out; optionally ``softcap * tanh(logits /
    softcap)``."""

    graph_safe = True
    accepts_deferred_norm = True

    def __init__(self, prefix: str, vocab_size: int, width: int, tensor_name: str | None = None,
                 embedding=None, softcap: float | None = None) -> None:
        super().__init__(prefix)
        self.vocab_size, self.width = vocab_size, width
        # logits <- softcap * tanh(logits / softcap): monotonic, so a greedy choice taken on the way stays right
        self.softcap = None if not softcap else float(softcap)
        self.tensor_name = tensor_name if tensor_name is not None else self.prefix + "weight"
        self.weight = None

    def tensor_specs(self):
        return {self.tensor_name: TensorSpec((self.vocab_size, self.width), "matrix", "fan_in")}

    def bind(self, tensors) -> None:
        self.weight = tensors.get(self.tensor_name)

    def forward(self, ctx, y):
        greedy_out = getattr(ctx, "greedy_out", None)
        if greedy_out is not None:
            logits, ctx.greedy_taken = ctx.ops.logits(y, self.weight, greedy_out,
                                                      getattr(ctx, "greedy_vocab_limit", None))
        else:
            logits = ctx.ops.logits(y, self.weight)
        return logits if self.softcap is None else ctx.ops.softcap_(logits, self.softcap)
