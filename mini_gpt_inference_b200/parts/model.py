"""A decoder put together from a ``ModelSpec``.

The reference's forward (src/minigpt_infer/model.py:152-187): embed, run the blocks,
final norm, head.  Differences that matter: the order of layers is the spec's list, the
final norm and the head run only on the rows whose logits are wanted (a norm over rows is
row-wise, so selecting first changes nothing), and logits are 32-bit.
"""

from __future__ import annotations

from typing import Any, Mapping

from .base import (ARRANGEMENTS, CONNECTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                   POSITION_ENCODINGS, SIDE_INPUTS, STREAM_ENTRIES)
from .block import Layer, stream_after
from .spec import ModelSpec, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding, "")
        self.position = POSITION_ENCODINGS.build(spec.position, "")
        self.layers: list[Layer] = []
        for layer_spec in spec.layers:
            p = layer_spec.prefix
            parts, roles = {}, {}
            for name, part_spec in layer_spec.parts.items():
                role = roles[name] = layer_spec.role_of(name)
                if role == "mixer":
                    parts[name] = MIXERS.build(part_spec, p, position=self.position)
                else:
                    registry = {"norm": NORMS, "feed_forward": FEED_FORWARDS, "connection": CONNECTIONS,
                                "side_input": SIDE_INPUTS}[role]
                    parts[name] = registry.build(part_spec, p)
            self.layers.append(Layer(parts, roles, ARRANGEMENTS.get(layer_spec.arrangement), p))
        self.entries = [STREAM_ENTRIES.build(entry, "") for entry in spec.entries]
        self.final_norm = NORMS.build(spec.final_norm, "")
        self.head = HEADS.build(spec.head, "", embedding=self.embedding)
        self.layer_order = spec.layer_order
        # Cache entries: the ones the run order names (one per layer unless the spec says otherwise),
        # then one for the embedding if it keeps something per request.
        self._layer_of_cache: dict[int, int] = {}
        for call in spec.layer_order:
            self._layer_of_cache.setdefault(call.cache_layer, call.layer)
        self.embedding_cache = spec.num_caches if self._embedding_cache_spec() is not None else None

    # ---- tensors ----------------------------------------------------------------------
    def parts(self) -> list[Any]:
        out = [self.embedding, self.position]
        for layer in self.layers:
            out.extend(layer.parts())
        out.extend(self.entries)
        out.extend([self.final_norm, self.head])
        return out

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for part in self.parts():
            for name, spec in part.tensor_specs().items():
                if name in specs:
                    raise ValueError(f"two parts claim the tensor {name!r}")
                specs[name] = spec
        return specs

    def bind(self, tensors: Mapping[str, Any]) -> None:
        for part in self.parts():
            part.bind(tensors)

    @property
    def max_positions(self) -> int | None:
        return self.position.max_positions

    def _embedding_cache_spec(self):
        spec = getattr(self.embedding, "cache_spec", None)
        return spec() if spec is not None else None

    def cache_specs(self) -> list[Any]:
        """What each cache entry keeps per request: the wish of the layer that runs against it (an
        entry that no call names keeps nothing), then the embedding's, if it has one."""
        specs = [self.layers[self._layer_of_cache[c]].cache_spec() if c in self._layer_of_cache else None
                 for c in range(self.spec.num_caches)]
        if self.embedding_cache is not None:
            specs.append(self._embedding_cache_spec())
        return specs

    # ---- one step ------------------------------------------------------------------------
    def forward(self, ctx):
        """Run ``ctx``'s tokens; return 32-bit logits ``[len(ctx.logit_rows), vocab]``."""
        if getattr(ctx, "shared", None) is not None:
            ctx.shared.clear()
        if self.embedding_cache is not None:
            x = self.embedding.forward(ctx, self.position, ctx.cache_view(self.embedding_cache, True))
        else:
            x = self.embedding.forward(ctx, self.position)
        # layers add into the stream in place: what a stream entry wants of the embedding's output is a copy
        x_embedded = ctx.ops.clone(x) if self.entries else None
        if self.spec.streams is not None:
            x = ctx.ops.streams_spread(x, self.spec.streams)          # [streams, tokens, width]
        for call in self.layer_order:
            layer = self.layers[call.layer]
            if call.enter is not None:
                x = self.entries[call.enter].forward(ctx, x, x_embedded, call.enter_index)
            x = stream_after(layer.run(ctx, layer, ctx.cache_view(call.cache_layer, call.writes_cache), x), x)
        if ctx.logit_rows.numel() == 0:
            return None
        if self.spec.streams is not None:
            x = ctx.ops.streams_sum(x)
        if getattr(self.head, "accepts_deferred_norm", False):
            return self.head.forward(ctx, self.final_norm.defer(ctx, x, ctx.logit_rows))
        rows = ctx.ops.gather_rows(x, ctx.logit_rows)
        return self.head.forward(ctx, self.final_norm.forward(ctx, rows))
