"""Plain-data description of a model: which part sits where, and in which order layers run.

A ``ModelSpec`` is what an architecture's ``describe(config)`` returns.  It holds no
tensors and no code: parts are named by registry key (``kind``) with their sizes and
constants as ``params``; ``layer_order`` is a list, so a layer may run twice or use
another layer's cache.  ``parts.build`` turns it into runnable parts.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


ROLES = ("norm", "mixer", "feed_forward", "connection", "side_input")


@dataclass(frozen=True)
class PartSpec:
    kind: str                               # key in the part registry of its role
    params: Mapping[str, Any] = field(default_factory=dict)
    name: str = ""                          # weight-name prefix inside its parent ("ln1", "attn")
    role: str = ""                          # inside a layer: "norm" | "mixer" | "feed_forward" | "connection" | "side_input"; if empty,
                                            # taken from the part's name in the layer (see LayerSpec)


@dataclass(frozen=True)
class LayerSpec:
    """A layer is a bag of named parts and the name of the arrangement that wires them.  What
    names an arrangement expects is the arrangement's business (``pre_norm`` wants ``norm1``,
    ``mixer``, ``norm2``, ``feed_forward``); a layer with one norm, without a feed-forward or
    with two mixers is another arrangement over another bag, not another schema."""

    prefix: str                             # weight-name prefix of the layer ("blocks.0.")
    parts: Mapping[str, PartSpec]           # name in the layer -> part
    arrangement: str = "pre_norm"           # key in the block-arrangement registry

    def role_of(self, name: str) -> str:
        role = self.parts[name].role
        if not role:
            role = next((r for r in ROLES if name == r or name.startswith(r)), "")
        if role not in ROLES:
            raise ValueError(f"layer {self.prefix!r}: part {name!r} has no role; set PartSpec.role to "
                             f"one of {ROLES} or name it after its role")
        return role


def pre_norm_layer(prefix: str, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec,
                   feed_forward: PartSpec) -> LayerSpec:
    """The usual block: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))``."""
    return LayerSpec(prefix, {"norm1": norm1, "mixer": mixer, "norm2": norm2,
                              "feed_forward": feed_forward}, "pre_norm")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run ``layer`` against the cache entry ``cache_layer``.  By
    default the model has one cache entry per layer; a model whose layers run several times, each
    time with a cache or state of its own, names more (``ModelSpec.n_caches``).  ``enter``: index of
    a stream-entry part (``ModelSpec.entries``) that transforms the residual stream right before
    this call, with ``enter_index`` as its argument (the number of the pass that begins here)."""

    layer: int
    cache_layer: int
    writes_cache: bool = True
    enter: int | None = None
    enter_index: int = 0


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    width: int
    vocab_size: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    layer_order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    n_caches: int | None = None             # cache entries that layer_order names (None: one per layer)
    streams: int | None = None              # residual streams side by side (None: one stream, handed on as it is);
                                            # the embedding's output is copied into each, their sum feeds the final norm
    entries: tuple[PartSpec, ...] = ()      # stream-entry parts that layer_order's ``enter`` names

    @property
    def num_caches(self) -> int:
        return len(self.layers) if self.n_caches is None else self.n_caches

    def __post_init__(self) -> None:
        n = len(self.layers)
        owner: dict[int, int] = {}
        for call in self.layer_order:
            if not (0 <= call.layer < n and 0 <= call.cache_layer < self.num_caches):
                raise ValueError(f"layer_order entry {call} names a layer outside 0..{n - 1} or a cache "
                                 f"entry outside 0..{self.num_caches - 1}")
            if call.enter is not None and not 0 <= call.enter < len(self.entries):
                raise ValueError(f"layer_order entry {call} names a stream entry outside 0..{len(self.entries) - 1}")
            if self.n_caches is not None and owner.setdefault(call.cache_layer, call.layer) != call.layer:
                raise ValueError(f"cache entry {call.cache_layer} is used by two different layers")


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects in the checkpoint."""

    shape: tuple[int, ...]      # a dimension of -1 is taken from the checkpoint (see ``fill``)
    role: str = "matrix"        # "matrix": stored in the compute dtype; "vector": kept in 32-bit;
                                # "table": integer table kept as int32
    init: str = "normal"        # random-weights mode: "normal" | "residual_proj" | "norm_gain" |
                                # "norm_shift" | "bias" | "unit_interval" (a number in 0..1)
    optional_alias_of: str | None = None   # e.g. lm_head.weight may repeat tok_emb.weight
    optional: bool = False      # a checkpoint may hold it or not (a tensor the model never reads)
    fill: tuple[int, ...] | None = None    # the shape that random-weights mode gives a tensor with free dimensions

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(w in (-1, g) for w, g in zip(self.shape, shape))

    @property
    def init_shape(self) -> tuple[int, ...]:
        if -1 in self.shape:
            if self.fill is None:
                raise ValueError(f"a tensor of shape {self.shape} has no size to be made with")
            return tuple(self.fill)
        return tuple(self.shape)
