"""Typed configuration of the Lunelorn decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``, an optional ``loop`` (``start``, ``stop``,
``times``), an optional ``token_side`` (``dim``) and a list ``layers``; each entry has ``type`` (the mixer's kind:
``retention``, ``parallel`` or ``wkv``), ``mixer`` (its sizes and constants) and ``mlp`` (routed experts, or null for
none).  Every size and constant is read from the file; a missing key is an error, a key that this engine does not
know a warning.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .fakilorn_config import _keys, _number, _positive_int
from .model_config import ConfigError

MIXER_TYPES = ("retention", "parallel", "wkv")


@dataclass(frozen=True)
class LunelornAttentionConfig:
    """The attention side of a ``parallel`` mixer."""

    heads: int
    kv_heads: int
    dim: int                  # features of a query or key head
    vdim: int                 # features of a value head
    scale: float              # factor on q . k
    rot_dims: int             # features of a query or key head that turn with the position
    rot_base: float

    @classmethod
    def from_dict(cls, raw, what: str) -> "LunelornAttentionConfig":
        _keys(raw, ("heads", "kv_heads", "dim", "vdim", "scale", "rot"), (), what)
        _keys(raw["rot"], ("dims", "base"), (), what + ".rot")
        heads, kv_heads = _positive_int(raw["heads"], what + ".heads"), _positive_int(raw["kv_heads"], what + ".kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{what}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim, vdim = _positive_int(raw["dim"], what + ".dim"), _positive_int(raw["vdim"], what + ".vdim")
        dims = raw["rot"]["dims"]
        if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{what}.rot.dims must be an even number of at most dim ({dim}), got {dims!r}")
        if vdim % 2:
            raise ConfigError(f"{what}.vdim ({vdim}) must be even: the values turn in pairs")
        base = _number(raw["rot"]["base"], what + ".rot.base")
        if base <= 0:
            raise ConfigError(f"{what}.rot.base must be positive, got {base!r}")
        return cls(heads, kv_heads, dim, vdim, _number(raw["scale"], what + ".scale"), dims, base)

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class LunelornMixerConfig:
    """Sizes and constants of one mixer; fields that a kind does not have are None."""

    kind: str
    heads: int = 0                                    # retention, wkv
    dim: int = 0                                      # retention, wkv: features of a query / key head
    vdim: int = 0                                     # retention (wkv: equal to dim)
    decay: tuple[float, ...] | None = None            # retention: the fixed decay of every head
    left: LunelornAttentionConfig | None = None       # parallel
    right_width: int | None = None                    # parallel: features of the gated recurrence
    left_scale: float | None = None
    right_scale: float | None = None

    @classmethod
    def from_dict(cls, kind: str, raw, what: str) -> "LunelornMixerConfig":
        if kind == "retention":
            _keys(raw, ("heads", "dim", "vdim", "decay"), (), what)
            heads = _positive_int(raw["heads"], what + ".heads")
            decay = raw["decay"]
            if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                raise ConfigError(f"{what}.decay must list one decay per head ({heads}), got {decay!r}")
            decay = tuple(_number(a, f"{what}.decay[{i}]") for i, a in enumerate(decay))
            if not all(0.0 <= a <= 1.0 for a in decay):
                raise ConfigError(f"{what}.decay: every decay lies in 0..1, got {list(decay)!r}")
            return cls(kind, heads, _positive_int(raw["dim"], what + ".dim"), _positive_int(raw["vdim"], what + ".vdim"),
                       decay=decay)
        if kind == "wkv":
            _keys(raw, ("heads", "dim"), (), what)
            dim = _positive_int(raw["dim"], what + ".dim")
            return cls(kind, _positive_int(raw["heads"], what + ".heads"), dim, dim)
        _keys(raw, ("left", "right", "left_scale", "right_scale"), (), what)
        _keys(raw["right"], ("width",), (), what + ".right")
        return cls(kind, left=LunelornAttentionConfig.from_dict(raw["left"], what + ".left"),
                   right_width=_positive_int(raw["right"]["width"], what + ".right.width"),
                   left_scale=_number(raw["left_scale"], what + ".left_scale"),
                   right_scale=_number(raw["right_scale"], what + ".right_scale"))

    def to_dict(self) -> dict:
        if self.kind == "retention":
            return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.kind == "wkv":
            return {"dim": self.dim, "heads": self.heads}
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": {"width": self.right_width},
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class LunelornExpertsConfig:
    ff: int                   # hidden width of an expert
    experts: int
    top: int

    @classmethod
    def from_dict(cls, raw, what: str) -> "LunelornExpertsConfig":
        if not isinstance(raw, Mapping) or raw.get("kind") != "moe":
            raise ConfigError(f"{what} must be an object of kind 'moe', got {raw!r}")
        _keys(raw, ("kind", "expert", "router"), (), what)
        _keys(raw["expert"], ("ff",), (), what + ".expert")
        _keys(raw["router"], ("experts", "top"), (), what + ".router")
        experts, top = _positive_int(raw["router"]["experts"], what + ".router.experts"), _positive_int(raw["router"]["top"], what + ".router.top")
        if top > experts:
            raise ConfigError(f"{what}: top ({top}) exceeds experts ({experts})")
        return cls(_positive_int(raw["expert"]["ff"], what + ".expert.ff"), experts, top)

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class LunelornLayerConfig:
    type: str
    mixer: LunelornMixerConfig
    mlp: LunelornExpertsConfig | None

    @classmethod
    def from_dict(cls, raw, what: str) -> "LunelornLayerConfig":
        _keys(raw, ("type", "mixer"), ("mlp",), what)
        if raw["type"] not in MIXER_TYPES:
            raise ConfigError(f"{what}.type {raw['type']!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
        mlp = raw.get("mlp")
        return cls(raw["type"], LunelornMixerConfig.from_dict(raw["type"], raw["mixer"], what + ".mixer"),
                   None if mlp is None else LunelornExpertsConfig.from_dict(mlp, what + ".mlp"))

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class LunelornConfig:
    vocab: int
    width: int
    layers: tuple[LunelornLayerConfig, ...]
    norm_eps: float
    logit_softcap: float | None = None     # logits <- cap * tanh(logits / cap); None: as they are
    side_dim: int | None = None            # features of a layer's token input; None: the model has none
    loop_start: int = 0                    # layers loop_start .. loop_stop-1 run loop_times times in a row;
    loop_stop: int = 0                     # loop_times 0: the file names no loop
    loop_times: int = 0
    architecture: str = "Lunelorn"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], architecture: str | None = None) -> "LunelornConfig":
        _keys(raw, ("vocab", "width", "layers", "norm"),
              ("loop", "token_side", "logit_softcap", "architecture", "architectures", "model_type", "dtype", "torch_dtype"),
              "config.json")
        _keys(raw["norm"], ("eps",), (), "norm")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one layer")
        layers = tuple(LunelornLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(raw["layers"]))
        eps = _number(raw["norm"]["eps"], "norm.eps")
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps!r}")
        cap = raw.get("logit_softcap")
        if cap is not None:
            cap = _number(cap, "logit_softcap")
            if cap <= 0:
                raise ConfigError(f"logit_softcap must be positive, got {cap!r}")
        side = raw.get("token_side")
        if side is not None:
            _keys(side, ("dim",), (), "token_side")
            side = _positive_int(side["dim"], "token_side.dim")
        start = stop = times = 0
        loop = raw.get("loop")
        if loop is not None:
            _keys(loop, ("start", "stop", "times"), (), "loop")
            start, stop = loop["start"], loop["stop"]
            times = _positive_int(loop["times"], "loop.times")
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(layers)):
                raise ConfigError(f"loop: layers {start!r} .. {stop!r} are not a range of the {len(layers)} layers")
        return cls(_positive_int(raw["vocab"], "vocab"), _positive_int(raw["width"], "width"), layers, eps, cap, side,
                   start, stop, times, architecture or "Lunelorn")

    @classmethod
    def from_json(cls, path: str | Path) -> "LunelornConfig":
        from .model_config import read_config_json

        path = Path(path)
        return cls.from_dict(read_config_json(path / "config.json" if path.is_dir() else path))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop_times:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    def run_order(self) -> list[tuple[int, int | None]]:
        """``(layer, pass)`` in the order the layers run; ``pass`` is None outside the loop."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        order: list[tuple[int, int | None]] = [(i, None) for i in range(self.loop_start)]
        for p in range(self.loop_times):
            order += [(i, p) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, n)]

    def num_parameters(self) -> int:
        c = self.width
        total = 2 * self.vocab * c + 2 * c + self.loop_times * c
        if self.side_dim is not None:
            total += self.vocab * self.side_dim * len(self.layers)
        for layer in self.layers:
            m = layer.mixer
            total += 2 * c
            if m.kind == "retention":
                total += c * (2 * m.heads * m.dim + 3 * m.heads * m.vdim)
            elif m.kind == "wkv":
                n = m.heads * m.dim
                total += 5 * c + 5 * n * c + 3 * n        # plus the two decay matrices, whose rank the checkpoint gives
            else:
                a = m.left
                total += c * ((a.heads + a.kv_heads) * a.dim + a.kv_heads * a.vdim + a.heads * a.vdim)
                total += 4 * c * m.right_width + 2 * m.right_width
            if self.side_dim is not None:
                total += 2 * c * self.side_dim + c
            f = layer.mlp
            if f is not None:
                total += 2 * c + f.experts * (c + 3 * c * f.ff)
        return total

    def save(self, model_dir: str | Path) -> Path:
        model_dir = Path(model_dir)
        model_dir.mkdir(parents=True, exist_ok=True)
        path = model_dir / "config.json"
        path.write_text(json.dumps(self.to_dict(), indent=1) + "\n")
        return path
