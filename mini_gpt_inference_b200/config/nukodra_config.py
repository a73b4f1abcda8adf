"""Typed configuration of the Nukodra decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``streams`` (residual streams side by side), ``norm.eps`` and a
list ``layers``; each entry has ``type`` (the mixer's kind: ``attention``, ``latent_attention`` or
``mamba2``), ``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null for none).  Every
size and constant is read from the file; a missing key is an error, a key that this engine does not
know a warning.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .fakilorn_config import _keys, _number, _positive_int
from .model_config import ConfigError

MIXER_TYPES = ("attention", "latent_attention", "mamba2")
MAX_STREAMS = 8          # what the stream kernels hold in registers


def _rotation(raw, what: str, most: int) -> tuple[int, float]:
    """``rot``: how many features of a head turn with the position, and the base of their frequencies."""
    _keys(raw, ("base", "dims"), (), what)
    dims = raw["dims"]
    if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"{what}.dims must be an even number of 0..{most} features, got {dims!r}")
    base = _number(raw["base"], what + ".base")
    if base <= 0:
        raise ConfigError(f"{what}.base must be positive, got {base!r}")
    return dims, base


@dataclass(frozen=True)
class NukodraMixerConfig:
    """Sizes and constants of one mixer; fields that a kind does not have are None."""

    kind: str
    heads: int
    vdim: int                         # features of a value head
    dim: int | None = None            # attention kinds: features of a query or key head (the part that does not
                                      # turn, for latent attention)
    scale: float | None = None        # attention kinds: factor on q . k
    rot_dims: int | None = None       # attention kinds: features of a head that turn with the position
    rot_base: float | None = None
    kv_heads: int | None = None       # attention
    window: int | None = None         # attention: a query sees itself and the window - 1 tokens before it
    softcap: float | None = None      # attention: scores pass cap * tanh(s / cap)
    kv_rank: int | None = None        # latent attention: size of the cached latent
    rot_dim: int | None = None        # latent attention: size of the turning part of queries and of the shared key part
    kv_from: int | None = None        # latent attention: the layer whose latents this one reads (None: its own)
    conv: int | None = None           # mamba2: taps of the causal convolution
    groups: int | None = None         # mamba2: groups of heads that share B and C
    norm_groups: int | None = None    # mamba2: equal parts of the gated output that are RMS-normed apart
    state: int | None = None          # mamba2: rows of a head's state matrix

    @classmethod
    def from_dict(cls, kind: str, raw, what: str) -> "NukodraMixerConfig":
        if kind == "mamba2":
            _keys(raw, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), (), what)
            heads, groups = _positive_int(raw["heads"], what + ".heads"), _positive_int(raw["groups"], what + ".groups")
            vdim = _positive_int(raw["vdim"], what + ".vdim")
            parts = _positive_int(raw["norm_groups"], what + ".norm_groups")
            if heads % groups:
                raise ConfigError(f"{what}: heads ({heads}) must be a multiple of groups ({groups})")
            if (heads * vdim) % parts:
                raise ConfigError(f"{what}: {heads * vdim} features do not form {parts} equal parts")
            return cls(kind, heads, vdim, conv=_positive_int(raw["conv"], what + ".conv"), groups=groups,
                       norm_groups=parts, state=_positive_int(raw["state"], what + ".state"))
        if kind == "latent_attention":
            _keys(raw, ("heads", "dim", "vdim", "kv_rank", "rot_dim", "rot", "scale"), ("kv_from",), what)
            rot_dim = raw["rot_dim"]
            if not isinstance(rot_dim, int) or isinstance(rot_dim, bool) or rot_dim < 0 or rot_dim % 2:
                raise ConfigError(f"{what}.rot_dim must be an even number of features, got {rot_dim!r}")
            dims, base = _rotation(raw["rot"], what + ".rot", rot_dim)
            if dims != rot_dim:
                raise ConfigError(f"{what}: the turning part has {rot_dim} features, rot.dims says {dims}")
            source = raw.get("kv_from")
            if source is not None and (not isinstance(source, int) or isinstance(source, bool) or source < 0):
                raise ConfigError(f"{what}.kv_from must be a layer's number, got {source!r}")
            return cls(kind, _positive_int(raw["heads"], what + ".heads"), _positive_int(raw["vdim"], what + ".vdim"),
                       dim=_positive_int(raw["dim"], what + ".dim"), scale=_number(raw["scale"], what + ".scale"),
                       rot_dims=dims, rot_base=base, kv_rank=_positive_int(raw["kv_rank"], what + ".kv_rank"),
                       rot_dim=rot_dim, kv_from=source)
        _keys(raw, ("heads", "kv_heads", "dim", "vdim", "scale"), ("mask", "rot", "softcap"), what)
        heads = _positive_int(raw["heads"], what + ".heads")
        kv_heads = _positive_int(raw["kv_heads"], what + ".kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{what}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive_int(raw["dim"], what + ".dim")
        dims, base = _rotation(raw["rot"], what + ".rot", dim) if raw.get("rot") is not None else (0, 1.0)
        window = None
        if raw.get("mask") is not None:
            _keys(raw["mask"], ("size",), (), what + ".mask")
            window = _positive_int(raw["mask"]["size"], what + ".mask.size")
        cap = None
        if raw.get("softcap") is not None:
            cap = _number(raw["softcap"], what + ".softcap")
            if cap <= 0:
                raise ConfigError(f"{what}.softcap must be positive, got {cap!r}")
        return cls(kind, heads, _positive_int(raw["vdim"], what + ".vdim"), dim=dim,
                   scale=_number(raw["scale"], what + ".scale"), rot_dims=dims, rot_base=base, kv_heads=kv_heads,
                   window=window, softcap=cap)

    def to_dict(self) -> dict:
        if self.kind == "mamba2":
            return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                    "state": self.state, "vdim": self.vdim}
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.kind == "latent_attention":
            out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot": rot,
                                   "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
            if self.kv_from is not None:
                out["kv_from"] = self.kv_from
            return out
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": rot, "scale": self.scale,
               "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class NukodraFeedForwardConfig:
    kind: str                          # "dense"
    ff: int                            # hidden width

    @classmethod
    def from_dict(cls, raw, what: str) -> "NukodraFeedForwardConfig":
        if not isinstance(raw, Mapping) or "kind" not in raw:
            raise ConfigError(f"{what} must be an object with a 'kind'")
        if raw["kind"] != "dense":
            raise ConfigError(f"{what}.kind {raw['kind']!r} is not known (dense)")
        _keys(raw, ("kind", "ff"), (), what)
        return cls("dense", _positive_int(raw["ff"], what + ".ff"))

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": self.kind}


@dataclass(frozen=True)
class NukodraLayerConfig:
    type: str
    mixer: NukodraMixerConfig
    mlp: NukodraFeedForwardConfig | None

    @classmethod
    def from_dict(cls, raw, what: str) -> "NukodraLayerConfig":
        _keys(raw, ("type", "mixer"), ("mlp",), what)
        if raw["type"] not in MIXER_TYPES:
            raise ConfigError(f"{what}.type {raw['type']!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
        mlp = raw.get("mlp")
        return cls(raw["type"], NukodraMixerConfig.from_dict(raw["type"], raw["mixer"], what + ".mixer"),
                   None if mlp is None else NukodraFeedForwardConfig.from_dict(mlp, what + ".mlp"))

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class NukodraConfig:
    vocab: int
    width: int
    layers: tuple[NukodraLayerConfig, ...]
    norm_eps: float
    streams: int | None = None         # residual streams side by side; None: one stream and plain residual sums
    architecture: str = "Nukodra"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], architecture: str | None = None) -> "NukodraConfig":
        _keys(raw, ("vocab", "width", "layers", "norm"),
              ("streams", "architecture", "architectures", "model_type", "dtype", "torch_dtype"), "config.json")
        _keys(raw["norm"], ("eps",), (), "norm")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one layer")
        layers = tuple(NukodraLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(raw["layers"]))
        eps = _number(raw["norm"]["eps"], "norm.eps")
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps!r}")
        streams = raw.get("streams")
        if streams is not None:
            streams = _positive_int(streams, "streams")
            if streams > MAX_STREAMS:
                raise ConfigError(f"streams: at most {MAX_STREAMS}, got {streams}")
        for i, layer in enumerate(layers):
            m = layer.mixer
            if m.kv_from is None:
                continue
            src = layers[m.kv_from].mixer if m.kv_from < i else None
            if src is None or src.kind != "latent_attention" or src.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from: layer {m.kv_from} is not an earlier latent-attention "
                                  "layer with latents of its own")
            if (src.kv_rank, src.rot_dim, src.rot_base) != (m.kv_rank, m.rot_dim, m.rot_base):
                raise ConfigError(f"layers[{i}].mixer: its latents' sizes and rotation differ from layer {m.kv_from}'s")
        return cls(_positive_int(raw["vocab"], "vocab"), _positive_int(raw["width"], "width"), layers, eps, streams,
                   architecture or "Nukodra")

    @classmethod
    def from_json(cls, path: str | Path) -> "NukodraConfig":
        from .model_config import read_config_json

        path = Path(path)
        return cls.from_dict(read_config_json(path / "config.json" if path.is_dir() else path))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    def num_parameters(self) -> int:
        c = self.width
        per_sublayer = 0 if self.streams is None else 2 * self.streams + self.streams ** 2
        total = self.vocab * c + c
        for layer in self.layers:
            m = layer.mixer
            total += c + per_sublayer
            if m.kind == "attention":
                q, kv = m.heads * m.dim, m.kv_heads * m.dim
                total += (q + kv + m.kv_heads * m.vdim) * (c + 1) + q + kv + m.heads + 2 * m.heads * m.vdim * c
            elif m.kind == "latent_attention":
                total += m.heads * (m.dim + m.rot_dim) * c + m.heads * (m.dim + m.vdim) * m.kv_rank + 2 * m.heads * m.vdim * c
                if m.kv_from is None:
                    total += (m.kv_rank + m.rot_dim) * c + m.kv_rank
            else:
                inner, bc = m.heads * m.vdim, 2 * m.groups * m.state
                total += (2 * inner + bc + m.heads) * c + (inner + bc) * (m.conv + 1) + 3 * m.heads + inner + c * inner
            if layer.mlp is not None:
                total += c + per_sublayer + 3 * c * layer.mlp.ff
        return total

    def save(self, model_dir: str | Path) -> Path:
        model_dir = Path(model_dir)
        model_dir.mkdir(parents=True, exist_ok=True)
        path = model_dir / "config.json"
        path.write_text(json.dumps(self.to_dict(), indent=1) + "\n")
        return path
