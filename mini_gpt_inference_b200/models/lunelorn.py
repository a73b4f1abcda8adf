"""The Lunelorn decoder as data: which part sits in which layer, and in which order layers run.

Token embedding followed by an RMS norm; layers with a norm on both sides of each sublayer whose mixer is retention
(a matrix memory with one fixed decay per head), RWKV-style time mixing, or an attention with rotated, unit-norm
values beside a minGRU recurrence, and whose feed-forward is routed experts or none; behind the sublayers every
layer adds its own slice of a second token embedding, gated by the stream; a range of layers that runs several times
with the same weights, every pass with a cache or state of its own and, in front of it, the embedding's output
(from the second pass on) and a learned vector added to the stream; a final RMS norm, an untied head and a soft cap
on the logits.  Tensor names: ``embed``, ``embed.norm``, ``side.embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.lunelorn_config import LunelornConfig
from ..config.registry import register_model
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _norm(cfg: LunelornConfig, name: str, optional: bool = False) -> PartSpec:
    return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "offset": 0.0, "weight_name": name,
                                "optional": optional}, "", "norm")


def _mixer(cfg: LunelornConfig, m) -> PartSpec:
    if m.kind == "retention":
        return PartSpec("retention", {"width": cfg.width, "n_head": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                                      "decay": list(m.decay), "eps": cfg.norm_eps}, "mix")
    if m.kind == "wkv":
        return PartSpec("wkv", {"width": cfg.width, "n_head": m.heads, "head_dim": m.dim, "eps": cfg.norm_eps}, "mix")
    a = m.left
    left = {"kind": "gated_unit_attention", "params": {
        "width": cfg.width, "n_head": a.heads, "n_kv_head": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
        "scale": a.scale, "eps": cfg.norm_eps, "unit_norm": False, "gate": False, "rot_dims": a.rot_dims,
        "rot_base": a.rot_base, "value_unit_norm": True, "value_rot": True, "init": "fan_in"}}
    right = {"kind": "min_gru", "params": {"width": cfg.width, "inner": m.right_width}}
    return PartSpec("parallel_mixers", {"left": left, "right": right, "left_scale": m.left_scale,
                                        "right_scale": m.right_scale}, "mix")


@register_model("Lunelorn", "lunelorn", config_class=LunelornConfig)
def describe_lunelorn(cfg: LunelornConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm1": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, layer.mixer), "norm1b": _norm(cfg, p + "norm1b")}
        if layer.mlp is None:
            # (a checkpoint may still hold the feed-forward's norms of a layer without one)
            parts["norm2"] = _norm(cfg, p + "norm2", optional=True)
            parts["norm2b"] = _norm(cfg, p + "norm2b", optional=True)
        else:
            parts["norm2"], parts["norm2b"] = _norm(cfg, p + "norm2"), _norm(cfg, p + "norm2b")
            parts["feed_forward"] = PartSpec("routed_experts", {
                "width": cfg.width, "n_experts": layer.mlp.experts, "top": layer.mlp.top, "inner": layer.mlp.ff,
                "shared_inner": None, "init": "fan_in"}, "mlp")
        if cfg.side_dim is not None:
            parts["side_input"] = PartSpec("token_side_input", {
                "width": cfg.width, "vocab_size": cfg.vocab, "dim": cfg.side_dim, "index": i, "parts": len(cfg.layers),
                "eps": cfg.norm_eps, "table_name": "side.embed", "owns_table": i == 0}, "side")
        layers.append(LayerSpec(p, parts, "sandwich_norm"))
    # every run of a layer has a cache entry of its own; a pass of the loop begins with the re-entry step
    order = []
    for n, (i, loop_pass) in enumerate(cfg.run_order()):
        begins = loop_pass is not None and i == cfg.loop_start
        order.append(LayerCall(i, n, True, 0 if begins else None, loop_pass if begins else 0))
    entries = ()
    if cfg.loop_times:
        entries = (PartSpec("additive_reentry", {"width": cfg.width, "passes": cfg.loop_times}, "loop"),)
    return ModelSpec(
        architecture=cfg.architecture,
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width, "tensor_name": "embed",
                                               "norm_name": "embed.norm", "norm_eps": cfg.norm_eps,
                                               "init": "unit_normal"}, ""),
        position=PartSpec("none", {}, ""),
        layers=tuple(layers),
        layer_order=tuple(order),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "width": cfg.width, "tensor_name": "head",
                                      "softcap": cfg.logit_softcap}, ""),
        n_caches=len(order),
        entries=entries)
