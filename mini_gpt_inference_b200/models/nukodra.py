"""The Nukodra decoder as data: which part sits in which layer, and in which order layers run.

Token embedding without positions, copied into several residual streams; pre-norm layers (RMS norms with
gains stored around zero) whose sublayers read from and write to the streams through small learned
connections; a mixer per layer out of three: attention with grouped key heads, biases, a norm over the whole
query and key projections, rotary positions, capped scores, a sliding window, a sink in the softmax and an output
gate; attention over cached latents (a layer may read an earlier layer's latents); a Mamba-2 state-space mixer;
a gated silu feed-forward, or none; a final RMS norm over the summed streams and a head that shares the
embedding's matrix.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.hc1.*``, ``l<i>.norm2``,
``l<i>.mlp.*``, ``l<i>.hc2.*``, ``final.norm``.
"""

from __future__ import annotations

from ..config.nukodra_config import NukodraConfig
from ..config.registry import register_model
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _norm(cfg: NukodraConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "offset": 1.0, "weight_name": name}, "", "norm")


def _mixer(cfg: NukodraConfig, m) -> PartSpec:
    if m.kind == "mamba2":
        return PartSpec("state_space_duality", {
            "width": cfg.width, "n_head": m.heads, "v_head_dim": m.vdim, "state": m.state, "groups": m.groups,
            "taps": m.conv, "norm_groups": m.norm_groups, "eps": cfg.norm_eps}, "mix")
    if m.kind == "latent_attention":
        return PartSpec("latent_attention", {
            "width": cfg.width, "n_head": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
            "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "rot_base": m.rot_base, "gate": True,
            "own_latents": m.kv_from is None, "init": "fan_in"}, "mix")
    return PartSpec("gated_unit_attention", {
        "width": cfg.width, "n_head": m.heads, "n_kv_head": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
        "scale": m.scale, "eps": cfg.norm_eps, "unit_norm": True, "norm_weights": True, "norm_scope": "projection",
        "gate": True, "bias": ("q", "k", "v"), "window": m.window, "rot_dims": m.rot_dims, "rot_base": m.rot_base,
        "softcap": m.softcap, "sink": True, "init": "fan_in"}, "mix")


@register_model("Nukodra", "nukodra", config_class=NukodraConfig)
def describe_nukodra(cfg: NukodraConfig) -> ModelSpec:
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm1": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, layer.mixer)}
        many = cfg.streams is not None
        if many:
            parts["connection1"] = PartSpec("stream_connection", {"streams": cfg.streams}, "hc1")
        if layer.mlp is not None:
            parts["norm2"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = PartSpec("gated_mlp", {"width": cfg.width, "inner": layer.mlp.ff,
                                                           "activation": "silu"}, "mlp")
            if many:
                parts["connection2"] = PartSpec("stream_connection", {"streams": cfg.streams}, "hc2")
            arrangement = "multi_stream_pre_norm" if many else "pre_norm"
        else:
            arrangement = "multi_stream_mixer_only" if many else "pre_norm_mixer_only"
        layers.append(LayerSpec(p, parts, arrangement))
        # a layer that reads an earlier layer's latents runs against that layer's cache entry, read-only
        source = layer.mixer.kv_from
        order.append(LayerCall(i, i, True) if source is None else LayerCall(i, source, False))
    return ModelSpec(
        architecture=cfg.architecture,
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width, "tensor_name": "embed"}, ""),
        position=PartSpec("none", {}, ""),
        layers=tuple(layers),
        layer_order=tuple(order),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("tied_head", {"vocab_size": cfg.vocab, "width": cfg.width, "tied_to": "embed",
                                    "stored_again": False}, ""),
        streams=cfg.streams)
