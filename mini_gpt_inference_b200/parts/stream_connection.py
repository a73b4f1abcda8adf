"""Several residual streams side by side, and the layer arrangements that use them.

Instead of one residual stream ``x`` the model carries ``S`` streams ``x_0 .. x_(S-1)``, all equal to the
embedding's output at the start and summed in front of the final norm.  A sublayer has a connection with three
small tensors: ``in`` ``[S]``, ``out`` ``[S]`` and ``mix`` ``[S, S]`` (indexed ``[from, to]``):

    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x'_t = sum_s mix[s, t] x_s + out[t] y   (all t from the old x)

which takes the place of the residual sum ``x += sublayer(norm(x))``.  The streams are one 32-bit tensor
``[S, tokens, width]``; all of this is 32-bit.  Mixers and feed-forwards stay as they are: they add their output
into the tensor they are given as the residual stream, which here is a buffer of zeros that the connection's
read fills on its way, so what they leave there is ``y``.

Arrangements: ``multi_stream_pre_norm`` (``norm1``, ``mixer``, ``connection1``, ``norm2``, ``feed_forward``,
``connection2``) and ``multi_stream_mixer_only`` (the first three).  Where a layer has both sublayers, the write
of the first and the read of the second are one kernel.
"""

from __future__ import annotations

from .base import Part, register_arrangement, register_connection
from .block import _normed, stream_after
from .spec import TensorSpec


@register_connection("stream_connection")
class StreamConnection(Part):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, streams: int, names: dict | None = None) -> None:
        super().__init__(prefix)
        self.streams = int(streams)
        self.names = {"in": "in", "out": "out", "mix": "mix", **(names or {})}
        self.read_weights = self.write_weights = self.mix = None

    def tensor_specs(self):
        p, s, n = self.prefix, self.streams, self.names
        return {p + n["in"]: TensorSpec((s,), "vector", "norm_gain"),
                p + n["out"]: TensorSpec((s,), "vector", "norm_gain"),
                p + n["mix"]: TensorSpec((s, s), "vector", "near_identity")}

    def bind(self, tensors) -> None:
        p, n = self.prefix, self.names
        self.read_weights, self.write_weights = tensors.get(p + n["in"]), tensors.get(p + n["out"])
        self.mix = tensors.get(p + n["mix"])

    def read(self, ctx, streams32):
        """``(u, zeros)``: the sublayer's input before its norm, and the buffer it will add its output into."""
        return ctx.ops.streams_read(streams32, self.read_weights, want_zeros=True)

    def write(self, ctx, streams32, y32, then=None):
        """Mix the streams and add the sublayer's output (in place).  ``then``: the connection of the sublayer that
        follows; its read happens on the way and ``(u, zeros)`` for it is returned."""
        return ctx.ops.streams_write(streams32, self.mix, self.write_weights, y32,
                                     next_read=None if then is None else then.read_weights)


def _sublayer_mixer(ctx, layer, cache, u, zeros):
    return stream_after(layer.mixer.forward(ctx, cache, _normed(ctx, layer.norm1, layer.mixer, u), zeros), zeros)


def multi_stream_pre_norm(ctx, layer, cache, streams32):
    u, zeros = layer.connection1.read(ctx, streams32)
    y = _sublayer_mixer(ctx, layer, cache, u, zeros)
    u, zeros = layer.connection1.write(ctx, streams32, y, then=layer.connection2)
    ff = layer.feed_forward
    y = stream_after(ff.forward(ctx, _normed(ctx, layer.norm2, ff, u), zeros), zeros)
    layer.connection2.write(ctx, streams32, y)
    return None


multi_stream_pre_norm.requires = ("norm1", "mixer", "connection1", "norm2", "feed_forward", "connection2")
register_arrangement("multi_stream_pre_norm")(multi_stream_pre_norm)


def multi_stream_mixer_only(ctx, layer, cache, streams32):
    u, zeros = layer.connection1.read(ctx, streams32)
    layer.connection1.write(ctx, streams32, _sublayer_mixer(ctx, layer, cache, u, zeros))
    return None


multi_stream_mixer_only.requires = ("norm1", "mixer", "connection1")
register_arrangement("multi_stream_mixer_only")(multi_stream_mixer_only)
