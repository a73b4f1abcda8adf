from . import (attention, block, embedding, gated_attention, gated_recurrence, latent_attention, layernorm, loop_entry,  # noqa: F401  (register)
               matrix_memory, mlp, moe, positions, rmsnorm, stream_connection, token_side)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                   POSITION_ENCODINGS, FeedForward, Mixer, Norm, Part, PositionEncoding,
                   register_arrangement, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position_encoding,
                   register_stream_entry, STREAM_ENTRIES, StreamEntry)
from .context import HostBatch, StepContext, StepPlan
from .model import DecoderModel
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec, pre_norm_layer

__all__ = [n for n in dir() if not n.startswith("_")]
