"""Typed descriptions of a decoder, one small record per part.

A model configuration (read from an architecture's own ``config.json`` keys)
is lowered into these records; the generic decoder in ``agave_b200.models``
builds parts from them through the part registries and never looks at the
architecture's name.  Every size and constant of a part is a field here, so
that two layers of one model may carry different mixers, feed-forwards,
windows or rotary bases.

The reference keeps the same facts as flat fields of one model struct
(src/models/gemma3.zig:59-85) and decides "local or global" per layer inside
the forward pass (src/models/gemma3.zig:736); here that decision is data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the key."""


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding on split halves (i, i + rotary_dim/2).

    angle(p, i) = (p / factor) * theta ** (-2 i / rotary_dim)
    (src/backend/kernels/cpu/rope.zig:11-47, src/models/gemma3.zig:884-902).
    """
    kind: str = "rotary"
    theta: float = 10000.0
    factor: float = 1.0
    rotary_dim: int = 0          # 0 means the whole head

    def key(self) -> Tuple:
        return (self.kind, float(self.theta), float(self.factor), int(self.rotary_dim))


@dataclass(frozen=True)
class NormSpec:
    """RMS norm; ``zero_centered`` stores w and applies (1 + w)
    (src/models/gemma3.zig:199-202,943-949)."""
    kind: str = "rmsnorm"
    eps: float = 1e-6
    zero_centered: bool = True


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a key/value cache.

    ``window`` None keeps every key; an integer W lets position p see the keys
    j with p - W < j <= p (src/models/gemma4.zig:1153-1155).  ``scale``
    multiplies the dot product (src/backend/kernels/cpu/sdpa.zig:58).
    """
    kind: str = "attention"
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None      # per-head norm of q and k, before the rotation
    position: Optional[RotarySpec] = None


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """down(act(gate x) * up x), dense (src/models/gemma3.zig:840-872)."""
    kind: str = "gated_dense"
    intermediate_size: int = 0
    activation: str = "gelu_tanh"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: a mixer and a feed-forward between norms.

    arrangement "sandwich": h += post(mixer(pre(h))); h += post(ffn(pre(h)))
    (src/models/gemma3.zig:708-709,824-826,835-836,876-878);
    arrangement "pre": the same without the two post norms.
    ``kind`` names the block class in the block registry; "sequential" is the
    class that runs the mixer and then the feed-forward, as above.  Another
    arrangement of parts (both branches from one norm, no feed-forward at all)
    is another block class under another kind, with a spec of its own if it
    needs other fields.
    """
    mixer: object = None
    feed_forward: object = None
    norm: NormSpec = NormSpec()
    arrangement: str = "sandwich"
    kind: str = "sequential"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be called twice);
    ``cache`` names the cache entry the mixer uses and ``writes_cache`` says
    whether this call appends to it (False: it reads what another call wrote).
    """
    block: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """The whole decoder as data."""
    hidden_size: int
    vocab_size: int
    embed_scale: float
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tie_embeddings: bool = True
    max_positions: int = 0
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    # a position encoding that is added to the stream after the embedding (a learned
    # table, say), by its kind in the stream-position registry; None: there is none
    stream_position: Optional[object] = None

    def n_cache_entries(self) -> int:
        return 1 + max(c.cache for c in self.schedule) if self.schedule else 0


def default_schedule(n_blocks: int) -> Tuple[LayerCall, ...]:
    return tuple(LayerCall(block=i, cache=i) for i in range(n_blocks))
