"""What every part declares, and the registries that build parts from specs.

A part is a mixer, a feed-forward, a norm or a position encoding.  It is
built from its own spec record (``agave_b200.config.base``) and the hidden
size; it never learns which model it sits in.  Each part class gives

* ``param_specs(spec, hidden_size) -> {local name: ParamSpec}`` (a class
  method, usable without a GPU: the loader and the random-weights writer need
  only this), and
* an instance with ``load(tensors)`` and ``forward(...)`` (see the part kinds
  below for the exact ``forward`` signature of each kind).

A block is the arrangement of such parts in one layer; it has a registry of
its own (``register_block``), so that an arrangement the library does not
have is added like a part.  A stream position is a position encoding that is
added to the residual stream right after the embedding (as opposed to one
that rotates q and k inside a mixer); it too is registered by kind.

Registries map ``spec.kind`` to the part class; registering under a new kind
is all that a new part needs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """Shape and role of one tensor of a part.

    role "matrix": a projection [out, in], kept in the compute dtype;
    role "embedding": a table [rows, width], kept in the compute dtype;
    role "norm": a norm weight, kept in 32-bit (``zero_centered`` ones are
    stored as w and used as 1 + w);
    role "table_int": an integer table, kept as int32;
    role "float32": kept in 32-bit whatever the compute dtype is.
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    zero_centered: bool = False


# ---- cache needs a mixer can state ------------------------------------------
@dataclass(frozen=True)
class KVRequest:
    """Keys and values per position; ``window`` None keeps all of them, W keeps
    the last W."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A fixed number of 32-bit values per sequence, zero when a slot is taken."""
    numel: int


_MIXERS: Dict[str, type] = {}
_FEED_FORWARDS: Dict[str, type] = {}
_NORMS: Dict[str, type] = {}
_POSITIONS: Dict[str, type] = {}
_BLOCKS: Dict[str, type] = {}
_STREAM_POSITIONS: Dict[str, type] = {}


def register_mixer(kind: str, cls: type) -> None:
    _MIXERS[kind] = cls


def register_feed_forward(kind: str, cls: type) -> None:
    _FEED_FORWARDS[kind] = cls


def register_norm(kind: str, cls: type) -> None:
    _NORMS[kind] = cls


def register_position(kind: str, cls: type) -> None:
    _POSITIONS[kind] = cls


def register_block(kind: str, cls: type) -> None:
    """A block class: ``param_specs(spec, hidden) -> {name: ParamSpec}`` (class method),
    ``__init__(spec, hidden, dtype, device)``, ``load(tensors, dtype, device)``,
    ``entry_norm`` (the norm part that feeds its first branch; the block before it
    applies that norm in the launch that also adds its own last branch),
    ``cache_request()`` and
    ``forward(h, x, ctx, cache_entry, writes_cache, next_norm) -> x_next``: h is the
    32-bit stream [T, H], updated in place; x = entry_norm(h); x_next = next_norm(h)
    after the update, or None when next_norm is None."""
    _BLOCKS[kind] = cls


def register_stream_position(kind: str, cls: type) -> None:
    """A position encoding added to the stream after the embedding:
    ``param_specs(spec, hidden)`` (class method), ``__init__(spec, hidden, dtype,
    device)``, ``load(tensors, device)`` and ``forward(h, ctx)``, which adds to the
    32-bit stream h [T, H] in place from ``ctx.positions``."""
    _STREAM_POSITIONS[kind] = cls


def _lookup(table: Dict[str, type], what: str, kind: str) -> type:
    if kind not in table:
        raise KeyError(f"no {what} registered under kind {kind!r}; "
                       f"registered: {', '.join(sorted(table)) or '(none)'}")
    return table[kind]


def mixer_class(kind: str) -> type:
    return _lookup(_MIXERS, "mixer", kind)


def feed_forward_class(kind: str) -> type:
    return _lookup(_FEED_FORWARDS, "feed-forward", kind)


def norm_class(kind: str) -> type:
    return _lookup(_NORMS, "norm", kind)


def position_class(kind: str) -> type:
    return _lookup(_POSITIONS, "position encoding", kind)


def block_class(kind: str) -> type:
    return _lookup(_BLOCKS, "block", kind)


def stream_position_class(kind: str) -> type:
    return _lookup(_STREAM_POSITIONS, "stream position", kind)
