"""Weights by tensor name, with one error that says everything that is wrong.

The model states which tensors it needs (``ParamSpec`` per internal name) and
the architecture gives each internal name its checkpoint name; this module
matches that list against the files.  Tensors stay as stored: bfloat16 stays
bfloat16, a tensor stored in 32-bit stays 32-bit, half floats are widened
(exactly) to 32-bit and integer tables become int32.  The cast to the compute
dtype is the model's business, not the loader's.

The reference reports a missing tensor only when a layer first asks for it
(``MissingTensor``, src/models/gemma3.zig:352, src/format/safetensors.zig:333-349);
here the whole list is checked before anything is copied to the device.

A folder may hold more than the decoder: checkpoints of the multimodal family
members carry a vision tower and a projector beside ``language_model.*``.  The
reference looks tensors up by name and never sees the rest
(src/format/safetensors.zig:333-349, prefixes 517-521).  Here a tensor that
the decoder does not ask for is *unexpected* (an error) when it lies under the
decoder's own prefix, where a stray name is most likely a mistake, and
*ignored* when it lies elsewhere in the folder; ``strict=True`` makes every
unrequested tensor an error.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Sequence, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsFolder


class WeightsError(ValueError):
    """Lists missing tensors, unexpected tensors and wrong shapes in one message."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: List[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"{where}: the tensors do not match the configuration"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {dt}" for n, dt in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOATS = ("F32", "BF16", "F16", "F64")
_INTS = ("I64", "I32", "I16", "I8", "U8")


def _as_stored(t: torch.Tensor, role: str) -> torch.Tensor:
    if role == "table_int":
        return t.to(torch.int32)
    if t.dtype == torch.bfloat16 or t.dtype == torch.float32:
        return t
    return t.to(torch.float32)


def choose_prefix(file_names, expected_suffixes: Sequence[str], prefixes: Sequence[str]) -> str:
    """The prefix under which most of the expected names are present."""
    names = set(file_names)
    best, best_hits = prefixes[0], -1
    for p in prefixes:
        hits = sum(1 for s in expected_suffixes if p + s in names)
        if hits > best_hits:
            best, best_hits = p, hits
    return best


def head_is_stored(folder: str, checkpoint_name: Callable[[str, str], str],
                   prefixes: Sequence[str]) -> bool:
    """Whether the folder holds an output head of its own (``lm_head.weight``
    beside the decoder it belongs to)."""
    files = SafetensorsFolder(folder)
    prefix = choose_prefix(files.names(), [checkpoint_name("embed.weight", ""),
                                           checkpoint_name("final_norm.weight", "")], prefixes)
    return checkpoint_name("lm_head.weight", prefix) in files.tensors


class LoadedWeights(dict):
    """{internal name: CPU tensor as stored}, with what the folder held besides:
    ``prefix`` (where the decoder's tensors sit) and ``ignored`` (names outside it)."""
    prefix: str = ""
    ignored: List[str] = []


def load_weights(folder: str, param_specs: Dict[str, ParamSpec],
                 checkpoint_name: Callable[[str, str], str],
                 prefixes: Sequence[str] = ("",), strict: bool = False,
                 ignore_prefixes: Sequence[str] = ()) -> "LoadedWeights":
    """{internal name: CPU tensor as stored}; raises ``WeightsError``.

    ``checkpoint_name(internal, prefix)`` gives the name in the files.  Tensors
    the model does not ask for are an error under the decoder's prefix and
    ignored elsewhere (and under ``ignore_prefixes``); with ``strict`` all of
    them are errors.  The names ignored are in the result's ``ignored``.
    """
    files = SafetensorsFolder(folder)
    probe = [checkpoint_name(n, "") for n in param_specs]
    prefix = choose_prefix(files.names(), probe, prefixes)
    wanted = {checkpoint_name(n, prefix): n for n in param_specs}

    missing, wrong_shape, wrong_dtype = [], [], []
    for ck, internal in wanted.items():
        info = files.tensors.get(ck)
        spec = param_specs[internal]
        if info is None:
            missing.append(ck)
            continue
        if tuple(info.shape) != tuple(spec.shape):
            wrong_shape.append((ck, tuple(info.shape), tuple(spec.shape)))
        ok = _INTS if spec.role == "table_int" else _FLOATS
        if info.dtype not in ok:
            wrong_dtype.append((ck, info.dtype))
    unexpected, ignored = [], []
    for n in sorted(files.names()):
        if n in wanted:
            continue
        outside = (not n.startswith(prefix)) or any(n.startswith(p) for p in ignore_prefixes)
        (ignored if outside and not strict else unexpected).append(n)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(folder, sorted(missing), unexpected, wrong_shape, wrong_dtype)
    out = LoadedWeights((internal, _as_stored(files.tensor(ck), param_specs[internal].role))
                        for ck, internal in wanted.items())
    out.prefix, out.ignored = prefix, ignored
    return out
