"""Seeded random weights: tensors for a model, or a whole model folder.

Each tensor has its own generator keyed by (seed, internal name), so a tensor
is the same whatever the order or the subset that is drawn.  Matrices and
tables are N(0, std); norm weights are N(0, norm_std) around zero for
zero-centred norms (they are used as 1 + w) and around one otherwise.
The reference has no such mode; its nearest relative are the synthetic fills
of its micro-benchmarks (src/micro_bench.zig:533-575).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Optional

import torch

from ..parts.base import ParamSpec
from .safetensors_io import save_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: ParamSpec, seed: int, std: float, norm_std: float,
                  dtype: torch.dtype, device: str = "cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    if spec.role == "table_int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.role == "norm":
        t = t * norm_std
        if not spec.zero_centered:
            t = t + 1.0
        return t.to(dtype)
    return (t * std).to(dtype)


def random_tensors(param_specs: Dict[str, ParamSpec], seed: int, std: float = 0.02,
                   norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    return {n: random_tensor(n, s, seed, std, norm_std, dtype, device)
            for n, s in param_specs.items()}


def write_model_folder(folder: str, raw_config: dict, seed: int, std: float = 0.02,
                       norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for a configuration.

    ``raw_config`` holds the architecture's own config.json keys (it must name
    the architecture); the tensors get the names a checkpoint of that
    architecture has.
    """
    from ..config import resolve_architecture
    from ..models.decoder import decoder_param_specs
    entry = resolve_architecture(raw_config)
    config = entry.config_class.from_dict(raw_config)
    specs = decoder_param_specs(config.to_model_spec())
    plan = entry.weight_names(config)
    tensors = random_tensors(specs, seed, std, norm_std, dtype)
    named = {plan.checkpoint_name(n, plan.prefixes[0]): t for n, t in tensors.items()}
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw_config, f, indent=1)
    save_safetensors(os.path.join(folder, "model.safetensors"), named)
    return folder
