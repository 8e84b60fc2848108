"""Typed configuration of the Gemma 3 text decoder, read from its own
``config.json`` keys (the names Hugging Face checkpoints carry).

Which keys exist and what they mean follows the reference's reader
(src/models/gemma3.zig:149-202 with the key map in
src/format/safetensors.zig:641-664): heads, head_dim (not hidden/heads),
query_pre_attn_scalar for the score scale, two rotary bases, a layer pattern
in which layer l is local iff (l + 1) % pattern != 0
(src/models/gemma3.zig:736), and eps inside the square root.  Two things the
reference cannot reach from config.json are read here: the window size
(``sliding_window``) and the nested ``rope_scaling.factor`` for global layers.

Only the defaults the reference itself documents are kept (eps 1e-6, rotary
bases 1e6 / 1e4, pattern 6, query_pre_attn_scalar = head_dim, factor 1);
every size must be present.  The ``text_config`` of the multimodal family
members leaves out the sizes that equal their library defaults (head count,
kv head count, head_dim, vocab_size); the reference falls back to the 1B
sizes there (src/models/gemma3.zig:40-52), which is wrong for every other
member.  Here a size that config.json omits is read from the shapes of the
checkpoint's own tensors when the caller can show them (``shapes``), and is an
error otherwise.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import (AttentionSpec, BlockSpec, ConfigError, GatedFeedForwardSpec,
                   ModelSpec, NormSpec, RotarySpec, default_schedule)

_ACTIVATIONS = {
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_tanh": "gelu_tanh",
    "silu": "silu",
    "swish": "silu",
}

_LOCAL = "sliding_attention"
_GLOBAL = "full_attention"


def _need(d: Dict[str, Any], key: str, typ=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                return int(v)
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    return v


def _opt(d, key, default, typ=float):
    if key not in d or d[key] is None:
        return default
    return _need(d, key, typ)


@dataclass(frozen=True)
class Gemma3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    query_pre_attn_scalar: float
    rms_norm_eps: float
    rope_theta: float
    rope_local_base_freq: float
    rope_scaling_factor: float
    sliding_window: Optional[int]
    layer_types: Tuple[str, ...]
    hidden_activation: str
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]

    architecture = "Gemma3ForCausalLM"

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, raw: Dict[str, Any], shapes=None) -> "Gemma3Config":
        """``shapes(suffix)``: the shape of the checkpoint tensor whose name ends
        with ``suffix`` (under whatever prefix), or None; used only for sizes
        that config.json leaves out."""
        d = dict(raw)
        # keys under text_config override top-level ones
        # (src/format/safetensors.zig:1827-1831)
        if isinstance(d.get("text_config"), dict):
            d.update(d["text_config"])
        if shapes is not None:
            cls._sizes_from_shapes(d, shapes)
        n_layers = _need(d, "num_hidden_layers")
        hidden = _need(d, "hidden_size")
        n_heads = _need(d, "num_attention_heads")
        n_kv = _opt(d, "num_key_value_heads", n_heads, int)
        head_dim = _need(d, "head_dim")
        qpas = _opt(d, "query_pre_attn_scalar", float(head_dim), float)
        window = _opt(d, "sliding_window", None, int)

        # rotary bases and scaling: flat keys, or the per-layer-type table
        # newer checkpoints carry under rope_parameters
        theta = _opt(d, "rope_theta", 1e6, float)
        local_theta = _opt(d, "rope_local_base_freq", 1e4, float)
        factor = 1.0
        scaling = d.get("rope_scaling")
        params = d.get("rope_parameters")
        if isinstance(params, dict):
            if isinstance(params.get(_GLOBAL), dict) or isinstance(params.get(_LOCAL), dict):
                g = params.get(_GLOBAL) or {}
                l = params.get(_LOCAL) or {}
                theta = float(g.get("rope_theta", theta))
                local_theta = float(l.get("rope_theta", local_theta))
                scaling = g
                cls._check_scaling(l, "rope_parameters.sliding_attention", allow_factor=False)
            else:
                theta = float(params.get("rope_theta", theta))
                scaling = params
        if isinstance(scaling, dict):
            factor = cls._check_scaling(scaling, "rope_scaling", allow_factor=True)
        elif scaling is not None:
            raise ConfigError("config.json: 'rope_scaling' must be null or an object")

        # which layers are local: an explicit list, else the pattern
        if d.get("layer_types") is not None:
            lt = d["layer_types"]
            if not isinstance(lt, list) or len(lt) != n_layers:
                raise ConfigError(
                    f"config.json: 'layer_types' must list {n_layers} entries, got "
                    f"{len(lt) if isinstance(lt, list) else type(lt).__name__}")
            for t in lt:
                if t not in (_LOCAL, _GLOBAL):
                    raise ConfigError(f"config.json: unknown layer type {t!r} in 'layer_types'")
            layer_types = tuple(lt)
        else:
            pattern = _opt(d, "sliding_window_pattern", 6 if window is not None else 0, int)
            if pattern < 0:
                raise ConfigError("config.json: 'sliding_window_pattern' must be >= 0")
            layer_types = tuple(
                _LOCAL if (pattern > 0 and (l + 1) % pattern != 0) else _GLOBAL
                for l in range(n_layers))

        act = d.get("hidden_activation", d.get("hidden_act", "gelu_pytorch_tanh"))
        if act is None:
            act = "gelu_pytorch_tanh"
        if act not in _ACTIVATIONS:
            raise ConfigError(f"config.json: hidden_activation {act!r} is not supported "
                              f"(supported: {sorted(_ACTIVATIONS)})")

        eos = d.get("eos_token_id", 1)     # default 1: src/models/gemma3.zig:189
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, list):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        bos = d.get("bos_token_id", 2)     # default 2: src/main.zig:1186-1196

        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            if d.get(key):
                raise ConfigError(
                    f"config.json: '{key}' = {d[key]!r} is not supported: this decoder "
                    "applies no soft cap (src/models/gemma3.zig:197)")
        if d.get("attention_bias"):
            raise ConfigError("config.json: 'attention_bias' = true is not supported "
                              "(no bias tensors are read, src/models/gemma3.zig:714-719)")

        cfg = cls(
            vocab_size=_need(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size"),
            num_hidden_layers=n_layers,
            num_attention_heads=n_heads,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            query_pre_attn_scalar=float(qpas),
            rms_norm_eps=_opt(d, "rms_norm_eps", 1e-6, float),
            rope_theta=theta,
            rope_local_base_freq=local_theta,
            rope_scaling_factor=float(factor),
            sliding_window=window,
            layer_types=layer_types,
            hidden_activation=_ACTIVATIONS[act],
            max_position_embeddings=_opt(d, "max_position_embeddings", 0, int),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
            bos_token_id=None if bos is None else int(bos),
            eos_token_ids=eos_ids,
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _sizes_from_shapes(d: Dict[str, Any], shapes) -> None:
        """Fill sizes that config.json omits from the tensors that have them."""
        def rows(suffix):
            sh = shapes(suffix)
            return int(sh[0]) if sh else None
        if d.get("head_dim") is None:
            hd = rows("layers.0.self_attn.q_norm.weight")
            if hd:
                d["head_dim"] = hd
        hd = d.get("head_dim")
        if isinstance(hd, int) and hd > 0:
            for key, suffix in (("num_attention_heads", "layers.0.self_attn.q_proj.weight"),
                                ("num_key_value_heads", "layers.0.self_attn.k_proj.weight")):
                if d.get(key) is None:
                    r = rows(suffix)
                    if r and r % hd == 0:
                        d[key] = r // hd
        if d.get("vocab_size") is None:
            v = rows("embed_tokens.weight")
            if v:
                d["vocab_size"] = v

    @staticmethod
    def _check_scaling(s: Dict[str, Any], where: str, allow_factor: bool) -> float:
        kind = s.get("rope_type", s.get("type", "default"))
        if kind in (None, "default"):
            return 1.0
        if kind != "linear":
            raise ConfigError(f"config.json: {where} type {kind!r} is not supported "
                              "(supported: linear)")
        f = s.get("factor", 1.0)
        if not isinstance(f, (int, float)) or isinstance(f, bool) or f <= 0:
            raise ConfigError(f"config.json: {where}.factor must be a positive number")
        if not allow_factor and float(f) != 1.0:
            raise ConfigError(f"config.json: {where}.factor on sliding layers is not supported")
        return float(f)

    def validate(self) -> None:
        pos = ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
               "num_attention_heads", "num_key_value_heads", "head_dim"]
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: '{k}' must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a "
                f"multiple of num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even")
        if self.query_pre_attn_scalar <= 0:
            raise ConfigError("config.json: 'query_pre_attn_scalar' must be positive")
        if self.rms_norm_eps <= 0:
            raise ConfigError("config.json: 'rms_norm_eps' must be positive")
        if self.rope_theta <= 0 or self.rope_local_base_freq <= 0:
            raise ConfigError("config.json: rotary bases must be positive")
        if _LOCAL in self.layer_types:
            if self.sliding_window is None or self.sliding_window < 1:
                raise ConfigError("config.json: 'sliding_window' (>= 1) is required when a "
                                  "layer is sliding_attention")

    @classmethod
    def from_model_dir(cls, folder: str) -> "Gemma3Config":
        with open(os.path.join(folder, "config.json"), "r") as f:
            return cls.from_dict(json.load(f))

    # ----------------------------------------------------------------- write
    def to_dict(self) -> Dict[str, Any]:
        """The same configuration under its config.json keys."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "gemma3_text",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "query_pre_attn_scalar": self.query_pre_attn_scalar,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_local_base_freq": self.rope_local_base_freq,
            "rope_scaling": (None if self.rope_scaling_factor == 1.0 else
                             {"rope_type": "linear", "factor": self.rope_scaling_factor}),
            "sliding_window": self.sliding_window,
            "layer_types": list(self.layer_types),
            "hidden_activation": ("gelu_pytorch_tanh" if self.hidden_activation == "gelu_tanh"
                                  else self.hidden_activation),
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1
            else self.eos_token_ids[0],
        }
        return d

    # ----------------------------------------------------------------- lower
    def is_local(self, layer: int) -> bool:
        return self.layer_types[layer] == _LOCAL

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(eps=self.rms_norm_eps, zero_centered=True)
        ffn = GatedFeedForwardSpec(intermediate_size=self.intermediate_size,
                                   activation=self.hidden_activation)
        scale = 1.0 / math.sqrt(self.query_pre_attn_scalar)   # src/models/gemma3.zig:190-194
        local_rope = RotarySpec(theta=self.rope_local_base_freq, factor=1.0,
                                rotary_dim=self.head_dim)
        global_rope = RotarySpec(theta=self.rope_theta, factor=self.rope_scaling_factor,
                                 rotary_dim=self.head_dim)
        blocks = []
        for l in range(self.num_hidden_layers):
            local = self.is_local(l)
            attn = AttentionSpec(
                n_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim, scale=scale,
                window=self.sliding_window if local else None,
                qk_norm=norm, position=local_rope if local else global_rope)
            blocks.append(BlockSpec(mixer=attn, feed_forward=ffn, norm=norm,
                                    arrangement="sandwich"))
        return ModelSpec(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            embed_scale=math.sqrt(float(self.hidden_size)),   # src/models/gemma3.zig:195
            blocks=tuple(blocks), schedule=default_schedule(len(blocks)),
            final_norm=norm, tie_embeddings=self.tie_word_embeddings,
            max_positions=self.max_position_embeddings,
            bos_token_id=self.bos_token_id, eos_token_ids=self.eos_token_ids)
