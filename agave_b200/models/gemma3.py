"""Gemma 3 text decoder: the registry entry and the names of its tensors.

The layer structure itself is data (``Gemma3Config.to_model_spec``); what is
left to say here is how the generic decoder's tensor names map to the names
in a checkpoint (src/format/safetensors.zig:468-481,525-540) and under which
prefixes they may sit (src/format/safetensors.zig:517-521).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

from ..config.gemma3 import Gemma3Config
from ..config.registry import register_architecture

_BLOCK_NAMES = {
    "pre_mixer_norm.weight": "input_layernorm.weight",
    "post_mixer_norm.weight": "post_attention_layernorm.weight",
    "pre_ffn_norm.weight": "pre_feedforward_layernorm.weight",
    "post_ffn_norm.weight": "post_feedforward_layernorm.weight",
    "mixer.q_proj.weight": "self_attn.q_proj.weight",
    "mixer.k_proj.weight": "self_attn.k_proj.weight",
    "mixer.v_proj.weight": "self_attn.v_proj.weight",
    "mixer.o_proj.weight": "self_attn.o_proj.weight",
    "mixer.q_norm.weight": "self_attn.q_norm.weight",
    "mixer.k_norm.weight": "self_attn.k_norm.weight",
    "ffn.gate_proj.weight": "mlp.gate_proj.weight",
    "ffn.up_proj.weight": "mlp.up_proj.weight",
    "ffn.down_proj.weight": "mlp.down_proj.weight",
}


_HEAD_PREFIX = {"model.": "", "language_model.model.": "language_model.",
                "model.language_model.": "", "": ""}


@dataclass(frozen=True)
class Gemma3WeightNames:
    prefixes: Tuple[str, ...] = ("model.", "language_model.model.", "model.language_model.", "")
    # what a multimodal folder holds beside the text decoder; never read here
    ignore_prefixes: Tuple[str, ...] = ("vision_tower.", "multi_modal_projector.",
                                        "model.vision_tower.", "model.multi_modal_projector.")

    def checkpoint_name(self, internal: str, prefix: str) -> str:
        if internal == "embed.weight":
            return prefix + "embed_tokens.weight"
        if internal == "final_norm.weight":
            return prefix + "norm.weight"
        if internal == "lm_head.weight":
            # the head sits beside the decoder, not inside it
            return _HEAD_PREFIX.get(prefix, "") + "lm_head.weight"
        parts = internal.split(".", 2)
        if parts[0] == "blocks" and parts[2] in _BLOCK_NAMES:
            return f"{prefix}layers.{parts[1]}.{_BLOCK_NAMES[parts[2]]}"
        raise KeyError(f"Gemma 3 has no checkpoint name for '{internal}'")


def _weight_names(config: Gemma3Config) -> Gemma3WeightNames:
    return Gemma3WeightNames()


register_architecture("Gemma3ForCausalLM", Gemma3Config, _weight_names,
                      model_types=("gemma3_text", "gemma3"))
