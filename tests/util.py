"""Shared fixtures of the tests: the two tiny configurations, model folders in
temporary directories, and the comparison rule."""
import json
import os
import sys
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Gemma 3 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
    "num_hidden_layers": 4, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 16, "query_pre_attn_scalar": 16,
    "intermediate_size": 128, "vocab_size": 256, "sliding_window": 8,
    "sliding_window_pattern": 2, "rope_local_base_freq": 10000.0, "rope_theta": 1000000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 1024, "hidden_activation": "gelu_pytorch_tanh",
    "bos_token_id": 2, "eos_token_id": 1,
}
TINY_B = {
    "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
    "num_hidden_layers": 7, "hidden_size": 96, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 32, "query_pre_attn_scalar": 24,
    "intermediate_size": 224, "vocab_size": 384, "sliding_window": 16,
    "sliding_window_pattern": 3, "rope_local_base_freq": 5000.0, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0}, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 2048,
    "hidden_activation": "gelu_pytorch_tanh", "bos_token_id": 2, "eos_token_id": [1, 106],
}
# A third one with a head size of 64, the smallest that takes the kernels the full-size
# models run on (tcgen05 prompt attention, decode attention with the q/k norm, the
# rotation and the cache store inside): two query heads per kv head, three kv heads.
TINY_C = {
    "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
    "num_hidden_layers": 5, "hidden_size": 192, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 64, "query_pre_attn_scalar": 48,
    "intermediate_size": 320, "vocab_size": 500, "sliding_window": 24,
    "sliding_window_pattern": 4, "rope_local_base_freq": 8000.0, "rope_theta": 200000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 4.0}, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 1024,
    "hidden_activation": "gelu_pytorch_tanh", "bos_token_id": 2, "eos_token_id": 1,
}
TINY = {"A": (TINY_A, 0, 0.02, 0.1), "B": (TINY_B, 1, 0.03, 0.2), "C": (TINY_C, 2, 0.03, 0.15)}

_FOLDERS = {}


def _cleanup():
    import shutil
    for d in _FOLDERS.values():
        shutil.rmtree(d, ignore_errors=True)


import atexit
atexit.register(_cleanup)


def model_folder(name: str, dtype=torch.float32, std_scale: float = 1.0) -> str:
    """A temporary model folder for tiny configuration ``name`` (made once per run)."""
    key = (name, dtype, std_scale)
    if key not in _FOLDERS:
        from agave_b200.weights import write_model_folder
        cfg, seed, std, norm_std = TINY[name]
        d = tempfile.mkdtemp(prefix=f"agave_tiny_{name}_")
        write_model_folder(d, cfg, seed, std * std_scale, norm_std, dtype)
        _FOLDERS[key] = d
    return _FOLDERS[key]


def random_tokens(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(3, vocab, (n,), generator=g).tolist()


def plain_logits(folder: str, tokens, dtype=torch.float64):
    from plain import gemma3_plain as P
    cfg = P.read_config(folder)
    w = P.read_weights(folder, dtype)
    return P.forward_logits(cfg, w, tokens)


def close(got: torch.Tensor, ref: torch.Tensor, rel: float):
    """max |got - ref| <= rel * max |ref|, per comparison (logit rows share a scale)."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), "non-finite values"
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= rel * scale, f"max error {err:.3e} exceeds {rel:g} * {scale:.3e}"
    return err / max(scale, 1e-30)


# relative tolerances on logits (max error over max magnitude)
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
