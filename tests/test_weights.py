"""Safetensors reading, weight errors and the random-weights mode (no GPU)."""
import json
import os
import shutil
import struct
import tempfile

import pytest
import torch

import agave_b200  # noqa: F401
from agave_b200.config import load_config
from agave_b200.models.decoder import decoder_param_specs
from agave_b200.weights import (SafetensorsError, SafetensorsFolder, WeightsError, load_weights,
                                save_safetensors, write_model_folder)
from util import TINY_A, TINY_B, model_folder


def _load(folder):
    entry, cfg = load_config(folder)
    names = entry.weight_names(cfg)
    specs = decoder_param_specs(cfg.to_model_spec())
    return load_weights(folder, specs, names.checkpoint_name, names.prefixes), specs


def test_random_folder_loads_and_keeps_dtypes():
    for dtype in (torch.bfloat16, torch.float32):
        folder = model_folder("A", dtype)
        tensors, specs = _load(folder)
        assert set(tensors) == set(specs)
        for n, t in tensors.items():
            assert tuple(t.shape) == tuple(specs[n].shape)
            assert t.dtype == dtype          # stored bf16 stays bf16, stored f32 stays f32
        names = set(SafetensorsFolder(folder).names())
        assert "model.embed_tokens.weight" in names
        assert "model.layers.3.self_attn.q_norm.weight" in names
        assert "model.layers.0.pre_feedforward_layernorm.weight" in names


def test_random_weights_are_seeded_and_per_tensor():
    a1 = tempfile.mkdtemp(); a2 = tempfile.mkdtemp(); a3 = tempfile.mkdtemp()
    write_model_folder(a1, TINY_A, seed=5)
    write_model_folder(a2, TINY_A, seed=5)
    write_model_folder(a3, TINY_A, seed=6)
    f1, f2, f3 = SafetensorsFolder(a1), SafetensorsFolder(a2), SafetensorsFolder(a3)
    for n in f1.names():
        assert torch.equal(f1.tensor(n), f2.tensor(n))
    assert not torch.equal(f1.tensor("model.embed_tokens.weight"),
                           f3.tensor("model.embed_tokens.weight"))
    w = f1.tensor("model.layers.0.mlp.up_proj.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002
    nw = f1.tensor("model.layers.0.input_layernorm.weight").float()
    assert abs(nw.mean().item()) < 0.05 and 0.05 < nw.std().item() < 0.15


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    src = model_folder("A", torch.float32)
    d = tempfile.mkdtemp()
    shutil.copy(os.path.join(src, "config.json"), d)
    f = SafetensorsFolder(src)
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.1.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 63)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightsError) as e:
        _load(d)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 63), (16, 64))]
    msg = str(err)
    for piece in ("missing", "unexpected", "wrong shape", "model.norm.weight",
                  "model.layers.9.extra.weight", "[16, 63]"):
        assert piece in msg


def test_prefixed_names_and_untied_head():
    src = model_folder("B", torch.float32)
    d = tempfile.mkdtemp()
    cfg = dict(TINY_B); cfg["tie_word_embeddings"] = False
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    f = SafetensorsFolder(src)
    t = {"language_model." + n: f.tensor(n).clone() for n in f.names()}
    t["language_model.lm_head.weight"] = torch.randn(384, 96)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    tensors, specs = _load(d)
    assert "lm_head.weight" in tensors and tensors["lm_head.weight"].shape == (384, 96)
    del t["language_model.lm_head.weight"]
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightsError) as e:
        _load(d)
    assert e.value.missing == ["language_model.lm_head.weight"]


def multimodal_folder(prefix: str, head_name: str, d=None):
    """A folder laid out like the multimodal family members: ``model_type`` gemma3, the
    sizes under ``text_config`` (with the keys those leave out left out), the decoder
    under ``prefix``, a head of its own, and tensors of a vision tower and a projector."""
    src = model_folder("B", torch.float32)
    d = d or tempfile.mkdtemp()
    text = {k: v for k, v in TINY_B.items()
            if k not in ("architectures", "num_attention_heads", "num_key_value_heads",
                         "head_dim", "vocab_size", "tie_word_embeddings")}
    cfg = {"architectures": ["Gemma3ForConditionalGeneration"], "model_type": "gemma3",
           "text_config": text, "vision_config": {"hidden_size": 8, "model_type": "siglip"},
           "mm_tokens_per_image": 4}
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    f = SafetensorsFolder(src)
    t = {prefix + n[len("model."):]: f.tensor(n).clone() for n in f.names()}
    t[head_name] = torch.randn(384, 96)
    vis = "" if prefix.startswith("language_model") else "model."
    t[vis + "vision_tower.vision_model.encoder.layers.0.self_attn.q_proj.weight"] = torch.zeros(8, 8)
    t[vis + "vision_tower.vision_model.embeddings.position_embedding.weight"] = torch.zeros(4, 8)
    t[vis + "multi_modal_projector.mm_input_projection_weight"] = torch.zeros(8, 96)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    return d, t


@pytest.mark.parametrize("prefix,head", [("language_model.model.", "language_model.lm_head.weight"),
                                         ("model.language_model.", "lm_head.weight")])
def test_multimodal_folder_gives_the_text_decoder(prefix, head):
    d, t = multimodal_folder(prefix, head)
    entry, cfg = load_config(d)
    assert entry.name == "Gemma3ForCausalLM"
    # the sizes text_config leaves out come from the tensors
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
            cfg.vocab_size) == (6, 2, 32, 384)
    names = entry.weight_names(cfg)
    import dataclasses
    from agave_b200.weights import head_is_stored
    assert head_is_stored(d, names.checkpoint_name, names.prefixes)
    spec = dataclasses.replace(cfg.to_model_spec(), tie_embeddings=False)
    specs = decoder_param_specs(spec)
    tensors = load_weights(d, specs, names.checkpoint_name, names.prefixes,
                           ignore_prefixes=names.ignore_prefixes)
    assert set(tensors) == set(specs) and tensors.prefix == prefix
    assert torch.equal(tensors["lm_head.weight"], t[head])
    assert len(tensors.ignored) == 3 and all("vision" in n or "projector" in n
                                             for n in tensors.ignored)
    # the strict switch keeps the old rule: every unrequested tensor is an error
    with pytest.raises(WeightsError) as e:
        load_weights(d, specs, names.checkpoint_name, names.prefixes, strict=True)
    assert len(e.value.unexpected) == 3 and not e.value.missing
    # a stray name inside the decoder is still an error without it
    t[prefix + "layers.0.self_attn.extra.weight"] = torch.zeros(2)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightsError) as e:
        load_weights(d, specs, names.checkpoint_name, names.prefixes,
                     ignore_prefixes=names.ignore_prefixes)
    assert e.value.unexpected == [prefix + "layers.0.self_attn.extra.weight"]


def test_sizes_left_out_of_config_need_the_tensors():
    from agave_b200.config import ConfigError, Gemma3Config
    raw = {k: v for k, v in TINY_B.items() if k not in ("head_dim", "vocab_size")}
    with pytest.raises(ConfigError):
        Gemma3Config.from_dict(raw)
    shapes = {"layers.0.self_attn.q_norm.weight": (32,), "embed_tokens.weight": (384, 96)}
    cfg = Gemma3Config.from_dict(raw, shapes=shapes.get)
    assert cfg.head_dim == 32 and cfg.vocab_size == 384


def test_sharded_folder_with_index():
    src = model_folder("A", torch.bfloat16)
    d = tempfile.mkdtemp()
    shutil.copy(os.path.join(src, "config.json"), d)
    f = SafetensorsFolder(src)
    names = sorted(f.names())
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half],
             "model-00002-of-00002.safetensors": names[half:]}
    wm = {}
    for fn, ns in parts.items():
        save_safetensors(os.path.join(d, fn), {n: f.tensor(n).clone() for n in ns})
        wm.update({n: fn for n in ns})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    tensors, specs = _load(d)
    assert set(tensors) == set(specs)
    wm[names[0]] = "../evil.safetensors"
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    with pytest.raises(SafetensorsError):
        _load(d)


def test_truncated_and_inconsistent_files_are_refused():
    src = model_folder("A", torch.float32)
    path = os.path.join(src, "model.safetensors")
    raw = open(path, "rb").read()
    d = tempfile.mkdtemp()
    shutil.copy(os.path.join(src, "config.json"), d)
    target = os.path.join(d, "model.safetensors")
    for blob in (raw[:4], raw[:len(raw) - 100], struct.pack("<Q", 10 ** 12) + raw[8:]):
        with open(target, "wb") as fh:
            fh.write(blob)
        with pytest.raises(SafetensorsError):
            SafetensorsFolder(d)
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    k = next(iter(header))
    header[k]["data_offsets"][1] += 4
    hb = json.dumps(header).encode()
    with open(target, "wb") as fh:
        fh.write(struct.pack("<Q", len(hb)) + hb + raw[8 + n:])
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(d)
