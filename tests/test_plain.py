"""The plain implementation itself (no GPU): against the reference's own Python
kernel references (committed golden file), and its own invariants."""
import math
import os

import numpy as np
import torch

from plain import gemma3_plain as P
from util import TINY_A, TINY_B, model_folder, random_tokens

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                      "reference_kernels.npz")


def _t(a):
    return torch.from_numpy(np.asarray(a)).double()


def test_parts_match_the_reference_python_functions():
    g = np.load(GOLDEN)
    y = P.rms_norm(_t(g["norm_x"]), _t(g["norm_w"]), 1e-5, add_one=False)
    assert torch.allclose(y, _t(g["norm_y"]), atol=1e-5)
    assert torch.allclose(P.gelu_tanh(_t(g["gelu_x"])), _t(g["gelu_y"]), atol=1e-6)
    nh, nkv, hd, pos, theta = g["rope_meta"]
    nh, nkv, hd, pos = int(nh), int(nkv), int(hd), int(pos)
    ang = P.rope_angles(torch.tensor([pos]), hd, float(theta), 1.0)
    qo = P.apply_rope(_t(g["rope_q"]).reshape(1, nh, hd), ang).reshape(-1)
    ko = P.apply_rope(_t(g["rope_k"]).reshape(1, nkv, hd), ang).reshape(-1)
    assert torch.allclose(qo, _t(g["rope_qo"]), atol=2e-5)
    assert torch.allclose(ko, _t(g["rope_ko"]), atol=2e-5)
    nh, nkv, hd, sl, scale = g["sdpa_meta"]
    nh, nkv, hd, sl = int(nh), int(nkv), int(hd), int(sl)
    # the golden query sits after sl cached positions: last row of a causal pass
    k = _t(g["sdpa_k"]).reshape(sl, nkv, hd)
    v = _t(g["sdpa_v"]).reshape(sl, nkv, hd)
    q = torch.zeros(sl, nh, hd, dtype=torch.float64)
    q[-1] = _t(g["sdpa_q"]).reshape(nh, hd)
    o = P.attention(q, k, v, float(scale), None)[-1]
    assert torch.allclose(o, _t(g["sdpa_o"]), atol=1e-5)


def test_window_mask_convention():
    m = P.visible(6, 3)
    # position p sees p-2..p: exactly W keys once p >= W-1
    assert m[5].tolist() == [False, False, False, True, True, True]
    assert m[1].tolist() == [True, True, False, False, False, False]
    assert P.visible(4, None)[3].all()


def test_logits_are_causal_and_windows_matter():
    folder = model_folder("A", torch.float32)
    cfg, w = P.read_config(folder), P.read_weights(folder)
    toks = random_tokens(24, 256, 3)
    full = P.forward_logits(cfg, w, toks)
    part = P.forward_logits(cfg, w, toks[:13])
    assert torch.allclose(full[:13], part, atol=1e-9)        # later tokens change nothing earlier
    cfg2 = dict(cfg)
    cfg2["sliding_window"] = 1000
    wide = P.forward_logits(cfg2, w, toks)
    assert torch.allclose(wide[:8], full[:8], atol=1e-9)     # inside the window: same
    assert (wide[12:] - full[12:]).abs().max() > 1e-6        # beyond it: the mask shows


def test_scaling_factor_only_touches_global_layers():
    folder = model_folder("B", torch.float32)
    cfg, w = P.read_config(folder), P.read_weights(folder)
    assert P.rope_factor(cfg) == 2.0
    assert [P.layer_is_local(cfg, l) for l in range(7)] == [True, True, False, True, True,
                                                            False, True]
    a = P.rope_angles(torch.arange(4), 32, 500000.0, 2.0)
    b = P.rope_angles(torch.arange(4), 32, 500000.0, 1.0)
    assert torch.allclose(a * 2, b)


def test_sampling_reference_functions():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert P.argmax_first(logits) == 1
    w = P.filtered_weights(logits, 1.0, 2, 1.0)
    assert (w > 0).tolist() == [False, True, True, False, False]
    w = P.filtered_weights(logits, 0.5, 0, 0.9)
    assert (w > 0).tolist() == [False, True, True, False, False]
    assert P.draw(torch.tensor([0.0, 2.0, 2.0]), 0.49) == 1
    assert P.draw(torch.tensor([0.0, 2.0, 2.0]), 0.51) == 2
    pen = P.repeat_penalty(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 1], 2.0)
    assert pen.tolist() == [1.0, -8.0, 1.0]


def test_greedy_generate_stops():
    folder = model_folder("A", torch.float32)
    cfg, w = P.read_config(folder), P.read_weights(folder)
    out = P.greedy_generate(cfg, w, [2, 9, 77], 5)
    assert len(out) == 5
    stop = out[2]
    first = out.index(stop)
    assert P.greedy_generate(cfg, w, [2, 9, 77], 5, stop=[stop]) == out[:first]


def _reference_walk():
    """The reference's whole-model walk (tests/golden/reference_model.npz): its weights
    under the names and in the form a safetensors checkpoint has (norm weights as w, the
    file holds 1 + w), a configuration for them, and its stages."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_model.npz"))
    E, nh, nkv, hd, ff, L, V, theta, eps = z["meta"]
    cfg = {"hidden_size": int(E), "num_attention_heads": int(nh), "num_key_value_heads": int(nkv),
           "head_dim": int(hd), "intermediate_size": int(ff), "num_hidden_layers": int(L),
           "vocab_size": int(V), "rope_theta": float(theta), "rope_local_base_freq": float(theta),
           "rms_norm_eps": float(eps), "sliding_window": None, "sliding_window_pattern": 0}
    names = {"attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj",
             "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
             "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
             "attn_output": "self_attn.o_proj", "post_attention_norm": "post_attention_layernorm",
             "ffn_norm": "pre_feedforward_layernorm", "ffn_gate": "mlp.gate_proj",
             "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
             "post_ffw_norm": "post_feedforward_layernorm"}      # src/format/safetensors.zig:468-481
    w = {}
    for key in z.files:
        if not key.startswith("w:"):
            continue
        t = torch.from_numpy(z[key]).double()
        name = key[2:-len(".weight")]
        if name == "token_embd":
            w["embed_tokens.weight"] = t
        elif name == "output_norm":
            w["norm.weight"] = t - 1.0
        else:
            _, l, short = name.split(".")
            w[f"layers.{l}.{names[short]}.weight"] = t - 1.0 if short.endswith("norm") else t
    stages = {k[2:]: torch.from_numpy(z[k]).double() for k in z.files if k.startswith("s:")}
    return cfg, w, stages


def test_whole_model_order_against_the_reference_walk():
    """research/gemma3_ref.py ran the BOS token through a tiny 32-bit model; the plain
    implementation must reproduce every stage it printed: the parts of layer 0 one by
    one, the stream after each layer, the final norm and the logits."""
    cfg, w, st = _reference_walk()
    eps, nh, nkv, hd = cfg["rms_norm_eps"], cfg["num_attention_heads"], \
        cfg["num_key_value_heads"], cfg["head_dim"]
    tol = dict(rtol=2e-5, atol=2e-6)              # the walk computes in 32-bit

    def same(got, name):
        assert torch.allclose(got.reshape(-1), st[name], **tol), name

    pos = torch.arange(1)
    h0 = P.embed([2], w["embed_tokens.weight"], cfg["hidden_size"])
    same(h0, "embedding")
    p = "layers.0."
    x = P.rms_norm(h0, w[p + "input_layernorm.weight"], eps)
    same(x, "after_norm")
    q = (x @ w[p + "self_attn.q_proj.weight"].T).reshape(1, nh, hd)
    k = (x @ w[p + "self_attn.k_proj.weight"].T).reshape(1, nkv, hd)
    v = (x @ w[p + "self_attn.v_proj.weight"].T).reshape(1, nkv, hd)
    same(q, "Q"); same(k, "K"); same(v, "V")
    qn = P.rms_norm(q, w[p + "self_attn.q_norm.weight"], eps)
    kn = P.rms_norm(k, w[p + "self_attn.k_norm.weight"], eps)
    same(qn, "Q_normed"); same(kn, "K_normed")
    ang = P.rope_angles(pos, hd, cfg["rope_theta"], 1.0)
    same(P.apply_rope(qn, ang), "Q_rope")
    ao = P.attention(P.apply_rope(qn, ang), P.apply_rope(kn, ang), v, hd ** -0.5, None)
    same(ao, "attn_out")
    y = P.attention_block(cfg, w, 0, x, pos)
    same(y, "out_proj")
    h = h0 + P.rms_norm(y, w[p + "post_attention_layernorm.weight"], eps)
    same(h, "hidden_L0_attn")
    x2 = P.rms_norm(h, w[p + "pre_feedforward_layernorm.weight"], eps)
    same(x2, "after_ffn_norm")
    same(P.gelu_tanh(x2 @ w[p + "mlp.gate_proj.weight"].T) * (x2 @ w[p + "mlp.up_proj.weight"].T),
         "geglu_out")
    same(P.geglu(x2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                 w[p + "mlp.down_proj.weight"]), "ffn_down")
    # the layer function itself, layer after layer
    hl = h0
    for l in range(cfg["num_hidden_layers"]):
        hl = P.decoder_layer(cfg, w, l, hl, pos)
        same(hl, "hidden_L0_full" if l == 0 else f"hidden_L{l}")
    same(P.rms_norm(hl, w["norm.weight"], eps), "final_normed")
    same(P.forward_logits(cfg, w, [2]), "logits")
    assert int(P.forward_logits(cfg, w, [2]).argmax()) == int(st["logits"].argmax())
