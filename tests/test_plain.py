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
