"""A plain, slow Gemma 3 text decoder for comparison: whole sequences, no cache.

One function per part, written from the formulas of the reference engine
(maci0/agave); every function cites the file and lines it restates.  Nothing
here is imported by, or imports, the library under test: this file reads
``config.json`` as a dictionary and the weights through the ``safetensors``
package.

The reference's own model code is Zig and cannot be compiled here (no Zig
toolchain), so the whole-model result rests on the formulas.  The parts that
the reference also has as importable Python (research/kernels/reference.py:
rms_norm, gelu, rope, sdpa) are compared once with these functions by
``tests/golden/make_golden.py``, whose small outputs are committed.

Arithmetic runs in the dtype of the tensors handed in (float64 by default).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

PREFIXES = ("model.", "language_model.model.", "model.language_model.", "")
# src/format/safetensors.zig:517-521


# --------------------------------------------------------------------- inputs
def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        d = json.load(f)
    if isinstance(d.get("text_config"), dict):      # src/format/safetensors.zig:1827-1831
        d = {**d, **d["text_config"]}
    return d


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    out = {}
    for name in sorted(os.listdir(folder)):
        if name.endswith(".safetensors"):
            for k, v in load_file(os.path.join(folder, name)).items():
                out[k] = v.to(dtype)
    for p in PREFIXES:
        if p + "embed_tokens.weight" in out:
            n = len(p)
            named = {(k[n:] if k.startswith(p) else k): v for k, v in out.items()}
            # a head of its own sits beside the decoder, under the outer part of the
            # prefix or none (src/format/safetensors.zig:531-540)
            for k in list(named):
                if k.endswith("lm_head.weight") and k != "lm_head.weight":
                    named["lm_head.weight"] = named.pop(k)
            return named
    raise KeyError("embed_tokens.weight not found under any known prefix")


def layer_is_local(cfg: dict, layer: int) -> bool:
    """src/models/gemma3.zig:736: local iff pattern > 0 and (l+1) % pattern != 0;
    an explicit ``layer_types`` list, where the file has one, says the same."""
    if cfg.get("layer_types") is not None:
        return cfg["layer_types"][layer] == "sliding_attention"
    pattern = cfg.get("sliding_window_pattern")
    if pattern is None:     # src/models/gemma3.zig:185-187
        pattern = 6 if cfg.get("sliding_window") is not None else 0
    return pattern > 0 and (layer + 1) % pattern != 0


def rope_factor(cfg: dict) -> float:
    """Linear scaling factor of global layers (src/models/gemma3.zig:179-183)."""
    s = cfg.get("rope_scaling")
    if isinstance(s, dict) and s.get("rope_type", s.get("type")) == "linear":
        return float(s.get("factor", 1.0))
    return 1.0


# ---------------------------------------------------------------------- parts
def embed(tokens: Sequence[int], table: torch.Tensor, hidden: int) -> torch.Tensor:
    """h0 = E[token] * sqrt(H) (src/models/gemma3.zig:195,1017-1046)."""
    idx = torch.as_tensor(list(tokens), dtype=torch.long)
    return table[idx] * math.sqrt(float(hidden))


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, add_one: bool = True) -> torch.Tensor:
    """x * w' / sqrt(mean(x^2) + eps) over the last axis, eps inside the root
    (src/backend/kernels/cpu/norm.zig:29-39); w' = 1 + w for safetensors
    checkpoints (src/models/gemma3.zig:199-202,943-949)."""
    ww = w + 1.0 if add_one else w
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * ww


def rope_angles(positions: torch.Tensor, rotary_dim: int, theta: float, factor: float,
                dtype=torch.float64) -> torch.Tensor:
    """angle[p, i] = (p / factor) * theta^(-2i/rotary_dim)
    (src/backend/kernels/cpu/rope.zig:11-27; scaled: src/models/gemma3.zig:884-902)."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    freq = torch.exp(-math.log(theta) * 2.0 * i / rotary_dim)
    p = positions.to(torch.float64) * (1.0 / factor)
    return (p[:, None] * freq[None, :]).to(dtype)


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, hd]; pairs (i, i + half) rotate together
    (src/backend/kernels/cpu/rope.zig:29-47)."""
    half = angles.shape[1]
    c = torch.cos(angles)[:, None, :].to(x.dtype)
    s = torch.sin(angles)[:, None, :].to(x.dtype)
    re, im = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = re * c - im * s
    out[..., half:2 * half] = re * s + im * c
    return out


def visible(n: int, window: Optional[int]) -> torch.Tensor:
    """mask[p, j]: causal j <= p (src/backend/kernels/cuda/sdpa_prefill.zig:50);
    with a window W also p - W < j (start = sl - W for sl = p + 1 > W,
    src/models/gemma4.zig:1153-1155)."""
    p = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    m = j <= p
    if window is not None:
        m = m & (j > p - window)
    return m


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int]) -> torch.Tensor:
    """q: [T, nh, hd], k, v: [T, nkv, hd] -> [T, nh*hd].  Query head h uses kv
    head h // (nh/nkv) (src/backend/kernels/cpu/sdpa.zig:36-37); score =
    (q . k) * scale (sdpa.zig:58); softmax with the maximum subtracted
    (sdpa.zig:184-234); no soft cap, no sinks."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    mask = visible(T, window)
    out = torch.zeros(T, nh, hd, dtype=q.dtype)
    for h in range(nh):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        e = torch.exp(s)
        a = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = a @ v[:, g, :]
    return out.reshape(T, nh * hd)


def gelu_tanh(t: torch.Tensor) -> torch.Tensor:
    """0.5 t (1 + tanh(sqrt(2/pi) (t + 0.044715 t^3))) (src/ops/math.zig:8-10,
    src/backend/kernels/cpu/activation.zig:69-112)."""
    return 0.5 * t * (1.0 + torch.tanh(0.7978845608028654 * (t + 0.044715 * t * t * t)))


def geglu(x: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """down(gelu(gate x) * up x), no biases (src/models/gemma3.zig:840-872)."""
    return (gelu_tanh(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def attention_block(cfg: dict, w: Dict[str, torch.Tensor], l: int, x: torch.Tensor,
                    positions: torch.Tensor) -> torch.Tensor:
    """q/k/v projections, per-head q and k norms before the rotation, rotation
    with the layer kind's base, attention, output projection
    (src/models/gemma3.zig:714-748,795-820)."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = x.shape[0]
    pre = f"layers.{l}.self_attn."
    q = (x @ w[pre + "q_proj.weight"].T).reshape(T, nh, hd)
    k = (x @ w[pre + "k_proj.weight"].T).reshape(T, nkv, hd)
    v = (x @ w[pre + "v_proj.weight"].T).reshape(T, nkv, hd)
    q = rms_norm(q, w[pre + "q_norm.weight"], eps)
    k = rms_norm(k, w[pre + "k_norm.weight"], eps)
    local = layer_is_local(cfg, l)
    if local:
        ang = rope_angles(positions, hd, cfg.get("rope_local_base_freq", 1e4), 1.0, x.dtype)
    else:
        ang = rope_angles(positions, hd, cfg.get("rope_theta", 1e6), rope_factor(cfg), x.dtype)
    q, k = apply_rope(q, ang), apply_rope(k, ang)
    qpas = cfg.get("query_pre_attn_scalar", hd)          # src/models/gemma3.zig:190-194
    o = attention(q, k, v, 1.0 / math.sqrt(qpas), cfg["sliding_window"] if local else None)
    return o @ w[pre + "o_proj.weight"].T


def decoder_layer(cfg: dict, w: Dict[str, torch.Tensor], l: int, h: torch.Tensor,
                  positions: torch.Tensor) -> torch.Tensor:
    """Norm before each branch, norm on the branch's output, then the sum
    (src/models/gemma3.zig:708-709,824-826,835-836,876-878)."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    p = f"layers.{l}."
    y = attention_block(cfg, w, l, rms_norm(h, w[p + "input_layernorm.weight"], eps), positions)
    h = h + rms_norm(y, w[p + "post_attention_layernorm.weight"], eps)
    d = geglu(rms_norm(h, w[p + "pre_feedforward_layernorm.weight"], eps),
              w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
              w[p + "mlp.down_proj.weight"])
    return h + rms_norm(d, w[p + "post_feedforward_layernorm.weight"], eps)


def forward_hidden(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """The stream [T, H] after the last layer of one whole sequence starting at
    position 0: embedding, then the layers in order (src/models/gemma3.zig:331-351)."""
    T = len(tokens)
    positions = torch.arange(T)
    h = embed(tokens, w["embed_tokens.weight"], cfg["hidden_size"])
    for l in range(cfg["num_hidden_layers"]):
        h = decoder_layer(cfg, w, l, h, positions)
    return h


def logits_at(cfg: dict, w: Dict[str, torch.Tensor], h: torch.Tensor,
              rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Final norm and head on the given rows of the stream (all by default): the
    head is tied to the embedding unless the file has lm_head.weight; no soft cap
    (src/models/gemma3.zig:352-367)."""
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rms_norm(h, w["norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w.get("lm_head.weight", w["embed_tokens.weight"])
    return x @ head.T


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] of one whole sequence starting at position 0
    (src/models/gemma3.zig:331-368)."""
    return logits_at(cfg, w, forward_hidden(cfg, w, tokens))


# ----------------------------------------------------------------- generation
def argmax_first(row: torch.Tensor) -> int:
    """Greatest value, first index on ties (src/ops/math.zig:32-50)."""
    m = row.max()
    return int(torch.nonzero(row >= m)[0, 0])


def greedy_generate(cfg: dict, w, prompt: Sequence[int], n_new: int,
                    stop: Sequence[int] = ()) -> List[int]:
    """Whole-sequence recomputation per token; a stop token ends the sequence
    and is not returned (src/main.zig:2366-2369)."""
    seq = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        t = argmax_first(forward_logits(cfg, w, seq)[-1])
        if t in stop:
            break
        out.append(t)
        seq.append(t)
    return out


# ------------------------------------------------------------------- sampling
def repeat_penalty(logits: torch.Tensor, recent: Sequence[int], penalty: float) -> torch.Tensor:
    """Positive logits divided, others multiplied (src/ops/math.zig:186-197)."""
    out = logits.clone()
    for t in recent:
        if t < out.numel():
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def filtered_weights(logits: torch.Tensor, temperature: float, top_k: int,
                     top_p: float) -> torch.Tensor:
    """Unnormalised weights the draw is made from (src/ops/math.zig:209-362):
    logits / T; keep values >= the k-th greatest; exp(x - max); then keep
    weights >= the one at which the descending cumulative sum first reaches
    top_p * total."""
    x = logits.to(torch.float64) / temperature
    n = x.numel()
    if 0 < top_k < n:
        kth = torch.topk(x, top_k).values[-1]
        x = torch.where(x < kth, torch.full_like(x, float("-inf")), x)
    wts = torch.exp(x - x.max())
    if 0.0 < top_p < 1.0:
        srt = torch.sort(wts, descending=True).values
        cum = torch.cumsum(srt, 0)
        idx = int(torch.nonzero(cum >= top_p * wts.sum())[0, 0])
        wts = torch.where(wts >= srt[idx], wts, torch.zeros_like(wts))
    return wts


def draw(weights: torch.Tensor, u: float) -> int:
    """First index whose running sum exceeds u * total, else the last
    (src/ops/math.zig:364-371)."""
    thr = u * float(weights.sum())
    cum = torch.cumsum(weights, 0)
    hit = torch.nonzero(cum > thr)
    return int(hit[0, 0]) if hit.numel() else weights.numel() - 1
