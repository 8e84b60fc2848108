"""Makes the golden files from the reference's own Python code (maci0/agave),
which imports on a CPU without any checkpoint.

    python tests/golden/make_golden.py /path/to/agave

``reference_kernels.npz``: the part-level functions of
research/kernels/reference.py (rms_norm, gelu, rope, sdpa).

``reference_model.npz``: the reference's whole-model walk,
research/gemma3_ref.py, which runs the BOS token through every layer of a GGUF
file and prints each stage.  Here it is given a tiny 32-bit GGUF file written
by this script (norm weights with the +1 baked in, as GGUF files have them,
docs/MODELS.md:32) and its ``dump`` is replaced by a collector, so the stages
(embedding, normed q and k, attention output, the stream after each branch and
each layer, the final norm, the logits) are stored beside the weights that made
them.  That pins the order of operations of a whole layer and of the model on
the reference's own output: the embedding scale, norm before and after each
branch, the per-head q/k norm, one kv head serving several query heads, the
gated feed-forward, the final norm and the tied head.  What that walk cannot
show (it runs one token at position 0 with one rotary base): the window, the
two rotary bases and the scaling of global layers, the 1 + w of safetensors
norm weights; those rest on the formulas cited in tests/plain/gemma3_plain.py.

The reference's model code proper is Zig and cannot be compiled here.  Inputs
are seeded and stored with the outputs, so the comparison needs neither the
reference nor a seed.
"""
import contextlib
import importlib.util
import io
import os
import struct
import sys
import tempfile

import numpy as np
import torch

# the tiny model of the whole-model walk: three layers, two query heads on one kv head
MODEL = dict(n_embd=32, n_head=2, n_head_kv=1, head_dim=16, n_ff=48, n_layers=3, vocab=64,
             rope_theta=10000.0, rms_eps=1e-5)


def _gguf_string(s):
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, meta, tensors):
    """A GGUF (version 3) file of 32-bit tensors.  ``meta``: {key: int | float | str};
    ``tensors``: {name: array}; a matrix [out, in] is listed with its dims reversed, as
    GGUF does (research/gemma3_ref.py:62-70, 211)."""
    head = b"GGUF" + struct.pack("<I", 3) + struct.pack("<Q", len(tensors)) + \
        struct.pack("<Q", len(meta))
    for k, v in meta.items():
        head += _gguf_string(k)
        if isinstance(v, str):
            head += struct.pack("<I", 8) + _gguf_string(v)
        elif isinstance(v, float):
            head += struct.pack("<If", 6, v)
        else:
            head += struct.pack("<II", 4, v)
    offset, blobs = 0, []
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        head += _gguf_string(name) + struct.pack("<I", arr.ndim)
        for d in reversed(arr.shape):
            head += struct.pack("<Q", d)
        head += struct.pack("<IQ", 0, offset)
        blob = arr.tobytes()
        blob += b"\0" * ((32 - len(blob) % 32) % 32)
        blobs.append(blob)
        offset += len(blob)
    head += b"\0" * ((32 - len(head) % 32) % 32)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


def whole_model(root):
    m = MODEL
    g = torch.Generator().manual_seed(4321)

    def mat(*shape, std=0.08):
        return (torch.randn(*shape, generator=g) * std).numpy().astype(np.float32)

    def norm(n):      # as a GGUF file holds it: 1 + w
        return (1.0 + torch.randn(n, generator=g) * 0.2).numpy().astype(np.float32)

    E, nh, nkv, hd, ff = m["n_embd"], m["n_head"], m["n_head_kv"], m["head_dim"], m["n_ff"]
    t = {"token_embd.weight": mat(m["vocab"], E, std=0.5), "output_norm.weight": norm(E)}
    for l in range(m["n_layers"]):
        b = f"blk.{l}."
        t[b + "attn_norm.weight"] = norm(E)
        t[b + "attn_q.weight"] = mat(nh * hd, E)
        t[b + "attn_k.weight"] = mat(nkv * hd, E)
        t[b + "attn_v.weight"] = mat(nkv * hd, E)
        t[b + "attn_q_norm.weight"] = norm(hd)
        t[b + "attn_k_norm.weight"] = norm(hd)
        t[b + "attn_output.weight"] = mat(E, nh * hd)
        t[b + "post_attention_norm.weight"] = norm(E)
        t[b + "ffn_norm.weight"] = norm(E)
        t[b + "ffn_gate.weight"] = mat(ff, E)
        t[b + "ffn_up.weight"] = mat(ff, E)
        t[b + "ffn_down.weight"] = mat(E, ff)
        t[b + "post_ffw_norm.weight"] = norm(E)
    meta = {"general.architecture": "gemma3", "gemma3.embedding_length": E,
            "gemma3.attention.head_count": nh, "gemma3.attention.head_count_kv": nkv,
            "gemma3.attention.key_length": hd, "gemma3.feed_forward_length": ff,
            "gemma3.block_count": m["n_layers"], "gemma3.rope.freq_base": m["rope_theta"],
            "gemma3.attention.layer_norm_rms_epsilon": m["rms_eps"]}
    path = os.path.join(root, "research", "gemma3_ref.py")
    spec = importlib.util.spec_from_file_location("agave_gemma3_ref", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    stages = {}
    ref.dump = lambda label, v: stages.__setitem__(label, np.array(v, dtype=np.float32))
    with tempfile.TemporaryDirectory() as d:
        gguf = os.path.join(d, "tiny.gguf")
        write_gguf(gguf, meta, t)
        argv, sys.argv = sys.argv, ["gemma3_ref.py", gguf]
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                ref.main()
        finally:
            sys.argv = argv
    out = {"w:" + k: v for k, v in t.items()}
    out.update({"s:" + k: v for k, v in stages.items()})
    out["meta"] = np.array([E, nh, nkv, hd, ff, m["n_layers"], m["vocab"], m["rope_theta"],
                            m["rms_eps"]], dtype=np.float64)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_model.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes;", len(stages), "stages:",
          ", ".join(stages))


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/agave")
    root = sys.argv[1]
    path = os.path.join(root, "research", "kernels", "reference.py")
    spec = importlib.util.spec_from_file_location("agave_reference_kernels", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = torch.Generator().manual_seed(1234)
    out = {}
    # rms_norm: x / sqrt(mean(x^2) + eps) * weight (weight applied as given)
    x = torch.randn(96, generator=g)
    w = torch.randn(96, generator=g) * 0.2 + 1.0
    out["norm_x"], out["norm_w"] = x.numpy(), w.numpy()
    out["norm_y"] = ref.rms_norm(x, w, eps=1e-5).numpy()
    # gelu (tanh form)
    t = torch.linspace(-6, 6, 97)
    out["gelu_x"], out["gelu_y"] = t.numpy(), ref.gelu(t).numpy()
    # rope: 3 q heads / 1 k head of 32, position 37, theta 5000
    nh, nkv, hd, pos, theta = 3, 1, 32, 37, 5000.0
    q = torch.randn(nh * hd, generator=g)
    k = torch.randn(nkv * hd, generator=g)
    # the reference function takes q and k of equal head count: call it once for each
    qo, _ = ref.rope(q, q, pos, hd, hd, theta)
    ko, _ = ref.rope(k, k, pos, hd, hd, theta)
    out["rope_q"], out["rope_k"] = q.numpy(), k.numpy()
    out["rope_qo"], out["rope_ko"] = qo.numpy(), ko.numpy()
    out["rope_meta"] = np.array([nh, nkv, hd, pos, theta], dtype=np.float64)
    # sdpa: one query over 9 cached positions, 4 heads / 2 kv heads of 16
    nh, nkv, hd, sl = 4, 2, 16, 9
    q = torch.randn(nh * hd, generator=g)
    keys = torch.randn(sl * nkv * hd, generator=g)
    vals = torch.randn(sl * nkv * hd, generator=g)
    scale = 1.0 / 24 ** 0.5
    out["sdpa_q"], out["sdpa_k"], out["sdpa_v"] = q.numpy(), keys.numpy(), vals.numpy()
    out["sdpa_o"] = ref.sdpa(q, keys, vals, nh, nkv, hd, scale).numpy()
    out["sdpa_meta"] = np.array([nh, nkv, hd, sl, scale], dtype=np.float64)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz")
    np.savez(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")
    whole_model(root)


if __name__ == "__main__":
    main()
