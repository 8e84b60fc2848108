"""Makes tests/golden/reference_kernels.npz from the reference's own Python
kernel references (research/kernels/reference.py of maci0/agave), which import
on a CPU without any checkpoint.

    python tests/golden/make_golden.py /path/to/agave

The reference's model code is Zig and cannot be compiled here, so only these
part-level functions anchor the plain implementation (rms_norm, gelu, rope,
sdpa); the whole model rests on the formulas.  Inputs are seeded and stored
with the outputs, so the comparison needs neither the reference nor a seed.
"""
import importlib.util
import os
import sys

import numpy as np
import torch


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


if __name__ == "__main__":
    main()
