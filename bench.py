#!/usr/bin/env python3
"""Measures decoding and prefill of Gemma 3 layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--shapes 1b|4b|27b] [--prompt-lens LO HI] [--prefill-tokens N]

Prints ONE JSON line.  ``value`` is decoded tokens per second of K decode
steps (random bfloat16 weights, context 8,192), timed on the device with CUDA
events; ``e2e`` is the same through ``Engine.generate`` with host token ids in
and out every step.  ``prefill`` is one 2,048-token prompt: ``ms`` for a
length whose step has been recorded, ``first_seen_ms`` for lengths never run
before (no recording: the host launches the step, through the library's C++
step function), ``first_seen_128_tokens_ms`` the same for prompts of about 128
tokens.
``roofline`` relates the decode step to the bytes it has to read; ``points``
holds decoding at the other batch sizes of the schedule.

Schedules (``--shapes``; the default, 1b, is the benchmark configuration):
  1b   batch 8 (and 1, 64), prompts of unequal lengths 128..2,048, K steps
  4b   batch 8, prompts of unequal lengths 256..4,096, 256 decoded tokens
  27b  batch 16 (and 1), prompts of 2,048 tokens, 128 decoded tokens (54 GB of weights)
A step's inputs (the weights, gigabytes) are larger than the 126 MB L2, so
every timed iteration reads them from HBM; ``config.l2`` says how many bytes.
``--layers``, ``--prompt-lens`` and ``--prefill-tokens`` measure fewer layers,
other contexts and other prompts; what they were is in ``config`` and
``prefill``.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Gemma 3 1B layer sizes (random weights, seed 2, N(0, 0.02) bfloat16)
CONFIG_1B = {
    "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
    "num_hidden_layers": 26, "hidden_size": 1152, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 256, "query_pre_attn_scalar": 256,
    "intermediate_size": 6912, "vocab_size": 262144, "sliding_window": 512,
    "sliding_window_pattern": 6, "rope_local_base_freq": 10000.0, "rope_theta": 1000000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "hidden_activation": "gelu_pytorch_tanh",
    "bos_token_id": 2, "eos_token_id": 1,
}
# layer sizes of the larger family members (--shapes 4b / 27b); the default run is 1b
CONFIG_4B = dict(CONFIG_1B, num_hidden_layers=34, hidden_size=2560, num_attention_heads=8,
                 num_key_value_heads=4, head_dim=256, query_pre_attn_scalar=256,
                 intermediate_size=10240, vocab_size=262208, sliding_window=1024,
                 rope_scaling={"rope_type": "linear", "factor": 8.0}, max_position_embeddings=131072)
CONFIG_27B = dict(CONFIG_4B, num_hidden_layers=62, hidden_size=5376, num_attention_heads=32,
                  num_key_value_heads=16, head_dim=128, query_pre_attn_scalar=168,
                  intermediate_size=21504)
SHAPES = {"1b": (CONFIG_1B, 2), "4b": (CONFIG_4B, 3), "27b": (CONFIG_27B, 4)}
# per shape: headline batch, the other batch sizes, prompt lengths, decode steps (None: --steps)
SCHEDULES = {"1b": dict(batch=8, others=(1, 64), lens=(128, 2048), steps=None),
             "4b": dict(batch=8, others=(), lens=(256, 4096), steps=256),
             "27b": dict(batch=16, others=(1,), lens=(2048, 2048), steps=128)}
CONTEXT = 8192
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6
                          for i in range(4) if s[2 + i].lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(mhz)}


def layer_kinds(cfg):
    P = cfg["sliding_window_pattern"]
    return [(P > 0 and (l + 1) % P != 0) for l in range(cfg["num_hidden_layers"])]


def decode_bytes(cfg, lens):
    """Bytes one decode step must read: every weight once, and the live cache."""
    H, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    L = cfg["num_hidden_layers"]
    per_layer = (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * ff) * 2 + (4 * H + 2 * hd) * 4
    weights = L * per_layer + V * H * 2 + H * 4
    kv = 0
    W = cfg["sliding_window"]
    for local in layer_kinds(cfg):
        for n in lens:
            kv += (min(n, W) if local else n) * nkv * hd * 2 * 2
    return weights + kv


def prefill_flops(cfg, T, rows):
    H, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    W = cfg["sliding_window"]
    lin = 2 * T * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * ff)
    total = 0
    for local in layer_kinds(cfg):
        vis = sum(min(t + 1, W) if local else t + 1 for t in range(T))
        total += lin + 4 * nh * hd * vis
    return total + 2 * rows * H * V


def run_reference(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "maci0/agave is a Zig program (build.zig); pip reports 'Neither setup.py "
                       "nor pyproject.toml found' and no zig toolchain is installed, so it "
                       "cannot be built or run here"}))
    return 0


def timed_decode(engine, torch, batch, steps, warmup, seed, lo=128, hi=2048):
    """K decode steps at one batch size, device-timed; returns (ms/step, lens, launches/step).

    The steps are the engine's own: each is staged by ``Engine._stage_step`` (the routine
    the generation loop stages its steps with), kept in a device array, and replayed
    through the engine's recorded decode step; only the token ids are this function's."""
    from agave_b200.engine.generate import RequestState
    from agave_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(seed)
    V = engine.spec.vocab_size
    lens = torch.linspace(lo, hi, batch).round().int().tolist() if batch > 1 else [(lo + hi) // 2]
    prompts = [torch.randint(3, V, (n,), generator=g).tolist() for n in lens]
    reqs = [RequestState(i, p, 1 << 30, output=[3]) for i, p in enumerate(prompts)]
    for r in reqs:
        r.slot = engine.acquire()
    # prompts in chunks of sequences, to bound the prompt step's activations
    for i in range(0, batch, 8):
        part = reqs[i:i + 8]
        engine.step([(r.slot, r.prompt) for r in part], [[] for _ in part])
    params = SamplingParams()
    total = warmup + steps
    toks = torch.randint(3, V, (total, batch), generator=g, dtype=torch.int32)
    staged = None
    for k in range(total):
        graph = engine._stage_step(reqs, params, 0, k, 0)       # the step k steps ahead
        a = graph.hosts_np[0]
        a[:batch] = toks[k].numpy()
        a[graph.flag_at] = 0                                    # token ids come from the host
        if staged is None:
            staged = torch.zeros((total, a.size), dtype=torch.int32)
        staged[k] = graph.hosts[0]
    engine.runner.cache.flush()
    staged_dev = staged.to(engine.device)
    torch.cuda.synchronize()
    per_step = graph.kernels_per_step
    for k in range(warmup):
        graph.dev.copy_(staged_dev[k])
        graph.graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for k in range(warmup, total):
        graph.dev.copy_(staged_dev[k])
        graph.graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # the last step's choices are real tokens of the vocabulary (the step ran, on these ids)
    chosen = graph.next_dev[:batch].cpu()
    assert int(chosen.min()) >= 0 and int(chosen.max()) < V, "the decode step chose no tokens"
    book = engine.runner.cache.book
    final_lens = [book.length[r.slot] + total for r in reqs]
    for r in reqs:
        engine.release(r.slot)
    return ms, final_lens, per_step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shapes", default="1b", choices=sorted(SHAPES),
                    help="layer sizes to run (the default, 1b, is the benchmark configuration)")
    ap.add_argument("--prompt-lens", type=int, nargs=2, default=None, metavar=("LO", "HI"),
                    help="the decode batches' prompt lengths run from LO to HI (default: the "
                         "schedule's, 128 to 2,048 for the benchmark configuration)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (default: the benchmark configuration's)")
    args = ap.parse_args()
    sched = SCHEDULES[args.shapes]
    lo, hi = args.prompt_lens or sched["lens"]
    steps = args.steps if sched["steps"] is None else sched["steps"]
    n_pre = args.prefill_tokens
    if not (0 < lo <= hi and hi + steps + max(3, args.warmup) + 1 <= CONTEXT
            and 8 <= n_pre <= CONTEXT):
        print(f"bench.py: prompts and the decoded tokens must fit the context of {CONTEXT}")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus must be 1")
        return 2
    args.warmup = max(3, args.warmup)

    import torch
    from agave_b200.engine.api import Engine

    base_cfg, seed = SHAPES[args.shapes]
    cfg = dict(base_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    batch = sched["batch"]
    max_batch = max((batch,) + tuple(sched["others"]))
    engine = Engine.from_config(cfg, seed=seed, std=0.02, norm_std=0.1, dtype="bfloat16",
                                max_tokens=max_batch * CONTEXT, ctx_size=CONTEXT,
                                max_batch=max_batch)
    V = engine.spec.vocab_size
    g = torch.Generator().manual_seed(5)

    def timed_prompt(tokens):
        s = engine.acquire()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([(s, tokens)], [[len(tokens) - 1]])
        e1.record()
        torch.cuda.synchronize()
        engine.release(s)
        return e0.elapsed_time(e1)

    # ---- prefill: one prompt (2,048 tokens by default), logits of its last token ----
    prompt = torch.randint(3, V, (n_pre,), generator=g).tolist()
    # lengths never run before: no recorded step, the host launches kernel by kernel
    # (the first of them also pays what a kernel's first use costs, so it is not counted)
    first_seen = sorted(timed_prompt(prompt[:n_pre - k]) for k in (7, 5, 3, 1))[:3]
    first_seen_ms = sorted(first_seen)[1]
    # the same for short prompts (time to the first token of a chat turn): what the host
    # needs to launch a step bounds these
    short = sorted(timed_prompt(prompt[:128 - k]) for k in (7, 5, 3, 1))[:3]
    short_ms = sorted(short)[1]
    pre_ms = [timed_prompt(prompt) for _ in range(3 + 5)][3:]
    pre_ms = sorted(pre_ms)[len(pre_ms) // 2]
    pflops = prefill_flops(cfg, n_pre, 1)
    prefill = {"value": round(n_pre / pre_ms * 1e3, 1), "tokens": n_pre,
               "ms": round(pre_ms, 3),
               "frac": round(pflops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "first_seen_ms": round(first_seen_ms, 3),
               "first_seen_128_tokens_ms": round(short_ms, 3)}

    # ---- decode at the headline batch, with clocks sampled meanwhile ----
    clocks = ClockSampler()
    clocks.start()
    ms_b, lens_b, launches = timed_decode(engine, torch, batch, steps, args.warmup, 8, lo, hi)
    clock_rec = clocks.stop()
    value = batch / ms_b * 1e3
    nbytes = decode_bytes(cfg, lens_b)
    achieved = nbytes / (ms_b * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                "of": pk["source"], "bytes_per_step": nbytes}

    # ---- the other batch sizes ----
    points = {}
    for b in sched["others"]:
        k = steps if b <= 16 else max(8, steps // 2)
        ms, _, _ = timed_decode(engine, torch, b, k, args.warmup, b, lo, hi)
        points[f"decode_b{b}"] = round(b / ms * 1e3, 1)

    # ---- end to end through the Python entry point ----
    lens = torch.linspace(lo, hi, batch).round().int().tolist()
    prompts = [torch.randint(3, V, (n,), generator=g).tolist() for n in lens]
    n_new = steps + 1
    engine.generate(prompts, max_new_tokens=4, stop_token_ids=[])           # warm-up
    engine.generate(prompts, max_new_tokens=n_new, stop_token_ids=[])
    st = engine.stats
    e2e_val = st["decode_tokens"] / st["decode_seconds"]
    graph = next(iter(engine._graphs.values()))
    e2e = {"value": round(e2e_val, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int(graph.hosts[0].numel() * 4),
           "d2h_bytes_per_step": int(graph.next_hosts[0].numel() * 4)}

    weight_gb = (decode_bytes(cfg, [0]) / 1e9)
    out = {
        "metric": f"Gemma3-{args.shapes.upper()} bf16 decode tokens/s at batch {batch} "
                  f"(context {CONTEXT})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(ms_b, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"gemma3-{args.shapes}-shapes-random", "layers": cfg["num_hidden_layers"],
            "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "sliding_window": cfg["sliding_window"],
            "local_per_global": cfg["sliding_window_pattern"] - 1, "global_batch": batch,
            "seq_len": CONTEXT, "prompt_lens": f"{lo}..{hi}" + (" unequal" if lo != hi else ""),
            "seed": seed, "parallelism": "single-gpu", "cache": "paged bf16",
            "l2": f"inputs larger than L2 ({weight_gb:.1f} GB weights per step)"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": int(launches * steps), "clocks": clock_rec,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
