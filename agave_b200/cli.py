"""Command line in the manner of the reference's ``agave`` program.

    python -m agave_b200 [OPTIONS] <model-dir> [prompt]

Option names and meanings are the reference's where it has them
(src/main.zig:325-382, usage text 801-901): ``-n/--max-tokens`` (512),
``-t/--temperature`` (0 = greedy), ``--top-p`` (1.0), ``--top-k`` (0),
``--repeat-penalty`` (1.0), ``--seed`` (random), ``--ctx-size`` (0 = the model's
own limit; default min(model, 4096)), ``-q/--quiet``, ``--json``,
``--model-info``, ``-V/--verbose``, ``-d/--debug``, ``-v/--version``.
Options of what this library does not have (other backends, quantised caches,
server, vision, speculative decoding, grammars) are not offered.  Added here:
``--tokens`` (a prompt as token ids), ``--dtype``, ``--max-batch``,
``--random-weights SEED`` (the folder then needs only ``config.json``: seeded random
weights are drawn on the device) and ``--strict`` (refuse folders that hold tensors the
decoder does not ask for).  ``--profile`` prints the reference's per-operation table
(src/perf.zig:84-130), with device times, for a run whose steps go launch by launch.

A text prompt needs ``tokenizer.json`` in the model folder; it is wrapped in
the Gemma chat template (src/chat_template.zig:153-161) after the BOS token
(src/main.zig:2199-2208).  Without a tokenizer, give ``--tokens``; the output
is then token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, List, Optional

from . import __version__

DEFAULT_CTX = 4096        # src/main.zig:1102-1113


class SimpleTokenizer:
    """Greedy longest-match over the vocabulary of ``tokenizer.json``, spaces as
    the SentencePiece mark, no dummy prefix (src/tokenizer/bpe.zig:396-430);
    decoding joins the pieces (bpe.zig:566).  Enough for the command line; the
    library's contract is token ids."""

    SPACE = "▁"

    def __init__(self, path: str):
        with open(path, "r", encoding="utf-8") as f:
            data = json.load(f)
        vocab = data.get("model", {}).get("vocab", {})
        if isinstance(vocab, list):          # unigram form: [[piece, score], ...]
            vocab = {p[0]: i for i, p in enumerate(vocab)}
        for t in data.get("added_tokens", []):
            vocab.setdefault(t["content"], t["id"])
        if not vocab:
            raise ValueError(f"{path}: no vocabulary found")
        self.vocab: Dict[str, int] = vocab
        self.pieces = {i: p for p, i in vocab.items()}
        self.max_len = max(len(p) for p in vocab)
        self.specials = sorted((t["content"] for t in data.get("added_tokens", [])),
                               key=len, reverse=True)

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        norm_cache: Dict[int, str] = {}
        while i < len(text):
            hit = next((s for s in self.specials if text.startswith(s, i)), None)
            if hit is not None:
                out.append(self.vocab[hit])
                i += len(hit)
                continue
            for n in range(min(self.max_len, len(text) - i), 0, -1):
                piece = text[i:i + n].replace(" ", self.SPACE)
                if piece in self.vocab:
                    out.append(self.vocab[piece])
                    i += n
                    break
            else:
                for b in text[i].encode("utf-8"):        # byte fallback pieces
                    key = f"<0x{b:02X}>"
                    if key in self.vocab:
                        out.append(self.vocab[key])
                i += 1
        return out

    def decode(self, ids: List[int]) -> str:
        return "".join(self.pieces.get(i, "") for i in ids).replace(self.SPACE, " ")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(
        prog="agave_b200", add_help=False,
        description="Gemma 3 generation on one B200 (after the agave command line).")
    p.add_argument("model", nargs="?", help="model folder (config.json + safetensors)")
    p.add_argument("prompt", nargs="?", help="text prompt (needs tokenizer.json)")
    g = p.add_argument_group("GENERAL")
    g.add_argument("-h", "--help", action="help", help="Show this help message and exit.")
    g.add_argument("-v", "--version", action="store_true", help="Print version and exit.")
    g.add_argument("-q", "--quiet", action="store_true",
                   help="Suppress banner and stats (raw output only).")
    g = p.add_argument_group("GENERATION")
    g.add_argument("-n", "--max-tokens", type=int, default=512,
                   help="Maximum tokens to generate [default: 512].")
    g.add_argument("-t", "--temperature", type=float, default=0.0,
                   help="Sampling temperature, 0 = greedy [default: 0].")
    g.add_argument("--top-p", type=float, default=1.0,
                   help="Nucleus sampling threshold [default: 1.0].")
    g.add_argument("--top-k", type=int, default=0,
                   help="Top-k sampling, 0 = disabled [default: 0].")
    g.add_argument("--repeat-penalty", type=float, default=1.0,
                   help="Repetition penalty [default: 1.0].")
    g.add_argument("--seed", type=int, default=None,
                   help="Random seed for sampling [default: random].")
    g.add_argument("--system", default=None, help="System prompt for chat formatting.")
    g.add_argument("--tokens", default=None,
                   help="Prompt as comma-separated token ids; several prompts separated by ';'.")
    g = p.add_argument_group("MODEL")
    g.add_argument("--ctx-size", type=int, default=None,
                   help="Context window size; 0 = full model context [default: min(model, 4096)].")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                   help="Compute dtype [default: bfloat16].")
    g.add_argument("--max-batch", type=int, default=None,
                   help="Most sequences in one batch [default: as many as prompts].")
    g.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="Draw seeded random weights for the folder's config.json instead of "
                        "reading tensors.")
    g.add_argument("--strict", action="store_true",
                   help="Refuse a folder that holds tensors the decoder does not ask for.")
    g = p.add_argument_group(
        "OPTIONS OF THE REFERENCE WITHOUT A COUNTERPART HERE",
        "Accepted where they name what this library does anyway, refused with the reason where "
        "they ask for what it does not have.")
    g.add_argument("--backend", default="auto",
                   help="Compute backend: only auto and cuda exist here [default: auto].")
    g.add_argument("--color", default="auto", help="Color mode (output here is plain; ignored).")
    g.add_argument("--no-color", action="store_true", help="Same as --color=never (ignored).")
    g.add_argument("--mmap", action="store_true",
                   help="Lazy weight mapping (weights are read straight to the GPU; ignored).")
    g.add_argument("--prefill-batch-size", type=int, default=None,
                   help="Prefill chunk size (a prompt runs as one step here; ignored).")
    g.add_argument("--allow-cpu-fallback", action="store_true", help="Refused: there is no CPU path.")
    g.add_argument("--kv-type", default=None,
                   help="Cache element type: bf16 (f16 is read as bf16) with --dtype bfloat16, f32 "
                        "with --dtype float32; quantised caches are refused.")
    for name in ("--kv-type-k", "--kv-type-v", "--cache-type-k", "--cache-type-v"):
        g.add_argument(name, default=None, help="As --kv-type.")
    for name, why in (("--kv-tiers", "tiered caches"), ("--kv-eviction", "cache eviction"),
                      ("--grammar", "constrained decoding"), ("--grammar-string", "constrained decoding"),
                      ("--draft-model", "speculative decoding"), ("--mmproj", "vision input"),
                      ("--image", "vision input")):
        g.add_argument(name, default=None, help=f"Refused: no {why} here.")
    for name, why in (("--json-output", "constrained decoding"), ("--serve", "server"),
                      ("--megakernel", "quantised single-launch kernels")):
        g.add_argument(name, action="store_true", help=f"Refused: no {why} here.")
    g = p.add_argument_group("DIAGNOSTICS")
    g.add_argument("-V", "--verbose", action="store_true",
                   help="Show technical details (params, load times, EOG).")
    g.add_argument("-d", "--debug", action="store_true",
                   help="Enable debug logging (token IDs); implies --verbose.")
    g.add_argument("--json", action="store_true", help="Output results as JSON (implies --quiet).")
    g.add_argument("--model-info", action="store_true",
                   help="Print model metadata and exit (supports --json).")
    g.add_argument("--profile", action="store_true",
                   help="Print a per-operation table of device times (steps then run launch by "
                        "launch).")
    return p


def _peaks() -> dict:
    """Measured memory and tensor peaks of this GPU, if a record of them is around:
    the JSON file $AGAVE_B200_PEAKS names, else MEASURED_PEAKS.json beside the package."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for path in (os.environ.get("AGAVE_B200_PEAKS"), os.path.join(here, "MEASURED_PEAKS.json")):
        if path and os.path.isfile(path):
            try:
                with open(path) as f:
                    p = json.load(f)
                return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"])}
            except (OSError, ValueError, KeyError):
                pass
    return {}


def _fail(msg: str) -> int:
    print(f"Error: {msg}", file=sys.stderr)
    return 1


def _unsupported(args) -> Optional[str]:
    """Why an option of the reference's command line cannot be honoured here, or None."""
    if args.backend not in ("auto", "cuda"):
        return f"--backend {args.backend}: this library runs on CUDA (sm_100a) only"
    if args.allow_cpu_fallback:
        return "--allow-cpu-fallback: there is no CPU path"
    want = {"bfloat16": ("bf16", "f16", "fp16", "bfloat16", "float16"),
            "float32": ("f32", "fp32", "float32")}[args.dtype]
    for name in ("kv_type", "kv_type_k", "kv_type_v", "cache_type_k", "cache_type_v"):
        v = getattr(args, name)
        if v is not None and v.lower() not in want:
            return (f"--{name.replace('_', '-')} {v}: the cache holds {args.dtype} with --dtype "
                    f"{args.dtype}; there are no quantised or mixed caches")
    for name, why in (("kv_tiers", "tiered caches"), ("kv_eviction", "cache eviction"),
                      ("grammar", "constrained decoding"), ("grammar_string", "constrained decoding"),
                      ("json_output", "constrained decoding"), ("draft_model", "speculative decoding"),
                      ("mmproj", "vision input"), ("image", "vision input"), ("serve", "a server"),
                      ("megakernel", "quantised single-launch kernels")):
        v = getattr(args, name)
        if v not in (None, False) and not (name == "kv_eviction" and v == "none"):
            return f"--{name.replace('_', '-')}: this library has no {why}"
    return None


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.version:
        print(f"agave_b200 {__version__}")
        return 0
    if not args.model:
        build_parser().print_usage(sys.stderr)
        return _fail("no model folder given")
    if not os.path.isdir(args.model):
        return _fail(f"'{args.model}' is not a model folder")
    if args.random_weights is not None and args.strict:
        return _fail("--strict is about tensors in files; --random-weights reads none")
    refusal = _unsupported(args)
    if refusal:
        return _fail(refusal)
    # the reference's own validation (src/main.zig:555-573)
    if args.temperature < 0:
        return _fail("--temperature must be >= 0")
    if not (0.0 < args.top_p <= 1.0):
        return _fail("--top-p must be in (0, 1]")
    if args.repeat_penalty <= 0:
        return _fail("--repeat-penalty must be > 0")
    if args.max_tokens < 0:
        return _fail("--max-tokens must be >= 0")
    args.verbose = args.verbose or args.debug
    quiet = args.quiet or args.json

    from .config import ConfigError, load_config, read_config_json, resolve_architecture
    from .weights import SafetensorsError, WeightsError
    try:
        if args.random_weights is not None:
            raw_config = read_config_json(args.model)
            entry = resolve_architecture(raw_config)
            config = entry.config_class.from_dict(raw_config)
        else:
            entry, config = load_config(args.model)
    except ConfigError as e:
        return _fail(str(e))
    spec = config.to_model_spec()
    model_ctx = spec.max_positions or DEFAULT_CTX
    if args.ctx_size is None:
        ctx = min(model_ctx, DEFAULT_CTX)
    elif args.ctx_size == 0:
        ctx = model_ctx
    else:
        ctx = min(args.ctx_size, model_ctx)

    tok = None
    tok_path = os.path.join(args.model, "tokenizer.json")
    if os.path.isfile(tok_path):
        tok = SimpleTokenizer(tok_path)
    prompts: List[List[int]] = []
    if args.tokens is not None:
        try:
            for part in args.tokens.split(";"):
                ids = [int(t) for t in part.replace(" ", "").split(",") if t != ""]
                if ids:
                    prompts.append(ids)
        except ValueError:
            return _fail("--tokens takes comma-separated integers")
    elif not args.model_info and (args.prompt is not None or not sys.stdin.isatty()):
        text = args.prompt if args.prompt is not None else sys.stdin.read().strip()
        if not text:
            return _fail("no prompt: give text, --tokens, or pipe text in (there is no REPL here)")
        if tok is None:
            return _fail(f"{args.model} has no tokenizer.json: give the prompt as --tokens")
        chat = ""
        if args.system:
            chat += f"<start_of_turn>user\n{args.system}\n\n{text}<end_of_turn>\n"
        else:
            chat += f"<start_of_turn>user\n{text}<end_of_turn>\n"
        chat += "<start_of_turn>model\n"
        ids = tok.encode(chat)
        if spec.bos_token_id is not None and spec.bos_token_id > 0:
            ids = [spec.bos_token_id] + ids
        prompts.append(ids)
    if not prompts and not args.model_info:
        return _fail("no prompt: give text, --tokens, or pipe text in (there is no REPL here)")

    from .engine.api import Engine
    n = max(1, len(prompts))
    max_batch = args.max_batch or n
    t0 = time.time()
    sizes = dict(dtype=args.dtype, max_tokens=max_batch * ((ctx + 63) // 64 * 64), ctx_size=ctx,
                 max_batch=max_batch)
    try:
        if args.random_weights is not None:
            engine = Engine.from_config(raw_config, seed=args.random_weights, **sizes)
        else:
            engine = Engine(args.model, strict=args.strict, **sizes)
    except (WeightsError, SafetensorsError, ConfigError, RuntimeError) as e:
        return _fail(str(e))
    info = engine.model_info()
    c = info["config"]
    if args.model_info:
        meta = {"version": __version__, "name": os.path.basename(os.path.normpath(args.model)),
                "arch": entry.name, "quant": info["dtype"], "backend": "cuda-sm100a",
                "format": "safetensors", "layers": c.get("num_hidden_layers"),
                "embed": c.get("hidden_size"), "heads": c.get("num_attention_heads"),
                "kv_heads": c.get("num_key_value_heads"), "head_dim": c.get("head_dim"),
                "ff_dim": c.get("intermediate_size"), "vocab_size": c.get("vocab_size"),
                "ctx_size": engine.max_seq_len, "rope_theta": c.get("rope_theta"),
                "weight_bytes": info["weight_bytes"], "cache_bytes": info["cache_bytes"]}
        if args.json:
            print(json.dumps(meta))
        else:
            for k, v in meta.items():
                print(f"{k:>14}: {v}")
        return 0
    if not quiet:
        print(f"agave_b200 {__version__} · {entry.name} · {info['dtype']} · ctx {engine.max_seq_len}"
              f" · loaded in {engine.load_seconds:.1f}s", file=sys.stderr)
    if args.verbose:
        print(f"weights {info['weight_bytes'] / 1e6:.1f} MB · cache {info['cache_bytes'] / 1e6:.1f} MB"
              f" · EOG {list(spec.eos_token_ids)}", file=sys.stderr)
        if engine.ignored_tensors:
            print(f"ignored {len(engine.ignored_tensors)} tensors outside the text decoder: "
                  + ", ".join(engine.ignored_tensors[:8])
                  + (" ..." if len(engine.ignored_tensors) > 8 else ""), file=sys.stderr)
    stops = list(spec.eos_token_ids)
    if tok is not None:
        for name in ("<end_of_turn>", "<eos>"):          # src/main.zig:1213-1222
            if name in tok.vocab and tok.vocab[name] not in stops:
                stops.append(tok.vocab[name])
    counters = None
    try:
        if args.profile:
            from .perf import PerfCounters
            counters = PerfCounters()
            counters.__enter__()
        outs = engine.generate(prompts, max_new_tokens=args.max_tokens,
                               temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                               repeat_penalty=args.repeat_penalty, seed=args.seed,
                               stop_token_ids=stops)
    except (ValueError, RuntimeError) as e:
        return _fail(str(e))
    finally:
        if counters is not None:
            counters.__exit__(None, None, None)
    st = engine.stats
    n_tok = sum(len(o) for o in outs)
    gen_ms = st["decode_seconds"] * 1e3
    pre_ms = st["prefill_seconds"] * 1e3
    tps = st["decode_tokens"] / st["decode_seconds"] if st["decode_seconds"] > 0 else 0.0
    if args.debug:
        for i, o in enumerate(outs):
            print(f"[debug] request {i}: prompt {prompts[i]} -> {o} "
                  f"({engine.finish_reasons[i]})", file=sys.stderr)
    texts = [tok.decode(o) if (tok is not None and args.tokens is None) else
             ",".join(str(t) for t in o) for o in outs]
    if args.json:
        rec = {"model": os.path.basename(os.path.normpath(args.model)), "arch": entry.name,
               "quant": info["dtype"], "backend": "cuda-sm100a", "version": __version__,
               "output": texts[0] if len(texts) == 1 else texts,
               "output_ids": outs[0] if len(outs) == 1 else outs,
               "tokens": n_tok, "tok_per_sec": tps, "prefill_tokens": st["prefill_tokens"],
               "prefill_ms": pre_ms,
               "prefill_tok_per_sec": st["prefill_tokens"] / st["prefill_seconds"]
               if st["prefill_seconds"] > 0 else 0.0,
               "gen_ms": gen_ms}
        print(json.dumps(rec))
    else:
        for t in texts:
            print(t)
        if not quiet:
            print(f"{n_tok} tok · {tps:.1f} tok/s · {pre_ms:.0f}ms prefill", file=sys.stderr)
    if args.profile:
        print(f"[profile] load {engine.load_seconds * 1e3:.0f} ms · prefill {pre_ms:.1f} ms "
              f"({st['prefill_tokens']} tok) · decode {gen_ms:.1f} ms ({st['decode_steps']} steps, "
              f"{st['batches']} batches)", file=sys.stderr)
        pk = _peaks()
        print(counters.report(pk.get("hbm_gbs", 0.0), pk.get("bf16_tflops", 0.0)),
              file=sys.stderr)
    return 0
