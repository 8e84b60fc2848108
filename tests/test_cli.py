"""The command line's own pieces: the small tokenizer (no GPU), and on the GPU the
text-prompt branch, ``--random-weights`` and the per-operation ``--profile`` table."""
import json
import os
import shutil
import subprocess
import sys
import tempfile

import pytest
import torch

from util import ROOT, TINY_A, model_folder

PIECES = ["<pad>", "<eos>", "<bos>", "<unk>", "<start_of_turn>", "<end_of_turn>", "\n", "▁",
          "user", "model", "▁the", "▁cat", "▁sat", "▁on", "▁mat", "the", "cat", "c", "a", "t",
          "s", "o", "n", "m", "h", "e", "▁a", "at", "<0xC3>", "<0xA9>", ".", "u", "r", "d", "l"]


def write_tokenizer(folder):
    vocab = {p: i for i, p in enumerate(PIECES)}
    added = [{"id": vocab[p], "content": p, "special": True}
             for p in ("<pad>", "<eos>", "<bos>", "<unk>", "<start_of_turn>", "<end_of_turn>")]
    with open(os.path.join(folder, "tokenizer.json"), "w", encoding="utf-8") as f:
        json.dump({"model": {"type": "BPE", "vocab": vocab}, "added_tokens": added}, f)
    return vocab


def test_simple_tokenizer_round_trip():
    from agave_b200.cli import SimpleTokenizer
    with tempfile.TemporaryDirectory() as d:
        vocab = write_tokenizer(d)
        tok = SimpleTokenizer(os.path.join(d, "tokenizer.json"))
    # longest match first, spaces as the SentencePiece mark, no dummy prefix
    ids = tok.encode("the cat sat on the mat.")
    assert [PIECES[i] for i in ids] == ["the", "▁cat", "▁sat", "▁on", "▁the", "▁mat", "."]
    assert tok.decode(ids) == "the cat sat on the mat."
    # special tokens are matched whole, wherever they stand
    ids = tok.encode("<start_of_turn>user\nthe cat<end_of_turn>\n<start_of_turn>model\n")
    assert ids[0] == vocab["<start_of_turn>"] and ids[1] == vocab["user"]
    assert ids.count(vocab["<start_of_turn>"]) == 2 and vocab["<end_of_turn>"] in ids
    assert tok.decode(ids) == "<start_of_turn>user\nthe cat<end_of_turn>\n<start_of_turn>model\n"
    # a character without a piece falls back to its bytes; one without those is dropped
    ids = tok.encode("caté")
    assert [PIECES[i] for i in ids] == ["cat", "<0xC3>", "<0xA9>"]
    assert tok.encode("z") == []
    # greedy longest match: "a" + "t" is never preferred over "at"
    assert [PIECES[i] for i in tok.encode("at")] == ["at"]


def test_options_of_the_reference_without_a_counterpart():
    """Accepted where they name what happens anyway, refused with the reason otherwise;
    none ends in a usage error."""
    from agave_b200.cli import build_parser, _unsupported
    p = build_parser()
    ok = p.parse_args(["m", "--backend", "cuda", "--no-color", "--color", "never", "--mmap",
                       "--prefill-batch-size", "512", "--kv-type", "f16", "--kv-eviction", "none"])
    assert _unsupported(ok) is None
    for argv, word in ((["--backend", "vulkan"], "CUDA"), (["--allow-cpu-fallback"], "CPU"),
                       (["--kv-type", "q8_0"], "quantised"), (["--kv-type-k", "f32"], "bfloat16"),
                       (["--kv-tiers", "vram+ram"], "tiered"), (["--grammar", "g.gbnf"], "constrained"),
                       (["--json-output"], "constrained"), (["--draft-model", "d"], "speculative"),
                       (["--image", "a.png"], "vision"), (["--serve"], "server"),
                       (["--megakernel"], "single-launch"), (["--kv-eviction", "norm"], "eviction")):
        msg = _unsupported(p.parse_args(["m"] + argv))
        assert msg is not None and word in msg, (argv, msg)
    assert _unsupported(p.parse_args(["m", "--dtype", "float32", "--kv-type", "f32"])) is None


def _run(cmd, env=None):
    return subprocess.run([sys.executable, "-m", "agave_b200"] + cmd, capture_output=True,
                          text=True, cwd=ROOT, timeout=900,
                          env=dict(os.environ, **env) if env else None)


@pytest.mark.gpu
def test_text_prompt_random_weights_and_profile():
    src = model_folder("A", torch.float32)
    with tempfile.TemporaryDirectory() as d:
        for n in os.listdir(src):
            shutil.copy(os.path.join(src, n), d)
        vocab = write_tokenizer(d)
        # a text prompt: BOS, then the chat template around it, ids from the tokenizer
        r = _run([d, "the cat sat", "-n", "5", "--json", "--dtype", "float32", "-d"])
        assert r.returncode == 0, r.stderr[-2000:]
        rec = json.loads(r.stdout.strip().splitlines()[-1])
        from agave_b200.cli import SimpleTokenizer
        tok = SimpleTokenizer(os.path.join(d, "tokenizer.json"))
        want = [TINY_A["bos_token_id"]] + tok.encode(
            "<start_of_turn>user\nthe cat sat<end_of_turn>\n<start_of_turn>model\n")
        assert f"prompt {want}" in r.stderr                 # what -d prints is what was run
        from plain import gemma3_plain as P
        cfg, w = P.read_config(d), P.read_weights(d)
        stops = [cfg["eos_token_id"], vocab["<end_of_turn>"]]
        ids = P.greedy_generate(cfg, w, want, 5, stop=stops)
        assert rec["output_ids"] == ids and rec["output"] == tok.decode(ids)
        # per-operation timing: a table with the operations of a layer and a total
        r = _run([d, "--tokens", "2,17,99,5", "-n", "4", "--profile", "--dtype", "bfloat16"])
        assert r.returncode == 0, r.stderr[-2000:]
        for op in ("embed", "norm", "qkv", "attention", "out_proj", "gate_up", "down", "lm_head",
                   "TOTAL"):
            assert op in r.stderr, (op, r.stderr[-1500:])
    # a folder with nothing but config.json, weights drawn from a seed: the same seed gives
    # the same tokens, another seed other weights
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(TINY_A, f)
        outs = []
        for seed in ("3", "3", "4"):
            r = _run([d, "--random-weights", seed, "--tokens", "2,9,30,77,5", "-n", "8", "--json"])
            assert r.returncode == 0, r.stderr[-2000:]
            outs.append(json.loads(r.stdout.strip().splitlines()[-1])["output_ids"])
        assert outs[0] == outs[1] and len(outs[0]) <= 8
        # one sequence decoded through the tensor-core products instead of the dot products
        # that steps of one and two tokens take by default: the same tokens
        r = _run([d, "--random-weights", "3", "--tokens", "2,9,30,77,5", "-n", "8", "--json"],
                 env={"AGAVE_B200_FEW_TOKENS": "0"})
        assert r.returncode == 0, r.stderr[-2000:]
        assert json.loads(r.stdout.strip().splitlines()[-1])["output_ids"] == outs[0]
        # every launch named by an NVTX range (steps then go through the Python parts):
        # the same tokens
        r = _run([d, "--random-weights", "3", "--tokens", "2,9,30,77,5", "-n", "8", "--json"],
                 env={"AGAVE_B200_NVTX": "1"})
        assert r.returncode == 0, r.stderr[-2000:]
        assert json.loads(r.stdout.strip().splitlines()[-1])["output_ids"] == outs[0]
        r = _run([d, "--tokens", "2,9", "-n", "2"])
        assert r.returncode != 0 and "safetensors" in r.stderr
