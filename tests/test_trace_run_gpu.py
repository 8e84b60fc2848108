"""bin/trace_run and the command line, as a user runs them: separate processes,
model folders in a temporary place."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from util import ROOT, TINY, TOL, close, model_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def replay(folder, dtype, steps, max_tokens=1024):
    out = tempfile.mkdtemp(prefix="agave_trace_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens)],
                       input=text, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    import atexit, shutil
    atexit.register(shutil.rmtree, out, ignore_errors=True)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_whole_then_one_by_one_and_unequal_batches(dtype):
    name = "B"
    V = TINY[name][0]["vocab_size"]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = model_folder(name, store)
    a, b, c = (random_tokens(n, V, 200 + n) for n in (40, 9, 21))
    refs = {k: plain_logits(folder, s) for k, s in (("a", a), ("b", b), ("c", c))}
    steps = []
    # batch 1: a, b, c start together; b ends first, then c
    steps.append({"step": 0, "entries": [
        {"id": "a", "tokens": a[:30], "want": list(range(30))},
        {"id": "b", "tokens": b[:5], "want": [4]},
        {"id": "c", "tokens": c[:20], "want": []}], "end": []})
    n = 1
    for k in range(10):
        ent, end = [], []
        for rid, s, start in (("a", a, 30), ("b", b, 5), ("c", c, 20)):
            if start + k < len(s):
                ent.append({"id": rid, "tokens": [s[start + k]], "want": [0]})
                if start + k == len(s) - 1:
                    end.append(rid)
        steps.append({"step": n, "entries": ent, "end": end})
        n += 1
    # batch 2 reuses the slots: c whole, alone
    steps.append({"step": n, "entries": [{"id": "c2", "tokens": c, "want": list(range(len(c)))}],
                  "end": ["c2"]})
    out = replay(folder, dtype, steps)
    tol = TOL[dtype]

    def rows(step):
        return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4")
                                .reshape(-1, V).copy())
    first = rows(0)
    assert first.shape[0] == 31
    close(first[:30], refs["a"][:30], tol)
    close(first[30:], refs["b"][4:5], tol)
    for k in range(10):
        got = rows(1 + k)
        i = 0
        for rid, s, start in (("a", a, 30), ("b", b, 5), ("c", c, 20)):
            if start + k < len(s):
                close(got[i:i + 1], refs[rid][start + k:start + k + 1], tol)
                i += 1
        assert i == got.shape[0]
    close(rows(n), refs["c"], tol)


def test_command_line_generates_token_ids():
    folder = model_folder("A", torch.bfloat16)
    cmd = [sys.executable, "-m", "agave_b200", folder, "--tokens", "2,17,99,5;2,8", "-n", "6",
           "--json", "--dtype", "float32"]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["arch"] == "Gemma3ForCausalLM" and rec["tokens"] <= 12
    ids = rec["output_ids"]
    assert len(ids) == 2 and all(len(o) <= 6 for o in ids)
    from plain import gemma3_plain as P
    cfg, w = P.read_config(folder), P.read_weights(folder)
    stops = [cfg["eos_token_id"]]
    assert ids[0] == P.greedy_generate(cfg, w, [2, 17, 99, 5], 6, stop=stops)
    # sampling with a seed is repeatable; model info prints and exits
    cmd2 = [sys.executable, "-m", "agave_b200", folder, "--tokens", "2,17,99,5", "-n", "5", "-t",
            "0.9", "--top-k", "20", "--top-p", "0.95", "--repeat-penalty", "1.1", "--seed", "7",
            "--json"]
    r1 = subprocess.run(cmd2, capture_output=True, text=True, cwd=ROOT, timeout=600)
    r2 = subprocess.run(cmd2, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r1.returncode == 0 and r2.returncode == 0, r1.stderr[-2000:]
    assert json.loads(r1.stdout.splitlines()[-1])["output_ids"] == \
        json.loads(r2.stdout.splitlines()[-1])["output_ids"]
    r3 = subprocess.run([sys.executable, "-m", "agave_b200", folder, "--model-info", "--json"],
                        capture_output=True, text=True, cwd=ROOT, timeout=600)
    info = json.loads(r3.stdout.splitlines()[-1])
    assert info["layers"] == 4 and info["head_dim"] == 16 and info["vocab_size"] == 256
