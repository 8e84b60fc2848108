"""Schedules and sizes beyond the tiny configurations' defaults, on the GPU, against
the plain implementation: generation cut into several batches by the slot limit and by
the token budget, the end of the cache with a step in flight, the step function's
refusals, sampling that does not depend on a sequence's company, windows as large as
their ring (64 and 128 positions) with decoding past the wrap, the layer sizes of the
1B model with its vocabulary of 262,144 and its window of 512, a folder that holds more
than the text decoder, the cancel flag, and a bounded wait that runs out."""
import json
import os
import tempfile
import threading

import pytest
import torch

from util import TINY, TINY_B, TOL, close, model_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def _engine(name, dtype, **kw):
    from agave_b200.engine.api import Engine
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = model_folder(name, store)
    return Engine(folder, dtype=dtype, **kw), folder


def _all_back(eng):
    book = eng.runner.cache.book
    assert book.slots.n_free == book.slots.n_slots
    for pool in book.pools:
        assert pool.n_free == pool.n_pages
    assert not book.length and not book.pages


def _check_greedy(folder, prompts, outs, dtype):
    """Teacher-forced: each chosen token is the plain arg max given the engine's own
    prefix, or as good as it within the dtype's tolerance."""
    from plain import gemma3_plain as P
    cfg, w = P.read_config(folder), P.read_weights(folder)
    for p, g in zip(prompts, outs):
        if not g:
            continue
        ref = P.forward_logits(cfg, w, list(p) + list(g))
        for k, t in enumerate(g):
            row = ref[len(p) - 1 + k]
            best = int(row.argmax())
            if t != best:
                margin = (row[best] - row[t]).item()
                assert margin <= 2 * TOL[dtype] * row.abs().max().item(), (k, t, best, margin)


# ------------------------------------------------------------ several batches
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_cut_into_batches_by_the_slot_limit(dtype):
    """Five prompts through an engine with two slots: three batches, slots reused."""
    eng, folder = _engine("B", dtype, max_tokens=4096, max_batch=2)
    V = TINY["B"][0]["vocab_size"]
    prompts = [random_tokens(L, V, 700 + L) for L in (3, 33, 9, 20, 14)]
    outs = eng.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    assert eng.stats["batches"] == 3 and [len(o) for o in outs] == [10] * 5
    _check_greedy(folder, prompts, outs, dtype)
    _all_back(eng)
    if dtype == "float32":
        # the 32-bit products add in one order whatever the batch: the same tokens
        # as when every request runs alone
        alone = [eng.generate([p], max_new_tokens=10, stop_token_ids=[])[0] for p in prompts]
        assert alone == outs
    # a stop token in the second batch ends that request only
    stop = outs[3][4]
    again = eng.generate(prompts, max_new_tokens=10, stop_token_ids=[stop])
    for o, a in zip(outs, again):
        assert a == (o[:o.index(stop)] if stop in o else o)
    _all_back(eng)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_cut_by_the_token_budget_and_clamped_by_the_context(dtype):
    V = TINY["A"][0]["vocab_size"]
    # a budget of two pages: two of the three requests (a page each) fit a batch
    eng, folder = _engine("A", dtype, max_tokens=128, max_batch=4)
    prompts = [random_tokens(L, V, 800 + L) for L in (30, 40, 50)]
    outs = eng.generate(prompts, max_new_tokens=12, stop_token_ids=[])
    assert eng.stats["batches"] == 2 and [len(o) for o in outs] == [12] * 3
    assert eng.finish_reasons == ["length"] * 3
    _check_greedy(folder, prompts, outs, dtype)
    _all_back(eng)
    # one page in all: a prompt of 50 may grow to 64 positions; the token sampled from
    # the last of them is still returned, and the reason says why it ended
    eng1, folder = _engine("A", dtype, max_tokens=64, max_batch=2)
    assert eng1.max_seq_len == 64
    p = random_tokens(50, V, 900)
    out = eng1.generate([p, p[:7]], max_new_tokens=40, stop_token_ids=[])
    assert len(out[0]) == 15 and eng1.finish_reasons[0] == "context"
    assert len(out[1]) == 40 and eng1.finish_reasons[1] == "length"
    assert eng1.stats["batches"] == 2
    _check_greedy(folder, [p, p[:7]], out, dtype)
    _all_back(eng1)
    with pytest.raises(ValueError):
        eng1.generate([random_tokens(65, V, 1)], max_new_tokens=2)
    _all_back(eng1)


# ------------------------------------------------------------------- refusals
def test_the_step_function_refuses_what_it_cannot_run():
    from agave_b200.cache import CacheError, CacheFull
    from agave_b200.engine.step import StepError
    eng, folder = _engine("A", "float32", max_tokens=192, max_batch=4)
    V = TINY["A"][0]["vocab_size"]
    book = eng.runner.cache.book
    a, b = eng.acquire(), eng.acquire()
    with pytest.raises(StepError, match="at least one"):
        eng.step([], [])
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([(a, [1, V])], [[0]])
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([(a, [-1])], [[0]])
    with pytest.raises(StepError, match="twice"):
        eng.step([(a, [1, 2]), (a, [3])], [[0], [0]])
    with pytest.raises(StepError, match="not held"):
        eng.step([(3, [1, 2])], [[0]])
    with pytest.raises(StepError, match="no tokens"):
        eng.step([(a, [])], [[]])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([(a, [1, 2])], [[2]])
    with pytest.raises(StepError, match="one list per sequence"):
        eng.step([(a, [1, 2])], [[0], [0]])
    assert book.length[a] == 0 and not any(book.pages[a])        # nothing was reserved
    eng.step([(a, [5, 6, 7])], [[]])
    with pytest.raises(StepError, match="either all start"):        # a started and a fresh one
        eng.step([(a, [8]), (b, [9, 10])], [[0], [0]])
    with pytest.raises(StepError, match="either all start"):        # two tokens onto a started one
        eng.step([(a, [8, 9])], [[0]])
    # the budget is three pages: a second sequence of 130 positions does not fit beside the
    # first one's page, and the page reserved for the step's first entry goes back
    free = [p.n_free for p in book.pools]
    c = eng.acquire()
    with pytest.raises(CacheFull):
        eng.step([(c, random_tokens(60, V, 1)), (b, random_tokens(130, V, 2))], [[], []])
    assert [p.n_free for p in book.pools] == free and not any(book.pages[c])
    assert book.length[c] == 0 and book.length[b] == 0
    with pytest.raises(CacheFull):                                   # longer than the cache allows
        eng.step([(c, random_tokens(193, V, 3))], [[]])
    # what was refused changed nothing: the started sequence goes on and is right
    toks = [5, 6, 7, 8]
    got = eng.step([(a, [8])], [[0]])
    close(got, plain_logits(folder, toks)[-1:], TOL["float32"])
    for s in (a, b, c):
        eng.release(s)
    with pytest.raises(CacheError):
        eng.release(a)
    _all_back(eng)


# ------------------------------------------------------------------- sampling
def test_a_sampled_sequence_does_not_depend_on_its_company():
    """The draw of a request is keyed by (seed, request index, tokens generated so far);
    in 32-bit the logits do not depend on the batch either, so the tokens are equal."""
    eng, _ = _engine("B", "float32", max_tokens=4096)
    V = TINY["B"][0]["vocab_size"]
    p0, p1, p2 = (random_tokens(L, V, 40 + L) for L in (9, 21, 4))
    kw = dict(max_new_tokens=12, temperature=0.9, top_k=40, top_p=0.95, seed=7, stop_token_ids=[])
    a = eng.generate([p0, p1], **kw)
    b = eng.generate([p0, p2], **kw)
    c = eng.generate([p0], **kw)
    assert a[0] == b[0] == c[0] and len(a[0]) == 12
    assert a[1] != b[1]
    # another seed draws other tokens; no seed means another seed each call, and neither
    # records a decode step anew: the options are step inputs, not part of a recording
    n_graphs = len(eng._graphs)
    d = eng.generate([p0], **dict(kw, seed=8))
    assert d[0] != a[0]
    eng.generate([p0], **dict(kw, seed=None))
    eng.generate([p0], **dict(kw, temperature=0.5, top_k=0, top_p=1.0))
    assert len(eng._graphs) == n_graphs
    _all_back(eng)


# ------------------------------------------------- windows as large as their ring
WINDOWED = {
    # window 128 = two pages, head size 64 (bfloat16 then decodes with the fused kernel)
    "W128": {"architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
             "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 4,
             "num_key_value_heads": 2, "head_dim": 64, "query_pre_attn_scalar": 64,
             "intermediate_size": 256, "vocab_size": 320, "sliding_window": 128,
             "sliding_window_pattern": 3, "rope_local_base_freq": 10000.0,
             "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
             "eos_token_id": 1},
    # window 64 = one page exactly, one kv head, every second layer global
    "W64": {"architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
            "num_hidden_layers": 4, "hidden_size": 192, "num_attention_heads": 3,
            "num_key_value_heads": 1, "head_dim": 64, "query_pre_attn_scalar": 32,
            "intermediate_size": 384, "vocab_size": 270, "sliding_window": 64,
            "sliding_window_pattern": 2, "rope_local_base_freq": 9000.0,
            "rope_theta": 400000.0, "rope_scaling": {"rope_type": "linear", "factor": 2.0},
            "rms_norm_eps": 1e-5, "max_position_embeddings": 1024, "eos_token_id": 1},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["W128", "W64"])
def test_windows_as_large_as_their_ring(name, dtype):
    """A prompt longer than the ring, then decoding well past several wraps; and a prompt
    of exactly the window, so that the first decoded token is the first to overwrite."""
    from agave_b200.engine.api import Engine
    from agave_b200.weights import write_model_folder
    cfg = WINDOWED[name]
    W, V = cfg["sliding_window"], cfg["vocab_size"]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, cfg, seed=21, std=0.05, norm_std=0.2, dtype=store)
        eng = Engine(d, dtype=dtype, max_tokens=2048, max_batch=4)
        for g in eng.runner.cache.book.groups:
            if g.window is not None:
                assert g.cap == W and g.window == W          # the ring holds the window exactly
        seqs = [random_tokens(n, V, 60 + n) for n in (2 * W + 60, W + 45, 3 * W + 10)]
        starts = [W + 72, W, 1]
        refs = [plain_logits(d, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in range(3)],
                   [list(range(starts[i])) for i in range(3)])
    got, o = [], 0
    for i in range(3):
        got.append([out[o:o + starts[i]]]); o += starts[i]
    pos = list(starts)
    live = [0, 1, 2]
    while live:
        res = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live], [[0]] * len(live))
        for j, i in enumerate(live):
            got[i].append(res[j:j + 1]); pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            eng.release(slots[i]); live.remove(i)
    for i in range(3):
        g = torch.cat(got[i])
        close(g, refs[i], TOL[dtype])
        # around the first wrap and the window's edge, on their own
        for at in (W - 1, W, W + 1, 2 * W):
            if at < len(seqs[i]):
                close(g[at:at + 1], refs[i][at:at + 1], TOL[dtype])
    _all_back(eng)


def test_prompt_steps_with_the_qkv_epilogue(monkeypatch):
    """The q/k/v product that norms, rotates and stores in its epilogue is chosen only when
    a CTA gets several tiles (the larger models); here it is forced on a small model so
    that a whole prompt step and the decoding that follows from its cache run through it:
    two prompts, one longer than its ring."""
    from agave_b200.engine.api import Engine
    from agave_b200.weights import write_model_folder
    monkeypatch.setenv("AGAVE_B200_FUSED_QKV_PREFILL", "2")
    cfg = WINDOWED["W128"]
    V = cfg["vocab_size"]
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, cfg, seed=22, std=0.05, norm_std=0.2, dtype=torch.bfloat16)
        eng = Engine(d, dtype="bfloat16", max_tokens=2048, max_batch=4)
        seqs = [random_tokens(n, V, 90 + n) for n in (230, 150)]
        starts = [222, 141]
        refs = [plain_logits(d, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in range(2)],
                   [list(range(starts[i])) for i in range(2)])
    got = [[out[:starts[0]]], [out[starts[0]:]]]
    for k in range(9):
        live = [i for i in range(2) if starts[i] + k < len(seqs[i])]
        res = eng.step([(slots[i], [seqs[i][starts[i] + k]]) for i in live], [[0]] * len(live))
        for j, i in enumerate(live):
            got[i].append(res[j:j + 1])
    for i in range(2):
        close(torch.cat(got[i]), refs[i], TOL["bfloat16"])
        eng.release(slots[i])
    _all_back(eng)


# --------------------------------------------------------- the 1B layer sizes
CFG_1B_TWO_LAYERS = {
    "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
    "num_hidden_layers": 2, "hidden_size": 1152, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 256, "query_pre_attn_scalar": 256,
    "intermediate_size": 6912, "vocab_size": 262144, "sliding_window": 512,
    "sliding_window_pattern": 2, "rope_local_base_freq": 10000.0, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 32768,
    "eos_token_id": 1,
}


@pytest.fixture(scope="module")
def folder_1b():
    from agave_b200.weights import write_model_folder
    from plain import gemma3_plain as P
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, CFG_1B_TWO_LAYERS, seed=2, std=0.02, norm_std=0.1,
                           dtype=torch.bfloat16)
        yield d, P.read_config(d), P.read_weights(d, torch.float32)


def _plain_rows(cfg, w, tokens, rows):
    from plain import gemma3_plain as P
    return P.logits_at(cfg, w, P.forward_hidden(cfg, w, tokens), rows)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_the_1b_layer_sizes_through_the_step_function(folder_1b, dtype):
    """One sliding and one global layer at the benchmark model's sizes (width 1,152, four
    heads of 256 on one kv head, vocabulary 262,144, window 512): a prompt of 700 tokens and
    40 decoded ones (past the ring's wrap at 512), then a batch of unequal prompts."""
    from agave_b200.engine.api import Engine
    d, cfg, w = folder_1b
    V = cfg["vocab_size"]
    eng = Engine(d, dtype=dtype, max_tokens=4096, ctx_size=2048, max_batch=4)
    n, head = 740, 700
    toks = random_tokens(n, V, 77)
    rows = [0, 511, 512, 513, 698, 699] + list(range(head, n, 3))
    ref = _plain_rows(cfg, w, toks, rows)
    s = eng.acquire()
    got = {}
    out = eng.step([(s, toks[:head])], [[r for r in rows if r < head]])
    for j, r in enumerate([r for r in rows if r < head]):
        got[r] = out[j]
    for i in range(head, n):
        out = eng.step([(s, [toks[i]])], [[0]] if i in rows else [[]])
        if i in rows:
            got[i] = out[0]
    eng.release(s)
    close(torch.stack([got[r] for r in rows]), ref, TOL[dtype])
    # a batch of unequal prompts, shorter ones ending earlier
    lens, decode = (530, 70, 9), (6, 4, 8)
    seqs = [random_tokens(L + k, V, 300 + L) for L, k in zip(lens, decode)]
    slots = [eng.acquire() for _ in seqs]
    out = eng.step([(slots[i], seqs[i][:lens[i]]) for i in range(3)], [[L - 1] for L in lens])
    got = [[out[i:i + 1]] for i in range(3)]
    pos, live = list(lens), [0, 1, 2]
    while live:
        res = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live], [[0]] * len(live))
        for j, i in enumerate(live):
            got[i].append(res[j:j + 1]); pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            eng.release(slots[i]); live.remove(i)
    for i in range(3):
        ref = _plain_rows(cfg, w, seqs[i], list(range(lens[i] - 1, len(seqs[i]))))
        close(torch.cat(got[i]), ref, TOL[dtype])
    _all_back(eng)


def test_the_1b_layer_sizes_through_generate(folder_1b):
    """The recorded decode step sized for a context of 8,192, greedy choice at a
    vocabulary of 262,144, unequal prompts one of which is past its ring's wrap."""
    from agave_b200.engine.api import Engine
    from plain import gemma3_plain as P
    d, cfg, w = folder_1b
    V = cfg["vocab_size"]
    eng = Engine(d, dtype="bfloat16", max_tokens=4 * 8192, ctx_size=8192, max_batch=4)
    prompts = [random_tokens(L, V, 500 + L) for L in (600, 33, 140)]
    outs = eng.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    assert [len(o) for o in outs] == [10, 10, 10]
    for p, g in zip(prompts, outs):
        rows = list(range(len(p) - 1, len(p) + len(g) - 1))
        ref = _plain_rows(cfg, w, list(p) + list(g), rows)
        for k, t in enumerate(g):
            row = ref[k]
            best = int(row.argmax())
            if t != best:
                margin = (row[best] - row[t]).item()
                assert margin <= 2 * TOL["bfloat16"] * row.abs().max().item(), (k, t, best)
    _all_back(eng)


# ------------------------------------------- a folder with more than the decoder
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_multimodal_folder_runs_as_its_text_decoder(dtype):
    from agave_b200.engine.api import Engine
    from agave_b200.weights import SafetensorsFolder, WeightsError, save_safetensors
    from plain import gemma3_plain as P
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    src = model_folder("B", store)
    with tempfile.TemporaryDirectory() as d:
        text = {k: v for k, v in TINY_B.items()
                if k not in ("architectures", "num_attention_heads", "num_key_value_heads",
                             "head_dim", "vocab_size", "tie_word_embeddings")}
        with open(os.path.join(d, "config.json"), "w") as fh:
            json.dump({"architectures": ["Gemma3ForConditionalGeneration"],
                       "model_type": "gemma3", "text_config": text,
                       "vision_config": {"hidden_size": 8}}, fh)
        f = SafetensorsFolder(src)
        t = {"language_model." + n: f.tensor(n).clone() for n in f.names()}
        g = torch.Generator().manual_seed(3)
        t["language_model.lm_head.weight"] = (torch.randn(384, 96, generator=g) * 0.05).to(store)
        t["vision_tower.vision_model.encoder.layers.0.self_attn.q_proj.weight"] = torch.zeros(8, 8)
        t["multi_modal_projector.mm_input_projection_weight"] = torch.zeros(8, 96)
        save_safetensors(os.path.join(d, "model.safetensors"), t)
        eng = Engine(d, dtype=dtype, max_tokens=512)
        assert len(eng.ignored_tensors) == 2 and not eng.spec.tie_embeddings
        with pytest.raises(WeightsError):
            Engine(d, dtype=dtype, max_tokens=512, strict=True)
        toks = random_tokens(40, 384, 9)
        cfg, w = P.read_config(d), P.read_weights(d)
        assert "lm_head.weight" in w
        # the plain implementation needs the sizes the text_config leaves out
        cfg.update(num_attention_heads=6, num_key_value_heads=2, head_dim=32, vocab_size=384)
        ref = P.forward_logits(cfg, w, toks)
    s = eng.acquire()
    got = [eng.step([(s, toks[:30])], [list(range(30))])]
    for i in range(30, 40):
        got.append(eng.step([(s, [toks[i]])], [[0]]))
    eng.release(s)
    close(torch.cat(got), ref, TOL[dtype])


# ----------------------------------------------- the two host sides of a step
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_the_cpp_host_step_launches_what_the_python_parts_launch(name, dtype):
    """A model of standard blocks runs its steps through one call into the library, which
    makes the dispatch decisions itself; the Python parts make them launch by launch for
    every other model.  Both must launch the same kernels with the same arguments: the
    logits of a prompt step, of decode steps and of a batch are equal bit for bit."""
    eng, folder = _engine(name, dtype, max_tokens=4096)
    assert eng.model.native is not None
    V = TINY[name][0]["vocab_size"]
    seqs = [random_tokens(n, V, 400 + n) for n in (150, 7, 41)]

    def run():
        slots = [eng.acquire() for _ in seqs]
        outs = [eng.step([(slots[i], seqs[i][:-4]) for i in range(3)],
                         [list(range(len(seqs[i]) - 4)) for i in range(3)])]
        for k in range(4, 0, -1):
            outs.append(eng.step([(slots[i], [seqs[i][-k]]) for i in range(3)], [[0]] * 3))
        outs.append(eng.step([(slots[0], [7])], [[0]]))
        for s in slots:
            eng.release(s)
        return torch.cat(outs)

    native = run()
    close(native[:146], plain_logits(folder, seqs[0])[:146], TOL[dtype])
    keep, eng.model.native = eng.model.native, None
    try:
        python = run()
    finally:
        eng.model.native = keep
    assert torch.equal(native, python)
    # and through the generation loop (recorded decode steps, arg max in the head's epilogue)
    prompts = [s[:9] for s in seqs]
    a = eng.generate(prompts, max_new_tokens=8, stop_token_ids=[])
    keep, eng.model.native = eng.model.native, None
    eng._graphs.clear()
    try:
        b = eng.generate(prompts, max_new_tokens=8, stop_token_ids=[])
    finally:
        eng.model.native = keep
        eng._graphs.clear()
    assert a == b


# ------------------------------------------------------------------ cancelling
def test_cancel_from_another_thread():
    """``Engine.cancel`` stops an eager step between two blocks (nothing is committed, the
    reserved room goes back) and a generation between two steps (what was generated so far
    is returned, every slot comes back); the engine then works as before."""
    from agave_b200.engine.api import Engine
    from agave_b200.engine.batch import Cancelled
    folder = model_folder("B", torch.float32)
    eng = Engine(folder, dtype="float32", max_tokens=4096, use_graphs=False)
    V = TINY["B"][0]["vocab_size"]
    toks = random_tokens(50, V, 3)
    ref = plain_logits(folder, toks)
    # a step: the flag is up before it starts, so it stops before its first block
    s = eng.acquire()
    eng.cancel()
    with pytest.raises(Cancelled):
        eng.step([(s, toks[:40])], [[39]])
    book = eng.runner.cache.book
    assert book.length[s] == 0 and not any(book.pages[s])
    close(eng.step([(s, toks[:40])], [[39]]), ref[39:40], TOL["float32"])    # the flag was cleared
    eng.release(s)
    # a generation: a thread raises the flag once some tokens are out
    started = threading.Event()
    orig = eng._stage_step
    count = {"n": 0}

    def counting(*a, **k):
        count["n"] += 1
        if count["n"] == 6:
            started.set()
        return orig(*a, **k)

    eng._stage_step = counting
    t = threading.Thread(target=lambda: (started.wait(60), eng.cancel()))
    t.start()
    outs = eng.generate([toks[:9], toks[:20]], max_new_tokens=4000, stop_token_ids=[])
    t.join()
    eng._stage_step = orig
    assert eng.finish_reasons == ["cancelled", "cancelled"]
    assert 2 <= len(outs[0]) < 4000 and len(outs[0]) == len(outs[1])
    _all_back(eng)
    full = eng.generate([toks[:9]], max_new_tokens=len(outs[0]), stop_token_ids=[])
    assert full[0] == outs[0] and eng.finish_reasons == ["length"]


# ------------------------------------------------------- a wait that runs out
def test_a_bounded_wait_that_runs_out_returns_its_status():
    """The unit kernel whose barriers nobody arrives on: every wait gives up after its
    limit, the kernel records the loader's or the epilogue's code, frees its tensor memory
    and returns; the next product on the tensor cores is right and its status is clean."""
    from agave_b200 import kernels
    assert kernels.linear_tc_status() == 0
    for limit, ctas in ((500, 1), (3000, 8)):
        status, cycles = kernels.selftest_bounded_wait(limit, ctas)
        assert status in ((1 << 8) | 0, 3 << 8), status
        assert cycles > 0
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(24, 512, generator=g) * 0.5).to(torch.bfloat16).cuda()
    w = (torch.randn(384, 512, generator=g) * 0.1).to(torch.bfloat16).cuda()
    out = torch.empty(24, 384, dtype=torch.float32, device="cuda")
    kernels.linear_tc(x, w, out)
    assert kernels.linear_tc_status() == 0
    close(out, x.float() @ w.float().T, 1e-5)
