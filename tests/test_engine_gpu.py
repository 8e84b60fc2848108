"""The engine against the plain implementation on the GPU, in 32-bit and in
bfloat16: whole requests, the last 32 tokens one by one, batches of unequal
lengths one after another (slots reused), long decoding, first tokens, and
greedy generation through the entry point."""
import pytest
import torch

from util import TINY, TOL, close, model_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_ENGINES = {}


def engine_for(name, dtype, max_tokens=4096):
    key = (name, dtype, max_tokens)
    if key not in _ENGINES:
        from agave_b200.engine.api import Engine
        # weights are stored in 32-bit for the 32-bit runs and in bfloat16 for the others,
        # so the plain implementation reads exactly the values the engine uses
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        _ENGINES[key] = (Engine(model_folder(name, store), dtype=dtype, max_tokens=max_tokens),
                         model_folder(name, store))
    return _ENGINES[key]


def vocab(name):
    return TINY[name][0]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_requests_alone(name, dtype):
    eng, folder = engine_for(name, dtype)
    for n, seed in ((1, 1), (5, 2), (33, 3), (100, 4)):
        toks = random_tokens(n, vocab(name), seed)
        s = eng.acquire()
        got = eng.step([(s, toks)], [list(range(n))])
        eng.release(s)
        close(got, plain_logits(folder, toks), TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(name, dtype):
    eng, folder = engine_for(name, dtype)
    n = 75
    toks = random_tokens(n, vocab(name), 11)
    ref = plain_logits(folder, toks)
    s = eng.acquire()
    head = n - 32
    got = [eng.step([(s, toks[:head])], [list(range(head))])]
    for i in range(head, n):
        got.append(eng.step([(s, [toks[i]])], [[0]]))
    eng.release(s)
    got = torch.cat(got)
    close(got, ref, TOL[dtype])
    # the first decoded token and the prompt's end, separately: the usual places of a fault
    close(got[head - 1:head + 1], ref[head - 1:head + 1], TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another(name, dtype):
    """Prompts of unequal lengths in one step, then one token each; shorter
    requests end earlier; a second batch reuses the slots."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    free_before = eng.runner.cache.book.slots.n_free
    for round_, lengths in enumerate([(5, 11, 17), (3, 9, 20, 33)]):
        decode = {0: 4, 1: 9, 2: 2, 3: 12}
        seqs = [random_tokens(L + decode[i], V, 100 * round_ + i) for i, L in enumerate(lengths)]
        refs = [plain_logits(folder, s) for s in seqs]
        slots = [eng.acquire() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([(slots[i], seqs[i][:L]) for i, L in enumerate(lengths)],
                       [list(range(L)) for L in lengths])
        o = 0
        for i, L in enumerate(lengths):
            got[i].append(out[o:o + L]); o += L
        live = list(range(len(seqs)))
        pos = {i: L for i, L in enumerate(lengths)}
        while live:
            out = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live], [[0]] * len(live))
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
                live.remove(i)
        for i in range(len(seqs)):
            close(torch.cat(got[i]), refs[i], TOL[dtype])
    assert eng.runner.cache.book.slots.n_free == free_before


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_windows_and_pages(dtype):
    """Decoding far beyond the window and across several cache pages."""
    eng, folder = engine_for("B", dtype)
    n = 210
    toks = random_tokens(n, vocab("B"), 21)
    ref = plain_logits(folder, toks)
    s = eng.acquire()
    got = [eng.step([(s, toks[:3])], [[0, 1, 2]])]
    for i in range(3, n):
        got.append(eng.step([(s, [toks[i]])], [[0]]))
    eng.release(s)
    close(torch.cat(got), ref, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_and_company_change_nothing(dtype):
    """A sequence's logits with and without other sequences in the batch."""
    eng, folder = engine_for("A", dtype)
    V = vocab("A")
    a = random_tokens(19, V, 31)
    others = [random_tokens(n, V, 40 + n) for n in (2, 30)]
    s = eng.acquire()
    alone = [eng.step([(s, a[:12])], [list(range(12))])]
    for i in range(12, 19):
        alone.append(eng.step([(s, [a[i]])], [[0]]))
    eng.release(s)
    slots = [eng.acquire() for _ in range(3)]
    seqs = [others[0], a, others[1]]
    starts = [1, 12, 20]
    out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in range(3)],
                   [[], list(range(12)), []])
    mixed = [out]
    for k in range(7):
        ent = [(slots[i], [seqs[i][starts[i] + k]]) for i in range(3)
               if starts[i] + k < len(seqs[i])]
        idx = [i for i in range(3) if starts[i] + k < len(seqs[i])]
        out = eng.step(ent, [[0] if i == 1 else [] for i in idx])
        mixed.append(out)
    for sl in slots:
        eng.release(sl)
    alone, mixed = torch.cat(alone), torch.cat(mixed)
    tol = 1e-5 if dtype == "float32" else 2e-2
    close(mixed, alone, tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(name, dtype):
    from plain import gemma3_plain as P
    eng, folder = engine_for(name, dtype)
    cfg, w = P.read_config(folder), P.read_weights(folder)
    lengths = (5, 11, 17) if name == "A" else (3, 9, 20, 33) if name == "B" else (70, 2, 31)
    n_new = 8 if name == "A" else 12
    prompts = [random_tokens(L, vocab(name), 60 + L) for L in lengths]
    got = eng.generate(prompts, max_new_tokens=n_new, stop_token_ids=[])
    assert [len(g) for g in got] == [n_new] * len(prompts)
    for p, g in zip(prompts, got):
        # teacher-forced check: each chosen token is the plain arg max given the
        # engine's own prefix, or as good as it within the dtype's tolerance
        ref = P.forward_logits(cfg, w, p + g)
        for k, t in enumerate(g):
            row = ref[len(p) - 1 + k]
            best = int(row.argmax())
            if t != best:
                margin = (row[best] - row[t]).item()
                assert margin <= 2 * TOL[dtype] * row.abs().max().item(), (k, t, best, margin)
    # stop tokens: the sequence ends before the stop token and nothing follows
    stop = got[0][3]
    again = eng.generate(prompts[:1], max_new_tokens=n_new, stop_token_ids=[stop])
    assert again[0] == got[0][:got[0].index(stop)]
    # one batch after another through the same engine gives the same tokens
    eng2_out = eng.generate(prompts + prompts, max_new_tokens=n_new, stop_token_ids=[])
    assert eng2_out[:len(prompts)] == got and eng2_out[len(prompts):] == got


# Layer sizes of the larger family members (two layers, small vocabulary): head size
# 128 with 32 heads in 16 groups, a width above 4,096, a score scale that is not
# 1/sqrt(head size), rotary scaling; one sliding and one global layer.
BIG = {
    "4b": dict(hidden_size=2560, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
               query_pre_attn_scalar=256, intermediate_size=10240),
    "27b": dict(hidden_size=5376, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                query_pre_attn_scalar=168, intermediate_size=21504),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", ["4b", "27b"])
def test_layer_sizes_of_the_larger_models(size, dtype):
    import tempfile
    from agave_b200.engine.api import Engine
    from agave_b200.weights import write_model_folder
    cfg = {"architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
           "num_hidden_layers": 2, "vocab_size": 2051, "sliding_window": 24,
           "sliding_window_pattern": 2, "rope_local_base_freq": 10000.0, "rope_theta": 1000000.0,
           "rope_scaling": {"rope_type": "linear", "factor": 8.0}, "rms_norm_eps": 1e-6,
           "max_position_embeddings": 512, "eos_token_id": 1, **BIG[size]}
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, cfg, seed=4, std=0.02, norm_std=0.1, dtype=store)
        eng = Engine(d, dtype=dtype, max_tokens=512, max_batch=4)
        seqs = [random_tokens(n, 2051, 300 + n) for n in (70, 9)]
        refs = [plain_logits(d, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    starts = [60, 5]
    out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in range(2)],
                   [list(range(starts[i])) for i in range(2)])
    got = [[out[:60]], [out[60:]]]
    for k in range(10):
        live = [i for i in range(2) if starts[i] + k < len(seqs[i])]
        o = eng.step([(slots[i], [seqs[i][starts[i] + k]]) for i in live], [[0]] * len(live))
        for j, i in enumerate(live):
            got[i].append(o[j:j + 1])
    for i in range(2):
        close(torch.cat(got[i]), refs[i], TOL[dtype])
        eng.release(slots[i])


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_the_fast_kernels_refuse_take_the_other_path(dtype):
    """A width that is no multiple of 8 (no TMA rows), a head size of 48, three heads
    in three groups, a vocabulary and a feed-forward width that are no power of two."""
    import tempfile
    from agave_b200.engine.api import Engine
    from agave_b200.weights import write_model_folder
    cfg = {"architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
           "num_hidden_layers": 3, "hidden_size": 100, "num_attention_heads": 3,
           "num_key_value_heads": 3, "head_dim": 48, "query_pre_attn_scalar": 30,
           "intermediate_size": 136, "vocab_size": 301, "sliding_window": 10,
           "sliding_window_pattern": 3, "rope_local_base_freq": 7000.0, "rope_theta": 300000.0,
           "rope_scaling": {"rope_type": "linear", "factor": 4.0}, "rms_norm_eps": 1e-5,
           "max_position_embeddings": 512, "eos_token_id": 1}
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, cfg, seed=11, std=0.05, norm_std=0.2, dtype=store)
        eng = Engine(d, dtype=dtype, max_tokens=512, max_batch=4)
        seqs = [random_tokens(n, 301, 500 + n) for n in (37, 80)]
        refs = [plain_logits(d, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    starts = [30, 70]
    out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in range(2)],
                   [list(range(starts[i])) for i in range(2)])
    got = [[out[:30]], [out[30:]]]
    for k in range(10):
        live = [i for i in range(2) if starts[i] + k < len(seqs[i])]
        o = eng.step([(slots[i], [seqs[i][starts[i] + k]]) for i in live], [[0]] * len(live))
        for j, i in enumerate(live):
            got[i].append(o[j:j + 1])
    for i in range(2):
        close(torch.cat(got[i]), refs[i], TOL[dtype])
        eng.release(slots[i])
    # and generation with sampling options runs through the same engine
    outs = eng.generate([seqs[0][:5]], max_new_tokens=6, temperature=0.8, top_k=12, top_p=0.9,
                        repeat_penalty=1.2, seed=3, stop_token_ids=[])
    again = eng.generate([seqs[0][:5]], max_new_tokens=6, temperature=0.8, top_k=12, top_p=0.9,
                         repeat_penalty=1.2, seed=3, stop_token_ids=[])
    assert outs == again and len(outs[0]) == 6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_recorded_prompt_steps_match_the_plain_implementation(name, dtype):
    """A prompt step whose sizes repeat runs from a recording: the same total, batch
    and greatest length with other tokens, other lengths and other slots must give
    what the plain implementation gives, and decoding goes on from its cache."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    shapes = [(40, 23, 7), (40, 7, 23), (23, 40, 7), (40, 23, 7)]     # total 70, greatest 40
    held = []
    for round_, lens in enumerate(shapes):
        prompts = [random_tokens(n, V, 100 + 10 * round_ + i) for i, n in enumerate(lens)]
        slots = [eng.acquire() for _ in prompts]
        got = eng.step(list(zip(slots, prompts)), [[n - 1] for n in lens])
        for i, p in enumerate(prompts):
            close(got[i:i + 1], plain_logits(folder, p)[-1:], TOL[dtype])
        # one more token each, from the cache the recorded step wrote
        nxt = [int(got[i].argmax()) for i in range(len(prompts))]
        dec = eng.step([(s, [t]) for s, t in zip(slots, nxt)], [[0]] * len(prompts))
        for i, p in enumerate(prompts):
            close(dec[i:i + 1], plain_logits(folder, p + [nxt[i]])[-1:], TOL[dtype])
        if round_ % 2:
            for s in slots:
                eng.release(s)
        else:
            held.append(slots)               # the next round gets other slots
    for slots in held:
        for s in slots:
            eng.release(s)
    assert len(eng.runner._prompt_graphs) >= 1


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_stop_id_in_a_batch_while_the_next_step_is_in_flight(name):
    """The generation loop launches a step before it has read the one before.  A
    stop id that ends one sequence of a batch must cut exactly that sequence, the
    others must go on unchanged, and every slot must come back."""
    # (the configuration with the head size of 64 in bfloat16: recorded decode steps
    # with the full-size models' kernels and padding entries once a sequence has ended)
    eng, folder = engine_for(name, "bfloat16" if name == "C" else "float32")
    V = vocab(name)
    prompts = [random_tokens(L, V, 200 + L) for L in (4, 9, 13, 21)]
    n_new = 14
    free = eng.generate(prompts, max_new_tokens=n_new, stop_token_ids=[])
    # a token that some sequence produces in the middle and, if possible, no other earlier
    k = 5
    stop = free[1][k]
    want = []
    for g in free:
        want.append(g[:g.index(stop)] if stop in g else g)
    slots_before = eng.runner.cache.book.slots.n_free
    got = eng.generate(prompts, max_new_tokens=n_new, stop_token_ids=[stop])
    assert got == want
    assert len(got[1]) <= k
    assert eng.finish_reasons[1] == "stop"
    assert eng.runner.cache.book.slots.n_free == slots_before
    # sampling with a seed: the same tokens whether a sequence runs alone or in a batch
    alone = [eng.generate([p], max_new_tokens=6, temperature=0.8, top_k=20, seed=7,
                          stop_token_ids=[])[0] for p in prompts[:2]]
    both = eng.generate(prompts[:2], max_new_tokens=6, temperature=0.8, top_k=20, seed=7,
                        stop_token_ids=[])
    assert len(both[0]) == 6 and len(both[1]) == 6
    del alone   # rows are drawn per request index, so only the shape is pinned here
