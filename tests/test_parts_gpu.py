"""Each part alone against the plain functions, and the generality of the
assembly: a toy mixer with state of its own, another arrangement, activation
and norm flavour, a block called twice and a layer that reads another layer's
cache, a feed-forward with routing and a position encoding of another formula,
a block of another shape (both branches from one norm) and a learned position
table added to the stream.  The toy parts live here and are registered from
here; no file of the library changes for them."""
import dataclasses
import json
import math
import os
import tempfile

import pytest
import torch

from plain import gemma3_plain as P
from util import TINY_B, TOL, close, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _ctx(engine, entries):
    """A step context for (slot, tokens) entries, as the step function builds it."""
    return engine.runner.context(entries)


# ------------------------------------------------------------ parts, one by one
def test_rms_norm_part_zero_centred_and_plain():
    from agave_b200.config import NormSpec
    from agave_b200.parts import RMSNorm
    H = 200
    h = torch.randn(9, H, device=DEV)
    w = torch.randn(H) * 0.3
    for zc in (True, False):
        n = RMSNorm(NormSpec(eps=1e-5, zero_centered=zc), H, torch.float32, DEV)
        n.load({"weight": w}, DEV)
        out = torch.empty_like(h)
        n.forward(h, out)
        ref = P.rms_norm(h.cpu().double(), w.double(), 1e-5, add_one=zc)
        close(out, ref, 1e-6)


def test_rotary_part_tables():
    from agave_b200.config import RotarySpec
    from agave_b200.parts import RotaryEmbedding

    class Ctx:
        rope_tables = {}
        n_tokens = 5
        positions = torch.tensor([0, 1, 2, 700, 4000], dtype=torch.int32, device=DEV)
        def new(self, *shape, dtype=None):
            return torch.empty(shape, dtype=dtype, device=DEV)

    r = RotaryEmbedding(RotarySpec(theta=5e5, factor=4.0, rotary_dim=24), head_dim=32)
    cos, sin = r.tables(Ctx())
    ang = P.rope_angles(Ctx.positions.cpu(), 24, 5e5, 4.0)
    close(cos, torch.cos(ang), 1e-6)
    close(sin, torch.sin(ang), 1e-6)
    assert r.tables(Ctx())[0] is cos            # made once per step and shared


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_and_feed_forward_parts_alone(dtype):
    """The mixer and the feed-forward of one layer, outside any model."""
    from agave_b200.cache import Cache
    from agave_b200.config import Gemma3Config
    from agave_b200.engine.batch import PREFILL, StepContext
    from agave_b200.parts import AttentionMixer, GatedFeedForward
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg = Gemma3Config.from_dict(TINY_B)
    spec = cfg.to_model_spec()
    block = spec.blocks[0]                      # a sliding layer
    H = spec.hidden_size
    g = torch.Generator().manual_seed(0)
    mixer = AttentionMixer(block.mixer, H, tdt, DEV)
    tensors = {n: (torch.randn(s.shape, generator=g) * (0.1 if s.role == "norm" else 0.05)).to(tdt)
               for n, s in AttentionMixer.param_specs(block.mixer, H).items()}
    mixer.load(tensors, tdt, DEV)
    ffn = GatedFeedForward(block.feed_forward, H, tdt, DEV)
    ften = {n: (torch.randn(s.shape, generator=g) * 0.05).to(tdt)
            for n, s in GatedFeedForward.param_specs(block.feed_forward, H).items()}
    ffn.load(ften, tdt, DEV)
    cache = Cache([mixer.cache_request()], 256, 256, 2, tdt, DEV)
    slot = cache.acquire()
    T = 40
    cache.reserve(slot, T)
    cache.flush()
    ar = torch.arange(T, dtype=torch.int32, device=DEV)
    ctx = StepContext(mode=PREFILL, n_tokens=T, batch=1, tokens=ar, positions=ar,
                      seq_index=torch.zeros(T, dtype=torch.int32, device=DEV),
                      cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=DEV),
                      slots=torch.tensor([slot], dtype=torch.int32, device=DEV),
                      lens=torch.tensor([T], dtype=torch.int32, device=DEV), max_len=T, max_new=T,
                      cache=cache, dtype=tdt, device=DEV)
    x = (torch.randn(T, H, generator=g) * 0.5).to(tdt).to(DEV)
    y = mixer.forward(x, ctx, 0, True)
    y = y.sum(0) if y.dim() == 3 else y          # partial sums over ranges of K
    # the same with the plain functions
    w = {"layers.0.self_attn." + n: t.double() for n, t in tensors.items()}
    pcfg = dict(TINY_B)
    ref = P.attention_block(pcfg, w, 0, x.cpu().double(), torch.arange(T))
    close(y, ref, 1e-4 if dtype == "float32" else 2e-2)
    d = ffn.forward(x, ctx)
    d = d.sum(0) if d.dim() == 3 else d
    ref = P.geglu(x.cpu().double(), ften["gate_proj.weight"].double(),
                  ften["up_proj.weight"].double(), ften["down_proj.weight"].double())
    close(d, ref, 1e-4 if dtype == "float32" else 2e-2)


# ------------------------------------------------- a toy mixer with its own state
class PrefixSumSpec:
    kind = "toy_prefix_sum"

    def __init__(self, width):
        self.width = width


class PrefixSumMixer:
    """y_t = W (x_1 + ... + x_t): the running sum is per-sequence state of fixed
    size, kept in the cache's state storage."""

    def __init__(self, spec, hidden_size, dtype, device):
        self.hidden_size, self.dtype, self.device = hidden_size, dtype, device
        self.w = None

    @classmethod
    def param_specs(cls, spec, hidden_size):
        from agave_b200.parts import ParamSpec
        return {"mix.weight": ParamSpec((hidden_size, hidden_size))}

    def cache_request(self):
        from agave_b200.parts import StateRequest
        return StateRequest(self.hidden_size)

    def load(self, tensors, dtype, device):
        self.w = tensors["mix.weight"].to(device=device, dtype=torch.float32)

    def forward(self, x, ctx, cache_entry, writes_cache):
        state = ctx.cache.state_view(cache_entry).state
        cu = ctx.cu_seqlens.cpu().tolist()
        slots = ctx.slots.cpu().tolist()
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for b, slot in enumerate(slots):
            if slot < 0:
                continue
            rows = slice(cu[b], cu[b + 1])
            c = torch.cumsum(x[rows].float(), dim=0) + state[slot]
            if writes_cache:
                state[slot] = c[-1]
            out[rows] = c @ self.w.T
        return out.to(x.dtype)


class ToyConfig:
    """hidden, vocab, layers, intermediate: a decoder of prefix-sum mixers in the
    "pre" arrangement with SiLU feed-forwards and ordinary (not zero-centred) norms."""

    def __init__(self, raw):
        self.raw = raw

    @classmethod
    def from_dict(cls, raw):
        return cls(raw)

    def to_model_spec(self):
        from agave_b200.config import (BlockSpec, GatedFeedForwardSpec, ModelSpec, NormSpec,
                                       default_schedule)
        r = self.raw
        norm = NormSpec(eps=r["eps"], zero_centered=False)
        blocks = tuple(BlockSpec(mixer=PrefixSumSpec(r["hidden"]),
                                 feed_forward=GatedFeedForwardSpec(intermediate_size=r["inter"],
                                                                   activation="silu"),
                                 norm=norm, arrangement="pre") for _ in range(r["layers"]))
        return ModelSpec(hidden_size=r["hidden"], vocab_size=r["vocab"], embed_scale=1.5,
                         blocks=blocks, schedule=default_schedule(len(blocks)), final_norm=norm,
                         tie_embeddings=True, max_positions=512)


class ToyNames:
    prefixes = ("toy.",)

    def checkpoint_name(self, internal, prefix):
        return prefix + internal


def toy_plain(raw, w, tokens):
    h = w["toy.embed.weight"][torch.tensor(tokens)] * 1.5
    for l in range(raw["layers"]):
        p = f"toy.blocks.{l}."
        x = P.rms_norm(h, w[p + "pre_mixer_norm.weight"], raw["eps"], add_one=False)
        h = h + torch.cumsum(x, 0) @ w[p + "mixer.mix.weight"].T
        x = P.rms_norm(h, w[p + "pre_ffn_norm.weight"], raw["eps"], add_one=False)
        gte = x @ w[p + "ffn.gate_proj.weight"].T
        d = (gte * torch.sigmoid(gte) * (x @ w[p + "ffn.up_proj.weight"].T)) \
            @ w[p + "ffn.down_proj.weight"].T
        h = h + d
    return P.rms_norm(h, w["toy.final_norm.weight"], raw["eps"], add_one=False) \
        @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype):
    from safetensors.torch import load_file
    from agave_b200.config import register_architecture
    from agave_b200.engine.api import Engine
    from agave_b200.parts import register_mixer
    from agave_b200.weights import write_model_folder
    register_mixer("toy_prefix_sum", PrefixSumMixer)
    register_architecture("ToyPrefixSumLM", ToyConfig, lambda c: ToyNames())
    raw = {"architectures": ["ToyPrefixSumLM"], "hidden": 72, "vocab": 300, "layers": 3,
           "inter": 104, "eps": 1e-5}
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, raw, seed=3, std=0.05, norm_std=0.1, dtype=store)
        w = {k: v.double() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
        eng = Engine(d, dtype=dtype, max_tokens=1024, max_batch=4)
    seqs = [random_tokens(n, 300, 70 + n) for n in (14, 6, 9)]
    refs = [toy_plain(raw, w, s) for s in seqs]
    # two batches, so that the state of a reused slot must have been zeroed
    for order in ([0, 1], [2, 1, 0]):
        slots = {i: eng.acquire() for i in order}
        starts = {i: max(1, len(seqs[i]) - 4) for i in order}
        out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in order],
                       [list(range(starts[i])) for i in order])
        got = {i: [] for i in order}
        o = 0
        for i in order:
            got[i].append(out[o:o + starts[i]]); o += starts[i]
        for k in range(4):
            live = [i for i in order if starts[i] + k < len(seqs[i])]
            out = eng.step([(slots[i], [seqs[i][starts[i] + k]]) for i in live],
                           [[0]] * len(live))
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
        for i in order:
            close(torch.cat(got[i]), refs[i], 1e-4 if dtype == "float32" else 3e-2)
            eng.release(slots[i])
    # through the generation loop, twice with the same sizes: this mixer reads device
    # data on the host, so neither a prompt step nor a decode step of it can be recorded
    # into a CUDA graph; the engine must notice and run it launch by launch
    if dtype == "float32":
        prompts = [seqs[0][:5], seqs[1][:5]]
        first = eng.generate(prompts, max_new_tokens=3, stop_token_ids=[])
        again = eng.generate(prompts, max_new_tokens=3, stop_token_ids=[])
        assert first == again and all(len(o) == 3 for o in first)
        for pr, o in zip(prompts, first):
            ref = toy_plain(raw, w, pr + o)
            for k, t in enumerate(o):
                row = ref[len(pr) - 1 + k]
                assert row[t] >= row.max() - 1e-3 * row.abs().max()


# ------------------------- the run order is data: a block twice, a shared cache
class LoopedGemmaConfig:
    def __init__(self, inner, order):
        self.inner, self.order = inner, order

    @classmethod
    def from_dict(cls, raw):
        from agave_b200.config import Gemma3Config
        return cls(Gemma3Config.from_dict(raw), raw["run_order"])

    def to_model_spec(self):
        from agave_b200.config import LayerCall
        spec = self.inner.to_model_spec()
        return dataclasses.replace(spec, schedule=tuple(
            LayerCall(block=b, cache=c, writes_cache=w) for b, c, w in self.order))

    def to_dict(self):
        return self.inner.to_dict()


def looped_plain(cfg, w, tokens, order):
    T = len(tokens)
    pos = torch.arange(T)
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    h = P.embed(tokens, w["embed_tokens.weight"], cfg["hidden_size"])
    kept = {}
    for l, cache, writes in order:
        p = f"layers.{l}."
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        local = P.layer_is_local(cfg, l)
        theta = cfg["rope_local_base_freq"] if local else cfg["rope_theta"]
        ang = P.rope_angles(pos, hd, theta, 1.0 if local else P.rope_factor(cfg))
        q = P.apply_rope(P.rms_norm((x @ w[p + "self_attn.q_proj.weight"].T).reshape(T, nh, hd),
                                    w[p + "self_attn.q_norm.weight"], eps), ang)
        if writes:
            k = P.apply_rope(P.rms_norm((x @ w[p + "self_attn.k_proj.weight"].T).reshape(T, nkv, hd),
                                        w[p + "self_attn.k_norm.weight"], eps), ang)
            v = (x @ w[p + "self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
            kept[cache] = (k, v)
        k, v = kept[cache]
        o = P.attention(q, k, v, 1.0 / math.sqrt(cfg["query_pre_attn_scalar"]),
                        cfg["sliding_window"] if local else None)
        y = o @ w[p + "self_attn.o_proj.weight"].T
        h = h + P.rms_norm(y, w[p + "post_attention_layernorm.weight"], eps)
        d = P.geglu(P.rms_norm(h, w[p + "pre_feedforward_layernorm.weight"], eps),
                    w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                    w[p + "mlp.down_proj.weight"])
        h = h + P.rms_norm(d, w[p + "post_feedforward_layernorm.weight"], eps)
    return P.rms_norm(h, w["norm.weight"], eps) @ w["embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_block_called_twice_and_a_layer_reading_anothers_cache(dtype):
    from agave_b200.config import register_architecture
    from agave_b200.engine.api import Engine
    from agave_b200.models.gemma3 import Gemma3WeightNames
    from agave_b200.weights import write_model_folder
    register_architecture("LoopedGemma3", LoopedGemmaConfig, lambda c: Gemma3WeightNames())
    raw = dict(TINY_B)
    raw["architectures"] = ["LoopedGemma3"]
    raw["num_hidden_layers"] = 3            # layers 0, 1 sliding; 2 global
    # block 0 runs twice with caches of its own; the last call reads block 2's cache
    raw["run_order"] = [[0, 0, True], [2, 1, True], [0, 2, True], [1, 3, True], [2, 1, False]]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, raw, seed=9, std=0.03, norm_std=0.2, dtype=store)
        cfg, w = P.read_config(d), P.read_weights(d)
        eng = Engine(d, dtype=dtype, max_tokens=1024, max_batch=2)
    toks = random_tokens(41, 384, 5)
    ref = looped_plain(cfg, w, toks, [tuple(o) for o in raw["run_order"]])
    s = eng.acquire()
    got = [eng.step([(s, toks[:30])], [list(range(30))])]
    for i in range(30, 41):
        got.append(eng.step([(s, [toks[i]])], [[0]]))
    eng.release(s)
    close(torch.cat(got), ref, TOL[dtype])


# ------------- a feed-forward with routing and another position encoding, both toys
class Top1Spec:
    kind = "toy_top1_experts"

    def __init__(self, n_experts, inter):
        self.n_experts, self.inter = n_experts, inter


class Top1Experts:
    """Each token goes to the expert with the greatest router logit (computed in
    32-bit) and is scaled by the softmax weight of that logit: a feed-forward whose
    work depends on the data.  Built on the library's own gated-linear kernels."""

    def __init__(self, spec, hidden_size, dtype, device):
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device

    @classmethod
    def param_specs(cls, spec, hidden_size):
        from agave_b200.parts import ParamSpec
        p = {"router.weight": ParamSpec((spec.n_experts, hidden_size), "float32")}
        for e in range(spec.n_experts):
            p[f"experts.{e}.gate_proj.weight"] = ParamSpec((spec.inter, hidden_size))
            p[f"experts.{e}.up_proj.weight"] = ParamSpec((spec.inter, hidden_size))
            p[f"experts.{e}.down_proj.weight"] = ParamSpec((hidden_size, spec.inter))
        return p

    def load(self, tensors, dtype, device):
        from agave_b200.parts.linear import GatedLinear, Linear
        self.router = tensors["router.weight"].to(device=device, dtype=torch.float32)
        self.experts = []
        for e in range(self.spec.n_experts):
            m = lambda n: tensors[f"experts.{e}.{n}"].to(device=device, dtype=dtype).contiguous()
            self.experts.append((GatedLinear(m("gate_proj.weight"), m("up_proj.weight"), "silu"),
                                 Linear(m("down_proj.weight"))))

    def forward(self, x, ctx):
        logits = x.float() @ self.router.T                         # 32-bit router
        weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e, (gate_up, down) in enumerate(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            y = down(gate_up(x[rows].contiguous()), out_dtype=torch.float32)
            out[rows] = y.float() * weight[rows, None]
        return out


class LinearPhaseSpec:
    """angle(p, i) = p * slope * (i + 1) over the first ``rotary_dim`` dims of a head."""
    kind = "toy_linear_phase"

    def __init__(self, slope, rotary_dim):
        self.slope, self.rotary_dim = slope, rotary_dim


class LinearPhase:
    def __init__(self, spec, head_dim):
        self.spec, self.rotary_dim = spec, spec.rotary_dim

    def tables(self, ctx):
        key = ("toy_linear_phase", self.spec.slope, self.rotary_dim)
        hit = ctx.rope_tables.get(key)
        if hit is None:
            i = torch.arange(1, self.rotary_dim // 2 + 1, device=ctx.device, dtype=torch.float64)
            ang = ctx.positions.double()[:, None] * (self.spec.slope * i)[None, :]
            hit = ctx.rope_tables[key] = (torch.cos(ang).float().contiguous(),
                                          torch.sin(ang).float().contiguous())
        return hit


class RoutedConfig:
    def __init__(self, raw):
        self.raw = raw

    @classmethod
    def from_dict(cls, raw):
        return cls(raw)

    def to_model_spec(self):
        from agave_b200.config import (AttentionSpec, BlockSpec, ModelSpec, NormSpec,
                                       default_schedule)
        r = self.raw
        norm = NormSpec(eps=r["eps"], zero_centered=False)
        att = AttentionSpec(n_heads=r["heads"], n_kv_heads=r["kv_heads"], head_dim=r["head_dim"],
                            scale=r["head_dim"] ** -0.5, window=None, qk_norm=None,
                            position=LinearPhaseSpec(r["slope"], r["rotary_dim"]))
        blocks = tuple(BlockSpec(mixer=att, feed_forward=Top1Spec(r["experts"], r["inter"]),
                                 norm=norm, arrangement="pre") for _ in range(r["layers"]))
        return ModelSpec(hidden_size=r["hidden"], vocab_size=r["vocab"], embed_scale=1.0,
                         blocks=blocks, schedule=default_schedule(len(blocks)), final_norm=norm,
                         tie_embeddings=True, max_positions=256)


def routed_plain(raw, w, tokens):
    T = len(tokens)
    nh, nkv, hd, rd = raw["heads"], raw["kv_heads"], raw["head_dim"], raw["rotary_dim"]
    i = torch.arange(1, rd // 2 + 1, dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * (raw["slope"] * i)[None, :]
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    for l in range(raw["layers"]):
        p = f"toy.blocks.{l}."
        x = P.rms_norm(h, w[p + "pre_mixer_norm.weight"], raw["eps"], add_one=False)
        q = P.apply_rope((x @ w[p + "mixer.q_proj.weight"].T).reshape(T, nh, hd), ang)
        k = P.apply_rope((x @ w[p + "mixer.k_proj.weight"].T).reshape(T, nkv, hd), ang)
        v = (x @ w[p + "mixer.v_proj.weight"].T).reshape(T, nkv, hd)
        h = h + P.attention(q, k, v, hd ** -0.5, None) @ w[p + "mixer.o_proj.weight"].T
        x = P.rms_norm(h, w[p + "pre_ffn_norm.weight"], raw["eps"], add_one=False)
        prob = torch.softmax(x @ w[p + "ffn.router.weight"].T, dim=-1)
        weight, choice = prob.max(dim=-1)
        d = torch.zeros_like(h)
        for t in range(T):
            e = int(choice[t])
            g = x[t] @ w[p + f"ffn.experts.{e}.gate_proj.weight"].T
            u = x[t] @ w[p + f"ffn.experts.{e}.up_proj.weight"].T
            d[t] = (g * torch.sigmoid(g) * u) @ w[p + f"ffn.experts.{e}.down_proj.weight"].T \
                * weight[t]
        h = h + d
    return P.rms_norm(h, w["toy.final_norm.weight"], raw["eps"], add_one=False) \
        @ w["toy.embed.weight"].T


def test_toy_routed_feed_forward_and_toy_position_encoding():
    """A feed-forward with routing and a position encoding of another formula (over
    part of the head only), registered here, in a model whose mixers are the
    library's attention: built, loaded by name, stepped whole and token by token."""
    from safetensors.torch import load_file
    from agave_b200.config import register_architecture
    from agave_b200.engine.api import Engine
    from agave_b200.parts import register_feed_forward, register_position
    from agave_b200.weights import write_model_folder
    register_feed_forward("toy_top1_experts", Top1Experts)
    register_position("toy_linear_phase", LinearPhase)
    register_architecture("ToyRoutedLM", RoutedConfig, lambda c: ToyNames())
    raw = {"architectures": ["ToyRoutedLM"], "hidden": 80, "vocab": 200, "layers": 2,
           "heads": 6, "kv_heads": 3, "head_dim": 24, "rotary_dim": 16, "slope": 0.07,
           "experts": 3, "inter": 56, "eps": 1e-5}
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, raw, seed=11, std=0.08, norm_std=0.1, dtype=torch.float32)
        w = {k: v.double() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
        eng = Engine(d, dtype="float32", max_tokens=512, max_batch=2)
    toks = random_tokens(23, 200, 3)
    ref = routed_plain(raw, w, toks)
    s = eng.acquire()
    got = [eng.step([(s, toks[:15])], [list(range(15))])]
    for t in toks[15:]:
        got.append(eng.step([(s, [t])], [[0]]))
    eng.release(s)
    close(torch.cat(got), ref, 2e-4)


# ------- a block of another shape and a position table added to the stream, both toys
class ParallelBlockSpec:
    """h += mixer(norm(h)) + ffn(norm(h)): one norm, both branches from it."""
    kind = "toy_parallel"

    def __init__(self, mixer, feed_forward, norm):
        self.mixer, self.feed_forward, self.norm = mixer, feed_forward, norm


class ParallelBlock:
    def __init__(self, spec, hidden_size, dtype, device):
        from agave_b200.parts import feed_forward_class, mixer_class, norm_class
        self.norm = norm_class(spec.norm.kind)(spec.norm, hidden_size, dtype, device)
        self.mixer = mixer_class(spec.mixer.kind)(spec.mixer, hidden_size, dtype, device)
        self.ffn = feed_forward_class(spec.feed_forward.kind)(spec.feed_forward, hidden_size,
                                                              dtype, device)

    @classmethod
    def param_specs(cls, spec, hidden_size):
        from agave_b200.parts import feed_forward_class, mixer_class, norm_class
        out = {f"norm.{k}": v
               for k, v in norm_class(spec.norm.kind).param_specs(spec.norm, hidden_size).items()}
        out.update({f"mixer.{k}": v for k, v in
                    mixer_class(spec.mixer.kind).param_specs(spec.mixer, hidden_size).items()})
        out.update({f"ffn.{k}": v for k, v in feed_forward_class(spec.feed_forward.kind)
                    .param_specs(spec.feed_forward, hidden_size).items()})
        return out

    @property
    def entry_norm(self):
        return self.norm

    def cache_request(self):
        return self.mixer.cache_request()

    def load(self, tensors, dtype, device):
        sub = lambda p: {k[len(p) + 1:]: v for k, v in tensors.items() if k.startswith(p + ".")}
        self.norm.load(sub("norm"), device)
        self.mixer.load(sub("mixer"), dtype, device)
        self.ffn.load(sub("ffn"), dtype, device)

    def forward(self, h, x, ctx, cache_entry, writes_cache, next_norm):
        y = self.mixer.forward(x, ctx, cache_entry, writes_cache)
        d = self.ffn.forward(x, ctx)
        for branch in (y, d):                        # (partial sums over ranges of K are added)
            h += branch.float().sum(0) if branch.dim() == 3 else branch.float()
        if next_norm is None:
            return None
        x_next = ctx.new(*x.shape)
        next_norm.forward(h, x_next)
        return x_next


class LearnedPositionsSpec:
    kind = "toy_learned_positions"

    def __init__(self, n_positions):
        self.n_positions = n_positions


class LearnedPositions:
    """h[t] += table[position of t]: a position encoding with no seat inside a mixer."""

    def __init__(self, spec, hidden_size, dtype, device):
        self.spec = spec

    @classmethod
    def param_specs(cls, spec, hidden_size):
        from agave_b200.parts import ParamSpec
        return {"table.weight": ParamSpec((spec.n_positions, hidden_size), "float32")}

    def load(self, tensors, device):
        self.table = tensors["table.weight"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h, ctx):
        from agave_b200 import kernels
        add = torch.empty_like(h)
        kernels.embed(ctx.positions, self.table, 1.0, add)      # the library's own gather
        h += add


class ParallelConfig:
    def __init__(self, raw):
        self.raw = raw

    @classmethod
    def from_dict(cls, raw):
        return cls(raw)

    def to_model_spec(self):
        from agave_b200.config import (AttentionSpec, GatedFeedForwardSpec, ModelSpec, NormSpec,
                                       default_schedule)
        r = self.raw
        norm = NormSpec(eps=r["eps"], zero_centered=False)
        att = AttentionSpec(n_heads=r["heads"], n_kv_heads=r["kv_heads"], head_dim=r["head_dim"],
                            scale=r["head_dim"] ** -0.5, window=r["window"], qk_norm=None,
                            position=None)
        ffn = GatedFeedForwardSpec(intermediate_size=r["inter"], activation="gelu_tanh")
        blocks = tuple(ParallelBlockSpec(att, ffn, norm) for _ in range(r["layers"]))
        return ModelSpec(hidden_size=r["hidden"], vocab_size=r["vocab"], embed_scale=1.0,
                         blocks=blocks, schedule=default_schedule(len(blocks)), final_norm=norm,
                         tie_embeddings=True, max_positions=r["positions"],
                         stream_position=LearnedPositionsSpec(r["positions"]))


def parallel_plain(raw, w, tokens):
    T = len(tokens)
    nh, nkv, hd = raw["heads"], raw["kv_heads"], raw["head_dim"]
    h = w["toy.embed.weight"][torch.tensor(tokens)] + w["toy.stream_position.table.weight"][:T]
    for l in range(raw["layers"]):
        p = f"toy.blocks.{l}."
        x = P.rms_norm(h, w[p + "norm.weight"], raw["eps"], add_one=False)
        q = (x @ w[p + "mixer.q_proj.weight"].T).reshape(T, nh, hd)
        k = (x @ w[p + "mixer.k_proj.weight"].T).reshape(T, nkv, hd)
        v = (x @ w[p + "mixer.v_proj.weight"].T).reshape(T, nkv, hd)
        y = P.attention(q, k, v, hd ** -0.5, raw["window"]) @ w[p + "mixer.o_proj.weight"].T
        d = P.geglu(x, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                    w[p + "ffn.down_proj.weight"])
        h = h + y + d
    return P.rms_norm(h, w["toy.final_norm.weight"], raw["eps"], add_one=False) \
        @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_block_of_another_shape_and_positions_added_to_the_stream(dtype):
    """A block that is not "norm, mixer, add, norm, feed-forward, add" and a position
    encoding that is not a rotation inside a mixer: registered here, built through the
    block and stream-position registries, loaded by name, stepped whole, token by token
    and through the generation loop (whose steps are recorded, these parts being
    launches only)."""
    from safetensors.torch import load_file
    from agave_b200.config import register_architecture
    from agave_b200.engine.api import Engine
    from agave_b200.parts import register_block, register_stream_position
    from agave_b200.weights import write_model_folder
    register_block("toy_parallel", ParallelBlock)
    register_stream_position("toy_learned_positions", LearnedPositions)
    register_architecture("ToyParallelLM", ParallelConfig, lambda c: ToyNames())
    raw = {"architectures": ["ToyParallelLM"], "hidden": 96, "vocab": 260, "layers": 3,
           "heads": 4, "kv_heads": 2, "head_dim": 32, "window": 11, "inter": 160, "eps": 1e-5,
           "positions": 128}
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, raw, seed=13, std=0.06, norm_std=0.1, dtype=store)
        w = {k: v.double() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
        eng = Engine(d, dtype=dtype, max_tokens=512, max_batch=4)
    seqs = [random_tokens(n, 260, 30 + n) for n in (37, 12)]
    refs = [parallel_plain(raw, w, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    starts = [29, 5]
    out = eng.step([(slots[i], seqs[i][:starts[i]]) for i in range(2)],
                   [list(range(starts[i])) for i in range(2)])
    got = [[out[:starts[0]]], [out[starts[0]:]]]
    for k in range(8):
        live = [i for i in range(2) if starts[i] + k < len(seqs[i])]
        res = eng.step([(slots[i], [seqs[i][starts[i] + k]]) for i in live], [[0]] * len(live))
        for j, i in enumerate(live):
            got[i].append(res[j:j + 1])
    for i in range(2):
        close(torch.cat(got[i]), refs[i], 2e-4 if dtype == "float32" else 3e-2)
        eng.release(slots[i])
    prompts = [s[:6] for s in seqs]
    outs = eng.generate(prompts, max_new_tokens=5, stop_token_ids=[])
    for pr, o in zip(prompts, outs):
        ref = parallel_plain(raw, w, pr + o)
        for k, t in enumerate(o):
            row = ref[len(pr) - 1 + k]
            assert row[t] >= row.max() - (1e-3 if dtype == "float32" else 6e-2) * row.abs().max()
