"""The Python entry point: a model folder (or a configuration and a seed) in,
token ids out.

    engine = Engine("model-dir", dtype="bfloat16", max_tokens=65536)
    outs = engine.generate([[2, 17, 5], [2, 9]], max_new_tokens=32)

``Engine.step`` is the step function that trace replay drives; ``generate``
is the loop above it.  Decode steps of ``generate`` are recorded once per
batch size as a CUDA graph and replayed; per step the host writes the batch's
token ids, positions and slots into pinned memory, copies them to the graph's
fixed input buffers and reads the chosen tokens back.
"""
from __future__ import annotations

import dataclasses
import json
import os
import threading
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..cache import PAGE, CacheError, round_up
from ..config import load_config, resolve_architecture
from ..models.decoder import DecoderModel, decoder_param_specs
from ..sampling import Sampler, SamplingParams
from ..weights import head_is_stored, load_weights, random_tensors
from .batch import DECODE, PREFILL, Cancelled, StepContext
from .generate import GenerationPlan, RequestState
from .step import Runner, StepError

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def _bucket(n: int) -> int:
    """Padded size of a decode batch: powers of two up to 8, then multiples of 8."""
    if n <= 8:
        b = 1
        while b < n:
            b *= 2
        return b
    return round_up(n, 8)


class _DecodeGraph:
    """One recorded decode step for a padded batch size and a kind of choice (arg
    max or a draw, with or without the repeat penalty).  The sampling options
    themselves (temperature, top_k, top_p, seed, penalty) are step inputs on the
    device, so one recording serves every setting of its kind."""

    def __init__(self, engine: "Engine", size: int, params: SamplingParams, seed: int):
        self.size = size
        dev = engine.device
        B = size
        n_int = round_up(3 * B + 3 * B + 1 + B + 1, 2)  # step arrays, sampling steps, flag; even
        total = n_int + 2 * B + kernels.SAMPLING_WORDS  # + sequence ids (64-bit) + sampling words
        # two pinned staging buffers: the next step's arrays are filled while the
        # copy of this step's may still be in flight
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.host, self.host_np = self.hosts[0], self.hosts_np[0]
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        d = self.dev
        self.words_at = n_int + 2 * B
        self.words = d[self.words_at:]
        o = 3 * B
        self.views = dict(tokens=d[:B], positions=d[B:2 * B], seq_index=d[2 * B:3 * B],
                          cu=d[o:o + B + 1], slots=d[o + B + 1:o + 2 * B + 1],
                          lens=d[o + 2 * B + 1:o + 3 * B + 1],
                          steps=d[o + 3 * B + 1:o + 4 * B + 1],
                          take=d[o + 4 * B + 1:o + 4 * B + 2])
        self.flag_at = o + 4 * B + 1
        self.seq_ids = d[n_int:n_int + 2 * B].view(torch.int64)
        self.n_int = n_int
        self.rows = torch.arange(B, dtype=torch.int32, device=dev)
        self.next_dev = torch.zeros(B, dtype=torch.int32, device=dev)
        # one result buffer and one event per staging buffer: a step may be launched
        # before the result of the step before it has been read
        self.next_hosts = [torch.zeros(B, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.done = [torch.cuda.Event() for _ in range(2)]
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_step = 0
        self._record(engine, params, seed)

    def _body(self, engine: "Engine", params: SamplingParams, seed: int,
              lens_host=None) -> None:
        v = self.views
        runner = engine.runner
        # a step launched ahead takes its token ids from the choices of the step before
        kernels.take_tokens(v["tokens"], self.next_dev, v["take"], runner.vocab_size)
        ctx = StepContext(mode=DECODE, n_tokens=self.size, batch=self.size, tokens=v["tokens"],
                          positions=v["positions"], seq_index=v["seq_index"],
                          cu_seqlens=v["cu"], slots=v["slots"], lens=v["lens"],
                          max_len=runner.cache.max_seq_len, max_new=1, cache=runner.cache,
                          dtype=runner.dtype, device=runner.device, lens_host=lens_host)
        engine.sampler.note_inputs(v["tokens"], v["slots"])
        fused = params.greedy and params.repeat_penalty == 1.0 and engine.fused_greedy
        self.logits = runner.model.run_step(ctx, self.rows,
                                            choose_into=self.next_dev if fused else None)
        if self.logits is None:
            return                     # the greatest logit was found in the head's epilogue
        engine.sampler.choose(self.logits, self.next_dev, params, seed, v["slots"], self.seq_ids,
                              v["steps"], penalise=True, dev_params=self.words)

    def _record(self, engine: "Engine", params: SamplingParams, seed: int) -> None:
        if not engine.use_graphs:
            return
        self.host_np[:] = 0
        B = self.size
        self.host_np[3 * B + B + 1:3 * B + 2 * B + 1] = -1      # all padding while recording
        self.dev.copy_(self.host)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = kernels.launch_count()
        try:
            with torch.cuda.graph(g):
                self._body(engine, params, seed)
        except RuntimeError:
            # a part that cannot be recorded (one that reads device data on the host,
            # say): this batch size runs launch by launch
            torch.cuda.synchronize()
            self.kernels_per_step = kernels.launch_count() - n0
            return
        self.kernels_per_step = kernels.launch_count() - n0
        self.graph = g

    def launch(self, engine: "Engine", params: SamplingParams, seed: int, which: int = 0) -> None:
        """Copy staging buffer ``which`` in, run the step, start the copy of the
        chosen tokens out; returns without waiting."""
        self.dev.copy_(self.hosts[which], non_blocking=True)
        if kernels._perf is not None:
            # per-operation timing: the step runs launch by launch, lengths known to the host
            B = self.size
            lens = self.hosts_np[which][5 * B + 1:6 * B + 1].copy()
            kernels._perf.n_tokens += int((lens > 0).sum())
            self._body(engine, params, seed, lens_host=lens)
        elif self.graph is not None:
            self.graph.replay()
        else:
            self._body(engine, params, seed)
        self.next_hosts[which].copy_(self.next_dev, non_blocking=True)
        self.done[which].record()

    def wait(self, which: int = 0) -> "np.ndarray":
        """The tokens chosen by the step launched from staging buffer ``which``."""
        self.done[which].synchronize()
        return self.next_hosts[which].numpy()

    def run(self, engine: "Engine", params: SamplingParams, seed: int) -> None:
        self.launch(engine, params, seed)
        self.wait()


class Engine:
    """A loaded model with its cache, step function and generation loop."""

    def __init__(self, model_dir: Optional[str] = None, *, dtype: str = "bfloat16",
                 max_tokens: int = 65536, ctx_size: int = 0, max_batch: Optional[int] = None,
                 device: str = "cuda:0", use_graphs: bool = True, strict: bool = False,
                 _raw_config: Optional[dict] = None, _tensors: Optional[dict] = None):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype {dtype!r} is not supported (bfloat16, float32)")
        if not torch.cuda.is_available():
            raise RuntimeError("agave_b200 needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        arch = kernels.device_arch()
        if arch // 10 != 10:
            raise RuntimeError(f"the kernels are built for sm_100a; this device is sm_{arch}")
        self.dtype = _DTYPES[dtype]
        t0 = time.time()
        if model_dir is not None:
            self.entry, self.config = load_config(model_dir)
        else:
            self.entry = resolve_architecture(_raw_config)
            self.config = self.entry.config_class.from_dict(_raw_config)
        self.spec = self.config.to_model_spec()
        names = self.entry.weight_names(self.config)
        self.ignored_tensors: List[str] = []
        if model_dir is not None and self.spec.tie_embeddings and head_is_stored(
                model_dir, names.checkpoint_name, names.prefixes):
            # a head of its own in the files wins over the configuration's word: the
            # reference ties by absence (src/format/safetensors.zig:531-540)
            self.spec = dataclasses.replace(self.spec, tie_embeddings=False)
        self.model = DecoderModel(self.spec, self.dtype, self.device)
        if model_dir is not None:
            tensors = load_weights(model_dir, self.model.param_specs(), names.checkpoint_name,
                                   names.prefixes, strict=strict,
                                   ignore_prefixes=getattr(names, "ignore_prefixes", ()))
            self.ignored_tensors = list(tensors.ignored)
        else:
            tensors = _tensors
        self.model.load(tensors)
        del tensors
        self.load_seconds = time.time() - t0
        # context: 0 = the model's own limit (src/main.zig:1102-1113 caps it at 4096
        # by default; here the cache's token budget is the cap)
        limit = self.spec.max_positions or max_tokens
        max_seq_len = min(ctx_size or limit, limit)
        if max_batch is None:
            max_batch = max(1, min(1024, round_up(max_tokens, PAGE) // PAGE))
        self.max_batch, self.max_tokens = max_batch, max_tokens
        self.runner = Runner(self.model, max_tokens, max_seq_len, max_batch,
                             use_graphs=use_graphs)
        self.max_seq_len = self.runner.cache.max_seq_len
        self.sampler = Sampler(max_batch, self.device)
        kernels.prepare_device(self.device)
        self.use_graphs = use_graphs
        self._graphs: Dict[Tuple, _DecodeGraph] = {}
        self.stats: Dict[str, float] = {}
        # greedy decoding takes the arg max in the head product's epilogue
        self.fused_greedy = os.environ.get("AGAVE_B200_FUSED_GREEDY", "1") != "0"
        self._cancel = threading.Event()
        self.runner.cancel_flag = self._cancel

    @classmethod
    def from_config(cls, raw_config: dict, seed: int = 0, std: float = 0.02,
                    norm_std: float = 0.1, **kw) -> "Engine":
        """A model with seeded random weights, drawn on the device."""
        entry = resolve_architecture(raw_config)
        config = entry.config_class.from_dict(raw_config)
        specs = decoder_param_specs(config.to_model_spec())
        dtype = _DTYPES[kw.get("dtype", "bfloat16")]
        device = kw.get("device", "cuda:0")
        tensors = random_tensors(specs, seed, std, norm_std, dtype, device)
        return cls(None, _raw_config=raw_config, _tensors=tensors, **kw)

    # ------------------------------------------------------------ step level
    def acquire(self) -> int:
        s = self.runner.acquire()
        self.sampler.reset(s)
        return s

    def release(self, slot: int) -> None:
        self.runner.release(slot)

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Sequence[Sequence[int]]) -> torch.Tensor:
        """See ``Runner.step``.  Raises ``Cancelled`` (and runs nothing further) when
        ``cancel()`` was called; the flag is cleared by that."""
        try:
            return self.runner.step(entries, want)
        except Cancelled:
            self._cancel.clear()
            raise

    def cancel(self) -> None:
        """Stop the running ``generate`` or ``step`` at its next check, from any thread
        (src/models/model.zig:443-446).  A step that runs launch by launch stops between
        two blocks (src/models/gemma3.zig:342,435); a recorded step runs to its end, and
        the generation loop stops before the next one.  ``generate`` then returns what
        was generated so far, with the finish reason "cancelled" for what it cut."""
        self._cancel.set()

    # ------------------------------------------------------------- generate
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 512,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 repeat_penalty: float = 1.0, seed: Optional[int] = None,
                 stop_token_ids: Optional[Sequence[int]] = None) -> List[List[int]]:
        """Token ids generated for each prompt (stop tokens excluded).

        Option names and defaults are the reference's (src/main.zig:333-338):
        temperature 0 is greedy.  ``stop_token_ids`` defaults to the
        configuration's end-of-sequence ids.
        """
        params = SamplingParams(temperature, top_k, top_p, repeat_penalty, seed).validate()
        seed_v = 0 if params.greedy else params.resolved_seed()
        stops = self.spec.eos_token_ids if stop_token_ids is None else tuple(stop_token_ids)
        plan = GenerationPlan(prompts, max_new_tokens, stops, self.max_batch, self.max_tokens,
                              self.max_seq_len)
        stats = dict(prefill_tokens=0, prefill_seconds=0.0, decode_tokens=0, decode_seconds=0.0,
                     decode_steps=0, batches=0)
        try:
            while True:
                batch = plan.next_batch()
                if not batch:
                    break
                stats["batches"] += 1
                try:
                    self._run_batch(plan, batch, params, seed_v, stats)
                except Cancelled:
                    plan.cancel()
                if self._cancel.is_set():
                    plan.cancel()
        finally:
            self._cancel.clear()
        self.stats = stats
        self.finish_reasons = [r.finish_reason for r in plan.requests]
        return plan.outputs()

    def _run_batch(self, plan: GenerationPlan, batch, params: SamplingParams, seed: int,
                   stats: dict) -> None:
        dev = self.device
        for r in batch:
            r.slot = self.acquire()
        try:
            # the prompts, in one step; logits of each last token
            t0 = time.perf_counter()
            entries = [(r.slot, r.prompt) for r in batch]
            logits = self.step(entries, [[len(r.prompt) - 1] for r in batch])
            B = len(batch)
            slots = torch.tensor([r.slot for r in batch], dtype=torch.int32).to(dev)
            seq_ids = torch.tensor([r.index for r in batch], dtype=torch.int64).to(dev)
            steps = torch.zeros(B, dtype=torch.int32, device=dev)
            first = torch.empty(B, dtype=torch.int32, device=dev)
            self.sampler.choose(logits, first, params, seed, slots, seq_ids, steps,
                                penalise=False)
            first_host = first.cpu()
            stats["prefill_seconds"] += time.perf_counter() - t0
            stats["prefill_tokens"] += sum(len(r.prompt) for r in batch)
            ended = plan.accept({r.index: int(first_host[i]) for i, r in enumerate(batch)})
            for r in ended:
                self.release(r.slot)
                r.slot = -1
            # one token each until the batch is empty
            t0 = time.perf_counter()
            self._decode_loop(plan, params, seed, stats)
            stats["decode_seconds"] += time.perf_counter() - t0
        finally:
            for r in batch:
                if r.slot >= 0:
                    self.release(r.slot)
                    r.slot = -1

    def _graph_for(self, size: int, params: SamplingParams, seed: int) -> _DecodeGraph:
        # what is fixed in a recording: the padded batch and which kernels choose the token
        key = (size, params.greedy, params.repeat_penalty != 1.0)
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= 64:
                self._graphs.clear()
            g = self._graphs[key] = _DecodeGraph(self, size, params, seed)
        return g

    def _stage_step(self, live, params: SamplingParams, seed: int, ahead: int, which: int):
        """Fill staging buffer ``which`` of the live set's graph with everything a
        decode step needs except the token ids, for the step ``ahead`` steps after
        the last committed one; reserves the cache rows it will write."""
        n = len(live)
        B = _bucket(n)
        g = self._graph_for(B, params, seed)
        book = self.runner.cache.book
        for r in live:
            self.runner.cache.reserve(r.slot, book.length[r.slot] + ahead + 1)
        a = g.hosts_np[which]
        lens = np.fromiter((book.length[r.slot] + ahead for r in live), dtype=np.int32, count=n)
        a[:2 * B] = 0
        a[B:B + n] = lens
        a[2 * B:3 * B] = np.arange(B, dtype=np.int32)
        o = 3 * B
        a[o:o + B + 1] = np.arange(B + 1, dtype=np.int32)
        a[o + B + 1:o + 2 * B + 1] = -1
        a[o + B + 1:o + B + 1 + n] = np.fromiter((r.slot for r in live), dtype=np.int32, count=n)
        a[o + 2 * B + 1:o + 4 * B + 1] = 0
        a[o + 2 * B + 1:o + 2 * B + 1 + n] = lens + 1
        a[o + 3 * B + 1:o + 3 * B + 1 + n] = np.fromiter((len(r.output) + ahead for r in live),
                                                        dtype=np.int32, count=n)
        ids = a[g.n_int:g.words_at].view(np.int64)
        ids[:] = 0
        ids[:n] = np.fromiter((r.index for r in live), dtype=np.int64, count=n)
        a[g.words_at:] = kernels.sampling_words(params.temperature, params.top_k, params.top_p,
                                                seed, params.repeat_penalty)
        return g

    def _decode_loop(self, plan: GenerationPlan, params: SamplingParams, seed: int,
                     stats: dict) -> None:
        """One token for every live sequence per step until the batch is empty.

        A step is launched before the host has read the step before it (its token
        ids come from that step's choices on the device), unless a sequence reaches
        its token limit with the step in flight; so the GPU does not idle while the
        host reads tokens and checks stop ids.  When a stop id turns up, the step
        already in flight still ran the ended sequence: its token is dropped and its
        slot is released once that step has been read.
        """
        book = self.runner.cache.book
        cache = self.runner.cache
        live = plan.live()
        which = 0
        inflight = None                    # (graph, staging buffer, requests) launched, not read
        held: List[RequestState] = []      # ended, but a step in flight still uses their slots
        while live or inflight is not None:
            if self._cancel.is_set() and inflight is None:
                # between two steps, nothing in flight: the live sequences end here
                for r in plan.cancel():
                    self.release(r.slot)
                    r.slot = -1
                return
            if inflight is None:
                n = len(live)
                g = self._stage_step(live, params, seed, 0, which)
                g.hosts_np[which][:n] = np.fromiter((r.output[-1] for r in live), dtype=np.int32,
                                                    count=n)
                g.hosts_np[which][g.flag_at] = 0
                cache.flush()
                g.launch(self, params, seed, which)
                inflight = (g, which, list(live))
            g, w, reqs = inflight
            # the step after it, for the same sequences
            ahead = None
            if (not self._cancel.is_set() and
                    all(not r.done and len(r.output) + 1 < r.max_new for r in reqs)):
                try:
                    g2 = self._stage_step(reqs, params, seed, 1, 1 - w)
                    g2.hosts_np[1 - w][g2.flag_at] = 1
                    cache.flush()
                    g2.launch(self, params, seed, 1 - w)
                    ahead = (g2, 1 - w, reqs)
                except (CacheError, StepError):
                    ahead = None           # a sequence is at the end of its room
            out = g.wait(w)
            current = [(i, r) for i, r in enumerate(reqs) if not r.done]
            sampled = {r.index: int(out[i]) for i, r in current}
            for _, r in current:
                book.set_length(r.slot, book.length[r.slot] + 1)
            stats["decode_steps"] += 1
            stats["decode_tokens"] += len(current)
            ended = plan.accept(sampled)
            if ahead is not None:
                held.extend(ended)
                inflight = ahead
            else:
                for r in held + ended:
                    self.release(r.slot)
                    r.slot = -1
                held = []
                inflight = None
                live = plan.live()
                which = 1 - w

    # ----------------------------------------------------------------- info
    def model_info(self) -> dict:
        """What ``--model-info`` prints (src/main.zig:376)."""
        c = self.config
        return {
            "architecture": self.entry.name,
            "config": c.to_dict() if hasattr(c, "to_dict") else {},
            "dtype": str(self.dtype).replace("torch.", ""),
            "weight_bytes": self.model.weight_bytes(),
            "cache_bytes": self.runner.cache.bytes_held(),
            "max_seq_len": self.max_seq_len,
            "max_tokens": self.max_tokens,
            "max_batch": self.max_batch,
        }
