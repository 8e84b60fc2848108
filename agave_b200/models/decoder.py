"""The generic decoder: embedding, blocks run in the order the spec lists,
final norm, head.  It is built from a ``ModelSpec`` through the part
registries and knows no architecture by name.

Internal tensor names (what ``decoder_param_specs`` lists and ``load`` takes):
``embed.weight``, ``blocks.{i}.<block-local name>``, ``final_norm.weight`` and,
unless the head is tied to the embedding, ``lm_head.weight``.  An
architecture maps these to the names its checkpoints use.

Flow of one step (src/models/gemma3.zig:331-368 for one token, :413-442 for a
prompt chunk): embedding times the spec's scale into a 32-bit stream, the
blocks, the final norm on the rows whose logits are wanted, the head in
32-bit output.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..config.base import ModelSpec
from ..engine.batch import DECODE, Cancelled
from ..parts import block as _block      # registers the "sequential" block
from ..parts.base import ParamSpec, block_class, norm_class, stream_position_class
from ..parts.linear import Linear


def decoder_param_specs(spec: ModelSpec) -> Dict[str, ParamSpec]:
    out: Dict[str, ParamSpec] = {
        "embed.weight": ParamSpec((spec.vocab_size, spec.hidden_size), "embedding")}
    for i, b in enumerate(spec.blocks):
        B = block_class(getattr(b, "kind", "sequential"))
        for k, v in B.param_specs(b, spec.hidden_size).items():
            out[f"blocks.{i}.{k}"] = v
    if spec.stream_position is not None:
        S = stream_position_class(spec.stream_position.kind)
        for k, v in S.param_specs(spec.stream_position, spec.hidden_size).items():
            out[f"stream_position.{k}"] = v
    N = norm_class(spec.final_norm.kind)
    for k, v in N.param_specs(spec.final_norm, spec.hidden_size).items():
        out[f"final_norm.{k}"] = v
    if not spec.tie_embeddings:
        out["lm_head.weight"] = ParamSpec((spec.vocab_size, spec.hidden_size), "matrix")
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype {dtype} is not supported (float32, bfloat16)")
        self.spec, self.dtype, self.device = spec, dtype, device
        self.blocks: List[object] = [
            block_class(getattr(b, "kind", "sequential"))(b, spec.hidden_size, dtype, device)
            for b in spec.blocks]
        self.stream_position = None
        if spec.stream_position is not None:
            self.stream_position = stream_position_class(spec.stream_position.kind)(
                spec.stream_position, spec.hidden_size, dtype, device)
        self.final_norm = norm_class(spec.final_norm.kind)(spec.final_norm, spec.hidden_size,
                                                           dtype, device)
        self.embed_table: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None
        self.native = None             # the C++ host side of a step, if the model allows it
        self.standard = False          # every block the standard arrangement of the library's parts
        for call in spec.schedule:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"the run order names block {call.block}, which does not exist")
        writers = {}
        for call in spec.schedule:
            if call.writes_cache:
                if call.cache in writers:
                    raise ValueError(f"cache entry {call.cache} is written by two calls")
                writers[call.cache] = call.block
        for call in spec.schedule:
            if not call.writes_cache and call.cache not in writers:
                raise ValueError(f"cache entry {call.cache} is read but never written")
        self._writers = writers

    # ----------------------------------------------------------------- cache
    def cache_requests(self) -> List[object]:
        """What each cache entry must hold, in entry order (None: nothing)."""
        n = self.spec.n_cache_entries()
        out: List[object] = [None] * n
        for entry, block in self._writers.items():
            out[entry] = self.blocks[block].cache_request()
        return out

    # --------------------------------------------------------------- weights
    def param_specs(self) -> Dict[str, ParamSpec]:
        return decoder_param_specs(self.spec)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take tensors under their internal names (any device, as stored)."""
        dt, dev = self.dtype, self.device
        self.embed_table = tensors["embed.weight"].to(device=dev, dtype=dt).contiguous()
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}."
            b.load({k[len(p):]: v for k, v in tensors.items() if k.startswith(p)}, dt, dev)
        if self.stream_position is not None:
            p = "stream_position."
            self.stream_position.load({k[len(p):]: v for k, v in tensors.items()
                                       if k.startswith(p)}, dev)
        self.final_norm.load({"weight": tensors["final_norm.weight"]}, dev)
        if self.spec.tie_embeddings:
            self.head = Linear(self.embed_table, role="lm_head")
        else:
            self.head = Linear(tensors["lm_head.weight"].to(device=dev, dtype=dt).contiguous(),
                               role="lm_head")
        from .native import NativeStep, standard_blocks
        self.standard = standard_blocks(self)
        self.native = NativeStep.build(self)

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        def visit(o):
            nonlocal n
            if isinstance(o, torch.Tensor):
                if o.data_ptr() not in seen:
                    seen.add(o.data_ptr())
                    n += o.numel() * o.element_size()
            elif isinstance(o, (list, tuple)):
                for i in o:
                    visit(i)
            elif hasattr(o, "__dict__") and not isinstance(o, (type, torch.dtype, torch.device)):
                if id(o) in seen:
                    return
                seen.add(id(o))
                for v in vars(o).values():
                    visit(v)
        visit(self.blocks); visit(self.final_norm); visit(self.embed_table); visit(self.head)
        visit(self.stream_position)
        return n

    # --------------------------------------------------------------- forward
    def _few_tokens(self, ctx) -> bool:
        """Whether this step is a decode step of so few tokens that its projections run as
        dot products with the joins in their prologues (``kernels.gemv_few``)."""
        T = ctx.n_tokens
        if ctx.mode != DECODE or not self.standard or self.dtype != torch.bfloat16 or \
                not 1 <= T <= kernels.FEW_TOKENS or not self.spec.schedule:
            return False
        H = self.spec.hidden_size
        for call in self.spec.schedule:
            b = self.blocks[call.block]
            s = b.mixer.spec
            width = (s.n_heads + 2 * s.n_kv_heads) * s.head_dim
            rd = b.mixer.position.rotary_dim if b.mixer.position is not None else 0
            ff = b.ffn.spec.intermediate_size
            # (a layer of more than 96 MB is bound by how fast its weights stream, and there
            # the tensor-core products, fed by TMA, are ahead)
            if 2 * (width * H + H * s.n_heads * s.head_dim + 3 * ff * H) > 96 * 1024 * 1024:
                return False
            if not (kernels.attention_decode_fused_supported(self.dtype, s.head_dim, rd) and
                    kernels.gemv_few_supported(T, width, H, join=True) and
                    kernels.gemv_few_supported(T, H, s.n_heads * s.head_dim, s.n_heads * s.head_dim) and
                    kernels.gemv_few_supported(T, ff, H, join=True) and
                    kernels.gemv_few_supported(T, H, ff, ff)):
                return False
        return True

    def _blocks_few_tokens(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """The blocks of such a step; returns the buffer that holds the stream afterwards
        (it alternates between two, because all CTAs of a projection read the stream while
        one of them writes the joined one)."""
        T, H = h.shape
        cur, other = h, ctx.new(T, H, dtype=torch.float32)
        y_down = ctx.new(T, H, dtype=torch.float32)
        pend = None                                    # (branch output, its norm) the next join adds
        sched = self.spec.schedule
        for i, call in enumerate(sched):
            if ctx.cancel is not None and ctx.cancel.is_set():
                raise Cancelled(f"cancelled before block {i} of {len(sched)}")
            b = self.blocks[call.block]
            m, s = b.mixer, b.mixer.spec
            nh, nkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
            width = (nh + 2 * nkv) * hd
            cos = sin = None
            if m.position is not None:
                cos, sin = m.position.tables(ctx)
            view = ctx.cache.kv_view(call.cache)
            qkv = ctx.new(T, width, dtype=torch.float32)
            post = pend[1] if pend is not None else None
            kernels.gemv_few(m.qkv.weight, qkv, h_in=cur, h_out=other if pend is not None else None,
                             y=pend[0] if pend is not None else None,
                             w_post=post.weight if post is not None else None,
                             w_next=b.pre_mixer_norm.weight,
                             eps_post=post.eps if post is not None else 0.0,
                             eps_next=b.pre_mixer_norm.eps, op="qkv")
            if pend is not None:
                cur, other = other, cur
            att = ctx.new(T, nh * hd)
            kernels.attention_decode_fused(
                qkv.view(1, T, width), m.q_norm_weight, m.k_norm_weight,
                s.qk_norm.eps if s.qk_norm is not None else 0.0, cos, sin, True, att, view, ctx, nh,
                nkv, hd, s.scale, s.window or 0)
            y_out = ctx.new(T, H, dtype=torch.float32)
            kernels.gemv_few(m.out.weight, y_out, x=att, op="out_proj")
            z = ctx.new(T, b.ffn.spec.intermediate_size)
            pm = b.post_mixer_norm
            kernels.gemv_few(b.ffn.gate_up.w_gate, z, w2=b.ffn.gate_up.w_up,
                             activation=b.ffn.spec.activation, h_in=cur, h_out=other, y=y_out,
                             w_post=pm.weight if pm is not None else None,
                             w_next=b.pre_ffn_norm.weight, eps_post=pm.eps if pm is not None else 0.0,
                             eps_next=b.pre_ffn_norm.eps, op="gate_up")
            cur, other = other, cur
            kernels.gemv_few(b.ffn.down.weight, y_down, x=z, op="down")
            pend = (y_down, b.post_ffn_norm)
        if pend is not None:                           # the last block's branch joins the stream
            post = pend[1]
            kernels.norm_residual(cur, pend[0], post.weight if post is not None else None, None, None,
                                  eps_post=post.eps if post is not None else 0.0)
        return cur

    def hidden_states(self, ctx) -> torch.Tensor:
        """The 32-bit stream [T, H] after the last block (before the final norm)."""
        spec = self.spec
        T = ctx.n_tokens
        h = ctx.new(T, spec.hidden_size, dtype=torch.float32)
        kernels.embed(ctx.tokens, self.embed_table, spec.embed_scale, h)
        if self.stream_position is not None:
            self.stream_position.forward(h, ctx)
        sched = spec.schedule
        if not sched:
            return h
        if self._few_tokens(ctx):
            return self._blocks_few_tokens(h, ctx)
        x = ctx.new(T, spec.hidden_size)
        self.blocks[sched[0].block].entry_norm.forward(h, x)
        for i, call in enumerate(sched):
            if ctx.cancel is not None and ctx.cancel.is_set():
                raise Cancelled(f"cancelled before block {i} of {len(sched)}")
            nxt = self.blocks[sched[i + 1].block].entry_norm if i + 1 < len(sched) else None
            x = self.blocks[call.block].forward(h, x, ctx, call.cache, call.writes_cache, nxt)
        return h

    def logits(self, h: torch.Tensor, rows: torch.Tensor, ctx,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """32-bit logits [len(rows), V] of the stream rows ``rows`` (int32)."""
        R = rows.numel()
        x = ctx.new(R, self.spec.hidden_size)
        self.final_norm.forward(h, x, rows=rows)
        if out is None:
            out = ctx.new(R, self.spec.vocab_size, dtype=torch.float32)
        return self.head(x, out=out)

    def greedy_tokens(self, h: torch.Tensor, rows: torch.Tensor, ctx,
                      out: torch.Tensor) -> bool:
        """out[r] = first index of the greatest logit of stream row rows[r], without the
        logits ever being written (the head product takes the arg max in its epilogue;
        the reference chooses in the same place, src/models/gemma3.zig:352-367).
        Returns False, having done nothing, where the head has no such kernel (32-bit
        weights, more rows than it takes): the caller then asks for ``logits``."""
        x = ctx.new(rows.numel(), self.spec.hidden_size)
        if not kernels.linear_argmax_supported(x, self.head.weight):
            return False
        self.final_norm.forward(h, x, rows=rows)
        kernels.linear_argmax(x, self.head.weight, out)
        return True

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        return self.logits(self.hidden_states(ctx), rows, ctx)

    def run_step(self, ctx, rows: Optional[torch.Tensor],
                 choose_into: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """A whole step: 32-bit logits [len(rows), V] of the stream rows ``rows`` (None:
        the step only fills the cache and nothing is returned); or, with ``choose_into``
        (int32, len(rows)), the index of each row's greatest logit goes there without the
        logits being written, where the head has that kernel (else the logits are
        returned and nothing is chosen).

        Models of standard blocks take the C++ host path (one call into the library for
        the whole step); others, and any step whose operations are being timed, run
        through the Python parts launch by launch."""
        n_rows = rows.numel() if rows is not None else 0
        if ctx.cancel is not None and ctx.cancel.is_set():
            raise Cancelled("cancelled before the step")
        greedy = (choose_into is not None and n_rows > 0 and self.dtype == torch.bfloat16 and
                  n_rows <= kernels.ARGMAX_MAX_ROWS and self.spec.hidden_size % 8 == 0 and
                  self.head.weight.data_ptr() % 16 == 0)
        if self.native is not None and kernels._perf is None and not kernels.NVTX:
            if n_rows == 0:
                self.native.run(ctx, None)
                return None
            if greedy:
                self.native.run(ctx, rows, argmax_out=choose_into)
                return None
            out = ctx.new(n_rows, self.spec.vocab_size, dtype=torch.float32)
            self.native.run(ctx, rows, logits=out)
            return out
        h = self.hidden_states(ctx)
        if n_rows == 0:
            return None
        if greedy and self.greedy_tokens(h, rows, ctx, choose_into):
            return None
        return self.logits(h, rows, ctx)
