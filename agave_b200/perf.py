"""Per-operation timing of eager steps, after the reference's ``--profile``
(src/perf.zig:28-130: an operation enum, start/end around every call site, a
table of calls, total, average and share printed after generation).

The reference brackets host calls with wall-clock stamps and a device
synchronisation; here every kernel launcher is bracketed with two CUDA events
on the launching stream, so the numbers are device times and nothing is
synchronised until the report is made.  Each span also carries the bytes the
kernel has to move and the flops it has to do (from its shapes), so the report
gives each operation's share of the measured memory and tensor peaks.

Timing applies to steps that run launch by launch; a recorded step (a CUDA
graph) is one opaque launch, so the engine runs steps eagerly while a
``PerfCounters`` is active.  Dependent launch lets a kernel's prologue overlap
its predecessor's tail; with an event between them that overlap goes away, so
the sum over operations is somewhat above the time of an untimed eager step.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


NULL_SPAN = _Null()


class NvtxSpan:
    """An NVTX range around one launch: with ``AGAVE_B200_NVTX=1`` every operation is
    named on a profiler's timeline (steps then run launch by launch through the Python
    parts, also while a CUDA graph is recorded: a range is a host-side mark)."""
    __slots__ = ("op",)

    def __init__(self, op: str):
        self.op = op

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.op)
        return self

    def __exit__(self, *a):
        torch.cuda.nvtx.range_pop()
        return False


class _Span:
    __slots__ = ("owner", "op", "nbytes", "flops", "e0")

    def __init__(self, owner, op, nbytes, flops):
        self.owner, self.op, self.nbytes, self.flops = owner, op, nbytes, flops

    def __enter__(self):
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e0.record()
        return self

    def __exit__(self, *a):
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record()
        self.owner.records.append((self.op, self.e0, e1, self.nbytes, self.flops))
        return False


class PerfCounters:
    """Collects (operation, device time, bytes, flops) for every kernel launched
    while it is active (``with counters:``)."""

    def __init__(self):
        self.records: List[Tuple] = []
        self.n_tokens = 0
        self._role: Optional[str] = None

    def span(self, op: str, nbytes: int = 0, flops: int = 0) -> _Span:
        return _Span(self, op, int(nbytes), int(flops))

    def __enter__(self):
        from . import kernels
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("operations cannot be timed while a CUDA graph is recorded")
        self._prev = kernels._perf
        kernels._perf = self
        return self

    def __exit__(self, *a):
        from . import kernels
        kernels._perf = self._prev
        return False

    # ---------------------------------------------------------------- report
    def table(self) -> "OrderedDict[str, Dict[str, float]]":
        """{operation: calls, total_us, bytes, flops}, in order of first use."""
        torch.cuda.synchronize()
        out: "OrderedDict[str, Dict[str, float]]" = OrderedDict()
        for op, e0, e1, nbytes, flops in self.records:
            row = out.setdefault(op, dict(calls=0, total_us=0.0, bytes=0, flops=0))
            row["calls"] += 1
            row["total_us"] += e0.elapsed_time(e1) * 1e3
            row["bytes"] += nbytes
            row["flops"] += flops
        return out

    def report(self, hbm_gbs: float = 0.0, tflops: float = 0.0, title: str = "") -> str:
        """The table as text.  With the measured peaks given, each row also shows its
        achieved GB/s and TFLOP/s and the larger of the two as a share of its peak."""
        rows = self.table()
        total = sum(r["total_us"] for r in rows.values()) or 1.0
        head = f"── Profile {title}({self.n_tokens} tokens, {total / 1e3:.2f} ms in kernels) ──"
        lines = [head, f"{'Operation':<18} {'Calls':>6} {'Total(ms)':>10} {'Avg(us)':>9} {'%':>6} "
                       f"{'GB/s':>8} {'TFLOP/s':>8} {'of peak':>8}", "─" * 80]
        for op, r in rows.items():
            sec = r["total_us"] * 1e-6
            gbs = r["bytes"] / sec / 1e9 if sec > 0 else 0.0
            tf = r["flops"] / sec / 1e12 if sec > 0 else 0.0
            frac = max(gbs / hbm_gbs if hbm_gbs else 0.0, tf / tflops if tflops else 0.0)
            lines.append(f"{op:<18} {r['calls']:>6d} {r['total_us'] / 1e3:>10.3f} "
                         f"{r['total_us'] / r['calls']:>9.1f} {100 * r['total_us'] / total:>5.1f}% "
                         f"{gbs:>8.0f} {tf:>8.1f} {frac:>8.2f}")
        lines += ["─" * 80, f"{'TOTAL':<18} {'':>6} {total / 1e3:>10.3f}"]
        return "\n".join(lines)
