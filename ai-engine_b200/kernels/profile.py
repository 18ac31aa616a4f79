"""Opt-in timers around the kernels, by class of kernel.

The reference's profile run prints wall-clock per decode step
(crates/ai-engine-runtime/examples/profile_decode.rs:97-127) and its binary traces
spans (crates/ai-engine/src/lib.rs:11-30).  Here every launcher of `kernels.ops` sits
in a `region(cls, bytes, flops)`: when profiling is on, a pair of CUDA events on
the launching stream times it and an NVTX range of the same name is pushed for
external tools; when it is off (the default) a region costs one attribute test.
Times are taken eagerly, kernel by kernel (no CUDA graphs, no overlap of one
kernel's start with the previous one's end), so the shares compare and the sum
exceeds what the same step takes when it is replayed from a graph.

    from ai_engine_b200.kernels import profile
    profile.start(); ...steps...; rows = profile.stop(hbm_gbs, tflops)
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Dict, List

import torch

_ON = [False]
_RECORDS: List[tuple] = []        # (class, start event, end event, bytes, flops)


def enabled() -> bool:
    return _ON[0]


def start() -> None:
    """Begin recording (also turns CUDA-graph replay off for runners built afterwards: see
    engine.step.StepRunner)."""
    _RECORDS.clear()
    _ON[0] = True


@contextmanager
def _timed(cls: str, nbytes: float, flops: float):
    torch.cuda.nvtx.range_push(cls)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    try:
        yield
    finally:
        b.record()
        torch.cuda.nvtx.range_pop()
        _RECORDS.append((cls, a, b, float(nbytes), float(flops)))


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


_NULL = _Null()


def region(cls: str, nbytes: float = 0.0, flops: float = 0.0):
    """Context manager around one launch: `cls` is the kernel class, `nbytes` the bytes it has to
    move (operands read once + results written), `flops` its floating-point operations."""
    if not _ON[0]:
        return _NULL
    return _timed(cls, nbytes, flops)


def stop(hbm_gbs: float, tflops: float) -> List[Dict[str, object]]:
    """End recording; one row per class, by time: calls, ms, GB moved, GFLOP, achieved GB/s and
    TFLOP/s, and `frac` = the larger of (bytes / hbm_gbs) and (flops / tflops), over the time."""
    _ON[0] = False
    torch.cuda.synchronize()
    agg: Dict[str, list] = {}
    for cls, a, b, nb, fl in _RECORDS:
        r = agg.setdefault(cls, [0, 0.0, 0.0, 0.0])
        r[0] += 1
        r[1] += a.elapsed_time(b)
        r[2] += nb
        r[3] += fl
    _RECORDS.clear()
    total = sum(r[1] for r in agg.values()) or 1.0
    rows = []
    for cls, (n, ms, nb, fl) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        s = ms * 1e-3
        ideal = max(nb / (hbm_gbs * 1e9), fl / (tflops * 1e12))
        rows.append(dict(kernel=cls, calls=n, ms=round(ms, 4), share=round(ms / total, 4),
                         gb=round(nb / 1e9, 4), gflop=round(fl / 1e9, 2),
                         gb_s=round(nb / s / 1e9, 1) if s else 0.0,
                         tflop_s=round(fl / s / 1e12, 2) if s else 0.0,
                         frac=round(ideal / s, 4) if s else 0.0))
    return rows


def table(rows: List[Dict[str, object]]) -> str:
    head = f"{'kernel class':<28}{'calls':>7}{'ms':>10}{'share':>8}{'GB':>9}{'GFLOP':>11}{'GB/s':>9}{'TFLOP/s':>9}{'frac':>7}"
    lines = [head, "-" * len(head)]
    for r in rows:
        lines.append(f"{r['kernel']:<28}{r['calls']:>7}{r['ms']:>10.3f}{r['share']:>8.3f}{r['gb']:>9.3f}"
                     f"{r['gflop']:>11.1f}{r['gb_s']:>9.0f}{r['tflop_s']:>9.1f}{r['frac']:>7.3f}")
    return "\n".join(lines)
