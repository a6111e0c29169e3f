"""How much of a training step the GPU spends idle between kernels (is the host the limit?).

A step is a few thousand kernel launches.  If the host cannot enqueue them as fast as the device retires them,
the device timeline shows gaps between consecutive kernels; if the launch queue stays ahead, it does not.  This
module records the device timeline of a few steps with ``torch.profiler`` (CUPTI activity records: start and end
of every kernel and copy on every stream of this process's GPU), merges the intervals of all streams and reports
the busy time, the idle time and the largest gaps.

The recording itself makes every launch a little more expensive on the host, so the idle share it reports is an
UPPER bound; step times are never taken from a profiled run.
"""
from __future__ import annotations

import torch


def merge_intervals(intervals: list[tuple[float, float]]) -> list[tuple[float, float]]:
    """Union of possibly overlapping [start, end) intervals, sorted."""
    out: list[list[float]] = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            if e > out[-1][1]:
                out[-1][1] = e
        else:
            out.append([s, e])
    return [(a, b) for a, b in out]


def summarize(intervals: list[tuple[float, float]], steps: int, gap_floor_us: float = 2.0) -> dict:
    """``intervals`` in microseconds -> per-step busy / idle milliseconds and gap statistics.

    The trace begins with a start-up gap that steady-state training does not have (the first traced step starts
    with an empty launch queue: the device waits while the host prepares the step, and in a multi-rank run also for
    the slowest rank's tracer).  A gap in the first 15 % of the timeline that is larger than a millisecond is
    therefore reported on its own (``startup_gap_ms``) and left out of the idle time."""
    merged = merge_intervals(intervals)
    if not merged:
        return {"kernels": 0}
    t0, t1 = merged[0][0], merged[-1][1]
    gaps = [(merged[i + 1][0] - merged[i][1], merged[i][1]) for i in range(len(merged) - 1)]
    startup = 0.0
    early = [(g, at) for g, at in gaps if at - t0 < 0.15 * (t1 - t0) and g > 1000.0]
    if early:
        startup = max(g for g, _ in early)
    span = (t1 - t0) - startup
    busy = sum(b - a for a, b in merged)
    big = sorted((g for g, _ in gaps if g > gap_floor_us and g != startup), reverse=True)
    return {"kernels": len(intervals), "steps": steps,
            "span_ms_per_step": span / 1e3 / steps, "busy_ms_per_step": busy / 1e3 / steps,
            "idle_ms_per_step": (span - busy) / 1e3 / steps, "idle_share": (span - busy) / span if span else 0.0,
            "startup_gap_ms": startup / 1e3,
            "gaps_over_floor_per_step": len(big) / steps, "gap_floor_us": gap_floor_us,
            "largest_gaps_us": [round(g, 1) for g in big[:5]]}


def short_name(name: str) -> str:
    """Kernel name without its return type, namespaces' template arguments and parameter list."""
    name = name.replace("(anonymous namespace)::", "").split("(")[0]
    if name.startswith("void "):
        name = name[5:]
    depth, out = 0, []
    for ch in name:                   # drop everything inside <...>
        if ch == "<":
            depth += 1
        elif ch == ">":
            depth -= 1
        elif depth == 0:
            out.append(ch)
    return "".join(out).strip()[:80]


def measure(step_fn, steps: int = 2, ready=None, top_kernels: int = 16) -> dict:
    """Run ``step_fn()`` ``steps`` times under a CUDA activity trace and summarise the device timeline.

    ``ready`` is called once the trace is recording and before the first step: in a multi-rank run pass a barrier,
    so that the ranks that are not traced do not start (and wait in bounded device-side waits) while this rank is
    still bringing the tracer up."""
    from torch.autograd import DeviceType
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        if ready is not None:
            ready()
        for _ in range(steps):
            step_fn()
        torch.cuda.synchronize()
    iv = []
    by_name: dict[str, list[float]] = {}
    for e in prof.events():
        if e.device_type == DeviceType.CUDA:
            r = e.time_range
            iv.append((float(r.start), float(r.end)))
            acc = by_name.setdefault(short_name(e.name), [0.0, 0.0])
            acc[0] += 1
            acc[1] += float(r.end) - float(r.start)
    out = summarize(iv, steps)
    top = sorted(by_name.items(), key=lambda kv: -kv[1][1])[:top_kernels]
    out["top_kernels"] = [{"kernel": k, "launches_per_step": round(v[0] / steps, 1),
                           "ms_per_step": round(v[1] / 1e3 / steps, 3)} for k, v in top]
    out["note"] = ("device timeline of this rank recorded with CUPTI activity tracing in a phase of its own after all "
                   "timed regions; tracing slows the host's launches, so the idle share is an upper bound")
    return out
