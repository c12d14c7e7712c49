"""Per-step time breakdown of a training job from a kernel timeline.

Counterpart of ``tools/zuku-timeline.py:1-560`` (which reads an Nsight Systems database): here
the timeline comes from ``torch.profiler`` (CUPTI) - either live, through :func:`profile`, or
from a Chrome trace file it exported. Kernels are put into the classes

    Compute | NCCL AG | NCCL AR/RS | NCCL other | Fused comm | Reshard | Memcpy | CUDA idle | Pipeline idle

per device, joined to the enclosing task range (the runtime opens one named range per task
launch), and reported as "current" against a speed-of-light column that keeps only the compute
time. *CUDA idle* is the time without a running kernel inside task ranges (launch gaps, host
stalls); *Pipeline idle* is the time without a running kernel outside every task range (bubbles,
waiting for another stage).

    python -m multimesh_jax_b200.utils.timeline trace.json [--device 0] [--json]
"""
from __future__ import annotations

import argparse
import contextlib
import json
import re
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

CLASSES = ("Compute", "NCCL AG", "NCCL AR/RS", "NCCL other", "Fused comm", "Reshard", "Memcpy",
           "CUDA idle", "Pipeline idle")

_RULES: Sequence[Tuple[str, str]] = (
    (r"nccl.*AllGather", "NCCL AG"),
    (r"nccl.*(AllReduce|ReduceScatter)", "NCCL AR/RS"),
    (r"nccl", "NCCL other"),
    (r"reshard_pull|wait_flags_timeout|set_flags_kernel|wait_flag_kernel|set_flag_kernel", "Reshard"),
    (r"AllReduceHook|allreduce|gemm_ar|allgather_gemm|moe_route_dispatch|moe_dispatch|moe_combine|reduce_pull|fsdp_",
     "Fused comm"),
    (r"[Mm]emcpy|[Mm]emset", "Memcpy"),
)
TASK_PREFIX = "mm.task:"
RESHARD_PREFIX = "mm.reshard:"


def classify(kernel_name: str) -> str:
    for pat, cls in _RULES:
        if re.search(pat, kernel_name):
            return cls
    return "Compute"


@dataclass
class Span:
    name: str
    start: float   # microseconds
    dur: float
    device: int = 0
    kind: str = "kernel"   # "kernel" | "range"

    @property
    def end(self) -> float:
        return self.start + self.dur


@dataclass
class Breakdown:
    device: int
    wall_us: float
    classes: Dict[str, float] = field(default_factory=dict)
    per_task: Dict[str, Dict[str, float]] = field(default_factory=dict)
    top_kernels: List[Tuple[str, float, int]] = field(default_factory=list)
    # cross-stream ordering of the step: edges the runtime context enforced with an event wait
    # (from its dependence analysis) and the event calls the profiler saw on the host
    event_edges: List[dict] = field(default_factory=list)
    host_event_calls: Dict[str, int] = field(default_factory=dict)

    def speed_of_light_us(self) -> float:
        return self.classes.get("Compute", 0.0)

    def to_dict(self) -> dict:
        return {"device": self.device, "wall_us": round(self.wall_us, 1),
                "classes_us": {k: round(v, 1) for k, v in self.classes.items()},
                "classes_pct": {k: round(100.0 * v / self.wall_us, 2) if self.wall_us else 0.0
                                for k, v in self.classes.items()},
                "speed_of_light_us": round(self.speed_of_light_us(), 1),
                "per_task_us": {t: {k: round(v, 1) for k, v in c.items()} for t, c in self.per_task.items()},
                "top_kernels": [{"name": n[:96], "us": round(u, 1), "count": c} for n, u, c in self.top_kernels],
                "event_edges": self.edge_summary(), "host_event_calls": dict(self.host_event_calls)}

    STREAMS = ("compute", "communication", "auxiliary")

    def edge_summary(self) -> dict:
        """Event edges by (stream of the earlier task -> stream of the waiting task), with examples."""
        out: Dict[str, dict] = {}
        for e in self.event_edges:
            key = f"{self.STREAMS[e['from_stream']]}->{self.STREAMS[e['to_stream']]}"
            d = out.setdefault(key, {"count": 0, "examples": []})
            d["count"] += 1
            if len(d["examples"]) < 3:
                d["examples"].append(f"{e['from_name']} -> {e['to_name']}")
        return out

    def format(self) -> str:
        lines = [f"device {self.device}: wall {self.wall_us / 1e3:.2f} ms", f"{'class':<16}{'current ms':>12}{'%':>8}{'SoL ms':>10}"]
        for c in CLASSES:
            v = self.classes.get(c, 0.0)
            sol = v if c == "Compute" else 0.0
            lines.append(f"{c:<16}{v / 1e3:>12.3f}{100 * v / self.wall_us if self.wall_us else 0:>8.1f}{sol / 1e3:>10.3f}")
        if self.event_edges or self.host_event_calls:
            lines.append(f"event edges between streams: {len(self.event_edges)}  (host calls: "
                         + ", ".join(f"{k} x{v}" for k, v in sorted(self.host_event_calls.items())) + ")")
            for key, d in self.edge_summary().items():
                lines.append(f"  {key:<28} x{d['count']:<5} e.g. {d['examples'][0][:90]}")
        lines.append("top kernels:")
        for n, u, cnt in self.top_kernels:
            lines.append(f"  {u / 1e3:>10.3f} ms  x{cnt:<6} {n[:100]}")
        return "\n".join(lines)


def _merge(intervals: List[Tuple[float, float]]) -> List[Tuple[float, float]]:
    out: List[Tuple[float, float]] = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            out[-1] = (out[-1][0], max(out[-1][1], e))
        else:
            out.append((s, e))
    return out


def _overlap(a: List[Tuple[float, float]], b: List[Tuple[float, float]]) -> float:
    i = j = 0
    tot = 0.0
    while i < len(a) and j < len(b):
        lo, hi = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if hi > lo:
            tot += hi - lo
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return tot


def breakdown(spans: Iterable[Span], device: int = 0, window: Optional[Tuple[float, float]] = None,
              top: int = 12) -> Breakdown:
    """Classifies the kernels of ``device`` inside ``window`` (default: first kernel start to
    last kernel end). Overlapping kernels (several streams) are charged by priority: time in
    which a communication kernel runs alone counts as communication, time in which any compute
    kernel runs counts as compute (communication hidden under compute costs nothing)."""
    spans = [s for s in spans if s.device == device]
    kernels = [s for s in spans if s.kind == "kernel"]
    ranges = [s for s in spans if s.kind == "range"]
    if not kernels:
        return Breakdown(device, 0.0, {c: 0.0 for c in CLASSES})
    t0 = min(k.start for k in kernels) if window is None else window[0]
    t1 = max(k.end for k in kernels) if window is None else window[1]
    clip = lambda s, e: (max(s, t0), min(e, t1))
    by_class: Dict[str, List[Tuple[float, float]]] = {}
    agg: Dict[str, List[float]] = {}
    for k in kernels:
        s, e = clip(k.start, k.end)
        if e <= s:
            continue
        by_class.setdefault(classify(k.name), []).append((s, e))
        a = agg.setdefault(k.name, [0.0, 0])
        a[0] += e - s
        a[1] += 1
    merged = {c: _merge(v) for c, v in by_class.items()}
    classes = {c: 0.0 for c in CLASSES}
    covered: List[Tuple[float, float]] = []
    for c in ("Compute", "Fused comm", "Reshard", "NCCL AR/RS", "NCCL AG", "NCCL other", "Memcpy"):
        iv = merged.get(c, [])
        total = sum(e - s for s, e in iv)
        classes[c] = total - _overlap(iv, covered)
        covered = _merge(covered + iv)
    busy = sum(e - s for s, e in covered)
    wall = t1 - t0
    task_iv = _merge([clip(r.start, r.end) for r in ranges if r.name.startswith((TASK_PREFIX, RESHARD_PREFIX))
                      and min(r.end, t1) > max(r.start, t0)])
    in_task = sum(e - s for s, e in task_iv)
    busy_in_task = _overlap(covered, task_iv)
    if task_iv:
        classes["CUDA idle"] = max(0.0, in_task - busy_in_task)
        classes["Pipeline idle"] = max(0.0, (wall - in_task) - (busy - busy_in_task))
    else:
        classes["CUDA idle"] = max(0.0, wall - busy)
    per_task: Dict[str, Dict[str, float]] = {}
    for r in ranges:
        if not r.name.startswith(TASK_PREFIX):
            continue
        s, e = clip(r.start, r.end)
        if e <= s:
            continue
        d = per_task.setdefault(r.name[len(TASK_PREFIX):], {"range": 0.0, "count": 0})
        d["range"] += e - s
        d["count"] += 1
    top_k = sorted(((n, v[0], v[1]) for n, v in agg.items()), key=lambda x: -x[1])[:top]
    return Breakdown(device, wall, classes, per_task, top_k)


# ---------------------------------------------------------------------------- sources
def spans_from_chrome_trace(path: str) -> List[Span]:
    """Spans from a Chrome trace exported by ``torch.profiler`` (``export_chrome_trace``)."""
    with open(path) as f:
        doc = json.load(f)
    events = doc["traceEvents"] if isinstance(doc, dict) else doc
    out: List[Span] = []
    for e in events:
        if e.get("ph") != "X":
            continue
        cat = e.get("cat", "")
        args = e.get("args", {})
        if cat in ("kernel", "gpu_memcpy", "gpu_memset"):
            out.append(Span(e["name"], float(e["ts"]), float(e.get("dur", 0.0)), int(args.get("device", 0)), "kernel"))
        elif cat == "gpu_user_annotation" and e["name"].startswith((TASK_PREFIX, RESHARD_PREFIX)):
            out.append(Span(e["name"], float(e["ts"]), float(e.get("dur", 0.0)), int(args.get("device", e.get("pid", 0)) or 0),
                            "range"))
    return out


def spans_from_profiler(prof) -> List[Span]:
    """Spans from a finished ``torch.profiler.profile`` object."""
    out: List[Span] = []
    for ev in prof.events():
        dt = str(getattr(ev, "device_type", ""))
        if "CUDA" not in dt:
            continue
        name = ev.name
        dev = int(getattr(ev, "device_index", 0) or 0)
        tr = ev.time_range
        kind = "range" if name.startswith((TASK_PREFIX, RESHARD_PREFIX)) else "kernel"
        out.append(Span(name, float(tr.start), float(tr.end - tr.start), dev, kind))
    return out


def host_event_calls(prof) -> Dict[str, int]:
    """How often the profiled region called the CUDA event API on the host."""
    out: Dict[str, int] = {}
    for ev in prof.events():
        if ev.name in ("cudaStreamWaitEvent", "cudaEventRecord", "cudaEventRecordWithFlags", "cudaEventSynchronize",
                       "cudaStreamSynchronize", "cudaDeviceSynchronize"):
            out[ev.name] = out.get(ev.name, 0) + 1
    return out


@contextlib.contextmanager
def profile(result: dict, device: int = 0, context=None):
    """Runs the body under ``torch.profiler`` and stores the :class:`Breakdown` of ``device`` in
    ``result['breakdown']``. ``context``: the executable's runtime context; when it records
    cross-stream event edges (``CudaContext``) the edges of the profiled region are attached to
    the breakdown. Timings taken inside the body are perturbed by the profiler and must not be
    reported as benchmark values."""
    import torch
    from torch.profiler import ProfilerActivity, profile as _profile
    from .. import state
    old = state.knobs["task_ranges"]
    state.knobs["task_ranges"] = True
    if context is not None and hasattr(context, "edges"):
        context.clear_event_log()
    try:
        with _profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            yield
            if torch.cuda.is_available():
                torch.cuda.synchronize()
    finally:
        state.knobs["task_ranges"] = old
    result["breakdown"] = breakdown(spans_from_profiler(prof), device)
    result["breakdown"].host_event_calls = host_event_calls(prof)
    if context is not None and hasattr(context, "edges"):
        result["breakdown"].event_edges = list(context.edges())
    result["profiler"] = prof


def main(argv: Optional[Sequence[str]] = None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("trace")
    p.add_argument("--device", type=int, default=0)
    p.add_argument("--json", action="store_true")
    ns = p.parse_args(argv)
    b = breakdown(spans_from_chrome_trace(ns.trace), ns.device)
    print(json.dumps(b.to_dict()) if ns.json else b.format())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
