"""What a training step's GPU timeline is made of, from a torch-profiler Chrome trace.

Reads the JSON that ``benchmarks/profile_step.py`` (or any ``torch.profiler``
export) writes and reports, for the GPU events of one rank:

* device time per kernel family -- this package's tcgen05 GEMMs, its peer-memory
  and tensor-parallel kernels, its multi-tensor and model kernels, NCCL, library
  GEMMs, attention, copies -- with launch counts;
* how much of the communication (NCCL kernels, peer copies, this package's peer
  kernels) ran WHILE a compute kernel was running on another stream, and how much
  was exposed;
* idle gaps of the device (no kernel on any stream) above a threshold, the
  longest ones with the kernels on either side: the places where launch latency or
  a host synchronisation shows;
* the ``dmuon.*`` ``record_function`` ranges (host side) with count and total.

It runs no GPU code and imports neither torch nor this package, so a trace taken
on a training host can be analysed anywhere:

    python benchmarks/analyze_trace.py rank0.trace.json --gap-us 200 --json-out summary.json

(The reference ships ``benchmarks/analyze_tp_trace.py`` for its TP benchmark; this
tool answers the same question -- is the communication hidden, and where are the
bubbles -- for every placement.)
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from pathlib import Path
from typing import Any, Iterable

GPU_CATEGORIES = ("kernel", "gpu_memcpy", "gpu_memset")

#: (family, substrings of the lower-cased kernel name); first match wins
FAMILIES: tuple[tuple[str, tuple[str, ...]], ...] = (
    ("own tcgen05 gemm", ("gemm_tcgen05", "pull_linear_kernel")),
    ("own peer / tp kernels", ("peer_prologue", "peer_pull", "multicast_copy", "signal_peers", "wait_flags", "tp_gather_prologue",
                               "tp_apply_delta", "scalar_allreduce", "peer_")),
    ("own multi-tensor kernels", ("prologue_kernel", "adamw_kernel", "cast_kernel", "clip_sumsq", "clip_scale", "norm_scales",
                                  "multi_tensor")),
    ("own model kernels", ("swiglu", "geglu", "rope_", "rotary", "xent", "cross_entropy_kernel")),
    ("nccl", ("nccl",)),
    ("attention (library)", ("fmha", "flash", "attention", "sdpa", "cudnn_generated")),
    ("gemm (library)", ("gemm", "cutlass", "cublas", "nvjet", "xmma", "sm100_", "sm90_")),
    ("copy", ("memcpy", "memset")),
    ("elementwise / reduce (torch)", ("elementwise", "reduce_kernel", "vectorized", "cat", "index", "fill")),
)

COMM_FAMILIES = ("nccl", "own peer / tp kernels")


def load_events(path: Path) -> list[dict[str, Any]]:
    payload = json.loads(Path(path).read_text())
    return list(payload.get("traceEvents", [])) if isinstance(payload, dict) else list(payload)


def family_of(event: dict[str, Any]) -> str:
    name = str(event.get("name", "")).lower()
    cat = event.get("cat")
    if cat in ("gpu_memcpy", "gpu_memset"):
        # peer-to-peer copies are communication, everything else is a local copy
        return "peer copy (copy engines)" if ("ptop" in name or "peer" in name) else "copy"
    for fam, keys in FAMILIES:
        if any(k in name for k in keys):
            return fam
    return "other"


def _gpu_events(events: Iterable[dict[str, Any]]) -> list[dict[str, Any]]:
    out = []
    for e in events:
        if e.get("ph") == "X" and e.get("cat") in GPU_CATEGORIES and float(e.get("dur", 0.0)) >= 0.0:
            out.append(e)
    out.sort(key=lambda e: float(e["ts"]))
    return out


def _union(intervals: list[tuple[float, float]]) -> list[tuple[float, float]]:
    merged: list[tuple[float, float]] = []
    for lo, hi in sorted(intervals):
        if merged and lo <= merged[-1][1]:
            if hi > merged[-1][1]:
                merged[-1] = (merged[-1][0], hi)
        else:
            merged.append((lo, hi))
    return merged


def _overlap(a: list[tuple[float, float]], b: list[tuple[float, float]]) -> float:
    """Total length of the intersection of two sorted disjoint interval lists."""
    i = j = 0
    total = 0.0
    while i < len(a) and j < len(b):
        lo, hi = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if hi > lo:
            total += hi - lo
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return total


def _ranges(events: list[dict[str, Any]]) -> dict[str, dict[str, Any]]:
    ranges: dict[str, dict[str, float]] = defaultdict(lambda: {"us": 0.0, "count": 0})
    for e in events:
        name = str(e.get("name", ""))
        if e.get("ph") == "X" and name.startswith("dmuon.") and e.get("cat") not in GPU_CATEGORIES:
            # collapse per-layer suffixes ("dmuon.tp_gather.layers.3" -> "dmuon.tp_gather")
            key = ".".join(name.split(".")[:3]) if name.count(".") > 2 else name
            ranges[key]["us"] += float(e.get("dur", 0.0))
            ranges[key]["count"] += 1
    return {
        k: {"count": int(v["count"]), "host_ms": round(v["us"] / 1e3, 3)}
        for k, v in sorted(ranges.items(), key=lambda kv: -kv[1]["us"])
    }


def analyze(events: list[dict[str, Any]], gap_us: float = 200.0, top_gaps: int = 10) -> dict[str, Any]:
    gpu = _gpu_events(events)
    if not gpu:
        return {"gpu_events": 0, "ranges": _ranges(events)}
    t0 = min(float(e["ts"]) for e in gpu)
    t1 = max(float(e["ts"]) + float(e.get("dur", 0.0)) for e in gpu)

    per_family: dict[str, dict[str, float]] = defaultdict(lambda: {"us": 0.0, "launches": 0})
    per_kernel: dict[str, dict[str, float]] = defaultdict(lambda: {"us": 0.0, "launches": 0})
    comm_iv: list[tuple[float, float]] = []
    compute_iv: list[tuple[float, float]] = []
    all_iv: list[tuple[float, float, str]] = []
    for e in gpu:
        fam = family_of(e)
        lo = float(e["ts"])
        hi = lo + float(e.get("dur", 0.0))
        per_family[fam]["us"] += hi - lo
        per_family[fam]["launches"] += 1
        short = str(e.get("name", ""))[:96]
        per_kernel[short]["us"] += hi - lo
        per_kernel[short]["launches"] += 1
        is_comm = fam in COMM_FAMILIES or fam == "peer copy (copy engines)"
        (comm_iv if is_comm else compute_iv).append((lo, hi))
        all_iv.append((lo, hi, short))

    comm_u, compute_u = _union(comm_iv), _union(compute_iv)
    busy_u = _union([(lo, hi) for lo, hi, _ in all_iv])
    comm_total = sum(hi - lo for lo, hi in comm_u)
    hidden = _overlap(comm_u, compute_u)
    busy = sum(hi - lo for lo, hi in busy_u)

    # idle gaps of the whole device, with the kernels that end / start them
    gaps = []
    ends = sorted(all_iv, key=lambda t: t[1])
    starts = sorted(all_iv, key=lambda t: t[0])
    for (lo_a, hi_a), (lo_b, _hi_b) in zip(busy_u, busy_u[1:]):
        width = lo_b - hi_a
        if width >= gap_us:
            before = next((n for lo, hi, n in reversed(ends) if abs(hi - hi_a) < 1e-3), "?")
            after = next((n for lo, hi, n in starts if abs(lo - lo_b) < 1e-3), "?")
            gaps.append({"at_us": round(hi_a - t0, 1), "us": round(width, 1), "after_kernel": before, "before_kernel": after})
    gaps.sort(key=lambda g: -g["us"])

    span = t1 - t0
    return {
        "gpu_events": len(gpu),
        "span_ms": round(span / 1e3, 3),
        "device_busy_ms": round(busy / 1e3, 3),
        "device_busy_fraction": round(busy / span, 4) if span > 0 else None,
        "families": {
            k: {"ms": round(v["us"] / 1e3, 3), "launches": int(v["launches"]),
                "share_of_busy": round(v["us"] / busy, 4) if busy > 0 else None}
            for k, v in sorted(per_family.items(), key=lambda kv: -kv[1]["us"])
        },
        "top_kernels": [
            {"name": k, "ms": round(v["us"] / 1e3, 3), "launches": int(v["launches"])}
            for k, v in sorted(per_kernel.items(), key=lambda kv: -kv[1]["us"])[:15]
        ],
        "communication": {
            "ms": round(comm_total / 1e3, 3),
            "hidden_behind_compute_ms": round(hidden / 1e3, 3),
            "exposed_ms": round((comm_total - hidden) / 1e3, 3),
            "hidden_fraction": round(hidden / comm_total, 4) if comm_total > 0 else None,
        },
        "idle_gaps": {
            "threshold_us": gap_us,
            "count": len(gaps),
            "total_ms": round(sum(g["us"] for g in gaps) / 1e3, 3),
            "longest": gaps[:top_gaps],
        },
        "ranges": _ranges(events),
    }


def _format_ranges(s: dict[str, Any]) -> list[str]:
    if not s.get("ranges"):
        return []
    lines = ["", f"{'range':44s} {'count':>7s} {'host ms':>10s}"]
    for k, v in s["ranges"].items():
        lines.append(f"{k:44s} {v['count']:7d} {v['host_ms']:10.3f}")
    return lines


def format_report(s: dict[str, Any]) -> str:
    if not s.get("gpu_events"):
        return "\n".join(["no GPU events in this trace"] + _format_ranges(s)) + "\n"
    lines = [
        f"GPU events {s['gpu_events']}, span {s['span_ms']} ms, device busy {s['device_busy_ms']} ms "
        f"({100 * s['device_busy_fraction']:.1f} %)",
        "",
        f"{'kernel family':34s} {'ms':>10s} {'launches':>9s} {'of busy':>8s}",
    ]
    for k, v in s["families"].items():
        lines.append(f"{k:34s} {v['ms']:10.3f} {v['launches']:9d} {100 * (v['share_of_busy'] or 0):7.1f}%")
    c = s["communication"]
    lines += [
        "",
        f"communication {c['ms']} ms: {c['hidden_behind_compute_ms']} ms behind compute on another stream, "
        f"{c['exposed_ms']} ms exposed" + (f" ({100 * c['hidden_fraction']:.1f} % hidden)" if c["hidden_fraction"] is not None else ""),
        f"idle gaps >= {s['idle_gaps']['threshold_us']} us: {s['idle_gaps']['count']}, {s['idle_gaps']['total_ms']} ms in total",
    ]
    for g in s["idle_gaps"]["longest"]:
        lines.append(f"  +{g['at_us'] / 1e3:9.3f} ms  {g['us']:9.1f} us   {g['after_kernel'][:40]}  ->  {g['before_kernel'][:40]}")
    lines += _format_ranges(s)
    return "\n".join(lines) + "\n"


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("trace", type=Path)
    ap.add_argument("--gap-us", type=float, default=200.0, help="report device-idle gaps of at least this many microseconds")
    ap.add_argument("--top-gaps", type=int, default=10)
    ap.add_argument("--json-out", type=Path, default=None)
    args = ap.parse_args()
    summary = analyze(load_events(args.trace), args.gap_us, args.top_gaps)
    print(format_report(summary), end="")
    if args.json_out is not None:
        args.json_out.write_text(json.dumps(summary, indent=2) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
