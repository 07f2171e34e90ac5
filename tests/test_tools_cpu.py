"""The analysis tools that ship beside the benchmarks (no GPU needed)."""
import importlib.util
import json
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _load(name):
    spec = importlib.util.spec_from_file_location(name, ROOT / "benchmarks" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _k(name, ts, dur, cat="kernel", tid=7):
    return {"ph": "X", "cat": cat, "name": name, "ts": ts, "dur": dur, "pid": 0, "tid": tid}


def test_trace_analysis_separates_hidden_from_exposed_communication(tmp_path):
    at = _load("analyze_trace")
    events = [
        # compute stream: two of this package's GEMMs with a 500 us hole between them
        _k("void dmuon::gemm_tcgen05_pair_kernel<...>(KParams)", 1000.0, 400.0),
        _k("void dmuon::gemm_tcgen05_pair_kernel<...>(KParams)", 1900.0, 600.0),
        # communication stream: an NCCL kernel half behind the first GEMM, half in the hole ...
        _k("ncclDevKernel_Reduce_Sum_bf16_RING_LL(...)", 1200.0, 400.0, tid=9),
        # ... and a peer-to-peer copy fully behind the second GEMM
        _k("Memcpy PtoP (Device -> Device)", 2000.0, 100.0, cat="gpu_memcpy", tid=11),
        # a library GEMM and an attention kernel later on
        _k("nvjet_tst_128x256_64x4_2x1_v_bz_TNN", 2600.0, 50.0),
        _k("cudnn_generated_fort_native_sdpa_sm100_flash_fprop", 2650.0, 50.0),
        # host ranges: two layers of the same phase collapse into one line
        {"ph": "X", "cat": "user_annotation", "name": "dmuon.tp_gather.layers.0", "ts": 900.0, "dur": 30.0},
        {"ph": "X", "cat": "user_annotation", "name": "dmuon.tp_gather.layers.1", "ts": 950.0, "dur": 20.0},
        {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 900.0, "dur": 10.0},
    ]
    path = tmp_path / "t.json"
    path.write_text(json.dumps({"traceEvents": events}))
    s = at.analyze(at.load_events(path), gap_us=50.0)
    assert s["gpu_events"] == 6
    fam = s["families"]
    assert fam["own tcgen05 gemm"]["launches"] == 2 and abs(fam["own tcgen05 gemm"]["ms"] - 1.0) < 1e-9
    assert fam["nccl"]["launches"] == 1 and fam["peer copy (copy engines)"]["launches"] == 1
    assert fam["gemm (library)"]["launches"] == 1 and fam["attention (library)"]["launches"] == 1
    c = s["communication"]
    # NCCL 1200-1600: 1200-1400 behind the first GEMM, 1400-1600 exposed; the copy is fully hidden
    assert abs(c["ms"] - 0.5) < 1e-9 and abs(c["hidden_behind_compute_ms"] - 0.3) < 1e-9 and abs(c["exposed_ms"] - 0.2) < 1e-9
    # device idle: 1600-1900 (between the NCCL kernel and the second GEMM) and 2500-2600
    gaps = s["idle_gaps"]
    assert gaps["count"] == 2 and abs(gaps["longest"][0]["us"] - 300.0) < 1e-6
    assert gaps["longest"][0]["after_kernel"].startswith("ncclDevKernel") and "gemm_tcgen05" in gaps["longest"][0]["before_kernel"]
    assert s["ranges"] == {"dmuon.tp_gather.layers": {"count": 2, "host_ms": 0.05}}
    text = at.format_report(s)
    assert "own tcgen05 gemm" in text and "exposed" in text


def test_trace_analysis_without_gpu_events_still_lists_ranges():
    at = _load("analyze_trace")
    s = at.analyze([{"ph": "X", "cat": "user_annotation", "name": "dmuon.peer.publish_owned", "ts": 1.0, "dur": 2000.0}])
    assert s["gpu_events"] == 0 and s["ranges"]["dmuon.peer.publish_owned"]["count"] == 1
    assert "no GPU events" in at.format_report(s)


def test_ownership_benchmark_arms_follow_the_same_trajectory():
    """``benchmarks/bench_e2e.py`` on two gloo ranks: plain FSDP2 with every rank
    orthogonalising the all-gathered gradient (no ownership, nothing of this
    package's placement code) and dedicated ownership must reach the same loss --
    an end-to-end oracle that shares only the model and the Newton-Schulz function."""
    import socket
    import subprocess
    import sys

    with socket.socket() as sock:                     # a port nobody holds right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
        "--master-port", str(port), str(ROOT / "benchmarks" / "bench_e2e.py"), "--cpu", "--arms", "redundant,owned",
        "--layers", "2", "--width", "128", "--heads", "4", "--vocab", "512", "--batch", "2", "--seq", "64",
        "--steps", "3", "--warmup", "1",
    ]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    recs = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    arms = {r["arm"]: r for r in recs if "arm" in r}
    assert set(arms) == {"redundant", "owned"}
    assert abs(arms["redundant"]["loss"] - arms["owned"]["loss"]) < 2e-3, arms
    assert any(r.get("summary") and "owned_vs_redundant_speedup" in r for r in recs)
