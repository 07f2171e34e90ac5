"""The parts of ``bench.py`` that need no GPU: argument defaults of the driver's
contract, model dimensions, the MFU and AdamW-table arithmetic, data-plane
naming and the parsing of the clock samples."""
import importlib.util
import json
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("_bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_default_arguments_follow_the_contract(bench, monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = bench.parse_args()
    assert (a.gpus, a.impl, a.model, a.optimizer, a.parallelism) == (1, "ours", "llama3-8b", "muon", "fsdp")
    assert a.steps >= 1 and a.warmup >= 3
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "8", "--steps", "20", "--warmup", "5"])
    a = bench.parse_args()
    assert (a.impl, a.gpus, a.steps, a.warmup) == ("reference", 8, 20, 5)


def test_model_dimensions_of_the_headline_configuration(bench):
    d = bench.model_dims(SimpleNamespace(model="llama3-8b", seq=0, micro_batch=0))
    assert (d["d_model"], d["n_layers"], d["n_heads"], d["n_kv_heads"], d["head_dim"], d["ffn_hidden"]) == (4096, 32, 32, 8, 128, 14336)
    assert (d["vocab_size"], d["seq"], d["mb"]) == (128256, 8192, 1)
    d = bench.model_dims(SimpleNamespace(model="llama3-8b", seq=1024, micro_batch=4))
    assert (d["seq"], d["mb"]) == (1024, 4)


def test_mfu_counts_six_flops_per_parameter_and_token_plus_causal_attention(bench):
    args = SimpleNamespace(model="llama3-8b")
    dims = bench.model_dims(SimpleNamespace(model="llama3-8b", seq=0, micro_batch=0))
    per_layer = 4096 * 4096 * 2 + 2 * 4096 * 1024 + 3 * 4096 * 14336
    params = 32 * per_layer + 128256 * 4096
    attn = 6 * 32 * 4096 * 8192
    tokens = 8192
    want = tokens * (6 * params + attn) / 0.5 / (1 * 2250e12)
    assert abs(bench.mfu(args, dims, tokens, 500.0, 1) - round(want, 4)) < 1e-4
    assert bench.mfu(SimpleNamespace(model="pi0"), dims, tokens, 500.0, 1) is None


def test_adamw_table_lookup_is_keyed_by_model_implementation_placement_and_ranks(bench):
    table = json.load(open(ROOT / "baseline" / "adamw_step_ms.json"))
    key = "llama3-8b|own|fsdp|1"
    assert key in table and table[key]["ms"] > 0
    args = SimpleNamespace(model="llama3-8b", impl="ours", model_impl="own", parallelism="fsdp")
    assert bench.adamw_step_ms(args, 1) == float(table[key]["ms"])
    assert bench.adamw_step_ms(args, 3) is None                                   # a cell nobody measured
    args.impl = "reference"
    assert bench.adamw_step_ms(args, 1) == (float(table["llama3-8b|hf|fsdp|1"]["ms"]) if "llama3-8b|hf|fsdp|1" in table else None)


def test_data_plane_names(bench):
    assert bench._plane_name(None) == "nccl"
    assert bench._plane_name(SimpleNamespace(peer_runtime=None, tp_exchanges={})) == "nccl"
    assert "tensor-parallel shards read in place" in bench._plane_name(SimpleNamespace(peer_runtime=None, tp_exchanges={1: object()}))
    rt = SimpleNamespace(reduce_via="ce", publish_via="ce", copy_mode="ce", nvls_publish="lane")
    name = bench._plane_name(SimpleNamespace(peer_runtime=rt))
    assert name.startswith("peer memory [ce]") and "copy engines" in name
    rt = SimpleNamespace(reduce_via="nvls", publish_via="nvls", copy_mode="nvls", nvls_publish="epilogue")
    name = bench._plane_name(SimpleNamespace(peer_runtime=rt))
    assert "multimem.st" in name and "multimem.ld_reduce" in name and "epilogue" in name


def test_clock_samples_are_summarised_under_load_only(bench, tmp_path):
    s = bench.ClockSampler(enabled=True)
    s.path = str(tmp_path / "clocks.csv")
    Path(s.path).write_text(
        "0, 345, 1965, 120.5, 0x0, Not Active, Not Active, Not Active, Not Active\n"      # idle sample: ignored
        "0, 1400, 1965, 990.1, 0x4, Not Active, Not Active, Not Active, Active\n"
        "0, 1300, 1965, 1001.7, 0x4, Not Active, Not Active, Not Active, Active\n"
        "0, 1500, 1965, 985.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"
        "garbage line\n"
    )

    class _Proc:
        def terminate(self): pass
        def wait(self, timeout=None): return 0
        def kill(self): pass

    s.proc = _Proc()
    out = s.stop()
    assert out["sm_mhz"] == 1400 and out["sm_max_mhz"] == 1965 and out["samples_under_load"] == 3
    assert out["reasons"] == ["sw_power_cap"]
    assert bench.ClockSampler(enabled=False).stop()["reasons"] == ["unsampled"]
