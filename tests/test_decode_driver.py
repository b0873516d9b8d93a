"""Host-side pieces of the vLLM decode driver and of the benchmark's tensor-parallel sharding (no GPU)."""
import importlib.metadata as metadata
import importlib.util
import json
import os
import sys
from pathlib import Path

import pytest

vllm = pytest.importorskip("vllm")
from hygemm_vllm import decode  # noqa: E402

ROOT = Path(__file__).resolve().parent.parent


def test_model_directory_carries_the_selection_rule(tmp_path):
    folder = decode.write_model_dir(tmp_path / "m", "qwen2.5-7b", layers=2)
    config = json.loads((folder / "config.json").read_text())
    assert (config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]) == (3584, 18944, 2)
    assert config["quantization_config"] == {"quant_method": "hygemm",
                                             "selection": {"rule": "l2norm", "fraction": 0.1, "multiple": 128}}
    dense = json.loads((decode.write_model_dir(tmp_path / "d", "mistral-7b", dense=True) / "config.json").read_text())
    assert "quantization_config" not in dense and dense["num_key_value_heads"] == 8


def test_engine_arguments_follow_the_decode_protocol(tmp_path):
    kw = decode.engine_arguments(tmp_path, [16, 1, 128], prompt=128, steps=128, dense=False, tp=2)
    assert kw["quantization"] == "hygemm" and kw["load_format"] == "dummy" and kw["tensor_parallel_size"] == 2
    assert kw["max_num_seqs"] == 128 and kw["max_model_len"] >= 256 and not kw["enable_prefix_caching"]
    cc = kw["compilation_config"]
    assert cc["mode"] == 0 and cc["cudagraph_mode"] == "FULL" and cc["cudagraph_capture_sizes"] == [1, 16, 128]
    assert cc["cudagraph_num_of_warmups"] >= 1                 # GEMM handles are created in the eager warm-up
    assert kw["worker_extension_cls"] == "hygemm_vllm.worker.AuditWorkerExtension"
    assert decode.engine_arguments(tmp_path, [1], 8, 8, dense=True)["quantization"] is None


def test_plugin_entry_point_is_published_for_worker_processes(monkeypatch):
    monkeypatch.setenv("PYTHONPATH", "")
    before = list(sys.path)
    try:
        decode.ensure_plugin_entry_point()
        names = {ep.name: ep.value for ep in metadata.entry_points(group="vllm.general_plugins")}
        assert names["hygemm_quantization"] == "hygemm_vllm:register"
        first = os.environ["PYTHONPATH"].split(os.pathsep)
        assert any((Path(p) / "hygemm_vllm").is_dir() for p in first) and any(Path(p).name.startswith("hygemm_plugin_") for p in first)
        decode.ensure_plugin_entry_point()                      # idempotent
        assert os.environ["PYTHONPATH"].split(os.pathsep) == first
    finally:
        sys.path[:] = before


def test_benchmark_shards_cover_the_layer_at_every_world_size():
    spec = importlib.util.spec_from_file_location("bench_module_cpu", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(bench)
    finally:
        sys.argv = argv
    for world in (2, 4, 8):
        for k in (3584, 18944):
            pieces = [bench.k_block_shard(k, r, world) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == k
            assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
            assert all((e - b) % 128 == 0 and e > b for b, e in pieces)
            assert max(e - b for b, e in pieces) - min(e - b for b, e in pieces) <= 128


def test_cell_summary_follows_the_reference_protocol(tmp_path):
    """Median of the samples, population coefficient of variation, tokens/s = batch * 1000 / median ms
    (integrations/vllm/formal/benchmark.py:84-89 of the reference), and the markdown row of a cell."""
    samples = [{"decode_ms_per_step": t, "steps": 127, "graph_steps": 127, "sum_step_gpu_ms": 100.0 * t,
                "context_min": 128, "context_max": 255} for t in (2.0, 2.2, 2.1, 2.05, 2.15)]
    cell = decode.summarise(samples, 16)
    assert cell["median_ms_per_step"] == 2.1 and abs(cell["decode_tokens_per_s"] - 16000 / 2.1) < 1e-9
    import statistics
    assert abs(cell["cv"] - statistics.pstdev([2.0, 2.2, 2.1, 2.05, 2.15]) / 2.1) < 1e-12 and cell["cv"] < 0.05
    assert cell["context"] == [128, 255] and cell["steps"] == 127
    row = dict(cell, arch="qwen2.5-7b", dense=False, tp=1, batch=16, prompt=128, attempts=1)
    table = tmp_path / "t.md"
    decode.append_table(table, [row], " + fused SwiGLU producer")
    decode.append_table(table, [dict(row, dense=True)])
    lines = table.read_text().splitlines()
    assert lines[0].startswith("| arch | linears") and len(lines) == 4
    assert "hybrid + fused SwiGLU producer" in lines[2] and "dense bf16" in lines[3] and "127/127" in lines[2]
