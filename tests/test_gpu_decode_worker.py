"""The decode driver and the worker extension on a GPU: a two-layer random-init Qwen2.5-7B-shaped model served by
the installed vLLM with the `hygemm` method, FULL CUDA graphs, pure decode steps timed by `formal_begin` /
`formal_end` (integrations/vllm/hygemm_vllm/worker.py:6-73 and formal/benchmark.py:76-91 of the reference).
Runs in a child process: an engine wants a process of its own."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_two_layer_model_decodes_under_full_graphs_with_every_linear_hybrid():
    pytest.importorskip("vllm")
    env = dict(os.environ, HYGEMM_FUSE_SILU="1", VLLM_LOGGING_LEVEL="WARNING")
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT / "comp2029-hybridgemm_b200"), env.get("PYTHONPATH", "")])
    done = subprocess.run([sys.executable, "-m", "hygemm_vllm.decode", "--layers", "2", "--batch", "1,4", "--prompt", "16",
                           "--steps", "24", "--samples", "2"], env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    rows = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    cells = [r for r in rows if "batch" in r]
    audit = [r for r in rows if "audit_layers" in r]
    assert [c["batch"] for c in cells] == [1, 4]
    for c in cells:
        assert c["steps"] >= 16 and c["graph_steps"] == c["steps"]          # every timed step was a FULL graph
        assert c["decode_tokens_per_s"] > 0 and c["context"][0] >= 16
    assert audit and audit[0]["audit_layers"] == 8                           # 2 layers x (qkv, o, gate_up, down)
    first = audit[0]["first"]
    assert first["high"] % 128 == 0 and 0 < first["high"] < first["outputs"] and sum(first["calls_by_tokens"].values()) > 0
