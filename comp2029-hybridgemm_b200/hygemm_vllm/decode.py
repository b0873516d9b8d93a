"""Fixed-batch decode benchmark of a random-init 7B-class model served by vLLM with the hybrid linear method.

Counterpart of the reference's `integrations/vllm/formal/benchmark.py` (engine settings, uniform random
token-id prompts, pure-decode timing through the worker extension) for models that exist only as an
architecture: weights are vLLM's dummy initialisation, the MXFP8 channels of every linear are the 10 % of
output channels with the largest weight-row L2 norm (quota rounded to 128), chosen at load time.

    python -m hygemm_vllm.decode --arch qwen2.5-7b --batch 1,16,128 --prompt 128,1024 --steps 128 [--dense]

prints one JSON line per (prompt length, batch size): decode tokens/s from the median milliseconds per step
over the span of the timed steps (engine gaps included), the coefficient of variation of the samples, and the
audit of the hybrid layers.  Per cell the reference's protocol (formal/benchmark.py:76-91): one warm-up
generation, then `--samples` timed ones; a cell whose coefficient of variation exceeds `--cv` is repeated, at
most three attempts.  `--dense` serves the same model with plain bf16 linears for comparison; `--table FILE`
appends the rows as a markdown table.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
from pathlib import Path

ARCHITECTURES = {
    "qwen2.5-7b": {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 3584,
                   "intermediate_size": 18944, "num_hidden_layers": 28, "num_attention_heads": 28,
                   "num_key_value_heads": 4, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "vocab_size": 152064,
                   "max_position_embeddings": 32768, "hidden_act": "silu", "tie_word_embeddings": False},
    "mistral-7b": {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_size": 4096,
                   "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32,
                   "num_key_value_heads": 8, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "vocab_size": 32000,
                   "max_position_embeddings": 32768, "hidden_act": "silu", "tie_word_embeddings": False,
                   "sliding_window": None},
}


def write_model_dir(folder, arch: str, dense: bool = False, fraction: float = 0.1, layers: int | None = None) -> Path:
    """A model directory holding only `config.json` (served with `load_format="dummy"`)."""
    config = dict(ARCHITECTURES[arch], torch_dtype="bfloat16")
    if layers:
        config["num_hidden_layers"] = layers
    if not dense:
        config["quantization_config"] = {"quant_method": "hygemm",
                                         "selection": {"rule": "l2norm", "fraction": fraction, "multiple": 128}}
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


def engine_arguments(model_dir, batches, prompt: int, steps: int, dense: bool, tp: int = 1, memory: float = 0.6) -> dict:
    """Keyword arguments of `vllm.LLM` (reference: formal/benchmark.py:44-49): no compilation, FULL CUDA graphs
    captured for exactly the measured batch sizes after one eager warm-up each (the hybrid layers create their
    GEMM handles in that warm-up)."""
    return dict(model=str(model_dir), skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16",
                quantization=None if dense else "hygemm", max_model_len=prompt + steps + 16,
                max_num_seqs=max(batches), max_num_batched_tokens=max(2048, prompt * 2),
                gpu_memory_utilization=memory, tensor_parallel_size=tp, enable_prefix_caching=False, seed=0,
                generation_config="vllm", worker_extension_cls="hygemm_vllm.worker.AuditWorkerExtension",
                compilation_config={"mode": 0, "cudagraph_mode": "FULL", "cudagraph_capture_sizes": sorted(batches),
                                    "max_cudagraph_capture_size": max(batches), "cudagraph_num_of_warmups": 1})


def ensure_plugin_entry_point() -> None:
    """vLLM loads `vllm.general_plugins` entry points in every worker process.  When this package is used from
    its source tree (not pip-installed) no entry point exists, so one is published the way an editable install
    would: a `*.dist-info` with `entry_points.txt` in a temporary directory that, together with the package
    root, is put on `PYTHONPATH` for the worker processes."""
    import importlib.metadata as metadata
    import sys
    if any(ep.name == "hygemm_quantization" for ep in metadata.entry_points(group="vllm.general_plugins")):
        return
    root = Path(tempfile.mkdtemp(prefix="hygemm_plugin_"))
    info = root / "hygemm_vllm_b200-0.1.dist-info"
    info.mkdir()
    (info / "METADATA").write_text("Metadata-Version: 2.1\nName: hygemm-vllm-b200\nVersion: 0.1\n")
    (info / "entry_points.txt").write_text("[vllm.general_plugins]\nhygemm_quantization = hygemm_vllm:register\n")
    package_root = str(Path(__file__).resolve().parent.parent)
    os.environ["PYTHONPATH"] = os.pathsep.join(p for p in (str(root), package_root, os.environ.get("PYTHONPATH", "")) if p)
    sys.path.insert(0, str(root))


def summarise(samples: list[dict], batch: int) -> dict:
    """Median, coefficient of variation and tokens/s of one cell's samples (reference: formal/benchmark.py:84-89)."""
    import statistics
    times = [x["decode_ms_per_step"] for x in samples]
    median = statistics.median(times)
    cv = statistics.pstdev(times) / statistics.mean(times) if len(times) > 1 else 0.0
    return {"median_ms_per_step": median, "cv": cv, "decode_tokens_per_s": batch * 1000.0 / median,
            "steps": min(x["steps"] for x in samples), "graph_steps": min(x["graph_steps"] for x in samples),
            "gpu_ms_per_step": statistics.median(x["sum_step_gpu_ms"] / x["steps"] for x in samples),
            "context": [min(x["context_min"] for x in samples), max(x["context_max"] for x in samples)]}


def run(arch: str, batches, prompts, steps: int, dense: bool = False, layers: int | None = None, tp: int = 1,
        samples: int = 5, cv_gate: float = 0.05, attempts: int = 3):
    import torch
    if tp == 1:
        os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")   # engine in this process: the plugin is registered here
    else:
        ensure_plugin_entry_point()                                    # worker processes find the plugin themselves
    import hygemm_vllm
    hygemm_vllm.register()
    from vllm import LLM, SamplingParams
    prompts = [prompts] if isinstance(prompts, int) else list(prompts)
    results = []
    with tempfile.TemporaryDirectory() as tmp:
        model_dir = write_model_dir(Path(tmp) / arch, arch, dense, layers=layers)
        llm = LLM(**engine_arguments(model_dir, batches, max(prompts), steps, dense, tp))
        vocab = ARCHITECTURES[arch]["vocab_size"]
        sampling = SamplingParams(max_tokens=steps, ignore_eos=True, temperature=0.0, detokenize=False)
        for prompt in prompts:
            g = torch.Generator().manual_seed(20261024 + prompt)
            for batch in batches:
                ids = [{"prompt_token_ids": torch.randint(0, vocab, (prompt,), generator=g).tolist()} for _ in range(batch)]

                def timed():
                    llm.collective_rpc("formal_begin", args=(batch,))
                    llm.generate(ids, sampling, use_tqdm=False)
                    return llm.collective_rpc("formal_end")[0]
                for attempt in range(attempts):
                    llm.generate(ids, sampling, use_tqdm=False)                  # warm-up pass
                    cell = summarise([timed() for _ in range(samples)], batch)
                    if cell["cv"] <= cv_gate:
                        break
                row = {"arch": arch, "dense": dense, "tp": tp, "batch": batch, "prompt": prompt, "samples": samples,
                       "attempts": attempt + 1, "stable": cell["cv"] <= cv_gate, **cell,
                       "decode_ms_per_step": cell["median_ms_per_step"]}
                results.append(row)
                print(json.dumps(row), flush=True)
        if not dense:
            audit = llm.collective_rpc("hygemm_model_audit")[0]
            print(json.dumps({"audit_layers": len(audit), "first": audit[0] if audit else None}), flush=True)
    return results


def append_table(path, rows, note: str = "") -> None:
    """Markdown rows `arch | linears | tp | prompt | batch | tokens/s | ms/step | CV | attempts` appended to `path`."""
    path = Path(path)
    fresh = not path.exists()
    with path.open("a") as f:
        if fresh:
            f.write("| arch | linears | TP | prompt | batch | decode tokens/s | ms/step (median) | CV | attempts | FULL-graph steps |\n")
            f.write("|---|---|---|---|---|---|---|---|---|---|\n")
        for r in rows:
            f.write(f"| {r['arch']} | {'dense bf16' if r['dense'] else 'hybrid' + note} | {r['tp']} | {r['prompt']} | {r['batch']} | "
                    f"{r['decode_tokens_per_s']:.0f} | {r['median_ms_per_step']:.3f} | {r['cv']:.3f} | {r['attempts']} | "
                    f"{r['graph_steps']}/{r['steps']} |\n")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--arch", default="qwen2.5-7b", choices=sorted(ARCHITECTURES))
    ap.add_argument("--batch", default="1,16,128")
    ap.add_argument("--prompt", default="128", help="prompt length, or several separated by commas")
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--layers", type=int, default=None, help="fewer decoder layers (smoke runs)")
    ap.add_argument("--dense", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (one worker process per GPU)")
    ap.add_argument("--samples", type=int, default=5, help="timed generations per cell after one warm-up")
    ap.add_argument("--cv", type=float, default=0.05, help="largest accepted coefficient of variation of a cell")
    ap.add_argument("--table", default=None, help="append the rows as a markdown table to this file")
    args = ap.parse_args(argv)
    rows = run(args.arch, [int(b) for b in args.batch.split(",")], [int(v) for v in args.prompt.split(",")], args.steps,
               args.dense, args.layers, args.tp, args.samples, args.cv)
    if args.table:
        fused = os.environ.get("HYGEMM_FUSE_SILU", "0") == "1"
        append_table(args.table, rows, " + fused SwiGLU producer" if fused and not args.dense else "")


if __name__ == "__main__":
    main()
