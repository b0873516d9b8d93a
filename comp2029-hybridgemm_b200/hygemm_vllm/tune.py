"""M-bucket schedule tuner and bound plan files for the B200 library.

Counterpart of the reference's `integrations/vllm/performance/tune.py` (resident screen, cold refinement,
2 % switch margin) and `performance/bind_plan.py` (plans bound to the binary they were tuned on).  The
search space is this library's: one tcgen05 kernel with the tile schedules of include/hygemm.h (1
data-parallel, 2 split-K, 3 stream-K; 0 lets the library choose) and, up to four tokens, the SIMT pair
kernel behind policies `gemv_pair1/2/4`.

    python -m hygemm_vllm.tune --shapes 4608x3584x512,3584x18944x384 --tokens 1,16,128 --out plans.json

writes `{"hygemm": [{"out","k","high","tokens","low_id","high_id","policy","us",...}], "binding": {...}}`,
which `PlanTable` (plans.py) loads through the `tuning_plan` key of the quantization config.  Every candidate
is validated against a dequantise-and-matmul of the same operands (atol .01, rtol .003 as the reference's
tuner) before it is timed.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import statistics
from pathlib import Path

import torch

from . import native
from .fp4_quant import decode_logical
from .offline_weights import logical_scales
from .plans import LAYOUT

SCHEDULES = (1, 2, 3)
SWITCH_MARGIN = 1.02          # a tuned choice replaces the library's own only if it is at least 2 % faster
EVICTION_BYTES = 256 << 20    # larger than the 126 MB L2


def dequantised_weight(layer: native.DualLinear) -> torch.Tensor:
    """fp32 `[N, K]` of what the layer's stored codes and scales represent."""
    w = torch.empty(layer.outputs, layer.k, dtype=torch.float32, device=layer.w4.device)
    if layer.lo.numel():
        w[layer.lo.long()] = decode_logical(layer.w4, logical_scales(layer.sf4, layer.lo.numel(), layer.k), layer.k)
    if layer.hi.numel():
        scale = torch.exp2(logical_scales(layer.sf8, layer.hi.numel(), layer.k).float() - 127)
        codes = layer.w8.view(torch.float8_e4m3fn).float().reshape(layer.hi.numel(), layer.k // 32, 32)
        w[layer.hi.long()] = (codes * scale.unsqueeze(-1)).reshape(layer.hi.numel(), layer.k)
    return w


def dequantised_activation(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    rows, k = q.shape
    scale = torch.exp2(logical_scales(sf, rows, k).float() - 127)
    return (q.view(torch.float8_e4m3fn).float().reshape(rows, k // 32, 32) * scale.unsqueeze(-1)).reshape(rows, k)


class Timer:
    """CUDA-graph replay timing as the reference's tuner does it (performance/tune.py:27-46): resident = eight
    calls per replay, one median of three replays; cold = one call per replay with the L2 evicted by an untimed
    read-modify-write of 256 MiB before each, median of three medians of three."""

    def __init__(self, device):
        self.eviction = torch.zeros(EVICTION_BYTES, dtype=torch.uint8, device=device)

    def measure(self, layer, q, sf, config, expected, cold):
        layer.low_id, layer.high_id, layer.concurrent = config["low_id"], config["high_id"], native.POLICIES[config["policy"]]
        y = layer.run_packed(q, sf)
        torch.testing.assert_close(y, expected, atol=.01, rtol=.003)
        count = 1 if cold else 8
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for _ in range(count):
                layer.run_packed(q, sf)
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        samples = []
        for _ in range(3):
            times = []
            for _ in range(3 if cold else 1):
                if cold:
                    self.eviction.add_(1)
                start.record()
                graph.replay()
                stop.record()
                stop.synchronize()
                times.append(start.elapsed_time(stop) * 1000 / count)
            samples.append(statistics.median(times))
        return {**config, "us": statistics.median(samples), "samples_us": samples,
                "cv": statistics.pstdev(samples) / statistics.mean(samples), "validated_full_output": True}


def candidates(tokens: int):
    configs = [{"low_id": s, "high_id": s, "policy": "serial"} for s in SCHEDULES]
    if tokens <= 4:
        configs += [{"low_id": 28, "high_id": 28, "policy": p} for p in ("gemv_pair1", "gemv_pair2", "gemv_pair4")]
    return configs


def tune_shape(outputs, k, high, token_buckets, device, timer=None, seed=20261026, log=None):
    """Plan rows of one (N, K, H) shape: resident screen of every candidate, cold refinement of the best three
    plus the library's own choice, and the 2 % switch rule."""
    timer = timer or Timer(device)
    g = torch.Generator().manual_seed(seed)
    # IEEE half, as the reference's tuner: its 11-bit significand is what the validation tolerance assumes.
    weight = (torch.randn(outputs, k, generator=g) * .04).to(torch.float16).to(device)
    ids = torch.sort(torch.randperm(outputs, generator=g)[:high]).values.to(device)
    layer = native.DualLinear(weight, ids)
    reference = dequantised_weight(layer)
    default = {"low_id": 0, "high_id": 0, "policy": "serial"}
    rows = []
    for tokens in token_buckets:
        x = torch.randn(tokens, k, generator=g).to(torch.float16).to(device)
        q, sf = native.pack(x)
        expected = (dequantised_activation(q, sf) @ reference.t()).to(torch.float16)
        screen = [timer.measure(layer, q, sf, c, expected, cold=False) for c in candidates(tokens)]
        shortlist = [{key: s[key] for key in ("low_id", "high_id", "policy")} for s in sorted(screen, key=lambda s: s["us"])[:3]]
        base = timer.measure(layer, q, sf, default, expected, cold=True)
        refined = [timer.measure(layer, q, sf, c, expected, cold=True) for c in shortlist]
        best = min(refined, key=lambda s: s["us"])
        chosen = best if base["us"] / best["us"] >= SWITCH_MARGIN else base
        if log is not None:
            log.append({"key": [outputs, k, high, tokens], "screen": screen, "base": base, "refined": refined})
        rows.append({"out": outputs, "k": k, "high": high, "tokens": tokens, **chosen})
    layer.low_id = layer.high_id = 0
    layer.close()
    return rows


def bind(rows, library=None):
    """Plan document bound to the library binary and scale layout (reference: performance/bind_plan.py:24-33,
    hygemm_vllm/plans.py:9-19)."""
    library = Path(library or native.library_path())
    return {"hygemm": rows, "binding": {"library_sha256": hashlib.sha256(library.read_bytes()).hexdigest(), "layout": LAYOUT,
                                         "bucket_rule": "smallest covering bucket"}}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shapes", required=True, help="comma-separated OUTxKxHIGH")
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64,128")
    ap.add_argument("--out", type=Path, required=True)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("tuning needs a CUDA device")
    device = torch.device("cuda", torch.cuda.current_device())
    buckets = sorted(int(t) for t in args.tokens.split(","))
    timer, rows, log = Timer(device), [], []
    for spec in args.shapes.split(","):
        outputs, k, high = (int(v) for v in spec.split("x"))
        rows += tune_shape(outputs, k, high, buckets, device, timer, log=log)
        print("tuned", spec, [(r["tokens"], r["low_id"], r["policy"], round(r["us"], 2)) for r in rows if (r["out"], r["k"], r["high"]) == (outputs, k, high)], flush=True)
    args.out.write_text(json.dumps(bind(rows), indent=1))
    args.out.with_suffix(".raw.json").write_text(json.dumps(log))


if __name__ == "__main__":
    main()
