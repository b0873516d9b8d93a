"""Benchmark of the hybrid MXFP4/MXFP8 linear hot path on B200.

Workload (`config.workload`): the Qwen2.5-7B layer-shape sweep — qkv 3584->4608,
o_proj 3584->3584, gate_up 3584->37888, down 18944->3584 (10 % MXFP8 channels
rounded to a multiple of 128), M in {1,2,4,8,16,32,64,128}.  One STEP is one
pass of that sweep: for every M, one layer's worth of the hot path —
quantise(x) -> qkv GEMM, quantise -> o_proj GEMM, quantise -> gate_up GEMM,
SwiGLU+quantise -> down GEMM (8 kernels per M, 64 per step).  Two distinct
weight sets (272 MB) alternate between consecutive M so every GEMM streams its
weights from HBM, not from L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

* `value`: whole-job TFLOP/s (2*M*N*K over all GEMMs of the timed steps) with
  inputs resident in HBM, the step replayed as one CUDA graph.
* `e2e`: the same metric through the plugin-facing Python API
  (`DualLinear.__call__`, `linear_silu` path) with HOST buffers: pinned-host ->
  device copies of the step's activations and device -> host reads of its
  outputs inside the timed region.
* `roofline`: the tcgen05 GEMM kernel; algorithmic bytes per launch
  (L*K/2 + H*K + N*K/32 + 4N + M*K + M*K/32 + 2*M*N) over the CUDA-event
  duration of each launch in the same weight-cycling sequence.
* `cpu_baseline`: the PyTorch port of the reference's dequantise-and-matmul path
  on the host cores, on a bounded sample of the workload.
* N > 1: the layer is sharded by tensor parallelism (column-parallel qkv /
  gate_up on N, row-parallel o_proj / down on K with an NCCL all-reduce);
  total work is fixed, so `scaling` is "strong".
* `--impl reference`: the CPU port alone, same metric and unit (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "comp2029-hybridgemm_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402

SEED = 20261024
HIDDEN, INTER = 3584, 18944
M_SWEEP = [1, 2, 4, 8, 16, 32, 64, 128]
# name: (K, {projection: width}) of the unsharded layer
SHAPES = {"qkv": (HIDDEN, {"q": 3584, "k": 512, "v": 512}), "o_proj": (HIDDEN, {"o": HIDDEN}),
          "gate_up": (HIDDEN, {"gate": INTER, "up": INTER}), "down": (INTER, {"down": HIDDEN})}
ROW_PARALLEL = {"o_proj", "down"}
METRIC = "hybrid_gemm_tflops_qwen2.5-7b_layer_sweep_M1-128"


def high_quota(n: int) -> int:
    return 128 * round(0.1 * n / 128)


def gemm_bytes(m, k, n, h):
    """Algorithmic HBM bytes of one hybrid GEMM call."""
    low = n - h
    return low * k // 2 + h * k + n * k // 32 + 4 * n + m * k + m * k // 32 + 2 * m * n


# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the same launch, from the ncu
# captures summarised under profiles/ (one per shape class; cold weights, weight copies cycled).  The ratio
# does not move with the token count inside a class: the weights are read once and dominate.  Above 32 tokens
# part of the output is still in L2 when the launch ends (gate_up at 128 tokens: 9.7 MB written, 3.8 MB reach DRAM).
DRAM_TRAFFIC_RATIO = {("gate_up", "decode"): 1.01, ("down", "decode"): 1.00, ("qkv", "decode"): 0.99,
                      ("o_proj", "decode"): 0.99, ("gate_up", "wide"): 0.93, ("down", "wide"): 0.98,
                      ("qkv", "wide"): 0.99, ("o_proj", "wide"): 0.99}


def dram_traffic_ratio(name: str, m: int) -> float:
    return DRAM_TRAFFIC_RATIO[(name, "decode" if m <= 32 else "wide")]


def k_block_shard(k: int, rank: int, world: int) -> tuple[int, int]:
    """Row-parallel K range of `rank`, in whole K128 blocks (uneven when blocks % world != 0)."""
    blocks = k // 128
    base, rem = divmod(blocks, world)
    begin = rank * base + min(rank, rem)
    return begin * 128, (begin + base + (1 if rank < rem else 0)) * 128


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, begin: float, end: float) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.samples if begin - 0.05 <= t <= end + 0.15 and len(r) >= 7] or \
               [r for _, r in self.samples if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]

        def num(s):
            try:
                return float(s)
            except ValueError:
                return None
        sm = [num(r[0]) for r in rows if num(r[0]) is not None]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": num(rows[0][1]),
                "power_w_max": max((num(r[2]) or 0) for r in rows), "samples": len(rows), "reasons": reasons}


# ------------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------------

def build_layer(device, layer_seed: int, rank: int, world: int):
    """One transformer layer's four hybrid linears (this rank's tensor-parallel shard)."""
    from hygemm_vllm import native
    g = torch.Generator().manual_seed(layer_seed)
    layer = {}
    for name, (k, parts) in SHAPES.items():
        n = sum(parts.values())
        w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
        high = torch.sort(torch.randperm(n, generator=g)[: high_quota(n)]).values
        if world > 1:
            if name in ROW_PARALLEL:
                begin, end = k_block_shard(k, rank, world)
                w = w[:, begin:end].contiguous()
            else:
                keep, offset = [], 0
                for width in parts.values():
                    if name == "gate_up":
                        # gate and up keep the intermediate channels of this rank's K shard of down_proj (whole
                        # K128 blocks, uneven when 148 blocks do not divide by the world size)
                        begin, end = k_block_shard(width, rank, world)
                    else:
                        begin, end = rank * (width // world), (rank + 1) * (width // world)
                    keep.append(torch.arange(offset + begin, offset + end))
                    offset += width
                keep = torch.cat(keep)
                mask = torch.zeros(n, dtype=torch.bool)
                mask[high] = True
                w = w[keep].contiguous()
                high = torch.where(mask[keep])[0]
        layer[name] = native.DualLinear(w.to(device), high.to(device))
    return layer


def launches_of(rt, tokens):
    """Kernels one hybrid GEMM call launches: 1, or 2 when its cut tiles are summed by the reduce kernel."""
    import ctypes as C
    from hygemm_vllm import native
    header = (C.c_int * 12)()
    props = torch.cuda.get_device_properties(rt.w4.device)
    native.check(native.library().hg_plan(int(rt.lo.numel()), int(rt.hi.numel()), tokens, rt.k,
                                          props.multi_processor_count, rt.low_id, header, None, 0))
    return 1 + header[10]


def shard_stats(layer):
    """(K, N, H) of each GEMM as this rank runs it."""
    return {name: (rt.k, rt.outputs, int(rt.hi.numel())) for name, rt in layer.items()}


class Sweep:
    """Device buffers and the launch sequence of one step."""

    def __init__(self, device, layers, world, group):
        from hygemm_vllm import native, producer
        self.native, self.producer = native, producer
        self.layers, self.world, self.group, self.device = layers, world, group, device
        g = torch.Generator().manual_seed(SEED + 1)
        self.host, self.dev = {}, {}
        k_o = layers[0]["o_proj"].k
        for m in M_SWEEP:
            x = torch.randn(3, m, HIDDEN, generator=g)
            cols = torch.randperm(HIDDEN, generator=g)[: -(-HIDDEN // 100)]
            x[:, :, cols] *= 20
            x = x.to(torch.bfloat16)
            self.host[m] = {"x_qkv": x[0].contiguous().pin_memory(), "x_gate": x[2].contiguous().pin_memory(),
                            "x_o": x[1][:, :k_o].contiguous().pin_memory()}
            self.dev[m] = {n: t.to(device) for n, t in self.host[m].items()}
        # quantiser launches per M (one SwiGLU-quantiser; three activation quantisers unless they are fused
        # into the GEMM launch) plus the GEMM launches (a GEMM whose cut tiles are summed by the separate
        # reduce kernel counts two)
        def quantisers(i, m):
            separate = [name for name in ("qkv", "o_proj", "gate_up")
                        if m > native.FUSED_QUANT_TOKENS or self.layer_for(i)[name].outputs > native.FUSED_QUANT_MAX_OUTPUTS]
            return 1 + len(separate)
        self.launches_per_step = sum(quantisers(i, m) + sum(launches_of(self.layer_for(i)[name], m) for name in SHAPES)
                                     for i, m in enumerate(M_SWEEP))
        self.event_factory = lambda: torch.cuda.Event(enable_timing=True)
        # Row-parallel layers under tensor parallelism: the GEMM writes its partial sums into a peer-mapped
        # buffer and a second launch pulls every rank's partials over NVLink and sums them
        # (HYGEMM_TP_EXCHANGE=0: GEMM + NCCL all-reduce).
        self.exchange, self.exchange_note = None, None
        if world > 1 and os.environ.get("HYGEMM_TP_EXCHANGE", "1") != "0":
            try:
                from hygemm_vllm import tp
                self.exchange = tp.PeerExchange(group, max(M_SWEEP) * HIDDEN, torch.bfloat16, device)
                self.launches_per_step += 2 * len(M_SWEEP)
                self.exchange_note = self.verify_exchange()
            except Exception as exc:     # no peer access between these GPUs, or symmetric memory unavailable
                self.exchange = None
                self.exchange_note = f"NCCL all-reduce ({type(exc).__name__}: {exc})"[:200]

    def verify_exchange(self):
        """The fused exchange against GEMM + NCCL all-reduce on the same inputs, once, before timing."""
        worst = 0.0
        for i, m in enumerate((16, 128)):
            layer = self.layer_for(i)
            q, sf = self.native.pack(self.dev[m]["x_o"])
            want = layer["o_proj"].run_packed(q, sf)
            torch.distributed.all_reduce(want, group=self.group)
            got = layer["o_proj"].run_exchange(self.exchange, q=q, sf=sf)
            worst = max(worst, ((got.float() - want.float()).abs().max() / want.float().abs().max()).item())
        status = self.exchange.status()
        if status or not worst < 0.02:
            raise RuntimeError(f"exchange disagrees with NCCL: status {status}, max relative difference {worst}")
        return (f"GEMM writes its partial to a peer-mapped buffer (fp32 up to 16 tokens) + one launch that pulls all ranks' "
                f"partials over NVLink and adds them; max relative difference to NCCL {worst:.2e}")

    def layer_for(self, i):
        return self.layers[i % len(self.layers)]

    def run_m(self, i, m, x, events=None):
        """One layer's hot path at M tokens.  `events` (optional) collects (name, m, start, end) around GEMMs."""
        layer = self.layer_for(i)
        native, producer = self.native, self.producer
        out = {}

        def timed(name, call):
            if events is None:
                return call()
            a, b = self.event_factory(), self.event_factory()
            a.record()
            y = call()
            b.record()
            events.append((name, m, a, b))
            return y

        # What `layer(x)` (the plugin-facing call) does: up to 16 tokens the activations are quantised inside
        # the GEMM launch (hg_run_x); above that the quantiser is its own launch.  Events bracket the GEMM launch.
        def linear(name, xin, row_parallel=False):
            rt = layer[name]
            if row_parallel and self.exchange is not None:
                if m <= native.FUSED_QUANT_TOKENS:
                    return timed(name, lambda: rt.run_exchange(self.exchange, x=xin))
                q, sf = native.pack(xin)
                return timed(name, lambda: rt.run_exchange(self.exchange, q=q, sf=sf))
            if m <= native.FUSED_QUANT_TOKENS and rt.outputs <= native.FUSED_QUANT_MAX_OUTPUTS:
                return timed(name, lambda: rt(xin))
            q, sf = native.pack(xin)
            return timed(name, lambda: rt.run_packed(q, sf))

        out["qkv"] = linear("qkv", x["x_qkv"])
        y_o = linear("o_proj", x["x_o"], row_parallel=True)
        if self.world > 1 and self.exchange is None:
            torch.distributed.all_reduce(y_o, group=self.group)
        gate_up = linear("gate_up", x["x_gate"])
        q, sf = producer.silu_pack(gate_up, 0)
        if self.exchange is not None:
            y_d = timed("down", lambda: layer["down"].run_exchange(self.exchange, q=q, sf=sf))
        else:
            y_d = timed("down", lambda: layer["down"].run_packed(q, sf))
            if self.world > 1:
                torch.distributed.all_reduce(y_d, group=self.group)
        out["o_proj"], out["down"] = y_o, y_d
        return out

    def step_resident(self, events=None):
        outs = None
        for i, m in enumerate(M_SWEEP):
            outs = self.run_m(i, m, self.dev[m], events)
        return outs

    def step_e2e(self, host_out, overlap=False):
        """Host buffers in, host buffers out: the call a user of the plugin-facing API makes.

        `overlap`: the copies run on their own streams (inputs of every M are sent ahead, each M's results
        leave while the next M computes); used when the step is captured into a CUDA graph, where every
        tensor stays alive until the capture ends."""
        h2d = d2h = 0
        if not overlap:
            for i, m in enumerate(M_SWEEP):
                x = {n: t.to(self.device, non_blocking=True) for n, t in self.host[m].items()}
                h2d += sum(t.numel() * t.element_size() for t in self.host[m].values())
                out = self.run_m(i, m, x)
                for name in ("qkv", "o_proj", "down"):
                    host_out[m][name].copy_(out[name], non_blocking=True)
                    d2h += out[name].numel() * out[name].element_size()
            return h2d, d2h
        main = torch.cuda.current_stream()
        if not hasattr(self, "copy_streams"):
            self.copy_streams = (torch.cuda.Stream(), torch.cuda.Stream())
        cin, cout = self.copy_streams
        keep = []                                                  # nothing is freed (and reused) mid-capture
        cin.wait_stream(main)
        cout.wait_stream(main)
        arrived = []
        with torch.cuda.stream(cin):
            for m in M_SWEEP:
                x = {n: t.to(self.device, non_blocking=True) for n, t in self.host[m].items()}
                h2d += sum(t.numel() * t.element_size() for t in self.host[m].values())
                event = torch.cuda.Event()
                event.record(cin)
                arrived.append((x, event))
        for i, m in enumerate(M_SWEEP):
            x, event = arrived[i]
            main.wait_event(event)
            out = self.run_m(i, m, x)
            done = torch.cuda.Event()
            done.record(main)
            keep.append((x, out))
            with torch.cuda.stream(cout):
                cout.wait_event(done)
                for name in ("qkv", "o_proj", "down"):
                    host_out[m][name].copy_(out[name], non_blocking=True)
                    d2h += out[name].numel() * out[name].element_size()
        main.wait_stream(cin)
        main.wait_stream(cout)
        self.keep = keep
        return h2d, d2h


def total_flops(stats):
    return sum(2 * m * n * k for m in M_SWEEP for (k, n, h) in stats.values())


# ------------------------------------------------------------------------------------------------
# CPU baseline (the oracle port; the only place the benchmark executes oracle code)
# ------------------------------------------------------------------------------------------------

_CPU_CASES = None


def _cpu_cases():
    """Quantised qkv and o_proj operands of the CPU sample (prepared once, outside any timed region)."""
    global _CPU_CASES
    if _CPU_CASES is None:
        import oracle
        g = torch.Generator().manual_seed(SEED)
        cases = []
        for name in ("qkv", "o_proj"):
            k, parts = SHAPES[name]
            n = sum(parts.values())
            w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
            high = torch.sort(torch.randperm(n, generator=g)[: high_quota(n)]).values.numpy()
            lo, hi = oracle.partition(n, high)
            w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True)
            w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False)
            xs = {m: torch.randn(m, k, generator=g).to(torch.bfloat16) for m in (1, 16, 128)}
            cases.append((k, n, lo, hi, w4, sf4, w8, sf8, xs))
        _CPU_CASES = cases
    return _CPU_CASES


def cpu_reference_sample(min_seconds: float = 0.0, passes: int = 1):
    """Bounded sample of the workload on the host cores: qkv and o_proj shapes at M in {1,16,128} through the
    PyTorch port of the reference's `reference()` (activations quantised, weights re-dequantised per call,
    fp32 matmul — what the reference literally does).  Runs `passes` passes, then more until `min_seconds`."""
    from oracle import torch_path
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    cases = _cpu_cases()
    flops, done, begin = 0, 0, time.perf_counter()
    while done < passes or time.perf_counter() - begin < min_seconds:
        for k, n, lo, hi, w4, sf4, w8, sf8, xs in cases:
            for m, x in xs.items():
                torch_path.reference_linear(x, w4, sf4, lo, w8, sf8, hi, n, redequantise=True)
                flops += 2 * m * n * k
        done += 1
    seconds = time.perf_counter() - begin
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"qkv+o_proj shapes x M in (1,16,128), {done} pass(es), weights re-dequantised per call "
                      f"as reference() does; {seconds:.1f} s of CPU work"}, seconds


def run_reference_arm(args, rank):
    if rank != 0:
        return
    for _ in range(args.warmup):                              # page-in, thread pool
        cpu_reference_sample()
    base, seconds = cpu_reference_sample(passes=args.steps)   # one step = one pass over the sample
    value = base["value"]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / max(1, args.steps),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "mxfp4/mxfp8 x mxfp8 -> fp32 accumulate -> bf16", "data": "synthetic",
            "config": {"workload": "Qwen2.5-7B layer-shape GEMM sweep (bounded CPU sample: qkv + o_proj, M in 1/16/128)"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# single-GEMM mode (small, self-ending case for ncu captures)
# ------------------------------------------------------------------------------------------------

def run_single_gemm(args, device):
    """`--gemm NAME:M[:SCHEDULE]`: one shape, `steps` launches alternating between enough weight copies to
    exceed L2, each bracketed by CUDA events; prints one JSON line with the median duration."""
    from hygemm_vllm import native
    fields = args.gemm.split(":")
    name, m = fields[0], int(fields[1])
    schedule = int(fields[2]) if len(fields) > 2 else 0
    k, parts = SHAPES[name]
    n = sum(parts.values())
    h = high_quota(n) if len(fields) < 4 or fields[3] == '' else int(round(float(fields[3]) * n))
    fused = len(fields) > 4 and fields[4] == 'fused'
    weight_bytes = (n - h) * k // 2 + h * k
    copies = max(2, -(-300_000_000 // weight_bytes))            # > 2x the 126 MB L2 between reuses
    g = torch.Generator().manual_seed(SEED)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(device)
    high = torch.sort(torch.randperm(n, generator=g)[:h]).values.to(device)
    layers = []
    for c in range(copies):
        layers.append(native.DualLinear(torch.roll(w, c, 0) if c else w, high, schedule, schedule))
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(device)
    q, sf = native.pack(x)
    for layer in layers[:2]:
        layer.run_packed(q, sf)
    torch.cuda.synchronize()
    import ctypes as C
    stream = torch.cuda.current_stream().cuda_stream
    for layer in layers:
        if not layer.handles:
            layer.run_packed(q, sf)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    calls = []
    for layer in layers:
        low, hi = layer.problems(q, sf, y)
        calls.append((layer.handles[next(iter(layer.handles))], low, hi))
    lib = native.library()

    def enqueue(count):
        stream = torch.cuda.current_stream().cuda_stream      # the capture stream while a graph is recorded
        for i in range(count):
            handle, low, hi = calls[i % copies]
            if fused:
                native.check(lib.hg_run_x(handle, C.byref(low), C.byref(hi), x.data_ptr(), 1, stream))
            else:
                native.check(lib.hg_run(handle, C.byref(low), C.byref(hi), stream, 0))

    # `count` launches back to back (weight copies cycled) as one CUDA graph, so the host launch rate
    # does not bound what is measured; one event pair around each replay.
    count = max(args.steps, copies)
    enqueue(copies)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue(count)
    stream = torch.cuda.current_stream().cuda_stream
    times = []
    for _ in range(6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e-3 / count)
    times = times[1:]
    seconds = statistics.median(times)
    nbytes = gemm_bytes(m, k, n, h)
    info = layers[0].info(m)
    line = {"gemm": name, "M": m, "K": k, "N": n, "H": h, "schedule": info[0], "n_tile": info[2],
            "stages": info[4], "copies": copies, "us_median": seconds * 1e6, "us_min": min(times) * 1e6,
            "GBps": nbytes / seconds / 1e9, "algorithmic_bytes": nbytes,
            "status": [layer.status() for layer in layers][:2]}
    if args.timeline:
        line["timeline"] = cta_timeline(lib, [c[0] for c in calls], stream)
    print(json.dumps(line))


TIMELINE_POINTS = ["entry", "setup_done", "wait_released", "first_full_stage", "unit0_committed", "unit1_committed",
                   "unit2_committed", "unit3_committed", "epilogue0_start", "epilogue0_end", "epilogue1_start",
                   "epilogue1_end", "epilogue2_start", "epilogue2_end"]


def cta_timeline(lib, handles, stream):
    """Per-CTA time stamps of the last launch of each handle (trace build of the library): for the launch that ran
    last, microseconds after its first CTA entered, as [min, median, 90th percentile, max] over the grid per point,
    and the distance to the first entry of the launch before it.  The global timer ticks in steps of up to 0.5 us."""
    import ctypes as C
    import numpy as np
    traces = []
    for handle in handles:
        buf = (C.c_uint64 * (16 * 1024))()
        count = C.c_int(0)
        from hygemm_vllm import native
        native.check(lib.hg_trace(handle, stream, buf, len(buf), C.byref(count)))
        traces.append(np.frombuffer(buf, dtype=np.uint64, count=count.value).reshape(-1, 16).astype(np.int64))
    traces.sort(key=lambda a: a[:, 0].min())
    last, before = traces[-1], traces[-2]
    t0 = last[:, 0].min()
    out = {"ctas": int(last.shape[0]), "period_us": round(float(t0 - before[:, 0].min()) / 1e3, 2)}
    for i, point in enumerate(TIMELINE_POINTS):
        column = last[:, i]
        if (column > 0).any():
            v = (column[column > 0] - t0) / 1e3
            out[point] = [round(float(np.percentile(v, q)), 1) for q in (0, 50, 90, 100)]
    return out


def run_single_quant(args, device):
    """`--quant act:ROWS:K` or `--quant silu:ROWS:K`: the activation quantiser or the SwiGLU + quantiser alone,
    `steps` launches as one CUDA graph over enough distinct inputs to exceed L2; one JSON line (a small,
    self-ending case for ncu captures)."""
    from hygemm_vllm import native, producer
    kind, rows, k = args.quant.split(":")
    rows, k = int(rows), int(k)
    width = 2 * k if kind == "silu" else k
    in_bytes = rows * width * 2
    copies = max(2, min(64, -(-300_000_000 // max(in_bytes, 1))))
    g = torch.Generator().manual_seed(SEED)
    xs = [(torch.randn(rows, width, generator=g) * (2.0 if kind == "silu" else 1.0)).to(torch.bfloat16).to(device)
          for _ in range(copies)]

    def call(x):
        return producer.silu_pack(x, 0) if kind == "silu" else native.pack(x)
    count = max(args.steps, copies)
    keep = [call(x) for x in xs]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        keep = [call(xs[i % copies]) for i in range(count)]
    times = []
    for _ in range(6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e-3 / count)
    seconds = statistics.median(times[1:])
    nbytes = in_bytes + rows * k + rows * k // 32
    print(json.dumps({"quant": kind, "rows": rows, "K": k, "copies": copies, "us_median": seconds * 1e6,
                      "GBps": nbytes / seconds / 1e9, "algorithmic_bytes": nbytes}))


def run_single_clip(args, device):
    """`--clip ROWS:K`: the offline MXFP4 exponent search (`hg_clip_pack`) on a seeded random weight matrix, timed
    with CUDA events; one JSON line with the kernel's rate (it reads 2 B and writes 0.53 B per weight) and the
    error statistics of the search (a small, self-ending case for ncu captures of the load-time path)."""
    import ctypes as C
    from hygemm_vllm import fp4_quant, native
    rows, k = (int(v) for v in args.clip.split(":"))
    g = torch.Generator().manual_seed(SEED)
    w = (torch.randn(rows, k, generator=g) * 0.02).to(torch.bfloat16).to(device)
    importance = (torch.rand(k, generator=g) * 2).to(device)
    q4, scales, stats = fp4_quant.quantize(w, importance)
    lib = native.library()
    shifts = (C.c_int * 3)(0, -1, -2)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(max(3, args.steps)):
        start.record()
        native.check(lib.hg_clip_pack(w.data_ptr(), importance.data_ptr(), q4.data_ptr(), scales.data_ptr(), rows, k,
                                      shifts, 3, native.DTYPES[w.dtype], torch.cuda.current_stream().cuda_stream))
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop) * 1e-3)
    seconds = statistics.median(times)
    moved = w.numel() * 2 + q4.numel() + scales.numel()
    print(json.dumps({"rows": rows, "k": k, "us": seconds * 1e6, "GBps": moved / seconds / 1e9,
                      "algorithmic_bytes": moved, **stats}))


# ------------------------------------------------------------------------------------------------
# main
# ------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--step-only", action="store_true",
                    help="skip the hot per-shape rows and the prefill rows (launch-list captures of the step itself)")
    ap.add_argument("--gemm", default=None, metavar="NAME:M[:SCHEDULE[:HIGH_FRACTION[:fused]]]",
                    help="profiling aid: run only this GEMM (e.g. gate_up:16) a few times on cold weights and exit")
    ap.add_argument("--timeline", action="store_true",
                    help="with --gemm: load the trace build of the library (build.py --trace) and add the per-CTA "
                         "timeline of the last launch to the JSON line")
    ap.add_argument("--quant", default=None, metavar="act|silu:ROWS:K",
                    help="profiling aid: run only this quantiser launch a few times on cold inputs and exit")
    ap.add_argument("--clip", default=None, metavar="ROWS:K",
                    help="profiling aid: time the offline MXFP4 exponent search on a random ROWS x K matrix and exit")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run); got {world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if args.gemm:
        if args.timeline:
            trace_library = ROOT / "comp2029-hybridgemm_b200" / "lib" / "libhygemm_b200_trace.so"
            if not trace_library.exists():
                raise SystemExit(f"--timeline needs {trace_library} (python comp2029-hybridgemm_b200/build.py --trace)")
            os.environ["HYGEMM_LIBRARY"] = str(trace_library)
        run_single_gemm(args, device)
        return
    if args.quant:
        run_single_quant(args, device)
        return
    if args.clip:
        run_single_clip(args, device)
        return
    import torch.distributed as dist
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    layers = [build_layer(device, SEED + 100 * i, rank, world) for i in range(2)]
    stats = shard_stats(layers[0])
    sweep = Sweep(device, layers, world, group)
    flops_step_rank = total_flops(stats)
    flops_step = flops_step_rank
    if world > 1:
        t = torch.tensor([float(flops_step_rank)], device=device, dtype=torch.float64)
        dist.all_reduce(t)
        flops_step = t.item()

    # ---- warm every shape (handles are created outside capture), then capture the step as a graph
    for _ in range(2):
        sweep.step_resident()
    barrier()
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sweep.step_resident()
    except Exception as exc:                                   # e.g. a collective that cannot be captured
        graph = None
        torch.cuda.synchronize()
        note = f"step not graph-captured ({type(exc).__name__}); eager launches timed"
    else:
        note = "step replayed as one CUDA graph"

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            sweep.step_resident()

    for _ in range(args.warmup):
        one_step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    begin_wall = time.time()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        one_step()
    stop.record()
    barrier()
    end_wall = time.time()
    ms = start.elapsed_time(stop)
    clocks = sampler.stop(begin_wall, end_wall) if sampler else None
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    value = flops_step * args.steps / (ms * 1e-3) / 1e12

    # ---- end to end through the plugin-facing API with host buffers
    host_out = {m: {"qkv": torch.empty(m, layers[0]["qkv"].outputs, dtype=torch.bfloat16).pin_memory(),
                    "o_proj": torch.empty(m, HIDDEN, dtype=torch.bfloat16).pin_memory(),
                    "down": torch.empty(m, HIDDEN, dtype=torch.bfloat16).pin_memory()} for m in M_SWEEP}
    for _ in range(args.warmup):
        sweep.step_e2e(host_out)
    barrier()
    e2e_steps = max(3, min(args.steps, 20))
    start.record()
    for _ in range(e2e_steps):
        h2d, d2h = sweep.step_e2e(host_out)
    stop.record()
    barrier()
    e2e_eager_ms = start.elapsed_time(stop)
    # The same calls, host buffers included, recorded once into a CUDA graph and replayed (what a serving
    # engine does with the plugin): the copies become memcpy nodes on side streams and overlap the GEMMs.
    e2e_graph, e2e_api = None, "hygemm_vllm.native.DualLinear.__call__ / producer.silu_pack + run_packed, eager"
    e2e_ms = e2e_eager_ms
    if graph is not None:
        try:
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph):
                h2d, d2h = sweep.step_e2e(host_out, overlap=True)
            for _ in range(args.warmup):
                e2e_graph.replay()
            barrier()
            start.record()
            for _ in range(e2e_steps):
                e2e_graph.replay()
            stop.record()
            barrier()
            e2e_ms = start.elapsed_time(stop)
            e2e_api = ("hygemm_vllm.native.DualLinear.__call__ / producer.silu_pack + run_packed with pinned host inputs "
                       "and outputs, captured once into a CUDA graph (copies as memcpy nodes on side streams) and replayed")
        except Exception as exc:
            torch.cuda.synchronize()
            e2e_graph, e2e_ms = None, e2e_eager_ms
            e2e_api += f" (graph capture of the host-buffer step failed: {type(exc).__name__})"
    if world > 1:
        t = torch.tensor([e2e_ms, e2e_eager_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, e2e_eager_ms = t.tolist()
    e2e_value = flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12

    # ---- per-launch GEMM durations in the same weight-cycling sequence: CUDA events recorded INSIDE a graph
    # of the step (event-record nodes on the launch stream), so the host launch path is not in the number.
    timed_graph = None
    per, how = {}, "event-record nodes around each GEMM inside a CUDA graph of the step, 5 replays"
    try:
        if graph is None:
            raise RuntimeError("step is not graph-captured")
        events = []
        sweep.event_factory = lambda: torch.cuda.Event(enable_timing=True, external=True)
        timed_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(timed_graph):
            sweep.step_resident(events)
        for _ in range(5):
            timed_graph.replay()
            torch.cuda.synchronize()
            for name, m, a, b in events:
                per.setdefault((name, m), []).append(a.elapsed_time(b) * 1e-3)
    except Exception as exc:
        torch.cuda.synchronize()
        per, events = {}, []
        how = f"eager launches bracketed by events ({type(exc).__name__}: in-graph events unavailable); includes host launch latency"
        sweep.event_factory = lambda: torch.cuda.Event(enable_timing=True)
        for _ in range(5):
            sweep.step_resident(events)
        torch.cuda.synchronize()
        for name, m, a, b in events:
            per.setdefault((name, m), []).append(a.elapsed_time(b) * 1e-3)
    # ---- hot (L2-resident) figure per shape: the same GEMM on the same weights, back to back in one graph.
    # gate_up (79 MB of weights) only just fits the 126 MB L2; the other three stay resident.
    hot = {}
    try:
        from hygemm_vllm import native as _native
        for m in ([] if args.step_only else M_SWEEP):
            x = sweep.dev[m]
            gate_up_out = layers[0]["gate_up"].run_packed(*_native.pack(x["x_gate"]))
            packed = {"qkv": _native.pack(x["x_qkv"]), "o_proj": _native.pack(x["x_o"]), "gate_up": _native.pack(x["x_gate"]),
                      "down": sweep.producer.silu_pack(gate_up_out, 0)}
            for name in SHAPES:
                if world > 1 and name in ROW_PARALLEL:
                    continue                                   # the exchange needs every rank in step: cold rows only
                rt, (q, sf) = layers[0][name], packed[name]
                rt.run_packed(q, sf)
                torch.cuda.synchronize()
                burst = torch.cuda.CUDAGraph()
                with torch.cuda.graph(burst):
                    for _ in range(10):
                        rt.run_packed(q, sf)
                samples = []
                for _ in range(4):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    burst.replay()
                    b.record()
                    torch.cuda.synchronize()
                    samples.append(a.elapsed_time(b) * 1e-3 / 10)
                hot[(name, m)] = statistics.median(samples[1:])
                del burst
    except Exception as exc:                                   # never lose the main line to the diagnostic rows
        hot = {}
        print(f"hot rows skipped: {type(exc).__name__}: {exc}", file=sys.stderr)
    # ---- prefill buckets (the reference's plans reach 2048 tokens): the same kernel in rows of 128-token
    # tiles, the two weight sets alternating so the weights come from HBM; outside the step and its metric.
    prefill = []
    if world == 1 and not args.step_only:
        try:
            from hygemm_vllm import native as _native
            g2 = torch.Generator().manual_seed(SEED + 7)
            for m in (256, 1024, 2048):
                for name, (k, _parts) in SHAPES.items():
                    q, sf = _native.pack(torch.randn(m, k, generator=g2).to(torch.bfloat16).to(device))
                    for layer in layers:
                        layer[name].run_packed(q, sf)
                    torch.cuda.synchronize()
                    burst = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(burst):
                        for i in range(4):
                            layers[i % 2][name].run_packed(q, sf)
                    samples = []
                    for _ in range(4):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record()
                        burst.replay()
                        b.record()
                        torch.cuda.synchronize()
                        samples.append(a.elapsed_time(b) * 1e-3 / 4)
                    del burst
                    prefill.append((name, m, statistics.median(samples[1:])))
        except Exception as exc:
            prefill = []
            print(f"prefill rows skipped: {type(exc).__name__}: {exc}", file=sys.stderr)
    status = [rt.status() for layer in layers for rt in layer.values()]
    if any(s[0] for s in status):
        raise SystemExit(f"device reported a stuck wait: {status}")
    if sweep.exchange is not None and sweep.exchange.status():
        raise SystemExit("a tensor-parallel exchange gave up waiting for a peer")

    if rank == 0:
        peaks = {}
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peaks = json.loads(peaks_file.read_text())
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        # Dense FP8 tensor peak: none is measured on this pool, so twice the measured bf16 cuBLAS burst figure
        # stands in (FP8 issues at twice the bf16 rate), as `tensor_peak_source` says.
        tensor_peak = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
        sweep_rows, bytes_sum, time_sum, traffic_sum = [], 0, 0.0, 0.0
        for (name, m), durations in sorted(per.items(), key=lambda kv: (list(SHAPES).index(kv[0][0]), kv[0][1])):
            k, n, h = stats[name]
            seconds = statistics.median(durations)
            nbytes = gemm_bytes(m, k, n, h)
            bytes_sum += nbytes
            time_sum += seconds
            traffic_sum += nbytes * dram_traffic_ratio(name, m)
            flops = 2 * m * n * k
            row = {"gemm": name, "M": m, "K": k, "N": n, "H": h, "us": round(seconds * 1e6, 2),
                   "GBps": round(nbytes / seconds / 1e9, 1), "TFLOPs": round(flops / seconds / 1e12, 2),
                   "hbm_frac": round(nbytes / seconds / 1e9 / hbm_peak, 3)}
            if (name, m) in hot:
                hs = hot[(name, m)]
                row.update({"hot_us": round(hs * 1e6, 2), "hot_TFLOPs": round(flops / hs / 1e12, 2)})
            if m >= 64:                                       # the tensor-pipe side of the roofline, cold and hot
                row["tensor_frac"] = round(flops / seconds / 1e12 / tensor_peak, 3)
                if (name, m) in hot:
                    row["hot_tensor_frac"] = round(flops / hot[(name, m)] / 1e12 / tensor_peak, 3)
            sweep_rows.append(row)
        # Two figures for the same 32 GEMM launches.  `bracketed`: each launch between its own pair of event
        # nodes, which serialises it against its neighbours (no programmatic overlap of prologue and tail) and
        # adds the event nodes' own cost, so the durations sum to more than the step.  `achieved`: the GEMM
        # bytes over the whole timed step, i.e. with the quantiser launches counted as GEMM time; it is a
        # lower bound of the kernel's rate in the sequence that is actually timed.
        bracketed = bytes_sum / time_sum / 1e9
        achieved = bytes_sum / (ms / args.steps * 1e-3) / 1e9 if sweep_rows else 0.0
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "mxfp4/mxfp8 x mxfp8 -> fp32 accumulate -> bf16", "data": "synthetic",
            "config": {"workload": "Qwen2.5-7B layer-shape hybrid GEMM sweep: qkv 3584->4608, o_proj 3584->3584, "
                                   "gate_up 3584->37888, down 18944->3584; M in 1,2,4,8,16,32,64,128; 10% MXFP8 channels",
                       "step": "per M: quantise+qkv, quantise+o_proj, quantise+gate_up, SwiGLU-quantise+down "
                               "(M<=16: the three activation quantisers run inside their GEMM launch)",
                       "parallelism": f"tp{world}" if world > 1 else "single GPU",
                       **({"row_parallel_sum": sweep.exchange_note} if world > 1 else {}),
                       "l2": "inputs larger than L2: two weight sets (272 MB) alternate between consecutive M",
                       "launch": note, "seed": SEED},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps, "api": e2e_api,
                    "eager_value": flops_step * e2e_steps / (e2e_eager_ms * 1e-3) / 1e12,
                    "eager_ms_per_step": e2e_eager_ms / e2e_steps},
            "gpu_launches": sweep.launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak,
                         "bracketed": {"achieved": bracketed, "frac": bracketed / hbm_peak},
                         # DRAM bytes per launch: algorithmic bytes of each launch times the read+write ratio its
                         # shape class showed under ncu (`dram_traffic_ratio`), averaged over the step's GEMM launches.
                         "traffic": traffic_sum / len(sweep_rows), "traffic_unit": "bytes per GEMM launch (mean)",
                         "tensor_peak": tensor_peak, "tensor_peak_unit": "TFLOP/s",
                         "tensor_peak_source": "2 x measured bf16 cuBLAS burst (no FP8 peak is measured on this pool)"
                                               if peaks else "2 x fallback bf16 figure",
                         "kernel": "hybrid_gemm_tc_kernel", "peak_source": "of measured" if peaks else "of fallback",
                         "how": "achieved: algorithmic bytes of the 32 GEMM launches of a step / CUDA-event time of "
                                "the whole timed step (quantiser launches included in the time); bracketed: the same "
                                "bytes / sum of the launches' median CUDA-event durations, " + how},
            "sweep": sweep_rows,
            "prefill": [{"gemm": name, "M": m, "us": round(sec * 1e6, 1),
                         "TFLOPs": round(2 * m * stats[name][1] * stats[name][0] / sec / 1e12, 1),
                         "tensor_frac": round(2 * m * stats[name][1] * stats[name][0] / sec / 1e12 / tensor_peak, 3)}
                        for name, m, sec in prefill],
        }
        if not args.no_cpu_baseline and world == 1:
            cpu_reference_sample()
            line["cpu_baseline"], _ = cpu_reference_sample(min_seconds=10.0)
            # The GPU on EXACTLY the CPU sample (qkv + o_proj at 1, 16 and 128 tokens, cold weights), so one
            # like-for-like quotient stands beside the whole-sweep value.
            same = [r for r in sweep_rows if r["gemm"] in ("qkv", "o_proj") and r["M"] in (1, 16, 128)]
            if len(same) == 6:
                gpu_same = sum(2 * r["M"] * r["N"] * r["K"] for r in same) / sum(r["us"] for r in same) / 1e6
                line["cpu_baseline"]["gpu_on_same_sample"] = {"value": gpu_same, "unit": "TFLOP/s",
                                                              "ratio": gpu_same / line["cpu_baseline"]["value"],
                                                              "how": "the six GEMM launches of the sample, cold weights, "
                                                                     "per-launch CUDA-event durations from the step"}
        print(json.dumps(line))
    if world > 1:
        # Graphs that captured NCCL kernels must go before the communicator; a watchdog ends the process
        # if the communicator teardown does not return (the result line is already printed and flushed).
        sys.stdout.flush()
        graph = timed_graph = e2e_graph = None  # noqa: F841
        torch.cuda.synchronize()
        watchdog = threading.Timer(30.0, os._exit, args=(0,))
        watchdog.daemon = True
        watchdog.start()
        dist.barrier()
        dist.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
