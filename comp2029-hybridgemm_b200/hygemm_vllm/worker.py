"""vLLM worker extension: per-layer audit and timing of pure fixed-batch decode steps.

Counterpart of the reference's `integrations/vllm/hygemm_vllm/worker.py` (same RPC names and the same
result dictionary), written against the worker interface of the vLLM installed with this library
(`Worker.execute_model(scheduler_output)`, `Worker.sample_tokens(grammar_output)`,
`model_runner.cudagraph_dispatcher.dispatch(...) -> (CUDAGraphMode, BatchDescriptor)`).

Use: `LLM(..., worker_extension_cls="hygemm_vllm.worker.AuditWorkerExtension")`, then
`llm.collective_rpc("formal_begin", args=(batch,))`, generate, `llm.collective_rpc("formal_end")`.

What is timed (reference: worker.py:6-11, docs/formal_decode_protocol.md:107-124): every engine step whose
batch is exactly `batch` requests, each scheduled for one token and each past its prompt, from the call of
`execute_model` to the return of `sample_tokens`, with CUDA events and no device synchronisation per step.
`decode_span_ms` runs from the first such step's start to the last one's end and therefore includes the
engine's idle gaps between steps; prefill and mixed steps are excluded.  Every timed step must have been
dispatched to a FULL CUDA graph, otherwise `formal_end` raises.
"""
from __future__ import annotations

EVENT_POOL = 1024


class _DecodeTimer:
    """State of one measurement window and the three hooks installed on a worker."""

    def __init__(self, worker):
        import torch
        from vllm.config import CUDAGraphMode
        self.worker = worker
        self.enabled = False
        self.full_mode = CUDAGraphMode.FULL
        self.events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                       for _ in range(EVENT_POOL)]
        self.execute, self.sample = worker.execute_model, worker.sample_tokens
        self.dispatcher = worker.model_runner.cudagraph_dispatcher
        self.dispatch = self.dispatcher.dispatch
        worker.execute_model, worker.sample_tokens = self.on_execute, self.on_sample
        self.dispatcher.dispatch = self.on_dispatch
        self.reset(0)

    def reset(self, batch):
        self.batch = int(batch)
        self.records, self.prompt_length, self.position = [], {}, {}
        self.pending, self.engine_steps, self.graph_steps = None, 0, 0

    # -- hooks -------------------------------------------------------------------------------------------
    def is_pure_decode(self, scheduled):
        for request in scheduled.scheduled_new_reqs:
            self.prompt_length[request.req_id] = len(request.prompt_token_ids or ())
            self.position[request.req_id] = request.num_computed_tokens
        cached = scheduled.scheduled_cached_reqs
        for req_id, computed in zip(cached.req_ids, cached.num_computed_tokens):
            self.position[req_id] = computed
        tokens = scheduled.num_scheduled_tokens
        if len(tokens) != self.batch:
            return False
        return all(count == 1 and self.position.get(req_id, -1) >= self.prompt_length.get(req_id, 1 << 60)
                   for req_id, count in tokens.items())

    def on_execute(self, scheduled, *args, **kwargs):
        self.pending = None
        if self.enabled:
            if self.is_pure_decode(scheduled):
                if len(self.records) >= len(self.events):
                    raise RuntimeError("Timing event pool exhausted")
                start, stop = self.events[len(self.records)]
                self.pending = [start, stop, [self.position[r] for r in scheduled.num_scheduled_tokens], False]
                start.record()
            self.engine_steps += 1
        return self.execute(scheduled, *args, **kwargs)

    def on_dispatch(self, *args, **kwargs):
        mode, descriptor = self.dispatch(*args, **kwargs)
        if self.enabled and self.pending is not None and mode == self.full_mode and not self.pending[3]:
            self.pending[3] = True
            self.graph_steps += 1
        return mode, descriptor

    def on_sample(self, *args, **kwargs):
        output = self.sample(*args, **kwargs)
        if self.enabled and self.pending is not None:
            start, stop, positions, _ = self.pending
            stop.record()
            self.records.append((start, stop, positions))
            self.pending = None
        return output


class AuditWorkerExtension:
    def hygemm_model_audit(self):
        from .quantization import model_audit
        return model_audit(self.model_runner.model)

    def formal_begin(self, batch):
        import torch
        if not hasattr(self, "_hygemm_timer"):
            self._hygemm_timer = _DecodeTimer(self)
        torch.cuda.synchronize()
        self._hygemm_timer.reset(batch)
        self._hygemm_timer.enabled = True
        return True

    def formal_end(self):
        import torch
        timer = self._hygemm_timer
        timer.enabled = False
        torch.cuda.synchronize()
        rows = timer.records
        if not rows:
            raise RuntimeError("No fixed-batch pure decode steps were recorded")
        if timer.graph_steps != len(rows):
            raise RuntimeError("A measured decode step did not use FULL Graph")
        per_step = [start.elapsed_time(stop) for start, stop, _ in rows]
        span = rows[0][0].elapsed_time(rows[-1][1])
        return {"batch": timer.batch, "steps": len(rows), "graph_steps": timer.graph_steps,
                "total_engine_steps": timer.engine_steps, "decode_span_ms": span,
                "decode_ms_per_step": span / len(rows), "sum_step_gpu_ms": sum(per_step), "step_gpu_ms": per_step,
                "context_min": min(min(p) for _, _, p in rows), "context_max": max(max(p) for _, _, p in rows)}
