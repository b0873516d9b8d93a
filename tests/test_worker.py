"""Decode-step timing extension on fakes (no GPU, no engine): which steps count as pure fixed-batch decode,
the FULL-graph requirement, and the result dictionary of the reference's `formal_end`."""
import types

import pytest
import torch

vllm = pytest.importorskip("vllm")
from hygemm_vllm import worker as W  # noqa: E402


class FakeEvent:
    clock = 0.0

    def __init__(self, enable_timing=True):
        self.at = None

    def record(self):
        FakeEvent.clock += 1.0
        self.at = FakeEvent.clock

    def elapsed_time(self, other):
        return other.at - self.at


class FakeWorker(W.AuditWorkerExtension):
    def __init__(self, full_mode, graph=True):
        self.executed, self.sampled = [], 0
        self.graph = graph
        outer = self

        class Dispatcher:
            def dispatch(self, num_tokens, **kwargs):
                return (full_mode if outer.graph else "NONE"), types.SimpleNamespace(num_tokens=num_tokens)

        self.model_runner = types.SimpleNamespace(cudagraph_dispatcher=Dispatcher(), model=torch.nn.Module())

    def execute_model(self, scheduled):
        self.executed.append(scheduled)
        self.model_runner.cudagraph_dispatcher.dispatch(num_tokens=len(scheduled.num_scheduled_tokens))
        return None

    def sample_tokens(self, grammar_output):
        self.sampled += 1
        return "sampled"


def step(new=(), cached=(), tokens=None):
    return types.SimpleNamespace(
        scheduled_new_reqs=[types.SimpleNamespace(req_id=r, prompt_token_ids=list(range(n)), num_computed_tokens=0) for r, n in new],
        scheduled_cached_reqs=types.SimpleNamespace(req_ids=[r for r, _ in cached], num_computed_tokens=[c for _, c in cached]),
        num_scheduled_tokens=tokens)


@pytest.fixture
def fakes(monkeypatch):
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(W, "EVENT_POOL", 8)
    from vllm.config import CUDAGraphMode
    return CUDAGraphMode.FULL


def test_only_pure_fixed_batch_decode_steps_are_timed(fakes):
    worker = FakeWorker(fakes)
    assert worker.formal_begin(2) is True
    run = lambda s: (worker.execute_model(s), worker.sample_tokens(None))  # noqa: E731
    run(step(new=[("a", 4), ("b", 4)], tokens={"a": 4, "b": 4}))                      # prefill
    run(step(cached=[("a", 4), ("b", 4)], tokens={"a": 1, "b": 1}))                    # decode, context 4
    run(step(cached=[("a", 5), ("b", 5)], tokens={"a": 1, "b": 1}))                    # decode, context 5
    run(step(new=[("c", 3)], cached=[("a", 6)], tokens={"a": 1, "c": 3}))              # mixed step
    run(step(cached=[("a", 7)], tokens={"a": 1}))                                      # wrong batch
    out = worker.formal_end()
    assert (out["batch"], out["steps"], out["graph_steps"], out["total_engine_steps"]) == (2, 2, 2, 5)
    assert (out["context_min"], out["context_max"]) == (4, 5)
    assert out["step_gpu_ms"] == [1.0, 1.0] and out["sum_step_gpu_ms"] == 2.0
    assert out["decode_span_ms"] == 3.0 and out["decode_ms_per_step"] == 1.5
    assert worker.sampled == 5 and len(worker.executed) == 5
    # a second window starts clean and the hooks are installed once
    # (a request whose prefill was not seen inside the window is never counted, as in the reference)
    worker.formal_begin(1)
    run(step(cached=[("a", 8)], tokens={"a": 1}))
    run(step(new=[("d", 3)], tokens={"d": 3}))
    run(step(cached=[("d", 3)], tokens={"d": 1}))
    out = worker.formal_end()
    assert (out["steps"], out["total_engine_steps"], out["context_min"]) == (1, 3, 3)


def test_a_step_outside_a_full_graph_is_refused(fakes):
    worker = FakeWorker(fakes, graph=False)
    worker.formal_begin(1)
    worker.execute_model(step(new=[("a", 2)], tokens={"a": 2}))
    worker.sample_tokens(None)
    with pytest.raises(RuntimeError, match="No fixed-batch pure decode"):
        worker.formal_end()
    worker.formal_begin(1)
    worker.execute_model(step(new=[("b", 2)], tokens={"b": 2}))
    worker.sample_tokens(None)
    worker.execute_model(step(cached=[("b", 2)], tokens={"b": 1}))
    worker.sample_tokens(None)
    with pytest.raises(RuntimeError, match="did not use FULL Graph"):
        worker.formal_end()


def test_event_pool_is_bounded_and_audit_is_exposed(fakes):
    worker = FakeWorker(fakes)
    worker.formal_begin(1)
    worker.execute_model(step(new=[("a", 1)], tokens={"a": 1}))
    for i in range(8):
        worker.execute_model(step(cached=[("a", 1 + i)], tokens={"a": 1}))
        worker.sample_tokens(None)
    with pytest.raises(RuntimeError, match="pool exhausted"):
        worker.execute_model(step(cached=[("a", 20)], tokens={"a": 1}))
    assert worker.hygemm_model_audit() == []
