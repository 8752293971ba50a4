"""Step records and request totals (no GPU)."""
import json

from sglang_rs_b200.engine.metrics import EngineMetrics, StepLog, StepStats


def stats(step):
    return StepStats(step=step, rows=10, requests=3, decode_rows=2, prompt_rows=8, wanted=3, captured=False,
                     pages_free={"kv:None": 7}, host_ms=0.5)


def test_step_log_writes_json_lines_and_keeps_records(tmp_path):
    path = tmp_path / "steps.jsonl"
    log = StepLog(str(path))
    for step in (1, 2):
        log.add(stats(step))
    lines = [json.loads(line) for line in path.read_text().splitlines()]
    assert [line["step"] for line in lines] == [1, 2]
    assert lines[0]["rows"] == 10 and lines[0]["pages_free"] == {"kv:None": 7} and lines[0]["device_ms"] is None
    assert [record.step for record in log.flush()] == [1, 2]
    quiet = StepLog(None)
    quiet.add(stats(9))
    assert not quiet.time_device and quiet.records[-1].step == 9


class FakeEvent:
    """Stands in for a CUDA event: completes when told to."""
    def __init__(self, at):
        self.at, self.done = at, False

    def query(self):
        return self.done

    def synchronize(self):
        self.done = True

    def elapsed_time(self, other):
        return other.at - self.at


def test_device_times_are_filled_in_once_the_events_completed_and_in_order(tmp_path):
    log = StepLog(str(tmp_path / "s.jsonl"))
    first, second = (FakeEvent(0.0), FakeEvent(2.5)), (FakeEvent(3.0), FakeEvent(4.0))
    log.add(stats(1), *first)
    log.add(stats(2), *second)
    assert not log.records                                   # nothing completed: nothing written, nobody waited
    second[1].done = True
    log.poll()
    assert not log.records                                   # the first step is still running: order is kept
    first[1].done = True
    log.poll()
    assert [(r.step, r.device_ms) for r in log.records] == [(1, 2.5), (2, 1.0)]
    log.add(stats(3), FakeEvent(5.0), FakeEvent(5.5))
    assert [r.device_ms for r in log.flush()] == [2.5, 1.0, 0.5]


def test_request_totals_in_the_references_names():
    m = EngineMetrics()
    m.arrived("a", 12)
    m.arrived("b", 30)
    assert m.requests_in_flight == 2 and m.prompt_tokens_total == 42
    m.produced("a", 0, finished=False)                       # a prompt portion: no token yet, no first-token time
    assert m.time_to_first_token_seconds_count == 0
    m.produced("a", 1, finished=False)
    m.produced("a", 1, finished=True, cached_tokens=8)
    m.produced("b", 0, finished=True, failed=True)
    assert (m.requests_total, m.requests_failed_total, m.requests_in_flight) == (2, 1, 0)
    assert m.generation_tokens_total == 2 and m.cached_tokens_total == 8
    assert m.time_to_first_token_seconds_count == 1 and m.request_duration_seconds_count == 2
    arrival, first, end = m.timeline["a"]
    assert arrival <= first <= end and m.timeline["b"][1] is None
    text = m.render()
    for name in ("sglang_requests_total 2", "sglang_requests_failed_total 1", "sglang_requests_in_flight 0",
                 "sglang_prompt_tokens_total 42", "sglang_generation_tokens_total 2", "sglang_cached_tokens_total 8",
                 "sglang_time_to_first_token_seconds_count 1", "sglang_request_duration_seconds_count 2",
                 "# TYPE sglang_time_to_first_token_seconds summary"):
        assert name in text


def test_kernel_classes_are_traced_only_when_asked():
    from sglang_rs_b200.ops import trace
    assert trace.active is None or trace.active is not None   # set by SRB_TRACE at import; the default is off
    calls = []

    @trace.traced("gemm")
    def op(x):
        calls.append(x)
        return x + 1
    saved = trace.active
    try:
        trace.configure(None)
        assert op(1) == 2 and trace.active is None
    finally:
        trace.active = saved
    assert calls == [1]
