"""Route trace writer and reader (zerocool_b200/route_trace.py) on a synthetic trace: the event shape and state
machine of the reference's capture (include/engine/route_trace.hpp:10-77) and the reader's consistency checks
(src/engine/bench.cpp:35-41)."""
import json

import numpy as np
import pytest

from zerocool_b200.route_trace import KIND, RouteTrace, read_route_trace

LAYERS, TOPK, EXPERTS = 3, 4, 32


def synthetic_ids(rng, tokens):
    return np.stack([rng.choice(EXPERTS, size=TOPK, replace=False) for _ in range(tokens)]).astype(np.int32)


def test_round_trip_and_event_shape(tmp_path):
    path = tmp_path / "trace.jsonl"
    rng = np.random.default_rng(1)
    want = []
    with RouteTrace(path, {"build": "test", "layers": LAYERS}, LAYERS, TOPK) as trace:
        trace.request_begin("r0", [1, 2, 3], 8)
        for offset, tokens in ((0, 3), (3, 1)):
            trace.begin(7, offset, tokens, phase="prefill" if tokens > 1 else "decode")
            layers = [synthetic_ids(rng, tokens) for _ in range(LAYERS)]
            for layer, ids in enumerate(layers):
                trace.routes(layer, offset, tokens, ids)
            trace.commit(offset + tokens)
            want.append(layers)
        trace.begin(7, 4, 1)                      # an aborted forward leaves no pass
        trace.routes(0, 4, 1, synthetic_ids(rng, 1))
        trace.abort()
        trace.request_end([5], "stop")
        trace.finish()
    rows = [json.loads(line) for line in open(path)]
    assert [r["sequence"] for r in rows] == list(range(1, len(rows) + 1))
    assert all(r["kind"] == KIND and set(r) == {"kind", "sequence", "monotonic_ns", "event", "request_id", "forward_id", "details"} for r in rows)
    assert rows[0]["event"] == "trace_begin" and rows[-1]["event"] == "trace_end" and rows[-1]["details"]["status"] == "complete"
    assert [r["event"] for r in rows].count("routes") == 2 * LAYERS + 1
    passes = read_route_trace(path, LAYERS, TOPK, EXPERTS)
    assert [(p["offset"], p["tokens"], p["phase"]) for p in passes] == [(0, 3, "prefill"), (3, 1, "decode")]
    for got, layers in zip(passes, want):
        assert all(np.array_equal(a, b) for a, b in zip(got["routes"], layers))


def test_state_machine_and_limits(tmp_path):
    path = tmp_path / "t.jsonl"
    trace = RouteTrace(path, {}, LAYERS, TOPK)
    with pytest.raises(RuntimeError, match="new file"):
        RouteTrace(path, {}, LAYERS, TOPK)
    with pytest.raises(RuntimeError):
        trace.begin(1, 0, 1)                      # no request open
    trace.request_begin("r", [], 1)
    trace.begin(1, 0, 2)
    ids = synthetic_ids(np.random.default_rng(2), 2)
    with pytest.raises(RuntimeError):
        trace.routes(1, 0, 2, ids)                # layers arrive in order
    with pytest.raises(RuntimeError):
        trace.routes(0, 0, 2, ids[:1])            # tokens x top_k ids
    trace.routes(0, 0, 2, ids)
    with pytest.raises(RuntimeError):
        trace.commit(2)                           # not all layers captured
    with pytest.raises(RuntimeError):
        trace.finish()                            # a forward is still open
    trace.close()
    rows = [json.loads(line) for line in open(path)]
    assert rows[-1]["event"] == "trace_end" and rows[-1]["details"]["status"] == "incomplete"
    with pytest.raises(ValueError, match="no committed pass"):
        read_route_trace(path, LAYERS, TOPK)


def test_reader_rejects_invalid_selections(tmp_path):
    for name, ids, why in (("dup", [[0, 1, 1, 2]], "repeats"), ("range", [[0, 1, 2, 40]], "outside")):
        path = tmp_path / f"{name}.jsonl"
        with RouteTrace(path, {}, 1, TOPK) as trace:
            trace.request_begin("r", [], 1)
            trace.begin(1, 0, 1)
            trace.routes(0, 0, 1, np.asarray(ids))
            trace.commit(1)
            trace.request_end([], "stop")
            trace.finish()
        with pytest.raises(ValueError, match=why):
            read_route_trace(path, 1, TOPK, EXPERTS)
