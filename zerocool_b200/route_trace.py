"""Route trace: the per-layer expert selections of a forward pass as a JSON-lines file, and its reader.

Mirrors the reference's coordinator-side capture (include/engine/route_trace.hpp:10-77): one line per event with
the fields ``kind`` ("qwen_route_trace_v1"), ``sequence``, ``monotonic_ns``, ``event``, ``request_id``,
``forward_id`` and ``details``; the events ``trace_begin``, ``request_begin``, ``forward_begin``, ``routes`` (one per
layer, in layer order: ``{"layer": l, "routes": [tokens x top_k ids]}``), ``forward_commit`` / ``forward_abort``,
``request_end``, ``cache_reset`` and ``trace_end``; the same state machine (a route is tentative until its forward is
committed) and the same limits (a new file only, at most 20000 events, 64 KiB per line, 16 MiB per trace). The layer
count and top-k, compile-time constants in the reference, come from the caller.

The reader returns the committed passes, which `bench.py --replay-routes` and `Moe.moe_routed` replay
(src/engine/bench.cpp:43-104 does the same with the reference's expert executor).
"""
import json
import os
import time

import numpy as np

KIND = "qwen_route_trace_v1"
MAX_EVENTS, MAX_LINE, MAX_BYTES, MAX_POSITION = 20000, 65536, 16 << 20, 8192


class RouteTrace:
    def __init__(self, path, identity, layers, top_k):
        self.layers, self.top_k = int(layers), int(top_k)
        try:
            fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        except FileExistsError:
            raise RuntimeError(f"route trace must be a new file: {path}") from None
        self._stream = os.fdopen(fd, "w")
        self._sequence = self._bytes = self._request_id = self._forward_id = 0
        self._offset = self._tokens = self._next_layer = 0
        self._request = self._forward = self._terminal = False
        try:
            self._emit("trace_begin", {"identity": identity})
        except Exception:
            self._stream.close()
            self._stream = None
            raise

    # -- events ---------------------------------------------------------------------------------------
    def request_begin(self, name, prompt, max_tokens, prime=False):
        if self._request or self._forward or self._terminal:
            raise RuntimeError("route request already active")
        self._request = True
        self._request_id += 1
        self._emit("request_begin", {"name": name, "input_token_ids": [int(t) for t in prompt], "max_tokens": int(max_tokens), "prime": bool(prime)})

    def request_end(self, output, reason, reused=0):
        if not self._request or self._forward or self._terminal:
            raise RuntimeError("route request not complete")
        self._emit("request_end", {"output_token_ids": [int(t) for t in output], "finish_reason": reason, "reused_tokens": int(reused)})
        self._request = False

    def begin(self, session, offset, tokens, phase="decode", slots=0, input_token_ids=None):
        """Start of one forward pass over `tokens` tokens at position `offset` (input_token_ids optional: the MoE path has none)."""
        if not self._request or self._forward or self._terminal or tokens < 1 or offset + tokens > MAX_POSITION or not session:
            raise RuntimeError("invalid route forward start")
        self._forward = True
        self._forward_id += 1
        self._next_layer, self._offset, self._tokens = 0, int(offset), int(tokens)
        self._emit("forward_begin", {"session_id": str(session), "offset": int(offset), "tokens": int(tokens),
                                     "input_token_ids": [] if input_token_ids is None else [int(t) for t in input_token_ids],
                                     "request_phase": phase, "expert_slots": int(slots)})

    def routes(self, layer, offset, tokens, selected):
        selected = np.asarray(selected).reshape(-1)
        if (not self._forward or self._terminal or layer != self._next_layer or layer >= self.layers or offset != self._offset
                or tokens != self._tokens or selected.size != tokens * self.top_k):
            raise RuntimeError("route pass does not match active forward")
        self._emit("routes", {"layer": int(layer), "routes": [int(v) for v in selected]})
        self._next_layer += 1

    def commit(self, position):
        if not self._forward or self._terminal or self._next_layer != self.layers or position != self._offset + self._tokens:
            raise RuntimeError("route forward did not complete all layers")
        self._emit("forward_commit", {"position": int(position)})
        self._forward = False

    def abort(self):
        if self._forward and not self._terminal:
            self._emit("forward_abort", {"captured_layers": self._next_layer})
            self._forward = False

    def cache_reset(self):
        self._emit("cache_reset", {})

    def finish(self):
        if self._request or self._forward or self._terminal:
            raise RuntimeError("route trace is incomplete")
        self._emit("trace_end", {"status": "complete"})
        self._terminal = True
        self.close()

    def close(self):
        if self._stream is not None:
            if not self._terminal:
                try:
                    self._emit("trace_end", {"status": "incomplete"})
                except Exception:
                    pass
            self._stream.close()
            self._stream = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _emit(self, event, details):
        if self._sequence >= MAX_EVENTS:
            raise RuntimeError("route trace event limit exceeded")
        line = json.dumps({"kind": KIND, "sequence": self._sequence + 1, "monotonic_ns": time.monotonic_ns(), "event": event,
                           "request_id": self._request_id, "forward_id": self._forward_id, "details": details}, separators=(",", ":")) + "\n"
        if len(line) > MAX_LINE or self._bytes + len(line) > MAX_BYTES:
            raise RuntimeError("route trace byte limit exceeded")
        self._stream.write(line)
        self._stream.flush()
        self._sequence += 1
        self._bytes += len(line)


def read_route_trace(path, layers, top_k, experts=None):
    """Committed forward passes of a trace: a list of dicts(offset, tokens, phase, routes=[layers x int32 [tokens, top_k]]).
    Raises ValueError on a malformed trace (wrong kind, gaps in the sequence, a pass that is not `layers` consistent
    layers, ids outside the expert range or repeated inside a token)."""
    passes, current, sequence = [], None, 0
    with open(path) as f:
        for raw in f:
            if not raw.strip():
                continue
            row = json.loads(raw)
            sequence += 1
            if row.get("kind") != KIND or row.get("sequence") != sequence:
                raise ValueError("not a route trace, or events are missing")
            event, d = row["event"], row["details"]
            if event == "forward_begin":
                current = dict(offset=int(d["offset"]), tokens=int(d["tokens"]), phase=d.get("request_phase", ""), routes=[], forward_id=row["forward_id"])
            elif event == "routes":
                if current is None or row["forward_id"] != current["forward_id"] or d["layer"] != len(current["routes"]):
                    raise ValueError("route trace is not a consistent pass")
                ids = np.asarray(d["routes"], np.int32)
                if ids.size != current["tokens"] * top_k:
                    raise ValueError("route row does not hold tokens x top_k ids")
                ids = ids.reshape(current["tokens"], top_k)
                if experts is not None and (ids.min() < 0 or ids.max() >= experts):
                    raise ValueError("invalid recorded selection: expert id outside the model")
                if any(len(set(r)) != top_k for r in ids.tolist()):
                    raise ValueError("invalid recorded selection: an expert repeats inside a token")
                current["routes"].append(ids)
            elif event == "forward_commit":
                if current is None or len(current["routes"]) != layers or d["position"] != current["offset"] + current["tokens"]:
                    raise ValueError(f"route trace is not a consistent {layers}-layer pass")
                passes.append(current)
                current = None
            elif event == "forward_abort":
                current = None
    if not passes:
        raise ValueError("route trace holds no committed pass")
    return passes
