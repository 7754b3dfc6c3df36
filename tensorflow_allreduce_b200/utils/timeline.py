"""Per-collective records as a Chrome-trace timeline (load it in chrome://tracing or Perfetto).

The reference has no tracing of its own; under TensorFlow's `RunOptions.trace_level` an
allreduce shows up as one async op whose span runs from enqueue to completion, negotiation wait
included (`tensorflow/python/client/timeline.py`). Here every collective contributes two spans:
"negotiate" (enqueue -> go-ahead from the coordinator) and "launch"/"run" (go-ahead -> kernel
enqueued on the private stream for CUDA tensors, or ring finished for CPU tensors); an allreduce
in two levels adds its three steps. Records that carry a device time (`set_device_timing`,
`DistributedOptimizer(timing_every=...)`) add a span of that length on a lane per channel
(`tid` 10 + channel), placed at the host time of the launch: the length is measured on the
device, the position is when the host queued it.
"""
from __future__ import annotations

import json
from typing import Iterable, List, Optional

from .. import core


def chrome_trace(records: Optional[Iterable[dict]] = None, pid: Optional[int] = None) -> List[dict]:
    """Chrome-trace events for `records` (default: `stats()` of this process)."""
    recs = list(records) if records is not None else core.stats()
    pid = core.rank() if pid is None and core.is_initialized() else (pid or 0)
    if not recs:
        return []
    t0 = min(r["t_enqueue"] for r in recs)
    ev = []
    for r in recs:
        args = {"bytes": r["bytes"], "algo": r["algo"], "blocks": r["blocks"], "device": "cuda" if r["device"] else "cpu"}
        ev.append({"name": r["name"], "cat": r["op"] + ".negotiate", "ph": "X", "pid": pid, "tid": 0,
                   "ts": (r["t_enqueue"] - t0) * 1e6, "dur": max(0.0, (r["t_negotiated"] - r["t_enqueue"]) * 1e6), "args": args})
        ev.append({"name": r["name"], "cat": r["op"] + (".launch" if r["device"] else ".run"), "ph": "X", "pid": pid, "tid": 1,
                   "ts": (r["t_negotiated"] - t0) * 1e6, "dur": max(0.0, (r["t_done"] - r["t_negotiated"]) * 1e6), "args": args})
        if r.get("device_us", -1) > 0:
            ev.append({"name": r["name"], "cat": r["op"] + ".device", "ph": "X", "pid": pid, "tid": 10 + int(r.get("channel", 0)),
                       "ts": (r["t_done"] - t0) * 1e6, "dur": r["device_us"],
                       "args": dict(args, bus_gbs=round(r.get("bus_gbs", 0.0), 2), link_frac=round(r.get("link_frac", 0.0), 4))})
        if r.get("two_level_s"):
            # an allreduce over several hosts: its three steps, one after the other, on a row of their own
            ts = (r["t_negotiated"] - t0) * 1e6
            for step, sec in zip(("inside the host", "rail between hosts", "gather inside the host"), r["two_level_s"]):
                ev.append({"name": step, "cat": r["op"] + ".two_level", "ph": "X", "pid": pid, "tid": 2, "ts": ts, "dur": sec * 1e6,
                           "args": {"collective": r["name"]}})
                ts += sec * 1e6
    return ev


def dump(path: str, records: Optional[Iterable[dict]] = None) -> None:
    """Write the timeline of this process to `path` as Chrome-trace JSON."""
    with open(path, "w") as f:
        json.dump({"traceEvents": chrome_trace(records), "displayTimeUnit": "ms"}, f)


def summary(records: Optional[Iterable[dict]] = None) -> dict:
    """Counters per (operation, algorithm): calls, bytes, mean negotiation and launch/run time, and
    over the records that were timed on the device their number, mean device time and mean bus GB/s."""
    recs = list(records) if records is not None else core.stats()
    out = {}
    for r in recs:
        k = f'{r["op"]}/{r["algo"]}'
        s = out.setdefault(k, {"calls": 0, "bytes": 0, "negotiation_us": 0.0, "run_us": 0.0, "device_timed": 0, "device_us": 0.0,
                               "bus_gbs": 0.0})
        s["calls"] += 1
        s["bytes"] += r["bytes"]
        s["negotiation_us"] += (r["t_negotiated"] - r["t_enqueue"]) * 1e6
        s["run_us"] += (r["t_done"] - r["t_negotiated"]) * 1e6
        if r.get("device_us", -1) > 0:
            s["device_timed"] += 1
            s["device_us"] += r["device_us"]
            s["bus_gbs"] += r.get("bus_gbs", 0.0)
    for s in out.values():
        s["negotiation_us"] /= s["calls"]
        s["run_us"] /= s["calls"]
        if s["device_timed"]:                       # means over the records that were timed on the device
            s["device_us"] /= s["device_timed"]
            s["bus_gbs"] /= s["device_timed"]
    return out
