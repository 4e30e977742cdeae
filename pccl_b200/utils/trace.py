"""Putting the per-rank instruction traces of ``Engine.trace()`` on one time line.

Every rank records its own Chrome-trace document (process id = rank, thread id = instruction stream).  Host time
stamps of ranks on one machine share a clock; device stamps (``%globaltimer``) and ranks of different machines do not,
so ``merge_traces`` can shift every rank to start at zero, which is enough to compare the shape of the schedules."""
from __future__ import annotations

import json
from typing import Dict, Iterable, List, Optional, Union

Doc = Union[str, Dict]


def _load(d: Doc) -> Dict:
    if isinstance(d, dict):
        return d
    with open(d) as f:
        return json.load(f)


def merge_traces(docs: Iterable[Doc], out: Optional[str] = None, align: bool = False) -> Dict:
    """One document out of several ranks' documents (dicts or paths).  ``align``: subtract each rank's first time
    stamp.  Adds process-name records so that the viewer shows "rank N" instead of a bare number."""
    events: List[Dict] = []
    seen = set()
    for d in docs:
        ev = list(_load(d).get("traceEvents", []))
        if align and ev:
            by_pid: Dict[int, float] = {}
            for e in ev:
                if "ts" in e:
                    by_pid[e["pid"]] = min(by_pid.get(e["pid"], e["ts"]), e["ts"])
            ev = [dict(e, ts=e["ts"] - by_pid[e["pid"]]) if "ts" in e else e for e in ev]
        for e in ev:
            if e.get("pid") not in seen and e.get("ph") != "M":
                seen.add(e.get("pid"))
                events.append({"name": "process_name", "ph": "M", "pid": e.get("pid"), "args": {"name": f"rank {e.get('pid')}"}})
        events.extend(ev)
    doc = {"traceEvents": events, "displayTimeUnit": "ns"}
    if out:
        with open(out, "w") as f:
            json.dump(doc, f)
    return doc


def summarize(doc: Doc) -> Dict[str, Dict[str, float]]:
    """Per instruction kind: count, total microseconds, bytes, and GB/s of the instructions that move data."""
    acc: Dict[str, Dict[str, float]] = {}
    for e in _load(doc).get("traceEvents", []):
        if e.get("ph") != "X":
            continue
        a = acc.setdefault(e["name"], {"count": 0, "us": 0.0, "bytes": 0})
        a["count"] += 1
        a["us"] += float(e.get("dur", 0.0))
        a["bytes"] += int(e.get("args", {}).get("bytes", 0))
    for a in acc.values():
        a["gbs"] = a["bytes"] / a["us"] / 1e3 if a["us"] > 0 and a["bytes"] else 0.0
    return acc


__all__ = ["merge_traces", "summarize"]
