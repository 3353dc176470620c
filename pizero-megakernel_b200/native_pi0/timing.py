"""Reduction of the per-instruction time stamps of a launch into per-stage figures.

The device records, for every instruction of every worker, eight global-timer values in nanoseconds (start, producers
ready, end, copies issued, first operands landed, MMAs issued, first accumulator ready, last stores done).  The
reference reduces its per-instruction cycle slots the same way (``benchmarks/profile_native_components.py:58-92``):
per stage the number of active workers and the median / maximum duration of its instructions, per operation type the
median over layers, per worker the span between its first and last instruction.  Pure NumPy: usable without a GPU on
recorded stamps.
"""
from __future__ import annotations

import statistics

import numpy as np

START, READY, END = 0, 1, 2


def _valid(stamps, code):
    return (code[:, :, 0] != 0) & (stamps[:, :, READY] > 0) & (stamps[:, :, END] > 0)


def stage_spans(stamps, code, names):
    """[(name, first_ready_ns, last_end_ns, instructions)] per stage that ran, relative to the earliest ready stamp."""
    stamps, code = np.asarray(stamps), np.asarray(code)
    valid = _valid(stamps, code)
    if not valid.any():
        return []
    stage_of = code[:, :, 1]
    start, end = stamps[:, :, READY], stamps[:, :, END]
    origin = start[valid].min()
    first = np.full(len(names), np.iinfo(np.int64).max, dtype=np.int64)
    last = np.zeros(len(names), dtype=np.int64)
    count = np.zeros(len(names), dtype=np.int64)
    np.minimum.at(first, stage_of[valid], start[valid] - origin)
    np.maximum.at(last, stage_of[valid], end[valid] - origin)
    np.add.at(count, stage_of[valid], 1)
    return [(names[i], int(first[i]), int(last[i]), int(count[i])) for i in range(len(names)) if count[i]]


def stage_statistics(stamps, code, names):
    """{stage index: {name, active_workers, instructions, busy_ns_median, busy_ns_max}}: busy = end - producers ready."""
    stamps, code = np.asarray(stamps), np.asarray(code)
    valid = _valid(stamps, code)
    busy = stamps[:, :, END].astype(np.int64) - stamps[:, :, READY].astype(np.int64)
    out = {}
    for stage in np.unique(code[:, :, 1][valid]):
        mask = valid & (code[:, :, 1] == stage)
        out[int(stage)] = {"name": names[int(stage)], "active_workers": int(mask.any(axis=1).sum()), "instructions": int(mask.sum()),
                           "busy_ns_median": int(np.median(busy[mask])), "busy_ns_max": int(busy[mask].max())}
    return out


def operation_report(stamps, code, names):
    """Stages grouped by operation (the last component of the stage name: qkv, attention, o_proj, ...) within each phase
    (the first component): layers, median active workers, median of the stages' median busy time, and the chain time -
    the sum over the stages of (last end of the stage - last end of the stage before it)."""
    stats = stage_statistics(stamps, code, names)
    spans = {name: (first, last) for name, first, last, _ in stage_spans(stamps, code, names)}
    groups, previous_end = {}, None
    for stage in sorted(stats):
        item = stats[stage]
        phase, operation = item["name"].split(".")[0], item["name"].rsplit(".", 1)[-1]
        last = spans[item["name"]][1]
        step = 0 if previous_end is None else max(0, last - previous_end)
        previous_end = last if previous_end is None else max(previous_end, last)
        groups.setdefault((phase, operation), []).append((item, step))
    report = {}
    for (phase, operation), items in groups.items():
        report.setdefault(phase, {})[operation] = {
            "layers": len(items),
            "active_workers_median": statistics.median(i["active_workers"] for i, _ in items),
            "busy_ns_median": statistics.median(i["busy_ns_median"] for i, _ in items),
            "chain_ns_total": int(sum(step for _, step in items)),
        }
    return report


def worker_spans(stamps, code):
    """Nanoseconds between the first start and the last end of every worker that ran anything."""
    stamps, code = np.asarray(stamps), np.asarray(code)
    valid = _valid(stamps, code)
    return [int(stamps[w, valid[w], END].max() - stamps[w, valid[w], START].min()) for w in range(code.shape[0]) if valid[w].any()]
