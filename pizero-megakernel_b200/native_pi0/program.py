"""Static instruction-stream compiler for the persistent pi0 VM kernel.

Same surface as the reference ``native_pi0/program.py`` (``LinearWork`` ``:7-10``,
``linear_streams`` ``:13-33``, ``program_summary`` ``:36-40``): every stage's
tiles are cut into at most ``workers`` contiguous ranges, and ranges are handed
to the workers that currently carry the least accumulated cost.  An instruction
is 32 int32 words ``[opcode, stage, first_tile, tile_count, 0...]``; opcode 0 is
an empty slot.  Assignment happens once at setup; the device never fetches work
from a shared queue.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

WIDTH = 32          # int32 words per instruction
MAX_WORKERS = 148   # SMs on a B200


@dataclass(frozen=True)
class LinearWork:
    tiles: int
    k: int


def linear_streams(stages, workers):
    """Return ``int32[workers, length, 32]`` streams for a list of ``LinearWork``."""
    if not isinstance(workers, int) or workers < 1 or workers > MAX_WORKERS:
        raise ValueError("Expected 1..148 B200 workers")
    stages = tuple(stages)
    if not stages or any(w.tiles < 1 or w.k < 64 or w.k % 64 for w in stages):
        raise ValueError("Invalid linear stage geometry")
    load = np.zeros(workers, dtype=np.int64)
    rows = [[] for _ in range(workers)]
    for index, work in enumerate(stages):
        parts = min(workers, work.tiles)
        small, extra = divmod(work.tiles, parts)
        # stable sort: ties in cost resolve to the lower worker index
        order = np.argsort(load, kind="stable")[:parts]
        start = 0
        for rank, worker in enumerate(order.tolist()):
            count = small + (1 if rank < extra else 0)
            rows[worker].append((1, index, start, count))
            load[worker] += count * work.k
            start += count
    length = max(len(r) for r in rows)
    code = np.zeros((workers, length, WIDTH), dtype=np.int32)
    for worker, entries in enumerate(rows):
        if entries:
            code[worker, :len(entries), :4] = np.asarray(entries, dtype=np.int32)
    return code


def spread_streams(stages, workers, sources, kinds=None):
    """Streams in the layout of ``linear_streams`` for a chain of short, dependent stages.

    ``linear_streams`` hands each stage to the least loaded workers. A worker that has just run a tile of a stage
    is the last to learn that the next stage may start: it still has to publish, fetch its next instruction and
    issue its first copies, while an idle worker has done all that in advance and only polls a counter (a
    difference of 2-3 microseconds per stage on B200). Here the tiles of a stage go first to workers whose previous
    instruction is NOT one of the stage's sources (``sources[i]``: indices of the stages stage ``i`` waits for);
    among those, to the least loaded, ties to the lower index. Stages with at least as many tiles as workers
    are split exactly as in ``linear_streams``.

    ``kinds`` (optional, one label per stage: the code path its tiles execute): among the workers that are not late,
    those that ran the stage's kind most recently come first, so that a worker keeps to few kinds of instruction and
    its SM's instruction cache to few code paths."""
    if not isinstance(workers, int) or workers < 1 or workers > MAX_WORKERS:
        raise ValueError("Expected 1..148 B200 workers")
    stages = tuple(stages)
    if not stages or len(sources) != len(stages) or any(w.tiles < 1 or w.k < 64 or w.k % 64 for w in stages):
        raise ValueError("Invalid stage geometry")
    load = np.zeros(workers, dtype=np.int64)
    last = np.full(workers, -1, dtype=np.int64)          # the stage of each worker's previous instruction
    rows = [[] for _ in range(workers)]
    index_of = np.arange(workers)
    known = {}                                           # kind -> per worker: the last stage of this kind it ran (-1: none)
    if kinds is not None and len(kinds) != len(stages):
        raise ValueError("Expected one kind per stage")
    for index, work in enumerate(stages):
        parts = min(workers, work.tiles)
        small, extra = divmod(work.tiles, parts)
        src = [s for s in sources[index] if s is not None and s >= 0]
        late = np.isin(last, src).astype(np.int64) if src else np.zeros(workers, dtype=np.int64)
        if kinds is None:
            order = np.lexsort((index_of, load, late))[:parts]        # keys: late first, then load, then index
        else:
            ran = known.setdefault(kinds[index], np.full(workers, -1, dtype=np.int64))
            order = np.lexsort((index_of, load, -ran, late))[:parts]      # late, then most recent run of this kind, load, index
            ran[order] = index
        start = 0
        for rank, worker in enumerate(order.tolist()):
            count = small + (1 if rank < extra else 0)
            rows[worker].append((1, index, start, count))
            load[worker] += count * work.k
            last[worker] = index
            start += count
    length = max(len(r) for r in rows)
    code = np.zeros((workers, length, WIDTH), dtype=np.int32)
    for worker, entries in enumerate(rows):
        if entries:
            code[worker, :len(entries), :4] = np.asarray(entries, dtype=np.int32)
    return code


def program_summary(code):
    code = np.asarray(code)
    used = code[:, :, 0] != 0
    return {
        "workers": int(code.shape[0]),
        "stream_length": int(code.shape[1]),
        "instructions": int(used.sum()),
        "compute_tiles": int(code[:, :, 3][used].sum()),
        "largest_tile_range": int(code[:, :, 3].max()),
        "dynamic_fetch": False,
        "ready_queue": False,
    }


def validate_streams(code, stage_tiles):
    """Host-side static check of a program (the rule the reference applies in
    ``native_pi0/model.cu:263-268``): stage indices never decrease along a worker
    stream and every tile of every stage is covered exactly once."""
    code = np.asarray(code)
    if code.ndim != 3 or code.shape[2] != WIDTH:
        raise ValueError("Program must be int32[workers, length, 32]")
    seen = [np.zeros(t, dtype=np.int32) for t in stage_tiles]
    for worker in range(code.shape[0]):
        last = -1
        ended = False
        for op, stage, first, count in code[worker, :, :4].tolist():
            if op == 0:
                ended = True
                continue
            if ended:
                raise ValueError(f"worker {worker}: instruction after an empty slot")
            if not 0 <= stage < len(stage_tiles) or stage < last:
                raise ValueError(f"worker {worker}: stage order violated at stage {stage}")
            if count < 1 or first < 0 or first + count > stage_tiles[stage]:
                raise ValueError(f"worker {worker}: tile range outside stage {stage}")
            seen[stage][first:first + count] += 1
            last = stage
    for stage, cover in enumerate(seen):
        if not np.all(cover == 1):
            raise ValueError(f"stage {stage}: tiles not covered exactly once")
    return True
