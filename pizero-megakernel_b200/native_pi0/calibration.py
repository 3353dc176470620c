"""Offline activation calibration records and cache identities.

Drop-in for the reference ``native_pi0/calibration.py`` (``checkpoint_digest``
``:15-27``, ``cache_key`` ``:30-36``, ``ActivationCalibration`` ``:39-83``,
``fp32_descale`` ``:86-92``).  Nothing here runs during inference: the engine
reads the finished per-operation scales at setup.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

_DIGEST_TAG = b"native-pi0-checkpoint-v1\0"
_CHUNK = 8 << 20


def _file_sha256(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            block = f.read(_CHUNK)
            if not block:
                break
            h.update(block)
    return h.digest()


def checkpoint_digest(files):
    """SHA-256 over (name, content hash) of every shard, in name order."""
    paths = sorted(Path(f) for f in files)
    names = [p.name for p in paths]
    if not paths or len(set(names)) != len(names):
        raise ValueError("Supply nonempty checkpoint files with unique names")
    outer = hashlib.sha256(_DIGEST_TAG)
    for p in paths:
        outer.update(p.name.encode() + b"\0" + _file_sha256(p))
    return outer.hexdigest()


def cache_key(checkpoint, config, dataset_digest):
    if not checkpoint or not dataset_digest:
        raise ValueError("Checkpoint and observation dataset identities are required")
    body = json.dumps({"version": 1, "checkpoint": checkpoint, "config": config,
                       "dataset": dataset_digest},
                      sort_keys=True, separators=(",", ":"), allow_nan=False)
    return hashlib.sha256(body.encode()).hexdigest()


class ActivationCalibration:
    """Collects one |max| per (operation, observation, denoising step)."""

    def __init__(self):
        self._amax = {}          # operation -> {(sample, step): amax}

    def observe(self, operation, values, *, sample, step=None):
        arr = np.asarray(values, dtype=np.float32)
        if not isinstance(operation, str) or not operation:
            raise ValueError("Operation name is required")
        if arr.size == 0 or not np.all(np.isfinite(arr)):
            raise ValueError("Calibration activations must be nonempty and finite")
        if not isinstance(sample, str) or not sample:
            raise ValueError("Observation identity is required")
        if step is not None and not (isinstance(step, int) and step >= 0):
            raise ValueError("Denoising step must be nonnegative")
        table = self._amax.setdefault(operation, {})
        if (sample, step) in table:
            raise ValueError("Duplicate operation/observation/step record")
        table[(sample, step)] = float(np.max(np.abs(arr)))

    def finalize(self, *, percentile=99.9, required_steps=None):
        if not self._amax or not 0 <= percentile <= 100:
            raise ValueError("Nonempty calibration and percentile in [0,100] required")
        need = None if required_steps is None else set(required_steps)
        report = {}
        for operation in sorted(self._amax):
            table = self._amax[operation]
            stepped = sorted({st for _, st in table if st is not None})
            if stepped and need is not None:
                by_sample = {}
                for smp, st in table:
                    by_sample.setdefault(smp, set()).add(st)
                for smp, have in by_sample.items():
                    if have != need:
                        raise ValueError(f"Incomplete denoising coverage for {operation}/{smp}")
            amax = np.fromiter(table.values(), dtype=np.float64, count=len(table))
            chosen = np.float32(np.percentile(amax, percentile))
            scale = np.float32(max(float(chosen) / 448, 1e-12))
            report[operation] = {
                "fp8_scale": float(scale),
                "percentile": percentile,
                "selected_amax": float(chosen),
                "max_amax": float(amax.max()),
                "records": len(table),
                "observations": len({smp for smp, _ in table}),
                "amax_records_above_range": int(np.count_nonzero(amax > float(scale) * 448)),
                "per_step_max": {str(st): max(v for (_, s2), v in table.items() if s2 == st)
                                 for st in stepped},
            }
        return report


def fp32_descale(activation_scale, weight_scale):
    a = np.float32(activation_scale)
    w = np.float32(weight_scale)
    with np.errstate(over="ignore", invalid="ignore"):
        product = np.float32(a * w)
    if not np.isfinite(product) or min(a, w, product) <= 0:
        raise ValueError("Descale factors must be finite and positive")
    return product


# ---------------------------------------------------------------------------------------------------------------
# Extensions: from a finished calibration to the engine's per-site operand formats, and a file cache for it.
NVFP4_AMAX_LIMIT = 6.0 * 448.0          # largest magnitude an NVFP4 block can hold with tensor scale 1 (E2M1 6 x E4M3 448)


def site_precisions(report, *, sensitive=("*.qkv",), amax_limit=NVFP4_AMAX_LIMIT, default="nvfp4"):
    """Precision dict for ``NativePi0(precision=...)`` from ``ActivationCalibration.finalize()``.

    ``sensitive`` site patterns run on BF16 operands regardless of statistics (query / key projections lose the most
    under 4-bit operands: their error moves the softmax).  Every calibrated operation whose selected |max| exceeds
    ``amax_limit`` - it would saturate an NVFP4 block at tensor scale 1 - runs in BF16 as well.  Operation names are the
    engine's site names (``prefix.3.down``, ``expert.7.qkv``, ...)."""
    chosen = {pattern: "bf16" for pattern in sensitive}
    for operation in sorted(report):
        if float(report[operation]["selected_amax"]) > amax_limit:
            chosen[operation] = "bf16"
    chosen["default"] = default
    return chosen


def cached_calibration(directory, key, build):
    """``build()`` -> report, stored as ``<directory>/<key>.json`` and read back on the next call with the same key
    (``cache_key`` of checkpoint digest, engine configuration and observation set)."""
    path = Path(directory) / f"{key}.json"
    if path.exists():
        return json.loads(path.read_text())
    report = build()
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(report, sort_keys=True, indent=1))
    return report
