"""Static stream compiler and calibration records against reference golden outputs."""
import json
import tempfile
from pathlib import Path

import numpy as np
import pytest

from native_pi0.calibration import ActivationCalibration, cache_key, checkpoint_digest, fp32_descale
from native_pi0.program import LinearWork, linear_streams, program_summary, spread_streams, validate_streams


def test_linear_streams_match_reference(golden_dir):
    gold = np.load(golden_dir / "program.npz")
    lists = json.loads((golden_dir / "program.json").read_text())
    for key, lst in lists.items():
        for workers in (1, 20, 148):
            code = linear_streams([LinearWork(t, k) for t, k in lst], workers)
            np.testing.assert_array_equal(code, gold[f"{key}_{workers}"])
            assert validate_streams(code, [t for t, _ in lst])
            s = program_summary(code)
            assert s["compute_tiles"] == sum(t for t, _ in lst)
            assert s["workers"] == workers and not s["dynamic_fetch"]


def test_linear_streams_errors():
    for workers in (0, 149, 1.5):
        with pytest.raises(ValueError):
            linear_streams([LinearWork(1, 64)], workers)
    for bad in ([], [LinearWork(0, 64)], [LinearWork(1, 32)], [LinearWork(1, 96)]):
        with pytest.raises(ValueError):
            linear_streams(bad, 4)


def test_spread_streams_avoid_the_workers_of_a_stage_sources():
    """The latency-oriented scheduler covers every tile exactly once, keeps stage order per worker and never gives a
    worker two consecutive dependent stages while idle workers exist; wide stages are split as by linear_streams."""
    tiles = [7, 40, 104, 16, 7, 128, 16] * 4 + [1536, 96, 7]
    work = [LinearWork(t, 1024) for t in tiles]
    sources = [[i - 1, -1, -1, -1] for i in range(len(tiles))]
    code = spread_streams(work, 148, sources)
    validate_streams(code, tiles)
    assert code.shape[0] == 148 and code.dtype == np.int32
    avoidable = 0
    for worker in range(148):
        stages = [row[1] for row in code[worker, :, :4].tolist() if row[0]]
        avoidable += sum(1 for a, b in zip(stages, stages[1:]) if b == a + 1 and tiles[a] + tiles[b] <= 148)
    assert avoidable == 0
    wide = tiles.index(1536)
    counts = sorted(int(row[3]) for worker in range(148) for row in code[worker, :, :4].tolist() if row[0] and row[1] == wide)
    assert counts[0] == 10 and counts[-1] == 11 and sum(counts) == 1536
    # a chain without declared sources degenerates to the reference policy
    np.testing.assert_array_equal(spread_streams(work, 148, [[-1] * 4] * len(tiles)), linear_streams(work, 148))
    with pytest.raises(ValueError):
        spread_streams(work, 148, sources[:-1])
    with pytest.raises(ValueError):
        spread_streams(work, 0, sources)


def test_spread_streams_keep_workers_to_the_kinds_they_ran():
    """With stage kinds the scheduler still never makes a worker late where it can be avoided, covers every tile once,
    and a worker runs fewer kinds of instruction than without them."""
    names = ["qkv", "attention", "o_proj", "gate_up", "down"]
    tiles = [40, 104, 32, 128, 32] * 12
    kinds = names * 12
    work = [LinearWork(t, 1024) for t in tiles]
    sources = [[i - 1, -1, -1, -1] for i in range(len(tiles))]

    def kinds_per_worker(code):
        validate_streams(code, tiles)
        late = 0
        seen = []
        for worker in range(148):
            stages = [row[1] for row in code[worker, :, :4].tolist() if row[0]]
            late += sum(1 for a, b in zip(stages, stages[1:]) if b == a + 1 and tiles[a] + tiles[b] <= 148)
            seen.append(len({kinds[s] for s in stages[len(stages) // 2:]}))
        assert late == 0
        return sum(seen) / 148.0

    plain = kinds_per_worker(spread_streams(work, 148, sources))
    affine = kinds_per_worker(spread_streams(work, 148, sources, kinds))
    assert affine < plain - 0.5
    with pytest.raises(ValueError):
        spread_streams(work, 148, sources, kinds[:-1])


def test_validator_rejects_corrupt_programs():
    code = linear_streams([LinearWork(10, 64), LinearWork(7, 128)], 4)
    tiles = [10, 7]
    assert validate_streams(code, tiles)
    broken = code.copy()
    broken[0, 0, 3] += 1                       # overlapping coverage
    with pytest.raises(ValueError):
        validate_streams(broken, tiles)
    broken = code.copy()
    broken[1, 0, 0] = 0                        # a missing producer range
    with pytest.raises(ValueError):
        validate_streams(broken, tiles)
    broken = code.copy()
    broken[2, 0, 1], broken[2, 1, 1] = 1, 0    # stage order reversed
    with pytest.raises(ValueError):
        validate_streams(broken, tiles)


def test_calibration_matches_reference(golden_dir):
    gold = json.loads((golden_dir / "calibration.json").read_text())
    c = ActivationCalibration()
    for op, values, sample, step in gold["observations"]:
        c.observe(op, values, sample=sample, step=step)
    assert c.finalize(required_steps=range(4)) == gold["finalize_99_9"]
    assert c.finalize(percentile=50) == gold["finalize_50"]
    assert cache_key("abc", {"views": 3, "steps": 10}, "obs-v1") == gold["cache_key"]
    assert float(fp32_descale(.0123, .0456)) == gold["fp32_descale"]


def test_calibration_known_answers():             # reference test_calibration.py:10-51
    c = ActivationCalibration()
    for sample in ("camera_a", "camera_b"):
        for step in range(10):
            c.observe("expert.0.qkv", [0, -(step + 1) * 448], sample=sample, step=step)
    rec = c.finalize(percentile=100, required_steps=range(10))["expert.0.qkv"]
    assert rec["fp8_scale"] == 10 and rec["per_step_max"]["9"] == 4480
    assert rec["observations"] == 2 and rec["amax_records_above_range"] == 0
    assert c.finalize(percentile=0)["expert.0.qkv"]["fp8_scale"] == 1
    with pytest.raises(ValueError):
        c.finalize(required_steps=range(11))
    with pytest.raises(ValueError):
        c.observe("expert.0.qkv", [1], sample="camera_a", step=0)
    z = ActivationCalibration()
    z.observe("prefix.qkv", [0], sample="zero")
    assert z.finalize()["prefix.qkv"]["fp8_scale"] > 0
    for v in (float("nan"), float("inf")):
        with pytest.raises(ValueError):
            z.observe("bad", [v], sample="bad")
    assert fp32_descale(.0123, .0456) == np.float32(.0123) * np.float32(.0456)
    with pytest.raises(ValueError):
        fp32_descale(1e30, 1e30)


def test_checkpoint_identity():
    with tempfile.TemporaryDirectory() as d:
        p = Path(d) / "model.safetensors"
        p.write_bytes(b"a" * 70000)
        before = checkpoint_digest([p])
        with p.open("r+b") as f:
            f.seek(69999)
            f.write(b"b")
        after = checkpoint_digest([p])
        assert before != after
        k = cache_key(after, {"steps": 10, "views": 3}, "observations-v1")
        assert k == cache_key(after, {"views": 3, "steps": 10}, "observations-v1")
        assert k != cache_key(after, {"steps": 5, "views": 3}, "observations-v1")
        with pytest.raises(ValueError):
            checkpoint_digest([])


def test_timing_reducer_on_recorded_stamps():
    """The per-stage reduction of instruction time stamps (``native_pi0.timing``) on a hand-made recording: three stages
    over four workers, one worker idle, one instruction that never ran (zero stamps)."""
    from native_pi0.timing import operation_report, stage_spans, stage_statistics, worker_spans
    names = ["prefix.0.qkv", "prefix.0.attention", "prefix.1.qkv"]
    code = np.zeros((4, 3, 32), dtype=np.int32)
    stamps = np.zeros((4, 3, 8), dtype=np.int64)

    def put(worker, slot, stage, start, ready, end):
        code[worker, slot, :4] = (1, stage, 0, 1)
        stamps[worker, slot, :3] = (start, ready, end)

    put(0, 0, 0, 1000, 1100, 1600); put(1, 0, 0, 1000, 1150, 1700); put(2, 0, 0, 1000, 1100, 1500)
    put(0, 1, 1, 1600, 1750, 2600); put(1, 1, 1, 1700, 1760, 2900)
    put(2, 1, 2, 1500, 2950, 3300)
    code[2, 2, :4] = (1, 2, 1, 1)                      # scheduled, but no stamps: ignored
    spans = stage_spans(stamps, code, names)
    assert spans == [("prefix.0.qkv", 0, 600, 3), ("prefix.0.attention", 650, 1800, 2), ("prefix.1.qkv", 1850, 2200, 1)]
    stats = stage_statistics(stamps, code, names)
    assert stats[0] == {"name": "prefix.0.qkv", "active_workers": 3, "instructions": 3, "busy_ns_median": 500, "busy_ns_max": 550}
    assert stats[1]["busy_ns_max"] == 1140 and stats[2]["active_workers"] == 1
    report = operation_report(stamps, code, names)
    assert report["prefix"]["qkv"]["layers"] == 2 and report["prefix"]["attention"]["chain_ns_total"] == 1200
    assert report["prefix"]["qkv"]["chain_ns_total"] == 400            # the second qkv ends 400 ns after the attention before it
    assert worker_spans(stamps, code) == [1600, 1900, 2300]
    assert stage_spans(np.zeros_like(stamps), code, names) == []
