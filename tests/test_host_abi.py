"""CPU-side checks: the C-ABI library builds, loads and exports every symbol the header declares (no compute
calls without a GPU), argument validation that needs no device, and the replica plumbing on gloo."""
import ctypes
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def libraries():
    from native_pi0 import _native
    _native.build()
    return ctypes.CDLL(str(_native.LIBRARY)), ctypes.CDLL(str(_native.TRACE_LIBRARY))


def declared_functions():
    text = (ROOT / "include" / "pi0_native.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|const char\*)\s+(\w+)\s*\(", text)))


def test_header_symbols_are_exported(libraries):
    engine, trace = libraries
    names = declared_functions()
    assert len(names) >= 45
    for name in names:
        owner = trace if "launch_trace" in name else engine
        assert hasattr(owner, name), f"{name} declared in include/pi0_native.h but not exported"


def test_every_exported_entry_point_is_declared():
    """The other direction: nothing is exported behind the header's back."""
    declared = set(declared_functions())
    for source in ("pi0_native.cu", "launch_trace.cpp"):
        text = (ROOT / "pizero-megakernel_b200" / "csrc" / source).read_text()
        exported = set(re.findall(r'extern "C"\s+(?:int|const char\*)\s+(\w+)\s*\(', text))
        assert exported and not exported - declared, sorted(exported - declared)


def test_timing_record_width_matches_the_header():
    header = (ROOT / "include" / "pi0_native.h").read_text()
    source = (ROOT / "pizero-megakernel_b200" / "csrc" / "pi0_native.cu").read_text()
    assert "int64 [workers, length, 8]" in header
    assert "static_cast<size_t>(8) * prog->workers * prog->length" in source


def test_loader_signatures_cover_the_header():
    from native_pi0 import _native
    missing = set(declared_functions()) - set(_native.EXPORTS) - {"begin_launch_trace", "end_launch_trace", "launch_trace_error"}
    assert not missing, missing


def test_missing_library_fails_loudly(tmp_path):
    from native_pi0 import _native
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _native.load(tmp_path / "absent.so")


def test_null_handles_need_no_device(libraries):
    engine, _ = libraries
    for name in ("destroy_resident_fp4", "destroy_norm", "destroy_attention", "destroy_op", "destroy_native_model", "destroy_native_linear"):
        fn = getattr(engine, name)
        fn.argtypes, fn.restype = [ctypes.c_void_p], ctypes.c_int
        assert fn(None) == 0
    engine.launch_resident_fp4.argtypes, engine.launch_resident_fp4.restype = [ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int
    assert engine.launch_resident_fp4(None, None) == 1


def test_python_surface_imports_without_cuda():
    import native_pi0
    from native_pi0.calibration import ActivationCalibration  # noqa: F401
    from native_pi0.program import linear_streams  # noqa: F401
    from native_pi0.quantization import pack_nvfp4  # noqa: F401
    from native_pi0.weights import Pi0Config, parameter_shapes
    assert native_pi0.__all__ == ["NativePi0"]
    shapes = parameter_shapes(Pi0Config())
    total = sum(int(torch.tensor(s).prod()) for s, _, _ in shapes.values())
    assert 3.2e9 < total < 3.4e9          # SigLIP 0.41 B + Gemma-2B 2.5 B (incl. embedding) + expert 0.31 B


def test_replica_round_robin():
    from native_pi0.replicas import requests_for
    assert requests_for(0, 2, 5) == [0, 2, 4] and requests_for(1, 2, 5) == [1, 3]
    assert sorted(sum((requests_for(r, 8, 37) for r in range(8)), [])) == list(range(37))
    with pytest.raises(ValueError):
        requests_for(2, 2, 5)


WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch.distributed as dist
from native_pi0.replicas import reduce_stats, requests_for
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
mine = requests_for(rank, world, 9)
lat = [10.0 + rank] * len(mine)          # replica 1 is the slow one
dist.barrier()
out = reduce_stats(lat, 50)
assert out["p50_ms"] == 10.0 + (world - 1), out
assert abs(out["actions_per_s"] - sum(50e3 / (10.0 + r) for r in range(world))) < 1e-6, out
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_replica_statistics_world_size_2_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29531", str(script), str(ROOT / "pizero-megakernel_b200")]
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert result.returncode == 0, result.stdout + result.stderr
    assert result.stdout.count("ok") == 2


def test_bench_reference_arm_prints_one_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU restatement on a bounded sample and prints exactly
    one JSON line on stdout with the keys the benchmark contract names (everything else goes to stderr)."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    run = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=900, cwd=root)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [line for line in run.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "pi0_10step_action_chunk_latency_p50_ms" and line["unit"] == "ms"
    assert line["higher_is_better"] is False and line["n_gpus"] == 1 and line["steps"] == 1 and line["gpu_launches"] == 0
    assert line["value"] > 0 and line["ms_per_step"] == line["value"]
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and line["data"] == "synthetic"
