"""Whole-model GPU tests: one persistent launch against the oracle, replay, partitioned launches, launch
counting, chained GEMM programs with counters, and a clean device-side timeout.

Tolerances.  NVFP4 is not a contraction: a perturbation of 1e-3 ahead of a quantiser moves ~0.5 % of the codes
by a whole step, so two correct implementations drift apart layer by layer until they differ by about the
quantisation noise itself.  The per-operator tests (test_gpu_ops.py) are the tight ones; here the gates are
action NRMSE <= 0.1 against the dequantised-NVFP4 emulation and <= 1.3 x the emulation's own distance from
the BF16 eager model.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from native_pi0 import _native
from native_pi0.linear import NativeLinearProgram
from native_pi0.model import EngineCache, NativePi0
from native_pi0.primitives import ResidentNVFP4
from native_pi0.quantization import PackedNVFP4, pack_nvfp4, unswizzle_scales
from native_pi0.weights import Pi0Config, StateDictModel
from oracle import nvfp4 as oracle
from oracle.pi0_torch import Pi0Dims, Pi0Torch, init_state_dict

SMALL = dict(vision_layers=2, prefix_layers=3, expert_layers=2, mlp=2048, expert_mlp=1024, vocab=1024)


def nrmse(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def inputs(views, chunk, prompt, vocab, seed=7):
    g = torch.Generator(device="cpu").manual_seed(seed)
    images = (torch.rand(views, 224, 224, 3, generator=g) * 2 - 1).cuda()
    state = torch.randn(1, 32, generator=g).cuda()
    noise = torch.randn(1, chunk, 32, generator=g).cuda()
    tokens = torch.randint(0, vocab, (1, prompt), generator=g).cuda()
    return images, state, noise, tokens


@pytest.fixture(scope="module")
def small_model():
    dims, cfg = Pi0Dims(**SMALL), Pi0Config(**SMALL)
    sd = init_state_dict(dims, seed=101, device="cuda")
    return dims, cfg, sd


@pytest.mark.parametrize("views,chunk,prompt", [(3, 50, 0), (3, 63, 16), (1, 7, 3)])
def test_forward_matches_oracle(small_model, views, chunk, prompt):
    dims, cfg, sd = small_model
    x = inputs(views, chunk, prompt, dims.vocab)
    emulation = Pi0Torch(dims, sd, mode="nvfp4").sample_actions(*x)
    eager = Pi0Torch(dims, sd, mode="bf16").sample_actions(*x)
    with NativePi0.from_model(StateDictModel(cfg, sd), num_views=views, prompt_len=prompt, chunk_size=chunk) as engine:
        out = engine.forward(*x).clone()
        assert engine.status()["code"] == 0
        assert out.shape == (1, chunk, 32) and out.dtype == torch.float32 and torch.isfinite(out).all()
        assert nrmse(out, emulation) <= 0.1
        assert nrmse(out, eager) <= 1.3 * max(nrmse(emulation, eager), 0.05)
        # same inputs again: bit-exact; the returned tensor is the reused output buffer
        again = engine.forward(*x)
        assert again.data_ptr() == engine.output.data_ptr() and torch.equal(again, out)
        # changed noise changes the result and is still within the gate
        x2 = (x[0], x[1], torch.randn_like(x[2]), x[3])
        out2 = engine.forward(*x2).clone()
        assert not torch.equal(out2, out)
        assert nrmse(out2, Pi0Torch(dims, sd, mode="nvfp4").sample_actions(*x2)) <= 0.1
        assert engine.epoch == 3 and engine.precision_policy == "nvfp4"
        assert engine.plan["compute_tiles"] == sum(engine.stage_tiles)
        assert set(engine.component_ranges) == {"vision", "prefix", "expert"}


@pytest.mark.parametrize("precision,policy", [("bf16", "bf16_reference"), ({"*.qkv": "bf16"}, "mixed"),
                                              ({"default": "bf16", "vision.*": "nvfp4", "expert.*.down": "nvfp4"}, "mixed")])
def test_site_precisions(small_model, precision, policy):
    """Operand format chosen site by site: the engine against the oracle emulating the same choice.  With every site in
    BF16 the engine has to meet the reference's own action gate against BF16 eager (``scripts/validate_native_pi0.py
    :149-150``: NRMSE <= 2 BF16 eps, max error <= 0.0625 RMS, cosine >= 0.999)."""
    dims, cfg, sd = small_model
    x = inputs(3, 50, 16, dims.vocab)
    emulation = Pi0Torch(dims, sd, mode="nvfp4", precision=precision).sample_actions(*x)
    eager = Pi0Torch(dims, sd, mode="bf16").sample_actions(*x)
    with NativePi0(StateDictModel(cfg, sd), prompt_len=16, precision=precision) as engine:
        out = engine.forward(*x).clone()
        assert engine.status()["code"] == 0 and engine.precision_policy == policy
        assert torch.equal(engine.forward(*x), out)
        formats = set(engine.site_precisions.values())
    assert formats == ({"bf16"} if policy == "bf16_reference" else {"bf16", "nvfp4"})
    if policy == "bf16_reference":
        assert nrmse(out, emulation) <= 0.0156
        assert nrmse(out, eager) <= 0.015625
        assert float((out - eager).abs().max() / eager.square().mean().sqrt()) <= 0.0625
        assert float(torch.nn.functional.cosine_similarity(out.flatten(), eager.flatten(), dim=0)) >= 0.999
    else:
        assert nrmse(out, emulation) <= 0.1
        assert nrmse(out, eager) <= 1.3 * max(nrmse(emulation, eager), 0.05)


def test_checkpoint_file_and_calibrated_precisions(small_model, tmp_path):
    """The checkpoint path: a ``model.safetensors`` with OpenPI parameter names is read by ``from_openpi`` (dimensions
    from the tensors) and gives the same bits as the in-memory state dict; a BF16 engine records activation maxima for
    two observations, and the finished calibration picks the operand formats of the serving engine (cached by key)."""
    from safetensors.torch import save_file
    from native_pi0.calibration import ActivationCalibration, cache_key, cached_calibration, checkpoint_digest, site_precisions
    dims, cfg, sd = small_model
    path = tmp_path / "model.safetensors"
    save_file({k: v.contiguous() for k, v in sd.items()}, str(path))
    x = inputs(3, 50, 0, dims.vocab)
    with NativePi0.from_openpi(tmp_path) as loaded, NativePi0(StateDictModel(cfg, sd)) as direct:
        assert loaded.config.vision_layers == cfg.vision_layers and loaded.config.mlp == cfg.mlp and loaded.config.expert_mlp == cfg.expert_mlp
        assert torch.equal(loaded.forward(*x), direct.forward(*x))

    def observe():
        record = ActivationCalibration()
        with NativePi0.from_openpi(path, precision="bf16", flow_steps=3) as reference:
            for n in range(2):
                reference.calibrate(record, f"observation-{n}", *inputs(3, 50, 0, dims.vocab, seed=40 + n))
            assert reference.status()["code"] == 0
        return record.finalize(required_steps=range(3))

    key = cache_key(checkpoint_digest([path]), {"views": 3, "chunk": 50, "steps": 3}, "two-synthetic-observations")
    report = cached_calibration(tmp_path / "calibration", key, observe)
    assert report == cached_calibration(tmp_path / "calibration", key, lambda: pytest.fail("cache miss"))
    assert "expert.1.down" in report and report["expert.1.down"]["records"] == 6 and "prefix.0.o_proj" in report
    chosen = site_precisions(report)
    assert chosen["*.qkv"] == "bf16" and chosen["default"] == "nvfp4"
    forced = site_precisions(report, amax_limit=0.5 * report["prefix.1.down"]["selected_amax"])
    assert forced["prefix.1.down"] == "bf16"
    with NativePi0.from_openpi(path, precision=chosen) as engine:
        out = engine.forward(*x)
        assert engine.status()["code"] == 0 and engine.precision_policy == "mixed" and torch.isfinite(out).all()
        assert engine.site_precisions["prefix.0.qkv"] == "bf16" and engine.site_precisions["prefix.0.down"] == "nvfp4"


def test_engine_cache_shares_weights_between_shapes(small_model):
    """Several (views, prompt, chunk) shapes over one weight store: same bits as engines built alone, one packed copy of
    every weight, least recently used shape evicted."""
    dims, cfg, sd = small_model
    shapes = [(3, 0, 50), (3, 16, 63), (1, 3, 7)]
    with EngineCache(StateDictModel(cfg, sd), capacity=2) as cache:
        first = cache.get(*shapes[0])
        packed = len(cache.weights)
        second = cache.get(*shapes[1])
        assert len(cache.weights) == packed and cache.get(*shapes[0]) is first               # no weight was packed a second time
        for shape, engine in ((shapes[0], first), (shapes[1], second)):
            x = inputs(shape[0], shape[2], shape[1], dims.vocab)
            with NativePi0(StateDictModel(cfg, sd), num_views=shape[0], prompt_len=shape[1], chunk_size=shape[2]) as alone:
                assert torch.equal(engine.forward(*x), alone.forward(*x))
        third = cache.get(*shapes[2])                       # capacity 2: the least recently used shape (the second) is closed
        assert not second.handle.value and first.handle.value and third.handle.value
        assert set(cache.engines) == {shapes[0], shapes[2]}


def test_norm_stages_instead_of_folded_norms(small_model):
    """``fold_norms=False`` keeps every RMSNorm as a stage of its own (normalised rows are quantised, plain weights):
    more stages, and agreement with the oracle emulating that arithmetic."""
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    emulation = Pi0Torch(dims, sd, mode="nvfp4", fold_norms=False).sample_actions(*x)
    with NativePi0(StateDictModel(cfg, sd), fold_norms=False) as plain, NativePi0(StateDictModel(cfg, sd)) as folded:
        out = plain.forward(*x).clone()
        assert plain.status()["code"] == 0
        assert len(plain.stages) > len(folded.stages)
        assert any(n.endswith("norm2") for n in plain.stage_names) and not any(n.endswith("norm2") for n in folded.stage_names)
    assert nrmse(out, emulation) <= 0.1


@pytest.mark.parametrize("engine_kw,oracle_kw", [
    (dict(fold_layernorms=False), dict(fold_layernorms=False)),                      # SigLIP norms as stages, RMSNorms folded
    (dict(attention_path="mma.sync"), dict(head_blocks=False)),                      # quantiser stage behind the SigLIP attention
    (dict(expert_block_n=64, vision_block_n=128), dict()),                           # one tile width everywhere
    (dict(expert_block_n={"qkv": 32, "o_proj": 32, "gate_up": 64, "down": 32}), dict()),
])
def test_engine_options_against_their_emulation(small_model, engine_kw, oracle_kw):
    """Constructor options that change the arithmetic (what is quantised where) agree with the oracle run the same way;
    options that only change the tiling agree with the default oracle."""
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    emulation = Pi0Torch(dims, sd, mode="nvfp4", **oracle_kw).sample_actions(*x)
    with NativePi0(StateDictModel(cfg, sd), **engine_kw) as engine:
        out = engine.forward(*x).clone()
        assert engine.status()["code"] == 0
        names = engine.stage_names
    assert torch.isfinite(out).all() and nrmse(out, emulation) <= 0.1
    if engine_kw.get("fold_layernorms") is False:
        assert sum(n.endswith(".ln1") or n.endswith(".ln2") for n in names) == 2 * cfg.vision_layers
    if engine_kw.get("attention_path") == "mma.sync":
        assert any(n.endswith("attention_quant") for n in names)


def test_partitioned_and_stage_range_launches_are_bit_exact(small_model):
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    with NativePi0(StateDictModel(cfg, sd)) as one, NativePi0(StateDictModel(cfg, sd), partitioned=True) as three:
        a = one.forward(*x).clone()
        b = three.forward(*x).clone()
        assert torch.equal(a, b)
        # every stage as its own launch
        for s in range(len(one.stages)):
            one.launch_range(s, s + 1, *x, new_epoch=(s == 0))
        assert one.status()["code"] == 0
        assert torch.equal(one.output, a)


def test_schedules_and_split_counts_agree(small_model):
    """Which worker runs which tile never changes a bit of the result: the reference's least-loaded policy and the
    source-avoiding one give identical actions. The number of KV splits changes the order of the softmax sums (and the
    BF16 partial rows), so different split counts agree only to the NVFP4 noise gate."""
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    with NativePi0(StateDictModel(cfg, sd), schedule="spread") as spread, NativePi0(StateDictModel(cfg, sd), schedule="linear") as linear, \
            NativePi0(StateDictModel(cfg, sd)) as affine:
        a = spread.forward(*x).clone()
        b = linear.forward(*x).clone()
        c = affine.forward(*x).clone()
        assert spread.status()["code"] == 0 and linear.status()["code"] == 0 and affine.status()["code"] == 0
        assert affine.schedule == "affine"
        assert not np.array_equal(spread.code, linear.code) and not np.array_equal(spread.code, affine.code)
        assert torch.equal(a, b) and torch.equal(a, c)
    with NativePi0(StateDictModel(cfg, sd), expert_splits=4, prefix_splits=1) as other:
        c = other.forward(*x).clone()
        assert other.status()["code"] == 0
        assert nrmse(c, a) <= 0.1
    with pytest.raises(ValueError):
        NativePi0(StateDictModel(cfg, sd), schedule="random")


def test_progress_marks_come_from_the_full_kernel_variant(small_model):
    """Progress marks are off by default and the all-NVFP4 program launches the lean kernel variant; with marks on the
    same program launches the full variant, gives the same bits, and every warp of every worker ends on the last
    teardown mark."""
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    with NativePi0(StateDictModel(cfg, sd)) as engine:
        lib = engine.lib
        assert engine.plan["kernel"] == "lean"
        a = engine.forward(*x).clone()
        lean = C.c_int(-1)
        _native.check(lib.enable_native_model_debug(engine.handle, 1), "marks on")
        _native.check(lib.native_model_kernel_variant(engine.handle, C.byref(lean)), "variant")
        assert lean.value == 0
        b = engine.forward(*x).clone()
        torch.cuda.synchronize()
        assert engine.status()["code"] == 0 and torch.equal(a, b)
        marks = (C.c_int * (engine.workers * 8))()
        _native.check(lib.read_native_model_debug(engine.handle, marks, len(marks)), "marks")
        assert set(marks) == {900004}
        _native.check(lib.enable_native_model_debug(engine.handle, 0), "marks off")
        _native.check(lib.native_model_kernel_variant(engine.handle, C.byref(lean)), "variant")
        assert lean.value == 1
        assert torch.equal(engine.forward(*x), a)


def test_single_launch_is_counted_by_cupti(small_model):
    from native_pi0.launch_trace import LaunchTrace
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    with NativePi0(StateDictModel(cfg, sd)) as engine:
        engine.forward(*x)
        torch.cuda.synchronize()
        try:
            with LaunchTrace() as trace:
                engine.forward(*x)
                torch.cuda.synchronize()
        except RuntimeError as error:            # CUPTI not available to this process
            pytest.skip(str(error))
        assert trace.count == 1
        assert "pi0_vm_kernel" in trace.symbol


def test_input_validation_and_capture_rejection(small_model):
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    with pytest.raises(ValueError):
        NativePi0(StateDictModel(cfg, sd), precision="fp8")
    with pytest.raises(ValueError):
        NativePi0(StateDictModel(cfg, sd), precision={"*.qkv": "int4"})
    with pytest.raises(ValueError):
        NativePi0(StateDictModel(cfg, sd), num_views=4)
    with NativePi0(StateDictModel(cfg, sd)) as engine:
        with pytest.raises(ValueError):
            engine.forward(x[0][:2], x[1], x[2], x[3])
        with pytest.raises(ValueError):
            engine.forward(x[0].double(), x[1], x[2], x[3])
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with pytest.raises(RuntimeError, match="900"):
                with torch.cuda.graph(graph, stream=stream):
                    engine.forward(*x)
        torch.cuda.synchronize()
        host = engine.sample_actions(*[t.cpu() for t in x])
        assert host.device.type == "cpu" and torch.equal(host.cuda(), engine.forward(*x))
    with pytest.raises(RuntimeError):
        engine.forward(*x)


def test_device_wait_timeout_is_reported_not_hung(small_model):
    """A wait that cannot be satisfied in time ends with a status word; the context and the handle stay usable."""
    dims, cfg, sd = small_model
    x = inputs(3, 50, 0, dims.vocab)
    with NativePi0(StateDictModel(cfg, sd)) as engine:
        good = engine.forward(*x).clone()
        _native.check(engine.lib.set_native_model_wait_budget(engine.handle, 20_000), "budget")    # 20 microseconds
        engine.forward(*x)
        status = engine.status()
        assert status["code"] in (1, 2) and status["aborted"] == 1
        assert -1 <= status["stage"] < len(engine.stages)
        _native.check(engine.lib.set_native_model_wait_budget(engine.handle, 2_000_000_000), "budget")
        assert torch.equal(engine.forward(*x), good)
        assert engine.status()["code"] == 0


def test_chained_gemm_program_counters():
    """Two NVFP4 projections in one launch: stage 1 consumes the packed output of stage 0 band by band."""
    rng = np.random.default_rng(31)
    m, k, n0, n1 = 256, 512, 1024, 384
    a = rng.normal(size=(m, k)).astype(np.float32)
    w0 = rng.normal(scale=0.05, size=(n0, k)).astype(np.float32)
    w1 = rng.normal(scale=0.05, size=(n1, n0)).astype(np.float32)
    pa, p0, p1 = pack_nvfp4(a), pack_nvfp4(w0, scale_policy="ceil"), pack_nvfp4(w1, scale_policy="ceil")
    placeholder = pack_nvfp4(np.zeros((m, n0), np.float32))
    with ResidentNVFP4(None, pa, p0, workers=16, output_dtype=torch.uint8, output_relu2=True) as s0:
        with ResidentNVFP4(None, placeholder, p1, workers=16, activation_buffers=(s0.output, s0.output_scales)) as s1:
            s1.output.fill_(float("nan"))
            with NativeLinearProgram(None, [s0, s1], workers=24) as program:
                out = program.forward().cpu().numpy()
                assert program.status()["code"] == 0
                counters = program.read_counters()
                np.testing.assert_array_equal(counters["counts"], counters["expected"])
                assert counters["epoch"] == 1
                out2 = program.forward().cpu().numpy()
                counters = program.read_counters()
                np.testing.assert_array_equal(counters["counts"], counters["expected"])
                np.testing.assert_array_equal(out, out2)
            # the same two stages as separate launches give the same bits
            s0.forward()
            np.testing.assert_array_equal(s1.forward().cpu().numpy(), out)
            mid = PackedNVFP4(s0.output.cpu().numpy(), unswizzle_scales(s0.output_scales.cpu().numpy(), m, n0 // 16), np.float32(1), (m, n0))
    ref = oracle.gemm(mid.data, mid.scales, 1.0, p1.data, p1.scales, 1.0, m, n1, n0)
    assert np.isfinite(out).all()
    np.testing.assert_allclose(out, ref, rtol=3e-5, atol=1e-5 * np.abs(ref).max())
    with pytest.raises(ValueError):
        NativeLinearProgram(None, [])
