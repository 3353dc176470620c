"""Small, self-contained workloads for profilers (Nsight Compute) and quick timing.

    python -m native_pi0.profile_case --case model_small --launches 3
    python -m native_pi0.profile_case --case gemm_gate_up --launches 3

``model_small`` is pi0 at full widths with 2 vision / 3 prefix / 2 expert layers and all 10 Euler steps:
one launch of the persistent kernel touches ~0.25 GB of NVFP4 weights (more than the 126 MB L2), finishes in a
few milliseconds and holds well under 2 GB on the device, so a multi-pass capture ends by itself quickly.
``gemm_gate_up`` is the Gemma-2B gate/up projection with the fused GeGLU -> NVFP4 epilogue
(M 768, N 32768, K 2048) on 148 workers; ``attention_prefix`` is the 768 x 768 MQA prefix attention with three KV
splits (tcgen05 tiles; the ``*_mma_sync`` cases force the mma.sync tiles on the same shapes).  The other
cases are the stand-alone operator shapes the reference publishes timings for: ``gemm_expert_qkv`` (51 rows padded
to 128, N 2560, K 1024, BF16 out), ``gemm_prefix_qkv`` (768 x 2560 x 2048), ``gemm_vision_qkv`` (256 x 3456 x 1152),
``geglu_expert`` (51 x 8192 x 1024), ``attention_expert`` (51 queries over 819 keys, unsplit) and
``attention_expert_split8``, ``attention_vision`` (3 x 256 x 256, 16 heads of 72), ``norm_prefix`` (768 x 2048 RMS ->
NVFP4), ``norm_expert`` (51 x 1024) and ``mlp_block`` (RMSNorm -> gate/up + GeGLU -> down + residual at
768 x 2048 x 16384 as one three-stage launch).  ``--case all`` runs every operator case.
Prints the mean time per launch measured with CUDA events.
"""
import argparse

import numpy as np
import torch


def model_small(launches):
    from native_pi0.model import NativePi0
    from native_pi0.weights import Pi0Config, StateDictModel, random_state_dict
    cfg = Pi0Config(vision_layers=2, prefix_layers=3, expert_layers=2, vocab=1024)
    sd = random_state_dict(cfg, seed=0, device="cuda")
    g = torch.Generator(device="cpu").manual_seed(0)
    inputs = [(torch.rand(3, 224, 224, 3, generator=g) * 2 - 1).cuda(), torch.randn(1, 32, generator=g).cuda(),
              torch.randn(1, 50, 32, generator=g).cuda(), torch.zeros(1, 0, dtype=torch.int64).cuda()]
    with NativePi0(StateDictModel(cfg, sd)) as engine:
        return timed(lambda: engine.forward(*inputs), launches, engine.status)


def gemm_gate_up(launches):
    return _gemm(768, 32768, 2048, launches, output_dtype=torch.uint8, output_geglu=True)


def attention_prefix(launches):
    return _attention(1, 768, 768, 8, 1, 256, launches, splits=3)


def attention_prefix_mma_sync(launches):
    return _attention(1, 768, 768, 8, 1, 256, launches, splits=3, path="mma.sync")


def _random_packed(rng, rows, k):
    from native_pi0.quantization import PackedNVFP4
    return PackedNVFP4(rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8),
                       rng.integers(40, 60, size=(rows, k // 16), dtype=np.uint8), np.float32(1.0), (rows, k))


def _gemm(m, n, k, launches, *, rows=None, workers=148, tiled=True, block_n=128, **kw):
    from native_pi0.primitives import ResidentNVFP4
    rng = np.random.default_rng(0)
    with ResidentNVFP4(None, _random_packed(rng, m, k), _random_packed(rng, n, k), workers=workers, rows=rows, block_n=block_n,
                       tiled_weight=tiled and k % 256 == 0, **kw) as op:
        return timed(op.forward, launches, op.status)


def gemm_expert_qkv(launches):
    return _gemm(128, 2560, 1024, launches, rows=51, block_n=64, output_dtype=torch.bfloat16)


def gemm_prefix_qkv(launches):
    return _gemm(768, 2560, 2048, launches, output_dtype=torch.bfloat16)


def gemm_vision_qkv(launches):
    return _gemm(256, 3456, 1152, launches, output_dtype=torch.bfloat16)


def geglu_expert(launches):
    return _gemm(128, 8192, 1024, launches, rows=51, block_n=64, output_dtype=torch.uint8, output_geglu=True)


def _attention(b, nq, nk, h, hk, hd, launches, *, prefix=None, splits=1, workers=148, stored=None, path=None):
    """``stored``: elements a head occupies in memory (zeros behind the head); ``path``: None (by geometry), "mma.sync" or "tcgen05"."""
    from native_pi0.attention import ResidentAttention
    torch.manual_seed(0)
    stored = stored or hd
    def heads(rows, count):
        t = torch.zeros(b, rows, count, stored, device="cuda")
        t[..., :hd] = torch.randn(b, rows, count, hd, device="cuda")
        return t.bfloat16()
    q, k, v = heads(nq, h), heads(nk, hk), heads(nk, hk)
    tiles = b * ((nq + 127) // 128) * h * splits
    with ResidentAttention(None, q, k, v, workers=workers, prefix=prefix, splits=splits, fused_merge=splits > 1 and tiles <= workers,
                           head_dim=hd, path=path) as op:
        return timed(op.forward, launches, op.status)


def attention_expert(launches):
    return _attention(1, 51, 819, 8, 1, 256, launches, prefix=768)


def attention_expert_split8(launches):
    return _attention(1, 51, 819, 8, 1, 256, launches, prefix=768, splits=8)


def attention_vision(launches):
    return _attention(3, 256, 256, 16, 16, 72, launches, stored=128)


def attention_vision_mma_sync(launches):
    return _attention(3, 256, 256, 16, 16, 72, launches)


def attention_expert_split13(launches):
    return _attention(1, 51, 819, 8, 1, 256, launches, prefix=768, splits=13)


def attention_expert_split13_mma_sync(launches):
    return _attention(1, 51, 819, 8, 1, 256, launches, prefix=768, splits=13, path="mma.sync")


def _norm(rows, width, launches):
    from native_pi0.normalization import ResidentNorm
    torch.manual_seed(0)
    x = torch.randn(rows, width).bfloat16()
    with ResidentNorm(None, x, kind="rms", gamma=torch.ones(width), workers=148, row_alignment=128) as op:
        return timed(op.forward, launches, op.status)


def norm_prefix(launches):
    return _norm(768, 2048, launches)


def norm_expert(launches):
    return _norm(51, 1024, launches)


def mlp_block(launches):
    from native_pi0.linear import NativeStageProgram
    from native_pi0.normalization import ResidentNorm
    from native_pi0.primitives import ResidentNVFP4
    from native_pi0.quantization import PackedNVFP4
    rng = np.random.default_rng(0)
    m, width, mlp = 768, 2048, 16384
    x = torch.randn(m, width).bfloat16()
    empty = lambda k: PackedNVFP4(np.zeros((m, k // 2), np.uint8), np.zeros((m, k // 16), np.uint8), np.float32(1), (m, k))
    with ResidentNorm(None, x, kind="rms", gamma=torch.ones(width), workers=148, row_alignment=128) as norm, \
            ResidentNVFP4(None, empty(width), _random_packed(rng, 2 * mlp, width), workers=148, output_dtype=torch.uint8, output_geglu=True,
                          activation_buffers=(norm.output, norm.output_scales), tiled_weight=True) as gu, \
            ResidentNVFP4(None, empty(mlp), _random_packed(rng, width, mlp), workers=148, output_dtype=torch.bfloat16, residual=x,
                          activation_buffers=(gu.output, gu.output_scales), tiled_weight=True) as dn, \
            NativeStageProgram(None, [(norm, []), (gu, [(0, 0)]), (dn, [(1, 0)])], workers=148) as program:
        return timed(program.forward, launches, program.status)


def _linear32(rows, n, k, flags, launches):
    """The FP32 linear operator of the expert's head and tail (flags: 1 BF16 input, 2 BF16 output, 4 SiLU, 8 RMS factor,
    16 Euler update)."""
    import ctypes
    from native_pi0 import _native
    lib = _native.load()
    torch.manual_seed(0)
    x = torch.randn(128, k, device="cuda")
    x = x.bfloat16() if flags & 1 else x
    w, b, prev = torch.randn(n, k, device="cuda") * 0.05, torch.randn(n, device="cuda"), torch.randn(rows, n, device="cuda")
    out = torch.zeros(128, n, device="cuda", dtype=torch.bfloat16 if flags & 2 else torch.float32)
    h = ctypes.c_void_p()
    _native.check(lib.create_linear32(ctypes.byref(h), x.data_ptr(), w.data_ptr(), b.data_ptr(), prev.data_ptr() if flags & 16 else None,
                                      out.data_ptr(), rows, n, k, k, n, flags, 0, 0, 0, -0.1, 1e-6, 148), "FP32 linear setup")
    try:
        return timed(lambda: _native.check(lib.launch_op(h, None), "launch"), launches, lambda: _native.status(lib, h))
    finally:
        lib.destroy_op(h)


def linear_time_out(launches):
    return _linear32(50, 1024, 1024, 2, launches)


def linear_euler(launches):
    return _linear32(50, 32, 1024, 1 | 8 | 16, launches)


def timed(call, launches, status):
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(launches):
        call()
    stop.record()
    torch.cuda.synchronize()
    state = status()
    if state["code"]:
        raise RuntimeError(f"device status {state}")
    return start.elapsed_time(stop) / launches


CASES = {"model_small": model_small, "gemm_gate_up": gemm_gate_up, "attention_prefix": attention_prefix,
         "gemm_expert_qkv": gemm_expert_qkv, "gemm_prefix_qkv": gemm_prefix_qkv, "gemm_vision_qkv": gemm_vision_qkv,
         "geglu_expert": geglu_expert, "attention_expert": attention_expert, "attention_expert_split8": attention_expert_split8,
         "attention_vision": attention_vision, "attention_vision_mma_sync": attention_vision_mma_sync,
         "attention_prefix_mma_sync": attention_prefix_mma_sync, "attention_expert_split13": attention_expert_split13,
         "attention_expert_split13_mma_sync": attention_expert_split13_mma_sync, "norm_prefix": norm_prefix, "norm_expert": norm_expert, "mlp_block": mlp_block,
         "linear_time_out": linear_time_out, "linear_euler": linear_euler}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", choices=sorted(CASES) + ["all"], default="model_small")
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    for case in ([c for c in sorted(CASES) if c != "model_small"] if args.case == "all" else [args.case]):
        ms = CASES[case](args.launches)
        print(f"{case}: {ms:.4f} ms per launch over {args.launches} launches (+3 warm-up)", flush=True)


if __name__ == "__main__":
    main()
