"""Small, self-contained workloads for profilers (Nsight Compute) and quick timing.

    python -m native_pi0.profile_case --case model_small --launches 3
    python -m native_pi0.profile_case --case gemm_gate_up --launches 3

``model_small`` is pi0 at full widths with 2 vision / 3 prefix / 2 expert layers and all 10 Euler steps:
one launch of the persistent kernel touches ~0.25 GB of NVFP4 weights (more than the 126 MB L2), finishes in a
few milliseconds and holds well under 2 GB on the device, so a multi-pass capture ends by itself quickly.
``gemm_gate_up`` is the Gemma-2B gate/up projection with the fused GeGLU -> NVFP4 epilogue
(M 768, N 32768, K 2048) on 148 workers; ``attention_prefix`` is the 768 x 768 MQA prefix attention.
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
    from native_pi0.primitives import ResidentNVFP4
    from native_pi0.quantization import PackedNVFP4
    rng = np.random.default_rng(0)
    m, n, k = 768, 32768, 2048

    def random_packed(rows):
        return PackedNVFP4(rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8),
                           rng.integers(40, 60, size=(rows, k // 16), dtype=np.uint8), np.float32(1.0), (rows, k))

    with ResidentNVFP4(None, random_packed(m), random_packed(n), workers=148, output_dtype=torch.uint8, output_geglu=True) as op:
        return timed(op.forward, launches, op.status)


def attention_prefix(launches):
    from native_pi0.attention import ResidentAttention
    torch.manual_seed(0)
    q = torch.randn(1, 768, 8, 256, device="cuda").bfloat16()
    k = torch.randn(1, 768, 1, 256, device="cuda").bfloat16()
    v = torch.randn(1, 768, 1, 256, device="cuda").bfloat16()
    with ResidentAttention(None, q, k, v, workers=148) as op:
        return timed(op.forward, launches, op.status)


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


CASES = {"model_small": model_small, "gemm_gate_up": gemm_gate_up, "attention_prefix": attention_prefix}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", choices=sorted(CASES), default="model_small")
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    ms = CASES[args.case](args.launches)
    print(f"{args.case}: {ms:.4f} ms per launch over {args.launches} launches (+3 warm-up)")


if __name__ == "__main__":
    main()
