// The persistent worker kernel: every CTA walks its own static instruction stream.
#pragma once
#include "op_attention.cuh"
#include "op_gemm.cuh"
#include "op_norm.cuh"
#include "op_small.cuh"

namespace pi0 {

__global__ void __launch_bounds__(kThreads, 1) pi0_vm_kernel(const __grid_constant__ VmProgram prog) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    Ctl* ctl = reinterpret_cast<Ctl*>(base);
    uint8_t* data = base + kCtlBytes;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);      // one arrival per epilogue warp
        }
        ctl->abort = 0;
        ctl->dep_ok = 1;
        mbar_fence_init();
    }
    if (warp == 2) {
        tmem_alloc(&ctl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    PipeState ps;
    const int4* stream = prog.code + static_cast<size_t>(blockIdx.x) * prog.length;
    for (int ip = 0; ip < prog.length; ++ip) {
        const int4 ins = stream[ip];
        if (ins.x == 0 || ins.y >= prog.stage_end) break;
        if (ins.y < prog.stage_begin) continue;
        const StageDesc& st = prog.stages[ins.y];
        if (prog.timings && threadIdx.x == 0) prog.timings[(static_cast<size_t>(blockIdx.x) * prog.length + ip) * 2] = clock64();
        if (st.kind == OP_GEMM) {
            gemm_instruction(prog, ctl, data, tmem, st, ins.y, ins.z, ins.w, ps);
            if (ctl->abort) break;
        } else {
            // CTA-wide operator: every warp (including GEMM roles still draining) meets here first.
            __syncthreads();
            if (ctl->abort) break;
            switch (st.kind) {
                case OP_NORM: norm_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                case OP_ATTN: attn_instruction(prog, ctl, data, st, ins.y, ins.z, ins.w); break;
                case OP_MERGE: merge_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                case OP_PATCH: patch_instruction(prog, ctl, data, st, ins.y, ins.z, ins.w); break;
                case OP_EMBED: embed_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                case OP_LINEAR32: linear32_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                case OP_SUFFIX: suffix_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                default:
                    if (threadIdx.x == 0) { report(prog, 3, ins.y, -1, st.kind, 0); ctl->abort = 1; }
                    break;
            }
            __syncthreads();
            if (ctl->abort) break;
        }
        if (prog.timings && threadIdx.x == 0) prog.timings[(static_cast<size_t>(blockIdx.x) * prog.length + ip) * 2 + 1] = clock64();
    }

    // Teardown. After an abort, give copies and MMAs that may still be in flight a bounded moment to land.
    if (ctl->abort) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace pi0
