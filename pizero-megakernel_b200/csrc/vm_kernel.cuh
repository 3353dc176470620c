// The persistent worker kernel: every CTA walks its own static instruction stream.
//
// Warp 2 runs kAhead instructions ahead of the others and copies each upcoming instruction and its stage
// descriptor from global memory into a shared-memory slot with asynchronous copies that arrive on the slot's
// mbarrier, so the working warps never chase pointers through global memory between two dependent stages: they
// wait on a shared-memory barrier, read the descriptor, poll the (precomputed) producer counters in parallel and
// start.  A slot is recycled once all eight warps have released it.
#pragma once
#include "op_attention_tc.cuh"
#include "op_gemm.cuh"
#include "op_norm.cuh"
#include "op_small.cuh"

namespace pi0 {

__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Instruction `ip` of this worker, or a terminator when the stream (or the requested stage range) is over.
__device__ __forceinline__ int4 fetch_instruction(const VmProgram& prog, const int4* stream, int ip) {
    if (ip >= prog.length) return make_int4(0, 0, 0, 0);
    int4 ins = __ldg(stream + ip);
    if (ins.x == 0 || ins.y >= prog.stage_end) return make_int4(0, 0, 0, 0);
    return ins;
}

// Whole prefetch warp: fill slot (seq % kRing) with instruction `ins`. Returns false on abort.
__device__ __forceinline__ bool prefetch_slot(const VmProgram& prog, Ctl* ctl, const int4* stream, uint32_t seq, int ip, int4 ins) {
    const int lane = lane_id();
    const uint32_t slot = seq % kRing, use = seq / kRing;
    if (use > 0 && !mbar_wait_warp(prog, ctl, &ctl->release[slot], (use - 1) & 1u, ins.y)) return false;
    Slot* dst = &ctl->slot[slot];
    if (ins.x == 0) {
        if (lane == 0) dst->ins = ins;
        __syncwarp();
        mbar_arrive(&ctl->ready[slot]);
        return true;
    }
    const char* src = reinterpret_cast<const char*>(prog.stages + ins.y);
    char* out = reinterpret_cast<char*>(&dst->desc);
    for (int off = lane * 16; off < static_cast<int>(sizeof(StageDesc)); off += 32 * 16) cp_async16(out + off, src + off, true);
    if (lane == 31) cp_async16(&dst->ins, stream + ip, true);
    cp_async_arrive_noinc(&ctl->ready[slot]);
    return true;
}

// LEAN = true: the variant for programs made of the pi0 model's own NVFP4 operators only (what build_program calls
// lean); LEAN = false runs every operator and option.  Same VM, same protocol; the lean one is simply a smaller kernel.
// TIMED = false: without the per-instruction time stamps (the lean variant is built both ways, so that a stage profile
// times the kernel that serves, and serving does not carry the stamp tests: 0.5 % of the pi0 forward).
template <bool LEAN, bool TIMED = true>
__global__ void __launch_bounds__(kThreads, 1) pi0_vm_kernel(const __grid_constant__ VmProgram prog) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    Ctl* ctl = reinterpret_cast<Ctl*>(base);
    uint8_t* data = base + kCtlBytes;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; s++) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);      // one arrival per epilogue warp
        }
        for (int r = 0; r < kRing; r++) {
            mbar_init(&ctl->ready[r], 32);         // every lane of the prefetch warp
            mbar_init(&ctl->release[r], kThreads / 32);
        }
        for (int b = 0; b < 4; b++) mbar_init(&ctl->attn_bar[b], 1);
        mbar_init(&ctl->gather, kThreads / 32);
        mbar_init(&ctl->done, kThreads / 32);
        ctl->abort = 0;
        ctl->deps_seen = 0;
        ctl->dep_ok = 1;
        ctl->gate = 0;
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

    const int4* stream = prog.code + static_cast<size_t>(blockIdx.x) * prog.length;
    // first instruction of the requested stage range (streams are sorted by stage)
    int ip0 = 0;
    if (prog.stage_begin > 0) {
        while (ip0 < prog.length) {
            const int4 ins = __ldg(stream + ip0);
            if (ins.x == 0 || ins.y >= prog.stage_begin) break;
            ip0++;
        }
    }
    int4 pending = make_int4(0, 0, 0, 0);
    if (warp == kPrefetchWarp) {
        for (int s = 0; s < kAhead; s++) prefetch_slot(prog, ctl, stream, s, ip0 + s, fetch_instruction(prog, stream, ip0 + s));
        pending = fetch_instruction(prog, stream, ip0 + kAhead);
    }

    PipeState ps;
    uint32_t gathers = 0;        // CTA-wide operators executed so far (phase of the gather barrier)
    uint32_t tc_tiles = 0;       // tensor-core attention tiles executed so far (phase of their barriers)
    for (uint32_t seq = 0;; ++seq) {
        if (warp == kPrefetchWarp) {
            if (!prefetch_slot(prog, ctl, stream, seq + kAhead, ip0 + seq + kAhead, pending)) break;
            pending = fetch_instruction(prog, stream, ip0 + seq + kAhead + 1);      // consumed one iteration later
            // warm the TMA descriptors of the next instruction if its slot has already landed
            const uint32_t nslot = (seq + 1) % kRing;
            if (lane_id() < 2 && mbar_try_wait(&ctl->ready[nslot], ((seq + 1) / kRing) & 1u)) {
                const Slot& nx = ctl->slot[nslot];
                if (nx.ins.x != 0 && nx.desc.kind == OP_GEMM) prefetch_tmap(lane_id() == 0 ? nx.desc.p.gemm.tmap_a : nx.desc.p.gemm.tmap_b);
            }
        }
        const uint32_t slot = seq % kRing;
        if (!mbar_wait_warp(prog, ctl, &ctl->ready[slot], (seq / kRing) & 1u, -1)) break;
        const int4 ins = ctl->slot[slot].ins;
        if (ins.x == 0) break;
        const StageDesc& st = ctl->slot[slot].desc;
        long long* stamp = !TIMED ? nullptr : prog.timings ? prog.timings + (static_cast<size_t>(blockIdx.x) * prog.length + ip0 + seq) * 8 : nullptr;
        if (stamp && threadIdx.x == 0) stamp[0] = static_cast<long long>(global_ns());
        if (st.kind == OP_GEMM) {
            if constexpr (!LEAN) mark(prog, 800000 + ins.y);
            gemm_instruction<LEAN>(prog, ctl, data, tmem, st, ins.y, ins.z, ins.w, ps, stamp);
            // one decision per warp: the lanes with a role return later than the others and must not leave alone
            if (__any_sync(0xffffffffu, ctl->abort != 0)) break;
        } else {
            // CTA-wide operator: every warp (including GEMM roles still draining) meets here first, on an mbarrier
            // with a bounded, abort-aware wait and an all-or-nothing outcome (gather_enter). Behind the gate all
            // eight warps are present, so the hardware barriers of the operator body are safe; the next abort
            // decision is the CTA-wide one of cta_wait_sources.
            if constexpr (!LEAN) mark(prog, 600000 + ins.y);
            __syncwarp();
            if (!gather_enter(prog, ctl, gathers, ins.y)) break;
            gathers++;
            if constexpr (!LEAN) mark(prog, 700000 + ins.y);
            if (st.kind == OP_NORM) {
                // the norm weights do not depend on any stage: fetch them while the CTA waits for its input rows
                const NormParams& np = st.p.norm;
                const int lines = (np.width * 4 + 127) >> 7;
                for (int i = threadIdx.x; i < lines; i += kThreads) {
                    if (np.gamma) prefetch_l1(np.gamma + i * 32);
                    if (np.beta) prefetch_l1(np.beta + i * 32);
                }
            }
            // (an attention instruction waits for its sources itself, behind its index arithmetic)
            if (st.kind != OP_ATTN && !cta_wait_sources(prog, ctl, st, ins.y, ins.z, ins.w, stamp)) break;
            switch (st.kind) {
                case OP_NORM: norm_instruction<LEAN>(prog, ctl, data, st, ins.y, ins.z, ins.w); break;
                case OP_ATTN: attn_instruction<LEAN>(prog, ctl, data, tmem, tc_tiles, st, ins.y, ins.z, ins.w, stamp); break;
                case OP_MERGE: merge_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                case OP_PATCH: patch_instruction(prog, ctl, data, st, ins.y, ins.z, ins.w); break;
                case OP_EMBED: embed_instruction(prog, ctl, st, ins.y, ins.z, ins.w); break;
                case OP_LINEAR32: linear32_instruction(prog, ctl, data, st, ins.y, ins.z, ins.w, stamp); break;
                case OP_SUFFIX:
                    if constexpr (!LEAN) suffix_instruction(prog, ctl, st, ins.y, ins.z, ins.w);
                    break;
                case OP_PROBE:
                    if constexpr (!LEAN) probe_instruction(prog, ctl, st, tmem, ins.z, ins.w);
                    break;
                case OP_ATTN_PREP:
                    if constexpr (!LEAN) prep_instruction(prog, ctl, st, ins.z, ins.w);
                    break;
                default:
                    if (threadIdx.x == 0) { report(prog, 3, ins.y, -1, st.kind, 0); ctl->abort = 1; }
                    break;
            }
            __syncthreads();
            if (ctl->abort) break;
            if (stamp && threadIdx.x == 0) stamp[2] = static_cast<long long>(global_ns());
        }
        __syncwarp();
        if (lane_id() == 0) mbar_arrive(&ctl->release[slot]);
    }

    if constexpr (!LEAN) mark(prog, 900001);
    // Teardown. After an abort, give copies and MMAs that may still be in flight a bounded moment to land.
    if (ctl->abort) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    if constexpr (!LEAN) mark(prog, 900002);
    cp_async_wait<0>();
    tc_fence_before();
    __syncwarp();
    if (lane_id() == 0) mbar_arrive(&ctl->done);
    if (warp == 2) {
        // the warp that allocated tensor memory frees it once every warp is out of the loop (bounded wait: after
        // an abort a warp may be late, the memory is still returned)
        mbar_wait_warp(prog, ctl, &ctl->done, 0u, -1);
        if constexpr (!LEAN) mark(prog, 900003);
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    if constexpr (!LEAN) mark(prog, 900004);
}

}  // namespace pi0
