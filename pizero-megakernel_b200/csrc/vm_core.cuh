// Worker-CTA control block, bounded waits and the inter-SM dependency protocol.
#pragma once
#include "ptx.cuh"
#include "vm_types.h"

namespace pi0 {

constexpr int kStages = 5;                                   // shared-memory ring depth of the GEMM pipeline
constexpr int kTileABytes = 128 * 128;                       // 128 rows x 128 bytes (256 FP4 along K)
constexpr int kSfBytes = 4 * 512;                            // four 64-wide K groups of scale atoms
constexpr int kStageBytes = 2 * kTileABytes + 2 * kSfBytes;  // A | B | SFA | SFB = 36 KiB
constexpr int kCtlBytes = 1024;
constexpr int kDataBytes = 216 * 1024;                       // operator scratch behind the control block
constexpr int kSmemBytes = kCtlBytes + kDataBytes + 1024;    // + slack for 1 KiB alignment
constexpr int kTmemCols = 512;
constexpr int kSfCol0 = 256;                                 // accumulators use columns [0,256)
static_assert(kStages * kStageBytes <= kDataBytes, "GEMM ring exceeds the data region");

struct Ctl {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    volatile int abort;          // CTA-local copy of the abort decision
    volatile int dep_ok;         // broadcast slot for CTA-wide operators
    float red[32];               // small reduction scratch
};
static_assert(sizeof(Ctl) <= kCtlBytes, "control block too large");

struct PipeState {
    uint32_t prod_it = 0;        // K stages issued by the TMA lane
    uint32_t mma_it = 0;         // K stages consumed by the MMA lane
    uint32_t mma_tile = 0;       // accumulator tiles produced
    uint32_t epi_tile = 0;       // accumulator tiles drained
};

__device__ __forceinline__ void report(const VmProgram& prog, int code, int stage, int band, unsigned int observed,
                                       unsigned int expected) {
    VmStatus* s = prog.status;
    if (atomicCAS(&s->abort, 0, 1) == 0) {
        s->code = code;
        s->worker = blockIdx.x;
        s->stage = stage;
        s->band = band;
        s->observed = observed;
        s->expected = expected;
        __threadfence();
    }
}

// Wait on an mbarrier phase with a time budget. Returns false when the budget expires or the
// program has been aborted; the caller leaves its loop.
__device__ __forceinline__ bool mbar_wait(const VmProgram& prog, Ctl* ctl, uint64_t* bar, uint32_t parity, int stage) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long start = global_ns();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (ctl->abort) return false;
            if (global_ns() - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                report(prog, 2, stage, -1, parity, 0);
                ctl->abort = 1;
                return false;
            }
        }
    }
}

// Single-thread wait until counter >= target.
__device__ __forceinline__ bool counter_wait(const VmProgram& prog, Ctl* ctl, const unsigned int* counter,
                                             unsigned int target, int stage, int band) {
    unsigned int seen = ld_acquire(counter);
    if (seen >= target) return true;
    unsigned long long start = global_ns();
    for (uint32_t spin = 1;; ++spin) {
        __nanosleep(20);
        seen = ld_acquire(counter);
        if (seen >= target) return true;
        if ((spin & 63u) == 0u) {
            if (ctl->abort) return false;
            if (global_ns() - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                report(prog, 1, stage, band, seen, target);
                ctl->abort = 1;
                return false;
            }
        }
    }
}

// Wait (one thread) for every source of `st` that this tile band reads.
__device__ __forceinline__ bool wait_sources(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage, int band) {
#pragma unroll
    for (int i = 0; i < kMaxSources; i++) {
        int src = st.src[i];
        if (src < 0 || src < prog.stage_begin) continue;
        const StageDesc& ps = prog.stages[src];
        int lo = 0, hi = ps.bands;
        if (st.src_mode[i] == SRC_SAME_BAND) {
            lo = min(band, ps.bands - 1);
            hi = lo + 1;
        }
        for (int b = lo; b < hi; b++) {
            int c = ps.counter_base + b;
            if (!counter_wait(prog, ctl, prog.counters + c, prog.expected[c] * prog.epoch, stage, b)) return false;
        }
    }
    return true;
}

__device__ __forceinline__ int tile_band(const StageDesc& st, int tile) { return min(tile / st.band_div, st.bands - 1); }

// Publish progress of a tile. Call from ONE thread after a barrier (CTA or warp) that covers every
// writer thread it speaks for. A stage's tile is complete after `units_per_tile` such calls.
__device__ __forceinline__ void publish_tile(const VmProgram& prog, const StageDesc& st, int tile) {
    __threadfence();
    red_release_add(prog.counters + st.counter_base + tile_band(st, tile), 1u);
}

// CTA-wide operators: thread 0 waits, everybody learns the outcome. Returns false on abort.
__device__ __forceinline__ bool cta_wait_sources(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage, int band) {
    if (threadIdx.x == 0) ctl->dep_ok = wait_sources(prog, ctl, st, stage, band) ? 1 : 0;
    __syncthreads();
    bool ok = ctl->dep_ok != 0;
    __syncthreads();
    return ok;
}
__device__ __forceinline__ void cta_publish_tile(const VmProgram& prog, const StageDesc& st, int tile) {
    fence_proxy_async_global();
    __syncthreads();
    if (threadIdx.x == 0) publish_tile(prog, st, tile);
}

}  // namespace pi0
