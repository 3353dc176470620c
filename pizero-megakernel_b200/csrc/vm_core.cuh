// Worker-CTA control block, instruction prefetch ring, bounded waits and the inter-SM dependency protocol.
#pragma once
#include "ptx.cuh"
#include "vm_types.h"

namespace pi0 {

// GEMM pipeline: a ring of slots, each holding kChunks consecutive 256-wide K chunks of A and B plus their scale
// atoms. One slot is filled by four copies (A, B, SFA, SFB). The ring is laid out per GEMM by the host (slot size from
// the rows that are really copied, as many slots as fit): kStages slots of kStageBytes for full tiles, up to
// kMaxStages for the narrowest ones.
constexpr int kStages = 3;                                   // slots in flight with full-size tiles (128 rows of A and of B)
constexpr int kMaxStages = 5;                                // slots in flight with the narrowest tiles (64 rows of each)
constexpr int kChunks = 2;                                   // 256-wide K chunks per slot
constexpr int kTileABytes = 128 * 128;                       // one chunk of one operand: 128 rows x 128 bytes
constexpr int kSfBytes = kChunks * 4 * 512;                  // scale atoms of one operand: four 64-wide K groups per chunk
constexpr int kStageBytes = 2 * kChunks * kTileABytes + 2 * kSfBytes;   // largest slot: 72 KiB
constexpr int kCtlBytes = 3072;
constexpr int kDataBytes = 216 * 1024;                       // operator scratch behind the control block: three full-size slots
constexpr int kSmemBytes = kCtlBytes + kDataBytes + 1024;    // + slack for 1 KiB alignment
constexpr int kTmemCols = 512;
constexpr int kSfCol0 = 256;                                 // accumulators use columns [0,256)
constexpr int kRing = 4;                                     // instruction slots resident in shared memory
constexpr int kAhead = 2;                                    // the prefetch warp runs this many instructions ahead
constexpr int kPrefetchWarp = 2;
static_assert(kStages * kStageBytes <= kDataBytes, "GEMM ring exceeds the data region");
static_assert(sizeof(StageDesc) % 16 == 0, "descriptors are copied in 16-byte pieces");

// One decoded instruction: the stream entry and a private copy of its stage descriptor.
struct alignas(16) Slot {
    int4 ins;                    // {opcode, stage, first_tile, tile_count}; opcode 0 terminates the stream
    StageDesc desc;
};

struct Ctl {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t ready[kRing];       // slot filled (32 asynchronous-copy arrivals of the prefetch warp)
    uint64_t release[kRing];     // slot no longer read (one arrival per warp)
    uint64_t attn_bar[4];        // tensor-core attention: Q+K landed, S complete, V landed, O complete (one use each per tile)
    uint64_t gather;             // all warps have reached a CTA-wide operator (one arrival per warp)
    uint64_t done;               // all warps have left the instruction loop
    uint32_t tmem_base;
    volatile uint32_t deps_seen; // GEMM instructions of this CTA whose sources its copy warp has seen complete (monotonic)
    volatile int abort;          // CTA-local copy of the abort decision
    volatile int dep_ok;         // broadcast slot for CTA-wide operators
    volatile int flag;           // second broadcast slot (outcome of the split-KV ticket wait)
    int gate;                    // CTA-wide operators entered so far, or -1 once a warp has given up on one (gather_enter)
    Slot slot[kRing];
};
static_assert(sizeof(Ctl) <= kCtlBytes, "control block too large");

// The ring geometry (slot count and size) belongs to the GEMM, so positions are kept per barrier: bit s of
// prod_bits / mma_bits is the parity of the fills / drains slot s has seen. Producer and MMA lane walk the same slot
// sequence: the cursor continues from one instruction to the next and restarts at 0 when the geometry changes.
struct PipeState {
    uint32_t prod_slot = 0, prod_bits = 0, prod_geo = 0;     // TMA lane
    uint32_t mma_slot = 0, mma_bits = 0, mma_geo = 0;        // MMA lane
    uint32_t mma_it = 0;         // K stages consumed by the MMA lane (rotates the scale columns in tensor memory)
    uint32_t mma_tile = 0;       // accumulator tiles produced
    uint32_t epi_tile = 0;       // accumulator tiles drained
    uint32_t gemm_seq = 0;       // GEMM instructions this warp has been through (every warp counts them)
};

// Progress mark of this warp (debugging aid, host-mapped; see the instruction loop).  Only the instruction loop of the
// full kernel variant writes marks: inside the wait helpers, which are inlined into every pipeline loop, the test of
// the mark pointer alone cost 1.3 % of the pi0 forward.
__device__ __forceinline__ void mark(const VmProgram& prog, int code) {
    if (prog.debug && lane_id() == 0) {
        volatile int* p = prog.debug + blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
        *p = code;
    }
}

// (out of line: it runs once, when a launch gives up, and its stores need not sit in every wait loop)
__device__ __noinline__ void report(const VmProgram& prog, int code, int stage, int band, unsigned int observed,
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
    // Reading the global timer costs about a microsecond, so the clock is only consulted once a wait has
    // already lasted for several tries (the budget counts from that first reading).
    unsigned long long start = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;          // each try suspends for at most ~1 us
        if (ctl->abort) return false;
        if ((spin & 15u) == 0u) {
            const unsigned long long now = global_ns();
            if (start == 0) start = now;
            if (now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                report(prog, 2, stage, -1, parity, 0);
                ctl->abort = 1;
                return false;
            }
        }
    }
}

// The same wait for a whole warp (all 32 lanes call it, converged).  Every lane tries the barrier itself and the warp
// votes, so the common case - the phase is already complete, or completes within one try - is one instruction and a
// vote, and every lane has observed the completed phase when the call returns.  Only lane 0 keeps the time budget; its
// verdict is broadcast, so a time-out can never split the warp in front of a warp-collective instruction.
// (A version in which lane 0 waited alone and the others adopted its result measured 3 % slower on the pi0 forward:
// these helpers sit in every pipeline loop.)
__device__ __forceinline__ bool mbar_wait_warp(const VmProgram& prog, Ctl* ctl, uint64_t* bar, uint32_t parity, int stage) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    unsigned long long start = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;   // each try suspends for at most ~1 us
        if (__any_sync(0xffffffffu, ctl->abort != 0)) return false;
        if ((spin & 15u) == 0u) {
            int stop = 0;
            if (lane_id() == 0) {
                const unsigned long long now = global_ns();
                if (start == 0) start = now;
                if (now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                    report(prog, 2, stage, -1, parity, 0);
                    ctl->abort = 1;
                    stop = 1;
                }
            }
            if (__shfl_sync(0xffffffffu, stop, 0)) return false;
        }
    }
}

// Wait (bounded, abort-aware, one decision per warp) until the copy warp of this CTA has seen the sources of GEMM instruction
// number `seq` complete: from then on everything those sources wrote - and everything that was final before they ran - may
// be read, so an epilogue warp can request its residual rows and row statistics while the operands are still on their way.
__device__ __forceinline__ bool wait_deps_seen(const VmProgram& prog, Ctl* ctl, uint32_t seq, int stage) {
    unsigned long long start = 0;
    for (uint32_t spin = 1;; ++spin) {
        uint32_t seen;                                       // (every lane reads the word: no broadcast on the way out)
        asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(seen) : "r"(smem_u32(const_cast<uint32_t*>(&ctl->deps_seen))) : "memory");
        if (__all_sync(0xffffffffu, seen > seq)) return true;
        if (__any_sync(0xffffffffu, ctl->abort != 0)) return false;
        __nanosleep(32);
        if ((spin & 255u) == 0u) {
            int stop = 0;
            if (lane_id() == 0) {
                const unsigned long long now = global_ns();
                if (start == 0) start = now;
                if (now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                    report(prog, 2, stage, -1, seq, 0);
                    ctl->abort = 1;
                    stop = 1;
                }
            }
            if (__shfl_sync(0xffffffffu, stop, 0)) return false;
        }
    }
}

// Entry of a CTA-wide operator: all eight warps go in, or none does.
//
// The operator body synchronises with hardware barriers, which never time out, so a warp may only enter when every
// other warp is certain to follow. Each warp arrives on the gather barrier and waits with the usual bounds; what it
// saw (phase complete, or time-out / abort) is turned into one decision per operator by a compare-and-swap on
// ctl->gate: the first warp to finish its wait moves the gate from k (operators entered so far) to k + 1 ("all
// arrived, enter") or to -1 ("somebody gave up, leave"), and every other warp adopts that outcome whatever it
// observed itself. A warp that timed out but finds the gate at k + 1 enters (the phase did complete); a warp that
// saw the phase complete but finds -1 leaves.
__device__ __forceinline__ bool gather_enter(const VmProgram& prog, Ctl* ctl, uint32_t k, int stage) {
    const int open = static_cast<int>(k), entered = open + 1;
    int pass = 0;
    if (lane_id() == 0) mbar_arrive(&ctl->gather);
    __syncwarp();
    unsigned long long start = 0;
    for (uint32_t spin = 1;; ++spin) {                       // (the whole warp tries the barrier: see mbar_wait_warp)
        if (__all_sync(0xffffffffu, mbar_try_wait(&ctl->gather, k & 1u))) {
            if (lane_id() == 0) {
                const int seen = atomicCAS(&ctl->gate, open, entered);
                pass = (seen == open || seen == entered) ? 1 : 0;
            }
            break;
        }
        int give_up = __any_sync(0xffffffffu, ctl->abort != 0) ? 1 : 0;
        if (!give_up && (spin & 15u) == 0u) {
            if (lane_id() == 0) {
                const unsigned long long now = global_ns();
                if (start == 0) start = now;
                if (now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                    report(prog, 2, stage, -2, k, 0);
                    give_up = 1;
                }
            }
            give_up = __shfl_sync(0xffffffffu, give_up, 0);
        }
        if (give_up) {
            if (lane_id() == 0) {
                pass = atomicCAS(&ctl->gate, open, -1) == entered ? 1 : 0;
                if (!pass) ctl->abort = 1;
            }
            break;
        }
    }
    return __shfl_sync(0xffffffffu, pass, 0) != 0;
}

__device__ __forceinline__ int tile_band(const StageDesc& st, int tile) { return min(tile / st.band_div, st.bands - 1); }

// Warp-cooperative dependency wait (all 32 lanes of one warp call it): every counter this tile range reads
// is polled by its own lane, so a stage with several producers and bands costs one memory round trip, not
// one per counter.  Bands [band_lo, band_hi] of the consumer are covered.  Returns false on abort / timeout.
__device__ __forceinline__ bool warp_wait_sources(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage,
                                                  int band_lo, int band_hi) {
    const int lane = lane_id();
    const unsigned int* mine = nullptr;
    unsigned int target = 0;
    int my_band = -1, n = 0;
#pragma unroll
    for (int i = 0; i < kMaxSources; i++) {
        const int src = st.src[i];
        if (src < 0 || src < prog.stage_begin) continue;
        const int sb = st.src_bands[i];
        int lo = 0, hi = sb - 1;
        if (st.src_mode[i] == SRC_SAME_BAND) {
            lo = min(band_lo, sb - 1);
            hi = min(band_hi, sb - 1);
        }
        const int b = lo + lane - n;                 // lanes n .. n + (hi - lo) take this source's bands lo .. hi
        if (b >= lo && b <= hi) {
            mine = prog.counters + st.src_counter_base[i] + b;
            target = (b == sb - 1 ? st.src_expected_last[i] : st.src_expected[i]) * prog.epoch;
            my_band = b;
        }
        n += hi - lo + 1;
    }
    // (a consumer never reads more than 32 counters; the host rejects programs that would)
    unsigned int seen = mine ? ld_acquire(mine) : 0u;
    bool ok = mine == nullptr || seen >= target;
    if (__all_sync(0xffffffffu, ok)) return true;
    unsigned long long start = 0;                 // the global timer is slow to read: first consulted after 64 polls
    for (uint32_t spin = 1;; ++spin) {
        if (!ok) {
            __nanosleep(20);
            seen = ld_acquire(mine);
            ok = seen >= target;
        }
        if (__all_sync(0xffffffffu, ok)) return true;
        if ((spin & 63u) == 0u) {
            bool stop = ctl->abort != 0;
            const unsigned long long now = global_ns();
            if (start == 0) start = now;
            if (!stop && (now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort))) {
                if (!ok) report(prog, 1, stage, my_band, seen, target);
                stop = true;
            }
            if (__any_sync(0xffffffffu, stop)) {
                ctl->abort = 1;
                return false;
            }
        }
    }
}

// Publish progress of a tile. Call from ONE thread after a barrier (CTA or warp) that covers every
// writer thread it speaks for. A stage's tile is complete after `units_per_tile` such calls.
__device__ __forceinline__ void publish_tile(const VmProgram& prog, const StageDesc& st, int tile) {
    red_release_add(prog.counters + st.counter_base + tile_band(st, tile), 1u);
}

// CTA-wide operators: warp 0 waits for the bands of the whole tile range, everybody learns the outcome.
__device__ __forceinline__ bool cta_wait_sources(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage,
                                                 int first, int count, long long* stamp) {
    if (threadIdx.x < 32) {
        const bool ok = warp_wait_sources(prog, ctl, st, stage, tile_band(st, first), tile_band(st, first + count - 1));
        if (threadIdx.x == 0) {
            ctl->dep_ok = (ok && !ctl->abort) ? 1 : 0;       // one decision for the CTA, taken behind the entry gate
            if (stamp) stamp[1] = static_cast<long long>(global_ns());
        }
    }
    __syncthreads();
    return ctl->dep_ok != 0;
}
__device__ __forceinline__ void cta_publish_tile(const VmProgram& prog, const StageDesc& st, int tile) {
    fence_proxy_async_global();
    __syncthreads();
    if (threadIdx.x == 0) publish_tile(prog, st, tile);
}

}  // namespace pi0
