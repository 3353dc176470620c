// Attention tile on the 5th-generation tensor cores: softmax(scale * Q K^T + mask) V for one
// (batch, head, 128-query tile, KV split) with S, P and O never leaving the SM.
//
//   TMA  : Q [128 x hd] and the tile's keys K [<= 256 x hd] arrive as 64-element (128-byte) column chunks with the
//          128-byte swizzle, the layout tcgen05 reads as a K-major operand; V follows into K's place once S is done.
//   S    : tcgen05.mma kind::f16, M 128, N = keys of the tile (<= 256), K = hd -> FP32 in tensor memory columns [0, 256)
//   P    : every thread owns one query row of one half of the 32-column chunks (tcgen05.ld 32x32b): row maximum, exp2,
//          row sum in FP32; P is rounded to BF16 and written over Q in the same swizzled K-major layout
//   O    : tcgen05.mma, A = P (K-major), B = V as it lies in memory (hd contiguous: the "MN-major" operand form, one
//          128-byte row per key) -> FP32 in tensor memory columns [256, 256 + hd)
//   out  : O / l as BF16 rows, or with KV splits the un-normalised BF16 rows plus (m, l) for the merge
//
// A tile holds all its keys' scores at once (at most 256 keys), so there is no running maximum and no rescaling of O;
// longer key ranges are covered by KV splits and the split merge.  Heads of 72 (SigLIP) are stored padded to 128 with
// zeros by the producing projection, so every chunk is a full 128-byte row.  Waits are bounded like all others
// (cta_wait_phase).
#pragma once
#include "op_attention.cuh"

namespace pi0 {

constexpr int kTcQBytes = 64 * 1024;                    // Q chunks (later P chunks): up to four of 128 rows x 128 bytes
constexpr int kTcKvBytes = 128 * 1024;                  // K chunks (later V chunks): up to four of 256 rows x 128 bytes
constexpr int kTcScratch = kTcQBytes + kTcKvBytes;      // row maxima / sums of the two column halves: 2 x 2 x 128 floats
static_assert(kTcScratch + 2048 <= kDataBytes, "tensor-core attention exceeds the data region");

// CTA-wide wait on a phase: every warp tries the barrier itself (so each thread has observed the completed phase);
// warp 0 keeps the time budget and raises the CTA's abort flag, which ends every warp's spin; one hardware barrier
// behind the spins makes the outcome the same for all threads.
__device__ __forceinline__ bool cta_wait_phase(const VmProgram& prog, Ctl* ctl, uint64_t* bar, uint32_t parity, int stage) {
    unsigned long long start = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) break;
        if (__any_sync(0xffffffffu, ctl->abort != 0)) break;
        if (threadIdx.x < 32 && (spin & 15u) == 0u) {
            int stop = 0;
            if (threadIdx.x == 0) {
                const unsigned long long now = global_ns();
                if (start == 0) start = now;
                if (now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                    report(prog, 2, stage, -1, parity, 0);
                    ctl->abort = 1;
                    stop = 1;
                }
            }
            if (__shfl_sync(0xffffffffu, stop, 0)) break;
        }
    }
    __syncthreads();
    return ctl->abort == 0;
}

// HDP: elements per head in memory and in the MMAs (128 or 256); a.head_dim: logical width that is stored.
// `uses` counts the tensor-core attention tiles this CTA has run (phase parity of the four barriers).
// MASK: the operator's boolean visibility mask is consulted (instantiated for the full kernel variant only).
template <int HDP, bool MASK = false>
// deps: when not null, the stage whose sources this call waits for itself (tile range dep_first, dep_count) - after its
// index arithmetic and just before the first copies, so that the arithmetic is off the dependent path.
__device__ bool attn_tile_tc(const VmProgram& prog, Ctl* ctl, const AttnParams& a, int tile, uint8_t* data, uint32_t tmem,
                             uint32_t uses, int stage, long long* stamp, const StageDesc* deps, int dep_first, int dep_count) {
    constexpr int CHUNKS = HDP / 64;
    uint8_t* sQ = data;                                  // Q, then P
    uint8_t* sKV = data + kTcQBytes;                     // K, then V
    float* xm = reinterpret_cast<float*>(data + kTcScratch);           // [2][128] row maxima of the two column halves
    float* xl = xm + 256;                                               // [2][128] row sums

    const int warp = threadIdx.x >> 5, lane = lane_id();
    const int split = tile % a.splits;
    const int t2 = tile / a.splits;
    const int head = t2 % a.heads;
    const int qbg = t2 / a.heads;
    const int qtiles = (a.nq + kAttnQRows - 1) / kAttnQRows;
    const int batch = qbg / qtiles, qt = qbg - batch * qtiles;
    const int q0 = qt * kAttnQRows;
    const int q_valid = min(kAttnQRows, a.nq - q0);
    const int kvh = head / (a.heads / a.kv_heads);
    const int per = (a.nk + a.splits - 1) / a.splits;
    const int k_begin = split * per, k_end = min(a.nk, k_begin + per);
    const int keys = max(k_end - k_begin, 0);
    const int n_s = a.k_box;                             // score columns computed (multiple of 16, >= keys)
    const uint32_t parity = uses & 1u;
    uint64_t* bar_qk = &ctl->attn_bar[0];
    uint64_t* bar_s = &ctl->attn_bar[1];
    uint64_t* bar_v = &ctl->attn_bar[2];
    uint64_t* bar_o = &ctl->attn_bar[3];

    if (deps && !cta_wait_sources(prog, ctl, *deps, stage, dep_first, dep_count, stamp)) return false;

    // ---- Q and K
    if (threadIdx.x == 0) {
        const uint32_t q_bytes = static_cast<uint32_t>(a.q_box) * 128u, k_bytes = static_cast<uint32_t>(a.k_box) * 128u;
        mbar_expect_tx(bar_qk, CHUNKS * (q_bytes + k_bytes));
        const int q_row = batch * a.q_batch_rows + q0, k_row = batch * a.kv_batch_rows + k_begin;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            tma_load_2d(sQ + c * 16384, a.tmap_q, bar_qk, head * HDP + c * 64, q_row);
            tma_load_2d(sKV + c * k_bytes, a.tmap_k, bar_qk, kvh * HDP + c * 64, k_row);
        }
    }
    // ---- S = Q K^T  (only the issuing warp waits for Q and K: nobody else touches them; if its wait gives up, the abort
    //      flag is set and the CTA-wide wait for S below ends for everybody)
    constexpr uint64_t kKMajor = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);       // 128-byte swizzle, 8-row groups 1 KiB apart
    const uint32_t q16 = (smem_u32(sQ) & 0x3FFFFu) >> 4, kv16 = (smem_u32(sKV) & 0x3FFFFu) >> 4;
    const uint32_t kchunk16 = static_cast<uint32_t>(a.k_box) * 8u;                                  // one K/V chunk in 16-byte units
    if (warp == 0 && mbar_wait_warp(prog, ctl, bar_qk, parity, stage)) {
        if (stamp && lane == 0) stamp[4] = static_cast<long long>(global_ns());
        if (elect_one()) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n_s >> 3) << 17) | (8u << 24);
#pragma unroll
            for (int i = 0; i < HDP / 16; ++i) {
                const uint32_t c = static_cast<uint32_t>(i) >> 2, sub = static_cast<uint32_t>(i) & 3u;
                tc_mma_f16(tmem, kKMajor | static_cast<uint64_t>(q16 + c * 1024u + 2u * sub),
                           kKMajor | static_cast<uint64_t>(kv16 + c * kchunk16 + 2u * sub), idesc, i != 0 ? 1u : 0u);
            }
            tc_commit(bar_s);
        }
        __syncwarp();
    }
    if (!cta_wait_phase(prog, ctl, bar_s, parity, stage)) return false;
    tc_fence_after();

    // ---- V into K's place (its copies overlap the softmax)
    if (threadIdx.x == 0) {
        const uint32_t k_bytes = static_cast<uint32_t>(a.k_box) * 128u;
        mbar_expect_tx(bar_v, CHUNKS * k_bytes);
        const int k_row = batch * a.kv_batch_rows + k_begin;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) tma_load_2d(sKV + c * k_bytes, a.tmap_v, bar_v, kvh * HDP + c * 64, k_row);
    }

    // ---- softmax: thread = query row, the two warp groups take alternate 32-column chunks
    const int wg = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;                                // query row inside the tile = tensor-memory lane
    const int qrow = q0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = a.scale * 1.4426950408889634f;
    const int chunks32 = (n_s + 31) >> 5;
    const int visible_end = (a.prefix >= 0 && qrow == 0) ? min(keys, a.prefix + 1 - k_begin) : keys;   // keys [0, visible_end) of this tile
    // bit i of the result: key j * 32 + i of this tile is visible to this thread's query row under the boolean mask
    auto mask_bits = [&](int j) -> uint32_t {
        if constexpr (!MASK) return 0xffffffffu;
        if (qrow >= a.nq) return 0u;
        const uint8_t* m = a.mask + (static_cast<size_t>(batch) * a.nq + qrow) * a.nk + k_begin + j * 32;
        uint32_t bits = 0u;
#pragma unroll 8
        for (int i = 0; i < 32; i++)
            if (j * 32 + i < keys && __ldg(m + i)) bits |= 1u << i;
        return bits;
    };
    float m_part = -INFINITY;
    for (int j = wg; j < chunks32; j += 2) {
        uint32_t raw[32];
        tmem_ld32(tmem + lane_addr + j * 32, raw);
        const uint32_t vis = mask_bits(j);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++)
            if (j * 32 + i < visible_end && ((vis >> i) & 1u)) m_part = fmaxf(m_part, __uint_as_float(raw[i]));
    }
    xm[wg * 128 + row] = m_part;
    __syncthreads();
    const float m_raw = fmaxf(xm[row], xm[128 + row]);
    const float m_use = m_raw == -INFINITY ? 0.f : m_raw * sl2;
    float l_part = 0.f;
    for (int j = wg; j < chunks32; j += 2) {
        uint32_t raw[32];
        tmem_ld32(tmem + lane_addr + j * 32, raw);
        const uint32_t vis = mask_bits(j);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int k0 = j * 32 + 2 * i;
            const float p0 = k0 < visible_end && ((vis >> (2 * i)) & 1u) ? exp2f(__uint_as_float(raw[2 * i]) * sl2 - m_use) : 0.f;
            const float p1 = k0 + 1 < visible_end && ((vis >> (2 * i + 1)) & 1u) ? exp2f(__uint_as_float(raw[2 * i + 1]) * sl2 - m_use) : 0.f;
            l_part += p0 + p1;
            packed[i] = pack2_bf16(p0, p1);
        }
        // P chunk of 64 keys = 128 rows x 128 bytes, 16-byte units swizzled with the row (what the K-major descriptor expects)
        uint8_t* prow = sQ + (j >> 1) * 16384 + row * 128;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int unit = ((j & 1) * 4 + u) ^ (row & 7);
            *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
        }
    }
    xl[wg * 128 + row] = l_part;
    tc_fence_before();
    fence_proxy_async_smem();                            // P (generic stores) must be visible to the tensor core's reads
    __syncthreads();

    // ---- O = P V  (again only the issuing warp waits for V)
    if (warp == 0 && mbar_wait_warp(prog, ctl, bar_v, parity, stage)) {
        if (stamp && lane == 0) stamp[5] = static_cast<long long>(global_ns());
        tc_fence_after();
        if (elect_one()) {
            // B = V with hd contiguous (MN-major): 64-element blocks of hd are one chunk (k_box rows x 128 bytes) apart,
            // groups of 8 keys 1 KiB apart
            const uint64_t v_major = (static_cast<uint64_t>(kchunk16) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(HDP >> 3) << 17) | (8u << 24);
            const int steps = n_s >> 4;
            for (int j = 0; j < steps; ++j) {
                const uint32_t c = static_cast<uint32_t>(j) >> 2, sub = static_cast<uint32_t>(j) & 3u;
                tc_mma_f16(tmem + 256u, kKMajor | static_cast<uint64_t>(q16 + c * 1024u + 2u * sub),
                           v_major | static_cast<uint64_t>(kv16 + static_cast<uint32_t>(j) * 128u), idesc, j != 0 ? 1u : 0u);
            }
            tc_commit(bar_o);
        }
        __syncwarp();
    }
    if (!cta_wait_phase(prog, ctl, bar_o, parity, stage)) return false;
    tc_fence_after();
    if (stamp && threadIdx.x == 0) stamp[6] = static_cast<long long>(global_ns());

    // ---- output: thread = row, warp group = half of the head's columns
    const float l_sum = xl[row] + xl[128 + row];
    const bool row_ok = row < q_valid;
    constexpr int HALF = HDP / 2;
    const int col_begin = wg * HALF;
    if (a.splits > 1) {
        __nv_bfloat16* po = reinterpret_cast<__nv_bfloat16*>(a.partial_o) + (static_cast<size_t>(tile) * kAttnQRows + row) * a.head_dim;
        for (int c0 = col_begin; c0 < col_begin + HALF; c0 += 32) {
            uint32_t raw[32];
            tmem_ld32(tmem + 256u + lane_addr + c0, raw);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (c0 + 8 * u < a.head_dim)
                        *reinterpret_cast<uint4*>(po + c0 + 8 * u) =
                            make_uint4(pack2_bf16(__uint_as_float(raw[8 * u]), __uint_as_float(raw[8 * u + 1])),
                                       pack2_bf16(__uint_as_float(raw[8 * u + 2]), __uint_as_float(raw[8 * u + 3])),
                                       pack2_bf16(__uint_as_float(raw[8 * u + 4]), __uint_as_float(raw[8 * u + 5])),
                                       pack2_bf16(__uint_as_float(raw[8 * u + 6]), __uint_as_float(raw[8 * u + 7])));
                }
            }
        }
        if (wg == 0 && row_ok) {
            float* pml = a.partial_ml + (static_cast<size_t>(tile) * kAttnQRows + row) * 2;
            pml[0] = m_raw == -INFINITY ? -INFINITY : m_use;
            pml[1] = l_sum;
        }
    } else {
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        const size_t grow = static_cast<size_t>(batch) * a.q_batch_rows + q0 + row;
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.out) + grow * a.ldo + head * a.head_dim;
        for (int c0 = col_begin; c0 < col_begin + HALF; c0 += 32) {
            uint32_t raw[32];
            tmem_ld32(tmem + 256u + lane_addr + c0, raw);
            tmem_ld_wait();
            if (row_ok && a.out) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (c0 + 8 * u < a.head_dim)
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * u) =
                            make_uint4(pack2_bf16(__uint_as_float(raw[8 * u]) * inv, __uint_as_float(raw[8 * u + 1]) * inv),
                                       pack2_bf16(__uint_as_float(raw[8 * u + 2]) * inv, __uint_as_float(raw[8 * u + 3]) * inv),
                                       pack2_bf16(__uint_as_float(raw[8 * u + 4]) * inv, __uint_as_float(raw[8 * u + 5]) * inv),
                                       pack2_bf16(__uint_as_float(raw[8 * u + 6]) * inv, __uint_as_float(raw[8 * u + 7]) * inv));
                }
            }
            if (a.out_fp4 && row_ok) {
                // NVFP4 copy of the BF16-rounded rows: every head occupies fp4_pitch columns (a multiple of 16 >= head_dim;
                // the accumulator columns beyond head_dim are exact zeros because V is zero there)
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const int cb = c0 + 16 * half;
                    if (cb < a.fp4_pitch) {
                        float v[16];
#pragma unroll
                        for (int e = 0; e < 16; e++)
                            v[e] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(raw[16 * half + e]) * inv)) * a.out_inv_gs;
                        uint32_t code;
                        const uint2 bytes = quantize_block16(v, 0, code);
                        const int col = head * a.fp4_pitch + cb;
                        *reinterpret_cast<uint2*>(a.out_fp4 + grow * a.ld_fp4 + (col >> 1)) = bytes;
                        a.out_scales[scale_offset(static_cast<int>(grow), col >> 4, a.out_blocks)] = static_cast<uint8_t>(code);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();                                     // tensor memory and the operand buffers are free for the next tile
    return true;
}

}  // namespace pi0
