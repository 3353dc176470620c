// Small FP32 operators around the transformer blocks: patch embedding, token embedding, FP32 linears with fused
// SiLU / RMS factor / Euler update, and the expert-input assembly. All are CTA-wide, coalesced CUDA-core code.
#pragma once
#include "vm_core.cuh"
#include "op_norm.cuh"
#include "op_attention.cuh"

namespace pi0 {

constexpr int kPatchTokens = 16;      // tokens per tile
constexpr int kPatchCols = 256;       // output columns per tile (one per thread)
constexpr int kPatchK = 14 * 14 * 3;  // 588

// out[t, n] = sum_k patch[t, k] * W[k, n] + bias[n] + pos[t % 256, n];  k = (dy*14 + dx)*3 + c, images are NHWC.
__device__ __forceinline__ void patch_tile(const PatchParams& p, const float* images, int tile, uint8_t* data) {
    float* sp = reinterpret_cast<float*>(data);                    // [16][588]
    const int ntiles = (p.width + kPatchCols - 1) / kPatchCols;
    const int tt = tile / ntiles, nt = tile - tt * ntiles;
    // gather the 16 patches: loads are issued in batches of 8 per thread before any is stored
    for (int base = 0; base < kPatchTokens * kPatchK; base += kThreads * 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = base + j * kThreads + threadIdx.x;
            v[j] = 0.f;
            if (i < kPatchTokens * kPatchK) {
                const int tok = i / kPatchK, k = i - tok * kPatchK;
                const int dy = k / 42, rem = k - dy * 42;
                const int t = tt * kPatchTokens + tok;
                const int view = t >> 8, pidx = t & 255, py = pidx >> 4, px = pidx & 15;
                v[j] = __ldg(images + ((static_cast<size_t>(view) * 224 + py * 14 + dy) * 224 + px * 14) * 3 + rem);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = base + j * kThreads + threadIdx.x;
            if (i < kPatchTokens * kPatchK) sp[i] = v[j];
        }
    }
    __syncthreads();
    const int n = nt * kPatchCols + threadIdx.x;
    if (n < p.width) {
        float acc[kPatchTokens];
#pragma unroll
        for (int i = 0; i < kPatchTokens; i++) acc[i] = 0.f;
        for (int k0 = 0; k0 < kPatchK; k0 += 4) {           // 588 = 4 * 147: four weight loads in flight
            float w[4];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = __ldg(p.weight + static_cast<size_t>(k0 + j) * p.width + n);
#pragma unroll
            for (int i = 0; i < kPatchTokens; i++) {
                const float4 x = *reinterpret_cast<const float4*>(sp + i * kPatchK + k0);
                acc[i] = fmaf(x.w, w[3], fmaf(x.z, w[2], fmaf(x.y, w[1], fmaf(x.x, w[0], acc[i]))));
            }
        }
        const float b = p.bias[n];
#pragma unroll
        for (int i = 0; i < kPatchTokens; i++) {
            const int t = tt * kPatchTokens + i;
            const float y = acc[i] + b + p.pos[static_cast<size_t>(t & 255) * p.width + n];
            static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(t) * p.width + n] = __float2bfloat16_rn(y);
        }
    }
}

__device__ __forceinline__ void patch_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, const StageDesc& st,
                                                  int stage_index, int first, int count) {
    const PatchParams& p = st.p.patch;
    const float* images = p.images ? p.images : prog.in.images;
    for (int t = first; t < first + count; ++t) {
        patch_tile(p, images, t, data);
        cta_publish_tile(prog, st, t);
    }
}

// Token rows: out[row_base + i, :] = bf16(table[token_i, :] * scale); eight tokens per tile, one warp each.
__device__ __forceinline__ void embed_instruction(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage_index,
                                                  int first, int count) {
    const EmbedParams& e = st.p.embed;
    const long long* tokens = e.tokens ? e.tokens : prog.in.tokens;
    const int warp = threadIdx.x >> 5, lane = lane_id();
    for (int t = first; t < first + count; ++t) {
        const int i = t * 8 + warp;
        if (i < e.count) {
            long long tok = tokens[i];
            tok = tok < 0 ? 0 : (tok >= e.vocab ? e.vocab - 1 : tok);
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(e.table) + static_cast<size_t>(tok) * e.width;
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(e.out) + static_cast<size_t>(e.row_base + i) * e.width;
            for (int c = lane; c < e.width; c += 32) dst[c] = __float2bfloat16_rn(__bfloat162float(src[c]) * e.scale);
        }
        cta_publish_tile(prog, st, t);
    }
}

// out[r, n] = f(sum_k x[r, k] * W[n, k]) in FP32.  A tile is 16 output columns for a block of rows (64; 32 or 16 when
// that still leaves every tile a CTA of its own: each tile stages all of its x rows, so shorter blocks mean fewer
// bytes per CTA, and an operator with few columns would otherwise occupy one or two CTAs). K runs in chunks of 128 through a four-deep
// cp.async ring in shared memory (x rows as stored, FP32 or BF16, and the 16 weight rows), so the L2 latency of a
// chunk is paid once per tile, not once per chunk. Thread (col = tid % 16, ty = tid / 16) owns rows ty, ty + 16, ...
// of its column; every shared-memory read is a 16-byte broadcast or conflict-free access.
constexpr int kLinCols = 16;
constexpr int kLinRows = 64;
constexpr int kLinChunk = 128;
constexpr int kLinLd = kLinChunk + 4;                                  // floats per staged row (padded)
constexpr int kLinStages = 4;
constexpr int kLinStageBytes = (kLinRows + kLinCols) * kLinLd * 4;     // x block + weight rows
static_assert(kLinStages * kLinStageBytes <= kDataBytes, "linear32 ring exceeds the data region");

__device__ __forceinline__ void linear32_issue(const Linear32Params& p, const void* xbase, uint8_t* stage, int col0, int r0,
                                               int row_block, int kc) {
    const int kw = min(kLinChunk, p.k - kc);
    float* xs = reinterpret_cast<float*>(stage);
    float* ws = xs + kLinRows * kLinLd;
    if (p.x_bf16) {
        // BF16 rows are staged as stored (8 elements per 16-byte copy) in the first half of each padded row
        const int per_row = kw >> 3;
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(xbase);
        for (int i = threadIdx.x; i < row_block * per_row; i += kThreads) {
            const int r = i / per_row, c = i - r * per_row;
            const bool ok = r0 + r < p.rows;
            const __nv_bfloat16* from = ok ? src + static_cast<size_t>(r0 + r + p.x_row_offset) * p.ldx + kc + c * 8 : src;
            cp_async16(reinterpret_cast<__nv_bfloat16*>(xs + r * kLinLd) + c * 8, from, ok);
        }
    } else {
        const int per_row = kw >> 2;
        const float* src = static_cast<const float*>(xbase);
        for (int i = threadIdx.x; i < row_block * per_row; i += kThreads) {
            const int r = i / per_row, c = i - r * per_row;
            const bool ok = r0 + r < p.rows;
            const float* from = ok ? src + static_cast<size_t>(r0 + r + p.x_row_offset) * p.ldx + kc + c * 4 : src;
            cp_async16(xs + r * kLinLd + c * 4, from, ok);
        }
    }
    const int per_row = kw >> 2;
    for (int i = threadIdx.x; i < kLinCols * per_row; i += kThreads) {
        const int r = i / per_row, c = i - r * per_row;
        const bool ok = col0 + r < p.n;
        const float* from = ok ? p.w + static_cast<size_t>(col0 + r) * p.k + kc + c * 4 : p.w;
        cp_async16(ws + r * kLinLd + c * 4, from, ok);
    }
}

// Four groups of 64 threads split every K chunk between them; inside a group thread (tx = t % 4, ty = t / 4) owns
// columns 4 tx .. 4 tx + 3 of rows ty, ty + 16, ... (16 R outputs), so a step of four k values costs 4 + R 16-byte
// shared-memory reads for 16 R fused multiply-adds (the operator is bound by shared-memory bandwidth, not by the
// FP32 pipe). The four partial sums of an output meet in shared memory at the end and are added in a fixed order.
template <int R>
__device__ __forceinline__ void linear32_tile(const Linear32Params& p, const void* xbase, const float* prev, int tile,
                                              uint8_t* data, long long* stamp) {
    constexpr int row_block = 16 * R;
    const int col_tiles = (p.n + kLinCols - 1) / kLinCols;
    const int ct = tile % col_tiles, r0 = (tile / col_tiles) * row_block;
    const int col0 = ct * kLinCols;
    const int kg = threadIdx.x >> 6, t64 = threadIdx.x & 63;
    const int tx = t64 & 3, ty = t64 >> 2;
    const int nchunks = (p.k + kLinChunk - 1) / kLinChunk;
    const bool rms = p.rms != 0, x_bf16 = p.x_bf16 != 0;
    float acc[R][4], ss[R];
#pragma unroll
    for (int i = 0; i < R; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; ss[i] = 0.f; }
    __syncthreads();                                   // the previous tile's readers are done with the ring
    for (int s = 0; s < kLinStages - 1; ++s) {
        if (s < nchunks) linear32_issue(p, xbase, data + s * kLinStageBytes, col0, r0, row_block, s * kLinChunk);
        cp_async_commit();
    }
    for (int c = 0; c < nchunks; ++c) {
        cp_async_wait<kLinStages - 2>();               // chunk c has landed (this thread's copies) ...
        __syncthreads();                               // ... and everybody's; the buffer of chunk c - 1 is free
        if (stamp && c == 0 && threadIdx.x == 0) stamp[4] = static_cast<long long>(global_ns());
        const int next = c + kLinStages - 1;
        if (next < nchunks) linear32_issue(p, xbase, data + (next % kLinStages) * kLinStageBytes, col0, r0, row_block, next * kLinChunk);
        cp_async_commit();
        const float* xs = reinterpret_cast<const float*>(data + (c % kLinStages) * kLinStageBytes);
        const float4* ws4 = reinterpret_cast<const float4*>(xs + kLinRows * kLinLd) + 4 * tx * (kLinLd / 4);
        const int kw4 = min(kLinChunk, p.k - c * kLinChunk) >> 2;
        const int q_end = min(kw4, kg * 8 + 8);
#pragma unroll 2
        for (int q = kg * 8; q < q_end; q++) {
            float4 w4[4], x4[R];
#pragma unroll
            for (int cc = 0; cc < 4; cc++) w4[cc] = ws4[cc * (kLinLd / 4) + q];
#pragma unroll
            for (int i = 0; i < R; i++) {
                if (x_bf16) {
                    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(xs + (ty + 16 * i) * kLinLd) + q * 4);
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
                    x4[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
                } else {
                    x4[i] = *reinterpret_cast<const float4*>(xs + (ty + 16 * i) * kLinLd + q * 4);
                }
            }
#pragma unroll
            for (int i = 0; i < R; i++) {
#pragma unroll
                for (int cc = 0; cc < 4; cc++)
                    acc[i][cc] = fmaf(x4[i].x, w4[cc].x, fmaf(x4[i].y, w4[cc].y, fmaf(x4[i].z, w4[cc].z, fmaf(x4[i].w, w4[cc].w, acc[i][cc]))));
                if (rms) ss[i] = fmaf(x4[i].x, x4[i].x, fmaf(x4[i].y, x4[i].y, fmaf(x4[i].z, x4[i].z, fmaf(x4[i].w, x4[i].w, ss[i]))));
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                   // the ring is free: it now holds the partial sums
    if (stamp && threadIdx.x == 0) stamp[5] = static_cast<long long>(global_ns());
    float* red = reinterpret_cast<float*>(data);       // [4 groups][row_block][16 columns]
    float* red_ss = red + 4 * row_block * kLinCols;    // [4 groups][row_block]
#pragma unroll
    for (int i = 0; i < R; i++) {
        *reinterpret_cast<float4*>(red + (kg * row_block + ty + 16 * i) * kLinCols + 4 * tx) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        if (tx == 0) red_ss[kg * row_block + ty + 16 * i] = ss[i];
    }
    __syncthreads();
    for (int o = threadIdx.x; o < row_block * kLinCols; o += kThreads) {
        const int rl = o >> 4, cl = o & 15;
        const int r = r0 + rl, n = col0 + cl;
        if (r >= p.rows || n >= p.n) continue;
        float v = 0.f, sq = 0.f;
#pragma unroll
        for (int k4 = 0; k4 < 4; k4++) {
            v += red[(k4 * row_block + rl) * kLinCols + cl];
            sq += red_ss[k4 * row_block + rl];
        }
        if (rms) v *= rsqrtf(sq / static_cast<float>(p.k) + p.eps);
        if (p.bias) v += p.bias[n];
        if (p.silu) v = v / (1.f + expf(-v));
        if (p.euler) v = __fadd_rn(__ldcg(prev + static_cast<size_t>(r) * p.n + n), __fmul_rn(p.dt, v));
        if (p.out_bf16) static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(r) * p.ldo + n] = __float2bfloat16_rn(v);
        else static_cast<float*>(p.out)[static_cast<size_t>(r) * p.ldo + n] = v;
    }
    if (stamp && threadIdx.x == 0) stamp[6] = static_cast<long long>(global_ns());
    // Optional extra row: FP32 values of this tile's columns copied (as BF16) to the row in front of the output,
    // which is how the state token joins the action tokens without a stage of its own.
    if (p.row0_src && r0 == 0 && threadIdx.x < kLinCols && col0 + threadIdx.x < p.n)
        static_cast<__nv_bfloat16*>(p.row0_dst)[col0 + threadIdx.x] = __float2bfloat16_rn(__ldcg(p.row0_src + col0 + threadIdx.x));
}

__device__ __forceinline__ void linear32_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, const StageDesc& st,
                                                     int stage_index, int first, int count, long long* stamp) {
    const Linear32Params& p = st.p.lin;
    const void* xbase = p.slot == 2 ? static_cast<const void*>(prog.in.state)
                        : p.slot == 3 ? static_cast<const void*>(prog.in.noise) : p.x;
    const float* prev = p.prev_slot == 3 ? prog.in.noise : p.prev;
    for (int t = first; t < first + count; ++t) {
        long long* stamp_t = t == first ? stamp : nullptr;
        if (p.row_block == 16) linear32_tile<1>(p, xbase, prev, t, data, stamp_t);
        else if (p.row_block == 32) linear32_tile<2>(p, xbase, prev, t, data, stamp_t);
        else linear32_tile<4>(p, xbase, prev, t, data, stamp_t);
        cta_publish_tile(prog, st, t);
    }
}

// Expert input: row 0 = state embedding, rows 1..chunk = action/time embeddings, as BF16. Eight rows per tile.
__device__ __forceinline__ void suffix_instruction(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage_index,
                                                   int first, int count) {
    const SuffixParams& p = st.p.suffix;
    const int warp = threadIdx.x >> 5, lane = lane_id();
    for (int t = first; t < first + count; ++t) {
        const int r = t * 8 + warp;
        if (r <= p.chunk) {
            const float* src = r == 0 ? p.state_emb : p.action_emb + static_cast<size_t>(r - 1) * p.width;
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(r) * p.width;
            for (int c = lane; c < p.width; c += 32) dst[c] = __float2bfloat16_rn(__ldcg(src + c));
        }
        cta_publish_tile(prog, st, t);
    }
}

}  // namespace pi0
