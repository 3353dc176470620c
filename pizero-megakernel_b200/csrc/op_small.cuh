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

// out[r, n] = f(sum_k x[r, k] * W[n, k]) in FP32.  A tile is 16 output columns for a block of 32 rows (16 for an operator
// with few rows or few columns, which would otherwise occupy one or two CTAs). K runs in chunks of 256 through a four-deep
// cp.async ring in shared memory (x rows as stored, FP32 or BF16, and the 16 weight rows), so the L2 latency of a
// chunk is paid once per tile, not once per chunk.
//
// With eight warps per SM the operator is bound by instruction issue, so the inner loop is built for few instructions:
// every warp owns one eighth of each K chunk (32 values) and computes the WHOLE tile for it - lane (rg = lane / 4,
// cg = lane % 4) holds rows rg, rg + 8, ... and columns cg, cg + 4, cg + 8, cg + 12 - with packed FP32 multiply-adds
// (fma.rn.f32x2: two products per instruction, accumulated as separate even / odd partial sums).  A step of four k
// values costs RT + 4 16-byte shared-memory reads (conflict-free: rows are 132 floats apart) for 8 RT packed
// multiply-adds.  The eight partial tiles meet in shared memory at the end and are added in a fixed order.
constexpr int kLinCols = 16;
constexpr int kLinRows = 32;
constexpr int kLinChunk = 256;
constexpr int kLinLd = kLinChunk + 4;                                  // floats per staged row (padded)
constexpr int kLinStages = 4;
constexpr int kLinStageBytes = (kLinRows + kLinCols) * kLinLd * 4;     // x block + weight rows
static_assert(kLinStages * kLinStageBytes <= kDataBytes, "linear32 ring exceeds the data region");
static_assert(8 * (kLinRows * kLinCols + kLinRows) * 4 <= kLinStages * kLinStageBytes, "partial sums exceed the ring");

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)), "l"(*reinterpret_cast<const uint64_t*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}

// Geometry of one tile, read once from the (shared-memory) descriptor.
struct LinTile {
    const void* x;
    const float* w;
    int rows, n, k, ldx, x_row_offset, x_bf16;
    int col0, r0;
};

// One K chunk into a ring stage: warp w copies rows w, w + 8, ...; lane l the l-th 16-byte piece of the row.
__device__ __forceinline__ void linear32_issue(const LinTile& t, uint8_t* stage, int row_block, int kc) {
    const int warp = threadIdx.x >> 5, lane = lane_id();
    const int kw = min(kLinChunk, t.k - kc);
    float* xs = reinterpret_cast<float*>(stage);
    float* ws = xs + kLinRows * kLinLd;
    if (t.x_bf16) {
        // BF16 rows are staged as stored (8 elements per 16-byte copy) in the first half of each padded row
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(t.x);
        for (int c = lane; c < (kw >> 3); c += 32)
            for (int r = warp; r < row_block; r += 8) {
                const bool ok = t.r0 + r < t.rows;
                const __nv_bfloat16* from = ok ? src + static_cast<size_t>(t.r0 + r + t.x_row_offset) * t.ldx + kc + c * 8 : src;
                cp_async16(reinterpret_cast<__nv_bfloat16*>(xs + r * kLinLd) + c * 8, from, ok);
            }
    } else {
        const float* src = static_cast<const float*>(t.x);
        for (int c = lane; c < (kw >> 2); c += 32)
            for (int r = warp; r < row_block; r += 8) {
                const bool ok = t.r0 + r < t.rows;
                const float* from = ok ? src + static_cast<size_t>(t.r0 + r + t.x_row_offset) * t.ldx + kc + c * 4 : src;
                cp_async16(xs + r * kLinLd + c * 4, from, ok);
            }
    }
    for (int c = lane; c < (kw >> 2); c += 32)
        for (int r = warp; r < kLinCols; r += 8) {
            const bool ok = t.col0 + r < t.n;
            const float* from = ok ? t.w + static_cast<size_t>(t.col0 + r) * t.k + kc + c * 4 : t.w;
            cp_async16(ws + r * kLinLd + c * 4, from, ok);
        }
}

template <int RT>
__device__ __forceinline__ void linear32_tile(const Linear32Params& p, const void* xbase, const float* prev, int tile,
                                              uint8_t* data, long long* stamp) {
    constexpr int row_block = 8 * RT;
    const int col_tiles = (p.n + kLinCols - 1) / kLinCols;
    LinTile t;
    t.x = xbase; t.w = p.w;
    t.rows = p.rows; t.n = p.n; t.k = p.k; t.ldx = p.ldx; t.x_row_offset = p.x_row_offset; t.x_bf16 = p.x_bf16;
    t.col0 = (tile % col_tiles) * kLinCols;
    t.r0 = (tile / col_tiles) * row_block;
    const int warp = threadIdx.x >> 5, lane = lane_id();
    const int rg = lane >> 2, cg = lane & 3;
    const int nchunks = (t.k + kLinChunk - 1) / kLinChunk;
    const bool rms = p.rms != 0, x_bf16 = t.x_bf16 != 0;
    float2 acc[RT][4], ss[RT];
#pragma unroll
    for (int i = 0; i < RT; i++) {
        ss[i] = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = make_float2(0.f, 0.f);
    }
    __syncthreads();                                   // the previous tile's readers are done with the ring
    for (int s = 0; s < kLinStages - 1; ++s) {
        if (s < nchunks) linear32_issue(t, data + s * kLinStageBytes, row_block, s * kLinChunk);
        cp_async_commit();
    }
    for (int c = 0; c < nchunks; ++c) {
        cp_async_wait<kLinStages - 2>();               // chunk c has landed (this thread's copies) ...
        __syncthreads();                               // ... and everybody's; the buffer of chunk c - 1 is free
        if (stamp && c == 0 && threadIdx.x == 0) stamp[4] = static_cast<long long>(global_ns());
        const int next = c + kLinStages - 1;
        if (next < nchunks) linear32_issue(t, data + (next % kLinStages) * kLinStageBytes, row_block, next * kLinChunk);
        cp_async_commit();
        const float* xs = reinterpret_cast<const float*>(data + (c % kLinStages) * kLinStageBytes);
        const float* ws = xs + kLinRows * kLinLd;
        const int kw4 = min(kLinChunk, t.k - c * kLinChunk) >> 2;
#pragma unroll 1
        for (int j = 0; j < kLinChunk / 32; j++) {     // (not unrolled: the operator runs a few times per pass, from a cold instruction cache)
            const int q = warp * (kLinChunk / 32) + j; // this warp's share of the chunk: k values 32 warp .. 32 warp + 31
            if (q < kw4) {
                float4 w4[4];
#pragma unroll
                for (int cc = 0; cc < 4; cc++) w4[cc] = *reinterpret_cast<const float4*>(ws + (cg + 4 * cc) * kLinLd + q * 4);
                constexpr int XB = RT < 4 ? RT : 4;    // rows in flight at a time (register budget)
#pragma unroll
                for (int i0 = 0; i0 < RT; i0 += XB) {
                    float4 x4[XB];
#pragma unroll
                    for (int i = 0; i < XB; i++) {
                        if (x_bf16) {
                            const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(xs + (rg + 8 * (i0 + i)) * kLinLd) + q * 4);
                            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
                            x4[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
                        } else {
                            x4[i] = *reinterpret_cast<const float4*>(xs + (rg + 8 * (i0 + i)) * kLinLd + q * 4);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < XB; i++) {
                        const float2 xa = make_float2(x4[i].x, x4[i].y), xb = make_float2(x4[i].z, x4[i].w);
#pragma unroll
                        for (int cc = 0; cc < 4; cc++)
                            acc[i0 + i][cc] = fma2(xb, make_float2(w4[cc].z, w4[cc].w), fma2(xa, make_float2(w4[cc].x, w4[cc].y), acc[i0 + i][cc]));
                        if (rms) ss[i0 + i] = fma2(xb, xb, fma2(xa, xa, ss[i0 + i]));
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                   // the ring is free: it now holds the partial sums
    if (stamp && threadIdx.x == 0) stamp[5] = static_cast<long long>(global_ns());
    float* red = reinterpret_cast<float*>(data);       // [8 warps][row_block][16 columns]
    float* red_ss = red + 8 * row_block * kLinCols;    // [8 warps][row_block]
#pragma unroll
    for (int i = 0; i < RT; i++) {
#pragma unroll
        for (int cc = 0; cc < 4; cc++) red[(warp * row_block + rg + 8 * i) * kLinCols + cg + 4 * cc] = acc[i][cc].x + acc[i][cc].y;
        if (cg == 0) red_ss[warp * row_block + rg + 8 * i] = ss[i].x + ss[i].y;
    }
    __syncthreads();
    for (int o = threadIdx.x; o < row_block * kLinCols; o += kThreads) {
        const int rl = o >> 4, cl = o & 15;
        const int r = t.r0 + rl, n = t.col0 + cl;
        if (r >= t.rows || n >= t.n) continue;
        float v = 0.f, sq = 0.f;
#pragma unroll
        for (int k8 = 0; k8 < 8; k8++) {
            v += red[(k8 * row_block + rl) * kLinCols + cl];
            sq += red_ss[k8 * row_block + rl];
        }
        if (rms) v *= rsqrtf(sq / static_cast<float>(t.k) + p.eps);
        if (p.bias) v += p.bias[n];
        if (p.silu) v = v / (1.f + expf(-v));
        if (p.euler) v = __fadd_rn(__ldcg(prev + static_cast<size_t>(r) * t.n + n), __fmul_rn(p.dt, v));
        if (p.out_bf16) static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(r) * p.ldo + n] = __float2bfloat16_rn(v);
        else static_cast<float*>(p.out)[static_cast<size_t>(r) * p.ldo + n] = v;
    }
    if (stamp && threadIdx.x == 0) stamp[6] = static_cast<long long>(global_ns());
    // Optional extra row: FP32 values of this tile's columns copied (as BF16) to the row in front of the output,
    // which is how the state token joins the action tokens without a stage of its own.
    if (p.row0_src && t.r0 == 0 && threadIdx.x < kLinCols && t.col0 + threadIdx.x < t.n)
        static_cast<__nv_bfloat16*>(p.row0_dst)[t.col0 + threadIdx.x] = __float2bfloat16_rn(__ldcg(p.row0_src + t.col0 + threadIdx.x));
}

__device__ __forceinline__ void linear32_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, const StageDesc& st,
                                                     int stage_index, int first, int count, long long* stamp) {
    const Linear32Params& p = st.p.lin;
    const void* xbase = p.slot == 2 ? static_cast<const void*>(prog.in.state)
                        : p.slot == 3 ? static_cast<const void*>(prog.in.noise) : p.x;
    const float* prev = p.prev_slot == 3 ? prog.in.noise : p.prev;
    for (int t = first; t < first + count; ++t) {
        long long* stamp_t = t == first ? stamp : nullptr;
        if (p.row_block == 16) linear32_tile<2>(p, xbase, prev, t, data, stamp_t);
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

// Attention operand preparation: a tile is eight rows (a warp each) of the concatenated row space Q | K | V.
constexpr int kPrepRows = 8;
__device__ __forceinline__ int prep_tiles(const PrepParams& p) {
    return (p.rows[0] + kPrepRows - 1) / kPrepRows + (p.rows[1] + kPrepRows - 1) / kPrepRows + (p.rows[2] + kPrepRows - 1) / kPrepRows;
}
__device__ __forceinline__ void prep_instruction(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int first, int count) {
    const PrepParams& p = st.p.prep;
    const int warp = threadIdx.x >> 5, lane = lane_id();
    const int tq = (p.rows[0] + kPrepRows - 1) / kPrepRows, tk = (p.rows[1] + kPrepRows - 1) / kPrepRows;
    const int half = p.head_dim >> 1;
    for (int t = first; t < first + count; ++t) {
        const int part = t < tq ? 0 : (t < tq + tk ? 1 : 2);
        const int row = (t - (part == 0 ? 0 : part == 1 ? tq : tq + tk)) * kPrepRows + warp;
        if (row < p.rows[part]) {
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.src[part]) + static_cast<size_t>(row) * p.ld_src[part];
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.dst[part]) + static_cast<size_t>(row) * p.ld_dst[part];
            const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(p.bias[part]);
            const __nv_bfloat16* cs = part < 2 && p.cos[part] ? static_cast<const __nv_bfloat16*>(p.cos[part]) + static_cast<size_t>(row) * p.head_dim : nullptr;
            const __nv_bfloat16* sn = part < 2 && p.sin[part] ? static_cast<const __nv_bfloat16*>(p.sin[part]) + static_cast<size_t>(row) * p.head_dim : nullptr;
            for (int i = lane; i < p.heads[part] * half; i += 32) {
                const int h = i / half, d = i - h * half;
                float lo = __bfloat162float(src[h * p.src_pitch + d]), hi = __bfloat162float(src[h * p.src_pitch + half + d]);
                if (bias) {
                    lo += __bfloat162float(bias[h * p.head_dim + d]);
                    hi += __bfloat162float(bias[h * p.head_dim + half + d]);
                }
                if (cs) {
                    const float c = __bfloat162float(cs[d]), s = __bfloat162float(sn[d]);
                    const float rl = lo * c - hi * s, rh = hi * c + lo * s;
                    lo = rl; hi = rh;
                }
                dst[h * p.pitch + d] = __float2bfloat16_rn(lo);
                dst[h * p.pitch + half + d] = __float2bfloat16_rn(hi);
            }
        }
        cta_publish_tile(prog, st, t);
    }
}

// Resource probe (run_vm_probe): for every tile - one instruction each - every warp writes the CTA's tensor-memory base
// + 1 into its two slots, so the host sees that all eight warps took part in every instruction and that the allocation
// they saw never changed.
__device__ __forceinline__ void probe_instruction(const VmProgram& prog, Ctl* ctl, const StageDesc& st, uint32_t tmem, int first, int count) {
    const ProbeParams& p = st.p.probe;
    const int warp = threadIdx.x >> 5;
    for (int t = first; t < first + count; ++t) {
        if (lane_id() == 0) {
            p.out[t * 16 + warp] = static_cast<int>(tmem) + 1;
            p.out[t * 16 + warp + 8] = static_cast<int>(tmem) + 1;
        }
        cta_publish_tile(prog, st, t);
    }
}

}  // namespace pi0
