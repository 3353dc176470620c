// Small FP32 operators around the transformer blocks: patch embedding, token embedding, FP32 linears with fused
// SiLU / RMS factor / Euler update, and the expert-input assembly. All are CTA-wide, coalesced CUDA-core code.
#pragma once
#include "vm_core.cuh"
#include "op_norm.cuh"

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

// out[r, n] = f(sum_k x[r, k] * W[n, k]) in FP32.  A tile is 16 output columns for all rows: the CTA stages K-chunks
// of x (up to 64 rows) and of the 16 weight rows in shared memory; thread (col = tid % 16, ty = tid / 16) owns rows
// ty, ty+16, ty+32, ty+48 of its column, so every shared-memory read is a 16-byte broadcast or conflict-free access.
constexpr int kLinCols = 16;
constexpr int kLinRows = 64;
constexpr int kLinChunk = 128;
constexpr int kLinLd = kLinChunk + 4;

__device__ __forceinline__ void linear32_tile(const Linear32Params& p, const void* xbase, const float* prev, int tile,
                                              uint8_t* data) {
    float4* xs = reinterpret_cast<float4*>(data);                                   // [64][kLinLd] floats
    float4* ws = xs + kLinRows * kLinLd / 4;                                        // [16][kLinLd] floats
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int n = tile * kLinCols + tx;
    for (int r0 = 0; r0 < p.rows; r0 += kLinRows) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, ss[4] = {0.f, 0.f, 0.f, 0.f};
        for (int kc = 0; kc < p.k; kc += kLinChunk) {
            const int kw4 = min(kLinChunk, p.k - kc) >> 2;
            __syncthreads();
            // stage the chunk: all loads of a thread (8 of x, 2 of w for a full chunk) are issued before any store
            constexpr int kXLoads = kLinRows * (kLinChunk / 4) / kThreads, kWLoads = kLinCols * (kLinChunk / 4) / kThreads;
            float4 xv[kXLoads], wv[kWLoads];
#pragma unroll
            for (int j = 0; j < kXLoads; j++) {
                const int i = j * kThreads + threadIdx.x;
                const int r = i / kw4, c = i - r * kw4;
                xv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < kLinRows * kw4 && r0 + r < p.rows) {
                    const size_t off = static_cast<size_t>(r0 + r + p.x_row_offset) * p.ldx + kc + c * 4;
                    if (p.x_bf16) {
                        uint2 u = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(xbase) + off));
                        float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.x));
                        float2 hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.y));
                        xv[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
                    } else {
                        xv[j] = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(xbase) + off));
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < kWLoads; j++) {
                const int i = j * kThreads + threadIdx.x;
                const int r = i / kw4, c = i - r * kw4;
                const int col = tile * kLinCols + r;
                wv[j] = (i < kLinCols * kw4 && col < p.n) ? __ldg(reinterpret_cast<const float4*>(p.w + static_cast<size_t>(col) * p.k + kc) + c)
                                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < kXLoads; j++) {
                const int i = j * kThreads + threadIdx.x;
                if (i < kLinRows * kw4) xs[(i / kw4) * (kLinLd / 4) + (i % kw4)] = xv[j];
            }
#pragma unroll
            for (int j = 0; j < kWLoads; j++) {
                const int i = j * kThreads + threadIdx.x;
                if (i < kLinCols * kw4) ws[(i / kw4) * (kLinLd / 4) + (i % kw4)] = wv[j];
            }
            __syncthreads();
            if (p.rms) {
#pragma unroll 4
                for (int c = 0; c < kw4; c++) {
                    const float4 w4 = ws[tx * (kLinLd / 4) + c];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float4 x4 = xs[(ty + 16 * i) * (kLinLd / 4) + c];
                        acc[i] = fmaf(x4.x, w4.x, fmaf(x4.y, w4.y, fmaf(x4.z, w4.z, fmaf(x4.w, w4.w, acc[i]))));
                        ss[i] = fmaf(x4.x, x4.x, fmaf(x4.y, x4.y, fmaf(x4.z, x4.z, fmaf(x4.w, x4.w, ss[i]))));
                    }
                }
            } else {
#pragma unroll 4
                for (int c = 0; c < kw4; c++) {
                    const float4 w4 = ws[tx * (kLinLd / 4) + c];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float4 x4 = xs[(ty + 16 * i) * (kLinLd / 4) + c];
                        acc[i] = fmaf(x4.x, w4.x, fmaf(x4.y, w4.y, fmaf(x4.z, w4.z, fmaf(x4.w, w4.w, acc[i]))));
                    }
                }
            }
        }
        if (n < p.n) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = r0 + ty + 16 * i;
                if (r >= p.rows) continue;
                float v = acc[i];
                if (p.rms) v *= rsqrtf(ss[i] / static_cast<float>(p.k) + p.eps);
                if (p.bias) v += p.bias[n];
                if (p.silu) v = v / (1.f + expf(-v));
                if (p.euler) v = __fadd_rn(__ldcg(prev + static_cast<size_t>(r) * p.n + n), __fmul_rn(p.dt, v));
                if (p.out_bf16) static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(r) * p.ldo + n] = __float2bfloat16_rn(v);
                else static_cast<float*>(p.out)[static_cast<size_t>(r) * p.ldo + n] = v;
            }
        }
    }
}

__device__ __forceinline__ void linear32_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, const StageDesc& st,
                                                     int stage_index, int first, int count) {
    const Linear32Params& p = st.p.lin;
    const void* xbase = p.slot == 2 ? static_cast<const void*>(prog.in.state)
                        : p.slot == 3 ? static_cast<const void*>(prog.in.noise) : p.x;
    const float* prev = p.prev_slot == 3 ? prog.in.noise : p.prev;
    for (int t = first; t < first + count; ++t) {
        linear32_tile(p, xbase, prev, t, data);
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
