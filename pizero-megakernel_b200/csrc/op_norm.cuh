// Fused LayerNorm / RMSNorm -> NVFP4 producer (also plain BF16 -> NVFP4 quantisation).
//
// RMSNorm stages let two warps share a row (four rows per tile): a lane owns the 16-element scale blocks
// part*32 + lane, + 64, ...; each block is two 16-byte loads, statistics are warp-shuffle reductions in FP32 joined
// through shared memory in a fixed order, and a block leaves as one 8-byte store of E2M1 codes plus one E4M3 scale
// byte in the swizzled 128x4 atom layout. The chain a lane walks alone (load, normalise, quantise, store, block after
// block) is what a norm stage costs, so it is kept short: one block per lane at width 1024 (3.5 instead of 5.6 us per
// expert norm stage). `norm_row` is the one-warp-per-row form used by the stand-alone quantiser kernel.
#pragma once
#include "vm_core.cuh"

namespace pi0 {

constexpr int kNormRowsPerTile = 8;           // one warp per row: the stand-alone quantiser kernel
constexpr int kNormPairRows = 4;              // two warps per row: rows a CTA normalises at a time
constexpr int kNormMaxBlocksPerLane = 4;      // one warp per row, normalising modes: width <= 2048
constexpr int kNormPairBlocksPerLane = 2;     // two warps per row

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void load_block16(const __nv_bfloat16* src, float (&v)[16]) {
    const uint4* p = reinterpret_cast<const uint4*>(src);
    uint4 a = __ldcg(p), b = __ldcg(p + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
        float2 f = __bfloat1622float2(h);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// Input block (row, block): x, plus the residual when one is bound; the sum is stored for the next residual connection
// and, with round_residual, the statistics continue from its BF16 rounding.
// LEAN (here and below): the norm of the lean kernel variant - NVFP4 output only, no fused residual, no inverse scale.
template <bool LEAN = false>
__device__ __forceinline__ void load_input16(const NormParams& n, int row, int block, float (&v)[16]) {
    load_block16(static_cast<const __nv_bfloat16*>(n.in) + static_cast<size_t>(row) * n.ld_in + block * 16, v);
    if (!LEAN && n.residual) {
        float r[16];
        load_block16(static_cast<const __nv_bfloat16*>(n.residual) + static_cast<size_t>(row) * n.width + block * 16, r);
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float a = v[2 * i] + r[2 * i], b = v[2 * i + 1] + r[2 * i + 1];
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
            const float2 back = __bfloat1622float2(h);
            v[2 * i] = n.round_residual ? back.x : a;
            v[2 * i + 1] = n.round_residual ? back.y : b;
        }
        if (n.residual_out) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(n.residual_out) + static_cast<size_t>(row) * n.width + block * 16);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
    }
}

template <bool LEAN = false>
__device__ __forceinline__ void store_block16(const NormParams& n, int row, int block, float (&v)[16]) {
    if (!LEAN && n.inv_scale) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(n.inv_scale + block * 16) + q);
            v[4 * q] *= s4.x; v[4 * q + 1] *= s4.y; v[4 * q + 2] *= s4.z; v[4 * q + 3] *= s4.w;
        }
        if (n.round_norm) {
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = bf16_round(v[i]);
        }
    }
    if (!LEAN && n.out_fp8) {
        uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int i = 0; i < 16; i++)
            w[i >> 2] |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] * n.inv_gs, __NV_SATFINITE, __NV_E4M3)) << (8 * (i & 3));
        *reinterpret_cast<uint4*>(n.out_fp8 + static_cast<size_t>(row) * n.width + block * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (!LEAN && n.out_bf16) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(n.out_bf16) + static_cast<size_t>(row) * n.width + block * 16);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
    if (n.out) {
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] *= n.inv_gs;
        uint32_t code;
        uint2 bytes = quantize_block16(v, n.policy, code);
        *reinterpret_cast<uint2*>(n.out + static_cast<size_t>(row) * n.ld_out + block * 8) = bytes;
        n.out_scales[scale_offset(row, block, n.out_blocks)] = static_cast<uint8_t>(code);
    }
}

__device__ __forceinline__ void norm_row(const NormParams& n, int row) {
    const int lane = lane_id();
    const int blocks = n.width >> 4;
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(n.in) + static_cast<size_t>(row) * n.ld_in;
    if (n.mode == 2) {                       // quantise only: stream blocks, nothing cached
        for (int b = lane; b < blocks; b += 32) {
            float v[16];
            load_block16(src + b * 16, v);
            store_block16(n, row, b, v);
        }
        return;
    }
    float cache[kNormMaxBlocksPerLane][16];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kNormMaxBlocksPerLane; j++) {
        const int b = lane + 32 * j;
        if (b < blocks) {
            load_input16(n, row, b, cache[j]);
#pragma unroll
            for (int i = 0; i < 16; i++) sum += cache[j][i];
        }
    }
    const float inv_width = 1.f / static_cast<float>(n.width);
    const float mean = n.mode == 1 ? warp_sum(sum) * inv_width : 0.f;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < kNormMaxBlocksPerLane; j++) {
        const int b = lane + 32 * j;
        if (b < blocks) {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float d = cache[j][i] - mean;
                sq += d * d;
            }
        }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_width + n.eps);
    if (n.out_factor) {                      // only the row factor is wanted
        if (lane == 0) n.out_factor[row] = rstd;
        return;
    }
#pragma unroll
    for (int j = 0; j < kNormMaxBlocksPerLane; j++) {
        const int b = lane + 32 * j;
        if (b < blocks) {
            float v[16], gm[16], bt[16];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 g4 = n.gamma ? __ldg(reinterpret_cast<const float4*>(n.gamma + b * 16) + q) : make_float4(1.f, 1.f, 1.f, 1.f);
                const float4 b4 = n.beta ? __ldg(reinterpret_cast<const float4*>(n.beta + b * 16) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                gm[4 * q] = g4.x; gm[4 * q + 1] = g4.y; gm[4 * q + 2] = g4.z; gm[4 * q + 3] = g4.w;
                bt[4 * q] = b4.x; bt[4 * q + 1] = b4.y; bt[4 * q + 2] = b4.z; bt[4 * q + 3] = b4.w;
            }
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float y = (cache[j][i] - mean) * rstd;
                if (n.gamma) y *= gm[i];
                if (n.beta) y += bt[i];
                v[i] = (n.round_norm && !n.inv_scale) ? bf16_round(y) : y;     // (with an inverse scale the rounding follows it)
            }
            store_block16(n, row, b, v);
        }
    }
}

// Two warps per row: `part` (0/1) selects this warp's half of the blocks; `red` is shared memory for 2 x 4 x 2 floats.
// Called by every warp of the CTA (it contains CTA barriers); `valid` is false for warps whose row does not exist.
template <bool LEAN = false>
__device__ __forceinline__ void norm_row_pair(const NormParams& n, int row, int local_row, int part, bool valid, float* red) {
    const int lane = lane_id();
    const int blocks = n.width >> 4;
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(n.in) + static_cast<size_t>(row) * n.ld_in;
    if (n.mode == 2) {                       // quantise only: stream blocks, nothing cached, no statistics
        if (valid) {
            for (int b = part * 32 + lane; b < blocks; b += 64) {
                float v[16];
                load_block16(src + b * 16, v);
                store_block16<LEAN>(n, row, b, v);
            }
        }
        return;
    }
    float cache[kNormPairBlocksPerLane][16];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kNormPairBlocksPerLane; j++) {
        const int b = part * 32 + lane + 64 * j;
        if (valid && b < blocks) {
            load_input16<LEAN>(n, row, b, cache[j]);
#pragma unroll
            for (int i = 0; i < 16; i++) sum += cache[j][i];
        }
    }
    const float inv_width = 1.f / static_cast<float>(n.width);
    float mean = 0.f;
    if (n.mode == 1) {                       // LayerNorm: the mean first (two-pass variance)
        sum = warp_sum(sum);
        if (lane == 0) red[local_row * 2 + part] = sum;
        __syncthreads();
        mean = (red[local_row * 2] + red[local_row * 2 + 1]) * inv_width;
    }
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < kNormPairBlocksPerLane; j++) {
        const int b = part * 32 + lane + 64 * j;
        if (valid && b < blocks) {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float d = cache[j][i] - mean;
                sq += d * d;
            }
        }
    }
    sq = warp_sum(sq);
    if (lane == 0) red[8 + local_row * 2 + part] = sq;
    __syncthreads();
    const float rstd = rsqrtf((red[8 + local_row * 2] + red[8 + local_row * 2 + 1]) * inv_width + n.eps);
    if (!valid) return;
    if (!LEAN && n.out_factor) {             // only the row factor is wanted
        if (part == 0 && lane == 0) n.out_factor[row] = rstd;
        return;
    }
#pragma unroll
    for (int j = 0; j < kNormPairBlocksPerLane; j++) {
        const int b = part * 32 + lane + 64 * j;
        if (b < blocks) {
            float v[16], gm[16], bt[16];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 g4 = n.gamma ? __ldg(reinterpret_cast<const float4*>(n.gamma + b * 16) + q) : make_float4(1.f, 1.f, 1.f, 1.f);
                const float4 b4 = n.beta ? __ldg(reinterpret_cast<const float4*>(n.beta + b * 16) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                gm[4 * q] = g4.x; gm[4 * q + 1] = g4.y; gm[4 * q + 2] = g4.z; gm[4 * q + 3] = g4.w;
                bt[4 * q] = b4.x; bt[4 * q + 1] = b4.y; bt[4 * q + 2] = b4.z; bt[4 * q + 3] = b4.w;
            }
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float y = (cache[j][i] - mean) * rstd;
                if (n.gamma) y *= gm[i];
                if (n.beta) y += bt[i];
                v[i] = (n.round_norm && (LEAN || !n.inv_scale)) ? bf16_round(y) : y;     // (with an inverse scale the rounding follows it)
            }
            store_block16<LEAN>(n, row, b, v);
        }
    }
}

template <bool LEAN = false>
__device__ __forceinline__ void norm_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, const StageDesc& st, int stage_index,
                                                 int first, int count) {
    const NormParams& n = st.p.norm;
    const int warp = threadIdx.x >> 5;
    float* red = reinterpret_cast<float*>(data);
    // A tile is four rows (RMSNorm: shortest chain per stage) or eight rows taken four at a time (LayerNorm and
    // quantise-only stages of the 768-row vision phase: half the tiles, so the stage still fits one wave of CTAs).
    const int passes = n.rows_per_tile / kNormPairRows;
    for (int t = first; t < first + count; ++t) {
        for (int pass = 0; pass < passes; ++pass) {
            const int local_row = warp >> 1;
            const int row = t * n.rows_per_tile + pass * kNormPairRows + local_row;
            norm_row_pair<LEAN>(n, row, local_row, warp & 1, row < n.rows, red);
            if (pass + 1 < passes) __syncthreads();      // `red` is reused by the next pass
        }
        cta_publish_tile(prog, st, t);          // (its barrier also separates this tile's use of `red` from the next one's)
    }
}

}  // namespace pi0
