// GEMM instruction:  out[M,N] = epilogue(alpha * A[M,K] . B[N,K]^T), FP32 accumulation in tensor memory.
// Operands: NVFP4 (packed E2M1 with E4M3 block scales, tcgen05.mma kind::mxf4nvf4.block_scale), BF16 (kind::f16) or
// FP8 E4M3 (kind::f8f6f4).  In every format a row of K is cut into 128-byte chunks and one MMA consumes 32 bytes of
// each operand row (64 FP4, 16 BF16 or 32 FP8 elements), so the copy ring and the issue loop are the same code.
//
//   warp 0 / lane 0 : TMA producer  - operand tiles (128 B swizzled rows) and scale atoms into a ring of slots; the ring
//                                     is laid out per GEMM: 3 slots of 72 KiB for full NVFP4 tiles, up to 5 for narrow ones
//   warp 1          : MMA issuer    - warp-uniform loop, one elected lane issues tcgen05.cp (scales smem->TMEM, NVFP4
//                                     only) and tcgen05.mma, 32 operand bytes of K each
//   warps 4..7      : epilogue      - tcgen05.ld of a 128xN FP32 accumulator (one row per thread), fused math, stores
//
// Two TMEM accumulators alternate, so the epilogue of tile t overlaps the MMAs of tile t+1. Pipeline positions live in
// registers (PipeState) and carry over from one instruction to the next; barriers are never re-initialised.
#pragma once
#include "vm_core.cuh"

namespace pi0 {

// Whole warp 0: the dependency wait is lane-parallel, lane 0 issues the copies.
//
// Weights never depend on another stage, so for the first tile of an instruction the B tiles and B scales of the
// first slots are requested BEFORE the dependency wait (their bytes are announced with expect_tx without an
// arrival); when the producers are done only the activation half (A, A scales) is still to be fetched.
__device__ __forceinline__ void gemm_producer(const VmProgram& prog, Ctl* ctl, uint8_t* data, const StageDesc& st,
                                              int stage_index, int first, int count, PipeState& ps, long long* stamp) {
    const GemmParams& g = st.p.gemm;
    const int lane = lane_id();
    uint32_t p_slot = ps.prod_slot, p_bits = ps.prod_bits;
    const int chunks = (g.k_groups + 3) >> 2;                        // 256-wide K chunks
    const int slots = (chunks + kChunks - 1) / kChunks;
    const uint32_t a_bytes = static_cast<uint32_t>(kChunks) * 128u * static_cast<uint32_t>(g.a_box_rows);
    const uint32_t b_bytes = static_cast<uint32_t>(kChunks) * 128u * static_cast<uint32_t>(g.block_n);
    const uint32_t ring = static_cast<uint32_t>(g.ring_stages), stride = static_cast<uint32_t>(g.slot_stride);
    const uint32_t sf_unit = g.operands == GEMM_NVFP4 ? 512u : 0u;      // scale-atom bytes per MMA group and operand
    if (ps.prod_geo != stride) {
        // Slots of the previous geometry overlap the new ones at other indices: every copy issued so far must have
        // been read by its MMAs before the first new copy lands (waits for the last release of each slot).
        int alive0 = 1;
        if (lane == 0)
            for (int s = 0; s < kMaxStages && alive0; ++s)
                alive0 = mbar_wait(prog, ctl, &ctl->empty[s], ((p_bits >> s) & 1u) ^ 1u, stage_index) ? 1 : 0;
        alive0 = __shfl_sync(0xffffffffu, alive0, 0);
        if (!alive0) return;
        ps.prod_geo = stride;
        p_slot = 0;
    }
    int current_band = -1;
    for (int t = first; t < first + count; ++t) {
        const int m_tile = t / g.n_tiles, n_tile = t - m_tile * g.n_tiles;
        const int band = tile_band(st, t);
        // B scales: the 128-row atom that holds the tile's rows, or - 32-wide tiles - an atom of the tile's own
        const int sfb_tile = g.block_n == 32 ? n_tile : (n_tile * g.block_n) >> 7;
        int early = 0;                                               // slots whose weight half is already in flight
        int alive = 1;
        if (band != current_band) {
            if (t == first) {
                if (lane == 0) {
                    early = min(slots, g.ring_stages);
                    for (int ks = 0; ks < early; ++ks) {
                        const uint32_t s = (p_slot + ks) % ring;
                        if (!mbar_wait(prog, ctl, &ctl->empty[s], ((p_bits >> s) & 1u) ^ 1u, stage_index)) { alive = 0; break; }
                        const int groups = min(4 * kChunks, g.k_groups - ks * 4 * kChunks);
                        uint8_t* slot = data + s * stride;
                        mbar_expect_tx_only(&ctl->full[s], b_bytes + groups * sf_unit);
                        if (g.b_tiled) tma_load_2d(slot + g.off_b, g.tmap_b, &ctl->full[s], 0, (n_tile * chunks + ks * kChunks) * g.block_n);
                        else tma_load_3d(slot + g.off_b, g.tmap_b, &ctl->full[s], 0, n_tile * g.block_n, ks * kChunks);
                        if (sf_unit)
                            bulk_load(slot + g.off_sfb, g.sfb + (static_cast<size_t>(sfb_tile) * g.k_groups + ks * 4 * kChunks) * 512,
                                      groups * 512u, &ctl->full[s]);
                    }
                }
                early = __shfl_sync(0xffffffffu, early, 0);
                alive = __shfl_sync(0xffffffffu, alive, 0);
                if (!alive) return;
            }
            if (!warp_wait_sources(prog, ctl, st, stage_index, band, band)) return;
            if (lane == 0) {
                fence_proxy_async_global();
                if (current_band < 0)       // tell the epilogue warps: the sources of this instruction's first band are complete
                    asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(&ctl->deps_seen))), "r"(ps.gemm_seq + 1u) : "memory");
                if (stamp && current_band < 0) stamp[1] = static_cast<long long>(global_ns());
            }
            current_band = band;
        }
        if (lane == 0) {
            for (int ks = 0; ks < slots; ++ks) {
                const uint32_t s = p_slot;
                const int groups = min(4 * kChunks, g.k_groups - ks * 4 * kChunks);
                uint8_t* slot = data + s * stride;
                const bool weights_issued = ks < early;
                if (!weights_issued && !mbar_wait(prog, ctl, &ctl->empty[s], ((p_bits >> s) & 1u) ^ 1u, stage_index)) { alive = 0; break; }
                // Boxes always deliver kChunks chunks (beyond K the copy engine fills zeros or, inside a padded
                // allocation, bytes that no MMA reads).  a_box_rows < 128 (few logical rows): only the rows that
                // exist are copied; the MMA still reads 128 rows, the rest lands in accumulator rows never stored.
                mbar_expect_tx(&ctl->full[s], a_bytes + groups * sf_unit + (weights_issued ? 0u : b_bytes + groups * sf_unit));
                tma_load_3d(slot, g.tmap_a, &ctl->full[s], 0, m_tile * 128, ks * kChunks);
                if (sf_unit)
                    bulk_load(slot + g.off_sfa, g.sfa + (static_cast<size_t>(m_tile) * g.k_groups + ks * 4 * kChunks) * 512, groups * 512u,
                              &ctl->full[s]);
                if (!weights_issued) {
                    if (g.b_tiled) tma_load_2d(slot + g.off_b, g.tmap_b, &ctl->full[s], 0, (n_tile * chunks + ks * kChunks) * g.block_n);
                    else tma_load_3d(slot + g.off_b, g.tmap_b, &ctl->full[s], 0, n_tile * g.block_n, ks * kChunks);
                    if (sf_unit)
                        bulk_load(slot + g.off_sfb, g.sfb + (static_cast<size_t>(sfb_tile) * g.k_groups + ks * 4 * kChunks) * 512,
                                  groups * 512u, &ctl->full[s]);
                }
                p_bits ^= 1u << s;
                p_slot = s + 1 == ring ? 0u : s + 1;
            }
        }
        alive = __shfl_sync(0xffffffffu, alive, 0);
        if (!alive) return;
    }
    ps.prod_slot = p_slot;
    ps.prod_bits = p_bits;
}

// Whole warp 1, converged: the loop and all operand arithmetic are warp-uniform and only the tcgen05 instructions are
// issued by one elected lane. (Run by a single lane inside a divergent branch, every descriptor and address has to be
// moved from per-thread to uniform registers for each instruction, which measured about 250 cycles per 64-wide K
// group and made this lane, not the copies or the tensor core, the pace of a narrow GEMM.)
// (One instantiation per operand format, so each issue loop carries only its own instructions.)
template <int OPERANDS>
__device__ __forceinline__ void gemm_mma(const VmProgram& prog, Ctl* ctl, uint8_t* data, uint32_t tmem_in, const StageDesc& st,
                                         int stage_index, int first_in, int count_in, PipeState& ps, long long* stamp) {
    const GemmParams& g = st.p.gemm;
    const int first = uniform_i32(first_in), count = uniform_i32(count_in);
    const int k_groups = uniform_i32(g.k_groups), n_tiles = uniform_i32(g.n_tiles), block_n = uniform_i32(g.block_n);
    const int chunks = (k_groups + 3) >> 2;
    const int slots = (chunks + kChunks - 1) / kChunks;
    const uint32_t a_chunk16 = uniform_u32(static_cast<uint32_t>(g.a_box_rows)) * 8u, b_chunk16 = static_cast<uint32_t>(block_n) * 8u;   // 16-byte units
    const uint32_t ring = uniform_u32(static_cast<uint32_t>(g.ring_stages)), stride = uniform_u32(static_cast<uint32_t>(g.slot_stride));
    const uint32_t off_b16 = uniform_u32(static_cast<uint32_t>(g.off_b)) >> 4, off_sfa16 = uniform_u32(static_cast<uint32_t>(g.off_sfa)) >> 4,
                   off_sfb16 = uniform_u32(static_cast<uint32_t>(g.off_sfb)) >> 4;
    const uint32_t idesc = uniform_u32(g.idesc);
    const uint32_t tmem = uniform_u32(tmem_in);
    const uint32_t data16 = uniform_u32((smem_u32(data) & 0x3FFFFu) >> 4), stride16 = stride >> 4;
    // descriptor high words: K-major 128-byte swizzle (8-row groups 1024 bytes apart, version 1) and the scale atoms
    // (no swizzle, 8-line groups 128 bytes apart)
    constexpr uint64_t kOperandHi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
    constexpr uint64_t kScaleHi = (1ull << 16) | (8ull << 32) | (1ull << 46);
    if (ps.mma_geo != stride) { ps.mma_geo = stride; ps.mma_slot = 0; }
    uint32_t slot = uniform_u32(ps.mma_slot), bits = uniform_u32(ps.mma_bits), it = uniform_u32(ps.mma_it), tile_no = uniform_u32(ps.mma_tile);
    bool first_slot = true;
    for (int t = first; t < first + count; ++t) {
        const int n_tile = t % n_tiles;
        const uint32_t buf = tile_no & 1u, acc_phase = (tile_no >> 1) & 1u;
        if (!mbar_wait_warp(prog, ctl, &ctl->acc_empty[buf], acc_phase ^ 1u, stage_index)) return;
        tc_fence_after();
        const uint32_t d = tmem + buf * 128u;
        // Scale rows of a 64-wide B tile sit in the 32-row sub-columns 0 or 2 of their 128-row atom (the scale operand of
        // the MMA must start at an even sub-column); 32-wide tiles bring atoms of their own with the rows in sub-column 0.
        const uint32_t sfb_sub = block_n == 32 ? 0u : static_cast<uint32_t>((n_tile * block_n) & 127) >> 5;
        for (int ks = 0; ks < slots; ++ks) {
            const uint32_t s = slot;
            if (!mbar_wait_warp(prog, ctl, &ctl->full[s], (bits >> s) & 1u, stage_index)) return;
            if (stamp && first_slot && lane_id() == 0) stamp[4] = static_cast<long long>(global_ns());
            first_slot = false;
            const int groups = min(4 * kChunks, k_groups - ks * 4 * kChunks);
            const uint32_t a16 = data16 + s * stride16;
            const uint32_t sf_cols = tmem + kSfCol0 + (it & 3u) * (4 * kChunks * 8);
            if constexpr (OPERANDS != GEMM_NVFP4) {
                // BF16 / FP8 rows: the same descriptors and the same 32-byte advance along K, no scale factors
                if (elect_one()) {
#pragma unroll
                    for (int gi = 0; gi < 4 * kChunks; ++gi) {
                        if (gi < groups) {
                            const uint32_t chunk = static_cast<uint32_t>(gi) >> 2, sub = static_cast<uint32_t>(gi) & 3u;
                            const uint64_t da = kOperandHi | static_cast<uint64_t>(a16 + chunk * a_chunk16 + 2u * sub);
                            const uint64_t db = kOperandHi | static_cast<uint64_t>(a16 + off_b16 + chunk * b_chunk16 + 2u * sub);
                            const uint32_t acc = gi != 0 ? 1u : static_cast<uint32_t>(ks != 0);
                            if constexpr (OPERANDS == GEMM_BF16) tc_mma_f16(d, da, db, idesc, acc);
                            else tc_mma_f8(d, da, db, idesc, acc);
                        }
                    }
                    tc_commit(&ctl->empty[s]);
                }
            } else if (elect_one()) {
#pragma unroll
                for (int gi = 0; gi < 4 * kChunks; ++gi) {
                    if (gi < groups) {
                        const uint32_t chunk = static_cast<uint32_t>(gi) >> 2, sub = static_cast<uint32_t>(gi) & 3u;
                        const uint32_t sfa_t = sf_cols + gi * 8, sfb_t = sfa_t + 4;
                        tc_copy_sf(sfa_t, kScaleHi | static_cast<uint64_t>(a16 + off_sfa16 + gi * 32));
                        tc_copy_sf(sfb_t, kScaleHi | static_cast<uint64_t>(a16 + off_sfb16 + gi * 32));
                        // 64 FP4 = 32 bytes along K inside the 128-byte swizzled row: advance the start address by 2 units.
                        tc_mma_nvfp4(d, kOperandHi | static_cast<uint64_t>(a16 + chunk * a_chunk16 + 2u * sub),
                                     kOperandHi | static_cast<uint64_t>(a16 + off_b16 + chunk * b_chunk16 + 2u * sub), idesc, sfa_t,
                                     sfb_t + sfb_sub, gi != 0 ? 1u : static_cast<uint32_t>(ks != 0));
                    }
                }
                tc_commit(&ctl->empty[s]);     // slot reusable once these MMAs have read it
            }
            __syncwarp();
            bits ^= 1u << s;
            slot = s + 1 == ring ? 0u : s + 1;
            it++;
        }
        if (elect_one()) tc_commit(&ctl->acc_full[buf]);    // accumulator complete
        __syncwarp();
        tile_no++;
    }
    ps.mma_slot = slot; ps.mma_bits = bits; ps.mma_it = it; ps.mma_tile = tile_no;
    if (stamp && lane_id() == 0) stamp[5] = static_cast<long long>(global_ns());
}

// ---- epilogue helpers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(h);
}
__device__ __forceinline__ float gelu_sigmoid(float x) {
    // x * sigmoid(2u), u = sqrt(2/pi)(x + 0.044715 x^3): identical to the tanh form.
    float z = 1.5957691216057308f * x * (1.f + 0.044715f * x * x);
    return __fdividef(x, 1.f + __expf(-z));
}

// One 32-column chunk of one accumulator row (thread == row).
// (Instantiated per epilogue kind: each accumulator drain carries only its own arithmetic and registers.)
// LEAN: without the options only the BF16 model uses (rounding before the residual, GELU on BF16 output) and without ReLU^2.
template <int EPI, bool LEAN = false>
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmParams& g, const uint32_t (&raw)[32], int row, int col0,
                                                    bool row_ok, float row_scale, float row_shift, float& sumsq, float& sum) {
    float v[32];
    if (!row_ok) return;
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(raw[i]) * row_scale;
    if constexpr (EPI == EPI_BF16_EXT || EPI == EPI_FP4) {
        if (g.col_center) {
            // folded LayerNorm: subtract the row mean's share, mean * rstd * (sum over K of weight row n)
            const float4* c4 = reinterpret_cast<const float4*>(g.col_center + col0);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 c = __ldg(c4 + i);
                v[4 * i] = fmaf(row_shift, c.x, v[4 * i]);
                v[4 * i + 1] = fmaf(row_shift, c.y, v[4 * i + 1]);
                v[4 * i + 2] = fmaf(row_shift, c.z, v[4 * i + 2]);
                v[4 * i + 3] = fmaf(row_shift, c.w, v[4 * i + 3]);
            }
        }
    }
    if constexpr (EPI == EPI_GEGLU_FP4) {
        // interleaved (gate, up) column pairs -> 16 outputs = one scale block
        float h[16];
#pragma unroll
        for (int i = 0; i < 16; i++) h[i] = gelu_sigmoid(v[2 * i]) * v[2 * i + 1] * g.out_inv_gs;
        uint32_t code;
        uint2 bytes = quantize_block16(h, 0, code);
        const int out_col = col0 >> 1;
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(g.out) + static_cast<size_t>(row) * g.ldo + (out_col >> 1)) = bytes;
        g.out_scales[scale_offset(row, out_col >> 4, g.out_blocks)] = static_cast<uint8_t>(code);
        return;
    }
    if constexpr (EPI == EPI_GEGLU_BF16) {
        // bf16(gelu(bf16 gate)) * bf16(up), rounded once more: the BF16 model's GeGLU on interleaved (gate, up) columns
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float h0 = bf16_round(gelu_tanh(bf16_round(v[4 * i]))) * bf16_round(v[4 * i + 1]);
            const float h1 = bf16_round(gelu_tanh(bf16_round(v[4 * i + 2]))) * bf16_round(v[4 * i + 3]);
            w[i] = pack_bf16x2(h0, h1);
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.ldo + (col0 >> 1));
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        return;
    }
    const bool early_bias = !LEAN && EPI == EPI_BF16_EXT && g.bias && g.residual && g.round_before_residual;
    if (early_bias) {
        const uint4* b = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(g.bias) + col0);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint4 u = __ldg(b + i);
            float2 f;
            f = unpack_bf16x2(u.x); v[8 * i + 0] += f.x; v[8 * i + 1] += f.y;
            f = unpack_bf16x2(u.y); v[8 * i + 2] += f.x; v[8 * i + 3] += f.y;
            f = unpack_bf16x2(u.z); v[8 * i + 4] += f.x; v[8 * i + 5] += f.y;
            f = unpack_bf16x2(u.w); v[8 * i + 6] += f.x; v[8 * i + 7] += f.y;
        }
    }
    if (g.residual) {
        if (!LEAN && EPI == EPI_BF16_EXT && g.round_before_residual) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = bf16_round(v[i]);
        }
        const uint4* r = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(g.residual) +
                                                        static_cast<size_t>(row) * g.ldr + col0);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint4 u = __ldcg(r + i);
            float2 f;
            f = unpack_bf16x2(u.x); v[8 * i + 0] += f.x; v[8 * i + 1] += f.y;
            f = unpack_bf16x2(u.y); v[8 * i + 2] += f.x; v[8 * i + 3] += f.y;
            f = unpack_bf16x2(u.z); v[8 * i + 4] += f.x; v[8 * i + 5] += f.y;
            f = unpack_bf16x2(u.w); v[8 * i + 6] += f.x; v[8 * i + 7] += f.y;
        }
    }
    if (g.bias && !early_bias) {
        // (residual first, bias second: the order of the reference epilogue, whose BF16 result the tests reproduce bit for bit)
        const uint4* b = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(g.bias) + col0);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint4 u = __ldg(b + i);
            float2 f;
            f = unpack_bf16x2(u.x); v[8 * i + 0] += f.x; v[8 * i + 1] += f.y;
            f = unpack_bf16x2(u.y); v[8 * i + 2] += f.x; v[8 * i + 3] += f.y;
            f = unpack_bf16x2(u.z); v[8 * i + 4] += f.x; v[8 * i + 5] += f.y;
            f = unpack_bf16x2(u.w); v[8 * i + 6] += f.x; v[8 * i + 7] += f.y;
        }
    }
    if constexpr (EPI == EPI_F32) {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(g.out) + static_cast<size_t>(row) * g.ldo + col0);
#pragma unroll
        for (int i = 0; i < 8; i++) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        return;
    }
    if constexpr (EPI == EPI_STREAM) {
        // the residual stream in BF16 ...
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.ldo + col0);
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        // ... and, from the rounded values a norm stage would have read back, the sum of squares and the NVFP4 copy
        uint32_t words[4];
        uint32_t codes = 0;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            float h[16];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float2 f = unpack_bf16x2(w[8 * half + i]);
                sumsq = __fmaf_rn(f.x, f.x, sumsq);
                sumsq = __fmaf_rn(f.y, f.y, sumsq);
                sum += f.x;
                sum += f.y;
                h[2 * i] = f.x * g.out_inv_gs;
                h[2 * i + 1] = f.y * g.out_inv_gs;
            }
            uint32_t code;
            uint2 bytes = quantize_block16(h, 0, code);
            words[2 * half] = bytes.x;
            words[2 * half + 1] = bytes.y;
            codes |= code << (8 * half);
        }
        *reinterpret_cast<uint4*>(g.copy_fp4 + static_cast<size_t>(row) * g.ld_copy + (col0 >> 1)) = make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint16_t*>(g.out_scales + scale_offset(row, col0 >> 4, g.out_blocks)) = static_cast<uint16_t>(codes);
        return;
    }
    if constexpr (EPI == EPI_BF16 || EPI == EPI_BF16_EXT) {
        if (!LEAN && EPI == EPI_BF16_EXT && g.gelu_cols > 0) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = col0 + i < g.gelu_cols ? gelu_tanh(bf16_round(v[i])) : 0.f;
        }
        if (EPI == EPI_BF16_EXT && g.pad_from > 0) {
            // heads written pad_to columns apart (8-column pieces never straddle a head: pad_from is a multiple of 8)
            __nv_bfloat16* base = static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.ldo;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = col0 + 8 * i, head = c / g.pad_from;
                *reinterpret_cast<uint4*>(base + head * g.pad_to + (c - head * g.pad_from)) =
                    make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                               pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
            }
            return;
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.ldo + col0);
#pragma unroll
        for (int i = 0; i < 4; i++)
            dst[i] = make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                                pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
        return;
    }
    if constexpr (EPI == EPI_FP4) {
        if (g.act == 1) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = gelu_sigmoid(v[i]);
        } else if (!LEAN && g.act == 3) {
#pragma unroll
            for (int i = 0; i < 32; i++) { float r = fmaxf(v[i], 0.f); v[i] = r * r; }
        }
        uint32_t words[4];
        uint32_t codes = 0;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            float h[16];
#pragma unroll
            for (int i = 0; i < 16; i++) h[i] = v[16 * half + i] * g.out_inv_gs;
            uint32_t code;
            uint2 bytes = quantize_block16(h, 0, code);
            words[2 * half] = bytes.x;
            words[2 * half + 1] = bytes.y;
            codes |= code << (8 * half);
        }
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(g.out) + static_cast<size_t>(row) * g.ldo + (col0 >> 1)) =
            make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint16_t*>(g.out_scales + scale_offset(row, col0 >> 4, g.out_blocks)) = static_cast<uint16_t>(codes);
        return;
    }
    // EPI_QKV_ROPE: values are first rounded to BF16 (the projection output), then rotated.
    if constexpr (EPI == EPI_QKV_ROPE) {
        const int hd = g.head_dim, half = hd >> 1;
        const int kv0 = g.q_cols;                      // K columns [kv0, kv0+hd), V columns [kv0+hd, kv0+2hd)
        const bool is_v = col0 >= kv0 + hd;
        const bool is_k = !is_v && col0 >= kv0;
        const int in_head = is_v ? col0 - kv0 - hd : (is_k ? col0 - kv0 : col0 % hd);
        uint32_t packed[16];
        if (is_v) {
#pragma unroll
            for (int i = 0; i < 16; i++) packed[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
        } else {
            // Q and K heads are stored pair-interleaved: column 2i holds original dim i, column 2i+1 holds dim i+hd/2.
            const __nv_bfloat16* cs = static_cast<const __nv_bfloat16*>(g.rope_cos) + static_cast<size_t>(row) * hd;
            const __nv_bfloat16* sn = static_cast<const __nv_bfloat16*>(g.rope_sin) + static_cast<size_t>(row) * hd;
            // the 16 pairs of this chunk use table entries [dim0, dim0+16) and [dim0+half, dim0+half+16): 8 vector loads
            const int dim0 = in_head >> 1;
            uint32_t tc[2][8], ts[2][8];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint4* pc = reinterpret_cast<const uint4*>(cs + dim0 + h * half);
                const uint4* ps = reinterpret_cast<const uint4*>(sn + dim0 + h * half);
                const uint4 c0 = __ldg(pc), c1 = __ldg(pc + 1), s0 = __ldg(ps), s1 = __ldg(ps + 1);
                tc[h][0] = c0.x; tc[h][1] = c0.y; tc[h][2] = c0.z; tc[h][3] = c0.w;
                tc[h][4] = c1.x; tc[h][5] = c1.y; tc[h][6] = c1.z; tc[h][7] = c1.w;
                ts[h][0] = s0.x; ts[h][1] = s0.y; ts[h][2] = s0.z; ts[h][3] = s0.w;
                ts[h][4] = s1.x; ts[h][5] = s1.y; ts[h][6] = s1.z; ts[h][7] = s1.w;
            }
            // Packed BF16 arithmetic, two lanes = the two members of a rotation pair: with X = (x1, x2), C = (c1, c2),
            // S = (s1, s2) and X' = (-x2, x1) the rotated pair is  bf16(X * C) + bf16(X' * S)  lane by lane - every
            // product rounded to BF16 before the sum, as the reference's rotate-half does.
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;          // high or low halves of the two table words
                const uint32_t cw = __byte_perm(tc[0][i >> 1], tc[1][i >> 1], sel);
                const uint32_t sw = __byte_perm(ts[0][i >> 1], ts[1][i >> 1], sel);
                const uint32_t xw = pack_bf16x2(v[2 * i], v[2 * i + 1]);   // (x1, x2) rounded to BF16
                const uint32_t xr = __byte_perm(xw, xw, 0x1032u) ^ 0x00008000u;   // (-x2, x1)
                const __nv_bfloat162 p = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&xw), *reinterpret_cast<const __nv_bfloat162*>(&cw));
                const __nv_bfloat162 q = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&xr), *reinterpret_cast<const __nv_bfloat162*>(&sw));
                const __nv_bfloat162 o = __hadd2_rn(p, q);                  // (_rn: never contracted into a fused multiply-add)
                packed[i] = *reinterpret_cast<const uint32_t*>(&o);
            }
        }
        __nv_bfloat16* dst;
        if (is_v) dst = static_cast<__nv_bfloat16*>(g.cache_v) + static_cast<size_t>(g.cache_base + row) * hd + in_head;
        else if (is_k) dst = static_cast<__nv_bfloat16*>(g.cache_k) + static_cast<size_t>(g.cache_base + row) * hd + in_head;
        else dst = static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.ldo + col0;
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int i = 0; i < 4; i++) d4[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    }
}

// LEAN: the drain of the lean kernel variant; the residual-stream and plain BF16 drains there carry no row-statistics code
// (the host sends programs that give those two epilogues row statistics to the full variant).
template <int EPI, bool LEAN = false>
__device__ __forceinline__ void gemm_epilogue(const VmProgram& prog, Ctl* ctl, uint32_t tmem, const StageDesc& st,
                                              int stage_index, int first, int count, PipeState& ps, long long* stamp) {
    const GemmParams& g = st.p.gemm;
    constexpr bool kStats = !(LEAN && (EPI == EPI_STREAM || EPI == EPI_BF16));
    const int quarter = (threadIdx.x >> 5) & 3;          // TMEM lane quarter this warp may read
    const int lane = lane_id();
    for (int t = first; t < first + count; ++t) {
        const int m_tile = t / g.n_tiles, n_tile = t - m_tile * g.n_tiles;
        const uint32_t buf = ps.epi_tile & 1u, phase = (ps.epi_tile >> 1) & 1u;
        const int row = m_tile * 128 + quarter * 32 + lane;
        const bool row_ok = row < g.rows;
        if (EPI == EPI_QKV_ROPE && row_ok) {
            // while the MMAs run: bring this row's rotary table entries (constant data) close
            const int hd = g.head_dim, col_a = n_tile * g.block_n;
            if (col_a < g.q_cols + hd) {                                   // a Q or K tile
                const int in_head = col_a >= g.q_cols ? col_a - g.q_cols : col_a % hd;
                const __nv_bfloat16* cs = static_cast<const __nv_bfloat16*>(g.rope_cos) + static_cast<size_t>(row) * hd + (in_head >> 1);
                const __nv_bfloat16* sn = static_cast<const __nv_bfloat16*>(g.rope_sin) + static_cast<size_t>(row) * hd + (in_head >> 1);
                prefetch_l1(cs); prefetch_l1(cs + (hd >> 1)); prefetch_l1(sn); prefetch_l1(sn + (hd >> 1));
            }
        }
        if ((EPI == EPI_BF16_EXT || EPI == EPI_FP4) && g.col_center && lane < (g.block_n >> 5))
            prefetch_l1(g.col_center + n_tile * g.block_n + lane * 32);    // constant data: close by when the accumulator is ready
        // A single-tile instruction that reads row statistics (the few-row projections behind a folded norm, whose epilogue
        // is serial time): once the copy warp has seen the sources complete, the statistics are read and the row factor
        // computed while the operands are still on their way, instead of after the accumulator is ready.  (Requesting the
        // residual rows early as well was measured and lost: o_proj 7.9 vs 7.7 us.)
        const int chunks = g.block_n >> 5;
        // (compiled into the drains of the projections that stand behind a folded norm in the model; the others read their
        // statistics, if they are given any, once the accumulator is ready)
        constexpr bool kEarly = EPI == EPI_QKV_ROPE || EPI == EPI_GEGLU_FP4 || EPI == EPI_FP4 || EPI == EPI_BF16_EXT;
        const bool early = kEarly && count == 1 && (g.row_sumsq != nullptr || g.row_factor != nullptr);
        if (early) {
            if (!wait_deps_seen(prog, ctl, ps.gemm_seq, stage_index)) return;
        } else {
            if (!mbar_wait_warp(prog, ctl, &ctl->acc_full[buf], phase, stage_index)) return;
        }
        // alpha, times the row's 1/rms where the projection reads un-normalised rows (norm weight folded into B): given
        // as a factor, or as the producer's per-tile sums of squares (complete: the operands behind this accumulator
        // were only copied after the producer stage had finished)
        float row_scale = g.alpha, row_shift = 0.f, sumsq = 0.f, sum = 0.f;
        if (kStats && row_ok && g.row_factor) row_scale *= __ldcg(g.row_factor + row);
        if (kStats && row_ok && g.row_sumsq) {
            const float4* part = reinterpret_cast<const float4*>(g.row_sumsq + static_cast<size_t>(row) * g.sumsq_parts);
            const int quads = g.sumsq_parts >> 2;
            float total = 0.f;
            if ((EPI == EPI_BF16_EXT || EPI == EPI_FP4) && g.row_sum) {
                // LayerNorm: the per-tile sums (same layout) are requested together with the sums of squares; the mean
                // from the sums, the variance as E[x^2] - mean^2
                const float4* spart = reinterpret_cast<const float4*>(g.row_sum + static_cast<size_t>(row) * g.sumsq_parts);
                float stotal = 0.f;
                for (int i0 = 0; i0 < quads; i0 += 4) {
                    float4 q[4], sq[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        q[j] = i0 + j < quads ? __ldcg(part + i0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        sq[j] = i0 + j < quads ? __ldcg(spart + i0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {                    // fixed order: the same bits on every launch
                        if (i0 + j < quads) {
                            total += q[j].x; total += q[j].y; total += q[j].z; total += q[j].w;
                            stotal += sq[j].x; stotal += sq[j].y; stotal += sq[j].z; stotal += sq[j].w;
                        }
                    }
                }
                const float mean = stotal * g.sumsq_inv_width;
                const float rstd = rsqrtf(fmaxf(total * g.sumsq_inv_width - mean * mean, 0.f) + g.sumsq_eps);
                row_scale *= rstd;
                row_shift = -mean * rstd;
            } else {
                for (int i0 = 0; i0 < quads; i0 += 8) {              // eight loads in flight: one L2 round trip per 128 bytes
                    float4 q[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) q[j] = i0 + j < quads ? __ldcg(part + i0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < 8; j++) {                    // fixed order: the same bits on every launch
                        if (i0 + j < quads) { total += q[j].x; total += q[j].y; total += q[j].z; total += q[j].w; }
                    }
                }
                row_scale *= rsqrtf(total * g.sumsq_inv_width + g.sumsq_eps);
            }
        }
        if (early && !mbar_wait_warp(prog, ctl, &ctl->acc_full[buf], phase, stage_index)) return;
        tc_fence_after();
        if (stamp && t == first && threadIdx.x == 128) stamp[6] = static_cast<long long>(global_ns());
        const uint32_t taddr = tmem + buf * 128u + (static_cast<uint32_t>(quarter * 32) << 16);
        for (int c = 0; c < chunks; ++c) {
            uint32_t raw[32];
            tmem_ld32(taddr + c * 32, raw);
            tmem_ld_wait();
            if (c == chunks - 1) {
                // every column of this accumulator is in registers: hand the buffer back to the MMA lane
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
            }
            gemm_epilogue_chunk<EPI, LEAN>(g, raw, row, n_tile * g.block_n + c * 32, row_ok, row_scale, row_shift, sumsq, sum);
        }
        if (EPI == EPI_STREAM && row_ok) {
            g.sumsq_out[static_cast<size_t>(row) * g.sumsq_ld + n_tile] = sumsq;
            if (g.sum_out) g.sum_out[static_cast<size_t>(row) * g.sumsq_ld + n_tile] = sum;
        }
        // each epilogue warp publishes its own 32 rows (a GEMM tile counts 4 units): no CTA barrier on this path
        if (stamp && t == first + count - 1 && threadIdx.x == 128) stamp[7] = static_cast<long long>(global_ns());
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) publish_tile(prog, st, t);
        ps.epi_tile++;
    }
}

// Dispatch of one GEMM instruction onto the warp roles. Warps 2 and 3 have no role and fall through.
// LEAN: the kernel variant for programs made only of NVFP4 projections with the pi0 model's epilogues (the host checks
// this when it builds a program); it carries neither the dense issue loops nor the other drain loops.
template <bool LEAN>
__device__ __forceinline__ void gemm_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, uint32_t tmem,
                                                 const StageDesc& st, int stage_index, int first, int count,
                                                 PipeState& ps, long long* stamp) {
    const int warp = threadIdx.x >> 5;
    if (warp == 0) {
        gemm_producer(prog, ctl, data, st, stage_index, first, count, ps, stamp);
        if (stamp && threadIdx.x == 0) stamp[3] = static_cast<long long>(global_ns());
    } else if (warp == 1) {
        const int operands = st.p.gemm.operands;
        if (LEAN || operands == GEMM_NVFP4) gemm_mma<GEMM_NVFP4>(prog, ctl, data, tmem, st, stage_index, first, count, ps, stamp);
        else if (operands == GEMM_BF16) gemm_mma<GEMM_BF16>(prog, ctl, data, tmem, st, stage_index, first, count, ps, stamp);
        else gemm_mma<GEMM_FP8>(prog, ctl, data, tmem, st, stage_index, first, count, ps, stamp);
    } else if (warp >= 4) {
        const int epilogue = st.p.gemm.epilogue;            // one drain loop per epilogue kind: only its own arithmetic and registers
        if (epilogue == EPI_BF16) gemm_epilogue<EPI_BF16, LEAN>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else if (epilogue == EPI_STREAM) gemm_epilogue<EPI_STREAM, LEAN>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else if (epilogue == EPI_GEGLU_FP4) gemm_epilogue<EPI_GEGLU_FP4, LEAN>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else if (epilogue == EPI_FP4) gemm_epilogue<EPI_FP4, LEAN>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else if (epilogue == EPI_QKV_ROPE) gemm_epilogue<EPI_QKV_ROPE, LEAN>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else if (LEAN || epilogue == EPI_BF16_EXT) gemm_epilogue<EPI_BF16_EXT, LEAN>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else if (epilogue == EPI_F32) gemm_epilogue<EPI_F32>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        else gemm_epilogue<EPI_GEGLU_BF16>(prog, ctl, tmem, st, stage_index, first, count, ps, stamp);
        if (stamp && threadIdx.x == 128) stamp[2] = static_cast<long long>(global_ns());
    }
    ps.gemm_seq++;                                          // (every warp: the ordinal of the next GEMM instruction of this CTA)
}

}  // namespace pi0
