// Attention instruction: softmax(scale * Q K^T + mask) V for one (batch, head, 128-query tile, KV split).
//
// Eight warps, 16 query rows each. K/V stream through shared memory in 64-key chunks (cp.async, double buffered);
// QK^T and PV run on the tensor cores (mma.sync m16n8k16, BF16 in, FP32 accumulate) with an online softmax in the
// exp2 domain. MQA/GQA: the KV head is head / (heads / kv_heads). The pi0 suffix mask hides keys beyond `prefix` from
// query row 0 (the state token). With splits > 1 the tile writes un-normalised partials (o as BF16; m, l as FP32) for the merge;
// otherwise it normalises, rounds to BF16, and optionally quantises the rows to NVFP4 in the same pass.
#pragma once
#include "vm_core.cuh"

namespace pi0 {

constexpr int kAttnQRows = 128;
constexpr int kAttnChunk = 64;
// Shared memory an attention tile may touch (head dimension 256): Q, two K buffers, two V buffers of 264-element rows,
// and for split-KV tiles of at most 64 queries the partial-row staging area 4 KiB into the V buffers.
constexpr int kAttnOperandBytes = 3 * kAttnQRows * (256 + 8) * 2;
constexpr int kAttnStageEnd = 2 * kAttnQRows * (256 + 8) * 2 + 4096 + 8 * 16 * (128 + 16) * 2;
constexpr int kAttnSmemBytes = kAttnStageEnd > kAttnOperandBytes ? kAttnStageEnd : kAttnOperandBytes;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;       // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD>
__device__ __forceinline__ void attn_load_rows(__nv_bfloat16* dst, const __nv_bfloat16* src, int ld, int rows_total,
                                               int row0, int valid_rows, int head_dim) {
    // rows_total rows of HD (padded) elements into dst[row][HD+8]; rows >= valid_rows and columns >= head_dim are zero.
    constexpr int LD = HD + 8, CPR = HD / 8;
    for (int i = threadIdx.x; i < rows_total * CPR; i += kThreads) {
        const int r = i / CPR, c = i - r * CPR;
        const bool ok = r < valid_rows && c * 8 < head_dim;
        const __nv_bfloat16* s = ok ? src + static_cast<size_t>(row0 + r) * ld + c * 8 : src;
        cp_async16(dst + r * LD + c * 8, s, ok);
    }
}

template <int HD>
__device__ void attn_tile(const AttnParams& a, int tile, uint8_t* data, long long* stamp) {
    constexpr int LD = HD + 8;
    constexpr int KSTEPS = HD / 16;           // along the head dimension
    constexpr int ONT = HD / 8;               // output n-tiles
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(data);
    __nv_bfloat16* sK = sQ + kAttnQRows * LD;
    __nv_bfloat16* sV = sK + 2 * kAttnChunk * LD;

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
    const int nchunks = (max(k_end - k_begin, 0) + kAttnChunk - 1) / kAttnChunk;

    const int head_stride = a.hd_pad > a.head_dim ? a.hd_pad : a.head_dim;       // elements from one head to the next in q / k / v
    const __nv_bfloat16* qsrc = static_cast<const __nv_bfloat16*>(a.q) + static_cast<size_t>(batch) * a.q_batch_rows * a.ldq + head * head_stride;
    const __nv_bfloat16* ksrc = static_cast<const __nv_bfloat16*>(a.k) + static_cast<size_t>(batch) * a.kv_batch_rows * a.ldkv + kvh * head_stride;
    const __nv_bfloat16* vsrc = static_cast<const __nv_bfloat16*>(a.v) + static_cast<size_t>(batch) * a.kv_batch_rows * a.ldkv + kvh * head_stride;

    attn_load_rows<HD>(sQ, qsrc, a.ldq, kAttnQRows, q0, q_valid, a.head_dim);
    if (nchunks > 0) {
        attn_load_rows<HD>(sK, ksrc, a.ldkv, kAttnChunk, k_begin, min(kAttnChunk, k_end - k_begin), a.head_dim);
        attn_load_rows<HD>(sV, vsrc, a.ldkv, kAttnChunk, k_begin, min(kAttnChunk, k_end - k_begin), a.head_dim);
    }
    cp_async_commit();

    float o[ONT][4];
#pragma unroll
    for (int j = 0; j < ONT; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sl2 = a.scale * 1.4426950408889634f;
    // At most 64 query rows: warps 0-3 and 4-7 own the same four 16-row blocks and take the first and the second
    // 32 keys of every chunk; the two halves are combined through shared memory after the last chunk.
    const bool paired = q_valid <= 64;
    const int rb = paired ? (warp & 3) : warp;            // 16-row block of this warp
    const int khalf = paired ? (warp >> 2) : -1;          // the half of each chunk this warp takes (-1: both)
    const bool warp_active = rb * 16 < q_valid;
    const int row_a = rb * 16 + (lane >> 2);              // local query rows of this thread: row_a, row_a + 8
    const __nv_bfloat16* q_lane = sQ + (rb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8;

    for (int c = 0; c < nchunks; ++c) {
        const int buf = c & 1;
        if (c + 1 < nchunks) {
            const int kb = k_begin + (c + 1) * kAttnChunk;
            attn_load_rows<HD>(sK + (buf ^ 1) * kAttnChunk * LD, ksrc, a.ldkv, kAttnChunk, kb, min(kAttnChunk, k_end - kb), a.head_dim);
            attn_load_rows<HD>(sV + (buf ^ 1) * kAttnChunk * LD, vsrc, a.ldkv, kAttnChunk, kb, min(kAttnChunk, k_end - kb), a.head_dim);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (stamp && c == 0 && threadIdx.x == 0) stamp[4] = static_cast<long long>(global_ns());
        if (warp_active) {
            const __nv_bfloat16* kbuf = sK + buf * kAttnChunk * LD;
            const __nv_bfloat16* vbuf = sV + buf * kAttnChunk * LD;
            const int key_base = k_begin + c * kAttnChunk;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (key_base + half * 32 >= k_end) break;
                if (khalf >= 0 && half != khalf) continue;
                float s[4][4];
#pragma unroll
                for (int j = 0; j < 4; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
                const __nv_bfloat16* k_lane = kbuf + (half * 32 + (lane & 7) + (lane >> 4) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    uint32_t qa[4];
                    ldsm_x4(qa, q_lane + kk * 16);
#pragma unroll
                    for (int jp = 0; jp < 2; ++jp) {
                        uint32_t kb4[4];
                        ldsm_x4(kb4, k_lane + jp * 16 * LD + kk * 16);
                        mma_bf16(s[2 * jp], qa, kb4[0], kb4[1]);
                        mma_bf16(s[2 * jp + 1], qa, kb4[2], kb4[3]);
                    }
                }
                // scale, mask, online softmax
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 4; j++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int key = key_base + half * 32 + j * 8 + 2 * (lane & 3) + (e & 1);
                        const int qrow = q0 + row_a + (e >> 1) * 8;
                        bool visible = key < k_end;
                        if (a.prefix >= 0 && qrow == 0 && key > a.prefix) visible = false;
                        float val = visible ? s[j][e] * sl2 : -INFINITY;
                        s[j][e] = val;
                        mx[e >> 1] = fmaxf(mx[e >> 1], val);
                    }
                }
                float corr[2], m_use[2];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    const float m_new = fmaxf(m_run[r], mx[r]);
                    m_use[r] = m_new == -INFINITY ? 0.f : m_new;
                    corr[r] = exp2f(m_run[r] - m_use[r]);
                    m_run[r] = m_new;
                }
                float psum[2] = {0.f, 0.f};
                uint32_t pa[2][4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
                    const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
                    psum[0] += p0 + p1;
                    psum[1] += p2 + p3;
                    pa[j >> 1][(j & 1) * 2 + 0] = pack2_bf16(p0, p1);
                    pa[j >> 1][(j & 1) * 2 + 1] = pack2_bf16(p2, p3);
                }
#pragma unroll
                for (int r = 0; r < 2; r++) l_run[r] = l_run[r] * corr[r] + psum[r];
#pragma unroll
                for (int j = 0; j < ONT; j++) {
                    o[j][0] *= corr[0]; o[j][1] *= corr[0];
                    o[j][2] *= corr[1]; o[j][3] *= corr[1];
                }
                const __nv_bfloat16* v_lane = vbuf + (half * 32 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8;
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
                    for (int dp = 0; dp < ONT / 2; ++dp) {
                        uint32_t vb4[4];
                        ldsm_x4_trans(vb4, v_lane + ks * 16 * LD + dp * 16);
                        mma_bf16(o[2 * dp], pa[ks], vb4[0], vb4[1]);
                        mma_bf16(o[2 * dp + 1], pa[ks], vb4[2], vb4[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    if (nchunks == 0) { cp_async_wait<0>(); __syncthreads(); }
    if (stamp && threadIdx.x == 0) stamp[5] = static_cast<long long>(global_ns());

    // quad-reduce the row sums
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }

    // Columns of the output this warp finishes: all of them, or (paired warps) one half each - the two warps of a
    // row block swap the halves they do not keep, so the combine, the staging and the stores are shared by all
    // eight warps instead of falling on four.
    constexpr int HALF = ONT / 2;
    const bool upper = paired && khalf == 1;              // keeps n-tiles [HALF, ONT)
    if (paired) {
        // the loop's last barrier has passed: K and V buffers are free
        float4* xo = reinterpret_cast<float4*>(sK);                       // [2 senders][4 blocks][HALF][32 lanes]
        float4* xml = reinterpret_cast<float4*>(sV);                      // [2 senders][4 blocks][32 lanes]: m0, m1, l0, l1
        if (warp_active) {
#pragma unroll
            for (int j = 0; j < ONT; j++)
                if ((j >= HALF) != upper) xo[((khalf * 4 + rb) * HALF + (j % HALF)) * 32 + lane] = make_float4(o[j][0], o[j][1], o[j][2], o[j][3]);
            xml[(khalf * 4 + rb) * 32 + lane] = make_float4(m_run[0], m_run[1], l_run[0], l_run[1]);
        }
        __syncthreads();
        if (warp_active) {
            const float4 other = xml[((khalf ^ 1) * 4 + rb) * 32 + lane];
            const float om[2] = {other.x, other.y}, ol[2] = {other.z, other.w};
            float ca[2], cb[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const float m_new = fmaxf(m_run[r], om[r]);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                ca[r] = exp2f(m_run[r] - m_use);
                cb[r] = exp2f(om[r] - m_use);
                // the same operation order in both warps (first-half warp's term first): identical row sums
                l_run[r] = upper ? __fmaf_rn(ol[r], cb[r], __fmul_rn(l_run[r], ca[r])) : __fmaf_rn(l_run[r], ca[r], __fmul_rn(ol[r], cb[r]));
                m_run[r] = m_new;
            }
#pragma unroll
            for (int j = 0; j < ONT; j++) {
                if ((j >= HALF) == upper) {
                    const float4 x = xo[(((khalf ^ 1) * 4 + rb) * HALF + (j % HALF)) * 32 + lane];
                    o[j][0] = o[j][0] * ca[0] + x.x * cb[0]; o[j][1] = o[j][1] * ca[0] + x.y * cb[0];
                    o[j][2] = o[j][2] * ca[1] + x.z * cb[1]; o[j][3] = o[j][3] * ca[1] + x.w * cb[1];
                }
            }
        }
    }
    const int col_lo = upper ? HALF * 8 : 0;               // first output column this warp finishes

    if (a.splits > 1) {
        if (warp_active) {
            // The un-normalised rows go through shared memory (each warp's own slice of the now idle K/V buffers)
            // so that they leave as whole row pieces, 512 contiguous bytes per store instruction, instead of
            // 8-byte pieces scattered over eight rows.
            // Partials are kept as BF16: they are combined with FP32 weights and the result is rounded to BF16 (and
            // then to NVFP4) anyway, while the bytes a tile has to store and its peers have to fetch are what this
            // stage spends its time on (a CTA moves about 30 GB/s through ordinary loads and stores).
            constexpr int SLD = HD + 16, SLDH = HALF * 8 + 16;               // staged row lengths in BF16 elements
            // (paired warps: behind the exchange areas, which other warps may still be reading)
            __nv_bfloat16* stage = paired ? reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(sV) + 4096) + warp * 16 * SLDH
                                          : reinterpret_cast<__nv_bfloat16*>(sK) + warp * 16 * SLD;
            const int sld = paired ? SLDH : SLD;
            static_assert(kAttnStageEnd <= kDataBytes, "partial staging exceeds the data region");
#pragma unroll
            for (int r = 0; r < 2; r++) {
                __nv_bfloat16* srow = stage + ((lane >> 2) + r * 8) * sld + 2 * (lane & 3);
#pragma unroll
                for (int j = 0; j < ONT; j++)
                    if (!paired || (j >= HALF) == upper)
                        *reinterpret_cast<uint32_t*>(srow + (paired ? j % HALF : j) * 8) = pack2_bf16(o[j][2 * r], o[j][2 * r + 1]);
            }
            __syncwarp();
            __nv_bfloat16* po = reinterpret_cast<__nv_bfloat16*>(a.partial_o) + static_cast<size_t>(tile) * kAttnQRows * a.head_dim + col_lo;
            float* pml = a.partial_ml + static_cast<size_t>(tile) * kAttnQRows * 2;
            const int row0 = rb * 16;
            const int width = paired ? a.head_dim / 2 : a.head_dim;
            // 16-byte pieces: a row piece of `width` elements takes width / 8 lanes; the other lanes take the next row
            const int lanes_per_row = width >> 3, rows_per_pass = 32 / lanes_per_row;
            const int lr = lane / lanes_per_row, lc = (lane - lr * lanes_per_row) * 8;
            for (int r = lr; r < 16 && row0 + r < q_valid; r += rows_per_pass)
                *reinterpret_cast<uint4*>(po + static_cast<size_t>(row0 + r) * a.head_dim + lc) = *reinterpret_cast<const uint4*>(stage + r * sld + lc);
            if (!upper) {
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int row = row_a + r * 8;
                    if (row < q_valid && (lane & 3) == 0) {
                        pml[row * 2] = m_run[r];
                        pml[row * 2 + 1] = l_run[r];
                    }
                }
            }
        }
        return;
    }

    // normalise, round to BF16, stage the tile in the (now free) Q rows of this warp's row block
    if (warp_active) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
            __nv_bfloat16* dst = sQ + (row_a + r * 8) * LD + 2 * (lane & 3);
#pragma unroll
            for (int j = 0; j < ONT; j++)
                if (!paired || (j >= HALF) == upper)
                    *reinterpret_cast<uint32_t*>(dst + j * 8) = pack2_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
        }
    }
    __syncthreads();
    const size_t grow0 = static_cast<size_t>(batch) * a.q_batch_rows + q0;
    if (a.out) {
        const int cpr = a.head_dim / 8;
        for (int i = threadIdx.x; i < q_valid * cpr; i += kThreads) {
            const int r = i / cpr, c = i - r * cpr;
            uint4 val = *reinterpret_cast<const uint4*>(sQ + r * LD + c * 8);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + (grow0 + r) * a.ldo + head * a.head_dim + c * 8) = val;
        }
    }
    if (a.out_fp4) {
        const int bpr = a.head_dim / 16;
        for (int i = threadIdx.x; i < q_valid * bpr; i += kThreads) {
            const int r = i / bpr, b = i - r * bpr;
            const uint4* sp = reinterpret_cast<const uint4*>(sQ + r * LD + b * 16);
            uint4 u0 = sp[0], u1 = sp[1];
            const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
            float v[16];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
                v[2 * e] = f.x * a.out_inv_gs;
                v[2 * e + 1] = f.y * a.out_inv_gs;
            }
            uint32_t code;
            uint2 bytes = quantize_block16(v, 0, code);
            const int grow = static_cast<int>(grow0) + r;
            const int col = head * a.head_dim + b * 16;
            *reinterpret_cast<uint2*>(a.out_fp4 + static_cast<size_t>(grow) * a.ld_fp4 + (col >> 1)) = bytes;
            a.out_scales[scale_offset(grow, col >> 4, a.out_blocks)] = static_cast<uint8_t>(code);
        }
    }
}

// Split-KV merge: out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s.  A tile is 16 query rows of one head: one
// (row, 16-column block) per thread, all partial loads of a thread independent of each other.
constexpr int kMergeRows = 16;

// acc += w * (16 BF16 values of one partial row block)
__device__ __forceinline__ void merge_accumulate(float (&acc)[16], float w, const uint4 (&x)[2]) {
    const uint32_t u[8] = {x[0].x, x[0].y, x[0].z, x[0].w, x[1].x, x[1].y, x[1].z, x[1].w};
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[e]));
        acc[2 * e] += w * f.x;
        acc[2 * e + 1] += w * f.y;
    }
}

// Normalise one (row, 16-column block), round to BF16 and store it (BF16 and / or NVFP4 with its block scale).
__device__ __forceinline__ void merge_store(const MergeParams& g, int head, int grow, int b, const float (&acc)[16], float denom) {
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    float v[16];
#pragma unroll
    for (int e = 0; e < 16; e++) v[e] = bf16_round(acc[e] * inv);
    const int col = head * g.head_dim + b * 16;
    if (g.out) {
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; e++) w[e] = pack2_bf16(v[2 * e], v[2 * e + 1]);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(grow) * g.ldo + col);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
    if (g.out_fp4) {
#pragma unroll
        for (int e = 0; e < 16; e++) v[e] *= g.out_inv_gs;
        uint32_t code;
        uint2 bytes = quantize_block16(v, 0, code);
        *reinterpret_cast<uint2*>(g.out_fp4 + static_cast<size_t>(grow) * g.ld_fp4 + (col >> 1)) = bytes;
        g.out_scales[scale_offset(grow, col >> 4, g.out_blocks)] = static_cast<uint8_t>(code);
    }
}

// One (query row, 16-column block) of one group (a head of one 128-query tile); r counts rows inside the query tile.
__device__ __forceinline__ void merge_item(const MergeParams& g, int group, int r, int b) {
    {
        const int head = group % g.heads;
        const int grow = (group / g.heads) * kAttnQRows + r;          // row in the output
        const float* ml = g.partial_ml + (static_cast<size_t>(group) * g.splits * kAttnQRows + r) * 2;
        const __nv_bfloat16* po = reinterpret_cast<const __nv_bfloat16*>(g.partial_o) + (static_cast<size_t>(group) * g.splits * kAttnQRows + r) * g.head_dim + b * 16;
        float acc[16];
#pragma unroll
        for (int e = 0; e < 16; e++) acc[e] = 0.f;
        float denom = 0.f;
        if (g.splits <= 4) {
            // everything the item needs in one batch of independent loads: one round trip to L2 (the reference maximum
            // comes from the same pairs)
            float2 pair[4];
            uint4 x[4][2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int s = min(j, g.splits - 1);
                pair[j] = __ldcg(reinterpret_cast<const float2*>(ml + static_cast<size_t>(s) * kAttnQRows * 2));
                const uint4* src = reinterpret_cast<const uint4*>(po + static_cast<size_t>(s) * kAttnQRows * g.head_dim);
                x[j][0] = __ldcg(src);
                x[j][1] = __ldcg(src + 1);
            }
            const float big = fmaxf(fmaxf(pair[0].x, pair[1].x), fmaxf(pair[2].x, pair[3].x));
            const float ref = big == -INFINITY ? 0.f : big;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float w = j < g.splits ? exp2f(pair[j].x - ref) : 0.f;          // 0 for a fully masked split
                denom += w * pair[j].y;
                merge_accumulate(acc, w, x[j]);
            }
            merge_store(g, head, grow, b, acc, denom);
            return;
        }
        float big = -INFINITY;
#pragma unroll 8
        for (int s = 0; s < g.splits; s++) big = fmaxf(big, __ldcg(ml + static_cast<size_t>(s) * kAttnQRows * 2));
        const float ref = big == -INFINITY ? 0.f : big;
        // four splits at a time: their (m, l) pairs and their 16 output values are requested together, the
        // weights are computed afterwards, so no load waits for arithmetic
        for (int s0 = 0; s0 < g.splits; s0 += 4) {
            float2 pair[4];
            uint4 x[4][2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int s = min(s0 + j, g.splits - 1);
                pair[j] = __ldcg(reinterpret_cast<const float2*>(ml + static_cast<size_t>(s) * kAttnQRows * 2));
                const uint4* src = reinterpret_cast<const uint4*>(po + static_cast<size_t>(s) * kAttnQRows * g.head_dim);
                x[j][0] = __ldcg(src);
                x[j][1] = __ldcg(src + 1);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float w = s0 + j < g.splits ? exp2f(pair[j].x - ref) : 0.f;     // 0 for a fully masked split
                denom += w * pair[j].y;
                merge_accumulate(acc, w, x[j]);
            }
        }
        merge_store(g, head, grow, b, acc, denom);
    }
}

// The same for 5..16 splits with four adjacent lanes per (row, block): each lane fetches the partials of splits
// sub, sub + 4, sub + 8, sub + 12 in one batch of independent loads and the lanes combine with shuffles, so an item
// costs one round trip to L2 instead of one per four splits. All 32 lanes of a warp must call it together.
__device__ __forceinline__ void merge_item_wide(const MergeParams& g, int group, int r, int b, bool valid) {
    const int sub = threadIdx.x & 3;
    const int head = group % g.heads;
    const int grow = (group / g.heads) * kAttnQRows + r;
    const float* ml = g.partial_ml + (static_cast<size_t>(group) * g.splits * kAttnQRows + r) * 2;
    const __nv_bfloat16* po = reinterpret_cast<const __nv_bfloat16*>(g.partial_o) + (static_cast<size_t>(group) * g.splits * kAttnQRows + r) * g.head_dim + b * 16;
    float2 pair[4];
    uint4 x[4][2];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int sp = sub + 4 * j;
        const bool ok = valid && sp < g.splits;
        pair[j] = make_float2(-INFINITY, 0.f);
        x[j][0] = x[j][1] = make_uint4(0u, 0u, 0u, 0u);
        if (ok) {
            pair[j] = __ldcg(reinterpret_cast<const float2*>(ml + static_cast<size_t>(sp) * kAttnQRows * 2));
            const uint4* src = reinterpret_cast<const uint4*>(po + static_cast<size_t>(sp) * kAttnQRows * g.head_dim);
            x[j][0] = __ldcg(src);
            x[j][1] = __ldcg(src + 1);
        }
    }
    float big = fmaxf(fmaxf(pair[0].x, pair[1].x), fmaxf(pair[2].x, pair[3].x));
    big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, 1));
    big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, 2));
    const float ref = big == -INFINITY ? 0.f : big;
    float acc[16];
#pragma unroll
    for (int e = 0; e < 16; e++) acc[e] = 0.f;
    float denom = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float w = exp2f(pair[j].x - ref);               // 0 for an absent or fully masked split
        denom += w * pair[j].y;
        merge_accumulate(acc, w, x[j]);
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
        denom += __shfl_xor_sync(0xffffffffu, denom, o);
#pragma unroll
        for (int e = 0; e < 16; e++) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
    }
    if (valid && sub == 0) merge_store(g, head, grow, b, acc, denom);
}

// `rows` rows of one group, starting at `first_row` with stride `row_step`, all 16-column blocks: the whole CTA.
__device__ __forceinline__ void merge_rows(const MergeParams& g, int group, int first_row, int row_step, int rows) {
    const int bpr = g.head_dim / 16;
    const int items = rows * bpr;
    if (g.splits > 4 && g.splits <= 16) {
        for (int base = 0; base < items; base += kThreads / 4) {          // warp-uniform trip count
            const int i = base + (threadIdx.x >> 2);
            const bool valid = i < items;
            const int ii = valid ? i : 0;
            merge_item_wide(g, group, first_row + (ii / bpr) * row_step, ii % bpr, valid);
        }
    } else {
        for (int i = threadIdx.x; i < items; i += kThreads) merge_item(g, group, first_row + (i / bpr) * row_step, i % bpr);
    }
}

__device__ __forceinline__ void merge_tile(const MergeParams& g, int tile) {
    const int chunks = (min(g.nq, kAttnQRows) + kMergeRows - 1) / kMergeRows;
    const int group = tile / chunks, r0 = (tile - group * chunks) * kMergeRows;
    const int q_valid = min(kAttnQRows, g.nq - (group / g.heads) * kAttnQRows);
    merge_rows(g, group, r0, 1, max(0, min(kMergeRows, q_valid - r0)));
}

__device__ __forceinline__ void merge_instruction(const VmProgram& prog, Ctl* ctl, const StageDesc& st, int stage_index,
                                                  int first, int count) {
    for (int t = first; t < first + count; ++t) {
        merge_tile(st.p.merge, t);
        cta_publish_tile(prog, st, t);
    }
}

// One attention instruction.  With a fused split-KV merge the tiles of a head of one query tile (one per split,
// resident on different SMs at the same time) meet on a per-group ticket counter that grows by `splits` per launch; once all partials of
// the head are published, every tile merges its share of the query rows (row % splits == split), so the merge
// costs neither a stage of its own nor a serial tail on one SM.
template <int HDP, bool MASK>
__device__ bool attn_tile_tc(const VmProgram& prog, Ctl* ctl, const AttnParams& a, int tile, uint8_t* data, uint32_t tmem,
                             uint32_t uses, int stage, long long* stamp, const StageDesc* deps, int dep_first, int dep_count);

// LEAN: kernel variant for programs whose attention stages all run on the tcgen05 tiles (no mma.sync tile code).
// The instruction waits for its sources itself (the instruction loop does not): the tcgen05 tile does so after its
// index arithmetic, the other tiles up front.
template <bool LEAN>
__device__ __forceinline__ void attn_instruction(const VmProgram& prog, Ctl* ctl, uint8_t* data, uint32_t tmem, uint32_t& tc_tiles,
                                                 const StageDesc& st, int stage_index, int first, int count, long long* stamp) {
    const AttnParams& a = st.p.attn;
    if (!(LEAN || a.tc) && !cta_wait_sources(prog, ctl, st, stage_index, first, count, stamp)) return;
    for (int t = first; t < first + count; ++t) {
        long long* stamp_t = t == first ? stamp : nullptr;
        const StageDesc* deps = t == first ? &st : nullptr;
        if (LEAN || a.tc) {
            bool ok = false;
            if (!LEAN && a.mask) {
                if constexpr (!LEAN)
                    ok = a.hd_pad > 128 ? attn_tile_tc<256, true>(prog, ctl, a, t, data, tmem, tc_tiles, stage_index, stamp_t, deps, first, count)
                                        : attn_tile_tc<128, true>(prog, ctl, a, t, data, tmem, tc_tiles, stage_index, stamp_t, deps, first, count);
            } else {
                ok = a.hd_pad > 128 ? attn_tile_tc<256, false>(prog, ctl, a, t, data, tmem, tc_tiles, stage_index, stamp_t, deps, first, count)
                                    : attn_tile_tc<128, false>(prog, ctl, a, t, data, tmem, tc_tiles, stage_index, stamp_t, deps, first, count);
            }
            tc_tiles++;
            if (!ok) return;                                   // uniform: a wait gave up, the abort flag is set
        } else if constexpr (!LEAN) {
            if (a.head_dim > 128) attn_tile<256>(a, t, data, stamp_t);
            else attn_tile<80>(a, t, data, stamp_t);
        }
        if (a.splits > 1 && a.fused_merge) {
            const int split = t % a.splits, group = t / a.splits;         // group: one head of one 128-query tile
            // The barrier orders every thread's partial stores before thread 0's release increment below, which
            // is cumulative at GPU scope: no per-thread fence is needed.
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int target = static_cast<unsigned int>(a.splits) * prog.epoch;
                red_release_add(a.tickets + group, 1u);
                int ok = 1;
                unsigned long long start = 0;           // the global timer is slow to read: first consulted after 64 polls
                for (uint32_t spin = 1; ld_acquire(a.tickets + group) < target; ++spin) {
                    __nanosleep(20);
                    if ((spin & 63u) != 0u) continue;
                    const unsigned long long now = global_ns();
                    if (start == 0) start = now;
                    if (ctl->abort || now - start > prog.wait_budget_ns || ld_relaxed_int(&prog.status->abort)) {
                        report(prog, 1, stage_index, group, ld_acquire(a.tickets + group), target);
                        ctl->abort = 1;
                        ok = 0;
                        break;
                    }
                }
                ctl->flag = ok;
            }
            __syncthreads();
            if (!ctl->flag) return;                            // uniform: the abort flag is set, the caller leaves the loop
            if (stamp_t && threadIdx.x == 0) stamp_t[6] = static_cast<long long>(global_ns());
            MergeParams g;
            g.partial_o = a.partial_o; g.partial_ml = a.partial_ml;
            g.heads = a.heads; g.nq = a.nq; g.head_dim = a.head_dim; g.splits = a.splits;
            g.out = a.out; g.ldo = a.ldo;
            g.out_fp4 = a.out_fp4; g.out_scales = a.out_scales; g.out_blocks = a.out_blocks;
            g.out_inv_gs = a.out_inv_gs; g.ld_fp4 = a.ld_fp4;
            const int q_valid = min(kAttnQRows, a.nq - (group / a.heads) * kAttnQRows);
            const int my_rows = (q_valid - split + a.splits - 1) / a.splits;       // rows split, split+splits, ...
            merge_rows(g, group, split, a.splits, max(0, my_rows));
            if (stamp_t && threadIdx.x == 0) stamp_t[7] = static_cast<long long>(global_ns());
        }
        cta_publish_tile(prog, st, t);
    }
}

}  // namespace pi0
