// Shared host/device description of a pi0 VM program.
//
// A program is a list of stages (one operator instance each) plus, per worker
// CTA, a static stream of instructions {opcode, stage, first_tile, tile_count}.
// Dependencies between stages are expressed with monotonically growing counters:
// every finished tile adds 1 to the counter of its 128-row band, and a consumer
// waits until the bands it reads have reached epoch * expected.
#pragma once
#include <stdint.h>
#include <vector_types.h>

namespace pi0 {

constexpr int kThreads = 256;            // 8 warps per worker CTA
constexpr int kMaxSources = 4;
constexpr int kBandRows = 128;

enum OpKind : int {
    OP_NONE = 0,
    OP_GEMM = 1,        // tcgen05 GEMM (NVFP4 block-scaled, BF16 or FP8 operands), fused epilogue
    OP_NORM = 2,        // LayerNorm / RMSNorm (or plain copy) -> NVFP4 / BF16
    OP_ATTN = 3,        // softmax(QK^T)V on tensor cores, optional split-KV partials
    OP_MERGE = 4,       // split-KV merge (+ NVFP4 quantize)
    OP_PATCH = 5,       // FP32 patch embedding (14x14x3 conv) + bias + position embedding
    OP_EMBED = 6,       // token embedding rows * sqrt(width)
    OP_LINEAR32 = 7,    // small FP32 linear (+bias, SiLU, RMS factor, Euler update)
    OP_SUFFIX = 8,      // assemble expert input rows: state token + action tokens
    OP_PROBE = 9,       // resource probe: every warp reports the CTA's tensor-memory base for every instruction
    OP_ATTN_PREP = 10,  // attention operands with bias / rotate-half RoPE applied, copied into the padded head layout
    OP_KINDS
};

enum SrcMode : int { SRC_SAME_BAND = 0, SRC_ALL_BANDS = 1 };

enum GemmEpilogue : int {
    EPI_F32 = 0,        // alpha*acc -> FP32
    EPI_BF16 = 1,       // alpha*acc + bias + residual -> BF16 (one rounding)
    EPI_FP4 = 2,        // alpha*acc + bias (+residual) [GELU|ReLU^2] -> NVFP4 + swizzled scales
    EPI_GEGLU_FP4 = 3,  // gelu_tanh(gate)*up on interleaved columns -> NVFP4, width N/2
    EPI_QKV_ROPE = 4,   // BF16, RoPE on Q/K heads, K/V rows appended to the KV cache
    EPI_GEGLU_BF16 = 5, // bf16(gelu_tanh(bf16 gate)) * bf16(up) on interleaved columns -> BF16, width N/2
    EPI_BF16_EXT = 6,   // EPI_BF16 with the BF16 model's options: round before the residual add, GELU with a column limit
    EPI_STREAM = 7      // EPI_BF16 (residual stream) + an NVFP4 copy of the stored rows + per-tile sums of their squares
};

enum GemmOperands : int {
    GEMM_NVFP4 = 0,     // packed E2M1 + E4M3 block scales, kind::mxf4nvf4, 64 K-elements per MMA
    GEMM_BF16 = 1,      // BF16 rows, kind::f16, 16 K-elements per MMA
    GEMM_FP8 = 2        // E4M3 rows, kind::f8f6f4, 32 K-elements per MMA
};

struct GemmParams {
    const void* tmap_a;          // CUtensorMap in global memory: A rows as bytes [M_pad, row_bytes] (NVFP4: K/2, BF16: 2K, FP8: K)
    const void* tmap_b;          // CUtensorMap: B rows [N_pad, row_bytes]
    const uint8_t* sfa;          // swizzled E4M3 block scales of A (NVFP4 only)
    const uint8_t* sfb;
    int operands;                // GemmOperands
    int m_tiles, n_tiles;        // 128-row x block_n-column output tiles
    int k_groups;                // row_bytes / 32: one MMA each (64 FP4, 16 BF16 or 32 FP8 elements of K)
    int block_n;                 // 128 (default), 64 or 32
    int b_tiled;                 // B stored tile-major: block (n_tile, k_stage) is block_n contiguous 128-byte rows
    int a_box_rows;              // rows of A copied per tile: 128, or fewer (a multiple of 8) when there are fewer logical rows
    int ring_stages;             // operand ring of this GEMM: slots in flight (2..kMaxStages) ...
    int slot_stride;             // ... bytes from one slot to the next (multiple of 1024) ...
    int off_b, off_sfa, off_sfb; // ... and where B, the A scales and the B scales start inside a slot (A starts at 0)
    float alpha;                 // global_scale(A) * global_scale(B)
    int epilogue;
    int act;                     // EPI_FP4: 0 none, 1 GELU(tanh), 3 ReLU^2
    const float* row_factor;     // FP32 [M] multiplied into every accumulator row (1/rms of the input row) or null
    int round_before_residual;   // EPI_BF16: (+bias) round to BF16, then add the residual and round again
    int gelu_cols;               // EPI_BF16: > 0 applies GELU(tanh) to bf16(value) in columns < gelu_cols and stores 0 beyond
    int pad_from, pad_to;        // EPI_BF16_EXT: > 0 stores column c at (c / pad_from) * pad_to + c % pad_from (heads of pad_from
                                 // columns written pad_to apart, the gap left untouched); pad_from a multiple of 8
    // EPI_STREAM: the BF16 rows are also quantised, un-normalised, to NVFP4 (out_scales / out_blocks / out_inv_gs describe
    // the copy) and every tile stores the sum of squares of its part of each row, so that the projection that follows can
    // apply the RMS normalisation as a row factor instead of running behind a norm stage
    uint8_t* copy_fp4;           // packed codes [M_pad, ld_copy bytes]
    int ld_copy;
    float* sumsq_out;            // FP32 [M_pad, sumsq_ld] (sumsq_ld >= n_tiles: slot n of a row belongs to column tile n)
    float* sum_out;              // FP32 [M_pad, sumsq_ld] or null: per-tile sums of the same rounded rows (LayerNorm consumers)
    int sumsq_ld;
    // consumer side: row factor rsqrt(sum(row_sumsq[row, 0..sumsq_parts)) * sumsq_inv_width + sumsq_eps), times alpha.
    // With row_sum (per-tile sums, same layout) the rows are LayerNorm-ed instead: mean m and variance from the two sums,
    // acc * alpha * rstd - m * rstd * col_center[n], where col_center[n] is the sum over K of the weight row n as the MMA
    // reads it (the weight columns carry the norm's gamma, the bias its beta)
    const float* row_sumsq;
    const float* row_sum;
    const float* col_center;     // FP32 [N]
    int sumsq_parts;
    float sumsq_inv_width, sumsq_eps;
    int rows;                    // logical rows (rows >= this are written as zero codes / skipped)
    void* out;                   // FP32 / BF16 / packed FP4
    int ldo;                     // elements (FP32/BF16) or bytes (FP4) per output row
    const void* bias;            // BF16 [N] or null
    const void* residual;        // BF16 [M, ldr] or null
    int ldr;
    uint8_t* out_scales;         // swizzled scales of the FP4 output
    int out_blocks;              // 16-wide blocks per output row (scale layout width)
    float out_inv_gs;            // 1 / global scale of the FP4 output
    // EPI_QKV_ROPE
    const void* rope_cos;        // BF16 [rows, head_dim]
    const void* rope_sin;
    void* cache_k;               // BF16 [cache_rows, head_dim]
    void* cache_v;
    int q_cols;                  // heads * head_dim (0 when the projection has no Q part)
    int head_dim;
    int cache_base;              // first cache row written by this projection
    uint32_t idesc;              // tcgen05 instruction descriptor
};

struct NormParams {
    const void* in;              // BF16 [rows, width]
    const float* gamma;          // FP32 [width] or null (RMS: already 1+w)
    const float* beta;           // FP32 [width] or null
    int rows, width;
    int mode;                    // 0 = RMSNorm, 1 = LayerNorm, 2 = none (quantize only)
    int round_norm;              // round normalised value to BF16 before quantisation
    float eps;
    float inv_gs;                // 1 / global scale of the FP4 output
    int policy;                  // 0 nearest (activations), 1 ceil (weights)
    uint8_t* out;                // packed FP4 [rows_pad, width/2] or null
    uint8_t* out_scales;         // swizzled scales
    int out_blocks;              // blocks per row of the scale layout (>= width/16)
    void* out_bf16;              // optional BF16 copy of the normalised rows
    int ld_in;                   // input row stride in elements
    int ld_out;                  // FP4 output row stride in bytes
    int rows_per_tile;           // 4 (RMSNorm stages) or 8 (LayerNorm, quantise-only); two warps share a row
    const void* residual;        // BF16 [rows, width] added to the input before the statistics, or null
    void* residual_out;          // BF16 [rows, width]: the sum (what the next residual connection reads), or null
    int round_residual;          // continue from the BF16-rounded sum (what a separate add kernel would have stored)
    const float* inv_scale;      // FP32 [width] multiplied in after gamma / beta (AWQ-style inverse smoothing scale) or null
    uint8_t* out_fp8;            // E4M3 [rows, width] of value / global scale (format 8), or null
    float* out_factor;           // FP32 [rows]: only 1 / sqrt(mean square + eps) of every row (format 17), or null
};

struct AttnParams {
    const void* q;               // BF16; element (b, r, h, d) at q + ((b*q_batch_rows + r)*ldq + h*head_dim + d)
    const void* k;               // BF16; key (b, j, hk, d) at k + ((b*kv_batch_rows + j)*ldkv + hk*head_dim + d)
    const void* v;
    void* out;                   // BF16 [.., heads*head_dim] (ldo elements) or null when partial
    int ldq, ldkv, ldo;
    int batches, nq, nk;         // queries / keys per batch
    int q_batch_rows, kv_batch_rows;
    int heads, kv_heads, head_dim;
    float scale;
    int prefix;                  // >= 0: pi0 suffix mask, query 0 sees keys [0, prefix]; -1: no mask
    int splits;                  // KV splits (1 = none)
    uint16_t* partial_o;         // BF16 bits [tasks, 128, head_dim] when splits > 1: un-normalised partial rows
    float* partial_ml;           // FP32 [tasks, 128, 2]
    // fused NVFP4 quantisation of the output (splits == 1)
    uint8_t* out_fp4;
    uint8_t* out_scales;
    int out_blocks;
    float out_inv_gs;
    int ld_fp4;
    int fp4_pitch;               // columns one head occupies in the FP4 output (a multiple of 16 >= head_dim; tcgen05 tiles only otherwise head_dim)
    // splits > 1 with the merge inside the attention stage: one arrival ticket per (128-query tile, head); once all
    // splits of a group have arrived every tile merges its share of the rows. Tickets are program counters (they grow
    // by `splits` per launch and are reset with them); 0 / null selects the separate OP_MERGE stage
    unsigned int* tickets;
    int fused_merge;
    // Tensor-core path (tcgen05, operands by TMA): chosen by the host when the geometry allows it
    int tc;                      // 0: mma.sync tiles, 1: tcgen05 tiles
    int hd_pad;                  // elements one head occupies in q / k / v (128 or 256; >= head_dim, the rest zeros)
    int q_box, k_box;            // rows per TMA box of Q (<= 128) and of K / V (keys per tile rounded up to 16, <= 256)
    const uint8_t* mask;         // bool [batches, nq, nk], 1 = visible, or null (tcgen05 tiles of the full kernel variant only)
    const void* tmap_q;          // CUtensorMaps in global memory: BF16 [rows, ld] with boxes of 64 columns
    const void* tmap_k;
    const void* tmap_v;
};

struct MergeParams {
    const uint16_t* partial_o;
    const float* partial_ml;
    int heads, nq, head_dim, splits;
    void* out;                   // BF16 [nq, heads*head_dim] or null
    int ldo;
    uint8_t* out_fp4;
    uint8_t* out_scales;
    int out_blocks;
    float out_inv_gs;
    int ld_fp4;
};

struct PatchParams {
    const float* images;         // FP32 [views,224,224,3] (null: bound at launch, slot 1)
    const float* weight;         // FP32 [588, width]  (k = (py*14+px)*3 + c)
    const float* bias;           // FP32 [width]
    const float* pos;            // FP32 [256, width]
    void* out;                   // BF16 [views*256, width]
    int views, width;
};

struct EmbedParams {
    const long long* tokens;     // null: bound at launch (slot 4)
    const void* table;           // BF16 [vocab, width]
    void* out;                   // BF16 rows [row_base, row_base+count)
    int count, width, row_base, vocab;
    float scale;
};

struct Linear32Params {
    const void* x;               // FP32 or BF16 [rows, ldx]; null: launch slot
    const float* w;              // FP32 [n, k] row major
    const float* bias;           // FP32 [n] or null
    const float* prev;           // Euler: FP32 [rows, n] previous value (null with slot: launch noise)
    void* out;                   // FP32 [rows, ldo] or BF16
    int rows, n, k, ldx, ldo;
    int x_bf16, out_bf16;
    int silu, rms;               // rms: multiply by rsqrt(mean(x^2)+eps) of the input row
    int euler;                   // out = prev + dt * value   (separately rounded mul and add)
    int slot, prev_slot;         // 0 pointer, 2 state, 3 noise
    int x_row_offset;            // first input row
    int row_block;               // rows per tile: 32 or 16
    const float* row0_src;       // optional FP32 [n] row ...
    void* row0_dst;              // ... stored as BF16 [n] by the tiles of the first row block (null: none)
    float dt, eps;
};

struct SuffixParams {
    const float* state_emb;      // FP32 [1, width]
    const float* action_emb;     // FP32 [chunk, width]
    void* out;                   // BF16 [rows_pad, width]
    int chunk, width;
};

// Operand preparation of the attention operator: part p (0 Q, 1 K, 2 V) has rows[p] rows of heads[p] heads;
// dst[r, h, :] = rope(src[r, h, :] + bias[h, :]) in FP32, rounded to BF16, every head on `pitch` elements (zeros behind
// head_dim: the destination is zeroed once at set-up).  Rotate-half with the first half of the tables' angles.
struct PrepParams {
    const void* src[3];          // BF16, row r / head h at src + r * ld_src + h * src_pitch
    void* dst[3];                // BF16, row r / head h at dst + r * ld_dst + h * pitch
    const void* bias[3];         // BF16 [heads, head_dim] or null
    const void* cos[2];          // BF16 [rows, head_dim] for Q and K, or null
    const void* sin[2];
    int rows[3], heads[3], ld_src[3], ld_dst[3];
    int head_dim, src_pitch, pitch;
};

struct ProbeParams {
    int* out;                    // int32 [tiles, 16]: slots w and w + 8 of a tile belong to warp w
};

struct alignas(16) StageDesc {
    int kind;
    int tiles;
    int bands;
    int counter_base;
    int band_div;                // band(tile) = min(tile / band_div, bands - 1)
    int src[kMaxSources];
    int src_mode[kMaxSources];
    int aux_base, aux_count;     // extra program counters owned by the stage (attention: one ticket per head)
    int units_per_tile;          // counter increments one finished tile contributes (GEMM: one per epilogue warp)
    // Filled by the host when the program is built, so a consumer polls counters without touching its producers'
    // descriptors: first counter, band count and the per-launch contribution of a full / of the last band.
    int src_counter_base[kMaxSources];
    int src_bands[kMaxSources];
    unsigned int src_expected[kMaxSources];
    unsigned int src_expected_last[kMaxSources];
    union {
        GemmParams gemm;
        NormParams norm;
        AttnParams attn;
        MergeParams merge;
        PatchParams patch;
        EmbedParams embed;
        Linear32Params lin;
        SuffixParams suffix;
        ProbeParams probe;
        PrepParams prep;
    } p;
};

// Written by the device when a bounded wait expires or a check fails.
struct VmStatus {
    int code;                    // 0 ok, 1 dependency wait timed out, 2 pipeline barrier timed out, 3 bad instruction
    int worker, stage, band;
    unsigned int observed, expected;
    int abort;                   // set once; every wait polls it
    int pad;
};

struct LaunchInputs {
    const float* images;
    const float* state;
    const float* noise;
    const long long* tokens;
};

struct VmProgram {
    const StageDesc* stages;
    const int4* code;            // [workers][length] compacted instructions
    unsigned int* counters;
    const unsigned int* expected;
    VmStatus* status;
    long long* timings;          // optional [workers][length][8] global-timer stamps (ns): start, sources ready, end, copies issued,
                                 // first operands landed, MMAs issued, first accumulator ready, last stores done
    int num_stages, length;
    unsigned int epoch;
    int stage_begin, stage_end;  // execute stages in [begin, end); sources < begin are treated as complete
    unsigned long long wait_budget_ns;
    LaunchInputs in;
    int* debug;                  // optional host-mapped progress marks, one word per warp (diagnostics)
};

}  // namespace pi0
