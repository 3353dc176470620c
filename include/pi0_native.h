/* C ABI of libpi0_native.so - the B200 (sm_100a) pi0 inference engine.
 *
 * Every function returns a cudaError_t as int (0 = success).  Argument errors return
 * cudaErrorInvalidValue (1); a device that is not compute capability 10.x, or more workers than SMs,
 * returns cudaErrorInvalidConfiguration (9); a handle used on another device returns
 * cudaErrorInvalidDevice (101); launching on a capturing stream returns
 * cudaErrorStreamCaptureUnsupported (900).  On failure *handle is set to NULL.  destroy_*(NULL) succeeds.
 *
 * Ownership: the caller owns every tensor it passes (weights, activations, caches, outputs) and keeps it
 * alive while the handle lives; the library owns only its programs, counters, tensor maps and status words.
 * Calls on one handle must be stream ordered.  All pointers are device pointers unless noted.
 *
 * The entry points mirror the ctypes surface of the reference project (file:line of the interface each one
 * replaces is given); extensions that the reference has no counterpart for are marked "extension".
 */
#ifndef PI0_NATIVE_H
#define PI0_NATIVE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------------
 * NVFP4 block-scaled GEMM:  out[M,N] = epilogue(alpha * deq(A)[M,K] . deq(B)[N,K]^T)
 * A, B: packed E2M1 (two per byte, low nibble first) [M, K/2], [N, K/2];  sfa, sfb: E4M3 block scales in the
 * 128x4 swizzled atom layout;  M, N multiples of 128, K a multiple of 64;  default output FP32 [M, N].
 * Replaces: native_pi0/nvfp4_probe.cu:293-401 (create_resident_fp4, launch_resident_fp4,
 * configure_resident_fp4_bf16, configure_resident_fp4_quantized, resident_fp4_resources,
 * destroy_resident_fp4), bound in native_pi0/primitives.py:57-112.
 */
int create_resident_fp4(void** handle, const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                        int m, int n, int k, int workers, float alpha);
int launch_resident_fp4(void* handle, void* stream);
/* BF16 output [M, N] = alpha*acc + residual + bias, rounded once.  bias BF16 [N], residual BF16 [M, N]. */
int configure_resident_fp4_bf16(void* handle, const void* bias, const void* residual, void* out);
/* NVFP4 output: packed [M, No/2] + swizzled scales; activation 0 none, 1 GELU(tanh), 2 GeGLU over interleaved
 * gate/up columns (No = N/2), 3 ReLU^2; otherwise No = N.  global_scale is the output's tensor scale. */
int configure_resident_fp4_quantized(void* handle, const void* bias, const void* residual, void* out, void* scales,
                                     float global_scale, int activation);
int resident_fp4_resources(void* handle, int* values, int count);
int destroy_resident_fp4(void* handle);
/* extension: fused QKV epilogue - BF16 Q [M, ldq] (heads stored pair-interleaved), rotate-half RoPE with BF16
 * cos/sin [rows, head_dim], K and V rows written to cache_k/cache_v [*, head_dim] at row cache_base + r.
 * Replaces the BF16 path's configure_dense_qkv_rope (native_pi0/dense.cu:231-253). */
int configure_resident_fp4_qkv_rope(void* handle, void* out_q, int ldq, const void* cos, const void* sin, void* cache_k,
                                    void* cache_v, int q_cols, int head_dim, int cache_base);
/* extension: residual-stream epilogue.  out BF16 [M, N] = alpha*acc + residual + bias as configure_resident_fp4_bf16;
 * the rounded rows are also quantised, un-normalised, to NVFP4 (copy_fp4 packed [M, N/2], copy_scales swizzled with
 * N/16 blocks per row, tensor scale copy_global_scale), and sumsq FP32 [M, N / tile width] receives, per output tile,
 * the sum of squares of its part of each row.  With configure_resident_fp4_row_rms on the projection that reads the
 * copy (whose weight has the norm weight folded in) this replaces an RMSNorm stage between the two projections
 * (the reference folds the norm the same way for its BF16 model: native_pi0/model.py:163-164,203-204 and the
 * rms_factors of native_pi0/dense.cu:86-89). */
int configure_resident_fp4_stream(void* handle, const void* bias, const void* residual, void* out, void* copy_fp4,
                                  void* copy_scales, float copy_global_scale, float* sumsq);
/* extension: every accumulator row r is multiplied by rsqrt(sum(sumsq[r, 0..parts)) / width + eps); parts % 4 == 0.
 * The sum runs in index order, so the factor has the same bits on every launch. */
int configure_resident_fp4_row_rms(void* handle, const float* sumsq, int parts, int width, float eps);
/* extension: LayerNorm folded the same way.  configure_resident_fp4_stream_sums (after configure_resident_fp4_stream and
 * the tile width) makes the producing projection also leave the per-tile SUMS of its rounded rows, and gives both
 * statistics arrays a row stride of ld floats (>= N / tile width, a multiple of 4; slots beyond the tile count are never
 * written: zero them once).  configure_resident_fp4_row_layernorm on the reading projection turns every accumulator row
 * r into rstd_r * (alpha * acc - mean_r * center[n]), mean and variance (E[x^2] - mean^2) from the two sums over `width`
 * values, center FP32 [N] = the sum over K of weight row n as the MMA reads it (dequantised); the weight columns carry
 * the norm's gamma and the bias, added afterwards as always, its beta (bias + W beta).  Offered by the BF16 epilogue
 * with extended options (head-padded store, GELU column limit) and by the NVFP4-output epilogue. */
int configure_resident_fp4_stream_sums(void* handle, float* sums, int ld);
int configure_resident_fp4_row_layernorm(void* handle, const float* sumsq, const float* sums, int parts, int width, float eps,
                                         const float* center);
/* extension: logical row count (rows >= this are never stored; with at most 64 rows only 64 rows of A are
 * copied per tile) and output tile width: 128, 64, or 32 (NVFP4 operands only).  With 32-wide tiles the weight scales
 * given at creation are read in a layout of their own: one 512-byte atom per (32-row tile, group of four 16-element
 * blocks) - [N / 32][K / 64][512] - holding the tile's 32 rows in the first 32-row sub-column of the atom (bytes
 * 16 r + b for row r, block b) and zeros elsewhere, i.e. four times the bytes of the standard layout.  Narrow tiles are
 * for projections of a few rows, whose time is the bytes one SM takes in and the serial epilogue of one tile. */
int configure_resident_fp4_rows(void* handle, int rows);
int configure_resident_fp4_tile(void* handle, int block_n);
/* extension: tiled = 1 declares that B is stored tile-major (K a multiple of 256): for every output tile n and every
 * 256-wide K stage s the block_n x 128 bytes of that block are contiguous, at byte offset
 * ((n * K/256 + s) * block_n) * 128; one TMA box is then one contiguous read.  Set the tile width first. */
int configure_resident_fp4_weight_layout(void* handle, int tiled);

/* ------------------------------------------------------------------------------------------------------
 * Dense projection:  out[M,N] = epilogue(alpha * A[M,K] . B[N,K]^T), A and B both BF16 (fp8 == 0) or both FP8 E4M3
 * (fp8 == 1), row-major with K contiguous, FP32 accumulation on tcgen05 (kind::f16 / kind::f8f6f4) through the same
 * TMA ring and tensor-memory accumulators as the NVFP4 GEMM.  M, N multiples of 128; K a multiple of 64 (BF16) or 128
 * (FP8); all pointers 16-byte aligned.  bf16 == 1: BF16 output, else FP32; bias BF16 [N] and residual BF16 [M, N]
 * are added in FP32 (residual first, then bias) before the single rounding.
 * Replaces: native_pi0/dense.cu:142-253 (create_dense, launch_dense, destroy_dense and the six configure_dense_*),
 * bound in native_pi0/dense.py:8-129; the GEMM itself replaces native_pi0/tcgen_probe.cu:35-125.
 */
int create_dense(void** handle, const void* a, const void* b, void* out, const void* bias, const void* residual,
                 int m, int n, int k, int workers, int fp8, int bf16, float alpha);
int launch_dense(void* handle, void* stream);
int destroy_dense(void* handle);
/* The configure calls below need a BF16 output.  (The reference also demands BF16 operands; these epilogues do not
 * depend on the operand format, so they accept FP8 and NVFP4 projection handles as well.) */
/* (+bias) is rounded to BF16 first, then the residual is added and the sum rounded again (needs a residual). */
int configure_dense_round_before_residual(void* handle);
/* Interleaved (gate, up) column pairs -> compact BF16 [M, N/2] = bf16(bf16(gelu_tanh(bf16 gate)) * bf16 up); no bias,
 * no residual, N a multiple of 256. */
int configure_dense_geglu(void* handle, void* compact_output);
/* GELU(tanh) of the BF16-rounded value in columns < logical_columns, zeros beyond (no residual). */
int configure_dense_gelu(void* handle, int logical_columns);
/* Every accumulator row r is multiplied by factors[r] (FP32 [M]): the 1/rms of an un-normalised input row whose
 * norm weight has been folded into B (no bias, no residual). */
int configure_dense_rms_factor(void* handle, const float* factors);
/* At most 64 logical rows (M == 128): only 64 rows of A are copied per tile and rows >= 64 are never stored. */
int configure_dense_skinny(void* handle);
/* Fused QKV epilogue of a [M, key_offset + 512] projection: Q heads (columns < key_offset) stay in `out`, rotated;
 * the K head (columns key_offset..+256) is rotated and written to cache_k row cache_base + r; the V head to cache_v.
 * cos/sin BF16 [rows, 256].  Layout note: the rotation is done on ADJACENT column pairs, so the rows of the Q and K
 * heads of B must be ordered (0, 128, 1, 129, ...) inside each head (the Python wrapper does this); Q in `out` and K in
 * the cache are then in that same pair order, which attention over them does not see. */
int configure_dense_qkv_rope(void* handle, const void* cos, const void* sin, void* cache_k, void* cache_v, int logical_rows,
                             int key_offset, int cache_base);
/* extension: head-padded BF16 output - column c is stored at (c / from) * to + c % from of a row of ld elements, so
 * heads of `from` columns start `to` columns apart (from, to multiples of 8); the gaps are never written: zero the
 * buffer once and they stay zero.  Gives 72-wide SigLIP heads the 128-element pitch the tcgen05 attention tiles read
 * (configure_attention_head_pad).  No residual. */
int configure_dense_head_pad(void* handle, int from, int to, int ld);
/* extension: logical row count and output tile width (128 or 64) of a dense projection.  The NVFP4 GEMM's
 * configure_resident_fp4_{bf16, quantized, qkv_rope, rows, tile} calls accept dense handles too (a dense projection
 * may emit NVFP4 for an NVFP4 consumer); configure_resident_fp4_weight_layout does not. */
int configure_dense_rows(void* handle, int rows);
int configure_dense_tile(void* handle, int block_n);

/* ------------------------------------------------------------------------------------------------------
 * LayerNorm / RMSNorm producer -> NVFP4 (format 4: packed codes + swizzled scales), FP8 E4M3 (format 8: value / global
 * scale, [rows, width] bytes), BF16 (format 16) or only the FP32 row factor 1 / sqrt(mean square + eps) (format 17,
 * output FP32 [rows]).  Optional fused residual: input + residual (BF16 [rows, width]) is normalised, the sum is stored
 * to residual_output when given, and with round_residual the statistics continue from its BF16 rounding.  gamma / beta
 * / inverse_scale (an AWQ-style per-channel factor applied after gamma and beta) are FP32 [width]; RMSNorm gamma
 * already holds 1+w.
 * Replaces: native_pi0/norm.cu:138-176 (create_norm, launch_norm, destroy_norm), bound in
 * native_pi0/normalization.py:43-66.  Not offered: FP16 input (fp16 == 1) and legacy_ties == 1 (a rounding variant of
 * an older quantiser) return cudaErrorInvalidValue.
 */
int create_norm(void** handle, const void* input, const void* residual, const float* gamma, const float* beta,
                const float* inverse_scale, void* residual_output, void* output, void* scales, int rows, int width,
                int workers, int fp16, int format, int layer, int round_norm, int round_residual, int legacy_ties,
                float epsilon, float global_scale);
int launch_norm(void* handle, void* stream);
int destroy_norm(void* handle);
/* extension: skip normalisation (plain BF16 -> NVFP4 quantiser); policy 0 nearest, 1 ceil (weights). */
int configure_norm_quantize_only(void* handle, int policy);
/* extension: also store the normalised rows as BF16 [rows, width]. */
int configure_norm_bf16_copy(void* handle, void* out_bf16);
/* extension: input row stride (elements), FP4 output row stride (bytes), scale-layout blocks per row. */
int configure_norm_layout(void* handle, int ld_in, int ld_out, int out_blocks);

/* ------------------------------------------------------------------------------------------------------
 * Attention (MHA / GQA / MQA), BF16 in, FP32 softmax, BF16 out.
 * Replaces: native_pi0/attention.cu:544-666 (create_attention, launch_attention, destroy_attention,
 * configure_attention_splits, configure_attention_cache, attention_resources), bound in
 * native_pi0/attention.py:60-110.  BF16 only (fp16 == 0); head_dim a multiple of 8 up to 256 (the reference: 64, 72,
 * 128, 256).  prefix >= 0 selects the pi0 suffix mask (query 0 sees keys [0, prefix]); prefix < 0: none.
 * Element (b, r, h, d) of q is q[((b*nq + r)*ldq) + h*hd + d]; keys likewise with ldkv and nk.
 * Optional arguments as in the reference: q_bias / k_bias / v_bias BF16 [heads, head_dim] ([kv_heads, head_dim] for K and
 * V) added to the operands; q_cos / q_sin BF16 [batches * nq, head_dim] and k_cos / k_sin [batches * nk, head_dim]:
 * rotate-half RoPE with the first half of each table; mask: bytes [batches, nq, nk], non-zero = visible, applied on top
 * of the suffix mask (a query with no visible key gives a zero row).  Biases, tables and head sizes other than 72 / 256
 * add an operand-preparation stage (attention_prepare_handle) that writes Q, K and V - bias added, rotated, FP32
 * arithmetic rounded to BF16 - into library-owned buffers with every head on a 128- or 256-element pitch.  Prepared
 * operands and the mask run on the tcgen05 tiles only: at most 256 keys per tile (use configure_attention_splits beyond
 * that; cudaErrorInvalidValue otherwise), no KV cache, and programs that contain them launch the full kernel variant.
 */
int create_attention(void** handle, const void* q, const void* k, const void* v, const void* q_bias, const void* k_bias,
                     const void* v_bias, const void* q_cos, const void* q_sin, const void* k_cos, const void* k_sin,
                     void* out, const void* mask, int batches, int nq, int nk, int heads, int kv_heads, int head_dim,
                     int ldq, int ldkv, int out_ld, int fp16, int workers, int prefix, float scale);
int launch_attention(void* handle, void* stream);
int destroy_attention(void* handle);
int attention_resources(int* values, int count);
/* Split the key range into `splits` parts; partial (o, m, l) go to library-owned scratch and a merge stage
 * produces the output. */
int configure_attention_splits(void* handle, int splits);
/* extension: with splits > 1, let the tile that finishes last for a head merge the partials itself instead of running
 * a separate merge stage (call after configure_attention_splits and configure_attention_fp4_output). */
int configure_attention_fused_merge(void* handle, int enable);
/* Read keys/values from a KV cache [rows, head_dim] (BF16) instead of k/v; rows = total keys visible. */
int configure_attention_cache(void* handle, const void* cache_k, const void* cache_v, int rows, int prefix_rows);
/* extension: also quantise the output rows to NVFP4: every head occupies `pitch` columns of the FP4 rows (head_dim unless
 * configure_attention_fp4_pitch was called first), ld_bytes >= heads * pitch / 2, out_blocks >= heads * pitch / 16. */
int configure_attention_fp4_output(void* handle, void* out_fp4, void* scales, int ld_bytes, int out_blocks,
                                   float global_scale);
/* extension: head pitch of the FP4 output (a multiple of 16 with head_dim <= pitch <= the padded head size of
 * configure_attention_head_pad); columns from head_dim up to the pitch are stored as zeros, so a projection whose weight has
 * zero columns at the same places reads the rows as they are - 72-wide SigLIP heads on an 80-column pitch feed the output
 * projection without a separate quantisation stage.  Before configure_attention_fp4_output; a pitch other than head_dim
 * exists only in the unsplit tcgen05 tiles (cudaErrorInvalidValue otherwise). */
int configure_attention_fp4_pitch(void* handle, int pitch);
/* extension: tile implementation.  -1 (default) picks the tcgen05 tiles (Q, K, V by TMA, S / P / O in tensor memory)
 * whenever the geometry allows them - heads that occupy 128 or 256 elements in memory, at most 256 keys per tile (use KV
 * splits beyond that) - and the mma.sync tiles otherwise; 0 forces the mma.sync
 * tiles, 1 the tcgen05 tiles (cudaErrorInvalidValue when the geometry does not allow them). */
int configure_attention_path(void* handle, int path);
/* extension: every head occupies `elements` (128 or 256) elements in q, k and v, zeros beyond head_dim (what a projection
 * with configure_dense_head_pad writes); the row strides given at creation must cover heads * elements.  Lets 72-wide
 * SigLIP heads run on the tcgen05 tiles.  Output rows stay head_dim wide. */
int configure_attention_head_pad(void* handle, int elements);
/* extension: handle of the operand-preparation stage owned by an attention handle created with biases, rotary tables
 * or a head size other than 72 / 256 (NULL otherwise); a program lists it as a stage in front of the attention. */
int attention_prepare_handle(void* handle, void** prepare);
/* extension: cudaSuccess when the handle can run as configured - an operator with prepared operands or a mask whose key
 * range per tile exceeds 256 (or whose path was forced to mma.sync) cannot; launches and programs refuse it too. */
int attention_validate(void* handle);
/* extension: handle of the merge stage owned by an attention handle with splits > 1 (NULL otherwise). */
int attention_merge_handle(void* handle, void** merge);
/* Development diagnostics of a split attention handle (splits >= 2), never part of a forward pass.
 * Replaces: native_pi0/attention.cu:629-656 (attention_split_diagnostics, attention_poison_partials).
 * attention_poison_partials fills the partial rows and their (max, sum) statistics with 0xFF bytes on `stream`, so
 * that a launch which read a partial it had not written itself would produce NaNs.  attention_split_diagnostics
 * returns, per (128-query tile, head) group, how many split tiles have arrived over all stand-alone launches so
 * far (capacity >= number of groups) and the launch count `epoch`; every count equals splits * epoch after a clean
 * launch. */
int attention_poison_partials(void* handle, void* stream);
int attention_split_diagnostics(void* handle, unsigned long long* counts, int capacity, unsigned int* epoch);

/* Split-KV attention that allocates nothing.  No counterpart in the reference.
 * For callers that cannot call cudaMalloc when they need the result - a control loop that must not block on the
 * driver's allocator, or a process whose device memory all belongs to another runtime's pool.  The split-KV partials
 * live in a fixed device array inside the library (about 4.1 MiB per GPU that loads it, held until exit) instead of
 * an allocated buffer; the call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 * q BF16 [nq, heads*256] (row stride ldq), k and v BF16 [nk, kv_heads*256] (row stride ldkv), out BF16 [nq, heads*256]
 * (row stride out_ld); prefix >= 0 selects the pi0 suffix mask, < 0 none.  Limits (cudaErrorInvalidValue beyond them):
 * head_dim == 256, nq <= 128, splits >= 1, heads * splits <= 64; all four pointers 16-byte aligned.  Same arithmetic as
 * create_attention + configure_attention_splits on the mma.sync tiles (configure_attention_path 0); with splits == 1 every head is one tile that writes `out` directly
 * and the array is not touched.
 * The first call on a device looks up the array's device address and raises the kernel's shared-memory limit; make
 * that first call before any stream capture begins.  All calls on a GPU share the one array, which keeps the last
 * call's partials: every word read is rewritten first by the same call, but two calls that overlap on the GPU
 * (different streams) race on it - serialise them. */
int attention_split_noalloc(const void* q, const void* k, const void* v, void* out, int nq, int nk, int heads, int kv_heads,
                            int head_dim, int ldq, int ldkv, int out_ld, int prefix, int splits, float scale, void* stream);

/* ------------------------------------------------------------------------------------------------------
 * Small FP32 operators (the reference's NativeTensorOp modes 5, 6, 8, 10: native_pi0/model.cu:95-183,
 * created from native_pi0/model.py:95-104,136-145).  extension: each is an operator handle of its own.
 */
/* patch embedding: images FP32 [views,224,224,3] (NULL = bound at launch), weight FP32 [588, width] with
 * k = (dy*14+dx)*3+c, bias FP32 [width], pos FP32 [256, width], out BF16 [views*256, width]. */
int create_patch_embed(void** handle, const float* images, const float* weight, const float* bias, const float* pos,
                       void* out, int views, int width, int workers);
/* token embedding rows: out[row_base+i, :] = bf16(table[tokens[i], :] * scale); tokens NULL = bound at launch. */
int create_token_embed(void** handle, const long long* tokens, const void* table, void* out, int count, int width,
                       int row_base, int vocab, float scale, int workers);
/* out[r, n] = f(sum_k x[r + x_row_offset, k] w[n, k]);  flags: 1 x is BF16, 2 out is BF16, 4 SiLU, 8 multiply by
 * rsqrt(mean(x^2)+eps), 16 Euler update out = prev + dt*value.  slot 0: x pointer, 2: launch state, 3: launch
 * noise; prev_slot 3: previous value is the launch noise. */
int create_linear32(void** handle, const void* x, const float* w, const float* bias, const float* prev, void* out,
                    int rows, int n, int k, int ldx, int ldo, int flags, int slot, int prev_slot, int x_row_offset,
                    float dt, float eps, int workers);
/* extension: the tiles of the operator's first row block also store src (FP32 [n]) as BF16 [n] at dst; with the output
 * pointing one row below dst this makes the state token row 0 of the action-expert input without a stage of its own. */
int configure_linear32_extra_row(void* handle, const float* src, void* dst);
/* expert input rows: row 0 = state embedding, rows 1..chunk = action embeddings, BF16 [*, width]. */
int create_suffix_assemble(void** handle, const float* state_emb, const float* action_emb, void* out, int chunk,
                           int width, int workers);
int launch_op(void* handle, void* stream);      /* any operator handle, as a one-stage program */
int destroy_op(void* handle);
/* tiles, 128-row bands and K-cost of an operator handle (what the stream compiler needs). */
int op_geometry(void* handle, int* tiles, int* bands, int* cost);

/* ------------------------------------------------------------------------------------------------------
 * Whole-model program: one persistent launch over static per-worker instruction streams.
 * Replaces: native_pi0/model.cu:188-303 (create_native_model, launch_native_model,
 * read_native_model_timings, destroy_native_model), bound in native_pi0/model.py:286,303-305,318-337.
 * NativeSpec is versioned against the reference's struct (native_pi0/model.cu:8-12): every stage is an
 * operator handle, with up to four producer stages and a wait mode each (0 = same 128-row band, 1 = all).
 * code: int32 [workers, length, 32] = {opcode, stage, first_tile, tile_count, 0...}; opcode 0 ends a stream.
 */
typedef struct NativeSpec {
    int kind;            /* 0 GEMM, 1 attention, 2 norm, 3 small operator, 4 split-KV merge */
    void* handle;
    int sources[4];      /* producer stage index or -1 */
    int modes[4];
} NativeSpec;
int create_native_model(void** handle, int count, const NativeSpec* specs, const int* code, int workers, int length);
int launch_native_model(void* handle, void* stream, const float* images, const float* state, const float* noise,
                        const long long* tokens);
/* extension: run only stages [begin, end); producers before `begin` are taken as complete.  new_epoch != 0
 * starts a new forward pass (first range of a pass). */
int launch_native_model_range(void* handle, void* stream, const float* images, const float* state, const float* noise,
                              const long long* tokens, int begin, int end, int new_epoch);
/* per-instruction global-timer stamps (ns), int64 [workers, length, 8] = {start, producers ready, end, copies
 * issued, first operands landed, MMAs issued, first accumulator ready, last stores done} (the last five only for
 * GEMM and attention instructions); enable before the launch to record.  `count` must be 8 * workers * length.
 * The reference's slots are int32 clock samples (native_pi0/model.cu:292-298); these are 64-bit nanoseconds. */
int enable_native_model_timings(void* handle, int enable);
int read_native_model_timings(void* handle, long long* out, size_t count);
/* extension: synchronises the device and returns {code, worker, stage, band, observed, expected, aborted, epoch};
 * code 0 ok, 1 dependency wait timed out, 2 pipeline barrier timed out, 3 bad instruction.  A non-zero status
 * is cleared and the counters are reset so the handle stays usable. */
int read_native_model_status(void* handle, int* values, int count);
/* extension: counters uint32 [n] and the expected value per counter for the current epoch. */
int read_native_model_counters(void* handle, unsigned int* counts, unsigned int* expected, int n, int* total);
/* extension: which kernel variant the program launches: *lean = 1 for the smaller kernel that carries only the NVFP4
 * projections with the pi0 model's epilogues and the tcgen05 attention tiles (chosen when every stage allows it), 0 for
 * the kernel with every operator and option.  Same protocol, same results. */
int native_model_kernel_variant(void* handle, int* lean);
/* extension (debugging): host-mapped progress marks, one word per warp of every worker, written as the warp moves
 * through its instruction loop (which instruction it has entered, where in the teardown it is); readable while a
 * launch is still running.  Off by default; while on, the program launches the full kernel variant. */
int enable_native_model_debug(void* handle, int enable);
int read_native_model_debug(void* handle, int* out, int n);      /* n >= workers * 8 */
/* extension: time budget of every device-side wait in nanoseconds (default 2e9). */
int set_native_model_wait_budget(void* handle, unsigned long long nanoseconds);
int destroy_native_model(void* handle);

/* Chain of GEMM stages in one launch with row-band counters.
 * Replaces: native_pi0/native.cu:174-236 (create_native_linear, launch_native_linear, read_native_linear,
 * destroy_native_linear), bound in native_pi0/linear.py:37-45. */
int create_native_linear(void** handle, int count, void* const* stages, const int* parents, const int* code, int workers,
                         int length);
int launch_native_linear(void* handle, void* stream);
int read_native_linear(void* handle, unsigned long long* counters, int count, unsigned long long* epoch);
int destroy_native_linear(void* handle);

/* ------------------------------------------------------------------------------------------------------
 * extension: stand-alone BF16 -> NVFP4 quantiser (setup-time weight packing on the device).
 * in BF16 [rows, ld_in]; out packed [rows, width/2]; scales swizzled with `out_blocks` blocks per row;
 * policy 0 nearest, 1 ceil.  Bit-exact with pack_nvfp4 (native_pi0/quantization.py:48-93). */
int quantize_nvfp4(const void* in, void* out, void* scales, int rows, int width, int ld_in, int out_blocks,
                   float global_scale, int policy, void* stream);

/* ------------------------------------------------------------------------------------------------------
 * Launch counting through CUPTI driver callbacks (proves "one launch per forward").
 * Replaces: native_pi0/launch_trace.cpp:25-47, bound in native_pi0/launch_trace.py:7-17.  Returns CUptiResult. */
int begin_launch_trace(void** handle);
int end_launch_trace(void* handle, int* count, char* symbol, int symbol_bytes);
const char* launch_trace_error(int code);

/* ------------------------------------------------------------------------------------------------------
 * Self-contained probes with HOST pointers: each call allocates device memory, copies the operands, launches, copies
 * the results back and frees.  Development and validation aids, never on the path of a forward pass.
 * Replaces: native_pi0/tcgen_probe.cu (run_tcgen_probe, run_fp8_probe, run_k_probe, run_grid_probe; bound by
 * scripts/validate_tcgen.py:26-83), native_pi0/nvfp4_probe.cu:293-299 (scripts/validate_nvfp4.py:31-72) and
 * native_pi0/vm_probe.cu:34 (scripts/validate_vm.py:23-36).
 * GEMM probes: a [m, k] and b [n, k] row major - BF16 (precision 0), FP8 E4M3 (precision 1) or packed NVFP4 with
 * swizzled scale atoms sa / sb; out FP32 [repetitions, m, n], every repetition one launch = alpha * a b^T with
 * alpha = a_scale * w_scale (1 for run_tcgen_probe); m, n multiples of 128, k a multiple of 64; the single-tile probes
 * are m = n = 128 (k = 64 unless given).
 * run_vm_probe: `workers` CTAs run `instructions` instructions each in one launch; host_output int32 [workers,
 * instructions, 16] receives the CTA's tensor-memory base + 1 per instruction and reporting slot (this kernel has eight
 * warps: warp w fills slots w and w + 8), so every entry is positive and all entries of a worker are equal. */
int run_tcgen_probe(const void* a, const void* b, float* out, int repetitions);
int run_fp8_probe(const void* a, const void* b, float* out, int repetitions, float a_scale, float w_scale);
int run_k_probe(const void* a, const void* b, float* out, int repetitions, int k, int precision, float a_scale, float w_scale);
int run_grid_probe(const void* a, const void* b, float* out, int repetitions, int m, int n, int k, int workers, int precision,
                   float a_scale, float w_scale);
int run_nvfp4_probe(const void* a, const void* b, const void* sa, const void* sb, float* out, int repetitions, float alpha, int k);
int run_nvfp4_grid_probe(const void* a, const void* b, const void* sa, const void* sb, float* out, int repetitions, int m, int n,
                         int k, int workers, float alpha);
int run_vm_probe(int workers, int instructions, int* host_output);

#ifdef __cplusplus
}
#endif
#endif /* PI0_NATIVE_H */
