// Host runtime and C ABI of libpi0_native.so: operator handles, program assembly (counters, expected
// contributions, compacted instruction streams), TMA tensor maps and the single persistent launch.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "../../include/pi0_native.h"
#include "vm_kernel.cuh"

namespace pi0 {
namespace {

constexpr uint32_t kOpMagic = 0x7069304f;       // "pi0O"
constexpr uint32_t kProgramMagic = 0x70693050;  // "pi0P"

// Current device, checked to be compute capability 10.x. The capability is looked up once per device (one attribute
// query), so steady-state callers pay only cudaGetDevice.
int check_device(int* device_out) {
    static int major_of[64] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    int major = device >= 0 && device < 64 ? major_of[device] : 0;
    if (major == 0) {
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) return e;
        if (device >= 0 && device < 64) major_of[device] = major;
    }
    if (major != 10) return cudaErrorInvalidConfiguration;
    *device_out = device;
    return cudaSuccess;
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int sm_count(int device) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
    return n;
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}
// Operand matrix [rows, row_bytes] seen as [chunk][row][128 bytes]: a box is kChunks consecutive 128-byte chunks of K
// (256 FP4, 64 BF16 or 128 FP8 elements each) of box_rows rows, each chunk landing as box_rows 128-byte rows with the
// 128-byte swizzle.
int encode_operand(CUtensorMap* map, const void* base, int rows, size_t row_bytes_in, int box_rows) {
    EncodeTiled fn = encoder();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t row_bytes = static_cast<cuuint64_t>(row_bytes_in);
    cuuint64_t dims[3] = {128u, static_cast<cuuint64_t>(rows), (row_bytes + 127) / 128};
    cuuint64_t strides[2] = {row_bytes, 128u};
    cuuint32_t box[3] = {128u, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(kChunks)};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}
// Tile-major weight: [blocks * block_n rows][128 bytes]; a box is kChunks consecutive blocks of one output tile.
int encode_tiled(CUtensorMap* map, const void* base, int total_rows, int box_rows) {
    EncodeTiled fn = encoder();
    if (!fn) return cudaErrorNotSupported;
    cuuint64_t dims[2] = {128u, static_cast<cuuint64_t>(total_rows)};
    cuuint64_t strides[1] = {128u};
    cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// BF16 matrix [rows, ld] with boxes of 64 columns (128 bytes, 128-byte swizzle) x box_rows rows: attention operands.
int encode_bf16_rows(CUtensorMap* map, const void* base, size_t rows, int ld, int box_rows) {
    EncodeTiled fn = encoder();
    if (!fn) return cudaErrorNotSupported;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2u};
    cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

struct Program;

struct Op {
    uint32_t magic = kOpMagic;
    int device = 0;
    int workers = 1;
    int cost = 64;                     // K-like weight for the stream compiler
    StageDesc desc{};
    // GEMM bookkeeping (tensor maps are rebuilt when the tile width changes)
    const void *a = nullptr, *b = nullptr;
    int m = 0, n = 0, k = 0;
    int operands = GEMM_NVFP4;
    CUtensorMap* maps = nullptr;       // device: [0] = A, [1] = B
    // attention bookkeeping
    Op* merge = nullptr;               // owned merge stage (splits > 1)
    uint16_t* partial_o = nullptr;
    float* partial_ml = nullptr;
    size_t partial_bytes = 0, stat_bytes = 0;
    CUtensorMap* attn_maps = nullptr;  // device: Q, K, V maps of the tensor-core path
    int attn_path = -1;                // -1 choose by geometry, 0 mma.sync tiles, 1 tcgen05 tiles
    Op* prep = nullptr;                // owned operand-preparation stage (bias / RoPE / head sizes other than 72 and 256)
    void* prep_scratch = nullptr;      // its padded BF16 copies of Q, K and V
    Program* solo = nullptr;           // lazily built one/two-stage program for stand-alone launches
    bool solo_dirty = true;
};

struct Program {
    uint32_t magic = kProgramMagic;
    int device = 0;
    int workers = 0, length = 0;
    std::vector<StageDesc> stages;
    std::vector<unsigned int> expected;
    StageDesc* d_stages = nullptr;
    int4* d_code = nullptr;
    unsigned int* d_counters = nullptr;
    unsigned int* d_expected = nullptr;
    VmStatus* d_status = nullptr;
    long long* d_timings = nullptr;
    bool timings_on = false;
    bool lean = false;                 // every stage is one the lean kernel variant runs
    unsigned int epoch = 0;
    unsigned long long budget_ns = 2000000000ull;
    int* h_debug = nullptr;            // host-mapped progress marks (enable_native_model_debug)
    ~Program() {
        cudaFree(d_stages);
        cudaFree(d_code);
        cudaFree(d_counters);
        cudaFree(d_expected);
        cudaFree(d_status);
        cudaFree(d_timings);
        if (h_debug) cudaFreeHost(h_debug);
    }
};

int units_of(const StageDesc& d) { return d.kind == OP_GEMM ? 4 : 1; }

// Fill counter bookkeeping of a stage from its geometry.
void finish_desc(StageDesc& d) {
    d.units_per_tile = units_of(d);
    for (int i = 0; i < kMaxSources; i++) {
        d.src[i] = -1;
        d.src_mode[i] = SRC_ALL_BANDS;
    }
}

// Least-loaded contiguous tile ranges, the same policy as native_pi0.program.linear_streams.
std::vector<int> compile_streams(const std::vector<std::pair<int, int>>& work, int workers, int* length_out) {
    std::vector<std::vector<int>> rows(workers);
    std::vector<long long> load(workers, 0);
    for (size_t s = 0; s < work.size(); s++) {
        int tiles = work[s].first, k = work[s].second;
        int parts = std::min(workers, tiles), small = tiles / parts, extra = tiles % parts;
        std::vector<int> order(workers);
        for (int i = 0; i < workers; i++) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return load[x] < load[y]; });
        int start = 0;
        for (int r = 0; r < parts; r++) {
            int w = order[r], count = small + (r < extra ? 1 : 0);
            rows[w].insert(rows[w].end(), {1, static_cast<int>(s), start, count});
            load[w] += static_cast<long long>(count) * k;
            start += count;
        }
    }
    size_t length = 1;
    for (auto& r : rows) length = std::max(length, r.size() / 4);
    std::vector<int> code(static_cast<size_t>(workers) * length * 4, 0);
    for (int w = 0; w < workers; w++) std::copy(rows[w].begin(), rows[w].end(), code.begin() + static_cast<size_t>(w) * length * 4);
    *length_out = static_cast<int>(length);
    return code;
}

// Stages the lean kernel variant runs: NVFP4 projections with the model's epilogues, attention on the tcgen05 tiles, and
// every operator without variants (norm, merge, patch, embed, FP32 linear, suffix).
bool lean_stage(const StageDesc& d) {
    if (d.kind == OP_GEMM) {
        const GemmParams& g = d.p.gemm;
        const bool stats = g.row_sumsq || g.row_factor;     // (the lean residual-stream and plain BF16 drains read none)
        if (stats && (g.epilogue == EPI_BF16 || g.epilogue == EPI_STREAM)) return false;
        if (g.round_before_residual || g.gelu_cols > 0 || g.act == 3) return false;       // options the lean drains leave out
        return g.operands == GEMM_NVFP4 && (g.epilogue == EPI_BF16 || g.epilogue == EPI_STREAM || g.epilogue == EPI_GEGLU_FP4 ||
                                            g.epilogue == EPI_FP4 || g.epilogue == EPI_QKV_ROPE || g.epilogue == EPI_BF16_EXT);
    }
    if (d.kind == OP_ATTN) return d.p.attn.tc != 0 && !d.p.attn.mask;
    if (d.kind == OP_NORM) {                                 // the lean norm writes NVFP4 only: no fused residual, inverse scale, other outputs
        const NormParams& n = d.p.norm;
        return n.out && !n.residual && !n.inv_scale && !n.out_fp8 && !n.out_bf16 && !n.out_factor;
    }
    return d.kind != OP_ATTN_PREP && d.kind != OP_SUFFIX && d.kind != OP_PROBE;
}

// Build a program from stage descriptors (sources already set) and compact int4 instructions.
int build_program(Program** out, int device, const std::vector<StageDesc>& stages_in, const std::vector<int>& code4,
                  int workers, int length) {
    auto prog = std::make_unique<Program>();
    prog->device = device;
    prog->workers = workers;
    prog->length = length;
    prog->stages = stages_in;
    int counters = 0;
    for (auto& d : prog->stages) {
        d.counter_base = counters;
        counters += d.bands;
    }
    for (auto& d : prog->stages) {                     // auxiliary counters (nobody waits on them: expected stays 0)
        d.aux_base = counters;
        counters += d.aux_count;
    }
    prog->expected.assign(counters, 0);
    for (auto& d : prog->stages)
        for (int t = 0; t < d.tiles; t++) prog->expected[d.counter_base + std::min(t / d.band_div, d.bands - 1)] += d.units_per_tile;
    // static validation: stage order per worker, every tile exactly once, sources earlier than consumers
    std::vector<std::vector<int>> cover(prog->stages.size());
    for (size_t s = 0; s < prog->stages.size(); s++) {
        cover[s].assign(prog->stages[s].tiles, 0);
        for (int i = 0; i < kMaxSources; i++)
            if (prog->stages[s].src[i] >= static_cast<int>(s)) return cudaErrorInvalidValue;
    }
    for (int w = 0; w < workers; w++) {
        int last = -1;
        bool ended = false;
        for (int i = 0; i < length; i++) {
            const int* ins = &code4[(static_cast<size_t>(w) * length + i) * 4];
            if (ins[0] == 0) { ended = true; continue; }
            if (ended) return cudaErrorInvalidValue;
            int s = ins[1];
            if (s < 0 || s >= static_cast<int>(prog->stages.size()) || s < last) return cudaErrorInvalidValue;
            if (ins[3] < 1 || ins[2] < 0 || ins[2] + ins[3] > prog->stages[s].tiles) return cudaErrorInvalidValue;
            for (int t = ins[2]; t < ins[2] + ins[3]; t++) cover[s][t]++;
            // tiles of a fused split-KV attention wait for each other: each needs a worker of its own
            if (prog->stages[s].kind == OP_ATTN && prog->stages[s].p.attn.fused_merge && ins[3] != 1) return cudaErrorInvalidValue;
            last = s;
        }
    }
    for (auto& c : cover)
        for (int v : c)
            if (v != 1) return cudaErrorInvalidValue;
    // consumer-side wait lists: counter range and per-launch contribution of each producer
    for (auto& d : prog->stages) {
        int polled = 0;
        for (int i = 0; i < kMaxSources; i++) {
            d.src_counter_base[i] = 0; d.src_bands[i] = 0; d.src_expected[i] = 0; d.src_expected_last[i] = 0;
            if (d.src[i] < 0) continue;
            const StageDesc& src = prog->stages[d.src[i]];
            d.src_counter_base[i] = src.counter_base;
            d.src_bands[i] = src.bands;
            d.src_expected[i] = prog->expected[src.counter_base];
            d.src_expected_last[i] = prog->expected[src.counter_base + src.bands - 1];
            for (int b = 0; b + 1 < src.bands; b++)
                if (prog->expected[src.counter_base + b] != d.src_expected[i]) return cudaErrorInvalidValue;
            polled += d.src_mode[i] == SRC_SAME_BAND ? std::min(d.bands, src.bands) : src.bands;
        }
        if (polled > 32) return cudaErrorInvalidValue;     // one lane per polled counter
    }

    cudaError_t e = cudaMalloc(&prog->d_stages, sizeof(StageDesc) * prog->stages.size());
    if (e == cudaSuccess) e = cudaMalloc(&prog->d_code, sizeof(int4) * static_cast<size_t>(workers) * length);
    if (e == cudaSuccess) e = cudaMalloc(&prog->d_counters, sizeof(unsigned int) * std::max(counters, 1));
    if (e == cudaSuccess) e = cudaMalloc(&prog->d_expected, sizeof(unsigned int) * std::max(counters, 1));
    if (e == cudaSuccess) e = cudaMalloc(&prog->d_status, sizeof(VmStatus));
    if (e == cudaSuccess) {
        for (auto& d : prog->stages)
            if (d.kind == OP_ATTN && d.aux_count) d.p.attn.tickets = prog->d_counters + d.aux_base;
        e = cudaMemcpy(prog->d_stages, prog->stages.data(), sizeof(StageDesc) * prog->stages.size(), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) e = cudaMemcpy(prog->d_code, code4.data(), sizeof(int4) * static_cast<size_t>(workers) * length, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(prog->d_counters, 0, sizeof(unsigned int) * std::max(counters, 1));
    if (e == cudaSuccess && counters) e = cudaMemcpy(prog->d_expected, prog->expected.data(), sizeof(unsigned int) * counters, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(prog->d_status, 0, sizeof(VmStatus));
    if (e == cudaSuccess) {
        static bool configured[64] = {};
        if (device < 64 && !configured[device]) {
            e = cudaFuncSetAttribute(pi0_vm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(pi0_vm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(pi0_vm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            configured[device] = e == cudaSuccess;
        }
        prog->lean = true;
        for (const auto& d : prog->stages) prog->lean = prog->lean && lean_stage(d);
    }
    if (e != cudaSuccess) return e;
    *out = prog.release();
    return cudaSuccess;
}

int launch_program(Program* prog, cudaStream_t stream, LaunchInputs in, int begin, int end, bool new_epoch) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device != prog->device) return cudaErrorInvalidDevice;
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(stream, &capture);
    if (e != cudaSuccess) return e;
    if (capture != cudaStreamCaptureStatusNone) return cudaErrorStreamCaptureUnsupported;
    if (new_epoch) {
        if (prog->epoch >= (1u << 20)) {          // keep expected * epoch far from 2^32
            e = cudaMemsetAsync(prog->d_counters, 0, sizeof(unsigned int) * std::max<size_t>(prog->expected.size(), 1), stream);
            if (e != cudaSuccess) return e;
            prog->epoch = 0;
        }
        prog->epoch++;
    }
    VmProgram p{};
    p.stages = prog->d_stages;
    p.code = prog->d_code;
    p.counters = prog->d_counters;
    p.expected = prog->d_expected;
    p.status = prog->d_status;
    p.timings = prog->timings_on ? prog->d_timings : nullptr;
    p.num_stages = static_cast<int>(prog->stages.size());
    p.length = prog->length;
    p.epoch = prog->epoch;
    p.stage_begin = begin;
    p.stage_end = end;
    p.wait_budget_ns = prog->budget_ns;
    p.in = in;
    p.debug = prog->h_debug;
    if (prog->lean && !prog->h_debug && !p.timings) pi0_vm_kernel<true, false><<<prog->workers, kThreads, kSmemBytes, stream>>>(p);
    else if (prog->lean && !prog->h_debug) pi0_vm_kernel<true><<<prog->workers, kThreads, kSmemBytes, stream>>>(p);
    else pi0_vm_kernel<false><<<prog->workers, kThreads, kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}

Op* as_op(void* h) {
    Op* op = static_cast<Op*>(h);
    return op && op->magic == kOpMagic ? op : nullptr;
}
Program* as_program(void* h) {
    Program* p = static_cast<Program*>(h);
    return p && p->magic == kProgramMagic ? p : nullptr;
}

int new_op(Op** out, int workers) {
    int device = 0;
    int e = check_device(&device);
    if (e) return e;
    if (workers < 1 || workers > sm_count(device)) return cudaErrorInvalidConfiguration;
    Op* op = new Op();
    op->device = device;
    op->workers = workers;
    *out = op;
    return cudaSuccess;
}

void free_op(Op* op) {
    if (!op) return;
    if (op->merge) free_op(op->merge);
    if (op->prep) free_op(op->prep);
    cudaFree(op->prep_scratch);
    delete op->solo;
    cudaFree(op->maps);
    cudaFree(op->partial_o);
    cudaFree(op->partial_ml);
    cudaFree(op->attn_maps);
    op->magic = 0;
    delete op;
}

// Bytes of one operand row: K elements of 4, 16 or 8 bits.
size_t operand_row_bytes(int operands, int k) {
    return operands == GEMM_NVFP4 ? static_cast<size_t>(k) / 2 : operands == GEMM_BF16 ? static_cast<size_t>(k) * 2 : static_cast<size_t>(k);
}

int gemm_refresh(Op* op) {
    GemmParams& g = op->desc.p.gemm;
    CUtensorMap host[2];
    const size_t row_bytes = operand_row_bytes(op->operands, op->k);
    int e = encode_operand(&host[0], op->a, op->m, row_bytes, g.a_box_rows);
    if (!e) e = g.b_tiled ? encode_tiled(&host[1], op->b, op->n * (op->k / 256), kChunks * g.block_n)
                          : encode_operand(&host[1], op->b, op->n, row_bytes, g.block_n);
    if (e) return e;
    if (!op->maps) {
        cudaError_t ce = cudaMalloc(&op->maps, 2 * sizeof(CUtensorMap));
        if (ce != cudaSuccess) return ce;
    }
    cudaError_t ce = cudaMemcpy(op->maps, host, sizeof(host), cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) return ce;
    g.tmap_a = op->maps;
    g.tmap_b = op->maps + 1;
    g.m_tiles = op->m / 128;
    g.n_tiles = op->n / g.block_n;
    if (!g.sum_out || g.sumsq_ld < g.n_tiles) g.sumsq_ld = g.n_tiles;      // statistics rows: one slot per column tile
    g.operands = op->operands;
    g.k_groups = static_cast<int>(row_bytes / 32);
    // Operand ring: a slot holds kChunks chunks of the rows that are actually copied (A: a_box_rows, B: block_n) and,
    // for NVFP4, 4 KiB of scale atoms per operand. The MMA always reads 128 rows of A; with fewer copied rows the others are
    // whatever follows in the slot (B, scales) and end in accumulator rows that are never stored, so the read only
    // has to stay inside shared memory, which the slot's own B and scale regions guarantee.
    g.off_b = kChunks * 128 * g.a_box_rows;
    const int sf_bytes = op->operands == GEMM_NVFP4 ? kSfBytes : 0;
    g.off_sfa = g.off_b + kChunks * 128 * g.block_n;
    g.off_sfb = g.off_sfa + sf_bytes;
    g.slot_stride = g.off_sfb + sf_bytes;
    g.ring_stages = std::max(kStages, std::min(kMaxStages, kDataBytes / g.slot_stride));
    if (g.slot_stride % 1024 || g.ring_stages * g.slot_stride > kDataBytes ||
        (kChunks - 1) * 128 * g.a_box_rows + kTileABytes > g.slot_stride)
        return cudaErrorInvalidValue;
    // tcgen05 instruction descriptor: operand formats at bits 7 and 10 (block-scaled kind: 1 = E2M1; kind::f16: 1 = BF16;
    // kind::f8f6f4: 0 = E4M3), FP32 accumulator (bit 4) for the dense kinds, N / 8 at bit 17, M / 16 at bit 24; both
    // operands K-major.
    const uint32_t fmt = op->operands == GEMM_FP8 ? 0u : 1u;
    const uint32_t acc_f32 = op->operands == GEMM_NVFP4 ? 0u : (1u << 4);
    g.idesc = acc_f32 | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(g.block_n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
    op->desc.tiles = g.m_tiles * g.n_tiles;
    op->desc.bands = g.m_tiles;
    op->desc.band_div = g.n_tiles;
    op->cost = op->k;
    op->solo_dirty = true;
    return cudaSuccess;
}

// Stand-alone program of one operator (plus its merge stage when the attention is split).
int solo_program(Op* op) {
    if (op->solo && !op->solo_dirty) return cudaSuccess;
    delete op->solo;
    op->solo = nullptr;
    std::vector<StageDesc> stages;
    std::vector<std::pair<int, int>> work;
    StageDesc self = op->desc;
    if (op->prep) {                                    // operand preparation first; the attention stage waits for all of it
        stages.push_back(op->prep->desc);
        work.push_back({op->prep->desc.tiles, 64});
        self.src[0] = 0;
        self.src_mode[0] = SRC_ALL_BANDS;
    }
    stages.push_back(self);
    work.push_back({op->desc.tiles, op->cost});
    if (op->merge && !op->desc.p.attn.fused_merge) {
        StageDesc m = op->merge->desc;
        m.src[0] = static_cast<int>(stages.size()) - 1;
        m.src_mode[0] = SRC_ALL_BANDS;
        stages.push_back(m);
        work.push_back({m.tiles, 64});
    }
    int length = 0;
    std::vector<int> code = compile_streams(work, op->workers, &length);
    int e = build_program(&op->solo, op->device, stages, code, op->workers, length);
    if (!e) op->solo_dirty = false;
    return e;
}

int launch_solo(void* handle, void* stream) {
    Op* op = as_op(handle);
    if (!op) return cudaErrorInvalidValue;
    int device = 0;
    cudaError_t ce = cudaGetDevice(&device);
    if (ce != cudaSuccess) return ce;
    if (device != op->device) return cudaErrorInvalidDevice;
    int e = solo_program(op);
    if (e) return e;
    return launch_program(op->solo, static_cast<cudaStream_t>(stream), LaunchInputs{}, 0, static_cast<int>(op->solo->stages.size()), true);
}

int destroy_checked(void* handle) {
    if (!handle) return cudaSuccess;
    Op* op = as_op(handle);
    if (!op) return cudaErrorInvalidValue;
    int device = 0;
    cudaError_t ce = cudaGetDevice(&device);
    if (ce != cudaSuccess) return ce;
    if (device != op->device) return cudaErrorInvalidDevice;
    free_op(op);
    return cudaSuccess;
}

__global__ void quantize_rows_kernel(NormParams n) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row < n.rows) norm_row(n, row);
}

}  // namespace
}  // namespace pi0

using namespace pi0;

// =====================================================================================================
extern "C" int create_resident_fp4(void** handle, const void* a, const void* b, const void* sfa, const void* sfb, void* out,
                                   int m, int n, int k, int workers, float alpha) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!a || !b || !sfa || !sfb || !out || m < 128 || m % 128 || n < 128 || n % 128 || k < 64 || k % 64 ||
        !std::isfinite(alpha) || alpha <= 0)
        return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    op->a = a; op->b = b; op->m = m; op->n = n; op->k = k;
    StageDesc& d = op->desc;
    d.kind = OP_GEMM;
    finish_desc(d);
    GemmParams& g = d.p.gemm;
    g.sfa = static_cast<const uint8_t*>(sfa);
    g.sfb = static_cast<const uint8_t*>(sfb);
    g.block_n = 128;
    g.a_box_rows = 128;
    g.alpha = alpha;
    g.epilogue = EPI_F32;
    g.rows = m;
    g.out = out;
    g.ldo = n;
    g.out_inv_gs = 1.f;
    e = gemm_refresh(op);
    if (e) { free_op(op); return e; }
    *handle = op;
    return cudaSuccess;
}
extern "C" int launch_resident_fp4(void* handle, void* stream) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM) return cudaErrorInvalidValue;
    return launch_solo(handle, stream);
}
extern "C" int configure_resident_fp4_bf16(void* handle, const void* bias, const void* residual, void* out) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || !out) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    g.epilogue = EPI_BF16;
    g.round_before_residual = 0; g.gelu_cols = 0; g.pad_from = 0; g.pad_to = 0;
    g.bias = bias; g.residual = residual; g.ldr = op->n;
    g.out = out; g.ldo = op->n;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_resident_fp4_quantized(void* handle, const void* bias, const void* residual, void* out, void* scales,
                                                float global_scale, int activation) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || !out || !scales || !std::isfinite(global_scale) || global_scale <= 0 ||
        activation < 0 || activation > 3)
        return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if (activation == 2 && (bias || residual || op->n % 256)) return cudaErrorInvalidValue;
    const int width = activation == 2 ? op->n / 2 : op->n;
    g.epilogue = activation == 2 ? EPI_GEGLU_FP4 : EPI_FP4;
    g.act = activation == 2 ? 0 : activation;
    g.bias = bias; g.residual = residual; g.ldr = op->n;
    g.out = out; g.ldo = width / 2;
    g.out_scales = static_cast<uint8_t*>(scales);
    g.out_blocks = width / 16;
    g.out_inv_gs = 1.f / global_scale;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_resident_fp4_qkv_rope(void* handle, void* out_q, int ldq, const void* cos, const void* sin,
                                               void* cache_k, void* cache_v, int q_cols, int head_dim, int cache_base) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || !cos || !sin || !cache_k || !cache_v || head_dim < 32 || head_dim % 32 ||
        q_cols < 0 || q_cols % head_dim || q_cols + 2 * head_dim != op->n || (q_cols && !out_q) || cache_base < 0)
        return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    g.epilogue = EPI_QKV_ROPE;
    g.bias = nullptr; g.residual = nullptr;
    g.out = out_q; g.ldo = ldq;
    g.rope_cos = cos; g.rope_sin = sin;
    g.cache_k = cache_k; g.cache_v = cache_v;
    g.q_cols = q_cols; g.head_dim = head_dim; g.cache_base = cache_base;
    op->solo_dirty = true;
    return cudaSuccess;
}
// Residual-stream epilogue: BF16 rows (+bias +residual) and, from those rounded rows, an un-normalised NVFP4 copy plus the
// per-tile sums of squares [M, N / tile width] that let the next projection apply RMSNorm as a row factor.
extern "C" int configure_resident_fp4_stream(void* handle, const void* bias, const void* residual, void* out, void* copy_fp4,
                                             void* copy_scales, float copy_global_scale, float* sumsq) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || !out || !copy_fp4 || !copy_scales || !sumsq || !std::isfinite(copy_global_scale) ||
        copy_global_scale <= 0 || !aligned16(out) || !aligned16(copy_fp4) || !aligned16(bias) || !aligned16(residual) || !aligned16(sumsq))
        return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    g.epilogue = EPI_STREAM;
    g.round_before_residual = 0; g.gelu_cols = 0;
    g.bias = bias; g.residual = residual; g.ldr = op->n;
    g.out = out; g.ldo = op->n;
    g.copy_fp4 = static_cast<uint8_t*>(copy_fp4); g.ld_copy = op->n / 2;
    g.out_scales = static_cast<uint8_t*>(copy_scales);
    g.out_blocks = op->n / 16;
    g.out_inv_gs = 1.f / copy_global_scale;
    g.sumsq_out = sumsq;
    g.sum_out = nullptr;
    g.sumsq_ld = op->n / g.block_n;
    op->solo_dirty = true;
    return cudaSuccess;
}
// extension: a residual-stream projection also leaves the per-tile SUMS of its rounded rows (for a LayerNorm folded into
// the projection that follows), and the row stride of both statistics arrays becomes ld floats (>= N / tile width, a multiple
// of 4; slots beyond the tile count are never written: zero them once).  After configure_resident_fp4_stream and the tile width.
extern "C" int configure_resident_fp4_stream_sums(void* handle, float* sums, int ld) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || op->desc.p.gemm.epilogue != EPI_STREAM || !sums || !aligned16(sums)) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if (ld < op->n / g.block_n || ld % 4) return cudaErrorInvalidValue;
    g.sum_out = sums;
    g.sumsq_ld = ld;
    op->solo_dirty = true;
    return cudaSuccess;
}
// Consumer side: multiply every accumulator row by rsqrt(sum(sumsq[row, 0..parts)) / width + eps); parts a multiple of 4.
extern "C" int configure_resident_fp4_row_rms(void* handle, const float* sumsq, int parts, int width, float eps) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || !sumsq || parts < 4 || parts % 4 || width < 1 || !std::isfinite(eps) || eps <= 0 || !aligned16(sumsq))
        return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    g.row_sumsq = sumsq; g.sumsq_parts = parts; g.sumsq_inv_width = 1.f / static_cast<float>(width); g.sumsq_eps = eps;
    g.row_sum = nullptr; g.col_center = nullptr;
    op->solo_dirty = true;
    return cudaSuccess;
}
// extension: the LayerNorm form of configure_resident_fp4_row_rms.  sums / sumsq FP32 [M, parts] are the per-tile sums and sums
// of squares a residual-stream projection left (configure_resident_fp4_stream_sums); every accumulator row r becomes
// rstd_r * (alpha * acc - mean_r * center[n]) with mean and variance (E[x^2] - mean^2) of the `width` values of row r, and
// center FP32 [N] the sum over K of weight row n as the MMA reads it (dequantised).  The weight columns carry the norm's
// gamma, the bias (added afterwards, as always) its beta: bias + W beta.  Epilogues: BF16 with the extended options
// (a head-padded store or a GELU column limit selects them) and NVFP4 output.
extern "C" int configure_resident_fp4_row_layernorm(void* handle, const float* sumsq, const float* sums, int parts, int width,
                                                    float eps, const float* center) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || !sumsq || !sums || !center || parts < 4 || parts % 4 || width < 1 || !std::isfinite(eps) ||
        eps <= 0 || !aligned16(sumsq) || !aligned16(sums) || !aligned16(center))
        return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if (g.epilogue == EPI_BF16) g.epilogue = EPI_BF16_EXT;           // (the drain loop that carries the correction)
    if (g.epilogue != EPI_BF16_EXT && g.epilogue != EPI_FP4) return cudaErrorInvalidValue;
    g.row_sumsq = sumsq; g.row_sum = sums; g.col_center = center;
    g.sumsq_parts = parts; g.sumsq_inv_width = 1.f / static_cast<float>(width); g.sumsq_eps = eps;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_resident_fp4_rows(void* handle, int rows) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || rows < 1 || rows > op->m) return cudaErrorInvalidValue;
    op->desc.p.gemm.rows = rows;
    // rows of A copied per tile: the logical rows in whole 8-row swizzle groups (at least 32, so that the 128 rows the MMA
    // reads stay inside the slot for every tile width)
    if (op->m == 128 && op->operands == GEMM_NVFP4) op->desc.p.gemm.a_box_rows = std::min(128, std::max(32, (rows + 7) / 8 * 8));
    else op->desc.p.gemm.a_box_rows = (rows <= 64 && op->m == 128) ? 64 : 128;
    return gemm_refresh(op);
}
extern "C" int configure_resident_fp4_weight_layout(void* handle, int tiled) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || (tiled != 0 && tiled != 1) || (tiled && (op->k % 256 || op->operands != GEMM_NVFP4)))
        return cudaErrorInvalidValue;
    op->desc.p.gemm.b_tiled = tiled;
    return gemm_refresh(op);
}
extern "C" int configure_resident_fp4_tile(void* handle, int block_n) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || (block_n != 128 && block_n != 64 && block_n != 32) ||
        (block_n == 32 && op->operands != GEMM_NVFP4))
        return cudaErrorInvalidValue;
    op->desc.p.gemm.block_n = block_n;
    return gemm_refresh(op);
}
extern "C" int resident_fp4_resources(void* handle, int* values, int count) {
    Op* op = as_op(handle);
    if (!op || !values || count < 8) return cudaErrorInvalidValue;
    cudaFuncAttributes attr{};
    cudaError_t e = cudaFuncGetAttributes(&attr, pi0_vm_kernel<false>);
    if (e != cudaSuccess) return e;
    cudaDeviceProp prop{};
    e = cudaGetDeviceProperties(&prop, op->device);
    if (e != cudaSuccess) return e;
    values[0] = attr.numRegs;
    values[1] = static_cast<int>(attr.sharedSizeBytes);
    values[2] = kSmemBytes;
    values[3] = static_cast<int>(attr.localSizeBytes);
    values[4] = 1;
    values[5] = kThreads;
    values[6] = prop.maxThreadsPerMultiProcessor;
    values[7] = prop.multiProcessorCount;
    return cudaSuccess;
}
extern "C" int destroy_resident_fp4(void* handle) { return destroy_checked(handle); }

// =====================================================================================================
// Dense (BF16 / FP8 E4M3) projections on the same tcgen05 pipeline, with the BF16 model's epilogues.
extern "C" int create_dense(void** handle, const void* a, const void* b, void* out, const void* bias, const void* residual,
                            int m, int n, int k, int workers, int fp8, int bf16, float alpha) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!a || !b || !out || m < 128 || m % 128 || n < 128 || n % 128 || k < 64 || k % 64 || (fp8 != 0 && fp8 != 1) ||
        (bf16 != 0 && bf16 != 1) || !std::isfinite(alpha) || alpha <= 0 || (fp8 && k % 128) ||
        !aligned16(a) || !aligned16(b) || !aligned16(out) || !aligned16(bias) || !aligned16(residual))
        return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    op->a = a; op->b = b; op->m = m; op->n = n; op->k = k;
    op->operands = fp8 ? GEMM_FP8 : GEMM_BF16;
    StageDesc& d = op->desc;
    d.kind = OP_GEMM;
    finish_desc(d);
    GemmParams& g = d.p.gemm;
    g.block_n = 128;
    g.a_box_rows = 128;
    g.alpha = alpha;
    g.epilogue = bf16 ? EPI_BF16 : EPI_F32;
    g.rows = m;
    g.out = out;
    g.ldo = n;
    g.bias = bias;
    g.residual = residual;
    g.ldr = n;
    g.out_inv_gs = 1.f;
    e = gemm_refresh(op);
    if (e) { free_op(op); return e; }
    *handle = op;
    return cudaSuccess;
}
namespace {
// A GEMM handle whose output is BF16: what every configure_dense_* call requires. (The reference also demands BF16
// operands; here the epilogues are independent of the operand format, so an NVFP4 or FP8 projection may use them.)
Op* dense_bf16(void* handle) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM) return nullptr;
    const int epilogue = op->desc.p.gemm.epilogue;
    return epilogue == EPI_BF16 || epilogue == EPI_BF16_EXT || epilogue == EPI_GEGLU_BF16 || epilogue == EPI_QKV_ROPE ? op : nullptr;
}
}  // namespace
extern "C" int launch_dense(void* handle, void* stream) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || op->operands == GEMM_NVFP4) return cudaErrorInvalidValue;
    return launch_solo(handle, stream);
}
extern "C" int destroy_dense(void* handle) { return destroy_checked(handle); }
extern "C" int configure_dense_round_before_residual(void* handle) {
    Op* op = dense_bf16(handle);
    const bool plain = op && (op->desc.p.gemm.epilogue == EPI_BF16 || op->desc.p.gemm.epilogue == EPI_BF16_EXT);
    if (!plain || !op->desc.p.gemm.residual) return cudaErrorInvalidValue;
    op->desc.p.gemm.epilogue = EPI_BF16_EXT;
    op->desc.p.gemm.round_before_residual = 1;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_dense_geglu(void* handle, void* compact_output) {
    Op* op = dense_bf16(handle);
    if (!op || !compact_output || !aligned16(compact_output)) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if (g.epilogue != EPI_BF16 || g.bias || g.residual || op->n % 256) return cudaErrorInvalidValue;
    g.epilogue = EPI_GEGLU_BF16;
    g.out = compact_output;
    g.ldo = op->n / 2;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_dense_gelu(void* handle, int logical_columns) {
    Op* op = dense_bf16(handle);
    if (!op) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if ((g.epilogue != EPI_BF16 && g.epilogue != EPI_BF16_EXT) || g.residual || logical_columns < 1 || logical_columns > op->n)
        return cudaErrorInvalidValue;
    g.epilogue = EPI_BF16_EXT;
    g.gelu_cols = logical_columns;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_dense_rms_factor(void* handle, const float* factors) {
    Op* op = dense_bf16(handle);
    if (!op || !factors) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if (g.bias || g.residual) return cudaErrorInvalidValue;
    g.row_factor = factors;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_dense_skinny(void* handle) {
    Op* op = dense_bf16(handle);
    if (!op || op->m != 128) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    g.a_box_rows = 64;                      // only 64 rows of A are copied per tile ...
    g.rows = std::min(g.rows, 64);          // ... and only those rows are ever stored
    return gemm_refresh(op);
}
extern "C" int configure_dense_qkv_rope(void* handle, const void* cos, const void* sin, void* cache_k, void* cache_v,
                                        int logical_rows, int key_offset, int cache_base) {
    Op* op = dense_bf16(handle);
    if (!op || !cos || !sin || !cache_k || !cache_v || logical_rows < 1 || key_offset < 0 || key_offset % 256 || cache_base < 0 ||
        !aligned16(cos) || !aligned16(sin) || !aligned16(cache_k) || !aligned16(cache_v))
        return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if (g.epilogue != EPI_BF16 || g.bias || g.residual || logical_rows > op->m || key_offset + 512 != op->n)
        return cudaErrorInvalidValue;
    g.epilogue = EPI_QKV_ROPE;
    g.rope_cos = cos; g.rope_sin = sin;
    g.cache_k = cache_k; g.cache_v = cache_v;
    g.q_cols = key_offset; g.head_dim = 256; g.cache_base = cache_base;
    g.rows = std::min(g.rows, logical_rows);
    op->solo_dirty = true;
    return cudaSuccess;
}
// extension: store the BF16 output with every group of `from` columns (a head) starting `to` columns after the previous
// one, in rows of `ld` elements; the columns between the heads are not written (keep them zero).  No residual.
extern "C" int configure_dense_head_pad(void* handle, int from, int to, int ld) {
    Op* op = dense_bf16(handle);
    if (!op) return cudaErrorInvalidValue;
    GemmParams& g = op->desc.p.gemm;
    if ((g.epilogue != EPI_BF16 && g.epilogue != EPI_BF16_EXT) || g.residual || from < 8 || from % 8 || to < from || to % 8 ||
        ld < (op->n + from - 1) / from * to || ld % 8)
        return cudaErrorInvalidValue;
    g.epilogue = EPI_BF16_EXT;
    g.pad_from = from; g.pad_to = to; g.ldo = ld;
    op->solo_dirty = true;
    return cudaSuccess;
}
// extension: logical rows (as configure_resident_fp4_rows) and output tile width of a dense projection.
extern "C" int configure_dense_rows(void* handle, int rows) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || op->operands == GEMM_NVFP4 || rows < 1 || rows > op->m) return cudaErrorInvalidValue;
    op->desc.p.gemm.rows = rows;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_dense_tile(void* handle, int block_n) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_GEMM || op->operands == GEMM_NVFP4 || (block_n != 128 && block_n != 64)) return cudaErrorInvalidValue;
    op->desc.p.gemm.block_n = block_n;
    return gemm_refresh(op);
}

// =====================================================================================================
extern "C" int create_norm(void** handle, const void* input, const void* residual, const float* gamma, const float* beta,
                           const float* inverse_scale, void* residual_output, void* output, void* scales, int rows, int width,
                           int workers, int fp16, int format, int layer, int round_norm, int round_residual, int legacy_ties,
                           float epsilon, float global_scale) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    const bool known_format = format == 4 || format == 8 || format == 16 || format == 17;
    if (!input || !output || rows < 1 || width < 16 || width % 16 || !known_format || (format == 4 && !scales) || fp16 ||
        (residual_output && !residual) || legacy_ties || !std::isfinite(epsilon) || epsilon <= 0 ||
        !std::isfinite(global_scale) || global_scale <= 0 || width > 2048 || !aligned16(input) || !aligned16(residual) ||
        !aligned16(residual_output) || !aligned16(output) || !aligned16(gamma) || !aligned16(beta) || !aligned16(inverse_scale))
        return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    StageDesc& d = op->desc;
    d.kind = OP_NORM;
    finish_desc(d);
    const int rows_per_tile = layer ? 2 * kNormPairRows : kNormPairRows;
    d.tiles = (rows + rows_per_tile - 1) / rows_per_tile;
    d.bands = (rows + kBandRows - 1) / kBandRows;
    d.band_div = kBandRows / rows_per_tile;
    NormParams& n = d.p.norm;
    n.rows_per_tile = rows_per_tile;
    n.in = input; n.gamma = gamma; n.beta = beta;
    n.residual = residual; n.residual_out = residual_output; n.round_residual = round_residual;
    n.inv_scale = inverse_scale;
    n.rows = rows; n.width = width;
    n.mode = layer ? 1 : 0;
    n.round_norm = round_norm;
    n.eps = epsilon;
    n.inv_gs = 1.f / global_scale;
    n.policy = 0;
    if (format == 4) { n.out = static_cast<uint8_t*>(output); n.out_scales = static_cast<uint8_t*>(scales); }
    else if (format == 8) n.out_fp8 = static_cast<uint8_t*>(output);
    else if (format == 16) n.out_bf16 = output;
    else n.out_factor = static_cast<float*>(output);
    n.out_blocks = width / 16;
    n.ld_in = width;
    n.ld_out = width / 2;
    *handle = op;
    return cudaSuccess;
}
extern "C" int launch_norm(void* handle, void* stream) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_NORM) return cudaErrorInvalidValue;
    return launch_solo(handle, stream);
}
extern "C" int destroy_norm(void* handle) { return destroy_checked(handle); }
extern "C" int configure_norm_quantize_only(void* handle, int policy) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_NORM || (policy != 0 && policy != 1)) return cudaErrorInvalidValue;
    NormParams& n = op->desc.p.norm;
    n.mode = 2;
    n.policy = policy;
    n.rows_per_tile = 2 * kNormPairRows;
    op->desc.tiles = (n.rows + n.rows_per_tile - 1) / n.rows_per_tile;
    op->desc.band_div = kBandRows / n.rows_per_tile;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_norm_bf16_copy(void* handle, void* out_bf16) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_NORM) return cudaErrorInvalidValue;
    op->desc.p.norm.out_bf16 = out_bf16;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_norm_layout(void* handle, int ld_in, int ld_out, int out_blocks) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_NORM) return cudaErrorInvalidValue;
    NormParams& n = op->desc.p.norm;
    if (ld_in < n.width || ld_in % 8 || ld_out < n.width / 2 || ld_out % 8 || out_blocks < n.width / 16) return cudaErrorInvalidValue;
    n.ld_in = ld_in; n.ld_out = ld_out; n.out_blocks = out_blocks;
    op->solo_dirty = true;
    return cudaSuccess;
}

// =====================================================================================================
// Tile geometry of an attention operator and the choice between the two tile implementations.  The tcgen05 tiles need
// heads that occupy 128 or 256 elements in memory (hd_pad), at most 256 keys per tile (more keys: more KV splits) and,
// without splits, no fused NVFP4 output; everything else runs on the mma.sync tiles.
static int attention_geometry(Op* op) {
    AttnParams& a = op->desc.p.attn;
    const int qtiles = (a.nq + kAttnQRows - 1) / kAttnQRows;
    op->desc.tiles = a.batches * qtiles * a.heads * a.splits;
    op->desc.bands = a.batches * qtiles;
    op->desc.band_div = a.heads * a.splits;
    op->cost = std::max(64, ((a.nk / a.splits) * a.head_dim / 64 + 63) / 64 * 64);
    op->solo_dirty = true;
    const int per = (a.nk + a.splits - 1) / a.splits;
    const bool layout_ok = (a.hd_pad == 128 || a.hd_pad == 256) && a.hd_pad >= a.head_dim && a.head_dim % 8 == 0 &&
                           a.ldq >= a.heads * a.hd_pad && a.ldkv >= a.kv_heads * a.hd_pad;
    const bool eligible = layout_ok && per <= 256 && (a.splits == 1 || a.head_dim % 16 == 0);    // (the merge works on 16-column blocks)
    a.tc = op->attn_path == 0 ? 0 : eligible ? 1 : 0;
    if (op->attn_path == 1 && !eligible) return cudaErrorInvalidValue;
    // an FP4 output on a head pitch other than head_dim exists only in the unsplit tcgen05 tile
    if (a.out_fp4 && a.fp4_pitch != a.head_dim && !(a.tc && a.splits == 1)) return cudaErrorInvalidValue;
    if (!a.tc) return cudaSuccess;
    a.q_box = std::min(128, (std::min(a.nq, 128) + 7) / 8 * 8);
    a.k_box = std::min(256, (per + 15) / 16 * 16);
    CUtensorMap host[3];
    int e = encode_bf16_rows(&host[0], a.q, static_cast<size_t>(a.batches) * a.q_batch_rows, a.ldq, a.q_box);
    if (!e) e = encode_bf16_rows(&host[1], a.k, static_cast<size_t>(a.batches) * a.kv_batch_rows, a.ldkv, a.k_box);
    if (!e) e = encode_bf16_rows(&host[2], a.v, static_cast<size_t>(a.batches) * a.kv_batch_rows, a.ldkv, a.k_box);
    if (e) return e;
    if (!op->attn_maps) {
        cudaError_t ce = cudaMalloc(&op->attn_maps, sizeof(host));
        if (ce != cudaSuccess) return ce;
    }
    cudaError_t ce = cudaMemcpy(op->attn_maps, host, sizeof(host), cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) return ce;
    a.tmap_q = op->attn_maps; a.tmap_k = op->attn_maps + 1; a.tmap_v = op->attn_maps + 2;
    return cudaSuccess;
}
extern "C" int create_attention(void** handle, const void* q, const void* k, const void* v, const void* q_bias, const void* k_bias,
                                const void* v_bias, const void* q_cos, const void* q_sin, const void* k_cos, const void* k_sin,
                                void* out, const void* mask, int batches, int nq, int nk, int heads, int kv_heads, int head_dim,
                                int ldq, int ldkv, int out_ld, int fp16, int workers, int prefix, float scale) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!q || !k || !v || !out || fp16 || batches < 1 || nq < 1 || nk < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads ||
        head_dim < 8 || head_dim > 256 || head_dim % 8 || (q_cos == nullptr) != (q_sin == nullptr) || (k_cos == nullptr) != (k_sin == nullptr) ||
        ldq < heads * head_dim || ldq % 8 || ldkv < kv_heads * head_dim || ldkv % 8 || out_ld < heads * head_dim || out_ld % 8 ||
        !std::isfinite(scale) || scale <= 0 || (prefix >= 0 && batches != 1) ||
        !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))     // rows move in 16-byte pieces
        return cudaErrorInvalidValue;
    // Biases, rotary tables and head sizes other than 72 / 256 go through an operand-preparation stage that writes Q, K and V
    // (bias added, rotated) into library-owned buffers with every head on a 128- or 256-element pitch, which the tcgen05
    // tiles read; the boolean mask is applied inside those tiles.
    const bool prepared = q_bias || k_bias || v_bias || q_cos || k_cos || (head_dim != 72 && head_dim != 256);
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    StageDesc& d = op->desc;
    d.kind = OP_ATTN;
    finish_desc(d);
    AttnParams& a = d.p.attn;
    a.mask = static_cast<const uint8_t*>(mask);
    if (prepared) {
        const int pitch = head_dim <= 128 ? 128 : 256;
        const size_t q_elems = static_cast<size_t>(batches) * nq * heads * pitch, kv_elems = static_cast<size_t>(batches) * nk * kv_heads * pitch;
        cudaError_t ce = cudaMalloc(&op->prep_scratch, (q_elems + 2 * kv_elems) * sizeof(uint16_t));
        if (ce == cudaSuccess) ce = cudaMemset(op->prep_scratch, 0, (q_elems + 2 * kv_elems) * sizeof(uint16_t));
        if (ce != cudaSuccess) { free_op(op); return ce; }
        uint16_t* base = static_cast<uint16_t*>(op->prep_scratch);
        e = new_op(&op->prep, workers);
        if (e) { free_op(op); return e; }
        StageDesc& pd = op->prep->desc;
        pd.kind = OP_ATTN_PREP;
        finish_desc(pd);
        PrepParams& pp = pd.p.prep;
        pp.src[0] = q; pp.src[1] = k; pp.src[2] = v;
        pp.dst[0] = base; pp.dst[1] = base + q_elems; pp.dst[2] = base + q_elems + kv_elems;
        pp.bias[0] = q_bias; pp.bias[1] = k_bias; pp.bias[2] = v_bias;
        pp.cos[0] = q_cos; pp.sin[0] = q_sin; pp.cos[1] = k_cos; pp.sin[1] = k_sin;
        pp.rows[0] = batches * nq; pp.rows[1] = pp.rows[2] = batches * nk;
        pp.heads[0] = heads; pp.heads[1] = pp.heads[2] = kv_heads;
        pp.ld_src[0] = ldq; pp.ld_src[1] = pp.ld_src[2] = ldkv;
        pp.ld_dst[0] = heads * pitch; pp.ld_dst[1] = pp.ld_dst[2] = kv_heads * pitch;
        pp.head_dim = head_dim; pp.src_pitch = head_dim; pp.pitch = pitch;
        pd.tiles = (pp.rows[0] + 7) / 8 + 2 * ((pp.rows[1] + 7) / 8);
        pd.bands = 1;
        pd.band_div = pd.tiles;
        q = pp.dst[0]; k = pp.dst[1]; v = pp.dst[2];
        ldq = pp.ld_dst[0]; ldkv = pp.ld_dst[1];
    }
    a.q = q; a.k = k; a.v = v; a.out = out;
    a.ldq = ldq; a.ldkv = ldkv; a.ldo = out_ld;
    a.batches = batches; a.nq = nq; a.nk = nk;
    a.q_batch_rows = nq; a.kv_batch_rows = nk;
    a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
    a.scale = scale;
    a.prefix = prefix >= 0 ? prefix : -1;
    a.splits = 1;
    a.out_inv_gs = 1.f;
    a.fp4_pitch = head_dim;
    a.hd_pad = prepared ? (head_dim <= 128 ? 128 : 256) : head_dim == 256 ? 256 : 0;   // 72-wide heads as given: the tensor-core tiles only after configure_attention_head_pad
    e = attention_geometry(op);
    if (e) { free_op(op); return e; }
    *handle = op;
    return cudaSuccess;
}
// Prepared operands and the boolean mask exist for the tcgen05 tiles only (at most 256 keys per tile: use KV splits).  Checked when
// the operator is launched or placed in a program, so that splits can still be configured after creation.
static bool attention_runnable(const Op* op) {
    const AttnParams& a = op->desc.p.attn;
    return a.tc || !(a.mask || op->prep);
}
extern "C" int attention_validate(void* handle) {
    Op* op = as_op(handle);
    return op && op->desc.kind == OP_ATTN && attention_runnable(op) ? cudaSuccess : cudaErrorInvalidValue;
}
extern "C" int launch_attention(void* handle, void* stream) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || !attention_runnable(op)) return cudaErrorInvalidValue;
    return launch_solo(handle, stream);
}
extern "C" int destroy_attention(void* handle) { return destroy_checked(handle); }
extern "C" int attention_resources(int* values, int count) {
    if (!values || count < 4) return cudaErrorInvalidValue;
    cudaFuncAttributes attr{};
    cudaError_t e = cudaFuncGetAttributes(&attr, pi0_vm_kernel<false>);
    if (e != cudaSuccess) return e;
    values[0] = attr.numRegs;
    values[1] = static_cast<int>(attr.localSizeBytes);
    values[2] = kSmemBytes;
    values[3] = kThreads;
    return cudaSuccess;
}
extern "C" int configure_attention_splits(void* handle, int splits) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || splits < 1 || splits > 64) return cudaErrorInvalidValue;
    AttnParams& a = op->desc.p.attn;
    if (splits > 1 && (a.batches != 1 || a.head_dim % 16)) return cudaErrorInvalidValue;
    // Allocate first; the handle changes only when everything it needs exists (a failed call leaves it as it was).
    uint16_t* partial_o = nullptr;
    float* partial_ml = nullptr;
    const int groups = a.heads * ((a.nq + kAttnQRows - 1) / kAttnQRows);          // heads x 128-query tiles
    const size_t tasks = static_cast<size_t>(groups) * splits;
    if (splits > 1) {
        cudaError_t e = cudaMalloc(&partial_o, tasks * kAttnQRows * a.head_dim * sizeof(uint16_t));
        if (e == cudaSuccess) e = cudaMalloc(&partial_ml, tasks * kAttnQRows * 2 * sizeof(float));
        if (e != cudaSuccess) {
            cudaFree(partial_o);
            cudaFree(partial_ml);
            return e;
        }
    }
    if (op->merge) { free_op(op->merge); op->merge = nullptr; }
    cudaFree(op->partial_o);
    cudaFree(op->partial_ml);
    op->partial_o = partial_o;
    op->partial_ml = partial_ml;
    op->partial_bytes = splits > 1 ? tasks * kAttnQRows * a.head_dim * sizeof(uint16_t) : 0;
    op->stat_bytes = splits > 1 ? tasks * kAttnQRows * 2 * sizeof(float) : 0;
    a.splits = splits;
    a.fused_merge = 0;
    a.partial_o = partial_o;
    a.partial_ml = partial_ml;
    op->desc.aux_count = 0;
    if (splits > 1) {
        Op* mg = new Op();
        mg->device = op->device;
        mg->workers = op->workers;
        mg->desc.kind = OP_MERGE;
        finish_desc(mg->desc);
        mg->desc.tiles = groups * ((std::min(a.nq, kAttnQRows) + kMergeRows - 1) / kMergeRows);
        mg->desc.bands = 1;
        mg->desc.band_div = mg->desc.tiles;
        MergeParams& g = mg->desc.p.merge;
        g.partial_o = partial_o; g.partial_ml = partial_ml;
        g.heads = a.heads; g.nq = a.nq; g.head_dim = a.head_dim; g.splits = splits;
        g.out = a.out; g.ldo = a.ldo;
        g.out_fp4 = a.out_fp4; g.out_scales = a.out_scales; g.out_blocks = a.out_blocks; g.out_inv_gs = a.out_inv_gs; g.ld_fp4 = a.ld_fp4;
        op->merge = mg;
    }
    return attention_geometry(op);
}
// Fill the split-KV scratch (partial rows and their softmax statistics) with 0xFF bytes - NaN patterns in both
// formats - so a run that read a partial it had not written in the same launch would show it in its output.
extern "C" int attention_poison_partials(void* handle, void* stream) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || op->desc.p.attn.splits < 2) return cudaErrorInvalidValue;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device != op->device) return cudaErrorInvalidDevice;
    e = cudaMemsetAsync(op->partial_o, 255, op->partial_bytes, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(op->partial_ml, 255, op->stat_bytes, static_cast<cudaStream_t>(stream));
    return e;
}
// Arrival counts of the split-KV groups (one per head of each 128-query tile) after the launches so far, and the launch
// count they are measured against: a group is complete when its count equals splits * epoch. With the merge as a stage
// of its own the counts are those of the attention stage's row bands scaled to tiles per group.
extern "C" int attention_split_diagnostics(void* handle, unsigned long long* counts, int capacity, unsigned int* epoch) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || !counts || !epoch) return cudaErrorInvalidValue;
    const AttnParams& a = op->desc.p.attn;
    const int groups = a.heads * ((a.nq + kAttnQRows - 1) / kAttnQRows);
    if (a.splits < 2 || capacity < groups) return cudaErrorInvalidValue;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device != op->device) return cudaErrorInvalidDevice;
    *epoch = op->solo ? op->solo->epoch : 0u;
    for (int g = 0; g < groups; g++) counts[g] = 0;
    if (!op->solo) return cudaSuccess;
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    const StageDesc& d = op->solo->stages[0];
    std::vector<unsigned int> raw(op->solo->expected.size());
    e = cudaMemcpy(raw.data(), op->solo->d_counters, raw.size() * sizeof(unsigned int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (a.fused_merge && d.aux_count == groups) {
        for (int g = 0; g < groups; g++) counts[g] = raw[d.aux_base + g];
    } else {
        // one counter per 128-query tile: heads * splits tiles each, every head of the tile has the same share
        for (int g = 0; g < groups; g++) counts[g] = raw[d.counter_base + g / a.heads] / static_cast<unsigned int>(a.heads);
    }
    return cudaSuccess;
}
extern "C" int configure_attention_fused_merge(void* handle, int enable) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || (enable != 0 && enable != 1)) return cudaErrorInvalidValue;
    AttnParams& a = op->desc.p.attn;
    if (enable && a.splits < 2) return cudaErrorInvalidValue;
    a.fused_merge = enable;
    op->desc.aux_count = enable ? a.heads * ((a.nq + kAttnQRows - 1) / kAttnQRows) : 0;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int configure_attention_cache(void* handle, const void* cache_k, const void* cache_v, int rows, int prefix_rows) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || !cache_k || !cache_v || rows < 1 || prefix_rows < 0 || prefix_rows > rows ||
        !aligned16(cache_k) || !aligned16(cache_v))
        return cudaErrorInvalidValue;
    AttnParams& a = op->desc.p.attn;
    if (a.batches != 1 || a.kv_heads != 1 || op->prep) return cudaErrorInvalidValue;    // (prepared operands are copies: no cache)
    a.k = cache_k; a.v = cache_v; a.ldkv = a.head_dim; a.nk = rows; a.kv_batch_rows = rows;
    return attention_geometry(op);
}
extern "C" int configure_attention_fp4_output(void* handle, void* out_fp4, void* scales, int ld_bytes, int out_blocks, float global_scale) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || !out_fp4 || !scales || !std::isfinite(global_scale) || global_scale <= 0) return cudaErrorInvalidValue;
    AttnParams& a = op->desc.p.attn;
    if (a.fp4_pitch % 16 || ld_bytes < a.heads * a.fp4_pitch / 2 || out_blocks < a.heads * a.fp4_pitch / 16) return cudaErrorInvalidValue;
    a.out_fp4 = static_cast<uint8_t*>(out_fp4); a.out_scales = static_cast<uint8_t*>(scales);
    a.ld_fp4 = ld_bytes; a.out_blocks = out_blocks; a.out_inv_gs = 1.f / global_scale;
    if (op->merge) {
        MergeParams& g = op->merge->desc.p.merge;
        g.out_fp4 = a.out_fp4; g.out_scales = a.out_scales; g.ld_fp4 = ld_bytes; g.out_blocks = out_blocks; g.out_inv_gs = a.out_inv_gs;
    }
    return attention_geometry(op);
}
// extension: columns one head occupies in the FP4 output (a multiple of 16, head_dim <= pitch <= the padded head size).  The
// columns from head_dim up to the pitch are written as zeros, so a following projection whose K is heads * pitch (zero weight
// columns at the same places) reads the output directly.  Set it before configure_attention_fp4_output; only the unsplit
// tcgen05 tiles offer a pitch other than head_dim.
extern "C" int configure_attention_fp4_pitch(void* handle, int pitch) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN) return cudaErrorInvalidValue;
    AttnParams& a = op->desc.p.attn;
    if (pitch % 16 || pitch < a.head_dim || (pitch != a.head_dim && pitch > a.hd_pad) || a.out_fp4) return cudaErrorInvalidValue;
    a.fp4_pitch = pitch;
    return attention_geometry(op);
}
// extension: choose the tile implementation: -1 by geometry (default), 0 mma.sync tiles, 1 tcgen05 tiles (an error when the
// geometry does not allow them).
extern "C" int configure_attention_path(void* handle, int path) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || path < -1 || path > 1) return cudaErrorInvalidValue;
    const int before = op->attn_path;
    op->attn_path = path;
    const int e = attention_geometry(op);
    if (e) { op->attn_path = before; attention_geometry(op); }
    return e;
}
// extension: declare that every head occupies `elements` (128 or 256) elements in q, k and v, the columns beyond
// head_dim being zeros (as a projection with the head-padded epilogue writes them).  The row strides given at creation
// must cover heads * elements.  Output rows stay head_dim wide.
extern "C" int configure_attention_head_pad(void* handle, int elements) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || (elements != 128 && elements != 256) || elements < op->desc.p.attn.head_dim || op->prep)
        return cudaErrorInvalidValue;
    AttnParams& a = op->desc.p.attn;
    if (a.ldq < a.heads * elements || a.ldkv < a.kv_heads * elements) return cudaErrorInvalidValue;
    a.hd_pad = elements;
    return attention_geometry(op);
}
// extension: handle of the operand-preparation stage an attention handle owns when it was created with biases, rotary
// tables or a head size other than 72 / 256 (NULL otherwise); a program lists it in front of the attention stage.
extern "C" int attention_prepare_handle(void* handle, void** prepare) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || !prepare) return cudaErrorInvalidValue;
    *prepare = op->prep;
    return cudaSuccess;
}
extern "C" int attention_merge_handle(void* handle, void** merge) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_ATTN || !merge) return cudaErrorInvalidValue;
    *merge = op->merge;
    return cudaSuccess;
}

// =====================================================================================================
extern "C" int create_patch_embed(void** handle, const float* images, const float* weight, const float* bias, const float* pos,
                                  void* out, int views, int width, int workers) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!weight || !bias || !pos || !out || views < 1 || width < 1) return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    StageDesc& d = op->desc;
    d.kind = OP_PATCH;
    finish_desc(d);
    const int ntiles = (width + kPatchCols - 1) / kPatchCols;
    d.tiles = views * 256 / kPatchTokens * ntiles;
    d.bands = views * 256 / kBandRows;
    d.band_div = kBandRows / kPatchTokens * ntiles;
    op->cost = 576;
    d.p.patch = PatchParams{images, weight, bias, pos, out, views, width};
    *handle = op;
    return cudaSuccess;
}
extern "C" int create_token_embed(void** handle, const long long* tokens, const void* table, void* out, int count, int width,
                                  int row_base, int vocab, float scale, int workers) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!table || !out || count < 1 || width < 1 || row_base < 0 || vocab < 1) return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    StageDesc& d = op->desc;
    d.kind = OP_EMBED;
    finish_desc(d);
    d.tiles = (count + 7) / 8;
    d.bands = 1;
    d.band_div = d.tiles;
    d.p.embed = EmbedParams{tokens, table, out, count, width, row_base, vocab, scale};
    *handle = op;
    return cudaSuccess;
}
extern "C" int create_linear32(void** handle, const void* x, const float* w, const float* bias, const float* prev, void* out,
                               int rows, int n, int k, int ldx, int ldo, int flags, int slot, int prev_slot, int x_row_offset,
                               float dt, float eps, int workers) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!w || !out || rows < 1 || n < 1 || k < 4 || k % 4 || ldx < k || ldo < n || (slot != 0 && slot != 2 && slot != 3) ||
        (slot == 0 && !x) || (prev_slot != 0 && prev_slot != 3) || ((flags & 16) && prev_slot == 0 && !prev) || x_row_offset < 0 ||
        ldx % 4 || ((flags & 1) && (k % 8 || ldx % 8)))            // rows are staged with 16-byte asynchronous copies
        return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    StageDesc& d = op->desc;
    d.kind = OP_LINEAR32;
    finish_desc(d);
    // few columns (the action head): blocks of 16 rows, so that more than one or two CTAs share the operator
    const int row_block = (rows <= 16 || n <= 64) ? 16 : kLinRows;
    d.tiles = ((n + kLinCols - 1) / kLinCols) * ((rows + row_block - 1) / row_block);
    d.bands = 1;
    d.band_div = d.tiles;
    op->cost = std::max(64, (k * std::min(rows, row_block) / 16 + 63) / 64 * 64);
    Linear32Params& p = d.p.lin;
    p.row_block = row_block;
    p.x = x; p.w = w; p.bias = bias; p.prev = prev; p.out = out;
    p.rows = rows; p.n = n; p.k = k; p.ldx = ldx; p.ldo = ldo;
    p.x_bf16 = flags & 1; p.out_bf16 = (flags >> 1) & 1; p.silu = (flags >> 2) & 1; p.rms = (flags >> 3) & 1; p.euler = (flags >> 4) & 1;
    p.slot = slot; p.prev_slot = prev_slot; p.x_row_offset = x_row_offset; p.dt = dt; p.eps = eps;
    *handle = op;
    return cudaSuccess;
}
// Extension: the tiles of the first row block also store `src` (FP32 [n]) as BF16 at `dst`.
extern "C" int configure_linear32_extra_row(void* handle, const float* src, void* dst) {
    Op* op = as_op(handle);
    if (!op || op->desc.kind != OP_LINEAR32 || !src || !dst) return cudaErrorInvalidValue;
    op->desc.p.lin.row0_src = src;
    op->desc.p.lin.row0_dst = dst;
    op->solo_dirty = true;
    return cudaSuccess;
}
extern "C" int create_suffix_assemble(void** handle, const float* state_emb, const float* action_emb, void* out, int chunk,
                                      int width, int workers) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (!state_emb || !action_emb || !out || chunk < 1 || width < 1) return cudaErrorInvalidValue;
    Op* op = nullptr;
    int e = new_op(&op, workers);
    if (e) return e;
    StageDesc& d = op->desc;
    d.kind = OP_SUFFIX;
    finish_desc(d);
    d.tiles = (chunk + 1 + 7) / 8;
    d.bands = 1;
    d.band_div = d.tiles;
    d.p.suffix = SuffixParams{state_emb, action_emb, out, chunk, width};
    *handle = op;
    return cudaSuccess;
}
extern "C" int launch_op(void* handle, void* stream) { return launch_solo(handle, stream); }
extern "C" int destroy_op(void* handle) { return destroy_checked(handle); }
extern "C" int op_geometry(void* handle, int* tiles, int* bands, int* cost) {
    Op* op = as_op(handle);
    if (!op) return cudaErrorInvalidValue;
    if (tiles) *tiles = op->desc.tiles;
    if (bands) *bands = op->desc.bands;
    if (cost) *cost = op->cost;
    return cudaSuccess;
}

// =====================================================================================================
extern "C" int create_native_model(void** handle, int count, const NativeSpec* specs, const int* code, int workers, int length) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (count < 1 || !specs || !code || workers < 1 || length < 1) return cudaErrorInvalidValue;
    int device = 0;
    int e = check_device(&device);
    if (e) return e;
    if (workers > sm_count(device)) return cudaErrorInvalidConfiguration;
    std::vector<StageDesc> stages;
    stages.reserve(count);
    for (int i = 0; i < count; i++) {
        Op* op = as_op(specs[i].handle);
        if (!op || op->device != device) return cudaErrorInvalidValue;
        const int want = op->desc.kind == OP_GEMM ? 0 : op->desc.kind == OP_ATTN ? 1 : op->desc.kind == OP_NORM ? 2 : op->desc.kind == OP_MERGE ? 4 : 3;
        if (specs[i].kind != want) return cudaErrorInvalidValue;
        if (op->desc.kind == OP_ATTN && !attention_runnable(op)) return cudaErrorInvalidValue;
        StageDesc d = op->desc;
        for (int s = 0; s < kMaxSources; s++) {
            d.src[s] = specs[i].sources[s];
            d.src_mode[s] = specs[i].modes[s] ? SRC_ALL_BANDS : SRC_SAME_BAND;
            if (d.src[s] >= i || d.src[s] < -1) return cudaErrorInvalidValue;
        }
        stages.push_back(d);
    }
    std::vector<int> code4(static_cast<size_t>(workers) * length * 4);
    for (size_t i = 0; i < static_cast<size_t>(workers) * length; i++) {
        const int* ins = code + i * 32;
        code4[i * 4 + 0] = ins[0] ? stages[std::min(std::max(ins[1], 0), count - 1)].kind : 0;
        code4[i * 4 + 1] = ins[1];
        code4[i * 4 + 2] = ins[2];
        code4[i * 4 + 3] = ins[3];
    }
    Program* prog = nullptr;
    e = build_program(&prog, device, stages, code4, workers, length);
    if (e) return e;
    *handle = prog;
    return cudaSuccess;
}
extern "C" int launch_native_model_range(void* handle, void* stream, const float* images, const float* state, const float* noise,
                                         const long long* tokens, int begin, int end, int new_epoch) {
    Program* prog = as_program(handle);
    if (!prog || begin < 0 || end > static_cast<int>(prog->stages.size()) || begin >= end) return cudaErrorInvalidValue;
    return launch_program(prog, static_cast<cudaStream_t>(stream), LaunchInputs{images, state, noise, tokens}, begin, end, new_epoch != 0);
}
extern "C" int launch_native_model(void* handle, void* stream, const float* images, const float* state, const float* noise,
                                   const long long* tokens) {
    Program* prog = as_program(handle);
    if (!prog) return cudaErrorInvalidValue;
    return launch_program(prog, static_cast<cudaStream_t>(stream), LaunchInputs{images, state, noise, tokens}, 0,
                          static_cast<int>(prog->stages.size()), true);
}
extern "C" int enable_native_model_timings(void* handle, int enable) {
    Program* prog = as_program(handle);
    if (!prog) return cudaErrorInvalidValue;
    if (enable && !prog->d_timings) {
        const size_t bytes = sizeof(long long) * 8 * prog->workers * prog->length;
        cudaError_t e = cudaMalloc(&prog->d_timings, bytes);
        if (e == cudaSuccess) e = cudaMemset(prog->d_timings, 0, bytes);
        if (e != cudaSuccess) return e;
    }
    prog->timings_on = enable != 0;
    return cudaSuccess;
}
extern "C" int read_native_model_timings(void* handle, long long* out, size_t count) {
    Program* prog = as_program(handle);
    if (!prog || !out || !prog->d_timings || count != static_cast<size_t>(8) * prog->workers * prog->length) return cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    return cudaMemcpy(out, prog->d_timings, count * sizeof(long long), cudaMemcpyDeviceToHost);
}
static int read_status(Program* prog, int* values, int count) {
    if (!values || count < 8) return cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    VmStatus st{};
    e = cudaMemcpy(&st, prog->d_status, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    values[0] = st.code; values[1] = st.worker; values[2] = st.stage; values[3] = st.band;
    values[4] = static_cast<int>(st.observed); values[5] = static_cast<int>(st.expected); values[6] = st.abort;
    values[7] = static_cast<int>(prog->epoch);
    if (st.abort || st.code) {
        e = cudaMemset(prog->d_status, 0, sizeof(VmStatus));
        if (e == cudaSuccess) e = cudaMemset(prog->d_counters, 0, sizeof(unsigned int) * std::max<size_t>(prog->expected.size(), 1));
        prog->epoch = 0;
    }
    return e;
}
extern "C" int read_native_model_status(void* handle, int* values, int count) {
    Program* prog = as_program(handle);
    if (!prog) {
        Op* op = as_op(handle);          // operator handles answer for their stand-alone program
        if (!op || !op->solo) return cudaErrorInvalidValue;
        prog = op->solo;
    }
    return read_status(prog, values, count);
}
extern "C" int read_native_model_counters(void* handle, unsigned int* counts, unsigned int* expected, int n, int* total) {
    Program* prog = as_program(handle);
    if (!prog) {
        Op* op = as_op(handle);
        if (!op || !op->solo) return cudaErrorInvalidValue;
        prog = op->solo;
    }
    const int have = static_cast<int>(prog->expected.size());
    if (total) *total = have;
    if (!counts && !expected) return cudaSuccess;
    if (n < have) return cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    if (counts) {
        e = cudaMemcpy(counts, prog->d_counters, sizeof(unsigned int) * have, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return e;
    }
    if (expected)
        for (int i = 0; i < have; i++) expected[i] = prog->expected[i] * prog->epoch;
    return cudaSuccess;
}
// extension: the kernel variant a program launches: 1 = the lean kernel (NVFP4 projections with the model's epilogues and
// tcgen05 attention only), 0 = the kernel with every operator and option.
extern "C" int native_model_kernel_variant(void* handle, int* lean) {
    Program* prog = as_program(handle);
    if (!prog || !lean) return cudaErrorInvalidValue;
    *lean = (prog->lean && !prog->h_debug) ? 1 : 0;             // (progress marks are written by the full variant only)
    return cudaSuccess;
}
extern "C" int enable_native_model_debug(void* handle, int enable) {
    Program* prog = as_program(handle);
    if (!prog) return cudaErrorInvalidValue;
    if (enable && !prog->h_debug) {
        const size_t bytes = sizeof(int) * prog->workers * (kThreads / 32);
        cudaError_t e = cudaHostAlloc(&prog->h_debug, bytes, cudaHostAllocMapped);
        if (e != cudaSuccess) { prog->h_debug = nullptr; return e; }
        memset(prog->h_debug, 0, bytes);
    } else if (!enable && prog->h_debug) {
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) return e;
        cudaFreeHost(prog->h_debug);
        prog->h_debug = nullptr;
    }
    return cudaSuccess;
}
extern "C" int read_native_model_debug(void* handle, int* out, int n) {
    Program* prog = as_program(handle);
    if (!prog || !prog->h_debug || !out || n < prog->workers * (kThreads / 32)) return cudaErrorInvalidValue;
    memcpy(out, prog->h_debug, sizeof(int) * prog->workers * (kThreads / 32));
    return cudaSuccess;
}
extern "C" int set_native_model_wait_budget(void* handle, unsigned long long nanoseconds) {
    Program* prog = as_program(handle);
    if (!prog) {
        Op* op = as_op(handle);
        if (!op) return cudaErrorInvalidValue;
        int e = solo_program(op);
        if (e) return e;
        prog = op->solo;
    }
    if (nanoseconds < 1000) return cudaErrorInvalidValue;
    prog->budget_ns = nanoseconds;
    return cudaSuccess;
}
extern "C" int destroy_native_model(void* handle) {
    if (!handle) return cudaSuccess;
    Program* prog = as_program(handle);
    if (!prog) return cudaErrorInvalidValue;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device != prog->device) return cudaErrorInvalidDevice;
    prog->magic = 0;
    delete prog;
    return cudaSuccess;
}

// =====================================================================================================
extern "C" int create_native_linear(void** handle, int count, void* const* stage_handles, const int* parents, const int* code,
                                    int workers, int length) {
    if (!handle) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (count < 1 || !stage_handles || !parents) return cudaErrorInvalidValue;
    std::vector<NativeSpec> specs(count);
    for (int i = 0; i < count; i++) {
        Op* op = as_op(stage_handles[i]);
        if (!op || op->desc.kind != OP_GEMM) return cudaErrorInvalidValue;
        specs[i].kind = 0;
        specs[i].handle = stage_handles[i];
        for (int s = 0; s < 4; s++) { specs[i].sources[s] = -1; specs[i].modes[s] = 0; }
        if (parents[i] < -1 || parents[i] >= i) return cudaErrorInvalidValue;
        specs[i].sources[0] = parents[i];
    }
    return create_native_model(handle, count, specs.data(), code, workers, length);
}
extern "C" int launch_native_linear(void* handle, void* stream) { return launch_native_model(handle, stream, nullptr, nullptr, nullptr, nullptr); }
extern "C" int read_native_linear(void* handle, unsigned long long* counters, int count, unsigned long long* epoch) {
    Program* prog = as_program(handle);
    if (!prog || !counters || !epoch || count != static_cast<int>(prog->expected.size())) return cudaErrorInvalidValue;
    std::vector<unsigned int> raw(count);
    int e = read_native_model_counters(handle, raw.data(), nullptr, count, nullptr);
    if (e) return e;
    // reported in tiles (a GEMM tile is four warp contributions)
    for (int i = 0; i < count; i++) counters[i] = raw[i] / 4;
    *epoch = prog->epoch;
    return cudaSuccess;
}
extern "C" int destroy_native_linear(void* handle) { return destroy_native_model(handle); }

// =====================================================================================================
extern "C" int quantize_nvfp4(const void* in, void* out, void* scales, int rows, int width, int ld_in, int out_blocks,
                              float global_scale, int policy, void* stream) {
    if (!in || !out || !scales || rows < 1 || width < 16 || width % 16 || ld_in < width || ld_in % 8 || out_blocks < width / 16 ||
        !std::isfinite(global_scale) || global_scale <= 0 || (policy != 0 && policy != 1))
        return cudaErrorInvalidValue;
    int device = 0;
    int e = check_device(&device);
    if (e) return e;
    NormParams n{};
    n.in = in; n.rows = rows; n.width = width; n.mode = 2; n.inv_gs = 1.f / global_scale; n.policy = policy;
    n.out = static_cast<uint8_t*>(out); n.out_scales = static_cast<uint8_t*>(scales);
    n.out_blocks = out_blocks; n.ld_in = ld_in; n.ld_out = width / 2;
    quantize_rows_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(n);
    return cudaGetLastError();
}

// =====================================================================================================
// Allocation-free split-KV attention.
//
// Some callers may not allocate device memory at the moment they need attention: a robot control loop that
// must never block on the driver's allocator (cudaMalloc takes a process-wide lock and synchronises the
// device, which can cost milliseconds in the middle of a 20 ms control period), or a process that has handed
// all of its device memory to another runtime's pool at start-up.  For them the split-KV partials live in a
// file-scope device array of fixed size instead of a buffer obtained from cudaMalloc.  The array exists once
// per GPU that loads this library (about 4.1 MiB each, held until the process exits), is shared by every
// call, and keeps the previous call's contents.
namespace pi0 {
namespace {

constexpr int kNoAllocMaxParts = 64;                 // heads * splits
constexpr int kNoAllocHeadDim = 256;
constexpr size_t kNoAllocPartialO = static_cast<size_t>(kNoAllocMaxParts) * kAttnQRows * kNoAllocHeadDim * sizeof(uint16_t);   // BF16 rows
constexpr size_t kNoAllocPartialMl = static_cast<size_t>(kNoAllocMaxParts) * kAttnQRows * 2 * sizeof(float);
constexpr int kNoAllocSmem = kAttnSmemBytes + 1024;     // operands and partial-row staging of attn_tile, plus alignment slack

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPartialO + kNoAllocPartialMl];

__global__ void __launch_bounds__(kThreads, 1) noalloc_attention_kernel(AttnParams a) {
    extern __shared__ uint8_t noalloc_smem[];
    uint8_t* data = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(noalloc_smem) + 1023) & ~static_cast<uintptr_t>(1023));
    attn_tile<kNoAllocHeadDim>(a, blockIdx.x, data, nullptr);
}
__global__ void __launch_bounds__(kThreads, 1) noalloc_merge_kernel(MergeParams g) { merge_tile(g, blockIdx.x); }

// Device address of the scratch array, looked up once per device.  In host code the array's name is only a
// handle for the runtime, never an address a kernel could use, so the address must come from
// cudaGetSymbolAddress with the owning device current.
struct NoAllocDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;
};
NoAllocDevice g_noalloc_device[64];
std::mutex g_noalloc_mutex;

int noalloc_setup(int device, unsigned char** scratch) {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocDevice& d = g_noalloc_device[device];
    if (!d.ready) {
        void* address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&address, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(noalloc_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kNoAllocSmem);
        if (e != cudaSuccess) return e;
        d.scratch = static_cast<unsigned char*>(address);
        d.ready = true;
    }
    *scratch = d.scratch;
    return cudaSuccess;
}

}  // namespace
}  // namespace pi0

extern "C" int attention_split_noalloc(const void* q, const void* k, const void* v, void* out, int nq, int nk, int heads,
                                       int kv_heads, int head_dim, int ldq, int ldkv, int out_ld, int prefix, int splits,
                                       float scale, void* stream) {
    if (!q || !k || !v || !out || nq < 1 || nk < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads || splits < 1 ||
        ldq < heads * head_dim || ldq % 8 || ldkv < kv_heads * head_dim || ldkv % 8 || out_ld < heads * head_dim || out_ld % 8 ||
        !std::isfinite(scale) || scale <= 0 || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
        return cudaErrorInvalidValue;
    // limits of the fixed scratch array: 256-wide heads, at most 128 queries, heads * splits <= 64
    if (head_dim != kNoAllocHeadDim || nq > kAttnQRows || heads * splits > kNoAllocMaxParts) return cudaErrorInvalidValue;
    int device = 0;
    int e = check_device(&device);
    if (e) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    unsigned char* scratch = nullptr;
    e = noalloc_setup(device, &scratch);
    if (e) return e;
    uint16_t* partial_o = reinterpret_cast<uint16_t*>(scratch);
    float* partial_ml = reinterpret_cast<float*>(scratch + kNoAllocPartialO);
    AttnParams a{};
    a.q = q; a.k = k; a.v = v;
    a.ldq = ldq; a.ldkv = ldkv; a.ldo = out_ld;
    a.batches = 1; a.nq = nq; a.nk = nk; a.q_batch_rows = nq; a.kv_batch_rows = nk;
    a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
    a.scale = scale;
    a.prefix = prefix >= 0 ? prefix : -1;
    a.splits = splits;
    a.out_inv_gs = 1.f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (splits == 1) {
        // One part per head: the tile normalises and stores its rows itself; no partials, no merge, the array is unused.
        a.out = out;
        noalloc_attention_kernel<<<heads, kThreads, kNoAllocSmem, s>>>(a);
        return cudaGetLastError();
    }
    a.out = nullptr;
    a.partial_o = partial_o; a.partial_ml = partial_ml;
    MergeParams g{};
    g.partial_o = partial_o; g.partial_ml = partial_ml;
    g.heads = heads; g.nq = nq; g.head_dim = head_dim; g.splits = splits;
    g.out = out; g.ldo = out_ld;
    g.out_inv_gs = 1.f;
    // Every partial word the merge reads (rows < nq of each head/split) is written by the attention kernel of
    // this same call first, so nothing in the shared array has to be cleared beforehand.
    noalloc_attention_kernel<<<heads * splits, kThreads, kNoAllocSmem, s>>>(a);
    cudaError_t launch = cudaGetLastError();
    if (launch != cudaSuccess) return launch;
    noalloc_merge_kernel<<<heads * ((nq + kMergeRows - 1) / kMergeRows), kThreads, 0, s>>>(g);
    return cudaGetLastError();
}

// =====================================================================================================
// Self-contained probes with HOST pointers (the reference builds them as separate libraries for its validation
// scripts: native_pi0/vm_probe.cu, tcgen_probe.cu, nvfp4_probe.cu).  Each call allocates, copies, launches, copies back
// and frees; nothing of it is on the path of a forward pass.
namespace {
struct DeviceBuffers {                               // frees whatever a probe allocated, on every return path
    std::vector<void*> owned;
    ~DeviceBuffers() { for (void* p : owned) cudaFree(p); }
    cudaError_t get(void** out, size_t bytes) {
        cudaError_t e = cudaMalloc(out, std::max<size_t>(bytes, 16));
        if (e == cudaSuccess) { owned.push_back(*out); e = cudaMemset(*out, 0, std::max<size_t>(bytes, 16)); }
        return e;
    }
};

// `repetitions` launches of one projection, each result copied to its own [m, n] FP32 slab of the host output.
// operands: GEMM_NVFP4 (sfa / sfb swizzled scale atoms), GEMM_BF16 or GEMM_FP8; k_pad >= k is the device row length.
int probe_gemm(int operands, const void* a, const void* b, const void* sfa, const void* sfb, float* out, int repetitions, int m,
               int n, int k, int workers, float alpha) {
    if (!a || !b || !out || repetitions < 1 || m < 128 || m % 128 || n < 128 || n % 128 || k < 64 || k % 64 || workers < 1 ||
        (operands == GEMM_NVFP4 && (!sfa || !sfb)) || !std::isfinite(alpha) || alpha <= 0)
        return cudaErrorInvalidValue;
    const int k_pad = operands == GEMM_FP8 ? (k + 127) / 128 * 128 : k;
    const size_t row = operand_row_bytes(operands, k), row_pad = operand_row_bytes(operands, k_pad);
    DeviceBuffers mem;
    void *da = nullptr, *db = nullptr, *dsa = nullptr, *dsb = nullptr, *dout = nullptr;
    cudaError_t e = mem.get(&da, row_pad * m);
    if (e == cudaSuccess) e = mem.get(&db, row_pad * n);
    if (e == cudaSuccess) e = mem.get(&dout, sizeof(float) * m * n);
    if (e == cudaSuccess) e = cudaMemcpy2D(da, row_pad, a, row, row, m, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy2D(db, row_pad, b, row, row, n, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && operands == GEMM_NVFP4) {
        const size_t groups = (static_cast<size_t>(k) / 16 + 3) / 4;
        const size_t bytes_a = static_cast<size_t>(m / 128) * groups * 512, bytes_b = static_cast<size_t>(n / 128) * groups * 512;
        e = mem.get(&dsa, bytes_a);
        if (e == cudaSuccess) e = mem.get(&dsb, bytes_b);
        if (e == cudaSuccess) e = cudaMemcpy(dsa, sfa, bytes_a, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(dsb, sfb, bytes_b, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) return e;
    void* handle = nullptr;
    int code = operands == GEMM_NVFP4 ? create_resident_fp4(&handle, da, db, dsa, dsb, dout, m, n, k, workers, alpha)
                                      : create_dense(&handle, da, db, dout, nullptr, nullptr, m, n, k_pad, workers, operands == GEMM_FP8, 0, alpha);
    if (code) return code;
    for (int r = 0; r < repetitions && !code; r++) {
        code = cudaMemsetAsync(dout, 0xFF, sizeof(float) * m * n, nullptr);          // a repetition that stored nothing would show
        if (!code) code = launch_solo(handle, nullptr);
        if (!code) code = cudaMemcpy(out + static_cast<size_t>(r) * m * n, dout, sizeof(float) * m * n, cudaMemcpyDeviceToHost);
        int status[8] = {};
        if (!code) code = read_native_model_status(handle, status, 8);
        if (!code && status[0]) code = cudaErrorLaunchFailure;
    }
    const int freed = destroy_checked(handle);
    return code ? code : freed;
}
}  // namespace

// Replaces: native_pi0/tcgen_probe.cu (run_tcgen_probe, run_fp8_probe, run_k_probe, run_grid_probe) - BF16 (precision 0) or
// FP8 E4M3 (precision 1) host operands a [m, k], b [n, k]; out FP32 [repetitions, m, n] = (a_scale * w_scale) * a b^T.
extern "C" int run_tcgen_probe(const void* a, const void* b, float* out, int repetitions) {
    return probe_gemm(GEMM_BF16, a, b, nullptr, nullptr, out, repetitions, 128, 128, 64, 1, 1.f);
}
extern "C" int run_fp8_probe(const void* a, const void* b, float* out, int repetitions, float a_scale, float w_scale) {
    return probe_gemm(GEMM_FP8, a, b, nullptr, nullptr, out, repetitions, 128, 128, 64, 1, a_scale * w_scale);
}
extern "C" int run_k_probe(const void* a, const void* b, float* out, int repetitions, int k, int precision, float a_scale, float w_scale) {
    if (precision != 0 && precision != 1) return cudaErrorInvalidValue;
    return probe_gemm(precision ? GEMM_FP8 : GEMM_BF16, a, b, nullptr, nullptr, out, repetitions, 128, 128, k, 1, a_scale * w_scale);
}
extern "C" int run_grid_probe(const void* a, const void* b, float* out, int repetitions, int m, int n, int k, int workers, int precision,
                              float a_scale, float w_scale) {
    if (precision != 0 && precision != 1) return cudaErrorInvalidValue;
    return probe_gemm(precision ? GEMM_FP8 : GEMM_BF16, a, b, nullptr, nullptr, out, repetitions, m, n, k, workers, a_scale * w_scale);
}
// Replaces: native_pi0/nvfp4_probe.cu:293-299 - packed NVFP4 host operands with swizzled scale atoms.
extern "C" int run_nvfp4_probe(const void* a, const void* b, const void* sa, const void* sb, float* out, int repetitions, float alpha, int k) {
    return probe_gemm(GEMM_NVFP4, a, b, sa, sb, out, repetitions, 128, 128, k, 1, alpha);
}
extern "C" int run_nvfp4_grid_probe(const void* a, const void* b, const void* sa, const void* sb, float* out, int repetitions, int m, int n,
                                    int k, int workers, float alpha) {
    return probe_gemm(GEMM_NVFP4, a, b, sa, sb, out, repetitions, m, n, k, workers, alpha);
}
// Replaces: native_pi0/vm_probe.cu:34 - `workers` CTAs run `instructions` instructions each; host_output int32
// [workers, instructions, 16] receives, per instruction and reporting slot, the CTA's tensor-memory base + 1 (this kernel has
// eight warps: warp w fills slots w and w + 8), so every entry is positive and equal within a worker.
extern "C" int run_vm_probe(int workers, int instructions, int* host_output) {
    if (workers < 1 || instructions < 1 || !host_output) return cudaErrorInvalidValue;
    int device = 0;
    int code = check_device(&device);
    if (code) return code;
    if (workers > sm_count(device)) return cudaErrorInvalidConfiguration;
    const size_t count = static_cast<size_t>(workers) * instructions;
    DeviceBuffers mem;
    void* dout = nullptr;
    cudaError_t e = mem.get(&dout, count * 16 * sizeof(int));
    if (e != cudaSuccess) return e;
    StageDesc d{};
    d.kind = OP_PROBE;
    finish_desc(d);
    d.tiles = static_cast<int>(count);
    d.bands = 1;
    d.band_div = d.tiles;
    d.p.probe.out = static_cast<int*>(dout);
    std::vector<int> code4(count * 4);
    for (int w = 0; w < workers; w++)
        for (int i = 0; i < instructions; i++) {
            int* ins = &code4[(static_cast<size_t>(w) * instructions + i) * 4];
            ins[0] = 1; ins[1] = 0; ins[2] = w * instructions + i; ins[3] = 1;
        }
    Program* prog = nullptr;
    code = build_program(&prog, device, std::vector<StageDesc>{d}, code4, workers, instructions);
    if (code) return code;
    std::unique_ptr<Program> owner(prog);
    code = launch_program(prog, nullptr, LaunchInputs{}, 0, 1, true);
    int status[8] = {};
    if (!code) code = read_status(prog, status, 8);
    if (!code && status[0]) code = cudaErrorLaunchFailure;
    if (!code) code = cudaMemcpy(host_output, dout, count * 16 * sizeof(int), cudaMemcpyDeviceToHost);
    return code;
}
