// C ABI of libllmini_b200.so: argument validation, the Muon plan (workspace carving, tile
// lists, TMA descriptors) and the step driver.  Host side of the reference's
// `OptimizerModule` / `Nvfp4QuantModule` launch wrappers
// (crates/cuda-kernels/src/gpt/optimizer/launcher/*.rs, .../utils/nvfp4/quant/*.rs).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "internal.h"

using namespace b2;

namespace {

constexpr uint32_t kChunkHost = 2048;  // values per streaming chunk (kChunk on the device side)
// Largest tensor any entry point accepts: the kernels index elements and chunks in 32 bits, and
// (len + 2047) / 2048 must not wrap.
constexpr uint64_t kMaxFlatElements = 0xfffff000ull;
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
};
// Current device and its SM count; fails when no CUDA device is usable.
cudaError_t device_info(DeviceInfo &out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static std::mutex mu;
    static int cached[64];
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (cached[dev] == 0) {
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        cached[dev] = n;
    }
    out.device = dev;
    out.sm_count = cached[dev];
    return cudaSuccess;
}
int stream_grid_cap(const DeviceInfo &d) { return d.sm_count * 8; }  // 8 x 256 threads per SM

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}
// 2-D row-major tensor [rows][cols] with `pitch_bytes` between rows; box = box_cols x box_rows,
// 128-byte swizzle, zero fill outside the tensor.
bool make_map(CUtensorMap *m, void *base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
              uint32_t box_cols, uint32_t box_rows, bool swizzle = true) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    return fn(m, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// crates/cuda-kernels/src/gpt/optimizer/muon/polar/fused/coefficients.rs:9-42
void reference_coefficients(uint32_t iter, float &a, float &b, float &c) {
    static const float raw[5][3] = {{8.287212f, -23.595886f, 17.300388f},
                                    {4.107059f, -2.94785f, 0.5448431f},
                                    {3.948691f, -2.9089022f, 0.55181915f},
                                    {3.3184197f, -2.488488f, 0.5100489f},
                                    {2.300652f, -1.668904f, 0.4188073f}};
    if (iter < 5) {
        a = raw[iter][0] / 1.01f;
        b = raw[iter][1] / 1.030301f;
        c = raw[iter][2] / 1.0510101f;
    } else {
        a = 1.875f; b = -1.25f; c = 0.375f;
    }
}

double slot_flops(uint32_t rows, uint32_t cols) {
    double n = std::min(rows, cols), m = std::max(rows, cols);
    return 4.0 * n * n * m + 2.0 * n * n * n;
}

enum ProblemType { kGram0 = 0, kGram1, kPoly, kApply0, kApply1, kLast0, kLast1, kProblemTypes };
// load maps: *K = box 64 (K) x 128 rows for K-major use, *M = box 64 x 64 for MN-major use
enum MapKind { kLX0K = 0, kLX1K, kLX0M, kLX1M, kLG, kLQ, kMapsPerSlot };

struct SlotLayout {
    uint32_t rows, cols, n, m, ldg, tiles_m_nn, tiles_n_nn, sub_m_nn;
    uint64_t len;
    size_t off_x[2], off_u, off_g16, off_q16, off_frag, off_factors;
};
struct Layout {
    std::vector<SlotLayout> slots;
    std::vector<uint32_t> chunk_prefix;  // slot_count + 1
    std::vector<uint32_t> unit_prefix;   // slot_count + 1: NorMuon work units (32 rows or 128 columns)
    std::vector<uint32_t> items;         // work list of the fused update + encode launch
    std::vector<uint32_t> group_item_begin;   // groups + 1 entries: where each finish group's part of `items` begins
    uint32_t chain_tiles = 0;            // entries of the chained Newton-Schulz work list (0: not built)
    uint32_t chain_iterations = 0;
    uint32_t gp_tiles = 0;               // entries of ONE fused Gram + polynomial work list (0: not built); three lists
    uint32_t gp_widest = 0;              // most Gram tiles any one matrix has
    uint32_t total_chunks = 0;
    int bn = 256;
    int pair = 0;   // 1: two-CTA 256 x 256 tiles
    int symmetric = 0;  // 1: Gram / Poly compute the upper triangle of tiles only
    int tile_m = 128;
    size_t off_prefix, off_partials, off_inv_norm, off_amax_x, off_status, off_x0_ptrs, off_x1_ptrs, off_u_ptrs, off_maps,
        off_problems, off_tiles_nn, off_tiles_out, off_unit_prefix, off_factor_ptrs, off_unit_partials, off_slot_stats,
        off_items, off_fused_sync, off_chain, off_gp, off_chain_sync, off_meta_end, total;
    uint32_t tiles_nn = 0, tiles_out = 0;
};

bool valid_shape(uint32_t rows, uint32_t cols, const b2_muon_options &o) {
    if ((uint64_t)rows * cols == 0) return true;  // padding slot, skipped
    if (cols % 16 != 0) return false;
    if ((uint64_t)rows * cols > kMaxFlatElements) return false;
    // tile indices are 16-bit (GemmTile): at most 65535 tiles of 128 along either dimension
    if ((std::max(rows, cols) + 127u) / 128u > 65535u) return false;
    if (o.scale_layout == B2_SCALES_CSF && cols % 128 != 0) return false;
    return true;
}

// Tile configuration: reserved[0] = 128 / 256 forces the single-CTA kernel with that width,
// 512 forces the two-CTA pair; 0 picks the cheapest by padded tensor work, weighted by how
// well each configuration feeds the tensor core (measured: the pair streams 1.5x fewer bytes
// per FLOP than 128 x 256, which in turn beats 128 x 128).
void pick_tiles(const uint32_t *rows, const uint32_t *cols, uint32_t count, const b2_muon_options &o, int &bn,
                int &pair) {
    if (o.tile_override == 128 || o.tile_override == 256) { bn = (int)o.tile_override; pair = 0; return; }
    if (o.tile_override == 512) { bn = 256; pair = 1; return; }
    const int tm[3] = {128, 128, 256}, tn[3] = {128, 256, 256};
    const double weight[3] = {1.9, 1.45, 1.0};
    double cost[3] = {0, 0, 0};
    for (int ci = 0; ci < 3; ++ci) {
        for (uint32_t s = 0; s < count; ++s) {
            if ((uint64_t)rows[s] * cols[s] == 0) continue;
            double n = std::min(rows[s], cols[s]), m = std::max(rows[s], cols[s]);
            auto pad = [](double v, double t) { return std::ceil(v / t) * t; };
            bool tall = rows[s] > cols[s];
            double nn = pad(n, tm[ci]) * pad(n, tn[ci]);
            double out = tall ? pad(m, tm[ci]) * pad(n, tn[ci]) : pad(n, tm[ci]) * pad(m, tn[ci]);
            cost[ci] += weight[ci] * (nn * m + nn * n + out * n);
        }
    }
    int best = 0;
    for (int ci = 1; ci < 3; ++ci)
        if (cost[ci] < cost[best]) best = ci;
    bn = tn[best];
    pair = best == 2;
}

// Work list of the fused update + encode launch, for the slot groups [first[g], first[g + 1]): the lists of the
// groups follow one another in L.items, group g's being items[group_item_begin[g] .. group_item_begin[g + 1]).
// Within a group: update chunks in slot order; the encode spans (B2_FUSED_ENCODE_SPAN chunks each) of a matrix
// become eligible kLag update chunks after its last one -- late enough that they never wait in practice, early
// enough that the updated weights are still in L2 -- and are then fed in one per kEvery update chunks (they
// arrive at one per B2_FUSED_ENCODE_SPAN), so that the issue-bound encode work is spread over the memory-bound
// update work instead of arriving as a block (measured 390 us against 405 us; with kLag 4000, or a feed slower
// than the arrival, the weights have left L2 and it is 420 us).  A group's list ends with the encode spans still
// pending, so every group is complete in itself and the total length does not depend on the grouping.
void build_items(Layout &L, const std::vector<uint32_t> &first) {
    const uint32_t kLag = 1200, kEvery = 3, kEncodeFlag = 0x80000000u;
    L.items.clear();
    L.group_item_begin.assign(1, 0u);
    for (size_t g = 0; g + 1 < first.size(); ++g) {
        std::vector<std::pair<uint32_t, uint32_t>> pending;   // (eligible at update position, encode item)
        size_t head = 0;
        uint32_t since = 0;
        for (uint32_t s = first[g]; s < first[g + 1]; ++s) {
            const uint32_t lo = L.chunk_prefix[s], hi = L.chunk_prefix[s + 1];
            for (uint32_t c = lo; c < hi; ++c) {
                L.items.push_back(c);
                if (++since >= kEvery && head < pending.size() && pending[head].first <= c) {
                    L.items.push_back(pending[head++].second);
                    since = 0;
                }
            }
            for (uint32_t c = lo; c < hi; c += B2_FUSED_ENCODE_SPAN) pending.emplace_back(hi - 1 + kLag, kEncodeFlag | c);
        }
        while (head < pending.size()) L.items.push_back(pending[head++].second);
        L.group_item_begin.push_back((uint32_t)L.items.size());
    }
}

bool build_layout(const uint32_t *rows, const uint32_t *cols, uint32_t count, const b2_muon_options &o, Layout &L) {
    pick_tiles(rows, cols, count, o, L.bn, L.pair);
    L.tile_m = L.pair ? 256 : 128;
    L.symmetric = (L.pair && L.bn == 256) ? 1 : 0;
#ifdef B2_MEASURE
    if (o.measure_flags & 4u) L.symmetric = 0;   // all tiles of the symmetric outputs
#endif
    L.slots.resize(count);
    L.chunk_prefix.assign(count + 1, 0);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t at = off;
        off = align_up(off + bytes, 1024);
        return at;
    };
    uint32_t chunks = 0;
    for (uint32_t s = 0; s < count; ++s) {
        if (!valid_shape(rows[s], cols[s], o)) return false;
        L.chunk_prefix[s] = chunks;
        chunks += (uint32_t)(((uint64_t)rows[s] * cols[s] + kChunkHost - 1) / kChunkHost);
    }
    L.chunk_prefix[count] = chunks;
    L.total_chunks = chunks;
    L.unit_prefix.assign(count + 1, 0);
    for (uint32_t s = 0; s < count; ++s) {
        uint32_t units = 0;
        if ((uint64_t)rows[s] * cols[s] != 0) units = rows[s] >= cols[s] ? (rows[s] + B2_NORMUON_ROWS_PER_UNIT - 1) / B2_NORMUON_ROWS_PER_UNIT : (cols[s] + 127) / 128;
        L.unit_prefix[s + 1] = L.unit_prefix[s] + units;
    }
    // ---- metadata region (uploaded at plan creation) ----
    L.off_prefix = take((count + 1) * sizeof(uint32_t));
    L.off_x0_ptrs = take(count * sizeof(uint64_t));
    L.off_u_ptrs = take(count * sizeof(uint64_t));
    L.off_x1_ptrs = take(count * sizeof(uint64_t));
    build_items(L, std::vector<uint32_t>{0u, count});
    L.off_items = take(std::max<size_t>(L.items.size(), 1) * sizeof(uint32_t));
    L.off_unit_prefix = take((count + 1) * sizeof(uint32_t));
    L.off_factor_ptrs = take(count * sizeof(uint64_t));
    L.off_maps = take((size_t)count * kMapsPerSlot * sizeof(CUtensorMap));
    L.off_problems = take((size_t)kProblemTypes * count * sizeof(GemmProblem));
    L.tiles_nn = L.tiles_out = 0;
    for (uint32_t s = 0; s < count; ++s) {
        SlotLayout &sl = L.slots[s];
        sl.rows = rows[s]; sl.cols = cols[s];
        sl.len = (uint64_t)rows[s] * cols[s];
        sl.n = std::min(rows[s], cols[s]); sl.m = std::max(rows[s], cols[s]);
        sl.ldg = (uint32_t)align_up(sl.n, 8);
        sl.tiles_m_nn = (sl.n + L.tile_m - 1) / L.tile_m;
        sl.tiles_n_nn = (sl.n + L.bn - 1) / L.bn;
        sl.sub_m_nn = sl.tiles_m_nn * (L.tile_m / kGemmBlockM);  // 128-row sub-tiles (fragment scratch)
        if (sl.len == 0) continue;
        L.tiles_nn += L.symmetric ? sl.tiles_m_nn * (sl.tiles_m_nn + 1) / 2 : sl.tiles_m_nn * sl.tiles_n_nn;
        uint32_t M = rows[s] > cols[s] ? sl.m : sl.n, N = rows[s] > cols[s] ? sl.n : sl.m;
        L.tiles_out += ((M + L.tile_m - 1) / L.tile_m) * ((N + L.bn - 1) / L.bn);
    }
    L.off_tiles_nn = take((size_t)std::max(L.tiles_nn, 1u) * sizeof(GemmTile));
    L.off_tiles_out = take((size_t)std::max(L.tiles_out, 1u) * sizeof(GemmTile));
    // the whole Newton-Schulz loop as one work list, for the iteration count the plan is made for
    L.chain_iterations = 0;
    L.chain_tiles = 0;
    if (o.ns_schedule == B2_NS_CHAINED && o.max_iterations <= kMaxChainIterations && count <= 0xffffu) {
        L.chain_iterations = o.max_iterations;
        L.chain_tiles = o.max_iterations * (2 * L.tiles_nn + L.tiles_out);
    }
    L.off_chain = take((size_t)std::max(L.chain_tiles, 1u) * sizeof(ChainTile));
    // fused Gram + polynomial tiles: one list for the first iteration, one for odd and one for later even ones
    L.gp_tiles = (o.ns_schedule == B2_NS_FUSED_GRAM_POLY && count <= 0xffffu) ? L.tiles_nn : 0u;
    L.off_gp = take((size_t)std::max(3u * L.gp_tiles, 1u) * sizeof(ChainTile));
    L.off_meta_end = off;
    // ---- per-step scratch ----
    L.off_partials = take((size_t)std::max(chunks, 1u) * B2_ONE_PASS_PARTIALS * sizeof(double));
    L.off_inv_norm = take(count * sizeof(float));
    L.off_amax_x = take(count * sizeof(float));
    L.off_status = take(sizeof(uint32_t));
    L.off_unit_partials = take((size_t)std::max(L.unit_prefix[count], 1u) * 4 * sizeof(double));
    L.off_slot_stats = take((size_t)count * 4 * sizeof(float));
    L.off_fused_sync = take(fused_sync_bytes(count));
    L.off_chain_sync = take(chain_sync_bytes(count));
    for (uint32_t s = 0; s < count; ++s) {
        SlotLayout &sl = L.slots[s];
        if (sl.len == 0) continue;
        sl.off_x[0] = take(sl.len * 2);
        sl.off_x[1] = take(sl.len * 2);
        sl.off_u = take(sl.len * 4);
        sl.off_g16 = take((size_t)sl.n * sl.ldg * 2);
        sl.off_q16 = take((size_t)sl.n * sl.ldg * 2);
        sl.off_frag = take((size_t)sl.sub_m_nn * sl.tiles_n_nn * kGemmBlockM * L.bn * 4);
        sl.off_factors = take((size_t)sl.m * 4);
    }
    L.total = off;
    return true;
}

b2_muon_options normalized(const b2_muon_options *o) {
    b2_muon_options r;
    std::memset(&r, 0, sizeof(r));
    if (o) r = *o;
    if (r.max_iterations == 0) r.max_iterations = 5;
#ifndef B2_MEASURE
    r.measure_phase_mask = r.measure_flags = 0;   // honoured only by a library built with -DB2_MEASURE
#endif
    return r;
}

}  // namespace

struct b2_muon_plan {
    Layout layout;
    b2_muon_options options;
    DeviceInfo dev;
    uint8_t *ws = nullptr;
    std::vector<uint8_t> meta;  // host image of the metadata region
    double flops_per_iteration = 0.0;
    uint64_t fused_wait_ns = 2000000000ull;   // limit of the completion-counter wait in the update + encode launch
    uint32_t resident_groups = 0;             // CTAs (pairs) of the ticketed GEMM kernel the device runs at once

    template <typename T>
    T *at(size_t off) const { return reinterpret_cast<T *>(ws + off); }
    SlotView view(const b2_muon_slot_descriptor *d_slots) const {
        SlotView v;
        v.slots = d_slots;
        v.chunk_prefix = at<uint32_t>(layout.off_prefix);
        v.slot_count = (uint32_t)layout.slots.size();
        v.total_chunks = layout.total_chunks;
        v.grid = stream_grid_cap(dev);
        return v;
    }
    NeuronView neurons() const {
        NeuronView nv;
        nv.unit_prefix = at<uint32_t>(layout.off_unit_prefix);
        nv.total_units = layout.unit_prefix.back();
        nv.factor_ptrs = at<uint64_t>(layout.off_factor_ptrs);
        nv.partials = at<double>(layout.off_unit_partials);
        nv.slot_stats = at<float>(layout.off_slot_stats);
        return nv;
    }
};

extern "C" {

uint32_t b2_abi_version(void) { return B2_ABI_VERSION; }

const char *b2_error_string(int code) {
    if (code == B2_SUCCESS) return "success";
    return cudaGetErrorString(static_cast<cudaError_t>(code));
}

int b2_verify_storage_layout(void *stream) {
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    // The echo needs three words of device memory; borrow them from a stream-ordered
    // allocation-free place: a kernel argument cannot carry output, so use mapped pinned memory.
    uint32_t *host = nullptr;
    e = cudaHostAlloc(reinterpret_cast<void **>(&host), 3 * sizeof(uint32_t), cudaHostAllocMapped);
    if (e != cudaSuccess) return (int)e;
    host[0] = host[1] = host[2] = 0;
    uint32_t *dev_view = nullptr;
    e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&dev_view), host, 0);
    if (e == cudaSuccess) e = launch_layout_echo(dev_view, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    bool ok = e == cudaSuccess && host[0] == B2_MUON_STORAGE_LAYOUT_VERSION &&
              host[1] == sizeof(b2_muon_slot_descriptor) && host[2] == B2_ABI_VERSION;
    cudaFreeHost(host);
    if (e != cudaSuccess) return (int)e;
    return ok ? B2_SUCCESS : B2_ERROR_INVALID_VALUE;
}

size_t b2_muon_workspace_bytes(const uint32_t *rows, const uint32_t *cols, uint32_t slot_count,
                               const b2_muon_options *options) {
    if (!rows || !cols || slot_count == 0 || slot_count > 65535) return 0;
    Layout L;
    b2_muon_options o = normalized(options);
    if (!build_layout(rows, cols, slot_count, o, L)) return 0;
    return L.total;
}

int b2_muon_plan_create(b2_muon_plan **out, const uint32_t *rows, const uint32_t *cols, uint32_t slot_count,
                        const b2_muon_options *options, void *d_workspace, size_t workspace_bytes, void *stream) {
    if (!out || !rows || !cols || slot_count == 0 || slot_count > 65535 || !d_workspace) return B2_ERROR_INVALID_VALUE;
    if (reinterpret_cast<uintptr_t>(d_workspace) % 1024 != 0) return B2_ERROR_INVALID_VALUE;
    b2_muon_options o = normalized(options);
    if (o.operand_format > B2_OPERAND_F16 || o.scale_layout > B2_SCALES_SM100 || o.quantize_target > B2_QUANTIZE_Y ||
        o.normalize_mode > B2_NORMALIZE_DEFERRED || o.ns_schedule > B2_NS_FUSED_GRAM_POLY || o.update_input > B2_UPDATE_16BIT)
        return B2_ERROR_INVALID_VALUE;
    // an un-normalised update can leave F16's range: the one-pass prepare is for BF16 operands
    if (o.normalize_mode == B2_NORMALIZE_DEFERRED && o.operand_format != B2_OPERAND_BF16) return B2_ERROR_INVALID_VALUE;
    b2_muon_plan *p = new (std::nothrow) b2_muon_plan();
    if (!p) return (int)cudaErrorMemoryAllocation;
    p->options = o;
    cudaError_t e = device_info(p->dev);
    if (e != cudaSuccess) { delete p; return (int)e; }
    Layout &L = p->layout;
    if (!build_layout(rows, cols, slot_count, o, L) || L.total > workspace_bytes) { delete p; return B2_ERROR_INVALID_VALUE; }
    p->ws = static_cast<uint8_t *>(d_workspace);
    e = gemm_configure(L.bn, L.pair);
    if (e != cudaSuccess) { delete p; return (int)e; }
    p->resident_groups = (uint32_t)std::max(gemm_resident_groups(L.bn, L.pair, p->dev.sm_count), 0);

    p->meta.assign(L.off_meta_end, 0);
    uint8_t *h = p->meta.data();
    std::memcpy(h + L.off_prefix, L.chunk_prefix.data(), (slot_count + 1) * sizeof(uint32_t));
    uint64_t *x0p = reinterpret_cast<uint64_t *>(h + L.off_x0_ptrs);
    uint64_t *up = reinterpret_cast<uint64_t *>(h + L.off_u_ptrs);
    uint64_t *x1p = reinterpret_cast<uint64_t *>(h + L.off_x1_ptrs);
    uint64_t *fp = reinterpret_cast<uint64_t *>(h + L.off_factor_ptrs);
    std::memcpy(h + L.off_unit_prefix, L.unit_prefix.data(), (slot_count + 1) * sizeof(uint32_t));
    if (!L.items.empty()) std::memcpy(h + L.off_items, L.items.data(), L.items.size() * sizeof(uint32_t));
    CUtensorMap *maps = reinterpret_cast<CUtensorMap *>(h + L.off_maps);
    GemmProblem *probs = reinterpret_cast<GemmProblem *>(h + L.off_problems);
    auto dmap = [&](uint32_t s, int kind) {
        return reinterpret_cast<uint64_t>(p->ws + L.off_maps + ((size_t)s * kMapsPerSlot + kind) * sizeof(CUtensorMap));
    };
    bool ok = true;
    for (uint32_t s = 0; s < slot_count; ++s) {
        const SlotLayout &sl = L.slots[s];
        if (sl.len == 0) continue;
        p->flops_per_iteration += slot_flops(sl.rows, sl.cols);
        x0p[s] = reinterpret_cast<uint64_t>(p->ws + sl.off_x[0]);
        up[s] = reinterpret_cast<uint64_t>(p->ws + sl.off_u);
        x1p[s] = reinterpret_cast<uint64_t>(p->ws + sl.off_x[1]);
        fp[s] = reinterpret_cast<uint64_t>(p->ws + sl.off_factors);
        CUtensorMap *ms = maps + (size_t)s * kMapsPerSlot;
        const uint64_t xp = (uint64_t)sl.cols * 2, gp = (uint64_t)sl.ldg * 2;
        ok &= make_map(ms + kLX0K, p->ws + sl.off_x[0], 2, sl.rows, sl.cols, xp, 64, 128);
        ok &= make_map(ms + kLX1K, p->ws + sl.off_x[1], 2, sl.rows, sl.cols, xp, 64, 128);
        ok &= make_map(ms + kLX0M, p->ws + sl.off_x[0], 2, sl.rows, sl.cols, xp, 64, 64);
        ok &= make_map(ms + kLX1M, p->ws + sl.off_x[1], 2, sl.rows, sl.cols, xp, 64, 64);
        ok &= make_map(ms + kLG, p->ws + sl.off_g16, 2, sl.n, sl.n, gp, 64, 128);
        ok &= make_map(ms + kLQ, p->ws + sl.off_q16, 2, sl.n, sl.n, gp, 64, 128);
        const bool tall = sl.rows > sl.cols;
        const uint64_t frag = reinterpret_cast<uint64_t>(p->ws + sl.off_frag);
        for (int b = 0; b < 2; ++b) {
            GemmProblem &g = probs[(size_t)(kGram0 + b) * slot_count + s];
            g.map_a = g.map_b = dmap(s, (tall ? kLX0M : kLX0K) + b);
            g.out16 = reinterpret_cast<uint64_t>(p->ws + sl.off_g16);
            g.pitch16 = sl.ldg;
            g.frag32 = frag;
            g.M = g.N = sl.n; g.K = sl.m;
            g.a_mn_major = g.b_mn_major = tall ? 1u : 0u;
            g.tiles_n = sl.tiles_n_nn;
            for (int last = 0; last < 2; ++last) {
                GemmProblem &a = probs[(size_t)((last ? kLast0 : kApply0) + b) * slot_count + s];
                if (tall) {  // Y' = Y Q : A = Y [m][n] K-major, B = Q [n][n] K-major
                    a.map_a = dmap(s, kLX0K + b); a.map_b = dmap(s, kLQ);
                    a.a_mn_major = 0; a.b_mn_major = 0;
                    a.M = sl.m; a.N = sl.n;
                } else {     // X' = Q X : A = Q K-major, B = X [n][m] read as MN-major
                    a.map_a = dmap(s, kLQ); a.map_b = dmap(s, kLX0M + b);
                    a.a_mn_major = 0; a.b_mn_major = 1;
                    a.M = sl.n; a.N = sl.m;
                }
                a.K = sl.n;
                a.out16 = reinterpret_cast<uint64_t>(p->ws + sl.off_x[1 - b]);
                a.pitch16 = sl.cols;
                a.out32 = reinterpret_cast<uint64_t>(p->ws + sl.off_u);
                a.pitch32 = sl.cols;
                a.tiles_n = (a.N + L.bn - 1) / L.bn;
            }
        }
        GemmProblem &q = probs[(size_t)kPoly * slot_count + s];
        q.map_a = q.map_b = dmap(s, kLG);
        q.out16 = reinterpret_cast<uint64_t>(p->ws + sl.off_q16);
        q.pitch16 = sl.ldg;
        q.frag32 = frag;
        q.M = q.N = q.K = sl.n;
        q.tiles_n = sl.tiles_n_nn;
    }
    if (!ok) { delete p; return B2_ERROR_NOT_SUPPORTED; }
    // tile lists, most expensive slots first so the round-robin over CTAs ends evenly
    std::vector<uint32_t> order;
    for (uint32_t s = 0; s < slot_count; ++s)
        if (L.slots[s].len) order.push_back(s);
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
        const SlotLayout &x = L.slots[a], &y = L.slots[b];
        if (x.m != y.m) return x.m > y.m;
        return x.n > y.n;
    });
    GemmTile *tnn = reinterpret_cast<GemmTile *>(h + L.off_tiles_nn);
    GemmTile *tout = reinterpret_cast<GemmTile *>(h + L.off_tiles_out);
    uint32_t inn = 0, iout = 0;
    for (uint32_t s : order) {
        const SlotLayout &sl = L.slots[s];
        for (uint32_t i = 0; i < sl.tiles_m_nn; ++i)
            for (uint32_t j = 0; j < sl.tiles_n_nn; ++j) {
                // square 256 x 256 tiles: G and Q are symmetric, so only tiles on or above the
                // diagonal are computed and the others are written as transposes
                if (L.symmetric && j < i) continue;
                tnn[inn++] = GemmTile{(uint16_t)s, (uint16_t)i, (uint16_t)j, (uint16_t)((L.symmetric && j > i) ? 1 : 0)};
            }
    }
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return L.slots[a].n > L.slots[b].n; });
    for (uint32_t s : order) {
        const SlotLayout &sl = L.slots[s];
        const bool tall = sl.rows > sl.cols;
        uint32_t M = tall ? sl.m : sl.n, N = tall ? sl.n : sl.m;
        uint32_t tm = (M + L.tile_m - 1) / L.tile_m, tn = (N + L.bn - 1) / L.bn;
        for (uint32_t i = 0; i < tm; ++i)
            for (uint32_t j = 0; j < tn; ++j) tout[iout++] = GemmTile{(uint16_t)s, (uint16_t)i, (uint16_t)j, 0};
    }
    if (L.chain_tiles) {
        // Phase after phase, iteration after iteration, each phase in the order of its per-phase list.  `need`
        // of a tile = progress increments of its matrix's earlier phases (every tile is finished by `warps`
        // epilogue warps).
        ChainTile *ct = reinterpret_cast<ChainTile *>(h + L.off_chain);
        const uint32_t warps = chain_epilogue_warps(L.bn, L.pair);
        std::vector<uint32_t> done(slot_count, 0), nn_tiles(slot_count, 0), out_tiles(slot_count, 0);
        for (uint32_t i = 0; i < inn; ++i) ++nn_tiles[tnn[i].problem];
        for (uint32_t i = 0; i < iout; ++i) ++out_tiles[tout[i].problem];
        const bool deferred = o.normalize_mode == B2_NORMALIZE_DEFERRED;
        uint32_t n = 0;
        auto emit = [&](const GemmTile &t, uint32_t type, uint32_t epi, uint32_t scale_pow, uint32_t it) {
            ChainTile c = {};
            c.problem = type * slot_count + t.problem;
            c.tile_m = t.tile_m;
            c.tile_n = t.tile_n;
            c.slot = t.problem;
            c.epilogue = (uint8_t)epi;
            c.flags = (uint8_t)((t.reserved ? 1u : 0u) | (scale_pow << 1) | (it << 3));
            c.need = warps * done[t.problem];
            ct[n++] = c;
        };
        for (uint32_t it = 0; it < L.chain_iterations; ++it) {
            const uint32_t b = it & 1u;
            const bool last32 = it + 1 == L.chain_iterations && o.update_input == B2_UPDATE_F32;   // FP32 result
            const bool first_scaled = it == 0 && deferred;
            for (uint32_t i = 0; i < inn; ++i) emit(tnn[i], kGram0 + b, kEpiGram, first_scaled ? 2u : 0u, it);
            for (uint32_t s = 0; s < slot_count; ++s) done[s] += nn_tiles[s];
            for (uint32_t i = 0; i < inn; ++i) emit(tnn[i], kPoly, kEpiPoly, 0u, it);
            for (uint32_t s = 0; s < slot_count; ++s) done[s] += nn_tiles[s];
            for (uint32_t i = 0; i < iout; ++i)
                emit(tout[i], (last32 ? kLast0 : kApply0) + b, last32 ? kEpiApplyLast : kEpiApply, first_scaled ? 1u : 0u, it);
            for (uint32_t s = 0; s < slot_count; ++s) done[s] += out_tiles[s];
        }
    }
    if (L.gp_tiles) {
        // One entry per Gram tile, a matrix's entries next to each other: the CTA (pair) that draws it computes the
        // Gram tile, publishes its 16-bit form, waits for the matrix's other Gram tiles (need2) and goes on to the
        // polynomial tile of the same position.  The progress counts start from zero in every launch.
        ChainTile *gp = reinterpret_cast<ChainTile *>(h + L.off_gp);
        const uint32_t warps = chain_epilogue_warps(L.bn, L.pair);
        std::vector<uint32_t> nn_tiles(slot_count, 0);
        for (uint32_t i = 0; i < inn; ++i) ++nn_tiles[tnn[i].problem];
        L.gp_widest = 0;
        for (uint32_t s = 0; s < slot_count; ++s) L.gp_widest = std::max(L.gp_widest, nn_tiles[s]);
        const bool deferred = o.normalize_mode == B2_NORMALIZE_DEFERRED;
        for (uint32_t list = 0; list < 3; ++list) {
            const uint32_t b = list == 1 ? 1u : 0u;
            const uint32_t scale_pow = (list == 0 && deferred) ? 2u : 0u;
            for (uint32_t i = 0; i < inn; ++i) {
                ChainTile c = {};
                c.problem = (kGram0 + b) * slot_count + tnn[i].problem;
                c.tile_m = tnn[i].tile_m;
                c.tile_n = tnn[i].tile_n;
                c.slot = tnn[i].problem;
                c.epilogue = (uint8_t)kEpiGramPoly;
                c.flags = (uint8_t)((tnn[i].reserved ? 1u : 0u) | (scale_pow << 1));
                c.need = 0;
                c.problem2 = kPoly * slot_count + tnn[i].problem;
                c.need2 = warps * nn_tiles[tnn[i].problem];
                gp[(size_t)list * L.gp_tiles + i] = c;
            }
        }
    }
    e = cudaMemcpyAsync(p->ws, h, L.off_meta_end, cudaMemcpyHostToDevice, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(p->ws + L.off_status, 0, sizeof(uint32_t), as_stream(stream));
    if (e == cudaSuccess)
        e = cudaMemsetAsync(p->ws + L.off_chain_sync, 0, chain_sync_bytes(slot_count), as_stream(stream));
    if (e == cudaSuccess)
        e = cudaMemsetAsync(p->ws + L.off_fused_sync, 0, fused_sync_bytes(slot_count), as_stream(stream));
    if (e != cudaSuccess) { delete p; return (int)e; }
    *out = p;
    return B2_SUCCESS;
}

void b2_muon_plan_destroy(b2_muon_plan *plan) { delete plan; }

double b2_muon_plan_flops_per_iteration(const b2_muon_plan *plan) { return plan ? plan->flops_per_iteration : 0.0; }

static int check_step(const b2_muon_plan *plan, const b2_muon_step_args *a) {
    if (!plan || !a) return B2_ERROR_INVALID_VALUE;
    if (a->iterations == 0 || a->iterations > plan->options.max_iterations) return B2_ERROR_INVALID_VALUE;
    return B2_SUCCESS;
}

static MomentumParams momentum_params(const b2_muon_step_args *a) {
    MomentumParams mp;
    mp.mu = a->mu;
    mp.grad_scale = a->grad_scale;
    mp.d_grad_scale = a->d_grad_scale;
    mp.nesterov = (int)a->nesterov;
    mp.variance_adaptive = a->variance_adaptive ? 1 : 0;
    mp.bias_correction_inv = a->variance_adaptive ? a->bias_correction_inv : 1.0f;
    return mp;
}
static UpdateParams update_params(const b2_muon_step_args *a) {
    UpdateParams up;
    up.update_format = 0;
    up.lr = a->learning_rate;
    up.wd = a->weight_decay;
    up.c_avg = a->average_coefficient;
    up.beta = a->schedule_beta;
    up.d_qk_clip_factors = a->d_qk_clip_factors;
    up.normuon = 0;
    up.factor_ptrs = nullptr;
    up.slot_stats = nullptr;
    up.symexp_beta = a->symexp_lin_beta > 0.0f ? a->symexp_lin_beta : 0.0f;
    up.symexp_slots = a->d_symexp_lin_slots;
    return up;
}

int b2_muon_prepare_polar(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, const b2_muon_step_args *a,
                          void *stream) {
    if (!plan || !a || !d_slots) return B2_ERROR_INVALID_VALUE;
    const Layout &L = plan->layout;
    cudaStream_t s = as_stream(stream);
    SlotView v = plan->view(d_slots);
    double *partials = plan->at<double>(L.off_partials);
    float *inv = plan->at<float>(L.off_inv_norm);
    const MomentumParams mp = momentum_params(a);
    if (plan->options.normalize_mode == B2_NORMALIZE_DEFERRED) {
        // one pass over the gradients; the scalar goes to the first Newton-Schulz iteration (b2_muon_polar)
        cudaError_t e = launch_muon_momentum_sumsq(v, mp, plan->at<uint64_t>(L.off_x0_ptrs), partials,
                                                   plan->at<float>(L.off_amax_x), s);
        if (e == cudaSuccess) e = launch_muon_inv_norm(v, partials, inv, B2_ONE_PASS_PARTIALS, s);
        return (int)e;
    }
    cudaError_t e = launch_muon_sumsq(v, mp, partials, plan->at<float>(L.off_amax_x), s);
    if (e == cudaSuccess) e = launch_muon_inv_norm(v, partials, inv, 1u, s);
    if (e == cudaSuccess)
        e = launch_muon_momentum_normalize(v, mp, inv, plan->at<uint64_t>(L.off_x0_ptrs),
                                           plan->options.operand_format == B2_OPERAND_F16, s);
    return (int)e;
}

int b2_muon_polar(b2_muon_plan *plan, const b2_muon_step_args *a, void *stream) {
    int rc = check_step(plan, a);
    if (rc) return rc;
    const Layout &L = plan->layout;
    cudaStream_t s = as_stream(stream);
    const uint32_t count = (uint32_t)L.slots.size();
    const GemmProblem *probs = plan->at<GemmProblem>(L.off_problems);
    const GemmTile *tnn = plan->at<GemmTile>(L.off_tiles_nn), *tout = plan->at<GemmTile>(L.off_tiles_out);
    uint32_t *status = plan->at<uint32_t>(L.off_status);
    const int f16 = plan->options.operand_format == B2_OPERAND_F16;
    const int grid = plan->dev.sm_count;
    cudaError_t e = cudaSuccess;
    bool whole_loop = L.chain_tiles != 0 && a->iterations == L.chain_iterations;
#ifdef B2_MEASURE
    if (plan->options.measure_phase_mask) whole_loop = false;
#endif
    if (whole_loop) {
        // every GEMM of every iteration as one grid, ordered by per-matrix progress counts
        GemmCoefficients coef = {};
        for (uint32_t it = 0; it < a->iterations; ++it) {
            if (a->coefficients) {
                for (int k = 0; k < 3; ++k) coef.v[3 * it + k] = a->coefficients[3 * it + k];
            } else {
                reference_coefficients(it, coef.v[3 * it], coef.v[3 * it + 1], coef.v[3 * it + 2]);
            }
        }
        const float *scale = plan->options.normalize_mode == B2_NORMALIZE_DEFERRED ? plan->at<float>(L.off_inv_norm) : nullptr;
        return (int)launch_ns_chain(L.bn, L.pair, probs, plan->at<ChainTile>(L.off_chain), L.chain_tiles, f16, coef, scale,
                                    status, plan->ws + L.off_chain_sync, count, plan->options.measure_flags, grid, s);
    }
    // The fused form needs all Gram tiles of a matrix in flight at once: one CTA (pair) each.
    const bool fused_gram_poly = L.gp_tiles != 0 && L.gp_widest <= plan->resident_groups;
    for (uint32_t it = 0; it < a->iterations && e == cudaSuccess; ++it) {
        float ca, cb, cc;
        if (a->coefficients) {
            ca = a->coefficients[3 * it]; cb = a->coefficients[3 * it + 1]; cc = a->coefficients[3 * it + 2];
        } else {
            reference_coefficients(it, ca, cb, cc);
        }
        const uint32_t b = it & 1u;
        const bool last = it + 1 == a->iterations && plan->options.update_input == B2_UPDATE_F32;   // FP32 result
        // measurement builds only: phase mask (1 Gram, 2 Poly, 4 Apply; 0 = all) and kernel flags
        const uint32_t mask = plan->options.measure_phase_mask ? plan->options.measure_phase_mask : 7u;
        const uint32_t dbg = plan->options.measure_flags;
        // after a one-pass prepare the first iteration's operand is not normalised: its Gram output takes
        // s^2 and its Apply output s, s = inv_norm[slot]
        const float *scale = (it == 0 && plan->options.normalize_mode == B2_NORMALIZE_DEFERRED)
                                 ? plan->at<float>(L.off_inv_norm) : nullptr;
        if (fused_gram_poly && (mask & 3u) == 3u) {
            // Gram and polynomial tile of one position on one CTA (pair): the FP32 Gram tile stays in tensor memory
            GemmCoefficients coef = {};
            coef.v[0] = ca; coef.v[1] = cb; coef.v[2] = cc;
            const uint32_t list = it == 0 ? 0u : ((it & 1u) ? 1u : 2u);
            e = launch_ns_chain(L.bn, L.pair, probs, plan->at<ChainTile>(L.off_gp) + (size_t)list * L.gp_tiles, L.gp_tiles,
                                f16, coef, scale, status, plan->ws + L.off_chain_sync, count, dbg, grid, s, true);
        } else {
            if (mask & 1u)
                e = launch_ns_gemm(L.bn, L.pair, probs + (size_t)(kGram0 + b) * count, tnn, L.tiles_nn, kEpiGram, f16, ca, cb,
                                   cc, scale, 2u, status, dbg, grid, s);
            if (e == cudaSuccess && (mask & 2u))
                e = launch_ns_gemm(L.bn, L.pair, probs + (size_t)kPoly * count, tnn, L.tiles_nn, kEpiPoly, f16, ca, cb, cc,
                                   nullptr, 0u, status, dbg, grid, s);
        }
        if (e == cudaSuccess && (mask & 4u))
            e = launch_ns_gemm(L.bn, L.pair, probs + (size_t)((last ? kLast0 : kApply0) + b) * count, tout, L.tiles_out,
                               last ? kEpiApplyLast : kEpiApply, f16, ca, cb, cc, scale, 1u, status, dbg, grid, s);
    }
    return (int)e;
}

// group < 0: every slot of the plan; otherwise the slots of that finish group (fused update + encode launch only)
static int finish_impl(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, const b2_muon_step_args *a,
                       bool quantize, void *stream, int group = -1) {
    if (!plan || !a || !d_slots) return B2_ERROR_INVALID_VALUE;
    const Layout &L = plan->layout;
    if (group >= 0 && (size_t)group + 1 >= L.group_item_begin.size()) return B2_ERROR_INVALID_VALUE;
    cudaStream_t s = as_stream(stream);
    SlotView v = plan->view(d_slots);
    float *amax_x = plan->at<float>(L.off_amax_x);
    UpdateParams up = update_params(a);
    cudaError_t e = cudaSuccess;
    // where the Newton-Schulz result is: the FP32 buffer, or the 16-bit operand buffer the last iteration wrote
    const uint64_t *u_ptrs = plan->at<uint64_t>(L.off_u_ptrs);
    if (plan->options.update_input == B2_UPDATE_16BIT) {
        if (a->normuon) return B2_ERROR_NOT_SUPPORTED;
        if (a->iterations == 0 || a->iterations > plan->options.max_iterations) return B2_ERROR_INVALID_VALUE;
        u_ptrs = plan->at<uint64_t>((a->iterations & 1u) ? L.off_x1_ptrs : L.off_x0_ptrs);
        up.update_format = plan->options.operand_format == B2_OPERAND_F16 ? 2 : 1;
    }
    if (a->normuon) {
        const NeuronView nv = plan->neurons();
        e = launch_normuon_stats(v, nv, plan->at<uint64_t>(L.off_u_ptrs), 0, s);
        up.normuon = 1;
        up.factor_ptrs = nv.factor_ptrs;
        up.slot_stats = nv.slot_stats;
    }
    const int quantize_y = plan->options.quantize_target == B2_QUANTIZE_Y;
    // one launch for the plain update; NorMuon / qk-clip steps (and measurement flag 16) take two
    if (quantize && !(plan->options.measure_flags & 16u) && !up.normuon && !up.d_qk_clip_factors &&
        up.symexp_beta == 0.0f) {
        const uint32_t begin = group < 0 ? 0u : L.group_item_begin[group];
        const uint32_t end = group < 0 ? (uint32_t)L.items.size() : L.group_item_begin[group + 1];
        if (e == cudaSuccess && end > begin)
            e = launch_muon_update_encode(v, plan->at<uint32_t>(L.off_items) + begin, end - begin,
                                          u_ptrs, amax_x, up, quantize_y,
                                          (int)plan->options.scale_layout, plan->ws + L.off_fused_sync,
                                          plan->at<uint32_t>(L.off_status), plan->fused_wait_ns, s);
        return (int)e;
    }
    if (group >= 0) return B2_ERROR_NOT_SUPPORTED;   // the two-launch forms work on the whole plan
    if (e == cudaSuccess) e = launch_muon_update(v, u_ptrs, amax_x, up, s);
    if (e == cudaSuccess && quantize)
        e = launch_muon_encode(v, amax_x, quantize_y, (int)plan->options.scale_layout, s);
    return (int)e;
}
int b2_muon_finish_update(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, const b2_muon_step_args *a,
                          void *stream) {
    return finish_impl(plan, d_slots, a, true, stream);
}
int b2_muon_finish_update_deferred_quantization(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                                                const b2_muon_step_args *a, void *stream) {
    return finish_impl(plan, d_slots, a, false, stream);
}
int b2_muon_plan_set_finish_groups(b2_muon_plan *plan, const uint32_t *first_slot, uint32_t group_count, void *stream) {
    if (!plan || !first_slot || group_count == 0) return B2_ERROR_INVALID_VALUE;
    Layout &L = plan->layout;
    const uint32_t count = (uint32_t)L.slots.size();
    std::vector<uint32_t> first(first_slot, first_slot + group_count);
    if (first[0] != 0) return B2_ERROR_INVALID_VALUE;
    for (uint32_t g = 1; g < group_count; ++g)
        if (first[g] < first[g - 1] || first[g] > count) return B2_ERROR_INVALID_VALUE;
    first.push_back(count);
    const size_t before = L.items.size();
    build_items(L, first);
    if (L.items.size() != before) return B2_ERROR_INVALID_VALUE;   // (cannot happen: the grouping only reorders)
    if (L.items.empty()) return B2_SUCCESS;
    return (int)cudaMemcpyAsync(plan->ws + L.off_items, L.items.data(), L.items.size() * sizeof(uint32_t),
                                cudaMemcpyHostToDevice, as_stream(stream));
}
int b2_muon_finish_update_group(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, const b2_muon_step_args *a,
                                uint32_t group, void *stream) {
    if (group > 0x7fffffffu) return B2_ERROR_INVALID_VALUE;
    return finish_impl(plan, d_slots, a, true, stream, (int)group);
}

int b2_muon_materialize_master_weights(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, void *stream) {
    if (!plan || !d_slots) return B2_ERROR_INVALID_VALUE;
    SlotView v = plan->view(d_slots);
    return (int)launch_muon_encode(v, plan->at<float>(plan->layout.off_amax_x), 0, (int)plan->options.scale_layout,
                                   as_stream(stream));
}

int b2_muon_finish_hyperball_update_deferred_quantization(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                                                          const b2_muon_step_args *a, uint32_t use_schedule_free,
                                                          void *stream) {
    if (!plan || !a || !d_slots) return B2_ERROR_INVALID_VALUE;
    if (plan->options.update_input != B2_UPDATE_F32) return B2_ERROR_NOT_SUPPORTED;   // its statistics read FP32
    const Layout &L = plan->layout;
    cudaStream_t s = as_stream(stream);
    SlotView v = plan->view(d_slots);
    const NeuronView nv = plan->neurons();
    UpdateParams up = update_params(a);
    up.normuon = 1;
    up.factor_ptrs = nv.factor_ptrs;
    up.slot_stats = nv.slot_stats;
    cudaError_t e = launch_normuon_stats(v, nv, plan->at<uint64_t>(L.off_u_ptrs), 1, s);
    if (e == cudaSuccess)
        e = launch_muon_hyperball_update(v, plan->at<uint64_t>(L.off_u_ptrs), plan->at<float>(L.off_amax_x), up,
                                         use_schedule_free ? 1 : 0, s);
    return (int)e;
}

int b2_muon_sign_update_deferred_quantization(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                                              const b2_muon_step_args *a, void *stream) {
    if (!plan || !a || !d_slots) return B2_ERROR_INVALID_VALUE;
    SlotView v = plan->view(d_slots);
    return (int)launch_muon_sign_update(v, momentum_params(a), update_params(a),
                                        plan->at<float>(plan->layout.off_amax_x), as_stream(stream));
}

int b2_muon_mega_update(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, const b2_muon_step_args *a,
                        void *stream) {
    int rc = check_step(plan, a);
    if (rc) return rc;
    if (!d_slots) return B2_ERROR_INVALID_VALUE;
    rc = b2_muon_prepare_polar(plan, d_slots, a, stream);
    if (rc == 0) rc = b2_muon_polar(plan, a, stream);
    if (rc == 0) rc = b2_muon_finish_update(plan, d_slots, a, stream);
    return rc;
}

int b2_muon_plan_scratch(b2_muon_plan *plan, uint32_t slot, uint32_t which, void **d_ptr, size_t *bytes) {
    if (!plan || !d_ptr || !bytes) return B2_ERROR_INVALID_VALUE;
    const Layout &L = plan->layout;
    if (which == 4) { *d_ptr = plan->ws + L.off_status; *bytes = 4; return B2_SUCCESS; }
    if (which == 11) {
        *d_ptr = plan->ws + L.off_chain_sync;
        *bytes = chain_sync_bytes((uint32_t)L.slots.size());
        return B2_SUCCESS;
    }
    if (which == 10) {
        *d_ptr = plan->ws + L.off_fused_sync;
        *bytes = fused_sync_bytes((uint32_t)L.slots.size());
        return B2_SUCCESS;
    }
    if (slot >= L.slots.size()) return B2_ERROR_INVALID_VALUE;
    const SlotLayout &sl = L.slots[slot];
    if (sl.len == 0) return B2_ERROR_INVALID_VALUE;
    switch (which) {
        case 0: *d_ptr = plan->ws + sl.off_x[0]; *bytes = sl.len * 2; break;
        case 1: *d_ptr = plan->ws + sl.off_u; *bytes = sl.len * 4; break;
        case 2: *d_ptr = plan->ws + L.off_inv_norm + slot * 4; *bytes = 4; break;
        case 3: *d_ptr = plan->ws + L.off_amax_x + slot * 4; *bytes = 4; break;
        case 5: *d_ptr = plan->ws + sl.off_g16; *bytes = (size_t)sl.n * sl.ldg * 2; break;
        case 6: *d_ptr = plan->ws + sl.off_q16; *bytes = (size_t)sl.n * sl.ldg * 2; break;
        case 7: *d_ptr = plan->ws + sl.off_x[1]; *bytes = sl.len * 2; break;
        case 8: *d_ptr = plan->ws + sl.off_factors; *bytes = (size_t)sl.m * 4; break;
        case 9: *d_ptr = plan->ws + L.off_slot_stats + (size_t)slot * 16; *bytes = 16; break;
        default: return B2_ERROR_INVALID_VALUE;
    }
    return B2_SUCCESS;
}

int b2_muon_plan_status(b2_muon_plan *plan, void *stream) {
    if (!plan) return B2_ERROR_INVALID_VALUE;
    uint32_t st = 0;
    cudaStream_t s = as_stream(stream);
    uint32_t *d = plan->at<uint32_t>(plan->layout.off_status);
    cudaError_t e = cudaMemcpyAsync(&st, d, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(d, 0, 4, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return (int)e;
    return st ? B2_ERROR_LAUNCH_TIMEOUT : B2_SUCCESS;
}

// ---- quantiser ------------------------------------------------------------------------------
int b2_tensor_amax_f32(const float *d_x, float *d_chunk_amax, float *d_out, uint32_t n, void *stream) {
    if (!d_x || !d_chunk_amax || !d_out || n > kMaxFlatElements) return B2_ERROR_INVALID_VALUE;
    cudaError_t e = launch_tensor_chunk_amax(d_x, d_chunk_amax, n, as_stream(stream));
    if (e == cudaSuccess) e = launch_tensor_amax_from_chunks(d_chunk_amax, d_out, (n + 2047) / 2048, as_stream(stream));
    return (int)e;
}
int b2_tensor_amax_from_chunks_f32(const float *d_chunk_amax, float *d_out, uint32_t chunk_count, void *stream) {
    if (!d_chunk_amax || !d_out) return B2_ERROR_INVALID_VALUE;
    return (int)launch_tensor_amax_from_chunks(d_chunk_amax, d_out, chunk_count, as_stream(stream));
}
int b2_fp32_to_nvfp4_four_six(const float *d_x, const float *d_amax, uint8_t *d_out_fp4, uint8_t *d_out_scales,
                              float *d_out_global_scale, uint32_t group_count, uint32_t scale_layout, void *stream) {
    if (!d_x || !d_amax || !d_out_fp4 || !d_out_scales || !d_out_global_scale) return B2_ERROR_INVALID_VALUE;
    if (scale_layout > B2_SCALES_RAW || group_count > kMaxFlatElements / 16) return B2_ERROR_INVALID_VALUE;
    if (scale_layout == B2_SCALES_CSF && group_count % 8 != 0) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_quantize_flat(d_x, nullptr, nullptr, 0.f, 0, d_amax, d_out_fp4, d_out_scales, d_out_global_scale,
                                     group_count, (int)scale_layout, stream_grid_cap(d), as_stream(stream));
}
size_t b2_nvfp4_sm100_scales_bytes(uint32_t rows, uint32_t cols) {
    return (size_t)((rows + 127) / 128) * ((cols / 16 + 3) / 4) * 512;
}
int b2_nvfp4_scales_to_sm100(const uint8_t *d_scales, uint32_t src_layout, uint32_t rows, uint32_t cols,
                             uint8_t *d_out, void *stream) {
    if (!d_scales || !d_out || src_layout > B2_SCALES_RAW) return B2_ERROR_INVALID_VALUE;
    if (cols % 16 != 0 || (src_layout == B2_SCALES_CSF && cols % 128 != 0)) return B2_ERROR_INVALID_VALUE;
    if ((uint64_t)rows * cols > 0xfffff000ull) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_scales_to_sm100(d_scales, src_layout == B2_SCALES_CSF, rows, cols, d_out, stream_grid_cap(d),
                                       as_stream(stream));
}
int b2_materialize_master(uint8_t *d_bytes, uint8_t *d_scales, float *d_global_scale, const float *d_master,
                          float *d_amax, float *d_chunk_amax, uint32_t len, uint32_t scale_layout, void *stream) {
    if (len % 16 != 0 || len > kMaxFlatElements) return B2_ERROR_INVALID_VALUE;
    int rc = b2_tensor_amax_f32(d_master, d_chunk_amax, d_amax, len, stream);
    if (rc) return rc;
    return b2_fp32_to_nvfp4_four_six(d_master, d_amax, d_bytes, d_scales, d_global_scale, len / 16, scale_layout, stream);
}

static int check_sf(const b2_schedule_free_materialize_args *a) {
    if (!a || !a->bytes || !a->scales || !a->global_scale || !a->z_master || !a->x_master || !a->amax)
        return B2_ERROR_INVALID_VALUE;
    if (a->len % 16 != 0 || a->len > kMaxFlatElements || a->scale_layout > B2_SCALES_RAW) return B2_ERROR_INVALID_VALUE;
    if (a->scale_layout == B2_SCALES_CSF && a->len % 128 != 0) return B2_ERROR_INVALID_VALUE;
    if ((uint64_t)a->scale_rows * a->scale_k < a->len) return B2_ERROR_INVALID_VALUE;
    if (!(a->symexp_lin_beta >= 0.0f)) return B2_ERROR_INVALID_VALUE;
    const bool any = a->symexp_lin_scales[0] != nullptr;
    for (int k = 0; k < 6; ++k)   // the six scale scalars come together or not at all
        if ((a->symexp_lin_scales[k] != nullptr) != any) return B2_ERROR_INVALID_VALUE;
    return B2_SUCCESS;
}
static SymExpLinParams symexp_params(const b2_schedule_free_materialize_args *a) {
    SymExpLinParams sp;
    sp.beta = a->symexp_lin_beta;
    for (int k = 0; k < 6; ++k) sp.scales[k] = a->symexp_lin_scales[k];
    return sp;
}
int b2_materialize_schedule_free_precomputed(const b2_schedule_free_materialize_args *a, void *stream) {
    int rc = check_sf(a);
    if (rc) return rc;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    if (a->precomputed_values)
        return (int)launch_quantize_flat(a->precomputed_values, nullptr, nullptr, 0.f, 0, a->amax, a->bytes, a->scales,
                                         a->global_scale, a->len / 16, (int)a->scale_layout, stream_grid_cap(d),
                                         as_stream(stream));
    const SymExpLinParams sp = symexp_params(a);
    return (int)launch_quantize_flat(nullptr, a->z_master, a->x_master, a->beta, 1, a->amax, a->bytes, a->scales,
                                     a->global_scale, a->len / 16, (int)a->scale_layout, stream_grid_cap(d),
                                     as_stream(stream), &sp);
}
int b2_materialize_schedule_free(const b2_schedule_free_materialize_args *a, void *stream) {
    int rc = check_sf(a);
    if (rc) return rc;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    cudaStream_t s = as_stream(stream);
    e = cudaMemsetAsync(a->amax, 0, sizeof(float), s);  // launcher/update.rs:14-23 (zero_amax)
    const SymExpLinParams sp = symexp_params(a);
    if (e == cudaSuccess)
        e = launch_schedule_free_amax(a->z_master, a->x_master, a->beta, a->len, a->amax, stream_grid_cap(d), s, &sp);
    if (e == cudaSuccess)
        e = launch_quantize_flat(nullptr, a->z_master, a->x_master, a->beta, 1, a->amax, a->bytes, a->scales,
                                 a->global_scale, a->len / 16, (int)a->scale_layout, stream_grid_cap(d), s, &sp);
    return (int)e;
}

static int check_adam(const b2_adamw_update_args *a, bool need_quant, bool need_amax) {
    if (!a || !a->z_master || !a->x_master || !a->grad || !a->first_moment || !a->second_moment)
        return B2_ERROR_INVALID_VALUE;
    if (a->len > kMaxFlatElements) return B2_ERROR_INVALID_VALUE;
    if (need_quant && (a->len % 16 != 0 || !a->bytes || !a->scales || !a->global_scale || !a->amax || !a->chunk_amax))
        return B2_ERROR_INVALID_VALUE;
    if (need_amax && (a->len % 16 != 0 || !a->amax)) return B2_ERROR_INVALID_VALUE;
    return B2_SUCCESS;
}
int b2_apply_fp32_adamw_update(const b2_adamw_update_args *a, void *stream) {
    int rc = check_adam(a, false, false);
    if (rc) return rc;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_adamw(*a, 0, stream_grid_cap(d), as_stream(stream));
}
int b2_apply_adamw_update(const b2_adamw_update_args *a, void *stream) {
    int rc = check_adam(a, true, false);
    if (rc) return rc;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    // The reference runs the update, then materialize_master (two amax kernels + encode).  Here
    // the update kernel raises max|x'| itself (atomicMax, order-independent, so the same value),
    // which saves the extra read of x'; `chunk_amax` is left untouched.
    cudaStream_t s = as_stream(stream);
    e = cudaMemsetAsync(a->amax, 0, sizeof(float), s);
    if (e == cudaSuccess) e = launch_adamw(*a, 2, stream_grid_cap(d), s);
    if (e != cudaSuccess) return (int)e;
    return b2_fp32_to_nvfp4_four_six(a->x_master, a->amax, a->bytes, a->scales, a->global_scale, a->len / 16,
                                     a->scale_layout, stream);
}
int b2_apply_adamw_update_deferred_quantization(const b2_adamw_update_args *a, void *stream) {
    int rc = check_adam(a, false, true);
    if (rc) return rc;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_adamw(*a, 1, stream_grid_cap(d), as_stream(stream));
}
int b2_adamw_table_prepare(b2_adamw_slot_descriptor *t, uint32_t count, uint32_t *total_chunks) {
    if ((!t && count) || !total_chunks) return B2_ERROR_INVALID_VALUE;
    uint64_t chunks = 0;
    for (uint32_t i = 0; i < count; ++i) {
        if (t[i].mode > 2 || t[i].scale_layout > B2_SCALES_RAW || t[i].len > kMaxFlatElements) return B2_ERROR_INVALID_VALUE;
        if (t[i].mode != 0 && (t[i].len % 16 != 0 || !t[i].amax)) return B2_ERROR_INVALID_VALUE;
        if (t[i].mode == 2 && (!t[i].bytes || !t[i].scales || !t[i].global_scale)) return B2_ERROR_INVALID_VALUE;
        if (t[i].mode == 2 && t[i].scale_layout == B2_SCALES_CSF && t[i].len % 128 != 0) return B2_ERROR_INVALID_VALUE;
        if (t[i].len && (!t[i].z_master || !t[i].x_master || !t[i].grad || !t[i].first_moment || !t[i].second_moment))
            return B2_ERROR_INVALID_VALUE;
        t[i].chunk_begin = (uint32_t)chunks;
        chunks += (t[i].len + kChunkHost - 1) / kChunkHost;
        if (chunks > 0xffffffffull) return B2_ERROR_INVALID_VALUE;
    }
    *total_chunks = (uint32_t)chunks;
    return B2_SUCCESS;
}
int b2_apply_adamw_update_multi(const b2_adamw_slot_descriptor *d_table, uint32_t count, uint32_t total_chunks,
                                const b2_adamw_update_args *scalars, void *stream) {
    if (!scalars || (!d_table && count)) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_adamw_multi(d_table, count, total_chunks, *scalars, stream_grid_cap(d), as_stream(stream));
}
int b2_adamw_materialize_training_weights(const b2_adamw_slot_descriptor *d_table, uint32_t count,
                                          uint32_t total_chunks, float schedule_beta, int values_cached,
                                          void *stream) {
    if (!d_table && count) return B2_ERROR_INVALID_VALUE;
    if (!std::isfinite(schedule_beta)) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_adamw_multi_materialize(d_table, count, total_chunks, schedule_beta, values_cached != 0,
                                               stream_grid_cap(d), as_stream(stream));
}
int b2_muon_materialize_training_weights(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, void *stream) {
    if (!plan || !d_slots) return B2_ERROR_INVALID_VALUE;
    SlotView v = plan->view(d_slots);
    return (int)launch_muon_encode(v, plan->at<float>(plan->layout.off_amax_x), 1, (int)plan->options.scale_layout,
                                   as_stream(stream));
}
int b2_symexp_lin_zero_scale_grads(const b2_symexp_lin_slot_descriptor *d_slots, uint32_t slot_count, void *stream) {
    if (!d_slots && slot_count) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_symexp_zero_scale_grads(d_slots, slot_count, as_stream(stream));
}
int b2_symexp_lin_scale_adamw_update(const b2_symexp_lin_slot_descriptor *d_slots, uint32_t slot_count,
                                     const b2_symexp_lin_adamw_args *args, void *stream) {
    if (!args || (!d_slots && slot_count)) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_symexp_scale_adamw(d_slots, slot_count, *args, as_stream(stream));
}
int b2_symexp_lin_congruent_inverse_in_place(float *d_raw, uint32_t len, float beta, void *stream) {
    if ((!d_raw && len) || !(beta > 0.0f) || !std::isfinite(beta)) return B2_ERROR_INVALID_VALUE;  // symexp_lin.rs:67
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_symexp_congruent_inverse(d_raw, len, beta, as_stream(stream));
}
int b2_clip_gradients(const b2_gradient_clip_args *a, void *stream) {
    if (!a || !a->scale || !a->norm) return B2_ERROR_INVALID_VALUE;
    if (a->chunk_count && (!a->chunk_ptrs || !a->chunk_lens || !a->chunk_sums)) return B2_ERROR_INVALID_VALUE;
    if (a->extra_sum_count && !a->extra_sums) return B2_ERROR_INVALID_VALUE;
    DeviceInfo d;
    cudaError_t e = device_info(d);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_grad_clip(*a, stream_grid_cap(d), as_stream(stream));
}
int b2_zero_f32_pointer_table(const uint64_t *d_pointers, uint32_t pointer_count, void *stream) {
    if (!d_pointers && pointer_count) return B2_ERROR_INVALID_VALUE;
    return (int)launch_zero_pointer_table(d_pointers, pointer_count, as_stream(stream));
}

int b2_debug_muon_fused_wait_expiry(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, uint32_t slot,
                                    uint64_t wait_ns, void *stream) {
    if (!plan || !d_slots || wait_ns == 0 || wait_ns > 1000000000ull) return B2_ERROR_INVALID_VALUE;
    const Layout &L = plan->layout;
    if (slot >= L.slots.size() || L.slots[slot].len == 0) return B2_ERROR_INVALID_VALUE;
    cudaStream_t s = as_stream(stream);
    // A one-item list: the encode span at the slot's first chunk, with none of the slot's update chunks in
    // the list, so the completion count it waits for is never reached.  The list borrows the first
    // word of the per-step partial sums (rewritten by the next prepare).
    const uint32_t item = 0x80000000u | L.chunk_prefix[slot];
    uint32_t *d_item = plan->at<uint32_t>(L.off_partials);
    cudaError_t e = cudaMemcpyAsync(d_item, &item, sizeof(item), cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(s);   // `item` lives on this frame
    if (e != cudaSuccess) return (int)e;
    SlotView v = plan->view(d_slots);
    b2_muon_step_args zero;
    std::memset(&zero, 0, sizeof(zero));
    const UpdateParams up = update_params(&zero);
    return (int)launch_muon_update_encode(v, d_item, 1u, plan->at<uint64_t>(L.off_u_ptrs), plan->at<float>(L.off_amax_x),
                                          up, 0, (int)plan->options.scale_layout, plan->ws + L.off_fused_sync,
                                          plan->at<uint32_t>(L.off_status), wait_ns, s);
}

int b2_debug_rcp_approx_ftz(const float *d_in, float *d_out, uint32_t count, void *stream) {
    if (!d_in || !d_out) return B2_ERROR_INVALID_VALUE;
    return (int)launch_debug_rcp(d_in, d_out, count, as_stream(stream));
}
int b2_debug_quantize_literal(const float *d_x, const float *d_amax, uint8_t *d_out_fp4, uint8_t *d_out_raw_scales,
                              float *d_out_global_scale, uint32_t group_count, void *stream) {
    if (!d_x || !d_amax || !d_out_fp4 || !d_out_raw_scales || !d_out_global_scale) return B2_ERROR_INVALID_VALUE;
    return (int)launch_debug_quantize_literal(d_x, d_amax, d_out_fp4, d_out_raw_scales, d_out_global_scale, group_count,
                                              as_stream(stream));
}

}  // extern "C"
