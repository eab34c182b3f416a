// Host-side prototypes shared by the translation units of libllmini_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/llmini_b200.h"

namespace b2 {

// ---- multi-slot streaming stages (stream_kernels.cu) --------------------------------------
struct SlotView {
    const b2_muon_slot_descriptor *slots;  // device
    const uint32_t *chunk_prefix;          // device, slot_count + 1 entries
    uint32_t slot_count;
    uint32_t total_chunks;
    int grid;                              // CTAs to launch (multiple of the SM count)
};

struct MomentumParams {
    float mu, grad_scale;
    const float *d_grad_scale;
    int nesterov, variance_adaptive;
    float bias_correction_inv;
};
#define B2_NORMUON_ROWS_PER_UNIT 32
// NorMuon / Hyperball scratch of a plan: work units are B2_NORMUON_ROWS_PER_UNIT rows (slots with rows >= cols) or 128
// columns (rows < cols) of one slot; `unit_prefix` counts them like `chunk_prefix` counts chunks.
struct NeuronView {
    const uint32_t *unit_prefix;   // device, slot_count + 1 entries
    uint32_t total_units;
    const uint64_t *factor_ptrs;   // device, per slot: f32[max(rows, cols)] factors
    double *partials;              // device, 4 per unit: raw, scaled, parameter, dot
    float *slot_stats;             // device, 4 per slot: normuon_scale, update_norm, radius, dot
};
struct UpdateParams {
    float lr, wd, c_avg, beta;
    const float *d_qk_clip_factors;
    int normuon;                   // 1: scale U by factor[neuron] * normuon_scale
    const uint64_t *factor_ptrs;
    const float *slot_stats;
    int update_format;             // how `u_ptrs` buffers hold the Newton-Schulz result: 0 f32, 1 bf16, 2 f16
    float symexp_beta;             // > 0: SymExpLin forward on y, scales from the slot table (or unit)
    const b2_symexp_lin_slot_descriptor *symexp_slots;
};
cudaError_t launch_muon_sumsq(const SlotView &v, const MomentumParams &mp, double *partials, float *amax_x,
                              cudaStream_t s);
// One-pass form of stages M+N: momentum state, un-normalised BF16 operand and the chunk sums in one launch.
cudaError_t launch_muon_momentum_sumsq(const SlotView &v, const MomentumParams &mp, const uint64_t *x0_ptrs,
                                       double *partials, float *amax_x, cudaStream_t s);
// `partials_per_chunk`: 1 after launch_muon_sumsq, B2_ONE_PASS_PARTIALS after launch_muon_momentum_sumsq.
#define B2_ONE_PASS_PARTIALS 8
cudaError_t launch_muon_inv_norm(const SlotView &v, const double *partials, float *inv_norm,
                                 uint32_t partials_per_chunk, cudaStream_t s);
cudaError_t launch_muon_momentum_normalize(const SlotView &v, const MomentumParams &mp, const float *inv_norm,
                                           const uint64_t *x0_ptrs, int f16, cudaStream_t s);
cudaError_t launch_muon_update(const SlotView &v, const uint64_t *u_ptrs, float *amax_x, const UpdateParams &up,
                               cudaStream_t s);
// Stages U and Q in one launch over an item list (bit 31: encode span of B2_FUSED_ENCODE_SPAN chunks, else update
// chunk; low bits: flat chunk index).  `sync` is fused_sync_bytes(slot_count) of device scratch,
// zeroed once by the owner; every launch leaves it zeroed again.  `wait_ns` bounds an encode span's wait for
// its matrix's update chunks; when it runs out the launch sets *status and returns.
#define B2_FUSED_ENCODE_SPAN 4
size_t fused_sync_bytes(uint32_t slot_count);
cudaError_t launch_muon_update_encode(const SlotView &v, const uint32_t *items, uint32_t item_count,
                                      const uint64_t *u_ptrs, float *amax_x, const UpdateParams &up, int quantize_y,
                                      int scale_layout, void *sync, uint32_t *status, uint64_t wait_ns,
                                      cudaStream_t s);
cudaError_t launch_normuon_stats(const SlotView &v, const NeuronView &nv, const uint64_t *u_ptrs, int hyperball,
                                 cudaStream_t s);
cudaError_t launch_muon_hyperball_update(const SlotView &v, const uint64_t *u_ptrs, float *amax_x,
                                         const UpdateParams &up, int use_schedule_free, cudaStream_t s);
cudaError_t launch_muon_sign_update(const SlotView &v, const MomentumParams &mp, const UpdateParams &up,
                                    float *amax_x, cudaStream_t s);
cudaError_t launch_muon_encode(const SlotView &v, const float *amax_x, int quantize_y,
                               int scale_layout, cudaStream_t s);

// ---- single-tensor kernels (stream_kernels.cu) ---------------------------------------------
cudaError_t launch_tensor_chunk_amax(const float *x, float *chunk_amax, uint32_t n, cudaStream_t s);
cudaError_t launch_tensor_amax_from_chunks(const float *chunk_amax, float *out, uint32_t count,
                                           cudaStream_t s);
// SymExpLin forward of the schedule values: beta <= 0 is the identity; scale pointers as in
// b2_schedule_free_materialize_args (all NULL = unit scales).
struct SymExpLinParams {
    float beta;
    const float *scales[6];
};
cudaError_t launch_quantize_flat(const float *x, const float *z, const float *xm, float beta,
                                 int mode, const float *amax, uint8_t *fp4, uint8_t *scales,
                                 float *gs, uint32_t group_count, int scale_layout, int grid_cap,
                                 cudaStream_t s, const SymExpLinParams *symexp = nullptr);
cudaError_t launch_schedule_free_amax(const float *z, const float *x, float beta, uint32_t len,
                                      float *amax, int grid_cap, cudaStream_t s,
                                      const SymExpLinParams *symexp = nullptr);
cudaError_t launch_adamw(const b2_adamw_update_args &a, int mode, int grid_cap,
                         cudaStream_t s);
cudaError_t launch_adamw_multi(const b2_adamw_slot_descriptor *table, uint32_t count, uint32_t total_chunks,
                              const b2_adamw_update_args &scalars, int grid_cap, cudaStream_t s);
cudaError_t launch_adamw_multi_materialize(const b2_adamw_slot_descriptor *table, uint32_t count,
                                          uint32_t total_chunks, float beta, bool cached, int grid_cap,
                                          cudaStream_t s);
cudaError_t launch_grad_clip(const b2_gradient_clip_args &a, int grid_cap, cudaStream_t s);
cudaError_t launch_scales_to_sm100(const uint8_t *src, int src_csf, uint32_t rows, uint32_t cols, uint8_t *out,
                                   int grid_cap, cudaStream_t s);
cudaError_t launch_symexp_scale_adamw(const b2_symexp_lin_slot_descriptor *slots, uint32_t n,
                                      const b2_symexp_lin_adamw_args &a, cudaStream_t s);
cudaError_t launch_symexp_zero_scale_grads(const b2_symexp_lin_slot_descriptor *slots, uint32_t n, cudaStream_t s);
cudaError_t launch_symexp_congruent_inverse(float *raw, uint32_t len, float beta, cudaStream_t s);
cudaError_t launch_zero_pointer_table(const uint64_t *ptrs, uint32_t n, cudaStream_t s);
cudaError_t launch_layout_echo(uint32_t *out, cudaStream_t s);
cudaError_t launch_debug_rcp(const float *in, float *out, uint32_t n, cudaStream_t s);
cudaError_t launch_debug_quantize_literal(const float *x, const float *amax, uint8_t *fp4,
                                          uint8_t *raw_scales, float *gs, uint32_t group_count,
                                          cudaStream_t s);

// ---- Newton-Schulz GEMMs (ns_gemm_sm100.cu) --------------------------------------------------
enum GemmEpilogue : uint32_t {
    kEpiGram = 0,   // out16 = r16(acc), frag32 = acc
    kEpiPoly = 1,   // out16 = r16(fma(c, acc, fma(b, frag32, a * delta_ij)))
    kEpiApply = 2,  // out16 = r16(acc)
    kEpiApplyLast = 3,  // out32 = acc (f32, storage layout)
    // Work-list entries of the ticketed launch only.  kEpiGramPoly: the CTA (pair) computes the Gram tile, keeps its
    // FP32 accumulator in tensor memory, waits until every Gram tile of the matrix has been stored, computes the
    // polynomial tile of the same position into the other accumulator buffer and combines the two in registers,
    // so the FP32 Gram tile never leaves the SM.  The kernel runs it as the two parts below.
    kEpiGramPoly = 4,
    kEpiGramHold = 5,   // out16 = r16(acc); the accumulator buffer stays occupied
    kEpiPolyFused = 6,  // out16 = r16(fma(c, acc, fma(b, held Gram accumulator, a * delta_ij))); frees both buffers
};

// One GEMM of one slot: D[M][N] = A * B^T with A, B described by TMA maps.  Lives in device
// memory; built once per plan.
struct alignas(16) GemmProblem {
    uint64_t map_a;      // device address of the CUtensorMap of operand A (16-bit; box 64 x 128
                         // rows when K-major, 64 x 64 when MN-major)
    uint64_t map_b;
    uint64_t out16;      // 16-bit result, row-major with `pitch16` elements per row — unused for kEpiApplyLast
    uint64_t out32;      // f32 result, row-major with `pitch32` elements per row — kEpiApplyLast only
    uint64_t frag32;     // f32 accumulator tiles in fragment order (Gram writes, Poly reads)
    uint32_t M, N, K;
    uint32_t a_mn_major;  // 0: A is [M][K] K-contiguous; 1: A is [K][M] M-contiguous
    uint32_t b_mn_major;  // 0: B is [N][K]; 1: B is [K][N]
    uint32_t tiles_n;     // number of BN-wide tile columns (for frag32 addressing)
    uint32_t pitch16;     // >= N, a multiple of 8 (columns N .. pitch16 of a row are padding and may be written)
    uint32_t pitch32;
};
struct GemmTile {
    uint16_t problem;
    uint16_t tile_m;
    uint16_t tile_n;
    uint16_t reserved;   // 1: also store the transposed tile (symmetric output, tile above the diagonal)
};

constexpr int kGemmBlockM = 128;
constexpr int kGemmBlockK = 64;

// Polynomial coefficients (a, b, c) per Newton-Schulz iteration, passed by value to the kernel.
constexpr uint32_t kMaxChainIterations = 8;
struct GemmCoefficients {
    float v[3 * kMaxChainIterations];
};
// One entry of the work list of the chained launch, which runs every GEMM of every iteration of the plan's
// matrices as ONE grid: `need` is the value the matrix's progress count (epilogue warps that have finished a
// tile of the matrix, over all earlier phases) must have reached before this tile's operands are read.  A
// matrix's phases follow one another strictly (Gram -> Poly -> Apply -> next Gram), so one count per matrix
// orders every read after the writes it depends on, and every overwrite after the reads of the old contents.
struct alignas(16) ChainTile {
    uint32_t problem;      // index into the plan's GemmProblem array (type * slot_count + slot)
    uint16_t tile_m, tile_n;
    uint16_t slot;
    uint8_t epilogue;      // GemmEpilogue
    uint8_t flags;         // bit 0: also store the transposed tile; bits 1-2: power of the slot scale applied to
                           // the accumulator (one-pass prepare); bits 3-7: iteration (coefficient triple)
    uint32_t need;
    // kEpiGramPoly only: the polynomial GEMM of the tile and the progress count at which every Gram tile of the
    // matrix has been stored (need + epilogue warps x Gram tiles of the matrix)
    uint32_t problem2;
    uint32_t need2;
    uint32_t reserved[2];
};
static_assert(sizeof(ChainTile) == 32, "ChainTile is read as two 16-byte words");

cudaError_t gemm_configure(int block_n, int pair);
// CTAs (pairs of CTAs when `pair`) of the ticketed kernel that the device runs at the same time, 0 if unknown.
// Call after gemm_configure.
int gemm_resident_groups(int block_n, int pair, int sm_count);
// `slot_scale` (may be null): per-slot scalars s; the Gram epilogue multiplies the accumulator by s^scale_pow
// (scale_pow = 2) and the Apply epilogues by s (scale_pow = 1).  Used by the first iteration after a
// one-pass prepare, whose operand is not normalised yet.
cudaError_t launch_ns_gemm(int block_n, int pair, const GemmProblem *problems, const GemmTile *tiles,
                           uint32_t tile_count, uint32_t epilogue, int f16, float ca, float cb,
                           float cc, const float *slot_scale, uint32_t scale_pow, uint32_t *status,
                           uint32_t debug_flags, int grid, cudaStream_t s);

// The ticketed launch over a ChainTile list.  `fused_list`: the list holds kEpiGramPoly entries, whose second part
// waits for tiles with LARGER tickets of the same matrix; a CTA then never holds a ticket it has not started
// while it waits, every matrix's entries must be contiguous in the list, and no matrix may have more Gram tiles
// than the launch has CTAs (pairs).  `sync` is chain_sync_bytes(slot_count) of device memory, zeroed once by
// the owner; every launch leaves it zeroed.  chain_epilogue_warps: progress-count increments per finished tile.
size_t chain_sync_bytes(uint32_t slot_count);
uint32_t chain_epilogue_warps(int block_n, int pair);
cudaError_t launch_ns_chain(int block_n, int pair, const GemmProblem *problems, const ChainTile *tiles,
                            uint32_t tile_count, int f16, const GemmCoefficients &coef, const float *slot_scale,
                            uint32_t *status, void *sync, uint32_t slot_count, uint32_t debug_flags, int grid,
                            cudaStream_t s, bool fused_list = false);

}  // namespace b2
