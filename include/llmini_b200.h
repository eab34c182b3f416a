/*
 * llmini_b200 — C ABI of the B200 (sm_100a) implementation of llmini's AMUSE/Muon matrix
 * update + NVFP4 requantisation path.
 *
 * Every entry point replaces one method of the reference's Rust kernel host API
 * (`OptimizerModule`, `Nvfp4QuantModule`) or one host helper beside it; the reference
 * file:line is cited per declaration (paths relative to the reference repository root).
 *
 * Conventions
 *  - Return value: int, 0 on success, otherwise a CUDA error code (the numeric values of
 *    cudaError_t and CUresult coincide; precondition violations return 1 =
 *    CUDA_ERROR_INVALID_VALUE where the reference panics with `assert!`).
 *  - `stream` is a `cudaStream_t` / `CUstream` passed as `void*`; all work is enqueued on
 *    it in program order and nothing synchronises unless stated.
 *  - All pointers named `d_*` or typed as device buffers are device pointers owned by the
 *    caller.  No compute call allocates device memory: scratch comes from the caller-sized
 *    workspace (`b2_muon_workspace_bytes`).  (`b2_peer_buffer_alloc` allocates, because that is what it is asked
 *    for: a buffer other processes can map.)
 *  - No CPU fallback exists.  Without a CUDA device every compute entry point returns an
 *    error.
 *  - Sizes: a tensor has at most 0xfffff000 elements (elements and 2048-value chunks are indexed in
 *    32 bits) and a matrix at most 65535 * 128 rows or columns; larger arguments are refused with
 *    B2_ERROR_INVALID_VALUE.
 */
#ifndef LLMINI_B200_H
#define LLMINI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_ABI_VERSION 2u
/* crates/cuda-kernels/src/gpt/optimizer/storage.rs:4 (MUON_STORAGE_LAYOUT_VERSION) */
#define B2_MUON_STORAGE_LAYOUT_VERSION 1u

#define B2_SUCCESS 0
#define B2_ERROR_INVALID_VALUE 1
#define B2_ERROR_NOT_SUPPORTED 801
#define B2_ERROR_LAUNCH_TIMEOUT 702 /* a bounded device-side wait ran out */
#define B2_ERROR_NO_DEVICE 100

/* Per-matrix pointer table entry.  Same field order, sizes and 104-byte stride as
 * `MuonSlotDescriptor` (crates/cuda-kernels/src/gpt/optimizer/args/muon.rs:3-21), so the
 * reference's device-resident slot table can be passed through unchanged. */
typedef struct b2_muon_slot_descriptor {
    uint64_t grad;            /* f32 [rows][cols]; overwritten with y = z' + beta (x' - z') */
    uint64_t momentum;        /* bf16 [rows][cols] */
    uint64_t variance;        /* bf16 [rows][cols]; read and written only with variance_adaptive */
    uint64_t second_momentum; /* f32 [max(rows, cols)]: NorMuon per-neuron second moment; read and written
                                 only with b2_muon_step_args.normuon or the Hyperball finish */
    uint64_t z_master;        /* f32 */
    uint64_t x_master;        /* f32 */
    uint64_t schedule_amax;   /* f32[1]: max |y| */
    uint64_t bytes;           /* u8 [len/2] packed E2M1 codes */
    uint64_t scales;          /* u8: CSF block-scale storage with its 128-byte header
                                 pre-filled, or a raw [len/16] plane (b2_muon_options) */
    uint64_t global_scale;    /* f32[1] */
    uint32_t rows;
    uint32_t cols;
    float learning_rate_multiplier;
    uint32_t qk_clip_factor_offset; /* UINT32_MAX = no qk-clip; else index of this slot's first head
                                       in b2_muon_step_args.d_qk_clip_factors */
    uint32_t qk_clip_head_dim;
    uint32_t reserved_padding;
} b2_muon_slot_descriptor;

/* Same field order and 152-byte stride as `SymExpLinSlotDescriptor`
 * (crates/cuda-kernels/src/gpt/optimizer/args/symexp_lin.rs:5-26).  Only the six scale scalars
 * (f32[1] each, as schedule-free z / x pairs) are read on this path. */
typedef struct b2_symexp_lin_slot_descriptor {
    uint64_t grad, z_master, x_master;
    uint64_t exponential_z, exponential_x, exponential_grad, exponential_first, exponential_second;
    uint64_t linear_z, linear_x, linear_grad, linear_first, linear_second;
    uint64_t curvature_z, curvature_x, curvature_grad, curvature_first, curvature_second;
    uint32_t rows, cols;
} b2_symexp_lin_slot_descriptor;

enum { B2_OPERAND_BF16 = 0, B2_OPERAND_F16 = 1 };
enum { B2_SCALES_CSF = 0, B2_SCALES_RAW = 1,
       B2_SCALES_SM100 = 2 /* the block-scale operand layout of sm_100a's `tcgen05.mma
                              kind::mxf4nvf4.block_scale` (what cuBLASLt calls VEC16_UE4M3): 512-byte
                              tiles of 128 rows x 4 scale columns, tile (row/128, kblock/4) row-major,
                              byte (row%32)*16 + (row%128)/32*4 + kblock%4 inside a tile; rows padded
                              to 128 and scale columns to 4 (padding bytes are never written: zero the
                              buffer once).  Accepted by the Muon plan only */ };
enum { B2_QUANTIZE_X = 0, B2_QUANTIZE_Y = 1 };
/* Where the Frobenius normalisation of stage N is applied.
 * B2_NORMALIZE_TWO_PASS: X0 = r16(u * s), the reference's rounding point
 *   (crates/cuda-kernels/src/gpt/optimizer/muon/polar/fused/normalize.rs:91-145); the gradients are read twice.
 * B2_NORMALIZE_DEFERRED: one pass over the gradients writes X0 = r16(u); s enters through the first
 *   Newton-Schulz iteration, which is linear in it (G = s^2 X0 X0^T, X1 = s Q X0).  Same algebra, the operand
 *   is rounded before instead of after the scaling; BF16 operands only. */
enum { B2_NORMALIZE_TWO_PASS = 0, B2_NORMALIZE_DEFERRED = 1 };
/* How the Newton-Schulz loop is launched.
 * B2_NS_PER_PHASE: three launches per iteration (Gram, polynomial, apply), each over all matrices, chained with
 *   programmatic dependent launch.
 * B2_NS_CHAINED: every GEMM of every iteration of every matrix as ONE persistent grid (the reference runs its loop
 *   inside one cooperative kernel with grid-wide barriers, .../muon/polar/fused.rs:64-92).  CTAs claim tiles
 *   from one work list with an atomic ticket; a matrix's Gram, polynomial and apply tiles are ordered by a
 *   progress count of that matrix instead of launch boundaries, so phases of different matrices overlap.  Used
 *   when a step runs exactly `max_iterations` iterations (at most 8); other steps take the per-phase form.
 *   Bit-identical results; measured equal to the per-phase form on one GPU and slower when a rank owns few
 *   matrices, so it is not the default.
 * B2_NS_FUSED_GRAM_POLY: two launches per iteration.  In the first, the CTA (pair) that computes a Gram tile keeps
 *   its FP32 accumulator in tensor memory, stores the 16-bit tile, waits (bounded) until the matrix's other Gram
 *   tiles are stored, computes the polynomial tile of the same position into the second accumulator buffer and
 *   combines the two in registers: the FP32 Gram tile never goes through memory.  Tiles are drawn with an atomic
 *   ticket as in the chained form.  Needs every Gram tile of a matrix in flight at once, so a plan with a matrix
 *   of more Gram tiles than the GPU has CTA slots (pairs: SMs / 2) takes the per-phase form.  Bit-identical
 *   results. */
enum { B2_NS_PER_PHASE = 0, B2_NS_CHAINED = 1, B2_NS_FUSED_GRAM_POLY = 2 };
/* Precision in which the Newton-Schulz result reaches stage U.
 * B2_UPDATE_F32: the last Apply GEMM stores FP32 (the reference's `polar_update` is f32:
 *   crates/cuda-kernels/src/gpt/optimizer/muon/fused/update/one.rs:46-85).
 * B2_UPDATE_16BIT: it stores the operand type (BF16 or F16) like the other iterations, and stage U reads that:
 *   two bytes per element less to write and to read (18.56 instead of 20.56 bytes per element in the
 *   update + quantise pass, before the schedule cache).  The update direction carries one more 16-bit rounding.
 *   Plain finish entry points only (b2_muon_finish_update[_deferred_quantization], b2_muon_mega_update): steps
 *   with NorMuon scaling or the Hyperball finish, whose statistics read the FP32 result, are refused with
 *   B2_ERROR_NOT_SUPPORTED. */
enum { B2_UPDATE_F32 = 0, B2_UPDATE_16BIT = 1 };

typedef struct b2_muon_options {
    uint32_t operand_format;  /* B2_OPERAND_*: 16-bit type the Newton-Schulz GEMM operands are
                                 rounded to (the reference rounds to F16:
                                 .../muon/polar/fused/stage.rs:51-55) */
    uint32_t scale_layout;    /* B2_SCALES_* */
    uint32_t quantize_target; /* B2_QUANTIZE_X: the averaged weights x' (mega path,
                                 .../muon/fused/body.rs:90-101); B2_QUANTIZE_Y: the
                                 schedule-free training weights y */
    uint32_t max_iterations;  /* upper bound on b2_muon_step_args.iterations (0 -> 5) */
    uint32_t tile_override;   /* GEMM tile shape: 0 = choose; 128 / 256 = one CTA per 128 x N tile;
                                 512 = two-CTA 256 x 256 tiles */
    uint32_t measure_phase_mask; /* leave 0.  Read only by a library built with -DB2_MEASURE: which GEMMs of an */
    uint32_t measure_flags;      /* iteration run, and kernel variants used to attribute time */
    uint32_t normalize_mode;  /* B2_NORMALIZE_* */
    uint32_t ns_schedule;     /* B2_NS_* */
    uint32_t update_input;    /* B2_UPDATE_* */
    uint32_t reserved[2];     /* must be 0 */
} b2_muon_options;

/* Step scalars: `MuonMegaUpdateArgs` (.../optimizer/args/muon.rs:25-44) and
 * `MuonUpdateScalars` (.../muon/fused/types.rs:55-63). */
typedef struct b2_muon_step_args {
    float mu;
    float grad_scale;
    float learning_rate;
    float weight_decay;
    float average_coefficient;
    float schedule_beta;        /* the mega kernel passes 1.0 (.../muon/fused/body.rs:82) */
    uint32_t iterations;
    uint32_t nesterov;          /* the mega kernel passes true (.../muon/fused/body.rs:34) */
    const float *coefficients;  /* host pointer, iterations x (a, b, c); NULL selects the
                                   reference table (.../muon/polar/fused/coefficients.rs:9-42) */
    const float *d_grad_scale;  /* optional DEVICE pointer to the clip scale written by
                                   b2_clip_gradients; when non-NULL it replaces `grad_scale`, so
                                   the step needs no host read-back of the gradient norm */
    uint32_t variance_adaptive; /* Muon-VS (.../muon/fused/momentum.rs:72-158): slots carry a bf16
                                   `variance` buffer; `MuonTmaPrepareArgs::variance_adaptive` */
    float bias_correction_inv;  /* `MuonTmaPrepareArgs::bias_correction_inv`; used with Muon-VS */
    const float *d_qk_clip_factors; /* optional DEVICE table of per-head factors (`qk_clip_factors` of
                                   `MuonTmaFinishArgs`): slots whose qk_clip_factor_offset is not
                                   UINT32_MAX scale z', x', momentum (and variance) of their query/key
                                   rows (row < 2*cols, head = (row % cols) / qk_clip_head_dim) */
    float symexp_lin_beta;      /* > 0: y = SymExpLin(z' + beta (x' - z')) (.../optimizer/symexp_lin.rs:8-26) in
                                   the finish, Hyperball and sign entry points; 0 = identity */
    const struct b2_symexp_lin_slot_descriptor *d_symexp_lin_slots; /* DEVICE table, one entry per slot
                                   (`symexp_lin_slots` of MuonTmaFinishArgs); NULL or an entry whose
                                   exponential_z is 0 means unit scales */
    uint32_t normuon;           /* 1: the finish stage first updates every slot's `second_momentum`
                                   (beta2 0.95) from the orthogonalised update and scales each neuron by
                                   1/sqrt(second moment), renormalised to the update's Frobenius norm
                                   (`muon_tma_normuon`, .../launcher/muon_mega.rs:283-325; the reference's
                                   split finish always does, its mega kernel never) */
    uint32_t reserved_padding;
} b2_muon_step_args;

typedef struct b2_muon_plan b2_muon_plan;

/* ---- handshake ------------------------------------------------------------------- */
uint32_t b2_abi_version(void);
const char *b2_error_string(int code);
/* `OptimizerModule::verify_storage_layout` (.../optimizer/launcher/mod.rs:43-56): a device
 * kernel echoes the layout version and sizeof(b2_muon_slot_descriptor); synchronises. */
int b2_verify_storage_layout(void *stream);

/* ---- Muon matrix step ------------------------------------------------------------- */
/* Scratch sizing replaces the reference's pre-sized buffers
 * (src/training/optimizer_tc_scratch.rs:43-66). */
size_t b2_muon_workspace_bytes(const uint32_t *rows, const uint32_t *cols, uint32_t slot_count,
                               const b2_muon_options *options);
/* Builds the tile lists and TMA descriptors for a fixed set of matrix shapes and uploads
 * them into `d_workspace` (enqueued on `stream`; the plan must outlive queued work). */
int b2_muon_plan_create(b2_muon_plan **plan, const uint32_t *rows, const uint32_t *cols,
                        uint32_t slot_count, const b2_muon_options *options, void *d_workspace,
                        size_t workspace_bytes, void *stream);
void b2_muon_plan_destroy(b2_muon_plan *plan);

/* `OptimizerModule::muon_mega_update` (.../optimizer/launcher/muon_mega.rs:24-51; device
 * body .../muon/fused/body.rs:14-102): momentum -> normalise -> Newton-Schulz -> update ->
 * NVFP4 requantisation for every slot with rows*cols > 0. */
int b2_muon_mega_update(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                        const b2_muon_step_args *args, void *stream);
/* The three stages on their own.  `b2_muon_prepare_polar`:
 * `OptimizerModule::muon_tma_prepare_polar` (.../launcher/muon_mega.rs:53-115) without the
 * variance-adaptive branch.  `b2_muon_polar`: the Newton-Schulz loop
 * (.../muon/polar/fused.rs:64-92).  `b2_muon_finish_update[_deferred_quantization]`:
 * `OptimizerModule::muon_tma_finish_update[_deferred_quantization]`
 * (.../launcher/muon_mega.rs:139-165) without NorMuon / qk-clip / SymExpLin. */
int b2_muon_prepare_polar(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                          const b2_muon_step_args *args, void *stream);
int b2_muon_polar(b2_muon_plan *plan, const b2_muon_step_args *args, void *stream);
int b2_muon_finish_update(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                          const b2_muon_step_args *args, void *stream);
int b2_muon_finish_update_deferred_quantization(b2_muon_plan *plan,
                                                const b2_muon_slot_descriptor *d_slots,
                                                const b2_muon_step_args *args, void *stream);
/* Finish groups: the plan's slots cut into `group_count` contiguous runs, run g starting at slot first_slot[g]
 * (first_slot[0] = 0, ascending; a run may be empty), so that stage U + Q can be launched run by run and whatever
 * consumes a run's packed weights (the all-gather of a multi-GPU step) can start while the next run is updated.
 * `b2_muon_plan_set_finish_groups` rebuilds the work list of the fused update + encode launch accordingly and
 * uploads it on `stream` (call it once after plan creation, with no finish launch of the plan in flight; a new
 * plan has one group).  `b2_muon_finish_update_group` is `b2_muon_finish_update` for the slots of one group:
 * plain steps only (no NorMuon / qk-clip / SymExpLin; B2_ERROR_NOT_SUPPORTED otherwise), an empty group is a
 * no-op.  `b2_muon_finish_update` still runs all groups in one launch.  No counterpart in the reference, whose
 * finish works per slot (.../launcher/muon_mega.rs:139-165). */
int b2_muon_plan_set_finish_groups(b2_muon_plan *plan, const uint32_t *first_slot, uint32_t group_count,
                                   void *stream);
int b2_muon_finish_update_group(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                                const b2_muon_step_args *args, uint32_t group, void *stream);
/* `OptimizerModule::muon_tma_finish_hyperball_update_deferred_quantization`
 * (.../launcher/muon_mega.rs:166-228): NorMuon factors, then a step of relative size
 * learning_rate along the update followed by projection back onto the sphere of the matrix's
 * Frobenius radius; x' averages towards z' when use_schedule_free, else x' = z'.  No weight decay. */
int b2_muon_finish_hyperball_update_deferred_quantization(b2_muon_plan *plan,
                                                          const b2_muon_slot_descriptor *d_slots,
                                                          const b2_muon_step_args *args,
                                                          uint32_t use_schedule_free, void *stream);
/* `OptimizerModule::muon_tma_sign_update_deferred_quantization` (.../launcher/muon_mega.rs:229-283;
 * device code .../muon/fused/update/one.rs:88-167) for every slot of the plan: momentum (and
 * variance) update, z' = z (1 - lr wd) - lr sign(m'), x', y into the gradient buffer, both amax
 * words.  No Newton-Schulz, no quantisation. */
int b2_muon_sign_update_deferred_quantization(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots,
                                              const b2_muon_step_args *args, void *stream);
/* Scratch views for tests and tracing (the reference's `MUON_TMA_TRACE`,
 * src/training/optimizer_muon/tma.rs:1210-1276).  which: 0 = X0 (16-bit, [rows][cols]),
 * 1 = Newton-Schulz result U (f32, [rows][cols]; with B2_UPDATE_16BIT the result is in the operand buffer 0 or 7
 * that the last iteration wrote: 7 for an odd iteration count, 0 for an even one), 2 = inverse norm (f32[1]),
 * 3 = max|x'| (f32[1]), 4 = device status word (u32[1], plan-wide).
 * 5 = Gram (16-bit, [n][ld]) and 6 = polynomial Q (16-bit, [n][ld]) of the LAST iteration,
 * 7 = the second operand buffer X1, 8 = NorMuon factors (f32[max(rows, cols)]),
 * 9 = NorMuon / Hyperball slot scalars (f32[4]: normuon_scale, update_norm, radius, dot),
 * 10 = the ticket, abort and completion words of the one-launch update + encode (u32[4 + slots], plan-wide;
 * all zero between launches), 11 = the abort, exit and per-matrix progress words of the chained Newton-Schulz
 * launch (u32[4 + slots], plan-wide; all zero between launches). */
int b2_muon_plan_scratch(b2_muon_plan *plan, uint32_t slot, uint32_t which, void **d_ptr,
                         size_t *bytes);
/* Reads back and clears the plan's device status word (synchronises `stream`): 0 when no
 * bounded wait ran out, else B2_ERROR_LAUNCH_TIMEOUT. */
int b2_muon_plan_status(b2_muon_plan *plan, void *stream);
/* Algorithmic FLOPs of one Newton-Schulz iteration over all slots: sum of 4 n^2 m + 2 n^3. */
double b2_muon_plan_flops_per_iteration(const b2_muon_plan *plan);

/* ---- NVFP4 quantiser (Nvfp4QuantModule) -------------------------------------------- */
/* `Nvfp4QuantModule::tensor_amax_f32` (crates/cuda-kernels/src/utils/nvfp4/quant/amax.rs:19-23;
 * kernels .../quant/kernels/row_amax.rs:92-136).  chunk_amax needs ceil(n/2048) floats. */
int b2_tensor_amax_f32(const float *d_x, float *d_chunk_amax, float *d_out, uint32_t element_count,
                       void *stream);
/* `Nvfp4QuantModule::tensor_amax_from_chunks_f32` (.../quant/amax.rs:25-39). */
int b2_tensor_amax_from_chunks_f32(const float *d_chunk_amax, float *d_out, uint32_t chunk_count,
                                   void *stream);
/* `Nvfp4QuantModule::fp32_to_nvfp4_four_six` (.../quant/four_six.rs:19-30; kernel
 * .../quant/kernels/four_six.rs:104-152,1838-1901, flat layout).  `d_out_scales` is CSF
 * storage whose header the caller has filled (b2_csf_encode_host of zeros does that), or a
 * raw plane when scale_layout == B2_SCALES_RAW. */
int b2_fp32_to_nvfp4_four_six(const float *d_x, const float *d_amax, uint8_t *d_out_fp4,
                              uint8_t *d_out_scales, float *d_out_global_scale,
                              uint32_t group_count, uint32_t scale_layout, void *stream);

/* ---- materialisation + AdamW (OptimizerModule) ------------------------------------- */
/* No single counterpart in the reference, whose forward GEMMs run on sm_120a and repack scales with
 * crates/cuda-kernels/src/utils/nvfp4_tma_matmul/scale_pack.rs:29-175: size of, and conversion into,
 * the B2_SCALES_SM100 layout from a raw plane or CSF storage of a [rows][cols] tensor (cols % 16 == 0;
 * CSF: cols % 128 == 0).  The converter writes every byte of the destination, padding as zero. */
size_t b2_nvfp4_sm100_scales_bytes(uint32_t rows, uint32_t cols);
int b2_nvfp4_scales_to_sm100(const uint8_t *d_scales, uint32_t src_layout, uint32_t rows, uint32_t cols,
                             uint8_t *d_out, void *stream);
/* `OptimizerModule::materialize_master` (.../optimizer/launcher/mod.rs:67-95): tensor maximum (two
 * kernels over `d_chunk_amax`, ceil(len/2048) floats) and the four-six quantiser.  len % 16 == 0. */
int b2_materialize_master(uint8_t *d_bytes, uint8_t *d_scales, float *d_global_scale,
                          const float *d_master, float *d_amax, float *d_chunk_amax, uint32_t len,
                          uint32_t scale_layout, void *stream);

/* No counterpart in the reference.  Same result as b2_materialize_master, for callers that
 * cannot supply the two scratch buffers and cannot allocate them either: code that receives only
 * the master tensor and the NVFP4 destination (an export or evaluation hook beside the trainer,
 * an embedder whose device memory is fully reserved before the first step), where cudaMalloc
 * would fail or would stall the training stream by synchronising the device.  The scratch is an
 * array built into the library (about 128 KiB on every GPU the library's module is loaded on, until exit), which
 * limits one call to B2_STATIC_MAX_ELEMENTS values; longer tensors are refused with
 * B2_ERROR_INVALID_VALUE.  The call allocates nothing.  The first call on each device looks up the
 * array's device address and should therefore be made outside any stream capture.  That first call is
 * also the moment the CUDA runtime loads the library's module onto the device (modules load lazily by
 * default), which is when the driver sets the array's 128 KiB aside: a process that is about to reserve
 * all device memory should make one warm-up call (len = 0 is enough) at start-up, before that
 * reservation, or the first real call can fail with an out-of-memory error.  From the second call on a
 * device nothing is looked up, loaded or reserved.  The looked-up address is kept for the life of the
 * process; after cudaDeviceReset it is stale.  All calls on a device share the one array: it needs no
 * clearing between calls, but two calls whose kernels can overlap on the GPU (different streams) race
 * on it — serialise them. */
#define B2_STATIC_MAX_ELEMENTS (1u << 26)
int b2_materialize_master_static(uint8_t *d_bytes, uint8_t *d_scales, float *d_global_scale,
                                 const float *d_master, uint32_t len, uint32_t scale_layout,
                                 void *stream);

/* `ScheduleFreeMaterializeArgs` / `...PrecomputedArgs`
 * (.../optimizer/args/schedule_free.rs:13-45).  symexp_lin_beta > 0 applies the SymExpLin forward
 * transform (.../optimizer/symexp_lin.rs:8-26) to every schedule value before it is measured and
 * quantised; symexp_lin_scales are the six device scalars of `SymExpLinScaleRefs` (exponential z, x;
 * linear z, x; curvature z, x), all NULL for the unit scales the reference uses without them. */
typedef struct b2_schedule_free_materialize_args {
    uint8_t *bytes;
    uint8_t *scales;
    float *global_scale;
    const float *z_master;
    const float *x_master;
    const float *precomputed_values; /* precomputed variant only; may be NULL */
    float *amax;                      /* written by materialize_schedule_free, read by _precomputed */
    uint32_t len;
    uint32_t scale_rows;
    uint32_t scale_k;
    float beta;
    float symexp_lin_beta;
    uint32_t scale_layout;
    const float *symexp_lin_scales[6];
} b2_schedule_free_materialize_args;
/* `OptimizerModule::materialize_schedule_free` (.../launcher/update.rs:77-133). */
int b2_materialize_schedule_free(const b2_schedule_free_materialize_args *args, void *stream);
/* `OptimizerModule::materialize_schedule_free_precomputed` (.../launcher/update.rs:25-75). */
int b2_materialize_schedule_free_precomputed(const b2_schedule_free_materialize_args *args,
                                             void *stream);

/* `AdamWUpdateArgs` / `Fp32AdamWUpdateArgs` (.../optimizer/args/adam.rs:3-45). */
typedef struct b2_adamw_update_args {
    uint8_t *bytes;
    uint8_t *scales;
    float *global_scale;
    float *z_master;
    float *x_master;
    float *grad;
    float grad_scale;
    uint32_t scale_layout;
    float *first_moment;
    float *second_moment;
    float *amax;
    float *chunk_amax;
    uint32_t len;
    float learning_rate;
    float weight_decay;
    float beta1;
    float beta2;
    float beta1_correction;
    float beta2_correction;
    float eps;
    float average_coefficient;
    float schedule_beta;
    const float *d_grad_scale; /* optional DEVICE pointer; replaces grad_scale when non-NULL */
} b2_adamw_update_args;
/* `OptimizerModule::apply_adamw_update` (.../launcher/adam.rs:9-21). */
int b2_apply_adamw_update(const b2_adamw_update_args *args, void *stream);
/* `OptimizerModule::apply_adamw_update_deferred_quantization` (.../launcher/adam.rs:23-28). */
int b2_apply_adamw_update_deferred_quantization(const b2_adamw_update_args *args, void *stream);
/* `OptimizerModule::apply_fp32_adamw_update` (.../launcher/adam.rs:45-72); uses z_master,
 * x_master, grad, grad_scale, the moments, len and the scalar hyper-parameters only. */
int b2_apply_fp32_adamw_update(const b2_adamw_update_args *args, void *stream);
/* Multi-tensor forms (no counterpart as a single call in the reference, which issues one to four
 * launches per tensor: src/training/optimizer_apply/adam.rs:18-157,
 * src/training/schedule_free/materialize.rs:44-91).  One device-resident table describes every
 * AdamW tensor; three launches cover all of them.  mode: 0 = apply_fp32_adamw_update,
 * 1 = apply_adamw_update_deferred_quantization (y into grad, max|y| into amax),
 * 2 = apply_adamw_update (requantise x'; max|x'| into amax). */
typedef struct b2_adamw_slot_descriptor {
    uint64_t z_master, x_master, grad, first_moment, second_moment;
    uint64_t amax;          /* f32[1]; modes 1 and 2 */
    uint64_t bytes, scales, global_scale; /* mode 2; mode 1 when materialised later */
    uint32_t len;
    uint32_t chunk_begin;   /* filled by b2_adamw_table_prepare */
    uint32_t mode;
    uint32_t scale_layout;
} b2_adamw_slot_descriptor;
/* Fills chunk_begin of a HOST copy of the table (upload it afterwards); returns the chunk total. */
int b2_adamw_table_prepare(b2_adamw_slot_descriptor *host_table, uint32_t count, uint32_t *total_chunks);
/* Hyper-parameters are taken from `scalars` (pointer fields and len are ignored). */
int b2_apply_adamw_update_multi(const b2_adamw_slot_descriptor *d_table, uint32_t count, uint32_t total_chunks,
                                const b2_adamw_update_args *scalars, void *stream);
/* `Materializer::adam` for every mode-1 entry of the table at once
 * (src/training/schedule_free/tensor.rs:71-89): quantises the schedule-free values with the max|y|
 * the deferred update left in `amax` into bytes / scales / global_scale.  values_cached != 0 reads
 * y from each entry's gradient buffer (where the update left it); 0 rebuilds
 * y = z + schedule_beta * (x - z) from the masters, as the reference does when its cached values
 * are stale (`scheduled_values_valid`, tensor.rs:245).  Entries of other modes are skipped. */
int b2_adamw_materialize_training_weights(const b2_adamw_slot_descriptor *d_table, uint32_t count,
                                          uint32_t total_chunks, float schedule_beta, int values_cached,
                                          void *stream);
/* Stages Q1 + Q2 for every matrix of the plan from the masters x' and the max|x'| the last finish of
 * this plan left in the workspace: a deferred finish followed by this call writes what
 * b2_muon_finish_update writes (crates/cuda-kernels/src/gpt/optimizer/muon/fused/quant/encode.rs:13-60). */
int b2_muon_materialize_master_weights(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, void *stream);
/* `Materializer::muon_precomputed` for every matrix of the plan at once
 * (src/training/schedule_free/tensor.rs:128-153): quantises the cached schedule-free values y
 * (left in each slot's gradient buffer by the update) with the cached schedule_amax. */
int b2_muon_materialize_training_weights(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, void *stream);

/* `OptimizerModule::zero_f32_pointer_table` (.../launcher/adam.rs:30-43). */
int b2_zero_f32_pointer_table(const uint64_t *d_pointers, uint32_t pointer_count, void *stream);

/* ---- SymExpLin scale scalars ------------------------------------------------------------------ */
/* `OptimizerModule::symexp_lin_zero_scale_grads` (.../launcher/symexp_lin.rs:9-22): clears the three
 * scale gradients of every slot that has scale scalars. */
int b2_symexp_lin_zero_scale_grads(const b2_symexp_lin_slot_descriptor *d_slots, uint32_t slot_count, void *stream);
/* `OptimizerModule::symexp_lin_scale_adamw_update` (.../launcher/symexp_lin.rs:24-59): schedule-free
 * AdamW on the exponential, linear (same learning rate, with weight decay) and curvature (own learning
 * rate, no weight decay) scalars of every slot. */
typedef struct b2_symexp_lin_adamw_args {
    float grad_scale;
    float exponential_linear_learning_rate;
    float curvature_learning_rate;
    float weight_decay;
    float beta1, beta2;
    float beta1_correction, beta2_correction;
    float eps;
    float average_coefficient;
} b2_symexp_lin_adamw_args;
int b2_symexp_lin_scale_adamw_update(const b2_symexp_lin_slot_descriptor *d_slots, uint32_t slot_count,
                                     const b2_symexp_lin_adamw_args *args, void *stream);
/* `OptimizerModule::symexp_lin_congruent_inverse_in_place` (.../launcher/symexp_lin.rs:61-75): replaces
 * every value t by the r with (exp(beta r) - 1 + r) / beta = t (sign kept), ten Newton steps from
 * log1p(beta |t|) / beta. */
int b2_symexp_lin_congruent_inverse_in_place(float *d_raw, uint32_t len, float beta, void *stream);

/* ---- global gradient-norm clip (the producer of grad_scale) --------------------------------- */
/* `GradientClipArgs` (crates/cuda-kernels/src/gpt/optimizer/args/grad_clip.rs:3-15). */
typedef struct b2_gradient_clip_args {
    const uint64_t *chunk_ptrs; /* device: f32 pointers, one per chunk (the reference cuts 4096-value chunks) */
    const uint32_t *chunk_lens; /* device: values per chunk */
    float *chunk_sums;          /* device scratch, chunk_count floats */
    const float *extra_sums;    /* device: sums of squares computed elsewhere; may be NULL when count is 0 */
    float *scale;               /* device f32[1]: norm > max_norm ? max_norm / (norm + 1e-6) : 1 */
    float *norm;                /* device f32[1] */
    uint32_t chunk_count;
    uint32_t extra_sum_count;
    float max_norm;
    uint32_t apply;             /* non-zero: also multiply every chunk by the scale */
} b2_gradient_clip_args;
/* `OptimizerModule::clip_gradients` (kernels: .../optimizer/grad_clip/{sumsq,scale,apply}.rs).
 * The reference reads `scale` back to the host after this call; here it can stay on the device
 * and be passed to the step as `d_grad_scale`. */
int b2_clip_gradients(const b2_gradient_clip_args *args, void *stream);

/* ---- CSF block-scale storage, host side -------------------------------------------- */
/* crates/cuda-kernels/src/utils/nvfp4/csf.rs:8-17 (encoded_len). */
size_t b2_csf_encoded_len(size_t rows, size_t k);
/* csf.rs:36-95 (encode_host).  Returns bytes written, 0 on a violated precondition. */
size_t b2_csf_encode_host(const uint8_t *raw, size_t raw_len, size_t rows, size_t k, uint8_t *out,
                          size_t out_capacity);
/* csf.rs:139-147 (scale_at). */
uint8_t b2_csf_scale_at(const uint8_t *encoded, size_t group);

/* ---- host schedules feeding the step scalars ---------------------------------------- */
/* src/training/learning_rate/schedule.rs:24-34, :36-47 + :60-65, :49-58. */
float b2_schedule_free_beta(uint32_t step, uint32_t warmup_steps, float beta1, float rho);
float b2_schedule_free_average_coefficient(uint32_t step, uint32_t warmup_steps, float start_ratio,
                                           float *weight_sum);
float b2_warmup_multiplier(uint32_t step, uint32_t warmup_steps, float start_ratio);

/* ---- multi-GPU: whole-matrix sharding + all-gather of packed weights ------------------ */
/* No counterpart in the reference (single GPU).  Greedy longest-processing-time assignment
 * of whole matrices to ranks by 4 n^2 m + 2 n^3; the slot order follows the reference's
 * work sort (src/training/optimizer_muon/groups/slots.rs:104-106).  owner[i] in [0, world). */
int b2_shard_plan(const uint32_t *rows, const uint32_t *cols, uint32_t slot_count, uint32_t world,
                  uint32_t *owner, double *rank_flops);
/* NCCL plumbing over the process's already-loaded libnccl (resolved with dlopen).
 * unique_id is the 128-byte ncclUniqueId; rank 0 obtains it with b2_comm_unique_id and the
 * caller broadcasts it out of band. */
typedef struct b2_comm b2_comm;
int b2_comm_unique_id(uint8_t unique_id[128]);
int b2_comm_create(b2_comm **comm, const uint8_t unique_id[128], int rank, int world);
void b2_comm_destroy(b2_comm *comm);
/* In-place all-gather of equally sized per-rank arenas: rank r's packed codes, scales and
 * tensor scales live at d_arena + r * bytes_per_rank. */
int b2_allgather_nvfp4(b2_comm *comm, void *d_arena, size_t bytes_per_rank, void *stream);

/* The same exchange without a library collective: every rank's arena lives in a buffer that the other ranks map
 * (one process per GPU, CUDA IPC, NVLink peer access), and a rank copies its slice into the same offset of every
 * peer's buffer with plain stores from one small kernel, which ends by telling every peer how many copies this
 * rank has completed.  All ranks issue the same sequence of copies; `b2_peer_wait` returns (on the stream) once
 * every peer's count has reached this rank's own, i.e. every copy enqueued before it, by any rank, has landed
 * here.  The wait is bounded (`wait_ns`, at most and by default 2e9): when it runs out the kernel sets a status
 * word and returns, and `b2_peer_status` (synchronises) reports B2_ERROR_LAUNCH_TIMEOUT once.  The fixed cost of
 * a copy is a few microseconds, against 50-80 us for an ncclAllGather, so small buckets pay.
 *   b2_peer_buffer_alloc: cudaMalloc of arena_bytes plus a 256-byte control block, zeroed; `handle` is the
 *     64-byte IPC handle to send to the other ranks.  b2_peer_buffer_open maps another rank's buffer
 *     (b2_peer_buffer_close unmaps it); b2_peer_buffer_free releases one's own.
 *   b2_peer_group: world, rank, the arena size given to b2_peer_buffer_alloc, and base[r] = the address at which
 *     this process sees rank r's buffer (its own allocation for r == rank).
 *   b2_peer_push: offset and bytes are multiples of 16 inside the arena; `ctas` caps the grid (0: 48).  Copies and
 *     the wait of one group go on ONE stream. */
#define B2_MAX_PEERS 16
typedef struct b2_peer_group {
    uint32_t world, rank;
    uint64_t arena_bytes;
    uint64_t base[B2_MAX_PEERS];
} b2_peer_group;
int b2_peer_buffer_alloc(size_t arena_bytes, void **d_ptr, uint8_t handle[64]);
int b2_peer_buffer_open(const uint8_t handle[64], void **d_ptr);
int b2_peer_buffer_close(void *d_ptr);
int b2_peer_buffer_free(void *d_ptr);
int b2_peer_push(const b2_peer_group *group, size_t offset, size_t bytes, uint32_t ctas, void *stream);
int b2_peer_wait(const b2_peer_group *group, uint64_t wait_ns, void *stream);
int b2_peer_status(const b2_peer_group *group, void *stream);

/* ---- debug helpers used by the parity tests ------------------------------------------- */
/* Makes the bounded completion-counter wait of the one-launch update + encode run out, harmlessly:
 * launches that kernel as ONE CTA on a one-item list (the encode span at `slot`'s first chunk, none of the
 * slot's update chunks), so the count it waits for is never reached; after `wait_ns` (at most 1e9) the CTA
 * raises the abort and status words, leaves, and clears the ticket and completion words as every launch
 * does.  Nothing is updated or encoded.  b2_muon_plan_status then reports B2_ERROR_LAUNCH_TIMEOUT once.
 * Synchronises `stream` before the launch. */
int b2_debug_muon_fused_wait_expiry(b2_muon_plan *plan, const b2_muon_slot_descriptor *d_slots, uint32_t slot,
                                    uint64_t wait_ns, void *stream);
/* Evaluates `rcp.approx.ftz.f32` (crates/cuda-kernels/src/utils/float_ptx.rs:31-33). */
int b2_debug_rcp_approx_ftz(const float *d_in, float *d_out, uint32_t count, void *stream);
/* Literal one-thread-per-group transcription of the reference quantiser
 * (.../quant/kernels/four_six/helpers.rs:41-94), raw scale plane; the optimised kernels
 * must equal it bit for bit. */
int b2_debug_quantize_literal(const float *d_x, const float *d_amax, uint8_t *d_out_fp4,
                              uint8_t *d_out_raw_scales, float *d_out_global_scale,
                              uint32_t group_count, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LLMINI_B200_H */
