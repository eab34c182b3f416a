//! Rust binding of libllmini_b200.so and a forwarding `OptimizerModule` / `Nvfp4QuantModule` with the
//! reference's method names and argument structs
//! (crates/cuda-kernels/src/gpt/optimizer/launcher/{mod,muon_mega,update,adam,grad_clip,symexp_lin}.rs,
//! crates/cuda-kernels/src/utils/nvfp4/quant/{amax,four_six}.rs).
//!
//! NOT COMPILED HERE: the image this library is built in has no rustc.  The `ffi` module is kept in step
//! with include/llmini_b200.h by a test that parses both files; the forwarding layer is written against the
//! reference's `cuda-core` types (`CudaStream`, `DeviceBuffer<T>`, `DriverError`) and has not been built.
//!
//! Differences from the reference's call surface, all of them on the host:
//! * The five `polar_*` scratch buffers, `normuon_*`, `hyperball_chunks` and `update_chunks` arguments are
//!   accepted and ignored: scratch lives in the plan's workspace, sized by `b2_muon_workspace_bytes`.
//! * The reference's split path is called once per slot (`slot_index`).  The library runs a stage for every
//!   slot of the plan in one call, so the per-slot methods run the stage when they are called for the
//!   plan's FIRST non-empty slot and return `Ok` for the other slots: the trainer's loop over slots stays as
//!   it is (src/training/optimizer_muon/tma.rs:74-199), provided it visits the first slot first and passes
//!   the same scalars for every slot of a group, which it does.
//! * Preconditions the reference asserts come back as `DriverError(1)`.

#![allow(clippy::too_many_arguments)]

use std::cell::Cell;

use cuda_core::{CudaStream, DeviceBuffer, DriverError};

pub mod ffi {
    //! Mirror of include/llmini_b200.h: same names, same field order.
    use std::ffi::c_void;

    pub type CUdeviceptr = u64;
    pub type CUstream = *mut c_void;

    pub const B2_ABI_VERSION: u32 = 2;
    pub const B2_SUCCESS: i32 = 0;
    pub const B2_ERROR_INVALID_VALUE: i32 = 1;
    pub const B2_ERROR_LAUNCH_TIMEOUT: i32 = 702;
    pub const B2_OPERAND_BF16: u32 = 0;
    pub const B2_OPERAND_F16: u32 = 1;
    pub const B2_SCALES_CSF: u32 = 0;
    pub const B2_SCALES_RAW: u32 = 1;
    pub const B2_SCALES_SM100: u32 = 2;
    pub const B2_QUANTIZE_X: u32 = 0;
    pub const B2_QUANTIZE_Y: u32 = 1;
    pub const B2_NORMALIZE_TWO_PASS: u32 = 0;
    pub const B2_NORMALIZE_DEFERRED: u32 = 1;
    pub const B2_NS_PER_PHASE: u32 = 0;
    pub const B2_NS_CHAINED: u32 = 1;
    pub const B2_NS_FUSED_GRAM_POLY: u32 = 2;
    pub const B2_UPDATE_F32: u32 = 0;
    pub const B2_UPDATE_16BIT: u32 = 1;
    pub const B2_STATIC_MAX_ELEMENTS: u32 = 1 << 26;
    pub const B2_MAX_PEERS: usize = 16;

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct b2_muon_slot_descriptor {
        pub grad: u64,
        pub momentum: u64,
        pub variance: u64,
        pub second_momentum: u64,
        pub z_master: u64,
        pub x_master: u64,
        pub schedule_amax: u64,
        pub bytes: u64,
        pub scales: u64,
        pub global_scale: u64,
        pub rows: u32,
        pub cols: u32,
        pub learning_rate_multiplier: f32,
        pub qk_clip_factor_offset: u32,
        pub qk_clip_head_dim: u32,
        pub reserved_padding: u32,
    }

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct b2_symexp_lin_slot_descriptor {
        pub grad: u64,
        pub z_master: u64,
        pub x_master: u64,
        pub exponential_z: u64,
        pub exponential_x: u64,
        pub exponential_grad: u64,
        pub exponential_first: u64,
        pub exponential_second: u64,
        pub linear_z: u64,
        pub linear_x: u64,
        pub linear_grad: u64,
        pub linear_first: u64,
        pub linear_second: u64,
        pub curvature_z: u64,
        pub curvature_x: u64,
        pub curvature_grad: u64,
        pub curvature_first: u64,
        pub curvature_second: u64,
        pub rows: u32,
        pub cols: u32,
    }

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct b2_muon_options {
        pub operand_format: u32,
        pub scale_layout: u32,
        pub quantize_target: u32,
        pub max_iterations: u32,
        pub tile_override: u32,
        pub measure_phase_mask: u32,
        pub measure_flags: u32,
        pub normalize_mode: u32,
        pub ns_schedule: u32,
        pub update_input: u32,
        pub reserved: [u32; 2],
    }

    #[repr(C)]
    #[derive(Clone, Copy)]
    pub struct b2_muon_step_args {
        pub mu: f32,
        pub grad_scale: f32,
        pub learning_rate: f32,
        pub weight_decay: f32,
        pub average_coefficient: f32,
        pub schedule_beta: f32,
        pub iterations: u32,
        pub nesterov: u32,
        pub coefficients: *const f32,
        pub d_grad_scale: CUdeviceptr,
        pub variance_adaptive: u32,
        pub bias_correction_inv: f32,
        pub d_qk_clip_factors: CUdeviceptr,
        pub symexp_lin_beta: f32,
        pub d_symexp_lin_slots: CUdeviceptr,
        pub normuon: u32,
        pub reserved_padding: u32,
    }

    #[repr(C)]
    #[derive(Clone, Copy)]
    pub struct b2_schedule_free_materialize_args {
        pub bytes: CUdeviceptr,
        pub scales: CUdeviceptr,
        pub global_scale: CUdeviceptr,
        pub z_master: CUdeviceptr,
        pub x_master: CUdeviceptr,
        pub precomputed_values: CUdeviceptr,
        pub amax: CUdeviceptr,
        pub len: u32,
        pub scale_rows: u32,
        pub scale_k: u32,
        pub beta: f32,
        pub symexp_lin_beta: f32,
        pub scale_layout: u32,
        pub symexp_lin_scales: [CUdeviceptr; 6],
    }

    #[repr(C)]
    #[derive(Clone, Copy)]
    pub struct b2_adamw_update_args {
        pub bytes: CUdeviceptr,
        pub scales: CUdeviceptr,
        pub global_scale: CUdeviceptr,
        pub z_master: CUdeviceptr,
        pub x_master: CUdeviceptr,
        pub grad: CUdeviceptr,
        pub grad_scale: f32,
        pub scale_layout: u32,
        pub first_moment: CUdeviceptr,
        pub second_moment: CUdeviceptr,
        pub amax: CUdeviceptr,
        pub chunk_amax: CUdeviceptr,
        pub len: u32,
        pub learning_rate: f32,
        pub weight_decay: f32,
        pub beta1: f32,
        pub beta2: f32,
        pub beta1_correction: f32,
        pub beta2_correction: f32,
        pub eps: f32,
        pub average_coefficient: f32,
        pub schedule_beta: f32,
        pub d_grad_scale: CUdeviceptr,
    }

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct b2_peer_group {
        pub world: u32,
        pub rank: u32,
        pub arena_bytes: u64,
        pub base: [u64; B2_MAX_PEERS],
    }

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct b2_adamw_slot_descriptor {
        pub z_master: u64,
        pub x_master: u64,
        pub grad: u64,
        pub first_moment: u64,
        pub second_moment: u64,
        pub amax: u64,
        pub bytes: u64,
        pub scales: u64,
        pub global_scale: u64,
        pub len: u32,
        pub chunk_begin: u32,
        pub mode: u32,
        pub scale_layout: u32,
    }

    #[repr(C)]
    #[derive(Clone, Copy)]
    pub struct b2_symexp_lin_adamw_args {
        pub grad_scale: f32,
        pub exponential_linear_learning_rate: f32,
        pub curvature_learning_rate: f32,
        pub weight_decay: f32,
        pub beta1: f32,
        pub beta2: f32,
        pub beta1_correction: f32,
        pub beta2_correction: f32,
        pub eps: f32,
        pub average_coefficient: f32,
    }

    #[repr(C)]
    #[derive(Clone, Copy)]
    pub struct b2_gradient_clip_args {
        pub chunk_ptrs: CUdeviceptr,
        pub chunk_lens: CUdeviceptr,
        pub chunk_sums: CUdeviceptr,
        pub extra_sums: CUdeviceptr,
        pub scale: CUdeviceptr,
        pub norm: CUdeviceptr,
        pub chunk_count: u32,
        pub extra_sum_count: u32,
        pub max_norm: f32,
        pub apply: u32,
    }

    #[repr(C)]
    pub struct b2_muon_plan {
        _opaque: [u8; 0],
    }
    #[repr(C)]
    pub struct b2_comm {
        _opaque: [u8; 0],
    }

    extern "C" {
        pub fn b2_abi_version() -> u32;
        pub fn b2_error_string(code: i32) -> *const std::ffi::c_char;
        pub fn b2_verify_storage_layout(stream: CUstream) -> i32;
        pub fn b2_muon_workspace_bytes(rows: *const u32, cols: *const u32, slot_count: u32,
                                       options: *const b2_muon_options) -> usize;
        pub fn b2_muon_plan_create(plan: *mut *mut b2_muon_plan, rows: *const u32, cols: *const u32, slot_count: u32,
                                   options: *const b2_muon_options, d_workspace: CUdeviceptr, workspace_bytes: usize,
                                   stream: CUstream) -> i32;
        pub fn b2_muon_plan_destroy(plan: *mut b2_muon_plan);
        pub fn b2_muon_mega_update(plan: *mut b2_muon_plan, d_slots: CUdeviceptr, args: *const b2_muon_step_args,
                                   stream: CUstream) -> i32;
        pub fn b2_muon_prepare_polar(plan: *mut b2_muon_plan, d_slots: CUdeviceptr, args: *const b2_muon_step_args,
                                     stream: CUstream) -> i32;
        pub fn b2_muon_polar(plan: *mut b2_muon_plan, args: *const b2_muon_step_args, stream: CUstream) -> i32;
        pub fn b2_muon_finish_update(plan: *mut b2_muon_plan, d_slots: CUdeviceptr, args: *const b2_muon_step_args,
                                     stream: CUstream) -> i32;
        pub fn b2_muon_finish_update_deferred_quantization(plan: *mut b2_muon_plan, d_slots: CUdeviceptr,
                                                           args: *const b2_muon_step_args, stream: CUstream) -> i32;
        pub fn b2_muon_plan_set_finish_groups(plan: *mut b2_muon_plan, first_slot: *const u32, group_count: u32,
                                              stream: CUstream) -> i32;
        pub fn b2_muon_finish_update_group(plan: *mut b2_muon_plan, d_slots: CUdeviceptr, args: *const b2_muon_step_args,
                                           group: u32, stream: CUstream) -> i32;
        pub fn b2_muon_finish_hyperball_update_deferred_quantization(plan: *mut b2_muon_plan, d_slots: CUdeviceptr,
                                                                     args: *const b2_muon_step_args,
                                                                     use_schedule_free: u32, stream: CUstream) -> i32;
        pub fn b2_muon_sign_update_deferred_quantization(plan: *mut b2_muon_plan, d_slots: CUdeviceptr,
                                                         args: *const b2_muon_step_args, stream: CUstream) -> i32;
        pub fn b2_muon_plan_scratch(plan: *mut b2_muon_plan, slot: u32, which: u32, d_ptr: *mut CUdeviceptr,
                                    bytes: *mut usize) -> i32;
        pub fn b2_muon_plan_status(plan: *mut b2_muon_plan, stream: CUstream) -> i32;
        pub fn b2_muon_plan_flops_per_iteration(plan: *const b2_muon_plan) -> f64;
        pub fn b2_tensor_amax_f32(d_x: CUdeviceptr, d_chunk_amax: CUdeviceptr, d_out: CUdeviceptr, element_count: u32,
                                  stream: CUstream) -> i32;
        pub fn b2_tensor_amax_from_chunks_f32(d_chunk_amax: CUdeviceptr, d_out: CUdeviceptr, chunk_count: u32,
                                              stream: CUstream) -> i32;
        pub fn b2_fp32_to_nvfp4_four_six(d_x: CUdeviceptr, d_amax: CUdeviceptr, d_out_fp4: CUdeviceptr,
                                         d_out_scales: CUdeviceptr, d_out_global_scale: CUdeviceptr, group_count: u32,
                                         scale_layout: u32, stream: CUstream) -> i32;
        pub fn b2_nvfp4_sm100_scales_bytes(rows: u32, cols: u32) -> usize;
        pub fn b2_nvfp4_scales_to_sm100(d_scales: CUdeviceptr, src_layout: u32, rows: u32, cols: u32, d_out: CUdeviceptr,
                                        stream: CUstream) -> i32;
        pub fn b2_materialize_master(d_bytes: CUdeviceptr, d_scales: CUdeviceptr, d_global_scale: CUdeviceptr,
                                     d_master: CUdeviceptr, d_amax: CUdeviceptr, d_chunk_amax: CUdeviceptr, len: u32,
                                     scale_layout: u32, stream: CUstream) -> i32;
        pub fn b2_materialize_master_static(d_bytes: CUdeviceptr, d_scales: CUdeviceptr, d_global_scale: CUdeviceptr,
                                            d_master: CUdeviceptr, len: u32, scale_layout: u32, stream: CUstream) -> i32;
        pub fn b2_materialize_schedule_free(args: *const b2_schedule_free_materialize_args, stream: CUstream) -> i32;
        pub fn b2_materialize_schedule_free_precomputed(args: *const b2_schedule_free_materialize_args,
                                                        stream: CUstream) -> i32;
        pub fn b2_apply_adamw_update(args: *const b2_adamw_update_args, stream: CUstream) -> i32;
        pub fn b2_apply_adamw_update_deferred_quantization(args: *const b2_adamw_update_args, stream: CUstream) -> i32;
        pub fn b2_apply_fp32_adamw_update(args: *const b2_adamw_update_args, stream: CUstream) -> i32;
        pub fn b2_adamw_table_prepare(host_table: *mut b2_adamw_slot_descriptor, count: u32,
                                      total_chunks: *mut u32) -> i32;
        pub fn b2_apply_adamw_update_multi(d_table: CUdeviceptr, count: u32, total_chunks: u32,
                                           scalars: *const b2_adamw_update_args, stream: CUstream) -> i32;
        pub fn b2_adamw_materialize_training_weights(d_table: CUdeviceptr, count: u32, total_chunks: u32,
                                                     schedule_beta: f32, values_cached: i32, stream: CUstream) -> i32;
        pub fn b2_muon_materialize_master_weights(plan: *mut b2_muon_plan, d_slots: CUdeviceptr, stream: CUstream) -> i32;
        pub fn b2_muon_materialize_training_weights(plan: *mut b2_muon_plan, d_slots: CUdeviceptr,
                                                    stream: CUstream) -> i32;
        pub fn b2_zero_f32_pointer_table(d_pointers: CUdeviceptr, pointer_count: u32, stream: CUstream) -> i32;
        pub fn b2_symexp_lin_zero_scale_grads(d_slots: CUdeviceptr, slot_count: u32, stream: CUstream) -> i32;
        pub fn b2_symexp_lin_scale_adamw_update(d_slots: CUdeviceptr, slot_count: u32,
                                                args: *const b2_symexp_lin_adamw_args, stream: CUstream) -> i32;
        pub fn b2_symexp_lin_congruent_inverse_in_place(d_raw: CUdeviceptr, len: u32, beta: f32, stream: CUstream) -> i32;
        pub fn b2_clip_gradients(args: *const b2_gradient_clip_args, stream: CUstream) -> i32;
        pub fn b2_csf_encoded_len(rows: usize, k: usize) -> usize;
        pub fn b2_csf_encode_host(raw: *const u8, raw_len: usize, rows: usize, k: usize, out: *mut u8,
                                  out_capacity: usize) -> usize;
        pub fn b2_csf_scale_at(encoded: *const u8, group: usize) -> u8;
        pub fn b2_schedule_free_beta(step: u32, warmup_steps: u32, beta1: f32, rho: f32) -> f32;
        pub fn b2_schedule_free_average_coefficient(step: u32, warmup_steps: u32, start_ratio: f32,
                                                    weight_sum: *mut f32) -> f32;
        pub fn b2_warmup_multiplier(step: u32, warmup_steps: u32, start_ratio: f32) -> f32;
        pub fn b2_shard_plan(rows: *const u32, cols: *const u32, slot_count: u32, world: u32, owner: *mut u32,
                             rank_flops: *mut f64) -> i32;
        pub fn b2_comm_unique_id(unique_id: *mut u8) -> i32;
        pub fn b2_comm_create(comm: *mut *mut b2_comm, unique_id: *const u8, rank: i32, world: i32) -> i32;
        pub fn b2_comm_destroy(comm: *mut b2_comm);
        pub fn b2_allgather_nvfp4(comm: *mut b2_comm, d_arena: CUdeviceptr, bytes_per_rank: usize, stream: CUstream) -> i32;
        pub fn b2_peer_buffer_alloc(arena_bytes: usize, d_ptr: *mut CUdeviceptr, handle: *mut u8) -> i32;
        pub fn b2_peer_buffer_open(handle: *const u8, d_ptr: *mut CUdeviceptr) -> i32;
        pub fn b2_peer_buffer_close(d_ptr: CUdeviceptr) -> i32;
        pub fn b2_peer_buffer_free(d_ptr: CUdeviceptr) -> i32;
        pub fn b2_peer_push(group: *const b2_peer_group, offset: usize, bytes: usize, ctas: u32, stream: CUstream) -> i32;
        pub fn b2_peer_wait(group: *const b2_peer_group, wait_ns: u64, stream: CUstream) -> i32;
        pub fn b2_peer_status(group: *const b2_peer_group, stream: CUstream) -> i32;
        pub fn b2_debug_muon_fused_wait_expiry(plan: *mut b2_muon_plan, d_slots: CUdeviceptr, slot: u32, wait_ns: u64,
                                               stream: CUstream) -> i32;
        pub fn b2_debug_rcp_approx_ftz(d_in: CUdeviceptr, d_out: CUdeviceptr, count: u32, stream: CUstream) -> i32;
        pub fn b2_debug_quantize_literal(d_x: CUdeviceptr, d_amax: CUdeviceptr, d_out_fp4: CUdeviceptr,
                                         d_out_raw_scales: CUdeviceptr, d_out_global_scale: CUdeviceptr, group_count: u32,
                                         stream: CUstream) -> i32;
    }
}

use ffi::*;

fn check(code: i32) -> Result<(), DriverError> {
    if code == B2_SUCCESS {
        Ok(())
    } else {
        Err(DriverError(code as u32))
    }
}
fn ptr<T>(b: &DeviceBuffer<T>) -> CUdeviceptr {
    b.cu_deviceptr()
}
fn opt_ptr<T>(b: Option<&DeviceBuffer<T>>) -> CUdeviceptr {
    b.map_or(0, |b| b.cu_deviceptr())
}

// ---------------------------------------------------------------------------------------------------------
// Argument structs: the reference's, field for field (crates/cuda-kernels/src/gpt/optimizer/args/*.rs).
// ---------------------------------------------------------------------------------------------------------
pub type MuonSlotDescriptor = b2_muon_slot_descriptor; // args/muon.rs:3-21 (+ the 4 bytes of tail padding, named)
pub type SymExpLinSlotDescriptor = b2_symexp_lin_slot_descriptor; // args/symexp_lin.rs:5-26

/// args/muon.rs:25-44
pub struct MuonMegaUpdateArgs<'a> {
    pub stream: &'a CudaStream,
    pub slots: &'a DeviceBuffer<MuonSlotDescriptor>,
    pub oriented: &'a mut DeviceBuffer<f32>,
    pub polar_next: &'a mut DeviceBuffer<f32>,
    pub polar_x: &'a mut DeviceBuffer<f32>,
    pub polar_gram: &'a mut DeviceBuffer<f32>,
    pub polar_ax: &'a mut DeviceBuffer<f32>,
    pub polar_chunks: &'a mut DeviceBuffer<f32>,
    pub slot_count: u32,
    pub max_len: u32,
    pub max_ax_len: u32,
    pub max_dim: u32,
    pub mu: f32,
    pub grad_scale: f32,
    pub learning_rate: f32,
    pub weight_decay: f32,
    pub average_coefficient: f32,
    pub iterations: u32,
}
/// args/muon.rs:46-60
pub struct MuonTmaPrepareArgs<'a> {
    pub stream: &'a CudaStream,
    pub slots: &'a DeviceBuffer<MuonSlotDescriptor>,
    pub oriented: &'a mut DeviceBuffer<f32>,
    pub polar_x: &'a mut DeviceBuffer<f32>,
    pub polar_chunks: &'a mut DeviceBuffer<f32>,
    pub polar_x_chunk_amax: &'a mut DeviceBuffer<f32>,
    pub slot_index: u32,
    pub matrix_len: u32,
    pub mu: f32,
    pub grad_scale: f32,
    pub nesterov: u32,
    pub variance_adaptive: u32,
    pub bias_correction_inv: f32,
}
/// args/muon.rs:62-83
pub struct MuonTmaFinishArgs<'a> {
    pub stream: &'a CudaStream,
    pub slots: &'a DeviceBuffer<MuonSlotDescriptor>,
    pub symexp_lin_slots: &'a DeviceBuffer<SymExpLinSlotDescriptor>,
    pub polar_update: &'a DeviceBuffer<f32>,
    pub polar_bound_amax: &'a DeviceBuffer<f32>,
    pub polar_chunks: &'a mut DeviceBuffer<f32>,
    pub normuon_factors: &'a mut DeviceBuffer<f32>,
    pub normuon_chunks: &'a mut DeviceBuffer<f32>,
    pub qk_clip_factors: &'a DeviceBuffer<f32>,
    pub slot_index: u32,
    pub matrix_len: u32,
    pub matrix_rows: u32,
    pub matrix_cols: u32,
    pub polar_cols: u32,
    pub learning_rate: f32,
    pub weight_decay: f32,
    pub average_coefficient: f32,
    pub schedule_beta: f32,
    pub symexp_lin_beta: f32,
    pub apply_polar_sqrt_bound: u32,
}
/// args/muon.rs:85-89
pub struct MuonTmaHyperballFinishArgs<'a> {
    pub finish: MuonTmaFinishArgs<'a>,
    pub hyperball_chunks: &'a mut DeviceBuffer<f32>,
    pub use_schedule_free: bool,
}
/// args/muon.rs:91-107
pub struct MuonTmaSignUpdateArgs<'a> {
    pub stream: &'a CudaStream,
    pub slots: &'a DeviceBuffer<MuonSlotDescriptor>,
    pub symexp_lin_slots: &'a DeviceBuffer<SymExpLinSlotDescriptor>,
    pub update_chunks: &'a mut DeviceBuffer<f32>,
    pub qk_clip_factors: &'a DeviceBuffer<f32>,
    pub slot_index: u32,
    pub matrix_len: u32,
    pub mu: f32,
    pub grad_scale: f32,
    pub variance_adaptive: u32,
    pub learning_rate: f32,
    pub weight_decay: f32,
    pub average_coefficient: f32,
    pub schedule_beta: f32,
    pub symexp_lin_beta: f32,
}
/// args/schedule_free.rs:3-11
#[derive(Clone, Copy)]
pub struct SymExpLinScaleRefs<'a> {
    pub exponential_z: &'a DeviceBuffer<f32>,
    pub exponential_x: &'a DeviceBuffer<f32>,
    pub linear_z: &'a DeviceBuffer<f32>,
    pub linear_x: &'a DeviceBuffer<f32>,
    pub curvature_z: &'a DeviceBuffer<f32>,
    pub curvature_x: &'a DeviceBuffer<f32>,
}
/// args/schedule_free.rs:13-28
pub struct ScheduleFreeMaterializeArgs<'a> {
    pub stream: &'a CudaStream,
    pub bytes: &'a mut DeviceBuffer<u8>,
    pub scales: &'a mut DeviceBuffer<u8>,
    pub global_scale: &'a mut DeviceBuffer<f32>,
    pub z_master: &'a DeviceBuffer<f32>,
    pub x_master: &'a DeviceBuffer<f32>,
    pub amax: &'a mut DeviceBuffer<f32>,
    pub chunk_amax: &'a mut DeviceBuffer<f32>,
    pub len: u32,
    pub scale_rows: u32,
    pub scale_k: u32,
    pub beta: f32,
    pub symexp_lin_beta: f32,
    pub symexp_lin_scales: Option<SymExpLinScaleRefs<'a>>,
}
/// args/schedule_free.rs:30-45
pub struct ScheduleFreeMaterializePrecomputedArgs<'a> {
    pub stream: &'a CudaStream,
    pub bytes: &'a mut DeviceBuffer<u8>,
    pub scales: &'a mut DeviceBuffer<u8>,
    pub global_scale: &'a mut DeviceBuffer<f32>,
    pub z_master: &'a DeviceBuffer<f32>,
    pub x_master: &'a DeviceBuffer<f32>,
    pub precomputed_values: Option<&'a DeviceBuffer<f32>>,
    pub amax: &'a DeviceBuffer<f32>,
    pub len: u32,
    pub scale_rows: u32,
    pub scale_k: u32,
    pub beta: f32,
    pub symexp_lin_beta: f32,
    pub symexp_lin_scales: Option<SymExpLinScaleRefs<'a>>,
}
/// args/adam.rs:3-26
pub struct AdamWUpdateArgs<'a> {
    pub stream: &'a CudaStream,
    pub bytes: &'a mut DeviceBuffer<u8>,
    pub scales: &'a mut DeviceBuffer<u8>,
    pub global_scale: &'a mut DeviceBuffer<f32>,
    pub z_master: &'a mut DeviceBuffer<f32>,
    pub x_master: &'a mut DeviceBuffer<f32>,
    pub grad: &'a mut DeviceBuffer<f32>,
    pub grad_scale: f32,
    pub first_moment: &'a mut DeviceBuffer<f32>,
    pub second_moment: &'a mut DeviceBuffer<f32>,
    pub amax: &'a mut DeviceBuffer<f32>,
    pub chunk_amax: &'a mut DeviceBuffer<f32>,
    pub len: u32,
    pub learning_rate: f32,
    pub weight_decay: f32,
    pub beta1: f32,
    pub beta2: f32,
    pub beta1_correction: f32,
    pub beta2_correction: f32,
    pub eps: f32,
    pub average_coefficient: f32,
    pub schedule_beta: f32,
}
/// args/adam.rs:28-45
pub struct Fp32AdamWUpdateArgs<'a> {
    pub stream: &'a CudaStream,
    pub z_master: &'a mut DeviceBuffer<f32>,
    pub x_master: &'a mut DeviceBuffer<f32>,
    pub grad: &'a DeviceBuffer<f32>,
    pub grad_scale: f32,
    pub first_moment: &'a mut DeviceBuffer<f32>,
    pub second_moment: &'a mut DeviceBuffer<f32>,
    pub len: u32,
    pub learning_rate: f32,
    pub weight_decay: f32,
    pub beta1: f32,
    pub beta2: f32,
    pub beta1_correction: f32,
    pub beta2_correction: f32,
    pub eps: f32,
    pub average_coefficient: f32,
}
/// args/grad_clip.rs:3-15
pub struct GradientClipArgs<'a> {
    pub stream: &'a CudaStream,
    pub chunk_ptrs: &'a DeviceBuffer<u64>,
    pub chunk_lens: &'a DeviceBuffer<u32>,
    pub chunk_sums: &'a mut DeviceBuffer<f32>,
    pub extra_sums: &'a DeviceBuffer<f32>,
    pub scale: &'a mut DeviceBuffer<f32>,
    pub norm: &'a mut DeviceBuffer<f32>,
    pub chunk_count: u32,
    pub extra_sum_count: u32,
    pub max_norm: f32,
    pub apply: bool,
}
/// crates/cuda-kernels/src/utils/nvfp4/quant/args/basic.rs:3-11
pub struct Nvfp4QuantArgs<'a, 'b> {
    pub stream: &'a CudaStream,
    pub x: &'b DeviceBuffer<f32>,
    pub amax: &'b DeviceBuffer<f32>,
    pub out_fp4: &'b mut DeviceBuffer<u8>,
    pub out_scales: &'b mut DeviceBuffer<u8>,
    pub out_global_scale: &'b mut DeviceBuffer<f32>,
    pub group_count: u32,
}
/// crates/cuda-kernels/src/utils/nvfp4/quant/args/basic.rs:100-106
pub struct TensorAmaxArgs<'a, 'b> {
    pub stream: &'a CudaStream,
    pub x: &'b DeviceBuffer<f32>,
    pub chunk_amax: &'b mut DeviceBuffer<f32>,
    pub out: &'b mut DeviceBuffer<f32>,
    pub element_count: u32,
}

// ---------------------------------------------------------------------------------------------------------
// Nvfp4QuantModule (crates/cuda-kernels/src/utils/nvfp4/quant/launcher.rs:7-16)
// ---------------------------------------------------------------------------------------------------------
pub struct Nvfp4QuantModule {
    /// B2_SCALES_CSF for the reference's storage; B2_SCALES_RAW where `k % 128 != 0`.
    pub scale_layout: u32,
}

impl Nvfp4QuantModule {
    /// quant/amax.rs:19-23
    pub fn tensor_amax_f32(&self, args: TensorAmaxArgs<'_, '_>) -> Result<(), DriverError> {
        check(unsafe {
            b2_tensor_amax_f32(ptr(args.x), ptr(args.chunk_amax), ptr(args.out), args.element_count, args.stream.cu_stream())
        })
    }
    /// quant/amax.rs:25-39
    pub fn tensor_amax_from_chunks_f32(&self, stream: &CudaStream, chunk_amax: &DeviceBuffer<f32>,
                                       out: &mut DeviceBuffer<f32>, chunk_count: u32) -> Result<(), DriverError> {
        check(unsafe { b2_tensor_amax_from_chunks_f32(ptr(chunk_amax), ptr(out), chunk_count, stream.cu_stream()) })
    }
    /// quant/four_six.rs:19-30
    pub fn fp32_to_nvfp4_four_six(&self, args: Nvfp4QuantArgs<'_, '_>) -> Result<(), DriverError> {
        check(unsafe {
            b2_fp32_to_nvfp4_four_six(ptr(args.x), ptr(args.amax), ptr(args.out_fp4), ptr(args.out_scales),
                                      ptr(args.out_global_scale), args.group_count, self.scale_layout,
                                      args.stream.cu_stream())
        })
    }
}

// ---------------------------------------------------------------------------------------------------------
// OptimizerModule (crates/cuda-kernels/src/gpt/optimizer/launcher/mod.rs:20-26)
// ---------------------------------------------------------------------------------------------------------
/// Host copy of the slot shapes the plan was built for (the reference keeps `host_slots` beside the device
/// table: src/training/optimizer_muon/groups.rs:36-41).
pub struct MuonPlan {
    raw: *mut b2_muon_plan,
    first_slot: u32,
    options: b2_muon_options,
    _workspace: DeviceBuffer<u8>,
}

impl MuonPlan {
    /// Replaces the allocation of the five scratch buffers in src/training/optimizer_tc_scratch.rs:43-66.
    pub fn new(stream: &CudaStream, rows: &[u32], cols: &[u32], options: b2_muon_options) -> Result<Self, DriverError> {
        assert_eq!(rows.len(), cols.len());
        let n = rows.len() as u32;
        let bytes = unsafe { b2_muon_workspace_bytes(rows.as_ptr(), cols.as_ptr(), n, &options) };
        if bytes == 0 {
            return Err(DriverError(B2_ERROR_INVALID_VALUE as u32));
        }
        // 1 KiB alignment: cuMemAlloc returns at least 256-byte aligned blocks, so over-allocate
        let workspace: DeviceBuffer<u8> = DeviceBuffer::zeroed(stream, bytes + 1024)?;
        let base = (workspace.cu_deviceptr() + 1023) & !1023u64;
        let mut raw: *mut b2_muon_plan = std::ptr::null_mut();
        check(unsafe {
            b2_muon_plan_create(&mut raw, rows.as_ptr(), cols.as_ptr(), n, &options, base, bytes, stream.cu_stream())
        })?;
        let first_slot = rows.iter().zip(cols).position(|(r, c)| (*r as u64) * (*c as u64) != 0).unwrap_or(0) as u32;
        Ok(Self { raw, first_slot, options, _workspace: workspace })
    }
    /// Cuts the plan's slots into contiguous runs for `OptimizerModule::muon_tma_finish_update_group`.
    pub fn set_finish_groups(&self, stream: &CudaStream, first_slot: &[u32]) -> Result<(), DriverError> {
        check(unsafe {
            b2_muon_plan_set_finish_groups(self.raw, first_slot.as_ptr(), first_slot.len() as u32, stream.cu_stream())
        })
    }
    /// Whether a bounded device-side wait ran out since the last call (synchronises the stream).
    pub fn status(&self, stream: &CudaStream) -> Result<(), DriverError> {
        check(unsafe { b2_muon_plan_status(self.raw, stream.cu_stream()) })
    }
}
impl Drop for MuonPlan {
    fn drop(&mut self) {
        unsafe { b2_muon_plan_destroy(self.raw) }
    }
}

pub struct OptimizerModule {
    pub plan: MuonPlan,
    quant: Nvfp4QuantModule,
    /// Scalars of the prepare call of the current group, needed again by `b2_muon_polar`.
    iterations: Cell<u32>,
}

impl OptimizerModule {
    pub fn new(plan: MuonPlan, iterations: u32) -> Self {
        let scale_layout = plan.options.scale_layout;
        Self { plan, quant: Nvfp4QuantModule { scale_layout }, iterations: Cell::new(iterations) }
    }

    fn step_args(mu: f32, grad_scale: f32, learning_rate: f32, weight_decay: f32, average_coefficient: f32,
                 schedule_beta: f32, iterations: u32, nesterov: u32) -> b2_muon_step_args {
        b2_muon_step_args {
            mu,
            grad_scale,
            learning_rate,
            weight_decay,
            average_coefficient,
            schedule_beta,
            iterations,
            nesterov,
            coefficients: std::ptr::null(), // the reference's coefficient table
            d_grad_scale: 0,
            variance_adaptive: 0,
            bias_correction_inv: 1.0,
            d_qk_clip_factors: 0,
            symexp_lin_beta: 0.0,
            d_symexp_lin_slots: 0,
            normuon: 0,
            reserved_padding: 0,
        }
    }
    fn finish_args(&self, a: &MuonTmaFinishArgs<'_>, normuon: u32) -> b2_muon_step_args {
        let mut s = Self::step_args(0.0, 1.0, a.learning_rate, a.weight_decay, a.average_coefficient, a.schedule_beta,
                                    self.iterations.get(), 1);
        s.d_qk_clip_factors = if a.qk_clip_factors.is_empty() { 0 } else { ptr(a.qk_clip_factors) };
        s.symexp_lin_beta = a.symexp_lin_beta;
        s.d_symexp_lin_slots = if a.symexp_lin_slots.is_empty() { 0 } else { ptr(a.symexp_lin_slots) };
        s.normuon = normuon;
        s
    }

    /// launcher/mod.rs:43-56
    pub fn verify_storage_layout(&self, stream: &CudaStream) -> Result<(), DriverError> {
        if unsafe { b2_abi_version() } != B2_ABI_VERSION {
            return Err(DriverError(B2_ERROR_INVALID_VALUE as u32));
        }
        check(unsafe { b2_verify_storage_layout(stream.cu_stream()) })
    }

    /// launcher/mod.rs:67-95
    pub fn materialize_master(&self, stream: &CudaStream, bytes: &mut DeviceBuffer<u8>, scales: &mut DeviceBuffer<u8>,
                              global_scale: &mut DeviceBuffer<f32>, master: &DeviceBuffer<f32>,
                              amax: &mut DeviceBuffer<f32>, chunk_amax: &mut DeviceBuffer<f32>,
                              len: u32) -> Result<(), DriverError> {
        check(unsafe {
            b2_materialize_master(ptr(bytes), ptr(scales), ptr(global_scale), ptr(master), ptr(amax), ptr(chunk_amax), len,
                                  self.quant.scale_layout, stream.cu_stream())
        })
    }
    /// No counterpart in the reference: `materialize_master` for call sites without scratch buffers
    /// (b2_materialize_master_static; at most B2_STATIC_MAX_ELEMENTS values, calls must not overlap on the GPU).
    pub fn materialize_master_static(&self, stream: &CudaStream, bytes: &mut DeviceBuffer<u8>,
                                     scales: &mut DeviceBuffer<u8>, global_scale: &mut DeviceBuffer<f32>,
                                     master: &DeviceBuffer<f32>, len: u32) -> Result<(), DriverError> {
        check(unsafe {
            b2_materialize_master_static(ptr(bytes), ptr(scales), ptr(global_scale), ptr(master), len,
                                         self.quant.scale_layout, stream.cu_stream())
        })
    }

    /// launcher/muon_mega.rs:24-51.  The scratch buffers of the argument struct are not used.
    pub fn muon_mega_update(&self, args: MuonMegaUpdateArgs<'_>) -> Result<(), DriverError> {
        let step = Self::step_args(args.mu, args.grad_scale, args.learning_rate, args.weight_decay,
                                   args.average_coefficient, 1.0, args.iterations, 1);
        check(unsafe { b2_muon_mega_update(self.plan.raw, ptr(args.slots), &step, args.stream.cu_stream()) })
    }

    /// launcher/muon_mega.rs:53-115.  Runs stages M+N and the Newton-Schulz loop for every slot of the plan
    /// when called for the plan's first slot; the reference returns the number of amax chunks it wrote, which
    /// has no meaning here (0).
    pub fn muon_tma_prepare_polar(&self, args: MuonTmaPrepareArgs<'_>) -> Result<u32, DriverError> {
        if args.slot_index != self.plan.first_slot {
            return Ok(0);
        }
        let mut step = Self::step_args(args.mu, args.grad_scale, 0.0, 0.0, 1.0, 1.0, self.iterations.get(), args.nesterov);
        step.variance_adaptive = args.variance_adaptive;
        step.bias_correction_inv = args.bias_correction_inv;
        check(unsafe { b2_muon_prepare_polar(self.plan.raw, ptr(args.slots), &step, args.stream.cu_stream()) })?;
        check(unsafe { b2_muon_polar(self.plan.raw, &step, args.stream.cu_stream()) })?;
        Ok(0)
    }
    /// launcher/muon_mega.rs:117-137: the same stage; the cooperative form is the reference's own cross-check.
    pub fn muon_tma_prepare_polar_cooperative_reference(&self, args: MuonTmaPrepareArgs<'_>) -> Result<(), DriverError> {
        self.muon_tma_prepare_polar(args).map(|_| ())
    }

    /// launcher/muon_mega.rs:139-157 (NorMuon scaling, master update, requantisation of x').
    pub fn muon_tma_finish_update(&self, args: MuonTmaFinishArgs<'_>) -> Result<(), DriverError> {
        if args.slot_index != self.plan.first_slot {
            return Ok(());
        }
        if args.apply_polar_sqrt_bound != 0 {
            return Err(DriverError(B2_ERROR_INVALID_VALUE as u32)); // belongs to the NVFP4-precision loop: not built
        }
        let step = self.finish_args(&args, 1);
        check(unsafe { b2_muon_finish_update(self.plan.raw, ptr(args.slots), &step, args.stream.cu_stream()) })
    }
    /// `muon_tma_finish_update` for the slots of one finish group (multi-GPU steps gather a group's packed weights
    /// while the next group is updated); called once per group, whatever `args.slot_index` is.
    pub fn muon_tma_finish_update_group(&self, args: MuonTmaFinishArgs<'_>, group: u32) -> Result<(), DriverError> {
        if args.apply_polar_sqrt_bound != 0 {
            return Err(DriverError(B2_ERROR_INVALID_VALUE as u32));
        }
        let step = self.finish_args(&args, 0);
        check(unsafe { b2_muon_finish_update_group(self.plan.raw, ptr(args.slots), &step, group, args.stream.cu_stream()) })
    }
    /// launcher/muon_mega.rs:159-165
    pub fn muon_tma_finish_update_deferred_quantization(&self, args: MuonTmaFinishArgs<'_>) -> Result<(), DriverError> {
        if args.slot_index != self.plan.first_slot {
            return Ok(());
        }
        if args.apply_polar_sqrt_bound != 0 {
            return Err(DriverError(B2_ERROR_INVALID_VALUE as u32));
        }
        let step = self.finish_args(&args, 1);
        check(unsafe {
            b2_muon_finish_update_deferred_quantization(self.plan.raw, ptr(args.slots), &step, args.stream.cu_stream())
        })
    }
    /// launcher/muon_mega.rs:468-518: the cooperative finish (no NorMuon) the reference keeps as a cross-check.
    pub fn muon_tma_finish_update_cooperative_reference(&self, args: MuonTmaFinishArgs<'_>) -> Result<(), DriverError> {
        if args.slot_index != self.plan.first_slot {
            return Ok(());
        }
        let step = self.finish_args(&args, 0);
        check(unsafe { b2_muon_finish_update(self.plan.raw, ptr(args.slots), &step, args.stream.cu_stream()) })
    }
    /// launcher/muon_mega.rs:166-228
    pub fn muon_tma_finish_hyperball_update_deferred_quantization(&self, args: MuonTmaHyperballFinishArgs<'_>)
                                                                  -> Result<(), DriverError> {
        if args.finish.slot_index != self.plan.first_slot {
            return Ok(());
        }
        let step = self.finish_args(&args.finish, 1);
        check(unsafe {
            b2_muon_finish_hyperball_update_deferred_quantization(self.plan.raw, ptr(args.finish.slots), &step,
                                                                  args.use_schedule_free as u32,
                                                                  args.finish.stream.cu_stream())
        })
    }
    /// launcher/muon_mega.rs:229-283
    pub fn muon_tma_sign_update_deferred_quantization(&self, args: MuonTmaSignUpdateArgs<'_>) -> Result<(), DriverError> {
        if args.slot_index != self.plan.first_slot {
            return Ok(());
        }
        let mut step = Self::step_args(args.mu, args.grad_scale, args.learning_rate, args.weight_decay,
                                       args.average_coefficient, args.schedule_beta, self.iterations.get(), 1);
        step.variance_adaptive = args.variance_adaptive;
        step.d_qk_clip_factors = if args.qk_clip_factors.is_empty() { 0 } else { ptr(args.qk_clip_factors) };
        step.symexp_lin_beta = args.symexp_lin_beta;
        step.d_symexp_lin_slots = if args.symexp_lin_slots.is_empty() { 0 } else { ptr(args.symexp_lin_slots) };
        check(unsafe {
            b2_muon_sign_update_deferred_quantization(self.plan.raw, ptr(args.slots), &step, args.stream.cu_stream())
        })
    }
    /// `Materializer::muon_precomputed` for every matrix at once (src/training/schedule_free/tensor.rs:128-153).
    pub fn muon_materialize_training_weights(&self, stream: &CudaStream,
                                             slots: &DeviceBuffer<MuonSlotDescriptor>) -> Result<(), DriverError> {
        check(unsafe { b2_muon_materialize_training_weights(self.plan.raw, ptr(slots), stream.cu_stream()) })
    }
    /// Stages Q1 + Q2 of every matrix after a deferred finish (.../muon/fused/quant/encode.rs:13-60).
    pub fn muon_materialize_master_weights(&self, stream: &CudaStream,
                                           slots: &DeviceBuffer<MuonSlotDescriptor>) -> Result<(), DriverError> {
        check(unsafe { b2_muon_materialize_master_weights(self.plan.raw, ptr(slots), stream.cu_stream()) })
    }

    fn sf_args(bytes: CUdeviceptr, scales: CUdeviceptr, global_scale: CUdeviceptr, z_master: CUdeviceptr,
               x_master: CUdeviceptr, precomputed_values: CUdeviceptr, amax: CUdeviceptr, len: u32, scale_rows: u32,
               scale_k: u32, beta: f32, symexp_lin_beta: f32, scale_layout: u32,
               refs: Option<SymExpLinScaleRefs<'_>>) -> b2_schedule_free_materialize_args {
        let symexp_lin_scales = match refs {
            Some(r) => [ptr(r.exponential_z), ptr(r.exponential_x), ptr(r.linear_z), ptr(r.linear_x), ptr(r.curvature_z),
                        ptr(r.curvature_x)],
            None => [0; 6],
        };
        b2_schedule_free_materialize_args {
            bytes,
            scales,
            global_scale,
            z_master,
            x_master,
            precomputed_values,
            amax,
            len,
            scale_rows,
            scale_k,
            beta,
            symexp_lin_beta,
            scale_layout,
            symexp_lin_scales,
        }
    }
    /// launcher/update.rs:25-75
    pub fn materialize_schedule_free_precomputed(&self, args: ScheduleFreeMaterializePrecomputedArgs<'_>)
                                                 -> Result<(), DriverError> {
        let a = Self::sf_args(ptr(args.bytes), ptr(args.scales), ptr(args.global_scale), ptr(args.z_master),
                              ptr(args.x_master), opt_ptr(args.precomputed_values), ptr(args.amax), args.len,
                              args.scale_rows, args.scale_k, args.beta, args.symexp_lin_beta, self.quant.scale_layout,
                              args.symexp_lin_scales);
        check(unsafe { b2_materialize_schedule_free_precomputed(&a, args.stream.cu_stream()) })
    }
    /// launcher/update.rs:77-133 (`chunk_amax` is not used: the maximum is raised with an atomic).
    pub fn materialize_schedule_free(&self, args: ScheduleFreeMaterializeArgs<'_>) -> Result<(), DriverError> {
        let a = Self::sf_args(ptr(args.bytes), ptr(args.scales), ptr(args.global_scale), ptr(args.z_master),
                              ptr(args.x_master), 0, ptr(args.amax), args.len, args.scale_rows, args.scale_k, args.beta,
                              args.symexp_lin_beta, self.quant.scale_layout, args.symexp_lin_scales);
        check(unsafe { b2_materialize_schedule_free(&a, args.stream.cu_stream()) })
    }

    fn adam_args(&self, a: &AdamWUpdateArgs<'_>) -> b2_adamw_update_args {
        b2_adamw_update_args {
            bytes: ptr(a.bytes),
            scales: ptr(a.scales),
            global_scale: ptr(a.global_scale),
            z_master: ptr(a.z_master),
            x_master: ptr(a.x_master),
            grad: ptr(a.grad),
            grad_scale: a.grad_scale,
            scale_layout: self.quant.scale_layout,
            first_moment: ptr(a.first_moment),
            second_moment: ptr(a.second_moment),
            amax: ptr(a.amax),
            chunk_amax: ptr(a.chunk_amax),
            len: a.len,
            learning_rate: a.learning_rate,
            weight_decay: a.weight_decay,
            beta1: a.beta1,
            beta2: a.beta2,
            beta1_correction: a.beta1_correction,
            beta2_correction: a.beta2_correction,
            eps: a.eps,
            average_coefficient: a.average_coefficient,
            schedule_beta: a.schedule_beta,
            d_grad_scale: 0,
        }
    }
    /// launcher/adam.rs:9-21
    pub fn apply_adamw_update(&self, args: AdamWUpdateArgs<'_>) -> Result<(), DriverError> {
        let a = self.adam_args(&args);
        check(unsafe { b2_apply_adamw_update(&a, args.stream.cu_stream()) })
    }
    /// launcher/adam.rs:23-28
    pub fn apply_adamw_update_deferred_quantization(&self, args: AdamWUpdateArgs<'_>) -> Result<(), DriverError> {
        let a = self.adam_args(&args);
        check(unsafe { b2_apply_adamw_update_deferred_quantization(&a, args.stream.cu_stream()) })
    }
    /// launcher/adam.rs:30-43
    pub fn zero_f32_pointer_table(&self, stream: &CudaStream, pointers: &DeviceBuffer<u64>,
                                  pointer_count: u32) -> Result<(), DriverError> {
        check(unsafe { b2_zero_f32_pointer_table(ptr(pointers), pointer_count, stream.cu_stream()) })
    }
    /// launcher/adam.rs:45-72
    pub fn apply_fp32_adamw_update(&self, args: Fp32AdamWUpdateArgs<'_>) -> Result<(), DriverError> {
        let a = b2_adamw_update_args {
            bytes: 0,
            scales: 0,
            global_scale: 0,
            z_master: ptr(args.z_master),
            x_master: ptr(args.x_master),
            grad: ptr(args.grad),
            grad_scale: args.grad_scale,
            scale_layout: self.quant.scale_layout,
            first_moment: ptr(args.first_moment),
            second_moment: ptr(args.second_moment),
            amax: 0,
            chunk_amax: 0,
            len: args.len,
            learning_rate: args.learning_rate,
            weight_decay: args.weight_decay,
            beta1: args.beta1,
            beta2: args.beta2,
            beta1_correction: args.beta1_correction,
            beta2_correction: args.beta2_correction,
            eps: args.eps,
            average_coefficient: args.average_coefficient,
            schedule_beta: 0.0,
            d_grad_scale: 0,
        };
        check(unsafe { b2_apply_fp32_adamw_update(&a, args.stream.cu_stream()) })
    }
    /// One launch for every AdamW tensor of a device-resident table (no single counterpart:
    /// src/training/optimizer_apply/adam.rs:18-157 loops over tensors).  `scalars` carries the hyper-parameters.
    pub fn apply_adamw_update_multi(&self, stream: &CudaStream, table: &DeviceBuffer<b2_adamw_slot_descriptor>,
                                    count: u32, total_chunks: u32,
                                    scalars: &b2_adamw_update_args) -> Result<(), DriverError> {
        check(unsafe { b2_apply_adamw_update_multi(ptr(table), count, total_chunks, scalars, stream.cu_stream()) })
    }
    /// `Materializer::adam` for every deferred tensor of the table (src/training/schedule_free/tensor.rs:71-89).
    pub fn adamw_materialize_training_weights(&self, stream: &CudaStream,
                                              table: &DeviceBuffer<b2_adamw_slot_descriptor>, count: u32,
                                              total_chunks: u32, schedule_beta: f32,
                                              values_cached: bool) -> Result<(), DriverError> {
        check(unsafe {
            b2_adamw_materialize_training_weights(ptr(table), count, total_chunks, schedule_beta, values_cached as i32,
                                                  stream.cu_stream())
        })
    }

    /// launcher/grad_clip.rs:9-50.  The scale stays on the device: hand `args.scale` to the step as
    /// `d_grad_scale` instead of reading it back.
    pub fn clip_gradients(&self, args: GradientClipArgs<'_>) -> Result<(), DriverError> {
        let a = b2_gradient_clip_args {
            chunk_ptrs: ptr(args.chunk_ptrs),
            chunk_lens: ptr(args.chunk_lens),
            chunk_sums: ptr(args.chunk_sums),
            extra_sums: if args.extra_sum_count == 0 { 0 } else { ptr(args.extra_sums) },
            scale: ptr(args.scale),
            norm: ptr(args.norm),
            chunk_count: args.chunk_count,
            extra_sum_count: args.extra_sum_count,
            max_norm: args.max_norm,
            apply: args.apply as u32,
        };
        check(unsafe { b2_clip_gradients(&a, args.stream.cu_stream()) })
    }

    /// launcher/symexp_lin.rs:9-22
    pub fn symexp_lin_zero_scale_grads(&self, stream: &CudaStream, slots: &DeviceBuffer<SymExpLinSlotDescriptor>,
                                       slot_count: u32) -> Result<(), DriverError> {
        check(unsafe { b2_symexp_lin_zero_scale_grads(ptr(slots), slot_count, stream.cu_stream()) })
    }
    /// launcher/symexp_lin.rs:24-59
    pub fn symexp_lin_scale_adamw_update(&self, stream: &CudaStream, slots: &DeviceBuffer<SymExpLinSlotDescriptor>,
                                         slot_count: u32, grad_scale: f32, exponential_linear_learning_rate: f32,
                                         curvature_learning_rate: f32, weight_decay: f32, beta1: f32, beta2: f32,
                                         beta1_correction: f32, beta2_correction: f32, eps: f32,
                                         average_coefficient: f32) -> Result<(), DriverError> {
        let a = b2_symexp_lin_adamw_args {
            grad_scale,
            exponential_linear_learning_rate,
            curvature_learning_rate,
            weight_decay,
            beta1,
            beta2,
            beta1_correction,
            beta2_correction,
            eps,
            average_coefficient,
        };
        check(unsafe { b2_symexp_lin_scale_adamw_update(ptr(slots), slot_count, &a, stream.cu_stream()) })
    }
    /// launcher/symexp_lin.rs:61-75
    pub fn symexp_lin_congruent_inverse_in_place(&self, stream: &CudaStream, raw: &mut DeviceBuffer<f32>,
                                                 beta: f32) -> Result<(), DriverError> {
        check(unsafe { b2_symexp_lin_congruent_inverse_in_place(ptr(raw), raw.len() as u32, beta, stream.cu_stream()) })
    }
}

// ---------------------------------------------------------------------------------------------------------
// host schedules (src/training/learning_rate/schedule.rs:24-65) and CSF helpers (utils/nvfp4/csf.rs)
// ---------------------------------------------------------------------------------------------------------
pub fn schedule_free_beta(step: u32, warmup_steps: u32, beta1: f32, rho: f32) -> f32 {
    unsafe { b2_schedule_free_beta(step, warmup_steps, beta1, rho) }
}
pub fn schedule_free_average_coefficient(step: u32, warmup_steps: u32, start_ratio: f32, weight_sum: &mut f32) -> f32 {
    unsafe { b2_schedule_free_average_coefficient(step, warmup_steps, start_ratio, weight_sum) }
}
pub fn warmup_multiplier(step: u32, warmup_steps: u32, start_ratio: f32) -> f32 {
    unsafe { b2_warmup_multiplier(step, warmup_steps, start_ratio) }
}
pub fn csf_encoded_len(rows: usize, k: usize) -> usize {
    unsafe { b2_csf_encoded_len(rows, k) }
}
pub fn csf_encode_host(raw: &[u8], rows: usize, k: usize) -> Vec<u8> {
    let mut out = vec![0u8; csf_encoded_len(rows, k)];
    let n = unsafe { b2_csf_encode_host(raw.as_ptr(), raw.len(), rows, k, out.as_mut_ptr(), out.len()) };
    assert!(n != 0, "csf_encode_host: k % 128, rows * k or the raw length violate csf.rs:36-49");
    out.truncate(n);
    out
}
pub fn csf_scale_at(encoded: &[u8], group: usize) -> u8 {
    unsafe { b2_csf_scale_at(encoded.as_ptr(), group) }
}
/// Whole-matrix shard plan for N ranks (no counterpart in the single-GPU reference).
pub fn shard_plan(rows: &[u32], cols: &[u32], world: u32) -> Result<(Vec<u32>, Vec<f64>), DriverError> {
    let mut owner = vec![0u32; rows.len()];
    let mut load = vec![0f64; world as usize];
    check(unsafe { b2_shard_plan(rows.as_ptr(), cols.as_ptr(), rows.len() as u32, world, owner.as_mut_ptr(), load.as_mut_ptr()) })?;
    Ok((owner, load))
}
