"""ctypes binding of libllmini_b200.so (the C ABI declared in include/llmini_b200.h).

The library is the product; this module only loads it and declares signatures.  There is no
fallback: if the shared object is missing or fails to load, importing raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libllmini_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "llmini_b200.h")

SCALES_CSF, SCALES_RAW, SCALES_SM100 = 0, 1, 2
OPERAND_BF16, OPERAND_F16 = 0, 1
QUANTIZE_X, QUANTIZE_Y = 0, 1
NORMALIZE_TWO_PASS, NORMALIZE_DEFERRED = 0, 1
NS_PER_PHASE, NS_CHAINED, NS_FUSED_GRAM_POLY = 0, 1, 2
UPDATE_F32, UPDATE_16BIT = 0, 1
ERROR_INVALID_VALUE, ERROR_NOT_SUPPORTED, ERROR_LAUNCH_TIMEOUT = 1, 801, 702


class MuonSlotDescriptor(C.Structure):
    """`MuonSlotDescriptor` (crates/cuda-kernels/src/gpt/optimizer/args/muon.rs:3-21), 104 bytes."""
    _fields_ = [
        ("grad", C.c_uint64), ("momentum", C.c_uint64), ("variance", C.c_uint64),
        ("second_momentum", C.c_uint64), ("z_master", C.c_uint64), ("x_master", C.c_uint64),
        ("schedule_amax", C.c_uint64), ("bytes", C.c_uint64), ("scales", C.c_uint64),
        ("global_scale", C.c_uint64), ("rows", C.c_uint32), ("cols", C.c_uint32),
        ("learning_rate_multiplier", C.c_float), ("qk_clip_factor_offset", C.c_uint32),
        ("qk_clip_head_dim", C.c_uint32), ("reserved_padding", C.c_uint32),
    ]


class MuonOptions(C.Structure):
    _fields_ = [("operand_format", C.c_uint32), ("scale_layout", C.c_uint32), ("quantize_target", C.c_uint32),
                ("max_iterations", C.c_uint32), ("tile_override", C.c_uint32), ("measure_phase_mask", C.c_uint32),
                ("measure_flags", C.c_uint32), ("normalize_mode", C.c_uint32), ("ns_schedule", C.c_uint32),
                ("update_input", C.c_uint32), ("reserved", C.c_uint32 * 2)]


class MuonStepArgs(C.Structure):
    _fields_ = [("mu", C.c_float), ("grad_scale", C.c_float), ("learning_rate", C.c_float),
                ("weight_decay", C.c_float), ("average_coefficient", C.c_float), ("schedule_beta", C.c_float),
                ("iterations", C.c_uint32), ("nesterov", C.c_uint32), ("coefficients", C.POINTER(C.c_float)),
                ("d_grad_scale", C.c_void_p), ("variance_adaptive", C.c_uint32), ("bias_correction_inv", C.c_float),
                ("d_qk_clip_factors", C.c_void_p), ("symexp_lin_beta", C.c_float),
                ("d_symexp_lin_slots", C.c_void_p), ("normuon", C.c_uint32), ("reserved_padding", C.c_uint32)]


class SymExpLinSlotDescriptor(C.Structure):
    """`SymExpLinSlotDescriptor` (args/symexp_lin.rs:5-26), 152 bytes."""
    _fields_ = [(n, C.c_uint64) for n in (
        "grad", "z_master", "x_master", "exponential_z", "exponential_x", "exponential_grad", "exponential_first",
        "exponential_second", "linear_z", "linear_x", "linear_grad", "linear_first", "linear_second", "curvature_z",
        "curvature_x", "curvature_grad", "curvature_first", "curvature_second")] + [("rows", C.c_uint32), ("cols", C.c_uint32)]


class SymExpLinAdamWArgs(C.Structure):
    _fields_ = [(n, C.c_float) for n in (
        "grad_scale", "exponential_linear_learning_rate", "curvature_learning_rate", "weight_decay", "beta1", "beta2",
        "beta1_correction", "beta2_correction", "eps", "average_coefficient")]


class ScheduleFreeMaterializeArgs(C.Structure):
    _fields_ = [("bytes", C.c_void_p), ("scales", C.c_void_p), ("global_scale", C.c_void_p),
                ("z_master", C.c_void_p), ("x_master", C.c_void_p), ("precomputed_values", C.c_void_p),
                ("amax", C.c_void_p), ("len", C.c_uint32), ("scale_rows", C.c_uint32), ("scale_k", C.c_uint32),
                ("beta", C.c_float), ("symexp_lin_beta", C.c_float), ("scale_layout", C.c_uint32),
                ("symexp_lin_scales", C.c_void_p * 6)]


class AdamWUpdateArgs(C.Structure):
    _fields_ = [("bytes", C.c_void_p), ("scales", C.c_void_p), ("global_scale", C.c_void_p),
                ("z_master", C.c_void_p), ("x_master", C.c_void_p), ("grad", C.c_void_p),
                ("grad_scale", C.c_float), ("scale_layout", C.c_uint32),
                ("first_moment", C.c_void_p), ("second_moment", C.c_void_p), ("amax", C.c_void_p),
                ("chunk_amax", C.c_void_p), ("len", C.c_uint32), ("learning_rate", C.c_float),
                ("weight_decay", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("beta1_correction", C.c_float), ("beta2_correction", C.c_float), ("eps", C.c_float),
                ("average_coefficient", C.c_float), ("schedule_beta", C.c_float), ("d_grad_scale", C.c_void_p)]


class AdamWSlotDescriptor(C.Structure):
    _fields_ = [("z_master", C.c_uint64), ("x_master", C.c_uint64), ("grad", C.c_uint64),
                ("first_moment", C.c_uint64), ("second_moment", C.c_uint64), ("amax", C.c_uint64),
                ("bytes", C.c_uint64), ("scales", C.c_uint64), ("global_scale", C.c_uint64),
                ("len", C.c_uint32), ("chunk_begin", C.c_uint32), ("mode", C.c_uint32), ("scale_layout", C.c_uint32)]


MAX_PEERS = 16


class PeerGroup(C.Structure):
    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("arena_bytes", C.c_uint64),
                ("base", C.c_uint64 * MAX_PEERS)]


class GradientClipArgs(C.Structure):
    _fields_ = [("chunk_ptrs", C.c_void_p), ("chunk_lens", C.c_void_p), ("chunk_sums", C.c_void_p),
                ("extra_sums", C.c_void_p), ("scale", C.c_void_p), ("norm", C.c_void_p),
                ("chunk_count", C.c_uint32), ("extra_sum_count", C.c_uint32), ("max_norm", C.c_float),
                ("apply", C.c_uint32)]


def declared_symbols() -> list[str]:
    """Names of every function the public header declares."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def _declare(L: C.CDLL) -> None:
    vp, u32, u64, f32, sz, i = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_size_t, C.c_int
    u32p, f32p, u8p = C.POINTER(C.c_uint32), C.POINTER(C.c_float), C.POINTER(C.c_uint8)
    sig = {
        "b2_abi_version": (u32, []),
        "b2_error_string": (C.c_char_p, [i]),
        "b2_verify_storage_layout": (i, [vp]),
        "b2_muon_workspace_bytes": (sz, [u32p, u32p, u32, C.POINTER(MuonOptions)]),
        "b2_muon_plan_create": (i, [C.POINTER(vp), u32p, u32p, u32, C.POINTER(MuonOptions), vp, sz, vp]),
        "b2_muon_plan_destroy": (None, [vp]),
        "b2_muon_mega_update": (i, [vp, vp, C.POINTER(MuonStepArgs), vp]),
        "b2_muon_prepare_polar": (i, [vp, vp, C.POINTER(MuonStepArgs), vp]),
        "b2_muon_polar": (i, [vp, C.POINTER(MuonStepArgs), vp]),
        "b2_muon_finish_update": (i, [vp, vp, C.POINTER(MuonStepArgs), vp]),
        "b2_muon_finish_update_deferred_quantization": (i, [vp, vp, C.POINTER(MuonStepArgs), vp]),
        "b2_muon_plan_set_finish_groups": (i, [vp, C.POINTER(C.c_uint32), C.c_uint32, vp]),
        "b2_muon_finish_update_group": (i, [vp, vp, C.POINTER(MuonStepArgs), C.c_uint32, vp]),
        "b2_muon_finish_hyperball_update_deferred_quantization": (i, [vp, vp, C.POINTER(MuonStepArgs), C.c_uint32, vp]),
        "b2_muon_sign_update_deferred_quantization": (i, [vp, vp, C.POINTER(MuonStepArgs), vp]),
        "b2_nvfp4_sm100_scales_bytes": (C.c_size_t, [C.c_uint32, C.c_uint32]),
        "b2_nvfp4_scales_to_sm100": (i, [vp, C.c_uint32, C.c_uint32, C.c_uint32, vp, vp]),
        "b2_symexp_lin_zero_scale_grads": (i, [vp, C.c_uint32, vp]),
        "b2_symexp_lin_scale_adamw_update": (i, [vp, C.c_uint32, C.POINTER(SymExpLinAdamWArgs), vp]),
        "b2_symexp_lin_congruent_inverse_in_place": (i, [vp, C.c_uint32, C.c_float, vp]),
        "b2_muon_plan_scratch": (i, [vp, u32, u32, C.POINTER(vp), C.POINTER(sz)]),
        "b2_muon_plan_status": (i, [vp, vp]),
        "b2_muon_plan_flops_per_iteration": (C.c_double, [vp]),
        "b2_tensor_amax_f32": (i, [vp, vp, vp, u32, vp]),
        "b2_tensor_amax_from_chunks_f32": (i, [vp, vp, u32, vp]),
        "b2_fp32_to_nvfp4_four_six": (i, [vp, vp, vp, vp, vp, u32, u32, vp]),
        "b2_materialize_master": (i, [vp, vp, vp, vp, vp, vp, u32, u32, vp]),
        "b2_materialize_master_static": (i, [vp, vp, vp, vp, u32, u32, vp]),
        "b2_materialize_schedule_free": (i, [C.POINTER(ScheduleFreeMaterializeArgs), vp]),
        "b2_materialize_schedule_free_precomputed": (i, [C.POINTER(ScheduleFreeMaterializeArgs), vp]),
        "b2_apply_adamw_update": (i, [C.POINTER(AdamWUpdateArgs), vp]),
        "b2_apply_adamw_update_deferred_quantization": (i, [C.POINTER(AdamWUpdateArgs), vp]),
        "b2_apply_fp32_adamw_update": (i, [C.POINTER(AdamWUpdateArgs), vp]),
        "b2_zero_f32_pointer_table": (i, [vp, u32, vp]),
        "b2_clip_gradients": (i, [C.POINTER(GradientClipArgs), vp]),
        "b2_adamw_table_prepare": (i, [C.POINTER(AdamWSlotDescriptor), u32, u32p]),
        "b2_apply_adamw_update_multi": (i, [vp, u32, u32, C.POINTER(AdamWUpdateArgs), vp]),
        "b2_adamw_materialize_training_weights": (i, [vp, u32, u32, C.c_float, C.c_int, vp]),
        "b2_muon_materialize_training_weights": (i, [vp, vp, vp]),
        "b2_muon_materialize_master_weights": (i, [vp, vp, vp]),
        "b2_csf_encoded_len": (sz, [sz, sz]),
        "b2_csf_encode_host": (sz, [u8p, sz, sz, sz, u8p, sz]),
        "b2_csf_scale_at": (C.c_uint8, [u8p, sz]),
        "b2_schedule_free_beta": (f32, [u32, u32, f32, f32]),
        "b2_schedule_free_average_coefficient": (f32, [u32, u32, f32, f32p]),
        "b2_warmup_multiplier": (f32, [u32, u32, f32]),
        "b2_shard_plan": (i, [u32p, u32p, u32, u32, u32p, C.POINTER(C.c_double)]),
        "b2_comm_unique_id": (i, [u8p]),
        "b2_comm_create": (i, [C.POINTER(vp), u8p, i, i]),
        "b2_comm_destroy": (None, [vp]),
        "b2_allgather_nvfp4": (i, [vp, vp, sz, vp]),
        "b2_peer_buffer_alloc": (i, [sz, C.POINTER(vp), u8p]),
        "b2_peer_buffer_open": (i, [u8p, C.POINTER(vp)]),
        "b2_peer_buffer_close": (i, [vp]),
        "b2_peer_buffer_free": (i, [vp]),
        "b2_peer_push": (i, [C.POINTER(PeerGroup), sz, sz, u32, vp]),
        "b2_peer_wait": (i, [C.POINTER(PeerGroup), u64, vp]),
        "b2_peer_status": (i, [C.POINTER(PeerGroup), vp]),
        "b2_debug_muon_fused_wait_expiry": (i, [vp, vp, u32, u64, vp]),
        "b2_debug_rcp_approx_ftz": (i, [vp, vp, u32, vp]),
        "b2_debug_quantize_literal": (i, [vp, vp, vp, vp, vp, u32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m llmini_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        L = C.CDLL(LIB_PATH)
        _declare(L)
        _lib = L
    return _lib


class B2Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().b2_error_string(code)
        super().__init__(f"{where}: error {code} ({msg.decode() if msg else '?'})")


def check(code: int, where: str) -> None:
    if code != 0:
        raise B2Error(code, where)
