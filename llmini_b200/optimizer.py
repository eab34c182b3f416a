"""Host mirror of the reference's `OptimizerModule` hot-path methods over the C ABI.

Reference interface: crates/cuda-kernels/src/gpt/optimizer/launcher/{mod,muon_mega,update,adam}.rs
with argument structs in .../optimizer/args/{muon,schedule_free,adam}.rs.  Method and field
names follow the reference so its tests read the same here.  Tensors are torch CUDA tensors
used purely as device buffers; all arithmetic happens inside libllmini_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import _ffi
from ._ffi import (AdamWSlotDescriptor, AdamWUpdateArgs as _CAdam, GradientClipArgs as _CClip, MuonOptions, MuonSlotDescriptor, MuonStepArgs, OPERAND_BF16,
                   NORMALIZE_DEFERRED, NORMALIZE_TWO_PASS, NS_CHAINED, NS_FUSED_GRAM_POLY, NS_PER_PHASE, OPERAND_F16, UPDATE_16BIT, UPDATE_F32, QUANTIZE_X, QUANTIZE_Y, SCALES_CSF, SCALES_RAW, SCALES_SM100,
                   ScheduleFreeMaterializeArgs as _CSf, check)
from .nvfp4 import Nvfp4QuantModule, sm100_scales_bytes, zero_scales

U32_MAX = 0xFFFFFFFF


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> int:
    if t is None:
        return 0
    assert t.is_cuda and t.is_contiguous()
    return t.data_ptr()


@dataclass
class MuonSlot:
    """Device buffers of one matrix (the fields of `MuonSlotDescriptor`)."""
    grad: torch.Tensor           # f32 [rows, cols]; receives y
    momentum: torch.Tensor       # bf16 [rows, cols]
    z_master: torch.Tensor       # f32
    x_master: torch.Tensor       # f32
    schedule_amax: torch.Tensor  # f32[1]
    bytes: torch.Tensor          # u8 [len/2]
    scales: torch.Tensor         # u8 CSF (pre-headed) or raw plane
    global_scale: torch.Tensor   # f32[1]
    rows: int
    cols: int
    learning_rate_multiplier: float = 1.0
    variance: Optional[torch.Tensor] = None  # bf16 [rows, cols], Muon-VS only
    second_momentum: Optional[torch.Tensor] = None  # f32 [max(rows, cols)], NorMuon / Hyperball only
    qk_clip_factor_offset: int = U32_MAX
    qk_clip_head_dim: int = 0

    @staticmethod
    def allocate(rows: int, cols: int, scale_layout: int = SCALES_CSF, device="cuda") -> "MuonSlot":
        n = rows * cols
        if n == 0:  # padding slot: skipped by every kernel
            scales = torch.zeros(1, dtype=torch.uint8, device=device)
        elif scale_layout == SCALES_CSF:
            if cols % 128 != 0:
                raise ValueError("CSF block-scale storage needs cols % 128 == 0; use SCALES_RAW")
            scales = zero_scales(rows, cols, device)
        elif scale_layout == SCALES_SM100:  # padding bytes stay zero: the kernels never write them
            scales = torch.zeros(sm100_scales_bytes(rows, cols), dtype=torch.uint8, device=device)
        else:
            scales = torch.zeros(max(n // 16, 1), dtype=torch.uint8, device=device)
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)
        return MuonSlot(z(rows, cols), z(rows, cols, dt=torch.bfloat16), z(rows, cols), z(rows, cols), z(1),
                        torch.zeros(max(n // 2, 1), dtype=torch.uint8, device=device), scales, z(1), rows, cols)

    def descriptor(self) -> MuonSlotDescriptor:
        return MuonSlotDescriptor(_ptr(self.grad), _ptr(self.momentum), _ptr(self.variance),
                                  _ptr(self.second_momentum), _ptr(self.z_master),
                                  _ptr(self.x_master), _ptr(self.schedule_amax), _ptr(self.bytes), _ptr(self.scales),
                                  _ptr(self.global_scale), self.rows, self.cols, self.learning_rate_multiplier,
                                  self.qk_clip_factor_offset, self.qk_clip_head_dim, 0)


def slot_table(slots: Sequence[MuonSlot], device="cuda") -> torch.Tensor:
    """Device-resident `MuonSlotDescriptor` table (104 bytes per entry)."""
    arr = (MuonSlotDescriptor * len(slots))(*[s.descriptor() for s in slots])
    host = np.frombuffer(bytes(arr), dtype=np.uint8).copy()
    return torch.from_numpy(host).to(device)


@dataclass
class MuonMegaUpdateArgs:
    """`MuonMegaUpdateArgs` (args/muon.rs:25-44) minus the scratch buffers, which the plan owns."""
    mu: float = 0.95
    grad_scale: float = 1.0
    learning_rate: float = 1.0e-4
    weight_decay: float = 0.025
    average_coefficient: float = 1.0
    iterations: int = 5
    schedule_beta: float = 1.0
    nesterov: bool = True
    coefficients: Optional[np.ndarray] = None  # iterations x 3; None = reference table
    grad_scale_device: Optional[torch.Tensor] = None  # f32[1] on the device; replaces grad_scale
    variance_adaptive: bool = False                    # Muon-VS; slots need a `variance` buffer
    bias_correction_inv: float = 1.0
    qk_clip_factors: Optional[torch.Tensor] = None     # f32 per-head factors on the device
    normuon: bool = False                              # slots need a `second_momentum` buffer
    symexp_lin_beta: float = 0.0                       # > 0: SymExpLin forward on y
    symexp_lin_slots: Optional[torch.Tensor] = None    # device table of SymExpLinSlotDescriptor, or None

    def c_args(self):
        co = None
        keep = None
        if self.coefficients is not None:
            keep = np.ascontiguousarray(self.coefficients, dtype=np.float32).reshape(-1)
            assert keep.size >= 3 * self.iterations
            co = keep.ctypes.data_as(C.POINTER(C.c_float))
        a = MuonStepArgs(self.mu, self.grad_scale, self.learning_rate, self.weight_decay, self.average_coefficient,
                         self.schedule_beta, self.iterations, int(self.nesterov), co, _ptr(self.grad_scale_device),
                         int(self.variance_adaptive), self.bias_correction_inv, _ptr(self.qk_clip_factors),
                         self.symexp_lin_beta, _ptr(self.symexp_lin_slots), int(self.normuon), 0)
        return a, keep


class MuonPlan:
    """Shapes-only plan: workspace, tile lists and TMA descriptors for a fixed slot list."""

    def __init__(self, shapes: Sequence[tuple[int, int]], operand_format: int = OPERAND_BF16,
                 scale_layout: int = SCALES_CSF, quantize_target: int = QUANTIZE_X, max_iterations: int = 5,
                 tile_n: int = 0, device="cuda", debug_phase_mask: int = 0, debug_flags: int = 0,
                 normalize_mode: int = NORMALIZE_TWO_PASS, ns_schedule: int = NS_PER_PHASE,
                 update_input: int = UPDATE_F32):
        """`normalize_mode`: NORMALIZE_TWO_PASS keeps the reference's rounding point X0 = r16(u * s);
        NORMALIZE_DEFERRED reads the gradients once and lets s enter through the first iteration (BF16
        operands only).  `ns_schedule`: NS_PER_PHASE runs three launches per iteration, NS_CHAINED the whole
        Newton-Schulz loop as one persistent grid ordered by per-matrix progress counts (steps of exactly
        `max_iterations` iterations), NS_FUSED_GRAM_POLY two launches per iteration, the Gram and polynomial tile of a
        position computed by one CTA pair with the FP32 Gram tile kept in tensor memory.  `update_input`: UPDATE_16BIT lets the last iteration store the 16-bit operand type instead of
        FP32 and the update read that (plain finish only).  `debug_*` are read only by a library built with -DB2_MEASURE."""
        self._lib = _ffi.lib()
        self.shapes = [(int(r), int(c)) for r, c in shapes]
        n = len(self.shapes)
        self._rows = (C.c_uint32 * n)(*[r for r, _ in self.shapes])
        self._cols = (C.c_uint32 * n)(*[c for _, c in self.shapes])
        self.options = MuonOptions(operand_format, scale_layout, quantize_target, max_iterations, tile_n, debug_phase_mask, debug_flags, normalize_mode, ns_schedule,
                                   update_input, (C.c_uint32 * 2)())
        nbytes = self._lib.b2_muon_workspace_bytes(self._rows, self._cols, n, C.byref(self.options))
        if nbytes == 0:
            raise _ffi.B2Error(_ffi.ERROR_INVALID_VALUE, "muon_workspace_bytes")
        self.workspace_bytes = int(nbytes)
        # torch's caching allocator returns 512-byte aligned blocks; over-allocate and align to 1 KiB
        self._buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        base = (self._buf.data_ptr() + 1023) // 1024 * 1024
        self._handle = C.c_void_p()
        check(self._lib.b2_muon_plan_create(C.byref(self._handle), self._rows, self._cols, n, C.byref(self.options),
                                            base, nbytes, _stream()), "muon_plan_create")

    def close(self):
        if getattr(self, "_handle", None) and self._handle.value:
            torch.cuda.synchronize()
            self._lib.b2_muon_plan_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._handle

    def flops_per_iteration(self) -> float:
        return float(self._lib.b2_muon_plan_flops_per_iteration(self._handle))

    def status(self) -> int:
        return int(self._lib.b2_muon_plan_status(self._handle, _stream()))

    def set_finish_groups(self, first_slots: Sequence[int]) -> None:
        """Cuts the plan's slots into contiguous runs starting at `first_slots` (first entry 0, ascending; a run
        may be empty) for OptimizerModule.muon_tma_finish_update_group (b2_muon_plan_set_finish_groups)."""
        arr = (C.c_uint32 * len(first_slots))(*[int(v) for v in first_slots])
        check(self._lib.b2_muon_plan_set_finish_groups(self._handle, arr, len(first_slots), _stream()),
              "muon_plan_set_finish_groups")

    def debug_fused_wait_expiry(self, slots: torch.Tensor, slot: int, wait_ns: int) -> None:
        """Test hook: one CTA of the update + encode launch waits `wait_ns` for a completion count that cannot
        arrive, gives up and reports through the status word (b2_debug_muon_fused_wait_expiry)."""
        check(self._lib.b2_debug_muon_fused_wait_expiry(self._handle, _ptr(slots), slot, wait_ns, _stream()),
              "debug_muon_fused_wait_expiry")

    def scratch(self, slot: int, which: int) -> torch.Tensor:
        """View of a scratch buffer as a torch tensor (see b2_muon_plan_scratch)."""
        p, n = C.c_void_p(), C.c_size_t()
        check(self._lib.b2_muon_plan_scratch(self._handle, slot, which, C.byref(p), C.byref(n)), "muon_plan_scratch")
        off = p.value - self._buf.data_ptr()
        raw = self._buf[off:off + n.value]
        rows, cols = self.shapes[slot] if which not in (4, 10, 11) else (0, 0)
        if which in (0, 7):
            dt = torch.float16 if self.options.operand_format == OPERAND_F16 else torch.bfloat16
            return raw.view(dt).view(rows, cols)
        if which == 1:
            return raw.view(torch.float32).view(rows, cols)
        if which in (5, 6):
            dt = torch.float16 if self.options.operand_format == OPERAND_F16 else torch.bfloat16
            n_ = min(rows, cols)
            return raw.view(dt).view(n_, -1)[:, :n_]
        if which in (4, 10, 11):
            return raw.view(torch.int32)
        return raw.view(torch.float32)


class OptimizerModule:
    """`OptimizerModule` (crates/cuda-kernels/src/gpt/optimizer/launcher/mod.rs:20-26)."""

    def __init__(self):
        self._lib = _ffi.lib()
        self.quant = Nvfp4QuantModule()

    # launcher/mod.rs:43-56
    def verify_storage_layout(self) -> None:
        check(self._lib.b2_verify_storage_layout(_stream()), "verify_storage_layout")

    # launcher/muon_mega.rs:24-51
    def muon_mega_update(self, plan: MuonPlan, slots: torch.Tensor, args: MuonMegaUpdateArgs) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_mega_update(plan.handle, _ptr(slots), C.byref(a), _stream()), "muon_mega_update")
        del keep

    # launcher/muon_mega.rs:53-115
    def muon_tma_prepare_polar(self, plan: MuonPlan, slots: torch.Tensor, args: MuonMegaUpdateArgs) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_prepare_polar(plan.handle, _ptr(slots), C.byref(a), _stream()), "muon_prepare_polar")
        del keep

    def muon_polar(self, plan: MuonPlan, args: MuonMegaUpdateArgs) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_polar(plan.handle, C.byref(a), _stream()), "muon_polar")
        del keep

    # launcher/muon_mega.rs:139-157
    def muon_tma_finish_update(self, plan: MuonPlan, slots: torch.Tensor, args: MuonMegaUpdateArgs) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_finish_update(plan.handle, _ptr(slots), C.byref(a), _stream()), "muon_finish_update")
        del keep

    def muon_tma_finish_update_group(self, plan: MuonPlan, slots: torch.Tensor, args: MuonMegaUpdateArgs,
                                     group: int) -> None:
        """muon_tma_finish_update for the slots of one finish group of the plan (MuonPlan.set_finish_groups)."""
        a, keep = args.c_args()
        check(self._lib.b2_muon_finish_update_group(plan.handle, _ptr(slots), C.byref(a), int(group), _stream()),
              "muon_finish_update_group")
        del keep

    # launcher/muon_mega.rs:159-165
    def muon_tma_finish_update_deferred_quantization(self, plan: MuonPlan, slots: torch.Tensor,
                                                     args: MuonMegaUpdateArgs) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_finish_update_deferred_quantization(plan.handle, _ptr(slots), C.byref(a), _stream()),
              "muon_finish_update_deferred_quantization")
        del keep

    # stages Q1 + Q2 of every matrix from x' and the max|x'| the last finish left in the plan
    def muon_materialize_master_weights(self, plan: MuonPlan, slots: torch.Tensor) -> None:
        check(self._lib.b2_muon_materialize_master_weights(plan.handle, _ptr(slots), _stream()),
              "muon_materialize_master_weights")

    # launcher/muon_mega.rs:166-228
    def muon_tma_finish_hyperball_update_deferred_quantization(self, plan: MuonPlan, slots: torch.Tensor,
                                                               args: MuonMegaUpdateArgs,
                                                               use_schedule_free: bool = True) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_finish_hyperball_update_deferred_quantization(
            plan.handle, _ptr(slots), C.byref(a), int(use_schedule_free), _stream()), "muon_finish_hyperball_update")
        del keep

    # launcher/muon_mega.rs:229-283
    def muon_tma_sign_update_deferred_quantization(self, plan: MuonPlan, slots: torch.Tensor,
                                                   args: MuonMegaUpdateArgs) -> None:
        a, keep = args.c_args()
        check(self._lib.b2_muon_sign_update_deferred_quantization(plan.handle, _ptr(slots), C.byref(a), _stream()),
              "muon_sign_update_deferred_quantization")
        del keep

    # launcher/mod.rs:67-95
    def materialize_master(self, bytes_: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                           master: torch.Tensor, amax: torch.Tensor, chunk_amax: torch.Tensor, len_: int,
                           scale_layout: int = SCALES_CSF) -> None:
        check(self._lib.b2_materialize_master(_ptr(bytes_), _ptr(scales), _ptr(global_scale), _ptr(master), _ptr(amax),
                                              _ptr(chunk_amax), len_, scale_layout, _stream()), "materialize_master")

    STATIC_MAX_ELEMENTS = 1 << 26

    def materialize_master_static(self, bytes_: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                                  master: torch.Tensor, len_: int, scale_layout: int = SCALES_CSF) -> None:
        """`materialize_master` for callers with no scratch to give and no way to allocate it (an
        export or evaluation hook that only holds the weight buffers): the chunk maxima and the
        tensor maximum live in an array inside the library, so `len_` is limited to
        STATIC_MAX_ELEMENTS and calls that may overlap on the GPU must be serialised."""
        check(self._lib.b2_materialize_master_static(_ptr(bytes_), _ptr(scales), _ptr(global_scale), _ptr(master),
                                                     len_, scale_layout, _stream()), "materialize_master_static")

    def _sf_args(self, *, bytes, scales, global_scale, z_master, x_master, amax, len, scale_rows, scale_k, beta,
                 symexp_lin_beta=0.0, symexp_lin_scales=None, precomputed_values=None, scale_layout=SCALES_CSF,
                 **_ignored):
        # symexp_lin_scales: `SymExpLinScaleRefs`, six f32[1] device tensors (exponential z, x; linear z, x;
        # curvature z, x), or None for unit scales
        ptrs = (C.c_void_p * 6)(*[_ptr(t) for t in (symexp_lin_scales or [None] * 6)])
        return _CSf(_ptr(bytes), _ptr(scales), _ptr(global_scale), _ptr(z_master), _ptr(x_master),
                    _ptr(precomputed_values), _ptr(amax), len, scale_rows, scale_k, beta, symexp_lin_beta, scale_layout,
                    ptrs)

    # launcher/update.rs:77-133
    def materialize_schedule_free(self, **kw) -> None:
        a = self._sf_args(**kw)
        check(self._lib.b2_materialize_schedule_free(C.byref(a), _stream()), "materialize_schedule_free")

    # launcher/update.rs:25-75
    def materialize_schedule_free_precomputed(self, **kw) -> None:
        a = self._sf_args(**kw)
        check(self._lib.b2_materialize_schedule_free_precomputed(C.byref(a), _stream()),
              "materialize_schedule_free_precomputed")

    def _adam_args(self, *, z_master, x_master, grad, grad_scale, first_moment, second_moment, len, learning_rate,
                   weight_decay, beta1, beta2, beta1_correction, beta2_correction, eps, average_coefficient,
                   schedule_beta=0.0, bytes=None, scales=None, global_scale=None, amax=None, chunk_amax=None,
                   scale_layout=SCALES_CSF, grad_scale_device=None):
        return _CAdam(_ptr(bytes), _ptr(scales), _ptr(global_scale), _ptr(z_master), _ptr(x_master), _ptr(grad),
                      grad_scale, scale_layout, _ptr(first_moment), _ptr(second_moment), _ptr(amax), _ptr(chunk_amax),
                      len, learning_rate, weight_decay, beta1, beta2, beta1_correction, beta2_correction, eps,
                      average_coefficient, schedule_beta, _ptr(grad_scale_device))

    # launcher/adam.rs:9-21
    def apply_adamw_update(self, **kw) -> None:
        a = self._adam_args(**kw)
        check(self._lib.b2_apply_adamw_update(C.byref(a), _stream()), "apply_adamw_update")

    # launcher/adam.rs:23-28
    def apply_adamw_update_deferred_quantization(self, **kw) -> None:
        a = self._adam_args(**kw)
        check(self._lib.b2_apply_adamw_update_deferred_quantization(C.byref(a), _stream()),
              "apply_adamw_update_deferred_quantization")

    # launcher/adam.rs:45-72
    def apply_fp32_adamw_update(self, **kw) -> None:
        a = self._adam_args(**kw)
        check(self._lib.b2_apply_fp32_adamw_update(C.byref(a), _stream()), "apply_fp32_adamw_update")

    def adamw_table(self, tensors: Sequence[dict], device="cuda"):
        """Builds the device table for `apply_adamw_update_multi` from dicts with the tensor fields
        of `AdamWUpdateArgs` plus `mode` (0 fp32 only, 1 deferred, 2 requantise).
        -> (device table tensor, count, total_chunks)."""
        n = len(tensors)
        arr = (AdamWSlotDescriptor * n)()
        for d, t in zip(arr, tensors):
            for k in ("z_master", "x_master", "grad", "first_moment", "second_moment", "amax", "bytes", "scales", "global_scale"):
                setattr(d, k, _ptr(t.get(k)))
            d.len, d.mode, d.scale_layout = t["len"], t.get("mode", 0), t.get("scale_layout", SCALES_CSF)
        total = C.c_uint32(0)
        check(self._lib.b2_adamw_table_prepare(arr, n, C.byref(total)), "adamw_table_prepare")
        host = np.frombuffer(bytes(arr), dtype=np.uint8).copy()
        return torch.from_numpy(host).to(device), n, int(total.value)

    def apply_adamw_update_multi(self, table: torch.Tensor, count: int, total_chunks: int, **scalars) -> None:
        a = self._adam_args(z_master=None, x_master=None, grad=None, first_moment=None, second_moment=None, len=0, **scalars)
        check(self._lib.b2_apply_adamw_update_multi(_ptr(table), count, total_chunks, C.byref(a), _stream()),
              "apply_adamw_update_multi")

    # Materializer::adam for all deferred tensors of the table (src/training/schedule_free/tensor.rs:71-89)
    def adamw_materialize_training_weights(self, table: torch.Tensor, count: int, total_chunks: int,
                                           schedule_beta: float, values_cached: bool = True) -> None:
        check(self._lib.b2_adamw_materialize_training_weights(_ptr(table), count, total_chunks, schedule_beta,
                                                              int(values_cached), _stream()),
              "adamw_materialize_training_weights")

    # Materializer::muon_precomputed for all matrices (src/training/schedule_free/tensor.rs:128-153)
    def muon_materialize_training_weights(self, plan: "MuonPlan", slots: torch.Tensor) -> None:
        check(self._lib.b2_muon_materialize_training_weights(plan.handle, _ptr(slots), _stream()),
              "muon_materialize_training_weights")

    # OptimizerModule::clip_gradients (args/grad_clip.rs:3-15)
    def clip_gradients(self, *, chunk_ptrs, chunk_lens, chunk_sums, extra_sums, scale, norm, chunk_count,
                       extra_sum_count, max_norm, apply) -> None:
        a = _CClip(_ptr(chunk_ptrs), _ptr(chunk_lens), _ptr(chunk_sums), _ptr(extra_sums), _ptr(scale), _ptr(norm),
                   chunk_count, extra_sum_count, max_norm, int(bool(apply)))
        check(self._lib.b2_clip_gradients(C.byref(a), _stream()), "clip_gradients")

    # launcher/symexp_lin.rs:9-75
    def symexp_lin_zero_scale_grads(self, slots: torch.Tensor, slot_count: int) -> None:
        check(self._lib.b2_symexp_lin_zero_scale_grads(_ptr(slots), slot_count, _stream()), "symexp_lin_zero_scale_grads")

    def symexp_lin_scale_adamw_update(self, slots: torch.Tensor, slot_count: int, grad_scale: float,
                                      exponential_linear_learning_rate: float, curvature_learning_rate: float,
                                      weight_decay: float, beta1: float, beta2: float, beta1_correction: float,
                                      beta2_correction: float, eps: float, average_coefficient: float) -> None:
        a = _ffi.SymExpLinAdamWArgs(grad_scale, exponential_linear_learning_rate, curvature_learning_rate, weight_decay,
                                    beta1, beta2, beta1_correction, beta2_correction, eps, average_coefficient)
        check(self._lib.b2_symexp_lin_scale_adamw_update(_ptr(slots), slot_count, C.byref(a), _stream()),
              "symexp_lin_scale_adamw_update")

    def symexp_lin_congruent_inverse_in_place(self, raw: torch.Tensor, beta: float) -> None:
        check(self._lib.b2_symexp_lin_congruent_inverse_in_place(_ptr(raw), raw.numel(), beta, _stream()),
              "symexp_lin_congruent_inverse_in_place")

    # launcher/adam.rs:30-43
    def zero_f32_pointer_table(self, pointers: torch.Tensor, pointer_count: int) -> None:
        check(self._lib.b2_zero_f32_pointer_table(_ptr(pointers), pointer_count, _stream()), "zero_f32_pointer_table")


# ---- host schedules (src/training/learning_rate/schedule.rs) ---------------------------------
def schedule_free_beta(step: int, warmup_steps: int = 5, beta1: float = 0.2, rho: float = 0.5) -> float:
    return float(_ffi.lib().b2_schedule_free_beta(step, warmup_steps, beta1, rho))


def warmup_multiplier(step: int, warmup_steps: int = 5, start_ratio: float = 0.05) -> float:
    return float(_ffi.lib().b2_warmup_multiplier(step, warmup_steps, start_ratio))


class AverageCoefficient:
    """Running `schedule_free_average_coefficient` (schedule.rs:36-47)."""

    def __init__(self, warmup_steps: int = 5, start_ratio: float = 0.05):
        self.warmup_steps, self.start_ratio = warmup_steps, start_ratio
        self._sum = C.c_float(0.0)

    def step(self, step: int) -> float:
        return float(_ffi.lib().b2_schedule_free_average_coefficient(step, self.warmup_steps, self.start_ratio,
                                                                     C.byref(self._sum)))
