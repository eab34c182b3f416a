"""Host mirror of the reference's `Nvfp4QuantModule` and CSF helpers over the C ABI.

Reference interface: crates/cuda-kernels/src/utils/nvfp4/quant/{launcher,amax,four_six}.rs,
crates/cuda-kernels/src/utils/nvfp4/csf.rs, and the `Nvfp4Tensor` triple
(crates/gpt2-nvfp4/src/tensor/nvfp4.rs:17-21).  Tensors are torch CUDA tensors used purely as
device buffers.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _ffi
from ._ffi import SCALES_CSF, SCALES_RAW, SCALES_SM100, check


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor) -> int:
    assert t.is_cuda and t.is_contiguous()
    return t.data_ptr()


# ---- CSF host helpers ---------------------------------------------------------------------
def csf_encoded_len(rows: int, k: int) -> int:
    """`csf::encoded_len` (csf.rs:8-17)."""
    return int(_ffi.lib().b2_csf_encoded_len(rows, k))


def csf_encode_host(raw, rows: int, k: int) -> np.ndarray:
    """`csf::encode_host` (csf.rs:36-44); raises where the reference asserts."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    cap = 128 + ((rows + 127) // 128) * ((k + 127) // 128) * 1024 + k // 16
    out = np.zeros(cap, dtype=np.uint8)
    u8p = C.POINTER(C.c_uint8)
    n = _ffi.lib().b2_csf_encode_host(raw.ctypes.data_as(u8p), raw.size, rows, k, out.ctypes.data_as(u8p), cap)
    if n == 0:
        raise ValueError("csf_encode_host: precondition violated (k % 128, rows * k, raw length)")
    return out[:n].copy()


def csf_scale_at(encoded: np.ndarray, group: int) -> int:
    """`csf::scale_at` (csf.rs:139-147)."""
    encoded = np.ascontiguousarray(encoded, dtype=np.uint8)
    return int(_ffi.lib().b2_csf_scale_at(encoded.ctypes.data_as(C.POINTER(C.c_uint8)), group))


def zero_scales(rows: int, k: int, device="cuda") -> torch.Tensor:
    """Pre-headed CSF scale storage, as the reference's fixtures build it
    (crates/cuda-kernels/tests/optimizer/muon/buffers.rs:135-142)."""
    enc = csf_encode_host(np.zeros(rows * k // 16, np.uint8), rows, k)
    return torch.from_numpy(enc).to(device)


def sm100_scales_bytes(rows: int, cols: int) -> int:
    """Bytes of the sm_100 block-scale operand layout of a [rows][cols] tensor (128 x 4 tiles, padded)."""
    return int(_ffi.lib().b2_nvfp4_sm100_scales_bytes(rows, cols))


def scales_to_sm100(scales: torch.Tensor, src_layout: int, rows: int, cols: int) -> torch.Tensor:
    """Block scales (raw plane or CSF storage, on the device) -> the layout `tcgen05.mma
    kind::mxf4nvf4.block_scale` operands use; every byte of the result is written."""
    out = torch.empty(sm100_scales_bytes(rows, cols), dtype=torch.uint8, device=scales.device)
    check(_ffi.lib().b2_nvfp4_scales_to_sm100(scales.data_ptr(), src_layout, rows, cols, out.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream), "nvfp4_scales_to_sm100")
    return out


@dataclass
class Nvfp4Tensor:
    """bytes (packed E2M1), scales (CSF or raw plane), global_scale f32[1]."""
    bytes: torch.Tensor
    scales: torch.Tensor
    global_scale: torch.Tensor
    rows: int
    k: int
    scale_layout: int = SCALES_CSF

    @staticmethod
    def empty(rows: int, k: int, scale_layout: int = SCALES_CSF, device="cuda") -> "Nvfp4Tensor":
        n = rows * k
        scales = zero_scales(rows, k, device) if scale_layout == SCALES_CSF else torch.zeros(n // 16, dtype=torch.uint8, device=device)
        return Nvfp4Tensor(torch.zeros(n // 2, dtype=torch.uint8, device=device), scales,
                           torch.zeros(1, dtype=torch.float32, device=device), rows, k, scale_layout)


class Nvfp4QuantModule:
    """`Nvfp4QuantModule` (crates/cuda-kernels/src/utils/nvfp4/quant/launcher.rs:7-16)."""

    def __init__(self):
        self._lib = _ffi.lib()

    def tensor_amax_f32(self, x: torch.Tensor, chunk_amax: torch.Tensor, out: torch.Tensor, element_count: int) -> None:
        assert chunk_amax.numel() >= (element_count + 2047) // 2048
        check(self._lib.b2_tensor_amax_f32(_ptr(x), _ptr(chunk_amax), _ptr(out), element_count, _stream()), "tensor_amax_f32")

    def tensor_amax_from_chunks_f32(self, chunk_amax: torch.Tensor, out: torch.Tensor, chunk_count: int) -> None:
        check(self._lib.b2_tensor_amax_from_chunks_f32(_ptr(chunk_amax), _ptr(out), chunk_count, _stream()),
              "tensor_amax_from_chunks_f32")

    def fp32_to_nvfp4_four_six(self, x: torch.Tensor, amax: torch.Tensor, out_fp4: torch.Tensor,
                               out_scales: torch.Tensor, out_global_scale: torch.Tensor, group_count: int,
                               scale_layout: int = SCALES_CSF) -> None:
        assert x.numel() >= group_count * 16 and out_fp4.numel() >= group_count * 8
        check(self._lib.b2_fp32_to_nvfp4_four_six(_ptr(x), _ptr(amax), _ptr(out_fp4), _ptr(out_scales),
                                                   _ptr(out_global_scale), group_count, scale_layout, _stream()),
              "fp32_to_nvfp4_four_six")

    # debug helpers used by the parity tests
    def debug_rcp_approx_ftz(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        check(self._lib.b2_debug_rcp_approx_ftz(_ptr(x), _ptr(out), x.numel(), _stream()), "debug_rcp")
        return out

    def debug_quantize_literal(self, x: torch.Tensor, amax: torch.Tensor):
        n = x.numel()
        fp4 = torch.zeros(n // 2, dtype=torch.uint8, device=x.device)
        sc = torch.zeros(n // 16, dtype=torch.uint8, device=x.device)
        gs = torch.zeros(1, dtype=torch.float32, device=x.device)
        check(self._lib.b2_debug_quantize_literal(_ptr(x), _ptr(amax), _ptr(fp4), _ptr(sc), _ptr(gs), n // 16, _stream()),
              "debug_quantize_literal")
        return fp4, sc, gs
