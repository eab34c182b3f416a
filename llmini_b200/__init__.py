"""llmini_b200: B200 (sm_100a) implementation of llmini's AMUSE/Muon + NVFP4 requantisation path.

The product is the C-ABI shared library built from ``csrc/`` (see ``include/llmini_b200.h``);
the Python modules here mirror the reference's Rust host interface on top of it.
"""
from ._ffi import (B2Error, NORMALIZE_DEFERRED, NORMALIZE_TWO_PASS, NS_CHAINED, NS_FUSED_GRAM_POLY, NS_PER_PHASE, OPERAND_BF16, OPERAND_F16, QUANTIZE_X, QUANTIZE_Y, SCALES_CSF, SCALES_RAW, SCALES_SM100, UPDATE_16BIT, UPDATE_F32, lib)
from .nvfp4 import (Nvfp4QuantModule, Nvfp4Tensor, csf_encode_host, csf_encoded_len, csf_scale_at, scales_to_sm100,
                    sm100_scales_bytes, zero_scales)
from .optimizer import (AverageCoefficient, MuonMegaUpdateArgs, MuonPlan, MuonSlot, OptimizerModule,
                        schedule_free_beta, slot_table, warmup_multiplier)

__all__ = [
    "B2Error", "NORMALIZE_DEFERRED", "NORMALIZE_TWO_PASS", "NS_CHAINED", "NS_FUSED_GRAM_POLY", "NS_PER_PHASE", "OPERAND_BF16", "OPERAND_F16", "QUANTIZE_X", "QUANTIZE_Y", "SCALES_CSF", "SCALES_RAW", "SCALES_SM100", "UPDATE_16BIT", "UPDATE_F32", "lib",
    "Nvfp4QuantModule", "Nvfp4Tensor", "csf_encode_host", "csf_encoded_len", "csf_scale_at", "scales_to_sm100",
    "sm100_scales_bytes", "zero_scales",
    "AverageCoefficient", "MuonMegaUpdateArgs", "MuonPlan", "MuonSlot", "OptimizerModule", "schedule_free_beta",
    "slot_table", "warmup_multiplier",
]
