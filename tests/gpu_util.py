"""Helpers shared by the GPU parity tests (device <-> numpy, rcp tables from the device)."""
import numpy as np
import torch

import llmini_b200 as b2
from oracle import oracle as o


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host(t):
    return t.detach().cpu().numpy()


def bf16_from_bits(bits):
    """uint16 bit patterns -> torch bfloat16 CUDA tensor."""
    return torch.from_numpy(np.ascontiguousarray(bits, dtype=np.uint16).view(np.int16)).cuda().view(torch.bfloat16)


def bf16_bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rcp_table(global_scales, contract=False):
    """Reciprocals the quantiser can need for the given tensor scales, evaluated with
    `rcp.approx.ftz.f32` on the device: (in_bits, out_bits) for the oracle."""
    q = b2.Nvfp4QuantModule()
    ins = np.concatenate([o.rcp_inputs(gs, contract) for gs in np.atleast_1d(global_scales)]).astype(np.float32)
    outs = host(q.debug_rcp_approx_ftz(dev(ins)))
    return ins.view(np.uint32).copy(), outs.view(np.uint32).copy()


def decode_scales(slot_scales, rows, cols, layout):
    s = host(slot_scales)
    if layout == b2.SCALES_RAW:
        return s[: rows * cols // 16]
    return o.csf_decode_matrix(s, rows, cols)
