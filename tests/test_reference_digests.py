"""Golden digests the reference holds for the four-six NVFP4 quantiser: FNV-1a over the packed
E2M1 bytes, the decoded E4M3 block-scale bytes and the little-endian FP32 tensor scale, captured
from the reference's own PTX (crates/cuda-kernels/tests/csf_quantization.rs:505-572,
`persistent_materialization_128_columns_preserves_original_bytes`).  They pin codes, block scales
and tensor scale of the oracle (CPU) and of this build's kernels (GPU) bit for bit."""
import numpy as np
import pytest

import llmini_b200 as b2
from oracle import oracle as o

F = np.float32
LEN = 128 * 128
DIRECT_DIGEST = 0x8B6E8A7E1DFFF073       # fp32_to_nvfp4_four_six on x
SCHEDULED_DIGEST = 0xD8F0E69E822B79DF    # materialize_schedule_free, beta 0.7, symexp_lin_beta 12.5, no scale slots


def fnv1a(*parts) -> int:
    h = 0xCBF29CE484222325
    for part in parts:
        for byte in bytes(part):
            h = ((h ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def inputs():
    i = np.arange(LEN)
    x = (((i * 17 + 13) % 251).astype(F) - F(125.0)) * F(0.001)
    z = (((i * 29 + 7) % 277).astype(F) - F(138.0)) * F(0.001)
    return x.astype(F), z.astype(F)


def test_oracle_quantiser_reproduces_the_reference_digest():
    x, _ = inputs()
    codes, raw, gs, _ = o.nvfp4_quantize(x, amax=np.max(np.abs(x)))
    assert codes.size + raw.size + 4 == 9220
    assert fnv1a(codes.tobytes(), raw.tobytes(), F(gs).tobytes()) == DIRECT_DIGEST


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [b2.SCALES_CSF, b2.SCALES_RAW])
def test_gpu_quantiser_reproduces_the_reference_digest(layout):
    import torch
    from tests.gpu_util import dev, host
    x, _ = inputs()
    q = b2.Nvfp4QuantModule()
    t = b2.Nvfp4Tensor.empty(128, 128, layout)
    amax = dev(np.array([np.max(np.abs(x))], F))
    q.fp32_to_nvfp4_four_six(dev(x), amax, t.bytes, t.scales, t.global_scale, LEN // 16, layout)
    torch.cuda.synchronize()
    stored = host(t.scales)
    raw = stored[: LEN // 16] if layout == b2.SCALES_RAW else \
        np.array([b2.csf_scale_at(stored, g) for g in range(LEN // 16)], np.uint8)
    assert fnv1a(host(t.bytes).tobytes(), raw.tobytes(), host(t.global_scale).tobytes()) == DIRECT_DIGEST


@pytest.mark.gpu
def test_gpu_schedule_free_materialisation_with_symexp_lin_reproduces_the_reference_digest():
    # the second digest of the same reference test: y = SymExpLin(z + beta (x - z)) with beta 0.7,
    # symexp_lin_beta 12.5 and no scale slots, measured and quantised by materialize_schedule_free.
    # It goes through ex2.approx, un-fused multiply-adds and IEEE division exactly as assumed here.
    import torch
    from tests.gpu_util import dev, host
    x, z = inputs()
    opt = b2.OptimizerModule()
    t = b2.Nvfp4Tensor.empty(128, 128, b2.SCALES_CSF)
    amax = dev(np.array([np.max(np.abs(x))], F))
    opt.materialize_schedule_free(bytes=t.bytes, scales=t.scales, global_scale=t.global_scale, z_master=dev(z),
                                  x_master=dev(x), amax=amax, len=LEN, scale_rows=128, scale_k=128, beta=0.7,
                                  symexp_lin_beta=12.5, scale_layout=b2.SCALES_CSF)
    torch.cuda.synchronize()
    stored = host(t.scales)
    raw = np.array([b2.csf_scale_at(stored, g) for g in range(LEN // 16)], np.uint8)
    assert fnv1a(host(t.bytes).tobytes(), raw.tobytes(), host(t.global_scale).tobytes()) == SCHEDULED_DIGEST


# Digests of the reference's row-wise quantiser (csf_quantization.rs:574-655): the same four-six
# arithmetic with every row as its own tensor (tensor scale = row amax / 1536, zero rows included),
# FNV-1a over all packed bytes, then each row's block-scale bytes, then the row scales.
ROWWISE = [(1, 16, 0x7AE32C9F6169785E), (3, 80, 0xF787EA4CA1E768FC), (3, 128, 0xBA595E1D681332C4),
           (129, 256, 0x484EB3D70045C086), (17, 2048, 0xABE7DBF7EA809134), (17, 8192, 0x65FA8FFA758B9DC1)]


def rowwise_input(rows, cols):
    i = np.arange(rows * cols)
    return np.where((i // cols) % 17 == 0, F(0.0), (((i * 17 + 13) % 251).astype(F) - F(125.0)) * F(0.003)).astype(F)


@pytest.mark.parametrize("rows,cols,digest", ROWWISE)
def test_oracle_reproduces_the_rowwise_digests(rows, cols, digest):
    x = rowwise_input(rows, cols).reshape(rows, cols)
    out = [o.nvfp4_quantize(row, amax=np.max(np.abs(row))) for row in x]
    assert fnv1a(*[c.tobytes() for c, _, _, _ in out], *[s.tobytes() for _, s, _, _ in out],
                 *[F(gs).tobytes() for _, _, gs, _ in out]) == digest


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,digest", ROWWISE)
def test_gpu_quantiser_reproduces_the_rowwise_digests(rows, cols, digest):
    import torch
    from tests.gpu_util import dev, host
    x = rowwise_input(rows, cols).reshape(rows, cols)
    q = b2.Nvfp4QuantModule()
    xd = dev(x)
    codes = torch.zeros(rows, cols // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, cols // 16, dtype=torch.uint8, device="cuda")
    gs = torch.zeros(rows, device="cuda")
    amax = xd.abs().amax(dim=1).contiguous()
    for r in range(rows):   # every row through the tensor quantiser with the row's own maximum
        q.fp32_to_nvfp4_four_six(xd[r], amax[r:r + 1], codes[r], scales[r], gs[r:r + 1], cols // 16, b2.SCALES_RAW)
    torch.cuda.synchronize()
    assert fnv1a(host(codes).tobytes(), host(scales).tobytes(), host(gs).tobytes()) == digest
