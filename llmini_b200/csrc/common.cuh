// Shared device helpers: PTX wrappers for the conversions the NVFP4 recipe is defined by,
// warp/block reductions and small vector load/store helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/llmini_b200.h"

namespace b2 {

constexpr int kThreads = 256;            // CTA size of every streaming kernel
constexpr int kChunk = 2048;             // values per chunk (8 per thread), as the reference's
                                         // NVFP4_TENSOR_AMAX_VALUES_PER_BLOCK
constexpr int kMaxResidentCtasPerSm = 8; // 2048 threads / 256
constexpr float kDenomEps = 1.0e-20f;    // crates/cuda-kernels/src/utils/nvfp4/quant/kernels/convert.rs:6

// ---- PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ float rcp_approx_ftz(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// low byte = E4M3(lo), high byte = E4M3(hi)
__device__ __forceinline__ uint16_t cvt_e4m3x2(float hi, float lo) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// low nibble = E2M1(lo), high nibble = E2M1(hi)
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }"
        : "=h"(r)
        : "f"(hi), "f"(lo));
    return (uint32_t)r & 0xffu;
}
// value of the E4M3 code in the LOW byte of `bits`
__device__ __forceinline__ float e4m3_value(uint16_t bits) {
    float v;
    asm("{ .reg .b32 h2; .reg .b16 lo, hi; cvt.rn.f16x2.e4m3x2 h2, %1; mov.b32 {lo, hi}, h2; "
        "cvt.f32.f16 %0, lo; }"
        : "=f"(v)
        : "h"(bits));
    return v;
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
// round-to-nearest-even; same result as the reference's host helper for finite inputs
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ uint32_t f32_to_f16_bits(float v) {
    uint16_t r;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
    return r;
}
// packs two floats into one 32-bit word of 16-bit operands: low half = a, high half = b
__device__ __forceinline__ uint32_t pack_operands(float a, float b, int f16) {
    uint32_t r;
    if (f16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}

// ---- NVFP4 recipe ------------------------------------------------------------------------
// crates/cuda-kernels/src/utils/nvfp4/quant/kernels/four_six/helpers.rs:32-38
__device__ __forceinline__ float four_six_global_scale(float tensor_amax) {
    float gs = (tensor_amax == 0.0f) ? 1.0f : tensor_amax * 1.0f / (256.0f * 6.0f);
    return gs == 0.0f ? 1.0f : gs;
}
// Block scale of one 16-value group from its amax: convert.rs:64-85 (local_scale_bits),
// then the code reciprocal: convert.rs:23-25 (nvfp4_inv_scale).  gs is already non-zero.
__device__ __forceinline__ uint32_t group_scale_and_inv(float group_amax, float gs, float &inv) {
    float t = group_amax * 1.0f * rcp_approx_ftz(6.0f * gs + kDenomEps);
    uint16_t sb = cvt_e4m3x2(0.0f, t);
    float s = e4m3_value(sb);
    float sn = (s == 0.0f) ? 1.0f : s;
    inv = rcp_approx_ftz(sn * gs + kDenomEps);
    return (uint32_t)sb & 0xffu;
}
// Four consecutive values of a group -> 16-bit payload (convert.rs:27-43 pair packing).
__device__ __forceinline__ uint32_t pack_quad(float v0, float v1, float v2, float v3, float inv) {
    uint32_t p01 = cvt_e2m1x2(v1 * inv, v0 * inv);
    uint32_t p23 = cvt_e2m1x2(v3 * inv, v2 * inv);
    return p01 | (p23 << 8);
}

// ---- CSF record store (crates/cuda-kernels/src/utils/nvfp4/csf.rs:19-30,193-261) ---------
__device__ __forceinline__ uint32_t csf_code_offset(uint32_t r) {
    return (r / 16) * 96 + (r % 8) * 12 + (r % 16 / 8) * 3;
}
__device__ __forceinline__ uint32_t csf_compact6(uint32_t w) {
    return (w & 63) | ((w & 0x3f00) >> 2) | ((w & 0x3f0000) >> 4) | ((w & 0x3f000000) >> 6);
}
__device__ __forceinline__ uint32_t csf_high1(uint32_t w) {
    return (((w >> 6) & 0x01010101u) * 0x01020408u) >> 24;
}
__device__ __forceinline__ void csf_store24(uint8_t *d, uint32_t v) {
    d[0] = (uint8_t)v;
    d[1] = (uint8_t)(v >> 8);
    d[2] = (uint8_t)(v >> 16);
}
// floor(2^32 / groups-per-row) (one less for a power of two): the multiplier csf_store_record
// divides by.  Computed once per tensor, not once per record.
__device__ __forceinline__ uint32_t csf_row_magic(uint32_t k, uint32_t rows) {
    return (rows == 1 || k < 16) ? 0u : 0xffffffffu / (k / 16);
}
// Eight consecutive block scales (a = groups 0..3, b = groups 4..7) of flat group index g0
// (a multiple of 8).  `scales` points at the CSF header; k and rows are read from it, and
// magic = csf_row_magic(k, rows) when USE_MAGIC (ignored otherwise).
template <bool USE_MAGIC>
__device__ __forceinline__ void csf_store_record(uint8_t *scales, uint32_t k, uint32_t rows, uint32_t magic,
                                                 uint32_t g0, uint32_t a, uint32_t b) {
    if (rows == 1) {
        uint32_t *p = reinterpret_cast<uint32_t *>(scales + 128 + g0);
        p[0] = a;
        p[1] = b;
        return;
    }
    const uint32_t groups = k / 16;
    uint32_t row, kg;
    if (USE_MAGIC) {
        // row = g0 / groups by multiplication: floor(g0 * magic / 2^32) is the quotient or one less
        row = __umulhi(g0, magic);
        kg = g0 - row * groups;
        if (kg >= groups) {
            ++row;
            kg -= groups;
        }
    } else {
        row = g0 / groups;
        kg = g0 - row * groups;
    }
    uint32_t t = row / 128 * (k / 128) + kg / 8;
    uint32_t r = row % 128;
    uint8_t *d = scales + 128;
    uint32_t at = t * 896 + csf_code_offset(r);
    csf_store24(d + at, csf_compact6(a));
    csf_store24(d + at + 6, csf_compact6(b));
    d[t * 896 + 768 + r] = (uint8_t)(csf_high1(a) | (csf_high1(b) << 4));
}

// One block scale out of CSF storage (the device twin of b2_csf_scale_at).
__device__ __forceinline__ uint32_t csf_load_scale(const uint8_t *s, uint32_t g) {
    if (s[8] == 255) return s[128 + g];
    const uint32_t k = reinterpret_cast<const uint32_t *>(s)[0], groups = k / 16;
    const uint32_t row = g / groups, kg = g - row * groups;
    const uint32_t bytes = (uint32_t)s[9] - 6;
    const uint8_t *d = s + 128;
    const uint32_t t = row / 128 * (k / 128) + kg / 8, r = row % 128, stride = 768 + 128 * bytes;
    const size_t at = (size_t)t * stride + csf_code_offset(r) + (kg % 8 / 4) * 6;
    const uint32_t shift = (kg % 4) * 6, bits = shift % 8;
    const size_t byte = at + shift / 8;
    const uint32_t lo = d[byte], hi = bits > 2 ? d[byte + 1] : 0;
    const uint32_t q = ((lo | (hi << 8)) >> bits) & 63u;
    const size_t am = (size_t)t * stride + 768 + (size_t)r * bytes;
    if (bytes == 1) return q | (((d[am] >> (kg % 8)) & 1u) << 6);
    return q | (((d[am + kg % 8 / 4] >> ((kg % 4) * 2)) & 3u) << 6);
}
// Byte offset of the scale of (row, 16-value block kb) in the sm_100 block-scale operand layout:
// 512-byte tiles of 128 rows x 4 blocks, `kb_tiles` = ceil(blocks per row / 4) tiles per row band.
__device__ __forceinline__ size_t sm100_scale_offset(uint32_t row, uint32_t kb, uint32_t kb_tiles) {
    return ((size_t)(row >> 7) * kb_tiles + (kb >> 2)) * 512 + (row & 31u) * 16 + ((row >> 5) & 3u) * 4 + (kb & 3u);
}

// ---- SymExpLin forward (crates/cuda-kernels/src/gpt/optimizer/symexp_lin.rs:8-26) -------------
struct SymExpLin {
    float beta, exponential, linear, curvature;
};
// exp_f32 of the reference: ex2.approx.ftz.f32(x * log2(e)) (crates/cuda-kernels/src/utils/float_ptx.rs:46-51)
__device__ __forceinline__ float exp_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
    return r;
}
// ln_f32 / log1p_f32 of the reference (float_ptx.rs:53-57, 103-108)
__device__ __forceinline__ float ln_approx(float x) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r * 0.6931471805599453f;
}
__device__ __forceinline__ float log1p_compensated(float x) {
    const float u = 1.0f + x;
    return u == 1.0f ? x : ln_approx(u) * (x / (u - 1.0f));
}
__device__ __forceinline__ float symexp_forward(float raw, const SymExpLin &s) {
    if (s.beta <= 0.0f) return raw;
    const float sign = raw > 0.0f ? 1.0f : (raw < 0.0f ? -1.0f : 0.0f);
    if (sign == 0.0f) return 0.0f;
    const float exponential = s.exponential * (exp_approx(s.beta * s.curvature * fabsf(raw)) - 1.0f) / s.beta;
    return sign * (exponential + s.linear * raw / s.beta);
}

// ---- reductions ----------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// non-negative floats order like their bit patterns
__device__ __forceinline__ void atomic_max_nonneg(float *addr, float v) {
    atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

// ---- streaming loads/stores ------------------------------------------------------------------
__device__ __forceinline__ float4 ld_stream(const float *p) {
    return __ldcs(reinterpret_cast<const float4 *>(p));
}
__device__ __forceinline__ void st_stream(float *p, float4 v) {
    __stcs(reinterpret_cast<float4 *>(p), v);
}

// Slot that owns global chunk `c`: largest s with prefix[s] <= c.
__device__ __forceinline__ uint32_t find_slot(const uint32_t *prefix, uint32_t slot_count, uint32_t c) {
    uint32_t lo = 0, hi = slot_count;
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= c) lo = mid;
        else hi = mid;
    }
    return lo;
}

}  // namespace b2
