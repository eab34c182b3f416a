/*
 * CPU oracle for the AMUSE/Muon + NVFP4 requantisation path of JustKitting/llmini.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference's
 * arithmetic, used to check the CUDA library and to time a CPU baseline.  Nothing in the
 * shipped library links, loads or calls it.
 *
 * Parity status.  The reference is Rust compiled to PTX by cuda-oxide (pinned at commit
 * 971e353af258a05279aee7f805dfcfe8e95a0e30 in Cargo.lock) and cannot be built or run where
 * this oracle was written, so the oracle is pinned against the known answers that the
 * reference's own tests hold (see tests/test_oracle_known_answers.py) and not against
 * reference outputs.  The NVFP4 codes, block scales and tensor scale ARE pinned against a
 * reference output: the FNV-1a digest that crates/cuda-kernels/tests/csf_quantization.rs:526
 * holds for `fp32_to_nvfp4_four_six` on a 128 x 128 tensor, captured from the reference's own
 * PTX, is reproduced by orc_nvfp4_quantize (tests/test_reference_digests.py).  Two things
 * cannot be read from the reference's source and are switches here: whether `a*b + c`
 * expressions are contracted to FMA (`contract`; the second digest of that test, which the
 * GPU library reproduces, says they are not), and the exact result of `rcp.approx.ftz.f32`
 * (hardware-defined; callers may pass a table of reciprocals taken from the GPU, otherwise
 * the correctly rounded reciprocal is used).
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference's repository root).
 */
#include "oracle.h"

#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------ */
/* scalar conversions                                                                    */
/* ------------------------------------------------------------------------------------ */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* Round-to-nearest-even f32 -> bf16 bits.
 * crates/cuda-kernels/tests/common/mod.rs:74-78 (f32_to_bf16_bits). */
uint16_t orc_f32_to_bf16_bits(float v) {
    uint32_t bits = f2u(v);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x40); /* NaN */
    uint32_t bias = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}
float orc_bf16_bits_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }
float orc_round_bf16(float v) { return orc_bf16_bits_to_f32(orc_f32_to_bf16_bits(v)); }

/* IEEE binary16 round-to-nearest-even, subnormals kept: what `cvt.rn.f16.f32` does
 * (crates/cuda-kernels/src/utils/f16_tc_matmul/convert.rs:23-25). */
uint16_t orc_f32_to_f16_bits(float v) {
    uint32_t x = f2u(v);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (ax >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536 -> inf */
    if (ax < 0x38800000u) { /* below 2^-14: subnormal half or zero */
        if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to 0 */
        float a = u2f(ax);
        /* a * 2^24 is exact; rint is RNE in the default rounding mode */
        uint32_t q = (uint32_t)nearbyintf(a * 16777216.0f);
        return (uint16_t)(sign | q);
    }
    uint32_t mant = ax & 0x7fffffu;
    uint32_t exp = (ax >> 23) - 127 + 15;
    uint32_t half = (exp << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half += 1; /* carries into exp */
    return (uint16_t)(sign | half); /* 65520..65535.99 -> 0x7c00 = inf by the carry */
}
float orc_f16_bits_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t mant = h & 0x3ff;
    if (exp == 0) {
        float v = (float)mant * 5.9604644775390625e-8f; /* 2^-24 */
        return u2f(f2u(v) | sign);
    }
    if (exp == 31) return u2f(sign | 0x7f800000u | (mant << 13));
    return u2f(sign | ((exp - 15 + 127) << 23) | (mant << 13));
}
float orc_round_f16(float v) { return orc_f16_bits_to_f32(orc_f32_to_f16_bits(v)); }

/* The reference's HOST helper flushes binary16 subnormals to zero
 * (crates/cuda-kernels/tests/optimizer/polar_reference/rounding.rs:1-32). */
float orc_round_f16_host_flush(float v) {
    uint32_t bits = f2u(v);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int exp = (int)((bits >> 23) & 0xff) - 127 + 15;
    uint32_t mant = bits & 0x7fffffu;
    if (exp <= 0) return 0.0f;
    if (exp >= 0x1f) return INFINITY;
    uint32_t hm = mant >> 13;
    uint32_t rb = mant & 0x1fffu;
    if (rb > 0x1000u || (rb == 0x1000u && (hm & 1u))) {
        hm += 1;
        if (hm == 0x400u) { hm = 0; exp += 1; }
    }
    uint32_t half = sign | ((uint32_t)exp << 10) | hm;
    int e2 = (int)((half >> 10) & 0x1f);
    uint32_t m2 = half & 0x3ff;
    if (e2 == 0) return 0.0f;
    return u2f(((half & 0x8000u) << 16) | ((uint32_t)(e2 - 15 + 127) << 23) | (m2 << 13));
}

float orc_round_operand(float v, int mode) {
    switch (mode) {
        case ORC_ROUND_F16: return orc_round_f16(v);
        case ORC_ROUND_BF16: return orc_round_bf16(v);
        case ORC_ROUND_F16_HOST: return orc_round_f16_host_flush(v);
        default: return v;
    }
}

/* Generic small-float encoder, round-to-nearest-even, saturating to max_code.
 * Restates `cvt.rn.satfinite.e4m3x2.f32` / `cvt.rn.satfinite.e2m1x2.f32` for one value
 * (crates/cuda-kernels/src/utils/nvfp4/quant/kernels/convert.rs:64-105). */
static uint8_t encode_small_float(float v, int exp_bits, int man_bits, int bias,
                                  uint8_t max_code, uint8_t nan_code) {
    uint32_t bits = f2u(v);
    uint8_t sign = (uint8_t)((bits >> 31) << (exp_bits + man_bits));
    if ((bits & 0x7fffffffu) > 0x7f800000u) return nan_code;
    double a = fabs((double)v);
    double max_val;
    {
        int e = (max_code >> man_bits);
        int m = max_code & ((1 << man_bits) - 1);
        max_val = ldexp(1.0 + (double)m / (double)(1 << man_bits), e - bias);
    }
    if (a >= max_val) return (uint8_t)(sign | max_code);
    double min_normal = ldexp(1.0, 1 - bias);
    uint32_t code;
    if (a < min_normal) {
        double q = nearbyint(ldexp(a, bias - 1 + man_bits)); /* quantum 2^(1-bias-man) */
        code = (uint32_t)q;                                  /* q == 2^man -> min normal */
    } else {
        int e;
        double fr = frexp(a, &e); /* a = fr * 2^e, fr in [0.5,1) */
        e -= 1;                   /* a = (2 fr) * 2^e */
        double m = nearbyint((fr * 2.0 - 1.0) * (double)(1 << man_bits));
        uint32_t mi = (uint32_t)m;
        uint32_t eb = (uint32_t)(e + bias);
        if (mi == (1u << man_bits)) { mi = 0; eb += 1; }
        code = (eb << man_bits) | mi;
    }
    if (code > max_code) code = max_code;
    return (uint8_t)(sign | code);
}

uint8_t orc_f32_to_e4m3(float v) { return encode_small_float(v, 4, 3, 7, 0x7e, 0x7f); }
/* For E2M1, NaN converts to positive MAX_NORM under .satfinite. */
uint8_t orc_f32_to_e2m1(float v) { return encode_small_float(v, 2, 1, 1, 0x7, 0x7); }

/* crates/cuda-kernels/src/utils/nvfp4/cast.rs:50-63 (e4m3_value); decode table in
 * src/training/schedule_free/materialize.rs:380-386. */
float orc_e4m3_value(uint8_t code) {
    int sign = code >> 7;
    int e = (code >> 3) & 15;
    int m = code & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = (float)m * 0.001953125f; /* 2^-9 */
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return sign ? -v : v;
}
/* crates/cuda-kernels/src/utils/nvfp4/cast.rs:4-19 (e2m1_value); table
 * {0,.5,1,1.5,2,3,4,6} in src/training/schedule_free/materialize.rs:388. */
float orc_e2m1_value(uint8_t code) {
    static const float t[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = t[code & 7];
    return (code & 8) ? -v : v;
}

/* ------------------------------------------------------------------------------------ */
/* reciprocal provider: rcp.approx.ftz.f32                                               */
/* ------------------------------------------------------------------------------------ */

static float ftz(float v) {
    uint32_t b = f2u(v);
    if ((b & 0x7f800000u) == 0) return u2f(b & 0x80000000u);
    return v;
}
/* Correctly rounded stand-in with flush-to-zero on input and output
 * (crates/cuda-kernels/src/utils/float_ptx.rs:31-33). */
float orc_rcp_exact_ftz(float x) {
    x = ftz(x);
    return ftz(1.0f / x);
}
static float rcp_lookup(const orc_rcp_table *t, float x, uint64_t *misses) {
    if (t && t->count) {
        uint32_t key = f2u(x);
        for (uint32_t i = 0; i < t->count; ++i)
            if (t->in_bits[i] == key) return u2f(t->out_bits[i]);
        if (misses) *misses += 1;
    }
    return orc_rcp_exact_ftz(x);
}

static inline float mul_add(float a, float b, float c, int contract) {
    if (contract) return fmaf(a, b, c);
    volatile float p = a * b; /* volatile: keep the compiler from fusing */
    return p + c;
}

/* ------------------------------------------------------------------------------------ */
/* NVFP4 quantiser                                                                       */
/* ------------------------------------------------------------------------------------ */

/* crates/cuda-kernels/src/utils/nvfp4/quant/kernels/four_six/helpers.rs:32-38
 * (four_six_global_scale) + convert.rs:9-15 (nonzero_global_scale). */
float orc_four_six_global_scale(float tensor_amax) {
    float gs = (tensor_amax == 0.0f) ? 1.0f : tensor_amax * 1.0f / (256.0f * 6.0f);
    return gs == 0.0f ? 1.0f : gs;
}

/* The rcp inputs one tensor can need: index 0 is the block-scale denominator
 * `6*gs + 1e-20` (convert.rs:72-73), index 1+c the code denominator for E4M3 code c
 * (convert.rs:23-25).  Returns the count written (1 + 127). */
uint32_t orc_nvfp4_rcp_inputs(float global_scale, int contract, float *out) {
    float gs = global_scale == 0.0f ? 1.0f : global_scale;
    out[0] = mul_add(6.0f, gs, 1.0e-20f, contract);
    for (int c = 0; c < 127; ++c) {
        float s = orc_e4m3_value((uint8_t)c);
        float sn = (s == 0.0f) ? 1.0f : s;
        out[1 + c] = mul_add(sn, gs, 1.0e-20f, contract);
    }
    return 128;
}

/* One 16-value group: helpers.rs:41-94 (six_grid_group_scale), convert.rs:64-85
 * (local_scale_bits), convert.rs:23-43 (nvfp4_inv_scale, candidate pair payload). */
static void quantize_group(const float *v, float gs_in, int contract, const orc_rcp_table *rcp,
                           uint64_t *misses, uint8_t *scale_out, uint8_t *codes_out /*8 bytes*/) {
    float gs = gs_in == 0.0f ? 1.0f : gs_in;
    float ga = 0.0f;
    for (int i = 0; i < 16; ++i) {
        float a = fabsf(v[i]);
        /* max.f32: NaN operands are dropped, like PTX max */
        if (a > ga) ga = a;
    }
    float denom = mul_add(6.0f, gs, 1.0e-20f, contract);
    float t = ga * 1.0f * rcp_lookup(rcp, denom, misses);
    uint8_t sb = orc_f32_to_e4m3(t);
    float s = orc_e4m3_value(sb);
    float sn = (s == 0.0f) ? 1.0f : s;
    float inv = rcp_lookup(rcp, mul_add(sn, gs, 1.0e-20f, contract), misses);
    for (int i = 0; i < 8; ++i) {
        uint8_t lo = orc_f32_to_e2m1(v[2 * i] * inv);
        uint8_t hi = orc_f32_to_e2m1(v[2 * i + 1] * inv);
        codes_out[i] = (uint8_t)(lo | (hi << 4));
    }
    *scale_out = sb;
}

float orc_tensor_amax(const float *x, uint64_t len) {
    float m = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        float a = fabsf(x[i]);
        if (a > m) m = a;
    }
    return m;
}

/* Flat-tensor quantisation with a given tensor amax:
 * crates/cuda-kernels/src/gpt/optimizer/muon/fused/quant/encode.rs:13-60 and
 * crates/cuda-kernels/src/utils/nvfp4/quant/kernels/four_six.rs:104-152,1838-1901
 * (layout 2).  `raw_scales` receives one E4M3 byte per group (row-major plane). */
uint64_t orc_nvfp4_quantize(const float *x, uint64_t len, float tensor_amax, int contract,
                            const orc_rcp_table *rcp, uint8_t *codes, uint8_t *raw_scales,
                            float *global_scale) {
    float gs = orc_four_six_global_scale(tensor_amax);
    uint64_t groups = len / 16;
    uint64_t misses = 0;
#pragma omp parallel for reduction(+ : misses) schedule(static)
    for (uint64_t g = 0; g < groups; ++g) {
        uint64_t local = 0;
        quantize_group(x + 16 * g, gs, contract, rcp, &local, raw_scales + g, codes + 8 * g);
        misses += local;
    }
    *global_scale = gs;
    return misses;
}

/* Dequantise (decode tables of src/training/optimizer_muon/tma_tests.rs:96-116). */
void orc_nvfp4_dequantize(const uint8_t *codes, const uint8_t *raw_scales, float global_scale,
                          uint64_t len, float *out) {
    for (uint64_t i = 0; i < len; ++i) {
        uint8_t q = (codes[i / 2] >> ((i % 2) * 4)) & 15;
        out[i] = orc_e2m1_value(q) * orc_e4m3_value(raw_scales[i / 16]) * global_scale;
    }
}

/* ------------------------------------------------------------------------------------ */
/* CSF packed block-scale storage (crates/cuda-kernels/src/utils/nvfp4/csf.rs)           */
/* ------------------------------------------------------------------------------------ */

static inline uint32_t csf_code_offset(uint32_t r) { /* csf.rs:19-21 */
    return (r / 16) * 96 + (r % 8) * 12 + (r % 16 / 8) * 3;
}
static inline uint32_t csf_compact6(uint32_t w) { /* csf.rs:23-25 */
    return (w & 63) | ((w & 0x3f00) >> 2) | ((w & 0x3f0000) >> 4) | ((w & 0x3f000000) >> 6);
}
static inline uint8_t csf_high1(uint32_t w) { /* csf.rs:27-29 */
    return (uint8_t)((((w >> 6) & 0x01010101u) * 0x01020408u) >> 24);
}
static inline uint8_t csf_high2(uint32_t w) { /* csf.rs:31-35 */
    uint32_t v = (w >> 6) & 0x03030303u;
    v = (v | (v >> 6)) & 0x000f000fu;
    return (uint8_t)((v | (v >> 12)) & 255);
}
uint64_t orc_csf_encoded_len(uint64_t rows, uint64_t k) { /* csf.rs:8-17 */
    if (rows == 1) return 128 + k / 16;
    return 128 + ((rows + 127) / 128) * ((k + 127) / 128) * 896;
}
/* csf.rs:36-95 (encode_host + encode_matrix + encode_vector).  Returns bytes written, 0 on
 * a violated precondition (the reference asserts).  `raw_len` may be shorter than
 * rows*k/16; the missing tail reads as zero. */
uint64_t orc_csf_encode(const uint8_t *raw, uint64_t raw_len, uint64_t rows, uint64_t k,
                        uint8_t *out, uint64_t out_cap) {
    if (k < 128 || k % 128 != 0) return 0;
    if (rows * k > 0xffffffffull) return 0;
    if (raw_len > rows * k / 16) return 0;
    if (rows == 1) {
        uint64_t n = 128 + k / 16;
        if (out_cap < n) return 0;
        memset(out, 0, n);
        uint32_t k32 = (uint32_t)k, one = 1;
        memcpy(out, &k32, 4);
        memcpy(out + 4, &one, 4);
        out[8] = 255;
        out[9] = 8;
        memcpy(out + 128, raw, raw_len);
        return n;
    }
    int bytes = 1;
    for (uint64_t i = 0; i < raw_len; ++i)
        if (raw[i] >= 128) { bytes = 2; break; }
    uint64_t stride = 768 + 128 * (uint64_t)bytes;
    uint64_t padded = (rows + 127) / 128 * 128;
    uint64_t tiles = padded / 128 * (k / 128);
    uint64_t n = 128 + tiles * stride;
    if (out_cap < n) return 0;
    memset(out, 0, n);
    uint32_t k32 = (uint32_t)k, r32 = (uint32_t)rows;
    memcpy(out, &k32, 4);
    memcpy(out + 4, &r32, 4);
    {
        uint32_t g = (uint32_t)(k / 16), tz = 0;
        while (((g >> tz) & 1u) == 0) ++tz;
        out[8] = (uint8_t)tz;
    }
    out[9] = (uint8_t)(6 + bytes);
    uint64_t groups = k / 16;
    for (uint64_t row = 0; row < padded; ++row) {
        for (uint64_t kg = 0; kg < groups; kg += 8) {
            uint8_t v[8];
            for (int i = 0; i < 8; ++i) {
                uint64_t idx = row * groups + kg + (uint64_t)i;
                v[i] = (row < rows && kg + (uint64_t)i < groups && idx < raw_len) ? raw[idx] : 0;
            }
            uint32_t a = (uint32_t)v[0] | ((uint32_t)v[1] << 8) | ((uint32_t)v[2] << 16) |
                         ((uint32_t)v[3] << 24);
            uint32_t b = (uint32_t)v[4] | ((uint32_t)v[5] << 8) | ((uint32_t)v[6] << 16) |
                         ((uint32_t)v[7] << 24);
            uint64_t t = row / 128 * (k / 128) + kg / 8;
            uint64_t at = 128 + t * stride + csf_code_offset((uint32_t)(row % 128));
            uint32_t ca = csf_compact6(a), cb = csf_compact6(b);
            out[at] = (uint8_t)ca; out[at + 1] = (uint8_t)(ca >> 8); out[at + 2] = (uint8_t)(ca >> 16);
            out[at + 6] = (uint8_t)cb; out[at + 7] = (uint8_t)(cb >> 8); out[at + 8] = (uint8_t)(cb >> 16);
            uint64_t am = 128 + t * stride + 768 + (row % 128) * (uint64_t)bytes;
            if (bytes == 1) out[am] = (uint8_t)(csf_high1(a) | (csf_high1(b) << 4));
            else { out[am] = csf_high2(a); out[am + 1] = csf_high2(b); }
        }
    }
    return n;
}
/* csf.rs:97-179 (read6, matrix_scale_at_bits, scale_at, flat_scale_coordinates). */
uint8_t orc_csf_scale_at(const uint8_t *s, uint64_t g) {
    if (s[8] == 255) return s[128 + g];
    uint32_t k; memcpy(&k, s, 4);
    uint32_t groups = k / 16;
    uint32_t row = (uint32_t)(g / groups), kg = (uint32_t)(g % groups);
    uint32_t bytes = (uint32_t)s[9] - 6;
    const uint8_t *d = s + 128;
    uint32_t t = row / 128 * (k / 128) + kg / 8;
    uint32_t r = row % 128;
    uint32_t stride = 768 + 128 * bytes;
    uint64_t at = (uint64_t)t * stride + csf_code_offset(r) + (kg % 8 / 4) * 6;
    uint32_t shift = (kg % 4) * 6;
    uint64_t byte = at + shift / 8;
    uint32_t bits = shift % 8;
    uint32_t a = d[byte];
    uint32_t b = bits > 2 ? d[byte + 1] : 0;
    uint8_t q = (uint8_t)(((a | (b << 8)) >> bits) & 63);
    uint64_t am = (uint64_t)t * stride + 768 + (uint64_t)r * bytes;
    if (bytes == 1) return (uint8_t)(q | (((d[am] >> (kg % 8)) & 1) << 6));
    return (uint8_t)(q | (((d[am + kg % 8 / 4] >> ((kg % 4) * 2)) & 3) << 6));
}

/* ------------------------------------------------------------------------------------ */
/* Muon stages                                                                           */
/* ------------------------------------------------------------------------------------ */

/* Stage M: crates/cuda-kernels/src/gpt/optimizer/muon/fused/momentum.rs:42-68.
 * `oriented` is written in the storage layout [rows][cols] (no transpose); callers that
 * want the reference's polar orientation transpose afterwards.  Returns sum of u^2 in
 * double. */
double orc_momentum(const float *grad, uint16_t *momentum_bf16, float *u_out, uint64_t len,
                    float mu, float grad_scale, int nesterov, int contract) {
    double s = 0.0;
    for (uint64_t i = 0; i < len; ++i) {
        float g = grad[i] * grad_scale;
        float pm = orc_bf16_bits_to_f32(momentum_bf16[i]);
        float omg;
        { volatile float t = (1.0f - mu) * g; omg = t; }
        float nm = mul_add(mu, pm, omg, contract);
        float u = nesterov ? mul_add(mu, nm, omg, contract) : nm;
        momentum_bf16[i] = orc_f32_to_bf16_bits(nm);
        u_out[i] = u;
        s += (double)u * (double)u;
    }
    return s;
}

/* Stage M, variance-adaptive branch (Muon-VS):
 * crates/cuda-kernels/src/gpt/optimizer/muon/fused/momentum.rs:72-158. */
double orc_momentum_vs(const float *grad, uint16_t *momentum_bf16, uint16_t *variance_bf16, float *u_out,
                       uint64_t len, float mu, float grad_scale, int nesterov, float bias_correction_inv) {
    double s = 0.0;
    volatile float one_minus_mu = 1.0f - mu;
    volatile float variance_factor = mu * one_minus_mu;
    volatile float nesterov_factor = mu / one_minus_mu;
    for (uint64_t i = 0; i < len; ++i) {
        volatile float g = grad[i] * grad_scale;
        float pm = orc_bf16_bits_to_f32(momentum_bf16[i]);
        float pv = orc_bf16_bits_to_f32(variance_bf16[i]);
        volatile float a = mu * pm, b = one_minus_mu * g;
        float nm = a + b;
        volatile float innovation = pm - g;
        volatile float c0 = mu * pv, c1 = variance_factor * innovation;
        volatile float c2 = c1 * innovation;
        float nv = c0 + c2;
        volatile float corrected = nm * bias_correction_inv;
        float numerator;
        if (nesterov) { volatile float t = nesterov_factor * corrected; numerator = g + t; }
        else numerator = corrected;
        volatile float vb = nv * bias_correction_inv;
        float root = sqrtf(vb > 0.0f ? vb : 0.0f);
        float u = numerator / (root + 1.0e-8f);
        momentum_bf16[i] = orc_f32_to_bf16_bits(nm);
        variance_bf16[i] = orc_f32_to_bf16_bits(nv);
        u_out[i] = u;
        s += (double)u * (double)u;
    }
    return s;
}

static float qk_factor(const float *factors, uint32_t offset, uint32_t head_dim, uint32_t rows, uint32_t cols,
                       uint64_t index) {
    /* update.rs:58-66 with cols == one chunk: rows below 2*cols are query/key rows, one factor per head */
    (void)rows;
    if (!factors || offset == 0xffffffffu || head_dim == 0) return 1.0f;
    uint64_t row = index / cols;
    if (row >= 2ull * cols) return 1.0f;
    return factors[offset + (uint32_t)((row % cols) / head_dim)];
}

/* Stage U with qk-clip: crates/cuda-kernels/src/gpt/optimizer/muon/fused/update/one.rs:46-85.
 * momentum (and variance when given) are rescaled for clipped rows. */
void orc_update_clip(const float *U, float *z, float *x, float *y, uint16_t *momentum_bf16, uint16_t *variance_bf16,
                     uint64_t len, uint32_t rows, uint32_t cols, float lr, float wd, float c_avg, float beta,
                     const float *factors, uint32_t offset, uint32_t head_dim, float *amax) {
    float fr = (float)rows, fc = (float)cols;
    float scale = 0.2f * sqrtf(fr > fc ? fr : fc);
    volatile float lw = lr * wd;
    float decay = 1.0f - lw;
    float ax = 0.0f, ay = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        volatile float upd = scale * U[i];
        volatile float p1 = z[i] * decay, p2 = lr * upd;
        volatile float nz = p1 - p2;
        volatile float d1 = nz - x[i];
        volatile float p3 = c_avg * d1;
        volatile float nx = x[i] + p3;
        float f = qk_factor(factors, offset, head_dim, rows, cols, i);
        if (f != 1.0f) {
            nz = nz * f;
            nx = nx * f;
            volatile float cm = orc_bf16_bits_to_f32(momentum_bf16[i]) * f;
            momentum_bf16[i] = orc_f32_to_bf16_bits(cm);
            if (variance_bf16) {
                volatile float cv = orc_bf16_bits_to_f32(variance_bf16[i]) * f;
                volatile float cv2 = cv * f;
                variance_bf16[i] = orc_f32_to_bf16_bits(cv2);
            }
        }
        volatile float d2 = nx - nz;
        volatile float p4 = beta * d2;
        float yy = nz + p4;
        z[i] = nz; x[i] = nx;
        if (y) y[i] = yy;
        if (fabsf(nx) > ax) ax = fabsf(nx);
        if (fabsf(yy) > ay) ay = fabsf(yy);
    }
    amax[0] = ax; amax[1] = ay;
}

/* NorMuon per-neuron second moment and Hyperball statistics:
 * crates/cuda-kernels/src/gpt/optimizer/muon/fused/tma_split.rs:285-477.
 * U is given in STORAGE orientation [rows][cols]; a neuron is an index along the larger dimension
 * (a row when rows >= cols, else a column: update/one.rs:48-53), its mean is taken over the
 * smaller one.  Sums are accumulated in double (the kernel's summation order is not part of the
 * contract; the reference's own tests allow 2e-6 / 2e-5).  stats = { normuon_scale,
 * update_norm, radius, dot }; radius and dot only when z is given. */
void orc_normuon_stats(const float *U, const float *z, uint32_t rows, uint32_t cols, float *second_momentum,
                       float *factors, float *stats) {
    const uint32_t neurons = rows >= cols ? rows : cols, span = rows >= cols ? cols : rows;
    double raw_total = 0.0, scaled_total = 0.0, param_total = 0.0, dot_total = 0.0;
    for (uint32_t nidx = 0; nidx < neurons; ++nidx) {
        double raw = 0.0, dot = 0.0;
        for (uint32_t k = 0; k < span; ++k) {
            uint64_t i = rows >= cols ? (uint64_t)nidx * cols + k : (uint64_t)k * cols + nidx;
            raw += (double)U[i] * U[i];
            if (z) { param_total += (double)z[i] * z[i]; dot += (double)z[i] * U[i]; }
        }
        volatile float mean = (float)raw / (float)span;
        volatile float a = 0.95f * second_momentum[nidx], b = (1.0f - 0.95f) * mean;
        float next = a + b;
        float factor = 1.0f / sqrtf(fmaxf(next, 1.0e-10f));
        second_momentum[nidx] = next;
        factors[nidx] = factor;
        raw_total += raw;
        scaled_total += (double)((float)raw * factor * factor);
        dot_total += (double)((float)dot * factor);
    }
    float scaled = fmaxf((float)scaled_total, 1.0e-10f);
    stats[0] = sqrtf((float)raw_total / scaled);
    stats[1] = sqrtf(scaled);
    stats[2] = z ? sqrtf(fmaxf((float)param_total, 1.0e-10f)) : 0.0f;
    stats[3] = z ? (float)dot_total : 0.0f;
}

/* Stage U with NorMuon factors: update/one.rs:46-60; factors == NULL is the plain update. */
void orc_update_normuon(const float *U, float *z, float *x, float *y, uint64_t len, uint32_t rows, uint32_t cols,
                        float lr, float wd, float c_avg, float beta, const float *factors, float normuon_scale,
                        float *amax) {
    float fr = (float)rows, fc = (float)cols;
    float scale = 0.2f * sqrtf(fr > fc ? fr : fc);
    volatile float lw = lr * wd;
    float decay = 1.0f - lw;
    float ax = 0.0f, ay = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        uint32_t row = (uint32_t)(i / cols), col = (uint32_t)(i - (uint64_t)row * cols);
        volatile float nf = factors ? factors[rows >= cols ? row : col] * normuon_scale : 1.0f;
        volatile float un = U[i] * nf;
        volatile float upd = scale * un;
        volatile float p1 = z[i] * decay, p2 = lr * upd;
        volatile float nz = p1 - p2;
        volatile float d1 = nz - x[i];
        volatile float p3 = c_avg * d1;
        volatile float nx = x[i] + p3;
        volatile float d2 = nx - nz;
        volatile float p4 = beta * d2;
        float yy = nz + p4;
        z[i] = nz; x[i] = nx;
        if (y) y[i] = yy;
        if (fabsf(nx) > ax) ax = fabsf(nx);
        if (fabsf(yy) > ay) ay = fabsf(yy);
    }
    amax[0] = ax; amax[1] = ay;
}

/* Hyperball projection: tma_split.rs:516-527 (scalars) and hyperball.rs:107-173 (elements).
 * lr is learning_rate * learning_rate_multiplier; stats as written by orc_normuon_stats. */
void orc_hyperball_update(const float *U, float *z, float *x, float *y, uint16_t *momentum_bf16,
                          uint16_t *variance_bf16, uint32_t rows, uint32_t cols, float lr, float c_avg, float beta,
                          int use_schedule_free, const float *factors, const float *stats, const float *clip_factors,
                          uint32_t offset, uint32_t head_dim, float *amax) {
    const uint64_t len = (uint64_t)rows * cols;
    const float radius = stats[2], dot = stats[3];
    const float update_norm = fmaxf(stats[1], 1.0e-10f);
    volatile float s0 = lr * radius;
    const float step_scale = s0 / update_norm;
    volatile float c0 = radius * radius;
    volatile float c1 = 2.0f * step_scale;
    volatile float c2 = c1 * dot;
    volatile float c3 = step_scale * step_scale;
    volatile float c4 = c3 * update_norm;
    volatile float c5 = c4 * update_norm;
    volatile float c6 = c0 - c2;
    volatile float c7 = c6 + c5;
    const float projection = radius / sqrtf(fmaxf(c7, 1.0e-10f));
    float ax = 0.0f, ay = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        uint32_t row = (uint32_t)(i / cols), col = (uint32_t)(i - (uint64_t)row * cols);
        volatile float direction = U[i] * factors[rows >= cols ? row : col];
        volatile float p0 = step_scale * direction;
        volatile float p1 = z[i] - p0;
        volatile float pz = p1 * projection;
        volatile float nx = pz;
        if (use_schedule_free) {
            volatile float d1 = pz - x[i];
            volatile float p3 = c_avg * d1;
            nx = x[i] + p3;
        }
        float f = qk_factor(clip_factors, offset, head_dim, rows, cols, i);
        if (f != 1.0f) {
            volatile float cm = orc_bf16_bits_to_f32(momentum_bf16[i]) * f;
            momentum_bf16[i] = orc_f32_to_bf16_bits(cm);
            if (variance_bf16) {
                volatile float cv = orc_bf16_bits_to_f32(variance_bf16[i]) * f;
                volatile float cv2 = cv * f;
                variance_bf16[i] = orc_f32_to_bf16_bits(cv2);
            }
            pz = pz * f; nx = nx * f;
        }
        volatile float d2 = nx - pz;
        volatile float p4 = beta * d2;
        float yy = pz + p4;
        z[i] = pz; x[i] = nx;
        if (y) y[i] = yy;
        if (fabsf(nx) > ax) ax = fabsf(nx);
        if (fabsf(yy) > ay) ay = fabsf(yy);
    }
    amax[0] = ax; amax[1] = ay;
}

/* sign-Muon: crates/cuda-kernels/src/gpt/optimizer/muon/fused/update/one.rs:88-167 (update_one_sign). */
void orc_sign_update(float *grad_inout_y, uint16_t *momentum_bf16, uint16_t *variance_bf16, float *z, float *x,
                     uint64_t len, uint32_t rows, uint32_t cols, float mu, float grad_scale, int variance_adaptive,
                     float lr, float wd, float c_avg, float beta, const float *factors, uint32_t offset,
                     uint32_t head_dim, float *amax) {
    volatile float one_minus_mu = 1.0f - mu;
    volatile float lw = lr * wd;
    float decay = 1.0f - lw;
    float ax = 0.0f, ay = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        volatile float g = grad_inout_y[i] * grad_scale;
        float pm = orc_bf16_bits_to_f32(momentum_bf16[i]);
        volatile float a = mu * pm, b = one_minus_mu * g;
        volatile float nm = a + b;
        volatile float nv = 0.0f;
        if (variance_adaptive) {
            volatile float innovation = pm - g;
            volatile float c0 = mu * orc_bf16_bits_to_f32(variance_bf16[i]);
            volatile float vf = mu * one_minus_mu;
            volatile float c1 = vf * innovation;
            volatile float c2 = c1 * innovation;
            nv = c0 + c2;
        }
        float dir = nm > 0.0f ? 1.0f : (nm < 0.0f ? -1.0f : 0.0f);
        volatile float p1 = z[i] * decay, p2 = lr * dir;
        volatile float nz = p1 - p2;
        volatile float d1 = nz - x[i];
        volatile float p3 = c_avg * d1;
        volatile float nx = x[i] + p3;
        volatile float cm = nm;
        float f = qk_factor(factors, offset, head_dim, rows, cols, i);
        if (f != 1.0f) {
            nz = nz * f; nx = nx * f; cm = cm * f;
            if (variance_adaptive) { volatile float ff = f * f; nv = nv * ff; }
        }
        if (variance_adaptive) variance_bf16[i] = orc_f32_to_bf16_bits(nv);
        momentum_bf16[i] = orc_f32_to_bf16_bits(cm);
        volatile float d2 = nx - nz;
        volatile float p4 = beta * d2;
        float yy = nz + p4;
        z[i] = nz; x[i] = nx; grad_inout_y[i] = yy;
        if (fabsf(nx) > ax) ax = fabsf(nx);
        if (fabsf(yy) > ay) ay = fabsf(yy);
    }
    amax[0] = ax; amax[1] = ay;
}

/* Number of host threads the OpenMP loops below use (0 = leave the runtime's default). */
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Stage N scalar: crates/cuda-kernels/src/gpt/optimizer/muon/polar/fused/normalize.rs:8-9,82-86. */
float orc_inv_norm(float sumsq, int contract) {
    float r = sqrtf(sumsq);
    float d = mul_add(r, 1.01f, 1.0e-7f, contract);
    return 1.0f / d;
}

/* C[i][j] = sum_k A[i][k]*B[j][k]; A is [M][K], B is [N][K]. */
static void gemm_nt(const float *A, const float *B, float *C, int M, int N, int K) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int i0 = 0; i0 < M; i0 += 4) {
        for (int j0 = 0; j0 < N; j0 += 4) {
            float acc[4][4] = {{0}};
            int im = (M - i0 < 4) ? M - i0 : 4, jm = (N - j0 < 4) ? N - j0 : 4;
            if (im == 4 && jm == 4) {
                const float *a0 = A + (size_t)(i0 + 0) * K, *a1 = A + (size_t)(i0 + 1) * K;
                const float *a2 = A + (size_t)(i0 + 2) * K, *a3 = A + (size_t)(i0 + 3) * K;
                const float *b0 = B + (size_t)(j0 + 0) * K, *b1 = B + (size_t)(j0 + 1) * K;
                const float *b2 = B + (size_t)(j0 + 2) * K, *b3 = B + (size_t)(j0 + 3) * K;
                float c00 = 0, c01 = 0, c02 = 0, c03 = 0, c10 = 0, c11 = 0, c12 = 0, c13 = 0;
                float c20 = 0, c21 = 0, c22 = 0, c23 = 0, c30 = 0, c31 = 0, c32 = 0, c33 = 0;
#pragma omp simd reduction(+ : c00, c01, c02, c03, c10, c11, c12, c13, c20, c21, c22, c23, c30, c31, c32, c33)
                for (int k = 0; k < K; ++k) {
                    float x0 = a0[k], x1 = a1[k], x2 = a2[k], x3 = a3[k];
                    float y0 = b0[k], y1 = b1[k], y2 = b2[k], y3 = b3[k];
                    c00 += x0 * y0; c01 += x0 * y1; c02 += x0 * y2; c03 += x0 * y3;
                    c10 += x1 * y0; c11 += x1 * y1; c12 += x1 * y2; c13 += x1 * y3;
                    c20 += x2 * y0; c21 += x2 * y1; c22 += x2 * y2; c23 += x2 * y3;
                    c30 += x3 * y0; c31 += x3 * y1; c32 += x3 * y2; c33 += x3 * y3;
                }
                acc[0][0] = c00; acc[0][1] = c01; acc[0][2] = c02; acc[0][3] = c03;
                acc[1][0] = c10; acc[1][1] = c11; acc[1][2] = c12; acc[1][3] = c13;
                acc[2][0] = c20; acc[2][1] = c21; acc[2][2] = c22; acc[2][3] = c23;
                acc[3][0] = c30; acc[3][1] = c31; acc[3][2] = c32; acc[3][3] = c33;
            } else {
                for (int i = 0; i < im; ++i)
                    for (int j = 0; j < jm; ++j) {
                        float s = 0;
                        for (int k = 0; k < K; ++k)
                            s += A[(size_t)(i0 + i) * K + k] * B[(size_t)(j0 + j) * K + k];
                        acc[i][j] = s;
                    }
            }
            for (int i = 0; i < im; ++i)
                for (int j = 0; j < jm; ++j) C[(size_t)(i0 + i) * N + (j0 + j)] = acc[i][j];
        }
    }
}
/* C[i][j] = sum_k A[i][k]*B[k][j]; A is [M][K], B is [K][N]. */
static void gemm_nn(const float *A, const float *B, float *C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i) {
        float *c = C + (size_t)i * N;
        for (int j = 0; j < N; ++j) c[j] = 0.0f;
        for (int k = 0; k < K; ++k) {
            float a = A[(size_t)i * K + k];
            const float *b = B + (size_t)k * N;
#pragma omp simd
            for (int j = 0; j < N; ++j) c[j] += a * b[j];
        }
    }
}
static void round_into(const float *src, float *dst, size_t n, int mode) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) dst[i] = orc_round_operand(src[i], mode);
}

/* Stage P, Gram form, as the device code computes it:
 * crates/cuda-kernels/src/gpt/optimizer/muon/polar/fused.rs:64-92 with the epilogue of
 * .../polar/fused/store/plain.rs:175-178 (polynomial_value) and operand rounding at
 * staging (.../polar/fused/stage.rs:51-55,74-83).  X is [n][m] row-major with n <= m,
 * overwritten with the result.  coeffs holds `iterations` triples (a, b, c). */
void orc_polar_gram(float *X, int n, int m, int iterations, const float *coeffs, int round_mode) {
    orc_polar_gram_scaled(X, n, m, iterations, coeffs, round_mode, 1.0f);
}

/* The same recurrence with the Frobenius normalisation deferred into the first iteration
 * (the one-pass form of stages M+N in the CUDA library): X arrives UN-normalised, is rounded to
 * 16 bits as it is, and s = 1 / (1.01 |X| + 1e-7) enters through the first iteration's outputs,
 *     G = (s * s) * (r16(X) r16(X)^T),   X1 = s * (r16(Q) r16(X)),
 * which is algebraically the reference's normalize.rs:137-143 followed by fused.rs:64-92 but rounds the
 * operand before instead of after the scaling.  first_scale = 1 gives the reference's order. */
void orc_polar_gram_scaled(float *X, int n, int m, int iterations, const float *coeffs, int round_mode,
                           float first_scale) {
    size_t nm = (size_t)n * m, nn = (size_t)n * n;
    float *Xr = (float *)malloc(nm * 4), *G = (float *)malloc(nn * 4);
    float *Gr = (float *)malloc(nn * 4), *Q = (float *)malloc(nn * 4);
    float *Y = (float *)malloc(nm * 4);
    for (int it = 0; it < iterations; ++it) {
        float a = coeffs[3 * it], b = coeffs[3 * it + 1], c = coeffs[3 * it + 2];
        round_into(X, Xr, nm, round_mode);
        gemm_nt(Xr, Xr, G, n, n, m);
        if (it == 0 && first_scale != 1.0f) {
            const float s2 = first_scale * first_scale;
#pragma omp parallel for schedule(static)
            for (size_t i = 0; i < nn; ++i) G[i] = G[i] * s2;
        }
        round_into(G, Gr, nn, round_mode);
        gemm_nt(Gr, Gr, Q, n, n, n); /* G symmetric: G*G == G*G^T */
#pragma omp parallel for schedule(static)
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < n; ++j) {
                float ident = (i == j) ? a : 0.0f;
                Q[(size_t)i * n + j] = fmaf(c, Q[(size_t)i * n + j], fmaf(b, G[(size_t)i * n + j], ident));
            }
        round_into(Q, Gr, nn, round_mode);
        gemm_nn(Gr, Xr, Y, n, m, n);
        if (it == 0 && first_scale != 1.0f) {
#pragma omp parallel for schedule(static)
            for (size_t i = 0; i < nm; ++i) Y[i] = Y[i] * first_scale;
        }
        memcpy(X, Y, nm * 4);
    }
    free(Xr); free(G); free(Gr); free(Q); free(Y);
}

/* Stage P in the tall orientation: Y is [m][n] row-major with m >= n; computes the same
 * recurrence on Y^T without materialising it: G = Y^T Y, Y <- Y Q.  (The CUDA library
 * works on the storage orientation; this mirrors its operand order.) */
void orc_polar_gram_tall(float *Y, int m, int n, int iterations, const float *coeffs, int round_mode) {
    orc_polar_gram_tall_scaled(Y, m, n, iterations, coeffs, round_mode, 1.0f);
}
void orc_polar_gram_tall_scaled(float *Y, int m, int n, int iterations, const float *coeffs, int round_mode,
                                float first_scale) {
    size_t nm = (size_t)n * m;
    float *Xt = (float *)malloc(nm * 4);
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) Xt[(size_t)j * m + i] = Y[(size_t)i * n + j];
    orc_polar_gram_scaled(Xt, n, m, iterations, coeffs, round_mode, first_scale);
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) Y[(size_t)i * n + j] = Xt[(size_t)j * m + i];
    free(Xt);
}

/* Stage P as the reference's HOST oracle computes it (three products, sequential f32 sums):
 * crates/cuda-kernels/tests/optimizer/polar_reference/ops.rs:5-48. */
void orc_polar_three_product(float *X, int n, int m, int iterations, const float *coeffs,
                             int round_mode) {
    size_t nm = (size_t)n * m, nn = (size_t)n * n;
    float *G = (float *)malloc(nn * 4), *AX = (float *)malloc(nm * 4), *AAX = (float *)malloc(nm * 4);
    for (int it = 0; it < iterations; ++it) {
        float a = coeffs[3 * it], b = coeffs[3 * it + 1], c = coeffs[3 * it + 2];
        for (int r = 0; r < n; ++r)
            for (int q = 0; q < n; ++q) {
                float s = 0.0f;
                for (int k = 0; k < m; ++k)
                    s += orc_round_operand(X[(size_t)r * m + k], round_mode) *
                         orc_round_operand(X[(size_t)q * m + k], round_mode);
                G[(size_t)r * n + q] = s;
            }
        for (int r = 0; r < n; ++r)
            for (int q = 0; q < m; ++q) {
                float s = 0.0f;
                for (int k = 0; k < n; ++k)
                    s += orc_round_operand(G[(size_t)r * n + k], round_mode) *
                         orc_round_operand(X[(size_t)k * m + q], round_mode);
                AX[(size_t)r * m + q] = s;
            }
        for (int r = 0; r < n; ++r)
            for (int q = 0; q < m; ++q) {
                float s = 0.0f;
                for (int k = 0; k < n; ++k)
                    s += orc_round_operand(G[(size_t)r * n + k], round_mode) *
                         orc_round_operand(AX[(size_t)k * m + q], round_mode);
                AAX[(size_t)r * m + q] = s;
            }
        for (size_t i = 0; i < nm; ++i) X[i] = fmaf(c, AAX[i], fmaf(a, X[i], b * AX[i]));
    }
    free(G); free(AX); free(AAX);
}

/* Stage U: crates/cuda-kernels/src/gpt/optimizer/muon/fused/update/one.rs:46-85 with
 * scale from .../update.rs:54.  U is indexed like z/x (storage layout).  y may be NULL.
 * amax[0] = max|x'|, amax[1] = max|y|. */
void orc_update(const float *U, float *z, float *x, float *y, uint64_t len, uint32_t rows,
                uint32_t cols, float lr, float wd, float c_avg, float beta, int contract,
                float *amax) {
    float fr = (float)rows, fc = (float)cols;
    float scale = 0.2f * sqrtf(fr > fc ? fr : fc);
    float decay;
    { volatile float t = lr * wd; decay = 1.0f - t; }
    if (contract) decay = fmaf(-lr, wd, 1.0f);
    float ax = 0.0f, ay = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        float mu_upd = scale * (U[i] * 1.0f * 1.0f);
        float nz, nx, yy;
        if (contract) {
            /* z*decay - lr*upd  ->  fma(z, decay, -(lr*upd)) */
            nz = fmaf(z[i], decay, -(lr * mu_upd));
            nx = fmaf(c_avg, nz - x[i], x[i]);
            yy = fmaf(beta, nx - nz, nz);
        } else {
            volatile float p1 = z[i] * decay, p2 = lr * mu_upd;
            nz = p1 - p2;
            volatile float d1 = nz - x[i];
            volatile float p3 = c_avg * d1;
            nx = x[i] + p3;
            volatile float d2 = nx - nz;
            volatile float p4 = beta * d2;
            yy = nz + p4;
        }
        z[i] = nz;
        x[i] = nx;
        if (y) y[i] = yy;
        if (fabsf(nx) > ax) ax = fabsf(nx);
        if (fabsf(yy) > ay) ay = fabsf(yy);
    }
    amax[0] = ax;
    amax[1] = ay;
}

/* crates/cuda-kernels/src/gpt/optimizer/schedule_free/value.rs:7-18: y = z + beta*(x - z). */
float orc_schedule_free_values(const float *z, const float *x, float *y, uint64_t len, float beta,
                               int contract) {
    float am = 0.0f;
    for (uint64_t i = 0; i < len; ++i) {
        float v;
        if (contract) v = fmaf(beta, x[i] - z[i], z[i]);
        else { volatile float d = x[i] - z[i]; volatile float p = beta * d; v = z[i] + p; }
        if (y) y[i] = v;
        if (fabsf(v) > am) am = fabsf(v);
    }
    return am;
}

/* crates/cuda-kernels/src/gpt/optimizer/adam/mod.rs:86-131
 * (fp32_adamw_update_schedule_amax_kernel; y and amax optional). */
float orc_adamw(float *z, float *x, const float *grad, float *y, float *m1, float *m2, uint64_t len,
                float grad_scale, float lr, float wd, float beta1, float beta2, float bc1, float bc2,
                float eps, float c_avg, float sched_beta, int contract) {
    float am = 0.0f;
    float decay;
    { volatile float t = lr * wd; decay = 1.0f - t; }
    if (contract) decay = fmaf(-lr, wd, 1.0f);
    for (uint64_t i = 0; i < len; ++i) {
        float g = grad[i] * grad_scale;
        float m, v, nz, nx, yy;
        volatile float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
        if (contract) {
            m = fmaf(beta1, m1[i], omb1 * g);
            v = fmaf(beta2, m2[i], (omb2 * g) * g);
        } else {
            volatile float a = beta1 * m1[i], b = omb1 * g;
            m = a + b;
            volatile float c0 = beta2 * m2[i], d0 = omb2 * g;
            volatile float d1 = d0 * g;
            v = c0 + d1;
        }
        float upd = (m / bc1) / (sqrtf(v / bc2) + eps);
        if (contract) {
            nz = fmaf(z[i], decay, -(lr * upd));
            nx = fmaf(c_avg, nz - x[i], x[i]);
            yy = fmaf(sched_beta, nx - nz, nz);
        } else {
            volatile float p1 = z[i] * decay, p2 = lr * upd;
            nz = p1 - p2;
            volatile float e1 = nz - x[i];
            volatile float p3 = c_avg * e1;
            nx = x[i] + p3;
            volatile float e2 = nx - nz;
            volatile float p4 = sched_beta * e2;
            yy = nz + p4;
        }
        m1[i] = m; m2[i] = v; z[i] = nz; x[i] = nx;
        if (y) { y[i] = yy; if (fabsf(yy) > am) am = fabsf(yy); }
    }
    return am;
}

/* crates/cuda-kernels/tests/optimizer/polar_reference/scalar.rs:3-19 — closed form for a
 * constant matrix after one iteration with the reference's first coefficient triple. */
float orc_polar_first_iteration_scalar(float x, int rows, int cols) {
    int r = rows >= cols ? rows : cols, c = rows >= cols ? cols : rows;
    float inv_norm = 1.0f / (sqrtf((float)(r * c) * x * x) * 1.01f + 1.0e-7f);
    x = x * inv_norm;
    float xh = orc_round_f16_host_flush(x);
    float gram = (float)r * xh * xh;
    float gramh = orc_round_f16_host_flush(gram);
    float gram2 = (float)c * gramh * gramh;
    float off = fmaf(17.300388f / 1.0510101f, gram2, (-23.595886f / 1.030301f) * gram);
    float diag = off + 8.287212f / 1.01f;
    return xh * (orc_round_f16_host_flush(diag) + ((float)c - 1.0f) * orc_round_f16_host_flush(off));
}

/* The per-iteration coefficient table of
 * crates/cuda-kernels/src/gpt/optimizer/muon/polar/fused/coefficients.rs:9-42. */
void orc_polar_express_coefficients(int iterations, float *out) {
    static const float raw[5][3] = {{8.287212f, -23.595886f, 17.300388f},
                                    {4.107059f, -2.94785f, 0.5448431f},
                                    {3.948691f, -2.9089022f, 0.55181915f},
                                    {3.3184197f, -2.488488f, 0.5100489f},
                                    {2.300652f, -1.668904f, 0.4188073f}};
    for (int i = 0; i < iterations; ++i) {
        if (i < 5) {
            out[3 * i] = raw[i][0] / 1.01f;
            out[3 * i + 1] = raw[i][1] / 1.030301f;
            out[3 * i + 2] = raw[i][2] / 1.0510101f;
        } else {
            out[3 * i] = 1.875f; out[3 * i + 1] = -1.25f; out[3 * i + 2] = 0.375f;
        }
    }
}

/* Whole matrix step as the mega path orders it
 * (crates/cuda-kernels/src/gpt/optimizer/muon/fused/body.rs:14-102): momentum -> normalise
 * -> Newton-Schulz -> update (beta = sched_beta; the mega kernel passes 1.0) -> quantise x'.
 * Works in the storage orientation.  Outputs: momentum, z, x, y(=grad buffer), codes,
 * raw scales, global_scale, schedule_amax.  `U_out` (optional) receives the NS result in
 * storage layout.  Returns rcp-table misses. */
uint64_t orc_muon_step(float *grad_inout_y, uint16_t *momentum, float *z, float *x, uint32_t rows,
                       uint32_t cols, const orc_muon_params *p, const orc_rcp_table *rcp,
                       uint8_t *codes, uint8_t *raw_scales, float *global_scale,
                       float *schedule_amax, float *U_out) {
    uint64_t len = (uint64_t)rows * cols;
    float *u = (float *)malloc(len * 4);
    double s = orc_momentum(grad_inout_y, momentum, u, len, p->mu, p->grad_scale, p->nesterov,
                            p->contract);
    float inv = orc_inv_norm((float)s, p->contract);
    float first_scale = 1.0f;
    if (p->deferred_normalize) first_scale = inv;   /* one-pass prepare: s enters through iteration 0 */
    else for (uint64_t i = 0; i < len; ++i) u[i] = u[i] * inv;
    if (rows > cols)
        orc_polar_gram_tall_scaled(u, (int)rows, (int)cols, p->iterations, p->coeffs, p->round_mode, first_scale);
    else
        orc_polar_gram_scaled(u, (int)rows, (int)cols, p->iterations, p->coeffs, p->round_mode, first_scale);
    if (U_out) memcpy(U_out, u, len * 4);
    float amax[2];
    orc_update(u, z, x, grad_inout_y, len, rows, cols, p->learning_rate, p->weight_decay,
               p->average_coefficient, p->schedule_beta, p->contract, amax);
    free(u);
    *schedule_amax = amax[1];
    const float *q = p->quantize_y ? grad_inout_y : x;
    float qa = p->quantize_y ? amax[1] : amax[0];
    return orc_nvfp4_quantize(q, len, qa, p->contract, rcp, codes, raw_scales, global_scale);
}

/* Global gradient-norm clip: crates/cuda-kernels/src/gpt/optimizer/grad_clip/sumsq.rs:9-41
 * (per-chunk sum of squares) and scale.rs:10-46 (norm and scale).  Sums are taken in double
 * here; the reference sums in f32 in a grid-dependent order, so norm parity is a tolerance. */
float orc_grad_clip(const float *const *chunks, const uint32_t *lens, uint32_t chunk_count,
                    const float *extra_sums, uint32_t extra_count, float max_norm, float *norm_out) {
    double t = 0.0;
    for (uint32_t c = 0; c < chunk_count; ++c) {
        double s = 0.0;
        for (uint32_t i = 0; i < lens[c]; ++i) s += (double)chunks[c][i] * (double)chunks[c][i];
        t += (double)(float)s;
    }
    for (uint32_t i = 0; i < extra_count; ++i) t += (double)extra_sums[i];
    float norm = sqrtf((float)t);
    if (norm_out) *norm_out = norm;
    return norm > max_norm ? max_norm / (norm + 1.0e-6f) : 1.0f;
}

/* Host schedules: src/training/learning_rate/schedule.rs:24-65. */
float orc_warmup_only(uint32_t step, uint32_t warmup_steps, float start_ratio) {
    if (step < 1) step = 1;
    if (step <= warmup_steps) {
        float progress = (float)step / (float)warmup_steps;
        return start_ratio + (1.0f - start_ratio) * progress;
    }
    return 1.0f;
}
float orc_schedule_free_beta(uint32_t step, uint32_t warmup_steps, float beta1, float rho) {
    if (step < 1) step = 1;
    uint32_t warmup = warmup_steps < 2 ? 2 : warmup_steps;
    if (step <= warmup) return beta1;
    float ratio = (float)(warmup - 1) / (float)(step - 1);
    return 1.0f - powf(ratio, rho) * (1.0f - beta1);
}
float orc_schedule_free_average_coefficient(uint32_t step, uint32_t warmup_steps, float start_ratio,
                                            float *weight_sum) {
    if (step < 1) step = 1;
    float lr_max = orc_warmup_only(step, warmup_steps, start_ratio);
    float weight = powf((float)step, 0.0f) * powf(lr_max, 2.0f);
    *weight_sum += weight;
    return *weight_sum > 0.0f ? weight / *weight_sum : 0.0f;
}
