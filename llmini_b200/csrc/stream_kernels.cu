// HBM-bound stages of the Muon + NVFP4 path as coalesced, 128-bit vectorised streaming
// kernels: momentum / Nesterov / Frobenius norm (stages M+N), master update with the
// schedule-free interpolation (stage U), NVFP4 absmax -> scale -> pack (stage Q), AdamW and
// the stand-alone quantiser entry points.
//
// Multi-slot kernels walk a flat list of 2048-value chunks over every matrix of the plan
// (grid-stride, grid = SM count x resident CTAs), so one launch covers the whole step.
// The file is compiled with -fmad=false: `a*b + c` is never fused unless written as fmaf,
// which is how the reference's Rust expressions behave.
#include <algorithm>

#include <cuda_fp16.h>

#include "common.cuh"
#include "internal.h"

namespace b2 {

// ---------------------------------------------------------------------------------------------
// stage M arithmetic: crates/cuda-kernels/src/gpt/optimizer/muon/fused/momentum.rs:46-55
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float momentum_update(float graw, float pm, float mu, float grad_scale,
                                                 int nesterov, float &next_m) {
    float g = graw * grad_scale;
    float omg = (1.0f - mu) * g;
    next_m = mu * pm + omg;
    return nesterov ? mu * next_m + omg : next_m;
}

// Same stage with the variance-adaptive branch (Muon-VS, momentum.rs:86-133); `next_v` is the
// new variance state.  Operation order follows the reference expression by expression.
__device__ __forceinline__ float momentum_update_vs(float graw, float pm, float pv, float mu, float grad_scale,
                                                    int nesterov, float bias_correction_inv, float &next_m,
                                                    float &next_v) {
    const float g = graw * grad_scale;
    const float one_minus_mu = 1.0f - mu;
    const float variance_factor = mu * one_minus_mu;
    next_m = mu * pm + one_minus_mu * g;
    const float innovation = pm - g;
    next_v = mu * pv + variance_factor * innovation * innovation;
    const float corrected = next_m * bias_correction_inv;
    const float numerator = nesterov ? g + (mu / one_minus_mu) * corrected : corrected;
    return numerator / (sqrtf(fmaxf(next_v * bias_correction_inv, 0.0f)) + 1.0e-8f);
}
// Four consecutive elements of stage M in either variant.
struct Quad { float u[4], m[4], v[4]; };
template <int VS>
__device__ __forceinline__ Quad momentum_quad(const float *grad, const uint16_t *mom, const uint16_t *var, uint32_t i,
                                              const MomentumParams &mp, bool streaming) {
    Quad q;
    const float4 g = streaming ? __ldcs(reinterpret_cast<const float4 *>(grad + i))
                               : *reinterpret_cast<const float4 *>(grad + i);
    const uint2 m = *reinterpret_cast<const uint2 *>(mom + i);
    const float gr[4] = {g.x, g.y, g.z, g.w};
    const float pm[4] = {bf16_bits_to_f32(m.x & 0xffffu), bf16_bits_to_f32(m.x >> 16),
                         bf16_bits_to_f32(m.y & 0xffffu), bf16_bits_to_f32(m.y >> 16)};
    if (VS) {
        const uint2 v = *reinterpret_cast<const uint2 *>(var + i);
        const float pv[4] = {bf16_bits_to_f32(v.x & 0xffffu), bf16_bits_to_f32(v.x >> 16),
                             bf16_bits_to_f32(v.y & 0xffffu), bf16_bits_to_f32(v.y >> 16)};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            q.u[e] = momentum_update_vs(gr[e], pm[e], pv[e], mp.mu, mp.grad_scale, mp.nesterov,
                                        mp.bias_correction_inv, q.m[e], q.v[e]);
    } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            q.u[e] = momentum_update(gr[e], pm[e], mp.mu, mp.grad_scale, mp.nesterov, q.m[e]);
            q.v[e] = 0.0f;
        }
    }
    return q;
}
__device__ __forceinline__ uint2 pack_bf16x4(const float *v) {
    uint2 o;
    o.x = f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16);
    o.y = f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16);
    return o;
}
// Per-head qk-clip factor of element `i` (update.rs:58-66; one row of `cols` values per chunk there).
// `row` = element index / cols, computed once by the caller (integer division is the expensive
// part of this stage's index arithmetic).
__device__ __forceinline__ float qk_clip_factor(const b2_muon_slot_descriptor &d, const float *factors, uint32_t row) {
    if (factors == nullptr || d.qk_clip_factor_offset == 0xffffffffu || d.qk_clip_head_dim == 0) return 1.0f;
    if (row >= 2u * d.cols) return 1.0f;
    const uint32_t in_block = row >= d.cols ? row - d.cols : row;   // row % cols for row < 2 cols
    return __ldg(factors + d.qk_clip_factor_offset + in_block / d.qk_clip_head_dim);
}

struct ChunkCtx {
    uint32_t slot;
    uint32_t local_chunk;
    uint32_t len;
    b2_muon_slot_descriptor d;
};
__device__ __forceinline__ ChunkCtx chunk_ctx(const b2_muon_slot_descriptor *slots,
                                              const uint32_t *prefix, uint32_t slot_count,
                                              uint32_t c) {
    ChunkCtx x;
    x.slot = find_slot(prefix, slot_count, c);
    x.local_chunk = c - prefix[x.slot];
    x.d = slots[x.slot];
    x.len = x.d.rows * x.d.cols;
    return x;
}

// Pass 1 of stages M+N: sum of u^2 per chunk: an f32 fma chain over a thread's eight values,
// then f64 across threads, warps and chunks, so the grid shape does not change the result.  Also clears the two amax
// words the update kernel later raises with atomicMax.
template <int VS>
__global__ void __launch_bounds__(kThreads, VS ? 4 : 6)
k_muon_sumsq(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
             uint32_t total_chunks, MomentumParams mp, double *partials, float *amax_x) {
    // Two chunks per trip: both chunks' loads are in flight together and one pair of barriers
    // serves both block reductions.  Every chunk still leaves its own partial, summed in the same
    // order as before, so the result does not depend on the pairing.
    __shared__ double warp_part[2][kThreads / 32];
    const int tid = threadIdx.x;
    if (mp.d_grad_scale) mp.grad_scale = __ldg(mp.d_grad_scale);
    for (uint32_t c0 = 2 * blockIdx.x; c0 < total_chunks; c0 += 2 * gridDim.x) {
        float local[2] = {0.0f, 0.0f};
        uint32_t reset_slot[2] = {0xffffffffu, 0xffffffffu};
        uint64_t reset_amax[2] = {0, 0};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t c = c0 + k;
            if (c >= total_chunks) break;   // CTA-uniform
            ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
            const float *grad = reinterpret_cast<const float *>(cx.d.grad);
            const uint16_t *mom = reinterpret_cast<const uint16_t *>(cx.d.momentum);
            const uint16_t *var = reinterpret_cast<const uint16_t *>(cx.d.variance);
            const uint32_t base = cx.local_chunk * kChunk;
            if (cx.local_chunk == 0) {
                reset_slot[k] = cx.slot;
                reset_amax[k] = cx.d.schedule_amax;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t i = base + h * (kChunk / 2) + tid * 4;
                if (i < cx.len) {
                    const Quad q = momentum_quad<VS>(grad, mom, var, i, mp, false);
                    // per-thread chain as in the reference (momentum.rs:63: fma(update, update, sum));
                    // eight terms at most, so the chain's rounding stays below 1e-7 relative
#pragma unroll
                    for (int e = 0; e < 4; ++e) local[k] = fmaf(q.u[e], q.u[e], local[k]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const double acc = warp_sum((double)local[k]);
            if ((tid & 31) == 0) warp_part[k][tid >> 5] = acc;
        }
        __syncthreads();
        if (tid < 2 && c0 + tid < total_chunks) {
            double s = 0.0;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) s += warp_part[tid][w];
            partials[c0 + tid] = s;
            const uint32_t rs = tid == 0 ? reset_slot[0] : reset_slot[1];
            const uint64_t ra = tid == 0 ? reset_amax[0] : reset_amax[1];
            if (rs != 0xffffffffu) {
                amax_x[rs] = 0.0f;
                *reinterpret_cast<float *>(ra) = 0.0f;
            }
        }
        __syncthreads();
    }
}

// One CTA per slot: fixed-order sum of the slot's chunk partials, then
// inv = 1 / (sqrt(S) * 1.01 + 1e-7)
// (crates/cuda-kernels/src/gpt/optimizer/muon/polar/fused/normalize.rs:8-9,82-86).
__global__ void __launch_bounds__(kThreads)
k_muon_inv_norm(const uint32_t *prefix, const double *partials, float *inv_norm, uint32_t per_chunk) {
    __shared__ double warp_part[kThreads / 32];
    const uint32_t s = blockIdx.x;
    const uint32_t begin = prefix[s] * per_chunk, end = prefix[s + 1] * per_chunk;
    double acc = 0.0;
    for (uint32_t c = begin + threadIdx.x; c < end; c += kThreads) acc += partials[c];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) t += warp_part[w];
        float sum = (float)t;
        inv_norm[s] = 1.0f / (sqrtf(sum) * 1.01f + 1.0e-7f);
    }
}

// Pass 2 of stages M+N: stores the BF16 momentum state and X0 = r16(u * inv) in the storage
// layout [rows][cols] (momentum.rs:56-63 and normalize.rs:137-143; operand rounding
// .../polar/fused/stage.rs:51-55).  No transpose: the GEMMs read either orientation.
template <int VS>
__global__ void __launch_bounds__(kThreads, VS ? 4 : 8)
k_muon_momentum_normalize(const b2_muon_slot_descriptor *slots, const uint32_t *prefix,
                          uint32_t slot_count, uint32_t total_chunks, MomentumParams mp,
                          const float *inv_norm, const uint64_t *x0_ptrs, int f16) {
    const int tid = threadIdx.x;
    if (mp.d_grad_scale) mp.grad_scale = __ldg(mp.d_grad_scale);
    for (uint32_t c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
        const float *grad = reinterpret_cast<const float *>(cx.d.grad);
        uint16_t *mom = reinterpret_cast<uint16_t *>(cx.d.momentum);
        uint16_t *var = reinterpret_cast<uint16_t *>(cx.d.variance);
        uint16_t *x0 = reinterpret_cast<uint16_t *>(x0_ptrs[cx.slot]);
        const float inv = inv_norm[cx.slot];
        const uint32_t base = cx.local_chunk * kChunk;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t i = base + h * (kChunk / 2) + tid * 4;
            if (i < cx.len) {
                const Quad q = momentum_quad<VS>(grad, mom, var, i, mp, true);
                *reinterpret_cast<uint2 *>(mom + i) = pack_bf16x4(q.m);
                if (VS) *reinterpret_cast<uint2 *>(var + i) = pack_bf16x4(q.v);
                uint2 xo;
                xo.x = pack_operands(q.u[0] * inv, q.u[1] * inv, f16);
                xo.y = pack_operands(q.u[2] * inv, q.u[3] * inv, f16);
                *reinterpret_cast<uint2 *>(x0 + i) = xo;
            }
        }
    }
}

// Stages M+N in ONE pass over the gradients: BF16 momentum state, the UN-normalised 16-bit operand
// X0 = r16(u) in the storage layout, and the sum of u^2 (taken over the FP32 u, as normalize.rs:35-79 does).
// The Frobenius scale s = 1 / (1.01 |u| + 1e-7) is not known until every chunk of the matrix has been
// summed, so it is left to the first Newton-Schulz iteration, which is linear in it: G = (s s) X0 X0^T and
// X1 = s (Q X0) (the Gram and Apply epilogues multiply by the slot's scalar).  10 bytes per element cross
// the memory interface instead of 16.  The operand is rounded before instead of after the scaling, which is
// not the reference's rounding point; the two-pass kernels above keep that one.  BF16 operands only: an
// un-normalised F16 operand could leave F16's range.
// Every warp leaves its own f64 partial per chunk (kThreads / 32 per chunk, summed in a fixed order by
// k_muon_inv_norm), so no CTA-wide barrier sits between a chunk's loads and the next chunk's.  Two chunks
// per trip keep eight 128-bit loads per thread in flight.  Also clears the two amax words of each slot.
constexpr uint32_t kWarpsPerCta = kThreads / 32;
static_assert(kWarpsPerCta == B2_ONE_PASS_PARTIALS, "partials per chunk of the one-pass prepare");
template <int VS>
__global__ void __launch_bounds__(kThreads, VS ? 4 : 8)
k_muon_momentum_sumsq(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
                      uint32_t total_chunks, MomentumParams mp, const uint64_t *x0_ptrs, double *partials,
                      float *amax_x) {
    const int tid = threadIdx.x;
    if (mp.d_grad_scale) mp.grad_scale = __ldg(mp.d_grad_scale);
    for (uint32_t c0 = 2 * blockIdx.x; c0 < total_chunks; c0 += 2 * gridDim.x) {
        float local[2] = {0.0f, 0.0f};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t c = c0 + k;
            if (c >= total_chunks) break;   // CTA-uniform
            ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
            const float *grad = reinterpret_cast<const float *>(cx.d.grad);
            uint16_t *mom = reinterpret_cast<uint16_t *>(cx.d.momentum);
            uint16_t *var = reinterpret_cast<uint16_t *>(cx.d.variance);
            uint16_t *x0 = reinterpret_cast<uint16_t *>(x0_ptrs[cx.slot]);
            const uint32_t base = cx.local_chunk * kChunk;
            if (cx.local_chunk == 0 && tid == 0) {
                amax_x[cx.slot] = 0.0f;
                *reinterpret_cast<float *>(cx.d.schedule_amax) = 0.0f;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t i = base + h * (kChunk / 2) + tid * 4;
                if (i < cx.len) {
                    const Quad q = momentum_quad<VS>(grad, mom, var, i, mp, true);
                    *reinterpret_cast<uint2 *>(mom + i) = pack_bf16x4(q.m);
                    if (VS) *reinterpret_cast<uint2 *>(var + i) = pack_bf16x4(q.v);
                    uint2 xo;
                    xo.x = pack_operands(q.u[0], q.u[1], 0);
                    xo.y = pack_operands(q.u[2], q.u[3], 0);
                    *reinterpret_cast<uint2 *>(x0 + i) = xo;
#pragma unroll
                    for (int e = 0; e < 4; ++e) local[k] = fmaf(q.u[e], q.u[e], local[k]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (c0 + k >= total_chunks) break;
            const double acc = warp_sum((double)local[k]);
            if ((tid & 31) == 0) partials[(size_t)(c0 + k) * kWarpsPerCta + (tid >> 5)] = acc;
        }
    }
}

// Per-slot SymExpLin scalars for the update kernels (tma_split.rs:38-55): identity unless the step
// asks for the transform; unit scales unless the slot's entry carries scale scalars.
__device__ __forceinline__ SymExpLin symexp_for_slot(const UpdateParams &up, uint32_t slot) {
    SymExpLin s = {up.symexp_beta, 1.0f, 1.0f, 1.0f};
    if (up.symexp_beta > 0.0f && up.symexp_slots != nullptr) {
        const b2_symexp_lin_slot_descriptor &d = up.symexp_slots[slot];
        if (d.exponential_z != 0) {
            const uint64_t p[6] = {d.exponential_z, d.exponential_x, d.linear_z, d.linear_x, d.curvature_z, d.curvature_x};
            float v[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float z = __ldg(reinterpret_cast<const float *>(p[2 * k]));
                const float x = __ldg(reinterpret_cast<const float *>(p[2 * k + 1]));
                v[k] = z + up.beta * (x - z);
            }
            s.exponential = v[0]; s.linear = v[1]; s.curvature = v[2];
        }
    }
    return s;
}

// NorMuon factors of four consecutive elements (update/one.rs:48-56): the neuron is the row when
// rows >= cols, else the column; `with_scale` multiplies in the per-slot normuon_scale.
__device__ __forceinline__ void neuron_factors(const ChunkCtx &cx, const UpdateParams &up, uint32_t i, uint32_t row,
                                               int with_scale, float *nf) {
    nf[0] = nf[1] = nf[2] = nf[3] = 1.0f;
    if (!up.normuon) return;
    const float *fp = reinterpret_cast<const float *>(up.factor_ptrs[cx.slot]);
    const float sc = with_scale ? up.slot_stats[cx.slot * 4] : 1.0f;
    if (cx.d.rows >= cx.d.cols) {
        const float f = with_scale ? __ldg(fp + row) * sc : __ldg(fp + row);
        nf[0] = nf[1] = nf[2] = nf[3] = f;
    } else {
        const float4 f = __ldg(reinterpret_cast<const float4 *>(fp + (i - row * cx.d.cols)));
        nf[0] = f.x; nf[1] = f.y; nf[2] = f.z; nf[3] = f.w;
        if (with_scale) {
#pragma unroll
            for (int e = 0; e < 4; ++e) nf[e] *= sc;
        }
    }
}

// Stage U: crates/cuda-kernels/src/gpt/optimizer/muon/fused/update/one.rs:46-85, scale from
// .../fused/update.rs:54, per-slot learning rate from .../fused/mega/slot.rs:26-29.
// U is in the storage layout, so every access is a coalesced 128-bit one.  One call handles one
// 2048-value chunk, including the CTA's contribution to both maxima.  EXT = 1: NorMuon factors,
// qk-clip or the SymExpLin transform are in play.  keep_y: y is the tensor that gets quantised
// next, so y stays cacheable and x' is streamed; otherwise the other way round.
// UFMT: how the Newton-Schulz result arrives: 0 = FP32, 1 = BF16, 2 = F16 (the 16-bit output of an Apply GEMM,
// two bytes per element less to write there and to read here).
__device__ __forceinline__ float4 load_update16(const uint16_t *U, uint32_t i, int f16) {
    uint2 w;
    asm volatile("ld.global.cs.v2.u32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(U + i));
    if (f16) {
        const __half2 a = *reinterpret_cast<const __half2 *>(&w.x), b = *reinterpret_cast<const __half2 *>(&w.y);
        const float2 fa = __half22float2(a), fb = __half22float2(b);
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
    return make_float4(bf16_bits_to_f32(w.x & 0xffffu), bf16_bits_to_f32(w.x >> 16), bf16_bits_to_f32(w.y & 0xffffu),
                       bf16_bits_to_f32(w.y >> 16));
}
template <int EXT, int UFMT = 0>
__device__ __forceinline__ void update_chunk(const ChunkCtx &cx, const uint64_t *u_ptrs, float *amax_x,
                                             const UpdateParams &up, bool keep_y, float *warp_ax, float *warp_ay) {
    const float lr = up.lr, wd = up.wd, c_avg = up.c_avg, beta = up.beta;
    const int tid = threadIdx.x;
    const float *U = reinterpret_cast<const float *>(u_ptrs[cx.slot]);
    const uint16_t *U16 = reinterpret_cast<const uint16_t *>(u_ptrs[cx.slot]);
    float *z = reinterpret_cast<float *>(cx.d.z_master);
    float *x = reinterpret_cast<float *>(cx.d.x_master);
    float *y = reinterpret_cast<float *>(cx.d.grad);
    const float lr_s = lr * cx.d.learning_rate_multiplier;
    const float scale = 0.2f * sqrtf(fmaxf((float)cx.d.rows, (float)cx.d.cols));
    const float decay = 1.0f - lr_s * wd;
    const uint32_t base = cx.local_chunk * kChunk;
    const SymExpLin sx = EXT ? symexp_for_slot(up, cx.slot) : SymExpLin{0.0f, 1.0f, 1.0f, 1.0f};
    float ax = 0.0f, ay = 0.0f;
    // all six loads of the thread go out before the first store: the stores below could alias
    // them as far as the compiler knows, so it would not hoist the second half by itself
    float4 lu[2], lz[2], lx[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t i = base + h * (kChunk / 2) + tid * 4;
        if (i < cx.len) {
            lu[h] = UFMT == 0 ? ld_stream(U + i) : load_update16(U16, i, UFMT == 2);
            lz[h] = ld_stream(z + i);
            lx[h] = ld_stream(x + i);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t i = base + h * (kChunk / 2) + tid * 4;
        if (i < cx.len) {
            const float4 u = lu[h], zv = lz[h], xv = lx[h];
            float uu[4] = {u.x, u.y, u.z, u.w};
            float zz[4] = {zv.x, zv.y, zv.z, zv.w};
            float xx[4] = {xv.x, xv.y, xv.z, xv.w};
            float yy[4];
            // the four elements share a row (cols % 16 == 0), hence one clip factor
            float nf[4] = {1.0f, 1.0f, 1.0f, 1.0f};
            const uint32_t row = EXT ? i / cx.d.cols : 0u;
            if (EXT) neuron_factors(cx, up, i, row, 1, nf);
            const float clip = EXT ? qk_clip_factor(cx.d, up.d_qk_clip_factors, row) : 1.0f;
            if (clip != 1.0f) {  // one.rs:63-72: momentum (and variance) follow the clipped weights
                uint16_t *mom = reinterpret_cast<uint16_t *>(cx.d.momentum);
                const uint2 m = *reinterpret_cast<const uint2 *>(mom + i);
                const float cm[4] = {bf16_bits_to_f32(m.x & 0xffffu) * clip, bf16_bits_to_f32(m.x >> 16) * clip,
                                     bf16_bits_to_f32(m.y & 0xffffu) * clip, bf16_bits_to_f32(m.y >> 16) * clip};
                *reinterpret_cast<uint2 *>(mom + i) = pack_bf16x4(cm);
                if (cx.d.variance != 0) {
                    uint16_t *var = reinterpret_cast<uint16_t *>(cx.d.variance);
                    const uint2 v = *reinterpret_cast<const uint2 *>(var + i);
                    const float cv[4] = {bf16_bits_to_f32(v.x & 0xffffu) * clip * clip, bf16_bits_to_f32(v.x >> 16) * clip * clip,
                                         bf16_bits_to_f32(v.y & 0xffffu) * clip * clip, bf16_bits_to_f32(v.y >> 16) * clip * clip};
                    *reinterpret_cast<uint2 *>(var + i) = pack_bf16x4(cv);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float upd = scale * (uu[e] * 1.0f * nf[e]);
                float nz = zz[e] * decay - lr_s * upd;
                float nx = xx[e] + c_avg * (nz - xx[e]);
                if (clip != 1.0f) {
                    nz *= clip;
                    nx *= clip;
                }
                float sv = nz + beta * (nx - nz);
                if (EXT) sv = symexp_forward(sv, sx);
                zz[e] = nz;
                xx[e] = nx;
                yy[e] = sv;
                ax = fmaxf(ax, fabsf(nx));
                ay = fmaxf(ay, fabsf(sv));
            }
            const float4 xo = make_float4(xx[0], xx[1], xx[2], xx[3]), yo = make_float4(yy[0], yy[1], yy[2], yy[3]);
            st_stream(z + i, make_float4(zz[0], zz[1], zz[2], zz[3]));
            // the tensor that the encode pass reads again stays cacheable
            if (keep_y) {
                st_stream(x + i, xo);
                *reinterpret_cast<float4 *>(y + i) = yo;
            } else {
                *reinterpret_cast<float4 *>(x + i) = xo;
                st_stream(y + i, yo);
            }
        }
    }
    ax = warp_max(ax);
    ay = warp_max(ay);
    if ((tid & 31) == 0) {
        warp_ax[tid >> 5] = ax;
        warp_ay[tid >> 5] = ay;
    }
    __syncthreads();
    if (tid == 0) {
        float mx = 0.0f, my = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            mx = fmaxf(mx, warp_ax[w]);
            my = fmaxf(my, warp_ay[w]);
        }
        atomic_max_nonneg(amax_x + cx.slot, mx);
        atomic_max_nonneg(reinterpret_cast<float *>(cx.d.schedule_amax), my);
    }
}

template <int EXT, int UFMT>
__global__ void __launch_bounds__(kThreads, 5)
k_muon_update(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
              uint32_t total_chunks, const uint64_t *u_ptrs, float *amax_x, UpdateParams up) {
    __shared__ float warp_ax[kThreads / 32], warp_ay[kThreads / 32];
    for (uint32_t c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
        update_chunk<EXT, UFMT>(cx, u_ptrs, amax_x, up, false, warp_ax, warp_ay);
        __syncthreads();
    }
}

// NorMuon second moment per neuron, and the Hyperball statistics when `hyperball` is set:
// crates/cuda-kernels/src/gpt/optimizer/muon/fused/tma_split.rs:285-443.  U is in the storage
// layout here, so a neuron's values are one row (rows >= cols: a warp per row) or one column
// (rows < cols: 128 columns per CTA, the eight warps striding over the rows); both read whole
// 512-byte row segments.  Per unit four partial sums leave the CTA: raw, scaled, parameter, dot.
// COLS = 0 handles the row-neuron units, COLS = 1 the column-neuron ones; each instance skips the
// other's units, so the register-hungry column form (eight loads in flight per thread) does not
// take the occupancy of the row form down with it.
template <int COLS>
__global__ void __launch_bounds__(kThreads, COLS ? 2 : 4)
k_normuon_stats(const b2_muon_slot_descriptor *slots, uint32_t slot_count, NeuronView nv, const uint64_t *u_ptrs,
                int hyperball) {
    __shared__ float col_raw[COLS ? kThreads / 32 : 1][128], col_dot[COLS ? kThreads / 32 : 1][128];
    __shared__ double part[kThreads / 32][4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t unit = blockIdx.x; unit < nv.total_units; unit += gridDim.x) {
        const uint32_t slot = find_slot(nv.unit_prefix, slot_count, unit);
        if ((slots[slot].rows < slots[slot].cols) != (COLS != 0)) continue;   // CTA-uniform
        const b2_muon_slot_descriptor d = slots[slot];
        const uint32_t local = unit - nv.unit_prefix[slot];
        const float *U = reinterpret_cast<const float *>(u_ptrs[slot]);
        const float *z = reinterpret_cast<const float *>(d.z_master);
        float *state = reinterpret_cast<float *>(d.second_momentum);
        float *factors = reinterpret_cast<float *>(nv.factor_ptrs[slot]);
        double s_raw = 0.0, s_scaled = 0.0, s_param = 0.0, s_dot = 0.0;  // meaningful on one thread per neuron
        if (!COLS) {
            // B2_NORMUON_ROWS_PER_UNIT rows per unit, kRowsPerWarp per warp, one after the other: the
            // unit's fixed cost (slot lookup, descriptor, block reduction) is paid once for all of them
            constexpr uint32_t kRowsPerWarp = B2_NORMUON_ROWS_PER_UNIT / (kThreads / 32);
            const uint32_t row0 = local * B2_NORMUON_ROWS_PER_UNIT + warp * kRowsPerWarp;
            // the old second moments are needed last: ask for them first
            float old_state[kRowsPerWarp];
#pragma unroll
            for (uint32_t j = 0; j < kRowsPerWarp; ++j)
                old_state[j] = (lane == 0 && state && row0 + j < d.rows) ? __ldcg(state + row0 + j) : 0.0f;
#pragma unroll
            for (uint32_t j = 0; j < kRowsPerWarp; ++j) {
                const uint32_t row = row0 + j;
                if (row >= d.rows) break;   // warp-uniform
                float raw = 0.0f, param = 0.0f, dot = 0.0f;
                const size_t base = (size_t)row * d.cols;
#pragma unroll 4
                for (uint32_t c = lane * 4; c < d.cols; c += 128) {
                    const float4 u = *reinterpret_cast<const float4 *>(U + base + c);
                    raw = fmaf(u.x, u.x, raw); raw = fmaf(u.y, u.y, raw);
                    raw = fmaf(u.z, u.z, raw); raw = fmaf(u.w, u.w, raw);
                    if (hyperball) {
                        const float4 p = *reinterpret_cast<const float4 *>(z + base + c);
                        param = fmaf(p.x, p.x, param); param = fmaf(p.y, p.y, param);
                        param = fmaf(p.z, p.z, param); param = fmaf(p.w, p.w, param);
                        dot = fmaf(p.x, u.x, dot); dot = fmaf(p.y, u.y, dot);
                        dot = fmaf(p.z, u.z, dot); dot = fmaf(p.w, u.w, dot);
                    }
                }
                const double r = warp_sum((double)raw), pp = warp_sum((double)param), dd = warp_sum((double)dot);
                if (lane == 0) {
                    float factor = 1.0f;
                    if (state) {
                        const float mean = (float)r / (float)d.cols;
                        const float next = 0.95f * old_state[j] + (1.0f - 0.95f) * mean;
                        factor = 1.0f / sqrtf(fmaxf(next, 1.0e-10f));
                        state[row] = next;
                    }
                    factors[row] = factor;
                    s_raw += r; s_scaled += (double)((float)r * factor * factor);
                    s_param += pp; s_dot += (double)((float)dd * factor);
                }
            }
        } else {
            const uint32_t c0 = local * 128 + lane * 4;
            float raw[4] = {0.f, 0.f, 0.f, 0.f}, dot[4] = {0.f, 0.f, 0.f, 0.f}, param = 0.0f;
            if (c0 < d.cols) {
                // eight rows per step and warp: eight independent 128-bit loads in flight per thread
                // (one at a time left each 128-column unit latency-bound at about 100 us)
                constexpr uint32_t kRowsInFlight = 8, kWarps = kThreads / 32;
                for (uint32_t r0 = warp; r0 < d.rows; r0 += kWarps * kRowsInFlight) {
                    float4 u[kRowsInFlight], p[kRowsInFlight];
#pragma unroll
                    for (uint32_t k = 0; k < kRowsInFlight; ++k) {
                        const uint32_t r = r0 + k * kWarps;
                        const size_t at = (size_t)r * d.cols + c0;
                        u[k] = r < d.rows ? *reinterpret_cast<const float4 *>(U + at) : make_float4(0.f, 0.f, 0.f, 0.f);
                        if (hyperball)
                            p[k] = r < d.rows ? *reinterpret_cast<const float4 *>(z + at) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (uint32_t k = 0; k < kRowsInFlight; ++k) {
                        const float uu[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) raw[e] = fmaf(uu[e], uu[e], raw[e]);
                        if (hyperball) {
                            const float pp[4] = {p[k].x, p[k].y, p[k].z, p[k].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                param = fmaf(pp[e], pp[e], param);
                                dot[e] = fmaf(pp[e], uu[e], dot[e]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                col_raw[warp][lane * 4 + e] = raw[e];
                col_dot[warp][lane * 4 + e] = dot[e];
            }
            s_param = (double)param;
            __syncthreads();
            const uint32_t col = local * 128 + tid;
            if (tid < 128 && col < d.cols) {
                double r = 0.0, dd = 0.0;
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w) {
                    r += (double)col_raw[w][tid];
                    dd += (double)col_dot[w][tid];
                }
                float factor = 1.0f;
                if (state) {
                    const float mean = (float)r / (float)d.rows;
                    const float next = 0.95f * state[col] + (1.0f - 0.95f) * mean;
                    factor = 1.0f / sqrtf(fmaxf(next, 1.0e-10f));
                    state[col] = next;
                }
                factors[col] = factor;
                s_raw = r; s_scaled = (double)((float)r * factor * factor);
                s_dot = (double)((float)dd * factor);
            }
        }
        s_raw = warp_sum(s_raw); s_scaled = warp_sum(s_scaled);
        s_param = warp_sum(s_param); s_dot = warp_sum(s_dot);
        if (lane == 0) {
            part[warp][0] = s_raw; part[warp][1] = s_scaled; part[warp][2] = s_param; part[warp][3] = s_dot;
        }
        __syncthreads();
        if (tid < 4) {
            double t = 0.0;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) t += part[w][tid];
            nv.partials[(size_t)unit * 4 + tid] = t;
        }
        __syncthreads();
    }
}

// One CTA per slot: fixed-order sums of the unit partials, then the four slot scalars
// (tma_split.rs:445-477 and hyperball.rs:78-105).
__global__ void __launch_bounds__(kThreads)
k_normuon_reduce(const b2_muon_slot_descriptor *slots, NeuronView nv) {
    __shared__ double part[kThreads / 32][4];
    const uint32_t slot = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t lo = nv.unit_prefix[slot], hi = nv.unit_prefix[slot + 1];
    if (lo == hi) return;
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    for (uint32_t u = lo + tid; u < hi; u += kThreads)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] += nv.partials[(size_t)u * 4 + k];
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] = warp_sum(acc[k]);
    if (lane == 0)
#pragma unroll
        for (int k = 0; k < 4; ++k) part[warp][k] = acc[k];
    __syncthreads();
    if (tid == 0) {
        double t[4] = {0.0, 0.0, 0.0, 0.0};
        for (int w = 0; w < kThreads / 32; ++w)
#pragma unroll
            for (int k = 0; k < 4; ++k) t[k] += part[w][k];
        const float scaled = fmaxf((float)t[1], 1.0e-10f);
        float *st = nv.slot_stats + slot * 4;
        st[0] = sqrtf((float)t[0] / scaled);
        st[1] = sqrtf(scaled);
        st[2] = sqrtf(fmaxf((float)t[2], 1.0e-10f));
        st[3] = (float)t[3];
    }
}

// Hyperball: the step keeps the matrix on the sphere of its current Frobenius radius
// (tma_split.rs:498-558 scalars, hyperball.rs:107-173 elements).  No weight decay on this path.
__global__ void __launch_bounds__(kThreads)
k_muon_hyperball_update(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
                        uint32_t total_chunks, const uint64_t *u_ptrs, float *amax_x, UpdateParams up,
                        int use_schedule_free) {
    __shared__ float warp_ax[kThreads / 32], warp_ay[kThreads / 32];
    const int tid = threadIdx.x;
    for (uint32_t c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
        const float *U = reinterpret_cast<const float *>(u_ptrs[cx.slot]);
        float *z = reinterpret_cast<float *>(cx.d.z_master);
        float *x = reinterpret_cast<float *>(cx.d.x_master);
        float *y = reinterpret_cast<float *>(cx.d.grad);
        const float *st = up.slot_stats + cx.slot * 4;
        const float radius = st[2], dot = st[3];
        const float update_norm = fmaxf(st[1], 1.0e-10f);
        const float step_scale = up.lr * cx.d.learning_rate_multiplier * radius / update_norm;
        const float candidate = fmaxf(radius * radius - 2.0f * step_scale * dot +
                                          step_scale * step_scale * update_norm * update_norm, 1.0e-10f);
        const float projection = radius / sqrtf(candidate);
        const SymExpLin sx = symexp_for_slot(up, cx.slot);
        const uint32_t base = cx.local_chunk * kChunk;
        float ax = 0.0f, ay = 0.0f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t i = base + h * (kChunk / 2) + tid * 4;
            if (i < cx.len) {
                const float4 u = ld_stream(U + i), zv = ld_stream(z + i), xv = ld_stream(x + i);
                const float uu[4] = {u.x, u.y, u.z, u.w};
                float zz[4] = {zv.x, zv.y, zv.z, zv.w}, xx[4] = {xv.x, xv.y, xv.z, xv.w}, yy[4], nf[4];
                const uint32_t row = i / cx.d.cols;
                neuron_factors(cx, up, i, row, 0, nf);
                const float clip = qk_clip_factor(cx.d, up.d_qk_clip_factors, row);
                if (clip != 1.0f) {
                    uint16_t *mom = reinterpret_cast<uint16_t *>(cx.d.momentum);
                    const uint2 m = *reinterpret_cast<const uint2 *>(mom + i);
                    const float cm[4] = {bf16_bits_to_f32(m.x & 0xffffu) * clip, bf16_bits_to_f32(m.x >> 16) * clip,
                                         bf16_bits_to_f32(m.y & 0xffffu) * clip, bf16_bits_to_f32(m.y >> 16) * clip};
                    *reinterpret_cast<uint2 *>(mom + i) = pack_bf16x4(cm);
                    if (cx.d.variance != 0) {
                        uint16_t *var = reinterpret_cast<uint16_t *>(cx.d.variance);
                        const uint2 v = *reinterpret_cast<const uint2 *>(var + i);
                        const float cv[4] = {bf16_bits_to_f32(v.x & 0xffffu) * clip * clip, bf16_bits_to_f32(v.x >> 16) * clip * clip,
                                             bf16_bits_to_f32(v.y & 0xffffu) * clip * clip, bf16_bits_to_f32(v.y >> 16) * clip * clip};
                        *reinterpret_cast<uint2 *>(var + i) = pack_bf16x4(cv);
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float direction = uu[e] * nf[e];
                    float pz = (zz[e] - step_scale * direction) * projection;
                    float nx = use_schedule_free ? xx[e] + up.c_avg * (pz - xx[e]) : pz;
                    if (clip != 1.0f) {
                        pz *= clip;
                        nx *= clip;
                    }
                    const float sv = symexp_forward(pz + up.beta * (nx - pz), sx);
                    zz[e] = pz; xx[e] = nx; yy[e] = sv;
                    ax = fmaxf(ax, fabsf(nx));
                    ay = fmaxf(ay, fabsf(sv));
                }
                st_stream(z + i, make_float4(zz[0], zz[1], zz[2], zz[3]));
                *reinterpret_cast<float4 *>(x + i) = make_float4(xx[0], xx[1], xx[2], xx[3]);
                *reinterpret_cast<float4 *>(y + i) = make_float4(yy[0], yy[1], yy[2], yy[3]);
            }
        }
        ax = warp_max(ax);
        ay = warp_max(ay);
        if ((tid & 31) == 0) {
            warp_ax[tid >> 5] = ax;
            warp_ay[tid >> 5] = ay;
        }
        __syncthreads();
        if (tid == 0) {
            float mx = 0.0f, my = 0.0f;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                mx = fmaxf(mx, warp_ax[w]);
                my = fmaxf(my, warp_ay[w]);
            }
            atomic_max_nonneg(amax_x + cx.slot, mx);
            atomic_max_nonneg(reinterpret_cast<float *>(cx.d.schedule_amax), my);
        }
        __syncthreads();
    }
}

// Clears the two amax words of every slot (the prepare stage does this on the Newton-Schulz path).
__global__ void k_muon_reset_amax(const b2_muon_slot_descriptor *slots, uint32_t slot_count, float *amax_x) {
    uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < slot_count && slots[s].rows * slots[s].cols != 0) {
        amax_x[s] = 0.0f;
        *reinterpret_cast<float *>(slots[s].schedule_amax) = 0.0f;
    }
}

// sign-Muon: crates/cuda-kernels/src/gpt/optimizer/muon/fused/update/one.rs:88-167
// (update_one_sign / update_sign_pair): the direction is sign(m'), no orthogonalisation.
__global__ void __launch_bounds__(kThreads)
k_muon_sign_update(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
                   uint32_t total_chunks, MomentumParams mp, UpdateParams up, float *amax_x) {
    __shared__ float warp_ax[kThreads / 32], warp_ay[kThreads / 32];
    const int tid = threadIdx.x;
    if (mp.d_grad_scale) mp.grad_scale = __ldg(mp.d_grad_scale);
    for (uint32_t c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
        float *grad = reinterpret_cast<float *>(cx.d.grad);
        uint16_t *mom = reinterpret_cast<uint16_t *>(cx.d.momentum);
        uint16_t *var = reinterpret_cast<uint16_t *>(cx.d.variance);
        float *z = reinterpret_cast<float *>(cx.d.z_master);
        float *x = reinterpret_cast<float *>(cx.d.x_master);
        const float lr_s = up.lr * cx.d.learning_rate_multiplier;
        const float decay = 1.0f - lr_s * up.wd;
        const float one_minus_mu = 1.0f - mp.mu;
        const SymExpLin sx = symexp_for_slot(up, cx.slot);
        const uint32_t base = cx.local_chunk * kChunk;
        float ax = 0.0f, ay = 0.0f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t i = base + h * (kChunk / 2) + tid * 4;
            if (i < cx.len) {
                const float4 gv = ld_stream(grad + i);
                const uint2 mb = *reinterpret_cast<const uint2 *>(mom + i);
                const float4 zv = ld_stream(z + i), xv = ld_stream(x + i);
                const float gr[4] = {gv.x, gv.y, gv.z, gv.w};
                const float pm[4] = {bf16_bits_to_f32(mb.x & 0xffffu), bf16_bits_to_f32(mb.x >> 16),
                                     bf16_bits_to_f32(mb.y & 0xffffu), bf16_bits_to_f32(mb.y >> 16)};
                float pv[4] = {0.f, 0.f, 0.f, 0.f};
                if (mp.variance_adaptive) {
                    const uint2 vb = *reinterpret_cast<const uint2 *>(var + i);
                    pv[0] = bf16_bits_to_f32(vb.x & 0xffffu); pv[1] = bf16_bits_to_f32(vb.x >> 16);
                    pv[2] = bf16_bits_to_f32(vb.y & 0xffffu); pv[3] = bf16_bits_to_f32(vb.y >> 16);
                }
                float zz[4] = {zv.x, zv.y, zv.z, zv.w}, xx[4] = {xv.x, xv.y, xv.z, xv.w};
                float nm[4], nv[4], yy[4];
                const float clip = up.d_qk_clip_factors ? qk_clip_factor(cx.d, up.d_qk_clip_factors, i / cx.d.cols) : 1.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float g = gr[e] * mp.grad_scale;
                    nm[e] = mp.mu * pm[e] + one_minus_mu * g;
                    nv[e] = 0.0f;
                    if (mp.variance_adaptive) {
                        const float innovation = pm[e] - g;
                        nv[e] = mp.mu * pv[e] + (mp.mu * one_minus_mu) * innovation * innovation;
                    }
                    const float dir = nm[e] > 0.0f ? 1.0f : (nm[e] < 0.0f ? -1.0f : 0.0f);
                    float nz = zz[e] * decay - lr_s * dir;
                    float nx = xx[e] + up.c_avg * (nz - xx[e]);
                    if (clip != 1.0f) {
                        nz *= clip;
                        nx *= clip;
                        nm[e] *= clip;
                        if (mp.variance_adaptive) nv[e] *= clip * clip;
                    }
                    const float sv = symexp_forward(nz + up.beta * (nx - nz), sx);
                    zz[e] = nz; xx[e] = nx; yy[e] = sv;
                    ax = fmaxf(ax, fabsf(nx));
                    ay = fmaxf(ay, fabsf(sv));
                }
                if (mp.variance_adaptive) *reinterpret_cast<uint2 *>(var + i) = pack_bf16x4(nv);
                *reinterpret_cast<uint2 *>(mom + i) = pack_bf16x4(nm);
                st_stream(z + i, make_float4(zz[0], zz[1], zz[2], zz[3]));
                *reinterpret_cast<float4 *>(x + i) = make_float4(xx[0], xx[1], xx[2], xx[3]);
                *reinterpret_cast<float4 *>(grad + i) = make_float4(yy[0], yy[1], yy[2], yy[3]);
            }
        }
        ax = warp_max(ax);
        ay = warp_max(ay);
        if ((tid & 31) == 0) {
            warp_ax[tid >> 5] = ax;
            warp_ay[tid >> 5] = ay;
        }
        __syncthreads();
        if (tid == 0) {
            float mx = 0.0f, my = 0.0f;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                mx = fmaxf(mx, warp_ax[w]);
                my = fmaxf(my, warp_ay[w]);
            }
            atomic_max_nonneg(amax_x + cx.slot, mx);
            atomic_max_nonneg(reinterpret_cast<float *>(cx.d.schedule_amax), my);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// stage Q: one 2048-value chunk = 128 groups of 16, one thread per group (CTAs of 128 threads).
// The arithmetic per group is that of
// crates/cuda-kernels/src/utils/nvfp4/quant/kernels/four_six/helpers.rs:41-94 and
// .../muon/fused/quant/encode.rs:37-60; the reference spreads a group over four lanes and
// repeats the scale arithmetic in each, which makes the pass issue-bound on B200 — here the
// scale is computed once per group; the loads stay fully coalesced through a per-warp
// shared-memory exchange.
// MODE 0: values come from `src`; MODE 1: values are z + beta (x - z) computed on the fly
// (crates/cuda-kernels/src/gpt/optimizer/schedule_free/value.rs:21-34).
// ---------------------------------------------------------------------------------------------
constexpr int kEncodeThreads = kChunk / 16;

// Scalars of the transform: the three scales are schedule-free pairs themselves
// (symexp_lin.rs:164-196: z + beta (x - z) with the SCHEDULE beta); no pointers = unit scales.
__device__ __forceinline__ SymExpLin symexp_resolve(const SymExpLinParams &p, float schedule_beta) {
    SymExpLin s = {p.beta, 1.0f, 1.0f, 1.0f};
    if (p.beta > 0.0f && p.scales[0] != nullptr) {
        float v[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const float z = __ldg(p.scales[2 * k]), x = __ldg(p.scales[2 * k + 1]);
            v[k] = z + schedule_beta * (x - z);
        }
        s.exponential = v[0]; s.linear = v[1]; s.curvature = v[2];
    }
    return s;
}

// The raw loads of one warp's span of a chunk (four float4 per lane, eight in MODE 1), kept apart
// from the arithmetic so that a kernel can have the next chunk's loads in flight while it encodes
// the current one.
template <int MODE>
struct EncodeRaw {
    float4 a[4];
    float4 b[MODE == 1 ? 4 : 1];
};
template <int MODE, bool L2_ONLY = false>
__device__ __forceinline__ void encode_fetch(EncodeRaw<MODE> &r, const float *src, const float *z, const float *xm,
                                             uint32_t len, uint32_t base) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t warp_first = (base / 16 + warp * 32) * 16;   // first element of this warp's span
    if (!L2_ONLY && warp_first + 512 <= len) {                  // the whole span exists (warp-uniform)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t e = warp_first + (j * 32 + lane) * 4;
            if (MODE == 0) {
                r.a[j] = L2_ONLY ? __ldcg(reinterpret_cast<const float4 *>(src + e)) : ld_stream(src + e);
            } else {
                r.a[j] = ld_stream(z + e);
                r.b[j] = ld_stream(xm + e);
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t e = warp_first + (j * 32 + lane) * 4;
        r.a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE == 1) r.b[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < len) {
            if (MODE == 0) {
                r.a[j] = L2_ONLY ? __ldcg(reinterpret_cast<const float4 *>(src + e)) : ld_stream(src + e);
            } else {
                r.a[j] = ld_stream(z + e);
                r.b[j] = ld_stream(xm + e);
            }
        }
    }
}
template <int MODE, int THREADS = kEncodeThreads, bool USE_MAGIC = true>
__device__ __forceinline__ void encode_finish(const EncodeRaw<MODE> &r, float beta, uint32_t len, uint32_t base,
                                              float gs, uint8_t *fp4, uint8_t *scales, int scale_layout,
                                              uint32_t csf_k, uint32_t csf_rows, uint32_t csf_magic,
                                              const SymExpLin sx) {
    // Each warp owns 32 consecutive groups = 2048 contiguous bytes.  It has read them with four
    // fully coalesced 128-bit loads per lane; it parks them in shared memory and every lane picks
    // up its own group.  A 128-bit access is served a quarter-warp at a time, and a group's four
    // 16-byte slots cover half of the 32 banks, so slot k of group g sits at k ^ ((g >> 1) & 3):
    // eight consecutive lanes then touch eight different bank quads on the read side (lanes =
    // groups) as well as on the write side (lanes = two groups x four slots).
    __shared__ float4 stage[THREADS / 32][128];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t group = base / 16 + threadIdx.x;
    const uint32_t i = group * 16;
    const bool valid = i < len;
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t f4 = j * 32 + lane;                       // float4 index inside the span
        float4 t = r.a[j];
        if (MODE == 1) {
            const float4 zv = r.a[j], xv = r.b[j];
            t.x = symexp_forward(zv.x + beta * (xv.x - zv.x), sx);
            t.y = symexp_forward(zv.y + beta * (xv.y - zv.y), sx);
            t.z = symexp_forward(zv.z + beta * (xv.z - zv.z), sx);
            t.w = symexp_forward(zv.w + beta * (xv.w - zv.w), sx);
        }
        const uint32_t g = f4 >> 2, k = f4 & 3;
        stage[warp][g * 4 + (k ^ ((g >> 1) & 3))] = t;
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float4 t = stage[warp][lane * 4 + (k ^ ((lane >> 1) & 3))];
        v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
    }
    __syncwarp();
    float ga = 0.0f;
#pragma unroll
    for (int e = 0; e < 16; ++e) ga = fmaxf(ga, fabsf(v[e]));
    float inv;
    const uint32_t sb = group_scale_and_inv(ga, gs, inv);
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t p0 = cvt_e2m1x2(v[8 * h + 1] * inv, v[8 * h + 0] * inv);
        uint32_t p1 = cvt_e2m1x2(v[8 * h + 3] * inv, v[8 * h + 2] * inv);
        uint32_t p2 = cvt_e2m1x2(v[8 * h + 5] * inv, v[8 * h + 4] * inv);
        uint32_t p3 = cvt_e2m1x2(v[8 * h + 7] * inv, v[8 * h + 6] * inv);
        w[h] = p0 | (p1 << 8) | (p2 << 16) | (p3 << 24);
    }
    if (valid) *reinterpret_cast<uint2 *>(fp4 + (size_t)group * 8) = make_uint2(w[0], w[1]);
    if (scale_layout == B2_SCALES_RAW) {
        if (valid) scales[group] = (uint8_t)sb;
    } else if (scale_layout == B2_SCALES_SM100) {
        // csf_k carries the row length here; a warp's 32 groups land in eight 4-byte runs
        const uint32_t per_row = csf_k / 16, row = group / per_row, kb = group - row * per_row;
        if (valid) scales[sm100_scale_offset(row, kb, (per_row + 3) / 4)] = (uint8_t)sb;
    } else {
        // eight consecutive groups (one CSF record, crates/cuda-kernels/src/utils/nvfp4/csf.rs:193-232)
        // sit in eight consecutive lanes: fold their scale bytes into the first of them
        uint32_t s2 = sb | (__shfl_down_sync(0xffffffffu, sb, 1) << 8);
        uint32_t a = s2 | (__shfl_down_sync(0xffffffffu, s2, 2) << 16);
        uint32_t b = __shfl_down_sync(0xffffffffu, a, 4);
        if ((lane & 7) == 0 && valid) csf_store_record<USE_MAGIC>(scales, csf_k, csf_rows, csf_magic, group, a, b);
    }
}
template <int MODE, int THREADS = kEncodeThreads, bool L2_ONLY = false>
__device__ __forceinline__ void encode_chunk(const float *src, const float *z, const float *xm,
                                             float beta, uint32_t len, uint32_t base, float gs,
                                             uint8_t *fp4, uint8_t *scales, int scale_layout,
                                             uint32_t csf_k, uint32_t csf_rows,
                                             const SymExpLin sx = SymExpLin{0.0f, 1.0f, 1.0f, 1.0f}) {
    EncodeRaw<MODE> r;
    encode_fetch<MODE, L2_ONLY>(r, src, z, xm, len, base);
    encode_finish<MODE, THREADS, false>(r, beta, len, base, gs, fp4, scales, scale_layout, csf_k, csf_rows, 0u, sx);
}

// Where one chunk of a stand-alone encode pass reads and writes.  `skip` marks a chunk the pass
// leaves alone (len and base are valid all the same).
struct EncodeTarget {
    const float *src, *z, *xm;
    uint8_t *fp4, *scales;
    float *gs_out;           // written by thread 0 of the tensor's first chunk
    uint32_t len, base, k, rows, magic;
    float gs;
    int layout;
    bool skip;
};
// The chunk loop of a stand-alone encode pass.  Every CTA takes one contiguous share of the chunk
// list, so the description of a tensor (descriptor, tensor maximum, scale header: a chain of
// dependent loads and a division) is worked out once per tensor and CTA and a step to the next
// chunk is one addition; `target_of(c)` gives the full description of chunk c.  Within a tensor
// the loop is software-pipelined one chunk deep: the loads of the next chunk are issued before the
// current one is encoded, so a CTA always has 8 KB (16 KB in MODE 1) in flight.  The two buffers
// swap roles in the unrolled body instead of being copied; the pipeline drains where the share
// crosses into the next tensor.
template <int MODE, typename F>
__device__ __forceinline__ void encode_pipeline(uint32_t total_chunks, float beta, const SymExpLin sx, F target_of) {
    const uint32_t per = total_chunks / gridDim.x, rem = total_chunks % gridDim.x;
    uint32_t c = blockIdx.x * per + min(blockIdx.x, rem);
    const uint32_t end = c + per + (blockIdx.x < rem ? 1u : 0u);
    EncodeRaw<MODE> ra, rb;
    while (c < end) {
        EncodeTarget t = target_of(c);
        // chunks of this tensor inside the share
        const uint32_t left = (t.len - t.base + kChunk - 1) / kChunk;
        uint32_t n = max(min(left, end - c), 1u);   // never stands still, whatever the table says
        c += n;
        if (t.skip) continue;
        if (t.base == 0 && threadIdx.x == 0) *t.gs_out = t.gs;
        encode_fetch<MODE>(ra, t.src, t.z, t.xm, t.len, t.base);
        for (;;) {
            if (n > 1) encode_fetch<MODE>(rb, t.src, t.z, t.xm, t.len, t.base + kChunk);
            encode_finish<MODE>(ra, beta, t.len, t.base, t.gs, t.fp4, t.scales, t.layout, t.k, t.rows, t.magic, sx);
            if (--n == 0) break;
            t.base += kChunk;
            if (n > 1) encode_fetch<MODE>(ra, t.src, t.z, t.xm, t.len, t.base + kChunk);
            encode_finish<MODE>(rb, beta, t.len, t.base, t.gs, t.fp4, t.scales, t.layout, t.k, t.rows, t.magic, sx);
            if (--n == 0) break;
            t.base += kChunk;
        }
    }
}

__global__ void __launch_bounds__(kEncodeThreads)
k_muon_encode(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
              uint32_t total_chunks, const float *amax_x, int quantize_y, int scale_layout) {
    encode_pipeline<0>(total_chunks, 0.f, SymExpLin{0.0f, 1.0f, 1.0f, 1.0f}, [&](uint32_t c) {
        const uint32_t slot = find_slot(prefix, slot_count, c);
        const b2_muon_slot_descriptor *d = slots + slot;
        EncodeTarget t;
        t.src = reinterpret_cast<const float *>(quantize_y ? d->grad : d->x_master);
        t.z = t.xm = nullptr;
        const float amax = quantize_y ? *reinterpret_cast<const float *>(d->schedule_amax) : amax_x[slot];
        // crates/cuda-kernels/src/gpt/optimizer/muon/fused/quant/reduce_scale.rs:66-71
        t.gs = four_six_global_scale(amax);
        t.scales = reinterpret_cast<uint8_t *>(d->scales);
        t.fp4 = reinterpret_cast<uint8_t *>(d->bytes);
        t.gs_out = reinterpret_cast<float *>(d->global_scale);
        t.k = t.rows = 0;
        if (scale_layout == B2_SCALES_CSF) {
            t.k = reinterpret_cast<const uint32_t *>(t.scales)[0];
            t.rows = reinterpret_cast<const uint32_t *>(t.scales)[1];
        } else if (scale_layout == B2_SCALES_SM100) {
            t.k = d->cols;
            t.rows = d->rows;
        }
        t.magic = scale_layout == B2_SCALES_CSF ? csf_row_magic(t.k, t.rows) : 0u;
        t.len = d->rows * d->cols;
        t.base = (c - prefix[slot]) * kChunk;
        t.layout = scale_layout;
        t.skip = false;
        return t;
    });
}

// Stand-alone flat quantiser: `fp32_to_nvfp4_four_six_kernel`
// (crates/cuda-kernels/src/utils/nvfp4/quant/kernels/four_six.rs:104-152) and
// `schedule_free_four_six_kernel` (.../optimizer/schedule_free/four_six.rs:12-54).
// Stages U and Q of every slot in ONE launch.  The tensor scale of a matrix depends on the maximum
// over the whole matrix, so its blocks can only be encoded once every update chunk of that matrix
// is done.  Work items (update chunk / encode span of 4096 values) sit in a list built with the
// plan, ordered so that the encode items of a matrix follow its own update items by a few hundred
// positions: the updated weights are then still in L2 when they are read back, and DRAM sees each
// weight once.  CTAs claim items in list order through an atomic ticket; an encode item waits
// (bounded) on its matrix's completion counter.  Every item such a wait depends on has a smaller
// ticket, hence is held by a running CTA and never waits itself, so the kernel makes progress
// whatever the number of resident CTAs.
__device__ __forceinline__ uint64_t stream_globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
struct FusedSync {   // all zero between launches: the last CTA to leave clears it again
    uint32_t ticket;
    uint32_t abort;
    uint32_t exited;
    uint32_t reserved;
    uint32_t done[1];  // slot_count entries: update chunks of the slot that are complete
};
constexpr uint32_t kItemEncode = 0x80000000u;
constexpr uint32_t kEncodeSpan = B2_FUSED_ENCODE_SPAN;  // chunks per encode item (list built by the plan)

template <int UFMT>
__global__ void __launch_bounds__(kThreads, 5)
k_muon_update_encode(const b2_muon_slot_descriptor *slots, const uint32_t *prefix, uint32_t slot_count,
                     const uint32_t *items, uint32_t item_count, const uint64_t *u_ptrs, float *amax_x,
                     UpdateParams up, int quantize_y, int scale_layout, FusedSync *sync, uint32_t *status,
                     uint64_t wait_ns) {
    __shared__ float warp_ax[kThreads / 32], warp_ay[kThreads / 32];
    __shared__ uint32_t s_ticket[2], s_ok;
    const int tid = threadIdx.x;
    if (tid == 0) s_ticket[0] = atomicAdd(&sync->ticket, 1u);
    __syncthreads();
    for (uint32_t it = 0;; ++it) {
        const uint32_t t = s_ticket[it & 1];
        if (t >= item_count) break;
        // claim the next item now and park it in a register; its latency hides behind this item
        uint32_t next_ticket = 0;
        if (tid == 0) next_ticket = atomicAdd(&sync->ticket, 1u);
        const uint32_t item = items[t];
        const uint32_t c = item & ~kItemEncode;
        ChunkCtx cx = chunk_ctx(slots, prefix, slot_count, c);
        if (!(item & kItemEncode)) {
            update_chunk<0, UFMT>(cx, u_ptrs, amax_x, up, quantize_y != 0, warp_ax, warp_ay);
            // Publish.  The barrier orders every thread's stores before thread 0's fence, which is
            // cumulative; thread 0 raised the two maxima before it.  (Letting the other warps run
            // ahead of the fence, or publishing one item late, both measured slower.)
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                atomicAdd(&sync->done[cx.slot], 1u);
            }
        } else {
            if (tid == 0) {
                const uint32_t need = prefix[cx.slot + 1] - prefix[cx.slot];
                uint32_t ok = 1;
                if (ld_acquire_u32(&sync->done[cx.slot]) < need) {
                    const uint64_t start = stream_globaltimer();
                    while (ld_acquire_u32(&sync->done[cx.slot]) < need) {
                        if (ld_acquire_u32(&sync->abort) != 0 || stream_globaltimer() - start > wait_ns) {
                            ok = 0;
                            break;
                        }
                        __nanosleep(200);
                    }
                }
                if (!ok) {
                    atomicExch(&sync->abort, 1u);
                    atomicExch(status, 1u);
                }
                __threadfence();
                s_ok = ok;
            }
            __syncthreads();
            if (!s_ok) break;   // uniform: s_ok is shared
            const float *src = reinterpret_cast<const float *>(quantize_y ? cx.d.grad : cx.d.x_master);
            const float amax = __ldcg(quantize_y ? reinterpret_cast<const float *>(cx.d.schedule_amax)
                                                 : amax_x + cx.slot);
            const float gs = four_six_global_scale(amax);
            uint8_t *scales = reinterpret_cast<uint8_t *>(cx.d.scales);
            uint32_t k = 0, rows = 0;
            if (scale_layout == B2_SCALES_CSF) {
                k = reinterpret_cast<const uint32_t *>(scales)[0];
                rows = reinterpret_cast<const uint32_t *>(scales)[1];
            } else if (scale_layout == B2_SCALES_SM100) {
                k = cx.d.cols;
                rows = cx.d.rows;
            }
            if (cx.local_chunk == 0 && tid == 0) *reinterpret_cast<float *>(cx.d.global_scale) = gs;
            // 256 threads x one 16-value group per call: kEncodeSpan chunks of the same slot
#pragma unroll
            for (uint32_t part = 0; part < kEncodeSpan / 2; ++part) {
                const uint32_t base = (cx.local_chunk + 2 * part) * kChunk;
                if (base < cx.len)
                    encode_chunk<0, kThreads, true>(src, nullptr, nullptr, 0.f, cx.len, base, gs,
                                                    reinterpret_cast<uint8_t *>(cx.d.bytes), scales, scale_layout, k, rows);
            }
        }
        if (tid == 0) s_ticket[(it + 1) & 1] = next_ticket;
        __syncthreads();
    }
    // leave the words as the next launch expects them (a memset node per step costs more)
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&sync->exited, 1u) == gridDim.x - 1) {
            for (uint32_t k = 0; k < slot_count; ++k) sync->done[k] = 0;
            sync->ticket = 0;
            sync->abort = 0;
            sync->exited = 0;
        }
    }
}

template <int MODE>
__global__ void __launch_bounds__(kEncodeThreads)
k_quantize_flat(const float *src, const float *z, const float *xm, float beta, const float *amax,
                uint8_t *fp4, uint8_t *scales, float *out_gs, uint32_t group_count,
                int scale_layout, SymExpLinParams sp) {
    const SymExpLin sx = symexp_resolve(sp, beta);
    const uint32_t len = group_count * 16;
    const uint32_t chunks = (len + kChunk - 1) / kChunk;
    const float gs = four_six_global_scale(amax[0]);
    uint32_t k = 0, rows = 0;
    if (scale_layout == B2_SCALES_CSF) {
        k = reinterpret_cast<const uint32_t *>(scales)[0];
        rows = reinterpret_cast<const uint32_t *>(scales)[1];
    }
    const uint32_t magic = scale_layout == B2_SCALES_CSF ? csf_row_magic(k, rows) : 0u;
    if (chunks == 0) {  // an empty tensor still gets its global scale
        if (blockIdx.x == 0 && threadIdx.x == 0) out_gs[0] = gs;
        return;
    }
    encode_pipeline<MODE>(chunks, beta, sx, [&](uint32_t c) {
        return EncodeTarget{src, z, xm, fp4, scales, out_gs, len, c * kChunk, k, rows, magic, gs, scale_layout, false};
    });
}

// `tensor_chunk_amax_f32_kernel` / `tensor_amax_from_chunks_f32_kernel`
// (crates/cuda-kernels/src/utils/nvfp4/quant/kernels/row_amax.rs:92-136).
__global__ void __launch_bounds__(kThreads)
k_tensor_chunk_amax(const float *x, float *chunk_amax, uint32_t n) {
    __shared__ float warp_part[kThreads / 32];
    const int tid = threadIdx.x;
    const uint32_t base = blockIdx.x * kChunk;
    float m = 0.0f;
    if (base + kChunk <= n && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float4 v = ld_stream(x + base + h * (kChunk / 2) + tid * 4);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (uint32_t i = base + tid; i < n && i < base + kChunk; i += kThreads) m = fmaxf(m, fabsf(x[i]));
    }
    m = warp_max(m);
    if ((tid & 31) == 0) warp_part[tid >> 5] = m;
    __syncthreads();
    if (tid == 0) {
        float r = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) r = fmaxf(r, warp_part[w]);
        chunk_amax[blockIdx.x] = r;
    }
}
__global__ void __launch_bounds__(kThreads)
k_tensor_amax_from_chunks(const float *chunk_amax, float *out, uint32_t count) {
    __shared__ float warp_part[kThreads / 32];
    float m = 0.0f;
    for (uint32_t i = threadIdx.x; i < count; i += kThreads) m = fmaxf(m, chunk_amax[i]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) r = fmaxf(r, warp_part[w]);
        out[0] = r;
    }
}

// `schedule_free_amax_kernel` (crates/cuda-kernels/src/gpt/optimizer/schedule_free/amax.rs:16-68).
__global__ void __launch_bounds__(kThreads)
k_schedule_free_amax(const float *z, const float *x, float beta, uint32_t len, float *amax, SymExpLinParams sp) {
    __shared__ float warp_part[kThreads / 32];
    const SymExpLin sx = symexp_resolve(sp, beta);
    const int tid = threadIdx.x;
    const uint32_t chunks = (len + kChunk - 1) / kChunk;
    float m = 0.0f;
    for (uint32_t c = blockIdx.x; c < chunks; c += gridDim.x) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t i = c * kChunk + h * (kChunk / 2) + tid * 4;
            if (i + 4 <= len) {
                float4 zv = ld_stream(z + i), xv = ld_stream(x + i);
                m = fmaxf(m, fabsf(symexp_forward(zv.x + beta * (xv.x - zv.x), sx)));
                m = fmaxf(m, fabsf(symexp_forward(zv.y + beta * (xv.y - zv.y), sx)));
                m = fmaxf(m, fabsf(symexp_forward(zv.z + beta * (xv.z - zv.z), sx)));
                m = fmaxf(m, fabsf(symexp_forward(zv.w + beta * (xv.w - zv.w), sx)));
            } else {
                for (uint32_t j = i; j < len && j < i + 4; ++j)
                    m = fmaxf(m, fabsf(symexp_forward(z[j] + beta * (x[j] - z[j]), sx)));
            }
        }
    }
    m = warp_max(m);
    if ((tid & 31) == 0) warp_part[tid >> 5] = m;
    __syncthreads();
    if (tid == 0) {
        float r = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) r = fmaxf(r, warp_part[w]);
        atomic_max_nonneg(amax, r);
    }
}

// `fp32_adamw_update_kernel` / `fp32_adamw_update_schedule_amax_kernel`
// (crates/cuda-kernels/src/gpt/optimizer/adam/mod.rs:28-131).
struct AdamScalars {
    float grad_scale, lr, wd, beta1, beta2, bc1, bc2, eps, c_avg, sched_beta;
};
__device__ __forceinline__ void adam_one(float &z, float &x, float &g_io, float &m1, float &m2,
                                         const AdamScalars &a, float decay, float &sched) {
    float g = g_io * a.grad_scale;
    float m = a.beta1 * m1 + (1.0f - a.beta1) * g;
    float v = a.beta2 * m2 + (1.0f - a.beta2) * g * g;
    float update = (m / a.bc1) / (sqrtf(v / a.bc2) + a.eps);
    float next = z * decay - a.lr * update;
    float nx = x + a.c_avg * (next - x);
    m1 = m;
    m2 = v;
    z = next;
    x = nx;
    sched = next + a.sched_beta * (nx - next);
}
// MODE 0: masters and moments only; 1: also y into the gradient buffer and max|y| (deferred
// quantisation); 2: also max|x'|, which the requantisation that follows needs, so that x' is not
// read a second time just for its maximum.
template <int MODE>
__global__ void __launch_bounds__(kThreads)
k_adamw(float *z, float *x, float *grad, float *m1, float *m2, float *amax, AdamScalars a,
        const float *d_grad_scale, uint32_t len) {
    __shared__ float warp_part[kThreads / 32];
    if (d_grad_scale) a.grad_scale = __ldg(d_grad_scale);
    const int tid = threadIdx.x;
    const float decay = 1.0f - a.lr * a.wd;
    const bool aligned = ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(x) |
                           reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m1) |
                           reinterpret_cast<uintptr_t>(m2)) & 15) == 0;
    const uint32_t chunks = (len + kChunk - 1) / kChunk;
    float am = 0.0f;
    for (uint32_t c = blockIdx.x; c < chunks; c += gridDim.x) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t i = c * kChunk + h * (kChunk / 2) + tid * 4;
            if (aligned && i + 4 <= len) {
                float4 zv = ld_stream(z + i), xv = ld_stream(x + i), gv = ld_stream(grad + i);
                float4 av = ld_stream(m1 + i), bv = ld_stream(m2 + i);
                float4 sv;
                adam_one(zv.x, xv.x, gv.x, av.x, bv.x, a, decay, sv.x);
                adam_one(zv.y, xv.y, gv.y, av.y, bv.y, a, decay, sv.y);
                adam_one(zv.z, xv.z, gv.z, av.z, bv.z, a, decay, sv.z);
                adam_one(zv.w, xv.w, gv.w, av.w, bv.w, a, decay, sv.w);
                st_stream(z + i, zv);
                *reinterpret_cast<float4 *>(x + i) = xv;
                st_stream(m1 + i, av);
                st_stream(m2 + i, bv);
                if (MODE == 1) {
                    *reinterpret_cast<float4 *>(grad + i) = sv;
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(sv.x), fabsf(sv.y)), fmaxf(fabsf(sv.z), fabsf(sv.w))));
                } else if (MODE == 2) {
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(xv.x), fabsf(xv.y)), fmaxf(fabsf(xv.z), fabsf(xv.w))));
                }
            } else {
                for (uint32_t j = i; j < len && j < i + 4; ++j) {
                    float zz = z[j], xx = x[j], gg = grad[j], aa = m1[j], bb = m2[j], ss;
                    adam_one(zz, xx, gg, aa, bb, a, decay, ss);
                    z[j] = zz; x[j] = xx; m1[j] = aa; m2[j] = bb;
                    if (MODE == 1) {
                        grad[j] = ss;
                        am = fmaxf(am, fabsf(ss));
                    } else if (MODE == 2) {
                        am = fmaxf(am, fabsf(xx));
                    }
                }
            }
        }
    }
    if (MODE != 0) {
        am = warp_max(am);
        if ((tid & 31) == 0) warp_part[tid >> 5] = am;
        __syncthreads();
        if (tid == 0) {
            float r = 0.0f;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) r = fmaxf(r, warp_part[w]);
            atomic_max_nonneg(amax, r);
        }
    }
}

// Multi-tensor AdamW: one table entry per tensor, chunks of all tensors in one flat list.
__device__ __forceinline__ uint32_t find_adam_slot(const b2_adamw_slot_descriptor *t, uint32_t count, uint32_t c) {
    uint32_t lo = 0, hi = count;
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) >> 1;
        if (t[mid].chunk_begin <= c) lo = mid;
        else hi = mid;
    }
    return lo;
}
__global__ void k_adamw_multi_reset(const b2_adamw_slot_descriptor *t, uint32_t count) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count && t[i].mode != 0 && t[i].len != 0) *reinterpret_cast<float *>(t[i].amax) = 0.0f;
}
__global__ void __launch_bounds__(kThreads)
k_adamw_multi(const b2_adamw_slot_descriptor *t, uint32_t count, uint32_t total_chunks, AdamScalars a,
              const float *d_grad_scale) {
    __shared__ float warp_part[kThreads / 32];
    const int tid = threadIdx.x;
    if (d_grad_scale) a.grad_scale = __ldg(d_grad_scale);
    const float decay = 1.0f - a.lr * a.wd;
    for (uint32_t c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        const uint32_t slot = find_adam_slot(t, count, c);
        const b2_adamw_slot_descriptor d = t[slot];
        float *z = reinterpret_cast<float *>(d.z_master), *x = reinterpret_cast<float *>(d.x_master);
        float *grad = reinterpret_cast<float *>(d.grad);
        float *m1 = reinterpret_cast<float *>(d.first_moment), *m2 = reinterpret_cast<float *>(d.second_moment);
        const uint32_t base = (c - d.chunk_begin) * kChunk;
        float am = 0.0f;
        const bool aligned = ((d.z_master | d.x_master | d.grad | d.first_moment | d.second_moment) & 15) == 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t i = base + h * (kChunk / 2) + tid * 4;
            if (aligned && i + 4 <= d.len) {
                float4 zv = ld_stream(z + i), xv = ld_stream(x + i), gv = ld_stream(grad + i);
                float4 av = ld_stream(m1 + i), bv = ld_stream(m2 + i);
                float4 sv;
                adam_one(zv.x, xv.x, gv.x, av.x, bv.x, a, decay, sv.x);
                adam_one(zv.y, xv.y, gv.y, av.y, bv.y, a, decay, sv.y);
                adam_one(zv.z, xv.z, gv.z, av.z, bv.z, a, decay, sv.z);
                adam_one(zv.w, xv.w, gv.w, av.w, bv.w, a, decay, sv.w);
                st_stream(z + i, zv);
                *reinterpret_cast<float4 *>(x + i) = xv;
                st_stream(m1 + i, av);
                st_stream(m2 + i, bv);
                if (d.mode == 1) {
                    *reinterpret_cast<float4 *>(grad + i) = sv;
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(sv.x), fabsf(sv.y)), fmaxf(fabsf(sv.z), fabsf(sv.w))));
                } else if (d.mode == 2) {
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(xv.x), fabsf(xv.y)), fmaxf(fabsf(xv.z), fabsf(xv.w))));
                }
            } else {
                for (uint32_t j = i; j < d.len && j < i + 4; ++j) {
                    float zz = z[j], xx = x[j], gg = grad[j], aa = m1[j], bb = m2[j], ss;
                    adam_one(zz, xx, gg, aa, bb, a, decay, ss);
                    z[j] = zz; x[j] = xx; m1[j] = aa; m2[j] = bb;
                    if (d.mode == 1) {
                        grad[j] = ss;
                        am = fmaxf(am, fabsf(ss));
                    } else if (d.mode == 2) {
                        am = fmaxf(am, fabsf(xx));
                    }
                }
            }
        }
        am = warp_max(am);
        if ((tid & 31) == 0) warp_part[tid >> 5] = am;
        __syncthreads();
        if (tid == 0 && d.mode != 0) {
            float r = 0.0f;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) r = fmaxf(r, warp_part[w]);
            atomic_max_nonneg(reinterpret_cast<float *>(d.amax), r);
        }
        __syncthreads();
    }
}
// mode 2 entries: x' -> NVFP4; with `deferred` set, mode 1 entries instead: the schedule-free values
// (cached in the gradient buffer when MODE == 0, rebuilt from the masters when MODE == 1).
template <int MODE>
__device__ __forceinline__ EncodeTarget adam_encode_target(const b2_adamw_slot_descriptor *t, uint32_t count,
                                                           uint32_t c, bool deferred) {
    const uint32_t slot = find_adam_slot(t, count, c);
    const b2_adamw_slot_descriptor *d = t + slot;
    EncodeTarget e;
    e.len = d->len;
    e.base = (c - d->chunk_begin) * kChunk;
    e.skip = d->mode != (deferred ? 1u : 2u);
    if (e.skip) return e;
    e.src = reinterpret_cast<const float *>(deferred ? d->grad : d->x_master);
    e.z = reinterpret_cast<const float *>(d->z_master);
    e.xm = reinterpret_cast<const float *>(d->x_master);
    e.gs = four_six_global_scale(*reinterpret_cast<const float *>(d->amax));
    e.scales = reinterpret_cast<uint8_t *>(d->scales);
    e.fp4 = reinterpret_cast<uint8_t *>(d->bytes);
    e.gs_out = reinterpret_cast<float *>(d->global_scale);
    e.layout = (int)d->scale_layout;
    e.k = e.rows = 0;
    if (d->scale_layout == B2_SCALES_CSF) {
        e.k = reinterpret_cast<const uint32_t *>(e.scales)[0];
        e.rows = reinterpret_cast<const uint32_t *>(e.scales)[1];
    }
    e.magic = d->scale_layout == B2_SCALES_CSF ? csf_row_magic(e.k, e.rows) : 0u;
    return e;
}
__global__ void __launch_bounds__(kEncodeThreads)
k_adamw_multi_encode(const b2_adamw_slot_descriptor *t, uint32_t count, uint32_t total_chunks) {
    encode_pipeline<0>(total_chunks, 0.f, SymExpLin{0.0f, 1.0f, 1.0f, 1.0f},
                       [&](uint32_t c) { return adam_encode_target<0>(t, count, c, false); });
}

// `Materializer::adam` for every deferred (mode 1) entry of the table at once
// (src/training/schedule_free/tensor.rs:71-89 -> materialize_schedule_free_precomputed):
// quantises the schedule-free values with the max|y| the update left in `amax`.  CACHED reads y
// from the gradient buffer; otherwise y = z + beta * (x - z) is rebuilt from the masters.
template <bool CACHED>
__global__ void __launch_bounds__(kEncodeThreads)
k_adamw_multi_materialize(const b2_adamw_slot_descriptor *t, uint32_t count, uint32_t total_chunks, float beta) {
    encode_pipeline<CACHED ? 0 : 1>(total_chunks, beta, SymExpLin{0.0f, 1.0f, 1.0f, 1.0f}, [&](uint32_t c) {
        return adam_encode_target<CACHED ? 0 : 1>(t, count, c, true);
    });
}

// Global gradient-norm clip: per-chunk sums of squares, the scale, and the optional in-place
// scaling (crates/cuda-kernels/src/gpt/optimizer/grad_clip/{sumsq,scale,apply}.rs).
__global__ void __launch_bounds__(kThreads)
k_grad_clip_sumsq(const uint64_t *chunk_ptrs, const uint32_t *chunk_lens, float *chunk_sums, uint32_t chunk_count) {
    __shared__ float warp_part[kThreads / 32];
    for (uint32_t c = blockIdx.x; c < chunk_count; c += gridDim.x) {
        const float *p = reinterpret_cast<const float *>(chunk_ptrs[c]);
        const uint32_t len = chunk_lens[c];
        float local = 0.0f;
        if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
            for (uint32_t i = threadIdx.x * 4; i < len; i += kThreads * 4) {
                if (i + 4 <= len) {
                    float4 v = ld_stream(p + i);
                    local += v.x * v.x; local += v.y * v.y; local += v.z * v.z; local += v.w * v.w;
                } else {
                    for (uint32_t j = i; j < len; ++j) local += p[j] * p[j];
                }
            }
        } else {
            for (uint32_t i = threadIdx.x; i < len; i += kThreads) local += p[i] * p[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = local;
        __syncthreads();
        if (threadIdx.x == 0) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) sum += warp_part[w];
            chunk_sums[c] = sum;
        }
        __syncthreads();
    }
}
__global__ void __launch_bounds__(kThreads)
k_grad_clip_scale(const float *chunk_sums, const float *extra_sums, float *scale, float *norm_out,
                  uint32_t chunk_count, uint32_t extra_count, float max_norm) {
    __shared__ double warp_part[kThreads / 32];
    double local = 0.0;
    for (uint32_t i = threadIdx.x; i < chunk_count; i += kThreads) local += (double)chunk_sums[i];
    for (uint32_t i = threadIdx.x; i < extra_count; i += kThreads) local += (double)extra_sums[i];
    local = warp_sum(local);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) t += warp_part[w];
        const float norm = sqrtf((float)t);
        scale[0] = norm > max_norm ? max_norm / (norm + 1.0e-6f) : 1.0f;  // grad_clip/scale.rs:38-43
        norm_out[0] = norm;
    }
}
__global__ void __launch_bounds__(kThreads)
k_grad_clip_apply(const uint64_t *chunk_ptrs, const uint32_t *chunk_lens, const float *scale, uint32_t chunk_count) {
    const float sc = scale[0];
    if (sc == 1.0f) return;
    for (uint32_t c = blockIdx.x; c < chunk_count; c += gridDim.x) {
        float *p = reinterpret_cast<float *>(chunk_ptrs[c]);
        const uint32_t len = chunk_lens[c];
        for (uint32_t i = threadIdx.x; i < len; i += kThreads) p[i] *= sc;
    }
}

// `zero_f32_pointer_table_kernel` (crates/cuda-kernels/src/gpt/optimizer/adam/mod.rs:18-26).
__global__ void k_zero_pointer_table(const uint64_t *ptrs, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) *reinterpret_cast<float *>(ptrs[i]) = 0.0f;
}
// `muon_storage_layout_signature_kernel` (crates/cuda-kernels/src/gpt/optimizer/storage.rs:4-17).
__global__ void k_layout_echo(uint32_t *out) {
    if (threadIdx.x == 0) {
        out[0] = B2_MUON_STORAGE_LAYOUT_VERSION;
        out[1] = (uint32_t)sizeof(b2_muon_slot_descriptor);
        out[2] = B2_ABI_VERSION;
    }
}
__global__ void k_debug_rcp(const float *in, float *out, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = rcp_approx_ftz(in[i]);
}
// One thread per group, same instruction sequence as the reference, raw scale plane.
__global__ void k_debug_quantize_literal(const float *x, const float *amax, uint8_t *fp4,
                                         uint8_t *raw_scales, float *out_gs, uint32_t group_count) {
    uint32_t g = blockIdx.x * blockDim.x + threadIdx.x;
    const float gs = four_six_global_scale(amax[0]);
    if (g == 0) out_gs[0] = gs;
    if (g >= group_count) return;
    const float *v = x + (size_t)g * 16;
    float ga = 0.0f;
    for (int i = 0; i < 16; ++i) ga = fmaxf(ga, fabsf(v[i]));
    float inv;
    uint32_t sb = group_scale_and_inv(ga, gs, inv);
    raw_scales[g] = (uint8_t)sb;
    for (int i = 0; i < 8; ++i) fp4[(size_t)g * 8 + i] = (uint8_t)cvt_e2m1x2(v[2 * i + 1] * inv, v[2 * i] * inv);
}

// ---------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------
static inline int clamp_grid(uint32_t chunks, int cap) {
    if (chunks == 0) return 0;
    return (int)(chunks < (uint32_t)cap ? chunks : (uint32_t)cap);
}

cudaError_t launch_muon_sumsq(const SlotView &v, const MomentumParams &mp, double *partials, float *amax_x,
                              cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    if (mp.variance_adaptive)
        k_muon_sumsq<1><<<clamp_grid((v.total_chunks + 1) / 2, v.grid), kThreads, 0, s>>>(
            v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, partials, amax_x);
    else
        k_muon_sumsq<0><<<clamp_grid((v.total_chunks + 1) / 2, v.grid), kThreads, 0, s>>>(
            v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, partials, amax_x);
    return cudaGetLastError();
}
cudaError_t launch_muon_momentum_sumsq(const SlotView &v, const MomentumParams &mp, const uint64_t *x0_ptrs,
                                       double *partials, float *amax_x, cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    if (mp.variance_adaptive)
        k_muon_momentum_sumsq<1><<<clamp_grid((v.total_chunks + 1) / 2, v.grid), kThreads, 0, s>>>(
            v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, x0_ptrs, partials, amax_x);
    else
        k_muon_momentum_sumsq<0><<<clamp_grid((v.total_chunks + 1) / 2, v.grid), kThreads, 0, s>>>(
            v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, x0_ptrs, partials, amax_x);
    return cudaGetLastError();
}
cudaError_t launch_muon_inv_norm(const SlotView &v, const double *partials, float *inv_norm,
                                 uint32_t partials_per_chunk, cudaStream_t s) {
    if (v.slot_count == 0) return cudaSuccess;
    k_muon_inv_norm<<<v.slot_count, kThreads, 0, s>>>(v.chunk_prefix, partials, inv_norm, partials_per_chunk);
    return cudaGetLastError();
}
cudaError_t launch_muon_momentum_normalize(const SlotView &v, const MomentumParams &mp, const float *inv_norm,
                                           const uint64_t *x0_ptrs, int f16, cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    if (mp.variance_adaptive)
        k_muon_momentum_normalize<1><<<clamp_grid(v.total_chunks, v.grid), kThreads, 0, s>>>(
            v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, inv_norm, x0_ptrs, f16);
    else
        k_muon_momentum_normalize<0><<<clamp_grid(v.total_chunks, v.grid), kThreads, 0, s>>>(
            v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, inv_norm, x0_ptrs, f16);
    return cudaGetLastError();
}
cudaError_t launch_muon_update(const SlotView &v, const uint64_t *u_ptrs, float *amax_x, const UpdateParams &up,
                               cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    const bool ext = up.normuon || up.d_qk_clip_factors || up.symexp_beta > 0.0f;
    const int grid = clamp_grid(v.total_chunks, v.grid);
#define B2_LAUNCH_UPDATE(EXT, UFMT)                                                                          \
    k_muon_update<EXT, UFMT><<<grid, kThreads, 0, s>>>(v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, \
                                                       u_ptrs, amax_x, up)
    if (up.update_format == 0) { if (ext) B2_LAUNCH_UPDATE(1, 0); else B2_LAUNCH_UPDATE(0, 0); }
    else if (up.update_format == 1) { if (ext) B2_LAUNCH_UPDATE(1, 1); else B2_LAUNCH_UPDATE(0, 1); }
    else { if (ext) B2_LAUNCH_UPDATE(1, 2); else B2_LAUNCH_UPDATE(0, 2); }
#undef B2_LAUNCH_UPDATE
    return cudaGetLastError();
}
// ---- SymExpLin scale scalars (crates/cuda-kernels/src/gpt/optimizer/symexp_lin.rs:98-283) -----
__device__ __forceinline__ void scalar_adamw(uint64_t z_p, uint64_t x_p, uint64_t g_p, uint64_t m1_p, uint64_t m2_p,
                                             const b2_symexp_lin_adamw_args &a, float lr, float wd) {
    float *z = reinterpret_cast<float *>(z_p), *x = reinterpret_cast<float *>(x_p);
    float *m1 = reinterpret_cast<float *>(m1_p), *m2 = reinterpret_cast<float *>(m2_p);
    const float g = *reinterpret_cast<const float *>(g_p) * a.grad_scale;
    const float m = a.beta1 * *m1 + (1.0f - a.beta1) * g;
    const float v = a.beta2 * *m2 + (1.0f - a.beta2) * g * g;
    const float update = (m / a.beta1_correction) / (sqrtf(v / a.beta2_correction) + a.eps);
    const float decay = 1.0f - lr * wd;
    const float next = *z * decay - lr * update;
    const float xv = *x;
    *m1 = m;
    *m2 = v;
    *z = next;
    *x = xv + a.average_coefficient * (next - xv);
}
__global__ void k_symexp_scale_adamw(const b2_symexp_lin_slot_descriptor *slots, uint32_t slot_count,
                                     b2_symexp_lin_adamw_args a) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= slot_count) return;
    const b2_symexp_lin_slot_descriptor d = slots[i];
    if (d.exponential_z == 0) return;
    scalar_adamw(d.exponential_z, d.exponential_x, d.exponential_grad, d.exponential_first, d.exponential_second, a,
                 a.exponential_linear_learning_rate, a.weight_decay);
    scalar_adamw(d.linear_z, d.linear_x, d.linear_grad, d.linear_first, d.linear_second, a,
                 a.exponential_linear_learning_rate, a.weight_decay);
    scalar_adamw(d.curvature_z, d.curvature_x, d.curvature_grad, d.curvature_first, d.curvature_second, a,
                 a.curvature_learning_rate, 0.0f);
}
__global__ void k_symexp_zero_scale_grads(const b2_symexp_lin_slot_descriptor *slots, uint32_t slot_count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= slot_count) return;
    const b2_symexp_lin_slot_descriptor d = slots[i];
    if (d.exponential_grad == 0) return;
    *reinterpret_cast<float *>(d.exponential_grad) = 0.0f;
    *reinterpret_cast<float *>(d.linear_grad) = 0.0f;
    *reinterpret_cast<float *>(d.curvature_grad) = 0.0f;
}
__global__ void k_symexp_congruent_inverse(float *raw, uint32_t len, float beta) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= len) return;
    const float target = raw[i];
    if (beta <= 0.0f || target == 0.0f) return;
    const float sign = target > 0.0f ? 1.0f : -1.0f;
    const float t = fabsf(target), inv_beta = 1.0f / beta;
    float mag = log1p_compensated(beta * t) * inv_beta;   // a tight upper bound to start from
    for (int it = 0; it < 10; ++it) {
        const float ex = exp_approx(beta * mag);
        const float residual = (ex - 1.0f + mag) * inv_beta - t;
        mag -= residual / (ex + inv_beta);
        if (mag < 0.0f) mag = 0.0f;
    }
    raw[i] = sign * mag;
}
cudaError_t launch_symexp_scale_adamw(const b2_symexp_lin_slot_descriptor *slots, uint32_t n,
                                      const b2_symexp_lin_adamw_args &a, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    k_symexp_scale_adamw<<<(n + 255) / 256, 256, 0, s>>>(slots, n, a);
    return cudaGetLastError();
}
cudaError_t launch_symexp_zero_scale_grads(const b2_symexp_lin_slot_descriptor *slots, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    k_symexp_zero_scale_grads<<<(n + 255) / 256, 256, 0, s>>>(slots, n);
    return cudaGetLastError();
}
cudaError_t launch_symexp_congruent_inverse(float *raw, uint32_t len, float beta, cudaStream_t s) {
    if (len == 0) return cudaSuccess;
    k_symexp_congruent_inverse<<<(len + 255) / 256, 256, 0, s>>>(raw, len, beta);
    return cudaGetLastError();
}

// Raw plane or CSF storage -> sm_100 block-scale operand layout; one thread per destination byte,
// so the padding of the last row band and scale-column group is written (as zero) too.
__global__ void __launch_bounds__(kThreads)
k_scales_to_sm100(const uint8_t *src, int src_csf, uint32_t rows, uint32_t per_row, uint32_t kb_tiles,
                  uint8_t *out, size_t out_bytes) {
    for (size_t o = (size_t)blockIdx.x * kThreads + threadIdx.x; o < out_bytes; o += (size_t)gridDim.x * kThreads) {
        const size_t tile = o >> 9;
        const uint32_t in = (uint32_t)(o & 511u);
        const uint32_t row = (uint32_t)(tile / kb_tiles) * 128 + ((in >> 2) & 3u) * 32 + (in >> 4);
        const uint32_t kb = (uint32_t)(tile % kb_tiles) * 4 + (in & 3u);
        uint32_t v = 0;
        if (row < rows && kb < per_row) {
            const uint32_t g = row * per_row + kb;
            v = src_csf ? csf_load_scale(src, g) : src[g];
        }
        out[o] = (uint8_t)v;
    }
}
cudaError_t launch_scales_to_sm100(const uint8_t *src, int src_csf, uint32_t rows, uint32_t cols, uint8_t *out,
                                   int grid_cap, cudaStream_t s) {
    const uint32_t per_row = cols / 16, kb_tiles = (per_row + 3) / 4;
    const size_t bytes = (size_t)((rows + 127) / 128) * kb_tiles * 512;
    if (bytes == 0) return cudaSuccess;
    const size_t blocks = (bytes + kThreads - 1) / kThreads;
    k_scales_to_sm100<<<(unsigned)std::min<size_t>(blocks, (size_t)grid_cap), kThreads, 0, s>>>(src, src_csf, rows, per_row,
                                                                                            kb_tiles, out, bytes);
    return cudaGetLastError();
}
size_t fused_sync_bytes(uint32_t slot_count) { return sizeof(FusedSync) + sizeof(uint32_t) * slot_count; }
cudaError_t launch_muon_update_encode(const SlotView &v, const uint32_t *items, uint32_t item_count,
                                      const uint64_t *u_ptrs, float *amax_x, const UpdateParams &up, int quantize_y,
                                      int scale_layout, void *sync, uint32_t *status, uint64_t wait_ns,
                                      cudaStream_t s) {
    if (item_count == 0) return cudaSuccess;
    // the plain update only: with NorMuon factors or qk-clip the two-launch form measured faster
    if (up.normuon || up.d_qk_clip_factors || up.symexp_beta > 0.0f) return cudaErrorInvalidValue;
    const int grid = clamp_grid(item_count, v.grid);
#define B2_LAUNCH_FUSED(UFMT)                                                                                     \
    k_muon_update_encode<UFMT><<<grid, kThreads, 0, s>>>(v.slots, v.chunk_prefix, v.slot_count, items, item_count,   \
                                                         u_ptrs, amax_x, up, quantize_y, scale_layout,               \
                                                         static_cast<FusedSync *>(sync), status, wait_ns)
    if (up.update_format == 0) B2_LAUNCH_FUSED(0);
    else if (up.update_format == 1) B2_LAUNCH_FUSED(1);
    else B2_LAUNCH_FUSED(2);
#undef B2_LAUNCH_FUSED
    return cudaGetLastError();
}
cudaError_t launch_normuon_stats(const SlotView &v, const NeuronView &nv, const uint64_t *u_ptrs, int hyperball,
                                 cudaStream_t s) {
    if (nv.total_units == 0) return cudaSuccess;
    k_normuon_stats<0><<<clamp_grid(nv.total_units, v.grid), kThreads, 0, s>>>(v.slots, v.slot_count, nv, u_ptrs, hyperball);
    k_normuon_stats<1><<<clamp_grid(nv.total_units, v.grid), kThreads, 0, s>>>(v.slots, v.slot_count, nv, u_ptrs, hyperball);
    k_normuon_reduce<<<v.slot_count, kThreads, 0, s>>>(v.slots, nv);
    return cudaGetLastError();
}
cudaError_t launch_muon_hyperball_update(const SlotView &v, const uint64_t *u_ptrs, float *amax_x,
                                         const UpdateParams &up, int use_schedule_free, cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    k_muon_hyperball_update<<<clamp_grid(v.total_chunks, v.grid), kThreads, 0, s>>>(
        v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, u_ptrs, amax_x, up, use_schedule_free);
    return cudaGetLastError();
}
cudaError_t launch_muon_sign_update(const SlotView &v, const MomentumParams &mp, const UpdateParams &up,
                                    float *amax_x, cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    k_muon_reset_amax<<<(v.slot_count + 255) / 256, 256, 0, s>>>(v.slots, v.slot_count, amax_x);
    k_muon_sign_update<<<clamp_grid(v.total_chunks, v.grid), kThreads, 0, s>>>(
        v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, mp, up, amax_x);
    return cudaGetLastError();
}
// Grid of a pipelined encode pass: exactly the CTAs that are resident at once (the pass is a
// grid-stride loop, so a second wave would only add a tail).  grid_cap is 8 CTAs per SM.
template <typename K>
static int encode_grid(K kernel, uint32_t chunks, int grid_cap) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kEncodeThreads, 0) != cudaSuccess || per_sm < 1)
        per_sm = 4;
    return clamp_grid(chunks, (grid_cap / 8) * per_sm);
}
cudaError_t launch_muon_encode(const SlotView &v, const float *amax_x, int quantize_y,
                               int scale_layout, cudaStream_t s) {
    if (v.total_chunks == 0) return cudaSuccess;
    k_muon_encode<<<encode_grid(k_muon_encode, v.total_chunks, v.grid), kEncodeThreads, 0, s>>>(
        v.slots, v.chunk_prefix, v.slot_count, v.total_chunks, amax_x, quantize_y, scale_layout);
    return cudaGetLastError();
}
cudaError_t launch_tensor_chunk_amax(const float *x, float *chunk_amax, uint32_t n, cudaStream_t s) {
    uint32_t chunks = (n + kChunk - 1) / kChunk;
    if (chunks == 0) return cudaSuccess;
    k_tensor_chunk_amax<<<chunks, kThreads, 0, s>>>(x, chunk_amax, n);
    return cudaGetLastError();
}
cudaError_t launch_tensor_amax_from_chunks(const float *chunk_amax, float *out, uint32_t count,
                                           cudaStream_t s) {
    k_tensor_amax_from_chunks<<<1, kThreads, 0, s>>>(chunk_amax, out, count);
    return cudaGetLastError();
}
cudaError_t launch_quantize_flat(const float *x, const float *z, const float *xm, float beta,
                                 int mode, const float *amax, uint8_t *fp4, uint8_t *scales,
                                 float *gs, uint32_t group_count, int scale_layout, int grid_cap,
                                 cudaStream_t s, const SymExpLinParams *symexp) {
    SymExpLinParams sp = {};
    if (symexp) sp = *symexp;
    uint32_t chunks = (group_count * 16 + kChunk - 1) / kChunk;
    int grid = mode == 0 ? encode_grid(k_quantize_flat<0>, chunks, grid_cap) : encode_grid(k_quantize_flat<1>, chunks, grid_cap);
    if (grid == 0) grid = 1;  // still writes the global scale
    if (mode == 0)
        k_quantize_flat<0><<<grid, kEncodeThreads, 0, s>>>(x, z, xm, beta, amax, fp4, scales, gs, group_count, scale_layout, sp);
    else
        k_quantize_flat<1><<<grid, kEncodeThreads, 0, s>>>(x, z, xm, beta, amax, fp4, scales, gs, group_count, scale_layout, sp);
    return cudaGetLastError();
}
cudaError_t launch_schedule_free_amax(const float *z, const float *x, float beta, uint32_t len,
                                      float *amax, int grid_cap, cudaStream_t s, const SymExpLinParams *symexp) {
    SymExpLinParams sp = {};
    if (symexp) sp = *symexp;
    uint32_t chunks = (len + kChunk - 1) / kChunk;
    if (chunks == 0) return cudaSuccess;
    k_schedule_free_amax<<<clamp_grid(chunks, grid_cap), kThreads, 0, s>>>(z, x, beta, len, amax, sp);
    return cudaGetLastError();
}
cudaError_t launch_adamw(const b2_adamw_update_args &a, int mode, int grid_cap,
                         cudaStream_t s) {
    uint32_t chunks = (a.len + kChunk - 1) / kChunk;
    if (chunks == 0) return cudaSuccess;
    AdamScalars sc{a.grad_scale, a.learning_rate, a.weight_decay, a.beta1, a.beta2,
                   a.beta1_correction, a.beta2_correction, a.eps, a.average_coefficient, a.schedule_beta};
    int grid = clamp_grid(chunks, grid_cap);
    if (mode == 1)
        k_adamw<1><<<grid, kThreads, 0, s>>>(a.z_master, a.x_master, a.grad, a.first_moment, a.second_moment, a.amax, sc, a.d_grad_scale, a.len);
    else if (mode == 2)
        k_adamw<2><<<grid, kThreads, 0, s>>>(a.z_master, a.x_master, a.grad, a.first_moment, a.second_moment, a.amax, sc, a.d_grad_scale, a.len);
    else
        k_adamw<0><<<grid, kThreads, 0, s>>>(a.z_master, a.x_master, a.grad, a.first_moment, a.second_moment, nullptr, sc, a.d_grad_scale, a.len);
    return cudaGetLastError();
}
cudaError_t launch_adamw_multi(const b2_adamw_slot_descriptor *table, uint32_t count, uint32_t total_chunks,
                              const b2_adamw_update_args &a, int grid_cap, cudaStream_t s) {
    if (count == 0 || total_chunks == 0) return cudaSuccess;
    AdamScalars sc{a.grad_scale, a.learning_rate, a.weight_decay, a.beta1, a.beta2,
                   a.beta1_correction, a.beta2_correction, a.eps, a.average_coefficient, a.schedule_beta};
    k_adamw_multi_reset<<<(count + 255) / 256, 256, 0, s>>>(table, count);
    k_adamw_multi<<<clamp_grid(total_chunks, grid_cap), kThreads, 0, s>>>(table, count, total_chunks, sc, a.d_grad_scale);
    k_adamw_multi_encode<<<encode_grid(k_adamw_multi_encode, total_chunks, grid_cap), kEncodeThreads, 0, s>>>(table, count, total_chunks);
    return cudaGetLastError();
}
cudaError_t launch_adamw_multi_materialize(const b2_adamw_slot_descriptor *table, uint32_t count,
                                          uint32_t total_chunks, float beta, bool cached, int grid_cap,
                                          cudaStream_t s) {
    if (count == 0 || total_chunks == 0) return cudaSuccess;
    if (cached)
        k_adamw_multi_materialize<true><<<encode_grid(k_adamw_multi_materialize<true>, total_chunks, grid_cap),
                                          kEncodeThreads, 0, s>>>(table, count, total_chunks, beta);
    else
        k_adamw_multi_materialize<false><<<encode_grid(k_adamw_multi_materialize<false>, total_chunks, grid_cap),
                                           kEncodeThreads, 0, s>>>(table, count, total_chunks, beta);
    return cudaGetLastError();
}
cudaError_t launch_grad_clip(const b2_gradient_clip_args &a, int grid_cap, cudaStream_t s) {
    if (a.chunk_count) {
        k_grad_clip_sumsq<<<clamp_grid(a.chunk_count, grid_cap), kThreads, 0, s>>>(a.chunk_ptrs, a.chunk_lens, a.chunk_sums, a.chunk_count);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    k_grad_clip_scale<<<1, kThreads, 0, s>>>(a.chunk_sums, a.extra_sums, a.scale, a.norm, a.chunk_count, a.extra_sum_count, a.max_norm);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || !a.apply || a.chunk_count == 0) return e;
    k_grad_clip_apply<<<clamp_grid(a.chunk_count, grid_cap), kThreads, 0, s>>>(a.chunk_ptrs, a.chunk_lens, a.scale, a.chunk_count);
    return cudaGetLastError();
}
cudaError_t launch_zero_pointer_table(const uint64_t *ptrs, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    k_zero_pointer_table<<<(n + 255) / 256, 256, 0, s>>>(ptrs, n);
    return cudaGetLastError();
}
cudaError_t launch_layout_echo(uint32_t *out, cudaStream_t s) {
    k_layout_echo<<<1, 32, 0, s>>>(out);
    return cudaGetLastError();
}
cudaError_t launch_debug_rcp(const float *in, float *out, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    k_debug_rcp<<<(n + 255) / 256, 256, 0, s>>>(in, out, n);
    return cudaGetLastError();
}
cudaError_t launch_debug_quantize_literal(const float *x, const float *amax, uint8_t *fp4,
                                          uint8_t *raw_scales, float *gs, uint32_t group_count,
                                          cudaStream_t s) {
    uint32_t blocks = group_count == 0 ? 1 : (group_count + 255) / 256;
    k_debug_quantize_literal<<<blocks, 256, 0, s>>>(x, amax, fp4, raw_scales, gs, group_count);
    return cudaGetLastError();
}

}  // namespace b2
