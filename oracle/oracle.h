/* CPU oracle (test infrastructure only; see oracle.c for the parity statement). */
#ifndef LLMINI_B200_ORACLE_H
#define LLMINI_B200_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_ROUND_NONE = 0, ORC_ROUND_F16 = 1, ORC_ROUND_BF16 = 2, ORC_ROUND_F16_HOST = 3 };

/* Optional table of `rcp.approx.ftz.f32` results taken from a GPU: in_bits[i] -> out_bits[i]. */
typedef struct orc_rcp_table {
    const uint32_t *in_bits;
    const uint32_t *out_bits;
    uint32_t count;
} orc_rcp_table;

typedef struct orc_muon_params {
    float mu, grad_scale, learning_rate, weight_decay, average_coefficient, schedule_beta;
    int32_t iterations;
    int32_t nesterov;
    int32_t round_mode;  /* ORC_ROUND_* applied to every GEMM operand */
    int32_t contract;    /* 1: a*b+c expressions fused to FMA */
    int32_t quantize_y;  /* 0: quantise x' (mega path); 1: quantise y */
    int32_t deferred_normalize; /* 1: operands rounded before the Frobenius scaling, which enters through the
                                   first iteration (orc_polar_gram_scaled); 0: the reference's order */
    const float *coeffs; /* iterations x (a, b, c) */
} orc_muon_params;

uint16_t orc_f32_to_bf16_bits(float v);
float orc_bf16_bits_to_f32(uint16_t b);
float orc_round_bf16(float v);
uint16_t orc_f32_to_f16_bits(float v);
float orc_f16_bits_to_f32(uint16_t h);
float orc_round_f16(float v);
float orc_round_f16_host_flush(float v);
float orc_round_operand(float v, int mode);
uint8_t orc_f32_to_e4m3(float v);
uint8_t orc_f32_to_e2m1(float v);
float orc_e4m3_value(uint8_t code);
float orc_e2m1_value(uint8_t code);
float orc_rcp_exact_ftz(float x);

float orc_four_six_global_scale(float tensor_amax);
uint32_t orc_nvfp4_rcp_inputs(float global_scale, int contract, float *out);
float orc_tensor_amax(const float *x, uint64_t len);
uint64_t orc_nvfp4_quantize(const float *x, uint64_t len, float tensor_amax, int contract,
                            const orc_rcp_table *rcp, uint8_t *codes, uint8_t *raw_scales,
                            float *global_scale);
void orc_nvfp4_dequantize(const uint8_t *codes, const uint8_t *raw_scales, float global_scale,
                          uint64_t len, float *out);

uint64_t orc_csf_encoded_len(uint64_t rows, uint64_t k);
uint64_t orc_csf_encode(const uint8_t *raw, uint64_t raw_len, uint64_t rows, uint64_t k,
                        uint8_t *out, uint64_t out_cap);
uint8_t orc_csf_scale_at(const uint8_t *s, uint64_t g);

double orc_momentum(const float *grad, uint16_t *momentum_bf16, float *u_out, uint64_t len,
                    float mu, float grad_scale, int nesterov, int contract);
float orc_inv_norm(float sumsq, int contract);
double orc_momentum_vs(const float *grad, uint16_t *momentum_bf16, uint16_t *variance_bf16, float *u_out,
                       uint64_t len, float mu, float grad_scale, int nesterov, float bias_correction_inv);
void orc_update_clip(const float *U, float *z, float *x, float *y, uint16_t *momentum_bf16, uint16_t *variance_bf16,
                     uint64_t len, uint32_t rows, uint32_t cols, float lr, float wd, float c_avg, float beta,
                     const float *factors, uint32_t offset, uint32_t head_dim, float *amax);
void orc_sign_update(float *grad_inout_y, uint16_t *momentum_bf16, uint16_t *variance_bf16, float *z, float *x,
                     uint64_t len, uint32_t rows, uint32_t cols, float mu, float grad_scale, int variance_adaptive,
                     float lr, float wd, float c_avg, float beta, const float *factors, uint32_t offset,
                     uint32_t head_dim, float *amax);
void orc_normuon_stats(const float *U, const float *z, uint32_t rows, uint32_t cols, float *second_momentum,
                       float *factors, float *stats);
void orc_update_normuon(const float *U, float *z, float *x, float *y, uint64_t len, uint32_t rows, uint32_t cols,
                        float lr, float wd, float c_avg, float beta, const float *factors, float normuon_scale,
                        float *amax);
void orc_hyperball_update(const float *U, float *z, float *x, float *y, uint16_t *momentum_bf16,
                          uint16_t *variance_bf16, uint32_t rows, uint32_t cols, float lr, float c_avg, float beta,
                          int use_schedule_free, const float *factors, const float *stats, const float *clip_factors,
                          uint32_t offset, uint32_t head_dim, float *amax);
void orc_polar_gram(float *X, int n, int m, int iterations, const float *coeffs, int round_mode);
void orc_polar_gram_tall(float *Y, int m, int n, int iterations, const float *coeffs, int round_mode);
void orc_polar_gram_scaled(float *X, int n, int m, int iterations, const float *coeffs, int round_mode,
                           float first_scale);
void orc_polar_gram_tall_scaled(float *Y, int m, int n, int iterations, const float *coeffs, int round_mode,
                                float first_scale);
void orc_set_threads(int n);
int orc_max_threads(void);
void orc_polar_three_product(float *X, int n, int m, int iterations, const float *coeffs,
                             int round_mode);
void orc_update(const float *U, float *z, float *x, float *y, uint64_t len, uint32_t rows,
                uint32_t cols, float lr, float wd, float c_avg, float beta, int contract,
                float *amax);
float orc_schedule_free_values(const float *z, const float *x, float *y, uint64_t len, float beta,
                               int contract);
float orc_adamw(float *z, float *x, const float *grad, float *y, float *m1, float *m2, uint64_t len,
                float grad_scale, float lr, float wd, float beta1, float beta2, float bc1, float bc2,
                float eps, float c_avg, float sched_beta, int contract);
float orc_polar_first_iteration_scalar(float x, int rows, int cols);
void orc_polar_express_coefficients(int iterations, float *out);
uint64_t orc_muon_step(float *grad_inout_y, uint16_t *momentum, float *z, float *x, uint32_t rows,
                       uint32_t cols, const orc_muon_params *p, const orc_rcp_table *rcp,
                       uint8_t *codes, uint8_t *raw_scales, float *global_scale,
                       float *schedule_amax, float *U_out);

float orc_grad_clip(const float *const *chunks, const uint32_t *lens, uint32_t chunk_count,
                    const float *extra_sums, uint32_t extra_count, float max_norm, float *norm_out);
float orc_warmup_only(uint32_t step, uint32_t warmup_steps, float start_ratio);
float orc_schedule_free_beta(uint32_t step, uint32_t warmup_steps, float beta1, float rho);
float orc_schedule_free_average_coefficient(uint32_t step, uint32_t warmup_steps, float start_ratio,
                                            float *weight_sum);

#ifdef __cplusplus
}
#endif
#endif
