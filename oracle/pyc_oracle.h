/*
 * pyc_oracle.h -- TEST INFRASTRUCTURE ONLY: CPU restatement of PyC's
 * deterministic executor and of the ops it lacks (see pyc_oracle.c for the
 * PyC file:line each function follows and for which ones are unpinned).
 */
#ifndef PYC_ORACLE_H
#define PYC_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#include "pyc_b200_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_F32 = 0, ORACLE_BF16 = 1, ORACLE_F16 = 2 };

void oracle_set_threads(int n);
int oracle_get_threads(void);

uint16_t oracle_f32_to_bf16(float f);
float oracle_bf16_to_f32(uint16_t h);
uint16_t oracle_f32_to_f16(float f);
float oracle_f16_to_f32(uint16_t h);
float oracle_e4m3_to_f32(uint8_t v);
uint8_t oracle_f32_to_e4m3(float f);
void oracle_widen(int dtype, const void* src, float* dst, size_t n);
void oracle_narrow(int dtype, const float* src, void* dst, size_t n);

void oracle_matmul_f32(const float* a, const float* b, float* c, size_t m, size_t k, size_t n);
void oracle_add(const float* a, const float* b, float* out, size_t n);
void oracle_add_row_bias(const float* a, const float* bias, float* out, size_t rows, size_t cols);
void oracle_add_scalar(const float* a, float s, float* out, size_t n);
void oracle_relu(const float* a, float* out, size_t n);
void oracle_gelu(const float* a, float* out, size_t n);
void oracle_layernorm(const float* x, const float* gamma, const float* beta, float* out, size_t rows, size_t cols, float eps);
void oracle_reduce_sum(const float* x, float* out, size_t rows, size_t cols);
void oracle_softmax(const float* x, float* out, size_t rows, size_t cols);
void oracle_attention(const float* q, const float* k, const float* v, float* out, int batch_heads, int seq, int d, float scale, int causal);
void oracle_conv2d_nhwc(const float* in, const float* w, const float* bias, float* out, int N, int H, int W, int C, int K, int R, int S,
                        int pad_h, int pad_w, int stride_h, int stride_w, int relu);
int oracle_run_module(const pyc_ir_module* m, const pyc_tensor* inputs, size_t input_count, pyc_tensor* outputs, size_t output_count);

#ifdef __cplusplus
}
#endif
#endif
