// Activation math shared by the kernels' epilogues.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

// 2^x on the special-function unit (2 ulp; subnormal results flush to zero).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// GELU, erf form: 0.5 * v * (1 + erf(v / sqrt(2))).
// erfc(x), x = |v|/sqrt(2), is evaluated as 2^(-x * Q(x)) with Q a degree-7 polynomial fitted on [0, 4.2] to
// -log2(erfc(x))/x, weighted by the sensitivity of erfc to Q (absolute error of erfc 1.6e-8 in exact arithmetic,
// 7.5e-8 in fp32; beyond 4.2 erfc < 3e-9 and x is clamped).  Seven FMAs and one special-function op per element;
// the two signs are assembled without cancellation: v < 0 uses 0.5*v*erfc(x) directly.
__device__ __forceinline__ float gelu_erf(float v) {
    const float x = fminf(fabsf(v) * 0.70710678118654752f, 4.2f);
    float q = 4.536098769e-05f;
    q = fmaf(q, x, -4.455243683e-04f);
    q = fmaf(q, x, 1.489487318e-03f);
    q = fmaf(q, x, 7.745675391e-04f);
    q = fmaf(q, x, -2.825363673e-02f);
    q = fmaf(q, x, 1.484815990e-01f);
    q = fmaf(q, x, 9.184163958e-01f);
    q = fmaf(q, x, 1.627908593e+00f);
    const float c = ex2_approx(-x * q);       // erfc(|x|)
    const float h = 0.5f * v * c;             // v < 0: the result; v >= 0: the part to take away from v
    return v < 0.0f ? h : v - h;
}

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == 1 /* PYC_B200_ACT_RELU */) return v > 0.0f ? v : 0.0f;
    if (act == 2 /* PYC_B200_ACT_GELU */) return gelu_erf(v);
    return v;
}

}  // namespace b200
