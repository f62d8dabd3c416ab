// Activation math shared by the kernels' epilogues.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

// GELU, erf form: 0.5 * v * (1 + erf(v / sqrt(2))).
// erfc(|x|) is evaluated with the five-term rational approximation of Abramowitz & Stegun 7.1.26
// (absolute error of erf <= 1.5e-7, i.e. about one fp32 ulp of 1.0) as poly(t) * exp(-x^2), t = 1/(1 + p|x|),
// and the two signs are assembled without cancellation: v < 0 uses 0.5*v*erfc(|x|) directly.
// About a third of the instructions of erff(); the epilogues are otherwise bound by it.
__device__ __forceinline__ float gelu_erf(float v) {
    const float x = fabsf(v) * 0.70710678118654752f;
    const float t = __fdividef(1.0f, fmaf(0.3275911f, x, 1.0f));  // approximate reciprocal: 1 ulp, inside the formula's own 1.5e-7
    float p = fmaf(1.061405429f, t, -1.453152027f);
    p = fmaf(p, t, 1.421413741f);
    p = fmaf(p, t, -0.284496736f);
    p = fmaf(p, t, 0.254829592f);
    const float c = p * t * __expf(-x * x);   // erfc(|x|)
    const float h = 0.5f * v * c;             // v < 0: the result; v >= 0: the part to take away from v
    return v < 0.0f ? h : v - h;
}

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == 1 /* PYC_B200_ACT_RELU */) return v > 0.0f ? v : 0.0f;
    if (act == 2 /* PYC_B200_ACT_GELU */) return gelu_erf(v);
    return v;
}

}  // namespace b200
