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

// Two fp32 lanes per instruction (fma/mul .f32x2): the polynomial of two elements costs the issue slots of one.
// Matters where the activation runs beside a tensor-core main loop whose single issuing thread needs those slots.
__device__ __forceinline__ unsigned long long f32x2_pack(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f32x2_unpack(unsigned long long v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long f32x2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long f32x2_mul(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long f32x2_add(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long f32x2_splat(float a) { return f32x2_pack(a, a); }

// gelu_erf on two values at once; same polynomial, same results as the scalar form up to the sign assembly, which is
// written as max(v, 0) - |0.5 * v * erfc(x)| (equal to the scalar form's two cases).
__device__ __forceinline__ void gelu_erf_x2(float& v0, float& v1) {
    const float x0 = fminf(fabsf(v0) * 0.70710678118654752f, 4.2f), x1 = fminf(fabsf(v1) * 0.70710678118654752f, 4.2f);
    const unsigned long long x = f32x2_pack(x0, x1);
    unsigned long long q = f32x2_splat(-4.536098769e-05f);      // coefficients negated: the product below is -x * Q(x)
    q = f32x2_fma(q, x, f32x2_splat(4.455243683e-04f));
    q = f32x2_fma(q, x, f32x2_splat(-1.489487318e-03f));
    q = f32x2_fma(q, x, f32x2_splat(-7.745675391e-04f));
    q = f32x2_fma(q, x, f32x2_splat(2.825363673e-02f));
    q = f32x2_fma(q, x, f32x2_splat(-1.484815990e-01f));
    q = f32x2_fma(q, x, f32x2_splat(-9.184163958e-01f));
    q = f32x2_fma(q, x, f32x2_splat(-1.627908593e+00f));
    float t0, t1;
    f32x2_unpack(f32x2_mul(x, q), t0, t1);
    const float h0 = v0 * ex2_approx(t0), h1 = v1 * ex2_approx(t1);   // v * erfc(x)
    v0 = fmaf(-0.5f, fabsf(h0), fmaxf(v0, 0.0f));
    v1 = fmaf(-0.5f, fabsf(h1), fmaxf(v1, 0.0f));
}

// The same for results that are stored in a 16-bit type: a degree-4 exponent polynomial (three packed FMAs fewer per pair).
// Fitted like the degree-7 one; absolute error of GELU 1.1e-6, relative error 1.1e-3 wherever |GELU| > 1e-3 -- under half a
// bf16 step (2e-3) and about one f16 step (1e-3), so the stored value differs from the exact-erf result by at most one
// rounding step of the 16-bit type.
__device__ __forceinline__ void gelu_erf_x2_16bit(float& v0, float& v1) {
    // No clamp of x here: beyond the fitted range the polynomial keeps growing (Q(5) = 8.1, Q(6) = 9.9, ...), so 2^(-x Q)
    // underflows to zero as erfc does (absolute error < 1e-12 * |v|), and for huge |v| the chain saturates to -inf -> 0.
    const float a0 = fabsf(v0), a1 = fabsf(v1);
    const unsigned long long av = f32x2_pack(a0, a1);
    const unsigned long long x = f32x2_mul(av, f32x2_splat(0.70710678118654752f));
    unsigned long long q = f32x2_splat(-2.944164920e-03f);      // coefficients negated: the product below is -x * Q(x)
    q = f32x2_fma(q, x, f32x2_splat(2.959006855e-02f));
    q = f32x2_fma(q, x, f32x2_splat(-1.486656611e-01f));
    q = f32x2_fma(q, x, f32x2_splat(-9.185093504e-01f));
    q = f32x2_fma(q, x, f32x2_splat(-1.627889008e+00f));
    float t0, t1;
    f32x2_unpack(f32x2_mul(x, q), t0, t1);
    const unsigned long long e = f32x2_pack(ex2_approx(t0), ex2_approx(t1));          // erfc(x)
    const unsigned long long pos = f32x2_pack(fmaxf(v0, 0.0f), fmaxf(v1, 0.0f));
    f32x2_unpack(f32x2_fma(f32x2_mul(av, e), f32x2_splat(-0.5f), pos), v0, v1);       // max(v, 0) - 0.5 |v| erfc(x)
}

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == 1 /* PYC_B200_ACT_RELU */) return v > 0.0f ? v : 0.0f;
    if (act == 2 /* PYC_B200_ACT_GELU */) return gelu_erf(v);
    return v;
}

}  // namespace b200
