/*
 * pyc_oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement, on the CPU, of what PyC's deterministic executor
 * computes for the compiler-next hot path, plus CPU definitions for the ops
 * that executor lacks.  Only tests, the smoke check and the benchmark's CPU
 * baseline leg may link or load this file; the product library never does.
 *
 * Parity pins: oracle_matmul_f32 / oracle_add / oracle_relu and
 * oracle_run_module are checked (tests/test_oracle.py) against the
 * known-answer vectors of PyC's own tests
 *   tests/compiler_next/test_cpu_execution.c:56-59   (2x3 * 3x2 -> 22,28,49,64)
 *   tests/compiler_next/test_cpu_execution.c:135-138 (add+relu -> 1,0,1,3)
 *   tests/compiler_next/test_cuda_backend.c:84-89    (row bias + relu -> 4.5,0,2.5,13.5)
 *   tests/compiler_next/test_cuda_backend.c:261-262  (bf16 passthrough bytes)
 * and, bit for bit, against PyC's own executor compiled from its sources
 * (oracle/Makefile target `ref`, fixtures in tests/golden/).
 * GELU, LayerNorm, ReduceSum, softmax, attention, conv2d and fp8 decode have
 * no test or implementation in PyC: for those, parity is UNPINNED and the
 * definitions below are the ones the GPU kernels are held to.
 *
 * Build: gcc -O3 -ffp-contract=off -fPIC -shared -pthread (no -ffast-math, no
 * FMA contraction: PyC builds its executor with plain -O3 for baseline x86-64,
 * so every a*b+c is two roundings).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "pyc_oracle.h"

/* ------------------------------------------------------------------------ *
 * Threads: rows are independent, so splitting rows never changes a result.  *
 * ------------------------------------------------------------------------ */
static int g_threads = 1;
void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int oracle_get_threads(void) { return g_threads; }

typedef void (*row_fn)(size_t r0, size_t r1, void* ctx);
typedef struct { row_fn fn; size_t r0, r1; void* ctx; } row_job;
static void* row_worker(void* p) { row_job* j = (row_job*)p; j->fn(j->r0, j->r1, j->ctx); return NULL; }

static void parallel_rows(size_t rows, row_fn fn, void* ctx) {
    size_t nt = (size_t)g_threads;
    if (nt > rows) nt = rows;
    if (nt <= 1) { fn(0, rows, ctx); return; }
    pthread_t th[256]; row_job jobs[256];
    size_t per = (rows + nt - 1) / nt, t, started = 0;
    for (t = 0; t < nt; ++t) {
        size_t b = t * per, e = b + per > rows ? rows : b + per;
        if (b >= rows) break;
        jobs[t].fn = fn; jobs[t].r0 = b; jobs[t].r1 = e; jobs[t].ctx = ctx;
        if (pthread_create(&th[t], NULL, row_worker, &jobs[t]) != 0) { fn(b, rows, ctx); break; }
        started++;
    }
    for (t = 0; t < started; ++t) pthread_join(th[t], NULL);
}

/* ------------------------------------------------------------------------ *
 * dtype conversions                                                         *
 * ------------------------------------------------------------------------ */
/* bf16 round-to-nearest-even, the conversion PyC's bench uses
 * (benchmark/benchmarks/gpu/workloads/pyc_compiler_next_bench.c:248-256). */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float oracle_bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }

float oracle_f16_to_f32(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1f, m = h & 0x3ff, u;
    if (e == 0) {
        if (m == 0) u = s;
        else { int sh = 0; while (!(m & 0x400)) { m <<= 1; sh++; } m &= 0x3ff; u = s | ((uint32_t)(113 - sh) << 23) | (m << 13); }
    } else if (e == 31) u = s | 0x7f800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}
uint16_t oracle_f32_to_f16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    uint32_t s = (u >> 16) & 0x8000u; int32_t e = (int32_t)((u >> 23) & 0xff) - 127 + 15; uint32_t m = u & 0x7fffffu;
    if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0));
    if (e >= 31) return (uint16_t)(s | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        m |= 0x800000u; uint32_t shift = (uint32_t)(14 - e);
        uint32_t r = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) r++;
        return (uint16_t)(s | r);
    }
    uint32_t r = ((uint32_t)e << 10) | (m >> 13), rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
    return (uint16_t)(s | r);
}

/* fp8 e4m3 ("fn" variant: no infinities, 0x7f/0xff = NaN, max finite 448).
 * PyC has no fp8 code; this is the OCP 8-bit floating point definition. */
float oracle_e4m3_to_f32(uint8_t v) {
    int s = v >> 7, e = (v >> 3) & 0xf, m = v & 7; float r;
    if (e == 0xf && m == 7) return NAN;
    if (e == 0) r = ldexpf((float)m, -9); else r = ldexpf((float)(8 + m), e - 10);
    return s ? -r : r;
}
uint8_t oracle_f32_to_e4m3(float f) { /* RNE, saturating to +-448 */
    uint8_t s = signbit(f) ? 0x80 : 0; float a = fabsf(f);
    if (isnan(f)) return (uint8_t)(s | 0x7f);
    if (a >= 448.0f) return (uint8_t)(s | 0x7e);
    if (a < ldexpf(1.0f, -10)) return s; /* below half the smallest subnormal */
    int e; float fr = frexpf(a, &e);     /* a = fr * 2^e, fr in [0.5,1) */
    int E = e - 1 + 7;                    /* biased exponent of 1.x form */
    float q;
    if (E <= 0) { q = rintf(ldexpf(a, 9)); if (q >= 8.0f) return (uint8_t)(s | 0x08); return (uint8_t)(s | (uint8_t)q); }
    q = rintf(ldexpf(fr, 4));             /* 8..16 */
    if (q >= 16.0f) { q = 8.0f; E += 1; }
    if (E > 15 || (E == 15 && q > 14.0f)) return (uint8_t)(s | 0x7e);
    return (uint8_t)(s | (uint8_t)(E << 3) | ((uint8_t)q - 8));
}

void oracle_widen(int dtype, const void* src, float* dst, size_t n) {
    size_t i;
    if (dtype == ORACLE_F32) memcpy(dst, src, n * 4);
    else if (dtype == ORACLE_BF16) for (i = 0; i < n; ++i) dst[i] = oracle_bf16_to_f32(((const uint16_t*)src)[i]);
    else if (dtype == ORACLE_F16) for (i = 0; i < n; ++i) dst[i] = oracle_f16_to_f32(((const uint16_t*)src)[i]);
}
void oracle_narrow(int dtype, const float* src, void* dst, size_t n) {
    size_t i;
    if (dtype == ORACLE_F32) memcpy(dst, src, n * 4);
    else if (dtype == ORACLE_BF16) for (i = 0; i < n; ++i) ((uint16_t*)dst)[i] = oracle_f32_to_bf16(src[i]);
    else if (dtype == ORACLE_F16) for (i = 0; i < n; ++i) ((uint16_t*)dst)[i] = oracle_f32_to_f16(src[i]);
}

/* ------------------------------------------------------------------------ *
 * matmul: src/compiler/compiler_api.c:1747-1781 (matmul_compute_rows).       *
 * Per output element one fp32 accumulator, products added in ascending k,    *
 * a*b rounded before the add.  The k-blocking of 64 and the 8-way column     *
 * unroll there do not change any element's summation order, so the plain     *
 * i-k-j loop below is bit-identical.                                         *
 * ------------------------------------------------------------------------ */
typedef struct { const float* a; const float* b; float* c; size_t k, n; } mm_ctx;
static void mm_rows(size_t r0, size_t r1, void* p) {
    mm_ctx* x = (mm_ctx*)p; size_t r, kk, j;
    for (r = r0; r < r1; ++r) {
        const float* ar = x->a + r * x->k; float* cr = x->c + r * x->n;
        memset(cr, 0, x->n * sizeof(float));
        for (kk = 0; kk < x->k; ++kk) {
            float av = ar[kk]; const float* br = x->b + kk * x->n;
            for (j = 0; j < x->n; ++j) cr[j] += av * br[j];
        }
    }
}
void oracle_matmul_f32(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    mm_ctx x = { a, b, c, k, n };
    parallel_rows(m, mm_rows, &x);
}

/* add: compiler_api.c:1974-2014 (same shape); the row-bias and scalar forms
 * follow the GPU path's own CPU stand-in, cuda_backend.c:1556-1568. */
void oracle_add(const float* a, const float* b, float* out, size_t n) { size_t i; for (i = 0; i < n; ++i) out[i] = a[i] + b[i]; }
void oracle_add_row_bias(const float* a, const float* bias, float* out, size_t rows, size_t cols) {
    size_t r, c; for (r = 0; r < rows; ++r) for (c = 0; c < cols; ++c) out[r * cols + c] = a[r * cols + c] + bias[c];
}
void oracle_add_scalar(const float* a, float s, float* out, size_t n) { size_t i; for (i = 0; i < n; ++i) out[i] = a[i] + s; }
/* relu: compiler_api.c:2015-2052 */
void oracle_relu(const float* a, float* out, size_t n) { size_t i; for (i = 0; i < n; ++i) out[i] = a[i] > 0.0f ? a[i] : 0.0f; }

/* GELU, exact erf form 0.5*x*(1+erf(x/sqrt2)) -- UNPINNED: PyC's executor
 * rejects the op (compiler_api.c:2076-2083); the only hint is torch.nn.GELU()
 * in benchmark/benchmarks/gpu/workloads/standard_workload.py:58-62. Computed in
 * double and rounded once. */
void oracle_gelu(const float* a, float* out, size_t n) {
    size_t i; for (i = 0; i < n; ++i) { double x = a[i]; out[i] = (float)(0.5 * x * (1.0 + erf(x * 0.70710678118654752440))); }
}

/* LayerNorm over the last axis, biased variance, eps inside the sqrt, optional
 * affine -- UNPINNED (nn.LayerNorm(hidden) in
 * benchmark/benchmarks/gpu/ground_truth/encoder_ground_truth.py:117-121).
 * Statistics in double. */
void oracle_layernorm(const float* x, const float* gamma, const float* beta, float* out,
                      size_t rows, size_t cols, float eps) {
    size_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols; float* o = out + r * cols; double s = 0, ss = 0;
        for (c = 0; c < cols; ++c) s += xr[c];
        double mean = s / (double)cols;
        for (c = 0; c < cols; ++c) { double d = xr[c] - mean; ss += d * d; }
        double rstd = 1.0 / sqrt(ss / (double)cols + (double)eps);
        for (c = 0; c < cols; ++c) {
            double v = (xr[c] - mean) * rstd;
            if (gamma) v *= gamma[c];
            if (beta) v += beta[c];
            o[c] = (float)v;
        }
    }
}

/* ReduceSum over the trailing `cols` elements of each row -- UNPINNED. */
void oracle_reduce_sum(const float* x, float* out, size_t rows, size_t cols) {
    size_t r, c; for (r = 0; r < rows; ++r) { double s = 0; for (c = 0; c < cols; ++c) s += x[r * cols + c]; out[r] = (float)s; }
}

/* Row softmax -- UNPINNED (no softmax op in PyC's IR). */
void oracle_softmax(const float* x, float* out, size_t rows, size_t cols) {
    size_t r, c;
    for (r = 0; r < rows; ++r) {
        const float* xr = x + r * cols; float* o = out + r * cols; double mx = -INFINITY, s = 0;
        for (c = 0; c < cols; ++c) if (xr[c] > mx) mx = xr[c];
        for (c = 0; c < cols; ++c) s += exp(xr[c] - mx);
        for (c = 0; c < cols; ++c) o[c] = (float)(exp(xr[c] - mx) / s);
    }
}

/* Attention, one head per (batch*head) slice: softmax(scale * Q K^T [+causal]) V,
 * the definition in the header comment of
 * src/compiler/cutlass_kernels/attention/kernel.cu:6-8 (the kernel body there
 * copies Q) -- UNPINNED.  Scores and sums in double. */
typedef struct { const float *q, *k, *v; float* out; int s, d; float scale; int causal; } att_ctx;
static void att_rows(size_t r0, size_t r1, void* p) {
    att_ctx* x = (att_ctx*)p; size_t gr; int S = x->s, D = x->d;
    double* sc = (double*)malloc(sizeof(double) * (size_t)S);
    double* acc = (double*)malloc(sizeof(double) * (size_t)D);
    for (gr = r0; gr < r1; ++gr) {
        size_t bh = gr / (size_t)S; int i = (int)(gr % (size_t)S), j, t;
        const float* q = x->q + (bh * S + i) * D; const float* kb = x->k + bh * S * D; const float* vb = x->v + bh * S * D;
        int lim = x->causal ? i + 1 : S; double mx = -INFINITY, den = 0;
        for (j = 0; j < lim; ++j) { double s = 0; for (t = 0; t < D; ++t) s += (double)q[t] * kb[(size_t)j * D + t]; s *= x->scale; sc[j] = s; if (s > mx) mx = s; }
        for (t = 0; t < D; ++t) acc[t] = 0;
        for (j = 0; j < lim; ++j) { double pj = exp(sc[j] - mx); den += pj; for (t = 0; t < D; ++t) acc[t] += pj * vb[(size_t)j * D + t]; }
        for (t = 0; t < D; ++t) x->out[(bh * S + i) * D + t] = (float)(acc[t] / den);
    }
    free(sc); free(acc);
}
void oracle_attention(const float* q, const float* k, const float* v, float* out,
                      int batch_heads, int seq, int d, float scale, int causal) {
    att_ctx x = { q, k, v, out, seq, d, scale, causal };
    parallel_rows((size_t)batch_heads * (size_t)seq, att_rows, &x);
}

/* conv2d forward, NHWC input, KRSC filter, cross-correlation, dilation 1,
 * groups 1, symmetric padding -- the problem PyC hands to CUTLASS at
 * src/compiler/cutlass_kernels/conv2d/kernel.cu:92-98 -- UNPINNED (PyC has no
 * CPU conv).  fp32 accumulate in (r,s,c) order; bias and ReLU optional. */
typedef struct { const float *in, *w, *bias; float* out; int N, H, W, C, K, R, S, ph, pw, sh, sw, P, Q, relu; } conv_ctx;
static void conv_rows(size_t r0, size_t r1, void* p) {
    conv_ctx* x = (conv_ctx*)p; size_t row;
    for (row = r0; row < r1; ++row) { /* row = (n*P + p)*Q + q */
        int q = (int)(row % (size_t)x->Q), pp = (int)((row / (size_t)x->Q) % (size_t)x->P), n = (int)(row / ((size_t)x->Q * x->P)), k, r, s, c;
        for (k = 0; k < x->K; ++k) {
            float acc = 0.0f;
            for (r = 0; r < x->R; ++r) { int h = pp * x->sh - x->ph + r; if (h < 0 || h >= x->H) continue;
                for (s = 0; s < x->S; ++s) { int w = q * x->sw - x->pw + s; if (w < 0 || w >= x->W) continue;
                    const float* ip = x->in + (((size_t)n * x->H + h) * x->W + w) * x->C;
                    const float* wp = x->w + (((size_t)k * x->R + r) * x->S + s) * x->C;
                    for (c = 0; c < x->C; ++c) acc += ip[c] * wp[c]; } }
            if (x->bias) acc += x->bias[k];
            if (x->relu && acc < 0.0f) acc = 0.0f;
            x->out[row * (size_t)x->K + k] = acc;
        }
    }
}
void oracle_conv2d_nhwc(const float* in, const float* w, const float* bias, float* out,
                        int N, int H, int W, int C, int K, int R, int S,
                        int pad_h, int pad_w, int stride_h, int stride_w, int relu) {
    conv_ctx x = { in, w, bias, out, N, H, W, C, K, R, S, pad_h, pad_w, stride_h, stride_w,
                   (H - R + 2 * pad_h) / stride_h + 1, (W - S + 2 * pad_w) / stride_w + 1, relu };
    parallel_rows((size_t)N * x.P * x.Q, conv_rows, &x);
}

/* ------------------------------------------------------------------------ *
 * Graph walk: compiler_api.c:1877-2092 (execute_cpu_graph), widened to every *
 * op kind of the IR and to bf16/f16 storage.  All arithmetic is fp32 on the   *
 * widened inputs; outputs are narrowed once at the OUTPUT op.  ADD accepts    *
 * the three operand forms of cuda_backend.c:1201-1230.                        *
 * ------------------------------------------------------------------------ */
static size_t shape_elems(const pyc_shape* s) {
    size_t i, t = 1; if (s->rank == 0) return 0;
    for (i = 0; i < s->rank; ++i) { if (s->dims[i] <= 0) return 0; t *= (size_t)s->dims[i]; }
    return t;
}
static int dtype_tag(pyc_dtype d) { return d == PYC_DTYPE_F32 ? ORACLE_F32 : d == PYC_DTYPE_BF16 ? ORACLE_BF16 : d == PYC_DTYPE_F16 ? ORACLE_F16 : -1; }

int oracle_run_module(const pyc_ir_module* m, const pyc_tensor* inputs, size_t input_count,
                      pyc_tensor* outputs, size_t output_count) {
    float** val = (float**)calloc(m->op_count, sizeof(float*));
    size_t* ne = (size_t*)calloc(m->op_count, sizeof(size_t));
    size_t i, in_i = 0, out_i = 0; int rc = 0;
    if (!val || !ne) { free(val); free(ne); return -1; }
    for (i = 0; i < m->op_count && rc == 0; ++i) {
        const pyc_ir_op* op = &m->ops[i]; size_t n = shape_elems(&op->shape), j;
        ne[i] = n;
        for (j = 0; j < op->input_count; ++j) if (op->input_ids[j] < 0 || (size_t)op->input_ids[j] >= i || !val[op->input_ids[j]]) rc = -1;
        if (rc) break;
        switch (op->kind) {
        case PYC_IR_OP_INPUT: {
            int tag;
            if (in_i >= input_count || !inputs[in_i].data || n == 0 || (tag = dtype_tag(inputs[in_i].dtype)) < 0) { rc = -1; break; }
            if (inputs[in_i].size_bytes < n * (tag == ORACLE_F32 ? 4u : 2u)) { rc = -1; break; }
            val[i] = (float*)malloc(n * 4); oracle_widen(tag, inputs[in_i].data, val[i], n); in_i++; break; }
        case PYC_IR_OP_MATMUL: {
            const pyc_ir_op *a = &m->ops[op->input_ids[0]], *b = &m->ops[op->input_ids[1]];
            if (op->input_count < 2 || a->shape.rank != 2 || b->shape.rank != 2 || a->shape.dims[1] != b->shape.dims[0]) { rc = -1; break; }
            size_t M = (size_t)a->shape.dims[0], K = (size_t)a->shape.dims[1], N = (size_t)b->shape.dims[1];
            ne[i] = M * N; val[i] = (float*)malloc(M * N * 4);
            oracle_matmul_f32(val[op->input_ids[0]], val[op->input_ids[1]], val[i], M, K, N); break; }
        case PYC_IR_OP_ADD: {
            if (op->input_count < 2) { rc = -1; break; }
            int ia = op->input_ids[0], ib = op->input_ids[1];
            if (ne[ia] < ne[ib]) { int t = ia; ia = ib; ib = t; }
            size_t na = ne[ia], nb = ne[ib]; ne[i] = na; val[i] = (float*)malloc(na * 4);
            const pyc_shape* sa = &m->ops[ia].shape; size_t cols = sa->rank ? (size_t)sa->dims[sa->rank - 1] : 0;
            if (nb == na) oracle_add(val[ia], val[ib], val[i], na);
            else if (nb == 1) oracle_add_scalar(val[ia], val[ib][0], val[i], na);
            else if (cols && nb == cols) oracle_add_row_bias(val[ia], val[ib], val[i], na / cols, cols);
            else rc = -1;
            break; }
        case PYC_IR_OP_RELU: case PYC_IR_OP_GELU: {
            if (op->input_count < 1) { rc = -1; break; }
            size_t na = ne[op->input_ids[0]]; ne[i] = na; val[i] = (float*)malloc(na * 4);
            if (op->kind == PYC_IR_OP_RELU) oracle_relu(val[op->input_ids[0]], val[i], na); else oracle_gelu(val[op->input_ids[0]], val[i], na);
            break; }
        case PYC_IR_OP_LAYERNORM: {
            if (op->input_count < 1) { rc = -1; break; }
            int ix = op->input_ids[0]; const pyc_shape* sx = &m->ops[ix].shape; size_t na = ne[ix];
            size_t cols = sx->rank ? (size_t)sx->dims[sx->rank - 1] : 0; if (!cols) { rc = -1; break; }
            const float* g = op->input_count > 1 ? val[op->input_ids[1]] : NULL; const float* bt = op->input_count > 2 ? val[op->input_ids[2]] : NULL;
            ne[i] = na; val[i] = (float*)malloc(na * 4);
            oracle_layernorm(val[ix], g, bt, val[i], na / cols, cols, 1e-5f); break; }
        case PYC_IR_OP_REDUCE_SUM: {
            if (op->input_count < 1 || n == 0) { rc = -1; break; }
            size_t na = ne[op->input_ids[0]]; if (na % n) { rc = -1; break; }
            val[i] = (float*)malloc(n * 4); oracle_reduce_sum(val[op->input_ids[0]], val[i], n, na / n); break; }
        case PYC_IR_OP_OUTPUT: {
            int tag; if (op->input_count < 1 || out_i >= output_count || !outputs[out_i].data) { rc = -1; break; }
            int src = op->input_ids[0]; tag = dtype_tag(outputs[out_i].dtype);
            if (tag < 0 || outputs[out_i].size_bytes < ne[src] * (tag == ORACLE_F32 ? 4u : 2u)) { rc = -1; break; }
            /* INPUT -> OUTPUT keeps the stored bytes (test_cuda_backend.c:252-312). */
            oracle_narrow(tag, val[src], outputs[out_i].data, ne[src]);
            val[i] = (float*)malloc(4); ne[i] = ne[src]; out_i++; break; }
        default: rc = -1; break; /* CONST carries no data in the IR: compiler_api.c:2076 rejects it too */
        }
    }
    for (i = 0; i < m->op_count; ++i) free(val[i]);
    free(val); free(ne);
    return rc;
}
