/*
 * bw_oracle.c -- CPU restatement of the Bitween RTN quantize/pack, dequantize and
 * QuantizedLinear-forward arithmetic.  TEST INFRASTRUCTURE ONLY: this file is the
 * checker the CUDA kernels are compared against and the timed CPU baseline.  It is
 * never linked into, imported by, or called from the shipped library.
 *
 * Parity status: PINNED.  Every function here is checked (tests/test_oracle_golden.py)
 * against fixtures under tests/golden/ that were produced by running the reference's
 * own bitween/functional.py on CPU (tests/golden/gen_golden.py).
 *
 * Each function cites the reference lines it restates (paths are relative to the
 * reference project root).  Arithmetic notes:
 *   - torch evaluates every elementwise op of a float16/bfloat16 tensor in float32
 *     and rounds the result back to the tensor dtype, so `rnd(dtype, v)` is applied
 *     after each op; for float32 it is the identity.
 *   - torch.round is round-half-to-even (nearbyintf under the default FE_TONEAREST).
 *   - tensor.to(int32) of NaN yields INT32_MIN on x86 (cvttss2si "integer indefinite").
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp, no -ffast-math, -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define BWO_F32 0
#define BWO_F16 1
#define BWO_BF16 2
#define BWO_I32 3

/* ---------- scalar format helpers ------------------------------------------------ */

static inline float f16_bits_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f32_to_f16_bits(float f) {
    _Float16 v = (_Float16)f; /* IEEE round-to-nearest-even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}
static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb; /* round-to-nearest-even on the dropped 16 bits */
    return (uint16_t)(u >> 16);
}
static inline float rnd(int dtype, float v) {
    if (dtype == BWO_F16) return f16_bits_to_f32(f32_to_f16_bits(v));
    if (dtype == BWO_BF16) return bf16_bits_to_f32(f32_to_bf16_bits(v));
    return v;
}
static inline float load_as_f32(const void *p, int dtype, int64_t i) {
    if (dtype == BWO_F32) return ((const float *)p)[i];
    if (dtype == BWO_F16) return f16_bits_to_f32(((const uint16_t *)p)[i]);
    if (dtype == BWO_BF16) return bf16_bits_to_f32(((const uint16_t *)p)[i]);
    return (float)((const int32_t *)p)[i];
}
static inline void store_from_f32(void *p, int dtype, int64_t i, float v) {
    if (dtype == BWO_F32) ((float *)p)[i] = v;
    else if (dtype == BWO_F16) ((uint16_t *)p)[i] = f32_to_f16_bits(v);
    else ((uint16_t *)p)[i] = f32_to_bf16_bits(v);
}
/* torch amin/amax propagate NaN. */
static inline float min_nanprop(float a, float b) { return (a != a) ? a : ((b != b) ? b : (b < a ? b : a)); }
static inline float max_nanprop(float a, float b) { return (a != a) ? a : ((b != b) ? b : (b > a ? b : a)); }
/* torch.clamp(lo, hi): NaN stays NaN; otherwise min(max(v, lo), hi). */
static inline float clampf(float v, float lo, float hi) {
    if (v != v) return v;
    return v < lo ? lo : (v > hi ? hi : v);
}
static inline int32_t to_i32(float v) { return (v != v) ? INT32_MIN : (int32_t)v; }

/* ---------- quantize_rtn : bitween/functional.py:3-45 ---------------------------- */
/*
 * w        [N,K] row-major, dtype in {F32,F16,BF16}; arithmetic runs in that dtype
 * q_packed [N, K/vpi] int32, vpi = 32/bits; element e = j*vpi + i of the flat
 *          row-major code array sits in word j at bits [i*bits, (i+1)*bits)
 *          (functional.py:35-40)
 * scale    [N, K/g] in the weight dtype (functional.py:25, :45)
 * zp       [N, K/g] int32 (functional.py:26)
 * returns 0, or -1 for bad bits, -2 when K % g != 0 (functional.py:12-17),
 *          -3 when K % vpi != 0 (the view at functional.py:42-43 would fail).
 */
int bwo_quantize_rtn(const void *w, int dtype, int64_t N, int64_t K, int bits, int g,
                     int32_t *q_packed, void *scale, int32_t *zp) {
    if (bits != 2 && bits != 4 && bits != 8) return -1;
    if (g < 1 || K % g != 0) return -2;
    const int vpi = 32 / bits;
    if (K % vpi != 0) return -3;
    const int64_t G = K / g;
    const float Qmax = (float)((1 << bits) - 1);            /* functional.py:8-9 */
    const float floor_s = rnd(dtype, 1e-8f);                /* clamp(min=1e-8) in the tensor dtype */

#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        int32_t *qrow = q_packed + n * (K / vpi);
        memset(qrow, 0, sizeof(int32_t) * (size_t)(K / vpi));
        for (int64_t gi = 0; gi < G; ++gi) {
            const int64_t base = n * K + gi * g;
            float mn = load_as_f32(w, dtype, base), mx = mn;  /* functional.py:22-23 */
            for (int j = 1; j < g; ++j) {
                float v = load_as_f32(w, dtype, base + j);
                mn = min_nanprop(mn, v);
                mx = max_nanprop(mx, v);
            }
            /* functional.py:25  scale = ((w_max - w_min) / Qmax).clamp(min=1e-8) */
            float s = rnd(dtype, mx - mn);
            s = rnd(dtype, s / Qmax);
            if (s == s && s < floor_s) s = floor_s;
            /* functional.py:26  zero_point = round(-w_min / scale).clamp(Qmin, Qmax).int32 */
            float z = rnd(dtype, (-mn) / s);
            z = clampf(nearbyintf(z), 0.0f, Qmax);
            const int32_t zi = to_i32(z);
            store_from_f32(scale, dtype, n * G + gi, s);
            zp[n * G + gi] = zi;
            /* int32 zero_point is promoted to the weight dtype for the add (functional.py:29) */
            const float zf = rnd(dtype, (float)zi);
            for (int j = 0; j < g; ++j) {
                float v = load_as_f32(w, dtype, base + j);
                float t = rnd(dtype, v / s);
                t = rnd(dtype, t + zf);
                t = clampf(nearbyintf(t), 0.0f, Qmax);
                const uint32_t code = (uint32_t)to_i32(t);
                const int64_t k = gi * g + j;
                /* functional.py:38-40  q_packed |= q_flat[i::vpi] << (i*bits)  (int32 shift wraps) */
                qrow[k / vpi] = (int32_t)((uint32_t)qrow[k / vpi] | (code << ((k % vpi) * bits)));
            }
        }
    }
    return 0;
}

/* ---------- dequantize_rtn : bitween/functional.py:47-71 ------------------------- */
/*
 * out[n,k] = float(scale[n,k/g]) * ( float(q[n,k]) - float(zp[n,k/g]) ), fp32
 * (functional.py:70).  Codes are extracted with an arithmetic shift then a mask
 * (functional.py:58-62), so negative words are handled.
 */
int bwo_dequantize_rtn(const int32_t *q_packed, const void *scale, int scale_dtype,
                       const void *zp, int zp_dtype, int64_t N, int64_t K, int bits, int g,
                       float *out) {
    if (bits != 2 && bits != 4 && bits != 8) return -1;
    if (g < 1 || K % g != 0) return -2;
    const int vpi = 32 / bits;
    if (K % vpi != 0) return -3;
    const int64_t G = K / g;
    const int32_t mask = (1 << bits) - 1;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) {
            const int32_t word = q_packed[n * (K / vpi) + k / vpi];
            const int32_t code = (word >> ((k % vpi) * bits)) & mask;
            const float s = load_as_f32(scale, scale_dtype, n * G + k / g);
            const float z = load_as_f32(zp, zp_dtype, n * G + k / g);
            out[n * K + k] = s * ((float)code - z);
        }
    }
    return 0;
}

/* ---------- dequantize_weights_kernel : bitween/modules.py:10-58 ----------------- */
/*
 * The module's device kernel: fp16 scale and fp16 zero_point buffers,
 * weights = scales * (q.to(fp32) - zps) in fp32 (modules.py:55), stored as fp16
 * (modules.py:58).  `out_dtype` F16 reproduces it; BF16 / F32 are this build's
 * documented extensions (same fp32 expression, different final rounding).
 */
int bwo_dequantize_module(const int32_t *q_packed, const uint16_t *scale_h, const uint16_t *zp_h,
                          int64_t N, int64_t K, int bits, int g, void *out, int out_dtype) {
    if (bits != 2 && bits != 4 && bits != 8) return -1;
    if (g < 1 || K % g != 0) return -2;
    const int vpi = 32 / bits;
    if (K % vpi != 0) return -3;
    const int64_t G = K / g;
    const int32_t mask = (1 << bits) - 1;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) {
            const int32_t word = q_packed[n * (K / vpi) + k / vpi];
            const int32_t code = (word >> ((k % vpi) * bits)) & mask;
            const float s = f16_bits_to_f32(scale_h[n * G + k / g]);
            const float z = f16_bits_to_f32(zp_h[n * G + k / g]);
            store_from_f32(out, out_dtype, n * K + k, s * ((float)code - z));
        }
    }
    return 0;
}

/* ---------- QuantizedLinearFunction.forward : bitween/modules.py:61-106 ---------- */
/*
 * x        [M,K] activations already cast to `act_dtype` (modules.py:74 casts to fp16;
 *          BF16 is this build's extension)
 * W        = act_dtype( scale_h * (q - zp_h) )            (modules.py:55,58)
 * c        = act_dtype( sum_k x[m,k] * W[n,k] )           (modules.py:97; the GEMM library
 *          accumulates in fp32 in an unspecified order -- the sum here is taken in
 *          double, which is what tolerance-based parity compares against)
 * out      = act_dtype( c + bias )                         (modules.py:100-101)
 * out_acc  (optional, may be NULL) receives the fp32-rounded double sum before any
 *          16-bit rounding and before bias, for the "fp32 accumulate" checks.
 */
int bwo_qlinear_forward(const uint16_t *x, int act_dtype, int64_t M, int64_t N, int64_t K,
                        const int32_t *q_packed, const uint16_t *scale_h, const uint16_t *zp_h,
                        const uint16_t *bias, int bits, int g, uint16_t *out, float *out_acc) {
    if (bits != 2 && bits != 4 && bits != 8) return -1;
    if (g < 1 || K % g != 0) return -2;
    const int vpi = 32 / bits;
    if (K % vpi != 0) return -3;
    if (act_dtype != BWO_F16 && act_dtype != BWO_BF16) return -4;
    const int64_t G = K / g;
    const int32_t mask = (1 << bits) - 1;
    int err = 0;
#pragma omp parallel
    {
        float *wrow = (float *)malloc(sizeof(float) * (size_t)K);
        if (!wrow) {
#pragma omp atomic write
            err = -5;
        }
#pragma omp barrier
        if (!err) {
#pragma omp for schedule(static)
            for (int64_t n = 0; n < N; ++n) {
                for (int64_t k = 0; k < K; ++k) {
                    const int32_t word = q_packed[n * (K / vpi) + k / vpi];
                    const int32_t code = (word >> ((k % vpi) * bits)) & mask;
                    const float s = f16_bits_to_f32(scale_h[n * G + k / g]);
                    const float z = f16_bits_to_f32(zp_h[n * G + k / g]);
                    wrow[k] = rnd(act_dtype, s * ((float)code - z));
                }
                for (int64_t m = 0; m < M; ++m) {
                    const uint16_t *xr = x + m * K;
                    double acc = 0.0;
                    if (act_dtype == BWO_F16)
                        for (int64_t k = 0; k < K; ++k) acc += (double)f16_bits_to_f32(xr[k]) * (double)wrow[k];
                    else
                        for (int64_t k = 0; k < K; ++k) acc += (double)bf16_bits_to_f32(xr[k]) * (double)wrow[k];
                    const float accf = (float)acc;
                    if (out_acc) out_acc[m * N + n] = accf;
                    if (out) {
                        float c = rnd(act_dtype, accf);
                        if (bias) c = rnd(act_dtype, c + load_as_f32(bias, act_dtype, n));
                        store_from_f32(out, act_dtype, m * N + n, c);
                    }
                }
            }
        }
        free(wrow);
    }
    return err;
}

/* ---------- grad_input of QuantizedLinearFunction.backward : modules.py:108-141 -- */
/*
 * W = scale * (q.float() - zero_point.float()) in fp32 (modules.py:131-135), cast to the
 * grad dtype (modules.py:139), grad_input[m,k] = sum_n grad_out[m,n] * W[n,k].
 * Summed in double; result rounded to grad dtype (F16/BF16/F32).
 */
int bwo_qlinear_grad_input(const void *grad_out, int grad_dtype, int64_t M, int64_t N, int64_t K,
                           const int32_t *q_packed, const uint16_t *scale_h, const uint16_t *zp_h,
                           int bits, int g, void *grad_in) {
    if (bits != 2 && bits != 4 && bits != 8) return -1;
    if (g < 1 || K % g != 0) return -2;
    const int vpi = 32 / bits;
    if (K % vpi != 0) return -3;
    const int64_t G = K / g;
    const int32_t mask = (1 << bits) - 1;
    double *acc = (double *)calloc((size_t)(M * K), sizeof(double));
    if (!acc) return -5;
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) {
            const int32_t word = q_packed[n * (K / vpi) + k / vpi];
            const int32_t code = (word >> ((k % vpi) * bits)) & mask;
            const float s = f16_bits_to_f32(scale_h[n * G + k / g]);
            const float z = f16_bits_to_f32(zp_h[n * G + k / g]);
            const double wv = (double)rnd(grad_dtype, s * ((float)code - z));
            for (int64_t m = 0; m < M; ++m)
                acc[m * K + k] += (double)load_as_f32(grad_out, grad_dtype, m * N + n) * wv;
        }
    }
    for (int64_t i = 0; i < M * K; ++i) store_from_f32(grad_in, grad_dtype, i, (float)acc[i]);
    free(acc);
    return 0;
}

/* Sets the number of OpenMP threads of the later calls (launchers such as torchrun export
 * OMP_NUM_THREADS=1 to their workers; the timed CPU baseline wants all host threads). */
int bwo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
    return 0;
}

int bwo_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp master
        n = omp_get_num_threads();
    }
#endif
    return n;
}
