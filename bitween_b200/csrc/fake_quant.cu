// Fake-quantized weights with learnable parameters for sm_100a.
//
// Replaces the elementwise tensor program of the reference's
// WrapperLinear._quantize_weight_with_learnable_params (bitween/wrapper.py:116-172), evaluated on
// every training step of the trainable / gradual modes: given the per-group scale and (float,
// unrounded) zero point that the learnable min/max factors produce, and the learnable rounding
// perturbation `value`,
//     t   = w / scale + zero_point (+ value)          bitween/wrapper.py:143-149
//     w_q = clamp(round(t), 0, 2^bits - 1)             :152   (round half to even)
//     w_dq = scale * (w_q - zero_point)                :155
// -- about ten full passes over [N,K] in eager mode, one here: every weight (and perturbation)
// is read once, w_dq (and, if asked for, w_q) written once.  All arithmetic is fp32 with the
// reference's operation order and one rounding per operation (the division is the correctly
// rounded quotient), so the outputs are bit-identical to the reference run in fp32; 16-bit
// weights are up-cast exactly, which is what torch's type promotion does once any fp32 parameter
// takes part (the perturbation may be fp32 or 16-bit for the same reason).  HBM-bound:
// sizeof(w) + sizeof(value) in, 4 (+4) out per weight.
#include "bw_common.cuh"

namespace bw {
namespace {

// torch.clamp keeps NaN; fminf/fmaxf would drop it.
__device__ __forceinline__ float clamp_keepnan(float v, float hi) { return (v != v) ? v : fminf(fmaxf(v, 0.0f), hi); }

template <typename T> __device__ __forceinline__ void load4(const T *p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float *p, float (&v)[4]) {
    const float4 a = __ldcs(reinterpret_cast<const float4 *>(p));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void load4<__half>(const __half *p, float (&v)[4]) {
    const uint2 a = __ldcs(reinterpret_cast<const uint2 *>(p));
    const __half2 *h = reinterpret_cast<const __half2 *>(&a);
    const float2 lo = __half22float2(h[0]), hi = __half22float2(h[1]);
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16 *p, float (&v)[4]) {
    const uint2 a = __ldcs(reinterpret_cast<const uint2 *>(p));
    v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xffff0000u);
    v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xffff0000u);
}

// Eight consecutive elements: one 16-byte load for 16-bit types, two for fp32.
template <typename T> __device__ __forceinline__ void load8(const T *p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float *p, float (&v)[8]) {
    const float4 a = __ldcs(reinterpret_cast<const float4 *>(p)), b = __ldcs(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__half>(const __half *p, float (&v)[8]) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(p));
    const __half2 *h = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        v[2 * j] = f.x; v[2 * j + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(p));
    const uint32_t r[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(r[j] << 16); v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
    }
}
template <int V, typename T> __device__ __forceinline__ void loadv(const T *p, float (&v)[V]) {
    if constexpr (V == 8) load8<T>(p, v); else load4<T>(p, v);
}

template <int V, typename T, typename VT>
__global__ void __launch_bounds__(256)
fake_quant_kernel(const T *__restrict__ w, int64_t quads, int g, float qmax, const float *__restrict__ scale,
                  const float *__restrict__ zp, const VT *__restrict__ value, float *__restrict__ dq,
                  float *__restrict__ wq) {
    // one thread = V consecutive elements of one group (group_size % V == 0)
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e0 = i * V, grp = e0 / g;
        const float s = __ldg(scale + grp), z = __ldg(zp + grp);
        float v[V], pv[V], q[V], d[V];
        loadv<V, T>(w + e0, v);
        if (value) loadv<V, VT>(value + e0, pv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            float t = __fadd_rn(__fdiv_rn(v[j], s), z);
            if (value) t = __fadd_rn(t, pv[j]);
            q[j] = clamp_keepnan(rintf(t), qmax);
            d[j] = __fmul_rn(s, __fsub_rn(q[j], z));
        }
#pragma unroll
        for (int j = 0; j < V; j += 4) {
            __stcs(reinterpret_cast<float4 *>(dq + e0 + j), make_float4(d[j], d[j + 1], d[j + 2], d[j + 3]));
            if (wq) __stcs(reinterpret_cast<float4 *>(wq + e0 + j), make_float4(q[j], q[j + 1], q[j + 2], q[j + 3]));
        }
    }
}

template <typename T, typename VT>
__global__ void __launch_bounds__(256)
fake_quant_scalar_kernel(const T *__restrict__ w, int64_t total, int g, float qmax, const float *__restrict__ scale,
                         const float *__restrict__ zp, const VT *__restrict__ value, float *__restrict__ dq,
                         float *__restrict__ wq) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const float s = scale[e / g], z = zp[e / g];
        float t = __fadd_rn(__fdiv_rn(to_f32<T>(w[e]), s), z);
        if (value) t = __fadd_rn(t, to_f32<VT>(value[e]));
        const float q = clamp_keepnan(rintf(t), qmax);
        dq[e] = __fmul_rn(s, __fsub_rn(q, z));
        if (wq) wq[e] = q;
    }
}

template <typename T, typename VT>
int launch(const void *w, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp, const void *value,
           float *dq, float *wq, cudaStream_t st) {
    const int64_t total = N * K;
    const float qmax = (float)((1 << bits) - 1);
    const bool out_ok = aligned_to(dq, 16) && aligned_to(wq, 16);
    const bool vec8 = out_ok && g % 8 == 0 && aligned_to(w, 8 * sizeof(T)) && aligned_to(value, 8 * sizeof(VT));
    const bool vec = out_ok && g % 4 == 0 && aligned_to(w, 4 * sizeof(T)) && aligned_to(value, 4 * sizeof(VT));
    const int64_t work = vec8 ? total / 8 : vec ? total / 4 : total;
    int64_t blocks = (work + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (vec8)
        fake_quant_kernel<8, T, VT><<<(unsigned)blocks, 256, 0, st>>>((const T *)w, work, g, qmax, scale, zp, (const VT *)value, dq, wq);
    else if (vec)
        fake_quant_kernel<4, T, VT><<<(unsigned)blocks, 256, 0, st>>>((const T *)w, work, g, qmax, scale, zp, (const VT *)value, dq, wq);
    else
        fake_quant_scalar_kernel<T, VT><<<(unsigned)blocks, 256, 0, st>>>((const T *)w, work, g, qmax, scale, zp, (const VT *)value, dq, wq);
    return check_launch("fake_quant_kernel");
}

// The same pass when EVERYTHING is 16-bit (16-bit weights, min/max tuning off, so no fp32 tensor
// promotes the arithmetic): the reference's torch ops then round every intermediate to the
// weight's dtype -- w/scale, + zero_point, + value, the difference and the product -- which is
// reproduced here by rounding after each fp32 operation (the fp32 result of one operation on two
// 16-bit values, rounded to 16 bits, is the correctly rounded 16-bit result).  scale, zero_point,
// value and both outputs have the weight's dtype.
template <typename T> __device__ __forceinline__ float rnd16(float v) { return to_f32<T>(from_f32<T>(v)); }
template <typename T>
__global__ void __launch_bounds__(256)
fake_quant_native_kernel(const T *__restrict__ w, int64_t total, int g, float qmax, const T *__restrict__ scale,
                         const T *__restrict__ zp, const T *__restrict__ value, T *__restrict__ dq, T *__restrict__ wq) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const float s = to_f32<T>(scale[e / g]), z = to_f32<T>(zp[e / g]);
        float t = rnd16<T>(__fadd_rn(rnd16<T>(__fdiv_rn(to_f32<T>(w[e]), s)), z));
        if (value) t = rnd16<T>(__fadd_rn(t, to_f32<T>(value[e])));
        const float q = clamp_keepnan(rintf(t), qmax);
        dq[e] = from_f32<T>(__fmul_rn(s, rnd16<T>(__fsub_rn(q, z))));
        if (wq) wq[e] = from_f32<T>(q);
    }
}

// Backward of the pass above for the per-group parameters.  round() has zero gradient in the
// reference's autograd graph, so w_dq = scale * (w_q - zero_point) gives
//     d/d scale      = sum_group grad * (w_q - zero_point)
//     d/d zero_point = -scale * sum_group grad
// and nothing for `value`.  w_q is recomputed from the weights instead of being kept from the
// forward: sizeof(w) + sizeof(value) + 4 bytes read per weight, nothing written but [N,G] sums.
// One thread = V elements; the g/V lanes of a group (a power of two <= 32) reduce by shuffles.
template <int V, typename T, typename VT>
__global__ void __launch_bounds__(256)
fake_quant_backward_kernel(const T *__restrict__ w, int64_t quads, int g, float qmax, const float *__restrict__ scale,
                           const float *__restrict__ zp, const VT *__restrict__ value, const float *__restrict__ grad,
                           float *__restrict__ gscale, float *__restrict__ gzp) {
    const int lanes = g / V;
    const int64_t quads_padded = (quads + 31) & ~(int64_t)31;      // whole warps stay in the loop together
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads_padded; i += (int64_t)gridDim.x * blockDim.x) {
        const bool live = i < quads;
        const int64_t e0 = i * V, grp = e0 / g;
        float a = 0.0f, b = 0.0f, s = 1.0f, z = 0.0f;
        if (live) {
            s = __ldg(scale + grp); z = __ldg(zp + grp);
            float v[V], pv[V], gr[V];
            loadv<V, T>(w + e0, v);
            loadv<V, float>(grad + e0, gr);
            if (value) loadv<V, VT>(value + e0, pv);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float t = __fadd_rn(__fdiv_rn(v[j], s), z);
                if (value) t = __fadd_rn(t, pv[j]);
                const float q = clamp_keepnan(rintf(t), qmax);
                a = fmaf(gr[j], __fsub_rn(q, z), a);
                b += gr[j];
            }
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            b += __shfl_xor_sync(0xffffffffu, b, o);
        }
        if (live && (threadIdx.x & (lanes - 1)) == 0) {
            gscale[grp] = a;
            gzp[grp] = -s * b;
        }
    }
}

template <typename T, typename VT>
int launch_bwd(const void *w, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp, const void *value,
               const float *grad, float *gscale, float *gzp, cudaStream_t st) {
    const bool vec8 = g % 8 == 0 && g / 8 <= 32 && aligned_to(w, 8 * sizeof(T)) && aligned_to(value, 8 * sizeof(VT)) && aligned_to(grad, 32);
    if (!vec8 && !(g % 4 == 0 && g / 4 <= 32 && ((g / 4) & (g / 4 - 1)) == 0)) return BW_ERR_ALIGN;
    const int64_t quads = N * K / (vec8 ? 8 : 4);
    int64_t blocks = (quads + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    const float qmax = (float)((1 << bits) - 1);
    if (vec8)
        fake_quant_backward_kernel<8, T, VT><<<(unsigned)blocks, 256, 0, st>>>((const T *)w, quads, g, qmax, scale, zp,
                                                                               (const VT *)value, grad, gscale, gzp);
    else
        fake_quant_backward_kernel<4, T, VT><<<(unsigned)blocks, 256, 0, st>>>((const T *)w, quads, g, qmax, scale, zp,
                                                                               (const VT *)value, grad, gscale, gzp);
    return check_launch("fake_quant_backward_kernel");
}

template <typename T>
int launch_bwd_v(const void *w, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp, const void *value,
                 int value_dtype, const float *grad, float *gscale, float *gzp, cudaStream_t st) {
    if (!value || value_dtype == BW_F32) return launch_bwd<T, float>(w, N, K, bits, g, scale, zp, value, grad, gscale, gzp, st);
    if (value_dtype == BW_F16) return launch_bwd<T, __half>(w, N, K, bits, g, scale, zp, value, grad, gscale, gzp, st);
    if (value_dtype == BW_BF16) return launch_bwd<T, __nv_bfloat16>(w, N, K, bits, g, scale, zp, value, grad, gscale, gzp, st);
    return BW_ERR_DTYPE;
}

template <typename T>
int launch_v(const void *w, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp, const void *value,
             int value_dtype, float *dq, float *wq, cudaStream_t st) {
    if (!value || value_dtype == BW_F32) return launch<T, float>(w, N, K, bits, g, scale, zp, value, dq, wq, st);
    if (value_dtype == BW_F16) return launch<T, __half>(w, N, K, bits, g, scale, zp, value, dq, wq, st);
    if (value_dtype == BW_BF16) return launch<T, __nv_bfloat16>(w, N, K, bits, g, scale, zp, value, dq, wq, st);
    return BW_ERR_DTYPE;
}

}  // namespace

int fake_quant_native(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, const void *scale, const void *zp,
                      const void *value, void *dq, void *wq, cudaStream_t st) {
    const int64_t total = N * K;
    if (total == 0) return BW_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    const float qmax = (float)((1 << bits) - 1);
    if (w_dtype == BW_F16)
        fake_quant_native_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half *)w, total, g, qmax, (const __half *)scale,
                                                                          (const __half *)zp, (const __half *)value, (__half *)dq, (__half *)wq);
    else if (w_dtype == BW_BF16)
        fake_quant_native_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16 *)w, total, g, qmax,
                                                                                 (const __nv_bfloat16 *)scale, (const __nv_bfloat16 *)zp,
                                                                                 (const __nv_bfloat16 *)value, (__nv_bfloat16 *)dq,
                                                                                 (__nv_bfloat16 *)wq);
    else
        return BW_ERR_DTYPE;
    return check_launch("fake_quant_native_kernel");
}

int fake_quant(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp,
               const void *value, int value_dtype, float *dq, float *wq, cudaStream_t st) {
    if (N * K == 0) return BW_OK;
    switch (w_dtype) {
        case BW_F32: return launch_v<float>(w, N, K, bits, g, scale, zp, value, value_dtype, dq, wq, st);
        case BW_F16: return launch_v<__half>(w, N, K, bits, g, scale, zp, value, value_dtype, dq, wq, st);
        case BW_BF16: return launch_v<__nv_bfloat16>(w, N, K, bits, g, scale, zp, value, value_dtype, dq, wq, st);
        default: return BW_ERR_DTYPE;
    }
}


// group_size must be 4 * 2^j (j <= 5) or 8 * 2^j (j <= 5), w / value / grad aligned to four elements.
int fake_quant_backward(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp,
                        const void *value, int value_dtype, const float *grad, float *gscale, float *gzp, cudaStream_t st) {
    if (N * K == 0) return BW_OK;
    const auto pow2_lanes = [](int lanes) { return lanes >= 1 && lanes <= 32 && (lanes & (lanes - 1)) == 0; };
    if (!((g % 4 == 0 && pow2_lanes(g / 4)) || (g % 8 == 0 && pow2_lanes(g / 8)))) return BW_ERR_GROUP;
    const size_t wa = 4 * (size_t)dtype_size(w_dtype), va = value ? 4 * (size_t)dtype_size(value_dtype) : 1;
    if (!aligned_to(w, wa) || !aligned_to(value, va) || !aligned_to(grad, 16)) return BW_ERR_ALIGN;
    switch (w_dtype) {
        case BW_F32: return launch_bwd_v<float>(w, N, K, bits, g, scale, zp, value, value_dtype, grad, gscale, gzp, st);
        case BW_F16: return launch_bwd_v<__half>(w, N, K, bits, g, scale, zp, value, value_dtype, grad, gscale, gzp, st);
        case BW_BF16: return launch_bwd_v<__nv_bfloat16>(w, N, K, bits, g, scale, zp, value, value_dtype, grad, gscale, gzp, st);
        default: return BW_ERR_DTYPE;
    }
}

}  // namespace bw
