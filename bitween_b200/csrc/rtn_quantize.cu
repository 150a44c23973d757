// RTN group-wise quantize + pack for sm_100a.
//
// Replaces the eager tensor program of the reference's quantize_rtn
// (bitween/functional.py:3-45): amin/amax per group, scale, zero-point, round/clamp and
// the 32/bits-iteration shift-OR packing loop -- about a dozen full passes over [N,K]
// plus an int32 temporary -- by ONE pass: each weight is read once, codes are packed in
// registers and only the packed words, scales and zero-points are written.
//
// Bit-exactness: every arithmetic step uses the correctly rounded IEEE intrinsic
// (__fsub_rn, __fdiv_rn, __fadd_rn, rintf) in the order torch evaluates the expression,
// with an extra rounding to the tensor dtype after each step when the weights are
// fp16/bf16 and "native" arithmetic is requested (torch computes 16-bit elementwise ops
// in fp32 and rounds the result back).  No fast-math, no reciprocal, no FMA contraction.
//
// Data layout: weights are read as 16-byte vectors, lane-contiguous, so a warp
// instruction covers 512 contiguous bytes; a quantization group occupies g/V
// consecutive lanes (V = elements per 16 bytes), its min/max are reduced with xor
// shuffles inside that lane segment, and a packed word is assembled with xor shuffles
// over the 32/bits/V lanes that hold its codes.  The kernel is HBM-bound:
// bytes per weight = sizeof(T) in, bits/8 out, plus (scale+zp)/g.
#include "bw_common.cuh"

namespace bw {
namespace {

__device__ __forceinline__ float min_nanprop(float a, float b) {
    return (a != a) ? a : ((b != b) ? b : fminf(a, b));
}
__device__ __forceinline__ float max_nanprop(float a, float b) {
    return (a != a) ? a : ((b != b) ? b : fmaxf(a, b));
}
// torch.clamp keeps NaN; fminf/fmaxf would drop it.
__device__ __forceinline__ float clamp_keepnan(float v, float hi) {
    return (v != v) ? v : fminf(fmaxf(v, 0.0f), hi);
}
// tensor.to(int32): NaN becomes INT32_MIN ("integer indefinite"), as the CPU reference does.
__device__ __forceinline__ int32_t to_i32_like_torch(float v) {
    return (v != v) ? INT32_MIN : (int32_t)v;
}

template <typename T, bool NATIVE> __device__ __forceinline__ float rnd(float v) {
    if constexpr (NATIVE) return to_f32<T>(from_f32<T>(v));
    else return v;
}

template <typename T> struct Elems16 { static constexpr int V = 16 / sizeof(T); };

template <typename T> __device__ __forceinline__ void load16(const T *p, float (&out)[Elems16<T>::V]);
template <> __device__ __forceinline__ void load16<float>(const float *p, float (&out)[4]) {
    const float4 v = __ldcs(reinterpret_cast<const float4 *>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> __device__ __forceinline__ void load16<__half>(const __half *p, float (&out)[8]) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(p));
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16 *p, float (&out)[8]) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(p));
    const uint32_t *u = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(u[i] << 16);
        out[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

template <typename ZT> __device__ __forceinline__ void store_zp(ZT *p, int32_t z);
template <> __device__ __forceinline__ void store_zp<int32_t>(int32_t *p, int32_t z) { *p = z; }
template <> __device__ __forceinline__ void store_zp<__half>(__half *p, int32_t z) { *p = __int2half_rn(z); }

// The per-group parameters of bitween/functional.py:25-26.
template <typename T, bool NATIVE>
__device__ __forceinline__ void group_params(float mn, float mx, float qmax, float floor_s, float &s,
                                             int32_t &zi, float &zf) {
    s = rnd<T, NATIVE>(__fsub_rn(mx, mn));
    s = rnd<T, NATIVE>(__fdiv_rn(s, qmax));
    if (s < floor_s) s = floor_s;                     // clamp(min=1e-8); NaN stays NaN
    float z = rnd<T, NATIVE>(__fdiv_rn(-mn, s));
    z = clamp_keepnan(rintf(z), qmax);                // torch.round is half-to-even
    zi = to_i32_like_torch(z);
    zf = rnd<T, NATIVE>((float)zi);                   // int32 -> weight dtype promotion for the add
}
// One code, bitween/functional.py:29.
template <typename T, bool NATIVE>
__device__ __forceinline__ uint32_t code_of(float v, float s, float zf, float qmax) {
    float t = rnd<T, NATIVE>(__fdiv_rn(v, s));
    t = rnd<T, NATIVE>(__fadd_rn(t, zf));
    t = clamp_keepnan(rintf(t), qmax);
    return (uint32_t)to_i32_like_torch(t);
}

// ---- fast path: g = V * 2^j, g/V <= 32 -------------------------------------------------
template <typename T, bool NATIVE, int BITS, int L, typename ST, typename ZT>
__global__ void __launch_bounds__(256)
rtn_quantize_pack_kernel(const T *__restrict__ w, int64_t total_chunks, int cpg_log2, float floor_s,
                         int32_t *__restrict__ qweight, ST *__restrict__ scale, ZT *__restrict__ zp) {
    constexpr int V = Elems16<T>::V;
    constexpr int VPI = 32 / BITS;
    constexpr float QMAX = (float)((1 << BITS) - 1);
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t c0 = warp * (32 * L) + lane;
    const int cpg = 1 << cpg_log2;

    float v[L][V];
#pragma unroll
    for (int l = 0; l < L; ++l) {
        const int64_t c = c0 + l * 32;
        if (c < total_chunks) load16<T>(w + c * V, v[l]);
        else {
#pragma unroll
            for (int j = 0; j < V; ++j) v[l][j] = 0.0f;
        }
    }
#pragma unroll
    for (int l = 0; l < L; ++l) {
        const int64_t c = c0 + l * 32;
        float mn = v[l][0], mx = v[l][0];
#pragma unroll
        for (int j = 1; j < V; ++j) { mn = min_nanprop(mn, v[l][j]); mx = max_nanprop(mx, v[l][j]); }
        for (int off = cpg >> 1; off > 0; off >>= 1) {
            mn = min_nanprop(mn, __shfl_xor_sync(0xffffffffu, mn, off));
            mx = max_nanprop(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        }
        float s, zf; int32_t zi;
        group_params<T, NATIVE>(mn, mx, QMAX, floor_s, s, zi, zf);
        if (c < total_chunks && (lane & (cpg - 1)) == 0) {
            const int64_t gidx = c >> cpg_log2;
            scale[gidx] = from_f32<ST>(s);
            store_zp<ZT>(zp + gidx, zi);
        }
        if constexpr (V >= VPI) {
            // this thread owns V/VPI whole words
            constexpr int WPC = V / VPI;
            uint32_t words[WPC];
#pragma unroll
            for (int wi = 0; wi < WPC; ++wi) {
                uint32_t acc = 0;
#pragma unroll
                for (int i = 0; i < VPI; ++i)
                    acc |= code_of<T, NATIVE>(v[l][wi * VPI + i], s, zf, QMAX) << (i * BITS);
                words[wi] = acc;
            }
            if (c < total_chunks) {
                if constexpr (WPC == 1) qweight[c] = (int32_t)words[0];
                else if constexpr (WPC == 2)
                    *reinterpret_cast<uint2 *>(qweight + c * 2) = make_uint2(words[0], words[1]);
                else {
#pragma unroll
                    for (int wi = 0; wi < WPC; ++wi) qweight[c * WPC + wi] = (int32_t)words[wi];
                }
            }
        } else {
            // VPI/V consecutive lanes hold the codes of one word
            constexpr int LPW = VPI / V;
            const int pos0 = (lane & (LPW - 1)) * V;
            uint32_t acc = 0;
#pragma unroll
            for (int j = 0; j < V; ++j)
                acc |= code_of<T, NATIVE>(v[l][j], s, zf, QMAX) << ((pos0 + j) * BITS);
#pragma unroll
            for (int off = 1; off < LPW; off <<= 1) acc |= __shfl_xor_sync(0xffffffffu, acc, off);
            if (c < total_chunks && (lane & (LPW - 1)) == 0) qweight[c / LPW] = (int32_t)acc;
        }
    }
}

// ---- general path: any group_size >= 1 with K % group_size == 0 and K % (32/bits) == 0 --
// One warp per span of lcm(group_size, 32/bits) elements: it first reduces each group of
// the span (parameters kept in shared memory), then its lanes assemble the span's words.
template <typename T, bool NATIVE, int BITS, typename ST, typename ZT>
__global__ void __launch_bounds__(128)
rtn_quantize_pack_general_kernel(const T *__restrict__ w, int64_t num_spans, int span, int g,
                                 float floor_s, int32_t *__restrict__ qweight,
                                 ST *__restrict__ scale, ZT *__restrict__ zp) {
    constexpr int VPI = 32 / BITS;
    constexpr float QMAX = (float)((1 << BITS) - 1);
    __shared__ float sh_s[4][VPI];
    __shared__ float sh_zf[4][VPI];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int64_t sp = (int64_t)blockIdx.x * 4 + wib;
    if (sp >= num_spans) return;          // whole warps leave together; no block-wide sync below
    const int64_t e0 = sp * span;
    const int gps = span / g;             // groups per span, <= VPI
    for (int gi = 0; gi < gps; ++gi) {
        const T *p = w + e0 + (int64_t)gi * g;
        float mn = to_f32<T>(p[0]), mx = mn;  // every lane seeds with element 0 of the group
        for (int j = lane; j < g; j += 32) {
            const float x = to_f32<T>(p[j]);
            mn = min_nanprop(mn, x);
            mx = max_nanprop(mx, x);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            mn = min_nanprop(mn, __shfl_xor_sync(0xffffffffu, mn, off));
            mx = max_nanprop(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        }
        float s, zf; int32_t zi;
        group_params<T, NATIVE>(mn, mx, QMAX, floor_s, s, zi, zf);
        if (lane == 0) {
            const int64_t gidx = e0 / g + gi;
            scale[gidx] = from_f32<ST>(s);
            store_zp<ZT>(zp + gidx, zi);
            sh_s[wib][gi] = s;
            sh_zf[wib][gi] = zf;
        }
    }
    __syncwarp();
    const int wps = span / VPI;           // words per span
    for (int wi = lane; wi < wps; wi += 32) {
        uint32_t acc = 0;
#pragma unroll
        for (int i = 0; i < VPI; ++i) {
            const int off = wi * VPI + i;
            const int gi = off / g;
            acc |= code_of<T, NATIVE>(to_f32<T>(w[e0 + off]), sh_s[wib][gi], sh_zf[wib][gi], QMAX)
                   << (i * BITS);
        }
        qweight[e0 / VPI + wi] = (int32_t)acc;
    }
}

int64_t gcd64(int64_t a, int64_t b) { while (b) { int64_t t = a % b; a = b; b = t; } return a; }

template <typename T, bool NATIVE, int BITS, typename ST, typename ZT>
int launch_typed(const T *w, int64_t N, int64_t K, int g, int32_t *q, ST *scale, ZT *zp, float floor_s,
                 cudaStream_t st) {
    constexpr int V = Elems16<T>::V;
    constexpr int VPI = 32 / BITS;
    constexpr int L = (sizeof(T) == 4) ? 4 : 2;
    const int64_t total = N * K;
    if (total == 0) return BW_OK;
    int cpg_log2 = -1;
    if (g % V == 0) {
        const int cpg = g / V;
        if (cpg <= 32 && (cpg & (cpg - 1)) == 0) { cpg_log2 = 0; while ((1 << cpg_log2) < cpg) ++cpg_log2; }
    }
    if (cpg_log2 >= 0 && aligned_to(w, 16) && aligned_to(q, 8)) {
        const int64_t chunks = total / V;
        const int64_t warps = (chunks + 32 * L - 1) / (32 * L);
        const int64_t blocks = (warps + 7) / 8;
        if (blocks > 0x7fffffff) return BW_ERR_SHAPE;
        rtn_quantize_pack_kernel<T, NATIVE, BITS, L, ST, ZT><<<(unsigned)blocks, 256, 0, st>>>(
            w, chunks, cpg_log2, floor_s, q, scale, zp);
        return check_launch("rtn_quantize_pack_kernel");
    }
    const int64_t span = (int64_t)g / gcd64(g, VPI) * VPI;
    if (span > 0x7fffffff) return BW_ERR_SHAPE;
    const int64_t spans = total / span;
    const int64_t blocks = (spans + 3) / 4;
    if (blocks > 0x7fffffff) return BW_ERR_SHAPE;
    rtn_quantize_pack_general_kernel<T, NATIVE, BITS, ST, ZT><<<(unsigned)blocks, 128, 0, st>>>(
        w, spans, (int)span, g, floor_s, q, scale, zp);
    return check_launch("rtn_quantize_pack_general_kernel");
}

template <typename T, bool NATIVE, typename ST, typename ZT>
int launch_bits(const T *w, int64_t N, int64_t K, int bits, int g, int32_t *q, ST *scale, ZT *zp,
                float floor_s, cudaStream_t st) {
    switch (bits) {
        case 2: return launch_typed<T, NATIVE, 2, ST, ZT>(w, N, K, g, q, scale, zp, floor_s, st);
        case 4: return launch_typed<T, NATIVE, 4, ST, ZT>(w, N, K, g, q, scale, zp, floor_s, st);
        default: return launch_typed<T, NATIVE, 8, ST, ZT>(w, N, K, g, q, scale, zp, floor_s, st);
    }
}

template <typename T, bool NATIVE, typename ST>
int launch_zp(const T *w, int64_t N, int64_t K, int bits, int g, int32_t *q, ST *scale, void *zp,
              int zp_dtype, float floor_s, cudaStream_t st) {
    if (zp_dtype == BW_I32)
        return launch_bits<T, NATIVE, ST, int32_t>(w, N, K, bits, g, q, scale, (int32_t *)zp, floor_s, st);
    return launch_bits<T, NATIVE, ST, __half>(w, N, K, bits, g, q, scale, (__half *)zp, floor_s, st);
}

template <typename T, bool NATIVE>
int launch_scale(const T *w, int64_t N, int64_t K, int bits, int g, int32_t *q, void *scale,
                 int scale_dtype, void *zp, int zp_dtype, float floor_s, cudaStream_t st) {
    switch (scale_dtype) {
        case BW_F32: return launch_zp<T, NATIVE, float>(w, N, K, bits, g, q, (float *)scale, zp, zp_dtype, floor_s, st);
        case BW_F16: return launch_zp<T, NATIVE, __half>(w, N, K, bits, g, q, (__half *)scale, zp, zp_dtype, floor_s, st);
        default: return launch_zp<T, NATIVE, __nv_bfloat16>(w, N, K, bits, g, q, (__nv_bfloat16 *)scale, zp, zp_dtype, floor_s, st);
    }
}

}  // namespace

int rtn_quantize_pack(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g,
                      int32_t *q, void *scale, int scale_dtype, void *zp, int zp_dtype,
                      unsigned flags, cudaStream_t st) {
    const bool native = !(flags & BW_RTN_UPCAST_F32);
    switch (w_dtype) {
        case BW_F32:
            return launch_scale<float, false>((const float *)w, N, K, bits, g, q, scale, scale_dtype, zp, zp_dtype, 1e-8f, st);
        case BW_F16:
            // clamp(min=1e-8) on a float16 tensor compares against float16(1e-8) == 0
            if (native) return launch_scale<__half, true>((const __half *)w, N, K, bits, g, q, scale, scale_dtype, zp, zp_dtype, 0.0f, st);
            return launch_scale<__half, false>((const __half *)w, N, K, bits, g, q, scale, scale_dtype, zp, zp_dtype, 1e-8f, st);
        case BW_BF16:
            if (native) return launch_scale<__nv_bfloat16, true>((const __nv_bfloat16 *)w, N, K, bits, g, q, scale, scale_dtype, zp, zp_dtype, __bfloat162float(__float2bfloat16_rn(1e-8f)), st);
            return launch_scale<__nv_bfloat16, false>((const __nv_bfloat16 *)w, N, K, bits, g, q, scale, scale_dtype, zp, zp_dtype, 1e-8f, st);
        default:
            return BW_ERR_DTYPE;
    }
}

}  // namespace bw
