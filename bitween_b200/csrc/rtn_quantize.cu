// RTN group-wise quantize + pack for sm_100a.
//
// Replaces the eager tensor program of the reference's quantize_rtn
// (bitween/functional.py:3-45): amin/amax per group, scale, zero-point, round/clamp and
// the 32/bits-iteration shift-OR packing loop -- about a dozen full passes over [N,K]
// plus an int32 temporary -- by ONE pass: each weight is read once, codes are packed in
// registers and only the packed words, scales and zero-points are written.
//
// Bit-exactness: every arithmetic step produces the correctly rounded IEEE result in the
// order torch evaluates the expression (__fsub_rn, __fdiv_rn, __fadd_rn, rintf, or a
// provably equivalent form -- see the fast path below), with an extra rounding to the
// tensor dtype after each step when the weights are fp16/bf16 and "native" arithmetic is
// requested (torch computes 16-bit elementwise ops in fp32 and rounds the result back).
// No fast-math, no approximate reciprocal, no FMA contraction.
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

// 16 bytes already in registers -> fp32 elements
template <typename T> __device__ __forceinline__ void unpack16(const uint4 &v, float (&out)[Elems16<T>::V]);
template <> __device__ __forceinline__ void unpack16<float>(const uint4 &v, float (&out)[4]) {
    out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y);
    out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4 &v, float (&out)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4 &v, float (&out)[8]) {
    const uint32_t *u = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(u[i] << 16);
        out[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

// min / max of the elements of one 16-byte chunk (NaNs dropped, as fminf / fmaxf do): on packed
// 16-bit pairs where the input is 16-bit -- min and max are exact in any format and cost one
// instruction per two elements there.
template <typename T> __device__ __forceinline__ void lane_minmax(const uint4 &raw, const float (&v)[Elems16<T>::V], float &mn, float &mx);
template <> __device__ __forceinline__ void lane_minmax<float>(const uint4 &, const float (&v)[4], float &mn, float &mx) {
    mn = fminf(fminf(v[0], v[1]), fminf(v[2], v[3]));
    mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
}
template <> __device__ __forceinline__ void lane_minmax<__half>(const uint4 &raw, const float (&)[8], float &mn, float &mx) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
    const __half2 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
    const __half2 hi = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    mn = fminf(__low2float(lo), __high2float(lo));
    mx = fmaxf(__low2float(hi), __high2float(hi));
}
template <> __device__ __forceinline__ void lane_minmax<__nv_bfloat16>(const uint4 &raw, const float (&)[8], float &mn, float &mx) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
    const __nv_bfloat162 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
    const __nv_bfloat162 hi = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    mn = fminf(__low2float(lo), __high2float(lo));
    mx = fmaxf(__low2float(hi), __high2float(hi));
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
//
// Per-element arithmetic on the common path (finite weights, scale within 2^-40..2^40):
//   * w/scale: the correctly rounded fp32 quotient torch computes, obtained from one
//     correctly rounded reciprocal per group and four FMAs per element (div_by_recip).
//   * round-half-even + clamp + int conversion: clamp(rint(t),0,Q) == rint(clamp(t,0,Q)), and
//     for 0 <= t <= 255 the sum t + 1.5*2^23 is rounded to an integer by the fp32 adder itself
//     (half-to-even), leaving the code in the low mantissa bits.
// Groups with a NaN/Inf weight or an out-of-range scale take the step-by-step path below,
// which mirrors torch's NaN/Inf propagation (bitween/functional.py:25-29 on such inputs).
// Correctly rounded fp32 quotient v/s from the correctly rounded reciprocal r = RN(1/s)
// (one __frcp_rn per group) with fused multiply-adds only:
//   q0 = RN(v*r)                      within 1.5 ulp of v/s
//   q1 = RN(q0 + RN(v - s*q0) * r)    a faithful rounding (error <= 1/2 ulp + 2^-22 ulp)
//   q2 = RN(q1 + (v - s*q1) * r)      the residual of a faithful quotient is exact, and
//                                     Markstein's theorem (correction of a faithful quotient
//                                     with the correctly rounded reciprocal) gives RN(v/s)
// Valid for normal operands without over/underflow: the caller guarantees |v| <= 2^40 and
// 2^-40 <= s <= 2^40.  For |v| < 2^-79 the residual may underflow, but then |v/s| < 2^-39 and
// the code does not depend on the quotient's low bits (adding the integer zero-point absorbs
// it).  tests/test_gpu_parity.py compares this against __fdiv_rn on 2^28 operand pairs.
__device__ __forceinline__ float div_by_recip(float v, float s, float r) {
    const float q0 = __fmul_rn(v, r);
    const float q1 = __fmaf_rn(__fmaf_rn(-s, q0, v), r, q0);
    return __fmaf_rn(__fmaf_rn(-s, q1, v), r, q1);
}

// The same division for two elements at a time with the packed fp32 instructions of sm_100
// (fma.rn.f32x2 / mul.rn.f32x2 / add.rn.f32x2: each lane of the pair is an IEEE operation with
// round-to-nearest-even, so the sequence above stays exact; one issue slot instead of two).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
        " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    float2 d;
    asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n"
        " mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    float2 d;
    asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n"
        " add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 div_by_recip2(float2 v, float s, float r) {
    const float2 s2 = make_float2(-s, -s), r2 = make_float2(r, r);
    const float2 q0 = fmul2(v, r2);
    const float2 q1 = ffma2(ffma2(s2, q0, v), r2, q0);
    return ffma2(ffma2(s2, q1, v), r2, q1);
}

// One 16-byte chunk per lane: group min/max over the lane segment, group parameters, codes,
// packed words and the group's scale / zero-point.  `c` is the global chunk index of this lane.
template <typename T, bool NATIVE, int BITS, typename ST, typename ZT>
__device__ __forceinline__ void rtn_slot(const uint4 &raw, int64_t c, bool in_range, int lane, int cpg,
                                         int cpg_log2, uint32_t seg_mask, float floor_s,
                                         int32_t *__restrict__ qweight, ST *__restrict__ scale,
                                         ZT *__restrict__ zp) {
    constexpr int V = Elems16<T>::V;
    constexpr int VPI = 32 / BITS;
    constexpr float QMAX = (float)((1 << BITS) - 1);
    constexpr float MAGIC = 12582912.0f;                 // 1.5 * 2^23
    constexpr uint32_t MAGIC_BITS = 0x4B400000u;
    float v[V];
    unpack16<T>(raw, v);
    float mn, mx;
    lane_minmax<T>(raw, v, mn, mx);
    // NaN/Inf detector on the FMA pipe: a sum is NaN or Inf as soon as one addend is; a sum of
    // finite values that overflows only sends the group down the slow, still exact, path.
    // fminf/fmaxf drop NaNs, so they cannot serve as the detector.
    float2 sum2 = make_float2(v[0], v[1]);
#pragma unroll
    for (int j = 2; j < V; j += 2) sum2 = fadd2(sum2, make_float2(v[j], v[j + 1]));
    const float sum = __fadd_rn(sum2.x, sum2.y);
    for (int off = cpg >> 1; off > 0; off >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    // bad: a NaN/Inf in this lane's elements, or a weight beyond +-2^40 in the group
    const bool bad = !(fabsf(sum) <= 3.0e38f) || !(mn >= -1.0995116e12f) || !(mx <= 1.0995116e12f);
    const bool group_bad = (__ballot_sync(0xffffffffu, bad) & seg_mask) != 0u;
    // (all lanes of the warp are together here; the vote is used by the fast path below)
    const bool lower_clamp = !NATIVE && __any_sync(0xffffffffu, !(mn <= 0.0f && mx >= 0.0f));
    float s, zf; int32_t zi;
    uint32_t words[V >= VPI ? V / VPI : 1];
    bool fast = !group_bad;
    float r = 0.0f;
    if (fast) {
        // group parameters with the same reciprocal+FMA division (the divisor Qmax is a constant)
        constexpr float RQ = 1.0f / QMAX;                     // correctly rounded at compile time
        s = rnd<T, NATIVE>(__fsub_rn(mx, mn));
        s = rnd<T, NATIVE>(div_by_recip(s, QMAX, RQ));        // a range below 2^-79 ends at the floor anyway
        if (s < floor_s) s = floor_s;
        fast = (s >= 9.094947e-13f) && (s <= 1.0995116e12f);  // 2^-40 <= scale <= 2^40
        r = __frcp_rn(s);
        float z = rnd<T, NATIVE>(div_by_recip(-mn, s, r));    // |min| < 2^-79 gives |z| < 2^-39 -> 0 either way
        z = fminf(fmaxf(rintf(z), 0.0f), QMAX);
        zi = (int32_t)z;
        zf = rnd<T, NATIVE>((float)zi);
    }
    if (fast) {
        const int pos0 = (V >= VPI) ? 0 : (lane & (VPI / V - 1)) * V;
        // When a group's range contains zero, zero_point = round(-min/scale) is not clamped and
        // w/scale + zero_point >= -1/2 for every element (RN(min/scale) = -RN(-min/scale) and the
        // division is monotonic), which the magic-number rounding below turns into code 0: the
        // lower clamp does nothing.  Weights almost always look like that, so the whole warp
        // votes (above, where all lanes are still together) and skips it (one instruction per element).
#pragma unroll
        for (int wi = 0; wi < (V >= VPI ? V / VPI : 1); ++wi) {
            // word = sum_i code_i * 2^(pos_i*bits); the codes arrive as MAGIC_BITS + code_i, so
            // one integer multiply-add per element accumulates them and the constant
            // MAGIC_BITS * sum_i 2^(pos_i*bits) is removed once at the end (mod 2^32).
            uint32_t acc = 0, bias = 0;
            if constexpr (!NATIVE) {
                // fp32 arithmetic: two elements per packed instruction
#pragma unroll
                for (int i = 0; i < (V >= VPI ? VPI : V); i += 2) {
                    float2 t = div_by_recip2(make_float2(v[wi * VPI + i], v[wi * VPI + i + 1]), s, r);
                    t = fadd2(t, make_float2(zf, zf));
                    if (lower_clamp) { t.x = fmaxf(t.x, 0.0f); t.y = fmaxf(t.y, 0.0f); }
                    t.x = fminf(t.x, QMAX);
                    t.y = fminf(t.y, QMAX);
                    t = fadd2(t, make_float2(MAGIC, MAGIC));
                    const uint32_t mul0 = 1u << ((pos0 + i) * BITS), mul1 = 1u << ((pos0 + i + 1) * BITS);
                    acc += __float_as_uint(t.x) * mul0;
                    acc += __float_as_uint(t.y) * mul1;
                    bias += MAGIC_BITS * mul0 + MAGIC_BITS * mul1;
                }
            } else {
#pragma unroll
                for (int i = 0; i < (V >= VPI ? VPI : V); ++i) {
                    const float x = v[wi * VPI + i];
                    float t = rnd<T, NATIVE>(div_by_recip(x, s, r));
                    t = rnd<T, NATIVE>(__fadd_rn(t, zf));
                    t = fminf(fmaxf(t, 0.0f), QMAX);
                    const uint32_t mul = 1u << ((pos0 + i) * BITS);
                    acc += __float_as_uint(__fadd_rn(t, MAGIC)) * mul;
                    bias += MAGIC_BITS * mul;
                }
            }
            words[wi] = acc - bias;
        }
    } else {
        // step-by-step path with torch's NaN propagation (amin/amax keep NaN)
        float mn2 = v[0], mx2 = v[0];
#pragma unroll
        for (int j = 1; j < V; ++j) { mn2 = min_nanprop(mn2, v[j]); mx2 = max_nanprop(mx2, v[j]); }
        for (int off = cpg >> 1; off > 0; off >>= 1) {
            // only lanes of this group's segment hold meaningful values; the shuffle is
            // executed by the lanes that took this branch
            mn2 = min_nanprop(mn2, __shfl_xor_sync(__activemask(), mn2, off));
            mx2 = max_nanprop(mx2, __shfl_xor_sync(__activemask(), mx2, off));
        }
        group_params<T, NATIVE>(mn2, mx2, QMAX, floor_s, s, zi, zf);
        const int pos0 = (V >= VPI) ? 0 : (lane & (VPI / V - 1)) * V;
#pragma unroll
        for (int wi = 0; wi < (V >= VPI ? V / VPI : 1); ++wi) {
            uint32_t acc = 0;
#pragma unroll
            for (int i = 0; i < (V >= VPI ? VPI : V); ++i)
                acc |= code_of<T, NATIVE>(v[wi * VPI + i], s, zf, QMAX) << ((pos0 + i) * BITS);
            words[wi] = acc;
        }
    }
    if (in_range && (lane & (cpg - 1)) == 0) {
        const int64_t gidx = c >> cpg_log2;
        scale[gidx] = from_f32<ST>(s);
        store_zp<ZT>(zp + gidx, zi);
    }
    if constexpr (V >= VPI) {
        constexpr int WPC = V / VPI;     // this thread owns V/VPI whole words
        if (in_range) {
            if constexpr (WPC == 1) qweight[c] = (int32_t)words[0];
            else if constexpr (WPC == 2)
                *reinterpret_cast<uint2 *>(qweight + c * 2) = make_uint2(words[0], words[1]);
            else {
#pragma unroll
                for (int wi = 0; wi < WPC; ++wi) qweight[c * WPC + wi] = (int32_t)words[wi];
            }
        }
    } else {
        constexpr int LPW = VPI / V;     // VPI/V consecutive lanes hold the codes of one word
        uint32_t acc = words[0];
#pragma unroll
        for (int off = 1; off < LPW; off <<= 1) acc |= __shfl_xor_sync(0xffffffffu, acc, off);
        if (in_range && (lane & (LPW - 1)) == 0) qweight[c / LPW] = (int32_t)acc;
    }
}

template <typename T, bool NATIVE, int BITS, int L, typename ST, typename ZT>
__global__ void __launch_bounds__(256)
rtn_quantize_pack_kernel(const T *__restrict__ w, int64_t total_chunks, int cpg_log2, float floor_s,
                         int32_t *__restrict__ qweight, ST *__restrict__ scale, ZT *__restrict__ zp) {
    constexpr int V = Elems16<T>::V;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t c0 = warp * (32 * L) + lane;
    const int cpg = 1 << cpg_log2;
    const uint32_t seg_mask = (cpg == 32) ? 0xffffffffu : (((1u << cpg) - 1u) << (lane & ~(cpg - 1)));
    uint4 raw[L];
#pragma unroll
    for (int l = 0; l < L; ++l) {
        const int64_t c = c0 + l * 32;
        raw[l] = (c < total_chunks) ? __ldcs(reinterpret_cast<const uint4 *>(w + c * V)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int l = 0; l < L; ++l) {
        const int64_t c = c0 + l * 32;
        rtn_slot<T, NATIVE, BITS, ST, ZT>(raw[l], c, c < total_chunks, lane, cpg, cpg_log2, seg_mask, floor_s,
                                          qweight, scale, zp);
    }
}

// ---- several weight matrices in one launch ---------------------------------------------------
// The per-layer loops of the callers (bitween/quantizer/quantizer.py:72-80,
// bitween/gradual/base_wrapper.py:300-311) quantize one layer after the other; for the six or
// seven linears of a decoder block the launches, not the kernel, are the cost.  Here a table in
// device memory lists the matrices (all of one dtype, bit width and group size); every block
// looks up the matrix its index falls into and then runs the single-matrix code on it.
struct RtnBatchEntry {
    const void *w;
    int32_t *q;
    void *scale;
    void *zp;
    long long chunks;        // 16-byte chunks of the matrix
    long long first_block;   // first block index of the matrix in the batched grid
};

template <typename T, bool NATIVE, int BITS, int L, typename ST, typename ZT>
__global__ void __launch_bounds__(256)
rtn_quantize_pack_batch_kernel(const RtnBatchEntry *__restrict__ table, int njobs, int cpg_log2, float floor_s) {
    constexpr int V = Elems16<T>::V;
    __shared__ int job_s;
    if (threadIdx.x == 0) {
        int lo = 0, hi = njobs - 1;                      // last entry with first_block <= blockIdx.x
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (table[mid].first_block <= (long long)blockIdx.x) lo = mid; else hi = mid - 1;
        }
        job_s = lo;
    }
    __syncthreads();
    const RtnBatchEntry e = table[job_s];
    const T *w = reinterpret_cast<const T *>(e.w);
    const int lane = threadIdx.x & 31;
    const int64_t warp = (((int64_t)blockIdx.x - e.first_block) * blockDim.x + threadIdx.x) >> 5;
    const int64_t c0 = warp * (32 * L) + lane;
    const int cpg = 1 << cpg_log2;
    const uint32_t seg_mask = (cpg == 32) ? 0xffffffffu : (((1u << cpg) - 1u) << (lane & ~(cpg - 1)));
    uint4 raw[L];
#pragma unroll
    for (int l = 0; l < L; ++l) {
        const int64_t c = c0 + l * 32;
        raw[l] = (c < e.chunks) ? __ldcs(reinterpret_cast<const uint4 *>(w + c * V)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int l = 0; l < L; ++l) {
        const int64_t c = c0 + l * 32;
        rtn_slot<T, NATIVE, BITS, ST, ZT>(raw[l], c, c < e.chunks, lane, cpg, cpg_log2, seg_mask, floor_s, e.q,
                                          reinterpret_cast<ST *>(e.scale), reinterpret_cast<ZT *>(e.zp));
    }
}

// ---- streaming variant of the fast path: bulk-async copies into a shared-memory ring ------
//
// HBM latency under load on B200 is about 2 us, so ~100 KB per SM have to be in flight to
// approach the bandwidth roofline -- more than register-resident loads of a compute-heavy
// kernel can hold.  Persistent CTAs therefore pull the (fully contiguous) weight stream with
// cp.async.bulk (the 1-D form of the TMA engine) into a STAGES-deep ring of 16 KB tiles,
// completion signalled on mbarriers; all threads then read their 16-byte chunks from
// shared memory (lane-contiguous, conflict-free) and run the same per-chunk code as above.
// Every wait is bounded: a wait that runs out sets g_rtn_status and the thread returns.
__device__ int g_rtn_status = 0;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

constexpr int RTN_STAGES = 4;
constexpr int RTN_THREADS = 512;
constexpr int RTN_L = 2;                                   // 16-byte chunks per thread per tile
constexpr int RTN_TILE_CHUNKS = RTN_THREADS * RTN_L;       // 16 KB tiles
constexpr unsigned RTN_WAIT_LIMIT = 1u << 22;

template <typename T, bool NATIVE, int BITS, typename ST, typename ZT>
__global__ void __launch_bounds__(RTN_THREADS, 3)
rtn_quantize_pack_stream_kernel(const T *__restrict__ w, int64_t total_chunks, int64_t num_tiles, int cpg_log2,
                                float floor_s, int32_t *__restrict__ qweight, ST *__restrict__ scale,
                                ZT *__restrict__ zp) {
    constexpr int V = Elems16<T>::V;
    extern __shared__ __align__(128) unsigned char rtn_smem[];
    uint4 *ring = reinterpret_cast<uint4 *>(rtn_smem);                         // [STAGES][TILE_CHUNKS]
    uint64_t *full = reinterpret_cast<uint64_t *>(ring + RTN_STAGES * RTN_TILE_CHUNKS);
    const int tid = threadIdx.x, lane = tid & 31;
    const int cpg = 1 << cpg_log2;
    const uint32_t seg_mask = (cpg == 32) ? 0xffffffffu : (((1u << cpg) - 1u) << (lane & ~(cpg - 1)));
    const uint4 *src = reinterpret_cast<const uint4 *>(w);

    auto tile_of = [&](int64_t it) { return (int64_t)blockIdx.x + it * gridDim.x; };
    auto issue = [&](int64_t it) {                          // thread 0 only
        const int64_t tile = tile_of(it);
        if (tile >= num_tiles) return;
        const int st = (int)(it % RTN_STAGES);
        const int64_t first = tile * RTN_TILE_CHUNKS;
        const int64_t n = (total_chunks - first < RTN_TILE_CHUNKS) ? (total_chunks - first) : RTN_TILE_CHUNKS;
        mbar_expect_tx(&full[st], (unsigned)(n * 16));
        bulk_g2s(ring + st * RTN_TILE_CHUNKS, src + first, (unsigned)(n * 16), &full[st]);
    };
    if (tid == 0) {
        for (int s = 0; s < RTN_STAGES; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        for (int s = 0; s < RTN_STAGES; ++s) issue(s);
    }
    for (int64_t it = 0; tile_of(it) < num_tiles; ++it) {
        const int st = (int)(it % RTN_STAGES);
        const unsigned parity = (unsigned)((it / RTN_STAGES) & 1);
        unsigned tries = 0;
        while (!mbar_try_wait(&full[st], parity)) {
            if (++tries > RTN_WAIT_LIMIT) { atomicExch(&g_rtn_status, 1); return; }
        }
        const int64_t first = tile_of(it) * RTN_TILE_CHUNKS;
        const uint4 *tile = ring + st * RTN_TILE_CHUNKS;
        uint4 v[RTN_L];
#pragma unroll
        for (int l = 0; l < RTN_L; ++l) {
            const int cl = (tid >> 5) * (32 * RTN_L) + l * 32 + lane;
            v[l] = (first + cl < total_chunks) ? tile[cl] : make_uint4(0, 0, 0, 0);
        }
        // generic-proxy reads of the stage are ordered before the bulk copy that refills it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();                                    // the whole CTA has read this stage
        if (tid == 0) issue(it + RTN_STAGES);
#pragma unroll
        for (int l = 0; l < RTN_L; ++l) {
            const int64_t c = first + (tid >> 5) * (32 * RTN_L) + l * 32 + lane;
            rtn_slot<T, NATIVE, BITS, ST, ZT>(v[l], c, c < total_chunks, lane, cpg, cpg_log2, seg_mask, floor_s,
                                              qweight, scale, zp);
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

// The bulk-async variant is correct and tested but currently slower than the register-load
// kernel (both are instruction-issue bound, about 30 instructions per weight), so it is opt-in
// per call (BW_RTN_TMA_STREAM); the flag of the call in progress on this thread:
thread_local bool t_rtn_stream = false;
// A batched call in progress on this thread: the device table, its length and the grid size.
struct RtnBatchCall { const RtnBatchEntry *table; int njobs; long long blocks; };
thread_local RtnBatchCall t_rtn_batch = {nullptr, 0, 0};

int64_t gcd64(int64_t a, int64_t b) { while (b) { int64_t t = a % b; a = b; b = t; } return a; }

template <typename T, bool NATIVE, int BITS, typename ST, typename ZT>
int launch_typed(const T *w, int64_t N, int64_t K, int g, int32_t *q, ST *scale, ZT *zp, float floor_s,
                 cudaStream_t st) {
    constexpr int V = Elems16<T>::V;
    constexpr int VPI = 32 / BITS;
    constexpr int L = 4;
    const int64_t total = N * K;
    if (total == 0) return BW_OK;
    int cpg_log2 = -1;
    if (g % V == 0) {
        const int cpg = g / V;
        if (cpg <= 32 && (cpg & (cpg - 1)) == 0) { cpg_log2 = 0; while ((1 << cpg_log2) < cpg) ++cpg_log2; }
    }
    if (t_rtn_batch.njobs > 0) {
        // (the caller has checked that every matrix of the batch takes the fast path)
        if (cpg_log2 < 0) return BW_ERR_UNSUPPORTED;
        rtn_quantize_pack_batch_kernel<T, NATIVE, BITS, L, ST, ZT><<<(unsigned)t_rtn_batch.blocks, 256, 0, st>>>(
            t_rtn_batch.table, t_rtn_batch.njobs, cpg_log2, floor_s);
        return check_launch("rtn_quantize_pack_batch_kernel");
    }
    if (cpg_log2 >= 0 && aligned_to(w, 16) && aligned_to(q, 8)) {
        const int64_t chunks = total / V;
        const int64_t warps = (chunks + 32 * L - 1) / (32 * L);
        const int64_t blocks = (warps + 7) / 8;
        if (blocks > 0x7fffffff) return BW_ERR_SHAPE;
        const int64_t tiles = (chunks + RTN_TILE_CHUNKS - 1) / RTN_TILE_CHUNKS;
        if (t_rtn_stream && tiles >= 148 * 4) {
            auto kern = rtn_quantize_pack_stream_kernel<T, NATIVE, BITS, ST, ZT>;
            const size_t smem = (size_t)RTN_STAGES * RTN_TILE_CHUNKS * 16 + RTN_STAGES * sizeof(uint64_t);
            BW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            const int64_t grid = tiles < 148 * 3 ? tiles : 148 * 3;
            kern<<<(unsigned)grid, RTN_THREADS, smem, st>>>(w, chunks, tiles, cpg_log2, floor_s, q, scale, zp);
            return check_launch("rtn_quantize_pack_stream_kernel");
        }
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

// Test hook: compares div_by_recip with __fdiv_rn on pseudo-random operand pairs inside the
// fast path's domain (plus adversarial significands); returns the number of mismatches.
__global__ void div_check_kernel(uint64_t n, uint64_t seed, unsigned long long *mismatches) {
    unsigned long long bad = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t z = (i + 1) * 0x9E3779B97F4A7C15ull + seed;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
        uint32_t mv = (uint32_t)z & 0x7fffffu, ms = (uint32_t)(z >> 23) & 0x7fffffu;
        const uint32_t kind = (uint32_t)(z >> 60);
        if (kind == 0) ms = 0x7fffffu;                 // all-ones divisor significand
        else if (kind == 1) ms = 0;                    // power of two
        else if (kind == 2) ms = 0x7ffffeu;
        else if (kind == 3) mv = 0x7fffffu;
        else if (kind == 4) mv = ms;                   // quotient exactly 1 * 2^k
        else if (kind == 5) ms &= 0x7ff000u;           // short divisor significands (fp16/bf16 scales)
        const float qconst = kind == 6 ? 15.0f : (kind == 7 ? 255.0f : (kind == 8 ? 3.0f : 0.0f));
        const int ev = 127 - 38 + (int)((z >> 46) % 77);   // |v| in [2^-38, 2^38]
        const int es = 127 - 39 + (int)((z >> 53) % 78);   // s in [2^-39, 2^38]
        const float v = __uint_as_float(((uint32_t)(z >> 45) & 1u) << 31 | (uint32_t)ev << 23 | mv);
        const float s = qconst != 0.0f ? qconst : __uint_as_float((uint32_t)es << 23 | ms);   // Qmax divisors too
        const float a = div_by_recip(v, s, __frcp_rn(s)), b = __fdiv_rn(v, s);
        if (__float_as_uint(a) != __float_as_uint(b)) ++bad;
        // the packed form, with a second numerator in the other lane
        const float v2 = -v * 0.75f;
        const float2 p = div_by_recip2(make_float2(v, v2), s, __frcp_rn(s));
        if (__float_as_uint(p.x) != __float_as_uint(b) || __float_as_uint(p.y) != __float_as_uint(__fdiv_rn(v2, s))) ++bad;
    }
    if (bad) atomicAdd(mismatches, bad);
}
long long div_self_check(unsigned long long n, unsigned long long seed) {
    unsigned long long *d = nullptr, h = 0;
    if (cudaMalloc(&d, sizeof(h)) != cudaSuccess) return -1;
    cudaMemset(d, 0, sizeof(h));
    div_check_kernel<<<148 * 8, 256>>>(n, seed, d);
    const cudaError_t e = cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
    cudaFree(d);
    return e == cudaSuccess ? (long long)h : -1;
}

// Reads and clears the status word the bounded waits set (0 = no wait ever ran out).
int rtn_device_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_rtn_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) (void)cudaMemcpyToSymbol(g_rtn_status, &zero, sizeof(int));
    return v;
}

int rtn_quantize_pack(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g,
                      int32_t *q, void *scale, int scale_dtype, void *zp, int zp_dtype,
                      unsigned flags, cudaStream_t st) {
    const bool native = !(flags & BW_RTN_UPCAST_F32);
    t_rtn_stream = (flags & BW_RTN_TMA_STREAM) != 0;
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

size_t rtn_batch_table_bytes(int njobs) { return njobs > 0 ? (size_t)njobs * sizeof(RtnBatchEntry) : 0; }

// Quantizes `njobs` matrices with ONE kernel launch when all of them take the fast path (group a
// power-of-two multiple of 16 bytes of weights, 16-byte aligned weights, 8-byte aligned packed
// words), else one launch per matrix.  `table_dev` receives the job table (one asynchronous copy).
int rtn_quantize_pack_batch(const bw_rtn_job *jobs, int njobs, int w_dtype, int bits, int g, int scale_dtype,
                            int zp_dtype, unsigned flags, void *table_dev, cudaStream_t st) {
    const int v = 16 / (int)dtype_size(w_dtype), lpt = 4;
    bool fast = table_dev != nullptr && g % v == 0 && (g / v) <= 32 && ((g / v) & (g / v - 1)) == 0 && njobs <= 4096;
    for (int j = 0; j < njobs && fast; ++j)
        fast = aligned_to(jobs[j].w, 16) && aligned_to(jobs[j].qweight, 8);
    if (!fast) {
        for (int j = 0; j < njobs; ++j) {
            if (jobs[j].N * jobs[j].K == 0) continue;
            const int rc = rtn_quantize_pack(jobs[j].w, w_dtype, jobs[j].N, jobs[j].K, bits, g, jobs[j].qweight, jobs[j].scale,
                                             scale_dtype, jobs[j].zero_point, zp_dtype, flags, st);
            if (rc != BW_OK) return rc;
        }
        return BW_OK;
    }
    static thread_local RtnBatchEntry host_table[4096];
    long long blocks = 0;
    int used = 0, first = -1;
    for (int j = 0; j < njobs; ++j) {
        const long long chunks = (long long)(jobs[j].N * jobs[j].K) / v;
        if (chunks == 0) continue;
        if (first < 0) first = j;
        host_table[used++] = {jobs[j].w, jobs[j].qweight, jobs[j].scale, jobs[j].zero_point, chunks, blocks};
        const long long warps = (chunks + 32 * lpt - 1) / (32 * lpt);
        blocks += (warps + 7) / 8;
    }
    if (used == 0) return BW_OK;
    if (blocks > 0x7fffffff) return BW_ERR_SHAPE;
    // (pageable source: the runtime stages the table before the call returns)
    BW_CUDA_TRY(cudaMemcpyAsync(table_dev, host_table, (size_t)used * sizeof(RtnBatchEntry), cudaMemcpyHostToDevice, st));
    t_rtn_batch = {reinterpret_cast<const RtnBatchEntry *>(table_dev), used, blocks};
    const int rc = rtn_quantize_pack(jobs[first].w, w_dtype, jobs[first].N, jobs[first].K, bits, g, jobs[first].qweight,
                                     jobs[first].scale, scale_dtype, jobs[first].zero_point, zp_dtype, flags, st);
    t_rtn_batch = {nullptr, 0, 0};
    return rc;
}

}  // namespace bw
