// Dequantize packed weights: out[n][k] = OutT( float(scale) * (float(code) - float(zp)) ).
//
// One kernel for the three places the reference reconstructs weights: dequantize_rtn
// (bitween/functional.py:47-71, fp32 out), the module's Triton kernel
// (bitween/modules.py:10-58, fp16 scale/zero-point in, fp16 out) and the backward pass
// (bitween/modules.py:121-135).  The expression is evaluated in fp32 exactly as written
// there (one subtract, one multiply, both IEEE-rounded, no FMA contraction), so results
// are bit-identical.
//
// Each thread expands one packed int32 word (read once, unlike the reference kernel
// where every word is re-fetched by 32/bits lanes) into 32/bits outputs stored as one
// vector.  HBM-bound: bits/8 bytes in, sizeof(OutT) bytes out per weight.
#include "bw_common.cuh"

namespace bw {
namespace {

template <int BITS, typename ST, typename ZT, typename OutT>
__global__ void __launch_bounds__(256)
dequantize_kernel(const int32_t *__restrict__ qweight, const ST *__restrict__ scale,
                  const ZT *__restrict__ zp, int64_t total_words, int64_t words_per_row, int64_t G,
                  int g, bool word_in_one_group, OutT *__restrict__ out) {
    constexpr int VPI = 32 / BITS;
    constexpr int32_t MASK = (1 << BITS) - 1;
    const int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= total_words) return;
    const int32_t word = __ldcs(qweight + wi);
    const int64_t n = wi / words_per_row;
    const int64_t k0 = (wi - n * words_per_row) * VPI;
    alignas(16) OutT vals[VPI];
    if (word_in_one_group) {
        const int64_t gi = n * G + k0 / g;
        const float s = to_f32<ST>(scale[gi]);
        const float z = to_f32<ZT>(zp[gi]);
#pragma unroll
        for (int i = 0; i < VPI; ++i) {
            const int32_t code = (word >> (i * BITS)) & MASK;   // arithmetic shift, then mask
            vals[i] = from_f32<OutT>(__fmul_rn(s, __fsub_rn((float)code, z)));
        }
    } else {
#pragma unroll
        for (int i = 0; i < VPI; ++i) {
            const int64_t gi = n * G + (k0 + i) / g;
            const float s = to_f32<ST>(scale[gi]);
            const float z = to_f32<ZT>(zp[gi]);
            const int32_t code = (word >> (i * BITS)) & MASK;
            vals[i] = from_f32<OutT>(__fmul_rn(s, __fsub_rn((float)code, z)));
        }
    }
    OutT *dst = out + wi * VPI;
    constexpr int BYTES = VPI * sizeof(OutT);
    if constexpr (BYTES % 16 == 0) {
        if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < BYTES / 16; ++j)
                __stcs(reinterpret_cast<uint4 *>(dst) + j, reinterpret_cast<const uint4 *>(vals)[j]);
            return;
        }
    } else if constexpr (BYTES == 8) {
        if ((reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
            __stcs(reinterpret_cast<uint2 *>(dst), *reinterpret_cast<const uint2 *>(vals));
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < VPI; ++i) dst[i] = vals[i];
}

template <int BITS, typename ST, typename ZT, typename OutT>
int launch4(const int32_t *q, const ST *s, const ZT *z, int64_t N, int64_t K, int g, OutT *out,
            cudaStream_t st) {
    constexpr int VPI = 32 / BITS;
    const int64_t wpr = K / VPI;
    const int64_t total = N * wpr;
    if (total == 0) return BW_OK;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffff) return BW_ERR_SHAPE;
    dequantize_kernel<BITS, ST, ZT, OutT><<<(unsigned)blocks, 256, 0, st>>>(
        q, s, z, total, wpr, K / g, g, g % VPI == 0, out);
    return check_launch("dequantize_kernel");
}

template <int BITS, typename ST, typename ZT>
int launch3(const int32_t *q, const ST *s, const ZT *z, int64_t N, int64_t K, int g, void *out,
            int out_dtype, cudaStream_t st) {
    switch (out_dtype) {
        case BW_F32: return launch4<BITS, ST, ZT, float>(q, s, z, N, K, g, (float *)out, st);
        case BW_F16: return launch4<BITS, ST, ZT, __half>(q, s, z, N, K, g, (__half *)out, st);
        case BW_BF16: return launch4<BITS, ST, ZT, __nv_bfloat16>(q, s, z, N, K, g, (__nv_bfloat16 *)out, st);
        default: return BW_ERR_DTYPE;
    }
}

template <int BITS, typename ST>
int launch2(const int32_t *q, const ST *s, const void *z, int zp_dtype, int64_t N, int64_t K, int g,
            void *out, int out_dtype, cudaStream_t st) {
    switch (zp_dtype) {
        case BW_I32: return launch3<BITS, ST, int32_t>(q, s, (const int32_t *)z, N, K, g, out, out_dtype, st);
        case BW_F32: return launch3<BITS, ST, float>(q, s, (const float *)z, N, K, g, out, out_dtype, st);
        case BW_F16: return launch3<BITS, ST, __half>(q, s, (const __half *)z, N, K, g, out, out_dtype, st);
        case BW_BF16: return launch3<BITS, ST, __nv_bfloat16>(q, s, (const __nv_bfloat16 *)z, N, K, g, out, out_dtype, st);
        default: return BW_ERR_DTYPE;
    }
}

template <int BITS>
int launch1(const int32_t *q, const void *s, int scale_dtype, const void *z, int zp_dtype, int64_t N,
            int64_t K, int g, void *out, int out_dtype, cudaStream_t st) {
    switch (scale_dtype) {
        case BW_F32: return launch2<BITS, float>(q, (const float *)s, z, zp_dtype, N, K, g, out, out_dtype, st);
        case BW_F16: return launch2<BITS, __half>(q, (const __half *)s, z, zp_dtype, N, K, g, out, out_dtype, st);
        case BW_BF16: return launch2<BITS, __nv_bfloat16>(q, (const __nv_bfloat16 *)s, z, zp_dtype, N, K, g, out, out_dtype, st);
        default: return BW_ERR_DTYPE;
    }
}

}  // namespace

int dequantize(const int32_t *q, const void *scale, int scale_dtype, const void *zp, int zp_dtype,
               int64_t N, int64_t K, int bits, int g, void *out, int out_dtype, cudaStream_t st) {
    switch (bits) {
        case 2: return launch1<2>(q, scale, scale_dtype, zp, zp_dtype, N, K, g, out, out_dtype, st);
        case 4: return launch1<4>(q, scale, scale_dtype, zp, zp_dtype, N, K, g, out, out_dtype, st);
        case 8: return launch1<8>(q, scale, scale_dtype, zp, zp_dtype, N, K, g, out, out_dtype, st);
        default: return BW_ERR_BITS;
    }
}

}  // namespace bw
