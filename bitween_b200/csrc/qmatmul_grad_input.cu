// grad_input of the QuantizedLinear backward pass: grad_in[M,K] = grad_out[M,N] . W[N,K],
// W = GradT( scale * (code - zero_point) ) evaluated in fp32 and cast to the gradient dtype.
//
// Replaces the eager unpack loop + fp32 dequantize + matmul of
// QuantizedLinearFunction.backward (bitween/modules.py:108-141) without materialising W.
// Each thread owns one packed word column (32/bits consecutive k) for a block of up to 8
// tokens and walks down the rows, so packed words are read coalesced across the warp and
// each is expanded once per token block.  This is the drop-in completeness path for LoRA /
// retraining callers, not one of the measured configurations.
#include "bw_common.cuh"

namespace bw {
namespace {

constexpr int TOK = 8;

template <int BITS, typename GT>
__global__ void __launch_bounds__(128)
grad_input_kernel(const GT *__restrict__ go, int64_t M, int64_t N, int64_t K,
                  const int32_t *__restrict__ q, const __half *__restrict__ scale,
                  const __half *__restrict__ zp, GT *__restrict__ gi, int g, int words_per_row,
                  int64_t G) {
    constexpr int VPI = 32 / BITS;
    constexpr int32_t MASK = (1 << BITS) - 1;
    const int wi = blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t m0 = (int64_t)blockIdx.y * TOK;
    if (wi >= words_per_row) return;
    float acc[TOK][VPI];
#pragma unroll
    for (int j = 0; j < TOK; ++j)
#pragma unroll
        for (int i = 0; i < VPI; ++i) acc[j][i] = 0.0f;
    const bool one_group = (g % VPI) == 0;
    for (int64_t n = 0; n < N; ++n) {
        const int32_t word = q[n * words_per_row + wi];
        float wv[VPI];
        if (one_group) {
            const int64_t gidx = n * G + ((int64_t)wi * VPI) / g;
            const float s = __half2float(scale[gidx]), z = __half2float(zp[gidx]);
#pragma unroll
            for (int i = 0; i < VPI; ++i)
                wv[i] = to_f32<GT>(from_f32<GT>(__fmul_rn(s, __fsub_rn((float)((word >> (i * BITS)) & MASK), z))));
        } else {
#pragma unroll
            for (int i = 0; i < VPI; ++i) {
                const int64_t gidx = n * G + ((int64_t)wi * VPI + i) / g;
                const float s = __half2float(scale[gidx]), z = __half2float(zp[gidx]);
                wv[i] = to_f32<GT>(from_f32<GT>(__fmul_rn(s, __fsub_rn((float)((word >> (i * BITS)) & MASK), z))));
            }
        }
#pragma unroll
        for (int j = 0; j < TOK; ++j) {
            if (m0 + j < M) {
                const float gv = to_f32<GT>(go[(m0 + j) * N + n]);
#pragma unroll
                for (int i = 0; i < VPI; ++i) acc[j][i] = fmaf(gv, wv[i], acc[j][i]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < TOK; ++j) {
        if (m0 + j < M) {
#pragma unroll
            for (int i = 0; i < VPI; ++i) gi[(m0 + j) * K + (int64_t)wi * VPI + i] = from_f32<GT>(acc[j][i]);
        }
    }
}

template <int BITS, typename GT>
int launch(const void *go, int64_t M, int64_t N, int64_t K, const int32_t *q, const __half *scale,
           const __half *zp, void *gi, int g, cudaStream_t st) {
    const int wpr = (int)(K / (32 / BITS));
    const int64_t mblocks = (M + TOK - 1) / TOK;
    if (mblocks > 65535) return BW_ERR_SHAPE;
    dim3 grid((unsigned)((wpr + 127) / 128), (unsigned)mblocks, 1);
    grad_input_kernel<BITS, GT><<<grid, 128, 0, st>>>((const GT *)go, M, N, K, q, scale, zp, (GT *)gi, g,
                                                      wpr, K / g);
    return check_launch("grad_input_kernel");
}

template <int BITS>
int launch_dt(const void *go, int dt, int64_t M, int64_t N, int64_t K, const int32_t *q,
              const __half *scale, const __half *zp, void *gi, int g, cudaStream_t st) {
    switch (dt) {
        case BW_F32: return launch<BITS, float>(go, M, N, K, q, scale, zp, gi, g, st);
        case BW_F16: return launch<BITS, __half>(go, M, N, K, q, scale, zp, gi, g, st);
        case BW_BF16: return launch<BITS, __nv_bfloat16>(go, M, N, K, q, scale, zp, gi, g, st);
        default: return BW_ERR_DTYPE;
    }
}

}  // namespace

int qmatmul_grad_input(const void *go, int dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                       const __half *scale, const __half *zp, void *gi, int bits, int g, cudaStream_t st) {
    if (K > (int64_t)1 << 31) return BW_ERR_SHAPE;
    switch (bits) {
        case 2: return launch_dt<2>(go, dtype, M, N, K, q, scale, zp, gi, g, st);
        case 4: return launch_dt<4>(go, dtype, M, N, K, q, scale, zp, gi, g, st);
        case 8: return launch_dt<8>(go, dtype, M, N, K, q, scale, zp, gi, g, st);
        default: return BW_ERR_BITS;
    }
}

}  // namespace bw
