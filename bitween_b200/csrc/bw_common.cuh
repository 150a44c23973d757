// Shared helpers of the sm_100a kernels behind the C ABI in include/bitween_b200.h.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bitween_b200.h"

namespace bw {

// Records a failed CUDA runtime call for bw_last_cuda_error(); returns BW_ERR_CUDA.
int record_cuda_error(cudaError_t e, const char *where);
void set_last_kernel(const char *name);

#define BW_CUDA_TRY(expr)                                              \
    do {                                                               \
        cudaError_t _e = (expr);                                       \
        if (_e != cudaSuccess) return ::bw::record_cuda_error(_e, #expr); \
    } while (0)

inline int check_launch(const char *where) {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BW_OK : record_cuda_error(e, where);
}

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline size_t dtype_size(int dt) {
    switch (dt) {
        case BW_F32: case BW_I32: return 4;
        case BW_F16: case BW_BF16: return 2;
        default: return 0;
    }
}

// Validates the (bits, group_size, K) triple the way the reference does
// (bitween/functional.py:6,12-17 and the reshape at :42-43).
inline int check_quant_shape(int64_t N, int64_t K, int bits, int group_size) {
    if (bits != 2 && bits != 4 && bits != 8) return BW_ERR_BITS;
    if (group_size < 1) return BW_ERR_GROUP;
    if (N < 0 || K < 0) return BW_ERR_SHAPE;
    if (K % group_size != 0) return BW_ERR_GROUP;
    if (K % (32 / bits) != 0) return BW_ERR_SHAPE;
    if (N > 0 && K > (int64_t)1 << 40) return BW_ERR_SHAPE;
    if (N * K < 0 || (K > 0 && N > ((int64_t)1 << 62) / K)) return BW_ERR_SHAPE;
    return BW_OK;
}

// ---- device-side element load/store in fp32 ---------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<int32_t>(int32_t v) { return (float)v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- output epilogue shared by the quantized-matmul kernels ------------------------------
// What follows the linear in a decoder block, done on the value before it leaves the SM instead
// of by one more elementwise kernel each (the reference adds even the bias with a separate
// kernel, bitween/modules.py:100-101): activation (ReLU, the OPT feed-forward) and residual add.
// fp16 outputs reproduce the eager op-by-op result: fp16(acc), + bias, relu, + residual, each
// rounded to fp16 like the separate torch ops would.
struct Epilogue {
    int act;                  // BW_ACT_NONE | BW_ACT_RELU | BW_ACT_SILU_MUL
    const __half *residual;   // [M, N] fp16, added last, or null
};
// The epilogue of the bw_qmatmul_fused call in progress on this thread (none otherwise).
Epilogue current_epilogue();

__device__ __forceinline__ void store_output(void *out, int out_dtype, int64_t idx, float v, bool has_bias, __half bias,
                                             const Epilogue &ep) {
    if (out_dtype == BW_F16) {
        __half c = __float2half_rn(v);                       // the GEMM's fp16 output rounding
        if (has_bias) c = __hadd(c, bias);                   // separate fp16 bias add
        if (ep.act == BW_ACT_RELU) c = __hmax(c, __float2half(0.0f));
        if (ep.residual) c = __hadd(c, ep.residual[idx]);
        reinterpret_cast<__half *>(out)[idx] = c;
    } else {
        if (has_bias) v += __half2float(bias);
        if (ep.act == BW_ACT_RELU) v = fmaxf(v, 0.0f);
        if (ep.residual) v += __half2float(ep.residual[idx]);
        if (out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(out)[idx] = __float2bfloat16_rn(v);
        else reinterpret_cast<float *>(out)[idx] = v;
    }
}


// BW_ACT_SILU_MUL: the packed weight holds gate row i in row 2i and up row i in row 2i+1 (one
// [2*ffn, K] GEMM for the gated feed-forward), and the output [M, N/2] is silu(gate) * up:
// g = the two linears' outputs as the plain call would round them, silu evaluated in fp32 and
// rounded like a torch op on an fp16 tensor, the product rounded once more, then the residual.
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ void store_output_silu_mul(void *out, int out_dtype, int64_t idx, float g, float u, bool has_bias,
                                                      __half bias_g, __half bias_u, const Epilogue &ep) {
    if (out_dtype == BW_F16) {
        __half gh = __float2half_rn(g), uh = __float2half_rn(u);
        if (has_bias) { gh = __hadd(gh, bias_g); uh = __hadd(uh, bias_u); }
        __half c = __hmul(__float2half_rn(silu_f32(__half2float(gh))), uh);
        if (ep.residual) c = __hadd(c, ep.residual[idx]);
        reinterpret_cast<__half *>(out)[idx] = c;
    } else {
        if (has_bias) { g += __half2float(bias_g); u += __half2float(bias_u); }
        float v = silu_f32(g) * u;
        if (ep.residual) v += __half2float(ep.residual[idx]);
        if (out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(out)[idx] = __float2bfloat16_rn(v);
        else reinterpret_cast<float *>(out)[idx] = v;
    }
}

}  // namespace bw
