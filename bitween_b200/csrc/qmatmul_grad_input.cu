// grad_input of the QuantizedLinear backward pass: grad_in[M,K] = grad_out[M,N] . W[N,K],
// W = GradT( scale * (code - zero_point) ) evaluated in fp32 and cast to the gradient dtype.
//
// Replaces the eager unpack loop + fp32 dequantize + matmul of
// QuantizedLinearFunction.backward (bitween/modules.py:108-141) without materialising W.
// Each thread owns one packed word column (32/bits consecutive k) for a block of up to 8
// tokens and walks down the rows, so packed words are read coalesced across the warp and
// each is expanded once per token block.  That CUDA-core kernel serves fp32 gradients and
// layouts the tensor-core kernel below cannot take.
//
// fp16 / bf16 gradients (what LoRA fine-tuning and mixed-precision retraining produce) run on
// the tensor cores: a CTA owns 128 tokens x 64 k of grad_in and walks over N in steps of 64 rows;
// each step the CTA expands the [64 rows x 64 k] block of W ONCE (exactly GradT(scale * (code -
// zp)), fp32 arithmetic, one rounding) into shared memory, transposed and padded so that the
// mma.sync B fragments are conflict-free 32-bit loads, while the eight warps multiply the
// previous block: mma.sync.m16n8k16 with grad_out as the row-major A operand, fp32 accumulators.
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

// ---- tensor-core kernel --------------------------------------------------------------------
constexpr int GI_BM = 128, GI_BK = 64, GI_BN = 64;   // tokens x k per CTA, weight rows per step
constexpr int GI_PITCH = GI_BN + 8;                  // elements between k columns of the expanded block: conflict-free
                                                     // 32-bit fragment loads (36 words: 8 columns land on banks 0,4,...,28)

template <typename GT> __device__ __forceinline__ void mma_grad(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_grad<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_grad<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Each step the CTA expands the [64 rows x 64 k] block of W once into shared memory (transposed,
// [k][row]) while the eight warps multiply the previous block; the packed words, their scales and
// zero points and the grad_out fragments of the NEXT step are already in registers by then, so
// the global-memory latency hides behind the 32 MMAs of a step.
template <int BITS, typename GT>
__global__ void __launch_bounds__(256)
grad_input_tc_kernel(const GT *__restrict__ go, int64_t M, int64_t N, int64_t K, const int32_t *__restrict__ q,
                     const __half *__restrict__ scale, const __half *__restrict__ zp, GT *__restrict__ gi, int g,
                     int words_per_row, int64_t G) {
    constexpr int VPI = 32 / BITS;
    constexpr int32_t MASK = (1 << BITS) - 1;
    constexpr int WPB = GI_BK / VPI;                       // packed words per row of the block: 16 / 8 / 4
    constexpr int WPT = GI_BN * WPB / 256;                 // words per thread and step: 4 / 2 / 1
    __shared__ __align__(16) GT wt[2][GI_BK * GI_PITCH];   // [buffer][k][row] expanded weights
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
    const int64_t k0 = (int64_t)blockIdx.x * GI_BK, m0 = (int64_t)blockIdx.y * GI_BM + warp * 16;
    const bool one_group = (g % VPI) == 0;                 // a packed word lies in one quantization group
    float acc[GI_BK / 8][4];
#pragma unroll
    for (int j = 0; j < GI_BK / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;

    // registers holding the next step's global data
    int32_t words[WPT];
    float sv[WPT], zv[WPT];
    uint32_t a_next[GI_BN / 16][4];
    auto fetch = [&](int64_t n0) {
#pragma unroll
        for (int u = 0; u < WPT; ++u) {
            const int w = tid + u * 256, er = w % GI_BN, ew = w / GI_BN;   // rows vary fastest: conflict-free stores below
            const int64_t n = n0 + er, kw = k0 + (int64_t)ew * VPI;
            words[u] = 0; sv[u] = 0.0f; zv[u] = 0.0f;
            if (n < N && kw < K) {
                words[u] = __ldg(q + n * words_per_row + kw / VPI);
                const int64_t gidx = n * G + kw / g;
                sv[u] = __half2float(__ldg(scale + gidx));
                zv[u] = __half2float(__ldg(zp + gidx));
            }
        }
#pragma unroll
        for (int sub = 0; sub < GI_BN / 16; ++sub)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int64_t m = m0 + gq + (e & 1) * 8, n = n0 + sub * 16 + 2 * t + (e >> 1) * 8;
                a_next[sub][e] = (m < M && n < N) ? __ldg(reinterpret_cast<const unsigned int *>(go + m * N + n)) : 0u;
            }
    };
    auto expand = [&](int64_t n0, int buf) {
#pragma unroll
        for (int u = 0; u < WPT; ++u) {
            const int w = tid + u * 256, er = w % GI_BN, ew = w / GI_BN;
            const int64_t n = n0 + er, kw = k0 + (int64_t)ew * VPI;
            GT *dst = wt[buf] + (size_t)(ew * VPI) * GI_PITCH + er;
            const bool live = n < N && kw < K;
#pragma unroll
            for (int i = 0; i < VPI; ++i) {
                float s1 = sv[u], z1 = zv[u];
                if (!one_group && live) {
                    const int64_t gidx = n * G + (kw + i) / g;
                    s1 = __half2float(__ldg(scale + gidx));
                    z1 = __half2float(__ldg(zp + gidx));
                }
                const float wv = live ? __fmul_rn(s1, __fsub_rn((float)((words[u] >> (i * BITS)) & MASK), z1)) : 0.0f;
                dst[(size_t)i * GI_PITCH] = from_f32<GT>(wv);
            }
        }
    };
    const int64_t steps = (N + GI_BN - 1) / GI_BN;
    fetch(0);
    expand(0, 0);
    uint32_t a_cur[GI_BN / 16][4];
#pragma unroll
    for (int sub = 0; sub < GI_BN / 16; ++sub)
#pragma unroll
        for (int e = 0; e < 4; ++e) a_cur[sub][e] = a_next[sub][e];
    __syncthreads();
    for (int64_t st = 0; st < steps; ++st) {
        const int buf = (int)(st & 1);
        if (st + 1 < steps) fetch((st + 1) * GI_BN);              // in flight during the MMAs below
        const GT *wb = wt[buf];
#pragma unroll
        for (int sub = 0; sub < GI_BN / 16; ++sub)
#pragma unroll
            for (int j = 0; j < GI_BK / 8; ++j) {
                const GT *col = wb + (size_t)(j * 8 + gq) * GI_PITCH + sub * 16 + 2 * t;
                mma_grad<GT>(acc[j], a_cur[sub], *reinterpret_cast<const uint32_t *>(col), *reinterpret_cast<const uint32_t *>(col + 8));
            }
        if (st + 1 < steps) {
            expand((st + 1) * GI_BN, buf ^ 1);
#pragma unroll
            for (int sub = 0; sub < GI_BN / 16; ++sub)
#pragma unroll
                for (int e = 0; e < 4; ++e) a_cur[sub][e] = a_next[sub][e];
        }
        __syncthreads();
    }
    // C fragment: rows m0+gq / +8, columns k0 + 8j + 2t, +1
#pragma unroll
    for (int j = 0; j < GI_BK / 8; ++j) {
        const int64_t k = k0 + j * 8 + 2 * t;
        if (k >= K) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t m = m0 + gq + h * 8;
            if (m >= M) continue;
            GT pair[2] = {from_f32<GT>(acc[j][2 * h]), from_f32<GT>(acc[j][2 * h + 1])};
            *reinterpret_cast<uint32_t *>(gi + m * K + k) = *reinterpret_cast<const uint32_t *>(pair);
        }
    }
}

template <int BITS, typename GT>
int launch_tc(const void *go, int64_t M, int64_t N, int64_t K, const int32_t *q, const __half *scale,
              const __half *zp, void *gi, int g, cudaStream_t st) {
    const int64_t kblocks = (K + GI_BK - 1) / GI_BK, mblocks = (M + GI_BM - 1) / GI_BM;
    if (kblocks > 0x7fffffff || mblocks > 65535) return BW_ERR_SHAPE;
    dim3 grid((unsigned)kblocks, (unsigned)mblocks, 1);
    grad_input_tc_kernel<BITS, GT><<<grid, 256, 0, st>>>((const GT *)go, M, N, K, q, scale, zp, (GT *)gi, g,
                                                         (int)(K / (32 / BITS)), K / g);
    return check_launch("grad_input_tc_kernel");
}

// 16-bit gradients whose rows allow 32-bit accesses at even columns run on the tensor cores.
inline bool grad_tc_ok(const void *go, const void *gi, int dt, int64_t N, int64_t K) {
    return (dt == BW_F16 || dt == BW_BF16) && N % 2 == 0 && K % 2 == 0 && aligned_to(go, 4) && aligned_to(gi, 4);
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
    if (grad_tc_ok(go, gi, dt, N, K)) {
        if (dt == BW_F16) return launch_tc<BITS, __half>(go, M, N, K, q, scale, zp, gi, g, st);
        return launch_tc<BITS, __nv_bfloat16>(go, M, N, K, q, scale, zp, gi, g, st);
    }
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
