// Large-M ("prefill") quantized matmul for sm_100a on the 5th-generation tensor cores:
//   out[M,N] = x[M,K] . W[N,K]^T (+bias),   W = fp16(scale * (code - zero_point)).
//
// Replaces, for many tokens, the reference forward (bitween/modules.py:85-101: Triton
// dequantize to a temporary fp16 [N,K] in HBM, then a library GEMM, then a bias kernel) by one
// kernel that dequantizes straight into the tensor-core operand buffers.
//
// Shape of the computation ("swap-AB"): the MMA's M dimension (128 rows, one TMEM lane each)
// holds 128 WEIGHT rows, its N dimension holds up to 256 TOKENS, so every dequantized weight is
// used by up to 256 tokens of one CTA and the accumulator D^T[n, m] lives in 128 lanes x BN
// fp32 columns of tensor memory.
//
// Warp roles in a CTA of 320 threads (one output tile of 128 weight rows x BN tokens):
//   warp 0       TMA producer: cp.async.bulk.tensor loads the [BN tokens x 64 k] fp16 tile of
//                the activations (128-byte swizzle, no multicast) for each pipeline stage
//   warp 1       allocates tensor memory; one elected lane issues tcgen05.mma (kind::f16,
//                M=128, N=BN, K=16, four per stage) and commits stages / the accumulator
//   warps 2..9   two groups of 128 dequantization threads (one per weight row; the groups take
//                alternate pipeline stages): stream that row's packed
//                words (prefetched one own stage ahead in registers), expand them to fp16 in
//                natural k order and store them as the A operand in the canonical K-major
//                128-byte-swizzled layout; afterwards the same warps are the epilogue:
//                tcgen05.ld of their TMEM lane quadrant, fp16 rounding + bias, coalesced stores
// Stages are handed over with mbarriers (full_a, full_b, empty, acc_full).  Every wait is
// bounded: a wait that runs out records an error in g_tc_status, the CTA drains, frees its
// tensor memory and returns.
#include <cuda.h>

#include "bw_common.cuh"
#include "qmm_dequant.cuh"

namespace bw {
namespace {

constexpr int TC_BM = 128;        // weight rows per tile (MMA M)
constexpr int TC_BK = 64;         // k per stage: 64 fp16 = one 128-byte swizzle row
constexpr int TC_STAGES = 4;
constexpr int TC_DQ_GROUPS = 4;   // dequantization warp groups (4 warps each) taking alternate stages
constexpr int TC_THREADS = 64 + TC_DQ_GROUPS * 128;
constexpr unsigned TC_WAIT_LIMIT = 1u << 22;   // polls of >= 20 ns each: gives up after ~0.1-1 s

__device__ int g_tc_status = 0;

// ---- PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Non-blocking test of a phase (the bounded loop around it does the waiting).
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records the error) when the limit is hit or another
// thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, volatile int *abort_flag, int code) {
    unsigned tries = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        __nanosleep(20);
        if (++tries > TC_WAIT_LIMIT) {
            *abort_flag = code;
            atomicExch(&g_tc_status, code);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_in_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_in_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes (64 fp16)
// stored with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the
// leading byte offset is unused for swizzled K-major layouts, descriptor version 1 (sm_100),
// layout type 2 (SWIZZLE_128B).  `addr` may be advanced by 32 bytes per 16-element k step.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);          // bits [0,14): start address >> 4
    d |= (uint64_t)1 << 16;                           // bits [16,30): leading byte offset >> 4 (ignored)
    d |= (uint64_t)(1024u >> 4) << 32;                // bits [32,46): stride byte offset >> 4
    d |= (uint64_t)1 << 46;                           // bits [46,48): descriptor version
    d |= (uint64_t)2 << 61;                           // bits [61,64): SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: fp16 A and B (format 0), fp32 accumulator (1), both
// operands K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t umma_idesc_f16(int bn) {
    uint32_t d = 0;
    d |= 1u << 4;                                     // c_format = F32
    d |= (uint32_t)(bn >> 3) << 17;                   // n_dim
    d |= (uint32_t)(TC_BM >> 4) << 24;                // m_dim
    return d;
}

struct TcParams {
    const int32_t *q;
    const __half *scale;
    const __half *zp;
    const __half *bias;
    void *out;
    int64_t M, N, K;
    int out_dtype;
    int g_shift;        // log2(group_size)
    int G;              // groups per row
    int words_per_row;  // K / vpi
    int k_stages;       // ceil(K / 64)
    int bn;             // tokens per tile: 32, 64, 128 or 256
};

// Words of one row for one 64-k stage, as 16-byte vectors, and the natural-order expansion.
template <int BITS> struct StageGeom {
    static constexpr int VPI = 32 / BITS;             // codes per word
    static constexpr int WPS = TC_BK / VPI;           // words per row per stage: 4 / 8 / 16
    static constexpr int VPS = WPS / 4;               // 16-byte vectors per row per stage: 1 / 2 / 4
};

// Expands the WPS words of one stage into the row's eight 16-byte chunks (8 consecutive k each).
template <int BITS>
__device__ __forceinline__ void expand_stage(const uint32_t (&w)[StageGeom<BITS>::WPS], const GroupConst (&gc)[4],
                                             int kbase, int g_shift, int grp0, uint4 (&chunk)[8]) {
    constexpr int VPI = 32 / BITS;
    constexpr int WPS = StageGeom<BITS>::WPS;
    Dequant<BITS> dq;
    int cur = -1;
#pragma unroll
    for (int j = 0; j < WPS; ++j) {
        const int gl = min(((kbase + j * VPI) >> g_shift) - grp0, 3);
        if (gl != cur) { dq.set(gc[gl]); cur = gl; }
        if constexpr (BITS == 4) {
            uint32_t p[4];
            dq.run(w[j], p);                          // (c0,c4) (c1,c5) (c2,c6) (c3,c7)
            chunk[j] = make_uint4(pair_lo(p[0], p[1]), pair_lo(p[2], p[3]), pair_hi(p[0], p[1]), pair_hi(p[2], p[3]));
        } else if constexpr (BITS == 8) {
            uint32_t p[2];
            dq.run(w[j], p);                          // (c0,c2) (c1,c3)
            const uint32_t lo = pair_lo(p[0], p[1]), hi = pair_hi(p[0], p[1]);
            if (j & 1) { chunk[j >> 1].z = lo; chunk[j >> 1].w = hi; }
            else { chunk[j >> 1].x = lo; chunk[j >> 1].y = hi; }
        } else {
            uint32_t p[8];
            dq.run(w[j], p);                          // (c_i, c_{i+8}), i = 0..7
            chunk[2 * j] = make_uint4(pair_lo(p[0], p[1]), pair_lo(p[2], p[3]), pair_lo(p[4], p[5]), pair_lo(p[6], p[7]));
            chunk[2 * j + 1] = make_uint4(pair_hi(p[0], p[1]), pair_hi(p[2], p[3]), pair_hi(p[4], p[5]), pair_hi(p[6], p[7]));
        }
    }
}

template <int BITS>
__global__ void __launch_bounds__(TC_THREADS, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap x_map, const TcParams p) {
    using SG = StageGeom<BITS>;
    extern __shared__ unsigned char tc_smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle pattern
    unsigned char *smem = tc_smem_raw + ((1024u - (smem_addr(tc_smem_raw) & 1023u)) & 1023u);
    const int bn = p.bn;
    unsigned char *a_tiles = smem;                                        // [STAGES][128][128 B]
    unsigned char *b_tiles = smem + TC_STAGES * TC_BM * 128;              // [STAGES][bn][128 B]
    uint64_t *bars = reinterpret_cast<uint64_t *>(b_tiles + (size_t)TC_STAGES * bn * 128);
    uint64_t *full_a = bars, *full_b = bars + TC_STAGES, *empty = bars + 2 * TC_STAGES, *acc_full = bars + 3 * TC_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * TC_STAGES + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * TC_BM;
    const int m0 = blockIdx.y * bn;
    const uint32_t tmem_cols = bn < 32 ? 32u : (uint32_t)bn;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&full_a[s], 4); mbar_init(&full_b[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer: activations ----
        if (lane == 0) {
            for (int kt = 0; kt < p.k_stages; ++kt) {
                const int s = kt % TC_STAGES;
                const unsigned ph = (unsigned)(kt / TC_STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, 1)) break;
                mbar_expect_tx(&full_b[s], (unsigned)bn * 128u);
                tma_load_2d(b_tiles + (size_t)s * bn * 128, &x_map, kt * TC_BK, m0, &full_b[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(bn);
            bool ok = true;
            for (int kt = 0; kt < p.k_stages && ok; ++kt) {
                const int s = kt % TC_STAGES;
                const unsigned ph = (unsigned)(kt / TC_STAGES) & 1u;
                ok = mbar_wait(&full_a[s], ph, abort_flag, 2) && mbar_wait(&full_b[s], ph, abort_flag, 3);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_addr(a_tiles + (size_t)s * TC_BM * 128);
                const uint32_t b_addr = smem_addr(b_tiles + (size_t)s * bn * 128);
#pragma unroll
                for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                    umma_f16(tmem_base, umma_smem_desc(a_addr + k4 * 32), umma_smem_desc(b_addr + k4 * 32), idesc,
                             (kt | k4) != 0 ? 1u : 0u);
                umma_commit(&empty[s]);       // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(acc_full);    // accumulator complete
        }
    } else {
        // ---- dequantization threads (one weight row each), then epilogue ----
        const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
        const int dgroup = (warp - 2) >> 2;              // this group expands stages dgroup, dgroup+2, ...
        const int row = quad * 32 + lane;                // tile row == TMEM lane
        int64_t n = (int64_t)n0 + row;
        const bool n_ok = n < p.N;
        if (!n_ok) n = p.N - 1;
        const uint4 *qrow = reinterpret_cast<const uint4 *>(p.q + n * p.words_per_row);
        const __half *srow = p.scale + n * p.G, *zrow = p.zp + n * p.G;
        const int vec_per_row = p.words_per_row >> 2;
        const int gps = max(1, TC_BK >> p.g_shift);      // groups per stage (<= 4)

        uint4 wv[SG::VPS];
        GroupConst gcs[4];
        auto prefetch = [&](int kt) {
#pragma unroll
            for (int i = 0; i < SG::VPS; ++i) {
                const int v = min(kt * SG::VPS + i, vec_per_row - 1);   // past-the-end k meets zero activations
                wv[i] = __ldg(qrow + v);
            }
            const int grp0 = (kt * TC_BK) >> p.g_shift;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i < gps) {
                    const int grp = min(grp0 + i, p.G - 1);
                    gcs[i].s2 = h2_as_u32(__half2half2(__ldg(srow + grp)));
                    gcs[i].z1024 = h2_as_u32(__hadd2(__half2half2(__ldg(zrow + grp)), __float2half2_rn(1024.0f)));
                } else {
                    gcs[i] = gcs[0];
                }
            }
        };
        if (dgroup < p.k_stages) prefetch(dgroup);
        bool ok = true;
        for (int kt = dgroup; kt < p.k_stages; kt += TC_DQ_GROUPS) {
            const int s = kt % TC_STAGES;
            const unsigned ph = (unsigned)(kt / TC_STAGES) & 1u;
            uint32_t w[SG::WPS];
#pragma unroll
            for (int i = 0; i < SG::VPS; ++i) { w[4 * i] = wv[i].x; w[4 * i + 1] = wv[i].y; w[4 * i + 2] = wv[i].z; w[4 * i + 3] = wv[i].w; }
            GroupConst gc_now[4] = {gcs[0], gcs[1], gcs[2], gcs[3]};
            if (kt + TC_DQ_GROUPS < p.k_stages) prefetch(kt + TC_DQ_GROUPS);
            uint4 chunk[8];
            expand_stage<BITS>(w, gc_now, kt * TC_BK, p.g_shift, (kt * TC_BK) >> p.g_shift, chunk);
            ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, abort_flag, 4));   // warp-uniform
            if (!ok) break;
            uint4 *arow = reinterpret_cast<uint4 *>(a_tiles + (size_t)s * TC_BM * 128 + (size_t)row * 128);
#pragma unroll
            for (int c = 0; c < 8; ++c) arow[c ^ (row & 7)] = chunk[c];
            fence_proxy_async_smem();                    // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_a[s]);
        }
        // ---- epilogue ----
        if (__all_sync(0xffffffffu, ok && mbar_wait(acc_full, 0u, abort_flag, 5))) {
            tc_fence_after();
            const __half bias_h = (p.bias && n_ok) ? p.bias[n] : __float2half(0.0f);
            // the warp groups share the lane quadrants and split the token columns
            const int nblk = bn / 32, per = (nblk + TC_DQ_GROUPS - 1) / TC_DQ_GROUPS;
            for (int cb = dgroup * per; cb < min(nblk, (dgroup + 1) * per); ++cb) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), r);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int64_t m = (int64_t)m0 + cb * 32 + j;
                    if (n_ok && m < p.M) {
                        float v = __uint_as_float(r[j]);
                        if (p.out_dtype == BW_F16) {
                            __half c = __float2half_rn(v);
                            if (p.bias) c = __hadd(c, bias_h);
                            reinterpret_cast<__half *>(p.out)[m * p.N + n] = c;
                        } else {
                            if (p.bias) v += __half2float(bias_h);
                            if (p.out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[m * p.N + n] = __float2bfloat16_rn(v);
                            else reinterpret_cast<float *>(p.out)[m * p.N + n] = v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// Activations that are not fp16 are cast once (bitween/modules.py:74) into caller scratch.
template <typename XT>
__global__ void __launch_bounds__(256) cast_to_f16_kernel(const XT *__restrict__ x, __half *__restrict__ y, int64_t n) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i + 8 <= n) {
        alignas(16) __half h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = from_f32<__half>(to_f32<XT>(x[i + j]));
        *reinterpret_cast<uint4 *>(y + i) = *reinterpret_cast<const uint4 *>(h);
    } else {
        for (int64_t j = i; j < n; ++j) y[j] = from_f32<__half>(to_f32<XT>(x[j]));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

template <int BITS>
int launch_tc(const CUtensorMap &map, const TcParams &p, cudaStream_t st) {
    auto kern = qmm_tc_kernel<BITS>;
    const size_t smem = (size_t)TC_STAGES * TC_BM * 128 + (size_t)TC_STAGES * p.bn * 128 + 256 + 1024;
    static size_t configured[64] = {};
    int dev = 0;
    BW_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
        BW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    const dim3 grid((unsigned)((p.N + TC_BM - 1) / TC_BM), (unsigned)((p.M + p.bn - 1) / p.bn), 1);
    kern<<<grid, TC_THREADS, smem, st>>>(map, p);
    return check_launch("qmm_tc_kernel");
}

}  // namespace

static bool g_tc_enabled = true;
void set_tc_enabled(int on) { g_tc_enabled = on != 0; }

// Layout preconditions of the tensor-core kernel (others run on the streaming / general kernels).
bool tc_path_ok(int64_t M, int64_t N, int64_t K, const int32_t *q, int bits, int g) {
    if (!g_tc_enabled) return false;
    const int vpi = 32 / bits;
    if (M < 1 || N < 1 || K < 1) return false;
    if (g & (g - 1)) return false;                    // power-of-two groups
    if (g < 16 || g < vpi) return false;              // at most four groups per 64-k stage
    if (K % (4 * vpi) != 0) return false;             // whole 16-byte vectors of packed words per row
    if (K % 8 != 0) return false;                     // TMA: row pitch of the fp16 activations % 16 bytes
    if (M > 0x7fffffff || K > 0x7fffffff || N > ((int64_t)1 << 31) - 256) return false;
    if (!aligned_to(q, 16)) return false;
    return encode_tiled_fn() != nullptr;
}

size_t tc_workspace_bytes(int64_t M, int64_t K) { return (size_t)M * (size_t)K * 2; }

int tc_device_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) (void)cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    return v;
}

// x: [M,K] fp16/bf16/fp32 (non-fp16 is cast into `workspace`, M*K*2 bytes, 16-byte aligned).
int qmatmul_tc(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
               const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype, int bits,
               int g, void *workspace, cudaStream_t st) {
    const __half *xh = reinterpret_cast<const __half *>(x);
    if (x_dtype != BW_F16 || !aligned_to(x, 16)) {
        if (!workspace || !aligned_to(workspace, 16)) return BW_ERR_WORKSPACE;
        __half *y = reinterpret_cast<__half *>(workspace);
        const int64_t n = M * K;
        const unsigned blocks = (unsigned)((n / 8 + 255) / 256 + 1);
        switch (x_dtype) {
            case BW_F16: cast_to_f16_kernel<__half><<<blocks, 256, 0, st>>>((const __half *)x, y, n); break;
            case BW_BF16: cast_to_f16_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16 *)x, y, n); break;
            default: cast_to_f16_kernel<float><<<blocks, 256, 0, st>>>((const float *)x, y, n); break;
        }
        int rc = check_launch("cast_to_f16_kernel");
        if (rc != BW_OK) return rc;
        xh = y;
    }
    TcParams p = {};
    p.q = q; p.scale = scale; p.zp = zp; p.bias = bias; p.out = out;
    p.M = M; p.N = N; p.K = K; p.out_dtype = out_dtype;
    int gs = 0;
    while ((1 << gs) < g) ++gs;
    p.g_shift = gs;
    p.G = (int)(K / g);
    p.words_per_row = (int)(K / (32 / bits));
    p.k_stages = (int)((K + TC_BK - 1) / TC_BK);
    p.bn = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : 32));

    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};                 // bytes between token rows
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)p.bn};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xh), dims,
                                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return BW_ERR_UNSUPPORTED;
    set_last_kernel("qmm_tc_kernel");
    switch (bits) {
        case 2: return launch_tc<2>(map, p, st);
        case 4: return launch_tc<4>(map, p, st);
        default: return launch_tc<8>(map, p, st);
    }
}

}  // namespace bw
