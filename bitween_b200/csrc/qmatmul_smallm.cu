// Small-M ("decode") quantized matmul for sm_100a:  out[M,N] = x[M,K] . W[N,K]^T (+bias),
// W = fp16(scale * (code - zero_point)), for M <= 64 tokens per launch.
//
// Replaces, for few tokens, the three-launch forward of the reference
// (bitween/modules.py:85-101: allocate fp16 [N,K], Triton dequantize, cuBLAS matmul, bias
// add), which moves about N*K*(bits/8 + 4) bytes; this path streams the packed words once
// (N*K*bits/8 bytes) and never materialises W.
//
// Two kernels:
//   qmm_xprep_kernel   casts the activations to fp16 (bitween/modules.py:74) and writes
//                      them ONCE, already permuted into tensor-core fragment order, to a
//                      small scratch buffer (K * 8*ceil(M/8) * 2 bytes, L2 resident).
//   qmm_smallm_kernel  the streaming kernel.  "Swap-AB": the packed weight rows fill the
//                      16-row dimension of mma.sync.m16n8k16 and the 1..64 tokens are its
//                      8-wide dimension, so a 16x16 weight tile costs one tensor instruction
//                      per 8 tokens and the kernel stays HBM-bound.
//     * every warp is independent in the k loop (no block-wide barrier): each lane streams
//       16-byte vectors of packed words of rows r and r+8 into a register prefetch ring,
//       reads its B fragments as coalesced 16-byte loads from the prepared activations
//       (served by L1/L2) and keeps its rows' group constants in a warp-private slice of
//       shared memory
//     * codes become fp16 in registers by the magic-number trick (lop3/prmt into
//       1024+code, subtract 1024+zp, multiply by scale): the subtraction is exact and the
//       product is rounded once to fp16, so W is bit-identical to the reference's fp16
//       weights (bitween/modules.py:55-58)
//     * the order of the k slots inside an MMA is free as long as A and B agree; the
//       prepared activations are stored in the order the code extraction produces
//       ((c_j, c_{j+vpi/2}) pairs)
//     * split-K runs across the CTAs of a thread-block cluster; partial tiles are summed
//       through distributed shared memory (barrier.cluster: no global scratch, no flags
//       to spin on) and the owning CTA writes fp16(fp16(acc)+bias)
// Both kernels use programmatic dependent launch: they let the next kernel of the stream
// start early (griddepcontrol.launch_dependents) and wait for their own predecessor
// (griddepcontrol.wait) only right before touching data it may have produced, so that the
// weight prefetch of one layer overlaps the tail of the previous one.
#include <cooperative_groups.h>

#include "bw_common.cuh"
#include "qmm_dequant.cuh"

namespace cg = cooperative_groups;

namespace bw {
namespace {

constexpr int PF = 2;       // granularity of the activation/group-constant staging blocks
#ifndef BW_SMALLM_THREADS
#define BW_SMALLM_THREADS 1024
#endif
constexpr int STAGES = 4;   // depth of each warp's shared-memory ring of packed-word vectors

struct SmallMParams {
    const void *x;        // raw activations (general kernel only)
    const uint4 *xp;      // prepared activations [chunks_total][NX][MT][32] x 16 bytes
    const int32_t *q;
    const __half *scale;
    const __half *zp;
    const __half *bias;
    void *out;
    int64_t M, N, K;
    int x_dtype, out_dtype;
    int g_shift;          // log2(group_size)
    int G;                // groups per row
    int words_per_row;    // K / vpi
    int chunks_total;     // ceil(K / KC)
    int chunks_per_cta;   // k-chunks handled by one CTA of the split-K cluster
    int gblock;           // k-chunks whose activations and group constants are staged at once (multiple of PF)
    int splits;           // cluster size along y
    Epilogue ep;          // activation / residual add on the way out
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16-byte streaming load of packed words: read once, do not keep in L1
__device__ __forceinline__ uint4 ld_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}
// Programmatic dependent launch: no-ops when the kernel was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int BITS> struct Geometry {
    static constexpr int VPI = 32 / BITS;    // codes per word
    static constexpr int KL = 4 * VPI;       // k values per lane load (one uint4)
    static constexpr int KC = 4 * KL;        // k values per warp step (4 lanes along k)
    static constexpr int NX = KL / 8;        // 16-byte activation pieces per lane load per token tile
    static constexpr int UNIT = VPI > 8 ? VPI : 8;  // k values permuted together when preparing x
};

// ---- activation preparation ------------------------------------------------------------
template <typename XT> __device__ __forceinline__ __half x_to_half(XT v);
template <> __device__ __forceinline__ __half x_to_half<__half>(__half v) { return v; }
template <> __device__ __forceinline__ __half x_to_half<__nv_bfloat16>(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }
template <> __device__ __forceinline__ __half x_to_half<float>(float v) { return __float2half_rn(v); }

// One thread per unit of UNIT consecutive k of one token: load, cast to fp16, permute into
// the (c_j, c_{j+vpi/2}) pair order and store at the slot the consuming lane reads with one
// 16-byte load:  xp[((chunk*NX + piece)*mt + m/8)*32 + (m%8)*4 + t].
template <int BITS, typename XT>
__global__ void __launch_bounds__(256)
qmm_xprep_kernel(const XT *__restrict__ x, int64_t M, int64_t K, int mt, int chunks_total,
                 uint4 *__restrict__ xp) {
    using Geo = Geometry<BITS>;
    constexpr int UNIT = Geo::UNIT;
    constexpr int UPC = Geo::KC / UNIT;
    pdl_launch_dependents();
    const int upr = chunks_total * UPC;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= upr * mt * 8) return;
    const int m = idx / upr;
    const int u = idx - m * upr;
    const int cl = u / UPC, uc = u % UPC;
    const int64_t k = (int64_t)u * UNIT;
    pdl_wait();   // x may come from the previous kernel; xp may still be read by it
    uint32_t r[UNIT / 2];
    if (m < M && k < K) {
        alignas(16) XT tmp[UNIT];
        const uint4 *src = reinterpret_cast<const uint4 *>(x + m * K + k);
#pragma unroll
        for (int j = 0; j < (int)(UNIT * sizeof(XT) / 16); ++j) reinterpret_cast<uint4 *>(tmp)[j] = __ldg(src + j);
#pragma unroll
        for (int e = 0; e < UNIT / 2; ++e)
            r[e] = h2_as_u32(__halves2half2(x_to_half<XT>(tmp[2 * e]), x_to_half<XT>(tmp[2 * e + 1])));
    } else {
#pragma unroll
        for (int e = 0; e < UNIT / 2; ++e) r[e] = 0u;
    }
    const int tok = (m >> 3) * 32 + (m & 7) * 4;
    if constexpr (BITS == 4) {
        const int t = uc >> 2, px = uc & 3;
        xp[((cl * Geo::NX + px) * mt) * 32 + tok + t] =
            make_uint4(pair_lo(r[0], r[2]), pair_hi(r[0], r[2]), pair_lo(r[1], r[3]), pair_hi(r[1], r[3]));
    } else if constexpr (BITS == 8) {
        const int t = uc >> 1, px = uc & 1;
        xp[((cl * Geo::NX + px) * mt) * 32 + tok + t] =
            make_uint4(pair_lo(r[0], r[1]), pair_hi(r[0], r[1]), pair_lo(r[2], r[3]), pair_hi(r[2], r[3]));
    } else {
        const int t = uc >> 2, px = 2 * (uc & 3);
        xp[((cl * Geo::NX + px) * mt) * 32 + tok + t] =
            make_uint4(pair_lo(r[0], r[4]), pair_hi(r[0], r[4]), pair_lo(r[1], r[5]), pair_hi(r[1], r[5]));
        xp[((cl * Geo::NX + px + 1) * mt) * 32 + tok + t] =
            make_uint4(pair_lo(r[2], r[6]), pair_hi(r[2], r[6]), pair_lo(r[3], r[7]), pair_hi(r[3], r[7]));
    }
}

// ---- warp-private group constants ---------------------------------------------------------
// The CTA of cluster rank r owns the k-chunks r, r+S, r+2S, ... (cyclic, so that the S CTAs of
// a cluster stream S adjacent 64-byte pieces of every row at the same time and DRAM sees long
// sequential bursts).  Lane `task` < 2*R owns one (row, array) pair -- scale or zero-point of
// one of the warp's R rows -- and copies the groups that cover local chunks [i0, i0+nb).
// Table layout: gcw[((il * GPC + j) * R + r) * 2 + which], il = chunk index inside the block,
// j = group inside the chunk (GPC = groups per chunk, 1 when a group spans several chunks).
template <int R, int KC>
__device__ __forceinline__ void stage_group_consts(const SmallMParams &p, int64_t row0, int c_first, int stride,
                                                   int i0, int nb, int gpc, uint32_t *gcw, int lane) {
    for (int task = lane; task < 2 * R; task += 32) {
        const int r = task % R, which = task / R;          // which: 0 = scale, 1 = zero point
        int64_t n = row0 + r;
        if (n >= p.N) n = p.N - 1;
        const __half *src = (which ? p.zp : p.scale) + n * p.G;
        const __half2 off = which ? __float2half2_rn(1024.0f) : __float2half2_rn(0.0f);
        for (int il = 0; il < nb; ++il) {
            const int grp0 = (int)(((int64_t)(c_first + (i0 + il) * stride) * KC) >> p.g_shift);
            for (int j = 0; j < gpc; ++j) {
                const int grp = grp0 + j;
                uint32_t v = 0u;                           // groups past the end of the row
                if (grp < p.G) v = h2_as_u32(__hadd2(__half2half2(__ldg(src + grp)), off));
                gcw[((il * gpc + j) * R + r) * 2 + which] = v;
            }
        }
    }
}

template <int MT, int RT, int WARPS> struct Occupancy {
    // CTAs per SM the register allocator should leave room for: 64 registers per thread for
    // one row tile and up to 16 tokens, 128 otherwise.
    static constexpr int THREADS = (MT <= 2 && RT == 1) ? BW_SMALLM_THREADS : ((MT <= 2) ? 512 : 256);
    static constexpr int MIN_BLOCKS = THREADS / (WARPS * 32) > 0 ? THREADS / (WARPS * 32) : 1;
};

template <int BITS, int MT, int RT, int WARPS, bool TWO_GROUPS>
__global__ void __launch_bounds__(WARPS * 32, Occupancy<MT, RT, WARPS>::MIN_BLOCKS)
qmm_smallm_kernel(const SmallMParams p) {
    using Geo = Geometry<BITS>;
    constexpr int R = RT * 16;                            // rows per warp
    constexpr int ROWS = WARPS * R;
    constexpr int MTOK = MT * 8;
    constexpr int SLOTS = 2 * RT;                         // uint4 per lane per k-chunk
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_launch_dependents();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    // cyclic split-K: this CTA owns chunks c_first, c_first + stride, ...
    const int c_first = blockIdx.y, stride = p.splits;
    const int nloc = (p.chunks_total - c_first + stride - 1) / stride;
    const int gpc = max(1, Geo::KC >> p.g_shift);             // groups per chunk
    const int gcap = p.gblock * gpc;                          // table entries per row
    uint4 *xs = reinterpret_cast<uint4 *>(smem_raw) + (size_t)WARPS * STAGES * SLOTS * 32;   // [gblock][NX][MT][32]
    uint32_t *gcw = reinterpret_cast<uint32_t *>(xs + (size_t)p.gblock * Geo::NX * MT * 32) +
                    (size_t)warp * gcap * R * 2;

    // rows streamed by this lane (clamped so that loads stay in range; stores are masked)
    const uint4 *rowp[SLOTS];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int64_t n = (int64_t)n0 + warp * R + rt * 16 + h * 8 + g;
            if (n >= p.N) n = p.N - 1;
            rowp[rt * 2 + h] = reinterpret_cast<const uint4 *>(p.q + n * p.words_per_row) + t;
        }
    }
    // Warp-private shared-memory ring, STAGES k-chunks deep, filled with cp.async: each lane
    // later reads back exactly the 16-byte slots it filled itself, so the k loop needs no
    // barrier.  HBM latency under load is about 2 us; ~100 KB per SM must be in flight.
    uint4 *ring = reinterpret_cast<uint4 *>(smem_raw) + (size_t)warp * STAGES * SLOTS * 32 + lane;
    const int vec_per_row = p.words_per_row >> 2;
    // Vectors past the end of a row are clamped to its last vector: the prepared activations
    // are zero there and group constants past the row end are zero, so they contribute exactly 0.
    const int vmax = vec_per_row - 1 - t;
    auto issue = [&](int i) {   // i = local chunk index; always commits a (possibly empty) group
        if (i < nloc) {
            const int v = min((c_first + i * stride) * 4, vmax);   // uint4 index of lane column 0 in the row
#pragma unroll
            for (int s = 0; s < SLOTS; ++s)
                cp_async16(ring + ((i & (STAGES - 1)) * SLOTS + s) * 32, rowp[s] + v);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int d = 0; d < STAGES - 1; ++d) issue(d);

    float acc[RT][MT][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[rt][mt][e] = 0.0f;

    for (int xb = 0; xb < nloc; xb += p.gblock) {     // p.gblock is a multiple of PF
        const int nb = min(p.gblock, nloc - xb);
        if (xb > 0) __syncthreads();   // every warp is done with the previous block's activations
        stage_group_consts<R, Geo::KC>(p, (int64_t)n0 + warp * R, c_first, stride, xb, nb, gpc, gcw, lane);
        if (xb == 0) pdl_wait();       // the prepared activations come from the preceding kernel
        {
            constexpr int VPC = Geo::NX * MT * 32;   // 16-byte vectors of activations per chunk
            for (int i = threadIdx.x; i < nb * VPC; i += WARPS * 32) {
                const int il = i / VPC, e = i - il * VPC;
                cp_async16(xs + i, p.xp + (size_t)(c_first + (xb + il) * stride) * VPC + e);
            }
            cp_async_commit_wait_all();
            __syncthreads();
        }
        const GroupConst *gc = reinterpret_cast<const GroupConst *>(gcw);

        for (int cl = 0; cl < nb; ++cl) {
            {
            {
            const int i = xb + cl;
            issue(i + STAGES - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
            uint4 wv[SLOTS];
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) wv[s] = ring[((i & (STAGES - 1)) * SLOTS + s) * 32];

            const int kc0 = (c_first + i * stride) * Geo::KC;       // first k of the chunk
            const int kl = kc0 + t * Geo::KL;                       // first k of this lane's vectors
            const int gl0 = cl * gpc + ((kl >> p.g_shift) - (kc0 >> p.g_shift));
            const int gl1 = TWO_GROUPS ? (cl * gpc + (((kl + Geo::KL / 2) >> p.g_shift) - (kc0 >> p.g_shift))) : gl0;
            Dequant<BITS> dq[SLOTS][TWO_GROUPS ? 2 : 1];
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int r = (s >> 1) * 16 + (s & 1) * 8 + g;
                dq[s][0].set(gc[gl0 * R + r]);
                if constexpr (TWO_GROUPS) dq[s][1].set(gc[gl1 * R + r]);
            }
            const uint4 *xc = xs + (size_t)cl * Geo::NX * MT * 32 + lane;
            uint4 xq8[MT];   // 8-bit codes: one 16-byte piece feeds two consecutive words
            (void)xq8;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const int gs = TWO_GROUPS ? (wi >> 1) : 0;   // words 0,1 -> first group, 2,3 -> second
                if constexpr (BITS == 4) {
                    uint4 xf[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) xf[mt] = xc[(wi * MT + mt) * 32];
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt) {
                        uint32_t pa[4], pb[4];
                        dq[rt * 2][gs].run((&wv[rt * 2].x)[wi], pa);
                        dq[rt * 2 + 1][gs].run((&wv[rt * 2 + 1].x)[wi], pb);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_16816(acc[rt][mt], pa[0], pb[0], pa[1], pb[1], xf[mt].x, xf[mt].y);
                            mma_16816(acc[rt][mt], pa[2], pb[2], pa[3], pb[3], xf[mt].z, xf[mt].w);
                        }
                    }
                } else if constexpr (BITS == 8) {
                    // piece wi/2 holds the activations of words 2*(wi/2) and 2*(wi/2)+1
                    if ((wi & 1) == 0) {
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) xq8[mt] = xc[((wi >> 1) * MT + mt) * 32];
                    }
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt) {
                        uint32_t pa[2], pb[2];
                        dq[rt * 2][gs].run((&wv[rt * 2].x)[wi], pa);
                        dq[rt * 2 + 1][gs].run((&wv[rt * 2 + 1].x)[wi], pb);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            if (wi & 1) mma_16816(acc[rt][mt], pa[0], pb[0], pa[1], pb[1], xq8[mt].z, xq8[mt].w);
                            else mma_16816(acc[rt][mt], pa[0], pb[0], pa[1], pb[1], xq8[mt].x, xq8[mt].y);
                        }
                    }
                } else {
                    uint4 xf0[MT], xf1[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        xf0[mt] = xc[((2 * wi) * MT + mt) * 32];
                        xf1[mt] = xc[((2 * wi + 1) * MT + mt) * 32];
                    }
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt) {
                        uint32_t pa[8], pb[8];
                        dq[rt * 2][gs].run((&wv[rt * 2].x)[wi], pa);
                        dq[rt * 2 + 1][gs].run((&wv[rt * 2 + 1].x)[wi], pb);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_16816(acc[rt][mt], pa[0], pb[0], pa[1], pb[1], xf0[mt].x, xf0[mt].y);
                            mma_16816(acc[rt][mt], pa[2], pb[2], pa[3], pb[3], xf0[mt].z, xf0[mt].w);
                            mma_16816(acc[rt][mt], pa[4], pb[4], pa[5], pb[5], xf1[mt].x, xf1[mt].y);
                            mma_16816(acc[rt][mt], pa[6], pb[6], pa[7], pb[7], xf1[mt].z, xf1[mt].w);
                        }
                    }
                }
            }
            }
          }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (nloc == 0) pdl_wait();   // every CTA orders its output writes after the predecessor

    // ---- epilogue ---------------------------------------------------------------------
    auto store_out = [&](int64_t m, int64_t n, float v) {
        store_output(p.out, p.out_dtype, m * p.N + n, v, p.bias != nullptr, p.bias ? p.bias[n] : __half(), p.ep);
    };

    if (p.splits == 1) {
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int64_t n = (int64_t)n0 + warp * R + rt * 16 + (e >> 1) * 8 + g;
                    const int64_t m = mt * 8 + 2 * t + (e & 1);
                    if (n < p.N && m < p.M) store_out(m, n, acc[rt][mt][e]);
                }
        return;
    }

    // split-K: sum the cluster's partial tiles through distributed shared memory
    cg::cluster_group cluster = cg::this_cluster();
    float *red = reinterpret_cast<float *>(smem_raw);   // [MTOK][ROWS], reuses the constants area
    __syncthreads();                                    // every warp is done with its constants
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = warp * R + rt * 16 + (e >> 1) * 8 + g;
                const int m = mt * 8 + 2 * t + (e & 1);
                red[m * ROWS + r] = acc[rt][mt][e];
            }
    cluster.sync();
    {
        const int rank = (int)cluster.block_rank();
        const int nranks = (int)cluster.num_blocks();
        const int total = MTOK * ROWS;
        const int per = (total + nranks - 1) / nranks;
        const int e_end = min((rank + 1) * per, total);
        for (int e = rank * per + (int)threadIdx.x; e < e_end; e += WARPS * 32) {
            float v = 0.0f;
            for (int q = 0; q < nranks; ++q) v += cluster.map_shared_rank(red, q)[e];
            const int m = e / ROWS, r = e % ROWS;
            const int64_t n = (int64_t)n0 + r;
            if (n < p.N && m < p.M) store_out(m, n, v);
        }
    }
    cluster.sync();   // keep this CTA's shared memory alive until every peer has read it
}

// ---- general kernel: any group_size / K layout the reference accepts -------------------
// One warp per output row; lanes stride over packed words; per-element group lookup.
// Correct for every legal (bits, group_size, K); used when the streaming kernel's layout
// preconditions do not hold (group size not a power of two, K not a multiple of 4 words,
// unaligned pointers) -- still on the GPU, never a CPU path.
template <int BITS, typename XT>
__global__ void __launch_bounds__(128)
qmm_general_kernel(const SmallMParams p, int g, int64_t m0, int mcount) {
    constexpr int VPI = 32 / BITS;
    constexpr int32_t MASK = (1 << BITS) - 1;
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (n >= p.N) return;
    const XT *x = reinterpret_cast<const XT *>(p.x);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int wi = lane; wi < p.words_per_row; wi += 32) {
        const int32_t word = p.q[n * p.words_per_row + wi];
#pragma unroll
        for (int i = 0; i < VPI; ++i) {
            const int64_t k = (int64_t)wi * VPI + i;
            const int64_t gi = n * p.G + k / g;
            const float s = __half2float(p.scale[gi]);
            const float z = __half2float(p.zp[gi]);
            const float wv = __half2float(__float2half_rn(__fmul_rn(s, __fsub_rn((float)((word >> (i * BITS)) & MASK), z))));
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j < mcount) acc[j] += __half2float(x_to_half<XT>(x[(m0 + j) * p.K + k])) * wv;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
    if (lane == 0) {
        for (int j = 0; j < mcount; ++j) {
            const int64_t m = m0 + j;
            store_output(p.out, p.out_dtype, m * p.N + n, acc[j], p.bias != nullptr, p.bias ? p.bias[n] : __half(), p.ep);
        }
    }
}

static bool g_pdl = true;   // programmatic dependent launch between the library's kernels

template <typename Kern, typename... Args>
int launch_ex(Kern kern, dim3 grid, dim3 block, size_t smem, int cluster_y, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (cluster_y > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = (unsigned)cluster_y;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (g_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, args...));
    return BW_OK;
}

template <int BITS>
int launch_xprep(const SmallMParams &p, int mt, uint4 *xp, cudaStream_t st) {
    using Geo = Geometry<BITS>;
    const int64_t total = (int64_t)p.chunks_total * (Geo::KC / Geo::UNIT) * mt * 8;
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    switch (p.x_dtype) {
        case BW_F16: return launch_ex(qmm_xprep_kernel<BITS, __half>, grid, block, 0, 1, st, (const __half *)p.x, p.M, p.K, mt, p.chunks_total, xp);
        case BW_BF16: return launch_ex(qmm_xprep_kernel<BITS, __nv_bfloat16>, grid, block, 0, 1, st, (const __nv_bfloat16 *)p.x, p.M, p.K, mt, p.chunks_total, xp);
        default: return launch_ex(qmm_xprep_kernel<BITS, float>, grid, block, 0, 1, st, (const float *)p.x, p.M, p.K, mt, p.chunks_total, xp);
    }
}

template <int BITS, int MT, int RT, int WARPS, bool TWO_GROUPS>
int launch_cfg(SmallMParams p, cudaStream_t st) {
    using Geo = Geometry<BITS>;
    constexpr int R = RT * 16;
    constexpr int ROWS = WARPS * R;
    constexpr int MTOK = MT * 8;
    auto kern = qmm_smallm_kernel<BITS, MT, RT, WARPS, TWO_GROUPS>;
    // shared memory: the CTA's slice of the prepared activations + warp-private group
    // constants (the split-K reduction tile reuses the same bytes)
    const size_t red_bytes = (size_t)MTOK * ROWS * sizeof(float);
    const size_t x_per_chunk = (size_t)Geo::NX * MT * 32 * 16;
    const size_t budget = 48 * 1024;
    int gblock = (p.chunks_per_cta + PF - 1) / PF * PF;
    const int gpc = (Geo::KC >> p.g_shift) > 0 ? (Geo::KC >> p.g_shift) : 1;
    auto gc_bytes = [&](int gb) { return (size_t)WARPS * gb * gpc * R * sizeof(GroupConst); };
    while (gblock > PF && gblock * x_per_chunk + gc_bytes(gblock) > budget) gblock -= PF;
    p.gblock = gblock;
    const size_t ring_bytes = (size_t)WARPS * STAGES * 2 * RT * 32 * 16;
    size_t smem = ring_bytes + gblock * x_per_chunk + gc_bytes(gblock);
    if (p.splits > 1 && smem < red_bytes) smem = red_bytes;
    static size_t configured[64] = {};   // per instantiation and device; grows monotonically
    int dev = 0;
    BW_CUDA_TRY(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || smem > configured[dev])) {
        BW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    const dim3 grid((unsigned)((p.N + ROWS - 1) / ROWS), (unsigned)p.splits, 1);
    return launch_ex(kern, grid, dim3(WARPS * 32, 1, 1), smem, p.splits, st, p);
}

template <int BITS, int MT, bool TWO_GROUPS>
int launch_rows(const SmallMParams &p, int rt, int warps, cudaStream_t st) {
    if constexpr (TWO_GROUPS) return launch_cfg<BITS, MT, 1, 4, TWO_GROUPS>(p, st);
    else {
        if (rt == 1 && warps == 4) return launch_cfg<BITS, MT, 1, 4, TWO_GROUPS>(p, st);
        if (rt == 2 && warps == 4) return launch_cfg<BITS, MT, 2, 4, TWO_GROUPS>(p, st);
        if constexpr (MT <= 2) {
            if (rt == 2 && warps == 8) return launch_cfg<BITS, MT, 2, 8, TWO_GROUPS>(p, st);
            if (rt == 1 && warps == 8) return launch_cfg<BITS, MT, 1, 8, TWO_GROUPS>(p, st);
        }
        return launch_cfg<BITS, MT, 1, 4, TWO_GROUPS>(p, st);
    }
}

template <int BITS, bool TWO_GROUPS>
int launch_mt(const SmallMParams &p, int mt, int rt, int warps, cudaStream_t st) {
    switch (mt) {
        case 1: return launch_rows<BITS, 1, TWO_GROUPS>(p, rt, warps, st);
        case 2: return launch_rows<BITS, 2, TWO_GROUPS>(p, rt, warps, st);
        case 4: return launch_rows<BITS, 4, TWO_GROUPS>(p, rt, warps, st);
        default: return launch_rows<BITS, 8, TWO_GROUPS>(p, rt, warps, st);
    }
}

template <int BITS>
int launch_general(const SmallMParams &p, int g, cudaStream_t st) {
    const unsigned blocks = (unsigned)((p.N + 3) / 4);
    for (int64_t m0 = 0; m0 < p.M; m0 += 8) {
        const int mc = (int)((p.M - m0 < 8) ? (p.M - m0) : 8);
        switch (p.x_dtype) {
            case BW_F16: qmm_general_kernel<BITS, __half><<<blocks, 128, 0, st>>>(p, g, m0, mc); break;
            case BW_BF16: qmm_general_kernel<BITS, __nv_bfloat16><<<blocks, 128, 0, st>>>(p, g, m0, mc); break;
            default: qmm_general_kernel<BITS, float><<<blocks, 128, 0, st>>>(p, g, m0, mc); break;
        }
        int rc = check_launch("qmm_general_kernel");
        if (rc != BW_OK) return rc;
    }
    return BW_OK;
}

}  // namespace

// Tuning override for experiments: row tiles per warp, warps per CTA, split-K factor
// (0 = automatic), programmatic dependent launch on/off.  Not part of the C ABI.
struct SmallMTuning { int rt, warps, splits; };
static SmallMTuning g_tuning = {0, 0, 0};
void set_smallm_tuning(int rt, int warps, int splits) { g_tuning = {rt, warps, splits}; }
void set_smallm_pdl(int on) { g_pdl = on != 0; }

bool smallm_fast_path_ok(const void *x, int x_dtype, int64_t K, const int32_t *q, int bits, int g) {
    const int vpi = 32 / bits;
    const int kl = 4 * vpi;
    if (K == 0) return false;
    if (g & (g - 1)) return false;                      // power-of-two groups only
    if (g < kl / 2) return false;
    if (K % kl != 0) return false;                      // rows start 16-byte aligned, vectors whole
    if (K > (int64_t)1 << 30) return false;
    if (!aligned_to(q, 16)) return false;
    const int unit = vpi > 8 ? vpi : 8;
    if (!aligned_to(x, 16) || (K * dtype_size(x_dtype)) % 16 != 0 || K % unit != 0) return false;
    return true;
}

// ---- built-in scratch for bw_qmatmul_noalloc ------------------------------------------------
// Some callers may not allocate device memory at all: code running while a CUDA graph is being
// captured, real-time serving loops that forbid allocator calls after start-up, and plugins
// whose host hands them only input/output buffers.  For them the prepared-activation scratch
// lives in this fixed array instead of a caller-supplied workspace.  Every GPU that loads the
// library reserves these 2 MiB until the process exits.  All calls on a device share the
// array, so calls that overlap on the GPU (different streams) would race on it.
constexpr size_t NOALLOC_SCRATCH_BYTES = (size_t)2 << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// Device address of the built-in scratch on the CURRENT device.  In host code the array's
// name is only a handle for the runtime, not a device pointer, so the address is looked up
// with cudaGetSymbolAddress -- once per device, with that device current -- and cached.
int noalloc_scratch(void **ptr, size_t *bytes) {
    static void *cached[64] = {};
    int dev = 0;
    BW_CUDA_TRY(cudaGetDevice(&dev));
    void *p = (dev >= 0 && dev < 64) ? cached[dev] : nullptr;
    if (!p) {
        BW_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        if (dev >= 0 && dev < 64) cached[dev] = p;   // racing first calls store the same value
    }
    *ptr = p;
    *bytes = NOALLOC_SCRATCH_BYTES;
    return BW_OK;
}

// Scratch bytes the streaming kernel needs for the prepared activations of one launch.
size_t smallm_workspace_bytes(int64_t M, int64_t K, int bits) {
    const int kc = 16 * (32 / bits);
    const int64_t mtok = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    return (size_t)((K + kc - 1) / kc * kc) * mtok * 2;
}

// One launch pair (prepare + stream) for up to 64 tokens (the caller loops over token
// blocks), or the general kernel when the layout preconditions do not hold.
int qmatmul_smallm(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                   const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype,
                   int bits, int g, void *workspace, cudaStream_t st) {
    if (M == 0 || N == 0) return BW_OK;
    SmallMParams p = {};
    p.x = x; p.q = q; p.scale = scale; p.zp = zp; p.bias = bias; p.out = out;
    p.M = M; p.N = N; p.K = K; p.x_dtype = x_dtype; p.out_dtype = out_dtype;
    p.ep = current_epilogue();
    p.G = (int)(K / g);
    p.words_per_row = (int)(K / (32 / bits));
    if (!smallm_fast_path_ok(x, x_dtype, K, q, bits, g)) {
        set_last_kernel("qmm_general_kernel");
        switch (bits) {
            case 2: return launch_general<2>(p, g, st);
            case 4: return launch_general<4>(p, g, st);
            default: return launch_general<8>(p, g, st);
        }
    }
    if (M > 64) return BW_ERR_UNSUPPORTED;
    if (!workspace || !aligned_to(workspace, 16)) return BW_ERR_WORKSPACE;
    const int vpi = 32 / bits, kc = 16 * vpi;
    int gs = 0;
    while ((1 << gs) < g) ++gs;
    p.g_shift = gs;
    p.chunks_total = (int)((K + kc - 1) / kc);
    p.xp = reinterpret_cast<const uint4 *>(workspace);
    const bool two_groups = g < 4 * vpi;
    const int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));

    int rt = g_tuning.rt, warps = g_tuning.warps, splits = g_tuning.splits;
    if (rt == 0 || warps == 0) {
        rt = 1;
        warps = (mt <= 2 && N >= 8192) ? 8 : 4;
    }
    if (two_groups || mt > 2) { if (warps > 4) warps = 4; }
    if (two_groups) rt = 1;
    const int rows = rt * warps * 16;
    const int row_blocks = (int)((N + rows - 1) / rows);
    if (splits == 0) {
        // fill the CTA slots of the 148 SMs in one wave
        const int threads_per_sm = (mt <= 2) ? 1024 : 256;
        const int slots = 148 * (threads_per_sm / (warps * 32) > 0 ? threads_per_sm / (warps * 32) : 1);
        splits = slots / row_blocks;
        if (splits > 8) splits = 8;
        const int max_by_chunks = p.chunks_total / 2 > 0 ? p.chunks_total / 2 : 1;
        if (splits > max_by_chunks) splits = max_by_chunks;
        if (splits < 1) splits = 1;
    }
    if (splits > 8) splits = 8;
    p.chunks_per_cta = (p.chunks_total + splits - 1) / splits;
    p.splits = splits;
    set_last_kernel("qmm_smallm_kernel");
    int rc;
    switch (bits) {
        case 2: rc = launch_xprep<2>(p, mt, reinterpret_cast<uint4 *>(workspace), st); break;
        case 4: rc = launch_xprep<4>(p, mt, reinterpret_cast<uint4 *>(workspace), st); break;
        default: rc = launch_xprep<8>(p, mt, reinterpret_cast<uint4 *>(workspace), st); break;
    }
    if (rc != BW_OK) return rc;
    if (two_groups) {
        switch (bits) {
            case 2: rc = launch_mt<2, true>(p, mt, rt, warps, st); break;
            case 4: rc = launch_mt<4, true>(p, mt, rt, warps, st); break;
            default: rc = launch_mt<8, true>(p, mt, rt, warps, st); break;
        }
    } else {
        switch (bits) {
            case 2: rc = launch_mt<2, false>(p, mt, rt, warps, st); break;
            case 4: rc = launch_mt<4, false>(p, mt, rt, warps, st); break;
            default: rc = launch_mt<8, false>(p, mt, rt, warps, st); break;
        }
    }
    return rc;
}

}  // namespace bw
