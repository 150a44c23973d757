// Decode ("few tokens") quantized matmul for sm_100a: out[M,N] = x[M,K] . W[N,K]^T (+bias) for
// M <= 32, W = fp16(scale * (code - zero_point)) bit-identical to the reference's dequantized
// weights (bitween/modules.py:55-58), fp32 accumulation, fp16 output rounding and a separate
// fp16 bias add as in bitween/modules.py:97,101.  ONE kernel per call; nothing else is launched.
//
// The kernel is bound by HBM traffic and instruction issue, so it is built like this:
//   * persistent CTAs, at most one per SM, each owning a contiguous range of the
//     [N/128] x [K-tiles] grid of weight tiles (128 rows x 128 bytes of packed words).  When there
//     are fewer row blocks than SMs every row block gets the same number of CTAs; otherwise the
//     tile list is cut into equal ranges ("stream-K");
//   * warp 16 (one elected lane issues) keeps a shared-memory ring full with TMA, without multicast: per
//     tile one 128-byte-swizzled box of packed words, one box each of the rows' scales and zero
//     points (8 groups wide, so the box starts on a 16-byte boundary) and one box of the RAW
//     activations of the tile's k range; completion on mbarriers, so no thread holds a load in
//     flight.  The first two tiles' weights, scales and zero points are requested before
//     griddepcontrol.wait, the activations after it (they may come from the preceding kernel);
//   * warps 17.. (2 for up to 8 tokens, else 4) cast each tile's raw activations to fp16 (as
//     bitween/modules.py:74) into tensor-core fragment order, pairing values the way the
//     dequantizer pairs codes;
//   * warps 0..15 (8 row slices x 2 chunk parities) are the consumers: each reads its part of
//     the swizzled weight tile without bank conflicts, expands the codes with the exact
//     magic-number dequantization and feeds mma.sync.m16n8k16 with the weights as the A operand
//     (16 weight rows x 8 tokens);
//   * the last 4 warps take the finished sums of each row-block share off the consumers' hands:
//     whole row blocks are stored; the CTAs of a row block that form a thread-block cluster
//     exchange slices of their shares through distributed shared memory and each adds and
//     stores one slice (rank order); stream-K shares go to a global scratch and the last CTA
//     to arrive for a row block (a wrapping atomic counter per row block, in library-owned
//     memory) sums them in CTA order.  Outside a cluster no CTA ever waits for another.
// Every mbarrier wait is bounded; a wait that runs out records an error in g_dec_status and the
// CTA stops waiting.
#include <cuda.h>

#include <mutex>

#include "bw_common.cuh"
#include "qmm_dequant.cuh"

namespace bw {
namespace {

constexpr int DK_ROWS = 128;                       // weight rows per tile
constexpr int DK_ROW_BYTES = 128;                  // packed bytes per row per tile (one swizzle row)
constexpr int DK_WORDS = DK_ROW_BYTES / 4;         // words per row per tile
constexpr int DK_W_BYTES = DK_ROWS * DK_ROW_BYTES; // 16 KB of packed words per tile
constexpr int DK_GBOX = 8;                         // groups per row in a tile's box of scales / zero points
constexpr int DK_C_BYTES = DK_ROWS * DK_GBOX * 2;  // 2 KB per array per tile
constexpr int DK_CWARPS = 16;                      // consumer warps
constexpr int DK_HWARPS = 4;                       // hand-over warps (row-block sums -> outputs / scratch)
constexpr int DK_HTHREADS = DK_HWARPS * 32;
// converter warps (raw activations -> fp16 fragments): 2 for one token tile, 4 for more
template <int MT> struct DecWarps {
    static constexpr int X = MT == 1 ? 2 : 4;                       // converter warps
    static constexpr int HANDOVER0 = DK_CWARPS + 1 + X;             // first hand-over warp
    static constexpr int THREADS = (DK_CWARPS + 1 + X + DK_HWARPS) * 32;
};
constexpr int DK_PRODUCER = DK_CWARPS;             // warp index of the producer
constexpr int DK_CONVERTER0 = DK_CWARPS + 1;       // first converter warp
constexpr int DK_MAX_CTAS = 160;                   // upper bound of the grid (sizes the scratch)
constexpr int DK_MAX_STAGES = 12;
constexpr int DK_XBOX = 256;                       // widest TMA box of raw activations (elements)
constexpr unsigned DK_WAIT_LIMIT = 1u << 22;       // polls of >= 20 ns each
constexpr int DK_CNT_PER_WS = 4096;                // row-block counters per registered workspace
constexpr int DK_CNT_WS = 64;                      // workspaces per device that can use the kernel at a time

__device__ int g_dec_status = 0;
// Arrival counters of the row blocks.  atomicInc wraps them back to 0 when the last share of a
// row block arrives, so a completed call leaves them ready for the next one; they live here,
// not in the caller's scratch, because they must be zero before the first call.
__device__ unsigned g_dec_cnt[DK_CNT_WS * DK_CNT_PER_WS];

struct DecParams {
    unsigned *cnt;        // this call's slice of g_dec_cnt
    float *part;          // partial tiles [2 * cta + which][MTOK][128] fp32
    const __half *bias;
    void *out;
    int64_t M, N, K;
    int x_dtype, out_dtype;
    int g_shift;          // log2(group_size)
    int KT;               // k-tiles per row
    int RB;               // row blocks
    int tiles;            // RB * KT
    int stages;           // ring depth
    int raw_bytes;        // raw activation bytes per tile
    int cluster;          // CTAs per row block when they form a thread-block cluster (sums through DSMEM), else 1
    int cluster_leader;   // 1: the cluster's first CTA collects the shares; 0: every CTA collects one slice
};

template <int BITS> struct DecGeom {
    static constexpr int VPI = 32 / BITS;
    static constexpr int TILE_K = DK_WORDS * VPI;            // k values per tile: 128 / 256 / 512
    static constexpr int CHUNK_K = 4 * VPI;                  // k values per 16-byte chunk of a row
    static constexpr int NXC = VPI / 2;                      // 16-byte activation pieces per chunk per lane
    static constexpr int UNIT = VPI > 8 ? VPI : 8;           // k values the converter handles at a time
    static constexpr int UPCH = CHUNK_K / UNIT;              // units per chunk
    static constexpr int UPT = TILE_K / UNIT;                // units per tile
    static constexpr int BOXK = TILE_K < DK_XBOX ? TILE_K : DK_XBOX;   // k per box of raw activations
};
template <int BITS, int MT> struct DecX { static constexpr int BYTES = 2 * DecGeom<BITS>::NXC * MT * 512; };   // prepared activations per tile

// ---- PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up (recording `code`) after DK_WAIT_LIMIT polls or as soon as another
// thread of the CTA has given up; the caller carries on without waiting any more.
__device__ __forceinline__ void mbar_wait(uint64_t *bar, unsigned parity, volatile int *dead, int code) {
    if (mbar_test(bar, parity)) return;
    unsigned tries = 0;
    while (!mbar_test(bar, parity)) {
        if (*dead) return;
        __nanosleep(20);
        if (++tries > DK_WAIT_LIMIT) {
            *dead = code;
            atomicExch(&g_dec_status, code);
            return;
        }
    }
}
// The producer warp calls these two with all lanes and warp-uniform arguments; one elected lane
// issues (a single divergent lane pays for moving every operand into uniform registers).
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "{\n .reg .pred q;\n elect.sync _|q, 0xffffffff;\n"
        " @q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n}"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_elect(uint64_t *bar, unsigned bytes) {
    asm volatile(
        "{\n .reg .pred q;\n elect.sync _|q, 0xffffffff;\n"
        " @q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n}" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// ---- thread-block cluster helpers (row-block shares summed through distributed shared memory) ----
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t remote_smem(const void *local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ void remote_store4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void remote_arrive_release(uint32_t bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ bool mbar_test_cluster(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void handover_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DK_HTHREADS) : "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- activation tiles: raw [token][k] -> fp16 in fragment order ----------------------------
// Two adjacent activations -> packed fp16 pair (round to nearest even, as a torch .to(float16)).
template <typename XT> __device__ __forceinline__ uint32_t x_pair_to_h2(const XT *v);
template <> __device__ __forceinline__ uint32_t x_pair_to_h2<__half>(const __half *v) { return *reinterpret_cast<const uint32_t *>(v); }
template <> __device__ __forceinline__ uint32_t x_pair_to_h2<__nv_bfloat16>(const __nv_bfloat16 *v) {
    const uint32_t u = *reinterpret_cast<const uint32_t *>(v);           // bf16 -> fp32 is a 16-bit shift
    return h2_as_u32(__floats2half2_rn(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u)));
}
template <> __device__ __forceinline__ uint32_t x_pair_to_h2<float>(const float *v) { return h2_as_u32(__floats2half2_rn(v[0], v[1])); }

// The converter threads convert one tile together: each takes units of UNIT consecutive k of one
// token slot, casts them to fp16, pairs the values the way the dequantizer pairs codes (c_j with
// c_{j+vpi/2}) and stores them where the consuming lane reads them with one 16-byte load:
//   xs[(block*MT + m/8)*32 + (((m%8)*4 + t) ^ (block & 7))],  block = parity*NXC + piece, chunk = 2*t + parity
// (the XOR spreads the stores of a quarter warp, which differ in block, over the banks; a
// consuming warp still reads 32 distinct 16-byte slots).
// The raw tile is [box][token slot][BOXK] as the TMA boxes arrive (token slots past M and k past
// K are zeros there).
template <int BITS, int MT, typename XT>
__device__ __forceinline__ void convert_tile(const unsigned char *raw, uint4 *xs, int xtid) {
    using Geo = DecGeom<BITS>;
    constexpr int UNIT = Geo::UNIT, MTOK = MT * 8;
    const XT *src = reinterpret_cast<const XT *>(raw);
    constexpr int XTHREADS = DecWarps<MT>::X * 32;
#pragma unroll
    for (int it = 0; it < Geo::UPT * MTOK / XTHREADS; ++it) {
        const int idx = xtid + it * XTHREADS;
        const int m = idx / Geo::UPT, ud = idx % Geo::UPT;
        const int k = ud * UNIT;
        const XT *u = src + ((k / Geo::BOXK) * MTOK + m) * Geo::BOXK + (k % Geo::BOXK);
        alignas(16) XT tmp[UNIT];
#pragma unroll
        for (int j = 0; j < (int)(UNIT * sizeof(XT) / 16); ++j)
            reinterpret_cast<uint4 *>(tmp)[j] = reinterpret_cast<const uint4 *>(u)[j];
        uint32_t r[UNIT / 2];
#pragma unroll
        for (int e = 0; e < UNIT / 2; ++e)
            r[e] = x_pair_to_h2<XT>(tmp + 2 * e);
        const int c = ud / Geo::UPCH, sub = ud % Geo::UPCH;
        const int t = c >> 1, par = c & 1;
        const int piece0 = (BITS == 2) ? 2 * sub : sub;
        const int blk = par * Geo::NXC + piece0, pos = (m & 7) * 4 + t;
        uint4 *dst = xs + (blk * MT + (m >> 3)) * 32;
        if constexpr (BITS == 4) {
            dst[pos ^ (blk & 7)] = make_uint4(pair_lo(r[0], r[2]), pair_hi(r[0], r[2]), pair_lo(r[1], r[3]), pair_hi(r[1], r[3]));
        } else if constexpr (BITS == 8) {
            dst[pos ^ (blk & 7)] = make_uint4(pair_lo(r[0], r[1]), pair_hi(r[0], r[1]), pair_lo(r[2], r[3]), pair_hi(r[2], r[3]));
        } else {
            dst[pos ^ (blk & 7)] = make_uint4(pair_lo(r[0], r[4]), pair_hi(r[0], r[4]), pair_lo(r[1], r[5]), pair_hi(r[1], r[5]));
            dst[MT * 32 + (pos ^ ((blk + 1) & 7))] = make_uint4(pair_lo(r[2], r[6]), pair_hi(r[2], r[6]), pair_lo(r[3], r[7]), pair_hi(r[3], r[7]));
        }
    }
}

// ---- the streaming kernel --------------------------------------------------------------------
// Tiles are numbered tile = row_block * KT + k_tile; CTA c owns tiles [c*T/C, (c+1)*T/C).
__device__ __forceinline__ int64_t dec_first_tile(int64_t c, int64_t tiles, int64_t ctas) { return c * tiles / ctas; }
// The CTA that owns a tile: the largest c with dec_first_tile(c) <= tile.
__device__ __forceinline__ int dec_cta_of(int64_t tile, int64_t tiles, int64_t ctas) {
    return (int)(((tile + 1) * ctas - 1) / tiles);
}

// EPI: the output stage applies an activation / residual add (bw_qmatmul_fused); a separate
// instantiation, so that the plain kernel's code is not touched by it.
template <int BITS, int MT, bool EPI>
__global__ void __launch_bounds__(DecWarps<MT>::THREADS, 1)
qmm_decode_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap s_map,
                  const __grid_constant__ CUtensorMap z_map, const __grid_constant__ CUtensorMap x_map,
                  const DecParams p, const Epilogue ep) {
    using Geo = DecGeom<BITS>;
    constexpr int MTOK = MT * 8;
    constexpr int XB = DecX<BITS, MT>::BYTES;
    constexpr int NACC = MT == 1 ? 2 : 1;             // two accumulation chains when there is one token tile
    constexpr int RED = MTOK * DK_ROWS;               // fp32 sums of one tile of outputs
    constexpr int NRED = MT == 4 ? 1 : 2;             // hand-over buffers
    extern __shared__ unsigned char smem_dyn[];
    pdl_launch_dependents();

    const int S = p.stages;
    unsigned char *base = smem_dyn + ((1024u - (smem_addr(smem_dyn) & 1023u)) & 1023u);   // swizzled tiles: 1024-byte aligned
    unsigned char *wst = base;                                       // [S][16 KB] packed words
    unsigned char *cst = wst + (size_t)S * DK_W_BYTES;               // [S][scale box 2 KB | zero-point box 2 KB]
    unsigned char *xst = cst + (size_t)S * 2 * DK_C_BYTES;           // [S][XB] activations in fragment order
    unsigned char *rst = xst + (size_t)S * XB;                       // [S][raw_bytes] raw activations
    float *red = reinterpret_cast<float *>(rst + (size_t)S * p.raw_bytes);   // [NRED buffers][2 parities][MTOK][128]
    uint64_t *full = reinterpret_cast<uint64_t *>(red + NRED * 2 * RED);
    uint64_t *empty = full + DK_MAX_STAGES;
    uint64_t *xdone = empty + DK_MAX_STAGES;                          // [S] activations of the stage are converted
    uint64_t *cdone = xdone + DK_MAX_STAGES;                          // [1] the peers' shares of this CTA's slice have arrived
    uint64_t *red_full = cdone + 1;                     // [2] consumers -> hand-over warps
    uint64_t *red_free = red_full + 2;                               // [2] hand-over warps -> consumers
    volatile int *flags = reinterpret_cast<volatile int *>(red_free + 2);   // [0] a wait ran out, [1] last arriver, [2] c_lo, [3] nc
    int *slots = const_cast<int *>(flags) + 4;                       // [DK_MAX_CTAS] scratch slots of one row block's shares
    float4 *cpart = reinterpret_cast<float4 *>(                      // [cluster ranks][slice] the peers' shares of this CTA's slice of the outputs
        (reinterpret_cast<uintptr_t>(slots + DK_MAX_CTAS) + 15) & ~(uintptr_t)15);
    volatile int *dead = flags;
    const unsigned stage_tx = DK_W_BYTES + 2 * DK_C_BYTES + (unsigned)p.raw_bytes;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t ctas = gridDim.x;
    const int64_t t0 = dec_first_tile(blockIdx.x, p.tiles, ctas);
    const int nt = (int)(dec_first_tile(blockIdx.x + 1, p.tiles, ctas) - t0);
    const int rb0 = (int)(t0 / p.KT), kt0 = (int)(t0 % p.KT);

    if (threadIdx.x < S) {                       // one thread per stage initialises its barriers
        mbar_init(full + threadIdx.x, 1);
        mbar_init(empty + threadIdx.x, DK_CWARPS);
        mbar_init(xdone + threadIdx.x, DecWarps<MT>::X);
    }
    if (threadIdx.x == 32) {
        for (int b = 0; b < 2; ++b) { mbar_init(red_full + b, DK_CWARPS); mbar_init(red_free + b, 1); }
        mbar_init(cdone, (unsigned)(p.cluster > 1 ? (p.cluster - 1) * DK_HWARPS : 1));   // one arrival per peer hand-over warp
        flags[0] = 0;
    }
    if (threadIdx.x < S || threadIdx.x == 32) {
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Every CTA's barriers must exist before a peer arrives on them: all threads arrive on the cluster
    // barrier here; only the hand-over warps, the only ones that touch a peer, wait for it (later).
    if (p.cluster > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    if (warp == DK_PRODUCER) {
        // ---- producer: the warp runs the loop, one elected lane issues each copy ----
        {
            if (lane == 0) {
                asm volatile("prefetch.tensormap [%0];" ::"l"(&w_map) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"(&s_map) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"(&z_map) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"(&x_map) : "memory");
            }
            __syncwarp();
            auto load_weights = [&](int s, int rb, int kt) {
                mbar_expect_tx_elect(full + s, stage_tx);
                tma_load_2d(wst + (size_t)s * DK_W_BYTES, &w_map, kt * DK_WORDS, rb * DK_ROWS, full + s);
                const int grp0 = ((kt * Geo::TILE_K) >> p.g_shift) & ~(DK_GBOX - 1);   // TMA boxes start on 16-byte boundaries
                tma_load_2d(cst + (size_t)s * 2 * DK_C_BYTES, &s_map, grp0, rb * DK_ROWS, full + s);
                tma_load_2d(cst + (size_t)s * 2 * DK_C_BYTES + DK_C_BYTES, &z_map, grp0, rb * DK_ROWS, full + s);
            };
            auto load_x = [&](int s, int kt) {
                unsigned char *dst = rst + (size_t)s * p.raw_bytes;
#pragma unroll
                for (int b = 0; b < Geo::TILE_K / Geo::BOXK; ++b)
                    tma_load_2d(dst + (size_t)b * (p.raw_bytes / (Geo::TILE_K / Geo::BOXK)), &x_map,
                                kt * Geo::TILE_K + b * Geo::BOXK, 0, full + s);
            };
            const int npro = nt < S ? nt : S;
            const int early = npro < 2 ? npro : 2;
            int rb = rb0, kt = kt0;
            // Weights, scales and zero points do not depend on the preceding kernel: the first two
            // tiles are requested before waiting for it.  (Not more: the activations can only be
            // requested after the wait and would queue behind megabytes of weight traffic.)
            for (int i = 0; i < early; ++i) {
                load_weights(i, rb, kt);
                if (++kt == p.KT) { kt = 0; ++rb; }
            }
            pdl_wait();   // the activations may be written by the preceding kernel
            int kx = kt0;
            for (int i = 0; i < early; ++i) {
                load_x(i, kx);
                if (++kx == p.KT) kx = 0;
            }
            for (int i = early; i < npro; ++i) {
                load_weights(i, rb, kt);
                load_x(i, kt);
                if (++kt == p.KT) { kt = 0; ++rb; }
            }
            int s = 0;
            unsigned ph = 0;
            for (int i = npro; i < nt; ++i) {
                mbar_wait(empty + s, ph, dead, 1);
                load_weights(s, rb, kt);
                load_x(s, kt);
                if (++kt == p.KT) { kt = 0; ++rb; }
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp >= DK_CONVERTER0 && warp < DecWarps<MT>::HANDOVER0) {
        // ---- converters: each tile's raw activations -> fp16 fragments, ahead of the consumers ----
        const int xtid = threadIdx.x - DK_CONVERTER0 * 32;
        int s = 0;
        unsigned ph = 0;
        for (int i = 0; i < nt; ++i) {
            mbar_wait(full + s, ph, dead, 5);
            const unsigned char *raw = rst + (size_t)s * p.raw_bytes;
            uint4 *xw = reinterpret_cast<uint4 *>(xst + (size_t)s * XB);
            if (p.x_dtype == BW_F16) convert_tile<BITS, MT, __half>(raw, xw, xtid);
            else if (p.x_dtype == BW_BF16) convert_tile<BITS, MT, __nv_bfloat16>(raw, xw, xtid);
            else convert_tile<BITS, MT, float>(raw, xw, xtid);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // reads of the raw tile before its refill by TMA
            __syncwarp();
            if (lane == 0) mbar_arrive(xdone + s);
            if (++s == S) { s = 0; ph ^= 1u; }
        }
    } else if (warp >= DecWarps<MT>::HANDOVER0) {
        // ---- hand-over warps: take the finished sums of each row-block share off the consumers'
        // hands: whole row blocks are stored, shares go to the scratch and the last CTA to
        // arrive for a row block sums them in CTA order ----
        auto store_out = [&](int64_t m, int64_t n, float v) {
            if constexpr (EPI) {
                store_output(p.out, p.out_dtype, m * p.N + n, v, p.bias != nullptr, p.bias ? p.bias[n] : __half(), ep);
            } else if (p.out_dtype == BW_F16) {
                __half c = __float2half_rn(v);                       // the GEMM's fp16 output rounding
                if (p.bias) c = __hadd(c, p.bias[n]);                // separate fp16 bias add
                reinterpret_cast<__half *>(p.out)[m * p.N + n] = c;
            } else {
                if (p.bias) v += __half2float(p.bias[n]);
                if (p.out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[m * p.N + n] = __float2bfloat16_rn(v);
                else reinterpret_cast<float *>(p.out)[m * p.N + n] = v;
            }
        };
        pdl_wait();   // outputs, scratch and counters may still be in use by the preceding kernel
        if (p.cluster > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // the peers' barriers are initialised
        const int htid = threadIdx.x - DecWarps<MT>::HANDOVER0 * 32;          // 0..DK_HTHREADS-1
        constexpr int V4 = RED / 4 / DK_HTHREADS;                      // float4 per thread: 2 / 4 / 8
        int rb = rb0, kt = kt0, f = 0;
        for (int i = 0; i < nt; ++f) {
            const int len = min(p.KT - kt, nt - i);
            const bool whole = (kt == 0) && (len == p.KT);
            const int b = f % NRED, use = f / NRED;
            const float4 *r0 = reinterpret_cast<const float4 *>(red + (size_t)b * 2 * RED), *r1 = r0 + RED / 4;
            const int64_t nbase = (int64_t)rb * DK_ROWS;
            mbar_wait(red_full + b, (unsigned)use & 1u, dead, 3);
            float4 v[V4];
#pragma unroll
            for (int j = 0; j < V4; ++j) {
                const float4 a = r0[htid + j * DK_HTHREADS], c = r1[htid + j * DK_HTHREADS];
                v[j] = make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w);
            }
            handover_sync();
            if (htid == 0) mbar_arrive(red_free + b);           // the consumers may refill this buffer
            auto store_f4 = [&](int idx, float4 val) {           // idx: float4 index into the [MTOK][128] tile
                const int e = idx * 4;
                const int m = e / DK_ROWS, r = e % DK_ROWS;
                if constexpr (EPI) {
                    if (ep.act == BW_ACT_SILU_MUL) {
                        // rows come in (gate, up) pairs: two outputs of the [M, N/2] result per float4
                        if (m < p.M) {
                            const int64_t n = nbase + r, half_n = p.N >> 1;
                            if (n + 1 < p.N)
                                store_output_silu_mul(p.out, p.out_dtype, m * half_n + (n >> 1), val.x, val.y, p.bias != nullptr,
                                                      p.bias ? p.bias[n] : __half(), p.bias ? p.bias[n + 1] : __half(), ep);
                            if (n + 3 < p.N)
                                store_output_silu_mul(p.out, p.out_dtype, m * half_n + (n >> 1) + 1, val.z, val.w, p.bias != nullptr,
                                                      p.bias ? p.bias[n + 2] : __half(), p.bias ? p.bias[n + 3] : __half(), ep);
                        }
                        return;
                    }
                }
                if (m < p.M) {
                    if (nbase + r + 0 < p.N) store_out(m, nbase + r + 0, val.x);
                    if (nbase + r + 1 < p.N) store_out(m, nbase + r + 1, val.y);
                    if (nbase + r + 2 < p.N) store_out(m, nbase + r + 2, val.z);
                    if (nbase + r + 3 < p.N) store_out(m, nbase + r + 3, val.w);
                }
            };
            auto store4 = [&](int j) { store_f4(htid + j * DK_HTHREADS, v[j]); };
            if (p.cluster > 1 && p.cluster_leader) {
                // This CTA's only share of its row block.  Small shares go to the cluster's first
                // CTA through distributed shared memory; it adds them in rank order and stores,
                // while the other CTAs are already gone.
                const uint32_t rank = cluster_rank();
                if (rank != 0) {
                    const uint32_t dst = remote_smem(cpart + (size_t)(rank - 1) * (RED / 4), 0);
#pragma unroll
                    for (int j = 0; j < V4; ++j) remote_store4(dst + (uint32_t)(htid + j * DK_HTHREADS) * 16u, v[j]);
                    __syncwarp();                                    // the lanes' stores are ordered before lane 0's arrival
                    if ((htid & 31) == 0) remote_arrive_release(remote_smem(cdone, 0));
                } else {
                    unsigned tries = 0;
                    while (!mbar_test_cluster(cdone, 0u)) {
                        if (*dead) break;
                        __nanosleep(20);
                        if (++tries > DK_WAIT_LIMIT) { *dead = 7; atomicExch(&g_dec_status, 7); break; }
                    }
                    for (int r = 0; r < p.cluster - 1; ++r) {
#pragma unroll
                        for (int j = 0; j < V4; ++j) {
                            const float4 a = cpart[(size_t)r * (RED / 4) + htid + j * DK_HTHREADS];
                            v[j].x += a.x; v[j].y += a.y; v[j].z += a.z; v[j].w += a.w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < V4; ++j) store4(j);
                }
            } else if (p.cluster > 1) {
                // Large shares: the cluster's CTAs split the block's outputs into equal slices: every CTA sends slice d of its sums to CTA d through
                // distributed shared memory, and CTA d adds the shares in rank order and stores.
                const uint32_t rank = cluster_rank(), nranks = (uint32_t)p.cluster;
                const int SL = RED / 4 / p.cluster;                  // float4 per slice
#pragma unroll
                for (int j = 0; j < V4; ++j) {
                    const int idx = htid + j * DK_HTHREADS;
                    const uint32_t d = (uint32_t)(idx / SL);
                    float4 *slot = cpart + (size_t)rank * SL + (idx - (int)d * SL);
                    if (d == rank) *slot = v[j];
                    else remote_store4(remote_smem(slot, d), v[j]);
                }
                __syncwarp();                                        // the lanes' stores are ordered before lane 0's arrivals
                if ((htid & 31) == 0) {
                    for (uint32_t d = 0; d < nranks; ++d)
                        if (d != rank) remote_arrive_release(remote_smem(cdone, d));
                }
                handover_sync();                                     // this CTA's own slice is in place
                unsigned tries = 0;
                while (!mbar_test_cluster(cdone, 0u)) {
                    if (*dead) break;
                    __nanosleep(20);
                    if (++tries > DK_WAIT_LIMIT) { *dead = 7; atomicExch(&g_dec_status, 7); break; }
                }
                for (int o = htid; o < SL; o += DK_HTHREADS) {
                    float4 a = cpart[o];
                    for (uint32_t r = 1; r < nranks; ++r) {
                        const float4 c = cpart[(size_t)r * SL + o];
                        a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
                    }
                    store_f4((int)rank * SL + o, a);
                }
            } else if (whole) {
#pragma unroll
                for (int j = 0; j < V4; ++j) store4(j);
            } else {
                float4 *mine = reinterpret_cast<float4 *>(p.part + ((size_t)2 * blockIdx.x + (rb != rb0 ? 1 : 0)) * RED);
#pragma unroll
                for (int j = 0; j < V4; ++j) __stcg(mine + htid + j * DK_HTHREADS, v[j]);
                __threadfence();
                handover_sync();
                if (htid == 0) {
                    const int c_lo = dec_cta_of((int64_t)rb * p.KT, p.tiles, ctas);
                    const int nc = dec_cta_of((int64_t)rb * p.KT + p.KT - 1, p.tiles, ctas) - c_lo + 1;
                    flags[1] = (atomicInc(reinterpret_cast<unsigned *>(p.cnt) + rb, (unsigned)(nc - 1)) == (unsigned)(nc - 1)) ? 1 : 0;   // wraps to 0: ready for the next call
                    flags[2] = c_lo;
                    flags[3] = nc;
                }
                handover_sync();
                if (flags[1]) {
                    // last CTA to arrive for this row block: sum the shares in CTA order
                    __threadfence();
                    const int c_lo = flags[2], nc = flags[3];
                    for (int j = htid; j < nc; j += DK_HTHREADS) {
                        const int first_rb = (int)(dec_first_tile(c_lo + j, p.tiles, ctas) / p.KT);
                        slots[j] = 2 * (c_lo + j) + (rb != first_rb ? 1 : 0);
                    }
                    handover_sync();
#pragma unroll
                    for (int j = 0; j < V4; ++j) v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
                    for (int c = 0; c < nc; ++c) {
                        const float4 *src = reinterpret_cast<const float4 *>(p.part + (size_t)slots[c] * RED);
#pragma unroll
                        for (int j = 0; j < V4; ++j) {
                            const float4 a = __ldcg(src + htid + j * DK_HTHREADS);
                            v[j].x += a.x; v[j].y += a.y; v[j].z += a.z; v[j].w += a.w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < V4; ++j) store4(j);
                }
                handover_sync();                                 // flags and slots may be reused
            }
            i += len; kt = 0; ++rb;
        }
    } else {
        // ---- consumers ----
        const int wr = warp & 7, par = warp >> 3;           // row slice, chunk parity
        const int g = lane >> 2, t = lane & 3;
        const int chunk = 2 * t + par;                      // 16-byte chunk of the 128-byte row this lane expands
        const uint32_t w_off = (uint32_t)(wr * 16 + g) * DK_ROW_BYTES + (uint32_t)((chunk ^ g) << 4);
        const int x_blk0 = par * Geo::NXC;                  // first activation block of this warp's chunk parity
        const int row_a = wr * 16 + g;

        // this lane's group inside the tile's box of scales / zero points (row pitch 16 bytes)
        const int goff = (4 * chunk * Geo::VPI) >> p.g_shift;
        const uint32_t c_off = (uint32_t)row_a * (DK_GBOX * 2) + (uint32_t)goff * 2;
        auto make_const = [&](const unsigned char *cbox) {   // {scale, scale} and {1024 + zp, 1024 + zp}
            GroupConst c;
            const uint32_t sr = *reinterpret_cast<const unsigned short *>(cbox);
            const uint32_t zr = *reinterpret_cast<const unsigned short *>(cbox + DK_C_BYTES);
            c.s2 = __byte_perm(sr, sr, 0x1010);
            c.z1024 = h2_as_u32(__hadd2(u32_as_h2(__byte_perm(zr, zr, 0x1010)), __float2half2_rn(1024.0f)));
            return c;
        };

        float acc[NACC][MT][4];
#pragma unroll
        for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[a][mt][e] = 0.0f;

        int kt = kt0, f = 0;
        int s = 0;
        unsigned ph = 0;

        for (int i = 0; i < nt; ++i) {
            mbar_wait(full + s, ph, dead, 2);               // packed words, scales, zero points
            mbar_wait(xdone + s, ph, dead, 6);              // activations converted
            Dequant<BITS> dqa, dqb;
            {
                const int gtile = ((kt * Geo::TILE_K) >> p.g_shift) & (DK_GBOX - 1);   // the tile's first group inside its box
                const unsigned char *cb = cst + (size_t)s * 2 * DK_C_BYTES + c_off + gtile * 2;
                dqa.set(make_const(cb));
                dqb.set(make_const(cb + 8 * DK_GBOX * 2));
            }
            const unsigned char *wt = wst + (size_t)s * DK_W_BYTES + w_off;
            const uint4 wa = *reinterpret_cast<const uint4 *>(wt);
            const uint4 wb = *reinterpret_cast<const uint4 *>(wt + 8 * DK_ROW_BYTES);
            const uint4 *xs = reinterpret_cast<const uint4 *>(xst + (size_t)s * XB);
            auto x_at = [&](int piece, int mt) { const int blk = x_blk0 + piece; return xs[(blk * MT + mt) * 32 + (lane ^ (blk & 7))]; };
            uint4 xq8[MT];
            (void)xq8;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t wwa = (&wa.x)[wi], wwb = (&wb.x)[wi];
                if constexpr (BITS == 4) {
                    uint4 xf[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) xf[mt] = x_at(wi, mt);
                    uint32_t pa[4], pb[4];
                    dqa.run(wwa, pa);
                    dqb.run(wwb, pb);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_16816(acc[0][mt], pa[0], pb[0], pa[1], pb[1], xf[mt].x, xf[mt].y);
                        mma_16816(acc[NACC - 1][mt], pa[2], pb[2], pa[3], pb[3], xf[mt].z, xf[mt].w);
                    }
                } else if constexpr (BITS == 8) {
                    if ((wi & 1) == 0) {
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) xq8[mt] = x_at(wi >> 1, mt);
                    }
                    uint32_t pa[2], pb[2];
                    dqa.run(wwa, pa);
                    dqb.run(wwb, pb);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        if (wi & 1) mma_16816(acc[NACC - 1][mt], pa[0], pb[0], pa[1], pb[1], xq8[mt].z, xq8[mt].w);
                        else mma_16816(acc[0][mt], pa[0], pb[0], pa[1], pb[1], xq8[mt].x, xq8[mt].y);
                    }
                } else {
                    uint4 xf0[MT], xf1[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        xf0[mt] = x_at(2 * wi, mt);
                        xf1[mt] = x_at(2 * wi + 1, mt);
                    }
                    uint32_t pa[8], pb[8];
                    dqa.run(wwa, pa);
                    dqb.run(wwb, pb);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_16816(acc[0][mt], pa[0], pb[0], pa[1], pb[1], xf0[mt].x, xf0[mt].y);
                        mma_16816(acc[NACC - 1][mt], pa[2], pb[2], pa[3], pb[3], xf0[mt].z, xf0[mt].w);
                        mma_16816(acc[0][mt], pa[4], pb[4], pa[5], pb[5], xf1[mt].x, xf1[mt].y);
                        mma_16816(acc[NACC - 1][mt], pa[6], pb[6], pa[7], pb[7], xf1[mt].z, xf1[mt].w);
                    }
                }
            }
            // generic-proxy reads of the stage are ordered before the TMA write that refills it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);          // this warp is done with the stage
            if (++s == S) { s = 0; ph ^= 1u; }

            if (kt == p.KT - 1 || i == nt - 1) {
                // ---- end of this CTA's share of a row block: leave the sums to the hand-over warp ----
                const int b = f % NRED, use = f / NRED;
                mbar_wait(red_free + b, ((unsigned)use & 1u) ^ 1u, dead, 4);   // passes at once the first time round
                float *r = red + ((size_t)b * 2 + par) * RED + row_a;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        r[(mt * 8 + 2 * t + (e & 1)) * DK_ROWS + (e >> 1) * 8] = acc[0][mt][e] + (NACC > 1 ? acc[NACC - 1][mt][e] : 0.0f);
                        acc[0][mt][e] = 0.0f;
                        acc[NACC - 1][mt][e] = 0.0f;
                    }
                __syncwarp();
                if (lane == 0) mbar_arrive(red_full + b);
                ++f;
                kt = 0;
            } else {
                ++kt;
            }
        }
    }
    // A CTA that gave up on a wait may still have copies in flight, and -- in a cluster -- peers
    // that have not reached their hand-over yet would store into its shared memory: it lingers for
    // longer than any peer can spend in its own bounded waits (each gives up after DK_WAIT_LIMIT
    // polls, ~0.1 s) before its shared memory is handed to another CTA.  (A closing cluster
    // barrier would make this airtight, but costs every healthy launch of the small shapes
    // 0.4-0.6 us: the CTAs that have delivered their shares would wait for the one that stores.)
    if (*dead) {
        for (int i = 0; i < (p.cluster > 1 ? 400000 : 2000); ++i) __nanosleep(1000);
    }
}

// ---- host side ---------------------------------------------------------------------------------
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

int encode_2d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t inner, uint64_t outer,
              uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_tiled_fn()(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BW_OK : BW_ERR_UNSUPPORTED;
}

struct DecTuning { int enabled, smem_kb, max_ctas, pdl; };
DecTuning g_dec = {1, 0, 0, 1};

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

}  // namespace

// The slice of g_dec_cnt that calls with this workspace use.  Calls that may overlap on the GPU
// already need distinct workspaces, so they also get distinct counters.  Slices are handed out
// per workspace address; when all are taken the least recently used one is reassigned (a call
// leaves its counters at zero, so a slice can change hands as long as no kernel of its previous
// owner is still running -- that would take more than DK_CNT_WS workspaces with work in flight
// on one device at a time).
unsigned *counter_slice(const void *workspace) {
    static std::mutex mu;
    static const void *owner[64][DK_CNT_WS] = {};
    static unsigned long long used[64][DK_CNT_WS] = {};
    static unsigned long long tick = 0;
    static unsigned *base[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!base[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dec_cnt) != cudaSuccess) return nullptr;
        base[dev] = reinterpret_cast<unsigned *>(p);
    }
    int pick = -1;
    for (int i = 0; i < DK_CNT_WS; ++i) {
        if (owner[dev][i] == workspace) { pick = i; break; }
        if (!owner[dev][i]) { pick = i; break; }
    }
    if (pick < 0) {
        pick = 0;
        for (int i = 1; i < DK_CNT_WS; ++i)
            if (used[dev][i] < used[dev][pick]) pick = i;
    }
    owner[dev][pick] = workspace;
    used[dev][pick] = ++tick;
    return base[dev] + (size_t)pick * DK_CNT_PER_WS;
}

namespace {

inline int dec_token_tiles(int64_t M) { return M <= 8 ? 1 : (M <= 16 ? 2 : 4); }

template <typename Kern, typename... Args>
int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, int cluster, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (cluster > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)cluster;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (g_dec.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, args...));
    return BW_OK;
}

struct DecMaps { CUtensorMap w, s, z, x; };

template <int BITS, int MT, bool EPI>
int launch_dec(const DecMaps &maps, DecParams p, const Epilogue &ep, cudaStream_t st) {
    auto kern = qmm_decode_kernel<BITS, MT, EPI>;
    constexpr size_t XB = DecX<BITS, MT>::BYTES;
    constexpr int NRED = MT == 4 ? 1 : 2;
    const size_t stage = DK_W_BYTES + 2 * DK_C_BYTES + XB + (size_t)p.raw_bytes;

    int ctas = sm_count();
    if (ctas > DK_MAX_CTAS) ctas = DK_MAX_CTAS;
    if (g_dec.max_ctas > 0) {
        if (ctas > g_dec.max_ctas) ctas = g_dec.max_ctas;
    } else if (g_dec.max_ctas == 0 && p.RB <= ctas) {
        // no more row blocks than SMs: give each row block the same number of CTAs, 1, 2, 4 or 8,
        // launched as one thread-block cluster that adds its shares through distributed shared
        // memory (no round trips through L2)
        int per_rb = 1;
        while (per_rb * 2 <= 8 && p.RB * per_rb * 2 <= ctas && per_rb * 2 <= p.KT) per_rb *= 2;
        ctas = p.RB * per_rb;
        p.cluster = per_rb;
        p.cluster_leader = (size_t)(per_rb - 1) * MT * 8 * DK_ROWS * 4 <= 32 * 1024 ? 1 : 0;
    }
    if (ctas > p.tiles) ctas = p.tiles;
    // the first CTA's buffer for the other CTAs' shares, or one [MTOK][128] tile (ranks x slices)
    const size_t cpart_bytes = p.cluster > 1 ? (size_t)(p.cluster_leader ? p.cluster - 1 : 1) * MT * 8 * DK_ROWS * 4 : 0;
    const size_t fixed = 1024 /*alignment slack*/ + (size_t)NRED * 2 * MT * 8 * DK_ROWS * 4 + (3 * DK_MAX_STAGES + 5) * 8 +
                         16 + DK_MAX_CTAS * 4 + cpart_bytes + 64;
    const size_t budget = (size_t)(g_dec.smem_kb > 0 ? g_dec.smem_kb : 224) * 1024;
    if (budget < fixed + 2 * stage) return BW_ERR_UNSUPPORTED;
    int stages = (int)((budget - fixed) / stage);
    const int per_cta = (p.tiles + ctas - 1) / ctas;
    if (stages > per_cta) stages = per_cta;           // a ring deeper than the CTA's tile count is never filled
    if (stages > DK_MAX_STAGES) stages = DK_MAX_STAGES;
    if (stages < 1) stages = 1;
    p.stages = stages;
    const size_t smem = fixed + (size_t)stages * stage;
    static size_t configured[64] = {};   // per instantiation and device; grows monotonically
    int dev = 0;
    BW_CUDA_TRY(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || smem > configured[dev])) {
        BW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    return launch_pdl(kern, dim3((unsigned)ctas), dim3(DecWarps<MT>::THREADS), smem, p.cluster, st, maps.w, maps.s, maps.z, maps.x, p, ep);
}

template <int BITS>
int launch_dec_mt(const DecMaps &maps, const DecParams &p, int mt, cudaStream_t st) {
    const Epilogue ep = current_epilogue();
    if (ep.act != BW_ACT_NONE || ep.residual) {
        switch (mt) {
            case 1: return launch_dec<BITS, 1, true>(maps, p, ep, st);
            case 2: return launch_dec<BITS, 2, true>(maps, p, ep, st);
            default: return launch_dec<BITS, 4, true>(maps, p, ep, st);
        }
    }
    switch (mt) {
        case 1: return launch_dec<BITS, 1, false>(maps, p, ep, st);
        case 2: return launch_dec<BITS, 2, false>(maps, p, ep, st);
        default: return launch_dec<BITS, 4, false>(maps, p, ep, st);
    }
}

}  // namespace

void set_decode_tuning(int enabled, int smem_kb, int max_ctas, int pdl) { g_dec = {enabled, smem_kb, max_ctas, pdl}; }

int decode_device_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_dec_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) {
        // a CTA that gave up may have left row-block counters half way: clear them all
        (void)cudaMemcpyToSymbol(g_dec_status, &zero, sizeof(int));
        void *cnt = nullptr;
        if (cudaGetSymbolAddress(&cnt, g_dec_cnt) == cudaSuccess) (void)cudaMemset(cnt, 0, sizeof(unsigned) * DK_CNT_WS * DK_CNT_PER_WS);
    }
    return v;
}

// Layout preconditions of the persistent decode kernel: at most 32 tokens, power-of-two groups
// that hold a lane's 16-byte chunk (4 words), rows of packed words, scales, zero points and
// activations that TMA can stride over (whole 16-byte units, 16-byte aligned bases).
bool decode_path_ok(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                    const void *scale, const void *zp, int bits, int g) {
    if (!g_dec.enabled) return false;
    if (bits != 2 && bits != 4 && bits != 8) return false;
    const int vpi = 32 / bits;
    if (M < 1 || M > 32 || N < 1 || K < 1) return false;
    if (g & (g - 1)) return false;
    if (g < 4 * vpi) return false;
    if (K % (4 * vpi) != 0) return false;
    if (K > (int64_t)1 << 30 || N > (int64_t)DK_CNT_PER_WS * DK_ROWS) return false;
    if ((N + DK_ROWS - 1) / DK_ROWS * ((K / vpi + DK_WORDS - 1) / DK_WORDS) > (int64_t)1 << 30) return false;
    if (!aligned_to(q, 16)) return false;
    if ((K / g) % 8 != 0 || !aligned_to(scale, 16) || !aligned_to(zp, 16)) return false;
    if (!aligned_to(x, 16) || (K * dtype_size(x_dtype)) % 16 != 0) return false;
    return encode_tiled_fn() != nullptr;
}

// Scratch: the row-block shares of the CTAs, two slots of [8*ceil(M/8)][128] fp32 per CTA.
size_t decode_workspace_bytes(int64_t M, int64_t N, int64_t K, int bits) {
    (void)N; (void)K; (void)bits;
    return (size_t)2 * DK_MAX_CTAS * dec_token_tiles(M) * 8 * DK_ROWS * sizeof(float);
}

// Returns BW_ERR_UNSUPPORTED (nothing launched) when no ring of two stages fits; the caller then uses the cluster split-K kernel.
int qmatmul_decode(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                   const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype,
                   int bits, int g, void *workspace, cudaStream_t st) {
    if (!workspace || !aligned_to(workspace, 16)) return BW_ERR_WORKSPACE;
    const int vpi = 32 / bits, mt = dec_token_tiles(M);
    const int tile_k = DK_WORDS * vpi;
    DecParams p = {};
    p.cnt = counter_slice(workspace);
    if (!p.cnt) return BW_ERR_UNSUPPORTED;
    p.part = reinterpret_cast<float *>(workspace);
    p.bias = bias; p.out = out;
    p.M = M; p.N = N; p.K = K; p.x_dtype = x_dtype; p.out_dtype = out_dtype;
    int gs = 0;
    while ((1 << gs) < g) ++gs;
    p.g_shift = gs;
    p.KT = (int)((K / vpi + DK_WORDS - 1) / DK_WORDS);
    p.RB = (int)((N + DK_ROWS - 1) / DK_ROWS);
    p.tiles = p.KT * p.RB;
    p.raw_bytes = mt * 8 * tile_k * (int)dtype_size(x_dtype);
    p.cluster = 1;

    DecMaps maps;
    // packed words [N rows][K/vpi int32]: boxes of 128 rows x 32 words, 128-byte swizzle; scales
    // and zero points [N rows][K/g fp16]: boxes of 128 rows x 8 groups; raw activations [M][K]:
    // boxes of 8*ceil(M/8) token slots x up to 256 k.  Everything outside a tensor arrives as zeros.
    int rc = encode_2d(&maps.w, CU_TENSOR_MAP_DATA_TYPE_INT32, q, (uint64_t)(K / vpi), (uint64_t)N, (uint64_t)(K / vpi) * 4,
                       DK_WORDS, DK_ROWS, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == BW_OK) rc = encode_2d(&maps.s, CU_TENSOR_MAP_DATA_TYPE_UINT16, scale, (uint64_t)(K / g), (uint64_t)N, (uint64_t)(K / g) * 2,
                                    DK_GBOX, DK_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc == BW_OK) rc = encode_2d(&maps.z, CU_TENSOR_MAP_DATA_TYPE_UINT16, zp, (uint64_t)(K / g), (uint64_t)N, (uint64_t)(K / g) * 2,
                                    DK_GBOX, DK_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc == BW_OK) rc = encode_2d(&maps.x, x_dtype == BW_F32 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, x,
                                    (uint64_t)K, (uint64_t)M, (uint64_t)K * dtype_size(x_dtype),
                                    (uint32_t)(tile_k < DK_XBOX ? tile_k : DK_XBOX), (uint32_t)(mt * 8), CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != BW_OK) return rc;
    switch (bits) {
        case 2: rc = launch_dec_mt<2>(maps, p, mt, st); break;
        case 4: rc = launch_dec_mt<4>(maps, p, mt, st); break;
        default: rc = launch_dec_mt<8>(maps, p, mt, st); break;
    }
    if (rc == BW_OK) set_last_kernel("qmm_decode_kernel");
    return rc;
}

}  // namespace bw
