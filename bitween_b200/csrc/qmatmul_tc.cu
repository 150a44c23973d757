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
// fp32 columns of tensor memory.  The dequantized weights (the A operand) never touch shared
// memory: each dequantization thread owns one weight row = one TMEM lane and writes its 64 fp16
// of a k-stage into 32 columns of that lane with tcgen05.st; the MMAs read A from tensor
// memory and only the activations (B) from shared memory.
//
// Warp roles in a CTA of 608 threads (one output tile of 128 weight rows x BN tokens, BN from
// 16 to 256 by token count):
//   warp 0       TMA producer (one lane) of the [BN tokens x 64 k] fp16 activation tile (128-byte
//                swizzle) of each k-stage: cp.async.bulk.tensor loads, without multicast
//   warp 18      TMA producer (one lane) of the packed-word slots [128 rows x 128 bytes] (2, 4 or
//                8 k-stages, 128-byte swizzle: whole 128-byte row segments keep the weight
//                stream's DRAM accesses efficient); the two rings are independent
//   warp 1       allocates tensor memory (accumulator + eight A stages); the whole warp runs the
//                issue loop and one elected lane issues
//                tcgen05.mma (kind::f16, A in TMEM, M=128, N=BN, K=16, four per stage) and one
//                tcgen05.commit per stage (it frees the A stage for its dequantization group
//                and the activation slot for the producer) / one for the accumulator
//   warps 2..17  four groups of 128 dequantization threads (one per weight row; group g takes
//                k-stages g, g+4, ...): fetch the row's packed words from the ring, expand them to
//                fp16 in natural k order and store them as the A operand into their TMEM lane
//                (tcgen05.st); afterwards the same warps are the epilogue:
//                tcgen05.ld of their TMEM lane quadrant, fp16 rounding + bias, coalesced stores
// Small problems split K over the CTAs of a thread-block cluster; the partial tiles are summed
// through distributed shared memory.  Stages are handed over with mbarriers; every wait is
// bounded: a wait that runs out records an error in g_tc_status, the CTA drains, frees its
// tensor memory and returns.  Ring positions and phases are tracked with counters (a division
// per stage on the single MMA-issuing thread cost 15 % of the throughput).
#include <cooperative_groups.h>
#include <cuda.h>

#include "bw_common.cuh"
#include "qmm_dequant.cuh"

namespace cgx = cooperative_groups;

namespace bw {
namespace {

constexpr int TC_BM = 128;        // weight rows per tile (MMA M)
constexpr int TC_BK = 64;         // k per stage: 64 fp16 = one 128-byte swizzle row
constexpr int TC_STAGES = 8;       // A-operand stages in tensor memory (8 x 32 columns next to a 256-column accumulator)
constexpr int TC_DQ_GROUPS = 4;   // dequantization warp groups (4 warps each) taking alternate stages
constexpr int TC_THREADS = 64 + TC_DQ_GROUPS * 128 + 32;
constexpr int TC_WPROD_WARP = TC_THREADS / 32 - 1;   // the last warp: producer of the packed-word ring
static_assert(TC_STAGES % TC_DQ_GROUPS == 0, "each dequantization group owns whole A stages (phase parity)");
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
// (Called by all lanes of the issuing warp; one elected lane issues.)
// Same MMA with the A operand (128 rows x 16 k, two fp16 per 32-bit column, one row per lane) in
// tensor memory: only the B operand is read from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n elect.sync _|q, 0xffffffff;\n"
        " @q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Each thread of the warp writes 32 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Arrives on the mbarrier once all tcgen05.mma issued so far by this warp's elected lane have
// completed (called by all lanes of the issuing warp).
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile(
        "{\n .reg .pred q;\n elect.sync _|q, 0xffffffff;\n"
        " @q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}" ::"r"(smem_addr(bar)) : "memory");
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
// Instruction descriptor for kind::f16: fp16 A (format 0), fp16 or bf16 B, fp32 accumulator
// (1), both operands K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t umma_idesc_f16(int bn, int b_is_bf16) {
    uint32_t d = 0;
    d |= 1u << 4;                                     // c_format = F32
    d |= (b_is_bf16 ? 1u : 0u) << 10;                 // b_format: 0 = F16, 1 = BF16 (A stays F16)
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
    int bn;             // tokens per tile: 16, 32, 64, 128 or 256
    int x_stages;       // depth of the TMA ring of activation tiles
    int w_stages;       // depth of the TMA ring of packed-word slots (a power of two)
    int w_stages_log2;
    int splits;         // split-K factor = cluster size along grid z
    int kper;           // k-stages per split
    int n_tiles;        // row tiles (N / 128, rounded up)
    int tiles;          // output tiles: n_tiles x token tiles
    int persistent;     // 1: grid.x CTAs walk the tile list (tile = blockIdx.x, += gridDim.x); 0: one tile per CTA
    int tma_store;      // 1: output blocks leave through a shared-memory staging tile and TMA stores
    int pdl;            // 1: launched with programmatic stream serialisation behind the kernel that casts the activations
    int x_is_bf16;      // always 0: kind::f16 MMAs take both operands in one 16-bit format
    Epilogue ep;        // activation / residual add on the way out
};

// Words of one row for one 64-k stage, as 16-byte vectors, and the natural-order expansion.
template <int BITS> struct StageGeom {
    static constexpr int VPI = 32 / BITS;             // codes per word
    static constexpr int WPS = TC_BK / VPI;           // words per row per stage: 4 / 8 / 16
    static constexpr int VPS = WPS / 4;               // 16-byte vectors per row per stage: 1 / 2 / 4
    static constexpr int SPS = 32 / WPS;              // k-stages per 128-byte row segment of a packed-word slot: 8 / 4 / 2
};

// Expands the WPS words of one stage into the row's eight 16-byte chunks (8 consecutive k each).
// ONE: the whole stage lies in one quantization group (group_size >= 64): no per-word lookup.
template <int BITS, bool ONE>
__device__ __forceinline__ void expand_stage(const uint32_t (&w)[StageGeom<BITS>::WPS], const GroupConst (&gc)[4],
                                             int kbase, int g_shift, int grp0, uint4 (&chunk)[8]) {
    constexpr int VPI = 32 / BITS;
    constexpr int WPS = StageGeom<BITS>::WPS;
    Dequant<BITS> dq;
    int cur = -1;
    if constexpr (ONE) dq.set(gc[0]);
#pragma unroll
    for (int j = 0; j < WPS; ++j) {
        if constexpr (!ONE) {
            const int gl = min(((kbase + j * VPI) >> g_shift) - grp0, 3);
            if (gl != cur) { dq.set(gc[gl]); cur = gl; }
        }
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

template <int BITS, bool PERSIST, bool TMAST>
__global__ void __launch_bounds__(TC_THREADS, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
              const __grid_constant__ CUtensorMap out_map, const TcParams p) {
    using SG = StageGeom<BITS>;
    // one slot of the packed-word ring: 128 rows x 128 bytes (SPS k-stages), 128-byte swizzle; whole
    // 128-byte row segments keep the DRAM accesses of the weight stream efficient
    constexpr int W_STAGE_BYTES = TC_BM * 128;
    extern __shared__ unsigned char tc_smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle pattern
    unsigned char *smem = tc_smem_raw + ((1024u - (smem_addr(tc_smem_raw) & 1023u)) & 1023u);
    const int bn = p.bn, NSX = p.x_stages, NSW = p.w_stages;
    unsigned char *x_tiles = smem;                                        // [NSX][bn][128 B]         activations
    unsigned char *w_tiles = x_tiles + (size_t)NSX * bn * 128;            // [NSW][128][128 B]        packed words
    // output staging of the TMA-store epilogue: per dequantization group one block [32 tokens][128 rows]
    unsigned char *o_stage = w_tiles + (size_t)NSW * W_STAGE_BYTES;
    const int o_esize = p.out_dtype == BW_F32 ? 4 : 2;
    const size_t o_bytes = TMAST ? (size_t)TC_DQ_GROUPS * 32 * TC_BM * o_esize : 0;
    uint64_t *bars = reinterpret_cast<uint64_t *>(o_stage + o_bytes);
    uint64_t *a_full = bars, *a_empty = bars + TC_STAGES, *x_full = bars + 2 * TC_STAGES;
    uint64_t *w_full = x_full + NSX, *w_empty = w_full + NSW, *acc_full = w_empty + NSW, *acc_empty = acc_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Tile schedule.  Persistent launches (no split-K) walk the list tile = mt * n_tiles + nt from
    // blockIdx.x in steps of gridDim.x: barriers, rings and tensor memory are set up once, the
    // producer runs ahead into the next tile while the current one drains, and only the epilogue
    // separates the MMAs of consecutive tiles.  Otherwise a CTA owns the tile its block index names.
    const int first_tile = PERSIST ? (int)blockIdx.x : (int)(blockIdx.y * p.n_tiles + blockIdx.x);
    const int tile_step = PERSIST ? (int)gridDim.x : p.tiles;
    // split-K over the CTAs of a cluster (grid z): this CTA owns k-stages [kt0, kt1)
    const int kt0 = blockIdx.z * p.kper;
    const int kt1 = min(kt0 + p.kper, p.k_stages);
    const int nk = max(kt1 - kt0, 0);
    const int nslots = (nk + SG::SPS - 1) / SG::SPS;   // packed-word slots per tile of this CTA's k range
    // tensor memory: the accumulator (bn columns) followed by TC_STAGES tiles of dequantized
    // weights (the A operand: 128 lanes x 32 columns = 128 rows x 64 fp16 each)
    const uint32_t acc_cols = bn < 32 ? 32u : (uint32_t)bn;
    uint32_t tmem_cols = 32;
    while (tmem_cols < acc_cols + TC_STAGES * (TC_BK / 2)) tmem_cols *= 2;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&a_full[s], 4); mbar_init(&a_empty[s], 1); }   // a_full: the four warps of one group
        for (int s = 0; s < NSX; ++s) mbar_init(&x_full[s], 1);
        for (int s = 0; s < NSW; ++s) { mbar_init(&w_full[s], 1); mbar_init(&w_empty[s], SG::SPS * 4); }   // w_empty: 4 reader warps per k-stage of the slot
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, TC_DQ_GROUPS * 4);          // every epilogue warp has read its part of the accumulator
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
        // ---- TMA producer of the activation tiles (one thread) ----
        // (Each ring has its own producer thread: one thread serving both spent ~250 cycles per k-stage
        // on mbarrier round trips and TMA issue, which bounded a k-stage of small token tiles.)
        if (lane == 0) {
            int sx = 0, gx = 0;                     // ring slot; activation stages requested so far, over all tiles
            bool alive = true;
            // Launched behind the activations' cast with programmatic stream serialisation: set-up and the
            // packed-word requests (weights never depend on the preceding kernel) run beside it, the
            // first activation request waits for it.
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
            int t = first_tile;
            do {   // (one trip, known at compile time, when not persistent)
                const int m0 = (t / p.n_tiles) * bn;
                for (int ix = 0; ix < nk && alive; ++ix, ++gx) {
                    // the slot is free once the MMAs of the stage NSX positions back have completed:
                    // that is the commit that also frees the A stage of that k-stage (one per stage)
                    const int jf = gx - NSX;
                    if (jf >= 0 && !mbar_wait(&a_empty[jf % TC_STAGES], (unsigned)(jf / TC_STAGES) & 1u, abort_flag, 1)) { alive = false; break; }
                    mbar_expect_tx(&x_full[sx], (unsigned)bn * 128u);
                    tma_load_2d(x_tiles + (size_t)sx * bn * 128, &x_map, (kt0 + ix) * TC_BK, m0, &x_full[sx]);
                    if (++sx == NSX) sx = 0;
                }
            } while (PERSIST && alive && (t += tile_step) < p.tiles);
        }
    } else if (warp == TC_WPROD_WARP) {
        // ---- TMA producer of the packed-word slots (one thread) ----
        // (the slots are freed by the dequantization warps as soon as they have been read into
        // registers, so this ring runs far ahead of the tensor core)
        if (lane == 0) {
            int sw = 0;
            unsigned phw = 0;
            bool alive = true;
            int t = first_tile;
            do {
                const int n0 = (t % p.n_tiles) * TC_BM;
                for (int iw = 0; iw < nslots && alive; ++iw) {
                    if (!mbar_wait(&w_empty[sw], phw ^ 1u, abort_flag, 1)) { alive = false; break; }
                    mbar_expect_tx(&w_full[sw], (unsigned)W_STAGE_BYTES);
                    tma_load_2d(w_tiles + (size_t)sw * W_STAGE_BYTES, &w_map, (kt0 + iw * SG::SPS) * SG::WPS, n0, &w_full[sw]);
                    if (++sw == NSW) { sw = 0; phw ^= 1u; }
                }
            } while (PERSIST && alive && (t += tile_step) < p.tiles);
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        // The whole warp runs the loop and one elected lane issues each tcgen05 instruction, so
        // that addresses and descriptors are warp-uniform values: issued from a single divergent
        // lane, every tcgen05.mma / tcgen05.commit took 80-90 cycles to issue (operands moved
        // one by one into uniform registers) and the issuing thread, not the tensor pipe, set
        // the pace of the kernel.
        const uint32_t idesc = umma_idesc_f16(bn, 0);
        bool ok = true;
        int si = 0, gi = 0, tile_iter = 0;          // gi: k-stages issued so far, over all tiles
        unsigned phx = 0;
        int t = first_tile;
        do {
            if (PERSIST && tile_iter > 0) {
                // the epilogue warps have read the previous tile's sums out of the accumulator
                ok = __all_sync(0xffffffffu, mbar_wait(acc_empty, (unsigned)(tile_iter - 1) & 1u, abort_flag, 7));
                if (!ok) break;
                tc_fence_after();
            }
            for (int i = 0; i < nk && ok; ++i, ++gi) {
                const int sa = gi % TC_STAGES;
                const bool got = mbar_wait(&a_full[sa], (unsigned)(gi / TC_STAGES) & 1u, abort_flag, 2) &&
                                 mbar_wait(&x_full[si], phx, abort_flag, 3);
                ok = __all_sync(0xffffffffu, got);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_taddr = tmem_base + acc_cols + (uint32_t)sa * (TC_BK / 2);
                const uint32_t b_addr = smem_addr(x_tiles + (size_t)si * bn * 128);
#pragma unroll
                for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                    umma_f16_ts(tmem_base, a_taddr + k4 * 8, umma_smem_desc(b_addr + k4 * 32), idesc,
                                (i | k4) != 0 ? 1u : 0u);
                umma_commit(&a_empty[sa]);     // the A stage and the activation slot are free once these MMAs have read them
                if (++si == NSX) { si = 0; phx ^= 1u; }
            }
            if (ok) umma_commit(acc_full);     // accumulator complete (arrives at once when nk == 0)
            ++tile_iter;
        } while (PERSIST && ok && (t += tile_step) < p.tiles);
    } else {
        // ---- dequantization threads (one weight row each), then epilogue ----
        const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
        const int dgroup = (warp - 2) >> 2;              // this group expands the stages whose running index is dgroup mod 4
        const int row = quad * 32 + lane;                // tile row == TMEM lane
        const int gps = max(1, TC_BK >> p.g_shift);      // groups per stage (<= 4)
        const int swz = (row & 7);                       // 128-byte swizzle of the packed-word slots
        bool ok = true;
        int gbase = 0, slot_base = 0, tile_iter = 0;     // running stage / slot index of the tile's first stage
        int t = first_tile;
        do {
            const int n0 = (t % p.n_tiles) * TC_BM, m0 = (t / p.n_tiles) * bn;
            int64_t n = (int64_t)n0 + row;
            const bool n_ok = n < p.N;
            if (!n_ok) n = p.N - 1;
            const __half *srow = p.scale + n * p.G, *zrow = p.zp + n * p.G;

            GroupConst gcs[4];
            auto prefetch_consts = [&](int kt) {             // kt = global k-stage index
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
            const int i0 = (dgroup - gbase) & (TC_DQ_GROUPS - 1);   // this group's first stage of the tile
            if (i0 < nk) prefetch_consts(kt0 + i0);
            for (int i = i0; i < nk; i += TC_DQ_GROUPS) {
                const int gi = gbase + i;
                const int sa = gi % TC_STAGES;
                const int kt = kt0 + i;
                GroupConst gc_now[4] = {gcs[0], gcs[1], gcs[2], gcs[3]};
                if (i + TC_DQ_GROUPS < nk) prefetch_consts(kt + TC_DQ_GROUPS);
                uint32_t w[SG::WPS];
                {
                    // stage i lies in slot i / SPS of this tile, at position (i % SPS) of each 128-byte row
                    const int slot = slot_base + i / SG::SPS, si = slot & (NSW - 1);
                    const unsigned phw = (unsigned)(slot >> p.w_stages_log2) & 1u;
                    ok = __all_sync(0xffffffffu, mbar_wait(&w_full[si], phw, abort_flag, 6));
                    if (!ok) break;
                    const uint4 *src = reinterpret_cast<const uint4 *>(w_tiles + (size_t)si * W_STAGE_BYTES + (size_t)row * 128);
                    const int c0 = (i % SG::SPS) * SG::VPS;
#pragma unroll
                    for (int v = 0; v < SG::VPS; ++v) {
                        const uint4 tq = src[(c0 + v) ^ swz];
                        w[4 * v] = tq.x; w[4 * v + 1] = tq.y; w[4 * v + 2] = tq.z; w[4 * v + 3] = tq.w;
                    }
                    // generic-proxy reads of the slot must be ordered before the async-proxy (TMA) write
                    // that refills it: without this fence random rows read the next stage's words
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&w_empty[si]);    // the packed words are in registers now
                }
                uint4 chunk[8];
                if (gps == 1) expand_stage<BITS, true>(w, gc_now, kt * TC_BK, p.g_shift, (kt * TC_BK) >> p.g_shift, chunk);
                else expand_stage<BITS, false>(w, gc_now, kt * TC_BK, p.g_shift, (kt * TC_BK) >> p.g_shift, chunk);
                ok = __all_sync(0xffffffffu, mbar_wait(&a_empty[sa], ((unsigned)(gi / TC_STAGES) & 1u) ^ 1u, abort_flag, 4));
                if (!ok) break;
                tc_fence_after();                            // the MMAs that read this stage come before the stores below
                {
                    // this thread's row of the A tile: 64 fp16 in k order = 32 columns of its TMEM lane
                    uint32_t a_regs[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) { a_regs[4 * c] = chunk[c].x; a_regs[4 * c + 1] = chunk[c].y; a_regs[4 * c + 2] = chunk[c].z; a_regs[4 * c + 3] = chunk[c].w; }
                    tmem_st_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc_cols + (uint32_t)sa * (TC_BK / 2), a_regs);
                }
                tc_fence_before();                           // the stores are ordered before the arrival
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[sa]);
            }
            // ---- epilogue of this tile ----
            const bool acc_ok = __all_sync(0xffffffffu, ok && mbar_wait(acc_full, (unsigned)tile_iter & 1u, abort_flag, 5));
            if (acc_ok) tc_fence_after();
            const int nblk = bn < 32 ? 1 : bn / 32, per = (nblk + TC_DQ_GROUPS - 1) / TC_DQ_GROUPS;
            const __half bias_h = (p.bias && n_ok) ? p.bias[n] : __float2half(0.0f);
            auto store_out = [&](int64_t m, float v) {
                store_output(p.out, p.out_dtype, m * p.N + n, v, p.bias != nullptr, bias_h, p.ep);
            };
            if (p.splits == 1) {
                if (TMAST && acc_ok) {
                    // Each group turns its blocks of 32 tokens into [32 tokens][128 rows] tiles of the output
                    // dtype in shared memory (lane = row: consecutive lanes write consecutive elements) and
                    // one thread hands each tile to a TMA store, which writes whole 256- or 512-byte row
                    // segments and clips at the edges of the output.  (Two-byte stores straight from the
                    // registers, 64 bytes per warp instruction, took 9 us of a 35 us tile.)
                    unsigned char *stage = o_stage + (size_t)dgroup * 32 * TC_BM * o_esize;
                    const bool issuer = quad == 0 && lane == 0;
                    const int cb_end = min(nblk, (dgroup + 1) * per);
                    for (int cb = dgroup * per; cb < cb_end; ++cb) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), r);
                        if (cb == cb_end - 1) {
                            // this warp's last read of the accumulator: the next tile's first MMA may overwrite it
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(acc_empty);
                        }
                        // the previous store out of this staging tile has finished reading it
                        if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        asm volatile("bar.sync %0, 128;" ::"r"(1 + dgroup) : "memory");
                        if (p.out_dtype == BW_F16) {
                            __half *dst = reinterpret_cast<__half *>(stage) + row;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                __half c = __float2half_rn(__uint_as_float(r[j]));       // the GEMM's fp16 output rounding
                                if (p.bias) c = __hadd(c, bias_h);                       // separate fp16 bias add
                                if (p.ep.act == BW_ACT_RELU) c = __hmax(c, __float2half(0.0f));
                                dst[j * TC_BM] = c;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float v = __uint_as_float(r[j]);
                                if (p.bias) v += __half2float(bias_h);
                                if (p.ep.act == BW_ACT_RELU) v = fmaxf(v, 0.0f);
                                if (p.out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(stage)[j * TC_BM + row] = __float2bfloat16_rn(v);
                                else reinterpret_cast<float *>(stage)[j * TC_BM + row] = v;
                            }
                        }
                        fence_proxy_async_smem();                  // generic-proxy writes before the async-proxy read
                        asm volatile("bar.sync %0, 128;" ::"r"(1 + dgroup) : "memory");
                        if (issuer) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                         ::"l"(&out_map), "r"(smem_addr(stage)), "r"(n0), "r"(m0 + cb * 32) : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                    if (cb_end <= dgroup * per) {
                        // a group without a block of this tile still owes its arrivals
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty);
                    }
                } else if (acc_ok) {
                    // the warp groups share the lane quadrants and split the token columns
                    for (int cb = dgroup * per; cb < min(nblk, (dgroup + 1) * per); ++cb) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), r);
                        if (p.ep.act == BW_ACT_SILU_MUL) {
                            // adjacent lanes hold a (gate, up) row pair: the even lane takes both and stores
                            const __half bias_u = __shfl_xor_sync(0xffffffffu, bias_h, 1);
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const float up = __shfl_xor_sync(0xffffffffu, __uint_as_float(r[j]), 1);
                                const int64_t m = (int64_t)m0 + cb * 32 + j;
                                if ((lane & 1) == 0 && n + 1 < p.N && n_ok && m < p.M)
                                    store_output_silu_mul(p.out, p.out_dtype, m * (p.N >> 1) + (n >> 1), __uint_as_float(r[j]), up,
                                                          p.bias != nullptr, bias_h, bias_u, p.ep);
                            }
                            continue;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int64_t m = (int64_t)m0 + cb * 32 + j;
                            if (n_ok && m < p.M) store_out(m, __uint_as_float(r[j]));
                        }
                    }
                    // the accumulator may be overwritten by the next tile's first MMA
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty);
                }
            } else {
                // split-K: park this CTA's partial tile in its own shared memory (the input ring
                // is idle by now) as red[column][row]; the cluster sums it below
                float *red = reinterpret_cast<float *>(x_tiles);
                if (acc_ok) {
                    for (int cb = dgroup * per; cb < min(nblk, (dgroup + 1) * per); ++cb) {
                        uint32_t r[32];
                        if (nk > 0) tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(cb * 32), r);
#pragma unroll
                        for (int j = 0; j < 32; ++j) red[(cb * 32 + j) * TC_BM + row] = nk > 0 ? __uint_as_float(r[j]) : 0.0f;
                    }
                }
            }
            if (!acc_ok) break;
            ++tile_iter; gbase += nk; slot_base += nslots;
        } while (PERSIST && (t += tile_step) < p.tiles);
    }
    if (p.splits > 1) {
        // every thread of every CTA of the cluster reaches these barriers (also after an abort)
        cgx::cluster_group cluster = cgx::this_cluster();
        float *red = reinterpret_cast<float *>(x_tiles);
        const int n0 = blockIdx.x * TC_BM, m0 = blockIdx.y * bn;     // split-K launches are never persistent
        cluster.sync();
        if (warp >= 2 && warp < TC_WPROD_WARP && *abort_flag == 0) {
            const int rank = (int)cluster.block_rank(), nranks = (int)cluster.num_blocks();
            const int cols = bn < 32 ? 32 : bn;
            const int per_rank = (cols + nranks - 1) / nranks;
            const int row = (warp & 3) * 32 + lane, dgroup = (warp - 2) >> 2;
            const int64_t n = (int64_t)n0 + row;
            const __half bias_h = (p.bias && n < p.N) ? p.bias[n] : __float2half(0.0f);
            for (int c = rank * per_rank + dgroup; c < min(cols, (rank + 1) * per_rank); c += TC_DQ_GROUPS) {
                float v = 0.0f;
                for (int q = 0; q < nranks; ++q) v += cluster.map_shared_rank(red, q)[c * TC_BM + row];
                const int64_t m = (int64_t)m0 + c;
                if (p.ep.act == BW_ACT_SILU_MUL) {
                    // (the loop bounds do not depend on the lane: the whole warp is here)
                    const float up = __shfl_xor_sync(0xffffffffu, v, 1);
                    const __half bias_u = __shfl_xor_sync(0xffffffffu, bias_h, 1);
                    if ((lane & 1) == 0 && n + 1 < p.N && m < p.M)
                        store_output_silu_mul(p.out, p.out_dtype, m * (p.N >> 1) + (n >> 1), v, up, p.bias != nullptr, bias_h, bias_u, p.ep);
                    continue;
                }
                if (n < p.N && m < p.M)
                    store_output(p.out, p.out_dtype, m * p.N + n, v, p.bias != nullptr, bias_h, p.ep);
            }
        }
        cluster.sync();   // keep shared memory alive until every peer has read it
    }
    // the staging tiles must outlive the bulk stores that read them
    if (TMAST) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// Activations that are not fp16 are cast once (bitween/modules.py:74) into caller scratch.
template <typename XT>
__global__ void __launch_bounds__(256) cast_to_f16_kernel(const XT *__restrict__ x, __half *__restrict__ y, int64_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the GEMM behind it may start its set-up
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

int g_tc_splits = 0;   // experiments: force the split-K factor (0 = automatic)

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
int launch_tc(const CUtensorMap &xmap, const CUtensorMap &wmap, const CUtensorMap &omap, TcParams p, cudaStream_t st) {
    using SG = StageGeom<BITS>;
    // (the kernel is chosen below, once the schedule is known)
    const size_t w_stage = (size_t)TC_BM * 128, x_stage = (size_t)p.bn * 128;
    const size_t o_stage = p.tma_store ? (size_t)TC_DQ_GROUPS * 32 * TC_BM * (p.out_dtype == BW_F32 ? 4 : 2) : 0;
    const size_t fixed = 1024 /*alignment slack*/ + 1024 /*barriers*/ + o_stage;
    // Packed-word ring: 4 slots of 16 KB for small token tiles (the weight stream is what is being
    // waited for), 2 for large ones.  Each slot is always read by the same dequantization groups,
    // once per phase (a waiter that skipped a phase could not tell phase k from phase k-2).
    int nsw = p.bn >= 128 ? 2 : 4;
    int nsx = (int)((227 * 1024 - fixed - (size_t)nsw * w_stage) / x_stage);
    if (nsx > TC_STAGES) nsx = TC_STAGES;   // activation slots are released by the commits of the A stages
    if (nsx < 2) return BW_ERR_UNSUPPORTED;
    p.x_stages = nsx;
    p.w_stages = nsw;
    p.w_stages_log2 = nsw == 4 ? 2 : 1;
    // split-K (cluster along z) only for small tiles that would leave most SMs idle
    const int64_t tiles = ((p.N + TC_BM - 1) / TC_BM) * ((p.M + p.bn - 1) / p.bn);
    int splits = 1;
    if (g_tc_splits > 0) splits = g_tc_splits;
    else if (tiles < 148) {
        splits = (int)(148 / tiles);
        if (splits > 8) splits = 8;
        if (splits > p.k_stages / 4) splits = p.k_stages / 4;
        if (splits < 1) splits = 1;
    }
    const size_t red_bytes = (size_t)(p.bn < 32 ? 32 : p.bn) * TC_BM * 4;
    if (splits > 8 || red_bytes > (size_t)nsx * x_stage + (size_t)nsw * w_stage) splits = 1;
    if (splits > 1) p.tma_store = 0;   // split-K tiles are summed by the cluster and stored from registers
    p.splits = splits;
    p.kper = (p.k_stages + splits - 1) / splits;
    if (tiles > ((int64_t)1 << 30)) return BW_ERR_UNSUPPORTED;
    p.n_tiles = (int)((p.N + TC_BM - 1) / TC_BM);
    p.tiles = (int)tiles;
    // More tiles than SMs: one persistent CTA per SM walks the tile list (whole packed-word slots per
    // tile, so that every slot of the ring collects its full count of releases).
    int sms = 148;
    {
        int dev_id = 0, v = 0;
        if (cudaGetDevice(&dev_id) == cudaSuccess &&
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev_id) == cudaSuccess && v > 0)
            sms = v;
    }
    // (tiles of 256 tokens and K <= 4096 only: for smaller token tiles and for longer K the per-tile costs
    // it removes are a small share, and the one-tile instantiation, with fewer registers, measured faster:
    // 7 % on a 28672 x 8192 layer at 4096 tokens)
    p.persistent = (splits == 1 && p.bn == 256 && p.k_stages <= 64 && tiles > sms && p.k_stages % SG::SPS == 0) ? 1 : 0;
    const size_t smem = fixed + (size_t)nsx * x_stage + (size_t)nsw * w_stage;
    static size_t configured[64] = {};
    int dev = 0;
    BW_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
        BW_CUDA_TRY(cudaFuncSetAttribute(qmm_tc_kernel<BITS, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        BW_CUDA_TRY(cudaFuncSetAttribute(qmm_tc_kernel<BITS, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        BW_CUDA_TRY(cudaFuncSetAttribute(qmm_tc_kernel<BITS, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        BW_CUDA_TRY(cudaFuncSetAttribute(qmm_tc_kernel<BITS, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = p.persistent ? dim3((unsigned)sms, 1, 1)
                               : dim3((unsigned)p.n_tiles, (unsigned)((p.M + p.bn - 1) / p.bn), (unsigned)splits);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = (unsigned)splits;
        ++na;
    }
    if (p.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (p.persistent && p.tma_store) BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_tc_kernel<BITS, true, true>, xmap, wmap, omap, p));
    else if (p.persistent) BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_tc_kernel<BITS, true, false>, xmap, wmap, omap, p));
    else if (p.tma_store) BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_tc_kernel<BITS, false, true>, xmap, wmap, omap, p));
    else BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_tc_kernel<BITS, false, false>, xmap, wmap, omap, p));
    return BW_OK;
}

}  // namespace

static bool g_tc_enabled = true;
void set_tc_enabled(int on) { g_tc_enabled = on != 0; }
void set_tc_splits(int s) { g_tc_splits = s; }

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
    // fp16 activations are read by TMA as they are; bf16 / fp32 (or misaligned) activations are
    // cast to fp16 first, as the reference does (bitween/modules.py:74).  kind::f16 MMAs want
    // both operands in the same 16-bit format: an fp16 A with a bf16 B raised an illegal
    // instruction on sm_100a, so the B-format bit of the descriptor stays 0.
    const bool direct = x_dtype == BW_F16 && aligned_to(x, 16);
    if (!direct) {
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
    p.bn = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : (M > 16 ? 32 : 16)));
    p.x_is_bf16 = 0;
    p.pdl = direct ? 0 : 1;      // the cast kernel precedes this launch in the stream
    p.ep = current_epilogue();

    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};                 // bytes between token rows
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)p.bn};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_tiled_fn()(&map, p.x_is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xh), dims,
                                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return BW_ERR_UNSUPPORTED;
    // packed words: [N rows][K/vpi int32], one box = 128 rows x the words of one 64-k stage
    CUtensorMap wmap;
    const cuuint64_t wdims[2] = {(cuuint64_t)p.words_per_row, (cuuint64_t)N};
    const cuuint64_t wstrides[1] = {(cuuint64_t)p.words_per_row * 4};
    const cuuint32_t wbox[2] = {32u, (cuuint32_t)TC_BM};   // 128 bytes of every row: 2, 4 or 8 k-stages
    const CUresult rw = encode_tiled_fn()(&wmap, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(q), wdims,
                                          wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rw != CUDA_SUCCESS) return BW_ERR_UNSUPPORTED;
    // output [M tokens][N]: boxes of 32 tokens x 128 rows for the TMA-store epilogue (needs a 16-byte
    // aligned base and row pitch; a residual operand is read per element, so it takes the direct path)
    CUtensorMap omap = wmap;
    const size_t oes = dtype_size(out_dtype);
    p.tma_store = 0;
    // (token tiles of 64 and more: timed inside the kernel, the register-store epilogue of a 64-token tile
    // took 3 us of a 25 us launch)
    if (p.bn >= 64 && N >= TC_BM && (N * oes) % 16 == 0 && aligned_to(out, 16) && !p.ep.residual && p.ep.act != BW_ACT_SILU_MUL) {
        const cuuint64_t odims[2] = {(cuuint64_t)N, (cuuint64_t)M};
        const cuuint64_t ostrides[1] = {(cuuint64_t)N * oes};
        const cuuint32_t obox[2] = {(cuuint32_t)TC_BM, 32u};
        const CUresult ro = encode_tiled_fn()(&omap, out_dtype == BW_F32 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16,
                                              2, out, odims, ostrides, obox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (ro == CUDA_SUCCESS) p.tma_store = 1;
    }
    set_last_kernel("qmm_tc_kernel");
    switch (bits) {
        case 2: return launch_tc<2>(map, wmap, omap, p, st);
        case 4: return launch_tc<4>(map, wmap, omap, p, st);
        default: return launch_tc<8>(map, wmap, omap, p, st);
    }
}

}  // namespace bw
