// Small-M ("decode") quantized matmul for sm_100a:  out[M,N] = x[M,K] . W[N,K]^T (+bias),
// W = fp16(scale * (code - zero_point)), for M <= 64 tokens per launch.
//
// Replaces, for few tokens, the three-launch forward of the reference
// (bitween/modules.py:85-101: allocate fp16 [N,K], Triton dequantize, cuBLAS matmul, bias
// add), which moves about N*K*(bits/8 + 4) bytes; this kernel streams the packed words
// once (N*K*bits/8 bytes) and never materialises W.
//
// Shape of the computation ("swap-AB"): the packed weight rows fill the 16-row dimension
// of mma.sync.m16n8k16 and the 1..64 tokens are its 8-wide dimension, so a 16x16 weight
// tile costs one tensor instruction per 8 tokens and the kernel stays HBM-bound.
//
//   * each lane streams 16-byte vectors of packed words of rows r and r+8 with cp.async
//     into a private 4-stage shared-memory ring (no block-wide barrier in the k loop)
//   * codes become fp16 in registers by the magic-number trick (lop3/prmt into
//     1024+code, subtract 1024+zp, multiply by scale) -- the subtraction is exact and the
//     product is rounded once to fp16, so W is bit-identical to the reference's fp16
//     weights (bitween/modules.py:55-58)
//   * the order of the k slots inside an MMA is free as long as A and B agree; activations
//     are staged once per CTA into shared memory already permuted to the order the
//     code extraction produces ((c_j, c_{j+vpi/2}) pairs), as one conflict-free 16-byte
//     load per lane per MMA pair
//   * split-K runs across the CTAs of a thread-block cluster; partial tiles are summed
//     through distributed shared memory (barrier.cluster, no global scratch, no flags to
//     spin on) and the owning CTA writes fp16(fp16(acc)+bias)
#include <cooperative_groups.h>

#include "bw_common.cuh"

namespace cg = cooperative_groups;

namespace bw {
namespace {

constexpr int STAGES = 4;

struct SmallMParams {
    const void *x;
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
    int xblock;           // k-chunks whose activations are staged in shared memory at once
    int splits;           // cluster size along y
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return d;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // src-size 0 => the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Per-(row, group) dequantization constants kept in shared memory: {scale,scale} and
// {1024+zp, 1024+zp} as half2 pairs.
struct GroupConst { uint32_t s2, z1024; };

template <int BITS> struct Geometry {
    static constexpr int VPI = 32 / BITS;    // codes per word
    static constexpr int KL = 4 * VPI;       // k values per lane load (one uint4)
    static constexpr int KC = 4 * KL;        // k values per warp step (4 lanes along k)
    static constexpr int NX = KL / 8;        // 16-byte activation pieces per lane load per token tile
    static constexpr int UNIT = VPI > 8 ? VPI : 8;  // k values permuted together when staging x
};

// ---- code extraction: word -> fp16 pairs (c_j, c_{j+VPI/2}), already scaled --------
template <int BITS> struct Dequant;

template <> struct Dequant<4> {
    uint32_t s2, z1024, n64;
    __device__ __forceinline__ void set(GroupConst c) {
        s2 = c.s2; z1024 = c.z1024;
        n64 = h2_as_u32(__hsub2(__float2half2_rn(960.0f), u32_as_h2(c.z1024)));  // -(64+zp)
    }
    // out[j] = (c_j, c_{j+4}) for j = 0..3
    __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[4]) const {
        constexpr uint32_t LO = 0x000f000fu, HI = 0x00f000f0u, EX = 0x64006400u;
        const __half2 sixteenth = __float2half2_rn(0.0625f);
        const uint32_t w8 = w >> 8;
        const __half2 t0 = __hsub2(u32_as_h2(lop3_and_or(w, LO, EX)), u32_as_h2(z1024));
        const __half2 t1 = __hfma2(u32_as_h2(lop3_and_or(w, HI, EX)), sixteenth, u32_as_h2(n64));
        const __half2 t2 = __hsub2(u32_as_h2(lop3_and_or(w8, LO, EX)), u32_as_h2(z1024));
        const __half2 t3 = __hfma2(u32_as_h2(lop3_and_or(w8, HI, EX)), sixteenth, u32_as_h2(n64));
        out[0] = h2_as_u32(__hmul2(t0, u32_as_h2(s2)));
        out[1] = h2_as_u32(__hmul2(t1, u32_as_h2(s2)));
        out[2] = h2_as_u32(__hmul2(t2, u32_as_h2(s2)));
        out[3] = h2_as_u32(__hmul2(t3, u32_as_h2(s2)));
    }
};

template <> struct Dequant<8> {
    uint32_t s2, z1024;
    __device__ __forceinline__ void set(GroupConst c) { s2 = c.s2; z1024 = c.z1024; }
    // out[j] = (c_j, c_{j+2}) for j = 0..1
    __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[2]) const {
        constexpr uint32_t EX = 0x64646464u;
        const uint32_t p0 = __byte_perm(w, EX, 0x4240);  // bytes [c0, 0x64, c2, 0x64]
        const uint32_t p1 = __byte_perm(w, EX, 0x4341);  // bytes [c1, 0x64, c3, 0x64]
        out[0] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(p0), u32_as_h2(z1024)), u32_as_h2(s2)));
        out[1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(p1), u32_as_h2(z1024)), u32_as_h2(s2)));
    }
};

template <> struct Dequant<2> {
    uint32_t s2, z1024, n256, n64, n16, n4;
    __device__ __forceinline__ void set(GroupConst c) {
        s2 = c.s2; z1024 = c.z1024;
        const __half2 z = u32_as_h2(c.z1024);
        n256 = h2_as_u32(__hsub2(__float2half2_rn(768.0f), z));    // -(256+zp)
        n64 = h2_as_u32(__hsub2(__float2half2_rn(960.0f), z));     // -(64+zp)
        n16 = h2_as_u32(__hsub2(__float2half2_rn(1008.0f), z));    // -(16+zp)
        n4 = h2_as_u32(__hsub2(__float2half2_rn(1020.0f), z));     // -(4+zp)
    }
    // out[j] = (c_j, c_{j+8}) for j = 0..7
    __device__ __forceinline__ void run(uint32_t w, uint32_t (&out)[8]) const {
        constexpr uint32_t EX = 0x64006400u;
        const __half2 q4 = __float2half2_rn(0.25f), q16 = __float2half2_rn(0.0625f);
        const __half2 q64 = __float2half2_rn(0.015625f), q256 = __float2half2_rn(0.00390625f);
        const uint32_t w10 = w >> 10;
        const __half2 s = u32_as_h2(s2);
        __half2 t;
        t = __hsub2(u32_as_h2(lop3_and_or(w, 0x00030003u, EX)), u32_as_h2(z1024));            out[0] = h2_as_u32(__hmul2(t, s));
        t = __hfma2(u32_as_h2(lop3_and_or(w, 0x000c000cu, EX)), q4, u32_as_h2(n256));          out[1] = h2_as_u32(__hmul2(t, s));
        t = __hfma2(u32_as_h2(lop3_and_or(w, 0x00300030u, EX)), q16, u32_as_h2(n64));          out[2] = h2_as_u32(__hmul2(t, s));
        t = __hfma2(u32_as_h2(lop3_and_or(w, 0x00c000c0u, EX)), q64, u32_as_h2(n16));          out[3] = h2_as_u32(__hmul2(t, s));
        t = __hfma2(u32_as_h2(lop3_and_or(w, 0x03000300u, EX)), q256, u32_as_h2(n4));          out[4] = h2_as_u32(__hmul2(t, s));
        t = __hsub2(u32_as_h2(lop3_and_or(w10, 0x00030003u, EX)), u32_as_h2(z1024));          out[5] = h2_as_u32(__hmul2(t, s));
        t = __hfma2(u32_as_h2(lop3_and_or(w10, 0x000c000cu, EX)), q4, u32_as_h2(n256));        out[6] = h2_as_u32(__hmul2(t, s));
        t = __hfma2(u32_as_h2(lop3_and_or(w10, 0x00300030u, EX)), q16, u32_as_h2(n64));        out[7] = h2_as_u32(__hmul2(t, s));
    }
};

// ---- activation staging: UNIT consecutive k of one token -> fp16, permuted -----------
template <typename XT> __device__ __forceinline__ __half x_to_half(XT v);
template <> __device__ __forceinline__ __half x_to_half<__half>(__half v) { return v; }
template <> __device__ __forceinline__ __half x_to_half<__nv_bfloat16>(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }
template <> __device__ __forceinline__ __half x_to_half<float>(float v) { return __float2half_rn(v); }

template <int UNIT, typename XT>
__device__ __forceinline__ void load_unit(const XT *src, bool valid, __half (&h)[UNIT]) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < UNIT; ++i) h[i] = __ushort_as_half(0);
        return;
    }
    constexpr int BYTES = UNIT * sizeof(XT);
    alignas(16) XT tmp[UNIT];
#pragma unroll
    for (int j = 0; j < BYTES / 16; ++j)
        reinterpret_cast<uint4 *>(tmp)[j] = __ldg(reinterpret_cast<const uint4 *>(src) + j);
#pragma unroll
    for (int i = 0; i < UNIT; ++i) h[i] = x_to_half<XT>(tmp[i]);
}

// (lo16 of x, lo16 of y) and (hi16 of x, hi16 of y)
__device__ __forceinline__ uint32_t pair_lo(uint32_t x, uint32_t y) { return __byte_perm(x, y, 0x5410); }
__device__ __forceinline__ uint32_t pair_hi(uint32_t x, uint32_t y) { return __byte_perm(x, y, 0x7632); }

template <typename XT> __device__ __forceinline__ uint32_t pair_to_half2(uint32_t raw);
template <> __device__ __forceinline__ uint32_t pair_to_half2<__half>(uint32_t raw) { return raw; }
template <> __device__ __forceinline__ uint32_t pair_to_half2<__nv_bfloat16>(uint32_t raw) {
    return h2_as_u32(__floats2half2_rn(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u)));
}

// Shared-memory slot (in uint4 units) of activation piece `px` of lane column `t`, token m.
template <int BITS, int MT>
__device__ __forceinline__ int x_slot(int cl, int px, int m, int t) {
    return ((cl * Geometry<BITS>::NX + px) * MT + (m >> 3)) * 32 + (m & 7) * 4 + t;
}

// Stages the activations of k-chunks [chunk0, chunk0+nchunks) and the per-(group,row)
// constants.  16-bit activations go global->shared with cp.async (all copies of a thread in
// flight at once) and are converted/permuted in place by the thread that copied them; fp32
// activations take a batched register path.
template <int BITS, int MT, int RT, int WARPS, bool TWO_GROUPS, typename XT>
__device__ __forceinline__ void stage_block(const SmallMParams &p, int chunk0, int nchunks, int n0,
                                            uint4 *xs, GroupConst *gc, int grp0, int ngrp) {
    using Geo = Geometry<BITS>;
    constexpr int UNIT = Geo::UNIT;
    constexpr int ROWS = WARPS * RT * 16;
    constexpr int MTOK = MT * 8;
    constexpr int NTHR = WARPS * 32;
    constexpr int UPC = Geo::KC / UNIT;                  // staging units per chunk
    const int tid = threadIdx.x;
    const XT *x = reinterpret_cast<const XT *>(p.x);
    const int upr = nchunks * UPC;                       // units per token row (k fastest => coalesced)
    const int total_units = upr * MTOK;

    // decode unit index -> (token, chunk, unit-in-chunk); slots of its one or two pieces
    auto slots_of = [&](int i, int &m, int64_t &k, int &s0, int &s1) {
        const int u = i % upr;
        m = i / upr;
        const int cl = u / UPC, uc = u % UPC;
        k = (int64_t)(chunk0 + cl) * Geo::KC + (int64_t)uc * UNIT;
        if constexpr (BITS == 4) { s0 = x_slot<BITS, MT>(cl, uc & 3, m, uc >> 2); s1 = s0; }
        else if constexpr (BITS == 8) { s0 = x_slot<BITS, MT>(cl, uc & 1, m, uc >> 1); s1 = s0; }
        else { s0 = x_slot<BITS, MT>(cl, 2 * (uc & 3), m, uc >> 2); s1 = x_slot<BITS, MT>(cl, 2 * (uc & 3) + 1, m, uc >> 2); }
    };
    auto permute_store = [&](const uint32_t (&r)[UNIT / 2], int s0, int s1) {
        if constexpr (BITS == 4) {
            xs[s0] = make_uint4(pair_lo(r[0], r[2]), pair_hi(r[0], r[2]), pair_lo(r[1], r[3]), pair_hi(r[1], r[3]));
        } else if constexpr (BITS == 8) {
            xs[s0] = make_uint4(pair_lo(r[0], r[1]), pair_hi(r[0], r[1]), pair_lo(r[2], r[3]), pair_hi(r[2], r[3]));
        } else {
            xs[s0] = make_uint4(pair_lo(r[0], r[4]), pair_hi(r[0], r[4]), pair_lo(r[1], r[5]), pair_hi(r[1], r[5]));
            xs[s1] = make_uint4(pair_lo(r[2], r[6]), pair_hi(r[2], r[6]), pair_lo(r[3], r[7]), pair_hi(r[3], r[7]));
        }
    };

    if constexpr (sizeof(XT) == 2) {
        for (int i = tid; i < total_units; i += NTHR) {
            int m, s0, s1; int64_t k;
            slots_of(i, m, k, s0, s1);
            const bool valid = (m < p.M) && (k < p.K);
            const XT *src = x + (valid ? ((int64_t)m * p.K + k) : 0);
            cp_async16(xs + s0, src, valid);
            if constexpr (UNIT == 16) cp_async16(xs + s1, src + 8, valid);
        }
        cp_async_commit();
    }

    // --- per-(group,row) constants, loads batched four at a time ---
    const int total_gc = ngrp * ROWS;
    for (int base = tid; base < total_gc; base += NTHR * 4) {
        __half sv[4], zv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = base + j * NTHR;
            if (i < total_gc) {
                const int gl = i % ngrp, r = i / ngrp;
                int64_t n = (int64_t)n0 + r;
                if (n >= p.N) n = p.N - 1;
                int grp = grp0 + gl;
                if (grp >= p.G) grp = p.G - 1;
                sv[j] = p.scale[n * p.G + grp];
                zv[j] = p.zp[n * p.G + grp];
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = base + j * NTHR;
            if (i < total_gc) {
                const int gl = i % ngrp, r = i / ngrp;
                GroupConst c;
                c.s2 = h2_as_u32(__half2half2(sv[j]));
                c.z1024 = h2_as_u32(__hadd2(__half2half2(zv[j]), __float2half2_rn(1024.0f)));
                gc[gl * ROWS + r] = c;
            }
        }
    }

    if constexpr (sizeof(XT) == 2) {
        cp_async_wait<0>();   // this thread's own copies (and its weight prefetches) have landed
        for (int i = tid; i < total_units; i += NTHR) {
            int m, s0, s1; int64_t k;
            slots_of(i, m, k, s0, s1);
            uint32_t r[UNIT / 2];
            const uint4 a = xs[s0];
            r[0] = pair_to_half2<XT>(a.x); r[1] = pair_to_half2<XT>(a.y);
            r[2] = pair_to_half2<XT>(a.z); r[3] = pair_to_half2<XT>(a.w);
            if constexpr (UNIT == 16) {
                const uint4 b = xs[s1];
                r[4] = pair_to_half2<XT>(b.x); r[5] = pair_to_half2<XT>(b.y);
                r[6] = pair_to_half2<XT>(b.z); r[7] = pair_to_half2<XT>(b.w);
            }
            permute_store(r, s0, s1);
        }
    } else {
        // fp32 activations: rounded to fp16 (bitween/modules.py:74), two units per batch
        for (int base = tid; base < total_units; base += NTHR * 2) {
            float v[2][UNIT];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int i = base + j * NTHR;
                int m, s0, s1; int64_t k;
                if (i < total_units) {
                    slots_of(i, m, k, s0, s1);
                    const bool valid = (m < p.M) && (k < p.K);
                    const float4 *src = reinterpret_cast<const float4 *>(x + (valid ? ((int64_t)m * p.K + k) : 0));
#pragma unroll
                    for (int e = 0; e < UNIT / 4; ++e) {
                        const float4 f = valid ? __ldg(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                        v[j][4 * e] = f.x; v[j][4 * e + 1] = f.y; v[j][4 * e + 2] = f.z; v[j][4 * e + 3] = f.w;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int i = base + j * NTHR;
                if (i < total_units) {
                    int m, s0, s1; int64_t k;
                    slots_of(i, m, k, s0, s1);
                    uint32_t r[UNIT / 2];
#pragma unroll
                    for (int e = 0; e < UNIT / 2; ++e) r[e] = h2_as_u32(__floats2half2_rn(v[j][2 * e], v[j][2 * e + 1]));
                    permute_store(r, s0, s1);
                }
            }
        }
    }
}

template <int BITS, int MT, int RT, int WARPS, bool TWO_GROUPS>
__global__ void __launch_bounds__(WARPS * 32)
qmm_smallm_kernel(const SmallMParams p) {
    using Geo = Geometry<BITS>;
    constexpr int ROWS = WARPS * RT * 16;
    constexpr int MTOK = MT * 8;
    constexpr int SLOTS = 2 * RT;                         // uint4 per lane per stage
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4 *ring = reinterpret_cast<uint4 *>(smem_raw);                       // [WARPS][STAGES][SLOTS][32]
    uint4 *xs = ring + WARPS * STAGES * SLOTS * 32;                          // [xblock][NX][MT][32]
    GroupConst *gc = reinterpret_cast<GroupConst *>(xs + (size_t)p.xblock * Geo::NX * MT * 32);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int split = blockIdx.y;
    const int c_begin = split * p.chunks_per_cta;
    const int c_end = min(c_begin + p.chunks_per_cta, p.chunks_total);
    const int nloc = max(c_end - c_begin, 0);

    // rows streamed by this lane (clamped so that loads stay in range; stores are masked)
    const int32_t *rowp[SLOTS];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int64_t n = (int64_t)n0 + warp * (RT * 16) + rt * 16 + h * 8 + g;
            if (n >= p.N) n = p.N - 1;
            rowp[rt * 2 + h] = p.q + n * p.words_per_row;
        }
    }
    uint4 *myring = ring + (size_t)warp * STAGES * SLOTS * 32 + lane;
    auto issue = [&](int i) {   // i = local chunk index; always commits a group (possibly empty)
        if (i < nloc) {
            const int word0 = (c_begin + i) * (Geo::KC / Geo::VPI) + t * 4;
            const bool valid = word0 < p.words_per_row;
            const int wsafe = valid ? word0 : 0;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s)
                cp_async16(myring + ((i % STAGES) * SLOTS + s) * 32, rowp[s] + wsafe, valid);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) issue(i);

    float acc[RT][MT][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[rt][mt][e] = 0.0f;

    for (int xb = 0; xb < nloc; xb += p.xblock) {
        const int nb = min(p.xblock, nloc - xb);
        const int chunk0 = c_begin + xb;
        const int grp0 = (int)(((int64_t)chunk0 * Geo::KC) >> p.g_shift);
        const int grp_last = (int)((((int64_t)(chunk0 + nb) * Geo::KC) - 1) >> p.g_shift);
        const int ngrp = grp_last - grp0 + 1;
        if (xb > 0) __syncthreads();
        switch (p.x_dtype) {
            case BW_F16: stage_block<BITS, MT, RT, WARPS, TWO_GROUPS, __half>(p, chunk0, nb, n0, xs, gc, grp0, ngrp); break;
            case BW_BF16: stage_block<BITS, MT, RT, WARPS, TWO_GROUPS, __nv_bfloat16>(p, chunk0, nb, n0, xs, gc, grp0, ngrp); break;
            default: stage_block<BITS, MT, RT, WARPS, TWO_GROUPS, float>(p, chunk0, nb, n0, xs, gc, grp0, ngrp); break;
        }
        __syncthreads();

        for (int cl = 0; cl < nb; ++cl) {
            const int i = xb + cl;
            issue(i + STAGES - 1);
            cp_async_wait<STAGES - 1>();
            uint4 wv[SLOTS];
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) wv[s] = myring[((i % STAGES) * SLOTS + s) * 32];

            const int kl = (chunk0 + cl) * Geo::KC + t * Geo::KL;   // first k of this lane's vectors
            const int gl0 = (kl >> p.g_shift) - grp0;
            const int gl1 = TWO_GROUPS ? (((kl + Geo::KL / 2) >> p.g_shift) - grp0) : gl0;
            Dequant<BITS> dq[SLOTS][TWO_GROUPS ? 2 : 1];
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int r = warp * (RT * 16) + (s >> 1) * 16 + (s & 1) * 8 + g;
                dq[s][0].set(gc[gl0 * ROWS + r]);
                if constexpr (TWO_GROUPS) dq[s][1].set(gc[gl1 * ROWS + r]);
            }
            const uint4 *xc = xs + (size_t)cl * Geo::NX * MT * 32 + lane;
            uint4 xq8[MT];   // 8-bit codes: one 16-byte piece feeds two consecutive words
            (void)xq8;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                constexpr int GSEL_DIV = 2;  // words 0,1 -> first group, 2,3 -> second (TWO_GROUPS)
                const int gs = TWO_GROUPS ? (wi / GSEL_DIV) : 0;
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
    cp_async_wait<0>();

    // ---- epilogue ---------------------------------------------------------------------
    auto store_out = [&](int64_t m, int64_t n, float v) {
        if (p.out_dtype == BW_F16) {
            __half c = __float2half_rn(v);                       // the GEMM's fp16 output rounding
            if (p.bias) c = __hadd(c, p.bias[n]);                // separate fp16 bias add
            reinterpret_cast<__half *>(p.out)[m * p.N + n] = c;
        } else {
            if (p.bias) v += __half2float(p.bias[n]);
            if (p.out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[m * p.N + n] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(p.out)[m * p.N + n] = v;
        }
    };

    if (p.splits == 1) {
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int64_t n = (int64_t)n0 + warp * (RT * 16) + rt * 16 + (e >> 1) * 8 + g;
                    const int64_t m = mt * 8 + 2 * t + (e & 1);
                    if (n < p.N && m < p.M) store_out(m, n, acc[rt][mt][e]);
                }
        return;
    }

    // split-K: sum the cluster's partial tiles through distributed shared memory
    cg::cluster_group cluster = cg::this_cluster();
    float *red = reinterpret_cast<float *>(xs);       // [MTOK][ROWS], reuses the activation area
    __syncthreads();                                  // every warp is done reading xs / gc
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = warp * (RT * 16) + rt * 16 + (e >> 1) * 8 + g;
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
            float v = acc[j];
            const int64_t m = m0 + j;
            if (p.out_dtype == BW_F16) {
                __half c = __float2half_rn(v);
                if (p.bias) c = __hadd(c, p.bias[n]);
                reinterpret_cast<__half *>(p.out)[m * p.N + n] = c;
            } else {
                if (p.bias) v += __half2float(p.bias[n]);
                if (p.out_dtype == BW_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[m * p.N + n] = __float2bfloat16_rn(v);
                else reinterpret_cast<float *>(p.out)[m * p.N + n] = v;
            }
        }
    }
}

template <int BITS, int MT, int RT, int WARPS, bool TWO_GROUPS>
int launch_cfg(SmallMParams p, cudaStream_t st) {
    using Geo = Geometry<BITS>;
    constexpr int ROWS = WARPS * RT * 16;
    constexpr int MTOK = MT * 8;
    auto kern = qmm_smallm_kernel<BITS, MT, RT, WARPS, TWO_GROUPS>;
    const int g = 1 << p.g_shift;
    // shared memory: weight ring + activation block + group constants (or the reduction tile)
    const size_t ring_bytes = (size_t)WARPS * STAGES * 2 * RT * 32 * 16;
    const size_t x_per_chunk = (size_t)Geo::NX * MT * 32 * 16;
    const size_t gc_per_chunk = (size_t)((Geo::KC + g - 1) / g + 1) * ROWS * sizeof(GroupConst);
    const size_t red_bytes = (size_t)MTOK * ROWS * sizeof(float);
    const size_t budget = 96 * 1024;
    int xblock = p.chunks_per_cta;
    while (xblock > 1 && ring_bytes + xblock * (x_per_chunk + gc_per_chunk) > budget) --xblock;
    p.xblock = xblock;
    size_t xs_bytes = xblock * x_per_chunk;
    size_t tail = xblock * gc_per_chunk;
    if (xs_bytes + tail < red_bytes) tail = red_bytes - xs_bytes;
    const size_t smem = ring_bytes + xs_bytes + tail;
    static size_t configured[64] = {};   // per instantiation and device; grows monotonically
    int dev = 0;
    BW_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
        BW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.N + ROWS - 1) / ROWS), (unsigned)p.splits, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)p.splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    return BW_OK;
}

template <int BITS, int MT, bool TWO_GROUPS>
int launch_rows(const SmallMParams &p, int rt, int warps, cudaStream_t st) {
    if constexpr (TWO_GROUPS) return launch_cfg<BITS, MT, 1, 4, TWO_GROUPS>(p, st);
    if (rt == 1 && warps == 4) return launch_cfg<BITS, MT, 1, 4, TWO_GROUPS>(p, st);
    if (rt == 2 && warps == 4) return launch_cfg<BITS, MT, 2, 4, TWO_GROUPS>(p, st);
    if constexpr (MT <= 2) {
        if (rt == 2 && warps == 8) return launch_cfg<BITS, MT, 2, 8, TWO_GROUPS>(p, st);
        if (rt == 1 && warps == 8) return launch_cfg<BITS, MT, 1, 8, TWO_GROUPS>(p, st);
    }
    return launch_cfg<BITS, MT, 1, 4, TWO_GROUPS>(p, st);
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

// Tuning override for experiments: rows-tiles per warp, warps per CTA, split-K factor
// (0 = automatic).  Not part of the C ABI.
struct SmallMTuning { int rt, warps, splits; };
static SmallMTuning g_tuning = {0, 0, 0};
void set_smallm_tuning(int rt, int warps, int splits) { g_tuning = {rt, warps, splits}; }

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

// Runs one launch of the streaming kernel for up to 64 tokens (the caller loops over token
// blocks), or the general kernel when the layout preconditions do not hold.
int qmatmul_smallm(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                   const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype,
                   int bits, int g, cudaStream_t st) {
    if (M == 0 || N == 0) return BW_OK;
    SmallMParams p = {};
    p.x = x; p.q = q; p.scale = scale; p.zp = zp; p.bias = bias; p.out = out;
    p.M = M; p.N = N; p.K = K; p.x_dtype = x_dtype; p.out_dtype = out_dtype;
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
    const int vpi = 32 / bits, kc = 16 * vpi;
    int gs = 0;
    while ((1 << gs) < g) ++gs;
    p.g_shift = gs;
    p.chunks_total = (int)((K + kc - 1) / kc);
    const bool two_groups = g < 4 * vpi;
    const int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));

    int rt = g_tuning.rt, warps = g_tuning.warps, splits = g_tuning.splits;
    if (rt == 0 || warps == 0) {
        if (mt >= 4) { rt = 1; warps = 4; }
        else if (N >= 2048) { rt = 2; warps = 4; }
        else { rt = 1; warps = 4; }
    }
    const int rows = rt * warps * 16;
    const int row_blocks = (int)((N + rows - 1) / rows);
    if (splits == 0) {
        splits = (296 + row_blocks - 1) / row_blocks;
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
