// Code extraction shared by the quantized-matmul kernels: packed int32 words -> fp16 weights
// W = fp16(scale * (code - zero_point)), bit-identical to the reference's dequantized weights
// (bitween/modules.py:55-58).  Codes are turned into 1024+code (or 1024 + 4^j*code for the
// higher fields) with one lop3/prmt, the zero-point is removed with an exact fp16 subtract or
// FMA, and one fp16 multiply by the scale performs the single rounding.
#pragma once
#include "bw_common.cuh"

namespace bw {

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return d;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// Per-(row, group) dequantization constants kept in shared memory: {scale,scale} and
// {1024+zp, 1024+zp} as half2 pairs.
struct GroupConst { uint32_t s2, z1024; };

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

// (lo16 of x, lo16 of y) and (hi16 of x, hi16 of y)
__device__ __forceinline__ uint32_t pair_lo(uint32_t x, uint32_t y) { return __byte_perm(x, y, 0x5410); }
__device__ __forceinline__ uint32_t pair_hi(uint32_t x, uint32_t y) { return __byte_perm(x, y, 0x7632); }

}  // namespace bw
