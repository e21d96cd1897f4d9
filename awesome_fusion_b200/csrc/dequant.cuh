// In-register unpack of packed int8 / int4 weights to exact bf16 pairs.
//
// The reference kernel splices each byte into the mantissa of 2^23 and subtracts
// 2^23 + 128 in fp32 (bf16gemm_kernel_gfx90a.s:18-27, constants :204-210).  bf16 has an
// 8-bit significand, so on sm_100a the same idea is done directly in packed bf16:
//   int8:  v = (v & 0x7f) - 128 * bit7.   0x4300 | (v & 0x7f) is the bf16 128 + (v & 0x7f)
//          and 0xC300 | (v & 0x80) is the bf16 -128 (bit7 = 0) or -256 (bit7 = 1); their
//          bf16 sum is the exact integer v.  Two weights per 32-bit lane operation.
//   int4:  0x4300 | (q ^ 8) is the bf16 128 + (q + 8); subtracting 136 gives q exactly.
// All results are integers of magnitude <= 128, exactly representable in bf16.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>
#include "afb_capi.h"

namespace afb {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// (a & b) | c
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// (a & b) ^ c
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// x holds two two's-complement int8 values in bits [0,8) and [16,24) (other bits ignored).
// Returns the two exact bf16 values, low half = the value from bits [0,8).
__device__ __forceinline__ uint32_t s8pair_to_bf16x2(uint32_t x) {
    const uint32_t lo = lop3_and_or(x, 0x007f007fu, 0x43004300u);  // 128 + (v & 0x7f)
    const uint32_t hi = lop3_and_or(x, 0x00800080u, 0xC300C300u);  // -128 - 128 * bit7
    return bf16x2_add(lo, hi);
}

// Four consecutive int8 (two's complement) of word w -> {k0,k1} and {k2,k3} as bf16x2.
__device__ __forceinline__ void s8x4_to_bf16_natural(uint32_t w, uint32_t& p01, uint32_t& p23) {
    p01 = s8pair_to_bf16x2(prmt(w, 0u, 0x4140u));
    p23 = s8pair_to_bf16x2(prmt(w, 0u, 0x4342u));
}
// Same bytes, cheaper pairing: {k0,k2} and {k1,k3} (the consumer permutes its other operand).
__device__ __forceinline__ void s8x4_to_bf16_strided(uint32_t w, uint32_t& p02, uint32_t& p13) {
    p02 = s8pair_to_bf16x2(w);
    p13 = s8pair_to_bf16x2(w >> 8);
}

// The same for either storage encoding without a separate flip: `hi` = 0xC300C300 (two's complement) or 0xC380C380 (value + 128).
// With value + 128 the top bit is inverted, so the sign half is -256 + 128 * bit7 = the bf16 pattern 0xC380 with bit 7 toggled off.
__device__ __forceinline__ uint32_t s8pair_enc_to_bf16x2(uint32_t x, uint32_t hi) {
    const uint32_t lo = lop3_and_or(x, 0x007f007fu, 0x43004300u);   // 128 + (v & 0x7f)
    return bf16x2_add(lo, lop3_and_xor(x, 0x00800080u, hi));         // two's complement: -128 - 128 * bit7; offset: -256 + 128 * bit7
}
__device__ __forceinline__ void s8x4_enc_to_bf16_strided(uint32_t w, uint32_t hi, uint32_t& p02, uint32_t& p13) {
    p02 = s8pair_enc_to_bf16x2(w, hi);
    p13 = s8pair_enc_to_bf16x2(w >> 8, hi);
}

// magic = 0x43084308 for two's-complement nibbles, 0x43004300 for offset-binary (+8) nibbles.
// x holds two nibbles in bits [0,4) and [16,20) (other bits ignored) -> two exact bf16.
// `sub` is the packed-bf16 constant that is subtracted: 136 without zero-points, 136 + zero with them (the same instruction).
__device__ __forceinline__ uint32_t s4pair_to_bf16x2(uint32_t x, uint32_t magic, uint32_t sub = 0x43084308u) {
    return bf16x2_sub(lop3_and_xor(x, 0x000f000fu, magic), sub);
}
// Eight consecutive nibbles of w (k0 in bits [0,4)) -> {k0,k1},{k2,k3},{k4,k5},{k6,k7}.
__device__ __forceinline__ void s4x8_to_bf16_natural(uint32_t w, uint32_t magic, uint32_t p[4], uint32_t sub = 0x43084308u) {
    const uint32_t sh = w >> 4;
    p[0] = s4pair_to_bf16x2(prmt(w, sh, 0x0400u), magic, sub);
    p[1] = s4pair_to_bf16x2(prmt(w, sh, 0x0501u), magic, sub);
    p[2] = s4pair_to_bf16x2(prmt(w, sh, 0x0602u), magic, sub);
    p[3] = s4pair_to_bf16x2(prmt(w, sh, 0x0703u), magic, sub);
}
// Cheaper pairing: {k0,k4},{k1,k5},{k2,k6},{k3,k7}.
__device__ __forceinline__ void s4x8_to_bf16_strided(uint32_t w, uint32_t magic, uint32_t p[4], uint32_t sub = 0x43084308u) {
    p[0] = s4pair_to_bf16x2(w, magic, sub);
    p[1] = s4pair_to_bf16x2(w >> 4, magic, sub);
    p[2] = s4pair_to_bf16x2(w >> 8, magic, sub);
    p[3] = s4pair_to_bf16x2(w >> 12, magic, sub);
}

// Consecutive-k pairs {k0,k1},{k2,k3} of a word, whichever way the word is laid out: plain [k0,k1,k2,k3] needs two byte
// permutes, the pre-packed order [k0,k2,k1,k3] (afb_prepack) is what the cheap routine reads as pairs.
__device__ __forceinline__ void s8x4_to_bf16_pairs(uint32_t w, bool packed, uint32_t& p01, uint32_t& p23) {
    if (packed) s8x4_to_bf16_strided(w, p01, p23);
    else s8x4_to_bf16_natural(w, p01, p23);
}
__device__ __forceinline__ void s4x8_to_bf16_pairs(uint32_t w, uint32_t magic, bool packed, uint32_t p[4], uint32_t sub = 0x43084308u) {
    if (packed) s4x8_to_bf16_strided(w, magic, p, sub);
    else s4x8_to_bf16_natural(w, magic, p, sub);
}
// Zero-points: a byte in the weights' own encoding -> the packed-bf16 constant the unpack subtracts.
//   int8: the decoded zero itself, both halves (one extra sub.bf16x2 per pair; |q - z| <= 255 is exact in bf16);
//   int4: 136 + decoded zero, which takes the place of the 136 the unpack subtracts anyway (no extra instruction).
__device__ __forceinline__ uint32_t zero8_const(uint32_t zbyte, uint32_t enc) {
    const int z = enc == AFB_ENC_OFFSET_BINARY ? (int)zbyte - 128 : (int)(int8_t)zbyte;
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)z)) * 0x00010001u;
}
__device__ __forceinline__ uint32_t zero4_const(uint32_t zbyte, uint32_t enc) {
    const int nib = (int)(zbyte & 0xFu);
    const int z = enc == AFB_ENC_OFFSET_BINARY ? nib - 8 : ((nib ^ 8) - 8);
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn((float)(136 + z))) * 0x00010001u;
}
// Place of weight k inside its word in the pre-packed layout (int8: bytes [k0,k2,k1,k3]; int4: nibbles [k0,k2,k4,k6,k1,k3,k5,k7]).
__host__ __device__ __forceinline__ uint32_t packed_pos(uint32_t bits, uint32_t k) {
    if (bits == 8) { const uint32_t i = k & 3u; return (k & ~3u) | ((i >> 1) | ((i & 1u) << 1)); }
    const uint32_t i = k & 7u;
    return (k & ~7u) | ((i >> 1) | ((i & 1u) << 2));
}

__device__ __forceinline__ uint32_t bf16_dup(uint16_t s) { return (uint32_t)s * 0x00010001u; }

}  // namespace afb
