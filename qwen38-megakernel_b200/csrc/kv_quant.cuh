// Device-side quantizer of one K / V row, one warp per row: lane l holds values 8 l .. 8 l + 7, a 32-value block is the four
// lanes of a quad (lanes 4 j .. 4 j + 3). The stored bytes are the reference's (qwen38_mk.cu:2003-2097) bit for bit; the
// golden vectors under tests/golden/ pin them. What the format fixes is the fp32 arithmetic of the scale and of the index
// (every such operation below is an explicitly rounded intrinsic, so no compiler flag can change a byte) and the byte layout;
// how the block's extreme value is found and how the bytes are assembled is this file's own:
//   - magnitudes are compared as the integer bit patterns of |v| (same order as the floats for finite values) and reduced over
//     the quad with one redux.sync;
//   - the signed extreme of a 4 .. 7-bit block ("largest magnitude, ties to the larger value") is +max if any value of the block
//     equals +max, else -max, found with one quad vote;
//   - indices are packed four to a word with byte permutes, nibbles and high-bit fields are cut out of those words.
#pragma once
#include <cuda_fp16.h>

#include "kv_format.h"

namespace mkkv {

constexpr unsigned FULL = 0xffffffffu;

// the lanes of this lane's quad, as a member mask
__device__ __forceinline__ unsigned quad_mask(int lane) { return 0xfu << (lane & 28); }

// 256-point Walsh-Hadamard transform x 1/16 (orthonormal, self-inverse). fp32 sums do not commute in rounding, so the stage
// order is the format's (qwen38_mk.cu:2049-2069): index bits 1, 2, 4 inside the lane, then lane bits 1 .. 16; in every stage the
// element whose bit is clear becomes a + b, the other a - b with a the clear-bit element. Across lanes that is
// partner + own for a clear lane bit and partner - own = partner + (-own) for a set one: one add of a sign-adjusted value.
__device__ __forceinline__ void fwht256(float (&v)[8], int lane) {
#pragma unroll
    for (int stride = 1; stride < 8; stride *= 2)
#pragma unroll
        for (int base = 0; base < 8; base += 2 * stride)
#pragma unroll
            for (int j = base; j < base + stride; j++) {
                const float lo = v[j], hi = v[j + stride];
                v[j] = __fadd_rn(lo, hi);
                v[j + stride] = __fsub_rn(lo, hi);
            }
#pragma unroll
    for (int bit = 1; bit < 32; bit *= 2) {
        const unsigned flip = (lane & bit) ? 0x80000000u : 0u; // own value enters negated where the lane bit is set
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float partner = __shfl_xor_sync(FULL, v[k], bit);
            v[k] = __fadd_rn(partner, __uint_as_float(__float_as_uint(v[k]) ^ flip));
        }
    }
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = __fmul_rn(v[k], 0.0625f);
}

// bit pattern of the block's largest magnitude (the block: this lane's quad)
__device__ __forceinline__ unsigned block_absmax_bits(const float (&v)[8], int lane) {
    unsigned m = 0u;
#pragma unroll
    for (int k = 0; k < 8; k++) m = max(m, __float_as_uint(v[k]) & 0x7fffffffu);
    return __reduce_max_sync(quad_mask(lane), m);
}
// four small non-negative integers (each < 256) as the bytes of one word, a in the lowest
__device__ __forceinline__ unsigned bytes4(int a, int b, int c, int d) {
    return __byte_perm(__byte_perm((unsigned) a, (unsigned) b, 0x0040), __byte_perm((unsigned) c, (unsigned) d, 0x0040), 0x5410);
}

// q8_0 row (qwen38_mk.cu:2005-2023): q = rint(v * (127 / absmax)) to even, scale = half(absmax / 127)
__device__ __forceinline__ void store_q8(uint8_t * q, uint16_t * sc, const float (&v)[8], int lane) {
    const float am = __uint_as_float(block_absmax_bits(v, lane));
    const float inv = am > 0.f ? __fdiv_rn(127.0f, am) : 0.f;
    int n[8];
#pragma unroll
    for (int k = 0; k < 8; k++) n[k] = __float2int_rn(__fmul_rn(v[k], inv)) & 0xff; // two's-complement byte
    *reinterpret_cast<uint2 *>(q + lane * 8) = make_uint2(bytes4(n[0], n[1], n[2], n[3]), bytes4(n[4], n[5], n[6], n[7]));
    if ((lane & 3) == 0) sc[lane >> 2] = __half_as_ushort(__float2half_rn(__fdiv_rn(am, 127.0f)));
}

// 4 .. 7-bit row (qwen38_mk.cu:2029-2046, 2075-2097): d = (value of largest magnitude, ties to the larger value) / -2^(bits-1),
// index n = min(2^bits - 1, trunc(fma(v, 1 / d, 2^(bits-1) + 0.5))). Bytes 0 .. 127: lane word of low nibbles (values 0 .. 3 in the
// low, 4 .. 7 in the high nibbles of bytes 0 .. 3); then bits - 4 bytes per lane of high bits, value k at bit (bits - 4) k.
__device__ __forceinline__ void store_qn(uint8_t * q, uint16_t * sc, const float (&v)[8], int bits, int lane) {
    const int half_range = 1 << (bits - 1), hb = bits - 4;
    const unsigned am_bits = block_absmax_bits(v, lane);
    bool has_pos = false; // does the block hold +max itself?
#pragma unroll
    for (int k = 0; k < 8; k++) has_pos |= __float_as_uint(v[k]) == am_bits;
    const bool any_pos = (__ballot_sync(FULL, has_pos) & quad_mask(lane)) != 0u;
    // an all-zero block keeps the search's initial +0 whatever the zeros' signs, so its scale is -0 (+0 / -2^(bits-1))
    const float extreme = __uint_as_float(am_bits == 0u || any_pos ? am_bits : am_bits | 0x80000000u);
    const float d = __fdiv_rn(extreme, (float) -half_range), inv = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
    const float offset = (float) half_range + 0.5f;
    int n[8];
#pragma unroll
    for (int k = 0; k < 8; k++) n[k] = min(2 * half_range - 1, (int) __fmaf_rn(v[k], inv, offset));
    const unsigned first = bytes4(n[0], n[1], n[2], n[3]), second = bytes4(n[4], n[5], n[6], n[7]); // one index per byte
    *reinterpret_cast<unsigned *>(q + lane * 4) = (first & 0x0f0f0f0fu) | ((second & 0x0f0f0f0fu) << 4);
    if (hb > 0) {
        const unsigned top[2] = {(first >> 4) & 0x0f0f0f0fu, (second >> 4) & 0x0f0f0f0fu}; // the indices' bits 4 and up, one per byte
        unsigned field = 0u;
#pragma unroll
        for (int k = 0; k < 8; k++) field |= ((top[k >> 2] >> (8 * (k & 3))) & 0xfu) << (hb * k);
        uint8_t * dst = q + 128 + lane * hb;
        for (int b = 0; b < hb; b++) dst[b] = (uint8_t) (field >> (8 * b));
    }
    if ((lane & 3) == 0) sc[lane >> 2] = __half_as_ushort(__float2half_rn(d));
}

__device__ __forceinline__ void store_row(uint8_t * q, uint16_t * sc, const float (&v)[8], int bits, int lane) {
    if (bits == 8) store_q8(q, sc, v, lane);
    else store_qn(q, sc, v, bits, lane);
}

// the integers of lane word `lane` of a row (8 values): int8 for 8 bits, else n - 2^(bits-1) (qwen38_mk.cu:2336-2343,2458-2468)
__device__ __forceinline__ void row_ints(const uint8_t * row, int bits, int lane, int (&q)[8]) {
    if (bits == 8) {
        const uint2 w = *reinterpret_cast<const uint2 *>(row + lane * 8);
#pragma unroll
        for (int k = 0; k < 8; k++) q[k] = (int) (int8_t) ((k < 4 ? w.x : w.y) >> (8 * (k & 3)));
        return;
    }
    const unsigned wd = *reinterpret_cast<const unsigned *>(row + lane * 4);
    const int hb = bits - 4, mid = 1 << (bits - 1);
    unsigned hi = 0;
    for (int k = 0; k < hb; k++) hi |= (unsigned) row[128 + lane * hb + k] << (8 * k);
    const unsigned m = (1u << hb) - 1u;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const unsigned byte = (wd >> (8 * (k & 3))) & 0xffu, nib = k < 4 ? (byte & 0xfu) : (byte >> 4);
        q[k] = (int) (nib | (((hi >> (hb * k)) & m) << 4)) - mid;
    }
}

} // namespace mkkv
