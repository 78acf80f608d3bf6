// Device-side quantizer of one K / V row, one warp per row: lane l holds values 8 l .. 8 l + 7, a 32-value block is lanes
// 4 j .. 4 j + 3. Bytes and rounding follow the reference exactly (qwen38_mk.cu:2003-2097): every fp32 operation below is
// an explicitly rounded intrinsic so no compiler flag can change a stored byte.
#pragma once
#include <cuda_fp16.h>

#include "kv_format.h"

namespace mkkv {

constexpr unsigned FULL = 0xffffffffu;

// 256-point Walsh-Hadamard transform x 1/16 (orthonormal, self-inverse): the in-lane index bits first, then the lane
// bits, the same butterfly order as qwen38_mk.cu:2049-2069 (fp32 sums do not commute in rounding)
__device__ __forceinline__ void fwht256(float (&v)[8], int lane) {
#pragma unroll
    for (int m = 1; m < 8; m <<= 1)
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (!(k & m)) {
                const float a = v[k], b = v[k | m];
                v[k] = __fadd_rn(a, b);
                v[k | m] = __fsub_rn(a, b);
            }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1)
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float o = __shfl_xor_sync(FULL, v[k], m);
            v[k] = (lane & m) ? __fsub_rn(o, v[k]) : __fadd_rn(v[k], o);
        }
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = __fmul_rn(v[k], 0.0625f);
}

// q8_0 row (qwen38_mk.cu:2005-2023): q = rint(v * (127 / absmax)) to even, scale = half(absmax / 127)
__device__ __forceinline__ void store_q8(uint8_t * q, uint16_t * sc, const float (&v)[8], int lane) {
    float am = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) am = fmaxf(am, fabsf(v[k]));
    am = fmaxf(am, __shfl_xor_sync(FULL, am, 1));
    am = fmaxf(am, __shfl_xor_sync(FULL, am, 2));
    const float id = am > 0.f ? __fdiv_rn(127.0f, am) : 0.f;
    unsigned w[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        unsigned x = 0;
#pragma unroll
        for (int k = 0; k < 4; k++) x |= ((unsigned) __float2int_rn(__fmul_rn(v[4 * h + k], id)) & 0xffu) << (8 * k);
        w[h] = x;
    }
    *reinterpret_cast<uint2 *>(q + lane * 8) = make_uint2(w[0], w[1]);
    if ((lane & 3) == 0) sc[lane >> 2] = __half_as_ushort(__float2half_rn(__fdiv_rn(am, 127.0f)));
}

// 4 .. 7-bit row (qwen38_mk.cu:2029-2046, 2075-2097): d = (value of largest magnitude, ties to the larger value) / -2^(bits-1),
// index n = min(2^bits - 1, trunc(fma(v, 1 / d, 2^(bits-1) + 0.5))). Bytes 0 .. 127: lane word of low nibbles (values 0 .. 3 in the
// low, 4 .. 7 in the high nibbles of bytes 0 .. 3); then bits - 4 bytes per lane of high bits, value k at bit (bits - 4) k.
__device__ __forceinline__ void store_qn(uint8_t * q, uint16_t * sc, const float (&v)[8], int bits, int lane) {
    const int h = 1 << (bits - 1), hb = bits - 4;
    float am = 0.f, sv = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++)
        if (fabsf(v[k]) > am || (fabsf(v[k]) == am && v[k] > sv)) { am = fabsf(v[k]); sv = v[k]; }
#pragma unroll
    for (int m = 1; m <= 2; m <<= 1) {
        const float oa = __shfl_xor_sync(FULL, am, m), os = __shfl_xor_sync(FULL, sv, m);
        if (oa > am || (oa == am && os > sv)) { am = oa; sv = os; }
    }
    const float d = __fdiv_rn(sv, (float) -h), id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
    const float c = (float) h + 0.5f;
    unsigned lo = 0, hi = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const unsigned n = (unsigned) min(2 * h - 1, (int) __fmaf_rn(v[k], id, c));
        lo |= (n & 15u) << (k < 4 ? 8 * k : 8 * (k - 4) + 4);
        hi |= (n >> 4) << (hb * k);
    }
    *reinterpret_cast<unsigned *>(q + lane * 4) = lo;
    for (int k = 0; k < hb; k++) q[128 + lane * hb + k] = (uint8_t) ((hi >> (8 * k)) & 0xffu);
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
    for (int k = 0; k < 8; k++)
        q[k] = (int) (((wd >> (k < 4 ? 8 * k : 8 * (k - 4) + 4)) & 0xfu) | (((hi >> (hb * k)) & m) << 4)) - mid;
}

} // namespace mkkv
