// The unpack step of the tensor-core decode-attention kernel: one thread turns one position x 32 dims of a staged packed tile into
// four 16-byte units of exact fp16(d * q) operand values (kv_unpack.h states the bit assembly in host-checkable form).
#pragma once
#include <cuda_fp16.h>

#include "kv_attend_common.cuh"
#include "kv_unpack.h"

namespace mkkv {
namespace tc {

using namespace attn_common;

// ---- one worker step: position `row` of a staged tile, dims 32 jb .. 32 jb + 31 -> four 16-byte operand units ----
// A unit holds the 8 values of one lane word in the order UNIT_PERM (kv_unpack.h: pair_words and friends are the host-checkable
// statement of what follows). The instructions are chosen by hand -- one AND-OR per pair for the high bits under the bias, one for
// the nibbles, a subtract and a multiply in fp16 pairs -- because the compiler re-associates the plain C form into half as many
// again. raw, dst: shared-space addresses; dst: the thread's unit of dim group 4 (jb & 3) of the slot, the next dim groups are 2048
// bytes apart. valid false (a row past the chunk end holds stale bytes): zeros.
__device__ __forceinline__ unsigned and_or(unsigned a, unsigned mask, unsigned c) { // (a & mask) | c
    unsigned d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(c));
    return d;
}
template <unsigned MASK> __device__ __forceinline__ unsigned and_or_imm(unsigned a, unsigned c) { // (a & MASK) | c, the mask an immediate
    unsigned d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "n"(MASK), "r"(c));
    return d;
}
// fp16(d * q) of a pair held as (bias + n): the difference is exact, the product is rounded once
template <unsigned SUB> __device__ __forceinline__ unsigned pair_val(unsigned x, unsigned d) {
    unsigned r;
    asm("{\n\t.reg .b32 t;\n\tsub.f16x2 t, %1, %2;\n\tmul.f16x2 %0, t, %3;\n\t}" : "=r"(r) : "r"(x), "r"(SUB), "r"(d));
    return r;
}
__device__ __forceinline__ void sts128(unsigned addr, unsigned a, unsigned b, unsigned c, unsigned d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds128(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint2 lds64(unsigned addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned lds32(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned lds16(unsigned addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
    return v;
}
// one unit: the pairs' high-bit words y0 .. y3 (bias included) and the lane word -> four values, stored
template <int BITS> __device__ __forceinline__ void unit_out(unsigned dst, unsigned word, unsigned y0, unsigned y1, unsigned y2, unsigned y3, unsigned d) {
    constexpr unsigned SA = MAGIC_A + (0x00010001u << (BITS - 1)), SB = MAGIC_B + (0x00100010u << (BITS - 1));
    const unsigned w8 = word >> 8;
    sts128(dst, pair_val<SA>(and_or_imm<NIB_A>(word, y0), d), pair_val<SB>(and_or_imm<NIB_B>(word, y1), d),
           pair_val<SA>(and_or_imm<NIB_A>(w8, y2), d), pair_val<SB>(and_or_imm<NIB_B>(w8, y3), d));
}
// the packed bytes of one (position, 32-dim block): lane words, high-bit words, scale pair
template <int BITS> struct PackedBlock {
    unsigned w[BITS == 8 ? 8 : 4]; // 8 bits: the 32 int8 values; else the four lane words
    unsigned h[3];                 // the block's high bits: 4 (5 bits), 8 (6 bits) or 12 bytes (7 bits)
    unsigned d;                    // the block's scale as an fp16 pair (0 for a row past the chunk end)
};
template <int BITS> __device__ __forceinline__ void dq_load(PackedBlock<BITS> & b, unsigned raw, int row, int jb, bool valid) {
    const unsigned sc = valid ? lds16(raw + TILE_SC_OFF + (row * 8 + jb) * 2) : 0u;
    b.d = sc | (sc << 16);
    const unsigned rp = raw + row * (32 * BITS);
    if constexpr (BITS == 8) {
        const uint4 v0 = lds128(rp + 32 * jb), v1 = lds128(rp + 32 * jb + 16);
        b.w[0] = v0.x, b.w[1] = v0.y, b.w[2] = v0.z, b.w[3] = v0.w, b.w[4] = v1.x, b.w[5] = v1.y, b.w[6] = v1.z, b.w[7] = v1.w;
    } else {
        const uint4 nv = lds128(rp + 16 * jb);
        b.w[0] = nv.x, b.w[1] = nv.y, b.w[2] = nv.z, b.w[3] = nv.w;
        if constexpr (BITS == 5) b.h[0] = lds32(rp + 128 + 4 * jb);
        if constexpr (BITS == 6) {
            const uint2 h = lds64(rp + 128 + 8 * jb);
            b.h[0] = h.x, b.h[1] = h.y;
        }
        if constexpr (BITS == 7) b.h[0] = lds32(rp + 128 + 12 * jb), b.h[1] = lds32(rp + 132 + 12 * jb), b.h[2] = lds32(rp + 136 + 12 * jb);
    }
}
template <int BITS> __device__ __forceinline__ void dq_emit(const PackedBlock<BITS> & b, unsigned dst) {
    const unsigned d = b.d;
    if constexpr (BITS == 8) {
        constexpr unsigned S8 = MAGIC_A + 0x00800080u;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const unsigned lo = b.w[2 * u] ^ 0x80808080u, hi = b.w[2 * u + 1] ^ 0x80808080u; // q + 128
            sts128(dst + u * 2048, pair_val<S8>(__byte_perm(lo, MAGIC_A, 0x7270), d), // (value 0, value 2) under the exponent of 1024
                   pair_val<S8>(__byte_perm(hi, MAGIC_A, 0x7270), d),                 // (4, 6)
                   pair_val<S8>(__byte_perm(lo, MAGIC_A, 0x7371), d),                 // (1, 3)
                   pair_val<S8>(__byte_perm(hi, MAGIC_A, 0x7371), d));                // (5, 7)
        }
    } else if constexpr (BITS == 4) {
#pragma unroll
        for (int u = 0; u < 4; u++) unit_out<4>(dst + u * 2048, b.w[u], MAGIC_A, MAGIC_B, MAGIC_A, MAGIC_B, d);
    } else if constexpr (BITS == 5) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            // bit k of the word's byte of high bits at 4 + k and 18 + k; the copy one lower serves the odd values
            const unsigned hb = __byte_perm(b.h[0], 0u, 0x4440 + u), t = hb * 0x00040010u, t1 = hb * 0x00020008u;
            unit_out<5>(dst + u * 2048, b.w[u], and_or_imm<0x00100010u>(t, MAGIC_A), and_or_imm<0x01000100u>(t, MAGIC_B),
                        and_or_imm<0x00100010u>(t1, MAGIC_A), and_or_imm<0x01000100u>(t1, MAGIC_B), d);
        }
    } else if constexpr (BITS == 6) {
        const unsigned hw[4] = {b.h[0], b.h[0] >> 16, b.h[1], b.h[1] >> 16};
#pragma unroll
        for (int u = 0; u < 4; u++) {
            // even values' 2-bit fields at bits 0, 4, 8, 12 of he, odd values' of ho: the gaps keep the shifted copies' sums apart
            const unsigned he = hw[u] & 0x3333u, ho = (hw[u] >> 2) & 0x3333u;
            unit_out<6>(dst + u * 2048, b.w[u], and_or_imm<0x00300030u>(he * 0x00010010u, MAGIC_A), and_or_imm<0x03000300u>(he * 0x00001001u, MAGIC_B),
                        and_or_imm<0x00300030u>(ho * 0x00010010u, MAGIC_A), and_or_imm<0x03000300u>(ho * 0x00001001u, MAGIC_B), d);
        }
    } else { // 7 bits: every pair under the 1024 bias (pair_words7)
        const unsigned hw[4] = {b.h[0], __funnelshift_r(b.h[0], b.h[1], 24), __funnelshift_r(b.h[1], b.h[2], 16), b.h[2] >> 8}; // (bits above 23: not read)
        constexpr unsigned S7 = MAGIC_A + 0x00400040u;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            unsigned x[4];
            pair_words7(b.w[u], hw[u], x);
            sts128(dst + u * 2048, pair_val<S7>(x[0], d), pair_val<S7>(x[1], d), pair_val<S7>(x[2], d), pair_val<S7>(x[3], d));
        }
    }
}
// one block
template <int BITS> __device__ __forceinline__ void dq_item(unsigned raw, int row, int jb, bool valid, unsigned dst) {
    PackedBlock<BITS> b;
    dq_load<BITS>(b, raw, row, jb, valid);
    dq_emit<BITS>(b, dst);
}
} // namespace tc
} // namespace mkkv
