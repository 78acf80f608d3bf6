// Integer unpacking of packed KV rows, usable from host and device so that every map can be checked on the CPU.
//
// Row formats (qwen38_mk.cu:2071-2097): a b-bit row (b = 4 .. 7) is 32 lane words (word w: the low nibbles of values
// 8 w .. 8 w + 3 in the low and of values 8 w + 4 .. 8 w + 7 in the high nibbles of its 4 bytes) followed by b - 4 bytes per
// word of high bits (value k of the word at bit (b - 4) k); an 8-bit row is 256 int8 values.
//
// Two unpackers live here.
//
// 1. pair_words: the tensor-core kernel's. The 8 values of one lane word become four fp16 PAIRS, assembled directly as the
//    bit patterns of (bias + n) without building bytes first: a nibble that sits at bits 0 .. 3 of a 16-bit half is OR-ed
//    under the exponent of 1024 (0x6400: one mantissa step = 1), a nibble at bits 4 .. 7 under the exponent of 64 (0x5400:
//    one mantissa step = 1/16, so the nibble's steps are again whole numbers). The high bits of a value land right above its
//    nibble. One AND-OR gives a pair; the kernel then subtracts (bias + 2^(b-1)) and multiplies by the scale, both in fp16
//    pairs, which reproduces fp16(d * q) with a single rounding. The pairs come out in the order
//        (v0, v2) (v4, v6) (v1, v3) (v5, v7)
//    i.e. position j of the 8-value unit holds value UNIT_PERM[j]; queries are staged in the same order and the output
//    dims of P V are mapped back through it.
//
// 2. quad_bytes: the mma.sync kernel's: four values as four index bytes n (the kernel turns them into fp16 with a byte
//    permute).
#pragma once
#include "kv_format.h"

namespace mkkv {

// value index held at position j of an unpacked 8-value unit
constexpr int UNIT_PERM[8] = {0, 2, 4, 6, 1, 3, 5, 7};
MKKV_HD int unit_perm(int j) { return ((j & 3) << 1) | (j >> 2); }

constexpr unsigned MAGIC_A = 0x64006400u; // pair of 1024.0
constexpr unsigned MAGIC_B = 0x54005400u; // pair of 64.0
constexpr unsigned NIB_A = 0x000f000fu;   // the nibbles under MAGIC_A
constexpr unsigned NIB_B = 0x00f000f0u;   // the nibbles under MAGIC_B

// what the kernel subtracts from an A / B pair of a BITS-bit row: bias + 2^(BITS-1), as an fp16 pair
template <int BITS> MKKV_HD unsigned pair_sub_a() { return MAGIC_A + (BITS < 8 ? (0x00010001u << (BITS - 1)) : 0x00800080u); }
template <int BITS> MKKV_HD unsigned pair_sub_b() { return MAGIC_B + (0x00100010u << (BITS - 1)); }
// 7- and 8-bit rows use the 1024 bias for every pair (their indices do not fit under 64)
template <int BITS> MKKV_HD bool pair_is_a(int p) { return BITS >= 7 || !(p & 1); }

// Lane word `word` of a 4 .. 6-bit row and its high bits -> the four pairs. hi: BITS == 5: the word's byte of high bits (bit k:
// value k), no other bit set; BITS == 6: its 16 bits (bits 2 k, 2 k + 1: value k), higher bits are ignored.
template <int BITS> MKKV_HD void pair_words(unsigned word, unsigned hi, unsigned (&x)[4]) {
    static_assert(BITS >= 4 && BITS <= 6, "pair_words: 4 .. 6 bits");
    const unsigned w8 = word >> 8;
    unsigned y0 = MAGIC_A, y1 = MAGIC_B, y2 = MAGIC_A, y3 = MAGIC_B;
    if constexpr (BITS == 5) {
        // hi * (2^4 + 2^18): bit k of hi at 4 + k and at 18 + k; the copy shifted down by one serves the odd values
        const unsigned t = hi * 0x00040010u, t1 = hi * 0x00020008u;
        y0 |= t & 0x00100010u;  // value 0 -> bit 4, value 2 -> bit 20
        y1 |= t & 0x01000100u;  // value 4 -> bit 8, value 6 -> bit 24
        y2 |= t1 & 0x00100010u; // values 1, 3
        y3 |= t1 & 0x01000100u; // values 5, 7
    } else if constexpr (BITS == 6) {
        // even values' fields at bits 0, 4, 8, 12 of he, odd values' of ho; the gaps keep the shifted copies' sums apart
        const unsigned he = hi & 0x3333u, ho = (hi >> 2) & 0x3333u;
        y0 |= (he * 0x00010010u) & 0x00300030u; // value 0 -> bits 4-5, value 2 -> bits 20-21
        y1 |= (he * 0x00001001u) & 0x03000300u; // value 4 -> bits 8-9, value 6 -> bits 24-25
        y2 |= (ho * 0x00010010u) & 0x00300030u;
        y3 |= (ho * 0x00001001u) & 0x03000300u;
    }
    x[0] = (word & NIB_A) | y0;
    x[1] = (word & NIB_B) | y1;
    x[2] = (w8 & NIB_A) | y2;
    x[3] = (w8 & NIB_B) | y3;
}
// 7-bit rows: every pair under the 1024 bias; hi: the word's 24 bits (bits 3 k .. 3 k + 2: value k)
MKKV_HD void pair_words7(unsigned word, unsigned hi, unsigned (&x)[4]) {
    x[0] = (word & NIB_A) | ((hi << 4) & 0x70u) | ((hi << 14) & 0x700000u) | MAGIC_A;          // values 0, 2
    x[1] = ((word >> 4) & NIB_A) | ((hi >> 8) & 0x70u) | ((hi << 2) & 0x700000u) | MAGIC_A;    // values 4, 6
    x[2] = ((word >> 8) & NIB_A) | ((hi << 1) & 0x70u) | ((hi << 11) & 0x700000u) | MAGIC_A;   // values 1, 3
    x[3] = ((word >> 12) & NIB_A) | ((hi >> 11) & 0x70u) | ((hi >> 1) & 0x700000u) | MAGIC_A;  // values 5, 7
}
// 8-bit rows: the 8 int8 values of a unit (lo: values 0 .. 3, hi: 4 .. 7) with the sign bit flipped (q + 128) under the 1024 bias.
// (On the device the byte moves are one PRMT each.)
MKKV_HD unsigned byte_pair(unsigned w, int a, int b) { return ((w >> (8 * a)) & 0xffu) | (((w >> (8 * b)) & 0xffu) << 16) | MAGIC_A; }
MKKV_HD void pair_words8(unsigned lo, unsigned hi, unsigned (&x)[4]) {
    lo ^= 0x80808080u;
    hi ^= 0x80808080u;
    x[0] = byte_pair(lo, 0, 2);
    x[1] = byte_pair(hi, 0, 2);
    x[2] = byte_pair(lo, 1, 3);
    x[3] = byte_pair(hi, 1, 3);
}

// ---- the mma.sync kernel's byte form ----
// Values 4 half .. 4 half + 3 of one lane word (half = 0: low nibbles, 1: high nibbles) as four index bytes n.
// word: the lane word; hi: the word's high bits (8 HB bits, value k at bit HB k)
template <int HB> MKKV_HD unsigned quad_bytes(unsigned word, unsigned hi, int half) {
    unsigned x = (word >> (4 * half)) & 0x0f0f0f0fu;
    if constexpr (HB > 0) {
        const unsigned f = hi >> (4 * HB * half), m = (1u << HB) - 1u;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int k = 0; k < 4; k++) x |= ((f >> (HB * k)) & m) << (8 * k + 4);
    }
    return x;
}

// ---- fragment maps of the mma.sync kernel (m16n8k16; lane = 4 g8 + tig) ----
// S = Q K^T of one 32-position tile: n-tile nt (0 .. 3) holds positions 8 nt + pos_of_n(n), n = 0 .. 7. The permutation lets
// the P V loads of four consecutive lanes (tig = 0 .. 3) hit rows that differ mod 4 (different shared-memory banks for
// 160-byte rows) while a lane still owns pairs (n, n + 1) of adjacent MMA indices.
MKKV_HD int pos_of_n(int n) { return n < 4 ? n : (n ^ 1); } // 0 1 2 3 5 4 7 6
// The K value quadruple of MMA k-step ks = 4 G + s (G = 0 .. 3, s = 0 .. 3) held by lane (g8, tig): dims
// 64 G + 16 tig + 4 s .. + 3 of position 8 nt + pos_of_n(g8); b0 = (v0, v1), b1 = (v2, v3). The query fragment of the same lane
// is the same four dims of rows g8 and g8 + 8 (one 8-byte load each).
MKKV_HD int k_dim0(int G, int s, int tig) { return 64 * G + 16 * tig + 4 * s; }
// P V of one 32-position tile, k-step ks (0, 1) covers MMA columns 16 ks .. 16 ks + 15 of the P tile; MMA k index
// x = 2 tig + j + 8 h is column 16 ks + x, i.e. position 16 ks + 8 h + pos_of_n(2 tig + j). A P V warp owns 32 dims (dg);
// lane g8 holds the four values 4 (g8 & 1) .. + 3 of lane word 4 dg + (g8 >> 1), value v going to n-tile v:
MKKV_HD int v_dim(int dg, int g8, int v) { return 32 * dg + 8 * (g8 >> 1) + 4 * (g8 & 1) + v; }

} // namespace mkkv
