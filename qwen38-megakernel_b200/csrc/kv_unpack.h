// Integer unpacking of packed KV rows and the fragment index maps of the fast decode-attention kernel.
// Everything here is plain integer arithmetic usable from host and device, so the maps can be checked on the CPU.
//
// Row formats (qwen38_mk.cu:2071-2097): a b-bit row (b = 4 .. 7) is 32 lane words (word w: the low nibbles of values
// 8 w .. 8 w + 3 in the low and of values 8 w + 4 .. 8 w + 7 in the high nibbles of its 4 bytes) followed by b - 4 bytes per
// word of high bits (value k of the word at bit (b - 4) k); an 8-bit row is 256 int8 values. "Biased byte" below is the index
// n = q + 2^(b-1) (b < 8) or q + 128 (b = 8): the kernels turn it into fp16 with one PRMT and subtract the bias there.
#pragma once
#include "kv_format.h"

namespace mkkv {

// the four HB-bit fields k = 0 .. 3 of x (field k at bit HB k) moved to bits 4 .. 4 + HB - 1 of byte k
template <int HB> MKKV_HD unsigned spread4(unsigned x) {
    if constexpr (HB == 1) return ((x & 0xfu) * 0x02040810u) & 0x10101010u;
    if constexpr (HB == 2) {
        x = ((x & 0xffu) * 0x10010u) & 0x00f000f0u;
        return (x * 0x41u) & 0x30303030u;
    }
    if constexpr (HB == 3) {
        x &= 0xfffu;
        x = (x | (x << 10)) & 0x003f003fu;
        x = (x | (x << 5)) & 0x07070707u;
        return x << 4;
    }
    return 0u;
}

// Values 4 half .. 4 half + 3 of one lane word (half = 0: low nibbles, 1: high nibbles) as four biased bytes.
// word: the lane word; hi: the word's high bits (8 HB bits, value k at bit HB k)
template <int HB> MKKV_HD unsigned quad_bytes(unsigned word, unsigned hi, int half) {
    unsigned x = (word >> (4 * half)) & 0x0f0f0f0fu;
    if constexpr (HB > 0) x |= spread4<HB>(hi >> (4 * HB * half));
    return x;
}

// ---- fragment maps of the fast kernel (mma.sync m16n8k16; lane = 4 g8 + tig) ----
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
