// CPU check of the integer unpackers in csrc/kv_unpack.h (host + device code): for every row format, random packed words decode,
// through the fp16 bit patterns the tensor-core kernel assembles, to the integers the row holds, in the unit order UNIT_PERM.
// Built and run by tests/test_unpack_cpu.py.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "kv_unpack.h"

using namespace mkkv;

// value of an fp16 bit pattern that is a normal number (all patterns met here are)
static double half_val(unsigned h) {
    const int e = (h >> 10) & 31, m = h & 0x3ff;
    double v = (1.0 + m / 1024.0);
    for (int i = 15; i < e; i++) v *= 2;
    for (int i = e; i < 15; i++) v /= 2;
    return (h & 0x8000) ? -v : v;
}
static uint64_t rng = 0x243F6A8885A308D3ull;
static unsigned rnd() {
    rng ^= rng << 13;
    rng ^= rng >> 7;
    rng ^= rng << 17;
    return (unsigned) (rng >> 16);
}
// value k of lane word `word` with high-bit field `hi` (bits HB k ..): the index n
static int index_of(unsigned word, unsigned hi, int hb, int k) {
    const unsigned byte = (word >> (8 * (k & 3))) & 0xff;
    const unsigned nib = k < 4 ? (byte & 15) : (byte >> 4);
    return (int) (nib | (((hi >> (hb * k)) & ((1u << hb) - 1u)) << 4));
}
template <int BITS> static int check_bits() {
    int bad = 0;
    const int hb = BITS - 4;
    for (int it = 0; it < 200000; it++) {
        const unsigned word = rnd(), hi = hb ? rnd() & ((1u << (8 * hb)) - 1u) : 0u;
        unsigned x[4];
        if constexpr (BITS == 7) pair_words7(word, hi | (rnd() << 24), x); // (bits above 23 must be ignored)
        else if constexpr (BITS == 6) pair_words<6>(word, hi | (rnd() << 16), x); // (bits above 15 must be ignored)
        else pair_words<BITS>(word, hi, x);
        for (int j = 0; j < 8; j++) {
            const int p = j >> 1;
            const unsigned h16 = (x[p] >> (16 * (j & 1))) & 0xffff;
            const unsigned sub = pair_is_a<BITS>(p) ? pair_sub_a<BITS>() : pair_sub_b<BITS>();
            const double q = half_val(h16) - half_val(sub & 0xffff);
            const int want = index_of(word, hi, hb, unit_perm(j)) - (1 << (BITS - 1));
            if (q != (double) want) {
                if (bad++ < 5) printf("bits %d word %08x hi %x unit pos %d: got %g want %d\n", BITS, word, hi, j, q, want);
            }
        }
        // the byte form of the mma.sync kernel
        for (int half = 0; half < 2; half++) {
            unsigned qb;
            if constexpr (BITS == 4) qb = quad_bytes<0>(word, hi, half);
            else if constexpr (BITS == 5) qb = quad_bytes<1>(word, hi, half);
            else if constexpr (BITS == 6) qb = quad_bytes<2>(word, hi, half);
            else qb = quad_bytes<3>(word, hi, half);
            for (int k = 0; k < 4; k++)
                if ((int) ((qb >> (8 * k)) & 0xff) != index_of(word, hi, hb, 4 * half + k)) {
                    if (bad++ < 5) printf("bits %d quad_bytes half %d value %d differs\n", BITS, half, k);
                }
        }
    }
    return bad;
}
int main() {
    int bad = check_bits<4>() + check_bits<5>() + check_bits<6>() + check_bits<7>();
    for (int it = 0; it < 200000; it++) { // 8-bit rows: int8 values
        const unsigned lo = rnd(), hi = rnd();
        unsigned x[4];
        pair_words8(lo, hi, x);
        for (int j = 0; j < 8; j++) {
            const int k = unit_perm(j);
            const int want = (int) (int8_t) (((k < 4 ? lo : hi) >> (8 * (k & 3))) & 0xff);
            const double q = half_val((x[j >> 1] >> (16 * (j & 1))) & 0xffff) - half_val(pair_sub_a<8>() & 0xffff);
            if (q != (double) want && bad++ < 5) printf("q8 unit pos %d: got %g want %d\n", j, q, want);
        }
    }
    for (int j = 0; j < 8; j++)
        if (unit_perm(j) != UNIT_PERM[j]) bad++;
    printf(bad ? "FAILED: %d\n" : "OK %d\n", bad);
    return bad ? 1 : 0;
}
