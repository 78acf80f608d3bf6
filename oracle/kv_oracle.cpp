// TEST INFRASTRUCTURE ONLY -- the CPU parity oracle of the KV-cache hot path.
//
// A plain C++17 restatement (no CUDA, no product code) of the arithmetic and byte layout of the reference engine's
// KV quantizer, cache layout, decode attention, split merge, ring refill, host-store item order and state digest.
// Only tests, the smoke check and the benchmark's CPU-baseline leg may load this library; nothing shipped links it.
//
// Parity pin: the quantizer, rotation and dequantisation are checked against the reference's own device functions
// (cut from its source at build time into oracle/_ref and run on a GPU; see oracle/ref_witness.cu) through the golden
// vectors in tests/golden/kv_quant_golden.npz. The attention arithmetic is checked against the reference's own decode-attention
// kernels (cut from its source by its own generator script and run on a GPU behind oracle/ref_attn_witness.cu): the per-chunk
// running maxima, sums and un-normalised outputs and the merged output those kernels produced on seeded caches are stored in
// tests/golden/attn_golden.npz (made by tests/golden/make_attn_golden.py), together with the rows the reference's store
// kernels wrote, which must equal this file's bytes.
//
// Every function cites the reference lines it follows (paths relative to the reference project root).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr int NH = 24, NKV = 4, HD = 256, GQ = NH / NKV; // mk_shared.cuh:215
constexpr int ATP = 32, ATT_NCH = 20, ATT_BUCKET = 640;  // mk_shared.cuh:263-265
constexpr int KV_PAD = 16;                               // mk_shared.cuh:247
constexpr int MAX_LAYERS = 17;                           // mk_shared.cuh:251 (N_ATT_SLOTS)

thread_local std::string g_err;

// ---- fp16 <-> fp32 (IEEE binary16, round to nearest even), bit-level so no compiler flag changes it ----
inline float h2f(uint16_t h) {
    const uint32_t s = (uint32_t) (h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) u = s;
        else { // subnormal: m * 2^-24
            float f = (float) m * 5.9604644775390625e-8f;
            memcpy(&u, &f, 4);
            u |= s;
        }
    } else if (e == 31) u = s | 0x7f800000u | (m << 13);
    else u = s | ((e + 112u) << 23) | (m << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f2h(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t s = (u >> 16) & 0x8000u;
    u &= 0x7fffffffu;
    if (u >= 0x7f800000u) return (uint16_t) (s | 0x7c00u | (u > 0x7f800000u ? 0x200u : 0u));
    if (u >= 0x477ff000u) return (uint16_t) (s | 0x7c00u); // >= 65520 rounds to inf
    if (u < 0x38800000u) {                                 // below the smallest normal half: subnormal or zero
        if (u < 0x33000000u) return (uint16_t) s;          // < 2^-25 rounds to zero (2^-25 itself ties to even = 0)
        const int e = (int) (u >> 23);                     // value = 1.m * 2^(e-127)
        const uint32_t m = (u & 0x7fffffu) | 0x800000u;
        const int sh = 126 - e;                            // result = m >> sh in units of 2^-24 (sh in 14..24)
        const uint32_t q = m >> sh, r = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
        return (uint16_t) (s | (q + ((r > half || (r == half && (q & 1u))) ? 1u : 0u)));
    }
    const uint32_t m = u & 0x1fffu; // 13 dropped bits
    uint32_t v = (u - 0x38000000u) >> 13;
    if (m > 0x1000u || (m == 0x1000u && (v & 1u))) v++;
    return (uint16_t) (s | v);
}

// CUDA's __float2int_rn: round to nearest even, saturating, NaN -> 0
inline int f2i_rn(float x) {
    if (x != x) return 0;
    if (x >= 2147483648.0f) return 2147483647;
    if (x <= -2147483648.0f) return (-2147483647 - 1);
    return (int) std::nearbyintf(x); // default rounding mode: to nearest even
}
// CUDA's (int) float: truncation, saturating, NaN -> 0
inline int f2i_rz(float x) {
    if (x != x) return 0;
    if (x >= 2147483648.0f) return 2147483647;
    if (x <= -2147483648.0f) return (-2147483647 - 1);
    return (int) x;
}

// ---- quantizer: qwen38_mk.cu:2003-2116 ----

// 256-point Walsh-Hadamard transform, the reference's butterfly order: element index i = 8 lane + k, bits of k first
// (1, 2, 4), then the lane bits (1 .. 16), then x 1/16. qwen38_mk.cu:2049-2069
void fwht256(float * v) {
    for (int m = 1; m < 8; m <<= 1)
        for (int i = 0; i < HD; i++)
            if (!(i & m)) {
                const float a = v[i], b = v[i | m];
                v[i] = a + b;
                v[i | m] = a - b;
            }
    for (int m = 8; m < HD; m <<= 1) // lane bit m / 8: lane without the bit gets own + partner, with it partner - own
        for (int i = 0; i < HD; i++)
            if (!(i & m)) {
                const float a = v[i], b = v[i | m];
                v[i] = a + b;
                v[i | m] = a - b;
            }
    for (int i = 0; i < HD; i++) v[i] *= 0.0625f;
}

// q8_0 row: qwen38_mk.cu:2005-2023
void quant_q8(const float * v, uint8_t * q, uint16_t * sc) {
    for (int b = 0; b < HD / 32; b++) {
        float am = 0.f;
        for (int i = 0; i < 32; i++) am = std::fmax(am, std::fabs(v[32 * b + i]));
        const float id = am > 0.f ? 127.0f / am : 0.f;
        for (int i = 0; i < 32; i++) {
            const volatile float prod = v[32 * b + i] * id; // one fp32 multiply, then the conversion
            q[32 * b + i] = (uint8_t) (f2i_rn(prod) & 0xff);
        }
        sc[b] = f2h(am / 127.0f);
    }
}

// 4 .. 7-bit row: qwen38_mk.cu:2029-2046 (4 bits), :2075-2097 (5 .. 7 bits); 32 * bits bytes
void quant_qn(const float * v, int bits, uint8_t * q, uint16_t * sc) {
    const int h = 1 << (bits - 1), hb = bits - 4;
    memset(q, 0, (size_t) 32 * bits);
    for (int b = 0; b < HD / 32; b++) {
        // (am, sv) per lane in value order, then combined over the 4 lanes by xor 1, xor 2 under the same rule
        float lam[4], lsv[4];
        for (int l = 0; l < 4; l++) {
            float am = 0.f, sv = 0.f;
            for (int k = 0; k < 8; k++) {
                const float x = v[32 * b + 8 * l + k];
                if (std::fabs(x) > am || (std::fabs(x) == am && x > sv)) { am = std::fabs(x); sv = x; }
            }
            lam[l] = am;
            lsv[l] = sv;
        }
        for (int m = 1; m <= 2; m <<= 1) {
            float nam[4], nsv[4];
            for (int l = 0; l < 4; l++) {
                const float oa = lam[l ^ m], os = lsv[l ^ m];
                nam[l] = lam[l];
                nsv[l] = lsv[l];
                if (oa > lam[l] || (oa == lam[l] && os > lsv[l])) { nam[l] = oa; nsv[l] = os; }
            }
            memcpy(lam, nam, sizeof lam);
            memcpy(lsv, nsv, sizeof lsv);
        }
        const float sv = lsv[0];
        const float d = sv / (float) -h, id = d != 0.f ? 1.0f / d : 0.f;
        for (int l = 0; l < 4; l++) {
            const int lane = 4 * b + l;
            unsigned lo = 0, hi = 0;
            for (int k = 0; k < 8; k++) {
                // v * id + (h + 0.5) is one fused multiply-add in the reference binary (nvcc contracts it)
                const int t = f2i_rz(std::fmaf(v[8 * lane + k], id, (float) h + 0.5f));
                const unsigned n = (unsigned) std::min(2 * h - 1, t);
                lo |= (n & 15u) << (k < 4 ? 8 * k : 8 * (k - 4) + 4);
                hi |= (n >> 4) << (hb * k);
            }
            for (int j = 0; j < 4; j++) q[4 * lane + j] = (uint8_t) (lo >> (8 * j));
            for (int j = 0; j < hb; j++) q[128 + lane * hb + j] = (uint8_t) (hi >> (8 * j));
        }
        sc[b] = f2h(d);
    }
}

inline int row_bytes(int bits) { return 32 * bits; }

void quant_row(const float * v, int bits, uint8_t * q, uint16_t * sc) {
    if (bits == 8) quant_q8(v, q, sc);
    else quant_qn(v, bits, q, sc);
}

// the integer of value i of a row: int8 (8 bits) or n - 2^(bits-1). qwen38_mk.cu:2336-2343,2458-2468
inline int row_int(const uint8_t * q, int bits, int i) {
    if (bits == 8) return (int) (int8_t) q[i];
    const int lane = i >> 3, k = i & 7, hb = bits - 4;
    const unsigned byte = q[4 * lane + (k & 3)];
    unsigned n = k < 4 ? (byte & 15u) : (byte >> 4);
    if (hb > 0) {
        unsigned hi = 0;
        for (int j = 0; j < hb; j++) hi |= (unsigned) q[128 + lane * hb + j] << (8 * j);
        n |= ((hi >> (hb * k)) & ((1u << hb) - 1u)) << 4;
    }
    return (int) n - (1 << (bits - 1));
}
// d * q in fp32 (exact): what ring refill re-quantizes. qwen38_mk.cu:2498-2512
void dequant_f32(const uint8_t * q, const uint16_t * sc, int bits, float * out) {
    for (int i = 0; i < HD; i++) out[i] = h2f(sc[i >> 5]) * (float) row_int(q, bits, i);
}
// d * q rounded once to fp16: the attention operands. qwen38_mk.cu:2336-2343,2458-2468
void dequant_f16(const uint8_t * q, const uint16_t * sc, int bits, float * out) {
    for (int i = 0; i < HD; i++) out[i] = h2f(f2h(h2f(sc[i >> 5]) * (float) row_int(q, bits, i)));
}

// ---- window / partition: qwen38_mk.cu:2122-2126, 2548-2551, loader.cu:1479-1486, mk_shared.cuh:288-291 ----
int kv_ws(int L, int win) {
    if (win <= 0) return 0;
    const int ws = (L + ATT_BUCKET - 1) / ATT_BUCKET - 1 - (win + ATT_BUCKET - 1) / ATT_BUCKET;
    return ws > 0 ? ws * ATT_BUCKET : 0;
}
int kv_rc(int win) { return win > 0 ? ((win + ATT_BUCKET - 1) / ATT_BUCKET + 1) * ATT_BUCKET + ATP : 0; }
void attn_dims(int L, int & nch, int & cs) {
    cs = ATP * std::max(1, (L + ATT_BUCKET - 1) / ATT_BUCKET);
    nch = std::max(1, (L + cs - 1) / cs);
}
int att_cap_T(int n, int T) {
    const int lim = ATT_BUCKET * ((n + ATT_BUCKET) / ATT_BUCKET) - n;
    return T < lim ? T : lim;
}

// ---- MK_KV spec: loader.cu:1329-1366 ----
// Grammar: items separated by commas, each <K|V|*><layer|*|nothing>=<4..8>[r]; a later item overrides an earlier one; every
// side starts as 8 bits, not rotated. Errors carry the reference's messages.
bool parse_spec(const char * spec, int layers, int (*kvb)[MAX_LAYERS], int (*rot)[MAX_LAYERS]) {
    for (int s = 0; s < MAX_LAYERS; s++) {
        kvb[0][s] = kvb[1][s] = 8;
        rot[0][s] = rot[1][s] = 0;
    }
    const char * p = spec ? spec : "";
    while (*p) {
        const char * end = strchr(p, ',');
        const std::string item = end ? std::string(p, end) : std::string(p);
        p = end ? end + 1 : p + item.size();
        if (item.empty()) continue;
        // side letter, layer field, '=', format field
        const size_t eq = item.find('=');
        const bool side_ok = item[0] == 'K' || item[0] == 'V' || item[0] == '*';
        if (eq == std::string::npos || eq == 0 || !side_ok) { g_err = "MK_KV: bad item " + item; return false; }
        const std::string layer_field = item.substr(1, eq - 1), fmt = item.substr(eq + 1);
        int bits = 0, rotated = 0;
        if (fmt.size() >= 1 && fmt.size() <= 2 && fmt[0] >= '4' && fmt[0] <= '8' && (fmt.size() == 1 || fmt[1] == 'r')) {
            bits = fmt[0] - '0';
            rotated = fmt.size() == 2;
        } else {
            g_err = "MK_KV: expected 4..8 or 4r..8r in " + item;
            return false;
        }
        int lo = 0, hi = layers; // the layers the item names: all, or one
        if (!layer_field.empty() && layer_field != "*") {
            long v = -1;
            if (layer_field.find_first_not_of("0123456789") == std::string::npos && layer_field.size() < 7) v = atol(layer_field.c_str());
            if (v < 0 || v >= layers) { g_err = "MK_KV: bad slot in " + item; return false; }
            lo = (int) v;
            hi = lo + 1;
        }
        for (int l = lo; l < hi; l++) {
            if (item[0] != 'V') kvb[0][l] = bits, rot[0][l] = rotated;
            if (item[0] != 'K') kvb[1][l] = bits, rot[1][l] = rotated;
        }
    }
    return true;
}

// ---- the cache: mk_shared.cuh:385-403, loader.cu:1457-1503 ----
struct Cache {
    int layers = 0, ctx = 0, ctxp = 0, win = 0, rc = 0;
    int kvb[2][MAX_LAYERS], rot[2][MAX_LAYERS];
    bool has_ring[2][MAX_LAYERS];
    std::vector<uint8_t> val[2][MAX_LAYERS], rval[2][MAX_LAYERS];   // [g][ctxp][32 bits] / [g][rc][256]
    std::vector<uint16_t> sc[2][MAX_LAYERS], rsc[2][MAX_LAYERS];    // [g][ctxp][8] / [g][rc][8]
    int kv_top = 0;

    uint8_t * vrow(int w, int l, int g, int p) { return val[w][l].data() + ((size_t) g * ctxp + p) * row_bytes(kvb[w][l]); }
    uint16_t * srow(int w, int l, int g, int p) { return sc[w][l].data() + ((size_t) g * ctxp + p) * 8; }
    uint8_t * rvrow(int w, int l, int g, int r) { return rval[w][l].data() + ((size_t) g * rc + r) * HD; }
    uint16_t * rsrow(int w, int l, int g, int r) { return rsc[w][l].data() + ((size_t) g * rc + r) * 8; }
};

// one K / V row: rotate, main-format row, q8 ring row of the same (rotated) values. qwen38_mk.cu:2101-2116
void kv_store(Cache & c, int w, int l, int g, int pos, const float * vin) {
    float v[HD];
    memcpy(v, vin, sizeof v);
    if (c.rot[w][l]) fwht256(v);
    quant_row(v, c.kvb[w][l], c.vrow(w, l, g, pos), c.srow(w, l, g, pos));
    if (c.has_ring[w][l]) quant_q8(v, c.rvrow(w, l, g, pos % c.rc), c.rsrow(w, l, g, pos % c.rc));
}

// the rows of a tile's position: ring (q8) for positions of tiles at or after the window start. qwen38_mk.cu:2147-2166
inline void kv_src(Cache & c, int w, int l, int g, int p, int ws, const uint8_t *& q, const uint16_t *& s, int & bits) {
    const int p0 = p & ~(ATP - 1);
    if (c.has_ring[w][l] && p0 >= ws) {
        q = c.rvrow(w, l, g, p % c.rc);
        s = c.rsrow(w, l, g, p % c.rc);
        bits = 8;
    } else {
        q = c.vrow(w, l, g, p);
        s = c.srow(w, l, g, p);
        bits = c.kvb[w][l];
    }
}

// One (kv head, chunk) item of split-K flash decoding: qwen38_mk.cu:2756-3067 (attn_core_t's arithmetic).
// qf: [R][256] query rows as fp16 values (already rotated and scaled by 1/16), row r = (head % 6) T + t.
// Out: m[R], l[R], O[R][256] un-normalised.
void attn_item(Cache & c, int l, int g, int n, int T, int c0, int c1, int ws, const float * qf, float * om, float * ol, float * oO) {
    const int R = GQ * T;
    std::vector<float> kt((size_t) HD * ATP), vt((size_t) ATP * HD), S((size_t) R * ATP), P((size_t) R * ATP);
    std::vector<float> m(R, -INFINITY), ls(R, 0.f), O((size_t) R * HD, 0.f);
    float row[HD];
    for (int tb = c0; tb < c1; tb += ATP) {
        const int np = std::min(ATP, c1 - tb);
        for (int j = 0; j < ATP; j++) {
            if (j < np) {
                const uint8_t * q;
                const uint16_t * s;
                int bits;
                kv_src(c, 0, l, g, tb + j, ws, q, s, bits);
                dequant_f16(q, s, bits, row);
                for (int d = 0; d < HD; d++) kt[(size_t) d * ATP + j] = row[d];
                kv_src(c, 1, l, g, tb + j, ws, q, s, bits);
                dequant_f16(q, s, bits, vt.data() + (size_t) j * HD);
            } else { // rows past the chunk: zero scales (qwen38_mk.cu:2536-2538)
                for (int d = 0; d < HD; d++) kt[(size_t) d * ATP + j] = 0.f;
                memset(vt.data() + (size_t) j * HD, 0, HD * sizeof(float));
            }
        }
        // S = Q K^T, fp16 operands (products exact in fp32), fp32 accumulation over the head dimension in order
        for (int r = 0; r < R; r++) {
            float acc[ATP];
            for (int j = 0; j < ATP; j++) acc[j] = 0.f;
            const float * qr = qf + (size_t) r * HD;
            for (int d = 0; d < HD; d++) {
                const float qd = qr[d];
                const float * kd = kt.data() + (size_t) d * ATP;
                for (int j = 0; j < ATP; j++) acc[j] += qd * kd[j];
            }
            memcpy(S.data() + (size_t) r * ATP, acc, sizeof acc);
        }
        // online softmax per row, causal among the T new tokens: qwen38_mk.cu:2990-3016
        for (int r = 0; r < R; r++) {
            const int lim = n + (r % T);
            float * s = S.data() + (size_t) r * ATP;
            float mt = -INFINITY;
            for (int j = 0; j < ATP; j++) {
                if (j >= np || tb + j > lim) s[j] = -INFINITY;
                mt = std::fmax(mt, s[j]);
            }
            const float mold = m[r], mnew = std::fmax(mold, mt);
            float al = 1.f, ps = 0.f;
            float * p = P.data() + (size_t) r * ATP;
            if (mnew != -INFINITY) {
                for (int j = 0; j < ATP; j++) {
                    const float e = expf(s[j] - mnew);
                    ps += e;
                    p[j] = h2f(f2h(e));
                }
                al = expf(mold - mnew);
            } else {
                for (int j = 0; j < ATP; j++) p[j] = 0.f;
            }
            ls[r] = ls[r] * al + ps;
            m[r] = mnew;
            float * o = O.data() + (size_t) r * HD;
            if (al != 1.f)
                for (int d = 0; d < HD; d++) o[d] *= al;
            for (int j = 0; j < np; j++) {
                const float pj = p[j];
                if (pj == 0.f) continue;
                const float * vr = vt.data() + (size_t) j * HD;
                for (int d = 0; d < HD; d++) o[d] += pj * vr[d];
            }
        }
    }
    memcpy(om, m.data(), R * sizeof(float));
    memcpy(ol, ls.data(), R * sizeof(float));
    memcpy(oO, O.data(), (size_t) R * HD * sizeof(float));
}

} // namespace

extern "C" {

const char * orc_last_error() { return g_err.c_str(); }

int orc_kv_ws(int L, int win) { return kv_ws(L, win); }
int orc_kv_rc(int win) { return kv_rc(win); }
void orc_attn_dims(int L, int * nch, int * cs) { attn_dims(L, *nch, *cs); }
int orc_att_cap_T(int n, int T) { return att_cap_T(n, T); }
unsigned orc_f2h(float f) { return f2h(f); }
float orc_h2f(unsigned h) { return h2f((uint16_t) h); }
void orc_fwht256(float * v) { fwht256(v); }
int orc_row_bytes(int bits) { return row_bytes(bits); }
// v[256] fp32 -> row bytes + 8 fp16 scales, bits 4 .. 8
void orc_quant_row(const float * v, int bits, uint8_t * q, uint16_t * sc) { quant_row(v, bits, q, sc); }
void orc_dequant_f32(const uint8_t * q, const uint16_t * sc, int bits, float * out) { dequant_f32(q, sc, bits, out); }
void orc_dequant_f16(const uint8_t * q, const uint16_t * sc, int bits, float * out) { dequant_f16(q, sc, bits, out); }

// kvb / rot: [2][layers] ints (side-major). 0 ok, -1 error
int orc_parse_spec(const char * spec, int layers, int * kvb, int * rot) {
    int b[2][MAX_LAYERS], r[2][MAX_LAYERS];
    if (layers < 1 || layers > MAX_LAYERS) { g_err = "layers out of range"; return -1; }
    if (!parse_spec(spec, layers, b, r)) return -1;
    for (int w = 0; w < 2; w++)
        for (int s = 0; s < layers; s++) {
            kvb[w * layers + s] = b[w][s];
            rot[w * layers + s] = r[w][s];
        }
    return 0;
}

void * orc_new(int layers, int ctx, const char * spec, int win, int win_all) {
    if (layers < 1 || layers > MAX_LAYERS || ctx < 1) { g_err = "orc_new: bad shape"; return nullptr; }
    auto * c = new Cache;
    c->layers = layers;
    c->ctx = ctx;
    c->ctxp = ctx + KV_PAD;
    if (!parse_spec(spec, layers, c->kvb, c->rot)) { delete c; return nullptr; }
    const bool want = spec && spec[0];
    c->win = want && win > 0 ? win : 0;
    c->rc = kv_rc(c->win);
    for (int w = 0; w < 2; w++)
        for (int l = 0; l < layers; l++) {
            c->val[w][l].assign((size_t) NKV * c->ctxp * row_bytes(c->kvb[w][l]), 0);
            c->sc[w][l].assign((size_t) NKV * c->ctxp * 8, 0);
            c->has_ring[w][l] = c->win > 0 && (c->kvb[w][l] != 8 || win_all);
            if (c->has_ring[w][l]) {
                c->rval[w][l].assign((size_t) NKV * c->rc * HD, 0);
                c->rsc[w][l].assign((size_t) NKV * c->rc * 8, 0);
            }
        }
    return c;
}
void orc_free(void * h) { delete static_cast<Cache *>(h); }
int orc_ring_rows(void * h) { return static_cast<Cache *>(h)->rc; }
int orc_bits(void * h, int w, int l) { return static_cast<Cache *>(h)->kvb[w][l]; }
int orc_rot(void * h, int w, int l) { return static_cast<Cache *>(h)->rot[w][l]; }
int orc_has_ring(void * h, int w, int l) { return static_cast<Cache *>(h)->has_ring[w][l]; }

// K, V: fp16 [n][4][256] (post-norm, post-RoPE rows). Writes rows pos0 .. pos0 + n - 1 of the layer (main + ring)
int orc_append(void * h, int layer, int pos0, int n, const uint16_t * K, const uint16_t * V) {
    Cache & c = *static_cast<Cache *>(h);
    if (layer < 0 || layer >= c.layers || pos0 < 0 || n < 0 || pos0 + n > c.ctxp) { g_err = "orc_append: out of range"; return -1; }
    float v[HD];
    for (int t = 0; t < n; t++)
        for (int g = 0; g < NKV; g++)
            for (int w = 0; w < 2; w++) {
                const uint16_t * src = (w ? V : K) + ((size_t) t * NKV + g) * HD;
                for (int d = 0; d < HD; d++) v[d] = h2f(src[d]);
                kv_store(c, w, layer, g, pos0 + t, v);
            }
    c.kv_top = std::max(c.kv_top, pos0 + n);
    return 0;
}

// Decode attention of T query tokens at positions n .. n + T - 1 over positions 0 .. n + T - 1 (causal among the T).
// Q: fp16 [T][24][256] (post-norm, post-RoPE, unscaled); O: fp32 [T][24][256] normalised (rotated back if V is stored
// rotated). split > 1 cuts every chunk of the reference partition into that many pieces (partition-sensitivity probe).
// Prologue qwen38_mk.cu:2876-2883, partition :2548-2573, merge :4658-4685.
static int attend_impl(void * h, int layer, int n, int T, const uint16_t * Q, float * O, int nthreads, int split, float * out_m,
                       float * out_l, float * out_O, int ncuts = 0, const int * cuts = nullptr) {
    Cache & c = *static_cast<Cache *>(h);
    if (layer < 0 || layer >= c.layers || T < 1 || T > 8 || n < 0 || n + T > c.ctxp) { g_err = "orc_attend: out of range"; return -1; }
    const int L = n + T, R = GQ * T, ws = kv_ws(L, c.win);
    int nch, cs;
    attn_dims(L, nch, cs);
    // chunk list per kv head
    std::vector<std::pair<int, int>> ch;
    for (int k = 0; k < nch; k++) {
        const int c0 = k * cs, c1 = std::min(L, c0 + cs);
        if (ncuts > 0) { // the chunk cut again at the given positions (multiples of 32): a sequence split by position over GPUs
            int a = c0;
            for (int i = 0; i < ncuts; i++)
                if (cuts[i] > a && cuts[i] < c1) {
                    ch.push_back({a, cuts[i]});
                    a = cuts[i];
                }
            ch.push_back({a, c1});
        } else if (split <= 1) ch.push_back({c0, c1});
        else {
            const int tiles = (c1 - c0 + ATP - 1) / ATP, per = (tiles + split - 1) / split;
            for (int a = c0; a < c1; a += per * ATP) ch.push_back({a, std::min(c1, a + per * ATP)});
        }
    }
    const int nc = (int) ch.size();
    // query rows per kv head: fp16 -> fp32 -> (rotation) -> x 1/16 -> fp16
    std::vector<float> qf((size_t) NKV * R * HD);
    for (int hq = 0; hq < NH; hq++)
        for (int t = 0; t < T; t++) {
            float v[HD];
            const uint16_t * src = Q + ((size_t) t * NH + hq) * HD;
            for (int d = 0; d < HD; d++) v[d] = h2f(src[d]);
            if (c.rot[0][layer]) fwht256(v);
            float * dst = qf.data() + ((size_t) (hq / GQ) * R + (hq % GQ) * T + t) * HD;
            for (int d = 0; d < HD; d++) dst[d] = h2f(f2h(v[d] * 0.0625f));
        }
    std::vector<float> pm((size_t) NKV * nc * R), pl((size_t) NKV * nc * R), pO((size_t) NKV * nc * R * HD);
    std::atomic<int> next{0};
    auto work = [&]() {
        for (;;) {
            const int it = next.fetch_add(1);
            if (it >= NKV * nc) break;
            const int g = it / nc, k = it % nc;
            attn_item(c, layer, g, n, T, ch[k].first, ch[k].second, ws, qf.data() + (size_t) g * R * HD, pm.data() + (size_t) it * R,
                      pl.data() + (size_t) it * R, pO.data() + (size_t) it * R * HD);
        }
    };
    const int nt = std::max(1, std::min(nthreads, NKV * nc));
    std::vector<std::thread> th;
    for (int i = 1; i < nt; i++) th.emplace_back(work);
    work();
    for (auto & t : th) t.join();
    if (out_m) memcpy(out_m, pm.data(), pm.size() * sizeof(float));
    if (out_l) memcpy(out_l, pl.data(), pl.size() * sizeof(float));
    if (out_O) memcpy(out_O, pO.data(), pO.size() * sizeof(float));
    if (!O) return nc;
    // merge: qwen38_mk.cu:4658-4669
    for (int hq = 0; hq < NH; hq++)
        for (int t = 0; t < T; t++) {
            const int g = hq / GQ, r = (hq % GQ) * T + t;
            float M = -INFINITY;
            for (int k = 0; k < nc; k++) M = std::fmax(M, pm[((size_t) g * nc + k) * R + r]);
            float y[HD], den = 0.f;
            for (int d = 0; d < HD; d++) y[d] = 0.f;
            for (int k = 0; k < nc; k++) {
                const size_t it = (size_t) g * nc + k;
                const float mk = pm[it * R + r];
                const float wgt = mk == -INFINITY ? 0.f : expf(mk - M);
                const float * o = pO.data() + (it * R + r) * HD;
                for (int d = 0; d < HD; d++) y[d] += wgt * o[d];
                den += wgt * pl[it * R + r];
            }
            for (int d = 0; d < HD; d++) y[d] = y[d] / den;
            if (c.rot[1][layer]) fwht256(y);
            memcpy(O + ((size_t) t * NH + hq) * HD, y, sizeof y);
        }
    return nc;
}
int orc_attend(void * h, int layer, int n, int T, const uint16_t * Q, float * O, int nthreads, int split) {
    return attend_impl(h, layer, n, T, Q, O, nthreads, split, nullptr, nullptr, nullptr) < 0 ? -1 : 0;
}
// The same call, also giving the un-normalised split partials of the reference partition (what the reference's kernels leave in
// apart / aml, qwen38_mk.cu:3048-3064): item = kv head * chunks + chunk, row = (head % 6) T + t; m, l: [items][6 T],
// Op: [items][6 T][256]. O may be null (partials only). Returns the number of chunks per kv head, -1 on error.
int orc_attend_parts(void * h, int layer, int n, int T, const uint16_t * Q, float * O, int nthreads, float * m, float * l, float * Op) {
    return attend_impl(h, layer, n, T, Q, O, nthreads, 1, m, l, Op);
}
// The same attention with the reference's chunks cut again at `cuts` (ascending positions, multiples of 32): what a sequence split by
// position over several GPUs computes (every piece starts its running max afresh; the merge is the reference's).
int orc_attend_cuts(void * h, int layer, int n, int T, const uint16_t * Q, float * O, int nthreads, int ncuts, const int * cuts) {
    return attend_impl(h, layer, n, T, Q, O, nthreads, 1, nullptr, nullptr, nullptr, ncuts, cuts) < 0 ? -1 : 0;
}
// The merge alone (qwen38_mk.cu:4658-4685) over given partials of nc chunks per kv head in the layout above: O fp32 [T][24][256]
void orc_merge_parts(int T, int nc, int rot_v, const float * pm, const float * pl, const float * pO, float * O) {
    const int R = GQ * T;
    for (int hq = 0; hq < NH; hq++)
        for (int t = 0; t < T; t++) {
            const int g = hq / GQ, r = (hq % GQ) * T + t;
            float M = -INFINITY;
            for (int k = 0; k < nc; k++) M = std::fmax(M, pm[((size_t) g * nc + k) * R + r]);
            float y[HD], den = 0.f;
            for (int d = 0; d < HD; d++) y[d] = 0.f;
            for (int k = 0; k < nc; k++) {
                const size_t it = (size_t) g * nc + k;
                const float mk = pm[it * R + r];
                const float wgt = mk == -INFINITY ? 0.f : expf(mk - M);
                const float * o = pO + (it * R + r) * HD;
                for (int d = 0; d < HD; d++) y[d] += wgt * o[d];
                den += wgt * pl[it * R + r];
            }
            for (int d = 0; d < HD; d++) y[d] = y[d] / den;
            if (rot_v) fwht256(y);
            memcpy(O + ((size_t) t * NH + hq) * HD, y, sizeof y);
        }
}

// ring rows of positions [p0, p1) rebuilt from the main rows: qwen38_mk.cu:2488-2518
int orc_refill(void * h, int p0, int p1) {
    Cache & c = *static_cast<Cache *>(h);
    if (p0 < 0 || p1 > c.ctxp) { g_err = "orc_refill: out of range"; return -1; }
    float v[HD];
    for (int p = p0; p < p1; p++)
        for (int l = 0; l < c.layers; l++)
            for (int w = 0; w < 2; w++) {
                if (!c.has_ring[w][l]) continue;
                for (int g = 0; g < NKV; g++) {
                    dequant_f32(c.vrow(w, l, g, p), c.srow(w, l, g, p), c.kvb[w][l], v);
                    quant_q8(v, c.rvrow(w, l, g, p % c.rc), c.rsrow(w, l, g, p % c.rc));
                }
            }
    return 0;
}
// rewind to P with rows written up to kv_top: the refill range of ck_pool.cu:285-296; returns the rows refilled
int orc_ring_rewind(void * h, int P) {
    Cache & c = *static_cast<Cache *>(h);
    int done = 0;
    if (c.win > 0) {
        const int p0 = std::max(0, P - c.rc), p1 = std::min(P, c.kv_top - c.rc);
        if (p1 > p0) {
            orc_refill(h, p0, p1);
            done = p1 - p0;
        }
    }
    c.kv_top = std::min(c.kv_top, P);
    return done;
}
int orc_kv_top(void * h) { return static_cast<Cache *>(h)->kv_top; }

// The layer's buffers where they lie (the reference layout, mk_shared.cuh:385-403): kind 0 main values [4][ctxp][32 bits], 1 main
// scales [4][ctxp][8], 2 ring values [4][rc][256], 3 ring scales [4][rc][8] (null for a side without a ring). bytes: the size.
void * orc_buffer(void * h, int layer, int w, int kind, long long * bytes) {
    Cache & c = *static_cast<Cache *>(h);
    if (layer < 0 || layer >= c.layers || w < 0 || w > 1) return nullptr;
    switch (kind) {
    case 0: *bytes = (long long) c.val[w][layer].size(); return c.val[w][layer].data();
    case 1: *bytes = (long long) c.sc[w][layer].size() * 2; return c.sc[w][layer].data();
    case 2: *bytes = (long long) c.rval[w][layer].size(); return c.has_ring[w][layer] ? c.rval[w][layer].data() : nullptr;
    case 3: *bytes = (long long) c.rsc[w][layer].size() * 2; return c.has_ring[w][layer] ? c.rsc[w][layer].data() : nullptr;
    }
    return nullptr;
}
int orc_ctxp(void * h) { return static_cast<Cache *>(h)->ctxp; }

// one row's bytes: ring = 0 main row of position pos, ring = 1 the ring row of slot index pos. val: row bytes, sc: 8 halves
int orc_row(void * h, int layer, int w, int g, int pos, int ring, uint8_t * val, uint16_t * sc) {
    Cache & c = *static_cast<Cache *>(h);
    if (ring) {
        if (!c.has_ring[w][layer] || pos < 0 || pos >= c.rc) { g_err = "orc_row: no such ring row"; return -1; }
        memcpy(val, c.rvrow(w, layer, g, pos), HD);
        memcpy(sc, c.rsrow(w, layer, g, pos), 16);
        return HD;
    }
    if (pos < 0 || pos >= c.ctxp) { g_err = "orc_row: out of range"; return -1; }
    const int rb = row_bytes(c.kvb[w][layer]);
    memcpy(val, c.vrow(w, layer, g, pos), rb);
    memcpy(sc, c.srow(w, layer, g, pos), 16);
    return rb;
}

// engine.cu:1444-1455
static unsigned long long dg_hash(const void * p, size_t nb, unsigned long long h = 0xcbf29ce484222325ULL) {
    const unsigned char * b = static_cast<const unsigned char *>(p);
    size_t i = 0;
    for (; i + 8 <= nb; i += 8) {
        unsigned long long w;
        memcpy(&w, b + i, 8);
        h = (h ^ w) * 0x100000001b3ULL;
        h ^= h >> 31;
    }
    for (; i < nb; i++) h = (h ^ b[i]) * 0x100000001b3ULL;
    return h;
}
// The KV part of the state digest for a sequence of n positions: engine.cu:1438-1500 (header words 2 and 7, which
// describe the MTP block and the hidden-state ring, are written as 0). Returns the word count; writes up to cap words.
long long orc_digest(void * h, int n, unsigned long long * out, long long cap) {
    Cache & c = *static_cast<Cache *>(h);
    typedef unsigned long long u64;
    const int rc = c.win > 0 ? c.rc : 0, rlo = rc ? std::max(0, n - rc) : n;
    std::vector<u64> v = {0x4d4b444701ULL, (u64) n, 0, (u64) rc, (u64) rlo, (u64) c.layers, (u64) NKV, 0};
    for (int l = 0; l < c.layers; l++)
        for (int w = 0; w < 2; w++)
            for (int g = 0; g < NKV; g++)
                for (int p = 0; p < n; p++) v.push_back(dg_hash(c.srow(w, l, g, p), 16, dg_hash(c.vrow(w, l, g, p), row_bytes(c.kvb[w][l]))));
    for (int l = 0; l < c.layers; l++)
        for (int w = 0; w < 2; w++)
            for (int g = 0; g < NKV; g++)
                for (int p = rlo; p < n; p++)
                    v.push_back(rc && c.has_ring[w][l] ? dg_hash(c.rsrow(w, l, g, p % rc), 16, dg_hash(c.rvrow(w, l, g, p % rc), HD)) : 0ULL);
    if (out)
        for (long long i = 0; i < std::min<long long>(cap, (long long) v.size()); i++) out[i] = v[i];
    return (long long) v.size();
}

// The snapshot byte stream of rows [a, b) and ring slots [ra, rb): host_store.cu:77-107 (layer, side, kv head: values
// then scales; then the rings in the same order). out = NULL: the size only.
long long orc_snapshot(void * h, int a, int b, int ra, int rb, uint8_t * out) {
    Cache & c = *static_cast<Cache *>(h);
    long long pos = 0;
    auto put = [&](const void * src, size_t n) {
        if (out) memcpy(out + pos, src, n);
        pos += (long long) n;
    };
    if (b > a)
        for (int l = 0; l < c.layers; l++)
            for (int w = 0; w < 2; w++)
                for (int g = 0; g < NKV; g++) {
                    put(c.vrow(w, l, g, a), (size_t) (b - a) * row_bytes(c.kvb[w][l]));
                    put(c.srow(w, l, g, a), (size_t) (b - a) * 16);
                }
    if (c.win > 0 && rb > ra)
        for (int l = 0; l < c.layers; l++)
            for (int w = 0; w < 2; w++)
                if (c.has_ring[w][l])
                    for (int g = 0; g < NKV; g++) {
                        put(c.rvrow(w, l, g, ra), (size_t) (rb - ra) * HD);
                        put(c.rsrow(w, l, g, ra), (size_t) (rb - ra) * 16);
                    }
    return pos;
}

// The prompt-state file of the KV regions, state_files.cu:97-238: "MKSTATE1", u64 key length, key bytes, u64 hend, u64 region
// count, u64 size of every region, then the regions' bytes: for every layer, side, kv head the values of rows 0 .. hend - 1 and
// their scales (:103-110); then for every (layer, side) with a ring ALL heads' ring values, then all heads' ring scales
// (:115-119); then the caller's extra regions (the reference's own are its recurrent state: dstate, conv, h_hist, :120-122).
// Written to path + ".tmp<pid>" and renamed (:136, 178). Returns the file's size, -1 on an I/O error.
long long orc_state_save(void * h, const char * path, const uint8_t * key, long long key_len, int hend, int n_extra, const uint8_t * const * extra,
                         const long long * extra_sizes) {
    Cache & c = *static_cast<Cache *>(h);
    if (hend < 0 || hend > c.ctx) return -1;
    std::vector<std::pair<const void *, size_t>> R;
    for (int l = 0; l < c.layers; l++)
        for (int w = 0; w < 2; w++)
            for (int g = 0; g < NKV; g++) {
                R.push_back({c.vrow(w, l, g, 0), (size_t) hend * row_bytes(c.kvb[w][l])});
                R.push_back({c.srow(w, l, g, 0), (size_t) hend * 16});
            }
    for (int l = 0; l < c.layers; l++)
        for (int w = 0; w < 2; w++)
            if (c.has_ring[w][l]) {
                R.push_back({c.rval[w][l].data(), (size_t) NKV * c.rc * HD});
                R.push_back({c.rsc[w][l].data(), (size_t) NKV * c.rc * 16});
            }
    for (int i = 0; i < n_extra; i++) R.push_back({extra[i], (size_t) extra_sizes[i]});
    const std::string tmp = std::string(path) + ".tmp.oracle";
    FILE * f = fopen(tmp.c_str(), "wb");
    if (!f) return -1;
    bool ok = fwrite("MKSTATE1", 8, 1, f) == 1;
    auto w64 = [&](uint64_t v) { ok = ok && fwrite(&v, 8, 1, f) == 1; };
    w64((uint64_t) key_len);
    ok = ok && (key_len == 0 || fwrite(key, 1, (size_t) key_len, f) == (size_t) key_len);
    w64((uint64_t) hend);
    w64(R.size());
    long long tot = 8 + 8 + key_len + 8 + 8 + 8 * (long long) R.size();
    for (const auto & r : R) w64(r.second), tot += (long long) r.second;
    for (const auto & r : R) ok = ok && (r.second == 0 || fwrite(r.first, 1, r.second, f) == r.second);
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path) != 0) {
        remove(tmp.c_str());
        return -1;
    }
    return tot;
}

} // extern "C"
