// Fast decode attention for sm_100a: warp-specialised, register dequantisation, TMA bulk rings, all SMs busy on one sequence.
//
// Same arithmetic as the tensor-core kernel (the reference's attn_core_t, qwen38_mk.cu:2756-3067): the chunk
// partition attn_dims, 32-position tiles in order inside a chunk with a running max, P rounded to fp16, fp32 accumulation.
// What changes is who does the work:
//   - a chunk (up to thousands of positions) is cut into batches of B <= 8 tiles; a batch is a task. With one sequence the
//     tasks of a kv head are dealt to CPH = #SM / 4 CTAs in batch-major order, so every SM streams K / V rows;
//   - the running max a batch starts from is the max of all earlier batches of its chunk. Those batches run on other CTAs
//     at about the same time: each CTA publishes the cumulative row maxima up to its batch right after computing the scores
//     (which stay in registers meanwhile) and reads its predecessor's before it exponentiates. Waits are bounded; the launch is
//     cooperative so every CTA is resident;
//   - warps 0-7 compute S = Q K^T of one tile each (K rows unpacked from shared memory straight into MMA B fragments), run
//     the softmax on their registers and leave P (fp16) in shared memory; warps 8-15 own 32 output dims each, unpack V rows
//     into B fragments and accumulate O over every tile of every task of the CTA. K / V rows arrive by cp.async.bulk copies
//     completing on mbarriers: a score warp fetches its next tile into its own stage as soon as it has read the current
//     one; lane 0 of the first P V warp keeps a ring of V tiles full;
//   - a CTA writes one un-normalised partial (m, l, O); the merge kernel of kv_kernels.cu combines them.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <vector>

#include "kv_kernels.h"
#include "kv_quant.cuh"
#include "kv_unpack.h"
#include "kv_attend_common.cuh"

#ifndef MKKV_ABL
#define MKKV_ABL 0 // timing experiments only: bit 0 no P V math, bit 1 no score math, bit 2 no exp
#endif

namespace mkkv {

namespace fast {

using namespace attn_common;

constexpr int NTHREADS = 512;       // 16 warps: 8 score warps, 8 P V warps
constexpr int SW = 8;               // score warps = tiles per batch at most
constexpr int NSV = 6;              // V ring stages (K: one private stage per score warp)
constexpr int STAGE = ATP * HD + ATP * SCALE_ROW; // 32 q8 rows + their scales: 8704 bytes
constexpr int SC_OFF = ATP * HD;    // scales of a staged tile
constexpr int NPSLOT = 2 * SW;      // P tiles in flight: two batches
// Q and P live in shared memory in MMA A-fragment order: [row tile mt][k-step][lane] -> uint4 (a0, a1, a2, a3), so a
// fragment is one 16-byte load of consecutive lanes (no bank conflicts) and lands in registers in operand order.
constexpr int QF_KS = HD / 16;      // k-steps of Q (k-step 4 G + s covers dims 64 G + 16 tig + 4 s .. + 3 for lane (g8, tig))
constexpr int PF_KS = ATP / 16;     // k-steps of a P tile

struct PSlot {
    uint4 p[3][PF_KS][32];
    float alpha[AR]; // rescale of the accumulator rows before this tile
    int rescale[2];  // != 0: some alpha != 1 (one word per writing warp)
    int valid;       // 0: the batch has no such tile
    int pad;
};

struct Smem {
    uint8_t kst[SW][STAGE];
    uint8_t vst[NSV][STAGE];
    uint4 q[3][QF_KS][32];
    PSlot ps[NPSLOT];
    float tmax[2][SW][AR]; // row maxima of the batch's tiles (double-buffered by batch parity, as rs / carry / macc)
    float mrun[SW][AR];    // per score warp: the running max its tile's P is taken against
    float rs[2][SW][AR];   // row sums of P (fp32, before rounding)
    float carry[2][AR];    // mode 1: running max of the chunk after the previous batch
    float macc[2][AR];     // the reference max the accumulator rows are scaled to
    uint64_t k_full[SW], v_full[NSV], v_empty[NSV], p_full[NPSLOT], p_empty[NPSLOT];
    AttnJob job; // the CTA's job, copied here once: parameter / global reads stay out of the tile loops
    WaitLimit wl; // the launch's wait limit and the CTA's give-up flag
};

struct Args {
    AttnJob one;          // the job when jobs == null
    const AttnJob * jobs; // device array (mode 1)
    int njobs;
    int mode;  // 0: one job spread over the grid with the max exchange; 1: one CTA per (job, kv head, chunk)
    int cph;   // mode 0: CTAs per kv head
    int B;     // tiles per batch (<= SW)
    float * part;  // [slot][AR][HD]
    float2 * ml;   // [slot][AR]
    unsigned long long * xmax; // mode 0: [kv head][chunk][batch][AR] words {epoch : 32, float bits : 32}
    int nbmax;     // batches per chunk the exchange array holds
    int epoch;     // tag of this launch's words (differs from every earlier launch's)
    int * status;
    const AttnTask * tasks; // mode 0, optional: the task list of a kv head built on the host (position-range jobs), else null
    int ntasks;             // tasks per kv head in that list
    unsigned long long * prof; // optional: [CTA][PROF_BATCHES][PROF_STAMPS] globaltimer stamps (null: off)
    unsigned wait_rounds;      // failed tries of a wait before the CTA gives up
};
constexpr int PROF_BATCHES = 16, PROF_STAMPS = 20;
#define MKKV_STAMP(k)                                                                                                  \
    do {                                                                                                               \
        if (a.prof && lane == 0 && bcnt < PROF_BATCHES)                                                                \
            a.prof[((size_t) blockIdx.x * PROF_BATCHES + bcnt) * PROF_STAMPS + (k)] = globaltimer_ns();                \
    } while (0)

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}



// where a tile's rows live (ring from the window start on), its bits, its valid rows
__device__ __forceinline__ int tile_src(const KvView & kv, int w, int g, int tb, int ws, const uint8_t *& val, const uint16_t *& sc) {
    const KvSide & s = kv.s[w];
    if (s.rval && tb >= ws) {
        const size_t rr = (size_t) g * kv.rc + tb % kv.rc;
        val = s.rval + rr * HD;
        sc = s.rsc + rr * 8;
        return 8;
    }
    const size_t row = (size_t) g * kv.ctxp + (tb - kv.base);
    val = s.val + row * row_bytes(s.bits);
    sc = s.sc + row * 8;
    return s.bits;
}
__device__ __forceinline__ int tile_bits(const KvView & kv, int w, int tb, int ws) { return (kv.s[w].rval && tb >= ws) ? 8 : kv.s[w].bits; }

// ---- S = Q K^T of one staged 32-position tile, all in registers ----
// FMT 0 .. 3: rows of 4 + FMT bits; FMT 4: q8_0 rows. acc[mt][nt]: rows 16 mt + g8 (+ 8), MMA columns 2 tig, 2 tig + 1 of
// n-tile nt, i.e. positions 8 nt + pos_of_n(2 tig + e).
template <int MT, int FMT>
__device__ __forceinline__ void s_tile(const uint8_t * st, const uint4 * sq, float (&acc)[3][4][4], int lane) {
    const int g8 = lane >> 2, tig = lane & 3;
    constexpr int HB = FMT < 4 ? FMT : 0;
    constexpr int RB = FMT < 4 ? 32 * (4 + FMT) : HD;
    const __half bias = __float2half_rn(FMT < 4 ? 1024.f + (float) (1 << (3 + FMT)) : 1152.f);
    const __half2 sub = __half2half2(bias);
    const __half * scales = reinterpret_cast<const __half *>(st + SC_OFF);
    const int prow = pos_of_n(g8);
#pragma unroll
    for (int G = 0; G < 4; G++) {
        unsigned wA[4], wB[4], hA[4], hB[4], wC[4], wD[4];
        __half2 d[4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const int row = 8 * nt + prow;
            const uint8_t * rp = st + row * RB;
            if constexpr (FMT == 4) {
                const uint4 v = *reinterpret_cast<const uint4 *>(rp + 64 * G + 16 * tig);
                wA[nt] = v.x ^ 0x80808080u; // q + 128
                wB[nt] = v.y ^ 0x80808080u;
                wC[nt] = v.z ^ 0x80808080u;
                wD[nt] = v.w ^ 0x80808080u;
                hA[nt] = hB[nt] = 0u;
            } else {
                const uint2 v = *reinterpret_cast<const uint2 *>(rp + 32 * G + 8 * tig);
                wA[nt] = v.x;
                wB[nt] = v.y;
                wC[nt] = wD[nt] = 0u;
                if constexpr (HB == 1) {
                    const unsigned h = *reinterpret_cast<const unsigned short *>(rp + 128 + 8 * G + 2 * tig);
                    hA[nt] = h & 0xffu;
                    hB[nt] = h >> 8;
                } else if constexpr (HB == 2) {
                    const unsigned h = *reinterpret_cast<const unsigned *>(rp + 128 + 16 * G + 4 * tig);
                    hA[nt] = h & 0xffffu;
                    hB[nt] = h >> 16;
                } else if constexpr (HB == 3) {
                    const unsigned short * hp = reinterpret_cast<const unsigned short *>(rp + 128 + 24 * G + 6 * tig);
                    const unsigned h0 = hp[0], h1 = hp[1], h2 = hp[2];
                    hA[nt] = h0 | ((h1 & 0xffu) << 16);
                    hB[nt] = (h1 >> 8) | (h2 << 8);
                } else {
                    hA[nt] = hB[nt] = 0u;
                }
            }
            d[nt] = __half2half2(scales[row * 8 + 2 * G + (tig >> 1)]);
        }
#pragma unroll
        for (int s = 0; s < 4; s++) {
            uint4 a[3];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) a[mt] = sq[(mt * QF_KS + 4 * G + s) * 32 + lane];
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                unsigned x;
                if constexpr (FMT == 4) x = s == 0 ? wA[nt] : s == 1 ? wB[nt] : s == 2 ? wC[nt] : wD[nt];
                else x = quad_bytes<HB>(s < 2 ? wA[nt] : wB[nt], s < 2 ? hA[nt] : hB[nt], s & 1);
                const unsigned b0 = cvt_pair<0>(x, sub, d[nt]), b1 = cvt_pair<1>(x, sub, d[nt]);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) mma16816(acc[mt][nt], a[mt].x, a[mt].y, a[mt].z, a[mt].w, b0, b1);
            }
        }
    }
}

// ---- O += P V of one staged tile for the 32 dims of dim group dg ----
// acc[mt][v]: rows 16 mt + g8 (+ 8); MMA column x = 2 tig (+ 1) of n-tile v is dim 32 dg + 4 x + v. np: valid rows of the tile
// (rows past it hold stale bytes: their scale is forced to zero so 0 * garbage cannot make a NaN).
template <int MT, int FMT>
__device__ __forceinline__ void pv_tile(const uint8_t * st, const uint4 * sp, float (&acc)[3][4][4], int lane, int dg, int np) {
    const int g8 = lane >> 2, tig = lane & 3;
    constexpr int HB = FMT < 4 ? FMT : 0;
    constexpr int RB = FMT < 4 ? 32 * (4 + FMT) : HD;
    const __half bias = __float2half_rn(FMT < 4 ? 1024.f + (float) (1 << (3 + FMT)) : 1152.f);
    const __half2 sub = __half2half2(bias);
    const __half * scales = reinterpret_cast<const __half *>(st + SC_OFF);
#pragma unroll
    for (int ks = 0; ks < 2; ks++) {
        uint4 a[3];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) a[mt] = sp[(mt * PF_KS + ks) * 32 + lane];
        unsigned b[4][2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            unsigned x[2];
            __half dj[2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int row = 16 * ks + 8 * h + pos_of_n(2 * tig + j);
                const uint8_t * rp = st + row * RB;
                if constexpr (FMT == 4) {
                    x[j] = *reinterpret_cast<const unsigned *>(rp + 32 * dg + 4 * g8) ^ 0x80808080u;
                } else {
                    const int w = 4 * dg + (g8 >> 1);
                    const unsigned word = *reinterpret_cast<const unsigned *>(rp + 4 * w);
                    unsigned hi = 0u;
                    if constexpr (HB == 1) hi = rp[128 + w];
                    if constexpr (HB == 2) hi = *reinterpret_cast<const unsigned short *>(rp + 128 + 2 * w);
                    if constexpr (HB == 3) hi = (unsigned) rp[128 + 3 * w] | ((unsigned) rp[129 + 3 * w] << 8) | ((unsigned) rp[130 + 3 * w] << 16);
                    x[j] = quad_bytes<HB>(word, hi, g8 & 1);
                }
                dj[j] = row < np ? scales[row * 8 + dg] : __float2half_rn(0.f);
            }
            const __half2 dd = __halves2half2(dj[0], dj[1]);
            const unsigned y01 = __byte_perm(x[0], x[1], 0x5140), y23 = __byte_perm(x[0], x[1], 0x7362);
            b[0][h] = cvt_pair<0>(y01, sub, dd);
            b[1][h] = cvt_pair<1>(y01, sub, dd);
            b[2][h] = cvt_pair<0>(y23, sub, dd);
            b[3][h] = cvt_pair<1>(y23, sub, dd);
        }
#pragma unroll
        for (int v = 0; v < 4; v++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++) mma16816(acc[mt][v], a[mt].x, a[mt].y, a[mt].z, a[mt].w, b[v][0], b[v][1]);
    }
}

// format dispatch (warp-uniform): bits 4 .. 8
template <int MT> __device__ __forceinline__ void s_tile_any(int bits, const uint8_t * st, const uint4 * sq, float (&acc)[3][4][4], int lane) {
    switch (bits) {
    case 4: s_tile<MT, 0>(st, sq, acc, lane); break;
    case 5: s_tile<MT, 1>(st, sq, acc, lane); break;
    case 6: s_tile<MT, 2>(st, sq, acc, lane); break;
    case 7: s_tile<MT, 3>(st, sq, acc, lane); break;
    default: s_tile<MT, 4>(st, sq, acc, lane); break;
    }
}
template <int MT>
__device__ __forceinline__ void pv_tile_any(int bits, const uint8_t * st, const uint4 * sp, float (&acc)[3][4][4], int lane, int dg, int np) {
    switch (bits) {
    case 4: pv_tile<MT, 0>(st, sp, acc, lane, dg, np); break;
    case 5: pv_tile<MT, 1>(st, sp, acc, lane, dg, np); break;
    case 6: pv_tile<MT, 2>(st, sp, acc, lane, dg, np); break;
    case 7: pv_tile<MT, 3>(st, sp, acc, lane, dg, np); break;
    default: pv_tile<MT, 4>(st, sp, acc, lane, dg, np); break;
    }
}

__device__ __forceinline__ float quad_max(float x) { // over the 4 lanes of a quad (tig)
    x = fmaxf(x, __shfl_xor_sync(FULL, x, 1));
    return fmaxf(x, __shfl_xor_sync(FULL, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(FULL, x, 1);
    return x + __shfl_xor_sync(FULL, x, 2);
}

template <int MT>
__global__ void __launch_bounds__(NTHREADS, 1) attn_fast_kernel(const __grid_constant__ Args a) {
    extern __shared__ uint8_t smem_raw[];
    Smem & sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t) 127);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g8 = lane >> 2, tig = lane & 3;

    // ---- which job / kv head / tasks this CTA runs ----
    int g, c_fixed = 0, kk = 0;
    const int slot = blockIdx.x;
    {
        const AttnJob * Jp = &a.one;
        if (a.mode != 0 && a.jobs) {
            int j = 0;
            while (j + 1 < a.njobs && (int) blockIdx.x >= a.jobs[j + 1].item0) j++;
            Jp = &a.jobs[j];
        }
        const unsigned * src = reinterpret_cast<const unsigned *>(Jp);
        unsigned * dst = reinterpret_cast<unsigned *>(&sm.job);
        for (int i = tid; i < (int) (sizeof(AttnJob) / 4); i += NTHREADS) dst[i] = src[i];
    }
    if (tid < AR) {
        sm.carry[0][tid] = sm.carry[1][tid] = -CUDART_INF_F;
        sm.macc[0][tid] = sm.macc[1][tid] = -CUDART_INF_F;
    }
    if (tid == 0) {
        sm.wl.dead = 0;
        sm.wl.rounds = a.wait_rounds;
        for (int s = 0; s < SW; s++) mbar_init(&sm.k_full[s], 1);
        for (int s = 0; s < NSV; s++) { mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], SW); }
        for (int s = 0; s < NPSLOT; s++) { mbar_init(&sm.p_full[s], 1); mbar_init(&sm.p_empty[s], SW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const AttnJob & J = sm.job;
    const KvView & kv = J.kv;
    if (a.mode == 0) {
        g = blockIdx.x / a.cph;
        kk = blockIdx.x % a.cph;
    } else {
        const int item = (int) blockIdx.x - J.item0;
        g = item / J.nch;
        c_fixed = item % J.nch;
    }
    const int T = J.T, n = J.n, R = GQ * T, B = a.B, ws = J.ws;
    // per side: main-format bits and the first position served by the q8_0 ring (none: INT_MAX)
    const int kbits = kv.s[0].bits, vbits = kv.s[1].bits;
    const int kring0 = kv.s[0].rval ? ws : 0x7fffffff, vring0 = kv.s[1].rval ? ws : 0x7fffffff;
    const Geo geo = make_geo(J, B);
    // the CTA's task list: mode 0: tasks kk, kk + cph, .. of kv head g; mode 1: batches 0 .. nb - 1 of its chunk
    const int t_first = a.mode == 0 ? kk : 0, t_step = a.mode == 0 ? a.cph : 1;
    const int t_end = a.mode == 0 ? (a.tasks ? a.ntasks : geo.ntasks_head) : ((c_fixed == geo.nch - 1 ? geo.nt_last : geo.nt_full) + B - 1) / B;
    const AttnTask * const ttab = a.mode == 0 && a.tasks ? a.tasks : nullptr;
    auto get_task = [&](int t) -> Task { return ttab ? ttab[t] : make_task(geo, B, a.mode, t, c_fixed); };

    // query rows of the kv head: fp16 -> fp32 -> (K's rotation) -> x 1/16 -> fp16 (qwen38_mk.cu:2876-2883); row = (head % 6) T + t
    for (int r = warp; r < 16 * MT; r += NTHREADS / 32) {
        uint4 out = make_uint4(0, 0, 0, 0);
        if (r < R) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(J.Q + ((size_t) (r % T) * NH + g * GQ + r / T) * HD + lane * 8);
            const __half2 * hh = reinterpret_cast<const __half2 *>(&raw);
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float2 f = __half22float2(hh[k]);
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
            if (kv.s[0].rot) fwht256(v, lane);
            __half2 * h = reinterpret_cast<__half2 *>(&out);
#pragma unroll
            for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(__fmul_rn(v[2 * k], 0.0625f), __fmul_rn(v[2 * k + 1], 0.0625f));
        }
        // lane holds dims 8 lane .. + 7 of row r: two quadruples (k-steps) of the fragment word pair of this row
        {
            const int mt = r >> 4, g8r = r & 7, hh = (r >> 3) & 1, d0 = 8 * lane;
            const int G = d0 >> 6, tg = (d0 >> 4) & 3, s0 = (d0 >> 2) & 3; // dims d0 .. d0 + 3 -> k-step 4 G + s0, next quadruple s0 + 1
            unsigned * f0 = reinterpret_cast<unsigned *>(&sm.q[mt][4 * G + s0][4 * g8r + tg]);
            unsigned * f1 = reinterpret_cast<unsigned *>(&sm.q[mt][4 * G + s0 + 1][4 * g8r + tg]);
            f0[hh] = out.x;     // a0 / a1: dims + 0, + 1
            f0[hh + 2] = out.y; // a2 / a3: dims + 2, + 3
            f1[hh] = out.z;
            f1[hh + 2] = out.w;
        }
    }
    __syncthreads();

    if (warp >= SW) {
        // ---- P V warps: 32 output dims each, every tile of every task; lane 0 of the first one also feeds the V ring ----
        const int dg = warp - SW;
        const bool producer = dg == 0 && lane == 0;
        SideSrc vsrc;
        int vp_t = t_first, vp_j = 0, vp_nt = 0, vp_tb = 0, vp_c1 = 0; // the next tile the producer issues
        unsigned vp_cnt = 0;
        if (producer) vsrc = make_src(kv, 1, g, ws);
        auto v_issue = [&]() {
            if (vp_t >= t_end) return;
            if (vp_j == 0) { // a new task: its geometry once, then tiles by increment
                const Task k = get_task(vp_t);
                vp_nt = k.nt;
                vp_tb = k.pos0;
                vp_c1 = k.c1;
            }
            const int st = vp_cnt % NSV;
            mbar_wait(&sm.v_empty[st], ((vp_cnt / NSV) & 1) ^ 1, a.status, &sm.wl);
            issue_tile(vsrc, vp_tb, vp_c1, sm.vst[st], &sm.v_full[st]);
            vp_cnt++;
            vp_tb += ATP;
            if (++vp_j == vp_nt) {
                vp_j = 0;
                vp_t += t_step;
            }
        };
        if (producer)
            for (int i = 0; i < NSV - 2; i++) v_issue();
        float acc[3][4][4];
#pragma unroll
        for (int i = 0; i < 3; i++)
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int k = 0; k < 4; k++) acc[i][j][k] = 0.f;
        unsigned vcnt = 0, bcnt = 0;
        for (int t = t_first; t < t_end; t += t_step, bcnt++) {
            const Task k = get_task(t);
            if (dg == 0) MKKV_STAMP(8);
            for (int j = 0; j < SW; j++) {
                const int ps = (bcnt & 1) * SW + j;
                mbar_wait(&sm.p_full[ps], (bcnt >> 1) & 1, a.status, &sm.wl);
                if (dg == 0 && j == 0) MKKV_STAMP(9);
                const PSlot & P = sm.ps[ps];
                if (P.valid) {
                    if (dg == 0 && j == 1) MKKV_STAMP(18);
                    if (producer) v_issue(); // into the stage of the tile two before this one: every warp is past it
                    if (dg == 0 && j == 1) MKKV_STAMP(19);
                    __syncwarp();
                    const int st = vcnt % NSV, tb = k.pos0 + j * ATP, np = min(ATP, k.c1 - tb);
                    if (dg == 0 && j < 2) MKKV_STAMP(12 + 3 * j);
                    mbar_wait(&sm.v_full[st], (vcnt / NSV) & 1, a.status, &sm.wl);
                    if (dg == 0 && j < 2) MKKV_STAMP(13 + 3 * j);
                    if (P.rescale[0] | P.rescale[1]) {
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            const float al0 = P.alpha[16 * mt + g8], al1 = P.alpha[16 * mt + g8 + 8];
#pragma unroll
                            for (int v = 0; v < 4; v++) {
                                acc[mt][v][0] *= al0;
                                acc[mt][v][1] *= al0;
                                acc[mt][v][2] *= al1;
                                acc[mt][v][3] *= al1;
                            }
                        }
                    }
#if !(MKKV_ABL & 1)
                    pv_tile_any<MT>(tb >= vring0 ? 8 : vbits, sm.vst[st], &P.p[0][0][0], acc, lane, dg, np);
#endif
                    __syncwarp();
                    if (dg == 0 && j < 2) MKKV_STAMP(14 + 3 * j);
                    if (lane == 0) mbar_arrive(&sm.v_empty[st]);
                    vcnt++;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.p_empty[ps]);
            }
            if (dg == 0) MKKV_STAMP(10);
        }
        // the CTA's un-normalised O: MMA column x of n-tile v is dim 32 dg + 4 x + v
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int r = 16 * mt + g8 + 8 * hh;
                if (r < R) {
                    float * o = a.part + ((size_t) slot * AR + r) * HD + 32 * dg + 8 * tig;
                    *reinterpret_cast<float4 *>(o) = make_float4(acc[mt][0][2 * hh], acc[mt][1][2 * hh], acc[mt][2][2 * hh], acc[mt][3][2 * hh]);
                    *reinterpret_cast<float4 *>(o + 4) =
                        make_float4(acc[mt][0][2 * hh + 1], acc[mt][1][2 * hh + 1], acc[mt][2][2 * hh + 1], acc[mt][3][2 * hh + 1]);
                }
            }
    } else {
        // ---- score warps: tile `warp` of every batch ----
        const SideSrc ksrc = make_src(kv, 0, g, ws);
        // threads 0 .. 47 own one query row each: the max its accumulator row is scaled to, its sum, the carry between batches
        float m_acc = -CUDART_INF_F, l_acc = 0.f, carry = -CUDART_INF_F;
        unsigned kuse = 0, bcnt = 0;
        if (lane == 0 && t_first < t_end) { // the warp's first tile
            const Task k = get_task(t_first);
            if (warp < k.nt) issue_tile(ksrc, k.pos0 + warp * ATP, k.c1, sm.kst[warp], &sm.k_full[warp]);
        }
        for (int t = t_first; t < t_end; t += t_step, bcnt++) {
            const Task k = get_task(t);
            const int ps = (bcnt & 1) * SW + warp;
            float acc[3][4][4];
            const bool mine = warp < k.nt;
            const int tb = k.pos0 + warp * ATP;
            if (warp == 0) MKKV_STAMP(0);
            if (mine) {
#pragma unroll
                for (int i = 0; i < 3; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int q = 0; q < 4; q++) acc[i][j][q] = 0.f;
                mbar_wait(&sm.k_full[warp], kuse & 1, a.status, &sm.wl);
                kuse++;
                if (warp == 0) MKKV_STAMP(1);
#if !(MKKV_ABL & 2)
                s_tile_any<MT>(tb >= kring0 ? 8 : kbits, sm.kst[warp], &sm.q[0][0][0], acc, lane);
#endif
            }
            __syncwarp();
            if (warp == 0) MKKV_STAMP(2);
            if (lane == 0 && t + t_step < t_end) { // the stage is free: fetch this warp's tile of the next task
                const Task kn = get_task(t + t_step);
                if (warp < kn.nt) issue_tile(ksrc, kn.pos0 + warp * ATP, kn.c1, sm.kst[warp], &sm.k_full[warp]);
            }
            if (mine) {
                // mask (row token t sees positions <= n + t; rows past the chunk end; padding rows) and the tile's row maxima
                const bool need_mask = tb + ATP - 1 > min(k.c1 - 1, n) || R < 16 * MT; // (warp-uniform)
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const int r = 16 * mt + g8 + 8 * hh;
                        float mx = -CUDART_INF_F;
                        if (need_mask) {
                            const int lim = min(k.c1 - 1, n + (r % T));
#pragma unroll
                            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                                for (int e = 0; e < 2; e++) {
                                    const int p = tb + 8 * nt + pos_of_n(2 * tig + e);
                                    if (p > lim || r >= R) acc[mt][nt][2 * hh + e] = -CUDART_INF_F;
                                }
                        }
#pragma unroll
                        for (int nt = 0; nt < 4; nt++) mx = fmaxf(mx, fmaxf(acc[mt][nt][2 * hh], acc[mt][nt][2 * hh + 1]));
                        mx = quad_max(mx);
                        if (tig == 0) sm.tmax[0][warp][r] = mx;
                    }
            }
            if (warp == 0) MKKV_STAMP(3);
            named_bar(1, SW * 32); // the batch's tile maxima are complete
            if (warp == 0) MKKV_STAMP(4);
            // ---- rows (threads 0 .. 63 = warps 0, 1): incoming max of the batch, then per tile the running max and the
            // factor that brings the accumulator row to it ----
            if (warp < 2) {
                const int r = tid;
                float m_in = -CUDART_INF_F;
                unsigned long long * xm = nullptr;
                if (r < 16 * MT) {
                    if (a.mode == 0) {
                        if (k.nb > 1) {
                            // xmax[b][row] = {epoch, max over batches 0 .. b of the chunk}: an 8-byte word per row, valid when
                            // its tag is this launch's: no flag, fence or barrier, a row polls its own word (bounded)
                            xm = a.xmax + (((size_t) g * ATT_NCH + k.c) * a.nbmax) * AR + r;
                            if (k.b > 0) {
                                const unsigned long long * src = xm + (size_t) (k.b - 1) * AR;
                                unsigned long long w = __ldcv(src);
                                for (unsigned it = 0; (unsigned) (w >> 32) != (unsigned) a.epoch; it++) {
                                    if (sm.wl.dead) break;
                                    if (it >= sm.wl.rounds) {
                                        sm.wl.dead = 1;
                                        atomicExch(a.status, (int) KS_WAIT_TIMEOUT);
                                        break;
                                    }
                                    w = __ldcv(src);
                                }
                                m_in = __uint_as_float((unsigned) w);
                            }
                            if (k.b + 1 < k.nb) { // publish for the later batches
                                float bm = m_in;
                                for (int j = 0; j < k.nt; j++) bm = fmaxf(bm, sm.tmax[0][j][r]);
                                __stcg(xm + (size_t) k.b * AR, ((unsigned long long) (unsigned) a.epoch << 32) | __float_as_uint(bm));
                            }
                        }
                    } else if (k.b > 0) {
                        m_in = carry;
                    }
                }
                if (warp == 0) MKKV_STAMP(5);
                // the slots of this batch must have been released by the P V warps (two batches ago)
                for (int j = 0; j < SW; j++) mbar_wait(&sm.p_empty[(bcnt & 1) * SW + j], ((bcnt >> 1) & 1) ^ 1, a.status, &sm.wl);
                float m_ref = m_in;
                for (int j = 0; j < k.nt; j++) {
                    PSlot & Pj = sm.ps[(bcnt & 1) * SW + j];
                    float al = 1.f;
                    if (r < 16 * MT) {
                        const float mnew = fmaxf(m_ref, sm.tmax[0][j][r]);
                        if (mnew != -CUDART_INF_F) {
                            if (m_acc != -CUDART_INF_F) al = expf(fminf(m_acc - mnew, 64.f));
                            m_acc = mnew;
                        }
                        m_ref = mnew;
                        sm.mrun[j][r] = mnew;
                        Pj.alpha[r] = al;
                    }
                    const unsigned any = __ballot_sync(FULL, al != 1.f);
                    if (lane == 0) Pj.rescale[warp] = any != 0u;
                }
                carry = m_ref;
            }
            if (warp == 0) MKKV_STAMP(6);
            named_bar(1, SW * 32);
            if (warp == 0) MKKV_STAMP(7);
            // ---- P = fp16(exp(S - running max)) from the registers; row sums in fp32 ----
            PSlot & P = sm.ps[ps];
            if (mine) {
                // n-tile nt = 2 ks + h; the lane's half2 of row 16 mt + g8 + 8 hh is fragment word hh + 2 h of (mt, ks, lane)
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    unsigned w[PF_KS][4];
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const int r = 16 * mt + g8 + 8 * hh;
                        const float m = sm.mrun[warp][r];
                        float sum = 0.f;
#pragma unroll
                        for (int nt = 0; nt < 4; nt++) {
                            float p0 = 0.f, p1 = 0.f;
                            if (m != -CUDART_INF_F) {
#if MKKV_ABL & 4
                                p0 = acc[mt][nt][2 * hh] - m;
                                p1 = acc[mt][nt][2 * hh + 1] - m;
#else
                                p0 = expf(acc[mt][nt][2 * hh] - m);
                                p1 = expf(acc[mt][nt][2 * hh + 1] - m);
#endif
                            }
                            sum += p0 + p1;
                            const __half2 ph = __floats2half2_rn(p0, p1);
                            w[nt >> 1][hh + 2 * (nt & 1)] = *reinterpret_cast<const unsigned *>(&ph);
                        }
                        sum = quad_sum(sum);
                        if (tig == 0) sm.rs[0][warp][r] = sum;
                    }
#pragma unroll
                    for (int ks = 0; ks < PF_KS; ks++) P.p[mt][ks][lane] = make_uint4(w[ks][0], w[ks][1], w[ks][2], w[ks][3]);
                }
            }
            if (lane == 0) P.valid = mine ? 1 : 0;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_full[ps]);
            if (warp == 0) MKKV_STAMP(11);
            named_bar(1, SW * 32);
            if (tid < 16 * MT)
                for (int j = 0; j < k.nt; j++) l_acc = __fmaf_rn(l_acc, sm.ps[(bcnt & 1) * SW + j].alpha[tid], sm.rs[0][j][tid]);
        }
        if (tid < R) a.ml[(size_t) slot * AR + tid] = make_float2(m_acc, l_acc);
    }
}

} // namespace fast

size_t attend_fast_smem_bytes() { return sizeof(fast::Smem) + 128; }
size_t attend_fast_prof_words(int ctas) { return (size_t) ctas * fast::PROF_BATCHES * fast::PROF_STAMPS; }

// host copy of the partition arithmetic of fast::make_geo
static int fast_tasks_per_head(const AttnJob & J, int B, int & nb_full) {
    const int L = J.n + J.T, nt_full = J.cs / ATP, nt_last = (L - (J.nch - 1) * J.cs + ATP - 1) / ATP;
    nb_full = (nt_full + B - 1) / B;
    const int nb_last = (nt_last + B - 1) / B;
    return nb_last * J.nch + (nb_full - nb_last) * (J.nch - 1);
}

// Host-built task list for a job restricted to positions [pos_lo, pos_hi): the chunks of the partition clipped to the range,
// cut into batches of B tiles, batch-major so that a batch's predecessors (same chunk) are always earlier in the list.
int build_range_tasks(const AttnJob & J, int B, std::vector<AttnTask> & out) {
    out.clear();
    const int L = J.n + J.T;
    struct Ch { int c, c0, c1, ntc, nb; };
    std::vector<Ch> chs;
    int max_nb = 0;
    for (int c = 0; c < J.nch; c++) {
        const int c0 = std::max(c * J.cs, J.pos_lo), c1 = std::min(std::min(L, (c + 1) * J.cs), J.pos_hi);
        if (c1 <= c0) continue;
        const int ntc = (c1 - c0 + ATP - 1) / ATP, nb = (ntc + B - 1) / B;
        chs.push_back({c, c0, c1, ntc, nb});
        max_nb = std::max(max_nb, nb);
    }
    for (int b = 0; b < max_nb; b++)
        for (const Ch & h : chs)
            if (b < h.nb) out.push_back({h.c, b, h.nb, h.c0 + b * B * ATP, h.c1, std::min(B, h.ntc - b * B)});
    return max_nb;
}

template <int MT> static cudaError_t fast_launch_mt(const fast::Args & a, int grid, bool cooperative, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(fast::attn_fast_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) attend_fast_smem_bytes());
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    if (cooperative) { // every CTA resident: the CTAs of one chunk wait for one another's row maxima
        void * args[] = {const_cast<fast::Args *>(&a)};
        return cudaLaunchCooperativeKernel((const void *) fast::attn_fast_kernel<MT>, dim3(grid), dim3(fast::NTHREADS), args,
                                           attend_fast_smem_bytes(), stream);
    }
    fast::attn_fast_kernel<MT><<<grid, fast::NTHREADS, attend_fast_smem_bytes(), stream>>>(a);
    return cudaGetLastError();
}

cudaError_t preload_attend_fast() {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, (const void *) fast::attn_fast_kernel<1>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, (const void *) fast::attn_fast_kernel<2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, (const void *) fast::attn_fast_kernel<3>);
    return e;
}

cudaError_t launch_attend_fast(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int total_items, int max_T, int num_sms,
                               float * part, float2 * ml, int part_slots, unsigned long long * xmax, int nbmax, int epoch, int * status,
                               unsigned long long * prof, bool spread, cudaStream_t stream, const AttnTask * tasks_dev, int ntasks,
                               int tasks_B, float * raw_part, float2 * raw_ml) {
    fast::Args a;
    a.prof = prof;
    a.tasks = nullptr;
    a.ntasks = 0;
    a.one = jobs_host[0];
    a.jobs = njobs > 1 ? jobs_dev : nullptr;
    a.njobs = njobs;
    a.part = part;
    a.ml = ml;
    a.xmax = xmax;
    a.nbmax = nbmax;
    a.epoch = epoch;
    a.status = status;
    a.wait_rounds = attn_common::WAIT_ROUNDS_DEFAULT;
    int grid;
    AttnJob merge_job = jobs_host[0];
    if (njobs == 1 && spread) {
        // one sequence: spread its tasks over all SMs; pick the batch size that leaves the fewest idle rounds
        a.mode = 0;
        a.cph = num_sms / NKV;
        if (a.cph < 1 || a.cph > 64) return cudaErrorNotSupported; // (the merge holds a kv head's partial weights in two registers per lane)
        int best_B = 0, best_cost = 0x7fffffff;
        for (int B = fast::SW; B >= 4; B--) {
            int nb_full;
            const int tasks = fast_tasks_per_head(jobs_host[0], B, nb_full);
            if (nb_full > nbmax || nb_full > 64) continue;
            const int rounds = (tasks + a.cph - 1) / a.cph, cost = rounds * (B + 1);
            if (cost < best_cost) {
                best_cost = cost;
                best_B = B;
            }
        }
        if (tasks_dev) { // a position-range job: the host built its task list with tasks_B tiles per batch
            best_B = tasks_B;
            a.tasks = tasks_dev;
            a.ntasks = ntasks;
        }
        if (!best_B) return cudaErrorNotSupported;
        a.B = best_B;
        grid = NKV * a.cph;
        if (grid > part_slots) return cudaErrorNotSupported;
        merge_job.nch = a.cph; // the merge reads cph partials per kv head, slots g cph ..
        merge_job.item0 = 0;
    } else {
        a.mode = 1;
        a.cph = 0;
        a.B = fast::SW;
        grid = total_items;
        if (grid > part_slots) return cudaErrorNotSupported;
    }
    const int MT = (GQ * max_T + 15) / 16;
    cudaError_t e = MT == 1   ? fast_launch_mt<1>(a, grid, a.mode == 0, stream)
                    : MT == 2 ? fast_launch_mt<2>(a, grid, a.mode == 0, stream)
                              : fast_launch_mt<3>(a, grid, a.mode == 0, stream);
    if (e != cudaSuccess) return e;
    return launch_merge(jobs_dev, a.mode == 0 ? &merge_job : jobs_host, njobs, max_T, part, ml, stream, raw_part, raw_ml);
}

} // namespace mkkv
