// Decode attention on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory) for one sequence spread over
// every SM. Same arithmetic as the other two attention kernels (the reference's attn_core_t, qwen38_mk.cu:2756-3067): the
// chunk partition attn_dims, 32-position tiles in order inside a chunk with a running max, P = fp16(expf(S - max)), fp32
// accumulation. The structure is a dequantising GEMM main loop:
//   - the unit of work is a group of 4 consecutive tiles (128 positions) of one chunk; the groups of a kv head are dealt in
//     group-major order to the CTAs of that head (cooperative launch: all CTAs resident);
//   - one producer thread streams the packed K / V rows of the CTA's groups into a ring of shared-memory slots with bulk
//     copies completing on mbarriers;
//   - 16 worker warps turn packed rows into exact fp16(d * q) operands in the canonical no-swizzle UMMA layouts (one thread:
//     one position x 32 dims per step) -- K as the K-major A operand of S^T[128 pos x 48 rows] = K Q^T, V as the MN-major A
//     operand of O^T[256 dims x 48 rows] += V^T P^T;
//   - one issuer thread runs tcgen05.mma on the slots as they fill (mbarrier "full" from the workers, tcgen05.commit to
//     "empty"), S^T double-buffered in tensor memory, O^T (two 128-dim halves) resident there for the whole kernel;
//   - the workers read S^T back (tcgen05.ld: a thread owns one position and 12 query rows), take the tile maxima, exchange
//     the running max with the CTAs that hold the chunk's earlier groups through small global arrays (own group maxima and
//     cumulative maxima, 8-byte {launch tag, value} words, polled with a bound), and write P to shared memory as the B
//     operand. The accumulator is kept against a per-row reference max that moves rarely (when the running max passes it by
//     more than 8): P is multiplied by exp(running max - reference) in fp32 after its fp16 rounding and split into an fp16
//     high and low part (two MMAs), so the reference's fp16 P is reproduced and no per-tile accumulator rescale is needed;
//   - a CTA writes one un-normalised partial (m, l, O); attn_merge_kernel combines them.
// Every wait is bounded (about two seconds), then the status word is set and the kernel runs to its end and frees its
// tensor memory.
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kv_attend_common.cuh"
#include "kv_kernels.h"
#include "kv_quant.cuh"
#include "kv_unpack.h"

namespace mkkv {

namespace tc {

using namespace attn_common;

constexpr int NWORK = 16;                  // worker warps
constexpr int NTHREADS = (NWORK + 2) * 32; // + the MMA issuer warp + the copy producer warp
constexpr int GT = 4, GP = GT * ATP;       // tiles / positions per group: the M of one MMA
constexpr int RS = 12;                     // query rows per worker warp (4 warps share a tile: 48 rows)
constexpr int RAW_SLOT = ATP * HD + ATP * SCALE_ROW; // one tile of the widest format and its scales: 8704 bytes
constexpr int NRAW = 9;
constexpr int OP_SLOT = GP * 128 * 2;      // fp16 operand: 128 positions x 128 dims
constexpr int NOP = 3;
constexpr int Q_BYTES = AR * HD * 2, P_BYTES = AR * GP * 2;
constexpr unsigned S_COL0 = 0, S_COL1 = 64, O_COL0 = 128, O_COL1 = 192, TMEM_COLS = 256;
constexpr float REF_SLACK = 8.f; // the accumulator's reference max moves when the running max passes it by more than this

struct Smem {
    uint8_t op[NOP][OP_SLOT];   // [dim group 16][position group 16][8 positions][8 dims] fp16
    uint8_t raw[NRAW][RAW_SLOT];
    uint8_t q[Q_BYTES];         // [dim group 32][row group 6][8 rows][8 dims]
    uint8_t p[2][P_BYTES];      // high / low part: [row group 6][position group 16][8 positions][8 rows]
    float tmax[GT][AR];         // row maxima of the group's tiles
    float mrun[2][GT][AR];      // running max each tile's P is taken against (by group parity, as beta / fsc / resc)
    float beta[2][GT][AR];      // exp(running max - reference max)
    float fsc[2][AR];           // factor that brings the accumulator row to a moved reference max
    float lsum[GT][AR];
    int resc[2];
    unsigned char rtok[AR];     // token of a query row
    unsigned tmem_base;
    uint64_t raw_full[NRAW], raw_empty[NRAW], op_full[NOP], op_empty[NOP], s_full[2], s_empty[2], p_full, p_empty;
    AttnJob job;
};

struct Args {
    AttnJob one;
    int cph, ntasks;        // CTAs per kv head; tasks per kv head when a host-built list is given
    const AttnTask * tasks; // optional list (position-range jobs)
    float * part;           // [CTA][AR][HD]
    float2 * ml;            // [CTA][AR]
    unsigned long long * xa; // [kv head][chunk][group][AR]: the group's own row maxima {tag, value}
    unsigned long long * xb; // same shape: row maxima of the chunk up to and including the group
    int nbmax, epoch;
    int * status;
    unsigned long long * prof; // optional: [CTA][16 groups][20] globaltimer stamps of worker warp 0 (0 .. 15) and the issuer (16 .. 19)
};
#define TC_STAMP(grp, k)                                                                                               \
    do {                                                                                                               \
        if (a.prof && lane == 0 && (warp == 0 || warp == NWORK) && (grp) < 16)                                         \
            a.prof[((size_t) blockIdx.x * 16 + (grp)) * 20 + (k)] = globaltimer_ns();                                  \
    } while (0)

// ---- tcgen05 ----
__device__ __forceinline__ uint64_t smem_desc(unsigned addr, unsigned lbo, unsigned sbo) { // no swizzle, version 1
    return (uint64_t) ((addr >> 4) & 0x3fffu) | ((uint64_t) ((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t) ((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// D[128 x 48] (+)= A B, fp16 operands, fp32 accumulate; MN: both operands MN-major, else both K-major
constexpr unsigned IDESC_K = (1u << 4) | ((unsigned) (AR / 8) << 17) | ((unsigned) (GP / 16) << 24);
constexpr unsigned IDESC_MN = IDESC_K | (1u << 15) | (1u << 16);
__device__ __forceinline__ void umma(unsigned d_tmem, uint64_t da, uint64_t db, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// 12 consecutive columns of the warp's 32 lanes (thread: lane, 12 values)
__device__ __forceinline__ void tmem_ld12(unsigned taddr, float (&v)[RS]) {
    unsigned r[RS];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]) : "r"(taddr + 8));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < RS; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st12(unsigned taddr, const float (&v)[RS]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(__float_as_uint(v[0])),
                 "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
                 "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
                 : "memory");
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr + 8), "r"(__float_as_uint(v[8])),
                 "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11]))
                 : "memory");
}

// ---- one worker step: position `row` of a staged tile, dims 32 jb .. 32 jb + 31 -> four 16-byte operand units ----
// FMT 0 .. 3: rows of 4 + FMT bits; FMT 4: q8_0 rows. dst: the thread's unit of dim group 4 (jb & 3) of the slot; the next
// dim groups are 2048 bytes apart. valid false (a row past the chunk end holds stale bytes): zeros.
template <int FMT> __device__ __forceinline__ void dq_item(const uint8_t * raw, int row, int jb, bool valid, uint8_t * dst) {
    constexpr int HB = FMT < 4 ? FMT : 0;
    constexpr int RB = FMT < 4 ? 32 * (4 + FMT) : HD;
    const __half2 sub = __half2half2(__float2half_rn(FMT < 4 ? 1024.f + (float) (1 << (3 + FMT)) : 1152.f));
    const __half dsc = valid ? reinterpret_cast<const __half *>(raw + TILE_SC_OFF)[row * 8 + jb] : __float2half_rn(0.f);
    const __half2 d = __half2half2(dsc);
    const uint8_t * rp = raw + row * RB;
    if constexpr (FMT == 4) {
        const uint4 v0 = *reinterpret_cast<const uint4 *>(rp + 32 * jb), v1 = *reinterpret_cast<const uint4 *>(rp + 32 * jb + 16);
        const unsigned w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const unsigned x0 = w[2 * u] ^ 0x80808080u, x1 = w[2 * u + 1] ^ 0x80808080u; // q + 128
            *reinterpret_cast<uint4 *>(dst + u * 2048) =
                make_uint4(cvt_pair<0>(x0, sub, d), cvt_pair<1>(x0, sub, d), cvt_pair<0>(x1, sub, d), cvt_pair<1>(x1, sub, d));
        }
    } else {
        const uint4 nv = *reinterpret_cast<const uint4 *>(rp + 16 * jb);
        const unsigned nw[4] = {nv.x, nv.y, nv.z, nv.w};
        unsigned hw[4] = {0u, 0u, 0u, 0u};
        if constexpr (HB == 1) {
            const unsigned h = *reinterpret_cast<const unsigned *>(rp + 128 + 4 * jb);
            hw[0] = h, hw[1] = h >> 8, hw[2] = h >> 16, hw[3] = h >> 24;
        } else if constexpr (HB == 2) {
            const uint2 h = *reinterpret_cast<const uint2 *>(rp + 128 + 8 * jb);
            hw[0] = h.x, hw[1] = h.x >> 16, hw[2] = h.y, hw[3] = h.y >> 16;
        } else if constexpr (HB == 3) {
            const unsigned * hp = reinterpret_cast<const unsigned *>(rp + 128 + 12 * jb);
            const unsigned h0 = hp[0], h1 = hp[1], h2 = hp[2];
            hw[0] = h0, hw[1] = __funnelshift_r(h0, h1, 24), hw[2] = __funnelshift_r(h1, h2, 16), hw[3] = h2 >> 8;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const unsigned x0 = quad_bytes<HB>(nw[u], hw[u], 0), x1 = quad_bytes<HB>(nw[u], hw[u], 1);
            *reinterpret_cast<uint4 *>(dst + u * 2048) =
                make_uint4(cvt_pair<0>(x0, sub, d), cvt_pair<1>(x0, sub, d), cvt_pair<0>(x1, sub, d), cvt_pair<1>(x1, sub, d));
        }
    }
}
__device__ __forceinline__ void dq_item_any(int bits, const uint8_t * raw, int row, int jb, bool valid, uint8_t * dst) {
    switch (bits) {
    case 4: dq_item<0>(raw, row, jb, valid, dst); break;
    case 5: dq_item<1>(raw, row, jb, valid, dst); break;
    case 6: dq_item<2>(raw, row, jb, valid, dst); break;
    case 7: dq_item<3>(raw, row, jb, valid, dst); break;
    default: dq_item<4>(raw, row, jb, valid, dst); break;
    }
}

// order-preserving map float <-> int (for redux.sync.max)
__device__ __forceinline__ int f2key(float x) {
    const int i = __float_as_int(x);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float key2f(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }

// bounded poll of an exchange word until it carries this launch's tag
__device__ __forceinline__ float poll_word(const unsigned long long * src, unsigned long long w, int epoch, int * status) {
    if ((unsigned) (w >> 32) != (unsigned) epoch) {
        const unsigned long long t0 = globaltimer_ns();
        for (unsigned it = 0;; it++) {
            w = __ldcv(src);
            if ((unsigned) (w >> 32) == (unsigned) epoch) break;
            if ((it & 255u) == 255u && globaltimer_ns() - t0 > 2000000000ull) {
                atomicExch(status, (int) KS_WAIT_TIMEOUT);
                break;
            }
        }
    }
    return __uint_as_float((unsigned) w);
}

__global__ void __launch_bounds__(NTHREADS, 1) attn_tc_kernel(const __grid_constant__ Args a) {
    extern __shared__ uint8_t smem_raw[];
    Smem & sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t) 127);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    {
        const unsigned * src = reinterpret_cast<const unsigned *>(&a.one);
        unsigned * dst = reinterpret_cast<unsigned *>(&sm.job);
        for (int i = tid; i < (int) (sizeof(AttnJob) / 4); i += NTHREADS) dst[i] = src[i];
    }
    if (tid == 0) {
        for (int s = 0; s < NRAW; s++) { mbar_init(&sm.raw_full[s], 1); mbar_init(&sm.raw_empty[s], NWORK / GT); }
        for (int s = 0; s < NOP; s++) { mbar_init(&sm.op_full[s], NWORK); mbar_init(&sm.op_empty[s], 1); }
        for (int s = 0; s < 2; s++) { mbar_init(&sm.s_full[s], 1); mbar_init(&sm.s_empty[s], NWORK); }
        mbar_init(&sm.p_full, NWORK);
        mbar_init(&sm.p_empty, 1);
        sm.resc[0] = sm.resc[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == NWORK) { // tensor memory: S^T twice, O^T in two halves
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();
    const AttnJob & J = sm.job;
    const KvView & kv = J.kv;
    const int g = blockIdx.x / a.cph, kk = blockIdx.x % a.cph, slot = blockIdx.x;
    const int T = J.T, n = J.n, R = GQ * T, ws = J.ws;
    const Geo geo = make_geo(J, GT);
    const AttnTask * const ttab = a.tasks;
    const int t_end = ttab ? a.ntasks : geo.ntasks_head;
    auto get_task = [&](int t) -> Task { return ttab ? ttab[t] : make_task(geo, GT, 0, t, 0); };
    const int G = kk < t_end ? (t_end - kk + a.cph - 1) / a.cph : 0; // this CTA's groups: tasks kk, kk + cph, ..

    // query rows of the kv head: fp16 -> fp32 -> (K's rotation) -> x 1/16 -> fp16 (qwen38_mk.cu:2876-2883), row = (head % 6) T + t,
    // as the K-major B operand: lane holds dims 8 lane .. + 7 = one 16-byte unit
    for (int r = warp; r < AR; r += NTHREADS / 32) {
        uint4 out = make_uint4(0, 0, 0, 0);
        if (r < R) {
            const uint4 rawq = *reinterpret_cast<const uint4 *>(J.Q + ((size_t) (r % T) * NH + g * GQ + r / T) * HD + lane * 8);
            const __half2 * hh = reinterpret_cast<const __half2 *>(&rawq);
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
        *reinterpret_cast<uint4 *>(sm.q + lane * (AR / 8 * 128) + (r >> 3) * 128 + (r & 7) * 16) = out;
    }
    if (tid < AR) sm.rtok[tid] = (unsigned char) (tid % T);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tb = sm.tmem_base;

    if (warp == NWORK + 1) {
        // ---- producer: K(0), K(1), then V(i), K(i + 2) -- the order the workers consume ----
        if (lane == 0) {
            const SideSrc ksrc = make_src(kv, 0, g, ws), vsrc = make_src(kv, 1, g, ws);
            unsigned rseq = 0;
            auto load_unit = [&](const SideSrc & S, int i) {
                const Task k = get_task(kk + i * a.cph);
                for (int qq = 0; qq < GT; qq++, rseq++) {
                    const int rs = rseq % NRAW;
                    const unsigned round = rseq / NRAW;
                    if (round > 0) mbar_wait(&sm.raw_empty[rs], (round - 1) & 1, a.status);
                    if (qq < k.nt) issue_tile(S, k.pos0 + qq * ATP, k.c1, sm.raw[rs], &sm.raw_full[rs]);
                    else mbar_arrive(&sm.raw_full[rs]);
                }
            };
            if (G > 0) load_unit(ksrc, 0);
            if (G > 1) load_unit(ksrc, 1);
            for (int i = 0; i < G; i++) {
                load_unit(vsrc, i);
                if (i + 2 < G) load_unit(ksrc, i + 2);
            }
        }
    } else if (warp == NWORK) {
        // ---- issuer: S(0), S(1), then PV(i), S(i + 2) ----
        if (lane == 0) {
            unsigned oseq = 0;
            const unsigned qaddr = smem_u32(sm.q), phi = smem_u32(sm.p[0]), plo = smem_u32(sm.p[1]);
            auto do_S = [&](int j) {
                if (j >= 2) mbar_wait(&sm.s_empty[j & 1], ((j >> 1) - 1) & 1, a.status);
                const unsigned dcol = tb + ((j & 1) ? S_COL1 : S_COL0);
                for (int h = 0; h < 2; h++, oseq++) {
                    const int os = oseq % NOP;
                    mbar_wait(&sm.op_full[os], (oseq / NOP) & 1, a.status);
                    tc_fence_after();
                    const unsigned ab = smem_u32(sm.op[os]);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)
                        umma(dcol, smem_desc(ab + ks * 4096, 2048, 128), smem_desc(qaddr + (8 * h + ks) * (2 * AR / 8 * 128), AR / 8 * 128, 128), IDESC_K,
                             (unsigned) (h | ks));
                    umma_commit(&sm.op_empty[os]);
                }
                umma_commit(&sm.s_full[j & 1]);
            };
            auto do_PV = [&](int i) {
                TC_STAMP(i, 16);
                mbar_wait(&sm.p_full, i & 1, a.status);
                TC_STAMP(i, 17);
                for (int h = 0; h < 2; h++, oseq++) {
                    const int os = oseq % NOP;
                    mbar_wait(&sm.op_full[os], (oseq / NOP) & 1, a.status);
                    if (h == 0) TC_STAMP(i, 18);
                    tc_fence_after();
                    const unsigned ab = smem_u32(sm.op[os]), dcol = tb + (h ? O_COL1 : O_COL0);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint64_t da = smem_desc(ab + ks * 256, 128, 2048);
                        umma(dcol, da, smem_desc(phi + ks * 256, 128, 2048), IDESC_MN, (unsigned) (i | ks));
                        umma(dcol, da, smem_desc(plo + ks * 256, 128, 2048), IDESC_MN, 1u);
                    }
                    umma_commit(&sm.op_empty[os]);
                }
                umma_commit(&sm.p_empty);
                TC_STAMP(i, 19);
            };
            if (G > 0) do_S(0);
            if (G > 1) do_S(1);
            for (int i = 0; i < G; i++) {
                do_PV(i);
                if (i + 2 < G) do_S(i + 2);
            }
        }
    } else {
        // ---- workers: warp = 4 c + q: tile q (positions 32 q .. + 31 of a group, tensor-memory lanes 32 q ..), query rows
        // 12 c .. 12 c + 11 in the softmax, dims 32 (4 h + c) .. + 31 of half h in the unpacking ----
        const int q = warp & 3, c = warp >> 2, prow = ATP * q + lane;
        const unsigned pos_off = (prow >> 3) * 128 + (prow & 7) * 16; // the position's 16-byte unit inside a dim / row group
        const unsigned lane_addr = tb + ((unsigned) (ATP * q) << 16);
        const bool owner = q == 0 && lane < RS; // owns query row r_own: its running / reference max, the exchange
        const int r_own = RS * c + (lane < RS ? lane : 0);
        unsigned rseq = 0, oseq = 0;
        float l_acc[RS], s[RS];
#pragma unroll
        for (int i = 0; i < RS; i++) l_acc[i] = 0.f, s[i] = 0.f;
        float m_acc = -CUDART_INF_F;
        unsigned long long w0 = 0, w1 = 0, w2 = 0;

        // both 128-dim halves of one side of a group: packed rows -> operand slots
        auto unpack = [&](int side, const Task & k, int grp) {
            const int rs = (rseq + q) % NRAW;
            mbar_wait(&sm.raw_full[rs], ((rseq + q) / NRAW) & 1, a.status);
            TC_STAMP(grp, side ? 6 : 11);
            const int tbq = k.pos0 + q * ATP;
            const bool valid = q < k.nt && lane < k.c1 - tbq;
            const int bits = (kv.s[side].rval && tbq >= ws) ? 8 : kv.s[side].bits;
            for (int h = 0; h < 2; h++, oseq++) {
                const int os = oseq % NOP;
                const unsigned round = oseq / NOP;
                if (round > 0) mbar_wait(&sm.op_empty[os], (round - 1) & 1, a.status);
                TC_STAMP(grp, (side ? 7 : 12) + 2 * h);
                dq_item_any(bits, sm.raw[rs], lane, 4 * h + c, valid, sm.op[os] + 4 * c * 2048 + pos_off);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.op_full[os]);
                TC_STAMP(grp, (side ? 8 : 13) + 2 * h);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.raw_empty[rs]);
            rseq += GT;
        };
        auto xbase = [&](const Task & k) -> size_t { return (((size_t) g * ATT_NCH + k.c) * a.nbmax) * AR + r_own; };

        // S^T of group j is complete: scores to registers, mask, tile maxima, the group's own maxima published, the words
        // the running max will need requested
        auto scores = [&](int j, const Task & k) {
            mbar_wait(&sm.s_full[j & 1], (j >> 1) & 1, a.status);
            TC_STAMP(j - 1, 4);
            tc_fence_after();
            tmem_ld12(lane_addr + ((j & 1) ? S_COL1 : S_COL0) + RS * c, s);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.s_empty[j & 1]);
            const int p_abs = k.pos0 + prow;
            if (k.pos0 + GP - 1 > min(k.c1 - 1, n) || R < AR) { // (uniform) row token t sees positions <= n + t; chunk end; padding rows
#pragma unroll
                for (int i = 0; i < RS; i++) {
                    const int r = RS * c + i, lim = min(k.c1 - 1, n + (int) sm.rtok[r]);
                    if (p_abs > lim || r >= R) s[i] = -CUDART_INF_F;
                }
            }
            float mx[RS];
#pragma unroll
            for (int i = 0; i < RS; i++) mx[i] = key2f(__reduce_max_sync(FULL_MASK, f2key(s[i])));
            if (lane == 0) {
                float4 * d = reinterpret_cast<float4 *>(&sm.tmax[q][RS * c]);
                d[0] = make_float4(mx[0], mx[1], mx[2], mx[3]);
                d[1] = make_float4(mx[4], mx[5], mx[6], mx[7]);
                d[2] = make_float4(mx[8], mx[9], mx[10], mx[11]);
            }
            named_bar(1 + c, 4 * 32);
            if (owner && k.nb > 1) {
                const size_t xb0 = xbase(k);
                if (k.b + 1 < k.nb) {
                    const float gm = fmaxf(fmaxf(sm.tmax[0][r_own], sm.tmax[1][r_own]), fmaxf(sm.tmax[2][r_own], sm.tmax[3][r_own]));
                    __stcg(a.xa + xb0 + (size_t) k.b * AR, ((unsigned long long) (unsigned) a.epoch << 32) | __float_as_uint(gm));
                }
                if (k.b >= 1) w1 = __ldcv(a.xa + xb0 + (size_t) (k.b - 1) * AR);
                if (k.b >= 2) w2 = __ldcv(a.xa + xb0 + (size_t) (k.b - 2) * AR);
                if (k.b >= 3) w0 = __ldcv(a.xb + xb0 + (size_t) (k.b - 3) * AR);
            }
            TC_STAMP(j - 1, 5);
        };

        // P of group i from the scores in registers
        auto softmax = [&](int i, const Task & k) {
            const int par = i & 1;
            TC_STAMP(i, 0);
            if (owner) {
                float m_in = -CUDART_INF_F;
                const size_t xb0 = xbase(k);
                if (k.nb > 1) {
                    if (k.b >= 1) m_in = poll_word(a.xa + xb0 + (size_t) (k.b - 1) * AR, w1, a.epoch, a.status);
                    if (k.b >= 2) m_in = fmaxf(m_in, poll_word(a.xa + xb0 + (size_t) (k.b - 2) * AR, w2, a.epoch, a.status));
                    if (k.b >= 3) m_in = fmaxf(m_in, poll_word(a.xb + xb0 + (size_t) (k.b - 3) * AR, w0, a.epoch, a.status));
                }
                float mr[GT], m = m_in;
#pragma unroll
                for (int t = 0; t < GT; t++) {
                    m = fmaxf(m, sm.tmax[t][r_own]);
                    mr[t] = m;
                    sm.mrun[par][t][r_own] = m;
                }
                if (k.nb > 1 && k.b + 3 < k.nb) __stcg(a.xb + xb0 + (size_t) k.b * AR, ((unsigned long long) (unsigned) a.epoch << 32) | __float_as_uint(m));
                float f = 1.f;
                if (m != -CUDART_INF_F) {
                    if (m_acc == -CUDART_INF_F) m_acc = m;
                    else if (m > m_acc + REF_SLACK) {
                        f = expf(m_acc - m);
                        m_acc = m;
                    }
                }
#pragma unroll
                for (int t = 0; t < GT; t++) sm.beta[par][t][r_own] = mr[t] == -CUDART_INF_F ? 0.f : expf(mr[t] - m_acc);
                sm.fsc[par][r_own] = f;
                if (f != 1.f) atomicOr(&sm.resc[par], 1);
            }
            named_bar(5, NWORK * 32);
            if (tid == 0) sm.resc[par ^ 1] = 0;
            TC_STAMP(i, 1);
            if (i > 0) mbar_wait(&sm.p_empty, (i - 1) & 1, a.status); // P V of the previous group is complete: P is free, O^T at rest
            TC_STAMP(i, 2);
            tc_fence_after();
            if (sm.resc[par]) { // a reference max moved: bring the accumulator rows (and the row sums) to it
                float fs[RS], v[RS];
#pragma unroll
                for (int j = 0; j < RS; j++) fs[j] = sm.fsc[par][RS * c + j];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const unsigned ad = lane_addr + (h ? O_COL1 : O_COL0) + RS * c;
                    tmem_ld12(ad, v);
#pragma unroll
                    for (int j = 0; j < RS; j++) v[j] *= fs[j];
                    tmem_st12(ad, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < RS; j++) l_acc[j] *= fs[j];
            }
            float mq[RS], bq[RS];
            {
                const float4 * mp = reinterpret_cast<const float4 *>(&sm.mrun[par][q][RS * c]);
                const float4 * bp = reinterpret_cast<const float4 *>(&sm.beta[par][q][RS * c]);
#pragma unroll
                for (int j = 0; j < 3; j++) {
                    const float4 mv = mp[j], bv = bp[j];
                    mq[4 * j] = mv.x, mq[4 * j + 1] = mv.y, mq[4 * j + 2] = mv.z, mq[4 * j + 3] = mv.w;
                    bq[4 * j] = bv.x, bq[4 * j + 1] = bv.y, bq[4 * j + 2] = bv.z, bq[4 * j + 3] = bv.w;
                }
            }
            unsigned hi2[RS / 2], lo2[RS / 2];
#pragma unroll
            for (int j = 0; j < RS / 2; j++) {
                float p0 = 0.f, p1 = 0.f;
                if (mq[2 * j] != -CUDART_INF_F) p0 = expf(s[2 * j] - mq[2 * j]);
                if (mq[2 * j + 1] != -CUDART_INF_F) p1 = expf(s[2 * j + 1] - mq[2 * j + 1]);
                l_acc[2 * j] = __fmaf_rn(bq[2 * j], p0, l_acc[2 * j]);
                l_acc[2 * j + 1] = __fmaf_rn(bq[2 * j + 1], p1, l_acc[2 * j + 1]);
                const float2 pf = __half22float2(__floats2half2_rn(p0, p1)); // the reference's fp16 P
                const float x0 = __fmul_rn(pf.x, bq[2 * j]), x1 = __fmul_rn(pf.y, bq[2 * j + 1]);
                const __half2 hh = __floats2half2_rn(x0, x1);
                const float2 hf = __half22float2(hh);
                const __half2 ll = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
                hi2[j] = *reinterpret_cast<const unsigned *>(&hh);
                lo2[j] = *reinterpret_cast<const unsigned *>(&ll);
            }
            // rows 12 c .. 12 c + 11 of position prow: row group (12 c) >> 3 from its row (12 c) & 7 (0 or 4) on, then the next
            {
                const int ng0 = (RS * c) >> 3;
                uint8_t * ph = sm.p[0] + ng0 * 2048 + pos_off;
                uint8_t * pl = sm.p[1] + ng0 * 2048 + pos_off;
                if (c & 1) {
                    *reinterpret_cast<uint2 *>(ph + 8) = make_uint2(hi2[0], hi2[1]);
                    *reinterpret_cast<uint4 *>(ph + 2048) = make_uint4(hi2[2], hi2[3], hi2[4], hi2[5]);
                    *reinterpret_cast<uint2 *>(pl + 8) = make_uint2(lo2[0], lo2[1]);
                    *reinterpret_cast<uint4 *>(pl + 2048) = make_uint4(lo2[2], lo2[3], lo2[4], lo2[5]);
                } else {
                    *reinterpret_cast<uint4 *>(ph) = make_uint4(hi2[0], hi2[1], hi2[2], hi2[3]);
                    *reinterpret_cast<uint2 *>(ph + 2048) = make_uint2(hi2[4], hi2[5]);
                    *reinterpret_cast<uint4 *>(pl) = make_uint4(lo2[0], lo2[1], lo2[2], lo2[3]);
                    *reinterpret_cast<uint2 *>(pl + 2048) = make_uint2(lo2[4], lo2[5]);
                }
            }
            fence_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_full);
            TC_STAMP(i, 3);
        };

        if (G > 0) {
            Task kc = get_task(kk), kn = kc, k2 = kc;
            unpack(0, kc, 99);
            if (G > 1) {
                kn = get_task(kk + a.cph);
                unpack(0, kn, 99);
            }
            scores(0, kc);
            for (int i = 0; i < G; i++) {
                softmax(i, kc);
                if (i + 1 < G) scores(i + 1, kn);
                unpack(1, kc, i);
                if (i + 2 < G) {
                    k2 = get_task(kk + (i + 2) * a.cph);
                    unpack(0, k2, i);
                }
                kc = kn;
                kn = k2;
            }
            mbar_wait(&sm.p_empty, (G - 1) & 1, a.status);
            tc_fence_after();
        }
        // ---- the CTA's partial: O^T lanes are dims, columns are query rows ----
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float v[RS];
            if (G > 0) tmem_ld12(lane_addr + (h ? O_COL1 : O_COL0) + RS * c, v);
#pragma unroll
            for (int j = 0; j < RS; j++) {
                const int r = RS * c + j;
                if (r < R) a.part[((size_t) slot * AR + r) * HD + 128 * h + prow] = G > 0 ? v[j] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < RS; j++) {
            float x = l_acc[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(FULL_MASK, x, o);
            if (lane == 0) sm.lsum[q][RS * c + j] = x;
        }
        named_bar(5, NWORK * 32);
        if (owner && r_own < R)
            a.ml[(size_t) slot * AR + r_own] = make_float2(m_acc, sm.lsum[0][r_own] + sm.lsum[1][r_own] + sm.lsum[2][r_own] + sm.lsum[3][r_own]);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == NWORK) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(TMEM_COLS) : "memory");
}

} // namespace tc

size_t attend_tc_smem_bytes() { return sizeof(tc::Smem) + 128; }

cudaError_t launch_attend_tc(const AttnJob & job, int num_sms, float * part, float2 * ml, int part_slots, unsigned long long * xa,
                             unsigned long long * xb, int nbmax, int epoch, int * status, cudaStream_t stream, const AttnTask * tasks_dev,
                             int ntasks, int tasks_B, float * raw_part, float2 * raw_ml, unsigned long long * prof) {
    tc::Args a;
    a.prof = prof;
    a.one = job;
    a.cph = num_sms / NKV;
    if (a.cph < 1 || a.cph > 64 || NKV * a.cph > part_slots) return cudaErrorNotSupported; // (the merge keeps a head's weights in two registers per lane)
    a.tasks = nullptr;
    a.ntasks = 0;
    if (tasks_dev) {
        if (tasks_B != tc::GT) return cudaErrorNotSupported;
        a.tasks = tasks_dev;
        a.ntasks = ntasks;
    } else {
        const int nt_full = job.cs / ATP;
        if ((nt_full + tc::GT - 1) / tc::GT > nbmax) return cudaErrorNotSupported;
    }
    a.part = part;
    a.ml = ml;
    a.xa = xa;
    a.xb = xb;
    a.nbmax = nbmax;
    a.epoch = epoch;
    a.status = status;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(tc::attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) attend_tc_smem_bytes());
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    void * args[] = {&a};
    e = cudaLaunchCooperativeKernel((const void *) tc::attn_tc_kernel, dim3(NKV * a.cph), dim3(tc::NTHREADS), args, attend_tc_smem_bytes(), stream);
    if (e != cudaSuccess) return e;
    AttnJob merge_job = job;
    merge_job.nch = a.cph; // the merge reads cph partials per kv head, slots g cph ..
    merge_job.item0 = 0;
    return launch_merge(nullptr, &merge_job, 1, job.T, part, ml, stream, raw_part, raw_ml);
}

} // namespace mkkv
