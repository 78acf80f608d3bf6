// Decode attention on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory) for one sequence spread over
// every SM. Same arithmetic as the other attention kernel (the reference's attn_core_t, qwen38_mk.cu:2756-3067): the
// chunk partition attn_dims, 32-position tiles in order inside a chunk with a running max, P = fp16(exp(S - max)), fp32
// accumulation. The structure is a warp-specialised dequantising GEMM main loop:
//   - the unit of work is a group of 4 consecutive tiles (128 positions) of one chunk; the groups of a kv head are dealt in
//     group-major order to the CTAs of that head (cooperative launch: all CTAs resident);
//   - four producer lanes (a tile each) stream the packed K / V rows of the CTA's groups into a ring of shared-memory slots with
//     bulk copies completing on mbarriers;
//   - 16 unpack warps turn packed rows into exact fp16(d * q) operands in the canonical no-swizzle UMMA layouts (one thread:
//     one position x 32 dims per step; the fp16 pairs are assembled straight from the nibble words and high-bit fields with one
//     AND-OR each, kv_unpack.h, which leaves the 8 dims of a 16-byte unit in the order UNIT_PERM: the queries are staged in the
//     same order and the output dims are mapped back) -- K as the K-major A operand of S^T[128 pos x 48 rows] = K Q^T, V as the
//     MN-major A operand of O^T[256 dims x 48 rows] += V^T P^T;
//   - the queries arrive staged (qprep in kv_kernels.cu: rotated when K is, x 1/16, fp16, in the B operand's layout; made once per
//     (job, kv head) by the decode step's append launch or a small launch of its own) and are fetched with one bulk copy;
//   - one issuer thread runs tcgen05.mma on the slots as they fill (mbarrier "full" from the unpack warps, tcgen05.commit
//     to "empty"), S^T in five tensor-memory buffers (K runs five groups ahead of V), O^T (two 128-dim halves) resident there
//     for the whole kernel;
//   - 8 softmax warps read S^T back (tcgen05.ld: a thread owns one position and 24 query rows), take the tile maxima (two
//     groups ahead of P, so that a group's own maxima are published long before another CTA needs them), exchange the running
//     max with the CTAs that hold the chunk's earlier groups through small global arrays (own group maxima and cumulative
//     maxima, 8-byte {launch tag, value} words, polled with a bound), and write P to shared memory as the B operand. The
//     accumulator is kept against a per-row reference max that moves rarely (when the running max passes it by more than 10.5;
//     then the moved rows' accumulator columns are rescaled, one tensor-memory column per row and block): P, after its fp16 rounding, is multiplied by exp(running max - reference) and carried as an fp16
//     high and low part (one N = 96 MMA per k-step, two 48-column accumulator blocks), so the reference's fp16 P is reproduced
//     and no per-tile accumulator rescale is needed;
//   - a CTA writes one un-normalised partial (m, l, O); when the CTAs of a kv head have all written theirs (arrival count,
//     bounded wait) each merges one or two of the head's rows in the kernel's tail, four warps to a row;
//   - batch mode (several jobs): one CTA per (job, kv head, run of cpi chunks) in a plain launch, the chunks' groups in order on
//     that CTA with the running max carried in registers and started anew at every chunk; attn_merge_kernel afterwards.
// Every wait is bounded (about two seconds by default; the limits are launch arguments), then the status word and a CTA-wide
// flag are set, no later wait of the CTA blocks, the producer waits (bounded) for its copies still in flight, and the kernel
// runs to its end and frees its tensor memory.
#include <algorithm>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kv_attend_common.cuh"
#include "kv_kernels.h"
#include "kv_merge.cuh"
#include "kv_quant.cuh"
#include "kv_unpack.h"
#include "kv_attend_tc_unpack.cuh"

namespace mkkv {

namespace tc {

using namespace attn_common;

#ifndef MKKV_TC_NDQ
#define MKKV_TC_NDQ 16 // unpack warps: 16 (one 32-dim block of a half each, 28 warps per CTA) or 8 (two blocks each, 20 warps: measured
                       // 115 us against 105 on the one-layer case, the unpack needs the warps)
#endif
constexpr int NSL = 2;         // row slices of the softmax warps: 24 query rows each
constexpr int NSOFT = 4 * NSL; // softmax warps first: warp = 4 c2 + q, tile q (tensor-memory lanes 32 q ..), query rows RS c2 .. + RS - 1
constexpr int NDQ = MKKV_TC_NDQ; // then the unpack warps: 4 c + q, tile q, 32-dim blocks c, c + NDQ / 4, .. of each 128-dim half
constexpr int BPW = 16 / NDQ;  // blocks of a half per unpack warp
constexpr int W_ISSUE = NSOFT + NDQ, W_PROD = W_ISSUE + 1;
constexpr int NTHREADS = (W_PROD + 3) * 32; // two idle warps complete the last group of four (register reallocation is per group)
constexpr int GT = 4, GP = GT * ATP;        // tiles / positions per group: the M of one MMA
constexpr int RS = AR / NSL;                // query rows per softmax warp
// registers per thread after the reallocation (the launch gives 65536 / NTHREADS rounded down to 8; the three shares sum to at
// most the CTA's launch allocation -- a larger sum faults)
#if MKKV_TC_NDQ == 8
#define MKKV_TC_REGS_SOFT "128"
#define MKKV_TC_REGS_DQ "80"
#define MKKV_TC_REGS_CTL "56"
static_assert(NTHREADS == 640 && 8 * 128 + 8 * 80 + 4 * 56 <= 20 * 96, "register shares");
#else
#define MKKV_TC_REGS_SOFT "112"
#define MKKV_TC_REGS_DQ "56"
#define MKKV_TC_REGS_CTL "56"
static_assert(NTHREADS == 896 && 8 * 112 + 16 * 56 + 4 * 56 <= 28 * 72, "register shares");
#endif
constexpr int RAW_SLOT = ATP * HD + ATP * SCALE_ROW; // one tile of the widest format and its scales: 8704 bytes
constexpr int NRAW = 8;                     // packed tile slots: two side-groups (one being unpacked, one in flight)
static_assert(NRAW % GT == 0, "whole groups only: a 7-slot ring, tried once, was 20 % slower and its results changed from run to run");
constexpr int OP_SLOT = GP * 128 * 2;       // fp16 operand: 128 positions x 128 dims
constexpr int NOP = 3;
constexpr int NSB = 5;                      // S^T buffers: K runs NSB groups ahead of V
constexpr int NTASK = 16;
constexpr int Q_BYTES = AR * HD * 2, P_BYTES = AR * GP * 2;
constexpr unsigned S_COL = 0, S_STRIDE = 64, O_COL0 = NSB * 64, O_COL1 = O_COL0 + 2 * AR, TMEM_COLS = 512; // an O^T half: 48 columns for P's high part, 48 for its low part
static_assert(O_COL1 + 2 * AR <= TMEM_COLS, "tensor-memory columns");
static_assert(Q_BYTES == QP_HEAD_BYTES, "the staged query block of a kv head");
// The accumulator's reference max of a row is set REF_MARGIN above the running max it is taken from and moves when the running max
// passes it by more than REF_SLACK: exp(running - reference) stays within [e^-3 for the row's largest terms, e^10.5 < fp16 max].
constexpr float REF_SLACK = 10.5f, REF_MARGIN = 3.f;
constexpr float LOG2E = 1.4426950408889634f;

struct WaitCtl { // the launch's wait limits and the CTA's give-up flag
    int dead;
    unsigned hint, rounds, poll; // nanoseconds per failed try, failed tries of an mbarrier wait, failed polls of a global word
};

struct WarpScratch { // what the row-owner lanes of a softmax warp hand to all its lanes
    float m[RS];     // running max of the warp's tile (+inf where nothing is visible yet: exp2 gives 0)
    float beta[RS];  // exp(running max - reference max)
    float f[RS];     // factor of a moved reference max
    unsigned bh[RS / 2], bl[RS / 2]; // beta as fp16 high + low parts, rows (2 j, 2 j + 1) packed
};

struct Smem {
    uint8_t op[NOP][OP_SLOT];   // [dim group 16][position group 16][8 positions][8 dims] fp16
    uint8_t raw[NRAW][RAW_SLOT];
    uint8_t q[Q_BYTES];         // [dim group 32][row group 6][8 rows][8 dims]
    uint8_t p[2][P_BYTES];      // high / low part: [row group 6][position group 16][8 positions][8 rows]
    float tmax[4][GT][AR];      // row maxima of a group's tiles; by group % 4: a group's maxima are read while those of the next two
                                // groups exist or are being written, and a warp is never a whole group ahead of its slice.
                                // The first buffer holds the row sums at the end.
    WarpScratch ws[NSOFT];
    unsigned tmem_base;
    int merge_ok;               // the tail's merge: the head's CTAs have all arrived
    WaitCtl wc;                 // the launch's wait limits; dead: a wait of this CTA gave up, no later wait blocks
    AttnTask tasks[NTASK];      // the CTA's groups as the producer reaches them, by group % NTASK (no role is that far from it:
                                // the producer's K is at most NSB + 2 groups ahead of the softmax warps' group)
    uint64_t raw_full[NRAW], raw_empty[NRAW], op_full[NOP], op_empty[NOP], s_full[NSB], s_empty[NSB], p_full, p_empty, q_ready, fin;
    AttnJob job;
};

struct Args {
    AttnJob one;
    const AttnJob * jobs;   // batch mode: device array of njobs jobs, one CTA per (job, kv head, cpi chunks); else null: one job spread
    int njobs;              // over cph CTAs per kv head with the exchange of row maxima
    int cph, ntasks;        // CTAs per kv head; tasks per kv head when a host-built list is given
    const AttnTask * tasks; // optional list (position-range jobs)
    float * part;           // [CTA][AR][HD]
    float2 * ml;            // [CTA][AR]
    unsigned long long * xa; // [kv head][chunk][group][AR]: the group's own row maxima {tag, value}
    unsigned long long * xb; // same shape: row maxima of the chunk up to and including the group
    int nbmax, epoch;
    int * status;
    float * raw_part;       // fused merge, optional: the merged but un-normalised (m, l, O) per kv head goes here instead of O
    float2 * raw_ml;        // ([4][48][256] / [4][48]: the input of a later merge across GPUs)
    unsigned * done;        // fused merge: [kv head] count of CTAs whose partial is written, over all launches (wraps)
    unsigned done_target;   // the count that means "every CTA of the head, this launch"; done == null: separate merge launch
    unsigned long long * prof; // optional: [CTA][16 groups][20] globaltimer stamps: softmax warp 0 (0 .. 7), unpack warp 8 (8 .. 15),
                               // issuer (16 .. 19)
    unsigned wait_hint_ns, wait_rounds, poll_rounds; // limits of the waits: a failed mbarrier try suspends for up to wait_hint_ns,
                                                     // wait_rounds failed tries (poll_rounds failed polls of an exchange word) give up
};
#ifndef MKKV_ABL
#define MKKV_ABL 0 // experiments only (wrong results): 1 no unpack arithmetic, 2 no P arithmetic, 4 no tile maxima
#endif
#ifndef MKKV_TC_PROF
#define MKKV_TC_PROF 0 // 1: compile the phase stamps in (they cost a few per cent)
#endif
#if MKKV_TC_PROF
#define TC_STAMP(grp, k)                                                                                               \
    do {                                                                                                               \
        if (a.prof && lane == 0 && (grp) >= 0 && (grp) < 16)                                                           \
            a.prof[((size_t) blockIdx.x * 16 + (grp)) * 20 + (k)] = globaltimer_ns();                                  \
    } while (0)
#else
#define TC_STAMP(grp, k)                                                                                               \
    do {                                                                                                               \
    } while (0)
#endif

// Wait for a phase of an mbarrier. A failed try suspends the thread in hardware for up to the hinted time (it wakes when the phase
// completes), so waiting warps take next to no issue slots. Bounded: after `rounds` failed tries the status word and the CTA's
// `dead` flag are set; from then on no wait of this CTA blocks, and the kernel runs to its end.
constexpr unsigned WAIT_HINT_NS = 10000u, WAIT_ROUNDS = 200000u, POLL_ROUNDS = 1u << 21; // defaults: about two seconds each
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t * bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tc_wait(uint64_t * bar, unsigned parity, volatile WaitCtl * wc, int * status) {
    if (mbar_try_wait_hint(bar, parity, 0u)) return; // (the common case: no limit loaded)
    const unsigned hint = wc->hint, rounds = wc->rounds;
    for (unsigned it = 0; !mbar_try_wait_hint(bar, parity, hint); it++) {
        if (wc->dead) return;
        if (it >= rounds) {
            wc->dead = 1;
            atomicExch(status, (int) KS_WAIT_TIMEOUT);
            return;
        }
    }
}

// ---- tcgen05 ----
// Shared-memory matrix descriptors (no swizzle, version 1), as their 32-bit halves: the low half holds the start address and the
// byte distance between the two 8-element groups along K of one instruction ("leading"), the high half the distance between 8-row
// groups along M / N ("stride"). Only the low half changes between k-steps.
// D[128 x 48] (+)= A B, fp16 operands, fp32 accumulate; MN: both operands MN-major, else both K-major
constexpr unsigned IDESC_K = (1u << 4) | ((unsigned) (AR / 8) << 17) | ((unsigned) (GP / 16) << 24);
constexpr unsigned IDESC_MN = (1u << 4) | (1u << 15) | (1u << 16) | ((unsigned) (2 * AR / 8) << 17) | ((unsigned) (GP / 16) << 24); // N = 96
__device__ __forceinline__ void umma(unsigned d_tmem, unsigned a_lo, unsigned a_hi, unsigned b_lo, unsigned b_hi, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ unsigned desc_lo(unsigned addr, unsigned lbo) { return ((addr >> 4) & 0x3fffu) | (((lbo >> 4) & 0x3fffu) << 16); }
__device__ __forceinline__ unsigned desc_hi(unsigned sbo) { return ((sbo >> 4) & 0x3fffu) | (1u << 14); }
__device__ __forceinline__ void umma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned * p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// 8 consecutive columns, in flight until tmem_wait8 on the same registers (the wait names them so that no use can move above it)
__device__ __forceinline__ void tmem_ld8_async(unsigned taddr, unsigned (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait8(unsigned (&r)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])::"memory");
}
// 8 consecutive columns
__device__ __forceinline__ void tmem_ld8(unsigned taddr, float (&v)[8]) {
    unsigned r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st8(unsigned taddr, const float (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(__float_as_uint(v[0])),
                 "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
                 "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
                 : "memory");
}
#ifndef MKKV_TC_EXPF
#define MKKV_TC_EXPF 0 // 1: P through expf instead of ex2.approx (experiments)
#endif
// exp(x), relative error about 2^-21 (scale factors applied alike to the accumulator and the row sums)
__device__ __forceinline__ float exp_any(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(__fmul_rn(x, LOG2E)));
    return y;
}
// exp(x) for x <= 0 (and -inf -> 0)
__device__ __forceinline__ float exp_neg(float x) {
#if MKKV_TC_EXPF
    return expf(x);
#else
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(__fmul_rn(x, LOG2E)));
    return y;
#endif
}

// max over the warp (sm_100a: redux.sync on fp32)
__device__ __forceinline__ float warp_max(float x) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
    return r;
}

// bounded poll of an exchange word until it carries this launch's tag
__device__ __forceinline__ float poll_word(const unsigned long long * src, unsigned long long w, int epoch, volatile WaitCtl * wc, int * status) {
    if ((unsigned) (w >> 32) != (unsigned) epoch) {
        const unsigned rounds = wc->poll;
        for (unsigned it = 0; (unsigned) (w >> 32) != (unsigned) epoch; it++) {
            if (wc->dead) break;
            if (it >= rounds) { // (a round is a trip to the L2)
                wc->dead = 1;
                atomicExch(status, (int) KS_WAIT_TIMEOUT);
                break;
            }
            w = __ldcv(src);
        }
    }
    return __uint_as_float((unsigned) w);
}
// task t of a kv head (group-major over its chunks), 4 tiles per task; mul_*: ceil(2^32 / divisor) (exact quotients for t < 2^26)
struct Geo4 {
    Geo g;
    unsigned mul_nch, mul_nch1;
};
__device__ __forceinline__ Task make_task4(const Geo4 & G4, int t) {
    const Geo & g = G4.g;
    Task k;
    const int first = g.nb_last * g.nch;
    if (t < first) {
        k.b = g.nch > 1 ? (int) __umulhi((unsigned) t, G4.mul_nch) : t;
        k.c = t - k.b * g.nch;
    } else {
        const int u = t - first;
        const int qd = g.nch > 2 ? (int) __umulhi((unsigned) u, G4.mul_nch1) : u;
        k.b = g.nb_last + qd;
        k.c = u - qd * (g.nch - 1);
    }
    const int ntc = k.c == g.nch - 1 ? g.nt_last : g.nt_full;
    k.nb = (ntc + GT - 1) / GT;
    k.c1 = min(g.L, (k.c + 1) * g.cs);
    k.pos0 = k.c * g.cs + k.b * GP;
    k.nt = min(GT, ntc - k.b * GT);
    return k;
}

// KB / VB: the bits of the K / V main rows the instance is compiled for (0: any, decided per tile at run time). A compiled-in
// format leaves two unpack bodies per side (the format and the q8_0 ring) instead of five: a smaller instruction footprint.
// BATCH: the instance for several jobs (one CTA per job, kv head and run of chunks, no exchange between CTAs); the instance for one
// job spread over the SMs carries none of that mode's code (with both modes in one body the spread mode's loops came out 1.7 %
// slower).
template <int KB, int VB, bool BATCH> __global__ void __launch_bounds__(NTHREADS, 1) attn_tc_kernel(const __grid_constant__ Args a) {
    // (the dynamic shared memory starts on a 128-byte boundary -- there is no static shared memory in this kernel --, which is all the
    // bulk copies, matrix descriptors and barriers need; no pointer arithmetic here, so every access below is a shared-space one)
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem & sm = *reinterpret_cast<Smem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#if MKKV_TC_PROF
    const unsigned long long t_entry = globaltimer_ns();
#endif
    {
        const AttnJob * Jp = &a.one;
        if (BATCH) { // the job whose items contain this CTA
            int j = 0;
            while (j + 1 < a.njobs && (int) blockIdx.x >= a.jobs[j + 1].titem0) j++;
            Jp = &a.jobs[j];
        }
        const unsigned * src = reinterpret_cast<const unsigned *>(Jp);
        unsigned * dst = reinterpret_cast<unsigned *>(&sm.job);
        for (int i = tid; i < (int) (sizeof(AttnJob) / 4); i += NTHREADS) dst[i] = src[i];
    }
    if (tid == 0) {
        for (int s = 0; s < NRAW; s++) { mbar_init(&sm.raw_full[s], 1); mbar_init(&sm.raw_empty[s], NDQ / GT); }
        for (int s = 0; s < NOP; s++) { mbar_init(&sm.op_full[s], NDQ); mbar_init(&sm.op_empty[s], 1); }
        for (int s = 0; s < NSB; s++) { mbar_init(&sm.s_full[s], 1); mbar_init(&sm.s_empty[s], NSOFT); }
        mbar_init(&sm.p_full, NSOFT);
        mbar_init(&sm.p_empty, 1);
        mbar_init(&sm.fin, 1);
        mbar_init(&sm.q_ready, 1);
        sm.wc.dead = 0;
        sm.wc.hint = a.wait_hint_ns;
        sm.wc.rounds = a.wait_rounds;
        sm.wc.poll = a.poll_rounds;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == W_ISSUE) { // tensor memory: S^T five times, O^T in two halves
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const unsigned tb = sm.tmem_base;
    const AttnJob & J = sm.job;
    const KvView & kv = J.kv;
    // spread mode: CTA kk of kv head g runs tasks kk, kk + cph, .. of the head; batch mode: the CTA runs the groups of chunks c_first
    // .. c_first + cpi - 1 of kv head g of its job in order, chunk after chunk, the running max carried from group to group in
    // registers and started anew with every chunk; its partial is the head's slot number ci
    constexpr bool batch = BATCH;
    const int cpi = batch ? max(J.cpi, 1) : 1, nit = batch ? (J.nch + cpi - 1) / cpi : 1;
    const int item = batch ? (int) blockIdx.x - J.titem0 : 0, ci = item % nit;
    const int g = batch ? item / nit : (int) blockIdx.x / a.cph, kk = batch ? 0 : (int) blockIdx.x % a.cph;
    const int slot = batch ? J.item0 + g * J.nch + ci : (int) blockIdx.x;
    const int c_first = ci * cpi, c_count = batch ? min(cpi, J.nch - c_first) : 0, tstep = batch ? 1 : a.cph;
    const int T = J.T, n = J.n, R = GQ * T, ws = J.ws;
    Geo4 geo4;
    geo4.g = make_geo(J, GT);
    geo4.mul_nch = geo4.g.nch > 1 ? 0xffffffffu / (unsigned) geo4.g.nch + 1u : 0u;
    geo4.mul_nch1 = geo4.g.nch > 2 ? 0xffffffffu / (unsigned) (geo4.g.nch - 1) + 1u : 0u;
    const AttnTask * const ttab = a.tasks;
    // (batch mode: every chunk has nb_full groups but the job's last one, which is the last of its CTA too)
    const int t_end = batch ? c_count * geo4.g.nb_full - (c_first + c_count == geo4.g.nch ? geo4.g.nb_full - geo4.g.nb_last : 0)
                            : ttab ? a.ntasks : geo4.g.ntasks_head;
    auto get_task = [&](int t) -> Task {
        if (batch) {
            const int cc = t / geo4.g.nb_full;
            return make_task(geo4.g, GT, 1, t - cc * geo4.g.nb_full, c_first + cc);
        }
        return ttab ? ttab[t] : make_task4(geo4, t);
    };
    const int G = kk < t_end ? (t_end - kk + tstep - 1) / tstep : 0; // this CTA's groups: tasks kk, kk + tstep, ..

    // The kv head's query rows come staged (qprep: fp16 -> fp32 -> K's rotation -> x 1/16 -> fp16 in the K-major B operand's layout,
    // row = (head % 6) T + t): the producer fetches the block with one bulk copy, the issuer waits for it.
    // registers move from the unpack / control warps to the softmax warps
    if (warp >= W_ISSUE) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 " MKKV_TC_REGS_CTL ";");
    if (warp == W_PROD) {
        // ---- producer: K(0) .. K(NSB - 1), then V(i), K(i + NSB) -- the order the unpack warps consume. Lanes 0 .. 3 fetch one
        // tile of the group each ----
        if (lane == 0) { // the queries first
            mbar_expect_tx(&sm.q_ready, Q_BYTES);
            bulk_g2s(sm.q, reinterpret_cast<const uint8_t *>(J.Qp) + (size_t) g * Q_BYTES, Q_BYTES, &sm.q_ready);
        }
        if (lane < GT) {
            const SideSrc ksrc = make_src(kv, 0, g, ws), vsrc = make_src(kv, 1, g, ws);
            unsigned rseq = lane; // this lane's tile in the sequence of all tiles of all side-groups
            unsigned issued = 0xffffffu; // the lane's last three copies as bytes (slot << 1 | phase parity), 0xff: none
            for (int nk = 0, nv = 0; nv < G && !sm.wc.dead;) {
                const bool isK = nk < G && nk < nv + NSB;
                Task k;
                if (isK) { // a group's K comes first: its task is computed here, once, and left for the other roles (the waits on
                           // the copies' barriers order their reads after this write)
                    k = get_task(kk + nk * tstep);
                    if (lane == 0) sm.tasks[nk % NTASK] = k;
                } else {
                    k = sm.tasks[nv % NTASK];
                }
                __syncwarp(0xfu);
                const SideSrc & S = isK ? ksrc : vsrc;
                const int rs = rseq % NRAW;
                const unsigned round = rseq / NRAW;
                if (round > 0) tc_wait(&sm.raw_empty[rs], (round - 1) & 1, &sm.wc, a.status);
                if (sm.wc.dead) break; // (nothing is fetched into a slot that may still be read, no barrier is over-subscribed)
                if (lane < k.nt) {
                    issue_tile(S, k.pos0 + lane * ATP, k.c1, sm.raw[rs], &sm.raw_full[rs]);
                    issued = (issued << 8) | ((unsigned) rs << 1) | (round & 1u);
                } else {
                    mbar_arrive(&sm.raw_full[rs]);
                }
                rseq += GT;
                if (isK) nk++;
                else nv++;
            }
            // a CTA whose waits gave up reaches this point with copies possibly in flight: they must land before the CTA's shared
            // memory is released (bounded; in a normal run every copy was waited for by its consumer long ago)
            if (sm.wc.dead && lane == 0) // (the query block too)
                for (unsigned it = 0; it < (1u << 14) && !mbar_try_wait_hint(&sm.q_ready, 0u, 1000u); it++) {}
            if (sm.wc.dead)
                for (int j = 0; j < 3; j++) {
                    const unsigned e = (issued >> (8 * j)) & 0xffu;
                    if (e == 0xffu) continue;
                    for (unsigned it = 0; it < (1u << 14) && !mbar_try_wait_hint(&sm.raw_full[e >> 1], e & 1u, 1000u); it++) {}
                }
        }
    } else if (warp == W_ISSUE) {
        // ---- issuer: S(0) .. S(NSB - 1), then PV(i), S(i + NSB) ----
        if (lane == 0) {
            unsigned oseq = 0;
            tc_wait(&sm.q_ready, 0u, &sm.wc, a.status); // the queries are staged
            const unsigned q_lo = desc_lo(smem_u32(sm.q), AR / 8 * 128), p_lo0 = desc_lo(smem_u32(sm.p[0]), 128);
            const unsigned hi_k = desc_hi(128), hi_mn = desc_hi(2048); // K-major: 8-row groups 128 bytes apart; MN-major: 2048
            for (int nk = 0, nv = 0; nv < G && !sm.wc.dead;) {
                const bool isK = nk < G && nk < nv + NSB;
                if (isK) { // S^T(nk) = K Q^T
                    const int sb = nk % NSB;
                    if (nk >= NSB) tc_wait(&sm.s_empty[sb], ((nk / NSB) - 1) & 1, &sm.wc, a.status);
                    const unsigned dcol = tb + S_COL + S_STRIDE * sb;
#pragma unroll 1
                    for (int h = 0; h < 2; h++, oseq++) {
                        const int os = oseq % NOP;
                        tc_wait(&sm.op_full[os], (oseq / NOP) & 1, &sm.wc, a.status);
                        tc_fence_after();
                        const unsigned a_lo = desc_lo(smem_u32(sm.op[os]), 2048), b_lo = q_lo + ((8 * h) * (2 * AR / 8 * 128) >> 4);
#pragma unroll
                        for (int ks = 0; ks < 8; ks++)
                            umma(dcol, a_lo + (ks * 4096 >> 4), hi_k, b_lo + (ks * (2 * AR / 8 * 128) >> 4), hi_k, IDESC_K, (unsigned) (h | ks));
                        umma_commit(&sm.op_empty[os]);
                    }
                    umma_commit(&sm.s_full[sb]);
                    nk++;
                } else { // O^T += V^T P^T(nv), P as its high and low parts
#if MKKV_TC_PROF == 1
                    TC_STAMP(nv, 16);
#endif
                    tc_wait(&sm.p_full, nv & 1, &sm.wc, a.status);
#if MKKV_TC_PROF == 1
                    TC_STAMP(nv, 17);
#endif
#pragma unroll 1
                    for (int h = 0; h < 2; h++, oseq++) {
                        const int os = oseq % NOP;
                        tc_wait(&sm.op_full[os], (oseq / NOP) & 1, &sm.wc, a.status);
#if MKKV_TC_PROF == 1
                        if (h == 0) TC_STAMP(nv, 18);
#endif
                        tc_fence_after();
                        const unsigned a_lo = desc_lo(smem_u32(sm.op[os]), 128), dcol = tb + (h ? O_COL1 : O_COL0);
#pragma unroll
                        for (int ks = 0; ks < 8; ks++) // B: the 48 rows of P's high part, then the 48 of its low part (12 row groups)
                            umma(dcol, a_lo + (ks * 256 >> 4), hi_mn, p_lo0 + (ks * 256 >> 4), hi_mn, IDESC_MN, (unsigned) (nv | ks));
                        umma_commit(&sm.op_empty[os]);
                    }
                    umma_commit(&sm.p_empty);
#if MKKV_TC_PROF == 1
                    TC_STAMP(nv, 19);
#endif
                    nv++;
                }
            }
            // every instruction issued above is complete before the tensor memory is freed and the CTA's shared memory released
            // (bounded; in a normal run the softmax warps have already waited for the last one)
            umma_commit(&sm.fin);
            for (unsigned it = 0; it < (1u << 14) && !mbar_try_wait_hint(&sm.fin, 0u, 1000u); it++) {}
        }
    }
    } else if (warp >= NSOFT) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 " MKKV_TC_REGS_DQ ";");
        // ---- unpack warps: packed rows -> operand slots, both 128-dim halves of one side of a group at a time ----
        const int w = warp - NSOFT, q = w & 3, c = w >> 2, prow = ATP * q + lane;
        const unsigned pos_off = (prow >> 3) * 128 + (prow & 7) * 16; // the position's 16-byte unit inside a dim group
        const bool st = w == 0;
        int rs = q, rph = 0, os = 0, oph = 0; // raw slot / phase of this warp's tile, operand slot / phase
        bool owrap = false;
        for (int nk = 0, nv = 0; nv < G && !sm.wc.dead;) {
            const bool isK = nk < G && nk < nv + NSB;
            const int side = isK ? 0 : 1, grp = isK ? nk - NSB : nv;
            (void) grp; // (the stamps' group index)
            if (st) TC_STAMP(grp, side ? 8 : 11);
            tc_wait(&sm.raw_full[rs], rph, &sm.wc, a.status);
            if (st) TC_STAMP(grp, side ? 9 : 12);
            const AttnTask & kr = sm.tasks[(isK ? nk : nv) % NTASK];
            const int k_pos0 = kr.pos0;
            const int2 kt = *reinterpret_cast<const int2 *>(&kr.c1); // c1, nt
            const int tbq = k_pos0 + q * ATP;
            const bool valid = q < kt.y && lane < kt.x - tbq;
            const int bits = (kv.s[side].rval && tbq >= ws) ? 8 : kv.s[side].bits;
            // which 32-dim blocks of a half this lane unpacks: the warps of a tile cover the four blocks of every row, rotated with
            // the row so that the 16-byte loads of 8 consecutive lanes (rows 32 bits bytes apart) fall into 8 different bank groups
            const int jr = (c + (lane >> (bits == 6 ? 1 : (bits == 5 || bits == 7) ? 2 : 0))) & 3;
            // the packed bytes of both 128-dim halves are read first (they need no operand slot), then each half is written into its
            // slot as that slot frees up
            const unsigned rawa = smem_u32(sm.raw[rs]);
#define MKKV_SIDE(B)                                                                                                   \
    {                                                                                                                  \
        PackedBlock<B> b0[BPW], b1[BPW];                                                                               \
        _Pragma("unroll") for (int k = 0; k < BPW; k++) {                                                              \
            dq_load<B>(b0[k], rawa, lane, (jr + k * (NDQ / 4)) & 3, valid);                                            \
            dq_load<B>(b1[k], rawa, lane, 4 + ((jr + k * (NDQ / 4)) & 3), valid);                                      \
        }                                                                                                              \
        if (owrap) tc_wait(&sm.op_empty[os], oph ^ 1, &sm.wc, a.status);                                               \
        if (!(MKKV_ABL & 1))                                                                                           \
            _Pragma("unroll") for (int k = 0; k < BPW; k++)                                                            \
                dq_emit<B>(b0[k], smem_u32(sm.op[os]) + 4 * ((jr + k * (NDQ / 4)) & 3) * 2048 + pos_off);              \
        fence_async_smem();                                                                                            \
        __syncwarp();                                                                                                  \
        if (lane == 0) mbar_arrive(&sm.op_full[os]);                                                                   \
        if (++os == NOP) os = 0, oph ^= 1, owrap = true;                                                               \
        if (owrap) tc_wait(&sm.op_empty[os], oph ^ 1, &sm.wc, a.status);                                               \
        if (!(MKKV_ABL & 1))                                                                                           \
            _Pragma("unroll") for (int k = 0; k < BPW; k++)                                                            \
                dq_emit<B>(b1[k], smem_u32(sm.op[os]) + 4 * ((jr + k * (NDQ / 4)) & 3) * 2048 + pos_off);              \
        fence_async_smem();                                                                                            \
        __syncwarp();                                                                                                  \
        if (lane == 0) mbar_arrive(&sm.op_full[os]);                                                                   \
        if (++os == NOP) os = 0, oph ^= 1, owrap = true;                                                               \
    }
            const int fixed = side ? VB : KB; // the side's compiled-in main format, or 0: any
            if (bits == 8) MKKV_SIDE(8)
            else if (fixed == 4 || (!fixed && bits == 4)) MKKV_SIDE(4)
            else if (fixed == 5 || (!fixed && bits == 5)) MKKV_SIDE(5)
            else if (fixed == 6 || (!fixed && bits == 6)) MKKV_SIDE(6)
            else if (fixed == 7 || !fixed) MKKV_SIDE(7)
#undef MKKV_SIDE
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.raw_empty[rs]);
            if (st) TC_STAMP(grp, side ? 10 : 13);
            rs += GT;
            if (rs >= NRAW) rs -= NRAW, rph ^= 1;
            if (isK) nk++;
            else nv++;
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 " MKKV_TC_REGS_SOFT ";");
#if MKKV_TC_PROF
        const unsigned long long t_loop = globaltimer_ns();
#endif
        // ---- softmax warps: warp = 4 c2 + q: positions 32 q .. + 31 of a group (tensor-memory lanes 32 q ..), query rows
        // 24 c2 .. + 23. Lanes 0 .. 23 own one row each (its running / reference max; replicated over the four q) ----
        const int q = warp & 3, c2 = warp >> 2, prow = ATP * q + lane, row0 = RS * c2;
        const unsigned pos_off = (prow >> 3) * 128 + (prow & 7) * 16;
        const unsigned lane_addr = tb + ((unsigned) (ATP * q) << 16);
        const bool owner = lane < RS, st = warp == 0;
        const int r_own = row0 + (owner ? lane : 0);
        WarpScratch & W = sm.ws[warp];
        float l_acc[RS];
#pragma unroll
        for (int i = 0; i < RS; i++) l_acc[i] = 0.f;
        float m_acc = -CUDART_INF_F, carry = -CUDART_INF_F; // (carry: batch mode, the chunk's running max after the previous group)
        unsigned long long w0 = 0, w1 = 0, w2 = 0;
        auto xbase = [&](const Task & k) -> size_t { return (((size_t) g * ATT_NCH + k.c) * a.nbmax) * AR + r_own; };
        // the exchange arrays are only touched by a CTA that has not given up (after a give-up the task records of groups the
        // producer never reached are not valid) and only inside their bounds
        auto exch_ok = [&](const Task & k) -> bool { return !sm.wc.dead && (unsigned) k.c < (unsigned) ATT_NCH && (unsigned) k.b < (unsigned) a.nbmax; };
        // which of the warp's rows this thread's position must not see in group k: row token t sees positions <= n + t; positions
        // past the chunk end and padding rows see nothing (0 for almost every group: uniform test first)
        unsigned pad_mask = 0u; // the warp's rows beyond the job's 6 T (fewer than 8 tokens): never visible
#pragma unroll
        for (int i = 0; i < RS; i++)
            if (row0 + i >= R) pad_mask |= 1u << i;
        const int tok0 = row0 % T; // token of the warp's first row (row = (head % 6) T + t)
        auto row_mask = [&](const Task & k) -> unsigned {
            unsigned m = pad_mask;
            if (k.pos0 + GP - 1 > min(k.c1 - 1, n)) { // (the group reaches the chunk's end or the new tokens: the last groups only)
                const int p_abs = k.pos0 + prow;
                int t = tok0;
#pragma unroll 1
                for (int i = 0; i < RS; i++) {
                    if (p_abs > min(k.c1 - 1, n + t)) m |= 1u << i;
                    if (++t == T) t = 0;
                }
            }
            return m;
        };
        // rows row0 + 8 gq .. + 7 of S^T of group j: request, then (after the wait) as masked floats
        auto scores_request = [&](int j, int gq, unsigned (&r)[8]) { tmem_ld8_async(lane_addr + S_COL + S_STRIDE * (j % NSB) + row0 + 8 * gq, r); };
        auto scores_take = [&](unsigned (&r)[8], unsigned mask, int gq, float (&s)[8]) {
            tmem_wait8(r);
#pragma unroll
            for (int i = 0; i < 8; i++) s[i] = __uint_as_float(r[i]);
            if (__any_sync(FULL_MASK, mask != 0u)) {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    if ((mask >> (8 * gq + i)) & 1u) s[i] = -CUDART_INF_F;
            }
        };
        // tile maxima of group j, its own maxima published, the words its running max will need requested
        auto maxima = [&](int j) {
            if (st) TC_STAMP(j, 0);
            tc_wait(&sm.s_full[j % NSB], (j / NSB) & 1, &sm.wc, a.status);
            const Task k = sm.tasks[j % NTASK];
            if (st) TC_STAMP(j, 1);
            tc_fence_after();
#if !(MKKV_ABL & 4)
            unsigned rq[RS / 8][8];
#pragma unroll
            for (int gq = 0; gq < RS / 8; gq++) scores_request(j, gq, rq[gq]);
            const unsigned mask = row_mask(k);
#pragma unroll
            for (int gq = 0; gq < RS / 8; gq++) {
                float s[8];
                scores_take(rq[gq], mask, gq, s);
                float mx[8];
#pragma unroll
                for (int i = 0; i < 8; i++) mx[i] = warp_max(s[i]);
                if (lane == 0) {
                    float4 * d = reinterpret_cast<float4 *>(&sm.tmax[j & 3][q][row0 + 8 * gq]);
                    d[0] = make_float4(mx[0], mx[1], mx[2], mx[3]);
                    d[1] = make_float4(mx[4], mx[5], mx[6], mx[7]);
                }
            }
#endif
            named_bar(1 + c2, GT * 32);
            if (!batch && owner && q == 0 && k.nb > 1 && k.b + 1 < k.nb && exch_ok(k)) {
                const float(&tm)[GT][AR] = sm.tmax[j & 3];
                const float gk = fmaxf(fmaxf(tm[0][r_own], tm[1][r_own]), fmaxf(tm[2][r_own], tm[3][r_own]));
                __stcg(a.xa + xbase(k) + (size_t) k.b * AR, ((unsigned long long) (unsigned) a.epoch << 32) | __float_as_uint(gk));
            }
            if (st) TC_STAMP(j, 2);
        };
        // the words the running max of group k will need: requested one phase before they are used, when the CTAs that hold
        // the chunk's previous groups have most likely published them
        auto request_words = [&](const Task & k) {
            if (!batch && owner && k.nb > 1 && exch_ok(k)) {
                const size_t xb0 = xbase(k);
                if (k.b >= 1) w1 = __ldcv(a.xa + xb0 + (size_t) (k.b - 1) * AR);
                if (k.b >= 2) w2 = __ldcv(a.xa + xb0 + (size_t) (k.b - 2) * AR);
                if (k.b >= 3) w0 = __ldcv(a.xb + xb0 + (size_t) (k.b - 3) * AR);
            }
        };
        // P of group i
        auto softmax = [&](int i, const Task & k) {
            if (st) TC_STAMP(i, 3);
            float beta = 0.f, f = 1.f;
            if (owner && !(MKKV_ABL & 8)) {
                float m_in = batch && k.b > 0 ? carry : -CUDART_INF_F;
                const size_t xb0 = xbase(k);
                const bool alive = exch_ok(k);
                if (alive && !batch && k.nb > 1) {
                    if (k.b >= 1) m_in = poll_word(a.xa + xb0 + (size_t) (k.b - 1) * AR, w1, a.epoch, &sm.wc, a.status);
                    if (k.b >= 2) m_in = fmaxf(m_in, poll_word(a.xa + xb0 + (size_t) (k.b - 2) * AR, w2, a.epoch, &sm.wc, a.status));
                    if (k.b >= 3) m_in = fmaxf(m_in, poll_word(a.xb + xb0 + (size_t) (k.b - 3) * AR, w0, a.epoch, &sm.wc, a.status));
                }
                if (st) TC_STAMP(i, 7);
                const float(&tm)[GT][AR] = sm.tmax[i & 3];
                float mr = m_in; // running max after this warp's tile, M: after the whole group
#pragma unroll
                for (int t = 0; t < GT; t++)
                    if (t <= q) mr = fmaxf(mr, tm[t][r_own]);
                float M = mr;
#pragma unroll
                for (int t = 0; t < GT; t++)
                    if (t > q) M = fmaxf(M, tm[t][r_own]);
                if (alive && !batch && q == 0 && k.nb > 1 && k.b + 3 < k.nb) __stcg(a.xb + xb0 + (size_t) k.b * AR, ((unsigned long long) (unsigned) a.epoch << 32) | __float_as_uint(M));
                carry = M;
                if (M != -CUDART_INF_F) {
                    if (m_acc == -CUDART_INF_F) m_acc = M + REF_MARGIN;
                    else if (M > m_acc + REF_SLACK) {
                        f = exp_any(m_acc - (M + REF_MARGIN));
                        m_acc = M + REF_MARGIN;
                    }
                }
                beta = mr == -CUDART_INF_F ? 0.f : exp_any(mr - m_acc);
                W.m[lane] = mr == -CUDART_INF_F ? CUDART_INF_F : mr;
                W.beta[lane] = beta;
                W.f[lane] = f;
            }
            if (st) TC_STAMP(i, 14);
            const float bnext = __shfl_down_sync(FULL_MASK, beta, 1);
            if (owner && !(lane & 1)) {
                const __half2 bh = __floats2half2_rn(beta, bnext);
                const float2 bf = __half22float2(bh);
                const __half2 bl = __floats2half2_rn(beta - bf.x, bnext - bf.y);
                W.bh[lane >> 1] = *reinterpret_cast<const unsigned *>(&bh);
                W.bl[lane >> 1] = *reinterpret_cast<const unsigned *>(&bl);
            }
            const unsigned anyf = __ballot_sync(FULL_MASK, owner && f != 1.f);
            __syncwarp();
            if (st) TC_STAMP(i, 4);
            if (anyf) { // a reference max moved: the row sums follow at once, the accumulator when it is at rest (below)
#pragma unroll
                for (int j = 0; j < RS; j++) l_acc[j] *= W.f[j];
            }
            // P of the group into registers: the exponentials do not wait for the P buffer
            const unsigned mask = row_mask(k);
            unsigned ra[8], rb[8], hi[RS / 8][4], lo[RS / 8][4];
            scores_request(i, 0, ra);
#pragma unroll
            for (int gq = 0; gq < RS / 8; gq++) { // row groups of 8: one 16-byte unit of each P part; the next group's scores are in
                                                  // flight while this one's P is computed
                float s[8];
                if (gq + 1 < RS / 8) {
                    if (gq & 1) {
                        scores_take(rb, mask, gq, s);
                        scores_request(i, gq + 1, ra);
                    } else {
                        scores_take(ra, mask, gq, s);
                        scores_request(i, gq + 1, rb);
                    }
                } else {
                    scores_take((gq & 1) ? rb : ra, mask, gq, s);
                }
                if (gq == RS / 8 - 1) { // the last read of this S^T buffer
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm.s_empty[i % NSB]);
                }
#if MKKV_ABL & 2
                for (int j = 0; j < 4; j++) hi[gq][j] = lo[gq][j] = __float_as_uint(s[j]);
                continue;
#endif
                const float4 ma = *reinterpret_cast<const float4 *>(&W.m[8 * gq]), mb = *reinterpret_cast<const float4 *>(&W.m[8 * gq + 4]);
                const float4 ba = *reinterpret_cast<const float4 *>(&W.beta[8 * gq]), bb = *reinterpret_cast<const float4 *>(&W.beta[8 * gq + 4]);
                const uint4 bhv = *reinterpret_cast<const uint4 *>(&W.bh[4 * gq]), blv = *reinterpret_cast<const uint4 *>(&W.bl[4 * gq]);
                const float mm[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w}, be[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
                const unsigned bhw[4] = {bhv.x, bhv.y, bhv.z, bhv.w}, blw[4] = {blv.x, blv.y, blv.z, blv.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int r = 8 * gq + 2 * j;
                    const float p0 = exp_neg(s[2 * j] - mm[2 * j]), p1 = exp_neg(s[2 * j + 1] - mm[2 * j + 1]);
                    l_acc[r] = __fmaf_rn(be[2 * j], p0, l_acc[r]);
                    l_acc[r + 1] = __fmaf_rn(be[2 * j + 1], p1, l_acc[r + 1]);
                    const __half2 ph = __floats2half2_rn(p0, p1); // the reference's fp16 P
                    const __half2 bh = *reinterpret_cast<const __half2 *>(&bhw[j]), bl = *reinterpret_cast<const __half2 *>(&blw[j]);
                    const __half2 hh = __hmul2(ph, bh);                 // P beta = hh + ll up to 2^-22: the product's exact residual
                    const __half2 ll = __hfma2(ph, bl, __hfma2(ph, bh, __hneg2(hh))); // plus the low part of beta
                    hi[gq][j] = *reinterpret_cast<const unsigned *>(&hh);
                    lo[gq][j] = *reinterpret_cast<const unsigned *>(&ll);
                }
            }
            if (st && i < 15) TC_STAMP(i, 15);
            if (i > 0) tc_wait(&sm.p_empty, (i - 1) & 1, &sm.wc, a.status); // P V of the previous group is complete: P is free, O^T at rest
            if (st) TC_STAMP(i, 5);
            tc_fence_after();
#if MKKV_TC_PROF
            if (anyf && a.prof && st && lane == 0) a.prof[((size_t) blockIdx.x * 16 + 15) * 20 + 15] += 1ull | ((unsigned long long) __popc(anyf) << 32);
#endif
            if (anyf) { // bring the accumulator columns of the rows whose reference max moved (one, as a rule) to the new reference:
                        // a row is one column in each of the four blocks (two halves x high / low part); the four loads of a row
                        // are in flight together
                unsigned left = anyf;
#pragma unroll 1
                while (left) {
                    const int r = __ffs(left) - 1;
                    left &= left - 1;
                    const float fr = W.f[r];
                    const unsigned ad = lane_addr + row0 + r;
                    unsigned v0, v1, v2, v3;
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v0) : "r"(ad + O_COL0));
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v1) : "r"(ad + O_COL0 + AR));
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v2) : "r"(ad + O_COL1));
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v3) : "r"(ad + O_COL1 + AR));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v0), "+r"(v1), "+r"(v2), "+r"(v3)::"memory");
                    v0 = __float_as_uint(__uint_as_float(v0) * fr), v1 = __float_as_uint(__uint_as_float(v1) * fr);
                    v2 = __float_as_uint(__uint_as_float(v2) * fr), v3 = __float_as_uint(__uint_as_float(v3) * fr);
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(ad + O_COL0), "r"(v0) : "memory");
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(ad + O_COL0 + AR), "r"(v1) : "memory");
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(ad + O_COL1), "r"(v2) : "memory");
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(ad + O_COL1 + AR), "r"(v3) : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
#pragma unroll
            for (int gq = 0; gq < RS / 8; gq++) {
                const unsigned off = (unsigned) ((RS / 8) * c2 + gq) * 2048 + pos_off;
                *reinterpret_cast<uint4 *>(sm.p[0] + off) = make_uint4(hi[gq][0], hi[gq][1], hi[gq][2], hi[gq][3]);
                *reinterpret_cast<uint4 *>(sm.p[1] + off) = make_uint4(lo[gq][0], lo[gq][1], lo[gq][2], lo[gq][3]);
            }
            fence_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_full);
            if (st) TC_STAMP(i, 6);
        };

        if (G > 0) {
            // Tile maxima run ahead of P (tasks: left by the producer, see there), so that a group's own maxima are published well
            // before the CTAs that hold the chunk's next groups need them: the CTAs of a kv head may drift apart by a group
            // without a poll having to wait. The lead grows from none (the first P needs only its own group's scores) to two groups.
            constexpr int MAX_AHEAD = 2;
            int maxima_done = 0;
            for (int i = 0; i < G; i++) {
                const int want = min(G, i + 1 + min(i, MAX_AHEAD));
                while (maxima_done < want) maxima(maxima_done++);
                const Task kc = sm.tasks[i % NTASK];
                softmax(i, kc);
                if (i + 1 < maxima_done) { // (the next group's task record is known to be written: its scores have been waited for)
                    const Task kn = sm.tasks[(i + 1) % NTASK];
                    request_words(kn);
                } else {
                    w0 = w1 = w2 = 0ull; // (no early request: the polls fetch the words themselves)
                }
            }
            tc_wait(&sm.p_empty, (G - 1) & 1, &sm.wc, a.status);
            tc_fence_after();
        }
#if MKKV_TC_PROF
        if (warp == 0) { // the tail's stamps go to group slot 15 (stamps 8 .. 13, after the main loop's own use of them)
            if (a.prof && lane == 0) {
                a.prof[((size_t) blockIdx.x * 16 + 15) * 20 + 8] = t_entry;
                a.prof[((size_t) blockIdx.x * 16 + 15) * 20 + 9] = t_loop;
                unsigned smid;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                a.prof[((size_t) blockIdx.x * 16 + 15) * 20 + 14] = smid; // (which SM ran this CTA)
            }
            TC_STAMP(15, 10);
        }
#endif
        // ---- the CTA's partial: O^T lanes are dims (in the unpacked units' order: mapped back here), columns are query rows ----
        const int pdim = (prow & ~7) | unit_perm(prow & 7);
#pragma unroll
#pragma unroll 1
        for (int hg = 0; hg < 2 * (RS / 8); hg++) {
            const int h = hg / (RS / 8), gq = hg % (RS / 8);
            float v[8], w[8];
            if (G > 0) {
                tmem_ld8(lane_addr + (h ? O_COL1 : O_COL0) + row0 + 8 * gq, v);
                tmem_ld8(lane_addr + (h ? O_COL1 : O_COL0) + AR + row0 + 8 * gq, w);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int r = row0 + 8 * gq + j;
                if (r < R) a.part[((size_t) slot * AR + r) * HD + 128 * h + pdim] = G > 0 ? v[j] + w[j] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < RS; j++) {
            float x = l_acc[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(FULL_MASK, x, o);
            l_acc[j] = x;
        }
        named_bar(5, NSOFT * 32); // every softmax warp is past its last read of the tile maxima
        float(&lsum)[GT][AR] = *reinterpret_cast<float(*)[GT][AR]>(&sm.tmax[0][0][0]);
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < RS; j++) lsum[q][row0 + j] = l_acc[j];
        }
        named_bar(5, NSOFT * 32);
        if (owner && q == 0 && r_own < R)
            a.ml[(size_t) slot * AR + r_own] = make_float2(m_acc, lsum[0][r_own] + lsum[1][r_own] + lsum[2][r_own] + lsum[3][r_own]);
#if MKKV_TC_PROF
        if (warp == 0) TC_STAMP(15, 11);
#endif
        if (a.done) {
            // ---- the merge, in the kernel's tail: when every CTA of the kv head has written its partial, this CTA merges rows
            // kk and kk + cph of the head's 6 T. Four warps share a row (warp j of the team: partials j, j + 4, ..: all their loads
            // are in flight at once), the team's sums meet in shared memory (an operand slot: every MMA of the CTA is complete) ----
            __threadfence();
            named_bar(5, NSOFT * 32);
            if (warp == 0) {
                bool ok = true;
                if (lane == 0) {
                    atomicAdd(a.done + g, 1u);
                    unsigned it = 0;
                    while ((int) (ld_acquire_u32(a.done + g) - a.done_target) < 0) {
                        __nanosleep(100);
                        if (++it >= (sm.wc.poll << 2) || sm.wc.dead) { // (about a second)
                            atomicExch(a.status, (int) KS_WAIT_TIMEOUT);
                            ok = false;
                            break;
                        }
                    }
                    sm.merge_ok = ok;
                }
            }
            named_bar(5, NSOFT * 32);
#if MKKV_TC_PROF
            if (warp == 0) TC_STAMP(15, 12);
#endif
            const int team = warp >> 2, tj = warp & 3, rr = kk + team * a.cph;
            const bool has = sm.merge_ok && rr < GQ * T;
            float * const scratch = reinterpret_cast<float *>(sm.op[0]); // [warp][lane][8 sums], then [warp] weights' sums
            float num[8], den = 0.f, M = -CUDART_INF_F;
            if (has) {
                merge_accumulate(a.part, a.ml, (size_t) g * a.cph, (size_t) AR * HD, (size_t) AR, a.cph, tj, 4, rr, lane, num, den, M);
                float4 * d = reinterpret_cast<float4 *>(scratch + ((size_t) warp * 32 + lane) * 8);
                d[0] = make_float4(num[0], num[1], num[2], num[3]);
                d[1] = make_float4(num[4], num[5], num[6], num[7]);
                if (lane == 0) scratch[NSOFT * 32 * 8 + warp] = den;
            }
            named_bar(5, NSOFT * 32);
            if (has && tj == 0) {
#pragma unroll
                for (int w2 = 1; w2 < 4; w2++) {
                    const float4 * o = reinterpret_cast<const float4 *>(scratch + ((size_t) (warp + w2) * 32 + lane) * 8);
                    const float4 o0 = o[0], o1 = o[1];
                    num[0] += o0.x, num[1] += o0.y, num[2] += o0.z, num[3] += o0.w;
                    num[4] += o1.x, num[5] += o1.y, num[6] += o1.z, num[7] += o1.w;
                    den += scratch[NSOFT * 32 * 8 + warp + w2];
                }
                merge_finish(J, g * GQ + rr / T, rr % T, lane, a.raw_part != nullptr, a.raw_part, a.raw_ml, num, den, M);
            }
#if MKKV_TC_PROF
            if (warp == 0) TC_STAMP(15, 13);
#endif
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_ISSUE) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(TMEM_COLS) : "memory");
}

// ---- test probe of the unpack step ----
// nrows packed rows of BITS bits (values [nrows][32 BITS] bytes, scales [nrows][8] fp16) through the very code the unpack warps run
// (dq_load / dq_emit on a staged tile), back in natural dim order: out [nrows][256] fp16 bit patterns. One warp per 32-row tile.
template <int BITS> __global__ void __launch_bounds__(32) unpack_probe_kernel(const uint8_t * rows, const uint16_t * sc, int nrows, uint16_t * out) {
    __shared__ __align__(128) uint8_t raw[RAW_SLOT];
    __shared__ __align__(128) uint8_t op[4 * 2048]; // one 32-dim block: four dim groups of 128 positions x 16 bytes
    const int lane = threadIdx.x, row = blockIdx.x * ATP + lane;
    const bool valid = row < nrows;
    constexpr int RB = 32 * BITS;
    for (int i = lane; i < ATP * RB / 4; i += 32) { // the tile as the bulk copies leave it: rows, then the scale rows
        const int r = blockIdx.x * ATP + i / (RB / 4);
        reinterpret_cast<unsigned *>(raw)[i] = r < nrows ? reinterpret_cast<const unsigned *>(rows)[(size_t) blockIdx.x * ATP * RB / 4 + i] : 0u;
    }
    for (int i = lane; i < ATP * 8; i += 32) {
        const int r = blockIdx.x * ATP + i / 8;
        reinterpret_cast<uint16_t *>(raw + TILE_SC_OFF)[i] = r < nrows ? sc[(size_t) blockIdx.x * ATP * 8 + i] : (uint16_t) 0;
    }
    __syncwarp();
    for (int jb = 0; jb < 8; jb++) {
        dq_item<BITS>(smem_u32(raw), lane, jb, valid, smem_u32(op) + lane * 16);
        __syncwarp();
        if (valid)
            for (int u = 0; u < 4; u++) {
                const uint16_t * unit = reinterpret_cast<const uint16_t *>(op + u * 2048 + lane * 16);
                for (int j = 0; j < 8; j++) out[(size_t) row * HD + 32 * jb + 8 * u + unit_perm(j)] = unit[j];
            }
        __syncwarp();
    }
}

} // namespace tc

cudaError_t launch_unpack_probe(int bits, const uint8_t * rows, const uint16_t * sc, int nrows, uint16_t * out, cudaStream_t stream) {
    if (nrows < 1) return cudaSuccess;
    const int grid = (nrows + ATP - 1) / ATP;
    switch (bits) {
    case 4: tc::unpack_probe_kernel<4><<<grid, 32, 0, stream>>>(rows, sc, nrows, out); break;
    case 5: tc::unpack_probe_kernel<5><<<grid, 32, 0, stream>>>(rows, sc, nrows, out); break;
    case 6: tc::unpack_probe_kernel<6><<<grid, 32, 0, stream>>>(rows, sc, nrows, out); break;
    case 7: tc::unpack_probe_kernel<7><<<grid, 32, 0, stream>>>(rows, sc, nrows, out); break;
    case 8: tc::unpack_probe_kernel<8><<<grid, 32, 0, stream>>>(rows, sc, nrows, out); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

static_assert(sizeof(tc::Smem) + 128 <= 232448, "shared memory of one CTA");
size_t attend_tc_smem_bytes() { return sizeof(tc::Smem) + 128; }
// the kernel instance for a job's main formats: the served presets are compiled in, anything else runs the any-format instance
typedef void (*TcKernel)(const tc::Args);
static TcKernel tc_kernel_for(int kb, int vb, bool batch) {
    if (batch) {
        if (kb == 5 && vb == 6) return tc::attn_tc_kernel<5, 6, true>;
        if (kb == 5 && vb == 5) return tc::attn_tc_kernel<5, 5, true>;
        if (kb == 6 && vb == 5) return tc::attn_tc_kernel<6, 5, true>;
        if (kb == 8 && vb == 8) return tc::attn_tc_kernel<8, 8, true>;
        return tc::attn_tc_kernel<0, 0, true>;
    }
    if (kb == 5 && vb == 6) return tc::attn_tc_kernel<5, 6, false>;
    if (kb == 5 && vb == 5) return tc::attn_tc_kernel<5, 5, false>;
    if (kb == 6 && vb == 5) return tc::attn_tc_kernel<6, 5, false>;
    if (kb == 8 && vb == 8) return tc::attn_tc_kernel<8, 8, false>;
    return tc::attn_tc_kernel<0, 0, false>;
}
static const TcKernel tc_kernels[] = {tc::attn_tc_kernel<5, 6, false>, tc::attn_tc_kernel<5, 5, false>, tc::attn_tc_kernel<6, 5, false>,
                                      tc::attn_tc_kernel<8, 8, false>, tc::attn_tc_kernel<0, 0, false>,
                                      tc::attn_tc_kernel<5, 6, true>,  tc::attn_tc_kernel<5, 5, true>,  tc::attn_tc_kernel<6, 5, true>,
                                      tc::attn_tc_kernel<8, 8, true>,  tc::attn_tc_kernel<0, 0, true>};
// every instance may use the CTA's full shared memory (set once per device)
static cudaError_t tc_prepare() {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        for (TcKernel k : tc_kernels) {
            e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) attend_tc_smem_bytes());
            if (e != cudaSuccess) return e;
        }
        attr_set[dev] = true;
    }
    return cudaSuccess;
}
// the wait limits of the launches that follow (process-wide; diagnostics and the failure-path test)
static unsigned g_wait_hint_ns = tc::WAIT_HINT_NS, g_wait_rounds = tc::WAIT_ROUNDS, g_poll_rounds = tc::POLL_ROUNDS;
void attend_tc_set_wait_limits(unsigned hint_ns, unsigned rounds, unsigned polls) {
    g_wait_hint_ns = hint_ns;
    g_wait_rounds = rounds;
    g_poll_rounds = polls;
}
void attend_tc_default_wait_limits() { attend_tc_set_wait_limits(tc::WAIT_HINT_NS, tc::WAIT_ROUNDS, tc::POLL_ROUNDS); }
cudaError_t preload_attend_tc() {
    cudaFuncAttributes fa;
    for (TcKernel k : tc_kernels) {
        const cudaError_t e = cudaFuncGetAttributes(&fa, (const void *) k);
        if (e != cudaSuccess) return e;
    }
    return tc_prepare();
}

cudaError_t launch_attend_tc(const AttnJob & job, int num_sms, float * part, float2 * ml, int part_slots, unsigned long long * xa,
                             unsigned long long * xb, int nbmax, int epoch, int * status, cudaStream_t stream, const AttnTask * tasks_dev,
                             int ntasks, int tasks_B, float * raw_part, float2 * raw_ml, unsigned long long * prof, unsigned * done,
                             unsigned * done_seq) {
    if (!job.Qp) return cudaErrorNotSupported; // (the queries were not staged: the caller takes its other kernel)
    tc::Args a;
    a.prof = prof;
    a.one = job;
    a.jobs = nullptr;
    a.njobs = 1;
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
    a.wait_hint_ns = g_wait_hint_ns;
    a.wait_rounds = g_wait_rounds;
    a.poll_rounds = g_poll_rounds;
    cudaError_t e = tc_prepare();
    if (e != cudaSuccess) return e;
    // the merge runs in the kernel's tail (normalised into O, or un-normalised per kv head for a later merge across GPUs)
    const bool fused = done && done_seq && (raw_part ? raw_ml != nullptr : job.O != nullptr);
    a.raw_part = fused ? raw_part : nullptr;
    a.raw_ml = fused ? raw_ml : nullptr;
    a.done = fused ? done : nullptr;
    a.done_target = fused ? (*done_seq + 1u) * (unsigned) a.cph : 0u;
    void * args[] = {&a};
    e = cudaLaunchCooperativeKernel((const void *) tc_kernel_for(job.kv.s[0].bits, job.kv.s[1].bits, false), dim3(NKV * a.cph), dim3(tc::NTHREADS), args, attend_tc_smem_bytes(), stream);
    if (e != cudaSuccess) return e;
    if (fused) {
        *done_seq += 1u;
        return cudaSuccess;
    }
    AttnJob merge_job = job;
    merge_job.nch = a.cph; // the merge reads cph partials per kv head, slots g cph ..
    merge_job.item0 = 0;
    return launch_merge(nullptr, &merge_job, 1, job.T, part, ml, stream, raw_part, raw_ml);
}

// Batch mode: njobs jobs, one CTA per (job, kv head, run of the job's cpi chunks) in a plain launch (no CTA waits for another: the
// groups of a chunk run in order on one CTA), then the merge kernel over the jobs' partials (a head's partials: its first slots).
cudaError_t launch_attend_tc_batch(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int total_items, int max_T, float * part,
                                   float2 * ml, int part_slots, int * status, cudaStream_t stream) {
    if (njobs < 1 || total_items < 1 || total_items > part_slots || !jobs_dev) return cudaErrorNotSupported;
    for (int j = 0; j < njobs; j++)
        if (!jobs_host[j].Qp) return cudaErrorNotSupported; // (queries not staged)
    tc::Args a;
    a.one = jobs_host[0];
    a.jobs = jobs_dev;
    a.njobs = njobs;
    a.cph = 1;
    a.ntasks = 0;
    a.tasks = nullptr;
    a.part = part;
    a.ml = ml;
    a.xa = a.xb = nullptr;
    a.nbmax = 0;
    a.epoch = 0;
    a.status = status;
    a.done = nullptr;
    a.done_target = 0;
    a.raw_part = nullptr;
    a.raw_ml = nullptr;
    a.prof = nullptr;
    a.wait_hint_ns = g_wait_hint_ns;
    a.wait_rounds = g_wait_rounds;
    a.poll_rounds = g_poll_rounds;
    cudaError_t e = tc_prepare();
    if (e != cudaSuccess) return e;
    // (the jobs of one batch may differ in format: the any-format instance unless they all share a compiled-in pair)
    TcKernel kern = tc_kernel_for(jobs_host[0].kv.s[0].bits, jobs_host[0].kv.s[1].bits, true);
    for (int j = 1; j < njobs; j++)
        if (jobs_host[j].kv.s[0].bits != jobs_host[0].kv.s[0].bits || jobs_host[j].kv.s[1].bits != jobs_host[0].kv.s[1].bits) kern = tc::attn_tc_kernel<0, 0, true>;
    int grid = 0; // (the jobs' CTAs as step_batch planned them: titem0, cpi)
    for (int j = 0; j < njobs; j++) {
        const int cpi = std::max(jobs_host[j].cpi, 1);
        if (jobs_host[j].titem0 != grid) return cudaErrorInvalidValue;
        grid += NKV * ((jobs_host[j].nch + cpi - 1) / cpi);
    }
    if (grid > total_items) return cudaErrorInvalidValue;
    kern<<<grid, tc::NTHREADS, attend_tc_smem_bytes(), stream>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return launch_merge(jobs_dev, jobs_host, njobs, max_T, part, ml, stream, nullptr, nullptr, true);
}

} // namespace mkkv
