// Device helpers shared by the decode-attention kernels: PTX wrappers (mbarrier, bulk copies, named barriers), the exact
// packed-byte -> fp16(d * q) conversion, the task arithmetic of a job spread over the grid, and the tile fetch.
#pragma once
#include <cuda_fp16.h>

#include "kv_kernels.h"

namespace mkkv {
namespace attn_common {

constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr int TILE_SC_OFF = ATP * HD; // scales of a staged tile: after 32 rows of the widest format

// ---- PTX helpers ----
__device__ __forceinline__ unsigned smem_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t * bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait. A failed try_wait suspends the thread for a hardware-chosen time before it reports failure, so `rounds` failed
// tries (default 2^23) are seconds. On expiry the status word and the CTA's give-up flag are set and the caller goes on; from
// then on no wait of the CTA blocks, so the kernel always ends promptly (with a result the host rejects).
struct WaitLimit {
    int dead;        // a wait of this CTA gave up
    unsigned rounds; // failed tries of an mbarrier wait / failed polls of a global word before giving up
};
constexpr unsigned WAIT_ROUNDS_DEFAULT = 1u << 23;
__device__ __forceinline__ void mbar_wait(uint64_t * bar, unsigned parity, int * status, volatile WaitLimit * wl) {
    for (unsigned it = 0; !mbar_try_wait(bar, parity); it++) {
        if (wl->dead) return;
        if (it >= wl->rounds) {
            wl->dead = 1;
            if (status) atomicExch(status, (int) KS_WAIT_TIMEOUT);
            return;
        }
    }
}
__device__ __forceinline__ void bulk_g2s(void * dst, const void * src, unsigned bytes, uint64_t * bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void named_bar(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }
__device__ __forceinline__ int ld_acquire(const int * p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int * p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// biased bytes b0, b1 (SEL = 0) or b2, b3 (SEL = 1) of x -> half2 (1024 + b), minus (1024 + bias), times the scale pair:
// fp16(d * q) exactly, one rounding (the products 1024 + b and the difference are exact in fp16)
template <int SEL> __device__ __forceinline__ unsigned cvt_pair(unsigned x, __half2 sub, __half2 d) {
    const unsigned m = __byte_perm(x, 0x64646464u, SEL ? 0x4342 : 0x4140);
    const __half2 h = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&m), sub), d);
    return *reinterpret_cast<const unsigned *>(&h);
}

// ---- tasks ----
struct Geo { // the partition of one job
    int L, nch, cs, nt_full, nt_last, nb_full, nb_last, ntasks_head;
};
__device__ __forceinline__ Geo make_geo(const AttnJob & J, int B) {
    Geo g;
    g.L = J.n + J.T;
    g.nch = J.nch;
    g.cs = J.cs;
    g.nt_full = J.cs / ATP;
    g.nt_last = (g.L - (J.nch - 1) * J.cs + ATP - 1) / ATP;
    g.nb_full = (g.nt_full + B - 1) / B;
    g.nb_last = (g.nt_last + B - 1) / B;
    g.ntasks_head = g.nb_last * g.nch + (g.nb_full - g.nb_last) * (g.nch - 1);
    return g;
}
typedef AttnTask Task;
// mode 0: task t (batch-major over the chunks of one kv head); mode 1: batch t of chunk c_fixed
__device__ __forceinline__ Task make_task(const Geo & g, int B, int mode, int t, int c_fixed) {
    Task k;
    if (mode == 0) {
        const int first = g.nb_last * g.nch;
        if (t < first) {
            k.b = t / g.nch;
            k.c = t % g.nch;
        } else {
            const int u = t - first;
            k.b = g.nb_last + u / (g.nch - 1);
            k.c = u % (g.nch - 1);
        }
    } else {
        k.c = c_fixed;
        k.b = t;
    }
    const int ntc = k.c == g.nch - 1 ? g.nt_last : g.nt_full;
    k.nb = (ntc + B - 1) / B;
    k.c1 = min(g.L, (k.c + 1) * g.cs);
    k.pos0 = k.c * g.cs + k.b * B * ATP;
    k.nt = min(B, ntc - k.b * B);
    return k;
}

// where the tiles of one side of one kv head live: bases with the kv head's offset folded in (computed once per issuing thread)
struct SideSrc {
    const uint8_t * mval;  // main values, row 0 of the kv head
    const uint16_t * msc;  // main scales
    const uint8_t * rval;  // ring values (null: no ring)
    const uint16_t * rsc;
    int rb, bits, ring0, rc; // main row bytes / bits; first position served by the ring; ring rows
};
__device__ __forceinline__ SideSrc make_src(const KvView & kv, int w, int g, int ws) {
    const KvSide & s = kv.s[w];
    SideSrc r;
    r.bits = s.bits;
    r.rb = row_bytes(s.bits);
    // (row 0 of the buffer is position kv.base: fold it in; only positions >= base are ever fetched)
    r.mval = s.val + ((ptrdiff_t) g * kv.ctxp - kv.base) * r.rb;
    r.msc = s.sc + ((ptrdiff_t) g * kv.ctxp - kv.base) * 8;
    r.rval = s.rval ? s.rval + (size_t) g * kv.rc * HD : nullptr;
    r.rsc = s.rval ? s.rsc + (size_t) g * kv.rc * 8 : nullptr;
    r.ring0 = s.rval ? ws : 0x7fffffff;
    r.rc = kv.rc;
    return r;
}
// one side of one tile into a stage: rows then scales, completing on bar (one thread)
__device__ __forceinline__ void issue_tile(const SideSrc & S, int tb, int c1, uint8_t * stage, uint64_t * bar) {
    const int np = min(ATP, c1 - tb);
    const uint8_t * val;
    const uint16_t * sc;
    int rb;
    if (tb >= S.ring0) { // rc is a multiple of 32: a tile never wraps
        const int r = tb % S.rc;
        val = S.rval + (size_t) r * HD;
        sc = S.rsc + (size_t) r * 8;
        rb = HD;
    } else {
        val = S.mval + (size_t) tb * S.rb;
        sc = S.msc + (size_t) tb * 8;
        rb = S.rb;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the stage was read with ordinary loads before
    mbar_expect_tx(bar, np * rb + np * SCALE_ROW);
    bulk_g2s(stage, val, np * rb, bar);
    bulk_g2s(stage + TILE_SC_OFF, sc, np * SCALE_ROW, bar);
}

} // namespace attn_common
} // namespace mkkv
