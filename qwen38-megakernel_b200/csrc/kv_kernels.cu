// KV hot-path kernels for sm_100a: append + quantize, spill, ring refill, snapshot gather / scatter, and the baseline
// decode-attention kernel (TMA bulk staging + mbarrier pipeline, register dequant, fp16 tensor-core tiles) with its merge.
//
// Arithmetic contract (what the parity tests pin): stored bytes follow qwen38_mk.cu:2003-2116 bit for bit; attention
// follows attn_core_t (qwen38_mk.cu:2756-3067): operands fp16(d * q) and fp16(q / 16), fp32 scores, online softmax per
// 32-position tile with expf, P rounded to fp16, fp32 accumulation, the reference's chunk partition (attn_dims), and the
// merge of qwen38_mk.cu:4658-4685.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "kv_kernels.h"
#include "kv_quant.cuh"
#include "kv_merge.cuh"

namespace mkkv {

// --------------------------------------------------------------------------------------------------------------------
// small PTX helpers: mbarrier + bulk async copy (TMA), never multicast
// --------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t * bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
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
// Bounded wait: gives up after about two seconds, records KS_WAIT_TIMEOUT in *status and returns, so control flow stays
// uniform and the kernel ends (with a wrong result the host rejects) instead of hanging the GPU.
__device__ __forceinline__ void mbar_wait(uint64_t * bar, unsigned parity, int * status) {
    if (mbar_try_wait(bar, parity)) return;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned it = 0;; it++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 1023u) == 1023u && globaltimer_ns() - t0 > 2000000000ull) {
            if (status) atomicExch(status, (int) KS_WAIT_TIMEOUT);
            return;
        }
    }
}
// global -> shared bulk copy; dst, src 16-byte aligned, bytes a multiple of 16; completes on bar
__device__ __forceinline__ void bulk_g2s(void * dst, const void * src, unsigned bytes, uint64_t * bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// --------------------------------------------------------------------------------------------------------------------
// append / spill / refill: one warp per row
// --------------------------------------------------------------------------------------------------------------------
struct AppendArgs {
    KvView kv;
    const uint16_t * K;
    const uint16_t * V;
    int pos0, n;
};

__device__ __forceinline__ void load_row_f16(const uint16_t * src, int lane, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(src + lane * 8);
    const __half2 * h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 f = __half22float2(h[k]);
        v[2 * k] = f.x;
        v[2 * k + 1] = f.y;
    }
}

// one row: source fp16 row -> (shadow) -> rotation -> main-format row (eager, or no ring) and the ring's q8_0 row
__device__ __forceinline__ void append_row(const KvView & kv, int w, int g, int pos, const uint16_t * src, int lane) {
    const KvSide & s = kv.s[w];
    float v[8];
    load_row_f16(src, lane, v);
    if (s.shadow) { // spill mode: keep the source row so the main-format row can be made from the same values later
        const size_t rr = (size_t) g * kv.rc + pos % kv.rc;
        *reinterpret_cast<uint4 *>(s.shadow + rr * HD + lane * 8) = *reinterpret_cast<const uint4 *>(src + lane * 8);
    }
    if (s.rot) fwht256(v, lane);
    if (kv.eager || !s.rval) {
        const size_t row = (size_t) g * kv.ctxp + (pos - kv.base);
        store_row(s.val + row * row_bytes(s.bits), s.sc + row * 8, v, s.bits, lane);
    }
    if (s.rval) { // the ring keeps the same (rotated) values as q8_0: every tile of a side shares one basis
        const size_t rr = (size_t) g * kv.rc + pos % kv.rc;
        store_q8(s.rval + rr * HD, s.rsc + rr * 8, v, lane);
    }
}

__global__ void __launch_bounds__(256) append_kernel(const __grid_constant__ AppendArgs a) {
    const int lane = threadIdx.x & 31, idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (idx >= a.n * 2 * NKV) return;
    const int t = idx / (2 * NKV), w = (idx / NKV) & 1, g = idx % NKV, pos = a.pos0 + t;
    append_row(a.kv, w, g, pos, (w ? a.V : a.K) + ((size_t) t * NKV + g) * HD, lane);
}

// rows [p0, p1) x layers x ring sides x kv heads, one warp per row: fp16 shadow row -> main-format row
__global__ void __launch_bounds__(256) spill_kernel(const KvView * views, int layers, int p0, int p1) {
    const int lane = threadIdx.x & 31;
    const long long total = (long long) (p1 - p0) * layers * 2 * NKV;
    for (long long i = (long long) blockIdx.x * 8 + (threadIdx.x >> 5); i < total; i += (long long) gridDim.x * 8) {
        const int g = (int) (i % NKV), w = (int) ((i / NKV) & 1), l = (int) ((i / (2 * NKV)) % layers);
        const int pos = p0 + (int) (i / ((long long) 2 * NKV * layers));
        const KvView & kv = views[l];
        const KvSide & s = kv.s[w];
        if (!s.shadow) continue;
        float v[8];
        load_row_f16(s.shadow + ((size_t) g * kv.rc + pos % kv.rc) * HD, lane, v);
        if (s.rot) fwht256(v, lane);
        const size_t row = (size_t) g * kv.ctxp + (pos - kv.base);
        store_row(s.val + row * row_bytes(s.bits), s.sc + row * 8, v, s.bits, lane);
    }
}

// ring rows of positions [p0, p1) from the main rows: v = d * q in fp32, stored q8_0 again (qwen38_mk.cu:2488-2518)
__global__ void __launch_bounds__(256) refill_kernel(const KvView * views, int layers, int p0, int p1) {
    const int lane = threadIdx.x & 31;
    const long long total = (long long) (p1 - p0) * layers * 2 * NKV;
    for (long long i = (long long) blockIdx.x * 8 + (threadIdx.x >> 5); i < total; i += (long long) gridDim.x * 8) {
        const int g = (int) (i % NKV), w = (int) ((i / NKV) & 1), l = (int) ((i / (2 * NKV)) % layers);
        const int pos = p0 + (int) (i / ((long long) 2 * NKV * layers));
        const KvView & kv = views[l];
        const KvSide & s = kv.s[w];
        if (!s.rval) continue;
        const size_t row = (size_t) g * kv.ctxp + (pos - kv.base);
        int q[8];
        row_ints(s.val + row * row_bytes(s.bits), s.bits, lane, q);
        const float d = __half2float(__ushort_as_half(s.sc[row * 8 + (lane >> 2)]));
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = __fmul_rn(d, (float) q[k]);
        const size_t rr = (size_t) g * kv.rc + pos % kv.rc;
        store_q8(s.rval + rr * HD, s.rsc + rr * 8, v, lane);
    }
}

__global__ void __launch_bounds__(256) append_batch_kernel(const AppendJob * jobs) {
    const AppendJob & j = jobs[blockIdx.y];
    const int lane = threadIdx.x & 31, idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (idx >= j.n * 2 * NKV) return;
    const int t = idx / (2 * NKV), w = (idx / NKV) & 1, g = idx % NKV, pos = j.pos0 + t;
    append_row(j.kv, w, g, pos, (w ? j.V : j.K) + ((size_t) t * NKV + g) * HD, lane);
}
cudaError_t launch_append_batch(const AppendJob * jobs_dev, int njobs, int max_n, cudaStream_t stream) {
    if (njobs <= 0 || max_n <= 0) return cudaSuccess;
    append_batch_kernel<<<dim3((max_n * 2 * NKV + 7) / 8, njobs), 256, 0, stream>>>(jobs_dev);
    return cudaGetLastError();
}

cudaError_t launch_append(const KvView & kv, const uint16_t * K, const uint16_t * V, int pos0, int n, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    AppendArgs a{kv, K, V, pos0, n};
    append_kernel<<<(n * 2 * NKV + 7) / 8, 256, 0, stream>>>(a);
    return cudaGetLastError();
}
static int row_grid(long long rows) { return (int) std::min<long long>((rows + 7) / 8, 148 * 8); }
cudaError_t launch_spill(const KvView * views, int layers, int p0, int p1, cudaStream_t stream) {
    if (p1 <= p0) return cudaSuccess;
    spill_kernel<<<row_grid((long long) (p1 - p0) * layers * 2 * NKV), 256, 0, stream>>>(views, layers, p0, p1);
    return cudaGetLastError();
}
cudaError_t launch_refill(const KvView * views, int layers, int p0, int p1, cudaStream_t stream) {
    if (p1 <= p0) return cudaSuccess;
    refill_kernel<<<row_grid((long long) (p1 - p0) * layers * 2 * NKV), 256, 0, stream>>>(views, layers, p0, p1);
    return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------------------------------
// snapshot gather / restore scatter
// --------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_kernel(const CopyRegion * regions, int nregions, int a, int b, int ra, int rb,
                                                     unsigned long long off, unsigned long long len, uint8_t * staging, int scatter) {
    __shared__ unsigned long long start[MAX_REGIONS + 1]; // stream offset of every region
    for (int i = threadIdx.x; i < nregions; i += blockDim.x)
        start[i + 1] = (unsigned long long) regions[i].row_bytes * (unsigned long long) (regions[i].ring ? max(rb - ra, 0) : max(b - a, 0));
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long s = 0;
        for (int i = 0; i < nregions; i++) {
            const unsigned long long n = start[i + 1];
            start[i] = s;
            s += n;
        }
        start[nregions] = s;
    }
    __syncthreads();
    const unsigned long long units = len >> 4;
    for (unsigned long long u = (unsigned long long) blockIdx.x * blockDim.x + threadIdx.x; u < units;
         u += (unsigned long long) gridDim.x * blockDim.x) {
        const unsigned long long pos = off + (u << 4);
        int lo = 0, hi = nregions - 1; // last region whose start <= pos (empty regions share a start: skip to the last)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (start[mid] <= pos) lo = mid;
            else hi = mid - 1;
        }
        const CopyRegion r = regions[lo];
        uint4 * c = reinterpret_cast<uint4 *>(r.base + (unsigned long long) (r.ring ? ra : a) * r.row_bytes + (pos - start[lo]));
        uint4 * s = reinterpret_cast<uint4 *>(staging + (u << 4));
        if (scatter) *c = *s;
        else *s = *c;
    }
}
cudaError_t launch_gather(const CopyRegion * regions, int nregions, int a, int b, int ra, int rb, unsigned long long off,
                          unsigned long long len, uint8_t * staging, bool scatter, cudaStream_t stream) {
    if (len == 0) return cudaSuccess;
    const unsigned long long units = len >> 4;
    const int grid = (int) std::min<unsigned long long>((units + 255) / 256, 148ull * 8);
    gather_kernel<<<grid, 256, 0, stream>>>(regions, nregions, a, b, ra, rb, off, len, staging, scatter ? 1 : 0);
    return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------------------------------
// decode attention, baseline kernel: one CTA per (kv head, chunk) item
// --------------------------------------------------------------------------------------------------------------------
constexpr int A_THREADS = 512, A_WARPS = 16, A_STAGES = 3;
constexpr int LDH = HD + 8;   // fp16 tile row stride in halves: fragment loads hit distinct banks
constexpr int LDS = ATP + 1;  // score row stride (floats)
constexpr int LDP = ATP + 8;  // P row stride (halves)
constexpr int STAGE_SIDE = ATP * HD + ATP * SCALE_ROW; // one side of one stage: up to 32 q8 rows, then their scales

struct AttnSmem {
    uint8_t stage[A_STAGES][2][STAGE_SIDE];
    __half q[AR][LDH];
    __half k[ATP][LDH];
    __half v[ATP][LDH];
    float s[AR][LDS];
    __half p[AR][LDP];
    float m[AR], l[AR], al[AR];
    uint64_t full[A_STAGES];
    int job;
    AttnJob jobc; // the CTA's job, copied once: no parameter / global reads inside the tile loop
};
size_t attend_smem_bytes() { return sizeof(AttnSmem) + 128; }

struct AttnArgs {
    AttnJob one;          // the job when jobs == null
    const AttnJob * jobs; // device array of njobs jobs
    int njobs;
    float * part;   // [items][AR][HD]
    float2 * ml;    // [items][AR]
    int * status;
};

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) x = fmaxf(x, __shfl_xor_sync(FULL, x, m));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(FULL, x, m);
    return x;
}

// where tile tb (a multiple of 32) of side w of kv head g lives: ring rows for tiles at or after the window start
// (qwen38_mk.cu:2141-2159), else the main buffer in the side's bits
__device__ __forceinline__ int tile_src(const KvView & kv, int w, int g, int tb, int ws, const uint8_t *& val, const uint16_t *& sc) {
    const KvSide & s = kv.s[w];
    if (s.rval && tb >= ws) {
        const size_t rr = (size_t) g * kv.rc + tb % kv.rc; // rc is a multiple of 32: a tile never wraps
        val = s.rval + rr * HD;
        sc = s.rsc + rr * 8;
        return 8;
    }
    const size_t row = (size_t) g * kv.ctxp + (tb - kv.base);
    val = s.val + row * row_bytes(s.bits);
    sc = s.sc + row * 8;
    return s.bits;
}

__global__ void __launch_bounds__(A_THREADS, 1) attn_split_kernel(const __grid_constant__ AttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    AttnSmem & sm = *reinterpret_cast<AttnSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t) 127);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g8 = lane >> 2, tig = lane & 3;

    // which job this item belongs to
    if (tid == 0) {
        int j = 0;
        if (a.jobs)
            while (j + 1 < a.njobs && (int) blockIdx.x >= a.jobs[j + 1].item0) j++;
        sm.job = j;
#pragma unroll
        for (int s = 0; s < A_STAGES; s++) mbar_init(&sm.full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();
    {
        const unsigned * src = reinterpret_cast<const unsigned *>(a.jobs ? &a.jobs[sm.job] : &a.one);
        unsigned * dst = reinterpret_cast<unsigned *>(&sm.jobc);
        for (int i = tid; i < (int) (sizeof(AttnJob) / 4); i += A_THREADS) dst[i] = src[i];
    }
    __syncthreads();
    const AttnJob & J = sm.jobc;
    const int T = J.T, n = J.n, R = GQ * T, MT = (R + 15) >> 4, L = n + T;
    const int item = (int) blockIdx.x - J.item0, g = item / J.nch, c = item % J.nch;
    const int c0 = c * J.cs, c1 = min(L, c0 + J.cs), ntiles = (c1 - c0 + ATP - 1) / ATP;
    const KvView & kv = J.kv;

    auto issue = [&](int i) { // tile i of the chunk into stage i % A_STAGES (one thread)
        const int tb = c0 + i * ATP, np = min(ATP, c1 - tb), st = i % A_STAGES;
        const uint8_t *kq, *vq;
        const uint16_t *ks, *vs;
        const int kb = tile_src(kv, 0, g, tb, J.ws, kq, ks), vb = tile_src(kv, 1, g, tb, J.ws, vq, vs);
        const unsigned kbytes = np * row_bytes(kb), vbytes = np * row_bytes(vb), sbytes = np * SCALE_ROW;
        fence_proxy_async(); // the stage's previous contents were read with ordinary loads
        mbar_expect_tx(&sm.full[st], kbytes + vbytes + 2 * sbytes);
        bulk_g2s(sm.stage[st][0], kq, kbytes, &sm.full[st]);
        bulk_g2s(sm.stage[st][0] + ATP * HD, ks, sbytes, &sm.full[st]);
        bulk_g2s(sm.stage[st][1], vq, vbytes, &sm.full[st]);
        bulk_g2s(sm.stage[st][1] + ATP * HD, vs, sbytes, &sm.full[st]);
    };
    if (tid == 0)
        for (int i = 0; i < A_STAGES - 1 && i < ntiles; i++) issue(i);

    // query rows of this kv head: fp16 -> fp32 -> (K's rotation) -> x 1/16 -> fp16, row r = (head % 6) T + t (qwen38_mk.cu:2876-2883)
    for (int r = warp; r < 16 * MT; r += A_WARPS) {
        uint4 out = make_uint4(0, 0, 0, 0);
        if (r < R) {
            float v[8];
            load_row_f16(J.Q + ((size_t) (r % T) * NH + g * GQ + r / T) * HD, lane, v);
            if (kv.s[0].rot) fwht256(v, lane);
            __half2 * h = reinterpret_cast<__half2 *>(&out);
#pragma unroll
            for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(__fmul_rn(v[2 * k], 0.0625f), __fmul_rn(v[2 * k + 1], 0.0625f));
        }
        *reinterpret_cast<uint4 *>(&sm.q[r][lane * 8]) = out;
        for (int j = lane; j < LDP; j += 32) sm.p[r][j] = __float2half_rn(0.f); // padded rows of P stay zero
    }
    if (tid < AR) {
        sm.m[tid] = -CUDART_INF_F;
        sm.l[tid] = 0.f;
        sm.al[tid] = 1.f;
    }
    __syncthreads();

    constexpr int NTW = HD / 8 / A_WARPS; // 8-dim output tiles per warp in P V
    float acc[3][NTW][4];
#pragma unroll
    for (int i = 0; i < 3; i++)
#pragma unroll
        for (int j = 0; j < NTW; j++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[i][j][k] = 0.f;

    for (int i = 0; i < ntiles; i++) {
        const int tb = c0 + i * ATP, np = min(ATP, c1 - tb), st = i % A_STAGES;
        if (tid == 0 && i + A_STAGES - 1 < ntiles) issue(i + A_STAGES - 1); // (its stage was read in iteration i - 1)
        mbar_wait(&sm.full[st], (unsigned) ((i / A_STAGES) & 1), a.status);
        // staged rows -> fp16 tiles: value = fp16(d * q), one rounding (qwen38_mk.cu:2336-2343,2458-2468)
        const int kb = (kv.s[0].rval && tb >= J.ws) ? 8 : kv.s[0].bits, vb = (kv.s[1].rval && tb >= J.ws) ? 8 : kv.s[1].bits;
        for (int u = tid; u < 2 * ATP * 32; u += A_THREADS) {
            const int w = u >> 10, row = (u >> 5) & 31, cw = u & 31;
            uint4 out = make_uint4(0, 0, 0, 0);
            if (row < np) {
                const int bits = w ? vb : kb;
                const uint8_t * base = sm.stage[st][w];
                int q[8];
                row_ints(base + row * row_bytes(bits), bits, cw, q);
                const float d = __half2float(reinterpret_cast<const __half *>(base + ATP * HD)[row * 8 + (cw >> 2)]);
                __half2 * h = reinterpret_cast<__half2 *>(&out);
#pragma unroll
                for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(__fmul_rn(d, (float) q[2 * k]), __fmul_rn(d, (float) q[2 * k + 1]));
            }
            *reinterpret_cast<uint4 *>(w ? &sm.v[row][cw * 8] : &sm.k[row][cw * 8]) = out;
        }
        __syncthreads();
        // S = Q K^T: warp -> (row tile mt, positions 8 wn .. 8 wn + 7)
        if (warp < 4 * MT) {
            const int mt = warp >> 2, wn = warp & 3;
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            const __half * qa = &sm.q[16 * mt + g8][2 * tig];
            const __half * kp = &sm.k[8 * wn + g8][2 * tig];
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) {
                const unsigned a0 = *reinterpret_cast<const unsigned *>(qa + 16 * ks);
                const unsigned a1 = *reinterpret_cast<const unsigned *>(qa + 8 * LDH + 16 * ks);
                const unsigned a2 = *reinterpret_cast<const unsigned *>(qa + 16 * ks + 8);
                const unsigned a3 = *reinterpret_cast<const unsigned *>(qa + 8 * LDH + 16 * ks + 8);
                const unsigned b0 = *reinterpret_cast<const unsigned *>(kp + 16 * ks);
                const unsigned b1 = *reinterpret_cast<const unsigned *>(kp + 16 * ks + 8);
                mma16816(s, a0, a1, a2, a3, b0, b1);
            }
            float * so = &sm.s[16 * mt + g8][8 * wn + 2 * tig];
            so[0] = s[0];
            so[1] = s[1];
            so[8 * LDS] = s[2];
            so[8 * LDS + 1] = s[3];
        }
        __syncthreads();
        // online softmax per query row; row token t sees positions <= n + t (qwen38_mk.cu:2990-3016)
        for (int r = warp; r < R; r += A_WARPS) {
            const int lim = n + (r % T);
            float s0 = sm.s[r][lane];
            if (lane >= np || tb + lane > lim) s0 = -CUDART_INF_F;
            const float mt_ = warp_max(s0), mold = sm.m[r], mnew = fmaxf(mold, mt_);
            float p0 = 0.f, al = 1.f;
            if (mnew != -CUDART_INF_F) {
                p0 = expf(s0 - mnew);
                al = expf(mold - mnew);
            }
            const float ps = warp_sum(p0);
            sm.p[r][lane] = __float2half_rn(p0);
            __syncwarp();
            if (lane == 0) {
                sm.l[r] = __fmaf_rn(sm.l[r], al, ps);
                sm.m[r] = mnew;
                sm.al[r] = al;
            }
        }
        __syncthreads();
        // O = O alpha + P V: warp -> dims 8 NTW warp .. + 8 NTW - 1, all row tiles
#pragma unroll
        for (int mt = 0; mt < 3; mt++) {
            if (mt >= MT) break;
            const float al0 = sm.al[16 * mt + g8], al1 = sm.al[16 * mt + g8 + 8];
#pragma unroll
            for (int j = 0; j < NTW; j++) {
                acc[mt][j][0] *= al0;
                acc[mt][j][1] *= al0;
                acc[mt][j][2] *= al1;
                acc[mt][j][3] *= al1;
            }
            const __half * pa = &sm.p[16 * mt + g8][2 * tig];
#pragma unroll
            for (int ks = 0; ks < ATP / 16; ks++) {
                const unsigned a0 = *reinterpret_cast<const unsigned *>(pa + 16 * ks);
                const unsigned a1 = *reinterpret_cast<const unsigned *>(pa + 8 * LDP + 16 * ks);
                const unsigned a2 = *reinterpret_cast<const unsigned *>(pa + 16 * ks + 8);
                const unsigned a3 = *reinterpret_cast<const unsigned *>(pa + 8 * LDP + 16 * ks + 8);
#pragma unroll
                for (int j = 0; j < NTW; j++) {
                    const __half * vb_ = &sm.v[16 * ks + (lane & 15)][8 * (NTW * warp + j)];
                    unsigned b0, b1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(smem_u32(vb_)));
                    mma16816(acc[mt][j], a0, a1, a2, a3, b0, b1);
                }
            }
        }
        __syncthreads();
    }
    // un-normalised chunk result (m, l, O) (qwen38_mk.cu:3048-3064)
    const size_t it = blockIdx.x;
#pragma unroll
    for (int mt = 0; mt < 3; mt++) {
        if (mt >= MT) break;
#pragma unroll
        for (int j = 0; j < NTW; j++) {
            const int r0 = 16 * mt + g8, d0 = 8 * (NTW * warp + j) + 2 * tig;
            if (r0 < R) *reinterpret_cast<float2 *>(a.part + (it * AR + r0) * HD + d0) = make_float2(acc[mt][j][0], acc[mt][j][1]);
            if (r0 + 8 < R) *reinterpret_cast<float2 *>(a.part + (it * AR + r0 + 8) * HD + d0) = make_float2(acc[mt][j][2], acc[mt][j][3]);
        }
    }
    if (tid < R) a.ml[it * AR + tid] = make_float2(sm.m[tid], sm.l[tid]);
}

// merge of the chunk partials of one (query head, token), one warp per row (kv_merge.cuh)
__global__ void __launch_bounds__(256) attn_merge_kernel(const __grid_constant__ AttnArgs a, int rows_per_job, int raw, float * part_out,
                                                         float2 * ml_out) {
    const int lane = threadIdx.x & 31, idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int j = idx / rows_per_job, rr = idx % rows_per_job;
    if (j >= (a.jobs ? a.njobs : 1)) return;
    const AttnJob & J = a.jobs ? a.jobs[j] : a.one;
    if (rr >= NH * J.T) return;
    const int h = rr / J.T, t = rr % J.T, g = h / GQ;
    const size_t i0 = (size_t) J.item0 + (J.pstride > 1 ? (size_t) g : (size_t) g * J.nch);
    const size_t cstep = J.pstride > 1 ? (size_t) J.pstride : 1; // slots between consecutive partials of the kv head
    // (partials beyond 64 per kv head do not occur: nch <= 20, or #SM / 4 for the spread kernels)
    merge_row(J, a.part, a.ml, i0, cstep, J.nch, h, t, lane, raw, part_out, ml_out);
}

cudaError_t launch_attend(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int total_items, int max_T, float * part,
                          float2 * ml, int * status, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(attn_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) attend_smem_bytes());
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    AttnArgs a;
    a.one = jobs_host[0];
    a.jobs = njobs > 1 ? jobs_dev : nullptr;
    a.njobs = njobs;
    a.part = part;
    a.ml = ml;
    a.status = status;
    attn_split_kernel<<<total_items, A_THREADS, attend_smem_bytes(), stream>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int rows_per_job = NH * max_T;
    attn_merge_kernel<<<(njobs * rows_per_job + 7) / 8, 256, 0, stream>>>(a, rows_per_job, 0, nullptr, nullptr);
    return cudaGetLastError();
}

cudaError_t launch_merge(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int max_T, float * part, float2 * ml,
                         cudaStream_t stream, float * raw_part, float2 * raw_ml) {
    AttnArgs a;
    a.one = jobs_host[0];
    a.jobs = njobs > 1 ? jobs_dev : nullptr;
    a.njobs = njobs;
    a.part = part;
    a.ml = ml;
    a.status = nullptr;
    const int rows_per_job = NH * max_T;
    attn_merge_kernel<<<(njobs * rows_per_job + 7) / 8, 256, 0, stream>>>(a, rows_per_job, raw_part ? 1 : 0, raw_part, raw_ml);
    return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------------------------------
// attention with its scratch inside the device image (no allocator involved)
// --------------------------------------------------------------------------------------------------------------------
// In host code these names are only handles for cudaGetSymbolAddress: the kernels get the looked-up device addresses.
static __device__ __align__(256) float g_static_part[(size_t) STATIC_ITEMS * AR * HD];
static __device__ __align__(256) float2 g_static_ml[(size_t) STATIC_ITEMS * AR];

// Loads the library's kernels on the current device now (the runtime loads a kernel's code at its first launch otherwise, which
// takes device memory at that moment): after this, no launch of this library allocates anything.
cudaError_t preload_kernels() {
    cudaFuncAttributes fa;
    const void * fns[] = {(const void *) append_kernel, (const void *) spill_kernel, (const void *) refill_kernel, (const void *) append_batch_kernel,
                          (const void *) gather_kernel, (const void *) attn_split_kernel, (const void *) attn_merge_kernel};
    for (const void * f : fns) {
        const cudaError_t e = cudaFuncGetAttributes(&fa, f);
        if (e != cudaSuccess) return e;
    }
    void * p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_part);
    if (e != cudaSuccess) return e;
    e = preload_attend_fast();
    if (e != cudaSuccess) return e;
    return preload_attend_tc();
}

cudaError_t launch_attend_static(const AttnJob & job, int * status, cudaStream_t stream) {
    static float * part_addr[64] = {};
    static float2 * ml_addr[64] = {};
    if (NKV * job.nch > STATIC_ITEMS) return cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!part_addr[dev]) { // once per device, with that device current
        void * p = nullptr, * m = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_part);
        if (e != cudaSuccess) return e;
        e = cudaGetSymbolAddress(&m, g_static_ml);
        if (e != cudaSuccess) return e;
        ml_addr[dev] = static_cast<float2 *>(m);
        part_addr[dev] = static_cast<float *>(p);
    }
    AttnJob j = job;
    j.item0 = 0;
    // every partial row the merge reads is written by the split kernel of the same call: nothing has to start at zero.
    // One CTA per (kv head, chunk): that mode of the fast kernel needs no other scratch than the partials.
    const cudaError_t fe = launch_attend_fast(nullptr, &j, 1, NKV * j.nch, j.T, 0, part_addr[dev], ml_addr[dev], STATIC_ITEMS, nullptr, 0, 0,
                                              status, nullptr, false, stream);
    if (fe != cudaErrorNotSupported) return fe;
    return launch_attend(nullptr, &j, 1, NKV * j.nch, j.T, part_addr[dev], ml_addr[dev], status, stream);
}

} // namespace mkkv
