// KV hot-path kernels for sm_100a: append + quantize, spill, ring refill, snapshot gather / scatter, the merge of the
// decode-attention partials, and the attention entry whose scratch lives in the device image. The attention kernels
// themselves are in kv_attend_tc.cu (tcgen05) and kv_attend_fast.cu (mma.sync).
//
// Arithmetic contract (what the parity tests pin): stored bytes follow qwen38_mk.cu:2003-2116 bit for bit; the merge is
// qwen38_mk.cu:4658-4685.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <mutex>

#include "kv_kernels.h"
#include "kv_quant.cuh"
#include "kv_merge.cuh"
#include "kv_unpack.h"

namespace mkkv {

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
struct AttnArgs {
    AttnJob one;          // the job when jobs == null
    const AttnJob * jobs; // device array of njobs jobs
    int njobs;
    float * part;   // [items][AR][HD]
    float2 * ml;    // [items][AR]
};

// One staged query row: row r (0 .. 47) of kv head g = query head g 6 + r / T, token r % T. lane: dims 8 lane .. + 7 = one 16-byte
// unit of the operand layout.
__device__ __forceinline__ void qprep_row(const uint16_t * Q, uint16_t * qp, int T, int rot, int g, int r, int lane) {
    uint4 out = make_uint4(0, 0, 0, 0);
    if (r < GQ * T) {
        const uint4 rawq = *reinterpret_cast<const uint4 *>(Q + ((size_t) (r % T) * NH + g * GQ + r / T) * HD + lane * 8);
        const __half2 * hh = reinterpret_cast<const __half2 *>(&rawq);
        float v[8];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(hh[k]);
            v[2 * k] = f.x;
            v[2 * k + 1] = f.y;
        }
        if (rot) fwht256(v, lane);
        __half2 * h = reinterpret_cast<__half2 *>(&out);
#pragma unroll
        for (int k = 0; k < 4; k++) // the unit's dims in the order the unpack warps leave K's (unit_perm)
            h[k] = __floats2half2_rn(__fmul_rn(v[unit_perm(2 * k)], 0.0625f), __fmul_rn(v[unit_perm(2 * k + 1)], 0.0625f));
    }
    uint8_t * dst = reinterpret_cast<uint8_t *>(qp) + (size_t) g * QP_HEAD_BYTES + lane * (AR / 8 * 128) + (r >> 3) * 128 + (r & 7) * 16;
    *reinterpret_cast<uint4 *>(dst) = out;
}
constexpr int QP_BLOCKS = NKV * AR / 8; // blocks of 8 warps that stage one job's queries
__global__ void __launch_bounds__(256) qprep_kernel(const __grid_constant__ AttnArgs a) {
    const AttnJob & J = a.jobs ? a.jobs[blockIdx.y] : a.one;
    const int lane = threadIdx.x & 31, idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (!J.Qp) return;
    qprep_row(J.Q, const_cast<uint16_t *>(J.Qp), J.T, J.kv.s[0].rot, idx / AR, idx % AR, lane);
}
cudaError_t launch_qprep(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, cudaStream_t stream) {
    if (njobs <= 0) return cudaSuccess;
    AttnArgs a;
    a.one = jobs_host[0];
    a.jobs = njobs > 1 ? jobs_dev : nullptr;
    a.njobs = njobs;
    a.part = nullptr;
    a.ml = nullptr;
    qprep_kernel<<<dim3(QP_BLOCKS, njobs), 256, 0, stream>>>(a);
    return cudaGetLastError();
}

// the same rows for every layer of one sequence in one launch: layer = blockIdx.y, its K / V rows kv_stride bytes after the previous
// layer's (the views are the sequence's device-resident array, so a decode step uploads nothing). Blocks beyond the rows' stage the
// layer's queries for the attention launch that follows (Q != null).
__global__ void __launch_bounds__(256) append_layers_kernel(const KvView * views, const uint16_t * K, const uint16_t * V, size_t kv_stride, int pos0,
                                                            int n, const uint16_t * Q, size_t q_stride, uint16_t * qp, int T) {
    const KvView & kv = views[blockIdx.y];
    const int lane = threadIdx.x & 31, nab = (n * 2 * NKV + 7) / 8;
    if ((int) blockIdx.x >= nab) {
        const int idx = ((int) blockIdx.x - nab) * 8 + (threadIdx.x >> 5);
        qprep_row(reinterpret_cast<const uint16_t *>(reinterpret_cast<const char *>(Q) + blockIdx.y * q_stride),
                  reinterpret_cast<uint16_t *>(reinterpret_cast<char *>(qp) + (size_t) blockIdx.y * NKV * QP_HEAD_BYTES), T, kv.s[0].rot, idx / AR, idx % AR,
                  lane);
        return;
    }
    const int idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (idx >= n * 2 * NKV) return;
    const int t = idx / (2 * NKV), w = (idx / NKV) & 1, g = idx % NKV;
    const uint16_t * src = reinterpret_cast<const uint16_t *>(reinterpret_cast<const char *>(w ? V : K) + blockIdx.y * kv_stride);
    append_row(kv, w, g, pos0 + t, src + ((size_t) t * NKV + g) * HD, lane);
}
cudaError_t launch_append_layers(const KvView * views_dev, int nlayers, const uint16_t * K, const uint16_t * V, size_t kv_stride, int pos0, int n,
                                 cudaStream_t stream, const uint16_t * Q, size_t q_stride, uint16_t * qp, int T) {
    const bool stage = Q && qp && T > 0;
    if (nlayers <= 0 || (n <= 0 && !stage)) return cudaSuccess; // (n == 0 with queries: the staging alone)
    if (n < 0) n = 0;
    append_layers_kernel<<<dim3((n * 2 * NKV + 7) / 8 + (stage ? QP_BLOCKS : 0), nlayers), 256, 0, stream>>>(views_dev, K, V, kv_stride, pos0, n,
                                                                                                        stage ? Q : nullptr, q_stride, qp, T);
    return cudaGetLastError();
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
// merge of the decode-attention partials
// --------------------------------------------------------------------------------------------------------------------

// merge of the chunk partials of one (query head, token), one warp per row (kv_merge.cuh)
__global__ void __launch_bounds__(256) attn_merge_kernel(const __grid_constant__ AttnArgs a, int rows_per_job, int raw, float * part_out,
                                                         float2 * ml_out, int grouped) {
    const int lane = threadIdx.x & 31, idx = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int j = idx / rows_per_job, rr = idx % rows_per_job;
    if (j >= (a.jobs ? a.njobs : 1)) return;
    const AttnJob & J = a.jobs ? a.jobs[j] : a.one;
    if (rr >= NH * J.T) return;
    const int h = rr / J.T, t = rr % J.T, g = h / GQ;
    const size_t i0 = (size_t) J.item0 + (J.pstride > 1 ? (size_t) g : (size_t) g * J.nch);
    const size_t cstep = J.pstride > 1 ? (size_t) J.pstride : 1; // slots between consecutive partials of the kv head
    // (partials beyond 64 per kv head do not occur: nch <= 20, or #SM / 4 for the spread kernels)
    const bool packed = J.pstride > 1 && J.rstride != 0;
    // (grouped: the tensor-core kernel's batch mode left one partial per cpi chunks)
    const int count = grouped && J.cpi > 1 ? (J.nch + J.cpi - 1) / J.cpi : J.nch;
    merge_row(J, a.part, a.ml, i0, packed ? (size_t) J.rstride : cstep * AR * HD, packed ? (size_t) J.rstride / 2 : cstep * AR, count, h, t, lane, raw, part_out,
              ml_out);
}

cudaError_t launch_merge(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int max_T, float * part, float2 * ml,
                         cudaStream_t stream, float * raw_part, float2 * raw_ml, bool grouped) {
    AttnArgs a;
    a.one = jobs_host[0];
    a.jobs = njobs > 1 ? jobs_dev : nullptr;
    a.njobs = njobs;
    a.part = part;
    a.ml = ml;
    const int rows_per_job = NH * max_T;
    attn_merge_kernel<<<(njobs * rows_per_job + 7) / 8, 256, 0, stream>>>(a, rows_per_job, raw_part ? 1 : 0, raw_part, raw_ml, grouped ? 1 : 0);
    return cudaGetLastError();
}

// --------------------------------------------------------------------------------------------------------------------
// attention with its scratch inside the device image (no allocator involved)
// --------------------------------------------------------------------------------------------------------------------
// In host code these names are only handles for cudaGetSymbolAddress: the kernels get the looked-up device addresses.
static __device__ __align__(256) float g_static_part[(size_t) STATIC_ITEMS * AR * HD];
static __device__ __align__(256) float2 g_static_ml[(size_t) STATIC_ITEMS * AR];

// Loads the library's kernels on the current device now (the runtime loads a kernel's code at its first launch otherwise, which
// takes device memory at that moment): after this, no launch of this library allocates anything. Also looks up, once per device
// and with that device current, where the static scratch arrays live there (a handle of the engine's construction, never of a
// stream capture).
static std::mutex g_static_mu;
static float * g_static_part_addr[64] = {};
static float2 * g_static_ml_addr[64] = {};
cudaError_t preload_kernels() {
    cudaFuncAttributes fa;
    const void * fns[] = {(const void *) append_kernel, (const void *) spill_kernel, (const void *) refill_kernel, (const void *) append_batch_kernel, (const void *) append_layers_kernel, (const void *) qprep_kernel,
                          (const void *) gather_kernel, (const void *) attn_merge_kernel};
    for (const void * f : fns) {
        const cudaError_t e = cudaFuncGetAttributes(&fa, f);
        if (e != cudaSuccess) return e;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!g_static_part_addr[dev]) {
            void * p = nullptr, * m = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_part);
            if (e != cudaSuccess) return e;
            e = cudaGetSymbolAddress(&m, g_static_ml);
            if (e != cudaSuccess) return e;
            g_static_ml_addr[dev] = static_cast<float2 *>(m);
            g_static_part_addr[dev] = static_cast<float *>(p);
        }
    }
    e = preload_attend_fast();
    if (e != cudaSuccess) return e;
    return preload_attend_tc();
}

cudaError_t launch_attend_static(const AttnJob & job, int * status, cudaStream_t stream) {
    if (NKV * job.nch > STATIC_ITEMS) return cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    float * part;
    float2 * ml;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        part = g_static_part_addr[dev];
        ml = g_static_ml_addr[dev];
    }
    if (!part || !ml) return cudaErrorInitializationError; // (no engine was constructed on this device)
    AttnJob j = job;
    j.item0 = 0;
    j.cpi = 1;
    j.titem0 = 0;
    // every partial row the merge reads is written by the split kernel of the same call: nothing has to start at zero.
    // One CTA per (kv head, chunk): that mode of the mma.sync kernel needs no other scratch than the partials.
    return launch_attend_fast(nullptr, &j, 1, NKV * j.nch, j.T, 0, part, ml, STATIC_ITEMS, nullptr, 0, 0, status, nullptr, false, stream);
}

} // namespace mkkv
