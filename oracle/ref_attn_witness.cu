// TEST INFRASTRUCTURE ONLY. Driver around the reference project's own decode-attention kernels (attn_core_q8 / attn_core_q8m /
// attn_core_w48q / attn_core_w48m, qwen38_mk.cu:3276-4546), which oracle/build_ref.py cuts out of the reference source at build
// time (with the reference's own cutting script, bench/kvattn_gen.py) into ref_attn_cut.inc. The surrounding declarations the cut
// code expects (the constant Bufs views, the layer weights, the shared-memory block) follow what the reference's harness
// bench/kvattn_bench.cu:35-106 sets up; mk_shared.cuh is included from the reference tree where it lies.
//
// What this driver does differently from that harness: the KV cache is not random bytes but the caller's cache (main rows, scales
// and q8 rings of one layer, in the reference's layout), the RoPE table is all (cos, sin) = (1, 0) and the norm weights are one
// constant each, so that query / key rows whose mean square is exactly 1 pass the kernels' RMS-norm and RoPE prologue unchanged
// (the caller picks the constants so that rsqrtf(1 + eps) * weight rounds to 1.0f: see ref_rsqrt). The outputs are the kernels'
// split partials (apart, aml), the K / V rows they stored for the T new positions, and optionally their run time.
// Host wrappers take host buffers and do their own device allocation: this library is only ever loaded by tests, the fixture
// generator and the benchmark's reference-kernel timing, on a GPU box.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#define MK_SHARED_NS // (anonymous)
#include "mk_shared.cuh"

namespace {
__constant__ Bufs cBs[NVIEW];
__constant__ int cView;
__constant__ LayerW cL;
#define MK_ATT_PF_CTX (2 * ATT_BUCKET)
__shared__ int s_view;
#define cB cBs[s_view]
#define MK_VIEW_INIT()                          \
    do {                                        \
        if (threadIdx.x == 0) s_view = cView;   \
        __syncthreads();                        \
    } while (0)
extern __shared__ __align__(16) uint8_t smem[];

namespace kref {
__device__ __forceinline__ void attn_idle_pf(const Mat &, int, int) {}
#include "ref_attn_cut.inc"
} // namespace kref

__shared__ int s_call[4]; // the call's scalars through shared memory, as the engine passes them

template <int T> __device__ __forceinline__ void run_T(const LayerW & W, int q8, int slot, int n) {
    if constexpr (T > 5) {
        if (q8) kref::attn_core_w48q<T>(W, slot, n, -1, 0);
        else kref::attn_core_w48m<T>(W, slot, n, 0);
    } else {
        if (q8) kref::attn_core_q8<T>(W, slot, n, 0);
        else kref::attn_core_q8m<T>(W, slot, n, 0);
    }
}

__global__ void __launch_bounds__(NT, 1) w_attn(int q8, int T, int n_, int reps) {
    MK_VIEW_INIT();
    const LayerW W = cL;
    if (threadIdx.x == 0) s_call[0] = n_;
    __syncthreads();
    for (int rep = 0; rep < reps; rep++) {
        const int n = s_call[0];
        switch (T) {
        case 1: run_T<1>(W, q8, 0, n); break;
        case 2: run_T<2>(W, q8, 0, n); break;
        case 3: run_T<3>(W, q8, 0, n); break;
        case 4: run_T<4>(W, q8, 0, n); break;
        case 5: run_T<5>(W, q8, 0, n); break;
        default: run_T<8>(W, q8, 0, n); break;
        }
        __syncthreads();
    }
}

__global__ void w_rsqrt(const float * x, float * y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = rsqrtf(x[i]);
}

constexpr int GRID = 82; // the reference engine's grid (bench/kvattn_bench.cu:102)
constexpr size_t ITEMS = NKV * (ATT_NCH + 1);

struct Dev { // frees what it holds when the call returns
    std::vector<void *> p;
    ~Dev() {
        for (void * q : p) cudaFree(q);
    }
    template <class X> X * get(size_t n) {
        void * q = nullptr;
        if (cudaMalloc(&q, n * sizeof(X) + 256) != cudaSuccess) return nullptr;
        p.push_back(q);
        return static_cast<X *>(q);
    }
};
} // namespace

#define WCK(x)                                                                          \
    do {                                                                                \
        cudaError_t e_ = (x);                                                           \
        if (e_ != cudaSuccess) {                                                        \
            fprintf(stderr, "ref_attn_witness: %s: %s\n", #x, cudaGetErrorString(e_));  \
            return -1;                                                                  \
        }                                                                               \
    } while (0)

extern "C" {

// y[i] = rsqrtf(x[i]) as the GPU computes it (the kernels' RMS-norm factor)
int ref_rsqrt(const float * x, float * y, int n) {
    Dev d;
    float * dx = d.get<float>(n), * dy = d.get<float>(n);
    if (!dx || !dy) return -1;
    WCK(cudaMemcpy(dx, x, (size_t) n * 4, cudaMemcpyHostToDevice));
    w_rsqrt<<<(n + 127) / 128, 128>>>(dx, dy, n);
    WCK(cudaGetLastError());
    WCK(cudaMemcpy(y, dy, (size_t) n * 4, cudaMemcpyDeviceToHost));
    return 0;
}

// One decode-attention call of the reference kernels on the caller's cache of one layer.
//   kb, vb: bits of the K / V main rows; kr / vr: K / V stored rotated; win: MK_KV_WIN (0: no rings); ctxp: rows per kv head of the main
//   buffers; n, T: the T new tokens sit at positions n .. n + T - 1.
//   val[w] / sc[w]: main values [4][ctxp][32 bits] and scales [4][ctxp][8]; rval[w] / rsc[w]: ring values [4][rc][256] and scales
//   [4][rc][8] of a low-bit side when win > 0 (else null). Host buffers, holding positions < n.
//   q [T][24][256], k [T][4][256], v [T][4][256]: fp32 rows of the new tokens before the kernels' norm; qn, kn: the constant norm
//   weights.
//   Outputs (host): apart [84][48][256], aml [84][48][2] (item = kv head * chunks + chunk; row = (head % 6) T + t);
//   rows_val[w] [4][T][32 bits] + rows_sc[w] [4][T][8]: the main rows the call stored; rows_rval[w] [4][T][256] + rows_rsc[w]
//   [4][T][8]: the ring rows (ring sides only); us: device time of one call in microseconds (reps > 0: the median of reps timed
//   launches after 3 warm-up launches, CUDA events; reps == 0: not timed).
int ref_attn(int kb, int vb, int kr, int vr, int win, int ctxp, int n, int T, const uint8_t * const * val, const uint16_t * const * sc,
             const uint8_t * const * rval, const uint16_t * const * rsc, const float * q, const float * k, const float * v, float qn,
             float kn, float * apart, float * aml, uint8_t * const * rows_val, uint16_t * const * rows_sc, uint8_t * const * rows_rval,
             uint16_t * const * rows_rsc, int reps, float * us) {
    if (T < 1 || T > 8 || T == 6 || T == 7 || n < 0 || n + T > ctxp - 8) return -2;
    Dev d;
    Bufs hb;
    memset(&hb, 0, sizeof hb);
    const int bits[2] = {kb, vb};
    const int wb = (win + ATT_BUCKET - 1) / ATT_BUCKET, rc = win ? (wb + 1) * ATT_BUCKET + ATP : 0;
    int8_t * dval[2], * drval[2] = {nullptr, nullptr};
    __half * dsc[2], * drsc[2] = {nullptr, nullptr};
    for (int w = 0; w < 2; w++) {
        const size_t rb = (size_t) HD * bits[w] / 8, rows = (size_t) NKV * ctxp;
        dval[w] = d.get<int8_t>(rows * rb);
        dsc[w] = d.get<__half>(rows * 8);
        if (!dval[w] || !dsc[w]) return -1;
        WCK(cudaMemcpy(dval[w], val[w], rows * rb, cudaMemcpyHostToDevice));
        WCK(cudaMemcpy(dsc[w], sc[w], rows * 16, cudaMemcpyHostToDevice));
        if (win && bits[w] != 8) {
            drval[w] = d.get<int8_t>((size_t) NKV * rc * HD);
            drsc[w] = d.get<__half>((size_t) NKV * rc * 8);
            if (!drval[w] || !drsc[w]) return -1;
            WCK(cudaMemcpy(drval[w], rval[w], (size_t) NKV * rc * HD, cudaMemcpyHostToDevice));
            WCK(cudaMemcpy(drsc[w], rsc[w], (size_t) NKV * rc * 16, cudaMemcpyHostToDevice));
        }
        for (int s = 0; s < N_ATT_SLOTS; s++) {
            hb.kvp[w][s] = dval[w];
            hb.kvs[w][s] = dsc[w];
            hb.kvb[w][s] = bits[w];
            hb.kvrp[w][s] = drval[w];
            hb.kvrs[w][s] = drsc[w];
        }
    }
    for (int s = 0; s < N_ATT_SLOTS; s++) {
        hb.kvr[s] = kr;
        hb.kvrv[s] = vr;
    }
    hb.kvwin = win;
    hb.kvrc = rc;
    hb.ctx = ctxp;
    hb.kvq8 = 1;
    hb.dattn = 1;
    float * dq = d.get<float>((size_t) MAXD * QG + 64), * dk = d.get<float>((size_t) MAXD * KVD + 64), * dv = d.get<float>((size_t) MAXD * KVD + 64);
    float * dap = d.get<float>(ITEMS * AR * 256);
    float2 * dml = d.get<float2>(ITEMS * AR);
    float2 * drope = d.get<float2>((size_t) ctxp * 32);
    float * dqn = d.get<float>(HD), * dkn = d.get<float>(HD);
    if (!dq || !dk || !dv || !dap || !dml || !drope || !dqn || !dkn) return -1;
    {
        // the engine's q buffer holds, per token and head, 256 query values then 256 gate values (qwen38_mk.cu:2848)
        std::vector<float> hq((size_t) MAXD * QG, 0.f);
        for (int t = 0; t < T; t++)
            for (int h = 0; h < NH; h++) memcpy(&hq[(size_t) t * QG + (size_t) h * 512], q + ((size_t) t * NH + h) * HD, HD * 4);
        WCK(cudaMemcpy(dq, hq.data(), hq.size() * 4, cudaMemcpyHostToDevice));
        std::vector<float> hk((size_t) MAXD * KVD, 0.f), hv((size_t) MAXD * KVD, 0.f);
        memcpy(hk.data(), k, (size_t) T * KVD * 4);
        memcpy(hv.data(), v, (size_t) T * KVD * 4);
        WCK(cudaMemcpy(dk, hk.data(), hk.size() * 4, cudaMemcpyHostToDevice));
        WCK(cudaMemcpy(dv, hv.data(), hv.size() * 4, cudaMemcpyHostToDevice));
        std::vector<float2> hr((size_t) ctxp * 32, make_float2(1.f, 0.f));
        WCK(cudaMemcpy(drope, hr.data(), hr.size() * 8, cudaMemcpyHostToDevice));
        std::vector<float> w(HD, qn);
        WCK(cudaMemcpy(dqn, w.data(), HD * 4, cudaMemcpyHostToDevice));
        w.assign(HD, kn);
        WCK(cudaMemcpy(dkn, w.data(), HD * 4, cudaMemcpyHostToDevice));
    }
    hb.qbuf = dq;
    hb.kbuf = dk;
    hb.vbuf = dv;
    hb.apart = dap;
    hb.aml = dml;
    hb.rope = drope;
    LayerW hL;
    memset(&hL, 0, sizeof hL);
    hL.qn = dqn;
    hL.kn = dkn;
    WCK(cudaMemcpyToSymbol(cBs, &hb, sizeof hb));
    WCK(cudaMemcpyToSymbol(cL, &hL, sizeof hL));
    const int v0 = 0;
    WCK(cudaMemcpyToSymbol(cView, &v0, sizeof v0));
    WCK(cudaFuncSetAttribute(w_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL));
    WCK(cudaMemset(dap, 0xA5, ITEMS * AR * 256 * 4));
    WCK(cudaMemset(dml, 0xA5, ITEMS * AR * 8));
    int a_q8 = kb == 8 && vb == 8, a_T = T, a_n = n, a_reps = 1;
    void * args[] = {&a_q8, &a_T, &a_n, &a_reps};
    WCK(cudaLaunchCooperativeKernel((void *) w_attn, dim3(GRID), dim3(NT), args, SM_TOTAL, 0));
    WCK(cudaDeviceSynchronize());
    WCK(cudaMemcpy(apart, dap, ITEMS * AR * 256 * 4, cudaMemcpyDeviceToHost));
    WCK(cudaMemcpy(aml, dml, ITEMS * AR * 8, cudaMemcpyDeviceToHost));
    for (int w = 0; w < 2; w++) {
        const size_t rb = (size_t) HD * bits[w] / 8;
        for (int g = 0; g < NKV; g++) {
            const size_t r = (size_t) g * ctxp + n;
            WCK(cudaMemcpy(rows_val[w] + (size_t) g * T * rb, dval[w] + r * rb, (size_t) T * rb, cudaMemcpyDeviceToHost));
            WCK(cudaMemcpy(rows_sc[w] + (size_t) g * T * 8, dsc[w] + r * 8, (size_t) T * 16, cudaMemcpyDeviceToHost));
            if (drval[w])
                for (int t = 0; t < T; t++) {
                    const size_t rr = (size_t) g * rc + (n + t) % rc;
                    WCK(cudaMemcpy(rows_rval[w] + ((size_t) g * T + t) * HD, drval[w] + rr * HD, HD, cudaMemcpyDeviceToHost));
                    WCK(cudaMemcpy(rows_rsc[w] + ((size_t) g * T + t) * 8, drsc[w] + rr * 8, 16, cudaMemcpyDeviceToHost));
                }
        }
    }
    if (us) *us = 0.f;
    if (reps > 0 && us) {
        cudaEvent_t e0, e1;
        WCK(cudaEventCreate(&e0));
        WCK(cudaEventCreate(&e1));
        std::vector<float> t;
        for (int r = 0; r < reps + 3; r++) {
            WCK(cudaEventRecord(e0, 0));
            WCK(cudaLaunchCooperativeKernel((void *) w_attn, dim3(GRID), dim3(NT), args, SM_TOTAL, 0));
            WCK(cudaEventRecord(e1, 0));
            WCK(cudaEventSynchronize(e1));
            float ms = 0.f;
            WCK(cudaEventElapsedTime(&ms, e0, e1));
            if (r >= 3) t.push_back(ms * 1000.f);
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        for (size_t i = 1; i < t.size(); i++) // insertion sort: a handful of samples
            for (size_t j = i; j > 0 && t[j] < t[j - 1]; j--) {
                const float x = t[j];
                t[j] = t[j - 1];
                t[j - 1] = x;
            }
        *us = t[t.size() / 2];
    }
    return 0;
}

// The reference kernels' run time alone on a cache of random bytes (as the reference's own harness times them,
// bench/kvattn_bench.cu:258-283): device time of one call in microseconds, the median of reps launches after 3 warm-up launches.
int ref_attn_time(int kb, int vb, int kr, int win, int n, int T, int reps, float * us) {
    const int ctxp = n + T + 16 + 16;
    const int bits[2] = {kb, vb};
    const int wb = (win + ATT_BUCKET - 1) / ATT_BUCKET, rc = win ? (wb + 1) * ATT_BUCKET + ATP : 0;
    std::vector<uint8_t> hv[2], hrv[2];
    std::vector<uint16_t> hs[2], hrs[2];
    uint64_t s = 0x9E3779B97F4A7C15ull;
    auto next = [&]() {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        return s;
    };
    auto fill = [&](std::vector<uint8_t> & b, size_t nb) {
        b.resize(nb + 8);
        for (size_t i = 0; i + 8 <= nb + 8; i += 8) {
            const uint64_t x = next();
            memcpy(&b[i], &x, 8);
        }
    };
    auto fill_sc = [&](std::vector<uint16_t> & b, size_t nh) { // magnitudes around 0.1, both signs
        b.resize(nh);
        for (size_t i = 0; i < nh; i++) {
            const uint64_t x = next();
            b[i] = (uint16_t) ((((x >> 32) & 1) << 15) | ((9 + (x >> 8) % 8) << 10) | ((x >> 16) & 0x3ff));
        }
    };
    const uint8_t * pv[2], * prv[2] = {nullptr, nullptr};
    const uint16_t * ps[2], * prs[2] = {nullptr, nullptr};
    for (int w = 0; w < 2; w++) {
        fill(hv[w], (size_t) NKV * ctxp * HD * bits[w] / 8);
        fill_sc(hs[w], (size_t) NKV * ctxp * 8);
        pv[w] = hv[w].data();
        ps[w] = hs[w].data();
        if (win && bits[w] != 8) {
            fill(hrv[w], (size_t) NKV * rc * HD);
            fill_sc(hrs[w], (size_t) NKV * rc * 8);
            prv[w] = hrv[w].data();
            prs[w] = hrs[w].data();
        }
    }
    std::vector<float> q((size_t) T * NH * HD), k((size_t) T * KVD), v((size_t) T * KVD);
    for (auto * a : {&q, &k, &v})
        for (float & x : *a) x = (float) ((int) (next() % 129) - 64) / 32.f;
    std::vector<float> ap(ITEMS * AR * 256), ml(ITEMS * AR * 2);
    std::vector<uint8_t> rv[2], rrv[2];
    std::vector<uint16_t> rs[2], rrs[2];
    uint8_t * o_v[2], * o_rv[2];
    uint16_t * o_s[2], * o_rs[2];
    for (int w = 0; w < 2; w++) {
        rv[w].resize((size_t) NKV * T * HD);
        rrv[w].resize((size_t) NKV * T * HD);
        rs[w].resize((size_t) NKV * T * 8);
        rrs[w].resize((size_t) NKV * T * 8);
        o_v[w] = rv[w].data();
        o_rv[w] = rrv[w].data();
        o_s[w] = rs[w].data();
        o_rs[w] = rrs[w].data();
    }
    return ref_attn(kb, vb, kr, 0, win, ctxp, n, T, pv, ps, prv, prs, q.data(), k.data(), v.data(), 1.f, 1.f, ap.data(), ml.data(), o_v, o_s,
                    o_rv, o_rs, reps, us);
}
}
