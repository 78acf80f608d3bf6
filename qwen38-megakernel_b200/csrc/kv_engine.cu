// KvEngine implementation: see kv_engine.h. Host logic only; every device operation is a launcher from kv_kernels.h or a
// CUDA runtime copy. Compute runs on the engine's stream; snapshot / restore copies run on a side stream and are tied to
// the compute stream by events.
#include "kv_engine.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unistd.h>

namespace mkkv {

// A sticky error means the context is lost: nothing can be reset, the process ends with code 4 as the reference does
// (mk_shared.cuh:170-198). Everything else becomes MKCudaError and the C API resets the engine.
static bool context_lost(cudaError_t e) {
    switch (e) {
    case cudaErrorIllegalAddress:
    case cudaErrorLaunchFailure:
    case cudaErrorIllegalInstruction:
    case cudaErrorMisalignedAddress:
    case cudaErrorInvalidAddressSpace:
    case cudaErrorInvalidPc:
    case cudaErrorHardwareStackError:
    case cudaErrorLaunchTimeout:
    case cudaErrorECCUncorrectable:
    case cudaErrorAssert:
    case cudaErrorDevicesUnavailable:
        return true;
    default:
        return false;
    }
}
void cuda_fail(cudaError_t e, const char * what, const char * file, int line) {
    char msg[512];
    snprintf(msg, sizeof msg, "CUDA error %s (%s) at %s:%d", cudaGetErrorString(e), what, file, line);
    cudaGetLastError();
    // sticky = the context is lost: the error repeats after it was cleared (the reference's test, mk_shared.cuh:170-198)
    if (context_lost(e) || context_lost(cudaDeviceSynchronize())) {
        fprintf(stderr, "[mk] sticky %s: exiting with code 4\n", msg);
        fflush(stderr);
        std::_Exit(4);
    }
    cudaGetLastError();
    throw MKCudaError(msg);
}

constexpr int XCH_NB_MIN = 64; // fewest batches per chunk the exchange arrays of the spread attention kernels hold

namespace {
// One item of the MK_KV grammar (loader.cu:1329-1366): <K|V|*><layer|*|empty>=<4..8>[r]. The messages are the reference's.
struct SpecItem {
    bool sides[2]; // applies to K / to V
    int layer;     // -1: every layer
    int bits;
    bool rotated;
};
SpecItem parse_spec_item(const std::string & item, int layers) {
    const auto bad = [&](const std::string & what) -> std::runtime_error { return std::runtime_error("MK_KV: " + what); };
    const size_t eq = item.find('=');
    const char side = item.empty() ? 0 : item[0];
    if (eq == std::string::npos || eq == 0 || (side != 'K' && side != 'V' && side != '*')) throw bad("bad item " + item);
    SpecItem it;
    it.sides[0] = side != 'V';
    it.sides[1] = side != 'K';
    // the format: one digit 4 .. 8, optionally followed by r
    const std::string fmt = item.substr(eq + 1);
    const bool fmt_ok = (fmt.size() == 1 || (fmt.size() == 2 && fmt[1] == 'r')) && fmt[0] >= '4' && fmt[0] <= '8';
    if (!fmt_ok) throw bad("expected 4..8 or 4r..8r in " + item);
    it.bits = fmt[0] - '0';
    it.rotated = fmt.size() == 2;
    // the layer: nothing or * for all, else a decimal number below the layer count
    const std::string which = item.substr(1, eq - 1);
    it.layer = -1;
    if (!which.empty() && which != "*") {
        bool digits = true;
        long v = 0;
        for (char ch : which) {
            digits = digits && ch >= '0' && ch <= '9' && v < 100000;
            v = v * 10 + (ch - '0');
        }
        if (!digits || v >= layers) throw bad("bad slot in " + item + " (0.." + std::to_string(layers - 1) + " or *)");
        it.layer = (int) v;
    }
    return it;
}
// the items apply in order, later ones override earlier ones
bool parse_spec(const std::string & spec, int layers, int (*kvb)[MAX_LAYERS], int (*rot)[MAX_LAYERS]) {
    for (size_t at = 0; at <= spec.size();) {
        const size_t comma = std::min(spec.find(',', at), spec.size());
        if (comma > at) {
            const SpecItem it = parse_spec_item(spec.substr(at, comma - at), layers);
            for (int w = 0; w < 2; w++)
                for (int l = it.layer < 0 ? 0 : it.layer; it.sides[w] && l < (it.layer < 0 ? layers : it.layer + 1); l++) {
                    kvb[w][l] = it.bits;
                    rot[w][l] = it.rotated;
                }
        }
        at = comma + 1;
    }
    return true;
}
double ms_since(std::chrono::steady_clock::time_point t0) {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}
} // namespace

KvEngine::KvEngine(const EngineConfig & cfg) : cfg_(cfg) {
    if (cfg.layers < 1 || cfg.layers > MAX_LAYERS) throw std::runtime_error("layers must be 1.." + std::to_string(MAX_LAYERS));
    if (cfg.ctx < 1) throw std::runtime_error("ctx must be positive");
    for (int w = 0; w < 2; w++)
        for (int s = 0; s < MAX_LAYERS; s++) {
            kvb_[w][s] = 8;
            rot_[w][s] = 0;
            ring_[w][s] = false;
        }
    parse_spec(cfg.kv_spec, cfg.layers, kvb_, rot_);
    // the window needs a format spec, as in the reference (loader.cu:1478)
    if (cfg.kv_spec.empty() || cfg.win <= 0) cfg_.win = 0;
    rc_ = kv_ring_rows(cfg_.win);
    for (int w = 0; w < 2; w++)
        for (int s = 0; s < cfg.layers; s++) ring_[w][s] = cfg_.win > 0 && (kvb_[w][s] != 8 || cfg.win_all);
    if (cfg_.win <= 0) cfg_.spill = false;
    MKKV_CK(cudaGetDevice(&dev_));
    try {
        init_device_state();
    } catch (...) { // (a constructor that throws runs no destructor: what was made so far is released here)
        release();
        throw;
    }
}

void KvEngine::init_device_state() {
    const EngineConfig & cfg = cfg_;
    MKKV_CK(cudaStreamCreateWithFlags(&st_copy_, cudaStreamNonBlocking));
    MKKV_CK(cudaEventCreateWithFlags(&ev_compute_, cudaEventDisableTiming));
    MKKV_CK(cudaEventCreateWithFlags(&ev_copy_, cudaEventDisableTiming));
    MKKV_CK(cudaHostAlloc(reinterpret_cast<void **>(&h_status_), sizeof(int), cudaHostAllocMapped));
    *h_status_ = 0;
    MKKV_CK(cudaHostGetDevicePointer(reinterpret_cast<void **>(&d_status_), h_status_, 0));
    if (const char * c = getenv("MK_STORE_CHUNK_MIB")) {
        const long v = atol(c);
        if (v >= 1 && v <= 1024) hs_chunk_ = (size_t) v << 20;
    }
    MKKV_CK(cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, dev_));
    MKKV_CK(preload_kernels());
    // MK_KV_ATTN: "tc" (default: the tcgen05 kernel, the mma.sync kernel as its fallback) or "fast" (the mma.sync kernel only)
    if (const char * c = getenv("MK_KV_ATTN")) use_tc_ = strcmp(c, "fast") != 0;
    ensure_xch(((cfg.ctx + ATT_BUCKET - 1) / ATT_BUCKET + 3) / 4 + 2);
    MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&tc_done_), NKV * sizeof(unsigned)));
    MKKV_CK(cudaMemset(tc_done_, 0, NKV * sizeof(unsigned)));
    if (const char * c = getenv("MK_KV_PROFILE"))
        if (atoi(c) > 0) {
            MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&prof_), attend_fast_prof_words(num_sms_) * sizeof(unsigned long long)));
            MKKV_CK(cudaMemset(prof_, 0, attend_fast_prof_words(num_sms_) * sizeof(unsigned long long)));
        }
    alloc_seq(main_, cfg.ctx);
    ensure_work(std::max(NKV * ATT_NCH, num_sms_), 1);
    ensure_qprep(cfg.layers);
}

// exchange arrays of the spread attention kernels: two of [4][20][nb][48] words (zeroed: no word carries a launch tag yet)
void KvEngine::ensure_xch(int nb) {
    if (nb <= xnb_) return;
    nb = std::max(nb, XCH_NB_MIN);
    if (xmax_) {
        MKKV_CK(cudaStreamSynchronize(stream_));
        MKKV_CK(cudaFree(xmax_));
        xmax_ = nullptr;
    }
    const size_t words = 2 * (size_t) NKV * ATT_NCH * nb * AR;
    MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&xmax_), words * sizeof(unsigned long long)));
    MKKV_CK(cudaMemset(xmax_, 0, words * sizeof(unsigned long long)));
    xnb_ = nb;
}

// the decode-attention launches of one call: the tensor-core kernel, else the mma.sync one (spread over the grid, or, for shapes
// that mode does not take, one CTA per (kv head, chunk) item)
void KvEngine::launch_attention(const AttnJob * jobs_host, int njobs, int items, int max_T) {
    if (use_tc_ && njobs == 1) {
        const cudaError_t e = launch_attend_tc(jobs_host[0], num_sms_, part_, ml_, work_items_, xmax_, xmax_ + (size_t) NKV * ATT_NCH * xnb_ * AR,
                                               xnb_, ++epoch_, d_status_, stream_, nullptr, 0, 0, nullptr, nullptr, prof_, tc_done_, &tc_done_seq_);
        if (e == cudaSuccess) {
            launches_ += 1;
            return;
        }
        if (e != cudaErrorNotSupported && e != cudaErrorCooperativeLaunchTooLarge) MKKV_CK(e);
        cudaGetLastError();
    }
    if (use_tc_ && njobs > 1) {
        const cudaError_t e = launch_attend_tc_batch(d_jobs_, jobs_host, njobs, items, max_T, part_, ml_, work_items_, d_status_, stream_);
        if (e == cudaSuccess) {
            launches_ += 2;
            return;
        }
        if (e != cudaErrorNotSupported) MKKV_CK(e);
        cudaGetLastError();
    }
    {
        const cudaError_t e = launch_attend_fast(d_jobs_, jobs_host, njobs, items, max_T, num_sms_, part_, ml_, work_items_, xmax_,
                                                 std::min(xnb_, 64), ++epoch_, d_status_, njobs == 1 ? prof_ : nullptr, true, stream_);
        if (e == cudaSuccess) {
            launches_ += 2;
            return;
        }
        if (e != cudaErrorNotSupported && e != cudaErrorCooperativeLaunchTooLarge) MKKV_CK(e);
        cudaGetLastError();
    }
    MKKV_CK(launch_attend_fast(d_jobs_, jobs_host, njobs, items, max_T, num_sms_, part_, ml_, work_items_, nullptr, 0, 0, d_status_, nullptr,
                               false, stream_));
    launches_ += 2;
}

KvEngine::~KvEngine() { release(); }

void KvEngine::release() {
    cudaSetDevice(dev_);
    cudaDeviceSynchronize();
    free_seq(main_);
    for (auto & s : slots_) free_seq(s);
    for (auto & p : parked_)
        for (char * c : p.second.blob.chunks) cudaFreeHost(c);
    for (char * c : sw_blob_.chunks) cudaFreeHost(c);
    for (char * c : hs_free_) cudaFreeHost(c);
    for (auto & k : sw_cks_)
        if (k.ring) cudaFreeHost(k.ring);
    cudaFree(part_);
    cudaFree(ml_);
    cudaFree(d_jobs_);
    cudaFreeHost(h_jobs_);
    cudaFree(d_ajobs_);
    cudaFreeHost(h_ajobs_);
    cudaFree(d_tasks_);
    cudaFreeHost(h_tasks_);
    cudaFree(staging_);
    cudaFree(xmax_);
    cudaFree(tc_done_);
    cudaFree(qprep_);
    cudaFree(prof_);
    if (h_status_) cudaFreeHost(h_status_);
    if (ev_compute_) cudaEventDestroy(ev_compute_);
    if (ev_copy_) cudaEventDestroy(ev_copy_);
    if (st_copy_) cudaStreamDestroy(st_copy_);
    cudaGetLastError();
}

void KvEngine::use_device() const { MKKV_CK(cudaSetDevice(dev_)); }
void KvEngine::check_layer(int layer) const {
    if (layer < 0 || layer >= cfg_.layers) throw std::runtime_error("layer " + std::to_string(layer) + " out of range");
}
KvEngine::Seq & KvEngine::seq_ref(int seq) {
    if (seq == SEQ_MAIN) return main_;
    if (seq < 0 || seq >= (int) slots_.size()) throw std::runtime_error("no sequence slot " + std::to_string(seq));
    return slots_[seq];
}
const KvEngine::Seq & KvEngine::seq_ref(int seq) const { return const_cast<KvEngine *>(this)->seq_ref(seq); }

void KvEngine::alloc_seq(Seq & s, int ctx) {
    s.ctx = ctx;
    s.ctxp = ctx + KV_PAD;
    const size_t rows = (size_t) NKV * s.ctxp;
    size_t vb[2] = {0, 0};
    int nring = 0;
    for (int w = 0; w < 2; w++)
        for (int l = 0; l < cfg_.layers; l++) {
            vb[w] += rows * row_bytes(kvb_[w][l]);
            nring += ring_[w][l];
        }
    try {
        for (int w = 0; w < 2; w++) {
            MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.val[w]), vb[w]));
            MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.sc[w]), (size_t) cfg_.layers * rows * SCALE_ROW));
            MKKV_CK(cudaMemsetAsync(s.val[w], 0, vb[w], stream_));
            MKKV_CK(cudaMemsetAsync(s.sc[w], 0, (size_t) cfg_.layers * rows * SCALE_ROW, stream_));
            dev_bytes_ += vb[w] + (size_t) cfg_.layers * rows * SCALE_ROW;
        }
        const size_t rrows = (size_t) nring * NKV * rc_;
        if (rrows) {
            MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.ring_val), rrows * HD));
            MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.ring_sc), rrows * SCALE_ROW));
            MKKV_CK(cudaMemsetAsync(s.ring_val, 0, rrows * HD, stream_));
            MKKV_CK(cudaMemsetAsync(s.ring_sc, 0, rrows * SCALE_ROW, stream_));
            dev_bytes_ += rrows * (HD + SCALE_ROW);
            if (cfg_.spill) {
                MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.shadow), rrows * HD * 2));
                MKKV_CK(cudaMemsetAsync(s.shadow, 0, rrows * HD * 2, stream_));
                dev_bytes_ += rrows * HD * 2;
            }
        }
        s.views.assign(cfg_.layers, KvView{});
        s.regions.clear();
        size_t off[2] = {0, 0};
        int ri = 0;
        std::vector<CopyRegion> ring_regions;
        for (int l = 0; l < cfg_.layers; l++) {
            KvView & v = s.views[l];
            v.ctxp = s.ctxp;
            v.rc = rc_;
            v.win = cfg_.win;
            v.eager = cfg_.spill ? 0 : 1;
            v.base = 0;
            for (int w = 0; w < 2; w++) { // layers packed one after another in each side's allocation (loader.cu:1457-1468)
                KvSide & sd = v.s[w];
                sd.bits = kvb_[w][l];
                sd.rot = rot_[w][l];
                sd.val = s.val[w] + off[w];
                sd.sc = s.sc[w] + (size_t) l * rows * 8;
                off[w] += rows * row_bytes(sd.bits);
                sd.rval = nullptr;
                sd.rsc = nullptr;
                sd.shadow = nullptr;
                if (ring_[w][l]) {
                    sd.rval = s.ring_val + (size_t) ri * NKV * rc_ * HD;
                    sd.rsc = s.ring_sc + (size_t) ri * NKV * rc_ * 8;
                    if (s.shadow) sd.shadow = s.shadow + (size_t) ri * NKV * rc_ * HD;
                    ri++;
                }
                for (int g = 0; g < NKV; g++) {
                    s.regions.push_back({sd.val + (size_t) g * s.ctxp * row_bytes(sd.bits), (unsigned) row_bytes(sd.bits), 0u});
                    s.regions.push_back({reinterpret_cast<uint8_t *>(sd.sc + (size_t) g * s.ctxp * 8), (unsigned) SCALE_ROW, 0u});
                    if (sd.rval) {
                        ring_regions.push_back({sd.rval + (size_t) g * rc_ * HD, (unsigned) HD, 1u});
                        ring_regions.push_back({reinterpret_cast<uint8_t *>(sd.rsc + (size_t) g * rc_ * 8), (unsigned) SCALE_ROW, 1u});
                    }
                }
            }
        }
        s.regions.insert(s.regions.end(), ring_regions.begin(), ring_regions.end());
        MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.d_views), sizeof(KvView) * cfg_.layers));
        MKKV_CK(cudaMemcpy(s.d_views, s.views.data(), sizeof(KvView) * cfg_.layers, cudaMemcpyHostToDevice));
        MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&s.d_regions), sizeof(CopyRegion) * s.regions.size()));
        MKKV_CK(cudaMemcpy(s.d_regions, s.regions.data(), sizeof(CopyRegion) * s.regions.size(), cudaMemcpyHostToDevice));
        MKKV_CK(cudaEventCreateWithFlags(&s.copy_done, cudaEventDisableTiming));
        MKKV_CK(cudaStreamSynchronize(stream_));
    } catch (...) {
        free_seq(s);
        throw;
    }
    s.n = s.kv_top = 0;
    s.spilled.assign(cfg_.layers, 0);
    s.cks.clear();
}

void KvEngine::free_seq(Seq & s) {
    for (int w = 0; w < 2; w++) {
        cudaFree(s.val[w]);
        cudaFree(s.sc[w]);
        s.val[w] = nullptr;
        s.sc[w] = nullptr;
    }
    cudaFree(s.ring_val);
    cudaFree(s.ring_sc);
    cudaFree(s.shadow);
    cudaFree(s.d_views);
    cudaFree(s.d_regions);
    s.ring_val = nullptr;
    s.ring_sc = nullptr;
    s.shadow = nullptr;
    s.d_views = nullptr;
    s.d_regions = nullptr;
    for (auto & k : s.cks)
        if (k.ring) cudaFreeHost(k.ring);
    s.cks.clear();
    if (s.copy_done) cudaEventDestroy(s.copy_done);
    s.copy_done = nullptr;
}

void KvEngine::sync() {
    use_device();
    MKKV_CK(cudaStreamSynchronize(stream_));
    MKKV_CK(cudaStreamSynchronize(st_copy_));
    copies_in_flight_ = false;
    if (*h_status_ != KS_OK) {
        const int st = *h_status_;
        *h_status_ = KS_OK;
        throw MKCudaError("a kernel gave up waiting for its staged tiles (status " + std::to_string(st) + ")");
    }
}

int KvEngine::slots_open(int n, int ctx) {
    use_device();
    if (n < 0 || n > 1024) throw std::runtime_error("slots_open: n out of range");
    if (ctx <= 0) ctx = cfg_.ctx;
    sync();
    for (auto & s : slots_) free_seq(s);
    slots_.clear();
    slots_.resize(n);
    try {
        for (auto & s : slots_) alloc_seq(s, ctx);
    } catch (...) {
        for (auto & s : slots_) free_seq(s);
        slots_.clear();
        throw;
    }
    return ctx;
}

void KvEngine::drop_checkpoints(Seq & s, int after) {
    for (size_t i = 0; i < s.cks.size();)
        if (s.cks[i].pos > after) {
            if (s.cks[i].ring) cudaFreeHost(s.cks[i].ring);
            s.cks.erase(s.cks.begin() + i);
        } else i++;
}

void KvEngine::reset(int seq) {
    Seq & s = seq_ref(seq);
    s.n = s.kv_top = 0;
    std::fill(s.spilled.begin(), s.spilled.end(), s.base); // (a split sequence keeps its base: no main row below it exists)
    drop_checkpoints(s, -1);
    s.failed = false;
}
void KvEngine::reset_all() {
    reset(SEQ_MAIN);
    for (int i = 0; i < (int) slots_.size(); i++) reset(i);
    if (sw_on_) {
        sw_on_ = false;
        hs_release(sw_blob_);
        for (auto & k : sw_cks_)
            if (k.ring) cudaFreeHost(k.ring);
        sw_cks_.clear();
        sw_pieces_.clear();
    }
}
int KvEngine::position(int seq) const { return seq_ref(seq).n; }
int KvEngine::kv_top(int seq) const { return seq_ref(seq).kv_top; }
void KvEngine::commit(int seq, int len) {
    Seq & s = seq_ref(seq);
    if (len < 0 || len > s.kv_top) throw std::runtime_error("commit: length " + std::to_string(len) + " beyond the rows written (" + std::to_string(s.kv_top) + ")");
    s.n = len;
}

void KvEngine::wait_copies(Seq & s) {
    if (s.copy_pending) {
        MKKV_CK(cudaStreamWaitEvent(stream_, s.copy_done, 0));
        s.copy_pending = false;
    }
}

// spill mode: main-format rows of positions [spilled, upto) of one layer from the fp16 shadow
void KvEngine::spill_to(Seq & s, int layer, int upto) {
    if (!cfg_.spill || upto <= s.spilled[layer]) return;
    MKKV_CK(launch_spill(s.d_views + layer, 1, s.spilled[layer], upto, stream_));
    launches_++;
    s.spilled[layer] = upto;
}

void KvEngine::append(int seq, int layer, int pos0, int n, const void * K, const void * V) {
    use_device();
    check_layer(layer);
    Seq & s = seq_ref(seq);
    if (n < 0 || pos0 < s.base || (long long) pos0 + n - s.base > s.ctx)
        throw std::runtime_error("append: rows " + std::to_string(pos0) + " + " + std::to_string(n) + " outside the sequence's rows [" + std::to_string(s.base) + ", " + std::to_string(s.base + s.ctx) + ")");
    if (n == 0) return;
    if (!K || !V) throw std::runtime_error("append: null K / V");
    if (seq == SEQ_MAIN && sw_on_) sw_need(pos0 + n);
    wait_copies(s);
    const uint16_t * k = static_cast<const uint16_t *>(K), * v = static_cast<const uint16_t *>(V);
    if (cfg_.spill && rc_ > 0) {
        // a row's shadow slot is reused by the position rc later: rows about to be displaced are spilled first, and a long
        // run is cut into pieces of at most one ring so no piece displaces its own rows
        for (int done = 0; done < n;) {
            const int p = pos0 + done, m = std::min(n - done, rc_);
            spill_to(s, layer, std::min(p, p + m - rc_));
            MKKV_CK(launch_append(s.views[layer], k + (size_t) done * NKV * HD, v + (size_t) done * NKV * HD, p, m, stream_));
            launches_++;
            done += m;
        }
    } else {
        MKKV_CK(launch_append(s.views[layer], k, v, pos0, n, stream_));
        launches_++;
    }
    s.kv_top = std::max(s.kv_top, pos0 + n);
}

void KvEngine::step_layers(int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, void * O, size_t kv_stride,
                           size_t q_stride, size_t o_stride, int layer0) {
    use_device();
    if (nlayers < 0 || layer0 < 0 || layer0 + nlayers > cfg_.layers)
        throw std::runtime_error("step_layers: layers must lie in 0.." + std::to_string(cfg_.layers));
    if (nlayers == 0) return;
    Seq & s = seq_ref(seq);
    // The appends of all layers are independent of one another and of the previous layers' attention: they go out as one launch
    // (the per-layer form costs a launch between every two attention kernels), and the same launch stages the layers' queries
    // for the tensor-core kernel. Anything the single-layer append would do first is done first here too; a call it would
    // refuse takes the per-layer route and gets its message there.
    const bool one_launch = T >= 1 && T <= MAXT && K && V && n >= s.base && (long long) n + T - s.base <= s.ctx && kv_stride % 2 == 0;
    bool staged = false; // the layers' queries are staged by the append launch
    if (one_launch) {
        if (seq == SEQ_MAIN && sw_on_) sw_need(n + T);
        wait_copies(s);
        if (cfg_.spill && rc_ > 0)
            for (int l = layer0; l < layer0 + nlayers; l++) spill_to(s, l, n + T - rc_); // rows about to be displaced get their main-format row first
        const bool stage = use_tc_ && Q && q_stride % 16 == 0 && reinterpret_cast<uintptr_t>(Q) % 16 == 0;
        MKKV_CK(launch_append_layers(s.d_views + layer0, nlayers, static_cast<const uint16_t *>(K), static_cast<const uint16_t *>(V), kv_stride, n, T, stream_,
                                     stage ? static_cast<const uint16_t *>(Q) : nullptr, q_stride, qprep_ + (size_t) layer0 * NKV * (QP_HEAD_BYTES / 2), T));
        launches_++;
        s.kv_top = std::max(s.kv_top, n + T);
        staged = stage;
    }
    for (int l = 0; l < nlayers; l++) {
        if (!one_launch) append(seq, layer0 + l, n, T, static_cast<const char *>(K) + l * kv_stride, static_cast<const char *>(V) + l * kv_stride);
        attend_impl(seq, layer0 + l, n, T, static_cast<const char *>(Q) + l * q_stride, static_cast<char *>(O) + l * o_stride, staged);
    }
}

void KvEngine::ensure_qprep(int slots) {
    if (slots <= qprep_slots_) return;
    MKKV_CK(cudaStreamSynchronize(stream_));
    cudaFree(qprep_);
    qprep_ = nullptr;
    MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&qprep_), (size_t) slots * NKV * QP_HEAD_BYTES));
    qprep_slots_ = slots;
}
// the job's queries in the tensor-core kernel's operand layout: slot `slot` of the staging buffer, filled here by a launch of its own
// unless the caller (a decode step whose append launch staged every layer's queries a moment ago) says it is
void KvEngine::staged_q(AttnJob & j, int slot, bool staged) {
    j.Qp = qprep_ + (size_t) slot * NKV * (QP_HEAD_BYTES / 2);
    if (staged) return;
    MKKV_CK(launch_qprep(nullptr, &j, 1, stream_));
    launches_++;
}

void KvEngine::ensure_work(int items, int njobs) {
    if (items > work_items_) {
        MKKV_CK(cudaStreamSynchronize(stream_));
        cudaFree(part_);
        cudaFree(ml_);
        part_ = nullptr;
        ml_ = nullptr;
        MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&part_), (size_t) items * AR * HD * sizeof(float)));
        MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&ml_), (size_t) items * AR * sizeof(float2)));
        work_items_ = items;
    }
    if (njobs > work_jobs_) {
        MKKV_CK(cudaStreamSynchronize(stream_));
        cudaFree(d_jobs_);
        cudaFreeHost(h_jobs_);
        cudaFree(d_ajobs_);
        cudaFreeHost(h_ajobs_);
        d_jobs_ = nullptr;
        h_jobs_ = nullptr;
        d_ajobs_ = nullptr;
        h_ajobs_ = nullptr;
        MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&d_jobs_), sizeof(AttnJob) * njobs));
        MKKV_CK(cudaHostAlloc(reinterpret_cast<void **>(&h_jobs_), sizeof(AttnJob) * njobs, cudaHostAllocDefault));
        MKKV_CK(cudaMalloc(&d_ajobs_, sizeof(AppendJob) * njobs));
        MKKV_CK(cudaHostAlloc(&h_ajobs_, sizeof(AppendJob) * njobs, cudaHostAllocDefault));
        work_jobs_ = njobs;
    }
}
void KvEngine::reserve_batch(int njobs) {
    use_device();
    if (njobs < 1 || njobs > 4096) throw std::runtime_error("reserve_batch: njobs out of range");
    ensure_work(std::max(njobs * NKV * ATT_NCH, num_sms_), njobs);
    ensure_qprep(std::max(njobs, cfg_.layers));
}

// a call that needs the whole sequence on this GPU: not for a sequence whose rows start at a non-zero base (mk_kv_set_base)
void KvEngine::need_whole(const Seq & s, const char * what) const {
    if (s.base != 0)
        throw std::runtime_error(std::string(what) + ": not available on a sequence split by position (its rows start at position " +
                                 std::to_string(s.base) + "); use attend_partial / combine");
}

// The job of T query tokens at n over the whole context of one (sequence, layer), after the checks every attention entry shares:
// the rows exist; the T rows share one partition, i.e. n + 1 .. n + T do not cross a multiple of 640 (the reference's host rule,
// mk_shared.cuh:288-291: results are independent of T only then); the window's rows are still in the ring.
AttnJob KvEngine::whole_job(const Seq & s, const char * what, int layer, int n, int T, const void * Q, void * O) const {
    const std::string w(what);
    need_whole(s, what);
    if (T < 1 || T > MAXT) throw std::runtime_error(w + ": T must be 1.." + std::to_string(MAXT));
    if (n < 0 || n + T > s.kv_top) throw std::runtime_error(w + ": rows up to " + std::to_string(n + T) + " have not been appended (" + std::to_string(s.kv_top) + " written)");
    if (att_cap_T(n, T) < T)
        throw std::runtime_error(w + ": " + std::to_string(T) + " tokens at position " + std::to_string(n) + " cross a multiple of " + std::to_string(ATT_BUCKET) +
                                 " (at most " + std::to_string(att_cap_T(n, T)) + " share one partition: mk_kv_cap_T)");
    if (!Q || !O) throw std::runtime_error(w + ": null Q / O");
    AttnJob j;
    j.kv = s.views[layer];
    j.Q = static_cast<const uint16_t *>(Q);
    j.Qp = nullptr;
    j.O = static_cast<float *>(O);
    j.n = n;
    j.T = T;
    attn_dims(n + T, j.nch, j.cs);
    j.ws = kv_ws(n + T, cfg_.win);
    j.item0 = 0;
    j.cpi = 1;
    j.titem0 = 0;
    j.pos_lo = 0;
    j.pos_hi = n + T;
    j.pstride = 1;
    j.rstride = 0;
    // positions >= ws are read from the ring, which holds the newest rc rows written: an attend at an earlier n after rows far
    // beyond it were appended would read later positions' rows
    if (rc_ > 0 && (j.kv.s[0].rval || j.kv.s[1].rval) && s.kv_top > j.ws + rc_)
        throw std::runtime_error(w + ": the window rows of a call at position " + std::to_string(n) + " were overwritten (rows up to " +
                                 std::to_string(s.kv_top) + " written); truncate first");
    return j;
}

void KvEngine::attend(int seq, int layer, int n, int T, const void * Q, void * O) { attend_impl(seq, layer, n, T, Q, O, false); }
void KvEngine::attend_impl(int seq, int layer, int n, int T, const void * Q, void * O, bool q_staged) {
    use_device();
    check_layer(layer);
    Seq & s = seq_ref(seq);
    AttnJob j = whole_job(s, "attend", layer, n, T, Q, O);
    wait_copies(s);
    spill_to(s, layer, j.ws); // positions that left the window are read in the main format from now on
    if (use_tc_) staged_q(j, layer, q_staged);
    launch_attention(&j, 1, NKV * j.nch, T);
}

void KvEngine::set_base(int seq, int base) {
    use_device();
    Seq & s = seq_ref(seq);
    if (s.n != 0 || s.kv_top != 0) throw std::runtime_error("set_base: the sequence is not empty");
    if (base < 0 || base % ATP) throw std::runtime_error("set_base: the base must be a non-negative multiple of 32");
    MKKV_CK(cudaStreamSynchronize(stream_));
    s.base = base;
    for (auto & v : s.views) v.base = base;
    MKKV_CK(cudaMemcpy(s.d_views, s.views.data(), sizeof(KvView) * cfg_.layers, cudaMemcpyHostToDevice));
    std::fill(s.spilled.begin(), s.spilled.end(), base);
    s.kv_top = s.n = 0;
}

void KvEngine::attend_partial(int seq, int layer, int n, int T, const void * Q, int pos_lo, int pos_hi, void * part_out, void * ml_out) {
    attend_partial_impl(seq, layer, n, T, Q, pos_lo, pos_hi, part_out, ml_out, false);
}
void KvEngine::attend_partial_impl(int seq, int layer, int n, int T, const void * Q, int pos_lo, int pos_hi, void * part_out, void * ml_out,
                                   bool q_staged) {
    use_device();
    check_layer(layer);
    Seq & s = seq_ref(seq);
    if (T < 1 || T > MAXT) throw std::runtime_error("attend_partial: T must be 1.." + std::to_string(MAXT));
    if (!Q || !part_out || !ml_out) throw std::runtime_error("attend_partial: null argument");
    const int L = n + T;
    if (n < 0 || att_cap_T(n, T) < T)
        throw std::runtime_error("attend_partial: " + std::to_string(T) + " tokens at position " + std::to_string(n) + " cross a multiple of " + std::to_string(ATT_BUCKET));
    if (pos_hi != pos_lo && (pos_lo % ATP || pos_lo < s.base || pos_hi > L || pos_hi < pos_lo || (pos_hi != L && pos_hi % ATP)))
        throw std::runtime_error("attend_partial: bad position range [" + std::to_string(pos_lo) + ", " + std::to_string(pos_hi) + ")");
    if (pos_hi > pos_lo && pos_hi > s.kv_top) throw std::runtime_error("attend_partial: rows up to " + std::to_string(pos_hi) + " have not been appended (" + std::to_string(s.kv_top) + " written)");
    wait_copies(s);
    AttnJob j;
    j.kv = s.views[layer];
    j.Q = static_cast<const uint16_t *>(Q);
    j.Qp = nullptr;
    j.O = nullptr;
    j.n = n;
    j.T = T;
    attn_dims(L, j.nch, j.cs);
    j.ws = kv_ws(L, cfg_.win);
    j.item0 = 0;
    j.cpi = 1;
    j.titem0 = 0;
    j.pos_lo = pos_lo;
    j.pos_hi = pos_hi;
    j.pstride = 1;
    j.rstride = 0;
    if (pos_hi > pos_lo) spill_to(s, layer, std::min(j.ws, pos_hi)); // rows of this range that left the window
    if (use_tc_) staged_q(j, layer, q_staged);
    std::vector<AttnTask> tasks;
    bool tc = use_tc_;
    for (;; tc = false) { // the tensor-core kernel first (4 tiles per task), else the fast kernel (8)
        // the task list depends on the partition and the range only: a rank whose range does not end at the context's end keeps
        // the list of the previous step (no rebuild, no upload)
        const int B = tc ? 4 : 8;
        const long long key[5] = {j.nch, j.cs, pos_lo, pos_hi, B};
        int nt = tasks_n_;
        if (memcmp(key, tasks_key_, sizeof(key)) != 0 || tasks_n_ < 0) {
            const int max_nb = build_range_tasks(j, B, tasks);
            if (tc) ensure_xch(max_nb);
            else if (max_nb > std::min(xnb_, 64)) throw std::runtime_error("attend_partial: the context is too long for the exchange buffers");
            nt = (int) tasks.size();
            if (nt > tasks_cap_) {
                MKKV_CK(cudaStreamSynchronize(stream_));
                cudaFree(d_tasks_);
                cudaFreeHost(h_tasks_);
                d_tasks_ = nullptr;
                h_tasks_ = nullptr;
                tasks_cap_ = std::max(nt, 4096);
                MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&d_tasks_), sizeof(AttnTask) * tasks_cap_));
                MKKV_CK(cudaHostAlloc(reinterpret_cast<void **>(&h_tasks_), sizeof(AttnTask) * tasks_cap_, cudaHostAllocDefault));
            }
            MKKV_CK(cudaEventSynchronize(ev_compute_)); // the previous upload has been consumed
            if (nt) memcpy(h_tasks_, tasks.data(), sizeof(AttnTask) * nt);
            if (nt) MKKV_CK(cudaMemcpyAsync(d_tasks_, h_tasks_, sizeof(AttnTask) * nt, cudaMemcpyHostToDevice, stream_));
            MKKV_CK(cudaEventRecord(ev_compute_, stream_));
            memcpy(tasks_key_, key, sizeof(key));
            tasks_n_ = nt;
        }
        cudaError_t e;
        if (tc)
            e = launch_attend_tc(j, num_sms_, part_, ml_, work_items_, xmax_, xmax_ + (size_t) NKV * ATT_NCH * xnb_ * AR, xnb_, ++epoch_, d_status_,
                                 stream_, d_tasks_, nt, B, static_cast<float *>(part_out), static_cast<float2 *>(ml_out), nullptr, tc_done_, &tc_done_seq_);
        else
            e = launch_attend_fast(d_jobs_, &j, 1, NKV * j.nch, T, num_sms_, part_, ml_, work_items_, xmax_, std::min(xnb_, 64), ++epoch_, d_status_,
                                   nullptr, true, stream_, d_tasks_, nt, B, static_cast<float *>(part_out), static_cast<float2 *>(ml_out));
        if (e == cudaSuccess) {
            launches_ += tc ? 1 : 2; // (the tensor-core kernel merges in its tail)
            break;
        }
        if (!tc || (e != cudaErrorNotSupported && e != cudaErrorCooperativeLaunchTooLarge)) MKKV_CK(e);
        cudaGetLastError();
    }
}

void KvEngine::combine(int layer, int T, int nparts, const void * parts, const void * mls, void * O) {
    use_device();
    check_layer(layer);
    if (T < 1 || T > MAXT || nparts < 1 || nparts > 64 || !parts || !mls || !O) throw std::runtime_error("combine: bad arguments");
    AttnJob j;
    j.kv = main_.views[layer]; // (only the V rotation flag is read)
    j.Q = nullptr;
    j.Qp = nullptr;
    j.O = static_cast<float *>(O);
    j.n = 0;
    j.T = T;
    j.nch = nparts;
    j.cs = 0;
    j.ws = 0;
    j.item0 = 0;
    j.cpi = 1;
    j.titem0 = 0;
    j.pos_lo = j.pos_hi = 0;
    j.pstride = NKV; // partial p of kv head g is slot p * 4 + g
    j.rstride = 0;
    MKKV_CK(launch_merge(nullptr, &j, 1, T, const_cast<float *>(static_cast<const float *>(parts)),
                         const_cast<float2 *>(static_cast<const float2 *>(mls)), stream_));
    launches_ += 1;
}

// One decode step of a sequence split by position, all layers in one call (the host stays out of the per-layer loop): layer l
// appends the rows of [n, n + T) that fall into [own_lo, own_hi) and attends over [pos_lo, min(pos_hi, n + T)); its partial goes to
// parts + l * 4 * 48 * 256 floats and mls + l * 4 * 48 * 2 floats. The arrays of all ranks, gathered in rank order, are what
// combine_layers takes.
void KvEngine::step_layers_partial(int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, size_t kv_stride,
                                   size_t q_stride, int own_lo, int own_hi, int pos_lo, int pos_hi, void * parts, void * mls) {
    if (nlayers < 0 || nlayers > cfg_.layers) throw std::runtime_error("step_layers_partial: nlayers must be 0.." + std::to_string(cfg_.layers));
    if (T < 1 || T > MAXT) throw std::runtime_error("step_layers_partial: T must be 1.." + std::to_string(MAXT));
    const int a = std::max(n, own_lo), b = std::min(n + T, own_hi), hi = std::min(pos_hi, n + T);
    bool staged = false;
    if (nlayers > 0) { // the rows this rank owns, every layer in one launch (as step_layers), with the layers' queries staged
        use_device();
        Seq & s = seq_ref(seq);
        const int m = std::max(0, b - a);
        if (m > 0) {
            if (!K || !V) throw std::runtime_error("step_layers_partial: null K / V");
            if (a < s.base || (long long) b - s.base > s.ctx)
                throw std::runtime_error("step_layers_partial: rows " + std::to_string(a) + " .. " + std::to_string(b) + " outside the sequence's rows");
            if (seq == SEQ_MAIN && sw_on_) sw_need(b);
            wait_copies(s);
            if (cfg_.spill && rc_ > 0)
                for (int l = 0; l < nlayers; l++) spill_to(s, l, b - rc_);
        }
        const bool stage = use_tc_ && Q && q_stride % 16 == 0 && reinterpret_cast<uintptr_t>(Q) % 16 == 0;
        if (m > 0 || stage) {
            const size_t skip = (size_t) (m > 0 ? a - n : 0) * NKV * HD * 2;
            MKKV_CK(launch_append_layers(s.d_views, nlayers, reinterpret_cast<const uint16_t *>(static_cast<const char *>(K) + skip),
                                         reinterpret_cast<const uint16_t *>(static_cast<const char *>(V) + skip), kv_stride, a, m, stream_,
                                         stage ? static_cast<const uint16_t *>(Q) : nullptr, q_stride, qprep_, T));
            launches_++;
        }
        if (m > 0) s.kv_top = std::max(s.kv_top, b);
        staged = stage;
    }
    for (int l = 0; l < nlayers; l++) {
        attend_partial_impl(seq, l, n, T, static_cast<const char *>(Q) + l * q_stride, pos_lo, hi > pos_lo ? hi : pos_lo,
                            static_cast<float *>(parts) + (size_t) l * NKV * AR * HD, static_cast<float *>(mls) + (size_t) l * NKV * AR * 2, staged);
    }
}

// The merge of every layer's partials in one launch: parts [nparts][nlayers][4][48][256], mls [nparts][nlayers][4][48][2] (the ranks'
// step_layers_partial outputs gathered in rank order); layer l's output goes to O + l * o_stride bytes. rank_stride != 0: rank p's
// two arrays start rank_stride * p bytes after parts and mls (each rank's arrays packed into one exchange buffer).
void KvEngine::combine_layers(int nlayers, int T, int nparts, const void * parts, const void * mls, void * O, size_t o_stride, size_t rank_stride) {
    use_device();
    if (nlayers < 1 || nlayers > cfg_.layers || T < 1 || T > MAXT || nparts < 1 || nparts > 64 || !parts || !mls || !O)
        throw std::runtime_error("combine_layers: bad arguments");
    if (rank_stride % 8) throw std::runtime_error("combine_layers: the stride between the ranks' arrays must be a multiple of 8 bytes");
    ensure_work(work_items_, nlayers);
    MKKV_CK(cudaEventSynchronize(ev_compute_)); // the previous upload of the job table has been consumed
    for (int l = 0; l < nlayers; l++) {
        AttnJob & j = h_jobs_[l];
        j.kv = main_.views[l]; // (only the V rotation flag is read)
        j.Q = nullptr;
        j.Qp = nullptr;
        j.O = reinterpret_cast<float *>(static_cast<char *>(O) + l * o_stride);
        j.n = 0;
        j.T = T;
        j.nch = nparts;
        j.cs = 0;
        j.ws = 0;
        j.item0 = l * NKV;          // partial p of kv head g of layer l is slot (p * nlayers + l) * 4 + g
        j.cpi = 1;
        j.titem0 = 0;
        j.pos_lo = j.pos_hi = 0;
        j.pstride = nlayers * NKV;
        j.rstride = (long long) (rank_stride / 4); // (0: the ranks' arrays lie one after another)
    }
    MKKV_CK(cudaMemcpyAsync(d_jobs_, h_jobs_, sizeof(AttnJob) * nlayers, cudaMemcpyHostToDevice, stream_));
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    MKKV_CK(launch_merge(d_jobs_, h_jobs_, nlayers, T, const_cast<float *>(static_cast<const float *>(parts)),
                         const_cast<float2 *>(static_cast<const float2 *>(mls)), stream_));
    launches_ += 1;
}

void KvEngine::attend_static(int seq, int layer, int n, int T, const void * Q, void * O) {
    use_device();
    check_layer(layer);
    Seq & s = seq_ref(seq);
    if (T < 1 || T > MAXT) throw std::runtime_error("attend_static: T must be 1.." + std::to_string(MAXT) + " (the fixed scratch holds " + std::to_string(AR) + " query rows per item)");
    const AttnJob j = whole_job(s, "attend_static", layer, n, T, Q, O);
    if (NKV * j.nch > STATIC_ITEMS)
        throw std::runtime_error("attend_static: the call needs " + std::to_string(NKV * j.nch) + " partial items, the fixed scratch holds " + std::to_string(STATIC_ITEMS));
    wait_copies(s);
    spill_to(s, layer, j.ws);
    MKKV_CK(launch_attend_static(j, d_status_, stream_));
    launches_ += 2;
}

void KvEngine::step_batch(int njobs, const int * seqs, int layer, const int * n, const int * T, const void * K, const void * V, const void * Q,
                          void * O, bool do_append) {
    use_device();
    check_layer(layer);
    if (njobs < 1) return;
    if (njobs > work_jobs_) throw std::runtime_error("step_batch: call reserve_batch(" + std::to_string(njobs) + ") first");
    // the job tables are reused by every call: the previous call's upload must have been consumed
    MKKV_CK(cudaEventSynchronize(ev_compute_));
    AppendJob * aj = static_cast<AppendJob *>(h_ajobs_);
    int items = 0, tc_items = 0, maxT = 0;
    size_t row = 0;
    for (int j = 0; j < njobs; j++) {
        Seq & s = seq_ref(seqs[j]);
        for (int k = 0; k < j; k++)
            if (seqs[k] == seqs[j]) throw std::runtime_error("step_batch: sequence listed twice");
        if (T[j] < 1 || T[j] > MAXT) throw std::runtime_error("step_batch: T must be 1.." + std::to_string(MAXT));
        if (n[j] < 0 || n[j] + T[j] > (do_append ? s.ctx : s.kv_top)) throw std::runtime_error("step_batch: rows out of range for job " + std::to_string(j));
        need_whole(s, "step_batch");
        // a side request keeps the main sequence's rows aside lazily: they are copied out before this call overwrites them
        if (do_append && seqs[j] == SEQ_MAIN && sw_on_) sw_need(n[j] + T[j]);
        wait_copies(s);
        if (do_append && cfg_.spill && rc_ > 0) spill_to(s, layer, n[j] + T[j] - rc_);
        if (do_append) s.kv_top = std::max(s.kv_top, n[j] + T[j]);
        AttnJob & a = h_jobs_[j];
        a = whole_job(s, "step_batch", layer, n[j], T[j], static_cast<const uint16_t *>(Q) + row * NH * HD, static_cast<float *>(O) + row * NH * HD);
        a.item0 = items;
        if (use_tc_ && j < qprep_slots_) a.Qp = qprep_ + (size_t) j * NKV * (QP_HEAD_BYTES / 2); // (staged below, every job in one launch)
        items += NKV * a.nch;
        // the tensor-core kernel's CTAs: a CTA costs about two groups' time besides its groups, so chunks of fewer than
        // TC_ITEM_GROUPS groups of 128 positions share one (the long sequences' chunks stay one per CTA: they balance the SMs).
        // 32 sequences of 2,000 .. 100,000 positions, tokens per second: 13.2 k with one chunk per CTA, 14.2 k / 14.4 k / 14.7 k /
        // 14.5 k with 8 / 12 / 16 / 24 groups
        constexpr int TC_ITEM_GROUPS = 16;
        const int nb_full = (a.cs / ATP + 3) / 4;
        a.cpi = std::max(1, std::min(a.nch, (TC_ITEM_GROUPS + nb_full - 1) / std::max(nb_full, 1)));
        a.titem0 = tc_items;
        tc_items += NKV * ((a.nch + a.cpi - 1) / a.cpi);
        maxT = std::max(maxT, T[j]);
        aj[j].kv = a.kv;
        aj[j].K = static_cast<const uint16_t *>(K) + row * NKV * HD;
        aj[j].V = static_cast<const uint16_t *>(V) + row * NKV * HD;
        aj[j].pos0 = n[j];
        aj[j].n = T[j];
        row += T[j];
        spill_to(s, layer, a.ws);
    }
    if (items > work_items_) throw std::runtime_error("step_batch: call reserve_batch first");
    if (do_append) {
        MKKV_CK(cudaMemcpyAsync(d_ajobs_, h_ajobs_, sizeof(AppendJob) * njobs, cudaMemcpyHostToDevice, stream_));
        MKKV_CK(launch_append_batch(static_cast<const AppendJob *>(d_ajobs_), njobs, maxT, stream_));
        launches_++;
    }
    MKKV_CK(cudaMemcpyAsync(d_jobs_, h_jobs_, sizeof(AttnJob) * njobs, cudaMemcpyHostToDevice, stream_));
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    if (use_tc_ && h_jobs_[0].Qp) {
        MKKV_CK(launch_qprep(d_jobs_, h_jobs_, njobs, stream_));
        launches_++;
    }
    launch_attention(h_jobs_, njobs, items, maxT);
}

// ---- rewind ----

// ring rows of positions that the abandoned continuation overwrote are rebuilt from the main rows (ck_pool.cu:285-296)
void KvEngine::ring_rewind(Seq & s, int P) {
    if (cfg_.win > 0) {
        const int p0 = std::max(s.base, P - rc_), p1 = std::min(P, s.kv_top - rc_); // (a split sequence holds no rows below its base)
        if (p1 > p0) MKKV_CK(launch_refill(s.d_views, cfg_.layers, p0, p1, stream_));
    }
    s.kv_top = std::min(s.kv_top, P);
    for (int & sp : s.spilled) sp = std::min(sp, P);
}

void KvEngine::truncate(int seq, int len) {
    use_device();
    Seq & s = seq_ref(seq);
    if (s.base != 0 && len != 0) need_whole(s, "truncate");
    if (len < 0 || len > s.n) throw std::runtime_error("truncate: length " + std::to_string(len) + " not inside the sequence (" + std::to_string(s.n) + ")");
    wait_copies(s);
    ring_rewind(s, len);
    s.n = len;
    drop_checkpoints(s, len);
}

size_t KvEngine::ring_state_bytes() const {
    size_t nring = 0;
    for (int w = 0; w < 2; w++)
        for (int l = 0; l < cfg_.layers; l++) nring += ring_[w][l];
    return nring * NKV * rc_ * (HD + SCALE_ROW);
}

int KvEngine::checkpoint(int seq) {
    use_device();
    Seq & s = seq_ref(seq);
    need_whole(s, "checkpoint");
    const int pos = s.n;
    for (auto & k : s.cks)
        if (k.pos == pos) return pos;
    int max_slots = 8;
    if (const char * c = getenv("MK_CK_SLOTS")) max_slots = std::max(1, atoi(c));
    if ((int) s.cks.size() >= max_slots) { // the oldest goes (the reference thins by coverage; any policy keeps rewinds exact)
        if (s.cks.front().ring) cudaFreeHost(s.cks.front().ring);
        s.cks.erase(s.cks.begin());
    }
    Checkpoint k;
    k.pos = pos;
    const size_t rb = ring_state_bytes();
    if (cfg_.exact && rb) { // the rings as of pos, so a rewind restores them exactly (ck_pool.cu:135-158)
        MKKV_CK(cudaHostAlloc(reinterpret_cast<void **>(&k.ring), rb, cudaHostAllocDefault));
        const size_t vbytes = rb / (HD + SCALE_ROW) * HD;
        wait_copies(s);
        MKKV_CK(cudaEventRecord(ev_compute_, stream_));
        MKKV_CK(cudaStreamWaitEvent(st_copy_, ev_compute_, 0));
        MKKV_CK(cudaMemcpyAsync(k.ring, s.ring_val, vbytes, cudaMemcpyDeviceToHost, st_copy_));
        MKKV_CK(cudaMemcpyAsync(k.ring + vbytes, s.ring_sc, rb - vbytes, cudaMemcpyDeviceToHost, st_copy_));
        MKKV_CK(cudaEventRecord(s.copy_done, st_copy_));
        s.copy_pending = true; // the next launch that writes ring rows waits for the copy
        k.ring_ok = true;
    }
    s.cks.push_back(k);
    std::sort(s.cks.begin(), s.cks.end(), [](const Checkpoint & a, const Checkpoint & b) { return a.pos < b.pos; });
    return pos;
}

std::vector<int> KvEngine::checkpoints(int seq) const {
    std::vector<int> v;
    for (const auto & k : seq_ref(seq).cks) v.push_back(k.pos);
    return v;
}

bool KvEngine::rewind_to(int seq, int pos) {
    use_device();
    Seq & s = seq_ref(seq);
    need_whole(s, "rewind_to");
    const Checkpoint * ck = nullptr;
    for (const auto & k : s.cks)
        if (k.pos == pos && pos >= 0) ck = &k;
    if (!ck) return false;
    wait_copies(s);
    if (ck->ring_ok) { // exact mode: the rings go back to their state at pos (ck_pool.cu:208-214,279)
        const size_t rb = ring_state_bytes(), vbytes = rb / (HD + SCALE_ROW) * HD;
        MKKV_CK(cudaMemcpyAsync(s.ring_val, ck->ring, vbytes, cudaMemcpyHostToDevice, stream_));
        MKKV_CK(cudaMemcpyAsync(s.ring_sc, ck->ring + vbytes, rb - vbytes, cudaMemcpyHostToDevice, stream_));
        s.kv_top = std::min(s.kv_top, pos);
        for (int & sp : s.spilled) sp = std::min(sp, pos);
    } else {
        ring_rewind(s, pos);
    }
    s.n = pos;
    drop_checkpoints(s, pos);
    return true;
}

bool KvEngine::rewind_to_checkpoint(int seq) { // the last one (qwen38_mk.h:97-101)
    const Seq & s = seq_ref(seq);
    return !s.cks.empty() && rewind_to(seq, s.cks.back().pos);
}

// ---- host store ----

char * KvEngine::hs_new() {
    if (hs_alloc_ + hs_chunk_ > hs_budget_) return nullptr;
    char * c = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void **>(&c), hs_chunk_, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    hs_alloc_ += hs_chunk_;
    return c;
}
char * KvEngine::hs_take() {
    if (!hs_free_.empty()) {
        char * c = hs_free_.back();
        hs_free_.pop_back();
        return c;
    }
    return hs_new();
}
void KvEngine::hs_trim() {
    while (hs_alloc_ > hs_budget_ && !hs_free_.empty()) {
        cudaFreeHost(hs_free_.back());
        hs_free_.pop_back();
        hs_alloc_ -= hs_chunk_;
    }
}
void KvEngine::hs_release(Blob & b) {
    for (char * c : b.chunks) hs_free_.push_back(c);
    b = Blob();
    hs_trim();
}
// chunks for `bytes` more bytes of b; false: the budget is spent (b keeps what it has)
bool KvEngine::blob_room(Blob & b, size_t bytes) {
    const size_t need = (b.used + bytes + hs_chunk_ - 1) / hs_chunk_;
    while (b.chunks.size() < need) {
        char * c = hs_take();
        if (!c) return false;
        b.chunks.push_back(c);
    }
    return true;
}
size_t KvEngine::hs_used() const {
    size_t n = sw_blob_.chunks.size();
    for (const auto & p : parked_) n += p.second.blob.chunks.size();
    return n * hs_chunk_;
}
void KvEngine::store_budget(size_t bytes) {
    use_device();
    hs_budget_ = bytes;
    hs_trim();
}
void KvEngine::store_reserve(size_t bytes) {
    use_device();
    size_t free_b = hs_free_.size() * hs_chunk_;
    while (free_b < bytes) {
        char * c = hs_new();
        if (!c) break;
        hs_free_.push_back(c);
        free_b += hs_chunk_;
    }
}
KvEngine::StoreInfo KvEngine::store_info() const {
    StoreInfo i;
    i.budget = hs_budget_;
    i.allocated = hs_alloc_;
    i.used = hs_used();
    i.parked = (int) parked_.size();
    i.last_ms = hs_ms_;
    i.last_bytes = hs_bytes_;
    i.side_ms = sw_ms_;
    i.side_park_bytes = sw_park_bytes_;
    i.side_park_ms = sw_park_ms_;
    return i;
}
void KvEngine::kv_sizes(size_t * per_token, size_t * rings, size_t * state, size_t * checkpoint) const {
    size_t t = 0;
    for (int l = 0; l < cfg_.layers; l++)
        for (int w = 0; w < 2; w++) t += (size_t) NKV * (row_bytes(kvb_[w][l]) + SCALE_ROW);
    *per_token = t;
    *rings = ring_state_bytes();
    *state = 0; // no recurrent state on this path
    *checkpoint = cfg_.exact ? ring_state_bytes() : 0;
}

void KvEngine::ensure_staging() {
    if (!staging_) MKKV_CK(cudaMalloc(reinterpret_cast<void **>(&staging_), 2 * hs_chunk_));
}

size_t KvEngine::stream_bytes(const Seq & s, int a, int b, int ra, int rb) const {
    size_t t = 0;
    for (const auto & r : s.regions) t += (size_t) r.row_bytes * (size_t) std::max(0, r.ring ? rb - ra : b - a);
    return t;
}

void KvEngine::run_copy(Seq & s, int a, int b, int ra, int rb, Blob & blob, size_t blob_off, bool to_host) {
    ensure_staging();
    const size_t total = stream_bytes(s, a, b, ra, rb);
    int k = 0;
    for (size_t off = 0; off < total; k++) {
        const size_t bpos = blob_off + off, ci = bpos / hs_chunk_, co = bpos % hs_chunk_;
        const size_t len = std::min(total - off, hs_chunk_ - co);
        uint8_t * stage = staging_ + (size_t) (k & 1) * hs_chunk_;
        if (to_host) {
            MKKV_CK(launch_gather(s.d_regions, (int) s.regions.size(), a, b, ra, rb, off, len, stage, false, st_copy_));
            MKKV_CK(cudaMemcpyAsync(blob.chunks[ci] + co, stage, len, cudaMemcpyDeviceToHost, st_copy_));
        } else {
            MKKV_CK(cudaMemcpyAsync(stage, blob.chunks[ci] + co, len, cudaMemcpyHostToDevice, st_copy_));
            MKKV_CK(launch_gather(s.d_regions, (int) s.regions.size(), a, b, ra, rb, off, len, stage, true, st_copy_));
        }
        off += len;
    }
}

void KvEngine::store_wait() {
    use_device();
    MKKV_CK(cudaStreamSynchronize(st_copy_));
    copies_in_flight_ = false;
}

size_t KvEngine::park_need(int seq, int max_checkpoints) const {
    const Seq & s = seq_ref(seq);
    size_t t = stream_bytes(s, 0, s.n, 0, rc_);
    int k = 0;
    for (auto it = s.cks.rbegin(); it != s.cks.rend() && k < max_checkpoints; ++it, ++k)
        if (it->ring_ok) t += ring_state_bytes();
    return t;
}
size_t KvEngine::park_bytes(int id) const {
    const auto it = parked_.find(id);
    return it == parked_.end() ? 0 : it->second.blob.used;
}
void KvEngine::unpack_probe(int bits, const void * rows, const void * scales, int nrows, void * out) {
    use_device();
    if (bits < 4 || bits > 8 || nrows < 0 || (nrows && (!rows || !scales || !out))) throw std::runtime_error("unpack_probe: bad arguments");
    MKKV_CK(launch_unpack_probe(bits, static_cast<const uint8_t *>(rows), static_cast<const uint16_t *>(scales), nrows, static_cast<uint16_t *>(out), stream_));
    launches_++;
}

// ---- prompt-state file (state_files.cu:97-238) ----
// The regions in the file's order: for every layer, side, kv head the values of rows 0 .. hend - 1, then their scales (:103-110);
// then for every (layer, side) with a ring all heads' ring values, then all heads' ring scales (:115-119).
std::vector<std::pair<char *, size_t>> KvEngine::state_regions(Seq & s, int hend) const {
    std::vector<std::pair<char *, size_t>> r;
    for (int l = 0; l < cfg_.layers; l++)
        for (int w = 0; w < 2; w++) {
            const KvSide & sd = s.views[l].s[w];
            for (int g = 0; g < NKV; g++) {
                r.push_back({reinterpret_cast<char *>(sd.val + (size_t) g * s.ctxp * row_bytes(sd.bits)), (size_t) hend * row_bytes(sd.bits)});
                r.push_back({reinterpret_cast<char *>(sd.sc + (size_t) g * s.ctxp * 8), (size_t) hend * SCALE_ROW});
            }
        }
    for (int l = 0; l < cfg_.layers; l++)
        for (int w = 0; w < 2; w++) {
            const KvSide & sd = s.views[l].s[w];
            if (!sd.rval) continue;
            r.push_back({reinterpret_cast<char *>(sd.rval), (size_t) NKV * rc_ * HD});
            r.push_back({reinterpret_cast<char *>(sd.rsc), (size_t) NKV * rc_ * SCALE_ROW});
        }
    return r;
}

namespace {
constexpr char STATE_MAGIC[9] = "MKSTATE1";
constexpr size_t STATE_PIECE = (size_t) 32 << 20;
struct PinnedPiece { // one pinned staging buffer for the file's pieces
    uint8_t * p = nullptr;
    PinnedPiece() { if (cudaHostAlloc(reinterpret_cast<void **>(&p), STATE_PIECE, cudaHostAllocDefault) != cudaSuccess) p = nullptr, cudaGetLastError(); }
    ~PinnedPiece() { if (p) cudaFreeHost(p); }
};
} // namespace

long long KvEngine::state_save(int seq, const char * path, const void * key, size_t key_len, int hend, const void * const * extra,
                               const size_t * extra_sizes, int n_extra) {
    use_device();
    Seq & s = seq_ref(seq);
    need_whole(s, "state_save");
    if (!path || (key_len && !key) || n_extra < 0 || (n_extra && (!extra || !extra_sizes))) throw std::runtime_error("state_save: null argument");
    if (hend < 0 || hend != s.kv_top)
        throw std::runtime_error("state_save: hend (" + std::to_string(hend) + ") must equal the rows written (" + std::to_string(s.kv_top) + "): the rings in the file are those of exactly that state");
    for (int l = 0; l < cfg_.layers; l++) spill_to(s, l, hend); // spill mode: every position gets its main-format row first
    wait_copies(s);
    MKKV_CK(cudaStreamSynchronize(stream_));
    auto R = state_regions(s, hend);
    for (int i = 0; i < n_extra; i++) R.push_back({static_cast<char *>(const_cast<void *>(extra[i])), extra_sizes[i]});
    const std::string tmp = std::string(path) + ".tmp" + std::to_string((long long) getpid());
    FILE * f = fopen(tmp.c_str(), "wb");
    if (!f) throw std::runtime_error(std::string("state_save: cannot write ") + tmp);
    bool ok = fwrite(STATE_MAGIC, 8, 1, f) == 1;
    auto w64 = [&](uint64_t v) { ok = ok && fwrite(&v, 8, 1, f) == 1; };
    w64(key_len);
    ok = ok && (key_len == 0 || fwrite(key, 1, key_len, f) == key_len);
    w64((uint64_t) hend);
    w64(R.size());
    long long tot = 8 + 8 + (long long) key_len + 8 + 8 + 8 * (long long) R.size();
    for (const auto & r : R) w64(r.second), tot += (long long) r.second;
    PinnedPiece buf;
    if (!buf.p) {
        fclose(f);
        unlink(tmp.c_str());
        throw std::runtime_error("state_save: no pinned staging buffer");
    }
    try {
        for (const auto & r : R)
            for (size_t o = 0; ok && o < r.second; o += STATE_PIECE) {
                const size_t n = std::min(STATE_PIECE, r.second - o);
                MKKV_CK(cudaMemcpy(buf.p, r.first + o, n, cudaMemcpyDefault));
                ok = fwrite(buf.p, 1, n, f) == n;
            }
    } catch (...) { // (a CUDA error: no half-written file is left behind, state_files.cu:163-167)
        fclose(f);
        unlink(tmp.c_str());
        throw;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path) != 0) {
        unlink(tmp.c_str());
        throw std::runtime_error(std::string("state_save: writing ") + path + " failed");
    }
    return tot;
}

bool KvEngine::state_load(int seq, const char * path, const void * key, size_t key_len, int hend, void * const * extra, const size_t * extra_sizes,
                          int n_extra) {
    use_device();
    Seq & s = seq_ref(seq);
    need_whole(s, "state_load");
    if (!path || (key_len && !key) || n_extra < 0 || (n_extra && (!extra || !extra_sizes))) throw std::runtime_error("state_load: null argument");
    if (hend < 0 || hend > s.ctx) throw std::runtime_error("state_load: hend " + std::to_string(hend) + " does not fit the sequence's context");
    if (seq == SEQ_MAIN && sw_on_) throw std::runtime_error("state_load: a side request is active");
    FILE * f = fopen(path, "rb");
    if (!f) return false;
    auto R = state_regions(s, hend);
    for (int i = 0; i < n_extra; i++) R.push_back({static_cast<char *>(extra[i]), extra_sizes[i]});
    // the header must name this very state: key, hend, region count and every region's size, and the file must end with the
    // last region (state_files.cu:206-216); anything else is "no state file" and the caller rebuilds it
    bool ok = true;
    auto r64 = [&](uint64_t & v) { return fread(&v, 8, 1, f) == 1; };
    char magic[8];
    ok = fread(magic, 8, 1, f) == 1 && !memcmp(magic, STATE_MAGIC, 8);
    uint64_t kn = 0, h = 0, nr = 0, v = 0;
    ok = ok && r64(kn) && kn == key_len;
    if (ok && kn) {
        std::vector<char> kb(kn);
        ok = fread(kb.data(), 1, kn, f) == kn && !memcmp(kb.data(), key, kn);
    }
    ok = ok && r64(h) && h == (uint64_t) hend && r64(nr) && nr == R.size();
    unsigned long long tot = 0;
    for (size_t i = 0; ok && i < R.size(); i++) ok = r64(v) && v == R[i].second, tot += R[i].second;
    if (ok) {
        const long at = ftell(f);
        ok = at >= 0 && fseek(f, 0, SEEK_END) == 0 && (unsigned long long) ftell(f) == (unsigned long long) at + tot && fseek(f, at, SEEK_SET) == 0;
    }
    if (!ok) {
        fclose(f);
        return false;
    }
    PinnedPiece buf;
    if (!buf.p) {
        fclose(f);
        throw std::runtime_error("state_load: no pinned staging buffer");
    }
    reset(seq);
    wait_copies(s);
    MKKV_CK(cudaStreamSynchronize(stream_)); // (no earlier launch still reads the state, state_files.cu:217)
    try {
        for (const auto & r : R)
            for (size_t o = 0; o < r.second; o += STATE_PIECE) {
                const size_t n = std::min(STATE_PIECE, r.second - o);
                if (fread(buf.p, 1, n, f) != n) throw std::runtime_error(std::string("state_load: short read of ") + path);
                MKKV_CK(cudaMemcpy(r.first + o, buf.p, n, cudaMemcpyDefault));
            }
    } catch (...) {
        fclose(f);
        reset(seq); // (rows partly overwritten: the sequence is empty)
        throw;
    }
    fclose(f);
    s.n = hend;
    s.kv_top = hend; // (as a prefill of 0 .. hend - 1, state_files.cu:241)
    std::fill(s.spilled.begin(), s.spilled.end(), hend);
    return true;
}

int KvEngine::park_len(int id) const {
    const auto it = parked_.find(id);
    return it == parked_.end() ? -1 : it->second.n;
}

int KvEngine::park(int seq, int max_checkpoints, bool wait) {
    use_device();
    Seq & s = seq_ref(seq);
    need_whole(s, "park");
    if (s.n == 0) return 0;
    const auto t0 = std::chrono::steady_clock::now();
    // spill mode: every position of the sequence gets its main-format row first, so the entry is the reference's byte
    // stream (host_store.cu:243-265) and needs no fp16 shadow
    for (int l = 0; l < cfg_.layers; l++) spill_to(s, l, s.n);
    Parked e;
    e.n = s.n;
    e.kv_top = s.n;
    e.ctxp = s.ctxp;
    e.kv_bytes = stream_bytes(s, 0, s.n, 0, 0);
    e.ring_bytes = stream_bytes(s, 0, 0, 0, rc_);
    size_t need = e.kv_bytes + e.ring_bytes;
    std::vector<const Checkpoint *> keep;
    for (auto it = s.cks.rbegin(); it != s.cks.rend() && (int) keep.size() < max_checkpoints; ++it) keep.push_back(&*it);
    for (const Checkpoint * k : keep)
        if (k->ring_ok) need += ring_state_bytes();
    if (!blob_room(e.blob, need)) {
        hs_release(e.blob);
        return -1;
    }
    wait_copies(s);
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    MKKV_CK(cudaStreamWaitEvent(st_copy_, ev_compute_, 0));
    run_copy(s, 0, s.n, 0, rc_, e.blob, 0, true);
    MKKV_CK(cudaEventRecord(s.copy_done, st_copy_));
    s.copy_pending = true; // later launches on this sequence wait until the rows and rings are out
    e.blob.used = e.kv_bytes + e.ring_bytes;
    if (!keep.empty()) MKKV_CK(cudaStreamSynchronize(st_copy_)); // (a checkpoint's ring copy may still be in flight)
    for (const Checkpoint * k : keep) {
        Checkpoint c;
        c.pos = k->pos;
        c.ring_ok = k->ring_ok;
        e.cks.push_back(c);
        e.ck_off.push_back(e.blob.used);
        if (k->ring_ok) { // host item: memcpy over the chunk borders
            const size_t rb = ring_state_bytes();
            for (size_t done = 0; done < rb;) {
                const size_t bp = e.blob.used, ci = bp / hs_chunk_, co = bp % hs_chunk_, len = std::min(rb - done, hs_chunk_ - co);
                memcpy(e.blob.chunks[ci] + co, k->ring + done, len);
                done += len;
                e.blob.used += len;
            }
        }
    }
    copies_in_flight_ = true;
    if (wait) store_wait();
    const int id = park_next_++;
    hs_bytes_ = e.blob.used;
    hs_ms_ = ms_since(t0);
    parked_.emplace(id, std::move(e));
    return id;
}

bool KvEngine::unpark(int seq, int id, bool wait) {
    use_device();
    const auto it = parked_.find(id);
    if (it == parked_.end()) return false;
    Seq & s = seq_ref(seq);
    need_whole(s, "unpark");
    if (it->second.n > s.ctx) throw std::runtime_error("unpark: the parked conversation (" + std::to_string(it->second.n) + " positions) does not fit the sequence's context");
    if (seq == SEQ_MAIN && sw_on_) throw std::runtime_error("unpark: a side request is active (side_unpark continues a parked conversation inside it)");
    (void) wait;
    unpark_into(s, seq, id);
    return true;
}

// the sequence becomes parked entry id (which is freed): rows, rings, checkpoints (host_store.cu:457-483)
void KvEngine::unpark_into(Seq & s, int seq, int id) {
    const auto it = parked_.find(id);
    Parked & e = it->second;
    const auto t0 = std::chrono::steady_clock::now();
    reset(seq);
    // the side stream starts after the compute stream's pending work on this sequence
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    MKKV_CK(cudaStreamWaitEvent(st_copy_, ev_compute_, 0));
    run_copy(s, 0, e.n, 0, rc_, e.blob, 0, false);
    MKKV_CK(cudaEventRecord(s.copy_done, st_copy_));
    s.copy_pending = true;
    MKKV_CK(cudaStreamSynchronize(st_copy_)); // the chunks go back to the free list below
    for (size_t i = 0; i < e.cks.size(); i++) {
        Checkpoint c = e.cks[i];
        if (c.ring_ok) {
            const size_t rb = ring_state_bytes();
            MKKV_CK(cudaHostAlloc(reinterpret_cast<void **>(&c.ring), rb, cudaHostAllocDefault));
            size_t bp = e.ck_off[i];
            for (size_t done = 0; done < rb;) {
                const size_t ci = bp / hs_chunk_, co = bp % hs_chunk_, len = std::min(rb - done, hs_chunk_ - co);
                memcpy(c.ring + done, e.blob.chunks[ci] + co, len);
                done += len;
                bp += len;
            }
        }
        s.cks.push_back(c);
    }
    std::sort(s.cks.begin(), s.cks.end(), [](const Checkpoint & a, const Checkpoint & b) { return a.pos < b.pos; });
    s.n = e.n;
    s.kv_top = e.n;
    std::fill(s.spilled.begin(), s.spilled.end(), e.n);
    hs_bytes_ = e.blob.used;
    hs_release(e.blob);
    parked_.erase(it);
    hs_ms_ = ms_since(t0);
}

// Rows [0, P) of a parked conversation into the sequence, leaving the entry parked: the main rows of every region come
// straight from the pinned entry (one copy per region and chunk crossing), the window rings of the P positions are rebuilt
// from the main rows as a rewind does (ck_pool.cu:285-296 with every ring row stale).
bool KvEngine::restore_prefix(int seq, int id, int P, bool wait) {
    use_device();
    const auto it = parked_.find(id);
    if (it == parked_.end()) return false;
    Seq & s = seq_ref(seq);
    need_whole(s, "restore_prefix");
    const Parked & e = it->second;
    if (P < 0 || P > e.n || P > s.ctx) throw std::runtime_error("restore_prefix: position " + std::to_string(P) + " outside the parked conversation");
    const auto t0 = std::chrono::steady_clock::now();
    reset(seq);
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    MKKV_CK(cudaStreamWaitEvent(st_copy_, ev_compute_, 0));
    size_t off = 0, moved = 0;
    for (const auto & r : s.regions) {
        if (r.ring) break;
        const size_t want = (size_t) P * r.row_bytes;
        for (size_t done = 0; done < want;) {
            const size_t bp = off + done, ci = bp / hs_chunk_, co = bp % hs_chunk_, len = std::min(want - done, hs_chunk_ - co);
            MKKV_CK(cudaMemcpyAsync(r.base + done, e.blob.chunks[ci] + co, len, cudaMemcpyHostToDevice, st_copy_));
            done += len;
        }
        moved += want;
        off += (size_t) e.n * r.row_bytes;
    }
    if (cfg_.win > 0 && P > 0) MKKV_CK(launch_refill(s.d_views, cfg_.layers, std::max(0, P - rc_), P, st_copy_));
    MKKV_CK(cudaEventRecord(s.copy_done, st_copy_));
    s.copy_pending = true;
    copies_in_flight_ = true;
    s.n = P;
    s.kv_top = P;
    std::fill(s.spilled.begin(), s.spilled.end(), P);
    for (const auto & c : e.cks)
        if (c.pos <= P && !c.ring_ok) s.cks.push_back(c);
    if (wait) store_wait();
    hs_bytes_ = moved;
    hs_ms_ = ms_since(t0);
    return true;
}

bool KvEngine::park_drop(int id) {
    const auto it = parked_.find(id);
    if (it == parked_.end()) return false;
    use_device();
    MKKV_CK(cudaStreamSynchronize(st_copy_));
    hs_release(it->second.blob);
    parked_.erase(it);
    return true;
}

// ---- side request: the main sequence kept aside while a short unrelated one runs (host_store.cu:186-206,297-355) ----

bool KvEngine::side_begin() {
    use_device();
    if (sw_on_) throw std::runtime_error("side_begin: a side request is already active");
    if (hs_budget_ == 0) return false;
    Seq & s = main_;
    need_whole(s, "side_begin");
    for (int l = 0; l < cfg_.layers; l++) spill_to(s, l, s.n); // (the shadow rows will be overwritten: make the main rows now)
    sw_on_ = true;
    sw_broken_ = false;
    sw_n_ = s.n;
    sw_top_ = s.n;
    sw_hi_ = 0;
    sw_rings_saved_ = false;
    sw_spilled_ = s.spilled;
    sw_cks_ = std::move(s.cks);
    s.cks.clear();
    sw_pieces_.clear();
    sw_ms_ = 0;
    s.n = s.kv_top = 0;
    std::fill(s.spilled.begin(), s.spilled.end(), 0);
    return true;
}

// rows below X of the main buffers (and, once, the rings) are about to be overwritten by the side request: copy the kept
// sequence's rows [sw_hi, up) out first, 1024 rows at a time (host_store.cu:186-206)
void KvEngine::sw_need(int X) {
    if (!sw_on_ || sw_broken_) return;
    constexpr int SW_BLK = 1024;
    const int up = (X + MAXT + SW_BLK - 1) / SW_BLK * SW_BLK;
    const int want = std::max(sw_hi_, std::min(sw_top_, up));
    const bool rings = !sw_rings_saved_ && rc_ > 0;
    if (want <= sw_hi_ && !rings) return;
    const auto t0 = std::chrono::steady_clock::now();
    Seq & s = main_;
    const int ra = 0, rb = rings ? rc_ : 0;
    const size_t bytes = stream_bytes(s, sw_hi_, want, ra, rb);
    if (!blob_room(sw_blob_, bytes)) {
        sw_broken_ = true;
        fprintf(stderr, "[mk] side request: the host store is full at row %d: the kept sequence is dropped\n", X);
        return;
    }
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    MKKV_CK(cudaStreamWaitEvent(st_copy_, ev_compute_, 0));
    run_copy(s, sw_hi_, want, ra, rb, sw_blob_, sw_blob_.used, true);
    sw_pieces_.push_back({sw_hi_, want, rings, sw_blob_.used, bytes});
    sw_blob_.used += bytes;
    MKKV_CK(cudaStreamSynchronize(st_copy_)); // the launch that overwrites the rows comes next
    sw_hi_ = want;
    if (rings) sw_rings_saved_ = true;
    sw_ms_ += ms_since(t0);
}

int KvEngine::side_end() {
    use_device();
    if (!sw_on_) throw std::runtime_error("side_end: no side request");
    const auto t0 = std::chrono::steady_clock::now();
    Seq & s = main_;
    reset(SEQ_MAIN);
    if (sw_broken_) {
        side_drop();
        return 0;
    }
    MKKV_CK(cudaEventRecord(ev_compute_, stream_));
    MKKV_CK(cudaStreamWaitEvent(st_copy_, ev_compute_, 0));
    size_t moved = 0;
    for (const auto & p : sw_pieces_) {
        run_copy(s, p.a, p.b, 0, p.rings ? rc_ : 0, sw_blob_, p.off, false);
        moved += p.bytes;
    }
    MKKV_CK(cudaStreamSynchronize(st_copy_));
    s.n = sw_n_;
    s.kv_top = sw_top_;
    s.spilled = sw_spilled_;
    s.cks = std::move(sw_cks_);
    sw_cks_.clear();
    sw_on_ = false;
    sw_pieces_.clear();
    hs_bytes_ = moved;
    hs_release(sw_blob_);
    hs_ms_ = ms_since(t0);
    return 1;
}

// side_end with the side request's own conversation parked first (host_store.cu:371-396). *id: its entry, 0 when it is empty
// or the store has no room. 1: the kept sequence is back; 0: it was lost (the store ran full during the side request): the side
// request's conversation stays as the engine's sequence.
int KvEngine::side_end_park(int max_checkpoints, int * id) {
    use_device();
    if (!sw_on_) throw std::runtime_error("side_end_park: no side request");
    *id = 0;
    sw_park_bytes_ = 0;
    sw_park_ms_ = 0;
    const auto t0 = std::chrono::steady_clock::now();
    const int pid = park(SEQ_MAIN, max_checkpoints, true);
    if (pid > 0) {
        *id = pid;
        sw_park_bytes_ = park_bytes(pid);
        sw_park_ms_ = ms_since(t0);
    }
    if (sw_broken_) { // nothing to bring back: drop what was kept, leave the side request's conversation in place
        MKKV_CK(cudaStreamSynchronize(st_copy_));
        sw_on_ = false;
        sw_pieces_.clear();
        for (auto & k : sw_cks_)
            if (k.ring) cudaFreeHost(k.ring);
        sw_cks_.clear();
        hs_release(sw_blob_);
        return 0;
    }
    return side_end();
}

// Right after side_begin: the side request continues parked conversation id (the engine becomes it, the entry is freed) while
// the kept sequence stays aside: the rows and rings it overwrites go to the store first (host_store.cu:398-455).
// 1 done, 0 no room in the store (nothing changed), -1 no such entry.
int KvEngine::side_unpark(int id) {
    use_device();
    if (!sw_on_) throw std::runtime_error("side_unpark: no side request");
    const auto it = parked_.find(id);
    if (it == parked_.end()) return -1;
    Seq & s = main_;
    if (s.n != 0 || s.kv_top != 0) throw std::runtime_error("side_unpark: only right after side_begin");
    const int n = it->second.n;
    if (n > s.ctx) throw std::runtime_error("side_unpark: the parked conversation (" + std::to_string(n) + " positions) does not fit the context");
    if (sw_broken_) return 0;
    // the copy-out sw_need(n) would make, checked for room first so that a full store changes nothing
    constexpr int SW_BLK = 1024;
    const int up = (n + MAXT + SW_BLK - 1) / SW_BLK * SW_BLK, want = std::max(sw_hi_, std::min(sw_top_, up));
    const bool rings = !sw_rings_saved_ && rc_ > 0;
    if (!blob_room(sw_blob_, stream_bytes(s, sw_hi_, want, 0, rings ? rc_ : 0))) return 0;
    sw_need(n);
    if (sw_broken_) return 0;
    unpark_into(s, SEQ_MAIN, id);
    return 1;
}

void KvEngine::side_drop() {
    use_device();
    MKKV_CK(cudaStreamSynchronize(st_copy_));
    sw_on_ = false;
    sw_pieces_.clear();
    for (auto & k : sw_cks_)
        if (k.ring) cudaFreeHost(k.ring);
    sw_cks_.clear();
    hs_release(sw_blob_);
    reset(SEQ_MAIN);
}

// ---- test helpers ----

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

// Header of 8 words, then per (layer, side, kv head, position < n) the hash of its main row (values then scales), then per
// (layer, side, kv head, position in [ring_lo, n)) the hash of its ring row, 0 for a side without a ring (engine.cu:1438-1500).
// Words 2 and 7 of the reference's header describe state outside this path and are 0.
std::vector<unsigned long long> KvEngine::state_digest(int seq) {
    use_device();
    Seq & s = seq_ref(seq);
    need_whole(s, "state_digest");
    sync();
    typedef unsigned long long u64;
    const int n = s.n, rc = cfg_.win > 0 ? rc_ : 0, rlo = rc ? std::max(0, n - rc) : n;
    std::vector<u64> out = {0x4d4b444701ULL, (u64) n, 0, (u64) rc, (u64) rlo, (u64) cfg_.layers, (u64) NKV, 0};
    std::vector<unsigned char> vb, sb;
    auto d2h = [&](std::vector<unsigned char> & dst, const void * src, size_t nb) {
        dst.resize(std::max<size_t>(1, nb));
        if (nb) MKKV_CK(cudaMemcpy(dst.data(), src, nb, cudaMemcpyDeviceToHost));
    };
    for (int l = 0; l < cfg_.layers; l++)
        for (int w = 0; w < 2; w++)
            for (int g = 0; g < NKV; g++) {
                const KvSide & sd = s.views[l].s[w];
                const size_t rb = row_bytes(sd.bits);
                d2h(vb, sd.val + (size_t) g * s.ctxp * rb, n * rb);
                d2h(sb, sd.sc + (size_t) g * s.ctxp * 8, (size_t) n * SCALE_ROW);
                for (int p = 0; p < n; p++) out.push_back(dg_hash(sb.data() + (size_t) p * SCALE_ROW, SCALE_ROW, dg_hash(vb.data() + p * rb, rb)));
            }
    for (int l = 0; l < cfg_.layers; l++)
        for (int w = 0; w < 2; w++)
            for (int g = 0; g < NKV; g++) {
                const KvSide & sd = s.views[l].s[w];
                if (!rc || !sd.rval) {
                    out.insert(out.end(), n - rlo, 0ULL);
                    continue;
                }
                d2h(vb, sd.rval + (size_t) g * rc * HD, (size_t) rc * HD);
                d2h(sb, sd.rsc + (size_t) g * rc * 8, (size_t) rc * SCALE_ROW);
                for (int p = rlo; p < n; p++) {
                    const size_t r = p % rc;
                    out.push_back(dg_hash(sb.data() + r * SCALE_ROW, SCALE_ROW, dg_hash(vb.data() + r * HD, HD)));
                }
            }
    return out;
}

std::vector<unsigned long long> KvEngine::profile() {
    use_device();
    std::vector<unsigned long long> v;
    if (!prof_) return v;
    sync();
    v.resize(attend_fast_prof_words(num_sms_));
    MKKV_CK(cudaMemcpy(v.data(), prof_, v.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return v;
}

int KvEngine::read_row(int seq, int layer, int side, int g, int pos, bool ring, void * val, void * sc) {
    use_device();
    check_layer(layer);
    Seq & s = seq_ref(seq);
    if (side < 0 || side > 1 || g < 0 || g >= NKV) throw std::runtime_error("read_row: bad side / kv head");
    const KvSide & sd = s.views[layer].s[side];
    sync();
    if (ring) {
        if (!sd.rval || pos < 0 || pos >= rc_) throw std::runtime_error("read_row: no such ring row");
        MKKV_CK(cudaMemcpy(val, sd.rval + ((size_t) g * rc_ + pos) * HD, HD, cudaMemcpyDeviceToHost));
        MKKV_CK(cudaMemcpy(sc, sd.rsc + ((size_t) g * rc_ + pos) * 8, SCALE_ROW, cudaMemcpyDeviceToHost));
        return HD;
    }
    if (pos < s.base || pos - s.base >= s.ctxp) throw std::runtime_error("read_row: position out of range");
    const size_t rb = row_bytes(sd.bits), row = (size_t) g * s.ctxp + (pos - s.base);
    MKKV_CK(cudaMemcpy(val, sd.val + row * rb, rb, cudaMemcpyDeviceToHost));
    MKKV_CK(cudaMemcpy(sc, sd.sc + row * 8, SCALE_ROW, cudaMemcpyDeviceToHost));
    return (int) rb;
}

void KvEngine::write_row(int seq, int layer, int side, int g, int pos, bool ring, const void * val, const void * sc) {
    use_device();
    check_layer(layer);
    Seq & s = seq_ref(seq);
    if (side < 0 || side > 1 || g < 0 || g >= NKV) throw std::runtime_error("write_row: bad side / kv head");
    const KvSide & sd = s.views[layer].s[side];
    sync();
    if (ring) {
        if (!sd.rval || pos < 0 || pos >= rc_) throw std::runtime_error("write_row: no such ring row");
        MKKV_CK(cudaMemcpy(sd.rval + ((size_t) g * rc_ + pos) * HD, val, HD, cudaMemcpyHostToDevice));
        MKKV_CK(cudaMemcpy(sd.rsc + ((size_t) g * rc_ + pos) * 8, sc, SCALE_ROW, cudaMemcpyHostToDevice));
        return;
    }
    if (pos < s.base || pos - s.base >= s.ctxp) throw std::runtime_error("write_row: position out of range");
    const size_t rb = row_bytes(sd.bits), row = (size_t) g * s.ctxp + (pos - s.base);
    MKKV_CK(cudaMemcpy(sd.val + row * rb, val, rb, cudaMemcpyHostToDevice));
    MKKV_CK(cudaMemcpy(sd.sc + row * 8, sc, SCALE_ROW, cudaMemcpyHostToDevice));
    s.kv_top = std::max(s.kv_top, pos + 1);
}

} // namespace mkkv
