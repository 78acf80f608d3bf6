// extern "C" surface of the KV hot path (include/mk_kv.h). Conventions follow the reference's capi.cpp:201-263: exceptions
// become -1 with a thread-local message; a CUDA failure resets the engine first; a failed reset exits with code 4.
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../../include/mk_kv.h"
#include "kv_engine.h"

using mkkv::KvEngine;
using mkkv::MKCudaError;

namespace {
thread_local std::string g_err;

struct Handle {
    KvEngine * eng = nullptr;
};

[[noreturn]] void reset_failed(const char * why) {
    fprintf(stderr, "[mk] the reset after a CUDA error failed too (%s): exiting with code 4\n", why);
    fflush(stdout);
    fflush(stderr);
    std::_Exit(4);
}

template <class F> int guarded(void * hp, F f) {
    if (!hp) {
        g_err = "null handle";
        return -1;
    }
    auto * h = static_cast<Handle *>(hp);
    try {
        return f(h->eng);
    } catch (const MKCudaError & e) {
        g_err = e.what();
        try {
            h->eng->reset_all();
        } catch (const std::exception & e2) {
            reset_failed(e2.what());
        } catch (...) {
            reset_failed("unknown exception");
        }
        return -1;
    } catch (const std::exception & e) {
        g_err = e.what();
        return -1;
    } catch (...) {
        g_err = "unknown exception";
        return -1;
    }
}
template <class V> int copy_out(const V & v, int * out, int cap) {
    if (out)
        for (int i = 0; i < std::min((int) v.size(), cap); i++) out[i] = v[i];
    return (int) v.size();
}
} // namespace

extern "C" {

const char * mk_last_error(void) { return g_err.c_str(); }

unsigned long long mk_kv_abi_sig(void) {
    unsigned long long h = 0xcbf29ce484222325ULL;
    const unsigned long long w[] = {mkkv::NH, mkkv::NKV, mkkv::HD, mkkv::MAXT, mkkv::ATP, mkkv::ATT_NCH, mkkv::ATT_BUCKET, mkkv::KV_PAD,
                                    mkkv::MAX_LAYERS, sizeof(mkkv::KvView), sizeof(mkkv::AttnJob), 1 /* interface revision */};
    for (unsigned long long x : w) h = (h ^ x) * 0x100000001b3ULL;
    return h;
}

const char * mk_build_info(void) {
    static const std::string s = std::string("{\"commit\": \"unknown\", \"flags\": \"\", \"cuda\": \"") + std::to_string(CUDART_VERSION / 1000) + "." +
                                 std::to_string(CUDART_VERSION % 1000 / 10) + "\", \"arch\": \"sm_100a\"}";
    return s.c_str();
}

void * mk_kv_new(int layers, int ctx, const char * kv_spec, int kv_win, int flags) {
    try {
        mkkv::EngineConfig c;
        c.layers = layers;
        c.ctx = ctx;
        c.kv_spec = kv_spec ? kv_spec : "";
        c.win = kv_win;
        c.spill = (flags & MK_KV_SPILL) != 0;
        c.win_all = (flags & MK_KV_WIN_ALL) != 0;
        c.exact = (flags & MK_KV_EXACT) != 0;
        auto * h = new Handle;
        try {
            h->eng = new KvEngine(c);
        } catch (...) {
            delete h;
            throw;
        }
        return h;
    } catch (const std::exception & e) {
        g_err = e.what();
        return nullptr;
    }
}

void mk_free(void * hp) {
    if (!hp) return;
    auto * h = static_cast<Handle *>(hp);
    try {
        delete h->eng;
    } catch (...) {
    }
    delete h;
}

void mk_reset(void * hp) {
    guarded(hp, [](KvEngine * e) {
        e->sync();
        e->reset_all();
        return 0;
    });
}

int mk_kv_set_stream(void * hp, void * s) {
    return guarded(hp, [&](KvEngine * e) {
        e->set_stream(static_cast<cudaStream_t>(s));
        return 0;
    });
}
int mk_kv_sync(void * hp) {
    return guarded(hp, [](KvEngine * e) {
        e->sync();
        return 0;
    });
}

int mk_kv_wait_limits(unsigned hint_ns, unsigned rounds, unsigned polls) {
    if (hint_ns == 0 && rounds == 0 && polls == 0) mkkv::attend_tc_default_wait_limits();
    else mkkv::attend_tc_set_wait_limits(hint_ns, rounds, polls);
    return 0;
}
int mk_kv_wait_limits_expire_now(void) {
    mkkv::attend_tc_set_wait_limits(0u, 0u, 0u);
    return 0;
}

int mk_kv_append(void * hp, int seq, int layer, int pos0, int n, const void * K, const void * V) {
    return guarded(hp, [&](KvEngine * e) {
        e->append(seq, layer, pos0, n, K, V);
        return 0;
    });
}
int mk_kv_attend(void * hp, int seq, int layer, int n, int T, const void * Q, void * O) {
    return guarded(hp, [&](KvEngine * e) {
        e->attend(seq, layer, n, T, Q, O);
        return 0;
    });
}
int mk_kv_set_base(void * hp, int seq, int base) {
    return guarded(hp, [&](KvEngine * e) {
        e->set_base(seq, base);
        return 0;
    });
}
int mk_kv_attend_partial(void * hp, int seq, int layer, int n, int T, const void * Q, int pos_lo, int pos_hi, void * part_out, void * ml_out) {
    return guarded(hp, [&](KvEngine * e) {
        e->attend_partial(seq, layer, n, T, Q, pos_lo, pos_hi, part_out, ml_out);
        return 0;
    });
}
int mk_kv_combine(void * hp, int layer, int T, int nparts, const void * parts, const void * mls, void * O) {
    return guarded(hp, [&](KvEngine * e) {
        e->combine(layer, T, nparts, parts, mls, O);
        return 0;
    });
}
int mk_kv_step_layers_partial(void * hp, int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, size_t kv_stride,
                              size_t q_stride, int own_lo, int own_hi, int pos_lo, int pos_hi, void * parts, void * mls) {
    return guarded(hp, [&](KvEngine * e) {
        e->step_layers_partial(seq, nlayers, n, T, K, V, Q, kv_stride, q_stride, own_lo, own_hi, pos_lo, pos_hi, parts, mls);
        return 0;
    });
}
int mk_kv_combine_layers(void * hp, int nlayers, int T, int nparts, const void * parts, const void * mls, void * O, size_t o_stride) {
    return guarded(hp, [&](KvEngine * e) {
        e->combine_layers(nlayers, T, nparts, parts, mls, O, o_stride);
        return 0;
    });
}
int mk_kv_combine_layers_strided(void * hp, int nlayers, int T, int nparts, const void * parts, const void * mls, size_t rank_stride, void * O,
                                 size_t o_stride) {
    return guarded(hp, [&](KvEngine * e) {
        e->combine_layers(nlayers, T, nparts, parts, mls, O, o_stride, rank_stride);
        return 0;
    });
}
int mk_kv_attend_static(void * hp, int seq, int layer, int n, int T, const void * Q, void * O) {
    return guarded(hp, [&](KvEngine * e) {
        e->attend_static(seq, layer, n, T, Q, O);
        return 0;
    });
}
int mk_kv_step(void * hp, int seq, int layer, int n, int T, const void * K, const void * V, const void * Q, void * O) {
    return guarded(hp, [&](KvEngine * e) {
        e->step_layers(seq, 1, n, T, K, V, Q, O, 0, 0, 0, layer); // (one append launch that also stages the queries, then the attention)
        return 0;
    });
}
int mk_kv_step_layers(void * hp, int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, void * O,
                      size_t kv_stride, size_t q_stride, size_t o_stride) {
    return guarded(hp, [&](KvEngine * e) {
        e->step_layers(seq, nlayers, n, T, K, V, Q, O, kv_stride, q_stride, o_stride);
        return 0;
    });
}
int mk_kv_step_layers_at(void * hp, int seq, int layer0, int nlayers, int n, int T, const void * K, const void * V, const void * Q, void * O,
                         size_t kv_stride, size_t q_stride, size_t o_stride) {
    return guarded(hp, [&](KvEngine * e) {
        e->step_layers(seq, nlayers, n, T, K, V, Q, O, kv_stride, q_stride, o_stride, layer0);
        return 0;
    });
}
int mk_kv_reserve_batch(void * hp, int njobs) {
    return guarded(hp, [&](KvEngine * e) {
        e->reserve_batch(njobs);
        return 0;
    });
}
int mk_kv_step_batch(void * hp, int njobs, const int * seqs, int layer, const int * n, const int * T, const void * K, const void * V,
                     const void * Q, void * O) {
    return guarded(hp, [&](KvEngine * e) {
        e->step_batch(njobs, seqs, layer, n, T, K, V, Q, O, true);
        return 0;
    });
}
int mk_kv_attend_batch(void * hp, int njobs, const int * seqs, int layer, const int * n, const int * T, const void * Q, void * O) {
    return guarded(hp, [&](KvEngine * e) {
        e->step_batch(njobs, seqs, layer, n, T, nullptr, nullptr, Q, O, false);
        return 0;
    });
}
int mk_kv_commit(void * hp, int seq, int len) {
    return guarded(hp, [&](KvEngine * e) {
        e->commit(seq, len);
        return 0;
    });
}
int mk_kv_position(void * hp, int seq) {
    return guarded(hp, [&](KvEngine * e) { return e->position(seq); });
}
int mk_kv_cap_T(int n, int T_req) { return mkkv::att_cap_T(n, T_req); }

int mk_kv_truncate(void * hp, int seq, int len) {
    return guarded(hp, [&](KvEngine * e) {
        e->truncate(seq, len);
        return 0;
    });
}
int mk_truncate(void * hp, int len) { return mk_kv_truncate(hp, MK_SEQ_MAIN, len); }
int mk_kv_checkpoint(void * hp, int seq) {
    return guarded(hp, [&](KvEngine * e) { return e->checkpoint(seq); });
}
int mk_kv_checkpoints(void * hp, int seq, int * out, int cap) {
    return guarded(hp, [&](KvEngine * e) { return copy_out(e->checkpoints(seq), out, cap); });
}
int mk_checkpoints(void * hp, int * out, int cap) { return mk_kv_checkpoints(hp, MK_SEQ_MAIN, out, cap); }
int mk_kv_rewind_to(void * hp, int seq, int pos) {
    return guarded(hp, [&](KvEngine * e) { return e->rewind_to(seq, pos) ? 0 : -1; });
}
int mk_rewind_to(void * hp, int pos) { return mk_kv_rewind_to(hp, MK_SEQ_MAIN, pos); }
int mk_rewind_to_checkpoint(void * hp) {
    return guarded(hp, [](KvEngine * e) { return e->rewind_to_checkpoint(mkkv::SEQ_MAIN) ? 0 : -1; });
}

int mk_store_budget(void * hp, long long bytes) {
    return guarded(hp, [&](KvEngine * e) {
        e->store_budget((size_t) std::max(bytes, 0LL));
        return 0;
    });
}
int mk_store_reserve(void * hp, long long bytes) {
    return guarded(hp, [&](KvEngine * e) {
        e->store_reserve((size_t) std::max(bytes, 0LL));
        return 0;
    });
}
int mk_store_info(void * hp, long long * out, int cap) {
    return guarded(hp, [&](KvEngine * e) {
        const KvEngine::StoreInfo s = e->store_info();
        size_t pt, rings, state, ck;
        e->kv_sizes(&pt, &rings, &state, &ck);
        const long long v[] = {(long long) s.budget, (long long) s.allocated, (long long) s.used, s.parked, (long long) s.last_bytes,
                               (long long) (s.last_ms * 1000.0), (long long) (s.side_ms * 1000.0), (long long) pt,
                               (long long) s.side_park_bytes, (long long) (s.side_park_ms * 1000.0)};
        const int n = std::min(cap, (int) (sizeof v / sizeof v[0]));
        for (int i = 0; i < n; i++) out[i] = v[i];
        return n;
    });
}
void mk_kv_sizes(void * hp, long long * per_token, long long * rings, long long * state, long long * checkpoint) {
    guarded(hp, [&](KvEngine * e) {
        size_t a, b, c, d;
        e->kv_sizes(&a, &b, &c, &d);
        *per_token = (long long) a;
        *rings = (long long) b;
        *state = (long long) c;
        *checkpoint = (long long) d;
        return 0;
    });
}
int mk_kv_park(void * hp, int seq, int max_checkpoints) {
    return guarded(hp, [&](KvEngine * e) {
        const int id = e->park(seq, max_checkpoints);
        return id < 0 ? -3 : id;
    });
}
long long mk_kv_state_save(void * hp, int seq, const char * path, const void * key, size_t key_len, int hend, const void * const * extra,
                           const size_t * extra_sizes, int n_extra) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        r = e->state_save(seq, path, key, key_len, hend, extra, extra_sizes, n_extra);
        return 0;
    });
    return r;
}
int mk_kv_state_load(void * hp, int seq, const char * path, const void * key, size_t key_len, int hend, void * const * extra,
                     const size_t * extra_sizes, int n_extra) {
    return guarded(hp, [&](KvEngine * e) { return e->state_load(seq, path, key, key_len, hend, extra, extra_sizes, n_extra) ? 1 : 0; });
}
int mk_park(void * hp, int max_checkpoints) { return mk_kv_park(hp, MK_SEQ_MAIN, max_checkpoints); }
int mk_kv_unpark(void * hp, int seq, int id) {
    return guarded(hp, [&](KvEngine * e) {
        if (e->unpark(seq, id)) return 0;
        g_err = "no parked conversation " + std::to_string(id);
        return -1;
    });
}
int mk_unpark(void * hp, int id) { return mk_kv_unpark(hp, MK_SEQ_MAIN, id); }
int mk_park_drop(void * hp, int id) {
    return guarded(hp, [&](KvEngine * e) { return e->park_drop(id) ? 0 : -1; });
}
long long mk_park_need(void * hp, int max_checkpoints) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        r = (long long) e->park_need(MK_SEQ_MAIN, max_checkpoints);
        return 0;
    });
    return r;
}
long long mk_park_bytes(void * hp, int id) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        r = (long long) e->park_bytes(id);
        return 0;
    });
    return r;
}
int mk_kv_restore_prefix(void * hp, int seq, int id, int pos, int wait) {
    return guarded(hp, [&](KvEngine * e) {
        if (e->restore_prefix(seq, id, pos, wait != 0)) return 0;
        g_err = "no parked conversation " + std::to_string(id);
        return -1;
    });
}
int mk_kv_store_wait(void * hp) {
    return guarded(hp, [](KvEngine * e) {
        e->store_wait();
        return 0;
    });
}
int mk_side_begin(void * hp) {
    return guarded(hp, [](KvEngine * e) { return e->side_begin() ? 0 : 1; });
}
int mk_side_end(void * hp) {
    return guarded(hp, [](KvEngine * e) { return e->side_end(); });
}
int mk_side_end_park(void * hp, int max_checkpoints, int * id) {
    if (!id) {
        g_err = "mk_side_end_park: null id";
        return -1;
    }
    *id = 0;
    return guarded(hp, [&](KvEngine * e) { return e->side_end_park(max_checkpoints, id); });
}
int mk_side_unpark(void * hp, int id) {
    return guarded(hp, [&](KvEngine * e) {
        const int r = e->side_unpark(id);
        if (r < 0) g_err = "no parked conversation " + std::to_string(id);
        return r < 0 ? -1 : r == 1 ? 0 : 1;
    });
}
int mk_side_drop(void * hp) {
    return guarded(hp, [](KvEngine * e) {
        e->side_drop();
        return 0;
    });
}
int mk_side_active(void * hp) { return hp && static_cast<Handle *>(hp)->eng->side_active() ? 1 : 0; }

int mk_slots_open(void * hp, int n, int ctx) {
    return guarded(hp, [&](KvEngine * e) { return e->slots_open(n, ctx); });
}
int mk_slots_open2(void * hp, int n, int ctx, int seg_tokens) {
    (void) seg_tokens; // the reference's prefill segment length: this path has no token-level prefill
    return mk_slots_open(hp, n, ctx);
}
int mk_slots_count(void * hp) {
    return guarded(hp, [](KvEngine * e) { return e->slots_count(); });
}

long long mk_kv_state_digest(void * hp, int seq, unsigned long long * out, long long cap) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        const auto v = e->state_digest(seq);
        if (out)
            for (long long i = 0; i < std::min<long long>((long long) v.size(), cap); i++) out[i] = v[i];
        r = (long long) v.size();
        return 0;
    });
    return r;
}
int mk_state_digest(void * hp, unsigned long long * out, int cap) {
    const long long r = mk_kv_state_digest(hp, MK_SEQ_MAIN, out, cap);
    return r > INT_MAX ? INT_MAX : (int) r;
}
int mk_kv_read_row(void * hp, int seq, int layer, int side, int g, int pos, int ring, void * val, void * sc) {
    return guarded(hp, [&](KvEngine * e) { return e->read_row(seq, layer, side, g, pos, ring != 0, val, sc); });
}
int mk_kv_write_row(void * hp, int seq, int layer, int side, int g, int pos, int ring, const void * val, const void * sc) {
    return guarded(hp, [&](KvEngine * e) {
        e->write_row(seq, layer, side, g, pos, ring != 0, val, sc);
        return 0;
    });
}
int mk_kv_unpack_probe(void * hp, int bits, const void * rows, const void * scales, int nrows, void * out) {
    return guarded(hp, [&](KvEngine * e) {
        e->unpack_probe(bits, rows, scales, nrows, out);
        return 0;
    });
}
int mk_kv_bits(void * hp, int side, int layer) {
    return guarded(hp, [&](KvEngine * e) {
        if (side < 0 || side > 1 || layer < 0 || layer >= e->config().layers) throw std::runtime_error("mk_kv_bits: out of range");
        return e->bits(side, layer);
    });
}
int mk_kv_has_ring(void * hp, int side, int layer) {
    return guarded(hp, [&](KvEngine * e) {
        if (side < 0 || side > 1 || layer < 0 || layer >= e->config().layers) throw std::runtime_error("mk_kv_has_ring: out of range");
        return e->has_ring(side, layer) ? 1 : 0;
    });
}
int mk_kv_ring_rows(void * hp) {
    return guarded(hp, [](KvEngine * e) { return e->ring_rows(); });
}
long long mk_kv_profile(void * hp, unsigned long long * out, long long cap) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        const auto v = e->profile();
        if (out)
            for (long long i = 0; i < std::min<long long>((long long) v.size(), cap); i++) out[i] = v[i];
        r = (long long) v.size();
        return 0;
    });
    return r;
}
long long mk_kv_launches(void * hp) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        r = e->launches();
        return 0;
    });
    return r;
}
long long mk_kv_device_bytes(void * hp) {
    long long r = -1;
    guarded(hp, [&](KvEngine * e) {
        r = (long long) e->device_bytes();
        return 0;
    });
    return r;
}

} // extern "C"
