// KvEngine: the host side of the KV-cache hot path on one GPU -- cache ownership per sequence, MK_KV / MK_KV_WIN formats,
// append / attend launches, spill bookkeeping, ring rewind, checkpoints, the pinned host store (park / unpark / side
// requests) and the state digest. It mirrors the KV-relevant part of the reference's MKEngine (qwen38_mk.h:37-267) at
// tensor level: K / V / Q rows come in as device pointers instead of being computed from tokens.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "kv_format.h"
#include "kv_kernels.h"

namespace mkkv {

// a failed (non-sticky) CUDA call: the sequence state is undefined, the C API resets the engine (qwen38_mk.h:9-14)
struct MKCudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

[[noreturn]] void cuda_fail(cudaError_t e, const char * what, const char * file, int line);
#define MKKV_CK(x)                                                   \
    do {                                                             \
        cudaError_t e_ = (x);                                        \
        if (e_ != cudaSuccess) ::mkkv::cuda_fail(e_, #x, __FILE__, __LINE__); \
    } while (0)

constexpr int SEQ_MAIN = -1; // the engine's own sequence; parallel slots are 0 .. slots_count() - 1

struct EngineConfig {
    int layers = 16;
    int ctx = 4096;
    std::string kv_spec; // MK_KV grammar (loader.cu:1329-1366); empty: q8_0 everywhere
    int win = 0;         // MK_KV_WIN
    bool win_all = false; // MK_KV_WIN_ALL: rings for the 8-bit sides too (test knob, loader.cu:1487-1490)
    bool spill = false;   // main-format rows are written when a position leaves the window (fp16 shadow), not at append
    bool exact = false;   // MK_EXACT: checkpoints keep a copy of the window rings
};

struct Checkpoint {
    int pos = -1;
    char * ring = nullptr; // exact mode: pinned copy of every ring as of pos
    bool ring_ok = false;
};

// pinned host memory in chunks, entries laid end to end over chunks (host_store.cu:5-75)
struct Blob {
    std::vector<char *> chunks;
    size_t used = 0;
};

class KvEngine {
  public:
    explicit KvEngine(const EngineConfig & cfg);
    ~KvEngine();
    KvEngine(const KvEngine &) = delete;
    KvEngine & operator=(const KvEngine &) = delete;

    const EngineConfig & config() const { return cfg_; }
    int device() const { return dev_; }
    void set_stream(cudaStream_t s) { stream_ = s; }
    cudaStream_t stream() const { return stream_; }
    void sync(); // waits for all work of this engine and checks the kernels' status word

    // ---- sequences ----
    int slots_open(int n, int ctx); // n parallel sequences of ctx positions each (lanes.cu:291-326); returns ctx
    int slots_count() const { return (int) slots_.size(); }
    void reset(int seq);
    void reset_all();
    int position(int seq) const;
    int kv_top(int seq) const;
    void commit(int seq, int len); // the sequence is positions 0 .. len - 1 from now on (rows up to kv_top stay written)

    // ---- the hot path ----
    void append(int seq, int layer, int pos0, int n, const void * K, const void * V);
    void attend(int seq, int layer, int n, int T, const void * Q, void * O);
    // ---- one sequence split by position over several GPUs ----
    // This engine's copy of the sequence holds positions [base, base + ctx) (set while the sequence is empty; base a multiple of 32).
    void set_base(int seq, int base);
    // Attention of the T tokens at n over positions [pos_lo, pos_hi) only (inside this engine's rows; pos_lo a multiple of 32).
    // part_out [4][48][256] fp32, ml_out [4][48] (m, l): the un-normalised result per kv head, row (head % 6) T + t.
    void attend_partial(int seq, int layer, int n, int T, const void * Q, int pos_lo, int pos_hi, void * part_out, void * ml_out);
    // Merge of nparts such partials laid one after another (e.g. after an all-gather): O fp32 [T][24][256], normalised, rotated
    // back when the layer's V is stored rotated.
    void combine(int layer, int T, int nparts, const void * parts, const void * mls, void * O);
    // the same for every layer of one decode step in one call each (one collective per step between them)
    void step_layers_partial(int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, size_t kv_stride, size_t q_stride,
                             int own_lo, int own_hi, int pos_lo, int pos_hi, void * parts, void * mls);
    void combine_layers(int nlayers, int T, int nparts, const void * parts, const void * mls, void * O, size_t o_stride, size_t rank_stride = 0);
    // attend() with the split partials in the library's fixed device array: this call allocates nothing
    void attend_static(int seq, int layer, int n, int T, const void * Q, void * O);
    // one launch sequence for several sequences: job j appends T[j] rows at n[j] and attends; packed device buffers in job order
    void step_batch(int njobs, const int * seqs, int layer, const int * n, const int * T, const void * K, const void * V, const void * Q,
                    void * O, bool do_append);
    void reserve_batch(int njobs);

    // ---- rewind ----
    void truncate(int seq, int len);      // engine.cu:1233-1241
    int checkpoint(int seq);              // saves a checkpoint at the committed position; returns it
    std::vector<int> checkpoints(int seq) const;
    bool rewind_to(int seq, int pos);     // engine.cu:1197-1204, ck_pool.cu:268-296
    bool rewind_to_checkpoint(int seq);   // to the last checkpoint; false: none

    // ---- host store ----
    void store_budget(size_t bytes);
    void store_reserve(size_t bytes);
    struct StoreInfo {
        size_t budget = 0, allocated = 0, used = 0;
        int parked = 0;
        double last_ms = 0;
        size_t last_bytes = 0;
        double side_ms = 0;
        size_t side_park_bytes = 0; // the last side_end_park: its park of the side request's conversation (0: not parked)
        double side_park_ms = 0;
    };
    StoreInfo store_info() const;
    void kv_sizes(size_t * per_token, size_t * rings, size_t * state, size_t * checkpoint) const;
    // The reference's prompt-state file (state_files.cu:97-238) of rows 0 .. hend - 1, the rings and the caller's extra regions
    // (device or host pointers). save: the file's size; load: true when the file exists and matches key, hend and every region size.
    // one decode step over layers 0 .. nlayers - 1: one append launch for every layer's T rows at n, then the layers' attention
    void step_layers(int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, void * O, size_t kv_stride, size_t q_stride,
                     size_t o_stride, int layer0 = 0);
    void unpack_probe(int bits, const void * rows, const void * scales, int nrows, void * out); // (test probe of the unpack step)
    long long state_save(int seq, const char * path, const void * key, size_t key_len, int hend, const void * const * extra,
                         const size_t * extra_sizes, int n_extra);
    bool state_load(int seq, const char * path, const void * key, size_t key_len, int hend, void * const * extra, const size_t * extra_sizes,
                    int n_extra);
    int park(int seq, int max_checkpoints, bool wait = true); // id > 0; 0: empty sequence; -1: no room
    bool unpark(int seq, int id, bool wait = true);
    bool restore_prefix(int seq, int id, int P, bool wait = true); // rows [0, P) of a parked entry; rings refilled; entry kept
    bool park_drop(int id);
    size_t park_need(int seq, int max_checkpoints) const;
    size_t park_bytes(int id) const;
    int park_len(int id) const;
    void store_wait(); // completion of the copies enqueued by park / unpark / restore_prefix with wait = false
    bool side_begin();
    int side_end();
    int side_end_park(int max_checkpoints, int * id); // host_store.cu:371-396
    int side_unpark(int id);                          // host_store.cu:398-455
    void side_drop();
    bool side_active() const { return sw_on_; }

    // ---- test helpers ----
    std::vector<unsigned long long> state_digest(int seq); // engine.cu:1438-1500, KV words only
    // row bytes to host: ring = false: main row of position pos; ring = true: ring row index pos. Returns the value bytes.
    int read_row(int seq, int layer, int side, int g, int pos, bool ring, void * val, void * sc);
    void write_row(int seq, int layer, int side, int g, int pos, bool ring, const void * val, const void * sc);
    int ring_rows() const { return rc_; }
    int bits(int side, int layer) const { return kvb_[side][layer]; }
    bool has_ring(int side, int layer) const { return ring_[side][layer]; }
    size_t device_bytes() const { return dev_bytes_; }
    std::vector<unsigned long long> profile(); // MK_KV_PROFILE=1: the stamps of the last fast attention launch (else empty)
    long long launches() const { return launches_; } // kernels launched so far (every launcher call counts its kernels)

  private:
    struct Seq {
        int ctx = 0, ctxp = 0;
        uint8_t * val[2] = {nullptr, nullptr};
        uint16_t * sc[2] = {nullptr, nullptr};
        uint8_t * ring_val = nullptr;
        uint16_t * ring_sc = nullptr;
        uint16_t * shadow = nullptr;
        std::vector<KvView> views; // per layer
        KvView * d_views = nullptr;
        std::vector<CopyRegion> regions; // snapshot stream order
        CopyRegion * d_regions = nullptr;
        int n = 0, kv_top = 0, base = 0;
        std::vector<int> spilled; // per layer: main rows of ring sides exist for positions < spilled
        std::vector<Checkpoint> cks;
        cudaEvent_t copy_done = nullptr; // set while side-stream copies of this sequence are in flight
        bool copy_pending = false;
        bool failed = false;
    };
    struct Parked {
        Blob blob;
        int n = 0, kv_top = 0, ctxp = 0;
        size_t kv_bytes = 0, ring_bytes = 0;
        std::vector<Checkpoint> cks; // ring copies live inside the blob after the rings (host items)
        std::vector<size_t> ck_off;
    };

    void init_device_state(); // the constructor's device part
    void release();           // everything the engine owns (the destructor; the constructor when it fails part-way)
    Seq & seq_ref(int seq);
    const Seq & seq_ref(int seq) const;
    void alloc_seq(Seq & s, int ctx);
    void free_seq(Seq & s);
    void use_device() const;
    void check_layer(int layer) const;
    void need_whole(const Seq & s, const char * what) const;
    AttnJob whole_job(const Seq & s, const char * what, int layer, int n, int T, const void * Q, void * O) const;
    void unpark_into(Seq & s, int seq, int id);
    void ensure_qprep(int slots);
    void staged_q(AttnJob & j, int slot, bool staged); // j.Qp = the slot; staged false: filled by a launch of its own (true: the step's
                                                       // append launch has just done it)
    void attend_impl(int seq, int layer, int n, int T, const void * Q, void * O, bool q_staged);
    void attend_partial_impl(int seq, int layer, int n, int T, const void * Q, int pos_lo, int pos_hi, void * part_out, void * ml_out, bool q_staged);
    std::vector<std::pair<char *, size_t>> state_regions(Seq & s, int hend) const;
    void spill_to(Seq & s, int layer, int upto);
    void ring_rewind(Seq & s, int P);
    void drop_checkpoints(Seq & s, int after);
    void wait_copies(Seq & s); // the compute stream waits for side-stream copies touching s
    size_t stream_bytes(const Seq & s, int a, int b, int ra, int rb) const;
    // stream bytes of rows [a, b) + ring rows [ra, rb) of s <-> blob bytes [blob_off, ..) through the staging buffer
    void run_copy(Seq & s, int a, int b, int ra, int rb, Blob & blob, size_t blob_off, bool to_host);
    char * hs_take();
    char * hs_new();
    void hs_release(Blob & b);
    void hs_trim();
    bool blob_room(Blob & b, size_t bytes);
    size_t hs_used() const;
    size_t ring_state_bytes() const;
    void ensure_work(int items, int njobs);
    void ensure_staging();

    EngineConfig cfg_;
    int dev_ = 0;
    cudaStream_t stream_ = nullptr, st_copy_ = nullptr;
    cudaEvent_t ev_compute_ = nullptr, ev_copy_ = nullptr;
    int kvb_[2][MAX_LAYERS], rot_[2][MAX_LAYERS];
    bool ring_[2][MAX_LAYERS];
    int rc_ = 0;
    Seq main_;
    std::vector<Seq> slots_;
    size_t dev_bytes_ = 0;
    long long launches_ = 0;

    // attention workspace
    float * part_ = nullptr;
    float2 * ml_ = nullptr;
    int work_items_ = 0;
    AttnJob * d_jobs_ = nullptr;
    AttnJob * h_jobs_ = nullptr; // pinned
    void * d_ajobs_ = nullptr;   // batched append jobs
    void * h_ajobs_ = nullptr;
    int work_jobs_ = 0;
    AttnTask * d_tasks_ = nullptr; // task list of a position-range job
    AttnTask * h_tasks_ = nullptr; // pinned
    int tasks_cap_ = 0;
    long long tasks_key_[5] = {-1, -1, -1, -1, -1}; // (partition, range, tiles per task) of the list d_tasks_ holds
    int tasks_n_ = -1;
    int * h_status_ = nullptr; // mapped pinned word the kernels write
    int * d_status_ = nullptr;
    // fast attention path: exchange of row maxima between the CTAs of one chunk
    unsigned long long * xmax_ = nullptr;
    int epoch_ = 0, num_sms_ = 0;
    bool use_tc_ = true;
    int xnb_ = 0; // batches per chunk the exchange arrays hold
    uint16_t * qprep_ = nullptr;   // staged queries of the tensor-core kernel: [slot][4][QP_HEAD_BYTES]; slot = layer, or the job of a batch
    int qprep_slots_ = 0;
    unsigned * tc_done_ = nullptr; // fused merge of the tensor-core kernel: per kv head, CTAs done over all launches
    unsigned tc_done_seq_ = 0;     // launches that counted on it
    void ensure_xch(int nb);
    unsigned long long * prof_ = nullptr; // MK_KV_PROFILE=1: phase stamps of the last fast attention launch
    void launch_attention(const AttnJob * jobs_host, int njobs, int items, int max_T);

    // host store
    size_t hs_chunk_ = (size_t) 32 << 20, hs_budget_ = 0, hs_alloc_ = 0;
    std::vector<char *> hs_free_;
    std::map<int, Parked> parked_;
    int park_next_ = 1;
    double hs_ms_ = 0;
    size_t hs_bytes_ = 0;
    uint8_t * staging_ = nullptr; // device, 2 x hs_chunk_
    bool copies_in_flight_ = false;

    // side request: the main sequence kept aside
    bool sw_on_ = false, sw_broken_ = false;
    Blob sw_blob_;
    int sw_n_ = 0, sw_top_ = 0, sw_hi_ = 0;
    std::vector<int> sw_spilled_;
    std::vector<Checkpoint> sw_cks_;
    struct SwPiece { int a, b; bool rings; size_t off, bytes; };
    std::vector<SwPiece> sw_pieces_;
    bool sw_rings_saved_ = false;
    double sw_ms_ = 0, sw_park_ms_ = 0;
    size_t sw_park_bytes_ = 0;
    void sw_need(int X);
};

} // namespace mkkv
