/* mk_kv.h -- C ABI of the B200 KV-cache hot path (libmk_kv.so).
 *
 * Drop-in boundary for the KV path of the reference engine. The reference's own exported API (capi.cpp:261-802) is
 * token-level; its KV path is reached through the engine object. This header keeps the reference's names, return codes,
 * ownership and threading rules for every KV-relevant call it exports, and adds the tensor-level calls (mk_kv_*) that
 * the reference performs inside its decode cycle. Each declaration cites what it replaces (paths relative to the
 * reference project root).
 *
 * Conventions (capi.cpp:201-263):
 *   - every call catches all C++ exceptions: it returns -1 (or NULL) and the message is read with mk_last_error(), which is
 *     thread-local;
 *   - a failed CUDA call resets the engine before -1 is returned; a sticky CUDA error ends the process with exit code 4;
 *   - the caller owns every out-buffer and passes its capacity; out = NULL, cap = 0 returns the needed count;
 *   - one engine thread per handle; a handle binds to the CUDA device current at mk_kv_new;
 *   - K, V, Q, O are DEVICE pointers unless a parameter says "host"; no call allocates on behalf of the caller.
 *
 * Sequences: seq = MK_SEQ_MAIN (-1) is the engine's own sequence; 0 .. n-1 are the parallel slots opened by mk_slots_open.
 * Shapes: 24 query heads, 4 kv heads, head dimension 256 (mk_shared.cuh:215); at most 8 query tokens per call.
 */
#ifndef MK_KV_H
#define MK_KV_H

#ifdef __cplusplus
extern "C" {
#endif

#define MK_SEQ_MAIN (-1)
/* mk_kv_new flags */
#define MK_KV_SPILL 1   /* main-format rows are written when a position leaves the q8_0 window (fp16 shadow of the ring), not at append */
#define MK_KV_WIN_ALL 2 /* rings for the 8-bit sides too: MK_KV_WIN_ALL test knob, loader.cu:1487-1490 */
#define MK_KV_EXACT 4   /* checkpoints keep a copy of the window rings: MK_EXACT, ck_pool.cu:135-158 */

/* capi.cpp:263 */
const char * mk_last_error(void);
/* ABI check for bindings: a hash of the shapes and struct sizes this build uses (mk_shared.cuh:582-593 mk_abi_sig) */
unsigned long long mk_kv_abi_sig(void);
/* capi.cpp:787-800 */
const char * mk_build_info(void);

/* Replaces mk_new / mk_new2 (capi.cpp:266-312) for the KV path: instead of a model file, the shapes and the reference's
 * MK_KV / MK_KV_WIN settings (loader.cu:1329-1366, 1478-1503). layers: attention layers (1 .. 17); ctx: positions per
 * sequence; kv_spec: e.g. "K*=5r,V*=6" (NULL / "": q8_0); kv_win: e.g. 2048 (0: no window). NULL on error. */
void * mk_kv_new(int layers, int ctx, const char * kv_spec, int kv_win, int flags);
/* capi.cpp:418-424 */
void mk_free(void * h);
/* capi.cpp:564-569: clears every sequence (an error is only visible through mk_last_error) */
void mk_reset(void * h);
/* All later launches go to this cudaStream_t (default: the legacy default stream, as the reference: engine_impl.h:327) */
int mk_kv_set_stream(void * h, void * cuda_stream);
/* Waits for the engine's streams; -1 if a kernel reported a wait that ran out (the engine is reset), the reference's error-word
 * convention (mk_shared.cuh:170-203, capi.cpp:219-244) */
int mk_kv_sync(void * h);
/* Every device-side wait of the decode-attention kernel is bounded: a failed try of a shared-memory barrier suspends the thread for
 * up to hint_ns, after `rounds` failed tries (or `polls` failed reads of another CTA's exchange word) the CTA gives up: it sets the
 * status word mk_kv_sync reports, stops waiting, lets its copies in flight land, frees its tensor memory and returns. These calls
 * set the limits for the launches that follow, process-wide (defaults: 10,000 ns, 200,000, 2,097,152: about two seconds;
 * (0, 0, 0) restores them). mk_kv_wait_limits_expire_now makes the first wait that does not succeed at once give up: the
 * failure-path test uses it (nothing traps or hangs: the kernel returns with a wrong result the host rejects). The limits are the
 * tensor-core kernel's; the mma.sync kernel (MK_KV_ATTN=fast, and the fallback of the batched and no-allocation calls) has one
 * compiled-in limit of 8,388,608 tries per wait (seconds) and no early expiry: it does not wait for copies in flight before it
 * returns, which is safe only because no copy is still in flight after seconds. */
int mk_kv_wait_limits(unsigned hint_ns, unsigned rounds, unsigned polls);
int mk_kv_wait_limits_expire_now(void);

/* ---- the hot path ---- */
/* The reference's K / V row jobs (qwen38_mk.cu:2892-2926) and pk_attn_prep's store part (prefill.cuh:984-1023):
 * rows pos0 .. pos0 + n - 1 of one layer from fp16 K, V [n][4][256] (post-norm, post-RoPE). Rows at or past the committed
 * length may be rewritten. 0 / -1 */
int mk_kv_append(void * h, int seq, int layer, int pos0, int n, const void * K, const void * V);
/* attn_core + attn_combine (qwen38_mk.cu:4555-4690) without the model's gate: T query tokens at positions n .. n + T - 1
 * (their rows already appended), causal among the T. Q fp16 [T][24][256] (post-norm, post-RoPE, unscaled), O fp32
 * [T][24][256]. 0 / -1 */
int mk_kv_attend(void * h, int seq, int layer, int n, int T, const void * Q, void * O);
/* No counterpart in the reference. mk_kv_attend for callers that must not touch the CUDA allocator while they decode: a
 * plugin inside a server that has already handed every byte of device memory to its own pool (a cudaMalloc there fails or
 * stalls the whole device), or a real-time loop that may not take the allocator's locks and implicit synchronisation.
 * Same arguments, same result. The split-K partials go to a fixed array compiled into the library (3.96 MB on every GPU
 * that loads it, until the process exits) instead of the engine's allocated workspace; the call runs no cudaMalloc /
 * cudaFree or any other allocating routine. Limits: one sequence per call, T <= 8, at most 80 (kv head, chunk) items; a call
 * beyond that returns -1 with a message saying so. The array's device address is looked up when an engine is created on the device
 * (mk_kv_new), not in this call. All handles of a process share the one array per GPU, and it keeps the last
 * call's contents (nothing in it needs clearing: each call writes every partial it reads): two such calls that can
 * overlap on the GPU (different streams or handles) race and must be serialised by the caller. 0 / -1 */
int mk_kv_attend_static(void * h, int seq, int layer, int n, int T, const void * Q, void * O);
/* ---- one very long sequence split by position over several GPUs (no counterpart in the reference, which is single-GPU: its
 * split-K partials (qwen38_mk.cu:3048-3064) and merge (:4658-4669) are the unit that is exchanged) ----
 * mk_kv_set_base: this handle's copy of sequence seq holds positions [base, base + ctx) (empty sequence; base a multiple of 32).
 * mk_kv_attend_partial: the T tokens at n over positions [pos_lo, pos_hi) only, inside this handle's rows, with the reference's
 * chunk partition of the WHOLE context n + T; writes the un-normalised result per kv head: part_out fp32 [4][48][256] (row
 * (head % 6) T + t), ml_out fp32 [4][48][2] = (max, sum). Every rank passes the same Q.
 * mk_kv_combine: merges nparts such results laid one after another (as an all-gather leaves them) into O fp32 [T][24][256]. */
int mk_kv_set_base(void * h, int seq, int base);
int mk_kv_attend_partial(void * h, int seq, int layer, int n, int T, const void * Q, int pos_lo, int pos_hi, void * part_out, void * ml_out);
int mk_kv_combine(void * h, int layer, int T, int nparts, const void * parts, const void * mls, void * O);
/* The two calls above for every layer of one decode step, so that the ranks exchange once per step instead of once per layer:
 * mk_kv_step_layers_partial: layer l appends those of the T rows at n that fall into [own_lo, own_hi) (K, V + l kv_stride bytes, the
 * step's T rows) and attends with Q + l q_stride over [pos_lo, min(pos_hi, n + T)); its partial goes to parts + l * 4 * 48 * 256
 * floats and mls + l * 4 * 48 * 2 floats. mk_kv_combine_layers: parts [nparts][nlayers][4][48][256] and mls [nparts][nlayers][4][48][2]
 * (the ranks' arrays gathered in rank order) -> O + l o_stride bytes, every layer in one launch. */
int mk_kv_step_layers_partial(void * h, int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, size_t kv_stride,
                              size_t q_stride, int own_lo, int own_hi, int pos_lo, int pos_hi, void * parts, void * mls);
int mk_kv_combine_layers(void * h, int nlayers, int T, int nparts, const void * parts, const void * mls, void * O, size_t o_stride);
/* The same merge when every rank sends ONE buffer holding its parts array and its mls array (one all-gather per decode step): rank p's
 * arrays start p * rank_stride bytes after parts and after mls (rank_stride a multiple of 8). */
int mk_kv_combine_layers_strided(void * h, int nlayers, int T, int nparts, const void * parts, const void * mls, size_t rank_stride, void * O,
                                 size_t o_stride);
/* append + attend of one decode step's layer, as the reference's attention phase does in one pass */
int mk_kv_step(void * h, int seq, int layer, int n, int T, const void * K, const void * V, const void * Q, void * O);
/* One decode step over layers 0 .. nlayers - 1 in one call: layer l appends T rows at n from K + l kv_stride, V + l kv_stride
 * and attends with Q + l q_stride into O + l o_stride (strides in bytes). What the reference's forward pass does between its
 * layers' attention phases (engine.cu:1353-1413) with the host out of the loop; equal in result to nlayers calls of mk_kv_step (the
 * rows of all layers are appended by one launch before the first layer's attention: every K and V must be complete at the call). */
int mk_kv_step_layers(void * h, int seq, int nlayers, int n, int T, const void * K, const void * V, const void * Q, void * O,
                      size_t kv_stride, size_t q_stride, size_t o_stride);
/* The same for layers layer0 .. layer0 + nlayers - 1 (K, V, Q, O point at layer0's rows): a host that receives a step's rows in
 * blocks of layers overlaps the next block's copies with this block's attention. */
int mk_kv_step_layers_at(void * h, int seq, int layer0, int nlayers, int n, int T, const void * K, const void * V, const void * Q, void * O,
                         size_t kv_stride, size_t q_stride, size_t o_stride);
/* lanes_step (lanes.cu:452-560): one pass over several sequences; job j runs T[j] tokens at n[j] of sequence seqs[j].
 * K, V [sum T][4][256], Q [sum T][24][256], O [sum T][24][256] packed in job order. seqs, n, T are host arrays.
 * mk_kv_reserve_batch(njobs) must have been called once with at least this many jobs. */
int mk_kv_reserve_batch(void * h, int njobs);
int mk_kv_step_batch(void * h, int njobs, const int * seqs, int layer, const int * n, const int * T, const void * K, const void * V,
                     const void * Q, void * O);
int mk_kv_attend_batch(void * h, int njobs, const int * seqs, int layer, const int * n, const int * T, const void * Q, void * O);
/* The step's accepted count (engine.cu:1353-1413): the sequence is positions 0 .. len - 1 from now on */
int mk_kv_commit(void * h, int seq, int len);
int mk_kv_position(void * h, int seq);
/* att_cap_T (mk_shared.cuh:288-291): the most tokens a call at position n may carry so its rows share one partition */
int mk_kv_cap_T(int n, int T_req);

/* ---- rewind (main sequence: the reference's names; any sequence: the mk_kv_ forms) ---- */
/* capi.cpp:571-576 */
int mk_truncate(void * h, int len);
int mk_kv_truncate(void * h, int seq, int len);
/* Saves a checkpoint at the committed position (the reference saves them during a prefill: qwen38_mk.h:57-64); returns the position */
int mk_kv_checkpoint(void * h, int seq);
/* capi.cpp:593-599 */
int mk_checkpoints(void * h, int * out, int cap);
int mk_kv_checkpoints(void * h, int seq, int * out, int cap);
/* capi.cpp:600-603: 0, or -1 (no checkpoint there) */
int mk_rewind_to(void * h, int pos);
/* capi.cpp:590-592: to the last checkpoint; 0, or -1 (none) */
int mk_rewind_to_checkpoint(void * h);
int mk_kv_rewind_to(void * h, int seq, int pos);

/* ---- conversation state in pinned host memory (capi.cpp:644-741) ---- */
int mk_store_budget(void * h, long long bytes);
int mk_store_reserve(void * h, long long bytes);
/* capi.cpp:659-673. out[0..9]: budget, allocated, used bytes, parked entries, last copy's bytes and microseconds, side request's
 * copy-out microseconds, bytes per KV token, the last mk_side_end_park's park of the side request's conversation: bytes and
 * microseconds */
int mk_store_info(void * h, long long * out, int cap);
void mk_kv_sizes(void * h, long long * per_token, long long * rings, long long * state, long long * checkpoint);
/* The reference's prompt-state file for the KV regions (state_files.cu:97-238; the reference reaches it through MK_STATE inside its
 * generate call, engine.cu:1078-1130, and has no export for it): "MKSTATE1", u64 key length, key, u64 hend, u64 region count, u64
 * size of each region, then the regions: for every layer, side, kv head the values of rows 0 .. hend - 1 and their scales; for every
 * (layer, side) with a ring all heads' ring values, then all heads' ring scales; then n_extra caller regions (the reference appends
 * its recurrent-state buffers dstate, conv, h_hist there; device or host pointers). key is the caller's identity string of the state
 * (state_files.cu:44-95 builds it from the model file, the KV layout, the environment and the token prefix).
 * mk_kv_state_save: hend must equal the rows written; written to path + ".tmp<pid>" and renamed. Returns the file's size, -1 on error.
 * mk_kv_state_load: 1 = restored (the sequence then holds hend committed positions), 0 = no file or it does not match key, hend
 * or a region size (the caller recomputes and saves again), -1 error. */
long long mk_kv_state_save(void * h, int seq, const char * path, const void * key, size_t key_len, int hend, const void * const * extra,
                           const size_t * extra_sizes, int n_extra);
int mk_kv_state_load(void * h, int seq, const char * path, const void * key, size_t key_len, int hend, void * const * extra,
                     const size_t * extra_sizes, int n_extra);
/* id > 0, 0 (empty sequence), -3 (no room in the store), -1 error */
int mk_park(void * h, int max_checkpoints);
int mk_kv_park(void * h, int seq, int max_checkpoints);
/* 0, or -1 (no such entry / error) */
int mk_unpark(void * h, int id);
int mk_kv_unpark(void * h, int seq, int id);
int mk_park_drop(void * h, int id);
long long mk_park_need(void * h, int max_checkpoints);
long long mk_park_bytes(void * h, int id);
/* Rows [0, pos) of parked entry id become the sequence (the entry stays parked); the window rings of those positions are
 * rebuilt from the main rows exactly as mk_unpark followed by mk_rewind_to(pos) without a ring snapshot leaves them
 * (host_store.cu:457-483, ck_pool.cu:285-296). wait = 0 returns once the copies are enqueued on the side stream; later
 * launches on the sequence wait for them on the GPU, mk_kv_store_wait waits on the host. 0 / -1 */
int mk_kv_restore_prefix(void * h, int seq, int id, int pos, int wait);
int mk_kv_store_wait(void * h);
/* capi.cpp:683-711 */
int mk_side_begin(void * h);
int mk_side_end(void * h);
/* capi.cpp:696-700: mk_side_end with the side request's own conversation parked first (*id: its entry, 0: not parked). 1 the kept
 * sequence is back; 0 it was lost, the side request's conversation stays the engine's sequence; -1 error */
int mk_side_end_park(void * h, int max_checkpoints, int * id);
/* capi.cpp:702-707: right after mk_side_begin, the side request continues parked conversation id (the entry is freed; the kept
 * sequence stays aside). 0 done, 1 no room in the store (nothing changed), -1 no such entry / error */
int mk_side_unpark(void * h, int id);
int mk_side_drop(void * h);
int mk_side_active(void * h);

/* ---- parallel slots (capi.cpp mk_slots_open; lanes.cu:291-326): n sequences of ctx positions each; returns ctx ---- */
int mk_slots_open(void * h, int n, int ctx);
/* capi.cpp:318-326: the same with the reference's prefill segment length, which this path (no token-level prefill) ignores */
int mk_slots_open2(void * h, int n, int ctx, int seg_tokens);
int mk_slots_count(void * h);

/* ---- test helpers ---- */
/* capi.cpp:635-642 (state_digest, engine.cu:1438-1500: KV words) */
int mk_state_digest(void * h, unsigned long long * out, int cap);
long long mk_kv_state_digest(void * h, int seq, unsigned long long * out, long long cap);
/* One row's bytes to HOST buffers: ring = 0 the main row of position pos (32 * bits value bytes), ring = 1 ring row pos
 * (256 bytes); sc receives the 8 fp16 scales. Returns the value bytes, -1 on error */
int mk_kv_read_row(void * h, int seq, int layer, int side, int kv_head, int pos, int ring, void * val, void * sc);
int mk_kv_write_row(void * h, int seq, int layer, int side, int kv_head, int pos, int ring, const void * val, const void * sc);
/* format facts: bits of a side (0 K, 1 V) of a layer, 1 if it has a ring, ring rows per kv head, device bytes held */
/* Diagnostic, no counterpart in the reference: the operand values the tensor-core attention kernel's unpack step makes of nrows packed
 * rows of `bits` bits (device pointers: rows [nrows][32 bits] bytes, scales [nrows][8] fp16) -> out [nrows][256] fp16 in natural dim
 * order; they are fp16(d * q) of qwen38_mk.cu:2335-2343,2457-2468, which the parity tests check bit for bit. */
int mk_kv_unpack_probe(void * h, int bits, const void * rows, const void * scales, int nrows, void * out);
int mk_kv_bits(void * h, int side, int layer);
int mk_kv_has_ring(void * h, int side, int layer);
int mk_kv_ring_rows(void * h);
long long mk_kv_device_bytes(void * h);
/* Tracing, as the reference's -DMK_PROFILE barrier stamps (qwen38_mk.cu:143, engine.cu:377-560): with MK_KV_PROFILE=1 in the
 * environment at mk_kv_new, the decode-attention kernel records globaltimer stamps per phase for the first 16 batches of every
 * CTA; this copies the last launch's stamps ([CTA][16][20] words, nanoseconds) and returns the word count (0: off) */
long long mk_kv_profile(void * h, unsigned long long * out, long long cap);
/* kernels this engine has launched so far (append, spill, refill, attention split and merge) */
long long mk_kv_launches(void * h);

#ifdef __cplusplus
}
#endif
#endif
