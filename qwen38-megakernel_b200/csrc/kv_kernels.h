// Host-callable launchers of the KV hot-path kernels (sm_100a). Every launcher enqueues on `stream` and returns the
// launch's cudaError_t; none allocates or synchronises.
#pragma once
#include <cuda_runtime.h>

#include <vector>

#include "kv_format.h"

namespace mkkv {

// error word values a kernel may leave in the engine's mapped status word
enum KernelStatus : int { KS_OK = 0, KS_WAIT_TIMEOUT = 1 };

// rows pos0 .. pos0 + n - 1 of one (sequence, layer): K, V fp16 [n][4][256] -> ring q8 row (+ fp16 shadow) and, in eager
// mode or for a side without a ring, the main-format row
cudaError_t launch_append(const KvView & kv, const uint16_t * K, const uint16_t * V, int pos0, int n, cudaStream_t stream);
// spill mode: main-format rows of positions [p0, p1) of the layers' ring sides, quantized from the fp16 shadow.
// views: device array of KvView, one per layer
cudaError_t launch_spill(const KvView * views, int layers, int p0, int p1, cudaStream_t stream);
// ring rows of positions [p0, p1) rebuilt from the main rows (after a rewind), all layers of one sequence
cudaError_t launch_refill(const KvView * views, int layers, int p0, int p1, cudaStream_t stream);

// the merge alone: job j's partials are slots item0 + g nch .. + nch - 1 of kv head g (grouped: .. + ceil(nch / cpi) - 1, as the
// tensor-core kernel's batch mode leaves them)
// raw_part / raw_ml (one job only): write the merged but un-normalised result as one partial per kv head, [4][48][256] floats and
// [4][48] (m, l), instead of the job's O
cudaError_t launch_merge(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int max_T, float * part, float2 * ml,
                         cudaStream_t stream, float * raw_part = nullptr, float2 * raw_ml = nullptr, bool grouped = false);
// mma.sync path (kv_attend_fast.cu). One job: cooperative launch over num_sms CTAs with an
// exchange of row maxima through xmax ([4][20][nbmax][48] 8-byte words {epoch, value}, zeroed once; epoch must be non-zero and
// differ from every earlier launch's). Several jobs: one CTA per (job, kv head, chunk). part / ml hold part_slots partials.
// cudaErrorNotSupported: shape not handled (one job spread over the grid only: the one-CTA-per-item mode takes every shape).
cudaError_t launch_attend_fast(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int total_items, int max_T, int num_sms,
                               float * part, float2 * ml, int part_slots, unsigned long long * xmax, int nbmax, int epoch, int * status,
                               unsigned long long * prof, bool spread, cudaStream_t stream, const AttnTask * tasks_dev = nullptr,
                               int ntasks = 0, int tasks_B = 0, float * raw_part = nullptr, float2 * raw_ml = nullptr);
// A job restricted to positions [pos_lo, pos_hi) (one sequence split over GPUs): its task list for launch_attend_fast, batch-major;
// returns the most batches any chunk has. tasks_dev must hold the same list on the device; raw_part / raw_ml receive the job's
// merged, un-normalised (m, l, O) as one partial per kv head ([4][48][256], [4][48]).
int build_range_tasks(const AttnJob & J, int B, std::vector<AttnTask> & out);
size_t attend_fast_smem_bytes();
// prof (optional, null: off): globaltimer stamps of the first batches of every CTA, [CTA][16][20] words: 0 batch start,
// 1 K tile arrived, 2 scores done, 3 / 4 before / after the batch barrier, 5 incoming max known, 6 running maxima done,
// 7 barrier, 11 P written (score warp 0); 8 / 9 / 10 batch start, first P tile arrived, batch done (first P V warp)
size_t attend_fast_prof_words(int ctas);

// Tensor-core path (kv_attend_tc.cu, tcgen05 + tensor memory): one job spread over num_sms CTAs in a cooperative launch, then the
// merge. xa / xb: exchange arrays of [4][20][nbmax][48] 8-byte words each, zeroed once; epoch as for launch_attend_fast. A host-built
// task list must use 4 tiles per batch (build_range_tasks with B = 4). cudaErrorNotSupported: shape not handled.
// done (device, [4], zeroed once) + done_seq (host counter of launches that used it): the merge runs in the kernel's tail instead of
// a second launch (not when raw_part is given).
cudaError_t launch_attend_tc(const AttnJob & job, int num_sms, float * part, float2 * ml, int part_slots, unsigned long long * xa,
                             unsigned long long * xb, int nbmax, int epoch, int * status, cudaStream_t stream,
                             const AttnTask * tasks_dev = nullptr, int ntasks = 0, int tasks_B = 0, float * raw_part = nullptr,
                             float2 * raw_ml = nullptr, unsigned long long * prof = nullptr, unsigned * done = nullptr,
                             unsigned * done_seq = nullptr);
// batch mode of the same kernel: one CTA per (job, kv head, run of AttnJob::cpi chunks), plain launch, then the merge kernel
cudaError_t launch_attend_tc_batch(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, int total_items, int max_T, float * part,
                                   float2 * ml, int part_slots, int * status, cudaStream_t stream);
size_t attend_tc_smem_bytes();
// test probe: the tensor-core kernel's unpack step on nrows packed rows -> fp16 operand values [nrows][256] in natural dim order
cudaError_t launch_unpack_probe(int bits, const uint8_t * rows, const uint16_t * sc, int nrows, uint16_t * out, cudaStream_t stream);
// load every kernel of the library on the current device (no launch allocates afterwards); the engine calls it at construction
cudaError_t preload_kernels();
cudaError_t preload_attend_fast();
cudaError_t preload_attend_tc();
// Wait limits of the tensor-core kernel's launches that follow (process-wide; for diagnostics and the failure-path test): a failed
// mbarrier try suspends for up to hint_ns, `rounds` failed tries or `polls` failed polls of an exchange word make a CTA give up.
void attend_tc_set_wait_limits(unsigned hint_ns, unsigned rounds, unsigned polls);
void attend_tc_default_wait_limits();

// batched append: job j writes n rows at pos0 of its own (sequence, layer)
struct AppendJob {
    KvView kv;
    const uint16_t * K;
    const uint16_t * V;
    int pos0, n;
};
cudaError_t launch_append_batch(const AppendJob * jobs_dev, int njobs, int max_n, cudaStream_t stream);
// Queries staged for the tensor-core attention kernel (qwen38_mk.cu:2876-2883: fp16 -> fp32 -> K's rotation -> x 1/16 -> fp16), once
// per (job, kv head) instead of once per CTA: QP_HEAD_BYTES bytes per kv head in that kernel's B-operand layout
// [dim group 32][row group 6][8 rows][8 dims in the unpacked units' order], rows beyond 6 T zero. One bulk copy brings a head's block
// into shared memory.
constexpr int QP_HEAD_BYTES = AR * HD * 2;
cudaError_t launch_qprep(const AttnJob * jobs_dev, const AttnJob * jobs_host, int njobs, cudaStream_t stream);
// rows pos0 .. pos0 + n - 1 of layers 0 .. nlayers - 1 of one sequence in one launch (views_dev: the sequence's device array of views);
// Q != null: the same launch stages the T query tokens of every layer (Q + l q_stride bytes -> qp + l * 4 * QP_HEAD_BYTES bytes)
cudaError_t launch_append_layers(const KvView * views_dev, int nlayers, const uint16_t * K, const uint16_t * V, size_t kv_stride, int pos0, int n,
                                 cudaStream_t stream, const uint16_t * Q = nullptr, size_t q_stride = 0, uint16_t * qp = nullptr, int T = 0);

// Snapshot gather / restore scatter between the cache regions of one sequence and a contiguous staging buffer.
// The snapshot byte stream is, region after region, rows [a, b) of every main region and ring rows [ra, rb) of every ring
// region (host_store.cu:77-107 order: layer, side, kv head: values, scales; then the rings). This launch moves stream bytes
// [off, off + len) to / from staging[0 .. len). Row sizes are multiples of 16 bytes, so are off and len.
struct CopyRegion {
    uint8_t * base;     // first row of the region (one kv head's values or scales, main or ring)
    unsigned row_bytes; // bytes per row
    unsigned ring;      // 1: indexed by ring row, 0: by position
};
constexpr int MAX_REGIONS = MAX_LAYERS * 2 * NKV * 2 * 2;
cudaError_t launch_gather(const CopyRegion * regions, int nregions, int a, int b, int ra, int rb, unsigned long long off,
                          unsigned long long len, uint8_t * staging, bool scatter, cudaStream_t stream);


// Decode attention of ONE job whose split partials live in a fixed array inside the library's device image instead of
// memory obtained from the CUDA allocator. The array holds STATIC_ITEMS (kv head, chunk) items: enough for any single
// job (the partition never makes more than NKV * ATT_NCH), about 3.96 MB per GPU that loads the library, held until the
// process exits. The array's device address is looked up (cudaGetSymbolAddress) by preload_kernels, which every engine runs at
// construction. Returns cudaErrorInvalidValue if the job needs more items than the array holds.
constexpr int STATIC_ITEMS = NKV * ATT_NCH;
cudaError_t launch_attend_static(const AttnJob & job, int * status, cudaStream_t stream);

} // namespace mkkv
