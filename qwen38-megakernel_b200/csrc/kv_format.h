// KV-cache geometry, formats and the per-(sequence, layer) device view shared by host code and kernels.
//
// Layout (kept from the reference so snapshots and digests are byte-compatible):
//   main values  [kv head][ctx + 16][32 * bits] bytes, main scales [kv head][ctx + 16][8] fp16   (mk_shared.cuh:385-393)
//   ring values  [kv head][ring rows][256] int8,       ring scales [kv head][ring rows][8] fp16  (mk_shared.cuh:396-403)
// A run of positions of one kv head is contiguous in every buffer, so a tile of any number of rows is one bulk copy.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define MKKV_HD __host__ __device__ __forceinline__
#else
#define MKKV_HD inline
#endif

namespace mkkv {

constexpr int NH = 24, NKV = 4, HD = 256, GQ = NH / NKV; // query heads, kv heads, head dim, GQA group (mk_shared.cuh:215)
constexpr int MAXT = 8;                                  // most query tokens per call (mk_shared.cuh:221)
constexpr int AR = GQ * MAXT;                            // query rows per kv head (mk_shared.cuh:257)
constexpr int ATP = 32;                                  // positions per tile: the unit of the online softmax (mk_shared.cuh:263)
constexpr int ATT_NCH = 20, ATT_BUCKET = 640;            // split-K chunks per kv head, partition / window granularity (:264-265)
constexpr int KV_PAD = 16;                               // rows past the usable context (mk_shared.cuh:247)
constexpr int MAX_LAYERS = 17;                           // attention layers of the model + the MTP block (mk_shared.cuh:251)
constexpr int SCALE_ROW = 16;                            // bytes of one row's 8 fp16 block scales

MKKV_HD int row_bytes(int bits) { return 32 * bits; }

// window start for context length L: positions >= ws are read from the q8 ring (qwen38_mk.cu:2122-2126)
MKKV_HD int kv_ws(int L, int win) {
    if (win <= 0) return 0;
    const int ws = (L + ATT_BUCKET - 1) / ATT_BUCKET - 1 - (win + ATT_BUCKET - 1) / ATT_BUCKET;
    return ws > 0 ? ws * ATT_BUCKET : 0;
}
// ring rows per kv head for window win (loader.cu:1479-1486)
MKKV_HD int kv_ring_rows(int win) { return win > 0 ? ((win + ATT_BUCKET - 1) / ATT_BUCKET + 1) * ATT_BUCKET + ATP : 0; }
// split-K partition of L positions: a function of L's 640-bucket only (qwen38_mk.cu:2548-2551)
MKKV_HD void attn_dims(int L, int & nch, int & cs) {
    const int b = (L + ATT_BUCKET - 1) / ATT_BUCKET;
    cs = ATP * (b > 1 ? b : 1);
    const int n = (L + cs - 1) / cs;
    nch = n > 1 ? n : 1;
}
// largest T <= T_req whose rows n .. n + T - 1 share one partition (mk_shared.cuh:288-291)
MKKV_HD int att_cap_T(int n, int T_req) {
    const int lim = ATT_BUCKET * ((n + ATT_BUCKET) / ATT_BUCKET) - n;
    return T_req < lim ? T_req : lim;
}

// one side (K or V) of one layer of one sequence
struct KvSide {
    uint8_t * val;     // main values
    uint16_t * sc;     // main scales (fp16 bits)
    uint8_t * rval;    // ring values, or null (8-bit side without a window)
    uint16_t * rsc;    // ring scales
    uint16_t * shadow; // spill mode: fp16 copy of the ring's source rows [kv head][ring rows][256], else null
    int bits;          // 4 .. 8
    int rot;           // stored Hadamard-rotated
};
struct KvView {
    KvSide s[2]; // K, V
    int ctxp;    // rows per kv head in the main buffers (ctx + KV_PAD)
    int rc;      // ring rows per kv head (0: no window)
    int win;     // MK_KV_WIN
    int eager;   // 1: every appended row is also stored in its main format at once (the reference's state);
                 // 0: main rows are written when a position leaves the window (spill from the fp16 shadow)
    int base;    // position of main-buffer row 0 (0 unless the sequence is split by position over several GPUs); ring rows
                 // are always indexed by the global position
};

// one decode-attention job: T query tokens at positions n .. n + T - 1 of one (sequence, layer)
struct AttnJob {
    KvView kv;
    const uint16_t * Q; // fp16 [T][24][256], post-norm / post-RoPE, unscaled
    const uint16_t * Qp; // the same queries staged for the tensor-core kernel by qprep (kv_kernels.h): per kv head the 48 rows
                         // (head % 6) T + t, rotated when K is, x 1/16, fp16, in the operand layout; null: not staged
    float * O;          // fp32 [T][24][256]
    int n, T;
    int nch, cs, ws;    // partition and window start of L = n + T
    int item0;          // first (kv head, chunk) item of this job in the call's partial buffers
    int cpi, titem0;    // the tensor-core kernel's batch mode: a CTA runs cpi consecutive chunks of a kv head (short chunks are not
                        // worth a CTA each), so a head has ceil(nch / cpi) partials, in slots item0 + g nch + 0 ..; titem0: the job's
                        // first CTA in that grid. cpi <= 1: one chunk per CTA
    int pos_lo, pos_hi; // only positions in [pos_lo, pos_hi) are attended (multiples of 32 or the context end; whole context: 0, n + T)
    int pstride;        // merge: partial c of kv head g is slot item0 + g nch + c (pstride 1), else item0 + c pstride + g
    long long rstride;  // merge, pstride > 1 only: floats between partial c and c + 1 of both arrays when they are not pstride
                        // slots apart (each GPU's arrays packed into one exchange buffer); 0: pstride slots
};

// one batch of tiles of one chunk, as the fast attention kernel runs it (built on the host for position-range jobs)
struct AttnTask {
    int c, b, nb; // chunk, batch, batches of the chunk
    int pos0;     // position of the batch's first tile
    int c1;       // end of the chunk (clipped to the job's range)
    int nt;       // tiles of the batch
};

} // namespace mkkv
