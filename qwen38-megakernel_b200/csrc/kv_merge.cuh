// The merge of the partials of one (query head, token), shared by attn_merge_kernel and the tail of the tensor-core kernel.
#pragma once
#include <math_constants.h>

#include "kv_format.h"
#include "kv_quant.cuh"

namespace mkkv {

// y = sum_c w_c O_c / sum_c w_c l_c, w_c = exp(m_c - max m), then the inverse rotation when V is stored rotated
// (qwen38_mk.cu:4658-4685). One warp per row; lane holds dims 8 lane .. 8 lane + 7. The row's partials are slots i0, i0 + cstep, ..
// (count of them, at most 64) of part [slot][48][256] / ml [slot][48], row r = (head % 6) T + t.
// raw != 0: write the merged but un-normalised (m, l, O) of the row instead, as one partial per kv head (slot g of part_out /
// ml_out): the input of a later merge across GPUs
// pstep / mstep: floats / (m, l) pairs between consecutive partials of the row in part / ml.
// merge_accumulate: the weighted sums over partials first, first + step, .. < count of row r (lane: dims 8 lane .. + 7), with the
// weights taken against the maximum M over ALL count partials; merge_finish: the row's output from complete sums.
__device__ __forceinline__ void merge_accumulate(const float * part, const float2 * ml, size_t i0, size_t pstep, size_t mstep, int count, int first,
                                                 int step, int r, int lane, float (&num)[8], float & den, float & M) {
    // lane c (and c + 32) holds partial c's (m, l): all weights first, so the sums below run over independent loads
    float2 mla = lane < count ? __ldcg(&ml[i0 * AR + r + lane * mstep]) : make_float2(-CUDART_INF_F, 0.f);
    float2 mlb = lane + 32 < count ? __ldcg(&ml[i0 * AR + r + (lane + 32) * mstep]) : make_float2(-CUDART_INF_F, 0.f);
    M = fmaxf(mla.x, mlb.x);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) M = fmaxf(M, __shfl_xor_sync(FULL, M, m));
    const float wa = mla.x == -CUDART_INF_F ? 0.f : expf(mla.x - M), wb = mlb.x == -CUDART_INF_F ? 0.f : expf(mlb.x - M);
    den = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) num[k] = 0.f;
    const float * pbase = part + (i0 * AR + r) * HD + lane * 8;
#pragma unroll 4
    for (int c = first; c < count; c += step) {
        const float w = __shfl_sync(FULL, c < 32 ? wa : wb, c & 31), lc = __shfl_sync(FULL, c < 32 ? mla.y : mlb.y, c & 31);
        const float4 * o = reinterpret_cast<const float4 *>(pbase + (size_t) c * pstep);
        const float4 o0 = __ldcg(o), o1 = __ldcg(o + 1);
        num[0] = __fmaf_rn(w, o0.x, num[0]);
        num[1] = __fmaf_rn(w, o0.y, num[1]);
        num[2] = __fmaf_rn(w, o0.z, num[2]);
        num[3] = __fmaf_rn(w, o0.w, num[3]);
        num[4] = __fmaf_rn(w, o1.x, num[4]);
        num[5] = __fmaf_rn(w, o1.y, num[5]);
        num[6] = __fmaf_rn(w, o1.z, num[6]);
        num[7] = __fmaf_rn(w, o1.w, num[7]);
        den = __fmaf_rn(w, lc, den);
    }
}
__device__ __forceinline__ void merge_finish(const AttnJob & J, int h, int t, int lane, int raw, float * part_out, float2 * ml_out, const float (&num)[8],
                                             float den, float M) {
    const int g = h / GQ, r = (h % GQ) * J.T + t;
    if (raw) {
        float4 * dst = reinterpret_cast<float4 *>(part_out + ((size_t) g * AR + r) * HD + lane * 8);
        dst[0] = make_float4(num[0], num[1], num[2], num[3]);
        dst[1] = make_float4(num[4], num[5], num[6], num[7]);
        if (lane == 0) ml_out[(size_t) g * AR + r] = make_float2(M, den);
        return;
    }
    float y[8];
#pragma unroll
    for (int k = 0; k < 8; k++) y[k] = __fdiv_rn(num[k], den);
    if (J.kv.s[1].rot) fwht256(y, lane);
    float4 * dst = reinterpret_cast<float4 *>(J.O + ((size_t) t * NH + h) * HD + lane * 8);
    dst[0] = make_float4(y[0], y[1], y[2], y[3]);
    dst[1] = make_float4(y[4], y[5], y[6], y[7]);
}
__device__ __forceinline__ void merge_row(const AttnJob & J, const float * part, const float2 * ml, size_t i0, size_t pstep, size_t mstep, int count,
                                          int h, int t, int lane, int raw, float * part_out, float2 * ml_out) {
    float num[8], den, M;
    merge_accumulate(part, ml, i0, pstep, mstep, count, 0, 1, (h % GQ) * J.T + t, lane, num, den, M);
    merge_finish(J, h, t, lane, raw, part_out, ml_out, num, den, M);
}

} // namespace mkkv
