// TEST INFRASTRUCTURE ONLY. Driver around the reference project's own KV quantizer / dequantizer device functions, which
// oracle/build_ref.py cuts out of the reference source into ref_cut.inc at build time (qwen38_mk.cu:2003-2097, 2335-2368,
// 2457-2468). One warp per row, lane l holds values 8 l .. 8 l + 7, exactly as the reference calls them. Host wrappers take
// host buffers and do their own device allocation: this library is only ever loaded by tests on a GPU box.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#define HD 256
#include "ref_cut.inc"

__global__ void w_quant(const float * rows, int nrows, int bits, int rot, int8_t * q, __half * sc) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= nrows) return;
    float v[8];
    for (int k = 0; k < 8; k++) v[k] = rows[(size_t) row * 256 + lane * 8 + k];
    if (rot) fwht256(v);
    int8_t * qr = q + (size_t) row * 256; // rows are laid out at a 256-byte pitch whatever the format
    __half * sr = sc + (size_t) row * 8;
    if (bits == 8) kv_store_q8(qr, sr, v);
    else if (bits == 4) kv_store_q4(qr, sr, v);
    else kv_store_qn(qr, sr, v, bits);
}

__global__ void w_dequant(const uint8_t * q, const __half * sc, int nrows, int bits, __half * out) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= nrows) return;
    const uint8_t * rp = q + (size_t) row * 256;
    const float d = __half2float(sc[(size_t) row * 8 + (lane >> 2)]);
    __half2 h[4];
    if (bits == 8) q8_to_f16(*reinterpret_cast<const uint2 *>(rp + 8 * lane), d, h);
    else if (bits == 4) q4_to_f16(*reinterpret_cast<const unsigned *>(rp + 4 * lane), d, h);
    else qn_to_f16(*reinterpret_cast<const unsigned *>(rp + 4 * lane), kv_hi(rp + 128 + lane * (bits - 4), bits - 4), d, bits, h);
    *reinterpret_cast<int4 *>(out + (size_t) row * 256 + lane * 8) = *reinterpret_cast<int4 *>(h);
}

#define WCK(x)                                                                          \
    do {                                                                                \
        cudaError_t e_ = (x);                                                           \
        if (e_ != cudaSuccess) {                                                        \
            fprintf(stderr, "ref_witness: %s: %s\n", #x, cudaGetErrorString(e_));       \
            return -1;                                                                  \
        }                                                                               \
    } while (0)

extern "C" {
// rows: host fp32 [nrows][256] -> q: host [nrows][256] bytes (the row's 32 * bits bytes first), sc: host [nrows][8] fp16 bits
int ref_quant(const float * rows, int nrows, int bits, int rot, uint8_t * q, uint16_t * sc) {
    float * dr;
    int8_t * dq;
    __half * ds;
    WCK(cudaMalloc(&dr, (size_t) nrows * 1024));
    WCK(cudaMalloc(&dq, (size_t) nrows * 256));
    WCK(cudaMalloc(&ds, (size_t) nrows * 16));
    WCK(cudaMemset(dq, 0, (size_t) nrows * 256));
    WCK(cudaMemcpy(dr, rows, (size_t) nrows * 1024, cudaMemcpyHostToDevice));
    w_quant<<<(nrows + 7) / 8, 256>>>(dr, nrows, bits, rot, dq, ds);
    WCK(cudaGetLastError());
    WCK(cudaMemcpy(q, dq, (size_t) nrows * 256, cudaMemcpyDeviceToHost));
    WCK(cudaMemcpy(sc, ds, (size_t) nrows * 16, cudaMemcpyDeviceToHost));
    cudaFree(dr);
    cudaFree(dq);
    cudaFree(ds);
    return 0;
}
// q: host [nrows][256] bytes, sc: host [nrows][8] -> out: host fp16 bits [nrows][256], the operand values d * q rounded to half
int ref_dequant(const uint8_t * q, const uint16_t * sc, int nrows, int bits, uint16_t * out) {
    uint8_t * dq;
    __half *ds, *dout;
    WCK(cudaMalloc(&dq, (size_t) nrows * 256));
    WCK(cudaMalloc(&ds, (size_t) nrows * 16));
    WCK(cudaMalloc(&dout, (size_t) nrows * 512));
    WCK(cudaMemcpy(dq, q, (size_t) nrows * 256, cudaMemcpyHostToDevice));
    WCK(cudaMemcpy(ds, sc, (size_t) nrows * 16, cudaMemcpyHostToDevice));
    w_dequant<<<(nrows + 7) / 8, 256>>>(dq, ds, nrows, bits, dout);
    WCK(cudaGetLastError());
    WCK(cudaMemcpy(out, dout, (size_t) nrows * 512, cudaMemcpyDeviceToHost));
    cudaFree(dq);
    cudaFree(ds);
    cudaFree(dout);
    return 0;
}
}
