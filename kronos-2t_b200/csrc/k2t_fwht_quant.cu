// Activation rotation + int8 quantization kernel
// (Int8ChunkActivation::populate_fwht / populate_rmsnorm_fwht, src/kernels/simd_lut.rs:2954-3196).
// One warp per (token, 64-column chunk); 8 warps per CTA.  HBM traffic: 4 B/element in,
// 1 B/element + 8 B/chunk out.
#include "k2t_fwht.cuh"
#include "k2t_kernels.h"

namespace k2t {

__global__ void __launch_bounds__(256)
fwht_quant_kernel(const float *__restrict__ x, const float *__restrict__ norm_w,
                  const float *__restrict__ inv_rms, uint32_t n_tok, uint32_t nc, uint64_t chunk0,
                  int8_t *__restrict__ q, float *__restrict__ scales, int32_t *__restrict__ sums) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t item = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    // launched as a programmatic dependent: wait for the producer of x, then let the next kernel (a GEMV that
    // starts streaming its weights before it needs these activations) begin
    pdl_wait();
    pdl_trigger();
    if (item >= (uint64_t)n_tok * nc) return;   // whole warp leaves together
    const uint32_t t = (uint32_t)(item / nc), c = (uint32_t)(item % nc);
    const size_t base = (size_t)t * nc * 64 + (size_t)c * 64;
    float2 v = reinterpret_cast<const float2 *>(x + base)[lane];
    if (norm_w != nullptr) {
        const float inv = inv_rms[t];
        const float2 w = reinterpret_cast<const float2 *>(norm_w + (size_t)c * 64)[lane];
        v.x = __fmul_rn(__fmul_rn(v.x, inv), w.x);   // (x * inv_rms) * weight: two roundings
        v.y = __fmul_rn(__fmul_rn(v.y, inv), w.y);
    }
    warp_fwht64(v.x, v.y, chunk0 + c, lane);
    int q0, q1, sum;
    float scale;
    warp_quant64(v.x, v.y, q0, q1, scale, sum);
    reinterpret_cast<char2 *>(q + base)[lane] = make_char2((signed char)q0, (signed char)q1);
    if (lane == 0) {
        scales[(size_t)t * nc + c] = scale;
        sums[(size_t)t * nc + c] = sum;
    }
}

cudaError_t launch_fwht_quant(cudaStream_t stream, const float *x, const float *norm_w, const float *inv_rms,
                              uint32_t n_tok, uint32_t cols, uint64_t chunk0, int8_t *q, float *scales,
                              int32_t *sums) {
    const uint32_t nc = cols / 64;
    const uint64_t items = (uint64_t)n_tok * nc;
    if (items == 0) return cudaSuccess;
    return launch_kernel(fwht_quant_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, stream, true, x, norm_w, inv_rms, n_tok, nc, chunk0, q,
                         scales, sums);
}

}  // namespace k2t
