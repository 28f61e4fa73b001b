// Host-callable launchers of the sm_100a kernels (implemented in the .cu files of this folder).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "k2t_layout.h"

namespace k2t {

// Device-resident matrix (image produced by repack_matrix, uploaded once).
struct DeviceMatrix {
    MatrixGeom geom;
    uint8_t *d_base = nullptr;      // one allocation: code planes, scales (offsets in geom)
    size_t device_bytes = 0;
};

cudaError_t launch_fwht_quant(cudaStream_t stream, const float *x, const float *norm_w, const float *inv_rms,
                              uint32_t n_tok, uint32_t cols, uint64_t chunk0, int8_t *q, float *scales,
                              int32_t *sums);

// Quantized GEMV / small-N GEMM over all rows. n_tok in 1..4 (callers split longer batches). Returns the number of kernel launches
// in *launches. xsum may be null for NF formats.  pdl: launch as a programmatic dependent of the previous
// kernel in the stream (the weight pipeline starts before that kernel has finished).
cudaError_t launch_gemv(cudaStream_t stream, const DeviceMatrix &m, const int8_t *xq, const float *xs,
                        const int32_t *xsum, uint32_t n_tok, float *out, size_t out_stride, int32_t *int_dots,
                        int sm_count, uint32_t *err_flag, uint32_t *launches, bool pdl = false);

// The same product for any number of tokens: batches of sixteen tokens or more run on the tensor cores in one launch
// (k2t_gemm_tc.cu: exact int32 chunk dots by `tcgen05.mma`, the fp32 chains in the same order), shorter ones and calls that
// ask for the integer dots as 4-token weight passes.  Same results either way.
cudaError_t launch_gemv_batch(cudaStream_t stream, const DeviceMatrix &m, const int8_t *xq, const float *xs, const int32_t *xsum,
                              size_t n_tok, float *out, size_t out_stride, int32_t *int_dots, int sm_count, uint32_t *err_flag,
                              uint32_t *launches, bool pdl = false);

// Decode tables of one expert matrix (every expert of a MoE layer carries its own codebook): 64 bytes.
struct ExpertCodebook {
    uint32_t cb[8];      // expanded codebook, 4 centroids per word
    uint32_t tab[4];     // NF4 two-table decode
    int32_t nf4_offset;
    uint32_t pad[3];
};
// Fills `out` for matrix m and returns its kernel format index (FMT_*; FMT_COUNT = NF4 with the general decode).
int expert_codebook(const DeviceMatrix &m, ExpertCodebook &out);

// Expert-batched GEMV (one token): slot s of n_slot multiplies the matrix of expert route_ids[s] (device memory; all
// experts share the geometry of m0 and the kernel format `fmt`; bases[e] / books[e] = device image and decode tables of
// expert e) with activation row s (strides 0 = shared) into out + s * out_stride.
cudaError_t launch_gemv_experts(cudaStream_t stream, const DeviceMatrix &m0, int fmt, const ExpertCodebook *books, const uint8_t *const *bases,
                                const uint32_t *route_ids, uint32_t n_slot, const int8_t *xq, const float *xs, const int32_t *xsum,
                                size_t xq_stride, size_t xs_stride, float *out, size_t out_stride, int sm_count, uint32_t *err_flag, bool pdl,
                                uint32_t n_experts,
                                uint32_t route_group = 0, uint32_t route_stride = 0, uint32_t act_group = 1);

// Largest n_tok one launch_gemv call accepts for this matrix (4: the reference's tokens per weight tile in prompt batches).
uint32_t gemv_max_tokens(const DeviceMatrix &m);

}  // namespace k2t
