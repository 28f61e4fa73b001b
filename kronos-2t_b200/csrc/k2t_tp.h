// Tensor-parallel exchange kernel (k2t_tp.cu): argument block and launcher.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace k2t {

constexpr uint32_t TP_MAX = 8;

struct TpLink {
    float *peer_data[TP_MAX];       // exchange buffer of every rank (own buffer at index `rank`), mapped into this process
    uint32_t *peer_flags[TP_MAX];   // their flag words
    unsigned long long *peer_ll[TP_MAX];   // their (value, call number) words (one 64-bit word each) for the sums fused into the norm kernel: [2][tp][ll_slot]
    uint32_t tp, rank;
    uint32_t slot;                  // floats per (half, rank) slot
    uint32_t ll_slot;               // words per (half, rank) slot of the (value, call number) region
    uint32_t *epoch;                // this rank's call counter (device memory)
    uint32_t *err;                  // error word of the context
    uint32_t wait_polls;            // polls a kernel spends, in total, on words a peer has not written yet before it gives up (error word 3)
};
constexpr uint32_t TP_WAIT_POLLS_DEFAULT = 1u << 22;

// dst = sum over ranks of src (gather_stride = 0), or dst[r * gather_stride + i] = rank r's src[i] (gather_stride > 0).
// n floats (a multiple of 4, at most L.slot).  Every rank must make the same sequence of calls.
cudaError_t launch_tp_exchange(cudaStream_t s, const TpLink &L, const float *src, float *dst, uint32_t n, uint32_t gather_stride, bool pdl);

}  // namespace k2t
