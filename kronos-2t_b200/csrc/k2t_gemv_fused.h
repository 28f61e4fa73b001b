// Launchers of the GEMV kernels that build their own activation (k2t_gemv_fused.cu).
#pragma once
#include "k2t_kernels.h"

namespace k2t {

struct FusedPro;
struct GemvArgs;

// host helpers of k2t_gemv.cu
int fill_gemv_args(const DeviceMatrix &m, bool has_xsum, GemvArgs &a);
uint32_t gemv_warp_smem_bytes(int fmt_index);

// true when one CTA can hold the activation of this matrix (its columns) beside at least one GEMV warp
bool gemv_fused_fits(const DeviceMatrix &m, uint32_t mode);

// out[r] = W x for the activation x the prologue `p` describes (p.n = columns of m); one token
cudaError_t launch_gemv_fused(cudaStream_t stream, const DeviceMatrix &m, const FusedPro &p, float *out, int sm_count, uint32_t *err_flag, bool pdl);

// Expert-batched form: slot s of n_slot multiplies the matrix of expert route_ids[s] (see launch_gemv_experts) into
// out + s * out_stride.  PRO_NORM: every slot shares the activation; PRO_SWIGLU: slot s reads p.gate_up + s * gate_up_stride.
cudaError_t launch_gemv_fused_experts(cudaStream_t stream, const DeviceMatrix &m0, int fmt, const ExpertCodebook *books, const uint8_t *const *bases,
                                      const uint32_t *route_ids, uint32_t n_slot, uint32_t n_experts, const FusedPro &p, size_t gate_up_stride,
                                      float *out, size_t out_stride, int sm_count, uint32_t *err_flag, bool pdl);

}  // namespace k2t
