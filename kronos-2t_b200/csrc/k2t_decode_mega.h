// Whole-token decode kernel: argument blocks and launcher (k2t_decode_mega.cu).
#pragma once
#include "k2t_gemv_core.cuh"
#include "k2t_model_kernels.h"

namespace k2t {

struct MegaMatrix {          // lives in device memory
    GemvArgs g;              // matrix part only (activation / output pointers unused)
    uint32_t fmt;            // kernel format index (FMT_*, FMT_NF4G)
    uint32_t wk;             // warps per team: 1, 2, 4 or 8
};

struct MegaLayer {           // lives in device memory
    MegaMatrix qkv, o, gate_up, down;
    const float *input_norm, *post_norm, *qkv_bias, *q_norm, *k_norm;
};

struct MegaArgs {
    const MegaLayer *layers;
    const MegaMatrix *head;
    uint32_t n_layers, hidden, n_q, n_kv, head_dim, inter, vocab, max_seq, kv_bits;
    float eps, attn_scale;
    int32_t qk_norm_after_rope;
    const float *final_norm, *rope;
    EmbedArgs embed;         // `token` and `hidden` unused
    float *hidden_a, *hidden_b, *proj, *qkv, *gate_up, *logits, *attn_tap;
    int8_t *act_q; float *act_s; int32_t *act_m;           // o_proj activation (written by the attention CTAs)
    int8_t *k_q8, *v_q8; float *k_scale, *v_scale;
    int8_t *v_t;                 // block-transposed copy of the value rows (null when the engine keeps none)
    uint32_t *token, *pos, *step, *history;                // device scalars / token history
    uint32_t *barrier, *err_flag;                          // grid barrier counter (zero at launch), error word
    uint32_t first_token, pos0, n_steps;
    unsigned long long *trace; uint32_t trace_cap;         // optional phase trace: trace[0..cap) marks, trace[cap] = count
    uint32_t warp_smem, kmax;                              // shared-memory layout: bytes per warp region, longest activation
};

// Dynamic shared memory the kernel needs for this layout.
size_t decode_mega_smem(uint32_t warp_smem, uint32_t kmax);
// cudaSuccess when the kernel can run cooperatively with one CTA per SM on the current device.
cudaError_t decode_mega_check(size_t smem, int sm_count);
// Cooperative launch: n_steps greedy tokens in one kernel.  The barrier counter must be zero.
cudaError_t launch_decode_mega(cudaStream_t s, const MegaArgs &a, size_t smem, int sm_count);

// Host helpers of k2t_gemv.cu
int fill_gemv_args(const DeviceMatrix &m, bool has_xsum, GemvArgs &a);
uint32_t gemv_warp_smem_bytes(int fmt_index);

}  // namespace k2t
