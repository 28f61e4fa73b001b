// Quantized GEMV whose CTAs build their own activation (k2t_prologue.cuh) before they reduce: residual add + RMSNorm +
// rotation + int8 in front of qkv / gate_up / lm_head / the routed experts' gate_up, SwiGLU + rotation + int8 in front of
// down, the embedding lookup in front of the first layer's qkv.  One decode step then needs no kernel of its own for these
// operators (the reference's forward_token_sdot_megakernel folds them into its workers the same way,
// src/model/real_llm.rs:6723-6730, 6927-6953).  A CTA holds several independent GEMV teams (the warp pipeline of
// k2t_gemv_core.cuh, activations read from shared memory); the first weight stages of every warp are requested before
// the kernel waits for its predecessor, so the prologue runs while they arrive.
#include <algorithm>
#include <cstdlib>

#include "k2t_gemv_core.cuh"
#include "k2t_gemv_fused.h"
#include "k2t_prologue.cuh"

namespace k2t {

constexpr uint32_t FUSED_MAX_WARPS = 14, FUSED_MIN_WARPS = 4;
constexpr uint32_t FUSED_SMEM_LIMIT = 227u * 1024u;

struct FusedLayout { uint32_t warps, wk, teams; };      // warps per CTA, warps per team, teams per CTA (warps beyond teams * wk only help with the prologue)

template <int FMT>
__device__ __forceinline__ void fused_cta(const GemvArgs &a, const FusedPro &p, const FusedLayout &lay, const float *gate_up, float *out,
                                          uint8_t *smem, bool wait_first) {
    const uint32_t warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    const uint32_t team = warp / lay.wk;
    uint8_t *wsm = smem + (size_t)warp * warp_smem<FMT>(1);
    float *s_f = reinterpret_cast<float *>(smem + (size_t)W * warp_smem<FMT>(1)) + team * 32;
    const ActSmem act = act_carve(smem + (size_t)W * warp_smem<FMT>(1) + pro_round((size_t)W * 128), p.mode, p.n);
    __builtin_assume(__isShared(act.x)); __builtin_assume(__isShared(act.xq)); __builtin_assume(__isShared(act.xs));
    __builtin_assume(__isShared(act.xm)); __builtin_assume(__isShared(act.inv));
    if ((threadIdx.x & 31) == 0) gemv_init_barriers(wsm);
    __syncwarp();
    PipeState ps;
    // helper warps (beyond the CTA's teams) own no row block: gw = rows puts them past the last block
    const bool works = team < lay.teams;
    const uint32_t gw = works ? team * gridDim.x + blockIdx.x : 0xffffff00u, nw = lay.teams * gridDim.x;
    gemv_body<FMT, 1, false, true>(a, act.xq, act.xs, act.xm, out, wsm, s_f, gw, nw, warp % lay.wk, lay.wk, 1 + team, ps, [&] {
        if (wait_first) { pdl_wait(); pdl_trigger(); }
        cta_build_activation(act, p, gate_up);
    });
}

template <int FMT>
__global__ void __launch_bounds__(FUSED_MAX_WARPS * 32, 1) gemv_fused_kernel(const GemvArgs a, const FusedPro p, const FusedLayout lay) {
    extern __shared__ __align__(128) uint8_t smem[];
    fused_cta<FMT>(a, p, lay, p.gate_up, a.out, smem, true);
}

// Expert-batched form (grid.y = route slot): the matrix of expert route_ids[slot]; PRO_NORM builds one activation shared
// by all slots, PRO_SWIGLU the slot's own from its gate_up row.
struct FusedExperts {
    const ExpertCodebook *books;
    const uint8_t *const *bases;
    const uint8_t *base0;
    const uint32_t *route_ids;
    size_t gate_up_stride, out_stride;
    uint32_t n_experts;
};

template <int FMT>
__global__ void __launch_bounds__(FUSED_MAX_WARPS * 32, 1) gemv_fused_expert_kernel(GemvArgs a, const FusedPro p, const FusedLayout lay, const FusedExperts b) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_wait();
    pdl_trigger();
    const uint32_t slot = blockIdx.y, e = __ldcg(b.route_ids + slot);
    if (e >= b.n_experts) {
        if (threadIdx.x == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 4u);
        return;
    }
    const uint8_t *base = b.bases[e];
    if (base == nullptr) return;
    {
        const uint4 *bk = reinterpret_cast<const uint4 *>(b.books + e);
        const uint4 c0 = __ldg(bk), c1 = __ldg(bk + 1), t = __ldg(bk + 2), o = __ldg(bk + 3);
        a.cb[0] = c0.x; a.cb[1] = c0.y; a.cb[2] = c0.z; a.cb[3] = c0.w; a.cb[4] = c1.x; a.cb[5] = c1.y; a.cb[6] = c1.z; a.cb[7] = c1.w;
        a.tab[0] = t.x; a.tab[1] = t.y; a.tab[2] = t.z; a.tab[3] = t.w;
        a.nf4_offset = (int32_t)o.x;
    }
#pragma unroll
    for (int k = 0; k < 3; ++k) a.plane[k] = base + (a.plane[k] - b.base0);
    a.scales = reinterpret_cast<const uint16_t *>(base + (reinterpret_cast<const uint8_t *>(a.scales) - b.base0));
    fused_cta<FMT>(a, p, lay, p.gate_up != nullptr ? p.gate_up + slot * b.gate_up_stride : nullptr, a.out + slot * b.out_stride, smem, false);
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
struct FusedShape { FusedLayout lay; uint32_t ctas; uint32_t smem; };

static uint32_t env_u32(const char *name) { const char *v = std::getenv(name); return v ? (uint32_t)std::atoi(v) : 0u; }

// CTAs per SM and warps per CTA: as many resident warps as shared memory allows (at most FUSED_MAX_WARPS per SM), in two
// or three CTAs per SM when that costs little, so that the CTAs of the next kernel get onto an SM (and request their
// weights) as soon as one CTA of this kernel has left it.  Then the team shape by the cost model of choose_team in
// k2t_gemv.cu: few fat rounds beat many thin ones, every team gets the same number of row blocks.
static bool choose_fused(uint32_t n_rb, uint32_t np, uint32_t warp_bytes, uint32_t act_bytes, uint32_t n_slot, int sm_count, FusedShape &out) {
    static const uint32_t force_cps = env_u32("KRONOS_CUDA_FUSED_CPS"), force_w = env_u32("KRONOS_CUDA_FUSED_WARPS");      // measurement switches
    uint32_t best_total = 0, cps = 1, wmax = 0;
    uint32_t w_of[4] = {0, 0, 0, 0};
    for (uint32_t c = 1; c <= 3; ++c) {
        const uint32_t budget = FUSED_SMEM_LIMIT / c;
        if (budget < 1024u + act_bytes + 128u + warp_bytes + 128u) continue;
        uint32_t w = (budget - 1024u - act_bytes - 128u) / (warp_bytes + 128u);
        w = std::min(w, FUSED_MAX_WARPS / c);
        w_of[c] = w;
        best_total = std::max(best_total, w * c);
    }
    if (best_total == 0) return false;
    for (uint32_t c = 3; c >= 1; --c)
        if (w_of[c] > 0 && w_of[c] * c * 100u >= best_total * 85u) { cps = c; wmax = w_of[c]; break; }
    if (force_cps >= 1 && force_cps <= 3 && w_of[force_cps] > 0) { cps = force_cps; wmax = w_of[force_cps]; }
    if (force_w >= 1 && force_w <= wmax) wmax = force_w;
    FusedLayout best{0, 1, 1};
    uint32_t best_ctas = 0;
    float best_cost = 1e30f;
    for (uint32_t wk = 1; wk <= 8 && wk <= wmax && (wk == 1 || wk <= np); wk *= 2) {
        const uint32_t tpc_max = wmax / wk;
        const uint32_t cap = std::max(1u, tpc_max * cps * (uint32_t)sm_count / n_slot);
        const uint32_t J = (n_rb + cap - 1) / cap, teams = (n_rb + J - 1) / J;
        const uint32_t groups = (J + GB - 1) / GB, in_group = std::min(GB, J), rounds = (np + wk - 1) / wk;
        const float cost = (float)(groups * rounds) * (1.5f + 0.25f * (float)in_group);
        if (cost < 0.9f * best_cost) {
            best_cost = cost;
            // spread the teams over the SMs first: a CTA takes several teams only when there are more teams than SMs
            const uint32_t tpc = std::min(tpc_max, std::max(1u, (teams * n_slot + (uint32_t)sm_count * cps - 1) / ((uint32_t)sm_count * cps)));
            best.wk = wk; best.teams = tpc; best.warps = std::max(tpc * wk, std::min(FUSED_MIN_WARPS, wmax));
            best_ctas = (teams + tpc - 1) / tpc;
        }
    }
    if (best_ctas == 0) return false;
    out.lay = best; out.ctas = best_ctas;
    out.smem = best.warps * warp_bytes + (uint32_t)pro_round((size_t)best.warps * 128) + act_bytes;
    return true;
}

// the 1 KiB every CTA reserves in choose_fused also covers the few static bytes of a kernel (the E8Q2 template table)
template <typename K>
static cudaError_t allow_smem(K kernel, bool &) {
    return allow_dynamic_smem(reinterpret_cast<const void *>(kernel), FUSED_SMEM_LIMIT - 1024u);
}

template <int FMT>
static cudaError_t launch_fused_fmt(cudaStream_t stream, const GemvArgs &a, const FusedPro &p, int sm_count, bool pdl) {
    static bool attr_done = false;
    FusedShape sh;
    const uint32_t n_rb = (a.rows + RS - 1) / RS, np = (a.nc + 31) / 32;
    if (!choose_fused(n_rb, np, warp_smem<FMT>(1), (uint32_t)act_smem_bytes(p.mode, p.n), 1, sm_count, sh)) return cudaErrorInvalidValue;
    cudaError_t e = allow_smem(gemv_fused_kernel<FMT>, attr_done);
    if (e != cudaSuccess) return e;
    return launch_kernel(gemv_fused_kernel<FMT>, dim3(sh.ctas), dim3(32 * sh.lay.warps), sh.smem, stream, pdl, a, p, sh.lay);
}

template <int FMT>
static cudaError_t launch_fused_expert_fmt(cudaStream_t stream, const GemvArgs &a, const FusedPro &p, const FusedExperts &b, uint32_t n_slot, int sm_count, bool pdl) {
    static bool attr_done = false;
    FusedShape sh;
    const uint32_t n_rb = (a.rows + RS - 1) / RS, np = (a.nc + 31) / 32;
    if (!choose_fused(n_rb, np, warp_smem<FMT>(1), (uint32_t)act_smem_bytes(p.mode, p.n), n_slot, sm_count, sh)) return cudaErrorInvalidValue;
    cudaError_t e = allow_smem(gemv_fused_expert_kernel<FMT>, attr_done);
    if (e != cudaSuccess) return e;
    return launch_kernel(gemv_fused_expert_kernel<FMT>, dim3(sh.ctas, n_slot), dim3(32 * sh.lay.warps), sh.smem, stream, pdl, a, p, sh.lay, b);
}

bool gemv_fused_fits(const DeviceMatrix &m, uint32_t mode) {
    GemvArgs a;
    const int fmt = fill_gemv_args(m, true, a);
    if (fmt < 0) return false;
    FusedShape sh;
    return choose_fused((a.rows + RS - 1) / RS, (a.nc + 31) / 32, gemv_warp_smem_bytes(fmt), (uint32_t)act_smem_bytes(mode, m.geom.cols), 1, 148, sh);
}

cudaError_t launch_gemv_fused(cudaStream_t stream, const DeviceMatrix &m, const FusedPro &p, float *out, int sm_count, uint32_t *err_flag, bool pdl) {
    GemvArgs a;
    const int fmt = fill_gemv_args(m, true, a);
    if (fmt < 0 || p.n != m.geom.cols) return cudaErrorInvalidValue;
    a.out = out; a.err_flag = err_flag; a.out_stride = m.geom.rows; a.pdl = pdl ? 1u : 0u; a.n_tok = 1;
    switch (fmt) {
        case FMT_BP4: return launch_fused_fmt<FMT_BP4>(stream, a, p, sm_count, pdl);
        case FMT_BP5: return launch_fused_fmt<FMT_BP5>(stream, a, p, sm_count, pdl);
        case FMT_BP6: return launch_fused_fmt<FMT_BP6>(stream, a, p, sm_count, pdl);
        case FMT_NF4: return launch_fused_fmt<FMT_NF4>(stream, a, p, sm_count, pdl);
        case FMT_NF4G: return launch_fused_fmt<FMT_NF4G>(stream, a, p, sm_count, pdl);
        case FMT_NF3: return launch_fused_fmt<FMT_NF3>(stream, a, p, sm_count, pdl);
        case FMT_NF5: return launch_fused_fmt<FMT_NF5>(stream, a, p, sm_count, pdl);
        case FMT_E8Q2: return launch_fused_fmt<FMT_E8Q2>(stream, a, p, sm_count, pdl);
        default: return cudaErrorNotSupported;
    }
}

cudaError_t launch_gemv_fused_experts(cudaStream_t stream, const DeviceMatrix &m0, int fmt, const ExpertCodebook *books, const uint8_t *const *bases,
                                      const uint32_t *route_ids, uint32_t n_slot, uint32_t n_experts, const FusedPro &p, size_t gate_up_stride,
                                      float *out, size_t out_stride, int sm_count, uint32_t *err_flag, bool pdl) {
    if (n_slot == 0) return cudaSuccess;
    GemvArgs a;
    if (fill_gemv_args(m0, true, a) < 0 || p.n != m0.geom.cols) return cudaErrorInvalidValue;
    a.out = out; a.err_flag = err_flag; a.out_stride = m0.geom.rows; a.pdl = pdl ? 1u : 0u; a.n_tok = 1;
    const FusedExperts b{books, bases, m0.d_base, route_ids, gate_up_stride, out_stride, n_experts};
    switch (fmt) {
        case FMT_NF4: return launch_fused_expert_fmt<FMT_NF4>(stream, a, p, b, n_slot, sm_count, pdl);
        case FMT_NF4G: return launch_fused_expert_fmt<FMT_NF4G>(stream, a, p, b, n_slot, sm_count, pdl);
        case FMT_NF3: return launch_fused_expert_fmt<FMT_NF3>(stream, a, p, b, n_slot, sm_count, pdl);
        case FMT_NF5: return launch_fused_expert_fmt<FMT_NF5>(stream, a, p, b, n_slot, sm_count, pdl);
        case FMT_E8Q2: return launch_fused_expert_fmt<FMT_E8Q2>(stream, a, p, b, n_slot, sm_count, pdl);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace k2t
