// Stand-alone quantized GEMV / small-N GEMM kernel and its host launcher (body: k2t_gemv_core.cuh).
#include <algorithm>
#include <cstdlib>

#include "k2t_gemv_core.cuh"

namespace k2t {

// blockDim.x = 32 * WK: one team per CTA, persistent grid.
template <int FMT, int NT, bool DOTS>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t wid = threadIdx.x >> 5, WK = blockDim.x >> 5;
    uint8_t *wsm = smem + (size_t)wid * warp_smem<FMT>(NT);
    if ((threadIdx.x & 31) == 0) gemv_init_barriers(wsm);
    __syncwarp();
    PipeState ps;
    gemv_body<FMT, NT, DOTS, false>(a, a.xq, a.xs, a.xsum, a.out, wsm, reinterpret_cast<float *>(smem + (size_t)WK * warp_smem<FMT>(NT)),
                                    blockIdx.x, gridDim.x, wid, WK, 0, ps);
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
// Team shape for a launch: WK warps per team (they split the passes of their row blocks) and the number of teams.
// A team works through its J row blocks in groups of GB; each group costs one ROUND per WK passes, and a round pays a
// fixed latency (activation loads, first stage in flight, the hand-off of the fp32 chain) before its stages stream.
// So few fat rounds beat many thin ones: among the shapes that fit the SMs, take the one with the smallest
// groups x rounds x (latency + stages per round), with every team given the same number of blocks (no tail).
struct TeamShape { uint32_t wk, teams, smem; };
static TeamShape choose_team(uint32_t n_rb, uint32_t np, uint32_t warp_bytes, uint32_t extra_bytes, uint32_t n_slot, int sm_count) {
    TeamShape best{1, 1, warp_bytes + extra_bytes};
    float best_cost = 1e30f;
    static const uint32_t force_wk = [] { const char *v = std::getenv("KRONOS_CUDA_GEMV_WK"); return v ? (uint32_t)std::atoi(v) : 0u; }();   // measurement switch
    for (uint32_t wk = 1; wk <= 8 && (wk == 1 || wk <= np); wk *= 2) {
        if (force_wk && wk != force_wk && !(wk < force_wk && wk * 2 > std::min(8u, np))) continue;     // the forced size, or the largest one the passes allow
        const uint32_t smem = wk * warp_bytes + extra_bytes;
        uint32_t per_sm = (227u * 1024u) / (smem + 1024u);      // CTAs per SM by shared memory (1 KiB reserved per CTA)
        if (per_sm == 0) continue;
        per_sm = std::min(per_sm, 32u);
        if (per_sm * wk > 48) per_sm = 48 / wk;
        static const uint32_t force_per_sm = [] { const char *v = std::getenv("KRONOS_CUDA_GEMV_WARPS"); return v ? (uint32_t)std::atoi(v) : 0u; }();   // measurement switch
        if (force_per_sm && force_per_sm / wk >= 1 && force_per_sm / wk <= per_sm + 4) per_sm = force_per_sm / wk;
        const uint32_t cap = std::max(1u, per_sm * (uint32_t)sm_count / n_slot);
        const uint32_t J = (n_rb + cap - 1) / cap, teams = (n_rb + J - 1) / J;
        const uint32_t groups = (J + GB - 1) / GB, in_group = std::min(GB, J), rounds = (np + wk - 1) / wk;
        const float cost = (float)(groups * rounds) * (1.5f + 0.25f * (float)in_group);
        if (cost < 0.9f * best_cost) { best_cost = cost; best = TeamShape{wk, teams, smem}; }      // a larger team has to win clearly: its chain hand-offs are serial
    }
    return best;
}

template <int FMT, int NT, bool DOTS>
static cudaError_t launch_one(cudaStream_t stream, const GemvArgs &a, int sm_count) {
    const uint32_t n_rb = (a.rows + RS - 1) / RS, np = (a.nc + 31) / 32;
    const TeamShape t = choose_team(n_rb, np, warp_smem<FMT>(NT), NT * 32 * 4 + 16, 1, sm_count);      // hand-off array + turn counter
    cudaError_t e = cudaSuccess;
    e = allow_dynamic_smem(reinterpret_cast<const void *>(gemv_kernel<FMT, NT, DOTS>), t.smem);
    if (e != cudaSuccess) return e;
    return launch_kernel(gemv_kernel<FMT, NT, DOTS>, dim3(t.teams), dim3(32 * t.wk), t.smem, stream, a.pdl != 0, a);
}

template <int FMT>
static cudaError_t launch_fmt(cudaStream_t stream, const GemvArgs &a, uint32_t nt, int sm_count) {
    const bool dots = a.int_dots != nullptr;
    switch (nt) {
        case 1: return dots ? launch_one<FMT, 1, true>(stream, a, sm_count) : launch_one<FMT, 1, false>(stream, a, sm_count);
        case 2: return dots ? launch_one<FMT, 2, true>(stream, a, sm_count) : launch_one<FMT, 2, false>(stream, a, sm_count);
        default: return dots ? launch_one<FMT, 4, true>(stream, a, sm_count) : launch_one<FMT, 4, false>(stream, a, sm_count);
    }
}

uint32_t gemv_max_tokens(const DeviceMatrix &) { return 4; }

int fill_gemv_args(const DeviceMatrix &m, bool has_xsum, GemvArgs &a);

// Expert-batched GEMV: grid.y = route slot.  Every routed expert has the same geometry; slot s reads the matrix of
// expert route_ids[s] (written by the router kernel just before, so the ids are read after the dependency wait),
// its own activation rows (stride 0 = one activation shared by all slots) and writes its own output row.
struct ExpertBatch {
    const ExpertCodebook *books;   // device: decode tables of every expert (each expert has its own codebook)
    const uint8_t *const *bases;   // device: image base of every expert of the layer
    const uint8_t *base0;          // the base the GemvArgs plane pointers were filled with
    const uint32_t *route_ids;     // device [n_slot]
    size_t xq_stride, xs_stride;   // per-slot strides of the activation
    size_t out_stride;             // per-slot stride of the output
    uint32_t n_experts;            // entries of books / bases: a route id outside is refused (error word 4)
    // batches of tokens: slot = token * route_group + route; the token's routes start at route_ids + token * route_stride,
    // and act_group consecutive slots share one activation (the token's, for the gate_up projection)
    uint32_t route_group, route_stride, act_group;
};

template <int FMT>
__global__ void __launch_bounds__(256) gemv_expert_kernel(GemvArgs a, const ExpertBatch b) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t wid = threadIdx.x >> 5, WK = blockDim.x >> 5;
    uint8_t *wsm = smem + (size_t)wid * warp_smem<FMT>(1);
    if ((threadIdx.x & 31) == 0) gemv_init_barriers(wsm);
    __syncwarp();
    pdl_wait();
    const uint32_t slot = blockIdx.y, e = __ldcg(b.route_ids + (size_t)(slot / b.route_group) * b.route_stride + slot % b.route_group);
    const size_t ai = slot / b.act_group;
    if (e >= b.n_experts) {            // never produced by the router kernel; a foreign id must not index the tables
        if (threadIdx.x == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 4u);
        return;
    }
    const uint8_t *base = b.bases[e];
    if (base == nullptr) return;       // expert parallelism: another rank owns this expert (the whole CTA leaves, no copy is in flight)
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
    PipeState ps;
    gemv_body<FMT, 1, false, false>(a, a.xq + ai * b.xq_stride, a.xs + ai * b.xs_stride,
                                    a.xsum != nullptr ? a.xsum + ai * b.xs_stride : nullptr, a.out + slot * b.out_stride, wsm,
                                    reinterpret_cast<float *>(smem + (size_t)WK * warp_smem<FMT>(1)), blockIdx.x, gridDim.x, wid, WK, 0, ps);
}

template <int FMT>
static cudaError_t launch_expert_fmt(cudaStream_t stream, const GemvArgs &a, const ExpertBatch &b, uint32_t n_slot, int sm_count) {
    const uint32_t n_rb = (a.rows + RS - 1) / RS, np = (a.nc + 31) / 32;
    const TeamShape t = choose_team(n_rb, np, warp_smem<FMT>(1), 32 * 4 + 16, n_slot, sm_count);
    cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(gemv_expert_kernel<FMT>), t.smem);
    if (e != cudaSuccess) return e;
    return launch_kernel(gemv_expert_kernel<FMT>, dim3(t.teams, n_slot), dim3(32 * t.wk), t.smem, stream, a.pdl != 0, a, b);
}

int expert_codebook(const DeviceMatrix &m, ExpertCodebook &out) {
    GemvArgs a;
    const int fmt = fill_gemv_args(m, true, a);
    for (int i = 0; i < 8; ++i) out.cb[i] = a.cb[i];
    for (int i = 0; i < 4; ++i) out.tab[i] = a.tab[i];
    out.nf4_offset = a.nf4_offset;
    out.pad[0] = out.pad[1] = out.pad[2] = 0;
    return fmt;
}

cudaError_t launch_gemv_experts(cudaStream_t stream, const DeviceMatrix &m0, int fmt, const ExpertCodebook *books, const uint8_t *const *bases, const uint32_t *route_ids,
                                uint32_t n_slot, const int8_t *xq, const float *xs, const int32_t *xsum, size_t xq_stride,
                                size_t xs_stride, float *out, size_t out_stride, int sm_count, uint32_t *err_flag, bool pdl, uint32_t n_experts,
                                uint32_t route_group, uint32_t route_stride, uint32_t act_group) {
    if (n_slot == 0) return cudaSuccess;
    if (route_group == 0) { route_group = n_slot; route_stride = 0; }
    if (act_group == 0) act_group = 1;
    GemvArgs a;
    if (fill_gemv_args(m0, xsum != nullptr, a) < 0) return cudaErrorNotSupported;
    a.xq = xq; a.xs = xs; a.xsum = xsum; a.out = out; a.err_flag = err_flag; a.out_stride = m0.geom.rows; a.pdl = pdl ? 1u : 0u; a.n_tok = 1;
    ExpertBatch b{books, bases, m0.d_base, route_ids, xq_stride, xs_stride, out_stride, n_experts, route_group, route_stride, act_group};
    switch (fmt) {
        case FMT_NF4: return launch_expert_fmt<FMT_NF4>(stream, a, b, n_slot, sm_count);
        case FMT_NF4G: return launch_expert_fmt<FMT_NF4G>(stream, a, b, n_slot, sm_count);
        case FMT_NF3: return launch_expert_fmt<FMT_NF3>(stream, a, b, n_slot, sm_count);
        case FMT_NF5: return launch_expert_fmt<FMT_NF5>(stream, a, b, n_slot, sm_count);
        case FMT_E8Q2: return launch_expert_fmt<FMT_E8Q2>(stream, a, b, n_slot, sm_count);
        default: return cudaErrorNotSupported;       // experts are NF matrices (2..5 bits)
    }
}

// Fills the matrix part of GemvArgs (planes, codebooks) and returns the kernel format index
// (FMT_NF4G for an NF4 codebook the two-table decode cannot represent), or -1 when unsupported.
int fill_gemv_args(const DeviceMatrix &m, bool has_xsum, GemvArgs &a) {
    const MatrixGeom &g = m.geom;
    for (int k = 0; k < 3; ++k) a.plane[k] = m.d_base + g.plane_off[k];
    a.scales = reinterpret_cast<const uint16_t *>(m.d_base + g.scale_off);
    a.xq = nullptr; a.xs = nullptr; a.xsum = nullptr; a.out = nullptr; a.int_dots = nullptr; a.err_flag = nullptr;
    a.out_stride = g.rows; a.pdl = 0;
    a.rows = g.rows; a.rows_pad = g.rows_pad; a.cols = g.cols; a.nc = g.nc; a.nsg = g.nsg; a.sgc = g.sgc; a.n_tok = 1;
    a.sgc_shift = 32;
    for (uint32_t sh = 0; sh < 4; ++sh) if ((1u << sh) == g.sgc) a.sgc_shift = sh;
    a.max_odd = g.max_odd; a.nf4_offset = g.nf4_offset;
    for (int i = 0; i < 8; ++i) {
        const uint8_t *b = reinterpret_cast<const uint8_t *>(g.codebook32) + 4 * i;
        a.cb[i] = (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
    }
    for (int i = 0; i < 2; ++i) {
        const uint8_t *h = g.nf4_hi + 4 * i, *l = g.nf4_lo + 4 * i;
        a.tab[i] = (uint32_t)h[0] | ((uint32_t)h[1] << 8) | ((uint32_t)h[2] << 16) | ((uint32_t)h[3] << 24);
        a.tab[2 + i] = (uint32_t)l[0] | ((uint32_t)l[1] << 8) | ((uint32_t)l[2] << 16) | ((uint32_t)l[3] << 24);
    }
    if (g.fmt == FMT_NF4) return (g.nf4_split_ok && (g.nf4_offset == 0 || has_xsum)) ? (int)FMT_NF4 : (int)FMT_NF4G;
    return (int)g.fmt;
}

uint32_t gemv_warp_smem_bytes(int fmt_index) {
    switch (fmt_index) {
        case FMT_BP4: return warp_smem<FMT_BP4>(1);
        case FMT_BP5: return warp_smem<FMT_BP5>(1);
        case FMT_BP6: return warp_smem<FMT_BP6>(1);
        case FMT_NF4: return warp_smem<FMT_NF4>(1);
        case FMT_NF3: return warp_smem<FMT_NF3>(1);
        case FMT_NF4G: return warp_smem<FMT_NF4G>(1);
        case FMT_NF5: return warp_smem<FMT_NF5>(1);
        case FMT_E8Q2: return warp_smem<FMT_E8Q2>(1);
        default: return 0;
    }
}

cudaError_t launch_gemv(cudaStream_t stream, const DeviceMatrix &m, const int8_t *xq, const float *xs,
                        const int32_t *xsum, uint32_t n_tok, float *out, size_t out_stride, int32_t *int_dots,
                        int sm_count, uint32_t *err_flag, uint32_t *launches, bool pdl) {
    if (launches) *launches = 0;
    if (n_tok == 0) return cudaSuccess;
    if (n_tok > 4) return cudaErrorNotSupported;
    const uint32_t nt = n_tok <= 1 ? 1 : n_tok <= 2 ? 2 : 4;
    GemvArgs a;
    const int fmt = fill_gemv_args(m, xsum != nullptr, a);
    if (fmt < 0) return cudaErrorNotSupported;
    a.xq = xq; a.xs = xs; a.xsum = xsum; a.out = out; a.int_dots = int_dots; a.err_flag = err_flag;
    a.out_stride = out_stride; a.pdl = pdl ? 1u : 0u; a.n_tok = n_tok;
    cudaError_t e;
    switch (fmt) {
        case FMT_BP4: e = launch_fmt<FMT_BP4>(stream, a, nt, sm_count); break;
        case FMT_BP5: e = launch_fmt<FMT_BP5>(stream, a, nt, sm_count); break;
        case FMT_BP6: e = launch_fmt<FMT_BP6>(stream, a, nt, sm_count); break;
        case FMT_NF4: e = launch_fmt<FMT_NF4>(stream, a, nt, sm_count); break;
        case FMT_NF4G: e = launch_fmt<FMT_NF4G>(stream, a, nt, sm_count); break;
        case FMT_NF3: e = launch_fmt<FMT_NF3>(stream, a, nt, sm_count); break;
        case FMT_NF5: e = launch_fmt<FMT_NF5>(stream, a, nt, sm_count); break;
        case FMT_E8Q2: e = launch_fmt<FMT_E8Q2>(stream, a, nt, sm_count); break;
        default: return cudaErrorNotSupported;
    }
    if (e == cudaSuccess && launches) *launches = 1;
    return e;
}

}  // namespace k2t
