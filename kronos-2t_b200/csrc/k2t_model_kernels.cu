// Per-token kernels of the dense decode step around the GEMVs (reference: RealLlamaEngine::forward_token,
// src/model/real_llm.rs:6485-6790): embedding, RMSNorm + rotation + int8 quantization, bias / qk-norm /
// RoPE / KV store / query quantization, split-KV decode attention over the int8 Hadamard cache,
// SwiGLU + rotation + quantization, argmax.  Everything position dependent reads the position from
// device memory so that one captured CUDA graph serves every decode step.
#include <algorithm>

#include "k2t_model_device.cuh"

namespace k2t {

__global__ void __launch_bounds__(256) embed_kernel(const EmbedArgs a) {
    const uint32_t lane = threadIdx.x & 31, c = blockIdx.x * 8 + (threadIdx.x >> 5);
    pdl_wait();
    pdl_trigger();
    if (c >= a.nc) return;
    const uint32_t tok = __ldcg(a.token + blockIdx.y);          // blockIdx.y = token of the batch
    float *hidden = a.hidden + (size_t)blockIdx.y * a.nc * 64;
    float v0, v1;
    if (a.embed_bf16 != nullptr) {
        const uint16_t *row = a.embed_bf16 + (size_t)tok * a.nc * 64 + (size_t)c * 64;
        v0 = bf16_bits_to_f32(row[2 * lane]);
        v1 = bf16_bits_to_f32(row[2 * lane + 1]);
    } else {   // tied: lm_head row, dequantized in the rotated domain, rotated back
        v0 = cell_value(a, tok, c, 2 * lane);
        v1 = cell_value(a, tok, c, 2 * lane + 1);
        warp_ifwht64(v0, v1, c, lane);
    }
    reinterpret_cast<float2 *>(hidden + (size_t)c * 64)[lane] = make_float2(v0, v1);
}

// ------------------------------------------------------------------------------------------------
// residual add + RMSNorm + FWHT-64 + int8  (rms_norm 9858-9898 + exec_hidden_proj!)
// ------------------------------------------------------------------------------------------------
// One CTA per token, 256 to 1024 threads (a warp per 64-value chunk where that fits).  hidden += delta (if given, written back), then the activation of
// the next projection.  The sum of squares follows dot_f32_neon (real_llm.rs:9736-9800) exactly: 16 fma
// accumulators over 16-element strides (lanes 0..15 of warp 0 run the 16 chains over the staged vector),
// combined (a0+a1)+(a2+a3) lane-wise and then pairwise - so inv_rms is the CPU value bit for bit.
//
// Tensor parallel (tp.tp > 1, delta given): delta is this rank's PARTIAL projection output; the ranks' partials are
// exchanged here, so the residual update needs no launch of its own.  Every element is stored into each peer's buffer
// as one 64-bit (call number, value) word; the receiver polls (bounded) the words of call e in the half e & 1 of its own
// buffer and adds the ranks' values in rank order.  A rank cannot be two calls ahead of another (it needs the others'
// words of call e + 1, sent after they finished call e), so two halves suffice; the call counter is shared with
// tp_exchange_kernel (k2t_tp.cu) and advanced by the last CTA of the launch to finish.
template <bool TP>
__global__ void __launch_bounds__(1024) rmsnorm_quant_kernel(float *__restrict__ hidden, const float *__restrict__ delta,
                                                            const float *__restrict__ w, uint32_t n, float eps,
                                                            int8_t *__restrict__ q, float *__restrict__ scales,
                                                            int32_t *__restrict__ sums, float *__restrict__ x_norm,
                                                            const TpLink tp, uint32_t *__restrict__ tp_done) {
    extern __shared__ float s_x[];           // n floats
    __shared__ float s_inv;
    __shared__ uint32_t s_epoch;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nc = n / 64;
    const uint32_t tok = blockIdx.x;
    {   // blockIdx.x = token of the batch: every per-token vector is contiguous
        const size_t t = blockIdx.x;
        hidden += t * n; q += t * n; scales += t * nc; sums += t * nc;
        if (delta != nullptr) delta += t * n;
        if (x_norm != nullptr) x_norm += t * n;
    }
    const uint32_t nthr = blockDim.x, nwarp = nthr >> 5;
    // The norm weights do not depend on the predecessor: they are staged in shared memory before the wait (the weights of a
    // layer are read once per token, so this load goes all the way to HBM).  The loops of this kernel stay rolled: its code
    // runs once per launch, and instruction fetch, not issue, is what a long straight-line kernel waits for.
    float *s_w = s_x + (TP ? 2 : 1) * n;
#pragma unroll 1
    for (uint32_t i = tid; i < n / 4; i += nthr) reinterpret_cast<float4 *>(s_w)[i] = __ldg(reinterpret_cast<const float4 *>(w) + i);
    pdl_wait();
    pdl_trigger();
    const bool exchange = TP && tp.tp > 1 && delta != nullptr;
    uint32_t epoch = 0;
    float *s_d = s_x + n;                    // exchange: the summed delta (the launcher doubles the shared memory)
    if (TP && exchange) {
        __shared__ int s_gave_up;            // set by the first thread whose polls ran out: nobody polls on after that
        if (tid == 0) {
            s_epoch = *tp.epoch + 1;
            // a context whose error word is already set (an earlier exchange gave up: a peer has left) does not wait again
            s_gave_up = __ldcg(tp.err) != 0 ? 1 : 0;
        }
        __syncthreads();
        epoch = s_epoch;
        const size_t half_off = (size_t)(epoch & 1u) * tp.tp * tp.ll_slot + (size_t)tok * n;
        // send: every element travels with the call number in ONE 64-bit store (value in the low half), so the receiver
        // needs no fence and no flag round trip - it polls the words themselves, and a 64-bit access is single-copy atomic
        for (uint32_t i = tid; i < n; i += nthr) {
            const unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(__ldcg(delta + i));
            for (uint32_t p = 0; p < tp.tp; ++p) {
                if (p == tp.rank) continue;
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(tp.peer_ll[p] + half_off + (size_t)tp.rank * tp.ll_slot + i), "l"(word) : "memory");
            }
        }
        // receive and add in rank order, ((v0 + v1) + v2) + ...: the same bits on every rank.  The wait is bounded per
        // kernel, not per word: a thread counts its misses over ALL its words (wait_polls of them, about a third of a
        // microsecond each, is the time a rank may lag behind: first launches, a host thread that was descheduled), and
        // once one thread has given up the others stop at their next look at the shared mark.
        int failed = *(volatile int *)&s_gave_up;
        uint32_t misses = 0;
        const uint32_t poll_limit = min(tp.wait_polls, 0x40000000u);
        const unsigned long long *mine = tp.peer_ll[tp.rank] + half_off;
        for (uint32_t i = tid; i < n; i += nthr) {
            float acc = 0.0f;
            for (uint32_t r = 0; r < tp.tp; ++r) {
                float v;
                if (r == tp.rank) {
                    v = __ldcg(delta + i);
                } else {
                    unsigned long long word = 0;
                    for (;;) {
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(mine + (size_t)r * tp.ll_slot + i) : "memory");
                        if ((uint32_t)(word >> 32) == epoch || failed) break;
                        if ((++misses & 63u) == 0) {          // every 64 misses: out of polls, or has somebody else given up?
                            if (misses > poll_limit) { *(volatile int *)&s_gave_up = 1; failed = 1; break; }
                            if (*(volatile int *)&s_gave_up) { failed = 1; break; }
                        }
                    }
                    v = __uint_as_float((uint32_t)word);
                }
                acc = r == 0 ? v : __fadd_rn(acc, v);
            }
            s_d[i] = acc;
        }
        if (__syncthreads_or(failed) && tid == 0) atomicExch(tp.err, 3u);
    }
#pragma unroll 1
    for (uint32_t i = tid; i < n / 4; i += nthr) {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(hidden) + i);
        if (delta != nullptr) {
            const float4 d = exchange ? reinterpret_cast<const float4 *>(s_d)[i] : __ldcg(reinterpret_cast<const float4 *>(delta) + i);
            v.x = __fadd_rn(v.x, d.x); v.y = __fadd_rn(v.y, d.y); v.z = __fadd_rn(v.z, d.z); v.w = __fadd_rn(v.w, d.w);
            reinterpret_cast<float4 *>(hidden)[i] = v;
        }
        reinterpret_cast<float4 *>(s_x)[i] = v;
    }
    __syncthreads();
    if (warp == 0) {
        float acc = 0.0f;
        if (lane < 16) {
#pragma unroll 16
            for (uint32_t i = lane; i < n; i += 16) { const float v = s_x[i]; acc = __fmaf_rn(v, v, acc); }
        }
        float t = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4));      // lanes 0..3: a0+a1, lanes 8..11: a2+a3
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 8));                // lanes 0..3: the four vector lanes
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 1));                // lane 0: v0+v1, lane 2: v2+v3
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 2));
        if (lane == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), eps)));
    }
    __syncthreads();
    const float inv = s_inv;
#pragma unroll 1
    for (uint32_t c = warp; c < nc; c += nwarp) {
        float2 v = reinterpret_cast<const float2 *>(s_x + (size_t)c * 64)[lane];
        const float2 ww = reinterpret_cast<const float2 *>(s_w + (size_t)c * 64)[lane];
        v.x = __fmul_rn(__fmul_rn(v.x, inv), ww.x);
        v.y = __fmul_rn(__fmul_rn(v.y, inv), ww.y);
        if (x_norm != nullptr) reinterpret_cast<float2 *>(x_norm + (size_t)c * 64)[lane] = v;
        warp_fwht64(v.x, v.y, c, lane);
        int q0, q1, sum;
        float sc;
        warp_quant64(v.x, v.y, q0, q1, sc, sum);
        reinterpret_cast<char2 *>(q + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (lane == 0) { scales[c] = sc; sums[c] = sum; }
    }
    if (exchange && tid == 0 && atomicAdd(tp_done, 1u) + 1u == gridDim.x) {       // every CTA of the launch has read the counter
        *tp_done = 0;
        *tp.epoch = epoch;
    }
}

// ------------------------------------------------------------------------------------------------
// sparse-MoE FFN pieces (SparseMoeRuntime::forward_layer_single, sparse_moe.rs:961-1084)
// ------------------------------------------------------------------------------------------------
// The scalar paths of the reference call the platform expf; the correctly rounded value stands in for it here
// as in the CPU restatement these kernels are compared with.
__device__ __forceinline__ float exp_cr(float x) { return (float)exp((double)x); }

// Router.  Logits in the accumulator order of dot_f32_moe_neon (16 fma lanes over 16-element strides, (a0+a1)+(a2+a3),
// pairwise): half a warp per expert, eight experts per CTA, so the router matrix streams through many SMs at once (one
// CTA took 65 us for 128 experts of 2048).  The CTA that finishes last (device counter) does the small sequential part:
// softmax over all experts with the sum in expert order, top-k by rank (score descending, the earlier expert first among
// equals - what select_topk_by_score's strict '>' insertion produces), optional renormalisation in that order, sort by id.
constexpr uint32_t ROUTER_THREADS = 128, ROUTER_MAX_EXPERTS = 256, ROUTER_MAX_TOPK = 32;
constexpr uint32_t ROUTER_EXPERTS_PER_CTA = ROUTER_THREADS / 16;
__global__ void __launch_bounds__(ROUTER_THREADS) moe_router_kernel(RouterArgs a) {
    extern __shared__ __align__(128) float s_dyn[];      // x [hidden], then (staged form) the CTA's eight router rows [8][hidden + 16]
    float *s_xr = s_dyn;
    {   // blockIdx.y = token of the batch
        const size_t t = blockIdx.y;
        a.x += t * a.hidden; a.logits += t * a.n_experts; a.done += t; a.route_ids += t * a.route_stride; a.route_w += t * a.route_stride;
    }
    __shared__ float s_z[ROUTER_MAX_EXPERTS];
    __shared__ float s_sel_w[ROUTER_MAX_TOPK];
    __shared__ uint32_t s_sel_e[ROUTER_MAX_TOPK];
    __shared__ float s_max;
    __shared__ uint32_t s_last;
    __shared__ __align__(8) uint64_t s_bar;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, half = lane >> 4, l16 = lane & 15;
    // The router rows are weights: the CTA's eight rows are requested (one bulk copy each) BEFORE the dependency wait, so the
    // megabyte of router weights of a layer streams in while the norm kernel in front still runs.  (Read by the lanes from
    // global memory after the wait, 16 loads in flight per lane, the whole grid had 128 KB in flight: 15 us per layer for
    // 128 experts of 2048.)  staged = 0: the rows do not fit shared memory, the lanes read them from global memory.
    const uint32_t row_pitch = a.hidden + 16;             // floats: the two half-warps of a warp read different banks
    const uint32_t e0 = blockIdx.x * ROUTER_EXPERTS_PER_CTA;
    const uint32_t n_mine = e0 < a.n_experts ? min(ROUTER_EXPERTS_PER_CTA, a.n_experts - e0) : 0;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&s_bar);
    if (a.staged && tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        fence_proxy_async();
        mbar_expect_tx(bar, n_mine * a.hidden * 4);
        for (uint32_t j = 0; j < n_mine; ++j)
            bulk_g2s((uint32_t)__cvta_generic_to_shared(s_dyn + a.hidden + (size_t)j * row_pitch), a.w + (size_t)(e0 + j) * a.hidden, a.hidden * 4, bar);
    }
    // No early release of the successor: it is the expert-batched GEMV, which cannot request a byte before it has read the
    // routes this kernel writes, so its CTAs would only sit on the SMs (and slow the warps running there) until then.
    pdl_wait();
    {   // x: 16-byte loads, four in flight per thread (one load per loop trip cost an L2 round trip each)
        const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
        const uint32_t n4 = a.hidden / 4;
        uint32_t i = tid;
        for (; i + 3 * ROUTER_THREADS < n4; i += 4 * ROUTER_THREADS) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcg(x4 + i + u * ROUTER_THREADS);
#pragma unroll
            for (int u = 0; u < 4; ++u) reinterpret_cast<float4 *>(s_xr)[i + u * ROUTER_THREADS] = v[u];
        }
        for (; i < n4; i += ROUTER_THREADS) reinterpret_cast<float4 *>(s_xr)[i] = __ldcg(x4 + i);
    }
    __syncthreads();
    bool copy_failed = false;
    if (a.staged && n_mine > 0) {
        uint32_t ok = 0;
        for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) ok = mbar_try_wait(bar, 0);
        copy_failed = !ok;
    }
    {
        const uint32_t e = e0 + warp * 2 + half;
        float acc = 0.0f;
        if (e < a.n_experts && !copy_failed) {
            if (a.staged) {
                const float *row = s_dyn + a.hidden + (size_t)(warp * 2 + half) * row_pitch;
#pragma unroll 16
                for (uint32_t i = l16; i < a.hidden; i += 16) acc = __fmaf_rn(row[i], s_xr[i], acc);
            } else {
                const float *row = a.w + (size_t)e * a.hidden;
#pragma unroll 16
                for (uint32_t i = l16; i < a.hidden; i += 16) acc = __fmaf_rn(__ldg(row + i), s_xr[i], acc);
            }
        }
        float t = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4));      // within each half: lanes 0..3 and 8..11
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 8));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 1));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 2));
        if (l16 == 0 && e < a.n_experts) a.logits[e] = a.bias != nullptr ? __fadd_rn(t, __ldg(a.bias + e)) : t;
    }
    if (__syncthreads_or(copy_failed) && tid == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(a.done, 1u) + 1u == gridDim.x ? 1u : 0u;       // per token: its own counter
    __syncthreads();
    if (s_last == 0) return;
    __threadfence();
    if (tid == 0) *a.done = 0;               // ready for the next launch (launches of a stream do not overlap here)
    for (uint32_t e = tid; e < a.n_experts; e += ROUTER_THREADS) s_z[e] = __ldcg(a.logits + e);
    __syncthreads();
    if (warp == 0) {
        float m = -INFINITY;
        for (uint32_t e = lane; e < a.n_experts; e += 32) m = fmaxf(m, s_z[e]);
        m = warp_max(m);
        if (lane == 0) s_max = m;
    }
    __syncthreads();
    // scores: softmax numerators (normalised below), sigmoid values, or the raw logits (top-k softmax)
    for (uint32_t e = tid; e < a.n_experts; e += ROUTER_THREADS) {
        if (a.scoring == 0) s_z[e] = exp_cr(__fsub_rn(s_z[e], s_max));
        else if (a.scoring == 2) s_z[e] = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_cr(-s_z[e])));
    }
    __syncthreads();
    if (a.scoring == 0) {
        if (tid == 0) {
            float sum = 0.0f;
            for (uint32_t e = 0; e < a.n_experts; ++e) sum = __fadd_rn(sum, s_z[e]);
            s_max = sum > 0.0f ? __fdiv_rn(1.0f, sum) : __fdiv_rn(1.0f, (float)a.n_experts);
        }
        __syncthreads();
        const float inv_all = s_max;
        for (uint32_t e = tid; e < a.n_experts; e += ROUTER_THREADS) s_z[e] = __fmul_rn(s_z[e], inv_all);
        __syncthreads();
    }
    const uint32_t k = min(min(a.top_k, a.n_experts), ROUTER_MAX_TOPK);
    // Non-finite scores (a NaN ranks before nothing and after nothing) can leave ranks unassigned: every slot starts as
    // a valid route (expert i, weight 0), so the expert kernels never see an id outside [0, n_experts).
    if (tid < k) { s_sel_e[tid] = tid; s_sel_w[tid] = 0.0f; }
    __syncthreads();
    for (uint32_t e = tid; e < a.n_experts; e += ROUTER_THREADS) {       // rank of expert e in the descending order
        const float sc = s_z[e];
        uint32_t rank = 0;
        for (uint32_t j = 0; j < a.n_experts; ++j) {
            const float sj = s_z[j];
            rank += (sj > sc || (sj == sc && j < e)) ? 1u : 0u;
        }
        if (rank < k) { s_sel_e[rank] = e; s_sel_w[rank] = sc; }
    }
    __syncthreads();
    if (tid == 0) {
        // in place in shared memory (k is small; private arrays indexed by loop variables would live in local memory)
        uint32_t *ids = s_sel_e;
        float *w = s_sel_w;
        if (a.scoring == 1) {                 // k-way softmax over the selected logits, in selection order
            float max_z = -INFINITY, sum = 0.0f;
            for (uint32_t i = 0; i < k; ++i) max_z = fmaxf(max_z, w[i]);
            for (uint32_t i = 0; i < k; ++i) { w[i] = exp_cr(__fsub_rn(w[i], max_z)); sum = __fadd_rn(sum, w[i]); }
            const float inv = sum > 0.0f ? __fdiv_rn(1.0f, sum) : __fdiv_rn(1.0f, (float)k);
            for (uint32_t i = 0; i < k; ++i) w[i] = __fmul_rn(w[i], inv);
        } else if (a.norm_topk) {
            float top_sum = 0.0f;
            for (uint32_t i = 0; i < k; ++i) top_sum = __fadd_rn(top_sum, w[i]);
            if (top_sum > 0.0f) { const float inv_top = __fdiv_rn(1.0f, top_sum); for (uint32_t i = 0; i < k; ++i) w[i] = __fmul_rn(w[i], inv_top); }
        }
        for (uint32_t i = 1; i < k; ++i) {
            const uint32_t ce = ids[i]; const float cw = w[i];
            uint32_t j = i;
            while (j > 0 && ids[j - 1] > ce) { ids[j] = ids[j - 1]; w[j] = w[j - 1]; --j; }
            ids[j] = ce; w[j] = cw;
        }
        for (uint32_t i = 0; i < k; ++i) { a.route_ids[i] = min(ids[i], a.n_experts - 1u); a.route_w[i] = w[i]; }
    }
}

// SwiGLU of the routed experts' gate_up outputs [slot][2 * d_ff] (gate = rows [0, d_ff), up = the rest), chunk by chunk
// with the scalar-path exp, then rotation (chunk index c) + int8: the activation of each expert's down projection.
__global__ void __launch_bounds__(256) expert_swiglu_quant_kernel(const float *__restrict__ gate_up, uint32_t d_ff,
                                                                  int8_t *__restrict__ q, float *__restrict__ scales,
                                                                  int32_t *__restrict__ sums) {
    const uint32_t lane = threadIdx.x & 31, c = blockIdx.x * 8 + (threadIdx.x >> 5), nc = d_ff / 64;
    pdl_wait();                // the successor (an expert-batched GEMV) is released when this kernel's CTAs exit, see moe_router_kernel
    if (c >= nc) return;
    const size_t slot = blockIdx.y;
    gate_up += slot * 2 * d_ff; q += slot * d_ff; scales += slot * nc; sums += slot * nc;
    const float2 g = __ldcg(reinterpret_cast<const float2 *>(gate_up + (size_t)c * 64) + lane);
    const float2 u = __ldcg(reinterpret_cast<const float2 *>(gate_up + d_ff + (size_t)c * 64) + lane);
    float x0 = __fmul_rn(__fdiv_rn(g.x, __fadd_rn(1.0f, exp_cr(-g.x))), u.x);
    float x1 = __fmul_rn(__fdiv_rn(g.y, __fadd_rn(1.0f, exp_cr(-g.y))), u.y);
    warp_fwht64(x0, x1, c, lane);
    int q0, q1, sum;
    float sc;
    warp_quant64(x0, x1, q0, q1, sc, sum);
    reinterpret_cast<char2 *>(q + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
    if (lane == 0) { scales[c] = sc; sums[c] = sum; }
}

// out[i] = 0; for every route in ascending expert order: out[i] += w * expert_out[slot][i]   (separate multiply and add).
// Expert parallelism (owned != null): only the routes whose expert this rank holds (owned[e] != null) - a partial sum.
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *__restrict__ expert_out, const float *__restrict__ route_w,
                                                          uint32_t n_slot, uint32_t n, float *__restrict__ out,
                                                          const uint32_t *__restrict__ route_ids, const uint8_t *const *__restrict__ owned,
                                                          uint32_t n_experts, uint32_t route_stride,
                                                          const float *__restrict__ base, const float *__restrict__ base_scale) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    {   // blockIdx.y = token of the batch: its n_slot expert outputs, its routes, its output row
        const size_t t = blockIdx.y;
        expert_out += t * n_slot * n; route_w += t * route_stride; route_ids += t * route_stride; out += t * n;
        if (base != nullptr) base += t * n;
        if (base_scale != nullptr) base_scale += t;
    }
    pdl_wait();
    pdl_trigger();
    if (i >= n) return;
    // the shared expert's output comes first (SharedMoeExpert::forward_single writes `out`, the routed experts add to it),
    // scaled by its gate unless that is 1 within f32::EPSILON (sparse_moe.rs:307-311)
    float acc = 0.0f;
    if (base != nullptr) {
        acc = __ldcg(base + i);
        if (base_scale != nullptr) {
            const float sc = __ldcg(base_scale);
            if (fabsf(__fsub_rn(sc, 1.0f)) > 1.1920929e-07f) acc = __fmul_rn(acc, sc);
        }
    }
    for (uint32_t s = 0; s < n_slot; ++s) {
        if (owned != nullptr && (__ldcg(route_ids + s) >= n_experts || owned[__ldcg(route_ids + s)] == nullptr)) continue;
        acc = __fadd_rn(acc, __fmul_rn(__ldcg(route_w + s), __ldcg(expert_out + (size_t)s * n + i)));
    }
    out[i] = acc;
}

// ------------------------------------------------------------------------------------------------
// bias + qk-norm + RoPE + KV store + query quantization  (6609-6650, 8139-8178, 8303-8365, 9287-9326)
// ------------------------------------------------------------------------------------------------
// One warp per head of the fused qkv vector: heads [0, n_q) are queries, then n_kv keys, then n_kv values.
// Keys/values go to the int8 cache at position *pos; queries are rotated and quantized the same way
// (one scale per head) for the attention kernel.
__global__ void __launch_bounds__(128) qkv_post_kernel(const QkvPostArgs a) {
    __shared__ float s_head[4][128];
    __shared__ float s_qv[4][64], s_qc[4][64];     // NF4 quantizer scratch per warp
    __shared__ uint8_t s_qi[4][64];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t head = blockIdx.x * 4 + warp, hd = a.head_dim, half = hd / 2;
    pdl_wait();
    pdl_trigger();
    if (head >= a.n_q + 2 * a.n_kv) return;
    const uint32_t tok = blockIdx.y;             // token of the batch: its own fused qkv vector, position and query slots
    const uint32_t pos = __ldcg(a.pos) + a.pos_offset + tok;
    const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv;
    float *sh = s_head[warp];
    const float *src = a.qkv + (size_t)tok * (a.n_q + 2 * a.n_kv) * hd + (size_t)head * hd;
    for (uint32_t i = lane; i < hd; i += 32) {
        float v = __ldcg(src + i);
        if (a.bias != nullptr) v = __fadd_rn(v, a.bias[(size_t)head * hd + i]);
        sh[i] = v;
    }
    __syncwarp();
    const float *norm_w = is_q ? a.q_norm : (is_k ? a.k_norm : nullptr);
    const float *rope = a.rope + (size_t)pos * hd;
    auto do_rope = [&]() {
        for (uint32_t i = lane; i < half; i += 32) {
            const float x0 = sh[i], x1 = sh[half + i], c = rope[i], s = rope[half + i];
            sh[i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            sh[half + i] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
        }
        __syncwarp();
    };
    auto do_norm = [&]() {
        // dot_f32_neon order (16 fma accumulators, (a0+a1)+(a2+a3), pairwise), as in rmsnorm_quant_kernel
        float ss = 0.0f;
        if (lane < 16)
            for (uint32_t i = lane; i < hd; i += 16) ss = __fmaf_rn(sh[i], sh[i], ss);
        ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 4));
        ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 8));
        ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 1));
        ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 2));
        ss = __shfl_sync(0xffffffffu, ss, 0);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, __fdiv_rn(1.0f, (float)hd)), a.eps)));
        for (uint32_t i = lane; i < hd; i += 32) sh[i] = __fmul_rn(__fmul_rn(sh[i], inv), norm_w[i]);
        __syncwarp();
    };
    if (is_q || is_k) {
        if (a.qk_norm_after_rope) do_rope();
        if (norm_w != nullptr) do_norm();
        if (!a.qk_norm_after_rope) do_rope();
    }
    // rotate (block index = block within the head) and quantize with one scale for the whole head
    const uint32_t nb = hd / 64;
    float v0[2], v1[2], mx = 0.0f;
    for (uint32_t b = 0; b < nb; ++b) {
        v0[b] = sh[b * 64 + 2 * lane];
        v1[b] = sh[b * 64 + 2 * lane + 1];
        warp_fwht64(v0[b], v1[b], b, lane);
        mx = fmaxf(mx, fmaxf(fabsf(v0[b]), fabsf(v1[b])));
    }
    if (!is_q && a.kv_bits == 4) {       // NF4 cache entry: packed indices + one bf16 scale per 64 values (store_hadamard_q4_head_raw)
        const uint32_t kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
        const size_t slot = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq + a.ring.slot_of_pos(pos);
        uint8_t *row = reinterpret_cast<uint8_t *>(is_k ? a.k_q8 : a.v_q8) + slot * (hd / 2);
        uint16_t *sc = reinterpret_cast<uint16_t *>(is_k ? a.k_scale : a.v_scale) + slot * nb;
        for (uint32_t b = 0; b < nb; ++b) {
            uint16_t sb;
            const uint32_t byte = warp_quant64_q4(v0[b], v1[b], lane, s_qv[warp], s_qc[warp], s_qi[warp], &sb);
            row[b * 32 + lane] = (uint8_t)byte;
            if (lane == 0) sc[b] = sb;
        }
        return;
    }
    mx = warp_max(mx);
    int8_t *dst_q;
    float *dst_s;
    if (is_q) { dst_q = a.q_i8 + ((size_t)tok * a.n_q + head) * hd; dst_s = a.q_scale + (size_t)tok * a.n_q + head; }
    else {
        const uint32_t kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
        const size_t slot = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq + a.ring.slot_of_pos(pos);
        dst_q = (is_k ? a.k_q8 : a.v_q8) + slot * hd;
        dst_s = (is_k ? a.k_scale : a.v_scale) + slot;
    }
    const bool zero = mx <= 1.1920929e-07f;
    const float inv = zero ? 0.0f : __fdiv_rn(127.0f, mx);
    // value rows also go to the block-transposed copy the value chains read ([position / 16][dimension][16], sign flipped)
    int8_t *vt = nullptr;
    if (!is_q && !is_k && a.v_t != nullptr) {
        const uint32_t kvh = head - a.n_q - a.n_kv, row = a.ring.slot_of_pos(pos);
        vt = a.v_t + ((size_t)a.layer * a.n_kv + kvh) * a.max_seq * hd + (size_t)(row / 16) * hd * 16 + row % 16;
    }
    for (uint32_t b = 0; b < nb; ++b) {
        const int q0 = zero ? 0 : __float2int_rn(__fmul_rn(v0[b], inv)), q1 = zero ? 0 : __float2int_rn(__fmul_rn(v1[b], inv));
        reinterpret_cast<char2 *>(dst_q + b * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (vt != nullptr) {
            vt[(b * 64 + 2 * lane) * 16] = (int8_t)(q0 ^ 0x80);
            vt[(b * 64 + 2 * lane + 1) * 16] = (int8_t)(q1 ^ 0x80);
        }
    }
    if (lane == 0) *dst_s = zero ? 0.0f : __fdiv_rn(mx, 127.0f);
}

// v_t <- v_q8 for whole heads: thread = four dimensions of one cached row
__global__ void __launch_bounds__(256) vt_rebuild_kernel(const int8_t *__restrict__ v_q8, int8_t *__restrict__ v_t, size_t n_words, uint32_t rows_per_head,
                                                         uint32_t hd) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n_words; i += (size_t)gridDim.x * 256) {
        const size_t slot = i / (hd / 4), head = slot / rows_per_head;
        const uint32_t d0 = (uint32_t)(i % (hd / 4)) * 4, row = (uint32_t)(slot % rows_per_head);
        const uint32_t w = *reinterpret_cast<const uint32_t *>(v_q8 + slot * hd + d0) ^ 0x80808080u;
        int8_t *dst = v_t + head * rows_per_head * hd + (size_t)(row / 16) * hd * 16 + row % 16;
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[(d0 + k) * 16] = (int8_t)((w >> (8 * k)) & 0xffu);
    }
}
cudaError_t launch_vt_rebuild(cudaStream_t s, const int8_t *v_q8, int8_t *v_t, size_t heads, uint32_t rows_per_head, uint32_t head_dim) {
    const size_t n_words = heads * rows_per_head * (head_dim / 4);
    const unsigned grid = (unsigned)std::min<size_t>((n_words + 255) / 256, 148 * 16);
    return launch_kernel(vt_rebuild_kernel, dim3(grid), dim3(256), 0, s, false, v_q8, v_t, n_words, rows_per_head, head_dim);
}

// ------------------------------------------------------------------------------------------------
// split-KV decode attention over the Hadamard cache (causal_gqa_group_q8, 8471-8594; NF4: causal_gqa_group_q4_or_window)
// ------------------------------------------------------------------------------------------------
// One warp per (kv head, split).  The warp streams its positions through a ring of 32-position tiles in shared
// memory: lane 0 issues four bulk copies per tile (key rows, value rows and their scales are contiguous runs of the
// cache) that complete on the tile's mbarrier, several tiles ahead of the arithmetic, so the kernel is bound by the
// copy engine's bandwidth and not by one load latency per position.  A ragged last tile, or scale rows that do not
// start on 16 bytes, are copied by the lanes with plain loads instead.
// Scores: lane = position (its key row against the group's int8 queries with dp4a; the 16-byte vectors of a row are
// visited in a lane-dependent rotation so that a quarter-warp reads eight different bank groups - integer sums do
// not depend on the order); values: lane = four dimensions, the two half-warps take alternate positions.
// Used for contexts longer than ATTN_EXACT_CTX positions.  Scores (and so the maximum) are the CPU's bit for bit.
// Softmax is the online form; partial (max, sum, out) per split are merged by attn_finish_kernel.  Sums run in a
// different order than the CPU's position-ascending chains: the output agrees to fp32 rounding, not bit for bit.
template <int HD, bool KV4>
struct SplitTile {
    static constexpr uint32_t ROW = KV4 ? HD / 2 : HD;             // bytes of a cached key / value row
    static constexpr uint32_t SC = KV4 ? (HD / 64) * 2 : 4;        // scale bytes per position (bf16 per 64 values / fp32)
    static constexpr uint32_t K_OFF = 0, V_OFF = 32 * ROW, KS_OFF = 64 * ROW, VS_OFF = 64 * ROW + 32 * SC;
    static constexpr uint32_t BYTES = 64 * ROW + 64 * SC;
    static constexpr uint32_t NST = BYTES > 8000 ? 3 : 4;          // tiles in flight per warp
    static constexpr uint32_t WARP_BYTES = 64 + NST * BYTES;       // mbarriers first
};
template <int HD, bool KV4> constexpr size_t attn_partial_smem() { return 4 * SplitTile<HD, KV4>::WARP_BYTES; }

template <int HD, bool KV4>
__global__ void __launch_bounds__(128) attn_partial_kernel(const AttnArgs a) {
    using Tile = SplitTile<HD, KV4>;
    constexpr int QW = HD / 4;            // int32 words per query row
    constexpr int NB = HD / 64;
    constexpr uint32_t ROW = Tile::ROW, SC = Tile::SC, NST = Tile::NST, NV = ROW / 16;
    extern __shared__ __align__(128) uint8_t dyn_smem[];
    __shared__ __align__(16) int s_q[4][8][QW];       // [warp][query in group][words] (NF4 cache: gathered in the packed column order)
    __shared__ float s_p[4][8][KV4 ? NB : 1][32];     // value weights of the current 32 positions (per 64-value group for NF4)
    __shared__ float s_cb[16];            // NF4 centroids
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t split = blockIdx.x * 4 + warp, kvh = blockIdx.y;
    pdl_wait();
    pdl_trigger();
    if (split >= a.n_split) return;
    const uint32_t ctx = __ldcg(a.pos) + a.pos_offset + 1, G = a.group;
    if (ctx <= ATTN_EXACT_CTX) return;     // short contexts are computed in the CPU's order by attn_finish_kernel
    const uint32_t per = split_span(ctx, a.n_split);
    const uint32_t t_lo = min(ctx, split * per), t_hi = min(ctx, t_lo + per);
    const uint32_t n_tiles = (t_hi - t_lo + 31) / 32;
    const size_t slot0 = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq;
    const uint8_t *K = reinterpret_cast<const uint8_t *>(a.k_q8) + slot0 * ROW, *V = reinterpret_cast<const uint8_t *>(a.v_q8) + slot0 * ROW;
    const uint8_t *KS = reinterpret_cast<const uint8_t *>(a.k_scale) + slot0 * SC, *VS = reinterpret_cast<const uint8_t *>(a.v_scale) + slot0 * SC;
    uint8_t *wsm = dyn_smem + (size_t)warp * Tile::WARP_BYTES;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(wsm);
    uint8_t *stages = wsm + 64;
    if (lane == 0) {
        for (uint32_t st = 0; st < NST; ++st) mbar_init(bar0 + 8 * st, 1);
        fence_mbar_init();
    }
    __syncwarp();
    // bulk copies want 16-byte aligned sources: rows always are, the scale runs only for some cache lengths
    const bool sc_aligned = ((reinterpret_cast<uintptr_t>(KS + (size_t)t_lo * SC) | reinterpret_cast<uintptr_t>(VS + (size_t)t_lo * SC)) & 15u) == 0;
    auto tile_is_bulk = [&](uint32_t i) { return sc_aligned && t_lo + 32 * i + 32 <= t_hi; };
    auto fill = [&](uint32_t i) {         // tile i of the split into stage i % NST (every earlier read of that stage is done)
        const uint32_t t0 = t_lo + 32 * i, n = min(32u, t_hi - t0);
        uint8_t *st = stages + (i % NST) * Tile::BYTES;
        if (tile_is_bulk(i)) {
            if (lane == 0) {
                const uint32_t bar = bar0 + 8 * (i % NST), dst = (uint32_t)__cvta_generic_to_shared(st);
                fence_proxy_async();
                mbar_expect_tx(bar, Tile::BYTES);
                bulk_g2s(dst + Tile::K_OFF, K + (size_t)t0 * ROW, 32 * ROW, bar);
                bulk_g2s(dst + Tile::V_OFF, V + (size_t)t0 * ROW, 32 * ROW, bar);
                bulk_g2s(dst + Tile::KS_OFF, KS + (size_t)t0 * SC, 32 * SC, bar);
                bulk_g2s(dst + Tile::VS_OFF, VS + (size_t)t0 * SC, 32 * SC, bar);
            }
        } else {
            for (uint32_t v = lane; v < n * NV; v += 32) {
                reinterpret_cast<uint4 *>(st + Tile::K_OFF)[v] = __ldcg(reinterpret_cast<const uint4 *>(K + (size_t)t0 * ROW) + v);
                reinterpret_cast<uint4 *>(st + Tile::V_OFF)[v] = __ldcg(reinterpret_cast<const uint4 *>(V + (size_t)t0 * ROW) + v);
            }
            for (uint32_t v = lane; v < n * (SC / 2); v += 32) {
                reinterpret_cast<uint16_t *>(st + Tile::KS_OFF)[v] = __ldcg(reinterpret_cast<const uint16_t *>(KS + (size_t)t0 * SC) + v);
                reinterpret_cast<uint16_t *>(st + Tile::VS_OFF)[v] = __ldcg(reinterpret_cast<const uint16_t *>(VS + (size_t)t0 * SC) + v);
            }
        }
    };
    for (uint32_t i = 0; i < NST && i < n_tiles; ++i) fill(i);

    if (KV4 && lane < 16) s_cb[lane] = NF4_KV_CENTROIDS[lane];      // every warp writes the same values
    for (uint32_t i = lane; i < G * QW; i += 32) {
        const int8_t *qb = a.q_i8 + (size_t)(kvh * G + i / QW) * HD;
        const uint32_t wi = i % QW;
        if (KV4) {        // packed word w of a 64-value group holds columns (c, 16+c, c+1, 16+c+1 | c+2, ...) of a 32-column half
            const uint32_t g = wi / 16, w = (wi % 16) / 2, u = wi % 2;
            const int8_t *p = qb + g * 64 + (w / 4) * 32 + 4 * (w % 4);
            s_q[warp][i / QW][wi] = (int)((uint32_t)(uint8_t)__ldcg(p + 2 * u) | ((uint32_t)(uint8_t)__ldcg(p + 16 + 2 * u) << 8) |
                                          ((uint32_t)(uint8_t)__ldcg(p + 2 * u + 1) << 16) | ((uint32_t)(uint8_t)__ldcg(p + 16 + 2 * u + 1) << 24));
        } else {
            s_q[warp][i / QW][wi] = __ldcg(reinterpret_cast<const int *>(qb) + wi);
        }
    }
    __syncwarp();
    float qas[8], m[8], l[8], o[8][HD / 16];
    // value phase mapping: 16 lanes x 4 dims cover 64 dims; for HD = 128 each lane owns two such groups
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        qas[g] = g < (int)G ? __fmul_rn(__ldcg(a.q_scale + kvh * G + g), a.attn_scale) : 0.0f;
        m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int d = 0; d < HD / 16; ++d) o[g][d] = 0.0f;
    }
    const uint32_t hw = lane >> 4, dl = lane & 15;   // half-warp, dim group
    const uint32_t rot = (lane * NV / 8) % NV;       // vector rotation of this lane's key row
    uint32_t phase = 0;                              // parity bit per stage
    bool failed = false;
    for (uint32_t i = 0; i < n_tiles && !failed; ++i) {
        const uint32_t t0 = t_lo + 32 * i, stage = i % NST;
        const uint8_t *st = stages + stage * Tile::BYTES;
        if (tile_is_bulk(i)) {             // bounded wait for the tile
            uint32_t ok = 0;
            for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) ok = mbar_try_wait(bar0 + 8 * stage, (phase >> stage) & 1u);
            phase ^= 1u << stage;
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
                failed = true;
                break;
            }
        } else {
            __syncwarp();                  // the lanes' own stores
        }
        const uint32_t t = t0 + lane;
        const bool on = t < t_hi;
        const uint32_t tile0 = t & ~255u, tile_n = min(ctx, tile0 + 256u) - tile0;
        const bool grouped = t - tile0 < (tile_n & ~7u);
        float kst[KV4 ? NB : 1], vst[KV4 ? NB : 1];
        if (KV4) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                kst[b] = on ? bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(st + Tile::KS_OFF)[lane * NB + b]) : 0.0f;
                vst[b] = on ? bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(st + Tile::VS_OFF)[lane * NB + b]) : 0.0f;
            }
        } else {
            kst[0] = on ? reinterpret_cast<const float *>(st + Tile::KS_OFF)[lane] : 0.0f;
            vst[0] = on ? reinterpret_cast<const float *>(st + Tile::VS_OFF)[lane] : 0.0f;
        }
        // integer dots of position t with every query of the group
        int up[8][KV4 ? NB : 1], dn[8][KV4 ? NB : 1];
#pragma unroll
        for (int g = 0; g < 8; ++g)
#pragma unroll
            for (int b = 0; b < (KV4 ? NB : 1); ++b) { up[g][b] = 0; dn[g][b] = 0; }
        const uint4 *krow = reinterpret_cast<const uint4 *>(st + Tile::K_OFF + lane * ROW);
#pragma unroll
        for (uint32_t v = 0; v < NV; ++v) {
            const uint32_t vv = (v + rot) & (NV - 1);
            const uint4 kk = krow[vv];
            if (KV4) {
                const bool second = NB == 2 && vv >= NV / 2;      // the 64-value group this vector belongs to
                const uint32_t x[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if (g >= (int)G) break;
                    const int4 qa = *reinterpret_cast<const int4 *>(&s_q[warp][g][8 * vv]), qb = *reinterpret_cast<const int4 *>(&s_q[warp][g][8 * vv + 4]);
                    const int q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    int tu = 0, td = 0;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t y = x[c] ^ 0x88888888u;
                        tu = dp4a_us(prmt(NF4_KV_HI0, NF4_KV_HI1, y), q[2 * c], tu);
                        td = dp4a_us(prmt(NF4_KV_LO0, NF4_KV_LO1, x[c]), q[2 * c], td);
                        tu = dp4a_us(prmt(NF4_KV_HI0, NF4_KV_HI1, y >> 16), q[2 * c + 1], tu);
                        td = dp4a_us(prmt(NF4_KV_LO0, NF4_KV_LO1, x[c] >> 16), q[2 * c + 1], td);
                    }
                    if (NB == 2) {
                        up[g][0] += second ? 0 : tu; dn[g][0] += second ? 0 : td;
                        up[g][NB - 1] += second ? tu : 0; dn[g][NB - 1] += second ? td : 0;
                    } else {
                        up[g][0] += tu; dn[g][0] += td;
                    }
                }
            } else {
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if (g >= (int)G) break;
                    const int4 qq = *reinterpret_cast<const int4 *>(&s_q[warp][g][4 * vv]);
                    int d = up[g][0];
                    d = __dp4a((int)kk.x, qq.x, d); d = __dp4a((int)kk.y, qq.y, d); d = __dp4a((int)kk.z, qq.z, d); d = __dp4a((int)kk.w, qq.w, d);
                    up[g][0] = d;
                }
            }
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            if (g >= (int)G) break;
            float s = -INFINITY;
            if (KV4) {        // causal_gqa_group_q4_or_window: total += ((dot_b * ks_b) * q_s) per 64-value group
                if (on) {
                    s = 0.0f;
#pragma unroll
                    for (int b = 0; b < NB; ++b) s = __fadd_rn(s, __fmul_rn(__fmul_rn((float)(up[g][b] - dn[g][b]), kst[b]), qas[g]));
                }
            } else {
                // 256-position tiles: whole groups of 8 use dot*(ks*qas), the tile remainder (dot*ks)*qas (8992-9057)
                const int dot = up[g][0];
                s = !on ? -INFINITY
                  : grouped ? __fmul_rn((float)dot, __fmul_rn(kst[0], qas[g]))
                            : __fmul_rn(__fmul_rn((float)dot, kst[0]), qas[g]);
            }
            const float m_new = fmaxf(m[g], warp_max(s));
            const float corr = m[g] == -INFINITY ? 0.0f : exp_poly(m[g] - m_new);
            const float p = on ? exp_poly(s - m_new) : 0.0f;
            l[g] = __fmaf_rn(l[g], corr, warp_sum(p));
#pragma unroll
            for (int d = 0; d < HD / 16; ++d) o[g][d] *= corr;
            m[g] = m_new;
#pragma unroll
            for (int b = 0; b < (KV4 ? NB : 1); ++b) s_p[warp][g][b][lane] = __fmul_rn(p, vst[b]);     // weight of V row t
        }
        __syncwarp();
        // values: half-warp hw takes positions t0 + hw, t0 + hw + 2, ...
        const uint32_t n_here = min(32u, t_hi - t0);
        const uint8_t *vt = st + Tile::V_OFF;
#pragma unroll 4
        for (uint32_t j = hw; j < n_here; j += 2) {      // unrolled: the loads of four positions are in flight together
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float c0, c1, c2, c3;
                if (KV4) {    // dims 4 dl .. 4 dl + 3 of the group sit in one packed word: low nibbles for columns 0..15 of a half, high for 16..31
                    const uint32_t e = dl * 4, r = e % 32, shift = r < 16 ? 0u : 4u;
                    const uint32_t word = *reinterpret_cast<const uint32_t *>(vt + j * ROW + b * 32 + (e / 32) * 16 + (r % 16)) >> shift;
                    c0 = s_cb[word & 15u]; c1 = s_cb[(word >> 8) & 15u]; c2 = s_cb[(word >> 16) & 15u]; c3 = s_cb[(word >> 24) & 15u];
                } else {
                    // int8 -> fp32 without the conversion unit: 0x4B000000 | (b ^ 0x80) is the float 2^23 + 128 + (int8)b
                    const uint32_t v = *reinterpret_cast<const uint32_t *>(vt + j * ROW + b * 64 + dl * 4) ^ 0x80808080u;
                    c0 = __fsub_rn(__uint_as_float(prmt(v, 0x4B000000u, 0x7650u)), 8388736.0f);
                    c1 = __fsub_rn(__uint_as_float(prmt(v, 0x4B000000u, 0x7651u)), 8388736.0f);
                    c2 = __fsub_rn(__uint_as_float(prmt(v, 0x4B000000u, 0x7652u)), 8388736.0f);
                    c3 = __fsub_rn(__uint_as_float(prmt(v, 0x4B000000u, 0x7653u)), 8388736.0f);
                }
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if (g >= (int)G) break;
                    const float w = s_p[warp][g][KV4 ? b : 0][j];
                    o[g][4 * b + 0] = __fmaf_rn(c0, w, o[g][4 * b + 0]);
                    o[g][4 * b + 1] = __fmaf_rn(c1, w, o[g][4 * b + 1]);
                    o[g][4 * b + 2] = __fmaf_rn(c2, w, o[g][4 * b + 2]);
                    o[g][4 * b + 3] = __fmaf_rn(c3, w, o[g][4 * b + 3]);
                }
            }
        }
        __syncwarp();                      // the stage and the weights are free again
        if (i + NST < n_tiles) fill(i + NST);
    }
    if (failed) return;
    // combine the two half-warps and write the partial result
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        if (g >= (int)G) break;
        const uint32_t qh = kvh * G + g;
        float *po = a.part_o + ((size_t)qh * a.n_split + split) * HD;
#pragma unroll
        for (int d = 0; d < HD / 16; ++d) {
            const float other = __shfl_xor_sync(0xffffffffu, o[g][d], 16);
            if (hw == 0) po[(d / 4) * 64 + dl * 4 + (d % 4)] = o[g][d] + other;
        }
        if (lane == 0) { a.part_m[(size_t)qh * a.n_split + split] = m[g]; a.part_l[(size_t)qh * a.n_split + split] = l[g]; }
    }
}

// Finishes the attention of one query head (one CTA of HD threads, thread i = dimension i) and turns it
// into the int8 activation of o_proj.
//   context <= ATTN_EXACT_CTX: the whole head is computed here in the CPU's order (causal_gqa_group_q8,
//     8471-8594): scores, maximum, exp (polynomial body in groups of 4, correctly rounded exp for the
//     remainder), the 4-accumulator sum, then for every dimension the position-ascending fma chain over
//     the int8 values - bit for bit the CPU result; the split kernel above exits at once.
//   longer contexts: merges the split partials (sums in split order; fp32-rounding agreement).
// Then: inverse rotation (block index 0/1), forward rotation with the global chunk index
// qh*(hd/64)+b and quantization for o_proj (7059-7084).
constexpr uint32_t FINISH_THREADS = 256;     // also the largest split count the merge handles
template <int HD>
__global__ void __launch_bounds__(FINISH_THREADS) attn_finish_kernel(const AttnArgs a) {
    constexpr int NB = HD / 64, NG = FINISH_THREADS / HD;      // NG thread groups share the splits of a dimension
    __shared__ float s_w[FINISH_THREADS];
    __shared__ float s_part[NG][HD];
    __shared__ float s_red[FINISH_THREADS / 32], s_redl[FINISH_THREADS / 32];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    pdl_trigger();
    const uint32_t qh = blockIdx.x, ctx = __ldcg(a.pos) + a.pos_offset + 1;
    if (ctx <= ATTN_EXACT_CTX) return;         // those lengths belong to attn_fused_kernel
    const uint32_t per = split_span(ctx, a.n_split);
    const uint32_t used = (ctx + per - 1) / per;               // splits that hold positions (at most FINISH_THREADS)
    // thread s: weight of split s against the global maximum, and its share of the softmax denominator
    const float ms = tid < used ? __ldcg(a.part_m + (size_t)qh * a.n_split + tid) : -INFINITY;
    const float ls = tid < used ? __ldcg(a.part_l + (size_t)qh * a.n_split + tid) : 0.0f;
    float M = warp_max(ms);
    if (lane == 0) s_red[warp] = M;
    __syncthreads();
#pragma unroll
    for (uint32_t i = 0; i < FINISH_THREADS / 32; ++i) M = fmaxf(M, s_red[i]);
    const float wgt = tid < used ? exp_poly(ms - M) : 0.0f;
    s_w[tid] = wgt;
    const float lw = warp_sum(__fmul_rn(ls, wgt));
    if (lane == 0) s_redl[warp] = lw;
    __syncthreads();
    float L = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < FINISH_THREADS / 32; ++i) L = __fadd_rn(L, s_redl[i]);
    // group g of dimension d sums splits g, g + NG, ... (independent loads, one fma chain); the groups are added in order
    const uint32_t d = tid % HD, grp = tid / HD;
    float o = 0.0f;
    const float *po = a.part_o + (size_t)qh * a.n_split * HD + d;
#pragma unroll 16
    for (uint32_t sp = grp; sp < used; sp += NG) o = __fmaf_rn(__ldcg(po + (size_t)sp * HD), s_w[sp], o);
    s_part[grp][d] = o;
    __syncthreads();
    if (warp < NB) {
        const uint32_t b = warp;
        const float invL = __fdiv_rn(1.0f, L);
        float x0 = 0.0f, x1 = 0.0f;
#pragma unroll
        for (int g = 0; g < NG; ++g) { x0 = __fadd_rn(x0, s_part[g][b * 64 + 2 * lane]); x1 = __fadd_rn(x1, s_part[g][b * 64 + 2 * lane + 1]); }
        x0 = __fmul_rn(x0, invL); x1 = __fmul_rn(x1, invL);
        warp_ifwht64(x0, x1, b, lane);
        if (a.attn_out != nullptr) reinterpret_cast<float2 *>(a.attn_out + (size_t)qh * HD + b * 64)[lane] = make_float2(x0, x1);
        const uint32_t c = qh * NB + b;
        warp_fwht64(x0, x1, a.out_chunk0 + c, lane);
        int q0, q1, sum;
        float sc;
        warp_quant64(x0, x1, q0, q1, sc, sum);
        reinterpret_cast<char2 *>(a.out_q + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (lane == 0) { a.out_scales[c] = sc; a.out_sums[c] = sum; }
    }
}

// Contexts of up to ATTN_EXACT_CTX positions: bias / qk-norm / RoPE / KV store / attention / o_proj activation
// in one kernel, CTA q = query head q (attention_head_cta).  Longer contexts: returns at once, the split-KV
// kernels serve them.
__global__ void __launch_bounds__(ATTN_THREADS) attn_fused_kernel(const FusedAttnArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const bool early = a.early != 0;
    if (!early) pdl_wait();
    const uint32_t pos = __ldcg(a.pos) + a.pos_offset;
    if (pos + 1 > ATTN_EXACT_CTX) {
        if (early) pdl_wait();          // every kernel of the chain waits: completion of this one implies its predecessors'
        return;
    }
    attention_head_dispatch<true>(a, blockIdx.x, pos, attn_carve(smem, true), early ? 2 : 1);
}

// ------------------------------------------------------------------------------------------------
// SwiGLU + FWHT-64 + int8  (swiglu_activate_neon 9811-9842, then the down_proj activation)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_quant_kernel(const float *__restrict__ gate_up, uint32_t inter,
                                                           int8_t *__restrict__ q, float *__restrict__ scales,
                                                           int32_t *__restrict__ sums, float *__restrict__ dbg, uint32_t chunk0) {
    const uint32_t lane = threadIdx.x & 31, c = blockIdx.x * 8 + (threadIdx.x >> 5);
    const FwhtSigns sg = fwht_signs(chunk0 + c, lane);
    pdl_wait();
    pdl_trigger();
    if (c >= inter / 64) return;
    {   // blockIdx.y = token of the batch
        const size_t t = blockIdx.y;
        gate_up += t * 2 * inter; q += t * inter; scales += t * (inter / 64); sums += t * (inter / 64);
        if (dbg != nullptr) dbg += t * inter;
    }
    const float2 g = __ldcg(reinterpret_cast<const float2 *>(gate_up + (size_t)c * 64) + lane);
    const float2 u = __ldcg(reinterpret_cast<const float2 *>(gate_up + inter + (size_t)c * 64) + lane);
    float x0 = __fmul_rn(__fdiv_rn(g.x, __fadd_rn(1.0f, exp_poly(-g.x))), u.x);
    float x1 = __fmul_rn(__fdiv_rn(g.y, __fadd_rn(1.0f, exp_poly(-g.y))), u.y);
    if (dbg != nullptr) reinterpret_cast<float2 *>(dbg + (size_t)c * 64)[lane] = make_float2(x0, x1);
    warp_fwht64(x0, x1, sg, lane);
    int q0, q1, sum;
    float sc;
    warp_quant64(x0, x1, q0, q1, sc, sum);
    reinterpret_cast<char2 *>(q + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
    if (lane == 0) { scales[c] = sc; sums[c] = sum; }
}

// ------------------------------------------------------------------------------------------------
// greedy step: argmax (first maximum, argmax_scalar 9914-9924), record the token, advance the position
// ------------------------------------------------------------------------------------------------
// Many CTAs scan a slice of the logits each (a single CTA spent 12 - 25 us on 49K - 152K logits, one L2 round trip per
// thread and iteration); every CTA leaves its best (value, index) in `part`, and the CTA that finishes last (device
// counter) picks the winner among them - the first maximum, as a sequential scan would - and advances the step.
constexpr uint32_t ARGMAX_THREADS = 256, ARGMAX_MAX_CTAS = 256;
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_step_kernel(const float *__restrict__ logits, uint32_t n,
                                                                     uint32_t *__restrict__ token, uint32_t *__restrict__ pos,
                                                                     uint32_t *__restrict__ history, uint32_t *__restrict__ step,
                                                                     float *__restrict__ part_v, uint32_t *__restrict__ part_i,
                                                                     uint32_t *__restrict__ done) {
    __shared__ float s_v[ARGMAX_THREADS / 32];
    __shared__ uint32_t s_i[ARGMAX_THREADS / 32];
    __shared__ uint32_t s_last;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    pdl_wait();
    pdl_trigger();
    auto better = [](float v, uint32_t i, float bv2, uint32_t bi2) { return v > bv2 || (v == bv2 && i < bi2); };
    auto block_best = [&]() {            // best of the CTA in thread 0
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, m);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = bv; s_i[threadIdx.x >> 5] = bi; }
        __syncthreads();
        if (threadIdx.x == 0)
            for (uint32_t w = 1; w < ARGMAX_THREADS / 32; ++w)
                if (better(s_v[w], s_i[w], bv, bi)) { bv = s_v[w]; bi = s_i[w]; }
    };
    // slice of this CTA: contiguous, a multiple of 4 logits
    const uint32_t per = ((n + gridDim.x - 1) / gridDim.x + 3u) & ~3u;
    const uint32_t lo = min(n, blockIdx.x * per), hi = min(n, lo + per);
    for (uint32_t i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) {
        const float v = __ldcg(logits + i);
        if (v > bv) { bv = v; bi = i; }         // ascending i per thread: keeps the first maximum
    }
    block_best();
    if (threadIdx.x == 0) {
        part_v[blockIdx.x] = bv; part_i[blockIdx.x] = bi;
        __threadfence();
        s_last = atomicAdd(done, 1u) + 1u == gridDim.x ? 1u : 0u;
    }
    __syncthreads();
    if (s_last == 0) return;
    __threadfence();
    bv = -INFINITY; bi = 0xffffffffu;
    if (threadIdx.x < gridDim.x) { bv = __ldcg(part_v + threadIdx.x); bi = __ldcg(part_i + threadIdx.x); }
    __syncthreads();                            // s_v / s_i are reused
    block_best();
    if (threadIdx.x == 0) {
        *done = 0;                              // ready for the next launch
        if (bi == 0xffffffffu) bi = 0;          // all NaN / -inf: the scalar loop also returns 0
        *token = bi;
        const uint32_t st = __ldcg(step);
        if (history != nullptr) history[st] = bi;
        *step = st + 1;
        *pos = __ldcg(pos) + 1;
    }
}

// Keeps the stream busy for about `ns` nanoseconds of the global timer (bounded a second time by a poll count).
__global__ void delay_kernel(unsigned long long ns) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t i = 0; i < (1u << 24); ++i) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 >= ns) break;
        __nanosleep(200);
    }
}

__global__ void advance_pos_kernel(uint32_t *pos, uint32_t by) {
    pdl_wait();
    *pos = __ldcg(pos) + by;
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
cudaError_t launch_embed(cudaStream_t s, const EmbedArgs &a, uint32_t n_tok, bool pdl) {
    return launch_kernel(embed_kernel, dim3((a.nc + 7) / 8, n_tok), dim3(256), 0, s, pdl, a);
}
cudaError_t launch_rmsnorm_quant(cudaStream_t s, float *hidden, const float *delta, const float *w, uint32_t n, float eps,
                                 int8_t *q, float *scales, int32_t *sums, uint32_t n_tok, bool pdl) {
    return launch_rmsnorm_quant_x(s, hidden, delta, w, n, eps, q, scales, sums, nullptr, n_tok, pdl);
}
cudaError_t launch_moe_router(cudaStream_t s, const RouterArgs &a_in, bool pdl, uint32_t n_tok) {
    RouterArgs a = a_in;
    if (a.n_experts > ROUTER_MAX_EXPERTS || a.top_k > ROUTER_MAX_TOPK || a.hidden * 4 > 160 * 1024) return cudaErrorInvalidValue;
    // staged form: x and the CTA's eight rows in shared memory (rows padded by 16 floats); needs 16-byte rows
    const size_t staged_bytes = ((size_t)a.hidden + (size_t)ROUTER_EXPERTS_PER_CTA * (a.hidden + 16)) * 4;
    a.staged = (a.hidden % 4 == 0 && staged_bytes <= 200 * 1024 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0) ? 1u : 0u;
    const size_t smem = a.staged ? staged_bytes : (size_t)a.hidden * 4;
    {
        cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(moe_router_kernel), smem + 4096);      // beside 3 KiB of static shared memory
        if (e != cudaSuccess) return e;
    }
    if (a.logits == nullptr || a.done == nullptr) return cudaErrorInvalidValue;
    return launch_kernel(moe_router_kernel, dim3((a.n_experts + ROUTER_EXPERTS_PER_CTA - 1) / ROUTER_EXPERTS_PER_CTA, n_tok), dim3(ROUTER_THREADS), smem, s, pdl, a);
}
cudaError_t launch_expert_swiglu_quant(cudaStream_t s, const float *gate_up, uint32_t d_ff, uint32_t n_slot, int8_t *q, float *scales,
                                       int32_t *sums, bool pdl) {
    return launch_kernel(expert_swiglu_quant_kernel, dim3((d_ff / 64 + 7) / 8, n_slot), dim3(256), 0, s, pdl, gate_up, d_ff, q, scales, sums);
}
cudaError_t launch_moe_combine(cudaStream_t s, const float *expert_out, const float *route_w, uint32_t n_slot, uint32_t n, float *out,
                               bool pdl, const uint32_t *route_ids, const uint8_t *const *owned, uint32_t n_experts, uint32_t n_tok, uint32_t route_stride,
                               const float *base, const float *base_scale) {
    return launch_kernel(moe_combine_kernel, dim3((n + 255) / 256, n_tok), dim3(256), 0, s, pdl, expert_out, route_w, n_slot, n, out, route_ids, owned, n_experts,
                         route_stride, base, base_scale);
}

// Gate of a shared expert (SharedMoeExpert::gate_scale, sparse_moe.rs:241-249): sigmoid of dot_f32_moe(gate_w, x_norm), the
// dot in the 16-accumulator order of the router logits, the exp as in the scalar paths.  One warp per token.
__global__ void __launch_bounds__(32) shared_gate_kernel(const float *__restrict__ gate_w, const float *__restrict__ x_norm, uint32_t n,
                                                         float *__restrict__ scale) {
    const uint32_t lane = threadIdx.x, l16 = lane & 15;
    pdl_wait();
    pdl_trigger();
    const float *x = x_norm + (size_t)blockIdx.x * n;
    float acc = 0.0f;
    if (lane < 16)
        for (uint32_t i = l16; i < n; i += 16) acc = __fmaf_rn(__ldg(gate_w + i), __ldcg(x + i), acc);
    float t = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4));
    t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 8));
    t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 1));
    t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 2));
    if (lane == 0) scale[blockIdx.x] = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_cr(-t)));
}
cudaError_t launch_shared_gate(cudaStream_t s, const float *gate_w, const float *x_norm, uint32_t n, uint32_t n_tok, float *scale, bool pdl) {
    return launch_kernel(shared_gate_kernel, dim3(n_tok), dim3(32), 0, s, pdl, gate_w, x_norm, n, scale);
}
cudaError_t launch_rmsnorm_quant_x(cudaStream_t s, float *hidden, const float *delta, const float *w, uint32_t n, float eps,
                                   int8_t *q, float *scales, int32_t *sums, float *x_norm, uint32_t n_tok, bool pdl) {
    TpLink none{};
    return launch_rmsnorm_quant_tp(s, hidden, delta, w, n, eps, q, scales, sums, x_norm, n_tok, pdl, none, nullptr);
}
cudaError_t launch_rmsnorm_quant_tp(cudaStream_t s, float *hidden, const float *delta, const float *w, uint32_t n, float eps,
                                    int8_t *q, float *scales, int32_t *sums, float *x_norm, uint32_t n_tok, bool pdl,
                                    const TpLink &tp, uint32_t *tp_done) {
    if (tp.tp > 1 && ((size_t)n_tok * n > tp.ll_slot || tp_done == nullptr)) return cudaErrorInvalidValue;
    const bool with_tp = tp.tp > 1;
    const size_t smem = (size_t)n * sizeof(float) * (with_tp ? 3 : 2);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    {
        cudaError_t e = allow_dynamic_smem(with_tp ? reinterpret_cast<const void *>(rmsnorm_quant_kernel<true>) : reinterpret_cast<const void *>(rmsnorm_quant_kernel<false>), smem);
        if (e != cudaSuccess) return e;
    }
    // one warp per 64-value chunk where that fits: the load and the rotation each take one round
    const uint32_t threads = std::min(1024u, std::max(256u, (n / 64) * 32u));
    if (with_tp) return launch_kernel(rmsnorm_quant_kernel<true>, dim3(n_tok), dim3(threads), smem, s, pdl, hidden, delta, w, n, eps, q, scales, sums, x_norm, tp, tp_done);
    return launch_kernel(rmsnorm_quant_kernel<false>, dim3(n_tok), dim3(threads), smem, s, pdl, hidden, delta, w, n, eps, q, scales, sums, x_norm, tp, tp_done);
}
cudaError_t launch_qkv_post(cudaStream_t s, const QkvPostArgs &a, bool pdl, uint32_t n_tok) {
    const uint32_t heads = a.n_q + 2 * a.n_kv;
    return launch_kernel(qkv_post_kernel, dim3((heads + 3) / 4, n_tok), dim3(128), 0, s, pdl, a);
}
template <int HD, bool KV4>
static cudaError_t launch_partial(cudaStream_t s, dim3 grid, bool pdl, const AttnArgs &a) {
    constexpr size_t smem = attn_partial_smem<HD, KV4>();
    {
        cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(attn_partial_kernel<HD, KV4>), smem);
        if (e != cudaSuccess) return e;
    }
    return launch_kernel(attn_partial_kernel<HD, KV4>, grid, dim3(128), smem, s, pdl, a);
}
cudaError_t launch_attention(cudaStream_t s, const AttnArgs &a, bool pdl) {
    dim3 grid((a.n_split + 3) / 4, a.n_kv);
    cudaError_t e;
    if (a.head_dim == 64) e = a.kv_bits == 4 ? launch_partial<64, true>(s, grid, pdl, a) : launch_partial<64, false>(s, grid, pdl, a);
    else if (a.head_dim == 128) e = a.kv_bits == 4 ? launch_partial<128, true>(s, grid, pdl, a) : launch_partial<128, false>(s, grid, pdl, a);
    else return cudaErrorInvalidValue;
    if (e != cudaSuccess) return e;
    if (a.n_split > FINISH_THREADS) return cudaErrorInvalidValue;
    if (a.head_dim == 64) return launch_kernel(attn_finish_kernel<64>, dim3(a.n_kv * a.group), dim3(FINISH_THREADS), 0, s, pdl, a);
    return launch_kernel(attn_finish_kernel<128>, dim3(a.n_kv * a.group), dim3(FINISH_THREADS), 0, s, pdl, a);
}
cudaError_t launch_attention_fused(cudaStream_t s, const FusedAttnArgs &a, bool pdl) {
    const size_t smem = attn_smem_bytes(true);
    if (a.head_dim != 64 && a.head_dim != 128) return cudaErrorInvalidValue;
    cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(attn_fused_kernel), smem);
    if (e != cudaSuccess) return e;
    return launch_kernel(attn_fused_kernel, dim3(a.n_q), dim3(ATTN_THREADS), smem, s, pdl, a);
}
cudaError_t launch_swiglu_quant(cudaStream_t s, const float *gate_up, uint32_t inter, int8_t *q, float *scales, int32_t *sums,
                                float *dbg, uint32_t chunk0, uint32_t n_tok, bool pdl) {
    return launch_kernel(swiglu_quant_kernel, dim3((inter / 64 + 7) / 8, n_tok), dim3(256), 0, s, pdl, gate_up, inter, q, scales, sums, dbg, chunk0);
}
cudaError_t launch_argmax_step(cudaStream_t s, const float *logits, uint32_t n, uint32_t *token, uint32_t *pos,
                               uint32_t *history, uint32_t *step, float *scratch, bool pdl) {
    // scratch: ARGMAX_SCRATCH_WORDS 32-bit words, zero before the first launch: [256] values | [256] indices | counter
    if (scratch == nullptr) return cudaErrorInvalidValue;
    const uint32_t ctas = std::max(1u, std::min(ARGMAX_MAX_CTAS, n / 1024u));
    return launch_kernel(argmax_step_kernel, dim3(ctas), dim3(ARGMAX_THREADS), 0, s, pdl, logits, n, token, pos, history, step, scratch,
                         reinterpret_cast<uint32_t *>(scratch) + ARGMAX_MAX_CTAS, reinterpret_cast<uint32_t *>(scratch) + 2 * ARGMAX_MAX_CTAS);
}
cudaError_t launch_delay(cudaStream_t s, uint64_t ns) {
    return launch_kernel(delay_kernel, dim3(1), dim3(1), 0, s, false, (unsigned long long)ns);
}
cudaError_t launch_advance_pos(cudaStream_t s, uint32_t *pos, uint32_t by, bool pdl) {
    return launch_kernel(advance_pos_kernel, dim3(1), dim3(1), 0, s, pdl, pos, by);
}

}  // namespace k2t
