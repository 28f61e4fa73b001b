// Whole-token greedy decode in ONE cooperative kernel (counterpart of forward_token_sdot_megakernel,
// src/model/real_llm.rs:6794-7405: the reference's decode path that keeps its workers alive across the
// phases of a token instead of forking per projection).
//
// One CTA of 8 warps per SM stays resident for n_steps tokens.  A token is 5 phases per layer - qkv GEMV,
// attention, o GEMV, gate_up GEMV, down GEMV - plus the lm_head GEMV and the argmax, separated by grid
// barriers.  The small operators live in the prologue of the phase that consumes them and are computed by
// every CTA for itself in shared memory (a few KB of fp32 from L2, nothing to exchange):
//   residual add + RMSNorm + FWHT + int8   -> prologue of qkv / gate_up / lm_head
//   SwiGLU + FWHT + int8                   -> prologue of down
//   bias, qk-norm, RoPE, KV store, query quantization -> start of the attention phase (CTA q = query head q)
// The GEMV phases run the same warp pipeline as the stand-alone kernel (gemv_body), one team of WK warps
// per 4-row block, with the activations read from shared memory.  Arithmetic and summation orders are
// those of the per-operator kernels, so the outputs are identical to theirs bit for bit.
//
// Contexts are limited to ATTN_EXACT_CTX positions (the attention phase is the CPU-order kernel); the
// engine uses the per-operator path beyond.
//
// Grid barrier: one arrival counter in global memory, monotonically increasing; a CTA waits until the
// counter reaches (barriers so far) x (CTAs).  The wait is bounded: after BARRIER_LIMIT polls the CTA sets
// the error word and leaves the kernel (no bulk copy is in flight at a barrier), and so do the others
// when their own wait runs out.  Everything another CTA produced is read through L2 (ld.global.cg).
#include <cooperative_groups.h>

#include "k2t_decode_mega.h"
#include "k2t_model_device.cuh"

namespace k2t {

constexpr uint32_t MEGA_WARPS = 8, MEGA_THREADS = 256;
constexpr uint32_t BARRIER_LIMIT = 1u << 21;

struct MegaSmem {
    uint8_t *warp0;            // MEGA_WARPS regions of A.warp_smem bytes
    float *s_f;                // [8 teams][32]
    float *x;                  // fp32 staging of the vector being normalised [kmax]
    int8_t *xq;                // int8 activation [kmax]
    float *xs;                 // [kmax / 64]
    int32_t *xm;               // [kmax / 64]
    AttnSmem at;               // attention phase
};

__host__ __device__ inline size_t mega_round(size_t v) { return (v + 127) & ~(size_t)127; }

__device__ __forceinline__ MegaSmem carve(uint8_t *base, uint32_t warp_smem, uint32_t kmax) {
    MegaSmem s;
    size_t off = 0;
    s.warp0 = base; off += (size_t)MEGA_WARPS * warp_smem;
    s.s_f = reinterpret_cast<float *>(base + off); off += mega_round(8 * 32 * 4);
    s.x = reinterpret_cast<float *>(base + off); off += mega_round((size_t)kmax * 4);
    s.xq = reinterpret_cast<int8_t *>(base + off); off += mega_round(kmax);
    s.xs = reinterpret_cast<float *>(base + off); off += mega_round((size_t)kmax / 64 * 4);
    s.xm = reinterpret_cast<int32_t *>(base + off); off += mega_round((size_t)kmax / 64 * 4);
    s.at = attn_carve(base + off);
    return s;
}

size_t decode_mega_smem(uint32_t warp_smem, uint32_t kmax) {
    return (size_t)MEGA_WARPS * warp_smem + mega_round(8 * 32 * 4) + mega_round((size_t)kmax * 4) + mega_round(kmax) +
           2 * mega_round((size_t)kmax / 64 * 4) + attn_smem_bytes();
}

// ------------------------------------------------------------------------------------------------
// grid barrier (bounded)
// ------------------------------------------------------------------------------------------------
struct GridSync {
    uint32_t *counter, *err;
    uint32_t epoch = 0;
    // returns false when the wait gave up (the whole CTA must leave the kernel)
    __device__ __forceinline__ bool sync() {
        __syncthreads();
        int failed = 0;
        ++epoch;
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(counter, 1u);
            const uint32_t target = epoch * gridDim.x;
            uint32_t seen = 0, polls = 0;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                if (seen >= target) break;
                if (++polls > BARRIER_LIMIT) { failed = 1; atomicExch(err, 2u); break; }
            }
            __threadfence();
        }
        return __syncthreads_or(failed) == 0;
    }
};

// ------------------------------------------------------------------------------------------------
// per-CTA prologues: fill s.xq / s.xs / s.xm with the activation of the next GEMV
// ------------------------------------------------------------------------------------------------
// s.x holds n fp32 values: RMSNorm (CPU accumulator order, see rmsnorm_quant_kernel) + rotation + int8.
#define MEGA_SMEM_HINTS(s)                                                                                                   \
    __builtin_assume(__isShared((s).x)); __builtin_assume(__isShared((s).xq)); __builtin_assume(__isShared((s).xs));          \
    __builtin_assume(__isShared((s).xm)); __builtin_assume(__isShared((s).warp0)); __builtin_assume(__isShared((s).s_f));     \
    __builtin_assume(__isShared((s).at.inv)); __builtin_assume(__isShared((s).at.red));

__device__ __noinline__ void cta_norm_quant(const MegaSmem &s, const float *__restrict__ w, uint32_t n, float eps) {
    MEGA_SMEM_HINTS(s)
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nc = n / 64;
    if (warp == 0) {
        float acc = 0.0f;
        if (lane < 16) {
#pragma unroll 8
            for (uint32_t i = lane; i < n; i += 16) { const float v = s.x[i]; acc = __fmaf_rn(v, v, acc); }
        }
        float t = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 8));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 1));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 2));
        if (lane == 0) *s.at.inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), eps)));
    }
    __syncthreads();
    const float inv = *s.at.inv;
    for (uint32_t c = warp; c < nc; c += MEGA_WARPS) {
        float2 v = reinterpret_cast<const float2 *>(s.x + (size_t)c * 64)[lane];
        const float2 ww = __ldg(reinterpret_cast<const float2 *>(w + (size_t)c * 64) + lane);
        v.x = __fmul_rn(__fmul_rn(v.x, inv), ww.x);
        v.y = __fmul_rn(__fmul_rn(v.y, inv), ww.y);
        warp_fwht64(v.x, v.y, c, lane);
        int q0, q1, sum;
        float sc;
        warp_quant64(v.x, v.y, q0, q1, sc, sum);
        reinterpret_cast<char2 *>(s.xq + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (lane == 0) { s.xs[c] = sc; s.xm[c] = sum; }
    }
    __syncthreads();
}

// x = in + delta (delta may be null); CTA 0 also writes x to `out`.  Then norm + quant.
__device__ __noinline__ void cta_residual_norm_quant(const MegaSmem &s, const float *in, const float *delta, float *out,
                                                        const float *w, uint32_t n, float eps) {
    MEGA_SMEM_HINTS(s)
    for (uint32_t i = threadIdx.x; i < n / 4; i += MEGA_THREADS) {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(in) + i);
        if (delta != nullptr) {
            const float4 d = __ldcg(reinterpret_cast<const float4 *>(delta) + i);
            v.x = __fadd_rn(v.x, d.x); v.y = __fadd_rn(v.y, d.y); v.z = __fadd_rn(v.z, d.z); v.w = __fadd_rn(v.w, d.w);
        }
        reinterpret_cast<float4 *>(s.x)[i] = v;
        if (blockIdx.x == 0) reinterpret_cast<float4 *>(out)[i] = v;
    }
    __syncthreads();
    cta_norm_quant(s, w, n, eps);
}

// x = embedding of `tok` (embed_kernel); CTA 0 writes it to `out`.  Then norm + quant.
__device__ __noinline__ void cta_embed_norm_quant(const MegaSmem &s, const EmbedArgs &e, uint32_t tok, float *out, const float *w,
                                                     uint32_t n, float eps) {
    MEGA_SMEM_HINTS(s)
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t c = warp; c < e.nc; c += MEGA_WARPS) {
        float v0, v1;
        if (e.embed_bf16 != nullptr) {
            const uint16_t *row = e.embed_bf16 + (size_t)tok * e.nc * 64 + (size_t)c * 64;
            v0 = bf16_bits_to_f32(row[2 * lane]);
            v1 = bf16_bits_to_f32(row[2 * lane + 1]);
        } else {
            v0 = cell_value(e, tok, c, 2 * lane);
            v1 = cell_value(e, tok, c, 2 * lane + 1);
            warp_ifwht64(v0, v1, c, lane);
        }
        reinterpret_cast<float2 *>(s.x + (size_t)c * 64)[lane] = make_float2(v0, v1);
        if (blockIdx.x == 0) reinterpret_cast<float2 *>(out + (size_t)c * 64)[lane] = make_float2(v0, v1);
    }
    __syncthreads();
    cta_norm_quant(s, w, n, eps);
}

// SwiGLU of gate_up[2 * inter] + rotation + int8 (swiglu_quant_kernel)
__device__ __noinline__ void cta_swiglu_quant(const MegaSmem &s, const float *gate_up, uint32_t inter) {
    MEGA_SMEM_HINTS(s)
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t c = warp; c < inter / 64; c += MEGA_WARPS) {
        const float2 g = __ldcg(reinterpret_cast<const float2 *>(gate_up + (size_t)c * 64) + lane);
        const float2 u = __ldcg(reinterpret_cast<const float2 *>(gate_up + inter + (size_t)c * 64) + lane);
        float x0 = __fmul_rn(__fdiv_rn(g.x, __fadd_rn(1.0f, exp_poly(-g.x))), u.x);
        float x1 = __fmul_rn(__fdiv_rn(g.y, __fadd_rn(1.0f, exp_poly(-g.y))), u.y);
        warp_fwht64(x0, x1, c, lane);
        int q0, q1, sum;
        float sc;
        warp_quant64(x0, x1, q0, q1, sc, sum);
        reinterpret_cast<char2 *>(s.xq + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (lane == 0) { s.xs[c] = sc; s.xm[c] = sum; }
    }
    __syncthreads();
}

// copies an activation another phase left in global memory
__device__ __noinline__ void cta_load_act(const MegaSmem &s, const int8_t *q, const float *sc, const int32_t *sm, uint32_t n) {
    MEGA_SMEM_HINTS(s)
    for (uint32_t i = threadIdx.x; i < n / 16; i += MEGA_THREADS)
        reinterpret_cast<int4 *>(s.xq)[i] = __ldcg(reinterpret_cast<const int4 *>(q) + i);
    for (uint32_t i = threadIdx.x; i < n / 64; i += MEGA_THREADS) { s.xs[i] = __ldcg(sc + i); s.xm[i] = __ldcg(sm + i); }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------------
// GEMV phase
// ------------------------------------------------------------------------------------------------
struct TeamSlot { uint8_t *wsm; float *s_f; uint32_t gw, nw, wid, wk, bar; };

template <int FMT>
__device__ __noinline__ void mega_gemv_fmt(const MegaMatrix *mm, const int8_t *xq, const float *xs, const int32_t *xm, float *out,
                                           const TeamSlot t, PipeState &ps) {
    __builtin_assume(__isShared(xq)); __builtin_assume(__isShared(xs)); __builtin_assume(__isShared(xm));
    __builtin_assume(__isShared(t.wsm)); __builtin_assume(__isShared(t.s_f));
    const GemvArgs a = mm->g;
    gemv_body<FMT, 1, false, true>(a, xq, xs, xm, out, t.wsm, t.s_f, t.gw, t.nw, t.wid, t.wk, t.bar, ps);
}

__device__ __noinline__ void mega_gemv(const MegaMatrix *mm, float *out, const MegaSmem &s, uint32_t warp_smem, PipeState &ps) {
    const uint32_t fmt = mm->fmt, wk = mm->wk;
    const uint32_t warp = threadIdx.x >> 5, team = warp / wk, teams = MEGA_WARPS / wk;
    TeamSlot t;
    t.gw = team * gridDim.x + blockIdx.x; t.nw = teams * gridDim.x;     // consecutive blocks -> different SMs
    t.wid = warp % wk; t.wk = wk; t.bar = 1 + team;
    t.wsm = s.warp0 + (size_t)warp * warp_smem;
    t.s_f = s.s_f + team * 32;
    switch (fmt) {
        case FMT_BP4: mega_gemv_fmt<FMT_BP4>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        case FMT_BP5: mega_gemv_fmt<FMT_BP5>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        case FMT_BP6: mega_gemv_fmt<FMT_BP6>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        case FMT_NF4: mega_gemv_fmt<FMT_NF4>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        case FMT_NF3: mega_gemv_fmt<FMT_NF3>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        case FMT_NF5: mega_gemv_fmt<FMT_NF5>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        case FMT_E8Q2: mega_gemv_fmt<FMT_E8Q2>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
        default: mega_gemv_fmt<FMT_NF4G>(mm, s.xq, s.xs, s.xm, out, t, ps); break;
    }
}

// first maximum of logits[n] (argmax_scalar, real_llm.rs:9914-9924), by one CTA
__device__ __noinline__ uint32_t cta_argmax(const float *logits, uint32_t n, const MegaSmem &s) {
    MEGA_SMEM_HINTS(s)
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < n; i += MEGA_THREADS) {
        const float v = __ldcg(logits + i);
        if (v > bv) { bv = v; bi = i; }
    }
    auto better = [](float v, uint32_t i, float bv2, uint32_t bi2) { return v > bv2 || (v == bv2 && i < bi2); };
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, m);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    uint32_t *s_i = reinterpret_cast<uint32_t *>(s.at.red) + 8;      // s.red has room for 32 words
    if ((threadIdx.x & 31) == 0) { s.at.red[threadIdx.x >> 5] = bv; s_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    bv = s.at.red[0]; bi = s_i[0];
    for (uint32_t w = 1; w < MEGA_WARPS; ++w)
        if (better(s.at.red[w], s_i[w], bv, bi)) { bv = s.at.red[w]; bi = s_i[w]; }
    __syncthreads();
    return bi == 0xffffffffu ? 0u : bi;
}

// Phase trace (diagnostic): CTA 0 records the global timer at every phase boundary of the last step.
struct Trace {
    unsigned long long *buf;
    uint32_t n = 0, cap;
    bool on = false;
    __device__ __forceinline__ void mark() {
        if (on && threadIdx.x == 0 && n < cap) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            buf[n++] = t;
        }
    }
};

__global__ void __launch_bounds__(MEGA_THREADS, 1) decode_mega_kernel(const MegaArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    const MegaSmem s = carve(smem, A.warp_smem, A.kmax);
    const uint32_t warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) gemv_init_barriers(s.warp0 + (size_t)warp * A.warp_smem);
    __syncthreads();
    PipeState ps;
    GridSync grid{A.barrier, A.err_flag};
    const uint32_t h = A.hidden;
    uint32_t token = A.first_token;
    Trace tr{A.trace, 0, A.trace_cap};
    for (uint32_t step = 0; step < A.n_steps; ++step) {
        const uint32_t pos = A.pos0 + step;
        tr.on = A.trace != nullptr && blockIdx.x == 0 && step + 1 == A.n_steps;
        tr.mark();
        for (uint32_t l = 0; l < A.n_layers; ++l) {
            const MegaLayer *L = A.layers + l;
            // qkv (prologue: embedding or residual of the previous down_proj, input norm)
            if (l == 0) cta_embed_norm_quant(s, A.embed, token, A.hidden_b, L->input_norm, h, A.eps);
            else cta_residual_norm_quant(s, A.hidden_a, A.proj, A.hidden_b, L->input_norm, h, A.eps);
            tr.mark();
            mega_gemv(&L->qkv, A.qkv, s, A.warp_smem, ps);
            tr.mark();
            if (!grid.sync()) return;
            tr.mark();
            // attention (CTA q = query head q)
            if (blockIdx.x < A.n_q) {
                FusedAttnArgs fa;
                fa.qkv = A.qkv; fa.bias = L->qkv_bias; fa.q_norm = L->q_norm; fa.k_norm = L->k_norm; fa.rope = A.rope; fa.pos = nullptr;
                fa.k_q8 = A.k_q8; fa.v_q8 = A.v_q8; fa.k_scale = A.k_scale; fa.v_scale = A.v_scale;
                fa.attn_tap = l + 1 == A.n_layers ? A.attn_tap : nullptr;
                fa.out_q = A.act_q; fa.out_scales = A.act_s; fa.out_sums = A.act_m; fa.err_flag = A.err_flag;
                fa.n_q = A.n_q; fa.n_kv = A.n_kv; fa.head_dim = A.head_dim; fa.max_seq = A.max_seq; fa.layer = l;
                fa.eps = A.eps; fa.attn_scale = A.attn_scale; fa.qk_norm_after_rope = A.qk_norm_after_rope;
                fa.kv_bits = A.kv_bits; fa.out_chunk0 = 0; fa.pos_offset = 0; fa.trace = nullptr; fa.early = 0; fa.v_t = A.v_t;
                attention_head_dispatch<false>(fa, blockIdx.x, pos, s.at);
            }
            tr.mark();
            if (!grid.sync()) return;
            tr.mark();
            // o_proj
            cta_load_act(s, A.act_q, A.act_s, A.act_m, A.n_q * A.head_dim);
            tr.mark();
            mega_gemv(&L->o, A.proj, s, A.warp_smem, ps);
            tr.mark();
            if (!grid.sync()) return;
            tr.mark();
            // gate_up (prologue: residual of o_proj, post-attention norm)
            cta_residual_norm_quant(s, A.hidden_b, A.proj, A.hidden_a, L->post_norm, h, A.eps);
            tr.mark();
            mega_gemv(&L->gate_up, A.gate_up, s, A.warp_smem, ps);
            tr.mark();
            if (!grid.sync()) return;
            tr.mark();
            // down (prologue: SwiGLU)
            cta_swiglu_quant(s, A.gate_up, A.inter);
            tr.mark();
            mega_gemv(&L->down, A.proj, s, A.warp_smem, ps);
            tr.mark();
            if (!grid.sync()) return;
            tr.mark();
        }
        // lm_head (prologue: last residual, final norm)
        cta_residual_norm_quant(s, A.hidden_a, A.proj, A.hidden_b, A.final_norm, h, A.eps);
        tr.mark();
        mega_gemv(A.head, A.logits, s, A.warp_smem, ps);
        tr.mark();
        if (!grid.sync()) return;
        tr.mark();
        if (blockIdx.x == 0) {
            const uint32_t best = cta_argmax(A.logits, A.vocab, s);
            if (threadIdx.x == 0) {
                *A.token = best;
                A.history[step] = best;
                *A.step = step + 1;
                *A.pos = pos + 1;
            }
        }
        tr.mark();
        if (tr.on && threadIdx.x == 0) A.trace[A.trace_cap] = tr.n;
        if (step + 1 < A.n_steps) {
            if (!grid.sync()) return;
            token = __ldcg(A.token);
        }
    }
}

cudaError_t decode_mega_check(size_t smem, int sm_count) {
    int dev = 0, coop = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (e != cudaSuccess) return e;
    if (!coop) return cudaErrorNotSupported;
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    e = cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel, MEGA_THREADS, smem);
    if (e != cudaSuccess) return e;
    (void)sm_count;
    return per_sm >= 1 ? cudaSuccess : cudaErrorCooperativeLaunchTooLarge;
}

cudaError_t launch_decode_mega(cudaStream_t s, const MegaArgs &a, size_t smem, int sm_count) {
    MegaArgs copy = a;
    void *params[] = {&copy};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(decode_mega_kernel), dim3((unsigned)sm_count), dim3(MEGA_THREADS),
                                       params, smem, s);
}

}  // namespace k2t
