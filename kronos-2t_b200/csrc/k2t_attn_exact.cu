// Decode attention over the Hadamard KV cache in the reference's own summation order, for any context length
// (causal_gqa_group_q8, src/model/real_llm.rs:8471-8594; NF4 cache: causal_gqa_group_q4_or_window, 8794-8988):
//   scores for every position (exact integer dots), the global maximum, exp (NEON polynomial for whole groups of four
//   positions, correctly rounded exp for the remainder), the softmax denominator as four interleaved accumulators
//   combined (a0 + a1) + (a2 + a3) plus the remainder in order, then for every dimension ONE position-ascending fma
//   chain over the cached values.
// The output is the CPU's bit for bit at every length; the price is the serial part: ctx / 4 dependent adds for the
// denominator and ctx dependent fmas per dimension (about 4.5 cycles per position).  Two kernels after qkv_post_kernel:
//   attn_scores_kernel  - CTA = (128 positions, kv head): key rows staged by one bulk copy, lane = position, dp4a against
//                         the group's int8 queries; writes the scores and the maximum of every 128-position block;
//   attn_values_kernel  - CTA = query head: maximum, exp, denominator, value weights for all positions in shared memory,
//                         then the chains: thread = dimension, value rows streamed through a ring of 256-position tiles
//                         (bulk copies issued by a producer warp, full / empty mbarriers), sixteen positions loaded
//                         ahead of the chain; finally the inverse rotation, the forward rotation with the global chunk
//                         index and the int8 activation of o_proj (real_llm.rs:7059-7084).
#include <algorithm>

#include "k2t_model_device.cuh"

namespace k2t {

constexpr uint32_t SCORE_TILE = 128;          // positions per CTA of the scores kernel (= its threads)
constexpr uint32_t VAL_THREADS = 256;
constexpr uint32_t VAL_TILE = 256;            // positions per ring stage of the values kernel
constexpr uint32_t VAL_NST = 4;
constexpr uint32_t EXACT_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (uint32_t spin = 0; spin < EXACT_WAIT_LIMIT && !ok; ++spin) ok = mbar_try_wait(bar, parity);
    return ok != 0;
}

// ------------------------------------------------------------------------------------------------
// scores
// ------------------------------------------------------------------------------------------------
template <int HD, bool KV4>
__global__ void __launch_bounds__(SCORE_TILE) attn_scores_kernel(const ExactAttnArgs a) {
    constexpr int QW = HD / 4, NB = HD / 64;
    constexpr uint32_t ROW = KV4 ? HD / 2 : HD, NV = ROW / 16;
    __shared__ __align__(128) uint8_t s_k[SCORE_TILE * ROW];
    __shared__ __align__(16) int s_q[8][QW];
    __shared__ float s_red[8][SCORE_TILE / 32];
    __shared__ __align__(8) uint64_t s_bar;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t blk = blockIdx.x, kvh = blockIdx.y, tok = blockIdx.z, G = a.group, n_q = a.n_kv * G;
    pdl_wait();
    pdl_trigger();
    // sliding window: ctx = the active positions (sinks + the last window - sinks); index t -> position -> ring row
    const uint32_t seq_len = __ldcg(a.pos) + a.pos_offset + tok + 1, ctx = a.ring.active_len(seq_len), t0 = blk * SCORE_TILE;
    const bool windowed = a.ring.window > 0;
    if (t0 >= ctx) return;
    const uint32_t n = min(SCORE_TILE, ctx - t0);
    const size_t slot0 = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq;
    const uint8_t *K = reinterpret_cast<const uint8_t *>(a.k_q8) + (slot0 + t0) * ROW;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&s_bar);
    if (tid == 0 && !windowed) {
        mbar_init(bar, 1);
        fence_mbar_init();
        asm volatile("fence.proxy.async;" ::: "memory");      // the row qkv_post_kernel stored for this position is read by the copy engine
        mbar_expect_tx(bar, n * ROW);
        bulk_g2s((uint32_t)__cvta_generic_to_shared(s_k), K, n * ROW, bar);
    }
    // the group's int8 queries (NF4 cache: gathered in the packed column order of a cached row)
    for (uint32_t i = tid; i < G * QW; i += SCORE_TILE) {
        const int8_t *qb = a.q_i8 + ((size_t)tok * n_q + kvh * G + i / QW) * HD;
        const uint32_t wi = i % QW;
        if (KV4) {        // packed word w of a 64-value group holds columns (c, 16+c, c+1, 16+c+1 | c+2, ...) of a 32-column half
            const uint32_t g = wi / 16, w = (wi % 16) / 2, u = wi % 2;
            const int8_t *p = qb + g * 64 + (w / 4) * 32 + 4 * (w % 4);
            s_q[i / QW][wi] = (int)((uint32_t)(uint8_t)__ldcg(p + 2 * u) | ((uint32_t)(uint8_t)__ldcg(p + 16 + 2 * u) << 8) |
                                    ((uint32_t)(uint8_t)__ldcg(p + 2 * u + 1) << 16) | ((uint32_t)(uint8_t)__ldcg(p + 16 + 2 * u + 1) << 24));
        } else {
            s_q[i / QW][wi] = __ldcg(reinterpret_cast<const int *>(qb) + wi);
        }
    }
    const uint32_t t = t0 + tid;
    const bool on = tid < n;
    const uint32_t row = on ? a.ring.slot_of_pos(a.ring.active_pos(t, seq_len)) : 0u;      // cache row of this lane's position
    float kst[KV4 ? NB : 1];
    if (KV4) {
        const uint16_t *ks16 = reinterpret_cast<const uint16_t *>(a.k_scale) + (slot0 + row) * NB;
#pragma unroll
        for (int b = 0; b < NB; ++b) kst[b] = on ? bf16_bits_to_f32(__ldcg(ks16 + b)) : 0.0f;
    } else {
        kst[0] = on ? __ldcg(a.k_scale + slot0 + row) : 0.0f;
    }
    float qas[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) qas[g] = g < (int)G ? __fmul_rn(__ldcg(a.q_scale + (size_t)tok * n_q + kvh * G + g), a.attn_scale) : 0.0f;
    __syncthreads();                               // queries staged, barrier initialised
    if (!windowed) {
        const bool arrived = mbar_wait_bounded(bar, 0);
        if (__syncthreads_or(!arrived)) {
            if (tid == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
            return;
        }
    }
    int up[8][NB], dn[8][KV4 ? NB : 1];           // integer dots per 64-value group
#pragma unroll
    for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int b = 0; b < NB; ++b) { up[g][b] = 0; if (KV4) dn[g][b] = 0; }
    // the 16-byte vectors of a row are visited in a lane-dependent rotation, so that a quarter-warp reads eight different
    // bank groups (integer sums do not depend on the order); rows beyond n hold stale bytes and their scores are dropped.
    // With a window the rows are not contiguous in the ring: every lane reads its own row from the cache (L2) instead.
    const uint4 *krow = windowed ? reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(a.k_q8) + (slot0 + row) * ROW)
                                 : reinterpret_cast<const uint4 *>(s_k + (size_t)tid * ROW);
    const uint32_t rot = (lane * NV / 8) % NV;
#pragma unroll
    for (uint32_t v = 0; v < NV; ++v) {
        const uint32_t vv = (v + rot) & (NV - 1);
        const uint4 kk = krow[vv];
        if (KV4) {
            const bool second = NB == 2 && vv >= NV / 2;
            const uint32_t x[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g >= (int)G) break;
                const int4 qa = *reinterpret_cast<const int4 *>(&s_q[g][8 * vv]), qb = *reinterpret_cast<const int4 *>(&s_q[g][8 * vv + 4]);
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
                const int4 qq = *reinterpret_cast<const int4 *>(&s_q[g][4 * vv]);
                int d = 0;
                d = __dp4a((int)kk.x, qq.x, d); d = __dp4a((int)kk.y, qq.y, d); d = __dp4a((int)kk.z, qq.z, d); d = __dp4a((int)kk.w, qq.w, d);
                if (NB == 2 && vv >= NV / 2) up[g][NB - 1] += d;        // vector vv covers dimensions 16 vv .. 16 vv + 15
                else up[g][0] += d;
            }
        }
    }
    // int8 cache: 256-position tiles; whole groups of 8 use dot*(ks*qas), the tile remainder (dot*ks)*qas (8992-9057)
    const uint32_t tile0 = t & ~255u, tile_n = min(ctx, tile0 + 256u) - tile0;
    const bool grouped = t - tile0 < (tile_n & ~7u);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        if (g >= (int)G) break;
        float s = -INFINITY;
        if (on) {
            if (KV4) {        // total += ((dot_b * ks_b) * q_s) per 64-value group
                s = 0.0f;
#pragma unroll
                for (int b = 0; b < NB; ++b) s = __fadd_rn(s, __fmul_rn(__fmul_rn((float)(up[g][b] - dn[g][b]), kst[b]), qas[g]));
            } else if (windowed) {       // causal_gqa_group_q4_or_window with the int8 cache: one scale per slot, still a term per 64-value group
                s = 0.0f;
#pragma unroll
                for (int b = 0; b < NB; ++b) s = __fadd_rn(s, __fmul_rn(__fmul_rn((float)up[g][b], kst[0]), qas[g]));
            } else {
                const int dot = NB == 2 ? up[g][0] + up[g][NB - 1] : up[g][0];
                s = grouped ? __fmul_rn((float)dot, __fmul_rn(kst[0], qas[g])) : __fmul_rn(__fmul_rn((float)dot, kst[0]), qas[g]);
            }
            a.sc[((size_t)tok * n_q + kvh * G + g) * a.sc_stride + t] = s;
        }
        const float m = warp_max(s);
        if (lane == 0) s_red[g][warp] = m;
    }
    __syncthreads();
    if (tid < G) {
        float m = s_red[tid][0];
#pragma unroll
        for (uint32_t w = 1; w < SCORE_TILE / 32; ++w) m = fmaxf(m, s_red[tid][w]);
        a.bmax[((size_t)tok * n_q + kvh * G + tid) * a.blk_stride + blk] = m;
    }
    if (tid == 0 && !windowed) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ------------------------------------------------------------------------------------------------
// maximum, exp, denominator, value chains, o_proj activation
// ------------------------------------------------------------------------------------------------
template <int HD, bool KV4>
struct ValSmem {
    static constexpr uint32_t ROW = KV4 ? HD / 2 : HD;
    static constexpr uint32_t NW = KV4 ? HD / 64 : 1;             // weight vectors (one per 64-value group for NF4)
    static constexpr uint32_t STAGE = VAL_TILE * ROW;
    static __host__ __device__ size_t bytes(uint32_t ctx_cap) { return 128 + (size_t)VAL_NST * STAGE + (size_t)NW * ctx_cap * 4; }
};

#define VAL_MARK(i) do { if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) a.trace[i] = (unsigned long long)clock64(); } while (0)

template <int HD, bool KV4>
__global__ void __launch_bounds__(VAL_THREADS) attn_values_kernel(const ExactAttnArgs a) {
    using Sm = ValSmem<HD, KV4>;
    constexpr int NB = HD / 64;
    constexpr uint32_t ROW = Sm::ROW, CW = HD / 32;               // chain warps
    extern __shared__ __align__(128) uint8_t dyn[];
    __shared__ float s_red[VAL_THREADS / 32];
    __shared__ float s_inv, s_max;
    __shared__ float s_o[HD];
    __shared__ float s_cb[16];
    __shared__ uint32_t s_fail;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t qh = blockIdx.x, tok = blockIdx.y, G = a.group, kvh = qh / G, n_q = a.n_kv * G;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(dyn);           // full[VAL_NST], then empty[VAL_NST]
    uint8_t *stages = dyn + 128;
    float *W = reinterpret_cast<float *>(dyn + 128 + (size_t)VAL_NST * Sm::STAGE);
    if (tid == 0) {
        for (uint32_t s = 0; s < VAL_NST; ++s) { mbar_init(bar0 + 8 * s, 1); mbar_init(bar0 + 8 * (VAL_NST + s), CW); }
        fence_mbar_init();
        s_fail = 0;
    }
    if (KV4 && tid < 16) s_cb[tid] = NF4_KV_CENTROIDS[tid];
    pdl_wait();
    pdl_trigger();
    const uint32_t seq_len = __ldcg(a.pos) + a.pos_offset + tok + 1, ctx = a.ring.active_len(seq_len), cap = a.ctx_cap;
    const KvRing ring = a.ring;
    if (ctx > cap) {                       // the launcher sizes shared memory for the cache length: cannot happen
        if (tid == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 5u);
        return;
    }
    const size_t slot0 = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq;
    const uint8_t *V = reinterpret_cast<const uint8_t *>(a.v_q8) + slot0 * ROW;
    const uint32_t n_tiles = (ctx + VAL_TILE - 1) / VAL_TILE;
    __syncthreads();                       // barriers initialised
    VAL_MARK(0);
    // ---- producer: lane 0 of warp CW keeps the ring full; the first VAL_NST tiles go out at once
    auto fill = [&](uint32_t i) {
        const uint32_t st = i % VAL_NST, tl = i * VAL_TILE, n = min(VAL_TILE, ctx - tl);
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(stages + (size_t)st * Sm::STAGE);
        fence_proxy_async();
        mbar_expect_tx(bar0 + 8 * st, n * ROW);
        // the rows of consecutive active positions are consecutive cache rows except where the sinks end and where the ring
        // wraps: one bulk copy per run (one run without a window)
        uint32_t cur = tl;
        while (cur < tl + n) {
            const uint32_t p = ring.active_pos(cur, seq_len), row = ring.slot_of_pos(p);
            uint32_t run = tl + n - cur;
            if (ring.window > 0 && seq_len > ring.window && cur < ring.sinks) run = min(run, ring.sinks - cur);
            else if (ring.ring_len > 0 && p >= ring.sinks) run = min(run, ring.sinks + ring.ring_len - row);
            bulk_g2s(dst + (cur - tl) * ROW, V + (size_t)row * ROW, run * ROW, bar0 + 8 * st);
            cur += run;
        }
    };
    if (warp == CW && lane == 0)
        for (uint32_t i = 0; i < VAL_NST && i < n_tiles; ++i) fill(i);
    // ---- maximum over the blocks of the scores kernel
    {
        const uint32_t nblk = (ctx + SCORE_TILE - 1) / SCORE_TILE;
        float m = -INFINITY;
        for (uint32_t i = tid; i < nblk; i += VAL_THREADS) m = fmaxf(m, __ldcg(a.bmax + ((size_t)tok * n_q + qh) * a.blk_stride + i));
        m = warp_max(m);
        if (lane == 0) s_red[warp] = m;
        __syncthreads();
        if (tid == 0) {
            float mm = s_red[0];
            for (uint32_t w = 1; w < VAL_THREADS / 32; ++w) mm = fmaxf(mm, s_red[w]);
            s_max = mm;
        }
        __syncthreads();
    }
    // ---- exp: polynomial for whole groups of four positions, correctly rounded exp for the remainder (softmax_unnorm, 9603-9632)
    VAL_MARK(1);
    const float mx = s_max;
    const uint32_t n4 = ctx & ~3u;
    const float *sc = a.sc + ((size_t)tok * n_q + qh) * a.sc_stride;
    {   // eight loads in flight per thread (the scores come from L2)
        uint32_t t = tid;
        for (; t + 7 * VAL_THREADS < n4; t += 8 * VAL_THREADS) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(sc + t + u * VAL_THREADS);
#pragma unroll
            for (int u = 0; u < 8; ++u) W[t + u * VAL_THREADS] = exp_poly(__fsub_rn(v[u], mx));
        }
        for (; t < ctx; t += VAL_THREADS) {
            const float d = __fsub_rn(__ldcg(sc + t), mx);
            W[t] = t < n4 ? exp_poly(d) : (float)exp((double)d);
        }
    }
    __syncthreads();
    VAL_MARK(2);
    // ---- denominator: lanes 0..3 of warp 0 = the four accumulators (positions 4k + lane), sixteen loads ahead of the adds
    if (warp == 0) {
        float acc = 0.0f;
        if (lane < 4) {
            uint32_t t = lane;
            float cur[16], nxt[16];
            if (t + 60 < n4) {
#pragma unroll
                for (int u = 0; u < 16; ++u) cur[u] = W[t + 4 * u];
                for (; t + 124 < n4; t += 64) {
#pragma unroll
                    for (int u = 0; u < 16; ++u) nxt[u] = W[t + 64 + 4 * u];
#pragma unroll
                    for (int u = 0; u < 16; ++u) acc = __fadd_rn(acc, cur[u]);
#pragma unroll
                    for (int u = 0; u < 16; ++u) cur[u] = nxt[u];
                }
#pragma unroll
                for (int u = 0; u < 16; ++u) acc = __fadd_rn(acc, cur[u]);
                t += 64;
            }
            for (; t < n4; t += 4) acc = __fadd_rn(acc, W[t]);
        }
        acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 1));          // lane 0: a0 + a1, lane 2: a2 + a3
        acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 2));
        if (lane == 0) {
            for (uint32_t t = n4; t < ctx; ++t) acc = __fadd_rn(acc, W[t]);
            s_inv = __fdiv_rn(1.0f, acc);
        }
    }
    __syncthreads();
    VAL_MARK(3);
    // ---- value weights: (p * inv) * v_scale   (per 64-value group for the NF4 cache)
    const float inv = s_inv;
    if (KV4) {
        const uint16_t *vs16 = reinterpret_cast<const uint16_t *>(a.v_scale) + slot0 * NB;
        for (uint32_t t = tid; t < ctx; t += VAL_THREADS) {
            const float p_norm = __fmul_rn(W[t], inv);
            const size_t row = ring.slot_of_pos(ring.active_pos(t, seq_len));
            if (NB == 2) W[cap + t] = __fmul_rn(p_norm, bf16_bits_to_f32(__ldcg(vs16 + row * NB + 1)));
            W[t] = __fmul_rn(p_norm, bf16_bits_to_f32(__ldcg(vs16 + row * NB)));
        }
    } else {
        const float *vs = a.v_scale + slot0;
        uint32_t t = tid;
        for (; t + 7 * VAL_THREADS < ctx; t += 8 * VAL_THREADS) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(vs + ring.slot_of_pos(ring.active_pos(t + u * VAL_THREADS, seq_len)));
#pragma unroll
            for (int u = 0; u < 8; ++u) W[t + u * VAL_THREADS] = __fmul_rn(__fmul_rn(W[t + u * VAL_THREADS], inv), v[u]);
        }
        for (; t < ctx; t += VAL_THREADS) W[t] = __fmul_rn(__fmul_rn(W[t], inv), __ldcg(vs + ring.slot_of_pos(ring.active_pos(t, seq_len))));
    }
    __syncthreads();
    VAL_MARK(4);
    // ---- chains
    if (warp < CW) {
        // a zero weight adds +-0 (the CPU loop skips such positions: same bits, the values are finite and the sum starts at +0)
        float o = 0.0f;
        bool failed = false;
        long long t_wait = 0;
        const uint32_t d = tid;                                    // this thread's dimension
        uint32_t byte_off = d, shift = 0;
        const float *wp = W;
        if (KV4) {        // byte 16h + i of a 64-value group packs columns 32h + i (low nibble) and 32h + 16 + i (high)
            const uint32_t g = d / 64, e = d % 64, r = e % 32;
            byte_off = g * 32 + (e / 32) * 16 + (r % 16);
            shift = r < 16 ? 0u : 4u;
            wp = W + (size_t)g * cap;
        }
        auto value = [&](uint32_t b) -> float {
            if (KV4) return s_cb[(b >> shift) & 15u];
            return __fsub_rn(__uint_as_float(b ^ 0x4B000080u), 8388736.0f);      // int8 -> fp32 without the conversion unit
        };
        for (uint32_t i = 0; i < n_tiles; ++i) {
            const uint32_t st = i % VAL_NST, tl = i * VAL_TILE, n = min(VAL_TILE, ctx - tl);
            const long long tw0 = clock64();
            if (!mbar_wait_bounded(bar0 + 8 * st, (i / VAL_NST) & 1u)) { failed = true; break; }
            t_wait += clock64() - tw0;
            const uint8_t *vt = stages + (size_t)st * Sm::STAGE + byte_off;
            const float *wt = wp + tl;
            const uint32_t va = (uint32_t)__cvta_generic_to_shared(vt), wa = (uint32_t)__cvta_generic_to_shared(wt);
            uint32_t j = 0;
            if (n >= 16) {
                uint32_t cur[16], nxt[16];
                float4 wc[4], wn[4];
#pragma unroll
                for (int u = 0; u < 16; ++u) cur[u] = lds_u8(va + u * ROW);
#pragma unroll
                for (int u = 0; u < 4; ++u) wc[u] = lds_f32x4(wa + 16 * u);
                for (; j + 32 <= n; j += 16) {
#pragma unroll
                    for (int u = 0; u < 16; ++u) nxt[u] = lds_u8(va + (j + 16 + u) * ROW);
#pragma unroll
                    for (int u = 0; u < 4; ++u) wn[u] = lds_f32x4(wa + 4 * (j + 16) + 16 * u);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        o = __fmaf_rn(value(cur[4 * u + 0]), wc[u].x, o);
                        o = __fmaf_rn(value(cur[4 * u + 1]), wc[u].y, o);
                        o = __fmaf_rn(value(cur[4 * u + 2]), wc[u].z, o);
                        o = __fmaf_rn(value(cur[4 * u + 3]), wc[u].w, o);
                    }
#pragma unroll
                    for (int u = 0; u < 16; ++u) cur[u] = nxt[u];
#pragma unroll
                    for (int u = 0; u < 4; ++u) wc[u] = wn[u];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    o = __fmaf_rn(value(cur[4 * u + 0]), wc[u].x, o);
                    o = __fmaf_rn(value(cur[4 * u + 1]), wc[u].y, o);
                    o = __fmaf_rn(value(cur[4 * u + 2]), wc[u].z, o);
                    o = __fmaf_rn(value(cur[4 * u + 3]), wc[u].w, o);
                }
                j += 16;
            }
            for (; j < n; ++j) o = __fmaf_rn(value(vt[(size_t)j * ROW]), wt[j], o);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar0 + 8 * (VAL_NST + st));          // this warp is done with the stage
        }
        if (failed) atomicExch(&s_fail, 1u);
        if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) a.trace[8] = (unsigned long long)t_wait;
        s_o[d] = o;
    } else if (warp == CW && lane == 0) {
        for (uint32_t i = VAL_NST; i < n_tiles; ++i) {           // tile i reuses the stage of tile i - VAL_NST once every chain warp has left it
            if (!mbar_wait_bounded(bar0 + 8 * (VAL_NST + i % VAL_NST), ((i / VAL_NST) - 1u) & 1u)) { atomicExch(&s_fail, 1u); break; }
            fill(i);
        }
    }
    VAL_MARK(5);
    __syncthreads();
    VAL_MARK(6);
    if (s_fail != 0) {
        if (tid == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
        return;
    }
    // ---- inverse rotation (block index within the head), forward rotation with the global chunk index, int8 for o_proj
    if (warp < NB) {
        const uint32_t b = warp;
        float x0 = s_o[b * 64 + 2 * lane], x1 = s_o[b * 64 + 2 * lane + 1];
        warp_ifwht64(x0, x1, b, lane);
        if (a.attn_out != nullptr && tok + 1 == gridDim.y) reinterpret_cast<float2 *>(a.attn_out + (size_t)qh * HD + b * 64)[lane] = make_float2(x0, x1);
        const uint32_t c = qh * NB + b;
        warp_fwht64(x0, x1, a.out_chunk0 + c, lane);
        int q0, q1, sum;
        float scl;
        warp_quant64(x0, x1, q0, q1, scl, sum);
        const size_t row = (size_t)tok * n_q * NB;           // o_proj activation row of this token, in chunks
        reinterpret_cast<char2 *>(a.out_q + (row + c) * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (lane == 0) { a.out_scales[row + c] = scl; a.out_sums[row + c] = sum; }
    }
    VAL_MARK(7);
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
template <int HD, bool KV4>
static cudaError_t launch_exact(cudaStream_t s, const ExactAttnArgs &a, bool pdl, uint32_t n_tok) {
    const size_t smem = ValSmem<HD, KV4>::bytes(a.ctx_cap);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(attn_values_kernel<HD, KV4>), smem);
    if (e != cudaSuccess) return e;
    const uint32_t nblk = (a.ctx_cap + SCORE_TILE - 1) / SCORE_TILE;
    e = launch_kernel(attn_scores_kernel<HD, KV4>, dim3(nblk, a.n_kv, n_tok), dim3(SCORE_TILE), 0, s, pdl, a);
    if (e != cudaSuccess) return e;
    return launch_kernel(attn_values_kernel<HD, KV4>, dim3(a.n_kv * a.group, n_tok), dim3(VAL_THREADS), smem, s, pdl, a);
}

size_t attention_exact_max_ctx(uint32_t head_dim, uint32_t kv_bits) {
    const size_t ring = 128 + (size_t)VAL_NST * VAL_TILE * (kv_bits == 4 ? head_dim / 2 : head_dim);
    const size_t nw = kv_bits == 4 ? head_dim / 64 : 1;
    return (200 * 1024 - ring) / (4 * nw);
}

cudaError_t launch_attention_exact(cudaStream_t s, const ExactAttnArgs &a, bool pdl, uint32_t n_tok) {
    if (a.group > 8 || a.group == 0 || n_tok == 0) return cudaErrorInvalidValue;
    if (a.head_dim == 64) return a.kv_bits == 4 ? launch_exact<64, true>(s, a, pdl, n_tok) : launch_exact<64, false>(s, a, pdl, n_tok);
    if (a.head_dim == 128) return a.kv_bits == 4 ? launch_exact<128, true>(s, a, pdl, n_tok) : launch_exact<128, false>(s, a, pdl, n_tok);
    return cudaErrorInvalidValue;
}

}  // namespace k2t
