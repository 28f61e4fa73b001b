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
//   attn_values_kernel  - CTA = query head: maximum, exp and denominator for all positions in shared memory, then a
//                         three-stage pipeline over 256-position tiles: bulk copies of the value rows into a ring
//                         (producer lane), the other non-chain warps transpose each tile (dimension-major, see
//                         value_rows_transpose) and turn its softmax terms into value weights, and the chain warps
//                         (thread = dimension) run sixteen positions per 16-byte load; full / free mbarriers between
//                         the stages.  Finally the inverse rotation, the forward rotation with the global chunk index
//                         and the int8 activation of o_proj (real_llm.rs:7059-7084).
#include <algorithm>

#include "k2t_model_device.cuh"

namespace k2t {

constexpr uint32_t SCORE_TILE = 128;          // positions per CTA of the scores kernel (= its threads)
constexpr uint32_t VAL_THREADS = 288;        // chain warps, transposing warps, one producer warp (the ninth)
constexpr uint32_t VAL_TILE = 256;            // positions per ring stage of the values kernel
constexpr uint32_t VAL_TBUF = 2;              // transposed tiles in flight between the transposing warps and the chain warps
constexpr uint32_t EXACT_WAIT_LIMIT = 1u << 22;
constexpr uint32_t SCORE_TOK = 8;             // tokens of a prompt batch one scores CTA serves from one staged key tile

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (uint32_t spin = 0; spin < EXACT_WAIT_LIMIT && !ok; ++spin) ok = mbar_try_wait(bar, parity);
    return ok != 0;
}
// The same for warps that are ahead of the chain warps and share their schedulers: the hardware may park the thread for
// up to a microsecond per attempt (it wakes as soon as the phase completes), so waiting costs the running warps few issue slots.
__device__ __forceinline__ bool mbar_wait_bounded_idle(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (uint32_t spin = 0; spin < EXACT_WAIT_LIMIT && !ok; ++spin) {
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
    }
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
    // One CTA serves up to SCORE_TOK consecutive tokens of a batch from ONE staged key tile: token t of a prompt batch sees the
    // rows of the tokens before it (qkv_post_kernel has stored the whole batch), so the tile of the tile's last token holds
    // the rows of all of them; each token then takes the rows below its own context.
    const uint32_t blk = blockIdx.x, kvh = blockIdx.y, G = a.group, n_q = a.n_kv * G;
    const uint32_t tok_lo = blockIdx.z * SCORE_TOK, tok_hi = min(a.n_tok, tok_lo + SCORE_TOK);
    pdl_wait();
    pdl_trigger();
    // sliding window: ctx = the active positions (sinks + the last window - sinks); index t -> position -> ring row
    const uint32_t pos0 = __ldcg(a.pos) + a.pos_offset, t0 = blk * SCORE_TILE;
    const uint32_t ctx_hi = a.ring.active_len(pos0 + tok_hi);          // context of the tile's last token
    const bool windowed = a.ring.window > 0;
    if (t0 >= ctx_hi) return;
    const size_t slot0 = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq;
    const uint8_t *K = reinterpret_cast<const uint8_t *>(a.k_q8) + (slot0 + t0) * ROW;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&s_bar);
    if (tid == 0 && !windowed) {
        const uint32_t n_rows = min(SCORE_TILE, ctx_hi - t0);
        mbar_init(bar, 1);
        fence_mbar_init();
        asm volatile("fence.proxy.async;" ::: "memory");      // the rows qkv_post_kernel stored for these positions are read by the copy engine
        mbar_expect_tx(bar, n_rows * ROW);
        bulk_g2s((uint32_t)__cvta_generic_to_shared(s_k), K, n_rows * ROW, bar);
    }
    __syncthreads();                               // barrier initialised
    if (!windowed) {
        const bool arrived = mbar_wait_bounded(bar, 0);
        if (__syncthreads_or(!arrived)) {
            if (tid == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
            return;
        }
    }
    const uint32_t t = t0 + tid;
    for (uint32_t tok = tok_lo; tok < tok_hi; ++tok) {
    const uint32_t seq_len = pos0 + tok + 1, ctx = a.ring.active_len(seq_len);
    if (t0 >= ctx) continue;                       // the same for every thread of the CTA
    const uint32_t n = min(SCORE_TILE, ctx - t0);
    __syncthreads();                               // the token before is done with the staged queries and the maxima
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
    __syncthreads();                               // queries staged
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
    }          // tokens of the tile
    if (tid == 0 && !windowed) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ------------------------------------------------------------------------------------------------
// maximum, exp, denominator, value chains, o_proj activation
// ------------------------------------------------------------------------------------------------
template <int HD, bool KV4>
struct ValSmem {
    static constexpr uint32_t ROW = KV4 ? HD / 2 : HD;
    static constexpr uint32_t NW = KV4 ? HD / 64 : 1;             // weight vectors (one per 64-value group for NF4)
    static constexpr uint32_t STAGE = VAL_TILE * ROW;             // one tile of cache rows as stored
    static constexpr uint32_t NST = STAGE > 16 * 1024 ? 2 : 4;    // ring depth: 64 KB of rows in flight at most
    static constexpr uint32_t TILE_T = VAL_TILE * HD;             // one transposed tile: a byte per value, row = dimension
    static constexpr uint32_t W_OFF = 128 + NST * STAGE + VAL_TBUF * TILE_T;
    // barriers, row ring, transposed tiles, weights (16 floats of slack: the chain requests the next block's weights ahead)
    static __host__ __device__ uint32_t w_off(bool direct) { return direct ? 128 + NST * STAGE : W_OFF; }
    static __host__ __device__ size_t bytes(uint32_t ctx_cap, bool direct) { return w_off(direct) + (size_t)NW * (ctx_cap + 16) * 4; }
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
    __shared__ volatile uint32_t s_ready[4];       // direct mode: tiles whose value weights transposing warp w has written
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t qh = blockIdx.x, tok = blockIdx.y, G = a.group, kvh = qh / G, n_q = a.n_kv * G;
    // ring depth; transposing warps: the four that do not share a warp scheduler with a chain warp where that is possible
    // (head_dim 64: chain warps 0 and 1, transposing warps 2, 3, 6, 7, warps 4 and 5 idle during the chains; head_dim 128:
    // chain warps 0..3, transposing warps 4..7)
    constexpr uint32_t NST = Sm::NST, NTW = 4;
    // barriers: full[NST] (rows of a tile have landed), rows_free[NST] (every transposing warp has read them),
    // t_full[VAL_TBUF] (tile transposed and its weights written), t_free[VAL_TBUF] (every chain warp has left it)
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(dyn);
    const uint32_t bar_full = bar0, bar_rows_free = bar0 + 8 * NST, bar_t_full = bar0 + 16 * NST, bar_t_free = bar0 + 16 * NST + 8 * VAL_TBUF;
    uint8_t *stages = dyn + 128;
    const uint32_t tiles_t = (uint32_t)__cvta_generic_to_shared(dyn + 128 + (size_t)NST * Sm::STAGE);
    // direct: the cache holds a block-transposed copy of the value rows (ExactAttnArgs.v_t): tiles land ready for the chains,
    // the transposing warps only compute the value weights, and the chain warps free the ring stages themselves; no
    // transposed tiles exist then, and the weights follow the ring at once (the launcher sizes shared memory the same way)
    const bool direct = !KV4 && a.v_t != nullptr && a.ring.window == 0;
    float *W = reinterpret_cast<float *>(dyn + Sm::w_off(direct));
    const uint32_t w_stride = a.ctx_cap + 16;                                // floats between the weight vectors of the NF4 groups
    if (tid == 0) {
        for (uint32_t s = 0; s < NST; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_rows_free + 8 * s, direct ? CW : NTW); }
        for (uint32_t s = 0; s < VAL_TBUF; ++s) { mbar_init(bar_t_full + 8 * s, NTW); mbar_init(bar_t_free + 8 * s, CW); }
        fence_mbar_init();
        s_fail = 0;
        s_ready[0] = s_ready[1] = s_ready[2] = s_ready[3] = 0;
    }
    if (KV4 && tid < 16) s_cb[tid] = NF4_KV_CENTROIDS[tid];
    // The successor (the o_proj GEMV) is released when the chains reach their last two tiles, not here: its CTAs would sit
    // on this SM for the whole chain, and warps waiting for a predecessor slow the ones that run (the tail of this kernel
    // took eight times longer with them resident).
    pdl_wait();
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
        const uint32_t st = i % NST, tl = i * VAL_TILE, n = min(VAL_TILE, ctx - tl);
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(stages + (size_t)st * Sm::STAGE);
        fence_proxy_async();
        if (direct) {          // blocks of 16 positions x head_dim x 16 bytes, contiguous: one copy (whole blocks; the rows past ctx are unused)
            const uint32_t bytes = ((n + 15) / 16) * 16 * ROW;
            mbar_expect_tx(bar_full + 8 * st, bytes);
            bulk_g2s(dst, reinterpret_cast<const uint8_t *>(a.v_t) + slot0 * ROW + (size_t)tl * ROW, bytes, bar_full + 8 * st);
            return;
        }
        mbar_expect_tx(bar_full + 8 * st, n * ROW);
        // the rows of consecutive active positions are consecutive cache rows except where the sinks end and where the ring
        // wraps: one bulk copy per run (one run without a window)
        uint32_t cur = tl;
        while (cur < tl + n) {
            const uint32_t p = ring.active_pos(cur, seq_len), row = ring.slot_of_pos(p);
            uint32_t run = tl + n - cur;
            if (ring.window > 0 && seq_len > ring.window && cur < ring.sinks) run = min(run, ring.sinks - cur);
            else if (ring.ring_len > 0 && p >= ring.sinks) run = min(run, ring.sinks + ring.ring_len - row);
            bulk_g2s(dst + (cur - tl) * ROW, V + (size_t)row * ROW, run * ROW, bar_full + 8 * st);
            cur += run;
        }
    };
    if (warp == VAL_THREADS / 32 - 1 && lane == 0)
        for (uint32_t i = 0; i < NST && i < n_tiles; ++i) fill(i);
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
    // ---- denominator (softmax_body_sum in warp 0).  Meanwhile the transposing warps take the first VAL_TBUF tiles (rows only:
    // the weights need the denominator).
    const bool is_tw = CW == 4 ? (warp >= 4 && warp < 8) : (warp == 2 || warp == 3 || warp == 6 || warp == 7);
    const uint32_t tw = CW == 4 ? warp - 4 : (warp < 4 ? warp - 2 : warp - 4);          // transposing warp index 0..3 (0 = warp CW, the producer's)
    // tile i: rows of stage i % NST -> transposed tile i % VAL_TBUF; the producer lane refills the stage once all have read it
    auto transpose_tile = [&](uint32_t i) -> bool {
        const uint32_t st = i % NST, tb = i % VAL_TBUF, n = min(VAL_TILE, ctx - i * VAL_TILE);
        if (!mbar_wait_bounded(bar_full + 8 * st, (i / NST) & 1u)) return false;
        if (i >= VAL_TBUF && !mbar_wait_bounded(bar_t_free + 8 * tb, ((i / VAL_TBUF) - 1u) & 1u)) return false;
        value_rows_transpose<HD, KV4>((uint32_t)__cvta_generic_to_shared(stages + (size_t)st * Sm::STAGE), tiles_t + tb * Sm::TILE_T, VAL_TILE,
                                      (n + 15) / 16, tw, NTW, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rows_free + 8 * st);
        return true;
    };
    // producer (lane 0 of the ninth warp): tile i + NST goes into the stage of tile i once every transposing warp has read it
    auto refill_after = [&](uint32_t i) -> bool {
        if (i + NST >= n_tiles) return true;
        if (!mbar_wait_bounded_idle(bar_rows_free + 8 * (i % NST), (i / NST) & 1u)) return false;
        fill(i + NST);
        return true;
    };
    constexpr uint32_t PRODUCER_WARP = VAL_THREADS / 32 - 1;
    bool failed = false;
    const uint32_t li = tw * 32 + lane;                            // transposing warps: this lane's position within a tile (and li + NTW * 32)
    constexpr uint32_t PER = (VAL_TILE + NTW * 32 - 1) / (NTW * 32);
    float sc_first[4][PER];
    if (warp == 0) {
        float acc = softmax_body_sum((uint32_t)__cvta_generic_to_shared(W), n4, lane);
        if (lane == 0) {
            for (uint32_t t2 = n4; t2 < ctx; ++t2) acc = __fadd_rn(acc, W[t2]);
            s_inv = __fdiv_rn(1.0f, acc);
        }
    } else if (is_tw && direct) {
        // the value scales of the first four tiles are requested while the denominator is summed
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
#pragma unroll
            for (uint32_t k = 0; k < PER; ++k) {
                const uint32_t t = u * VAL_TILE + li + k * NTW * 32;
                sc_first[u][k] = (li + k * NTW * 32 < VAL_TILE && t < ctx) ? __ldcg(a.v_scale + slot0 + t) : 0.0f;
            }
    } else if (is_tw && !direct) {
        for (uint32_t i = 0; i < VAL_TBUF && i < n_tiles && !failed; ++i) failed = !transpose_tile(i);
    } else if (warp == PRODUCER_WARP && lane == 0 && !direct) {
        for (uint32_t i = 0; i < VAL_TBUF && i < n_tiles && !failed; ++i) failed = !refill_after(i);
    }
    __syncthreads();
    VAL_MARK(3);
    const float inv = s_inv;
    VAL_MARK(4);
    if (warp < CW) {
        // ---- chains: a zero weight adds +-0 (the CPU loop skips such positions: same bits, the values are finite and the sum
        // starts at +0)
        float o = 0.0f;
        long long t_wait = 0;
        const uint32_t d = tid, fd = vt_swz(d);                    // this thread's dimension
        const uint32_t cbfa = (uint32_t)__cvta_generic_to_shared(s_cb);
        const uint32_t wa0 = (uint32_t)__cvta_generic_to_shared(W + (KV4 ? (size_t)(d / 64) * w_stride : 0));
        for (uint32_t i = 0; i < n_tiles; ++i) {
            const uint32_t tb = i % VAL_TBUF, tl = i * VAL_TILE, n = min(VAL_TILE, ctx - tl);
            if (i + 2 >= n_tiles) pdl_trigger();       // one thread's call releases the CTA: only the chain warps call it
            const long long tw0 = clock64();
            const uint32_t st = i % NST;
            if (direct) {          // the tile's weights (the weight warps run ahead through all tiles) and its bytes
                uint32_t spin = 0;
                while (min(min(s_ready[0], s_ready[1]), min(s_ready[2], s_ready[3])) <= i && ++spin < EXACT_WAIT_LIMIT) {}
                __threadfence_block();
                if (spin >= EXACT_WAIT_LIMIT || !mbar_wait_bounded(bar_full + 8 * st, (i / NST) & 1u)) { failed = true; break; }
            } else if (!mbar_wait_bounded(bar_t_full + 8 * tb, (i / VAL_TBUF) & 1u)) { failed = true; break; }
            t_wait += clock64() - tw0;
            const uint32_t wa = wa0 + 4 * tl;
            // transposed tile: row d, swizzled chunks; direct: the ring stage as it landed, block b = [dimension][16]
            const uint32_t row = direct ? (uint32_t)__cvta_generic_to_shared(stages + (size_t)st * Sm::STAGE) + d * 16 : tiles_t + tb * Sm::TILE_T + d * VAL_TILE;
            auto chunk_at = [&](uint32_t b) { return direct ? row + b * (HD * 16) : row + (((b & ~7u) | ((b ^ fd) & 7u)) << 4); };
            const uint32_t n_full = n / 16, rem = n % 16;
            uint4 x = lds_u32x4(chunk_at(0));
            float4 w0 = lds_f32x4(wa), w1 = lds_f32x4(wa + 16), w2 = lds_f32x4(wa + 32), w3 = lds_f32x4(wa + 48);
            for (uint32_t b = 0; b < n_full; ++b) {
                // the next block's bytes and weights are requested before this block's sixteen steps (past the end of the
                // tile they are in bounds and unused)
                const uint32_t nb = b + 1 < VAL_TILE / 16 ? b + 1 : b;
                const uint4 xn = lds_u32x4(chunk_at(nb));
                const float4 n0 = lds_f32x4(wa + 64 * nb), n1 = lds_f32x4(wa + 64 * nb + 16), n2 = lds_f32x4(wa + 64 * nb + 32), n3 = lds_f32x4(wa + 64 * nb + 48);
                o = value_chain16<KV4>(o, x, w0, w1, w2, w3, cbfa);
                x = xn; w0 = n0; w1 = n1; w2 = n2; w3 = n3;
            }
            if (rem != 0) o = value_chain16<KV4>(o, x, w0, w1, w2, w3, cbfa, rem);
            __syncwarp();
            if (lane == 0) mbar_arrive(direct ? bar_rows_free + 8 * st : bar_t_free + 8 * tb);      // this warp is done with the tile
        }
        if (failed) atomicExch(&s_fail, 1u);
        if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) a.trace[8] = (unsigned long long)t_wait;
        s_o[d] = o;
    } else if (is_tw) {
        // ---- transposing warps: tile by tile, the value weights (p * inv) * v_scale of its positions (per 64-value group for
        // the NF4 cache), then - from the third tile on - the transposition; the scales of the next tile are requested first
        const float *vs = a.v_scale + slot0;
        const uint16_t *vs16 = reinterpret_cast<const uint16_t *>(a.v_scale) + slot0 * NB;
        float sc_next[PER][KV4 ? NB : 1];
        auto load_scales = [&](uint32_t i) {
#pragma unroll
            for (uint32_t k = 0; k < PER; ++k) {
                const uint32_t t = i * VAL_TILE + li + k * NTW * 32;
                const bool on = li + k * NTW * 32 < VAL_TILE && t < ctx;
                const size_t row = on ? ring.slot_of_pos(ring.active_pos(t, seq_len)) : 0;
                if (KV4) {
#pragma unroll
                    for (int g = 0; g < NB; ++g) sc_next[k][g] = on ? bf16_bits_to_f32(__ldcg(vs16 + row * NB + g)) : 0.0f;
                } else {
                    sc_next[k][0] = on ? __ldcg(vs + row) : 0.0f;
                }
            }
        };
        if (direct) {
            // no tile buffers to wait for: the weights of ALL tiles, the scales of four tiles (eight loads per lane) requested
            // at a time, each finished tile published through s_ready
            const float *vsd = a.v_scale + slot0;
            for (uint32_t i0 = 0; i0 < n_tiles; i0 += 4) {
                float sc[4][PER];
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u)
#pragma unroll
                    for (uint32_t k = 0; k < PER; ++k) {
                        const uint32_t t = (i0 + u) * VAL_TILE + li + k * NTW * 32;
                        sc[u][k] = i0 == 0 ? sc_first[u][k] : ((li + k * NTW * 32 < VAL_TILE && t < ctx) ? __ldcg(vsd + t) : 0.0f);
                    }
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    if (i0 + u >= n_tiles) break;
#pragma unroll
                    for (uint32_t k = 0; k < PER; ++k) {
                        const uint32_t t = (i0 + u) * VAL_TILE + li + k * NTW * 32;
                        if (li + k * NTW * 32 < VAL_TILE && t < ctx) W[t] = __fmul_rn(__fmul_rn(W[t], inv), sc[u][k]);
                    }
                    __syncwarp();
                    if (lane == 0) { __threadfence_block(); s_ready[tw] = i0 + u + 1; }
                }
            }
        }
        if (n_tiles > 0 && !direct) load_scales(0);
        for (uint32_t i = 0; i < n_tiles && !failed && !direct; ++i) {
            float sc_cur[PER][KV4 ? NB : 1];
#pragma unroll
            for (uint32_t k = 0; k < PER; ++k)
#pragma unroll
                for (int g = 0; g < (KV4 ? NB : 1); ++g) sc_cur[k][g] = sc_next[k][g];
            if (i + 1 < n_tiles) load_scales(i + 1);
            if (i >= VAL_TBUF) failed = !transpose_tile(i);
#pragma unroll
            for (uint32_t k = 0; k < PER; ++k) {
                const uint32_t t = i * VAL_TILE + li + k * NTW * 32;
                if (li + k * NTW * 32 < VAL_TILE && t < ctx) {
                    const float p_norm = __fmul_rn(W[t], inv);
                    if (KV4) {
#pragma unroll
                        for (int g = NB - 1; g >= 0; --g) W[(size_t)g * w_stride + t] = __fmul_rn(p_norm, sc_cur[k][g]);
                    } else {
                        W[t] = __fmul_rn(p_norm, sc_cur[k][0]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_t_full + 8 * (i % VAL_TBUF));
        }
        if (failed) atomicExch(&s_fail, 1u);
    } else if (warp == PRODUCER_WARP && lane == 0) {
        for (uint32_t i = direct ? 0u : VAL_TBUF; i < n_tiles && !failed; ++i) failed = !refill_after(i);
        if (failed) atomicExch(&s_fail, 1u);
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
    size_t smem = ValSmem<HD, KV4>::bytes(a.ctx_cap, !KV4 && a.v_t != nullptr && a.ring.window == 0);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    // One token: few CTAs, each a latency chain.  Asking for more than half an SM's shared memory keeps two of them off the
    // same SM (the block scheduler otherwise puts them wherever the scores kernel frees room first, and chain warps that
    // share a scheduler take turns: 103k against 86k cycles for 8192 positions).  Batches fill the SMs anyway.
    if (a.n_kv * a.group * n_tok <= 148) smem = std::max<size_t>(smem, 116 * 1024);
    cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(attn_values_kernel<HD, KV4>), smem);
    if (e != cudaSuccess) return e;
    const uint32_t nblk = (a.ctx_cap + SCORE_TILE - 1) / SCORE_TILE;
    ExactAttnArgs b = a;
    b.n_tok = n_tok;
    e = launch_kernel(attn_scores_kernel<HD, KV4>, dim3(nblk, a.n_kv, (n_tok + SCORE_TOK - 1) / SCORE_TOK), dim3(SCORE_TILE), 0, s, pdl, b);
    if (e != cudaSuccess) return e;
    return launch_kernel(attn_values_kernel<HD, KV4>, dim3(a.n_kv * a.group, n_tok), dim3(VAL_THREADS), smem, s, pdl, b);
}

size_t attention_exact_max_ctx(uint32_t head_dim, uint32_t kv_bits) {
    const size_t stage = (size_t)VAL_TILE * (kv_bits == 4 ? head_dim / 2 : head_dim);
    const size_t fixed = 128 + (stage > 16 * 1024 ? 2 : 4) * stage + (size_t)VAL_TBUF * VAL_TILE * head_dim;
    const size_t nw = kv_bits == 4 ? head_dim / 64 : 1;
    return (200 * 1024 - fixed) / (4 * nw) - 16;
}

cudaError_t launch_attention_exact(cudaStream_t s, const ExactAttnArgs &a, bool pdl, uint32_t n_tok) {
    if (a.group > 8 || a.group == 0 || n_tok == 0) return cudaErrorInvalidValue;
    if (a.head_dim == 64) return a.kv_bits == 4 ? launch_exact<64, true>(s, a, pdl, n_tok) : launch_exact<64, false>(s, a, pdl, n_tok);
    if (a.head_dim == 128) return a.kv_bits == 4 ? launch_exact<128, true>(s, a, pdl, n_tok) : launch_exact<128, false>(s, a, pdl, n_tok);
    return cudaErrorInvalidValue;
}

}  // namespace k2t
