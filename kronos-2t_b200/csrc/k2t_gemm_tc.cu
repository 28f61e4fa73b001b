// Wide-batch quantized GEMM on the tensor cores (prompt batches): the same arithmetic contract as the GEMV / small-N
// kernels (k2t_gemv_core.cuh; reference batch forms src/kernels/simd_lut.rs:4228-4331, 6689-7029), for 16..64 tokens per
// weight pass instead of 4.
//
// What the tensor cores can take over without changing a bit of the result is the INTEGER part: per row r, token t and
// 64-column chunk c the exact int32 dot  a = sum_i code_i * q_i.  The fp32 part stays a chain per (row, token) in
// ascending chunk order, f = fmaf((float)dot * xs[t][c], w_scale[r][c / sgc], f), and runs on the CUDA cores out of
// tensor memory.  So a CTA (128 rows x N tokens, N = 16 / 32 / 64; 25 warps) walks the chunks of its rows once:
//   * DECODE groups of 128 threads (thread = row; group g takes chunks g, g + G, ...): the row's cell of the chunk (2..3 x
//     16 bytes, fetched eight chunks ahead with `cp.async` into a thread-private ring) is expanded to 64 int8 codes and
//     stored as the A operand in the K-major no-swizzle UMMA layout (8-row x 16-byte core matrices); the same threads move
//     the tokens' int8 activations of the chunk into the B operand (N x 64 bytes, same layout);
//   * one thread issues two `tcgen05.mma.kind::i8` (M 128, N, K 32 each; signed x signed, int32 accumulators) per chunk into
//     the accumulator buffer of the chunk's stage (six stages, six buffers in tensor memory) and commits to the stage's
//     `done` mbarrier, which both frees the operands and publishes the accumulator;
//   * EPILOGUE warps (thread = row, two or four warps per 32-lane quarter splitting the tokens) read the chunk's dots of
//     their row with `tcgen05.ld` one chunk ahead of the arithmetic, hand the buffer back (`drained`: the decode threads
//     wait for it before they refill the stage, so the issuing thread never waits for the epilogue), and advance their
//     chains: one integer multiply-add folds the bit-plane correction (2a - (2^B - 1) * xsum) and the int -> float
//     conversion constant, then add, multiply, fma.  The row's weight scale of the chunk comes from shared memory: the
//     decode thread of the row carries it through its ring and publishes it per chunk (a row-strided global load in the
//     epilogue itself occupied the load / store path for 280 cycles per chunk, in front of the waits on the barriers).
// Activation scales and corrections of the CTA's tokens sit in shared memory, chunk-major, for the whole launch.  Every
// wait is bounded; a wait that gives up raises the context's error word and all roles leave their loops, the tensor
// memory is freed and the kernel returns.
// Measured (B200): 32 chunks in 14-24 us, 128 chunks in 49 us, whatever the rows up to one CTA per SM - 0.36 us per chunk
// for 16-token tiles, 0.65 us for 64: the serial hand-offs of a chunk through the roles and the per-chunk work of a warp
// (13 M warp instructions per 2048 x 16384 x 64 launch, half an instruction per scheduler and cycle, tensor pipe 4%
// active), not the tensor cores or HBM, bound it.  Against 4-token passes it wins from about 16 tokens on.
#include <algorithm>
#include <cstdlib>

#include "k2t_gemv_core.cuh"

namespace k2t {

int fill_gemv_args(const DeviceMatrix &m, bool has_xsum, GemvArgs &a);      // k2t_gemv.cu

namespace {

constexpr uint32_t TC_M = 128;              // rows per CTA = UMMA M
constexpr uint32_t TC_STAGES = 6;           // operand stages (A 8 KiB + B N x 64 bytes each), each with its own accumulator buffer
constexpr uint32_t TC_ACC = TC_STAGES;      // accumulator buffers in tensor memory (N columns each): chunk c uses stage and buffer c % 6
constexpr uint32_t TC_PF = 8;               // ring slots of the raw weights / activations (slot = chunk % TC_PF): chunks requested ahead
constexpr uint32_t TC_WARPS = 25;           // 24 decode + epilogue warps and the issuing warp
constexpr uint32_t TC_THREADS = TC_WARPS * 32;
// The 24 working warps are divided by the tile's width.  64 tokens: the chains are the larger part - sixteen epilogue warps
// (four per 32-lane quarter, a quarter of the tokens each) and two decode groups of 128 threads (group g expands chunks
// g, g + 2, ...).  16 / 32 tokens: the expansion is - eight epilogue warps (half the tokens each), four decode groups.
template <int N> struct TcRoles {
    static constexpr uint32_t EPI_WARPS = N == 64 ? 16 : 8;
    static constexpr uint32_t GROUPS = (TC_WARPS - 1 - EPI_WARPS) / 4;
    static constexpr uint32_t PFG = TC_PF / GROUPS;          // own chunks a decode group requests ahead
    static constexpr uint32_t NQ = N / (EPI_WARPS / 4);       // tokens per epilogue warp
};
constexpr uint32_t TC_A_STAGE = TC_M * 64;
constexpr uint32_t TC_HEADER = 1024;        // mbarriers, tensor-memory address, abort word
constexpr uint32_t TC_SMEM_MAX = 227u * 1024u;
constexpr uint32_t TC_LBO = 128, TC_SBO = 512;      // K-major no-swizzle: next core matrix along K / next 8-row group
constexpr int TC_MAGIC_I = 0x4B400000;      // bits of 12582912.0f = 1.5 * 2^23: as_float(MAGIC + d) - 12582912.0f == (float)d for |d| < 2^22
constexpr float TC_MAGIC_F = 12582912.0f;

__host__ __device__ constexpr uint32_t tc_tmem_cols(uint32_t n) { return TC_ACC * n <= 128 ? 128u : TC_ACC * n <= 256 ? 256u : 512u; }     // allocations are powers of two

template <int FMT> __host__ __device__ constexpr uint32_t tc_cell() { return Cell<FMT>::B0 + Cell<FMT>::B1 + Cell<FMT>::B2; }

struct TcLayout { uint32_t a, b, wring, bring, xs, bias, nz, ws, total; };
constexpr uint32_t TC_WS_SLOTS = 16;        // chunks the per-row weight scales stay published (more than the stages in flight)
template <int FMT, int N> __host__ __device__ inline TcLayout tc_layout(uint32_t nc) {
    TcLayout L;
    L.a = TC_HEADER;
    L.b = L.a + TC_STAGES * TC_A_STAGE;
    L.wring = L.b + TC_STAGES * N * 64;
    L.bring = L.wring + TC_PF * TC_M * (tc_cell<FMT>() + 4);      // a row's cell and the 4-byte word that holds its scale
    L.xs = L.bring + TC_PF * N * 64;
    L.bias = L.xs + nc * N * 4;
    L.nz = L.bias + (is_bitplane<FMT>() ? nc * N * 4 : 0u);       // codebook formats have no correction term
    L.ws = (L.nz + nc + 15u) & ~15u;                              // bf16 scale of (chunk % TC_WS_SLOTS, row)
    L.total = (L.ws + TC_WS_SLOTS * TC_M * 2 + 127u) & ~127u;
    return L;
}

struct TcArgs {
    GemvArgs g;
    uint32_t n_tok;            // tokens of the whole call; CTA (x, y) takes rows 128x.. and tokens N*y..
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {     // src_bytes 0: zero fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds_u32x4_tc(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint2 lds_u32x2_tc(uint32_t saddr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(saddr));
    return v;
}
__device__ __forceinline__ void sts_u32x4_tc(uint32_t saddr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t lds_u32_tc(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16_tc(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ void sts_u16_tc(uint32_t saddr, uint32_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(saddr), "r"(v) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int K> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr) : "memory");
}
// Waits for the thread's tensor-memory loads.  The loaded registers are operands so that no use of them can be scheduled
// above the wait (the loads complete asynchronously; the compiler sees only register names).
__device__ __forceinline__ void tc_ld_wait(int (&v)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])::"memory");
}
__device__ __forceinline__ void tc_ld_wait(int (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]),
                   "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])::"memory");
}
template <int K> __device__ __forceinline__ void tc_ld(uint32_t taddr, int (&v)[K]) {
#pragma unroll
    for (int k = 0; k < K / 8; ++k) tc_ld8(taddr + k * 8, *reinterpret_cast<int(*)[8]>(&v[k * 8]));
}
// Bounded wait on an mbarrier phase; gives up when the limit runs out or another role has given up.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_w) {
    for (uint32_t spin = 0; spin < WAIT_LIMIT; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u && *abort_w != 0) return false;
    }
    *abort_w = 1;
    return false;
}
#ifdef K2T_TC_TRACE
// Build-time diagnostic: cycles CTA 0 spends in the phases of its three roles (lane 0 of the first warp of each).
__device__ unsigned long long g_tc_trace[32];
#define TC_ACC_T(slot) do { if (blockIdx.x == 0 && blockIdx.y == 0) { const long long _t1 = clock64(); trace_acc[slot] += (unsigned long long)(_t1 - _tl); _tl = _t1; } } while (0)
#else
#define TC_ACC_T(slot) do {} while (0)
#endif

__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    // start address, leading (K) and stride (8-row group) byte offsets in 16-byte units, descriptor version 1, no swizzle
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)(TC_LBO >> 4) << 16) | ((uint64_t)(TC_SBO >> 4) << 32) | (1ull << 46);
}

template <int FMT, int N>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const TcArgs args) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const GemvArgs &a = args.g;
    constexpr uint32_t TC_EPI_WARPS = TcRoles<N>::EPI_WARPS, TC_GROUPS = TcRoles<N>::GROUPS, TC_PFG = TcRoles<N>::PFG, TC_DEC_WARPS = 4 * TC_GROUPS;
    constexpr uint32_t NQ = TcRoles<N>::NQ;              // tokens per epilogue warp
    constexpr uint32_t CELL = tc_cell<FMT>();
    constexpr bool BP = is_bitplane<FMT>();
    const TcLayout L = tc_layout<FMT, N>(a.nc);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t row0 = blockIdx.x * TC_M, tok0 = blockIdx.y * N;
    const uint32_t n_here = min((uint32_t)N, args.n_tok - tok0);
    const uint32_t nc = a.nc;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    // per stage: full (operands written: decode -> issue), done (the chunk's products are in tensor memory: issue -> decode, which may
    // reuse the stage, and -> epilogue), drained (the epilogue has read the accumulator: -> decode, which refills the stage only then,
    // so the issuing thread never waits for the epilogue itself)
    const uint32_t bar_full = sbase, bar_done = sbase + 64, bar_drained = sbase + 128;
    volatile uint32_t *s_tmem = reinterpret_cast<volatile uint32_t *>(smem + 256);
    volatile uint32_t *s_abort = reinterpret_cast<volatile uint32_t *>(smem + 260);

    if (tid == 0) {
        for (uint32_t i = 0; i < TC_STAGES; ++i) { mbar_init(bar_full + 8 * i, TC_M / 32); mbar_init(bar_done + 8 * i, 1); mbar_init(bar_drained + 8 * i, TC_EPI_WARPS); }
        *s_abort = 0;
        fence_mbar_init();
    }
    if (warp == TC_EPI_WARPS + TC_DEC_WARPS) {           // the issuing warp owns the tensor memory: TC_ACC x N columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + 256), "r"(tc_tmem_cols(N)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    if (warp < TC_EPI_WARPS) {
        // ------------------------------------------------------------------ epilogue: thread = row, NQ chains
        const uint32_t quarter = warp & 3u, part = warp >> 2;
        const uint32_t row = row0 + quarter * 32 + lane;
        float *s_xs = reinterpret_cast<float *>(smem + L.xs);
        int *s_bias = reinterpret_cast<int *>(smem + L.bias);
        uint8_t *s_nz = smem + L.nz;
        pdl_wait();
        // tables of the CTA's tokens, chunk-major: xs[c][t] and, for bit-planes, bias[c][t] = conversion constant -
        // (2^B - 1) * xsum[t][c]; nz[c] = no real token has a zero scale in chunk c (no chain step of the chunk is skipped)
        for (uint32_t c = tid; c < nc; c += TC_EPI_WARPS * 32) s_nz[c] = 1;
        asm volatile("bar.sync 1, %0;" ::"r"(TC_EPI_WARPS * 32) : "memory");
        for (uint32_t i = tid; i < nc * N; i += TC_EPI_WARPS * 32) {
            const uint32_t c = i / N, t = i % N;
            float sx = 1.0f;
            int sum = 0;
            if (t < n_here) {
                sx = __ldg(a.xs + (size_t)(tok0 + t) * nc + c);
                if (BP) sum = __ldg(a.xsum + (size_t)(tok0 + t) * nc + c);
                if (sx == 0.0f) s_nz[c] = 0;
            }
            s_xs[i] = sx;
            if (BP) s_bias[i] = TC_MAGIC_I - a.max_odd * sum;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(TC_EPI_WARPS * 32) : "memory");

        float f[NQ];
#pragma unroll
        for (uint32_t t = 0; t < NQ; ++t) f[t] = 0.0f;
        const uint32_t xs_sa = sbase + L.xs + part * NQ * 4, bias_sa = sbase + L.bias + part * NQ * 4;
        const uint32_t taddr0 = tmem + ((quarter * 32u) << 16) + part * NQ;
        const uint32_t ws_sa = sbase + L.ws + (quarter * 32 + lane) * 2;      // the row's scale of chunk c: slot c % TC_WS_SLOTS, written by the decode thread of the row
        bool ok = true;
#ifdef K2T_TC_TRACE
        unsigned long long trace_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long _tl = clock64();
#endif
        // chain steps of chunk c from the dots in v (already waited for)
        auto advance = [&](uint32_t c, const int (&v)[NQ]) {
            const float ws = bf16_bits_to_f32((uint16_t)lds_u16_tc(ws_sa + (c % TC_WS_SLOTS) * (TC_M * 2)));
            const uint32_t xo = c * (N * 4);
            if (s_nz[c] != 0) {
#pragma unroll
                for (uint32_t t = 0; t < NQ; t += 4) {
                    const float4 x4 = lds_f32x4(xs_sa + xo + t * 4);
                    uint4 b4 = make_uint4(TC_MAGIC_I, TC_MAGIC_I, TC_MAGIC_I, TC_MAGIC_I);
                    if (BP) b4 = lds_u32x4_tc(bias_sa + xo + t * 4);
                    const int d0 = BP ? v[t + 0] * 2 + (int)b4.x : v[t + 0] + (int)b4.x, d1 = BP ? v[t + 1] * 2 + (int)b4.y : v[t + 1] + (int)b4.y;
                    const int d2 = BP ? v[t + 2] * 2 + (int)b4.z : v[t + 2] + (int)b4.z, d3 = BP ? v[t + 3] * 2 + (int)b4.w : v[t + 3] + (int)b4.w;
                    f[t + 0] = __fmaf_rn(__fmul_rn(__fadd_rn(__int_as_float(d0), -TC_MAGIC_F), x4.x), ws, f[t + 0]);
                    f[t + 1] = __fmaf_rn(__fmul_rn(__fadd_rn(__int_as_float(d1), -TC_MAGIC_F), x4.y), ws, f[t + 1]);
                    f[t + 2] = __fmaf_rn(__fmul_rn(__fadd_rn(__int_as_float(d2), -TC_MAGIC_F), x4.z), ws, f[t + 2]);
                    f[t + 3] = __fmaf_rn(__fmul_rn(__fadd_rn(__int_as_float(d3), -TC_MAGIC_F), x4.w), ws, f[t + 3]);
                }
            } else {          // a token's zero scale skips its chain step (the reference skips the chunk)
#pragma unroll
                for (uint32_t t = 0; t < NQ; ++t) {
                    const float sx = s_xs[c * N + part * NQ + t];
                    const int bb = BP ? s_bias[c * N + part * NQ + t] : TC_MAGIC_I;
                    const int d = BP ? v[t] * 2 + bb : v[t] + bb;
                    const float r = __fmaf_rn(__fmul_rn(__fadd_rn(__int_as_float(d), -TC_MAGIC_F), sx), ws, f[t]);
                    f[t] = sx != 0.0f ? r : f[t];
                }
            }
        };
        // one step of the software pipeline: the dots of chunk c are on their way into `cur`; once they are in, the buffer goes
        // back to the issuing thread, the dots of chunk c + 1 are requested into `nxt`, and the chains advance meanwhile
        auto step = [&](uint32_t c, int (&cur)[NQ], int (&nxt)[NQ]) -> bool {
            TC_ACC_T(0);
            tc_ld_wait(cur);
            TC_ACC_T(1);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_drained + 8 * (c % TC_ACC));
            TC_ACC_T(4);
            if (c + 1 < nc) {
                TC_ACC_T(5);
                // `done` (the products) and `full` (already complete by then: it orders this thread after the decode threads' stores of the chunk's scales)
                if (!tc_wait(bar_done + 8 * ((c + 1) % TC_ACC), ((c + 1) / TC_ACC) & 1u, s_abort)) return false;
                if (!tc_wait(bar_full + 8 * ((c + 1) % TC_ACC), ((c + 1) / TC_ACC) & 1u, s_abort)) return false;
                TC_ACC_T(6);
                tc_fence_after();
                tc_ld<NQ>(taddr0 + ((c + 1) % TC_ACC) * N, nxt);
            }
            TC_ACC_T(2);
            advance(c, cur);
            TC_ACC_T(3);
            return true;
        };
        int v0[NQ], v1[NQ];
        ok = tc_wait(bar_done, 0u, s_abort) && tc_wait(bar_full, 0u, s_abort);
        if (ok) {
            tc_fence_after();
            tc_ld<NQ>(taddr0, v0);
            for (uint32_t c = 0; c < nc && ok; c += 2) {
                ok = step(c, v0, v1);
                if (ok && c + 1 < nc) ok = step(c + 1, v1, v0);
            }
        }
#ifdef K2T_TC_TRACE
        if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) for (int k = 0; k < 8; ++k) g_tc_trace[k] = trace_acc[k];
#endif
        if (!ok && lane == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
        if (ok && row < a.rows) {
#pragma unroll
            for (uint32_t t = 0; t < NQ; ++t) {
                const uint32_t tt = part * NQ + t;
                if (tt < n_here) a.out[(size_t)(tok0 + tt) * a.out_stride + row] = f[t];
            }
        }
    } else if (warp < TC_EPI_WARPS + TC_DEC_WARPS) {
        // ------------------------------------------------------------------ decode: group g, thread = row
        const uint32_t di = tid - TC_EPI_WARPS * 32, grp = di >> 7, i = di & 127u;
        const uint32_t row_c = min(row0 + i, a.rows_pad - 1);          // rows beyond the matrix repeat the last one (never stored)
        if (FMT == FMT_E8Q2) {
            uint32_t *tab = e8q2_templates_smem();
            if (di < 32) tab[di] = di < 28 ? E8Q2_TEMPLATE_WORDS[di] : 0u;
            asm volatile("bar.sync 2, %0;" ::"r"(TC_DEC_WARPS * 32) : "memory");
        }
        const uint32_t wring = sbase + L.wring, bring = sbase + L.bring;
        constexpr uint32_t B0 = Cell<FMT>::B0, B1 = Cell<FMT>::B1, B2 = Cell<FMT>::B2;
        constexpr uint32_t PIECES = (N * 4 + TC_M - 1) / TC_M;         // 16-byte activation pieces per thread and chunk
        // the row's cells of a pass are consecutive: bases per pass, recomputed when the pass changes
        uint32_t p_cur = 0xffffffffu;
        const uint8_t *wb0 = nullptr, *wb1 = nullptr, *wb2 = nullptr, *wsb = nullptr;
        uint32_t ws_g0 = 0;
        constexpr uint32_t SLOT = TC_M * (CELL + 4);
        auto request_w = [&](uint32_t c) {          // the row's cell of chunk c and the word with its scale -> ring slot c % TC_PF
            const uint32_t p = c >> 5;
            if (p != p_cur) {
                p_cur = p;
                const size_t r_n = (size_t)row_c * tile_chunks(nc, p);
                wb0 = a.plane[0] + tile_code_off(a.rows_pad, B0, p) + r_n * B0;
                if (B1) wb1 = a.plane[1] + tile_code_off(a.rows_pad, B1, p) + r_n * B1;
                if (B2) wb2 = a.plane[2] + tile_code_off(a.rows_pad, B2, p) + r_n * B2;
                wsb = reinterpret_cast<const uint8_t *>(a.scales) + tile_scale_off(a.rows_pad, p) + (size_t)row_c * tile_scale_pitch(nc, a.sgc, p);
                ws_g0 = scale_group_of(a, p * 32);
            }
            const uint32_t cc = c & 31u, slot = wring + (c % TC_PF) * SLOT;
            cp_async4(slot + TC_M * CELL + i * 4, wsb + (((scale_group_of(a, c) - ws_g0) * 2u) & ~3u));
            cp_async16(slot + i * B0, wb0 + cc * B0, 16);
            if (B1 == 16) cp_async16(slot + TC_M * B0 + i * 16, wb1 + cc * 16, 16);
            if (B1 == 8) cp_async8(slot + TC_M * B0 + i * 8, wb1 + cc * 8);
            if (B2 == 16) cp_async16(slot + TC_M * (B0 + B1) + i * 16, wb2 + cc * 16, 16);
            if (B2 == 8) cp_async8(slot + TC_M * (B0 + B1) + i * 8, wb2 + cc * 8);
        };
        // activation pieces of a chunk: piece j = (token j / 4, bytes 16 (j % 4) ..); tokens beyond the batch read as zeros
        const int8_t *xb[PIECES];
        uint32_t xb_bytes[PIECES];
#pragma unroll
        for (uint32_t k = 0; k < PIECES; ++k) {
            const uint32_t j = i + k * TC_M, t = j >> 2, kq = j & 3u, tt = min(t, n_here - 1);
            xb[k] = a.xq + (size_t)(tok0 + tt) * a.cols + kq * 16;
            xb_bytes[k] = t < n_here ? 16u : 0u;
        }
        auto request_b = [&](uint32_t c) {
            const uint32_t slot = bring + (c % TC_PF) * (N * 64);
#pragma unroll
            for (uint32_t k = 0; k < PIECES; ++k) {
                const uint32_t j = i + k * TC_M;
                if (j < N * 4) cp_async16(slot + j * 16, xb[k] + (size_t)c * 64, xb_bytes[k]);
            }
        };
        for (uint32_t k = 0; k < TC_PFG; ++k) if (grp + k * TC_GROUPS < nc) request_w(grp + k * TC_GROUPS);     // weights do not depend on the predecessor
        pdl_wait();
        pdl_trigger();
        for (uint32_t k = 0; k < TC_PFG; ++k) { if (grp + k * TC_GROUPS < nc) request_b(grp + k * TC_GROUPS); cp_async_commit(); }
        bool ok = true;
#ifdef K2T_TC_TRACE
        unsigned long long trace_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long _tl = clock64();
#endif
        for (uint32_t c = grp; c < nc; c += TC_GROUPS) {
            const uint32_t s = c % TC_STAGES;
            TC_ACC_T(0);
            cp_async_wait<TC_PFG - 1>();
            TC_ACC_T(1);
            // raw cell (and the word with the row's scale of this chunk) -> registers
            Raw<FMT> w;
            uint32_t ws_word;
            {
                const uint32_t slot = wring + (c % TC_PF) * SLOT;
                ws_word = lds_u32_tc(slot + TC_M * CELL + i * 4);
                const uint4 p0 = lds_u32x4_tc(slot + i * B0);
                w.w[0] = p0.x; w.w[1] = p0.y; w.w[2] = p0.z; w.w[3] = p0.w;
                if (B1 == 16) { const uint4 p1 = lds_u32x4_tc(slot + TC_M * B0 + i * 16); w.w[4] = p1.x; w.w[5] = p1.y; w.w[6] = p1.z; w.w[7] = p1.w; }
                if (B1 == 8) { const uint2 p1 = lds_u32x2_tc(slot + TC_M * B0 + i * 8); w.w[4] = p1.x; w.w[5] = p1.y; }
                if (B2 == 16) { const uint4 p2 = lds_u32x4_tc(slot + TC_M * (B0 + B1) + i * 16); w.w[8] = p2.x; w.w[9] = p2.y; w.w[10] = p2.z; w.w[11] = p2.w; }
                if (B2 == 8) { const uint2 p2 = lds_u32x2_tc(slot + TC_M * (B0 + B1) + i * 8); w.w[8] = p2.x; w.w[9] = p2.y; }
            }
            uint4 piece[PIECES];
            {
                const uint32_t slot = bring + (c % TC_PF) * (N * 64);
#pragma unroll
                for (uint32_t k = 0; k < PIECES; ++k) {
                    const uint32_t j = i + k * TC_M;
                    piece[k] = j < N * 4 ? lds_u32x4_tc(slot + j * 16) : make_uint4(0, 0, 0, 0);
                }
            }
            // the slot is free again: request the group's chunk after next (one copy group per chunk, also when nothing is left)
            if (c + TC_PF < nc) { request_w(c + TC_PF); request_b(c + TC_PF); }
            cp_async_commit();
            uint32_t u[16];
            decode<FMT>(w, a.cb, u);
            TC_ACC_T(2);
            if (c >= TC_STAGES) {
                ok = tc_wait(bar_done + 8 * s, ((c / TC_STAGES) - 1u) & 1u, s_abort) &&
                     tc_wait(bar_drained + 8 * s, ((c / TC_STAGES) - 1u) & 1u, s_abort);
                if (!ok) break;
            }
            TC_ACC_T(3);
            const uint32_t a_dst = sbase + L.a + s * TC_A_STAGE + (i >> 3) * TC_SBO + (i & 7u) * 16;
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) sts_u32x4_tc(a_dst + k * TC_LBO, u[4 * k], u[4 * k + 1], u[4 * k + 2], u[4 * k + 3]);
            const uint32_t b_stage = sbase + L.b + s * (N * 64);
#pragma unroll
            for (uint32_t k = 0; k < PIECES; ++k) {
                const uint32_t j = i + k * TC_M;
                if (j < N * 4) {
                    const uint32_t t = j >> 2, kq = j & 3u;
                    sts_u32x4_tc(b_stage + (t >> 3) * TC_SBO + kq * TC_LBO + (t & 7u) * 16, piece[k].x, piece[k].y, piece[k].z, piece[k].w);
                }
            }
            {   // the row's scale of this chunk, published for the epilogue (read after the chunk's `done`, which follows this `full`)
                const uint32_t g = scale_group_of(a, c) - scale_group_of(a, c & ~31u);
                sts_u16_tc(sbase + L.ws + ((c % TC_WS_SLOTS) * TC_M + i) * 2, (g & 1u) ? ws_word >> 16 : ws_word & 0xFFFFu);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full + 8 * s);
            TC_ACC_T(4);
        }
#ifdef K2T_TC_TRACE
        if (di == 0 && blockIdx.x == 0 && blockIdx.y == 0) for (int k = 0; k < 5; ++k) g_tc_trace[8 + k] = trace_acc[k];
#endif
        cp_async_wait<0>();
        if (!ok && lane == 0 && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
    } else if (lane == 0) {
        // ------------------------------------------------------------------ issue
        // instruction descriptor: int32 accumulators, signed 8-bit A and B, both K-major, N / 8, M / 16
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((TC_M >> 4) << 24);
        bool ok = true;
#ifdef K2T_TC_TRACE
        unsigned long long trace_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long _tl = clock64();
#endif
        for (uint32_t c = 0; c < nc; ++c) {
            const uint32_t s = c % TC_STAGES, b = c % TC_ACC;
            TC_ACC_T(0);
            ok = tc_wait(bar_full + 8 * s, (c / TC_STAGES) & 1u, s_abort);
            TC_ACC_T(1);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = tc_smem_desc(sbase + L.a + s * TC_A_STAGE), db = tc_smem_desc(sbase + L.b + s * (N * 64));
            const uint32_t d = tmem + b * N;
            tc_mma_i8(d, da, db, idesc, 0u);
            tc_mma_i8(d, da + ((2 * TC_LBO) >> 4), db + ((2 * TC_LBO) >> 4), idesc, 1u);      // columns 32..63: two core matrices on
            tc_commit(bar_done + 8 * s);
            TC_ACC_T(3);
        }
#ifdef K2T_TC_TRACE
        if (blockIdx.x == 0 && blockIdx.y == 0) for (int k = 0; k < 4; ++k) g_tc_trace[16 + k] = trace_acc[k];
#endif
        if (!ok && a.err_flag != nullptr) atomicExch(a.err_flag, 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_EPI_WARPS + TC_DEC_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tc_tmem_cols(N)) : "memory");
    }
}

template <int FMT, int N>
cudaError_t launch_tc_n(cudaStream_t stream, const TcArgs &args, bool pdl) {
    const TcLayout L = tc_layout<FMT, N>(args.g.nc);
    if (L.total > TC_SMEM_MAX) return cudaErrorNotSupported;
    cudaError_t e = allow_dynamic_smem(reinterpret_cast<const void *>(gemm_tc_kernel<FMT, N>), L.total);
    if (e != cudaSuccess) return e;
    const dim3 grid((args.g.rows + TC_M - 1) / TC_M, (args.n_tok + N - 1) / N);
    return launch_kernel(gemm_tc_kernel<FMT, N>, grid, dim3(TC_THREADS), L.total, stream, pdl, args);
}

template <int FMT>
cudaError_t launch_tc_fmt(cudaStream_t stream, const TcArgs &args, int sm_count, bool pdl) {
    // the narrowest token tile that holds the batch, halved while the grid would leave half the SMs idle: a CTA's time per
    // chunk is bounded by the expansion of its weights and the hand-offs between its roles, less by its tokens
    const uint32_t row_tiles = (args.g.rows + TC_M - 1) / TC_M;
    uint32_t n = args.n_tok > 32 ? 64 : args.n_tok > 16 ? 32 : 16;
    while (n > 16 && 2 * row_tiles * ((args.n_tok + n - 1) / n) <= (uint32_t)sm_count) n /= 2;
    for (; n >= 16; n /= 2) {          // a tile whose tables do not fit shared memory: try the next narrower one
        cudaError_t e = n == 64 ? launch_tc_n<FMT, 64>(stream, args, pdl) : n == 32 ? launch_tc_n<FMT, 32>(stream, args, pdl) : launch_tc_n<FMT, 16>(stream, args, pdl);
        if (e != cudaErrorNotSupported) return e;
    }
    return cudaErrorNotSupported;
}

uint32_t tc_min_tokens() {
    static const uint32_t v = [] {
        const char *s = std::getenv("KRONOS_CUDA_TC_MIN_TOKENS");          // 0 = never use the tensor-core path
        return s ? (uint32_t)std::atoi(s) : 16u;
    }();
    return v;
}

}  // namespace

// y[t] = W x[t] for any number of tokens: batches of at least `KRONOS_CUDA_TC_MIN_TOKENS` (16) go to the tensor-core kernel in
// one launch, shorter ones (and calls that ask for the integer dots) to the 4-token weight passes.
cudaError_t launch_gemv_batch(cudaStream_t stream, const DeviceMatrix &m, const int8_t *xq, const float *xs, const int32_t *xsum,
                              size_t n_tok, float *out, size_t out_stride, int32_t *int_dots, int sm_count, uint32_t *err_flag,
                              uint32_t *launches, bool pdl) {
    if (launches) *launches = 0;
    const MatrixGeom &g = m.geom;
    const uint32_t min_tok = tc_min_tokens();
    if (min_tok != 0 && n_tok >= min_tok && n_tok <= 0xFFFFu * 16u && int_dots == nullptr && (g.max_odd == 0 || xsum != nullptr)) {
        TcArgs args;
        int fmt = fill_gemv_args(m, xsum != nullptr, args.g);
        if (fmt == FMT_NF4) fmt = FMT_NF4G;          // the codes themselves go to the tensor cores: plain codebook decode
        args.g.xq = xq; args.g.xs = xs; args.g.xsum = xsum; args.g.out = out; args.g.err_flag = err_flag; args.g.out_stride = out_stride;
        args.n_tok = (uint32_t)n_tok;
        cudaError_t e = cudaErrorNotSupported;
        switch (fmt) {
            case FMT_BP4: e = launch_tc_fmt<FMT_BP4>(stream, args, sm_count, pdl); break;
            case FMT_BP5: e = launch_tc_fmt<FMT_BP5>(stream, args, sm_count, pdl); break;
            case FMT_BP6: e = launch_tc_fmt<FMT_BP6>(stream, args, sm_count, pdl); break;
            case FMT_NF4G: e = launch_tc_fmt<FMT_NF4G>(stream, args, sm_count, pdl); break;
            case FMT_NF3: e = launch_tc_fmt<FMT_NF3>(stream, args, sm_count, pdl); break;
            case FMT_NF5: e = launch_tc_fmt<FMT_NF5>(stream, args, sm_count, pdl); break;
            case FMT_E8Q2: e = launch_tc_fmt<FMT_E8Q2>(stream, args, sm_count, pdl); break;
            default: break;
        }
        if (e != cudaErrorNotSupported) {
            if (e == cudaSuccess && launches) *launches = 1;
            return e;
        }
    }
    const uint32_t max_t = gemv_max_tokens(m);
    for (size_t t0 = 0; t0 < n_tok; t0 += max_t) {
        uint32_t launched = 0;
        const uint32_t n = (uint32_t)std::min<size_t>(max_t, n_tok - t0);
        cudaError_t e = launch_gemv(stream, m, xq + t0 * g.cols, xs + t0 * g.nc, xsum ? xsum + t0 * g.nc : nullptr, n, out + t0 * out_stride, out_stride,
                                    int_dots ? int_dots + t0 * (size_t)g.rows * g.nc : nullptr, sm_count, err_flag, &launched, pdl);
        if (launches) *launches += launched;
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

#ifdef K2T_TC_TRACE
extern "C" int k2t_tc_trace_read(unsigned long long *out) { return (int)cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(unsigned long long) * 32); }
#endif

}  // namespace k2t
