// Small device helpers shared by the kernels (sm_100a).
#pragma once
#include <cstdint>
#include <mutex>
#include <vector>
#include <cuda_runtime.h>

namespace k2t {

// dp4a with unsigned bytes in `a` (codes, possibly pre-scaled) and signed bytes in `b` (int8 activations).
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// dp4a with signed bytes on both sides (codebook centroids x int8 activations).
__device__ __forceinline__ int dp4a_ss(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// (a & b) | c  and  a | (b & c) as single LOP3s
__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t b, uint32_t c) {  // a | (b & c)
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xF8;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// bytewise select: mask ? hi : lo
__device__ __forceinline__ uint32_t lop3_select(uint32_t lo, uint32_t hi, uint32_t mask) {
    uint32_t d;  // (lo & ~mask) | (hi & mask): truth table over (lo, hi, mask) = 0xCA with inputs (mask, hi, lo)
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(d) : "r"(mask), "r"(hi), "r"(lo));
    return d;
}
// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream still runs.  pdl_wait() returns once the predecessor grid has
// completed and its writes are visible; everything a kernel reads that another kernel wrote, and every
// global write, comes after it (weights are immutable and may be fetched before).  pdl_trigger() lets the
// successor start launching; kernels call it AFTER their own pdl_wait(), so that at most two consecutive
// kernels are ever resident together (a kernel two steps back can then no longer refill an SM's L1 with
// lines its successor is about to overwrite).  Both are no-ops for a kernel launched the ordinary way.
#ifndef K2T_TIMELINE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#else
// Build-time diagnostic (-DK2T_TIMELINE): thread 0 of block (0,0,0) of every kernel stamps %globaltimer when its dependency
// wait returns, i.e. when its predecessor has drained.  Consecutive stamps of a chained step are the in-chain durations
// of its kernels (launch gap included), which events around isolated launches cannot show.  The buffer is
// [count, capacity, stamps...]; each translation unit holds its own copy of the pointer, set through the registry below.
// The stamp costs the stamping thread one atomic round trip (well under a microsecond per kernel).
static __device__ unsigned long long *g_timeline;
inline std::vector<void (*)(unsigned long long *)> &timeline_setters() {
    static std::vector<void (*)(unsigned long long *)> v;
    return v;
}
static void timeline_set_here(unsigned long long *p) { cudaMemcpyToSymbol(g_timeline, &p, sizeof p); }
static const int timeline_registered = (timeline_setters().push_back(&timeline_set_here), 0);
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if ((threadIdx.x | threadIdx.y | blockIdx.x | blockIdx.y | blockIdx.z) == 0 && g_timeline != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const unsigned long long i = atomicAdd(g_timeline, 1ull);
        if (i < g_timeline[1]) g_timeline[2 + i] = t;
    }
}
#endif
#ifndef K2T_TRIGGER_AT_EXIT
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#else
__device__ __forceinline__ void pdl_trigger() {}       // measurement build: dependents launch when the CTAs exit
#endif

// Launches `kernel` on `stream`, optionally as a programmatic dependent of the previous kernel in the stream.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Raises a kernel's dynamic shared-memory limit once per (kernel, device) instead of on every launch: the value set so
// far is remembered per device, and cudaFuncSetAttribute is called only for a larger request.  (The attribute belongs
// to the function on the current device, so a process that drives several GPUs sets it on each.)
inline cudaError_t allow_dynamic_smem(const void *kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    constexpr int MAX_DEV = 16, SLOTS = 256;
    struct Entry { const void *fn; size_t bytes[MAX_DEV]; };
    static Entry table[SLOTS] = {};
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    Entry *slot = nullptr;
    for (int i = 0; i < SLOTS && dev < MAX_DEV; ++i) {
        if (table[i].fn == kernel) { slot = &table[i]; break; }
        if (table[i].fn == nullptr) { table[i].fn = kernel; slot = &table[i]; break; }
    }
    if (slot != nullptr && slot->bytes[dev] >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && slot != nullptr) slot->bytes[dev] = bytes;
    return e;
}

// E8Q2 even-coset templates (simd_lut.rs:4354-4383): four magnitudes per entry, packed little-endian.  The decode
// reads them from shared memory (28 words in 28 banks: lanes with different entries do not conflict).
__constant__ uint32_t E8Q2_TEMPLATE_WORDS[28] = {
    0x00000000u, 0x00002020u, 0x00200020u, 0x20000020u, 0x00202000u, 0x20002000u, 0x20200000u, 0x00000040u, 0x00004000u, 0x00400000u,
    0x40000000u, 0x20202020u, 0x00000020u, 0x00002000u, 0x00200000u, 0x20000000u, 0x00202020u, 0x20002020u, 0x20200020u, 0x20202000u,
    0x00000060u, 0x00006000u, 0x00600000u, 0x60000000u, 0x20202040u, 0x20204020u, 0x20402020u, 0x40202020u};

// ------------------------------------------------------------------------------------------------
// bulk-copy pipeline primitives
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// Shared-memory loads by shared-window address (from __cvta_generic_to_shared): where a pointer reaches a loop through a
// struct or a reference the compiler may fall back to generic loads, which cost about twice as much per access.
__device__ __forceinline__ uint32_t lds_u8(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ float4 lds_f32x4(uint32_t saddr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
    return v;
}

// Streaming 128-bit load that does not allocate in L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream(const uint2 *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// Rademacher sign of element i (0..63) of 64-block `block`: the SplitMix64 stream of
// rademacher_sign_masks_64 (src/kernels/hadamard.rs:29-44) evaluated at position i directly.
__device__ __forceinline__ uint32_t rademacher_sign(uint64_t block, uint32_t i) {
    const uint64_t G = 0x9E3779B97F4A7C15ull;
    uint64_t z = G + block * 0xBF58476D1CE4E5B9ull + (uint64_t)(i + 1) * G;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (uint32_t)(z & 1ull) << 31;
}

}  // namespace k2t
