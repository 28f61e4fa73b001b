// Tensor-parallel exchange: sum (all-reduce) or concatenation (all-gather) of one small fp32 vector per rank through
// peer memory over NVLink, one launch per rank, for batch-1 decode where a library collective's latency would dominate.
// No counterpart in the reference (single device).
//
// Every rank owns an exchange buffer: data[2][tp][slot] floats and flags[tp] words.  A call with epoch e (1, 2, ...; the
// parity picks the data half) does, on every rank r:
//   1. store its vector into data[e & 1][r] of EVERY rank's buffer (plain peer stores), then a system-scope fence;
//   2. store e into flags[r] of every rank's buffer (release, system scope);
//   3. wait until its own flags[0 .. tp) are all >= e (acquire, system scope; bounded: after L.wait_polls polls the error word
//      is set to 3 and the kernel carries on with whatever is there, so nothing hangs and the host sees the failure);
//   4. read data[e & 1][0 .. tp) of its OWN buffer through L2 and sum them in rank order, ((v0 + v1) + v2) + ... - every
//      rank gets the same bits - or copy them side by side (gather).
// A rank cannot run two calls ahead of another (step 3 of call e+1 needs everybody's step 2 of e+1, which follows their
// step 4 of e), so the two data halves suffice.  The kernels of the ranks run on different GPUs; they are never launched as
// several ranks on one device.  Loads and stores are ordinary peer accesses: no multicast objects.
#include "k2t_device.cuh"
#include "k2t_tp.h"

namespace k2t {

constexpr uint32_t TP_THREADS = 1024;

__global__ void __launch_bounds__(TP_THREADS) tp_exchange_kernel(const TpLink L, const float *__restrict__ src, float *__restrict__ dst,
                                                                 uint32_t n, uint32_t gather_stride) {
    __shared__ uint32_t s_epoch;
    const uint32_t tid = threadIdx.x;
    pdl_wait();
    pdl_trigger();
    if (tid == 0) s_epoch = *L.epoch + 1;
    __syncthreads();
    const uint32_t e = s_epoch, half = e & 1u;
    for (uint32_t p = 0; p < L.tp; ++p) {
        float4 *to = reinterpret_cast<float4 *>(L.peer_data[p] + ((size_t)half * L.tp + L.rank) * L.slot);
        for (uint32_t i = tid; i < n / 4; i += TP_THREADS) to[i] = __ldcg(reinterpret_cast<const float4 *>(src) + i);
    }
    __threadfence_system();
    __syncthreads();
    int failed = 0;
    if (tid < L.tp) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(L.peer_flags[tid] + L.rank), "r"(e) : "memory");
        // a context whose error word is already set (an earlier exchange gave up: a peer has left) does not wait again
        uint32_t seen = 0, polls = 0;
        const uint32_t limit = __ldcg(L.err) != 0 ? 0u : L.wait_polls;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(L.peer_flags[L.rank] + tid) : "memory");
            if (seen >= e) break;
            if (++polls > limit) { failed = 1; break; }
        }
    }
    if (__syncthreads_or(failed) && tid == 0) atomicExch(L.err, 3u);
    const float *mine = L.peer_data[L.rank] + (size_t)half * L.tp * L.slot;
    for (uint32_t i = tid; i < n / 4; i += TP_THREADS) {
        float4 acc = __ldcg(reinterpret_cast<const float4 *>(mine) + i);
        if (gather_stride != 0) reinterpret_cast<float4 *>(dst)[i] = acc;
        for (uint32_t r = 1; r < L.tp; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(mine + (size_t)r * L.slot) + i);
            if (gather_stride != 0) reinterpret_cast<float4 *>(dst + (size_t)r * gather_stride)[i] = v;
            else { acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w); }
        }
        if (gather_stride == 0) reinterpret_cast<float4 *>(dst)[i] = acc;
    }
    if (tid == 0) *L.epoch = e;
}

cudaError_t launch_tp_exchange(cudaStream_t s, const TpLink &L, const float *src, float *dst, uint32_t n, uint32_t gather_stride, bool pdl) {
    if (n % 4 || n > L.slot || (gather_stride % 4)) return cudaErrorInvalidValue;
    return launch_kernel(tp_exchange_kernel, dim3(1), dim3(TP_THREADS), 0, s, pdl, L, src, dst, n, gather_stride);
}

}  // namespace k2t
