// Private definitions shared by the files that implement the C ABI (contexts, matrices, helpers).
#pragma once
#include <string>

#include "../../include/kronos_cuda_ffi.h"
#include "k2t_kernels.h"

struct KronosCudaMatrix {
    k2t::DeviceMatrix dm;
    int device;
};

struct DeviceBuffer {   // grow-only scratch owned by a context
    void *p = nullptr;
    size_t cap = 0;
};

struct KronosCudaContext {
    int device = 0;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    std::string err;
    DeviceBuffer x, q, xs, xsum, out, dots, inv, normw;
    uint32_t *d_err = nullptr;      // device word kernels set when a bounded wait gives up
};

namespace k2t {

inline bool fail(KronosCudaContext *ctx, const std::string &msg) {
    if (ctx) ctx->err = msg;
    return false;
}
inline bool cuda_ok(KronosCudaContext *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    return fail(ctx, std::string(what) + ": " + cudaGetErrorString(e));
}
inline bool reserve(KronosCudaContext *ctx, DeviceBuffer &b, size_t bytes) {
    if (bytes <= b.cap) return true;
    if (b.p) { cudaFree(b.p); b.p = nullptr; b.cap = 0; }
    size_t want = (bytes + 255) & ~(size_t)255;
    if (!cuda_ok(ctx, cudaMalloc(&b.p, want), "cudaMalloc(scratch)")) return false;
    b.cap = want;
    return true;
}
inline void release(DeviceBuffer &b) {
    if (b.p) cudaFree(b.p);
    b.p = nullptr; b.cap = 0;
}
// Waits for the stream and reports a kernel-side timeout (a bounded wait that gave up) as an error.
inline bool sync_and_check(KronosCudaContext *ctx, const char *what) {
    uint32_t flag = 0;
    if (!cuda_ok(ctx, cudaMemcpyAsync(&flag, ctx->d_err, 4, cudaMemcpyDeviceToHost, ctx->stream), what) ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), what))
        return false;
    if (flag != 0) {
        // 3 stays set: a peer that did not answer once is not waited for again (the engine must be rebuilt)
        if (flag != 3) cudaMemsetAsync(ctx->d_err, 0, 4, ctx->stream);
        const char *why = flag == 2 ? "the grid barrier of the whole-token kernel gave up waiting"
                        : flag == 3 ? "a tensor- / expert-parallel exchange gave up waiting for a peer rank (the peer has left or never attached; recreate the engines)"
                        : flag == 4 ? "an expert kernel was handed a route id outside the layer's experts"
                        : flag == 5 ? "the attention kernel was launched for a context longer than it was sized for"
                        : "a kernel gave up waiting for its weight pipeline";
        return fail(ctx, std::string(what) + ": " + why + " (results invalid)");
    }
    return true;
}
inline bool make_current(KronosCudaContext *ctx) { return cuda_ok(ctx, cudaSetDevice(ctx->device), "cudaSetDevice"); }


}  // namespace k2t
