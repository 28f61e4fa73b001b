// kronos_cuda_linear_noalloc: y = W * rotate_quantize(x) on device buffers without allocating anything.
//
// Who needs this: hosts that must not (or cannot) call cudaMalloc on the decode path - an engine whose
// device memory is one arena planned at start-up, a real-time loop where the allocator's implicit
// device synchronisation is not acceptable, a process running under a memory cap that the driver
// allocator is not allowed to exceed.  kronos_cuda_linear keeps the quantized activations between its
// two kernels in scratch buffers the context grows with cudaMalloc on demand; this variant keeps
// them in a fixed array that is part of the library image instead.
//
// The scratch is a file-scope __device__ array: every GPU that loads the library holds its
// KRONOS_CUDA_NOALLOC_SCRATCH_BYTES until the process exits.  All calls (all contexts, all streams) on
// one device share it, and it keeps whatever the previous call left there:
//   * nothing in it has to start at zero - each call writes every byte it later reads (the int8
//     activations, their scales and sums of the tokens in flight) before the GEMV kernel runs;
//   * two calls that overlap on the GPU (different streams, or different contexts) race on it.
//     Calls issued on one stream are ordered and safe.
// In host code the array's name is only a host-side stand-in; the device address is fetched once per
// device with cudaGetSymbolAddress (that device current) and cached.  That happens in the first call
// on a device, so make the first call before any stream capture begins.
#include <mutex>

#include "k2t_context.h"

using namespace k2t;

namespace {

constexpr size_t kMaxCols = KRONOS_CUDA_NOALLOC_MAX_COLS;
constexpr size_t kTokens = 4;                                   // tokens per pass through the scratch
constexpr size_t kQBytes = kTokens * kMaxCols;                  // int8 activations
constexpr size_t kSBytes = kTokens * (kMaxCols / 64) * 4;       // fp32 scales; the int32 sums take the same
static_assert(kQBytes + 2 * kSBytes == KRONOS_CUDA_NOALLOC_SCRATCH_BYTES, "scratch size and header disagree");

static __device__ __align__(256) unsigned char g_noalloc_scratch[KRONOS_CUDA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned char *g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch on ctx's device (which must be current). Looked up once per device.
unsigned char *scratch_for(KronosCudaContext *ctx) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices) { fail(ctx, "linear_noalloc: device index too large"); return nullptr; }
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_scratch_addr[ctx->device] == nullptr) {
        void *p = nullptr;
        if (!cuda_ok(ctx, cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)")) return nullptr;
        g_scratch_addr[ctx->device] = static_cast<unsigned char *>(p);
    }
    return g_scratch_addr[ctx->device];
}

}  // namespace

extern "C" int32_t kronos_cuda_linear_noalloc(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *d_x,
                                              size_t n_tok, float *d_out) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!m) return fail(ctx, "linear_noalloc: matrix is NULL"), -1;
    if (m->device != ctx->device) return fail(ctx, "linear_noalloc: matrix lives on another device"), -1;
    if (!d_x || !d_out) return fail(ctx, "linear_noalloc: NULL buffer"), -1;
    const MatrixGeom &g = m->dm.geom;
    if (g.cols > kMaxCols)
        return fail(ctx, "linear_noalloc: matrix has " + std::to_string(g.cols) + " columns, the static scratch holds at most " +
                             std::to_string(kMaxCols) + " (use kronos_cuda_linear)"), -1;
    if (n_tok == 0) return 0;
    if (!make_current(ctx)) return -1;
    unsigned char *base = scratch_for(ctx);
    if (!base) return -1;
    int8_t *q = reinterpret_cast<int8_t *>(base);
    float *xs = reinterpret_cast<float *>(base + kQBytes);
    int32_t *xsum = reinterpret_cast<int32_t *>(base + kQBytes + kSBytes);
    // tokens go through the scratch four at a time; launches on one stream run in order, so a pass
    // may reuse the scratch of the pass before it
    for (size_t t0 = 0; t0 < n_tok; t0 += kTokens) {
        const uint32_t n = (uint32_t)std::min(kTokens, n_tok - t0);
        cudaError_t e = launch_fwht_quant(ctx->stream, d_x + t0 * g.cols, nullptr, nullptr, n, g.cols, 0, q, xs, xsum);
        ctx->launches += 1;
        if (!cuda_ok(ctx, e, "linear_noalloc: fwht_quant launch")) return -1;
        uint32_t launched = 0;
        e = launch_gemv(ctx->stream, m->dm, q, xs, xsum, n, d_out + t0 * g.rows, g.rows, nullptr, ctx->sm_count, ctx->d_err, &launched, true);
        ctx->launches += launched;
        if (!cuda_ok(ctx, e, "linear_noalloc: gemv launch")) return -1;
    }
    return 0;
}
