// C ABI of the backend (include/kronos_cuda_ffi.h): contexts, matrix upload, kernel entry points.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "k2t_context.h"
#include "k2t_model_kernels.h"

using namespace k2t;

namespace {

std::mutex g_err_mu;
std::string g_create_err = "";

bool check_gemv_args(KronosCudaContext *ctx, const KronosCudaMatrix *m, const void *xq, const void *xs,
                     const void *xsum, size_t n_tok, const void *out, size_t out_stride) {
    if (!m) return fail(ctx, "gemv: matrix is NULL");
    if (m->device != ctx->device) return fail(ctx, "gemv: matrix lives on another device");
    if (!xq || !xs || !out) return fail(ctx, "gemv: NULL buffer");
    if (m->dm.geom.max_odd != 0 && !xsum) return fail(ctx, "gemv: bit-plane matrices need xsum");
    if (n_tok == 0) return fail(ctx, "gemv: n_tok is 0");
    if (out_stride < m->dm.geom.rows) return fail(ctx, "gemv: out_stride smaller than rows");
    return true;
}

// Runs the GEMV over n_tok tokens (tensor-core kernel for batches, 4-token weight passes otherwise).
bool run_gemv(KronosCudaContext *ctx, const KronosCudaMatrix *m, const int8_t *d_xq, const float *d_xs,
              const int32_t *d_xsum, size_t n_tok, float *d_out, size_t out_stride, int32_t *d_dots) {
    uint32_t launched = 0;
    cudaError_t e = launch_gemv_batch(ctx->stream, m->dm, d_xq, d_xs, d_xsum, n_tok, d_out, out_stride, d_dots, ctx->sm_count, ctx->d_err, &launched, true);
    ctx->launches += launched;
    return cuda_ok(ctx, e, "gemv launch");
}

}  // namespace

extern "C" {

KronosCudaContext *kronos_cuda_context_create(int32_t device) {
    auto set_err = [](const std::string &m) { std::lock_guard<std::mutex> l(g_err_mu); g_create_err = m; };
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        set_err(std::string("no usable CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
        return nullptr;
    }
    if (device < 0 || device >= n) { set_err("device index out of range"); return nullptr; }
    cudaDeviceProp prop;
    if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
        set_err(std::string("cannot open device: ") + cudaGetErrorString(e));
        return nullptr;
    }
    if (prop.major != 10) {
        char buf[128];
        std::snprintf(buf, sizeof buf, "device is sm_%d%d; this library holds sm_100a code only", prop.major, prop.minor);
        set_err(buf);
        return nullptr;
    }
    KronosCudaContext *ctx = new (std::nothrow) KronosCudaContext();
    if (!ctx) { set_err("out of host memory"); return nullptr; }
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking)) != cudaSuccess) {
        set_err(std::string("cudaStreamCreate: ") + cudaGetErrorString(e));
        delete ctx;
        return nullptr;
    }
    ctx->stream = ctx->own_stream;
    if ((e = cudaMalloc(reinterpret_cast<void **>(&ctx->d_err), 4)) != cudaSuccess ||
        (e = cudaMemset(ctx->d_err, 0, 4)) != cudaSuccess) {
        set_err(std::string("cudaMalloc(error word): ") + cudaGetErrorString(e));
        cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return nullptr;
    }
    return ctx;
}

void kronos_cuda_context_destroy(KronosCudaContext *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (DeviceBuffer *b : {&ctx->x, &ctx->q, &ctx->xs, &ctx->xsum, &ctx->out, &ctx->dots, &ctx->inv, &ctx->normw}) release(*b);
    if (ctx->d_err) cudaFree(ctx->d_err);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
}

const char *kronos_cuda_last_error(const KronosCudaContext *ctx) {
    if (!ctx) {
        std::lock_guard<std::mutex> l(g_err_mu);
        static thread_local std::string copy;
        copy = g_create_err;
        return copy.c_str();
    }
    return ctx->err.c_str();
}

int32_t kronos_cuda_synchronize(KronosCudaContext *ctx) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!make_current(ctx)) return -1;
    return sync_and_check(ctx, "synchronize") ? 0 : -1;
}

uint64_t kronos_cuda_launch_count(const KronosCudaContext *ctx) { return ctx ? ctx->launches : 0; }

int32_t kronos_cuda_set_stream(KronosCudaContext *ctx, void *cuda_stream) {
    if (!ctx) return -1;
    ctx->err.clear();
    ctx->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
    return 0;
}

KronosCudaMatrix *kronos_cuda_matrix_upload(KronosCudaContext *ctx, const KronosCudaMatrixDesc *desc, uint32_t flags) {
    if (!ctx) return nullptr;
    ctx->err.clear();
    if (!desc) { fail(ctx, "matrix_upload: desc is NULL"); return nullptr; }
    MatrixGeom g;
    std::string why;
    if (!matrix_geometry(*desc, g, why)) { fail(ctx, why); return nullptr; }
    const bool interleave = (flags & KRONOS_CUDA_UPLOAD_GATE_UP_INTERLEAVE) != 0;
    if (interleave && (desc->rows % 128 != 0)) { fail(ctx, "gate_up interleaving requires rows divisible by 128"); return nullptr; }
    if (!make_current(ctx)) return nullptr;
    std::vector<uint8_t> image;
    try {
        image.resize(g.image_bytes());
    } catch (...) { fail(ctx, "matrix_upload: out of host memory"); return nullptr; }
    unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    repack_matrix(*desc, g, interleave, image.data(), std::min(hw, 16u));
    KronosCudaMatrix *m = new (std::nothrow) KronosCudaMatrix();
    if (!m) { fail(ctx, "matrix_upload: out of host memory"); return nullptr; }
    m->device = ctx->device;
    m->dm.geom = g;
    m->dm.device_bytes = image.size();
    if (!cuda_ok(ctx, cudaMalloc(reinterpret_cast<void **>(&m->dm.d_base), image.size()), "cudaMalloc(matrix)")) { delete m; return nullptr; }
    if (!cuda_ok(ctx, cudaMemcpyAsync(m->dm.d_base, image.data(), image.size(), cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpy(matrix)") ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "matrix upload sync")) {
        cudaFree(m->dm.d_base);
        delete m;
        return nullptr;
    }
    return m;
}

KronosCudaMatrix *kronos_cuda_matrix_clone(KronosCudaContext *ctx, const KronosCudaMatrix *src) {
    if (!ctx) return nullptr;
    ctx->err.clear();
    if (!src) { fail(ctx, "matrix_clone: matrix is NULL"); return nullptr; }
    if (src->device != ctx->device) { fail(ctx, "matrix_clone: matrix lives on another device"); return nullptr; }
    if (!make_current(ctx)) return nullptr;
    KronosCudaMatrix *m = new (std::nothrow) KronosCudaMatrix(*src);
    if (!m) { fail(ctx, "matrix_clone: out of host memory"); return nullptr; }
    m->dm.d_base = nullptr;
    if (!cuda_ok(ctx, cudaMalloc(reinterpret_cast<void **>(&m->dm.d_base), src->dm.device_bytes), "cudaMalloc(matrix)")) { delete m; return nullptr; }
    if (!cuda_ok(ctx, cudaMemcpyAsync(m->dm.d_base, src->dm.d_base, src->dm.device_bytes, cudaMemcpyDeviceToDevice, ctx->stream), "cudaMemcpy(matrix)") ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "matrix clone sync")) {
        cudaFree(m->dm.d_base);
        delete m;
        return nullptr;
    }
    return m;
}

void kronos_cuda_matrix_free(KronosCudaContext *ctx, KronosCudaMatrix *m) {
    if (!m) return;
    if (ctx) { cudaSetDevice(ctx->device); cudaStreamSynchronize(ctx->stream); }
    else cudaSetDevice(m->device);
    if (m->dm.d_base) cudaFree(m->dm.d_base);
    delete m;
}

size_t kronos_cuda_matrix_image(const KronosCudaMatrixDesc *desc, uint32_t flags, uint8_t *out, size_t cap) {
    if (!desc) return 0;
    MatrixGeom g;
    std::string why;
    if (!matrix_geometry(*desc, g, why)) return 0;
    const bool interleave = (flags & KRONOS_CUDA_UPLOAD_GATE_UP_INTERLEAVE) != 0;
    if (interleave && (desc->rows % 128 != 0)) return 0;
    const size_t need = g.image_bytes();
    if (out && cap >= need) repack_matrix(*desc, g, interleave, out, 4);
    return need;
}

size_t kronos_cuda_matrix_file_bytes(const KronosCudaMatrix *m) { return m ? m->dm.geom.file_bytes : 0; }
size_t kronos_cuda_matrix_device_bytes(const KronosCudaMatrix *m) { return m ? m->dm.device_bytes : 0; }

int32_t kronos_cuda_fwht_quant_dev(KronosCudaContext *ctx, const float *d_x, size_t n_tok, size_t cols,
                                   const float *d_norm_w, const float *d_inv_rms, uint64_t chunk0, int8_t *d_q,
                                   float *d_scales, int32_t *d_sums) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!d_x || !d_q || !d_scales || !d_sums) return fail(ctx, "fwht_quant: NULL buffer"), -1;
    if (cols == 0 || cols % 64 != 0) return fail(ctx, "fwht_quant: cols must be a positive multiple of 64"), -1;
    if (d_norm_w && !d_inv_rms) return fail(ctx, "fwht_quant: norm_w given without inv_rms"), -1;
    if (n_tok == 0) return 0;
    if (n_tok * (cols / 64) > 0x7fffffffull * 8) return fail(ctx, "fwht_quant: too many chunks"), -1;
    if (!make_current(ctx)) return -1;
    cudaError_t e = launch_fwht_quant(ctx->stream, d_x, d_norm_w, d_inv_rms, (uint32_t)n_tok, (uint32_t)cols, chunk0,
                                      d_q, d_scales, d_sums);
    ctx->launches += 1;
    return cuda_ok(ctx, e, "fwht_quant launch") ? 0 : -1;
}

int32_t kronos_cuda_gemv_dev(KronosCudaContext *ctx, const KronosCudaMatrix *m, const int8_t *d_xq, const float *d_xs,
                             const int32_t *d_xsum, size_t n_tok, float *d_out, size_t out_stride, int32_t *d_int_dots) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!check_gemv_args(ctx, m, d_xq, d_xs, d_xsum, n_tok, d_out, out_stride)) return -1;
    if (!make_current(ctx)) return -1;
    return run_gemv(ctx, m, d_xq, d_xs, d_xsum, n_tok, d_out, out_stride, d_int_dots) ? 0 : -1;
}

int32_t kronos_cuda_fwht_quant(KronosCudaContext *ctx, const float *x, size_t n_tok, size_t cols, const float *norm_w,
                               const float *inv_rms, uint64_t chunk0, int8_t *q, float *scales, int32_t *sums) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!x || !q || !scales || !sums) return fail(ctx, "fwht_quant: NULL buffer"), -1;
    if (cols == 0 || cols % 64 != 0) return fail(ctx, "fwht_quant: cols must be a positive multiple of 64"), -1;
    if (norm_w && !inv_rms) return fail(ctx, "fwht_quant: norm_w given without inv_rms"), -1;
    if (n_tok == 0) return 0;
    if (!make_current(ctx)) return -1;
    const size_t n = n_tok * cols, nch = n_tok * (cols / 64);
    cudaStream_t s = ctx->stream;
    if (!reserve(ctx, ctx->x, n * 4) || !reserve(ctx, ctx->q, n) || !reserve(ctx, ctx->xs, nch * 4) ||
        !reserve(ctx, ctx->xsum, nch * 4) || !reserve(ctx, ctx->normw, cols * 4) || !reserve(ctx, ctx->inv, n_tok * 4))
        return -1;
    if (!cuda_ok(ctx, cudaMemcpyAsync(ctx->x.p, x, n * 4, cudaMemcpyHostToDevice, s), "copy x")) return -1;
    if (norm_w) {
        if (!cuda_ok(ctx, cudaMemcpyAsync(ctx->normw.p, norm_w, cols * 4, cudaMemcpyHostToDevice, s), "copy norm_w") ||
            !cuda_ok(ctx, cudaMemcpyAsync(ctx->inv.p, inv_rms, n_tok * 4, cudaMemcpyHostToDevice, s), "copy inv_rms"))
            return -1;
    }
    if (kronos_cuda_fwht_quant_dev(ctx, (const float *)ctx->x.p, n_tok, cols, norm_w ? (const float *)ctx->normw.p : nullptr,
                                   norm_w ? (const float *)ctx->inv.p : nullptr, chunk0, (int8_t *)ctx->q.p,
                                   (float *)ctx->xs.p, (int32_t *)ctx->xsum.p) != 0)
        return -1;
    if (!cuda_ok(ctx, cudaMemcpyAsync(q, ctx->q.p, n, cudaMemcpyDeviceToHost, s), "copy q") ||
        !cuda_ok(ctx, cudaMemcpyAsync(scales, ctx->xs.p, nch * 4, cudaMemcpyDeviceToHost, s), "copy scales") ||
        !cuda_ok(ctx, cudaMemcpyAsync(sums, ctx->xsum.p, nch * 4, cudaMemcpyDeviceToHost, s), "copy sums") ||
        !cuda_ok(ctx, cudaStreamSynchronize(s), "fwht_quant sync"))
        return -1;
    return 0;
}

int32_t kronos_cuda_gemv(KronosCudaContext *ctx, const KronosCudaMatrix *m, const int8_t *xq, const float *xs,
                         const int32_t *xsum, size_t n_tok, float *out, size_t out_stride, int32_t *int_dots) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!check_gemv_args(ctx, m, xq, xs, xsum, n_tok, out, out_stride)) return -1;
    if (!make_current(ctx)) return -1;
    const MatrixGeom &g = m->dm.geom;
    const size_t n = n_tok * g.cols, nch = n_tok * g.nc, n_out = (n_tok - 1) * out_stride + g.rows;
    const size_t n_dots = int_dots ? n_tok * (size_t)g.rows * g.nc : 0;
    cudaStream_t s = ctx->stream;
    if (!reserve(ctx, ctx->q, n) || !reserve(ctx, ctx->xs, nch * 4) || !reserve(ctx, ctx->xsum, nch * 4) ||
        !reserve(ctx, ctx->out, n_out * 4) || !reserve(ctx, ctx->dots, n_dots * 4))
        return -1;
    if (!cuda_ok(ctx, cudaMemcpyAsync(ctx->q.p, xq, n, cudaMemcpyHostToDevice, s), "copy xq") ||
        !cuda_ok(ctx, cudaMemcpyAsync(ctx->xs.p, xs, nch * 4, cudaMemcpyHostToDevice, s), "copy xs"))
        return -1;
    if (xsum && !cuda_ok(ctx, cudaMemcpyAsync(ctx->xsum.p, xsum, nch * 4, cudaMemcpyHostToDevice, s), "copy xsum")) return -1;
    if (!cuda_ok(ctx, cudaMemsetAsync(ctx->out.p, 0, n_out * 4, s), "clear out")) return -1;
    if (!run_gemv(ctx, m, (const int8_t *)ctx->q.p, (const float *)ctx->xs.p, xsum ? (const int32_t *)ctx->xsum.p : nullptr,
                  n_tok, (float *)ctx->out.p, out_stride, int_dots ? (int32_t *)ctx->dots.p : nullptr))
        return -1;
    // copy back token by token so gaps between rows and out_stride in the caller's buffer stay untouched
    for (size_t t = 0; t < n_tok; ++t)
        if (!cuda_ok(ctx, cudaMemcpyAsync(out + t * out_stride, (const float *)ctx->out.p + t * out_stride,
                                          (size_t)g.rows * 4, cudaMemcpyDeviceToHost, s), "copy out")) return -1;
    if (int_dots && !cuda_ok(ctx, cudaMemcpyAsync(int_dots, ctx->dots.p, n_dots * 4, cudaMemcpyDeviceToHost, s), "copy dots")) return -1;
    return sync_and_check(ctx, "gemv") ? 0 : -1;
}

static int32_t linear_impl(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *x, size_t n_tok, float *out, bool wait) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!m) return fail(ctx, "linear: matrix is NULL"), -1;
    if (m->device != ctx->device) return fail(ctx, "linear: matrix lives on another device"), -1;
    if (!x || !out) return fail(ctx, "linear: NULL buffer"), -1;
    if (n_tok == 0) return 0;
    if (!make_current(ctx)) return -1;
    const MatrixGeom &g = m->dm.geom;
    const size_t n = n_tok * g.cols, nch = n_tok * g.nc, n_out = n_tok * (size_t)g.rows;
    cudaStream_t s = ctx->stream;
    if (!reserve(ctx, ctx->x, n * 4) || !reserve(ctx, ctx->q, n) || !reserve(ctx, ctx->xs, nch * 4) ||
        !reserve(ctx, ctx->xsum, nch * 4) || !reserve(ctx, ctx->out, n_out * 4))
        return -1;
    if (!cuda_ok(ctx, cudaMemcpyAsync(ctx->x.p, x, n * 4, cudaMemcpyHostToDevice, s), "copy x")) return -1;
    if (kronos_cuda_fwht_quant_dev(ctx, (const float *)ctx->x.p, n_tok, g.cols, nullptr, nullptr, 0, (int8_t *)ctx->q.p,
                                   (float *)ctx->xs.p, (int32_t *)ctx->xsum.p) != 0)
        return -1;
    if (!run_gemv(ctx, m, (const int8_t *)ctx->q.p, (const float *)ctx->xs.p, (const int32_t *)ctx->xsum.p, n_tok,
                  (float *)ctx->out.p, g.rows, nullptr))
        return -1;
    if (!cuda_ok(ctx, cudaMemcpyAsync(out, ctx->out.p, n_out * 4, cudaMemcpyDeviceToHost, s), "copy out")) return -1;
    if (!wait) return 0;
    return sync_and_check(ctx, "linear") ? 0 : -1;
}

int32_t kronos_cuda_moe_route(KronosCudaContext *ctx, const float *router_w, const float *router_bias, const float *x_norm,
                              uint32_t n_experts, uint32_t hidden, uint32_t top_k, int32_t norm_topk, uint32_t scoring,
                              uint32_t *route_ids, float *route_w) {
    if (!ctx) return -1;
    ctx->err.clear();
    if (!router_w || !x_norm || !route_ids || !route_w) return fail(ctx, "moe_route: NULL buffer"), -1;
    if (n_experts < 1 || n_experts > 256 || top_k < 1 || top_k > 32 || hidden == 0 || hidden % 4 || scoring > 2)
        return fail(ctx, "moe_route: 1..256 experts, 1..32 routes, hidden a multiple of 4, scoring 0..2"), -1;
    if (!make_current(ctx)) return -1;
    const size_t wb = (size_t)n_experts * hidden * 4;
    // scratch: weights | bias | x | logits[256] | done word | ids[32] | weights[32]
    const size_t off_b = wb, off_x = off_b + (size_t)n_experts * 4, off_l = off_x + (size_t)hidden * 4, off_d = off_l + 1024, off_i = off_d + 16, off_w = off_i + 128;
    if (!reserve(ctx, ctx->x, off_w + 128)) return -1;
    uint8_t *base = static_cast<uint8_t *>(ctx->x.p);
    cudaStream_t s = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpyAsync(base, router_w, wb, cudaMemcpyHostToDevice, s), "copy router") ||
        (router_bias && !cuda_ok(ctx, cudaMemcpyAsync(base + off_b, router_bias, (size_t)n_experts * 4, cudaMemcpyHostToDevice, s), "copy router bias")) ||
        !cuda_ok(ctx, cudaMemcpyAsync(base + off_x, x_norm, (size_t)hidden * 4, cudaMemcpyHostToDevice, s), "copy x") ||
        !cuda_ok(ctx, cudaMemsetAsync(base + off_d, 0, 16, s), "clear counter"))
        return -1;
    RouterArgs ra{};
    ra.w = reinterpret_cast<const float *>(base); ra.bias = router_bias ? reinterpret_cast<const float *>(base + off_b) : nullptr;
    ra.x = reinterpret_cast<const float *>(base + off_x);
    ra.n_experts = n_experts; ra.hidden = hidden; ra.top_k = top_k; ra.norm_topk = norm_topk; ra.scoring = scoring;
    ra.route_ids = reinterpret_cast<uint32_t *>(base + off_i); ra.route_w = reinterpret_cast<float *>(base + off_w);
    ra.logits = reinterpret_cast<float *>(base + off_l); ra.done = reinterpret_cast<uint32_t *>(base + off_d);
    const uint32_t k = std::min(top_k, n_experts);
    ctx->launches += 1;
    if (!cuda_ok(ctx, launch_moe_router(s, ra, false), "moe_router") ||
        !cuda_ok(ctx, cudaMemcpyAsync(route_ids, ra.route_ids, k * 4, cudaMemcpyDeviceToHost, s), "copy routes") ||
        !cuda_ok(ctx, cudaMemcpyAsync(route_w, ra.route_w, k * 4, cudaMemcpyDeviceToHost, s), "copy routes") ||
        !sync_and_check(ctx, "moe_route"))
        return -1;
    return (int32_t)k;
}

int32_t kronos_cuda_linear(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *x, size_t n_tok, float *out) {
    return linear_impl(ctx, m, x, n_tok, out, true);
}

int32_t kronos_cuda_linear_async(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *x, size_t n_tok, float *out) {
    return linear_impl(ctx, m, x, n_tok, out, false);
}

}  // extern "C"
