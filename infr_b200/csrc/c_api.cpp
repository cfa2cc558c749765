// extern "C" shell of libinfr_cuda.so: argument checks, locking, error text; no arithmetic here.
#include <cstring>
#include <string>

#include "backend.h"

using infr::CudaBackend;
using infr::Status;

namespace {
thread_local std::string g_create_error;

int32_t finish(infr_cuda_ctx *ctx, const Status &s) {
    if (!s.ok() && ctx && ctx->be) ctx->be->set_error(s);
    return s.code;
}

#define INFR_CTX_OR_RETURN(ctx)                  \
    if (!(ctx) || !(ctx)->be) return INFR_E_INVALID; \
    std::lock_guard<std::mutex> lock_((ctx)->be->mutex())

// Checks that [off, off+need) lies inside the buffer and returns the device address.
Status span(const infr_cuda_buf *b, size_t need, const char *what, uint8_t **out) {
    if (!b) return Status::Err(INFR_E_INVALID, std::string(what) + ": null buffer");
    if (b->len < need)
        return Status::Err(INFR_E_INVALID, std::string(what) + ": buffer holds " + std::to_string(b->len) +
                                               " bytes, call needs " + std::to_string(need));
    *out = static_cast<uint8_t *>(b->ptr);
    return Status::Ok();
}
}  // namespace

extern "C" {

int32_t infr_cuda_create(const infr_cuda_opts *opts, infr_cuda_ctx **out) {
    if (!out) return INFR_E_INVALID;
    infr_cuda_opts o;
    memset(&o, 0, sizeof o);
    if (opts) o = *opts;
    CudaBackend *be = nullptr;
    Status s = CudaBackend::create(o, &be);
    if (!s.ok()) {
        g_create_error = s.msg;
        return s.code;
    }
    *out = new infr_cuda_ctx{be};
    return INFR_OK;
}

void infr_cuda_destroy(infr_cuda_ctx *ctx) {
    if (!ctx) return;
    delete ctx->be;
    delete ctx;
}

int32_t infr_cuda_get_caps(infr_cuda_ctx *ctx, infr_cuda_caps *out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "get_caps: null output"));
    *out = ctx->be->capabilities();
    return INFR_OK;
}

int32_t infr_cuda_last_error(infr_cuda_ctx *ctx, char *dst, size_t cap) {
    const std::string &m = (ctx && ctx->be) ? ctx->be->last_error() : g_create_error;
    if (dst && cap) {
        const size_t n = m.size() < cap - 1 ? m.size() : cap - 1;
        memcpy(dst, m.data(), n);
        dst[n] = 0;
    }
    return (int32_t)m.size();
}

int32_t infr_cuda_alloc(infr_cuda_ctx *ctx, size_t bytes, int32_t usage, infr_cuda_buf **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "alloc: null output"));
    return finish(ctx, ctx->be->alloc(bytes, usage, true, out));
}

int32_t infr_cuda_alloc_uninit(infr_cuda_ctx *ctx, size_t bytes, int32_t usage, infr_cuda_buf **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "alloc_uninit: null output"));
    return finish(ctx, ctx->be->alloc(bytes, usage, false, out));
}

int32_t infr_cuda_wrap(infr_cuda_ctx *ctx, void *device_ptr, size_t bytes, int32_t usage, infr_cuda_buf **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "wrap: null output"));
    return finish(ctx, ctx->be->wrap(device_ptr, bytes, usage, out));
}

int32_t infr_cuda_comm_create(infr_cuda_ctx *ctx, int32_t rank, int32_t world, uint32_t max_floats, infr_cuda_comm **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "comm_create: null output"));
    return finish(ctx, ctx->be->comm_create(rank, world, max_floats, out));
}

int32_t infr_cuda_comm_export(infr_cuda_ctx *ctx, infr_cuda_comm *comm, uint8_t *handle64) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->comm_export(comm, handle64));
}

int32_t infr_cuda_comm_connect(infr_cuda_ctx *ctx, infr_cuda_comm *comm, const uint8_t *handles) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->comm_connect(comm, handles));
}

int32_t infr_cuda_comm_connect_silent(infr_cuda_ctx *ctx, infr_cuda_comm *comm, uint32_t spin_limit) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->comm_connect_silent(comm, spin_limit));
}

int32_t infr_cuda_all_reduce_f32(infr_cuda_ctx *ctx, infr_cuda_comm *comm, infr_cuda_buf *data, uint32_t n) {
    INFR_CTX_OR_RETURN(ctx);
    if (!data || (size_t)n * 4 > data->len) return finish(ctx, Status::Err(INFR_E_INVALID, "all_reduce: buffer smaller than n floats"));
    return finish(ctx, ctx->be->all_reduce_f32(comm, static_cast<float *>(data->ptr), n));
}

void infr_cuda_comm_destroy(infr_cuda_ctx *ctx, infr_cuda_comm *comm) {
    if (!ctx || !ctx->be) return;
    std::lock_guard<std::mutex> lock_(ctx->be->mutex());
    ctx->be->comm_destroy(comm);
}

void *infr_cuda_stream(infr_cuda_ctx *ctx) {
    if (!ctx || !ctx->be) return nullptr;
    return (void *)ctx->be->stream();
}

void infr_cuda_free(infr_cuda_ctx *ctx, infr_cuda_buf *buf) {
    if (!ctx || !ctx->be) return;
    std::lock_guard<std::mutex> lock_(ctx->be->mutex());
    ctx->be->free_buffer(buf);
}

size_t infr_cuda_buf_len(const infr_cuda_buf *buf) { return buf ? buf->len : 0; }
uint64_t infr_cuda_buf_device_ptr(const infr_cuda_buf *buf) { return buf ? (uint64_t)(uintptr_t)buf->ptr : 0; }

int32_t infr_cuda_upload(infr_cuda_ctx *ctx, infr_cuda_buf *dst, const void *src, size_t bytes) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->upload(dst, 0, src, bytes));
}

int32_t infr_cuda_upload_at(infr_cuda_ctx *ctx, infr_cuda_buf *dst, size_t dst_off, const void *src, size_t bytes) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->upload(dst, dst_off, src, bytes));
}

int32_t infr_cuda_download(infr_cuda_ctx *ctx, const infr_cuda_buf *src, void *dst, size_t bytes) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->download(src, dst, bytes));
}

int32_t infr_cuda_copy(infr_cuda_ctx *ctx, const infr_cuda_buf *src, infr_cuda_buf *dst, size_t bytes) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->copy_buffer(src, dst, bytes));
}

int32_t infr_cuda_host_alloc(infr_cuda_ctx *ctx, size_t bytes, void **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "host_alloc: null output"));
    return finish(ctx, ctx->be->cuda_status(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault), "cudaHostAlloc"));
}

void infr_cuda_host_free(infr_cuda_ctx *ctx, void *p) {
    if (!ctx || !ctx->be || !p) return;
    std::lock_guard<std::mutex> lock_(ctx->be->mutex());
    cudaFreeHost(p);
}

int32_t infr_cuda_sync(infr_cuda_ctx *ctx) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->sync());
}

int32_t infr_cuda_compile(infr_cuda_ctx *ctx, const infr_graph_desc *graph, infr_cuda_plan **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!graph || !out) return finish(ctx, Status::Err(INFR_E_INVALID, "compile: null argument"));
    return finish(ctx, ctx->be->compile(*graph, out));
}

void infr_cuda_plan_free(infr_cuda_ctx *ctx, infr_cuda_plan *plan) {
    if (!ctx || !ctx->be) return;
    std::lock_guard<std::mutex> lock_(ctx->be->mutex());
    ctx->be->free_plan(plan);
}

int32_t infr_cuda_execute(infr_cuda_ctx *ctx, infr_cuda_plan *plan, infr_cuda_buf *const *bindings, uint32_t n) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->execute(plan, bindings, n));
}

int32_t infr_cuda_quantize_q8(infr_cuda_ctx *ctx, int32_t gran, const infr_cuda_buf *x, uint32_t rows, uint32_t k,
                              infr_cuda_buf *qs, infr_cuda_buf *d, infr_cuda_buf *sums, infr_cuda_buf *sums16) {
    INFR_CTX_OR_RETURN(ctx);
    if (gran != 32 && gran != 256) return finish(ctx, Status::Err(INFR_E_INVALID, "quantize_q8: granularity must be 32 or 256"));
    uint8_t *px, *pq, *pd, *ps, *p16 = nullptr;
    Status s;
    const size_t n = (size_t)rows * k;
    if (!(s = span(x, n * 4, "quantize_q8 x", &px)).ok() || !(s = span(qs, n, "quantize_q8 qs", &pq)).ok() ||
        !(s = span(d, n / (size_t)gran * 4, "quantize_q8 d", &pd)).ok() ||
        !(s = span(sums, n / 32 * 4, "quantize_q8 sums", &ps)).ok())
        return finish(ctx, s);
    if (sums16 && !(s = span(sums16, n / 16 * 4, "quantize_q8 sums16", &p16)).ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->quantize_q8(gran, (const float *)px, rows, k, (int8_t *)pq, (float *)pd, (int32_t *)ps,
                                            (int32_t *)p16, nullptr, nullptr));
}

int32_t infr_cuda_quantize_q8_1(infr_cuda_ctx *ctx, const infr_cuda_buf *x, uint32_t rows, uint32_t k, infr_cuda_buf *qs,
                                infr_cuda_buf *dact, infr_cuda_buf *sact) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *px, *pq, *pd, *ps;
    Status s;
    const size_t n = (size_t)rows * k;
    if (!(s = span(x, n * 4, "quantize_q8_1 x", &px)).ok() || !(s = span(qs, n, "quantize_q8_1 qs", &pq)).ok() ||
        !(s = span(dact, n / 32 * 2, "quantize_q8_1 dact", &pd)).ok() ||
        !(s = span(sact, n / 32 * 2, "quantize_q8_1 sact", &ps)).ok())
        return finish(ctx, s);
    // The f32 scales and i32 sums the kernel also produces go to the context scratch.
    const size_t nb = n / 32;
    if (!(s = ctx->be->ensure_scratch(nb * 8 + 512)).ok()) return finish(ctx, s);
    float *d32 = reinterpret_cast<float *>(ctx->be->scratch());
    int32_t *s32 = reinterpret_cast<int32_t *>(ctx->be->scratch() + (nb * 4 + 255) / 256 * 256);
    return finish(ctx, ctx->be->quantize_q8(32, (const float *)px, rows, k, (int8_t *)pq, d32, s32, nullptr, (uint16_t *)pd,
                                            (uint16_t *)ps));
}

static Status linear_args(const infr_cuda_buf *w, uint64_t w_off, const infr_cuda_buf *x, const infr_cuda_buf *y, int32_t dtype,
                          uint32_t m, uint32_t in_f, uint32_t out_f, uint8_t **pw, uint8_t **px, uint8_t **py) {
    const int be = infr::block_elems(dtype), bb = infr::block_bytes(dtype);
    if (!bb || (dtype != INFR_DT_Q4K && dtype != INFR_DT_Q6K && dtype != INFR_DT_Q2_0))
        return Status::Err(INFR_E_UNSUPPORTED, "weight dtype code " + std::to_string(dtype) + " is not supported (Q4_K, Q6_K, Q2_0)");
    if (in_f == 0 || in_f % (uint32_t)be) return Status::Err(INFR_E_INVALID, "in_f is not a whole number of weight blocks");
    if (w_off % in_f) return Status::Err(INFR_E_INVALID, "w_off is not row-aligned");
    const size_t bpr = (size_t)(in_f / (uint32_t)be) * (size_t)bb;
    const size_t row0 = (size_t)(w_off / in_f);
    Status s;
    if (!(s = span(w, (row0 + out_f) * bpr, "weight", pw)).ok()) return s;
    *pw += row0 * bpr;
    if (!(s = span(x, (size_t)m * in_f * 4, "x", px)).ok()) return s;
    if (py && !(s = span(y, (size_t)m * out_f * 4, "y", py)).ok()) return s;
    return Status::Ok();
}

int32_t infr_cuda_gemv(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off, const infr_cuda_buf *x,
                       infr_cuda_buf *y, uint32_t m, uint32_t in_f, uint32_t out_f, int32_t act) {
    INFR_CTX_OR_RETURN(ctx);
    if (m > 8) return finish(ctx, Status::Err(INFR_E_INVALID, "gemv: m must be <= 8 (use infr_cuda_linear)"));
    uint8_t *pw, *px, *py;
    Status s = linear_args(w, w_off, x, y, dtype, m, in_f, out_f, &pw, &px, &py);
    if (!s.ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->linear(dtype, pw, (const float *)px, (float *)py, m, in_f, out_f, act));
}

int32_t infr_cuda_linear(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off, const infr_cuda_buf *x,
                         infr_cuda_buf *y, uint32_t m, uint32_t in_f, uint32_t out_f, int32_t act) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pw, *px, *py;
    Status s = linear_args(w, w_off, x, y, dtype, m, in_f, out_f, &pw, &px, &py);
    if (!s.ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->linear(dtype, pw, (const float *)px, (float *)py, m, in_f, out_f, act));
}

int32_t infr_cuda_linear_pair(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w1, uint64_t w_off1, infr_cuda_buf *y1, uint32_t out_f1,
                              const infr_cuda_buf *w2, uint64_t w_off2, infr_cuda_buf *y2, uint32_t out_f2, const infr_cuda_buf *x, uint32_t m,
                              uint32_t in_f, int32_t act) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pw1, *pw2, *px, *py1, *py2;
    Status s = linear_args(w1, w_off1, x, y1, dtype, m, in_f, out_f1, &pw1, &px, &py1);
    if (s.ok()) s = linear_args(w2, w_off2, x, y2, dtype, m, in_f, out_f2, &pw2, &px, &py2);
    if (!s.ok()) return finish(ctx, s);
    if (py1 == py2) return finish(ctx, Status::Err(INFR_E_INVALID, "linear_pair: the two results need different buffers"));
    return finish(ctx, ctx->be->linear_pair(dtype, pw1, (float *)py1, out_f1, pw2, (float *)py2, out_f2, (const float *)px, m, in_f, act));
}

int32_t infr_cuda_gemv_q8(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off, const infr_cuda_buf *qs,
                          const infr_cuda_buf *d, const infr_cuda_buf *sums, const infr_cuda_buf *sums16, infr_cuda_buf *y,
                          uint32_t m, uint32_t in_f, uint32_t out_f) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pw, *pq, *pd, *ps, *p16 = nullptr, *py;
    const int be = infr::block_elems(dtype), bb = infr::block_bytes(dtype);
    if (dtype != INFR_DT_Q4K && dtype != INFR_DT_Q6K && dtype != INFR_DT_Q2_0)
        return finish(ctx, Status::Err(INFR_E_UNSUPPORTED, "gemv_q8: weight dtype is not supported"));
    if (in_f == 0 || in_f % (uint32_t)be || w_off % in_f) return finish(ctx, Status::Err(INFR_E_INVALID, "gemv_q8: in_f / w_off"));
    const int gran = infr::act_gran(dtype);
    const size_t bpr = (size_t)(in_f / (uint32_t)be) * (size_t)bb, row0 = (size_t)(w_off / in_f), n = (size_t)m * in_f;
    Status s;
    if (!(s = span(w, (row0 + out_f) * bpr, "gemv_q8 weight", &pw)).ok() || !(s = span(qs, n, "gemv_q8 qs", &pq)).ok() ||
        !(s = span(d, n / (size_t)gran * 4, "gemv_q8 d", &pd)).ok() || !(s = span(sums, n / 32 * 4, "gemv_q8 sums", &ps)).ok() ||
        !(s = span(y, (size_t)m * out_f * 4, "gemv_q8 y", &py)).ok())
        return finish(ctx, s);
    if (sums16 && !(s = span(sums16, n / 16 * 4, "gemv_q8 sums16", &p16)).ok()) return finish(ctx, s);
    infr::Q8Dev a{(const int8_t *)pq, (const float *)pd, (const int32_t *)ps, (const int32_t *)p16, gran};
    return finish(ctx, ctx->be->gemv_q8(dtype, pw + row0 * bpr, a, (float *)py, m, in_f, out_f));
}

int32_t infr_cuda_gemv_q8_pair(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w1, uint64_t w_off1, infr_cuda_buf *y1, uint32_t out_f1,
                               const infr_cuda_buf *w2, uint64_t w_off2, infr_cuda_buf *y2, uint32_t out_f2, const infr_cuda_buf *qs,
                               const infr_cuda_buf *d, const infr_cuda_buf *sums, const infr_cuda_buf *sums16, uint32_t m, uint32_t in_f) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pw1, *pw2, *pq, *pd, *ps, *p16 = nullptr, *py1, *py2;
    const int be = infr::block_elems(dtype), bb = infr::block_bytes(dtype);
    if (dtype != INFR_DT_Q4K && dtype != INFR_DT_Q6K && dtype != INFR_DT_Q2_0)
        return finish(ctx, Status::Err(INFR_E_UNSUPPORTED, "gemv_q8_pair: weight dtype is not supported"));
    if (in_f == 0 || in_f % (uint32_t)be || w_off1 % in_f || w_off2 % in_f) return finish(ctx, Status::Err(INFR_E_INVALID, "gemv_q8_pair: in_f / w_off"));
    // (the row limit is infr_cuda_gemv_q8's: the backend checks it)
    if (m == 0 || out_f1 == 0 || out_f2 == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "gemv_q8_pair: m and both out_f must be positive"));
    const int gran = infr::act_gran(dtype);
    const size_t bpr = (size_t)(in_f / (uint32_t)be) * (size_t)bb, r1 = (size_t)(w_off1 / in_f), r2 = (size_t)(w_off2 / in_f), n = (size_t)m * in_f;
    Status s;
    if (!(s = span(w1, (r1 + out_f1) * bpr, "gemv_q8_pair weight 1", &pw1)).ok() || !(s = span(w2, (r2 + out_f2) * bpr, "gemv_q8_pair weight 2", &pw2)).ok() ||
        !(s = span(qs, n, "gemv_q8_pair qs", &pq)).ok() || !(s = span(d, n / (size_t)gran * 4, "gemv_q8_pair d", &pd)).ok() ||
        !(s = span(sums, n / 32 * 4, "gemv_q8_pair sums", &ps)).ok() || !(s = span(y1, (size_t)m * out_f1 * 4, "gemv_q8_pair y1", &py1)).ok() ||
        !(s = span(y2, (size_t)m * out_f2 * 4, "gemv_q8_pair y2", &py2)).ok())
        return finish(ctx, s);
    if (sums16 && !(s = span(sums16, n / 16 * 4, "gemv_q8_pair sums16", &p16)).ok()) return finish(ctx, s);
    if (dtype == INFR_DT_Q6K && !p16) return finish(ctx, Status::Err(INFR_E_INVALID, "gemv_q8_pair: Q6_K needs the per-16 sums"));
    infr::Q8Dev a{(const int8_t *)pq, (const float *)pd, (const int32_t *)ps, (const int32_t *)p16, gran};
    return finish(ctx, ctx->be->gemv_q8_pair(dtype, pw1 + r1 * bpr, (float *)py1, out_f1, pw2 + r2 * bpr, (float *)py2, out_f2, a, m, in_f));
}

int32_t infr_cuda_gemv_block_acc(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off,
                                 const infr_cuda_buf *x, infr_cuda_buf *acc, uint32_t in_f, uint32_t out_f) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pw, *px, *pa;
    Status s = linear_args(w, w_off, x, nullptr, dtype, 1, in_f, out_f, &pw, &px, nullptr);
    if (!s.ok()) return finish(ctx, s);
    const size_t per_row = dtype == INFR_DT_Q4K ? (size_t)in_f / 256 * 2 : (dtype == INFR_DT_Q6K ? (size_t)in_f / 256 : (size_t)in_f / 32);
    if (!(s = span(acc, (size_t)out_f * per_row * 4, "acc", &pa)).ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->gemv_block_acc(dtype, pw, (const float *)px, (int32_t *)pa, in_f, out_f));
}

// ---- the other ops of a dense decode step ----
int32_t infr_cuda_rms_norm(infr_cuda_ctx *ctx, const infr_cuda_buf *x, const infr_cuda_buf *weight, infr_cuda_buf *dst, uint32_t rows,
                           uint32_t dim, float eps) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0 || dim == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "rms_norm: rows and dim must be positive"));
    uint8_t *px, *pw, *pd;
    const size_t n = (size_t)rows * dim * 4;
    Status s;
    if (!(s = span(x, n, "rms_norm x", &px)).ok() || !(s = span(weight, (size_t)dim * 4, "rms_norm weight", &pw)).ok() ||
        !(s = span(dst, n, "rms_norm dst", &pd)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->rms_norm((const float *)px, nullptr, nullptr, (const float *)pw, (float *)pd, rows, dim, eps));
}

int32_t infr_cuda_add_rms_norm(infr_cuda_ctx *ctx, const infr_cuda_buf *a, const infr_cuda_buf *b, infr_cuda_buf *sum_dst,
                               const infr_cuda_buf *weight, infr_cuda_buf *norm_dst, uint32_t rows, uint32_t dim, float eps) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0 || dim == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "add_rms_norm: rows and dim must be positive"));
    uint8_t *pa, *pb, *ps, *pw, *pd;
    const size_t n = (size_t)rows * dim * 4;
    Status s;
    if (!(s = span(a, n, "add_rms_norm a", &pa)).ok() || !(s = span(b, n, "add_rms_norm b", &pb)).ok() ||
        !(s = span(sum_dst, n, "add_rms_norm sum_dst", &ps)).ok() || !(s = span(weight, (size_t)dim * 4, "add_rms_norm weight", &pw)).ok() ||
        !(s = span(norm_dst, n, "add_rms_norm norm_dst", &pd)).ok())
        return finish(ctx, s);
    if (pd == ps || pd == pa || pd == pb) return finish(ctx, Status::Err(INFR_E_INVALID, "add_rms_norm: norm_dst must not alias the sum or its inputs"));
    return finish(ctx, ctx->be->rms_norm((const float *)pa, (const float *)pb, (float *)ps, (const float *)pw, (float *)pd, rows, dim, eps));
}

int32_t infr_cuda_rope(infr_cuda_ctx *ctx, const infr_cuda_buf *x, const infr_cuda_buf *positions, infr_cuda_buf *dst, uint32_t rows,
                       uint32_t n_head, uint32_t head_dim, uint32_t rope_dim, float theta, int32_t neox) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0 || n_head == 0 || head_dim == 0 || rope_dim == 0 || rope_dim > head_dim || (rope_dim & 1))
        return finish(ctx, Status::Err(INFR_E_INVALID, "rope: rows, n_head, head_dim positive; rope_dim even and <= head_dim"));
    uint8_t *px, *pp, *pd;
    const size_t n = (size_t)rows * n_head * head_dim * 4;
    Status s;
    if (!(s = span(x, n, "rope x", &px)).ok() || !(s = span(positions, (size_t)rows * 4, "rope positions", &pp)).ok() ||
        !(s = span(dst, n, "rope dst", &pd)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->rope((const float *)px, (const int32_t *)pp, (float *)pd, rows, n_head, head_dim, rope_dim, theta, neox != 0));
}

int32_t infr_cuda_write_kv(infr_cuda_ctx *ctx, const infr_cuda_buf *src, infr_cuda_buf *cache, uint32_t rows, uint32_t row_stride,
                           uint32_t pos) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0 || row_stride == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "write_kv: rows and row_stride must be positive"));
    uint8_t *ps, *pc;
    const size_t n = (size_t)rows * row_stride;
    Status s;
    // the cache holds the whole context: a write past its end is an error, not a ring wrap
    if (!(s = span(src, n * 4, "write_kv src", &ps)).ok() || !(s = span(cache, ((size_t)pos * row_stride + n) * 2, "write_kv cache", &pc)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->write_kv((const float *)ps, pc + (size_t)pos * row_stride * 2, n));
}

namespace {
Status check_attn(const infr_attn_desc *d, const char *what, bool paged = false) {
    if (!d) return Status::Err(INFR_E_INVALID, std::string(what) + ": null descriptor");
    if (d->rows == 0 || d->n_head == 0 || d->n_kv == 0 || d->n_head % d->n_kv)
        return Status::Err(INFR_E_INVALID, std::string(what) + ": rows, n_head, n_kv positive and n_head a multiple of n_kv");
    const uint32_t g = d->n_head / d->n_kv;
    if ((d->head_dim != 64 && d->head_dim != 128) || (g != 1 && g != 2 && g != 4 && g != 8))
        return Status::Err(INFR_E_UNSUPPORTED, std::string(what) + ": head_dim 64 or 128 and n_head / n_kv in {1, 2, 4, 8}");
    if (!paged && d->n_seq > 1 && (d->seq_stride < (uint64_t)(d->pos + d->rows) * d->n_kv * d->head_dim || d->seq_stride % 8))
        return Status::Err(INFR_E_INVALID, std::string(what) + ": seq_stride must cover one sequence's rows and be a multiple of 8 elements");
    return Status::Ok();
}
}  // namespace

Status q8_out_args(const infr_q8_out *o, size_t rows, size_t k, const char *what, infr::Q8Dev *out);
static int32_t attention_entry(infr_cuda_ctx *ctx, const infr_attn_desc *d, const infr_cuda_buf *seq_pos, bool with_pos, const infr_cuda_buf *q,
                               const infr_cuda_buf *k_cache, const infr_cuda_buf *v_cache, infr_cuda_buf *dst, const infr_q8_out *out, bool q8_form) {
    INFR_CTX_OR_RETURN(ctx);
    const char *what = q8_form ? "attention_q8" : "attention";
    Status s = check_attn(d, what);
    if (!s.ok()) return finish(ctx, s);
    const size_t n_seq = d->n_seq ? d->n_seq : 1;
    const size_t qn = n_seq * d->rows * d->n_head * d->head_dim * 4;
    const size_t cn = ((n_seq - 1) * (size_t)d->seq_stride + (size_t)(d->pos + d->rows) * d->n_kv * d->head_dim) * 2;
    uint8_t *pq, *pk, *pv, *pd = nullptr, *pp = nullptr;
    if (!(s = span(q, qn, "attention q", &pq)).ok() || !(s = span(k_cache, cn, "attention k_cache", &pk)).ok() ||
        !(s = span(v_cache, cn, "attention v_cache", &pv)).ok())
        return finish(ctx, s);
    if (with_pos && !(s = span(seq_pos, n_seq * 4, "attention seq_pos", &pp)).ok()) return finish(ctx, s);
    if (q8_form) {
        infr::Q8Dev q8;
        if (!(s = q8_out_args(out, n_seq * d->rows, (size_t)d->n_head * d->head_dim, "attention_q8 output", &q8)).ok()) return finish(ctx, s);
        return finish(ctx, ctx->be->attention(*d, (const float *)pq, pk, pv, nullptr, &q8, (const int32_t *)pp));
    }
    if (!(s = span(dst, qn, "attention dst", &pd)).ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->attention(*d, (const float *)pq, pk, pv, (float *)pd, nullptr, (const int32_t *)pp));
}

int32_t infr_cuda_attention(infr_cuda_ctx *ctx, const infr_attn_desc *d, const infr_cuda_buf *q, const infr_cuda_buf *k_cache,
                            const infr_cuda_buf *v_cache, infr_cuda_buf *dst) {
    return attention_entry(ctx, d, nullptr, false, q, k_cache, v_cache, dst, nullptr, false);
}

int32_t infr_cuda_attention_seqpos(infr_cuda_ctx *ctx, const infr_attn_desc *d, const infr_cuda_buf *seq_pos, const infr_cuda_buf *q,
                                   const infr_cuda_buf *k_cache, const infr_cuda_buf *v_cache, infr_cuda_buf *dst) {
    return attention_entry(ctx, d, seq_pos, true, q, k_cache, v_cache, dst, nullptr, false);
}

int32_t infr_cuda_attention_seqpos_q8(infr_cuda_ctx *ctx, const infr_attn_desc *d, const infr_cuda_buf *seq_pos, const infr_cuda_buf *q,
                                      const infr_cuda_buf *k_cache, const infr_cuda_buf *v_cache, const infr_q8_out *out) {
    return attention_entry(ctx, d, seq_pos, true, q, k_cache, v_cache, nullptr, out, true);
}

// Paged caches: pools of n_pages pages of 128 rows, a table of pages per sequence.
static Status paged_args(const infr_attn_desc *d, const infr_cuda_buf *block_table, uint32_t table_stride, uint32_t n_pages, const infr_cuda_buf *k_pool,
                         const infr_cuda_buf *v_pool, uint8_t **pt, uint8_t **pk, uint8_t **pv) {
    const size_t n_seq = d->n_seq ? d->n_seq : 1;
    const size_t need_pages = ((size_t)d->pos + d->rows + 127) / 128;
    if (n_pages == 0 || n_pages > (1u << 24) || table_stride < need_pages)
        return Status::Err(INFR_E_INVALID, "paged cache: n_pages must be positive and table_stride must cover (pos + rows) / 128 pages");
    const size_t pool = (size_t)n_pages * 128 * d->n_kv * d->head_dim * 2;
    Status s;
    if (!(s = span(block_table, n_seq * table_stride * 4, "paged cache block_table", pt)).ok() || !(s = span(k_pool, pool, "paged cache k_pool", pk)).ok() ||
        !(s = span(v_pool, pool, "paged cache v_pool", pv)).ok())
        return s;
    return Status::Ok();
}

int32_t infr_cuda_attention_paged(infr_cuda_ctx *ctx, const infr_attn_desc *d, const infr_cuda_buf *seq_pos, const infr_cuda_buf *block_table,
                                  uint32_t table_stride, uint32_t n_pages, const infr_cuda_buf *q, const infr_cuda_buf *k_pool,
                                  const infr_cuda_buf *v_pool, infr_cuda_buf *dst, const infr_q8_out *out) {
    INFR_CTX_OR_RETURN(ctx);
    Status s = check_attn(d, "attention_paged", true);
    if (!s.ok()) return finish(ctx, s);
    if ((dst != nullptr) == (out != nullptr)) return finish(ctx, Status::Err(INFR_E_INVALID, "attention_paged: exactly one of dst and out"));
    const size_t n_seq = d->n_seq ? d->n_seq : 1, qn = n_seq * d->rows * d->n_head * d->head_dim * 4;
    uint8_t *pq, *pk, *pv, *pt, *pd = nullptr, *pp = nullptr;
    if (!(s = paged_args(d, block_table, table_stride, n_pages, k_pool, v_pool, &pt, &pk, &pv)).ok() || !(s = span(q, qn, "attention_paged q", &pq)).ok())
        return finish(ctx, s);
    if (seq_pos && !(s = span(seq_pos, n_seq * 4, "attention_paged seq_pos", &pp)).ok()) return finish(ctx, s);
    if (out) {
        infr::Q8Dev q8;
        if (!(s = q8_out_args(out, n_seq * d->rows, (size_t)d->n_head * d->head_dim, "attention_paged output", &q8)).ok()) return finish(ctx, s);
        return finish(ctx, ctx->be->attention(*d, (const float *)pq, pk, pv, nullptr, &q8, (const int32_t *)pp, (const int32_t *)pt, table_stride, n_pages));
    }
    if (!(s = span(dst, qn, "attention_paged dst", &pd)).ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->attention(*d, (const float *)pq, pk, pv, (float *)pd, nullptr, (const int32_t *)pp, (const int32_t *)pt, table_stride, n_pages));
}

int32_t infr_cuda_rope_write_kv_paged(infr_cuda_ctx *ctx, const infr_attn_desc *d, float theta, int32_t neox, infr_cuda_buf *q, const infr_cuda_buf *k,
                                      const infr_cuda_buf *v, const infr_cuda_buf *positions, const infr_cuda_buf *block_table, uint32_t table_stride,
                                      uint32_t n_pages, infr_cuda_buf *k_pool, infr_cuda_buf *v_pool) {
    INFR_CTX_OR_RETURN(ctx);
    Status s = check_attn(d, "rope_write_kv_paged", true);
    if (!s.ok()) return finish(ctx, s);
    const size_t n_seq = d->n_seq ? d->n_seq : 1, rows = n_seq * d->rows;
    uint8_t *pq, *pk, *pv, *pp, *pt, *pkc, *pvc;
    if (!(s = paged_args(d, block_table, table_stride, n_pages, k_pool, v_pool, &pt, &pkc, &pvc)).ok() ||
        !(s = span(q, rows * d->n_head * d->head_dim * 4, "rope_write_kv_paged q", &pq)).ok() ||
        !(s = span(k, rows * d->n_kv * d->head_dim * 4, "rope_write_kv_paged k", &pk)).ok() ||
        !(s = span(v, rows * d->n_kv * d->head_dim * 4, "rope_write_kv_paged v", &pv)).ok() ||
        !(s = span(positions, rows * 4, "rope_write_kv_paged positions", &pp)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->rope_write_kv(*d, theta, neox != 0, (float *)pq, (const float *)pk, (const float *)pv, (const int32_t *)pp, pkc, pvc, -1,
                                              (const int32_t *)pt, table_stride, n_pages));
}

int32_t infr_cuda_rope_write_kv(infr_cuda_ctx *ctx, const infr_attn_desc *d, float theta, int32_t neox, infr_cuda_buf *q, const infr_cuda_buf *k,
                                const infr_cuda_buf *v, const infr_cuda_buf *positions, infr_cuda_buf *k_cache, infr_cuda_buf *v_cache) {
    INFR_CTX_OR_RETURN(ctx);
    Status s = check_attn(d, "rope_write_kv");
    if (!s.ok()) return finish(ctx, s);
    const size_t n_seq = d->n_seq ? d->n_seq : 1, rows = n_seq * d->rows;
    const size_t cn = ((n_seq - 1) * (size_t)d->seq_stride + (size_t)(d->pos + d->rows) * d->n_kv * d->head_dim) * 2;
    uint8_t *pq, *pk, *pv, *pp, *pkc, *pvc;
    if (!(s = span(q, rows * d->n_head * d->head_dim * 4, "rope_write_kv q", &pq)).ok() ||
        !(s = span(k, rows * d->n_kv * d->head_dim * 4, "rope_write_kv k", &pk)).ok() ||
        !(s = span(v, rows * d->n_kv * d->head_dim * 4, "rope_write_kv v", &pv)).ok() ||
        !(s = span(positions, rows * 4, "rope_write_kv positions", &pp)).ok() || !(s = span(k_cache, cn, "rope_write_kv k_cache", &pkc)).ok() ||
        !(s = span(v_cache, cn, "rope_write_kv v_cache", &pvc)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->rope_write_kv(*d, theta, neox != 0, (float *)pq, (const float *)pk, (const float *)pv, (const int32_t *)pp, pkc, pvc));
}

namespace {
// Checks the four outputs of a fused quantiser for `rows` rows of `k` elements.
Status q8_out_args(const infr_q8_out *o, size_t rows, size_t k, const char *what, infr::Q8Dev *out) {
    if (!o) return Status::Err(INFR_E_INVALID, std::string(what) + ": null int8 output descriptor");
    if (k == 0 || k % 256) return Status::Err(INFR_E_INVALID, std::string(what) + ": the row width must be a multiple of 256");
    uint8_t *pq, *pd, *ps, *p16 = nullptr;
    Status s;
    const size_t n = rows * k;
    if (!(s = span(o->qs, n, what, &pq)).ok() || !(s = span(o->d, n / 256 * 4, what, &pd)).ok() || !(s = span(o->sums, n / 32 * 4, what, &ps)).ok())
        return s;
    if (o->sums16 && !(s = span(o->sums16, n / 16 * 4, what, &p16)).ok()) return s;
    *out = infr::Q8Dev{(const int8_t *)pq, (const float *)pd, (const int32_t *)ps, (const int32_t *)p16, 256};
    return Status::Ok();
}
}  // namespace

int32_t infr_cuda_add_rms_norm_q8(infr_cuda_ctx *ctx, const infr_cuda_buf *a, const infr_cuda_buf *b, infr_cuda_buf *sum_dst,
                                  const infr_cuda_buf *weight, uint32_t rows, uint32_t dim, float eps, const infr_q8_out *out) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "add_rms_norm_q8: rows must be positive"));
    infr::Q8Dev q8;
    Status s = q8_out_args(out, rows, dim, "add_rms_norm_q8 output", &q8);
    if (!s.ok()) return finish(ctx, s);
    uint8_t *pa, *pb = nullptr, *ps = nullptr, *pw;
    const size_t n = (size_t)rows * dim * 4;
    if (!(s = span(a, n, "add_rms_norm_q8 a", &pa)).ok() || !(s = span(weight, (size_t)dim * 4, "add_rms_norm_q8 weight", &pw)).ok())
        return finish(ctx, s);
    if (b && (!(s = span(b, n, "add_rms_norm_q8 b", &pb)).ok() || !(s = span(sum_dst, n, "add_rms_norm_q8 sum_dst", &ps)).ok()))
        return finish(ctx, s);
    return finish(ctx, ctx->be->rms_norm_q8((const float *)pa, (const float *)pb, (float *)ps, (const float *)pw, rows, dim, eps, q8));
}

int32_t infr_cuda_gemv_q8_push(infr_cuda_ctx *ctx, infr_cuda_comm *comm, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off, const infr_cuda_buf *qs,
                               const infr_cuda_buf *d, const infr_cuda_buf *sums, const infr_cuda_buf *sums16, uint32_t m, uint32_t in_f,
                               uint32_t out_f) {
    INFR_CTX_OR_RETURN(ctx);
    if (dtype != INFR_DT_Q4K && dtype != INFR_DT_Q6K) return finish(ctx, Status::Err(INFR_E_UNSUPPORTED, "gemv_q8_push: Q4_K and Q6_K weights"));
    if (in_f == 0 || in_f % 256 || w_off % in_f || m == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "gemv_q8_push: m / in_f / w_off"));
    uint8_t *pw, *pq, *pd, *ps, *p16 = nullptr;
    const size_t bpr = (size_t)(in_f / 256) * (size_t)infr::block_bytes(dtype), row0 = (size_t)(w_off / in_f), n = (size_t)m * in_f;
    Status s;
    if (!(s = span(w, (row0 + out_f) * bpr, "gemv_q8_push weight", &pw)).ok() || !(s = span(qs, n, "gemv_q8_push qs", &pq)).ok() ||
        !(s = span(d, n / 256 * 4, "gemv_q8_push d", &pd)).ok() || !(s = span(sums, n / 32 * 4, "gemv_q8_push sums", &ps)).ok())
        return finish(ctx, s);
    if (sums16 && !(s = span(sums16, n / 16 * 4, "gemv_q8_push sums16", &p16)).ok()) return finish(ctx, s);
    infr::Q8Dev a{(const int8_t *)pq, (const float *)pd, (const int32_t *)ps, (const int32_t *)p16, 256};
    return finish(ctx, ctx->be->gemv_q8_push(comm, dtype, pw + row0 * bpr, a, m, in_f, out_f));
}

int32_t infr_cuda_add_rms_norm_q8_pull(infr_cuda_ctx *ctx, infr_cuda_comm *comm, const infr_cuda_buf *a, infr_cuda_buf *sum_dst,
                                       const infr_cuda_buf *weight, uint32_t rows, uint32_t dim, float eps, const infr_q8_out *out) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "add_rms_norm_q8_pull: rows must be positive"));
    infr::Q8Dev q8;
    Status s = q8_out_args(out, rows, dim, "add_rms_norm_q8_pull output", &q8);
    if (!s.ok()) return finish(ctx, s);
    uint8_t *pa, *ps, *pw;
    const size_t n = (size_t)rows * dim * 4;
    if (!(s = span(a, n, "add_rms_norm_q8_pull a", &pa)).ok() || !(s = span(weight, (size_t)dim * 4, "add_rms_norm_q8_pull weight", &pw)).ok() ||
        !(s = span(sum_dst, n, "add_rms_norm_q8_pull sum_dst", &ps)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->rms_norm_q8_pull(comm, (const float *)pa, (float *)ps, (const float *)pw, rows, dim, eps, q8));
}

int32_t infr_cuda_gated_act_q8(infr_cuda_ctx *ctx, const infr_cuda_buf *gate, const infr_cuda_buf *up, uint32_t rows, uint32_t nff,
                               const infr_q8_out *out) {
    INFR_CTX_OR_RETURN(ctx);
    if (rows == 0) return finish(ctx, Status::Err(INFR_E_INVALID, "gated_act_q8: rows must be positive"));
    infr::Q8Dev q8;
    Status s = q8_out_args(out, rows, nff, "gated_act_q8 output", &q8);
    if (!s.ok()) return finish(ctx, s);
    uint8_t *pg, *pu;
    const size_t n = (size_t)rows * nff * 4;
    if (!(s = span(gate, n, "gated_act_q8 gate", &pg)).ok() || !(s = span(up, n, "gated_act_q8 up", &pu)).ok()) return finish(ctx, s);
    return finish(ctx, ctx->be->gated_act_q8((const float *)pg, (const float *)pu, rows, nff, q8));
}

int32_t infr_cuda_attention_q8(infr_cuda_ctx *ctx, const infr_attn_desc *d, const infr_cuda_buf *q, const infr_cuda_buf *k_cache,
                               const infr_cuda_buf *v_cache, const infr_q8_out *out) {
    return attention_entry(ctx, d, nullptr, false, q, k_cache, v_cache, nullptr, out, true);
}

int32_t infr_cuda_gated_act(infr_cuda_ctx *ctx, const infr_cuda_buf *gate, const infr_cuda_buf *up, infr_cuda_buf *dst, uint32_t rows,
                            uint32_t nff) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pg, *pu, *pd;
    const size_t n = (size_t)rows * nff;
    Status s;
    if (!(s = span(gate, n * 4, "gated_act gate", &pg)).ok() || !(s = span(up, n * 4, "gated_act up", &pu)).ok() ||
        !(s = span(dst, n * 4, "gated_act dst", &pd)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->gated_act((const float *)pg, (const float *)pu, (float *)pd, n));
}

int32_t infr_cuda_add(infr_cuda_ctx *ctx, const infr_cuda_buf *a, const infr_cuda_buf *b, infr_cuda_buf *dst, uint64_t n) {
    INFR_CTX_OR_RETURN(ctx);
    uint8_t *pa, *pb, *pd;
    Status s;
    if (!(s = span(a, (size_t)n * 4, "add a", &pa)).ok() || !(s = span(b, (size_t)n * 4, "add b", &pb)).ok() ||
        !(s = span(dst, (size_t)n * 4, "add dst", &pd)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->add((const float *)pa, (const float *)pb, (float *)pd, (size_t)n));
}

int32_t infr_cuda_argmax(infr_cuda_ctx *ctx, const infr_cuda_buf *x, infr_cuda_buf *dst, uint32_t n, uint32_t rows) {
    INFR_CTX_OR_RETURN(ctx);
    if (n == 0 || rows == 0 || rows > 65535) return finish(ctx, Status::Err(INFR_E_INVALID, "argmax: n positive, rows in 1..65535"));
    uint8_t *px, *pd;
    Status s;
    if (!(s = span(x, (size_t)rows * n * 4, "argmax x", &px)).ok() || !(s = span(dst, (size_t)rows * 4, "argmax dst", &pd)).ok())
        return finish(ctx, s);
    return finish(ctx, ctx->be->argmax((const float *)px, (uint32_t *)pd, n, rows));
}

int32_t infr_cuda_moe_ffn(infr_cuda_ctx *ctx, const infr_moe_desc *d, const infr_cuda_buf *x, const infr_cuda_buf *router_x,
                          const infr_cuda_buf *router, const infr_cuda_buf *gate, const infr_cuda_buf *up, const infr_cuda_buf *down,
                          infr_cuda_buf *dst, infr_cuda_buf *sel_ids, infr_cuda_buf *sel_w, infr_cuda_buf *logits) {
    INFR_CTX_OR_RETURN(ctx);
    if (!d) return finish(ctx, Status::Err(INFR_E_INVALID, "moe_ffn: null descriptor"));
    if (d->router_dtype != INFR_DT_F32) return finish(ctx, Status::Err(INFR_E_UNSUPPORTED, "moe_ffn: router weights must be F32"));
    auto bank_bytes = [&](int dt, size_t out_f, size_t in_f) -> size_t {
        const int be = infr::block_elems(dt), bb = infr::block_bytes(dt);
        if (!bb || in_f % (size_t)be) return (size_t)-1;
        return (size_t)(d->n_local ? d->n_local : d->n_expert) * out_f * (in_f / (size_t)be) * (size_t)bb;
    };
    if (d->n_local && ((uint64_t)d->expert_lo + d->n_local > d->n_expert))
        return finish(ctx, Status::Err(INFR_E_INVALID, "moe_ffn: the local expert range leaves [0, n_expert)"));
    const size_t rows = d->rows, ne = d->ne, nff = d->n_ff_exp;
    uint8_t *px, *prx, *pr, *pg, *pu, *pd, *pdst, *pids = nullptr, *pw = nullptr, *plog = nullptr;
    Status s;
    if (!(s = span(x, rows * ne * 4, "moe_ffn x", &px)).ok() || !(s = span(router_x, rows * ne * 4, "moe_ffn router_x", &prx)).ok() ||
        !(s = span(router, (size_t)d->n_expert * ne * 4, "moe_ffn router", &pr)).ok() ||
        !(s = span(gate, bank_bytes(d->gate_dtype, nff, ne), "moe_ffn gate_exps", &pg)).ok() ||
        !(s = span(up, bank_bytes(d->up_dtype, nff, ne), "moe_ffn up_exps", &pu)).ok() ||
        !(s = span(down, bank_bytes(d->down_dtype, ne, nff), "moe_ffn down_exps", &pd)).ok() ||
        !(s = span(dst, rows * ne * 4, "moe_ffn dst", &pdst)).ok())
        return finish(ctx, s);
    if (sel_ids && !(s = span(sel_ids, rows * d->n_used * 4, "moe_ffn sel_ids", &pids)).ok()) return finish(ctx, s);
    if (sel_w && !(s = span(sel_w, rows * d->n_used * 4, "moe_ffn sel_w", &pw)).ok()) return finish(ctx, s);
    if (logits && !(s = span(logits, rows * d->n_expert * 4, "moe_ffn logits", &plog)).ok()) return finish(ctx, s);
    CudaBackend::MoeArgs a{(const float *)px, (const float *)prx, (const float *)pr, pg, pu, pd, d->gate_dtype, d->up_dtype, d->down_dtype,
                           (float *)pdst, d->rows, d->ne, d->n_expert, d->n_used, d->n_ff_exp, d->scale, d->norm_w,
                           (int32_t *)pids, (float *)pw, (float *)plog, d->n_local ? d->expert_lo : 0u, d->n_local ? d->n_local : d->n_expert};
    return finish(ctx, ctx->be->moe_ffn(a));
}

int32_t infr_cuda_capture_begin(infr_cuda_ctx *ctx) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->capture_begin());
}
int32_t infr_cuda_capture_end(infr_cuda_ctx *ctx, infr_cuda_graph **out) {
    INFR_CTX_OR_RETURN(ctx);
    if (!out) return finish(ctx, Status::Err(INFR_E_INVALID, "capture_end: null output"));
    return finish(ctx, ctx->be->capture_end(out));
}
int32_t infr_cuda_graph_launch(infr_cuda_ctx *ctx, infr_cuda_graph *graph) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->graph_launch(graph));
}
void infr_cuda_graph_free(infr_cuda_ctx *ctx, infr_cuda_graph *graph) {
    if (!ctx || !ctx->be) return;
    std::lock_guard<std::mutex> lock_(ctx->be->mutex());
    ctx->be->graph_free(graph);
}
int32_t infr_cuda_timer_start(infr_cuda_ctx *ctx) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->timer_start());
}
int32_t infr_cuda_timer_stop(infr_cuda_ctx *ctx, float *ms) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->timer_stop(ms));
}
int32_t infr_cuda_flush_l2(infr_cuda_ctx *ctx) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->flush_l2());
}
int32_t infr_cuda_tensor_peak_i8(infr_cuda_ctx *ctx, uint32_t n_batches, uint32_t launches, float *ms, double *int8_ops) {
    INFR_CTX_OR_RETURN(ctx);
    return finish(ctx, ctx->be->tensor_peak_i8(n_batches, launches, ms, int8_ops));
}
uint64_t infr_cuda_launch_count(infr_cuda_ctx *ctx) {
    if (!ctx || !ctx->be) return 0;
    std::lock_guard<std::mutex> lock_(ctx->be->mutex());
    return ctx->be->launch_count();
}

}  // extern "C"
