// CudaBackend: device memory, graph walking and op dispatch (host side).
#include "backend.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace infr {

namespace {
std::string fmt(const char *f, ...) __attribute__((format(printf, 1, 2)));
std::string fmt(const char *f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof buf, f, ap);
    va_end(ap);
    return buf;
}
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

Status CudaBackend::cuda_status(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return Status::Ok();
    const int32_t code = e == cudaErrorMemoryAllocation ? INFR_E_OOM : INFR_E_CUDA;
    return Status::Err(code, fmt("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e)));
}

Status CudaBackend::create(const infr_cuda_opts &opts, CudaBackend **out) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0)
        return Status::Err(INFR_E_CUDA, fmt("no CUDA device: %s (this backend has no CPU fallback)",
                                            e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e)));
    if (opts.device < 0 || opts.device >= n)
        return Status::Err(INFR_E_INVALID, fmt("device %d out of range (%d present)", opts.device, n));
    auto *be = new CudaBackend();
    be->device_ = opts.device;
    be->reference_ = opts.reference != 0;
    Status s;
    if (!(s = be->cuda_status(cudaSetDevice(be->device_), "cudaSetDevice")).ok() ||
        !(s = be->cuda_status(cudaGetDeviceProperties(&be->prop_, be->device_), "cudaGetDeviceProperties")).ok()) {
        delete be;
        return s;
    }
    if (be->prop_.major != 10) {
        s = Status::Err(INFR_E_UNSUPPORTED, fmt("device %d is sm_%d%d; this library is built for sm_100a only",
                                                be->device_, be->prop_.major, be->prop_.minor));
        delete be;
        return s;
    }
    be->dev_.sm_count = be->prop_.multiProcessorCount;
    be->dev_.max_smem_optin = (int)be->prop_.sharedMemPerBlockOptin;
    be->dev_.l2_bytes = (size_t)be->prop_.l2CacheSize;
    if (!(s = be->cuda_status(cudaStreamCreateWithFlags(&be->stream_, cudaStreamNonBlocking), "cudaStreamCreate")).ok() ||
        !(s = be->cuda_status(cudaEventCreate(&be->ev0_), "cudaEventCreate")).ok() ||
        !(s = be->cuda_status(cudaEventCreate(&be->ev1_), "cudaEventCreate")).ok()) {
        delete be;
        return s;
    }
    be->gemv_impl_ = opts.gemv_kernel;
    be->mmq_impl_ = opts.mmq_kernel;
    if (!(s = be->cuda_status(cudaHostAlloc((void **)&be->status_host_, 64, cudaHostAllocMapped), "cudaHostAlloc")).ok() ||
        !(s = be->cuda_status(cudaHostGetDevicePointer((void **)&be->status_dev_, be->status_host_, 0), "cudaHostGetDevicePointer")).ok()) {
        delete be;
        return s;
    }
    *be->status_host_ = 0;
    if (!(s = be->cuda_status(cudaHostAlloc((void **)&be->up_ring_, kUpSlots * kUpSlotBytes, cudaHostAllocDefault), "cudaHostAlloc(upload ring)")).ok()) {
        delete be;
        return s;
    }
    for (int i = 0; i < kUpSlots; i++)
        if (!(s = be->cuda_status(cudaEventCreateWithFlags(&be->up_ev_[i], cudaEventDisableTiming), "cudaEventCreate")).ok()) {
            delete be;
            return s;
        }
    *out = be;
    return Status::Ok();
}

// A kernel whose bounded wait expired leaves a non-zero word in mapped host memory.
Status CudaBackend::check_device_status() {
    if (status_host_ && *(volatile uint32_t *)status_host_) {
        const uint32_t v = *(volatile uint32_t *)status_host_;
        *(volatile uint32_t *)status_host_ = 0;
        return Status::Err(INFR_E_TIMEOUT, fmt("a device-side wait expired (kernel status %u); results of this stream are invalid", v));
    }
    return Status::Ok();
}

CudaBackend::~CudaBackend() {
    cudaSetDevice(device_);
    if (stream_) cudaStreamSynchronize(stream_);
    if (scratch_) cudaFree(scratch_);
    if (flush_) cudaFree(flush_);
    for (auto &b : pool_) cudaFree(b.ptr);
    if (status_host_) cudaFreeHost(status_host_);
    if (up_ring_) cudaFreeHost(up_ring_);
    for (cudaEvent_t e : up_ev_)
        if (e) cudaEventDestroy(e);
    if (ev0_) cudaEventDestroy(ev0_);
    if (ev1_) cudaEventDestroy(ev1_);
    if (stream_) cudaStreamDestroy(stream_);
}

infr_cuda_caps CudaBackend::capabilities() const {
    infr_cuda_caps c;
    memset(&c, 0, sizeof c);
    snprintf(c.name, sizeof c.name, "%s", name());
    c.f16 = 1;
    c.i8 = 1;
    c.i8_dot = 1;
    c.integrated = 0;
    c.unified_memory = 0;
    c.decode_replay = 0;
    c.graph_input_inplace = 1;
    c.max_shared_memory_bytes = (uint32_t)dev_.max_smem_optin;
    c.sm_count = (uint32_t)dev_.sm_count;
    c.total_memory_bytes = (uint64_t)prop_.totalGlobalMem;
    c.l2_bytes = (uint64_t)dev_.l2_bytes;
    return c;
}

// ---------------------------------------------------------------------------------------- memory
Status CudaBackend::alloc(size_t bytes, int usage, bool zero, infr_cuda_buf **out) {
    if (capturing_) return Status::Err(INFR_E_INVALID, "alloc during stream capture");
    cudaSetDevice(device_);
    void *p = nullptr;
    // Round up so 16-byte vector accesses on the tail of a row never leave the allocation.
    const size_t padded = align_up(bytes ? bytes : 1, 256);
    Status s = cuda_status(cudaMalloc(&p, padded), "cudaMalloc");
    if (!s.ok()) return s;
    if (zero) {
        s = cuda_status(cudaMemsetAsync(p, 0, padded, stream_), "cudaMemsetAsync");
    } else {
        // only the padding must be defined
        if (padded > bytes) s = cuda_status(cudaMemsetAsync((uint8_t *)p + bytes, 0, padded - bytes, stream_), "cudaMemsetAsync");
    }
    if (!s.ok()) {
        cudaFree(p);
        return s;
    }
    auto *b = new infr_cuda_buf();
    b->ptr = p;
    b->len = bytes;
    b->usage = usage;
    b->uid = next_uid_++;
    *out = b;
    return Status::Ok();
}

Status CudaBackend::wrap(void *device_ptr, size_t bytes, int usage, infr_cuda_buf **out) {
    if (!device_ptr || !bytes) return Status::Err(INFR_E_INVALID, "wrap: null pointer or empty range");
    if ((uintptr_t)device_ptr % 16) return Status::Err(INFR_E_INVALID, "wrap: the device pointer must be 16-byte aligned");
    auto *b = new infr_cuda_buf();
    b->ptr = device_ptr;
    b->len = bytes;
    b->usage = usage;
    b->uid = next_uid_++;
    b->owned = false;
    *out = b;
    return Status::Ok();
}

void CudaBackend::free_buffer(infr_cuda_buf *b) {
    if (!b) return;
    cudaSetDevice(device_);
    if (!capturing_ && b->owned) cudaStreamSynchronize(stream_);  // a non-owning handle frees nothing
    if (b->owned) cudaFree(b->ptr);
    delete b;
}

Status CudaBackend::upload(infr_cuda_buf *dst, size_t dst_off, const void *src, size_t bytes) {
    if (!dst || (!src && bytes)) return Status::Err(INFR_E_INVALID, "upload: null argument");
    if (dst_off > dst->len || bytes > dst->len - dst_off)
        return Status::Err(INFR_E_INVALID, fmt("upload: %zu bytes at offset %zu into a %zu-byte buffer", bytes, dst_off, dst->len));
    if (capturing_) return Status::Err(INFR_E_INVALID, "upload during stream capture");
    cudaSetDevice(device_);
    // The caller may reuse `src` as soon as this returns (the trait takes a borrowed slice).  A small upload (a
    // decode step's activations) is copied into a pinned slot of the context's ring and sent from there, so that
    // the call returns without waiting for the stream; a slot is reused only after its copy has completed.
    if (bytes <= kUpSlotBytes) {
        const int slot = up_next_;
        up_next_ = (up_next_ + 1) % kUpSlots;
        Status s = cuda_status(cudaEventSynchronize(up_ev_[slot]), "upload slot");
        if (!s.ok()) return s;
        uint8_t *stage = up_ring_ + (size_t)slot * kUpSlotBytes;
        memcpy(stage, src, bytes);
        s = cuda_status(cudaMemcpyAsync((uint8_t *)dst->ptr + dst_off, stage, bytes, cudaMemcpyHostToDevice, stream_), "upload");
        if (!s.ok()) return s;
        return cuda_status(cudaEventRecord(up_ev_[slot], stream_), "upload event");
    }
    Status s = cuda_status(cudaMemcpyAsync((uint8_t *)dst->ptr + dst_off, src, bytes, cudaMemcpyHostToDevice, stream_), "upload");
    if (!s.ok()) return s;
    return cuda_status(cudaStreamSynchronize(stream_), "upload sync");
}

Status CudaBackend::download(const infr_cuda_buf *src, void *dst, size_t bytes) {
    if (!src || (!dst && bytes)) return Status::Err(INFR_E_INVALID, "download: null argument");
    if (bytes > src->len)
        return Status::Err(INFR_E_INVALID, fmt("download: %zu bytes from a %zu-byte buffer", bytes, src->len));
    if (capturing_) return Status::Err(INFR_E_INVALID, "download during stream capture");
    cudaSetDevice(device_);
    Status s = cuda_status(cudaMemcpyAsync(dst, src->ptr, bytes, cudaMemcpyDeviceToHost, stream_), "download");
    if (!s.ok()) return s;
    s = cuda_status(cudaStreamSynchronize(stream_), "download sync");
    return s.ok() ? check_device_status() : s;
}

Status CudaBackend::copy_buffer(const infr_cuda_buf *src, infr_cuda_buf *dst, size_t bytes) {
    if (!src || !dst) return Status::Err(INFR_E_INVALID, "copy: null buffer");
    if (bytes > src->len || bytes > dst->len)
        return Status::Err(INFR_E_INVALID, fmt("copy: %zu bytes between %zu- and %zu-byte buffers", bytes, src->len, dst->len));
    cudaSetDevice(device_);
    return cuda_status(cudaMemcpyAsync(dst->ptr, src->ptr, bytes, cudaMemcpyDeviceToDevice, stream_), "copy");
}

Status CudaBackend::sync() {
    if (capturing_) return Status::Err(INFR_E_INVALID, "sync during stream capture");
    cudaSetDevice(device_);
    Status s = cuda_status(cudaStreamSynchronize(stream_), "sync");
    return s.ok() ? check_device_status() : s;
}

Status CudaBackend::ensure_scratch(size_t bytes) {
    if (bytes <= scratch_bytes_) return Status::Ok();
    if (capturing_)
        return Status::Err(INFR_E_INVALID, "activation scratch would grow during stream capture; run the same calls once before capturing");
    cudaSetDevice(device_);
    Status s = cuda_status(cudaStreamSynchronize(stream_), "scratch sync");
    if (!s.ok()) return s;
    if (scratch_) cudaFree(scratch_);
    scratch_ = nullptr;
    scratch_bytes_ = 0;
    const size_t want = align_up(bytes, 1 << 20);
    s = cuda_status(cudaMalloc(&scratch_, want), "scratch cudaMalloc");
    if (!s.ok()) return s;
    scratch_bytes_ = want;
    scratch_gen_++;
    return Status::Ok();
}

// ------------------------------------------------------------------------------------------- ops
Status CudaBackend::quantize_q8(int gran, const float *x, uint32_t rows, uint32_t k, int8_t *qs, float *d,
                                int32_t *sums, int32_t *sums16, uint16_t *dact, uint16_t *sact) {
    if (gran != 32 && gran != 256) return Status::Err(INFR_E_INVALID, fmt("quantize_q8: granularity %d (32 or 256)", gran));
    if (k == 0 || k % (uint32_t)gran) return Status::Err(INFR_E_INVALID, fmt("quantize_q8: k=%u is not a multiple of %d", k, gran));
    cudaSetDevice(device_);
    Status s = cuda_status(launch_quantize_q8(x, (int)rows, (int)k, gran, qs, d, sums, sums16, dact, sact, stream_), "quantize_q8");
    if (s.ok() && rows) launches_++;
    return s;
}

// Lays the quantised rows out in the context scratch: qs | d | sums | sums16.
Status CudaBackend::quantize_for(int dtype, const float *x, uint32_t rows, uint32_t k, Q8Dev *out, size_t extra, uint8_t **extra_ptr) {
    const int gran = act_gran(dtype);
    const size_t qs_b = align_up((size_t)rows * k, 256);
    const size_t d_b = align_up((size_t)rows * (k / gran) * 4, 256);
    const size_t s_b = align_up((size_t)rows * (k / 32) * 4, 256);
    const size_t s16_b = dtype == DT_Q6K ? align_up((size_t)rows * (k / 16) * 4, 256) : 0;
    Status s = ensure_scratch(qs_b + d_b + s_b + s16_b + align_up(extra, 256));
    if (!s.ok()) return s;
    uint8_t *p = scratch();
    if (extra_ptr) *extra_ptr = p + qs_b + d_b + s_b + s16_b;
    int8_t *qs = reinterpret_cast<int8_t *>(p);
    float *d = reinterpret_cast<float *>(p + qs_b);
    int32_t *sums = reinterpret_cast<int32_t *>(p + qs_b + d_b);
    int32_t *sums16 = s16_b ? reinterpret_cast<int32_t *>(p + qs_b + d_b + s_b) : nullptr;
    s = quantize_q8(gran, x, rows, k, qs, d, sums, sums16, nullptr, nullptr);
    if (!s.ok()) return s;
    *out = Q8Dev{qs, d, sums, sums16, gran};
    return Status::Ok();
}

Status CudaBackend::linear(int dtype, const uint8_t *w, const float *x, float *y, uint32_t m, uint32_t in_f,
                           uint32_t out_f, int act) {
    if (dtype != DT_Q4K && dtype != DT_Q6K && dtype != DT_Q2_0)
        return Status::Err(INFR_E_UNSUPPORTED, fmt("linear: weight dtype code %d is not supported (Q4_K, Q6_K, Q2_0)", dtype));
    if (act != INFR_ACT_INT8 && act != INFR_ACT_F32) return Status::Err(INFR_E_INVALID, fmt("linear: activation mode %d", act));
    const int be = block_elems(dtype);
    if (in_f == 0 || in_f % (uint32_t)be) return Status::Err(INFR_E_INVALID, fmt("linear: in_f=%u is not a whole number of %d-element blocks", in_f, be));
    if (in_f % 16) return Status::Err(INFR_E_INVALID, fmt("linear: in_f=%u must be a multiple of 16", in_f));
    if (m == 0 || out_f == 0) return Status::Ok();
    cudaSetDevice(device_);
    // More than 8 rows with int8 activations: up to 32 rows (a decode step over that many sequences) take the wide
    // GEMV, which unpacks every weight byte once per 32 rows and is bound by the weight stream; beyond that Q4_K goes
    // to the tensor-memory GEMM (all rows quantised once, the weights unpacked once per 64 rows, K split across CTAs
    // when the row x token tiles alone would leave SMs idle: mmq_ws_k_splits).  mmq_kernel 2 sends every Q4_K batch
    // above 8 rows to the GEMM, 3 walks every batch through the GEMV 8 rows at a time (the parity tests and the bench
    // compare the three).
    if (wide_applies(dtype, m, in_f, act)) {
        Q8Dev a;
        uint8_t *partials = nullptr;
        Status s = quantize_for(dtype, x, m, in_f, &a, gemv_wide_partial_bytes(m < 32 ? (int)m : 32, (int)in_f, (int)out_f), &partials);
        return s.ok() ? wide_gemm(dtype, w, a, y, m, in_f, out_f, reinterpret_cast<float *>(partials)) : s;
    }
    const bool use_mmq = m > 8 && dtype == DT_Q4K && act == INFR_ACT_INT8 && gemv_impl_ == 0 && mmq_impl_ != 3;
    if (use_mmq && mmq_impl_ == 1) {
        Q8Dev a;
        uint8_t *rec = nullptr;
        Status s = quantize_for(dtype, x, m, in_f, &a, mmq_q4k_record_bytes((int)m, (int)in_f), &rec);
        if (!s.ok()) return s;
        s = cuda_status(launch_mmq_q4k(w, a, rec, y, (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_), "mmq_q4k");
        if (s.ok()) launches_ += 2;
        return s;
    }
    if (use_mmq) return mmq_linear(w, x, y, m, in_f, out_f, false);
    // Decode shapes (m <= 8) run the streaming GEMV; wider batches are walked 8 rows at a time, all rows quantised once.
    Q8Dev a_all{};
    // (a single Q4_K chunk quantises its rows inside the GEMV; with several chunks that would repeat the work in every CTA)
    const bool pre_quantised = act == INFR_ACT_INT8 && (!(dtype == DT_Q4K && gemv_impl_ == 0) || m > 8);
    if (pre_quantised) {
        Status s = quantize_for(dtype, x, m, in_f, &a_all);
        if (!s.ok()) return s;
    }
    for (uint32_t r0 = 0; r0 < m; r0 += 8) {
        const uint32_t mm = m - r0 < 8 ? m - r0 : 8;
        const float *xr = x + (size_t)r0 * in_f;
        float *yr = y + (size_t)r0 * out_f;
        if (act == INFR_ACT_F32) {
            Status s = cuda_status(launch_gemv_f32(dtype, w, xr, yr, (int)mm, (int)in_f, (int)out_f, dev_, stream_), "gemv_f32");
            if (!s.ok()) return s;
            launches_ += 1;
        } else if (!pre_quantised) {
            // Q4_K, one kernel: activation rows are quantised inside the GEMV while the first weights stream in.
            // Rows so long that `mm` staged activation rows exceed shared memory are run in narrower batches.
            uint32_t step = mm;
            for (uint32_t t0 = 0; t0 < mm;) {
                const uint32_t n = mm - t0 < step ? mm - t0 : step;
                cudaError_t e = launch_gemv_q4k_mma(w, nullptr, xr + (size_t)t0 * in_f, yr + (size_t)t0 * out_f, (int)n, (int)in_f,
                                                    (int)out_f, dev_, status_dev_, stream_);
                if (e == cudaErrorInvalidValue && step > 1) {
                    cudaGetLastError();
                    step /= 2;
                    continue;
                }
                Status s = cuda_status(e, "gemv_q4k");
                if (!s.ok()) return s;
                launches_ += 1;
                t0 += n;
            }
        } else {
            // this chunk's rows of the quantised batch
            Q8Dev a = a_all;
            Status s;
            const int gran = a.gran, ngr = (int)in_f / gran;
            a.qs = a_all.qs + (size_t)r0 * in_f;
            a.d = a_all.d + (size_t)r0 * ngr;
            a.sums = a_all.sums + (size_t)r0 * (in_f / 32);
            if (a_all.sums16) a.sums16 = a_all.sums16 + (size_t)r0 * (in_f / 16);
            // rows so long that `mm` staged activation rows exceed shared memory are run in narrower batches
            uint32_t step = mm;
            for (uint32_t t0 = 0; t0 < mm;) {
                const uint32_t n = mm - t0 < step ? mm - t0 : step;
                Q8Dev sub = a;
                sub.qs = a.qs + (size_t)t0 * in_f;
                sub.d = a.d + (size_t)t0 * ngr;
                sub.sums = a.sums + (size_t)t0 * (in_f / 32);
                if (a.sums16) sub.sums16 = a.sums16 + (size_t)t0 * (in_f / 16);
                float *yt = yr + (size_t)t0 * out_f;
                cudaError_t e = gemv_impl_ == 1   ? launch_gemv_q8(dtype, w, sub, yt, (int)n, (int)in_f, (int)out_f, nullptr, dev_, stream_)
                                : dtype == DT_Q4K ? launch_gemv_q4k_mma(w, &sub, nullptr, yt, (int)n, (int)in_f, (int)out_f, dev_, status_dev_, stream_)
                                                  : launch_gemv_stream(dtype, w, sub, yt, (int)n, (int)in_f, (int)out_f, dev_, status_dev_, stream_);
                if (e == cudaErrorInvalidValue && step > 1) {
                    cudaGetLastError();
                    step /= 2;
                    continue;
                }
                s = cuda_status(e, "gemv_q8");
                if (!s.ok()) return s;
                launches_ += 1;
                t0 += n;
            }
        }
    }
    return Status::Ok();
}

bool CudaBackend::wide_applies(int dtype, uint32_t m, uint32_t in_f, int act) const {
    if (act != INFR_ACT_INT8 || m <= 8 || gemv_impl_ != 0 || mmq_impl_ != 0 || in_f == 0 || in_f % 256) return false;
    if (dtype == DT_Q4K) return m <= 32;           // one pass of the weights; above, the tensor-memory GEMM is faster
    if (dtype == DT_Q6K) return in_f % 2048 == 0;  // (rows of a whole number of 16-byte units: the TMA stride rule)
    return false;
}

// y[m, out_f] from quantised rows, 32 rows per pass of the weights.
// w2 / y2 / out_f2: a second weight against the same rows in the same launches (partials sized for out_f + out_f2).
Status CudaBackend::wide_gemm(int dtype, const uint8_t *w, const Q8Dev &a, float *y, uint32_t m, uint32_t in_f, uint32_t out_f, float *partials,
                              const uint8_t *w2, float *y2, uint32_t out_f2) {
    const uint32_t nb = in_f / 256;
    for (uint32_t r0 = 0; r0 < m; r0 += 32) {
        const uint32_t mm = m - r0 < 32 ? m - r0 : 32;
        Q8Dev sub = a;
        sub.qs = a.qs + (size_t)r0 * in_f;
        sub.d = a.d + (size_t)r0 * nb;
        sub.sums = a.sums + (size_t)r0 * nb * 8;
        if (a.sums16) sub.sums16 = a.sums16 + (size_t)r0 * nb * 16;
        Status s = cuda_status(launch_gemv_wide(dtype, w, sub, y + (size_t)r0 * out_f, partials, (int)mm, (int)in_f, (int)out_f, dev_, status_dev_, stream_,
                                                nullptr, w2, y2 ? y2 + (size_t)r0 * out_f2 : nullptr, (int)out_f2),
                               "gemv_wide");
        if (!s.ok()) return s;
        launches_ += (uint64_t)gemv_wide_launches((int)in_f);
    }
    return Status::Ok();
}

// The tensor-memory GEMM from f32 rows.  The context scratch holds the activation planes (and the K-split partial
// results behind them); reuse = the planes are those of the previous call's rows (same x, m, in_f) and are not rebuilt.
Status CudaBackend::mmq_linear(const uint8_t *w, const float *x, float *y, uint32_t m, uint32_t in_f, uint32_t out_f, bool reuse) {
    const size_t rec_bytes = align_up(mmq_ws_record_bytes((int)m, (int)in_f), 256);
    // the partial results sit behind the planes at an offset that does not depend on out_f, so that two weights of
    // different height can share the planes
    const size_t part_bytes = mmq_ws_partial_bytes((int)m, (int)in_f, (int)out_f, dev_);
    Status s = ensure_scratch(rec_bytes + part_bytes);
    if (!s.ok()) return s;
    float *partials = part_bytes ? reinterpret_cast<float *>(scratch() + rec_bytes) : nullptr;
    s = cuda_status(launch_mmq_ws_q4k_f32(w, reuse ? nullptr : x, scratch(), y, (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_, partials),
                    "mmq_q4k");
    if (s.ok()) launches_ += (reuse ? 1 : 2) + (part_bytes ? 1 : 0);
    return s;
}

// Two weights of one format against the same f32 rows (q and k, gate and up): the rows are quantised once.
Status CudaBackend::linear_pair(int dtype, const uint8_t *w1, float *y1, uint32_t out_f1, const uint8_t *w2, float *y2, uint32_t out_f2,
                                const float *x, uint32_t m, uint32_t in_f, int act) {
    if (wide_applies(dtype, m, in_f, act) && out_f1 && out_f2) {
        cudaSetDevice(device_);
        const int mm = m < 32 ? (int)m : 32;
        Q8Dev a;
        uint8_t *partials = nullptr;
        Status s = quantize_for(dtype, x, m, in_f, &a, gemv_wide_partial_bytes(mm, (int)in_f, (int)(out_f1 + out_f2)), &partials);
        return s.ok() ? wide_gemm(dtype, w1, a, y1, m, in_f, out_f1, reinterpret_cast<float *>(partials), w2, y2, out_f2) : s;
    }
    const bool q4_gemm = m > 8 && dtype == DT_Q4K && act == INFR_ACT_INT8 && gemv_impl_ == 0 && (mmq_impl_ == 0 || mmq_impl_ == 2);
    if (q4_gemm && in_f && in_f % 256 == 0 && out_f1 && out_f2) {
        cudaSetDevice(device_);
        // scratch for the larger of the two before the first launch: growing it would drop the planes
        const size_t rec_bytes = align_up(mmq_ws_record_bytes((int)m, (int)in_f), 256);
        const size_t p1 = mmq_ws_partial_bytes((int)m, (int)in_f, (int)out_f1, dev_), p2 = mmq_ws_partial_bytes((int)m, (int)in_f, (int)out_f2, dev_);
        Status s = ensure_scratch(rec_bytes + (p1 > p2 ? p1 : p2));
        if (!s.ok()) return s;
        s = mmq_linear(w1, x, y1, m, in_f, out_f1, false);
        return s.ok() ? mmq_linear(w2, x, y2, m, in_f, out_f2, true) : s;
    }
    if (act == INFR_ACT_INT8 && m >= 1 && m <= 8 && (dtype == DT_Q4K || dtype == DT_Q6K || dtype == DT_Q2_0) && in_f &&
        in_f % (uint32_t)block_elems(dtype) == 0 && in_f % 16 == 0 && out_f1 && out_f2) {
        cudaSetDevice(device_);
        if (dtype == DT_Q4K && gemv_impl_ == 0 && in_f % 256 == 0) {
            // one kernel: the rows are quantised inside the GEMV while the first weights stream in
            const cudaError_t e = launch_gemv_q4k_mma_pair(w1, y1, (int)out_f1, w2, y2, (int)out_f2, nullptr, x, (int)m, (int)in_f, dev_,
                                                           status_dev_, stream_);
            if (e == cudaSuccess) {
                launches_++;
                return Status::Ok();
            }
            if (e != cudaErrorInvalidValue) return cuda_status(e, "linear_pair");
            cudaGetLastError();  // rows too long to stage m of them in one CTA: quantise first, then the pair
        }
        Q8Dev a;
        Status s = quantize_for(dtype, x, m, in_f, &a);
        return s.ok() ? gemv_q8_pair(dtype, w1, y1, out_f1, w2, y2, out_f2, a, m, in_f) : s;
    }
    Status s = linear(dtype, w1, x, y1, m, in_f, out_f1, act);
    return s.ok() ? linear(dtype, w2, x, y2, m, in_f, out_f2, act) : s;
}

Status CudaBackend::gemv_q8(int dtype, const uint8_t *w, const Q8Dev &a, float *y, uint32_t m, uint32_t in_f, uint32_t out_f) {
    if (dtype != DT_Q4K && dtype != DT_Q6K && dtype != DT_Q2_0)
        return Status::Err(INFR_E_UNSUPPORTED, fmt("gemv_q8: weight dtype code %d", dtype));
    const bool wide = m > 8 && wide_applies(dtype, m, in_f, INFR_ACT_INT8);
    if (m == 0 || (m > 8 && !wide))
        return Status::Err(INFR_E_INVALID, fmt("gemv_q8: m=%u (1..8; more rows where the wide GEMV applies: Q4_K up to 32, Q6_K with in_f a multiple of 2048)", m));
    if (in_f == 0 || in_f % (uint32_t)block_elems(dtype) || in_f % 16) return Status::Err(INFR_E_INVALID, fmt("gemv_q8: in_f=%u", in_f));
    if (a.gran != act_gran(dtype)) return Status::Err(INFR_E_INVALID, fmt("gemv_q8: activations have granularity %d, dtype needs %d", a.gran, act_gran(dtype)));
    if (dtype == DT_Q6K && !a.sums16) return Status::Err(INFR_E_INVALID, "gemv_q8: Q6_K needs the per-16 sums");
    cudaSetDevice(device_);
    if (wide) {
        // a decode batch of a few dozen rows: the context scratch holds the partial results of the K chunks
        const size_t pb = gemv_wide_partial_bytes(m < 32 ? (int)m : 32, (int)in_f, (int)out_f);
        Status s = ensure_scratch(pb);
        return s.ok() ? wide_gemm(dtype, w, a, y, m, in_f, out_f, reinterpret_cast<float *>(scratch())) : s;
    }
    Status s = cuda_status(gemv_impl_ == 1   ? launch_gemv_q8(dtype, w, a, y, (int)m, (int)in_f, (int)out_f, nullptr, dev_, stream_)
                           : (dtype == DT_Q4K && gemv_impl_ == 0)
                               ? launch_gemv_q4k_mma(w, &a, nullptr, y, (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_)
                               : launch_gemv_stream(dtype, w, a, y, (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_),
                           "gemv_q8");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::gemv_q8_pair(int dtype, const uint8_t *w1, float *y1, uint32_t out_f1, const uint8_t *w2, float *y2, uint32_t out_f2,
                                 const Q8Dev &a, uint32_t m, uint32_t in_f) {
    if (dtype == DT_Q4K && gemv_impl_ == 0 && m >= 1 && m <= 8 && in_f && in_f % 256 == 0 && out_f1 && out_f2 && a.gran == 256) {
        cudaSetDevice(device_);
        Status s = cuda_status(launch_gemv_q4k_mma_pair(w1, y1, (int)out_f1, w2, y2, (int)out_f2, &a, nullptr, (int)m, (int)in_f, dev_, status_dev_, stream_),
                               "gemv_q8_pair");
        if (s.ok()) launches_++;
        return s;
    }
    if (m > 8 && m <= 32 && out_f1 && out_f2 && wide_applies(dtype, m, in_f, INFR_ACT_INT8) && a.gran == 256 && (dtype != DT_Q6K || a.sums16)) {
        // a few dozen rows: both weights in one launch of the wide GEMV (and one launch that adds the K chunks of both)
        cudaSetDevice(device_);
        Status s = ensure_scratch(gemv_wide_partial_bytes((int)m, (int)in_f, (int)(out_f1 + out_f2)));
        return s.ok() ? wide_gemm(dtype, w1, a, y1, m, in_f, out_f1, reinterpret_cast<float *>(scratch()), w2, y2, out_f2) : s;
    }
    Status s = gemv_q8(dtype, w1, a, y1, m, in_f, out_f1);
    return s.ok() ? gemv_q8(dtype, w2, a, y2, m, in_f, out_f2) : s;
}

// ---- the other ops of a dense decode step ----
Status CudaBackend::rms_norm(const float *a, const float *b, float *sum_dst, const float *w, float *dst, uint32_t rows, uint32_t dim, float eps) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_rms_norm(a, b, sum_dst, w, dst, (int)rows, (int)dim, eps, stream_), "rms_norm");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::rope(const float *x, const int32_t *positions, float *dst, uint32_t rows, uint32_t n_head, uint32_t head_dim,
                         uint32_t rope_dim, float theta, int neox) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_rope(x, positions, dst, (int)rows, (int)n_head, (int)head_dim, (int)rope_dim, theta, neox, dev_, stream_), "rope");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::write_kv(const float *src, void *cache_at_pos, size_t n) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_write_kv_f16(src, cache_at_pos, n, dev_, stream_), "write_kv");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::rope_write_kv(const infr_attn_desc &d, float theta, int neox, float *q, const float *k, const float *v,
                                  const int32_t *positions, void *k_cache, void *v_cache, int write_pos, const int32_t *block_table,
                                  uint32_t table_stride, uint32_t n_pages) {
    cudaSetDevice(device_);
    const uint32_t n_seq = d.n_seq ? d.n_seq : 1;
    Status s = cuda_status(launch_rope_write_kv(q, k, v, positions, k_cache, v_cache, (int)(n_seq * d.rows), (int)d.n_head, (int)d.n_kv,
                                                (int)d.head_dim, theta, neox, (int)d.rows, block_table ? 0 : (size_t)d.seq_stride, dev_, stream_, write_pos, block_table,
                                                (int)table_stride, (int)n_pages),
                           "rope_write_kv");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::rms_norm_q8(const float *a, const float *b, float *sum_dst, const float *w, uint32_t rows, uint32_t dim, float eps, const Q8Dev &q8) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_rms_norm_q8(a, b, sum_dst, w, (int)rows, (int)dim, eps, const_cast<int8_t *>(q8.qs), const_cast<float *>(q8.d),
                                              const_cast<int32_t *>(q8.sums), const_cast<int32_t *>(q8.sums16), stream_),
                           "rms_norm_q8");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::gated_act_q8(const float *gate, const float *up, uint32_t rows, uint32_t nff, const Q8Dev &q8) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_gated_silu_q8(gate, up, (int)rows, (int)nff, const_cast<int8_t *>(q8.qs), const_cast<float *>(q8.d),
                                                const_cast<int32_t *>(q8.sums), const_cast<int32_t *>(q8.sums16), stream_),
                           "gated_act_q8");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::attention(const infr_attn_desc &d, const float *q, const void *k_cache, const void *v_cache, float *dst, const Q8Dev *q8,
                              const int32_t *seq_pos, const int32_t *block_table, uint32_t table_stride, uint32_t n_pages) {
    cudaSetDevice(device_);
    const uint32_t n_seq = d.n_seq ? d.n_seq : 1;
    const size_t ws = attention_workspace_bytes((int)(n_seq * d.rows), (int)d.n_head, (int)d.head_dim, (int)(d.pos + d.rows));
    Status s = ensure_scratch(ws);
    if (!s.ok()) return s;
    s = cuda_status(launch_attention(q, k_cache, v_cache, dst, scratch_, (int)n_seq, (int)d.rows, (int)d.n_head, (int)d.n_kv, (int)d.head_dim,
                                     d.scale, (int)d.pos, block_table ? 0 : (size_t)d.seq_stride, dev_.sm_count, stream_, status_dev_, q8 ? const_cast<int8_t *>(q8->qs) : nullptr,
                                     q8 ? const_cast<float *>(q8->d) : nullptr, q8 ? const_cast<int32_t *>(q8->sums) : nullptr,
                                     q8 ? const_cast<int32_t *>(q8->sums16) : nullptr, seq_pos, block_table, (int)table_stride, (int)n_pages),
                    "attention");
    if (s.ok()) launches_ += 2;
    return s;
}

Status CudaBackend::gated_act(const float *gate, const float *up, float *dst, size_t n) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_gated_silu(gate, up, dst, n, dev_, stream_), "gated_act");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::add(const float *a, const float *b, float *dst, size_t n) {
    cudaSetDevice(device_);
    Status s = cuda_status(launch_add(a, b, dst, n, dev_, stream_), "add");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::argmax(const float *x, uint32_t *dst, uint32_t n, uint32_t rows) {
    cudaSetDevice(device_);
    Status s = ensure_scratch(argmax_workspace_bytes(n, rows));
    if (!s.ok()) return s;
    s = cuda_status(launch_argmax(x, dst, scratch_, n, rows, stream_), "argmax");
    if (s.ok()) launches_ += 2;
    return s;
}

// rows == 1 or `reference`: every expert bank works on raw f32 activations (int8_ok false,
// crates/infr-cpu/src/lib.rs:2359): dequantised weight rows, f32 dot, pairs kept in (row, rank) order.
Status CudaBackend::moe_ffn_f32(const MoeArgs &a) {
    cudaSetDevice(device_);
    const size_t rows = a.rows, ne = a.ne, nff = a.n_ff, nu = a.n_used, nx = a.n_expert;
    const size_t n_pairs = rows * nu;
    if (n_pairs > 65535) return Status::Err(INFR_E_UNSUPPORTED, "moe_ffn (f32 path): more than 65535 routed pairs");
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes, 256);
        return o;
    };
    const size_t o_logits = take(rows * nx * 4), o_ids = take(n_pairs * 4), o_w = take(n_pairs * 4);
    const size_t o_g = take(n_pairs * nff * 4), o_u = take(n_pairs * nff * 4), o_act = take(n_pairs * nff * 4);
    const size_t o_q = take(n_pairs * nff), o_d = take(n_pairs * (nff / 256) * 4), o_s = take(n_pairs * (nff / 32) * 4);
    const size_t o_y = take(n_pairs * ne * 4);
    Status s = ensure_scratch(off);
    if (!s.ok()) return s;
    uint8_t *b = scratch();
    float *logits = a.logits ? a.logits : reinterpret_cast<float *>(b + o_logits);
    int32_t *ids = a.sel_ids ? a.sel_ids : reinterpret_cast<int32_t *>(b + o_ids);
    float *w = a.sel_w ? a.sel_w : reinterpret_cast<float *>(b + o_w);
    float *g = reinterpret_cast<float *>(b + o_g), *u = reinterpret_cast<float *>(b + o_u), *act = reinterpret_cast<float *>(b + o_act);
    float *y = reinterpret_cast<float *>(b + o_y);
    const size_t gu_stride = nff * (ne / 256) * 144, d_stride = ne * (nff / 256) * 144;
#define INFR_STEP(call, what)          \
    do {                               \
        s = cuda_status((call), what); \
        if (!s.ok()) return s;         \
        launches_++;                   \
    } while (0)
    INFR_STEP(launch_moe_router(a.router, a.router_x, logits, (int)rows, (int)ne, (int)nx, stream_), "moe router");
    INFR_STEP(launch_moe_route(logits, (int)rows, (int)nx, (int)nu, a.scale, a.norm_w, ids, w, stream_), "moe route");
    INFR_STEP(launch_gemv_q4k_f32_sel(a.gate, ids, gu_stride, a.x, (int)nu, g, (int)n_pairs, (int)ne, (int)nff, dev_, stream_), "moe gate f32");
    INFR_STEP(launch_gemv_q4k_f32_sel(a.up, ids, gu_stride, a.x, (int)nu, u, (int)n_pairs, (int)ne, (int)nff, dev_, stream_), "moe up f32");
    INFR_STEP(launch_moe_swiglu_quant(g, u, (int)n_pairs, (int)nff, reinterpret_cast<int8_t *>(b + o_q), reinterpret_cast<float *>(b + o_d),
                                      reinterpret_cast<int32_t *>(b + o_s), nullptr, act, stream_), "moe swiglu");
    INFR_STEP(launch_gemv_q4k_f32_sel(a.down, ids, d_stride, act, 0, y, (int)n_pairs, (int)nff, (int)ne, dev_, stream_), "moe down f32");
    INFR_STEP(launch_moe_combine(y, nullptr, w, (int)rows, (int)nu, (int)ne, a.dst, stream_), "moe combine");
#undef INFR_STEP
    return Status::Ok();
}

Status CudaBackend::moe_ffn(const MoeArgs &a) {
    auto bank_ok = [](int dt) { return dt == DT_Q4K || dt == DT_Q6K; };
    if (!bank_ok(a.gate_dt) || !bank_ok(a.up_dt) || !bank_ok(a.down_dt))
        return Status::Err(INFR_E_UNSUPPORTED, "moe_ffn: expert banks must be Q4_K or Q6_K");
    const bool any_q6 = a.gate_dt == DT_Q6K || a.up_dt == DT_Q6K || a.down_dt == DT_Q6K;
    if (a.ne == 0 || a.ne % 256 || a.n_ff == 0 || a.n_ff % 256)
        return Status::Err(INFR_E_UNSUPPORTED, fmt("moe_ffn: ne=%u and n_ff_exp=%u must be multiples of 256", a.ne, a.n_ff));
    if (a.n_expert == 0 || a.n_expert > 1024 || a.n_used == 0 || a.n_used > 32 || a.n_used > a.n_expert)
        return Status::Err(INFR_E_INVALID, fmt("moe_ffn: n_expert=%u (<=1024), n_used=%u (<=32)", a.n_expert, a.n_used));
    if (a.rows == 0) return Status::Ok();
    if (((size_t)a.rows * a.n_used + 31) / 32 * a.n_expert * 4 > (size_t)200 * 1024)
        return Status::Err(INFR_E_UNSUPPORTED, fmt("moe_ffn: %u rows x %u experts per row exceed what one call sorts (split the rows)", a.rows, a.n_used));
    if (a.rows < 2 || reference_) {
        if (a.n_local != a.n_expert) return Status::Err(INFR_E_UNSUPPORTED, "moe_ffn: a local expert range needs the int8 path (rows >= 2, no reference mode)");
        if (any_q6) return Status::Err(INFR_E_UNSUPPORTED, "moe_ffn: Q6_K expert banks run on the int8 path only (rows >= 2, no reference mode)");
        return moe_ffn_f32(a);
    }
    cudaSetDevice(device_);
    const size_t rows = a.rows, ne = a.ne, nff = a.n_ff, nu = a.n_used, nx = a.n_expert;
    const size_t n_pairs = rows * nu;
    const size_t max_items = n_pairs / 8 + nx + 1;
    // Experts that see a few dozen rows each run on the tensor-memory GEMM in grouped form (one 64-row slab of an
    // expert's rows per tile column: the expert's weights are unpacked once per slab); with only a handful of rows
    // per expert the 8-row grouped GEMV does less padded work.
    // (a Q6_K bank has no tensor-memory GEMM: such a layer takes 8-row items throughout)
    const bool grouped_gemm = !any_q6 && (mmq_impl_ == 2 || (mmq_impl_ == 0 && n_pairs >= (size_t)8 * a.n_local));
    const size_t max_slabs = n_pairs / 64 + a.n_local + 1;
    // scratch carve-up (all 256-byte aligned)
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes, 256);
        return o;
    };
    const size_t o_logits = take(rows * nx * 4), o_ids = take(n_pairs * 4), o_w = take(n_pairs * 4);
    const size_t o_prow = take(n_pairs * 4), o_pslot = take(n_pairs * 4);
    const size_t o_ie = take(max_items * 4), o_ip = take(max_items * 4), o_ic = take(max_items * 4), o_ni = take(4);
    const size_t o_xq = take(rows * ne), o_xd = take(rows * (ne / 256) * 4), o_xs = take(rows * (ne / 32) * 4);
    const size_t o_xs16 = any_q6 ? take(rows * (ne / 16) * 4) : 0, o_as16 = any_q6 ? take(n_pairs * (nff / 16) * 4) : 0;
    const size_t o_g = take(n_pairs * nff * 4), o_u = take(n_pairs * nff * 4);
    const size_t o_aq = take(n_pairs * nff), o_ad = take(n_pairs * (nff / 256) * 4), o_as = take(n_pairs * (nff / 32) * 4);
    const size_t o_y = take(n_pairs * ne * 4);
    const size_t o_px = grouped_gemm ? take(mmq_ws_record_bytes((int)max_slabs * 64, (int)ne)) : 0;
    const size_t o_pa = grouped_gemm ? take(mmq_ws_record_bytes((int)max_slabs * 64, (int)nff)) : 0;
    Status s = ensure_scratch(off);
    if (!s.ok()) return s;
    uint8_t *b = scratch();
    float *logits = a.logits ? a.logits : reinterpret_cast<float *>(b + o_logits);
    int32_t *ids = a.sel_ids ? a.sel_ids : reinterpret_cast<int32_t *>(b + o_ids);
    float *w = a.sel_w ? a.sel_w : reinterpret_cast<float *>(b + o_w);
    int32_t *prow = reinterpret_cast<int32_t *>(b + o_prow), *pslot = reinterpret_cast<int32_t *>(b + o_pslot);
    int32_t *ie = reinterpret_cast<int32_t *>(b + o_ie), *ip = reinterpret_cast<int32_t *>(b + o_ip);
    int32_t *ic = reinterpret_cast<int32_t *>(b + o_ic), *ni = reinterpret_cast<int32_t *>(b + o_ni);
    int8_t *xq = reinterpret_cast<int8_t *>(b + o_xq);
    float *xd = reinterpret_cast<float *>(b + o_xd);
    int32_t *xs = reinterpret_cast<int32_t *>(b + o_xs);
    float *g = reinterpret_cast<float *>(b + o_g), *u = reinterpret_cast<float *>(b + o_u);
    int8_t *aq = reinterpret_cast<int8_t *>(b + o_aq);
    float *ad = reinterpret_cast<float *>(b + o_ad);
    int32_t *as = reinterpret_cast<int32_t *>(b + o_as);
    float *y = reinterpret_cast<float *>(b + o_y);
#define INFR_STEP(call, what)                       \
    do {                                            \
        s = cuda_status((call), what);              \
        if (!s.ok()) return s;                      \
        launches_++;                                \
    } while (0)
    INFR_STEP(launch_moe_router(a.router, a.router_x, logits, (int)rows, (int)ne, (int)nx, stream_), "moe router");
    INFR_STEP(launch_moe_route(logits, (int)rows, (int)nx, (int)nu, a.scale, a.norm_w, ids, w, stream_), "moe route");
    INFR_STEP(launch_moe_bucket(ids, (int)rows, (int)nu, (int)nx, (int)a.expert_lo, (int)a.n_local, grouped_gemm ? 64 : 8, prow, pslot, ie, ip, ic, ni,
                                nullptr, stream_),
              "moe bucket");
    // stage A: every distinct row quantised once (lib.rs:2688-2718)
    int32_t *xs16 = any_q6 ? reinterpret_cast<int32_t *>(b + o_xs16) : nullptr, *as16 = any_q6 ? reinterpret_cast<int32_t *>(b + o_as16) : nullptr;
    INFR_STEP(launch_quantize_q8(a.x, (int)rows, (int)ne, 256, xq, xd, xs, xs16, nullptr, nullptr, stream_), "moe quantize x");
    Q8Dev xa{xq, xd, xs, xs16, 256};
    // one expert bank against the routed rows, 8-row items: Q4_K on the warp matrix unit, Q6_K on the byte-dot kernel
    auto bank_gemm = [&](int dt, const uint8_t *bank, const Q8Dev &acts, float *out, uint32_t k, uint32_t o, const int32_t *rows_of) {
        return dt == DT_Q4K ? launch_grouped_q4k_mma(bank, (int)a.n_local, acts, out, (int)k, (int)o, ie, ip, ic, ni, rows_of, (int)max_items, dev_,
                                                     status_dev_, stream_)
                            : launch_grouped_q6k(bank, acts, out, (int)k, (int)o, ie, ip, ic, ni, rows_of, (int)max_items, dev_, stream_);
    };
    if (grouped_gemm) {
        // stage B: both banks read the same gathered activation planes (laid out once); stage C; stage D on the
        // re-quantised pairs; stage E
        INFR_STEP(launch_mmq_ws_q4k_grouped(a.gate, (int)a.n_local, xa, b + o_px, g, (int)ne, (int)nff, ie, ip, ic, ni, prow, (int)max_slabs, true, dev_,
                                            status_dev_, stream_),
                  "moe gate (grouped gemm)");
        launches_++;  // the plane layout kernel
        INFR_STEP(launch_mmq_ws_q4k_grouped(a.up, (int)a.n_local, xa, b + o_px, u, (int)ne, (int)nff, ie, ip, ic, ni, prow, (int)max_slabs, false, dev_,
                                            status_dev_, stream_),
                  "moe up (grouped gemm)");
        INFR_STEP(launch_moe_swiglu_quant(g, u, (int)n_pairs, (int)nff, aq, ad, as, nullptr, nullptr, stream_), "moe swiglu");
        Q8Dev aa{aq, ad, as, nullptr, 256};
        INFR_STEP(launch_mmq_ws_q4k_grouped(a.down, (int)a.n_local, aa, b + o_pa, y, (int)nff, (int)ne, ie, ip, ic, ni, nullptr, (int)max_slabs, true, dev_,
                                            status_dev_, stream_),
                  "moe down (grouped gemm)");
        launches_++;
        INFR_STEP(launch_moe_combine(y, pslot, w, (int)rows, (int)nu, (int)ne, a.dst, stream_), "moe combine");
        return Status::Ok();
    }
    // stage B: gate and up expert GEMMs, rows gathered per pair
    INFR_STEP(bank_gemm(a.gate_dt, a.gate, xa, g, (uint32_t)ne, (uint32_t)nff, prow), "moe gate");
    INFR_STEP(bank_gemm(a.up_dt, a.up, xa, u, (uint32_t)ne, (uint32_t)nff, prow), "moe up");
    // stage C: SwiGLU and re-quantisation per pair
    INFR_STEP(launch_moe_swiglu_quant(g, u, (int)n_pairs, (int)nff, aq, ad, as, as16, nullptr, stream_), "moe swiglu");
    Q8Dev aa{aq, ad, as, as16, 256};
    // stage D: down GEMMs; stage E: rank-order combine
    INFR_STEP(bank_gemm(a.down_dt, a.down, aa, y, (uint32_t)nff, (uint32_t)ne, nullptr), "moe down");
    INFR_STEP(launch_moe_combine(y, pslot, w, (int)rows, (int)nu, (int)ne, a.dst, stream_), "moe combine");
#undef INFR_STEP
    return Status::Ok();
}

Status CudaBackend::gemv_block_acc(int dtype, const uint8_t *w, const float *x, int32_t *acc, uint32_t in_f, uint32_t out_f) {
    if (dtype != DT_Q4K && dtype != DT_Q6K && dtype != DT_Q2_0)
        return Status::Err(INFR_E_UNSUPPORTED, fmt("gemv_block_acc: dtype code %d", dtype));
    const int be = block_elems(dtype);
    if (in_f == 0 || in_f % (uint32_t)be || in_f % 16) return Status::Err(INFR_E_INVALID, fmt("gemv_block_acc: in_f=%u", in_f));
    cudaSetDevice(device_);
    Q8Dev a;
    Status s = quantize_for(dtype, x, 1, in_f, &a);
    if (!s.ok()) return s;
    s = cuda_status(launch_gemv_q8(dtype, w, a, nullptr, 1, (int)in_f, (int)out_f, acc, dev_, stream_), "gemv_block_acc");
    if (s.ok()) launches_++;
    return s;
}

// ------------------------------------------------------------------------------ capture and timing
Status CudaBackend::capture_begin() {
    if (capturing_) return Status::Err(INFR_E_INVALID, "capture_begin: already capturing");
    cudaSetDevice(device_);
    Status s = cuda_status(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    if (s.ok()) capturing_ = true;
    return s;
}

Status CudaBackend::capture_end(infr_cuda_graph **out) {
    if (!capturing_) return Status::Err(INFR_E_INVALID, "capture_end: not capturing");
    capturing_ = false;
    cudaSetDevice(device_);
    auto *g = new infr_cuda_graph();
    Status s = cuda_status(cudaStreamEndCapture(stream_, &g->graph), "cudaStreamEndCapture");
    if (s.ok()) s = cuda_status(cudaGraphInstantiate(&g->exec, g->graph, 0), "cudaGraphInstantiate");
    if (s.ok()) {
        size_t nn = 0;
        cudaGraphGetNodes(g->graph, nullptr, &nn);
        std::vector<cudaGraphNode_t> nodes(nn);
        if (nn) cudaGraphGetNodes(g->graph, nodes.data(), &nn);
        for (auto nd : nodes) {
            cudaGraphNodeType ty;
            if (cudaGraphNodeGetType(nd, &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) g->kernel_nodes++;
        }
    }
    if (!s.ok()) {
        graph_free(g);
        return s;
    }
    *out = g;
    return Status::Ok();
}

Status CudaBackend::graph_launch(infr_cuda_graph *g) {
    if (!g || !g->exec) return Status::Err(INFR_E_INVALID, "graph_launch: null graph");
    cudaSetDevice(device_);
    Status s = cuda_status(cudaGraphLaunch(g->exec, stream_), "cudaGraphLaunch");
    if (s.ok()) launches_ += g->kernel_nodes;
    return s;
}

void CudaBackend::graph_free(infr_cuda_graph *g) {
    if (!g) return;
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream_);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
}

Status CudaBackend::timer_start() {
    cudaSetDevice(device_);
    return cuda_status(cudaEventRecord(ev0_, stream_), "cudaEventRecord");
}

Status CudaBackend::timer_stop(float *ms) {
    if (!ms) return Status::Err(INFR_E_INVALID, "timer_stop: null output");
    cudaSetDevice(device_);
    Status s = cuda_status(cudaEventRecord(ev1_, stream_), "cudaEventRecord");
    if (s.ok()) s = cuda_status(cudaEventSynchronize(ev1_), "cudaEventSynchronize");
    if (s.ok()) s = cuda_status(cudaEventElapsedTime(ms, ev0_, ev1_), "cudaEventElapsedTime");
    return s.ok() ? check_device_status() : s;
}

Status CudaBackend::flush_l2() {
    cudaSetDevice(device_);
    if (!flush_) {
        if (capturing_) return Status::Err(INFR_E_INVALID, "flush_l2: first use during stream capture");
        flush_bytes_ = align_up(dev_.l2_bytes * 2 + (64u << 20), 1 << 20);
        Status s = cuda_status(cudaMalloc(&flush_, flush_bytes_), "flush cudaMalloc");
        if (!s.ok()) return s;
    }
    Status s = cuda_status(launch_fill_u32(static_cast<uint32_t *>(flush_), flush_bytes_ / 4, (uint32_t)launches_, stream_), "flush_l2");
    if (s.ok()) launches_++;
    return s;
}

Status CudaBackend::tensor_peak_i8(uint32_t n_batches, uint32_t launches, float *ms, double *ops) {
    if (!ms || !ops || launches == 0 || launches > 100000 || n_batches == 0 || n_batches > 4096)
        return Status::Err(INFR_E_INVALID, "tensor_peak_i8: 1..4096 batches, 1..100000 launches, non-null outputs");
    if (capturing_) return Status::Err(INFR_E_INVALID, "tensor_peak_i8 during stream capture");
    cudaSetDevice(device_);
    Status s = ensure_scratch(256);
    if (!s.ok()) return s;
    int32_t *check = reinterpret_cast<int32_t *>(scratch());
    if (!(s = cuda_status(cudaMemsetAsync(check, 0xff, 8, stream_), "tensor_peak memset")).ok()) return s;
    // one untimed launch: module load, first tensor-memory allocation
    if (!(s = cuda_status(launch_tensor_peak_i8(n_batches, check, dev_, status_dev_, stream_), "tensor_peak_i8")).ok()) return s;
    if (!(s = cuda_status(cudaEventRecord(ev0_, stream_), "cudaEventRecord")).ok()) return s;
    for (uint32_t i = 0; i < launches; i++)
        if (!(s = cuda_status(launch_tensor_peak_i8(n_batches, check, dev_, status_dev_, stream_), "tensor_peak_i8")).ok()) return s;
    launches_ += launches + 1;
    if (!(s = cuda_status(cudaEventRecord(ev1_, stream_), "cudaEventRecord")).ok()) return s;
    if (!(s = cuda_status(cudaEventSynchronize(ev1_), "cudaEventSynchronize")).ok()) return s;
    if (!(s = cuda_status(cudaEventElapsedTime(ms, ev0_, ev1_), "cudaEventElapsedTime")).ok()) return s;
    if (!(s = check_device_status()).ok()) return s;
    int32_t got[2] = {0, 0};
    if (!(s = cuda_status(cudaMemcpyAsync(got, check, 8, cudaMemcpyDeviceToHost, stream_), "tensor_peak readback")).ok()) return s;
    if (!(s = cuda_status(cudaStreamSynchronize(stream_), "tensor_peak sync")).ok()) return s;
    const int32_t want = tensor_peak_i8_expected(n_batches);
    if (got[0] != want || got[1] != want)
        return Status::Err(INFR_E_CUDA, fmt("tensor_peak_i8: accumulator check failed (got %d and %d, the operand pattern implies %d)", got[0], got[1], want));
    *ops = tensor_peak_i8_ops(n_batches, dev_) * launches;
    return Status::Ok();
}

}  // namespace infr
