// Small-message all-reduce over NVLink peer memory for the row-parallel Linears of a tensor-parallel decode
// step (the reference has no multi-GPU path; this is the exchange its Linear outputs need when a model's
// rows / columns are split over the GPUs of one box).
//
// One-shot push: every rank stores its n floats into slot [rank] of EVERY peer's staging buffer (plain
// remote stores through a CUDA IPC mapping: no TMA, no multicast), publishes a per-CTA flag on each peer
// after a system fence, waits — bounded — until the flags of all ranks have reached the current epoch in its
// OWN staging buffer, and then sums the slots in rank order, so every rank gets the same bits.  Staging and
// flags alternate between two parities by epoch: a peer can write parity p again only after the next
// exchange has finished, which needs this rank's flag, which is sent after this rank has read parity p.
// 16 KB (4096 floats) takes one CTA; a 64-float4-per-thread limit keeps the whole exchange a single wave.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "backend.h"

namespace infr {
namespace {

std::string fmt(const char *f, ...) {
    char buf[256];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof buf, f, ap);
    va_end(ap);
    return buf;
}

constexpr int kMaxWorld = 8;
constexpr int kArThreads = 1024;
constexpr int kArMaxCtas = 64;  // 64 x 1024 float4 = 256 K floats (1 MB) per exchange; one CTA per SM, all resident
constexpr uint32_t kArSpin = 1u << 22;
constexpr uint32_t kPushMaxFloats = 32 * 8192;  // a pushed GEMV result: at most 32 rows (2 MB of staged words per rank and parity)

struct ArPeers {
    float *stage[kMaxWorld];     // peer r's staging: [2][world][cap] f32
    uint32_t *flags[kMaxWorld];  // peer r's flags: [2][kArMaxCtas][world]
};

// ctrl[0] = epoch, ctrl[1] = CTAs done in the current launch (both in this rank's memory)
__global__ void __launch_bounds__(kArThreads, 1)
    allreduce_oneshot_kernel(float *__restrict__ data, uint32_t n4, int rank, int world, uint32_t cap, ArPeers peers,
                             uint32_t *__restrict__ ctrl, uint32_t *__restrict__ status, uint32_t spin) {
    __shared__ int s_bad;
    const uint32_t i = blockIdx.x * kArThreads + threadIdx.x;  // float4 index
    if (threadIdx.x == 0) s_bad = 0;
    // programmatic dependent launch: the next kernel may start its prologue now; this one waits for the previous
    // kernel (the producer of `data`, or this comm's previous exchange) before it reads `data` and the epoch word
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(ctrl);
    const uint32_t p = epoch & 1u, want = epoch + 1u;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < n4) {
        v = reinterpret_cast<const float4 *>(data)[i];
        for (int r = 0; r < world; r++)
            reinterpret_cast<float4 *>(peers.stage[r] + ((size_t)p * world + rank) * cap)[i] = v;
    }
    __syncthreads();  // the CTA's remote stores are ordered before the flags below (cumulative with the fence)
    if (threadIdx.x < world) {
        // this CTA's part of my slot is in place on peer `threadIdx.x`
        __threadfence_system();
        volatile uint32_t *f = peers.flags[threadIdx.x] + ((size_t)p * kArMaxCtas + blockIdx.x) * world + rank;
        *f = want;
        // wait for rank `threadIdx.x`'s part in MY staging buffer
        volatile uint32_t *fl = peers.flags[rank] + ((size_t)p * kArMaxCtas + blockIdx.x) * world + threadIdx.x;
        uint32_t it = 0;
        while (*fl != want && ++it < spin) {
        }
        if (*fl != want) {
            s_bad = 1;
            atomicExch(status, 10u);
        }
        __threadfence_system();
    }
    __syncthreads();
    if (i < n4 && !s_bad) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < world; r++) {
            const float4 t = __ldcg(reinterpret_cast<const float4 *>(peers.stage[rank] + ((size_t)p * world + r) * cap) + i);
            acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
        }
        reinterpret_cast<float4 *>(data)[i] = acc;
    }
    // the last CTA of the launch opens the next epoch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ctrl + 1, 1u) == gridDim.x - 1) {
            ctrl[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(ctrl) = epoch + 1u;
        }
    }
}

}  // namespace
}  // namespace infr

struct infr_cuda_comm {
    int rank = 0, world = 1;
    uint32_t cap = 0;            // floats per slot
    uint8_t *local = nullptr;    // this rank's allocation: staging | flags | ctrl
    size_t stage_bytes = 0, flag_bytes = 0;
    size_t push_off = 0, total_bytes = 0;  // the pushed GEMVs' staging ([2][world][push_cap] 8-byte words) follows the control words
    uint32_t push_cap = 0;
    void *peer_base[infr::kMaxWorld] = {};  // mapped allocations of the peers (own entry = local)
    bool connected = false;
    uint32_t spin = infr::kArSpin;  // polls a wait may take before it gives up
    uint8_t *silent = nullptr;      // comm_connect_silent: a stand-in for the peers that nobody ever writes to
    bool pushed = false;            // a GEMV has pushed its result and the consumer has not been enqueued yet
};

namespace infr {

Status CudaBackend::comm_create(int rank, int world, uint32_t max_floats, infr_cuda_comm **out) {
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return Status::Err(INFR_E_INVALID, fmt("comm: rank %d of %d (at most %d ranks)", rank, world, kMaxWorld));
    if (max_floats == 0 || max_floats % 4 || max_floats > (uint32_t)kArMaxCtas * kArThreads * 4)
        return Status::Err(INFR_E_INVALID, fmt("comm: %u floats per exchange (a multiple of 4, at most %d)", max_floats, kArMaxCtas * kArThreads * 4));
    if (capturing_) return Status::Err(INFR_E_INVALID, "comm_create during stream capture");
    cudaSetDevice(device_);
    auto *c = new infr_cuda_comm();
    c->rank = rank;
    c->world = world;
    c->cap = max_floats;
    c->stage_bytes = (size_t)2 * world * max_floats * 4;
    c->flag_bytes = (size_t)2 * kArMaxCtas * world * 4;
    c->push_off = c->stage_bytes + c->flag_bytes + 256;
    c->push_cap = max_floats < kPushMaxFloats ? max_floats : kPushMaxFloats;
    c->total_bytes = c->push_off + (size_t)2 * world * c->push_cap * 8;
    const size_t total = c->total_bytes;
    Status s = cuda_status(cudaMalloc((void **)&c->local, total), "cudaMalloc(comm)");
    if (s.ok()) s = cuda_status(cudaMemsetAsync(c->local, 0, total, stream_), "cudaMemsetAsync(comm)");
    if (s.ok()) s = cuda_status(cudaStreamSynchronize(stream_), "comm sync");
    if (!s.ok()) {
        if (c->local) cudaFree(c->local);
        delete c;
        return s;
    }
    c->peer_base[rank] = c->local;
    c->connected = world == 1;
    *out = c;
    return Status::Ok();
}

Status CudaBackend::comm_export(infr_cuda_comm *c, uint8_t *handle64) {
    if (!c || !handle64) return Status::Err(INFR_E_INVALID, "comm_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaSetDevice(device_);
    cudaIpcMemHandle_t h;
    Status s = cuda_status(cudaIpcGetMemHandle(&h, c->local), "cudaIpcGetMemHandle");
    if (s.ok()) memcpy(handle64, &h, 64);
    return s;
}

Status CudaBackend::comm_connect(infr_cuda_comm *c, const uint8_t *handles) {
    if (!c || !handles) return Status::Err(INFR_E_INVALID, "comm_connect: null argument");
    if (capturing_) return Status::Err(INFR_E_INVALID, "comm_connect during stream capture");
    cudaSetDevice(device_);
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank || c->peer_base[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        Status s = cuda_status(cudaIpcOpenMemHandle(&c->peer_base[r], h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        if (!s.ok()) return s;
    }
    c->connected = true;
    return Status::Ok();
}

// Failure-detection hook: every peer slot is mapped onto one private, zeroed buffer of THIS rank, so this rank's
// stores land somewhere harmless and the peers' flags never arrive; with a short poll limit the next exchange's
// wait runs out, the kernel returns, and the host sees INFR_E_TIMEOUT at its next sync.
Status CudaBackend::comm_connect_silent(infr_cuda_comm *c, uint32_t spin_limit) {
    if (!c) return Status::Err(INFR_E_INVALID, "comm_connect_silent: null comm");
    if (c->connected && c->world > 1) return Status::Err(INFR_E_INVALID, "comm_connect_silent: already connected");
    if (capturing_) return Status::Err(INFR_E_INVALID, "comm_connect_silent during stream capture");
    if (spin_limit == 0 || spin_limit > kArSpin) return Status::Err(INFR_E_INVALID, "comm_connect_silent: poll limit out of range");
    cudaSetDevice(device_);
    const size_t total = c->total_bytes;
    Status s = cuda_status(cudaMalloc((void **)&c->silent, total), "cudaMalloc(comm stand-in)");
    if (s.ok()) s = cuda_status(cudaMemsetAsync(c->silent, 0, total, stream_), "cudaMemsetAsync(comm stand-in)");
    if (s.ok()) s = cuda_status(cudaStreamSynchronize(stream_), "comm sync");
    if (!s.ok()) return s;
    for (int r = 0; r < c->world; r++)
        if (r != c->rank) c->peer_base[r] = c->silent;
    c->spin = spin_limit;
    c->connected = true;
    return Status::Ok();
}

Status CudaBackend::all_reduce_f32(infr_cuda_comm *c, float *data, uint32_t n) {
    if (!c || !data) return Status::Err(INFR_E_INVALID, "all_reduce: null argument");
    if (!c->connected) return Status::Err(INFR_E_INVALID, "all_reduce: the peers' buffers are not connected");
    if (c->pushed) return Status::Err(INFR_E_INVALID, "all_reduce: a pushed GEMV result is waiting for its consumer (rms_norm_q8_pull)");
    if (n == 0) return Status::Ok();
    if (n % 4 || n > c->cap || (uintptr_t)data % 16) return Status::Err(INFR_E_INVALID, fmt("all_reduce: %u floats (a multiple of 4, at most %u, 16-byte aligned)", n, c->cap));
    cudaSetDevice(device_);
    ArPeers peers;
    for (int r = 0; r < kMaxWorld; r++) {
        uint8_t *b = static_cast<uint8_t *>(c->peer_base[r < c->world ? r : c->rank]);
        peers.stage[r] = reinterpret_cast<float *>(b);
        peers.flags[r] = reinterpret_cast<uint32_t *>(b + c->stage_bytes);
    }
    uint32_t *ctrl = reinterpret_cast<uint32_t *>(c->local + c->stage_bytes + c->flag_bytes);
    const uint32_t n4 = n / 4;
    const unsigned grid = (n4 + kArThreads - 1) / kArThreads;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = stream_;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    Status s = cuda_status(cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel, data, n4, c->rank, c->world, c->cap, peers, ctrl, status_dev_, c->spin), "all_reduce");
    if (s.ok()) launches_ += 1;
    return s;
}

// The exchange fused into its producer and its consumer: the row-parallel GEMV's epilogue stores the rank's partial
// result into every rank's staging (slot [rank], the parity of the exchange count), each value in one 8-byte word with
// the exchange's sequence number; the norm that follows polls the words it adds, sums the slots in rank order and
// advances the count (the epoch word of the stand-alone all-reduce, so the two forms can alternate on one comm).  No
// kernel of its own, no fence, no arrival flag; the stores of a tile leave while the other tiles are still computed.
// A slot is written again two exchanges later: by then every rank has consumed it, because a rank pushes exchange
// e + 2 only after its consumer of e + 1 has finished, which needed every rank's push of e + 1, which follows that
// rank's consumer of e in its stream.
Status CudaBackend::gemv_q8_push(infr_cuda_comm *c, int dtype, const uint8_t *w, const Q8Dev &a, uint32_t m, uint32_t in_f, uint32_t out_f) {
    if (!c) return Status::Err(INFR_E_INVALID, "gemv_q8_push: null comm");
    if (!c->connected) return Status::Err(INFR_E_INVALID, "gemv_q8_push: the peers' buffers are not connected");
    if (c->pushed) return Status::Err(INFR_E_INVALID, "gemv_q8_push: the previous pushed result has not been consumed (rms_norm_q8_pull)");
    const bool wide = m > 8 && m <= 32 && wide_applies(dtype, m, in_f, INFR_ACT_INT8);
    if (m < 1 || (m > 8 && !wide))
        return Status::Err(INFR_E_INVALID, fmt("gemv_q8_push: m=%u (1..8; up to 32 where the wide GEMV applies)", m));
    if ((uint64_t)m * out_f > c->push_cap)
        return Status::Err(INFR_E_INVALID, fmt("gemv_q8_push: %u x %u results, the comm stages %u pushed floats", m, out_f, c->push_cap));
    const bool q4 = dtype == DT_Q4K && in_f && in_f % 256 == 0, q6 = dtype == DT_Q6K && in_f && in_f % 2048 == 0 && a.sums16;
    if (!q4 && !q6)
        return Status::Err(INFR_E_UNSUPPORTED, "gemv_q8_push: Q4_K rows of whole blocks or Q6_K rows of whole 2048-element chunks (with the per-16 sums)");
    if (a.gran != 256) return Status::Err(INFR_E_INVALID, "gemv_q8_push: activations quantised per 256 elements");
    cudaSetDevice(device_);
    GemvPush p;
    memset(&p, 0, sizeof p);
    for (int r = 0; r < kPushMaxWorld; r++)
        p.stage[r] = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(c->peer_base[r < c->world ? r : c->rank]) + c->push_off);
    p.ctrl = reinterpret_cast<const uint32_t *>(c->local + c->stage_bytes + c->flag_bytes);
    p.cap = c->push_cap;
    p.world = c->world;
    p.rank = c->rank;
    cudaError_t e;
    int n_launch = 1;
    if (wide) {
        // a few dozen rows: the wide GEMV; with several K chunks the kernel that adds them is the one that pushes
        const size_t pb = gemv_wide_partial_bytes((int)m, (int)in_f, (int)out_f);
        Status s = ensure_scratch(pb);
        if (!s.ok()) return s;
        e = launch_gemv_wide(dtype, w, a, nullptr, reinterpret_cast<float *>(scratch()), (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_, &p);
        n_launch = gemv_wide_launches((int)in_f);
    } else {
        e = q4 ? launch_gemv_q4k_mma(w, &a, nullptr, nullptr, (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_, &p)
               : launch_gemv_q6_mma(w, a, nullptr, (int)m, (int)in_f, (int)out_f, dev_, status_dev_, stream_, &p);
    }
    if (e == cudaErrorInvalidValue) return Status::Err(INFR_E_UNSUPPORTED, "gemv_q8_push: the matrix-unit GEMV does not take this shape");
    Status s = cuda_status(e, "gemv_q8_push");
    if (s.ok()) {
        launches_ += (uint64_t)n_launch;
        c->pushed = true;
    }
    return s;
}

Status CudaBackend::rms_norm_q8_pull(infr_cuda_comm *c, const float *a, float *sum_dst, const float *w, uint32_t rows, uint32_t dim, float eps,
                                     const Q8Dev &out) {
    if (!c) return Status::Err(INFR_E_INVALID, "rms_norm_q8_pull: null comm");
    if (!c->pushed) return Status::Err(INFR_E_INVALID, "rms_norm_q8_pull: no pushed GEMV result is waiting (gemv_q8_push comes first)");
    if (rows < 1 || dim == 0 || dim % 256 || (uint64_t)rows * dim > c->push_cap)
        return Status::Err(INFR_E_INVALID, fmt("rms_norm_q8_pull: %u rows of %u (a multiple of 256; the comm stages %u pushed floats)", rows, dim, c->push_cap));
    cudaSetDevice(device_);
    PullArgs p;
    p.stage = reinterpret_cast<const unsigned long long *>(c->local + c->push_off);
    p.ctrl = reinterpret_cast<uint32_t *>(c->local + c->stage_bytes + c->flag_bytes);
    p.cap = c->push_cap;
    p.spin = c->spin;
    p.world = c->world;
    p.status = status_dev_;
    Status s = cuda_status(launch_rms_norm_q8_pull(a, sum_dst, w, (int)rows, (int)dim, eps, const_cast<int8_t *>(out.qs), const_cast<float *>(out.d),
                                                   const_cast<int32_t *>(out.sums), const_cast<int32_t *>(out.sums16), p, stream_),
                           "rms_norm_q8_pull");
    if (s.ok()) {
        launches_++;
        c->pushed = false;
    }
    return s;
}

void CudaBackend::comm_destroy(infr_cuda_comm *c) {
    if (!c) return;
    cudaSetDevice(device_);
    if (!capturing_) cudaStreamSynchronize(stream_);
    for (int r = 0; r < c->world; r++)
        if (r != c->rank && c->peer_base[r] && c->peer_base[r] != c->silent) cudaIpcCloseMemHandle(c->peer_base[r]);
    if (c->silent) cudaFree(c->silent);
    if (c->local) cudaFree(c->local);
    delete c;
}

}  // namespace infr
