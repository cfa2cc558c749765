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
    void *peer_base[infr::kMaxWorld] = {};  // mapped allocations of the peers (own entry = local)
    bool connected = false;
    uint32_t spin = infr::kArSpin;  // polls a wait may take before it gives up
    uint8_t *silent = nullptr;      // comm_connect_silent: a stand-in for the peers that nobody ever writes to
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
    const size_t total = c->stage_bytes + c->flag_bytes + 256;
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
    const size_t total = c->stage_bytes + c->flag_bytes + 256;
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
