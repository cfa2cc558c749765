// A decode GEMV for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc (or anything that allocates) at the moment they
// need a matvec: a plugin that runs inside another engine's memory pool and is handed device pointers
// carved out of it, a real-time loop that has promised not to touch the driver's allocator after
// start-up, code running while a capture or another library forbids allocation.  The regular entry
// points keep their quantised activations in a context-owned buffer that grows on demand; this one
// keeps them in a fixed array that is part of the loaded module instead, so the call itself never
// allocates or frees anything.
//
// The array below is file-scope device memory: every GPU that loads the library holds its
// kNoAllocScratchBytes until the process exits.  In host code the NAME of such an array is only a
// host-side stand-in, not a device address — handing it to a kernel would fault (or, where the GPU
// can reach host memory, silently use the wrong bytes) — so the device address is fetched once per
// device with cudaGetSymbolAddress, with that device current, and that pointer is what the kernels get.
#include <mutex>

#include "../../include/infr_cuda.h"
#include "kernels.h"

namespace {

// Upper bounds of one call: m <= 8 rows of in_f <= 16384 activations.
constexpr uint32_t kNoAllocMaxM = 8;
constexpr uint32_t kNoAllocMaxInF = 16384;
// int8 codes + f32 scales (one per 32 at the finest) + i32 sums per 32 + i32 sums per 16
constexpr size_t kCodesBytes = (size_t)kNoAllocMaxM * kNoAllocMaxInF;
constexpr size_t kScaleBytes = (size_t)kNoAllocMaxM * (kNoAllocMaxInF / 32) * 4;
constexpr size_t kSum32Bytes = (size_t)kNoAllocMaxM * (kNoAllocMaxInF / 32) * 4;
constexpr size_t kSum16Bytes = (size_t)kNoAllocMaxM * (kNoAllocMaxInF / 16) * 4;
constexpr size_t kNoAllocScratchBytes = kCodesBytes + kScaleBytes + kSum32Bytes + kSum16Bytes;  // 192 KiB

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct PerDevice {
    bool ready = false;
    unsigned char *scratch = nullptr;  // device address of g_noalloc_scratch on this device
    infr::DeviceInfo info{};
};
constexpr int kMaxDevices = 64;
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;

void put_error(char *err, size_t cap, const char *msg) {
    if (!err || !cap) return;
    size_t i = 0;
    for (; msg[i] && i + 1 < cap; i++) err[i] = msg[i];
    err[i] = 0;
}

}  // namespace

extern "C" int32_t infr_cuda_gemv_noalloc(int32_t dtype, const void *w, const float *x, float *y, uint32_t m, uint32_t in_f,
                                          uint32_t out_f, void *stream, char *err, size_t err_cap) {
    using namespace infr;
    if (dtype != DT_Q4K && dtype != DT_Q6K && dtype != DT_Q2_0) {
        put_error(err, err_cap, "gemv_noalloc: weight dtype must be Q4_K, Q6_K or Q2_0");
        return INFR_E_UNSUPPORTED;
    }
    if (!w || !x || !y) {
        put_error(err, err_cap, "gemv_noalloc: null device pointer");
        return INFR_E_INVALID;
    }
    if (m == 0 || m > kNoAllocMaxM || in_f == 0 || in_f > kNoAllocMaxInF) {
        put_error(err, err_cap, "gemv_noalloc: the built-in scratch holds at most m = 8 rows of in_f = 16384 activations");
        return INFR_E_INVALID;
    }
    if (in_f % (uint32_t)block_elems(dtype) || in_f % 16) {
        put_error(err, err_cap, "gemv_noalloc: in_f is not a whole number of weight blocks");
        return INFR_E_INVALID;
    }
    // Raw pointers come from the caller's own pool, possibly at odd offsets: the quantiser reads x with 16-byte
    // loads, the Q4_K kernel reads whole 16-byte words of a block, Q6_K / Q2_0 blocks are read in 2-byte units and
    // y is written as f32.  A misaligned pointer must be an error here, not a fault on the device.
    const uintptr_t wa = reinterpret_cast<uintptr_t>(w), xa = reinterpret_cast<uintptr_t>(x), ya = reinterpret_cast<uintptr_t>(y);
    if (xa % 16 || ya % 4 || wa % (dtype == DT_Q4K ? 16u : 2u)) {
        put_error(err, err_cap,
                  "gemv_noalloc: misaligned pointer (x: 16 bytes, y: 4 bytes, w: 16 bytes for Q4_K, 2 bytes for Q6_K / Q2_0)");
        return INFR_E_INVALID;
    }
    if (out_f == 0) return INFR_OK;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        put_error(err, err_cap, "gemv_noalloc: no current CUDA device");
        return INFR_E_CUDA;
    }
    PerDevice *pd = &g_dev[device];
    {
        // One-time set-up per device (the first call on a device; make it before any stream capture).
        std::lock_guard<std::mutex> lock(g_mu);
        if (!pd->ready) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                put_error(err, err_cap, "gemv_noalloc: cudaGetSymbolAddress failed for the built-in scratch");
                return INFR_E_CUDA;
            }
            int sms = 0, smem = 0, l2 = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
                cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess ||
                cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, device) != cudaSuccess) {
                put_error(err, err_cap, "gemv_noalloc: cudaDeviceGetAttribute failed");
                return INFR_E_CUDA;
            }
            pd->scratch = static_cast<unsigned char *>(p);
            pd->info.sm_count = sms;
            pd->info.max_smem_optin = smem;
            pd->info.l2_bytes = (size_t)l2;
            pd->ready = true;
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int gran = act_gran(dtype);
    int8_t *qs = reinterpret_cast<int8_t *>(pd->scratch);
    float *d = reinterpret_cast<float *>(pd->scratch + kCodesBytes);
    int32_t *s32 = reinterpret_cast<int32_t *>(pd->scratch + kCodesBytes + kScaleBytes);
    int32_t *s16 = reinterpret_cast<int32_t *>(pd->scratch + kCodesBytes + kScaleBytes + kSum32Bytes);
    // Nothing in the scratch is accumulated into: the quantiser overwrites every byte the GEMV reads,
    // so there is nothing to clear between calls.
    cudaError_t e = launch_quantize_q8(x, (int)m, (int)in_f, gran, qs, d, s32, dtype == DT_Q6K ? s16 : nullptr, nullptr, nullptr, st);
    if (e == cudaSuccess) {
        Q8Dev a{qs, d, s32, dtype == DT_Q6K ? s16 : nullptr, gran};
        e = launch_gemv_q8(dtype, static_cast<const uint8_t *>(w), a, y, (int)m, (int)in_f, (int)out_f, nullptr, pd->info, st);
    }
    if (e != cudaSuccess) {
        put_error(err, err_cap, cudaGetErrorString(e));
        return INFR_E_CUDA;
    }
    return INFR_OK;
}
