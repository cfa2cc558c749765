// Dense int8 tensor-core peak of the device, measured: the denominator of the prefill GEMM's roofline.
//
// Every SM runs one CTA that issues `tcgen05.mma.cta_group::1.kind::i8` instructions of the largest shape
// (M = 128, N = 256, K = 32: 2 097 152 int8 multiply-adds each) from operands that already sit in shared memory
// in the layout the instruction reads (K-major 16-byte planes, no swizzle) — no unpacking, no epilogue, no global
// traffic inside the loop.  Two threads of different warps issue to their own 256-column accumulators in tensor
// memory (a single issuing thread is the limit for smaller shapes; with two the tensor pipe is never waiting for
// an issuer), in batches of 64 instructions closed by a commit; an issuer waits for batch i - 1 only after it has
// queued batch i, so the pipe never drains.  The instruction form, descriptors and layouts are those of the
// prefill GEMM (mmq_ws.cu), which the parity tests check bit for bit; on top of that the launch returns one
// accumulator element per issuer for the host to compare with the value the operand pattern implies.
// All waits are bounded; an expired wait sets the status word and the CTA frees its tensor memory and leaves.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace infr {
namespace {

constexpr int kPM = 128, kPN = 256, kPK = 256;            // K of the resident operands: 8 instructions of K = 32
constexpr int kABytes = kPK / 16 * kPM * 16;              // 32 KB
constexpr int kBBytes = kPK / 16 * kPN * 16;              // 64 KB
constexpr int kPeakSmem = 120 * 1024;                     // more than half an SM: one CTA (512 tensor-memory columns) per SM
constexpr int kBatch = 64;
constexpr uint32_t kPeakSpin = 1u << 22;

__device__ __forceinline__ uint32_t psu32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t peak_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ bool peak_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kPeakSpin; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}

// Operand pattern (also evaluated on the host): A[row][k] = (7 row + 13 k) mod 16 (the range of 4-bit codes),
// B[col][k] = (5 col + 11 k) mod 31 - 15.
__host__ __device__ inline int peak_a(int row, int k) { return (7 * row + 13 * k) & 15; }
__host__ __device__ inline int peak_b(int col, int k) { return (5 * col + 11 * k) % 31 - 15; }

__global__ void __launch_bounds__(128, 1)
    tensor_peak_i8_kernel(uint32_t n_batches, int32_t *__restrict__ check, uint32_t *__restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sA = smem;            // [kPK/16][kPM][16]
    uint8_t *sB = smem + kABytes;  // [kPK/16][kPN][16]
    __shared__ uint64_t bars[2][2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_bad;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        s_bad = 0;
        for (int i = 0; i < 4; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(psu32(&bars[i >> 1][i & 1])), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(psu32(&tmem_base_s)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    for (int i = tid; i < kPK / 16 * kPM; i += 128) {
        const int k16 = i / kPM, r = i % kPM;
        uint32_t w[4];
        for (int q = 0; q < 4; q++) {
            w[q] = 0;
            for (int b = 0; b < 4; b++) w[q] |= (uint32_t)peak_a(r, k16 * 16 + q * 4 + b) << (8 * b);
        }
        *reinterpret_cast<uint4 *>(sA + (size_t)i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (int i = tid; i < kPK / 16 * kPN; i += 128) {
        const int k16 = i / kPN, c = i % kPN;
        uint32_t w[4];
        for (int q = 0; q < 4; q++) {
            w[q] = 0;
            for (int b = 0; b < 4; b++) w[q] |= (uint32_t)(peak_b(c, k16 * 16 + q * 4 + b) & 0xff) << (8 * b);
        }
        *reinterpret_cast<uint4 *>(sB + (size_t)i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;

    if (lane == 0 && warp < 2) {
        const uint32_t dcol = tmem + (uint32_t)warp * kPN;
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kPN >> 3) << 17) | ((uint32_t)(kPM >> 4) << 24);
        bool ok = true;
        uint32_t first = 1;
        for (uint32_t batch = 0; batch < n_batches && ok; batch++) {
            for (int i = 0; i < kBatch; i++) {
                const int s = i & 7;
                const uint64_t da = peak_desc(psu32(sA + (size_t)(2 * s) * kPM * 16), kPM * 16, 128);
                const uint64_t db = peak_desc(psu32(sB + (size_t)(2 * s) * kPN * 16), kPN * 16, 128);
                const uint32_t acc = first ? 0u : 1u;
                first = 0;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(dcol),
                    "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(0)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(psu32(&bars[warp][batch & 1]))
                         : "memory");
            if (batch >= 1) ok = peak_wait(psu32(&bars[warp][(batch - 1) & 1]), ((batch - 1) >> 1) & 1u);
        }
        if (ok && n_batches >= 1) ok = peak_wait(psu32(&bars[warp][(n_batches - 1) & 1]), ((n_batches - 1) >> 1) & 1u);
        if (!ok) {
            // the expired wait lasted orders of magnitude longer than the two batches that can be queued behind it
            s_bad = 1;
            atomicExch(status, 20u);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!s_bad && blockIdx.x == 0 && warp == 0) {
        // element (row 0, column 0) of both accumulators: lane 0 of the first lane quarter, columns 0 and kPN
        uint32_t v0, v1;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v0) : "r"(tmem));
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v1) : "r"(tmem + (uint32_t)kPN));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (lane == 0) {
            check[0] = (int32_t)v0;
            check[1] = (int32_t)v1;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
}

}  // namespace

// One launch: every SM issues 2 x n_batches x 64 instructions.  `check` (device, 2 x int32) receives element
// (0, 0) of the two accumulators of CTA 0.
cudaError_t launch_tensor_peak_i8(uint32_t n_batches, int32_t *check, const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (n_batches == 0 || n_batches > 4096) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(tensor_peak_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem);
    if (e != cudaSuccess) return e;
    tensor_peak_i8_kernel<<<dev.sm_count, 128, kPeakSmem, st>>>(n_batches, check, status);
    return cudaGetLastError();
}

// int8 multiply-add operations (2 per MAC) of one launch, and the accumulator value the operand pattern implies
// after n_batches batches (int32 wrap-around included, as the hardware accumulates).
double tensor_peak_i8_ops(uint32_t n_batches, const DeviceInfo &dev) {
    return 2.0 * kPM * kPN * 32 * (double)kBatch * n_batches * 2.0 * dev.sm_count;
}
int32_t tensor_peak_i8_expected(uint32_t n_batches) {
    long long once = 0;  // one pass over the resident K = 256
    for (int k = 0; k < kPK; k++) once += (long long)peak_a(0, k) * peak_b(0, k);
    const long long total = once * (kBatch / 8) * (long long)n_batches;
    return (int32_t)(uint32_t)(unsigned long long)total;
}

}  // namespace infr
