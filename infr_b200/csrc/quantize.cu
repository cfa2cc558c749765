// On-GPU activation quantiser: f32 rows -> int8 codes + per-block scale + integer block sums.
//
// Arithmetic follows crates/infr-cpu/src/quant.rs:27-58 (`quantize_q8`, 256-element blocks) and
// :97-117 (`quantize_q8_32`, 32-element blocks) exactly: d = amax / 127 (IEEE division),
// id = d > 0 ? 1/d : 0, q = clamp(roundf(x * id), -127, 127) with round-half-away-from-zero, so the
// codes, scales and sums are bit-identical to the CPU implementation.  The optional f16 outputs are
// the "Q8_1" view of crates/infr-vulkan/shaders/quant_q8.comp:50-60 (dact = f16(d),
// sact = f16(d * float(sum q))).
//
// One warp quantises 256 consecutive elements of a row: lane l owns elements [4l, 4l+4) and
// [128+4l, 128+4l+4), so loads and stores are 16-byte / 4-byte coalesced and every reduction is a
// handful of shuffles.  The kernel is bandwidth-trivial (activations are KBs) and exists to keep the
// whole Linear on the device.
#include <cuda_fp16.h>

#include "kernels.h"
#include "pdl.cuh"
#include "q8_code.cuh"

namespace infr {

__device__ __forceinline__ float amax4(float4 v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

__device__ __forceinline__ int q1(float v, float id) { return q8_round_code(v, id); }

template <int GRAN>
__global__ void __launch_bounds__(256) quantize_q8_kernel(const float *__restrict__ x, int rows, int k,
                                                          int8_t *__restrict__ qs, float *__restrict__ d,
                                                          int32_t *__restrict__ sums,
                                                          int32_t *__restrict__ sums16,
                                                          __half *__restrict__ dact,
                                                          __half *__restrict__ sact) {
    pdl_go();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int cpr = (k + 255) / 256;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)rows * cpr) return;
    const int row = (int)(wg / cpr), chunk = (int)(wg % cpr);
    const int e[2] = {chunk * 256 + lane * 4, chunk * 256 + 128 + lane * 4};
    const float *xr = x + (size_t)row * k;
    float4 v[2];
    bool ok[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        ok[h] = e[h] < k;
        v[h] = ok[h] ? *reinterpret_cast<const float4 *>(xr + e[h]) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float a[2] = {amax4(v[0]), amax4(v[1])};
    float dd[2];
    if (GRAN == 256) {
        float m = fmaxf(a[0], a[1]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        dd[0] = dd[1] = m / 127.0f;
    } else {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float m = a[h];
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            dd[h] = m / 127.0f;
        }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float id = dd[h] > 0.0f ? 1.0f / dd[h] : 0.0f;
        const int q0 = q1(v[h].x, id), q1_ = q1(v[h].y, id), q2 = q1(v[h].z, id), q3 = q1(v[h].w, id);
        int s = q0 + q1_ + q2 + q3;
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        const int s16 = s;
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (!ok[h]) continue;
        const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1_ & 0xff) << 8) |
                                ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        *reinterpret_cast<uint32_t *>(qs + (size_t)row * k + e[h]) = packed;
        if (sums16 && (lane & 3) == 0) sums16[(size_t)row * (k / 16) + e[h] / 16] = s16;
        if ((lane & 7) == 0) {
            const size_t b32 = (size_t)row * (k / 32) + e[h] / 32;
            sums[b32] = s;
            if (GRAN == 32) {
                d[b32] = dd[h];
                if (dact) {
                    dact[b32] = __float2half_rn(dd[h]);
                    sact[b32] = __float2half_rn(__fmul_rn(dd[h], (float)s));
                }
            }
        }
    }
    if (GRAN == 256 && lane == 0) d[(size_t)row * (k / 256) + chunk] = dd[0];
}

cudaError_t launch_quantize_q8(const float *x, int rows, int k, int gran, int8_t *qs, float *d,
                               int32_t *sums, int32_t *sums16, uint16_t *dact, uint16_t *sact,
                               cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    const long long warps = (long long)rows * ((k + 255) / 256);
    const int threads = 256;
    const unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
    if (gran == 256)
        return launch_pdl(quantize_q8_kernel<256>, dim3(blocks), dim3(threads), 0, st, x, rows, k, qs, d, sums, sums16, (__half *)nullptr,
                          (__half *)nullptr);
    return launch_pdl(quantize_q8_kernel<32>, dim3(blocks), dim3(threads), 0, st, x, rows, k, qs, d, sums, sums16, reinterpret_cast<__half *>(dact),
                      reinterpret_cast<__half *>(sact));
}

__global__ void fill_u32_kernel(uint32_t *p, size_t n, uint32_t v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) p[i] = v;
}

cudaError_t launch_fill_u32(uint32_t *p, size_t n, uint32_t v, cudaStream_t st) {
    if (!n) return cudaSuccess;
    fill_u32_kernel<<<148 * 8, 256, 0, st>>>(p, n, v);
    return cudaGetLastError();
}

}  // namespace infr
