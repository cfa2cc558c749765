// Q2_0 (ternary, 64 elements / 18 bytes: f16 d + 16 bytes of 2-bit codes, w = (code - 1) * d) decode GEMV /
// small-batch GEMM (m <= 8) on the warp-level int8 matrix unit, for rows that are a whole number of
// 512-element chunks (8 blocks = 144 bytes, the 16-byte granule of a TMA box).
//
// Arithmetic of vec_dot_q2_0 (crates/infr-cpu/src/kernels.rs:5641-5668) with activations quantised per 32
// (quantize_q8_32): per 32-element group s of block b
//     iprod = sum_p code_p * q8_p  (exact int32)        y += d_b * d8_s * float(iprod - bsum_s)
//
// One `mma.sync.m16n8k32.u8.s8` is one 32-element group of 16 weight rows against up to 8 activation rows.
// The K index of the instruction is only a summation index: a lane feeds it the 8 codes of two code bytes
// (one 16-bit shared-memory read per row and group), expanded to bytes by two byte permutes and masks, and
// the 8 matching activation bytes, staged in the same order so that a lane reads them with one 64-bit load.  Everything around the block body (tiled TMA into warp-private rings, K split over
// the warps of a CTA, fixed-order reduction, programmatic dependent launch, bounded waits) is the scheme
// of the Q4_K kernel in gemv_mma.cu; the slot geometry is the same 16 rows x 144 bytes.
#include <cuda.h>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kRows = 16;
constexpr int kMaxSlots = 4;
constexpr int kChunkBytes = 144, kChunkElems = 512, kChunkGroups = 16;
constexpr int kSlotBytes = kRows * kChunkBytes;
constexpr int kLaneStride = 136;               // staged bytes of one K lane of a chunk (128 + 8: the four lanes hit distinct banks)
constexpr int kStagedChunk = 4 * kLaneStride;  // staged bytes of one chunk of one token
constexpr uint32_t kSpinQ2 = 1u << 22;

__device__ __forceinline__ uint32_t sm32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wait_parity(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinQ2; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void mma_q2(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// Eight 2-bit codes e0..e7 held in 16 bits -> two words of four bytes, in the order [e0 e4 e1 e5], [e2 e6 e3 e7]
// (a byte permute of x and x >> 2 lines up fields 0 and 1 of both code bytes; the activations are staged
// in the same order).
__device__ __forceinline__ void spread8(uint32_t x, uint32_t &lo, uint32_t &hi) {
    lo = __byte_perm(x, x >> 2, 0x5410) & 0x03030303u;
    hi = __byte_perm(x >> 4, x >> 6, 0x5410) & 0x03030303u;
}

struct Q2Geom {
    int nch;    // 512-element chunks per row
    int cpw;    // chunks per warp (K split)
    int slots;  // ring slots per warp
};

// Shared memory: rings [KW][slots][16 x 144 B]; staged activations per token n and chunk c: codes 544 B
// at (n*nch + c)*544, the 8 bytes of group s that lane t feeds at t*136 + s*8; d8 and bsum [group][8 tokens]
// (a lane's two result columns are neighbours).
template <int M, int KW>
__global__ void __launch_bounds__(KW * 32, 16 / KW)
    gemv_q2_mma_kernel(const __grid_constant__ CUtensorMap tmap, Q8Dev a, float *__restrict__ y, int m, int in_f, int out_f,
                       Q2Geom geo, uint32_t *__restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int nch = geo.nch, S = geo.slots, ng = nch * kChunkGroups;
    uint8_t *rings = smem;
    uint8_t *s_codes = smem + (size_t)KW * S * kSlotBytes;
    float *s_d8 = reinterpret_cast<float *>(s_codes + (size_t)M * nch * kStagedChunk);  // [ng][8]
    int32_t *s_bs = reinterpret_cast<int32_t *>(s_d8 + (size_t)8 * ng);               // [ng][8]
    float *s_part = reinterpret_cast<float *>(s_bs + (size_t)8 * ng);                  // [2][KW][16][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_part + 2 * KW * 128);  // [KW][kMaxSlots]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        for (int i = 0; i < KW * kMaxSlots; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm32(bars + i)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // balanced contiguous range of 16-row tiles of this CTA
    const int total_tiles = (out_f + kRows - 1) / kRows;
    const int G = gridDim.x, base = total_tiles / G, rem = total_tiles % G;
    const int t_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int n_tiles = base + (blockIdx.x < rem ? 1 : 0);
    const int r_begin = t_begin * kRows;
    const int c0 = warp * geo.cpw, c1 = min(nch, c0 + geo.cpw);
    const int my_chunks = max(0, c1 - c0);
    const int n_jobs = n_tiles * my_chunks;
    uint8_t *ring = rings + (size_t)warp * S * kSlotBytes;
    uint64_t *wbar = bars + warp * kMaxSlots;

    int j_issue = 0, i_tile = 0, i_ch = 0;
    auto issue = [&](int slot) {
        if (j_issue >= n_jobs) return;
        if (lane == 0) {
            const uint32_t bar = sm32(wbar + slot);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier reads of the slot come first
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kSlotBytes) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                             sm32(ring + (size_t)slot * kSlotBytes)),
                         "l"(&tmap), "r"((c0 + i_ch) * 36), "r"(r_begin + i_tile * kRows), "r"(bar)
                         : "memory");
        }
        __syncwarp();
        j_issue++;
        if (++i_ch == my_chunks) {
            i_ch = 0;
            i_tile++;
        }
    };
    for (int s = 0; s < S; s++) issue(s);

    // ---- activations (from the previous kernel in the stream) ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        // eight independent 8-byte loads in flight per thread (the copy is latency-bound)
        const int units = in_f / 8;
        for (int n = 0; n < M; n++) {
            const bool on = n < m;
            for (int u0 = threadIdx.x; u0 < units; u0 += 8 * KW * 32) {
                uint2 v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const int u = u0 + k * KW * 32;
                    v[k] = make_uint2(0, 0);
                    if (on && u < units) v[k] = *reinterpret_cast<const uint2 *>(a.qs + (size_t)n * in_f + (size_t)u * 8);
                }
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const int u = u0 + k * KW * 32;
                    const int c = u >> 6, uu = u & 63, s = uu >> 2, tt = uu & 3;
                    // bytes e0..e7 -> [e0 e4 e1 e5], [e2 e6 e3 e7]: the order spread8 gives the codes
                    const uint2 pv = make_uint2(__byte_perm(v[k].x, v[k].y, 0x5140), __byte_perm(v[k].x, v[k].y, 0x7362));
                    if (u < units) *reinterpret_cast<uint2 *>(s_codes + (size_t)(n * nch + c) * kStagedChunk + tt * kLaneStride + s * 8) = pv;
                }
            }
        }
        for (int i = threadIdx.x; i < ng * 8; i += KW * 32) {
            const int gi = i >> 3, n = i & 7;
            const bool on = n < m;
            s_d8[i] = on ? a.d[(size_t)n * ng + gi] : 0.f;
            s_bs[i] = on ? a.sums[(size_t)n * ng + gi] : 0;
        }
    }
    __syncthreads();

    // ---- consume ----
    const int gt = g < M ? g : 0;            // token whose codes this lane feeds as its B column
    const int n0 = 2 * t, n1 = 2 * t + 1;    // tokens of this lane's result columns
    int slot = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int tile = 0; tile < n_tiles; tile++) {
        float accf[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ci = 0; ci < my_chunks; ci++) {
            if (!dead && !wait_parity(sm32(wbar + slot), phase)) {
                dead = true;
                if (lane == 0) atomicExch(status, 3u);
            }
            if (!dead) {
                const int c = c0 + ci;
                const uint8_t *r0 = ring + (size_t)slot * kSlotBytes + (size_t)g * kChunkBytes, *r1 = r0 + 8 * kChunkBytes;
                const uint8_t *bp = s_codes + (size_t)(gt * nch + c) * kStagedChunk + t * kLaneStride;
#pragma unroll
                for (int bq = 0; bq < 8; bq++) {
                    const float d0 = h2f(*reinterpret_cast<const unsigned short *>(r0 + bq * 18));
                    const float d1 = h2f(*reinterpret_cast<const unsigned short *>(r1 + bq * 18));
#pragma unroll
                    for (int sub = 0; sub < 2; sub++) {
                        const int s = 2 * bq + sub;
                        const uint32_t x0 = *reinterpret_cast<const unsigned short *>(r0 + bq * 18 + 2 + 8 * sub + 2 * t);
                        const uint32_t x1 = *reinterpret_cast<const unsigned short *>(r1 + bq * 18 + 2 + 8 * sub + 2 * t);
                        const uint2 bv = *reinterpret_cast<const uint2 *>(bp + s * 8);
                        uint32_t a0, a1, a2, a3;
                        spread8(x0, a0, a2);
                        spread8(x1, a1, a3);
                        int pr[4];
                        mma_q2(pr, a0, a1, a2, a3, bv.x, bv.y);
                        // scales and sums of the lane's two result columns (zero for absent tokens: no branch)
                        const int gi = c * kChunkGroups + s;
                        const float2 e = *reinterpret_cast<const float2 *>(s_d8 + gi * 8 + n0);
                        const int2 bs = *reinterpret_cast<const int2 *>(s_bs + gi * 8 + n0);
                        accf[0] = fmaf(d0 * e.x, (float)(pr[0] - bs.x), accf[0]);
                        accf[2] = fmaf(d1 * e.x, (float)(pr[2] - bs.x), accf[2]);
                        if (M > 1) {
                            accf[1] = fmaf(d0 * e.y, (float)(pr[1] - bs.y), accf[1]);
                            accf[3] = fmaf(d1 * e.y, (float)(pr[3] - bs.y), accf[3]);
                        }
                    }
                }
            }
            __syncwarp();
            issue(slot);
            if (++slot == S) {
                slot = 0;
                phase ^= 1u;
            }
        }
        // partial sums of this warp's K range: [row 0..15][token 0..7]
        float *part = s_part + ((size_t)(tile & 1) * KW + warp) * 128;
        part[g * 8 + n0] = accf[0];
        part[g * 8 + n1] = accf[1];
        part[(g + 8) * 8 + n0] = accf[2];
        part[(g + 8) * 8 + n1] = accf[3];
        __syncthreads();
        if (threadIdx.x < kRows * 8) {  // 16 rows x 8 token columns; CTAs have at least 128 threads
            const int r = threadIdx.x >> 3, n = threadIdx.x & 7;
            const int row = r_begin + tile * kRows + r;
            if (n < m && row < out_f) {
                const float *pp = s_part + (size_t)(tile & 1) * KW * 128 + r * 8 + n;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < KW; w++) v += pp[w * 128];
                y[(size_t)n * out_f + row] = v;
            }
        }
    }
}

typedef CUresult (*EncQ2)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                          const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                          CUtensorMapFloatOOBfill);
EncQ2 enc_q2() {
    static EncQ2 fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncQ2>(p);
    }();
    return fn;
}

template <int M, int KW>
cudaError_t launch_cfg(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                       uint32_t *status, cudaStream_t st) {
    Q2Geom geo;
    geo.nch = in_f / kChunkElems;
    geo.cpw = (geo.nch + KW - 1) / KW;
    const size_t ng = (size_t)geo.nch * kChunkGroups;
    const size_t fixed = (size_t)M * geo.nch * kStagedChunk + ng * 64 + (size_t)2 * KW * 128 * 4 + (size_t)KW * kMaxSlots * 8 + 64;
    const size_t per_slot = (size_t)KW * kSlotBytes;
    if (fixed + 2 * per_slot > (size_t)dev.max_smem_optin - 1024) return cudaErrorInvalidValue;
    int per_sm = 16 / KW;
    while (per_sm > 1 && fixed + 2 * per_slot > (size_t)dev.max_smem_optin / per_sm - 2048) per_sm /= 2;
    const size_t budget = (size_t)dev.max_smem_optin / per_sm - (per_sm > 1 ? 2048 : 1024);
    int slots = (int)((budget - fixed) / per_slot);
    if (slots > kMaxSlots) slots = kMaxSlots;
    geo.slots = slots;
    const size_t smem = fixed + (size_t)slots * per_slot;
    int grid = (out_f + kRows - 1) / kRows;
    if (grid > dev.sm_count * per_sm) grid = dev.sm_count * per_sm;
    EncQ2 enc = enc_q2();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)geo.nch * 36, (cuuint64_t)out_f};
    const cuuint64_t gstride[1] = {(cuuint64_t)geo.nch * kChunkBytes};
    const cuuint32_t box[2] = {36, (cuuint32_t)kRows};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(w), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    auto kernel = gemv_q2_mma_kernel<M, KW>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(KW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tmap, a, y, m, in_f, out_f, geo, status);
}

template <int M>
cudaError_t launch_m(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                     uint32_t *status, cudaStream_t st) {
    const int nch = in_f / kChunkElems, tiles = (out_f + kRows - 1) / kRows;
    auto need = [&](int kw) { return (size_t)M * nch * kStagedChunk + (size_t)nch * kChunkGroups * 64 + (size_t)2 * kw * 512 + (size_t)kw * kMaxSlots * 8 + 64 + (size_t)2 * kw * kSlotBytes; };
    // as for Q4_K: few tiles -> more warps split a tile's K; many tiles -> four warps per tile
    int kw = tiles > 2 * dev.sm_count ? 4 : (tiles > dev.sm_count ? 8 : 16);
    while (kw < 16 && need(kw) > (size_t)dev.max_smem_optin / (16 / kw) - 2048) kw *= 2;
    while (kw > 4 && kw > nch) kw /= 2;
    while (kw > 4 && need(kw) > (size_t)dev.max_smem_optin - 1024) kw /= 2;
    if (kw == 16) return launch_cfg<M, 16>(w, a, y, m, in_f, out_f, dev, status, st);
    if (kw == 8) return launch_cfg<M, 8>(w, a, y, m, in_f, out_f, dev, status, st);
    return launch_cfg<M, 4>(w, a, y, m, in_f, out_f, dev, status, st);
}

}  // namespace

// cudaErrorInvalidValue when the shape does not qualify (rows not a whole number of 512-element chunks, or
// the staged activations do not fit): the caller falls back to the dp4a kernel.
cudaError_t launch_gemv_q2_mma(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                               uint32_t *status, cudaStream_t st) {
    if (m < 1 || m > 8 || in_f % kChunkElems || a.gran != 32) return cudaErrorInvalidValue;
    if (m == 1) return launch_m<1>(w, a, y, m, in_f, out_f, dev, status, st);
    if (m == 2) return launch_m<2>(w, a, y, m, in_f, out_f, dev, status, st);
    if (m <= 4) return launch_m<4>(w, a, y, m, in_f, out_f, dev, status, st);
    return launch_m<8>(w, a, y, m, in_f, out_f, dev, status, st);
}

}  // namespace infr
