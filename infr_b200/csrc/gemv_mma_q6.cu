// Q6_K (256 elements / 210 bytes: ql[128] low nibbles, qh[64] high 2 bits, 16 int8 sub-block scales, f16 d;
// w = d * sc_s * (q - 32)) decode GEMV / small-batch GEMM (m <= 8) on the warp-level int8 matrix unit, for
// rows whose byte length is a multiple of 16 (8 | blocks per row), the stride rule of a TMA tensor map.
//
// Arithmetic of vec_dot_q6k (vec_dot_q6k_scalar, crates/infr-cpu/src/kernels.rs:487-526): per block
//     isum = sum_s sc_s * (sum_{l in s} q_l a_l - 32 * bsum16_s)      exact int32, 16 sub-blocks of 16
//     y   += d * d8 * float(isum)
//
// One `mma.sync.m16n8k16.u8.s8` is one sub-block of 16 weight rows against up to 8 activation rows: the
// unsigned 6-bit codes go in as they are and the -32 is applied through the activation sums, themselves one
// more pair of instructions per block (A = the 16 scales, B = bsum16 split as 64 h + l).  The K index of the
// instruction is only a summation index; a lane feeds it 4 consecutive codes assembled from one word of ql
// and one of qh, and the 4 matching activation bytes, staged so that its 16 words of a block are contiguous.
//
// A 210-byte block starts at an even but not always 4-aligned address.  The TMA box of a block therefore
// starts at the 16-byte boundary below it and is 224 bytes wide; odd blocks sit 2 bytes off a word boundary
// and their words are put together from two aligned loads with a funnel shift.
// Everything around the block body (warp-private TMA rings, K split over the warps of a CTA, fixed-order
// reduction, programmatic dependent launch, bounded waits) is the scheme of the Q4_K kernel in gemv_mma.cu.
#include <cuda.h>

#include <cstring>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kRows6 = 16;
constexpr int kMaxSlots6 = 4;
constexpr int kPitch = 224;                     // bytes of one row of a slot: a block (210) + up to 14 bytes before it
constexpr int kSlotBytes6 = kRows6 * kPitch;
constexpr int kLane6 = 80;                      // staged bytes of one K lane of a block (64 + 16: distinct banks for 128-bit reads)
constexpr int kStagedBlock = 4 * kLane6 + 32;   // + bsum16 split: 16 bytes l, 16 bytes h
constexpr uint32_t kSpin6 = 1u << 22;

__device__ __forceinline__ uint32_t sm6(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wait_parity6(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpin6; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
// D = A(16x16, u8) * B(16x8, s8), int32, zero accumulator input
__device__ __forceinline__ void mma_k16_us(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void mma_k16_ss(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// word at byte offset `off` (a multiple of 4) of a block that starts at p; ODD: p is 2 bytes past a word boundary
template <bool ODD>
__device__ __forceinline__ uint32_t ldw(const uint8_t *p, int off) {
    if (!ODD) return *reinterpret_cast<const uint32_t *>(p + off);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(p + off - 2);
    return __funnelshift_r(q[0], q[1], 16);
}
__device__ __forceinline__ int sbyte(uint32_t w, int k) { return (int)(int8_t)(w >> (8 * k)); }

struct Q6Geom {
    int nb;     // blocks per row
    int bpw;    // blocks per warp (K split)
    int slots;  // ring slots per warp
};

template <int M, bool ODD>
__device__ __forceinline__ void block_q6(const uint8_t *p0, const uint8_t *p1, const uint8_t *st, const float *s_d8b, int t, int n0,
                                         float (&accf)[4]) {
    // the lane's 16 activation words of the block (one per sub-block) and its words of the split sums
    uint32_t bw[16];
    {
        const uint4 *bp = reinterpret_cast<const uint4 *>(st + t * kLane6);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 v = bp[i];
            bw[4 * i] = v.x, bw[4 * i + 1] = v.y, bw[4 * i + 2] = v.z, bw[4 * i + 3] = v.w;
        }
    }
    const uint32_t bl = *reinterpret_cast<const uint32_t *>(st + 4 * kLane6 + 4 * t);
    const uint32_t bh = *reinterpret_cast<const uint32_t *>(st + 4 * kLane6 + 16 + 4 * t);
    uint32_t sc0[4], sc1[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        sc0[i] = ldw<ODD>(p0, 192 + 4 * i);
        sc1[i] = ldw<ODD>(p1, 192 + 4 * i);
    }
    int isum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int n = 0; n < 2; n++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int o = n * 64 + j * 16 + 4 * t, oh = 128 + n * 32 + j * 16 + 4 * t;
            const uint32_t qa0 = ldw<ODD>(p0, o), qb0 = ldw<ODD>(p0, o + 32), qh0 = ldw<ODD>(p0, oh);
            const uint32_t qa1 = ldw<ODD>(p1, o), qb1 = ldw<ODD>(p1, o + 32), qh1 = ldw<ODD>(p1, oh);
            uint32_t a0[4], a1[4];
            a0[0] = (qa0 & 0x0F0F0F0Fu) | ((qh0 << 4) & 0x30303030u);
            a0[1] = (qb0 & 0x0F0F0F0Fu) | ((qh0 << 2) & 0x30303030u);
            a0[2] = ((qa0 >> 4) & 0x0F0F0F0Fu) | (qh0 & 0x30303030u);
            a0[3] = ((qb0 >> 4) & 0x0F0F0F0Fu) | ((qh0 >> 2) & 0x30303030u);
            a1[0] = (qa1 & 0x0F0F0F0Fu) | ((qh1 << 4) & 0x30303030u);
            a1[1] = (qb1 & 0x0F0F0F0Fu) | ((qh1 << 2) & 0x30303030u);
            a1[2] = ((qa1 >> 4) & 0x0F0F0F0Fu) | (qh1 & 0x30303030u);
            a1[3] = ((qb1 >> 4) & 0x0F0F0F0Fu) | ((qh1 >> 2) & 0x30303030u);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int s = n * 8 + 2 * c + j;  // sub-block = element / 16
                int pr[4];
                mma_k16_us(pr, a0[c], a1[c], bw[s]);
                const int s0 = sbyte(sc0[s >> 2], s & 3), s1 = sbyte(sc1[s >> 2], s & 3);
                isum[0] += s0 * pr[0];
                isum[2] += s1 * pr[2];
                if (M > 1) {
                    isum[1] += s0 * pr[1];
                    isum[3] += s1 * pr[3];
                }
            }
        }
    }
    // -32 * sum_s sc_s * bsum16_s, bsum16 = 64 h + l
    const uint32_t st0 = t == 0 ? sc0[0] : t == 1 ? sc0[1] : t == 2 ? sc0[2] : sc0[3];  // scales of sub-blocks 4t..4t+3
    const uint32_t st1 = t == 0 ? sc1[0] : t == 1 ? sc1[1] : t == 2 ? sc1[2] : sc1[3];
    int cl[4], ch[4];
    mma_k16_ss(cl, st0, st1, bl);
    mma_k16_ss(ch, st0, st1, bh);
    const float d0 = h2f(*reinterpret_cast<const unsigned short *>(p0 + 208));
    const float d1 = h2f(*reinterpret_cast<const unsigned short *>(p1 + 208));
    const float2 e = *reinterpret_cast<const float2 *>(s_d8b + n0);  // zero for absent tokens
    accf[0] = fmaf(d0 * e.x, (float)(isum[0] - 32 * (cl[0] + 64 * ch[0])), accf[0]);
    accf[2] = fmaf(d1 * e.x, (float)(isum[2] - 32 * (cl[2] + 64 * ch[2])), accf[2]);
    if (M > 1) {
        accf[1] = fmaf(d0 * e.y, (float)(isum[1] - 32 * (cl[1] + 64 * ch[1])), accf[1]);
        accf[3] = fmaf(d1 * e.y, (float)(isum[3] - 32 * (cl[3] + 64 * ch[3])), accf[3]);
    }
}

// Shared memory: rings [KW][slots][16 x 224 B]; staged activations per token n and block b: 352 B at
// (n*nb + b)*352 = four K lanes of 80 B (lane t: its 4 bytes of sub-block s at t*80 + s*4) + the split sums;
// d8 [block][8 tokens].
template <int M, int KW, bool PUSH>
__global__ void __launch_bounds__(KW * 32, 16 / KW)
    gemv_q6_mma_kernel(const __grid_constant__ CUtensorMap tmap, Q8Dev a, float *__restrict__ y, int m, int in_f, int out_f,
                       Q6Geom geo, uint32_t *__restrict__ status, const __grid_constant__ typename PushParam<PUSH>::type push) {
    __shared__ uint32_t s_epoch;  // push mode: exchanges completed before this launch
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = geo.nb, S = geo.slots;
    uint8_t *rings = smem;
    uint8_t *s_act = smem + (size_t)KW * S * kSlotBytes6;                              // [M][nb][352]
    float *s_d8 = reinterpret_cast<float *>(s_act + (size_t)M * nb * kStagedBlock);    // [nb][8]
    float *s_part = s_d8 + (size_t)nb * 8;                                             // [2][KW][16][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_part + 2 * KW * 128);              // [KW][kMaxSlots6]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        for (int i = 0; i < KW * kMaxSlots6; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm6(bars + i)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int total_tiles = (out_f + kRows6 - 1) / kRows6;
    const int G = gridDim.x, base = total_tiles / G, rem = total_tiles % G;
    const int t_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int n_tiles = base + (blockIdx.x < rem ? 1 : 0);
    const int r_begin = t_begin * kRows6;
    const int b0 = warp * geo.bpw, b1 = min(nb, b0 + geo.bpw);
    const int my_blocks = max(0, b1 - b0);
    const int n_jobs = n_tiles * my_blocks;
    uint8_t *ring = rings + (size_t)warp * S * kSlotBytes6;
    uint64_t *wbar = bars + warp * kMaxSlots6;

    int j_issue = 0, i_tile = 0, i_b = 0;
    auto issue = [&](int slot) {
        if (j_issue >= n_jobs) return;
        if (lane == 0) {
            const uint32_t bar = sm6(wbar + slot);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier reads of the slot come first
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kSlotBytes6) : "memory");
            // x in 16-bit elements: the 16-byte boundary at or below the block's first byte
            const int x = (((b0 + i_b) * 210) & ~15) >> 1;
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                             sm6(ring + (size_t)slot * kSlotBytes6)),
                         "l"(&tmap), "r"(x), "r"(r_begin + i_tile * kRows6), "r"(bar)
                         : "memory");
        }
        __syncwarp();
        j_issue++;
        if (++i_b == my_blocks) {
            i_b = 0;
            i_tile++;
        }
    };
    for (int s = 0; s < S; s++) issue(s);

    // ---- activations (from the previous kernel in the stream) ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (PUSH) {
        if (threadIdx.x == 0) s_epoch = *reinterpret_cast<const volatile uint32_t *>(push.ctrl);  // read by all after the barrier below
    }
    {
        // 16 bytes = the 16 codes of one sub-block = one word for each of the four K lanes; four loads in flight per
        // thread (the copy is latency-bound)
        // (flattened over tokens and units: with one token's few hundred units per pass most of the loads would be masked)
        const int units = in_f / 16, total = M * units;
        for (int i0 = threadIdx.x; i0 < total; i0 += 4 * KW * 32) {
            uint4 v[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = i0 + k * KW * 32, n = M == 1 ? 0 : i / units, u = i - n * units;
                v[k] = make_uint4(0, 0, 0, 0);
                if (i < total && n < m) v[k] = *reinterpret_cast<const uint4 *>(a.qs + (size_t)n * in_f + (size_t)u * 16);
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = i0 + k * KW * 32, n = M == 1 ? 0 : i / units, u = i - n * units;
                if (i < total) {
                    uint8_t *dst = s_act + (size_t)(n * nb + (u >> 4)) * kStagedBlock + (u & 15) * 4;
                    *reinterpret_cast<uint32_t *>(dst) = v[k].x;
                    *reinterpret_cast<uint32_t *>(dst + kLane6) = v[k].y;
                    *reinterpret_cast<uint32_t *>(dst + 2 * kLane6) = v[k].z;
                    *reinterpret_cast<uint32_t *>(dst + 3 * kLane6) = v[k].w;
                }
            }
        }
        for (int i = threadIdx.x; i < M * nb * 16; i += KW * 32) {
            const int n = i / (nb * 16), r = i - n * nb * 16, b = r >> 4, s = r & 15;
            const int bs = n < m ? a.sums16[(size_t)n * nb * 16 + r] : 0;
            uint8_t *sp = s_act + (size_t)(n * nb + b) * kStagedBlock + 4 * kLane6;
            sp[s] = (uint8_t)(bs & 63);
            sp[16 + s] = (uint8_t)(int8_t)(bs >> 6);
        }
        for (int i = threadIdx.x; i < nb * 8; i += KW * 32) {
            const int b = i >> 3, n = i & 7;
            s_d8[i] = n < m ? a.d[(size_t)n * nb + b] : 0.f;
        }
    }
    __syncthreads();

    // ---- consume ----
    const int gt = g < M ? g : 0;  // token whose codes this lane feeds as its B column
    const int n0 = 2 * t;          // first of this lane's two result columns
    int slot = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int tile = 0; tile < n_tiles; tile++) {
        float accf[4] = {0.f, 0.f, 0.f, 0.f};
        for (int bi = 0; bi < my_blocks; bi++) {
            if (!dead && !wait_parity6(sm6(wbar + slot), phase)) {
                dead = true;
                if (lane == 0) atomicExch(status, 3u);
            }
            if (!dead) {
                const int b = b0 + bi;
                const int off = (b * 210) & 15;
                const uint8_t *p0 = ring + (size_t)slot * kSlotBytes6 + (size_t)g * kPitch + off, *p1 = p0 + 8 * kPitch;
                const uint8_t *st = s_act + (size_t)(gt * nb + b) * kStagedBlock;
                if (b & 1)
                    block_q6<M, true>(p0, p1, st, s_d8 + b * 8, t, n0, accf);
                else
                    block_q6<M, false>(p0, p1, st, s_d8 + b * 8, t, n0, accf);
            }
            __syncwarp();
            issue(slot);
            if (++slot == S) {
                slot = 0;
                phase ^= 1u;
            }
        }
        float *part = s_part + ((size_t)(tile & 1) * KW + warp) * 128;
        part[g * 8 + n0] = accf[0];
        part[g * 8 + n0 + 1] = accf[1];
        part[(g + 8) * 8 + n0] = accf[2];
        part[(g + 8) * 8 + n0 + 1] = accf[3];
        __syncthreads();
        if (threadIdx.x < kRows6 * 8) {  // 16 rows x 8 token columns; CTAs have at least 128 threads
            const int r = threadIdx.x >> 3, n = threadIdx.x & 7;
            const int row = r_begin + tile * kRows6 + r;
            if (n < m && row < out_f) {
                const float *pp = s_part + (size_t)(tile & 1) * KW * 128 + r * 8 + n;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < KW; w++) v += pp[w * 128];
                if constexpr (PUSH)
                    push_store(push, s_epoch, (size_t)n * out_f + row, v);
                else
                    y[(size_t)n * out_f + row] = v;
            }
        }
    }
}

typedef CUresult (*EncQ6)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                          const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                          CUtensorMapFloatOOBfill);
EncQ6 enc_q6() {
    static EncQ6 fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncQ6>(p);
    }();
    return fn;
}

template <int M, int KW>
cudaError_t launch_cfg6(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                        uint32_t *status, cudaStream_t st, const GemvPush *push) {
    Q6Geom geo;
    geo.nb = in_f / 256;
    geo.bpw = (geo.nb + KW - 1) / KW;
    const size_t fixed = (size_t)M * geo.nb * kStagedBlock + (size_t)geo.nb * 32 + (size_t)2 * KW * 128 * 4 + (size_t)KW * kMaxSlots6 * 8 + 64;
    const size_t per_slot = (size_t)KW * kSlotBytes6;
    if (fixed + 2 * per_slot > (size_t)dev.max_smem_optin - 1024) return cudaErrorInvalidValue;
    int per_sm = 16 / KW;
    while (per_sm > 1 && fixed + 2 * per_slot > (size_t)dev.max_smem_optin / per_sm - 2048) per_sm /= 2;
    const size_t budget = (size_t)dev.max_smem_optin / per_sm - (per_sm > 1 ? 2048 : 1024);
    int slots = (int)((budget - fixed) / per_slot);
    if (slots > kMaxSlots6) slots = kMaxSlots6;
    geo.slots = slots;
    const size_t smem = fixed + (size_t)slots * per_slot;
    int grid = (out_f + kRows6 - 1) / kRows6;
    if (grid > dev.sm_count * per_sm) grid = dev.sm_count * per_sm;
    EncQ6 enc = enc_q6();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap tmap;
    // rows of nb * 105 16-bit elements; a box is 112 elements (224 B) x 16 rows and may run past the row's end (zero-filled)
    const cuuint64_t gdim[2] = {(cuuint64_t)geo.nb * 105, (cuuint64_t)out_f};
    const cuuint64_t gstride[1] = {(cuuint64_t)geo.nb * 210};
    const cuuint32_t box[2] = {(cuuint32_t)kPitch / 2, (cuuint32_t)kRows6};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<uint8_t *>(w), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    auto kernel = gemv_q6_mma_kernel<M, KW, false>;
    auto kernel_push = gemv_q6_mma_kernel<M, KW, true>;
    cudaError_t e = push ? cudaFuncSetAttribute(kernel_push, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
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
    if (push) return cudaLaunchKernelEx(&cfg, kernel_push, tmap, a, y, m, in_f, out_f, geo, status, *push);
    return cudaLaunchKernelEx(&cfg, kernel, tmap, a, y, m, in_f, out_f, geo, status, NoPush{});
}

template <int M>
cudaError_t launch_m6(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                      uint32_t *status, cudaStream_t st, const GemvPush *push) {
    const int nb = in_f / 256, tiles = (out_f + kRows6 - 1) / kRows6;
    auto need_slots = [&](int kw, int slots) {
        return (size_t)M * nb * kStagedBlock + (size_t)nb * 32 + (size_t)2 * kw * 512 + (size_t)kw * kMaxSlots6 * 8 + 64 +
               (size_t)slots * kw * kSlotBytes6;
    };
    auto need = [&](int kw) { return need_slots(kw, 2); };
    // as for Q4_K: few tiles -> more warps split a tile's K; many tiles -> four warps per tile
    int kw = tiles > 2 * dev.sm_count ? 4 : (tiles > dev.sm_count ? 8 : 16);
    // four-warp CTAs want three ring slots per warp (with two, a batch of 4 ran 20 % slower than 8-warp CTAs)
    if (kw == 4 && need_slots(4, 3) > (size_t)dev.max_smem_optin / 4 - 2048) kw = 8;
    while (kw < 16 && need(kw) > (size_t)dev.max_smem_optin / (16 / kw) - 2048) kw *= 2;
    while (kw > 4 && kw > nb) kw /= 2;
    while (kw > 4 && need(kw) > (size_t)dev.max_smem_optin - 1024) kw /= 2;
    if (kw == 16) return launch_cfg6<M, 16>(w, a, y, m, in_f, out_f, dev, status, st, push);
    if (kw == 8) return launch_cfg6<M, 8>(w, a, y, m, in_f, out_f, dev, status, st, push);
    return launch_cfg6<M, 4>(w, a, y, m, in_f, out_f, dev, status, st, push);
}

}  // namespace

// cudaErrorInvalidValue when the shape does not qualify (row bytes not a multiple of 16, no 16-element sums,
// or the staged activations do not fit): the caller falls back to the byte-dot kernel.
cudaError_t launch_gemv_q6_mma(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                               uint32_t *status, cudaStream_t st, const GemvPush *push) {
    if (m < 1 || m > 8 || in_f % 2048 || a.gran != 256 || !a.sums16) return cudaErrorInvalidValue;
    if (m == 1) return launch_m6<1>(w, a, y, m, in_f, out_f, dev, status, st, push);
    if (m == 2) return launch_m6<2>(w, a, y, m, in_f, out_f, dev, status, st, push);
    if (m <= 4) return launch_m6<4>(w, a, y, m, in_f, out_f, dev, status, st, push);
    return launch_m6<8>(w, a, y, m, in_f, out_f, dev, status, st, push);
}

}  // namespace infr
