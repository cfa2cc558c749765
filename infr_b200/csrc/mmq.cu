// Prefill MMQ: C[m, out_f] = Q8(x)[m, in_f] * Q4_K(W)^T on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), with the arithmetic of the production
// infr-cpu path (crates/infr-cpu/src/kernels.rs:151-184, batch form :1458-1509):
//     per 256-element super-block b:  sd = sum_s sc_s * sum_i q4 * q8,   sm = sum_s m_s * bsum_s
//     C += d8[tok, b] * (d[row, b] * float(sd) - dmin[row, b] * float(sm))      blocks in ascending order
// The f32 expression is evaluated per (row, token, block) with separately rounded multiply / subtract /
// add in block order, exactly as the CPU does, so the result is bit-identical to it.
//
// The 6-bit sub-block scale cannot ride inside an int8 operand (sc * q reaches 945) and rescaling the
// accumulator every 32 K would make the epilogue the bottleneck, so the scale is split in two 3-bit
// halves: A_lo = q * (sc & 7) and A_hi = q * (sc >> 3) are both <= 105, two MMAs per sub-block
// accumulate the whole super-block in tensor memory and sd = D_lo + 8 * D_hi is exact.  The min term
// is two more MMAs: A = the eight m_s bytes, B = bsum split as 64 * h + l.
//
// Operand layout in shared memory (no swizzle, K-major): 16-byte planes [k/16][row][16 B]; the
// descriptor of sub-block s starts at plane 2s with leading-dimension offset = one plane and stride
// offset = 128 B (8 rows).  One CTA owns a 128-row x 64-token tile: thread r unpacks weight row r,
// reads tensor-memory lane r in the epilogue and keeps the 64 running f32 sums of that row.
//
// Every mbarrier wait is bounded; on expiry the CTA records a status word and leaves (after freeing
// its tensor memory).
#include <cuda.h>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kTM = 128;  // weight rows per tile (MMA M)
constexpr int kTN = 64;   // tokens per tile (MMA N)
constexpr int kMathWarps = 16;                 // 4 per tensor-memory lane quarter
constexpr int kMathThreads = kMathWarps * 32;  // thread = (weight row, 16-column group)
constexpr int kCG = kTN / 4;                   // columns per thread in the epilogue
constexpr uint32_t kMmqSpin = 1u << 22;

__device__ __forceinline__ uint32_t sm_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

// Per (token, super-block) record the kernel fetches by TMA next to the int8 codes: 32 bytes =
// [l_0..l_7][h_0..h_7] (bsum_s = 64 * h_s + l_s) then the f32 scale d8 and 12 bytes of padding.
__global__ void mmq_prep_kernel(const int32_t *__restrict__ sums, const float *__restrict__ d, int n_rec,
                                uint32_t *__restrict__ rec) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rec) return;
    uint32_t l[2] = {0, 0}, h[2] = {0, 0};
#pragma unroll
    for (int s = 0; s < 8; s++) {
        const int bs = sums[(size_t)i * 8 + s];
        l[s >> 2] |= (uint32_t)(bs & 63) << (8 * (s & 3));
        h[s >> 2] |= (uint32_t)((bs >> 6) & 0xFF) << (8 * (s & 3));
    }
    uint4 *o = reinterpret_cast<uint4 *>(rec + (size_t)i * 8);
    o[0] = make_uint4(l[0], l[1], h[0], h[1]);
    o[1] = make_uint4(__float_as_uint(d[i]), 0, 0, 0);
}

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (uint32_t i = 0; i < kMmqSpin && !ok; i++)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

// Shared-memory plan (bytes): four load stages {raw weights 128 x 144, code planes [16][64][16], record
// planes [2][64][16]}, one operand buffer {A_lo [16][128][16], A_hi [16][128][16], A_ml [128][16],
// A_mh [128][16]}, one zero plane [128][16], three d8 rows [64] f32.  Tensor memory is double-buffered.
constexpr int kRawBytes = kTM * 144, kCodeBytes = 16 * kTN * 16, kRecBytes = 2 * kTN * 16;
constexpr int kStageBytes = kRawBytes + kCodeBytes + kRecBytes;
constexpr int kABufBytes = 2 * 16 * kTM * 16 + 2 * kTM * 16;
constexpr int kStages = 4;  // TMA latency is several block-times: keep four blocks in flight
constexpr int kSmemMmq = kStages * kStageBytes + kABufBytes + kTM * 16 + 3 * kTN * 4 + 256;

// Warps 0..15 are math warps: warp w works on tensor-memory lanes / weight rows 32*(w&3) .. +31 and on
// sub-block pair / column group (w>>2): it unpacks that pair of its rows, and in the epilogue folds 16
// token columns.  Warp 16 is the TMA producer.  Persistent CTA: it walks tiles blockIdx.x, +gridDim.x, ...
__global__ void __launch_bounds__(kMathThreads + 32, 1)
    mmq_q4k_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_r, float *__restrict__ C, int m, int in_f, int out_f,
                   uint32_t *__restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *stage0 = smem;
    uint8_t *abuf0 = smem + kStages * kStageBytes;
    uint8_t *zero_plane = abuf0 + kABufBytes;
    float *d8buf = reinterpret_cast<float *>(zero_plane + kTM * 16);  // [3][64]
    __shared__ uint64_t bars[2 * kStages + 2];  // full[kStages], mma_done[2], empty[kStages]
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int nb = in_f >> 8;
    const int row_tiles = (out_f + kTM - 1) / kTM, tok_tiles = (m + kTN - 1) / kTN;
    const int n_tiles = row_tiles * tok_tiles;
    int my_tiles = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) my_tiles++;
    (void)my_tiles;

    if (tid == 0) {
        s_dead = 0;
        for (int i = 0; i < 2 * kStages + 2; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm_u32(&bars[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_u32(&tmem_base_s)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    if (tid < kTM) *reinterpret_cast<uint4 *>(zero_plane + (size_t)tid * 16) = make_uint4(0, 0, 0, 0);
    const int row_in_tile = (warp & 3) * 32 + (tid & 31), cg = warp >> 2;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;

    if (warp == kMathWarps) {
        // ------------------------------------------------------------------ TMA producer
        if ((tid & 31) == 0) {
            int j = 0;
            for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                const int rt = t % row_tiles, tt = t / row_tiles;  // consecutive CTAs share a token tile
                for (int b = 0; b < nb; b++, j++) {
                    // stage j % kStages was last used by job j - kStages; its codes are free once that job's MMAs are done
                    // (a second commit of that job arrives on empty[stage]; a barrier per stage is never more than
                    // one phase ahead of this wait)
                    const int s = j % kStages;
                    if (j >= kStages && !mbar_wait_bounded(sm_u32(&bars[kStages + 2 + s]), (uint32_t)((j / kStages - 1) & 1))) {
                        atomicExch(status, 5u);
                        *(volatile int *)&s_dead = 1;
                        return;
                    }
                    if (*(volatile int *)&s_dead) return;
                    uint8_t *st = stage0 + (size_t)s * kStageBytes;
                    const uint32_t bar = sm_u32(&bars[s]);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kStageBytes) : "memory");
                    tma_2d(sm_u32(st), &map_w, b * 36, rt * kTM, bar);
                    tma_3d(sm_u32(st + kRawBytes), &map_q, 0, tt * kTN, b * 16, bar);
                    tma_3d(sm_u32(st + kRawBytes + kCodeBytes), &map_r, 0, tt * kTN, b * 2, bar);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- math warps
    const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(cg * kCG);
    float acc[kCG];
    float dw_prev = 0.f, dmin_prev = 0.f;
    bool dead = false;

    // epilogue of job j: fold the block's tensor-memory sums into the running f32 sums
    auto epilogue = [&](int j, float dw, float dminw) {
        const int s = j & 1;
        if (!mbar_wait_bounded(sm_u32(&bars[kStages + s]), (uint32_t)((j >> 1) & 1))) {
            *(volatile int *)&s_dead = 1;
            return;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float *d8 = d8buf + (j % 3) * kTN + cg * kCG;
        const uint32_t tb = lane_addr + (uint32_t)s * 256;
        int vlo[16], vhi[16], vml[16], vmh[16];
        tmem_ld16(tb, vlo);
        tmem_ld16(tb + kTN, vhi);
        tmem_ld16(tb + 2 * kTN, vml);
        tmem_ld16(tb + 3 * kTN, vmh);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < kCG; i++) {
            const int sd = vlo[i] + 8 * vhi[i];
            const int sm = vml[i] + 64 * vmh[i];
            const float t = __fsub_rn(__fmul_rn(dw, (float)sd), __fmul_rn(dminw, (float)sm));
            acc[i] = __fadd_rn(acc[i], __fmul_rn(d8[i], t));
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };
    auto store_tile = [&](int t) {
        const int rt = t % row_tiles, tt = t / row_tiles;
        const int row = rt * kTM + row_in_tile;
        if (row < out_f) {
#pragma unroll
            for (int i = 0; i < kCG; i++)
                if (tt * kTN + cg * kCG + i < m) C[(size_t)(tt * kTN + cg * kCG + i) * out_f + row] = acc[i];
        }
    };

    int j = 0, prev_tile = -1;
    for (int t = blockIdx.x; t < n_tiles && !dead; t += gridDim.x) {
        for (int b = 0; b < nb && !dead; b++, j++) {
            const int s = j & 1, ls = j % kStages;
            uint8_t *st = stage0 + (size_t)ls * kStageBytes;
            uint8_t *ab = abuf0;
            // ---- the previous block: its MMAs must be done before the operand buffer is rewritten ----
            if (j > 0) {
                epilogue(j - 1, dw_prev, dmin_prev);
                if (b == 0 && !*(volatile int *)&s_dead) store_tile(prev_tile);
            }
            if (b == 0) {
#pragma unroll
                for (int i = 0; i < kCG; i++) acc[i] = 0.f;
            }
            uint8_t *sA_lo = ab, *sA_hi = ab + 16 * kTM * 16, *sA_ml = ab + 2 * 16 * kTM * 16, *sA_mh = sA_ml + kTM * 16;
            // A thread whose bounded wait expires raises the CTA-wide flag but still walks to the next
            // barrier, where every thread sees the flag and leaves together.
            if (!mbar_wait_bounded(sm_u32(&bars[ls]), (uint32_t)((j / kStages) & 1))) *(volatile int *)&s_dead = 1;
            // ---- unpack weight row `tid` of this block from the raw tile ----
            const uint8_t *blk = st + (size_t)row_in_tile * 144;
            const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
            const float dw = h2f(hdr.x), dminw = h2f(hdr.x >> 16);
            {
                uint32_t sc[2], mn[2];
                sc[0] = hdr.y & 0x3F3F3F3Fu;
                mn[0] = hdr.z & 0x3F3F3F3Fu;
                sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                if (cg == 0) {
                    *reinterpret_cast<uint4 *>(sA_ml + (size_t)row_in_tile * 16) = make_uint4(mn[0], mn[1], 0, 0);
                    *reinterpret_cast<uint4 *>(sA_mh + (size_t)row_in_tile * 16) = make_uint4(0, 0, mn[0], mn[1]);
                }
                const int p = cg;  // this thread's sub-block pair (2p, 2p+1)
                const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 16 + p * 32);
                const uint4 q1 = *reinterpret_cast<const uint4 *>(blk + 32 + p * 32);
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                const uint32_t scp = sc[p >> 1] >> (16 * (p & 1));
#pragma unroll
                for (int hl = 0; hl < 2; hl++) {
                    const int sb = 2 * p + hl;
                    const uint32_t scs = (scp >> (8 * hl)) & 0xFFu;
                    const uint32_t f_lo = scs & 7u, f_hi = scs >> 3;
                    uint32_t lo[8], hi[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const uint32_t nib = (hl ? (w[i] >> 4) : w[i]) & 0x0F0F0F0Fu;
                        lo[i] = nib * f_lo;  // bytes <= 15 * 7: no carry between bytes
                        hi[i] = nib * f_hi;
                    }
                    // elements 0..15 of sub-block sb -> plane 2*sb, 16..31 -> plane 2*sb + 1
                    *reinterpret_cast<uint4 *>(sA_lo + ((size_t)(2 * sb) * kTM + row_in_tile) * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    *reinterpret_cast<uint4 *>(sA_lo + ((size_t)(2 * sb + 1) * kTM + row_in_tile) * 16) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                    *reinterpret_cast<uint4 *>(sA_hi + ((size_t)(2 * sb) * kTM + row_in_tile) * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(sA_hi + ((size_t)(2 * sb + 1) * kTM + row_in_tile) * 16) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                }
            }
            // d8 of this block's tokens: first word of record plane 1
            if (tid < kTN) d8buf[(j % 3) * kTN + tid] = *reinterpret_cast<const float *>(st + kRawBytes + kCodeBytes + kTN * 16 + (size_t)tid * 16);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, %0;" ::"r"(kMathThreads) : "memory");
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (*(volatile int *)&s_dead) {
                dead = true;
                break;
            }
            if (tid == 0) {
                const uint32_t td = tmem + (uint32_t)s * 256;
                const uint8_t *sB = st + kRawBytes, *sR = sB + kCodeBytes;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const uint64_t db = umma_desc(sm_u32(sB + (size_t)(2 * k) * kTN * 16), kTN * 16, 128);
                    umma_i8(td, umma_desc(sm_u32(sA_lo + (size_t)(2 * k) * kTM * 16), kTM * 16, 128), db, idesc, k > 0);
                    umma_i8(td + kTN, umma_desc(sm_u32(sA_hi + (size_t)(2 * k) * kTM * 16), kTM * 16, 128), db, idesc, k > 0);
                }
                // min term: the A operand's second K half is the zero plane, so record plane 1 (d8) is inert
                const uint64_t dbr = umma_desc(sm_u32(sR), kTN * 16, 128);
                umma_i8(td + 2 * kTN, umma_desc(sm_u32(sA_ml), (uint32_t)(zero_plane - sA_ml), 128), dbr, idesc, 0);
                umma_i8(td + 3 * kTN, umma_desc(sm_u32(sA_mh), (uint32_t)(zero_plane - sA_mh), 128), dbr, idesc, 0);
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sm_u32(&bars[kStages + s])) : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sm_u32(&bars[kStages + 2 + ls])) : "memory");
            }
            dw_prev = dw;
            dmin_prev = dminw;
        }
        prev_tile = t;
    }
    if (!dead && j > 0) epilogue(j - 1, dw_prev, dmin_prev);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"r"(kMathThreads) : "memory");
    if (*(volatile int *)&s_dead) {
        if (tid == 0) atomicExch(status, 4u);
    } else if (j > 0) {
        store_tile(prev_tile);
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn2 encode_tiled2() {
    static EncodeTiledFn2 fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn2>(p);
    }();
    return fn;
}

}  // namespace

size_t mmq_q4k_record_bytes(int m, int in_f) { return (size_t)m * (in_f / 256) * 32; }

cudaError_t launch_mmq_q4k(const uint8_t *w, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                           const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (m < 1 || in_f % 256 || out_f < 1) return cudaErrorInvalidValue;
    EncodeTiledFn2 enc = encode_tiled2();
    if (!enc) return cudaErrorNotSupported;
    const int nb = in_f / 256;
    const int n_rec = m * nb;
    mmq_prep_kernel<<<(n_rec + 255) / 256, 256, 0, st>>>(a.sums, a.d, n_rec, static_cast<uint32_t *>(records));
    CUtensorMap map_w, map_q, map_r;
    const cuuint32_t one3[3] = {1, 1, 1};
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)nb * 36, (cuuint64_t)out_f};
        const cuuint64_t gstr[1] = {(cuuint64_t)nb * 144};
        const cuuint32_t box[2] = {36, (cuuint32_t)kTM};
        if (enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(w), gdim, gstr, box, one3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        // codes [m][in_f] viewed as (16 bytes, token, 16-byte column): the box lands as planes [k/16][token][16]
        const cuuint64_t gdim[3] = {16, (cuuint64_t)m, (cuuint64_t)in_f / 16};
        const cuuint64_t gstr[2] = {(cuuint64_t)in_f, 16};
        const cuuint32_t box[3] = {16, (cuuint32_t)kTN, 16};
        if (enc(&map_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t *>(a.qs), gdim, gstr, box, one3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t gdim[3] = {16, (cuuint64_t)m, (cuuint64_t)nb * 2};
        const cuuint64_t gstr[2] = {(cuuint64_t)nb * 32, 16};
        const cuuint32_t box[3] = {16, (cuuint32_t)kTN, 2};
        if (enc(&map_r, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, records, gdim, gstr, box, one3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaFuncSetAttribute(mmq_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMmq);
    if (e != cudaSuccess) return e;
    const int n_tiles = ((out_f + kTM - 1) / kTM) * ((m + kTN - 1) / kTN);
    const int grid = n_tiles < dev.sm_count ? n_tiles : dev.sm_count;
    mmq_q4k_kernel<<<grid, kMathThreads + 32, kSmemMmq, st>>>(map_w, map_q, map_r, c, m, in_f, out_f, status);
    return cudaGetLastError();
}

}  // namespace infr
