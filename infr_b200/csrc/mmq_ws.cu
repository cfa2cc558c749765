// Prefill MMQ, warp-specialised: C[m, out_f] = Q8(x)[m, in_f] * Q4_K(W)^T on tcgen05.mma.
//
// Arithmetic (crates/infr-cpu/src/kernels.rs:151-184, batch form :1458-1509), per 256-element super-block b:
//     sd = sum_s sc_s * sum_i q4 * q8        int32, exact, tensor cores kind::i8
//     C += (d8[tok, b] * d[row, b]) * float(sd)                      per block, f32 FMA
//     C -= sum_b sum_s (dmin[row, b] * m_s) * (d8[tok, b] * bsum_s)  tensor cores kind::tf32, f32 accumulate
// The int32 block sums are the CPU's bit for bit.  The f32 result differs from the CPU's only by the
// order and fusion of f32 roundings (the min term is summed over the whole row in tensor memory instead
// of per block); both tf32 operands are split into exactly representable pieces (dmin * m_s = A1 + A2
// exactly, d8 * bsum_s = B1 + B2 up to 2^-22), so nothing is lost to the 10-bit tf32 mantissa.
//
// As in the bit-identical kernel the 6-bit sub-block scale is split: A_lo = q * (sc & 7), A_hi = q * (sc >> 3),
// sd = D_lo + 8 * D_hi.
//
// Roles in a CTA (one 128-row x 64-token tile at a time, persistent over tiles):
//   warps 0-3 / 4-7  unpack groups 0 / 1: thread = weight row; group g turns sub-block pairs g, g+2 of each
//                    block into int8 operand planes in its own 16 KB buffer (group 0 also the tf32 min planes)
//   warps 8-15       epilogue: warp = (tensor-memory lane quarter, 32-column half); folds each block's
//                    int32 sums into 32 running f32 sums per thread
//   warp 16          TMA producer (raw weights, activation codes, per-token records), four stages
//   warp 17          MMA issuer: 16 kind::i8 + 3 kind::tf32 instructions per block
// All hand-offs are mbarriers; tensor memory holds two {D_lo, D_hi} buffers and two min accumulators
// (by tile parity).  Every wait is bounded: on expiry the role raises a CTA flag and a status word,
// every role leaves its loop, in-flight copies are drained and the tensor memory is freed.
#include <cuda.h>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kTM = 128, kTN = 64;
constexpr int kStages = 4;
constexpr int kRing = 8;  // depth of the d / d8 rings read by the epilogue
constexpr int kRawBytes = kTM * 144, kCodeBytes = 16 * kTN * 16, kRecChunks = 5, kRecBytes = kRecChunks * kTN * 16;
constexpr int kStageBytes = kRawBytes + kCodeBytes + kRecBytes;
constexpr int kABuf = 2 * 4 * kTM * 16;  // {lo, hi} x 4 planes (two sub-blocks) x 128 rows x 16 B
constexpr int kMinBytes = 4 * kTM * 16;  // A1 planes [2], A2 planes [2]
constexpr int kSmem = kStages * kStageBytes + 2 * kABuf + kMinBytes + kRing * (kTM + kTN) * 4 + 1024;
constexpr int kThreadsWs = 18 * 32;
constexpr uint32_t kSpin = 1u << 22;

// barrier indices
constexpr int B_FULL = 0, B_EMPTY = B_FULL + kStages, B_AREADY = B_EMPTY + kStages, B_AFREE = B_AREADY + 2,
              B_DONE = B_AFREE + 2, B_ACCFREE = B_DONE + 2, B_COUNT = B_ACCFREE + 2;

__device__ __forceinline__ uint32_t su32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t mk_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void mma_i8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0)
        : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d),
        "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Bounded wait; gives up early when another role has raised the CTA flag.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int *dead) {
    for (uint32_t i = 0; i < kSpin; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
        if ((i & 1023u) == 1023u && *dead) return false;
    }
    return false;
}

__device__ __forceinline__ void tma2(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma3(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

}  // namespace

// Per (token, super-block) record, 80 bytes = five 16-byte chunks: B1[0..3], B1[4..7], B2[0..3], B2[4..7]
// (tf32 pieces of d8 * bsum_s), then {d8, 0, 0, 0}.
__global__ void mmq_ws_prep_kernel(const int32_t *__restrict__ sums, const float *__restrict__ d, int n_rec,
                                   uint32_t *__restrict__ rec) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rec) return;
    const float d8 = d[i];
    uint32_t b1[8], b2[8];
#pragma unroll
    for (int s = 0; s < 8; s++) {
        const float v = __fmul_rn(d8, (float)sums[(size_t)i * 8 + s]);
        const uint32_t hi = __float_as_uint(v) & 0xFFFFE000u;
        const float r = __fsub_rn(v, __uint_as_float(hi));
        b1[s] = hi;
        b2[s] = __float_as_uint(r) & 0xFFFFE000u;
    }
    uint4 *o = reinterpret_cast<uint4 *>(rec + (size_t)i * 20);
    o[0] = make_uint4(b1[0], b1[1], b1[2], b1[3]);
    o[1] = make_uint4(b1[4], b1[5], b1[6], b1[7]);
    o[2] = make_uint4(b2[0], b2[1], b2[2], b2[3]);
    o[3] = make_uint4(b2[4], b2[5], b2[6], b2[7]);
    o[4] = make_uint4(__float_as_uint(d8), 0, 0, 0);
}

namespace {

__device__ __forceinline__ bool wait_plain(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}

__global__ void __launch_bounds__(kThreadsWs, 1)
    mmq_ws_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                  const __grid_constant__ CUtensorMap map_r, float *__restrict__ C, int m, int in_f, int out_f,
                  uint32_t *__restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *stage0 = smem;
    uint8_t *abuf0 = smem + kStages * kStageBytes;
    uint8_t *minbuf = abuf0 + 2 * kABuf;
    float *dwring = reinterpret_cast<float *>(minbuf + kMinBytes);  // [kRing][kTM]
    float *d8ring = dwring + kRing * kTM;                           // [kRing][kTN]
    __shared__ uint64_t bars[B_COUNT + 1];                          // + drain barrier of the MMA issuer
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_dead;
    volatile int *dead = &s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = in_f >> 8;
    const int row_tiles = (out_f + kTM - 1) / kTM, tok_tiles = (m + kTN - 1) / kTN;
    const int n_tiles = row_tiles * tok_tiles;

    if (tid == 0) {
        s_dead = 0;
        for (int i = 0; i < B_COUNT + 1; i++) {
            const int cnt = (i >= B_AREADY && i < B_AREADY + 2) ? 4 : (i >= B_ACCFREE && i < B_ACCFREE + 2) ? 8 : 1;
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(su32(&bars[i])), "r"(cnt));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(su32(&tmem_base_s)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    auto bar = [&](int i) { return su32(&bars[i]); };

    if (warp == 16) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int j = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int rt = t % row_tiles, tt = t / row_tiles;  // consecutive CTAs share a token tile
                for (int b = 0; b < nb; b++, j++) {
                    const int s = j % kStages;
                    if (j >= kStages && !wait_bar(bar(B_EMPTY + s), (uint32_t)((j / kStages - 1) & 1), dead)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = stage0 + (size_t)s * kStageBytes;
                    const uint32_t fb = bar(B_FULL + s);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(kStageBytes) : "memory");
                    tma2(su32(st), &map_w, b * 36, rt * kTM, fb);
                    tma3(su32(st + kRawBytes), &map_q, 0, tt * kTN, b * 16, fb);
                    tma3(su32(st + kRawBytes + kCodeBytes), &map_r, 0, tt * kTN, b * kRecChunks, fb);
                }
            }
            if (!ok) {
                if (!*dead) atomicExch(status, 5u);
                *dead = 1;
            }
            if (*dead) {
                // copies still in flight must land before the CTA's shared memory is released
                for (int k = j > kStages ? j - kStages : 0; k < j; k++)
                    wait_plain(bar(B_FULL + k % kStages), (uint32_t)((k / kStages) & 1), 1u << 16);
            }
        }
    } else if (warp == 17) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_i8 = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
            const uint32_t idesc_tf = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
            const uint64_t a1 = mk_desc(su32(minbuf), kTM * 16, 128), a2 = mk_desc(su32(minbuf + 2 * kTM * 16), kTM * 16, 128);
            int j = 0, tile_i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, tile_i++) {
                const uint32_t tmin = tmem + 256 + (uint32_t)(tile_i & 1) * kTN;
                for (int b = 0; b < nb && ok; b++, j++) {
                    const int s = j & 1, ls = j % kStages;
                    if (!wait_bar(bar(B_FULL + ls), (uint32_t)((j / kStages) & 1), dead)) { ok = false; break; }
                    if (j >= 2 && !wait_bar(bar(B_ACCFREE + s), (uint32_t)(((j >> 1) - 1) & 1), dead)) { ok = false; break; }
                    tc_fence_after();
                    const uint8_t *sB = stage0 + (size_t)ls * kStageBytes + kRawBytes, *sR = sB + kCodeBytes;
                    const uint32_t td = tmem + (uint32_t)s * 2 * kTN;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int g = q & 1, n = 2 * j + (q >> 1);
                        if (!wait_bar(bar(B_AREADY + g), (uint32_t)(n & 1), dead)) { ok = false; break; }
                        tc_fence_after();
                        const uint8_t *ab = abuf0 + (size_t)g * kABuf;
#pragma unroll
                        for (int sl = 0; sl < 2; sl++) {
                            const int sb = 2 * q + sl;
                            const uint64_t db = mk_desc(su32(sB + (size_t)(2 * sb) * kTN * 16), kTN * 16, 128);
                            const uint32_t accum = (q > 0 || sl > 0) ? 1u : 0u;
                            mma_i8(td, mk_desc(su32(ab + (size_t)(2 * sl) * kTM * 16), kTM * 16, 128), db, idesc_i8, accum);
                            mma_i8(td + kTN, mk_desc(su32(ab + kABuf / 2 + (size_t)(2 * sl) * kTM * 16), kTM * 16, 128), db, idesc_i8, accum);
                        }
                        if (q == 0) {
                            const uint64_t b1 = mk_desc(su32(sR), kTN * 16, 128), b2 = mk_desc(su32(sR + 2 * kTN * 16), kTN * 16, 128);
                            mma_tf32(tmin, a1, b1, idesc_tf, b > 0 ? 1u : 0u);
                            mma_tf32(tmin, a2, b1, idesc_tf, 1u);
                            mma_tf32(tmin, a1, b2, idesc_tf, 1u);
                        }
                        mma_commit(bar(B_AFREE + g));
                    }
                    if (!ok) break;
                    mma_commit(bar(B_DONE + s));
                    mma_commit(bar(B_EMPTY + ls));
                }
            }
            if (!ok) {
                if (!*dead) atomicExch(status, 6u);
                *dead = 1;
            }
            // every issued MMA has completed before the tensor memory is freed
            mma_commit(bar(B_COUNT));
            wait_plain(bar(B_COUNT), 0u, 1u << 20);
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ unpack groups
        const int g = warp >> 2, row = (warp & 3) * 32 + lane;
        uint8_t *ab = abuf0 + (size_t)g * kABuf;
        int j = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            for (int b = 0; b < nb && ok; b++, j++) {
                const int ls = j % kStages;
                const uint8_t *st = stage0 + (size_t)ls * kStageBytes;
                if (!wait_bar(bar(B_FULL + ls), (uint32_t)((j / kStages) & 1), dead)) { ok = false; break; }
                const uint8_t *blk = st + (size_t)row * 144;
                const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
                uint32_t sc[2], mn[2];
                sc[0] = hdr.y & 0x3F3F3F3Fu;
                mn[0] = hdr.z & 0x3F3F3F3Fu;
                sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
#pragma unroll
                for (int qq = 0; qq < 2; qq++) {
                    const int p = 2 * qq + g, n = 2 * j + qq;
                    const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 16 + p * 32);
                    const uint4 q1 = *reinterpret_cast<const uint4 *>(blk + 32 + p * 32);
                    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    const uint32_t scp = sc[p >> 1] >> (16 * (p & 1));
                    if (n >= 1 && !wait_bar(bar(B_AFREE + g), (uint32_t)((n - 1) & 1), dead)) { ok = false; break; }
#pragma unroll
                    for (int hl = 0; hl < 2; hl++) {
                        const uint32_t scs = (scp >> (8 * hl)) & 0xFFu;
                        const uint32_t f_lo = scs & 7u, f_hi = scs >> 3;
                        uint32_t lo[8], hi[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const uint32_t nib = (hl ? (w[i] >> 4) : w[i]) & 0x0F0F0F0Fu;
                            lo[i] = nib * f_lo;  // bytes <= 15 * 7: no carry between bytes
                            hi[i] = nib * f_hi;
                        }
                        uint8_t *pl = ab + ((size_t)(2 * hl) * kTM + row) * 16;
                        *reinterpret_cast<uint4 *>(pl) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        *reinterpret_cast<uint4 *>(pl + kTM * 16) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                        *reinterpret_cast<uint4 *>(pl + kABuf / 2) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4 *>(pl + kABuf / 2 + kTM * 16) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                    }
                    if (g == 0 && qq == 0) {
                        // min planes: dmin * m_s = A1 + A2 exactly, both representable in tf32
                        const float dw = h2f(hdr.x), dminw = h2f(hdr.x >> 16);
                        uint32_t p1[8], p2[8];
#pragma unroll
                        for (int s8 = 0; s8 < 8; s8++) {
                            const float v = dminw * (float)((mn[s8 >> 2] >> (8 * (s8 & 3))) & 0xFFu);
                            p1[s8] = __float_as_uint(v) & 0xFFFFE000u;
                            p2[s8] = __float_as_uint(v - __uint_as_float(p1[s8]));
                        }
                        uint8_t *mp = minbuf + (size_t)row * 16;
                        *reinterpret_cast<uint4 *>(mp) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
                        *reinterpret_cast<uint4 *>(mp + kTM * 16) = make_uint4(p1[4], p1[5], p1[6], p1[7]);
                        *reinterpret_cast<uint4 *>(mp + 2 * kTM * 16) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
                        *reinterpret_cast<uint4 *>(mp + 3 * kTM * 16) = make_uint4(p2[4], p2[5], p2[6], p2[7]);
                        dwring[(j % kRing) * kTM + row] = dw;
                        if (row < kTN)
                            d8ring[(j % kRing) * kTN + row] =
                                *reinterpret_cast<const float *>(st + kRawBytes + kCodeBytes + 4 * kTN * 16 + (size_t)row * 16);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) bar_arrive(bar(B_AREADY + g));
                }
            }
        }
        if (!ok) {
            if (!*dead) atomicExch(status, 7u);
            *dead = 1;
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 8..15
        const int quarter = warp & 3, half = (warp - 8) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t tlane = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 32);
        float acc[32];
        int j = 0, tile_i = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, tile_i++) {
#pragma unroll
            for (int i = 0; i < 32; i++) acc[i] = 0.f;
            for (int b = 0; b < nb && ok; b++, j++) {
                const int s = j & 1;
                if (!wait_bar(bar(B_DONE + s), (uint32_t)((j >> 1) & 1), dead)) { ok = false; break; }
                tc_fence_after();
                const float dw = dwring[(j % kRing) * kTM + row];
                const float4 *d8p = reinterpret_cast<const float4 *>(d8ring + (j % kRing) * kTN + half * 32);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t lo[16], hi[16];
                    tld16(tlane + (uint32_t)(s * 2 * kTN + c * 16), lo);
                    tld16(tlane + (uint32_t)(s * 2 * kTN + kTN + c * 16), hi);
                    tld_wait();
                    if (c == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) bar_arrive(bar(B_ACCFREE + s));
                    }
#pragma unroll
                    for (int i4 = 0; i4 < 4; i4++) {
                        const float4 dd = d8p[c * 4 + i4];
                        const float ds[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const int i = i4 * 4 + k;
                            const int sd = (int)lo[i] + 8 * (int)hi[i];
                            acc[c * 16 + i] = fmaf(ds[k] * dw, (float)sd, acc[c * 16 + i]);
                        }
                    }
                }
            }
            if (!ok) break;
            // tile end: subtract the min term and store
            const int rt = t % row_tiles, tt = t / row_tiles;
            const int grow = rt * kTM + row;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t mv[16];
                tld16(tlane + (uint32_t)(256 + (tile_i & 1) * kTN + c * 16), mv);
                tld_wait();
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int tok = tt * kTN + half * 32 + c * 16 + i;
                    if (grow < out_f && tok < m) C[(size_t)tok * out_f + grow] = acc[c * 16 + i] - __uint_as_float(mv[i]);
                }
            }
            tc_fence_before();
        }
        if (!ok) {
            if (!*dead) atomicExch(status, 4u);
            *dead = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
}

typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                             const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

}  // namespace

size_t mmq_ws_record_bytes(int m, int in_f) { return (size_t)m * (in_f / 256) * 80; }

cudaError_t launch_mmq_ws_q4k(const uint8_t *w, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                              const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (m < 1 || in_f % 256 || out_f < 1) return cudaErrorInvalidValue;
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const int nb = in_f / 256;
    const int n_rec = m * nb;
    mmq_ws_prep_kernel<<<(n_rec + 255) / 256, 256, 0, st>>>(a.sums, a.d, n_rec, static_cast<uint32_t *>(records));
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
        const cuuint64_t gdim[3] = {16, (cuuint64_t)m, (cuuint64_t)nb * kRecChunks};
        const cuuint64_t gstr[2] = {(cuuint64_t)nb * kRecChunks * 16, 16};
        const cuuint32_t box[3] = {16, (cuuint32_t)kTN, (cuuint32_t)kRecChunks};
        if (enc(&map_r, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, records, gdim, gstr, box, one3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaFuncSetAttribute(mmq_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return e;
    const int n_tiles = ((out_f + kTM - 1) / kTM) * ((m + kTN - 1) / kTN);
    const int grid = n_tiles < dev.sm_count ? n_tiles : dev.sm_count;
    mmq_ws_kernel<<<grid, kThreadsWs, kSmem, st>>>(map_w, map_q, map_r, c, m, in_f, out_f, status);
    return cudaGetLastError();
}

}  // namespace infr
