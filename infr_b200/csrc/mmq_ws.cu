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
// Roles in a CTA (one 128-row x 64-token tile at a time, persistent over tiles; job = one super-block of a tile):
//   warps 0-7    unpack: thread = (weight row, half of the block); reads its 80 bytes of the Q4_K block straight
//                from global memory one job ahead and writes the int8 operand planes of the whole block into one
//                of two 64 KB buffers (the first four warps also the tf32 min planes and the row scale d)
//   warps 8-15   epilogue: warp = (tensor-memory lane quarter, 32-column half); folds each job's int32 sums
//                into 32 running f32 sums per thread
//   warp 16      TMA producer of the activation planes (codes and tf32 block-sum pieces), three stages
//   warps 17, 18 MMA issuers: issuer i runs the jobs j = i (mod 2) on operand buffer i and accumulator i,
//                16 kind::i8 + 3 kind::tf32 instructions per job and ONE commit
// A job's completion barrier (that one commit) releases its operand buffer, its activation stage and its
// accumulator to the epilogue at once; a single issuer thread doing one barrier operation per quarter block
// left the tensor pipe idle three quarters of the time.
// Every wait is bounded: on expiry the role raises a CTA flag and a status word, every role leaves its
// loop, in-flight copies are drained and the tensor memory is freed.
#include <cuda.h>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kTM = 128, kTN = 64;
constexpr int kStages = 3;                    // activation stages
constexpr int kPlanes = 20;                   // activation planes per super-block: 16 code planes + B1[2] + B2[2]
constexpr int kStageBytes = kPlanes * kTN * 16;
constexpr int kABuf = 2 * 16 * kTM * 16;      // {lo, hi} x 16 planes x 128 rows x 16 B: one whole super-block
constexpr int kMinBytes = 4 * kTM * 16;       // A1 planes [2], A2 planes [2]
constexpr int kRing = 4;                      // depth of the row-scale ring read by the epilogue
constexpr int kSmem = kStages * kStageBytes + 2 * (kABuf + kMinBytes) + kRing * kTM * 4;
constexpr int kThreadsWs = 19 * 32;
constexpr uint32_t kSpin = 1u << 22;

// barrier indices: FULL[stage] (TMA bytes), AREADY[buffer] (8 unpack warps), DONE[j % 4] (the job's commit),
// ACCFREE[accumulator] (8 epilogue warps), DRAIN[issuer]
constexpr int B_FULL = 0, B_AREADY = B_FULL + kStages, B_DONE = B_AREADY + 2, B_ACCFREE = B_DONE + 4, B_DRAIN = B_ACCFREE + 2,
              B_COUNT = B_DRAIN + 2;

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

// Warp-collective form: lane 0 polls, the result is broadcast (the shuffle also orders memory in the warp).
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, volatile int *dead) {
    int ok = 0;
    if ((threadIdx.x & 31) == 0) ok = wait_bar(bar, parity, dead) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void tma2(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
}  // namespace


// Re-lays the quantised activations for the kernel.  Output: for every super-block b, 20 planes of
// [m tokens][16 bytes]: planes 0..15 = the int8 codes of K chunk k/16, planes 16..19 = B1[0..3], B1[4..7],
// B2[0..3], B2[4..7] (tf32 pieces of d8 * bsum_s); a 64-token tile of one block is then 20 runs of 1 KB,
// which the copy engine moves at full rate (16-byte runs do not).  Behind the planes: d8 transposed to
// [nb][m_pad] f32 for the epilogue's broadcast loads.
__global__ void mmq_ws_prep_kernel(const int8_t *__restrict__ qs, const int32_t *__restrict__ sums, const float *__restrict__ d,
                                   int m, int m_pad, int nb, uint4 *__restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // token fastest: a warp writes 512 contiguous bytes per plane
    if (i >= m * nb) return;
    const int tok = i % m, b = i / m;
    const size_t rec = (size_t)tok * nb + b;
    uint4 *o = out + (size_t)b * kPlanes * m + tok;
    const uint4 *src = reinterpret_cast<const uint4 *>(qs + rec * 256);
#pragma unroll
    for (int k = 0; k < 16; k++) o[(size_t)k * m] = src[k];
    const float d8 = d[rec];
    uint32_t b1[8], b2[8];
#pragma unroll
    for (int s = 0; s < 8; s++) {
        const float v = __fmul_rn(d8, (float)sums[rec * 8 + s]);
        const uint32_t hi = __float_as_uint(v) & 0xFFFFE000u;
        const float r = __fsub_rn(v, __uint_as_float(hi));
        b1[s] = hi;
        b2[s] = __float_as_uint(r) & 0xFFFFE000u;
    }
    o[(size_t)16 * m] = make_uint4(b1[0], b1[1], b1[2], b1[3]);
    o[(size_t)17 * m] = make_uint4(b1[4], b1[5], b1[6], b1[7]);
    o[(size_t)18 * m] = make_uint4(b2[0], b2[1], b2[2], b2[3]);
    o[(size_t)19 * m] = make_uint4(b2[4], b2[5], b2[6], b2[7]);
    float *d8t = reinterpret_cast<float *>(out + (size_t)nb * kPlanes * m);
    d8t[(size_t)b * m_pad + tok] = d8;
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
__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(kThreadsWs, 1)
    mmq_ws_kernel(const __grid_constant__ CUtensorMap map_q, const uint8_t *__restrict__ W, const float *__restrict__ d8t,
                  float *__restrict__ C, int m, int m_pad, int in_f, int out_f, uint32_t *__restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *stage0 = smem;                              // [kStages][kStageBytes]
    uint8_t *abuf0 = smem + kStages * kStageBytes;       // [2][kABuf]
    uint8_t *minbuf0 = abuf0 + 2 * kABuf;                // [2][kMinBytes]
    float *dwring = reinterpret_cast<float *>(minbuf0 + 2 * kMinBytes);  // [kRing][kTM]
    __shared__ uint64_t bars[B_COUNT];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_dead;
    volatile int *dead = &s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = in_f >> 8;
    const int row_tiles = (out_f + kTM - 1) / kTM, tok_tiles = (m + kTN - 1) / kTN;
    const int n_tiles = row_tiles * tok_tiles;

    if (tid == 0) {
        s_dead = 0;
        for (int i = 0; i < B_COUNT; i++) {
            const int cnt = (i >= B_AREADY && i < B_AREADY + 2) ? 8 : (i >= B_ACCFREE && i < B_ACCFREE + 2) ? 8 : 1;
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
    // "job j is complete" = its issuer's commit has arrived
    auto wait_done = [&](int j) { return wait_bar(bar(B_DONE + (j & 3)), (uint32_t)((j >> 2) & 1), dead); };

    if (warp == 16) {
        // ------------------------------------------------------------------ TMA producer (activation planes)
        if (lane == 0) {
            int j = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int tt = t / row_tiles;  // consecutive CTAs share a token tile
                for (int b = 0; b < nb; b++, j++) {
                    const int s = j % kStages;
                    if (j >= kStages && !wait_done(j - kStages)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fb = bar(B_FULL + s);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(kStageBytes) : "memory");
                    tma2(su32(stage0 + (size_t)s * kStageBytes), &map_q, tt * kTN * 4, b * kPlanes, fb);
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
    } else if (warp >= 17) {
        // ------------------------------------------------------------------ MMA issuers
        const int me = warp - 17;
        if (lane == 0) {
            const uint32_t idesc_i8 = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
            const uint32_t idesc_tf = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
            const uint8_t *ab = abuf0 + (size_t)me * kABuf, *mb = minbuf0 + (size_t)me * kMinBytes;
            const uint64_t a1 = mk_desc(su32(mb), kTM * 16, 128), a2 = mk_desc(su32(mb + 2 * kTM * 16), kTM * 16, 128);
            const uint64_t alo = mk_desc(su32(ab), kTM * 16, 128), ahi = mk_desc(su32(ab + kABuf / 2), kTM * 16, 128);
            const uint32_t td = tmem + (uint32_t)me * 2 * kTN;
            int j = 0, tile_i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, tile_i++) {
                const uint32_t tmin = tmem + 256 + (uint32_t)(tile_i & 1) * 2 * kTN + (uint32_t)me * kTN;
                bool first = true;  // this issuer's first job of the tile starts its min accumulator
                for (int b = 0; b < nb; b++, j++) {
                    if ((j & 1) != me) continue;
                    const int ls = j % kStages;
                    if (!wait_bar(bar(B_FULL + ls), (uint32_t)((j / kStages) & 1), dead) ||
                        !wait_bar(bar(B_AREADY + me), (uint32_t)((j >> 1) & 1), dead) ||
                        (j >= 2 && !wait_bar(bar(B_ACCFREE + me), (uint32_t)(((j >> 1) - 1) & 1), dead))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sB = su32(stage0 + (size_t)ls * kStageBytes);
                    const uint64_t db0 = mk_desc(sB, kTN * 16, 128);
#pragma unroll
                    for (int sb = 0; sb < 8; sb++) {
                        // sub-block sb = planes 2sb, 2sb+1: the descriptor start address field counts 16-byte units
                        const uint64_t db = db0 + (uint64_t)(sb * 2 * kTN);
                        mma_i8(td, alo + (uint64_t)(sb * 2 * kTM), db, idesc_i8, sb > 0 ? 1u : 0u);
                        mma_i8(td + kTN, ahi + (uint64_t)(sb * 2 * kTM), db, idesc_i8, sb > 0 ? 1u : 0u);
                    }
                    const uint64_t b1 = db0 + (uint64_t)(16 * kTN), b2 = db0 + (uint64_t)(18 * kTN);
                    mma_tf32(tmin, a1, b1, idesc_tf, first ? 0u : 1u);
                    mma_tf32(tmin, a2, b1, idesc_tf, 1u);
                    mma_tf32(tmin, a1, b2, idesc_tf, 1u);
                    first = false;
                    mma_commit(bar(B_DONE + (j & 3)));
                }
            }
            if (!ok) {
                if (!*dead) atomicExch(status, 6u);
                *dead = 1;
            }
            // every issued MMA has completed before the tensor memory is freed
            mma_commit(bar(B_DRAIN + me));
            wait_plain(bar(B_DRAIN + me), 0u, 1u << 20);
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ unpack warps
        const int row = tid & 127, h = tid >> 7;
        // the thread's 80 bytes of a job's Q4_K block: header + the 64 nibble bytes of sub-blocks 4h..4h+3
        uint4 nh = make_uint4(0, 0, 0, 0), nq[4] = {nh, nh, nh, nh};
        auto fetch = [&](int t, int b) {
            const int grow = (t % row_tiles) * kTM + row;
            if (grow < out_f) {
                const uint8_t *p = W + ((size_t)grow * nb + b) * 144;
                nh = ldg_stream(p);
#pragma unroll
                for (int k = 0; k < 4; k++) nq[k] = ldg_stream(p + 16 + 64 * h + 16 * k);
            } else {
                nh = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int k = 0; k < 4; k++) nq[k] = nh;
            }
        };
        int j = 0;
        bool ok = true;
        if ((int)blockIdx.x < n_tiles) fetch(blockIdx.x, 0);
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            for (int b = 0; b < nb; b++, j++) {
                const uint4 hdr = nh;
                const uint32_t w[16] = {nq[0].x, nq[0].y, nq[0].z, nq[0].w, nq[1].x, nq[1].y, nq[1].z, nq[1].w,
                                        nq[2].x, nq[2].y, nq[2].z, nq[2].w, nq[3].x, nq[3].y, nq[3].z, nq[3].w};
                // next job's bytes are in flight while this one is unpacked
                if (b + 1 < nb) fetch(t, b + 1);
                else if (t + (int)gridDim.x < n_tiles) fetch(t + gridDim.x, 0);
                const int bi = j & 1;
                if (j >= 2 && !wait_bar_warp(bar(B_DONE + ((j - 2) & 3)), (uint32_t)(((j - 2) >> 2) & 1), dead)) {
                    ok = false;
                    break;
                }
                uint8_t *ab = abuf0 + (size_t)bi * kABuf;
                uint32_t sc[2], mn[2];
                sc[0] = hdr.y & 0x3F3F3F3Fu;
                mn[0] = hdr.z & 0x3F3F3F3Fu;
                sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                const uint32_t sc4 = sc[h];  // scales of sub-blocks 4h..4h+3
#pragma unroll
                for (int pp = 0; pp < 2; pp++) {
#pragma unroll
                    for (int hl = 0; hl < 2; hl++) {
                        const int sbl = 2 * pp + hl;  // sub-block 4h + sbl
                        const uint32_t scs = (sc4 >> (8 * sbl)) & 0xFFu;
                        const uint32_t f_lo = scs & 7u, f_hi = scs >> 3;
                        uint32_t lo[8], hi[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const uint32_t nib = (hl ? (w[8 * pp + i] >> 4) : w[8 * pp + i]) & 0x0F0F0F0Fu;
                            lo[i] = nib * f_lo;  // bytes <= 15 * 7: no carry between bytes
                            hi[i] = nib * f_hi;
                        }
                        uint8_t *pl = ab + ((size_t)(2 * (4 * h + sbl)) * kTM + row) * 16;
                        *reinterpret_cast<uint4 *>(pl) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        *reinterpret_cast<uint4 *>(pl + kTM * 16) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                        *reinterpret_cast<uint4 *>(pl + kABuf / 2) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4 *>(pl + kABuf / 2 + kTM * 16) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                    }
                }
                if (h == 0) {
                    // min planes: dmin * m_s = A1 + A2 exactly, both representable in tf32
                    const float dw = h2f(hdr.x), dminw = h2f(hdr.x >> 16);
                    uint32_t p1[8], p2[8];
#pragma unroll
                    for (int s8 = 0; s8 < 8; s8++) {
                        const float v = dminw * (float)((mn[s8 >> 2] >> (8 * (s8 & 3))) & 0xFFu);
                        p1[s8] = __float_as_uint(v) & 0xFFFFE000u;
                        p2[s8] = __float_as_uint(v - __uint_as_float(p1[s8]));
                    }
                    uint8_t *mp = minbuf0 + (size_t)bi * kMinBytes + (size_t)row * 16;
                    *reinterpret_cast<uint4 *>(mp) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
                    *reinterpret_cast<uint4 *>(mp + kTM * 16) = make_uint4(p1[4], p1[5], p1[6], p1[7]);
                    *reinterpret_cast<uint4 *>(mp + 2 * kTM * 16) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
                    *reinterpret_cast<uint4 *>(mp + 3 * kTM * 16) = make_uint4(p2[4], p2[5], p2[6], p2[7]);
                    dwring[(j % kRing) * kTM + row] = dw;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) bar_arrive(bar(B_AREADY + bi));
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
            const int rt = t % row_tiles, tt = t / row_tiles;
            const float4 *d8p = reinterpret_cast<const float4 *>(d8t + (size_t)tt * kTN + half * 32);
            const int j_tile = j;
#pragma unroll
            for (int i = 0; i < 32; i++) acc[i] = 0.f;
            for (int b = 0; b < nb; b++, j++) {
                const int s = j & 1;
                float4 dd[4];
#pragma unroll
                for (int i4 = 0; i4 < 4; i4++) dd[i4] = __ldg(d8p + (size_t)b * (m_pad / 4) + i4);
                if (!wait_bar_warp(bar(B_DONE + (j & 3)), (uint32_t)((j >> 2) & 1), dead)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const float dw = dwring[(j % kRing) * kTM + row];
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t lo[16], hi[16];
                    tld16(tlane + (uint32_t)(s * 2 * kTN + c * 16), lo);
                    tld16(tlane + (uint32_t)(s * 2 * kTN + kTN + c * 16), hi);
                    if (c == 1) {
#pragma unroll
                        for (int i4 = 0; i4 < 4; i4++) dd[i4] = __ldg(d8p + (size_t)b * (m_pad / 4) + 4 + i4);
                    }
                    tld_wait();
                    // the last job of a tile keeps its accumulator until the tile's min sums are read
                    if (c == 1 && b + 1 < nb) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) bar_arrive(bar(B_ACCFREE + s));
                    }
#pragma unroll
                    for (int i4 = 0; i4 < 4; i4++) {
                        const float ds[4] = {dd[i4].x, dd[i4].y, dd[i4].z, dd[i4].w};
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
            // tile end: subtract the min sums of the issuers that ran jobs of this tile, then store
            const int grow = rt * kTM + row;
            const bool use0 = nb >= 2 || (j_tile & 1) == 0, use1 = nb >= 2 || (j_tile & 1) == 1;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t m0[16], m1[16];
                const uint32_t tm = tlane + (uint32_t)(256 + (tile_i & 1) * 2 * kTN + c * 16);
                tld16(tm, m0);
                tld16(tm + kTN, m1);
                tld_wait();
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int tok = tt * kTN + half * 32 + c * 16 + i;
                    float v = acc[c * 16 + i];
                    if (use0) v -= __uint_as_float(m0[i]);
                    if (use1) v -= __uint_as_float(m1[i]);
                    if (grow < out_f && tok < m) C[(size_t)tok * out_f + grow] = v;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) bar_arrive(bar(B_ACCFREE + ((j - 1) & 1)));
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

size_t mmq_ws_record_bytes(int m, int in_f) {
    const size_t nb = in_f / 256, m_pad = ((size_t)m + kTN - 1) / kTN * kTN;
    return nb * kPlanes * (size_t)m * 16 + nb * m_pad * 4;
}

cudaError_t launch_mmq_ws_q4k(const uint8_t *w, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                              const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (m < 1 || in_f % 256 || out_f < 1) return cudaErrorInvalidValue;
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const int nb = in_f / 256, m_pad = (m + kTN - 1) / kTN * kTN;
    const int n_rec = m * nb;
    mmq_ws_prep_kernel<<<(n_rec + 255) / 256, 256, 0, st>>>(a.qs, a.sums, a.d, m, m_pad, nb, static_cast<uint4 *>(records));
    CUtensorMap map_q;
    const cuuint32_t one2[2] = {1, 1};
    {
        // activation planes [nb * 20][m][16 B] as rows of m * 4 words: a tile is 20 rows of 256 words
        const cuuint64_t gdim[2] = {(cuuint64_t)m * 4, (cuuint64_t)nb * kPlanes};
        const cuuint64_t gstr[1] = {(cuuint64_t)m * 16};
        const cuuint32_t box[2] = {(cuuint32_t)kTN * 4, (cuuint32_t)kPlanes};
        if (enc(&map_q, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, records, gdim, gstr, box, one2, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const float *d8t = reinterpret_cast<const float *>(static_cast<const uint8_t *>(records) + (size_t)nb * kPlanes * m * 16);
    cudaError_t e = cudaFuncSetAttribute(mmq_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return e;
    const int n_tiles = ((out_f + kTM - 1) / kTM) * ((m + kTN - 1) / kTN);
    const int grid = n_tiles < dev.sm_count ? n_tiles : dev.sm_count;
    mmq_ws_kernel<<<grid, kThreadsWs, kSmem, st>>>(map_q, w, d8t, c, m, m_pad, in_f, out_f, status);
    return cudaGetLastError();
}

}  // namespace infr
