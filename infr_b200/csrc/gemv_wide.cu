// Q4_K / Q6_K batched GEMV for 9..32 activation rows (a decode step over a few dozen sequences): every weight byte
// is fetched and unpacked once and meets all rows, instead of once per 8 rows.
//
// Arithmetic: that of the 8-row kernels (gemv_mma.cu, gemv_mma_q6.cu), i.e. the production infr-cpu dot products
// (crates/infr-cpu/src/kernels.rs:151-184 for Q4_K, :487-526 for Q6_K; the batch form :2318, :2347-2688 computes the
// same sums row by row): exact int32 sums per 256-element super-block on the warp-level int8 matrix unit, then
//     Q4_K  y += d8 * (d * float(sd) - dmin * float(sm))        Q6_K  y += d * d8 * float(isum)
// An unpacked A fragment (16 weight rows x one sub-block) feeds NT instructions, one per group of 8 activation rows,
// so the unpacking (the cost of the 8-row kernels) is paid once for up to 32 rows.
//
// Work split: K is cut into chunks of 8 super-blocks; a CTA (8 warps) owns one chunk and a contiguous range of 16-row
// weight tiles, warp w owns super-block w of the chunk for every tile.  The activations a warp needs are therefore
// the same for all its tiles and live in REGISTERS for the whole kernel (64 code words, the split block sums and the
// row scales per lane, fetched once after the dependency wait with every load in flight together): no shared-memory
// staging, no re-reads.  Weights arrive through warp-private rings filled by tiled TMA (prefetched before the
// dependency wait, evict-first in L2).  The 8 warps' partial sums of a tile meet in shared memory in warp order; with
// more than one K chunk the CTAs write partial results [chunk][row][out_f] that a second kernel adds in chunk order,
// so the result does not depend on timing.
//
// All mbarrier waits are bounded; an expired wait records a status word for the host and the warp stops consuming.
#include <cuda.h>

#include <cstring>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kWRows = 16;       // weight rows per tile
constexpr int kWWarps = 8;       // warps per CTA = super-blocks per K chunk
constexpr int kWSlots = 4;       // ring slots per warp
constexpr int kWPitch = 17;      // floats per token row of a warp's partial tile (16 + 1: distinct banks)
constexpr uint32_t kWSpin = 1u << 22;

__device__ __forceinline__ uint32_t sw32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wide_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWSpin; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void wide_tma(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
                 : "memory");
}
// D = A(16x32, u8) * B(32x8, s8), int32, zero accumulator input
__device__ __forceinline__ void wmma_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// D = A(16x16) * B(16x8), int32, zero accumulator input; A unsigned or signed bytes
__device__ __forceinline__ void wmma_k16_us(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void wmma_k16_ss(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

// ---------------------------------------------------------------------------------------------------------- Q4_K
// Lane (g = lane / 4, t = lane % 4) of the matrix instruction holds weight rows g and g + 8 and feeds K slots
// 4t..4t+3 and 16+4t..16+4t+3; the K index is only a summation index, so the lane takes the 8 nibble bytes
// [8t, 8t+8) of each 32-byte run of qs (elements l = 8t..8t+7 of sub-blocks 2p and 2p+1) and the activation codes
// of the same elements.
struct WideQ4 {
    static constexpr int kSlotBytes = kWRows * 144;
    static constexpr int kBWords = 18;  // per group of 8 rows: 16 code words + the split block sums (low 6 bits, high part)
    // box x coordinate (32-bit words) of super-block b
    __device__ static int tma_x(int b) { return b * 36; }
    // activation operands of token `row` for super-block b
    __device__ static void load_b(uint32_t (&bw)[kBWords], const Q8Dev &a, size_t row, int b, int nb, int in_f, int t, bool valid) {
        if (!valid) {
#pragma unroll
            for (int i = 0; i < kBWords; i++) bw[i] = 0u;
            return;
        }
        const int8_t *base = a.qs + row * (size_t)in_f + (size_t)b * 256 + t * 8;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            const uint2 v = *reinterpret_cast<const uint2 *>(base + s * 32);
            bw[2 * s] = v.x;
            bw[2 * s + 1] = v.y;
        }
        // bsum_s = 64 h + l: lanes t = 0 / 1 carry sub-blocks 0..3 / 4..7 (the other lanes meet zero A operands)
        const int4 sv = *reinterpret_cast<const int4 *>(a.sums + (row * nb + b) * 8 + (t & 1) * 4);
        bw[16] = pack4(sv.x & 63, sv.y & 63, sv.z & 63, sv.w & 63);
        bw[17] = pack4(sv.x >> 6, sv.y >> 6, sv.z >> 6, sv.w >> 6);
    }
    template <int NT>
    __device__ static void block(const uint8_t *sl, int b, int g, int t, const uint32_t (&bw)[NT][kBWords], const float2 (&e)[NT],
                                 float (&accf)[NT][4]) {
        const uint8_t *r0 = sl + (size_t)g * 144, *r1 = r0 + 8 * 144;
        const uint4 h0 = *reinterpret_cast<const uint4 *>(r0), h1 = *reinterpret_cast<const uint4 *>(r1);
        uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
        sc0[0] = h0.y & 0x3F3F3F3Fu, mn0[0] = h0.z & 0x3F3F3F3Fu;
        sc0[1] = (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u), mn0[1] = ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u);
        sc1[0] = h1.y & 0x3F3F3F3Fu, mn1[0] = h1.z & 0x3F3F3F3Fu;
        sc1[1] = (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u), mn1[1] = ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u);
        int sd[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) sd[nt][0] = sd[nt][1] = sd[nt][2] = sd[nt][3] = 0;
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint2 w0 = *reinterpret_cast<const uint2 *>(r0 + 16 + p * 32 + t * 8);
            const uint2 w1 = *reinterpret_cast<const uint2 *>(r1 + 16 + p * 32 + t * 8);
            const uint32_t l0 = w0.x & 0x0F0F0F0Fu, l1 = w1.x & 0x0F0F0F0Fu, l2 = w0.y & 0x0F0F0F0Fu, l3 = w1.y & 0x0F0F0F0Fu;
            const uint32_t u0 = (w0.x >> 4) & 0x0F0F0F0Fu, u1 = (w1.x >> 4) & 0x0F0F0F0Fu, u2 = (w0.y >> 4) & 0x0F0F0F0Fu,
                           u3 = (w1.y >> 4) & 0x0F0F0F0Fu;
            // scales of sub-block 2p (low nibbles) and 2p+1 (high nibbles) for rows g and g+8
            const uint32_t sel = (p & 1) ? 0x4442u : 0x4440u;
            const int sa_lo = (int)__byte_perm(sc0[p >> 1], 0, sel), sa_hi = (int)__byte_perm(sc0[p >> 1], 0, sel + 1);
            const int sb_lo = (int)__byte_perm(sc1[p >> 1], 0, sel), sb_hi = (int)__byte_perm(sc1[p >> 1], 0, sel + 1);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                int dlo[4], dhi[4];
                wmma_k32(dlo, l0, l1, l2, l3, bw[nt][4 * p], bw[nt][4 * p + 1]);
                wmma_k32(dhi, u0, u1, u2, u3, bw[nt][4 * p + 2], bw[nt][4 * p + 3]);
                sd[nt][0] += sa_lo * dlo[0] + sa_hi * dhi[0];
                sd[nt][1] += sa_lo * dlo[1] + sa_hi * dhi[1];
                sd[nt][2] += sb_lo * dlo[2] + sb_hi * dhi[2];
                sd[nt][3] += sb_lo * dlo[3] + sb_hi * dhi[3];
            }
        }
        // min term: K slots 0..7 carry the eight m_s (lanes t = 0, 1), the rest are zero
        const uint32_t am0 = t == 0 ? mn0[0] : (t == 1 ? mn0[1] : 0u), am1 = t == 0 ? mn1[0] : (t == 1 ? mn1[1] : 0u);
        const float d0 = h2f(h0.x), dm0 = h2f(h0.x >> 16), d1 = h2f(h1.x), dm1 = h2f(h1.x >> 16);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            int sml[4], smh[4];
            wmma_k32(sml, am0, am1, 0u, 0u, bw[nt][16], 0u);
            wmma_k32(smh, am0, am1, 0u, 0u, bw[nt][17], 0u);
            accf[nt][0] += e[nt].x * (d0 * (float)sd[nt][0] - dm0 * (float)(sml[0] + 64 * smh[0]));
            accf[nt][1] += e[nt].y * (d0 * (float)sd[nt][1] - dm0 * (float)(sml[1] + 64 * smh[1]));
            accf[nt][2] += e[nt].x * (d1 * (float)sd[nt][2] - dm1 * (float)(sml[2] + 64 * smh[2]));
            accf[nt][3] += e[nt].y * (d1 * (float)sd[nt][3] - dm1 * (float)(sml[3] + 64 * smh[3]));
        }
    }
};

// ---------------------------------------------------------------------------------------------------------- Q6_K
// One m16n8k16 instruction is one 16-element sub-block: the unsigned 6-bit codes go in as they are, the -32 is applied
// through the 16-element activation sums (A = the 16 scales, B = bsum16 split as 64 h + l).  A 210-byte block starts
// at an even address; its TMA box starts at the 16-byte boundary below it and is 224 bytes wide, and the words of odd
// blocks (2 bytes off a word boundary) are assembled with a funnel shift.
struct WideQ6 {
    static constexpr int kPitch = 224;
    static constexpr int kSlotBytes = kWRows * kPitch;
    static constexpr int kBWords = 18;  // 16 code words (one per sub-block) + the split sums
    // box x coordinate (16-bit elements) of block b
    __device__ static int tma_x(int b) { return ((b * 210) & ~15) >> 1; }
    __device__ static void load_b(uint32_t (&bw)[kBWords], const Q8Dev &a, size_t row, int b, int nb, int in_f, int t, bool valid) {
        if (!valid) {
#pragma unroll
            for (int i = 0; i < kBWords; i++) bw[i] = 0u;
            return;
        }
        const int8_t *base = a.qs + row * (size_t)in_f + (size_t)b * 256 + t * 4;
#pragma unroll
        for (int s = 0; s < 16; s++) bw[s] = *reinterpret_cast<const uint32_t *>(base + s * 16);
        // bsum16 of sub-blocks 4t..4t+3
        const int4 sv = *reinterpret_cast<const int4 *>(a.sums16 + (row * nb + b) * 16 + t * 4);
        bw[16] = pack4(sv.x & 63, sv.y & 63, sv.z & 63, sv.w & 63);
        bw[17] = pack4(sv.x >> 6, sv.y >> 6, sv.z >> 6, sv.w >> 6);
    }
    template <bool ODD>
    __device__ static uint32_t ldw(const uint8_t *p, int off) {
        if (!ODD) return *reinterpret_cast<const uint32_t *>(p + off);
        const uint32_t *q = reinterpret_cast<const uint32_t *>(p + off - 2);
        return __funnelshift_r(q[0], q[1], 16);
    }
    __device__ static int sbyte(uint32_t w, int k) { return (int)(int8_t)(w >> (8 * k)); }
    template <int NT, bool ODD>
    __device__ static void body(const uint8_t *p0, const uint8_t *p1, int t, const uint32_t (&bw)[NT][kBWords], const float2 (&e)[NT],
                                float (&accf)[NT][4]) {
        uint32_t sc0[4], sc1[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            sc0[i] = ldw<ODD>(p0, 192 + 4 * i);
            sc1[i] = ldw<ODD>(p1, 192 + 4 * i);
        }
        int isum[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) isum[nt][0] = isum[nt][1] = isum[nt][2] = isum[nt][3] = 0;
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
                    const int s0 = sbyte(sc0[s >> 2], s & 3), s1 = sbyte(sc1[s >> 2], s & 3);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        int pr[4];
                        wmma_k16_us(pr, a0[c], a1[c], bw[nt][s]);
                        isum[nt][0] += s0 * pr[0];
                        isum[nt][1] += s0 * pr[1];
                        isum[nt][2] += s1 * pr[2];
                        isum[nt][3] += s1 * pr[3];
                    }
                }
            }
        }
        // -32 * sum_s sc_s * bsum16_s, bsum16 = 64 h + l
        const uint32_t st0 = t == 0 ? sc0[0] : t == 1 ? sc0[1] : t == 2 ? sc0[2] : sc0[3];  // scales of sub-blocks 4t..4t+3
        const uint32_t st1 = t == 0 ? sc1[0] : t == 1 ? sc1[1] : t == 2 ? sc1[2] : sc1[3];
        const float d0 = h2f(*reinterpret_cast<const unsigned short *>(p0 + 208));
        const float d1 = h2f(*reinterpret_cast<const unsigned short *>(p1 + 208));
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            int cl[4], ch[4];
            wmma_k16_ss(cl, st0, st1, bw[nt][16]);
            wmma_k16_ss(ch, st0, st1, bw[nt][17]);
            accf[nt][0] = fmaf(d0 * e[nt].x, (float)(isum[nt][0] - 32 * (cl[0] + 64 * ch[0])), accf[nt][0]);
            accf[nt][1] = fmaf(d0 * e[nt].y, (float)(isum[nt][1] - 32 * (cl[1] + 64 * ch[1])), accf[nt][1]);
            accf[nt][2] = fmaf(d1 * e[nt].x, (float)(isum[nt][2] - 32 * (cl[2] + 64 * ch[2])), accf[nt][2]);
            accf[nt][3] = fmaf(d1 * e[nt].y, (float)(isum[nt][3] - 32 * (cl[3] + 64 * ch[3])), accf[nt][3]);
        }
    }
    template <int NT>
    __device__ static void block(const uint8_t *sl, int b, int g, int t, const uint32_t (&bw)[NT][kBWords], const float2 (&e)[NT],
                                 float (&accf)[NT][4]) {
        const uint8_t *p0 = sl + (size_t)g * kPitch + ((b * 210) & 15), *p1 = p0 + 8 * kPitch;
        if (b & 1)
            body<NT, true>(p0, p1, t, bw, e, accf);
        else
            body<NT, false>(p0, p1, t, bw, e, accf);
    }
};

// A second matrix of the same format and in_f against the same rows in the same launch (q and k, gate and up): its
// 16-row tiles follow the first matrix's in the CTAs' tile ranges.  out_f == 0: none.
struct WideSecond {
    CUtensorMap map;
    float *out;  // its result, or its partial results [K chunk][m][out_f]
    int out_f;
};

// Shared memory: rings [8 warps][slots][F::kSlotBytes], partial tiles [2][8 warps][8 NT tokens][17] f32, barriers.
template <class F, int NT, bool PUSH>
__global__ void __launch_bounds__(kWWarps * 32, 1)
    gemv_wide_kernel(const __grid_constant__ CUtensorMap tmap, Q8Dev a, float *__restrict__ out, int m, int in_f, int out_f, int slots,
                     uint32_t *__restrict__ status, const __grid_constant__ typename PushParam<PUSH>::type push,
                     const __grid_constant__ WideSecond sec) {
    constexpr int kPart = 8 * NT * kWPitch;  // floats of one warp's partial tile
    __shared__ uint32_t s_epoch;  // push mode (one K chunk only): exchanges completed before this launch
    extern __shared__ __align__(128) uint8_t smem[];
    const int S = slots;
    uint8_t *rings = smem;
    float *s_part = reinterpret_cast<float *>(rings + (size_t)kWWarps * S * F::kSlotBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_part + 2 * kWWarps * kPart);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nb = in_f >> 8;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kWWarps * kWSlots; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sw32(bars + i)), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this CTA's tiles (balanced contiguous ranges) and this warp's super-block
    const int tiles1 = (out_f + kWRows - 1) / kWRows, tiles = tiles1 + (sec.out_f + kWRows - 1) / kWRows;
    const int G = gridDim.x, base = tiles / G, rem = tiles % G;
    const int t_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int n_tiles = base + (blockIdx.x < rem ? 1 : 0);
    const int b = blockIdx.y * kWWarps + warp;
    const bool active = b < nb;
    const int n_jobs = active ? n_tiles : 0;
    uint8_t *ring = rings + (size_t)warp * S * F::kSlotBytes;
    uint64_t *wbar = bars + warp * kWSlots;

    uint64_t l2_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(l2_policy));
    int j_issue = 0;
    auto issue = [&](int slot) {
        if (j_issue >= n_jobs) return;
        if (lane == 0) {
            const uint32_t bar = sw32(wbar + slot);
            // order this warp's earlier reads of the slot before the engine overwrites it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)F::kSlotBytes) : "memory");
            const int T = t_begin + j_issue;
            if (T < tiles1)
                wide_tma(sw32(ring + (size_t)slot * F::kSlotBytes), &tmap, F::tma_x(b), T * kWRows, bar, l2_policy);
            else
                wide_tma(sw32(ring + (size_t)slot * F::kSlotBytes), &sec.map, F::tma_x(b), (T - tiles1) * kWRows, bar, l2_policy);
        }
        __syncwarp();
        j_issue++;
    };
    for (int s = 0; s < S; s++) issue(s);

    // ---- activations (from the previous kernel in the stream): this warp's super-block of every row, in registers ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (PUSH) {
        if (threadIdx.x == 0) s_epoch = *reinterpret_cast<const volatile uint32_t *>(push.ctrl);  // read after the tile barrier below
    }
    uint32_t bw[NT][F::kBWords];
    float2 e[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int n = nt * 8 + g;
        F::load_b(bw[nt], a, (size_t)n, b, nb, in_f, t, active && n < m);
        const int n0 = nt * 8 + 2 * t;  // the lane's two result columns
        e[nt].x = (active && n0 < m) ? a.d[(size_t)n0 * nb + b] : 0.f;
        e[nt].y = (active && n0 + 1 < m) ? a.d[(size_t)(n0 + 1) * nb + b] : 0.f;
    }

    // ---- consume ----
    float *dst = out + (size_t)blockIdx.y * (size_t)m * out_f;  // this K chunk's partial result
    float *dst2 = sec.out + (size_t)blockIdx.y * (size_t)m * sec.out_f;
    int slot = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int tile = 0; tile < n_tiles; tile++) {
        float accf[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) accf[nt][0] = accf[nt][1] = accf[nt][2] = accf[nt][3] = 0.f;
        if (active) {
            if (!dead && !wide_wait(sw32(wbar + slot), phase)) {
                dead = true;
                if (lane == 0) atomicExch(status, 3u);
            }
            if (!dead) F::template block<NT>(ring + (size_t)slot * F::kSlotBytes, b, g, t, bw, e, accf);
            __syncwarp();
            issue(slot);
            if (++slot == S) {
                slot = 0;
                phase ^= 1u;
            }
        }
        // this warp's partial tile: [token][row]
        float *part = s_part + ((size_t)(tile & 1) * kWWarps + warp) * kPart;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int n0 = nt * 8 + 2 * t;
            part[n0 * kWPitch + g] = accf[nt][0];
            part[(n0 + 1) * kWPitch + g] = accf[nt][1];
            part[n0 * kWPitch + g + 8] = accf[nt][2];
            part[(n0 + 1) * kWPitch + g + 8] = accf[nt][3];
        }
        __syncthreads();
        const int T = t_begin + tile;
        const bool second = T >= tiles1;
        const int row0 = (second ? T - tiles1 : T) * kWRows, of = second ? sec.out_f : out_f;
        for (int idx = threadIdx.x; idx < 8 * NT * kWRows; idx += kWWarps * 32) {
            const int n = idx >> 4, r = idx & 15;
            if (n < m && row0 + r < of) {
                const float *pp = s_part + (size_t)(tile & 1) * kWWarps * kPart + n * kWPitch + r;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kWWarps; w++) v += pp[w * kPart];
                if constexpr (PUSH)
                    push_store(push, s_epoch, (size_t)n * of + row0 + r, v);  // (no second matrix in push mode)
                else
                    (second ? dst2 : dst)[(size_t)n * of + row0 + r] = v;
            }
        }
    }
}

// y[i] = part[0][i] + part[1][i] + ... in chunk order (the same bits on every run).
// With push.world != 0 the sums go to the peers' staging instead (GemvPush).
// A second set of partial results (part2, n2 elements each) is added into y2 by the threads behind the first n.
__global__ void wide_sum_chunks_kernel(const float *__restrict__ part, float *__restrict__ y, size_t n, int kz, const __grid_constant__ GemvPush push,
                                       const float *__restrict__ part2, float *__restrict__ y2, size_t n2) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n + n2) return;
    if (i >= n) {
        i -= n;
        part = part2, y = y2, n = n2;
    }
    float acc = part[i];
    for (int s = 1; s < kz; s++) acc += part[(size_t)s * n + i];
    if (push.world)
        push_store(push, *reinterpret_cast<const volatile uint32_t *>(push.ctrl), i, acc);
    else
        y[i] = acc;
}

typedef CUresult (*EncWide)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                            const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                            CUtensorMapFloatOOBfill);
EncWide enc_wide() {
    static EncWide fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncWide>(p);
    }();
    return fn;
}

template <class F, int NT>
cudaError_t launch_wide_cfg(const CUtensorMap &tmap, const Q8Dev &a, float *y, float *partials, int m, int in_f, int out_f,
                            const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const GemvPush *push, const CUtensorMap *tmap2, float *y2,
                            int out_f2) {
    GemvPush none, mine;
    memset(&none, 0, sizeof none);
    mine = push ? *push : none;
    const int nb = in_f / 256, kz = (nb + kWWarps - 1) / kWWarps, tiles = (out_f + kWRows - 1) / kWRows + (out_f2 + kWRows - 1) / kWRows;
    WideSecond sec;
    memset(&sec, 0, sizeof sec);
    float *partials2 = partials ? partials + (size_t)kz * m * out_f : nullptr;
    if (out_f2 > 0) {
        sec.map = *tmap2;
        sec.out = kz > 1 ? partials2 : y2;
        sec.out_f = out_f2;
    }
    int gx = dev.sm_count / kz;
    if (gx < 1) gx = 1;
    if (gx > tiles) gx = tiles;
    int slots = (tiles + gx - 1) / gx;  // no more ring slots than a warp has jobs
    if (slots > kWSlots) slots = kWSlots;
    const size_t smem = (size_t)kWWarps * slots * F::kSlotBytes + (size_t)2 * kWWarps * 8 * NT * kWPitch * 4 + (size_t)kWWarps * kWSlots * 8 + 128;
    if (smem > (size_t)dev.max_smem_optin) return cudaErrorInvalidValue;
    // the GEMV itself pushes only when K is one chunk; otherwise the kernel that adds the chunks does
    const bool push_here = push && kz == 1;
    auto kernel = gemv_wide_kernel<F, NT, false>;
    auto kernel_push = gemv_wide_kernel<F, NT, true>;
    cudaError_t err = push_here ? cudaFuncSetAttribute(kernel_push, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                : cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, (unsigned)kz);
    cfg.blockDim = dim3(kWWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    err = push_here ? cudaLaunchKernelEx(&cfg, kernel_push, tmap, a, y, m, in_f, out_f, slots, status, mine, sec)
                    : cudaLaunchKernelEx(&cfg, kernel, tmap, a, kz > 1 ? partials : y, m, in_f, out_f, slots, status, NoPush{}, sec);
    if (err != cudaSuccess || kz == 1) return err;
    const size_t n = (size_t)m * out_f, n2 = (size_t)m * out_f2;
    cudaLaunchConfig_t c2 = {};
    c2.gridDim = dim3((unsigned)((n + n2 + 255) / 256));
    c2.blockDim = dim3(256);
    c2.stream = st;
    c2.attrs = attr;
    c2.numAttrs = 1;
    return cudaLaunchKernelEx(&c2, wide_sum_chunks_kernel, (const float *)partials, y, n, kz, mine, (const float *)partials2, y2, n2);
}

template <class F>
cudaError_t launch_wide_nt(const CUtensorMap &tmap, const Q8Dev &a, float *y, float *partials, int m, int in_f, int out_f,
                           const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const GemvPush *push, const CUtensorMap *tmap2 = nullptr,
                           float *y2 = nullptr, int out_f2 = 0) {
    if (m <= 16) return launch_wide_cfg<F, 2>(tmap, a, y, partials, m, in_f, out_f, dev, status, st, push, tmap2, y2, out_f2);
    if (m <= 24) return launch_wide_cfg<F, 3>(tmap, a, y, partials, m, in_f, out_f, dev, status, st, push, tmap2, y2, out_f2);
    return launch_wide_cfg<F, 4>(tmap, a, y, partials, m, in_f, out_f, dev, status, st, push, tmap2, y2, out_f2);
}

}  // namespace

// Scratch for the partial results of launch_gemv_wide (0 when K fits one chunk of 2048 elements).
size_t gemv_wide_partial_bytes(int m, int in_f, int out_f) {
    const int kz = (in_f / 256 + kWWarps - 1) / kWWarps;
    return kz > 1 ? (size_t)kz * (size_t)m * (size_t)out_f * 4 : 0;
}

// Launches on the given stream: 1 when K fits one chunk, else 2 (the GEMV and the sum of its chunks).
int gemv_wide_launches(int in_f) { return in_f / 256 > kWWarps ? 2 : 1; }

// y[m, out_f] for 1 <= m <= 32 pre-quantised rows (granularity 256; Q6_K also needs the 16-element sums) against a
// Q4_K or Q6_K matrix.  cudaErrorInvalidValue when the shape does not qualify (Q6_K rows whose byte length is not a
// multiple of 16 have no tensor map): the caller takes another kernel.
cudaError_t launch_gemv_wide(int dtype, const uint8_t *w, const Q8Dev &a, float *y, float *partials, int m, int in_f, int out_f,
                             const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const GemvPush *push, const uint8_t *w2, float *y2,
                             int out_f2) {
    if (m < 1 || m > 32 || in_f < 256 || in_f % 256 || out_f < 1 || a.gran != 256) return cudaErrorInvalidValue;
    if (out_f2 < 0 || (out_f2 > 0 && (!w2 || !y2 || push))) return cudaErrorInvalidValue;
    if (gemv_wide_partial_bytes(m, in_f, out_f + out_f2) && !partials) return cudaErrorInvalidValue;
    if ((in_f / 256 + kWWarps - 1) / kWWarps > 65535) return cudaErrorInvalidValue;
    if (((uintptr_t)a.qs % 8) || ((uintptr_t)a.sums % 16)) return cudaErrorInvalidValue;
    EncWide enc = enc_wide();
    if (!enc) return cudaErrorNotSupported;
    const int nb = in_f / 256;
    CUtensorMap tmap, tmap2;
    const cuuint32_t estr[2] = {1, 1};
    if (dtype == DT_Q4K) {
        auto encode = [&](CUtensorMap *map, const uint8_t *base, int rows) {
            const cuuint64_t gdim[2] = {(cuuint64_t)nb * 36, (cuuint64_t)rows};
            const cuuint64_t gstride[1] = {(cuuint64_t)nb * 144};
            const cuuint32_t box[2] = {36, (cuuint32_t)kWRows};
            return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        };
        if (!encode(&tmap, w, out_f) || (out_f2 > 0 && !encode(&tmap2, w2, out_f2))) return cudaErrorInvalidValue;
        return launch_wide_nt<WideQ4>(tmap, a, y, partials, m, in_f, out_f, dev, status, st, push, &tmap2, y2, out_f2);
    }
    if (dtype == DT_Q6K) {
        if (in_f % 2048 || !a.sums16 || ((uintptr_t)a.sums16 % 16)) return cudaErrorInvalidValue;
        // rows of nb * 105 16-bit elements; a box is 112 elements (224 B) x 16 rows and may run past the row's end (zero-filled)
        auto encode = [&](CUtensorMap *map, const uint8_t *base, int rows) {
            const cuuint64_t gdim[2] = {(cuuint64_t)nb * 105, (cuuint64_t)rows};
            const cuuint64_t gstride[1] = {(cuuint64_t)nb * 210};
            const cuuint32_t box[2] = {(cuuint32_t)WideQ6::kPitch / 2, (cuuint32_t)kWRows};
            return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<uint8_t *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        };
        if (!encode(&tmap, w, out_f) || (out_f2 > 0 && !encode(&tmap2, w2, out_f2))) return cudaErrorInvalidValue;
        return launch_wide_nt<WideQ6>(tmap, a, y, partials, m, in_f, out_f, dev, status, st, push, &tmap2, y2, out_f2);
    }
    return cudaErrorInvalidValue;
}

}  // namespace infr
