// Device helpers shared by the GEMV kernels: vector loads, the unsigned x signed byte dot product,
// Q4_K scale unpacking, and the shared-memory staging of quantised activations.
#pragma once
#include <cuda_fp16.h>

#include "kernels.h"

namespace infr {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint4 ldg16(const uint8_t *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t *p) {
    return (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p));
}
// 32-bit load from a 2-byte-aligned address (Q6_K / Q2_0 blocks are 210 / 18 bytes long).
__device__ __forceinline__ uint32_t ldg_u32_a2(const uint8_t *p) { return ldg_u16(p) | (ldg_u16(p + 2) << 16); }
// 4-way byte dot product, unsigned weight bytes x signed activation bytes, int32 accumulate.
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ float h2f(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)(bits16 & 0xffffu)));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- epilogue of a GEMV that pushes its result to the peers (GemvPush) ----
// The last parameter of such a kernel: the peers' staging (PUSH), or nothing at all - the ordinary kernel carries
// neither the parameter bytes nor the branch (the 148 bytes cost the 4096 x 4096 GEMV 2-3 % when they were always there).
struct NoPush {};
template <bool PUSH>
struct PushParam {
    typedef NoPush type;
};
template <>
struct PushParam<true> {
    typedef GemvPush type;
};
// One value of the result: slot [rank] of the exchange's parity on every rank, value and sequence number in one
// aligned 8-byte store.  The loop bound is a constant so that the pointer table is read from the kernel's parameters
// with constant indices.
__device__ __forceinline__ void push_store(const GemvPush &p, uint32_t done, size_t idx, float v) {
    const size_t off = ((size_t)(done & 1u) * p.world + p.rank) * p.cap + idx;
    const unsigned long long word = ((unsigned long long)(done + 1u) << 32) | (unsigned long long)__float_as_uint(v);
#pragma unroll
    for (int r = 0; r < kPushMaxWorld; r++)
        if (r < p.world) *reinterpret_cast<volatile unsigned long long *>(p.stage[r] + off) = word;
}

// get_scale_min_k4 (crates/infr-gguf/src/dequant.rs:73-83) for the sub-block pair (2j, 2j+1) of a
// Q4_K header held in registers: y = scales[0..3], z = scales[4..7], w = scales[8..11].
__device__ __forceinline__ void k4_pair(uint32_t y, uint32_t z, uint32_t w, int j, int &sc0, int &m0,
                                        int &sc1, int &m1) {
    const int sh = 16 * (j & 1);
    const uint32_t y2 = y >> sh, z2 = z >> sh, w2 = w >> sh;
    if (j < 2) {
        sc0 = y2 & 63;
        sc1 = (y2 >> 8) & 63;
        m0 = z2 & 63;
        m1 = (z2 >> 8) & 63;
    } else {
        sc0 = (w2 & 0xF) | (((y2 >> 6) & 3) << 4);
        sc1 = ((w2 >> 8) & 0xF) | (((y2 >> 14) & 3) << 4);
        m0 = ((w2 >> 4) & 0xF) | (((z2 >> 6) & 3) << 4);
        m1 = ((w2 >> 12) & 0xF) | (((z2 >> 14) & 3) << 4);
    }
}

// ------------------------------------------------------------------------------------------------
// Shared-memory staging of the quantised activations.
//   Q4_K : 16-byte unit u = 2*s + h of a 256-block (sub-block s, half h) moves to unit
//          (s&1)*8 + (s>>1)*2 + h, so the 8 lanes of a block read units 0..7 (even sub-blocks) and
//          8..15 (odd sub-blocks) as two contiguous 128-byte runs.
//   Q6_K : 4-byte word (half, k, l4) of block b moves to [b>>1][k][b&1][half][l4]: for a fixed k the
//          32 lanes of a warp (2 blocks x 2 halves x 8) hit 32 distinct banks.
//   Q2_0 : every 16-byte group is transposed 4x4 so word i holds elements (i, 4+i, 8+i, 12+i), the
//          order in which a 2-bit code word yields its fields.
// ------------------------------------------------------------------------------------------------
// Token t reads activation row row_of[row0 + t] (row_of == nullptr: row row0 + t) of the quantised rows in `a`.
template <int DT>
__device__ __forceinline__ void stage_q8(const Q8Dev &a, int m, int M, int in_f, int8_t *s_qa, float *s_d,
                                         int32_t *s_sum, const int32_t *row_of = nullptr, int row0 = 0) {
    const int units = in_f / 16;
    auto src_row = [&](int t) -> size_t { return (size_t)(row_of ? row_of[row0 + t] : row0 + t); };
    for (int idx = threadIdx.x; idx < M * units; idx += blockDim.x) {
        const int t = idx / units, u = idx - t * units;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < m) v = *reinterpret_cast<const uint4 *>(a.qs + src_row(t) * in_f + (size_t)u * 16);
        if (DT == DT_Q4K) {
            const int b = u >> 4, uu = u & 15, s = uu >> 1, h = uu & 1;
            const int nu = (s & 1) * 8 + (s >> 1) * 2 + h;
            reinterpret_cast<uint4 *>(s_qa + (size_t)t * in_f)[b * 16 + nu] = v;
        } else if (DT == DT_Q6K) {
            const int b = u >> 4, uu = u & 15;  // unit uu covers words 4uu..4uu+3 of the block
            uint32_t *dstw = reinterpret_cast<uint32_t *>(s_qa + (size_t)t * (((in_f >> 8) + 1) / 2 * 512));
            const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int w = uu * 4 + i, half = w >> 5, k = (w >> 3) & 3, l4 = w & 7;
                dstw[(b >> 1) * 128 + k * 32 + (b & 1) * 16 + half * 8 + l4] = vv[i];
            }
        } else {
            const uint32_t t01 = __byte_perm(v.x, v.y, 0x5140), t23 = __byte_perm(v.z, v.w, 0x5140);
            const uint32_t u01 = __byte_perm(v.x, v.y, 0x7362), u23 = __byte_perm(v.z, v.w, 0x7362);
            uint4 o;
            o.x = __byte_perm(t01, t23, 0x5410);
            o.y = __byte_perm(t01, t23, 0x7632);
            o.z = __byte_perm(u01, u23, 0x5410);
            o.w = __byte_perm(u01, u23, 0x7632);
            reinterpret_cast<uint4 *>(s_qa + (size_t)t * in_f)[u] = o;
        }
    }
    const int nd = in_f / a.gran;
    for (int idx = threadIdx.x; idx < M * nd; idx += blockDim.x) {
        const int t = idx / nd, i = idx - t * nd;
        s_d[idx] = t < m ? a.d[src_row(t) * nd + i] : 0.f;
    }
    const int ns = DT == DT_Q6K ? in_f / 16 : in_f / 32;
    const int32_t *src = DT == DT_Q6K ? a.sums16 : a.sums;
    for (int idx = threadIdx.x; idx < M * ns; idx += blockDim.x) {
        const int t = idx / ns, i = idx - t * ns;
        s_sum[idx] = t < m ? src[src_row(t) * ns + i] : 0;
    }
}


}  // namespace
}  // namespace infr
