// Streaming decode GEMV (int8 activations) for sm_100a: weights travel HBM -> shared memory through
// the bulk-copy engine (cp.async.bulk, 1-D TMA) and are consumed from there, so the bytes in flight per
// SM are set by the shared-memory rings, not by how many registers the math warps can hold.
//
// Work split.  The grid is up to two persistent CTAs per SM; CTA i owns a contiguous, balanced range
// of output rows and its warps claim rows from a CTA-local counter.  Every warp runs its OWN pipeline:
// lane 0 issues the bulk copy of the next K-slice of the warp's current row into one of the warp's
// private ring slots (completion on a per-slot mbarrier), the whole warp then reduces a landed slice
// against the staged activations and immediately refills the slot it has just drained.  Warps never
// wait on each other after the one barrier that publishes the staged activations.  A row's partial sum
// stays in registers across its slices, meets in one shuffle tree and is written once.  The arithmetic
// is the production infr-cpu arithmetic (crates/infr-cpu/src/kernels.rs:151-184, :487-526, :5641-5668):
// exact int32 block sums, f32 only for the per-block scale products.
//
// Q6_K / Q2_0 blocks are 210 / 18 bytes, so a slice of a row may start on any even address: the copy
// fetches the 16-byte-aligned superset and the consumer indexes from the remainder.
//
// Programmatic dependent launch: the weights do not depend on the previous kernel in the stream, so
// every warp puts its first slices in flight at once and only the activation staging waits on
// `griddepcontrol.wait`; `griddepcontrol.launch_dependents` lets the next kernel's CTAs begin their
// own weight stream while this one drains.
//
// Every mbarrier wait is bounded: when the limit is hit the warp records a status word for the host,
// stops claiming work, waits (bounded again) for the copies it still has in flight and returns.
#include <cstdlib>

#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kStreamWarps = 16;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kMaxSlots = 4;              // ring slots per warp
constexpr uint32_t kSpinLimit = 1u << 22; // polls of mbarrier.try_wait before giving up

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t lds_u16(const uint8_t *p) { return *reinterpret_cast<const unsigned short *>(p); }
__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t *p) { return lds_u16(p) | (lds_u16(p + 2) << 16); }

template <int DT>
struct Fmt;
template <>
struct Fmt<DT_Q4K> {
    static constexpr int kBlockBytes = 144, kBlockElems = 256, kSliceBlocks = 16, kStepBlocks = 8;
};
template <>
struct Fmt<DT_Q6K> {
    static constexpr int kBlockBytes = 210, kBlockElems = 256, kSliceBlocks = 16, kStepBlocks = 2;
};
template <>
struct Fmt<DT_Q2_0> {
    static constexpr int kBlockBytes = 18, kBlockElems = 64, kSliceBlocks = 128, kStepBlocks = 8;
};

// ---- per-format slice processors: `sl` points at the first block of this row's slice in shared
// memory, `nblk` blocks long, whose first block is block `gb0` of the row. --------------------------
// Q4_K: 4 lanes per super-block, lane j owns the 32 nibble bytes of sub-block pair (2j, 2j+1): the low
// nibbles are the 32 elements of sub-block 2j, the high nibbles those of 2j+1.  High nibbles are fed to
// the byte dot product unshifted (values 16x) and the sum is shifted back once, exactly.  A slice of 8
// blocks is one warp step.  Staged activations are laid out [block pair][k][block&1][j] in 16-byte
// units (k = 0,1: elements 0-15 / 16-31 of sub-block 2j; k = 2,3: of 2j+1) so that every 128-bit
// shared-memory read of a quarter-warp covers 128 contiguous bytes.
template <int M>
__device__ __forceinline__ void slice_q4k(const uint8_t *sl, int nblk, int gb0, int nb, int in_f, const int8_t *s_qa,
                                          const float *s_d, const int32_t *s_bs, int lane, float (&acc)[M]) {
    const int j = lane & 3;
    const int tok_stride = (nb + 1) / 2 * 512;
    for (int bl = lane >> 2; bl < nblk; bl += 8) {
    const int b = gb0 + bl;
    const uint8_t *blk = sl + bl * 144;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + j * 32);
    const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32 + j * 32);
    // get_scale_min_k4 for the pair (2j, 2j+1), on packed bytes
    uint32_t scw, mw;
    if (j < 2) {
        scw = hdr.y & 0x3F3F3F3Fu;
        mw = hdr.z & 0x3F3F3F3Fu;
    } else {
        scw = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        mw = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    }
    const uint32_t sel = (j & 1) ? 0x4442u : 0x4440u;  // byte 2 or byte 0, zero-extended
    const int sc0 = (int)__byte_perm(scw, 0, sel), sc1 = (int)__byte_perm(scw, 0, sel + 1);
    const int m0 = (int)__byte_perm(mw, 0, sel), m1 = (int)__byte_perm(mw, 0, sel + 1);
    const float d = h2f(hdr.x), dmin = h2f(hdr.x >> 16);
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int t = 0; t < M; t++) {
        const uint4 *au = reinterpret_cast<const uint4 *>(s_qa + (size_t)t * tok_stride) + (b >> 1) * 32 + (b & 1) * 4 + j;
        const uint4 a0 = au[0], a1 = au[8], a2 = au[16], a3 = au[24];
        const int al[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
        const int ah[8] = {(int)a2.x, (int)a2.y, (int)a2.z, (int)a2.w, (int)a3.x, (int)a3.y, (int)a3.z, (int)a3.w};
        int ilo = 0, ihi = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            ilo = dp4a_us(q[i] & 0x0F0F0F0Fu, al[i], ilo);
            ihi = dp4a_us(q[i] & 0xF0F0F0F0u, ah[i], ihi);
        }
        const int2 bs = *reinterpret_cast<const int2 *>(s_bs + (t * nb + b) * 8 + 2 * j);
        const int sd = sc0 * ilo + sc1 * (ihi >> 4);
        const int sm = m0 * bs.x + m1 * bs.y;
        acc[t] += s_d[t * nb + b] * (d * (float)sd - dmin * (float)sm);
    }
    }
}

template <int M>
__device__ __forceinline__ void slice_q6k(const uint8_t *sl, int nblk, int gb0, int nb, int in_f, const int8_t *s_qa,
                                          const float *s_d, const int32_t *s_bs, int lane, float (&acc)[M]) {
    const int hb = lane >> 4, r = lane & 15, half = r >> 3, l4 = r & 7;
    const int tok_stride = (nb + 1) / 2 * 512;
#pragma unroll 2
    for (int b0 = 0; b0 < nblk; b0 += 2) {
        const int bl = b0 + hb;
        if (bl < nblk) {
            const int b = gb0 + bl;
            const uint8_t *blk = sl + bl * 210;
            const uint32_t qla = lds_u32_a2(blk + half * 64 + l4 * 4);
            const uint32_t qlb = lds_u32_a2(blk + half * 64 + 32 + l4 * 4);
            const uint32_t qh = lds_u32_a2(blk + 128 + half * 32 + l4 * 4);
            const int8_t *scp = reinterpret_cast<const int8_t *>(blk + 192);
            const int is = l4 >> 2;
            int sc[4];
#pragma unroll
            for (int k = 0; k < 4; k++) sc[k] = (int)scp[half * 8 + is + 2 * k];
            const int scr = (int)scp[r];
            const float dw = h2f(lds_u16(blk + 208));
            uint32_t q[4];
            q[0] = (qla & 0x0F0F0F0Fu) | ((qh & 0x03030303u) << 4);
            q[1] = (qlb & 0x0F0F0F0Fu) | (((qh >> 2) & 0x03030303u) << 4);
            q[2] = ((qla >> 4) & 0x0F0F0F0Fu) | (((qh >> 4) & 0x03030303u) << 4);
            q[3] = ((qlb >> 4) & 0x0F0F0F0Fu) | (((qh >> 6) & 0x03030303u) << 4);
#pragma unroll
            for (int t = 0; t < M; t++) {
                const int *aw = reinterpret_cast<const int *>(s_qa + (size_t)t * tok_stride) + (b >> 1) * 128 +
                                (b & 1) * 16 + half * 8 + l4;
                int isum = 0;
#pragma unroll
                for (int k = 0; k < 4; k++) isum += sc[k] * dp4a_us(q[k], aw[k * 32], 0);
                isum -= 32 * scr * s_bs[(t * nb + b) * 16 + r];
                acc[t] += (dw * s_d[t * nb + b]) * (float)isum;
            }
        }
    }
}

// Q2_0: one LANE per 64-element block (a warp step is 32 blocks), so that the block's scale, its 18 bytes and the
// unpacking are fetched and done once per 64 elements: five aligned 32-bit reads cover the block wherever its even
// address falls, a funnel shift lines the four code words up.  A code word holds 16 two-bit codes; masking it at
// shifts 0 / 2 / 4 / 6 gives the codes of elements {0,4,8,12}, {1,5,9,13}, ... as bytes, which the staged activations
// are permuted to match.  Staged activations are laid out [quarter][block] in 16-byte units, so the lanes of a warp
// (consecutive blocks) read consecutive units.  Per 32-element group: (sum of code * x) - (sum of x), one float
// multiply-add with the group's two scales (crates/infr-cpu/src/kernels.rs:5641-5668).
template <int M>
__device__ __forceinline__ void slice_q2_0(const uint8_t *sl, int nblk, int gb0, int nb, int in_f, const int8_t *s_qa,
                                           const float *s_d, const int32_t *s_bs, int lane, float (&acc)[M]) {
    const int ns = nb * 2;
    for (int b0 = 0; b0 < nblk; b0 += 32) {
        const int bl = b0 + lane;
        if (bl < nblk) {
            const int b = gb0 + bl;
            const uint8_t *blk = sl + bl * 18;
            const uint32_t mis = (uint32_t)(smem_u32(blk) & 2u);  // the block starts on a 4-byte boundary, or 2 past one
            const uint32_t *wp = reinterpret_cast<const uint32_t *>(blk - mis);
            const uint32_t w0 = wp[0], w1 = wp[1], w2 = wp[2], w3 = wp[3], w4 = wp[4];
            const uint32_t sh = 16u + 8u * mis;  // 16, or 32 (= take the upper word)
            const float dw = h2f(w0 >> (8u * mis));
            const uint32_t c[4] = {__funnelshift_rc(w0, w1, sh), __funnelshift_rc(w1, w2, sh), __funnelshift_rc(w2, w3, sh),
                                   __funnelshift_rc(w3, w4, sh)};
            int ip[M][2];
#pragma unroll
            for (int t = 0; t < M; t++) ip[t][0] = ip[t][1] = 0;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t m0 = c[q] & 0x03030303u, m1 = (c[q] >> 2) & 0x03030303u, m2 = (c[q] >> 4) & 0x03030303u, m3 = (c[q] >> 6) & 0x03030303u;
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const uint4 av = reinterpret_cast<const uint4 *>(s_qa + (size_t)t * in_f)[q * nb + b];
                    int v = dp4a_us(m0, (int)av.x, ip[t][q >> 1]);
                    v = dp4a_us(m1, (int)av.y, v);
                    v = dp4a_us(m2, (int)av.z, v);
                    ip[t][q >> 1] = dp4a_us(m3, (int)av.w, v);
                }
            }
#pragma unroll
            for (int t = 0; t < M; t++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int s = 2 * b + h;
                    acc[t] += dw * s_d[t * ns + s] * (float)(ip[t][h] - s_bs[t * ns + s]);
                }
            }
        }
    }
}

struct StreamGeom {
    int nb;          // weight blocks per row
    int n_slices;    // K-slices per row
    int slot_bytes;  // shared-memory bytes per ring slot
    int slots;       // ring slots per warp
    uint32_t act_bytes;  // staged activations (codes + scales + sums), 16-byte aligned
};

template <int DT, int M>
__global__ void __launch_bounds__(kStreamThreads, (M <= 2 ? 2 : 1))
    gemv_stream_kernel(const uint8_t *__restrict__ W, Q8Dev a, float *__restrict__ y, int m, int in_f, int out_f,
                       StreamGeom geo, uint32_t *__restrict__ status) {
    using F = Fmt<DT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = geo.nb, S = geo.slots;
    uint8_t *act = smem + (size_t)kStreamWarps * S * geo.slot_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(act + geo.act_bytes);  // [warp][slot]
    int2 *meta = reinterpret_cast<int2 *>(bars + kStreamWarps * kMaxSlots); // [warp][slot] = (row, slice)
    __shared__ int s_next;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_next = 0;
        for (int i = 0; i < kStreamWarps * kMaxSlots; i++) mbar_init(smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    // balanced contiguous row range of this CTA
    const int G = gridDim.x, base = out_f / G, rem = out_f % G;
    const int r_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int r_count = base + (blockIdx.x < rem ? 1 : 0);
    const size_t row_bytes = (size_t)nb * F::kBlockBytes;
    uint8_t *ring = smem + (size_t)warp * S * geo.slot_bytes;
    uint64_t *wbar = bars + warp * kMaxSlots;
    int2 *wmeta = meta + warp * kMaxSlots;

    // ---- issue side (warp-uniform state; lane 0 talks to the copy engine) ----
    int i_row = -1, i_ks = 0;
    auto issue = [&](int slot) {
        if (i_ks == 0) {
            int idx = 0;
            if (lane == 0) idx = atomicAdd(&s_next, 1);
            idx = __shfl_sync(0xffffffffu, idx, 0);
            i_row = idx < r_count ? r_begin + idx : -1;
        }
        if (lane == 0) {
            wmeta[slot] = make_int2(i_row, i_ks);
            if (i_row >= 0) {
                const int blk0 = i_ks * F::kSliceBlocks;
                const int nblk = min(F::kSliceBlocks, nb - blk0);
                const size_t start = (size_t)W + (size_t)i_row * row_bytes + (size_t)blk0 * F::kBlockBytes;
                const size_t a0 = start & ~(size_t)15;
                const uint32_t bytes = (uint32_t)(((start + (size_t)nblk * F::kBlockBytes + 15) & ~(size_t)15) - a0);
                const uint32_t bar = smem_u32(wbar + slot);
                // order this warp's earlier reads of the slot before the engine overwrites it
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(bar, bytes);
                bulk_g2s(smem_u32(ring + (size_t)slot * geo.slot_bytes), reinterpret_cast<const void *>(a0), bytes, bar);
            }
        }
        __syncwarp();
        if (i_row >= 0) i_ks = (i_ks + 1 == geo.n_slices) ? 0 : i_ks + 1;
    };
    for (int s = 0; s < S; s++) issue(s);

    // ---- activations: produced by the previous kernel in the stream ----
    pdl_wait();
    int8_t *s_qa = reinterpret_cast<int8_t *>(act);
    const int code_bytes = DT != DT_Q2_0 ? M * ((nb + 1) / 2 * 512) : M * in_f;
    float *s_d = reinterpret_cast<float *>(act + code_bytes);
    const int nd = in_f / a.gran;
    int32_t *s_bs = reinterpret_cast<int32_t *>(act + code_bytes + ((M * nd * 4 + 15) & ~15));
    {
        const int tid = threadIdx.x, nthr = kStreamThreads;
        const int units = in_f / 16;
        for (int idx = tid; idx < M * units; idx += nthr) {
            const int t = idx / units, u = idx - t * units;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t < m) v = *reinterpret_cast<const uint4 *>(a.qs + (size_t)t * in_f + (size_t)u * 16);
            if (DT == DT_Q4K) {
                const int b = u >> 4, uu = u & 15, s = uu >> 1, h = uu & 1;
                const int k = (s & 1) * 2 + h, j = s >> 1;
                reinterpret_cast<uint4 *>(s_qa + (size_t)t * ((nb + 1) / 2 * 512))[(b >> 1) * 32 + k * 8 + (b & 1) * 4 + j] = v;
            } else if (DT == DT_Q6K) {
                const int b = u >> 4, uu = u & 15;
                uint32_t *dstw = reinterpret_cast<uint32_t *>(s_qa + (size_t)t * ((nb + 1) / 2 * 512));
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
                reinterpret_cast<uint4 *>(s_qa + (size_t)t * in_f)[(u & 3) * nb + (u >> 2)] = o;  // [quarter][block]
            }
        }
        for (int idx = tid; idx < M * nd; idx += nthr) {
            const int t = idx / nd, i = idx - t * nd;
            s_d[idx] = t < m ? a.d[(size_t)t * nd + i] : 0.f;
        }
        const int ns = DT == DT_Q6K ? in_f / 16 : in_f / 32;
        const int32_t *src = DT == DT_Q6K ? a.sums16 : a.sums;
        for (int idx = tid; idx < M * ns; idx += nthr) {
            const int t = idx / ns, i = idx - t * ns;
            s_bs[idx] = t < m ? src[(size_t)t * ns + i] : 0;
        }
    }
    __syncthreads();

    // ---- consume side ----
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; i++) acc[i] = 0.f;
    int slot = 0;
    uint32_t phase = 0;
    for (;;) {
        const int2 job = wmeta[slot];  // written by this warp's lane 0 before a __syncwarp
        const int row = job.x, ks = job.y;
        if (row < 0) break;
        if (!mbar_wait(smem_u32(wbar + slot), phase)) {
            if (lane == 0) atomicExch(status, 2u);
            // stop claiming work; give the copies still in flight a bounded chance to land
            for (int k = 1; k < S; k++) {
                const int s2 = (slot + k) % S;
                if (wmeta[s2].x >= 0) mbar_wait(smem_u32(wbar + s2), s2 > slot ? phase : phase ^ 1u);
            }
            return;
        }
        const int blk0 = ks * F::kSliceBlocks;
        const int nblk = min(F::kSliceBlocks, nb - blk0);
        const size_t start = (size_t)W + (size_t)row * row_bytes + (size_t)blk0 * F::kBlockBytes;
        const uint8_t *sl = ring + (size_t)slot * geo.slot_bytes + (DT == DT_Q4K ? 0 : (int)(start & 15));
        if (DT == DT_Q4K)
            slice_q4k<M>(sl, nblk, blk0, nb, in_f, s_qa, s_d, s_bs, lane, acc);
        else if (DT == DT_Q6K)
            slice_q6k<M>(sl, nblk, blk0, nb, in_f, s_qa, s_d, s_bs, lane, acc);
        else
            slice_q2_0<M>(sl, nblk, blk0, nb, in_f, s_qa, s_d, s_bs, lane, acc);
        __syncwarp();
        issue(slot);
        if (ks == geo.n_slices - 1) {
#pragma unroll
            for (int i = 0; i < M; i++) {
                const float v = warp_sum(acc[i]);
                if (lane == 0 && i < m) y[(size_t)i * out_f + row] = v;
                acc[i] = 0.f;
            }
        }
        if (++slot == S) {
            slot = 0;
            phase ^= 1u;
        }
    }
}

template <int DT, int M>
cudaError_t launch_stream_dt(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                             const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    using F = Fmt<DT>;
    StreamGeom geo;
    geo.nb = in_f / F::kBlockElems;
    geo.n_slices = (geo.nb + F::kSliceBlocks - 1) / F::kSliceBlocks;
    const int slice_bytes = (geo.nb < F::kSliceBlocks ? geo.nb : F::kSliceBlocks) * F::kBlockBytes;
    geo.slot_bytes = ((slice_bytes + 15) / 16 * 16) + 32;
    const size_t codes = DT != DT_Q2_0 ? (size_t)M * ((geo.nb + 1) / 2 * 512) : (size_t)M * in_f;
    const size_t acts = codes + (((size_t)M * (in_f / a.gran) * 4 + 15) & ~(size_t)15) +
                        (size_t)M * (DT == DT_Q6K ? in_f / 16 : in_f / 32) * 4;
    geo.act_bytes = (uint32_t)((acts + 15) / 16 * 16);
    const size_t fixed = geo.act_bytes + (size_t)kStreamWarps * kMaxSlots * 16 + 64;
    const size_t per_slot = (size_t)kStreamWarps * geo.slot_bytes;
    if (fixed + 2 * per_slot > (size_t)dev.max_smem_optin) return cudaErrorInvalidValue;
    // Two resident CTAs per SM when they fit with at least 2 ring slots per warp.
    const size_t half = (size_t)dev.max_smem_optin / 2 - 2048;
    int per_sm = (M <= 2 && fixed + 2 * per_slot <= half) ? 2 : 1;
    const size_t budget = per_sm == 2 ? half : (size_t)dev.max_smem_optin - 1024;
    int slots = (int)((budget - fixed) / per_slot);
    if (slots > kMaxSlots) slots = kMaxSlots;
    geo.slots = slots;
    const size_t smem = (size_t)slots * per_slot + fixed;
    int grid = (out_f + kStreamWarps - 1) / kStreamWarps;
    if (grid > dev.sm_count * per_sm) grid = dev.sm_count * per_sm;
    auto kernel = gemv_stream_kernel<DT, M>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, w, a, y, m, in_f, out_f, geo, status);
}

template <int M>
cudaError_t launch_stream_m(int dt, const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                            const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (dt == DT_Q4K) return launch_stream_dt<DT_Q4K, M>(w, a, y, m, in_f, out_f, dev, status, st);
    if (dt == DT_Q6K) return launch_stream_dt<DT_Q6K, M>(w, a, y, m, in_f, out_f, dev, status, st);
    return launch_stream_dt<DT_Q2_0, M>(w, a, y, m, in_f, out_f, dev, status, st);
}

}  // namespace

cudaError_t launch_gemv_stream(int dt, const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                               const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (m < 1 || m > 8 || (dt != DT_Q4K && dt != DT_Q6K && dt != DT_Q2_0)) return cudaErrorInvalidValue;
    if (dt == DT_Q2_0 && m > 1 && in_f % 512 == 0 && a.gran == 32) {
        // batches on rows of whole 512-element chunks take the matrix-unit kernel (1.6x faster at m = 4 and 8,
        // no gain at m = 1); it declines shapes whose staged activations do not fit, and those fall through
        // to the byte-dot kernel below
        const cudaError_t e = launch_gemv_q2_mma(w, a, y, m, in_f, out_f, dev, status, st);
        if (e != cudaErrorInvalidValue) return e;
        cudaGetLastError();
    }
    if (dt == DT_Q6K && in_f % 2048 == 0 && a.gran == 256 && a.sums16) {
        // rows whose byte length is a multiple of 16 take the matrix-unit kernel (same fall-through rule)
        const cudaError_t e = launch_gemv_q6_mma(w, a, y, m, in_f, out_f, dev, status, st);
        if (e != cudaErrorInvalidValue) return e;
        cudaGetLastError();
    }
    if (m == 1) return launch_stream_m<1>(dt, w, a, y, m, in_f, out_f, dev, status, st);
    if (m == 2) return launch_stream_m<2>(dt, w, a, y, m, in_f, out_f, dev, status, st);
    if (m <= 4) return launch_stream_m<4>(dt, w, a, y, m, in_f, out_f, dev, status, st);
    return launch_stream_m<8>(dt, w, a, y, m, in_f, out_f, dev, status, st);
}

}  // namespace infr
