// Streaming decode GEMV (int8 activations) for sm_100a: weights travel HBM -> shared memory through
// the bulk-copy engine (cp.async.bulk, 1-D TMA) into a multi-stage ring guarded by mbarriers, so the
// bytes in flight per SM are set by the ring size, not by how many registers the math warps can hold.
//
// Work split.  The grid is one persistent CTA per SM; CTA i owns a contiguous, balanced range of
// output rows.  Rows are taken kRows at a time (one per consumer warp) and every row is cut into
// K-slices of kSliceBytes; a ring stage holds one K-slice of kRows rows and is filled by kRows bulk
// copies issued in parallel by the lanes of the producer warp.  Consumer warp w accumulates row w
// across its K-slices in registers, reduces with one shuffle tree and writes y.  The arithmetic is
// the production infr-cpu arithmetic (crates/infr-cpu/src/kernels.rs:151-184, :487-526, :5641-5668):
// exact int32 block sums, f32 only for the per-block scale products.
//
// Q6_K / Q2_0 blocks are 210 / 18 bytes, so a slice of a row may start on any even address: the copy
// fetches the 16-byte-aligned superset and the consumer indexes from the remainder.
//
// Programmatic dependent launch: the weights do not depend on the previous kernel in the stream, so
// the producer starts streaming them immediately and only the activation staging waits on
// `griddepcontrol.wait`; `griddepcontrol.launch_dependents` lets the next kernel's CTAs begin their
// own weight stream while this one drains.
//
// Every mbarrier wait is bounded: when the limit is hit the kernel records a status word for the
// host, stops issuing work, drains the copies it has in flight (bounded again) and returns.
#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kRows = 16;                 // consumer warps == rows per ring stage
constexpr int kStreamThreads = (kRows + 1) * 32;
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
    static constexpr int kBlockBytes = 144, kBlockElems = 256, kSliceBlocks = 8;
};
template <>
struct Fmt<DT_Q6K> {
    static constexpr int kBlockBytes = 210, kBlockElems = 256, kSliceBlocks = 8;
};
template <>
struct Fmt<DT_Q2_0> {
    static constexpr int kBlockBytes = 18, kBlockElems = 64, kSliceBlocks = 64;
};

// ---- per-format slice processors: `sl` points at the first block of this row's slice in shared
// memory, `nblk` blocks long, whose first block is block `gb0` of the row. --------------------------
template <int M>
__device__ __forceinline__ void slice_q4k(const uint8_t *sl, int nblk, int gb0, int nb, int in_f, const int8_t *s_qa,
                                          const float *s_d, const int32_t *s_bs, int lane, float (&acc)[M]) {
    const int g = lane >> 3, c = lane & 7, j = c >> 1;
#pragma unroll 2
    for (int b0 = 0; b0 < nblk; b0 += 4) {
        const int bl = b0 + g;
        if (bl < nblk) {
            const int b = gb0 + bl;
            const uint8_t *blk = sl + bl * 144;
            const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
            const uint4 qv = *reinterpret_cast<const uint4 *>(blk + 16 + c * 16);
            int sc0, m0, sc1, m1;
            k4_pair(hdr.y, hdr.z, hdr.w, j, sc0, m0, sc1, m1);
            const float d = h2f(hdr.x), dmin = h2f(hdr.x >> 16);
            const int mc = (c & 1) ? m1 : m0;
            const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int t = 0; t < M; t++) {
                const uint4 alo = reinterpret_cast<const uint4 *>(s_qa + (size_t)t * in_f)[b * 16 + c];
                const uint4 ahi = reinterpret_cast<const uint4 *>(s_qa + (size_t)t * in_f)[b * 16 + 8 + c];
                const int al[4] = {(int)alo.x, (int)alo.y, (int)alo.z, (int)alo.w};
                const int ah[4] = {(int)ahi.x, (int)ahi.y, (int)ahi.z, (int)ahi.w};
                int ilo = 0, ihi = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    ilo = dp4a_us(q[i] & 0x0F0F0F0Fu, al[i], ilo);
                    ihi = dp4a_us((q[i] >> 4) & 0x0F0F0F0Fu, ah[i], ihi);
                }
                const int sd = sc0 * ilo + sc1 * ihi;
                const int sm = mc * s_bs[(t * nb + b) * 8 + c];
                acc[t] += s_d[t * nb + b] * (d * (float)sd - dmin * (float)sm);
            }
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

template <int M>
__device__ __forceinline__ void slice_q2_0(const uint8_t *sl, int nblk, int gb0, int nb, int in_f, const int8_t *s_qa,
                                           const float *s_d, const int32_t *s_bs, int lane, float (&acc)[M]) {
    const int g = lane >> 2, q = lane & 3;
    const int ns = nb * 2;
#pragma unroll 2
    for (int b0 = 0; b0 < nblk; b0 += 8) {
        const int bl = b0 + g;
        if (bl < nblk) {
            const int b = gb0 + bl;
            const int s = 2 * b + (q >> 1);
            const uint8_t *blk = sl + bl * 18;
            const float dw = h2f(lds_u16(blk));
            const uint32_t w = lds_u32_a2(blk + 2 + q * 4);
#pragma unroll
            for (int t = 0; t < M; t++) {
                const uint4 av = reinterpret_cast<const uint4 *>(s_qa + (size_t)t * in_f)[b * 4 + q];
                int ip = dp4a_us(w & 0x03030303u, (int)av.x, 0);
                ip = dp4a_us((w >> 2) & 0x03030303u, (int)av.y, ip);
                ip = dp4a_us((w >> 4) & 0x03030303u, (int)av.z, ip);
                ip = dp4a_us((w >> 6) & 0x03030303u, (int)av.w, ip);
                const int v = ip - ((q & 1) ? 0 : s_bs[t * ns + s]);
                acc[t] += dw * s_d[t * ns + s] * (float)v;
            }
        }
    }
}

struct StreamGeom {
    int nb;          // weight blocks per row
    int n_slices;    // K-slices per row
    int slot_bytes;  // shared-memory bytes reserved per (stage, row)
    int stages;
    uint32_t act_bytes;  // staged activations (codes + scales + sums), 16-byte aligned
};

template <int DT, int M>
__global__ void __launch_bounds__(kStreamThreads, (M <= 2 ? 2 : 1))
    gemv_stream_kernel(const uint8_t *__restrict__ W, Q8Dev a, float *__restrict__ y, int m, int in_f, int out_f,
                       StreamGeom geo, uint32_t *__restrict__ status) {
    using F = Fmt<DT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = geo.nb, S = geo.stages;
    uint8_t *ring = smem;
    uint8_t *act = smem + (size_t)S * kRows * geo.slot_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(act + geo.act_bytes);  // full[S], empty[S]
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < S; s++) {
            mbar_init(smem_u32(bars + s), 1);
            mbar_init(smem_u32(bars + S + s), kRows);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // balanced contiguous row range of this CTA
    const int G = gridDim.x, base = out_f / G, rem = out_f % G;
    const int r_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int r_count = base + (blockIdx.x < rem ? 1 : 0);
    const int n_groups = (r_count + kRows - 1) / kRows;
    const int n_tiles = n_groups * geo.n_slices;
    const size_t row_bytes = (size_t)nb * F::kBlockBytes;

    if (warp == kRows) {
        // ------------------------------------------------------------------ producer warp
        pdl_launch_dependents();
        bool ok = true;
        int issued = 0;
        for (int t = 0; t < n_tiles && ok; t++) {
            const int s = t % S, use = t / S;
            if (use > 0) ok = mbar_wait(smem_u32(bars + S + s), (uint32_t)((use - 1) & 1));
            if (*(volatile int *)&s_abort) ok = false;
            if (!ok) break;
            const int grp = t / geo.n_slices, ks = t - grp * geo.n_slices;
            const int row = r_begin + grp * kRows + lane;
            const int blk0 = ks * F::kSliceBlocks;
            const int nblk = min(F::kSliceBlocks, nb - blk0);
            uint32_t bytes = 0;
            const uint8_t *src = nullptr;
            if (lane < kRows && row < r_begin + r_count) {
                const size_t start = (size_t)W + (size_t)row * row_bytes + (size_t)blk0 * F::kBlockBytes;
                const size_t end = start + (size_t)nblk * F::kBlockBytes;
                const size_t a0 = start & ~(size_t)15, a1 = (end + 15) & ~(size_t)15;
                src = reinterpret_cast<const uint8_t *>(a0);
                bytes = (uint32_t)(a1 - a0);
            }
            uint32_t total = bytes;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0) mbar_expect_tx(smem_u32(bars + s), total);
            __syncwarp();
            if (bytes) bulk_g2s(smem_u32(ring + ((size_t)s * kRows + lane) * geo.slot_bytes), src, bytes, smem_u32(bars + s));
            issued = t + 1;
        }
        if (!ok) {
            if (lane == 0) {
                atomicExch(status, 1u);
                *(volatile int *)&s_abort = 1;
            }
            // drain: every stage filled but possibly not yet landed
            for (int t = max(0, issued - S); t < issued; t++) mbar_wait(smem_u32(bars + (t % S)), (uint32_t)((t / S) & 1));
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    pdl_wait();  // activations come from the previous kernel in the stream
    {
        int8_t *s_qa = reinterpret_cast<int8_t *>(act);
        const int code_bytes = DT == DT_Q6K ? M * ((nb + 1) / 2 * 512) : M * in_f;
        float *s_d = reinterpret_cast<float *>(act + code_bytes);
        const int nd = in_f / a.gran;
        int32_t *s_bs = reinterpret_cast<int32_t *>(s_d + M * nd);
        // stage_q8 strides by blockDim.x; only the consumer threads take part here
        const int tid = threadIdx.x, nthr = kRows * 32;
        const int units = in_f / 16;
        for (int idx = tid; idx < M * units; idx += nthr) {
            const int t = idx / units, u = idx - t * units;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t < m) v = *reinterpret_cast<const uint4 *>(a.qs + (size_t)t * in_f + (size_t)u * 16);
            if (DT == DT_Q4K) {
                const int b = u >> 4, uu = u & 15, s = uu >> 1, h = uu & 1;
                reinterpret_cast<uint4 *>(s_qa + (size_t)t * in_f)[b * 16 + (s & 1) * 8 + (s >> 1) * 2 + h] = v;
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
                reinterpret_cast<uint4 *>(s_qa + (size_t)t * in_f)[u] = o;
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
        // consumer-only barrier (named barrier 1, kRows warps)
        asm volatile("bar.sync 1, %0;" ::"r"(kRows * 32) : "memory");

        float acc[M];
        for (int t = 0; t < n_tiles; t++) {
            const int s = t % S, use = t / S;
            const int grp = t / geo.n_slices, ks = t - grp * geo.n_slices;
            if (ks == 0) {
#pragma unroll
                for (int i = 0; i < M; i++) acc[i] = 0.f;
            }
            if (!mbar_wait(smem_u32(bars + s), (uint32_t)(use & 1)) || *(volatile int *)&s_abort) {
                if (lane == 0) {
                    atomicExch(status, 2u);
                    *(volatile int *)&s_abort = 1;
                }
                return;
            }
            const int row = r_begin + grp * kRows + warp;
            const bool live = row < r_begin + r_count;
            const int blk0 = ks * F::kSliceBlocks;
            const int nblk = min(F::kSliceBlocks, nb - blk0);
            if (live) {
                const size_t start = (size_t)W + (size_t)row * row_bytes + (size_t)blk0 * F::kBlockBytes;
                const uint8_t *sl = ring + ((size_t)s * kRows + warp) * geo.slot_bytes + (start & 15);
                if (DT == DT_Q4K)
                    slice_q4k<M>(sl, nblk, blk0, nb, in_f, s_qa, s_d, s_bs, lane, acc);
                else if (DT == DT_Q6K)
                    slice_q6k<M>(sl, nblk, blk0, nb, in_f, s_qa, s_d, s_bs, lane, acc);
                else
                    slice_q2_0<M>(sl, nblk, blk0, nb, in_f, s_qa, s_d, s_bs, lane, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(bars + S + s));
            if (live && ks == geo.n_slices - 1) {
#pragma unroll
                for (int i = 0; i < M; i++) {
                    const float v = warp_sum(acc[i]);
                    if (lane == 0 && i < m) y[(size_t)i * out_f + row] = v;
                }
            }
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
    const size_t codes = DT == DT_Q6K ? (size_t)M * ((geo.nb + 1) / 2 * 512) : (size_t)M * in_f;
    const size_t acts = codes + (size_t)M * (in_f / a.gran) * 4 + (size_t)M * (DT == DT_Q6K ? in_f / 16 : in_f / 32) * 4;
    geo.act_bytes = (uint32_t)((acts + 15) / 16 * 16);
    // ring budget: leave room for a second CTA (the next kernel, launched early) on the same SM
    const size_t budget = (size_t)dev.max_smem_optin / 2 - 2048;
    if (geo.act_bytes + 64 + 2 * (size_t)kRows * geo.slot_bytes > (size_t)dev.max_smem_optin - 1024) return cudaErrorInvalidValue;
    size_t ring_budget = budget > geo.act_bytes ? budget - geo.act_bytes : 0;
    int stages = (int)(ring_budget / ((size_t)kRows * geo.slot_bytes));
    if (stages < 2) stages = 2;
    if (stages > 8) stages = 8;
    geo.stages = stages;
    const size_t smem = (size_t)stages * kRows * geo.slot_bytes + geo.act_bytes + 2 * stages * 8 + 16;
    int grid = (out_f + kRows - 1) / kRows;
    if (grid > dev.sm_count) grid = dev.sm_count;
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
    if (m == 1) return launch_stream_m<1>(dt, w, a, y, m, in_f, out_f, dev, status, st);
    if (m == 2) return launch_stream_m<2>(dt, w, a, y, m, in_f, out_f, dev, status, st);
    if (m <= 4) return launch_stream_m<4>(dt, w, a, y, m, in_f, out_f, dev, status, st);
    return launch_stream_m<8>(dt, w, a, y, m, in_f, out_f, dev, status, st);
}

}  // namespace infr
