// Q4_K decode GEMV for one activation row (m = 1), built around the launch-to-launch pipeline of a decode step.
//
// y[out_f] = x[in_f] * W^T with the production infr-cpu arithmetic (crates/infr-cpu/src/kernels.rs:151-184): per
// 256-element super-block  sd = sum_s sc_s * (sum_i q4_si * q8_si),  sm = sum_s m_s * bsum_s  in exact integer
// arithmetic, y += d8 * (d * sd - dmin * sm).
//
// A decode GEMV is a few microseconds of HBM streaming between two kernels that depend on each other, so what a
// launch costs is decided by what can happen BEFORE the previous kernel has finished:
//  * One CTA per SM that takes less than half of the SM (shared memory, threads, registers): the next GEMV of the
//    stream, started early by programmatic dependent launch, is resident beside this one and has its own weights in
//    flight while this one computes.
//  * A CTA owns a contiguous, balanced range of output rows — one contiguous byte range of W — and a control warp
//    streams it through a ring of shared-memory slots with 1-D bulk copies (cp.async.bulk; no tensor map, any
//    16-byte-aligned weight pointer), all of it issued before `griddepcontrol.wait`.
//  * The 16 compute warps split K: warp c owns super-block columns c, c + kw, ... of every row, a lane owns one
//    16-byte piece of such a block (8 lanes per block, 4 rows per warp step).  A lane's activation words therefore
//    never change: they are loaded ONCE into registers straight from global memory (one round trip, no staging in
//    shared memory, no CTA barrier), and the inner loop reads shared memory only for weights.
//  * Activations that were NOT written by the launch just before this one (the k and v projections after q, up
//    after gate, a batch of matrices against one input) may be read, and multiplied, before the wait; the host
//    tracks which buffers the previous launch wrote and picks that variant (`early_acts`).  It is legal only when
//    the previous kernel triggered its dependents AFTER its own wait (`late_trigger`), because then everything older
//    than the previous launch is complete and visible when this kernel starts; kernels launched in that variant
//    trigger late themselves, and results are stored only after the wait.
// Partial sums of the K split meet in shared memory once per batch of rows and are added in a fixed order, so the
// result does not depend on timing.  All waits are bounded; on expiry a status word is set for the host, the warps
// stop consuming, copies in flight are given time to land and the CTA leaves.
#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kCW = 16;                      // compute warps
constexpr int kRowsThreads = (kCW + 1) * 32;  // + the control warp
constexpr int kMaxRowSlots = 12;
constexpr int kBatchRows = 64;               // rows per cross-warp reduction
constexpr uint32_t kRowsSpin = 1u << 22;

__device__ __forceinline__ uint32_t r_su32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool r_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool r_wait(uint32_t bar, uint32_t parity, volatile int *dead, uint32_t limit = kRowsSpin) {
    for (uint32_t i = 0; i < limit; i++) {
        if (r_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *dead) return false;
    }
    return false;
}

struct RowsGeom {
    int nb;           // super-blocks per row
    int kw;           // warps that split K (a power of two <= 16); 16 / kw row groups work on different rows
    int step_rows;    // rows per ring slot = 4 * (16 / kw)
    int slots;        // ring depth
    uint32_t slot_bytes;
};

// NPOS = super-block columns per warp (ceil(nb / kw)); LATE = trigger dependents after the wait; EARLY = activations
// may be read before the wait (implies LATE).
template <int NPOS, bool LATE, bool EARLY>
__global__ void __launch_bounds__(kRowsThreads, 2)
    gemv_q4k_rows_kernel(const uint8_t *__restrict__ W, Q8Dev a, float *__restrict__ y, int in_f, int out_f, RowsGeom geo,
                         uint32_t *__restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = geo.nb, S = geo.slots, kw = geo.kw, step_rows = geo.step_rows;
    uint8_t *ring = smem;                                                            // [S][slot_bytes]
    float *part = reinterpret_cast<float *>(smem + (size_t)S * geo.slot_bytes);       // [2][kw][kBatchRows]
    uint64_t *bars = reinterpret_cast<uint64_t *>(part + 2 * kCW * kBatchRows);       // full[S], empty[S], dep
    __shared__ int s_dead;
    volatile int *dead = &s_dead;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto full = [&](int s) { return r_su32(bars + s); };
    auto empty = [&](int s) { return r_su32(bars + kMaxRowSlots + s); };
    const uint32_t dep = r_su32(bars + 2 * kMaxRowSlots);
    if (threadIdx.x == 0) {
        s_dead = 0;
        for (int s = 0; s < S; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full(s)), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty(s)), "r"(kCW) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dep), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // balanced contiguous row range of this CTA
    const int G = gridDim.x, base = out_f / G, rem = out_f % G;
    const int r_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int r_count = base + (blockIdx.x < rem ? 1 : 0);
    const int n_steps = (r_count + step_rows - 1) / step_rows;
    const size_t row_bytes = (size_t)nb * 144;

    if (warp == kCW) {
        // ------------------------------------------------------------------ control warp: copies and the dependency
        if (lane == 0) {
            auto issue = [&](int step) {
                const int slot = step % S, r0 = step * step_rows;
                const uint32_t bytes = (uint32_t)((size_t)min(step_rows, r_count - r0) * row_bytes);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full(slot)), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 r_su32(ring + (size_t)slot * geo.slot_bytes)),
                             "l"(W + (size_t)(r_begin + r0) * row_bytes), "r"(bytes), "r"(full(slot))
                             : "memory");
            };
            int issued = 0;
            for (; issued < S && issued < n_steps; issued++) issue(issued);
            if (!LATE) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (LATE) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dep) : "memory");
            bool ok = true;
            for (; issued < n_steps && ok; issued++) {
                const int slot = issued % S;
                // every compute warp has finished with the slot's previous rows
                ok = r_wait(empty(slot), (uint32_t)((issued / S - 1) & 1), dead);
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue(issued);
            }
            if (!ok) {
                if (!*dead) atomicExch(status, 8u);
                *dead = 1;
            }
            if (*dead)  // copies still in flight must land before the CTA's shared memory is released
                for (int k = issued > S ? issued - S : 0; k < issued; k++)
                    for (uint32_t i = 0; i < (1u << 16) && !r_try(full(k % S), (uint32_t)((k / S) & 1)); i++) {
                    }
        }
        return;
    }

    // ---------------------------------------------------------------------- compute warps
    const int cg = warp % kw, rg = warp / kw;   // K column group, row group
    const int g = lane >> 3, j = lane & 7;      // row inside the warp step, 16-byte piece of the block's nibbles
    const int p = j >> 1, h = j & 1;            // sub-block pair (2p, 2p+1), half of its elements
    // byte selectors: scales of sub-blocks 2p, 2p+1 and min j inside the packed words of k4_all
    const uint32_t sel_lo = 0x4440u + (uint32_t)(2 * (p & 1)), sel_hi = sel_lo + 1u, sel_m = 0x4440u + (uint32_t)(j & 3);
    const bool hi_words = p >= 2, hi_min = j >= 4;

    // this lane's activations: elements [16h, 16h+16) of sub-blocks 2p and 2p+1 of every column the warp owns
    uint32_t xl[NPOS][4], xh[NPOS][4];
    float d8[NPOS];
    int bs[NPOS];
    auto load_acts = [&]() {
#pragma unroll
        for (int q = 0; q < NPOS; q++) {
            const int b = cg + q * kw;
            uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
            d8[q] = 0.f;
            bs[q] = 0;
            if (b < nb) {
                const int8_t *xp = a.qs + (size_t)b * 256 + p * 64 + h * 16;
                v0 = __ldcg(reinterpret_cast<const uint4 *>(xp));
                v1 = __ldcg(reinterpret_cast<const uint4 *>(xp + 32));
                d8[q] = __ldcg(a.d + b);
                bs[q] = __ldcg(a.sums + b * 8 + j);
            }
            xl[q][0] = v0.x, xl[q][1] = v0.y, xl[q][2] = v0.z, xl[q][3] = v0.w;
            xh[q][0] = v1.x, xh[q][1] = v1.y, xh[q][2] = v1.z, xh[q][3] = v1.w;
        }
    };
    bool dep_seen = false;
    bool gone = false;  // warp-uniform: a wait expired somewhere in the CTA
    auto wait_dep = [&]() {
        if (dep_seen) return;
        if (!r_wait(dep, 0u, dead)) {
            if (lane == 0 && !*dead) atomicExch(status, 9u);
            *dead = 1;
            gone = true;
        }
        dep_seen = true;
    };
    if (!EARLY) wait_dep();
    load_acts();

    int batch = 0, row_in_batch0 = 0;  // rows of the CTA before the current step, inside the current batch
    for (int step = 0; step < n_steps; step++) {
        const int slot = step % S;
        if (!gone && !r_wait(full(slot), (uint32_t)((step / S) & 1), dead)) {
            if (lane == 0 && !*dead) atomicExch(status, 3u);
            *dead = 1;
            gone = true;
        }
        const int rloc = step * step_rows + rg * 4 + g;  // row inside the CTA's range
        float accf = 0.f;
        if (!gone && rloc < r_count) {
            const uint8_t *rowp = ring + (size_t)slot * geo.slot_bytes + (size_t)(rg * 4 + g) * row_bytes;
#pragma unroll
            for (int q = 0; q < NPOS; q++) {
                const int b = cg + q * kw;
                if (b < nb) {
                    const uint8_t *blk = rowp + (size_t)b * 144;
                    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
                    const uint4 w = *reinterpret_cast<const uint4 *>(blk + 16 + j * 16);
                    // get_scale_min_k4 (crates/infr-gguf/src/dequant.rs:73-83) on packed bytes
                    const uint32_t sc03 = hdr.y & 0x3F3F3F3Fu, mn03 = hdr.z & 0x3F3F3F3Fu;
                    const uint32_t sc47 = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                    const uint32_t mn47 = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                    const uint32_t scw = hi_words ? sc47 : sc03, mw = hi_min ? mn47 : mn03;
                    const int sc_lo = (int)__byte_perm(scw, 0, sel_lo), sc_hi = (int)__byte_perm(scw, 0, sel_hi);
                    const int mj = (int)__byte_perm(mw, 0, sel_m);
                    int ilo = 0, ihi = 0;  // ihi carries the high nibbles unshifted: 16 x the sum
                    ilo = dp4a_us(w.x & 0x0F0F0F0Fu, (int)xl[q][0], ilo);
                    ihi = dp4a_us(w.x & 0xF0F0F0F0u, (int)xh[q][0], ihi);
                    ilo = dp4a_us(w.y & 0x0F0F0F0Fu, (int)xl[q][1], ilo);
                    ihi = dp4a_us(w.y & 0xF0F0F0F0u, (int)xh[q][1], ihi);
                    ilo = dp4a_us(w.z & 0x0F0F0F0Fu, (int)xl[q][2], ilo);
                    ihi = dp4a_us(w.z & 0xF0F0F0F0u, (int)xh[q][2], ihi);
                    ilo = dp4a_us(w.w & 0x0F0F0F0Fu, (int)xl[q][3], ilo);
                    ihi = dp4a_us(w.w & 0xF0F0F0F0u, (int)xh[q][3], ihi);
                    const int sd16 = (sc_lo * 16) * ilo + sc_hi * ihi;  // 16 x this lane's share of sd (exact)
                    const int sm = mj * bs[q];                         // this lane's term of sm
                    const float dw = h2f(hdr.x) * 0.0625f, dminw = h2f(hdr.x >> 16);
                    accf = fmaf(d8[q], dw * (float)sd16 - dminw * (float)sm, accf);
                }
            }
        }
        // the eight lanes of a row
        accf += __shfl_xor_sync(0xffffffffu, accf, 1);
        accf += __shfl_xor_sync(0xffffffffu, accf, 2);
        accf += __shfl_xor_sync(0xffffffffu, accf, 4);
        float *pb = part + (size_t)(batch & 1) * kCW * kBatchRows + (size_t)cg * kBatchRows;
        if (j == 0) pb[row_in_batch0 + rg * 4 + g] = accf;
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty(slot)) : "memory");
        row_in_batch0 += step_rows;
        if (row_in_batch0 == kBatchRows || step == n_steps - 1) {
            // the K split meets: every row of the batch is the sum of kw partial sums, added in column-group order
            asm volatile("bar.sync 1, %0;" ::"r"(kCW * 32) : "memory");
            if (EARLY) wait_dep();  // results may be stored only once the previous kernel is complete
            const int t = threadIdx.x;
            const int rl = batch * kBatchRows + t;
            if (t < row_in_batch0 && rl < r_count && !*dead) {
                const float *pp = part + (size_t)(batch & 1) * kCW * kBatchRows + t;
                float v = 0.f;
                for (int c = 0; c < kw; c++) v += pp[(size_t)c * kBatchRows];
                y[r_begin + rl] = v;
            }
            batch++;
            row_in_batch0 = 0;
        }
    }
}

template <int NPOS, bool LATE, bool EARLY>
cudaError_t launch_rows_cfg(const uint8_t *w, const Q8Dev &a, float *y, int in_f, int out_f, const DeviceInfo &dev, uint32_t *status,
                            cudaStream_t st, RowsGeom geo, size_t smem, int grid) {
    auto kernel = gemv_q4k_rows_kernel<NPOS, LATE, EARLY>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kRowsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, w, a, y, in_f, out_f, geo, status);
}

template <int NPOS>
cudaError_t launch_rows_npos(int mode, const uint8_t *w, const Q8Dev &a, float *y, int in_f, int out_f, const DeviceInfo &dev,
                             uint32_t *status, cudaStream_t st, RowsGeom geo, size_t smem, int grid) {
    if (mode == 2) return launch_rows_cfg<NPOS, true, true>(w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
    if (mode == 1) return launch_rows_cfg<NPOS, true, false>(w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
    return launch_rows_cfg<NPOS, false, false>(w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
}

}  // namespace

// mode 0: activations come from the previous launch (dependents triggered at once, activations read after the wait);
// mode 1: the same reads, dependents triggered after the wait (the next launch may then read older data early);
// mode 2: activations are older than the previous launch, which triggered late: read and multiply before the wait.
// cudaErrorInvalidValue = shape not taken (the caller uses another kernel).
cudaError_t launch_gemv_q4k_rows(const uint8_t *w, const Q8Dev &a, float *y, int in_f, int out_f, int mode, const DeviceInfo &dev,
                                 uint32_t *status, cudaStream_t st) {
    if (in_f <= 0 || in_f % 256 || out_f < 1 || a.gran != 256) return cudaErrorInvalidValue;
    if (((uintptr_t)w % 16) || ((uintptr_t)a.qs % 16)) return cudaErrorInvalidValue;
    RowsGeom geo;
    geo.nb = in_f / 256;
    int kw = 1;
    while (kw * 2 <= geo.nb && kw < kCW) kw *= 2;
    geo.kw = kw;
    const int npos = (geo.nb + kw - 1) / kw;
    if (npos > 4) return cudaErrorInvalidValue;
    geo.step_rows = 4 * (kCW / kw);
    geo.slot_bytes = (uint32_t)((size_t)geo.step_rows * geo.nb * 144);
    const size_t fixed = (size_t)2 * kCW * kBatchRows * 4 + (size_t)(2 * kMaxRowSlots + 1) * 8 + 64;
    // less than half of the SM, so that the next launch is resident beside this one
    const size_t budget = (size_t)dev.max_smem_optin / 2 - 4096;
    if (fixed + 2 * (size_t)geo.slot_bytes > budget) return cudaErrorInvalidValue;
    int slots = (int)((budget - fixed) / geo.slot_bytes);
    if (slots > kMaxRowSlots) slots = kMaxRowSlots;
    geo.slots = slots;
    const size_t smem = fixed + (size_t)slots * geo.slot_bytes;
    int grid = (out_f + geo.step_rows - 1) / geo.step_rows;
    if (grid > dev.sm_count) grid = dev.sm_count;
    switch (npos) {
    case 1: return launch_rows_npos<1>(mode, w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
    case 2: return launch_rows_npos<2>(mode, w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
    case 3: return launch_rows_npos<3>(mode, w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
    default: return launch_rows_npos<4>(mode, w, a, y, in_f, out_f, dev, status, st, geo, smem, grid);
    }
}

}  // namespace infr
