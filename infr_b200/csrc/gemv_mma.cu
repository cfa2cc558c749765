// Q4_K decode GEMV / small-batch GEMM (m <= 8) on the warp-level int8 matrix unit.
//
// y[m,out_f] = x[m,in_f] * W^T with the production infr-cpu arithmetic
// (crates/infr-cpu/src/kernels.rs:151-184): per 256-element super-block
//     sd = sum_s sc_s * (sum_i q4_si * q8_si)      sm = sum_s m_s * bsum_s        (exact int32)
//     y += d8 * (d * float(sd) - dmin * float(sm))
//
// Why a matrix instruction for a matvec: the kernel is HBM-bound only if the SM can unpack 23 bytes
// of 4-bit weights per clock, and with scalar byte dot products the instruction stream (mask, dot,
// scale, reduce) needs more issue slots than an SM has.  `mma.sync.m16n8k32.u8.s8` takes 16 weight
// rows x 32 K per instruction and the 8 columns hold up to 8 activation rows, so the per-byte
// instruction count roughly halves and batch 1..8 all cost the same.  The K index of the instruction
// is only a summation index, so each lane feeds it the 8 nibble bytes it can fetch with one 64-bit
// shared-memory read; the activations are staged in shared memory in the matching order.  High
// nibbles are multiplied unshifted (x16) and the int32 result is shifted back, exactly.  The min term
// sm is one more instruction per half: A = the 8 min bytes, B = bsum split as 64*h + l (both int8).
//
// Data movement: weights go HBM -> shared memory by tiled TMA (cp.async.bulk.tensor.2d over a tensor
// map of the weight matrix viewed as [rows][row_bytes/4] 32-bit words; one instruction fetches the
// 16-row x K-step box of a ring slot, rows past the end of the matrix are zero-filled) into
// warp-private rings; a CTA owns a contiguous balanced row range, walks it 16 rows at a time and
// its 8 warps split K.  Partial sums meet in shared memory once per 16 rows in a fixed order (the
// result does not depend on timing).  Programmatic dependent launch: weights are prefetched before
// `griddepcontrol.wait`; only the activation staging waits for the previous kernel.
//
// When `x` is given instead of pre-quantised activations the CTA quantises the rows itself while the
// first weights are in flight (same arithmetic as quantize.cu, so the same bits), which makes a
// quantized Linear a single kernel.
//
// All mbarrier waits are bounded; an expired wait records a status word for the host and the warp
// stops consuming (the block still reaches its barriers, results of the launch are invalid).
#include <cuda.h>

#include <cstring>

#include "gemv_common.cuh"
#include "q8_code.cuh"

namespace infr {
namespace {

constexpr int kTileRows = 16;
constexpr int kMaxSlotsMma = 4;
constexpr int kLaneBytes = 80;               // staged codes of one K lane of a super-block (64 + 16: distinct banks for 128-bit reads)
constexpr int kStagedBytes = 4 * kLaneBytes;  // staged codes of one super-block of one token
constexpr uint32_t kSpin = 1u << 22;

__device__ __forceinline__ uint32_t s_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpin; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// Tiled TMA load of one box: x = word offset inside the row (a multiple of 4 -> 16-byte aligned), y = row; `policy` is
// an L2 eviction-priority hint.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
                 : "memory");
}
// D = A(16x32, u8) * B(32x8, s8), int32, zero accumulator input.
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// All eight (scale, min) pairs of a Q4_K header as bytes (get_scale_min_k4,
// crates/infr-gguf/src/dequant.rs:73-83): sc[0] = scales 0..3, sc[1] = 4..7, likewise mn.
__device__ __forceinline__ void k4_all(uint32_t y, uint32_t z, uint32_t w, uint32_t (&sc)[2], uint32_t (&mn)[2]) {
    sc[0] = y & 0x3F3F3F3Fu;
    mn[0] = z & 0x3F3F3F3Fu;
    sc[1] = (w & 0x0F0F0F0Fu) | ((y >> 2) & 0x30303030u);
    mn[1] = ((w >> 4) & 0x0F0F0F0Fu) | ((z >> 2) & 0x30303030u);
}


struct MmaGeom {
    int nb;         // super-blocks per row
    int bpw;        // super-blocks per warp (K split)
    int slots;      // ring slots per warp
    int act_bytes;  // staged activation bytes
};

// Grouped (mixture-of-experts) mode: blockIdx.y walks a device-built list of work items, each up to 8
// activation rows routed to one expert.  The weight bank holds the experts' matrices back to back, so
// expert e's rows start at e * out_f of the tensor map.  item_* == nullptr means an ordinary GEMV.
struct MmaGroup {
    const int *item_expert;  // [n_items] expert of the item
    const int *item_p0;      // [n_items] first routed pair of the item
    const int *item_cnt;     // [n_items] pairs in the item (1..8)
    const int *n_items;      // device scalar
    const int *pair_row;     // [n_pairs] activation row of each pair, or nullptr: pair p reads row p
};

// A second matrix with the same in_f and the same activations, multiplied in the same launch (the q and k
// projections, gate and up): its 16-row tiles follow the first matrix's in the CTAs' tile ranges.  out_f == 0: none.
struct MmaSecond {
    CUtensorMap map;
    float *y;
    int out_f;
};

// quantize_q8 (crates/infr-cpu/src/quant.rs:27-58) of NK 256-element blocks held by one warp (item K0 + k of the
// fetched set: lane l owns elements 8l..8l+7 of it), all NK worked on together phase by phase; the codes, the split
// sums and the scale go to the staged layout described below.  Item i = i0 + (K0 + k) * kw is token i / nb, block i % nb.
template <int NK, int K0>
__device__ __forceinline__ void quant_items(const float4 (&pa)[4], const float4 (&pb)[4], int i0, int kw, int nb, int lane, uint8_t *s_codes,
                                            uint8_t *s_bsplit, float *s_d8) {
    float am[NK], dd[NK], id[NK];
#pragma unroll
    for (int k = 0; k < NK; k++) {
        const float4 v0 = pa[K0 + k], v1 = pb[K0 + k];
        am[k] = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                      fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int k = 0; k < NK; k++) am[k] = fmaxf(am[k], __shfl_xor_sync(0xffffffffu, am[k], o));
    }
#pragma unroll
    for (int k = 0; k < NK; k++) {
        dd[k] = am[k] / 127.0f;
        id[k] = dd[k] > 0.0f ? 1.0f / dd[k] : 0.0f;
    }
    uint2 pk[NK];
    int sum[NK];
#pragma unroll
    for (int k = 0; k < NK; k++) {
        const float vv[8] = {pa[K0 + k].x, pa[K0 + k].y, pa[K0 + k].z, pa[K0 + k].w, pb[K0 + k].x, pb[K0 + k].y, pb[K0 + k].z, pb[K0 + k].w};
        int q[8];
        if (id[k] <= 3.0e38f) {  // (warp-uniform) the usual case: a finite scale, no clamp needed
#pragma unroll
            for (int e = 0; e < 8; e++) q[e] = q8_round_code_inrange(vv[e], id[k]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++) q[e] = q8_round_code(vv[e], id[k]);
        }
        pk[k].x = q8_pack4(q[0], q[1], q[2], q[3]);
        pk[k].y = q8_pack4(q[4], q[5], q[6], q[7]);
        sum[k] = q8_sum4(pk[k].x) + q8_sum4(pk[k].y);
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
#pragma unroll
        for (int k = 0; k < NK; k++) sum[k] += __shfl_xor_sync(0xffffffffu, sum[k], o);
    }
    // lane holds elements 8*lane..8*lane+7 = sub-block s = lane/4, l = 8*(lane&3)+e
    const int s = lane >> 2, tt = lane & 3;
#pragma unroll
    for (int k = 0; k < NK; k++) {
        const int i = i0 + (K0 + k) * kw, n = i / nb, b = i - n * nb;
        *reinterpret_cast<uint2 *>(s_codes + (size_t)(n * nb + b) * kStagedBytes + tt * kLaneBytes + s * 8) = pk[k];
        if (tt == 0) {
            s_bsplit[(size_t)(n * nb + b) * 16 + s] = (uint8_t)(sum[k] & 63);
            s_bsplit[(size_t)(n * nb + b) * 16 + 8 + s] = (uint8_t)(int8_t)(sum[k] >> 6);
        }
        if (lane == 0) s_d8[b * 8 + n] = dd[k];
    }
}

// Shared-memory layout of the staged activations, per token n (0..7) and super-block b:
//   codes  : 320 B at (n*nb + b)*320, element (sub-block s, l = 8t+i) at t*80 + s*8 + i
//   bsplit : 16 B at (n*nb + b)*16: bytes 0..7 = low 6 bits of bsum_s, bytes 8..15 = bsum_s >> 6
//   d8     : float [b][8 tokens], zero for absent tokens (a lane's two result columns are neighbours)
// KW = warps per CTA (they split K), SB = super-blocks per ring slot per row.
template <int M, bool FUSED, int KW, int SB, bool PUSH>
__global__ void __launch_bounds__(KW * 32, 16 / KW)
    gemv_q4k_mma_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ MmaSecond sec, Q8Dev a,
                        const float *__restrict__ x, float *__restrict__ y, int m, int in_f, int out_f, MmaGeom geo, MmaGroup grp,
                        uint32_t *__restrict__ status, const __grid_constant__ typename PushParam<PUSH>::type push) {
    constexpr int kW = KW, kThreadsMma = KW * 32, kStepBlocks = SB, kSlotBytes = kTileRows * SB * 144;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = geo.nb, S = geo.slots;
    uint8_t *rings = smem;                                         // [kW][S][kSlotBytes]
    uint8_t *s_codes = smem + (size_t)kW * S * kSlotBytes;         // [M][nb][256]
    uint8_t *s_bsplit = s_codes + (size_t)M * nb * kStagedBytes;   // [M][nb][16]
    float *s_d8 = reinterpret_cast<float *>(s_bsplit + (size_t)M * nb * 16);  // [nb][8]
    float *s_part = s_d8 + (size_t)nb * 8;                         // [2][kW][16][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_part + 2 * kW * 128);  // [kW][kMaxSlotsMma]
    __shared__ int s_bad;
    __shared__ uint32_t s_epoch;  // push mode: exchanges completed before this launch

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        s_bad = 0;
        for (int i = 0; i < kW * kMaxSlotsMma; i++) bar_init(s_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int row_base = 0, p0 = 0;  // grouped mode: first row of the expert in the bank, first pair of the item
    if (grp.item_expert) {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the work list comes from the previous kernels
        const int item = blockIdx.y;
        if (item >= *grp.n_items) return;
        row_base = grp.item_expert[item] * out_f;
        p0 = grp.item_p0[item];
        m = grp.item_cnt[item];
    }

    // balanced contiguous range of 16-row tiles of this CTA (only the matrix's last tile can be partial)
    const int tiles1 = (out_f + kTileRows - 1) / kTileRows;  // tiles of the first matrix; the second's follow
    const int total_tiles = tiles1 + (sec.out_f + kTileRows - 1) / kTileRows;
    const int G = gridDim.x, base = total_tiles / G, rem = total_tiles % G;
    const int t_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
    const int n_tiles = base + (blockIdx.x < rem ? 1 : 0);
    // this warp's K range
    const int kb0 = warp * geo.bpw;
    const int kb1 = min(nb, kb0 + geo.bpw);
    const int my_blocks = max(0, kb1 - kb0);
    const int steps_per_tile = (my_blocks + kStepBlocks - 1) / kStepBlocks;
    const int n_jobs = n_tiles * steps_per_tile;
    uint8_t *ring = rings + (size_t)warp * S * kSlotBytes;
    uint64_t *wbar = bars + warp * kMaxSlotsMma;

    // Weights are read once per launch: evict-first keeps them from pushing the activations (a few kilobytes that
    // every CTA of every launch reads) out of L2.
    uint64_t l2_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(l2_policy));
    // ---- issue side: one elected lane fetches the 16-row x K-step box of the slot ----
    int j_issue = 0, i_tile = 0, i_step = 0;
    auto issue = [&](int slot) {
        if (j_issue >= n_jobs) return;
        if (lane == 0) {
            const int blk0 = kb0 + i_step * kStepBlocks;
            const uint32_t bar = s_u32(wbar + slot);
            // order this warp's earlier reads of the slot before the engine overwrites it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            bar_expect_tx(bar, (uint32_t)kSlotBytes);
            const int T = t_begin + i_tile;
            if (T < tiles1)
                tma_load_2d_hint(s_u32(ring + (size_t)slot * kSlotBytes), &tmap, blk0 * 36, row_base + T * kTileRows, bar, l2_policy);
            else
                tma_load_2d_hint(s_u32(ring + (size_t)slot * kSlotBytes), &sec.map, blk0 * 36, (T - tiles1) * kTileRows, bar, l2_policy);
        }
        __syncwarp();
        j_issue++;
        if (++i_step == steps_per_tile) {
            i_step = 0;
            i_tile++;
        }
    };
    for (int s = 0; s < S; s++) issue(s);

    // ---- activations (from the previous kernel in the stream) ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (PUSH) {
        if (threadIdx.x == 0) s_epoch = *reinterpret_cast<const volatile uint32_t *>(push.ctrl);  // read by all after the barrier below
    }
    if (M < 8)  // scale columns of tokens the template does not stage
        for (int i = threadIdx.x; i < nb * 8; i += kThreadsMma)
            if ((i & 7) >= M) s_d8[i] = 0.f;
    if (FUSED) {
        // quantize_q8 (crates/infr-cpu/src/quant.rs:27-58) per 256-block, one warp per (row, block) item.  A warp
        // fetches up to four of its items before it works on the first, so the fetches share one round trip to L2.
        const int items = M * nb;
        for (int i0 = warp; i0 < items; i0 += 4 * kW) {
            float4 pa[4], pb[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = i0 + k * kW, n = i / nb, b = i - n * nb;
                pa[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                pb[k] = pa[k];
                if (i < items && n < m) {
                    const float *xp = x + (size_t)n * in_f + (size_t)b * 256;
                    pa[k] = *reinterpret_cast<const float4 *>(xp + lane * 8);
                    pb[k] = *reinterpret_cast<const float4 *>(xp + lane * 8 + 4);
                }
            }
            // Items are worked on together, phase by phase (all maxima, then all reductions, ...), so that their
            // dependent chains overlap: shuffles, two divisions and eight roundings per item are latency, not work.
            const int left = (items - i0 + kW - 1) / kW;  // items of this warp from i0 on (warp-uniform)
            if (left >= 4) {
                quant_items<4, 0>(pa, pb, i0, kW, nb, lane, s_codes, s_bsplit, s_d8);
            } else {
                if (left >= 2) quant_items<2, 0>(pa, pb, i0, kW, nb, lane, s_codes, s_bsplit, s_d8);
                if (left == 3) quant_items<1, 2>(pa, pb, i0, kW, nb, lane, s_codes, s_bsplit, s_d8);
                if (left == 1) quant_items<1, 0>(pa, pb, i0, kW, nb, lane, s_codes, s_bsplit, s_d8);
            }
        }
    } else {
        if (M == 1) {
            // One row.  Every global load of a thread is issued before its first shared-memory store (the compiler
            // may not move a load of a generic pointer across such a store), so the staging costs one round trip to
            // L2 instead of one per loop.
            const size_t ar = (size_t)(grp.pair_row ? grp.pair_row[p0] : p0);
            const int units = in_f / 8;
            const int8_t *qrow = a.qs + ar * in_f;
            const int32_t *srow = a.sums + ar * nb * 8;
            const float *drow = a.d + ar * nb;
            const int tid = threadIdx.x;
            const int sum0 = tid < nb * 8 ? srow[tid] : 0;
            const float d0 = tid < nb ? drow[tid] : 0.f;
            for (int u0 = tid; u0 < units; u0 += 4 * kThreadsMma) {
                uint2 v[4];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int u = u0 + k * kThreadsMma;
                    v[k] = make_uint2(0, 0);
                    if (u < units) v[k] = *reinterpret_cast<const uint2 *>(qrow + (size_t)u * 8);
                }
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int u = u0 + k * kThreadsMma;
                    const int b = u >> 5, uu = u & 31, s = uu >> 2, tt = uu & 3;
                    if (u < units) *reinterpret_cast<uint2 *>(s_codes + (size_t)b * kStagedBytes + tt * kLaneBytes + s * 8) = v[k];
                }
            }
            if (tid < nb * 8) {
                const int b = tid >> 3, s = tid & 7;
                s_bsplit[(size_t)b * 16 + s] = (uint8_t)(sum0 & 63);
                s_bsplit[(size_t)b * 16 + 8 + s] = (uint8_t)(int8_t)(sum0 >> 6);
            }
            if (tid < nb) s_d8[tid * 8] = d0;
            for (int r = tid + kThreadsMma; r < nb * 8; r += kThreadsMma) {
                const int b = r >> 3, s = r & 7, sum = srow[r];
                s_bsplit[(size_t)b * 16 + s] = (uint8_t)(sum & 63);
                s_bsplit[(size_t)b * 16 + 8 + s] = (uint8_t)(int8_t)(sum >> 6);
            }
            for (int b = tid + kThreadsMma; b < nb; b += kThreadsMma) s_d8[b * 8] = drow[b];
        } else {
        // activation row of column n: the item's n-th pair (gathered through pair_row when given)
        __shared__ uint32_t s_row[8];
        if (threadIdx.x < 8) s_row[threadIdx.x] = threadIdx.x < m ? (uint32_t)(grp.pair_row ? grp.pair_row[p0 + threadIdx.x] : p0 + threadIdx.x) : 0u;
        __syncthreads();
        // eight independent 8-byte loads in flight per thread: the copy is latency-bound, not bandwidth-bound
        // (flattened over tokens and units: with one token's few hundred units per pass most of the loads would be masked)
        const int units = in_f / 8, total = M * units;
        for (int i0 = threadIdx.x; i0 < total; i0 += 8 * kThreadsMma) {
            uint2 v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = i0 + k * kThreadsMma, n = i / units, u = i - n * units;
                v[k] = make_uint2(0, 0);
                if (i < total && n < m) v[k] = *reinterpret_cast<const uint2 *>(a.qs + (size_t)s_row[n] * in_f + (size_t)u * 8);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = i0 + k * kThreadsMma, n = i / units, u = i - n * units;
                const int b = u >> 5, uu = u & 31, s = uu >> 2, tt = uu & 3;
                if (i < total) *reinterpret_cast<uint2 *>(s_codes + (size_t)(n * nb + b) * kStagedBytes + tt * kLaneBytes + s * 8) = v[k];
            }
        }
        for (int i = threadIdx.x; i < M * nb * 8; i += kThreadsMma) {
            const int n = i / (nb * 8), r = i - n * nb * 8, b = r >> 3, s = r & 7;
            const int sum = n < m ? a.sums[(size_t)s_row[n] * nb * 8 + r] : 0;
            s_bsplit[(size_t)(n * nb + b) * 16 + s] = (uint8_t)(sum & 63);
            s_bsplit[(size_t)(n * nb + b) * 16 + 8 + s] = (uint8_t)(int8_t)(sum >> 6);
        }
        for (int i = threadIdx.x; i < M * nb; i += kThreadsMma) {
            const int n = i / nb, b = i - n * nb;
            s_d8[b * 8 + n] = n < m ? a.d[(size_t)s_row[n] * nb + b] : 0.f;
        }
        }
    }
    __syncthreads();

    // ---- consume ----
    const int gt = g < M ? g : 0;  // token whose codes this lane feeds as its B column
    int slot = 0, jc = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int tile = 0; tile < n_tiles; tile++) {
        float accf[4] = {0.f, 0.f, 0.f, 0.f};
        for (int step = 0; step < steps_per_tile; step++, jc++) {
            if (!dead && !bar_wait(s_u32(wbar + slot), phase)) {
                dead = true;
                if (lane == 0) {
                    atomicExch(status, 3u);
                    s_bad = 1;
                }
            }
            const int blk0 = kb0 + step * kStepBlocks;
            const int nblk = min(kStepBlocks, kb1 - blk0);
            const uint8_t *sl = ring + (size_t)slot * kSlotBytes;
            if (!dead) {
#pragma unroll
                for (int bl = 0; bl < kStepBlocks; bl++) {
                    if (bl >= nblk) break;
                    const int b = blk0 + bl;
                    const uint8_t *r0 = sl + (size_t)g * (kStepBlocks * 144) + bl * 144;
                    const uint8_t *r1 = r0 + 8 * (kStepBlocks * 144);
                    const uint4 h0 = *reinterpret_cast<const uint4 *>(r0);
                    const uint4 h1 = *reinterpret_cast<const uint4 *>(r1);
                    uint32_t sc0[2], mn0[2], sc1[2], mn1[2];
                    k4_all(h0.y, h0.z, h0.w, sc0, mn0);
                    k4_all(h1.y, h1.z, h1.w, sc1, mn1);
                    // B operands of this block for token g
                    // Output column n depends on B column n only, and columns >= M are never stored, so
                    // lanes of those columns simply re-read token gt; likewise the bsum words of lanes
                    // t >= 2 meet zero A operands.
                    uint32_t bq[16];
                    const uint4 *cp = reinterpret_cast<const uint4 *>(s_codes + (size_t)(gt * nb + b) * kStagedBytes + t * kLaneBytes);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint4 v = cp[i];
                        bq[4 * i] = v.x;
                        bq[4 * i + 1] = v.y;
                        bq[4 * i + 2] = v.z;
                        bq[4 * i + 3] = v.w;
                    }
                    const uint32_t bl_ = *reinterpret_cast<const uint32_t *>(s_bsplit + (size_t)(gt * nb + b) * 16 + (t & 1) * 4);
                    const uint32_t bh_ = *reinterpret_cast<const uint32_t *>(s_bsplit + (size_t)(gt * nb + b) * 16 + 8 + (t & 1) * 4);
                    int sdl[4] = {0, 0, 0, 0}, sdh[4] = {0, 0, 0, 0};  // low / high (x16) nibble sums, scaled
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const uint2 w0 = *reinterpret_cast<const uint2 *>(r0 + 16 + p * 32 + t * 8);
                        const uint2 w1 = *reinterpret_cast<const uint2 *>(r1 + 16 + p * 32 + t * 8);
                        int dlo[4], dhi[4];
                        mma_u8s8(dlo, w0.x & 0x0F0F0F0Fu, w1.x & 0x0F0F0F0Fu, w0.y & 0x0F0F0F0Fu, w1.y & 0x0F0F0F0Fu,
                                 bq[4 * p], bq[4 * p + 1]);
                        mma_u8s8(dhi, w0.x & 0xF0F0F0F0u, w1.x & 0xF0F0F0F0u, w0.y & 0xF0F0F0F0u, w1.y & 0xF0F0F0F0u,
                                 bq[4 * p + 2], bq[4 * p + 3]);
                        // scales of sub-block 2p (low nibbles) and 2p+1 (high nibbles) for rows g and g+8
                        const uint32_t sel = (p & 1) ? 0x4442u : 0x4440u;
                        const int sa_lo = (int)__byte_perm(sc0[p >> 1], 0, sel), sa_hi = (int)__byte_perm(sc0[p >> 1], 0, sel + 1);
                        const int sb_lo = (int)__byte_perm(sc1[p >> 1], 0, sel), sb_hi = (int)__byte_perm(sc1[p >> 1], 0, sel + 1);
                        sdl[0] += sa_lo * dlo[0];
                        sdh[0] += sa_hi * dhi[0];
                        sdl[2] += sb_lo * dlo[2];
                        sdh[2] += sb_hi * dhi[2];
                        if (M > 1) {
                            sdl[1] += sa_lo * dlo[1];
                            sdh[1] += sa_hi * dhi[1];
                            sdl[3] += sb_lo * dlo[3];
                            sdh[3] += sb_hi * dhi[3];
                        }
                    }
                    int sd[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) sd[i] = sdl[i] + (sdh[i] >> 4);  // exact: sdh is a multiple of 16
                    // min term: K slots 0..7 carry the eight m_s (lanes t = 0, 1), the rest are zero
                    int sml[4], smh[4];
                    const uint32_t am0 = t == 0 ? mn0[0] : (t == 1 ? mn0[1] : 0u), am1 = t == 0 ? mn1[0] : (t == 1 ? mn1[1] : 0u);
                    mma_u8s8(sml, am0, am1, 0u, 0u, bl_, 0u);
                    mma_u8s8(smh, am0, am1, 0u, 0u, bh_, 0u);
                    const float d0 = h2f(h0.x), dm0 = h2f(h0.x >> 16), d1 = h2f(h1.x), dm1 = h2f(h1.x >> 16);
                    const float2 e01 = *reinterpret_cast<const float2 *>(s_d8 + b * 8 + 2 * t);
                    const float e0 = e01.x;
                    accf[0] += e0 * (d0 * (float)sd[0] - dm0 * (float)(sml[0] + 64 * smh[0]));
                    accf[2] += e0 * (d1 * (float)sd[2] - dm1 * (float)(sml[2] + 64 * smh[2]));
                    if (M > 1) {
                        const float e1 = e01.y;
                        accf[1] += e1 * (d0 * (float)sd[1] - dm0 * (float)(sml[1] + 64 * smh[1]));
                        accf[3] += e1 * (d1 * (float)sd[3] - dm1 * (float)(sml[3] + 64 * smh[3]));
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
        float *part = s_part + ((size_t)(tile & 1) * kW + warp) * 128;
        part[g * 8 + 2 * t] = accf[0];
        part[g * 8 + 2 * t + 1] = accf[1];
        part[(g + 8) * 8 + 2 * t] = accf[2];
        part[(g + 8) * 8 + 2 * t + 1] = accf[3];
        __syncthreads();
        if (threadIdx.x < kTileRows * 8) {  // 16 rows x 8 token columns; CTAs have at least 128 threads
            const int r = threadIdx.x >> 3, n = threadIdx.x & 7;
            const int T = t_begin + tile;
            const bool second = T >= tiles1;
            const int row = (second ? T - tiles1 : T) * kTileRows + r, of = second ? sec.out_f : out_f;
            if (n < m && row < of) {
                const float *pp = s_part + (size_t)(tile & 1) * kW * 128 + r * 8 + n;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kW; w++) v += pp[w * 128];
                if constexpr (PUSH)
                    push_store(push, s_epoch, (size_t)n * of + row, v);
                else
                    (second ? sec.y : y)[(size_t)(p0 + n) * of + row] = v;
            }
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

template <int M, bool FUSED, int KW, int SB>
cudaError_t launch_mma_cfg(const uint8_t *w, const Q8Dev &a, const float *x, float *y, int m, int in_f, int out_f,
                           const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const MmaGroup &grp = MmaGroup{},
                           int n_experts = 1, int max_items = 1, const uint8_t *w2 = nullptr, float *y2 = nullptr, int out_f2 = 0,
                           const GemvPush *push = nullptr) {
    constexpr int kSlotBytes = kTileRows * SB * 144;
    MmaGeom geo;
    geo.nb = in_f / 256;
    geo.bpw = (geo.nb + KW - 1) / KW;
    const size_t acts = (size_t)M * geo.nb * (kStagedBytes + 16) + (size_t)geo.nb * 32;
    geo.act_bytes = (int)acts;
    const size_t fixed = acts + (size_t)2 * KW * 128 * 4 + (size_t)KW * kMaxSlotsMma * 8 + 64;
    const size_t per_slot = (size_t)KW * kSlotBytes;
    if (fixed + 2 * per_slot > (size_t)dev.max_smem_optin - 1024) return cudaErrorInvalidValue;
    // resident CTAs per SM: 16 math warps in total, each warp with at least two ring slots
    int per_sm = 16 / KW;
    while (per_sm > 1 && fixed + 2 * per_slot > (size_t)dev.max_smem_optin / per_sm - 2048) per_sm /= 2;
    const size_t budget = (size_t)dev.max_smem_optin / per_sm - (per_sm > 1 ? 2048 : 1024);
    int slots = (int)((budget - fixed) / per_slot);
    if (slots > kMaxSlotsMma) slots = kMaxSlotsMma;
    const int all_tiles = (out_f + kTileRows - 1) / kTileRows + (out_f2 + kTileRows - 1) / kTileRows;
    int grid = all_tiles;
    if (grid > dev.sm_count * per_sm) grid = dev.sm_count * per_sm;
    if (!grp.item_expert) {
        // no more ring slots than a warp has jobs: what a small matrix leaves of the SM's shared memory lets the
        // next kernel of the stream become resident, and prefetch its weights, while this one computes
        const int tiles = all_tiles, tiles_cta = (tiles + grid - 1) / grid;
        const int jobs = tiles_cta * ((geo.bpw + SB - 1) / SB);
        if (slots > jobs) slots = jobs < 1 ? 1 : jobs;
    }
    geo.slots = slots;
    const size_t smem = fixed + (size_t)slots * per_slot;
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap tmap;
    MmaSecond sec;
    memset(&sec, 0, sizeof sec);
    auto encode = [&](CUtensorMap *map, const uint8_t *base, cuuint64_t rows) {
        const cuuint64_t gdim[2] = {(cuuint64_t)geo.nb * 36, rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)geo.nb * 144};
        const cuuint32_t box[2] = {(cuuint32_t)SB * 36, (cuuint32_t)kTileRows};
        const cuuint32_t estr[2] = {1, 1};
        return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    if (!encode(&tmap, w, (cuuint64_t)out_f * (cuuint64_t)n_experts)) return cudaErrorInvalidValue;
    if (out_f2 > 0) {
        if (!encode(&sec.map, w2, (cuuint64_t)out_f2)) return cudaErrorInvalidValue;
        sec.y = y2;
        sec.out_f = out_f2;
    }
    // the pushing form exists for pre-quantised rows only
    auto kernel = gemv_q4k_mma_kernel<M, FUSED, KW, SB, false>;
    auto kernel_push = gemv_q4k_mma_kernel<M, false, KW, SB, true>;
    if (push && FUSED) return cudaErrorInvalidValue;
    cudaError_t e = push ? cudaFuncSetAttribute(kernel_push, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    if (grp.item_expert) {
        // many small (expert, 8-row) items: a few CTAs per item, the SMs fill up across items
        const int tiles = (out_f + kTileRows - 1) / kTileRows;
        grid = tiles < 4 ? tiles : 4;
    }
    cfg.gridDim = dim3((unsigned)grid, (unsigned)max_items);
    cfg.blockDim = dim3(KW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (push) return cudaLaunchKernelEx(&cfg, kernel_push, tmap, sec, a, x, y, m, in_f, out_f, geo, grp, status, *push);
    return cudaLaunchKernelEx(&cfg, kernel, tmap, sec, a, x, y, m, in_f, out_f, geo, grp, status, NoPush{});
}

// Few 16-row tiles (small matrices) -> more warps share a tile's K range so that a tile's latency is short;
// many tiles -> four warps per tile and the SM overlaps independent tiles instead.
template <int M, bool FUSED>
cudaError_t launch_mma_m(const uint8_t *w, const Q8Dev &a, const float *x, float *y, int m, int in_f, int out_f,
                         const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const uint8_t *w2 = nullptr, float *y2 = nullptr,
                         int out_f2 = 0, const GemvPush *push = nullptr) {
    const int nb = in_f / 256, tiles = (out_f + kTileRows - 1) / kTileRows + (out_f2 + kTileRows - 1) / kTileRows;
    // shared memory a configuration needs with two ring slots per warp of `sb` super-blocks each
    auto need_sb = [&](int kw, int sb) {
        return (size_t)M * nb * (kStagedBytes + 16) + (size_t)nb * 32 + (size_t)2 * kw * 512 + (size_t)kw * kMaxSlotsMma * 8 + 64 +
               (size_t)2 * kw * kTileRows * sb * 144;
    };
    auto need = [&](int kw) { return need_sb(kw, (nb + kw - 1) / kw == 1 ? 1 : 2); };
    // 16 math warps per SM: with kw warps per tile an SM holds 16/kw tiles at once.  Prefer the widest
    // split that still lets every tile be resident in the first wave.
    const int kw0 = tiles > 2 * dev.sm_count ? 4 : (tiles > dev.sm_count ? 8 : 16);
    int kw = kw0;
    // wide batches stage more activation bytes per CTA: let more warps share one staging copy so that
    // 16 math warps stay resident per SM
    while (kw < 16 && need(kw) > (size_t)dev.max_smem_optin / (16 / kw) - 2048) kw *= 2;
    while (kw > 4 && kw > nb) kw /= 2;
    // long rows with a wide batch may not fit at all with many warps: fall back to fewer
    while (kw > 4 && need(kw) > (size_t)dev.max_smem_optin - 1024) kw /= 2;
    int bpw = (nb + kw - 1) / kw;
    // one CTA of 16 warps per SM pays a 16-warp barrier and reduction per tile for one block of work per warp:
    // with many tiles, two CTAs of 8 warps and one-block ring slots are better when they fit
    if (kw == 16 && kw0 < 16 && nb >= 8 && need_sb(8, 1) <= (size_t)dev.max_smem_optin / 2 - 2048) {
        kw = 8;
        bpw = 1;  // selects SB = 1 below; the kernel walks a warp's blocks one slot at a time
    }
#define INFR_MMA(KW_, SB_) \
    return launch_mma_cfg<M, FUSED, KW_, SB_>(w, a, x, y, m, in_f, out_f, dev, status, st, MmaGroup{}, 1, 1, w2, y2, out_f2, push)
    if (kw == 16) {
        if (bpw == 1) INFR_MMA(16, 1);
        INFR_MMA(16, 2);
    }
    if (kw == 8) {
        if (bpw == 1) INFR_MMA(8, 1);
        INFR_MMA(8, 2);
    }
    if (bpw == 1) INFR_MMA(4, 1);
    INFR_MMA(4, 2);
#undef INFR_MMA
}

template <bool FUSED>
cudaError_t launch_mma(const uint8_t *w, const Q8Dev &a, const float *x, float *y, int m, int in_f, int out_f,
                       const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const uint8_t *w2 = nullptr, float *y2 = nullptr,
                       int out_f2 = 0, const GemvPush *push = nullptr) {
    if (m == 1) return launch_mma_m<1, FUSED>(w, a, x, y, m, in_f, out_f, dev, status, st, w2, y2, out_f2, push);
    if (m == 2) return launch_mma_m<2, FUSED>(w, a, x, y, m, in_f, out_f, dev, status, st, w2, y2, out_f2, push);
    if (m <= 4) return launch_mma_m<4, FUSED>(w, a, x, y, m, in_f, out_f, dev, status, st, w2, y2, out_f2, push);
    return launch_mma_m<8, FUSED>(w, a, x, y, m, in_f, out_f, dev, status, st, w2, y2, out_f2, push);
}

}  // namespace

cudaError_t launch_grouped_q4k_mma(const uint8_t *bank, int n_experts, const Q8Dev &a, float *y, int in_f, int out_f,
                                   const int *item_expert, const int *item_p0, const int *item_cnt, const int *n_items,
                                   const int *pair_row, int max_items, const DeviceInfo &dev, uint32_t *status,
                                   cudaStream_t st) {
    if (in_f % 256 || max_items < 1) return cudaErrorInvalidValue;
    MmaGroup grp{item_expert, item_p0, item_cnt, n_items, pair_row};
    const int nb = in_f / 256;
    // four warps per 16-row tile: an item has few tiles and few K blocks, so the per-tile barrier and
    // reduction are shared by two blocks per warp where the rows are long enough
    if ((nb + 3) / 4 == 1) return launch_mma_cfg<8, false, 4, 1>(bank, a, nullptr, y, 8, in_f, out_f, dev, status, st, grp, n_experts, max_items);
    return launch_mma_cfg<8, false, 4, 2>(bank, a, nullptr, y, 8, in_f, out_f, dev, status, st, grp, n_experts, max_items);
}

// Two Q4_K matrices with the same in_f against the same rows, one launch: pre-quantised rows (a), or f32 rows (x, a null)
// quantised inside the kernel.
cudaError_t launch_gemv_q4k_mma_pair(const uint8_t *w1, float *y1, int out_f1, const uint8_t *w2, float *y2, int out_f2, const Q8Dev *a,
                                     const float *x, int m, int in_f, const DeviceInfo &dev, uint32_t *status, cudaStream_t st) {
    if (m < 1 || m > 8 || in_f % 256 || out_f1 < 1 || out_f2 < 1) return cudaErrorInvalidValue;
    if (a) return launch_mma<false>(w1, *a, nullptr, y1, m, in_f, out_f1, dev, status, st, w2, y2, out_f2);
    Q8Dev none{nullptr, nullptr, nullptr, nullptr, 256};
    return launch_mma<true>(w1, none, x, y1, m, in_f, out_f1, dev, status, st, w2, y2, out_f2);
}

cudaError_t launch_gemv_q4k_mma(const uint8_t *w, const Q8Dev *a, const float *x, float *y, int m, int in_f, int out_f,
                                const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const GemvPush *push) {
    if (m < 1 || m > 8 || in_f % 256) return cudaErrorInvalidValue;
    if (a) return launch_mma<false>(w, *a, nullptr, y, m, in_f, out_f, dev, status, st, nullptr, nullptr, 0, push);
    Q8Dev none{nullptr, nullptr, nullptr, nullptr, 256};
    return launch_mma<true>(w, none, x, y, m, in_f, out_f, dev, status, st, nullptr, nullptr, 0, push);
}

}  // namespace infr
