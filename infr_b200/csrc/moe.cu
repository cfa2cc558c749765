// Mixture-of-experts routing and glue kernels around the grouped expert GEMMs.
//
// Follows the staged Op::MoeFfn of crates/infr-cpu/src/lib.rs:2264-2984 for the qwen3moe family
// (split gate/up banks, softmax gating, top-k by stable descending sort, optional renormalisation,
// SiLU gate, output-side weighting):
//   router logits  : F32 router rows against the raw f32 activations with the reference's `dot`
//                    (8 FMA lanes, lanes summed in order, kernels.rs:6557-6573) -> same bits as the CPU
//   route          : softmax over all experts with max shift, sequential sums (lib.rs:2427-2436),
//                    top-k = repeated arg-max with the lower expert id winning ties (:2527-2529),
//                    w = p / max(sum p_sel, 1e-20) * scale (:2536-2538)
//   bucket         : pairs (row, rank) grouped by expert, in (row, rank) order inside an expert
//                    (:2554-2587), plus the 8-row work items of the grouped GEMM
//   swiglu_quant   : act = silu(g) * u per pair (kernels.rs:6578-6597), re-quantised per 256
//                    (lib.rs:2862-2873) with the arithmetic of quantize.cu
//   combine        : out[r] += w * y in rank order, multiply and add rounded separately (:2970-2982)
#include "kernels.h"
#include "pdl.cuh"
#include "q8_code.cuh"

namespace infr {

// logits[r, e] = dot(router[e, :], x[r, :]).  Eight lanes per dot product replay the eight accumulators of the CPU
// `dot` (lane j takes elements j, 8 + j, ... in order, the lanes are then summed in order, the tail is added by fused
// multiply-adds).  A block computes 8 rows x 16 experts; a group of eight lanes holds a 2 x 2 corner of it, so every
// shared-memory read feeds two multiply-adds.  Rows and router rows are staged 256 columns at a time, coalesced;
// the row pitch (260 words) puts the four groups of a warp on disjoint banks.
constexpr int kRtRows = 8, kRtExperts = 16, kRtK = 256, kRtPitch = kRtK + 4;
__global__ void __launch_bounds__(256) moe_router_kernel(const float *__restrict__ router, const float *__restrict__ x,
                                                         float *__restrict__ logits, int rows, int ne, int n_expert) {
    pdl_go();
    pdl_wait();
    __shared__ float s_x[kRtRows * kRtPitch], s_w[kRtExperts * kRtPitch];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 3, j = lane & 7;
    const int rp = warp >> 1, ep = (warp & 1) * 4 + grp;  // row pair 0..3, expert pair 0..7
    const int r0 = blockIdx.x * kRtRows, e0 = blockIdx.y * kRtExperts;
    const int chunks = ne / 8;  // whole groups of eight columns; the rest is the tail
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    // Staging: 16-byte loads, the next 256 columns are fetched into registers while the current ones are multiplied
    // (rows start on 16-byte boundaries when ne is a multiple of 4; otherwise element loads).
    const bool vec = (ne & 3) == 0 && (((uintptr_t)x | (uintptr_t)router) & 15) == 0;
    const int kend = chunks * 8;
    float4 px[2], pw[4];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int u = 0; u < 6; u++) {
            const int i = threadIdx.x + u * 256;            // float4 slot: 0..511 rows of x, 512..1535 router rows
            const bool is_w = i >= 512;
            const int ii = is_w ? i - 512 : i, r = ii >> 6, k = (ii & 63) * 4;
            const int gr = (is_w ? e0 : r0) + r, lim = is_w ? n_expert : rows;
            const float *src = (is_w ? router : x) + (size_t)gr * ne + k0 + k;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gr < lim) {
                if (vec && k0 + k + 4 <= kend) {
                    v = __ldg(reinterpret_cast<const float4 *>(src));
                } else {
                    if (k0 + k < kend) v.x = src[0];
                    if (k0 + k + 1 < kend) v.y = src[1];
                    if (k0 + k + 2 < kend) v.z = src[2];
                    if (k0 + k + 3 < kend) v.w = src[3];
                }
            }
            if (is_w) pw[u - 2] = v; else px[u] = v;
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < 6; u++) {
            const int i = threadIdx.x + u * 256;
            const bool is_w = i >= 512;
            const int ii = is_w ? i - 512 : i, r = ii >> 6, k = (ii & 63) * 4;
            *reinterpret_cast<float4 *>((is_w ? s_w : s_x) + r * kRtPitch + k) = is_w ? pw[u - 2] : px[u];
        }
    };
    if (kend > 0) fetch(0);
    for (int k0 = 0; k0 < kend; k0 += kRtK) {
        const int kc = min(kRtK, kend - k0);
        __syncthreads();  // everybody has finished with the previous columns
        stash();
        __syncthreads();
        if (k0 + kRtK < kend) fetch(k0 + kRtK);
        const float *xa = s_x + (2 * rp) * kRtPitch + j, *xb = xa + kRtPitch;
        const float *wa = s_w + (2 * ep) * kRtPitch + j, *wb = wa + kRtPitch;
#pragma unroll 4
        for (int c = 0; c < kc / 8; c++) {
            const float x0 = xa[c * 8], x1 = xb[c * 8], w0 = wa[c * 8], w1 = wb[c * 8];
            acc[0][0] = fmaf(w0, x0, acc[0][0]);
            acc[0][1] = fmaf(w1, x0, acc[0][1]);
            acc[1][0] = fmaf(w0, x1, acc[1][0]);
            acc[1][1] = fmaf(w1, x1, acc[1][1]);
        }
    }
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 2; b++) {
            // s = ((((acc0 + acc1) + acc2) + ...) + acc7), then the FMA tail
            float sum = 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, acc[a][b], grp * 8 + k));
            const int r = r0 + 2 * rp + a, e = e0 + 2 * ep + b;
            if (r < rows && e < n_expert) {
                const float *w = router + (size_t)e * ne, *xr = x + (size_t)r * ne;
                for (int i = chunks * 8; i < ne; i++) sum = fmaf(w[i], xr[i], sum);
                if (j == 0) logits[(size_t)r * n_expert + e] = sum;
            }
        }
}

// One warp per row.  n_expert <= 1024.
__global__ void __launch_bounds__(128) moe_route_kernel(const float *__restrict__ logits, int rows, int n_expert, int n_used,
                                                        float scale, int norm_w, int32_t *__restrict__ sel_ids,
                                                        float *__restrict__ sel_w) {
    pdl_go();
    pdl_wait();
    extern __shared__ float s_p[];  // [warps][n_expert]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= rows) return;
    float *p = s_p + (size_t)warp * n_expert;
    const float *lg = logits + (size_t)r * n_expert;
    float mx = -INFINITY;
    for (int e = lane; e < n_expert; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int e = lane; e < n_expert; e += 32) p[e] = expf(lg[e] - mx);
    __syncwarp();
    float psum = 0.f;
    if (lane == 0)
        for (int e = 0; e < n_expert; e++) psum = __fadd_rn(psum, p[e]);  // the CPU sums in index order
    psum = __shfl_sync(0xffffffffu, psum, 0);
    for (int e = lane; e < n_expert; e += 32) p[e] = __fdiv_rn(p[e], psum);
    __syncwarp();
    // top-k: k rounds of arg-max; ties go to the lower expert id (what a stable descending sort does)
    float wsum = 0.f;
    float myw = 0.f;  // lane k keeps the k-th selected probability (n_used <= 32)
    int myid = 0;
    for (int k = 0; k < n_used; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < n_expert; e += 32) {
            const float v = p[e];
            if (v > best) {
                best = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (bi == 0x7fffffff) {
            // No probability compared greater than -inf: the row is all NaN (a NaN or infinite logit poisons the
            // softmax sum).  The CPU's stable sort leaves such a row in index order, so take the lowest expert
            // not selected yet; its NaN weight travels on as it does there.
            for (int e = lane; e < n_expert; e += 32)
                if (p[e] != -INFINITY) {
                    bi = e;
                    break;
                }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) bi = min(bi, __shfl_xor_sync(0xffffffffu, bi, o));
            if (bi < n_expert) best = p[bi];
        }
        wsum = __fadd_rn(wsum, best);
        if (lane == k) {
            myw = best;
            myid = bi < n_expert ? bi : 0;
        }
        if (lane == 0 && bi < n_expert) p[bi] = -INFINITY;  // never compares greater than the running best again
        __syncwarp();
    }
    wsum = fmaxf(wsum, 1e-20f);
    if (lane < n_used) {
        sel_ids[(size_t)r * n_used + lane] = myid;
        sel_w[(size_t)r * n_used + lane] = norm_w ? __fmul_rn(__fdiv_rn(myw, wsum), scale) : __fmul_rn(myw, scale);
    }
}

// One CTA of 32 warps lists the routed pairs by expert, in (row, rank) order inside an expert, and cuts every
// expert's pairs into work items of up to `item_rows` rows (8 for the grouped GEMV, 64 = one token tile for the
// grouped tensor-memory GEMM).
//   pair_row[p], pair_of_slot[r * n_used + rank] = p, item_{expert,p0,cnt}[], n_items
// Expert parallelism: only experts [e_lo, e_lo + n_local) are listed (item_expert is the index inside this
// rank's banks); pairs routed elsewhere get pair_of_slot = -1 and contribute nothing to this rank's output.
__global__ void __launch_bounds__(1024) moe_bucket_kernel(const int32_t *__restrict__ sel_ids, int rows, int n_used, int n_expert,
                                                          int e_lo, int n_local, int item_rows,
                                                          int32_t *__restrict__ pair_row, int32_t *__restrict__ pair_of_slot,
                                                          int32_t *__restrict__ item_expert, int32_t *__restrict__ item_p0,
                                                          int32_t *__restrict__ item_cnt, int32_t *__restrict__ n_items,
                                                          int32_t *__restrict__ counts_out, int n_chunks) {
    pdl_go();
    pdl_wait();
    // A stable counting sort over chunks of 32 pairs: hist[chunk][expert] = pairs of the expert inside the chunk
    // (lanes with the same expert find each other with a match), an exclusive scan down the chunks gives the place of
    // a chunk's first such pair inside its expert, and a pair's place is that plus its rank among the lanes before it:
    // (row, rank) order is kept and the work is linear in the number of pairs.
    __shared__ int s_cnt[1024], s_off[1024], s_ioff[1024];
    extern __shared__ int32_t s_hist[];  // [n_chunks][n_expert]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_pairs = rows * n_used;
    for (int i = threadIdx.x; i < n_chunks * n_expert; i += 1024) s_hist[i] = 0;
    __syncthreads();
    // the expert of pair i as this rank sees it: -1 for another rank's expert or an id outside the bank
    auto local_expert = [&](int i) {
        if (i >= n_pairs) return -1;
        const int e = sel_ids[i];
        return (e < e_lo || e >= e_lo + n_local || e < 0 || e >= n_expert) ? -1 : e;
    };
    for (int c = warp; c < n_chunks; c += 32) {
        const int e = local_expert(c * 32 + lane);
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (same & ((1u << lane) - 1u)) == 0) s_hist[c * n_expert + e] = __popc(same);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += 1024) {
        int run = 0;
        for (int c = 0; c < n_chunks; c++) {
            const int t = s_hist[c * n_expert + e];
            s_hist[c * n_expert + e] = run;
            run += t;
        }
        s_cnt[e] = run;
        if (counts_out) counts_out[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, ioff = 0;
        for (int k = 0; k < n_expert; k++) {
            s_off[k] = off;
            s_ioff[k] = ioff;
            off += s_cnt[k];
            ioff += (s_cnt[k] + item_rows - 1) / item_rows;
        }
        *n_items = ioff;
    }
    __syncthreads();
    for (int c = warp; c < n_chunks; c += 32) {
        const int i = c * 32 + lane;
        const int e = local_expert(i);
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        if (i < n_pairs) {
            int q = -1;  // pairs routed to an expert that is not listed contribute nothing to this rank's output
            if (e >= 0) {
                q = s_off[e] + s_hist[c * n_expert + e] + __popc(same & ((1u << lane) - 1u));
                pair_row[q] = i / n_used;
            }
            pair_of_slot[i] = q;
        }
    }
    for (int e = warp; e < n_expert; e += 32) {
        const int cnt = s_cnt[e];
        for (int c = lane * item_rows; c < cnt; c += 32 * item_rows) {
            const int it = s_ioff[e] + c / item_rows;
            item_expert[it] = e - e_lo;
            item_p0[it] = s_off[e] + c;
            item_cnt[it] = cnt - c < item_rows ? cnt - c : item_rows;
        }
    }
}

// One warp per (pair, 256-block): act = silu(gate) * up, then quantize_q8 of that block.
__global__ void __launch_bounds__(256) moe_swiglu_quant_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                               int n_pairs, int nff, int8_t *__restrict__ qs, float *__restrict__ d,
                                                               int32_t *__restrict__ sums, int32_t *__restrict__ sums16,
                                                               float *__restrict__ act_out) {
    pdl_go();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int nbk = nff / 256;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)n_pairs * nbk) return;
    const int p = (int)(wg / nbk), b = (int)(wg % nbk);
    const size_t base = (size_t)p * nff + (size_t)b * 256 + lane * 8;
    float v[8];
    float am = 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float4 g4 = *reinterpret_cast<const float4 *>(gate + base + h * 4);
        const float4 u4 = *reinterpret_cast<const float4 *>(up + base + h * 4);
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float sg = __fdiv_rn(gg[i], __fadd_rn(1.0f, expf(-gg[i])));
            v[h * 4 + i] = __fmul_rn(sg, uu[i]);
            am = fmaxf(am, fabsf(v[h * 4 + i]));
        }
    }
    if (act_out) {
#pragma unroll
        for (int i = 0; i < 8; i++) act_out[base + i] = v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float dd = am / 127.0f;
    const float id = dd > 0.0f ? 1.0f / dd : 0.0f;
    int q[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        q[i] = q8_round_code(v[i], id);
        sum += q[i];
    }
    uint2 pk;
    pk.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    pk.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(qs + base) = pk;
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (sums16 && (lane & 1) == 0) sums16[((size_t)p * nbk + b) * 16 + (lane >> 1)] = sum;  // Q6_K banks: sums per 16 codes
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((lane & 3) == 0) sums[((size_t)p * nbk + b) * 8 + (lane >> 2)] = sum;
    if (lane == 0) d[(size_t)p * nbk + b] = dd;
}

// out[r, i] = sum over ranks (in rank order) of w[r, rank] * y[pair_of_slot[r, rank], i].
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *__restrict__ y_pairs, const int32_t *__restrict__ pair_of_slot,
                                                          const float *__restrict__ sel_w, int rows, int n_used, int ne,
                                                          float *__restrict__ out) {
    pdl_go();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * ne) return;
    const int r = (int)(idx / ne), i = (int)(idx % ne);
    float o = 0.f;
    for (int k = 0; k < n_used; k++) {
        const int p = pair_of_slot ? pair_of_slot[(size_t)r * n_used + k] : r * n_used + k;
        if (p < 0) continue;  // routed to an expert of another rank
        o = __fadd_rn(o, __fmul_rn(sel_w[(size_t)r * n_used + k], y_pairs[(size_t)p * ne + i]));
    }
    out[idx] = o;
}

cudaError_t launch_moe_router(const float *router, const float *x, float *logits, int rows, int ne, int n_expert,
                              cudaStream_t st) {
    if (rows < 1 || n_expert < 1) return cudaErrorInvalidValue;
    const dim3 grid((unsigned)((rows + kRtRows - 1) / kRtRows), (unsigned)((n_expert + kRtExperts - 1) / kRtExperts));
    if (grid.y > 65535) return cudaErrorInvalidValue;
    return launch_pdl(moe_router_kernel, grid, dim3(256), 0, st, router, x, logits, rows, ne, n_expert);
}

cudaError_t launch_moe_route(const float *logits, int rows, int n_expert, int n_used, float scale, int norm_w,
                             int32_t *sel_ids, float *sel_w, cudaStream_t st) {
    if (n_expert > 1024 || n_used > 32 || n_used > n_expert) return cudaErrorInvalidValue;
    const int warps = 4;
    return launch_pdl(moe_route_kernel, dim3((unsigned)((rows + warps - 1) / warps)), dim3(warps * 32), (size_t)warps * n_expert * 4, st, logits, rows,
                      n_expert, n_used, scale, norm_w, sel_ids, sel_w);
}

cudaError_t launch_moe_bucket(const int32_t *sel_ids, int rows, int n_used, int n_expert, int e_lo, int n_local, int item_rows,
                              int32_t *pair_row, int32_t *pair_of_slot, int32_t *item_expert, int32_t *item_p0, int32_t *item_cnt,
                              int32_t *n_items, int32_t *counts_out, cudaStream_t st) {
    if (n_expert > 1024 || item_rows < 1) return cudaErrorInvalidValue;
    const int n_chunks = (rows * n_used + 31) / 32;
    const size_t hist_bytes = (size_t)n_chunks * n_expert * 4;
    if (hist_bytes > 200 * 1024) return cudaErrorInvalidValue;  // ~51 000 pairs of 128 experts; more would need a multi-CTA sort
    cudaError_t e = cudaFuncSetAttribute(moe_bucket_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_bytes);
    if (e != cudaSuccess) return e;
    return launch_pdl(moe_bucket_kernel, dim3(1), dim3(1024), hist_bytes, st, sel_ids, rows, n_used, n_expert, e_lo, n_local, item_rows, pair_row,
                      pair_of_slot, item_expert, item_p0, item_cnt, n_items, counts_out, n_chunks);
}

cudaError_t launch_moe_swiglu_quant(const float *gate, const float *up, int n_pairs, int nff, int8_t *qs, float *d,
                                    int32_t *sums, int32_t *sums16, float *act_out, cudaStream_t st) {
    if (nff % 256) return cudaErrorInvalidValue;
    const long long warps = (long long)n_pairs * (nff / 256);
    return launch_pdl(moe_swiglu_quant_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, st, gate, up, n_pairs, nff, qs, d, sums, sums16,
                      act_out);
}

cudaError_t launch_moe_combine(const float *y_pairs, const int32_t *pair_of_slot, const float *sel_w, int rows, int n_used,
                               int ne, float *out, cudaStream_t st) {
    const long long n = (long long)rows * ne;
    return launch_pdl(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, y_pairs, pair_of_slot, sel_w, rows, n_used, ne, out);
}

}  // namespace infr
