// Decode GEMV over GGUF block-quantized weights: y[m,out_f] = x[m,in_f] * W^T, m <= 8.
//
// Two arithmetic modes, both taken from the CPU reference:
//   * int8 activations (production): the activation rows are quantised once (quantize.cu) and every
//     weight block is reduced with integer dot products — crates/infr-cpu/src/kernels.rs:151-184
//     (Q4_K: sd = sum sc_s*iprod_s, sm = sum m_s*bsum_s, f = d8*(d*sd - dmin*sm)), :487-526 (Q6_K:
//     isum = sum sc_j*(sumi_j - 32*bsum_j), f = d*d8*isum), :5641-5668 (Q2_0: f = d*d8_s*(iprod_s -
//     bsum_s)).  The int32 block accumulators are exact, so they equal the reference's bit for bit
//     whatever the lane split; only the order of the final f32 additions differs.
//   * f32 activations (`kernels.cpu.reference`, crates/infr-cpu/src/lib.rs:1015-1031): weights are
//     dequantised with the two roundings of crates/infr-gguf/src/dequant.rs:31-47 and FMA'd.
//
// Layout / mapping.  The weight matrix is streamed exactly once with no reuse, so the kernel is
// HBM-bound: one warp owns one output row at a time and walks its blocks with every lane issuing
// 16-byte (Q4_K) loads that together cover contiguous 576-byte spans; partial results stay in
// registers and meet in one shuffle tree per row.  Activations are tiny and are staged once per CTA
// in shared memory, permuted so every lane's operand fetch is a conflict-free 16-byte read.  The grid
// is a multiple of the SM count and each CTA strides over rows (persistent CTAs), so the staging cost
// is paid once per SM.
#include "gemv_common.cuh"

namespace infr {

namespace {

// ------------------------------------------------------------------------------------------------
// Q4_K x Q8(256).  8 lanes per super-block (lane c owns the 16-byte nibble chunk c: 16 elements of
// sub-block 2*(c/2) in the low nibbles, 16 of sub-block 2*(c/2)+1 in the high ones), 4 blocks per
// warp step.
// ------------------------------------------------------------------------------------------------
template <int M, bool DUMP>
__global__ void __launch_bounds__(kThreads) gemv_q4k_q8_kernel(const uint8_t *__restrict__ W, Q8Dev a,
                                                               float *__restrict__ y, int m, int in_f,
                                                               int out_f, int32_t *__restrict__ acc_out) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = in_f >> 8;
    int8_t *s_qa = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * in_f);
    int32_t *s_bs = reinterpret_cast<int32_t *>(s_d + M * nb);
    stage_q8<DT_Q4K>(a, m, M, in_f, s_qa, s_d, s_bs);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 3, c = lane & 7, j = c >> 1;
    const size_t row_bytes = (size_t)nb * 144;
    for (int row = blockIdx.x * kWarps + warp; row < out_f; row += gridDim.x * kWarps) {
        const uint8_t *wr = W + (size_t)row * row_bytes;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = 0.f;
#pragma unroll 4
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int b = b0 + g;
            const bool live = b < nb;
            int sd[M], sm[M];
            float d = 0.f, dmin = 0.f;
            if (live) {
                const uint8_t *blk = wr + (size_t)b * 144;
                const uint4 hdr = ldg16(blk);
                const uint4 qv = ldg16(blk + 16 + c * 16);
                int sc0, m0, sc1, m1;
                k4_pair(hdr.y, hdr.z, hdr.w, j, sc0, m0, sc1, m1);
                d = h2f(hdr.x);
                dmin = h2f(hdr.x >> 16);
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
                    sd[t] = sc0 * ilo + sc1 * ihi;
                    sm[t] = mc * s_bs[(t * nb + b) * 8 + c];
                }
            } else {
#pragma unroll
                for (int t = 0; t < M; t++) sd[t] = sm[t] = 0;
            }
            if (DUMP) {
                int vd = sd[0], vm = sm[0];
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) {
                    vd += __shfl_xor_sync(0xffffffffu, vd, o, 8);
                    vm += __shfl_xor_sync(0xffffffffu, vm, o, 8);
                }
                if (live && c == 0) {
                    acc_out[((size_t)row * nb + b) * 2] = vd;
                    acc_out[((size_t)row * nb + b) * 2 + 1] = vm;
                }
            } else if (live) {
#pragma unroll
                for (int t = 0; t < M; t++)
                    acc[t] += s_d[t * nb + b] * (d * (float)sd[t] - dmin * (float)sm[t]);
            }
        }
        if (!DUMP) {
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float v = warp_sum(acc[t]);
                if (lane == 0 && t < m) y[(size_t)t * out_f + row] = v;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Q6_K x Q8(256).  16 lanes per super-block: lane (half, l4) owns l = 4*l4..4*l4+3 of that half, i.e.
// 4 bytes of ql[l], 4 of ql[l+32], 4 of qh[l] -> the 16 elements l, l+32, l+64, l+96 (x4).  Two blocks
// per warp step.
// ------------------------------------------------------------------------------------------------
// Body shared by the plain kernel and the expert-grouped one: token t reads activation row row_of[row0 + t]
// (row0 + t without a list) and writes row t of `y`, which the caller has offset to its first output row.
template <int M, bool DUMP>
__device__ __forceinline__ void q6k_q8_body(const uint8_t *__restrict__ W, const Q8Dev &a, float *__restrict__ y, int m, int in_f,
                                            int out_f, int32_t *__restrict__ acc_out, const int32_t *row_of, int row0) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = in_f >> 8;
    const int tok_stride = (nb + 1) / 2 * 512;  // bytes of staged codes per token (block pairs)
    int8_t *s_qa = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * tok_stride);
    int32_t *s_bs = reinterpret_cast<int32_t *>(s_d + M * nb);  // per-16 sums
    stage_q8<DT_Q6K>(a, m, M, in_f, s_qa, s_d, s_bs, row_of, row0);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hb = lane >> 4, r = lane & 15, half = r >> 3, l4 = r & 7;
    const size_t row_bytes = (size_t)nb * 210;
    for (int row = blockIdx.x * kWarps + warp; row < out_f; row += gridDim.x * kWarps) {
        const uint8_t *wr = W + (size_t)row * row_bytes;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = 0.f;
#pragma unroll 2
        for (int b0 = 0; b0 < nb; b0 += 2) {
            const int b = b0 + hb;
            const bool live = b < nb;
            int part[M];
            float dw = 0.f;
            if (live) {
                const uint8_t *blk = wr + (size_t)b * 210;
                const uint32_t qla = ldg_u32_a2(blk + half * 64 + l4 * 4);
                const uint32_t qlb = ldg_u32_a2(blk + half * 64 + 32 + l4 * 4);
                const uint32_t qh = ldg_u32_a2(blk + 128 + half * 32 + l4 * 4);
                const int8_t *scp = reinterpret_cast<const int8_t *>(blk + 192);
                const int is = l4 >> 2;
                int sc[4];
#pragma unroll
                for (int k = 0; k < 4; k++) sc[k] = (int)__ldg(scp + half * 8 + is + 2 * k);
                const int scr = (int)__ldg(scp + r);
                dw = h2f(ldg_u16(blk + 208));
                uint32_t q[4];
                q[0] = (qla & 0x0F0F0F0Fu) | ((qh & 0x03030303u) << 4);
                q[1] = (qlb & 0x0F0F0F0Fu) | (((qh >> 2) & 0x03030303u) << 4);
                q[2] = ((qla >> 4) & 0x0F0F0F0Fu) | (((qh >> 4) & 0x03030303u) << 4);
                q[3] = ((qlb >> 4) & 0x0F0F0F0Fu) | (((qh >> 6) & 0x03030303u) << 4);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const int *aw = reinterpret_cast<const int *>(s_qa + (size_t)t * tok_stride) +
                                    (b >> 1) * 128 + (b & 1) * 16 + half * 8 + l4;
                    int isum = 0;
#pragma unroll
                    for (int k = 0; k < 4; k++) isum += sc[k] * dp4a_us(q[k], aw[k * 32], 0);
                    isum -= 32 * scr * s_bs[(t * nb + b) * 16 + r];
                    part[t] = isum;
                }
            } else {
#pragma unroll
                for (int t = 0; t < M; t++) part[t] = 0;
            }
            if (DUMP) {
                int v = part[0];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o, 16);
                if (live && r == 0) acc_out[(size_t)row * nb + b] = v;
            } else if (live) {
#pragma unroll
                for (int t = 0; t < M; t++) acc[t] += (dw * s_d[t * nb + b]) * (float)part[t];
            }
        }
        if (!DUMP) {
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float v = warp_sum(acc[t]);
                if (lane == 0 && t < m) y[(size_t)t * out_f + row] = v;
            }
        }
    }
}

template <int M, bool DUMP>
__global__ void __launch_bounds__(kThreads) gemv_q6k_q8_kernel(const uint8_t *__restrict__ W, Q8Dev a,
                                                               float *__restrict__ y, int m, int in_f,
                                                               int out_f, int32_t *__restrict__ acc_out) {
    q6k_q8_body<M, DUMP>(W, a, y, m, in_f, out_f, acc_out, nullptr, 0);
}

// Expert-grouped form (mixture of experts): blockIdx.y walks the device-built list of work items, each up to 8
// routed pairs of one expert; the bank holds the experts' [out_f, in_f] matrices back to back; pair p reads
// activation row pair_row[p] (or p) and writes y row p.
__global__ void __launch_bounds__(kThreads) gemv_q6k_q8_grouped_kernel(const uint8_t *__restrict__ bank, Q8Dev a, float *__restrict__ y,
                                                                       int in_f, int out_f, const int *__restrict__ item_expert,
                                                                       const int *__restrict__ item_p0, const int *__restrict__ item_cnt,
                                                                       const int *__restrict__ n_items, const int *__restrict__ pair_row) {
    const int item = blockIdx.y;
    if (item >= *n_items) return;
    const int p0 = item_p0[item];
    const size_t w_off = (size_t)item_expert[item] * out_f * (size_t)(in_f >> 8) * 210;
    q6k_q8_body<8, false>(bank + w_off, a, y + (size_t)p0 * out_f, item_cnt[item], in_f, out_f, nullptr, pair_row, p0);
}

// ------------------------------------------------------------------------------------------------
// Q2_0 x Q8(32).  4 lanes per 64-element block: lane q owns 16 elements = one 32-bit word of 2-bit
// codes; field i of every byte comes out of (w >> 2i) & 0x03030303 and meets the transposed
// activation word i.  8 blocks per warp step.
// ------------------------------------------------------------------------------------------------
template <int M, bool DUMP>
__global__ void __launch_bounds__(kThreads) gemv_q2_0_q8_kernel(const uint8_t *__restrict__ W, Q8Dev a,
                                                                float *__restrict__ y, int m, int in_f,
                                                                int out_f, int32_t *__restrict__ acc_out) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = in_f >> 6, ns = in_f >> 5;
    int8_t *s_qa = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * in_f);
    int32_t *s_bs = reinterpret_cast<int32_t *>(s_d + M * ns);
    stage_q8<DT_Q2_0>(a, m, M, in_f, s_qa, s_d, s_bs);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const size_t row_bytes = (size_t)nb * 18;
    for (int row = blockIdx.x * kWarps + warp; row < out_f; row += gridDim.x * kWarps) {
        const uint8_t *wr = W + (size_t)row * row_bytes;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = 0.f;
#pragma unroll 4
        for (int b0 = 0; b0 < nb; b0 += 8) {
            const int b = b0 + g;
            const bool live = b < nb;
            const int s = 2 * b + (q >> 1);
            int part[M];
            float dw = 0.f;
            if (live) {
                const uint8_t *blk = wr + (size_t)b * 18;
                dw = h2f(ldg_u16(blk));
                const uint32_t w = ldg_u32_a2(blk + 2 + q * 4);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const uint4 av = reinterpret_cast<const uint4 *>(s_qa + (size_t)t * in_f)[b * 4 + q];
                    int ip = dp4a_us(w & 0x03030303u, (int)av.x, 0);
                    ip = dp4a_us((w >> 2) & 0x03030303u, (int)av.y, ip);
                    ip = dp4a_us((w >> 4) & 0x03030303u, (int)av.z, ip);
                    ip = dp4a_us((w >> 6) & 0x03030303u, (int)av.w, ip);
                    part[t] = ip;
                }
            } else {
#pragma unroll
                for (int t = 0; t < M; t++) part[t] = 0;
            }
            if (DUMP) {
                int v = part[0];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                if (live && (q & 1) == 0) acc_out[(size_t)row * ns + s] = v;
            } else if (live) {
#pragma unroll
                for (int t = 0; t < M; t++) {
                    const int v = part[t] - ((q & 1) ? 0 : s_bs[t * ns + s]);
                    acc[t] += dw * s_d[t * ns + s] * (float)v;
                }
            }
        }
        if (!DUMP) {
#pragma unroll
            for (int t = 0; t < M; t++) {
                const float v = warp_sum(acc[t]);
                if (lane == 0 && t < m) y[(size_t)t * out_f + row] = v;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// f32-activation (reference-mode) kernels: same lane ownership, weights dequantised exactly as
// dequant_block does (scale = d*sc, offset = dmin*(-m), value = scale*code + offset, two roundings).
// ------------------------------------------------------------------------------------------------
template <int M>
__device__ __forceinline__ void stage_f32(const float *x, int m, int in_f, float *s_x) {
    const int n4 = in_f / 4;
    for (int idx = threadIdx.x; idx < M * n4; idx += kThreads) {
        const int t = idx / n4, u = idx - t * n4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < m) v = *reinterpret_cast<const float4 *>(x + (size_t)t * in_f + (size_t)u * 4);
        reinterpret_cast<float4 *>(s_x)[idx] = v;
    }
}

// Expert selection for the f32 (single-row / reference) MoE path: blockIdx.y = routed pair p, whose
// weights are expert sel[p] of a bank, whose activation row is p / x_div (x_div = 0: row p) and whose
// output row is p.  sel == nullptr: an ordinary GEMV.
struct SelArgs {
    const int32_t *sel;
    size_t w_stride;
    int x_div;
};

template <int M>
__global__ void __launch_bounds__(kThreads) gemv_q4k_f32_kernel(const uint8_t *__restrict__ W,
                                                                const float *__restrict__ x,
                                                                float *__restrict__ y, int m, int in_f,
                                                                int out_f, SelArgs sa) {
    if (sa.sel) {
        const int p = blockIdx.y;
        W += (size_t)sa.sel[p] * sa.w_stride;
        x += (size_t)(sa.x_div ? p / sa.x_div : p) * in_f;
        y += (size_t)p * out_f;
    }
    extern __shared__ __align__(16) uint8_t smem[];
    float *s_x = reinterpret_cast<float *>(smem);
    stage_f32<M>(x, m, in_f, s_x);
    __syncthreads();
    const int nb = in_f >> 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 3, c = lane & 7, j = c >> 1, h = c & 1;
    const size_t row_bytes = (size_t)nb * 144;
    for (int row = blockIdx.x * kWarps + warp; row < out_f; row += gridDim.x * kWarps) {
        const uint8_t *wr = W + (size_t)row * row_bytes;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = 0.f;
#pragma unroll 2
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int b = b0 + g;
            if (b >= nb) continue;
            const uint8_t *blk = wr + (size_t)b * 144;
            const uint4 hdr = ldg16(blk);
            const uint4 qv = ldg16(blk + 16 + c * 16);
            int sc0, m0, sc1, m1;
            k4_pair(hdr.y, hdr.z, hdr.w, j, sc0, m0, sc1, m1);
            const float d = h2f(hdr.x), dmin = h2f(hdr.x >> 16);
            const float s0 = __fmul_rn(d, (float)sc0), n0 = __fmul_rn(dmin, (float)(-m0));
            const float s1 = __fmul_rn(d, (float)sc1), n1 = __fmul_rn(dmin, (float)(-m1));
            const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
            const int e0 = b * 256 + (2 * j) * 32 + h * 16;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t byte = (q[i >> 2] >> (8 * (i & 3))) & 0xFFu;
                const float wlo = __fadd_rn(__fmul_rn(s0, (float)(byte & 0xF)), n0);
                const float whi = __fadd_rn(__fmul_rn(s1, (float)(byte >> 4)), n1);
#pragma unroll
                for (int t = 0; t < M; t++) {
                    acc[t] = fmaf(wlo, s_x[t * in_f + e0 + i], acc[t]);
                    acc[t] = fmaf(whi, s_x[t * in_f + e0 + 32 + i], acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && t < m) y[(size_t)t * out_f + row] = v;
        }
    }
}

template <int M>
__global__ void __launch_bounds__(kThreads) gemv_q6k_f32_kernel(const uint8_t *__restrict__ W,
                                                                const float *__restrict__ x,
                                                                float *__restrict__ y, int m, int in_f,
                                                                int out_f) {
    extern __shared__ __align__(16) uint8_t smem[];
    float *s_x = reinterpret_cast<float *>(smem);
    stage_f32<M>(x, m, in_f, s_x);
    __syncthreads();
    const int nb = in_f >> 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hb = lane >> 4, r = lane & 15, half = r >> 3, l4 = r & 7;
    const size_t row_bytes = (size_t)nb * 210;
    for (int row = blockIdx.x * kWarps + warp; row < out_f; row += gridDim.x * kWarps) {
        const uint8_t *wr = W + (size_t)row * row_bytes;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 2) {
            const int b = b0 + hb;
            if (b >= nb) continue;
            const uint8_t *blk = wr + (size_t)b * 210;
            const uint32_t qla = ldg_u32_a2(blk + half * 64 + l4 * 4);
            const uint32_t qlb = ldg_u32_a2(blk + half * 64 + 32 + l4 * 4);
            const uint32_t qh = ldg_u32_a2(blk + 128 + half * 32 + l4 * 4);
            const int8_t *scp = reinterpret_cast<const int8_t *>(blk + 192);
            const float d = h2f(ldg_u16(blk + 208));
            uint32_t q[4];
            q[0] = (qla & 0x0F0F0F0Fu) | ((qh & 0x03030303u) << 4);
            q[1] = (qlb & 0x0F0F0F0Fu) | (((qh >> 2) & 0x03030303u) << 4);
            q[2] = ((qla >> 4) & 0x0F0F0F0Fu) | (((qh >> 4) & 0x03030303u) << 4);
            q[3] = ((qlb >> 4) & 0x0F0F0F0Fu) | (((qh >> 6) & 0x03030303u) << 4);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int sci = (int)__ldg(scp + half * 8 + (l4 >> 2) + 2 * k);
                const float sc = __fmul_rn(d, (float)sci), mn = __fmul_rn(d, (float)(-32 * sci));
                const int e0 = b * 256 + half * 128 + k * 32 + l4 * 4;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float wv = __fadd_rn(__fmul_rn(sc, (float)((q[k] >> (8 * i)) & 0xFFu)), mn);
#pragma unroll
                    for (int t = 0; t < M; t++) acc[t] = fmaf(wv, s_x[t * in_f + e0 + i], acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && t < m) y[(size_t)t * out_f + row] = v;
        }
    }
}

template <int M>
__global__ void __launch_bounds__(kThreads) gemv_q2_0_f32_kernel(const uint8_t *__restrict__ W,
                                                                 const float *__restrict__ x,
                                                                 float *__restrict__ y, int m, int in_f,
                                                                 int out_f) {
    extern __shared__ __align__(16) uint8_t smem[];
    float *s_x = reinterpret_cast<float *>(smem);
    stage_f32<M>(x, m, in_f, s_x);
    __syncthreads();
    const int nb = in_f >> 6;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const size_t row_bytes = (size_t)nb * 18;
    for (int row = blockIdx.x * kWarps + warp; row < out_f; row += gridDim.x * kWarps) {
        const uint8_t *wr = W + (size_t)row * row_bytes;
        float acc[M];
#pragma unroll
        for (int t = 0; t < M; t++) acc[t] = 0.f;
#pragma unroll 2
        for (int b0 = 0; b0 < nb; b0 += 8) {
            const int b = b0 + g;
            if (b >= nb) continue;
            const uint8_t *blk = wr + (size_t)b * 18;
            const float d = h2f(ldg_u16(blk));
            const uint32_t w = ldg_u32_a2(blk + 2 + q * 4);
            const int e0 = b * 64 + q * 16;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int code = (int)((w >> (2 * i)) & 3u);
                const float wv = __fmul_rn((float)(code - 1), d);
#pragma unroll
                for (int t = 0; t < M; t++) acc[t] = fmaf(wv, s_x[t * in_f + e0 + i], acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < M; t++) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && t < m) y[(size_t)t * out_f + row] = v;
        }
    }
}

// ------------------------------------------------------------------------------------------------
template <typename K>
cudaError_t set_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

int grid_for(int out_f, size_t smem, const DeviceInfo &dev) {
    const int need = (out_f + kWarps - 1) / kWarps;
    // resident CTAs per SM: limited by threads (2048/256 = 8) and by the staged activations
    int per_sm = 8;
    if (smem) per_sm = (int)((size_t)dev.max_smem_optin / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const int cap = dev.sm_count * per_sm;
    return need < cap ? need : cap;
}

size_t q8_smem(int dt, int M, int in_f) {
    if (dt == DT_Q4K) return (size_t)M * in_f + (size_t)M * (in_f / 256) * 4 + (size_t)M * (in_f / 32) * 4;
    if (dt == DT_Q6K)
        return (size_t)M * ((in_f / 256 + 1) / 2 * 512) + (size_t)M * (in_f / 256) * 4 + (size_t)M * (in_f / 16) * 4;
    return (size_t)M * in_f + (size_t)M * (in_f / 32) * 8;
}

template <int M>
cudaError_t launch_q8_m(int dt, const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                        int32_t *acc_out, const DeviceInfo &dev, cudaStream_t st) {
    const size_t smem = q8_smem(dt, M, in_f);
    if (smem > (size_t)dev.max_smem_optin) return cudaErrorInvalidValue;
    const int grid = grid_for(out_f, smem, dev);
    cudaError_t e;
#define INFR_LAUNCH(KERNEL)                                                   \
    do {                                                                      \
        if ((e = set_smem(KERNEL, smem)) != cudaSuccess) return e;            \
        KERNEL<<<grid, kThreads, smem, st>>>(w, a, y, m, in_f, out_f, acc_out); \
    } while (0)
    if (acc_out) {
        if constexpr (M == 1) {
            if (dt == DT_Q4K)
                INFR_LAUNCH((gemv_q4k_q8_kernel<1, true>));
            else if (dt == DT_Q6K)
                INFR_LAUNCH((gemv_q6k_q8_kernel<1, true>));
            else
                INFR_LAUNCH((gemv_q2_0_q8_kernel<1, true>));
        } else {
            return cudaErrorInvalidValue;
        }
    } else if (dt == DT_Q4K) {
        INFR_LAUNCH((gemv_q4k_q8_kernel<M, false>));
    } else if (dt == DT_Q6K) {
        INFR_LAUNCH((gemv_q6k_q8_kernel<M, false>));
    } else {
        INFR_LAUNCH((gemv_q2_0_q8_kernel<M, false>));
    }
#undef INFR_LAUNCH
    return cudaGetLastError();
}

template <int M>
cudaError_t launch_f32_m(int dt, const uint8_t *w, const float *x, float *y, int m, int in_f, int out_f,
                         const DeviceInfo &dev, cudaStream_t st) {
    const size_t smem = (size_t)M * in_f * 4;
    if (smem > (size_t)dev.max_smem_optin) return cudaErrorInvalidValue;
    const int grid = grid_for(out_f, smem, dev);
    cudaError_t e;
#define INFR_LAUNCH(KERNEL)                                          \
    do {                                                             \
        if ((e = set_smem(KERNEL, smem)) != cudaSuccess) return e;   \
        KERNEL<<<grid, kThreads, smem, st>>>(w, x, y, m, in_f, out_f); \
    } while (0)
    if (dt == DT_Q4K) {
        if ((e = set_smem(gemv_q4k_f32_kernel<M>, smem)) != cudaSuccess) return e;
        gemv_q4k_f32_kernel<M><<<grid, kThreads, smem, st>>>(w, x, y, m, in_f, out_f, SelArgs{nullptr, 0, 0});
    } else if (dt == DT_Q6K)
        INFR_LAUNCH(gemv_q6k_f32_kernel<M>);
    else
        INFR_LAUNCH(gemv_q2_0_f32_kernel<M>);
#undef INFR_LAUNCH
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemv_q4k_f32_sel(const uint8_t *bank, const int32_t *sel, size_t w_stride, const float *x, int x_div,
                                    float *y, int n_pairs, int in_f, int out_f, const DeviceInfo &dev, cudaStream_t st) {
    const size_t smem = (size_t)in_f * 4;
    if (smem > (size_t)dev.max_smem_optin || n_pairs < 1 || n_pairs > 65535) return cudaErrorInvalidValue;
    cudaError_t e = set_smem(gemv_q4k_f32_kernel<1>, smem);
    if (e != cudaSuccess) return e;
    int gx = (out_f + kWarps - 1) / kWarps;
    const int cap = (dev.sm_count * 4 + n_pairs - 1) / n_pairs;
    if (gx > cap) gx = cap < 1 ? 1 : cap;
    gemv_q4k_f32_kernel<1><<<dim3((unsigned)gx, (unsigned)n_pairs), kThreads, smem, st>>>(bank, x, y, 1, in_f, out_f, SelArgs{sel, w_stride, x_div});
    return cudaGetLastError();
}

cudaError_t launch_grouped_q6k(const uint8_t *bank, const Q8Dev &a, float *y, int in_f, int out_f, const int *item_expert, const int *item_p0,
                               const int *item_cnt, const int *n_items, const int *pair_row, int max_items, const DeviceInfo &dev,
                               cudaStream_t st) {
    if (in_f % 256 || max_items < 1 || !a.sums16 || a.gran != 256) return cudaErrorInvalidValue;
    const size_t smem = q8_smem(DT_Q6K, 8, in_f);
    if (smem > (size_t)dev.max_smem_optin) return cudaErrorInvalidValue;
    cudaError_t e = set_smem(gemv_q6k_q8_grouped_kernel, smem);
    if (e != cudaSuccess) return e;
    // a few CTAs per item (the staged activations are copied by each of them); the SMs fill up across items
    int gx = (out_f + kWarps - 1) / kWarps;
    if (gx > 8) gx = 8;
    gemv_q6k_q8_grouped_kernel<<<dim3((unsigned)gx, (unsigned)max_items), kThreads, smem, st>>>(bank, a, y, in_f, out_f, item_expert, item_p0,
                                                                                              item_cnt, n_items, pair_row);
    return cudaGetLastError();
}

cudaError_t launch_gemv_q8(int dt, const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                           int32_t *acc_out, const DeviceInfo &dev, cudaStream_t st) {
    if (m < 1 || m > 8 || (dt != DT_Q4K && dt != DT_Q6K && dt != DT_Q2_0)) return cudaErrorInvalidValue;
    if (m == 1) return launch_q8_m<1>(dt, w, a, y, m, in_f, out_f, acc_out, dev, st);
    if (acc_out) return cudaErrorInvalidValue;
    if (m == 2) return launch_q8_m<2>(dt, w, a, y, m, in_f, out_f, nullptr, dev, st);
    if (m <= 4) return launch_q8_m<4>(dt, w, a, y, m, in_f, out_f, nullptr, dev, st);
    return launch_q8_m<8>(dt, w, a, y, m, in_f, out_f, nullptr, dev, st);
}

cudaError_t launch_gemv_f32(int dt, const uint8_t *w, const float *x, float *y, int m, int in_f, int out_f,
                            const DeviceInfo &dev, cudaStream_t st) {
    if (m < 1 || m > 8 || (dt != DT_Q4K && dt != DT_Q6K && dt != DT_Q2_0)) return cudaErrorInvalidValue;
    // The f32 staging is 4 bytes per element per token: split wide batches so it fits shared memory.
    if (m == 1) return launch_f32_m<1>(dt, w, x, y, m, in_f, out_f, dev, st);
    if (m == 2 && (size_t)2 * in_f * 4 <= (size_t)dev.max_smem_optin)
        return launch_f32_m<2>(dt, w, x, y, m, in_f, out_f, dev, st);
    if (m <= 4 && (size_t)4 * in_f * 4 <= (size_t)dev.max_smem_optin)
        return launch_f32_m<4>(dt, w, x, y, m, in_f, out_f, dev, st);
    for (int t = 0; t < m; t++) {
        cudaError_t e = launch_f32_m<1>(dt, w, x + (size_t)t * in_f, y + (size_t)t * out_f, 1, in_f, out_f, dev, st);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace infr
