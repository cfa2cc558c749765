// The ops of a dense decode step that sit between the quantized Linears: RMSNorm (optionally fused with the
// residual add in front of it), RoPE, the f16 KV-cache write (optionally fused with RoPE of q and k), causal
// attention over an f16 KV cache with the keys split over CTAs, the SiLU gate, the residual add and argmax.
// Semantics follow the reference's CPU backend op by op (crates/infr-cpu/src/lib.rs: RmsNorm 801-825, Rope
// 1493-1553, WriteKv 1635-1673, Attention 1744-1888, GatedAct 1890-1944, Add 1972-1987, Argmax 2167-2187).
// All of them are HBM- or latency-bound elementwise / reduction kernels; every kernel waits for its producer
// with `griddepcontrol.wait` before its first read, so a chain of them can overlap launch with the tail of
// the previous kernel.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.h"

#include "pdl.cuh"
#include "q8_code.cuh"

namespace infr {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---------------------------------------------------------------------------------------------- RMSNorm
// One CTA per row.  With ADD the row is a + b, which is also written to sum_dst (the residual stream).
template <bool ADD>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const float *a, const float *b, float *sum_dst,  // sum_dst may alias a
                                                        const float *__restrict__ w, float *__restrict__ dst, int dim, float eps) {
    __shared__ float s_part[32];
    __shared__ float s_scale;
    pdl_go();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    const int n4 = (dim & 3) ? 0 : dim >> 2;  // 16-byte accesses only when every row starts on a 16-byte boundary
    float ss = 0.f;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 v = reinterpret_cast<const float4 *>(a + base)[i];
        if (ADD) {
            const float4 u = reinterpret_cast<const float4 *>(b + base)[i];
            v.x += u.x, v.y += u.y, v.z += u.z, v.w += u.w;
            reinterpret_cast<float4 *>(sum_dst + base)[i] = v;
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    for (int i = (n4 << 2) + threadIdx.x; i < dim; i += blockDim.x) {
        float v = a[base + i];
        if (ADD) {
            v += b[base + i];
            sum_dst[base + i] = v;
        }
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x + 31) / 32 ? s_part[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) s_scale = 1.0f / sqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float s = s_scale;
    const float *src = ADD ? sum_dst : a;  // a thread re-reads only what it wrote itself
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(src + base)[i];
        const float4 g = reinterpret_cast<const float4 *>(w)[i];
        reinterpret_cast<float4 *>(dst + base)[i] = make_float4(v.x * s * g.x, v.y * s * g.y, v.z * s * g.z, v.w * s * g.w);
    }
    for (int i = (n4 << 2) + threadIdx.x; i < dim; i += blockDim.x) dst[base + i] = src[base + i] * s * w[i];
}

// ---------------------------------------------------------------------------------------------- RoPE
// theta^(-2p/rope_dim): the exponent is formed in f32 like the reference's, the power in f64 and rounded once,
// which is what a correctly rounded f32 powf returns.
__device__ __forceinline__ float rope_freq(float theta, int p, int rope_dim) {
    const float e = -2.0f * (float)p / (float)rope_dim;
    return (float)pow((double)theta, (double)e);
}

__device__ __forceinline__ void rope_pair(float a, float b, float ang, float *oa, float *ob) {
    const float sn = sinf(ang), c = cosf(ang);
    *oa = a * c - b * sn;
    *ob = a * sn + b * c;
}

// thread = (row, head, pair or pass-through element)
__global__ void __launch_bounds__(256) rope_kernel(const float *__restrict__ x, const int32_t *__restrict__ positions,
                                                   float *__restrict__ dst, int rows, int n_head, int head_dim, int rope_dim,
                                                   float theta, int neox) {
    pdl_go();
    pdl_wait();
    const int hf = rope_dim / 2, per_head = hf + (head_dim - rope_dim);
    const size_t total = (size_t)rows * n_head * per_head;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int e = (int)(i % per_head);
        const size_t rh = i / per_head;
        const int r = (int)(rh / n_head);
        const size_t b = rh * head_dim;
        if (e < hf) {
            const int i0 = neox ? e : 2 * e, i1 = neox ? e + hf : 2 * e + 1;
            const float ang = (float)positions[r] * rope_freq(theta, e, rope_dim);
            float oa, ob;
            rope_pair(x[b + i0], x[b + i1], ang, &oa, &ob);
            dst[b + i0] = oa;
            dst[b + i1] = ob;
        } else {
            const int j = rope_dim + (e - hf);
            dst[b + j] = x[b + j];
        }
    }
}

// RoPE of q in place, RoPE of k straight into the f16 K cache, v into the f16 V cache: one launch instead of
// Rope, Rope, WriteKv, WriteKv (crates/infr-llama/src/seam/runner.rs:3611-3656).  Row r belongs to sequence
// r / rows_per_seq, whose caches start seq_stride elements after the previous sequence's, and lands at cache
// row positions[r].  Full-head rotation only (rope_dim == head_dim).
constexpr int kPageRows = 128;  // rows of a page of a paged KV cache = keys of an attention tile
__global__ void __launch_bounds__(256) rope_write_kv_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                            const int32_t *__restrict__ positions, __half *__restrict__ k_cache,
                                                            __half *__restrict__ v_cache, int rows, int n_head, int n_kv, int head_dim,
                                                            float theta, int neox, int rows_per_seq, size_t seq_stride, int write_pos,
                                                            const int32_t *__restrict__ block_table, int table_stride, int n_pages) {
    pdl_go();
    pdl_wait();
    const int hf = head_dim / 2;
    const size_t nq = (size_t)rows * n_head * hf, nk = (size_t)rows * n_kv * hf, total = nq + 2 * nk;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        if (i < nq) {
            const int p = (int)(i % hf);
            const size_t rh = i / hf;
            const int r = (int)(rh / n_head);
            const size_t b = rh * head_dim;
            const int i0 = neox ? p : 2 * p, i1 = neox ? p + hf : 2 * p + 1;
            float oa, ob;
            rope_pair(q[b + i0], q[b + i1], (float)positions[r] * rope_freq(theta, p, head_dim), &oa, &ob);
            q[b + i0] = oa;
            q[b + i1] = ob;
        } else {
            const bool is_v = i >= nq + nk;
            const size_t t = i - nq - (is_v ? nk : 0);
            const int p = (int)(t % hf);
            const size_t rh = t / hf;  // row * n_kv + head
            const int r = (int)(rh / n_kv), h = (int)(rh % n_kv);
            const size_t b = rh * head_dim;
            // cache row: the op's own `pos` + row when the caller gives one (Op::WriteKv), else the row's position
            const size_t crow = write_pos >= 0 ? (size_t)(write_pos + r % rows_per_seq) : (size_t)positions[r];
            size_t cb;
            if (block_table) {  // paged caches: row crow of the sequence lives in page table[seq][crow / 128] of the pool
                const int pg = min(max(block_table[(size_t)(r / rows_per_seq) * table_stride + crow / kPageRows], 0), n_pages - 1);
                cb = (((size_t)pg * kPageRows + crow % kPageRows) * n_kv + h) * head_dim;
            } else {
                cb = (size_t)(r / rows_per_seq) * seq_stride + (crow * n_kv + h) * head_dim;
            }
            if (is_v) {
                v_cache[cb + 2 * p] = __float2half_rn(v[b + 2 * p]);
                v_cache[cb + 2 * p + 1] = __float2half_rn(v[b + 2 * p + 1]);
            } else {
                const int i0 = neox ? p : 2 * p, i1 = neox ? p + hf : 2 * p + 1;
                float oa, ob;
                rope_pair(k[b + i0], k[b + i1], (float)positions[r] * rope_freq(theta, p, head_dim), &oa, &ob);
                k_cache[cb + i0] = __float2half_rn(oa);
                k_cache[cb + i1] = __float2half_rn(ob);
            }
        }
    }
}

__global__ void __launch_bounds__(256) write_kv_kernel(const float *__restrict__ src, __half *__restrict__ cache, size_t n) {
    pdl_go();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        cache[i] = __float2half_rn(src[i]);
}

// ---------------------------------------------------------------------------------------------- attention
constexpr int kAttnTile = 128;     // keys per CTA
constexpr int kAttnThreads = 256;  // eight warps: 16 keys each in the score phase, 16 output dims each in the value phase

// CTA = (key tile, KV head, query row).  The tile's 128 key rows and 128 value rows (head_dim halves each) are
// copied into shared memory with 16-byte cp.async, consecutive threads taking consecutive 16-byte pieces of a row, so
// every global request is a whole 128-byte line; all copies of the CTA are in flight together and none occupies a
// register.
//
// Both products run on the warp-level matrix unit in tf32 WITHOUT giving up f32 operands: an f16 cache value is exact
// in tf32 (10 mantissa bits), and the f32 operand (q, then the softmax weights p) is split into two tf32 pieces,
// hi = the top 11 significant bits, mid = the next 11 of the remainder, which sit in two neighbouring columns of the
// instruction's N dimension and are added afterwards; what is dropped is below 2^-22 of the operand, the size of the
// rounding of an f32 accumulation itself.  Products are exact, sums are f32.  This takes the instruction count of a tile
// from ~7100 (scalar FMAs on converted halves, which cost more issue slots than the tile's bytes cost HBM time) to
// ~2800.
// Phase 1: warp w scores keys 16w..16w+15 against the G query heads that share the KV head: A = the keys (ldmatrix,
// halves -> f32), B = the q pieces, K = head_dim in steps of 8.  Phase 2: one warp per head turns the tile's scores into
// exp(s - m), their sum, and the two tf32 pieces of each weight.  Phase 3: warp w owns output dims 16 (w mod HD/16):
// A = the values transposed (ldmatrix.trans), B = the weight pieces, K = the keys in steps of 8; with head_dim 64 the
// two halves of the keys go to two warps and meet in shared memory (over the key tile, dead by then).  The tile's
// (m, l, o) goes to the workspace for the merge kernel.
// The K index of the instruction is only a summation index: slot t takes element 2t of a group of 8 and slot t + 4
// element 2t + 1, which is how ldmatrix hands out halves in pairs.
template <int HD>
struct AttnSmem {
    static constexpr int kKeyStride = HD * 2 + 16;  // bytes; 16 past a multiple of 128: the 8 rows of an ldmatrix hit distinct banks
    static constexpr int kValStride = HD * 2 + 16;
    static constexpr int kBytes = kAttnTile * (kKeyStride + kValStride);
};

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Bounded wait for phase 0 of a copy barrier.
__device__ __forceinline__ bool attn_wait(uint64_t *bar) {
    const uint32_t b = (uint32_t)__cvta_generic_to_shared(bar);
    for (uint32_t i = 0; i < (1u << 22); i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(b), "r"(0u)
                     : "memory");
        if (ok) return true;
    }
    return false;
}

// Four 8x8 matrices of halves; lane l supplies the address of row l % 8 of matrix l / 8.  Plain: thread (g, t) gets
// elements [g][2t], [g][2t+1] of each matrix; .trans: elements [2t][g], [2t+1][g].
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void *row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(row)));
}
__device__ __forceinline__ void ldsm4_trans(uint32_t (&r)[4], const void *row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(row)));
}
// D += A(16x8, tf32) * B(8x8, tf32), f32 accumulate
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the two halves of a word as f32 bit patterns (exact, and representable in tf32)
__device__ __forceinline__ void half2_bits(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    lo = __float_as_uint(f.x);
    hi = __float_as_uint(f.y);
}
// tf32 pieces of an f32 value: piece 0 = its top 11 significant bits, piece 1 = the top 11 of what is left
__device__ __forceinline__ uint32_t tf32_piece(float v, int piece) {
    const uint32_t hi = __float_as_uint(v) & 0xFFFFE000u;
    return piece == 0 ? hi : (__float_as_uint(v - __uint_as_float(hi)) & 0xFFFFE000u);
}

template <int HD, int G, bool BULK>
__global__ void __launch_bounds__(kAttnThreads) attn_split_kernel(const float *__restrict__ q, const __half *__restrict__ k_cache,
                                                               const __half *__restrict__ v_cache, float *__restrict__ part_o,
                                                               float *__restrict__ part_ml, int rows, int n_head, int n_kv, int pos,
                                                               float scale, int n_splits, size_t seq_stride, uint32_t *__restrict__ status,
                                                               const int32_t *__restrict__ seq_pos, const int32_t *__restrict__ block_table,
                                                               int table_stride, int n_pages) {
    constexpr int CPR = HD * 2 / 16;           // 16-byte pieces per row
    constexpr int NT = (2 * G + 7) / 8;        // 8-column groups of the instruction: column c = head c / 2, piece c % 2
    constexpr int DG = HD / 16;                // 16-dim output groups
    constexpr int KP = (kAttnThreads / 32) / DG;  // warps per output group: they split the keys (1 for head_dim 128, 2 for 64)
    using L = AttnSmem<HD>;
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t *s_k = dyn_smem, *s_v = dyn_smem + kAttnTile * L::kKeyStride;
    float(*s_o)[G][HD] = reinterpret_cast<float(*)[G][HD]>(dyn_smem);  // KP x G x HD floats over the key tile (KP > 1 only)
    __shared__ __align__(16) float s_q[G * HD];
    __shared__ __align__(16) float s_pp[2][G][kAttnTile];  // [0]: scores, then the hi pieces of exp(s - m); [1]: the mid pieces
    __shared__ float s_ml[G][2];
    __shared__ __align__(8) uint64_t s_bar[2];
    static_assert(KP * G * HD * 4 <= kAttnTile * L::kKeyStride, "the partial outputs reuse the key tile");
    static_assert(KP >= 1 && KP * DG == kAttnThreads / 32, "head_dim 64 or 128");
    const int split = blockIdx.x, kvh = blockIdx.y, qr = blockIdx.z;
    const int seq = qr / rows, ti = qr % rows;
    const int key0 = split * kAttnTile;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
    pdl_go();
    pdl_wait();
    // sequences at positions of their own (seq_pos, written by an earlier kernel or the host): `pos` is their maximum
    const int n_keys = (seq_pos ? max(0, min(seq_pos[seq], pos)) : pos) + ti + 1;
    const size_t out_idx = ((size_t)qr * n_head + (size_t)kvh * G) * n_splits + split;  // + g * n_splits
    if (key0 >= n_keys) {  // a tile beyond this row's causal end contributes nothing
        if (tid < G) {
            part_ml[(out_idx + (size_t)tid * n_splits) * 2] = -INFINITY;
            part_ml[(out_idx + (size_t)tid * n_splits) * 2 + 1] = 0.f;
        }
        return;
    }
    const size_t kv_row = (size_t)n_kv * HD;
    // contiguous caches: the sequence's own; paged: the tile is one page of the pool (a page holds a tile's 128 rows)
    const size_t tile_off = block_table ? (size_t)min(max(block_table[(size_t)seq * table_stride + split], 0), n_pages - 1) * kAttnTile * kv_row
                                        : (size_t)seq * seq_stride + (size_t)key0 * kv_row;
    const __half *kbase = k_cache + (size_t)kvh * HD + tile_off;
    const __half *vbase = v_cache + (size_t)kvh * HD + tile_off;
    const int tile_keys = min(kAttnTile, n_keys - key0);
    // Two ways to fetch the tile.  BULK (many CTAs per SM over the launch: a batch of sequences): one bulk copy per row
    // (head_dim halves, contiguous in the cache) into the padded tile, thread r < 128 the key row r, thread 128 + r the
    // value row r, so a tile costs each warp two instructions instead of 32 cp.async with their address arithmetic (a
    // third of the kernel's instructions); keys and values complete on separate barriers.  Otherwise (a single wave of
    // CTAs, where the latency of the first byte is what counts): 16-byte cp.async, consecutive threads taking consecutive
    // pieces of a row.  Rows past the end of a partial tile are zeroed, so that the matrix unit multiplies 0 (not stale
    // bits) by the weight 0.
    if (BULK) {
        if (tid == 0) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t b = (uint32_t)__cvta_generic_to_shared(&s_bar[i]);
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b) : "memory");
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"((uint32_t)(tile_keys * HD * 2)) : "memory");
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();  // the barriers are armed before any copy can complete
        const int which = tid >> 7, r = tid & (kAttnTile - 1);  // 0: key row r, 1: value row r
        uint8_t *dst = (which ? s_v + r * L::kValStride : s_k + r * L::kKeyStride);
        if (r < tile_keys) {
            const __half *src = (which ? vbase : kbase) + (size_t)r * kv_row;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(dst)),
                         "l"(src), "r"((uint32_t)(HD * 2)), "r"((uint32_t)__cvta_generic_to_shared(&s_bar[which]))
                         : "memory");
        } else {
#pragma unroll
            for (int c = 0; c < CPR; c++) *reinterpret_cast<uint4 *>(dst + c * 16) = make_uint4(0, 0, 0, 0);
        }
    } else {
        for (int i = tid; i < tile_keys * CPR; i += kAttnThreads) {
            const int key = i / CPR, c = i % CPR;
            cp_async16(s_k + key * L::kKeyStride + c * 16, kbase + (size_t)key * kv_row + c * 8);
        }
        cp_async_commit();
        for (int i = tid; i < tile_keys * CPR; i += kAttnThreads) {
            const int key = i / CPR, c = i % CPR;
            cp_async16(s_v + key * L::kValStride + c * 16, vbase + (size_t)key * kv_row + c * 8);
        }
        cp_async_commit();
        for (int i = tid; i < (kAttnTile - tile_keys) * CPR; i += kAttnThreads) {
            const int key = tile_keys + i / CPR, c = i % CPR;
            *reinterpret_cast<uint4 *>(s_k + key * L::kKeyStride + c * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(s_v + key * L::kValStride + c * 16) = make_uint4(0, 0, 0, 0);
        }
    }
    const float *qrow = q + ((size_t)qr * n_head + (size_t)kvh * G) * HD;
    for (int i = tid; i < G * HD; i += kAttnThreads) s_q[i] = qrow[i];
    // the keys have landed; q is staged, the zeroed rows are in place.  (BULK: a bounded wait; if it runs out, the CTA
    // records it and leaves after the wait for the values has had its own limit, so that no copy can land in shared
    // memory that is no longer this CTA's.)
    if (BULK) {
        const bool k_ok = attn_wait(&s_bar[0]);
        if (!__syncthreads_and(k_ok)) {
            attn_wait(&s_bar[1]);
            if (tid == 0) atomicExch(status, 12u);
            return;
        }
    } else {
        cp_async_wait<1>();
        __syncthreads();
    }
    // ---- phase 1: scores of keys 16 warp .. 16 warp + 15
    {
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        // ldmatrix rows: matrices 0 / 1 = keys 0..7 / 8..15 at dims d0.., matrices 2 / 3 = the same keys at dims d0 + 8..
        const uint8_t *arow = s_k + (size_t)(16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8) * L::kKeyStride + (lane >> 4) * 16;
#pragma unroll 4
        for (int j = 0; j < HD / 16; j++) {
            uint32_t r[4];
            ldsm4(r, arow + j * 32);
            uint32_t a[2][4];  // [dim group of 8][a0..a3]
            half2_bits(r[0], a[0][0], a[0][2]);  // keys g8:     (slot t4, slot t4 + 4) = dims 2 t4, 2 t4 + 1
            half2_bits(r[1], a[0][1], a[0][3]);  // keys g8 + 8
            half2_bits(r[2], a[1][0], a[1][2]);
            half2_bits(r[3], a[1][1], a[1][3]);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int c = nt * 8 + g8, head = c >> 1, piece = c & 1;  // this lane's B column
                float2 q0 = make_float2(0.f, 0.f), q1 = q0;
                if (head < G) {
                    q0 = *reinterpret_cast<const float2 *>(s_q + head * HD + j * 16 + 2 * t4);
                    q1 = *reinterpret_cast<const float2 *>(s_q + head * HD + j * 16 + 8 + 2 * t4);
                }
                mma_tf32(acc[nt], a[0][0], a[0][1], a[0][2], a[0][3], tf32_piece(q0.x, piece), tf32_piece(q0.y, piece));
                mma_tf32(acc[nt], a[1][0], a[1][1], a[1][2], a[1][3], tf32_piece(q1.x, piece), tf32_piece(q1.y, piece));
            }
        }
        // columns 2 t4, 2 t4 + 1 of group nt = the two pieces of head 4 nt + t4; rows g8 and g8 + 8 of the warp's keys
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int head = nt * 4 + t4;
            if (head < G) {
                s_pp[0][head][16 * warp + g8] = acc[nt][0] + acc[nt][1];
                s_pp[0][head][16 * warp + g8 + 8] = acc[nt][2] + acc[nt][3];
            }
        }
    }
    // the values have landed; scores complete, key tile no longer read
    if (BULK) {
        const bool v_ok = attn_wait(&s_bar[1]);
        if (!__syncthreads_and(v_ok)) {
            if (tid == 0) atomicExch(status, 12u);
            return;
        }
    } else {
        cp_async_wait<0>();
        __syncthreads();
    }
    // ---- phase 2
    for (int g = warp; g < G; g += kAttnThreads / 32) {
        float v[4], m = -INFINITY;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int key = lane + 32 * e;
            v[e] = key < tile_keys ? s_pp[0][g][key] * scale : -INFINITY;
            m = fmaxf(m, v[e]);
        }
        m = warp_max(m);  // finite: the tile holds at least one valid key
        float l = 0.f;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float p = expf(v[e] - m);
            s_pp[0][g][lane + 32 * e] = __uint_as_float(tf32_piece(p, 0));
            s_pp[1][g][lane + 32 * e] = __uint_as_float(tf32_piece(p, 1));
            l += p;
        }
        l = warp_sum(l);
        if (lane == 0) s_ml[g][0] = m, s_ml[g][1] = l;
    }
    __syncthreads();
    // ---- phase 3: output dims 16 dg .. + 15 over this warp's share of the keys
    {
        const int dg = warp % DG, kp = warp / DG;
        constexpr int KEYS = kAttnTile / KP;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        // ldmatrix.trans rows: matrices 0 / 1 = keys 0..7 at dims 0..7 / 8..15 of the group, matrices 2 / 3 = keys 8..15
        const uint8_t *vrow = s_v + (size_t)(kp * KEYS + (lane & 7) + (lane >> 4) * 8) * L::kValStride + (size_t)(16 * dg + ((lane >> 3) & 1) * 8) * 2;
#pragma unroll 4
        for (int s16 = 0; s16 < KEYS / 16; s16++) {
            uint32_t r[4];
            ldsm4_trans(r, vrow + (size_t)s16 * 16 * L::kValStride);
            uint32_t a[2][4];  // [key group of 8][a0..a3]
            half2_bits(r[0], a[0][0], a[0][2]);  // dims g8:     (slot t4, slot t4 + 4) = keys 2 t4, 2 t4 + 1
            half2_bits(r[1], a[0][1], a[0][3]);  // dims g8 + 8
            half2_bits(r[2], a[1][0], a[1][2]);
            half2_bits(r[3], a[1][1], a[1][3]);
            const int k0 = kp * KEYS + s16 * 16 + 2 * t4;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int c = nt * 8 + g8, head = c >> 1, piece = c & 1;
                float2 p0 = make_float2(0.f, 0.f), p1 = p0;
                if (head < G) {
                    p0 = *reinterpret_cast<const float2 *>(&s_pp[piece][head][k0]);
                    p1 = *reinterpret_cast<const float2 *>(&s_pp[piece][head][k0 + 8]);
                }
                mma_tf32(acc[nt], a[0][0], a[0][1], a[0][2], a[0][3], __float_as_uint(p0.x), __float_as_uint(p0.y));
                mma_tf32(acc[nt], a[1][0], a[1][1], a[1][2], a[1][3], __float_as_uint(p1.x), __float_as_uint(p1.y));
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int head = nt * 4 + t4;
            if (head < G) {
                const float o0 = acc[nt][0] + acc[nt][1], o1 = acc[nt][2] + acc[nt][3];  // dims 16 dg + g8, + 8
                if (KP == 1) {
                    float *po = part_o + (out_idx + (size_t)head * n_splits) * HD + 16 * dg + g8;
                    po[0] = o0;
                    po[8] = o1;
                } else {
                    s_o[kp][head][16 * dg + g8] = o0;
                    s_o[kp][head][16 * dg + g8 + 8] = o1;
                }
            }
        }
    }
    if (KP > 1) {
        __syncthreads();
        for (int i = tid; i < G * HD; i += kAttnThreads) {
            const int g = i / HD, d = i % HD;
            float t = s_o[0][g][d];
#pragma unroll
            for (int w = 1; w < KP; w++) t += s_o[w][g][d];
            part_o[(out_idx + (size_t)g * n_splits) * HD + d] = t;
        }
    }
    if (tid < G) {
        part_ml[(out_idx + (size_t)tid * n_splits) * 2] = s_ml[tid][0];
        part_ml[(out_idx + (size_t)tid * n_splits) * 2 + 1] = s_ml[tid][1];
    }
}

// CTA = (query row, head), thread = output dim: merges the tiles' (m, l, o).
__global__ void attn_combine_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, float *__restrict__ dst,
                                    int head_dim, int n_splits) {
    pdl_go();
    pdl_wait();
    const size_t rh = blockIdx.x;
    const float *ml = part_ml + rh * n_splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, ml[2 * s]);
    float l = 0.f, o = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ls = ml[2 * s + 1];
        if (ls == 0.f) continue;
        const float wgt = expf(ml[2 * s] - m);
        l += wgt * ls;
        o = fmaf(wgt, part_o[(rh * n_splits + s) * head_dim + threadIdx.x], o);
    }
    dst[rh * head_dim + threadIdx.x] = o / l;
}

// ---------------------------------------------------------------------------------------------- elementwise
__global__ void __launch_bounds__(256) gated_silu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                         float *__restrict__ dst, size_t n) {
    pdl_go();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float g = gate[i];
        dst[i] = g / (1.0f + expf(-g)) * up[i];
    }
}

__global__ void __launch_bounds__(256) add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ dst, size_t n) {
    pdl_go();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = a[i] + b[i];
}

// Strict `>` with the lowest index on ties, per row.  Stage 1: CTA (chunk, row) -> best of its chunk;
// stage 2: one CTA per row over the chunk winners.
__device__ __forceinline__ void argmax_merge(float &bv, uint32_t &bi, float v, uint32_t i) {
    if (v > bv || (v == bv && i < bi)) bv = v, bi = i;
}
__device__ __forceinline__ void argmax_block(float bv, uint32_t bi, float *s_v, uint32_t *s_i, float *ov, uint32_t *oi) {
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t i = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_merge(bv, bi, v, i);
    }
    if ((threadIdx.x & 31) == 0) s_v[threadIdx.x >> 5] = bv, s_i[threadIdx.x >> 5] = bi;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = (blockDim.x + 31) / 32;
        bv = threadIdx.x < nw ? s_v[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? s_i[threadIdx.x] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float v = __shfl_xor_sync(0xffffffffu, bv, o);
            const uint32_t i = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_merge(bv, bi, v, i);
        }
        if (threadIdx.x == 0) *ov = bv, *oi = bi;
    }
}

__global__ void __launch_bounds__(256) argmax_stage1_kernel(const float *__restrict__ x, float *__restrict__ cand_v,
                                                            uint32_t *__restrict__ cand_i, uint32_t n, uint32_t chunk) {
    __shared__ float s_v[32];
    __shared__ uint32_t s_i[32];
    pdl_go();
    pdl_wait();
    const uint32_t lo = blockIdx.x * chunk, hi = min(n, lo + chunk);
    const float *row = x + (size_t)blockIdx.y * n;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_merge(bv, bi, row[i], i);
    argmax_block(bv, bi, s_v, s_i, cand_v + (size_t)blockIdx.y * gridDim.x + blockIdx.x, cand_i + (size_t)blockIdx.y * gridDim.x + blockIdx.x);
}

__global__ void __launch_bounds__(256) argmax_stage2_kernel(const float *__restrict__ cand_v, const uint32_t *__restrict__ cand_i,
                                                            uint32_t *__restrict__ dst, uint32_t n_chunks) {
    __shared__ float s_v[32];
    __shared__ uint32_t s_i[32];
    __shared__ float s_bv;
    __shared__ uint32_t s_bi;
    pdl_go();
    pdl_wait();
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t c = threadIdx.x; c < n_chunks; c += blockDim.x)
        argmax_merge(bv, bi, cand_v[(size_t)blockIdx.x * n_chunks + c], cand_i[(size_t)blockIdx.x * n_chunks + c]);
    argmax_block(bv, bi, s_v, s_i, &s_bv, &s_bi);
    __syncthreads();
    // a row with no value above -inf (all -inf or NaN) answers index 0, like the reference's scan
    if (threadIdx.x == 0) dst[blockIdx.x] = s_bi == 0xffffffffu ? 0u : s_bi;
}

// ---------------------------------------------------------------------------------------------- producers that emit int8
// The activation quantiser's arithmetic for one 256-element block held by one warp (lane l owns elements 4l..4l+3
// and 128+4l..128+4l+3): d = amax / 127, id = d > 0 ? 1/d : 0, q = clamp(roundf(x * id), -127, 127), plus the
// per-32 and per-16 code sums (crates/infr-cpu/src/quant.rs:27-58).  Same operations in the same order as
// quantize_q8_kernel<256>, so a producer that ends with this emits the bits the separate quantiser would.
__device__ __forceinline__ float q8_amax4(float4 v) { return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))); }
__device__ __forceinline__ int q8_code(float v, float id) { return q8_round_code(v, id); }
__device__ __forceinline__ void quantize_block256(const float4 v[2], int lane, size_t row, int k, int chunk, int8_t *__restrict__ qs,
                                                  float *__restrict__ d, int32_t *__restrict__ sums, int32_t *__restrict__ sums16) {
    float m = fmaxf(q8_amax4(v[0]), q8_amax4(v[1]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float dd = m / 127.0f;
    const float id = dd > 0.0f ? 1.0f / dd : 0.0f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int e = chunk * 256 + h * 128 + lane * 4;
        const int q0 = q8_code(v[h].x, id), q1 = q8_code(v[h].y, id), q2 = q8_code(v[h].z, id), q3 = q8_code(v[h].w, id);
        int sm = q0 + q1 + q2 + q3;
        sm += __shfl_xor_sync(0xffffffffu, sm, 1);
        sm += __shfl_xor_sync(0xffffffffu, sm, 2);
        const int s16 = sm;
        sm += __shfl_xor_sync(0xffffffffu, sm, 4);
        const uint32_t packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        *reinterpret_cast<uint32_t *>(qs + row * k + e) = packed;
        if (sums16 && (lane & 3) == 0) sums16[row * (k / 16) + e / 16] = s16;
        if ((lane & 7) == 0) sums[row * (k / 32) + e / 32] = sm;
    }
    if (lane == 0) d[row * (k / 256) + chunk] = dd;
}

// Sum of squares of four values with every product and sum rounded on its own (no fused multiply-add): two kernels
// that share this get the same bits whatever the compiler does around it, and it is how the CPU forms the sum.
__device__ __forceinline__ float sumsq4(const float4 v) {
    return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(v.x, v.x), __fmul_rn(v.y, v.y)), __fmul_rn(v.z, v.z)), __fmul_rn(v.w, v.w));
}

// RMSNorm (optionally of a + b, written to sum_dst) whose output goes straight to int8; dim % 256 == 0.
// Warp c owns the 256-element blocks c, c + warps, ...; with one block per warp (dim <= 256 * warps, the launcher's
// choice up to dim 8192) the row stays in registers between the sum of squares and the scaling.
// With Q8 false the scaled row is stored as f32 to dst instead: the same arithmetic, so both forms agree bit for bit.
template <bool ADD, bool Q8>
__global__ void __launch_bounds__(1024) rms_norm_q8_kernel(const float *a, const float *b, float *sum_dst, const float *__restrict__ w, int dim,
                                                           float eps, float *__restrict__ dst, int8_t *__restrict__ qs, float *__restrict__ d,
                                                           int32_t *__restrict__ sums, int32_t *__restrict__ sums16) {
    __shared__ float s_part[32];
    __shared__ float s_scale;
    pdl_go();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, chunks = dim / 256;
    const bool in_regs = chunks <= nw;
    // the norm weights do not depend on the previous kernel: fetch them before waiting for it
    float4 g[2];
    if (in_regs && warp < chunks) {
#pragma unroll
        for (int h = 0; h < 2; h++) g[h] = *reinterpret_cast<const float4 *>(w + warp * 256 + h * 128 + lane * 4);
    }
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    float4 x[2];
    float ss = 0.f;
    for (int chunk = warp; chunk < chunks; chunk += nw) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = chunk * 256 + h * 128 + lane * 4;
            float4 v = *reinterpret_cast<const float4 *>(a + base + e);
            if (ADD) {
                const float4 u = *reinterpret_cast<const float4 *>(b + base + e);
                v.x += u.x, v.y += u.y, v.z += u.z, v.w += u.w;
                *reinterpret_cast<float4 *>(sum_dst + base + e) = v;
            }
            ss = __fadd_rn(ss, sumsq4(v));
            x[h] = v;
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? s_part[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) s_scale = 1.0f / sqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float s = s_scale;
    const float *src = (ADD ? sum_dst : a) + base;  // re-read by the warp that wrote it
    for (int chunk = warp; chunk < chunks; chunk += nw) {
        float4 v[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = chunk * 256 + h * 128 + lane * 4;
            if (!in_regs) {
                x[h] = *reinterpret_cast<const float4 *>(src + e);
                g[h] = *reinterpret_cast<const float4 *>(w + e);
            }
            v[h] = make_float4(x[h].x * s * g[h].x, x[h].y * s * g[h].y, x[h].z * s * g[h].z, x[h].w * s * g[h].w);
        }
        if (Q8) {
            quantize_block256(v, lane, blockIdx.x, dim, chunk, qs, d, sums, sums16);
        } else {
#pragma unroll
            for (int h = 0; h < 2; h++) *reinterpret_cast<float4 *>(dst + base + chunk * 256 + h * 128 + lane * 4) = v[h];
        }
    }
}

// The consumer of a pushed row-parallel GEMV (GemvPush): row = a + sum over ranks of the partial results that the
// ranks' GEMV epilogues stored into this rank's staging, summed in rank order from zero (the order of the stand-alone
// all-reduce, so both forms give the same bits), written to sum_dst, then RMSNorm and the quantiser.  Every staged word
// carries its value and the exchange's sequence number: a thread polls, bounded, the four words of each rank that it
// is about to add, so nothing waits for data it does not read.  A thread whose poll runs out adds nothing and raises
// the status word.  The grid's last CTA opens the next exchange.  One CTA per row, dim % 256 == 0.
__device__ __forceinline__ void ld_words2(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__global__ void __launch_bounds__(1024) rms_norm_q8_pull_kernel(const float *a, float *sum_dst, const float *__restrict__ w, int dim, float eps,
                                                                int8_t *__restrict__ qs, float *__restrict__ d, int32_t *__restrict__ sums,
                                                                int32_t *__restrict__ sums16, PullArgs pull) {
    __shared__ float s_part[32];
    __shared__ float s_scale;
    pdl_go();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, chunks = dim / 256;
    const bool in_regs = chunks <= nw;
    // the norm weights do not depend on the previous kernel: fetch them before waiting for it
    float4 g[2];
    if (in_regs && warp < chunks) {
#pragma unroll
        for (int h = 0; h < 2; h++) g[h] = *reinterpret_cast<const float4 *>(w + warp * 256 + h * 128 + lane * 4);
    }
    pdl_wait();
    const uint32_t done = *reinterpret_cast<volatile uint32_t *>(pull.ctrl);
    const uint32_t par = done & 1u, want = done + 1u;
    const size_t base = (size_t)blockIdx.x * dim;
    float4 x[2];
    float ss = 0.f;
    for (int chunk = warp; chunk < chunks; chunk += nw) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = chunk * 256 + h * 128 + lane * 4;
            float4 v = *reinterpret_cast<const float4 *>(a + base + e);  // the residual row does not depend on the peers
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            bool all = true;
            for (int r = 0; r < pull.world; r++) {
                const unsigned long long *src = pull.stage + ((size_t)par * pull.world + r) * pull.cap + base + e;
                unsigned long long w0, w1, w2, w3;
                uint32_t it = 0;
                bool ok;
                do {
                    ld_words2(src, w0, w1);
                    ld_words2(src + 2, w2, w3);
                    ok = (uint32_t)(w0 >> 32) == want && (uint32_t)(w1 >> 32) == want && (uint32_t)(w2 >> 32) == want && (uint32_t)(w3 >> 32) == want;
                } while (!ok && ++it < pull.spin);
                all = all && ok;
                acc.x += __uint_as_float((uint32_t)w0), acc.y += __uint_as_float((uint32_t)w1);
                acc.z += __uint_as_float((uint32_t)w2), acc.w += __uint_as_float((uint32_t)w3);
            }
            if (all)
                v.x += acc.x, v.y += acc.y, v.z += acc.z, v.w += acc.w;
            else
                atomicExch(pull.status, 11u);
            *reinterpret_cast<float4 *>(sum_dst + base + e) = v;
            ss = __fadd_rn(ss, sumsq4(v));
            x[h] = v;
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? s_part[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) s_scale = 1.0f / sqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float s = s_scale;
    for (int chunk = warp; chunk < chunks; chunk += nw) {
        float4 v[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = chunk * 256 + h * 128 + lane * 4;
            if (!in_regs) {
                x[h] = *reinterpret_cast<const float4 *>(sum_dst + base + e);  // re-read by the warp that wrote it
                g[h] = *reinterpret_cast<const float4 *>(w + e);
            }
            v[h] = make_float4(x[h].x * s * g[h].x, x[h].y * s * g[h].y, x[h].z * s * g[h].z, x[h].w * s * g[h].w);
        }
        quantize_block256(v, lane, blockIdx.x, dim, chunk, qs, d, sums, sums16);
    }
    // every CTA has read the count and its words: the last one opens the next exchange
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(pull.ctrl + 1, 1u) == gridDim.x - 1) {
            pull.ctrl[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(pull.ctrl) = done + 1u;
        }
    }
}

// silu(gate) * up straight to int8: warp = (row, 256-element block); nff % 256 == 0.
__global__ void __launch_bounds__(256) gated_silu_q8_kernel(const float *__restrict__ gate, const float *__restrict__ up, int rows, int nff,
                                                            int8_t *__restrict__ qs, float *__restrict__ d, int32_t *__restrict__ sums,
                                                            int32_t *__restrict__ sums16) {
    pdl_go();
    pdl_wait();
    const int lane = threadIdx.x & 31, cpr = nff / 256;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)rows * cpr) return;
    const int row = (int)(wg / cpr), chunk = (int)(wg % cpr);
    float4 v[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const size_t e = (size_t)row * nff + chunk * 256 + h * 128 + lane * 4;
        const float4 g = *reinterpret_cast<const float4 *>(gate + e), u = *reinterpret_cast<const float4 *>(up + e);
        v[h] = make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y, g.z / (1.0f + expf(-g.z)) * u.z,
                           g.w / (1.0f + expf(-g.w)) * u.w);
    }
    quantize_block256(v, lane, (size_t)row, nff, chunk, qs, d, sums, sums16);
}

// The merge of the key tiles with the result quantised in place of an f32 store.  CTA = (query row, 256 outputs),
// 8 warps: warp h < heads-per-block first turns head h's tile maxima into weights exp(m_s - M) in shared memory,
// then warp w accumulates tiles w, w + 8, ... for the block's 256 outputs (lane = 2 x 4 dims), the eight partial
// sums meet in shared memory and warp 0 normalises and quantises.
// With Q8 false the same sums are stored as f32 instead, so the two forms agree bit for bit.
constexpr int kCombineMaxSplits = 512;
template <bool Q8>
__global__ void __launch_bounds__(256) attn_combine_wide_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int n_head,
                                                                int head_dim, int n_splits, float *__restrict__ dst, int8_t *__restrict__ qs,
                                                                float *__restrict__ d, int32_t *__restrict__ sums, int32_t *__restrict__ sums16) {
    __shared__ float s_w[4][kCombineMaxSplits];
    __shared__ float s_l[4];
    __shared__ __align__(16) float s_acc[8][256];
    pdl_go();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, k = n_head * head_dim, cpr = k / 256;
    const int row = blockIdx.x / cpr, chunk = blockIdx.x % cpr;
    const int heads = 256 / head_dim, head0 = chunk * heads;
    if (warp < heads) {
        const float *ml = part_ml + ((size_t)row * n_head + head0 + warp) * n_splits * 2;
        float m = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, ml[2 * s]);
        m = warp_max(m);
        float l = 0.f;
        for (int s = lane; s < n_splits; s += 32) {
            const float ls = ml[2 * s + 1];
            const float wgt = ls == 0.f ? 0.f : expf(ml[2 * s] - m);
            s_w[warp][s] = wgt;
            l += wgt * ls;
        }
        l = warp_sum(l);
        if (lane == 0) s_l[warp] = l;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int e = h * 128 + lane * 4, hh = e / head_dim, dim0 = e % head_dim;
        const float *po = part_o + ((size_t)row * n_head + head0 + hh) * n_splits * head_dim + dim0;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int s = warp; s < n_splits; s += 8) {
            const float wgt = s_w[hh][s];
            const float4 p = *reinterpret_cast<const float4 *>(po + (size_t)s * head_dim);
            acc.x = fmaf(wgt, p.x, acc.x), acc.y = fmaf(wgt, p.y, acc.y), acc.z = fmaf(wgt, p.z, acc.z), acc.w = fmaf(wgt, p.w, acc.w);
        }
        *reinterpret_cast<float4 *>(&s_acc[warp][e]) = acc;
    }
    __syncthreads();
    if (warp == 0) {
        float4 v[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int e = h * 128 + lane * 4;
            float4 t = *reinterpret_cast<const float4 *>(&s_acc[0][e]);
#pragma unroll
            for (int w = 1; w < 8; w++) {
                const float4 u = *reinterpret_cast<const float4 *>(&s_acc[w][e]);
                t.x += u.x, t.y += u.y, t.z += u.z, t.w += u.w;
            }
            const float l = s_l[e / head_dim];
            v[h] = make_float4(t.x / l, t.y / l, t.z / l, t.w / l);
        }
        if (Q8) {
            quantize_block256(v, lane, (size_t)row, k, chunk, qs, d, sums, sums16);
        } else {
#pragma unroll
            for (int h = 0; h < 2; h++) *reinterpret_cast<float4 *>(dst + (size_t)row * k + chunk * 256 + h * 128 + lane * 4) = v[h];
        }
    }
}

inline unsigned grid_for(size_t n, int block, const DeviceInfo &dev) {
    const size_t want = (n + (size_t)block - 1) / (size_t)block;
    const size_t cap = (size_t)dev.sm_count * 8;
    return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

cudaError_t launch_rms_norm(const float *a, const float *b, float *sum_dst, const float *w, float *dst, int rows, int dim, float eps,
                            cudaStream_t st) {
    if (rows <= 0 || dim <= 0) return cudaErrorInvalidValue;
    if (dim % 256 == 0) {  // the block-per-warp kernel, storing f32
        int t = dim / 256 * 32;
        t = t > 1024 ? 1024 : t;
        int8_t *nq = nullptr;
        float *nd = nullptr;
        int32_t *ns = nullptr;
        if (b) return launch_pdl(rms_norm_q8_kernel<true, false>, dim3(rows), dim3(t), 0, st, a, b, sum_dst, w, dim, eps, dst, nq, nd, ns, ns);
        return launch_pdl(rms_norm_q8_kernel<false, false>, dim3(rows), dim3(t), 0, st, a, (const float *)nullptr, nd, w, dim, eps, dst, nq, nd, ns, ns);
    }
    int threads = ((dim / 4 + 31) / 32) * 32;
    threads = threads < 32 ? 32 : (threads > 1024 ? 1024 : threads);
    if (b) return launch_pdl(rms_norm_kernel<true>, dim3(rows), dim3(threads), 0, st, a, b, sum_dst, w, dst, dim, eps);
    return launch_pdl(rms_norm_kernel<false>, dim3(rows), dim3(threads), 0, st, a, (const float *)nullptr, (float *)nullptr, w, dst, dim, eps);
}

cudaError_t launch_rope(const float *x, const int32_t *positions, float *dst, int rows, int n_head, int head_dim, int rope_dim, float theta,
                        int neox, const DeviceInfo &dev, cudaStream_t st) {
    if (rows <= 0 || n_head <= 0 || head_dim <= 0 || rope_dim <= 0 || rope_dim > head_dim || (rope_dim & 1)) return cudaErrorInvalidValue;
    const size_t total = (size_t)rows * n_head * (rope_dim / 2 + head_dim - rope_dim);
    return launch_pdl(rope_kernel, dim3(grid_for(total, 256, dev)), dim3(256), 0, st, x, positions, dst, rows, n_head, head_dim, rope_dim, theta,
                      neox);
}

cudaError_t launch_rope_write_kv(float *q, const float *k, const float *v, const int32_t *positions, void *k_cache, void *v_cache, int rows,
                                 int n_head, int n_kv, int head_dim, float theta, int neox, int rows_per_seq, size_t seq_stride,
                                 const DeviceInfo &dev, cudaStream_t st, int write_pos, const int32_t *block_table, int table_stride, int n_pages) {
    if (rows <= 0 || n_head <= 0 || n_kv <= 0 || head_dim <= 0 || (head_dim & 1) || rows_per_seq <= 0) return cudaErrorInvalidValue;
    const size_t total = (size_t)rows * (n_head + 2 * n_kv) * (head_dim / 2);
    return launch_pdl(rope_write_kv_kernel, dim3(grid_for(total, 256, dev)), dim3(256), 0, st, q, k, v, positions, (__half *)k_cache,
                      (__half *)v_cache, rows, n_head, n_kv, head_dim, theta, neox, rows_per_seq, seq_stride, write_pos, block_table, table_stride,
                      n_pages);
}

cudaError_t launch_write_kv_f16(const float *src, void *cache_at_pos, size_t n, const DeviceInfo &dev, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    return launch_pdl(write_kv_kernel, dim3(grid_for(n, 256, dev)), dim3(256), 0, st, src, (__half *)cache_at_pos, n);
}

size_t attention_workspace_bytes(int q_rows, int n_head, int head_dim, int max_keys) {
    const size_t n_splits = ((size_t)max_keys + kAttnTile - 1) / kAttnTile;
    return (size_t)q_rows * n_head * n_splits * ((size_t)head_dim + 2) * sizeof(float);
}

template <int HD, int G>
static cudaError_t launch_attn_one(dim3 grid, cudaStream_t st, const float *q, const __half *kc, const __half *vc, float *po, float *pml, int rows,
                                   int n_head, int n_kv, int pos, float scale, int n_splits, size_t seq_stride, uint32_t *status, bool bulk,
                                   const int32_t *seq_pos, const int32_t *block_table, int table_stride, int n_pages) {
    // the tile needs more than the default 48 KB of dynamic shared memory; the attribute is per device, so it is set
    // on every launch (cheap, allocates nothing) rather than remembered per process
    auto kernel = bulk ? attn_split_kernel<HD, G, true> : attn_split_kernel<HD, G, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<HD>::kBytes);
    if (e != cudaSuccess) return e;
    return launch_pdl(kernel, grid, dim3(kAttnThreads), (size_t)AttnSmem<HD>::kBytes, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits,
                      seq_stride, status, seq_pos, block_table, table_stride, n_pages);
}

template <int HD>
static cudaError_t launch_attn_hd(int group, dim3 grid, cudaStream_t st, const float *q, const __half *kc, const __half *vc, float *po, float *pml,
                                  int rows, int n_head, int n_kv, int pos, float scale, int n_splits, size_t seq_stride, uint32_t *status, bool bulk,
                                  const int32_t *seq_pos, const int32_t *block_table, int table_stride, int n_pages) {
    switch (group) {
        case 1: return launch_attn_one<HD, 1>(grid, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits, seq_stride, status, bulk, seq_pos, block_table,
                                                  table_stride, n_pages);
        case 2: return launch_attn_one<HD, 2>(grid, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits, seq_stride, status, bulk, seq_pos, block_table,
                                                  table_stride, n_pages);
        case 4: return launch_attn_one<HD, 4>(grid, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits, seq_stride, status, bulk, seq_pos, block_table,
                                                  table_stride, n_pages);
        case 8: return launch_attn_one<HD, 8>(grid, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits, seq_stride, status, bulk, seq_pos, block_table,
                                                  table_stride, n_pages);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_attention(const float *q, const void *k_cache, const void *v_cache, float *dst, void *workspace, int n_seq, int rows, int n_head,
                             int n_kv, int head_dim, float scale, int pos, size_t seq_stride, int sm_count, cudaStream_t st, uint32_t *status, int8_t *qs, float *d,
                             int32_t *sums, int32_t *sums16, const int32_t *seq_pos, const int32_t *block_table, int table_stride, int n_pages) {
    if (n_seq <= 0 || rows <= 0 || n_head <= 0 || n_kv <= 0 || n_head % n_kv || pos < 0) return cudaErrorInvalidValue;
    const int max_keys = pos + rows, n_splits = (max_keys + kAttnTile - 1) / kAttnTile, q_rows = n_seq * rows;
    if (n_kv > 65535 || q_rows > 65535) return cudaErrorInvalidValue;
    // the tiles are fetched with 16-byte-granular bulk copies of whole rows
    if (((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 || seq_stride % 8 || ((size_t)n_kv * head_dim) % 8) return cudaErrorInvalidValue;
    if (block_table && (n_pages < 1 || table_stride < n_splits)) return cudaErrorInvalidValue;
    float *po = static_cast<float *>(workspace);
    float *pml = po + (size_t)q_rows * n_head * n_splits * head_dim;
    const dim3 grid(n_splits, n_kv, q_rows);
    const __half *kc = static_cast<const __half *>(k_cache), *vc = static_cast<const __half *>(v_cache);
    cudaError_t e;
    // more than two waves of CTAs (three fit an SM): the per-tile instruction count decides, else the first byte's latency
    const bool bulk = (size_t)n_splits * n_kv * q_rows > (size_t)6 * (sm_count > 0 ? sm_count : 148);
    const int g = n_head / n_kv;
    if (head_dim == 128)
        e = launch_attn_hd<128>(g, grid, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits, seq_stride, status, bulk, seq_pos, block_table, table_stride,
                                n_pages);
    else if (head_dim == 64)
        e = launch_attn_hd<64>(g, grid, st, q, kc, vc, po, pml, rows, n_head, n_kv, pos, scale, n_splits, seq_stride, status, bulk, seq_pos, block_table, table_stride,
                               n_pages);
    else
        return cudaErrorInvalidValue;
    if (e != cudaSuccess) return e;
    if (qs) {  // the merged rows go straight to int8 (n_head * head_dim must be whole 256-element blocks)
        if ((n_head * head_dim) % 256 || n_splits > kCombineMaxSplits) return cudaErrorInvalidValue;
        return launch_pdl(attn_combine_wide_kernel<true>, dim3((unsigned)(q_rows * (n_head * head_dim / 256))), dim3(256), 0, st, (const float *)po,
                          (const float *)pml, n_head, head_dim, n_splits, (float *)nullptr, qs, d, sums, sums16);
    }
    if ((n_head * head_dim) % 256 == 0 && n_splits <= kCombineMaxSplits)
        return launch_pdl(attn_combine_wide_kernel<false>, dim3((unsigned)(q_rows * (n_head * head_dim / 256))), dim3(256), 0, st, (const float *)po,
                          (const float *)pml, n_head, head_dim, n_splits, dst, (int8_t *)nullptr, (float *)nullptr, (int32_t *)nullptr,
                          (int32_t *)nullptr);
    return launch_pdl(attn_combine_kernel, dim3(q_rows * n_head), dim3(head_dim), 0, st, (const float *)po, (const float *)pml, dst, head_dim, n_splits);
}

cudaError_t launch_rms_norm_q8_pull(const float *a, float *sum_dst, const float *w, int rows, int dim, float eps, int8_t *qs, float *d,
                                    int32_t *sums, int32_t *sums16, const PullArgs &pull, cudaStream_t st) {
    if (rows <= 0 || dim <= 0 || dim % 256 || pull.world < 1 || pull.world > kPushMaxWorld) return cudaErrorInvalidValue;
    int threads = dim / 256 * 32;
    threads = threads > 1024 ? 1024 : threads;
    return launch_pdl(rms_norm_q8_pull_kernel, dim3(rows), dim3(threads), 0, st, a, sum_dst, w, dim, eps, qs, d, sums, sums16, pull);
}

cudaError_t launch_rms_norm_q8(const float *a, const float *b, float *sum_dst, const float *w, int rows, int dim, float eps, int8_t *qs, float *d,
                               int32_t *sums, int32_t *sums16, cudaStream_t st) {
    if (rows <= 0 || dim <= 0 || dim % 256) return cudaErrorInvalidValue;
    int threads = dim / 256 * 32;
    threads = threads > 1024 ? 1024 : threads;
    float *none = nullptr;
    if (b) return launch_pdl(rms_norm_q8_kernel<true, true>, dim3(rows), dim3(threads), 0, st, a, b, sum_dst, w, dim, eps, none, qs, d, sums, sums16);
    return launch_pdl(rms_norm_q8_kernel<false, true>, dim3(rows), dim3(threads), 0, st, a, (const float *)nullptr, none, w, dim, eps, none, qs, d, sums,
                      sums16);
}

cudaError_t launch_gated_silu_q8(const float *gate, const float *up, int rows, int nff, int8_t *qs, float *d, int32_t *sums, int32_t *sums16,
                                 cudaStream_t st) {
    if (rows <= 0 || nff <= 0 || nff % 256) return cudaErrorInvalidValue;
    const long long warps = (long long)rows * (nff / 256);
    return launch_pdl(gated_silu_q8_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, st, gate, up, rows, nff, qs, d, sums, sums16);
}

cudaError_t launch_gated_silu(const float *gate, const float *up, float *dst, size_t n, const DeviceInfo &dev, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    return launch_pdl(gated_silu_kernel, dim3(grid_for(n, 256, dev)), dim3(256), 0, st, gate, up, dst, n);
}

cudaError_t launch_add(const float *a, const float *b, float *dst, size_t n, const DeviceInfo &dev, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    return launch_pdl(add_kernel, dim3(grid_for(n, 256, dev)), dim3(256), 0, st, a, b, dst, n);
}

size_t argmax_workspace_bytes(uint32_t n, uint32_t rows) {
    const uint32_t chunk = 4096, n_chunks = (n + chunk - 1) / chunk;
    return (size_t)rows * n_chunks * 8;
}

cudaError_t launch_argmax(const float *x, uint32_t *dst, void *workspace, uint32_t n, uint32_t rows, cudaStream_t st) {
    if (n == 0 || rows == 0 || rows > 65535) return cudaErrorInvalidValue;
    const uint32_t chunk = 4096, n_chunks = (n + chunk - 1) / chunk;
    float *cv = static_cast<float *>(workspace);
    uint32_t *ci = reinterpret_cast<uint32_t *>(cv + (size_t)rows * n_chunks);
    cudaError_t e = launch_pdl(argmax_stage1_kernel, dim3(n_chunks, rows), dim3(256), 0, st, x, cv, ci, n, chunk);
    if (e != cudaSuccess) return e;
    return launch_pdl(argmax_stage2_kernel, dim3(rows), dim3(256), 0, st, (const float *)cv, (const uint32_t *)ci, dst, n_chunks);
}

}  // namespace infr
