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
//   warps 0-7    unpack: thread = (weight row, K half of the block); turns its 4 sub-blocks into int8 operand words
//                and stores them into TENSOR MEMORY (tcgen05.st), a ring of three half-block slots; the A operand
//                of the MMAs is read from there, so shared memory carries only the token side
//                (warps 0-3 also write the tf32 min planes and the row scale d)
//   warps 8-15   epilogue: warp = (tensor-memory lane quarter, 32-column half); folds each job's int32 sums
//                into 32 running f32 sums per thread
//   warp 16      TMA producer: raw Q4_K rows + activation planes (codes, tf32 block-sum pieces), five stages
//   warps 17-19  MMA issuers, one per accumulator chain (D_lo: 8 kind::i8 per job, D_hi: 8, min sums: 3
//                kind::tf32): a tcgen05.mma holds its issuing thread ~90 cycles but threads issue concurrently
// Tensor memory (512 columns): accumulators {D_lo, D_hi} x 2 jobs = 256, min sums 64, operand ring 3 x 64.
//
// Measured on B200 and limiting this kernel: a tcgen05.mma with 32 bytes of K (kind::i8 K = 32, kind::tf32
// K = 8) occupies the issuing thread and the tensor pipe ~95 cycles for every N <= 128 (N = 256: 138), from
// shared-memory or tensor-memory operands alike — per issuing THREAD: two threads issue at twice the rate, which
// is why the job's 19 instructions are split over three issuer warps; accumulators leave tensor memory at ~128 B/clk per SM; one mbarrier
// operation costs its thread ~100 cycles.
// Every wait is bounded: on expiry the role raises a CTA flag and a status word, every role leaves its
// loop, in-flight copies are drained and the tensor memory is freed.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

#include "gemv_common.cuh"
#include "pdl.cuh"
#include "q8_code.cuh"

namespace infr {
namespace {

constexpr int kTM = 128, kTN = 64;
constexpr int kStages = 5;
constexpr int kPlanes = 20;                   // activation planes per super-block: 16 code planes + B1[2] + B2[2]
constexpr int kRawBytes = kTM * 144, kActBytes = kPlanes * kTN * 16;
constexpr int kStageBytes = kRawBytes + kActBytes;
constexpr int kMinBytes = 4 * kTM * 16;       // A1 planes [2], A2 planes [2]
constexpr int kRing = 4;                      // depth of the row-scale ring read by the epilogue
constexpr int kSmem = kStages * kStageBytes + 2 * kMinBytes + kRing * kTM * 4;
constexpr int kThreadsWs = 20 * 32;
constexpr uint32_t kSpin = 1u << 22;
// tensor-memory columns
constexpr uint32_t kColMin = 256, kColA = 320, kSlotCols = 64, kSlots = 3;

// barrier indices: FULL[stage] (TMA bytes), DONE[stage] (the job's last commit), AREADY/AFREE[operand slot],
// ACCFREE[accumulator] (8 epilogue warps), MINFREE (8 epilogue warps), MINREADY[min-plane buffer] (4 unpack warps), DRAIN
constexpr int B_FULL = 0, B_DONE = B_FULL + kStages, B_AREADY = B_DONE + kStages, B_AFREE = B_AREADY + kSlots,
              B_ACCFREE = B_AFREE + kSlots, B_MINFREE = B_ACCFREE + 2, B_MINREADY = B_MINFREE + 1, B_DRAIN = B_MINREADY + 2, B_COUNT = B_DRAIN + 3;

__device__ __forceinline__ uint32_t su32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t mk_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void mma_i8_ta(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d),
        "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc), "r"(0)
        : "memory");
}
__device__ __forceinline__ void tst8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tst_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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

// Warp-collective wait on up to 32 barriers at once: every lane names its own barrier (or need = false) and
// all lanes poll in the same instruction, so k waits cost the latency of one.
__device__ __forceinline__ bool wait_multi(uint32_t bar, uint32_t parity, bool need, volatile int *dead) {
    bool pending = need;
    for (uint32_t i = 0; i < kSpin; i++) {
        if (pending) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok)
                         : "r"(bar), "r"(parity)
                         : "memory");
            pending = !ok;
        }
        if (!__any_sync(0xffffffffu, pending)) return true;
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


// Grouped (mixture-of-experts) form: the token dimension is a list of 64-token slabs, each slab holding up to 64
// activation rows routed to ONE expert (moe_bucket_kernel with 64-row items); the weight rows of a slab's tiles are
// those of its expert inside the bank (experts back to back, out_f rows each) and its results go to the rows of
// its routed pairs.  slab_expert == nullptr: the plain GEMM.
struct MmqGroup {
    const int *slab_expert;  // [n_slabs] expert (index inside the bank) of the slab
    const int *slab_p0;      // [n_slabs] first routed pair of the slab; output row = pair
    const int *slab_cnt;     // [n_slabs] pairs in the slab (1..64)
    const int *n_slabs;      // device scalar
    const int *pair_row;     // [n_pairs] activation row of each pair, or nullptr: pair p reads row p
};

// Re-lays the quantised activations for the kernel.  Output: for every super-block b, 20 planes of
// [m tokens][16 bytes]: planes 0..15 = the int8 codes of K chunk k/16, planes 16..19 = B1[0..3], B1[4..7],
// B2[0..3], B2[4..7] (tf32 pieces of d8 * bsum_s); a 64-token tile of one block is then 20 runs of 1 KB,
// which the copy engine moves at full rate (16-byte runs do not).  Behind the planes: d8 transposed to
// [nb][m_pad] f32 for the epilogue's broadcast loads.
__global__ void mmq_ws_prep_kernel(const int8_t *__restrict__ qs, const int32_t *__restrict__ sums, const float *__restrict__ d,
                                   int m, int m_pad, int nb, uint4 *__restrict__ out, MmqGroup grp) {
    pdl_go();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // token fastest: a warp writes 512 contiguous bytes per plane
    if (i >= m * nb) return;
    const int tok = i % m, b = i / m;
    size_t rec = (size_t)tok * nb + b;
    uint4 *o = out + (size_t)b * kPlanes * m + tok;
    if (grp.slab_expert) {
        // `tok` is a slot of a slab: its activation row is the slab's pair, empty slots read as zero
        const int slab = tok / kTN, slot = tok - slab * kTN;
        if (slab >= *grp.n_slabs) return;
        if (slot >= grp.slab_cnt[slab]) {
            const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int k = 0; k < kPlanes; k++) o[(size_t)k * m] = z;
            reinterpret_cast<float *>(out + (size_t)nb * kPlanes * m)[(size_t)b * m_pad + tok] = 0.f;
            return;
        }
        const int pair = grp.slab_p0[slab] + slot;
        rec = (size_t)(grp.pair_row ? grp.pair_row[pair] : pair) * nb + b;
    }
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


// f32 activations straight to the kernel's planes: quantize_q8 (crates/infr-cpu/src/quant.rs:27-58, the operations of
// quantize.cu in the same order, so the same codes, scales and sums) and the re-layout above in one pass.  One warp per
// (token, super-block); lane l owns elements [4l, 4l+4) and [128+4l, 128+4l+4).
__global__ void __launch_bounds__(256) mmq_ws_quant_planes_kernel(const float *__restrict__ x, int m, int m_pad, int nb,
                                                                  uint32_t *__restrict__ out) {
    pdl_go();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)m * nb) return;
    const int tok = (int)(wg / nb), b = (int)(wg % nb);
    const float *xp = x + ((size_t)tok * nb + b) * 256;
    const float4 v0 = *reinterpret_cast<const float4 *>(xp + lane * 4), v1 = *reinterpret_cast<const float4 *>(xp + 128 + lane * 4);
    float am = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                     fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float dd = am / 127.0f;
    const float id = dd > 0.0f ? 1.0f / dd : 0.0f;
    auto q1 = [&](float v) { return q8_round_code(v, id); };
    uint32_t *pl = out + ((size_t)b * kPlanes * m + tok) * 4;  // word 0 of this token's entry in plane 0 of block b
    const size_t plane_words = (size_t)m * 4;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float4 v = h ? v1 : v0;
        const int q0 = q1(v.x), qq1 = q1(v.y), q2 = q1(v.z), q3 = q1(v.w);
        int sum = q0 + qq1 + q2 + q3;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        // elements [128h + 4l, +4) = 16-byte chunk 8h + l/4 of the block, word l%4 of the chunk
        pl[(size_t)(8 * h + (lane >> 2)) * plane_words + (lane & 3)] =
            (uint32_t)(q0 & 0xff) | ((uint32_t)(qq1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        if ((lane & 7) == 0) {
            // sub-block 4h + l/8: d8 * bsum as two tf32-representable pieces
            const float t = __fmul_rn(dd, (float)sum);
            const uint32_t hi = __float_as_uint(t) & 0xFFFFE000u;
            const float r = __fsub_rn(t, __uint_as_float(hi));
            pl[(size_t)(16 + h) * plane_words + (lane >> 3)] = hi;
            pl[(size_t)(18 + h) * plane_words + (lane >> 3)] = __float_as_uint(r) & 0xFFFFE000u;
        }
    }
    if (lane == 0) reinterpret_cast<float *>(out + (size_t)nb * kPlanes * m * 4)[(size_t)b * m_pad + tok] = dd;
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

__global__ void __launch_bounds__(kThreadsWs, 1)
    mmq_ws_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                  const float *__restrict__ d8t, float *__restrict__ C, int m, int m_pad, int in_f, int out_f,
                  uint32_t *__restrict__ status, MmqGroup grp, int kz) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *stage0 = smem;                                              // [kStages]{raw rows, activation planes}
    uint8_t *minbuf0 = smem + kStages * kStageBytes;                     // [2][kMinBytes]
    float *dwring = reinterpret_cast<float *>(minbuf0 + 2 * kMinBytes);  // [kRing][kTM]
    __shared__ uint64_t bars[B_COUNT];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_dead;
    volatile int *dead = &s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = in_f >> 8;
    pdl_go();
    // barriers and tensor memory do not depend on the previous kernel: they are set up while it finishes
    if (tid == 0) {
        s_dead = 0;
        for (int i = 0; i < B_COUNT; i++) {
            const int cnt = (i >= B_AREADY && i < B_AREADY + kSlots)  ? 4    // the four unpack warps of a K half
                            : (i >= B_MINREADY && i < B_MINREADY + 2) ? 4    // the four unpack warps that write the min planes
                            : (i >= B_ACCFREE && i <= B_MINFREE)      ? 8    // the epilogue warps
                            : (i >= B_AFREE && i < B_AFREE + kSlots)  ? 2    // the D_lo and D_hi issuers
                            : (i >= B_DONE && i < B_DONE + kStages)   ? 3    // all three issuers
                                                                      : 1;
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
    pdl_wait();  // every thread, before the first read of what the previous kernels wrote (planes, scales, slab lists)
    // grouped: one token tile per slab (their number is known only on the device)
    const int row_tiles = (out_f + kTM - 1) / kTM, tok_tiles = grp.slab_expert ? *grp.n_slabs : (m + kTN - 1) / kTN;
    // kz > 1: K is split kz ways across tiles (a batch of a few dozen rows against a matrix with few row tiles would
    // otherwise keep most SMs idle while a handful walk all of K); split s writes its partial result to C + s * m * out_f
    // and a second kernel adds the partial results in order.
    const int n_tiles = row_tiles * tok_tiles * kz;
    auto tile_of = [&](int t, int *rt, int *tt, int *b0, int *b1) {
        const int ks = t % kz, tr = t / kz;
        *rt = tr % row_tiles;  // consecutive CTAs share a token tile
        *tt = tr / row_tiles;
        *b0 = ks * nb / kz;
        *b1 = (ks + 1) * nb / kz;
        return ks;
    };

    const uint32_t tmem = tmem_base_s;
    auto bar = [&](int i) { return su32(&bars[i]); };

    if (warp == 16) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int j = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                int rt, tt, b0, b1;
                tile_of(t, &rt, &tt, &b0, &b1);
                const int wrow0 = (grp.slab_expert ? grp.slab_expert[tt] * out_f : 0) + rt * kTM;
                for (int b = b0; b < b1; b++, j++) {
                    const int s = j % kStages;
                    // the stage's previous job is complete (its operands were read by the MMAs, its rows unpacked)
                    if (j >= kStages && !wait_bar(bar(B_DONE + s), (uint32_t)((j / kStages - 1) & 1), dead)) {
                        ok = false;
                        break;
                    }
                    uint8_t *st = stage0 + (size_t)s * kStageBytes;
                    const uint32_t fb = bar(B_FULL + s);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(kStageBytes) : "memory");
                    tma2(su32(st), &map_w, b * 36, wrow0, fb);
                    tma2(su32(st + kRawBytes), &map_q, tt * kTN * 4, b * kPlanes, fb);
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
        // A tcgen05.mma keeps its issuing thread ~90 cycles whatever its size, but threads issue concurrently
        // (two threads: twice the rate), so the job's instructions are split over three warps by accumulator
        // chain: D_lo, D_hi, and the tf32 min sums.  Each issuer commits for itself; the barriers the chains
        // share count one arrival per issuer.  A role's waits are spread over lanes and complete together.
        const int role = warp - 17;  // 0: D_lo, 1: D_hi, 2: min sums
        const uint32_t idesc_i8 = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
        const uint32_t idesc_tf = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
        const uint32_t tmin = tmem + kColMin;
        int j = 0, tile_i = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, tile_i++) {
            int rt_, tt_, b0, b1;
            tile_of(t, &rt_, &tt_, &b0, &b1);
            for (int b = b0; b < b1 && ok; b++, j++) {
                const int s = j & 1, ls = j % kStages;
                const int slot0 = (2 * j) % (int)kSlots, n0 = (2 * j) / (int)kSlots;
                const int slot1 = (2 * j + 1) % (int)kSlots, n1 = (2 * j + 1) / (int)kSlots;
                uint32_t wb = 0, wp = 0;
                bool need = false;
                if (lane == 0) wb = bar(B_FULL + ls), wp = (uint32_t)((j / kStages) & 1), need = true;
                if (lane == 1) wb = bar(B_ACCFREE + s), wp = (uint32_t)(((j >> 1) - 1) & 1), need = role < 2 && j >= 2;
                if (lane == 2) wb = bar(B_AREADY + slot0), wp = (uint32_t)(n0 & 1), need = role < 2;
                if (lane == 3) wb = bar(B_AREADY + slot1), wp = (uint32_t)(n1 & 1), need = role < 2;
                // The min issuer has a barrier of its own for its operands.  It must not wait on AREADY: that barrier
                // advances with the D_lo / D_hi issuers alone, and an issuer held up at a tile boundary would find it two
                // phases ahead, which a parity wait cannot tell from "not yet".  MINREADY[s] can only be one phase
                // ahead: its next arrival needs the commit of this job.
                if (lane == 5) wb = bar(B_MINREADY + s), wp = (uint32_t)((j >> 1) & 1), need = role == 2;
                // the tile's first min MMA overwrites the sums of the previous tile: the epilogue has read them
                if (lane == 4) wb = bar(B_MINFREE), wp = (uint32_t)((tile_i - 1) & 1), need = role == 2 && b == b0 && tile_i >= 1;
                if (!wait_multi(wb, wp, need, dead)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t db0 = mk_desc(su32(stage0 + (size_t)ls * kStageBytes + kRawBytes), kTN * 16, 128);
                    if (role == 2) {
                        const uint8_t *mb = minbuf0 + (size_t)s * kMinBytes;
                        const uint64_t a1 = mk_desc(su32(mb), kTM * 16, 128), a2 = mk_desc(su32(mb + 2 * kTM * 16), kTM * 16, 128);
                        const uint64_t bd1 = db0 + (uint64_t)(16 * kTN), bd2 = db0 + (uint64_t)(18 * kTN);
                        mma_tf32(tmin, a1, bd1, idesc_tf, b > b0 ? 1u : 0u);
                        mma_tf32(tmin, a2, bd1, idesc_tf, 1u);
                        mma_tf32(tmin, a1, bd2, idesc_tf, 1u);
                    } else {
                        const uint32_t td = tmem + (uint32_t)s * 2 * kTN + (uint32_t)role * kTN;
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const uint32_t ta = tmem + kColA + (uint32_t)(h ? slot1 : slot0) * kSlotCols + (uint32_t)role * 32;
#pragma unroll
                            for (int sbl = 0; sbl < 4; sbl++) {
                                const int sb = 4 * h + sbl;
                                // sub-block sb = activation planes 2sb, 2sb+1: the descriptor start address counts 16-byte units
                                mma_i8_ta(td, ta + (uint32_t)(sbl * 8), db0 + (uint64_t)(sb * 2 * kTN), idesc_i8, sb > 0 ? 1u : 0u);
                            }
                            mma_commit(bar(B_AFREE + (h ? slot1 : slot0)));
                        }
                    }
                    mma_commit(bar(B_DONE + ls));
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            if (!*dead) atomicExch(status, 6u);
            *dead = 1;
        }
        if (lane == 0) {
            // every issued MMA has completed before the tensor memory is freed
            mma_commit(bar(B_DRAIN + role));
            wait_plain(bar(B_DRAIN + role), 0u, 1u << 20);
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ unpack warps
        const int quarter = warp & 3, h = warp >> 2, row = quarter * 32 + lane;
        const uint32_t tl = tmem + ((uint32_t)(quarter * 32) << 16) + kColA;
        int j = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            int rt_, tt_, b0, b1;
            tile_of(t, &rt_, &tt_, &b0, &b1);
            for (int b = b0; b < b1; b++, j++) {
                const int ls = j % kStages;
                const int r = 2 * j + h, slot = r % (int)kSlots, n = r / (int)kSlots;
                // two waits on two lanes: the rows have landed, the operand slot's previous MMAs are complete
                uint32_t wb = 0, wp = 0;
                bool need = false;
                if (lane == 0) wb = bar(B_FULL + ls), wp = (uint32_t)((j / kStages) & 1), need = true;
                if (lane == 1) wb = bar(B_AFREE + slot), wp = (uint32_t)((n - 1) & 1), need = n >= 1;
                // the min planes of job j - 2 (same buffer) have been read by the min issuer's MMAs
                if (lane == 2) wb = bar(B_DONE + (j - 2 + kStages) % kStages), wp = (uint32_t)((((j - 2) / kStages)) & 1), need = h == 0 && j >= 2;
                if (!wait_multi(wb, wp, need, dead)) {
                    ok = false;
                    break;
                }
                const uint8_t *blk = stage0 + (size_t)ls * kStageBytes + (size_t)row * 144;
                const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
                const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 64 * h), q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 64 * h);
                const uint4 q2 = *reinterpret_cast<const uint4 *>(blk + 48 + 64 * h), q3 = *reinterpret_cast<const uint4 *>(blk + 64 + 64 * h);
                const uint32_t w[16] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w, q3.x, q3.y, q3.z, q3.w};
                uint32_t sc[2], mn[2];
                sc[0] = hdr.y & 0x3F3F3F3Fu;
                mn[0] = hdr.z & 0x3F3F3F3Fu;
                sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                const uint32_t sc4 = sc[h];  // scales of sub-blocks 4h..4h+3
                tc_fence_after();
                const uint32_t ts = tl + (uint32_t)slot * kSlotCols;
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
                        // column c of a lane = K elements 4c..4c+3 of the row: 8 columns per sub-block
                        tst8(ts + (uint32_t)(sbl * 8), lo);
                        tst8(ts + 32 + (uint32_t)(sbl * 8), hi);
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
                    uint8_t *mp = minbuf0 + (size_t)(j & 1) * kMinBytes + (size_t)row * 16;
                    *reinterpret_cast<uint4 *>(mp) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
                    *reinterpret_cast<uint4 *>(mp + kTM * 16) = make_uint4(p1[4], p1[5], p1[6], p1[7]);
                    *reinterpret_cast<uint4 *>(mp + 2 * kTM * 16) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
                    *reinterpret_cast<uint4 *>(mp + 3 * kTM * 16) = make_uint4(p2[4], p2[5], p2[6], p2[7]);
                    dwring[(j % kRing) * kTM + row] = dw;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) bar_arrive(bar(B_MINREADY + (j & 1)));
                }
                tst_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) bar_arrive(bar(B_AREADY + slot));
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
            int rt, tt, b0, b1;
            const int ks = tile_of(t, &rt, &tt, &b0, &b1);
            float *Ct = C + (size_t)ks * m * out_f;  // this K split's partial result
            const float4 *d8p = reinterpret_cast<const float4 *>(d8t + (size_t)tt * kTN + half * 32);
#pragma unroll
            for (int i = 0; i < 32; i++) acc[i] = 0.f;
            for (int b = b0; b < b1; b++, j++) {
                const int s = j & 1;
                float4 dd[4];
#pragma unroll
                for (int i4 = 0; i4 < 4; i4++) dd[i4] = __ldg(d8p + (size_t)b * (m_pad / 4) + i4);
                if (!wait_bar_warp(bar(B_DONE + j % kStages), (uint32_t)((j / kStages) & 1), dead)) {
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
                    if (c == 1) {
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
            // tile end: subtract the min sums and store
            const int grow = rt * kTM + row;
            const int tok_lim = grp.slab_expert ? grp.slab_cnt[tt] : m - tt * kTN;      // valid token slots of the tile
            const size_t out_row0 = grp.slab_expert ? (size_t)grp.slab_p0[tt] : (size_t)tt * kTN;  // output row of slot 0
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t mv[16];
                tld16(tlane + kColMin + (uint32_t)(c * 16), mv);
                tld_wait();
                if (c == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) bar_arrive(bar(B_MINFREE));
                }
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int slot = half * 32 + c * 16 + i;
                    if (grow < out_f && slot < tok_lim) Ct[(out_row0 + slot) * out_f + grow] = acc[c * 16 + i] - __uint_as_float(mv[i]);
                }
            }
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

// How many ways K is split for C[m, out_f]: 1 when the row x token tiles alone fill the SMs, else enough splits to
// occupy them (at most one split per super-block, at most 16).
int mmq_ws_k_splits(int m, int in_f, int out_f, const DeviceInfo &dev) {
    const int tiles = ((out_f + kTM - 1) / kTM) * ((m + kTN - 1) / kTN), nb = in_f / 256;
    if (tiles * 2 > dev.sm_count) return 1;
    int kz = dev.sm_count / tiles;
    if (kz > nb) kz = nb;
    if (kz > 16) kz = 16;
    return kz < 1 ? 1 : kz;
}
size_t mmq_ws_partial_bytes(int m, int in_f, int out_f, const DeviceInfo &dev) {
    const int kz = mmq_ws_k_splits(m, in_f, out_f, dev);
    return kz > 1 ? (size_t)kz * m * out_f * 4 : 0;
}

// y[i] = part[0][i] + part[1][i] + ... in split order (the same bits on every run).
__global__ void mmq_ws_sum_splits_kernel(const float4 *__restrict__ part, float4 *__restrict__ y, size_t n4, int kz) {
    pdl_go();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 acc = part[i];
    for (int s = 1; s < kz; s++) {
        const float4 v = part[(size_t)s * n4 + i];
        acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    y[i] = acc;
}

namespace {
// Common launch: `m` token slots (a multiple of 64 in grouped mode: all slabs that can exist), weight tensor map over
// `w_rows` rows.  prep = false reuses the planes a previous call with the same activations and slabs has written.
cudaError_t launch_ws(const uint8_t *w, size_t w_rows, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                      const MmqGroup &grp, int max_tok_tiles, bool prep, const DeviceInfo &dev, uint32_t *status, cudaStream_t st,
                      int kz = 1, float *partials = nullptr, const float *x_f32 = nullptr) {
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const int nb = in_f / 256, m_pad = (m + kTN - 1) / kTN * kTN;
    const int n_rec = m * nb;
    cudaError_t pe = cudaSuccess;
    if (prep && x_f32)
        pe = launch_pdl(mmq_ws_quant_planes_kernel, dim3((unsigned)(((size_t)n_rec * 32 + 255) / 256)), dim3(256), 0, st, x_f32, m, m_pad, nb,
                        static_cast<uint32_t *>(records));
    else if (prep)
        pe = launch_pdl(mmq_ws_prep_kernel, dim3((unsigned)((n_rec + 255) / 256)), dim3(256), 0, st, a.qs, a.sums, a.d, m, m_pad, nb,
                        static_cast<uint4 *>(records), grp);
    if (pe != cudaSuccess) return pe;
    CUtensorMap map_w, map_q;
    const cuuint32_t one2[2] = {1, 1};
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)nb * 36, (cuuint64_t)w_rows};
        const cuuint64_t gstr[1] = {(cuuint64_t)nb * 144};
        const cuuint32_t box[2] = {36, (cuuint32_t)kTM};
        if (enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(w), gdim, gstr, box, one2, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
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
    const int n_tiles = ((out_f + kTM - 1) / kTM) * max_tok_tiles * kz;
    const int grid = n_tiles < dev.sm_count ? n_tiles : dev.sm_count;
    e = launch_pdl(mmq_ws_kernel, dim3((unsigned)grid), dim3(kThreadsWs), (size_t)kSmem, st, map_w, map_q, d8t, kz > 1 ? partials : c, m, m_pad, in_f,
                   out_f, status, grp, kz);
    if (e != cudaSuccess) return e;
    if (kz > 1) {
        const size_t n = (size_t)m * out_f;
        if (n % 4) return cudaErrorInvalidValue;  // (callers split K only when out_f is a multiple of 4)
        return launch_pdl(mmq_ws_sum_splits_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, reinterpret_cast<const float4 *>(partials),
                          reinterpret_cast<float4 *>(c), n / 4, kz);
    }
    return cudaSuccess;
}
}  // namespace

// `partials`: mmq_ws_partial_bytes(m, in_f, out_f) bytes of scratch (may be null when that is 0).
cudaError_t launch_mmq_ws_q4k(const uint8_t *w, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                              const DeviceInfo &dev, uint32_t *status, cudaStream_t st, float *partials) {
    if (m < 1 || in_f % 256 || out_f < 1) return cudaErrorInvalidValue;
    int kz = (out_f % 4 == 0 && partials && ((uintptr_t)c % 16) == 0) ? mmq_ws_k_splits(m, in_f, out_f, dev) : 1;
    return launch_ws(w, (size_t)out_f, a, records, c, m, in_f, out_f, MmqGroup{}, (m + kTN - 1) / kTN, true, dev, status, st, kz, partials);
}

// From f32 activations: x != nullptr quantises them straight into the planes in `records` (one kernel instead of the
// quantiser plus the re-layout); x == nullptr reuses the planes a previous call wrote for the same activations.
cudaError_t launch_mmq_ws_q4k_f32(const uint8_t *w, const float *x, void *records, float *c, int m, int in_f, int out_f,
                                  const DeviceInfo &dev, uint32_t *status, cudaStream_t st, float *partials) {
    if (m < 1 || in_f % 256 || out_f < 1) return cudaErrorInvalidValue;
    if (x && ((uintptr_t)x % 16)) return cudaErrorInvalidValue;
    int kz = (out_f % 4 == 0 && partials && ((uintptr_t)c % 16) == 0) ? mmq_ws_k_splits(m, in_f, out_f, dev) : 1;
    return launch_ws(w, (size_t)out_f, Q8Dev{}, records, c, m, in_f, out_f, MmqGroup{}, (m + kTN - 1) / kTN, x != nullptr, dev, status, st, kz,
                     partials, x);
}

// Expert-grouped GEMM over a bank of n_experts Q4_K matrices [out_f, in_f] stored back to back: slab i (a work item
// of moe_bucket_kernel with 64-row items) multiplies up to 64 quantised activation rows (pairs slab_p0[i]..+slab_cnt[i],
// gathered through pair_row when non-null) with expert slab_expert[i]; y is [n_pairs, out_f].  max_slabs bounds the
// number of slabs (n_pairs / 64 + n_experts); `records` holds mmq_ws_record_bytes(max_slabs * 64, in_f) bytes.
cudaError_t launch_mmq_ws_q4k_grouped(const uint8_t *bank, int n_experts, const Q8Dev &a, void *records, float *y, int in_f, int out_f,
                                      const int *slab_expert, const int *slab_p0, const int *slab_cnt, const int *n_slabs,
                                      const int *pair_row, int max_slabs, bool prep, const DeviceInfo &dev, uint32_t *status,
                                      cudaStream_t st) {
    if (in_f % 256 || out_f < 1 || max_slabs < 1 || n_experts < 1) return cudaErrorInvalidValue;
    MmqGroup grp{slab_expert, slab_p0, slab_cnt, n_slabs, pair_row};
    return launch_ws(bank, (size_t)n_experts * out_f, a, records, y, max_slabs * kTN, in_f, out_f, grp, max_slabs, prep, dev, status, st);
}

}  // namespace infr
