// Prefill MMQ: C[m, out_f] = Q8(x)[m, in_f] * Q4_K(W)^T on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), with the arithmetic of the production
// infr-cpu path (crates/infr-cpu/src/kernels.rs:151-184, batch form :1458-1509):
//     per 256-element super-block b:  sd = sum_s sc_s * sum_i q4 * q8,   sm = sum_s m_s * bsum_s
//     C += d8[tok, b] * (d[row, b] * float(sd) - dmin[row, b] * float(sm))      blocks in ascending order
// The f32 expression is evaluated per (row, token, block) with separately rounded multiply / subtract /
// add in block order, exactly as the CPU does, so the result is bit-identical to it.
//
// The 6-bit sub-block scale cannot ride inside an int8 operand (sc * q reaches 945) and rescaling the
// accumulator every 32 K would make the epilogue the bottleneck, so the scale is split in two 3-bit
// halves: A_lo = q * (sc & 7) and A_hi = q * (sc >> 3) are both <= 105, two MMAs per sub-block
// accumulate the whole super-block in tensor memory and sd = D_lo + 8 * D_hi is exact.  The min term
// is two more MMAs: A = the eight m_s bytes, B = bsum split as 64 * h + l.
//
// Operand layout in shared memory (no swizzle, K-major): 16-byte planes [k/16][row][16 B]; the
// descriptor of sub-block s starts at plane 2s with leading-dimension offset = one plane and stride
// offset = 128 B (8 rows).  One CTA owns a 128-row x 64-token tile: thread r unpacks weight row r,
// reads tensor-memory lane r in the epilogue and keeps the 64 running f32 sums of that row.
//
// Every mbarrier wait is bounded; on expiry the CTA records a status word and leaves (after freeing
// its tensor memory).
#include "gemv_common.cuh"

namespace infr {
namespace {

constexpr int kTM = 128;  // weight rows per tile (MMA M)
constexpr int kTN = 64;   // tokens per tile (MMA N)
constexpr uint32_t kMmqSpin = 1u << 22;

__device__ __forceinline__ uint32_t sm_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

__global__ void __launch_bounds__(kTM) mmq_q4k_kernel(const uint8_t *__restrict__ W, Q8Dev a, float *__restrict__ C, int m, int in_f,
                                                      int out_f, uint32_t *__restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sA_lo = smem;                        // [16][128][16]
    uint8_t *sA_hi = sA_lo + 16 * kTM * 16;       // [16][128][16]
    uint8_t *sA_m = sA_hi + 16 * kTM * 16;        // [2][128][16]
    uint8_t *sB = sA_m + 2 * kTM * 16;            // [16][64][16]
    uint8_t *sB_ml = sB + 16 * kTN * 16;          // [2][64][16]
    uint8_t *sB_mh = sB_ml + 2 * kTN * 16;        // [2][64][16]
    float *s_d8 = reinterpret_cast<float *>(sB_mh + 2 * kTN * 16);  // [64]
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int nb = in_f >> 8;
    const size_t row_bytes = (size_t)nb * 144;
    const int row0 = blockIdx.x * kTM, tok0 = blockIdx.y * kTN;
    const int row = row0 + tid;
    const bool row_ok = row < out_f;
    if (tid == 0) {
        s_dead = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm_u32(&bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_u32(&tmem_base_s)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // planes that never change: second half of the min-term operands is zero
    for (int i = tid; i < kTM; i += kTM) *reinterpret_cast<uint4 *>(sA_m + (size_t)(kTM + i) * 16) = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < kTN; i += kTM) {
        *reinterpret_cast<uint4 *>(sB_ml + (size_t)(kTN + i) * 16) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4 *>(sB_mh + (size_t)(kTN + i) * 16) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kTN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);

    float acc[kTN];
#pragma unroll
    for (int j = 0; j < kTN; j++) acc[j] = 0.f;
    uint32_t phase = 0;

    for (int b = 0; b < nb; b++) {
        // ---- unpack this thread's weight row: A_lo = q * (sc & 7), A_hi = q * (sc >> 3), A_m = m ----
        float dw = 0.f, dminw = 0.f;
        {
            uint4 hdr = make_uint4(0, 0, 0, 0);
            const uint8_t *blk = W + (size_t)(row_ok ? row : 0) * row_bytes + (size_t)b * 144;
            if (row_ok) hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
            dw = h2f(hdr.x);
            dminw = h2f(hdr.x >> 16);
            uint32_t sc[2], mn[2];
            sc[0] = hdr.y & 0x3F3F3F3Fu;
            mn[0] = hdr.z & 0x3F3F3F3Fu;
            sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
            mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
            *reinterpret_cast<uint4 *>(sA_m + (size_t)tid * 16) = make_uint4(mn[0], mn[1], 0, 0);
#pragma unroll
            for (int p = 0; p < 4; p++) {
                uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0;
                if (row_ok) {
                    q0 = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + p * 32));
                    q1 = __ldg(reinterpret_cast<const uint4 *>(blk + 32 + p * 32));
                }
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                for (int hl = 0; hl < 2; hl++) {  // hl = 0: low nibbles = sub-block 2p; 1: high nibbles = 2p+1
                    const int s = 2 * p + hl;
                    const uint32_t scs = (sc[s >> 2] >> (8 * (s & 3))) & 0xFFu;
                    const uint32_t f_lo = scs & 7u, f_hi = scs >> 3;
                    uint32_t lo[8], hi[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const uint32_t nib = (hl ? (w[i] >> 4) : w[i]) & 0x0F0F0F0Fu;
                        lo[i] = nib * f_lo;  // bytes <= 15 * 7: no carry between bytes
                        hi[i] = nib * f_hi;
                    }
                    // elements 0..15 of sub-block s -> plane 2s, 16..31 -> plane 2s + 1
                    *reinterpret_cast<uint4 *>(sA_lo + ((size_t)(2 * s) * kTM + tid) * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    *reinterpret_cast<uint4 *>(sA_lo + ((size_t)(2 * s + 1) * kTM + tid) * 16) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                    *reinterpret_cast<uint4 *>(sA_hi + ((size_t)(2 * s) * kTM + tid) * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(sA_hi + ((size_t)(2 * s + 1) * kTM + tid) * 16) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                }
            }
        }
        // ---- activations of this block: codes as planes, bsum split, d8 ----
        {
            const int tk = tid & (kTN - 1), half = tid >> 6;  // 2 threads per token, 8 planes each
            const int tok = tok0 + tk;
            const bool tok_ok = tok < m;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int k16 = half * 8 + k;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (tok_ok) v = *reinterpret_cast<const uint4 *>(a.qs + (size_t)tok * in_f + (size_t)b * 256 + k16 * 16);
                *reinterpret_cast<uint4 *>(sB + ((size_t)k16 * kTN + tk) * 16) = v;
            }
            if (half == 0) {
                uint32_t l[2] = {0, 0}, h[2] = {0, 0};
                if (tok_ok) {
#pragma unroll
                    for (int s = 0; s < 8; s++) {
                        const int bs = a.sums[((size_t)tok * nb + b) * 8 + s];
                        l[s >> 2] |= (uint32_t)(bs & 63) << (8 * (s & 3));
                        h[s >> 2] |= (uint32_t)((bs >> 6) & 0xFF) << (8 * (s & 3));
                    }
                }
                *reinterpret_cast<uint4 *>(sB_ml + (size_t)tk * 16) = make_uint4(l[0], l[1], 0, 0);
                *reinterpret_cast<uint4 *>(sB_mh + (size_t)tk * 16) = make_uint4(h[0], h[1], 0, 0);
                s_d8[tk] = tok_ok ? a.d[(size_t)tok * nb + b] : 0.f;
            }
        }
        // generic-proxy writes -> visible to the tensor core (async proxy); also orders the previous
        // block's tensor-memory reads before this block's MMAs overwrite the accumulators
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid == 0) {
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const uint64_t db = umma_desc(sm_u32(sB + (size_t)(2 * s) * kTN * 16), kTN * 16, 128);
                umma_i8(tmem + 0, umma_desc(sm_u32(sA_lo + (size_t)(2 * s) * kTM * 16), kTM * 16, 128), db, idesc, s > 0);
                umma_i8(tmem + kTN, umma_desc(sm_u32(sA_hi + (size_t)(2 * s) * kTM * 16), kTM * 16, 128), db, idesc, s > 0);
            }
            const uint64_t dam = umma_desc(sm_u32(sA_m), kTM * 16, 128);
            umma_i8(tmem + 2 * kTN, dam, umma_desc(sm_u32(sB_ml), kTN * 16, 128), idesc, 0);
            umma_i8(tmem + 3 * kTN, dam, umma_desc(sm_u32(sB_mh), kTN * 16, 128), idesc, 0);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sm_u32(&bar)) : "memory");
        }
        // ---- wait for the MMAs, then fold the block into the running sums ----
        {
            uint32_t ok = 0;
            for (uint32_t i = 0; i < kMmqSpin && !ok; i++)
                asm volatile(
                    "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                    : "=r"(ok)
                    : "r"(sm_u32(&bar)), "r"(phase)
                    : "memory");
            if (!ok) s_dead = 1;
        }
        phase ^= 1u;
        __syncthreads();
        if (s_dead) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < kTN; c0 += 16) {
            int vlo[16], vhi[16], vml[16], vmh[16];
            tmem_ld16(lane_addr + c0, vlo);
            tmem_ld16(lane_addr + kTN + c0, vhi);
            tmem_ld16(lane_addr + 2 * kTN + c0, vml);
            tmem_ld16(lane_addr + 3 * kTN + c0, vmh);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int sd = vlo[j] + 8 * vhi[j];
                const int sm = vml[j] + 64 * vmh[j];
                const float t = __fsub_rn(__fmul_rn(dw, (float)sd), __fmul_rn(dminw, (float)sm));
                acc[c0 + j] = __fadd_rn(acc[c0 + j], __fmul_rn(s_d8[c0 + j], t));
            }
        }
    }
    if (s_dead) {
        if (tid == 0) atomicExch(status, 4u);
    } else if (row_ok) {
#pragma unroll
        for (int j = 0; j < kTN; j++)
            if (tok0 + j < m) C[(size_t)(tok0 + j) * out_f + row] = acc[j];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256));
}

}  // namespace

cudaError_t launch_mmq_q4k(const uint8_t *w, const Q8Dev &a, float *c, int m, int in_f, int out_f, uint32_t *status,
                           cudaStream_t st) {
    if (m < 1 || in_f % 256 || out_f < 1) return cudaErrorInvalidValue;
    const size_t smem = (size_t)16 * kTM * 16 * 2 + 2 * kTM * 16 + 16 * kTN * 16 + 2 * 2 * kTN * 16 + kTN * 4 + 1024;
    cudaError_t e = cudaFuncSetAttribute(mmq_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((out_f + kTM - 1) / kTM), (unsigned)((m + kTN - 1) / kTN));
    mmq_q4k_kernel<<<grid, kTM, smem, st>>>(w, a, c, m, in_f, out_f, status);
    return cudaGetLastError();
}

}  // namespace infr
