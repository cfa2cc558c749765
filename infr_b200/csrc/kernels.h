// Internal launch interface between the host backend and the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace infr {

enum : int { DT_F32 = 0, DT_F16 = 1, DT_I32 = 3, DT_Q4K = 12, DT_Q6K = 14, DT_Q2_0 = 27 };

inline int block_elems(int dt) { return dt == DT_Q2_0 ? 64 : (dt == DT_Q4K || dt == DT_Q6K ? 256 : 1); }
inline int block_bytes(int dt) {
    switch (dt) {
    case DT_Q4K: return 144;
    case DT_Q6K: return 210;
    case DT_Q2_0: return 18;
    case DT_F32: return 4;
    case DT_F16: return 2;
    default: return 0;
    }
}
// Activation granularity of the production int8 path: 256 for the K-quants, 32 for Q2_0
// (crates/infr-cpu/src/lib.rs:1043-1076).
inline int act_gran(int dt) { return dt == DT_Q2_0 ? 32 : 256; }

// Quantised activation rows in device memory (struct Q8 / Q8x32, crates/infr-cpu/src/quant.rs:8-25, :90-95).
struct Q8Dev {
    const int8_t *qs;      // [rows, k]
    const float *d;        // [rows, k/gran]
    const int32_t *sums;   // [rows, k/32]
    const int32_t *sums16; // [rows, k/16] or null
    int gran;
};

struct DeviceInfo {
    int sm_count;
    int max_smem_optin;
    size_t l2_bytes;
};

// A row-parallel GEMV of a tensor-parallel step whose partial result goes straight to the peers: the epilogue stores
// every value, paired with the exchange's sequence number in ONE 8-byte word, into slot [rank] of EVERY rank's staging
// (plain remote stores over NVLink peer mappings) instead of y.  An aligned 8-byte store arrives whole, so a word
// that carries the expected number carries its value: no fence, no arrival flag, no count of finished CTAs.  The
// consumer (launch_rms_norm_q8_pull) polls the words of its own staging and sums the slots in rank order.
// world == 0: an ordinary GEMV (the result goes to y).
constexpr int kPushMaxWorld = 8;
struct GemvPush {
    unsigned long long *stage[kPushMaxWorld];  // rank r's staging: [2 parities][world][cap] words of (number << 32 | f32 bits)
    const uint32_t *ctrl;                      // this rank's control words: [0] = exchanges completed so far
    uint32_t cap;
    int world, rank;
};
// The consumer's view: this rank's own staging.
struct PullArgs {
    const unsigned long long *stage;
    uint32_t *ctrl;  // [0] exchanges completed (advanced by the consumer's last CTA), [1] consumer CTAs done
    uint32_t cap, spin;
    int world;
    uint32_t *status;
};

cudaError_t launch_quantize_q8(const float *x, int rows, int k, int gran, int8_t *qs, float *d,
                               int32_t *sums, int32_t *sums16, uint16_t *dact, uint16_t *sact,
                               cudaStream_t st);

// y[m,out_f] (m <= 8) from int8 activations; acc_out != null switches to the accumulator dump (m = 1).
cudaError_t launch_gemv_q8(int dt, const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                           int32_t *acc_out, const DeviceInfo &dev, cudaStream_t st);
// Same contract as launch_gemv_q8 without the accumulator dump: the bulk-copy ring kernel.  `status`
// is a device-visible word the kernel sets non-zero if a bounded wait expires.
cudaError_t launch_gemv_stream(int dt, const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f,
                               const DeviceInfo &dev, uint32_t *status, cudaStream_t st);
// Q2_0, m <= 8, rows of whole 512-element chunks, on the warp-level int8 matrix unit (activations quantised
// per 32).  cudaErrorInvalidValue = shape not taken (the caller uses the byte-dot kernel).
cudaError_t launch_gemv_q2_mma(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                               uint32_t *status, cudaStream_t st);
// Q6_K, m <= 8, rows of 8k blocks (row bytes a multiple of 16), on the warp-level int8 matrix unit; needs the
// 16-element activation sums.  cudaErrorInvalidValue = shape not taken.
cudaError_t launch_gemv_q6_mma(const uint8_t *w, const Q8Dev &a, float *y, int m, int in_f, int out_f, const DeviceInfo &dev,
                               uint32_t *status, cudaStream_t st, const GemvPush *push = nullptr);
// Q4_K, m <= 8, on the warp-level int8 matrix unit.  Exactly one of `a` (pre-quantised rows) and `x`
// (f32 rows, quantised inside the kernel) is non-null.
cudaError_t launch_gemv_q4k_mma(const uint8_t *w, const Q8Dev *a, const float *x, float *y, int m, int in_f, int out_f,
                                const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const GemvPush *push = nullptr);
// Two Q4_K matrices [out_f1, in_f] and [out_f2, in_f] against the same pre-quantised rows in ONE launch (q and k,
// gate and up: a decode step pays a fixed few microseconds per dependent launch).
cudaError_t launch_gemv_q4k_mma_pair(const uint8_t *w1, float *y1, int out_f1, const uint8_t *w2, float *y2, int out_f2, const Q8Dev *a,
                                     const float *x, int m, int in_f, const DeviceInfo &dev, uint32_t *status, cudaStream_t st);
// y[m,out_f] (m <= 8) from f32 activations and dequantised weights.
cudaError_t launch_gemv_f32(int dt, const uint8_t *w, const float *x, float *y, int m, int in_f, int out_f,
                            const DeviceInfo &dev, cudaStream_t st);

// Batched GEMV for 9..32 pre-quantised rows (Q4_K, Q6_K): every weight byte unpacked once for all rows, activations in
// registers, K cut into chunks of 2048 elements across CTAs (`partials`: gemv_wide_partial_bytes(...) bytes of scratch).
size_t gemv_wide_partial_bytes(int m, int in_f, int out_f);
int gemv_wide_launches(int in_f);
// w2 / y2 / out_f2: a second matrix of the same format and in_f against the same rows in the same launches (partials
// then holds gemv_wide_partial_bytes(m, in_f, out_f + out_f2)).
cudaError_t launch_gemv_wide(int dtype, const uint8_t *w, const Q8Dev &a, float *y, float *partials, int m, int in_f, int out_f,
                             const DeviceInfo &dev, uint32_t *status, cudaStream_t st, const GemvPush *push = nullptr, const uint8_t *w2 = nullptr,
                             float *y2 = nullptr, int out_f2 = 0);

// Prefill GEMM C[m,out_f] = Q8(256) activations x Q4_K weights on tcgen05 (kind::i8, TMEM accumulators);
// bit-identical to the CPU production path.
// `records` is scratch of mmq_q4k_record_bytes(m, in_f) bytes (per-token block sums and scales in the layout
// the kernel's TMA loads expect).
size_t mmq_q4k_record_bytes(int m, int in_f);
cudaError_t launch_mmq_q4k(const uint8_t *w, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                           const DeviceInfo &dev, uint32_t *status, cudaStream_t st);
// The same GEMM with specialised warps (unpack / MMA issue / epilogue overlap) and the min term summed in
// tensor memory by kind::tf32 MMAs: int32 block sums identical, f32 result within rounding of the CPU's.
size_t mmq_ws_record_bytes(int m, int in_f);
// Few row x token tiles (a batch of a few dozen rows, a few thousand outputs): K is split across CTAs and a second
// kernel adds the partial results in split order; `partials` is mmq_ws_partial_bytes(...) bytes of scratch.
int mmq_ws_k_splits(int m, int in_f, int out_f, const DeviceInfo &dev);
size_t mmq_ws_partial_bytes(int m, int in_f, int out_f, const DeviceInfo &dev);
cudaError_t launch_mmq_ws_q4k(const uint8_t *w, const Q8Dev &a, void *records, float *c, int m, int in_f, int out_f,
                              const DeviceInfo &dev, uint32_t *status, cudaStream_t st, float *partials = nullptr);
// The GEMM from f32 activations: x != nullptr quantises them straight into the kernel's layout in `records`; x == nullptr
// reuses what a previous call wrote there for the same activations (q and k, gate and up of a batch).
cudaError_t launch_mmq_ws_q4k_f32(const uint8_t *w, const float *x, void *records, float *c, int m, int in_f, int out_f,
                                  const DeviceInfo &dev, uint32_t *status, cudaStream_t st, float *partials = nullptr);
// The same tensor-memory GEMM over a bank of expert matrices, one 64-token slab of routed rows per tile column
// (mmq_ws.cu).  `records`: mmq_ws_record_bytes(max_slabs * 64, in_f) bytes; prep = false reuses planes already laid.
cudaError_t launch_mmq_ws_q4k_grouped(const uint8_t *bank, int n_experts, const Q8Dev &a, void *records, float *y, int in_f, int out_f,
                                      const int *slab_expert, const int *slab_p0, const int *slab_cnt, const int *n_slabs,
                                      const int *pair_row, int max_slabs, bool prep, const DeviceInfo &dev, uint32_t *status,
                                      cudaStream_t st);
// Grouped Q4_K GEMM over a bank of n_experts matrices [out_f, in_f] stored back to back: work item i
// multiplies up to 8 quantised activation rows (pairs item_p0[i]..+item_cnt[i], gathered through
// pair_row when non-null) with expert item_expert[i]; y is [n_pairs, out_f].
cudaError_t launch_grouped_q4k_mma(const uint8_t *bank, int n_experts, const Q8Dev &a, float *y, int in_f, int out_f,
                                   const int *item_expert, const int *item_p0, const int *item_cnt, const int *n_items,
                                   const int *pair_row, int max_items, const DeviceInfo &dev, uint32_t *status,
                                   cudaStream_t st);
// The same grouped product for a Q6_K bank (direct-load byte-dot kernel, any row length); `a` needs the sums per 16.
cudaError_t launch_grouped_q6k(const uint8_t *bank, const Q8Dev &a, float *y, int in_f, int out_f, const int *item_expert, const int *item_p0,
                               const int *item_cnt, const int *n_items, const int *pair_row, int max_items, const DeviceInfo &dev,
                               cudaStream_t st);
cudaError_t launch_moe_router(const float *router, const float *x, float *logits, int rows, int ne, int n_expert,
                              cudaStream_t st);
cudaError_t launch_moe_route(const float *logits, int rows, int n_expert, int n_used, float scale, int norm_w,
                             int32_t *sel_ids, float *sel_w, cudaStream_t st);
cudaError_t launch_moe_bucket(const int32_t *sel_ids, int rows, int n_used, int n_expert, int e_lo, int n_local, int item_rows,
                              int32_t *pair_row, int32_t *pair_of_slot, int32_t *item_expert, int32_t *item_p0, int32_t *item_cnt,
                              int32_t *n_items, int32_t *counts_out, cudaStream_t st);
cudaError_t launch_moe_swiglu_quant(const float *gate, const float *up, int n_pairs, int nff, int8_t *qs, float *d,
                                    int32_t *sums, int32_t *sums16, float *act_out, cudaStream_t st);
cudaError_t launch_moe_combine(const float *y_pairs, const int32_t *pair_of_slot, const float *sel_w, int rows, int n_used,
                               int ne, float *out, cudaStream_t st);

// f32-activation GEMV of routed pair p against expert sel[p] of a Q4_K bank (stride w_stride bytes):
// y[p, :] = dequant(bank[sel[p]]) * x[x_div ? p / x_div : p, :].
cudaError_t launch_gemv_q4k_f32_sel(const uint8_t *bank, const int32_t *sel, size_t w_stride, const float *x, int x_div,
                                    float *y, int n_pairs, int in_f, int out_f, const DeviceInfo &dev, cudaStream_t st);

// Dense int8 tensor-core peak microbenchmark (tensor_peak.cu): one launch = every SM issues 2 x n_batches x 64
// tcgen05 kind::i8 instructions of shape 128 x 256 x 32 from resident shared-memory operands.
cudaError_t launch_tensor_peak_i8(uint32_t n_batches, int32_t *check, const DeviceInfo &dev, uint32_t *status, cudaStream_t st);
double tensor_peak_i8_ops(uint32_t n_batches, const DeviceInfo &dev);
int32_t tensor_peak_i8_expected(uint32_t n_batches);

cudaError_t launch_fill_u32(uint32_t *p, size_t n, uint32_t v, cudaStream_t st);

// ---- dense decode-step ops (decode_ops.cu) ----
// RMSNorm of `rows` rows; with b != nullptr the row is a + b, also written to sum_dst (may alias a).
cudaError_t launch_rms_norm(const float *a, const float *b, float *sum_dst, const float *w, float *dst, int rows, int dim, float eps,
                            cudaStream_t st);
cudaError_t launch_rope(const float *x, const int32_t *positions, float *dst, int rows, int n_head, int head_dim, int rope_dim, float theta,
                        int neox, const DeviceInfo &dev, cudaStream_t st);
cudaError_t launch_rope_write_kv(float *q, const float *k, const float *v, const int32_t *positions, void *k_cache, void *v_cache, int rows,
                                 int n_head, int n_kv, int head_dim, float theta, int neox, int rows_per_seq, size_t seq_stride,
                                 const DeviceInfo &dev, cudaStream_t st, int write_pos = -1, const int32_t *block_table = nullptr, int table_stride = 0, int n_pages = 0);
cudaError_t launch_write_kv_f16(const float *src, void *cache_at_pos, size_t n, const DeviceInfo &dev, cudaStream_t st);
size_t attention_workspace_bytes(int q_rows, int n_head, int head_dim, int max_keys);
// With qs != nullptr the merged rows are quantised (256-element blocks) instead of stored to dst.
cudaError_t launch_attention(const float *q, const void *k_cache, const void *v_cache, float *dst, void *workspace, int n_seq, int rows, int n_head,
                             int n_kv, int head_dim, float scale, int pos, size_t seq_stride, int sm_count, cudaStream_t st, uint32_t *status,
                             int8_t *qs = nullptr, float *d = nullptr, int32_t *sums = nullptr, int32_t *sums16 = nullptr,
                             const int32_t *seq_pos = nullptr, const int32_t *block_table = nullptr, int table_stride = 0, int n_pages = 0);
// Producers that end in the activation quantiser (256-element blocks; sums16 may be null).
cudaError_t launch_rms_norm_q8(const float *a, const float *b, float *sum_dst, const float *w, int rows, int dim, float eps, int8_t *qs, float *d,
                               int32_t *sums, int32_t *sums16, cudaStream_t st);
// a + (the sum over ranks of the pushed partial results, in rank order) -> sum_dst, then RMSNorm and the quantiser.
cudaError_t launch_rms_norm_q8_pull(const float *a, float *sum_dst, const float *w, int rows, int dim, float eps, int8_t *qs, float *d,
                                    int32_t *sums, int32_t *sums16, const PullArgs &pull, cudaStream_t st);
cudaError_t launch_gated_silu_q8(const float *gate, const float *up, int rows, int nff, int8_t *qs, float *d, int32_t *sums, int32_t *sums16,
                                 cudaStream_t st);
cudaError_t launch_gated_silu(const float *gate, const float *up, float *dst, size_t n, const DeviceInfo &dev, cudaStream_t st);
cudaError_t launch_add(const float *a, const float *b, float *dst, size_t n, const DeviceInfo &dev, cudaStream_t st);
size_t argmax_workspace_bytes(uint32_t n, uint32_t rows);
cudaError_t launch_argmax(const float *x, uint32_t *dst, void *workspace, uint32_t n, uint32_t rows, cudaStream_t st);

}  // namespace infr
