/*
 * libinfr_cuda.so — C ABI of the sm_100a implementation of infr's block-quantized matmul path.
 *
 * This is the boundary a Rust `infr-cuda` crate binds with `extern "C"` to implement the reference's
 * `trait Backend` (crates/infr-core/src/backend.rs:486-662) and its companion `Buffer` / `Plan`
 * traits (:387-446).  Every entry point takes plain pointers and sizes; nothing here exposes C++,
 * CUDA or torch types.  All functions return an int32 status (0 = ok, negative = error); the text of
 * the last error of a context is fetched with infr_cuda_last_error().  Nothing in the library falls
 * back to the CPU: without a usable CUDA device infr_cuda_create() fails.
 *
 * Threading: a context serialises its own calls with an internal mutex (the reference holds a
 * backend as Arc<dyn Backend> and may call it from several threads, backend.rs:486).
 */
#ifndef INFR_CUDA_H
#define INFR_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define INFR_API
#else
#define INFR_API __attribute__((visibility("default")))
#endif

/* ---- status codes (map onto infr_core::error::Error, crates/infr-core/src/error.rs:6-25) ---- */
#define INFR_OK 0
#define INFR_E_INVALID (-1)     /* Error::Backend: bad size / shape / null / unbound handle */
#define INFR_E_UNSUPPORTED (-2) /* Error::Unsupported: op or dtype this backend does not run */
#define INFR_E_OOM (-3)         /* Error::Backend: device allocation failed */
#define INFR_E_CUDA (-4)        /* Error::Backend: a CUDA runtime call failed */
#define INFR_E_NCCL (-5)
#define INFR_E_TIMEOUT (-6)     /* a bounded device-side wait expired */

/* ---- dtype codes: the declaration order of `enum DType`, crates/infr-core/src/tensor.rs:7-57 ---- */
#define INFR_DT_F32 0
#define INFR_DT_F16 1
#define INFR_DT_I32 3
#define INFR_DT_Q4K 12
#define INFR_DT_Q6K 14
#define INFR_DT_Q2_0 27

/* ---- BufferUsage (crates/infr-core/src/backend.rs:359-380); advisory ---- */
#define INFR_USAGE_WEIGHTS 0
#define INFR_USAGE_ACTIVATIONS 1
#define INFR_USAGE_KV 2
#define INFR_USAGE_READBACK 3

/* ---- TensorKind (crates/infr-core/src/graph.rs:111-122) ---- */
#define INFR_TK_INPUT 0
#define INFR_TK_WEIGHT 1
#define INFR_TK_INTERNAL 2
#define INFR_TK_OUTPUT 3

/* ---- activation representation of a quantized Linear ---- */
#define INFR_ACT_INT8 0 /* production infr-cpu arithmetic: Q8 activations, integer block dots */
#define INFR_ACT_F32 1  /* `kernels.cpu.reference` arithmetic: dequantised weights, f32 dot */

typedef struct infr_cuda_ctx infr_cuda_ctx;
typedef struct infr_cuda_buf infr_cuda_buf;
typedef struct infr_cuda_plan infr_cuda_plan;
typedef struct infr_cuda_comm infr_cuda_comm;
typedef struct infr_cuda_graph infr_cuda_graph;

/* Options of infr_cuda_create.  `reference` mirrors CpuCfg::reference
 * (crates/infr-core/src/config/mod.rs:425-438): when non-zero every quantized Linear / MoeFfn run by
 * infr_cuda_execute uses INFR_ACT_F32 arithmetic. */
/* gemv_kernel / mmq_kernel choose between kernels that compute the same op (0 = the default dispatch); they exist
 * so that the parity tests can reach every kernel of the library on every shape:
 *   gemv_kernel 1: the direct-load byte-dot GEMV for all formats and batches;
 *   mmq_kernel  1: the Q4_K prefill GEMM whose f32 output is bit-identical to the CPU's (slower),
 *               2: the grouped tensor-memory GEMM also for MoE layers with a handful of rows per expert,
 *               3: no GEMM: batches of more than 8 rows are walked through the GEMV 8 rows at a time. */
typedef struct {
    int32_t device;
    int32_t reference;
    int32_t gemv_kernel;
    int32_t mmq_kernel;
    int32_t reserved[4];
} infr_cuda_opts;

/* The subset of `struct Capabilities` (crates/infr-core/src/backend.rs:43-213) this backend sets;
 * every field not listed is false / 0 / None on the Rust side. */
typedef struct {
    char name[32]; /* "cuda-sm100a" */
    int32_t f16, i8, i8_dot, integrated, unified_memory, decode_replay, graph_input_inplace;
    uint32_t max_shared_memory_bytes;
    uint32_t sm_count;
    uint64_t total_memory_bytes;
    uint64_t l2_bytes;
} infr_cuda_caps;

/* ---- lifecycle: `Backend::name/capabilities`, backend.rs:487-488 ---- */
INFR_API int32_t infr_cuda_create(const infr_cuda_opts *opts, infr_cuda_ctx **out);
INFR_API void infr_cuda_destroy(infr_cuda_ctx *ctx);
INFR_API int32_t infr_cuda_get_caps(infr_cuda_ctx *ctx, infr_cuda_caps *out);
/* Copies the NUL-terminated message of the most recent failing call on `ctx` (NULL = the failing
 * infr_cuda_create of this thread).  Returns the message length. */
INFR_API int32_t infr_cuda_last_error(infr_cuda_ctx *ctx, char *dst, size_t cap);

/* ---- memory: `Backend::alloc / alloc_uninit / upload / download / copy_buffer`, backend.rs:491-558;
 *      `Buffer::len_bytes`, backend.rs:387-398.  alloc is zero-initialised (calloc semantics). ---- */
INFR_API int32_t infr_cuda_alloc(infr_cuda_ctx *ctx, size_t bytes, int32_t usage, infr_cuda_buf **out);
INFR_API int32_t infr_cuda_alloc_uninit(infr_cuda_ctx *ctx, size_t bytes, int32_t usage, infr_cuda_buf **out);
/* No counterpart in the trait (its buffers are always the backend's own): a handle over device memory the
 * caller owns — a tensor of the host framework, a slice of another engine's pool — so that ops can read and
 * write it in place.  Nothing is allocated or copied; infr_cuda_free on such a handle drops the handle only.
 * The pointer must be 16-byte aligned and the range must stay valid while the handle is in use; ranges handed
 * to ops as weights must be readable 256 bytes past `bytes` rounded down to 16 (vector loads on a row's tail
 * never leave the backend's own padded allocations, and must not leave the caller's either). */
INFR_API int32_t infr_cuda_wrap(infr_cuda_ctx *ctx, void *device_ptr, size_t bytes, int32_t usage, infr_cuda_buf **out);
/* The CUDA stream (cudaStream_t as void*) the context enqueues all its work on, so that a caller can order
 * its own kernels and collectives with the context's without a device-wide synchronise. */
INFR_API void *infr_cuda_stream(infr_cuda_ctx *ctx);
INFR_API void infr_cuda_free(infr_cuda_ctx *ctx, infr_cuda_buf *buf);

/* No counterpart in the reference (it has no multi-GPU path): the exchange a row-parallel Linear needs when a
 * model is split over the GPUs of one box, one process per GPU.  In-place sum of n f32 (a multiple of 4, at
 * most max_floats <= 262144) over `world` <= 8 ranks, as one kernel over NVLink peer memory on the context's
 * stream (capturable in a CUDA graph); every rank gets the same bits (slots are summed in rank order).
 * Set-up: every rank creates a comm, exports its 64-byte handle (a CUDA IPC memory handle), the host program
 * gathers the handles of all ranks in rank order by whatever channel it has, and every rank connects.
 * All ranks must issue the same sequence of all-reduces.  A peer that never arrives makes the bounded wait
 * expire: the data is left unsummed and the next infr_cuda_sync returns INFR_E_TIMEOUT.
 * Ordering the host program owes (one process per GPU, so only the host can give it):
 *  - a host barrier over all ranks after every rank has connected and BEFORE the first exchange: the wait is a
 *    few seconds of polling, and a rank still loading weights or capturing a graph would let its peers' waits expire;
 *  - a host barrier after every rank has synchronised its last exchange and BEFORE any rank calls
 *    infr_cuda_comm_destroy: destroy frees memory the peers have mapped and may still be storing into.
 * Where the reference's multi-GPU sketch has one `group` object owning N devices in one process, this library has
 * one context and one comm per process; infr_cuda_comm_* stands in for a group constructor. */
INFR_API int32_t infr_cuda_comm_create(infr_cuda_ctx *ctx, int32_t rank, int32_t world, uint32_t max_floats, infr_cuda_comm **out);
INFR_API int32_t infr_cuda_comm_export(infr_cuda_ctx *ctx, infr_cuda_comm *comm, uint8_t *handle64);
INFR_API int32_t infr_cuda_comm_connect(infr_cuda_ctx *ctx, infr_cuda_comm *comm, const uint8_t *handles /* [world][64] */);
/* Failure-detection aid: instead of connecting real peers, map every peer slot onto a private buffer of this
 * rank that nobody writes, and let a wait give up after spin_limit polls (1 .. 4194304).  The next all-reduce
 * then returns without summing and infr_cuda_sync reports INFR_E_TIMEOUT; the context stays usable.  This is how
 * a host program (and this library's tests) exercise the path a vanished rank would take, without one. */
INFR_API int32_t infr_cuda_comm_connect_silent(infr_cuda_ctx *ctx, infr_cuda_comm *comm, uint32_t spin_limit);
INFR_API int32_t infr_cuda_all_reduce_f32(infr_cuda_ctx *ctx, infr_cuda_comm *comm, infr_cuda_buf *data, uint32_t n);
INFR_API void infr_cuda_comm_destroy(infr_cuda_ctx *ctx, infr_cuda_comm *comm);
INFR_API size_t infr_cuda_buf_len(const infr_cuda_buf *buf);
INFR_API uint64_t infr_cuda_buf_device_ptr(const infr_cuda_buf *buf);
/* upload/download reject a transfer larger than the buffer (check_copy_bytes, backend.rs:23-30).  `src` may be
 * reused as soon as upload returns: transfers of at most 64 KB are staged through pinned memory of the context and
 * return without waiting for the stream, larger ones wait for their copy; either way the data is in place for every
 * op enqueued afterwards.  download returns when `dst` holds the data. */
INFR_API int32_t infr_cuda_upload(infr_cuda_ctx *ctx, infr_cuda_buf *dst, const void *src, size_t bytes);
INFR_API int32_t infr_cuda_upload_at(infr_cuda_ctx *ctx, infr_cuda_buf *dst, size_t dst_off, const void *src, size_t bytes);
INFR_API int32_t infr_cuda_download(infr_cuda_ctx *ctx, const infr_cuda_buf *src, void *dst, size_t bytes);
INFR_API int32_t infr_cuda_copy(infr_cuda_ctx *ctx, const infr_cuda_buf *src, infr_cuda_buf *dst, size_t bytes);
/* Page-locked host memory for staging uploads/downloads (the reference's Vulkan backend stages
 * through host-visible memory the same way; no counterpart on the CPU backend). */
INFR_API int32_t infr_cuda_host_alloc(infr_cuda_ctx *ctx, size_t bytes, void **out);
INFR_API void infr_cuda_host_free(infr_cuda_ctx *ctx, void *p);
/* `Backend::sync`, backend.rs:596. */
INFR_API int32_t infr_cuda_sync(infr_cuda_ctx *ctx);

/* ---- graphs: `Backend::compile / execute`, backend.rs:561-562 ----
 * infr_graph_desc is a flat POD mirror of `Graph` (crates/infr-core/src/graph.rs:1317-1460): an
 * ordered op list over typed tensor handles; handle i is TensorId(i). */
typedef struct {
    uint32_t kind;  /* INFR_TK_* */
    uint32_t dtype; /* INFR_DT_* */
    uint64_t numel;
} infr_tensor_decl;

#define INFR_OP_LINEAR 1    /* Op::Linear, graph.rs:179-191 */
#define INFR_OP_MOE_FFN 2   /* Op::MoeFfn, graph.rs:918-1011 */
#define INFR_OP_RMS_NORM 3  /* Op::RmsNorm, graph.rs:141-148 */
#define INFR_OP_ROPE 4      /* Op::Rope, graph.rs:268-319 */
#define INFR_OP_WRITE_KV 5  /* Op::WriteKv, graph.rs:343-349 */
#define INFR_OP_ATTENTION 6 /* Op::Attention, graph.rs:353-397 */
#define INFR_OP_GATED_ACT 7 /* Op::GatedAct, graph.rs:707-736 */
#define INFR_OP_ADD 8       /* Op::Add, graph.rs:753-758 */
#define INFR_OP_ARGMAX 9    /* Op::Argmax, graph.rs:803-808 */
#define INFR_OP_COPY 10     /* Op::Copy, graph.rs:890-896 */

/* One op.  Field use per tag, in the field order of the Rust variant (an `Option` field travels as a has_* flag;
 * where this backend does not run the option the flag must be 0, else compile returns INFR_E_UNSUPPORTED):
 *  INFR_OP_LINEAR   : t = {x, weight, dst}; u = {m, in_f, out_f, w_off}
 *  INFR_OP_MOE_FFN  : t = {x, router_x, router, gate_exps, up_exps, down_exps, dst};
 *                     u = {ne, n_expert, n_used, n_ff_exp, norm_w, fused_gate_up, weight_before,
 *                          act (0 = SiLU), gating (0 = Softmax)}; f = {scale}
 *      Fields of Op::MoeFfn without a slot here (down_scale, swiglu_clamp, ep_band, exp_probs_b,
 *      expert groups, expert_ids) must be None/0 on the Rust side; the binding returns
 *      Error::Unsupported otherwise.  Banks: Q4_K or Q6_K (each bank on its own), router F32.
 *  INFR_OP_RMS_NORM : t = {x, weight, dst}; u = {rows, dim}; f = {eps}
 *  INFR_OP_ROPE     : t = {x, positions, dst}; u = {rows, n_head, head_dim, rope_dim, x_stride, neox, backward,
 *                     has_freq_factors}; f = {theta}          (x_stride 0 or packed; backward, freq_factors: not run)
 *  INFR_OP_WRITE_KV : t = {src, cache}; u = {rows, row_stride, pos}                       (cache dtype F16)
 *  INFR_OP_ATTENTION: t = {q, k_cache, v_cache, dst}; u = {rows, kv_len, n_head, n_kv, head_dim, mask (0 = Causal),
 *                     pos, has_sinks}; f = {scale}            (F16 caches, kv_len = pos + rows, no sinks)
 *  INFR_OP_GATED_ACT: t = {gate, up, dst}; u = {rows, nff, act (0 = SiLU), up_off, up_stride, gate_stride,
 *                     gate_block_width, has_swiglu_clamp}     (packed rows, SiLU, no clamp)
 *  INFR_OP_ADD      : t = {a, b, dst}; u = {n}
 *  INFR_OP_ARGMAX   : t = {x, dst}; u = {n, rows}             (dst holds u32 ids)
 *  INFR_OP_COPY     : t = {src, dst}; u = {src_off, dst_off, n}  (element offsets of 4-byte elements)
 * This is the op list `generate_dense_backend` emits for a Llama-family decode step when the backend advertises
 * the conservative capability set (crates/infr-llama/src/seam/runner.rs:2641-4493). */
typedef struct {
    uint32_t tag;
    uint32_t t[8];
    uint32_t u[12];
    float f[4];
} infr_op_desc;

typedef struct {
    const infr_tensor_decl *tensors;
    uint32_t n_tensors;
    const infr_op_desc *ops;
    uint32_t n_ops;
} infr_graph_desc;

INFR_API int32_t infr_cuda_compile(infr_cuda_ctx *ctx, const infr_graph_desc *graph, infr_cuda_plan **out);
INFR_API void infr_cuda_plan_free(infr_cuda_ctx *ctx, infr_cuda_plan *plan);
/* bindings[i] is the buffer bound to TensorId(i), NULL = unbound (`Bindings`, backend.rs:457-483).
 * Internal handles are backend scratch, zeroed before the walk (crates/infr-core/src/exec.rs:53-92).
 * An unbound Input/Weight/Output handle used by an op is INFR_E_INVALID (the CPU reference panics
 * there, crates/infr-cpu/src/lib.rs:754).
 * A plan of two or more launches that is run again on the same buffers is replayed as a CUDA graph from its second
 * run (one graph launch instead of one launch per op); other buffers, a reallocated context scratch or other kernel
 * options run it op by op again.  Inside a caller's own stream capture the ops are always issued directly. */
INFR_API int32_t infr_cuda_execute(infr_cuda_ctx *ctx, infr_cuda_plan *plan,
                                   infr_cuda_buf *const *bindings, uint32_t n_bindings);

/* ---- direct kernel entry points (what `execute` dispatches to; used by benches and tests) ----
 * All pointers are infr_cuda_buf handles; byte offsets select a sub-range. */

/* Activation quantiser.  gran = 256: `quantize_q8` (crates/infr-cpu/src/quant.rs:27-58): qs i8
 * [rows,k], d f32 [rows,k/256], sums i32 [rows,k/32] (`bsums`), sums16 i32 [rows,k/16] (nullable).
 * gran = 32: `quantize_q8_32` (quant.rs:97-117): d f32 [rows,k/32], sums i32 [rows,k/32]. */
INFR_API int32_t infr_cuda_quantize_q8(infr_cuda_ctx *ctx, int32_t gran, const infr_cuda_buf *x,
                                       uint32_t rows, uint32_t k, infr_cuda_buf *qs, infr_cuda_buf *d,
                                       infr_cuda_buf *sums, infr_cuda_buf *sums16);
/* The "Q8_1" view of the reference's GPU path (crates/infr-vulkan/shaders/quant_q8.comp:37-61):
 * same int8 codes as gran = 32, dact = f16(d), sact = f16(d * float(sum of codes)). */
INFR_API int32_t infr_cuda_quantize_q8_1(infr_cuda_ctx *ctx, const infr_cuda_buf *x, uint32_t rows,
                                         uint32_t k, infr_cuda_buf *qs, infr_cuda_buf *dact,
                                         infr_cuda_buf *sact);

/* y[m,out_f] = x[m,in_f] * W^T for m <= 8 (decode).  W is raw GGUF blocks, row-major [rows,in_f];
 * w_off is the ELEMENT offset of the first row used (Op::Linear::w_off).  act selects INFR_ACT_*.
 * Replaces the m == 1 / small-m arms of crates/infr-cpu/src/lib.rs:1035-1167. */
INFR_API int32_t infr_cuda_gemv(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off,
                                const infr_cuda_buf *x, infr_cuda_buf *y, uint32_t m, uint32_t in_f,
                                uint32_t out_f, int32_t act);
/* infr_cuda_gemv(INFR_ACT_INT8) on activations that are ALREADY quantised by infr_cuda_quantize_q8
 * (gran 256 for Q4_K / Q6_K — Q6_K also needs sums16 —, gran 32 for Q2_0): the CPU reference
 * quantises an activation row once and reuses it for every weight row and every projection that
 * reads it (crates/infr-cpu/src/lib.rs:1043-1062); this entry point is that reuse.  m <= 8, and more rows where the
 * wide GEMV applies (Q4_K: m <= 32; Q6_K with in_f a multiple of 2048: any m), so that a decode step over a few dozen
 * sequences keeps its activations in int8 between ops like a step over one. */
INFR_API int32_t infr_cuda_gemv_q8(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off,
                                   const infr_cuda_buf *qs, const infr_cuda_buf *d, const infr_cuda_buf *sums,
                                   const infr_cuda_buf *sums16, infr_cuda_buf *y, uint32_t m, uint32_t in_f,
                                   uint32_t out_f);
/* Two weights of one format against the same quantised rows (infr_cuda_gemv_q8 twice, same results): q and k, or gate
 * and up, of a decode step.  The reference gets the same effect from `w_off` slices of one fused weight
 * (crates/infr-llama/src/seam/runner.rs:3445-3461, :3842-3879); here the two weights may live anywhere, and Q4_K
 * pairs run as ONE launch (a decode step pays a fixed few microseconds per dependent launch). */
INFR_API int32_t infr_cuda_gemv_q8_pair(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w1, uint64_t w_off1, infr_cuda_buf *y1,
                                        uint32_t out_f1, const infr_cuda_buf *w2, uint64_t w_off2, infr_cuda_buf *y2, uint32_t out_f2,
                                        const infr_cuda_buf *qs, const infr_cuda_buf *d, const infr_cuda_buf *sums,
                                        const infr_cuda_buf *sums16, uint32_t m, uint32_t in_f);
/* No counterpart in the reference: a decode GEMV (INFR_ACT_INT8 arithmetic, same results as
 * infr_cuda_gemv) for callers that cannot allocate device memory when they need it — plugins living
 * inside another engine's memory pool, loops that must stay clear of the driver's allocator after
 * start-up.  It takes RAW device pointers (w: GGUF blocks of the first row used, x: f32 [m,in_f],
 * y: f32 [m,out_f]) and a cudaStream_t passed as void* (NULL = the default stream), needs no context,
 * and keeps its quantised activations in a 192 KiB array built into the library (held by every GPU
 * that loads it) instead of allocating: the call runs no cudaMalloc / cudaFree / allocating routine.
 * Limits: m <= 8, in_f <= 16384; larger sizes are rejected with INFR_E_INVALID.  Alignment: x on 16 bytes,
 * y on 4, w on 16 for Q4_K and on 2 for Q6_K / Q2_0; a misaligned pointer is INFR_E_INVALID.  The first call on a
 * device looks up the array's device address (cudaGetSymbolAddress) — make that call before any
 * stream capture.  All calls share the one array: calls that overlap on the GPU (different streams,
 * or threads) race on it; calls on one stream are ordered and need no clearing in between.  Work is
 * enqueued on `stream`; the caller synchronises.  On failure a message is copied into err. */
INFR_API int32_t infr_cuda_gemv_noalloc(int32_t dtype, const void *w, const float *x, float *y, uint32_t m,
                                        uint32_t in_f, uint32_t out_f, void *stream, char *err, size_t err_cap);
/* Same arithmetic as infr_cuda_gemv(INFR_ACT_INT8) for m = 1, but writes the per-block int32
 * accumulators instead of y: Q4_K -> acc[out_f][in_f/256][2] = (sd, sm) of
 * crates/infr-cpu/src/kernels.rs:161-181; Q6_K -> acc[out_f][in_f/256] = isum (:519-523);
 * Q2_0 -> acc[out_f][in_f/32] = iprod (:5655-5663). */
INFR_API int32_t infr_cuda_gemv_block_acc(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w,
                                          uint64_t w_off, const infr_cuda_buf *x, infr_cuda_buf *acc,
                                          uint32_t in_f, uint32_t out_f);

/* Op::Linear of any m (crates/infr-cpu/src/lib.rs:985-1492): dispatches to the GEMV (m <= 8) or the
 * MMQ GEMM.  act as above. */
INFR_API int32_t infr_cuda_linear(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off,
                                  const infr_cuda_buf *x, infr_cuda_buf *y, uint32_t m, uint32_t in_f,
                                  uint32_t out_f, int32_t act);

/* Two Op::Linear of one weight format on the same rows (q and k, gate and up), results as from two infr_cuda_linear
 * calls: the rows are quantised once (and laid out once for the prefill GEMM); for at most 8 rows of Q4_K the two
 * products are one launch.  infr_cuda_execute pairs neighbouring Linear ops of a graph the same way. */
INFR_API int32_t infr_cuda_linear_pair(infr_cuda_ctx *ctx, int32_t dtype, const infr_cuda_buf *w1, uint64_t w_off1, infr_cuda_buf *y1,
                                       uint32_t out_f1, const infr_cuda_buf *w2, uint64_t w_off2, infr_cuda_buf *y2, uint32_t out_f2,
                                       const infr_cuda_buf *x, uint32_t m, uint32_t in_f, int32_t act);

/* Op::MoeFfn as a direct call (crates/infr-core/src/graph.rs:918-1011; CPU semantics
 * crates/infr-cpu/src/lib.rs:2264-2984): F32 router [n_expert, ne], expert banks gate/up
 * [n_expert][n_ff_exp, ne] and down [n_expert][ne, n_ff_exp] as raw GGUF blocks (Q4_K or Q6_K, `expert_acts_kind`
 * Super of crates/infr-cpu/src/moe.rs:42-53; Q6_K banks on the int8 path, rows >= 2), softmax gating,
 * top-n_used with ties to the lower expert id, SiLU gate, output-side weighting.  dst is f32 [rows, ne].
 * Optional outputs for parity checks (NULL = not wanted): sel_ids i32 [rows, n_used] in rank order,
 * sel_w f32 [rows, n_used], logits f32 [rows, n_expert]. */
typedef struct {
    uint32_t rows, ne, n_expert, n_used, n_ff_exp;
    float scale;
    int32_t norm_w;
    int32_t router_dtype, gate_dtype, up_dtype, down_dtype; /* INFR_DT_* */
    /* Expert parallelism (no counterpart in the reference): n_local != 0 says the banks hold only experts
     * [expert_lo, expert_lo + n_local) — bank index = expert - expert_lo — and dst receives only their
     * contribution; the router stays whole and every rank routes every row, so the ranks' dst add up to the
     * unsharded result (the caller all-reduces them).  n_local == 0: all experts are here.  Needs rows >= 2. */
    uint32_t expert_lo, n_local;
} infr_moe_desc;
INFR_API int32_t infr_cuda_moe_ffn(infr_cuda_ctx *ctx, const infr_moe_desc *desc, const infr_cuda_buf *x,
                                   const infr_cuda_buf *router_x, const infr_cuda_buf *router,
                                   const infr_cuda_buf *gate_exps, const infr_cuda_buf *up_exps,
                                   const infr_cuda_buf *down_exps, infr_cuda_buf *dst, infr_cuda_buf *sel_ids,
                                   infr_cuda_buf *sel_w, infr_cuda_buf *logits);

/* ---- the other ops of a dense decode step (the reference's op sequence per layer:
 * crates/infr-llama/src/seam/runner.rs:2641-4286; semantics: the CPU backend's arms in
 * crates/infr-cpu/src/lib.rs).  All buffers hold f32 unless said otherwise. ---- */
/* Op::RmsNorm (graph.rs; cpu lib.rs:801-825): dst[r,i] = x[r,i] / sqrt(mean(x[r]^2) + eps) * weight[i]. */
INFR_API int32_t infr_cuda_rms_norm(infr_cuda_ctx *ctx, const infr_cuda_buf *x, const infr_cuda_buf *weight, infr_cuda_buf *dst,
                                    uint32_t rows, uint32_t dim, float eps);
/* Op::Add followed by Op::RmsNorm in one launch (runner.rs:3824-3838): sum_dst = a + b (sum_dst may be a),
 * norm_dst = rms_norm(sum_dst). */
INFR_API int32_t infr_cuda_add_rms_norm(infr_cuda_ctx *ctx, const infr_cuda_buf *a, const infr_cuda_buf *b, infr_cuda_buf *sum_dst,
                                        const infr_cuda_buf *weight, infr_cuda_buf *norm_dst, uint32_t rows, uint32_t dim, float eps);
/* Op::Rope without freq_factors (cpu lib.rs:1493-1553).  positions: int32 [rows].  neox = 0: pairs (2p, 2p+1). */
INFR_API int32_t infr_cuda_rope(infr_cuda_ctx *ctx, const infr_cuda_buf *x, const infr_cuda_buf *positions, infr_cuda_buf *dst,
                                uint32_t rows, uint32_t n_head, uint32_t head_dim, uint32_t rope_dim, float theta, int32_t neox);
/* Op::WriteKv into an f16 cache [max_ctx, row_stride] (cpu lib.rs:1635-1673): f32 -> f16, round to nearest even. */
INFR_API int32_t infr_cuda_write_kv(infr_cuda_ctx *ctx, const infr_cuda_buf *src, infr_cuda_buf *cache, uint32_t rows,
                                    uint32_t row_stride, uint32_t pos);
typedef struct infr_attn_desc {
    uint32_t rows;      /* query rows per sequence: consecutive positions pos .. pos+rows-1 (causal) */
    uint32_t pos;       /* position of the first query row; it attends keys [0, pos] */
    uint32_t n_head, n_kv, head_dim; /* head_dim 64 or 128; n_head / n_kv in {1, 2, 4, 8} */
    float scale;
    uint32_t n_seq;     /* 0 or 1: the reference's op.  > 1: independent sequences, q holds n_seq * rows rows */
    uint32_t reserved;
    uint64_t seq_stride; /* elements between the caches of consecutive sequences */
} infr_attn_desc;
/* Op::Attention with AttnMask::Causal over f16 K / V caches [max_ctx, n_kv * head_dim] (cpu lib.rs:1744-1888). */
INFR_API int32_t infr_cuda_attention(infr_cuda_ctx *ctx, const infr_attn_desc *desc, const infr_cuda_buf *q,
                                     const infr_cuda_buf *k_cache, const infr_cuda_buf *v_cache, infr_cuda_buf *dst);
/* Sequences at positions of their own (a batch that is served continuously: sequences join and finish at different
 * times).  No counterpart in the reference, whose Op::Attention takes one pos for all rows
 * (crates/infr-llama/src/parallel.rs:9-17 names the per-row KV table as the missing throughput lever).  seq_pos is an
 * int32 device array [n_seq]: the position of sequence s's first query row; desc->pos must be the largest of them (it
 * sizes the launch and the bounds checks; a larger seq_pos[s] is read as desc->pos).  Sequence s attends keys
 * [0, seq_pos[s] + row] of its own cache.  With infr_cuda_rope_write_kv, whose `positions` are per row already, a decode
 * step over sequences of different lengths needs nothing else. */
INFR_API int32_t infr_cuda_attention_seqpos(infr_cuda_ctx *ctx, const infr_attn_desc *desc, const infr_cuda_buf *seq_pos, const infr_cuda_buf *q,
                                            const infr_cuda_buf *k_cache, const infr_cuda_buf *v_cache, infr_cuda_buf *dst);
/* Rope(q) in place, Rope(k) and v straight into the f16 caches: the four ops of runner.rs:3611-3656 in one launch.
 * rope_dim == head_dim.  Row r belongs to sequence r / desc->rows and is written at cache row positions[r]. */
INFR_API int32_t infr_cuda_rope_write_kv(infr_cuda_ctx *ctx, const infr_attn_desc *desc, float theta, int32_t neox, infr_cuda_buf *q,
                                         const infr_cuda_buf *k, const infr_cuda_buf *v, const infr_cuda_buf *positions,
                                         infr_cuda_buf *k_cache, infr_cuda_buf *v_cache);
/* Op::GatedAct with Activation::Silu on dense [rows, nff] gate and up (cpu lib.rs:1890-1944). */
INFR_API int32_t infr_cuda_gated_act(infr_cuda_ctx *ctx, const infr_cuda_buf *gate, const infr_cuda_buf *up, infr_cuda_buf *dst,
                                     uint32_t rows, uint32_t nff);
/* Op::Add (cpu lib.rs:1972-1987). */
INFR_API int32_t infr_cuda_add(infr_cuda_ctx *ctx, const infr_cuda_buf *a, const infr_cuda_buf *b, infr_cuda_buf *dst, uint64_t n);
/* Producers fused with the activation quantiser: the result is written as the int8 codes, per-256 scales and code
 * sums that infr_cuda_quantize_q8 (granularity 256) would produce from the f32 result, bit for bit, ready for
 * infr_cuda_gemv_q8.  The row width (dim, nff, n_head * head_dim) must be a multiple of 256; sums16 may be NULL. */
typedef struct infr_q8_out {
    infr_cuda_buf *qs, *d, *sums, *sums16;
} infr_q8_out;
/* b == NULL: plain RmsNorm of a; else sum_dst = a + b (may be a) and the norm of the sum. */
INFR_API int32_t infr_cuda_add_rms_norm_q8(infr_cuda_ctx *ctx, const infr_cuda_buf *a, const infr_cuda_buf *b, infr_cuda_buf *sum_dst,
                                           const infr_cuda_buf *weight, uint32_t rows, uint32_t dim, float eps, const infr_q8_out *out);
INFR_API int32_t infr_cuda_gated_act_q8(infr_cuda_ctx *ctx, const infr_cuda_buf *gate, const infr_cuda_buf *up, uint32_t rows, uint32_t nff,
                                        const infr_q8_out *out);
/* The exchange of a row-parallel Linear with no kernel of its own (no counterpart in the reference, which has no
 * multi-GPU path; the reference's tensor-parallel sketch sums after the row-parallel Linears,
 * crates/infr-vulkan/src/tp_allreduce.rs:320).  infr_cuda_gemv_q8_push is infr_cuda_gemv_q8 (Q4_K rows of whole
 * blocks, or Q6_K rows of whole 2048-element chunks with sums16; m <= 8, or m <= 32 where infr_cuda_gemv_q8 takes that
 * many rows) whose epilogue stores the rank's partial [m, out_f] result into every rank's staging over NVLink peer
 * mappings instead of a buffer, each value in one 8-byte word with the exchange's sequence number (no fence, no flag);
 * infr_cuda_add_rms_norm_q8_pull is infr_cuda_add_rms_norm_q8 with b = the sum of all ranks' pushed results (polls,
 * bounded, the words it adds; sums in rank order from zero, so the result has the bits of infr_cuda_gemv_q8 +
 * infr_cuda_all_reduce_f32 + infr_cuda_add_rms_norm_q8).  The two calls come in pairs on one comm, in the same order on
 * every rank, m * out_f == rows * dim <= min(the comm's max_floats, 262144); other exchanges of the comm may come
 * between pairs, not inside one.  A rank that never pushes makes the poll run out: the row keeps `a` alone and the next
 * sync returns INFR_E_TIMEOUT. */
INFR_API int32_t infr_cuda_gemv_q8_push(infr_cuda_ctx *ctx, infr_cuda_comm *comm, int32_t dtype, const infr_cuda_buf *w, uint64_t w_off,
                                        const infr_cuda_buf *qs, const infr_cuda_buf *d, const infr_cuda_buf *sums, const infr_cuda_buf *sums16,
                                        uint32_t m, uint32_t in_f, uint32_t out_f);
INFR_API int32_t infr_cuda_add_rms_norm_q8_pull(infr_cuda_ctx *ctx, infr_cuda_comm *comm, const infr_cuda_buf *a, infr_cuda_buf *sum_dst,
                                                const infr_cuda_buf *weight, uint32_t rows, uint32_t dim, float eps, const infr_q8_out *out);
INFR_API int32_t infr_cuda_attention_q8(infr_cuda_ctx *ctx, const infr_attn_desc *desc, const infr_cuda_buf *q, const infr_cuda_buf *k_cache,
                                        const infr_cuda_buf *v_cache, const infr_q8_out *out);
INFR_API int32_t infr_cuda_attention_seqpos_q8(infr_cuda_ctx *ctx, const infr_attn_desc *desc, const infr_cuda_buf *seq_pos, const infr_cuda_buf *q,
                                               const infr_cuda_buf *k_cache, const infr_cuda_buf *v_cache, const infr_q8_out *out);
/* Paged caches (the per-row KV block table that crates/infr-llama/src/parallel.rs:9-17 names; no counterpart in the
 * reference): k_pool / v_pool hold n_pages pages of 128 rows [n_pages][128][n_kv * head_dim] f16 shared by all sequences,
 * block_table is an int32 device array [n_seq][table_stride] whose entry (s, i) is the page with rows 128 i .. 128 i + 127
 * of sequence s (an entry outside [0, n_pages) is read as the nearest valid page: a wrong table gives wrong numbers, not a
 * fault).  table_stride >= (desc->pos + desc->rows + 127) / 128; desc->seq_stride is ignored; seq_pos may be NULL (every
 * sequence at desc->pos).  attention_paged writes f32 rows to dst or, with dst NULL, the int8 form to out (exactly one).
 * rope_write_kv_paged is infr_cuda_rope_write_kv with row r of sequence s stored at page table[s][positions[r] / 128]. */
INFR_API int32_t infr_cuda_attention_paged(infr_cuda_ctx *ctx, const infr_attn_desc *desc, const infr_cuda_buf *seq_pos, const infr_cuda_buf *block_table,
                                           uint32_t table_stride, uint32_t n_pages, const infr_cuda_buf *q, const infr_cuda_buf *k_pool,
                                           const infr_cuda_buf *v_pool, infr_cuda_buf *dst, const infr_q8_out *out);
INFR_API int32_t infr_cuda_rope_write_kv_paged(infr_cuda_ctx *ctx, const infr_attn_desc *desc, float theta, int32_t neox, infr_cuda_buf *q,
                                               const infr_cuda_buf *k, const infr_cuda_buf *v, const infr_cuda_buf *positions,
                                               const infr_cuda_buf *block_table, uint32_t table_stride, uint32_t n_pages, infr_cuda_buf *k_pool,
                                               infr_cuda_buf *v_pool);
/* Op::Argmax (cpu lib.rs:2167-2187): dst uint32 [rows], lowest index on ties. */
INFR_API int32_t infr_cuda_argmax(infr_cuda_ctx *ctx, const infr_cuda_buf *x, infr_cuda_buf *dst, uint32_t n, uint32_t rows);

/* ---- stream capture and timing ----
 * capture_begin .. capture_end records every kernel the calls in between enqueue into a CUDA graph
 * that infr_cuda_graph_launch replays (decode replays a fixed kernel sequence every token).  Calls
 * that allocate or synchronise are rejected while capturing. */
INFR_API int32_t infr_cuda_capture_begin(infr_cuda_ctx *ctx);
INFR_API int32_t infr_cuda_capture_end(infr_cuda_ctx *ctx, infr_cuda_graph **out);
INFR_API int32_t infr_cuda_graph_launch(infr_cuda_ctx *ctx, infr_cuda_graph *graph);
INFR_API void infr_cuda_graph_free(infr_cuda_ctx *ctx, infr_cuda_graph *graph);
/* CUDA-event stopwatch on the context's stream: stop synchronises and returns milliseconds. */
INFR_API int32_t infr_cuda_timer_start(infr_cuda_ctx *ctx);
INFR_API int32_t infr_cuda_timer_stop(infr_cuda_ctx *ctx, float *ms);
/* Overwrites a context-owned buffer larger than L2 (evicts cached weights between timed runs). */
INFR_API int32_t infr_cuda_flush_l2(infr_cuda_ctx *ctx);
/* No counterpart in the reference: the device's dense int8 tensor-core rate, measured, as the denominator of the
 * prefill GEMM's roofline.  Runs `launches` launches of a kernel in which every SM issues 2 x n_batches x 64
 * tcgen05 kind::i8 instructions of shape 128 x 256 x 32 on operands resident in shared memory (no unpacking, no
 * epilogue), timed with CUDA events on the context's stream; *ms is the time, *int8_ops the operations (2 per
 * multiply-add) it covered.  One accumulator element per issuing thread is checked against the value the operand
 * pattern implies; a mismatch is INFR_E_CUDA.  n_batches 1..4096, launches 1..100000. */
INFR_API int32_t infr_cuda_tensor_peak_i8(infr_cuda_ctx *ctx, uint32_t n_batches, uint32_t launches, float *ms, double *int8_ops);
/* Number of kernels this context has launched since creation (graph replays count their nodes). */
INFR_API uint64_t infr_cuda_launch_count(infr_cuda_ctx *ctx);

/* ---- GGUF container: the weight file on the input side of the hot path ------------------------------------------
 * Replaces, for one file, Gguf::open / tensor_bytes / tensor_file_range and the Metadata getters of
 * crates/infr-gguf/src/lib.rs:82-145, :476, :893-930 (a gguf-split shard set is not read).  The file is mapped
 * read-only; tensor data is a pointer into the mapping, valid until infr_gguf_close, and goes to the device with
 * infr_cuda_upload_at (q / k / v back to back in one buffer give the `w_off` slices of a fused-QKV Linear,
 * crates/infr-llama/src/seam/runner.rs:3445-3461).  These entry points need no GPU.
 * Errors as in the reference's open (lib.rs:735-870): not GGUF, version other than 2 / 3, reads past the end, nesting
 * deeper than 64, general.alignment not a power of two or above 1 MiB, more than 8 dimensions, shape or byte-size
 * overflow, a quantised tensor that is not a whole number of blocks, data outside the file: INFR_E_INVALID
 * (Error::Loader) with a message in `err`; an unknown ggml type: INFR_E_UNSUPPORTED (Error::Unsupported). */
typedef struct infr_gguf infr_gguf;
typedef struct {
    const char *name;   /* NUL-terminated, owned by the infr_gguf */
    uint32_t ggml_type; /* the file's type code (12 = Q4_K, 14 = Q6_K, 42 = Q2_0, 0 = F32, 1 = F16, ...) */
    int32_t dtype;      /* the INFR_DT_* code this library runs the type under, or -1 */
    uint32_t n_dims;
    uint64_t dims[8];   /* dims[0] is the fastest-varying axis (the columns of a weight); unused entries are 1 */
    uint64_t numel, nbytes, file_offset;
} infr_gguf_tensor;
INFR_API int32_t infr_gguf_open(const char *path, infr_gguf **out, char *err, size_t err_len);
INFR_API void infr_gguf_close(infr_gguf *g);
INFR_API uint32_t infr_gguf_version(const infr_gguf *g);
INFR_API uint64_t infr_gguf_alignment(const infr_gguf *g);
INFR_API uint64_t infr_gguf_tensor_count(const infr_gguf *g);
INFR_API int32_t infr_gguf_tensor_at(const infr_gguf *g, uint64_t index, infr_gguf_tensor *out);
INFR_API int32_t infr_gguf_find(const infr_gguf *g, const char *name, infr_gguf_tensor *out);
INFR_API const void *infr_gguf_tensor_data(const infr_gguf *g, const infr_gguf_tensor *t);
/* Metadata.  Value type codes are the file's: 0 u8, 1 i8, 2 u16, 3 i16, 4 u32, 5 i32, 6 f32, 7 bool, 8 string,
 * 9 array, 10 u64, 11 i64, 12 f64; infr_gguf_meta_type returns -1 for an absent key.  _u64 takes any non-negative
 * integer or bool, _f64 any number; a string is a pointer into the mapping and a length (not NUL-terminated); an
 * array gives its element type and count and, for fixed-size element types, its packed elements. */
INFR_API uint64_t infr_gguf_meta_count(const infr_gguf *g);
INFR_API const char *infr_gguf_meta_key(const infr_gguf *g, uint64_t index);
INFR_API int32_t infr_gguf_meta_type(const infr_gguf *g, const char *key);
INFR_API int32_t infr_gguf_meta_u64(const infr_gguf *g, const char *key, uint64_t *out);
INFR_API int32_t infr_gguf_meta_f64(const infr_gguf *g, const char *key, double *out);
INFR_API int32_t infr_gguf_meta_str(const infr_gguf *g, const char *key, const char **s, uint64_t *len);
INFR_API int32_t infr_gguf_meta_array(const infr_gguf *g, const char *key, uint32_t *elem_type, uint64_t *count, const void **data);

#ifdef __cplusplus
}
#endif
#endif /* INFR_CUDA_H */
