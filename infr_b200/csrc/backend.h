// Host side of the CUDA backend: a C++ mirror of the reference's `trait Backend`
// (crates/infr-core/src/backend.rs:486-662) with the same method names, argument meaning and error
// behaviour (errors are returned, never thrown across the C ABI; bad sizes are errors, not panics —
// `check_copy_bytes`, backend.rs:23-30).  The C ABI in c_api.cpp is a thin shell over this class.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/infr_cuda.h"
#include "kernels.h"

// Opaque handles of the C ABI.
struct infr_cuda_buf {
    void *ptr = nullptr;
    size_t len = 0;  // logical size in bytes (Buffer::len_bytes, backend.rs:387-398)
    int usage = 0;
    uint64_t uid = 0;  // never reused: derived-data caches key on this, not on the address
    bool owned = true;  // false: the memory belongs to the caller (infr_cuda_wrap), free drops only the handle
};

struct infr_cuda_comm;  // comm.cu

// One launch group of a compiled plan: a single op, or neighbouring ops one kernel computes.
struct PlanStep {
    enum Kind { kSingle = 0, kAddRmsNorm = 1, kRopeWriteKv = 2, kLinearPair = 3 };
    int kind;
    uint32_t op0, n_ops;
};

struct infr_cuda_plan {
    std::vector<infr_tensor_decl> tensors;
    std::vector<infr_op_desc> ops;
    std::vector<PlanStep> steps;
    std::vector<void *> internal;  // device scratch of every Internal handle (null for the others), from the context's pool
    std::vector<size_t> internal_bytes;
    std::vector<char> needs_zero;  // the handle's zero fill is observable (read, or partly written, before a full overwrite)
    // The launch sequence of an execute kept as a CUDA graph: replayed while the bound buffers, the context scratch and
    // the kernel options are the ones it was captured with (a plan run again on the same buffers, as a decode loop or
    // a serving step does, then costs one graph launch on the host instead of one launch per op).
    struct infr_cuda_graph *cached = nullptr;
    std::vector<uint64_t> cached_key, last_key;
    bool no_graph = false;  // a capture of this plan failed once: it runs op by op from then on
};

struct infr_cuda_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernel_nodes = 0;
};

namespace infr {

struct Status {
    int32_t code = INFR_OK;
    std::string msg;
    bool ok() const { return code == INFR_OK; }
    static Status Ok() { return {}; }
    static Status Err(int32_t c, std::string m) { return {c, std::move(m)}; }
};

// Raw device view of an activation / weight operand (a buffer handle plus a byte offset).
struct DevSpan {
    uint8_t *ptr;
    size_t bytes;
};

class CudaBackend {
public:
    static Status create(const infr_cuda_opts &opts, CudaBackend **out);
    ~CudaBackend();

    const char *name() const { return "cuda-sm100a"; }
    infr_cuda_caps capabilities() const;

    // ---- memory ----
    Status alloc(size_t bytes, int usage, bool zero, infr_cuda_buf **out);
    void free_buffer(infr_cuda_buf *b);
    // A handle over device memory the caller owns (another engine's pool, a framework tensor): nothing is
    // allocated or copied, free_buffer drops the handle only.
    Status wrap(void *device_ptr, size_t bytes, int usage, infr_cuda_buf **out);
    // Small-message all-reduce over peer memory of the GPUs of one box (comm.cu).
    Status comm_create(int rank, int world, uint32_t max_floats, infr_cuda_comm **out);
    Status comm_export(infr_cuda_comm *c, uint8_t *handle64);
    Status comm_connect(infr_cuda_comm *c, const uint8_t *handles);
    Status comm_connect_silent(infr_cuda_comm *c, uint32_t spin_limit);
    Status all_reduce_f32(infr_cuda_comm *c, float *data, uint32_t n);
    // the exchange without a kernel of its own: pushed by the GEMV's epilogue, summed by the norm that follows
    Status gemv_q8_push(infr_cuda_comm *c, int dtype, const uint8_t *w, const Q8Dev &a, uint32_t m, uint32_t in_f, uint32_t out_f);
    Status rms_norm_q8_pull(infr_cuda_comm *c, const float *a, float *sum_dst, const float *w, uint32_t rows, uint32_t dim, float eps, const Q8Dev &out);
    void comm_destroy(infr_cuda_comm *c);
    Status upload(infr_cuda_buf *dst, size_t dst_off, const void *src, size_t bytes);
    Status download(const infr_cuda_buf *src, void *dst, size_t bytes);
    Status copy_buffer(const infr_cuda_buf *src, infr_cuda_buf *dst, size_t bytes);
    Status sync();

    // ---- graphs ----
    Status compile(const infr_graph_desc &g, infr_cuda_plan **out);
    void free_plan(infr_cuda_plan *p);
    Status execute(infr_cuda_plan *plan, infr_cuda_buf *const *bindings, uint32_t n);

    // ---- ops (device pointers already validated by the callers above / the C ABI) ----
    Status quantize_q8(int gran, const float *x, uint32_t rows, uint32_t k, int8_t *qs, float *d,
                       int32_t *sums, int32_t *sums16, uint16_t *dact, uint16_t *sact);
    Status linear(int dtype, const uint8_t *w, const float *x, float *y, uint32_t m, uint32_t in_f,
                  uint32_t out_f, int act);
    // Two Linears of one weight format on the same rows (q and k, gate and up): the rows are quantised once, and laid
    // out once for the tensor-memory GEMM; results are those of two `linear` calls.
    Status linear_pair(int dtype, const uint8_t *w1, float *y1, uint32_t out_f1, const uint8_t *w2, float *y2, uint32_t out_f2, const float *x,
                       uint32_t m, uint32_t in_f, int act);
    // Op::MoeFfn (crates/infr-cpu/src/lib.rs:2264-2984), qwen3moe configuration.  Optional debug outputs:
    // sel_ids [rows,n_used] i32, sel_w [rows,n_used] f32, logits [rows,n_expert] f32 (null = not wanted).
    struct MoeArgs {
        const float *x, *router_x, *router;
        const uint8_t *gate, *up, *down;
        int gate_dt, up_dt, down_dt;
        float *dst;
        uint32_t rows, ne, n_expert, n_used, n_ff;
        float scale;
        int norm_w;
        int32_t *sel_ids;
        float *sel_w, *logits;
        uint32_t expert_lo, n_local;  // the banks hold experts [expert_lo, expert_lo + n_local)
    };
    Status moe_ffn(const MoeArgs &a);
    Status moe_ffn_f32(const MoeArgs &a);
    Status gemv_q8(int dtype, const uint8_t *w, const Q8Dev &a, float *y, uint32_t m, uint32_t in_f, uint32_t out_f);
    // Two weights of one format against the same quantised rows: one launch where the format's kernel can (Q4_K).
    Status gemv_q8_pair(int dtype, const uint8_t *w1, float *y1, uint32_t out_f1, const uint8_t *w2, float *y2, uint32_t out_f2, const Q8Dev &a,
                        uint32_t m, uint32_t in_f);
    // ---- the other ops of a dense decode step (decode_ops.cu); arguments checked by the C ABI ----
    Status rms_norm(const float *a, const float *b, float *sum_dst, const float *w, float *dst, uint32_t rows, uint32_t dim, float eps);
    Status rope(const float *x, const int32_t *positions, float *dst, uint32_t rows, uint32_t n_head, uint32_t head_dim, uint32_t rope_dim,
                float theta, int neox);
    Status write_kv(const float *src, void *cache_at_pos, size_t n);
    // write_pos >= 0: cache row = write_pos + row (Op::WriteKv's `pos`); < 0: the row's own position
    Status rope_write_kv(const infr_attn_desc &d, float theta, int neox, float *q, const float *k, const float *v, const int32_t *positions,
                         void *k_cache, void *v_cache, int write_pos = -1,
                         const int32_t *block_table = nullptr, uint32_t table_stride = 0, uint32_t n_pages = 0);
    // seq_pos: optional device array of per-sequence positions (d.pos is then their maximum)
    // block_table: optional paged caches (int32 [n_seq][table_stride] on the device; k_cache / v_cache are then pools of n_pages pages)
    Status attention(const infr_attn_desc &d, const float *q, const void *k_cache, const void *v_cache, float *dst, const Q8Dev *q8 = nullptr,
                     const int32_t *seq_pos = nullptr, const int32_t *block_table = nullptr, uint32_t table_stride = 0, uint32_t n_pages = 0);
    Status rms_norm_q8(const float *a, const float *b, float *sum_dst, const float *w, uint32_t rows, uint32_t dim, float eps, const Q8Dev &q8);
    Status gated_act_q8(const float *gate, const float *up, uint32_t rows, uint32_t nff, const Q8Dev &q8);
    Status gated_act(const float *gate, const float *up, float *dst, size_t n);
    Status add(const float *a, const float *b, float *dst, size_t n);
    Status argmax(const float *x, uint32_t *dst, uint32_t n, uint32_t rows);
    Status gemv_block_acc(int dtype, const uint8_t *w, const float *x, int32_t *acc, uint32_t in_f,
                          uint32_t out_f);

    // ---- capture / timing ----
    Status capture_begin();
    Status capture_end(infr_cuda_graph **out);
    Status graph_launch(infr_cuda_graph *g);
    void graph_free(infr_cuda_graph *g);
    Status timer_start();
    Status timer_stop(float *ms);
    Status flush_l2();
    // Measures the dense int8 tensor-core rate: `launches` launches of the microbenchmark kernel, CUDA-event timed.
    Status tensor_peak_i8(uint32_t n_batches, uint32_t launches, float *ms, double *ops);
    uint64_t launch_count() const { return launches_; }

    std::mutex &mutex() { return mu_; }
    void set_error(const Status &s) { last_error_ = s.msg; }
    const std::string &last_error() const { return last_error_; }
    bool reference() const { return reference_; }
    cudaStream_t stream() const { return stream_; }
    const DeviceInfo &device_info() const { return dev_; }
    Status cuda_status(cudaError_t e, const char *what);
    // Grows the context's activation scratch; refused while capturing.
    Status ensure_scratch(size_t bytes);
    uint8_t *scratch() const { return static_cast<uint8_t *>(scratch_); }
    void count_launches(uint64_t n) { launches_ += n; }
    Status execute_steps(infr_cuda_plan *plan, infr_cuda_buf *const *bindings, uint32_t n);

private:
    CudaBackend() = default;
    // Quantises `rows` activation rows into the context scratch; `extra` more bytes are reserved behind them.
    Status quantize_for(int dtype, const float *x, uint32_t rows, uint32_t k, Q8Dev *out, size_t extra = 0,
                        uint8_t **extra_ptr = nullptr);

    int device_ = 0;
    bool reference_ = false;
    cudaStream_t stream_ = nullptr;
    cudaDeviceProp prop_{};
    DeviceInfo dev_{};
    std::mutex mu_;
    std::string last_error_;
    void *scratch_ = nullptr;
    uint64_t scratch_gen_ = 0;  // counts reallocations of the scratch: graphs captured before one hold stale pointers
    size_t scratch_bytes_ = 0;
    void *flush_ = nullptr;
    size_t flush_bytes_ = 0;
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
    bool capturing_ = false;
    uint64_t launches_ = 0;
    uint64_t next_uid_ = 1;
    uint32_t *status_host_ = nullptr;  // pinned + mapped: kernels report expired waits here
    uint32_t *status_dev_ = nullptr;
    // small uploads go through a ring of pinned slots, so that upload() can return without a stream sync
    static constexpr int kUpSlots = 8;
    static constexpr size_t kUpSlotBytes = 64 << 10;
    uint8_t *up_ring_ = nullptr;
    cudaEvent_t up_ev_[kUpSlots] = {};
    int up_next_ = 0;
    int gemv_impl_ = 0;                // 0 = bulk-copy ring kernel, 1 = direct-load kernel
    int mmq_impl_ = 0;                 // 0 = warp-specialised MMQ (f32 within rounding of the CPU), 1 = bit-identical MMQ
    Status check_device_status();
    // Batches of 9..32 rows (Q4_K) / any batch above 8 rows (Q6_K) through the wide GEMV, 32 rows per pass.
    bool wide_applies(int dtype, uint32_t m, uint32_t in_f, int act) const;
    Status wide_gemm(int dtype, const uint8_t *w, const Q8Dev &a, float *y, uint32_t m, uint32_t in_f, uint32_t out_f, float *partials,
                     const uint8_t *w2 = nullptr, float *y2 = nullptr, uint32_t out_f2 = 0);
    Status mmq_linear(const uint8_t *w, const float *x, float *y, uint32_t m, uint32_t in_f, uint32_t out_f, bool reuse);
    // Device blocks behind the Internal handles of compiled plans; a freed plan's blocks are reused by the next
    // compile (the reference rebuilds its graph every step, so compile must not cost an allocation each time).
    struct PoolBlock {
        void *ptr;
        size_t bytes;
        bool in_use;
    };
    std::vector<PoolBlock> pool_;
    Status pool_acquire(size_t bytes, void **out);
    void pool_release(void *p);
};

}  // namespace infr

struct infr_cuda_ctx {
    infr::CudaBackend *be;
};
