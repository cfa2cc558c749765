// Backend::compile / Backend::execute (crates/infr-core/src/backend.rs:561-562): the ordered op list of a `Graph`
// (crates/infr-core/src/graph.rs:8-14, 138-1074) walked on the context's stream.
//
// compile checks every op against what this backend runs (anything else is Error::Unsupported at compile time, so a
// caller finds out before it has uploaded a model), takes the scratch of the Internal handles from the context's pool
// and groups neighbouring ops that one launch can do:
//   Add, RmsNorm                      -> the residual add fused in front of the norm
//                                        (runner.rs:3824-3838 emits exactly this pair between the two halves of a layer)
//   Linear, Linear (same rows, same format) -> rows quantised once, one launch for a decode batch of Q4_K
//                                        (runner.rs:3476-3523 q/k/v, :3882-3933 gate/up)
//   Rope(k), Rope(q), WriteKv, WriteKv -> q rotated in place, k rotated and v cast straight into the f16 caches
//                                        (runner.rs:3611-3656), when the rotated k has no other reader
// The grouped norm and rope launches compute the same values with the same roundings as the separate ops (the kernels
// are the same templates); a pair of Linears has the separate ops' integer block sums and may add its f32 partial sums
// in a different order (K is split over a different number of warps).
// execute follows the provisioning contract of crates/infr-core/src/exec.rs:53-139: Internal handles are backend
// scratch that reads as zero until an op writes it, Inputs / Weights / Outputs are the caller's bound buffers,
// KV-cache Inputs are written in place, and every Output is in its bound buffer when the stream reaches the caller's
// download or sync.
#include <cstdarg>
#include <cstdio>

#include "backend.h"

namespace infr {
namespace {

std::string pfmt(const char *f, ...) __attribute__((format(printf, 1, 2)));
std::string pfmt(const char *f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof buf, f, ap);
    va_end(ap);
    return buf;
}
size_t up256(size_t v) { return (v + 255) / 256 * 256; }

size_t tensor_bytes(const infr_tensor_decl &t) {
    const int be = block_elems((int)t.dtype), bb = block_bytes((int)t.dtype);
    if (t.dtype == DT_I32) return (size_t)t.numel * 4;
    if (!bb) return 0;
    return (size_t)(t.numel / (uint64_t)be) * (size_t)bb;
}

// Number of tensor slots an op tag uses (the leading entries of infr_op_desc::t), or -1 for an unknown tag.
int op_tensors(uint32_t tag) {
    switch (tag) {
    case INFR_OP_LINEAR: return 3;
    case INFR_OP_MOE_FFN: return 7;
    case INFR_OP_RMS_NORM: return 3;
    case INFR_OP_ROPE: return 3;
    case INFR_OP_WRITE_KV: return 2;
    case INFR_OP_ATTENTION: return 4;
    case INFR_OP_GATED_ACT: return 3;
    case INFR_OP_ADD: return 3;
    case INFR_OP_ARGMAX: return 2;
    case INFR_OP_COPY: return 2;
    default: return -1;
    }
}

// Index (into t[]) of the tensor an op writes in full, and the number of elements it writes there; -1 when the op
// writes only part of its destination (WriteKv, Copy) — such a destination keeps needing its zero fill.
int op_full_dst(const infr_op_desc &op, uint64_t *numel) {
    switch (op.tag) {
    case INFR_OP_LINEAR: *numel = (uint64_t)op.u[0] * op.u[2]; return 2;
    case INFR_OP_RMS_NORM: *numel = (uint64_t)op.u[0] * op.u[1]; return 2;
    case INFR_OP_ROPE: *numel = (uint64_t)op.u[0] * op.u[1] * op.u[2]; return 2;
    case INFR_OP_ATTENTION: *numel = (uint64_t)op.u[0] * op.u[2] * op.u[4]; return 3;
    case INFR_OP_GATED_ACT: *numel = (uint64_t)op.u[0] * op.u[1]; return 2;
    case INFR_OP_ADD: *numel = op.u[0]; return 2;
    case INFR_OP_ARGMAX: *numel = op.u[1]; return 1;
    default: return -1;
    }
}

bool op_reads(const infr_op_desc &op, uint32_t id) {
    const int nt = op_tensors(op.tag);
    uint64_t dummy;
    const int dst = op_full_dst(op, &dummy);
    for (int k = 0; k < nt; k++) {
        if (op.t[k] != id) continue;
        if (k == dst) continue;  // pure destination
        if (op.tag == INFR_OP_MOE_FFN && k == 6) continue;
        if ((op.tag == INFR_OP_WRITE_KV || op.tag == INFR_OP_COPY) && k == 1) continue;
        return true;
    }
    return false;
}

}  // namespace

Status CudaBackend::pool_acquire(size_t bytes, void **out) {
    // best fit among the free blocks that are not wastefully large
    int best = -1;
    for (size_t i = 0; i < pool_.size(); i++)
        if (!pool_[i].in_use && pool_[i].bytes >= bytes && pool_[i].bytes <= 2 * bytes + 4096 &&
            (best < 0 || pool_[i].bytes < pool_[(size_t)best].bytes))
            best = (int)i;
    if (best >= 0) {
        pool_[(size_t)best].in_use = true;
        *out = pool_[(size_t)best].ptr;
        return Status::Ok();
    }
    if (capturing_) return Status::Err(INFR_E_INVALID, "compile would allocate plan scratch during stream capture");
    void *p = nullptr;
    Status s = cuda_status(cudaMalloc(&p, bytes), "plan scratch cudaMalloc");
    if (!s.ok()) return s;
    pool_.push_back(PoolBlock{p, bytes, true});
    *out = p;
    return Status::Ok();
}

void CudaBackend::pool_release(void *p) {
    for (auto &b : pool_)
        if (b.ptr == p) b.in_use = false;
}

Status CudaBackend::compile(const infr_graph_desc &g, infr_cuda_plan **out) {
    if ((g.n_tensors && !g.tensors) || (g.n_ops && !g.ops)) return Status::Err(INFR_E_INVALID, "compile: null graph arrays");
    auto plan = new infr_cuda_plan();
    plan->tensors.assign(g.tensors, g.tensors + g.n_tensors);
    plan->ops.assign(g.ops, g.ops + g.n_ops);
    plan->internal.assign(g.n_tensors, nullptr);
    plan->internal_bytes.assign(g.n_tensors, 0);
    plan->needs_zero.assign(g.n_tensors, 0);
    auto fail = [&](Status s) {
        free_plan(plan);
        return s;
    };
    auto unsupported = [&](uint32_t i, const char *what) {
        return fail(Status::Err(INFR_E_UNSUPPORTED, pfmt("compile: op %u: %s", i, what)));
    };
    auto dt = [&](uint32_t id) { return g.tensors[id].dtype; };
    for (uint32_t i = 0; i < g.n_ops; i++) {
        const infr_op_desc &op = g.ops[i];
        const int nt = op_tensors(op.tag);
        if (nt < 0) return unsupported(i, pfmt("tag %u is not an op this backend runs", op.tag).c_str());
        for (int k = 0; k < nt; k++)
            if (op.t[k] >= g.n_tensors) return fail(Status::Err(INFR_E_INVALID, pfmt("compile: op %u names tensor %u of %u", i, op.t[k], g.n_tensors)));
        switch (op.tag) {
        case INFR_OP_LINEAR: {
            const uint32_t in_f = op.u[1], w_off = op.u[3];
            const infr_tensor_decl &w = g.tensors[op.t[1]];
            if (w.dtype != DT_Q4K && w.dtype != DT_Q6K && w.dtype != DT_Q2_0) return unsupported(i, pfmt("Linear weight dtype code %u", w.dtype).c_str());
            if (in_f == 0 || w_off % in_f) return fail(Status::Err(INFR_E_INVALID, pfmt("compile: Linear w_off=%u is not row-aligned (in_f=%u)", w_off, in_f)));
            if ((uint64_t)w_off + (uint64_t)op.u[2] * in_f > w.numel)
                return fail(Status::Err(INFR_E_INVALID, pfmt("compile: Linear rows [%u,+%u) leave the %llu-element weight", w_off / in_f, op.u[2], (unsigned long long)w.numel)));
            break;
        }
        case INFR_OP_MOE_FFN:
            // u = {ne, n_expert, n_used, n_ff_exp, norm_w, fused_gate_up, weight_before, act, gating}
            if (op.u[5] || op.u[6] || op.u[7] || op.u[8]) return unsupported(i, "MoeFfn with fused gate/up, weight_before, a non-SiLU activation or non-softmax gating");
            if (dt(op.t[2]) != DT_F32) return unsupported(i, "MoeFfn router weights must be F32");
            for (int k = 3; k <= 5; k++)
                if (dt(op.t[k]) != DT_Q4K && dt(op.t[k]) != DT_Q6K) return unsupported(i, "MoeFfn expert banks must be Q4_K or Q6_K");
            break;
        case INFR_OP_RMS_NORM:
            if (op.u[0] == 0 || op.u[1] == 0) return fail(Status::Err(INFR_E_INVALID, pfmt("compile: op %u: RmsNorm of %u rows x %u", i, op.u[0], op.u[1])));
            if (dt(op.t[0]) != DT_F32 || dt(op.t[1]) != DT_F32 || dt(op.t[2]) != DT_F32) return unsupported(i, "RmsNorm on non-f32 tensors");
            break;
        case INFR_OP_ROPE:
            // u = {rows, n_head, head_dim, rope_dim, x_stride, neox, backward, has_freq_factors}
            if (op.u[7]) return unsupported(i, "Rope with freq_factors");
            if (op.u[6]) return unsupported(i, "Rope backward");
            if (op.u[4] && op.u[4] != op.u[1] * op.u[2]) return unsupported(i, "Rope with a row stride");
            if (op.u[0] == 0 || op.u[1] == 0 || op.u[2] == 0 || op.u[3] == 0 || op.u[3] > op.u[2] || (op.u[3] & 1))
                return fail(Status::Err(INFR_E_INVALID, pfmt("compile: op %u: Rope needs positive sizes and an even rope_dim <= head_dim", i)));
            if (dt(op.t[1]) != DT_I32) return unsupported(i, "Rope positions must be I32");
            break;
        case INFR_OP_WRITE_KV:
            if (dt(op.t[1]) != DT_F16) return unsupported(i, "WriteKv into a cache that is not F16");
            if (op.u[0] == 0 || op.u[1] == 0) return fail(Status::Err(INFR_E_INVALID, pfmt("compile: op %u: WriteKv of %u rows x %u", i, op.u[0], op.u[1])));
            break;
        case INFR_OP_ATTENTION: {
            // u = {rows, kv_len, n_head, n_kv, head_dim, mask, pos, has_sinks}
            if (op.u[5] != 0) return unsupported(i, "Attention with a mask other than Causal");
            if (op.u[7]) return unsupported(i, "Attention with sinks");
            if (dt(op.t[1]) != DT_F16 || dt(op.t[2]) != DT_F16) return unsupported(i, "Attention over caches that are not F16");
            if (op.u[1] != op.u[6] + op.u[0]) return unsupported(i, "Attention whose kv_len is not pos + rows");
            const uint32_t nh = op.u[2], nkv = op.u[3], hd = op.u[4];
            if (op.u[0] == 0 || nh == 0 || nkv == 0 || nh % nkv) return fail(Status::Err(INFR_E_INVALID, pfmt("compile: op %u: Attention head counts", i)));
            const uint32_t grp = nh / nkv;
            if ((hd != 64 && hd != 128) || (grp != 1 && grp != 2 && grp != 4 && grp != 8)) return unsupported(i, "Attention: head_dim 64 or 128, n_head / n_kv in {1, 2, 4, 8}");
            break;
        }
        case INFR_OP_GATED_ACT:
            // u = {rows, nff, act, up_off, up_stride, gate_stride, gate_block_width, has_clamp}
            if (op.u[2] != 0) return unsupported(i, "GatedAct with an activation other than SiLU");
            if (op.u[3] || (op.u[4] && op.u[4] != op.u[1]) || (op.u[5] && op.u[5] != op.u[1]) || op.u[6]) return unsupported(i, "GatedAct on strided or interleaved buffers");
            if (op.u[7]) return unsupported(i, "GatedAct with a clamp");
            break;
        case INFR_OP_ADD:
        case INFR_OP_ARGMAX:
        case INFR_OP_COPY: break;
        }
    }
    // ---- fusion groups ----
    for (uint32_t i = 0; i < g.n_ops;) {
        const infr_op_desc &a = g.ops[i];
        PlanStep st{PlanStep::kSingle, i, 1};
        if (a.tag == INFR_OP_ADD && i + 1 < g.n_ops) {
            const infr_op_desc &n = g.ops[i + 1];
            // norm of the sum just written; the norm's destination is a different tensor
            if (n.tag == INFR_OP_RMS_NORM && n.t[0] == a.t[2] && (uint64_t)n.u[0] * n.u[1] == a.u[0] && n.t[2] != a.t[2] && n.t[2] != a.t[0] &&
                n.t[2] != a.t[1])
                st = PlanStep{PlanStep::kAddRmsNorm, i, 2};
        }
        if (a.tag == INFR_OP_LINEAR && i + 1 < g.n_ops) {
            // two Linears of one weight format reading the same rows (q and k, gate and up): quantised once
            const infr_op_desc &n = g.ops[i + 1];
            if (n.tag == INFR_OP_LINEAR && n.t[0] == a.t[0] && n.u[0] == a.u[0] && n.u[1] == a.u[1] &&
                plan->tensors[n.t[1]].dtype == plan->tensors[a.t[1]].dtype && n.t[2] != a.t[2] && a.t[2] != a.t[0] && n.t[2] != a.t[0])
                st = PlanStep{PlanStep::kLinearPair, i, 2};
        }
        if (a.tag == INFR_OP_ROPE && i + 3 < g.n_ops) {
            const infr_op_desc &rq = g.ops[i + 1], &wk = g.ops[i + 2], &wv = g.ops[i + 3];
            bool ok = rq.tag == INFR_OP_ROPE && wk.tag == INFR_OP_WRITE_KV && wv.tag == INFR_OP_WRITE_KV;
            ok = ok && a.t[0] != a.t[2] && rq.t[0] == rq.t[2];                       // k -> k16, q in place
            ok = ok && a.t[1] == rq.t[1] && a.u[0] == rq.u[0];                       // same positions, same rows
            ok = ok && a.u[2] == rq.u[2] && a.u[3] == a.u[2] && rq.u[3] == rq.u[2];  // whole heads rotated, same head_dim
            ok = ok && a.u[5] == rq.u[5] && a.f[0] == rq.f[0];                       // same pairing and base
            ok = ok && wk.t[0] == a.t[2] && wk.u[0] == a.u[0] && wv.u[0] == a.u[0];  // the rotated k is what WriteKv stores
            ok = ok && wk.u[1] == a.u[1] * a.u[2] && wv.u[1] == wk.u[1] && wk.u[2] == wv.u[2] && wk.t[1] != wv.t[1];
            ok = ok && plan->tensors[a.t[2]].kind == INFR_TK_INTERNAL;
            if (ok) {
                const uint32_t nh = rq.u[1], nkv = a.u[1], hd = a.u[2];
                const uint32_t grp = nkv ? nh / nkv : 0;
                ok = nkv && nh % nkv == 0 && (hd == 64 || hd == 128) && (grp == 1 || grp == 2 || grp == 4 || grp == 8);
            }
            // the rotated k is never materialised by the grouped launch: nobody else may read it
            for (uint32_t j = i + 4; ok && j < g.n_ops; j++)
                if (op_reads(g.ops[j], a.t[2])) ok = false;
            if (ok) st = PlanStep{PlanStep::kRopeWriteKv, i, 4};
        }
        plan->steps.push_back(st);
        i += st.n_ops;
    }
    // ---- Internal handles: scratch from the pool; zero-filled only where an op could see the fill ----
    cudaSetDevice(device_);
    std::vector<char> written(g.n_tensors, 0);
    for (uint32_t i = 0; i < g.n_tensors; i++) plan->needs_zero[i] = 0;
    for (uint32_t i = 0; i < g.n_ops; i++) {
        const infr_op_desc &op = g.ops[i];
        const int nt = op_tensors(op.tag);
        uint64_t numel = 0;
        const int dst = op_full_dst(op, &numel);
        for (int k = 0; k < nt; k++) {
            const uint32_t id = op.t[k];
            if (plan->tensors[id].kind != INFR_TK_INTERNAL || written[id]) continue;
            if (k == dst && numel >= plan->tensors[id].numel && !op_reads(op, id)) continue;  // first touch overwrites all of it
            plan->needs_zero[id] = 1;
        }
        if (dst >= 0 && numel >= plan->tensors[op.t[dst]].numel) written[op.t[dst]] = 1;
    }
    for (uint32_t i = 0; i < g.n_tensors; i++) {
        if (g.tensors[i].kind != INFR_TK_INTERNAL) continue;
        const size_t bytes = up256(tensor_bytes(g.tensors[i]));
        if (!bytes) continue;
        Status s = pool_acquire(bytes, &plan->internal[i]);
        if (!s.ok()) return fail(s);
        plan->internal_bytes[i] = bytes;
    }
    *out = plan;
    return Status::Ok();
}

void CudaBackend::free_plan(infr_cuda_plan *p) {
    if (!p) return;
    // The blocks go back to the pool; work already enqueued on the stream that still uses them runs before
    // anything a later plan enqueues (one stream), so no synchronisation is needed here.
    for (void *q : p->internal)
        if (q) pool_release(q);
    if (p->cached) graph_free(p->cached);
    delete p;
}

// The second execute of a plan on the same buffers captures its launches into a CUDA graph (the first one ran op by
// op and sized the context scratch); later ones replay it.  Anything that changes what the kernels would be given
// (other buffers, a reallocated scratch, other kernel options) runs op by op again and starts over.  Inside a
// caller's own stream capture the ops are issued directly.
Status CudaBackend::execute(infr_cuda_plan *plan, infr_cuda_buf *const *bindings, uint32_t n) {
    if (!plan) return Status::Err(INFR_E_INVALID, "execute: null plan");
    if (capturing_ || plan->no_graph || plan->steps.size() < 2) return execute_steps(plan, bindings, n);
    cudaSetDevice(device_);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream_, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
        return execute_steps(plan, bindings, n);  // somebody else is capturing this stream
    std::vector<uint64_t> key;
    key.reserve(2 * (size_t)n + 5);
    key.push_back(n);
    key.push_back(scratch_gen_);
    key.push_back((uint64_t)reference_);
    key.push_back((uint64_t)gemv_impl_);
    key.push_back((uint64_t)mmq_impl_);
    for (uint32_t i = 0; i < n; i++) {
        key.push_back(bindings && bindings[i] ? (uint64_t)(uintptr_t)bindings[i]->ptr : 0);
        key.push_back(bindings && bindings[i] ? (uint64_t)bindings[i]->len : 0);
    }
    if (plan->cached && key == plan->cached_key) return graph_launch(plan->cached);
    if (key != plan->last_key) {
        plan->last_key = key;
        return execute_steps(plan, bindings, n);
    }
    // same buffers as the previous, op-by-op run: capture
    if (plan->cached) {
        graph_free(plan->cached);
        plan->cached = nullptr;
        plan->cached_key.clear();
    }
    const uint64_t launches_before = launches_;
    Status s = capture_begin();
    if (!s.ok()) return execute_steps(plan, bindings, n);
    Status run = execute_steps(plan, bindings, n);
    infr_cuda_graph *g = nullptr;
    s = capture_end(&g);
    launches_ = launches_before;  // nothing ran while capturing
    if (!run.ok() || !s.ok()) {
        // an op that cannot be captured: the plan runs op by op from now on
        if (g) graph_free(g);
        cudaGetLastError();
        plan->no_graph = true;
        return execute_steps(plan, bindings, n);
    }
    plan->cached = g;
    plan->cached_key = key;
    return graph_launch(g);
}


Status CudaBackend::execute_steps(infr_cuda_plan *plan, infr_cuda_buf *const *bindings, uint32_t n) {
    cudaSetDevice(device_);
    const uint32_t nt = (uint32_t)plan->tensors.size();
    // Provision: Internal handles read as zero until written (crates/infr-core/src/exec.rs:53-92).
    for (uint32_t i = 0; i < nt; i++)
        if (plan->internal[i] && plan->needs_zero[i]) {
            Status s = cuda_status(cudaMemsetAsync(plan->internal[i], 0, plan->internal_bytes[i], stream_), "zero internal");
            if (!s.ok()) return s;
        }
    auto resolve = [&](uint32_t id, size_t need, const char *role, DevSpan *out) -> Status {
        const infr_tensor_decl &d = plan->tensors[id];
        if (d.kind == INFR_TK_INTERNAL) {
            *out = DevSpan{static_cast<uint8_t *>(plan->internal[id]), plan->internal_bytes[id]};
        } else {
            if (id >= n || !bindings || !bindings[id]) return Status::Err(INFR_E_INVALID, pfmt("execute: %s handle %u is unbound", role, id));
            *out = DevSpan{static_cast<uint8_t *>(bindings[id]->ptr), bindings[id]->len};
        }
        if (out->bytes < need) return Status::Err(INFR_E_INVALID, pfmt("execute: %s handle %u holds %zu bytes, op needs %zu", role, id, out->bytes, need));
        return Status::Ok();
    };
#define INFR_RESOLVE(id, need, role, out)                     \
    do {                                                      \
        Status rs_ = resolve((id), (need), (role), (out));    \
        if (!rs_.ok()) return rs_;                            \
    } while (0)
    auto f32p = [](const DevSpan &s) { return reinterpret_cast<float *>(s.ptr); };

    for (const PlanStep &st : plan->steps) {
        const infr_op_desc &op = plan->ops[st.op0];
        Status s;
        if (st.kind == PlanStep::kAddRmsNorm) {
            const infr_op_desc &nm = plan->ops[st.op0 + 1];
            const uint32_t rows = nm.u[0], dim = nm.u[1];
            const size_t nb = (size_t)rows * dim * 4;
            DevSpan a, b, sum, w, dst;
            INFR_RESOLVE(op.t[0], nb, "Add a", &a);
            INFR_RESOLVE(op.t[1], nb, "Add b", &b);
            INFR_RESOLVE(op.t[2], nb, "Add dst", &sum);
            INFR_RESOLVE(nm.t[1], (size_t)dim * 4, "RmsNorm weight", &w);
            INFR_RESOLVE(nm.t[2], nb, "RmsNorm dst", &dst);
            s = rms_norm(f32p(a), f32p(b), f32p(sum), f32p(w), f32p(dst), rows, dim, nm.f[0]);
            if (!s.ok()) return s;
            continue;
        }
        if (st.kind == PlanStep::kLinearPair) {
            const infr_op_desc &o2 = plan->ops[st.op0 + 1];
            const uint32_t m = op.u[0], in_f = op.u[1];
            const int wdt = (int)plan->tensors[op.t[1]].dtype;
            const size_t bpr = (size_t)(in_f / block_elems(wdt)) * block_bytes(wdt);
            const size_t r1 = op.u[3] / in_f, r2 = o2.u[3] / in_f;
            DevSpan x, w1, w2, y1, y2;
            INFR_RESOLVE(op.t[0], (size_t)m * in_f * 4, "Linear x", &x);
            INFR_RESOLVE(op.t[1], (r1 + op.u[2]) * bpr, "Linear weight", &w1);
            INFR_RESOLVE(o2.t[1], (r2 + o2.u[2]) * bpr, "Linear weight", &w2);
            INFR_RESOLVE(op.t[2], (size_t)m * op.u[2] * 4, "Linear dst", &y1);
            INFR_RESOLVE(o2.t[2], (size_t)m * o2.u[2] * 4, "Linear dst", &y2);
            s = linear_pair(wdt, w1.ptr + r1 * bpr, f32p(y1), op.u[2], w2.ptr + r2 * bpr, f32p(y2), o2.u[2], f32p(x), m, in_f,
                            reference_ ? INFR_ACT_F32 : INFR_ACT_INT8);
            if (!s.ok()) return s;
            continue;
        }
        if (st.kind == PlanStep::kRopeWriteKv) {
            const infr_op_desc &rq = plan->ops[st.op0 + 1], &wk = plan->ops[st.op0 + 2], &wv = plan->ops[st.op0 + 3];
            const uint32_t rows = op.u[0], nkv = op.u[1], hd = op.u[2], nh = rq.u[1], pos = wk.u[2];
            DevSpan k, q, v, p, kc, vc;
            INFR_RESOLVE(op.t[0], (size_t)rows * nkv * hd * 4, "Rope x (k)", &k);
            INFR_RESOLVE(rq.t[0], (size_t)rows * nh * hd * 4, "Rope x (q)", &q);
            INFR_RESOLVE(wv.t[0], (size_t)rows * nkv * hd * 4, "WriteKv src (v)", &v);
            INFR_RESOLVE(op.t[1], (size_t)rows * 4, "Rope positions", &p);
            const size_t cache_need = ((size_t)pos + rows) * nkv * hd * 2;
            INFR_RESOLVE(wk.t[1], cache_need, "WriteKv cache (k)", &kc);
            INFR_RESOLVE(wv.t[1], cache_need, "WriteKv cache (v)", &vc);
            infr_attn_desc d{};
            d.rows = rows, d.pos = pos, d.n_head = nh, d.n_kv = nkv, d.head_dim = hd, d.scale = 0.f, d.n_seq = 1, d.seq_stride = 0;
            s = rope_write_kv(d, op.f[0], op.u[5] != 0, f32p(q), f32p(k), f32p(v), reinterpret_cast<const int32_t *>(p.ptr), kc.ptr, vc.ptr,
                              (int)pos);
            if (!s.ok()) return s;
            continue;
        }
        switch (op.tag) {
        case INFR_OP_LINEAR: {
            const uint32_t m = op.u[0], in_f = op.u[1], out_f = op.u[2], w_off = op.u[3];
            const int wdt = (int)plan->tensors[op.t[1]].dtype;
            const size_t bpr = (size_t)(in_f / block_elems(wdt)) * block_bytes(wdt);
            const size_t row0 = w_off / in_f;
            DevSpan x, w, y;
            INFR_RESOLVE(op.t[0], (size_t)m * in_f * 4, "Linear x", &x);
            INFR_RESOLVE(op.t[1], (row0 + out_f) * bpr, "Linear weight", &w);
            INFR_RESOLVE(op.t[2], (size_t)m * out_f * 4, "Linear dst", &y);
            s = linear(wdt, w.ptr + row0 * bpr, f32p(x), f32p(y), m, in_f, out_f, reference_ ? INFR_ACT_F32 : INFR_ACT_INT8);
            break;
        }
        case INFR_OP_MOE_FFN: {
            const uint32_t ne = op.u[0], nx = op.u[1], nu = op.u[2], nff = op.u[3];
            const infr_tensor_decl &xd = plan->tensors[op.t[0]];
            const uint32_t rows = ne ? (uint32_t)(xd.numel / ne) : 0;
            const int gdt = (int)plan->tensors[op.t[3]].dtype, udt = (int)plan->tensors[op.t[4]].dtype, ddt = (int)plan->tensors[op.t[5]].dtype;
            auto bank = [&](int bdt, size_t o, size_t k) { return (size_t)nx * o * (k / 256) * (size_t)block_bytes(bdt); };
            DevSpan x, rx, r, gt, up, dn, dst;
            INFR_RESOLVE(op.t[0], (size_t)rows * ne * 4, "MoeFfn x", &x);
            INFR_RESOLVE(op.t[1], (size_t)rows * ne * 4, "MoeFfn router_x", &rx);
            INFR_RESOLVE(op.t[2], (size_t)nx * ne * 4, "MoeFfn router", &r);
            INFR_RESOLVE(op.t[3], bank(gdt, nff, ne), "MoeFfn gate_exps", &gt);
            INFR_RESOLVE(op.t[4], bank(udt, nff, ne), "MoeFfn up_exps", &up);
            INFR_RESOLVE(op.t[5], bank(ddt, ne, nff), "MoeFfn down_exps", &dn);
            INFR_RESOLVE(op.t[6], (size_t)rows * ne * 4, "MoeFfn dst", &dst);
            MoeArgs a{f32p(x), f32p(rx), f32p(r), gt.ptr, up.ptr, dn.ptr, gdt, udt, ddt, f32p(dst), rows, ne, nx, nu, nff, op.f[0],
                      (int)op.u[4], nullptr, nullptr, nullptr, 0u, nx};
            s = moe_ffn(a);
            break;
        }
        case INFR_OP_RMS_NORM: {
            const uint32_t rows = op.u[0], dim = op.u[1];
            DevSpan x, w, dst;
            INFR_RESOLVE(op.t[0], (size_t)rows * dim * 4, "RmsNorm x", &x);
            INFR_RESOLVE(op.t[1], (size_t)dim * 4, "RmsNorm weight", &w);
            INFR_RESOLVE(op.t[2], (size_t)rows * dim * 4, "RmsNorm dst", &dst);
            s = rms_norm(f32p(x), nullptr, nullptr, f32p(w), f32p(dst), rows, dim, op.f[0]);
            break;
        }
        case INFR_OP_ROPE: {
            const uint32_t rows = op.u[0], nh = op.u[1], hd = op.u[2];
            const size_t nb = (size_t)rows * nh * hd * 4;
            DevSpan x, p, dst;
            INFR_RESOLVE(op.t[0], nb, "Rope x", &x);
            INFR_RESOLVE(op.t[1], (size_t)rows * 4, "Rope positions", &p);
            INFR_RESOLVE(op.t[2], nb, "Rope dst", &dst);
            s = rope(f32p(x), reinterpret_cast<const int32_t *>(p.ptr), f32p(dst), rows, nh, hd, op.u[3], op.f[0], op.u[5] != 0);
            break;
        }
        case INFR_OP_WRITE_KV: {
            const uint32_t rows = op.u[0], stride = op.u[1], pos = op.u[2];
            const size_t nel = (size_t)rows * stride;
            DevSpan src, cache;
            INFR_RESOLVE(op.t[0], nel * 4, "WriteKv src", &src);
            // the cache holds the whole context: a write past its end is an error, not a ring wrap
            INFR_RESOLVE(op.t[1], ((size_t)pos * stride + nel) * 2, "WriteKv cache", &cache);
            s = write_kv(f32p(src), cache.ptr + (size_t)pos * stride * 2, nel);
            break;
        }
        case INFR_OP_ATTENTION: {
            infr_attn_desc d{};
            d.rows = op.u[0], d.pos = op.u[6], d.n_head = op.u[2], d.n_kv = op.u[3], d.head_dim = op.u[4], d.scale = op.f[0], d.n_seq = 1;
            const size_t qn = (size_t)d.rows * d.n_head * d.head_dim * 4, cn = (size_t)op.u[1] * d.n_kv * d.head_dim * 2;
            DevSpan q, kc, vc, dst;
            INFR_RESOLVE(op.t[0], qn, "Attention q", &q);
            INFR_RESOLVE(op.t[1], cn, "Attention k_cache", &kc);
            INFR_RESOLVE(op.t[2], cn, "Attention v_cache", &vc);
            INFR_RESOLVE(op.t[3], qn, "Attention dst", &dst);
            s = attention(d, f32p(q), kc.ptr, vc.ptr, f32p(dst));
            break;
        }
        case INFR_OP_GATED_ACT: {
            const size_t nel = (size_t)op.u[0] * op.u[1];
            DevSpan gt, up, dst;
            INFR_RESOLVE(op.t[0], nel * 4, "GatedAct gate", &gt);
            INFR_RESOLVE(op.t[1], nel * 4, "GatedAct up", &up);
            INFR_RESOLVE(op.t[2], nel * 4, "GatedAct dst", &dst);
            s = gated_act(f32p(gt), f32p(up), f32p(dst), nel);
            break;
        }
        case INFR_OP_ADD: {
            const size_t nel = op.u[0];
            DevSpan a, b, dst;
            INFR_RESOLVE(op.t[0], nel * 4, "Add a", &a);
            INFR_RESOLVE(op.t[1], nel * 4, "Add b", &b);
            INFR_RESOLVE(op.t[2], nel * 4, "Add dst", &dst);
            s = add(f32p(a), f32p(b), f32p(dst), nel);
            break;
        }
        case INFR_OP_ARGMAX: {
            const uint32_t nel = op.u[0], rows = op.u[1];
            if (nel == 0 || rows == 0 || rows > 65535) return Status::Err(INFR_E_INVALID, "execute: Argmax needs n > 0 and 1..65535 rows");
            DevSpan x, dst;
            INFR_RESOLVE(op.t[0], (size_t)rows * nel * 4, "Argmax x", &x);
            INFR_RESOLVE(op.t[1], (size_t)rows * 4, "Argmax dst", &dst);
            s = argmax(f32p(x), reinterpret_cast<uint32_t *>(dst.ptr), nel, rows);
            break;
        }
        case INFR_OP_COPY: {
            // element offsets; both tensors hold 4-byte elements (f32 rows, i32 ids)
            const size_t so = op.u[0], dof = op.u[1], nel = op.u[2];
            DevSpan src, dst;
            INFR_RESOLVE(op.t[0], (so + nel) * 4, "Copy src", &src);
            INFR_RESOLVE(op.t[1], (dof + nel) * 4, "Copy dst", &dst);
            s = cuda_status(cudaMemcpyAsync(dst.ptr + dof * 4, src.ptr + so * 4, nel * 4, cudaMemcpyDeviceToDevice, stream_), "Copy");
            break;
        }
        default: return Status::Err(INFR_E_UNSUPPORTED, pfmt("execute: op %u tag %u", st.op0, op.tag));
        }
        if (!s.ok()) return s;
    }
#undef INFR_RESOLVE
    // Outputs live in their bound device buffers already; the caller's download (or sync) orders
    // after this stream's work, as Backend::execute + Backend::download do on the other backends.
    return Status::Ok();
}

}  // namespace infr
