#!/usr/bin/env python
"""Benchmark of the block-quantized decode GEMV path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--no-sweep]

Headline workload (config.workload): the Q4_K 4096x4096 matvec (x fp32 [1,4096], y fp32 [1,4096]),
the configuration the metric "Q4_K GEMV HBM GB/s" is quoted on.  One matrix is 9.4 MB and would sit in
the 126 MB L2, so a STEP is one pass over ROT = 64 device copies of the matrix at distinct addresses
(604 MB, > 4x L2): every launch streams its weights from HBM.  GB/s = ROT * 9 469 952 B / step time
(algorithmic bytes: packed weights + x + y).

  value     device-resident: one CUDA graph per step holding ROT x (quantise x -> int8, GEMV)
  roofline  the GEMV kernel alone on pre-quantised activations, timed live with CUDA events on the
            library's stream, against the measured HBM copy bandwidth in MEASURED_PEAKS.json
  e2e       the same pass through the Backend interface with HOST buffers: per step, one upload of the step's
            ROT input rows from pinned memory, one execute of a plan holding the step's ROT Linear ops, one download
            of the ROT result rows to pinned memory; beside it the latency of one synchronous upload / execute /
            download round trip per matrix (round_trip_us_per_call)
  sweep     (N=1) the other GEMV configurations: Q6_K 14336x4096 and ternary Q2_0 4096x14336 at
            batch 1/4/8, Q4_K 14336x4096; each rotated over > 4x L2 of distinct copies
  decode_step   (N=1) a whole 8B-shape decode step (32 layers: norms, Linears, RoPE + KV write, causal
            attention over a 4096-token f16 KV cache, SiLU gate, residual adds; head; argmax) at batch 1 and 32,
            one CUDA graph, tok/s = batch / step time
  cpu_baseline  the CPU restatement of infr-cpu on the host cores, bounded sample (N=1, rank 0)

--impl reference times the CPU restatement of infr-cpu (the reference is Rust; no Rust toolchain
exists here, so its own binary cannot be built) on all host threads on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

IN_F = OUT_F = 4096
ROT = 64
C1_BYTES = 4096 * 4096 // 256 * 144 + 4 * 4096 + 4 * 4096  # 9 469 952


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs."""

    BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                r = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for bit, name in self.BITS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self.nv:
            self._stop.clear()
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        if self._thr:
            self._stop.set()
            self._thr.join()
            self._thr = None

    def summary(self):
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def _dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist_.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist_.init_process_group("gloo")
        dist = dist_
    return rank, world, local, dist


def _barrier(dist):
    if dist is not None:
        dist.barrier()


def _max_over_ranks(dist, v: float) -> float:
    if dist is None:
        return v
    import torch

    t = torch.tensor([v], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------
def _rotation(be, infr_b200, dtype, out_f, in_f, seed, min_bytes):
    """Distinct device copies of one seeded weight; returns (buffers, host bytes)."""
    from infr_b200 import synth

    w = synth.weight(dtype, out_f, in_f, seed)
    n = max(2, int(np.ceil(min_bytes / w.nbytes)))
    first = be.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    bufs = [first]
    for _ in range(n - 1):
        b = be.alloc_uninit(w.nbytes, infr_b200.USAGE_WEIGHTS)
        be.copy_buffer(first, b, w.nbytes)
        bufs.append(b)
    be.sync()
    return bufs, w


def _time_graph(be, graph, steps, warmup, dist=None):
    for _ in range(warmup):
        graph.launch()
    be.sync()
    _barrier(dist)
    be.timer_start()
    for _ in range(steps):
        graph.launch()
    ms = be.timer_stop()
    return ms


def _gemv_case(be, infr_b200, dtype, out_f, in_f, m, seed, steps, warmup, l2_bytes, hbm_peak):
    """GB/s of quantise+GEMV and of the GEMV kernel alone for one configuration (rotated weights)."""
    from infr_b200 import synth

    bufs, w = _rotation(be, infr_b200, dtype, out_f, in_f, seed, 4 * l2_bytes + (64 << 20))
    rot = len(bufs)
    x = synth.normal(seed + 1, (m, in_f))
    xb = be.from_numpy(x)
    ys = [be.alloc(m * out_f * 4) for _ in range(rot)]
    gran = 32 if dtype == infr_b200.Q2_0 else 256
    qs, d = be.alloc(m * in_f), be.alloc(m * (in_f // gran) * 4)
    s32, s16 = be.alloc(m * (in_f // 32) * 4), be.alloc(m * (in_f // 16) * 4)
    be.gemv(dtype, bufs[0], xb, ys[0], m, in_f, out_f)  # warm the scratch before capture
    be.quantize_q8(gran, xb, m, in_f, qs, d, s32, s16 if gran == 256 else None)
    be.capture_begin()
    for i in range(rot):
        be.gemv(dtype, bufs[i], xb, ys[i], m, in_f, out_f)
    g_full = be.capture_end()
    be.capture_begin()
    for i in range(rot):
        be.gemv_q8(dtype, bufs[i], qs, d, s32, s16 if dtype == infr_b200.Q6K else None, ys[i], m, in_f, out_f)
    g_kern = be.capture_end()
    ms_full = _time_graph(be, g_full, steps, warmup)
    ms_kern = _time_graph(be, g_kern, steps, warmup)
    alg = w.nbytes + 4 * m * in_f + 4 * m * out_f
    res = {
        "workload": f"{synth.DTYPE_NAMES[dtype]} GEMV W {out_f}x{in_f} m={m}, {rot} distinct copies rotated",
        "alg_bytes_per_launch": alg,
        "gbs": alg * rot * steps / (ms_full * 1e-3) / 1e9,
        "kernel_us": ms_kern * 1e3 / (steps * rot),
        "kernel_gbs": alg * rot * steps / (ms_kern * 1e-3) / 1e9,
    }
    res["kernel_frac_of_measured_hbm"] = res["kernel_gbs"] / hbm_peak
    for g in (g_full, g_kern):
        g.close()
    for b in bufs + ys + [xb, qs, d, s32, s16]:
        b.close()
    return res


def _int8_peak(be):
    """Dense int8 tensor-core peak of this GPU, measured: tcgen05 kind::i8 128x256x32 instructions on operands resident
    in shared memory, two issuing threads per SM, no unpack and no epilogue (infr_cuda_tensor_peak_i8, which also
    checks one accumulator element per issuer).  `burst` is a few milliseconds (what a kernel timed alone sees),
    `sustained` is > 100 ms under the power cap."""
    ms_b, ops_b = be.tensor_peak_i8(n_batches=64, launches=10)
    ms_s, ops_s = be.tensor_peak_i8(n_batches=256, launches=100)
    return {"burst_tops": ops_b / (ms_b * 1e-3) / 1e12, "burst_ms": ms_b,
            "sustained_tops": ops_s / (ms_s * 1e-3) / 1e12, "sustained_ms": ms_s, "spec_tops": 4500.0,
            "how": "tcgen05.mma kind::i8 M=128 N=256 K=32 from resident shared-memory operands, 2 issuers per SM, CUDA events"}


def _mmq_case(be, infr_b200, m, in_f, out_f, seed, steps, warmup, peak=None):
    """Prefill MMQ (Linear with m > 8): int8 TOPS = 2*m*in_f*out_f / time; the activation quantiser is inside."""
    from infr_b200 import synth

    w = synth.weight(infr_b200.Q4K, out_f, in_f, seed)
    wb = be.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    xb = be.from_numpy(synth.normal(seed + 1, (m, in_f)))
    yb = be.alloc(m * out_f * 4)
    for _ in range(warmup):
        be.linear(infr_b200.Q4K, wb, xb, yb, m, in_f, out_f)
    be.sync()
    be.timer_start()
    for _ in range(steps):
        be.linear(infr_b200.Q4K, wb, xb, yb, m, in_f, out_f)
    ms = be.timer_stop()
    ops = 2.0 * m * in_f * out_f
    tops = ops * steps / (ms * 1e-3) / 1e12
    res = {"workload": f"prefill MMQ q4_k M={m} K={in_f} N={out_f} (quantise + tcgen05 kind::i8 GEMM)",
           "int8_ops": ops, "us": ms * 1e3 / steps, "tops": tops, "frac_of_4500_tops_spec": tops / 4500.0}
    if peak:
        # algorithmic ops 2*M*K*N; the kernel issues twice that on the tensor cores (the 6-bit sub-block scale is
        # split into two int8 operands so that the int32 block sums stay exact) plus the tf32 min term
        res["roofline"] = {"bound": "int8", "achieved": tops, "peak": peak["burst_tops"], "unit": "TOPS", "frac": tops / peak["burst_tops"],
                           "peak_source": "measured (infr_cuda_tensor_peak_i8, burst)", "peak_spec": 4500.0,
                           "alg_ops_per_launch": ops, "kernel": "quantize_q8 + mmq_ws_prep + mmq_ws_kernel"}
    for b in (wb, xb, yb):
        b.close()
    return res


def _moe_case(be, infr_b200, steps, warmup, hbm_peak=None):
    """Qwen3-30B-A3B-shaped MoE layer: 256 tokens, hidden 2048, 128 experts (gate/up 2048->768, down 768->2048,
    Q4_K), softmax top-8.  Bank bytes are random valid Q4_K blocks (timing does not depend on the values)."""
    from infr_b200 import synth

    rows, ne, nx, nu, nff = 256, 2048, 128, 8, 768
    gate = be.from_numpy(synth.random_blocks(infr_b200.Q4K, nx * nff * ne, 100), infr_b200.USAGE_WEIGHTS)
    up = be.from_numpy(synth.random_blocks(infr_b200.Q4K, nx * nff * ne, 101), infr_b200.USAGE_WEIGHTS)
    down = be.from_numpy(synth.random_blocks(infr_b200.Q4K, nx * ne * nff, 102), infr_b200.USAGE_WEIGHTS)
    router = be.from_numpy(synth.normal(7, (nx, ne), 1.0 / np.sqrt(ne)))
    x = be.from_numpy(synth.normal(8, (rows, ne)))
    dst = be.alloc(rows * ne * 4)
    kw = dict(rows=rows, ne=ne, n_expert=nx, n_used=nu, n_ff_exp=nff)
    for _ in range(warmup):
        be.moe_ffn(x, x, router, gate, up, down, dst, **kw)
    be.sync()
    be.timer_start()
    for _ in range(steps):
        be.moe_ffn(x, x, router, gate, up, down, dst, **kw)
    ms = be.timer_stop()
    w_bytes = 3 * nx * nff * ne // 256 * 144
    ops = rows * nu * 3 * 2.0 * ne * nff
    res = {"workload": "MoE layer 256 tok x hidden 2048, 128 experts x (2048->768->2048) Q4_K, softmax top-8 (9 kernels)",
           "us": ms * 1e3 / steps, "weight_bytes": w_bytes, "weights_gbs": w_bytes * steps / (ms * 1e-3) / 1e9,
           "int8_tops": ops * steps / (ms * 1e-3) / 1e12, "l2": "weights 340 MB > L2"}
    if hbm_peak:
        alg = w_bytes + 2 * rows * ne * 4  # every expert is hit with 2048 routed pairs: all banks once, x in, y out
        gbs = alg * steps / (ms * 1e-3) / 1e9
        res["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                           "alg_bytes_per_layer": alg, "peak_source": "measured HBM copy bandwidth"}
    for b in (gate, up, down, router, x, dst):
        b.close()
    return res


def _decode_linears_case(be, infr_b200, batch, steps, warmup):
    """The Linear ops of one Llama-3-8B-shaped decode step in the Q4_K_M mix (32 layers: q, k, o, gate, up in Q4_K,
    v and down in Q6_K; output head in Q6_K), every layer on its own device copy of the weights (4.9 GB, far
    beyond L2), captured in one CUDA graph.  Attention, norms and RoPE are not part of this path yet, so the
    figure is the matmul share of a decode step.  Weight bytes are random valid blocks."""
    from infr_b200 import synth

    Q4K, Q6K = infr_b200.Q4K, infr_b200.Q6K
    n_layer, h, kv, ff, vocab = 32, 4096, 1024, 14336, 128256
    shapes = [("wq", Q4K, h, h), ("wk", Q4K, kv, h), ("wv", Q6K, kv, h), ("wo", Q4K, h, h),
              ("gate", Q4K, ff, h), ("up", Q4K, ff, h), ("down", Q6K, h, ff)]
    masters = {name: be.from_numpy(synth.random_blocks(dt, o * i, 200 + k), infr_b200.USAGE_WEIGHTS)
               for k, (name, dt, o, i) in enumerate(shapes)}
    layers, total_bytes = [], 0
    for _ in range(n_layer):
        bufs = {}
        for name, dt, o, i in shapes:
            nbytes = o * i // synth.BLOCK_ELEMS[dt] * synth.BLOCK_BYTES[dt]
            b = be.alloc_uninit(nbytes, infr_b200.USAGE_WEIGHTS)
            be.copy_buffer(masters[name], b, nbytes)
            bufs[name] = b
            total_bytes += nbytes
        layers.append(bufs)
    head_bytes = vocab * h // 256 * 210
    head = be.from_numpy(synth.random_blocks(Q6K, vocab * h, 299), infr_b200.USAGE_WEIGHTS)
    total_bytes += head_bytes
    xh = be.from_numpy(synth.normal(31, (batch, h)))
    xf = be.from_numpy(synth.normal(32, (batch, ff)))
    yh, ykv, yff, ylog = be.alloc(batch * h * 4), be.alloc(batch * kv * 4), be.alloc(batch * ff * 4), be.alloc(batch * vocab * 4)

    def step():
        n = 0
        for L in layers:
            for name, dt, o, i in shapes:
                src = xf if i == ff else xh
                dst = yff if o == ff else (ykv if o == kv else yh)
                be.linear(dt, L[name], src, dst, batch, i, o)
                n += 1
        be.linear(Q6K, head, xh, ylog, batch, h, vocab)
        return n + 1

    step()  # sizes the context scratch before capture
    be.sync()
    l0 = be.launch_count()
    be.capture_begin()
    n_linear = step()
    graph = be.capture_end()
    kernels = be.launch_count() - l0
    ms = _time_graph(be, graph, steps, warmup)
    us = ms * 1e3 / steps
    res = {"workload": f"Linear ops of an 8B-shape decode step, batch {batch}: {n_linear} Linears, Q4_K_M mix "
                       f"(v/down/head Q6_K), {total_bytes / 1e9:.2f} GB of weights, one CUDA graph",
           "us_per_step": us, "tok_per_s_matmul_only": batch / (us * 1e-6), "weights_gbs": total_bytes / (us * 1e-6) / 1e9,
           "kernels_per_step": kernels, "not_included": "attention, norms, RoPE, sampling: see decode_step"}
    graph.close()
    for b in [head, xh, xf, yh, ykv, yff, ylog] + list(masters.values()) + [b for L in layers for b in L.values()]:
        b.close()
    return res


def _decode_step_case(be, infr_b200, batch, steps, warmup, hbm_peak, pos=4096, shard=1):
    """A whole Llama-3-8B-shape decode step: 32 layers of RmsNorm, q/k/v Linears, RoPE + f16 KV write, causal
    attention over a KV cache pre-filled to `pos` positions, o Linear, residual add + RmsNorm, gate/up Linears, SiLU
    gate, down Linear, residual add; then the output norm, the 128256-row head and argmax.  Q4_K_M mix (attn_v and
    ffn_down Q6_K, the rest Q4_K), every layer on its own device copy of the weights, `batch` independent sequences
    with their own caches, the step captured in one CUDA graph.  The input rows stand for the host-embedded token
    rows (the graph restores them at the start of every replay).  Weight bytes are random valid blocks; cache
    values are N(0,1) halves.
    shard = N > 1: ONE rank's share of the step split N ways (heads, padded FFN slice, vocabulary slice), alone on this
    GPU, its row-parallel results pushed to and pulled from a 1-rank comm: what a rank of the tensor-parallel step
    computes, with the kernels it launches, without the waiting for peers."""
    import numpy as np
    from infr_b200 import shard as shard_mod, synth
    from infr_b200.decode import DecodeStep, LlamaShape

    Q4K = infr_b200.Q4K
    s = LlamaShape()
    if shard > 1:
        s = LlamaShape(n_head=s.n_head // shard, n_kv=s.n_kv // shard, ffn=shard_mod.ffn_split(s.ffn, shard)[0][2], vocab=s.vocab // shard)
    max_ctx = pos + 8
    masters = {name: be.from_numpy(synth.random_blocks(dt, o * i, 200 + k), infr_b200.USAGE_WEIGHTS)
               for k, (name, dt, o, i) in enumerate(s.linears())}
    norm = be.from_numpy((1.0 + 0.02 * synth.normal(40, (s.hidden,))).astype(np.float32))
    layers, w_bytes, owned = [], 0, []
    for _ in range(s.n_layer):
        L = {"attn_norm": norm, "ffn_norm": norm}
        for name, dt, o, i in s.linears():
            nbytes = o * i // synth.BLOCK_ELEMS[dt] * synth.BLOCK_BYTES[dt]
            b = be.alloc_uninit(nbytes, infr_b200.USAGE_WEIGHTS)
            be.copy_buffer(masters[name], b, nbytes)
            L[name] = b
            owned.append(b)
            w_bytes += nbytes
        layers.append(L)
    head = be.from_numpy(synth.random_blocks(Q4K, s.vocab * s.hidden, 299), infr_b200.USAGE_WEIGHTS)
    w_bytes += s.vocab * s.hidden // 256 * 144
    seq_bytes = max_ctx * s.kv_dim * 2
    kv_master = be.from_numpy(synth.normal(9, (max_ctx, s.kv_dim)).astype(np.float16).view(np.uint16))
    kc, vc = [], []
    for _ in range(s.n_layer):
        for lst in (kc, vc):
            c = be.alloc_uninit(batch * seq_bytes, infr_b200.USAGE_ACTIVATIONS)
            for q in range(batch):
                view = be.wrap(c.device_ptr() + q * seq_bytes, seq_bytes, infr_b200.USAGE_ACTIVATIONS)
                be.copy_buffer(kv_master, view, seq_bytes)
                view.close()
            lst.append(c)
    comm = be.comm_create(0, 1, batch * s.hidden) if shard > 1 else None
    step = DecodeStep(be, s, batch, max_ctx, layers, norm, head, Q4K, kc, vc, comm=comm)
    hidden0 = be.from_numpy(synth.normal(31, (batch, s.hidden)))
    step.set_inputs(synth.normal(31, (batch, s.hidden)), pos)

    def one():
        be.copy_buffer(hidden0, step.hidden, batch * s.hidden * 4)
        return step.run(pos, fused=True)

    one()  # sizes the context scratch before capture
    be.sync()
    tok_eager = be.download(step.tok, np.uint32)
    l0 = be.launch_count()
    be.capture_begin()
    n_ops = one()
    graph = be.capture_end()
    kernels = be.launch_count() - l0
    ms = _time_graph(be, graph, steps, warmup)
    us = ms * 1e3 / steps
    tok = be.download(step.tok, np.uint32)
    kv_bytes = s.n_layer * 2 * (pos + 1) * s.kv_dim * 2 * batch
    alg = w_bytes + kv_bytes
    what = "8B-shape decode step" if shard == 1 else f"one rank's share of the 8B-shape decode step split {shard} ways (exchange with itself)"
    res = {"workload": f"{what}, batch {batch} (independent sequences), KV context {pos} (kv_len {pos + 1}), Q4_K_M mix, "
                       f"{n_ops} ops in one CUDA graph",
           "us_per_step": us, "tok_per_s": batch / (us * 1e-6), "weight_bytes": w_bytes, "kv_bytes_read": kv_bytes,
           "hbm_gbs": alg / (us * 1e-6) / 1e9, "frac_of_measured_hbm": alg / (us * 1e-6) / 1e9 / hbm_peak,
           "roofline": {"bound": "hbm", "achieved": alg / (us * 1e-6) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                        "frac": alg / (us * 1e-6) / 1e9 / hbm_peak, "alg_bytes_per_step": alg,
                        "peak_source": "measured HBM copy bandwidth (sustained over the step)"},
           "kernels_per_step": kernels, "tokens_same_eager_and_graph": bool((tok == tok_eager).all()),
           "first_token_ids": [int(t) for t in tok[:4]]}
    graph.close()
    if comm is not None:
        comm.close()
    for b in owned + kc + vc + [head, kv_master, hidden0, norm] + list(masters.values()):
        b.close()
    return res


def _tp_decode(be, infr_b200, dist, rank, world, local, steps, warmup):
    """Tensor-parallel form of the decode step's Linear ops (batch 1): q/k/v/gate/up and the output head are
    split by output rows, o and down by input columns with an NCCL all-reduce of the 4096-float result after each
    (2 per layer), the head's logits are all-gathered.  Activations live in torch tensors that the backend wraps
    in place (infr_cuda_wrap) and torch runs on the backend's stream (infr_cuda_stream), so the Linears and the
    collectives are ordered on one stream and the whole step is one CUDA graph when capture succeeds.
    Strong scaling: the same model on N GPUs."""
    import torch
    from infr_b200 import synth

    Q4K, Q6K = infr_b200.Q4K, infr_b200.Q6K
    dev = torch.device("cuda", local)
    N = world
    n_layer, h, kvd, ff, vocab = 32, 4096, 1024, 14336, 128256
    shapes = [("wq", Q4K, h // N, h), ("wk", Q4K, kvd // N, h), ("wv", Q6K, kvd // N, h), ("wo", Q4K, h, h // N),
              ("gate", Q4K, ff // N, h), ("up", Q4K, ff // N, h), ("down", Q6K, h, ff // N)]
    nbytes = lambda dt, o, i: o * i // synth.BLOCK_ELEMS[dt] * synth.BLOCK_BYTES[dt]
    masters = {name: be.from_numpy(synth.random_blocks(dt, o * i, 300 + k), infr_b200.USAGE_WEIGHTS)
               for k, (name, dt, o, i) in enumerate(shapes)}
    layers = []
    for _ in range(n_layer):
        L = {}
        for name, dt, o, i in shapes:
            L[name] = be.alloc_uninit(nbytes(dt, o, i), infr_b200.USAGE_WEIGHTS)
            be.copy_buffer(masters[name], L[name], nbytes(dt, o, i))
        layers.append(L)
    head = be.from_numpy(synth.random_blocks(Q6K, (vocab // N) * h, 399), infr_b200.USAGE_WEIGHTS)
    total_bytes = n_layer * sum(nbytes(dt, o, i) for _, dt, o, i in shapes) + nbytes(Q6K, vocab // N, h)
    f32 = dict(dtype=torch.float32, device=dev)
    t = {"x_h": torch.randn(h, **f32), "x_hs": torch.randn(h // N, **f32), "x_ffs": torch.randn(ff // N, **f32),
         "y_q": torch.empty(h // N, **f32), "y_kv": torch.empty(kvd // N, **f32), "y_o": torch.empty(h, **f32),
         "y_ff": torch.empty(ff // N, **f32), "y_d": torch.empty(h, **f32), "logits": torch.empty(vocab // N, **f32)}
    gathered = torch.empty(vocab // N * N, **f32)
    torch.cuda.synchronize(dev)
    b = {k: be.wrap(v.data_ptr(), v.numel() * 4, infr_b200.USAGE_ACTIVATIONS) for k, v in t.items()}

    # the library's own small-message all-reduce over NVLink peer memory (one kernel on the context's stream)
    comm, ar_us = None, None
    if N > 1:
        comm = be.comm_create(rank, N, h)
        handles = [None] * N
        dist.all_gather_object(handles, comm.export())
        comm.connect(handles)
        _barrier(dist)  # every rank is connected before the first exchange
        # same sums as NCCL on random data before it is trusted with the timing
        probe = torch.randn(h, **f32)
        ref = probe.clone()
        torch.cuda.synchronize(dev)
        pw = be.wrap(probe.data_ptr(), h * 4, infr_b200.USAGE_ACTIVATIONS)
        be.all_reduce(comm, pw, h)
        be.sync()
        dist.all_reduce(ref)
        torch.cuda.synchronize(dev)
        err = float((probe - ref).abs().max() / ref.abs().max())
        assert err < 1e-6, f"peer-memory all-reduce differs from NCCL: {err}"
        # latency of one exchange, back to back on the stream
        ar_us = {}
        with torch.cuda.stream(torch.cuda.ExternalStream(be.stream(), device=dev)) as _:
            for name, fn in (("own", lambda: be.all_reduce(comm, pw, h)), ("nccl", lambda: dist.all_reduce(probe))):
                for _ in range(20):
                    fn()
                be.sync()
                _barrier(dist)
                be.timer_start()
                for _ in range(200):
                    fn()
                ar_us[name] = _max_over_ranks(dist, be.timer_stop()) * 1e3 / 200
        pw.close()

    def step(own):
        def reduce_(name):
            if N == 1 or own is None:
                return
            if own:
                be.all_reduce(comm, b[name], h)
            else:
                dist.all_reduce(t[name])
        for L in layers:
            be.linear(Q4K, L["wq"], b["x_h"], b["y_q"], 1, h, h // N)
            be.linear(Q4K, L["wk"], b["x_h"], b["y_kv"], 1, h, kvd // N)
            be.linear(Q6K, L["wv"], b["x_h"], b["y_kv"], 1, h, kvd // N)
            be.linear(Q4K, L["wo"], b["x_hs"], b["y_o"], 1, h // N, h)      # row-parallel: partial sums of the full vector
            reduce_("y_o")
            be.linear(Q4K, L["gate"], b["y_o"], b["y_ff"], 1, h, ff // N)
            be.linear(Q4K, L["up"], b["y_o"], b["y_ff"], 1, h, ff // N)
            be.linear(Q6K, L["down"], b["x_ffs"], b["y_d"], 1, ff // N, h)  # row-parallel
            reduce_("y_d")
        be.linear(Q6K, head, b["y_d"], b["logits"], 1, h, vocab // N)
        if N > 1:
            dist.all_gather_into_tensor(gathered, t["logits"])

    ext = torch.cuda.ExternalStream(be.stream(), device=dev)

    def timed(own):
        mode = "cuda graph"
        with torch.cuda.stream(ext):
            for _ in range(3):
                step(own)  # sizes the context's scratch before capture
            ext.synchronize()
            graph = None
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=ext):
                    step(own)
            except Exception as e:  # capture refused (collectives or stream rules): time the eager step
                graph, mode = None, f"eager ({type(e).__name__}: {str(e)[:80]})"
            run = graph.replay if graph is not None else (lambda: step(own))
            for _ in range(warmup):
                run()
            ext.synchronize()
            _barrier(dist)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ext)
            for _ in range(steps):
                run()
            e1.record(ext)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            del graph
        return _max_over_ranks(dist, ms) * 1e3 / steps, mode

    us, mode = timed(True)
    us_nccl = timed(False)[0] if N > 1 else None
    us_none = timed(None)[0] if N > 1 else None  # the ranks' Linears alone (no exchange: not a valid step, a floor)
    be.sync()  # a bounded wait that expired in the exchange surfaces here
    _barrier(dist)  # every rank has synchronised its last exchange before any rank frees its staging
    if comm is not None:
        comm.close()
    for v in list(b.values()) + list(masters.values()) + [head] + [x for L in layers for x in L.values()]:
        v.close()
    return {"workload": f"tensor-parallel Linear ops of an 8B-shape decode step, batch 1, {N} GPU(s): 225 Linears per rank "
                        f"({total_bytes / 1e9:.2f} GB of weights per rank), {2 * n_layer if N > 1 else 0} all-reduces of 16 KB "
                        f"(peer-memory kernel of this library) + 1 NCCL all-gather",
            "us_per_step": us, "tok_per_s_matmul_only": 1e6 / us, "mode": mode, "scaling": "strong",
            "us_per_step_with_nccl_all_reduce": us_nccl, "us_per_step_without_all_reduce": us_none, "all_reduce_16KB_us": ar_us if N > 1 else None,
            "not_included": "attention, norms, RoPE, sampling: see decode_step"}


def _tp_decode_step(be, infr_b200, dist, rank, world, local, batch, steps, warmup, pos=4096, exchange="fused"):
    """Tensor-parallel form of the WHOLE 8B-shape decode step (section of the reference: tp.rs:7-21): q/k/v by heads,
    attention by KV head on the rank's own slice of the KV cache, gate/up by FFN slice, o and down by input columns
    with an all-reduce of the [batch, 4096] result after each (the library's peer-memory kernel while it fits its
    64 K-float limit, NCCL otherwise), norms and the residual stream replicated, the head by vocabulary slice with one
    NCCL all-gather of the logits.  One CUDA graph on the backend's stream.  Strong scaling: one model on N GPUs.

    Every rank builds the SAME seeded model on the host and uploads its shard of it (rows of q/k/v/gate/up/head,
    input columns of o/down, its KV heads' columns of the caches).  Before anything is timed, rank 0 also runs the
    unsharded step on its own GPU and the gathered logits of the sharded step are compared with it."""
    import numpy as np
    import torch
    from infr_b200 import shard, synth
    from infr_b200.decode import DecodeStep, LlamaShape

    Q4K = infr_b200.Q4K
    dev = torch.device("cuda", local)
    N = world
    full = LlamaShape()
    # the FFN is cut in whole 2048-column chunks while there are enough of them (14336 = 7 chunks: 4 + 3 on two ranks,
    # 2 + 2 + 2 + 1 on four): a Q6_K `down` whose rows are whole chunks keeps the wide GEMV (rows of 14336 / N columns
    # are 5880 or 2940 bytes: no TMA stride), and an uneven cut costs less than the 8-row walk it avoids
    # With more ranks than chunks (8 ranks: 1792 columns each) the slice is padded to whole chunks with zero blocks
    # (2048: 14 % more bytes of gate / up / down, and every Linear keeps its fast kernel and the pushed exchange).
    ffn_unit = 2048 if full.ffn // 2048 >= N else 256
    ffn_of = lambda r, n: shard.ffn_split(full.ffn, n)[r][:2]
    ffn_pad = lambda r, n: shard.ffn_split(full.ffn, n)[r][2]
    s = LlamaShape(n_head=full.n_head // N, n_kv=full.n_kv // N, ffn=ffn_pad(rank, N), vocab=full.vocab // N)
    max_ctx = pos + 8
    row_parallel = {"wo", "down"}  # input columns split, partial sums all-reduced
    host_full = {name: synth.random_blocks(dt, o * i, 300 + k) for k, (name, dt, o, i) in enumerate(full.linears())}
    host_head = synth.random_blocks(Q4K, full.vocab * full.hidden, 399)
    norm_h = (1.0 + 0.02 * synth.normal(40, (full.hidden,))).astype(np.float32)
    kv_full = synth.normal(9, (max_ctx, full.kv_dim)).astype(np.float16).view(np.uint16)
    hidden_h = synth.normal(31, (batch, full.hidden))

    def build(shape, n_ranks, r):
        """Device buffers of rank r's share of the model split n_ranks ways (n_ranks = 1: the whole model)."""
        masters = {}
        f0, f1 = ffn_of(r, n_ranks)
        fp = ffn_pad(r, n_ranks)
        for name, dt, o, i in full.linears():
            if name == "down":
                w, _, _ = shard.col_shard(dt, host_full[name], o, i, r, n_ranks, unit=ffn_unit)
                if fp != f1 - f0:
                    w = shard.pad_cols(dt, w, o, f1 - f0, fp)
            elif name in row_parallel:
                w, _, _ = shard.col_shard(dt, host_full[name], o, i, r, n_ranks, unit=256)
            elif name in ("gate", "up"):  # the rows that feed this rank's columns of `down`
                bpr = synth.row_bytes(dt, i)
                w = np.ascontiguousarray(host_full[name]).reshape(-1)[f0 * bpr:f1 * bpr]
                if fp != f1 - f0:
                    w = shard.pad_rows(dt, w, f1 - f0, i, fp)
            else:
                w, _, _ = shard.row_shard(dt, host_full[name], o, i, r, n_ranks)
            masters[name] = be.from_numpy(w, infr_b200.USAGE_WEIGHTS)
        norm = be.from_numpy(norm_h)
        layers, owned, w_bytes = [], [], 0
        for _ in range(shape.n_layer):
            L = {"attn_norm": norm, "ffn_norm": norm}
            for name, dt, o, i in shape.linears():
                nbytes = o * i // synth.BLOCK_ELEMS[dt] * synth.BLOCK_BYTES[dt]
                b_ = be.alloc_uninit(nbytes, infr_b200.USAGE_WEIGHTS)
                be.copy_buffer(masters[name], b_, nbytes)
                L[name] = b_
                owned.append(b_)
                w_bytes += nbytes
            layers.append(L)
        hw, _, _ = shard.row_shard(Q4K, host_head, full.vocab, full.hidden, r, n_ranks)
        head = be.from_numpy(hw, infr_b200.USAGE_WEIGHTS)
        w_bytes += hw.nbytes
        kvd = shape.kv_dim
        kv_master = be.from_numpy(np.ascontiguousarray(kv_full[:, r * kvd:(r + 1) * kvd]))
        seq_bytes = max_ctx * kvd * 2
        kc, vc = [], []
        for _ in range(shape.n_layer):
            for lst in (kc, vc):
                c = be.alloc_uninit(batch * seq_bytes, infr_b200.USAGE_ACTIVATIONS)
                for q in range(batch):
                    view = be.wrap(c.device_ptr() + q * seq_bytes, seq_bytes, infr_b200.USAGE_ACTIVATIONS)
                    be.copy_buffer(kv_master, view, seq_bytes)
                    view.close()
                lst.append(c)
        be.sync()
        return dict(layers=layers, owned=owned + kc + vc + [head, kv_master, norm] + list(masters.values()), head=head, norm=norm, kc=kc, vc=vc,
                    w_bytes=w_bytes)

    # ---- the unsharded step on rank 0 (eager, once): the result the sharded step has to reproduce ----
    ref_logits = None
    if N > 1 and rank == 0:
        m1 = build(full, 1, 0)
        st1 = DecodeStep(be, full, batch, max_ctx, m1["layers"], m1["norm"], m1["head"], Q4K, m1["kc"], m1["vc"])
        st1.set_inputs(hidden_h, pos)
        st1.run(pos, fused=True)
        ref_logits = be.download(st1.logits, np.float32).reshape(batch, full.vocab)
        for b_ in m1["owned"]:
            b_.close()
        del st1, m1

    mine = build(s, N, rank)
    f32 = dict(device=dev, dtype=torch.float32)
    sub_t = torch.zeros(batch * s.hidden, **f32)
    gathered = torch.empty(batch * s.vocab * N, **f32)
    torch.cuda.synchronize(dev)
    sub = be.wrap(sub_t.data_ptr(), sub_t.numel() * 4, infr_b200.USAGE_ACTIVATIONS)
    n_red = batch * s.hidden
    comm = None
    if N > 1 and n_red <= 262144:
        comm = be.comm_create(rank, N, n_red)
        handles = [None] * N
        dist.all_gather_object(handles, comm.export())
        comm.connect(handles)
        _barrier(dist)  # every rank is connected before the first exchange
    if N == 1:
        reduce = None
    elif comm is not None:
        reduce = lambda buf, n: be.all_reduce(comm, buf, n)
    else:
        reduce = lambda buf, n: dist.all_reduce(sub_t)
    # exchange == "fused": at most 8 sequences push from the GEMV epilogues and sum in the norms (no exchange kernel);
    # "kernel": the stand-alone all-reduce after every row-parallel GEMV
    step = DecodeStep(be, s, batch, max_ctx, mine["layers"], mine["norm"], mine["head"], Q4K, mine["kc"], mine["vc"], sub=sub, reduce=reduce,
                      argmax=N == 1, comm=comm if exchange == "fused" else None)
    pushed = N > 1 and step._push_ok()
    hidden0 = be.from_numpy(hidden_h)
    step.set_inputs(hidden_h, pos)
    logits_t = None
    if N > 1:  # the rank's logits slice as a torch tensor for the all-gather: copy through a wrapped view
        logits_t = torch.empty(batch * s.vocab, **f32)
        torch.cuda.synchronize(dev)
        logits_w = be.wrap(logits_t.data_ptr(), logits_t.numel() * 4, infr_b200.USAGE_ACTIVATIONS)

    def one():
        be.copy_buffer(hidden0, step.hidden, batch * s.hidden * 4)
        n = step.run(pos, fused=True)
        if N > 1:
            be.copy_buffer(step.logits, logits_w, batch * s.vocab * 4)
            dist.all_gather_into_tensor(gathered, logits_t)
        return n

    ext = torch.cuda.ExternalStream(be.stream(), device=dev)
    mode = "cuda graph"
    parity = None
    with torch.cuda.stream(ext):
        for _ in range(2):
            n_ops = one()  # sizes the context's scratch before capture
        ext.synchronize()
        if N > 1 and rank == 0:
            # gathered is [rank][row][vocab / N]: rank r holds vocabulary rows [r * vocab / N, (r + 1) * vocab / N)
            got = gathered.cpu().numpy().reshape(N, batch, s.vocab).transpose(1, 0, 2).reshape(batch, full.vocab)
            rel = float(np.linalg.norm(got - ref_logits) / np.linalg.norm(ref_logits))
            parity = {"vs": "the unsharded step on one GPU, same seeded model", "logits_rel_l2": rel,
                      "max_abs_diff": float(np.abs(got - ref_logits).max()),
                      "same_argmax": bool((got.argmax(axis=1) == ref_logits.argmax(axis=1)).all()), "bar_rel_l2": 1e-3}
            parity["within_bar"] = bool(rel < 1e-3 and parity["same_argmax"])
            # 32 layers of random weights amplify an int8 rounding that flips with the summation order of the exchange:
            # the stated bar is reported, a result that is wrong (not merely reordered) stops the run
            assert np.isfinite(got).all() and rel < 5e-2, f"tensor-parallel step differs from the single-GPU step: {parity}"
            if not parity["within_bar"]:
                print(f"[bench] tensor-parallel parity outside the 1e-3 bar: {parity}", file=sys.stderr)
        graph = None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=ext):
                one()
        except Exception as e:
            graph, mode = None, f"eager ({type(e).__name__}: {str(e)[:80]})"
        run = graph.replay if graph is not None else one
        for _ in range(warmup):
            run()
        ext.synchronize()
        _barrier(dist)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ext)
        for _ in range(steps):
            run()
        e1.record(ext)
        e1.synchronize()
        ms = e0.elapsed_time(e1)
        del graph
    us = _max_over_ranks(dist, ms) * 1e3 / steps
    be.sync()
    _barrier(dist)  # every rank has synchronised its last exchange before any rank frees its staging
    if comm is not None:
        comm.close()
    for b_ in mine["owned"] + [hidden0, sub]:
        b_.close()
    return {"workload": f"tensor-parallel 8B-shape decode step, batch {batch}, KV context {pos}, {N} GPU(s): heads, FFN and vocabulary "
                        f"split over the ranks ({mine['w_bytes'] / 1e9:.2f} GB of weights per rank), {2 * s.n_layer if N > 1 else 0} all-reduces of "
                        f"{n_red * 4 // 1024} KB ({'pushed from the GEMV epilogues, summed in the norms: no exchange kernel' if pushed else 'peer-memory kernel' if comm is not None else 'NCCL' if N > 1 else 'none'}) + 1 NCCL all-gather",
            "us_per_step": us, "tok_per_s": batch / (us * 1e-6), "ops_per_step": n_ops, "mode": mode, "scaling": "strong",
            "parity": parity}


def _ep_moe(be, infr_b200, dist, rank, world, local, steps, warmup):
    """Expert-parallel form of the C4 MoE layer: every rank holds 128 / N experts and all 256 tokens, routes all
    tokens (the router is replicated), runs its experts' grouped GEMMs and adds its share of the output; the
    shares are summed by one NCCL all-reduce of the [256, 2048] f32 result (2 MB) on the backend's stream, the
    layer and the exchange in one CUDA graph.  With all tokens resident everywhere no token dispatch is needed;
    an all-to-all dispatch (tokens sharded) is not built.  Strong scaling: one layer on N GPUs."""
    import torch
    from infr_b200 import synth

    dev = torch.device("cuda", local)
    rows, ne, nx, nu, nff = 256, 2048, 128, 8, 768
    n_local = nx // world
    lo = rank * n_local
    # every rank builds the same seeded banks on the host and uploads the band of its experts
    banks = [synth.random_blocks(infr_b200.Q4K, nx * nff * ne, 100 + k) for k in range(3)]
    per_expert = nff * ne // 256 * 144
    band = lambda a: a[lo * per_expert:(lo + n_local) * per_expert]
    router_h = synth.normal(7, (nx, ne), 1.0 / np.sqrt(ne))
    x_h = synth.normal(8, (rows, ne))
    router = be.from_numpy(router_h)
    x = be.from_numpy(x_h)
    ref = None
    if world > 1 and rank == 0:
        # the unsharded layer on this GPU: what the sum of the ranks' shares has to reproduce
        fg, fu, fd = (be.from_numpy(a, infr_b200.USAGE_WEIGHTS) for a in banks)
        ref_b = be.alloc(rows * ne * 4)
        be.moe_ffn(x, x, router, fg, fu, fd, ref_b, rows=rows, ne=ne, n_expert=nx, n_used=nu, n_ff_exp=nff)
        ref = be.download(ref_b, np.float32)
        for b in (fg, fu, fd, ref_b):
            b.close()
    gate, up, down = (be.from_numpy(band(a), infr_b200.USAGE_WEIGHTS) for a in banks)
    del banks
    out_t = torch.zeros(rows * ne, dtype=torch.float32, device=dev)
    torch.cuda.synchronize(dev)
    dst = be.wrap(out_t.data_ptr(), rows * ne * 4, infr_b200.USAGE_ACTIVATIONS)
    kw = dict(rows=rows, ne=ne, n_expert=nx, n_used=nu, n_ff_exp=nff, expert_lo=lo, n_local=n_local)

    def step():
        be.moe_ffn(x, x, router, gate, up, down, dst, **kw)
        if world > 1:
            dist.all_reduce(out_t)

    ext = torch.cuda.ExternalStream(be.stream(), device=dev)
    mode = "cuda graph"
    parity = None
    with torch.cuda.stream(ext):
        for _ in range(3):
            step()
        ext.synchronize()
        if ref is not None:
            got = out_t.cpu().numpy()
            rel = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
            parity = {"vs": "the unsharded layer on one GPU, same seeded banks", "rel_l2": rel, "max_abs_diff": float(np.abs(got - ref).max()),
                      "bar_rel_l2": 1e-3}
            assert rel < 1e-3, f"expert-parallel layer differs from the single-GPU layer: {parity}"
        graph = None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=ext):
                step()
        except Exception as e:
            graph, mode = None, f"eager ({type(e).__name__}: {str(e)[:80]})"
        run = graph.replay if graph is not None else step
        for _ in range(warmup):
            run()
        ext.synchronize()
        _barrier(dist)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ext)
        for _ in range(steps):
            run()
        e1.record(ext)
        e1.synchronize()
        ms = e0.elapsed_time(e1)
        del graph
    us = _max_over_ranks(dist, ms) * 1e3 / steps
    be.sync()
    for b in (dst, gate, up, down, router, x):
        b.close()
    return {"workload": f"expert-parallel MoE layer, {world} GPU(s): 256 tok x hidden 2048, {n_local} of 128 experts per rank "
                        f"(2048->768->2048, Q4_K), softmax top-8, tokens replicated, 1 NCCL all-reduce of 2 MB",
            "us_per_layer": us, "mode": mode, "scaling": "strong", "parity": parity}


def _mmq_sharded(be, infr_b200, dist, rank, world, steps, warmup, peak_tops=None):
    """The prefill configuration (M = 512 tokens, K = 4096, N = 14336 Q4_K rows) split by output rows over the ranks
    (the column-parallel half of the reference's tensor-parallel lowering, crates/infr-llama/src/seam/mod.rs:2711-2798):
    rank r multiplies the same 512 activation rows, quantised redundantly on every rank, with rows
    [r * 14336 / N, (r + 1) * 14336 / N) of one seeded weight.  No collective: a consumer of the full result would
    all-gather.  Reports per-GPU and aggregate int8 TOPS; rank 0 checks its shard against the unsharded product."""
    from infr_b200 import shard, synth

    m, in_f, out_f = 512, 4096, 14336
    w = synth.random_blocks(infr_b200.Q4K, out_f * in_f, 5)
    x = synth.normal(6, (m, in_f))
    xb = be.from_numpy(x)
    ws, lo, cnt = shard.row_shard(infr_b200.Q4K, w, out_f, in_f, rank, world)
    wb = be.from_numpy(ws, infr_b200.USAGE_WEIGHTS)
    yb = be.alloc(m * cnt * 4)
    parity = None
    if world > 1 and rank == 0:
        fb, fy = be.from_numpy(w, infr_b200.USAGE_WEIGHTS), be.alloc(m * out_f * 4)
        be.linear(infr_b200.Q4K, fb, xb, fy, m, in_f, out_f)
        be.linear(infr_b200.Q4K, wb, xb, yb, m, in_f, cnt)
        full = be.download(fy, np.float32).reshape(m, out_f)[:, lo:lo + cnt]
        mine = be.download(yb, np.float32).reshape(m, cnt)
        rel = float(np.linalg.norm(mine - full) / np.linalg.norm(full))
        parity = {"vs": "the same rows of the unsharded product on one GPU", "rel_l2": rel, "bit_identical": bool((mine == full).all())}
        assert rel < 1e-5, parity
        fb.close()
        fy.close()
    del w
    for _ in range(warmup):
        be.linear(infr_b200.Q4K, wb, xb, yb, m, in_f, cnt)
    be.sync()
    _barrier(dist)
    be.timer_start()
    for _ in range(steps):
        be.linear(infr_b200.Q4K, wb, xb, yb, m, in_f, cnt)
    ms = _max_over_ranks(dist, be.timer_stop())
    us = ms * 1e3 / steps
    agg = 2.0 * m * in_f * out_f / (us * 1e-6) / 1e12
    res = {"workload": f"prefill MMQ q4_k M={m} K={in_f} N={out_f} split by output rows over {world} GPU(s) ({cnt} rows on rank 0), "
                       f"activations quantised on every rank, no collective",
           "us": us, "aggregate_tops": agg, "per_gpu_tops": agg / world, "scaling": "strong", "parity": parity}
    if peak_tops:
        res["per_gpu_frac_of_measured_int8_peak"] = agg / world / peak_tops
    for b in (wb, xb, yb):
        b.close()
    return res


# ------------------------------------------------------------------------------------------------
def run_b200(args):
    import infr_b200
    from infr_b200 import synth

    rank, world, local, dist = _dist_setup(args.gpus)
    hbm_peak, peak_src = _peaks()
    be = infr_b200.CudaBackend(device=local)
    caps = be.capabilities()
    steps, warmup = args.steps, max(args.warmup, 3)

    w = synth.weight(infr_b200.Q4K, OUT_F, IN_F, seed=0)
    x = synth.normal(1, (1, IN_F))
    first = be.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    ws = [first]
    for _ in range(ROT - 1):
        b = be.alloc_uninit(w.nbytes, infr_b200.USAGE_WEIGHTS)
        be.copy_buffer(first, b, w.nbytes)
        ws.append(b)
    xb = be.from_numpy(x)
    ys = [be.alloc(OUT_F * 4) for _ in range(ROT)]
    qs, d, s32 = be.alloc(IN_F), be.alloc(IN_F // 256 * 4), be.alloc(IN_F // 32 * 4)
    be.gemv(infr_b200.Q4K, ws[0], xb, ys[0], 1, IN_F, OUT_F)
    be.quantize_q8(256, xb, 1, IN_F, qs, d, s32)
    be.sync()

    # ---- device-resident pass: one graph = ROT x (quantise + GEMV) ----
    be.capture_begin()
    for i in range(ROT):
        be.gemv(infr_b200.Q4K, ws[i], xb, ys[i], 1, IN_F, OUT_F)
    g_full = be.capture_end()
    be.capture_begin()
    for i in range(ROT):
        be.gemv_q8(infr_b200.Q4K, ws[i], qs, d, s32, None, ys[i], 1, IN_F, OUT_F)
    g_kern = be.capture_end()

    sampler = ClockSampler(local)
    for _ in range(warmup):
        g_full.launch()
    be.sync()
    l0 = be.launch_count()
    with sampler:
        ms = _time_graph(be, g_full, steps, 0, dist)
    launches = be.launch_count() - l0  # kernels of this library inside the timed region (graph nodes x steps)
    ms = _max_over_ranks(dist, ms)
    with sampler:
        ms_kern = _time_graph(be, g_kern, steps, warmup, dist)
    ms_kern = _max_over_ranks(dist, ms_kern)

    # ---- end to end through the Backend interface with host buffers ----
    # The step as a caller of the trait issues it: ONE plan holding the step's ROT Linear ops (one input, one weight
    # and one output handle each), one upload of the step's inputs from pinned memory (ROT rows of x, 1 MB), one
    # execute, one download of the step's results to pinned memory (1 MB; download waits for the stream).  The handles
    # are views into one input and one output allocation, so that a copy serves all of them.
    g = infr_b200.Graph()
    xids = [g.input(IN_F) for _ in range(ROT)]
    wids = [g.weight(OUT_F * IN_F, infr_b200.Q4K) for _ in range(ROT)]
    dids = [g.output(OUT_F) for _ in range(ROT)]
    for i in range(ROT):
        g.linear(xids[i], wids[i], dids[i], 1, IN_F, OUT_F)
    plan = be.compile(g)
    x_all, y_all = be.alloc(ROT * IN_F * 4), be.alloc(ROT * OUT_F * 4)
    views = [be.wrap(x_all.device_ptr() + i * IN_F * 4, IN_F * 4, infr_b200.USAGE_ACTIVATIONS) for i in range(ROT)]
    views += [be.wrap(y_all.device_ptr() + i * OUT_F * 4, OUT_F * 4, infr_b200.USAGE_ACTIVATIONS) for i in range(ROT)]
    bound = {}
    for i in range(ROT):
        bound[xids[i]], bound[wids[i]], bound[dids[i]] = views[i], ws[i], views[ROT + i]
    bound = be.bind(bound)
    hx = be.host_array((ROT, IN_F), np.float32)
    hy = be.host_array((ROT, OUT_F), np.float32)
    hx[:] = x[0]
    e2e_steps = max(3, min(steps, 50))

    def e2e_pass():
        be.upload_raw(x_all, hx.ctypes.data, ROT * IN_F * 4)
        be.execute(plan, bound)
        be.download_raw(y_all, hy.ctypes.data, ROT * OUT_F * 4)

    for _ in range(3):
        e2e_pass()
    _barrier(dist)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    e2e_s = _max_over_ranks(dist, time.perf_counter() - t0)
    # the same kernel on the same inputs as the device-resident pass: the rows that came back are those results
    for i in (0, ROT - 1):
        assert np.array_equal(hy[i], be.download(ys[i], np.float32).reshape(-1)), "end-to-end pass differs from the device-resident pass"

    # one synchronous round trip per matrix (upload x, execute a one-Linear plan, download y): the latency of a
    # single call through the interface, reported beside the throughput above
    g1 = infr_b200.Graph()
    xid, wid, did = g1.input(IN_F), g1.weight(OUT_F * IN_F, infr_b200.Q4K), g1.output(OUT_F)
    g1.linear(xid, wid, did, 1, IN_F, OUT_F)
    plan1 = be.compile(g1)

    def call_pass():
        for i in range(ROT):
            be.upload_raw(xb, hx.ctypes.data, IN_F * 4)
            be.execute(plan1, {xid: xb, wid: ws[i], did: ys[i]})
            be.download_raw(ys[i], hy[i].ctypes.data, OUT_F * 4)

    call_pass()
    t0 = time.perf_counter()
    for _ in range(3):
        call_pass()
    call_us = _max_over_ranks(dist, time.perf_counter() - t0) * 1e6 / (3 * ROT)

    total_bytes = C1_BYTES * ROT * world
    value = total_bytes * steps / (ms * 1e-3) / 1e9
    kern_gbs = C1_BYTES * ROT * steps / (ms_kern * 1e-3) / 1e9
    out = {
        "metric": "Q4_K GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 activations x 4-bit weights, int32 block accumulate, f32 out",
        "data": "synthetic",
        "config": {"workload": f"Q4_K GEMV W 4096x4096 (fp32 N(0,0.02) seed 0 -> Q4_K), x fp32 [1,4096] N(0,1); "
                               f"step = one pass over {ROT} device copies at distinct addresses",
                   "l2": f"inputs larger than L2: {ROT * w.nbytes / 1e6:.0f} MB of weights per step vs {caps.l2_bytes / 1e6:.0f} MB L2",
                   "parallelism": (f"weak scaling: rank r holds rows [r*4096, (r+1)*4096) of each of {ROT} Q4_K matrices of {world * 4096} x 4096 "
                                   f"(output-row shards, activations replicated, no collective; sharded results are checked against one GPU "
                                   f"in mmq_sharded / tp_decode_step / ep_moe)") if world > 1 else "1 GPU",
                   "fraction_of_8TBs": value / world / 8000.0},
        "roofline": {"bound": "hbm", "achieved": kern_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": kern_gbs / hbm_peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of this kernel at this shape from the committed
                     # ncu capture (profiles/gemv_q4k_mma_4096x4096_m1.md): 9 467 136 + 0 bytes per launch
                     "traffic": 9467136, "peak_source": f"{peak_src} HBM copy bandwidth",
                     "kernel": "gemv_q4k_mma_kernel (m=1, pre-quantised activations)", "kernel_us": ms_kern * 1e3 / (steps * ROT),
                     "alg_bytes_per_launch": C1_BYTES},
        "e2e": {"value": total_bytes * e2e_steps / e2e_s / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": ROT * IN_F * 4, "d2h_bytes_per_step": ROT * OUT_F * 4,
                "ms_per_step": e2e_s * 1e3 / e2e_steps, "steps": e2e_steps,
                "how": f"per step: one upload of the step's {ROT} input rows from pinned memory, one execute of a plan of {ROT} Linear ops, "
                       f"one download of the {ROT} result rows to pinned memory (waits for the stream)",
                "round_trip_us_per_call": call_us},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(),
    }
    # a parity spot check travels with the number (GPU vs GPU-free expectation is in tests/)
    y0 = be.download(ys[0], np.float32)
    out["config"]["y_checksum"] = float(np.abs(y0).sum())

    if rank == 0 and world == 1 and not args.no_sweep:
        sweep = []
        sw_steps = max(20, min(steps, 100))
        for dtype, o, i_, seed, ms_ in ((infr_b200.Q4K, 14336, 4096, 5, (1, 4, 8)), (infr_b200.Q6K, 14336, 4096, 2, (1, 4, 8)),
                                        (infr_b200.Q2_0, 4096, 14336, 3, (1, 4, 8))):
            for m in ms_:
                sweep.append(_gemv_case(be, infr_b200, dtype, o, i_, m, seed, sw_steps, 5, caps.l2_bytes, hbm_peak))
        out["sweep"] = sweep
        out["int8_peak"] = _int8_peak(be)
        out["mmq"] = _mmq_case(be, infr_b200, 512, 4096, 14336, 5, 20, 3, out["int8_peak"])
        out["moe"] = _moe_case(be, infr_b200, 20, 3, hbm_peak)
        out["decode_linears"] = [_decode_linears_case(be, infr_b200, b, 10, 3) for b in (1, 32)]
        out["decode_step"] = [_decode_step_case(be, infr_b200, b, 10, 3, hbm_peak) for b in (1, 32)]

    if not args.no_sweep:
        peak_tops = out["int8_peak"]["burst_tops"] if "int8_peak" in out else _int8_peak(be)["burst_tops"]
        mq = _mmq_sharded(be, infr_b200, dist, rank, world, 20, 3, peak_tops)
        if rank == 0:
            out["mmq_sharded"] = mq
        tp = _tp_decode(be, infr_b200, dist, rank, world, local, 10, 3)
        ep = _ep_moe(be, infr_b200, dist, rank, world, local, 20, 3)
        tps = [_tp_decode_step(be, infr_b200, dist, rank, world, local, b_, 10, 3) for b_ in (1, 32)] if world > 1 else None
        if tps:  # batch 1 again with the stand-alone exchange kernel, to show what the fused form saves
            tps.append(_tp_decode_step(be, infr_b200, dist, rank, world, local, 1, 10, 3, exchange="kernel"))
        dps = None
        if world > 1:
            # data-parallel replicas: every rank holds the whole model and decodes its own 32 sequences (no exchange)
            mine = _decode_step_case(be, infr_b200, 32, 5, 3, hbm_peak)
            us_dp = _max_over_ranks(dist, mine["us_per_step"])
            dps = {"workload": f"{world} replicas of the 8B-shape decode step, batch 32 each, KV context 4096, no exchange",
                   "us_per_step": us_dp, "tok_per_s": world * 32 / (us_dp * 1e-6), "scaling": "weak"}
        if rank == 0:
            out["tp_decode"] = tp
            out["ep_moe"] = ep
            if tps:
                out["tp_decode_step"] = tps
                out["dp_decode_step"] = dps

    if rank == 0 and world == 1 and not args.no_cpu:
        out["cpu_baseline"] = _cpu_baseline(w, x, budget_s=10.0)

    be.close()
    if rank == 0:
        _emit(out)
    if dist is not None:
        dist.destroy_process_group()


def run_profile_case(args):
    """A few plain launches of one GEMV configuration (for an ncu capture on a small case):
    --profile-case DTYPE:OUT_F:IN_F:M, e.g. q4_k:14336:4096:1; weights rotate over > L2 of copies."""
    import infr_b200
    from infr_b200 import synth

    name, out_f, in_f, m = args.profile_case.split(":")
    if name == "moe":
        be = infr_b200.CudaBackend(device=0)
        _emit(_moe_case(be, infr_b200, args.steps, 2, _peaks()[0]))
        be.close()
        return
    if name == "decode":  # decode:0:0:BATCH — the Linear ops of an 8B-shape decode step
        be = infr_b200.CudaBackend(device=0)
        _emit(_decode_linears_case(be, infr_b200, int(m), args.steps, 2))
        be.close()
        return
    if name == "step":  # step:SHARD:CONTEXT:BATCH — the whole 8B-shape decode step (SHARD > 1: one rank's share of it)
        be = infr_b200.CudaBackend(device=0)
        _emit(_decode_step_case(be, infr_b200, int(m), args.steps, 2, _peaks()[0], pos=int(in_f) or 4096, shard=max(int(out_f), 1)))
        be.close()
        return
    if name == "mmq":  # mmq:OUT_F:IN_F:M — the prefill GEMM (Linear with m > 8)
        be = infr_b200.CudaBackend(device=0)
        _emit(_mmq_case(be, infr_b200, int(m), int(in_f), int(out_f), 5, args.steps, 2))
        be.close()
        return
    dtype = {v: k for k, v in synth.DTYPE_NAMES.items()}[name]
    out_f, in_f, m = int(out_f), int(in_f), int(m)
    be = infr_b200.CudaBackend(device=0)
    caps = be.capabilities()
    bufs, w = _rotation(be, infr_b200, dtype, out_f, in_f, 5, caps.l2_bytes + (32 << 20))
    if args.copies:
        bufs = bufs[:args.copies]
    x = synth.normal(6, (m, in_f))
    xb = be.from_numpy(x)
    yb = be.alloc(m * out_f * 4)
    gran = 32 if dtype == infr_b200.Q2_0 else 256
    qs, d = be.alloc(m * in_f), be.alloc(m * (in_f // gran) * 4)
    s32, s16 = be.alloc(m * (in_f // 32) * 4), be.alloc(m * (in_f // 16) * 4)
    be.quantize_q8(gran, xb, m, in_f, qs, d, s32, s16 if gran == 256 else None)
    be.timer_start()
    for i in range(args.steps):
        if m > 8:  # batches of a few dozen rows: the whole Linear (quantise + wide GEMV [+ sum of the K chunks])
            be.linear(dtype, bufs[i % len(bufs)], xb, yb, m, in_f, out_f)
        else:
            be.gemv_q8(dtype, bufs[i % len(bufs)], qs, d, s32, s16 if dtype == infr_b200.Q6K else None, yb, m, in_f, out_f)
    ms = be.timer_stop()
    _emit({"profile_case": args.profile_case, "launches": args.steps, "copies": len(bufs),
           "alg_bytes_per_launch": w.nbytes + 4 * m * (in_f + out_f), "us_per_launch_incl_host": ms * 1e3 / args.steps})
    be.close()


def _cpu_baseline(w, x, budget_s):
    from oracle.cpu_oracle import Oracle, Q4K

    orc = Oracle()
    threads = os.cpu_count() or 1
    orc.linear(Q4K, w, x, 1, IN_F, OUT_F, threads=threads)
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < budget_s and n < 1000000:
        orc.linear(Q4K, w, x, 1, IN_F, OUT_F, threads=threads)
        n += 1
    dt = time.perf_counter() - t0
    return {"value": C1_BYTES * n / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{n} Q4_K 4096x4096 matvecs (production int8 path of the C restatement of infr-cpu, "
                      f"quantise + integer dots, OpenMP over rows), {dt:.1f} s; the matrix stays in the CPU caches"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from infr_b200 import synth
    from oracle.cpu_oracle import Oracle, Q4K

    orc = Oracle()
    threads = os.cpu_count() or 1
    steps, warmup = args.steps, args.warmup
    # each step: a bounded sample of the pass — `per` matvecs over distinct copies of the matrix
    per = 8
    w = synth.weight(Q4K, OUT_F, IN_F, seed=0)
    ws = [w.copy() for _ in range(per)]
    x = synth.normal(1, (1, IN_F))
    for _ in range(max(warmup, 1)):
        for wi in ws:
            orc.linear(Q4K, wi, x, 1, IN_F, OUT_F, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        for wi in ws:
            orc.linear(Q4K, wi, x, 1, IN_F, OUT_F, threads=threads)
    dt = time.perf_counter() - t0
    value = C1_BYTES * per * steps / dt / 1e9
    sample = (f"per step {per} of the {ROT} Q4_K 4096x4096 matvecs (distinct copies), production int8 path of the "
              f"C restatement of infr-cpu on {threads} host threads; the Rust reference cannot be built (no Rust toolchain)")
    out = {"impl": "reference", "metric": "Q4_K GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
           "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3 / steps, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "int8 activations x 4-bit weights, int32 block accumulate, f32 out",
           "data": "synthetic",
           "config": {"workload": "Q4_K GEMV W 4096x4096, x fp32 [1,4096]; CPU arm, bounded sample per step"},
           "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    _emit(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--copies", type=int, default=0, help="with --profile-case: use only this many weight copies")
    ap.add_argument("--profile-case", default=None, help="DTYPE:OUT_F:IN_F:M — plain launches of one GEMV case")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


_RESULT_STREAM = None


def _emit(obj):
    """The one JSON line of the contract, on the process's original stdout."""
    stream = _RESULT_STREAM or sys.stdout
    print(json.dumps(obj), file=stream)
    stream.flush()


if __name__ == "__main__":
    # Libraries write banners to stdout (NCCL prints its version there when NCCL_DEBUG asks for it): everything but
    # the result line goes to stderr.
    sys.stdout.flush()
    _RESULT_STREAM = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    main()
