"""Row sharding across ranks, exercised with two gloo ranks on CPU.

Each rank takes its row slice of a Q4_K / Q6_K weight, multiplies with the CPU restatement (the GPU is
not needed to check the partition and the gather) and the gathered result must equal the unsharded one
bit for bit — the op has no cross-rank arithmetic.
"""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, dt, out_f, in_f, m, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from infr_b200 import shard, synth
    from oracle.cpu_oracle import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        w = synth.weight(dt, out_f, in_f, seed=3)
        x = synth.normal(4, (m, in_f))
        mine, lo, n = shard.row_shard(dt, w, out_f, in_f, rank, world)
        y_local = orc.linear(dt, mine, x, m, in_f, n, threads=2)
        full = shard.gather_rows(dist, y_local, out_f, rank, world)
        want = orc.linear(dt, w, x, m, in_f, out_f, threads=2)
        q.put((rank, bool((full.view(np.uint32) == want.view(np.uint32)).all()), lo, n))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dt,out_f,in_f,m", [(12, 37, 512, 2), (14, 64, 256, 1)])
def test_row_shards_gather_to_the_unsharded_result(dt, out_f, in_f, m):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + dt) % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, dt, out_f, in_f, m, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in res)
    assert res[0][2] == 0 and res[0][2] + res[0][3] == res[1][2] and res[1][2] + res[1][3] == out_f


def _col_worker(rank, world, port, dt, out_f, in_f, m, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from infr_b200 import shard, synth
    from oracle.cpu_oracle import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        w = synth.weight(dt, out_f, in_f, seed=5)
        x = synth.normal(6, (m, in_f))
        mine, lo, n = shard.col_shard(dt, w, out_f, in_f, rank, world, unit=256)
        part = torch.from_numpy(orc.linear(dt, mine, np.ascontiguousarray(x[:, lo:lo + n]), m, n, out_f, threads=2))
        dist.all_reduce(part)  # the exchange of a row-parallel Linear
        want = orc.linear(dt, w, x, m, in_f, out_f, threads=2)
        rel = float(np.linalg.norm(part.numpy() - want) / np.linalg.norm(want))
        q.put((rank, rel, lo, n))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dt,out_f,in_f,m", [(12, 24, 1024, 2), (14, 16, 768, 1)])
def test_column_shards_sum_to_the_unsharded_result(dt, out_f, in_f, m):
    # whole 256-element granules per rank: every block term is the unsharded one, only the f32 sum order differs
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() + dt) % 2000
    procs = [ctx.Process(target=_col_worker, args=(r, 2, port, dt, out_f, in_f, m, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(rel < 1e-6 for _, rel, _, _ in res), res
    assert res[0][2] == 0 and res[0][2] + res[0][3] == res[1][2] and res[1][2] + res[1][3] == in_f


def test_col_range_keeps_blocks_and_granules_whole():
    sys.path.insert(0, ROOT)
    from infr_b200 import shard

    for dt, in_f, unit in ((12, 4096, 256), (14, 14336, 256), (27, 14336, 64), (27, 14336, 512)):
        for world in (1, 2, 4, 8):
            spans = [shard.col_range(dt, in_f, r, world, unit) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == in_f
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(a % unit == 0 and b % unit == 0 for a, b in spans)
    with pytest.raises(ValueError):
        shard.col_range(12, 4096 + 128, 0, 2)


def test_row_range_is_a_balanced_partition():
    sys.path.insert(0, ROOT)
    from infr_b200 import shard

    for out_f in (1, 7, 4096, 14336, 128256):
        for world in (1, 2, 3, 8):
            spans = [shard.row_range(out_f, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == out_f
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.row_range(10, 2, 2)


@pytest.mark.parametrize("dt", [12, 14])
def test_zero_padding_of_a_column_slice_changes_nothing(dt):
    """A slice of 1792 columns widened to 2048 with zero blocks (and its producer with zero rows): the padded product
    against zero-padded activations has the bits of the unpadded one, and the producer's extra rows are exactly 0."""
    sys.path.insert(0, ROOT)
    from infr_b200 import shard, synth
    from oracle.cpu_oracle import Oracle

    orc = Oracle()
    out_f, in_f, to, m = 24, 1792, 2048, 2
    w = synth.weight(dt, out_f, in_f, seed=5)
    x = synth.normal(6, (m, in_f))
    wp = shard.pad_cols(dt, w, out_f, in_f, to)
    xp = np.zeros((m, to), np.float32)
    xp[:, :in_f] = x
    want = orc.linear(dt, w, x, m, in_f, out_f, threads=2)
    got = orc.linear(dt, wp, xp, m, to, out_f, threads=2)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    # the producer side: rows appended to a [in_f_rows, k] weight give zeros
    k = 512
    g = synth.weight(dt, in_f, k, seed=7)
    gp = shard.pad_rows(dt, g, in_f, k, to)
    y = orc.linear(dt, gp, synth.normal(8, (1, k)), 1, k, to, threads=2)
    assert not y[0, in_f:].any() and y[0, :in_f].any()
    with pytest.raises(ValueError):
        shard.pad_cols(dt, w, out_f, in_f, 1024)


def test_ffn_split_of_a_tensor_parallel_step():
    sys.path.insert(0, ROOT)
    from infr_b200 import shard

    assert shard.ffn_split(14336, 1) == [(0, 14336, 14336)]
    assert [hi - lo for lo, hi, _ in shard.ffn_split(14336, 2)] == [8192, 6144]          # 4 + 3 chunks
    assert [hi - lo for lo, hi, _ in shard.ffn_split(14336, 4)] == [4096, 4096, 4096, 2048]
    eight = shard.ffn_split(14336, 8)                                                     # more ranks than chunks
    assert all(hi - lo == 1792 and pad == 2048 for lo, hi, pad in eight)
    for world in (1, 2, 3, 4, 7, 8):
        parts = shard.ffn_split(14336, world)
        assert parts[0][0] == 0 and parts[-1][1] == 14336
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert all(lo % 256 == 0 and hi % 256 == 0 and pad % 2048 == 0 and pad >= hi - lo and pad - (hi - lo) < 2048 for lo, hi, pad in parts)
        if world > 1:
            # what a rank's Q6_K `down` needs for the tiled copies: rows of whole 2048-column chunks
            assert all(pad % 2048 == 0 for _, _, pad in parts)
    assert [hi - lo for lo, hi, _ in shard.ffn_split(11008, 4)] == [2816, 2816, 2816, 2560]  # 5.375 chunks: cut in 256-column granules, padded
    assert all(pad == 4096 for _, _, pad in shard.ffn_split(11008, 4))
    with pytest.raises(ValueError):
        shard.ffn_split(1000, 2)
