"""Row (column-parallel) and column (row-parallel) sharding of a block-quantized weight across ranks.

The quantized matmul shards by OUTPUT rows with no exchange inside the op: rank r owns rows
[r*out_f/W, (r+1)*out_f/W) of the row-major [out_f, in_f] weight, whole GGUF blocks stay whole because a
row is a whole number of blocks, activations are replicated, and every rank produces its own slice of y.
This is the column-parallel half of the reference's tensor-parallel lowering
(crates/infr-llama/src/seam/mod.rs:2711-2798, `tp_slice_column`).  A collective is needed only where
the next consumer wants the full vector: `gather_rows` is that all-gather.
"""
from __future__ import annotations

import numpy as np

from .synth import row_bytes


def row_range(out_f: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous balanced row range of `rank` (the first out_f % world ranks get one extra row)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(out_f, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def row_shard(dtype: int, w_bytes: np.ndarray, out_f: int, in_f: int, rank: int, world: int) -> tuple[np.ndarray, int, int]:
    """(bytes of this rank's rows, first row, row count)."""
    bpr = row_bytes(dtype, in_f)
    w = np.ascontiguousarray(w_bytes, dtype=np.uint8).reshape(-1)
    if w.size != out_f * bpr:
        raise ValueError(f"weight holds {w.size} bytes, expected {out_f} rows x {bpr}")
    lo, hi = row_range(out_f, rank, world)
    return w[lo * bpr:hi * bpr], lo, hi - lo


def col_range(dtype: int, in_f: int, rank: int, world: int, unit: int = 0) -> tuple[int, int]:
    """Contiguous balanced range of INPUT columns of `rank`, in whole weight blocks (or multiples of `unit`
    elements when given: the activation quantiser's granule, 256 for Q4_K / Q6_K, must stay whole too so that a
    rank's int8 codes and scales are the unsharded ones).  This is the row-parallel half of the reference's
    tensor-parallel lowering (`tp_slice_row`, crates/infr-llama/src/seam/mod.rs:2711-2798): every rank multiplies
    its column slice with its slice of the activations and the partial results are summed (all-reduce)."""
    from .synth import BLOCK_ELEMS

    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    g = max(BLOCK_ELEMS[dtype], unit)
    if in_f % g:
        raise ValueError(f"in_f={in_f} is not a whole number of {g}-element granules")
    base, rem = divmod(in_f // g, world)
    lo = rank * base + min(rank, rem)
    return lo * g, (lo + base + (1 if rank < rem else 0)) * g


def col_shard(dtype: int, w_bytes: np.ndarray, out_f: int, in_f: int, rank: int, world: int, unit: int = 0) -> tuple[np.ndarray, int, int]:
    """(bytes of this rank's column slice as a dense [out_f, cols] weight, first column, column count)."""
    from .synth import BLOCK_BYTES, BLOCK_ELEMS

    bpr = row_bytes(dtype, in_f)
    w = np.ascontiguousarray(w_bytes, dtype=np.uint8).reshape(out_f, bpr)
    lo, hi = col_range(dtype, in_f, rank, world, unit)
    be, bb = BLOCK_ELEMS[dtype], BLOCK_BYTES[dtype]
    return np.ascontiguousarray(w[:, lo // be * bb:hi // be * bb]).reshape(-1), lo, hi - lo


def ffn_split(ffn: int, world: int, chunk: int = 2048, granule: int = 256) -> list[tuple[int, int, int]]:
    """How a tensor-parallel step cuts the FFN width over the ranks: per rank (first column, end column, padded width).
    While there are at least as many `chunk`-column pieces as ranks the cut is in whole chunks (uneven where they do
    not divide: 14336 = 7 chunks is 4 + 3 on two ranks, 2 + 2 + 2 + 1 on four), so that a rank's slice of a Q6_K `down`
    keeps rows the tiled copies can fetch; with more ranks than chunks the cut is in `granule`-column pieces (the
    activation quantiser's block) and every slice is padded up to whole chunks with zero blocks (pad_cols / pad_rows).
    One rank keeps the whole width unpadded."""
    if world < 1 or ffn % granule:
        raise ValueError(f"cannot split {ffn} columns over {world} ranks in pieces of {granule}")
    if world == 1:
        return [(0, ffn, ffn)]
    unit = chunk if ffn % chunk == 0 and ffn // chunk >= world else granule
    base, rem = divmod(ffn // unit, world)
    out, lo = [], 0
    for r in range(world):
        n = (base + (1 if r < rem else 0)) * unit
        out.append((lo, lo + n, -(-n // chunk) * chunk))
        lo += n
    return out


def pad_cols(dtype: int, w_bytes: np.ndarray, out_f: int, in_f: int, to: int) -> np.ndarray:
    """A dense [out_f, in_f] weight widened to `to` input columns with zero blocks (all-zero bytes are zero weights in
    Q4_K and Q6_K: d = 0).  A rank's column slice whose width is not one the fast kernels take (a Q6_K row must be whole
    2048-element chunks for the tiled copies) is padded instead of taking a slower kernel; the rows of the producer that
    feed the padding are zero rows (pad_rows), so the padded columns meet zero activations and add nothing."""
    from .synth import BLOCK_BYTES, BLOCK_ELEMS

    be, bb = BLOCK_ELEMS[dtype], BLOCK_BYTES[dtype]
    if to < in_f or to % be:
        raise ValueError(f"cannot pad {in_f} columns to {to}")
    w = np.ascontiguousarray(w_bytes, dtype=np.uint8).reshape(out_f, in_f // be * bb)
    out = np.zeros((out_f, to // be * bb), np.uint8)
    out[:, :w.shape[1]] = w
    return out.reshape(-1)


def pad_rows(dtype: int, w_bytes: np.ndarray, out_f: int, in_f: int, to: int) -> np.ndarray:
    """A dense [out_f, in_f] weight with zero rows appended up to `to` rows (their outputs are exactly 0)."""
    bpr = row_bytes(dtype, in_f)
    if to < out_f:
        raise ValueError(f"cannot pad {out_f} rows to {to}")
    out = np.zeros(to * bpr, np.uint8)
    out[:out_f * bpr] = np.ascontiguousarray(w_bytes, dtype=np.uint8).reshape(-1)[:out_f * bpr]
    return out


def gather_rows(dist, y_local: np.ndarray, out_f: int, rank: int, world: int) -> np.ndarray:
    """All-gather of the ranks' y slices [m, rows_r] into the full [m, out_f] (torch.distributed)."""
    import torch

    m = y_local.shape[0]
    counts = [row_range(out_f, r, world)[1] - row_range(out_f, r, world)[0] for r in range(world)]
    width = max(counts)
    pad = np.zeros((m, width), np.float32)
    pad[:, :y_local.shape[1]] = y_local
    mine = torch.from_numpy(pad)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    return np.concatenate([parts[r].numpy()[:, :counts[r]] for r in range(world)], axis=1)
