"""Sharding of the contractions over the GPUs of one box, one process per GPU.

The reference is single-device (its runtime opens devices[0] only,
t2s/src/AOT-OpenCL-Runtime.cpp:186-213); this is how the same calls scale out here. Every
operator has an independent output dimension, so ranks work on disjoint output slabs from
disjoint (or replicated) inputs and the data path needs no collective:

  GEMM     columns of B and C        (A replicated)
  conv     batch items n             (weights replicated)
  capsule  batch items n             (weights replicated)
  TTM      the j index of a(l,i,j)   (b replicated)
  MTTKRP   the k index (contraction) -> every rank holds a full partial d; the ONE exchange
           step of the whole scheme is the sum of those partials (all_reduce, or an ordered
           gather + sum when bitwise reproducibility across runs matters)

A slab of a column-sharded matrix is the same memory with a shifted base pointer and the full
row pitch, which is exactly what a halide_buffer_t (and the TMA descriptor made from it) can
describe, so shards are views, not copies. Results are gathered with torch.distributed only when
the caller wants them on every rank."""
import numpy as np

from .halide import Buffer, DTYPES


def split_range(total, world, rank):
    """Contiguous near-equal split of range(total); the first total % world ranks get one extra."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _elem_bytes(dtype):
    return (DTYPES[dtype][1] + 7) // 8


def column_slab_view(ptr, dtype, n_total, rows, lo, hi, on_device):
    """Halide view of columns [lo, hi) of a dense row-major (rows x n_total) matrix at `ptr`."""
    base = ptr + lo * _elem_bytes(dtype)
    if on_device:
        b = Buffer((hi - lo, rows), dtype, strides=(1, n_total))
        from . import wrap_device
        wrap_device(b, base)
        return b
    return Buffer((hi - lo, rows), dtype, host=base, strides=(1, n_total))


def gemm_shard(A, B_ptr, C_ptr, in_dtype, out_dtype, M, N, K, world, rank, on_device=False):
    """Buffers for this rank's part of C = A x B: all of A, columns [lo, hi) of B and C."""
    lo, hi = split_range(N, world, rank)
    b = column_slab_view(B_ptr, in_dtype, N, K, lo, hi, on_device)
    c = column_slab_view(C_ptr, out_dtype, N, M, lo, hi, on_device)
    return A, b, c, (lo, hi)


def gather_columns(local, N, dist):
    """all_gather of per-rank column slabs (torch tensors of shape [M, hi-lo]) into [M, N] on every rank."""
    import torch
    world = dist.get_world_size()
    M = local.shape[0]
    widths = [split_range(N, world, r)[1] - split_range(N, world, r)[0] for r in range(world)]
    wmax = max(widths)
    padded = torch.zeros((M, wmax), dtype=local.dtype, device=local.device)
    padded[:, :local.shape[1]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[:, :w] for p, w in zip(parts, widths)], dim=1)


def reduce_partials(local_partial, dist, ordered=True):
    """Sum of the per-rank MTTKRP partial results. ordered=True gathers and adds in rank order so
    that the fp32 result does not depend on the reduction tree; otherwise a plain all_reduce."""
    import torch
    if not ordered:
        out = local_partial.clone()
        dist.all_reduce(out)
        return out
    parts = [torch.empty_like(local_partial) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, local_partial)
    acc = parts[0].clone()
    for p in parts[1:]:
        acc += p
    return acc
