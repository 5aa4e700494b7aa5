"""Python front of the library's multi-GPU entries (include/t2sp_b200/runtime.h, csrc/multigpu.cpp):
sharding of the contractions over the GPUs of one box, one process per GPU.

The reference is single-device (its runtime opens devices[0] only,
t2s/src/AOT-OpenCL-Runtime.cpp:186-213); this is how the same calls scale out here. Every rank
calls the same entry with its rank and the world size on full-size buffers and works on its slab:

  gemm     columns of B and C        (A replicated)
  conv     batch items n             (weights replicated)
  capsule  batch items n             (weights replicated)
  ttm      the j index of a(l,i,j)   (b replicated)
  mttkrp   the k index (contraction) -> every rank holds a full-size partial d; the ONE exchange
           step of the whole scheme is the sum of those partials

A slab is the same memory with a shifted base pointer and unchanged strides, which is exactly what a
halide_buffer_t (and the TMA descriptor made from it) describes, so shards are views, not copies.
The slab arithmetic and the NCCL exchange steps live in the C library so that C hosts can use them;
this module only forwards, and offers torch.distributed forms of the two exchange steps for hosts
that already run a process group."""
import ctypes

from . import lib
from .halide import Buffer, HalideBuffer, HalideDimension


def _bind():
    L = lib()
    if getattr(L, "_shard_bound", False):
        return L
    P, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    L.t2sp_b200_split_range.argtypes = [i64, i32, i32, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    L.t2sp_b200_split_range.restype = None
    L.t2sp_b200_shard_view.argtypes = [P, i32, i32, i32, i32, P, P]
    for name, nbuf in (("gemm", 3), ("conv", 3), ("capsule", 3), ("ttm", 3), ("mttkrp", 4)):
        fn = getattr(L, f"t2sp_b200_{name}_shard")
        fn.argtypes = [P] * (nbuf + 1) + [i32, i32]
        fn.restype = ctypes.c_int
    L.t2sp_b200_nccl_unique_id.argtypes = [P, i32]
    L.t2sp_b200_comm_init.argtypes = [ctypes.POINTER(P), i32, P, i32]
    L.t2sp_b200_comm_destroy.argtypes = [P]
    L.t2sp_b200_gather_columns.argtypes = [P, P, i32, i32]
    L.t2sp_b200_reduce_partials.argtypes = [P, P, i32, i32, i32]
    L.t2sp_b200_broadcast.argtypes = [P, P, i32]
    L._shard_bound = True
    return L


def split_range(total, world, rank):
    """Contiguous near-equal split of range(total); the first total % world ranks get one extra."""
    lo, hi = ctypes.c_int64(), ctypes.c_int64()
    _bind().t2sp_b200_split_range(total, world, rank, ctypes.byref(lo), ctypes.byref(hi))
    return lo.value, hi.value


def shard_view(buf, dim, unit, rank, world):
    """This rank's slab of `buf` along dimension `dim` (in groups of `unit` indices) as a new Buffer
    that shares the memory. Raises on a halide error code."""
    out = Buffer([0] * buf.raw.dimensions, buf.dtype, keepalive=buf)
    rc = _bind().t2sp_b200_shard_view(buf.ptr, dim, unit, rank, world, ctypes.byref(out.raw),
                                      ctypes.cast(out.dims, ctypes.c_void_p))
    if rc != 0:
        raise ValueError(f"t2sp_b200_shard_view failed with halide error {rc}")
    out.extents = tuple(out.dims[d].extent for d in range(out.raw.dimensions))
    return out


def _desc(d):
    return ctypes.byref(d) if d is not None else None


def gemm_shard(A, B, C, rank, world, desc=None):
    """This rank's columns of C = A x B; B and C are the full-size buffers."""
    return _bind().t2sp_b200_gemm_shard(A.ptr, B.ptr, C.ptr, _desc(desc), rank, world)


def conv_shard(I, K, O, desc, rank, world):
    return _bind().t2sp_b200_conv_shard(I.ptr, K.ptr, O.ptr, _desc(desc), rank, world)


def capsule_shard(P, W, V, desc, rank, world):
    return _bind().t2sp_b200_capsule_shard(P.ptr, W.ptr, V.ptr, _desc(desc), rank, world)


def ttm_shard(a, b, c, rank, world, desc=None):
    return _bind().t2sp_b200_ttm_shard(a.ptr, b.ptr, c.ptr, _desc(desc), rank, world)


def mttkrp_shard(a, b, c, d_partial, rank, world, desc=None):
    return _bind().t2sp_b200_mttkrp_shard(a.ptr, b.ptr, c.ptr, d_partial.ptr, _desc(desc), rank, world)


class Comm:
    """An NCCL communicator made by the library for this rank's device. `exchange_id(id_bytes)` must hand
    rank 0's 128-byte id to every rank (e.g. a torch.distributed broadcast) and return it."""

    def __init__(self, rank, world, exchange_id):
        L = _bind()
        self.rank, self.world = rank, world
        raw = ctypes.create_string_buffer(128)
        if rank == 0:
            rc = L.t2sp_b200_nccl_unique_id(raw, 128)
            if rc != 0:
                raise RuntimeError(f"t2sp_b200_nccl_unique_id failed with halide error {rc}")
        idb = exchange_id(bytes(raw.raw))
        self.handle = ctypes.c_void_p()
        rc = L.t2sp_b200_comm_init(ctypes.byref(self.handle), world, ctypes.c_char_p(idb), rank)
        if rc != 0:
            raise RuntimeError(f"t2sp_b200_comm_init failed with halide error {rc}")

    def gather_columns(self, C):
        return _bind().t2sp_b200_gather_columns(C.ptr, self.handle, self.rank, self.world)

    def reduce_partials(self, d, ordered=True):
        return _bind().t2sp_b200_reduce_partials(d.ptr, self.handle, self.rank, self.world, 1 if ordered else 0)

    def broadcast(self, buf, root=0):
        return _bind().t2sp_b200_broadcast(buf.ptr, self.handle, root)

    def destroy(self):
        if self.handle:
            _bind().t2sp_b200_comm_destroy(self.handle)
            self.handle = ctypes.c_void_p()


def torch_id_exchange(dist, device=None):
    """exchange_id for Comm over an existing torch.distributed process group."""
    def exchange(idb):
        import torch
        t = torch.tensor(list(idb), dtype=torch.uint8, device=device or "cpu")
        dist.broadcast(t, src=0)
        return bytes(t.cpu().tolist())
    return exchange


# ---- torch.distributed forms of the exchange steps (any backend, e.g. gloo on CPU) ----------
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
