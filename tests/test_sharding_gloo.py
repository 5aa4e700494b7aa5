"""The multi-GPU host logic on CPU: two gloo ranks shard a GEMM by N-column slabs and an MTTKRP by
the contraction index, exactly as the GPU ranks do, with the CPU oracle standing in for the kernel
(the product has no CPU path). Checks the slab views (base pointer shift + full row pitch), the
column gather and the ordered reduction of partials."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import ctypes
    import torch
    import torch.distributed as dist
    from t2sp_b200 import shard
    from tests import oracle_lib as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- GEMM, N not divisible by the world size
        M, N, K = 24, 50, 40
        A, B = O.uniform(0, 1, (M, K)), O.uniform(0, 2, (K, N))
        C = np.zeros((M, N), np.float32)
        from t2sp_b200 import Buffer
        a = Buffer.from_numpy(A)
        _, b, c, (lo, hi) = shard.gemm_shard(a, B.ctypes.data, C.ctypes.data, "f32", "f32", M, N, K, world, rank)
        assert b.shape() == [(0, hi - lo, 1), (0, K, N)] and c.shape() == [(0, hi - lo, 1), (0, M, N)]
        # what the kernel would read/write through those views: gather the slab, compute, scatter back
        Bs = np.ctypeslib.as_array(ctypes.cast(b.raw.host, ctypes.POINTER(ctypes.c_float)), shape=(K * N - lo,))
        Bslab = np.lib.stride_tricks.as_strided(Bs, shape=(K, hi - lo), strides=(N * 4, 4)).copy()
        Cs = np.ctypeslib.as_array(ctypes.cast(c.raw.host, ctypes.POINTER(ctypes.c_float)), shape=(M * N - lo,))
        Cslab = np.lib.stride_tricks.as_strided(Cs, shape=(M, hi - lo), strides=(N * 4, 4))
        Cslab[:] = O.gemm_f32(A, Bslab)
        full = shard.gather_columns(torch.from_numpy(np.ascontiguousarray(C[:, lo:hi])), N, dist).numpy()
        ok_gemm = np.array_equal(full, O.gemm_f32(A, B)) and np.array_equal(C[:, lo:hi], full[:, lo:hi])
        # ---- MTTKRP sharded over the contraction index k: partials summed in rank order
        L, I, Kd, R = 16, 12, 10, 6
        at, bt, ct = O.uniform(1, 1, (Kd, I, L)), O.uniform(1, 2, (R, Kd)), O.uniform(1, 3, (R, L))
        k0, k1 = shard.split_range(Kd, world, rank)
        part = O.mttkrp_f32(np.ascontiguousarray(at[k0:k1]), np.ascontiguousarray(bt[:, k0:k1]), ct)
        total = shard.reduce_partials(torch.from_numpy(part), dist, ordered=True).numpy()
        ref = O.mttkrp_f32(at, bt, ct, acc64=True)
        ok_mttkrp = np.max(np.abs(total - ref)) / np.max(np.abs(ref)) < 1e-5
        q.put((rank, bool(ok_gemm), bool(ok_mttkrp), (lo, hi)))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_gather():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    results.sort()
    assert [r[0] for r in results] == [0, 1]
    assert all(r[1] and r[2] for r in results), results
    assert results[0][3] == (0, 25) and results[1][3] == (25, 50)


def test_split_range_covers_everything():
    from t2sp_b200.shard import split_range
    for total in (0, 1, 7, 64, 8192):
        for world in (1, 2, 3, 8):
            spans = [split_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
