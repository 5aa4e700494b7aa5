"""The multi-GPU host logic on CPU: two gloo ranks shard every operator exactly as the GPU ranks do
(GEMM by columns, conv and capsule by batch items, TTM by j, MTTKRP by the contraction index k), with
the CPU oracle standing in for the kernel (the product has no CPU path). The slab views come from the
C library (t2sp_b200_shard_view: shifted base pointer, unchanged strides); the test reads and writes
memory only through them, then gathers and compares with the oracle on the unsharded problem."""
import ctypes
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


def as_array(buf):
    """numpy view (numpy order: Halide's last dimension first) of the host memory a Buffer describes."""
    n = buf.raw.dimensions
    shape = tuple(buf.dims[d].extent for d in reversed(range(n)))
    strides = tuple(buf.dims[d].stride * 4 for d in reversed(range(n)))
    span = 1 + sum((buf.dims[d].extent - 1) * buf.dims[d].stride for d in range(n))
    if min(shape) == 0:
        return np.zeros(shape, np.float32)
    flat = np.ctypeslib.as_array(ctypes.cast(buf.raw.host, ctypes.POINTER(ctypes.c_float)), shape=(span,))
    return np.lib.stride_tricks.as_strided(flat, shape=shape, strides=strides)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from t2sp_b200 import Buffer, shard
    from tests import oracle_lib as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = {}
    try:
        def gathered(local):
            parts = [None] * world
            dist.all_gather_object(parts, local)
            return parts

        # ---- GEMM, N not divisible by the world size: columns of B and C
        M, N, K = 24, 50, 40
        A, B = O.uniform(0, 1, (M, K)), O.uniform(0, 2, (K, N))
        C = np.zeros((M, N), np.float32)
        bv = shard.shard_view(Buffer.from_numpy(B), 0, 1, rank, world)
        cv = shard.shard_view(Buffer.from_numpy(C), 0, 1, rank, world)
        lo, hi = shard.split_range(N, world, rank)
        assert bv.shape() == [(0, hi - lo, 1), (0, K, N)] and cv.shape() == [(0, hi - lo, 1), (0, M, N)]
        as_array(cv)[:] = O.gemm_f32(A, np.ascontiguousarray(as_array(bv)))
        full = shard.gather_columns(torch.from_numpy(np.ascontiguousarray(C[:, lo:hi])), N, dist).numpy()
        ok["gemm"] = np.array_equal(full, O.gemm_f32(A, B)) and np.array_equal(C[:, lo:hi], full[:, lo:hi]) and \
            not C[:, :lo].any() and not C[:, hi:].any()
        span = (lo, hi)

        # ---- conv: batch items n; dimension 0 of I and O is (channel + channels * n)
        Nb, CI, CO, KY, KX, OY, OX = 5, 4, 6, 3, 2, 4, 3
        IY, IX = OY + KY - 1, OX + KX - 1
        I2, K2 = O.uniform(1, 1, (IY * IX, CI * Nb)), O.uniform(1, 2, (CI * KY, CO * KX))
        O2 = np.zeros((OY * OX, CO * Nb), np.float32)
        iv = shard.shard_view(Buffer.from_numpy(I2), 0, CI, rank, world)
        ov = shard.shard_view(Buffer.from_numpy(O2), 0, CO, rank, world)
        n0, n1 = shard.split_range(Nb, world, rank)
        assert iv.shape() == [(0, CI * (n1 - n0), 1), (0, IY * IX, CI * Nb)]
        as_array(ov)[:] = O.conv_f32(np.ascontiguousarray(as_array(iv)), K2, n1 - n0, CI, CO, KY, KX, OY, OX)
        total = sum(gathered(O2))
        ok["conv"] = np.array_equal(total, O.conv_f32(I2, K2, Nb, CI, CO, KY, KX, OY, OX))

        # ---- capsule: batch items n; dimension 1 of P and V is (pixel + pixels * n)
        Nb, NN, CI, CII, CO, KY, KX, OY, OX, Mx, s = 3, 2, 4, 4, 2, 3, 3, 2, 2, 4, 2
        IY, IX = s * OY + KY - s, s * OX + KX - s
        P2 = O.uniform(2, 1, (IY * IX * Nb, CI * Mx * Mx * NN))
        W2 = O.uniform(2, 2, (CI * KY * KX * Mx, CO * Mx))
        V2 = np.zeros((OY * OX * Nb, CO * Mx * Mx * NN), np.float32)
        pv = shard.shard_view(Buffer.from_numpy(P2), 1, IY * IX, rank, world)
        vv = shard.shard_view(Buffer.from_numpy(V2), 1, OY * OX, rank, world)
        n0, n1 = shard.split_range(Nb, world, rank)
        as_array(vv)[:] = O.capsule_f32(np.ascontiguousarray(as_array(pv)), W2, n1 - n0, NN, CI, CII, CO, KY, KX, OY, OX,
                                        Mx, Mx, Mx, s)
        total = sum(gathered(V2))
        ok["capsule"] = np.array_equal(total, O.capsule_f32(P2, W2, Nb, NN, CI, CII, CO, KY, KX, OY, OX, Mx, Mx, Mx, s))

        # ---- TTM: the j index of a(l,i,j) and c(i,j,k)
        L, I, J, Kt = 12, 6, 7, 5
        a, b = O.uniform(3, 1, (J, I, L)), O.uniform(3, 2, (Kt, L))
        c = np.zeros((Kt, J, I), np.float32)
        av = shard.shard_view(Buffer.from_numpy(a), 2, 1, rank, world)
        cv3 = shard.shard_view(Buffer.from_numpy(c), 1, 1, rank, world)
        j0, j1 = shard.split_range(J, world, rank)
        assert cv3.shape() == [(0, I, 1), (0, j1 - j0, I), (0, Kt, I * J)]
        as_array(cv3)[:] = O.ttm_f32(np.ascontiguousarray(as_array(av)), b)
        total = sum(gathered(c))
        ok["ttm"] = np.array_equal(total, O.ttm_f32(a, b))

        # ---- MTTKRP sharded over the contraction index k: partials summed in rank order
        L, I, Kd, R = 16, 12, 10, 6
        at, bt, ct = O.uniform(4, 1, (Kd, I, L)), O.uniform(4, 2, (R, Kd)), O.uniform(4, 3, (R, L))
        av = shard.shard_view(Buffer.from_numpy(at), 2, 1, rank, world)
        bv = shard.shard_view(Buffer.from_numpy(bt), 0, 1, rank, world)
        part = O.mttkrp_f32(np.ascontiguousarray(as_array(av)), np.ascontiguousarray(as_array(bv)), ct)
        total = shard.reduce_partials(torch.from_numpy(part), dist, ordered=True).numpy()
        ref = O.mttkrp_f32(at, bt, ct, acc64=True)
        ok["mttkrp"] = bool(np.max(np.abs(total - ref)) / np.max(np.abs(ref)) < 1e-5)
        q.put((rank, {k: bool(v) for k, v in ok.items()}, span))
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
    results.sort(key=lambda r: r[0])
    assert [r[0] for r in results] == [0, 1]
    for r in results:
        assert set(r[1]) == {"gemm", "conv", "capsule", "ttm", "mttkrp"} and all(r[1].values()), results
    assert results[0][2] == (0, 25) and results[1][2] == (25, 50)


def test_split_range_covers_everything():
    from t2sp_b200.shard import split_range
    for total in (0, 1, 7, 64, 8192):
        for world in (1, 2, 3, 8):
            spans = [split_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1


def test_shard_entries_validate_before_touching_a_device():
    """Argument checks of the sharded entries run on the host: wrong world, tiled layouts and units that do not
    divide the extent are refused with halide error codes (no device is needed to get that far)."""
    import t2sp_b200
    from t2sp_b200 import Buffer, shard
    A = Buffer.from_numpy(np.zeros((8, 4), np.float32))
    B = Buffer.from_numpy(np.zeros((4, 6), np.float32))
    C = Buffer.from_numpy(np.zeros((8, 6), np.float32))
    assert shard.gemm_shard(A, B, C, rank=2, world=2) == -8       # constraint_violated: rank outside the world
    d = t2sp_b200.GemmDesc()
    d.layout = 1
    assert shard.gemm_shard(A, B, C, 0, 2, d) == -8
    cd = t2sp_b200.ConvDesc()
    cd.CI, cd.CO, cd.KY, cd.KX, cd.OY, cd.OX = 4, 4, 1, 1, 2, 2
    I = Buffer.from_numpy(np.zeros((4, 10), np.float32))          # 10 is not a whole number of 4-channel images
    assert shard.conv_shard(I, B, C, cd, 0, 2) == -8
    with pytest.raises(ValueError):
        shard.shard_view(A, 5, 1, 0, 2)
