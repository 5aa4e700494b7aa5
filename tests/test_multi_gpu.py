"""Two ranks on two GPUs (skipped on a one-GPU box): every rank runs its shard of a GEMM (columns of B
and C, A replicated), of an MTTKRP (a range of the contraction index k) and of a convolution (batch
items) through the library's sharded C entries on its own device; the column slabs are gathered and the
MTTKRP partials summed in rank order by the library's NCCL entries (t2sp_b200_gather_columns,
t2sp_b200_reduce_partials). No data-path collective is involved in the contractions themselves."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    import t2sp_b200
    from t2sp_b200 import Buffer, shard
    from tests import oracle_lib as O
    torch.cuda.set_device(rank)
    lib = t2sp_b200.lib()
    assert lib.t2sp_b200_set_device(rank) == 0
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        comm = shard.Comm(rank, world, shard.torch_id_exchange(dist, dev))   # the library's own NCCL communicator
        # ---- GEMM: bf16, N not divisible by 256 * world; full-size device buffers, the entry takes its columns
        M, N, K = 1024, 1280, 512
        A, B = O.to_bf16(O.uniform(51, 1, (M, K))), O.to_bf16(O.uniform(51, 2, (K, N)))
        dA = torch.from_numpy(A.view(np.int16)).to(dev)
        dB = torch.from_numpy(B.view(np.int16)).to(dev)
        dC = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
        a, b, c = Buffer((K, M), "bf16"), Buffer((N, K), "bf16"), Buffer((N, M), "f32")
        for buf, t in ((a, dA), (b, dB), (c, dC)):
            t2sp_b200.wrap_device(buf, t.data_ptr())
        assert shard.gemm_shard(a, b, c, rank, world) == 0
        torch.cuda.synchronize()
        lo, hi = shard.split_range(N, world, rank)
        untouched = bool(torch.isnan(dC[:, :lo]).all().item() and torch.isnan(dC[:, hi:]).all().item())
        assert comm.gather_columns(c) == 0                                   # ncclAllGather of the column slabs
        full = dC.cpu().numpy()
        truth = O.bf16_to_f32(A).astype(np.float64) @ O.bf16_to_f32(B).astype(np.float64)
        err_gemm = float(np.max(np.abs(full - truth)) / np.max(np.abs(truth)))
        # ---- MTTKRP: this rank's range of k from the full-size operands, partials added in rank order
        L, I, Kd, R = 128, 256, 48, 64
        at, bt, ct = O.uniform(52, 1, (Kd, I, L)), O.uniform(52, 2, (R, Kd)), O.uniform(52, 3, (R, L))
        dD = torch.full((R, I), float("nan"), dtype=torch.float32, device=dev)
        d = Buffer((I, R), "f32")
        t2sp_b200.wrap_device(d, dD.data_ptr())
        assert shard.mttkrp_shard(Buffer.from_numpy(at), Buffer.from_numpy(bt), Buffer.from_numpy(ct), d, rank, world) == 0
        assert comm.reduce_partials(d, ordered=True) == 0
        total = dD.cpu().numpy()
        ref = O.mttkrp_f32(at, bt, ct, acc64=True)
        err_mttkrp = float(np.max(np.abs(total - ref)) / np.max(np.abs(ref)))
        # ---- conv by batch items on host buffers: each rank fills its images of the full-size output
        Nb, CI, CO, KY, KX, OY, OX = 6, 64, 64, 3, 3, 6, 6
        IY, IX = OY + KY - 1, OX + KX - 1
        I2, K2 = O.uniform(53, 1, (IY * IX, CI * Nb)), O.uniform(53, 2, (CI * KY, CO * KX))
        O2 = np.zeros((OY * OX, CO * Nb), np.float32)
        cd = t2sp_b200.ConvDesc()
        cd.CI, cd.CO, cd.KY, cd.KX, cd.OY, cd.OX = CI, CO, KY, KX, OY, OX
        assert shard.conv_shard(Buffer.from_numpy(I2), Buffer.from_numpy(K2), Buffer.from_numpy(O2), cd, rank, world) == 0
        parts = [None] * world
        dist.all_gather_object(parts, O2)
        refc = O.conv_f32(I2, K2, Nb, CI, CO, KY, KX, OY, OX, acc64=True)
        err_conv = float(np.max(np.abs(sum(parts) - refc)) / np.max(np.abs(refc)))
        comm.destroy()
        q.put((rank, err_gemm, untouched, err_mttkrp, (lo, hi), err_conv))
    finally:
        dist.destroy_process_group()


def test_two_gpus_sharded_gemm_and_mttkrp():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results.sort()
    print(results)
    for rank, err_gemm, untouched, err_mttkrp, _, err_conv in results:
        assert err_gemm <= 1e-2 and untouched and err_mttkrp <= 1e-5 and err_conv <= 1e-5, results
    assert results[0][4] == (0, 640) and results[1][4] == (640, 1280)
