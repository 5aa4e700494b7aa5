"""Two ranks on two GPUs (skipped on a one-GPU box): every rank runs its shard of a GEMM (columns of B
and C, A replicated) and of an MTTKRP (a range of the contraction index k) through the C ABI on its own
device, with device-resident buffers; the column slabs are gathered and the MTTKRP partials summed in
rank order over NCCL. No data-path collective is involved in the contractions themselves."""
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
        # ---- GEMM: bf16, N not divisible by 256 * world
        M, N, K = 1024, 1280, 512
        A, B = O.to_bf16(O.uniform(51, 1, (M, K))), O.to_bf16(O.uniform(51, 2, (K, N)))
        dA = torch.from_numpy(A.view(np.int16)).to(dev)
        dB = torch.from_numpy(B.view(np.int16)).to(dev)
        dC = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
        a = Buffer((K, M), "bf16")
        t2sp_b200.wrap_device(a, dA.data_ptr())
        _, b, c, (lo, hi) = shard.gemm_shard(a, dB.data_ptr(), dC.data_ptr(), "bf16", "f32", M, N, K, world, rank,
                                             on_device=True)
        assert t2sp_b200.gemm(a, b, c) == 0
        torch.cuda.synchronize()
        full = shard.gather_columns(dC[:, lo:hi].contiguous(), N, dist).cpu().numpy()
        truth = O.bf16_to_f32(A).astype(np.float64) @ O.bf16_to_f32(B).astype(np.float64)
        err_gemm = float(np.max(np.abs(full - truth)) / np.max(np.abs(truth)))
        untouched = bool(torch.isnan(dC[:, :lo]).all().item() and torch.isnan(dC[:, hi:]).all().item())
        # ---- MTTKRP: this rank's range of k, partials added in rank order
        L, I, Kd, R = 128, 256, 48, 64
        at, bt, ct = O.uniform(52, 1, (Kd, I, L)), O.uniform(52, 2, (R, Kd)), O.uniform(52, 3, (R, L))
        k0, k1 = shard.split_range(Kd, world, rank)
        part = np.full((R, I), np.nan, np.float32)
        pb = Buffer.from_numpy(part)
        assert t2sp_b200.mttkrp(Buffer.from_numpy(np.ascontiguousarray(at[k0:k1])),
                                Buffer.from_numpy(np.ascontiguousarray(bt[:, k0:k1])), Buffer.from_numpy(ct), pb) == 0
        total = shard.reduce_partials(torch.from_numpy(pb.keepalive).to(dev), dist, ordered=True).cpu().numpy()
        ref = O.mttkrp_f32(at, bt, ct, acc64=True)
        err_mttkrp = float(np.max(np.abs(total - ref)) / np.max(np.abs(ref)))
        q.put((rank, err_gemm, untouched, err_mttkrp, (lo, hi)))
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
    for rank, err_gemm, untouched, err_mttkrp, _ in results:
        assert err_gemm <= 1e-2 and untouched and err_mttkrp <= 1e-5, results
    assert results[0][4] == (0, 640) and results[1][4] == (640, 1280)
