"""Column-parallel layer on 2 GPUs (NCCL): the gathered result must be bit-identical to the
same layer computed on one GPU. Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, mode, M, N, K, tmp):
    import torch
    import torch.distributed as dist
    from duqlinear4bitcuda_b200.parallel import ColumnParallelLinear4bit
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        x = torch.from_numpy(U.acts(M, K, 1, mean=0.1 if "asym" in mode else 0.0)).to(dev)
        t = lambda a: torch.from_numpy(a).to(dev)
        qw = t(U.rand_codes(N, K, 2)); sc1 = t(U.rand_scales(N, 3)); zc1 = t(U.rand_zeros(N, 4))
        sc2 = t(U.rand_scales(N, 5)); zc2 = t(U.rand_zeros(N, 6))
        bias = t(np.random.default_rng(7).standard_normal(N).astype(np.float16))
        asym, dual = mode.startswith("asym"), mode.endswith("dual")
        layer = ColumnParallelLinear4bit.from_full(mode, qw, sc1, zc1 if asym else None, sc2 if dual else None,
                                                   zc2 if mode == "asym_dual" else None, bias)
        y = layer(x)
        torch.cuda.synchronize()
        y_fused = layer(x, gather="fused").clone()   # epilogue peer stores instead of the collective
        y_fused2 = layer(x, gather="fused").clone()  # reuse of the shared buffer
        torch.cuda.synchronize()
        # the unsharded layer on this GPU alone
        single = ColumnParallelLinear4bit(mode, N, qw, sc1, zc1 if asym else None, sc2 if dual else None,
                                          zc2 if mode == "asym_dual" else None, bias, unsharded=True)
        y1 = single(x)
        torch.cuda.synchronize()
        ok = torch.equal(y.view(torch.int16), y1.view(torch.int16)) and tuple(y.shape) == (M, N)
        ok = ok and torch.equal(y_fused.view(torch.int16), y1.view(torch.int16))
        ok = ok and torch.equal(y_fused2.view(torch.int16), y1.view(torch.int16))
        open(os.path.join(tmp, f"r{rank}"), "w").write(str(int(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,M,N,K", [("sym", 8, 4096, 4096), ("sym_dual", 300, 1040, 512), ("asym_dual", 64, 2048, 1024),
                                        ("sym", 2048, 4096, 256), ("asym", 2000, 4200, 192)])   # the last two: CTA-pair kernel per rank
def test_two_gpu_column_parallel_matches_single_gpu(tmp_path, mode, M, N, K):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, mode, M, N, K, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"r{r}").read() == "1", f"rank {r}"


def _row_worker(rank, world, port, mode, M, N, K, tmp):
    import torch
    import torch.distributed as dist
    from duqlinear4bitcuda_b200.parallel import ColumnParallelLinear4bit, RowParallelLinear4bit, k_shard_bounds
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        x = torch.from_numpy(U.acts(M, K, 11, mean=0.1 if mode == "asym" else 0.0)).to(dev)
        t = lambda a: torch.from_numpy(a).to(dev)
        qw = t(U.rand_codes(N, K, 12)); sc = t(U.rand_scales(N, 13)); zc = t(U.rand_zeros(N, 14))
        bias = t(np.random.default_rng(15).standard_normal(N).astype(np.float16))
        layer = RowParallelLinear4bit.from_full(mode, qw, sc, zc if mode == "asym" else None, bias)
        b, e = k_shard_bounds(K, world, rank)
        y = layer(x[:, b:e])
        torch.cuda.synchronize()
        single = ColumnParallelLinear4bit(mode, N, qw, sc, zc if mode == "asym" else None, None, None, bias, unsharded=True)
        y1 = single(x)
        torch.cuda.synchronize()
        ok = torch.equal(y.view(torch.int16), y1.view(torch.int16)) and tuple(y.shape) == (M, N)
        open(os.path.join(tmp, f"r{rank}"), "w").write(str(int(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,M,N,K", [("sym", 8, 4096, 11008), ("asym", 300, 1040, 1024), ("sym", 512, 2048, 4096)])
def test_two_gpu_row_parallel_matches_single_gpu(tmp_path, mode, M, N, K):
    """K-sharded layer (int32 partial accumulators all-reduced before the dequant) == the whole layer
    on one GPU, bit for bit."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, port = 2, _free_port()
    mp.spawn(_row_worker, args=(world, port, mode, M, N, K, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"r{r}").read() == "1", f"rank {r}"
