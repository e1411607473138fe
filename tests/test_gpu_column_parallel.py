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
    import ctypes
    import torch
    import torch.distributed as dist
    import duqlinear4bitcuda_b200.lib as L
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
        y_fused = layer(x, gather="fused").clone()   # epilogue stores instead of the collective
        y_mc = layer(x, gather="fused_multicast").clone()   # one multimem.st per row segment where the switch offers a multicast mapping
        y_fused2 = layer(x, gather="fused").clone()  # reuse of the shared buffer
        y_peer = layer(x, gather="fused_peer").clone()   # one plain store per peer
        y_copy = layer(x, gather="copy").clone()         # local epilogue + copy-engine peer copies per row chunk
        y_copy2 = layer(x, gather="copy").clone()
        torch.cuda.synchronize()
        status = ctypes.c_int32(-1)
        L.call("duq4_last_device_status", L.current_stream(), ctypes.byref(status))
        # the unsharded layer on this GPU alone
        single = ColumnParallelLinear4bit(mode, N, qw, sc1, zc1 if asym else None, sc2 if dual else None,
                                          zc2 if mode == "asym_dual" else None, bias, unsharded=True)
        y1 = single(x)
        torch.cuda.synchronize()
        ok = torch.equal(y.view(torch.int16), y1.view(torch.int16)) and tuple(y.shape) == (M, N)
        ok = ok and torch.equal(y_fused.view(torch.int16), y1.view(torch.int16)) and torch.equal(y_mc.view(torch.int16), y1.view(torch.int16))
        ok = ok and torch.equal(y_fused2.view(torch.int16), y1.view(torch.int16))
        ok = ok and torch.equal(y_peer.view(torch.int16), y1.view(torch.int16)) and status.value == 0
        ok = ok and torch.equal(y_copy.view(torch.int16), y1.view(torch.int16)) and torch.equal(y_copy2.view(torch.int16), y1.view(torch.int16))
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


def _barrier_timeout_worker(rank, world, port, tmp):
    import ctypes
    import torch
    import torch.distributed as dist
    import duqlinear4bitcuda_b200.lib as L
    from duqlinear4bitcuda_b200.parallel import PeerOutput
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        peer = PeerOutput(8, 64, dev, use_multicast=False, barrier_timeout_ns=200_000_000)   # 0.2 s limit
        st = L.current_stream

        def status():
            v = ctypes.c_int32(-1)
            L.call("duq4_last_device_status", st(), ctypes.byref(v))   # synchronises the stream
            return v.value

        peer.barrier(); s1 = status()                     # everybody arrives: no time-out
        peer.barrier(arrive=(rank != 1)); s2 = status()   # rank 1 stays away (a host decision): the others' wait runs out
        flag = torch.tensor([s2], device=dev)
        seen = [torch.zeros_like(flag) for _ in range(world)]
        dist.all_gather(seen, flag)                       # nobody leaves while another rank still waits
        if rank == 1:
            peer.catch_up()                               # publish the missed epoch
        torch.cuda.synchronize(); dist.barrier()
        peer.barrier(); s3 = status()                     # the barrier is usable again
        want2 = 0 if rank == 1 else 301
        ok = s1 == 0 and s2 == want2 and s3 == 0 and [int(t.item()) for t in seen] == [301 if r != 1 else 0 for r in range(world)]
        open(os.path.join(tmp, f"r{rank}"), "w").write(f"{int(ok)} {s1} {s2} {s3}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_peer_barrier_times_out_instead_of_hanging(tmp_path, monkeypatch):
    """The library's device-side barrier has a bounded wait: when a rank is told (on the host) not to arrive,
    the other rank's barrier kernel gives up after its limit, the status word reads 301, the context stays
    usable and the next barrier works. Nothing traps or hangs; every rank stays until all have reported.
    Runs on plain peer loads/stores with NVLink multicast switched off in NCCL and in torch's symmetric memory."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    monkeypatch.setenv("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    world, port = 2, _free_port()
    mp.spawn(_barrier_timeout_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"r{r}").read().split()[0] == "1", (r, open(tmp_path / f"r{r}").read())


def _host_worker(rank, world, port, mode, M, N, K, tmp):
    import ctypes
    import torch
    import torch.distributed as dist
    import duqlinear4bitcuda_b200.lib as L
    from duqlinear4bitcuda_b200.parallel import ColumnParallelLinear4bit, SharedHostTensor
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    xh = oh = None
    try:
        dev = torch.device("cuda", rank)
        t = lambda a: torch.from_numpy(a).to(dev)
        qw = t(U.rand_codes(N, K, 2)); sc1 = t(U.rand_scales(N, 3)); zc1 = t(U.rand_zeros(N, 4))
        bias = t(np.random.default_rng(7).standard_normal(N).astype(np.float16))
        asym = mode == "asym"
        layer = ColumnParallelLinear4bit.from_full(mode, qw, sc1, zc1 if asym else None, None, None, bias)
        # ONE host input and ONE host result for the job, mapped and pinned by every rank
        if rank == 0:
            xh = SharedHostTensor(f"duq4_test_{port}_x", (M, K), torch.float16, create=True)
            oh = SharedHostTensor(f"duq4_test_{port}_o", (M, N), torch.float16, create=True)
            xh.tensor.copy_(torch.from_numpy(U.acts(M, K, 1, mean=0.1 if asym else 0.0)))
            oh.tensor.fill_(-3.0)
        dist.barrier()
        if rank != 0:
            xh = SharedHostTensor(f"duq4_test_{port}_x", (M, K), torch.float16, create=False)
            oh = SharedHostTensor(f"duq4_test_{port}_o", (M, N), torch.float16, create=False)
        # the whole layer on this GPU alone through the same host entry point
        single = ColumnParallelLinear4bit(mode, N, qw, sc1, zc1 if asym else None, None, None, bias, unsharded=True)
        want = torch.empty((M, N), dtype=torch.float16).pin_memory()
        single.forward_host(xh.tensor, want)
        torch.cuda.synchronize()
        ok = True
        # "rows": rows exchanged over NVLink by the epilogue, each rank downloads the contiguous rows it owns;
        # "columns": each rank downloads its column block. Twice each: staging, exchange buffers, flags and helper
        # streams are reused.
        for delivery, chunk in (("rows", 256), ("rows", 0), ("columns", 256), ("rows", 256)):
            if rank == 0:
                oh.tensor.fill_(-3.0)
            dist.barrier()
            layer.forward_host(xh.tensor, oh.tensor, chunk_rows=chunk, delivery=delivery)
            torch.cuda.synchronize()
            dist.barrier()
            ok = ok and torch.equal(oh.tensor.view(torch.int16), want.view(torch.int16))
            dist.barrier()
        status = ctypes.c_int32(-1)
        L.call("duq4_last_device_status", L.current_stream(), ctypes.byref(status))
        ok = ok and status.value == 0
        open(os.path.join(tmp, f"r{rank}"), "w").write(str(int(ok)))
        dist.barrier()
    finally:
        for h in (xh, oh):
            if h is not None:
                h.close()
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,M,N,K", [("sym", 8, 4096, 4096), ("asym", 701, 1040, 512), ("sym", 2048, 8192, 256)])
def test_two_gpu_host_result_assembled_by_slices_matches_single_gpu(tmp_path, mode, M, N, K):
    """Host-resident job on 2 GPUs: each rank uploads its row slice of the one shared pinned host input (ragged: 701
    rows), the slices are all-gathered over NVLink, and each rank delivers its column block into its slice of the one
    shared host result -- as contiguous rows after an exchange over NVLink written by the GEMM epilogue (default), or
    as its own column block; the assembled result equals the 1-GPU host entry point bit for bit (packed weights at 8
    tokens, the pre-laid-out int8 copy from 256 tokens on)."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, port = 2, _free_port()
    mp.spawn(_host_worker, args=(world, port, mode, M, N, K, str(tmp_path)), nprocs=world, join=True)
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
        y = layer(x[:, b:e]).clone()                 # fused: library pieces, partial sums stored to the owners, one dequant
        y_again = layer(x[:, b:e]).clone()           # the symmetric buffers are reused
        y_comp = layer(x[:, b:e], fused=False)       # composed from the reference-named operators + int32 all-reduce
        torch.cuda.synchronize()
        single = ColumnParallelLinear4bit(mode, N, qw, sc, zc if mode == "asym" else None, None, None, bias, unsharded=True)
        y1 = single(x)
        torch.cuda.synchronize()
        ok = torch.equal(y.view(torch.int16), y1.view(torch.int16)) and tuple(y.shape) == (M, N)
        ok = ok and torch.equal(y_again.view(torch.int16), y1.view(torch.int16)) and torch.equal(y_comp.view(torch.int16), y1.view(torch.int16))
        open(os.path.join(tmp, f"r{rank}"), "w").write(str(int(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,M,N,K", [("sym", 8, 4096, 11008), ("asym", 301, 1040, 1024), ("sym", 512, 2048, 4096), ("asym", 3, 264, 64)])
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
