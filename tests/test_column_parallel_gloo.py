"""Host logic of the column-parallel layer on CPU: two gloo ranks, the per-shard computation done
by the CPU oracle. Checks shard bounds, the global column offset handed to the dual-uniform
selectors, and that the all-gather reassembles the row-major [M, N] result of the unsharded layer
(even and ragged shard widths)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from duqlinear4bitcuda_b200.parallel import gather_columns, shard_bounds
from tests import _util as U


def test_shard_bounds_cover_and_align():
    for n in (28672, 4096, 1000, 8, 20, 12288 + 8):
        for w in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(b % 8 == 0 for b, e in spans if e > b)
    assert shard_bounds(28672, 8, 3) == (10752, 14336)
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, n_out, mode, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as o
        M, K = 5, 128
        qa = U.rand_codes(M, K, 1); qw = U.rand_codes(n_out, K, 2)
        sr = U.rand_scales(M, 3); zr = U.rand_zeros(M, 4)
        sc1 = U.rand_scales(n_out, 5); zc1 = U.rand_zeros(n_out, 6); sc2 = U.rand_scales(n_out, 7); zc2 = U.rand_zeros(n_out, 8)
        bias = np.random.default_rng(9).standard_normal(n_out).astype(np.float16)
        b, e = shard_bounds(n_out, world, rank)
        _, local = o.linear_w4a4(mode, qa, qw[b:e], sr, zr, sc1[b:e], zc1[b:e], sc2[b:e], zc2[b:e], bias[b:e], col0=b)
        full = gather_columns(torch.from_numpy(local.view(np.int16).astype(np.int32)), n_out)   # gloo has no fp16: move the bits as int32
        _, want = o.linear_w4a4(mode, qa, qw, sr, zr, sc1, zc1, sc2, zc2, bias, col0=0)
        ok = np.array_equal(full.numpy(), want.view(np.int16).astype(np.int32))
        # a wrong (local) column offset must be visible in the dual schemes: the test has teeth
        _, wrong = o.linear_w4a4(mode, qa, qw[b:e], sr, zr, sc1[b:e], zc1[b:e], sc2[b:e], zc2[b:e], bias[b:e], col0=0)
        differs = rank == 0 or not np.array_equal(wrong.view(np.int16), local.view(np.int16))
        open(os.path.join(tmp, f"r{rank}"), "w").write(f"{int(ok)} {int(differs)}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_out,mode", [(48, "sym_dual"), (40, "asym_dual"), (64, "sym")])
def test_two_rank_gather_matches_unsharded(tmp_path, n_out, mode):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, n_out, mode, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok, differs = open(tmp_path / f"r{r}").read().split()
        assert ok == "1", f"rank {r}: gathered result differs from the unsharded layer"
        if mode != "sym":
            assert differs == "1"


# ---- row-parallel (K-sharded) host logic -------------------------------------------------------
def test_k_shard_bounds_cover_and_align():
    from duqlinear4bitcuda_b200.parallel import k_shard_bounds
    for k in (64, 128, 4096, 11008, 8192, 28672):
        for w in (1, 2, 3, 4, 8):
            spans = [k_shard_bounds(k, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == k
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(b % 64 == 0 and e % 64 == 0 for b, e in spans)
    assert k_shard_bounds(11008, 8, 7) == (9856, 11008)
    assert k_shard_bounds(128, 4, 3) == (128, 128)   # more ranks than 64-channel blocks: trailing ranks are empty
    with pytest.raises(ValueError):
        k_shard_bounds(100, 2, 0)


def _row_worker(rank, world, port, mode, k_in, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as o
        from duqlinear4bitcuda_b200.parallel import (global_asym_scale_zeros, global_sym_scale, k_shard_bounds,
                                                     reduce_partial_accumulators)
        M, N = 6, 40
        x = U.acts(M, k_in, 21, mean=0.2 if mode == "asym" else 0.0)
        qw = U.rand_codes(N, k_in, 22)
        sc = U.rand_scales(N, 23); zc = U.rand_zeros(N, 24)
        b, e = k_shard_bounds(k_in, world, rank)
        xs = x[:, b:e]
        # per-rank statistics of the slice -> all-reduce -> the unsharded quantizer's scale (and zero-point)
        if mode == "sym":
            amax = np.abs(xs).max(axis=1) if e > b else np.zeros(M, np.float16)
            s = global_sym_scale(torch.from_numpy(amax.astype(np.float16)), 1.0).numpy()
            z = None
            s_want = o.sym_scales(x, 1.0)
        else:
            mn = xs.min(axis=1) if e > b else np.full(M, np.inf, np.float16)
            mx = xs.max(axis=1) if e > b else np.full(M, -np.inf, np.float16)
            s, z = (t.numpy() for t in global_asym_scale_zeros(torch.from_numpy(mn.astype(np.float16)),
                                                               torch.from_numpy(mx.astype(np.float16))))
            s_want, z_want = o.asym_scales_zeros(x)
        ok_stats = U.bits_equal(s, s_want) and (z is None or U.bits_equal(z, z_want))
        # slice codes with the global scale, partial int32 GEMM, exact sum over ranks, one dequant
        if e > b:
            q = o.sym_quant(np.ascontiguousarray(xs), s) if mode == "sym" else o.asym_quant(np.ascontiguousarray(xs), s, z)
            acc = o.matmul_4bit(q, np.ascontiguousarray(qw[:, b // 2: e // 2]))
        else:
            acc = np.zeros((M, N), np.int32)
        acc = reduce_partial_accumulators(torch.from_numpy(acc.copy())).numpy()
        got = o.sym_dequant(acc, s, sc) if mode == "sym" else o.asym_dequant(acc, s, z, sc, zc)
        # the unsharded layer
        if mode == "sym":
            qa = o.sym_quant(x, s_want); _, want = o.linear_w4a4("sym", qa, qw, s_want, None, sc, None, None, None)
        else:
            qa = o.asym_quant(x, s_want, z_want); _, want = o.linear_w4a4("asym", qa, qw, s_want, z_want, sc, zc, None, None)
        ok = U.f16_equal_nan(got, want)
        open(os.path.join(tmp, f"r{rank}"), "w").write(f"{int(ok_stats)} {int(ok)}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,k_in,world", [("sym", 256, 2), ("asym", 192, 2), ("sym", 128, 3)])
def test_row_parallel_partial_sums_match_unsharded(tmp_path, mode, k_in, world):
    """K-sharded layer on gloo ranks (per-shard arithmetic by the CPU oracle): all-reduced row statistics
    reproduce the unsharded quantizer's scale / zero-point bit for bit, and int32 partial accumulators
    summed before the dequant reproduce the unsharded output bit for bit (ragged and empty K-slices
    included: 192 = 128 + 64; 128 over 3 ranks leaves rank 2 empty)."""
    port = _free_port()
    mp.spawn(_row_worker, args=(world, port, mode, k_in, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok_stats, ok = open(tmp_path / f"r{r}").read().split()
        assert ok_stats == "1", f"rank {r}: all-reduced statistics differ from the unsharded quantizer"
        assert ok == "1", f"rank {r}: row-parallel result differs from the unsharded layer"


# ---- host-resident job: one shared host result assembled from per-rank column slices ----------------
def _host_slice_worker(rank, world, port, n_out, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shared = None
    try:
        from oracle import oracle as o
        from duqlinear4bitcuda_b200.parallel import SharedHostTensor, host_result_slice
        M, K = 7, 128
        qa = U.rand_codes(M, K, 1); qw = U.rand_codes(n_out, K, 2)
        sr = U.rand_scales(M, 3); sc1 = U.rand_scales(n_out, 5); sc2 = U.rand_scales(n_out, 7)
        name = f"duq4_gloo_{port}_out"
        if rank == 0:
            shared = SharedHostTensor(name, (M, n_out), torch.float16, create=True, pin=False)
            shared.tensor.fill_(-3.0)
        dist.barrier()
        if rank != 0:
            shared = SharedHostTensor(name, (M, n_out), torch.float16, create=False, pin=False)
        b, e = shard_bounds(n_out, world, rank)
        _, local = o.linear_w4a4("sym_dual", qa, qw[b:e], sr, None, sc1[b:e], None, sc2[b:e], None, None, col0=b)
        # deliver the block the way the host-buffer entry point does: base pointer + byte offset, row pitch ldo
        byte_off, ldo, width = host_result_slice(n_out, world, rank)
        assert (byte_off, ldo, width) == (2 * b, n_out, e - b)
        flat = shared.tensor.view(-1).numpy()
        for r in range(M):
            start = byte_off // 2 + r * ldo
            flat[start:start + width] = local[r]
        dist.barrier()
        _, want = o.linear_w4a4("sym_dual", qa, qw, sr, None, sc1, None, sc2, None, None, col0=0)
        ok = np.array_equal(shared.tensor.numpy().view(np.uint16), want.view(np.uint16))
        open(os.path.join(tmp, f"r{rank}"), "w").write(str(int(ok)))
        dist.barrier()
    finally:
        if shared is not None:
            shared.close()
        dist.destroy_process_group()


@pytest.mark.parametrize("n_out,world", [(48, 2), (40, 2), (72, 3)])
def test_host_result_assembled_from_rank_slices(tmp_path, n_out, world):
    """Every rank maps the ONE host result (POSIX shared memory) and writes its column block at the offset and
    pitch `host_result_slice` gives; together the slices are the unsharded layer's row-major [M, N] output
    (even and ragged shard widths). Per-shard arithmetic by the CPU oracle."""
    port = _free_port()
    mp.spawn(_host_slice_worker, args=(world, port, n_out, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"r{r}").read() == "1", f"rank {r}"
    assert not os.path.exists(f"/dev/shm/duq4_gloo_{port}_out")
