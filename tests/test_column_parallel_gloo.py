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
