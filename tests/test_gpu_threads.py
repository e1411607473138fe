"""Two host threads, each with its own stream, enter the library at the same moment in a fresh process, so
that the once-per-device set-up of every kernel (shared-memory opt-ins, occupancy queries, the TMA descriptor
cache, the driver entry point look-up) is reached concurrently. Both threads must get the oracle's results.
(The static-scratch entry point is excluded: its one array per GPU is shared by design.)"""
import os
import subprocess
import sys

import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu

CHILD = r'''
import ctypes, sys, threading
import numpy as np
import torch
sys.path.insert(0, %(root)r)
import duqlinear4bitcuda_b200.lib as L
from oracle import oracle as o
from tests import _util as U

shapes = [(1, 1000, 4096), (16, 9600, 4096), (40, 520, 1024), (300, 520, 256), (2000, 2100, 384)]   # every kernel family
start = threading.Barrier(2)
errors = []

def work(tid):
    try:
        torch.cuda.set_device(0)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            st = ctypes.c_void_p(stream.cuda_stream)
            cases = []
            for i, (M, N, K) in enumerate(shapes if tid == 0 else shapes[::-1]):
                qa = U.rand_codes(M, K, 10 * tid + i); qw = U.rand_codes(N, K, 100 + 10 * tid + i)
                sr = U.rand_scales(M, 3, 0.01, 0.3); sc = U.rand_scales(N, 4)
                t = [torch.from_numpy(v).cuda() for v in (qa, qw, sr, sc)]
                out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
                acc = torch.zeros((M, N), dtype=torch.int32, device="cuda")
                cases.append((qa, qw, sr, sc, t, out, acc, M, N, K))
            stream.synchronize()
            start.wait()                      # both threads hit their first launches together
            for rep in range(3):
                for (qa, qw, sr, sc, t, out, acc, M, N, K) in cases:
                    epi = L.make_epilogue("sym", t[2], None, t[3])
                    L.call("duq4_linear_w4a4", L.ptr(t[0]), L.ptr(t[1]), M, N, K, ctypes.byref(epi), L.ptr(out), L.ptr(acc), st)
            stream.synchronize()
            for (qa, qw, sr, sc, t, out, acc, M, N, K) in cases:
                acc_w, out_w = o.linear_w4a4("sym", qa, qw, sr, None, sc, None, None, None)
                assert np.array_equal(acc.cpu().numpy(), acc_w), (tid, M, N, K)
                assert U.f16_equal_nan(out.cpu().numpy(), out_w), (tid, M, N, K)
    except Exception as ex:   # report through the main thread
        errors.append(repr(ex))
        try:
            start.abort()
        except Exception:
            pass

ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
[t.start() for t in ts]
[t.join() for t in ts]
status = ctypes.c_int32(-1)
L.call("duq4_last_device_status", None, ctypes.byref(status))
assert not errors, errors
assert status.value == 0, status.value
print("threads ok")
'''


def test_two_host_threads_two_streams_first_use_race():
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": U.ROOT}], capture_output=True, text=True, cwd=U.ROOT, timeout=600)
    assert r.returncode == 0 and "threads ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
