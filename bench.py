#!/usr/bin/env python
"""Benchmark of the W4A4 linear hot path (per-token int4 quantize -> int4 GEMM -> dequant).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward of one W4A4 linear layer over a batch of synthetic tokens:
fp16 activations [M,K] -> fused per-token symmetric quantize -> int4 x int4 -> int32 GEMM on
tcgen05 tensor cores -> fp16 dequant epilogue, at the Llama-70B MLP up-projection shape
K=8192 -> N=28672 with M=4096 tokens (the M=4096 point of the headline metric). The M=1
point (decode, Llama-2-7B shapes, weight-bandwidth bound) is measured in the same run and
reported under "decode". With --gpus N > 1 the layer is column-sharded over N ranks (one
process per GPU, NCCL all-gather of the fp16 output shards) -- total work fixed: "strong".

`value` is timed with inputs resident in HBM; `e2e` is the same layer through the C-ABI
entry point with the activations coming from pinned host memory and the output going back
to it inside the timed region. `--impl reference` times the CPU restatement of the
reference arithmetic (oracle/) on the host cores over a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K_IN, N_OUT, M_TOK = 8192, 28672, 4096
DECODE_SHAPES = [(4096, 12288), (4096, 4096), (4096, 22016), (11008, 4096)]  # (K, N), Llama-2-7B
NOMINAL_HBM_GBS, NOMINAL_INT8_TOPS = 8000.0, 4500.0
WORKLOAD = f"prefill_llama70b_mlp_up_K{K_IN}_N{N_OUT}_M{M_TOK}_sym_w4a4"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle-reason samples taken (read-only, through NVML) while the timed
    region runs; a sample every few milliseconds from a helper thread."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.sm, self.bits, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._t = None
        self.err = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.idx < len(ids) and ids[self.idx].isdigit():
                return int(ids[self.idx])
        return self.idx

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as ex:  # NVML missing: report that instead of clocks
            self.err = f"nvml unavailable: {type(ex).__name__}"
            return
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception:
                pass
            time.sleep(0.003)

    def stop(self):
        if self._t is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err or "not sampled"]}
        self._stop.set()
        self._t.join(timeout=2)
        reasons = sorted(n for b, n in self.REASONS.items() if self.bits & b)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.sm), "reasons": reasons}


# ------------------------------------------------------------------------------------------
def synth_activations(torch, M, K, seed, pinned=True):
    """fp16 ~N(0,1) with 1% of the K channels scaled x20 (outliers); seeded on the CPU."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g, dtype=torch.float32)
    ch = torch.randperm(K, generator=g)[: K // 100]
    x[:, ch] *= 20.0
    x = x.to(torch.float16)
    return x.pin_memory() if pinned else x


def synth_weights(torch, N, K, seed, device):
    """Random-init weights ~N(0,0.015), per-output-channel symmetric int4 (scale = absmax/7,
    clamp [-8,7]), packed two per byte. Built on the GPU in row chunks."""
    from duqlinear4bitcuda_b200.tools.quantization import pack_i4
    g = torch.Generator(device=device).manual_seed(seed)
    qw = torch.empty((N, K // 2), dtype=torch.uint8, device=device)
    sw = torch.empty((N,), dtype=torch.float16, device=device)
    for r0 in range(0, N, 4096):
        r1 = min(N, r0 + 4096)
        w = (torch.randn((r1 - r0, K), generator=g, device=device, dtype=torch.float32) * 0.015).to(torch.float16)
        s = (w.abs().amax(dim=1, keepdim=True).float() / 7.0).to(torch.float16)
        q = torch.clamp(torch.round(w / s), -8, 7).to(torch.int8)
        qw[r0:r1] = pack_i4(q)
        sw[r0:r1] = s.view(-1)
    return qw, sw


_CPU_STATE = {}


def cpu_baseline(sample_rows=None, threads=None, budget_s=12.0):
    """CPU baselines on a bounded sample: the first `rows` tokens of the same workload against the full weight
    matrix, on all host cores. Two implementations of the reference's arithmetic are timed:
      reference-python : the reference's PyTorch fake-quant / integer-matmul path restated in torch ops
                         (oracle/torch_path.py: per-token scale, round/clamp, pack_i4, unpack_i4, the integer
                         contraction as a float matmul, fp16 dequant) -- the headline `value`;
      port             : the C restatement of the reference's CUDA kernels (oracle/duq_oracle.c, OpenMP).
    The weights are unpacked once outside the timed region in the torch path (a module holds its weights
    prepared); the C port reads the packed weights."""
    import numpy as np
    import torch
    from oracle import oracle as o
    from oracle import torch_path as tp
    threads = threads or os.cpu_count()
    os.environ["OMP_NUM_THREADS"] = str(threads)
    torch.set_num_threads(threads)
    state = _CPU_STATE   # weights are synthesised once per process
    if "qw" not in state:
        rng0 = np.random.default_rng(0)
        state["qw"] = rng0.integers(0, 256, (N_OUT, K_IN // 2), dtype=np.uint8)
        state["sw_np"] = (0.002 + 0.01 * rng0.random(N_OUT)).astype(np.float16)
    qw, sw = state["qw"], state["sw_np"]
    rng = np.random.default_rng(1)

    def run_port(rows):
        x = rng.standard_normal((rows, K_IN)).astype(np.float16)
        t0 = time.perf_counter()
        s = o.sym_scales(x)
        qa = o.sym_quant(x, s)
        acc = o.matmul_4bit(qa, qw)
        o.sym_dequant(acc, s, sw)
        return time.perf_counter() - t0

    def run_torch(rows):
        if "wf" not in state:
            state["wf"] = tp.unpack_i4(torch.from_numpy(qw)).float()
            state["sw"] = torch.from_numpy(sw)
        x = torch.from_numpy(rng.standard_normal((rows, K_IN)).astype(np.float16))
        t0 = time.perf_counter()
        tp.linear_w4a4_sym(x, state["wf"], state["sw"])
        return time.perf_counter() - t0

    if sample_rows is None:
        t = run_port(4)
        sample_rows = int(max(4, min(512, 4 * budget_s / max(t, 1e-3))))
    t_port = run_port(sample_rows)
    run_torch(min(sample_rows, 64))   # first call pays the one-off weight unpack and thread start-up
    t_torch = run_torch(sample_rows)
    tops = lambda t: 2.0 * sample_rows * N_OUT * K_IN / t / 1e12
    return {"value": tops(t_torch), "unit": "TOPS", "cores": threads, "kind": "reference-python",
            "sample": f"first {sample_rows} of {M_TOK} tokens x full {K_IN}->{N_OUT} layer (per-token scale, quantize, pack/unpack, "
                      f"integer matmul as float matmul, fp16 dequant) in torch on the host cores, {t_torch:.2f} s; the figure is normalised "
                      "to TOPS, so it is a sample of the workload, not the whole 4096-token step",
            "port": {"value": tops(t_port), "unit": "TOPS", "kind": "port", "seconds": round(t_port, 3),
                     "what": "oracle/duq_oracle.c (C restatement of the reference's CUDA kernels, OpenMP) on the same sample"}}, t_torch, sample_rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, rows = [], None
    for i in range(args.warmup + args.steps):
        cb, t, rows = cpu_baseline(sample_rows=rows, budget_s=6.0)
        if i >= args.warmup:
            times.append(t)
    t = sum(times) / len(times)
    tops = 2.0 * rows * N_OUT * K_IN / t / 1e12
    cb["value"] = tops
    line = {"impl": "reference", "metric": "w4a4_linear_tops_M4096", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4xint4->int32, fp16 epilogue", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample_rows_per_step": rows, "note": "CPU arm: the reference's PyTorch fake-quant / "
                       "integer-matmul path restated in torch (oracle/torch_path.py) on a token sample of the workload, all host cores; the C "
                       "port of the reference's CUDA kernels is timed beside it (cpu_baseline.port); the reference's CUDA kernels need a GPU"},
            "cpu_baseline": cb,
            "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
def time_decode(torch, L, device, peaks, Ms=(1, 2, 4, 8, 16)):
    """us/layer at M <= 16 tokens on the Llama-2-7B shapes with COLD weights: a CUDA graph walks over enough
    distinct weight buffers to exceed L2 (126 MB) before reusing one. Two kinds of rows:
      what = "layer"             the whole W4A4 linear, fp16 activations in -> fp16 out, through
                                 duq4_linear_w4a4_from_fp16 (activation quantizer included; one launch per layer)
      what = "gemv+dequant only" pre-quantized codes in -> fp16 out through duq4_linear_w4a4 (the quantizer is NOT
                                 in the timed region)
    each with the serving options on (weights declared static so consecutive layers overlap their weight
    streaming, next-layer L2 hint) and, for the layer rows, also with both off ("plain"). 1 and 16 tokens get all
    three rows, 2 / 4 / 8 tokens the first. us_per_layer is the median over ten graph replays of >= 100 layers each;
    p10 / p90 are given beside it."""
    out = []
    for (K, N) in DECODE_SHAPES:
        wbytes = N * K // 2
        ncopy = max(4, int(320e6 // wbytes) + 1)
        W = torch.randint(0, 256, (ncopy, N, K // 2), dtype=torch.uint8, device=device)
        sw = (torch.rand(N, device=device) * 0.01 + 0.002).to(torch.float16)
        for M in Ms:
            qa = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=device)
            sa = (torch.rand(M, device=device) * 0.1 + 0.01).to(torch.float16)
            x = torch.randn((M, K), device=device).to(torch.float16)
            y = torch.empty((M, N), dtype=torch.float16, device=device)
            ws_bytes = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
            ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=device)
            passes = -(-100 // ncopy)   # at least 100 layer invocations per graph replay
            kinds = (("layer", True), ("layer", False), ("gemv+dequant only", True)) if M in (1, 16) else (("layer", True),)
            for what, serving in kinds:
                if os.environ.get("DUQ4_BENCH_NO_PDL") and serving:
                    continue
                # one epilogue per layer: each names the NEXT layer's weights (L2 prefetch hint), as a model
                # runner that knows its layer order would
                epis = [L.make_epilogue("sym", None if what == "layer" else sa, None, sw,
                                        next_weights=W[(c + 1) % ncopy] if serving and not os.environ.get("DUQ4_BENCH_NO_HINT") else None)
                        for c in range(ncopy)]
                prev = L.cdll.duq4_set_static_weights(1 if serving else 0)

                def body():
                    for _ in range(passes):
                        for c in range(ncopy):
                            if what == "layer":
                                L.call("duq4_linear_w4a4_from_fp16", L.ptr(x), ctypes.c_void_p(W[c].data_ptr()), M, N, K, L.MODE_SYM, 1.0,
                                       ctypes.byref(epis[c]), L.ptr(y), L.ptr(ws), ws.numel(), L.current_stream())
                            else:
                                L.call("duq4_linear_w4a4", L.ptr(qa), ctypes.c_void_p(W[c].data_ptr()), M, N, K, ctypes.byref(epis[c]),
                                       L.ptr(y), None, L.current_stream())

                s = torch.cuda.Stream()
                with torch.cuda.stream(s):
                    body()
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=s):
                        body()
                    for _ in range(3):
                        g.replay()
                    torch.cuda.synchronize()
                    reps = 10
                    evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
                    evs[0].record(s)
                    for i in range(reps):
                        g.replay()
                        evs[i + 1].record(s)
                    torch.cuda.synchronize()
                L.cdll.duq4_set_static_weights(prev)
                per = sorted(evs[i].elapsed_time(evs[i + 1]) * 1e3 / (ncopy * passes) for i in range(reps))
                us = 0.5 * (per[reps // 2 - 1] + per[reps // 2])
                gbs = wbytes / (us * 1e-6) / 1e9
                out.append({"K": K, "N": N, "M": M, "what": what, "options": "static weights + next-layer hint" if serving else "plain",
                            "us_per_layer": round(us, 3), "us_p10": round(per[1], 3), "us_p90": round(per[-2], 3), "weight_GBps": round(gbs, 1),
                            "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4),
                            "frac_of_nominal_8TBps": round(gbs / NOMINAL_HBM_GBS, 4), "cold_weight_buffers": ncopy,
                            "layers_per_graph": ncopy * passes,
                            # fp16 tokens in: one launch at one token (the kernel quantizes the token itself), else the
                            # fused quantizer + the small-M kernel, the second launched programmatically behind the first
                            "launches_per_layer": 2 if (what == "layer" and M > 1) else 1})
                del g
        del W
    return out


def time_mlp_block(torch, L, device):
    """Quantized SiLU-gated MLP block of a random-init Llama-2-7B layer (hidden 4096, intermediate
    11008) on 32 x 512 = 16384 tokens, four launches either way:
      fused epilogue : quantize -> gate/up GEMM whose epilogue forms h = silu(g) * u (fp16 [T, I]; the
                       [T, 2I] gate/up tensor is never written) -> quantize h -> down GEMM
      glue kernel    : quantize -> gate/up GEMM (fp16 [T, 2I]) -> fused SiLU*mul + requantize -> down GEMM
    Both give bit-identical results. The fused-epilogue pipeline is the faster one (the gate/up GEMM
    variant runs 8 epilogue warps for the exp + IEEE divide per element and never writes the [T, 2I]
    tensor) and is reported as ms_per_block; the other is reported beside it."""
    T, H, I = 32 * 512, 4096, 11008
    st = L.current_stream
    x = synth_activations(torch, T, H, seed=3, pinned=False).to(device)
    w_gu, s_gu = synth_weights(torch, 2 * I, H, seed=11, device=device)
    w_dn, s_dn = synth_weights(torch, H, I, seed=12, device=device)
    a8 = torch.empty((T, H), dtype=torch.int8, device=device); sa = torch.empty(T, dtype=torch.float16, device=device)
    gu = torch.empty((T, 2 * I), dtype=torch.float16, device=device)
    h = torch.empty((T, I), dtype=torch.float16, device=device)
    h8 = torch.empty((T, I), dtype=torch.int8, device=device); sh = torch.empty(T, dtype=torch.float16, device=device)
    y = torch.empty((T, H), dtype=torch.float16, device=device)
    e1 = L.make_epilogue("sym", sa, None, s_gu)
    e2 = L.make_epilogue("sym", sh, None, s_dn)

    def block_fused_epilogue():
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), T, H, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
        L.call("duq4_linear_w4a4_gate_up_silu", L.ptr(a8), 1, L.ptr(w_gu), T, I, H, ctypes.byref(e1), L.ptr(h), st())
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(h), T, I, 1.0, L.ptr(h8), L.ptr(sh), None, None, None, st())
        L.call("duq4_linear_w4a4_preunpacked", L.ptr(h8), L.ptr(w_dn), T, H, I, ctypes.byref(e2), L.ptr(y), None, st())

    w8_gu = torch.empty((2 * I, H), dtype=torch.int8, device=device); w8_dn = torch.empty((H, I), dtype=torch.int8, device=device)
    L.call("duq4_weight_prelayout_i8", L.ptr(w_gu), 2 * I, H, L.ptr(w8_gu), st())
    L.call("duq4_weight_prelayout_i8", L.ptr(w_dn), H, I, L.ptr(w8_dn), st())
    split_ws = torch.empty(L.cdll.duq4_gemm_split_scratch_bytes(), dtype=torch.uint8, device=device)

    def block_prelaid():   # the fused-epilogue pipeline on pre-laid-out int8 weights (one-off re-layout outside the timing)
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), T, H, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
        L.call("duq4_linear_w4a4_gate_up_silu_prelaid", L.ptr(a8), L.ptr(w8_gu), T, I, H, ctypes.byref(e1), L.ptr(h), st())
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(h), T, I, 1.0, L.ptr(h8), L.ptr(sh), None, None, None, st())
        L.call("duq4_linear_w4a4_prelaid", L.ptr(h8), L.ptr(w8_dn), T, H, I, ctypes.byref(e2), L.ptr(y), None, L.ptr(split_ws), split_ws.numel(), st())

    def block_glue_kernel():
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), T, H, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
        L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), L.ptr(w_gu), T, 2 * I, H, ctypes.byref(e1), L.ptr(gu), None, st())
        L.call("duq4_silu_mul_quantize_fused", L.MODE_SYM, L.ptr(gu), T, I, 2 * I, I, 1.0, L.ptr(h8), 1, L.ptr(sh), None, st())
        L.call("duq4_linear_w4a4_preunpacked", L.ptr(h8), L.ptr(w_dn), T, H, I, ctypes.byref(e2), L.ptr(y), None, st())

    def run(block):
        for _ in range(3):
            block()
        torch.cuda.synchronize()
        e0, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            block()
        e1_.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1_) / reps

    ms_glue = run(block_glue_kernel)
    y_glue = y.clone()
    ms_packed = run(block_fused_epilogue)
    same = bool(torch.equal(y.view(torch.int16), y_glue.view(torch.int16)))
    ms = run(block_prelaid)
    same = same and bool(torch.equal(y.view(torch.int16), y_glue.view(torch.int16)))
    ops = 2.0 * T * H * 2 * I + 2.0 * T * I * H
    return {"tokens": T, "hidden": H, "intermediate": I, "ms_per_block": round(ms, 4), "tops": round(ops / (ms * 1e-3) / 1e12, 1),
            "launches_per_block": 4, "pipeline": "quantize, gate/up GEMM with SiLU*mul in its epilogue, quantize, down GEMM; both GEMMs on pre-laid-out int8 weights",
            "ms_per_block_packed_weights": round(ms_packed, 4),
            "ms_per_block_glue_kernel_variant": round(ms_glue, 4), "variants_bit_identical": same}


def time_tp_mlp_block(torch, L, dist, device, rank, world):
    """Tensor-parallel SiLU-gated MLP block of a random-init Llama-2-7B layer (hidden 4096, intermediate 11008) on
    16384 tokens over `world` GPUs, column -> row: every rank holds the gate and up rows of its slice of the hidden
    channels and the matching K slice of the down projection, so the block needs NO [T, I] all-gather:
      quantize x -> gate/up GEMM with SiLU*mul in its epilogue (h slice [T, I/G]) -> row-parallel down projection
      (slice statistics -> tiny all-reduce -> codes from the global statistics -> GEMM partial sums stored to the
      owners of the row blocks -> owner's reduce + dequant, result to every rank).
    Time = max over ranks, CUDA events, barrier on both sides; a checksum of the replicated result must agree on all ranks."""
    from duqlinear4bitcuda_b200.parallel import RowParallelLinear4bit, k_shard_bounds
    T, H, I = 32 * 512, 4096, 11008
    kb, ke = k_shard_bounds(I, world, rank)
    st = L.current_stream
    x = synth_activations(torch, T, H, seed=3, pinned=False).to(device)
    w_g, s_g = synth_weights(torch, I, H, seed=11, device=device)       # every rank synthesises the same full tensors, keeps its slice
    w_u, s_u = synth_weights(torch, I, H, seed=13, device=device)
    w_gu = torch.cat([w_g[kb:ke], w_u[kb:ke]]).contiguous(); s_gu = torch.cat([s_g[kb:ke], s_u[kb:ke]]).contiguous()
    del w_g, w_u
    w_dn, s_dn = synth_weights(torch, H, I, seed=12, device=device)
    down = RowParallelLinear4bit.from_full("sym", w_dn, s_dn)
    del w_dn
    a8 = torch.empty((T, H), dtype=torch.int8, device=device); sa = torch.empty(T, dtype=torch.float16, device=device)
    h = torch.empty((T, ke - kb), dtype=torch.float16, device=device)
    e1 = L.make_epilogue("sym", sa, None, s_gu)

    def block():
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), T, H, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
        L.call("duq4_linear_w4a4_gate_up_silu", L.ptr(a8), 1, L.ptr(w_gu), T, ke - kb, H, ctypes.byref(e1), L.ptr(h), st())
        return down(h)

    for _ in range(3):
        y = block()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    e0.record()
    for _ in range(reps):
        y = block()
    e1_.record()
    torch.cuda.synchronize(); dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1_) / reps], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    hsum = y.view(torch.int16).to(torch.int64).sum()
    lo, hi = hsum.clone(), hsum.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ops = 2.0 * T * H * 2 * I + 2.0 * T * I * H
    return {"tokens": T, "hidden": H, "intermediate": I, "gpus": world, "ms_per_block": round(float(ms.item()), 4),
            "tops": round(ops / (float(ms.item()) * 1e-3) / 1e12, 1), "replicated_result_checksum_equal": int(lo.item()) == int(hi.item()),
            "pipeline": "quantize, column-parallel gate/up GEMM with SiLU*mul epilogue, row-parallel down projection "
                        "(partial sums to row-block owners over NVLink, one dequant); no [T, I] gather"}


def time_prefill_sweep(torch, L, device, Ms=(512, 2048, 4096, 8192)):
    """Whole layer (fused per-token quantizer + GEMM with the dequant in its epilogue, one C-ABI call:
    duq4_linear_w4a4_from_fp16_prelaid, weights re-laid out to int8 once outside the timed region)
    on the Llama-2-70B MLP shapes with the asymmetric dual-uniform scheme: activations ~N(0.1, 1) with
    0.5 % of the channels x30, per-channel asymmetric weights (codes as signed nibbles, zero-points as
    per-channel vectors). `tops_packed_weights` is the same call on the packed weights (in-kernel unpack)."""
    rows = []
    for K, N in ((8192, 28672), (28672, 8192)):
        g = torch.Generator().manual_seed(100 + K % 97)
        qw = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g).to(device)
        sc1 = (torch.rand(N, generator=g) * 0.01 + 0.002).half().to(device); zc1 = torch.randint(0, 16, (N,), generator=g).half().to(device)
        sc2 = (torch.rand(N, generator=g) * 0.01 + 0.002).half().to(device); zc2 = torch.randint(0, 16, (N,), generator=g).half().to(device)
        epi = L.make_epilogue("asym_dual", None, None, sc1, zc1, sc2, zc2)
        w8 = torch.empty((N, K), dtype=torch.int8, device=device)
        L.call("duq4_weight_prelayout_i8", L.ptr(qw), N, K, L.ptr(w8), L.current_stream())
        for M in Ms:
            gd = torch.Generator(device=device).manual_seed(1000 + M)   # seeded on the device: 235 M values at the largest size
            x = torch.randn((M, K), generator=gd, dtype=torch.float32, device=device) + 0.1
            x[:, torch.randperm(K, generator=g)[: K // 200].to(device)] *= 30.0
            x = x.half()
            out = torch.empty((M, N), dtype=torch.float16, device=device)
            nbytes = L.cdll.duq4_linear_from_fp16_prelaid_workspace_bytes(M, K)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
            fn_packed = lambda: L.call("duq4_linear_w4a4_from_fp16", L.ptr(x), L.ptr(qw), M, N, K, L.MODES["asym_dual"], 1.0,
                                       ctypes.byref(epi), L.ptr(out), L.ptr(ws), nbytes, L.current_stream())
            fn = lambda: L.call("duq4_linear_w4a4_from_fp16_prelaid", L.ptr(x), L.ptr(w8), M, N, K, L.MODES["asym_dual"], 1.0,
                                ctypes.byref(epi), L.ptr(out), L.ptr(ws), nbytes, L.current_stream())
            res = []
            for f in (fn_packed, fn):
                for _ in range(3):
                    f()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 10
                e0.record()
                for _ in range(reps):
                    f()
                e1.record()
                torch.cuda.synchronize()
                res.append(e0.elapsed_time(e1) / reps)
            ms = res[1]
            rows.append({"K": K, "N": N, "M": M, "ms_per_layer": round(ms, 4), "tops": round(2.0 * M * N * K / (ms * 1e-3) / 1e12, 1),
                         "frac_of_nominal_4500": round(2.0 * M * N * K / (ms * 1e-3) / 1e12 / 4500.0, 3),
                         "tops_packed_weights": round(2.0 * M * N * K / (res[0] * 1e-3) / 1e12, 1)})
            del x, out, ws
        del w8
    return rows


def time_weight_prelayout_ablation(torch, L, device):
    """Headline layer (M=4096, 8192 -> 28672, symmetric) with the three operand formats the tensor-core kernel takes:
      packed x packed      activations and weights as packed int4 (the reference's formats; both unpacked in the CTA pair)
      int8 x packed        activations pre-unpacked by the fused quantizer, weights unpacked in the kernel (the default path)
      int8 x int8 prelaid  weights re-laid out ONCE to int8 (duq4_weight_prelayout_i8, twice the bytes), no in-kernel unpack
    Same result bits for all three; TOPS of the GEMM launch alone."""
    M, K, N = M_TOK, K_IN, N_OUT
    x = synth_activations(torch, M, K, seed=0, pinned=False).to(device)
    qw, sw = synth_weights(torch, N, K, seed=1000, device=device)
    a8 = torch.empty((M, K), dtype=torch.int8, device=device); a4 = torch.empty((M, K // 2), dtype=torch.uint8, device=device)
    w8 = torch.empty((N, K), dtype=torch.int8, device=device)
    sa = torch.empty(M, dtype=torch.float16, device=device)
    y = torch.empty((M, N), dtype=torch.float16, device=device)
    st = L.current_stream
    L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), M, K, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
    L.call("duq4_quantize_sym_fused", L.ptr(x), M, K, 1.0, L.ptr(a4), L.ptr(sa), st())
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record(); L.call("duq4_weight_prelayout_i8", L.ptr(qw), N, K, L.ptr(w8), st()); t1.record(); torch.cuda.synchronize()
    prelayout_ms = t0.elapsed_time(t1)
    split_ws = torch.empty(L.cdll.duq4_gemm_split_scratch_bytes(), dtype=torch.uint8, device=device)   # K-split of the last round of tiles
    epi = L.make_epilogue("sym", sa, None, sw)
    variants = {
        "packed x packed": lambda: L.call("duq4_linear_w4a4", L.ptr(a4), L.ptr(qw), M, N, K, ctypes.byref(epi), L.ptr(y), None, st()),
        "int8 x packed": lambda: L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), L.ptr(qw), M, N, K, ctypes.byref(epi), L.ptr(y), None, st()),
        "int8 x int8 prelaid": lambda: L.call("duq4_linear_w4a4_prelaid", L.ptr(a8), L.ptr(w8), M, N, K, ctypes.byref(epi), L.ptr(y), None, None, 0, st()),
    }
    res, ref = {}, None
    for name, fn in variants.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record(); torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        bits = y.view(torch.int16).clone()
        same = True if ref is None else bool(torch.equal(bits, ref))
        ref = bits if ref is None else ref
        res[name] = {"ms": round(ms, 4), "tops": round(2.0 * M * N * K / (ms * 1e-3) / 1e12, 1), "same_bits_as_first": same}
    res["one_off_prelayout_ms"] = round(prelayout_ms, 4)
    res["weight_bytes_packed_vs_prelaid"] = [N * K // 2, N * K]
    return res


def time_batched(torch, L, device):
    """B = 8 independent 4096 x 4096 weight sets over M = 256 tokens each, one batched launch with
    the asymmetric dequant in the epilogue."""
    B, M, N, K = 8, 256, 4096, 4096
    qa = torch.randint(0, 256, (B, M, K // 2), dtype=torch.uint8, device=device)
    qw = torch.randint(0, 256, (B, N, K // 2), dtype=torch.uint8, device=device)
    sr = torch.rand((B, M), device=device).half(); zr = torch.randint(0, 16, (B, M), device=device).half()
    sc = torch.rand((B, N), device=device).half(); zc = torch.randint(0, 16, (B, N), device=device).half()
    out = torch.empty((B, M, N), dtype=torch.float16, device=device)
    epi = L.make_epilogue("asym", sr, zr, sc, zc)
    fn = lambda: L.call("duq4_linear_w4a4_batched", L.ptr(qa), L.ptr(qw), M, N, K, B, ctypes.byref(epi), L.ptr(out), None,
                        L.current_stream())
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    return {"batch": B, "M": M, "N": N, "K": K, "us": round(ms * 1e3, 2), "tops": round(2.0 * B * M * N * K / (ms * 1e-3) / 1e12, 1)}


def int8_cublas_tops(torch, device):
    """cuBLASLt int8 GEMM (torch._int_mm) at 8192^3, best of 5: context for the tensor-pipe peak."""
    try:
        a = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device=device)
        b = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device=device).t()
        for _ in range(2):
            torch._int_mm(a, b)
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch._int_mm(a, b); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return round(2 * 8192 ** 3 / (best * 1e-3) / 1e12, 1)
    except Exception as ex:  # pragma: no cover
        return f"unavailable: {type(ex).__name__}"


def run_profile_case(args):
    """A few launches of one kernel on a reduced case, for `ncu` captures (no timing)."""
    import torch
    import duqlinear4bitcuda_b200.lib as L
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    st = L.current_stream
    if args.profile_case == "gemm":
        M, N, K = 2048, 8192, 8192
        x = torch.randn((M, K), device=dev).half()
        qw = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev)
        a8 = torch.empty((M, K), dtype=torch.int8, device=dev)
        sa = torch.empty(M, dtype=torch.float16, device=dev); sw = torch.rand(N, device=dev).half()
        y = torch.empty((M, N), dtype=torch.float16, device=dev)
        epi = L.make_epilogue("sym", sa, None, sw)
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), M, K, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
        for _ in range(4):
            L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), L.ptr(qw), M, N, K, ctypes.byref(epi), L.ptr(y), None, st())
    elif args.profile_case in ("gemm_prelaid", "gemm_headline", "gemm_m512"):
        # gemm_headline: the bench's own shape, with the K-split of the last round of tiles (0.6 GB on the device);
        # gemm_m512: the 512-token point of the prefill sweep (two row blocks: every weight tile is used by two pairs only)
        M, N, K = {"gemm_prelaid": (2048, 8192, 8192), "gemm_headline": (M_TOK, N_OUT, K_IN), "gemm_m512": (512, N_OUT, K_IN)}[args.profile_case]
        x = torch.randn((M, K), device=dev).half()
        qw = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev)
        a8 = torch.empty((M, K), dtype=torch.int8, device=dev); w8 = torch.empty((N, K), dtype=torch.int8, device=dev)
        sa = torch.empty(M, dtype=torch.float16, device=dev); sw = torch.rand(N, device=dev).half()
        y = torch.empty((M, N), dtype=torch.float16, device=dev)
        epi = L.make_epilogue("sym", sa, None, sw)
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), M, K, 1.0, L.ptr(a8), L.ptr(sa), None, None, None, st())
        L.call("duq4_weight_prelayout_i8", L.ptr(qw), N, K, L.ptr(w8), st())
        sk = torch.empty(L.cdll.duq4_gemm_split_scratch_bytes() if args.profile_case != "gemm_prelaid" else 0, dtype=torch.uint8, device=dev)
        for _ in range(4):
            L.call("duq4_linear_w4a4_prelaid", L.ptr(a8), L.ptr(w8), M, N, K, ctypes.byref(epi), L.ptr(y), None, L.ptr(sk) if sk.numel() else None, sk.numel(), st())
    elif args.profile_case in ("decode", "decode16", "decode_layer"):
        M, N, K = (16 if args.profile_case == "decode16" else 1), 22016, 4096
        W = torch.randint(0, 256, (8, N, K // 2), dtype=torch.uint8, device=dev)  # 8 x 45 MB: cold in L2
        qa = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev)
        x = torch.randn((M, K), device=dev).half()
        sa = torch.rand(M, device=dev).half(); sw = torch.rand(N, device=dev).half()
        y = torch.empty((M, N), dtype=torch.float16, device=dev)
        epi = L.make_epilogue("sym", sa, None, sw)
        ws = torch.empty(max(256, L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)), dtype=torch.uint8, device=dev)
        for c in range(8):
            if args.profile_case == "decode_layer":   # fp16 tokens in: the kernel quantizes them itself (one launch)
                L.call("duq4_linear_w4a4_from_fp16", L.ptr(x), ctypes.c_void_p(W[c].data_ptr()), M, N, K, L.MODE_SYM, 1.0, ctypes.byref(epi),
                       L.ptr(y), L.ptr(ws), ws.numel(), st())
            else:
                L.call("duq4_linear_w4a4", L.ptr(qa), ctypes.c_void_p(W[c].data_ptr()), M, N, K, ctypes.byref(epi), L.ptr(y), None, st())
    elif args.profile_case == "quantize":
        M, K = 4096, 8192
        xs = [torch.randn((M, K), device=dev).half() for _ in range(4)]  # 4 x 64 MB
        q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev); s = torch.empty(M, dtype=torch.float16, device=dev)
        for x in xs:
            L.call("duq4_quantize_sym_fused", L.ptr(x), M, K, 1.0, L.ptr(q), L.ptr(s), st())
    elif args.profile_case == "skinny":
        M, N, K = 64, 22016, 4096    # up to 128 tokens: narrow tiles, W streamed once (8 x 45 MB of cold weights)
        W = torch.randint(0, 256, (8, N, K // 2), dtype=torch.uint8, device=dev)
        a8 = (torch.randint(-8, 8, (M, K), dtype=torch.int8, device=dev) * 16)
        sa = torch.rand(M, device=dev).half(); sw = torch.rand(N, device=dev).half()
        y = torch.empty((M, N), dtype=torch.float16, device=dev)
        epi = L.make_epilogue("sym", sa, None, sw)
        for c in range(8):
            L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), ctypes.c_void_p(W[c].data_ptr()), M, N, K, ctypes.byref(epi), L.ptr(y), None, st())
    elif args.profile_case == "silu":
        T, I = 4096, 11008   # 180 MB of fp16 gate/up per launch (> L2)
        gu = (torch.randn((T, 2 * I), device=dev) * 2).half()
        h8 = torch.empty((T, I), dtype=torch.int8, device=dev); sh = torch.empty(T, dtype=torch.float16, device=dev)
        for _ in range(4):
            L.call("duq4_silu_mul_quantize_fused", L.MODE_SYM, L.ptr(gu), T, I, 2 * I, I, 1.0, L.ptr(h8), 1, L.ptr(sh), None, st())
    else:
        raise SystemExit("unknown --profile-case")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": args.profile_case, "ok": True}))


def run_ours(args):
    import torch
    import torch.distributed as dist
    import duqlinear4bitcuda_b200.lib as L  # raises if libduq4.so is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()
    M, K, N = M_TOK, K_IN, N_OUT
    assert N % world == 0
    Ns = N // world
    st = L.current_stream

    x_host = synth_activations(torch, M, K, seed=0)
    x = x_host.to(device)
    qw_full_seeded = synth_weights(torch, Ns, K, seed=1000 + rank, device=device)  # this rank's N-shard
    qw, sw = qw_full_seeded
    # Weight pre-layout (one-off, outside every timed region): int8 copy of this rank's packed weights in the tensor-core
    # kernel's operand layout; the packed tensor stays the format of record.
    w8 = torch.empty((Ns, K), dtype=torch.int8, device=device)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record(); L.call("duq4_weight_prelayout_i8", L.ptr(qw), Ns, K, L.ptr(w8), st()); t1.record(); torch.cuda.synchronize()
    prelayout_ms = t0.elapsed_time(t1)
    split_ws = torch.empty(L.cdll.duq4_gemm_split_scratch_bytes(), dtype=torch.uint8, device=device)   # K-split of the last round of tiles
    out_shard = torch.empty((M, Ns), dtype=torch.float16, device=device)
    out_full = torch.empty((M, N), dtype=torch.float16, device=device) if world > 1 else out_shard
    gathered = torch.empty((world, M, Ns), dtype=torch.float16, device=device) if world > 1 else None
    out_host = torch.empty((M, N), dtype=torch.float16).pin_memory()
    codes = torch.empty((M, K), dtype=torch.int8, device=device)   # tensor-core-ready activation codes
    sa = torch.empty((M,), dtype=torch.float16, device=device)
    epi = L.make_epilogue("sym", sa, None, sw, col_offset=rank * Ns)

    peer = None
    gather_mode = "none" if world == 1 else args.gather
    if world > 1 and args.gather in ("fused", "copy"):
        try:
            from duqlinear4bitcuda_b200.parallel import PeerOutput
            use_mc = args.gather == "fused" and (args.multicast == "on" or (args.multicast == "auto" and world >= 8))
            peer = PeerOutput(M, N, device, use_multicast=use_mc)
            epi_f = L.make_epilogue("sym", sa, None, sw, col_offset=rank * Ns, ldo=N, out_peers=peer.column_ptrs(rank * Ns),
                                    out_multicast=peer.multicast_column_ptr(rank * Ns))
            gather_mode = "fused, multimem.st through the NVLink switch" if peer.multicast_ptr else "fused, one st.global per peer"
            if args.gather == "copy":
                gather_mode = "copy engines: 2-D peer copies per row chunk, overlapped with the next chunk's GEMM"
                epi_c = L.make_epilogue("sym", None, None, sw, col_offset=rank * Ns, ldo=N, out_peers=peer.column_ptrs(rank * Ns))
                copy_staging_bytes = L.cdll.duq4_linear_pipeline_staging_bytes(0, 1, M, Ns, K, args.chunk_rows)
                copy_staging = torch.empty(copy_staging_bytes, dtype=torch.uint8, device=device)
        except Exception as ex:  # symmetric memory not available on this box: use the collective
            peer = None
            gather_mode = f"nccl (symmetric memory unavailable: {type(ex).__name__})"

    def step(ev=None):
        # the two launches duq4_linear_w4a4_from_fp16 makes, issued separately so that the GEMM
        # launch can be bracketed by its own events
        if peer is not None and args.gather == "copy":
            peer.barrier()   # every rank has consumed the previous result
            if ev:
                ev[0].record()
            L.call("duq4_linear_w4a4_from_fp16_to_peers", L.ptr(x), L.ptr(w8), 1, M, Ns, K, L.MODE_SYM, 1.0, ctypes.byref(epi_c), rank,
                   args.chunk_rows, L.ptr(copy_staging), copy_staging_bytes, st())
            if ev:
                ev[1].record()
            peer.barrier()   # every rank's block has landed everywhere
            return
        L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), M, K, 1.0, L.ptr(codes), L.ptr(sa), None, None, None, st())
        if ev:
            ev[0].record()
        if peer is not None:
            peer.barrier()   # every rank has consumed the previous result
            L.call("duq4_linear_w4a4_prelaid", L.ptr(codes), L.ptr(w8), M, Ns, K, ctypes.byref(epi_f), None, None, L.ptr(split_ws), split_ws.numel(), st())
            if ev:
                ev[1].record()
            peer.barrier()   # every rank's block has landed everywhere
            return
        L.call("duq4_linear_w4a4_prelaid", L.ptr(codes), L.ptr(w8), M, Ns, K, ctypes.byref(epi), L.ptr(out_shard), None, L.ptr(split_ws), split_ws.numel(), st())
        if ev:
            ev[1].record()
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(world * M, Ns), out_shard)
            out_full.view(M, world, Ns).copy_(gathered.permute(1, 0, 2))

    # e2e: the job's activations and result live in HOST memory. One GPU: pinned tensors of this process.
    # N GPUs: ONE input and ONE result in POSIX shared memory that every rank maps and page-locks for its own
    # GPU; each rank uploads the activations over its own PCIe link, computes its column block and delivers it
    # into columns [r*N/G, (r+1)*N/G) of the one row-major [M, N] host result -- the same C-ABI entry point as
    # on one GPU (output pitch N, pointer at the shard's first column), no device-side gather, no collective.
    shared_x = shared_out = None
    if world == 1:
        e2e_x, e2e_out = x_host, out_host
    else:
        from duqlinear4bitcuda_b200.parallel import SharedHostTensor
        tag = os.environ.get("MASTER_PORT", "0")
        if rank == 0:
            shared_x = SharedHostTensor(f"duq4_bench_{tag}_x", (M, K), torch.float16, create=True)
            shared_out = SharedHostTensor(f"duq4_bench_{tag}_out", (M, N), torch.float16, create=True)
            shared_x.tensor.copy_(x_host)
            shared_out.tensor.zero_()
        dist.barrier()
        if rank != 0:
            shared_x = SharedHostTensor(f"duq4_bench_{tag}_x", (M, K), torch.float16, create=False)
            shared_out = SharedHostTensor(f"duq4_bench_{tag}_out", (M, N), torch.float16, create=False)
        e2e_x, e2e_out = shared_x.tensor, shared_out.tensor
    # the public API of a host-resident job: ColumnParallelLinear4bit.forward_host (one GPU: the host-buffer entry
    # point; G GPUs: row-sharded upload, NVLink all-gather of the activations, then per --e2e-delivery)
    from duqlinear4bitcuda_b200.parallel import ColumnParallelLinear4bit
    host_layer = ColumnParallelLinear4bit("sym", N, qw, sw, unsharded=(world == 1))

    def step_e2e():
        host_layer.forward_host(e2e_x, e2e_out, delivery=args.e2e_delivery)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, per_kernel=False):
        for _ in range(warmup):
            fn()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)] if per_kernel else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(evs[i]) if per_kernel else fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        kms = [a.elapsed_time(b) for a, b in evs] if per_kernel else None
        return ms, kms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    total_ms, gemm_ms = timed(step, args.steps, args.warmup, per_kernel=True)
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms, _ = timed(step_e2e, args.steps, args.warmup)

    # Sustained figure: the same step back to back for at least two seconds (the burst above lasts a few
    # milliseconds at full SM clock; under continuous load the GPU settles at its power cap).
    sustained = None
    if world == 1 and not args.no_sustained:
        sampler2 = ClockSampler(local)
        sampler2.start()
        n_sus = max(args.steps, int(2.2 / (total_ms / args.steps * 1e-3)))
        sus_ms, sus_k = timed(step, n_sus, 3, per_kernel=True)
        c2 = sampler2.stop()
        sus_gemm_ms = sum(sus_k) / len(sus_k)
        sustained = {"steps": n_sus, "seconds": round(sus_ms * 1e-3, 3), "ms_per_step": round(sus_ms / n_sus, 4),
                     "value": round(2.0 * M * N * K / (sus_ms / n_sus * 1e-3) / 1e12, 2), "unit": "TOPS",
                     "gemm_launch_tops": round(2.0 * M * Ns * K / (sus_gemm_ms * 1e-3) / 1e12, 2),
                     "clocks": c2, "power_cap_seen": "sw_power_cap" in (c2.get("reasons") or []),
                     "frac_of_2x_bf16_sustained": round(2.0 * M * Ns * K / (sus_gemm_ms * 1e-3) / 1e12 / (2.0 * peaks["bf16_tflops_sustained"]), 4),
                     "frac_of_nominal_4500": round(2.0 * M * Ns * K / (sus_gemm_ms * 1e-3) / 1e12 / NOMINAL_INT8_TOPS, 4)}

    # ---- correctness of what was timed, computed OUTSIDE the timed regions -------------------------------
    checks = {}
    L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), M, K, 1.0, L.ptr(codes), L.ptr(sa), None, None, None, st())
    L.call("duq4_linear_w4a4_preunpacked", L.ptr(codes), L.ptr(qw), M, Ns, K, ctypes.byref(epi), L.ptr(out_shard), None, st())
    torch.cuda.synchronize()
    if world > 1:
        # (1) this rank's column slice of the gathered [M, N] buffer equals its local block bit for bit;
        # (2) a position-weighted checksum of the whole gathered buffer is the same number on every rank
        full = peer.buf if peer is not None else out_full
        mine = full[:, rank * Ns:(rank + 1) * Ns]
        slice_ok = bool(torch.equal(mine.view(torch.int16), out_shard.view(torch.int16)))
        hsum = torch.zeros((), dtype=torch.int64, device=device)
        wts = (torch.arange(N, device=device, dtype=torch.int64) % 8191) + 1
        for r0 in range(0, M, 512):
            hsum += (full[r0:r0 + 512].view(torch.int16).to(torch.int64) * wts).sum() * (1 + r0 // 512)
        lo, hi = hsum.clone(), hsum.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ok_t = torch.tensor([int(slice_ok)], device=device)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        checks["gather_check"] = "ok" if (int(ok_t.item()) == 1 and int(lo.item()) == int(hi.item())) else \
            f"FAILED (slice_ok_all_ranks={int(ok_t.item())}, checksum min/max {int(lo.item())}/{int(hi.item())})"
        # (3) the host result assembled from the ranks' slices equals the gathered device result
        dist.barrier()
        if rank == 0:
            host_ok = bool(torch.equal(e2e_out.view(torch.int16), full.cpu().view(torch.int16)))
            checks["e2e_host_result_check"] = "ok" if host_ok else "FAILED"
    else:
        checks["e2e_host_result_check"] = "ok" if bool(torch.equal(out_host.view(torch.int16), out_shard.cpu().view(torch.int16))) else "FAILED"

    status = ctypes.c_int32(-1)
    L.call("duq4_last_device_status", st(), ctypes.byref(status))
    if status.value != 0:
        raise SystemExit(f"device-side bounded wait expired (code {status.value}); result invalid")

    ops = 2.0 * M * N * K
    ms_step = total_ms / args.steps
    tops = ops / (ms_step * 1e-3) / 1e12
    e2e_tops = ops / (e2e_ms / args.steps * 1e-3) / 1e12
    gemm_avg_ms = sum(gemm_ms) / len(gemm_ms)
    gemm_tops = (2.0 * M * Ns * K) / (gemm_avg_ms * 1e-3) / 1e12  # this rank's GEMM launch
    # no int8 figure in MEASURED_PEAKS.json: dense int8 is nominally 2x dense bf16, so the denominator is twice
    # the measured cuBLAS bf16 burst rate (the kernel is timed alone over a few ms at full SM clock)
    int8_peak = 2.0 * peaks["bf16_tflops"]

    line = {"metric": "w4a4_linear_tops_M4096", "value": round(tops, 2), "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4xint4->int32 (kind::i8 tensor cores), fp16 epilogue", "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "K": K, "N": N, "parallelism": f"column-parallel N/{world}, gather={gather_mode}" if world > 1 else "single GPU",
                       "checks": "computed outside the timed regions: gathered buffer vs each rank's local block and a cross-rank checksum (gather_check), host result vs device result (e2e_host_result_check)",
                       "cache": "operands (weights 117 MB + activations 64 MB + output 235 MB) exceed the 126 MB L2; no flush",
                       "weights": "N(0,0.015) per-channel symmetric int4, packed [N, K/2]; the GEMM reads a one-off int8 re-layout of them "
                                  f"(duq4_weight_prelayout_i8, {prelayout_ms:.3f} ms outside the timed region, 2x the weight bytes); the in-kernel-unpack "
                                  "route on the packed tensor is timed under weight_prelayout_ablation", "activations": "N(0,1), 1% channels x20, per-token symmetric int4"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_tops, 2), "unit": "TOPS", "ms_per_step": round(e2e_ms / args.steps, 4),
                    "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                    "api": ("ColumnParallelLinear4bit.forward_host -> duq4_linear_w4a4_from_fp16_host (C ABI; pinned host activations in, pinned host result out, "
                            "copies pipelined with the arithmetic over row chunks)" if world == 1 else
                            "ColumnParallelLinear4bit.forward_host: one input and one result in shared pinned host memory; each rank uploads its row slice "
                            "of the activations over its own PCIe link, NCCL all-gather of the slices over NVLink, then "
                            + ("duq4_linear_w4a4_from_fp16_to_host_rows (C ABI): per row chunk the GEMM epilogue stores each row into the exchange buffer of "
                               "the rank that owns it (NVLink), a rank barrier, and every rank downloads the contiguous rows it owns while the next chunk is computed"
                               if args.e2e_delivery == "rows" else
                               "duq4_linear_w4a4_from_fp16_to_host (C ABI) per rank delivers its [M, N/G] column block into its column slice of the one host "
                               "result, download overlapped with the arithmetic"))},
            "checks": checks,
            "sustained": sustained,
            "gpu_launches": args.steps * ((2 * -(-M // max(256, -(-(args.chunk_rows or (M + 15) // 16) // 256) * 256)) + 2) if (peer is not None and args.gather == "copy")
                                          else (4 if peer is not None else 2)),   # per rank: quantize + GEMM (per row chunk with --gather copy) + two barrier kernels around a device-side gather
            "roofline": {"kernel": "gemm_tc2_kernel<WI8> (CTA pairs, 256x256x128 tiles, tcgen05.mma.cta_group::2.kind::i8; A int8 from the fused quantizer, W int8 pre-laid-out, both straight from TMA into the MMA ring)", "bound": "tensor",
                         "achieved": round(gemm_tops, 2), "peak": round(int8_peak, 1), "unit": "TOP/s",
                         "frac": round(gemm_tops / int8_peak, 4),
                         # dram read+write bytes per launch: ncu capture of this kernel at the bench's own size
                         # (the capture summarised under profiles/: 349.2 MB read + 218.7 MB written), scaled
                         # by this rank's share of the columns when the layer is sharded
                         "traffic": round(567.9e6 * Ns / N),
                         "traffic_note": "ncu dram__bytes_read+write of one full-size launch (M=4096, K=8192, N=28672: 349.2 MB read + 218.7 MB "
                                         "written; the tail of the result was still in L2 when the launch ended); algorithmic bytes "
                                         f"{M * K + Ns * K + 2 * M * Ns} (int8 activations + int8 weights + fp16 out)",
                         "avg_launch_ms": round(gemm_avg_ms, 4),
                         "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({peaks['source']}); no int8 entry there",
                         "frac_of_2x_bf16_sustained": round(gemm_tops / (2.0 * peaks["bf16_tflops_sustained"]), 4),
                         "frac_of_nominal_4500": round(gemm_tops / NOMINAL_INT8_TOPS, 4)}}
    if rank == 0 and world == 1:
        line["roofline"]["cublaslt_int8_8192cubed_tops"] = int8_cublas_tops(torch, device)
        if not args.no_decode:
            line["decode"] = time_decode(torch, L, device, peaks)
            line["mlp_block"] = time_mlp_block(torch, L, device)
            line["batched"] = time_batched(torch, L, device)
            line["weight_prelayout_ablation"] = time_weight_prelayout_ablation(torch, L, device)
            line["prefill_sweep"] = time_prefill_sweep(torch, L, device)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline()[0]
    if world > 1 and args.tp_mlp:
        tp = time_tp_mlp_block(torch, L, dist, device, rank, world)
        if rank == 0:
            line["tp_mlp_block"] = tp
    if world > 1:
        dist.barrier()
        for h in (shared_x, shared_out):
            if h is not None:
                h.close()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gather", default="fused", choices=["copy", "fused", "nccl"],
                    help="N>1: 'copy' = local epilogue + copy-engine peer copies per row chunk, overlapped with the next chunk's GEMM; "
                         "'fused' = GEMM epilogue stores into every rank's result buffer over NVLink; 'nccl' = all-gather")
    ap.add_argument("--multicast", default="auto", choices=["auto", "on", "off"], nargs="?", const="on",
                    help="N>1, --gather fused: one multimem.st per row segment through the NVLink switch instead of one plain store per peer; "
                         "auto = from 8 GPUs on (measured: plain stores win at 2 and 4 GPUs, where a rank's ingress is the limit; "
                         "multicast wins at 8, where its egress is)")
    ap.add_argument("--chunk-rows", type=int, default=0, help="N>1, --gather copy: rows per pipeline chunk (0 = M/16 rounded to 256)")
    ap.add_argument("--e2e-delivery", default="columns", choices=["rows", "columns"],
                    help="N>1, host-resident job: 'rows' = rows exchanged over NVLink by the epilogue, each rank downloads contiguous rows; "
                         "'columns' = each rank downloads its column block into its column slice of the host result")
    ap.add_argument("--tp-mlp", action="store_true", help="N>1: also time a tensor-parallel (column -> row) MLP block")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 2-second back-to-back run")
    ap.add_argument("--no-decode", action="store_true", help="skip the M<=16 decode sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--profile-case", default=None, choices=["gemm", "gemm_prelaid", "gemm_headline", "gemm_m512", "decode", "decode16", "decode_layer", "quantize", "silu", "skinny"],
                    help="run a few launches of one kernel on a reduced case (for ncu) and exit")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
