#!/usr/bin/env python
"""Benchmark of the B200 backend on the reference's headline partitions.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload mlp|gemm8192|...]

Headline workload (``config.workload``): BASELINE configs[2], the bf16 MLP chain
512 x (4096 -> 16384 -> 4096 -> 16384 -> 4096), bias + ReLU per layer, synthetic
inputs with benchgc's fill semantics (N(0,1) input, N(0,0.02) weights, zero biases).
One step = one pass of the whole partition.  Metric: TFLOPS (2*M*N*K per layer).

  value     device-resident inputs, CUDA events on the launching stream, max over ranks
  e2e       the same partition through dnnl_graph_compiler_execute with pinned HOST buffers:
            per step H2D of the activations, D2H of the result (weights are constant
            tensors: uploaded by the first call, resident afterwards)
  roofline  tensor-bound: algorithmic FLOPs per GEMM launch / average launch time in the
            timed region, against the measured cuBLAS bf16 peak of this pool
  cpu_baseline  the reference's CPU path on a bounded sample (rank 0, N=1)

Under torchrun (N>1) the layers are column/row tensor-parallel with one f32
all-reduce (NCCL) per layer pair; total work is fixed, so scaling is "strong".
``--impl reference`` times the reference's CPU implementation instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "graph-compiler_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

HIDDEN = (4096, 16384, 4096, 16384, 4096)
BATCH = 512
WORKLOAD = "mlp_bf16_b512_4096x16384x4096x16384x4096_bias_relu"


def mlp_flops(batch=BATCH, hidden=HIDDEN):
    return sum(2 * batch * hidden[i] * hidden[i + 1] for i in range(len(hidden) - 1))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], hbm=d["hbm_gbs"], source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


# --------------------------------------------------------------------------------------- clocks
class NvmlClockSampler:
    """SM clock and clock-event reasons read through NVML about once per millisecond while the timed region runs
    (the region is ~13 ms long at the default step count: nvidia-smi's 200 ms loop would see it once at best).
    Read-only queries; nothing on the GPU is changed."""

    def __init__(self, gpu_index: int):
        import pynvml

        self.nv = pynvml
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        self.samples, self.stop_flag, self.t = [], False, None

    def start(self):
        nv = self.nv

        def loop():
            while not self.stop_flag:
                try:
                    self.samples.append((nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM),
                                         nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)))
                except Exception:
                    pass
                time.sleep(0.001)

        self.t = threading.Thread(target=loop, daemon=True)
        self.t.start()

    def stop(self):
        nv = self.nv
        self.stop_flag = True
        self.t.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = sorted(n for n, bit in names.items() if any(r & bit for _, r in self.samples))
        try:
            mx = float(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
        except Exception:
            mx = None
        return {"sm_mhz": statistics.median(float(c) for c, _ in self.samples), "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(self.samples), "how": "NVML, 1 ms period, from the start of the device-timed region to the end of the end-to-end region"}


def make_clock_sampler(gpu_index: int):
    try:
        return NvmlClockSampler(gpu_index)
    except Exception:
        return ClockSampler(gpu_index)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs (used when NVML
    cannot be loaded)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------- CPU baseline
def cpu_reference_run(steps: int, warmup: int, rows: int | None = None):
    """The reference's CPU implementation of the path on this host's cores, on a bounded sample:
    `rows` rows of the 512-row batch through all four layers (rows of a batch are independent, so
    work scales linearly).  Uses the reference's own naive brgemm (oracle/_ref, compiled unmodified)
    driven by the restated deep-tile nest when present, else the oracle port."""
    import numpy as np

    import oracle

    cores = len(os.sched_getaffinity(0))
    oracle.set_num_threads(cores)
    kind = "reference" if oracle.have_ref() else "port"
    if rows is None:
        rows = 32 if kind == "reference" else 128
    rng = np.random.default_rng(0)
    X = oracle.f32_to_bf16(rng.standard_normal((rows, HIDDEN[0])).astype(np.float32))
    Ws = [oracle.f32_to_bf16((rng.standard_normal((HIDDEN[i], HIDDEN[i + 1])) * 0.02).astype(np.float32)) for i in range(4)]
    Bs = [np.zeros(HIDDEN[i + 1], np.uint16) for i in range(4)]

    def one():
        h = X
        for W, b in zip(Ws, Bs):
            if kind == "reference":
                h = oracle.linear_bf16_brgemm_nest(h, W, b, relu=True, backend="ref")
            else:
                h = oracle.linear_bf16(h, W, b, relu=True)
        return h

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    fl = mlp_flops(rows)
    sample = (f"{rows} of {BATCH} batch rows through all 4 layers ({fl / 1e9:.2f} GFLOP per step); "
              + ("reference BrgemmNaive.cpp (unmodified, oracle/_ref) driven by the restated deep-tile nest, OpenMP over output blocks"
                 if kind == "reference" else "oracle port (vectorised restatement), OpenMP over rows"))
    return dict(value=fl / dt / 1e12, unit="TFLOPS", cores=cores, kind=kind, sample=sample, ms_per_step=dt * 1e3)


def cpu_onednn_class(rows=BATCH):
    """Context only: torch CPU bf16 matmul (oneDNN brgemm, the kernel family BrgemmOnednn.cpp wraps)."""
    import torch

    torch.manual_seed(0)
    x = torch.randn(rows, HIDDEN[0]).bfloat16()
    ws = [(torch.randn(HIDDEN[i], HIDDEN[i + 1]) * 0.02).bfloat16() for i in range(4)]
    bs = [torch.zeros(HIDDEN[i + 1]).bfloat16() for i in range(4)]

    def one():
        h = x
        for w, b in zip(ws, bs):
            h = torch.relu(torch.mm(h, w) + b)
        return h

    one()
    t0 = time.perf_counter()
    n = 2
    for _ in range(n):
        one()
    dt = (time.perf_counter() - t0) / n
    return dict(value=mlp_flops(rows) / dt / 1e12, unit="TFLOPS", cores=torch.get_num_threads(),
                what="torch.mm bf16 on CPU (oneDNN), full batch")


# --------------------------------------------------------------------------------------- other BASELINE configs
def run_case(spec: str, steps: int = 20, warmup: int = 5, flush_mode: str = "auto", library: bool = False):
    """Time one kernel-level case with device-resident inputs (CUDA events on the launching stream).

    spec: gemm:M:N:K | decode | int8:M:N:K | attention:B:H:S:D:causal(0|1) | cfg1 | llama2
    Returns a dict with ms, value/unit, the roofline bound and fraction against the measured peak."""
    import math

    import torch

    from gc_b200 import lib

    peaks = measured_peaks()
    f = spec.split(":")
    kind = f[0]
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)

    def u(shape):
        return (torch.rand(shape, generator=g, device=dev) * 2 - 1).bfloat16()

    if kind in ("gemm", "decode", "cfg1"):
        M, N, K = (16, 28672, 8192) if kind == "decode" else (128, 256, 512) if kind == "cfg1" else map(int, f[1:4])
        A, B = u((M, K)), u((K, N))
        bias = u((N,)) if kind == "cfg1" else None
        Y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        fn = lambda: lib.matmul_bf16(A, B, bias, relu=(kind == "cfg1"), out=Y)
        work, unit = 2.0 * M * N * K, "TFLOPS"
        bytes_ = (M * K + K * N + M * N) * 2
        l2_flush = bytes_ < 256e6
    elif kind == "int8":
        M, N, K = map(int, f[1:4])
        A = torch.randint(0, 256, (M, K), generator=g, device=dev, dtype=torch.uint8)
        W = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
        sc = torch.rand(N, generator=g, device=dev) * 0.009 + 0.001
        bi = torch.rand(N, generator=g, device=dev) * 2 - 1
        comp = lib.colsum_s8(W, 128)
        out = torch.empty(M, N, device=dev)
        import ctypes as C
        l = lib.load()
        fn = lambda: lib.check(l.gcb200_matmul_u8s8(A.data_ptr(), W.data_ptr(), sc.data_ptr(), bi.data_ptr(), comp.data_ptr(),
                                                    out.data_ptr(), None, M, N, K, 0, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        work, unit = 2.0 * M * N * K, "TOPS"
        bytes_ = M * K + K * N + M * N * 4
        l2_flush = True
    elif kind == "attention":
        B_, H, S, D, causal = map(int, f[1:6])
        Q, Kt, V = (torch.randn(B_, H, S, D, generator=g, device=dev).bfloat16() for _ in range(3))
        O = torch.empty_like(Q)
        fn = lambda: lib.attention_bf16(Q, Kt, V, 1.0 / math.sqrt(D), bool(causal), out=O)
        work, unit = 4.0 * B_ * H * S * S * D * (0.5 if causal else 1.0), "TFLOPS"
        bytes_ = 4 * B_ * H * S * D * 2
        l2_flush = bytes_ < 256e6
    elif kind == "llama2":
        # the llama2 decoder MLP block of the reference's tests (onednn-graph-llama2.mlir:5-45), 1 x 32 tokens:
        # 25 steps, HBM-bound on its 302 MB of weights
        from gc_b200 import api, partitions
        Bq, S, H, I = 1, 32, 4096, 11008
        js, ids, outs = partitions.llama2_mlp(Bq, S, H, I)
        exe = api.GraphCompiler().compile(js)
        t = {"x": u((Bq, S, H)), "wo": u((H, H)) * 0.02, "resid": u((Bq, S, H)), "g1": u((H,)), "w_gate": u((I, H)) * 0.02,
             "w_up": u((I, H)) * 0.02, "w_down": u((H, I)) * 0.02, "g2": u((H,))}
        ins = {ids[k]: v.bfloat16() for k, v in t.items()}
        ins[ids["eps"]] = torch.full((1,), 1e-5, device=dev)
        o = {outs[0]: torch.empty(Bq, S, H, dtype=torch.bfloat16, device=dev), outs[1]: torch.empty(Bq, S, H, dtype=torch.bfloat16, device=dev)}
        fn = lambda: exe.execute_on_stream(ins, o)
        work, unit = 2.0 * S * (H * H + 3 * H * I), "TFLOPS"
        bytes_ = 2 * (H * H + 3 * H * I)
        l2_flush = False
    else:
        raise ValueError(spec)
    if flush_mode != "auto":
        l2_flush = flush_mode == "on"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if l2_flush else None

    def time_fn(f, n):
        if flush is None:
            st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record()
            for _ in range(n):
                f()
            en.record()
            torch.cuda.synchronize()
            return st.elapsed_time(en) / n
        tot = 0.0   # small working set: write a buffer larger than L2 between timed launches
        for _ in range(n):
            flush.zero_()
            st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record()
            f()
            en.record()
            torch.cuda.synchronize()
            tot += st.elapsed_time(en)
        return tot / n

    # Context only: the vendor library on the same tensors in the same run (cuBLAS through torch.matmul /
    # torch._int_mm, the library attention through torch SDPA) - the same-box bar the kernels are held against.
    lib_fn, lib_name = None, None
    if library and kind in ("gemm", "decode", "cfg1"):
        Yl = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        lib_fn, lib_name = (lambda: torch.matmul(A, B, out=Yl)), "cuBLAS bf16 via torch.matmul (no bias / ReLU)"
    elif library and kind == "int8" and M > 16 and M % 8 == 0 and N % 8 == 0 and K % 8 == 0:
        A8 = A.view(torch.int8)   # same bytes and work; torch._int_mm takes s8 x s8 only
        lib_fn, lib_name = (lambda: torch._int_mm(A8, W)), "cuBLASLt s8 x s8 -> s32 via torch._int_mm (no dequantisation)"
    elif library and kind == "attention":
        import torch.nn.functional as F
        lib_fn = lambda: F.scaled_dot_product_attention(Q, Kt, V, is_causal=bool(causal), scale=1.0 / math.sqrt(D))
        lib_name = "torch scaled_dot_product_attention (library flash attention)"
    lib_ms = None
    if lib_fn is not None:
        try:
            for _ in range(3):
                lib_fn()
            torch.cuda.synchronize()
            lib_ms = time_fn(lib_fn, max(3, steps // 2))
        except Exception as e:   # context only
            lib_name = f"unavailable: {type(e).__name__}"
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph_us = None
    if kind == "cfg1":
        # latency case: replay a CUDA graph of 50 launches so that host launch cost is not what is timed
        gr = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(gr, stream=side):
                for _ in range(50):
                    fn()
        torch.cuda.synchronize()
        gr.replay()
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        for _ in range(10):
            gr.replay()
        en.record()
        torch.cuda.synchronize()
        graph_us = st.elapsed_time(en) / 500 * 1e3
    l0 = lib.launch_count()
    ms = time_fn(fn, steps)
    launches = (lib.launch_count() - l0) // steps
    assert lib.device_error() == 0, "a kernel reported a bounded-wait time-out"
    r = {"case": spec, "ms": ms, "value": work / ms / 1e9, "unit": unit, "launches_per_step": int(launches),
         "l2": "flushed between launches" if flush is not None else "working set larger than L2"}
    if graph_us is not None:
        r["us_per_launch_graph_replay"] = graph_us
    if lib_name is not None:
        r["library"] = {"what": lib_name, "ms": lib_ms, "value": (work / lib_ms / 1e9 if lib_ms else None), "unit": unit,
                        "time_ratio_ours_over_library": (ms / lib_ms if lib_ms else None)}
    if kind in ("decode", "llama2"):
        r["roofline"] = {"bound": "hbm", "achieved": bytes_ / ms / 1e6, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": bytes_ / ms / 1e6 / peaks["hbm"]}
    elif kind == "int8":
        r["roofline"] = {"bound": "tensor", "achieved": work / ms / 1e9, "peak": 4500.0, "unit": "TOP/s", "frac": work / ms / 1e9 / 4500.0,
                         "peak_source": "vendor dense int8; the library figure of the 8192^3 case in the same sweep is the measured one"}
    else:
        r["roofline"] = {"bound": "tensor", "achieved": work / ms / 1e9, "peak": peaks["burst"], "unit": "TFLOP/s",
                         "frac": work / ms / 1e9 / peaks["burst"], "frac_of_vendor_dense_2250": work / ms / 1e9 / 2250.0}
    return r


def run_sharded_case(spec: str, steps: int, warmup: int, rank: int, world: int):
    """The kernel-level cases that shard across GPUs (one process per GPU, launched under torchrun):
    gemm:M:N:K and int8:M:N:K split along N with the all-gather of C done by the GEMM epilogue (peer stores, or multimem
    stores from four ranks on; GC_B200_GATHER=peer|multicast|nccl chooses, nccl being the library all-gather), decode (the same with the weight-stationary kernel), attention:B:H:S:D:causal split by (batch, head) with no collective.  Inputs are resident before
    timing; the time is the maximum over ranks of a CUDA-event bracket around `steps` steps."""
    import math

    import torch
    import torch.distributed as dist

    from gc_b200 import lib
    from gc_b200.tensor_parallel import PeerGatherGemm, ShardedAttention, ShardedGemm, ShardedQuantGemm, shard_range

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)          # same seed on every rank: replicated inputs are identical
    f = spec.split(":")
    kind = f[0]
    # From four ranks on each block leaves its GPU once through the NVSwitch multicast mapping instead of once per peer
    # (8 GPUs, same box: 16384^3 991 against 1217 us, 8192^3 269 against 289 us); PeerGatherGemm falls back to
    # peer stores where symmetric memory has no multicast mapping.
    gather = os.environ.get("GC_B200_GATHER", "multicast" if world >= 4 else "peer")
    fused, mcast = gather != "nccl", gather == "multicast"
    how = "n/a"
    if kind in ("gemm", "decode"):
        M, N, K = (16, 28672, 8192) if kind == "decode" else map(int, f[1:4])
        lo, hi = shard_range(N, world, rank)
        A = (torch.rand((M, K), generator=g, device=dev) * 2 - 1).bfloat16()
        Bs = (torch.rand((K, N), generator=g, device=dev) * 2 - 1).bfloat16()[:, lo:hi].contiguous()
        if fused:
            op = PeerGatherGemm(Bs, M, N, dev, multicast=mcast)
            fn, how = (lambda: op.step(A)), ("all-gather of C by multimem stores from the GEMM epilogue (NVSwitch multicast) + one barrier"
                                             if op.multicast else "all-gather of C by peer stores from the GEMM epilogue + one barrier")
        else:
            op = ShardedGemm(Bs, world, rank)
            fn, how = (lambda: op.step(A, gather=True)), "NCCL all-gather of C"
        work, unit = 2.0 * M * N * K, "TFLOPS"
    elif kind == "int8":
        M, N, K = map(int, f[1:4])
        lo, hi = shard_range(N, world, rank)
        A = torch.randint(0, 256, (M, K), generator=g, device=dev, dtype=torch.uint8)
        W = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)[:, lo:hi].contiguous()
        sc = (torch.rand(N, generator=g, device=dev) * 0.009 + 0.001)[lo:hi].contiguous()
        bi = (torch.rand(N, generator=g, device=dev) * 2 - 1)[lo:hi].contiguous()
        if fused:
            op = PeerGatherGemm(W, M, N, dev, bias_shard=bi, quant=(sc, 128), multicast=mcast)
            fn, how = (lambda: op.step(A)), ("all-gather of C by multimem stores from the GEMM epilogue (NVSwitch multicast) + one barrier"
                                             if op.multicast else "all-gather of C by peer stores from the GEMM epilogue + one barrier")
        else:
            op = ShardedQuantGemm(W, sc, bi, 128, world, rank)
            fn, how = (lambda: op.step(A, gather=True)), "NCCL all-gather of C"
        work, unit = 2.0 * M * N * K, "TOPS"
    elif kind == "attention":
        B_, H, S, D, causal = map(int, f[1:6])
        units = shard_range(B_ * H, world, rank)
        n = units[1] - units[0]
        Q, Kt, V = (torch.randn(n, 1, S, D, generator=g, device=dev).bfloat16() for _ in range(3))   # this rank's units, resident
        O = torch.empty_like(Q)
        fn, how = (lambda: lib.attention_bf16(Q, Kt, V, 1.0 / math.sqrt(D), bool(causal), out=O)), "no collective ((batch, head) units are independent)"
        work, unit = 4.0 * B_ * H * S * S * D * (0.5 if causal else 1.0), "TFLOPS"
    else:
        raise ValueError(f"{spec} does not shard")
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    l0 = lib.launch_count()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(steps):
        fn()
    en.record()
    torch.cuda.synchronize()
    t = torch.tensor([st.elapsed_time(en) / steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    assert lib.device_error() == 0
    return {"case": spec, "n_gpus": world, "ms": ms, "value": work / ms / 1e9, "unit": unit, "scaling": "strong",
            "launches_per_step_per_rank": int((lib.launch_count() - l0) // steps), "collective": how,
            "timing": "CUDA events, max over ranks, inputs resident"}


PARITY_ROWS = [0, 1, 63, 64, 127, 128, 129, 255, 256, 300, 383, 384, 447, 448, 510, 511]


def parity_rows(y_dev, X_host, W_host, B_host):
    """16 rows of the MLP output the timed step left on the device, against the CPU oracle fed the same rows (rows of a
    batch are independent).  Tolerance of the chain test: |diff| <= 1e-2 max(|want|, rms).  The oracle is used here as
    a checker only."""
    import numpy as np
    import torch

    import oracle

    def bits(t):
        return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)

    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    idx = torch.tensor(PARITY_ROWS)
    h = bits(X_host[idx])
    for W, b in zip(W_host, B_host):
        h = oracle.linear_bf16(h, bits(W), bits(b), relu=True)
    want = oracle.bf16_to_f32(h).astype(np.float64)
    got = oracle.bf16_to_f32(bits(y_dev[idx.to(y_dev.device)])).astype(np.float64)
    rms = float(np.sqrt(np.mean(want[want != 0] ** 2))) if (want != 0).any() else 0.0
    diff = np.abs(got - want)
    ok = bool((diff <= 1e-2 * np.maximum(np.abs(want), rms)).all())
    return {"rows": len(PARITY_ROWS), "max_abs": float(diff.max()), "bit_identical": float((got == want).mean()), "ok": ok,
            "rule": "|diff| <= 1e-2 max(|want|, rms) against the CPU oracle"}


SHARDED = ["gemm:8192:8192:8192", "gemm:16384:16384:16384", "decode", "int8:1024:4096:4096", "attention:16:32:2048:128:0",
           "attention:16:32:2048:128:1"]


def parallelism_of(world: int) -> str:
    """How the workload is spread over `world` GPUs: a function of the launch alone, so that the reference arm
    (which runs on the host) and this arm print the same `config`."""
    if world == 1:
        return "single GPU"
    return (f"tp{world}: layers 1,3 column-parallel, layers 2,4 row-parallel, f32 partial sums exchanged between the GPUs' "
            "own kernels over NVLink")


SWEEP = ["cfg1", "int8:1024:4096:4096", "int8:8192:8192:8192", "decode", "attention:16:32:2048:128:0", "attention:16:32:2048:128:1",
         "gemm:1024:1024:1024", "gemm:2048:2048:2048", "gemm:4096:4096:4096", "gemm:8192:8192:8192", "gemm:16384:16384:16384"]


# --------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sweep", dest="sweep", action="store_true", default=True,
                    help="also time the other BASELINE configs, each beside the vendor library on the same tensors (extra key 'sweep'; default)")
    ap.add_argument("--no-sweep", dest="sweep", action="store_false", help="headline workload only (profiling runs)")
    ap.add_argument("--case", default=None, help="time ONE kernel-level case instead (see run_case) and print its line; "
                                                  "used for ncu captures of a single kernel")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="after the timed region, run the device-resident step back to back for about this long and report it "
                         "under 'sustained' (0 = skip)")
    ap.add_argument("--tp-timeline", action="store_true",
                    help="under torchrun: print, per rank-0 kernel of one eagerly launched tensor-parallel step, the time it took "
                         "(CUDA events between the launches; waits for other ranks included), instead of the bench line")
    ap.add_argument("--flush", default="auto", choices=["auto", "on", "off"],
                    help="--case only: write a 256 MiB buffer between timed launches (auto: when the working set is below 256 MB)")
    a = ap.parse_args()
    if a.tp_timeline:
        os.environ["GC_B200_TP_TRACE"] = "1"   # read by the plan's first step
    a.warmup = max(a.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    config = {"workload": WORKLOAD, "batch": BATCH, "hidden": list(HIDDEN), "fill": "src N(0,1), weights N(0,0.02), bias 0 (benchgc fill flags)",
              "l2": "inputs larger than L2 (weights 512 MiB are re-read every step)"}

    config["parallelism"] = parallelism_of(world)
    if a.impl == "reference":
        if rank != 0:
            return
        # every step is a bounded sample (16 of the 512 batch rows through all four layers), so that the requested
        # step and warm-up counts are honoured and the whole run still ends within a few minutes on the host cores
        r = cpu_reference_run(max(1, a.steps), a.warmup, rows=16)
        line = {"impl": "reference", "metric": "TFLOPS", "value": r["value"], "unit": "TFLOPS", "n_gpus": a.gpus,
                "steps": max(1, a.steps), "warmup": a.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if a.case:
        import torch

        torch.cuda.set_device(local_rank)
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            try:
                r = run_sharded_case(a.case, a.steps, a.warmup, rank, world)
                if rank == 0:
                    print(json.dumps(r))
                torch.cuda.synchronize()
            finally:
                dist.destroy_process_group()
            return
        print(json.dumps(run_case(a.case, a.steps, a.warmup, a.flush)))
        return

    import torch
    import torch.distributed as dist

    from gc_b200 import api, lib, partitions
    from gc_b200 import benchgc_compat as bc
    from gc_b200.tensor_parallel import TensorParallelMLP, shard_weights

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- synthetic inputs (benchgc fills: seed + argument index)
    X_host = bc.fill_tensor((BATCH, HIDDEN[0]), "bf16", "N", (0, 1), 0).pin_memory()
    W_host = [bc.fill_tensor((HIDDEN[i], HIDDEN[i + 1]), "bf16", "N", (0, 0.02), 1 + i) for i in range(4)]
    B_host = [torch.zeros(HIDDEN[i + 1], dtype=torch.bfloat16) for i in range(4)]
    out_host = torch.empty(BATCH, HIDDEN[-1], dtype=torch.bfloat16).pin_memory()
    flops = mlp_flops()

    if world == 1:
        js, in_ids, out_id = partitions.mlp(BATCH, HIDDEN, "bf16", [True] * 4, "relu", constant_weights=True)
        exe = api.GraphCompiler().compile(js)
        Xd = X_host.to(dev)
        Wd = [w.to(dev) for w in W_host]
        Bd = [b.to(dev) for b in B_host]
        outd = torch.empty(BATCH, HIDDEN[-1], dtype=torch.bfloat16, device=dev)
        dev_in, dev_out = dict(zip(in_ids, [Xd] + Wd + Bd)), {out_id: outd}

        def step_device():
            exe.execute_on_stream(dev_in, dev_out)

        W_pin = [w.pin_memory() for w in W_host]
        B_pin = [b.pin_memory() for b in B_host]
        host_in, host_out = dict(zip(in_ids, [X_host] + W_pin + B_pin)), {out_id: out_host}

        bound = exe.bind(host_in, host_out)   # tensor structs built once, as a C caller would

        def step_e2e():
            bound.run()   # dnnl_graph_compiler_execute: H2D of X, 4 launches, D2H of the result, synchronous

        parallelism = "single GPU"
    fused_note = ""
    use_fused = world > 1 and os.environ.get("GC_B200_EXCHANGE", "fused_counters") == "fused_counters"
    if use_fused:
        # The tensor-parallel step behind the C ABI (gcb200_tp_mlp_*): GEMMs, exchange and every hand-off between the
        # GPUs are this library's own kernels; the step is replayed as a CUDA graph inside the library.
        from gc_b200.tensor_parallel import FusedTensorParallelMLP

        ws, bs = shard_weights([w.to(dev) for w in W_host], [b.to(dev) for b in B_host], world, rank)
        tpf = FusedTensorParallelMLP(ws, bs, BATCH, HIDDEN, dev, relu=True)
        Xd = X_host.to(dev)
        holder = {}
        # Every rank must come through one eager step, one captured step and one host-buffer call with a clean error
        # word; if any rank does not (a bounded wait ran out), all ranks fall back to the Python-driven exchange.
        ok = 1
        try:
            for _ in range(2):
                tpf.step(Xd)
            torch.cuda.synchronize()
            tpf.execute(X_host, None)
            ok = 1 if lib.device_error() == 0 else 0
        except Exception as e:
            ok, fused_note = 0, f"{type(e).__name__}: {e}"[:160]
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            use_fused = False
            fused_note = "fused tensor-parallel step failed its self-check on some rank" + (f" ({fused_note})" if fused_note else "")
            try:
                tpf.close()
            except Exception:
                pass

    if world > 1 and use_fused:

        if a.tp_timeline:
            for _ in range(a.warmup):
                tpf.step(Xd)
            torch.cuda.synchronize()
            dist.barrier()
            lines = []
            for _ in range(max(1, min(a.steps, 5))):
                lines.append(tpf.plan.timeline(Xd.data_ptr()))
            if rank == 0:
                print(f"tp{world} MLP step, rank 0, last of {len(lines)} eagerly launched steps (microseconds from the end of the "
                      "launch before to the end of this one):")
                print(lines[-1])
            # the same step as the bench times it (one CUDA-graph replay per step, back to back), read from the time
            # stamps the kernels write themselves
            dist.barrier()
            for _ in range(max(4, a.warmup)):
                tpf.step(Xd)
            torch.cuda.synchronize()
            trace = tpf.plan.trace()
            if rank == 0:
                print(f"tp{world} MLP step, rank 0, last of back-to-back graph replays, device time stamps:")
                print(trace)
            assert lib.device_error() == 0
            dist.barrier()
            tpf.close()
            dist.destroy_process_group()
            return

        def step_device():
            holder["y"] = tpf.step(Xd)

        def step_e2e():
            # gcb200_tp_mlp_execute: each rank copies its row block of the input over its own PCIe link, the blocks
            # cross NVLink, the step runs, rank 0 reads the whole result back; returns when all of it has finished
            holder["y"] = tpf.execute(X_host, out_host if rank == 0 else None)

        parallelism = (f"tp{world} behind the C ABI: row-parallel partial sums leave the GEMM epilogue for the rank that owns the rows "
                       "(peer stores), the owner reduces and stores the bf16 rows to every rank; hand-offs are device counters of "
                       "this library's kernels; one CUDA-graph replay per step")
    elif world > 1:
        from gc_b200.tensor_parallel import AllReduceExchange, CudaOps, PeerPushExchange, PeerReduceScatterExchange

        ws, bs = shard_weights([w.to(dev) for w in W_host], [b.to(dev) for b in B_host], world, rank)
        exchange, why = None, (" [" + fused_note + "]" if fused_note else "")
        # fused GEMM-epilogue exchanges: with two ranks sending the whole tile to the one peer is already minimal;
        # beyond that the partial sums are reduce-scattered by rows and the result all-gathered
        # every partial sum to every rank costs (g - 1) x 8 MiB of NVLink stores per rank and exchange: best at two ranks
        # (211 us per step against 228); the reduce-scatter form moves an all-reduce's traffic and wins beyond
        # (4 ranks: 171 us against 203; 8 ranks: 145 us against 289)
        want = os.environ.get("GC_B200_EXCHANGE", "fused_counters")
        if want == "fused_counters":
            want = "peer_push" if world <= 2 else "peer_reduce_scatter"
        if want in ("peer_push", "peer_push_multicast", "peer_reduce_scatter"):
            try:
                if want == "peer_reduce_scatter":
                    exchange = PeerReduceScatterExchange(BATCH, HIDDEN[-1], dev)
                else:
                    exchange = PeerPushExchange(BATCH, HIDDEN[-1], dev, multicast=(want == "peer_push_multicast"))
            except Exception as e:   # symmetric memory unavailable: NCCL all-reduce baseline
                why = f" (fused exchange unavailable: {type(e).__name__})"
        if exchange is None:
            exchange = AllReduceExchange(CudaOps())
        tp = TensorParallelMLP(ws, bs, relu=True, exchange=exchange)
        Xd = X_host.to(dev)
        holder = {}

        # One tensor-parallel step is 8 launches driven from Python; replay it as a CUDA graph so that the host
        # is out of the timed loop (every rank must take the same decision: all-reduce the outcome).
        graph, x_static = None, torch.empty_like(Xd)
        # Only with the peer-store exchange: a graph that holds NCCL kernels kept the communicator's
        # tear-down waiting at exit on this pool.
        if os.environ.get("GC_B200_TP_GRAPH", "1") != "0" and exchange.name != "all_reduce":
            ok = 1
            try:
                for _ in range(3):
                    tp.step(x_static)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                l0 = lib.launch_count()
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    holder["y"] = tp.step(x_static)
                holder["launches_per_replay"] = lib.launch_count() - l0   # this library's kernels inside the graph
                torch.cuda.synchronize()
            except Exception as e:   # capture not possible with this exchange: eager launches
                ok, graph = 0, None
                why += f" (graph capture failed: {type(e).__name__})"
                torch.cuda.synchronize()
            flag = torch.tensor([ok], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                graph = None

        def step_device():
            if graph is not None:
                x_static.copy_(Xd)     # device-to-device: the graph reads its own input buffer
                graph.replay()
                holder["replays"] = holder.get("replays", 0) + 1
            else:
                holder["y"] = tp.step(Xd)

        def step_e2e():
            if graph is not None:
                x_static.copy_(X_host, non_blocking=True)
                graph.replay()
                holder["replays"] = holder.get("replays", 0) + 1
                y = holder["y"]
            else:
                y = tp.step(X_host.to(dev, non_blocking=True))
            if rank == 0:
                out_host.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        parallelism = (f"tp{world}: layers 1,3 column-parallel, layers 2,4 row-parallel, f32 partial sums exchanged by "
                       + {"peer_push": "GEMM-epilogue peer stores over NVLink (every rank receives every partial sum) + local reduce",
                          "peer_push_multicast": "GEMM-epilogue multimem stores (one NVLink crossing per chunk, the NVSwitch writes every "
                                                 "rank's copy) + local reduce",
                          "peer_reduce_scatter": "GEMM-epilogue peer stores over NVLink to the row owner (reduce-scatter), owner reduces "
                                                 "and stores the bf16 rows to every rank (all-gather)",
                          "all_reduce": "NCCL all-reduce"}[exchange.name] + ("; one CUDA-graph replay per step" if graph is not None else "") + why)
    exchange_note = parallelism

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, sample_clocks=False):
        for _ in range(warmup):
            fn()
        barrier()
        sampler = make_clock_sampler(local_rank) if sample_clocks else None
        if sampler:
            sampler.start()
        l0 = lib.launch_count()
        r0 = holder.get("replays", 0) if world > 1 else 0
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        for _ in range(steps):
            fn()
        en.record()
        barrier()
        launches = lib.launch_count() - l0
        if world > 1:   # kernels launched by torch graph replays are not seen by the library's host-side counter
            launches += (holder.get("replays", 0) - r0) * holder.get("launches_per_replay", 0)
        ms = st.elapsed_time(en)
        clocks = sampler   # still running: it also covers the end-to-end region that follows and is stopped there
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, launches, clocks

    ms_dev, launches, sampler = timed(step_device, a.steps, a.warmup, sample_clocks=True)
    ms_e2e, _, _ = timed(step_e2e, max(3, a.steps // 2), a.warmup)
    clocks = sampler.stop()   # sampled from the start of the device-timed region to the end of the end-to-end one
    # The timed region above is milliseconds long (a burst at full clock).  The same step back to back for about two
    # seconds shows what the GPU holds once the power cap acts; compared with the sustained cuBLAS figure of this pool.
    sustained = None
    if a.sustained_seconds > 0:
        s2 = make_clock_sampler(local_rank)
        barrier()
        s2.start()
        n_s = max(a.steps, int(a.sustained_seconds * 1e3 / max(ms_dev, 1e-3)))
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        for _ in range(n_s):
            step_device()
        en.record()
        barrier()
        ms_s = st.elapsed_time(en) / n_s
        c2 = s2.stop()
        if world > 1:
            t = torch.tensor([ms_s], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_s = float(t.item())
        sustained = {"value": flops / ms_s / 1e9, "unit": "TFLOPS", "ms_per_step": ms_s, "steps": n_s, "seconds": ms_s * n_s / 1e3,
                     "sm_mhz_median": c2.get("sm_mhz"), "reasons": c2.get("reasons"),
                     "ms_x_mhz": (ms_s * c2["sm_mhz"] if c2.get("sm_mhz") else None)}
    assert lib.device_error() == 0, "a kernel reported a bounded-wait time-out"

    # ---- the step that was timed computed the right thing: 16 rows of its output against the CPU oracle (rank 0)
    parity = None
    if rank == 0:
        parity = parity_rows(outd if world == 1 else holder["y"], X_host, W_host, B_host)
    peaks = measured_peaks()
    gemm_launches = launches  # every launch in the timed region is one of this library's kernels
    per_launch_ms = ms_dev * a.steps / max(launches, 1)
    flops_per_launch = flops / (launches / a.steps) / world
    achieved = flops_per_launch / per_launch_ms / 1e9
    region_s = ms_dev * a.steps / 1e3
    peak_kind = "sustained" if region_s >= 1.0 else "burst"
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        traffic = json.load(open(tpath)).get("gemm_kernel_mlp_layer_bytes_per_launch")

    line = {
        "metric": "TFLOPS", "value": flops / ms_dev / 1e9, "unit": "TFLOPS", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config,
        "e2e": {"value": flops / ms_e2e / 1e9, "unit": "TFLOPS", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": X_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
                "note": ("weights are property_type=constant: uploaded by the first (warm-up) call, resident afterwards; the first and "
                         "last layer run as two row blocks so that the H2D / D2H copies overlap the other block's math") if world == 1 else
                        "per step: H2D of the activations on every rank, the tensor-parallel step, D2H of the result on rank 0"},
        "gpu_launches": int(gemm_launches),
        "exchange": exchange_note,
        "parity": parity,
        "sustained": sustained,
        "ms_x_mhz": (ms_dev * clocks["sm_mhz"] if clocks.get("sm_mhz") else None),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks[peak_kind], "unit": "TFLOP/s", "frac": achieved / peaks[peak_kind],
                     "traffic": traffic, "peak_source": f"{peaks['source']} cuBLAS bf16 {peak_kind}",
                     "kernel": "gemm_kernel<bf16, f32 accumulate> (tcgen05 + TMA), incl. launch gaps",
                     "frac_of_vendor_dense_2250": achieved / 2250.0},
    }
    if sustained is not None:
        sustained["frac_of_measured_sustained_peak"] = sustained["value"] / world / peaks["sustained"]
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        r = cpu_reference_run(1, 0)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        try:
            line["cpu_onednn_class"] = cpu_onednn_class()
        except Exception as e:  # context only
            line["cpu_onednn_class"] = {"error": repr(e)[:100]}
    if a.sweep and world == 1:
        line["sweep"] = [run_case(c, 10 if "16384" in c else 20, 3, library=True) for c in SWEEP]
    if a.sweep and world > 1:
        # the other configs that shard, at this number of ranks (strong scaling; the 1-GPU figures are in the N=1 line's sweep)
        if "tpf" in locals():
            tpf.close()
        sharded = []
        for c in SHARDED:
            try:
                sharded.append(run_sharded_case(c, 5 if "16384" in c else 10, 3, rank, world))
            except Exception as e:   # one case must not take the line down
                sharded.append({"case": c, "error": f"{type(e).__name__}: {e}"[:200]})
        line["sharded"] = sharded
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        # release the captured graph and the symmetric buffers before the process group goes away
        holder.clear()
        graph = None
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
