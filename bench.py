#!/usr/bin/env python
"""Benchmark of the adaptive hybrid quantization path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline metric (BASELINE.json): decode dequant-GEMV HBM GB/s on the
Llama-2-7B-shaped quantized linears (32 layers x q/k/v/o 4096x4096, gate/up
11008x4096, down 4096x11008), batch 1, bf16 activations.  One step = one pass
over all 224 linears (6.5 G weights, 6.7 GB of quantized data: every step
streams far more than the 126 MB L2, so nothing is served from cache).

  value     algorithmic bytes of a step / device time, inputs resident in HBM,
            the step replayed from a CUDA graph (one launch per linear)
  e2e       the same pass through QuantizedLinear.forward with host activations:
            every step copies the activations from pinned host memory to the
            device, replays a CUDA graph captured from the 224 module calls and
            copies all 224 outputs back to pinned host memory, inside the timed
            region (`extra.e2e_eager_gbs`: the same with copy-in, call and
            copy-out issued per linear from Python, no graph)
  extra     the other two figures BASELINE.json names (prefill GEMM TFLOP/s,
            quantize GB/s), GEMV at batch 4 and 16 and, with --gpus > 1, the
            70B-shaped column-parallel decode (batch 32, NCCL all-gather)

With --gpus N > 1 every rank runs the same pass on its own GPU (replicas, no
collective: the path shards by independent tensors) and `value` is the sum over
ranks / max time over ranks ("weak").  --impl reference times the reference's
forward on the host cores (rank 0 only): torch CPU F.linear on the cached fp16
weight, with the first-call dequantization (CPU oracle port) reported beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

LLAMA7B = dict(hidden=4096, inter=11008, layers=32)
LLAMA7B_LINEARS = [("q_proj", 4096, 4096), ("k_proj", 4096, 4096), ("v_proj", 4096, 4096),
                   ("o_proj", 4096, 4096), ("gate_proj", 11008, 4096), ("up_proj", 11008, 4096),
                   ("down_proj", 4096, 11008)]
LLAMA70B_LINEARS = [("q_proj", 8192, 8192), ("k_proj", 1024, 8192), ("v_proj", 1024, 8192),
                    ("o_proj", 8192, 8192), ("gate_proj", 28672, 8192), ("up_proj", 28672, 8192),
                    ("down_proj", 8192, 28672)]
BLOCK = 128
NO_GRAPH = False


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), tf_burst=float(p["bf16_tflops"]),
                    tf_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------- synthetic data
def synth_weight(n, k, gen, sigma=0.02, device="cuda"):
    """fp16 N(0, sigma) with 0.1 % of the entries replaced by +-U(0.1, 0.5) (seeded)."""
    w = torch.randn(n, k, generator=gen, device=device) * sigma
    cnt = round(1e-3 * n * k)
    pos = torch.randint(0, n * k, (cnt,), generator=gen, device=device)
    mag = torch.rand(cnt, generator=gen, device=device) * 0.4 + 0.1
    sgn = torch.where(torch.rand(cnt, generator=gen, device=device) < 0.5, -1.0, 1.0)
    w.view(-1)[pos] = mag * sgn
    return w.to(torch.float16)


def linear_bytes(n, k, n_out, m):
    """Algorithmic bytes of one quantized linear call: codes + scales + outliers (2 B value,
    4 B index) + activations in and out."""
    return (n * k - n_out) + (n * k // BLOCK) * 2 + n_out * 6 + m * k * 2 + m * n * 2


class Linear:
    """Device-resident kernel image of one quantized linear (canonical code stream dropped)."""

    def __init__(self, w, keep_module=False):
        import atlasinfer_b200 as ab
        from atlasinfer_b200.integration import atlas_wrappers as aw
        q = ab.quantize_tensor(w)
        self.n, self.k = w.shape
        self.n_out = q.fp16_outliers.numel()
        lay = aw.build_kernel_layout(q)
        torch.cuda.current_stream().synchronize()
        # the kernels read only the repacked layout; the canonical streams are not needed afterwards
        slim = ab.QuantizedTensor(torch.empty(0, dtype=torch.int8, device=w.device),
                                  torch.empty(0, dtype=torch.float16, device=w.device),
                                  torch.empty(0, dtype=torch.long, device=w.device),
                                  torch.empty(0, dtype=torch.float16, device=w.device),
                                  q.original_shape, q.block_size)
        self.q = slim
        self.layout = lay._replace(source=slim)
        self.module = None
        if keep_module:
            self.module = ab.QuantizedLinear(slim, None)
            self.module._kernel_layout = self.layout

    def forward(self, x, force=None):
        from atlasinfer_b200.integration import atlas_wrappers as aw
        return aw.quantized_linear_forward(x, self.layout, None, force)


def build_model(linears, layers, gen, sigma, rows_slice=None, keep_module=False):
    """`layers` x the given linears; rows_slice=(rank, world) keeps this rank's output rows."""
    out = []
    for _ in range(layers):
        for name, n, k in linears:
            if rows_slice is not None:
                r, wsz = rows_slice
                n = n // wsz
            w = synth_weight(n, k, gen, sigma)
            out.append((name, Linear(w, keep_module)))
            del w
    return out


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        # samples under load: the upper half of the observed clocks
        busy = sm[len(sm) // 2:] if sm else []
        med = busy[len(busy) // 2] if busy else None
        return dict(sm_mhz=med, sm_max_mhz=max(smax) if smax else None, reasons=sorted(reasons), samples=len(sm))


# ----------------------------------------------------------------------------- timing helpers
def time_steps(fn, steps, warmup, barrier=None):
    """Device time of `steps` calls of fn after `warmup` untimed ones (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[steps]) / 1e3  # seconds


def capture_graph(fn):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


# ----------------------------------------------------------------------------- measurements
def measure_gemv(model, m, steps, warmup, barrier=None, dtype=torch.bfloat16):
    """(bytes per step, seconds for `steps`, launches per step) of a graph-replayed decode pass."""
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(7 + m)
    xs = {k: torch.randn(m, k, generator=gen, device=dev).to(dtype) for k in {l.k for _, l in model}}
    outs = []

    def one_pass():
        outs.clear()
        for _, lin in model:
            outs.append(lin.forward(xs[lin.k]))   # the library's own dispatch for this batch size

    if NO_GRAPH:
        secs = time_steps(one_pass, steps, warmup, barrier)
    else:
        graph = capture_graph(one_pass)
        secs = time_steps(graph.replay, steps, warmup, barrier)
    nbytes = sum(linear_bytes(l.n, l.k, l.n_out, m) for _, l in model)
    return nbytes, secs, len(model)


def measure_e2e(model, m, steps, warmup, barrier=None, dtype=torch.bfloat16, eager=False):
    """The decode pass through the public module API (`QuantizedLinear.forward`) with host-resident activations.

    Every step copies the step's activations from pinned host memory to the device, runs the 224 module
    calls and copies all 224 outputs back to pinned host memory, then waits for them.  Default: the module
    calls are captured once in a CUDA graph (the way a serving loop drives a decode step) that reads static
    input tensors; `eager=True` instead issues copy-in, call, copy-out per linear from Python."""
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(11)
    hx = {k: torch.randn(m, k, generator=gen).to(dtype).pin_memory() for k in {l.k for _, l in model}}
    nbytes = sum(linear_bytes(l.n, l.k, l.n_out, m) for _, l in model)
    if eager:
        hy = {n: torch.empty(m, n, dtype=dtype).pin_memory() for n in {l.n for _, l in model}}

        def one_pass():
            for _, lin in model:
                x = hx[lin.k].to(dev, non_blocking=True)
                y = lin.module(x)
                hy[lin.n].copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller holds y on the host

        secs = time_steps(one_pass, steps, warmup, barrier)
        return nbytes, secs, sum(m * l.k * 2 for _, l in model), sum(m * l.n * 2 for _, l in model)

    dx = {k: torch.empty(m, k, dtype=dtype, device=dev) for k in hx}
    total_out = sum(m * l.n for _, l in model)
    hy = torch.empty(total_out, dtype=dtype).pin_memory()
    for k in hx:
        dx[k].copy_(hx[k])
    for _, lin in model[:8]:
        lin.module(dx[lin.k])           # warm the call path before capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = [lin.module(dx[lin.k]) for _, lin in model]
        flat = torch.cat([o.reshape(-1) for o in outs])

    def one_pass():
        for k in hx:
            dx[k].copy_(hx[k], non_blocking=True)
        graph.replay()
        hy.copy_(flat, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller holds every output on the host

    secs = time_steps(one_pass, steps, warmup, barrier)
    return nbytes, secs, sum(m * k * 2 for k in hx), total_out * 2


def measure_gemm(steps, warmup):
    """Prefill GEMM TFLOP/s: 2048 tokens against 11008x4096 and 4096x4096 (config 4)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(99)
    res = {}
    for n, k in ((11008, 4096), (4096, 4096)):
        # several distinct weights so that consecutive calls do not re-read one from L2
        reps = 4
        lins = [Linear(synth_weight(n, k, gen)) for _ in range(reps)]
        x = torch.randn(2048, k, generator=gen, device=dev).to(torch.bfloat16)
        ch = torch.randperm(k, generator=gen, device=dev)[: max(1, round(0.005 * k))]
        x[:, ch] *= 20

        def one():
            for l in lins:
                l.forward(x, "gemm")

        secs = time_steps(one, steps, warmup)
        res[f"{n}x{k}"] = 2.0 * 2048 * n * k * reps * steps / secs / 1e12
        del lins
    return res


def measure_quantize(steps, warmup):
    """Quantize GB/s on the 7B shapes: algorithmic bytes = 2 B read + codes + scales + 10 B per outlier."""
    import atlasinfer_b200 as ab
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(5)
    ws = [synth_weight(n, k, gen) for n, k in ((11008, 4096), (4096, 11008), (4096, 4096), (11008, 4096))]
    nbytes = 0
    for w in ws:
        q = ab.quantize_tensor(w)
        n_out = q.fp16_outliers.numel()
        nbytes += 2 * w.numel() + (w.numel() - n_out) + (w.numel() // BLOCK) * 2 + n_out * 10

    def one():
        for w in ws:
            ab.quantize_tensor(w)

    secs = time_steps(one, steps, warmup)
    return nbytes * steps / secs / 1e9


def measure_quantize_kernel(steps, warmup):
    """The quantize kernel alone, through the C ABI with caller-owned buffers and no host synchronisation
    (quantize_tensor adds allocations, a device-to-host read of the two stream lengths and two trims)."""
    from atlasinfer_b200 import _capi
    L = _capi.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(5)
    ws = [synth_weight(n, k, gen) for n, k in ((11008, 4096), (4096, 11008), (4096, 4096), (11008, 4096))]
    bufs, nbytes = [], 0
    for w in ws:
        flat = w.reshape(-1)
        n = flat.numel()
        cap = n // 8 + 1024
        b = dict(flat=flat, n=n, cap=cap, codes=torch.empty(n, dtype=torch.int8, device=dev),
                 ovals=torch.empty(cap, dtype=torch.float16, device=dev), oidx=torch.empty(cap, dtype=torch.int64, device=dev),
                 scales=torch.empty(n // BLOCK, dtype=torch.float16, device=dev),
                 counts=torch.zeros(4, dtype=torch.int64, device=dev))
        b["ws_bytes"] = int(L.atlas_quantize_workspace_bytes(n, BLOCK))
        b["ws"] = torch.empty(b["ws_bytes"], dtype=torch.uint8, device=dev)
        bufs.append(b)
    stream = _capi.stream_ptr(dev)

    def one():
        for b in bufs:
            rc = L.atlas_quantize(b["flat"].data_ptr(), b["n"], BLOCK, 3.0, b["codes"].data_ptr(), b["ovals"].data_ptr(),
                                  b["oidx"].data_ptr(), b["cap"], b["scales"].data_ptr(), b["counts"].data_ptr(),
                                  b["ws"].data_ptr(), b["ws_bytes"], stream)
            _capi.check(rc, "atlas_quantize")

    one()
    torch.cuda.synchronize()
    for b in bufs:
        n_codes, n_out, timed_out, _ = b["counts"].tolist()
        assert not timed_out and n_codes + n_out == b["n"]
        nbytes += 2 * b["n"] + n_codes + (b["n"] // BLOCK) * 2 + n_out * 10
    secs = time_steps(one, steps, warmup)
    return nbytes * steps / secs / 1e9


def measure_tp70b(rank, world, steps, warmup, barrier):
    """Config 5: Llama-3-70B-shaped decode, batch 32, column-parallel over `world` ranks.

    Every rank owns rows [r*N/g, (r+1)*N/g) of each linear (8 distinct layers, cycled ten times to
    stand for the 80 layers; one layer's shards already exceed L2 together with the gathers) and
    all-gathers its [32, N/g] output shard over NCCL.  Returns ms per token with and without the
    gathers, and the aggregate algorithmic GB/s of the weight streaming.
    """
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(777 + rank)
    layers, reps, m = 8, 10, 32
    model = build_model(LLAMA70B_LINEARS, layers, gen, 0.015, rows_slice=(rank, world))
    xs = {k: torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16) for k in {l.k for _, l in model}}
    gathered = {l.n: torch.empty(world * m, l.n, dtype=torch.bfloat16, device=dev) for _, l in model}

    def one_pass(gather):
        for _ in range(reps):
            for _, lin in model:
                y = lin.forward(xs[lin.k])
                if gather and world > 1:
                    dist.all_gather_into_tensor(gathered[lin.n], y)

    out = {}
    for name, gather in (("with_allgather", True), ("gemv_only", False)):
        fn = lambda: one_pass(gather)  # noqa: E731
        try:
            graph = capture_graph(fn)
            run = graph.replay
            mode = "graph"
        except Exception:  # noqa: BLE001 - capture of the collective not available: launch directly
            torch.cuda.synchronize()
            run, mode = fn, "eager"
        secs = time_steps(run, steps, warmup, barrier)
        t = torch.tensor([secs], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = dict(ms_per_token=float(t.item()) / steps * 1e3, launch=mode)
    nbytes = sum(linear_bytes(l.n, l.k, l.n_out, m) for _, l in model) * reps
    tot = torch.tensor([float(nbytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tot)
    out["aggregate_gbs_with_allgather"] = float(tot.item()) / (out["with_allgather"]["ms_per_token"] * 1e-3) / 1e9
    out["aggregate_gbs_gemv_only"] = float(tot.item()) / (out["gemv_only"]["ms_per_token"] * 1e-3) / 1e9
    out["config"] = "llama3-70b-shaped linears, 80 layers (8 distinct x 10), batch 32 bf16, rows sharded over %d ranks" % world
    del model
    torch.cuda.empty_cache()
    return out


def measure_quantize_sharded(rank, world, steps, warmup, barrier):
    """Whole-model quantization sharded by layer: every rank quantizes whole layers of its own
    (one 70B-shaped layer per step here), no collective.  Aggregate algorithmic GB/s."""
    import torch.distributed as dist
    import atlasinfer_b200 as ab
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(4242 + rank)
    ws = [synth_weight(n, k, gen, 0.015) for _, n, k in LLAMA70B_LINEARS]
    nbytes = 0
    for w in ws:
        q = ab.quantize_tensor(w)
        n_out = q.fp16_outliers.numel()
        nbytes += 2 * w.numel() + (w.numel() - n_out) + (w.numel() // BLOCK) * 2 + n_out * 10

    def one():
        for w in ws:
            ab.quantize_tensor(w)

    secs = time_steps(one, steps, warmup, barrier)
    t = torch.tensor([secs], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return world * nbytes * steps / float(t.item()) / 1e9


def cpu_linear_pass(linears, m):
    """The reference's forward on the host cores over `linears` [(n, k)].

    integration/atlas_wrappers.py:54-67 calls dequantize_tensor (adaptive_quantizer.py:156, which keeps the
    fp16 reconstruction in a cache keyed by the weight object) and then F.linear: the first call of a
    layer pays the dequantization, every later call multiplies by the cached fp16 weight.  Both are
    timed: the steady state with torch's own CPU F.linear on fp16 tensors (the very call the reference
    makes; fp32 if this torch build has no fp16 CPU matmul), the first call with the oracle's
    dequantizer in front of it.  Returns (algorithmic bytes, steady-state seconds, first-call seconds);
    the bytes are those of the quantized format, so the figure is comparable with the GPU lines.
    Weights are quantized (untimed) by the oracle first."""
    import torch.nn.functional as F
    from oracle import atlas_oracle as O
    gen = torch.Generator().manual_seed(3)
    prepared = []
    for n, k in linears:
        w = (torch.randn(n, k, generator=gen) * 0.02)
        cnt = round(1e-3 * n * k)
        w.view(-1)[torch.randint(0, n * k, (cnt,), generator=gen)] = 0.3
        q = O.quantize(w.half())
        x = torch.randn(m, k, generator=gen).half()
        prepared.append((q, x, linear_bytes(n, k, q.fp16_outliers.numel(), m)))
    t0 = time.perf_counter()
    cached = [O.dequantize(q) for q, _, _ in prepared]          # the reference's per-weight cache
    t_dequant = time.perf_counter() - t0
    try:
        F.linear(prepared[0][1], cached[0])
        xs = [x for _, x, _ in prepared]
    except RuntimeError:                                         # no fp16 matmul on this CPU build
        cached = [c.float() for c in cached]
        xs = [x.float() for _, x, _ in prepared]
    reps = 5
    t0 = time.perf_counter()
    for _ in range(reps):
        for x, wd in zip(xs, cached):
            F.linear(x, wd)
    t_steady = (time.perf_counter() - t0) / reps
    return sum(b for _, _, b in prepared), t_steady, t_steady + t_dequant


# ----------------------------------------------------------------------------- arms
def run_reference(args, rank, world):
    """CPU arm: the oracle port of the quantized linear forward on the host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import atlas_oracle as O
    O.build()
    sample = [(4096, 4096), (11008, 4096), (4096, 11008)]
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_linear_pass(sample[:1], 1)
    t_all, t_first, b_all = 0.0, 0.0, 0
    for _ in range(args.steps):
        b, t, tf = cpu_linear_pass(sample, 1)
        t_all += t
        t_first += tf
        b_all += b
    val = b_all / t_all / 1e9
    cores = torch.get_num_threads()
    desc = ("per step: q_proj 4096x4096 + gate_proj 11008x4096 + down_proj 4096x11008 at batch 1; steady state of "
            "the reference's forward = torch CPU F.linear on the cached fp16 weight; the first call of a layer "
            f"(dequantize_tensor, CPU oracle port, OpenMP, then F.linear) runs at {b_all / t_first / 1e9:.3f} GB/s")
    line = dict(
        impl="reference", metric="dequant_gemv_hbm_gbs", value=val, unit="GB/s", n_gpus=args.gpus,
        steps=args.steps, warmup=args.warmup, ms_per_step=t_all / args.steps * 1e3, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="fp16 weight rebuilt from int8 codes x fp16 scales (cached), torch CPU matmul",
        data="synthetic", config=workload_config(1), gpu_launches=0,
        cpu_baseline=dict(value=val, unit="GB/s", cores=cores, kind="port", sample=desc),
        e2e=dict(value=val, unit="GB/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


NCU_DRAM_BYTES_PER_WEIGHT = 1.039   # dram__bytes_read.sum + dram__bytes_write.sum per weight of gemv_strip_kernel


def weights_per_layer(linears):
    return float(sum(n * k for _, n, k in linears))


def workload_config(m):
    return dict(workload="llama2-7b decode linears: 32 layers x (q,k,v,o 4096x4096; gate,up 11008x4096; "
                         "down 4096x11008), block 128, z 3.0, weights N(0,0.02)+0.1% outliers",
                batch=m, activations="bf16 N(0,1)", l2="each step streams 6.7 GB of weights (>> 126 MB L2)",
                launch="one kernel per linear, step replayed from a CUDA graph")


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from atlasinfer_b200 import _capi
    _capi.load()  # fail here, loudly, if the CUDA library is missing
    barrier = None
    if world > 1:
        os.environ["NCCL_DEBUG"] = os.environ.get("ATLAS_NCCL_DEBUG", "WARN")  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
        barrier = dist.barrier
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    t_setup = time.perf_counter()
    model = build_model(LLAMA7B_LINEARS, args.layers, gen, 0.02, keep_module=True)
    torch.cuda.synchronize()
    t_setup = time.perf_counter() - t_setup

    sampler = ClockSampler(local_rank)
    sampler.start()
    nbytes, secs, launches = measure_gemv(model, 1, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    e_bytes, e_secs, h2d, d2h = measure_e2e(model, 1, args.steps, args.warmup, barrier)

    def allmax(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    secs, e_secs = allmax(secs), allmax(e_secs)
    value = world * nbytes * args.steps / secs / 1e9
    e2e_value = world * e_bytes * args.steps / e_secs / 1e9
    per_gpu = value / world

    extra = {}
    if rank == 0 and not args.headline_only:
        eb, es, _, _ = measure_e2e(model, 1, max(2, args.steps // 5), 2, eager=True)
        extra["e2e_eager_gbs"] = eb * max(2, args.steps // 5) / es / 1e9   # copy-in, call, copy-out per linear from Python
        for m in (4, 16):
            b, s, _ = measure_gemv(model, m, max(2, args.steps // 2), 3)
            extra[f"decode_m{m}_gbs"] = b * max(2, args.steps // 2) / s / 1e9
    del model
    torch.cuda.empty_cache()
    if world > 1 and not args.headline_only:
        try:
            tp = measure_tp70b(rank, world, max(2, args.steps // 5), 3, barrier)
            qs = measure_quantize_sharded(rank, world, 2, 1, barrier)
            if rank == 0:
                extra["tp70b_decode"] = tp
                extra["quantize_layer_sharded_gbs"] = qs
        except Exception as e:  # noqa: BLE001 - keep the headline line
            extra["tp70b_error"] = repr(e)
    if rank == 0 and not args.headline_only:
        try:
            extra["prefill_gemm_tflops"] = measure_gemm(max(2, args.steps // 4), 3)
            extra["quantize_gbs"] = measure_quantize(max(2, args.steps // 4), 3)
            extra["quantize_kernel_gbs"] = measure_quantize_kernel(max(2, args.steps // 4), 3)
        except Exception as e:  # noqa: BLE001 - secondary figures must not lose the headline line
            extra["error"] = repr(e)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import atlas_oracle as O
        O.build()
        b, t, tf = cpu_linear_pass([(4096, 4096), (11008, 4096)], 1)
        cpu = dict(value=b / t / 1e9, unit="GB/s", cores=torch.get_num_threads(), kind="port",
                   sample="q_proj 4096x4096 + gate_proj 11008x4096 at batch 1; steady state of the reference's "
                          "forward (torch CPU F.linear on the cached fp16 weight); with the first-call "
                          f"dequantization (CPU oracle port, OpenMP) in front: {b / tf / 1e9:.3f} GB/s")

    if rank == 0:
        line = dict(
            metric="dequant_gemv_hbm_gbs", value=value, unit="GB/s", n_gpus=world, steps=args.steps,
            warmup=args.warmup, ms_per_step=secs / args.steps * 1e3, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="int8 codes x fp16 scales -> fp16 MMA, fp32 accumulate", data="synthetic",
            config=dict(workload_config(1), layers=args.layers), clocks=clocks,
            e2e=dict(value=e2e_value, unit="GB/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                     method="per step: pinned-host activations -> device, CUDA-graph replay of the 224 "
                            "QuantizedLinear.forward calls, all 224 outputs -> pinned host, wait"),
            gpu_launches=launches * args.steps,
            roofline=dict(bound="hbm", achieved=per_gpu, peak=pk["hbm"], unit="GB/s", frac=per_gpu / pk["hbm"],
                          # DRAM bytes per launch, averaged over the step's launches: ncu measured 17.43 MB for a
                          # 4096x4096 linear and 46.82 MB for 4096x11008 (1.039 B per weight, equal to the
                          # algorithmic bytes); the 11008x4096 launches are taken at the same bytes per weight
                          traffic=NCU_DRAM_BYTES_PER_WEIGHT * weights_per_layer(LLAMA7B_LINEARS) / len(LLAMA7B_LINEARS),
                          traffic_unit="bytes per launch", algorithmic_bytes_per_launch=nbytes / launches,
                          avg_launch_us=secs / args.steps / launches * 1e6,
                          peak_source=pk["source"], kernel="gemv_strip_kernel",
                          frac_of_nominal_8tbs=per_gpu / 8000.0),
            cpu_baseline=cpu, extra=extra, setup_s=t_setup)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true", help="skip the secondary figures")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--layers", type=int, default=LLAMA7B["layers"],
                    help="decoder layers in the pass (default: the full 32; smaller only for profiler captures)")
    ap.add_argument("--no-graph", action="store_true", help="launch the pass directly instead of replaying a graph")
    ap.add_argument("--only", default=None, choices=["gemm", "quantize"],
                    help="run just one of the secondary measurements and print it (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    global NO_GRAPH
    NO_GRAPH = args.no_graph
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.only:
        torch.cuda.set_device(local_rank)
        if args.only == "gemm":
            out = {"gemm": measure_gemm(args.steps, args.warmup)}
        else:
            out = {"quantize": measure_quantize(args.steps, args.warmup),
                   "quantize_kernel": measure_quantize_kernel(args.steps, args.warmup)}
        print(json.dumps(out), flush=True)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
