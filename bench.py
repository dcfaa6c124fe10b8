#!/usr/bin/env python
"""Benchmark of the adaptive hybrid quantization path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline metric (BASELINE.json): decode dequant-GEMV HBM GB/s on the
Llama-2-7B-shaped quantized linears (32 layers x q/k/v/o 4096x4096, gate/up
11008x4096, down 4096x11008), batch 1, bf16 activations.  One step = one pass
over all 224 linears (6.5 G weights, 6.7 GB of quantized data: every step
streams far more than the 126 MB L2, so nothing is served from cache).  The
linears are `QuantizedLinear` modules built through the public API
(quantize_tensors -> QuantizedLinear -> fuse_linears for q/k/v and gate/up ->
offload_canonical), so a step is 4 launches per layer, 128 in all.

  value     algorithmic bytes of a step / device time, inputs resident in HBM,
            the step (the module calls) replayed from a CUDA graph
  e2e       the same pass with host activations: every step copies the
            activations from pinned host memory to the device, replays the
            graph and copies all 224 outputs back to pinned host memory, inside
            the timed region
  extra     the 70B-shaped column-parallel decode (batch 32) at this N, with the
            NCCL all-gather and with the kernels' own peer stores, and the
            layer-sharded quantization; in the single-GPU run also the figures
            that do not depend on N: the same pass without fusing (224
            launches), batch 4 / 16 / 32, batch 1 with fp16 activations (the
            reference's dtype), prefill GEMM TFLOP/s, quantize GB/s,
            the OPT-1.3B-architecture model end to end (quantize seconds,
            greedy decode tokens/s)

With --gpus N > 1 every rank runs the headline pass on its own GPU (replicas, no
collective: the path shards by independent tensors) and `value` is the sum over
ranks / max time over ranks ("weak"); the sharded 70B-shaped decode is the
config that communicates, reported per N in `extra.tp70b_decode`.
--impl reference times the reference's forward on the host cores (rank 0 only):
torch CPU F.linear on the cached fp16 weight, with the first-call
dequantization (CPU oracle port) reported beside it.
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
FUSED = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))
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


class Layer:
    """One decoder layer's quantized linears as the public API builds them."""

    def __init__(self, linears, gen, sigma, fuse, rows_slice=None):
        import atlasinfer_b200 as ab
        ws = []
        for _, n, k in linears:
            if rows_slice is not None:
                n = n // rows_slice[1]
            ws.append(synth_weight(n, k, gen, sigma))
        qs = ab.quantize_tensors(ws)                          # one host synchronisation for the layer
        del ws
        self.mods = {name: ab.QuantizedLinear(q, None) for (name, _, _), q in zip(linears, qs)}
        self.stats = {name: (int(q.original_shape[0]), int(q.original_shape[1]), q.fp16_outliers.numel())
                      for (name, _, _), q in zip(linears, qs)}
        self.groups = []
        if fuse:
            for names in FUSED:
                self.groups.append(ab.fuse_linears([self.mods[n] for n in names]))
        dev = qs[0].fp8_data.device
        for g in self.groups:
            g.build(dev)
        for mod in self.mods.values():
            mod.offload_canonical()        # the GPU keeps the kernel layout only (~1.03 B per weight)
        # the order a decoder layer calls them in; members of a fused group are called back to back with one input
        self.calls = list(self.mods.items())
        fused_names = {n for names in FUSED for n in names} if fuse else set()
        self.launches = len(self.groups) + sum(1 for n in self.mods if n not in fused_names)

    def nbytes(self, m):
        return sum(linear_bytes(n, k, no, m) for n, k, no in self.stats.values())


def build_model(linears, layers, gen, sigma, fuse=True, rows_slice=None):
    return [Layer(linears, gen, sigma, fuse, rows_slice) for _ in range(layers)]


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


def allmax(v, world, dev):
    if world == 1:
        return v
    import torch.distributed as dist
    t = torch.tensor([v], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ----------------------------------------------------------------------------- measurements
def decode_pass(model, xs, outs):
    """One decode step over `model`: every linear called through QuantizedLinear.forward with its input."""
    outs.clear()
    for layer in model:
        for name, mod in layer.calls:
            outs.append(mod(xs[mod.original_shape[1]]))


def measure_gemv(model, m, steps, warmup, barrier=None, dtype=torch.bfloat16):
    """(bytes per step, seconds for `steps`, launches per step) of a graph-replayed decode pass."""
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(7 + m)
    xs = {k: torch.randn(m, k, generator=gen, device=dev).to(dtype) for k in {s[1] for l in model for s in l.stats.values()}}
    outs = []
    fn = lambda: decode_pass(model, xs, outs)  # noqa: E731
    if NO_GRAPH:
        secs = time_steps(fn, steps, warmup, barrier)
    else:
        graph = capture_graph(fn)
        secs = time_steps(graph.replay, steps, warmup, barrier)
    return sum(l.nbytes(m) for l in model), secs, sum(l.launches for l in model)


def measure_e2e(model, m, steps, warmup, barrier=None, dtype=torch.bfloat16):
    """The decode pass with host-resident activations: per step the activations go from pinned host memory to the
    device, a CUDA graph captured from the module calls is replayed, all outputs go back to pinned host memory
    and the host waits for them."""
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(11)
    dims = {s[1] for l in model for s in l.stats.values()}
    hx = {k: torch.randn(m, k, generator=gen).to(dtype).pin_memory() for k in dims}
    dx = {k: torch.empty(m, k, dtype=dtype, device=dev) for k in hx}
    for k in hx:
        dx[k].copy_(hx[k])
    outs = []
    decode_pass(model, dx, outs)          # warm the call path before capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_pass(model, dx, outs)
        flat = torch.cat([o.reshape(-1) for o in outs])
    hy = torch.empty(flat.numel(), dtype=dtype).pin_memory()

    def one_pass():
        for k in hx:
            dx[k].copy_(hx[k], non_blocking=True)
        graph.replay()
        hy.copy_(flat, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller holds every output on the host

    secs = time_steps(one_pass, steps, warmup, barrier)
    return sum(l.nbytes(m) for l in model), secs, sum(m * k * 2 for k in hx), flat.numel() * 2


def measure_gemm(steps, warmup):
    """Prefill GEMM TFLOP/s: 2048 tokens against 11008x4096 and 4096x4096 (config 4)."""
    import atlasinfer_b200 as ab
    from atlasinfer_b200.integration import atlas_wrappers as aw
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(99)
    res = {}
    for n, k in ((11008, 4096), (4096, 4096)):
        # several distinct weights so that consecutive calls do not re-read one from L2
        reps = 4
        lays = [aw.build_kernel_layout(q) for q in ab.quantize_tensors([synth_weight(n, k, gen) for _ in range(reps)])]
        x = torch.randn(2048, k, generator=gen, device=dev).to(torch.bfloat16)
        ch = torch.randperm(k, generator=gen, device=dev)[: max(1, round(0.005 * k))]
        x[:, ch] *= 20

        def one():
            for lay in lays:
                aw.quantized_linear_forward(x, lay, None, "gemm")

        secs = time_steps(one, steps, warmup)
        res[f"{n}x{k}"] = 2.0 * 2048 * n * k * reps * steps / secs / 1e12
        del lays
    return res


def quantize_bytes(numel, n_out):
    return 2 * numel + (numel - n_out) + (numel // BLOCK) * 2 + n_out * 10


def measure_quantize(steps, warmup):
    """Quantize GB/s on the 7B shapes through the public API (quantize_tensors: one synchronisation per batch);
    algorithmic bytes = 2 B read + codes + scales + 10 B per outlier."""
    import atlasinfer_b200 as ab
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(5)
    ws = [synth_weight(n, k, gen) for n, k in ((11008, 4096), (4096, 11008), (4096, 4096), (11008, 4096))]
    nbytes = sum(quantize_bytes(w.numel(), q.fp16_outliers.numel()) for w, q in zip(ws, ab.quantize_tensors(ws)))
    secs = time_steps(lambda: ab.quantize_tensors(ws), steps, warmup)
    one = time_steps(lambda: [ab.quantize_tensor(w) for w in ws], steps, warmup)
    return nbytes * steps / secs / 1e9, nbytes * steps / one / 1e9


def measure_quantize_kernel(steps, warmup):
    """The quantize kernel alone, through the C ABI with caller-owned buffers and no host synchronisation."""
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
        nbytes += quantize_bytes(b["n"], n_out)
    secs = time_steps(one, steps, warmup)
    return nbytes * steps / secs / 1e9


def measure_opt13b():
    """Config 2: a random-init OPT-1.3B-architecture model quantized end to end on the GPU through the applier
    (fused q/k/v), then greedy decode of 128 new tokens from 128 seeded prompt ids (HF generate, eager)."""
    import atlasinfer_b200 as ab
    from transformers import OPTConfig, OPTForCausalLM
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = OPTConfig(vocab_size=50272, hidden_size=2048, ffn_dim=8192, num_hidden_layers=24, num_attention_heads=32,
                    max_position_embeddings=2048, word_embed_proj_dim=2048)
    with torch.device(dev):
        model = OPTForCausalLM(cfg).half().eval()
    gen = torch.Generator(device=dev).manual_seed(1234)
    n_weights = 0
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear) and "lm_head" not in name:
            mod.weight.data.copy_(synth_weight(*mod.weight.shape, gen))
            n_weights += mod.weight.numel()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ab.apply_atlas_quantization_to_model(model, "opt", {"block_size": BLOCK, "z_threshold": 3.0},
                                         keep_on_device=True, fuse=True, offload_canonical=True, verbose=False)
    torch.cuda.synchronize()
    t_quant = time.perf_counter() - t0
    ids = torch.randint(0, 50272, (1, 128), generator=torch.Generator().manual_seed(9)).to(dev)
    with torch.no_grad():
        model.generate(ids, max_new_tokens=4, min_new_tokens=4, do_sample=False)       # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model.generate(ids, max_new_tokens=128, min_new_tokens=128, do_sample=False)
        torch.cuda.synchronize()
        t_gen = time.perf_counter() - t0
    assert out.shape[1] == 256
    res = dict(linears=144, weights=n_weights, quantize_s=t_quant, quantize_gweights_per_s=n_weights / t_quant / 1e9,
               decode_tokens_per_s=128 / t_gen, decode="HF generate, eager, batch 1, 128 prompt + 128 new tokens")
    del model
    torch.cuda.empty_cache()
    return res


def measure_tp70b(rank, world, steps, warmup, barrier, all_forms=False, shard_of=None):
    """Config 5: Llama-3-70B-shaped decode, batch 32, column-parallel over `world` ranks.

    Every rank owns rows [r*N/g, (r+1)*N/g) of each linear (8 distinct layers, cycled ten times to stand for the
    80 layers; one layer's shards already exceed L2), q/k/v and gate/up fused into one launch each, and the
    [32, N/g] output shards are all-gathered after every launch: by NCCL (`nccl_allgather`), or by the ranks'
    own peer stores into symmetric buffers followed by a flag exchange (`peer_stores_stream`: in the streaming
    linear kernel's epilogue; `peer_stores_gemm`: in the tcgen05 path's second kernel; `peer_push`: a push kernel behind the default linear kernels; see
    atlasinfer_b200/peer.py).  Returns ms per token for each, the weight-streaming-only time and the aggregate
    algorithmic GB/s."""
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(777 + rank)
    layers, reps, m = 8, 10, 32
    # shard_of: time one rank's share of a `shard_of`-way split on this GPU alone (no gather partners)
    model = build_model(LLAMA70B_LINEARS, layers, gen, 0.015, fuse=True,
                        rows_slice=(rank, world) if shard_of is None else (0, shard_of))
    xs = {k: torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16) for k in (8192, 28672)}
    # what a layer launches: (kernel layout of the launch, output rows it produces on this rank)
    from atlasinfer_b200.integration import atlas_wrappers as aw
    launches = []
    for layer in model:
        by_first = {g.members[0]: g for g in layer.groups}
        for names in (("q_proj", "k_proj", "v_proj"), ("o_proj",), ("gate_proj", "up_proj"), ("down_proj",)):
            first = layer.mods[names[0]]
            lay = by_first[first].layout if first in by_first else first._kernel_layout
            launches.append((lay, lay.n_rows))
    widths = sorted({w for _, w in launches})
    gathered = {w: torch.empty(world * m, w, dtype=torch.bfloat16, device=dev) for w in widths}
    out = {}

    def one_pass(gather):
        for _ in range(reps):
            for lay, width in launches:
                y = aw.quantized_linear_forward(xs[lay.n_cols], lay, None)
                if gather and world > 1:
                    dist.all_gather_into_tensor(gathered[width], y)

    modes = [("gemv_only", False)] + ([("nccl_allgather", True)] if world > 1 else [])
    for name, gather in modes:
        fn = lambda: one_pass(gather)  # noqa: E731
        try:
            graph = capture_graph(fn)
            run, mode = graph.replay, "graph"
        except Exception:  # noqa: BLE001 - capture of the collective not available: launch directly
            torch.cuda.synchronize()
            run, mode = fn, "eager"
        secs = allmax(time_steps(run, steps, warmup, barrier), world, dev)
        out[name] = dict(ms_per_token=secs / steps * 1e3, launch=mode)
    # the ranks' own peer stores instead of the collective: fused into the streaming linear kernel, or as a push
    # kernel behind the default linear kernels (at one rank: the same launches, stores to the own buffer only)
    forms = [("peer_stores_gemm", "gemm")]
    if all_forms:
        forms += [("peer_stores_stream", "stream"), ("peer_push", "push")]
    for name, kernel in forms:
        try:
            out[name] = measure_tp_peer_stores(launches, xs, m, reps, steps, warmup, barrier, rank, world, dev, kernel)
        except Exception as e:  # noqa: BLE001 - keep the other figures
            out[name] = dict(error=repr(e))
    nbytes = sum(l.nbytes(m) for l in model) * reps
    tot = torch.tensor([float(nbytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tot)
    total = float(tot.item())
    pk = peaks()
    for name in list(out):
        if "ms_per_token" in out[name]:
            gbs = total / (out[name]["ms_per_token"] * 1e-3) / 1e9
            out[name]["aggregate_gbs"] = gbs
            out[name]["frac_of_n_x_hbm"] = gbs / (world * pk["hbm"])
    out["launches_per_token"] = len(launches) * reps
    out["config"] = ("llama3-70b-shaped linears, 80 layers (8 distinct x 10), batch 32 bf16, q/k/v and gate/up fused, "
                     "rows sharded over %d ranks" % world)
    del model
    torch.cuda.empty_cache()
    return out


def measure_tp_peer_stores(launches, xs, m, reps, steps, warmup, barrier, rank, world, dev, kernel):
    """The column-parallel decode pass with the ranks' own peer stores instead of NCCL: one gathered buffer per
    launch kind of a layer, every launch waiting (bounded) for the previous launch's arrivals from all ranks."""
    from atlasinfer_b200 import peer
    from atlasinfer_b200.integration import atlas_wrappers as aw
    per_layer = 4
    arena = peer.PeerArena(sum(m * lay.n_rows * world * 2 + 256 for lay, _ in launches[:per_layer]) + 4096, dev,
                           world=world, rank=rank, exchange=world > 1)
    try:
        kinds = [peer.GatheredLinear(arena, lay, m, torch.bfloat16, kernel=kernel) for lay, _ in launches[:per_layer]]

        def one_pass():
            for _ in range(reps):
                for i, (lay, _) in enumerate(launches):
                    g = kinds[i % per_layer]
                    g.layout = lay              # same shapes in every layer: one gathered buffer per kind, own weights
                    g(xs[lay.n_cols], wait=True)

        one_pass()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_pass()
        secs = allmax(time_steps(graph.replay, steps, warmup, barrier), world, dev)
        # a wait that ran out on ANY rank fails the measurement on EVERY rank (the ranks must stay in step for
        # the collectives that follow)
        bad = float(aw.status_word(dev).item() != 0)
        aw.status_word(dev).zero_()
        if allmax(bad, world, dev) > 0:
            return dict(error="a bounded wait on the other ranks' arrivals ran out")
        return dict(ms_per_token=secs / steps * 1e3, launch="graph")
    finally:
        arena.close()


def measure_quantize_sharded(rank, world, steps, warmup, barrier):
    """Whole-model quantization sharded by layer: every rank quantizes whole layers of its own
    (one 70B-shaped layer per step here), no collective.  Aggregate algorithmic GB/s."""
    import atlasinfer_b200 as ab
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(4242 + rank)
    ws = [synth_weight(n, k, gen, 0.015) for _, n, k in LLAMA70B_LINEARS]
    nbytes = sum(quantize_bytes(w.numel(), q.fp16_outliers.numel()) for w, q in zip(ws, ab.quantize_tensors(ws)))
    secs = allmax(time_steps(lambda: ab.quantize_tensors(ws), steps, warmup, barrier), world, dev)
    return world * nbytes * steps / secs / 1e9


CPU_SAMPLE = [(4096, 4096), (11008, 4096), (4096, 11008)]


def cpu_prepare(linears, m):
    """Quantized weights and activations of the CPU arm (oracle quantizer; untimed)."""
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
    return prepared


def cpu_linear_pass(prepared, reps=5):
    """The reference's forward on the host cores over prepared (weight, activation) pairs.

    integration/atlas_wrappers.py:54-67 calls dequantize_tensor (adaptive_quantizer.py:156, which keeps the
    fp16 reconstruction in a cache keyed by the weight object) and then F.linear: the first call of a
    layer pays the dequantization, every later call multiplies by the cached fp16 weight.  Both are
    timed: the steady state with torch's own CPU F.linear on fp16 tensors (the very call the reference
    makes; fp32 if this torch build has no fp16 CPU matmul), the first call with the oracle's
    dequantizer in front of it.  Returns (algorithmic bytes, steady-state seconds per pass, first-call seconds);
    the bytes are those of the quantized format, so the figure is comparable with the GPU lines."""
    import torch.nn.functional as F
    from oracle import atlas_oracle as O
    t0 = time.perf_counter()
    cached = [O.dequantize(q) for q, _, _ in prepared]          # the reference's per-weight cache
    t_dequant = time.perf_counter() - t0
    try:
        F.linear(prepared[0][1], cached[0])
        xs = [x for _, x, _ in prepared]
    except RuntimeError:                                         # no fp16 matmul on this CPU build
        cached = [c.float() for c in cached]
        xs = [x.float() for _, x, _ in prepared]
    t0 = time.perf_counter()
    for _ in range(reps):
        for x, wd in zip(xs, cached):
            F.linear(x, wd)
    t_steady = (time.perf_counter() - t0) / reps
    return sum(b for _, _, b in prepared), t_steady, t_steady + t_dequant


def host_threads():
    """Use every host core: under torch.distributed.run the environment pins OMP to one thread."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


# ----------------------------------------------------------------------------- arms
def run_reference(args, rank, world):
    """CPU arm: the oracle port of the quantized linear forward on the host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import atlas_oracle as O
    O.build()
    cores = host_threads()
    prepared = cpu_prepare(CPU_SAMPLE, 1)        # quantized once, outside the step loop
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_linear_pass(prepared[:1], 1)
    t_all, t_first, b_all = 0.0, 0.0, 0
    for _ in range(args.steps):
        b, t, tf = cpu_linear_pass(prepared, 1)
        t_all += t
        t_first += tf
        b_all += b
    val = b_all / t_all / 1e9
    desc = ("bounded sample of the workload per step: q_proj 4096x4096 + gate_proj 11008x4096 + down_proj 4096x11008 "
            "at batch 1; steady state of the reference's forward = torch CPU F.linear on the cached fp16 weight; the "
            f"first call of a layer (dequantize_tensor, CPU oracle port, OpenMP, then F.linear) runs at "
            f"{b_all / t_first / 1e9:.3f} GB/s")
    line = dict(
        impl="reference", metric="dequant_gemv_hbm_gbs", value=val, unit="GB/s", n_gpus=args.gpus,
        steps=args.steps, warmup=args.warmup, ms_per_step=t_all / args.steps * 1e3, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="int8 codes x fp16 scales -> fp16 MMA, fp32 accumulate",
        data="synthetic", config=workload_config(1, args.layers), gpu_launches=0,
        cpu_baseline=dict(value=val, unit="GB/s", cores=cores, kind="port", sample=desc),
        e2e=dict(value=val, unit="GB/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


NCU_DRAM_BYTES_PER_WEIGHT = 1.052   # dram__bytes_read.sum + dram__bytes_write.sum per weight over one layer's four fused launches (ncu capture)


_T0 = time.perf_counter()
PG_TIMEOUT = __import__("datetime").timedelta(seconds=180)   # a rank out of step ends the run in minutes, not in ten


def progress(rank, what):
    """One line per finished phase on stderr (rank 0), so a slow or stuck phase can be told from the log."""
    if rank == 0:
        print(f"[bench +{time.perf_counter() - _T0:6.1f}s] {what}", file=sys.stderr, flush=True)


def workload_config(m, layers):
    return dict(workload="llama2-7b decode linears: 32 layers x (q,k,v,o 4096x4096; gate,up 11008x4096; "
                         "down 4096x11008), block 128, z 3.0, weights N(0,0.02)+0.1% outliers",
                batch=m, activations="bf16 N(0,1)", l2="each step streams 6.7 GB of weights (>> 126 MB L2)",
                launch="q/k/v and gate/up fused: 4 kernels per layer, step replayed from a CUDA graph", layers=layers)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from atlasinfer_b200 import _capi
    _capi.load()  # fail here, loudly, if the CUDA library is missing
    barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=PG_TIMEOUT)
        barrier = dist.barrier
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    t_setup = time.perf_counter()
    model = build_model(LLAMA7B_LINEARS, args.layers, gen, 0.02, fuse=not args.no_fuse)
    torch.cuda.synchronize()
    t_setup = time.perf_counter() - t_setup
    resident = torch.cuda.memory_allocated(dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    nbytes, secs, launches = measure_gemv(model, 1, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    e_bytes, e_secs, h2d, d2h = measure_e2e(model, 1, args.steps, args.warmup, barrier)
    secs, e_secs = allmax(secs, world, dev), allmax(e_secs, world, dev)
    value = world * nbytes * args.steps / secs / 1e9
    e2e_value = world * e_bytes * args.steps / e_secs / 1e9
    per_gpu = value / world
    n_weights = sum(n * k for l in model for n, k, _ in l.stats.values())

    progress(rank, f"headline and end-to-end passes done ({value:.0f} / {e2e_value:.0f} GB/s)")
    extra = dict(resident_bytes_per_weight=resident / n_weights)
    half = max(2, args.steps // 2)
    # figures that do not depend on the number of ranks are taken in the single-GPU run only
    single = world == 1 and not args.headline_only
    if single:
        for m in (4, 16, 32):
            b, s, _ = measure_gemv(model, m, half, 3)
            extra[f"decode_m{m}_gbs"] = b * half / s / 1e9
        # the reference's own activation dtype (its F.linear takes fp16 only): no conversion inside the kernel
        b, s, _ = measure_gemv(model, 1, half, 3, dtype=torch.float16)
        extra["decode_m1_fp16_activations_gbs"] = b * half / s / 1e9
    del model
    torch.cuda.empty_cache()
    if single and not args.no_fuse:
        unfused = build_model(LLAMA7B_LINEARS, args.layers, torch.Generator(device=dev).manual_seed(99), 0.02, fuse=False)
        b, s, ln = measure_gemv(unfused, 1, half, 3)
        extra["unfused_gbs"] = b * half / s / 1e9
        extra["unfused_launches_per_step"] = ln
        del unfused
        torch.cuda.empty_cache()
    if not args.headline_only:
        try:
            tp = measure_tp70b(rank, world, max(2, args.steps // 5), 3, barrier, args.all_gather_forms)
            qs = measure_quantize_sharded(rank, world, 2, 1, barrier)
            if rank == 0:
                extra["tp70b_decode"] = tp
                extra["quantize_layer_sharded_gbs"] = qs
        except Exception as e:  # noqa: BLE001 - keep the headline line
            extra["tp70b_error"] = repr(e)
        progress(rank, "70B-shaped column-parallel decode and layer-sharded quantization done")
    if single:
        quarter = max(2, args.steps // 4)
        for name, fn in (("prefill_gemm_tflops", lambda: measure_gemm(quarter, 3)),
                         ("quantize_gbs", lambda: dict(zip(("batched", "one_by_one"), measure_quantize(quarter, 3)))),
                         ("quantize_kernel_gbs", lambda: measure_quantize_kernel(quarter, 3)),
                         ("opt_1p3b", measure_opt13b)):
            try:
                extra[name] = fn()
            except Exception as e:  # noqa: BLE001 - secondary figures must not lose the headline line
                extra[name + "_error"] = repr(e)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import atlas_oracle as O
        O.build()
        cores = host_threads()
        b, t, tf = cpu_linear_pass(cpu_prepare(CPU_SAMPLE[:2], 1))
        cpu = dict(value=b / t / 1e9, unit="GB/s", cores=cores, kind="port",
                   sample="q_proj 4096x4096 + gate_proj 11008x4096 at batch 1; steady state of the reference's "
                          "forward (torch CPU F.linear on the cached fp16 weight); with the first-call "
                          f"dequantization (CPU oracle port, OpenMP) in front: {b / tf / 1e9:.3f} GB/s")

    if rank == 0:
        cfg = workload_config(1, args.layers)
        if args.no_fuse:
            cfg["launch"] = "one kernel per linear, step replayed from a CUDA graph"
        line = dict(
            metric="dequant_gemv_hbm_gbs", value=value, unit="GB/s", n_gpus=world, steps=args.steps,
            warmup=args.warmup, ms_per_step=secs / args.steps * 1e3, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="int8 codes x fp16 scales -> fp16 MMA, fp32 accumulate", data="synthetic",
            config=cfg, clocks=clocks,
            e2e=dict(value=e2e_value, unit="GB/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                     method="per step: pinned-host activations -> device, CUDA-graph replay of the 224 "
                            "QuantizedLinear.forward calls, all 224 outputs -> pinned host, wait"),
            gpu_launches=launches * args.steps,
            roofline=dict(bound="hbm", achieved=per_gpu, peak=pk["hbm"], unit="GB/s", frac=per_gpu / pk["hbm"],
                          # DRAM bytes per launch from the ncu capture of the kernel (bytes per weight x the
                          # weights an average launch of the step covers)
                          traffic=NCU_DRAM_BYTES_PER_WEIGHT * n_weights / launches,
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
    ap.add_argument("--no-fuse", action="store_true", help="one launch per linear (224 per step) instead of 4 per layer")
    ap.add_argument("--layers", type=int, default=LLAMA7B["layers"],
                    help="decoder layers in the pass (default: the full 32; smaller only for profiler captures)")
    ap.add_argument("--all-gather-forms", action="store_true",
                    help="70B-shaped decode: also time the gather fused into the streaming kernel and the push kernel "
                         "(default: NCCL all-gather and the peer stores of the tcgen05 path)")
    ap.add_argument("--shard-of", type=int, default=None,
                    help="with --only tp70b on one GPU: time one rank's share of an N-way row split (no gathers)")
    ap.add_argument("--no-graph", action="store_true", help="launch the pass directly instead of replaying a graph")
    ap.add_argument("--only", default=None, choices=["gemm", "quantize", "opt13b", "tp70b"],
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
        elif args.only == "opt13b":
            out = {"opt_1p3b": measure_opt13b()}
        elif args.only == "tp70b":
            barrier = None
            if world > 1:
                import torch.distributed as dist
                dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=PG_TIMEOUT)
                barrier = dist.barrier
            out = {"tp70b_decode": measure_tp70b(rank, world, args.steps, args.warmup, barrier, args.all_gather_forms,
                                                 args.shard_of)}
            if world > 1:
                dist.barrier()
                dist.destroy_process_group()
            if rank != 0:
                return
        else:
            out = {"quantize": measure_quantize(args.steps, args.warmup),
                   "quantize_kernel": measure_quantize_kernel(args.steps, args.warmup)}
        print(json.dumps(out), flush=True)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
