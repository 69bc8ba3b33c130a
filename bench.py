#!/usr/bin/env python
"""Benchmark of the layer forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-ops]

One JSON line on stdout (rank 0). Headline workload ("int8_quant"): one PASS is the per-row
int8 configuration on one GPU's batch —
    quantise   bf16 [8192, 4096] (N(0,1), 0.1% outliers x20)      100,696,064 B
    dequantise the codes back to bf16                              100,696,064 B
    fused RMSNorm(4096) -> int8 on bf16 [16, 2048, 4096]           402,792,448 B
and one STEP is `passes_per_step` such passes over rotating input sets, so that the timed
region of K steps lasts long enough (>= 0.5 s) for clocks to be sampled inside it. `value` is
algorithmic GB/s (bytes that must move / time), whole job over all ranks, inputs resident in
HBM. Every rank owns its own batch (weak scaling, no collective on the data path). `e2e` is
the same pass through the public API from pinned host buffers with the copies inside the timed
region. `roofline` is the fused RMSNorm->int8 kernel (the dominant one) timed with CUDA events
inside the timed region. `ops` carries every other kernel of the path (norms, RoPE, GLUs,
attention variants, the decoder layer) on the benchmark shapes, batch-sharded over the ranks
(strong scaling for the kernels, the configuration's own 4 sequences per GPU for the layer),
each with the oracle's CPU time beside it at N = 1. `--impl reference` times the reference's
own CPU arithmetic (the oracle port) for the headline workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QUANT_SHAPE = (8192, 4096)
ACT_SHAPE = (16, 2048, 4096)
BYTES_QUANT = QUANT_SHAPE[0] * QUANT_SHAPE[1] * 3 + 4 * QUANT_SHAPE[0]
BYTES_DEQUANT = BYTES_QUANT
ACT_ROWS = ACT_SHAPE[0] * ACT_SHAPE[1]
BYTES_FUSED = ACT_ROWS * ACT_SHAPE[2] * 3 + 4 * ACT_ROWS + 2 * ACT_SHAPE[2]
BYTES_PASS = BYTES_QUANT + BYTES_DEQUANT + BYTES_FUSED
L2_BYTES = 126 * 1024 * 1024
METRIC = "int8_path_algorithmic_hbm_bandwidth"
WORKLOAD = ("int8_quant: quantize+dequantize bf16[8192,4096] (0.1% outliers x20) and fused "
            "RMSNorm(4096)->int8 on bf16[16,2048,4096]; this batch per GPU")
EST_PASS_MS = 0.12      # used only to size passes_per_step; the measured time is what is reported
TARGET_REGION_S = 0.8
E2E_REPEATS = 3         # end-to-end regions timed per mode; the median is reported


def config_block(world: int) -> dict:
    """The same for both arms (ours and --impl reference), key for key."""
    return {"workload": WORKLOAD, "parallelism": f"dp{world}",
            "bytes_per_pass_per_gpu": BYTES_PASS,
            "l2": "inputs rotate over 3 sets (960 MB), every read misses the 126 MB L2"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def profiled_traffic(kernel_key: str):
    """DRAM bytes (read + write) of one launch of a kernel, from the ncu summary committed under
    profiles/: a line `dram_traffic_bytes_per_launch[<kernel_key>] = <int>`. None if absent."""
    pat = re.compile(r"dram_traffic_bytes_per_launch\[" + re.escape(kernel_key) + r"\]\s*=\s*(\d+)")
    pdir = os.path.join(ROOT, "profiles")
    try:
        for name in sorted(os.listdir(pdir)):
            if name.endswith((".md", ".txt")):
                m = pat.search(open(os.path.join(pdir, name)).read())
                if m:
                    return {"bytes": int(m.group(1)), "source": f"profiles/{name}"}
    except OSError:
        pass
    return None


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """SM clock and throttle reasons, read through NVML every few milliseconds on a helper
    thread while the timed region runs (read-only queries; nothing is ever set). Falls back
    to one `nvidia-smi` query when the NVML binding is missing."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
               "sw_thermal_slowdown": 0x20}

    def __init__(self, gpu_index: int, period_s: float = 0.003):
        self.gpu, self.period = gpu_index, period_s
        self.samples, self.reason_bits, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            # torch's device index follows CUDA_VISIBLE_DEVICES; NVML wants the physical GPU
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.gpu
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if self.gpu < len(ids) and ids[self.gpu].isdigit():
                    phys = int(ids[self.gpu])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        if self._nvml is None:
            return self._smi_once()
        self._stop.set()
        self._thread.join(timeout=1.0)
        sm = sorted(self.samples)
        reasons = sorted(n for n, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                "sm_mhz_min": sm[0] if sm else None, "reasons": reasons, "samples": len(sm),
                "source": "nvml"}

    def _smi_once(self):
        try:
            out = subprocess.run(
                ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active",
                 "--format=csv,noheader,nounits", "-i", str(self.gpu)],
                capture_output=True, text=True, timeout=10).stdout.strip().split(",")
            return {"sm_mhz": float(out[0]), "sm_max_mhz": float(out[1]),
                    "reasons": [out[2].strip()], "samples": 1, "source": "nvidia-smi after the region"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}


# ----------------------------------------------------------------------------- helpers
def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def bind_rank_to_cores(local_rank: int, local_world: int):
    """Give each rank of a node its own slice of the host cores the job may use, before any
    pinned buffer is allocated (first-touch then places the pages near those cores). Returns
    the cores kept, or None when the platform has no affinity call or too few cores."""
    try:
        cores = sorted(os.sched_getaffinity(0))
    except AttributeError:
        return None
    if local_world <= 1 or len(cores) < 2 * local_world:
        return None
    per = len(cores) // local_world
    mine = cores[local_rank * per:(local_rank + 1) * per]
    try:
        os.sched_setaffinity(0, mine)
    except OSError:
        return None
    return mine


def make_inputs(seed: int, device, sets: int):
    """`sets` independent copies of the pass's inputs (rotated so reads come from HBM)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(sets):
        xq = torch.randn(QUANT_SHAPE, generator=g)
        mask = torch.rand(QUANT_SHAPE, generator=g) < 0.001
        xq = torch.where(mask, 20 * xq, xq).bfloat16()
        xa = torch.randn(ACT_SHAPE, generator=g).bfloat16()
        out.append((xq.to(device), xa.to(device)))
    w = (1 + 0.02 * torch.randn(ACT_SHAPE[2], generator=g)).bfloat16().to(device)
    return out, w


def capture(fn):
    """Capture fn() (kernel launches on the current stream, no host sync) into a CUDA graph,
    after one eager warm-up on a side stream. Launch-bound sequences of short kernels are
    replayed from graphs so that the GPU, not the Python interpreter, sets the pace."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        keep = fn()
    graph._keep = keep  # outputs live in the graph's private pool
    return graph


def event_ms(fn_list, warmup=3, iters=10):
    """Median device time in ms of ONE call, for calls that are rotated over `fn_list`
    (one callable per input set). All calls of one round are captured into one graph and
    the graph is replayed between two CUDA events."""
    def round_():
        return [f() for f in fn_list]
    graph = capture(round_)
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(iters)]
    for a, b in evs:
        a.record(); graph.replay(); b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return ts[len(ts) // 2] / len(fn_list)


def n_sets(bytes_per_set: int) -> int:
    """How many input sets to rotate over so that one round touches more than twice the L2."""
    return max(2, math.ceil(2.2 * L2_BYTES / max(1, bytes_per_set)))


# ----------------------------------------------------------------------------- per-op table
def bench_ops(device, pk, rank: int, world: int):
    """Every kernel of the path on the benchmark shapes, batch-sharded over `world` ranks:
    this rank runs rows / world (sequences / world) of each shape. Returns name -> entry with
    this rank's `ms` and the WHOLE-JOB work (`bytes` or `flop` over all ranks); the caller takes
    the maximum time over ranks. Inputs rotate over more than twice the L2."""
    import trinix_b200 as T
    from trinix_b200 import ops
    from trinix_b200.decoder import Int8DecoderLayer, random_layer_weights
    res = {}
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    rnd = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32).bfloat16()

    def hbm(name, nbytes_per_gpu, fns, **kw):
        res[name] = {"kind": "hbm", "ms": event_ms(fns, **kw), "bytes": nbytes_per_gpu * world}

    R_, C_ = ACT_ROWS // world, ACT_SHAPE[2]
    acts = [rnd(R_, C_) for _ in range(n_sets(R_ * C_ * 2))]
    pair = list(zip(acts, acts[1:] + acts[:1]))
    w = (1 + 0.02 * torch.randn(C_, generator=g, device=device)).bfloat16()
    b = torch.zeros(C_, device=device, dtype=torch.bfloat16)
    tag = f"{ACT_ROWS}x{C_}"
    hbm(f"rmsnorm_bf16_{tag}", R_ * C_ * 4 + 2 * C_, [lambda a=a: ops.rmsnorm(a, w, 1e-6) for a in acts])
    hbm(f"layernorm_bf16_{tag}", R_ * C_ * 4 + 4 * C_,
        [lambda a=a: ops.layernorm(a, w, b, 1e-5) for a in acts])
    # backward of the norms: read x and dy, write dx (6 B per element); dW / db via per-CTA fp32
    # partial sums and a second, small kernel (both inside the timed graph)
    hbm(f"rmsnorm_bwd_bf16_{tag}", R_ * C_ * 6 + 4 * C_,
        [lambda a=a, d=d: ops.rmsnorm_backward(d, a, w, 1e-6) for a, d in pair])
    hbm(f"layernorm_bwd_bf16_{tag}", R_ * C_ * 6 + 6 * C_,
        [lambda a=a, d=d: ops.layernorm_backward(d, a, w, 1e-5) for a, d in pair])
    hbm(f"rmsnorm_quant_i8_{tag}", R_ * C_ * 3 + 4 * R_ + 2 * C_,
        [lambda a=a: ops.rmsnorm_quantize(a, w, 1e-6) for a in acts])
    # residual forms (the step either side of the norm in a decoder layer), new residual stream
    # written: 2 reads + 2 writes of 2 bytes (8C), or 2 reads + 1 write + codes (7C + 4)
    hbm(f"residual_rmsnorm_sum_bf16_{tag}", R_ * C_ * 8 + 2 * C_,
        [lambda a=a, r=r: ops.residual_rmsnorm(a, r, w, 1e-6, True) for a, r in pair])
    hbm(f"residual_rmsnorm_quant_sum_i8_{tag}", R_ * C_ * 7 + 4 * R_ + 2 * C_,
        [lambda a=a, r=r: ops.residual_rmsnorm_quantize(a, r, w, 1e-6, True) for a, r in pair])
    hbm(f"residual_layernorm_sum_bf16_{tag}", R_ * C_ * 8 + 4 * C_,
        [lambda a=a, r=r: ops.residual_layernorm(a, r, w, b, 1e-5, True) for a, r in pair])
    for act in ("mish", "quickgelu", "squared_relu"):
        hbm(f"rmsnorm_{act}_bf16_{tag}", R_ * C_ * 4 + 2 * C_,
            [lambda a=a, act=act: ops.rmsnorm_activation(a, w, 1e-6, act) for a in acts])
    del acts, pair
    Rq, Cq = QUANT_SHAPE[0] // world, QUANT_SHAPE[1]
    xs = [rnd(Rq, Cq) for _ in range(n_sets(Rq * Cq * 3))]
    qtag = f"{QUANT_SHAPE[0]}x{Cq}"
    hbm(f"quant_i8_{qtag}", Rq * Cq * 3 + 4 * Rq, [lambda x=x: ops.quantize_rowwise(x) for x in xs])
    cs = [ops.quantize_rowwise(x) for x in xs]
    hbm(f"dequant_i8_{qtag}", Rq * Cq * 3 + 4 * Rq,
        [lambda c=c: ops.dequantize_rowwise(c[0], c[1], torch.bfloat16) for c in cs])
    del xs, cs
    # RoPE + GLUs (cfg: q[8,2048,32,128], k[8,2048,8,128]; gate/up [8,2048,11008])
    Bp = max(1, 8 // world)
    n_rope = n_sets(Bp * 2048 * 40 * 128 * 2)
    qs = [rnd(Bp, 2048, 32, 128) for _ in range(n_rope)]
    ks = [rnd(Bp, 2048, 8, 128) for _ in range(n_rope)]
    inv = 1.0 / 10000.0 ** (torch.arange(0, 128, 2, device=device).float() / 128)
    fr = torch.outer(torch.arange(2048, device=device).float(), inv)
    cos, sin = torch.cat([fr, fr], -1).cos(), torch.cat([fr, fr], -1).sin()
    hbm("rope_q32k8_8x2048x128", (qs[0].numel() + ks[0].numel()) * 4 + 2 * 2048 * 64 * 4,
        [lambda q=q, k=k: ops.rope(q, k, cos, sin) for q, k in zip(qs, ks)])
    del qs, ks
    Rg = 16384 // world
    xg = [rnd(Rg, 22016) for _ in range(n_sets(Rg * 22016 * 2))]
    for act in ("swiglu", "geglu", "reglu"):
        hbm(f"{act}_16384x11008", Rg * 11008 * 6, [lambda x=x, a=act: ops.glu(x, a) for x in xg])
    dyg = rnd(Rg, 11008)
    for act in ("swiglu", "geglu", "reglu"):  # backward: read dy, up, gate; write dup, dgate
        hbm(f"{act}_bwd_16384x11008", Rg * 11008 * 10,
            [lambda x=x, a=act: ops.glu_backward(dyg, x, a) for x in xg])
    del xg, dyg
    torch.cuda.empty_cache()
    # attention (cfg: q[16,4096,32,128], kv[16,4096,8,128]), 16 / world sequences on this rank
    B, S, H, Hk, D = max(1, 16 // world), 4096, 32, 8, 128
    q, k, v = rnd(B, S, H, D), rnd(B, S, Hk, D), rnd(B, S, Hk, D)
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / 32) for i in range(32)], device=device)
    causal_flop = 4 * B * H * S * S * D // 2
    win_pairs = 1024 * 1025 // 2 + 3072 * 1025
    variants = {
        "attn_causal": (dict(causal=True), causal_flop),
        "attn_causal_alibi": (dict(causal=True, alibi_slopes=slopes), causal_flop),
        "attn_window_1024_0": (dict(window=(1024, 0)), 4 * D * win_pairs * B * H),
    }
    attn_sampler = ClockSampler(device.index or 0)
    if rank == 0:
        attn_sampler.start()
    for name, (kw, flop) in variants.items():
        ms = event_ms([lambda kw=kw: ops.attention(q, k, v, **kw)], warmup=2, iters=5)
        res[name] = {"kind": "attn", "ms": ms, "flop": flop * world, "timing": "burst (5 launches)"}
    if rank == 0:
        res["attn_clocks_burst"] = {"kind": "info", **attn_sampler.stop()}
    if world == 1:
        # the same causal launch back to back for >= 2 s, clocks sampled inside: what the kernel
        # sustains under the power cap, and time x clock as a clock-independent figure
        reps = max(50, int(2000.0 / max(res["attn_causal"]["ms"], 0.05)))
        sus = ClockSampler(device.index or 0, period_s=0.02)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        out_buf = None
        sus.start()
        e0.record()
        for _ in range(reps):
            out_buf = ops.attention(q, k, v, causal=True)
        e1.record()
        torch.cuda.synchronize()
        ck = sus.stop()
        ms = e0.elapsed_time(e1) / reps
        res["attn_causal_sustained"] = {
            "kind": "attn", "ms": ms, "flop": causal_flop, "timing": f"{reps} launches back to back",
            "clocks": ck,
            "ms_times_sm_mhz": round(ms * ck["sm_mhz"], 1) if ck.get("sm_mhz") else None}
        del out_buf
    res["attn_status_word"] = {"kind": "info", "value": T.attention_status(device)}
    del q, k, v
    torch.cuda.empty_cache()
    # decoder layer (cfg5): x [32, 2048, 4096] over 8 GPUs = 4 sequences per GPU, at every N
    E, Hq, Hkv, FF, Bl, Sl = 4096, 32, 8, 11008, 4, 2048
    layer = Int8DecoderLayer(E, Hq, Hkv, FF, random_layer_weights(E, Hq, Hkv, FF, device, seed=0),
                             max_seq_len=Sl)
    x = torch.randn(Bl, Sl, E, generator=g, device=device).bfloat16()
    for name, fn in (("decoder_layer_modules", layer.forward_modules),
                     ("decoder_layer", layer.forward_fused)):
        res[name] = {"kind": "layer", "ms": event_ms([lambda fn=fn: fn(x)], warmup=2, iters=5),
                     "tokens": Bl * Sl * world}
    # where the layer's time goes: the GEMMs alone (cuBLAS), same shapes, weights already bf16
    wdq = layer.dequantised(("wq", "wk", "wv", "wo", "w_up_gate", "w_down"))
    x2 = x.view(-1, E)
    ff = torch.randn(Bl * Sl, FF, generator=g, device=device).bfloat16()

    def gemms():
        import torch.nn.functional as F
        return [F.linear(x2, wdq[n]) for n in ("wq", "wk", "wv", "wo", "w_up_gate")] + \
               [F.linear(ff, wdq["w_down"])]
    res["decoder_layer_gemms_only"] = {"kind": "layer_part", "ms": event_ms([gemms], warmup=2, iters=5)}
    res["decoder_layer_dequant_only"] = {
        "kind": "layer_part",
        "ms": event_ms([lambda: layer.dequantised(("wq", "wk", "wv", "wo", "w_up_gate", "w_down"))],
                       warmup=2, iters=5)}
    del layer, wdq, x, ff
    torch.cuda.empty_cache()
    return res


def finalize_ops(res: dict, pk: dict, world: int) -> dict:
    """Derived figures from the max-over-ranks times."""
    out = {}
    for name, e in res.items():
        kind = e.pop("kind")
        if kind == "info":
            out[name] = e.get("value", e) if set(e) == {"value"} else e
            continue
        ms = e["ms"]
        e["ms"] = round(ms, 5)
        if kind == "hbm":
            gbs = e["bytes"] / ms / 1e6
            e.update(gbs=round(gbs, 1), frac_hbm=round(gbs / world / pk["hbm_gbs"], 4),
                     frac_nominal_8tbs=round(gbs / world / 8000.0, 4))
        elif kind == "attn":
            tf = e["flop"] / ms / 1e9
            e.update(tflops=round(tf, 1),
                     frac_bf16_burst=round(tf / world / pk["bf16_tflops"], 4),
                     frac_bf16_sustained=round(tf / world / pk["bf16_tflops_sustained"], 4),
                     frac_nominal_2250=round(tf / world / 2250.0, 4))
        elif kind == "layer":
            e.update(tokens_per_s=round(e["tokens"] / ms * 1e3, 1),
                     note="4 sequences [4,2048,4096] bf16 per GPU, int8 weight store")
        if world > 1 and kind in ("hbm", "attn"):
            e["scaling"] = "strong: the benchmark shape split over the ranks by batch"
        out[name] = e
    if "decoder_layer" in out and "decoder_layer_gemms_only" in out:
        out["decoder_layer"]["gemm_ms"] = out["decoder_layer_gemms_only"]["ms"]
        out["decoder_layer"]["dequant_ms"] = out["decoder_layer_dequant_only"]["ms"]
    return out


# ----------------------------------------------------------------------------- CPU legs
def cpu_pass_sample(rows_q: int, rows_a: int, threads: int, reps: int = 1):
    """The oracle's arithmetic for a bounded sample of one pass; returns (seconds, bytes)."""
    from oracle import reference_port as R
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    xq = torch.randn(rows_q, QUANT_SHAPE[1], generator=g).bfloat16()
    xa = torch.randn(rows_a, ACT_SHAPE[2], generator=g).bfloat16()
    w = (1 + 0.02 * torch.randn(ACT_SHAPE[2], generator=g)).bfloat16()
    nbytes = rows_q * QUANT_SHAPE[1] * 6 + 8 * rows_q + rows_a * ACT_SHAPE[2] * 3 + 4 * rows_a
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        c, s = R.quantize_rowwise_ref(xq)
        R.dequantize_rowwise_ref(c, s, torch.bfloat16)
        R.rmsnorm_quantize_ref(xa, w, 1e-6)
        best = min(best, time.perf_counter() - t0)
    return best, nbytes


def cpu_ops_baseline(threads: int) -> dict:
    """The reference's PyTorch arithmetic (the oracle port) on the host cores for every row of
    `ops`, each on a bounded sample of the benchmark shape (stated), scaled to the full shape."""
    from oracle import reference_port as R
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    out = {}

    def timed(fn):
        fn()  # warm-up (thread pool, allocator)
        t0 = time.perf_counter()
        fn()
        return (time.perf_counter() - t0) * 1e3

    def put(name, ms_sample, factor, sample):
        out[name] = {"ms": round(ms_sample * factor, 2), "sample": sample, "cores": threads,
                     "kind": "port"}

    C = ACT_SHAPE[2]
    tag = f"{ACT_ROWS}x{C}"
    x = torch.randn(4096, C, generator=g).bfloat16()
    r = torch.randn(4096, C, generator=g).bfloat16()
    w = (1 + 0.02 * torch.randn(C, generator=g)).bfloat16()
    b = torch.zeros(C).bfloat16()
    s8 = "4096 of 32768 rows, x8"
    put(f"rmsnorm_bf16_{tag}", timed(lambda: R.rmsnorm_ref(x, w, 1e-6)), 8, s8)
    put(f"layernorm_bf16_{tag}", timed(lambda: R.layernorm_ref(x, w, b, 1e-5)), 8, s8)
    put(f"rmsnorm_quant_i8_{tag}", timed(lambda: R.rmsnorm_quantize_ref(x, w, 1e-6)), 8, s8)
    put(f"residual_rmsnorm_sum_bf16_{tag}", timed(lambda: R.residual_rmsnorm_ref(x, r, w, 1e-6)), 8, s8)
    put(f"residual_rmsnorm_quant_sum_i8_{tag}",
        timed(lambda: R.quantize_rowwise_ref(R.residual_rmsnorm_ref(x, r, w, 1e-6))), 8, s8)
    put(f"residual_layernorm_sum_bf16_{tag}",
        timed(lambda: R.residual_layernorm_ref(x, r, w, b, 1e-5)), 8, s8)
    for act in ("mish", "quickgelu", "squared_relu"):
        put(f"rmsnorm_{act}_bf16_{tag}", timed(lambda act=act: R.rmsnorm_activation_ref(x, w, 1e-6, act)), 8, s8)
    dy = torch.randn(4096, C, generator=g).bfloat16()
    put(f"rmsnorm_bwd_bf16_{tag}",
        timed(lambda: R.autograd_ref(lambda a, ww: R.rmsnorm_ref(a, ww, 1e-6), [x, w], dy)), 8, s8)
    put(f"layernorm_bwd_bf16_{tag}",
        timed(lambda: R.autograd_ref(lambda a, ww, bb: R.layernorm_ref(a, ww, bb, 1e-5), [x, w, b], dy)), 8, s8)
    xq = x[:2048]
    qtag = f"{QUANT_SHAPE[0]}x{QUANT_SHAPE[1]}"
    put(f"quant_i8_{qtag}", timed(lambda: R.quantize_rowwise_ref(xq)), 4, "2048 of 8192 rows, x4")
    c, s = R.quantize_rowwise_ref(xq)
    put(f"dequant_i8_{qtag}", timed(lambda: R.dequantize_rowwise_ref(c, s, torch.bfloat16)), 4,
        "2048 of 8192 rows, x4")
    q = torch.randn(1, 2048, 32, 128, generator=g).bfloat16()
    k = torch.randn(1, 2048, 8, 128, generator=g).bfloat16()
    cos, sin = R.rope_tables_ref(128, 2048, 10000.0, torch.float32)
    put("rope_q32k8_8x2048x128", timed(lambda: R.rope_ref(q, k, cos, sin)), 8, "1 of 8 sequences, x8")
    xg = torch.randn(2048, 22016, generator=g).bfloat16()
    dyg = torch.randn(2048, 11008, generator=g).bfloat16()
    for act, fn in (("swiglu", R.swiglu_ref), ("geglu", R.geglu_ref), ("reglu", R.reglu_ref)):
        put(f"{act}_16384x11008", timed(lambda fn=fn: fn(xg)), 8, "2048 of 16384 rows, x8")
        put(f"{act}_bwd_16384x11008", timed(lambda fn=fn: R.autograd_ref(fn, [xg], dyg)), 8,
            "2048 of 16384 rows, x8")
    del xg, dyg
    # attention: one sequence of the 16, eight query heads (two kv heads) at a time so that the
    # O(S^2) score tensor stays at 512 MiB; bf16 like the GPU arm
    S, D = 4096, 128
    qa = torch.randn(1, S, 32, D, generator=g).bfloat16()
    ka = torch.randn(1, S, 8, D, generator=g).bfloat16()
    va = torch.randn(1, S, 8, D, generator=g).bfloat16()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / 32) for i in range(32)])

    def attn(causal, window, sl):
        for h0 in range(0, 32, 8):
            R.attention_variant_ref(qa[:, :, h0:h0 + 8], ka[:, :, h0 // 4:h0 // 4 + 2],
                                    va[:, :, h0 // 4:h0 // 4 + 2], D ** -0.5, causal, window,
                                    None if sl is None else sl[h0:h0 + 8])
    sa = "1 of 16 sequences (8 query heads at a time), x16"
    put("attn_causal", timed(lambda: attn(True, None, None)), 16, sa)
    put("attn_causal_alibi", timed(lambda: attn(True, None, slopes)), 16, sa)
    put("attn_window_1024_0", timed(lambda: attn(False, (1024, 0), None)), 16, sa)
    # decoder layer: one sequence of the GPU's four
    E, FF = 4096, 11008
    p = {n: (0.02 * torch.randn(*sh, generator=g)).bfloat16() for n, sh in (
        ("wq", (E, E)), ("wk", (1024, E)), ("wv", (1024, E)), ("wo", (E, E)),
        ("w_up", (FF, E)), ("w_gate", (FF, E)), ("w_down", (E, FF)))}
    p["attn_norm"], p["ffn_norm"] = torch.ones(E).bfloat16(), torch.ones(E).bfloat16()
    xl = torch.randn(1, 2048, E, generator=g).bfloat16()
    ms = timed(lambda: R.decoder_layer_ref(xl, p, 32, 8))
    for name in ("decoder_layer", "decoder_layer_modules"):
        put(name, ms, 4, "1 of 4 sequences, x4 (weights already dequantised)")
    return out


def run_reference_arm(args):
    """The reference's CPU arithmetic for the same workload, all host threads; every step is a
    bounded sample of one pass (1/8 of its rows)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    threads = host_threads()
    rows_q, rows_a = QUANT_SHAPE[0] // 8, ACT_ROWS // 8
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_pass_sample(rows_q, rows_a, threads)
    t = 0.0
    nbytes = 0
    for _ in range(args.steps):
        dt, nb = cpu_pass_sample(rows_q, rows_a, threads)
        t += dt; nbytes += nb
    gbs = nbytes / t / 1e9
    sample = (f"each step = {rows_q} of {QUANT_SHAPE[0]} quant/dequant rows + {rows_a} of "
              f"{ACT_ROWS} fused rows (1/8 of one pass), one process on {threads} host threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3),
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(t / args.steps * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(world), "sample": sample,
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }))


def profile_case(name: str):
    """A handful of eager launches on benchmark-sized (but < 2 GB) inputs, for profiler captures:
    `ncu ... python bench.py --profile-case attention`. Prints nothing but a completion line."""
    from trinix_b200 import ops
    import trinix_b200 as T
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    g = torch.Generator(device=device).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32).bfloat16()
    if name == "int8":
        acts = [rnd(ACT_ROWS, ACT_SHAPE[2]) for _ in range(2)]  # 2 x 256 MB, each pass misses L2
        xq = [rnd(*QUANT_SHAPE) for _ in range(3)]
        w = torch.ones(ACT_SHAPE[2], device=device, dtype=torch.bfloat16)
        for i in range(4):
            ops.rmsnorm_quantize(acts[i % 2], w, 1e-6)
            c, sc = ops.quantize_rowwise(xq[i % 3])
            ops.dequantize_rowwise(c, sc, torch.bfloat16)
            ops.residual_rmsnorm_quantize(acts[i % 2], acts[(i + 1) % 2], w, 1e-6, True)
    elif name == "stream":
        acts = [rnd(ACT_ROWS, ACT_SHAPE[2]) for _ in range(2)]
        w = torch.ones(ACT_SHAPE[2], device=device, dtype=torch.bfloat16)
        b = torch.zeros(ACT_SHAPE[2], device=device, dtype=torch.bfloat16)
        q, k = rnd(8, 2048, 32, 128), rnd(8, 2048, 8, 128)
        inv = 1.0 / 10000.0 ** (torch.arange(0, 128, 2, device=device).float() / 128)
        fr = torch.outer(torch.arange(2048, device=device).float(), inv)
        cos, sin = torch.cat([fr, fr], -1).cos(), torch.cat([fr, fr], -1).sin()
        xg = rnd(8192, 22016)
        for i in range(3):
            ops.rmsnorm(acts[i % 2], w, 1e-6)
            ops.layernorm(acts[i % 2], w, b, 1e-5)
            ops.rope(q, k, cos, sin)
            ops.glu(xg, "swiglu")
    elif name == "backward":
        acts = [rnd(ACT_ROWS, ACT_SHAPE[2]) for _ in range(2)]
        w = torch.ones(ACT_SHAPE[2], device=device, dtype=torch.bfloat16)
        xg, dyg = rnd(8192, 22016), rnd(8192, 11008)
        for i in range(3):
            ops.rmsnorm_backward(acts[(i + 1) % 2], acts[i % 2], w, 1e-6)
            ops.layernorm_backward(acts[(i + 1) % 2], acts[i % 2], w, 1e-5)
            ops.glu_backward(dyg, xg, "swiglu")
    else:
        q, k, v = rnd(2, 4096, 32, 128), rnd(2, 4096, 8, 128), rnd(2, 4096, 8, 128)
        for _ in range(4):
            ops.attention(q, k, v, causal=True)
    torch.cuda.synchronize()
    print(f"profile case {name} done; attention status word {T.attention_status(device)}")


# ----------------------------------------------------------------------------- end to end
class E2E:
    """One pass through the public tensor API from pinned host buffers. The pass is cut into row
    chunks; host->device copies run on one stream into two preallocated device slots per input
    kind, kernels on a second stream, device->host copies of the results on a third, so both
    PCIe directions and the kernels overlap. Every byte of input crosses host->device and every
    byte of result device->host inside the timed region. `mode`: 'full' (copies + kernels),
    'copies' (the same schedule with the kernels left out: what the host side alone allows),
    'h2d' / 'd2h' (one direction alone)."""

    CH_Q, CH_A = 2048, 8192

    def __init__(self, device, w, seed):
        import trinix_b200 as T
        self.T, self.device, self.w = T, device, w
        g = torch.Generator().manual_seed(seed)
        self.h_xq = torch.randn(QUANT_SHAPE, generator=g).bfloat16().pin_memory()
        self.h_xa = torch.randn(ACT_SHAPE, generator=g).bfloat16().pin_memory()
        self.h_codes_q = torch.empty(QUANT_SHAPE, dtype=torch.int8).pin_memory()
        self.h_scales_q = torch.empty(QUANT_SHAPE[0], dtype=torch.float32).pin_memory()
        self.h_deq = torch.empty(QUANT_SHAPE, dtype=torch.bfloat16).pin_memory()
        self.h_codes_a = torch.empty(ACT_SHAPE, dtype=torch.int8).pin_memory()
        self.h_scales_a = torch.empty(ACT_SHAPE[:2], dtype=torch.float32).pin_memory()
        self.h2d = self.h_xq.numel() * 2 + self.h_xa.numel() * 2
        self.d2h = (self.h_codes_q.numel() + self.h_scales_q.numel() * 4 + self.h_deq.numel() * 2
                    + self.h_codes_a.numel() + self.h_scales_a.numel() * 4)
        self.s_in, self.s_k, self.s_out = (torch.cuda.Stream() for _ in range(3))
        self.xa2 = self.h_xa.view(-1, ACT_SHAPE[2])
        self.ca2 = self.h_codes_a.view(-1, ACT_SHAPE[2])
        self.sa2 = self.h_scales_a.view(-1)
        self.chunks = [("q", lo, lo + self.CH_Q) for lo in range(0, QUANT_SHAPE[0], self.CH_Q)]
        self.chunks += [("a", lo, lo + self.CH_A) for lo in range(0, ACT_ROWS, self.CH_A)]
        mk = lambda r, c, dt: [torch.empty(r, c, dtype=dt, device=device) for _ in range(2)]
        self.slots = {"q": mk(self.CH_Q, QUANT_SHAPE[1], torch.bfloat16),
                      "a": mk(self.CH_A, ACT_SHAPE[2], torch.bfloat16)}
        # result slots used by the copy-only modes (the full mode copies what the kernels return)
        self.r_codes = {"q": mk(self.CH_Q, QUANT_SHAPE[1], torch.int8),
                        "a": mk(self.CH_A, ACT_SHAPE[2], torch.int8)}
        self.r_deq = mk(self.CH_Q, QUANT_SHAPE[1], torch.bfloat16)
        self.r_scales = {"q": [torch.zeros(self.CH_Q, device=device) for _ in range(2)],
                         "a": [torch.zeros(self.CH_A, device=device) for _ in range(2)]}
        ev = lambda: [torch.cuda.Event() for _ in range(2)]
        self.ev_ready = {"q": ev(), "a": ev()}   # input slot filled
        self.ev_free = {"q": ev(), "a": ev()}    # input slot consumed
        self.ev_done = {"q": ev(), "a": ev()}    # results of the slot computed
        self.ev_out = {"q": ev(), "a": ev()}     # results of the slot copied out
        self.turn = {"q": 0, "a": 0}
        cur = torch.cuda.current_stream()
        for d in (self.ev_free, self.ev_out):
            for k in d:
                for e in d[k]:
                    e.record(cur)

    def one_pass(self, mode: str):
        T = self.T
        for kind, lo, hi in self.chunks:
            i = self.turn[kind] & 1
            self.turn[kind] += 1
            d_x = self.slots[kind][i]
            if mode != "d2h":
                with torch.cuda.stream(self.s_in):
                    self.s_in.wait_event(self.ev_free[kind][i])
                    d_x.copy_(self.h_xq[lo:hi] if kind == "q" else self.xa2[lo:hi], non_blocking=True)
                    self.ev_ready[kind][i].record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(self.ev_ready[kind][i])
                self.s_k.wait_event(self.ev_out[kind][i])  # the slot's previous results are out
                if mode == "full":
                    if kind == "q":
                        codes, scales = T.quantize_rowwise(d_x)
                        deq = T.dequantize_rowwise(codes, scales, torch.bfloat16)
                    else:
                        codes, scales = T.rmsnorm_quantize(d_x, self.w, 1e-6)
                        deq = None
                else:
                    codes, scales = self.r_codes[kind][i], self.r_scales[kind][i]
                    deq = self.r_deq[i] if kind == "q" else None
                self.ev_free[kind][i].record(self.s_k)
                self.ev_done[kind][i].record(self.s_k)
            if mode != "h2d":
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.ev_done[kind][i])
                    if kind == "q":
                        self.h_codes_q[lo:hi].copy_(codes, non_blocking=True)
                        self.h_scales_q[lo:hi].copy_(scales, non_blocking=True)
                        self.h_deq[lo:hi].copy_(deq, non_blocking=True)
                    else:
                        self.ca2[lo:hi].copy_(codes, non_blocking=True)
                        self.sa2[lo:hi].copy_(scales, non_blocking=True)
                    # tensors returned by the kernels are freed by the caching allocator on the
                    # kernel stream; tell it that the copy stream still reads them
                    for t in (codes, scales, deq):
                        if t is not None and mode == "full":
                            t.record_stream(self.s_out)
                    self.ev_out[kind][i].record(self.s_out)

    def timed(self, mode: str, passes: int, sync_all) -> float:
        """ms for `passes` passes in `mode`, bracketed by CUDA events on the current stream."""
        cur = torch.cuda.current_stream()
        streams = (self.s_in, self.s_k, self.s_out)
        for st in streams:
            st.wait_stream(cur)
        for _ in range(2):
            self.one_pass(mode)
        for st in streams:
            cur.wait_stream(st)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for st in streams:
            st.wait_stream(cur)
        for _ in range(passes):
            self.one_pass(mode)
        for st in streams:
            cur.wait_stream(st)
        e1.record()
        sync_all()
        return e0.elapsed_time(e1)


# ----------------------------------------------------------------------------- main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--passes-per-step", type=int, default=0,
                    help="passes of the int8 configuration per step (0 = sized for a 0.8 s region)")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-kernel table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--profile-case", choices=["int8", "stream", "backward", "attention"],
                    help="launch a few kernels of one family eagerly and exit (for ncu captures)")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: trinix_b200 has no CPU path")
    threads_total = host_threads()
    cores = bind_rank_to_cores(local, local_world)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    import trinix_b200 as T
    from trinix_b200 import build, ops, sharding
    if rank == 0 and not os.path.exists(build.LIB_PATH):
        build.build()
    if world > 1:
        dist.barrier()
    pk = peaks()
    warmup = max(args.warmup, 3)
    passes = args.passes_per_step or max(
        1, math.ceil(TARGET_REGION_S * 1e3 / (args.steps * EST_PASS_MS)))

    sets = 3  # 3 x (64 + 256) MB of inputs: every read misses the 126 MB L2
    inputs, w = make_inputs(1234 + rank, device, sets)

    # One pass = 3 kernels of 15-80 us each: replayed from CUDA graphs (one pair per input
    # set) so the timed region is not paced by the interpreter. The fused RMSNorm->int8 kernel
    # is a graph of its own so that CUDA events can bracket it inside the timed region.
    def qd(i):
        xq, _ = inputs[i]
        codes, scales = ops.quantize_rowwise(xq)
        return ops.dequantize_rowwise(codes, scales, torch.bfloat16), codes, scales

    def fused(i):
        return ops.rmsnorm_quantize(inputs[i][1], w, 1e-6)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    launches_before_capture = ops.launch_count
    g_qd = [capture(lambda i=i: qd(i)) for i in range(sets)]
    g_fused = [capture(lambda i=i: fused(i)) for i in range(sets)]
    kernels_per_pass = (ops.launch_count - launches_before_capture) // (2 * sets)  # eager + capture

    BRACKET_EVERY = 8  # the fused kernel is bracketed by events on every 8th pass
    n = 0
    for _ in range(warmup):
        for _ in range(passes):
            g_qd[n % sets].replay(); g_fused[n % sets].replay()
            n += 1
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fused_evs = []
    n = 0
    ev0.record()
    for _ in range(args.steps):
        for _ in range(passes):
            g_qd[n % sets].replay()
            if n % BRACKET_EVERY == 0:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g_fused[n % sets].replay()
                b.record()
                fused_evs.append((a, b))
            else:
                g_fused[n % sets].replay()
            n += 1
    ev1.record()
    sync_all()
    total_passes = n
    launches = kernels_per_pass * total_passes
    clocks = sampler.stop() if rank == 0 else None
    local_fused = sum(a.elapsed_time(b) for a, b in fused_evs) / len(fused_evs)
    total_ms, fused_ms = sharding.max_over_ranks([ev0.elapsed_time(ev1), local_fused], device)
    value = world * BYTES_PASS * total_passes / total_ms / 1e6  # GB/s

    # ---- informational: the same passes with the two independent halves on two streams --------
    # quantise -> dequantise on one stream, fused RMSNorm -> int8 on another: the fused kernel
    # leaves DRAM cycles idle that the other two can use. Reported beside the headline (which
    # stays the serial pass, so that the roofline line brackets the fused kernel alone).
    forked_ms = None
    if world == 1:
        cur = torch.cuda.current_stream()
        s_a, s_b = torch.cuda.Stream(), torch.cuda.Stream()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_forked = min(total_passes, 400)
        for timed in (False, True):
            if timed:
                f0.record(cur)
            s_a.wait_stream(cur); s_b.wait_stream(cur)
            for i in range(n_forked if timed else 2 * sets):
                with torch.cuda.stream(s_a):
                    g_qd[i % sets].replay()
                with torch.cuda.stream(s_b):
                    g_fused[i % sets].replay()
            cur.wait_stream(s_a); cur.wait_stream(s_b)
            if timed:
                f1.record(cur)
            torch.cuda.synchronize()
        forked_ms = f0.elapsed_time(f1) / n_forked

    # ---- untimed: the batch-sharded run reproduces the unsharded one bit for bit ----------------
    gc = torch.Generator().manual_seed(4321)  # the same tensors on every rank
    n_units = max(8, world)
    cx = torch.randn(n_units, 256, 4096, generator=gc)
    cx = torch.where(torch.rand(cx.shape, generator=gc) < 0.001, 20 * cx, cx).bfloat16().to(device)
    cq = torch.randn(n_units, 512, 8, 128, generator=gc).bfloat16().to(device)
    ckv = torch.randn(n_units, 512, 2, 128, generator=gc).bfloat16().to(device)
    cw = (1 + 0.02 * torch.randn(4096, generator=gc)).bfloat16().to(device)  # replicated weight
    cross = {
        "quantize": sharding.cross_rank_identical(lambda t: ops.quantize_rowwise(t), [cx], rank, world),
        "rmsnorm_quantize": sharding.cross_rank_identical(
            lambda t: ops.rmsnorm_quantize(t, cw, 1e-6), [cx], rank, world),
        "dequantize": sharding.cross_rank_identical(
            lambda t: ops.dequantize_rowwise(*ops.quantize_rowwise(t)), [cx], rank, world),
        "attention_causal": sharding.cross_rank_identical(
            lambda a, b_: ops.attention(a, b_, b_, causal=True), [cq, ckv], rank, world),
    }
    del cx, cq, ckv, cw

    # ---- end to end: pinned host buffers, copies inside the timed region -----------------------
    e2e = E2E(device, w, 99 + rank)
    e2e_passes = max(3, min(args.steps, 10))
    # Each mode is timed E2E_REPEATS times and the median kept: one repeat can catch the caching
    # allocator growing its pool (a synchronising cudaMalloc) or a neighbour on the host's PCIe
    # root, which says nothing about the schedule itself. All repeats are reported.
    modes, full_runs = {}, []
    for mode in ("full", "copies", "h2d", "d2h"):
        runs = sorted(e2e.timed(mode, e2e_passes, sync_all) for _ in range(E2E_REPEATS))
        modes[mode] = runs[len(runs) // 2]
        if mode == "full":
            full_runs = runs
    m_full, m_copies, m_h2d, m_d2h = sharding.max_over_ranks(
        [modes["full"], modes["copies"], modes["h2d"], modes["d2h"]], device)
    e2e_value = world * BYTES_PASS * e2e_passes / m_full / 1e6
    status = T.attention_status(device)

    # ---- per-kernel table, every rank on its shard ------------------------------------------------
    ops_res, ops_err = None, None
    if not args.no_ops:
        try:
            ops_res = bench_ops(device, pk, rank, world)
        except Exception as e:  # the headline line must still be printed
            ops_err = repr(e)
        if world > 1:  # all ranks must agree before the reduction below
            bad = torch.tensor([1 if ops_err else 0], device=device)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if int(bad.item()) and ops_res is not None:
                ops_res, ops_err = None, ops_err or "another rank failed"
        if ops_res is not None:
            timed_names = [k for k, e in ops_res.items() if e["kind"] != "info"]
            mx = sharding.max_over_ranks([ops_res[k]["ms"] for k in timed_names], device)
            for k, v in zip(timed_names, mx):
                ops_res[k]["ms"] = v

    out = None
    if rank == 0:
        achieved = BYTES_FUSED / fused_ms / 1e6
        traffic = profiled_traffic("rmsnorm_quant_i8")
        out = {
            "metric": METRIC, "value": round(value, 1),
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_block(world),
            "passes_per_step": passes, "ms_per_pass": round(total_ms / total_passes, 5),
            "timed_region_s": round(total_ms / 1e3, 3),
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": e2e.h2d,
                    "d2h_bytes_per_step": e2e.d2h, "passes": e2e_passes,
                    "repeats": E2E_REPEATS,
                    "repeat_values_this_rank": [
                        round(BYTES_PASS * e2e_passes / m / 1e6, 2) for m in full_runs],
                    "note": "one e2e step = one pass; algorithmic bytes of the pass / wall time; "
                            "median of the repeats, max over ranks",
                    "copy_only": {
                        "value": round(world * BYTES_PASS * e2e_passes / m_copies / 1e6, 2),
                        "unit": "GB/s", "note": "same chunk schedule, kernels left out",
                        "frac_of_e2e_time": round(m_copies / m_full, 3),
                        "h2d_alone_gbs": round(world * e2e.h2d * e2e_passes / m_h2d / 1e6, 2),
                        "d2h_alone_gbs": round(world * e2e.d2h * e2e_passes / m_d2h / 1e6, 2),
                        "both_directions_gbs": round(
                            world * (e2e.h2d + e2e.d2h) * e2e_passes / m_copies / 1e6, 2)},
                    "host_cores_of_this_rank": len(cores) if cores else threads_total},
            "gpu_launches": launches,
            "roofline": {"kernel": "row_kernel<RMSNORM_QUANT,bf16> (trx_rmsnorm_quant_i8)",
                         "bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                         "traffic": traffic["bytes"] if traffic else None,
                         "traffic_source": traffic["source"] if traffic else None,
                         "peak_source": pk["source"],
                         "algorithmic_bytes_per_launch": BYTES_FUSED,
                         "ms_per_launch": round(fused_ms, 5),
                         "launches_bracketed": len(fused_evs)},
            "peaks": pk, "attn_status_word": status,
            "cross_rank_identical": all(cross.values()), "cross_rank_checks": cross,
        }
        if forked_ms is not None:
            out["pass_on_two_streams"] = {
                "ms_per_pass": round(forked_ms, 5),
                "value": round(BYTES_PASS / forked_ms / 1e6, 1), "unit": "GB/s",
                "note": "informational: quantise->dequantise and the fused kernel overlapped on "
                        "two streams; the headline is the serial pass"}
    if world > 1:
        dist.barrier()
    if rank == 0:
        if ops_res is not None:
            out["ops"] = finalize_ops(ops_res, pk, world)
        elif ops_err:
            out["ops"] = {"error": ops_err}
        if not args.no_cpu and world == 1:
            threads = host_threads()
            cpu_pass_sample(256, 512, threads)
            dt, nb = cpu_pass_sample(2048, 8192, threads, reps=2)
            out["cpu_baseline"] = {"value": round(nb / dt / 1e9, 3), "unit": "GB/s",
                                   "cores": threads, "kind": "port",
                                   "sample": "2048 of 8192 quant/dequant rows + 8192 of 32768 fused "
                                             "rows (1/4 pass), best of 2"}
            if "ops" in out and "error" not in out["ops"]:
                try:
                    cpu = cpu_ops_baseline(threads)
                    for name, c in cpu.items():
                        if name in out["ops"]:
                            out["ops"][name]["cpu"] = c
                            out["ops"][name]["speedup_vs_cpu"] = round(c["ms"] / out["ops"][name]["ms"], 1)
                except Exception as e:
                    out["ops"]["cpu_error"] = repr(e)
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
