"""Benchmark of the KV-cache hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --impl reference-gpu      # context: the unmodified reference's own CUDA path on this GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one decode step of the hot path for a Qwen3-8B shaped
model): per GPU 36 layers, each a quantized cache of batch 64 x 8 kv heads x (4096 packed +
128 residual) tokens x head_dim 128, 32 query heads, 4-bit codes, group 64, fp16 metadata.
A step is, for every layer: append the new K/V token, flush the residual window when due,
and run the fused decode attention.  36 distinct layer caches (17 GB) are walked per step, so
every read comes from HBM, not L2.  Synthetic K/V: V~N(0,1), K~N(0,1) with log-normal channel
scales, q~N(0,1), seeded.

  value     tokens/s through the C ABI with all inputs resident in HBM
  e2e       tokens/s through the plug-in API (MuZeroCache.update + mu_zero_decode_attention_forward)
            with pinned host q/k/v copied in and the attention output copied out every step
            (copies on a second stream, overlapped with the layers' kernels)
  roofline  algorithmic bytes of one decode-attention call / its mean duration (CUDA events on
            the launch stream around one call per step of the timed region, a different layer each
            step) against the measured HBM copy bandwidth
  cpu_baseline / --impl reference
            the CPU restatement of the reference's PyTorch path (oracle/) on the host cores,
            on a bounded sample of the same workload
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, BATCH, KVH, QH, CTX, RES, D, GROUP = 36, 64, 8, 32, 4096, 128, 128, 64
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_mma_kernel launch at 4 bits, per sequence, from the
# ncu capture summarised in profiles/decode_mma_4bit_b32.md (batch 32: 168.20 MB + 4.91 MB); traffic is
# proportional to the batch, so a batch-64 launch is twice the captured one.
NCU_DRAM_BYTES_PER_SEQ_4BIT = (168_201_216 + 4_908_800) / 32
METRIC = ("decode tokens/sec of the KV-cache hot path (append + flush + quantized decode attention, 36 layers, "
          "batch 64/GPU, ctx 4096+128)")


def workload_config(bits: int, layers: int, batch: int, world: int, context: int) -> dict:
    """The `config` object both arms print: same keys, same values."""
    return {"workload": f"BASELINE config 1: standalone quantized decode attention, Qwen3-8B attention shape, {layers} layers/step",
            "bits": bits, "group": GROUP, "batch_per_gpu": batch, "global_batch": batch * world, "context": context,
            "residual_length": RES, "kv_heads": KVH, "q_heads": QH, "head_dim": D,
            "parallelism": f"batch-sharded x{world}, no collective",
            "l2_policy": f"inputs larger than L2: {layers} distinct layer caches walked per step"}


def algorithmic_bytes(bits: int, batch=BATCH, sq=CTX, res=RES, meta=2, elem=2, group=GROUP) -> int:
    """Bytes one decode-attention call must move: packed codes + metadata + residual + q/out."""
    per_pair = 2 * sq * D * bits // 8 + (sq // group) * D * 2 * meta + sq * (D // group) * 2 * meta + 2 * res * D * elem
    return batch * KVH * per_pair + 2 * batch * QH * D * elem


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_layers(bits: int, device: torch.device, layers: int, batch: int, seed: int, ctx: int = CTX, group: int = GROUP,
                 keep: list | None = None):
    """`layers` caches holding `ctx` quantized + RES residual tokens each (values drawn on the device).
    `keep`: receives host copies of sequence 0's K/V of the first cache (for the parity check)."""
    import muzero_b200 as mz
    gen = torch.Generator(device=device).manual_seed(seed)
    chan = torch.exp(torch.randn(D, device=device, generator=gen))
    out = []
    for li in range(layers):
        layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=group, residual_length=RES))
        layer.max_cache_length = ctx + RES + 1024
        k = (torch.randn(batch, KVH, ctx + RES, D, device=device, generator=gen) * chan).to(torch.bfloat16)
        v = torch.randn(batch, KVH, ctx + RES, D, device=device, generator=gen).to(torch.bfloat16)
        layer.update(k, v, {"materialize_full_kv": False})
        if li == 0 and keep is not None:
            keep.extend([k[:1].cpu(), v[:1].cpu()])
        del k, v
        out.append(layer)
    return out


def parity_check(layer, q: torch.Tensor, kept: list, bits: int) -> dict:
    """One fused decode-attention call of the benched shape against the CPU oracle on sequence 0 (outside any
    timed region): same bf16 K/V bits, same query, 2e-3 on the fp32 output, as in the parity tests."""
    import importlib.util
    from muzero_b200.cache.attention import decode_attention
    spec = importlib.util.spec_from_file_location("mz_oracle", os.path.join(ROOT, "oracle", "mz_oracle.py"))
    orc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(orc)
    ref = orc.OracleCacheLayer(bits=bits, group=GROUP, residual=RES)
    ref.append(kept[0], kept[1])
    want = orc.decode_attention_oracle(q[:1].cpu(), ref, D ** -0.5, QH // KVH, compute_dtype=torch.float32)
    got = decode_attention(layer, q, D ** -0.5, out_dtype=torch.float32)[:1].cpu()
    err = (got - want).abs().max().item()
    codes_equal = bool(torch.equal(layer._packed_key_q[:1].cpu(), ref.packed_k) and torch.equal(layer._packed_value_q[:1].cpu(), ref.packed_v))
    if err > 2e-3 or not codes_equal:
        raise RuntimeError(f"parity check failed: attention max-abs error {err}, codes equal: {codes_equal}")
    return {"against": "CPU oracle, sequence 0 of layer 0, full batch launch", "attention_max_abs_err": err, "tolerance": 2e-3,
            "codes_bit_exact": codes_equal}


def time_attention(bits: int, device, batch: int, ctx: int, layers: int, steps: int = 12, warmup: int = 3) -> dict:
    """Device time of one fused decode-attention call (main + merge kernel) on `layers` distinct caches (larger
    than L2 together), CUDA events on the launch stream."""
    from muzero_b200.cache.attention import build_decode_args
    from muzero_b200.kernels.loader import load_mu_zero_cuda_extension
    from muzero_b200.kernels._cabi import stream_ptr
    caches = build_layers(bits, device, layers, batch, seed=4321, ctx=ctx)
    q = torch.randn(batch, QH, 1, D, device=device).to(torch.bfloat16)
    outs = [torch.empty(batch, 1, QH, D, dtype=torch.bfloat16, device=device) for _ in caches]
    cargs = [build_decode_args(l, q, D ** -0.5, None, o) for l, o in zip(caches, outs)]
    lib, st = load_mu_zero_cuda_extension(), stream_ptr(device)
    for _ in range(warmup):
        for a in cargs:
            lib.mz_decode_attention(ctypes.byref(a), st)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        for a in cargs:
            lib.mz_decode_attention(ctypes.byref(a), st)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (steps * len(cargs))
    abytes = algorithmic_bytes(bits, batch=batch, sq=ctx)
    peak, _ = measured_peak_gbs()
    del caches, cargs
    torch.cuda.empty_cache()
    return {"bits": bits, "batch": batch, "context": ctx + RES, "us_per_launch": us, "bytes_per_launch": abytes,
            "achieved": abytes / us / 1e3, "frac": abytes / us / 1e3 / peak, "distinct_caches": layers}


class CabiSession:
    """Drives the C ABI directly: per layer one append, a flush when due, one fused attention."""

    def __init__(self, layers, q, k_new, v_new):
        from muzero_b200.cache.attention import build_decode_args
        from muzero_b200.kernels.loader import load_mu_zero_cuda_extension
        from muzero_b200.kernels._cabi import stream_ptr
        self.lib = load_mu_zero_cuda_extension()
        self.layers, self.q, self.k_new, self.v_new = layers, q, k_new, v_new
        self.stream = stream_ptr(q.device)
        self.outs = [torch.empty(q.shape[0], 1, q.shape[1], D, dtype=q.dtype, device=q.device) for _ in layers]
        self.build = build_decode_args
        self.launches = 0
        self.attn_events = []

    def step(self, timed_layer: int = -1):
        """One decode step.  `timed_layer`: the layer whose attention call is bracketed by CUDA events in this step
        (-1: none).  Only one call per step is bracketed: an event record between two kernels keeps the second
        from starting its prologue while the first drains (programmatic dependent launch), so events around every
        call would slow the step they measure."""
        lib, st = self.lib, self.stream
        for i, layer in enumerate(self.layers):
            before = layer._key_group_count
            layer.update(self.k_new, self.v_new, {"materialize_full_kv": False})   # append (+ flush when due)
            self.launches += 1 + (1 if layer._key_group_count != before else 0)
            args = self.build(layer, self.q, D ** -0.5, None, self.outs[i])
            timed = i == timed_layer
            if timed:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            rc = lib.mz_decode_attention(ctypes.byref(args), st)
            if timed:
                e1.record()
                self.attn_events.append((e0, e1))
            if rc != 0:
                raise RuntimeError("mz_decode_attention failed")
            self.launches += 2


def run_ours(args) -> dict:
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    import muzero_b200 as mz

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    bits, L, B = args.bits, args.layers, args.batch
    kept: list = []
    layers = build_layers(bits, device, L, B, seed=1234 + rank, keep=kept if rank == 0 else None)
    gen = torch.Generator(device=device).manual_seed(99 + rank)
    q = torch.randn(B, QH, 1, D, device=device, generator=gen).to(torch.bfloat16)
    parity = parity_check(layers[0], q, kept, bits) if rank == 0 else None
    k_new = torch.randn(B, KVH, 1, D, device=device, generator=gen).to(torch.bfloat16)
    v_new = torch.randn(B, KVH, 1, D, device=device, generator=gen).to(torch.bfloat16)

    # ---------------- device-resident throughput through the C ABI
    sess = CabiSession(layers, q, k_new, v_new)
    for _ in range(args.warmup):
        sess.step()
    barrier()
    sess.launches = 0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        sess.step(timed_layer=(7 * i) % L)     # one bracketed attention call per step, a different layer each time
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    attn_us = statistics.fmean(a.elapsed_time(b) for a, b in sess.attn_events) * 1e3
    launches = sess.launches
    ctx_now = layers[0].get_seq_length()

    # ---------------- end to end through the plug-in API with host buffers
    mz.patch_transformers()
    from types import SimpleNamespace
    cache = mz.MuZeroCache(layers[0].cfg)
    cache.layers = layers
    module = SimpleNamespace(num_key_value_groups=QH // KVH)
    # the step's inputs (one q/k/v slice per layer) sit in pinned host memory; a copy stream uploads them
    # slice by slice while the compute stream works on the layers whose slices have landed, and a third
    # stream reads each layer's output back as soon as it exists.  Nothing of a later step is touched early.
    host_q = [torch.randn(L, B, QH, 1, D).to(torch.bfloat16).pin_memory() for _ in range(2)]
    host_k = [torch.randn(L, B, KVH, 1, D).to(torch.bfloat16).pin_memory() for _ in range(2)]
    host_v = [torch.randn(L, B, KVH, 1, D).to(torch.bfloat16).pin_memory() for _ in range(2)]
    host_out = torch.empty(L, B, 1, QH, D, dtype=torch.bfloat16).pin_memory()
    dev_q, dev_k, dev_v = (torch.empty_like(t[0], device=device) for t in (host_q, host_k, host_v))
    h2d = (host_q[0].numel() + 2 * host_k[0].numel()) * 2
    d2h = host_out.numel() * 2
    copy_stream = torch.cuda.Stream(device)          # host -> device
    back_stream = torch.cuda.Stream(device)          # device -> host
    landed = [torch.cuda.Event() for _ in range(L)]
    computed = [torch.cuda.Event() for _ in range(L)]

    def e2e_step(i: int):
        compute = torch.cuda.current_stream()
        outs = []
        for li in range(L):
            with torch.cuda.stream(copy_stream):
                dev_q[li].copy_(host_q[i & 1][li], non_blocking=True)
                dev_k[li].copy_(host_k[i & 1][li], non_blocking=True)
                dev_v[li].copy_(host_v[i & 1][li], non_blocking=True)
                landed[li].record(copy_stream)
            compute.wait_event(landed[li])
            cache.update(dev_k[li], dev_v[li], li, {"materialize_full_kv": False})
            out, _ = mz.mu_zero_decode_attention_forward(module, dev_q[li], None, D ** -0.5, cache.get_attention_state(li))
            computed[li].record(compute)
            outs.append(out)
            with torch.cuda.stream(back_stream):
                back_stream.wait_event(computed[li])
                host_out[li].copy_(out, non_blocking=True)
        back_stream.synchronize()                      # the step's result is on the host
        compute.synchronize()

    for i in range(min(args.warmup, 3)):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)

    peak, peak_kind = measured_peak_gbs()
    abytes = algorithmic_bytes(bits, batch=B)
    achieved = abytes / (attn_us * 1e-6) / 1e9
    # ---------------- after the timed regions: the other points of the metric (rank 0's GPU; every rank measures so
    # that the GPUs stay in step): 2-bit codes at the same shape, and longer contexts at batch 64
    extra = {}
    if not args.no_sweep:
        del sess, cache
        layers.clear()
        torch.cuda.empty_cache()
        other = 2 if bits == 4 else 4
        extra[f"roofline_{other}bit"] = time_attention(other, device, B, CTX, layers=4)
        # the benched width again, calls back to back without events in between (what the step itself sees)
        extra[f"roofline_{bits}bit_back_to_back"] = time_attention(bits, device, B, CTX, layers=4)
        extra["ctx_sweep"] = [time_attention(bits, device, B, c, layers=2, steps=6) for c in (8192, 32768)]
        barrier()
        if world > 1:
            extra["kv_split"] = [kv_split_point(b_, device, rank, world, dist) for b_ in (4, 2)]
    result = {
        "metric": METRIC,
        "value": world * B * args.steps / (ms_total * 1e-3),
        "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"u{bits} codes, fp16 metadata, bf16 residual, f32 accumulation",
        "data": "synthetic",
        "config": workload_config(bits, L, B, world, ctx_now),
        "e2e": {"value": world * B * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_DRAM_BYTES_PER_SEQ_4BIT * B if bits == 4 else None, "peak_kind": peak_kind, "kernel": "decode_mma_kernel + combine_tiles_warp_kernel",
                     "bytes_per_launch": abytes, "us_per_launch": attn_us},
        "clocks": clocks,
        "parity_check": parity,
    }
    result.update(extra)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(bits, seconds=12.0)
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_attention_only(args) -> dict:
    """Small standalone case for profilers: `--layers` caches of `--batch` sequences, `--steps`
    rounds of one fused decode-attention call per cache, nothing else on the GPU."""
    from muzero_b200.cache.attention import build_decode_args
    from muzero_b200.kernels.loader import load_mu_zero_cuda_extension
    from muzero_b200.kernels._cabi import stream_ptr
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    layers = build_layers(args.bits, device, args.layers, args.batch, seed=1234, ctx=args.context, group=args.group)
    q = torch.randn(args.batch, QH, 1, D, device=device).to(torch.bfloat16)
    outs = [torch.empty(args.batch, 1, QH, D, dtype=torch.bfloat16, device=device) for _ in layers]
    cargs = [build_decode_args(l, q, D ** -0.5, None, o) for l, o in zip(layers, outs)]
    lib, st = load_mu_zero_cuda_extension(), stream_ptr(device)
    for _ in range(args.warmup):
        for a in cargs:
            lib.mz_decode_attention(ctypes.byref(a), st)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        for a in cargs:
            lib.mz_decode_attention(ctypes.byref(a), st)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * len(cargs))
    abytes = algorithmic_bytes(args.bits, batch=args.batch, sq=args.context, group=args.group)
    peak, kind = measured_peak_gbs()
    return {"mode": "attention-only", "bits": args.bits, "batch": args.batch, "layers": args.layers, "context": args.context,
            "group": args.group, "us_per_call": us,
            "bytes_per_call": abytes, "achieved_gbs": abytes / us / 1e3, "frac_of_peak": abytes / us / 1e3 / peak, "peak_kind": kind}


def kv_split_point(bits: int, device, rank: int, world: int, dist, batch: int = 8, context: int = 131072, layers: int = 2,
                   steps: int = 6, warmup: int = 2, group: int = GROUP) -> dict:
    """One point of the KV-sequence split: one very long context cut over the ranks' GPUs.
    Each rank holds a contiguous slice of `context` quantized tokens (the last one also the residual window),
    computes its partial (m, l, acc); the triples are all-gathered (NCCL) and merged on every rank.  CUDA events
    around whole calls (partial + all-gather + merge), max over ranks."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    from muzero_b200.distributed import kv_split_decode_attention, kv_split_ranges
    lo, hi = kv_split_ranges(context, world, group)[rank]
    res = RES if rank == world - 1 else 0
    gen = torch.Generator(device=device).manual_seed(77)            # same stream on every rank: identical q
    q = torch.randn(batch, QH, 1, D, device=device, generator=gen).to(torch.bfloat16)
    gen.manual_seed(1000 + rank)
    caches = []
    for _ in range(layers):
        layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=group, residual_length=res,
                                                    alpha_key=2.0, alpha_value=2.0))
        n = hi - lo + res
        k = torch.randn(batch, KVH, n, D, device=device, generator=gen).to(torch.bfloat16)
        v = torch.randn(batch, KVH, n, D, device=device, generator=gen).to(torch.bfloat16)
        layer.update(k, v, {"materialize_full_kv": False})
        del k, v
        caches.append(layer)

    def one_round():
        for layer in caches:
            if world > 1:
                kv_split_decode_attention(layer, q, D ** -0.5)
            else:
                decode_attention(layer, q, D ** -0.5)

    for _ in range(warmup):
        one_round()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one_round()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    us = ms.item() * 1e3 / (steps * len(caches))
    abytes = algorithmic_bytes(bits, batch=batch, sq=context, group=group)
    peak, kind = measured_peak_gbs()
    del caches
    torch.cuda.empty_cache()
    return {"mode": "kv-split", "n_gpus": world, "bits": bits, "group": group, "batch": batch, "context": context,
            "layers": layers, "us_per_call": us, "bytes_per_call_all_ranks": abytes,
            "achieved_gbs_all_ranks": abytes / us / 1e3, "frac_of_peak_per_gpu": abytes / us / 1e3 / peak / world,
            "collective": "all_gather of (m, l, acc) partials, then a local merge kernel" if world > 1 else "none", "peak_kind": kind}


def run_kv_split(args) -> dict:
    """Secondary workload on its own: `bench.py --kv-split [--gpus N]` (see kv_split_point)."""
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    out = kv_split_point(args.bits, device, rank, world, dist, batch=args.batch, context=args.context, layers=args.layers,
                         steps=args.steps, warmup=args.warmup, group=args.group)
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_generate(args) -> dict:
    """Secondary workload: greedy `generate()` on a random-init (std 0.02)
    Qwen3-8B-architecture decoder in bf16 through `patch_transformers()` and
    `cache_implementation="mu_zero_{bits}bit"`; decode-only tokens/s (prefill excluded, as the
    reference's throughput bench does).  `--cache dynamic` runs stock transformers for context;
    `--impl reference-gpu` runs the unmodified reference package from baseline/_ref instead of this one."""
    ours = args.impl != "reference-gpu"
    if not ours:
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "muzero")):
            return {"impl": "reference-gpu", "unavailable": "baseline/_ref holds no reference install"}
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(ref_dir, "_ext"))
        sys.path.insert(0, ref_dir)                  # ahead of the repo root, whose `muzero` is this package's alias
    import muzero
    assert ours or os.path.abspath(muzero.__file__).startswith(os.path.join(ROOT, "baseline")), muzero.__file__
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from transformers.generation.streamers import BaseStreamer
    muzero.patch_transformers()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    cfg = Qwen3Config(num_hidden_layers=args.layers, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                      head_dim=128, intermediate_size=12288, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6,
                      max_position_embeddings=40960, tie_word_embeddings=False)
    torch.manual_seed(0)
    with torch.device(device):
        model = Qwen3ForCausalLM(cfg).to(torch.bfloat16).eval()
        for prm in model.parameters():
            if prm.dim() > 1:
                prm.data.normal_(0.0, 0.02)
    gen = torch.Generator(device=device).manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.context), device=device, generator=gen)

    class Clock(BaseStreamer):
        """Records the wall-clock time (after a device sync) at which each new token arrives."""
        def __init__(self):
            self.stamps = []
        def put(self, value):
            torch.cuda.synchronize()
            self.stamps.append(time.perf_counter())
        def end(self):
            pass

    kwargs = dict(max_new_tokens=args.new_tokens, do_sample=False, pad_token_id=0)
    if args.prefill_chunk:
        kwargs["prefill_chunk_size"] = args.prefill_chunk      # long prompts: the model's own activations need it
        # ... and the cache quantizes chunk by chunk, as the reference's bench does in its chunked mode
        os.environ["MUZERO_QUANTIZE_PREFILL_CHUNKS"] = "1"
    if args.cache == "mu_zero":
        kwargs.update(cache_implementation=f"mu_zero_{args.bits}bit",
                      cache_config={"q_group_size": GROUP, "residual_length": RES, "backend": "cuda"})
    clock = Clock()
    grabbed = []          # the cache object generate() builds, for the cache-bytes columns
    if args.cache == "mu_zero" and ours:
        from muzero_b200.integrations import transformers_patch as tp
        real_init = tp.MuZeroCache.__init__
        def grabbing_init(self, *a, **kw):
            real_init(self, *a, **kw)
            grabbed.append(self)
        tp.MuZeroCache.__init__ = grabbing_init
    muzero.reset_mu_zero_decode_stats()
    torch.cuda.reset_peak_memory_stats()
    with torch.no_grad():
        out = model.generate(input_ids=ids, attention_mask=torch.ones_like(ids), streamer=clock, **kwargs)
    if args.cache == "mu_zero" and ours:
        tp.MuZeroCache.__init__ = real_init
    # stamps[0] = prompt echo, stamps[1] = first new token (end of prefill); decode = the rest
    t = clock.stamps
    decode_s = t[-1] - t[1]
    steps = len(t) - 2
    cache_mb = {}
    if args.cache == "mu_zero" and grabbed:
        # the reference's rule (benchmarks/bench_throughput.py:199-224): packed codes, metadata, residual buffers
        mb = lambda x: 0.0 if x is None else x.numel() * x.element_size() / 1024 ** 2
        packed = meta = resid = 0.0
        for layer in grabbed[0].layers:
            packed += mb(layer._packed_key_q) + mb(layer._packed_value_q)
            meta += sum(mb(getattr(layer, a)) for a in ("_key_mn", "_key_scale", "_value_mn", "_value_scale"))
            resid += mb(layer._key_buffer if layer._key_buffer is not None else layer.keys)
            resid += mb(layer._value_buffer if layer._value_buffer is not None else layer.values)
        cache_mb = {"cache_packed_mb": packed, "cache_meta_mb": meta, "cache_residual_mb": resid,
                    "cache_total_mb": packed + meta + resid}
    return {**cache_mb, "mode": "generate", "impl": args.impl, "cache": args.cache, "bits": args.bits, "layers": args.layers, "batch": args.batch,
            "context": args.context, "prefill_chunk": args.prefill_chunk, "new_tokens": int(out.shape[1] - ids.shape[1]),
            "prefill_s": t[1] - t[0], "decode_tokens_per_s": args.batch * steps / decode_s, "ms_per_decode_step": 1e3 * decode_s / steps,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30, "decode_stats": muzero.get_mu_zero_decode_stats()}


def cpu_baseline(bits: int, seconds: float) -> dict:
    """The oracle (CPU restatement of the reference's torch path) on a bounded sample of the workload."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("mz_oracle", os.path.join(ROOT, "oracle", "mz_oracle.py"))
    orc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(orc)
    sb, sl = 2, 2    # sequences and layers of the sample
    caches = []
    for li in range(sl):
        k, v, q = orc.synth_kv(sb, KVH, CTX + RES, D, QH, seed=li)
        layer = orc.OracleCacheLayer(bits=bits, group=GROUP, residual=RES)
        layer.append(k, v)
        caches.append((layer, q))
    k1 = torch.randn(sb, KVH, 1, D).to(torch.bfloat16)
    v1 = torch.randn(sb, KVH, 1, D).to(torch.bfloat16)
    steps, t0 = 0, time.perf_counter()
    while True:
        for layer, q in caches:
            layer.append(k1, v1)
            orc.decode_attention_oracle(q, layer, D ** -0.5, QH // KVH)
        steps += 1
        if time.perf_counter() - t0 > seconds or steps >= 64:
            break
    per_layer = (time.perf_counter() - t0) / (steps * sl)
    return {"value": sb / (per_layer * LAYERS), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sb} of {BATCH} sequences, {sl} of {LAYERS} layers, {steps} steps; per-layer time scaled to {LAYERS} layers",
            "host_cpus": os.cpu_count(), "torch": torch.__version__}


def run_reference(args) -> dict:
    """The reference arm: the reference's CPU (torch backend) implementation of the path, as restated in oracle/, on
    the host cores, on a bounded sample of the same workload.  Under a multi-rank launch rank 0 alone runs it (a CPU
    arm does not scale with the GPU count); it uses every host core (the launcher pins OMP_NUM_THREADS=1, which is undone)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    t0 = time.perf_counter()
    base = cpu_baseline(args.bits, seconds=max(10.0, min(90.0, 2.0 * args.steps)))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return {
        "impl": "reference",
        "metric": METRIC,
        "value": base["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * BATCH / base["value"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"u{args.bits} codes, fp16 metadata, bf16 residual (torch CPU ops in bf16, the reference's torch backend)",
        "data": "synthetic",
        "config": workload_config(args.bits, LAYERS, BATCH, world, CTX + RES + args.warmup + args.steps),
        "extrapolated": True,      # value and ms_per_step are scaled from the sample named in cpu_baseline.sample
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }


def run_reference_gpu(args) -> dict:
    """Context, not the reference arm the run is graded on: the UNMODIFIED reference package, installed under
    baseline/_ref (git-ignored), driven on cuda:0 through its own API - MuZeroCacheLayer.update() and
    mu_zero_decode_attention_forward() - on the same shape and synthetic data as `run_ours`, with its own JIT-built
    CUDA extension.  Two of its paths are timed: the stock decode path (qk kernel, softmax, av kernel, dense residual
    matmuls) and the fused chunked prefix decode it enables with MUZERO_FUSED_PREFIX_DECODE=1.  `--layers` distinct
    caches are walked per step (default 8 here: 2 GB of codes, larger than L2) and the per-layer time is scaled to 36."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "muzero")):
        return {"impl": "reference-gpu", "unavailable": "baseline/_ref holds no reference install"}
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(ref_dir, "_ext"))
    sys.path.insert(0, ref_dir)                      # ahead of the repo root, whose `muzero` is this package's alias
    import muzero as ref
    assert os.path.abspath(ref.__file__).startswith(ref_dir), ref.__file__
    from muzero.cache.attention import mu_zero_decode_attention_forward as ref_forward
    from muzero.cache.layer import MuZeroCacheLayer as RefLayer
    from types import SimpleNamespace
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    bits, L, B = args.bits, min(args.layers, 8), args.batch
    gen = torch.Generator(device=device).manual_seed(1234)
    chan = torch.exp(torch.randn(D, device=device, generator=gen))
    layers = []
    try:
        for _ in range(L):
            layer = RefLayer(ref.MuZeroConfig(bits=bits, q_group_size=GROUP, residual_length=RES, alpha_key=2.0, alpha_value=2.0))
            k = (torch.randn(B, KVH, CTX + RES, D, device=device, generator=gen) * chan).to(torch.bfloat16)
            v = torch.randn(B, KVH, CTX + RES, D, device=device, generator=gen).to(torch.bfloat16)
            layer.update(k, v, {"materialize_full_kv": False})
            del k, v
            layers.append(layer)
        q = torch.randn(B, QH, 1, D, device=device, generator=gen).to(torch.bfloat16)
        k_new = torch.randn(B, KVH, 1, D, device=device, generator=gen).to(torch.bfloat16)
        v_new = torch.randn(B, KVH, 1, D, device=device, generator=gen).to(torch.bfloat16)
        module = SimpleNamespace(num_key_value_groups=QH // KVH)

        def step(with_update: bool):
            for layer in layers:
                if with_update:
                    layer.update(k_new, v_new, {"materialize_full_kv": False})
                out = ref_forward(module, q, None, D ** -0.5, layer.get_attention_state())
                if out is None:
                    raise RuntimeError("the reference's decode forward declined the call")

        def timed(with_update: bool, steps: int) -> float:
            for _ in range(3):
                step(with_update)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step(with_update)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / (steps * L)       # us per layer

        res = {}
        for name, flag in (("stock", "0"), ("fused_chunked", "1")):
            os.environ["MUZERO_FUSED_PREFIX_DECODE"] = flag
            ref.reset_mu_zero_decode_stats()
            res[name] = {"attention_us_per_layer": timed(False, args.steps), "step_us_per_layer": timed(True, args.steps),
                         "decode_stats": {k: v for k, v in ref.get_mu_zero_decode_stats().items() if v}}
    except Exception as exc:                                  # a build or launch failure of the reference is the result
        return {"impl": "reference-gpu", "unavailable": f"{type(exc).__name__}: {str(exc)[-400:]}"}
    best = min(res.values(), key=lambda r: r["step_us_per_layer"])
    ms_step = best["step_us_per_layer"] * LAYERS / 1e3
    return {"impl": "reference-gpu", "metric": METRIC, "value": B / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": 3, "ms_per_step": ms_step, "higher_is_better": True,
            "dtype": f"u{bits} codes, fp16 metadata, bf16 residual", "data": "synthetic", "extrapolated": True,
            "config": workload_config(bits, L, B, 1, CTX + RES), "paths": res,
            "note": "the reference's own CUDA extension and torch ops on this GPU; per-layer time of the faster path scaled to 36 layers"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the measurements after the timed regions (2-bit, longer contexts, KV split)")
    ap.add_argument("--attention-only", action="store_true", help="small profiling case: only the fused attention calls")
    ap.add_argument("--kv-split", action="store_true", help="secondary workload: one long context split over the GPUs of the run")
    ap.add_argument("--generate", action="store_true", help="secondary workload: HF generate() on a Qwen3-8B shaped model")
    ap.add_argument("--cache", default="mu_zero", choices=["mu_zero", "dynamic"])
    ap.add_argument("--context", type=int, default=CTX, help="quantized tokens per sequence (--attention-only, --generate)")
    ap.add_argument("--group", type=int, default=GROUP, help="quantization group size (--attention-only)")
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--prefill-chunk", type=int, default=0, help="--generate: prefill the prompt in chunks of this many tokens")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.generate:
        print(json.dumps(run_generate(args)))
        return
    if args.attention_only:
        print(json.dumps(run_attention_only(args)))
        return
    if args.kv_split:
        out = run_kv_split(args)
        if out:
            print(json.dumps(out))
        return
    if args.impl == "reference-gpu":
        print(json.dumps(run_reference_gpu(args)))
        return
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
