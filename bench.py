"""Benchmark of the DartKV hot path on B200: fused packed-page decode attention (headline) and
quantize+pack append (reported beside it).

    python bench.py --gpus N --steps K --warmup W [--workload config5|config3] [--impl reference]

One JSON line on rank 0.  A step is one fused decode-attention pass over the whole resident
cache (one query token per sequence).  `value` is algorithmic HBM bytes per step (packed pages +
metadata + dense sink/tail + query/output, summed over all ranks) divided by the device time of a
step (max over ranks); `e2e` is the same through host buffers (pinned query -> device, attention,
output -> host).  Inputs are seeded synthetic tensors with the shapes and value distributions the
workload names (N(0,1) values, N(0,1) keys with 5 % of channels per head scaled x10).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # long-context batch-sharded decode: batch 128 split evenly over the GPUs, context 32768
    "config5": dict(batch=128, ctx=32768, seed=4),
    # packed-page fused GQA decode attention: batch 32, context 8192
    "config3": dict(batch=32, ctx=8192, seed=2),
}
GEOM = dict(query_heads=32, kv_heads=8, head_dim=128, page=128, key_group=128, value_group=64, sinks=32,
            promote_ratio=0.25, bits=2)


def cache_kwargs():
    return dict(bits=GEOM["bits"], promote_ratio=GEOM["promote_ratio"], page_size=GEOM["page"],
                key_group_size=GEOM["key_group"], value_group_size=GEOM["value_group"], sink_tokens=GEOM["sinks"],
                hold_partial_pages=True)


def bytes_per_bh(ctx: int) -> int:
    """Algorithmic bytes one (batch row, KV head) contributes to a decode step: bf16 sinks, packed
    pages (key 4096+1024+128+256+256, value 4096+512+512), bf16 dense tail."""

    pages = (ctx - GEOM["sinks"]) // GEOM["page"]
    tail = ctx - GEOM["sinks"] - pages * GEOM["page"]
    d = GEOM["head_dim"]
    return GEOM["sinks"] * d * 2 * 2 + pages * (5760 + 5120) + tail * d * 2 * 2


def step_bytes(batch: int, ctx: int) -> int:
    qo = 2 * batch * GEOM["query_heads"] * GEOM["head_dim"] * 2
    return batch * GEOM["kv_heads"] * bytes_per_bh(ctx) + qo


def outlier_channels(seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    count = int(0.05 * GEOM["head_dim"])
    return torch.stack([torch.randperm(GEOM["head_dim"], generator=gen)[:count] for _ in range(GEOM["kv_heads"])])


def build_device_cache(batch: int, ctx: int, seed: int, rank: int, device: torch.device):
    """Fill a cache with `ctx` tokens of synthetic K/V generated on the device, 1024 tokens per append."""

    import dartkv_b200 as dart

    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **cache_kwargs()), max_tokens=ctx + 256)
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    mult = torch.ones(GEOM["kv_heads"], GEOM["head_dim"], device=device)
    mult.scatter_(1, outlier_channels(seed).to(device), 10.0)
    mult = mult.view(1, GEOM["kv_heads"], 1, GEOM["head_dim"])
    done = 0
    first = True
    while done < ctx:
        step = GEOM["sinks"] if first else min(1024, ctx - done)
        first = False
        shape = (batch, GEOM["kv_heads"], step, GEOM["head_dim"])
        keys = (torch.randn(shape, generator=gen, device=device) * mult).to(torch.bfloat16)
        values = torch.randn(shape, generator=gen, device=device).to(torch.bfloat16)
        cache.append(keys, values)
        done += step
    query = torch.randn((batch, GEOM["query_heads"], 1, GEOM["head_dim"]), generator=gen, device=device).to(torch.bfloat16)
    torch.cuda.synchronize(device)
    return cache, query


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz, reasons, max_mhz = [], set(), None
        for parts in self.samples:
            try:
                mhz.append(float(parts[0]))
                max_mhz = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": max_mhz, "reasons": sorted(reasons),
                "samples": len(mhz)}


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------------------- CPU arm
def host_threads() -> int:
    """Threads the NumPy/BLAS legs may use: every core this process is allowed to run on."""

    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def cpu_oracle_decode(ctx: int, seed: int, rows: int, repeats: int):
    """Time the oracle port of the reference's page-streamed attention on `rows` batch rows.

    The BLAS pools are opened up to every host core for the duration (a launcher may have pinned them to one).
    """

    try:
        from threadpoolctl import threadpool_limits
    except ImportError:
        return _cpu_oracle_decode(ctx, seed, rows, repeats)
    with threadpool_limits(limits=host_threads()):
        return _cpu_oracle_decode(ctx, seed, rows, repeats)


def _cpu_oracle_decode(ctx: int, seed: int, rows: int, repeats: int):
    from oracle import dartkv_oracle as orc

    rng = np.random.default_rng(seed)
    h, d, hq = GEOM["kv_heads"], GEOM["head_dim"], GEOM["query_heads"]
    mult = np.ones((1, h, 1, d), dtype=np.float32)
    out = outlier_channels(seed).numpy()
    for head in range(h):
        mult[0, head, 0, out[head]] = 10.0
    keys = orc.round_to(rng.standard_normal((rows, h, ctx, d), dtype=np.float32) * mult, "bf16")
    values = orc.round_to(rng.standard_normal((rows, h, ctx, d), dtype=np.float32), "bf16")
    query = orc.round_to(rng.standard_normal((rows, hq, 1, d), dtype=np.float32), "bf16")
    cfg = dict(cache_kwargs())
    cache = orc.OracleCache(orc.CacheConfig(metadata_dtype="bf16", **cfg), "bf16")
    t0 = time.perf_counter()
    cache.append(keys[:, :, : GEOM["sinks"]], values[:, :, : GEOM["sinks"]])
    cache.append(keys[:, :, GEOM["sinks"]:], values[:, :, GEOM["sinks"]:])
    append_s = time.perf_counter() - t0
    orc.streamed_attention(query, cache, "bf16")  # warm-up
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.streamed_attention(query, cache, "bf16")
        times.append(time.perf_counter() - t0)
    return float(np.mean(times)), append_s


def reference_arm(args, wl) -> None:
    """`--impl reference`: the reference's CPU implementation of the path (oracle port), host cores only."""

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1
    step_s, _ = cpu_oracle_decode(wl["ctx"], wl["seed"], rows, max(1, min(args.steps, 3)))
    sample_bytes = rows * GEOM["kv_heads"] * bytes_per_bh(wl["ctx"]) + 2 * rows * GEOM["query_heads"] * GEOM["head_dim"] * 2
    value = sample_bytes / step_s / 1e9
    cores = host_threads()
    line = {
        "impl": "reference", "metric": "fused_decode_attention_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "batch": wl["batch"], "context": wl["ctx"]},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{rows} of {wl['batch']} batch rows, full context, NumPy port of the reference's "
                                   "page-streamed attention (BLAS threads = host cores)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- GPU arm
def append_microbench(device: torch.device, steps: int, warmup: int) -> dict:
    """Quantize+pack append microbench: bf16 K,V [16,8,4096,128], 2-bit + 0.25 promotion, 128 tokens per append."""

    import dartkv_b200 as dart

    b, h, t, d = 16, GEOM["kv_heads"], 4096, GEOM["head_dim"]
    gen = torch.Generator(device=device).manual_seed(1)
    mult = torch.ones(h, d, device=device)
    mult.scatter_(1, outlier_channels(1).to(device), 10.0)
    keys = (torch.randn((b, h, t, d), generator=gen, device=device) * mult.view(1, h, 1, d)).to(torch.bfloat16)
    values = torch.randn((b, h, t, d), generator=gen, device=device).to(torch.bfloat16)
    cfg = dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **cache_kwargs())
    start_evt, stop_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def run(chunk):
        cache = dart.DartKVCache(cfg, max_tokens=t + 256)
        cache.append(keys[:, :, :32], values[:, :, :32])
        torch.cuda.synchronize(device)
        start_evt.record()
        pos = 32
        while pos < t:
            n = min(chunk, t - pos)
            cache.append(keys[:, :, pos:pos + n], values[:, :, pos:pos + n])
            pos += n
        stop_evt.record()
        torch.cuda.synchronize(device)
        return start_evt.elapsed_time(stop_evt) * 1e-3

    out = {}
    pages = (t - 32) // 128
    read = 2 * b * h * (t - 32) * d * 2
    written = b * h * (pages * (5760 + 5120) + (t - 32 - pages * 128) * d * 2 * 2)
    for name, chunk in (("per_128_token_step", 128), ("bulk", t)):
        for _ in range(max(1, warmup)):
            run(chunk)
        secs = float(np.mean([run(chunk) for _ in range(max(1, steps))]))
        out[name] = {"gbs": (read + written) / secs / 1e9, "ms": secs * 1e3,
                     "appends": -(-(t - 32) // chunk)}
    out["bytes"] = {"read": read, "written": written}
    return out


def gpu_arm(args, wl) -> None:
    import torch.distributed as dist

    import dartkv_b200 as dart
    from dartkv_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        # the only collective is a gather of [B/N, Hq, D] outputs (1 MB in total): in-switch reduction buys nothing
        # here and its set-up dominates communicator creation on 8 GPUs
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    from dartkv_b200.sharding import shard_rows

    lo, hi = shard_rows(wl["batch"], world, rank)
    local_batch = hi - lo
    cache, query = build_device_cache(local_batch, wl["ctx"], wl["seed"], rank, device)
    hq, d = GEOM["query_heads"], GEOM["head_dim"]
    out = torch.empty((local_batch, hq, d), dtype=torch.bfloat16, device=device)
    gathered = torch.empty((world * local_batch, hq, d), dtype=torch.bfloat16, device=device) if world > 1 else None
    q3 = query[:, :, 0].contiguous()

    flavour = _lib.DEQUANT_FUSED if args.flavour == "fused" else _lib.DEQUANT_PER_OP

    def step():
        dart.decode_attention(q3, cache, out=out, flavour=flavour)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)  # the only cross-GPU traffic: final output gather

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    start_evt, stop_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = _lib.LIB.dartkv_launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        start_evt.record()
        for _ in range(args.steps):
            step()
        stop_evt.record()
        launches = _lib.LIB.dartkv_launch_count() - launches_before
        barrier()
        # keep the sampler alive long enough for at least a few readings under load
        elapsed_ms = start_evt.elapsed_time(stop_evt)
        if elapsed_ms < 600:
            t_end = time.time() + 0.6
            while time.time() < t_end:
                step()
            torch.cuda.synchronize(device)
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    total_bytes = step_bytes(wl["batch"], wl["ctx"])
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # dominant kernel alone (no gather), per-launch device time on the launching stream
    barrier()
    start_evt.record()
    for _ in range(args.steps):
        dart.decode_attention(q3, cache, out=out, flavour=flavour)
    stop_evt.record()
    torch.cuda.synchronize(device)
    kernel_ms = start_evt.elapsed_time(stop_evt) / args.steps
    local_bytes = step_bytes(local_batch, wl["ctx"])
    peak, peak_kind = measured_peak_gbs()
    achieved = local_bytes / (kernel_ms * 1e-3) / 1e9
    # DRAM traffic of one decode launch from the ncu capture of config 3 (profiles/decode_fast_kernel_config3.md):
    # 192.72 MB read + 6.54 MB written for 192.77 MB algorithmic; traffic grows with the pages processed, so
    # other workloads scale it by their algorithmic bytes
    traffic = int(round(local_bytes * (192.72e6 + 6.54e6) / 192774144))

    # end to end through host buffers: pinned query -> device, attention, output -> pinned host
    host_q = q3.cpu().pin_memory()
    host_out = torch.empty_like(out, device="cpu").pin_memory()
    dev_q = torch.empty_like(q3)

    def e2e_step():
        dev_q.copy_(host_q, non_blocking=True)
        dart.decode_attention(dev_q, cache, out=out, flavour=flavour)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)
            host_out.copy_(gathered[rank * local_batch:(rank + 1) * local_batch], non_blocking=True)
        else:
            host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9

    extra = {}
    if rank == 0 and world == 1 and not args.skip_extras:
        del gathered
        if args.flavour == "per_op":
            # the same call with the arithmetic of the reference's Triton kernels (dequantized values never rounded)
            for _ in range(3):
                dart.decode_attention(q3, cache, out=out, flavour=_lib.DEQUANT_FUSED)
            torch.cuda.synchronize(device)
            start_evt.record()
            for _ in range(args.steps):
                dart.decode_attention(q3, cache, out=out, flavour=_lib.DEQUANT_FUSED)
            stop_evt.record()
            torch.cuda.synchronize(device)
            fused_ms = start_evt.elapsed_time(stop_evt) / args.steps
            fused_gbs = local_bytes / (fused_ms * 1e-3) / 1e9
            extra["unrounded_fp32_variant"] = {
                "value": fused_gbs, "unit": "GB/s", "us_per_launch": fused_ms * 1e3, "frac": fused_gbs / peak,
                "note": "flavour DEQUANT_FUSED: code*scale+zero kept in fp32 like the reference's Triton kernels; "
                        "not the pinned oracle's arithmetic, so it is reported beside the headline, not as it"}
        extra["append"] = append_microbench(device, steps=3, warmup=1)
        rows = 1
        step_s, append_s = cpu_oracle_decode(wl["ctx"], wl["seed"], rows, 1)
        sample_bytes = rows * GEOM["kv_heads"] * bytes_per_bh(wl["ctx"]) + 2 * rows * hq * d * 2
        extra["cpu_baseline"] = {
            "value": sample_bytes / step_s / 1e9, "unit": "GB/s", "cores": host_threads(), "kind": "port",
            "sample": f"{rows} of {wl['batch']} batch rows, full context ({step_s:.2f} s per step; NumPy port of "
                      f"the reference's page-streamed attention, BLAS threads = host cores; oracle append of the "
                      f"sample took {append_s:.1f} s)"}
    if rank == 0:
        line = {
            "metric": "fused_decode_attention_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "us_per_step": ms_per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "batch": wl["batch"], "context": wl["ctx"], "per_gpu_batch": local_batch,
                       "query_heads": hq, "kv_heads": GEOM["kv_heads"], "head_dim": d, "page": GEOM["page"],
                       "bits": "2-bit + 0.25 promotion", "key_group": GEOM["key_group"], "value_group": GEOM["value_group"],
                       "sinks": GEOM["sinks"], "metadata": "bf16", "bytes_per_step": total_bytes,
                       "dequant": "per-op rounded (reference streamed path)" if args.flavour == "per_op"
                       else "unrounded fp32 (reference Triton kernels)",
                       "l2": f"per-GPU working set {local_bytes / 1e6:.0f} MB exceeds the 126 MB L2",
                       "parallelism": f"batch sharded over {world} GPU(s), output all-gather only"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_unit": "bytes per launch (ncu, config 3 capture scaled by algorithmic bytes)",
                         "peak_kind": peak_kind, "kernel": "decode attention call (all its kernels)",
                         "us_per_launch": kernel_ms * 1e3, "per_gpu_gbs": achieved},
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(q3.numel() * 2), "d2h_bytes_per_step": int(out.numel() * 2)},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def qwen3_decode(args) -> None:
    """Qwen3-8B-architecture greedy decode through DartHFCache + the fused decode hook (random bf16 weights)."""

    from transformers import Qwen3Config, Qwen3ForCausalLM

    import dartkv_b200 as dart
    from dartkv_b200 import _lib
    from dartkv_b200.integrations import DartHFCache, attach_dart_fused_attention
    from dartkv_b200.integrations import qwen3 as hook

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    batch, prompt_len, new_tokens = 8, 1024, max(2, args.steps if args.steps != 20 else 256)
    config = Qwen3Config(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                         num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                         rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, initializer_range=0.02)
    config._attn_implementation = "sdpa"
    torch.manual_seed(3)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(device):
        model = Qwen3ForCausalLM(config)
    torch.set_default_dtype(torch.float32)
    model.eval()
    attach_dart_fused_attention(model)
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, local_tokens=1, value_local_tokens=128,
                                 metadata_dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, config.vocab_size, (batch, prompt_len), generator=gen).to(device)

    # time spent inside the hot path (cache update + fused attention) per decode step, by CUDA events
    spans = []
    original = hook.fused_dart_attention
    original_update = DartHFCache.update

    def timed_attention(*a, **k):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = original(*a, **k)
        stop.record()
        spans.append((start, stop))
        return out

    def timed_update(self, *a, **k):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = original_update(self, *a, **k)
        stop.record()
        spans.append((start, stop))
        return out

    def run(measure: bool):
        cache = DartHFCache(cfg, max_tokens=prompt_len + new_tokens + 128)
        with torch.no_grad():
            logits = model(prompt, past_key_values=cache, use_cache=True).logits[:, -1]
            token = logits.argmax(-1, keepdim=True)
            torch.cuda.synchronize(device)
            if measure:
                hook.fused_dart_attention = timed_attention
                DartHFCache.update = timed_update
            launches = _lib.LIB.dartkv_launch_count()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(new_tokens):
                logits = model(token, past_key_values=cache, use_cache=True).logits[:, -1]
                token = logits.argmax(-1, keepdim=True)
            t1.record()
            torch.cuda.synchronize(device)
            hook.fused_dart_attention = original
            DartHFCache.update = original_update
        return t0.elapsed_time(t1), _lib.LIB.dartkv_launch_count() - launches, cache

    run(False)                       # warm-up: allocator, cuBLAS heuristics, kernel load
    spans.clear()
    with ClockSampler(0) as clocks:
        ms, launches, cache = run(True)
    hot_ms = sum(a.elapsed_time(b) for a, b in spans)
    line = {
        "metric": "qwen3_8b_arch_decode_tokens_per_s", "value": batch * new_tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": new_tokens, "warmup": 1, "ms_per_step": ms / new_tokens, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config4", "model": "Qwen3-8B architecture, random-init bf16 weights (std 0.02)",
                   "batch": batch, "prompt": prompt_len, "new_tokens": new_tokens,
                   "cache": "2-bit + 0.25 promotion, page 128, groups 128/64, 32 sinks, local 1, value local 128, bf16 metadata"},
        "attention_share_of_step": hot_ms / ms, "hot_path_ms_per_step": hot_ms / new_tokens,
        "compression_ratio": cache.compression_ratio, "gpu_launches": int(launches), "clocks": clocks.summary(),
        "e2e": {"value": batch * new_tokens / (ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0, "note": "token ids stay on the device between steps"},
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=sorted(WORKLOADS) + ["config4"], default="config5")
    parser.add_argument("--skip-extras", action="store_true", help="skip the append microbench and the CPU baseline")
    parser.add_argument("--flavour", choices=("per_op", "fused"), default="per_op",
                        help="dequantization arithmetic of the timed decode call (default: the pinned per-op rounding)")
    parser.add_argument("--batch", type=int, default=0, help="override the workload's batch (e.g. one rank's share)")
    parser.add_argument("--context", type=int, default=0, help="override the workload's context length")
    args = parser.parse_args()
    if args.workload == "config4":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "config4 needs the GPU model run; the CPU arm covers config5/config3"}))
            return
        qwen3_decode(args)
        return
    wl = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        wl["batch"] = args.batch
    if args.context > 0:
        wl["ctx"] = args.context
    if args.impl == "reference":
        reference_arm(args, wl)
    else:
        gpu_arm(args, wl)


if __name__ == "__main__":
    main()
