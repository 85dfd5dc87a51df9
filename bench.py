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
# DRAM bytes of ONE decode launch at config 3 measured with ncu (dram__bytes_read.sum / dram__bytes_write.sum of the
# tensor-core decode kernel, per-op flavour) next to that launch's algorithmic bytes
NCU_CONFIG3 = {"algorithmic": 192774144, "dram_read": 192.75e6, "dram_write": 6.55e6}
# the same numbers as dartkv_b200.synthetic.HEADLINE_GEOMETRY (kept here so that the CPU reference arm runs without
# loading the package or its CUDA library; the GPU arm asserts that the two agree)
GEOM = dict(query_heads=32, kv_heads=8, head_dim=128, page=128, key_group=128, value_group=64, sinks=32,
            promote_ratio=0.25, bits=2)
HEADLINE = dict(GEOM)   # --bits / --promote / --value-group change GEOM for runs off the headline geometry


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
    return GEOM["sinks"] * d * 2 * 2 + pages * page_bytes() + tail * d * 2 * 2


def page_bytes() -> int:
    """Packed bytes of one 128-token page of one (batch row, KV head), 16-bit metadata: 5760 + 5120 on the headline
    geometry.  Keys: code rows (2-bit rows plus a 2-bit plane and int32 indices for the promoted channels, or
    `bits`-wide rows), a scale and a zero point per channel and key group.  Values: code rows, a scale and a zero
    point per token and value group."""

    d, page = GEOM["head_dim"], GEOM["page"]
    promoted = min(d, int(d * GEOM["promote_ratio"] + 1e-6))
    key_meta = 2 * d * (page // GEOM["key_group"]) * 2
    if promoted:
        key = d * page // 4 + promoted * page // 4 + promoted * 4 + key_meta
    else:
        key = d * page * GEOM["bits"] // 8 + key_meta
    value = page * d * GEOM["bits"] // 8 + page * 2 * (d // GEOM["value_group"]) * 2
    return key + value


def step_bytes(batch: int, ctx: int) -> int:
    qo = 2 * batch * GEOM["query_heads"] * GEOM["head_dim"] * 2
    return batch * GEOM["kv_heads"] * bytes_per_bh(ctx) + qo


def outlier_channels(seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    count = int(0.05 * GEOM["head_dim"])
    return torch.stack([torch.randperm(GEOM["head_dim"], generator=gen)[:count] for _ in range(GEOM["kv_heads"])])


def build_device_cache(rows, ctx: int, seed: int, device: torch.device, keep_inputs: bool = False, heads=None):
    """The workload's cache for the global batch rows `rows` (see dartkv_b200.synthetic.build_headline_cache)."""

    from dartkv_b200.synthetic import HEADLINE_GEOMETRY, build_headline_cache

    assert HEADLINE_GEOMETRY == HEADLINE
    overrides = {{"bits": "bits", "promote_ratio": "promote_ratio", "value_group": "value_group_size"}[k]: GEOM[k]
                 for k in ("bits", "promote_ratio", "value_group") if GEOM[k] != HEADLINE[k]}
    rows = list(rows)
    got = build_headline_cache(rows, ctx, seed, device, heads=heads, keep_rows=rows if keep_inputs else None,
                               cache_overrides=overrides,
                               metadata_dtype=torch.float16 if GEOM.get("metadata") == "fp16" else torch.bfloat16)
    return got if keep_inputs else got[:2]


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
    """Threads the CPU legs may use: every core this process is allowed to run on."""

    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def reference_package():
    """The reference's own `dart` package when an install of it sits in oracle/_ref (made by oracle/make_ref.sh),
    else None.  It is only ever used as the timed CPU / GPU baseline, never by the product path."""

    path = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(path, "dart")):
        return None
    if path not in sys.path:
        sys.path.insert(0, path)
    try:
        import dart
    except Exception:   # an install that does not import here is the same as no install
        return None
    return dart


def synthetic_rows_cpu(ctx: int, seed: int, rows: int):
    """bf16 K, V [rows,H,ctx,D] and query [rows,Hq,1,D] as torch CPU tensors (same distributions as the GPU arm)."""

    rng = np.random.default_rng(seed)
    h, d, hq = GEOM["kv_heads"], GEOM["head_dim"], GEOM["query_heads"]
    mult = np.ones((1, h, 1, d), dtype=np.float32)
    out = outlier_channels(seed).numpy()
    for head in range(h):
        mult[0, head, 0, out[head]] = 10.0
    keys = torch.from_numpy(rng.standard_normal((rows, h, ctx, d), dtype=np.float32) * mult).to(torch.bfloat16)
    values = torch.from_numpy(rng.standard_normal((rows, h, ctx, d), dtype=np.float32)).to(torch.bfloat16)
    query = torch.from_numpy(rng.standard_normal((rows, hq, 1, d), dtype=np.float32)).to(torch.bfloat16)
    return keys, values, query


class CpuDecode:
    """The reference's CPU implementation of the path on `rows` batch rows of the workload at full context:
    its own package when installed (kind "reference"), else the NumPy port in oracle/ (kind "port")."""

    def __init__(self, ctx: int, seed: int, rows: int):
        self.cores = host_threads()
        torch.set_num_threads(self.cores)
        keys, values, query = synthetic_rows_cpu(ctx, seed, rows)
        dart = reference_package()
        t0 = time.perf_counter()
        if dart is not None:
            self.kind = "reference"
            cfg = dart.DartKVCacheConfig(metadata_dtype=torch.float16 if GEOM.get("metadata") == "fp16" else torch.bfloat16,
                                         **cache_kwargs())
            cache = dart.DartKVCache(cfg)
            cache.append(keys[:, :, : GEOM["sinks"]], values[:, :, : GEOM["sinks"]])
            cache.append(keys[:, :, GEOM["sinks"]:], values[:, :, GEOM["sinks"]:])
            self._step = lambda: dart.streamed_dart_attention(query, cache)
            self.what = "the reference's own streamed_dart_attention on torch CPU tensors"
        else:
            from threadpoolctl import threadpool_limits   # the port's matrix products run in the BLAS pool

            from oracle import dartkv_oracle as orc

            self.kind = "port"
            self._limits = threadpool_limits(limits=self.cores)
            cache = orc.OracleCache(orc.CacheConfig(metadata_dtype="f16" if GEOM.get("metadata") == "fp16" else "bf16",
                                                    **cache_kwargs()), "bf16")
            k32, v32, q32 = keys.float().numpy(), values.float().numpy(), query.float().numpy()
            cache.append(k32[:, :, : GEOM["sinks"]], v32[:, :, : GEOM["sinks"]])
            cache.append(k32[:, :, GEOM["sinks"]:], v32[:, :, GEOM["sinks"]:])
            self._step = lambda: orc.streamed_attention(q32, cache, "bf16")
            self.what = "NumPy port of the reference's page-streamed attention (BLAS threads = host cores)"
        self.append_s = time.perf_counter() - t0
        self.rows = rows
        self.bytes = rows * GEOM["kv_heads"] * bytes_per_bh(ctx) + 2 * rows * GEOM["query_heads"] * GEOM["head_dim"] * 2

    def time_steps(self, steps: int, warmup: int) -> float:
        """Mean seconds per step over exactly `steps` timed steps after `warmup` untimed ones."""

        for _ in range(warmup):
            self._step()
        t0 = time.perf_counter()
        for _ in range(steps):
            self._step()
        return (time.perf_counter() - t0) / steps


def workload_config(args, wl, world: int) -> dict:
    """The `config` object of the JSON line: identical for the GPU arm and the reference arm of one launch."""

    local_batch = -(-wl["batch"] // world) if wl["batch"] >= world else 1
    head_groups = 1 if wl["batch"] >= world else world // wl["batch"]
    local_bytes = step_bytes(local_batch, wl["ctx"]) // head_groups
    return {"workload": args.workload, "batch": wl["batch"], "context": wl["ctx"], "per_gpu_batch": local_batch,
            "query_heads": GEOM["query_heads"], "kv_heads": GEOM["kv_heads"], "head_dim": GEOM["head_dim"],
            "page": GEOM["page"],
            "bits": f"{GEOM['bits']}-bit values, " + (f"2+2-bit keys ({GEOM['promote_ratio']} promoted)" if GEOM["promote_ratio"] > 0
                                                       else f"{GEOM['bits']}-bit keys")
            if GEOM != HEADLINE else "2-bit + 0.25 promotion",
            "key_group": GEOM["key_group"],
            "value_group": GEOM["value_group"], "sinks": GEOM["sinks"], "metadata": GEOM.get("metadata", "bf16"),
            "bytes_per_step": step_bytes(wl["batch"], wl["ctx"]),
            "dequant": {"per_op": "per-op rounded (reference streamed path)",
                        "fp32": "fp32 with one rounding (reference streamed path on CUDA)",
                        "fused": "unrounded fp32 (reference Triton kernels)"}[args.flavour],
            "l2": f"per-GPU working set {local_bytes / 1e6:.0f} MB exceeds the 126 MB L2",
            "parallelism": (f"batch sharded over {world} GPU(s)" if head_groups == 1 else
                            f"batch x KV heads sharded over {world} GPU(s) ({head_groups} head groups)") +
                           ", output all-gather only"}


def reference_arm(args, wl) -> None:
    """`--impl reference`: the reference's CPU implementation of the path, host cores only, rank 0 only.

    A step is one decode-attention pass over a bounded sample of the workload (one batch row at full context);
    exactly `--steps` steps are timed after `--warmup` untimed ones.
    """

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuDecode(wl["ctx"], wl["seed"], rows=1)
    warmup = max(1, args.warmup)
    step_s = cpu.time_steps(args.steps, warmup)
    value = cpu.bytes / step_s / 1e9
    sample = (f"{cpu.rows} of {wl['batch']} batch rows at full context per step; {cpu.what}; building the "
              f"sample's cache took {cpu.append_s:.1f} s (untimed)")
    line = {
        "impl": "reference", "metric": "fused_decode_attention_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, wl, args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cpu.cores, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- GPU arm
# packed bytes per 128-token page and (batch, kv head): key page by key mode, value page by value bits
# (key group 128, value group 64, bf16 metadata)
KEY_PAGE_BYTES = {"mixed": 4096 + 1024 + 128 + 256 + 256, 2: 4096 + 512, 4: 8192 + 512, 8: 16384 + 512}
VALUE_PAGE_BYTES = {2: 4096 + 1024, 4: 8192 + 1024, 8: 16384 + 1024}
APPEND_VARIANTS = (("v2_mixed", 2, 0.25), ("v4_mixed", 4, 0.25), ("v8_mixed", 8, 0.25),
                   ("v2_uniform", 2, 0.0), ("v4_uniform", 4, 0.0), ("v8_uniform", 8, 0.0))


def append_microbench(device: torch.device, steps: int, warmup: int) -> dict:
    """Quantize+pack append microbench: bf16 K,V [16,8,4096,128], page 128, groups 128/64, 32 sinks; value bits
    2/4/8 with promoted 2+2-bit keys (ratio 0.25) or uniform keys of the same width; 128 tokens per append and,
    for the roofline figure, the whole tensor in one append."""

    import dartkv_b200 as dart

    b, h, t, d = 16, GEOM["kv_heads"], 4096, GEOM["head_dim"]
    gen = torch.Generator(device=device).manual_seed(1)
    mult = torch.ones(h, d, device=device)
    mult.scatter_(1, outlier_channels(1).to(device), 10.0)
    keys = (torch.randn((b, h, t, d), generator=gen, device=device) * mult.view(1, h, 1, d)).to(torch.bfloat16)
    values = torch.randn((b, h, t, d), generator=gen, device=device).to(torch.bfloat16)
    start_evt, stop_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pages = (t - 32) // 128
    read = 2 * b * h * (t - 32) * d * 2
    out = {}
    for name, bits, ratio in APPEND_VARIANTS:
        kwargs = dict(cache_kwargs(), bits=bits, promote_ratio=ratio)
        cfg = dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **kwargs)

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

        def run_graph():
            """The same 128-token appends replayed from a CUDA graph: device time per append without the host."""

            cache = dart.DartKVCache(cfg, max_tokens=t + 256)
            cache.append(keys[:, :, :32], values[:, :, :32])
            torch.cuda.synchronize(device)
            side = torch.cuda.Stream(device=device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    pos = 32
                    while pos < t:
                        n = min(128, t - pos)
                        cache.append(keys[:, :, pos:pos + n], values[:, :, pos:pos + n])
                        pos += n
            torch.cuda.synchronize(device)
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize(device)
            start_evt.record()
            for _ in range(max(1, steps)):
                graph.replay()
            stop_evt.record()
            torch.cuda.synchronize(device)
            cache.check_finite()
            return start_evt.elapsed_time(stop_evt) * 1e-3 / max(1, steps)

        key_page = KEY_PAGE_BYTES["mixed" if ratio > 0 else bits]
        written = b * h * (pages * (key_page + VALUE_PAGE_BYTES[bits]) + (t - 32 - pages * 128) * d * 2 * 2)
        entry = {"bytes_read": read, "bytes_written": written}
        for label, chunk in (("per_128_token_step", 128), ("bulk", t)):
            for _ in range(max(1, warmup)):
                run(chunk)
            secs = float(np.mean([run(chunk) for _ in range(max(1, steps))]))
            appends = -(-(t - 32) // chunk)
            entry[label] = {"gbs": (read + written) / secs / 1e9, "ms": secs * 1e3, "appends": appends,
                            "us_per_append": secs * 1e6 / appends}
        try:
            secs = run_graph()
            appends = -(-(t - 32) // 128)
            entry["per_128_token_step_cuda_graph"] = {"gbs": (read + written) / secs / 1e9, "ms": secs * 1e3,
                                                      "appends": appends, "us_per_append": secs * 1e6 / appends}
        except Exception as exc:   # graph capture refused by this driver / allocator state: the eager figure stands
            entry["per_128_token_step_cuda_graph"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}
        out[name] = entry
    # the headline variant keeps its place at the top level
    out["per_128_token_step"] = out["v2_mixed"]["per_128_token_step"]
    out["per_128_token_step_cuda_graph"] = out["v2_mixed"]["per_128_token_step_cuda_graph"]
    out["bulk"] = out["v2_mixed"]["bulk"]
    out["bytes"] = {"read": read, "written": out["v2_mixed"]["bytes_written"]}
    return out


def other_geometry_decode(device: torch.device, steps: int, peak: float) -> list:
    """Decode steps of the general tensor-core kernel on config 3's shape (batch 32, context 8192, same data) with
    other code widths and group sizes, and the fp32 flavour of the headline geometry: what a cache off the 2-bit
    headline geometry gets."""

    import dartkv_b200 as dart
    from dartkv_b200 import _lib

    saved = dict(GEOM)
    results = []
    variants = [("4-bit keys and values", dict(bits=4, promote_ratio=0.0), _lib.DEQUANT_PER_OP),
                ("2+2-bit keys, 4-bit values", dict(bits=4), _lib.DEQUANT_PER_OP),
                ("8-bit keys and values", dict(bits=8, promote_ratio=0.0), _lib.DEQUANT_PER_OP),
                ("headline widths, value groups of 32", dict(value_group=32), _lib.DEQUANT_PER_OP),
                ("headline geometry, fp32 flavour", dict(), _lib.DEQUANT_FP32),
                ("headline geometry, fp16 metadata beside the bf16 cache (the reference scripts' setting; per-op "
                 "kernel with operand casts)", dict(metadata="fp16"), _lib.DEQUANT_PER_OP)]
    start_evt, stop_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        for name, change, flavour in variants:
            GEOM.clear()
            GEOM.update(saved)
            GEOM.update(change)
            cache, query = build_device_cache(range(32), 8192, WORKLOADS["config3"]["seed"], device)
            q3 = query[:, :, 0].contiguous()
            out = torch.empty_like(q3)
            for _ in range(3):
                dart.decode_attention(q3, cache, out=out, flavour=flavour)
            torch.cuda.synchronize(device)
            start_evt.record()
            for _ in range(steps):
                dart.decode_attention(q3, cache, out=out, flavour=flavour)
            stop_evt.record()
            torch.cuda.synchronize(device)
            us = start_evt.elapsed_time(stop_evt) / steps * 1e3
            nbytes = step_bytes(32, 8192)
            results.append({"geometry": name, "us_per_step": us, "bytes_per_step": nbytes, "value": nbytes / us / 1e3,
                            "unit": "GB/s", "frac": nbytes / us / 1e3 / peak, "decode_status": cache.decode_status()})
            del cache
            torch.cuda.empty_cache()
    finally:
        GEOM.clear()
        GEOM.update(saved)
    return results


def decode_step_graph(device: torch.device, batch: int = 32, ctx: int = 8192, steps: int = 64) -> dict:
    """One generation step of a layer: append the new token's K and V, then decode attention.  Eager (host-planned
    append through the Python mirror, two library calls per step) against one CUDA graph that holds the
    device-planned append and the attention, captured once and replayed.  Config 3's shape is bound by the decode
    kernel either way; the shape of one Qwen3-8B layer in config 4 (batch 8, context 1024) is bound by the host."""

    import dartkv_b200 as dart

    cache, query = build_device_cache(range(batch), ctx, WORKLOADS["config3"]["seed"], device)
    capacity = ctx + 4 * steps + 256
    gen = torch.Generator(device=device).manual_seed(11)
    shape = (batch, GEOM["kv_heads"], 1, GEOM["head_dim"])
    new_k = torch.randn(shape, generator=gen, device=device).to(torch.bfloat16)
    new_v = torch.randn(shape, generator=gen, device=device).to(torch.bfloat16)
    out = torch.empty(batch, GEOM["query_heads"], GEOM["head_dim"], dtype=torch.bfloat16, device=device)
    start_evt, stop_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def eager_step():
        cache.append(new_k, new_v)
        dart.fused_dart_attention(query, cache, fallback=False, out=out)

    def planned_step():
        cache.append_device_planned(new_k, new_v)
        dart.fused_dart_attention(query, cache, fallback=False, out=out, token_capacity=capacity)

    cache._ensure_capacity(capacity // GEOM["page"] + 2, capacity)   # pools may not move under the graph
    for _ in range(3):
        eager_step()
    torch.cuda.synchronize(device)
    start_evt.record()
    for _ in range(steps):
        eager_step()
    stop_evt.record()
    torch.cuda.synchronize(device)
    eager_us = start_evt.elapsed_time(stop_evt) / steps * 1e3
    planned_step()
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        planned_step()
    graph.replay()
    torch.cuda.synchronize(device)
    start_evt.record()
    for _ in range(steps):
        cache.advance_device_planned(1)
        graph.replay()
    stop_evt.record()
    torch.cuda.synchronize(device)
    graph_us = start_evt.elapsed_time(stop_evt) / steps * 1e3
    status = cache.decode_status()
    del graph, cache
    torch.cuda.empty_cache()
    return {"what": f"append of one token per row + decode attention, batch {batch}, context {ctx} and growing",
            "eager_us_per_step": eager_us, "cuda_graph_us_per_step": graph_us, "steps": steps, "decode_status": status}


def reference_gpu_decode(wl, device: torch.device, steps: int) -> dict:
    """The reference's own Triton decode kernel (fused_dart_attention, fallback off) on this GPU, on a bounded
    sample of the workload: min(batch, 8) rows at full context, cache built by the reference's own append."""

    dart = reference_package()
    if dart is None:
        return {"unavailable": "no install of the reference under oracle/_ref"}
    rows = min(wl["batch"], 8)
    try:
        cache, query, keys, values = build_device_cache(range(rows), wl["ctx"], wl["seed"], device, keep_inputs=True)
        del cache
        cfg = dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **cache_kwargs())
        ref = dart.DartKVCache(cfg)
        ref.append(keys[:, :, : GEOM["sinks"]], values[:, :, : GEOM["sinks"]])
        ref.append(keys[:, :, GEOM["sinks"]:], values[:, :, GEOM["sinks"]:])
        del keys, values
        for _ in range(2):
            dart.fused_dart_attention(query, ref, fallback=False)
        torch.cuda.synchronize(device)
        start_evt, stop_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = max(1, min(steps, 5))
        start_evt.record()
        for _ in range(steps):
            dart.fused_dart_attention(query, ref, fallback=False)
        stop_evt.record()
        torch.cuda.synchronize(device)
        ms = start_evt.elapsed_time(stop_evt) / steps
    except Exception as exc:   # e.g. Triton cannot JIT on this device
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    sample_bytes = step_bytes(rows, wl["ctx"])
    return {"value": sample_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": steps,
            "sample": f"{rows} of {wl['batch']} batch rows at full context; the reference's Triton kernels "
                      "(one launch per page), same algorithmic bytes per row"}


def gpu_arm(args, wl) -> None:
    import datetime

    import torch.distributed as dist

    import dartkv_b200 as dart
    from dartkv_b200 import _lib
    from dartkv_b200.sharding import PeerGather, gather_outputs, shard_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        # the only collective is a gather of [B/N, Hq, D] outputs (1 MB in total): in-switch reduction buys nothing
        # here and its set-up dominates communicator creation on 8 GPUs.  The short timeout makes a rank that is
        # out of step give up with an error instead of spinning.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))

    shard = shard_plan(wl["batch"], GEOM["kv_heads"], world, rank)
    local_batch = shard.rows
    heads = (shard.head_begin, shard.head_end)
    cache, query = build_device_cache(range(shard.row_begin, shard.row_end), wl["ctx"], wl["seed"], device, heads=heads)
    hq, d = GEOM["query_heads"], GEOM["head_dim"]
    hq_local = query.shape[1]
    out = torch.empty((local_batch, hq_local, d), dtype=torch.bfloat16, device=device)
    gathered = torch.empty((wl["batch"], hq, d), dtype=torch.bfloat16, device=device) if world > 1 else None
    q3 = query[:, :, 0].contiguous()
    gather_kwargs = dict(shard=shard, batch=wl["batch"], kv_heads=GEOM["kv_heads"])
    q_lo, q_hi = shard.query_heads(hq, GEOM["kv_heads"])
    # how the outputs reach every rank: stored straight into the peers' gathered tensors by the kernel that
    # normalizes them ("peer", the default), or an NCCL all-gather after the decode call ("nccl")
    peer, gather_kind = None, "nccl all_gather_into_tensor"
    if world > 1 and args.gather == "peer":
        try:
            peer = PeerGather(shard, wl["batch"], hq, GEOM["kv_heads"], d, torch.bfloat16, device)
            gather_kind = "peer stores from the decode kernels (symmetric memory over NVLink, no multicast)"
        except Exception as exc:   # symmetric memory cannot be set up on this machine: NCCL does the gather
            gather_kind = f"nccl all_gather_into_tensor (peer stores unavailable: {type(exc).__name__}: {str(exc)[:120]})"

    flavour = {"per_op": _lib.DEQUANT_PER_OP, "fp32": _lib.DEQUANT_FP32, "fused": _lib.DEQUANT_FUSED}[args.flavour]

    def decode():
        dart.decode_attention(q3, cache, out=out, flavour=flavour)

    def step():
        nonlocal gathered
        if peer is not None:
            gathered = dart.decode_attention(q3, cache, out=out, flavour=flavour, peer_gather=peer)
            return
        decode()
        if world > 1:
            gather_outputs(out, gathered, **gather_kwargs)  # the only cross-GPU traffic: final output gather

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    warmup = max(3, args.warmup)
    for _ in range(warmup):
        step()
    barrier()

    # ---- the gathered result is checked once, outside the timed region: this rank's slice must be its own
    # output, and the first row of the next rank's slice must match a local recomputation of that batch row
    gather_check = None
    if world > 1:
        mine_ok = bool(torch.equal(gathered[shard.row_begin:shard.row_end, q_lo:q_hi], out))
        other = shard_plan(wl["batch"], GEOM["kv_heads"], world, (rank + 1) % world)
        peer_heads = (other.head_begin, other.head_end)
        peer_cache, peer_query = build_device_cache([other.row_begin], wl["ctx"], wl["seed"], device, heads=peer_heads)
        peer_out = torch.empty((1, peer_query.shape[1], d), dtype=torch.bfloat16, device=device)
        dart.decode_attention(peer_query[:, :, 0].contiguous(), peer_cache, out=peer_out, flavour=flavour)
        p_lo, p_hi = other.query_heads(hq, GEOM["kv_heads"])
        got = gathered[other.row_begin, p_lo:p_hi].float()
        diff = (got - peer_out[0].float()).abs()
        # the split of the work differs with the batch size, so the two fp32 sums may round differently: one
        # output ulp (or 2e-3) is allowed
        peer_ok = bool(((diff <= 2e-3) | (diff <= got.abs() * 2.0 ** -7)).all())
        flags = torch.tensor([int(mine_ok), int(peer_ok)], dtype=torch.int32, device=device)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        gather_check = {"own_slice_equal": bool(flags[0].item()), "peer_row_recomputed_within_1ulp": bool(flags[1].item()),
                        "peer_max_abs": float(diff.max().item())}
        del peer_cache, peer_query, peer_out
        if not (gather_check["own_slice_equal"] and gather_check["peer_row_recomputed_within_1ulp"]):
            raise SystemExit(f"gathered outputs are wrong: {gather_check}")
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
        elapsed_ms = start_evt.elapsed_time(stop_evt)
        # keep the GPU under the same load for ~0.6 s so that the 100 ms clock sampler sees it: a fixed number of
        # local decode calls, no collective (a collective count that depends on a rank's own clock deadlocks)
        extra = int(min(20000, max(0, (600.0 - elapsed_ms) / max(elapsed_ms / args.steps, 1e-3))))
        for _ in range(extra):
            decode()
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
        decode()
    stop_evt.record()
    torch.cuda.synchronize(device)
    kernel_ms = start_evt.elapsed_time(stop_evt) / args.steps
    local_bytes = step_bytes(local_batch, wl["ctx"]) * shard.heads // GEOM["kv_heads"]
    peak, peak_kind = measured_peak_gbs()
    achieved = local_bytes / (kernel_ms * 1e-3) / 1e9
    # DRAM traffic of one decode launch from the ncu capture of config 3; it grows with the pages processed, so
    # other workloads scale it by their algorithmic bytes
    traffic = int(round(local_bytes * (NCU_CONFIG3["dram_read"] + NCU_CONFIG3["dram_write"]) / NCU_CONFIG3["algorithmic"]))
    if GEOM != HEADLINE or args.flavour != "per_op":
        traffic = None   # the capture is of the headline geometry's per-op kernel

    # end to end through host buffers.  Every step copies its query from pinned host memory to the device, runs
    # the decode call (and the gather), and copies its output rows back to pinned host memory, all inside the timed
    # region.  Two arrangements are timed:
    #   blocking   the host waits for each step's output before it starts the next step;
    #   pipelined  (the reported figure) the copies go on a second stream with two buffers, so the query of step
    #              i+1 travels while step i computes and the host reads the output of step i one step later, the way
    #              a serving loop keeps a device busy.
    host_q = q3.cpu().pin_memory()
    host_out = [torch.empty_like(out, device="cpu").pin_memory() for _ in range(2)]
    dev_q = [torch.empty_like(q3) for _ in range(2)]
    dev_out = [torch.empty_like(out) for _ in range(2)]
    main_stream = torch.cuda.current_stream(device)
    copy_stream = torch.cuda.Stream(device=device)

    def decode_into(slot):
        if peer is not None:
            full = dart.decode_attention(dev_q[slot], cache, out=out, flavour=flavour, peer_gather=peer)
            dev_out[slot].copy_(full[shard.row_begin:shard.row_end, q_lo:q_hi])
        elif world > 1:
            dart.decode_attention(dev_q[slot], cache, out=out, flavour=flavour)
            gather_outputs(out, gathered, **gather_kwargs)
            dev_out[slot].copy_(gathered[shard.row_begin:shard.row_end, q_lo:q_hi])
        else:
            dart.decode_attention(dev_q[slot], cache, out=dev_out[slot], flavour=flavour)

    def e2e_blocking(steps):
        for _ in range(steps):
            dev_q[0].copy_(host_q, non_blocking=True)
            decode_into(0)
            host_out[0].copy_(dev_out[0], non_blocking=True)
            main_stream.synchronize()

    def e2e_pipelined(steps):
        ready = [torch.cuda.Event() for _ in range(2)]      # query of the slot has arrived
        done = [torch.cuda.Event() for _ in range(2)]       # output of the slot has been computed
        landed = [torch.cuda.Event() for _ in range(2)]     # output of the slot has reached the host
        with torch.cuda.stream(copy_stream):
            dev_q[0].copy_(host_q, non_blocking=True)
            ready[0].record(copy_stream)
        for i in range(steps):
            slot = i & 1
            main_stream.wait_event(ready[slot])
            if i >= 2:
                main_stream.wait_event(landed[slot])        # the slot's previous output has left the device
            decode_into(slot)
            done[slot].record(main_stream)
            with torch.cuda.stream(copy_stream):
                if i + 1 < steps:
                    dev_q[slot ^ 1].copy_(host_q, non_blocking=True)
                    ready[slot ^ 1].record(copy_stream)
                copy_stream.wait_event(done[slot])
                host_out[slot].copy_(dev_out[slot], non_blocking=True)
                landed[slot].record(copy_stream)
            if i >= 1:
                landed[slot ^ 1].synchronize()              # the host reads the previous step's output
        landed[(steps - 1) & 1].synchronize()

    def timed(fn):
        fn(3)
        barrier()
        t0 = time.perf_counter()
        fn(args.steps)
        barrier()
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
        worst = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        return float(worst.item())

    e2e_blocking_ms = timed(e2e_blocking)
    e2e_ms = timed(e2e_pipelined)
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9

    extra = {}
    if gather_check is not None:
        extra["gather_checked"] = True
        extra["gather_check"] = gather_check
        extra["gather"] = gather_kind
        extra["decode_status"] = cache.decode_status()
    if rank == 0 and world == 1 and not args.skip_extras:
        del gathered
        other = _lib.DEQUANT_FUSED if args.flavour == "per_op" else _lib.DEQUANT_PER_OP
        for _ in range(3):
            dart.decode_attention(q3, cache, out=out, flavour=other)
        torch.cuda.synchronize(device)
        start_evt.record()
        for _ in range(args.steps):
            dart.decode_attention(q3, cache, out=out, flavour=other)
        stop_evt.record()
        torch.cuda.synchronize(device)
        other_ms = start_evt.elapsed_time(stop_evt) / args.steps
        other_gbs = local_bytes / (other_ms * 1e-3) / 1e9
        if args.flavour == "per_op":
            extra["unrounded_fp32_variant"] = {
                "value": other_gbs, "unit": "GB/s", "us_per_launch": other_ms * 1e3, "frac": other_gbs / peak,
                "note": "flavour DEQUANT_FUSED: code*scale+zero kept in fp32 like the reference's Triton attention "
                        "kernels (checked against outputs of those kernels recorded on a B200); reported beside "
                        "the headline because the headline follows the reference's page-streamed attention"}
        else:
            extra["per_op_variant"] = {"value": other_gbs, "unit": "GB/s", "us_per_launch": other_ms * 1e3,
                                       "frac": other_gbs / peak}
        del cache
        torch.cuda.empty_cache()
        extra["reference_gpu"] = reference_gpu_decode(wl, device, args.steps)
        torch.cuda.empty_cache()
        if GEOM == HEADLINE:
            extra["other_geometries"] = other_geometry_decode(device, args.steps, peak)
            extra["decode_step_graph"] = [decode_step_graph(device, 32, 8192), decode_step_graph(device, 8, 1024)]
        extra["append"] = append_microbench(device, steps=3, warmup=1)
        cpu = CpuDecode(wl["ctx"], wl["seed"], rows=1)
        step_s = cpu.time_steps(3, 1)
        extra["cpu_baseline"] = {
            "value": cpu.bytes / step_s / 1e9, "unit": "GB/s", "cores": cpu.cores, "kind": cpu.kind,
            "sample": f"{cpu.rows} of {wl['batch']} batch rows at full context, 3 timed steps of {step_s:.2f} s; "
                      f"{cpu.what}; building the sample's cache took {cpu.append_s:.1f} s (untimed)"}
    if rank == 0:
        line = {
            "metric": "fused_decode_attention_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "us_per_step": ms_per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, wl, world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_unit": "bytes per launch (ncu, config 3 capture scaled by algorithmic bytes)",
                         "peak_kind": peak_kind, "kernel": "decode attention call (all its kernels)",
                         "us_per_launch": kernel_ms * 1e3, "per_gpu_gbs": achieved},
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(q3.numel() * 2), "d2h_bytes_per_step": int(out.numel() * 2),
                    "arrangement": "copies on a second stream, two buffers: every step's query copy, decode call"
                                   " and output copy are inside the timed region; the host reads a step's output"
                                   " while the next step computes",
                    "blocking_ms_per_step": e2e_blocking_ms,
                    "blocking_value": total_bytes / (e2e_blocking_ms * 1e-3) / 1e9},
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
                                 metadata_dtype=torch.float16)
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

    def run(measure: bool, graph_decode: bool = False):
        cache = DartHFCache(cfg, max_tokens=prompt_len + new_tokens + 128, graph_decode=graph_decode)
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
    # the same run with every layer's generation step (cache update + attention) replayed from a CUDA graph
    graph_ms, graph_launches, graph_cache = run(False, graph_decode=True)
    graph_status = max(graph_cache.layer_for_attention(i).decode_status() for i in (0, config.num_hidden_layers - 1))
    del graph_cache
    torch.cuda.empty_cache()
    # and with the whole generation step (all layers, the model's own modules included) as ONE CUDA graph
    from dartkv_b200.integrations import DartGraphedDecoder

    def run_graphed():
        cache = DartHFCache(cfg, max_tokens=prompt_len + new_tokens + 128)
        with torch.no_grad():
            logits = model(prompt, past_key_values=cache, use_cache=True).logits[:, -1]
            token = logits.argmax(-1, keepdim=True)
            decoder = DartGraphedDecoder(model, cache)
            for _ in range(3):           # host-planned first step, warm-up, capture
                token = decoder.step(token).argmax(-1, keepdim=True)
            torch.cuda.synchronize(device)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(new_tokens - 3):
                token = decoder.step(token).argmax(-1, keepdim=True)
            t1.record()
            torch.cuda.synchronize(device)
        status = max(cache.layer_for_attention(i).decode_status() for i in (0, config.num_hidden_layers - 1))
        return t0.elapsed_time(t1) / (new_tokens - 3), status, decoder.graph is not None

    step_ms, step_status, captured = run_graphed()
    torch.cuda.empty_cache()
    reference_gpu = reference_qwen3_decode(config, prompt, device, min(new_tokens, 16))
    line = {
        "metric": "qwen3_8b_arch_decode_tokens_per_s", "value": batch * new_tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": new_tokens, "warmup": 1, "ms_per_step": ms / new_tokens, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config4", "model": "Qwen3-8B architecture, random-init bf16 weights (std 0.02)",
                   "batch": batch, "prompt": prompt_len, "new_tokens": new_tokens,
                   "cache": "2-bit + 0.25 promotion, page 128, groups 128/64, 32 sinks, local 1, value local 128, fp16 metadata (the setting of the reference's benchmark script)"},
        "attention_share_of_step": hot_ms / ms, "hot_path_ms_per_step": hot_ms / new_tokens,
        "graph_decode": {"value": batch * new_tokens / (graph_ms * 1e-3), "unit": "tokens/s",
                         "ms_per_step": graph_ms / new_tokens, "decode_status": graph_status,
                         "what": "DartHFCache(graph_decode=True): from the third generated token on, every layer "
                                 "replays one CUDA graph holding the device-planned append and the decode attention"},
        "graph_step": {"value": batch / (step_ms * 1e-3), "unit": "tokens/s", "ms_per_step": step_ms,
                       "decode_status": step_status, "captured": captured,
                       "what": "DartGraphedDecoder: the model's whole forward for one new token (36 layers, their "
                               "device-planned cache appends and decode attention) replayed from one CUDA graph"},
        "reference_gpu": reference_gpu,
        "compression_ratio": cache.compression_ratio, "gpu_launches": int(launches), "clocks": clocks.summary(),
        "e2e": {"value": batch * new_tokens / (ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0, "note": "token ids stay on the device between steps"},
    }
    print(json.dumps(line), flush=True)


def reference_qwen3_decode(config, prompt, device, new_tokens: int) -> dict:
    """The same model and prompt through the reference's own DartHFCache and dart-engine hook (Triton kernels) on this
    GPU, for a few tokens: the GPU baseline of the Qwen3 decode figure."""

    dart_ref = reference_package()
    if dart_ref is None:
        return {"unavailable": "no install of the reference under oracle/_ref"}
    try:
        from transformers import Qwen3ForCausalLM

        from oracle.ref_compat import patch_reference_integrations

        patch_reference_integrations(dart_ref)
        from dart.integrations import DartHFCache as RefCache
        from dart.integrations import attach_dart_fused_attention as ref_attach

        torch.manual_seed(3)
        torch.set_default_dtype(torch.bfloat16)
        with torch.device(device):
            model = Qwen3ForCausalLM(config)
        torch.set_default_dtype(torch.float32)
        model = ref_attach(model.eval())
        cfg = dart_ref.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128,
                                         value_group_size=64, sink_tokens=32, hold_partial_pages=True, local_tokens=1,
                                         value_local_tokens=128, metadata_dtype=torch.float16)
        cache = RefCache(cfg)
        with torch.no_grad():
            logits = model(prompt, past_key_values=cache, use_cache=True).logits[:, -1]
            token = logits.argmax(-1, keepdim=True)
            for _ in range(2):   # Triton compiles on the first decode steps
                token = model(token, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(new_tokens):
                token = model(token, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
            t1.record()
            torch.cuda.synchronize(device)
        ms = t0.elapsed_time(t1)
        del model, cache
        torch.cuda.empty_cache()
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    return {"value": prompt.shape[0] * new_tokens / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms / new_tokens,
            "steps": new_tokens, "what": "the reference's DartHFCache + dart-engine hook (Triton page kernels) on this GPU, "
                                         "same architecture, weights seed, prompt and cache configuration"}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=sorted(WORKLOADS) + ["config4"], default="config5")
    parser.add_argument("--skip-extras", action="store_true", help="skip the append microbench and the CPU baseline")
    parser.add_argument("--flavour", choices=("per_op", "fp32", "fused"), default="per_op",
                        help="dequantization arithmetic of the timed decode call (default: the pinned per-op rounding; "
                             "fp32 runs the general tensor-core kernel that also serves 4/8-bit pages)")
    parser.add_argument("--bits", type=int, choices=(2, 4, 8), default=0, help="code width off the headline geometry")
    parser.add_argument("--promote", type=float, default=None, help="promoted key channel ratio off the headline geometry")
    parser.add_argument("--value-group", type=int, choices=(16, 32, 64, 128), default=0,
                        help="value group size off the headline geometry")
    parser.add_argument("--metadata", choices=("bf16", "fp16"), default="bf16",
                        help="dtype of scales and zero points (fp16 beside the bf16 cache: general tensor-core kernel)")
    parser.add_argument("--gather", choices=("peer", "nccl"), default="peer",
                        help="multi-GPU output gather: peer stores from the decode kernels (default) or NCCL")
    parser.add_argument("--batch", type=int, default=0, help="override the workload's batch (e.g. one rank's share)")
    parser.add_argument("--context", type=int, default=0, help="override the workload's context length")
    args = parser.parse_args()
    if args.bits:
        GEOM["bits"] = args.bits
    if args.promote is not None:
        GEOM["promote_ratio"] = args.promote
    if args.value_group:
        GEOM["value_group"] = args.value_group
    if args.metadata == "fp16":
        GEOM["metadata"] = "fp16"
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
