#!/usr/bin/env python
"""Benchmark of the cache-view decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

A step is one pass of the view-decode path of one attention layer over one batch of requests:
rotate-and-store of the new keys/values, the split-K walk over every request's view, the merge.
The workload is the shared-prefix decode configuration: per GPU 64 requests that all read one
shared 8192-token block plus a private 2048-token block each (Hq16 / Hkv2 / head_dim 256, bf16,
page size 16, page tables drawn from a random permutation of pool pages).

One JSON line is printed by rank 0:
  value      tokens/s with inputs and plan tables resident in HBM: the step is replayed from a CUDA
             graph in rounds of exactly ``--steps`` replays between two CUDA events; ms_per_step is the
             median round (max over ranks), enough rounds are timed to cover at least 100 ms
  e2e        tokens/s through the public API with HOST buffers: per step the pinned q/k/v rows go
             host->device, the step is planned (SharedCacheAttention.prepare), run, the output rows
             come back device->host and every write block grows by its token
  roofline   compulsory KV bytes / measured duration of the streaming kernel, against the measured
             HBM copy bandwidth of this pool's B200s
  cpu_baseline  the CPU oracle (port of the reference path) timed on this box's host cores; its
             output rows are also what the replayed step's rows are compared with (parity_checked)
  side       (1 GPU) the other configurations, briefly: view prefill, GDN decode step, GDN chunked
             prefill, block merge -- each with its own roofline and CPU baseline
With ``--impl reference`` the CPU oracle alone is timed on the same workload (rank 0 only).
``--workload prefill|gdn_step|gdn_prefill|block_merge`` prints one of the side lines alone.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "view_attn_decode_tokens_per_s"
UNIT = "tokens/s"
REQUESTS = 64
SHARED_LEN = 8192
PRIVATE_LEN = 2048
PAGE_SIZE = 16
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0
MIN_TIMED_MS = 100.0        # the rounds of the headline measurement cover at least this long
MIN_ROUNDS = 50
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the kernels of the default step, from the
# committed ncu summary profiles/view_decode_config2_step_traffic.md (same command as this bench with
# --kernel-only).  Only valid for the default workload; any other size reports traffic null.
NCU_STEP_TRAFFIC = {"view_decode_stream_kernel": 270_370_000, "view_dense_tc_kernel": 17_434_000}
SIDE_WORKLOADS = ("prefill", "gdn_step", "gdn_prefill", "block_merge")


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "config2 shared-prefix view decode: per GPU 64 requests x [shared 8192 | private 2048] "
                    "tokens, Hq16/Hkv2/D256, page 16, one attention layer",
        "requests_per_gpu": REQUESTS,
        "global_requests": REQUESTS * n_gpus,
        "parallelism": f"request-sharded x{n_gpus} (no data-path collective)",
        "l2": "inputs larger than L2 (285 MB of KV per step vs 126 MB L2)",
        "step": "store_kv + view_decode (streaming pass || dense tiles of the shared block, merge), "
                "plan resident, replayed from a CUDA graph",
        "e2e_step": "H2D q/k/v + plan_writes + prepare() + forward() + D2H out + append_token, one layer",
    }


def load_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm": float(p["hbm_gbs"]), "tflops": float(p["bf16_tflops"]),
                "tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "kind": "measured"}
    except Exception:
        return {"hbm": FALLBACK_HBM_GBS, "tflops": FALLBACK_TFLOPS, "tflops_sustained": 1400.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: the fields of
    ``nvidia-smi --query-gpu=clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.*`` read
    through NVML inside this process.  (Spawning nvidia-smi every 100 ms from the timed process
    re-initialises NVML on every sample and holds driver locks that the step's own launches and
    copies need: a host-bound step ran up to twice as long under it.)  Falls back to the
    nvidia-smi command line when the NVML binding is missing."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    _nvml = None      # (module, {cuda index: handle}) once initialised; False when unavailable

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    @classmethod
    def _handle(cls, gpu: int):
        if cls._nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                cls._nvml = (pynvml, {})
            except Exception:
                cls._nvml = False
        if not cls._nvml:
            return None, None
        nv, handles = cls._nvml
        if gpu not in handles:
            try:
                uuid = getattr(torch.cuda.get_device_properties(gpu), "uuid", None)
                handles[gpu] = (nv.nvmlDeviceGetHandleByUUID(f"GPU-{uuid}".encode()) if uuid is not None
                                else nv.nvmlDeviceGetHandleByIndex(gpu))
            except Exception:
                try:
                    handles[gpu] = nv.nvmlDeviceGetHandleByIndex(gpu)
                except Exception:
                    handles[gpu] = None
        return nv, handles[gpu]

    def _sample_nvml(self, nv, h) -> None:
        sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        try:
            watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
        except Exception:
            watts = float("nan")
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        r = int(get(h))
        bits = [getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)]
        self.samples.append([str(self.gpu), str(sm), str(mx), f"{watts:.1f}", hex(r)] +
                            ["Active" if r & b else "Not Active" for b in bits])

    def _sample_smi(self) -> None:
        out = subprocess.run(
            ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
             "-i", str(self.gpu)], capture_output=True, text=True, timeout=5).stdout.strip()
        if out:
            self.samples.append([c.strip() for c in out.split(",")])

    def _run(self):
        nv, h = self._handle(self.gpu)
        while not self._stop.is_set():
            try:
                if h is not None:
                    self._sample_nvml(nv, h)
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.05 if h is not None else 0.2)

    def __enter__(self):
        self._handle(self.gpu)     # NVML start-up happens before the timed region, not inside it
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.samples:
            try:
                sm.append(float(row[1]))
                mx.append(float(row[2]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, row[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvml" if self._nvml else "nvidia-smi"}


# ------------------------------------------------------------------------------------------------
# CPU legs (the only places that run oracle/)
def cpu_decode_step(case, repeats: int):
    """Time the CPU oracle on one full step (store + attention over all views); returns the median
    seconds and the step's output rows."""
    from oracle import view_oracle as vo

    pending, slots, positions = case.plan_writes()
    Hkv, D = case.num_kv_heads, case.head_dim
    times, out = [], None
    for _ in range(repeats + 1):
        k_pool, v_pool = case.k_pool, case.v_pool
        t0 = time.perf_counter()
        vo.store_kv(k_pool, v_pool, case.k_new.view(-1, Hkv, D), case.v_new.view(-1, Hkv, D),
                    positions.long(), slots.long(), case.cos_sin)
        out = vo.view_decode(case.q, k_pool, v_pool, case.group, pending, slots.tolist(), case.cos_sin,
                             case.num_q_heads)
        times.append(time.perf_counter() - t0)
    return statistics.median(times[1:] or times), out   # the first pass also warms the caches


def run_reference(args, rank: int) -> None:
    """The reference arm: the CPU port of the path on all host cores, same workload and metric.
    The host processes one 64-request shard per step whatever ``--gpus`` says: its throughput does
    not depend on how many GPUs the other arm uses."""
    if rank != 0:
        return
    import benchcases as wl

    torch.set_num_threads(os.cpu_count() or 1)
    case = wl.config2_decode(page_size=PAGE_SIZE, requests=REQUESTS, shared_len=SHARED_LEN,
                             private_len=PRIVATE_LEN)
    t0 = time.perf_counter()
    cpu_decode_step(case, 0)
    est = time.perf_counter() - t0
    # the run stays within a few minutes: fewer steps only if the host is far slower than expected
    budget = 150.0
    warmup = max(1, min(args.warmup, int(budget * 0.2 / est) or 1))
    steps = max(1, min(args.steps, int(budget * 0.8 / est) or 1))
    for _ in range(warmup - 1):            # the sizing pass above was the first warm-up step
        cpu_decode_step(case, 0)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_decode_step(case, 0)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    value = REQUESTS / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"one 64-request shard per step, {steps} timed steps (mean), torch CPU fp32; "
                                   "the host's throughput does not grow with the number of GPUs"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def time_graph(fn, iters: int, device) -> float:
    """Milliseconds per call of ``fn`` replayed from a CUDA graph (events on the replay stream)."""
    side = torch.cuda.Stream(device=device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def time_plain(fn, iters: int) -> float:
    """Median milliseconds per call of ``fn`` (for calls far longer than a launch): three untimed calls
    (first-use allocations, the caching allocator's pool), then every call timed by its own pair of
    CUDA events."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(max(iters, 5)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def timed_cpu(fn, repeats: int = 1) -> float:
    """Median wall seconds of ``fn`` after one warm-up call."""
    fn()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


# ------------------------------------------------------------------------------------------------
# Side workloads: the other rows of the scope table
def side_prefill(device, iters, peaks, with_cpu, requests=16):
    """Config 3: batched view-conditioned prefill (tensor bound)."""
    import benchcases as wl

    case = wl.config3_prefill(requests=requests)
    dp = wl.DevicePrefill(case, device)
    batch = dp.plan()
    ms = time_graph(lambda: dp.forward(batch), iters, device)
    dp.attn.check_status()
    achieved = case.flops() / ms / 1e9
    rows = sum(r["num_new"] for r in case.requests)
    res = {"metric": "view_prefill_tflops", "value": achieved, "unit": "TFLOP/s", "ms": ms,
           "tokens_per_s": rows / (ms * 1e-3),
           "config": {"workload": f"config3 view-conditioned prefill: {requests} requests x 512 new tokens, 2-6 "
                                  "context blocks of 1K-8K tokens, Hq32/Hkv8/D128, page 16, one layer",
                      "engine": dp.attn.dense_engine},
           "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                        "frac": achieved / peaks["tflops"], "peak_kind": f"{peaks['kind']} burst (kernel timed alone)",
                        "frac_of_sustained": achieved / peaks["tflops_sustained"], "traffic": None,
                        "algorithmic_flops": case.flops()}}
    if with_cpu:
        from oracle import view_oracle as vo

        one = wl.config3_prefill(requests=1)
        Hkv, D = one.num_kv_heads, one.head_dim
        k_pool, v_pool = one.k_pool.clone(), one.v_pool.clone()
        vo.store_kv(k_pool, v_pool, one.k_new.view(-1, Hkv, D), one.v_new.view(-1, Hkv, D),
                    one.positions.long(), one.out_loc.long(), one.cos_sin)
        sec = timed_cpu(lambda: vo.view_prefill(one.q, k_pool, v_pool, one.specs(), one.cos_sin, one.num_q_heads))
        res["cpu_baseline"] = {"value": one.flops() / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                               "kind": "port", "sample": "the first of the 16 requests (512 new tokens), one timed pass"}
    return res


def side_block_merge(device, iters, peaks, with_cpu):
    """Block merge: copy of two 8192-token blocks into a fresh block, right-hand keys re-rotated."""
    import benchcases as wl
    from async_llm_b200 import BlockOps, MHAKVCache, PageAllocator, SharedCacheAttention

    layers, Hkv, D, P, T = 24, 2, 256, PAGE_SIZE, 8192
    pages = 4 * T // P + 8
    pool = MHAKVCache(Hkv, layers, D, pages, P, torch.bfloat16, device)
    pool._buf.normal_()
    attn = SharedCacheAttention(pool, wl.cos_sin_table(D, 32768, 1e7).to(device), 16, Hkv, D, P,
                                torch.bfloat16, device)
    alloc = PageAllocator(pages, P, device)
    ops = BlockOps(pool, alloc, attn, P, device)
    left, right = ops.create_block(), ops.create_block()
    for b in (left, right):
        b.page_starts = alloc.alloc_pages(T // P).tolist()
        b.num_tokens = T
    src = torch.cat((left.token_slots_tensor(), right.token_slots_tensor()))
    dst = (alloc.alloc_pages(2 * T // P).to(torch.int32).unsqueeze(1)
           + torch.arange(P, dtype=torch.int32, device=device)).reshape(-1)
    alloc.free_pages(dst[::P].contiguous())
    kern_ms = time_graph(lambda: ops._copy_slots(src, dst, T, T), iters, device)

    def merge_and_free():
        ops.free_block(ops.merge_blocks(left, right))

    ms = time_plain(merge_and_free, max(2, iters // 2))
    attn.check_status()
    algo = 2 * T * layers * 2 * Hkv * D * 2 * 2      # tokens x layers x (K, V) rows, read + write
    achieved = algo / kern_ms / 1e6
    res = {"metric": "block_merge_gbs", "value": achieved, "unit": "GB/s", "ms": kern_ms,
           "config": {"workload": "merge of two 8192-token blocks into a fresh block: 24 layers, Hkv2/D256, page 16, "
                                  "right-hand keys rotated by 8192 positions; value = the copy kernel alone",
                      "merge_blocks_ms": ms},
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm"], "peak_kind": peaks["kind"], "traffic": None,
                        "algorithmic_bytes": algo}}
    if with_cpu:
        # the reference's per-layer gather / scatter (session.py:489-528) on the K rows of two layers
        kc = torch.randn(2, pages * P, Hkv, D).to(torch.bfloat16)
        s64, d64 = src.cpu().long(), dst.cpu().long()

        def two_layers():
            for layer in range(2):
                kc[layer].index_copy_(0, d64, kc[layer].index_select(0, s64))

        sec = timed_cpu(two_layers, 3)
        res["cpu_baseline"] = {"value": 2 * (2 * T) * Hkv * D * 2 * 2 / sec / 1e9, "unit": "GB/s",
                               "cores": torch.get_num_threads(), "kind": "port",
                               "sample": "K rows of 2 of the 24 layers, index_select + index_copy_, no rotation"}
    del pool
    return res


def _gdn_object(device, state_dtype=torch.float32):
    from async_llm_b200.view_gdn import SharedCacheGDN

    Hk, Hv, dk, dv = 16, 32, 128, 128
    ar = SharedCacheGDN(num_heads=Hv, head_k_dim=dk, head_v_dim=dv, conv_dim=2 * Hk * dk + Hv * dv,
                        conv_kernel=4, device=device, num_k_heads=Hk, state_dtype=state_dtype)
    return ar, Hk, Hv, dk, dv


def side_gdn_step(device, iters, peaks, with_cpu):
    """Config 4b: fused GDN decode step, 128 workers, chain [shared, private] (HBM bound)."""
    import benchcases as wl
    from async_llm_b200.blocks import CacheBlock

    ar, Hk, Hv, dk, dv = _gdn_object(device)
    W = 128
    shared = CacheBlock(device, PAGE_SIZE)
    shared.linear_affine[0] = wl.gdn_random_summary(Hv, dk, dv, 1, device)
    privs = []
    for w in range(W):
        b = CacheBlock(device, PAGE_SIZE)
        b.linear_affine[0] = wl.gdn_random_summary(Hv, dk, dv, 10 + w, device)
        privs.append(b)
    chains = [[shared, b] for b in privs]
    ar.set_context(chains, privs)
    ar.prepare_decode(1, torch.bfloat16)
    toks = wl.gdn_tokens(W, Hk, Hv, dk, dv, 4000)
    q, k, v, g, beta = (t.to(device) for t in toks)
    ms = time_graph(lambda: ar.decode_step(0, q, k, v, g, beta), iters, device)
    ar.finish_decode(False)
    algo = W * Hv * (dk * dk + dv * dk) * 4 * 2   # read + write of the write block's A_hat, B_hat
    achieved = algo / ms / 1e6
    res = {"metric": "gdn_step_gbs", "value": achieved, "unit": "GB/s", "ms": ms, "tokens_per_s": W / (ms * 1e-3),
           "config": {"workload": "config4b GDN decode step: 128 workers, chain [shared, private], Hk16/Hv32, "
                                  "dk=dv=128, fp32 summaries, one layer"},
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm"], "peak_kind": peaks["kind"], "traffic": None,
                        "algorithmic_bytes": algo}}
    # the same step over bf16-stored summaries (the reference's optional state_dtype): half the bytes
    ar16 = _gdn_object(device, torch.bfloat16)[0]
    for b in [shared] + privs:
        b.linear_affine[1] = tuple(t.to(torch.bfloat16) for t in b.linear_affine[0])
    ar16.set_context(chains, privs)
    ar16.prepare_decode(2, torch.bfloat16)
    ms16 = time_graph(lambda: ar16.decode_step(1, q, k, v, g, beta), iters, device)
    ar16.finish_decode(False)
    res["bf16_summaries"] = {"ms": ms16, "tokens_per_s": W / (ms16 * 1e-3), "achieved": algo / 2 / ms16 / 1e6, "unit": "GB/s",
                             "frac": algo / 2 / ms16 / 1e6 / peaks["hbm"], "algorithmic_bytes": algo // 2}
    if with_cpu:
        from oracle import gdn_oracle as go

        n = 16   # workers of the sample
        pairs = lambda b: (b.linear_affine[0][0].cpu(), b.linear_affine[0][1].cpu())
        cq, ck, cv, cg, cb = (t[:n] for t in toks)
        rep = lambda x: x.repeat_interleave(Hv // Hk, dim=1)
        chains_cpu = [[pairs(shared), pairs(privs[w])] for w in range(n)]
        targets_cpu = [pairs(privs[w]) for w in range(n)]
        sec = timed_cpu(lambda: go.decode_step(chains_cpu, targets_cpu, rep(cq), rep(ck), cv, cg, cb))
        res["cpu_baseline"] = {"value": algo * n / W / sec / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
                               "kind": "port", "tokens_per_s": n / sec,
                               "sample": "16 of the 128 workers: compose + one recurrent token + summary update"}
    return res


def side_gdn_prefill(device, iters, peaks, with_cpu):
    """Config 4a: chunked GDN prefill, 8 requests x 4 blocks of 2048 tokens written in order."""
    import benchcases as wl
    from async_llm_b200.blocks import CacheBlock

    ar, Hk, Hv, dk, dv = _gdn_object(device)
    R, T, NB = 8, 2048, 4
    toks = [tuple(t.to(device) for t in wl.gdn_tokens(R * T, Hk, Hv, dk, dv, 4100 + j)) for j in range(NB)]

    def four_blocks():
        # every request writes NB blocks in order; block j starts from the fold of blocks < j
        written = [[] for _ in range(R)]
        for j in range(NB):
            new = [CacheBlock(device, PAGE_SIZE) for _ in range(R)]
            ar.set_context([written[r] + [new[r]] for r in range(R)], new, prefill_segments=[T] * R)
            ar.prepare_prefill(1, torch.bfloat16, R * T)
            ar.prefill_scan(0, *toks[j])
            ar.finish_prefill(True)
            for r in range(R):
                written[r].append(new[r])

    ms = time_plain(four_blocks, max(2, iters // 4))
    tokens = R * T * NB
    chunked = ar.prefill_engine != "scan"
    # Per 64-token chunk and value head.  Pre-pass, computed ONCE for the three parts of the joint
    # state [S | A_hat | B_hat]: K K^T and Q K^T (64x64x128 each), W = T K' and U = T V' (64x128x64
    # each) plus the triangular inverse.  State pass, once per PART: W X (64x128x128) and
    # K^T Vnew (128x128x64); Q X (64x128x128) and P Vnew (64x128x64) for part 0 only.
    mm = lambda m, n, k: 2.0 * m * n * k
    pre = 2 * mm(64, 64, 128) + 2 * mm(64, 128, 64) + mm(64, 64, 64)
    state = 3 * (mm(64, 128, 128) + mm(128, 128, 64)) + mm(64, 128, 128) + mm(64, 128, 64)
    chunk_flops = (pre + state) / 64           # per token and head
    scan_flops = 3 * 3 * 2.0 * 128 * 128       # three parts x (decay, k^T S, rank-1) per token and head
    flops = tokens * Hv * (chunk_flops if chunked else scan_flops)
    achieved_tf = flops / ms / 1e9
    # q, k (16 heads), v, out (32 heads) bf16 per token + g, beta fp32: read once, out written once;
    # the scratch of the pre-pass (1.16 KB per token and head, written then read by three parts) and
    # the summaries come on top of this compulsory figure
    algo_bytes = tokens * ((2 * Hk * dk + 2 * Hv * dv) * 2 + 2 * Hv * 4)
    res = {"metric": "gdn_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "ms": ms,
           "config": {"workload": "config4a GDN prefill: 8 requests x 4 blocks of 2048 tokens written in order "
                                  "(block j starts from the fold of the earlier blocks' summaries), Hk16/Hv32, "
                                  "dk=dv=128, one layer; joint [S | A_hat | B_hat] pass; host planning between the "
                                  "blocks is inside the timed region", "engine": ar.prefill_engine},
           "roofline": {"bound": "tensor" if chunked else "fp32 fma", "achieved": achieved_tf, "unit": "TFLOP/s",
                        "peak": peaks["tflops"] if chunked else None,
                        "frac": achieved_tf / peaks["tflops"] if chunked else None, "peak_kind": peaks["kind"],
                        "algorithmic_flops": flops, "traffic": None,
                        "bytes": {"algorithmic_bytes": algo_bytes, "achieved_gbs": algo_bytes / ms / 1e6,
                                  "frac_of_hbm": algo_bytes / ms / 1e6 / peaks["hbm"]},
                        "note": "a chain of 32 dependent chunks per (block, request, head): neither bound is approached"}}
    if with_cpu:
        from oracle import gdn_oracle as go

        cq, ck, cv, cg, cb = (t[:T].cpu() for t in toks[0])
        rep = lambda x: x.repeat_interleave(Hv // Hk, dim=1)
        sec = timed_cpu(lambda: go.chunk_delta_rule(rep(cq)[None], rep(ck)[None], cv[None], cg[None], cb[None]))
        res["cpu_baseline"] = {"value": T / sec, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": "one request x one 2048-token block, the S scan only (no summary parts)"}
    return res


def run_hybrid(device, steps: int, warmup: int, peaks, rank: int, world: int, per_gpu: int = 32,
               profile_one_step: bool = False) -> dict:
    """Config 5: the random-init hybrid decoder ([GDN, GDN, GDN, attention] x 8) decoding over cache
    views, requests sharded over the GPUs.  Every rank takes part; returns the line on every rank
    (rank 0 prints it).  A step = partition of the global request list, write planning, attention +
    GDN planning into the captured tables, one replay of the captured forward, publish, append."""
    import torch.distributed as dist

    from async_llm_b200 import AsyncContext, CacheBlock
    from async_llm_b200.sharding import BlockReplicator, partition_contexts
    from hybrid_decoder import HybridConfig, HybridDecoder, HybridSession, synth_requests

    cfg = HybridConfig()
    P = cfg.page_size
    spec = synth_requests(per_gpu * world, seed=5000)
    shared_len = spec["shared_len"]
    cpu = torch.device("cpu")
    # host-only descriptors of every request of the job, for the partitioner (all ranks agree on them)
    shared_desc = CacheBlock(cpu, P)
    shared_desc.num_tokens = shared_len
    descs = []
    for lens in spec["private"]:
        blocks = []
        for n in lens:
            b = CacheBlock(cpu, P)
            b.num_tokens = n
            blocks.append(b)
        descs.append(AsyncContext(cache_view=[shared_desc] + blocks, output_block=blocks[-1]))
    part = partition_contexts(descs, world)
    sticky = {id(descs[i].output_block): g for g, shard in enumerate(part.shards) for i in shard}
    mine = part.shards[rank]
    max_workers = max(len(s) for s in part.shards)
    total_steps = steps + warmup + 4
    tokens_mine = sum(sum(spec["private"][i]) for i in mine)
    pages = (shared_len + tokens_mine) // P + 4 * len(mine) + len(mine) * (total_steps // P + 2) + max_workers + 64

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_init = time.perf_counter()
    model = HybridDecoder(cfg, device, seed=0)        # the same weights on every rank (replicated)
    sess = HybridSession(model, pages, max_workers, depth=4, max_seq_len=shared_len + 3 * 4096 + total_steps,
                         dense_fraction=0.25)
    gen = torch.Generator(device=device).manual_seed(7000 + rank)
    # the shared block is written on rank 0 and published once into every other GPU's own pages
    publish = {"bytes": 0, "ms": None}
    if world > 1:
        shared = sess.new_block(shared_len, gen) if rank == 0 else CacheBlock(device, P)
        rep = BlockReplicator(sess.kv_cache, sess.page_allocator)
        barrier()
        t0 = time.perf_counter()
        rep.publish(shared, src=0, gdn_layers=range(cfg.num_linear_layers))
        barrier()
        t = torch.tensor([rep.bytes_sent], dtype=torch.int64, device=device)
        dist.all_reduce(t)
        publish = {"bytes": int(t.item()), "ms": max_over_ranks((time.perf_counter() - t0) * 1e3),
                   "note": "shared 16K block: K/V rows of the 8 attention layers + summaries and conv windows of the "
                           "24 GDN layers, broadcast once from rank 0 (NCCL), host bookkeeping included"}
    else:
        shared = sess.new_block(shared_len, gen)
    contexts = {}
    for i in mine:
        blocks = [sess.new_block(n, gen) for n in spec["private"][i]]
        contexts[i] = AsyncContext(cache_view=[shared] + blocks, output_block=blocks[-1])
    sess.capture()
    torch.cuda.synchronize()
    init_s = time.perf_counter() - t_init

    def step(k: int):
        # the batch former: every rank deals the job's requests (pinned to the GPU holding their pages)
        shards = partition_contexts(descs, world, sticky).shards[rank]
        ctxs = [contexts[i] for i in shards]
        sess.run_step(ctxs, [(11 * k + i) % cfg.vocab for i in shards])
        for d in descs:
            d.output_block.num_tokens += 1

    # (the first steps after the capture also grow the caching allocator's pool of summary slabs --
    # every step hands each write block fresh A_hat / B_hat tensors, 3.2 GB at 32 requests -- and a
    # cudaMalloc synchronises the device: the warm-up has to reach the steady state of that pool)
    for k in range(warmup):
        step(k)
    barrier()
    if profile_one_step:
        # one step between cudaProfilerStart / Stop, for `ncu --profile-from-start off`
        torch.cuda.profiler.start()
        step(warmup)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return {"kernel_only": True, "workload": "hybrid"}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device.index or 0) as clocks:
        e0.record()
        for k in range(steps):
            step(warmup + k)
        e1.record()
        barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / steps)
    sess.sc_attn.check_status()
    # the captured forward alone (no host work between replays)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(5):
        sess.graph.replay()
    g1.record()
    g1.synchronize()
    graph_ms = max_over_ranks(g0.elapsed_time(g1) / 5)
    # per-layer-type time of one eager forward (same kernels, launched one by one)
    timers = {}
    shards = partition_contexts(descs, world, sticky).shards[rank]
    sess.forward_eager([contexts[i] for i in shards], [1] * len(shards))       # untimed: first-use allocations
    sess.forward_eager([contexts[i] for i in shards], [1] * len(shards), timers)
    torch.cuda.synchronize()
    by_type = {kind: sum(a.elapsed_time(b) for a, b in pairs) for kind, pairs in timers.items()}
    # bytes one step must move on this GPU
    kv_row = 2 * cfg.num_kv_heads * cfg.head_dim * 2
    private_tokens = sum(sum(spec["private"][i]) for i in mine)
    attn_bytes = cfg.num_attn_layers * (shared_len + private_tokens) * kv_row
    gdn_bytes = cfg.num_linear_layers * len(mine) * cfg.gdn_v_heads * 2 * (cfg.gdn_head_dim ** 2) * 4 * 2
    weight_bytes = cfg.param_bytes() - cfg.vocab * cfg.hidden * 2     # the embedding table is only indexed
    step_bytes = weight_bytes + attn_bytes + gdn_bytes
    n_req = per_gpu * world
    return {"metric": "hybrid_decode_tokens_per_s", "value": n_req / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "ms": ms_step, "higher_is_better": True,
            "scaling": "weak", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config5 hybrid decoder: 32 layers [GDN, GDN, GDN, attention] x 8, hidden 4096, attention "
                                   "Hq16/Hkv4/D256 (gated, q/k norm), GDN Hk16/Hv32/128, SwiGLU 12288, vocab 151936, random "
                                   f"bf16 weights replicated; {per_gpu} requests per GPU, views = shared 16384-token block + "
                                   "1-3 private blocks of 512-4096 tokens, page 16",
                       "global_requests": n_req, "requests_on_this_rank": len(mine), "captured_batch": max_workers,
                       "parallelism": f"request-sharded x{world} by partition_contexts (sticky), no collective in a step"},
            "graph_replay_ms": graph_ms, "host_ms_per_step": ms_step - graph_ms,
            "eager_ms_by_layer_type": by_type,
            "roofline": {"bound": "hbm", "achieved": step_bytes / graph_ms / 1e6, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": step_bytes / graph_ms / 1e6 / peaks["hbm"], "peak_kind": peaks["kind"], "traffic": None,
                         "algorithmic_bytes": step_bytes,
                         "bytes": {"weights": weight_bytes, "attention_kv": attn_bytes, "gdn_summaries": gdn_bytes},
                         "note": "bytes one captured forward must move on this GPU / its replay time; the replicated "
                                 "weight stream dominates at 32 requests per GPU"},
            "publish": publish, "init_s": init_s, "clocks": clocks.summary()}


SIDE_FUNCS = {"prefill": side_prefill, "gdn_step": side_gdn_step, "gdn_prefill": side_gdn_prefill,
              "block_merge": side_block_merge}


def run_side(name, device, iters, peaks, with_cpu) -> dict:
    torch.set_num_threads(os.cpu_count() or 1)
    res = SIDE_FUNCS[name](device, iters, peaks, with_cpu)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="skip the side workloads of the default run")
    ap.add_argument("--no-hybrid", action="store_true", help="skip the full-model (config 5) side line")
    # smaller cases of the same kernels for profiler captures (not a bench line)
    ap.add_argument("--requests", type=int, default=REQUESTS)
    ap.add_argument("--shared-len", type=int, default=SHARED_LEN)
    ap.add_argument("--private-len", type=int, default=PRIVATE_LEN)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hkv", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--workload", default="decode", choices=["decode", "hybrid", *SIDE_WORKLOADS],
                    help="decode = the headline metric (with the side workloads embedded); the others "
                         "print that side line alone")
    ap.add_argument("--kernel-only", action="store_true",
                    help="run warmup+steps steps of the workload and exit (for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the cache-view path has no CPU fallback")
    import torch.distributed as dist

    from async_llm_b200 import _lib
    import benchcases as wl

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    default_workload = (args.requests, args.shared_len, args.private_len, args.hq, args.hkv, args.head_dim,
                        args.page_size) == (REQUESTS, SHARED_LEN, PRIVATE_LEN, 16, 2, 256, PAGE_SIZE)

    if args.workload == "hybrid":
        line = run_hybrid(device, max(3, args.steps), args.warmup, peaks, rank, world,
                          profile_one_step=args.kernel_only)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    if args.workload != "decode":
        if rank == 0:
            if args.kernel_only:
                # a few launches of the side workload's kernels, nothing else (profiler captures)
                run_side(args.workload, device, max(3, args.steps), peaks, False)
                print(json.dumps({"kernel_only": True, "workload": args.workload}))
            else:
                line = run_side(args.workload, device, max(3, min(args.steps, 20)), peaks, not args.no_cpu_baseline)
                line["ms_per_step"] = line["ms"]
                line.update({"n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                             "side_workload": args.workload})
                print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    K, Wm = args.steps, args.warmup
    e2e_steps = min(max(K, 20), 50)
    # pages the end-to-end steps consume: every write block grows by one token per step
    e2e_pages = args.requests * (-(-(2 * e2e_steps + 8) // args.page_size) + 1)
    n_shared = -(-args.shared_len // args.page_size) + 8 if world > 1 else 0
    # every rank holds its own shard of requests; the shared block is replicated per GPU
    case = wl.config2_decode(page_size=args.page_size, seed=2000 + rank, requests=args.requests,
                             shared_len=args.shared_len, private_len=args.private_len,
                             num_q_heads=args.hq, num_kv_heads=args.hkv, head_dim=args.head_dim,
                             spare_pages=e2e_pages + n_shared)
    dv = wl.DeviceView(case, device)
    publish = {"bytes": 0, "ms": None}
    if world > 1:
        # the shared block is written on rank 0 and published once into every other GPU's own
        # pool pages (NCCL broadcast over NVLink); decode steps then run without any collective
        from async_llm_b200 import CacheBlock, PageAllocator
        from async_llm_b200.sharding import BlockReplicator

        alloc = PageAllocator(0, args.page_size, device)
        alloc.free_pages(torch.tensor(case.free_pages[-n_shared:], dtype=torch.int32))
        case.free_pages = case.free_pages[:-n_shared]
        rep = BlockReplicator(dv.pool, alloc)
        shared = case.blocks["shared"] if rank == 0 else CacheBlock(torch.device("cpu"), args.page_size)
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        rep.publish(shared, src=0)
        p1.record()
        barrier()
        case.blocks["shared"] = shared
        t = torch.tensor([rep.bytes_sent], dtype=torch.int64, device=device)
        dist.all_reduce(t)
        publish = {"bytes": int(t.item()), "ms": max_over_ranks(p0.elapsed_time(p1)),
                   "note": "one-time broadcast of the shared block's rows of every layer into each receiver's own "
                           "pages (host bookkeeping included); outside the timed steps"}
    batch = dv.plan()
    plan = batch.attn_metadata.plan
    if args.kernel_only:
        for _ in range(Wm + K):
            dv.decode(batch)
        torch.cuda.synchronize()
        dv.attn.check_status()
        print(json.dumps({"kernel_only": True, "requests": args.requests,
                          "kv_bytes_compulsory": case.kv_bytes_compulsory(),
                          "kv_bytes_logical": case.kv_bytes_logical()}))
        return

    # ---- resident-input throughput: the whole step (store + stream + merge) captured once in a
    # CUDA graph and replayed, so host launch latency is not part of the device-side number
    for _ in range(3):
        dv.decode(batch)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=device)
    step_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        dv.decode(batch)
        torch.cuda.synchronize()
        with torch.cuda.graph(step_graph, stream=side):
            graph_out = dv.decode(batch)
    for _ in range(Wm):
        step_graph.replay()
    torch.cuda.synchronize()
    # one untimed round sizes the measurement: rounds of exactly K replays until >= MIN_TIMED_MS
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        step_graph.replay()
    e1.record()
    e1.synchronize()
    est_round_ms = max_over_ranks(e0.elapsed_time(e1))
    rounds = int(max(MIN_ROUNDS, -(-MIN_TIMED_MS // max(est_round_ms, 1e-3))))
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(rounds)]
    barrier()
    with ClockSampler(local_rank) as clocks:
        t_wall = time.perf_counter()
        for a, b in events:
            a.record()
            for _ in range(K):
                step_graph.replay()
            b.record()
        barrier()
        timed_wall_ms = (time.perf_counter() - t_wall) * 1e3
        # keep the sampler alive for a few samples even when the region is short
        t_end = time.time() + 0.5
        while time.time() < t_end:
            step_graph.replay()
        torch.cuda.synchronize()
    per_step = sorted(a.elapsed_time(b) / K for a, b in events)
    ms_step = max_over_ranks(statistics.median(per_step))
    ms_step_min = max_over_ranks(per_step[0])
    dv.attn.check_status()
    gpu_rows = graph_out.float().cpu()

    # ---- the dominant kernel alone (streaming pass), for the roofline: one launch captured in
    # a graph, replayed back to back between two events on the launching stream
    import ctypes as C

    from async_llm_b200.kvpool import pool_struct

    pool = pool_struct(dv.pool, 0, case.num_q_heads, dv.attn._cos_sin, dv.attn.rotary_dim)
    out = torch.empty(args.requests, case.num_q_heads * case.head_dim, dtype=torch.bfloat16, device=device)

    def phase_ms(mask: int, iters: int) -> float:
        plan.struct.phase_mask = mask
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                rc = _lib.lib().va_view_decode(C.byref(pool), C.byref(plan.struct), dv.q.data_ptr(),
                                               dv.q.stride(0), out.data_ptr(), out.stride(0),
                                               dv.attn._partial_o.data_ptr(), dv.attn._partial_ml.data_ptr(),
                                               dv.attn.status().data_ptr(), _lib.stream_ptr())
        plan.struct.phase_mask = 0
        _lib.check(rc, "va_view_decode")
        for _ in range(10):
            g.replay()
        torch.cuda.synchronize()
        # five rounds of back-to-back replays, each between two events; the median round
        per_round = max(iters // 5, 1)
        rounds_ms = []
        for _ in range(5):
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            for _ in range(per_round):
                g.replay()
            k1.record()
            k1.synchronize()
            rounds_ms.append(k0.elapsed_time(k1) / per_round)
        return statistics.median(rounds_ms)

    n_kern = 200
    kern_avg_ms = phase_ms(2 | 4, n_kern)                 # streaming pass only
    dense_ms = phase_ms(1 | 2, n_kern) if plan.groups is not None else None   # shared-block tiles only
    # where the rest of the step goes: the same call with passes left out (no store kernel in these)
    phases = {"stream": kern_avg_ms, "dense_tiles": dense_ms, "stream_and_merge": phase_ms(4, n_kern),
              "stream_tiles_merge": phase_ms(0, n_kern)}
    # bytes the streaming kernel itself must read: the (row, kv head) key ranges in its items
    stream_keys = int(plan.host["items"][:, 2].sum()) if plan.num_items else 0
    algo_bytes = stream_keys * 2 * case.head_dim * 2
    step_bytes = case.kv_bytes_compulsory()
    achieved = algo_bytes / (kern_avg_ms * 1e-3) / 1e9

    # ---- CPU baseline of the same step, and the parity check of the replayed rows against it
    cpu_baseline, parity = None, {"parity_checked": False}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        sec, want = cpu_decode_step(case, 3)
        cpu_baseline = {"value": args.requests / sec, "unit": UNIT, "cores": torch.get_num_threads(),
                        "kind": "port",
                        "sample": f"full step: {args.requests} requests, 3 timed repeats (median), torch CPU fp32"}
        diff = (gpu_rows - want.float()).abs()
        parity = {"parity_checked": True, "parity_max_abs": float(diff.max()), "parity_mean_abs": float(diff.mean()),
                  "parity_ok": bool(diff.max() <= 2e-2 and diff.mean() <= 1e-3),
                  "parity_note": "rows of the graph-replayed step vs the CPU oracle's rows of the same step; "
                                 "bounds 2e-2 max-abs, 1e-3 mean-abs"}
        if not parity["parity_ok"]:
            raise SystemExit(f"bench: the replayed step does not match the oracle: {parity}")
    del graph_out

    # ---- end to end through the public API with host buffers; every step appends its token
    q_h, k_h, v_h = (t.cpu().pin_memory() for t in (case.q, case.k_new, case.v_new))
    out_h = torch.empty(args.requests, case.num_q_heads * case.head_dim, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (q_h, k_h, v_h))
    d2h = out_h.numel() * out_h.element_size()
    from types import SimpleNamespace

    group = case.group   # the serving engine keeps its worker group between steps
    targets = [case.blocks[n] for n in case.writes]
    snapshot = [(b, b.num_tokens, list(b.page_starts)) for b in targets], list(case.free_pages)

    def advance(pending):
        """Book-keeping after a step: every write block now holds its new token."""
        used = 0
        for b in targets:
            page = pending[id(b)]
            b.append_token(page)
            used += page is not None
        if used:
            del case.free_pages[:used]

    def e2e_step():
        pending, slots, positions = case.plan_writes()
        qd = q_h.to(device, non_blocking=True)
        kd = k_h.to(device, non_blocking=True)
        vd = v_h.to(device, non_blocking=True)
        meta = dv.attn.prepare(group, pending, slots)
        b = SimpleNamespace(attn_metadata=meta, positions=positions.to(device, non_blocking=True),
                            out_loc=slots.to(device, non_blocking=True), mrope_positions=None)
        o = dv.attn.forward(qd, kd, vd, 0, b)
        out_h.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
        advance(pending)
        return meta

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        meta = e2e_step()
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) / e2e_steps * 1e3)
    plan_bytes = meta.plan.host_blob.numel() * 4 + 2 * args.requests * 4

    # The same work with the host planning of step n+1 issued while the GPU runs step n (the plan
    # depends on block lengths, not on the sampled tokens): every step still copies its inputs in,
    # plans, runs, copies its result out and appends; only the wait for the result moves behind the
    # next step's planning.  Reported beside the strict number, not instead of it.
    def plan_step():
        pending, slots, positions = case.plan_writes()
        return dv.attn.prepare(group, pending, slots), positions, slots, pending

    def launch_step(planned):
        meta, positions, slots, _ = planned
        qd = q_h.to(device, non_blocking=True)
        kd = k_h.to(device, non_blocking=True)
        vd = v_h.to(device, non_blocking=True)
        b = SimpleNamespace(attn_metadata=meta, positions=positions.to(device, non_blocking=True),
                            out_loc=slots.to(device, non_blocking=True), mrope_positions=None)
        out_h.copy_(dv.attn.forward(qd, kd, vd, 0, b), non_blocking=True)

    def pipelined(n):
        planned = plan_step()
        for _ in range(n):
            launch_step(planned)
            advance(planned[3])          # the lengths after this step are known before its result is
            planned = plan_step()
            torch.cuda.synchronize()

    pipelined(3)
    barrier()
    t0 = time.perf_counter()
    pipelined(e2e_steps)
    barrier()
    e2e_pipelined_ms = max_over_ranks((time.perf_counter() - t0) / e2e_steps * 1e3)
    dv.attn.check_status()
    for b, n, pages in snapshot[0]:       # leave the case as it was
        b.num_tokens, b.page_starts = n, pages
    case.free_pages = snapshot[1]

    if rank == 0:
        launches_per_step = 4 if plan.groups is not None else 3
        stream_traffic = NCU_STEP_TRAFFIC["view_decode_stream_kernel"] if default_workload else None
        line = {
            "metric": METRIC, "value": args.requests * world / (ms_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": Wm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(world),
            "timing": {"rounds": rounds, "steps_per_round": K, "ms_per_step_median": ms_step,
                       "ms_per_step_min": ms_step_min, "timed_region_ms": timed_wall_ms,
                       "note": "every round is exactly --steps graph replays between two CUDA events; median round, "
                               "max over ranks"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm"], "traffic": stream_traffic,
                         "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel "
                                         "variant inside the step (ncu summary in profiles/)",
                         "peak_kind": peaks["kind"],
                         "kernel": f"view_decode_stream_kernel<{args.head_dim}>", "kernel_ms": kern_avg_ms,
                         "algorithmic_bytes": algo_bytes,
                         "stream_sms": plan.struct.num_lanes // (4 if args.head_dim == 256 else 6),
                         "dense_tiles_ms": dense_ms, "phases_ms": phases,
                         "dense_tiles_traffic": NCU_STEP_TRAFFIC["view_dense_tc_kernel"] if default_workload else None,
                         "step_compulsory_bytes": step_bytes,
                         "step_frac": step_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm"]},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": args.requests * world / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d + plan_bytes, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "steps": e2e_steps,
                    "pipelined_value": args.requests * world / (e2e_pipelined_ms * 1e-3),
                    "pipelined_note": "host planning of step n+1 overlapped with the GPU work of step n"},
            "gpu_launches": launches_per_step * K * rounds,
            "clocks": clocks.summary(),
            "publish": publish,
        }
        line.update(parity)
    sides = {}
    del dv
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_side:
        for name in SIDE_WORKLOADS:
            try:
                sides[name] = run_side(name, device, 10, peaks, not args.no_cpu_baseline)
            except Exception as exc:   # noqa: BLE001 -- a side line never costs the headline
                sides[name] = {"error": f"{type(exc).__name__}: {exc}"}
    if not args.no_side and not args.no_hybrid and default_workload:
        # the full-model workload runs on every rank (requests sharded over the GPUs)
        try:
            sides["hybrid"] = run_hybrid(device, 10, 8, peaks, rank, world)
        except Exception as exc:   # noqa: BLE001
            sides["hybrid"] = {"error": f"{type(exc).__name__}: {exc}"}
            if world > 1:
                raise
    if rank == 0:
        if sides:
            line["side"] = sides
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
