#!/usr/bin/env python
"""Benchmark of the cache-view decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

A step is one pass of the view-decode path of one attention layer over one batch of requests:
rotate-and-store of the new keys/values, the split-K walk over every request's view, the merge.
The workload is the shared-prefix decode configuration: per GPU 64 requests that all read one
shared 8192-token block plus a private 2048-token block each (Hq16 / Hkv2 / head_dim 256, bf16,
page size 16, page tables drawn from a random permutation of pool pages).

One JSON line is printed by rank 0:
  value      tokens/s with inputs and plan tables resident in HBM (CUDA events, max over ranks)
  e2e        tokens/s through the public API with HOST buffers: per step the pinned q/k/v rows go
             host->device, the step is planned (SharedCacheAttention.prepare), run, and the output
             rows come back device->host
  roofline   compulsory KV bytes / measured duration of the streaming kernel, against the measured
             HBM copy bandwidth of this pool's B200s
  cpu_baseline  the CPU oracle (port of the reference path) timed on this box's host cores
With ``--impl reference`` the CPU oracle alone is timed on the same workload (rank 0 only).
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
# dram__bytes_read.sum + dram__bytes_write.sum of the streaming kernel over its algorithmic bytes in the
# committed ncu capture (269.4 MB read + 7.1 MB of split-K partials written for 268.6 MB of K/V)
NCU_TRAFFIC_RATIO = 276.5 / 268.6


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
        "e2e_step": "H2D q/k/v + prepare() + forward() + D2H out, one layer",
    }


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                     "-i", str(self.gpu)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
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
                "samples": len(sm)}


def cpu_step_seconds(case, repeats: int):
    """Time the CPU oracle on one full step (store + attention over all views)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import view_oracle as vo

    pending, slots, positions = case.plan_writes()
    Hkv, D = case.num_kv_heads, case.head_dim
    times = []
    for _ in range(repeats + 1):
        k_pool, v_pool = case.k_pool, case.v_pool
        t0 = time.perf_counter()
        vo.store_kv(k_pool, v_pool, case.k_new.view(-1, Hkv, D), case.v_new.view(-1, Hkv, D),
                    positions.long(), slots.long(), case.cos_sin)
        vo.view_decode(case.q, k_pool, v_pool, case.group, pending, slots.tolist(), case.cos_sin,
                       case.num_q_heads)
        times.append(time.perf_counter() - t0)
    return statistics.median(times[1:] or times)   # the first pass also warms the caches


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    import benchcases as wl

    torch.set_num_threads(os.cpu_count() or 1)
    case = wl.config2_decode(page_size=PAGE_SIZE, requests=REQUESTS, shared_len=SHARED_LEN,
                             private_len=PRIVATE_LEN)
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_step_seconds(case, 0)
    steps = max(1, min(args.steps, 5))
    sec = cpu_step_seconds(case, steps)
    value = REQUESTS / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": "port",
                         "sample": f"full step: 64 requests, {steps} timed repeats (median), torch CPU fp32"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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
    """Milliseconds per call of ``fn`` launched back to back (for calls far longer than a launch)."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def run_side_workload(args, device) -> None:
    """Other rows of the scope table, one JSON line each (not the headline metric):
    view prefill (config 3), GDN decode step (config 4b), GDN prefill scan (config 4a)."""
    import benchcases as wl

    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    tflops = float(peaks.get("bf16_tflops", 1590.0))
    iters = max(3, min(args.steps, 20))
    if args.workload == "prefill":
        case = wl.config3_prefill(requests=args.requests if args.requests != REQUESTS else 16)
        dp = wl.DevicePrefill(case, device)
        batch = dp.plan()
        ms = time_graph(lambda: dp.forward(batch), iters, device)
        dp.attn.check_status()
        achieved = case.flops() / ms / 1e9
        line = {"metric": "view_prefill_tflops", "value": achieved, "unit": "TFLOP/s", "ms_per_step": ms,
                "config": {"workload": "config3 view-conditioned prefill: 16 requests x 512 new tokens, 2-6 context "
                                       "blocks of 1K-8K tokens, Hq32/Hkv8/D128, page 16", "engine": dp.attn.dense_engine},
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": tflops, "unit": "TFLOP/s",
                             "frac": achieved / tflops, "traffic": None, "algorithmic_flops": case.flops()}}
    elif args.workload == "block_merge":
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

        ms = time_plain(merge_and_free, iters)
        attn.check_status()

        def eager_copy():   # the reference's per-layer gather / scatter, without its key rotation
            s64, d64 = src.long(), dst.long()
            for i in range(layers):
                for cache in (pool.k_cache(i), pool.v_cache(i)):
                    flat = cache.reshape(-1, Hkv, D)
                    flat.index_copy_(0, d64, flat.index_select(0, s64))

        eager_ms = time_plain(eager_copy, max(2, iters // 4))
        algo = 2 * T * layers * 2 * Hkv * D * 2 * 2      # tokens x layers x (K, V) rows, read + write
        achieved = algo / kern_ms / 1e6
        line = {"metric": "block_merge_gbs", "value": achieved, "unit": "GB/s", "ms_per_step": kern_ms,
                "config": {"workload": "merge of two 8192-token blocks into a fresh block: 24 layers, Hkv2/D256, page 16, "
                                       "right-hand keys rotated by 8192 positions; value = the copy kernel alone",
                           "merge_blocks_ms": ms, "torch_eager_copy_only_ms": eager_ms},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                             "frac": achieved / hbm, "traffic": None, "algorithmic_bytes": algo}}
    else:
        from async_llm_b200.blocks import CacheBlock
        from async_llm_b200.view_gdn import SharedCacheGDN

        Hk, Hv, dk, dv = 16, 32, 128, 128
        ar = SharedCacheGDN(num_heads=Hv, head_k_dim=dk, head_v_dim=dv, conv_dim=2 * Hk * dk + Hv * dv,
                            conv_kernel=4, device=device, num_k_heads=Hk)
        if args.workload == "gdn_step":
            W = 128
            shared = CacheBlock(device, PAGE_SIZE)
            shared.linear_affine[0] = wl.gdn_random_summary(Hv, dk, dv, 1, device)
            privs = []
            for w in range(W):
                b = CacheBlock(device, PAGE_SIZE)
                b.linear_affine[0] = wl.gdn_random_summary(Hv, dk, dv, 10 + w, device)
                privs.append(b)
            ar.set_context([[shared, b] for b in privs], privs)
            ar.prepare_decode(1, torch.bfloat16)
            q, k, v, g, beta = (t.to(device) for t in wl.gdn_tokens(W, Hk, Hv, dk, dv, 4000))
            ms = time_graph(lambda: ar.decode_step(0, q, k, v, g, beta), iters, device)
            ar.finish_decode(False)
            algo = W * Hv * (dk * dk + dv * dk) * 4 * 2   # read + write of the write block's A_hat, B_hat
            achieved = algo / ms / 1e6
            line = {"metric": "gdn_step_gbs", "value": achieved, "unit": "GB/s", "ms_per_step": ms,
                    "config": {"workload": "config4b GDN decode step: 128 workers, chain [shared, private], Hk16/Hv32, "
                                           "dk=dv=128, fp32 summaries, one layer"},
                    "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                                 "frac": achieved / hbm, "traffic": None, "algorithmic_bytes": algo}}
        else:
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
            chunked = ar.prefill_engine == "chunk"
            # per token, head and part: scan 3 x 128 x 128 x 2 flops; chunk: the UT-transform products
            # (K K^T, Q K^T, W, U, W X, Q X, P Vnew, K^T Vnew) of _chunk_gated_delta_rule
            chunk_flops = 2.0 * (64 * 64 * 128 * 4 + 64 * 128 * 128 * 3 + 64 * 64 * 128) * 3 / 64
            scan_flops = 3 * 2.0 * 128 * 128 * 3
            tensor_peak = tflops
            achieved_tf = tokens * Hv * (chunk_flops if chunked else scan_flops) / ms / 1e9
            line = {"metric": "gdn_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
                    "ms_per_step": ms,
                    "config": {"workload": "config4a GDN prefill: 8 requests x 4 blocks of 2048 tokens written in order "
                                           "(block j starts from the fold of the earlier blocks' summaries), "
                                           "Hk16/Hv32, dk=dv=128, one layer; joint [S | A_hat | B_hat] pass; host "
                                           "planning between the blocks is inside the timed region",
                               "engine": ar.prefill_engine},
                    "roofline": {"bound": "tensor" if chunked else "fp32 fma", "achieved": achieved_tf, "unit": "TFLOP/s",
                                 "peak": tensor_peak if chunked else None,
                                 "frac": achieved_tf / tensor_peak if chunked else None, "traffic": None}}
    line.update({"n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                 "side_workload": args.workload})
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    # smaller cases of the same kernels for profiler captures (not a bench line)
    ap.add_argument("--requests", type=int, default=REQUESTS)
    ap.add_argument("--shared-len", type=int, default=SHARED_LEN)
    ap.add_argument("--private-len", type=int, default=PRIVATE_LEN)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hkv", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "gdn_step", "gdn_prefill", "block_merge"],
                    help="decode = the headline metric; the others print one extra JSON line each")
    ap.add_argument("--kernel-only", action="store_true",
                    help="run warmup+steps decode steps and exit (for ncu captures)")
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

    if args.workload != "decode":
        if rank == 0:
            run_side_workload(args, device)
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

    # every rank holds its own shard of requests; the shared block is replicated per GPU
    spare = -(-args.shared_len // args.page_size) + 8 if world > 1 else 0
    case = wl.config2_decode(page_size=args.page_size, seed=2000 + rank, requests=args.requests,
                             shared_len=args.shared_len, private_len=args.private_len,
                             num_q_heads=args.hq, num_kv_heads=args.hkv, head_dim=args.head_dim,
                             spare_pages=spare)
    dv = wl.DeviceView(case, device)
    replicated_bytes = 0
    if world > 1:
        # the shared block is written on rank 0 and published once into every other GPU's own
        # pool pages (NCCL broadcast over NVLink); decode steps then run without any collective
        from async_llm_b200 import CacheBlock, PageAllocator
        from async_llm_b200.sharding import BlockReplicator

        alloc = PageAllocator(0, args.page_size, device)
        alloc._free = torch.tensor(case.free_pages[len(case.writes):], dtype=torch.int32, device=device)
        case.free_pages = case.free_pages[: len(case.writes)]
        rep = BlockReplicator(dv.pool, alloc)
        shared = case.blocks["shared"] if rank == 0 else CacheBlock(torch.device("cpu"), args.page_size)
        rep.publish(shared, src=0)
        torch.cuda.synchronize()
        case.blocks["shared"] = shared
        t = torch.tensor([rep.bytes_sent], dtype=torch.int64, device=device)
        dist.all_reduce(t)
        replicated_bytes = int(t.item())
    batch = dv.plan()
    plan = batch.attn_metadata.plan
    K, Wm = args.steps, args.warmup
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
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for _ in range(K):
            step_graph.replay()
        e1.record()
        barrier()
        # keep the sampler alive for a few samples even when the region is short
        t_end = time.time() + 0.6
        while time.time() < t_end:
            step_graph.replay()
        torch.cuda.synchronize()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / K)
    dv.attn.check_status()
    del graph_out

    # ---- the dominant kernel alone (streaming pass), for the roofline: one launch captured in
    # a graph, replayed back to back between two events on the launching stream
    import ctypes as C

    from async_llm_b200.kvpool import pool_struct

    pool = pool_struct(dv.pool, 0, case.num_q_heads, dv.attn._cos_sin, dv.attn.rotary_dim)
    out = torch.empty(args.requests, case.num_q_heads * case.head_dim, dtype=torch.bfloat16, device=device)
    plan.struct.phase_mask = 2 | 4  # skip merge and dense tiles: the streaming pass only
    kern_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(kern_graph, stream=side):
            rc = _lib.lib().va_view_decode(C.byref(pool), C.byref(plan.struct), dv.q.data_ptr(),
                                           dv.q.stride(0), out.data_ptr(), out.stride(0),
                                           dv.attn._partial_o.data_ptr(), dv.attn._partial_ml.data_ptr(),
                                           dv.attn.status().data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "va_view_decode")
    plan.struct.phase_mask = 0
    for _ in range(3):
        kern_graph.replay()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_kern = max(10, min(K, 100))
    k0.record()
    for _ in range(n_kern):
        kern_graph.replay()
    k1.record()
    k1.synchronize()
    kern_avg_ms = k0.elapsed_time(k1) / n_kern
    # bytes the streaming kernel itself must read: the (row, kv head) key ranges in its items
    stream_keys = int(plan.host["items"][:, 2].sum()) if plan.num_items else 0
    algo_bytes = stream_keys * 2 * case.head_dim * 2
    step_bytes = case.kv_bytes_compulsory()
    peak, peak_kind = measured_peak()
    achieved = algo_bytes / (kern_avg_ms * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers
    q_h, k_h, v_h = (t.cpu().pin_memory() for t in (case.q, case.k_new, case.v_new))
    out_h = torch.empty(args.requests, case.num_q_heads * case.head_dim, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (q_h, k_h, v_h))
    d2h = out_h.numel() * out_h.element_size()
    from types import SimpleNamespace

    group = case.group   # the serving engine keeps its worker group between steps

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

    e2e_steps = min(K, 50)
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) / e2e_steps * 1e3)

    # The same work with the host planning of step n+1 issued while the GPU runs step n (the plan
    # depends on block lengths, not on the sampled tokens): every step still copies its inputs in,
    # plans, runs and copies its result out; only the wait for the result moves behind the next
    # step's planning.  Reported beside the strict number, not instead of it.
    def plan_step():
        pending, slots, positions = case.plan_writes()
        return dv.attn.prepare(group, pending, slots), positions, slots

    def launch_step(planned):
        meta, positions, slots = planned
        qd = q_h.to(device, non_blocking=True)
        kd = k_h.to(device, non_blocking=True)
        vd = v_h.to(device, non_blocking=True)
        b = SimpleNamespace(attn_metadata=meta, positions=positions.to(device, non_blocking=True),
                            out_loc=slots.to(device, non_blocking=True), mrope_positions=None)
        out_h.copy_(dv.attn.forward(qd, kd, vd, 0, b), non_blocking=True)

    planned = plan_step()
    for _ in range(3):
        launch_step(planned)
        planned = plan_step()
        torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        launch_step(planned)
        planned = plan_step()
        torch.cuda.synchronize()
    barrier()
    e2e_pipelined_ms = max_over_ranks((time.perf_counter() - t0) / e2e_steps * 1e3)
    h2d += plan.host_blob.numel() * 4 + 2 * args.requests * 4

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        sec = cpu_step_seconds(case, 3)
        cpu_baseline = {"value": args.requests / sec, "unit": UNIT, "cores": torch.get_num_threads(),
                        "kind": "port",
                        "sample": "full step: 64 requests, 3 timed repeats (median), torch CPU fp32"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": args.requests * world / (ms_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": Wm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": dict(workload_config(world), replicated_bytes_at_publish=replicated_bytes),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": int(algo_bytes * NCU_TRAFFIC_RATIO),
                         "traffic_note": "dram read+write of one ncu capture of this kernel on the same private "
                                         "blocks (276.5 MB for 268.6 MB of keys and values), scaled by the bytes "
                                         "streamed",
                         "peak_kind": peak_kind,
                         "kernel": f"view_decode_stream_kernel<{args.head_dim}>", "kernel_ms": kern_avg_ms,
                         "algorithmic_bytes": algo_bytes,
                         "stream_sms": plan.struct.num_lanes // (4 if args.head_dim == 256 else 6),
                         "step_compulsory_bytes": step_bytes,
                         "step_frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": args.requests * world / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "pipelined_value": args.requests * world / (e2e_pipelined_ms * 1e-3),
                    "pipelined_note": "host planning of step n+1 overlapped with the GPU work of step n"},
            "gpu_launches": (4 if plan.groups is not None else 3) * K,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
