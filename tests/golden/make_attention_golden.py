"""Generate tests/golden/attention_golden.npz: output rows of the REFERENCE attention path on a GPU.

The reference's attention core is FlashInfer (``BatchDecodeWithPagedKVCacheWrapper`` /
``BatchPrefillWithPagedKVCacheWrapper`` with backend "fa2" and ``merge_states``), which only runs on
a GPU, so this script -- unlike make_golden.py -- has to be run on a machine with one:

    python tests/golden/make_attention_golden.py /path/to/reference/python \
        [--flashinfer-aot DIR] [--out FILE] [--time]

It imports the unmodified ``minisgl.shared_cache`` from the given checkout (nothing is copied),
rebuilds the seeded cases of tests/attention_cases.py with the reference's own ``CacheBlock`` /
``WorkerGroup`` objects, runs ``SharedCacheAttention.prepare`` + ``forward`` (decode) and
``prepare_prefill_batch`` + ``forward`` (prefill) and stores the output rows as bf16 bit patterns,
together with the rotated keys the reference stored into the pool; it also runs the reference's
per-head q/k RMSNorm and sigmoid output gate of the gated attention layer on seeded rows (``layer/...``).

``--flashinfer-aot DIR`` points FlashInfer at prebuilt kernel modules (``DIR/<module>/<module>.so``)
so that nothing is compiled on the GPU machine.  ``--time`` also times the reference decode forward
of the shared-prefix benchmark case (CUDA events) and prints one JSON line.
"""
import argparse
import json
import os
import sys
import time
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
TESTS = os.path.dirname(HERE)
ROOT = os.path.dirname(TESTS)
for p in (ROOT, TESTS):
    if p not in sys.path:
        sys.path.insert(0, p)

MAX_ROWS = 64   # rows kept of a large output (evenly spaced, last row included)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().copy()


class TorchPool:
    """A KV pool behind the reference's BaseKVCachePool accessors whose store is an index_copy_:
    used when the reference's own pool (a JIT-compiled scatter kernel) cannot be built."""

    def __init__(self, k_pool, v_pool, device):
        self._k = [k_pool.to(device)]
        self._v = [v_pool.to(device)]
        self.device, self.dtype, self.num_layers = device, k_pool.dtype, 1

    def k_cache(self, i):
        return self._k[i]

    def v_cache(self, i):
        return self._v[i]

    def store_kv(self, k, v, out_loc, layer_id):
        kf = self._k[layer_id].view(-1, self._k[layer_id].shape[-2] * self._k[layer_id].shape[-1])
        vf = self._v[layer_id].view(kf.shape)
        keep = out_loc >= 0
        kf.index_copy_(0, out_loc[keep].long(), k.reshape(k.shape[0], -1)[keep])
        vf.index_copy_(0, out_loc[keep].long(), v.reshape(v.shape[0], -1)[keep])


def reference_pool(case, device, want_reference_store):
    """The reference's MHAKVCache holding the case's pool, or the torch stand-in."""
    if want_reference_store:
        try:
            from minisgl.distributed import DistributedInfo, set_tp_info
            from minisgl.kvcache.mha_pool import MHAKVCache

            try:
                set_tp_info(0, 1)
            except Exception:
                pass
            pool = MHAKVCache(case.num_kv_heads, 1, case.head_dim, case.num_pages, case.page_size,
                              torch.bfloat16, device)
            pool.k_cache(0).copy_(case.k_pool)
            pool.v_cache(0).copy_(case.v_pool)
            # one dry store into the dummy page proves the JIT kernel builds and runs
            z = torch.zeros(1, case.num_kv_heads * case.head_dim, dtype=torch.bfloat16, device=device)
            pool.store_kv(z, z, torch.tensor([(case.num_pages - 1) * case.page_size], dtype=torch.int32,
                                             device=device), 0)
            torch.cuda.synchronize()
            pool.k_cache(0).copy_(case.k_pool)
            pool.v_cache(0).copy_(case.v_pool)
            return pool, "reference MHAKVCache.store_kv"
        except Exception as exc:   # noqa: BLE001 -- any build / import problem selects the stand-in
            print(f"reference pool unavailable ({type(exc).__name__}: {exc}); using index_copy_ stand-in",
                  flush=True)
    return TorchPool(case.k_pool, case.v_pool, device), "torch index_copy_ stand-in"


def ref_blocks(case, device):
    """The case's blocks as the reference's own CacheBlock objects."""
    from minisgl.shared_cache.shared_block import CacheBlock

    out = {}
    for name, b in case.blocks.items():
        rb = CacheBlock(device, case.page_size)
        rb.page_starts = list(b.page_starts)
        rb.num_tokens = b.num_tokens
        out[name] = rb
    return out


def make_attention(case, pool, device):
    from minisgl.shared_cache.attention import SharedCacheAttention

    return SharedCacheAttention(pool, case.cos_sin.to(device), case.num_q_heads, case.num_kv_heads,
                                case.head_dim, case.page_size, torch.bfloat16, device)


def pick_rows(n):
    if n <= MAX_ROWS:
        return np.arange(n)
    rows = np.unique(np.concatenate((np.linspace(0, n - 1, MAX_ROWS).round().astype(np.int64), [n - 1])))
    return rows


def run_decode(case, device, want_reference_store):
    from minisgl.shared_cache.worker_group import WorkerGroup

    pool, store_kind = reference_pool(case, device, want_reference_store)
    attn = make_attention(case, pool, device)
    blocks = ref_blocks(case, device)
    group = WorkerGroup(cache_structure=[[blocks[n] for n in view] for view in case.views],
                        write_to=[blocks[n] for n in case.writes])
    pending_named, slots, positions = case.plan_writes()
    # plan_writes keys by the case's own block objects: re-key by the reference blocks
    by_id = {id(b): name for name, b in case.blocks.items()}
    pending = {id(blocks[by_id[k]]): v for k, v in pending_named.items()}
    meta = attn.prepare(group, pending, slots.to(device))
    batch = SimpleNamespace(attn_metadata=meta, positions=positions.to(device), out_loc=slots.to(device),
                            mrope_positions=None)
    q, k, v = (t.to(device) for t in (case.q, case.k_new, case.v_new))
    out = attn.forward(q, k, v, 0, batch)
    torch.cuda.synchronize()
    new_keys = pool.k_cache(0).view(-1, case.num_kv_heads * case.head_dim)[slots.to(device).long()]
    return out, new_keys, store_kind, (attn, group, pending, slots, positions, q, k, v)


def run_prefill(case, device, want_reference_store):
    from minisgl.shared_cache.attention import PrefillSpec

    pool, store_kind = reference_pool(case, device, want_reference_store)
    attn = make_attention(case, pool, device)
    blocks = ref_blocks(case, device)
    specs = []
    for req, pages in zip(case.requests, case.self_pages):
        wb = blocks[req["write"]]
        specs.append(PrefillSpec(context=[blocks[n] for n in req["context"]], self_page_starts=pages.to(device),
                                 num_new=req["num_new"], self_prefix_len=wb.num_tokens))
    meta = attn.prepare_prefill_batch(specs)
    batch = SimpleNamespace(attn_metadata=meta, positions=case.positions.to(device),
                            out_loc=case.out_loc.to(device), mrope_positions=None)
    q, k, v = (t.to(device) for t in (case.q, case.k_new, case.v_new))
    out = attn.forward(q, k, v, 0, batch)
    torch.cuda.synchronize()
    return out, store_kind


def time_reference_decode(handles, iters=20):
    """Milliseconds per reference decode forward (store + query copies + FlashInfer + merge) with the
    plan already made, and per prepare() + forward()."""
    attn, group, pending, slots, positions, q, k, v = handles
    device = q.device
    meta = attn.prepare(group, pending, slots.to(device))
    batch = SimpleNamespace(attn_metadata=meta, positions=positions.to(device), out_loc=slots.to(device),
                            mrope_positions=None)
    for _ in range(3):
        attn.forward(q, k, v, 0, batch)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        attn.forward(q, k, v, 0, batch)
    e1.record()
    e1.synchronize()
    fwd_ms = e0.elapsed_time(e1) / iters
    t0 = time.perf_counter()
    for _ in range(iters):
        meta = attn.prepare(group, pending, slots.to(device))
        batch.attn_metadata = meta
        attn.forward(q, k, v, 0, batch)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / iters * 1e3
    return fwd_ms, e2e_ms


def layer_step_inputs():
    """Seeded inputs of the gated attention layer's steps (the tests rebuild exactly these): rows of
    the fused qkv projection ``[n, (2*Hq + 2*Hkv) * D]``, the norm weights and an attention output."""
    out = {}
    for name, (n, hq, hkv, d) in {"d128": (37, 8, 2, 128), "d256": (21, 16, 4, 256)}.items():
        g = torch.Generator().manual_seed(909 + d)
        out[name] = dict(n=n, hq=hq, hkv=hkv, d=d, eps=1e-6,
                         qkv=(torch.randn(n, (2 * hq + 2 * hkv) * d, generator=g) * 1.5).to(torch.bfloat16),
                         q_weight=(torch.randn(d, generator=g) * 0.2).to(torch.bfloat16),
                         k_weight=(torch.randn(d, generator=g) * 0.2).to(torch.bfloat16),
                         o=torch.randn(n, hq * d, generator=g).to(torch.bfloat16))
    return out


def run_layer_steps(device):
    """The reference's per-head q/k RMSNorm (``RMSNorm(..., weight_plus_one=True)``: FlashInfer
    ``gemma_rmsnorm``, minisgl/layers/norm.py:8-22) and ``_sigmoid_output_gate``
    (minisgl/models/qwen3_5_attn.py:21-23) on the seeded rows, as ``Qwen3_5Attention.forward`` applies
    them (:103-114,136)."""
    from minisgl.layers.norm import RMSNorm
    from minisgl.models.qwen3_5_attn import _sigmoid_output_gate

    res = {}
    for name, c in layer_step_inputs().items():
        n, hq, hkv, d = c["n"], c["hq"], c["hkv"], c["d"]
        qkv = c["qkv"].to(device)
        q_gate, k, _ = qkv.split([2 * hq * d, hkv * d, hkv * d], dim=-1)
        q_gate = q_gate.view(n, hq, 2 * d)
        q, gate = q_gate[..., :d].contiguous(), q_gate[..., d:].contiguous()
        k = k.reshape(n, hkv, d)
        qn, kn = RMSNorm(d, c["eps"], weight_plus_one=True), RMSNorm(d, c["eps"], weight_plus_one=True)
        qn.weight, kn.weight = c["q_weight"].to(device), c["k_weight"].to(device)
        res[f"layer/{name}/q"] = bf16_bits(qn.forward(q).reshape(n, hq * d))
        res[f"layer/{name}/k"] = bf16_bits(kn.forward(k.contiguous()).reshape(n, hkv * d))
        res[f"layer/{name}/gated"] = bf16_bits(_sigmoid_output_gate(c["o"].to(device).view(n, hq, d), gate).reshape(n, hq * d))
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("reference_python", help="directory that holds the reference's `minisgl` package")
    ap.add_argument("--flashinfer-aot", default=None)
    ap.add_argument("--out", default=os.path.join(HERE, "attention_golden.npz"))
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--torch-store", action="store_true", help="do not try the reference's JIT store kernel")
    ap.add_argument("--only", default=None, help="comma-separated case names")
    args = ap.parse_args()

    sys.path.insert(0, os.path.abspath(args.reference_python))
    if args.flashinfer_aot:
        import pathlib

        from flashinfer.jit import env as jit_env

        jit_env.FLASHINFER_AOT_DIR = pathlib.Path(os.path.abspath(args.flashinfer_aot))
    import flashinfer

    from attention_cases import DECODE_CASES, PREFILL_CASES

    device = torch.device("cuda:0")
    only = set(args.only.split(",")) if args.only else None
    out = {}
    info = {"flashinfer": flashinfer.__version__, "torch": torch.__version__,
            "gpu": torch.cuda.get_device_name(0), "cases": {}}
    for name, build in DECODE_CASES.items():
        if only and name not in only:
            continue
        case = build()
        rows_out, new_keys, store_kind, handles = run_decode(case, device, not args.torch_store)
        rows = pick_rows(rows_out.shape[0])
        out[f"decode/{name}/rows"] = rows
        out[f"decode/{name}/out"] = bf16_bits(rows_out[torch.from_numpy(rows).to(device)])
        out[f"decode/{name}/new_keys"] = bf16_bits(new_keys)
        info["cases"][f"decode/{name}"] = {"store": store_kind, "rows": int(rows_out.shape[0])}
        print(f"decode/{name}: {tuple(rows_out.shape)} ({store_kind})", flush=True)
        if args.time and name == "config2_full":
            fwd_ms, e2e_ms = time_reference_decode(handles)
            W = rows_out.shape[0]
            line = {"reference_gpu": "SharedCacheAttention.forward (FlashInfer fa2 + torch glue), one layer",
                    "case": name, "forward_ms": fwd_ms, "tokens_per_s": W / (fwd_ms * 1e-3),
                    "prepare_plus_forward_ms": e2e_ms, "e2e_tokens_per_s": W / (e2e_ms * 1e-3),
                    "kv_bytes_compulsory": case.kv_bytes_compulsory(), "kv_bytes_logical": case.kv_bytes_logical(),
                    "logical_gbs": case.kv_bytes_logical() / (fwd_ms * 1e-3) / 1e9}
            info["timing"] = line
            print(json.dumps(line), flush=True)
        del handles
    for name, build in PREFILL_CASES.items():
        if only and name not in only:
            continue
        case = build()
        rows_out, store_kind = run_prefill(case, device, not args.torch_store)
        rows = pick_rows(rows_out.shape[0])
        out[f"prefill/{name}/rows"] = rows
        out[f"prefill/{name}/out"] = bf16_bits(rows_out[torch.from_numpy(rows).to(device)])
        info["cases"][f"prefill/{name}"] = {"store": store_kind, "rows": int(rows_out.shape[0])}
        print(f"prefill/{name}: {tuple(rows_out.shape)} ({store_kind})", flush=True)
    if not only or "layer" in only:
        try:
            out.update(run_layer_steps(device))
            info["layer_steps"] = "reference RMSNorm (flashinfer gemma_rmsnorm) + _sigmoid_output_gate"
            print("layer steps: done", flush=True)
        except Exception as exc:   # noqa: BLE001 -- the norm module may be missing; the rest still counts
            info["layer_steps"] = f"unavailable: {type(exc).__name__}: {exc}"
            print("layer steps unavailable:", info["layer_steps"], flush=True)
    out["info"] = np.frombuffer(json.dumps(info).encode(), dtype=np.uint8)
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, flush=True)


if __name__ == "__main__":
    main()
