"""Random-init hybrid decoder over cache views: the full-model decode workload of the benchmark.

32 layers in the pattern [GDN, GDN, GDN, full attention] x 8 (the reference's Qwen3.5-style hybrid,
minisgl/models/qwen3_5_attn.py and qwen3_5_delta.py): hidden 4096; attention Hq16 / Hkv4 / head_dim 256
with a 2x-wide q projection (query + sigmoid output gate) and per-head q/k RMSNorm; Gated DeltaNet
layers Hk16 / Hv32 / dk = dv = 128 with a conv window of 4; SwiGLU MLP 12288; vocabulary 151 936; bf16.
Weights are random (there are no checkpoints here), replicated on every GPU.

Projections, MLP GEMMs and the LM head are plain torch GEMMs; the residual add + RMSNorm between
sub-layers and the SwiGLU gate are ``decoder_glue.add_rmsnorm`` / ``silu_mul``; the attention
layers are ``GatedAttentionLayer`` (q/k norm, ``SharedCacheAttention.forward``, output gate) and the
GDN layers ``GatedDeltaNetLayer.forward_ar_decode``
-- the kernels of this package -- and the whole decode forward is captured ONCE in a CUDA graph
through ``SharedGraphIO`` and replayed every step after the host has re-planned the step's views
into the fixed-capacity tables.

``HybridSession`` is the minimum of a serving session around it: pool, allocator, blocks, one decode
step (write planning, attention + GDN planning, staging, replay, publish, append).  Requests are
sharded over GPUs by ``partition_contexts``; the shared block is published once with
``BlockReplicator``.  This file is benchmark / test infrastructure, not part of the package.
"""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from async_llm_b200 import AsyncContext, CacheBlock, MHAKVCache, PageAllocator, SharedCacheAttention, WorkerGroup
from async_llm_b200.attn_layer import GatedAttentionLayer
from async_llm_b200.decoder_glue import add_rmsnorm, silu_mul
from async_llm_b200.gdn_layer import GatedDeltaNetLayer
from async_llm_b200.graph_io import SharedGraphIO
from async_llm_b200.session_plan import plan_decode_writes
from async_llm_b200.view_gdn import SharedCacheGDN


@dataclass
class HybridConfig:
    num_layers: int = 32
    attn_every: int = 4            # layer i is full attention when (i + 1) % attn_every == 0
    hidden: int = 4096
    num_q_heads: int = 16
    num_kv_heads: int = 4
    head_dim: int = 256
    gdn_k_heads: int = 16
    gdn_v_heads: int = 32
    gdn_head_dim: int = 128
    conv_kernel: int = 4
    intermediate: int = 12288
    vocab: int = 151936
    eps: float = 1e-6
    rope_base: float = 1e7
    max_pos: int = 65536
    page_size: int = 16

    @staticmethod
    def small() -> "HybridConfig":
        """A few layers of the same structure for tests."""
        return HybridConfig(num_layers=4, hidden=256, num_q_heads=8, num_kv_heads=2, head_dim=128, gdn_k_heads=2,
                            gdn_v_heads=4, intermediate=512, vocab=1024, max_pos=8192)

    def is_attn(self, i: int) -> bool:
        return (i + 1) % self.attn_every == 0

    @property
    def num_attn_layers(self) -> int:
        return sum(self.is_attn(i) for i in range(self.num_layers))

    @property
    def num_linear_layers(self) -> int:
        return self.num_layers - self.num_attn_layers

    @property
    def conv_dim(self) -> int:
        return 2 * self.gdn_k_heads * self.gdn_head_dim + self.gdn_v_heads * self.gdn_head_dim

    def param_bytes(self) -> int:
        h, d = self.hidden, self.head_dim
        attn = ((2 * self.num_q_heads + 2 * self.num_kv_heads) * d * h + self.num_q_heads * d * h) * self.num_attn_layers
        vdim = self.gdn_v_heads * self.gdn_head_dim
        gdn = ((self.conv_dim + vdim + 2 * self.gdn_v_heads) * h + h * vdim) * self.num_linear_layers
        mlp = 3 * self.intermediate * h * self.num_layers
        return 2 * (attn + gdn + mlp + 2 * self.vocab * h)


def cos_sin_table(rotary_dim: int, max_pos: int, base: float, device) -> torch.Tensor:
    inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float, device=device) / rotary_dim))
    ang = torch.arange(max_pos, dtype=torch.float, device=device)[:, None] * inv[None, :]
    return torch.cat((ang.cos(), ang.sin()), dim=-1)


class HybridDecoder:
    """The layer stack; ``forward`` is one decode step over ``rows`` tokens (one per worker)."""

    def __init__(self, cfg: HybridConfig, device, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        g = torch.Generator(device=self.device).manual_seed(seed)
        h = cfg.hidden

        def w(rows, cols):
            return (torch.randn(rows, cols, generator=g, device=self.device, dtype=torch.float32)
                    * cols ** -0.5).to(torch.bfloat16)

        ones = lambda n: torch.ones(n, device=self.device, dtype=torch.bfloat16)
        self.embed = (torch.randn(cfg.vocab, h, generator=g, device=self.device, dtype=torch.float32) * 0.5).to(torch.bfloat16)
        self.layers: List[SimpleNamespace] = []
        kv_idx = lin_idx = 0
        d, hq, hkv, dv = cfg.head_dim, cfg.num_q_heads, cfg.num_kv_heads, cfg.gdn_head_dim
        for i in range(cfg.num_layers):
            layer = SimpleNamespace(norm_in=ones(h), norm_post=ones(h), w_gate_up=w(2 * cfg.intermediate, h),
                                    w_down=w(h, cfg.intermediate))
            if cfg.is_attn(i):
                layer.kind, layer.kv_idx = "attn", kv_idx
                kv_idx += 1
                layer.attn = GatedAttentionLayer(
                    layer.kv_idx, hq, hkv, d, w((2 * hq + 2 * hkv) * d, h), w(h, hq * d),   # [q | gate per head, k, v]
                    torch.randn(d, generator=g, device=self.device) * 0.1,                 # (1 + weight) form
                    torch.randn(d, generator=g, device=self.device) * 0.1, cfg.eps)
            else:
                layer.kind = "gdn"
                vdim, kdim = cfg.gdn_v_heads * dv, cfg.gdn_k_heads * dv
                layer.gdn = GatedDeltaNetLayer(
                    lin_idx, cfg.gdn_k_heads, cfg.gdn_v_heads, dv, dv, w(2 * kdim + vdim, h), w(vdim, h),
                    w(cfg.gdn_v_heads, h), w(cfg.gdn_v_heads, h), w(h, vdim),
                    (torch.randn(cfg.conv_dim, 1, cfg.conv_kernel, generator=g, device=self.device) * 0.5).to(torch.bfloat16),
                    torch.randn(cfg.gdn_v_heads, generator=g, device=self.device) * 0.5,
                    torch.randn(cfg.gdn_v_heads, generator=g, device=self.device),
                    torch.rand(dv, generator=g, device=self.device) + 0.5, cfg.eps)
                lin_idx += 1
            self.layers.append(layer)
        self.norm_final = ones(h)
        self.lm_head = w(cfg.vocab, h)

    def forward(self, input_ids: torch.Tensor, batch, ar, timers: Optional[Dict[str, list]] = None) -> torch.Tensor:
        """Logits ``[rows, vocab]`` (fp32) of one decode step; ``batch`` carries the attention plan,
        ``ar`` the prepared GDN seam object.  ``timers`` (eager runs only) collects one CUDA-event pair
        per section under "attn" / "gdn" / "mlp" / "head"."""
        def timed(kind, fn):
            if timers is None:
                return fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            timers.setdefault(kind, []).append((e0, e1))
            return out

        eps = self.cfg.eps
        h = self.embed[input_ids.long()]      # the residual stream, updated in place by the fused add + norm
        x = add_rmsnorm(h, None, self.layers[0].norm_in, eps)
        for i, layer in enumerate(self.layers):
            if layer.kind == "attn":
                a = timed("attn", lambda: layer.attn.forward(x, batch))
            else:
                a = timed("gdn", lambda: layer.gdn.forward_ar_decode(x, ar))
            x = add_rmsnorm(h, a, layer.norm_post, eps)
            m = timed("mlp", lambda: F.linear(silu_mul(F.linear(x, layer.w_gate_up)), layer.w_down))
            x = add_rmsnorm(h, m, self.layers[i + 1].norm_in if i + 1 < len(self.layers) else self.norm_final, eps)
        return timed("head", lambda: F.linear(x, self.lm_head).float())


class HybridSession:
    """Pool, allocator, seam objects and the decode step around a ``HybridDecoder``."""

    def __init__(self, model: HybridDecoder, num_pages: int, max_workers: int, depth: int, max_seq_len: int,
                 dense_fraction: float = 0.0):
        cfg = model.cfg
        self.model, self.cfg, self.device = model, cfg, model.device
        self.page_size = cfg.page_size
        self.dtype = torch.bfloat16
        self.num_linear_layers = cfg.num_linear_layers
        self.vocab_size = cfg.vocab
        self.kv_cache = MHAKVCache(cfg.num_kv_heads, cfg.num_attn_layers, cfg.head_dim, num_pages + 1, cfg.page_size,
                                   torch.bfloat16, self.device)
        self.page_allocator = PageAllocator(num_pages, cfg.page_size, self.device)
        self.sc_attn = SharedCacheAttention(self.kv_cache, cos_sin_table(cfg.head_dim, cfg.max_pos, cfg.rope_base, self.device),
                                            cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim, cfg.page_size,
                                            torch.bfloat16, self.device)
        self.sc_gdn = SharedCacheGDN(num_heads=cfg.gdn_v_heads, head_k_dim=cfg.gdn_head_dim, head_v_dim=cfg.gdn_head_dim,
                                     conv_dim=cfg.conv_dim, conv_kernel=cfg.conv_kernel, device=self.device,
                                     num_k_heads=cfg.gdn_k_heads)
        self.max_workers, self.depth = max_workers, depth
        self.io = SharedGraphIO(self, depth, dense_fraction=dense_fraction)
        self.io.init_capture_graph(max_seq_len, [max_workers])
        self._dummy_host = self.io.dummy_slots.cpu().numpy().astype("int32")
        # stable inputs of the captured forward
        self.input_ids = torch.zeros(max_workers, dtype=torch.int32, device=self.device)
        self.positions = torch.zeros(max_workers, dtype=torch.int32, device=self.device)
        self.out_loc = torch.zeros(max_workers, dtype=torch.int32, device=self.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self._batch = None
        self._stage_host = torch.zeros(3, max_workers, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self._stage_event = torch.cuda.Event() if self.device.type == "cuda" else None

    # ------------------------------------------------------------------ blocks with synthetic contents
    def new_block(self, num_tokens: int, gen: Optional[torch.Generator] = None, with_state: bool = True) -> CacheBlock:
        """A block of ``num_tokens`` tokens with random K/V rows in its pages and a plausible GDN
        summary / conv window per linear layer (no prefill is run for the benchmark)."""
        cfg = self.cfg
        b = CacheBlock(self.device, cfg.page_size)
        if num_tokens:
            pages = self.page_allocator.alloc_pages(-(-num_tokens // cfg.page_size))
            b.grow_pages(pages, num_tokens)
            slots = b.token_slots_tensor().long()
            for layer in range(cfg.num_attn_layers):
                for cache in (self.kv_cache.k_cache(layer), self.kv_cache.v_cache(layer)):
                    flat = cache.view(-1, cfg.num_kv_heads, cfg.head_dim)
                    flat[slots] = (torch.randn(num_tokens, cfg.num_kv_heads, cfg.head_dim, device=self.device,
                                               generator=gen) * 0.5).to(torch.bfloat16)
        if with_state and num_tokens:
            H, d = cfg.gdn_v_heads, cfg.gdn_head_dim
            eye = torch.eye(d, device=self.device)
            for layer in range(cfg.num_linear_layers):
                A = (0.9 * eye + 0.01 * torch.randn(1, H, d, d, device=self.device, generator=gen)).contiguous()
                Bm = 0.05 * torch.randn(1, H, d, d, device=self.device, generator=gen)
                b.linear_affine[layer] = (A, Bm)
                b.linear_conv_state[layer] = torch.randn(cfg.conv_dim, cfg.conv_kernel, device=self.device,
                                                         generator=gen).to(torch.bfloat16)
        return b

    # ------------------------------------------------------------------ capture
    def _make_batch(self, size: int, meta=None):
        return SimpleNamespace(size=size, padded_size=self.max_workers, is_prefill=False, is_decode=True,
                               input_ids=self.input_ids, positions=self.positions, out_loc=self.out_loc,
                               mrope_positions=None, attn_metadata=meta)

    def capture(self) -> None:
        """Capture the decode forward once, on a dummy topology of ``max_workers`` rows."""
        batch = self._make_batch(self.max_workers)
        self.io.prepare_for_capture(batch)
        self.model.forward(self.input_ids, batch, self.sc_gdn)     # warm-up outside the capture
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self.model.forward(self.input_ids, batch, self.sc_gdn)
        self.io.finish_capture(batch)
        self._batch = batch

    # ------------------------------------------------------------------ one decode step
    def plan_step(self, contexts: Sequence[AsyncContext], tokens: Sequence[int]):
        """Host side of a step: write planning, attention and GDN planning into the captured tables,
        staging of the padded inputs."""
        W, bs = len(contexts), self.max_workers
        if W > bs:
            raise ValueError(f"{W} workers exceed the captured batch size {bs}")
        group = WorkerGroup(list(contexts))
        pending, slots, positions = plan_decode_writes(group, self.page_allocator, self.page_size, torch.device("cpu"))
        meta = self.sc_attn.prepare(group, pending, slots, self.io.attention[bs])
        self.sc_gdn.set_context(group.cache_structure, group.write_to)
        self.sc_gdn.prepare_decode(self.num_linear_layers, self.dtype, buffers=self.io.gdn[bs])
        if self._stage_event is not None:
            self._stage_event.synchronize()
        hv = self._stage_host.numpy()
        hv[0, :W], hv[0, W:] = tokens, 0
        hv[1, :W], hv[1, W:] = positions, 0
        hv[2, :W] = slots.numpy()
        hv[2, W:] = self._dummy_host[W:bs]     # padding rows store into their own reserved page
        self.input_ids.copy_(self._stage_host[0], non_blocking=True)
        self.positions.copy_(self._stage_host[1], non_blocking=True)
        self.out_loc.copy_(self._stage_host[2], non_blocking=True)
        if self._stage_event is not None:
            self._stage_event.record()
        batch = self._make_batch(W, meta)
        self.io.prepare_for_replay(batch)
        return group, pending

    def run_step(self, contexts: Sequence[AsyncContext], tokens: Sequence[int]) -> torch.Tensor:
        """Plan, replay the captured forward, publish, append; returns the logits rows of the workers."""
        group, pending = self.plan_step(contexts, tokens)
        self.graph.replay()
        self.sc_gdn.finish_decode(True)
        for ctx in contexts:
            ctx.output_block.append_token(pending[id(ctx.output_block)])
        return self.logits[: len(contexts)]

    def forward_eager(self, contexts: Sequence[AsyncContext], tokens: Sequence[int],
                      timers: Optional[Dict[str, list]] = None) -> torch.Tensor:
        """The same step without graph or fixed-capacity tables (the cross-check of ``run_step``);
        publishes and appends like ``run_step``."""
        group = WorkerGroup(list(contexts))
        pending, slots, positions = plan_decode_writes(group, self.page_allocator, self.page_size, torch.device("cpu"))
        meta = self.sc_attn.prepare(group, pending, slots)
        self.sc_gdn.set_context(group.cache_structure, group.write_to)
        self.sc_gdn.prepare_decode(self.num_linear_layers, self.dtype)
        W = len(contexts)
        batch = SimpleNamespace(size=W, padded_size=W, is_prefill=False, is_decode=True, mrope_positions=None,
                                positions=torch.tensor(positions, dtype=torch.int32, device=self.device),
                                out_loc=slots.to(self.device), attn_metadata=meta)
        ids = torch.tensor(list(tokens), dtype=torch.int32, device=self.device)
        logits = self.model.forward(ids, batch, self.sc_gdn, timers)
        self.sc_gdn.finish_decode(True)
        for ctx in contexts:
            ctx.output_block.append_token(pending[id(ctx.output_block)])
        return logits


def synth_requests(n_requests: int, seed: int, shared_len: int = 16384, min_len: int = 512, max_len: int = 4096):
    """Seeded request shapes of the full-model workload: every request sees the shared block plus 1-3
    private blocks of U[min_len, max_len] tokens (views of 2-4 blocks) and writes its last block."""
    g = torch.Generator().manual_seed(seed)
    reqs = []
    for _ in range(n_requests):
        n_private = int(torch.randint(1, 4, (1,), generator=g))
        reqs.append([int(torch.randint(min_len, max_len + 1, (1,), generator=g)) for _ in range(n_private)])
    return {"shared_len": shared_len, "private": reqs}


__all__ = ["HybridConfig", "HybridDecoder", "HybridSession", "synth_requests", "cos_sin_table"]
