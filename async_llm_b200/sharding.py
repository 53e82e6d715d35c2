"""Request sharding of the cache-view path across the GPUs of one node.

The reference runs one GPU (``DistributedInfo(rank=0, size=1)``, minisgl/llm/async_llm.py:99-100)
and forms every decode batch in ``AsyncCacheEngine._run_decode_batch``
(minisgl/scheduler/async_engine.py:307-346).  Decode requests are independent given the blocks of
their views, so the batch former is where the work is split: one process per GPU, weights and
static shared blocks replicated, requests dealt to GPUs, and no collective inside a step.

``partition_contexts``  decides which GPU runs which request.  Requests coupled through a block
                        that is still being written this step (a thinker/writer pair sees the
                        other's current token, minisgl/shared_cache/attention.py:37-40) form one
                        component and stay together; components are bin-packed by the KV bytes
                        they stream.
``BlockReplicator``     copies a block's pages (and GDN summaries) into the other GPUs' own pools
                        when the block is published: one ``broadcast`` per publication over NCCL
                        (NVLink / NVSwitch), never per decode step.  Every GPU keeps its own page
                        list for its replica; kernels only ever read local memory.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .blocks import AsyncContext, CacheBlock


@dataclass
class Partition:
    """``assignment[i]`` is the GPU of request ``i``; ``shards[g]`` lists GPU ``g``'s requests in
    their original order; ``load[g]`` is the KV-token load the packer balanced."""

    assignment: List[int]
    shards: List[List[int]]
    load: List[int]
    components: List[List[int]]


def _find(parent: List[int], i: int) -> int:
    while parent[i] != i:
        parent[i] = parent[parent[i]]
        i = parent[i]
    return i


def partition_contexts(contexts: Sequence[AsyncContext], num_gpus: int,
                       sticky: Optional[Dict[int, int]] = None) -> Partition:
    """Deal one step's requests to ``num_gpus`` GPUs.

    Two requests are coupled when one reads a block the other writes in this step (including a
    request that writes a block it also reads with someone else).  ``sticky`` maps ``id(block)``
    of a write block to the GPU that already holds its private pages: such a component is pinned
    there, since private pages are not replicated.
    """
    n = len(contexts)
    parent = list(range(n))
    writer_of: Dict[int, int] = {}
    for i, ctx in enumerate(contexts):
        key = id(ctx.output_block)
        if key in writer_of:
            raise ValueError("two requests write the same block in one step")
        writer_of[key] = i
    for i, ctx in enumerate(contexts):
        for block in ctx.cache_view:
            j = writer_of.get(id(block))
            if j is not None and j != i:
                parent[_find(parent, i)] = _find(parent, j)
    groups: Dict[int, List[int]] = {}
    for i in range(n):
        groups.setdefault(_find(parent, i), []).append(i)
    components = sorted(groups.values(), key=lambda c: c[0])

    def cost(i: int) -> int:
        ctx = contexts[i]
        return sum(b.num_tokens for b in ctx.cache_view) + 1

    load = [0] * num_gpus
    assignment = [-1] * n
    free: List[List[int]] = []
    for comp in components:
        pinned = None
        if sticky:
            for i in comp:
                g = sticky.get(id(contexts[i].output_block))
                if g is not None:
                    if pinned is not None and pinned != g:
                        raise ValueError("coupled requests hold private pages on different GPUs")
                    pinned = g
        if pinned is None:
            free.append(comp)
        else:
            for i in comp:
                assignment[i] = pinned
            load[pinned] += sum(cost(i) for i in comp)
    # longest-processing-time-first bin packing of the unpinned components
    for comp in sorted(free, key=lambda c: -sum(cost(i) for i in c)):
        g = min(range(num_gpus), key=lambda x: (load[x], x))
        for i in comp:
            assignment[i] = g
        load[g] += sum(cost(i) for i in comp)
    shards = [[i for i in range(n) if assignment[i] == g] for g in range(num_gpus)]
    return Partition(assignment=assignment, shards=shards, load=load, components=components)


class BlockReplicator:
    """Publishes blocks written on one rank into the other ranks' own KV pools.

    Every rank calls ``publish`` with its local replica object of the same logical block (same
    call order on all ranks, as with any collective).  The source rank gathers the block's new
    K/V rows of every layer into one staging tensor, the group broadcasts it, and each receiver
    borrows pages from its OWN allocator and scatters the rows in; afterwards the replica's
    ``num_tokens`` / ``page_starts`` / GDN summaries describe the same tokens on every rank.
    """

    def __init__(self, kv_cache, page_allocator, group=None):
        self.kv_cache = kv_cache
        self.page_allocator = page_allocator
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.bytes_sent = 0

    def _flat(self, layer: int):
        k = self.kv_cache.k_cache(layer)
        v = self.kv_cache.v_cache(layer)
        return k.view(-1, k.shape[-2], k.shape[-1]), v.view(-1, v.shape[-2], v.shape[-1])

    def publish(self, block: CacheBlock, src: int, first_token: int = 0, total_tokens: Optional[int] = None,
                gdn_layers: Sequence[int] = ()) -> None:
        """Replicate tokens ``[first_token, total_tokens)`` of ``block`` from rank ``src``.

        ``total_tokens`` is the block's token count on the source after the write (receivers do not
        know it).  Receivers must hold the block's first ``first_token`` tokens already.
        """
        if self.world == 1:
            return
        device = self.kv_cache.device
        meta = [None]
        if self.rank == src:
            total = block.num_tokens if total_tokens is None else total_tokens
            gdn = []
            for layer in gdn_layers:
                pair = block.linear_affine.get(layer)
                conv = block.linear_conv_state.get(layer)
                if pair is None and conv is None:
                    continue
                gdn.append((layer,
                            None if pair is None else (tuple(pair[0].shape), tuple(pair[1].shape), str(pair[0].dtype)),
                            None if conv is None else (tuple(conv.shape), str(conv.dtype))))
            meta = [{"total": total, "span": block.mrope_span_override,
                     "token_ids": list(block.token_ids[first_token:total]), "gdn": gdn}]
        dist.broadcast_object_list(meta, src=src, group=self.group)
        info = meta[0]
        total = info["total"]
        n_new = total - first_token
        layers = self.kv_cache.num_layers
        k0, _ = self._flat(0)
        if n_new > 0:
            stage = torch.empty(layers, 2, n_new, k0.shape[1], k0.shape[2], dtype=k0.dtype, device=device)
            if self.rank == src:
                slots = block.token_slots_tensor().to(device).long()[first_token:total]
                for layer in range(layers):
                    kf, vf = self._flat(layer)
                    stage[layer, 0] = kf[slots]
                    stage[layer, 1] = vf[slots]
            dist.broadcast(stage, src=src, group=self.group)
            self.bytes_sent += stage.numel() * stage.element_size() if self.rank == src else 0
            if self.rank != src:
                assert block.num_tokens == first_token, "replica is missing earlier tokens of the block"
                fresh = self.page_allocator.alloc_pages(block.pages_needed(n_new))
                block.grow_pages(fresh, n_new)
                slots = block.token_slots_tensor().to(device).long()[first_token:total]
                for layer in range(layers):
                    kf, vf = self._flat(layer)
                    kf[slots] = stage[layer, 0]
                    vf[slots] = stage[layer, 1]
        if self.rank != src:
            # bookkeeping that does not depend on new rows having been sent (a publish may only
            # refresh the span or the recurrent state of a block whose tokens are already here)
            block.token_ids.extend(info["token_ids"])
            block.mrope_span_override = info["span"]

        def as_dtype(name: str) -> torch.dtype:
            return getattr(torch, name.split(".")[-1])

        # GDN state of the published layers: the affine pair and the conv window a reader of the
        # replica needs to continue the block (minisgl/shared_cache/gdn.py:127-207)
        for layer, pair_info, conv_info in info["gdn"]:
            if pair_info is not None:
                sa, sb, dt = pair_info
                if self.rank == src:
                    a, b = (t.to(device).contiguous() for t in block.linear_affine[layer])
                else:
                    a = torch.empty(sa, dtype=as_dtype(dt), device=device)
                    b = torch.empty(sb, dtype=as_dtype(dt), device=device)
                dist.broadcast(a, src=src, group=self.group)
                dist.broadcast(b, src=src, group=self.group)
                if self.rank == src:
                    self.bytes_sent += (a.numel() + b.numel()) * a.element_size()
                else:
                    block.linear_affine[layer] = (a, b)
            if conv_info is not None:
                sc, dt = conv_info
                if self.rank == src:
                    c = block.linear_conv_state[layer].to(device).contiguous()
                else:
                    c = torch.empty(sc, dtype=as_dtype(dt), device=device)
                dist.broadcast(c, src=src, group=self.group)
                if self.rank == src:
                    self.bytes_sent += c.numel() * c.element_size()
                else:
                    block.linear_conv_state[layer] = c


__all__ = ["Partition", "partition_contexts", "BlockReplicator"]
