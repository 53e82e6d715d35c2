"""Request partitioner and block replication (world_size 2 over gloo on the CPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from async_llm_b200 import AsyncContext, CacheBlock, MHAKVCache, PageAllocator
from async_llm_b200.sharding import BlockReplicator, partition_contexts


def blk(n):
    b = CacheBlock(torch.device("cpu"), 4)
    b.page_starts = [4 * i for i in range(-(-n // 4))]
    b.num_tokens = n
    return b


def test_partition_keeps_coupled_requests_together_and_balances():
    prompt = blk(4000)
    thinker, writer = blk(100), blk(50)
    privates = [blk(1000 + 100 * i) for i in range(6)]
    ctxs = [AsyncContext([prompt, writer, thinker], thinker),     # reads the block the next one writes
            AsyncContext([prompt, thinker, writer], writer)]
    ctxs += [AsyncContext([prompt, p], p) for p in privates]
    part = partition_contexts(ctxs, 4)
    assert part.assignment[0] == part.assignment[1]
    assert sorted(i for s in part.shards for i in s) == list(range(len(ctxs)))
    assert [0, 1] in part.components
    assert max(part.load) - min(part.load) <= 2 * (4000 + 1500 + 1)
    # a static shared block couples nobody
    assert all(len(c) == 1 for c in part.components if c != [0, 1])
    # private pages already resident on a GPU pin their request there
    sticky = {id(privates[0]): 3, id(privates[1]): 3}
    part2 = partition_contexts(ctxs, 4, sticky=sticky)
    assert part2.assignment[2] == 3 and part2.assignment[3] == 3
    with pytest.raises(ValueError):
        partition_contexts([AsyncContext([prompt], thinker), AsyncContext([prompt], thinker)], 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _replicate_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        P, layers, hkv, d = 4, 2, 2, 8
        pool = MHAKVCache(hkv, layers, d, 64, P, torch.bfloat16, torch.device("cpu"))
        pool._buf.zero_()
        # each rank hands out different pages first, so replicas never share page numbers
        alloc = PageAllocator(64, P, torch.device("cpu"))
        alloc.alloc_pages(5 + 7 * rank)
        rep = BlockReplicator(pool, alloc)
        block = CacheBlock(torch.device("cpu"), P)
        g = torch.Generator().manual_seed(9)
        rows = torch.randn(layers, 2, 42, hkv, d, generator=g).to(torch.bfloat16)

        def write(first, last):
            fresh = alloc.alloc_pages(block.pages_needed(last - first))
            block.grow_pages(fresh, last - first)
            block.token_ids.extend(range(first, last))
            slots = block.token_slots_tensor().long()[first:last]
            for layer in range(layers):
                pool.k_cache(layer).view(-1, hkv, d)[slots] = rows[layer, 0, first:last]
                pool.v_cache(layer).view(-1, hkv, d)[slots] = rows[layer, 1, first:last]

        if rank == 0:
            write(0, 37)
            block.linear_affine[1] = (torch.full((1, 2, 4, 4), 3.0), torch.full((1, 2, 4, 4), 5.0))
            block.linear_conv_state[1] = torch.full((6, 4), 7.0, dtype=torch.bfloat16)
            block.mrope_span_override = 30
        rep.publish(block, src=0, gdn_layers=(0, 1))
        ok0 = block.mrope_span == 30
        if rank == 0:
            write(37, 42)
            block.mrope_span_override = 33
        rep.publish(block, src=0, first_token=37)
        ok0 &= block.mrope_span == 33
        if rank == 0:
            # a publish without new rows still refreshes the span and the recurrent state
            block.mrope_span_override = 34
            block.linear_conv_state[1] = torch.full((6, 4), 9.0, dtype=torch.bfloat16)
        rep.publish(block, src=0, first_token=42, gdn_layers=(1,))
        ok0 &= block.mrope_span == 34 and float(block.linear_conv_state[1].float().mean()) == 9.0
        slots = block.token_slots_tensor().long()
        ok = ok0 and block.num_tokens == 42 and block.token_ids == list(range(42))
        ok &= 1 in block.linear_conv_state and 0 not in block.linear_conv_state
        for layer in range(layers):
            ok &= torch.equal(pool.k_cache(layer).view(-1, hkv, d)[slots], rows[layer, 0])
            ok &= torch.equal(pool.v_cache(layer).view(-1, hkv, d)[slots], rows[layer, 1])
        ok &= 1 in block.linear_affine and float(block.linear_affine[1][1].mean()) == 5.0
        ok &= 0 not in block.linear_affine
        out[rank] = (bool(ok), list(block.page_starts))
    finally:
        dist.destroy_process_group()


def test_block_replication_two_ranks():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_replicate_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[0][0] and out[1][0]
    assert out[0][1] != out[1][1], "every rank keeps its own page list for the replica"
