"""Host side of the fixed-capacity GDN tables (the graph contract of the GDN seam): addresses stay
put between steps, padding rows are zero, capacities are enforced before anything is copied."""
import numpy as np
import pytest
import torch

from async_llm_b200.blocks import CacheBlock
from async_llm_b200.view_gdn import (GDNDecodeBuffers, GDNPrefillBuffers, ROW_CHAIN_A, ROW_CONV_WRITE, ROW_READ_A,
                                     ROW_WRITE_A, SharedCacheGDN)

H, DK, DV, CONV, KW = 2, 128, 128, 512, 4
CPU = torch.device("cpu")


def make():
    return SharedCacheGDN(num_heads=H, head_k_dim=DK, head_v_dim=DV, conv_dim=CONV, conv_kernel=KW, device=CPU)


def block(layers=()):
    b = CacheBlock(CPU, 16)
    for layer in layers:
        b.linear_affine[layer] = (torch.zeros(1, H, DK, DK), torch.zeros(1, H, DV, DK))
        b.linear_conv_state[layer] = torch.zeros(CONV, KW, dtype=torch.bfloat16)
    return b


def test_decode_tables_keep_their_addresses_and_zero_the_padding():
    ar = make()
    bufs = GDNDecodeBuffers(ar, 2, 5, 3, torch.bfloat16)
    where = (bufs.tab.data_ptr(), bufs.rw.data_ptr())
    s, a, b = block((0, 1)), block((0,)), block()
    for chains, targets in (([[s, a], [s, b]], [a, b]), ([[a], [s, a, b], [s]], [a, b, block()])):
        ar.set_context(chains, targets)
        ar.prepare_decode(2, torch.bfloat16, buffers=bufs)
        st = ar._step
        assert (bufs.tab.data_ptr(), bufs.rw.data_ptr()) == where and st["tab"] is bufs.tab
        assert st["W"] == 5 and st["depth"] == 3 and st["real_W"] == len(chains)
        W = len(chains)
        tab = bufs.tab.numpy()
        assert (tab[:, :, W:, :] == 0).all(), "rows beyond the batch carry no address"
        assert (tab[ROW_WRITE_A, :, :W, 0] != 0).all() and (tab[ROW_CONV_WRITE, :, :W, 0] != 0).all()
        assert tab[ROW_CHAIN_A, 0, 0, 0] == chains[0][0].linear_affine[0][0].data_ptr()
        # the compact per-layer lists the kernels read are the [..., 0] columns of rows 2..7
        assert np.array_equal(bufs.rw.numpy(), tab[2:8, :, :, 0].transpose(1, 0, 2))
        assert np.array_equal(bufs.write_ptrs.numpy(), bufs.rw.numpy()[:, 3:6])
        ar.finish_decode(True)
        assert all(set(t.linear_affine) == {0, 1} for t in targets)
    assert bufs.prepare_count == 2


def test_capacities_are_enforced_before_anything_is_copied():
    ar = make()
    bufs = GDNDecodeBuffers(ar, 1, 2, 2, torch.bfloat16)
    three = [block() for _ in range(3)]
    ar.set_context([[t] for t in three], three)
    with pytest.raises(ValueError, match="workers exceeds"):
        ar.prepare_decode(1, torch.bfloat16, buffers=bufs)
    deep = [block(), block(), block()]
    ar.set_context([deep], [deep[-1]])
    with pytest.raises(ValueError, match="depth 3 exceeds"):
        ar.prepare_decode(1, torch.bfloat16, buffers=bufs)
    ar.set_context([[deep[0]]], [deep[0]])
    with pytest.raises(ValueError, match="layers"):
        ar.prepare_decode(2, torch.bfloat16, buffers=bufs)
    assert bufs.prepare_count == 0 and (bufs.tab == 0).all()
    assert ar._step is None


def test_prefill_segments_sit_at_a_fixed_address():
    ar = make()
    bufs = GDNPrefillBuffers(ar, 1, 4, 2, torch.bfloat16, rows=100)
    where = bufs.seg.data_ptr()
    a, b = block(), block()
    ar.set_context([[a], [b]], [a, b], prefill_segments=[30, 7])
    ar.prepare_prefill(1, torch.bfloat16, 100, buffers=bufs)
    assert bufs.seg.data_ptr() == where
    assert bufs.seg.tolist() == [0, 30, 37, 37, 37], "requests beyond the batch are empty ranges"
    ar.finish_prefill(False)
    assert not a.linear_affine, "a failed forward publishes nothing"
    ar.set_context([[a], [b]], [a, b], prefill_segments=[90, 20])
    with pytest.raises(ValueError, match="capacity"):
        ar.prepare_prefill(1, torch.bfloat16, 100, buffers=bufs)
    assert ar._step is None
