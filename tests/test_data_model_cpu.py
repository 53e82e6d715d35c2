"""The data model the kernels index: CacheBlock paging arithmetic, its change counters, WorkerGroup /
AsyncContext, the page allocator and the write planner -- integer code, checked exactly
(the behaviours of minisgl/shared_cache/shared_block.py, worker_group.py, async_context.py,
kvcache/page_allocator.py and session.py:1078-1141)."""
import pytest
import torch

from async_llm_b200 import AsyncContext, CacheBlock, PageAllocator, WorkerGroup
from async_llm_b200.session_plan import alloc_token_storage, plan_decode_writes

CPU = torch.device("cpu")


def block(P, pages, tokens):
    b = CacheBlock(CPU, P)
    b.page_starts = [p * P for p in pages]
    b.num_tokens = tokens
    return b


def test_token_slots_follow_the_page_list():
    b = block(4, [7, 2, 9], 10)
    assert [b.slot_of(i) for i in range(10)] == [28, 29, 30, 31, 8, 9, 10, 11, 36, 37]
    assert b.token_slots_tensor().tolist() == [b.slot_of(i) for i in range(10)]
    assert (b.num_pages, b.last_page_len, b.free_tail, b.has_capacity) == (3, 2, 2, True)
    assert b.page_numbers_tensor().tolist() == [7, 2, 9]
    assert (b.pages_needed(2), b.pages_needed(3), b.pages_needed(7)) == (0, 1, 2)
    empty = CacheBlock(CPU, 4)
    assert (empty.last_page_len, empty.has_capacity, empty.pages_needed(1)) == (0, False, 1)
    assert empty.token_slots_tensor().numel() == 0


def test_append_grow_and_clear():
    b = block(4, [1], 4)
    with pytest.raises(AssertionError):
        b.append_token(None)                      # the last page is full: a page must come along
    b.append_token(5 * 4)
    assert (b.num_tokens, list(b.page_starts)) == (5, [4, 20])
    with pytest.raises(AssertionError):
        b.append_token(6 * 4)                     # room left: no page may come along
    b.mrope_span_override = 9
    b.append_token(None)
    assert (b.num_tokens, b.mrope_span) == (6, 10)   # the span advances with the token count
    b.grow_pages(torch.tensor([36]), 5)           # 2 free slots, then one fresh page
    assert (b.num_tokens, list(b.page_starts)) == (11, [4, 20, 36])
    with pytest.raises(AssertionError):
        b.grow_pages(torch.tensor([40, 44]), 1)   # wrong number of pages for the tokens
    b.linear_affine[0] = (torch.zeros(1), torch.zeros(1))
    assert b.clear() == [4, 20, 36]
    assert (b.num_tokens, list(b.page_starts), b.mrope_span_override, dict(b.linear_affine)) == (0, [], None, {})


def test_page_numbers_follow_every_kind_of_list_change():
    b = block(4, [3, 5], 8)
    first = b.page_numbers()
    assert first.tolist() == [3, 5] and b.page_numbers() is first      # kept while nothing changes
    b.page_starts.append(36)
    assert b.page_numbers().tolist() == [3, 5, 9]
    b.page_starts += [44]
    assert b.page_numbers().tolist() == [3, 5, 9, 11]
    b.page_starts[0] = 8
    assert b.page_numbers().tolist() == [2, 5, 9, 11]
    b.page_starts = [16]                                               # replaced wholesale
    assert b.page_numbers().tolist() == [4]
    b.page_starts.clear()
    assert b.page_numbers().tolist() == []


def test_state_dictionaries_count_their_mutations():
    b = CacheBlock(CPU, 4)
    rev = b._gdn_revision
    b.linear_affine[3] = (torch.zeros(1), torch.ones(1))
    b.linear_conv_state.update({3: torch.zeros(2)})
    assert b._gdn_revision >= rev + 2
    rev = b._gdn_revision
    b._replace_linear_states({1: (torch.zeros(1), torch.zeros(1))}, {})
    assert b._gdn_revision > rev and list(b.linear_affine) == [1]
    rev = b._gdn_revision
    del b.linear_affine[1]
    assert b._gdn_revision > rev


def test_worker_group_forms_and_single_writer_rule():
    a, b, c = block(4, [1], 3), block(4, [2], 4), block(4, [3], 1)
    g = WorkerGroup(cache_structure=[[a, b], [a, c]])
    assert [w.output_block for w in g] == [b, c] and g.num_workers == len(g) == 2
    assert g[0].num_cached_tokens == 7 and g.write_to == [b, c]
    assert isinstance(g[:1], WorkerGroup) and g[:1].cache_structure == [[a, b]]
    outside = WorkerGroup(cache_structure=[[a]], write_to=[c])        # write block outside the view
    assert outside[0].output_block is c
    with pytest.raises(ValueError):
        WorkerGroup(cache_structure=[[a, b], [c, b]])                 # two writers of one block
    with pytest.raises(AssertionError):
        AsyncContext()                                                # neither view nor output block
    assert AsyncContext(cache_view=[a, c]).output_block is c


def test_page_allocator_hands_out_and_takes_back():
    alloc = PageAllocator(num_pages=6, page_size=4, device=CPU)
    first = alloc.alloc_pages(2)
    assert first.tolist() == [0, 4] and alloc.num_free_pages == 4
    assert alloc.pages_to_tokens(first).tolist() == [0, 1, 2, 3, 4, 5, 6, 7]
    with pytest.raises(RuntimeError):
        alloc.alloc_pages(5)                                          # nothing is handed out on failure
    assert alloc.num_free_pages == 4
    alloc.free_pages(first)
    assert alloc.num_free_pages == 6 and alloc.free_page_starts.tolist()[-2:] == [0, 4]
    assert alloc.alloc_pages(0).numel() == 0


def test_page_allocator_host_list_tracks_the_device_list():
    # the host copy answers the write planner without a device readback; it must hand out the same
    # pages in the same order as alloc_pages and see every page that comes back
    alloc = PageAllocator(num_pages=6, page_size=4, device=CPU)
    assert alloc.alloc_page_list(2) == [0, 4]
    assert alloc.alloc_pages(1).tolist() == [8]
    assert alloc.free_page_starts.tolist() == [12, 16, 20] and alloc.num_free_pages == 3
    alloc.free_pages(torch.tensor([4], dtype=torch.int32))
    alloc.free_pages([0])
    alloc.free_pages([])
    assert alloc.free_page_starts.tolist() == [12, 16, 20, 4, 0]
    assert alloc.alloc_page_list(4) == [12, 16, 20, 4]
    with pytest.raises(RuntimeError):
        alloc.alloc_page_list(2)
    assert alloc.alloc_page_list(1) == [0] and alloc.num_free_pages == 0


def test_write_planning_borrows_one_page_per_full_block():
    P = 4
    alloc = PageAllocator(num_pages=8, page_size=P, device=CPU)
    full, room, fresh = block(P, [6], 4), block(P, [7, 5], 6), CacheBlock(CPU, P)
    room.mrope_span_override = 11
    g = WorkerGroup(cache_structure=[[full], [room], [full, fresh]])
    pending, slots, positions = plan_decode_writes(g, alloc, P, CPU)
    assert pending == {id(full): 0, id(room): None, id(fresh): 4}     # one bulk allocation, in worker order
    assert slots.tolist() == [0, 5 * P + 2, 4] and slots.dtype == torch.int32
    assert positions == [4, 11, 0]                                    # the write position is the block's span
    assert alloc.num_free_pages == 6
    starts, token_slots = alloc_token_storage(alloc, P, CPU, 7, write_to=room)
    assert starts.tolist() == [8, 12] and token_slots.tolist() == [22, 23, 8, 9, 10, 11, 12]
    starts, token_slots = alloc_token_storage(alloc, P, CPU, 3)
    assert starts.tolist() == [16] and token_slots.tolist() == [16, 17, 18]


def test_state_dictionaries_build_deferred_entries_only_when_read():
    # a publisher may hand a block's per-layer entries over as a producer; nothing is built until the
    # dictionary is read, a later complete hand-over drops an earlier unbuilt one, and every hand-over
    # counts as a mutation for the planners' caches
    b = CacheBlock(torch.device("cpu"), 16)
    built = []

    def producer(tag):
        def make():
            built.append(tag)
            return [(layer, (tag, layer)) for layer in range(3)]
        return make

    rev = b._gdn_revision
    b.linear_affine.defer(producer("first"), range(3))
    assert b._gdn_revision > rev and built == []
    assert b.linear_affine.known_keys() == {0, 1, 2}
    b.linear_affine.defer(producer("second"), range(3))
    assert built == []                                   # the first hand-over was overwritten unbuilt
    assert b.linear_affine[1] == ("second", 1) and built == ["second"]
    assert len(b.linear_affine) == 3 and 2 in b.linear_affine and list(b.linear_affine) == [0, 1, 2]
    b.linear_affine.defer(producer("third"), range(3))
    b.linear_affine[7] = "x"                             # a plain write merges what is pending first
    assert built == ["second", "third"] and b.linear_affine.get(0) == ("third", 0) and b.linear_affine[7] == "x"
    b.linear_affine.defer(producer("fourth"), range(3))
    b.linear_affine.defer(lambda: [(9, "nine")], [9])    # a partial hand-over keeps the earlier one
    assert dict(b.linear_affine.items()) == {0: ("fourth", 0), 1: ("fourth", 1), 2: ("fourth", 2), 7: "x", 9: "nine"}
    b.linear_affine.defer(producer("fifth"), range(3))
    b.clear()
    assert len(b.linear_affine) == 0 and "fifth" not in built
