"""Host page allocator and block-table producer: reference counts, prefix sharing following
the reference's slot-reuse rule (g4b/scheduler.py:96-125), eviction, and the index contract
of prepare_prefill_inputs / prepare_decode_inputs (g4b/scheduler.py:133-212)."""
import numpy as np
import pytest

from g4b_b200.paging import OutOfPages, PageAllocator, PagedKVManager, shared_prefix_length


def test_allocator_refcounts_and_reuse():
    a = PageAllocator(4)
    p = a.alloc(3)
    assert p == [0, 1, 2] and a.free_pages == 1
    a.retain(p[:2])
    a.release(p)
    assert a.free_pages == 2 and a.refcount(0) == 1 and a.refcount(2) == 0
    a.release(p[:2])
    assert a.free_pages == 4
    with pytest.raises(RuntimeError):
        a.release([0])
    with pytest.raises(OutOfPages):
        a.alloc(5)


def test_shared_prefix_length_like_reference():
    assert shared_prefix_length([1, 2, 3], [1, 2, 4, 5]) == 2
    assert shared_prefix_length([], [1]) == 0
    assert shared_prefix_length([1, 2], [1, 2, 3]) == 2


def run_prefill(m, slot, start, n_tokens, chunk):
    """Feeds the prompt chunk by chunk the way the scheduler does (padded chunk counted in time)."""
    pos = start
    while pos < n_tokens:
        end = min(pos + chunk, n_tokens)
        off = [0] * m.max_batch
        tim = [0] * m.max_batch
        off[slot], tim[slot] = pos, pos + chunk
        m.prepare_prefill_inputs(None, off, tim)
        pos = end


def test_tables_cover_padded_chunk_and_idle_slots_are_unallocated():
    m = PagedKVManager(num_pages=64, max_batch=3, max_context=256, page_size=16, prefill_chunk=32)
    slot, pos = m.place_request(list(range(40)))
    assert pos == 0
    off, tim = [0] * 3, [0] * 3
    off[slot], tim[slot] = 0, 32
    bt, co, td, ph = m.prepare_prefill_inputs(None, off, tim)
    assert (bt[slot, :2] >= 0).all() and (bt[slot, 2:] == -1).all()
    assert ph.tolist() == [1 if b == slot else 0 for b in range(3)]
    off[slot], tim[slot] = 32, 64          # second chunk: 8 real tokens, padded to 32
    bt, co, td, ph = m.prepare_prefill_inputs(None, off, tim)
    assert (bt[slot, :4] >= 0).all() and td[slot] == 64 and co[slot] == 32
    assert len(set(bt[slot, :4].tolist())) == 4


def test_prefix_sharing_from_a_running_slot_and_rule_of_the_last_chunk():
    chunk = 32
    m = PagedKVManager(num_pages=64, max_batch=3, max_context=512, page_size=16, prefill_chunk=chunk)
    a_tokens = list(range(100))
    a, _ = m.place_request(a_tokens)
    run_prefill(m, a, 0, 100, chunk)
    # same first 70 tokens: whole chunks below token 69 -> 64 tokens = 4 pages shared, donor still active
    b_tokens = a_tokens[:70] + [999] * 10
    b, pos = m.place_request(b_tokens)
    assert b != a and pos == 64
    assert m.block_tables[b, :4].tolist() == m.block_tables[a, :4].tolist()
    assert all(m.alloc.refcount(p) == 2 for p in m.block_tables[a, :4])
    run_prefill(m, b, pos, len(b_tokens), chunk)
    assert m.block_tables[b, 4] not in m.block_tables[a].tolist()
    # identical prompt: the chunk holding the last token must still run (scheduler.py:118-122)
    c, pos_c = m.place_request(a_tokens[:64])
    assert pos_c == 32
    # the donor leaves; shared pages survive through the other owners
    m.retire(a)
    m.retire(b)
    m.retire(c)
    assert all(m.alloc.refcount(p) >= 1 for p in m.block_tables[a, :4])


def test_nothing_is_shared_before_the_donor_has_written_it():
    m = PagedKVManager(num_pages=64, max_batch=2, max_context=512, page_size=16, prefill_chunk=16)
    toks = list(range(200))
    a, _ = m.place_request(toks)
    off, tim = [0, 0], [0, 0]
    off[a], tim[a] = 0, 16
    m.prepare_prefill_inputs(None, off, tim)           # only the first 16 tokens are launched
    b, pos = m.place_request(toks)
    assert pos == 0                                    # (16 - 1) // 16 * 16


def test_free_donor_is_reused_in_place_and_its_tail_dropped():
    m = PagedKVManager(num_pages=16, max_batch=2, max_context=256, page_size=16, prefill_chunk=16)
    toks = list(range(90))
    a, _ = m.place_request(toks)
    run_prefill(m, a, 0, 90, 16)
    used = 16 - m.alloc.free_pages
    assert used == 6
    m.retire(a)
    b, pos = m.place_request(toks[:50] + [7, 7, 7])
    assert b == a and pos == 48
    assert 16 - m.alloc.free_pages == 3               # pages past the shared prefix went back


def test_eviction_of_retired_slots_oldest_first_then_out_of_pages():
    m = PagedKVManager(num_pages=8, max_batch=3, max_context=256, page_size=16, prefill_chunk=16)
    s0, _ = m.place_request([1] * 48)
    run_prefill(m, s0, 0, 48, 16)
    s1, _ = m.place_request([2] * 48)
    run_prefill(m, s1, 0, 48, 16)
    m.retire(s0)
    m.retire(s1)
    s2, pos = m.place_request([3] * 64)
    assert pos == 0 and s2 not in (s0, s1)
    run_prefill(m, s2, 0, 64, 16)                      # needs 4 pages, 2 free: drops s0 (oldest) only
    assert m.slots[s0].pages == [] and len(m.slots[s1].pages) == 3
    with pytest.raises(OutOfPages):
        m.ensure(s2, 16 * 9)                           # more than the whole pool


def test_decode_reservation_and_host_mirror_of_advance():
    m = PagedKVManager(num_pages=32, max_batch=2, max_context=96, page_size=16, prefill_chunk=16,
                       decode_reserve_pages=1)
    s, _ = m.place_request(list(range(30)))
    run_prefill(m, s, 0, 30, 16)
    off, tim = [0, 0], [0, 0]
    off[s], tim[s] = 30, 31                            # scheduler.py:199-203
    bt, co, td, ph = m.prepare_decode_inputs(None, off, tim)
    assert ph[s] == 2 and ph[1 - s] == 0
    assert (bt[s, :3] >= 0).all()                      # page of token 30 + one reserved
    uploads = 0
    for step in range(60):
        if int(m.time_dim_sizes[s]) >= 96:
            break
        changed = m.advance_decode()
        uploads += changed
        assert m.decode_steps_covered(s) >= 1 or int(m.time_dim_sizes[s]) == 96
        assert co[s] == 31 + step and td[s] == 32 + step
    assert 1 <= uploads <= 4                           # a new table only every page_size steps
    with pytest.raises(ValueError):
        m.ensure(s, 97)


def test_max_context_rounds_up_to_pages():
    m = PagedKVManager(num_pages=4, max_batch=1, max_context=40, page_size=16)
    assert m.block_tables.shape == (1, 3) and m.block_tables.dtype == np.int32
