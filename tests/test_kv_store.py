"""Bookkeeping of the paged K/V store (page = chunk = 64 tokens) on CPU tensors: page accounting, ragged
lengths, growth without copies, release and reuse, and the errors of a full pool."""
import pytest
import torch

from hils_attention_b200.kv_store import PagedKVStore, PagePool


def _store(num_pages=12, max_seqs=3, max_pages=4, **kw):
    return PagedKVStore(num_pages, max_seqs, max_pages, h_kv=2, head_dim=8, h_q=4, dtype=torch.float32, device="cpu", **kw)


def test_pool_hands_out_every_page_once_and_never_the_scratch_page():
    pool = PagePool(6)
    got = pool.take(5)
    assert sorted(got) == [1, 2, 3, 4, 5] and pool.free == 0
    with pytest.raises(MemoryError):
        pool.take(1)
    pool.give(got[:2])
    assert pool.free == 2 and set(pool.take(2)) == set(got[:2])
    with pytest.raises(ValueError):
        pool.give([0])


def test_prefill_round_trip_on_ragged_lengths():
    st = _store()
    g = torch.Generator().manual_seed(0)
    seqs = {}
    for T in (130, 64, 5):
        slot = st.allocate(T)
        k, v = torch.randn(T, 2, 8, generator=g), torch.randn(T, 2, 8, generator=g)
        n = T // 64
        st.write_prefill(slot, 0, k, v, torch.randn(n, 4, 8, generator=g) if n else None, torch.randn(n, 4, generator=g) if n else None)
        seqs[slot] = (k, v)
        assert len(st.pages_of(slot)) == (T + 63) // 64
    assert st.batch == 3 and st.pool.free == 11 - (3 + 1 + 1)
    for slot, (k, v) in seqs.items():
        gk, gv = st.gather(slot)
        assert torch.equal(gk, k) and torch.equal(gv, v)
    owned = [p for s in seqs for p in st.pages_of(s)]
    assert len(set(owned)) == len(owned) and 0 not in owned          # no page is shared, none is the scratch page
    assert st.lens.tolist() == [130, 64, 5]
    assert st.page_table[0, :3].tolist() == st.pages_of(0)


def test_growth_takes_a_page_only_at_chunk_boundaries_and_copies_nothing():
    st = _store()
    a, b = st.allocate(63), st.allocate(64)
    ptr_before = st.k_pages.data_ptr()
    free0 = st.pool.free
    assert st.begin_step() == 64
    assert st.pool.free == free0 - 1                                  # b stood at a boundary, a did not
    assert st.completing() == [a]                                     # a's token number 64 completes its chunk
    assert st.page_table[b, 1].item() == st.pages_of(b)[1]
    st.end_step()
    assert (st.length(a), st.length(b)) == (64, 65) and st.lens[:2].tolist() == [64, 65]
    st.begin_step()
    assert st.pool.free == free0 - 2 and st.completing() == []
    st.end_step()
    assert st.k_pages.data_ptr() == ptr_before                        # the pool never moved


def test_release_returns_pages_and_the_slot_is_reused():
    st = _store()
    a, b, c = st.allocate(100), st.allocate(10), st.allocate(70)
    free = st.pool.free
    st.release(b)
    assert st.pool.free == free + 1 and st.batch == 3 and st.active_slots() == [a, c]
    assert st.lens.tolist() == [100, 0, 70] and st.page_table[b].tolist() == [0, 0, 0, 0]
    st.begin_step()                                                   # the inactive row takes no page
    st.end_step()
    assert st.lens.tolist() == [101, 0, 71] and st.length(b) == 0
    assert st.allocate(3) == b
    st.release(c)
    assert st.batch == 2


def test_errors_when_the_pool_the_table_or_the_slots_run_out():
    st = _store(num_pages=4, max_seqs=2, max_pages=2)
    a = st.allocate(64)
    with pytest.raises(ValueError):
        st.allocate(128)                                              # no room left for a next token
    b = st.allocate(120)                                              # pool: 3 pages, all taken now
    with pytest.raises(MemoryError):
        st.allocate(1)                                                # no slot
    with pytest.raises(MemoryError):
        st.begin_step()                                               # a wants a page, none is free
    st.release(b)
    st.begin_step()
    with pytest.raises(RuntimeError):
        st.release(a)
    st.end_step()
    for _ in range(63):
        st.begin_step()
        st.end_step()
    assert st.length(a) == 128
    with pytest.raises(MemoryError):
        st.begin_step()                                               # the table of a is full


def test_pooled_keys_of_completed_chunks_land_in_their_rows():
    st = _store()
    a, b = st.allocate(63), st.allocate(127)
    st.begin_step()
    done = st.completing()
    assert done == [a, b]
    kc = st.chunk_keys(0, done)
    assert kc.shape == (2, 64, 2, 8)
    lk, pb = torch.ones(2, 4, 8), torch.full((2, 4), 3.0)
    st.put_chunk_keys(0, done, lk, pb)
    st.end_step()
    assert bool((st.lmk_k[0, a, 0] == 1).all()) and bool((st.lmk_k[0, b, 1] == 1).all())
    assert bool((st.lmk_k[0, b, 0] == 0).all()) and bool((st.prior_b[0, b, 1] == 3).all())
