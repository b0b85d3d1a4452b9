"""Paged K/V store for decode: the page is the chunk.

The reference's cache layer (utils/hils_cache_utils.py:9-76) re-allocates the whole cache with torch.cat on
every step (:61-62) and moves it to host memory beyond a length threshold (:19-23, :45-59); its serving
notes ask the serving engine for a page size of 64 (README.md:255,262), the chunk size.  This store keeps
that granularity: K and V live in one preallocated pool of pages of 64 tokens, a sequence owns a list of
pages (its page table), and growing a sequence by one token never copies anything - every 64 tokens it
takes one page from the free list.  Sequences of different lengths share one decode batch; the kernels
read the page table and the per-sequence lengths from device memory (ops.decode_step_paged).

Because a page is a chunk, the sparse branch reads each selected chunk as ONE page, and the sliding
window (whose left edge is snapped to a chunk boundary) walks whole pages: no kernel gathers rows across
a page boundary.  Inside a page the rows of one head are contiguous, (h_kv, 64, D): the chunk of one head
is a single 16 KB run (D = 128) where the token-major layout has 64 rows h_kv * D apart.  The pooled chunk keys and their prior bias - one row per completed chunk, 1/64 of the
store - are kept dense per sequence slot, since the selection streams all of them on every step.

Host-side bookkeeping (free list, tables, lengths) is plain Python and mirrors what sits on the device;
nothing here reads device memory back, so a decode step issues no synchronisation.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


class PagePool:
    """Free list of page ids.  Page 0 is reserved as the scratch page that inactive batch rows write to."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise ValueError("a pool needs at least two pages (page 0 is the scratch page)")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, 0, -1))   # pop() hands out 1, 2, 3, ...

    @property
    def free(self) -> int:
        return len(self._free)

    def shuffle(self, seed: int) -> None:
        """Hand the free pages out in a random order from now on (what a pool looks like after many sequences came
        and went); used to measure with a sequence's pages scattered over the pool."""
        import random
        random.Random(seed).shuffle(self._free)

    def take(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise MemoryError(f"paged store: {n} pages wanted, {len(self._free)} free of {self.num_pages - 1}")
        return [self._free.pop() for _ in range(n)]

    def give(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 < p < self.num_pages:
                raise ValueError(f"page id {p} is not a pool page")
        self._free.extend(reversed(list(pages)))


class PagedKVStore:
    """K/V pages, page tables, lengths and pooled chunk keys of up to `max_seqs` sequences and `num_layers` layers.

    Device tensors (all preallocated):
      k_pages, v_pages (num_layers, num_pages, h_kv, S, D)   the pool; one table serves every layer
      page_table       (max_seqs, max_pages) int32            page of chunk c of the sequence in slot b
      lens             (max_seqs) int32                       tokens the sequence in slot b holds
      lmk_k            (num_layers, max_seqs, max_pages, h_lmk, D)   pooled chunk keys
      prior_b          (num_layers, max_seqs, max_pages, h_q) fp32    prior bias of each chunk
    A decode batch is the slots [0, batch) with batch = 1 + the highest active slot; rows of inactive slots
    hold length 0 and point at the scratch page, so they cost one token of work and touch no sequence's data.
    """

    def __init__(self, num_pages: int, max_seqs: int, max_pages_per_seq: int, h_kv: int, head_dim: int, h_q: int,
                 h_lmk: Optional[int] = None, dtype: torch.dtype = torch.bfloat16, device="cuda", num_layers: int = 1,
                 page_size: int = 64):
        if page_size != 64:
            raise ValueError("the page is the chunk of the decode kernels: 64 tokens")
        self.S = page_size
        self.num_layers, self.max_seqs, self.max_pages = int(num_layers), int(max_seqs), int(max_pages_per_seq)
        self.h_kv, self.h_q, self.D = int(h_kv), int(h_q), int(head_dim)
        self.h_lmk = int(h_lmk if h_lmk is not None else h_q)
        self.pool = PagePool(num_pages)
        dev = torch.device(device)
        self.device, self.dtype = dev, dtype
        self.k_pages = torch.zeros((num_layers, num_pages, h_kv, self.S, head_dim), dtype=dtype, device=dev)
        self.v_pages = torch.zeros_like(self.k_pages)
        self.page_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=dev)   # 0 = scratch page
        self.lens = torch.zeros((max_seqs,), dtype=torch.int32, device=dev)
        self.lmk_k = torch.zeros((num_layers, max_seqs, max_pages_per_seq, self.h_lmk, head_dim), dtype=dtype, device=dev)
        self.prior_b = torch.zeros((num_layers, max_seqs, max_pages_per_seq, h_q), dtype=torch.float32, device=dev)
        self._active_dev = torch.zeros((max_seqs,), dtype=torch.int32, device=dev)
        # host mirrors
        self._tables: List[List[int]] = [[] for _ in range(max_seqs)]
        self._lens: List[int] = [0] * max_seqs
        self._active: List[bool] = [False] * max_seqs
        self._in_step = False

    # ---- bookkeeping ---------------------------------------------------------------------------------
    @property
    def batch(self) -> int:
        """Rows of a decode batch: 1 + the highest active slot."""
        for b in range(self.max_seqs - 1, -1, -1):
            if self._active[b]:
                return b + 1
        return 0

    def active_slots(self) -> List[int]:
        return [b for b in range(self.max_seqs) if self._active[b]]

    def length(self, slot: int) -> int:
        return self._lens[slot]

    def pages_of(self, slot: int) -> List[int]:
        return list(self._tables[slot])

    def _set_table(self, slot: int, first_chunk: int, pages: Sequence[int]) -> None:
        if not pages:
            return
        t = torch.tensor(list(pages), dtype=torch.int32)
        self.page_table[slot, first_chunk:first_chunk + len(pages)].copy_(t, non_blocking=True)

    def allocate(self, n_tokens: int = 0) -> int:
        """Activate the lowest free slot for a sequence that already has `n_tokens` tokens (to be written with
        write_prefill); reserves the pages those tokens need.  Returns the slot."""
        if self._in_step:
            raise RuntimeError("allocate() between begin_step() and end_step()")
        n_pages = (n_tokens + self.S - 1) // self.S
        if n_pages > self.max_pages or n_tokens >= self.max_pages * self.S:
            raise ValueError(f"{n_tokens} tokens do not fit {self.max_pages} pages per sequence")
        try:
            slot = self._active.index(False)
        except ValueError:
            raise MemoryError(f"paged store: all {self.max_seqs} sequence slots are in use") from None
        pages = self.pool.take(n_pages)
        self._tables[slot] = pages
        self._lens[slot] = int(n_tokens)
        self._active[slot] = True
        self._set_table(slot, 0, pages)
        self.lens[slot:slot + 1].fill_(int(n_tokens))
        self._active_dev[slot:slot + 1].fill_(1)
        return slot

    def release(self, slot: int) -> None:
        """Return the sequence's pages to the pool; the slot's row goes back to the scratch page."""
        if self._in_step:
            raise RuntimeError("release() between begin_step() and end_step()")
        if not self._active[slot]:
            raise ValueError(f"slot {slot} is not active")
        n = len(self._tables[slot])
        self.pool.give(self._tables[slot])
        self._tables[slot] = []
        self._lens[slot] = 0
        self._active[slot] = False
        if n:
            self.page_table[slot, :n].zero_()
        self.lens[slot:slot + 1].zero_()
        self._active_dev[slot:slot + 1].zero_()

    # ---- contents ------------------------------------------------------------------------------------
    def write_prefill(self, slot: int, layer: int, k: torch.Tensor, v: torch.Tensor, lmk_k: Optional[torch.Tensor] = None,
                      prior_b: Optional[torch.Tensor] = None) -> None:
        """Store the prefill of one sequence: k, v (T, h_kv, D) with T = the length given to allocate(); lmk_k
        (T // 64, h_lmk, D) and prior_b (T // 64, h_q) of its complete chunks."""
        T = self._lens[slot]
        if k.shape != (T, self.h_kv, self.D) or v.shape != k.shape:
            raise ValueError(f"write_prefill: expected ({T}, {self.h_kv}, {self.D}), got {tuple(k.shape)} / {tuple(v.shape)}")
        pages = self._tables[slot]
        full, rem = T // self.S, T % self.S
        if full:
            ids = torch.tensor(pages[:full], dtype=torch.long, device=self.device)
            def paged(x):   # (full * S, h, D) -> (full, h, S, D)
                return x[:full * self.S].reshape(full, self.S, self.h_kv, self.D).transpose(1, 2).to(self.dtype)
            self.k_pages[layer].index_copy_(0, ids, paged(k))
            self.v_pages[layer].index_copy_(0, ids, paged(v))
        if rem:
            self.k_pages[layer, pages[full], :, :rem].copy_(k[full * self.S:].transpose(0, 1))
            self.v_pages[layer, pages[full], :, :rem].copy_(v[full * self.S:].transpose(0, 1))
        if lmk_k is not None and full:
            if lmk_k.shape[0] != full:
                raise ValueError(f"write_prefill: {full} complete chunks but {lmk_k.shape[0]} chunk keys")
            self.lmk_k[layer, slot, :full].copy_(lmk_k)
            if prior_b is not None:
                self.prior_b[layer, slot, :full].copy_(prior_b)

    def gather(self, slot: int, layer: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense copies (T, h_kv, D) of a sequence's keys and values (tests, chunk-prefill against the history)."""
        T = self._lens[slot]
        n = (T + self.S - 1) // self.S
        ids = torch.tensor(self._tables[slot][:n], dtype=torch.long, device=self.device)
        k = self.k_pages[layer].index_select(0, ids).transpose(1, 2).reshape(n * self.S, self.h_kv, self.D)[:T]
        v = self.v_pages[layer].index_select(0, ids).transpose(1, 2).reshape(n * self.S, self.h_kv, self.D)[:T]
        return k, v

    # ---- the decode step -----------------------------------------------------------------------------
    def begin_step(self) -> int:
        """Make room for one more token in every active sequence (a sequence standing at a multiple of 64 tokens
        takes a page) and return max_len, the host-side bound of the lengths that the step call wants."""
        if self._in_step:
            raise RuntimeError("begin_step() twice without end_step()")
        need = [b for b in range(self.max_seqs) if self._active[b] and self._lens[b] % self.S == 0]
        for b in need:
            if len(self._tables[b]) >= self.max_pages:
                raise MemoryError(f"paged store: the sequence in slot {b} has reached {self.max_pages} pages")
        if len(need) > self.pool.free:
            raise MemoryError(f"paged store: {len(need)} pages wanted, {self.pool.free} free")
        for b in need:
            c = self._lens[b] // self.S
            if len(self._tables[b]) == c:          # the page of position lens[b] may already be reserved
                pg = self.pool.take(1)
                self._tables[b].extend(pg)
                self._set_table(b, c, pg)
        self._in_step = True
        return max((self._lens[b] for b in range(self.max_seqs) if self._active[b]), default=0)

    def step_args(self, layer: int):
        """(k_pages, v_pages, page_table, lens, lmk_k, prior_b) of one layer for the current batch."""
        n = self.batch
        return (self.k_pages[layer], self.v_pages[layer], self.page_table[:n], self.lens[:n], self.lmk_k[layer, :n],
                self.prior_b[layer, :n])

    def completing(self) -> List[int]:
        """Slots whose chunk is completed by the token of the current step (its pooled key is due after the step)."""
        return [b for b in range(self.max_seqs) if self._active[b] and (self._lens[b] + 1) % self.S == 0]

    def chunk_keys(self, layer: int, slots: Sequence[int]) -> torch.Tensor:
        """(n, 64, h_kv, D): the keys of the last chunk of each of `slots` (a token-major view of the pages)."""
        ids = torch.tensor([self._tables[b][self._lens[b] // self.S] for b in slots], dtype=torch.long, device=self.device)
        return self.k_pages[layer].index_select(0, ids).transpose(1, 2)

    def put_chunk_keys(self, layer: int, slots: Sequence[int], lmk_k: torch.Tensor, prior_b: Optional[torch.Tensor]) -> None:
        """Store the pooled key (n, h_lmk, D) and prior bias (n, h_q) of the chunk each of `slots` is completing."""
        rows = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        cols = torch.tensor([self._lens[b] // self.S for b in slots], dtype=torch.long, device=self.device)
        self.lmk_k[layer].index_put_((rows, cols), lmk_k.to(self.dtype))
        if prior_b is not None:
            self.prior_b[layer].index_put_((rows, cols), prior_b.to(torch.float32))

    def end_step(self) -> None:
        """Every active sequence is one token longer (after all layers ran the step)."""
        if not self._in_step:
            raise RuntimeError("end_step() without begin_step()")
        n = self.batch
        self.lens[:n].add_(self._active_dev[:n])
        for b in range(n):
            if self._active[b]:
                self._lens[b] += 1
        self._in_step = False

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.k_pages, self.v_pages, self.lmk_k, self.prior_b,
                                                          self.page_table, self.lens))
