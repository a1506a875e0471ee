"""Paged KV-cache bookkeeping on the host: fixed-size pages, per-sequence page tables,
reference-counted sharing (copy-on-write fork) and a token-prefix index so that requests with
a common prompt prefix reuse pages instead of recomputing them.

Capability parity with the reference's host-side ``PagedKvCache`` / ``PrefixCache``
(src/paged_kv/mod.rs:35-235, src/paged_kv/mod_compute_prefix.rs:20-170); unlike the reference
the page table produced here is what the GPU attention kernels index.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

FNV_OFFSET = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3


def fnv1a_tokens(tokens: Sequence[int], seed: int = FNV_OFFSET) -> int:
    h = seed
    for t in tokens:
        for shift in (0, 8, 16, 24):
            h ^= (t >> shift) & 0xFF
            h = (h * FNV_PRIME) & 0xFFFFFFFFFFFFFFFF
    return h


class OutOfPages(RuntimeError):
    pass


@dataclass
class SeqState:
    pages: List[int] = field(default_factory=list)
    length: int = 0          # tokens whose K/V are in the cache


@dataclass
class PagedKvStats:
    total_pages: int
    free_pages: int
    shared_pages: int
    sequences: int

    @property
    def utilization(self) -> float:
        return 1.0 - self.free_pages / max(1, self.total_pages)


class PagedKvCache:
    def __init__(self, num_pages: int, page_size: int = 16):
        self.num_pages, self.page_size = num_pages, page_size
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._ref = [0] * num_pages
        self.seqs: Dict[int, SeqState] = {}
        # prefix index: hash of the first (i+1)*page_size tokens -> page id holding tokens [i*ps, (i+1)*ps)
        self._prefix: Dict[int, int] = {}
        self._page_key: Dict[int, int] = {}

    # -- allocation ------------------------------------------------------------------------
    def free_page_count(self) -> int:
        return len(self._free)

    def _alloc(self) -> int:
        if not self._free:
            self._evict_prefix_pages(1)
        if not self._free:
            raise OutOfPages("KV cache has no free pages")
        p = self._free.pop()
        self._ref[p] = 1
        return p

    def _release(self, p: int) -> None:
        self._ref[p] -= 1
        if self._ref[p] == 0:
            key = self._page_key.pop(p, None)
            if key is not None and self._prefix.get(key) == p:
                del self._prefix[key]
            self._free.append(p)

    def _evict_prefix_pages(self, want: int) -> None:
        """Drop index-only references (pages kept alive just by the prefix index)."""
        for key, p in list(self._prefix.items()):
            if want <= 0:
                break
            if self._ref[p] == 1 and p in self._page_key and not any(p in s.pages for s in self.seqs.values()):
                del self._prefix[key]
                del self._page_key[p]
                self._ref[p] = 0
                self._free.append(p)
                want -= 1

    def pages_needed(self, length: int) -> int:
        return -(-length // self.page_size)

    def can_allocate(self, length: int) -> bool:
        return self.pages_needed(length) <= len(self._free)

    def add_sequence(self, seq_id: int) -> SeqState:
        if seq_id in self.seqs:
            raise KeyError(f"sequence {seq_id} already exists")
        self.seqs[seq_id] = SeqState()
        return self.seqs[seq_id]

    def reserve(self, seq_id: int, length: int) -> List[int]:
        """Make sure the sequence owns pages for ``length`` tokens; returns its page list."""
        s = self.seqs[seq_id]
        while len(s.pages) < self.pages_needed(length):
            s.pages.append(self._alloc())
        return s.pages

    def set_length(self, seq_id: int, length: int) -> None:
        self.seqs[seq_id].length = length

    def free_sequence(self, seq_id: int) -> None:
        s = self.seqs.pop(seq_id)
        for p in s.pages:
            self._release(p)

    def rollback(self, seq_id: int, length: int) -> None:
        """Forget tokens past ``length`` (speculative decoding rejects); frees whole pages."""
        s = self.seqs[seq_id]
        keep = self.pages_needed(length)
        for p in s.pages[keep:]:
            self._release(p)
        del s.pages[keep:]
        s.length = min(s.length, length)

    # -- sharing -----------------------------------------------------------------------------
    def fork(self, src_id: int, dst_id: int) -> SeqState:
        """Copy-on-write fork: the new sequence references the same pages."""
        src = self.seqs[src_id]
        dst = self.add_sequence(dst_id)
        dst.pages = list(src.pages)
        dst.length = src.length
        for p in dst.pages:
            self._ref[p] += 1
        return dst

    def ensure_writable(self, seq_id: int, page_index: int) -> Tuple[int, Optional[int]]:
        """Before writing into page ``page_index`` of a sequence: if the page is shared, give the
        sequence a private page.  Returns ``(page, copy_from)``; the caller copies the page
        contents on the device when ``copy_from`` is not None."""
        s = self.seqs[seq_id]
        p = s.pages[page_index]
        if self._ref[p] == 1:
            return p, None
        q = self._alloc()
        self._ref[p] -= 1
        s.pages[page_index] = q
        return q, p

    # -- prefix cache ------------------------------------------------------------------------
    def match_prefix(self, seq_id: int, tokens: Sequence[int]) -> int:
        """Attach cached pages covering the longest known full-page prefix of ``tokens`` to the
        (empty) sequence.  Returns the number of tokens covered.  The last prompt token is never
        covered so that its logits are still computed."""
        s = self.seqs[seq_id]
        assert not s.pages
        ps = self.page_size
        h = FNV_OFFSET
        covered = 0
        for i in range((len(tokens) - 1) // ps):
            h = fnv1a_tokens(tokens[i * ps:(i + 1) * ps], h)
            p = self._prefix.get(h)
            if p is None:
                break
            s.pages.append(p)
            self._ref[p] += 1
            covered += ps
        s.length = covered
        return covered

    def publish_prefix(self, seq_id: int, tokens: Sequence[int]) -> int:
        """Index the sequence's full pages by the hash of the tokens they hold (the index keeps
        a reference so pages survive the sequence).  Returns pages newly published."""
        s = self.seqs[seq_id]
        ps = self.page_size
        h = FNV_OFFSET
        new = 0
        for i in range(min(len(s.pages), len(tokens) // ps)):
            h = fnv1a_tokens(tokens[i * ps:(i + 1) * ps], h)
            if h not in self._prefix:
                p = s.pages[i]
                self._prefix[h] = p
                self._page_key[p] = h
                self._ref[p] += 1
                new += 1
        return new

    # -- introspection -----------------------------------------------------------------------
    def stats(self) -> PagedKvStats:
        shared = sum(1 for r in self._ref if r > 1)
        return PagedKvStats(self.num_pages, len(self._free), shared, len(self.seqs))

    def refcount(self, page: int) -> int:
        return self._ref[page]
