"""Paged KV cache bookkeeping: page allocator, per-sequence page tables, prefix sharing.

Pages hold 64 tokens.  A *block hash chain* identifies the content of every full page of a
prompt: ``h_i = H(h_{i-1}, tokens[64 i : 64 (i+1)], namespace)``; a page whose hash is already
published is shared (refcount + 1) instead of recomputed, after a token-by-token verify so a
hash collision can never alias two prompts.  Pages are published only after the step that filled
them has completed.  Unreferenced published pages stay in an LRU list and are reclaimed on demand.

Reference counterparts: the content-addressed KV block store (crates/plowrt/src/memory/kv_store.rs,
docs/arch/26-kv-block-store.md:206-330: chained token hash + token verify, Filling->Ready states,
reclaim LRU) and the unused vLLM-style allocator (memory/kv.rs) whose design this build ships.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass, field

PAGE = 64


class OutOfPages(RuntimeError):
    pass


def chain_hash(prev: bytes, tokens, namespace: bytes = b"") -> bytes:
    h = hashlib.blake2b(digest_size=16)
    h.update(prev)
    h.update(namespace)
    h.update(struct.pack(f"<{len(tokens)}i", *tokens))
    return h.digest()


@dataclass
class _Block:
    page: int
    tokens: tuple
    refs: int = 0


@dataclass
class SeqPages:
    pages: list = field(default_factory=list)     # physical page ids in logical order
    n_shared: int = 0                              # leading pages attached from the prefix cache
    hashes: list = field(default_factory=list)    # chain hash per full page (published or pending)
    published: int = 0                             # number of own pages already published


class PagePool:
    def __init__(self, n_pages: int, namespace: bytes = b"", enable_prefix: bool = True):
        self.n_pages = n_pages
        self.free = list(range(n_pages - 1, -1, -1))
        self.namespace = namespace
        self.enable_prefix = enable_prefix
        self.blocks: dict[bytes, _Block] = {}          # hash -> block
        self.page_hash: dict[int, bytes] = {}
        self.lru: OrderedDict[bytes, None] = OrderedDict()   # published blocks with refs == 0
        self.seqs: dict[int, SeqPages] = {}
        self.stats = dict(hits=0, misses=0, evictions=0, spilled=0, restored=0)
        # second tier (host memory): on_evict(page, hash, tokens) saves a published page that is about to be reused,
        # host_has(hash) / on_restore(page, hash) -> tokens bring it back on a later prefix match
        self.on_evict = None
        self.host_has = None
        self.on_restore = None

    # ---- capacity ------------------------------------------------------------------------------
    def available(self) -> int:
        return len(self.free) + len(self.lru)

    def _take(self) -> int:
        if self.free:
            return self.free.pop()
        if self.lru:
            h, _ = self.lru.popitem(last=False)
            blk = self.blocks.pop(h)
            self.page_hash.pop(blk.page, None)
            self.stats["evictions"] += 1
            if self.on_evict is not None:
                self.on_evict(blk.page, h, blk.tokens)
                self.stats["spilled"] += 1
            return blk.page
        raise OutOfPages("KV page pool exhausted")

    # ---- sequences -----------------------------------------------------------------------------
    def begin(self, slot: int, prompt: list) -> int:
        """Attach the longest cached prefix of `prompt`; returns the number of cached tokens
        (a multiple of PAGE, and strictly less than len(prompt) so at least one token is computed)."""
        assert slot not in self.seqs
        sp = SeqPages()
        self.seqs[slot] = sp
        if not self.enable_prefix:
            return 0
        prev = b""
        n_full = (len(prompt) - 1) // PAGE
        for i in range(n_full):
            toks = tuple(prompt[i * PAGE:(i + 1) * PAGE])
            h = chain_hash(prev, toks, self.namespace)
            blk = self.blocks.get(h)
            if blk is None and self.host_has is not None and self.host_has(h) and self.available() > 0:
                # the page was evicted to host memory: take a device page and copy it back
                page = self._take()
                if self.on_restore(page, h) == toks:
                    blk = _Block(page=page, tokens=toks, refs=0)
                    self.blocks[h] = blk
                    self.page_hash[page] = h
                    self.lru[h] = None
                    self.stats["restored"] += 1
                else:
                    self.free.append(page)
            if blk is None or blk.tokens != toks:
                self.stats["misses"] += 1
                break
            if blk.refs == 0:
                self.lru.pop(h, None)
            blk.refs += 1
            sp.pages.append(blk.page)
            sp.hashes.append(h)
            sp.n_shared += 1
            self.stats["hits"] += 1
            prev = h
        sp.published = sp.n_shared
        return sp.n_shared * PAGE

    def ensure(self, slot: int, n_tokens: int) -> list:
        """Make sure pages exist for positions [0, n_tokens); returns the page list."""
        sp = self.seqs[slot]
        need = (n_tokens + PAGE - 1) // PAGE
        if need - len(sp.pages) > self.available():
            raise OutOfPages(f"need {need - len(sp.pages)} pages, {self.available()} available")
        while len(sp.pages) < need:
            sp.pages.append(self._take())
        return sp.pages

    def publish(self, slot: int, tokens: list) -> int:
        """Publish every full page of `tokens` whose content is final (call after the step that
        wrote them has completed).  Returns how many pages were newly published."""
        if not self.enable_prefix:
            return 0
        sp = self.seqs[slot]
        n_full = min(len(tokens) // PAGE, len(sp.pages))
        new = 0
        prev = sp.hashes[sp.published - 1] if sp.published else b""
        for i in range(sp.published, n_full):
            toks = tuple(tokens[i * PAGE:(i + 1) * PAGE])
            h = chain_hash(prev, toks, self.namespace)
            if len(sp.hashes) <= i:
                sp.hashes.append(h)
            else:
                sp.hashes[i] = h
            if h not in self.blocks:
                self.blocks[h] = _Block(page=sp.pages[i], tokens=toks, refs=1)
                self.page_hash[sp.pages[i]] = h
                new += 1
            elif self.blocks[h].page != sp.pages[i]:
                # same content already published by another sequence: keep ours private
                pass
            prev = h
            sp.published = i + 1
        return new

    def release(self, slot: int) -> None:
        sp = self.seqs.pop(slot)
        for i, pg in enumerate(sp.pages):
            h = self.page_hash.get(pg)
            if h is not None and self.blocks.get(h) is not None and self.blocks[h].page == pg:
                blk = self.blocks[h]
                blk.refs -= 1
                if blk.refs == 0:
                    self.lru[h] = None
            else:
                self.free.append(pg)

    def truncate(self, slot: int, n_tokens: int) -> None:
        """Rewind a sequence (e.g. rejected speculative tokens): drop pages past n_tokens."""
        sp = self.seqs[slot]
        need = (n_tokens + PAGE - 1) // PAGE
        while len(sp.pages) > max(need, sp.published):
            self.free.append(sp.pages.pop())

    def cached_prefix_len(self, prompt: list) -> int:
        """Probe only (used by the data-parallel router to pick the rank with the longest hit)."""
        prev, n = b"", 0
        for i in range((len(prompt) - 1) // PAGE):
            toks = tuple(prompt[i * PAGE:(i + 1) * PAGE])
            h = chain_hash(prev, toks, self.namespace)
            blk = self.blocks.get(h)
            if blk is None or blk.tokens != toks:
                break
            n += PAGE
            prev = h
        return n

    def check(self) -> None:
        """Invariants: every page is in exactly one place; refcounts match holders."""
        held = {}
        for sp in self.seqs.values():
            for pg in sp.pages:
                held[pg] = held.get(pg, 0) + 1
        seen = set(self.free)
        assert len(seen) == len(self.free), "duplicate page in the free list"
        for h, blk in self.blocks.items():
            assert blk.page not in seen, "published page is also free"
            assert blk.refs == held.get(blk.page, 0), f"refcount {blk.refs} != holders {held.get(blk.page, 0)}"
            assert (blk.refs == 0) == (h in self.lru)
        for pg, n in held.items():
            if pg not in self.page_hash:
                assert n == 1 and pg not in seen, "private page shared or free"
        assert len(seen) + len({b.page for b in self.blocks.values()} | set(held)) == self.n_pages
