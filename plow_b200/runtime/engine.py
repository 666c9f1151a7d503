"""Engine interface shared by the CPU interpreter backend and the sm_100a backend.

An engine owns weights, the KV page pool and the per-step launch; the scheduler above it only
speaks token batches.  A :class:`TokenBatch` is the unified row format: every row carries its
token id, its position and the slot (sequence) it belongs to, so prefill chunks of several
requests, decode rows and mixed steps are all the same thing to the engine (the reference's
unified token batch: crates/plow-asset/src/token_batch.rs, exec/gpu/token_batch.rs:227).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..compiler import packet as pk
from .kv_pages import PAGE, PagePool


@dataclass
class TokenBatch:
    ids: np.ndarray           # int32 [rows]
    pos: np.ndarray           # int32 [rows]
    seq: np.ndarray           # int32 [rows] slot of each row
    sample_rows: np.ndarray   # int32 [n_sample] rows whose logits are wanted
    decode: bool = False      # one row per sequence
    want_logits: bool = False
    hidden: np.ndarray | None = None   # [rows, H] per-row hidden state (a prediction-module drafter's second input)
    want_hidden: bool = False          # return the packet's out.hidden rows in the StepResult

    @property
    def rows(self) -> int:
        return int(self.ids.shape[0])


@dataclass
class StepResult:
    ids: np.ndarray                    # int32 [n_sample] greedy tokens
    logits: np.ndarray | None = None   # float32 [n_sample, V] when requested
    hidden: np.ndarray | None = None   # out.hidden when requested: [rows, H] (a decoder) or [n_sample, H] (a drafter)
    device_ms: float = 0.0


class EngineHealth:
    HEALTHY, DEGRADED, DEAD = "healthy", "degraded", "dead"


class EngineError(RuntimeError):
    """A step failed; `fatal` means the backend is poisoned and every live slot must fail."""

    def __init__(self, msg, fatal=False):
        super().__init__(msg)
        self.fatal = fatal


class HostKvStore:
    """Second KV tier in host memory: published pages evicted from the device pool are kept here (LRU, bounded) and
    copied back when a later prompt matches their chain hash (reference: crates/plowrt/src/memory/kv_store.rs, the
    content-addressed block store with device and pinned-host slabs)."""

    def __init__(self, engine: "EngineBase", capacity_pages: int):
        from collections import OrderedDict
        self.engine, self.capacity = engine, capacity_pages
        self.blocks: "OrderedDict[bytes, tuple]" = OrderedDict()       # hash -> (tokens, {name: host array})
        pool = engine.pool
        pool.on_evict, pool.host_has, pool.on_restore = self.save, self.has, self.restore

    def has(self, h: bytes) -> bool:
        return h in self.blocks

    def save(self, page: int, h: bytes, tokens: tuple) -> None:
        from .kv_image import _to_numpy
        self.blocks[h] = (tokens, {n: _to_numpy(a, [page])[0] for n, a in self.engine.kv_arrays().items()})
        self.blocks.move_to_end(h)
        while len(self.blocks) > self.capacity:
            self.blocks.popitem(last=False)

    def restore(self, page: int, h: bytes):
        from .kv_image import _from_numpy
        tokens, arrays = self.blocks[h]
        self.blocks.move_to_end(h)
        for n, a in self.engine.kv_arrays().items():
            _from_numpy(a, [page], arrays[n][None])
        return tokens


class EngineBase:
    """Slot + page bookkeeping common to all backends."""

    def __init__(self, packet: pk.Packet, max_slots: int, n_pages: int, max_ctx: int, prefix_cache: bool = True):
        from ..models.config import ModelSpec
        self.packet = packet
        self.spec = ModelSpec.from_json(packet.sections["model.json"].decode())
        self.max_slots = max_slots
        self.max_ctx = max_ctx
        self.max_pages_per_seq = (max_ctx + PAGE - 1) // PAGE
        self.pool = PagePool(n_pages, namespace=packet.content_hash[:8], enable_prefix=prefix_cache)
        self.page_table = np.zeros((max_slots, self.max_pages_per_seq), dtype=np.int32)
        self.kvlen = np.zeros(max_slots, dtype=np.int32)
        self.tokens: dict[int, list] = {}
        self.health = EngineHealth.HEALTHY
        self.buckets = packet.section_json("serve.json")["buckets"]

    # ---- slots ---------------------------------------------------------------------------------
    def begin_slot(self, slot: int, prompt: list) -> int:
        """Seat a request; returns how many prompt tokens are already in the cache."""
        cached = self.pool.begin(slot, prompt)
        self.tokens[slot] = list(prompt[:cached])
        self.kvlen[slot] = cached
        self._sync_pages(slot)
        return cached

    def reserve(self, slot: int, n_tokens: int) -> None:
        if n_tokens > self.max_ctx:
            raise EngineError(f"slot {slot}: {n_tokens} tokens exceed max_ctx {self.max_ctx}")
        self.pool.ensure(slot, n_tokens)
        self._sync_pages(slot)

    def _sync_pages(self, slot: int) -> None:
        pages = self.pool.seqs[slot].pages
        self.page_table[slot, :len(pages)] = pages

    def commit(self, slot: int, new_tokens: list) -> None:
        """Record tokens whose KV is now in the cache and publish finished pages."""
        self.tokens[slot].extend(new_tokens)
        self.kvlen[slot] = len(self.tokens[slot])
        self.pool.publish(slot, self.tokens[slot])

    # ---- slot snapshot / rewind / resume (reference: crates/plowrt/src/exec/gpu.rs:8905-9149) ---------------------
    def snapshot_slot(self, slot: int) -> dict:
        """What a later rewind_slot needs: the committed tokens (their KV is in the cache) and the cached length."""
        return dict(tokens=list(self.tokens[slot]), kvlen=int(self.kvlen[slot]))

    def can_rewind(self, slot: int, n_tokens: int) -> bool:
        """A sequence can be cut back to n_tokens when no published (shared, content-addressed) page lies past the cut
        and the model keeps no recurrent state (which only exists for the sequence's current end)."""
        if slot not in self.tokens or n_tokens > len(self.tokens[slot]) or n_tokens < 0:
            return False
        if n_tokens == len(self.tokens[slot]):
            return True
        if self.has_recurrent_state:
            return False
        return n_tokens >= self.pool.seqs[slot].published * PAGE

    def rewind_slot(self, slot: int, n_tokens: int) -> None:
        """Forget the tokens past n_tokens (rejected drafts, a session whose next turn diverges): their pages go back
        to the pool and the next step writes position n_tokens."""
        if not self.can_rewind(slot, n_tokens):
            raise EngineError(f"slot {slot} cannot be rewound to {n_tokens} tokens")
        self.pool.truncate(slot, n_tokens)
        del self.tokens[slot][n_tokens:]
        self.kvlen[slot] = n_tokens
        self._sync_pages(slot)

    def resume_slot(self, slot: int, prompt: list) -> int:
        """Continue a retained sequence with a new prompt: keeps the longest common prefix (at most len(prompt) - 1, so
        the last prompt token is still computed and yields logits) and returns its length, or -1 when the slot cannot
        be cut back that far (the caller then retires it and seats the request afresh)."""
        have = self.tokens.get(slot)
        if have is None:
            return -1
        n = min(len(have), len(prompt) - 1)
        lcp = 0
        while lcp < n and have[lcp] == prompt[lcp]:
            lcp += 1
        if lcp == 0 or not self.can_rewind(slot, lcp):
            return -1
        self.rewind_slot(slot, lcp)
        return lcp

    def retire_slot(self, slot: int) -> None:
        self.pool.release(slot)
        self.tokens.pop(slot, None)
        self.kvlen[slot] = 0

    def enable_host_kv(self, capacity_pages: int) -> "HostKvStore":
        """Keep evicted prefix pages in host memory (call after the backend has bound its KV tensors)."""
        self.host_kv = HostKvStore(self, capacity_pages)
        return self.host_kv

    def kv_tokens_free(self) -> int:
        return self.pool.available() * PAGE

    # ---- programs ------------------------------------------------------------------------------
    def pick_program(self, rows: int, decode: bool) -> int:
        role = pk.Role.DECODE if decode else pk.Role.PREFILL
        best = None
        for i, p in enumerate(self.packet.programs):
            if p.role == role and p.rows >= rows and (best is None or p.rows < self.packet.programs[best].rows):
                best = i
        if best is None:
            raise EngineError(f"no {'decode' if decode else 'prefill'} program covers {rows} rows")
        return best

    def max_rows(self, decode: bool) -> int:
        return max(self.buckets["decode" if decode else "prefill"])

    def step(self, batch: TokenBatch) -> StepResult:   # pragma: no cover - interface
        raise NotImplementedError

    def step_multi(self, batch: TokenBatch, k: int) -> list:
        """k greedy decode steps of the same rows in one call: step i feeds the arg-max tokens of step i - 1 at the next
        position (the caller has reserved k more tokens per sequence and commits afterwards).  Returns the k
        StepResults.  This default is a host loop; the sm_100a engine chains the steps on the device
        (reference: crates/plowrt/src/exec/gpu.rs:10317, multi_step)."""
        out, ids = [], batch.ids
        for i in range(k):
            r = self.step(TokenBatch(ids, batch.pos + i, batch.seq, batch.sample_rows, decode=True))
            out.append(r)
            ids = np.asarray(r.ids, dtype=np.int32)
        return out

    # ---- lookahead-1 decode pipeline (reference: crates/plowrt/src/exec/gpu.rs:10667, pipe_step) ---------------------
    def step_launch(self, batch: TokenBatch, chain_from=None):
        """Start a decode step and return a handle for step_collect.  With ``chain_from`` (the handle of the step launched
        just before, same rows) the input ids are that step's output ids, which the host has not read yet: the caller
        can launch step n + 1 before it collects step n and do its own work for step n while the device runs n + 1.
        This default runs the step at once (the CPU backend); the sm_100a engine leaves it running on the device."""
        if chain_from is not None:
            batch = TokenBatch(np.asarray(chain_from["result"].ids[:batch.rows], np.int32), batch.pos, batch.seq, batch.sample_rows,
                               decode=batch.decode, want_logits=batch.want_logits)
        return dict(result=self.step(batch))

    def step_collect(self, handle) -> StepResult:
        return handle["result"]

    def bind_thread(self) -> None:
        """Called by a thread before it drives the engine (the current CUDA device is per host thread)."""

    # ---- rank groups ---------------------------------------------------------------------------
    lockstep = False          # True: the scheduler must call idle_step() whenever it has nothing to run

    def idle_step(self) -> bool:
        """Join the other ranks' step with an empty batch (engines in a lockstep rank group).  Returns False when no
        rank had work, so the caller may sleep."""
        return False

    def kv_arrays(self) -> dict:                       # pragma: no cover - interface
        """name -> page-indexed array of every KV tensor (for KV images and the host tier)."""
        raise NotImplementedError

    def state_arrays(self) -> dict:
        """name -> slot-indexed array of every recurrent-state tensor (empty for pure-attention models).  KV images
        carry a sequence's state entry next to its pages."""
        return {}

    @property
    def has_recurrent_state(self) -> bool:
        return any(t.tclass == pk.TClass.STATE for t in self.packet.tensors)
