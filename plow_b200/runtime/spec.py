"""Speculative decoding on the unified token batch: a drafter proposes k tokens, one verify step scores the pending
token plus the k drafts as k+1 rows of the same sequence, and the longest agreeing prefix is kept.  Greedy output is
identical to plain decoding by construction (every emitted token is the target model's arg-max given the accepted
prefix).  Two drafters: the prompt-lookup n-gram drafter (no second model) and the chain drafter over the checkpoint's
own prediction module (:class:`MtpDrafter`, a one-layer packet compiled by ``plowc --mtp``).  Reference:
crates/plowrt/src/exec/gpu/spec.rs:1-12 (chain drafter + span verify on decode rungs), crates/devgen/src/mtp.rs,
crates/plowrt/src/sched/spec.rs (depth plan)."""
from __future__ import annotations

import numpy as np

from .engine import EngineBase, TokenBatch


class NgramDrafter:
    """Propose the continuation that followed the most recent earlier occurrence of the trailing n-gram."""

    def __init__(self, max_ngram: int = 3, min_ngram: int = 1):
        self.max_ngram, self.min_ngram = max_ngram, min_ngram

    def propose(self, context: list, k: int) -> list:
        n_ctx = len(context)
        for n in range(min(self.max_ngram, n_ctx - 1), self.min_ngram - 1, -1):
            tail = context[n_ctx - n:]
            for start in range(n_ctx - n - 1, -1, -1):
                if context[start:start + n] == tail:
                    cont = context[start + n:start + n + k]
                    if cont:
                        return list(cont)
        return []


def _cat(blocks):
    import torch
    if len(blocks) == 1:
        return blocks[0]
    return torch.cat(list(blocks)) if torch.is_tensor(blocks[0]) else np.concatenate(blocks)


class MtpDrafter:
    """Chain drafter over a prediction-module packet (an engine opened on ``<assets>/mtp``).

    Row i of the module reads the decoder's normed hidden state of position i and token i + 1 and predicts token i + 2;
    it has a KV cache of its own, so it must see every position of a sequence exactly once with the decoder's hidden
    state: ``observe`` takes the rows a decoder step has just committed (prefill chunks, the accepted part of a verify
    step) and leaves the first draft of each sequence; ``propose_many`` extends it to k drafts by feeding the module its
    own hidden state and draft (one single-row step per further draft, all sequences in one launch).  Speculative rows
    are never committed: the next ``observe`` overwrites their cache entries with rows computed from decoder states.
    A sequence the drafter has not followed from position 0 without a gap (a prefix-cache hit, a plain decode step in
    between) is dropped and drafted by the fallback n-gram drafter instead."""
    needs_hidden = True

    def __init__(self, engine: EngineBase, fallback=None):
        self.eng = engine
        self.fallback = fallback or NgramDrafter()
        self.first: dict[int, tuple] = {}      # slot -> (draft id, module hidden row [1, H], next position)

    def begin(self, slot: int) -> None:
        self.retire(slot)
        self.eng.begin_slot(slot, [])

    def retire(self, slot: int) -> None:
        self.first.pop(slot, None)
        if slot in self.eng.tokens:
            self.eng.retire_slot(slot)

    def synced(self, slot: int, n_committed: int) -> bool:
        return slot in self.first and len(self.eng.tokens.get(slot, ())) == n_committed

    def propose(self, context: list, k: int) -> list:
        return self.fallback.propose(context, k)

    def observe(self, spans: list) -> None:
        """spans: (slot, start, next_ids, hidden) — the decoder committed positions start .. start + len(next_ids) - 1 of
        ``slot``; ``hidden`` [n, H] are its hidden states there and ``next_ids[i]`` is the token at position start + i + 1
        (the last one is the pending token)."""
        eng = self.eng
        ids, pos, seq, sample, blocks, kept = [], [], [], [], [], []
        cap = eng.max_rows(False)
        for slot, start, nxt, hidden in spans:
            n = len(nxt)
            if slot not in eng.tokens or len(eng.tokens[slot]) != start or n == 0 or len(ids) + n > cap \
                    or start + n + 2 > eng.max_ctx or len(kept) >= eng.buckets.get("max_seqs", 64):
                self.retire(slot)               # a gap (or no room): this sequence falls back to the n-gram drafter
                continue
            try:
                eng.reserve(slot, start + n + 1)
            except Exception:
                self.retire(slot)
                continue
            ids += [int(t) for t in nxt]
            pos += list(range(start, start + n))
            seq += [slot] * n
            sample.append(len(ids) - 1)
            blocks.append(hidden[:n])
            kept.append((slot, start, list(nxt)))
        if not kept:
            return
        one_each = len(ids) == len(kept) and len(ids) <= eng.max_rows(True)
        r = eng.step(TokenBatch(np.asarray(ids, np.int32), np.asarray(pos, np.int32), np.asarray(seq, np.int32),
                                np.asarray(sample, np.int32), decode=one_each, hidden=_cat(blocks), want_hidden=True))
        for k, (slot, start, nxt) in enumerate(kept):
            eng.commit(slot, nxt)
            self.first[slot] = (int(r.ids[k]), r.hidden[k:k + 1], start + len(nxt))

    def propose_many(self, slots: list, k: int) -> dict:
        """Up to k drafts for every slot that is in step with its decoder (others are absent from the result)."""
        eng = self.eng
        live = [s for s in sorted(slots) if s in self.first][:eng.max_rows(True)]
        out = {s: [self.first[s][0]] for s in live} if k > 0 else {}
        hid = {s: self.first[s][1] for s in live}
        for c in range(1, k):
            rows = [s for s in live if self.first[s][2] + c + 2 <= eng.max_ctx and len(out[s]) == c]
            if not rows:
                break
            try:
                for s in rows:
                    eng.reserve(s, self.first[s][2] + c + 1)
            except Exception:
                break
            r = eng.step(TokenBatch(np.asarray([out[s][-1] for s in rows], np.int32),
                                    np.asarray([self.first[s][2] + c - 1 for s in rows], np.int32),
                                    np.asarray(rows, np.int32), np.arange(len(rows), dtype=np.int32), decode=True,
                                    hidden=_cat([hid[s] for s in rows]), want_hidden=True))
            for i, s in enumerate(rows):
                out[s].append(int(r.ids[i]))
                hid[s] = r.hidden[i:i + 1]
        return out


class SpecStats:
    def __init__(self):
        self.steps = self.proposed = self.accepted = self.emitted = 0

    @property
    def tokens_per_step(self) -> float:
        return self.emitted / max(1, self.steps)


def plan_depth(accept_rate: float, max_depth: int, step_cost_per_row: float = 0.02) -> int:
    """Depth that maximises expected tokens per unit step time for a geometric acceptance model."""
    best, best_v = 0, 1.0
    for k in range(1, max_depth + 1):
        exp_tokens = sum(accept_rate ** i for i in range(k + 1))
        v = exp_tokens / (1.0 + step_cost_per_row * k)
        if v > best_v:
            best, best_v = k, v
    return best


def spec_decode(engine: EngineBase, slot: int, pending: int, max_new: int, drafter=None, depth: int = 4, eos=(),
                stats: SpecStats | None = None, prefill_hidden=None) -> list:
    """Continue ``slot`` (whose committed tokens are in the cache) from the not-yet-cached token ``pending``.  A drafter
    that reads hidden states (``needs_hidden``) also wants ``prefill_hidden``: the decoder's ``out.hidden`` rows of the
    whole committed sequence (the prefill step run with ``want_hidden``)."""
    drafter = drafter or NgramDrafter()
    stats = stats if stats is not None else SpecStats()
    model = getattr(drafter, "needs_hidden", False)
    if model:
        drafter.begin(slot)
        if prefill_hidden is not None:
            drafter.observe([(slot, 0, engine.tokens[slot][1:] + [pending], prefill_hidden)])
    out = [pending]
    cap = min(depth, engine.buckets.get("max_seqs", 8) - 1)
    while len(out) < max_new and out[-1] not in eos:
        n = len(engine.tokens[slot])
        room = max(0, min(cap, max_new - len(out) - 1))
        if model and drafter.synced(slot, n):
            draft = drafter.propose_many([slot], room).get(slot, [])[:room]
        else:
            draft = drafter.propose(engine.tokens[slot] + [out[-1]], cap)[:room]
        rows = [out[-1]] + draft
        engine.reserve(slot, n + len(rows) + 1)
        r = engine.step(TokenBatch(np.asarray(rows, np.int32), np.arange(n, n + len(rows), dtype=np.int32),
                                   np.full(len(rows), slot, np.int32), np.arange(len(rows), dtype=np.int32),
                                   decode=len(rows) == 1, want_hidden=model))
        got = [int(x) for x in r.ids[:len(rows)]]
        j = 0
        while j < len(draft) and draft[j] == got[j] and got[j] not in eos:
            j += 1
        engine.commit(slot, rows[:j + 1])                # KV of the pending token and the accepted drafts is valid
        new = draft[:j] + [got[j]]
        if model and r.hidden is not None:
            drafter.observe([(slot, n, new, r.hidden[:j + 1])])
        out.extend(new)
        stats.steps += 1
        stats.proposed += len(draft)
        stats.accepted += j
        stats.emitted += len(new)
    if model:
        drafter.retire(slot)
    return out[:max_new]
