"""Speculative decoding on the unified token batch: a drafter proposes k tokens, one verify step scores the pending
token plus the k drafts as k+1 rows of the same sequence, and the longest agreeing prefix is kept.  Greedy output is
identical to plain decoding by construction (every emitted token is the target model's arg-max given the accepted
prefix).  The drafter here is the prompt-lookup n-gram drafter (no second model); a model drafter plugs in through
the same ``propose`` interface.  Reference: crates/plowrt/src/exec/gpu/spec.rs:1-12 (chain drafter + span verify on
decode rungs), crates/plowrt/src/sched/spec.rs (depth plan)."""
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
                stats: SpecStats | None = None) -> list:
    """Continue ``slot`` (whose committed tokens are in the cache) from the not-yet-cached token ``pending``."""
    drafter = drafter or NgramDrafter()
    stats = stats if stats is not None else SpecStats()
    out = [pending]
    cap = min(depth, engine.buckets.get("max_seqs", 8) - 1)
    while len(out) < max_new and out[-1] not in eos:
        ctx = engine.tokens[slot] + [out[-1]]
        draft = drafter.propose(ctx, cap)[:max(0, max_new - len(out) - 1)]
        rows = [out[-1]] + draft
        n = len(engine.tokens[slot])
        engine.reserve(slot, n + len(rows) + 1)
        r = engine.step(TokenBatch(np.asarray(rows, np.int32), np.arange(n, n + len(rows), dtype=np.int32),
                                   np.full(len(rows), slot, np.int32), np.arange(len(rows), dtype=np.int32),
                                   decode=len(rows) == 1))
        got = [int(x) for x in r.ids[:len(rows)]]
        j = 0
        while j < len(draft) and draft[j] == got[j] and got[j] not in eos:
            j += 1
        engine.commit(slot, rows[:j + 1])                # KV of the pending token and the accepted drafts is valid
        new = draft[:j] + [got[j]]
        out.extend(new)
        stats.steps += 1
        stats.proposed += len(draft)
        stats.accepted += j
        stats.emitted += len(new)
    return out[:max_new]
