"""Decode-context parallelism, stage 1: the algebra, the row -> rank layout and the sizing rules.

KV rows of a sequence are dealt block-cyclically (block = one 64-token page) over the ``d`` ranks of a DCP group, so a
decode step reads 1/d of the context per rank; each rank runs flash attention over its shard and the partial results
are merged with the log-sum-exp rule (the same merge the split-KV kernels use, with ``nsplit = d * ns_local``).
This module is the planner and the numeric oracle; the kernels that consume it are the existing split-KV decode
kernels plus a head <-> row all-to-all that is not built.  Reference: crates/packet/src/dcp.rs,
docs/arch/21-decode-context-parallelism.md:1-170, crates/plowrt/src/sched/kv_budget.rs."""
from __future__ import annotations

import math

import torch

PAGE = 64


def owner_of_token(t: int, d: int) -> int:
    return (t // PAGE) % d


def local_index(t: int, d: int) -> int:
    """Position of token ``t`` inside its owner's shard."""
    return (t // PAGE // d) * PAGE + t % PAGE


def shard_lengths(n_tokens: int, d: int) -> list:
    """Tokens held by each rank for a context of ``n_tokens``."""
    full, rem = divmod(n_tokens, PAGE)
    out = [(full // d) * PAGE for _ in range(d)]
    for b in range(full % d):
        out[b] += PAGE
    out[full % d] += rem
    return out


def pages_needed(n_tokens: int, d: int) -> int:
    """KV pages per rank a sequence of ``n_tokens`` occupies (admission uses the max over ranks)."""
    return max((n + PAGE - 1) // PAGE for n in shard_lengths(n_tokens, d))


def kv_budget_tokens(pages_per_rank: int, d: int) -> int:
    """Largest context one sequence can reach when every rank offers ``pages_per_rank`` pages."""
    return pages_per_rank * PAGE * d


def merge_partials(outs: list, lses: list) -> torch.Tensor:
    """O = sum_s O_s * exp(lse_s - gm) / sum_s exp(lse_s - gm): the FLASH_MERGE rule over the ranks' partials.
    outs[s]: [..., D] normalised partial outputs; lses[s]: [...] natural-log log-sum-exp of the partial's scores."""
    lse = torch.stack(lses)                               # [d, ...]
    gm = lse.max(0).values
    w = torch.exp(lse - gm)
    w = torch.where(torch.isfinite(w), w, torch.zeros_like(w))
    num = (torch.stack(outs) * w.unsqueeze(-1)).sum(0)
    return num / w.sum(0).clamp_min(1e-30).unsqueeze(-1)


def reference_attention_sharded(q, k, v, d: int, scale=None):
    """Attention of one query block over a context sharded block-cyclically over ``d`` ranks, merged; equals the
    unsharded softmax attention.  q [H, D], k/v [T, H, D]."""
    T, H, D = k.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    outs, lses = [], []
    for r in range(d):
        idx = torch.tensor([t for t in range(T) if owner_of_token(t, d) == r], dtype=torch.long)
        if idx.numel() == 0:
            outs.append(torch.zeros(H, D))
            lses.append(torch.full((H,), -float("inf")))
            continue
        s = torch.einsum("hd,thd->ht", q.float(), k[idx].float()) * scale
        lses.append(torch.logsumexp(s, dim=-1))
        outs.append(torch.einsum("ht,thd->hd", torch.softmax(s, -1), v[idx].float()))
    return merge_partials(outs, lses)
