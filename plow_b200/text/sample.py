"""Host sampler: temperature / top-k / top-p / min-p with penalties and a per-request seed.

Greedy requests never reach this code (the device argmax result is used).  The device sampler in
``csrc/cuda`` implements the same filter order so both produce the same support set
(reference: crates/plowrt/src/text/sample.rs, runtime/nvidia/sample_sm120.cu).
"""
from __future__ import annotations

import numpy as np


def apply_penalties(logits: np.ndarray, history, presence=0.0, frequency=0.0, repetition=1.0) -> np.ndarray:
    if not history or (presence == 0.0 and frequency == 0.0 and repetition == 1.0):
        return logits
    out = logits.copy()
    ids, counts = np.unique(np.asarray(history, dtype=np.int64), return_counts=True)
    if repetition != 1.0:
        v = out[ids]
        out[ids] = np.where(v > 0, v / repetition, v * repetition)
    out[ids] -= presence + frequency * counts
    return out


def filter_probs(logits: np.ndarray, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0) -> np.ndarray:
    """Order: temperature -> top-k -> softmax -> top-p -> min-p -> renormalise."""
    x = logits.astype(np.float64) / max(temperature, 1e-6)
    if top_k and top_k < x.shape[0]:
        kth = np.partition(x, -top_k)[-top_k]
        x = np.where(x < kth, -np.inf, x)
    x = x - x.max()
    p = np.exp(x)
    p /= p.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cum = np.cumsum(p[order])
        cut = int(np.searchsorted(cum, top_p, side="left")) + 1
        mask = np.zeros_like(p, dtype=bool)
        mask[order[:cut]] = True
        p = np.where(mask, p, 0.0)
    if min_p > 0.0:
        p = np.where(p < min_p * p.max(), 0.0, p)
    return p / p.sum()


def sample(logits: np.ndarray, rng: np.random.Generator, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0) -> int:
    if temperature <= 0.0:
        return int(np.argmax(logits))
    p = filter_probs(logits, temperature, top_k, top_p, min_p)
    return int(rng.choice(p.shape[0], p=p))


def logprobs_of(logits: np.ndarray, token: int, top_n: int = 0):
    x = logits.astype(np.float64)
    lse = x.max() + np.log(np.exp(x - x.max()).sum())
    lp = x - lse
    top = []
    if top_n:
        idx = np.argsort(-lp, kind="stable")[:top_n]
        top = [(int(i), float(lp[i])) for i in idx]
    return float(lp[token]), top
