"""Device sampler (csrc/cuda/sampler.cu): temperature / top-k / top-p / min-p and the draw, one CTA per row."""
from __future__ import annotations

import torch

from . import native


def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, u=None, seed=None, step=0, out=None):
    """logits f32 [rows, V] -> int32 [rows].  Per-row parameter tensors may be None (neutral); ``u`` are the
    uniform variates in [0, 1) (else a counter hash of (seed[row], step) is used)."""
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    native.call("plow_sample", out, logits, logits.stride(0), rows, V, temperature, top_k, top_p, min_p, u, seed, int(step))
    return out


def reference(logits, temperature, top_k, top_p, min_p, u):
    """Plain PyTorch statement of the same filter order and inverse-CDF draw (ties at a cut are kept)."""
    out = []
    for r in range(logits.shape[0]):
        T = float(temperature[r])
        if T <= 0:
            out.append(int(logits[r].argmax()))
            continue
        x = logits[r].double() / max(T, 1e-6)
        k = int(top_k[r])
        if 0 < k < x.numel():
            kth = torch.topk(x, k).values[-1]
            x = torch.where(x < kth, torch.full_like(x, -float("inf")), x)
        p = torch.softmax(x, 0)
        tp = float(top_p[r])
        if tp < 1.0:
            sp, order = torch.sort(p, descending=True, stable=True)
            cum = torch.cumsum(sp, 0)
            cut = int(torch.searchsorted(cum, torch.tensor(tp, dtype=cum.dtype, device=cum.device))) + 1
            thr = sp[min(cut, sp.numel()) - 1]
            p = torch.where(p >= thr, p, torch.zeros_like(p))
        mp = float(min_p[r])
        if mp > 0:
            p = torch.where(p < mp * p.max(), torch.zeros_like(p), p)
        cdf = torch.cumsum(p, 0)
        target = float(u[r]) * float(cdf[-1])
        idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype, device=cdf.device), right=True))
        out.append(min(idx, x.numel() - 1))
    return out
