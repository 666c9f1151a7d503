"""Sparse-attention indexer ops (csrc/cuda/dsa.cu): index-key cache write, tcgen05 scores, exact top-k select.

Reference semantics: runtime/common/dev_isa.h:516-534, 1083-1115; runtime/nvidia/op_dsa.cuh."""
from __future__ import annotations

import torch

from . import native

FP8 = torch.float8_e4m3fn


def k_write(cache, cache_scale, k, gamma, beta, rope_tab, pos, seq, page_table, rot, pair_mode=0, eps=1e-6):
    """k bf16 [rows, 128] -> LayerNorm(+bias) + RoPE(first ``rot`` dims) -> e4m3 cache row + f32 scale."""
    rows = k.shape[0]
    native.call("plow_dsa_k_write", cache, cache_scale, k, k.stride(0), gamma, beta, rope_tab, pos, seq, page_table,
                page_table.shape[1], rows, rot, pair_mode, float(eps))


class SelectWorkspace:
    def __init__(self, rows, max_len, device):
        self.max_len = max_len
        self.scores = torch.empty(rows, (max_len + 127) // 128 * 128, dtype=torch.float32, device=device)
        self.q8 = torch.empty(rows, 64, 128, dtype=torch.uint8, device=device).view(FP8)
        self.wq = torch.empty(rows, 64, dtype=torch.float32, device=device)


def select(q, w, cache, cache_scale, rope_tab, pos, seq, page_table, top_k, ws: SelectWorkspace, rot, pair_mode=0, out=None):
    """q bf16 [rows, 64*128], w f32 [rows, 64] -> int32 [rows, top_k] selected positions (ascending; -1 padded)."""
    rows = q.shape[0]
    if out is None:
        out = torch.empty(rows, top_k, dtype=torch.int32, device=q.device)
    native.call("plow_dsa_select", out, ws.scores, ws.scores.stride(0), ws.q8, ws.wq, q, q.stride(0), w, w.stride(0), cache,
                cache_scale, cache.shape[0], rope_tab, pos, seq, page_table, page_table.shape[1], rows, rot, pair_mode,
                top_k, ws.max_len, native.status_word(q.device))
    return out


class CompactCache:
    """Per-row compact latent cache the dense MLA decode kernel walks after a sparse selection."""

    def __init__(self, rows, top_k, row_bytes, device):
        assert top_k % 64 == 0
        self.rows, self.top_k, self.pages_per = rows, top_k, top_k // 64
        n = rows * self.pages_per
        self.kv = torch.zeros(n, 64, row_bytes, dtype=torch.uint8, device=device).view(FP8)
        self.scale = torch.zeros(n, 64, dtype=torch.float32, device=device)
        self.smax = torch.zeros(n, 4, dtype=torch.float32, device=device)
        self.kvlen = torch.zeros(rows, dtype=torch.int32, device=device)
        self.page_table = torch.arange(n, dtype=torch.int32, device=device).view(rows, self.pages_per).contiguous()
        self.slot_of = torch.arange(rows, dtype=torch.int32, device=device)


def gather(cc: CompactCache, sel, cache, scale, pos, seq, page_table):
    """Copy every row's selected tokens (sel [rows, top_k], -1 padded) into its compact cache."""
    rows = sel.shape[0]
    native.call("plow_dsa_gather", cc.kv, cc.scale, cc.smax, cc.kvlen, sel, cc.top_k, cache, scale, pos, seq, page_table,
                page_table.shape[1], rows, cache.shape[2])


def _rope(x, tab, rot, pair_mode):
    half = rot // 2
    c, s = tab[..., :half], tab[..., half:]
    y = x.clone()
    if pair_mode == 0:
        a, b = x[..., :half], x[..., half:rot]
        y[..., :half] = a * c - b * s
        y[..., half:rot] = b * c + a * s
    else:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        y[..., 0:rot:2] = a * c - b * s
        y[..., 1:rot:2] = b * c + a * s
    return y


def reference_scores(q, w, cache, cache_scale, rope_tab, pos, seq, page_table, rot, pair_mode=0):
    """fp32 scores from the (already quantised) key cache; q is roped and quantised per head like the kernel."""
    rows = q.shape[0]
    out = []
    for r in range(rows):
        n = int(pos[r]) + 1
        t = torch.arange(n, device=q.device)
        pages = page_table[int(seq[r])][(t // 64).long()].long()
        k = cache[pages, (t % 64).long()].float() * cache_scale[pages, (t % 64).long()][:, None]     # [n, 128]
        qr = _rope(q[r].float().view(64, 128), rope_tab[int(pos[r])][None, :], rot, pair_mode)
        sc = qr.abs().amax(1, keepdim=True).clamp_min(1e-10) / 448.0
        qq = (qr / sc).to(FP8).float() * sc
        s = torch.relu(qq @ k.t())                                                                    # [64, n]
        out.append((w[r].float()[:, None] * s).sum(0))
    return out


def profile_topk(iters, timer):
    rows, ctx, top_k = 64, 32768, 2048
    pages_per = ctx // 64
    n_pages = rows * pages_per + 1
    dev = "cuda"
    cache = torch.randn(n_pages, 64, 128, device=dev).to(FP8)
    cs = torch.rand(n_pages, 64, device=dev) * 0.01 + 0.001
    pt = (torch.arange(rows * pages_per, dtype=torch.int32, device=dev).view(rows, pages_per) + 1).contiguous()
    seq = torch.arange(rows, dtype=torch.int32, device=dev)
    pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
    q = torch.randn(rows, 64 * 128, device=dev).bfloat16()
    w = torch.randn(rows, 64, device=dev)
    tab = torch.zeros(ctx, 64, device=dev)
    tab[:, :32] = 1.0
    ws = SelectWorkspace(rows, ctx, dev)
    out = torch.empty(rows, top_k, dtype=torch.int32, device=dev)
    us = timer(lambda: select(q, w, cache, cs, tab, pos, seq, pt, top_k, ws, 64, out=out), iters)
    return dict(us=us, flops=2.0 * rows * ctx * 64 * 128, bytes=1.0 * rows * ctx * 132 + 8.0 * rows * ctx * 4)
