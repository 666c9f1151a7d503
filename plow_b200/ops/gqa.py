"""Grouped-query attention ops over the paged KV cache, bf16 or e4m3 with one scale per (token, kv head)
(csrc/cuda/attn_gqa.cu).

``rope_kv`` is the fused head-norm + RoPE + cache-write row op (reference op HEADNORM_ROPE,
runtime/common/dev_isa.h:74-84); ``attention`` is the tcgen05 flash kernel that serves prefill
(causal by position) and decode (one row per sequence) from the same work list
(runtime/common/dev_isa.h:185-222).
"""
from __future__ import annotations

import math

import torch

from . import native

BF16 = torch.bfloat16


def rope_kv(qkv, kc, vc, rope_tab, pos, seq, page_table, nq, nkv, hd, rot=None, pair_mode=0,
            qn=None, kn=None, eps=1e-6, plus_one=False, q_out=None, gate_out=None, kv_scale=None):
    """qkv [rows, (nq+2*nkv)*hd] bf16 -> q_out [rows, nq, hd]; K (roped) and V rows land in their cache cells.
    With ``gate_out`` [rows, nq*hd] the query heads are [Q | gate] pairs (gated attention) and the gates are copied out.
    With ``kv_scale`` f32 [n_pages, 64, 2*nkv] the caches are e4m3 bytes (uint8 / float8 tensors) and every written cell
    stores amax / 448 there (k scales, then v scales of the token)."""
    rows = qkv.shape[0]
    if q_out is None:
        q_out = torch.empty(rows, nq, hd, dtype=BF16, device=qkv.device)
    native.call("plow_rope_kv", q_out, qkv, qkv.stride(0), kc, vc, qn, kn, rope_tab, pos, seq, page_table,
                page_table.shape[1], rows, nq, nkv, hd, hd if rot is None else rot, pair_mode, int(plus_one), float(eps), gate_out, kv_scale)
    return q_out


class AttnWorkspace:
    """Device scratch of one attention call shape: work list, split partials, per-row split counts."""

    def __init__(self, rows, nq, nkv, hd, max_ctx, device, tiles_per_split=None, max_splits=None):
        group = nq // nkv
        tq = max(1, 128 // group)
        tiles = (max_ctx + 63) // 64
        if max_splits is None:
            # enough (chunk, kv head, split) items to fill 148 SMs when the batch alone does not
            chunks = max(1, (rows + tq - 1) // tq) if rows > 256 else rows
            max_splits = max(1, min(16, (2 * 148 + chunks * nkv - 1) // (chunks * nkv), tiles))
        if tiles_per_split is None:
            tiles_per_split = max(2, (tiles + max_splits - 1) // max_splits)
        self.tiles_per_split, self.max_splits = tiles_per_split, max_splits
        self.item_cap = rows * nkv * max_splits
        self.items = torch.empty(self.item_cap * 8, dtype=torch.int32, device=device)
        self.n_items = torch.zeros(1, dtype=torch.int32, device=device)
        self.row_ns = torch.zeros(rows, dtype=torch.int32, device=device)
        if max_splits > 1:
            self.opart = torch.empty(rows, nq, max_splits, hd, dtype=torch.float32, device=device)
            self.lse = torch.empty(rows, nq, max_splits, dtype=torch.float32, device=device)
        else:
            self.opart = self.lse = None


def attention(q, kc, vc, page_table, seq, pos, ws: AttnWorkspace, scale=None, window=0, out=None, kv_scale=None):
    """q [rows, nq, hd] bf16; kc / vc [n_pages, 64, nkv, hd] bf16 (or e4m3 bytes with ``kv_scale`` f32
    [n_pages, 64, 2*nkv], head dim 128) -> out [rows, nq*hd] bf16."""
    rows, nq, hd = q.shape
    nkv = kc.shape[2]
    if out is None:
        out = torch.empty(rows, nq * hd, dtype=BF16, device=q.device)
    native.call("plow_gqa_attention", q, kc, vc, kc.shape[0], page_table, page_table.shape[1], seq, pos, rows, nq, nkv, hd,
                int(window), ws.tiles_per_split, ws.max_splits, ws.items, ws.item_cap, ws.n_items, ws.row_ns,
                ws.opart, ws.lse, out, float(scale if scale is not None else 1.0 / math.sqrt(hd)), kv_scale,
                native.status_word(q.device))
    return out


def quant_cache(c):
    """bf16 cache [n_pages, 64, nkv, hd] -> (e4m3 bytes as float8 tensor, f32 scales [n_pages, 64, nkv]) with the
    writer's rule (scale = amax / 448 per cell); ``dequant_cache`` is what the attention kernel's converter forms."""
    cf = c.float()
    sc = cf.abs().amax(dim=-1).clamp_min(1e-12) / 448.0
    return (cf / sc[..., None]).to(torch.float8_e4m3fn), sc


def dequant_cache(c8, sc):
    return (c8.float() * sc[..., None]).to(BF16)


def reference(q, kc, vc, page_table, seq, pos, scale=None, window=0):
    """Plain PyTorch fp32 statement of the op (the numerics oracle of the tests)."""
    rows, nq, hd = q.shape
    nkv = kc.shape[2]
    group = nq // nkv
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    out = torch.zeros(rows, nq * hd, dtype=torch.float32, device=q.device)
    for r in range(rows):
        p = int(pos[r])
        if p < 0:
            continue
        lo = max(0, p - window + 1) if window > 0 else 0
        t = torch.arange(lo, p + 1, device=q.device)
        pages = page_table[int(seq[r])][(t // 64).long()].long()
        k = kc[pages, (t % 64).long()].float()          # [n, nkv, hd]
        v = vc[pages, (t % 64).long()].float()
        qr = q[r].float().view(nkv, group, hd)
        s = torch.einsum("kgd,nkd->kgn", qr, k) * scale
        pr = torch.softmax(s, dim=-1)
        out[r] = torch.einsum("kgn,nkd->kgd", pr, v).reshape(-1)
    return out


def _paged_case(n_seq, ctx, nq, nkv, hd, rows_per_seq, device="cuda"):
    pages_per = (ctx + 63) // 64
    n_pages = n_seq * pages_per + 1
    kc = torch.randn(n_pages, 64, nkv, hd, device=device).to(BF16)
    vc = torch.randn(n_pages, 64, nkv, hd, device=device).to(BF16)
    pt = (torch.arange(n_seq * pages_per, dtype=torch.int32, device=device).view(n_seq, pages_per) + 1).contiguous()
    seq = torch.arange(n_seq, dtype=torch.int32, device=device).repeat_interleave(rows_per_seq)
    pos = (torch.arange(rows_per_seq, dtype=torch.int32, device=device) + (ctx - rows_per_seq)).repeat(n_seq)
    q = torch.randn(n_seq * rows_per_seq, nq, hd, device=device).to(BF16)
    return q, kc, vc, pt, seq, pos


def profile_decode(iters, timer):
    n_seq, ctx, nq, nkv, hd = 64, 4096, 32, 8, 128
    q, kc, vc, pt, seq, pos = _paged_case(n_seq, ctx, nq, nkv, hd, 1)
    ws = AttnWorkspace(n_seq, nq, nkv, hd, ctx, q.device)
    out = torch.empty(n_seq, nq * hd, dtype=BF16, device=q.device)
    us = timer(lambda: attention(q, kc, vc, pt, seq, pos, ws, out=out), iters)
    return dict(us=us, flops=4.0 * n_seq * ctx * nq * hd, bytes=2.0 * 2 * n_seq * ctx * nkv * hd)


def profile_decode_e4m3(iters, timer):
    """The decode case over an e4m3 cache: half the cache bytes (+ 8 bytes of scales per token and kv head pair)."""
    n_seq, ctx, nq, nkv, hd = 64, 4096, 32, 8, 128
    q, kc, vc, pt, seq, pos = _paged_case(n_seq, ctx, nq, nkv, hd, 1)
    k8, ks = quant_cache(kc)
    v8, vs = quant_cache(vc)
    sc = torch.cat([ks, vs], dim=-1).contiguous()
    del kc, vc
    ws = AttnWorkspace(n_seq, nq, nkv, hd, ctx, q.device)
    out = torch.empty(n_seq, nq * hd, dtype=BF16, device=q.device)
    us = timer(lambda: attention(q, k8, v8, pt, seq, pos, ws, out=out, kv_scale=sc), iters)
    return dict(us=us, flops=4.0 * n_seq * ctx * nq * hd, bytes=2.0 * n_seq * ctx * nkv * (hd + 4))


def profile_prefill_e4m3(iters, timer):
    ctx, nq, nkv, hd = 4096, 32, 8, 128
    q, kc, vc, pt, seq, pos = _paged_case(1, ctx, nq, nkv, hd, ctx)
    k8, ks = quant_cache(kc)
    v8, vs = quant_cache(vc)
    sc = torch.cat([ks, vs], dim=-1).contiguous()
    ws = AttnWorkspace(ctx, nq, nkv, hd, ctx, q.device, max_splits=1)
    out = torch.empty(ctx, nq * hd, dtype=BF16, device=q.device)
    us = timer(lambda: attention(q, k8, v8, pt, seq, pos, ws, out=out, kv_scale=sc), iters)
    return dict(us=us, flops=4.0 * ctx * ctx / 2 * nq * hd, bytes=2.0 * ctx * nkv * (hd + 4) + 2.0 * 2 * ctx * nq * hd)


def profile_prefill(iters, timer):
    ctx, nq, nkv, hd = 4096, 32, 8, 128
    q, kc, vc, pt, seq, pos = _paged_case(1, ctx, nq, nkv, hd, ctx)
    ws = AttnWorkspace(ctx, nq, nkv, hd, ctx, q.device, max_splits=1)
    out = torch.empty(ctx, nq * hd, dtype=BF16, device=q.device)
    us = timer(lambda: attention(q, kc, vc, pt, seq, pos, ws, out=out), iters)
    return dict(us=us, flops=4.0 * ctx * ctx / 2 * nq * hd, bytes=2.0 * (2 * ctx * nkv * hd + 2 * ctx * nq * hd))
