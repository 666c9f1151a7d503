"""Multi-head latent attention ops: query prep, latent-cache write, absorbed decode.

Decode path (reference op sequence: crates/devgen/src/mla.rs:6211-6323):
  q [T, heads*192] -> q_prep -> (q_nope_t [h][T][128], q_rope [h][T][64])
  q_abs = grouped GEMM(q_nope_t, W_uk^T per head)        [h][T][512]
  q8, sq = q_quant(q_abs, q_rope)                        e4m3 [h][T][576]
  kv_write: RMSNorm(latent) + RoPE(k_rope) -> one e4m3 row + f32 scale per token in the paged cache
  oacc = mla_decode(q8, sq, cache)                       [h][T][512]
  o = grouped GEMM(oacc, W_uv per head) -> [T, heads*128]
"""
from __future__ import annotations

import torch

from . import native

BF16, FP8 = torch.bfloat16, torch.float8_e4m3fn
MAX_SPLITS = 16          # KV splits per request the fold / merge kernels handle (kFoldSplits in csrc/cuda/mla_proj.cu)


def q_prep(q, rope_tab, pos, heads, nope, rope, pair_mode=1):
    T = q.shape[0]
    q_nope_t = torch.empty(heads, T, nope, dtype=BF16, device=q.device)
    q_rope = torch.empty(heads, T, rope, dtype=BF16, device=q.device)
    native.call("plow_mla_q_prep", q_nope_t, q_rope, q, q.stride(0), rope_tab, pos, T, heads, nope, rope, pair_mode)
    return q_nope_t, q_rope


def q_quant(q_abs, q_rope):
    heads, T, latent = q_abs.shape
    rope = q_rope.shape[2]
    q8 = torch.empty(heads, T, latent + rope, dtype=FP8, device=q_abs.device)
    sq = torch.empty(heads, T, dtype=torch.float32, device=q_abs.device)
    native.call("plow_mla_q_quant", q8, sq, q_abs, q_rope, T, heads, latent, rope)
    return q8, sq


def kv_write(kv8, kv_scale, kv_smax, kva, col_ofs, gamma, rope_tab, pos, slot_of, page_table, latent, rope, eps, pair_mode=1):
    T = kva.shape[0]
    native.call("plow_mla_kv_write", kv8, kv_scale, kv_smax, kva, kva.stride(0), col_ofs, gamma, rope_tab, pos, slot_of, page_table,
                page_table.shape[1], T, latent, rope, float(eps), pair_mode)


def absorb(q, wuk_t, rope_tab, pos, heads, pair_mode=1):
    """q [T, heads*192] bf16 -> (q8 e4m3 [heads][T][576], sq [heads][T]): W_uk absorb + RoPE + quantise, one kernel."""
    T = q.shape[0]
    q8 = torch.empty(heads, T, 576, dtype=FP8, device=q.device)
    sq = torch.empty(heads, T, dtype=torch.float32, device=q.device)
    native.call("plow_mla_absorb", q, q.stride(0), wuk_t, rope_tab, pos, q8, sq, T, heads, pair_mode, native.status_word(q.device))
    return q8, sq


def fold(ws, kvlen, wuv, T, heads, ao, want_fp8=False):
    """Merge the decode splits, multiply by W_uv per head, write token-major [T, heads*128] (+ e4m3 twin)."""
    aq = saq = None
    if want_fp8:
        aq = torch.empty(T, heads * 128, dtype=FP8, device=ao.device)
        saq = torch.empty(heads, T, dtype=torch.float32, device=ao.device)
    native.call("plow_mla_fold", ws.opart, ws.lse, kvlen, wuv, ao, aq, saq, T, T, heads, ws.max_splits, ws.tiles_per_split,
                native.status_word(ao.device))
    return aq, saq


class DecodeWorkspace:
    """Scratch of the split-KV decode kernel, sized once for (max rows, max context)."""

    def __init__(self, max_T, max_ctx, tiles_per_split=32, heads=128, latent=512, device="cuda"):
        self.tiles_per_split = tiles_per_split
        self.max_splits = max(1, -(-((max_ctx + 63) // 64) // tiles_per_split))
        self.items = torch.empty(2 * max_T * self.max_splits * 8, dtype=torch.int32, device=device)
        self.n_items = torch.zeros(1, dtype=torch.int32, device=device)
        self.claims = torch.zeros(256, dtype=torch.int32, device=device)    # work counters of the launches that share one list
        self.opart = torch.empty(max_T, self.max_splits, heads, latent, dtype=BF16, device=device)
        self.lse = torch.empty(max_T, self.max_splits, heads, dtype=torch.float32, device=device)


def build_items(kvlen, T, ws: DecodeWorkspace):
    """Work list of the split-KV decode kernel for rows with `kvlen` visible tokens.  It depends on the lengths only, so
    one call serves every layer of a step (pass ``build_items=False`` to :func:`decode`)."""
    native.call("plow_mla_build_items", kvlen, T, ws.tiles_per_split, ws.max_splits, ws.items, ws.n_items, ws.claims)


def decode(q8, sq, kv8, kv_scale, kv_smax, page_table, slot_of, kvlen, ws: DecodeWorkspace, softmax_scale, out=None, merge=True,
           build_items=True, claim_slot=0):
    """q8 [128][T][576] e4m3, sq [128][T]; kv8 [pages][64][576]; kv_smax f32 [pages][4] (element 0 bounds the
    page's scales from above); returns oacc bf16 [128][T][512]."""
    heads, T, _ = q8.shape
    assert heads == 128 and kv8.shape[1:] == (64, 576)
    if out is None and merge:
        out = torch.empty(heads, T, 512, dtype=BF16, device=q8.device)
    native.call("plow_mla_decode", q8, sq, kv8, kv_scale, kv_smax, kv8.shape[0], page_table, page_table.shape[1], slot_of, kvlen, T,
                ws.tiles_per_split, ws.max_splits, ws.items, ws.n_items, ws.opart, ws.lse, out, float(softmax_scale),
                int(build_items), ws.claims, int(claim_slot), native.status_word(q8.device))
    return out


# ---- materialised prefill ---------------------------------------------------------------------------------------
class PrefillWorkspace:
    """Scratch of the materialised prefill: the gathered latent of the step's prefilling requests, the K / V rebuilt
    from it for ONE layer (reused by every layer), the tile table and the attention work list.

    ``budget`` bounds the cached tokens (summed over the requests, each rounded up to 64) a step may rebuild; K / V
    take 64 KiB per token (128 heads x 256 dims bf16).
    """

    def __init__(self, budget, max_rows, n_slots, max_pages, heads=128, latent=512, rope=64, fp8_weight=True, device="cuda"):
        self.budget, self.max_rows, self.heads, self.latent, self.rope = budget, max_rows, heads, latent, rope
        self.fp8 = fp8_weight
        if fp8_weight:
            self.lat8 = torch.zeros(budget, latent + rope, dtype=FP8, device=device)
            self.lat_scale = torch.zeros(latent // 128, budget, dtype=torch.float32, device=device)
            self.lat16 = None
        else:
            self.lat8 = self.lat_scale = None
            self.lat16 = torch.zeros(budget, latent, dtype=BF16, device=device)
        self.krope = torch.zeros(budget, rope, dtype=BF16, device=device)
        self.kvb = torch.empty(budget, heads * 256, dtype=BF16, device=device)
        self.vpt = torch.zeros(n_slots, max_pages, dtype=torch.int32, device=device)
        chunks = (max_rows + 127) // 128 + n_slots
        # one (128-row chunk, head) item per CTA visit: with 128 heads even a single chunk fills the GPU, so the keys of
        # a chunk are never split
        self.tiles_per_split = 1 << 20
        self.max_splits = 1
        self.item_cap = chunks * heads * self.max_splits
        self.items = torch.empty(self.item_cap * 8, dtype=torch.int32, device=device)
        self.n_items = torch.zeros(1, dtype=torch.int32, device=device)
        self.row_ns = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.opart = self.lse = None


def latent_gather(ws: PrefillWorkspace, cache, scale, page_table, spans, n_spans, max_tiles):
    """cache e4m3 [pages, 64, latent+rope]; scale f32 [pages, 64]; spans int32 [>= n_spans, 4] (device)."""
    native.call("plow_mla_latent_gather", ws.lat8, ws.lat_scale, ws.budget, ws.lat16, ws.krope, ws.vpt, cache, scale, page_table,
                page_table.shape[1], spans, int(n_spans), int(max_tiles), ws.latent, ws.rope)


def q_rope(q, rope_tab, pos, heads, nope, rope, pair_mode=1):
    """Rotate the rotary part of every head of q [T, heads*(nope+rope)] in place (rows with pos < 0 untouched)."""
    native.call("plow_mla_q_rope", q, q.stride(0), rope_tab, pos, q.shape[0], heads, nope, rope, pair_mode)


def prefill_attention(q, ws: PrefillWorkspace, n_tokens, seq, pos, softmax_scale, out):
    """q [T, heads*192] bf16 (rotated); K / V from ws.kvb / ws.krope rows [0, n_tokens); out [T, heads*128] bf16.  Rows
    with pos < 0 are skipped (their rows of ``out`` are not written)."""
    T = q.shape[0]
    assert T <= ws.max_rows and n_tokens <= ws.budget
    native.call("plow_mla_prefill_attention", q, ws.kvb, ws.krope, int(n_tokens), ws.vpt, ws.vpt.shape[1], seq, pos, T, ws.heads,
                ws.tiles_per_split, ws.max_splits, ws.items, ws.item_cap, ws.n_items, ws.row_ns, ws.opart, ws.lse, out,
                float(softmax_scale), native.status_word(q.device))
    return out
