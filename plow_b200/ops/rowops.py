"""Python front ends of the row-wise kernels in ``csrc/cuda/rowops.cu`` (see that file for the
semantics and the reference counterparts)."""
from __future__ import annotations

import torch

from . import native

BF16, FP8 = torch.bfloat16, torch.float8_e4m3fn


def embed(table, ids, scale=1.0):
    out = torch.empty(ids.shape[0], table.shape[1], dtype=BF16, device=table.device)
    native.call("plow_embed", out, table, ids, ids.shape[0], table.shape[1], float(scale))
    return out


def _quant_bufs(R, W, dev, ld):
    ld = ld or R
    return torch.empty(R, W, dtype=FP8, device=dev), torch.empty(W // 128, ld, dtype=torch.float32, device=dev), ld


def rmsnorm(x, gamma, eps, plus_one=False, width=None, col_ofs=0, want_bf16=True, want_fp8=False, ld_sx=None):
    """RMSNorm over `width` columns starting at `col_ofs` of a (possibly wider) row.
    Returns (h bf16 | None, xq e4m3 | None, sx transposed | None)."""
    R = x.shape[0]
    W = width or x.shape[1]
    h = torch.empty(R, W, dtype=BF16, device=x.device) if want_bf16 else None
    xq = sx = None
    ld = 0
    if want_fp8:
        xq, sx, ld = _quant_bufs(R, W, x.device, ld_sx)
    xin = x if col_ofs == 0 else x[:, col_ofs:]
    native.call("plow_rmsnorm", h, xq, sx, ld, xin, gamma, R, W, x.stride(0), float(eps), int(plus_one))
    return h, xq, sx


def add_norm(x, delta, gamma, eps, plus_one=False, want_bf16=True, want_fp8=False, ld_sx=None):
    """x_out = bf16(x + delta); h = RMSNorm(x_out).  Returns (x_out, h | None, xq | None, sx | None)."""
    R, W = x.shape
    x_out = torch.empty_like(x)
    h = torch.empty(R, W, dtype=BF16, device=x.device) if want_bf16 else None
    xq = sx = None
    ld = 0
    if want_fp8:
        xq, sx, ld = _quant_bufs(R, W, x.device, ld_sx)
    native.call("plow_add_norm", h, xq, sx, ld, x_out, x, delta, gamma, R, W, float(eps), int(plus_one))
    return x_out, h, xq, sx


def quant_act(x, ld_sx=None):
    R, K = x.shape
    xq, sx, ld = _quant_bufs(R, K, x.device, ld_sx)
    native.call("plow_quant_act", xq, sx, ld, x, R, K, x.stride(0))
    return xq, sx


def router_topk(logits, bias, k, n_group=1, topk_group=1, sigmoid=True, norm_topk=True, route_scale=1.0):
    """Returns table int32 [T, k, 2]: (expert id, gate as float bits)."""
    T, E = logits.shape
    table = torch.empty(T, k, 2, dtype=torch.int32, device=logits.device)
    native.call("plow_router_topk", table, logits, bias, T, E, k, n_group, topk_group, int(sigmoid), int(norm_topk),
                float(route_scale))
    return table


def table_gates(table):
    return table[..., 1].contiguous().view(torch.float32)


def moe_align(table, e_base, e_local, shared_rows=0, shared_tok_base=0):
    """Expert-sorted row layout of the pairs routed to experts [e_base, e_base + e_local).  ``shared_rows`` > 0 appends
    one more group (index e_local) holding tokens [shared_tok_base, shared_tok_base + shared_rows): the shared expert
    stacked behind the routed ones; grp_off / tile_prefix then have e_local + 2 entries."""
    n_pairs = table.shape[0] * table.shape[1]
    dev = table.device
    ng = e_local + (1 if shared_rows else 0)
    grp_off = torch.empty(ng + 1, dtype=torch.int32, device=dev)
    tile_prefix = torch.empty(ng + 1, dtype=torch.int32, device=dev)
    row_of_pair = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    pair_of_row = torch.empty(n_pairs + shared_rows, dtype=torch.int32, device=dev)
    native.call("plow_moe_align", table, n_pairs, e_base, e_local, grp_off, tile_prefix, row_of_pair, pair_of_row,
                int(shared_rows), int(shared_tok_base), table.shape[1])
    return grp_off, tile_prefix, row_of_pair, pair_of_row


def moe_gather(xq, sx, pair_of_row, n_rows_dev, max_rows, top_k):
    K = xq.shape[1]
    xs = torch.empty(max_rows, K, dtype=FP8, device=xq.device)
    sxs = torch.empty(K // 128, max_rows, dtype=torch.float32, device=xq.device)
    native.call("plow_moe_gather", xs, sxs, max_rows, xq, sx, sx.stride(0), pair_of_row, n_rows_dev, max_rows, top_k, K)
    return xs, sxs


def moe_combine(y, shared, table, row_of_pair, T, H, shared_base=None, out=None):
    """``shared_base`` (int32 device scalar): the shared expert's rows start at y-row ``*shared_base`` of ``shared``."""
    if out is None:
        out = torch.empty(T, H, dtype=BF16, device=y.device)
    native.call("plow_moe_combine", out, y, shared, table, row_of_pair, T, table.shape[1], H, shared_base)
    return out


def argmax(logits):
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    native.call("plow_argmax", out, logits, R, V)
    return out


def row_gather(x, rows):
    out = torch.empty(rows.shape[0], x.shape[1], dtype=BF16, device=x.device)
    native.call("plow_row_gather", out, x, rows, rows.shape[0], x.shape[1])
    return out


def head_to_token(x, T, heads, W):
    out = torch.empty(T, heads * W, dtype=BF16, device=x.device)
    native.call("plow_head_to_token", out, x, T, heads, W)
    return out
