"""Analytical cost model: bytes, FLOPs and a roofline time per lowered op.

Used by the rewriter (is a fusion worth it), the scheduler (how to cut an op into slices and
balance them over compute units), the runtime planner (decode-rung admission, prefill chunk
sizing) and the bench tools (achieved / roofline).  Reference counterpart: crates/costmodel
(cost.rs, roofline.rs, mma.rs) and the M/D/1 service table of crates/plowrt/src/sched/mdq.rs.
"""
from __future__ import annotations

from dataclasses import dataclass

from .hwspec import GpuSpec

_BYTES = {"f32": 4, "bf16": 2, "f16": 2, "e4m3": 1, "fp8": 1, "i32": 4, "u8": 1, "i64": 8}


def dtype_bytes(dt: str) -> int:
    return _BYTES[dt]


@dataclass
class OpCost:
    flops: float = 0.0
    bytes: float = 0.0
    link_bytes: float = 0.0     # bytes that must cross NVLink (per GPU, one direction)
    launches: int = 1

    def time_us(self, hw: GpuSpec, dtype: str = "bf16", sustained: bool = True) -> float:
        bw, _ = hw.hbm_peak()
        tf, _ = hw.bf16_peak(sustained)
        if dtype in ("e4m3", "fp8"):
            tf *= 2.0
        t_mem = self.bytes / (bw * 1e3)            # GB/s -> bytes/us
        t_cmp = self.flops / (tf * 1e6)            # TFLOP/s -> flop/us
        t_lnk = self.link_bytes / (770.0 * 1e3)    # measured peer-copy bandwidth per direction
        return max(t_mem, t_cmp, t_lnk) + 2.0 * self.launches * 0.0  # launch latency hidden by graphs

    def bound(self, hw: GpuSpec, dtype: str = "bf16") -> str:
        bw, _ = hw.hbm_peak()
        tf, _ = hw.bf16_peak(True)
        if dtype in ("e4m3", "fp8"):
            tf *= 2.0
        t = {"memory": self.bytes / (bw * 1e3), "compute": self.flops / (tf * 1e6),
             "link": self.link_bytes / (770.0 * 1e3)}
        return max(t, key=t.get)


def gemm_cost(m: int, n: int, k: int, in_bytes: int = 2, out_bytes: int = 2) -> OpCost:
    return OpCost(flops=2.0 * m * n * k, bytes=float(m * k * in_bytes + n * k * in_bytes + m * n * out_bytes))


def attention_decode_cost(batch_kv_tokens: int, heads: int, kv_heads: int, hd_qk: int, hd_v: int,
                          kv_bytes: int = 2) -> OpCost:
    return OpCost(flops=2.0 * batch_kv_tokens * heads * (hd_qk + hd_v),
                  bytes=float(batch_kv_tokens * kv_heads * (hd_qk + hd_v) * kv_bytes))


def attention_prefill_cost(rows: int, ctx: int, heads: int, hd_qk: int, hd_v: int) -> OpCost:
    return OpCost(flops=2.0 * rows * ctx * heads * (hd_qk + hd_v) * 0.5,
                  bytes=float(2 * rows * heads * (hd_qk + hd_v)))


def rowwise_cost(rows: int, width: int, n_streams: int = 2, es: int = 2) -> OpCost:
    return OpCost(flops=4.0 * rows * width, bytes=float(rows * width * es * n_streams))


def allreduce_cost(rows: int, width: int, n_ranks: int, es: int = 2, one_shot: bool = True) -> OpCost:
    msg = rows * width * es
    link = (n_ranks - 1) * msg if one_shot else 2.0 * (n_ranks - 1) / n_ranks * msg
    return OpCost(flops=float(rows * width * n_ranks), bytes=float(msg * (n_ranks + 1)), link_bytes=float(link))


def pick_gemm_tile(m: int, n: int, fp8: bool, dual: bool) -> dict:
    """Orientation and UMMA N tile for a [m, k] x [n, k]^T product on tcgen05.

    m <= 128: weights ride the 128 TMEM lanes (swap) and the token tile is the smallest of
    32/64/128 that covers m, so each weight byte is read once.  Larger m: tokens on the lanes,
    256-wide feature tiles for bf16 (TMEM holds 2 x 256 fp32 columns), 128 for block-scaled fp8
    (the promotion registers bound the tile), halved when gate and up share a tile."""
    if m <= 128:
        cap = 64 if (fp8 and dual) else 128
        bn = next((b for b in (32, 64, 128) if m <= b and b <= cap), cap)
        return dict(swap=True, bn=bn)
    if fp8:
        return dict(swap=False, bn=64 if dual else 128)
    return dict(swap=False, bn=128 if dual else (256 if n >= 2048 else 128))


def decode_step_floor_us(spec, hw: GpuSpec, batch: int, mean_ctx: int, ep: int = 1, tp: int = 1) -> float:
    """Weight-stream + KV-stream floor of one decode step on one GPU (the reference certifies the
    same kind of lower bound: critical path + weight-stream floor, crates/plowc/src/main.rs:2045-2093)."""
    wbytes = 1 if spec.weight_quant != "none" else dtype_bytes(spec.dtype)
    total = 0.0
    h = spec.hidden
    for l in spec.layers:
        a, f = l.attn, l.ffn
        if a.kind == "gqa":
            total += wbytes * h * (a.n_heads + 2 * a.n_kv_heads + a.n_heads) * a.head_dim / tp
        elif a.kind == "mla":
            qh = a.qk_nope + a.qk_rope
            total += wbytes * ((h * a.q_lora + a.q_lora * a.n_heads * qh / tp) if a.q_lora else h * a.n_heads * qh / tp)
            total += wbytes * (h * (a.kv_lora + a.qk_rope) + a.kv_lora * a.n_heads * (a.qk_nope + a.v_head) / tp
                               + a.n_heads * a.v_head * h / tp)
        elif a.kind in ("gdn", "kda"):
            total += wbytes * h * (2 * a.gdn_k_heads + 3 * a.gdn_v_heads) * a.gdn_head_dim / tp
        if f.kind == "dense":
            total += wbytes * 3 * h * f.inter / tp
        else:
            hit = min(f.n_experts // ep, batch * ep * f.top_k)   # experts touched on this rank
            total += wbytes * 3 * h * f.moe_inter * (hit + f.n_shared)
    total += 2 * spec.vocab * h / tp                       # lm_head (bf16)
    total += spec.kv_bytes_per_token() * batch * mean_ctx  # KV stream
    bw, _ = hw.hbm_peak()
    return total / (bw * 1e3)
