"""Small, self-contained launches of the hot kernels for timing and for profiler captures.

    python -m plow_b200.ops.profile_cases <case> [--iters N]

Each case holds a few GB on the device at most, streams more than the 126 MB L2 per launch, runs
three warm-up launches and then ``--iters`` timed launches (CUDA events on the launching stream) and
prints one JSON line with the mean time, the algorithmic bytes / FLOPs and the achieved rates.  The
cases are small enough for a multi-pass profiler capture of one kernel to end by itself.

Cases
    gemm_bf16        8192 x 8192 x 8192 bf16 (BN=256 tile, persistent)
    gemm_fp8         8192 x 7168 x 8192 block-scaled e4m3
    gemm_fp8_swap    64 x 24576 x 7168 block-scaled e4m3, swap-AB decode shape
    gemm_moe         32 experts x (4096 -> 2x2048) grouped SwiGLU, 16 rows per expert
    mla_decode       74 requests x 4096 cached tokens, 128 heads, e4m3 latent cache
    gqa_decode       64 requests x 4096 cached tokens, 32/8 heads, hd128 bf16 paged cache
    gqa_decode_e4m3  the same over an e4m3 cache with per-cell scales
    gqa_prefill      one 4096-token prompt, 32/8 heads, hd128
    gqa_prefill_e4m3 the same over an e4m3 cache
    dsa_topk         64 rows x 32768 scores, exact top-2048
"""
from __future__ import annotations

import argparse
import json
import math

import torch

FP8 = torch.float8_e4m3fn


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / iters      # µs


def case_gemm_bf16(iters):
    from . import gemm
    M = N = K = 8192
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    us = _time(lambda: gemm.gemm(x, w), iters)
    return dict(us=us, flops=2.0 * M * N * K, bytes=2.0 * (M * K + N * K + M * N))


def case_gemm_fp8(iters):
    from . import gemm
    M, N, K = 8192, 7168, 8192
    x = torch.randn(M, K, device="cuda").to(FP8)
    w = torch.randn(N, K, device="cuda").to(FP8)
    sx = torch.rand(K // 128, M, device="cuda")
    sw = torch.rand(N // 128, K // 128, device="cuda")
    us = _time(lambda: gemm.gemm(x, w, sx=sx, sw=sw), iters)
    return dict(us=us, flops=2.0 * M * N * K, bytes=1.0 * (M * K + N * K) + 2.0 * M * N)


def case_gemm_fp8_swap(iters):
    from . import gemm
    M, N, K = 64, 24576, 7168
    x = torch.randn(M, K, device="cuda").to(FP8)
    w = torch.randn(N, K, device="cuda").to(FP8)
    sx = torch.rand(K // 128, M, device="cuda")
    sw = torch.rand(N // 128, K // 128, device="cuda")
    us = _time(lambda: gemm.gemm(x, w, sx=sx, sw=sw, swap=True, bn=64), iters)
    return dict(us=us, flops=2.0 * M * N * K, bytes=1.0 * N * K + 1.0 * M * K + 2.0 * M * N)


def case_gemm_moe(iters):
    from . import gemm
    E, H, I, rows = 32, 7168, 2048, 16
    w = torch.randn(E * 2 * I, H, device="cuda").to(FP8)
    sw = torch.rand(E * 2 * I // 128, H // 128, device="cuda")
    R = E * rows
    x = torch.randn(R, H, device="cuda").to(FP8)
    sx = torch.rand(H // 128, R, device="cuda")
    grp_off = (torch.arange(E + 1, dtype=torch.int32) * rows).cuda()
    tile_prefix = torch.arange(E + 1, dtype=torch.int32).cuda()
    us = _time(lambda: gemm.gemm(x, w, sx=sx, sw=sw, dual=True, n_out=I, swap=True, bn=32,
                                 grp_off=grp_off, tile_prefix=tile_prefix, n_experts=E), iters)
    return dict(us=us, flops=2.0 * E * rows * 2 * I * H, bytes=1.0 * E * 2 * I * H)


def case_gemm_fp8_dual_prefill(iters):
    """Dense SwiGLU up-projection of a 2048-row prefill chunk (7168 -> 2 x 18432), non-swap tiles."""
    from . import gemm
    M, N, K = 2048, 18432, 7168
    x = torch.randn(M, K, device="cuda").to(FP8)
    w = torch.randn(2 * N, K, device="cuda").to(FP8)
    sx = torch.rand(K // 128, M, device="cuda")
    sw = torch.rand(2 * N // 128, K // 128, device="cuda")
    us = _time(lambda: gemm.gemm(x, w, sx=sx, sw=sw, dual=True, n_out=N, swap=False), iters)
    return dict(us=us, flops=2.0 * M * 2 * N * K, bytes=1.0 * (M * K + 2 * N * K) + 2.0 * M * N)


def case_gemm_moe_prefill(iters):
    """Grouped SwiGLU GEMM of a 2048-token prefill chunk: 32 experts + the shared expert as a 33rd group, top-8 routing
    drawn uniformly (rows per expert vary around 512), non-swap 128-row token tiles."""
    from . import gemm
    E, H, I, T, k = 33, 7168, 2048, 2048, 8
    g = torch.Generator().manual_seed(0)
    counts = torch.bincount(torch.randint(0, 32, (T * k,), generator=g), minlength=32).tolist() + [T]
    off = [0]
    tiles = [0]
    for c in counts:
        off.append(off[-1] + c)
        tiles.append(tiles[-1] + (c + 127) // 128)
    R = off[-1]
    w = torch.randn(E * 2 * I, H, device="cuda").to(FP8)
    sw = torch.rand(E * 2 * I // 128, H // 128, device="cuda")
    x = torch.randn(R, H, device="cuda").to(FP8)
    sx = torch.rand(H // 128, R, device="cuda")
    grp_off = torch.tensor(off, dtype=torch.int32).cuda()
    tile_prefix = torch.tensor(tiles, dtype=torch.int32).cuda()
    us = _time(lambda: gemm.gemm(x, w, sx=sx, sw=sw, dual=True, n_out=I, swap=False, rows_hint=512,
                                 grp_off=grp_off, tile_prefix=tile_prefix, n_experts=E), iters)
    return dict(us=us, flops=2.0 * R * 2 * I * H, bytes=1.0 * E * 2 * I * H + 1.0 * R * H + 2.0 * R * I)


def case_mla_prefill(iters):
    """Materialised MLA prefill attention: one request, 2048 new rows after a 2048-token cached prefix, 128 heads,
    192-wide keys / 128-wide values (K / V already rebuilt)."""
    import math
    from . import mla
    T, L, H = 2048, 4096, 128
    ws = mla.PrefillWorkspace(L, T, 2, L // 64, device="cuda")
    ws.kvb.copy_(torch.randn(L, H * 256, device="cuda") * 0.5)
    ws.krope.copy_(torch.randn(L, 64, device="cuda") * 0.5)
    ws.vpt[1] = torch.arange(L // 64, dtype=torch.int32, device="cuda")
    q = (torch.randn(T, H * 192, device="cuda") * 0.5).bfloat16()
    seq = torch.ones(T, dtype=torch.int32, device="cuda")
    pos = torch.arange(L - T, L, dtype=torch.int32, device="cuda")
    out = torch.empty(T, H * 128, dtype=torch.bfloat16, device="cuda")
    us = _time(lambda: mla.prefill_attention(q, ws, L, seq, pos, 1.0 / math.sqrt(192), out), iters)
    pairs = T * (L - T) + T * (T + 1) / 2                   # attended (query, key) pairs per head
    return dict(us=us, flops=2.0 * H * pairs * (192 + 128), bytes=2.0 * (T * H * 192 + L * H * 256 + T * H * 128))


def case_mla_decode(iters):
    from . import mla
    T, ctx = 74, 4096
    n_pages = T * (ctx // 64) + 2
    kv8 = torch.randn(n_pages, 64, 576, device="cuda").to(FP8)
    ksc = torch.rand(n_pages, 64, device="cuda") * 0.01 + 0.005
    pt = torch.arange(T * (ctx // 64), dtype=torch.int32, device="cuda").view(T, -1)
    pt = torch.cat([pt, torch.zeros(T, 1, dtype=torch.int32, device="cuda")], 1).contiguous()
    q8 = torch.randn(128, T, 576, device="cuda").to(FP8)
    sq = torch.rand(128, T, device="cuda") * 0.01
    kvlen = torch.full((T,), ctx, dtype=torch.int32, device="cuda")
    slot_of = torch.arange(T, dtype=torch.int32, device="cuda")
    smax = torch.zeros(n_pages, 4, device="cuda")
    smax[:, 0] = ksc.amax(1)
    ws = mla.DecodeWorkspace(T, ctx + 64, tiles_per_split=64)
    out = torch.empty(128, T, 512, dtype=torch.bfloat16, device="cuda")
    us = _time(lambda: mla.decode(q8, sq, kv8, ksc, smax, pt, slot_of, kvlen, ws, 1 / math.sqrt(192), out=out), iters)
    return dict(us=us, flops=2.0 * T * ctx * 128 * (576 + 512), bytes=1.0 * T * ctx * 580)


def case_gqa_decode(iters):
    from . import gqa
    return gqa.profile_decode(iters, _time)


def case_gqa_decode_e4m3(iters):
    from . import gqa
    return gqa.profile_decode_e4m3(iters, _time)


def case_gqa_prefill_e4m3(iters):
    from . import gqa
    return gqa.profile_prefill_e4m3(iters, _time)


def case_gqa_prefill(iters):
    from . import gqa
    return gqa.profile_prefill(iters, _time)


def case_dsa_topk(iters):
    from . import dsa
    return dsa.profile_topk(iters, _time)


CASES = {k[5:]: v for k, v in list(globals().items()) if k.startswith("case_")}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    from . import native
    r = CASES[a.case](a.iters)
    native.check_status()
    r["case"] = a.case
    r["tflops"] = round(r["flops"] / r["us"] / 1e6, 1)
    r["gbs"] = round(r["bytes"] / r["us"] / 1e3, 1)
    r["us"] = round(r["us"], 2)
    print(json.dumps(r))


if __name__ == "__main__":
    main()
