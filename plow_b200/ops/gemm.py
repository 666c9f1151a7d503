"""tcgen05 GEMM family: Python front end of ``plow_gemm`` (csrc/cuda/gemm_api.h).

``linear`` picks the orientation from the row count: up to 128 rows the weights ride the
TMEM lanes (``swap``) and the rows become the UMMA N dimension, so a decode step streams each
weight tile exactly once at full tensor-core tile efficiency; larger row counts put tokens on
the lanes.  The reference makes the same split between its GEMV family (M <= 8..128 rows) and
its tiled prefill GEMM (runtime/nvidia/op_gemm.cuh:76, op_gemv_wide_sm90.cuh).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native

_BF16, _FP8 = 0, 1


def _ptr(t):
    return None if t is None else t.data_ptr()


def _pick_bn_swap(rows: int, fp8: bool, dual: bool) -> int:
    cap = 64 if (fp8 and dual) else 128
    for bn in (32, 64, 128):
        if rows <= bn and bn <= cap:
            return bn
    return cap


import os as _os

_STREAM_DEFAULT = _os.environ.get("PLOW_GEMM_STREAM", "1") != "0"
_WIDE_DEFAULT = _os.environ.get("PLOW_GEMM_WIDE", "1") != "0"
_SPLITK_WS = {}
SM_COUNT = 148          # B200; used only where no device is present (the device's own count is read otherwise)


_TUNED = {}


def _tuned(M, N, K, fp8, dual):
    """Measured (bn, splits) for a dense swap-mode shape from the tuning store, or None."""
    if "db" not in _TUNED:
        try:
            from ..compiler.tunedb import TuneDb
            db = TuneDb()
            _TUNED["db"] = db if db.root.exists() else None
        except Exception:
            _TUNED["db"] = None
    db = _TUNED["db"]
    if db is None:
        return None
    from ..compiler.tunedb import gemm_key
    rec = db.lookup("gemm", gemm_key(M, N, K, "e4m3" if fp8 else "bf16", dual))
    return rec["config"] if rec else None


def _splitk_ws(device):
    """fp32 partial workspace + self-resetting per-tile counters, one pair per device."""
    if device not in _SPLITK_WS:
        _SPLITK_WS[device] = (torch.empty(16 << 20, dtype=torch.float32, device=device),
                              torch.zeros(512 * 32, dtype=torch.int32, device=device))
    return _SPLITK_WS[device]


def reset_workspace(device) -> None:
    """Zero the split-K arrival counters of `device` (the kernels re-arm them only when a launch finishes cleanly)."""
    import torch as _t
    dev = _t.device(device)
    if dev in _SPLITK_WS:
        _SPLITK_WS[dev][1].zero_()


def sm_count(device=None) -> int:
    import torch as _t
    if not _t.cuda.is_available():
        return SM_COUNT
    return _t.cuda.get_device_properties(device if device is not None else _t.cuda.current_device()).multi_processor_count


def pick_splits(M, N, K, fp8, dual, bn) -> int:
    """Split-K factor for a dense swap-mode GEMM: fill the SMs when the tile count alone cannot.

    A swap-mode tile is 128 weight rows; a projection with fewer than 148 tiles leaves SMs idle while every
    busy SM is limited by its own load rate, so the K range of each tile is cut over ``s`` CTAs (all resident
    at once: tiles * s <= SM count) that reduce their partials through L2."""
    tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
    kb = (K + (127 if fp8 else 63)) // (128 if fp8 else 64)
    s = min(sm_count() // max(tiles, 1), kb // 4, bn // 4, 16)
    if s < 2:
        return 1
    acc = bn * (2 if dual else 1)
    if tiles * s * acc * 128 > (16 << 20) or tiles > 256:
        return 1
    return s


def gemm(x, w, *, sx=None, sw=None, out=None, residual=None, dual=False, n_out=None,
         grp_off=None, tile_prefix=None, n_experts=0, swap=None, bn=None, out_f32=False,
         out_scale=1.0, quant_out=False, rows_hint=None, ld_syq=None, wait=None, yq_out=None, syq_out=None, splits=None, ar=None,
         stream=None):
    """y = x @ w.T with the epilogue options of the kernel.

    x [M, K] bf16 or e4m3; w [(E*)N(*2), K] same dtype.  ``dual`` computes silu(gate)*up with
    w = [gate; up] stacked per expert.  Grouped mode (``n_experts`` > 0): rows of x are sorted
    by expert and ``grp_off`` [E+1] int32 (device) gives the ranges.  ``quant_out`` returns
    (yq e4m3, syq transposed scales) instead of bf16.  ``rows_hint``: expected rows per expert
    used to pick the token tile in grouped swap mode.  ``wait`` = (counter ptr, epoch ptr, multiplier,
    deadline ms): the kernel starts reading x once ``*counter >= *epoch * multiplier`` (rows written by
    peer GPUs during expert-parallel dispatch).  ``ar``: fuse the tensor-parallel all-reduce of the
    result into the kernel (see plow_b200/parallel/tp.py).  ``stream`` (swap mode; default on unless ``splits`` is
    given or PLOW_GEMM_STREAM=0): stream scheduling, every CTA runs the same number of K blocks and tiles whose K range
    is shared between CTAs are finished through fp32 partials in the workspace.
    """
    lib = native.cuda_lib()
    assert x.is_cuda and w.is_cuda and x.dim() == 2 and w.dim() == 2
    fp8 = x.dtype == torch.float8_e4m3fn
    assert w.dtype == x.dtype and (fp8 or x.dtype == torch.bfloat16)
    M, K = x.shape
    w_rows = w.shape[0]
    E = int(n_experts)
    if n_out is None:
        n_out = w_rows // (max(E, 1) * (2 if dual else 1))
    N = int(n_out)
    if swap is None:
        per = rows_hint if rows_hint is not None else M
        swap = per <= 128
    if swap and E == 0 and bn is None and splits is None and ar is None:
        cfg = _tuned(M, N, K, fp8, dual)
        if cfg and cfg.get("swap", True) and cfg["bn"] >= M:
            bn, splits = cfg["bn"], cfg.get("splits", 1)
    if fp8 and not swap and dual and _WIDE_DEFAULT and N % 128 == 0 and (bn is None or bn == 64):
        # large-M SwiGLU tiles: gate | up of 128 columns each (one N = 256 MMA, 256 TMEM columns per partial).  Measured
        # on the 2048-token prefill shapes: the grouped up-projection runs 1.2x faster than with 64 + 64 columns (fewer
        # operand bytes per FLOP through L2); the plain projections gain nothing from 256-wide tiles (fewer, longer tiles
        # leave the last wave of CTAs emptier) and keep 128.
        bn = 128
    if bn is None:
        if swap:
            bn = _pick_bn_swap(rows_hint if rows_hint is not None else M, fp8, dual)
        else:
            bn = (64 if dual else 128) if fp8 else (128 if dual else (256 if N >= 2048 else 128))
    y = yq = syq = None
    if quant_out:
        yq = yq_out if yq_out is not None else torch.empty(M, N, dtype=torch.float8_e4m3fn, device=x.device)
        ld_syq = ld_syq or M
        syq = syq_out if syq_out is not None else torch.empty((N + 127) // 128, ld_syq, dtype=torch.float32, device=x.device)
    else:
        y = out if out is not None else torch.empty(
            M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    ws = ws_ctr = None
    if ar is not None:
        splits = 1
    if stream is None:
        stream = bool(swap) and ar is None and splits is None and _STREAM_DEFAULT
        if stream and E == 0:
            # dense: worth it when the tile count is within a factor of a few of the SM count (a tile is then shared
            # by at most ~3 CTAs) and every CTA still gets a decent run of K blocks; few-tile problems keep the
            # split-K form, whose reduction is spread over the splits
            units = ((N + 127) // 128) * ((M + bn - 1) // bn)
            kb = (K + (127 if fp8 else 63)) // (128 if fp8 else 64)
            sms = sm_count(x.device)
            stream = units * 3 >= sms and units * kb >= 16 * sms
    stream = bool(stream) and bool(swap) and ar is None
    if stream:
        splits = 1
        ws, ws_ctr = _splitk_ws(x.device)
    elif swap and E == 0:
        if splits is None:
            splits = pick_splits(M, N, K, fp8, dual, bn)
        if splits > 1:
            ws, ws_ctr = _splitk_ws(x.device)
    else:
        splits = 1
    status = native.status_word(x.device)
    d = native.GemmDesc(
        x=_ptr(x), w=_ptr(w), y=_ptr(y), sx=_ptr(sx), sw=_ptr(sw), residual=_ptr(residual),
        yq=_ptr(yq), syq=_ptr(syq), grp_off=_ptr(grp_off), tile_prefix=_ptr(tile_prefix),
        status=status.data_ptr(), M=M, N=N, K=K, ldx=x.stride(0), ldw=w.stride(0), ldy=N,
        ld_sx=(sx.stride(0) if sx is not None else 0), ld_syq=(ld_syq or 0), E=E, w_rows=w_rows,
        dtype=_FP8 if fp8 else _BF16, dual=int(dual), swap=int(swap), bn=int(bn),
        out_f32=int(out_f32), out_scale=float(out_scale),
        ws=_ptr(ws), ws_ctr=_ptr(ws_ctr), splits=int(splits or 1), stream=int(stream),
        wait_ctr=(wait[0] if wait else None), wait_epoch=(wait[1] if wait else None),
        wait_mult=(int(wait[2]) if wait else 0), wait_deadline_ms=(int(wait[3]) if wait else 0))
    native.LAUNCHES["n"] += 1
    if ar is not None:
        # ar: dict(peers=[ptr...], part_ofs, flag_ofs, done_ofs, y_ofs, epoch_ptr, world, me)
        for i, pz in enumerate(ar["peers"]):
            d.ar_peer[i] = pz
        d.ar_part_ofs, d.ar_flag_ofs, d.ar_done_ofs, d.ar_y_ofs = ar["part_ofs"], ar["flag_ofs"], ar["done_ofs"], ar["y_ofs"]
        d.ar_epoch, d.ar_world, d.ar_me = ar["epoch_ptr"], ar["world"], ar["me"]
        d.wait_deadline_ms = ar.get("deadline_ms", 2000)
        d.ar_oneshot, d.ar_half_bytes = int(ar.get("oneshot", 0)), int(ar.get("half_bytes", 0))
        d.ar_mc, d.ar_tdone_ofs = ar.get("mc_ptr") or None, int(ar.get("tdone_ofs", 0))
    if native.PROFILE is not None:
        label = f"gemm M{M} N{N} K{K} E{E} {'fp8' if fp8 else 'bf16'}{' dual' if dual else ''}{' swap' if swap else ''} bn{bn}"
        rc = native.profiled(label, lambda: lib.plow_gemm(C.byref(d), native.stream_ptr()))
    else:
        rc = lib.plow_gemm(C.byref(d), native.stream_ptr())
    if rc != 0:
        raise native.NativeLibraryError(f"plow_gemm failed with code {rc} (bn={bn} swap={swap} dual={dual} fp8={fp8})")
    return (yq, syq) if quant_out else y


def linear(x, w, **kw):
    return gemm(x, w, **kw)
