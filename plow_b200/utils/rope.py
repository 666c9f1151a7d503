"""RoPE tables: computed in float64 and rounded once to float32.

Row layout ``[cos(rot/2) | sin(rot/2)]`` per position, so kernels read one contiguous row per
token.  Partial rotary is expressed by ``rot_dim < head_dim`` (dims beyond rot_dim pass through).
Scaling variants: ``linear``, ``llama3`` (piecewise wavelength remap) and ``yarn`` (NTK-by-parts
with attention factor folded into cos/sin).  Reference counterpart: crates/packet/src/rope.rs
(f64 generator incl. Llama-3 / YaRN), runtime/common/dev_blob.h:130-163.
"""
from __future__ import annotations

import math

import numpy as np


def inv_freq(theta: float, rot_dim: int, scaling: dict | None) -> tuple:
    half = rot_dim // 2
    f = 1.0 / (np.float64(theta) ** (np.arange(0, half, dtype=np.float64) * 2.0 / rot_dim))
    att = 1.0
    if not scaling:
        return f, att
    typ = scaling.get("type") or scaling.get("rope_type")
    factor = float(scaling.get("factor", 1.0))
    if typ == "nope":                                   # no rotary embedding: every angle is zero, the rotation is the identity
        f = f * 0.0
    elif typ == "linear":
        f = f / factor
    elif typ == "llama3":
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        orig = float(scaling.get("original_max_position_embeddings", 8192))
        wl = 2.0 * math.pi / f
        smooth = np.clip((orig / wl - lo) / (hi - lo), 0.0, 1.0)
        scaled = (1.0 - smooth) * f / factor + smooth * f
        f = np.where(wl < orig / hi, f, np.where(wl > orig / lo, f / factor, scaled))
    elif typ == "yarn":
        orig = float(scaling.get("original_max_position_embeddings", 4096))
        beta_fast = float(scaling.get("beta_fast", 32.0))
        beta_slow = float(scaling.get("beta_slow", 1.0))

        def corr_dim(n_rot):
            return rot_dim * math.log(orig / (n_rot * 2.0 * math.pi)) / (2.0 * math.log(theta))

        lo_f, hi_f = corr_dim(beta_fast), corr_dim(beta_slow)
        if scaling.get("truncate", True):           # gpt_oss sets truncate = false: the ramp's ends stay fractional
            lo_f, hi_f = math.floor(lo_f), math.ceil(hi_f)
        low = max(lo_f, 0)
        high = min(hi_f, half - 1)
        ramp = np.clip((np.arange(half, dtype=np.float64) - low) / max(high - low, 1e-3), 0.0, 1.0)
        mask = 1.0 - ramp
        f = f / factor * (1.0 - mask) + f * mask
        ms = float(scaling.get("mscale", 1.0))
        msa = float(scaling.get("mscale_all_dim", 0.0))

        def mscale(s, m):
            return 1.0 if s <= 1.0 else 0.1 * m * math.log(s) + 1.0

        att = float(scaling.get("attention_factor") or (mscale(factor, ms) / mscale(factor, msa) if msa else mscale(factor, ms)))
    else:
        raise ValueError(f"unknown rope scaling '{typ}'")
    return f, att


def rope_table(max_pos: int, rot_dim: int, theta: float, scaling: dict | None = None) -> np.ndarray:
    """float32 [max_pos, rot_dim]: cos in the first half of each row, sin in the second."""
    rot_dim = max(2, rot_dim)
    f, att = inv_freq(theta, rot_dim, scaling)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * f[None, :]
    return np.concatenate([np.cos(ang) * att, np.sin(ang) * att], axis=1).astype(np.float32)


def mla_softmax_factor(scaling: dict | None) -> float:
    """What multi-head latent attention multiplies its softmax scale by under YaRN: mscale(factor, mscale_all_dim)^2.
    The rotary table itself carries mscale(factor, mscale) / mscale(factor, mscale_all_dim) (1 when the two are equal),
    so without this factor a YaRN-extended checkpoint attends with logits about half as large as it was trained with."""
    if not scaling or (scaling.get("type") or scaling.get("rope_type")) != "yarn":
        return 1.0
    factor, msa = float(scaling.get("factor", 1.0)), float(scaling.get("mscale_all_dim") or 0.0)
    if factor <= 1.0 or msa == 0.0:
        return 1.0
    m = 0.1 * msa * math.log(factor) + 1.0
    return m * m
