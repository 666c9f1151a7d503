"""Block-scaled e4m3 quantisation (PyTorch reference forms).

Weights: 128x128 blocks, ``W_f32[n][k] = e4m3(Wq)[n][k] * S[n >> 7][k >> 7]``.
Activations: 1x128 groups along K, ``s = max(amax, 1e-10) / 448``; the scale tensor is kept
transposed ``[ceil(K/128), rows]`` so a GEMM tile reads the scales of consecutive rows with one
coalesced load.  Same conventions as the reference (runtime/nvidia/quant_group.cuh:1-4,
runtime/common/dev_isa.h:899-917).
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


def quant_weight_128x128(w: torch.Tensor):
    """w [N, K] float -> (e4m3 [N, K], scales f32 [ceil(N/128), ceil(K/128)])."""
    n, k = w.shape
    nb, kb = (n + 127) // 128, (k + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:n, :k] = w.float()
    blocks = wp.view(nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    # amax * (1 / 448), not amax / 448: a tensor divided by a host scalar is multiplied by the rounded reciprocal on the GPU
    # and truly divided on the CPU, which moves the scale by one ulp and one code in a thousand with it
    scale = amax.clamp_min(1e-10) * (1.0 / FP8_MAX)
    q = (blocks / scale[:, None, :, None]).view(nb * 128, kb * 128)[:n, :k].to(FP8)
    return q.contiguous(), scale.contiguous()


def dequant_weight_128x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    s = scale.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
    return q.float() * s


def quant_act_1x128(x: torch.Tensor, ld: int | None = None):
    """x [M, K] -> (e4m3 [M, K], scales f32 transposed [ceil(K/128), ld >= M])."""
    m, k = x.shape
    kb = (k + 127) // 128
    xp = torch.zeros(m, kb * 128, dtype=torch.float32, device=x.device)
    xp[:, :k] = x.float()
    g = xp.view(m, kb, 128)
    scale = g.abs().amax(dim=2).clamp_min(1e-10) / FP8_MAX          # [M, KB]
    q = (g / scale[:, :, None]).view(m, kb * 128)[:, :k].to(FP8)
    ld = ld or m
    st = torch.zeros(kb, ld, dtype=torch.float32, device=x.device)
    st[:, :m] = scale.t()
    return q.contiguous(), st


def dequant_act_1x128(q: torch.Tensor, st: torch.Tensor) -> torch.Tensor:
    m, k = q.shape
    s = st[:, :m].t().repeat_interleave(128, 1)[:, :k]
    return q.float() * s
