"""Gated delta-rule linear attention ops (csrc/cuda/gdn.cu).

Reference semantics: runtime/nvidia/op_qwen_gdn.cuh:1237-1247, runtime/common/dev_isa.h:1259-1280."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native

BF16 = torch.bfloat16


def gdn(qkvz, ba, conv_w, a_log, dt_bias, conv_state, ssm_state, pos, seq, hk, hv, head_dim=128, conv=4, out=None):
    """Conv + gates + state recurrence for every row of the step (rows of one sequence are consecutive)."""
    rows = qkvz.shape[0]
    if out is None:
        out = torch.empty(rows, hv * head_dim, dtype=BF16, device=qkvz.device)
    native.call("plow_gdn", out, conv_state, ssm_state, qkvz, qkvz.stride(0), ba, ba.stride(0), conv_w, a_log, dt_bias,
                pos, seq, rows, hk, hv, head_dim, conv)
    return out


def gated_norm(o, z_src, z_ofs, gamma, heads, head_dim, eps, out=None):
    rows = o.shape[0]
    if out is None:
        out = torch.empty_like(o)
    native.call("plow_gated_norm", out, o, z_src, z_src.stride(0), z_ofs, gamma, rows, heads, head_dim, float(eps))
    return out


def sigmoid_gate(a, gate, out=None):
    if out is None:
        out = torch.empty_like(a)
    native.call("plow_sigmoid_gate", out, a, gate, a.numel())
    return out


def reference(qkvz, ba, conv_w, a_log, dt_bias, hk, hv, d=128, conv=4, conv_hist=None, S=None):
    """fp32 recurrence for ONE sequence (rows in order).  Returns (out [T, hv*d], conv history [C, conv-1], S)."""
    T = qkvz.shape[0]
    C = (2 * hk + hv) * d
    x = qkvz[:, :C].float()
    hist = conv_hist if conv_hist is not None else torch.zeros(C, conv - 1, device=x.device)
    xp = torch.cat([hist.t(), x], 0)                                   # [conv-1+T, C]
    y = F.silu(F.conv1d(xp.t()[None], conv_w.float()[:, None, :], groups=C))[0].t()
    q = y[:, :hk * d].view(T, hk, d)
    k = y[:, hk * d:2 * hk * d].view(T, hk, d)
    v = y[:, 2 * hk * d:].view(T, hv, d)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    b, al = ba[:, :hv].float(), ba[:, hv:].float()
    beta = torch.sigmoid(b).bfloat16().float()
    alpha = torch.exp(-torch.exp(a_log.float()) * F.softplus(al + dt_bias.float()))
    rep = hv // hk
    S = torch.zeros(hv, d, d, device=x.device) if S is None else S.clone()
    out = torch.zeros(T, hv, d, device=x.device)
    for t in range(T):
        kt, qt = k[t].repeat_interleave(rep, 0), q[t].repeat_interleave(rep, 0)
        S = S * alpha[t, :, None, None]
        pred = torch.einsum("hvk,hk->hv", S, kt)
        S = S + beta[t, :, None, None] * torch.einsum("hv,hk->hvk", v[t] - pred, kt)
        out[t] = torch.einsum("hvk,hk->hv", S, qt) * d ** -0.5
    return out.reshape(T, -1), xp[-(conv - 1):].t().contiguous(), S
