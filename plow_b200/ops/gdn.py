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


# ---- chunked prefill (WY / UT form) -------------------------------------------------------------------------------
def chunked_prefill(qkvz, ba, conv_w, a_log, dt_bias, conv_hist, S, hk, hv, d=128, conv=4, chunk=64):
    """Gated delta rule over one sequence's consecutive rows in chunks of 64 tokens instead of token by token.

    Per head and chunk (state S0 [dv, dk] at the chunk start, g = running sum of log-decays inside the chunk,
    gamma = exp(g)):  the updates u_j = beta_j (v_j - alpha_j S_{j-1} k_j) solve the unit lower-triangular system
    (I + diag(beta) A) U = diag(beta) V - diag(beta gamma) K S0^T  with  A[j, m] = exp(g_j - g_m) (k_j . k_m), m < j,
    so with T = (I + diag(beta) A)^-1,  W = T diag(beta gamma) K  and  U~ = T diag(beta) V:   U = U~ - W S0^T.
    The state then moves by an affine map that does not depend on S0:  S_next = S0 (gamma_C I - W^T K^) + U~^T K^  with
    K^[j] = exp(g_C - g_j) k_j, so M_c and B_c of every chunk are formed in parallel and only  S <- S M_c + B_c  runs in
    sequence (one batched matrix product per chunk).  Outputs:  O = diag(gamma) Q S0^T + tril(Q K^T (.) exp(g_i - g_j)) U.
    Everything is f32 batched matrix algebra (cuBLAS / cuSOLVER through PyTorch: library GEMMs, not a hand-written
    kernel); the token-by-token kernel (csrc/cuda/gdn.cu) keeps decode and short runs.  Padding rows of the last chunk
    carry beta = 0, log-decay 0 and zero keys, which leaves the state untouched.

    qkvz [T, C + hv d] bf16, ba [T, 2 hv]; conv_hist [C, conv - 1] and S [hv, d, d] f32 are the sequence's state before
    these rows.  Returns (out [T, hv d] f32, new conv_hist, new S).  Same math as :func:`reference`
    (reference: runtime/nvidia/gdn_prefill_sm120.cu, chunked WY representation)."""
    T = qkvz.shape[0]
    C = (2 * hk + hv) * d
    dev = qkvz.device
    x = qkvz[:, :C].float()
    xp = torch.cat([conv_hist.float().t(), x], 0)
    y = F.silu(F.conv1d(xp.t()[None], conv_w.float()[:, None, :], groups=C))[0].t()
    new_hist = xp[-(conv - 1):].t().contiguous()
    q = y[:, :hk * d].view(T, hk, d)
    k = y[:, hk * d:2 * hk * d].view(T, hk, d)
    v = y[:, 2 * hk * d:].view(T, hv, d)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    b, al = ba[:, :hv].float(), ba[:, hv:].float()
    beta = torch.sigmoid(b).bfloat16().float()                                    # [T, hv]
    la = -torch.exp(a_log.float()) * F.softplus(al + dt_bias.float())             # log alpha, [T, hv]
    rep = hv // hk
    NC = (T + chunk - 1) // chunk
    Tp = NC * chunk

    def heads_chunks(t, width):                                                    # [T, h, w] -> [hv, NC, chunk, w]
        if t.shape[1] != hv:
            t = t.repeat_interleave(rep, 1)
        if Tp != T:
            t = torch.cat([t, torch.zeros(Tp - T, hv, width, device=dev)], 0)
        return t.permute(1, 0, 2).reshape(hv, NC, chunk, width)
    qc, kc, vc = heads_chunks(q, d), heads_chunks(k, d), heads_chunks(v, d)
    bc = heads_chunks(beta[:, :, None], 1)[..., 0]                                 # [hv, NC, chunk]
    g = torch.cumsum(heads_chunks(la[:, :, None], 1)[..., 0], -1)                  # [hv, NC, chunk]
    gam = torch.exp(g)
    decay = torch.exp((g[..., :, None] - g[..., None, :]).clamp(max=0.0))          # [.., i, j] = gamma_i / gamma_j for j <= i
    low = torch.tril(torch.ones(chunk, chunk, device=dev), -1)
    A = (kc @ kc.transpose(-1, -2)) * decay * low
    L = torch.eye(chunk, device=dev) + bc[..., None] * A
    rhs = torch.cat([(bc * gam)[..., None] * kc, bc[..., None] * vc], -1)
    sol = torch.linalg.solve_triangular(L, rhs, upper=False, unitriangular=True)
    W, Ut = sol[..., :d], sol[..., d:]                                             # [hv, NC, chunk, d]
    gC = g[..., -1]                                                                # [hv, NC]
    Kh = torch.exp(gC[..., None] - g)[..., None] * kc
    M = torch.exp(gC)[..., None, None] * torch.eye(d, device=dev) - W.transpose(-1, -2) @ Kh    # [hv, NC, dk, dk]
    B = Ut.transpose(-1, -2) @ Kh                                                  # [hv, NC, dv, dk]
    S_in = torch.empty(hv, NC, d, d, device=dev)
    cur = S.float().clone()
    for c in range(NC):                                                            # the only sequential part
        S_in[:, c] = cur
        cur = torch.baddbmm(B[:, c], cur, M[:, c])
    U = Ut - W @ S_in.transpose(-1, -2)
    P = (qc @ kc.transpose(-1, -2)) * decay * torch.tril(torch.ones(chunk, chunk, device=dev))
    O = gam[..., None] * (qc @ S_in.transpose(-1, -2)) + P @ U
    out = (O * d ** -0.5).reshape(hv, Tp, d)[:, :T].permute(1, 0, 2).reshape(T, hv * d)
    return out, new_hist, cur
