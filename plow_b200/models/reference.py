"""Plain PyTorch reference implementations (the numeric oracle) and random-init checkpoints.

Every model here consumes a ``state_dict`` keyed by the HF checkpoint tensor names and runs in
whatever dtype the tensors are promoted to (tests use fp32).  They are written for clarity, not
speed: full-sequence causal attention, dense expert loops.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F

from ..utils.rope import mla_softmax_factor, rope_table
from .config import ModelSpec, spec_from_config


# ------------------------------------------------------------------------------------------------
def rmsnorm(x, g, eps, plus_one=False):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if g is not None:
        y = y * ((1.0 + g.float()) if plus_one else g.float())
    return y.to(x.dtype)


def apply_rope(x, tab, pos, rot_dim, pair_mode):
    """x [..., T, heads, hd]; tab [max_pos, rot]; pos [T]."""
    half = rot_dim // 2
    cs = tab[pos, :half].to(x.dtype)[:, None, :]
    sn = tab[pos, half:rot_dim].to(x.dtype)[:, None, :]
    xr, xp = x[..., :rot_dim], x[..., rot_dim:]
    if pair_mode == "half":
        a, b = xr[..., :half], xr[..., half:]
        out = torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1)
    else:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cs - b * sn, b * cs + a * sn], dim=-1).flatten(-2)
    return torch.cat([out, xp], dim=-1)


def causal_attention(q, k, v, scale, window=0, keep=None, sinks=None):
    """q [T, nq, hd], k/v [T, nkv, hd(v)] -> [T, nq, hdv]; full causal mask (+ sliding window).  ``keep`` (bool [T, T],
    optional): sparse attention, query t attends only the keys s with keep[t, s].  ``sinks`` ([nq], optional): one more
    logit per head in every row's softmax, whose probability is dropped."""
    T, nq, _ = q.shape
    nkv = k.shape[1]
    k = k.repeat_interleave(nq // nkv, dim=1)
    v = v.repeat_interleave(nq // nkv, dim=1)
    s = torch.einsum("thd,shd->hts", q.float(), k.float()) * scale
    i = torch.arange(T, device=q.device)
    mask = i[None, :] > i[:, None]
    if keep is not None:
        mask = mask | ~keep
    if window:
        mask = mask | (i[None, :] <= i[:, None] - window)
    s = s.masked_fill(mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float()[:, None, None].expand(nq, T, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)[..., :T]
    return torch.einsum("hts,shd->thd", p, v.float()).to(q.dtype)


# ------------------------------------------------------------------------------------------------
class ReferenceModel:
    """Full-sequence forward of any supported family over a name-keyed state dict."""

    def __init__(self, spec: ModelSpec, state: dict, device="cpu", dtype=torch.float32):
        self.spec = spec
        self.w = {k: v.to(device=device, dtype=dtype if v.is_floating_point() else v.dtype) for k, v in state.items()}
        self.dsa_override: dict = {}      # layer prefix -> bool [T, T] selection to attend instead of the indexer's own
        self.dsa_last: dict = {}          # layer prefix -> the selection the last forward attended
        self.device, self.dtype = device, dtype
        r = spec.rope
        self.rope = torch.from_numpy(rope_table(min(r.max_pos, 1 << 17), r.rot_dim, r.theta, r.scaling)).to(device)
        self._ropes = {}             # rotary tables of layers with a base of their own

    def lin(self, x, name):
        y = x @ self.w[name].t()
        b = self.w.get(name[:-len("weight")] + "bias") if name.endswith("weight") else None
        return y if b is None else y + b

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [T] -> logits [T, V] (float32)."""
        return self.forward_hidden(ids)[0]

    @torch.no_grad()
    def forward_hidden(self, ids: torch.Tensor):
        """ids [T] -> (logits [T, V] float32, hidden [T, H] after the final norm: what a prediction module reads)."""
        spec = self.spec
        T = ids.shape[0]
        self.route_margin_last = float("inf")     # smallest routing gap of the last row over the MoE layers of this call
        pos = torch.arange(T, device=self.device)
        x = self.w["model.embed_tokens.weight"][ids] * spec.embed_scale
        for li, layer in enumerate(spec.layers):
            x = self._block(f"model.layers.{li}", x, pos, layer)
        x = rmsnorm(x, self.w["model.norm.weight"], spec.rms_eps, spec.norm_plus_one)
        return (x @ self._head().t()).float(), x

    @torch.no_grad()
    def mtp_forward(self, next_ids: torch.Tensor, hidden: torch.Tensor, k: int = 0):
        """Prediction module k over a whole sequence.  Row i reads ``hidden[i]`` (the decoder's normed hidden state at
        position i, or this module's own output for a chained draft) and ``next_ids[i]`` (token i + 1); its logits
        predict token i + 2.  Returns (logits [T, V] float32, the module's hidden [T, H] before its head norm).
        Weights: model.layers.<n_layers + k>.{enorm, hnorm, eh_proj, shared_head.norm} and a decoder block with the plan
        of the last layer; the embedding and the output head are the decoder's own."""
        spec = self.spec
        p = f"model.layers.{spec.n_layers + k}"
        pos = torch.arange(next_ids.shape[0], device=self.device)
        e = rmsnorm(self.w["model.embed_tokens.weight"][next_ids] * spec.embed_scale, self.w[f"{p}.enorm.weight"], spec.rms_eps, spec.norm_plus_one)
        h = rmsnorm(hidden.to(e.dtype), self.w[f"{p}.hnorm.weight"], spec.rms_eps, spec.norm_plus_one)
        x = torch.cat([e, h], dim=-1) @ self.w[f"{p}.eh_proj.weight"].t()
        x = self._block(p, x, pos, spec.layers[-1])
        hn = rmsnorm(x, self.w[f"{p}.shared_head.norm.weight"], spec.rms_eps, spec.norm_plus_one)
        return (hn @ self._head().t()).float(), x

    def _head(self):
        return self.w["model.embed_tokens.weight"] if self.spec.tie_embeddings else self.w["lm_head.weight"]

    def _block(self, p, x, pos, layer):
        spec = self.spec
        h = rmsnorm(x, self.w[f"{p}.input_layernorm.weight"], spec.rms_eps, spec.norm_plus_one)
        if layer.attn.kind == "gqa":
            o = self._gqa(p, h, pos, layer.attn)
        elif layer.attn.kind == "mla":
            o = self._mla(p, h, pos, layer.attn)
        elif layer.attn.kind == "kda":
            o = self._kda(p, h, layer.attn)
        else:
            o = self._gdn(p, h, layer.attn)
        if spec.sandwich_norms:
            o = rmsnorm(o, self.w[f"{p}.post_attention_layernorm.weight"], spec.rms_eps, spec.norm_plus_one)
        x = x + o
        pre = "pre_feedforward" if spec.sandwich_norms else "post_attention"
        h = rmsnorm(x, self.w[f"{p}.{pre}_layernorm.weight"], spec.rms_eps, spec.norm_plus_one)
        d = self._dense(f"{p}.mlp", h, act=layer.ffn.act) if layer.ffn.kind == "dense" else self._moe(f"{p}.{layer.ffn.block}", h, layer.ffn)
        if spec.sandwich_norms:
            d = rmsnorm(d, self.w[f"{p}.post_feedforward_layernorm.weight"], spec.rms_eps, spec.norm_plus_one)
        return x + d

    # ---- blocks --------------------------------------------------------------------------------
    def _dense(self, p, h, names="proj", act="silu"):
        g, u, d = ("w1", "w3", "w2") if names == "w123" else ("gate_proj", "up_proj", "down_proj")
        gate = self.lin(h, f"{p}.{g}.weight")
        gate = F.silu(gate) if act == "silu" else F.gelu(gate, approximate="tanh" if act == "gelu_tanh" else "none")
        return self.lin(gate * self.lin(h, f"{p}.{u}.weight"), f"{p}.{d}.weight")

    def _gqa(self, p, h, pos, a):
        spec = self.spec
        T = h.shape[0]
        q = self.lin(h, f"{p}.self_attn.q_proj.weight")
        gate = None
        if a.gated:
            q = q.view(T, a.n_heads, 2 * a.head_dim)
            q, gate = q[..., :a.head_dim], q[..., a.head_dim:].reshape(T, -1)
        q = q.reshape(T, a.n_heads, a.head_dim)
        k = self.lin(h, f"{p}.self_attn.k_proj.weight").view(T, a.n_kv_heads, a.head_dim)
        v = self.lin(h, f"{p}.self_attn.v_proj.weight").view(T, a.n_kv_heads, a.head_dim)
        if a.qk_norm:
            q = rmsnorm(q, self.w[f"{p}.self_attn.q_norm.weight"], spec.rms_eps, spec.norm_plus_one)
            k = rmsnorm(k, self.w[f"{p}.self_attn.k_norm.weight"], spec.rms_eps, spec.norm_plus_one)
        rope = self.rope
        if a.rope_theta and a.rope_theta != spec.rope.theta:
            if a.rope_theta not in self._ropes:
                self._ropes[a.rope_theta] = torch.from_numpy(rope_table(min(spec.rope.max_pos, 1 << 17), spec.rope.rot_dim, a.rope_theta, None)).to(self.device)
            rope = self._ropes[a.rope_theta]
        q = apply_rope(q, rope, pos, spec.rope.rot_dim, spec.rope.pair_mode)
        k = apply_rope(k, rope, pos, spec.rope.rot_dim, spec.rope.pair_mode)
        o = causal_attention(q, k, v, a.scale or a.head_dim ** -0.5, a.window,
                             sinks=self.w[f"{p}.self_attn.sinks"] if a.sinks else None).reshape(T, -1)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self.lin(o, f"{p}.self_attn.o_proj.weight")

    def _mla(self, p, h, pos, a):
        spec = self.spec
        T = h.shape[0]
        qh = a.qk_nope + a.qk_rope
        if a.q_lora:
            qa = rmsnorm(self.lin(h, f"{p}.self_attn.q_a_proj.weight"), self.w[f"{p}.self_attn.q_a_layernorm.weight"], spec.rms_eps)
            q = self.lin(qa, f"{p}.self_attn.q_b_proj.weight")
        else:
            q = self.lin(h, f"{p}.self_attn.q_proj.weight")
        q = q.view(T, a.n_heads, qh)
        kva = self.lin(h, f"{p}.self_attn.kv_a_proj_with_mqa.weight")
        c_kv = rmsnorm(kva[:, :a.kv_lora], self.w[f"{p}.self_attn.kv_a_layernorm.weight"], spec.rms_eps)
        k_rope = apply_rope(kva[:, a.kv_lora:].view(T, 1, a.qk_rope), self.rope, pos, a.qk_rope, spec.rope.pair_mode)
        q_nope, q_rope = q[..., :a.qk_nope], apply_rope(q[..., a.qk_nope:], self.rope, pos, a.qk_rope, spec.rope.pair_mode)
        kvb = self.lin(c_kv, f"{p}.self_attn.kv_b_proj.weight").view(T, a.n_heads, a.qk_nope + a.v_head)
        k = torch.cat([kvb[..., :a.qk_nope], k_rope.expand(T, a.n_heads, a.qk_rope)], dim=-1)
        v = kvb[..., a.qk_nope:]
        keep = None
        if a.index_heads:
            keep = self.dsa_override.get(p) if self.dsa_override else None      # tests: attend a given selection
            if keep is None:
                keep = self.dsa_select(p, h, qa if a.q_lora else h, pos, a)
            self.dsa_last[p] = keep
        o = causal_attention(torch.cat([q_nope, q_rope], -1), k, v, qh ** -0.5 * mla_softmax_factor(spec.rope.scaling), keep=keep).reshape(T, -1)
        return self.lin(o, f"{p}.self_attn.o_proj.weight")

    def dsa_scores(self, p, h, q_in, pos, a):
        """Sparse-attention indexer scores [T, T] (future keys at -inf): index queries of `index_heads` heads from the
        query latent, one index key per token (LayerNorm with bias, RoPE on the first rot dims, halves pairing), per-head
        weights from the hidden state; score[t, s] = sum_h w[t, h] relu(q[t, h] . k[s])."""
        T = h.shape[0]
        rot = self.spec.rope.rot_dim
        qi = self.lin(q_in, f"{p}.self_attn.indexer.wq_b.weight").view(T, a.index_heads, a.index_dim)
        ki = self.lin(h, f"{p}.self_attn.indexer.wk.weight")
        ki = torch.nn.functional.layer_norm(ki.float(), (a.index_dim,), self.w[f"{p}.self_attn.indexer.k_norm.weight"].float(),
                                            self.w[f"{p}.self_attn.indexer.k_norm.bias"].float(), 1e-6).to(h.dtype)
        wt = self.lin(h, f"{p}.self_attn.indexer.weights_proj.weight").float()
        qi = apply_rope(qi, self.rope, pos, rot, "half")
        ki = apply_rope(ki.view(T, 1, a.index_dim), self.rope, pos, rot, "half").view(T, a.index_dim)
        dots = torch.relu(torch.einsum("thd,sd->ths", qi.float(), ki.float()))
        sc = (wt[:, :, None] * dots).sum(1)
        i = torch.arange(T, device=h.device)
        return sc.masked_fill(i[None, :] > i[:, None], float("-inf"))

    def dsa_select(self, p, h, q_in, pos, a):
        """bool [T, T]: the index_topk best-scoring visible keys of every query (all of them while fewer are visible);
        ties go to the lower position."""
        sc = self.dsa_scores(p, h, q_in, pos, a)
        T = sc.shape[0]
        k = min(a.index_topk, T)
        idx = _stable_topk(sc, k)
        keep = torch.zeros(T, T, dtype=torch.bool, device=sc.device)
        keep.scatter_(1, idx, True)
        return keep & torch.isfinite(sc)

    def route(self, logits, f, bias=None):
        """Router semantics shared with the kernels (group-limited noaux_tc selection): returns
        (expert ids [T,k], gates [T,k]).  Selection uses score + bias, gates use the unbiased score."""
        scores = torch.sigmoid(logits.float()) if f.score == "sigmoid" else torch.softmax(logits.float(), -1)
        sel = scores + (bias.float() if bias is not None else 0.0)
        T, E = sel.shape
        if f.n_group > 1:
            grp = sel.view(T, f.n_group, E // f.n_group)
            gscore = grp.topk(2, dim=-1).values.sum(-1)
            keep = torch.zeros_like(gscore, dtype=torch.bool)
            keep.scatter_(1, _stable_topk(gscore, f.topk_group), True)
            sel = sel.masked_fill(~keep[:, :, None].expand_as(grp).reshape(T, E), float("-inf"))
        idx = _stable_topk(sel, f.top_k)
        g = scores.gather(1, idx)
        if f.norm_topk:
            g = g / g.sum(-1, keepdim=True).clamp_min(1e-20)
        return idx, g * f.route_scale

    def _moe_fused_experts(self, p, h, f):
        """gpt_oss: biased router, softmax over the chosen logits, experts read from the per-projection tensors."""
        logits = self.lin(h.float(), f"{p}.router.weight")
        idx, g = self.route(logits, f, None)
        gu, gub = self.w[f"{p}.experts.gate_up_proj"].float(), self.w[f"{p}.experts.gate_up_proj_bias"].float()
        dn, dnb = self.w[f"{p}.experts.down_proj"].float(), self.w[f"{p}.experts.down_proj_bias"].float()
        out = torch.zeros_like(h, dtype=torch.float32)
        for j in range(f.top_k):
            for e in idx[:, j].unique().tolist():
                m = idx[:, j] == e
                y = h[m].float() @ gu[e] + gub[e]
                gate, up = y[:, 0::2].clamp(max=f.swiglu_limit), y[:, 1::2].clamp(-f.swiglu_limit, f.swiglu_limit)
                act = (up + 1.0) * gate * torch.sigmoid(f.swiglu_alpha * gate)
                out[m] += g[m, j, None] * (act @ dn[e] + dnb[e])
        return out.to(h.dtype)

    def _moe(self, p, h, f):
        if f.fused_experts:
            return self._moe_fused_experts(p, h, f)
        bias = self.w.get(f"{p}.gate.e_score_correction_bias")
        logits = h.float() @ self.w[f"{p}.gate.weight"].float().t()
        idx, g = self.route(logits, f, bias)
        # how decisively the last row was routed: gap between the weakest chosen and the strongest rejected expert score
        # (a reduced-precision implementation may legitimately route such a row differently when the gap is tiny)
        sc = torch.sigmoid(logits[-1]) if f.score == "sigmoid" else torch.softmax(logits[-1], -1)
        sel = sc + (bias.float() if bias is not None else 0.0)
        top = torch.sort(sel, descending=True).values
        if f.top_k < top.numel():
            self.route_margin_last = min(self.route_margin_last, float(top[f.top_k - 1] - top[f.top_k]))
        out = torch.zeros_like(h, dtype=torch.float32)
        for j in range(f.top_k):
            for e in idx[:, j].unique().tolist():
                m = idx[:, j] == e
                out[m] += g[m, j, None] * self._dense(f"{p}.experts.{e}", h[m], f.expert_names).float()
        if f.n_shared:
            sp = f"{p}.shared_experts" if self.spec.family == "mla_moe" else f"{p}.shared_expert"
            out = out + self._dense(sp, h).float()
        return out.to(h.dtype)

    def _kda(self, p, h, a):
        """Kimi Delta Attention over a whole sequence, token by token."""
        T = h.shape[0]
        nh, d = a.gdn_v_heads, a.gdn_head_dim
        sa = f"{p}.self_attn"

        def conv(x, name):
            w = self.w[f"{sa}.{name}.weight"].float().reshape(nh * d, -1)
            xp = F.pad(x.float().t()[None], (a.gdn_conv - 1, 0))
            return F.silu(F.conv1d(xp, w[:, None, :], groups=w.shape[0]))[0].t().view(T, nh, d)

        q, k, v = (conv(self.lin(h, f"{sa}.{n}_proj.weight"), f"{n}_conv1d") for n in "qkv")
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(self.lin(h, f"{sa}.b_proj.weight").float())
        raw = self.lin(self.lin(h, f"{sa}.f_a_proj.weight"), f"{sa}.f_b_proj.weight").float() + self.w[f"{sa}.dt_bias"].float()
        ea = torch.exp(self.w[f"{sa}.A_log"].float().reshape(-1))[None, :, None]
        raw = raw.view(T, nh, d)
        g = a.kda_gate_floor * torch.sigmoid(ea * raw) if a.kda_gate_floor < 0 else -ea * F.softplus(raw)
        S = torch.zeros(nh, d, d, dtype=torch.float32, device=h.device)      # [head, v, k]
        out = torch.zeros(T, nh, d, dtype=torch.float32, device=h.device)
        for t in range(T):
            S = S * torch.exp(g[t])[:, None, :]
            pred = torch.einsum("hvk,hk->hv", S, k[t])
            S = S + beta[t, :, None, None] * torch.einsum("hv,hk->hvk", v[t] - pred, k[t])
            out[t] = torch.einsum("hvk,hk->hv", S, q[t])
        gate = self.lin(self.lin(h, f"{sa}.g_a_proj.weight"), f"{sa}.g_b_proj.weight").float().view(T, nh, d)
        on = rmsnorm(out, self.w[f"{sa}.o_norm.weight"], self.spec.rms_eps) * torch.sigmoid(gate)
        return self.lin(on.reshape(T, -1).to(h.dtype), f"{sa}.o_proj.weight")

    def _gdn(self, p, h, a):
        T = h.shape[0]
        hk, hv, d = a.gdn_k_heads, a.gdn_v_heads, a.gdn_head_dim
        la = f"{p}.linear_attn"
        if a.gdn_split_proj:
            qkvz = torch.cat([self.lin(h, f"{la}.in_proj_qkv.weight"), self.lin(h, f"{la}.in_proj_z.weight")], -1)
            ba = torch.cat([self.lin(h, f"{la}.in_proj_b.weight"), self.lin(h, f"{la}.in_proj_a.weight")], -1)
        else:
            qkvz = self.lin(h, f"{la}.in_proj_qkvz.weight")
            ba = self.lin(h, f"{la}.in_proj_ba.weight")
        qkv, z = qkvz[:, :(2 * hk + hv) * d], qkvz[:, (2 * hk + hv) * d:]
        w = self.w[f"{p}.linear_attn.conv1d.weight"].float()          # [C, W]
        xp = F.pad(qkv.float().t()[None], (a.gdn_conv - 1, 0))         # causal depthwise conv
        qkv = F.silu(F.conv1d(xp, w[:, None, :], groups=w.shape[0]))[0].t()
        q = qkv[:, :hk * d].view(T, hk, d)
        k = qkv[:, hk * d:2 * hk * d].view(T, hk, d)
        v = qkv[:, 2 * hk * d:].view(T, hv, d)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        b, al = ba[:, :hv].float(), ba[:, hv:].float()
        beta = torch.sigmoid(b)
        alpha = torch.exp(-torch.exp(self.w[f"{p}.linear_attn.A_log"].float()) * F.softplus(al + self.w[f"{p}.linear_attn.dt_bias"].float()))
        rep = hv // hk
        S = torch.zeros(hv, d, d, dtype=torch.float32, device=h.device)   # [v-head, V, K]
        out = torch.zeros(T, hv, d, dtype=torch.float32, device=h.device)
        for t in range(T):
            kt, qt = k[t].repeat_interleave(rep, 0), q[t].repeat_interleave(rep, 0)
            S = S * alpha[t, :, None, None]
            pred = torch.einsum("hvk,hk->hv", S, kt)
            S = S + beta[t, :, None, None] * torch.einsum("hv,hk->hvk", v[t] - pred, kt)
            out[t] = torch.einsum("hvk,hk->hv", S, qt) * d ** -0.5
        on = rmsnorm(out, self.w[f"{p}.linear_attn.norm.weight"], self.spec.rms_eps) * F.silu(z.float().view(T, hv, d))
        return self.lin(on.reshape(T, -1).to(h.dtype), f"{p}.linear_attn.out_proj.weight")


def _stable_topk(x, k):
    """top-k with the lowest index winning ties (the kernels' packed-key rule)."""
    order = torch.sort(x, dim=-1, descending=True, stable=True).indices
    return order[..., :k]


# ------------------------------------------------------------------------------------------------
def param_shapes(spec: ModelSpec) -> dict:
    """Checkpoint tensor name -> shape for a spec (HF naming)."""
    H, V = spec.hidden, spec.vocab
    s = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not spec.tie_embeddings:
        s["lm_head.weight"] = (V, H)
    blocks = list(enumerate(spec.layers)) + [(spec.n_layers + k, spec.layers[-1]) for k in range(spec.mtp_layers)]
    for li, layer in blocks:
        p = f"model.layers.{li}"
        a, f = layer.attn, layer.ffn
        if li >= spec.n_layers:      # a prediction module: two input norms, the [embedding | hidden] projection, a head norm
            s[f"{p}.enorm.weight"] = (H,)
            s[f"{p}.hnorm.weight"] = (H,)
            s[f"{p}.eh_proj.weight"] = (H, 2 * H)
            s[f"{p}.shared_head.norm.weight"] = (H,)
        s[f"{p}.input_layernorm.weight"] = (H,)
        s[f"{p}.post_attention_layernorm.weight"] = (H,)
        if spec.sandwich_norms:
            s[f"{p}.pre_feedforward_layernorm.weight"] = (H,)
            s[f"{p}.post_feedforward_layernorm.weight"] = (H,)
        if a.kind == "gqa":
            s[f"{p}.self_attn.q_proj.weight"] = (a.n_heads * a.head_dim * (2 if a.gated else 1), H)
            s[f"{p}.self_attn.k_proj.weight"] = (a.n_kv_heads * a.head_dim, H)
            s[f"{p}.self_attn.v_proj.weight"] = (a.n_kv_heads * a.head_dim, H)
            s[f"{p}.self_attn.o_proj.weight"] = (H, a.n_heads * a.head_dim)
            for proj in (("q_proj", "k_proj", "v_proj") if a.qkv_bias else ()) + (("o_proj",) if a.o_bias else ()):
                s[f"{p}.self_attn.{proj}.bias"] = (s[f"{p}.self_attn.{proj}.weight"][0],)
            if a.sinks:
                s[f"{p}.self_attn.sinks"] = (a.n_heads,)
            if a.qk_norm:
                s[f"{p}.self_attn.q_norm.weight"] = (a.head_dim,)
                s[f"{p}.self_attn.k_norm.weight"] = (a.head_dim,)
        elif a.kind == "kda":
            nh, d = a.gdn_v_heads, a.gdn_head_dim
            sa = f"{p}.self_attn"
            for nm in ("q", "k", "v"):
                s[f"{sa}.{nm}_proj.weight"] = (nh * d, H)
                s[f"{sa}.{nm}_conv1d.weight"] = (nh * d, 1, a.gdn_conv)
            s[f"{sa}.b_proj.weight"] = (nh, H)
            s[f"{sa}.f_a_proj.weight"], s[f"{sa}.f_b_proj.weight"] = (d, H), (nh * d, d)
            s[f"{sa}.g_a_proj.weight"], s[f"{sa}.g_b_proj.weight"] = (d, H), (nh * d, d)
            s[f"{sa}.A_log"], s[f"{sa}.dt_bias"] = (1, 1, nh, 1), (nh * d,)
            s[f"{sa}.o_norm.weight"] = (d,)
            s[f"{sa}.o_proj.weight"] = (H, nh * d)
        elif a.kind == "mla":
            qh = a.qk_nope + a.qk_rope
            if a.q_lora:
                s[f"{p}.self_attn.q_a_proj.weight"] = (a.q_lora, H)
                s[f"{p}.self_attn.q_a_layernorm.weight"] = (a.q_lora,)
                s[f"{p}.self_attn.q_b_proj.weight"] = (a.n_heads * qh, a.q_lora)
            else:
                s[f"{p}.self_attn.q_proj.weight"] = (a.n_heads * qh, H)
            s[f"{p}.self_attn.kv_a_proj_with_mqa.weight"] = (a.kv_lora + a.qk_rope, H)
            s[f"{p}.self_attn.kv_a_layernorm.weight"] = (a.kv_lora,)
            s[f"{p}.self_attn.kv_b_proj.weight"] = (a.n_heads * (a.qk_nope + a.v_head), a.kv_lora)
            s[f"{p}.self_attn.o_proj.weight"] = (H, a.n_heads * a.v_head)
            if a.index_heads:
                s[f"{p}.self_attn.indexer.wq_b.weight"] = (a.index_heads * a.index_dim, a.q_lora or H)
                s[f"{p}.self_attn.indexer.wk.weight"] = (a.index_dim, H)
                s[f"{p}.self_attn.indexer.weights_proj.weight"] = (a.index_heads, H)
                s[f"{p}.self_attn.indexer.k_norm.weight"] = (a.index_dim,)
                s[f"{p}.self_attn.indexer.k_norm.bias"] = (a.index_dim,)
        else:
            d = a.gdn_head_dim
            if a.gdn_split_proj:
                s[f"{p}.linear_attn.in_proj_qkv.weight"] = (2 * a.gdn_k_heads * d + a.gdn_v_heads * d, H)
                s[f"{p}.linear_attn.in_proj_z.weight"] = (a.gdn_v_heads * d, H)
                s[f"{p}.linear_attn.in_proj_b.weight"] = (a.gdn_v_heads, H)
                s[f"{p}.linear_attn.in_proj_a.weight"] = (a.gdn_v_heads, H)
            else:
                s[f"{p}.linear_attn.in_proj_qkvz.weight"] = (2 * a.gdn_k_heads * d + 2 * a.gdn_v_heads * d, H)
                s[f"{p}.linear_attn.in_proj_ba.weight"] = (2 * a.gdn_v_heads, H)
            s[f"{p}.linear_attn.conv1d.weight"] = ((2 * a.gdn_k_heads + a.gdn_v_heads) * d, a.gdn_conv)
            s[f"{p}.linear_attn.A_log"] = (a.gdn_v_heads,)
            s[f"{p}.linear_attn.dt_bias"] = (a.gdn_v_heads,)
            s[f"{p}.linear_attn.norm.weight"] = (d,)
            s[f"{p}.linear_attn.out_proj.weight"] = (H, a.gdn_v_heads * d)
        if f.kind == "dense":
            for nm, shp in (("gate_proj", (f.inter, H)), ("up_proj", (f.inter, H)), ("down_proj", (H, f.inter))):
                s[f"{p}.mlp.{nm}.weight"] = shp
        elif f.fused_experts:
            s[f"{p}.mlp.router.weight"] = (f.n_experts, H)
            s[f"{p}.mlp.router.bias"] = (f.n_experts,)
            s[f"{p}.mlp.experts.gate_up_proj"] = (f.n_experts, H, 2 * f.moe_inter)
            s[f"{p}.mlp.experts.gate_up_proj_bias"] = (f.n_experts, 2 * f.moe_inter)
            s[f"{p}.mlp.experts.down_proj"] = (f.n_experts, f.moe_inter, H)
            s[f"{p}.mlp.experts.down_proj_bias"] = (f.n_experts, H)
        else:
            s[f"{p}.{f.block}.gate.weight"] = (f.n_experts, H)
            if f.has_bias:
                s[f"{p}.{f.block}.gate.e_score_correction_bias"] = (f.n_experts,)
            gn, un, dn = ("w1", "w3", "w2") if f.expert_names == "w123" else ("gate_proj", "up_proj", "down_proj")
            for e in range(f.n_experts):
                for nm, shp in ((gn, (f.moe_inter, H)), (un, (f.moe_inter, H)), (dn, (H, f.moe_inter))):
                    s[f"{p}.{f.block}.experts.{e}.{nm}.weight"] = shp
            if f.n_shared:
                sp = f"{p}.{f.block}.shared_experts" if spec.family == "mla_moe" else f"{p}.{f.block}.shared_expert"
                w = f.moe_inter * f.n_shared
                for nm, shp in (("gate_proj", (w, H)), ("up_proj", (w, H)), ("down_proj", (H, w))):
                    s[f"{sp}.{nm}.weight"] = shp
    return s


def random_state(spec: ModelSpec, seed: int = 0, std: float = 0.02, dtype=torch.float32) -> dict:
    """Weights N(0, std), norm weights 1 (0 for (1+γ) models), router bias 0, A_log/dt_bias small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in param_shapes(spec).items():
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            t = torch.zeros(shape) if (spec.norm_plus_one and "linear_attn.norm" not in name) else torch.ones(shape)
        elif name.endswith("e_score_correction_bias") or name.endswith("k_norm.bias"):
            t = torch.zeros(shape)
        elif name.endswith("A_log"):
            t = torch.log(torch.rand(shape, generator=g) * 15 + 1)
        elif name.endswith("dt_bias"):
            t = torch.rand(shape, generator=g)
        elif name.endswith("proj.bias") or name.endswith("proj_bias") or name.endswith("router.bias") or name.endswith("sinks"):
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = torch.randn(shape, generator=g) * std
        out[name] = t.to(dtype if t.dim() > 1 and not name.endswith("conv1d.weight") else torch.float32)
    return out


def write_checkpoint(cfg: dict, out_dir, seed: int = 0, dtype=torch.float32, shard_bytes: int = 2 << 30) -> Path:
    """Random-init HF-layout checkpoint: config.json + model-0000x.safetensors (+ index)."""
    from safetensors.torch import save_file
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    spec = spec_from_config(cfg)
    state = random_state(spec, seed, dtype=dtype)
    (out / "config.json").write_text(json.dumps(cfg, indent=1))
    shards, cur, size = [], {}, 0
    for k, v in state.items():
        nb = v.numel() * v.element_size()
        if cur and size + nb > shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v.contiguous()
        size += nb
    shards.append(cur)
    index = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, str(out / fn))
        index.update({k: fn for k in sh})
    (out / "model.safetensors.index.json").write_text(json.dumps(dict(metadata={}, weight_map=index)))
    return out
