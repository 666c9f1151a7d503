"""Pipeline stage planning: cut the layer sequence into contiguous stages of balanced modelled time.

The cost of a layer is the cost model's decode-step time for its attention + FFN at the planned batch; embedding and
lm_head are charged to the first and last stage.  The planner minimises the slowest stage (the pipeline's beat) by
dynamic programming over cut points.  ``plowc stage-plan`` prints the plan; `parallel/pp.py` runs stages over
point-to-point sends.  Reference: crates/plowc/src/stage_plan.rs, docs/arch/30-heterogeneous-serving.md:127-143
(stage_boundary section design; the reference rejects ``--parallel pp`` at compile time)."""
from __future__ import annotations

from . import costmodel, hwspec


def layer_costs_us(spec, hw=None, batch: int = 64, ctx: int = 2048) -> list:
    hw = hw or hwspec.lookup("b200")
    es = costmodel.dtype_bytes(spec.dtype)
    wb = 1 if spec.weight_quant == "fp8_block128" else es
    out = []
    H = spec.hidden
    for layer in spec.layers:
        a, f = layer.attn, layer.ffn
        t = 0.0
        if a.kind == "gqa":
            qd = a.n_heads * a.head_dim * (2 if a.gated else 1)
            for n, k in ((qd + 2 * a.n_kv_heads * a.head_dim, H), (H, a.n_heads * a.head_dim)):
                t += costmodel.gemm_cost(batch, n, k, wb, es).time_us(hw, spec.dtype)
            t += costmodel.attention_decode_cost(batch * ctx, a.n_heads, a.n_kv_heads, a.head_dim, a.head_dim, es).time_us(hw)
        elif a.kind == "mla":
            qh = a.qk_nope + a.qk_rope
            for n, k in (((a.q_lora or 0) + a.kv_lora + a.qk_rope, H), (a.n_heads * qh, a.q_lora or H), (H, a.n_heads * a.v_head)):
                t += costmodel.gemm_cost(batch, n, k, wb, es).time_us(hw, spec.dtype)
            t += batch * ctx * (a.kv_lora + a.qk_rope) * (1 if spec.kv_dtype == "fp8" else es) / (hw.hbm_gbs * 1e3)
        else:
            d = a.gdn_head_dim
            for n, k in ((2 * a.gdn_k_heads * d + 2 * a.gdn_v_heads * d, H), (H, a.gdn_v_heads * d)):
                t += costmodel.gemm_cost(batch, n, k, wb, es).time_us(hw, spec.dtype)
            t += 2.0 * batch * a.gdn_v_heads * d * d * 4 / (hw.hbm_gbs * 1e3)
        if f.kind == "dense":
            t += costmodel.gemm_cost(batch, 2 * f.inter, H, wb, es).time_us(hw, spec.dtype) + costmodel.gemm_cost(batch, H, f.inter, wb, es).time_us(hw, spec.dtype)
        else:
            active = min(f.n_experts, batch * f.top_k)
            inter = f.moe_inter or f.inter
            t += 3.0 * active * inter * H * wb / (hw.hbm_gbs * 1e3)
            if f.n_shared:
                t += 3.0 * f.n_shared * inter * H * wb / (hw.hbm_gbs * 1e3)
        out.append(t)
    return out


def plan_stages(costs: list, n_stages: int, head_us: float = 0.0, tail_us: float = 0.0) -> dict:
    """Contiguous partition of ``costs`` into ``n_stages`` minimising the slowest stage.  Returns cut points
    (stage s runs layers [cuts[s], cuts[s+1])), per-stage times and the balance (mean / max)."""
    n = len(costs)
    if not 1 <= n_stages <= n:
        raise ValueError(f"cannot cut {n} layers into {n_stages} stages")
    pre = [0.0]
    for c in costs:
        pre.append(pre[-1] + c)

    def seg(i, j, s):
        return pre[j] - pre[i] + (head_us if s == 0 else 0.0) + (tail_us if s == n_stages - 1 else 0.0)
    INF = float("inf")
    best = [[INF] * (n + 1) for _ in range(n_stages + 1)]
    arg = [[0] * (n + 1) for _ in range(n_stages + 1)]
    best[0][0] = 0.0
    for s in range(1, n_stages + 1):
        for j in range(s, n + 1):
            for i in range(s - 1, j):
                v = max(best[s - 1][i], seg(i, j, s - 1))
                if v < best[s][j]:
                    best[s][j], arg[s][j] = v, i
    cuts = [n]
    j = n
    for s in range(n_stages, 0, -1):
        j = arg[s][j]
        cuts.append(j)
    cuts.reverse()
    times = [seg(cuts[s], cuts[s + 1], s) for s in range(n_stages)]
    return dict(cuts=cuts, stage_us=[round(t, 2) for t in times], beat_us=round(max(times), 2),
                balance=round(sum(times) / n_stages / max(times), 3))
