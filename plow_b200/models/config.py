"""Checkpoint ``config.json`` -> :class:`ModelSpec` (the per-layer plan the compiler lowers).

Families understood (by ``model_type`` / ``architectures``):

* dense GQA decoders: llama, mistral, qwen3 (per-head q/k RMSNorm), qwen2 (biases on q / k / v), llama-shaped models with
  ``attention_bias`` (o_proj too), gemma (``1+γ`` norms, GELU gate), gemma3_text (four norms per layer, local / global
  layers with their own rotary base); ``mlp_bias`` and gemma2 (capped logits) are refused by name.  The reference folds
  qwen2 into its qwen3 emitter with ``qkv_bias`` set (crates/nn-graph/src/models/config/mod.rs:233-248) and carries the
  bias as operand 7 of its GEMM (runtime/common/dev_isa.h:114-120);
* MLA + MoE decoders: deepseek_v3 / deepseek_v2, kimi_k2, glm_moe_dsa (adds the DSA indexer);
* hybrid linear-attention decoders: qwen3_next (gated delta rule + gated full attention, MoE), qwen3_5 / qwen3_5_moe (the
  same layers with split gated-delta-rule projections, ``layer_types`` and dense or MoE MLPs; language model only) and kimi_linear (Kimi Delta
  Attention layers + latent attention without rotary embedding; CPU backend);
* GQA + MoE decoders: qwen3_moe (per-head q/k norm, softmax router), mixtral (experts named w1 / w3 / w2 under
  ``block_sparse_moe``) and gpt_oss (attention sinks, biased projections / router / experts, clamped GLU, sliding and
  full layers in turn; bf16 experts or the release's MXFP4 blocks, dequantised at load).

The reference derives the same plan in crates/plowc/src/hf_config.rs (LayerPlan from config.json)
and dispatches emitters on ``model_type`` in crates/devgen/src/lib.rs:9518-9646.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass
class RopeSpec:
    theta: float = 10000.0
    rot_dim: int = 0              # rotated dims per head (partial rotary when < head_dim)
    pair_mode: str = "half"       # "half": (i, i + rot/2) NeoX; "interleaved": (2i, 2i+1) GPT-J
    scaling: dict | None = None   # {"type": "llama3"|"yarn"|"linear", ...}
    max_pos: int = 4096


@dataclass
class AttnSpec:
    kind: str = "gqa"             # gqa | mla | gdn | kda (gdn_* fields: heads, head_dim, conv; key heads = value heads)
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False
    window: int = 0               # 0 = full attention
    gated: bool = False           # per-head output gate (qwen3_next full attention)
    scale: float = 0.0            # softmax scale when it is not head_dim^-0.5 (gemma3: query_pre_attn_scalar^-0.5)
    rope_theta: float = 0.0       # rotary base of this layer when it differs from the model's (gemma3 local layers)
    qkv_bias: bool = False        # q / k / v projections carry a bias (qwen2; llama-style attention_bias)
    o_bias: bool = False          # the output projection carries one too (attention_bias)
    sinks: bool = False           # one learned logit per head joins every softmax and takes no value (gpt_oss)
    # MLA
    q_lora: int = 0
    kv_lora: int = 0
    qk_nope: int = 0
    qk_rope: int = 0
    v_head: int = 0
    # DSA indexer
    index_heads: int = 0
    index_dim: int = 0
    index_topk: int = 0
    # gated delta rule
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_head_dim: int = 0
    gdn_conv: int = 4
    gdn_split_proj: bool = False  # qwen3_5: in_proj_qkv / in_proj_z / in_proj_b / in_proj_a instead of in_proj_qkvz / in_proj_ba
    kda_gate_floor: float = 0.0   # kda: < 0 selects the bounded gate g = floor * sigmoid(exp(A_log) (x + dt_bias)); 0: -exp(A_log) softplus(.)


@dataclass
class FfnSpec:
    kind: str = "dense"           # dense | moe
    inter: int = 0
    act: str = "silu"
    n_experts: int = 0
    top_k: int = 0
    n_shared: int = 0
    moe_inter: int = 0
    n_group: int = 1
    topk_group: int = 1
    score: str = "softmax"        # softmax | sigmoid
    norm_topk: bool = True
    route_scale: float = 1.0
    has_bias: bool = False        # e_score_correction_bias
    block: str = "mlp"            # module that holds the router and the experts (mixtral: block_sparse_moe)
    expert_names: str = "proj"    # "proj": gate_proj / up_proj / down_proj; "w123": w1 (gate) / w3 (up) / w2 (down)
    # gpt_oss: all experts in one tensor per projection (gate_up_proj [E, H, 2F] with gate / up columns interleaved,
    # down_proj [E, F, H]) with biases, a biased router named `router`, and the clamped GLU
    # (up + 1) * g * sigmoid(alpha * g), g = min(gate, limit), up clamped to +-limit
    fused_experts: bool = False
    swiglu_limit: float = 0.0
    swiglu_alpha: float = 1.702


@dataclass
class LayerSpec:
    attn: AttnSpec
    ffn: FfnSpec


@dataclass
class ModelSpec:
    family: str
    model_type: str
    hidden: int
    vocab: int
    n_layers: int
    rms_eps: float
    tie_embeddings: bool
    rope: RopeSpec
    layers: list = field(default_factory=list)
    norm_plus_one: bool = False   # Gemma (1 + γ)
    embed_scale: float = 1.0
    dtype: str = "bf16"           # compute dtype of activations
    weight_quant: str = "none"    # none | fp8_block128
    kv_dtype: str = "bf16"        # bf16 | fp8 | f32
    max_ctx: int = 4096
    bos_token_id: int | None = None
    eos_token_ids: list = field(default_factory=list)
    sandwich_norms: bool = False  # gemma3: a norm after the attention and after the MLP too (four norms per layer)
    mtp_layers: int = 0           # next-token-prediction modules behind the decoder stack (num_nextn_predict_layers)
    role: str = "main"            # "mtp": this spec is one prediction module compiled as a drafter of its own
    name_base: int = 0            # checkpoint index of layers[0] (model.layers.<name_base + i>)

    def drafter_spec(self, k: int = 0) -> "ModelSpec":
        """The k-th prediction module as a one-layer model of its own.  Its block has the plan of the last decoder layer
        and its weights live at model.layers.<n_layers + k> (enorm, hnorm, eh_proj, shared_head.norm and the block)."""
        import copy
        if k >= self.mtp_layers:
            raise ValueError(f"the checkpoint has {self.mtp_layers} prediction module(s), asked for {k}")
        d = copy.deepcopy(self)
        d.layers, d.n_layers, d.mtp_layers, d.role, d.name_base = [copy.deepcopy(self.layers[-1])], 1, 0, "mtp", self.n_layers + k
        return d

    def to_json(self) -> str:
        return json.dumps(asdict(self), sort_keys=True)

    @staticmethod
    def from_json(s: str) -> "ModelSpec":
        d = json.loads(s)
        layers = [LayerSpec(AttnSpec(**l["attn"]), FfnSpec(**l["ffn"])) for l in d.pop("layers")]
        rope = RopeSpec(**d.pop("rope"))
        return ModelSpec(rope=rope, layers=layers, **d)

    # ---- sizes -------------------------------------------------------------------------
    def kv_bytes_per_token(self) -> int:
        """Bytes of KV cache one token occupies across all layers."""
        es = {"bf16": 2, "fp8": 1, "f32": 4}[self.kv_dtype]
        n = 0
        for l in self.layers:
            a = l.attn
            if a.kind == "gqa":
                n += 2 * a.n_kv_heads * a.head_dim * es + (8 * a.n_kv_heads if self.kv_dtype == "fp8" else 0)
            elif a.kind == "mla":
                n += (a.kv_lora + a.qk_rope) * es + (4 if self.kv_dtype == "fp8" else 0)
                if a.index_heads:
                    n += a.index_dim * (1 if self.kv_dtype == "fp8" else 2) + 4
        return n

    def param_count(self) -> int:
        h = self.hidden
        n = self.vocab * h * (1 if self.tie_embeddings else 2)
        for l in self.layers:
            a, f = l.attn, l.ffn
            if a.kind == "gqa":
                qd = a.n_heads * a.head_dim * (2 if a.gated else 1)
                n += h * (qd + 2 * a.n_kv_heads * a.head_dim) + a.n_heads * a.head_dim * h
            elif a.kind == "mla":
                qh = a.qk_nope + a.qk_rope
                n += (h * a.q_lora + a.q_lora * a.n_heads * qh) if a.q_lora else h * a.n_heads * qh
                n += h * (a.kv_lora + a.qk_rope) + a.kv_lora * a.n_heads * (a.qk_nope + a.v_head)
                n += a.n_heads * a.v_head * h
            elif a.kind == "gdn":
                kd, vd = a.gdn_k_heads * a.gdn_head_dim, a.gdn_v_heads * a.gdn_head_dim
                n += h * (2 * kd + 2 * vd) + h * 2 * a.gdn_v_heads + vd * h
            elif a.kind == "kda":
                hd_all, d = a.gdn_v_heads * a.gdn_head_dim, a.gdn_head_dim
                n += 4 * h * hd_all + h * a.gdn_v_heads + 2 * (h * d + d * hd_all)
            if f.kind == "dense":
                n += 3 * h * f.inter
            else:
                n += f.n_experts * 3 * h * f.moe_inter + f.n_shared * 3 * h * f.moe_inter + h * f.n_experts
        return n


def _rope_from(cfg: dict, head_dim: int, rot_dim: int | None = None, pair: str = "half") -> RopeSpec:
    sc = cfg.get("rope_scaling") or cfg.get("rope_parameters")
    scaling = None
    if isinstance(sc, dict) and (sc.get("rope_type") or sc.get("type")) not in (None, "default"):
        scaling = dict(sc)
        scaling["type"] = sc.get("rope_type") or sc.get("type")
    theta = cfg.get("rope_theta")
    if theta is None and isinstance(sc, dict):
        theta = sc.get("rope_theta")
    return RopeSpec(theta=float(theta or 10000.0), rot_dim=rot_dim if rot_dim is not None else head_dim,
                    pair_mode=pair, scaling=scaling, max_pos=int(cfg.get("max_position_embeddings", 4096)))


def _act(cfg: dict, moe: bool = False) -> str:
    """The gate activation of the GLU: silu, gelu_tanh or gelu.  Routed experts run SiLU only."""
    a = str(cfg.get("hidden_act") or cfg.get("hidden_activation") or "silu").lower()
    name = {"silu": "silu", "swish": "silu", "gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_tanh", "gelu_tanh": "gelu_tanh",
            "gelu_fast": "gelu_tanh", "gelu": "gelu"}.get(a)
    if name is None:
        raise ValueError(f"unsupported hidden_act '{a}' (silu, gelu_pytorch_tanh and gelu are)")
    if moe and name != "silu":
        raise ValueError(f"routed experts with hidden_act '{a}' are not supported (silu only)")
    return name


def _eos(cfg: dict) -> list:
    e = cfg.get("eos_token_id")
    if e is None:
        return []
    return list(e) if isinstance(e, (list, tuple)) else [int(e)]


def _quant(cfg: dict) -> str:
    q = cfg.get("quantization_config") or {}
    if q.get("quant_method") == "fp8" and q.get("weight_block_size") == [128, 128]:
        return "fp8_block128"
    return cfg.get("plow_weight_quant", "none")


def spec_from_config(cfg: dict) -> ModelSpec:
    mt = cfg.get("model_type", "")
    if cfg.get("mlp_bias") or (cfg.get("attention_bias") and mt not in ("llama", "mistral", "qwen3", "plow_dense")):
        raise ValueError(f"model_type '{mt}': this projection bias is not supported (attention biases are, on llama-shaped models and "
                         "qwen2); dropping it would compute a different model")
    if mt == "qwen2" and cfg.get("use_sliding_window"):
        raise ValueError("qwen2 with use_sliding_window is not supported: its window covers only the layers above max_window_layers")
    if mt in ("llama", "mistral", "qwen2", "qwen3", "gemma", "plow_dense"):
        return _dense_gqa(cfg, mt)
    if mt == "gpt_oss":
        return _gpt_oss(cfg)
    if mt == "kimi_linear":
        return _kimi_linear(cfg)
    if mt in ("gemma3_text", "gemma3"):
        return _gemma3(cfg.get("text_config", cfg) if mt == "gemma3" else cfg, "gemma3_text")
    if mt == "gemma2":
        raise ValueError("model_type 'gemma2' is not supported: it caps its attention and output logits; reading it as a "
                         "llama-shaped model would compute something else")
    if mt in ("deepseek_v3", "deepseek_v2", "kimi_k2", "glm_moe_dsa", "glm5_next", "deepseek_v32", "plow_mla_moe"):
        return _mla_moe(cfg, mt)
    if mt in ("qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text", "plow_gdn_hybrid"):
        return _gdn_hybrid(cfg, mt)
    if mt in ("qwen3_moe", "mixtral"):
        return _gqa_moe(cfg, mt)
    raise ValueError(f"unsupported model_type '{mt}'")


def load_spec(path) -> ModelSpec:
    """A checkpoint directory (its config.json), a config.json path, or a GGUF file (its metadata)."""
    from ..runtime.gguf import GgufFile, config_from_gguf, find_gguf
    g = find_gguf(path)
    if g is not None:
        return spec_from_config(config_from_gguf(GgufFile(g)))
    p = Path(path)
    if p.is_dir():
        p = p / "config.json"
    return spec_from_config(json.loads(p.read_text()))


def _dense_gqa(cfg: dict, mt: str) -> ModelSpec:
    h = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or h // nh
    n_layers = cfg["num_hidden_layers"]
    attn = AttnSpec(kind="gqa", n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm=(mt == "qwen3" or cfg.get("qk_norm", False)),
                    window=int(cfg.get("sliding_window") or 0) if cfg.get("use_sliding_window", mt == "mistral") else 0,
                    qkv_bias=(mt == "qwen2" or bool(cfg.get("attention_bias"))), o_bias=bool(cfg.get("attention_bias")) and mt != "qwen2")
    ffn = FfnSpec(kind="dense", inter=cfg["intermediate_size"], act=_act(cfg))
    gem = mt.startswith("gemma")
    return ModelSpec(
        family="dense_gqa", model_type=mt, hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        rope=_rope_from(cfg, hd), layers=[LayerSpec(attn, ffn) for _ in range(n_layers)],
        norm_plus_one=gem, embed_scale=(h ** 0.5 if gem else 1.0),
        dtype=cfg.get("plow_dtype", "bf16"), weight_quant=_quant(cfg), kv_dtype=cfg.get("plow_kv_dtype", cfg.get("plow_dtype", "bf16")),
        max_ctx=int(cfg.get("max_position_embeddings", 4096)), bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg),
        mtp_layers=int(cfg.get("num_nextn_predict_layers") or 0))


def _mla_moe(cfg: dict, mt: str) -> ModelSpec:
    h = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    n_layers = cfg["num_hidden_layers"]
    first_dense = int(cfg.get("first_k_dense_replace", 0))
    idx_heads = int(cfg.get("index_n_heads", 0))
    attn = AttnSpec(kind="mla", n_heads=nh, n_kv_heads=1, head_dim=cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"],
                    q_lora=int(cfg.get("q_lora_rank") or 0), kv_lora=cfg["kv_lora_rank"],
                    qk_nope=cfg["qk_nope_head_dim"], qk_rope=cfg["qk_rope_head_dim"], v_head=cfg["v_head_dim"],
                    index_heads=idx_heads, index_dim=int(cfg.get("index_head_dim", 0)),
                    index_topk=int(cfg.get("index_topk", 0)))
    dense = FfnSpec(kind="dense", inter=cfg["intermediate_size"], act=_act(cfg))
    moe = FfnSpec(kind="moe", act=_act(cfg, moe=bool(cfg.get("n_routed_experts"))), n_experts=cfg.get("n_routed_experts", 0),
                  top_k=cfg.get("num_experts_per_tok", 0), n_shared=cfg.get("n_shared_experts", 0),
                  moe_inter=cfg.get("moe_intermediate_size", 0), n_group=cfg.get("n_group", 1),
                  topk_group=cfg.get("topk_group", 1), score=cfg.get("scoring_func", "sigmoid"),
                  norm_topk=bool(cfg.get("norm_topk_prob", True)), route_scale=float(cfg.get("routed_scaling_factor", 1.0)),
                  has_bias=cfg.get("topk_method", "noaux_tc") == "noaux_tc")
    if moe.n_experts and moe.n_group > 1 and cfg.get("topk_method", "noaux_tc") not in ("noaux_tc", "greedy"):
        raise ValueError(f"topk_method '{cfg.get('topk_method')}' with expert groups is not supported: groups are ranked here by the "
                         "sum of their two best scores (noaux_tc), not by their best score")
    layers = [LayerSpec(attn, dense if (i < first_dense or not moe.n_experts) else moe) for i in range(n_layers)]
    return ModelSpec(
        family="mla_moe", model_type=mt, hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        rope=_rope_from(cfg, cfg["qk_rope_head_dim"], pair="interleaved"), layers=layers,
        dtype=cfg.get("plow_dtype", "bf16"), weight_quant=_quant(cfg), kv_dtype=cfg.get("plow_kv_dtype", "fp8" if _quant(cfg) != "none" else cfg.get("plow_dtype", "bf16")),
        max_ctx=int(cfg.get("max_position_embeddings", 4096)), bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg),
        mtp_layers=int(cfg.get("num_nextn_predict_layers") or 0))


def _gemma3(cfg: dict, mt: str) -> ModelSpec:
    """Gemma 3 text decoder: (1 + gamma) norms before AND after attention and MLP, per-head q / k norms, GELU-tanh gate,
    scaled embeddings, softmax scale from query_pre_attn_scalar, five sliding-window layers (local rotary base) for every
    global one (global base, optionally with linear scaling)."""
    h = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or 256
    n_layers = cfg["num_hidden_layers"]
    types = cfg.get("layer_types")
    if not types:
        pat = int(cfg.get("sliding_window_pattern", 6))
        types = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(n_layers)]
    scale = float(cfg.get("query_pre_attn_scalar", hd)) ** -0.5
    win = int(cfg.get("sliding_window") or 0)
    local = AttnSpec(kind="gqa", n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm=True, window=win, scale=scale,
                     rope_theta=float(cfg.get("rope_local_base_freq", 10000.0)))
    full = AttnSpec(kind="gqa", n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm=True, window=0, scale=scale)
    ffn = FfnSpec(kind="dense", inter=cfg["intermediate_size"], act=_act(dict(hidden_act=cfg.get("hidden_activation") or cfg.get("hidden_act") or "gelu_pytorch_tanh")))
    layers = [LayerSpec(full if t == "full_attention" else local, ffn) for t in types]
    return ModelSpec(
        family="dense_gqa", model_type=mt, hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(cfg.get("tie_word_embeddings", True)),
        rope=_rope_from(dict(cfg, rope_theta=cfg.get("rope_theta", 1000000.0)), hd), layers=layers, norm_plus_one=True, embed_scale=h ** 0.5,
        sandwich_norms=True, dtype=cfg.get("plow_dtype", "bf16"), weight_quant=_quant(cfg),
        kv_dtype=cfg.get("plow_kv_dtype", cfg.get("plow_dtype", "bf16")), max_ctx=int(cfg.get("max_position_embeddings", 4096)),
        bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg))


def _gqa_moe(cfg: dict, mt: str) -> ModelSpec:
    """Grouped-query attention + a routed MoE in (almost) every layer: qwen3_moe and mixtral."""
    h = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or h // nh
    n_layers = cfg["num_hidden_layers"]
    mix = mt == "mixtral"
    attn = AttnSpec(kind="gqa", n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm=not mix,
                    window=int(cfg.get("sliding_window") or 0) if (mix and cfg.get("sliding_window")) else 0)
    moe = FfnSpec(kind="moe", act=_act(cfg, moe=True), n_experts=cfg["num_local_experts" if mix else "num_experts"],
                  top_k=cfg["num_experts_per_tok"], moe_inter=cfg["intermediate_size" if mix else "moe_intermediate_size"],
                  score="softmax", norm_topk=True if mix else bool(cfg.get("norm_topk_prob", True)),
                  block="block_sparse_moe" if mix else "mlp", expert_names="w123" if mix else "proj")
    dense = FfnSpec(kind="dense", inter=cfg.get("intermediate_size", 0), act=_act(cfg))
    step, only = int(cfg.get("decoder_sparse_step", 1) or 1), set(cfg.get("mlp_only_layers") or [])
    layers = [LayerSpec(attn, moe if (mix or (i not in only and (i + 1) % step == 0)) else dense) for i in range(n_layers)]
    return ModelSpec(
        family="gqa_moe", model_type=mt, hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        rope=_rope_from(cfg, hd), layers=layers,
        dtype=cfg.get("plow_dtype", "bf16"), weight_quant=_quant(cfg), kv_dtype=cfg.get("plow_kv_dtype", cfg.get("plow_dtype", "bf16")),
        max_ctx=int(cfg.get("max_position_embeddings", 4096)), bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg))


def _gpt_oss(cfg: dict) -> ModelSpec:
    """gpt_oss: GQA with biased projections and per-head attention sinks, sliding-window and full layers in turn, YaRN
    rotary tables, and a routed MoE in every layer whose experts are biased and use the clamped GLU.  Experts are read
    from the bf16 export or from the MXFP4 blocks of the original release (dequantised at load).  Reference emitter: crates/devgen/src/gptoss.rs."""
    q = cfg.get("quantization_config") or {}
    if q and q.get("quant_method") != "mxfp4":
        raise ValueError(f"gpt_oss: quantization '{q.get('quant_method')}' is not supported (bf16 experts or the MXFP4 blocks are)")
    h = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or h // nh
    n_layers = cfg["num_hidden_layers"]
    win = int(cfg.get("sliding_window") or 0)
    kinds = cfg.get("layer_types") or ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n_layers)]
    if len(kinds) != n_layers or any(k not in ("sliding_attention", "full_attention") for k in kinds):
        raise ValueError("gpt_oss: layer_types must name sliding_attention or full_attention for every layer")

    def attn(kind):
        return AttnSpec(kind="gqa", n_heads=nh, n_kv_heads=nkv, head_dim=hd, window=win if kind == "sliding_attention" else 0,
                        qkv_bias=True, o_bias=True, sinks=True)

    moe = FfnSpec(kind="moe", n_experts=cfg["num_local_experts"], top_k=cfg.get("num_experts_per_tok") or cfg["experts_per_token"],
                  moe_inter=cfg["intermediate_size"], score="softmax", norm_topk=True, fused_experts=True,
                  swiglu_limit=float(cfg.get("swiglu_limit", 7.0)))
    return ModelSpec(
        family="gqa_moe", model_type="gpt_oss", hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-5)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        rope=_rope_from(cfg, hd), layers=[LayerSpec(attn(k), moe) for k in kinds],
        dtype=cfg.get("plow_dtype", "bf16"), weight_quant="none", kv_dtype=cfg.get("plow_kv_dtype", cfg.get("plow_dtype", "bf16")),
        max_ctx=int(cfg.get("max_position_embeddings", 4096)), bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg))


def _kimi_linear(cfg: dict) -> ModelSpec:
    """kimi_linear: Kimi Delta Attention layers (a gated delta rule whose forget gate is per key channel, fed by separate
    q / k / v short convolutions and low-rank gate projections) with a latent-attention layer every few layers, which
    carries no rotary embedding (``mla_use_nope``), and a sigmoid-routed MoE with a shared expert behind the first dense
    layers.  Reference emitters: crates/devgen/src/kda.rs, crates/devgen/src/k3.rs; op contract runtime/common/dev_isa.h:711-840."""
    h = cfg["hidden_size"]
    n_layers = cfg["num_hidden_layers"]
    lac = cfg.get("linear_attn_config") or {}
    kda_layers = {int(i) - 1 for i in lac.get("kda_layers", [])}           # the config counts layers from 1
    full_layers = {int(i) - 1 for i in lac.get("full_attn_layers", [])}
    if kda_layers | full_layers != set(range(n_layers)) or kda_layers & full_layers:
        raise ValueError("kimi_linear: linear_attn_config.kda_layers and full_attn_layers must split the layers between them")
    kda = AttnSpec(kind="kda", gdn_k_heads=lac["num_heads"], gdn_v_heads=lac["num_heads"], gdn_head_dim=lac["head_dim"],
                   gdn_conv=int(lac.get("short_conv_kernel_size", 4)), kda_gate_floor=float(lac.get("gate_lower_bound") or 0.0))
    mla = AttnSpec(kind="mla", n_heads=cfg["num_attention_heads"], n_kv_heads=1, head_dim=cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"],
                   q_lora=int(cfg.get("q_lora_rank") or 0), kv_lora=cfg["kv_lora_rank"], qk_nope=cfg["qk_nope_head_dim"],
                   qk_rope=cfg["qk_rope_head_dim"], v_head=cfg["v_head_dim"])
    first_dense = int(cfg.get("first_k_dense_replace", 0))
    dense = FfnSpec(kind="dense", inter=cfg["intermediate_size"], act=_act(cfg))
    moe = FfnSpec(kind="moe", act=_act(cfg, moe=True), n_experts=cfg["num_experts"], top_k=cfg.get("num_experts_per_token") or cfg["num_experts_per_tok"],
                  n_shared=int(cfg.get("num_shared_experts", 0)), moe_inter=cfg["moe_intermediate_size"],
                  n_group=int(cfg.get("num_expert_group", 1)), topk_group=int(cfg.get("topk_group", 1)),
                  score=cfg.get("moe_router_activation_func", "sigmoid"), norm_topk=bool(cfg.get("moe_renormalize", True)),
                  route_scale=float(cfg.get("routed_scaling_factor", 1.0)), has_bias=True, block="block_sparse_moe", expert_names="w123")
    layers = [LayerSpec(kda if i in kda_layers else mla, dense if i < first_dense else moe) for i in range(n_layers)]
    rope_cfg = dict(cfg, rope_scaling=dict(rope_type="nope")) if cfg.get("mla_use_nope", True) else cfg
    return ModelSpec(
        family="mla_moe", model_type="kimi_linear", hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-5)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        rope=_rope_from(rope_cfg, cfg["qk_rope_head_dim"], pair="interleaved"), layers=layers,
        dtype=cfg.get("plow_dtype", "bf16"), weight_quant="none", kv_dtype=cfg.get("plow_kv_dtype", cfg.get("plow_dtype", "bf16")),
        max_ctx=int(cfg.get("max_position_embeddings", 4096)), bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg))


def _gdn_hybrid(cfg: dict, mt: str) -> ModelSpec:
    q35 = mt.startswith("qwen3_5")
    if cfg.get("vision_config") is not None or "text_config" in cfg:
        raise ValueError(f"model_type '{mt}' with a vision tower is not supported: export the language model on its own "
                         "(tensor names model.layers.*)")
    if cfg.get("attention_bias"):
        raise ValueError(f"model_type '{mt}' with attention_bias is not supported")
    h = cfg["hidden_size"]
    n_layers = cfg["num_hidden_layers"]
    interval = int(cfg.get("full_attention_interval", 4))
    types = cfg.get("layer_types") or ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n_layers)]
    if len(types) != n_layers or any(t not in ("full_attention", "linear_attention") for t in types):
        raise ValueError(f"{mt}: layer_types must name linear_attention or full_attention for every layer")
    rp = cfg.get("rope_parameters") or {}
    hd = cfg.get("head_dim", 256)
    rot = int(hd * float(cfg.get("partial_rotary_factor", rp.get("partial_rotary_factor", 0.25))))
    full = AttnSpec(kind="gqa", n_heads=cfg["num_attention_heads"], n_kv_heads=cfg["num_key_value_heads"],
                    head_dim=hd, qk_norm=True, gated=bool(cfg.get("attn_output_gate", True)))
    lin = AttnSpec(kind="gdn", gdn_k_heads=cfg["linear_num_key_heads"], gdn_v_heads=cfg["linear_num_value_heads"],
                   gdn_head_dim=cfg.get("linear_key_head_dim", 128), gdn_conv=cfg.get("linear_conv_kernel_dim", 4), gdn_split_proj=q35)
    if cfg.get("num_experts"):
        ffn = FfnSpec(kind="moe", n_experts=cfg["num_experts"], top_k=cfg["num_experts_per_tok"],
                      n_shared=1 if cfg.get("shared_expert_intermediate_size") else 0,
                      moe_inter=cfg["moe_intermediate_size"], score="softmax", norm_topk=bool(cfg.get("norm_topk_prob", True)))
    else:                                              # qwen3_5 dense: a gated MLP in every layer
        ffn = FfnSpec(kind="dense", inter=cfg["intermediate_size"], act=_act(cfg))
    moe = ffn
    layers = [LayerSpec(full if t == "full_attention" else lin, moe) for t in types]
    return ModelSpec(
        family="gdn_hybrid", model_type=mt, hidden=h, vocab=cfg["vocab_size"], n_layers=n_layers,
        rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        rope=_rope_from(cfg, hd, rot_dim=rot), layers=layers, norm_plus_one=True,
        dtype=cfg.get("plow_dtype", "bf16"), weight_quant=_quant(cfg), kv_dtype=cfg.get("plow_kv_dtype", cfg.get("plow_dtype", "bf16")),
        max_ctx=int(cfg.get("max_position_embeddings", 4096)), bos_token_id=cfg.get("bos_token_id"), eos_token_ids=_eos(cfg))


# ---- the five benchmark configurations -------------------------------------------------------
def tiny_dense_config() -> dict:
    """CPU plumbing model: 4 layers, hidden 512, 8 q / 2 kv heads, hd 64, FFN 1408, fp32."""
    return dict(model_type="llama", hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                num_hidden_layers=4, intermediate_size=1408, rms_norm_eps=1e-6, rope_theta=10000.0,
                vocab_size=32000, tie_word_embeddings=True, max_position_embeddings=4096, plow_dtype="f32",
                plow_kv_dtype="f32", eos_token_id=2, bos_token_id=1)


def dense_8b_config() -> dict:
    return dict(model_type="llama", hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                num_hidden_layers=32, intermediate_size=14336, rms_norm_eps=1e-5, rope_theta=500000.0,
                vocab_size=128256, tie_word_embeddings=False, max_position_embeddings=8192, eos_token_id=128001)


def mla_moe_671b_config(n_experts: int = 256, n_layers: int = 61, dsa: bool = False) -> dict:
    cfg = dict(model_type="deepseek_v3", hidden_size=7168, num_attention_heads=128, num_hidden_layers=n_layers,
               q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
               intermediate_size=18432, first_k_dense_replace=3, n_routed_experts=n_experts, n_shared_experts=1,
               num_experts_per_tok=8, moe_intermediate_size=2048, n_group=8, topk_group=4, scoring_func="sigmoid",
               norm_topk_prob=True, routed_scaling_factor=2.5, topk_method="noaux_tc", rms_norm_eps=1e-6,
               rope_theta=10000.0, vocab_size=129280, tie_word_embeddings=False, max_position_embeddings=163840,
               quantization_config=dict(quant_method="fp8", weight_block_size=[128, 128]), eos_token_id=1)
    if dsa:
        cfg.update(model_type="glm_moe_dsa", index_n_heads=64, index_head_dim=128, index_topk=2048)
    return cfg


def qwen3_moe_30b_config() -> dict:
    """GQA + MoE decoder of the 30B-A3B shape: 48 layers, 128 experts, 8 active."""
    return dict(model_type="qwen3_moe", hidden_size=2048, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                head_dim=128, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, intermediate_size=6144,
                norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], rms_norm_eps=1e-6, rope_theta=1000000.0,
                vocab_size=151936, tie_word_embeddings=False, max_position_embeddings=40960, eos_token_id=151645)


def mixtral_8x7b_config() -> dict:
    return dict(model_type="mixtral", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                num_local_experts=8, num_experts_per_tok=2, intermediate_size=14336, rms_norm_eps=1e-5, rope_theta=1000000.0,
                vocab_size=32000, tie_word_embeddings=False, max_position_embeddings=32768, eos_token_id=2)


def kimi_linear_48b_config() -> dict:
    n = 27
    full = [4, 8, 12, 16, 20, 24, 27]
    return dict(model_type="kimi_linear", hidden_size=2304, num_hidden_layers=n, num_attention_heads=32, kv_lora_rank=512, q_lora_rank=None,
                qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, mla_use_nope=True,
                linear_attn_config=dict(kda_layers=[i for i in range(1, n + 1) if i not in full], full_attn_layers=full, num_heads=32,
                                        head_dim=128, short_conv_kernel_size=4),
                intermediate_size=9216, num_experts=256, num_experts_per_token=8, moe_intermediate_size=1024, num_shared_experts=1,
                first_k_dense_replace=1, moe_router_activation_func="sigmoid", moe_renormalize=True, routed_scaling_factor=2.446,
                num_expert_group=1, topk_group=1, rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=163840, tie_word_embeddings=False,
                max_position_embeddings=1048576, eos_token_id=163586)


def gpt_oss_120b_config() -> dict:
    return dict(model_type="gpt_oss", hidden_size=2880, num_hidden_layers=36, num_attention_heads=64, num_key_value_heads=8, head_dim=64,
                num_local_experts=128, num_experts_per_tok=4, intermediate_size=2880, sliding_window=128, swiglu_limit=7.0,
                layer_types=["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(36)], rms_norm_eps=1e-5,
                rope_theta=150000.0, rope_scaling=dict(rope_type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0,
                                                       original_max_position_embeddings=4096, truncate=False),
                vocab_size=201088, tie_word_embeddings=False, max_position_embeddings=131072, eos_token_id=200002)


def gdn_hybrid_80b_config() -> dict:
    return dict(model_type="qwen3_next", hidden_size=2048, num_hidden_layers=48, full_attention_interval=4,
                num_attention_heads=16, num_key_value_heads=2, head_dim=256, partial_rotary_factor=0.25,
                linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                linear_value_head_dim=128, linear_conv_kernel_dim=4, num_experts=512, num_experts_per_tok=10,
                moe_intermediate_size=512, shared_expert_intermediate_size=512, norm_topk_prob=True,
                rms_norm_eps=1e-6, rope_theta=10000000.0, vocab_size=151936, tie_word_embeddings=False,
                max_position_embeddings=262144, eos_token_id=151645)
