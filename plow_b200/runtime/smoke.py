"""One tiny prefill + decode of the flagship family (MLA + MoE, block-scaled e4m3 weights, e4m3
latent cache) on cuda:0 through the sm_100a kernels."""
from __future__ import annotations

import numpy as np
import torch


def small_mla_moe_config(n_layers=2, hidden=1024, experts=16) -> dict:
    from ..models.config import mla_moe_671b_config
    cfg = mla_moe_671b_config(n_experts=experts, n_layers=n_layers)
    cfg.update(hidden_size=hidden, q_lora_rank=256, intermediate_size=512, moe_intermediate_size=256,
               first_k_dense_replace=1, num_experts_per_tok=4, n_group=4, topk_group=2, vocab_size=1024,
               max_position_embeddings=4096)
    return cfg


def build_engine(cfg, max_slots=8, max_ctx=1024, prefill=(128,), decode=(8,), seed=0, cuda_graphs=True, ep=1, rank=0, comm=None):
    from ..compiler import emit, graph, hwspec, rewrite
    from ..models.config import spec_from_config
    from .gpu_engine import GpuEngine, SyntheticWeights
    spec = spec_from_config(cfg)
    g = graph.build_graph(spec, ep=ep, rank=rank)
    sites = rewrite.fuse(g)
    pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=list(prefill), decode=list(decode), max_seqs=max_slots), rank=rank)
    dev = torch.device("cuda", torch.cuda.current_device())
    return GpuEngine(packet=pkt, weights=SyntheticWeights(dev, seed=seed), max_slots=max_slots, max_ctx=max_ctx,
                     cuda_graphs=cuda_graphs, rank=rank, comm=comm)


def run() -> None:
    from .engine import TokenBatch
    eng = build_engine(small_mla_moe_config())
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 1024, size=100).astype(np.int32)
    eng.begin_slot(0, prompt.tolist())
    eng.reserve(0, 110)
    r = eng.step(TokenBatch(prompt, np.arange(100, dtype=np.int32), np.zeros(100, np.int32), np.array([99], np.int32)))
    eng.commit(0, prompt.tolist())
    tok = int(r.ids[0])
    for i in range(3):
        r = eng.step(TokenBatch(np.array([tok], np.int32), np.array([100 + i], np.int32), np.zeros(1, np.int32),
                                np.array([0], np.int32), decode=True))
        eng.commit(0, [tok])
        tok = int(r.ids[0])
    assert 0 <= tok < 1024
    print(f"smoke ok: last token {tok}, decode step {eng.step_ms_last:.3f} ms")
