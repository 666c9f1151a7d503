"""Checkpoint access: safetensors read in place, names are the contract, shards cut at bind.

* :class:`Checkpoint` discovers ``*.safetensors`` (+ index) in a directory and serves tensors by
  name without loading whole files; :func:`open_checkpoint` also accepts a GGUF file (runtime/gguf.py).
* :func:`shard_slice` applies the Megatron layout: column-parallel weights are split on axis 0
  (output features), row-parallel on axis 1 (input features), everything else is replicated.
* :func:`materialize` resolves one packet tensor entry: a checkpoint tensor, a derived tensor
  (row concatenation, stacked expert matrices, a column range), its block-scaled e4m3 twin, or a generated table.

Reference counterpart: crates/plowrt/src/asset/{checkpoint,shard}.rs, memory/container.rs,
crates/plow-asset/src/derived_weights.rs.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


class Checkpoint:
    def __init__(self, path):
        from safetensors import safe_open
        self.dir = Path(path)
        self._open = safe_open
        self.files: dict[str, str] = {}
        idx = self.dir / "model.safetensors.index.json"
        if idx.exists():
            self.files = dict(json.loads(idx.read_text())["weight_map"])
        else:
            for f in sorted(self.dir.glob("*.safetensors")):
                with safe_open(str(f), framework="pt") as h:
                    for k in h.keys():
                        self.files[k] = f.name
        self._handles: dict[str, object] = {}

    def names(self):
        return self.files.keys()

    def has(self, name: str) -> bool:
        return name in self.files

    def _h(self, fn):
        if fn not in self._handles:
            self._handles[fn] = self._open(str(self.dir / fn), framework="pt")
        return self._handles[fn]

    def get(self, name: str) -> torch.Tensor:
        if name not in self.files:
            raise KeyError(f"checkpoint has no tensor '{name}'")
        return self._h(self.files[name]).get_tensor(name)

    def get_slice(self, name: str, axis: int, start: int, stop: int) -> torch.Tensor:
        s = self._h(self.files[name]).get_slice(name)
        return s[start:stop] if axis == 0 else s[:, start:stop]

    def shape(self, name: str) -> tuple:
        return tuple(self._h(self.files[name]).get_slice(name).get_shape())


def open_checkpoint(path):
    """A safetensors directory, or a GGUF file (or a directory holding just one) behind the same interface."""
    from .gguf import GgufCheckpoint, find_gguf
    g = find_gguf(path)
    return GgufCheckpoint(g) if g is not None else Checkpoint(path)


FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)     # e2m1 codes 0..15


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """OCP microscaling fp4: ``blocks`` [..., G, 16] uint8 holds 32 e2m1 values per group (low nibble = the even element),
    ``scales`` [..., G] uint8 one E8M0 exponent per group (value 2^(s - 127)) -> [..., G * 32].  Exact in bf16: an e2m1
    value has two significant bits and the scale is a power of two."""
    lut = torch.tensor(FP4_VALUES, dtype=torch.float32)
    b = blocks.to(torch.int64)
    vals = torch.stack([lut[b & 0xF], lut[b >> 4]], dim=-1).reshape(*blocks.shape[:-1], 32)
    out = torch.ldexp(vals, (scales.to(torch.int32) - 127)[..., None])
    return out.reshape(*blocks.shape[:-2], -1).to(dtype)


def quant_mxfp4(w: torch.Tensor) -> tuple:
    """The inverse for writing test and converted checkpoints: [..., K] (K % 32 == 0) -> (blocks [..., K/32, 16], scales
    [..., K/32]); per group the smallest power-of-two scale that brings the largest magnitude within 6, values rounded
    to the nearest e2m1 code."""
    g = w.float().reshape(*w.shape[:-1], -1, 32)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    lut = torch.tensor(FP4_VALUES, dtype=torch.float32)
    code = ((g / torch.exp2(e)[..., None])[..., None] - lut).abs().argmin(-1).to(torch.uint8)
    return (code[..., 0::2] | (code[..., 1::2] << 4)).contiguous(), (e + 127).to(torch.uint8).contiguous()


def recipe_sources(recipe: dict) -> list:
    """Checkpoint tensors a derived-weight recipe reads."""
    if recipe["op"] == "cat":
        return list(recipe["parts"])
    if recipe["op"] == "stack_experts":
        return [f"{recipe['prefix']}.{e}.{part}.weight" for e in expert_range(recipe["n"], recipe.get("ep", 1), recipe.get("rank", 0))
                for part in recipe["parts"]] + list(recipe.get("tail", []))
    if recipe["op"] == "fused_experts":          # either the plain tensor or its fp4 blocks + scales
        return [recipe["src"]]
    if recipe["op"] == "cols":
        return [recipe["src"]]
    raise ValueError(f"unknown derived-weight recipe '{recipe['op']}'")


def missing_weights(pkt, ckpt) -> list:
    """Names the packet binds by (directly or through its derived-weight recipes) that the checkpoint does not hold."""
    from ..compiler.packet import TClass
    derived = pkt.section_json("derived_weights.json") or {}
    want = set()
    for t in pkt.tensors:
        if t.tclass == TClass.WEIGHT:
            want.add(t.name)
        elif t.tclass == TClass.DERIVED and t.name in derived:
            want.update(recipe_sources(derived[t.name]))
    return sorted(n for n in want if not ckpt.has(n) and not (ckpt.has(n + "_blocks") and ckpt.has(n + "_scales")))


SCALE_SUFFIX = "_scale_inv"      # block-quantised checkpoints: <name> holds e4m3 codes, <name>_scale_inv one f32 per 128 x 128 block


def is_block_fp8(ckpt, name: str) -> bool:
    return ckpt.has(name + SCALE_SUFFIX)


def dequant_block_fp8(q: torch.Tensor, scale_inv: torch.Tensor, row0: int = 0, col0: int = 0) -> torch.Tensor:
    """codes [n, k] (a slice starting at (row0, col0) of the full matrix) times their 128 x 128 block scales -> bf16."""
    n, k = q.shape
    r = (torch.arange(n) + row0) // 128
    c = (torch.arange(k) + col0) // 128
    return (q.float() * scale_inv.float()[r][:, c]).to(torch.bfloat16)


def shard_slice(ckpt: Checkpoint, name: str, shard_axis, tp: int, rank: int) -> torch.Tensor:
    """The rank's part of a checkpoint tensor.  A block-quantised tensor (e4m3 codes + ``_scale_inv``) comes back
    dequantised to bf16: callers that want the codes themselves use :func:`fp8_codes`."""
    if is_block_fp8(ckpt, name):
        scale = ckpt.get(name + SCALE_SUFFIX)
        if shard_axis is None or shard_axis == 0xFFFFFFFF or tp == 1:
            return dequant_block_fp8(ckpt.get(name), scale)
        n = ckpt.shape(name)[shard_axis]
        per = n // tp
        q = ckpt.get_slice(name, shard_axis, rank * per, (rank + 1) * per)
        return dequant_block_fp8(q, scale, rank * per if shard_axis == 0 else 0, rank * per if shard_axis == 1 else 0)
    if shard_axis is None or shard_axis == 0xFFFFFFFF or tp == 1:
        return ckpt.get(name)
    n = ckpt.shape(name)[shard_axis]
    if n % tp:
        raise ValueError(f"{name}: axis {shard_axis} of size {n} does not divide over tp={tp}")
    per = n // tp
    return ckpt.get_slice(name, shard_axis, rank * per, (rank + 1) * per)


def expert_range(n_experts: int, ep: int, rank: int) -> range:
    """Contiguous balanced expert ranges per rank."""
    per = n_experts // ep
    return range(rank * per, (rank + 1) * per)


def fp8_codes(name: str, ent, recipe: dict | None, ckpt, tp: int = 1, rank: int = 0):
    """(e4m3 codes, f32 block scales) of a packet tensor taken straight from a block-quantised checkpoint, or None when
    the checkpoint is not quantised that way or the pieces do not line up with 128-row blocks (the caller then
    dequantises and quantises again).  Covers plain tensors, row concatenations and stacked experts, unsharded."""
    if tp != 1:
        return None

    def one(n):
        if not is_block_fp8(ckpt, n):
            return None
        q, s = ckpt.get(n), ckpt.get(n + SCALE_SUFFIX).float()
        if q.dtype != torch.float8_e4m3fn or q.dim() != 2 or (q.shape[0] % 128 and recipe is not None):
            return None
        return q, s
    if recipe is None:
        return one(name)
    if recipe["op"] == "cat" and recipe.get("axis", 0) == 0:
        parts = [one(p) for p in recipe["parts"]]
    elif recipe["op"] == "stack_experts":
        names = [f"{recipe['prefix']}.{e}.{part}.weight" for e in expert_range(recipe["n"], recipe.get("ep", 1), recipe.get("rank", 0))
                 for part in recipe["parts"]] + list(recipe.get("tail", []))
        parts = [one(p) for p in names]
    else:
        return None
    if any(p is None for p in parts):
        return None
    return torch.cat([p[0].view(torch.uint8) for p in parts], 0).view(torch.float8_e4m3fn).contiguous(), torch.cat([p[1] for p in parts], 0).contiguous()


def materialize(name: str, ent, recipe: dict | None, ckpt: Checkpoint, tp: int = 1, rank: int = 0) -> torch.Tensor:
    """Build the tensor behind a WEIGHT or DERIVED packet entry (host memory, checkpoint dtype)."""
    if recipe is None:
        return shard_slice(ckpt, name, ent.shard_axis, tp, rank)
    if recipe["op"] == "cat":
        parts = [shard_slice(ckpt, p, recipe.get("shard_axis"), tp, rank) for p in recipe["parts"]]
        return torch.cat(parts, dim=recipe.get("axis", 0)).contiguous()
    if recipe["op"] == "stack_experts":
        rows = []
        for e in expert_range(recipe["n"], recipe.get("ep", 1), recipe.get("rank", 0)):
            for part in recipe["parts"]:
                rows.append(shard_slice(ckpt, f"{recipe['prefix']}.{e}.{part}.weight", None, 1, 0))
        for name in recipe.get("tail", []):      # shared expert stacked behind the routed ones (replicated on every rank)
            rows.append(shard_slice(ckpt, name, None, 1, 0))
        return torch.cat(rows, dim=0).contiguous()
    if recipe["op"] == "fused_experts":        # gpt_oss: every expert of a projection in one tensor
        er = list(expert_range(recipe["n"], recipe.get("ep", 1), recipe.get("rank", 0)))
        kind = recipe["kind"]
        if not ckpt.has(recipe["src"]) and ckpt.has(recipe["src"] + "_blocks"):
            # the original release: fp4 blocks of the transposed matrices, [E, 2F, H/32, 16] (gate / up rows interleaved)
            # and [E, H, F/32, 16]; this rank's experts are dequantised and are already row-major for the expert op
            dt = ckpt.get(recipe["src"] + "_bias").dtype if ckpt.has(recipe["src"] + "_bias") else torch.bfloat16     # the model's own dtype
            w = dequant_mxfp4(shard_slice(ckpt, recipe["src"] + "_blocks", None, 1, 0)[er],
                              shard_slice(ckpt, recipe["src"] + "_scales", None, 1, 0)[er], dt)
            if kind == "gate_up":
                return torch.cat([w[:, 0::2], w[:, 1::2]], 1).reshape(-1, w.shape[2]).contiguous()
            return w.reshape(-1, w.shape[2]).contiguous()
        t = shard_slice(ckpt, recipe["src"], None, 1, 0)[er]
        if kind == "gate_up":                  # [e, H, 2F], gate / up columns interleaved -> [e * (F gate rows + F up rows), H]
            return torch.cat([t[:, :, 0::2].transpose(1, 2), t[:, :, 1::2].transpose(1, 2)], 1).reshape(-1, t.shape[1]).contiguous()
        if kind == "down":                     # [e, F, H] -> [e * H, F]
            return t.transpose(1, 2).reshape(-1, t.shape[1]).contiguous()
        if kind == "gate_up_bias":             # [e, 2F] interleaved -> gate part then up part per expert
            return torch.cat([t[:, 0::2], t[:, 1::2]], 1).reshape(-1).contiguous()
        if kind == "down_bias":
            return t.reshape(-1).contiguous()
        raise ValueError(f"unknown fused-experts part '{kind}'")
    if recipe["op"] == "cols":                 # a column range of a checkpoint matrix (a half of eh_proj)
        if is_block_fp8(ckpt, recipe["src"]):
            return shard_slice(ckpt, recipe["src"], None, 1, 0)[:, recipe["start"]:recipe["stop"]].contiguous()
        return ckpt.get_slice(recipe["src"], 1, recipe["start"], recipe["stop"]).contiguous()
    raise ValueError(f"unknown derived-weight recipe '{recipe['op']}'")
