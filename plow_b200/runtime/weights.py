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


def shard_slice(ckpt: Checkpoint, name: str, shard_axis, tp: int, rank: int) -> torch.Tensor:
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
                rows.append(ckpt.get(f"{recipe['prefix']}.{e}.{part}.weight"))
        for name in recipe.get("tail", []):      # shared expert stacked behind the routed ones (replicated on every rank)
            rows.append(ckpt.get(name))
        return torch.cat(rows, dim=0).contiguous()
    if recipe["op"] == "cols":                 # a column range of a checkpoint matrix (a half of eh_proj)
        return ckpt.get_slice(recipe["src"], 1, recipe["start"], recipe["stop"]).contiguous()
    raise ValueError(f"unknown derived-weight recipe '{recipe['op']}'")
