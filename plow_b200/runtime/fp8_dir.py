"""Pre-quantised weight twins on disk.

The sm_100a engine runs the projections of a ``fp8_block128`` model on e4m3 weights with one f32 scale per 128 x 128
block.  Quantising them at every load costs a pass over the whole checkpoint; ``plowc --fp8-dir`` does it once and
writes the twins next to the packet (``<assets>/fp8[/rank<r>]``: safetensors shards with the e4m3 bytes under the packet
tensor's name and the scales under ``<name>.scale``, plus an index that records the packet's content hash).  The engine
takes a twin from there when the index matches the packet it loaded, and quantises on the spot otherwise.

Reference: crates/plowrt/src/asset/ (fp8 weight directories next to the checkpoint), crates/plow-asset/src/derived_weights.rs.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..compiler import packet as pk
from ..compiler.packet import Op

INDEX = "fp8_index.json"


def fp8_weight_handles(pkt: pk.Packet, weight_quant: str) -> set:
    """Handles of the weight tensors some instruction reads as block-scaled e4m3."""
    out = set()
    for p in pkt.programs:
        for ins in p.insts:
            if ins.op in (Op.GEMM, Op.GEMM_XREDUCE) and ins.i[2] & pk.GEMM_FP8_BLOCK:
                out.add(ins.t[2])
            if ins.op == Op.MOE_GEMM and weight_quant == "fp8_block128":
                out.update([ins.t[3], ins.t[4]])
    out.discard(pk.T_NONE)
    return out


def _dir(assets, rank: int) -> Path:
    return Path(assets) / "fp8" / (f"rank{rank}" if rank else "")


def write_fp8_dir(assets, packet_name: str = "model.pkt", rank: int = 0, tp: int = 1, shard_bytes: int = 2 << 30, device="cpu") -> dict:
    """Quantise every e4m3-read weight of the packet and store the twins; returns the index."""
    from safetensors.torch import save_file
    from ..models.config import ModelSpec
    from ..ops import quant
    from .weights import materialize, open_checkpoint
    assets = Path(assets)
    pkt = pk.read_packet(assets / packet_name)
    spec = ModelSpec.from_json(pkt.sections["model.json"].decode())
    derived = pkt.section_json("derived_weights.json") or {}
    ckpt = open_checkpoint(assets / "checkpoint")
    out = _dir(assets, rank)
    out.mkdir(parents=True, exist_ok=True)
    shards, cur, size, where = [], {}, 0, {}

    def flush():
        nonlocal cur, size
        if cur:
            fn = f"fp8-{len(shards) + 1:05d}.safetensors"
            save_file(cur, str(out / fn))
            shards.append(fn)
            for k in cur:
                where[k] = fn
            cur, size = {}, 0
    for h in sorted(fp8_weight_handles(pkt, spec.weight_quant)):
        ent = pkt.tensors[h]
        w = materialize(ent.name, ent, derived.get(ent.name), ckpt, tp, rank).to(device=device, dtype=torch.bfloat16)
        q, s = quant.quant_weight_128x128(w)
        cur[ent.name] = q.view(torch.uint8).cpu().contiguous()
        cur[ent.name + ".scale"] = s.float().cpu().contiguous()
        size += q.numel() + s.numel() * 4
        if size >= shard_bytes:
            flush()
    flush()
    index = dict(packet_sha256=pkt.content_hash.hex() if isinstance(pkt.content_hash, bytes) else str(pkt.content_hash),
                 rank=rank, tp=tp, block=128, weight_map=where)
    (out / INDEX).write_text(json.dumps(index, indent=1))
    return index


class Fp8Dir:
    """The twins of one rank, if they were written for the packet in hand."""

    def __init__(self, assets, pkt: pk.Packet, rank: int = 0):
        self.dir = _dir(assets, rank)
        self.map: dict = {}
        self._handles: dict = {}
        f = self.dir / INDEX
        if not f.exists():
            return
        idx = json.loads(f.read_text())
        have = pkt.content_hash.hex() if isinstance(pkt.content_hash, bytes) else str(pkt.content_hash)
        if idx.get("packet_sha256") != have or idx.get("rank") != rank:
            return                      # written for another build of the packet: not trusted
        self.map = idx["weight_map"]

    def __bool__(self) -> bool:
        return bool(self.map)

    def get(self, name: str, device):
        """(e4m3 [N, K], f32 scales) or None."""
        if name not in self.map or name + ".scale" not in self.map:
            return None
        from safetensors import safe_open
        fn = self.map[name]
        if fn not in self._handles:
            self._handles[fn] = safe_open(str(self.dir / fn), framework="pt")
        h = self._handles[fn]
        q = h.get_tensor(name).to(device).view(torch.float8_e4m3fn)
        s = self._handles[self.map[name + ".scale"]].get_tensor(name + ".scale") if self.map[name + ".scale"] == fn else None
        if s is None:
            fs = self.map[name + ".scale"]
            if fs not in self._handles:
                self._handles[fs] = safe_open(str(self.dir / fs), framework="pt")
            s = self._handles[fs].get_tensor(name + ".scale")
        return q, s.to(device)
