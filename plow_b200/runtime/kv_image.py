"""KV image: the cache content of one sequence as a self-describing blob, for prefill/decode disaggregation,
session retention and slot migration between engines of the same packet.

An image carries the token ids whose KV it holds, the packet hash it belongs to and, per KV tensor of the packet,
the sequence's pages in order ([n_pages, 64, ...]; e4m3 tensors travel as raw bytes).  ``import_slot`` seats the
sequence in another engine (prefix-cache hits on the destination are kept), copies the pages that are not already
there and publishes them, after which decoding continues at position ``len(tokens)``.
Reference: crates/plow-asset/src/kv_image.rs, crates/plowrt/src/exec/kv_image.rs, serve/pd.rs:1-8.
"""
from __future__ import annotations

import io
import json
from dataclasses import dataclass, field

import numpy as np

from .engine import EngineBase, EngineError
from .kv_pages import PAGE


@dataclass
class KvImage:
    packet_hash: str
    tokens: list
    arrays: dict = field(default_factory=dict)       # name -> np.ndarray [n_pages, 64, ...] (uint8 for e4m3)

    @property
    def n_pages(self) -> int:
        return (len(self.tokens) + PAGE - 1) // PAGE

    def nbytes(self) -> int:
        return sum(a.nbytes for a in self.arrays.values())

    def to_bytes(self) -> bytes:
        buf = io.BytesIO()
        meta = json.dumps(dict(packet_hash=self.packet_hash, tokens=self.tokens, names=list(self.arrays)))
        np.savez(buf, __meta__=np.frombuffer(meta.encode(), dtype=np.uint8), **{f"a{i}": a for i, a in enumerate(self.arrays.values())})
        return buf.getvalue()

    @staticmethod
    def from_bytes(b: bytes) -> "KvImage":
        z = np.load(io.BytesIO(b))
        meta = json.loads(bytes(z["__meta__"]).decode())
        return KvImage(meta["packet_hash"], meta["tokens"], {n: z[f"a{i}"] for i, n in enumerate(meta["names"])})


def _to_numpy(a, pages):
    if isinstance(a, np.ndarray):
        return a[pages].copy()
    import torch
    t = a[torch.as_tensor(pages, dtype=torch.long, device=a.device)]
    if t.dtype == torch.float8_e4m3fn:
        t = t.view(torch.uint8)
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy()
    return t.cpu().numpy()


def _from_numpy(a, pages, src):
    if isinstance(a, np.ndarray):
        a[pages] = src
        return
    import torch
    t = torch.from_numpy(np.ascontiguousarray(src)).to(a.device)
    if a.dtype == torch.float8_e4m3fn:
        t = t.view(torch.float8_e4m3fn)
    elif a.dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    a[torch.as_tensor(pages, dtype=torch.long, device=a.device)] = t


def export_slot(engine: EngineBase, slot: int) -> KvImage:
    tokens = list(engine.tokens[slot])
    n_pages = (len(tokens) + PAGE - 1) // PAGE
    pages = list(engine.pool.seqs[slot].pages[:n_pages])
    img = KvImage(engine.packet.content_hash.hex(), tokens)
    for name, arr in engine.kv_arrays().items():
        img.arrays[name] = _to_numpy(arr, pages)
    # recurrent state (gated delta rule: conv history + S matrix) is per slot, not per page
    for name, arr in engine.state_arrays().items():
        img.arrays["slot/" + name] = _to_numpy(arr, [slot])
    return img


def import_slot(engine: EngineBase, slot: int, img: KvImage) -> int:
    """Seat ``img`` in ``slot``; returns how many tokens were already cached on this engine."""
    if img.packet_hash != engine.packet.content_hash.hex():
        raise EngineError("KV image belongs to a different packet")
    state = engine.state_arrays()
    if state and any("slot/" + n not in img.arrays for n in state):
        raise EngineError("KV image carries no recurrent state for this packet")
    cached = engine.begin_slot(slot, img.tokens)
    engine.reserve(slot, len(img.tokens) + 1)
    first = cached // PAGE                      # pages fully covered by the destination's prefix cache stay untouched
    pages = list(engine.pool.seqs[slot].pages[first:img.n_pages])
    if pages:
        for name, arr in engine.kv_arrays().items():
            _from_numpy(arr, pages, img.arrays[name][first:img.n_pages])
    for name, arr in state.items():
        _from_numpy(arr, [slot], img.arrays["slot/" + name])
    engine.commit(slot, img.tokens[cached:])
    return cached
