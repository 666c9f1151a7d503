"""Prefill / decode disaggregation inside one server: a prefill engine runs the prompt, exports the slot's KV image,
a decode engine imports it and continues (reference: crates/plowrt/src/serve/pd.rs:1-8,
docs/arch/30-heterogeneous-serving.md:213-335).  Both engines load the same packet; they may sit on different GPUs."""
from __future__ import annotations

import numpy as np

from ..runtime.engine import EngineBase, TokenBatch
from ..runtime.kv_image import KvImage, export_slot, import_slot


class PdPipeline:
    def __init__(self, prefill: EngineBase, decode: EngineBase, wire: bool = False):
        self.p, self.d, self.wire = prefill, decode, wire
        self.bytes_moved = 0

    def prefill(self, slot: int, prompt: list, chunk: int | None = None) -> tuple:
        """Run the prompt on the prefill engine; returns (first generated token, KV image)."""
        eng = self.p
        cached = eng.begin_slot(slot, prompt)
        eng.reserve(slot, len(prompt) + 1)
        cached = min(cached, len(prompt) - 1)          # at least the last token is computed to get its logits
        chunk = chunk or eng.max_rows(False)
        first = None
        at = cached
        while at < len(prompt):
            part = prompt[at:at + chunk]
            r = eng.step(TokenBatch(np.asarray(part, np.int32), np.arange(at, at + len(part), dtype=np.int32),
                                    np.full(len(part), slot, np.int32), np.asarray([len(part) - 1], np.int32)))
            first = int(r.ids[0])
            eng.commit(slot, part) if at >= len(eng.tokens[slot]) else eng.commit(slot, part[len(eng.tokens[slot]) - at:])
            at += len(part)
        img = export_slot(eng, slot)
        eng.retire_slot(slot)
        return first, img

    def handoff(self, slot: int, img: KvImage) -> None:
        if self.wire:                                   # serialise as a cross-process transfer would
            b = img.to_bytes()
            self.bytes_moved += len(b)
            img = KvImage.from_bytes(b)
        else:
            self.bytes_moved += img.nbytes()
        import_slot(self.d, slot, img)

    def decode(self, slot: int, first: int, max_new: int, eos=()) -> list:
        eng = self.d
        out, cur = [first], first
        while len(out) < max_new and cur not in eos:
            n = len(eng.tokens[slot])
            eng.reserve(slot, n + 2)
            r = eng.step(TokenBatch(np.asarray([cur], np.int32), np.asarray([n], np.int32), np.asarray([slot], np.int32),
                                    np.asarray([0], np.int32), decode=True))
            eng.commit(slot, [cur])
            cur = int(r.ids[0])
            out.append(cur)
        return out

    def generate(self, prompt: list, max_new: int, p_slot: int = 0, d_slot: int = 0, eos=()) -> list:
        first, img = self.prefill(p_slot, prompt)
        self.handoff(d_slot, img)
        return self.decode(d_slot, first, max_new, eos)
