"""Device-memory budget of a packet: what the weights, the activation arenas, the recurrent state and the KV pages take,
and how many pages (tokens, full-length sequences) fit in what is left.

Everything is computed from the packet alone (tensor table, programs, metadata), so ``plowrt budget`` answers "does this
model fit, and with how much context" before a single byte is loaded, and a launcher can turn a memory share into an
explicit page count (``--kv-pages``).  Weights the programs read as block-scaled e4m3 count one byte per element plus
their 128 x 128 block scales, everything else its table dtype; every prepared program owns an arena, so the arenas are
reported both as their sum (all programs prepared) and as the largest one.

Reference: crates/plowrt/src/memory/budget.rs (weights + KV + activation budget against device memory),
crates/plow-asset/src/serve_manifest.rs (``KvGeometry``).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

from ..compiler import packet as pk
from .fp8_dir import fp8_weight_handles
from .kv_pages import PAGE


@dataclass
class MemoryPlan:
    weights_bytes: int
    fp8_weight_bytes: int            # the part of weights_bytes held as e4m3 codes + block scales
    arena_bytes_sum: int
    arena_bytes_max: int
    state_bytes: int                 # recurrent state of max_slots sequences
    page_bytes: int                  # one 64-token KV page across all layers (cells + scales)
    io_bytes: int                    # step inputs / outputs / logits
    budget_bytes: int                # what the KV pool may take
    n_pages: int
    kv_tokens: int
    full_sequences: int              # sequences of max_ctx tokens that fit at once
    pages_wanted: int                # max_slots sequences of max_ctx tokens
    fits: bool                       # weights + arenas + state + io + one full sequence fit

    def to_json(self) -> dict:
        return asdict(self)


def _nbytes(t: pk.TensorEnt, rows=0, samples=0, pages=1, slots=1) -> int:
    n = pk.DTYPE_BYTES[pk.DType(t.dtype)]
    for d in t.dims:
        n *= rows if d == -1 else samples if d == -2 else pages if d == -3 else slots if d == -4 else int(d)
    return n


def plan_memory(pkt: pk.Packet, device_bytes: int, max_slots: int, max_ctx: int, kv_fraction: float = 0.9,
                reserve_bytes: int = 2 << 30) -> MemoryPlan:
    """``device_bytes``: memory of the GPU (or what is free on it); ``kv_fraction``: share of what remains after the
    weights, arenas, state and a fixed reserve (library workspaces, graphs) that the KV pool may take."""
    from ..models.config import ModelSpec
    spec = ModelSpec.from_json(pkt.sections["model.json"].decode())
    fp8 = fp8_weight_handles(pkt, spec.weight_quant)
    weights = fp8_bytes = 0
    for h, t in enumerate(pkt.tensors):
        if t.tclass not in (pk.TClass.WEIGHT, pk.TClass.DERIVED, pk.TClass.GEN):
            continue
        if h in fp8 and len(t.dims) == 2:
            n, k = int(t.dims[0]), int(t.dims[1])
            b = n * k + 4 * ((n + 127) // 128) * ((k + 127) // 128)
            fp8_bytes += b
            weights += b
        else:
            weights += _nbytes(t)
    arenas = [int(p.arena_bytes) for p in pkt.programs]
    max_rows = max(p.rows for p in pkt.programs)
    state = sum(_nbytes(t, slots=max_slots + 1) for t in pkt.tensors if t.tclass == pk.TClass.STATE)
    page = sum(_nbytes(t, pages=1) for t in pkt.tensors if t.tclass == pk.TClass.KV)
    io = sum(_nbytes(t, rows=max_rows, samples=max_rows) for t in pkt.tensors if t.tclass in (pk.TClass.INPUT, pk.TClass.OUTPUT))
    fixed = weights + sum(arenas) + state + io + reserve_bytes
    budget = max(0, int((device_bytes - fixed) * kv_fraction))
    pages_per_seq = (max_ctx + PAGE - 1) // PAGE
    n_pages = budget // page if page else 0
    return MemoryPlan(weights_bytes=weights, fp8_weight_bytes=fp8_bytes, arena_bytes_sum=sum(arenas), arena_bytes_max=max(arenas),
                      state_bytes=state, page_bytes=page, io_bytes=io, budget_bytes=budget, n_pages=int(n_pages),
                      kv_tokens=int(n_pages) * PAGE, full_sequences=int(n_pages // pages_per_seq) if pages_per_seq else 0,
                      pages_wanted=max_slots * pages_per_seq, fits=bool(page == 0 or n_pages >= pages_per_seq))
