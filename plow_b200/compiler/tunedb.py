"""Measurement store keyed by hardware fingerprint.

Records live under ``<root>/<vendor>/<isa>/<sku>/<kind>.json`` (kinds: gemm, gemv, attention, projection,
moe_decode); a record maps a shape key to the measured best configuration and its time.  The compiler's tile picker
and the runtime's split-K choice consult the store first and fall back to the analytical model
(reference: crates/tunedb/src/{store,record}.rs; ``plowc tune``)."""
from __future__ import annotations

import json
import os
import time
from pathlib import Path

KINDS = ("gemm", "gemv", "attention", "projection", "moe_decode")


def fingerprint(vendor="nvidia", isa="sm_100a", sku="b200") -> tuple:
    return vendor, isa, sku


def device_fingerprint() -> tuple:
    try:
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            return "nvidia", f"sm_{p.major}{p.minor}{'a' if p.major >= 9 else ''}", p.name.lower().replace("nvidia ", "").replace(" ", "-")
    except Exception:
        pass
    return "cpu", "generic", "host"


def gemm_key(M, N, K, dtype, dual=False, grouped=0) -> str:
    return f"m{M}_n{N}_k{K}_{dtype}{'_glu' if dual else ''}{f'_e{grouped}' if grouped else ''}"


class TuneDb:
    def __init__(self, root=None, fp: tuple | None = None):
        self.root = Path(root or os.environ.get("PLOW_TUNEDB", Path(__file__).resolve().parent.parent / "tuning"))
        self.fp = fp or fingerprint()
        self._cache = {}

    def _path(self, kind: str) -> Path:
        if kind not in KINDS:
            raise ValueError(f"unknown record kind '{kind}'")
        return self.root.joinpath(*self.fp, f"{kind}.json")

    def _load(self, kind: str) -> dict:
        if kind not in self._cache:
            p = self._path(kind)
            self._cache[kind] = json.loads(p.read_text()) if p.exists() else {}
        return self._cache[kind]

    def lookup(self, kind: str, key: str):
        return self._load(kind).get(key)

    def record(self, kind: str, key: str, config: dict, us: float, note: str = "") -> bool:
        """Keep the faster of the stored and the new measurement; returns True when the store changed."""
        d = self._load(kind)
        old = d.get(key)
        if old is not None and old["us"] <= us:
            return False
        d[key] = dict(config=config, us=round(float(us), 3), when=int(time.time()), note=note)
        p = self._path(kind)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(".tmp")
        tmp.write_text(json.dumps(d, indent=1, sort_keys=True))
        tmp.replace(p)
        return True

    def keys(self, kind: str) -> list:
        return sorted(self._load(kind))


def tune_gemm(db: TuneDb, shapes, iters: int = 10) -> list:
    """Measure swap-mode tile width and split-K choices for decode GEMM shapes on the current GPU."""
    import torch

    from ..ops import gemm, native
    out = []
    for (M, N, K, fp8, dual) in shapes:
        if fp8:
            x = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
            w = torch.randn(N * (2 if dual else 1), K, device="cuda").to(torch.float8_e4m3fn)
            sx = torch.rand(K // 128, M, device="cuda")
            sw = torch.rand(w.shape[0] // 128, K // 128, device="cuda")
        else:
            x, w, sx, sw = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N * (2 if dual else 1), K, device="cuda").bfloat16(), None, None
        best = None
        for bn in (32, 64, 128):
            if bn < M:
                continue
            for s in sorted({1, gemm.pick_splits(M, N, K, fp8, dual, bn)}):
                try:
                    fn = lambda: gemm.gemm(x, w, sx=sx, sw=sw, dual=dual, n_out=N, swap=True, bn=bn, splits=s)
                    for _ in range(3):
                        fn()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for _ in range(4):
                            fn()
                    g.replay()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(iters):
                        g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / (iters * 4)
                except native.NativeLibraryError:
                    continue
                if best is None or us < best[1]:
                    best = (dict(swap=True, bn=bn, splits=s), us)
        if best:
            key = gemm_key(M, N, K, "e4m3" if fp8 else "bf16", dual)
            db.record("gemm", key, best[0], best[1])
            out.append((key, best))
    return out
