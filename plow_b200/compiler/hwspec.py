"""Hardware registry: the facts the cost model, the scheduler and the runtime planner share.

Only Blackwell B200 (sm_100a) is a compile target for device code; a ``cpu`` entry exists for the
hermetic CPU interpreter.  Peaks come in two flavours: nominal (datasheet) and measured (a JSON file
of measured copy bandwidth / GEMM throughput that the caller names, ``lookup(..., peaks_file=...)`` or
``--peaks`` on the tools), and every roofline fraction the tools print says which one it used.  Reference counterpart: crates/hwspec (registry.rs, isa.rs,
nvidia/blackwell.rs:57-118).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path


@dataclass(frozen=True)
class IsaCaps:
    mma_sync: bool = False
    wgmma: bool = False
    tcgen05: bool = False
    tmem: bool = False
    tma: bool = False
    clusters: bool = False
    nvls_multimem: bool = False
    fp8: bool = False
    fp4: bool = False


@dataclass(frozen=True)
class GpuSpec:
    name: str
    arch: str
    sm_count: int
    smem_per_cta: int           # bytes, opt-in maximum
    tmem_cols: int              # 32-bit columns x 128 lanes per SM
    l2_bytes: int
    hbm_bytes: int
    hbm_gbs: float              # nominal
    bf16_tflops: float          # nominal dense
    fp8_tflops: float
    fp4_tflops: float
    nvlink_gbs_dir: float       # per direction per GPU
    nvlink_domain: int
    sm_clock_mhz: int
    isa: IsaCaps = field(default_factory=IsaCaps)
    measured: dict = field(default_factory=dict)

    def hbm_peak(self) -> tuple:
        """(GB/s, 'measured'|'nominal')"""
        if "hbm_gbs" in self.measured:
            return float(self.measured["hbm_gbs"]), "measured"
        return self.hbm_gbs, "nominal"

    def bf16_peak(self, sustained: bool = False) -> tuple:
        key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
        if key in self.measured:
            return float(self.measured[key]), "measured"
        return self.bf16_tflops, "nominal"


B200_ISA = IsaCaps(mma_sync=True, wgmma=False, tcgen05=True, tmem=True, tma=True, clusters=True,
                   nvls_multimem=True, fp8=True, fp4=True)

_REGISTRY = {
    "b200": GpuSpec(name="NVIDIA B200", arch="sm_100a", sm_count=148, smem_per_cta=227 * 1024, tmem_cols=512,
                    l2_bytes=126 * 2 ** 20, hbm_bytes=180 * 10 ** 9, hbm_gbs=7700.0, bf16_tflops=2250.0,
                    fp8_tflops=4500.0, fp4_tflops=9000.0, nvlink_gbs_dir=900.0, nvlink_domain=8,
                    sm_clock_mhz=1965, isa=B200_ISA),
    "cpu": GpuSpec(name="host cpu", arch="cpu", sm_count=8, smem_per_cta=0, tmem_cols=0, l2_bytes=32 * 2 ** 20,
                   hbm_bytes=64 * 10 ** 9, hbm_gbs=100.0, bf16_tflops=1.0, fp8_tflops=1.0, fp4_tflops=1.0,
                   nvlink_gbs_dir=10.0, nvlink_domain=1, sm_clock_mhz=3000),
}

SUPPORTED_ARCHS = ("sm_100a", "cpu")


def lookup(name: str, peaks_file: str | Path | None = None) -> GpuSpec:
    """Registry entry for ``name``.  ``peaks_file`` (JSON with hbm_gbs / bf16_tflops / bf16_tflops_sustained measured on
    the machine at hand) attaches measured peaks; without it only the nominal figures are known."""
    key = name.lower().replace("nvidia ", "")
    if key not in _REGISTRY:
        raise KeyError(f"unknown device '{name}'; known: {sorted(_REGISTRY)}")
    spec = _REGISTRY[key]
    if key == "b200" and peaks_file is not None and Path(peaks_file).exists():
        try:
            m = json.loads(Path(peaks_file).read_text())
            spec = GpuSpec(**{**spec.__dict__, "measured": {k: m[k] for k in
                                                          ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") if k in m}})
        except (OSError, ValueError):
            pass
    return spec


def check_arch(arch: str) -> None:
    """This build emits device code for sm_100a only (and the CPU interpreter)."""
    if arch not in SUPPORTED_ARCHS:
        raise ValueError(f"--arch {arch}: no interpreter object is defined; supported: {', '.join(SUPPORTED_ARCHS)}")
