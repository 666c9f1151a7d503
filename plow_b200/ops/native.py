"""ctypes bindings of the in-tree native libraries.

The CUDA library is loaded lazily and *loudly*: on a machine with a GPU a missing or unloadable
``libplow_cuda.so`` raises instead of falling back to PyTorch, so a silent eager path can never
stand in for the hand-written kernels.
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache
from pathlib import Path

# PLOW_LIBDIR points at an alternative build of the libraries (e.g. one compiled with -DPLOW_DEVICE_TRACE)
LIBDIR = Path(os.environ["PLOW_LIBDIR"]) if os.environ.get("PLOW_LIBDIR") else Path(__file__).resolve().parent.parent / "lib"


class NativeLibraryError(RuntimeError):
    pass


class GemmDesc(C.Structure):
    """Mirror of ``PlowGemmDesc`` (csrc/cuda/gemm_api.h)."""
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("y", C.c_void_p), ("sx", C.c_void_p),
        ("sw", C.c_void_p), ("residual", C.c_void_p), ("yq", C.c_void_p), ("syq", C.c_void_p),
        ("grp_off", C.c_void_p), ("tile_prefix", C.c_void_p), ("status", C.c_void_p),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("ldx", C.c_int32), ("ldw", C.c_int32), ("ldy", C.c_int32), ("ld_sx", C.c_int32),
        ("ld_syq", C.c_int32), ("E", C.c_int32),
        ("w_rows", C.c_int64),
        ("dtype", C.c_int32), ("dual", C.c_int32), ("swap", C.c_int32), ("bn", C.c_int32),
        ("out_f32", C.c_int32), ("out_scale", C.c_float),
        ("ws", C.c_void_p), ("ws_ctr", C.c_void_p), ("splits", C.c_int32), ("stream", C.c_int32),
        ("ar_peer", C.c_void_p * 8), ("ar_part_ofs", C.c_uint64), ("ar_flag_ofs", C.c_uint64), ("ar_done_ofs", C.c_uint64),
        ("ar_y_ofs", C.c_uint64), ("ar_epoch", C.c_void_p), ("ar_world", C.c_int32), ("ar_me", C.c_int32),
        ("wait_ctr", C.c_void_p), ("wait_epoch", C.c_void_p), ("wait_mult", C.c_int32), ("wait_deadline_ms", C.c_int32),
        ("ar_oneshot", C.c_int32), ("ar_pad", C.c_int32), ("ar_half_bytes", C.c_uint64),
        ("ar_mc", C.c_void_p), ("ar_tdone_ofs", C.c_uint64),
    ]


def _ensure_built(name: str) -> Path:
    path = LIBDIR / name
    if not path.exists() and os.environ.get("PLOW_NO_AUTOBUILD") != "1":
        from .. import build
        (build.build_cuda if "cuda" in name else build.build_cpu)()
    if not path.exists():
        raise NativeLibraryError(f"{path} is missing; run `python -m plow_b200.build`")
    return path


@lru_cache(maxsize=None)
def cuda_lib() -> C.CDLL:
    """The sm_100a kernel library.  Raises if it cannot be loaded."""
    import torch  # noqa: F401  (loads libcudart / initialises the allocator first)
    lib = C.CDLL(str(_ensure_built("libplow_cuda.so")), mode=C.RTLD_GLOBAL)
    lib.plow_gemm.argtypes = [C.POINTER(GemmDesc), C.c_void_p]
    lib.plow_gemm.restype = C.c_int
    return lib


@lru_cache(maxsize=None)
def cpu_lib() -> C.CDLL:
    """The CPU packet interpreter + golden ops."""
    return C.CDLL(str(_ensure_built("libplow_cpu.so")))


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


_status = {}


def status_word(device=None):
    """One int32 device word per GPU that kernels write error codes into (0 = ok)."""
    import torch
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev not in _status:
        _status[dev] = torch.zeros(4, dtype=torch.int32, device=dev)
    return _status[dev]


STATUS_NAMES = {
    0: "ok", 1: "tma stage never landed", 2: "smem stage never freed", 3: "accumulator never completed",
    4: "accumulator never drained", 5: "peer flag never arrived", 6: "device bounds check failed",
    7: "in-grid counter wait ran out",
}


KERNEL_FAMILIES = {0: "?", 1: "gemm", 2: "mla_decode", 3: "mla_absorb/fold", 4: "gqa_attention", 5: "dsa", 6: "ep dispatch/combine",
                   7: "all-gather push", 8: "gdn", 9: "interpreter", 10: "tp all-reduce + norm"}


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises on a recorded device-side error.  The word is
    ``code | (kernel family << 8)`` (csrc/cuda/ptx.cuh)."""
    s = status_word(device)
    word = int(s[0].item())
    if word != 0:
        s.zero_()
        code, fam = word & 0xFF, word >> 8
        raise NativeLibraryError(f"device kernel reported status {code}: {STATUS_NAMES.get(code, '?')} "
                                 f"(kernel family: {KERNEL_FAMILIES.get(fam, fam)})")


# ---- compact ctypes signatures: p = pointer, i = int32, l = int64, f = float ----------------------
_SIGS = {
    "plow_embed": "pppiifp",
    "plow_rmsnorm": "pppipp" "iiifip",
    "plow_add_norm": "pppippppiifip",
    "plow_quant_act": "ppipiiip",
    "plow_mla_q_prep": "pppippiiiiip",
    "plow_mla_q_quant": "ppppiiiip",
    "plow_mla_kv_write": "ppppiipppppiiiifip",
    "plow_router_topk": "pppiiiiiiifp",
    "plow_moe_align": "piiippppiiip",
    "plow_moe_route": "pppipp" "iiiiiiii" "f" "iii" "pppp" "ii" "ppp" "p",
    "plow_moe_gather": "ppippipp" "iiip",
    "plow_moe_combine": "pppppiiipp",
    "plow_argmax": "ppiip",
    "plow_argmax_key": "ppiiip",
    "plow_argmax_fin": "ppiip",
    "plow_row_gather": "pppiip",
    "plow_head_to_token": "ppiiip",
    "plow_eltwise2": "pppl" "ip",
    "plow_mla_decode": "ppppplpipp" "iiipppppfipipp",
    "plow_mla_build_items": "piiipppp",
    "plow_mla_absorb": "pipppppiiipp",
    "plow_mla_fold": "pppppppiiiiipp",
    "plow_ep_counts": "ppipp",
    "plow_ep_push": "ppiippippppiip",
    "plow_ep_y_ready": "pp",
    "plow_ep_combine": "pppppiipip",
    "plow_wait_probe": "piLpp",
    "plow_ag_push": "pLLppiipiii" "Lipp",
    "plow_ag_release": "pLiip",
    "plow_tp_allreduce_norm": "pLLLp" "iii" "pipppp" "iifiipp",
    "plow_interp_run": "ppppppppppp" "IIIIp",
    "plow_sample": "ppiiipppppp" "Lp",
    "plow_dsa_k_write": "pppipppppp" "iiiifp",
    "plow_dsa_select": "ppippp" "ipipplp" "pppiiiiiipp",
    "plow_dsa_gather": "pppppi" "pppppi" "iip",
    "plow_gdn": "ppppipi" "ppppp" "iiiiip",
    "plow_gated_norm": "pppiipiiifp",
    "plow_sigmoid_gate": "ppplp",
    "plow_gqa_attention": "ppplpipp" "iiiiiii" "pi" "ppppp" "fppp",
    "plow_rope_kv": "ppi" "pppppppp" "i" "iiiiiii" "fppp",
    "plow_mla_prefill_attention": "ppplpipp" "iiii" "pi" "ppppp" "fpp",
    "plow_mla_latent_gather": "ppipppppp" "ipiiiip",
    "plow_mla_q_rope": "pippiiiiip",
}
_CT = {"p": C.c_void_p, "i": C.c_int32, "l": C.c_int64, "f": C.c_float, "L": C.c_uint64, "I": C.c_uint32}


def _arg(v):
    if v is None:
        return None
    if hasattr(v, "data_ptr"):
        return v.data_ptr()
    return v


LAUNCHES = {"n": 0}                       # kernels launched through this module (bench bookkeeping)
PROFILE: list | None = None               # when a list: (label, start event, end event) per launcher call (diagnostic)


def profiled(label: str, fn):
    """Run ``fn()`` between two CUDA events recorded on the current stream and log them under ``label``."""
    import torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    r = fn()
    b.record()
    PROFILE.append((label, a, b))
    return r


def profile_summary() -> list:
    """[(label, calls, total ms)] of the calls logged since PROFILE was set, longest first; clears the log."""
    import torch
    torch.cuda.synchronize()
    agg: dict = {}
    for label, a, b in PROFILE:
        e = agg.setdefault(label, [0, 0.0])
        e[0] += 1
        e[1] += a.elapsed_time(b)
    PROFILE.clear()
    return sorted(((k, c, t) for k, (c, t) in agg.items()), key=lambda x: -x[2])
_KERNELS_PER_CALL = {"plow_gqa_attention": 2, "plow_dsa_select": 3, "plow_mla_prefill_attention": 3}


def call(name: str, *args) -> None:
    """Invoke a kernel launcher of libplow_cuda.so on the current stream (appended as last arg)."""
    lib = cuda_lib()
    LAUNCHES["n"] += _KERNELS_PER_CALL.get(name, 1)
    fn = getattr(lib, name)
    if fn.argtypes is None:
        fn.argtypes = [_CT[c] for c in _SIGS[name]]
        fn.restype = C.c_int
    if PROFILE is not None:
        rc = profiled(name, lambda: fn(*[_arg(a) for a in args], stream_ptr()))
    else:
        rc = fn(*[_arg(a) for a in args], stream_ptr())
    if rc != 0:
        raise NativeLibraryError(f"{name} failed with code {rc}")
