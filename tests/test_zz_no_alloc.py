"""The allocation-free split-K GEMM entry point (csrc/cuda/gemm_noalloc.h), called through its exported
C symbol exactly as an external caller would, against the library's regular GEMM entry point.

Some callers of this library cannot allocate device memory when they need a GEMM (all HBM already
promised to weights and KV pages, or a decode thread that must not hit cudaMalloc's implicit device
synchronisation); for them the split-K scratch lives in a fixed device array inside the library.
This file is named so that pytest collects it last: a run that stops at the first failure has then
already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from plow_b200.ops import native
    lib = native.cuda_lib()
    fn = lib.plow_gemm_splitk_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.plow_gemm_noalloc_strerror.restype = C.c_char_p
    lib.plow_gemm_noalloc_strerror.argtypes = [C.c_int]
    return lib, fn


def _relerr(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("m,n,k,splits", [(64, 2176, 7168, 8), (17, 256, 4096, 16)])
def test_noalloc_matches_regular_entry_point_twice(m, n, k, splits):
    from plow_b200.ops import gemm, native
    lib, fn = _entry()
    g = torch.Generator(device="cuda").manual_seed(m)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                       # two calls in a row share the static scratch
        x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
        w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
        y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        rc = fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, splits, status.data_ptr(), stream)
        assert rc == 0, lib.plow_gemm_noalloc_strerror(rc)
        want = gemm.gemm(x, w, swap=True, bn=32 if m <= 32 else 64, splits=splits)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        native.check_status()
        assert _relerr(y, want) < 1e-2
        assert _relerr(y, x.float() @ w.float().t()) < 1e-2


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib, fn = _entry()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.zeros(128, 1024, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128 * 200, 1024, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(128, 128 * 200, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), 128, 128 * 200, 1024, 1, status.data_ptr(), s)   # 200 tiles
    assert rc == -2 and b"too large" in lib.plow_gemm_noalloc_strerror(rc)
    assert fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), 129, 256, 1024, 1, status.data_ptr(), s) == -1
    assert fn(None, w.data_ptr(), y.data_ptr(), 64, 256, 1024, 1, status.data_ptr(), s) == -1
    assert fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), 64, 256, 1020, 1, status.data_ptr(), s) == -1
