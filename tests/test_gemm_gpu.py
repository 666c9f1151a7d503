"""tcgen05 GEMM family vs a plain fp32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _relerr(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _mk(m, n, k, dual=False, experts=1, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(m, k, device="cuda", generator=g)
    w = torch.randn(experts * n * (2 if dual else 1), k, device="cuda", generator=g) * 0.05
    return x, w


def _ref(x, w, n, dual):
    if dual:
        g = x @ w[:n].t()
        u = x @ w[n:2 * n].t()
        return torch.nn.functional.silu(g) * u
    return x @ w.t()


@pytest.mark.parametrize("m,n,k,swap,bn", [
    (300, 512, 320, False, 128), (1000, 2048, 328, False, 256), (129, 640, 64, False, 128),
    (5, 512, 320, True, 32), (17, 384, 1024, True, 32), (64, 256, 512, True, 64),
    (100, 1000, 256, True, 128), (200, 512, 256, True, 64),
])
def test_bf16(m, n, k, swap, bn):
    from plow_b200.ops import gemm, native
    x, w = _mk(m, n, k)
    xb, wb = x.bfloat16(), w.bfloat16()
    y = gemm.gemm(xb, wb, swap=swap, bn=bn)
    native.check_status()
    ref = xb.float() @ wb.float().t()
    assert _relerr(y, ref) < 1e-2
    yf = gemm.gemm(xb, wb, swap=swap, bn=bn, out_f32=True)
    assert _relerr(yf, ref) < 1e-4


@pytest.mark.parametrize("m,n,k,swap,bn", [
    (300, 512, 320, False, 128), (7, 256, 512, True, 32), (100, 384, 256, True, 128),
])
def test_bf16_dual_residual(m, n, k, swap, bn):
    from plow_b200.ops import gemm, native
    x, w = _mk(m, n, k, dual=True)
    xb, wb = x.bfloat16(), w.bfloat16()
    y = gemm.gemm(xb, wb, dual=True, swap=swap, bn=bn)
    native.check_status()
    ref = _ref(xb.float(), wb.float(), n, True)
    assert _relerr(y, ref) < 1e-2
    res = torch.randn(m, n, device="cuda").bfloat16()
    x2, w2 = _mk(m, n, k, seed=3)
    y2 = gemm.gemm(x2.bfloat16(), w2.bfloat16(), residual=res, swap=swap, bn=bn)
    native.check_status()
    assert _relerr(y2, x2.bfloat16().float() @ w2.bfloat16().float().t() + res.float()) < 1e-2


@pytest.mark.parametrize("m,n,k,swap,bn,dual", [
    (300, 512, 512, False, 128, False), (260, 256, 1024, False, 64, True), (300, 512, 512, False, 256, False),
    (9, 512, 512, True, 32, False), (60, 256, 7168, True, 64, False), (128, 384, 256, True, 128, False),
    (20, 256, 512, True, 32, True), (50, 512, 2048, True, 64, True),
])
def test_fp8_block_scaled(m, n, k, swap, bn, dual):
    from plow_b200.ops import gemm, native, quant
    x, w = _mk(m, n, k, dual=dual)
    xq, sx = quant.quant_act_1x128(x)
    wq, sw = quant.quant_weight_128x128(w)
    y = gemm.gemm(xq, wq, sx=sx, sw=sw, dual=dual, swap=swap, bn=bn)
    native.check_status()
    ref = _ref(quant.dequant_act_1x128(xq, sx), quant.dequant_weight_128x128(wq, sw), n, dual)
    assert _relerr(y, ref) < 1e-2


@pytest.mark.parametrize("swap,bn,fp8", [(True, 32, False), (True, 32, True), (False, 128, False), (False, 128, True)])
def test_grouped(swap, bn, fp8):
    from plow_b200.ops import gemm, native, quant
    E, n, k = 6, 256, 512
    counts = torch.tensor([5, 0, 40, 1, 33, 17]) if swap else torch.tensor([130, 0, 300, 1, 128, 77])
    off = torch.zeros(E + 1, dtype=torch.int32)
    off[1:] = counts.cumsum(0)
    m = int(off[-1])
    tiles = (counts + 127) // 128
    tp = torch.zeros(E + 1, dtype=torch.int32)
    tp[1:] = tiles.cumsum(0)
    x, w = _mk(m, n, k, experts=E)
    if fp8:
        xq, sx = quant.quant_act_1x128(x)
        wq, sw = quant.quant_weight_128x128(w)
        xr, wr = quant.dequant_act_1x128(xq, sx), quant.dequant_weight_128x128(wq, sw)
    else:
        xq, wq, sx, sw = x.bfloat16(), w.bfloat16(), None, None
        xr, wr = xq.float(), wq.float()
    y = gemm.gemm(xq, wq, sx=sx, sw=sw, n_experts=E, grp_off=off.cuda(), tile_prefix=tp.cuda(),
                  swap=swap, bn=bn)
    native.check_status()
    ref = torch.empty(m, n, device="cuda")
    for e in range(E):
        ref[off[e]:off[e + 1]] = xr[off[e]:off[e + 1]] @ wr[e * n:(e + 1) * n].t()
    assert _relerr(y, ref) < 1e-2


@pytest.mark.parametrize("m,swap,bn,fp8", [(40, True, 64, True), (200, False, 128, False), (33, True, 64, False)])
def test_quant_epilogue(m, swap, bn, fp8):
    from plow_b200.ops import gemm, native, quant
    n, k = 256, 512
    dual = swap  # SwiGLU + requant is the decode MoE path
    x, w = _mk(m, n, k, dual=dual)
    if fp8:
        xq, sx = quant.quant_act_1x128(x)
        wq, sw = quant.quant_weight_128x128(w)
        xr, wr = quant.dequant_act_1x128(xq, sx), quant.dequant_weight_128x128(wq, sw)
    else:
        xq, wq, sx, sw = x.bfloat16(), w.bfloat16(), None, None
        xr, wr = xq.float(), wq.float()
    yq, syq = gemm.gemm(xq, wq, sx=sx, sw=sw, dual=dual, swap=swap, bn=bn, quant_out=True)
    native.check_status()
    ref = _ref(xr, wr, n, dual)
    got = quant.dequant_act_1x128(yq, syq)
    assert _relerr(got, ref) < 6e-2   # e4m3 has 3 mantissa bits
    sref = ref.view(m, n // 128, 128).abs().amax(2).clamp_min(1e-10) / 448.0
    assert _relerr(syq[:, :m].t(), sref) < 2e-2


@pytest.mark.parametrize("dual,bn,grouped", [(True, 128, False), (False, 256, False), (True, 128, True), (False, 256, True),
                                             (True, 64, True)])
def test_large_m_fp8_tiles_quant_epilogue(dual, bn, grouped, monkeypatch):
    """Token-major (non-swap) block-scaled tiles with eight epilogue warps: 256 accumulator columns per partial (gate | up
    of 128, or 256 plain) and the 64 + 64 form, with the e4m3 + 1x128-scale output, dense and grouped (an empty expert,
    ragged last tiles)."""
    from plow_b200.ops import gemm, native, quant
    if bn == 64:
        monkeypatch.setattr(gemm, "_WIDE_DEFAULT", False)
    E, n, k = (5, 512, 1024) if grouped else (0, 512, 1024)
    counts = torch.tensor([130, 0, 300, 1, 257]) if grouped else torch.tensor([333])
    off = torch.zeros(len(counts) + 1, dtype=torch.int32)
    off[1:] = counts.cumsum(0)
    m = int(off[-1])
    tp = torch.zeros(len(counts) + 1, dtype=torch.int32)
    tp[1:] = ((counts + 127) // 128).cumsum(0)
    x, w = _mk(m, n, k, dual=dual, experts=max(E, 1))
    xq, sx = quant.quant_act_1x128(x)
    wq, sw = quant.quant_weight_128x128(w)
    xr, wr = quant.dequant_act_1x128(xq, sx), quant.dequant_weight_128x128(wq, sw)
    kw = dict(n_experts=E, grp_off=off.cuda(), tile_prefix=tp.cuda()) if grouped else {}
    y = gemm.gemm(xq, wq, sx=sx, sw=sw, dual=dual, n_out=n, swap=False, bn=bn, **kw)
    if bn >= 128:      # the quantising epilogue needs a token's whole 1x128 group inside one tile
        yq, syq = gemm.gemm(xq, wq, sx=sx, sw=sw, dual=dual, n_out=n, swap=False, bn=bn, quant_out=True, **kw)
    native.check_status()
    per = n * (2 if dual else 1)
    ref = torch.empty(m, n, device="cuda")
    for e in range(len(counts)):
        ref[off[e]:off[e + 1]] = _ref(xr[off[e]:off[e + 1]], wr[e * per:(e + 1) * per], n, dual)
    assert _relerr(y, ref) < 1e-2
    if bn < 128:
        return
    got = quant.dequant_act_1x128(yq, syq)
    assert _relerr(got, ref) < 6e-2
    sref = ref.view(m, n // 128, 128).abs().amax(2).clamp_min(1e-10) / 448.0
    assert _relerr(syq[:, :m].t(), sref) < 2e-2


@pytest.mark.parametrize("m,n,k,fp8,dual,splits", [(64, 256, 7168, True, False, 7), (64, 512, 2048, True, True, 4),
                                                    (33, 384, 4096, False, False, 5), (64, 128, 7168, False, False, 28),
                                                    (20, 256, 1024, False, True, 3)])
def test_split_k(m, n, k, fp8, dual, splits):
    from plow_b200.ops import gemm, native, quant
    x, w = _mk(m, n, k, dual=dual)
    if fp8:
        xq, sx = quant.quant_act_1x128(x)
        wq, sw = quant.quant_weight_128x128(w)
        xr, wr = quant.dequant_act_1x128(xq, sx), quant.dequant_weight_128x128(wq, sw)
    else:
        xq, wq, sx, sw = x.bfloat16(), w.bfloat16(), None, None
        xr, wr = xq.float(), wq.float()
    ref = _ref(xr, wr, n, dual)
    for _ in range(2):      # twice: the tile counters must have reset themselves
        y = gemm.gemm(xq, wq, sx=sx, sw=sw, dual=dual, swap=True, bn=64, splits=splits, out_f32=True)
        native.check_status()
        assert _relerr(y, ref) < 2e-3
    if fp8 or not dual:
        yq, syq = gemm.gemm(xq, wq, sx=sx, sw=sw, dual=dual, swap=True, bn=64, splits=splits, quant_out=True)
        assert _relerr(quant.dequant_act_1x128(yq, syq), ref) < 6e-2
