"""GQA flash attention + fused RoPE/cache-write kernels against plain PyTorch fp32 (GPU)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _err(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())


@pytest.mark.parametrize("nq,nkv,hd", [(32, 8, 128), (8, 8, 128), (16, 2, 256)])
def test_decode(nq, nkv, hd):
    from plow_b200.ops import gqa, native
    torch.manual_seed(0)
    n_seq = 5
    lens = [1, 63, 64, 200, 777]
    pages_per = 13
    n_pages = n_seq * pages_per + 1
    kc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16()
    vc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16()
    perm = torch.randperm(n_pages - 1, device="cuda").int() + 1
    pt = perm[: n_seq * pages_per].view(n_seq, pages_per).contiguous()
    seq = torch.arange(n_seq, dtype=torch.int32, device="cuda")
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    q = torch.randn(n_seq, nq, hd, device="cuda").bfloat16()
    ref = gqa.reference(q, kc, vc, pt, seq, pos)
    for splits in (1, 4):
        ws = gqa.AttnWorkspace(n_seq, nq, nkv, hd, 13 * 64, q.device, tiles_per_split=2, max_splits=splits)
        out = gqa.attention(q, kc, vc, pt, seq, pos, ws)
        torch.cuda.synchronize()
        native.check_status()
        assert _err(out, ref) < 2e-2, (splits, _err(out, ref))


@pytest.mark.parametrize("window", [0, 100])
def test_prefill_causal_mixed_batch(window):
    from plow_b200.ops import gqa, native
    torch.manual_seed(1)
    nq, nkv, hd = 32, 8, 128
    # three sequences: a fresh 150-token prompt, a 70-token chunk appended at position 90, one decode row; one idle row
    pages_per = 6
    n_pages = 4 * pages_per + 1
    kc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16()
    vc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16()
    pt = (torch.arange(4 * pages_per, dtype=torch.int32, device="cuda").view(4, pages_per) + 1).contiguous()
    seq = torch.tensor([0] * 150 + [2] * 70 + [1] + [3], dtype=torch.int32, device="cuda")
    pos = torch.tensor(list(range(150)) + list(range(90, 160)) + [300] + [-1], dtype=torch.int32, device="cuda")
    rows = seq.numel()
    q = torch.randn(rows, nq, hd, device="cuda").bfloat16()
    ref = gqa.reference(q, kc, vc, pt, seq, pos, window=window)
    for splits in (1, 3):
        ws = gqa.AttnWorkspace(rows, nq, nkv, hd, pages_per * 64, q.device, tiles_per_split=1, max_splits=splits)
        out = torch.zeros(rows, nq * hd, dtype=torch.bfloat16, device="cuda")
        gqa.attention(q, kc, vc, pt, seq, pos, ws, window=window, out=out)
        torch.cuda.synchronize()
        native.check_status()
        assert _err(out, ref) < 2e-2, (splits, _err(out, ref))


@pytest.mark.parametrize("pair_mode,rot,norm", [(0, 128, False), (1, 64, True)])
def test_rope_kv(pair_mode, rot, norm):
    from plow_b200.ops import gqa
    torch.manual_seed(2)
    nq, nkv, hd, rows = 8, 2, 128, 37
    qkv = torch.randn(rows, (nq + 2 * nkv) * hd, device="cuda").bfloat16()
    tab = torch.randn(512, rot, device="cuda")
    pos = torch.randint(0, 300, (rows,), dtype=torch.int32, device="cuda")
    seq = torch.arange(rows, dtype=torch.int32, device="cuda")
    pt = (torch.arange(rows * 5, dtype=torch.int32, device="cuda").view(rows, 5)).contiguous()
    kc = torch.zeros(rows * 5, 64, nkv, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qn = torch.randn(hd, device="cuda").bfloat16() if norm else None
    kn = torch.randn(hd, device="cuda").bfloat16() if norm else None
    q_out = gqa.rope_kv(qkv, kc, vc, tab, pos, seq, pt, nq, nkv, hd, rot=rot, pair_mode=pair_mode, qn=qn, kn=kn, eps=1e-6)
    torch.cuda.synchronize()

    def ref_head(x, g, p):
        x = x.float()
        if g is not None:
            x = (x * torch.rsqrt((x * x).mean() + 1e-6) * g.float()).bfloat16().float()
        half = rot // 2
        c, s = tab[p, :half], tab[p, half:]
        y = x.clone()
        if pair_mode == 0:
            a, b = x[:half], x[half:rot]
            y[:half] = a * c - b * s
            y[half:rot] = b * c + a * s
        else:
            a, b = x[0:rot:2], x[1:rot:2]
            y[0:rot:2] = a * c - b * s
            y[1:rot:2] = b * c + a * s
        return y
    v = qkv.view(rows, nq + 2 * nkv, hd)
    for r in (0, 5, rows - 1):
        p = int(pos[r])
        cell_k = kc[int(pt[r, p // 64]), p % 64]
        cell_v = vc[int(pt[r, p // 64]), p % 64]
        for h in (0, nq - 1):
            assert _err(q_out[r, h], ref_head(v[r, h], qn, p)) < 1e-2
        for h in range(nkv):
            assert _err(cell_k[h], ref_head(v[r, nq + h], kn, p)) < 1e-2
            assert torch.equal(cell_v[h], v[r, nq + nkv + h])


def test_rope_kv_gated_heads():
    """Gated attention: query heads arrive as [Q | gate] pairs; Q is roped into q_out, the gates are copied out, K/V follow."""
    from plow_b200.ops import gqa
    torch.manual_seed(4)
    nq, nkv, hd, rows, rot = 4, 1, 256, 9, 64
    qkv = torch.randn(rows, nq * 2 * hd + 2 * nkv * hd, device="cuda").bfloat16()
    tab = torch.randn(64, rot, device="cuda")
    pos = torch.arange(rows, dtype=torch.int32, device="cuda")
    seq = torch.zeros(rows, dtype=torch.int32, device="cuda")
    pt = torch.tensor([[3, 4]], dtype=torch.int32, device="cuda")
    kc = torch.zeros(6, 64, nkv, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    gate = torch.zeros(rows, nq * hd, dtype=torch.bfloat16, device="cuda")
    q_out = gqa.rope_kv(qkv, kc, vc, tab, pos, seq, pt, nq, nkv, hd, rot=rot, pair_mode=0, gate_out=gate)
    torch.cuda.synchronize()
    qh = qkv[:, :nq * 2 * hd].view(rows, nq, 2 * hd)
    assert torch.equal(gate.view(rows, nq, hd), qh[..., hd:])
    half = rot // 2
    x = qh[..., :hd].float()
    c, s = tab[pos.long(), :half][:, None, :], tab[pos.long(), half:][:, None, :]
    want = x.clone()
    want[..., :half] = x[..., :half] * c - x[..., half:rot] * s
    want[..., half:rot] = x[..., half:rot] * c + x[..., :half] * s
    assert _err(q_out, want) < 1e-2
    assert torch.equal(vc[3, :rows, 0], qkv[:, nq * 2 * hd + hd:])


def _kv8(kc, vc):
    """e4m3 twins of bf16 caches + the packed [n_pages, 64, 2*nkv] scale tensor the kernels read."""
    from plow_b200.ops import gqa
    k8, ks = gqa.quant_cache(kc)
    v8, vs = gqa.quant_cache(vc)
    return k8, v8, torch.cat([ks, vs], dim=-1).contiguous(), gqa.dequant_cache(k8, ks), gqa.dequant_cache(v8, vs)


@pytest.mark.parametrize("nq,nkv", [(32, 8), (8, 8), (16, 1)])
def test_decode_e4m3_cache(nq, nkv):
    """The e4m3-cache instantiation (raw byte tiles by TMA, converter warps, same MMAs) against the fp32 statement over
    the dequantised cache: the only difference left is the bf16 kernel's own error."""
    from plow_b200.ops import gqa, native
    torch.manual_seed(3)
    hd, n_seq, pages_per = 128, 5, 13
    lens = [1, 63, 64, 200, 777]
    n_pages = n_seq * pages_per + 1
    kc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16() * 3.0
    vc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16() * 0.5
    k8, v8, sc, kd, vd = _kv8(kc, vc)
    perm = torch.randperm(n_pages - 1, device="cuda").int() + 1
    pt = perm[: n_seq * pages_per].view(n_seq, pages_per).contiguous()
    seq = torch.arange(n_seq, dtype=torch.int32, device="cuda")
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    q = (torch.randn(n_seq, nq, hd, device="cuda") * 0.3).bfloat16()
    ref = gqa.reference(q, kd, vd, pt, seq, pos)
    for splits in (1, 4):
        ws = gqa.AttnWorkspace(n_seq, nq, nkv, hd, 13 * 64, q.device, tiles_per_split=2, max_splits=splits)
        out = gqa.attention(q, k8, v8, pt, seq, pos, ws, kv_scale=sc)
        torch.cuda.synchronize()
        native.check_status()
        assert _err(out, ref) < 2e-2, (splits, _err(out, ref))
        assert _err(out, gqa.reference(q, kc, vc, pt, seq, pos)) < 8e-2        # and close to the unquantised cache


def test_prefill_e4m3_cache_mixed_batch():
    from plow_b200.ops import gqa, native
    torch.manual_seed(4)
    nq, nkv, hd, pages_per = 32, 8, 128, 6
    n_pages = 4 * pages_per + 1
    kc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16()
    vc = torch.randn(n_pages, 64, nkv, hd, device="cuda").bfloat16()
    k8, v8, sc, kd, vd = _kv8(kc, vc)
    pt = (torch.arange(4 * pages_per, dtype=torch.int32, device="cuda").view(4, pages_per) + 1).contiguous()
    seq = torch.tensor([0] * 150 + [2] * 70 + [1] + [3], dtype=torch.int32, device="cuda")
    pos = torch.tensor(list(range(150)) + list(range(90, 160)) + [300] + [-1], dtype=torch.int32, device="cuda")
    rows = seq.numel()
    q = (torch.randn(rows, nq, hd, device="cuda") * 0.3).bfloat16()
    for window in (0, 100):
        ref = gqa.reference(q, kd, vd, pt, seq, pos, window=window)
        for splits in (1, 3):
            ws = gqa.AttnWorkspace(rows, nq, nkv, hd, pages_per * 64, q.device, tiles_per_split=1, max_splits=splits)
            out = torch.zeros(rows, nq * hd, dtype=torch.bfloat16, device="cuda")
            gqa.attention(q, k8, v8, pt, seq, pos, ws, window=window, out=out, kv_scale=sc)
            torch.cuda.synchronize()
            native.check_status()
            assert _err(out, ref) < 2e-2, (window, splits, _err(out, ref))


def test_rope_kv_writes_e4m3_cells():
    """The fused writer with a scale tensor: every cell is the bf16 writer's row quantised with amax / 448."""
    from plow_b200.ops import gqa
    torch.manual_seed(5)
    nq, nkv, hd, rows, rot = 8, 2, 128, 37, 128
    qkv = torch.randn(rows, (nq + 2 * nkv) * hd, device="cuda").bfloat16()
    tab = torch.randn(512, rot, device="cuda")
    pos = torch.randint(0, 300, (rows,), dtype=torch.int32, device="cuda")
    seq = torch.arange(rows, dtype=torch.int32, device="cuda")
    pt = (torch.arange(rows * 5, dtype=torch.int32, device="cuda").view(rows, 5)).contiguous()
    kn = torch.randn(hd, device="cuda").bfloat16()
    qn = torch.randn(hd, device="cuda").bfloat16()
    kc = torch.zeros(rows * 5, 64, nkv, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q_ref = gqa.rope_kv(qkv, kc, vc, tab, pos, seq, pt, nq, nkv, hd, rot=rot, qn=qn, kn=kn)
    k8 = torch.zeros(rows * 5, 64, nkv, hd, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    v8 = torch.zeros(rows * 5, 64, nkv, hd, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    sc = torch.zeros(rows * 5, 64, 2 * nkv, device="cuda")
    q_out = gqa.rope_kv(qkv, k8, v8, tab, pos, seq, pt, nq, nkv, hd, rot=rot, qn=qn, kn=kn, kv_scale=sc)
    torch.cuda.synchronize()
    assert torch.equal(q_out, q_ref)
    for c16, c8, ofs in ((kc, k8, 0), (vc, v8, nkv)):
        want8, want_sc = gqa.quant_cache(c16)
        written = c16.float().abs().amax(dim=-1) > 0
        assert written.sum().item() == rows * nkv
        got_sc = sc[..., ofs:ofs + nkv]
        assert torch.allclose(got_sc[written], want_sc[written], rtol=1e-6, atol=0)
        assert (got_sc[~written] == 0).all()
        deq = c8.float() * got_sc[..., None]
        assert _err(deq[written], c16.float()[written]) < 0.07            # e4m3: 3 mantissa bits, error <= 2^-4 of amax
        # same bytes as the PyTorch quantiser, up to a rounding tie on a few cells
        same = (c8.view(torch.uint8)[written] == want8.view(torch.uint8)[written]).float().mean().item()
        assert same > 0.995, same
