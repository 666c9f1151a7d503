"""MLA kernels: query prep / quant, latent-cache write, absorbed tcgen05 decode vs fp32 PyTorch."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _rope_ref(x, tab, pos, interleaved=True):
    half = tab.shape[1] // 2
    c, s = tab[pos.long(), :half], tab[pos.long(), half:]
    if interleaved:
        a, b = x[..., 0::2].float(), x[..., 1::2].float()
        return torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def test_q_prep_and_quant():
    from plow_b200.ops import mla
    from plow_b200.utils.rope import rope_table
    T, H = 7, 128
    q = torch.randn(T, H * 192, device="cuda").bfloat16()
    tab = torch.from_numpy(rope_table(4096, 64, 10000.0)).cuda()
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    qn, qr = mla.q_prep(q, tab, pos, H, 128, 64, 1)
    q3 = q.view(T, H, 192)
    assert torch.equal(qn, q3[..., :128].permute(1, 0, 2))
    ref = _rope_ref(q3[..., 128:].permute(1, 0, 2), tab, pos)
    assert _rel(qr, ref) < 5e-3
    q_abs = torch.randn(H, T, 512, device="cuda").bfloat16()
    q8, sq = mla.q_quant(q_abs, qr)
    full = torch.cat([q_abs, qr], -1).float()
    assert _rel(sq, full.abs().amax(-1) / 448) < 1e-6
    assert _rel(q8.float() * sq[..., None], full) < 4e-2


def _build_cache(lens, n_pages, max_pages, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kv = (torch.randn(n_pages, 64, 576, device="cuda", generator=g) * 1.5)
    amax = kv.abs().amax(-1)
    scale = (amax / 448).clamp_min(1e-10)
    kv8 = (kv / scale[..., None]).to(torch.float8_e4m3fn)
    perm = torch.randperm(n_pages, device="cuda", generator=g).int()
    pt = torch.zeros(len(lens), max_pages, dtype=torch.int32, device="cuda")
    used = 0
    for r, n in enumerate(lens):
        np_ = (n + 63) // 64
        pt[r, :np_] = perm[used:used + np_]
        used += np_
    return kv8, scale.contiguous(), pt


@pytest.mark.parametrize("lens,tps", [([64], 32), ([1, 65, 130], 32), ([300, 2048, 777, 5], 8), ([5000, 100], 16)])
def test_mla_decode_vs_reference(lens, tps):
    from plow_b200.ops import mla, native
    T = len(lens)
    max_ctx = max(lens)
    max_pages = (max_ctx + 63) // 64 + 1
    n_pages = sum((n + 63) // 64 for n in lens) + 3
    kv8, ksc, pt = _build_cache(lens, n_pages, max_pages)
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(128, T, 576, device="cuda", generator=g) * 0.3
    sq = q.abs().amax(-1) / 448
    q8 = (q / sq[..., None]).to(torch.float8_e4m3fn)
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    slot_of = torch.arange(T, dtype=torch.int32, device="cuda")
    smax = torch.zeros(kv8.shape[0], 4, device='cuda'); smax[:, 0] = ksc.amax(1)
    ws = mla.DecodeWorkspace(T, max_ctx + 64, tiles_per_split=tps)
    scale = 1.0 / math.sqrt(192)
    out = mla.decode(q8, sq, kv8, ksc, smax, pt, slot_of, kvlen, ws, scale)
    native.check_status()
    qd = q8.float() * sq[..., None]
    for r, n in enumerate(lens):
        pages = pt[r, :(n + 63) // 64].long()
        kv = (kv8[pages].float() * ksc[pages][..., None]).view(-1, 576)[:n]
        s = (qd[:, r] @ kv.t()) * scale
        p = torch.softmax(s, -1)
        ref = p @ kv[:, :512]
        assert _rel(out[:, r], ref) < 6e-2, (r, n)


def test_kv_write_roundtrip():
    from plow_b200.ops import mla
    from plow_b200.utils.rope import rope_table
    T = 6
    kva = torch.randn(T, 2112, device="cuda").bfloat16()          # fused [q_a | kv_a] row, kv part at 1536
    gamma = (torch.rand(512, device="cuda") + 0.5).bfloat16()
    tab = torch.from_numpy(rope_table(1024, 64, 10000.0)).cuda()
    pos = torch.tensor([0, 63, 64, 130, 5, 700], dtype=torch.int32, device="cuda")
    slot = torch.tensor([0, 0, 0, 1, 2, 1], dtype=torch.int32, device="cuda")
    pt = torch.arange(3 * 16, dtype=torch.int32, device="cuda").view(3, 16).flip(1).contiguous()
    kv8 = torch.zeros(48, 64, 576, device="cuda").to(torch.float8_e4m3fn)
    ksc = torch.zeros(48, 64, device="cuda")
    smax = torch.zeros(48, 4, device='cuda')
    mla.kv_write(kv8, ksc, smax, kva, 1536, gamma, tab, pos, slot, pt, 512, 64, 1e-6, 1)
    src = kva[:, 1536:].float()
    lat = src[:, :512] * torch.rsqrt(src[:, :512].pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
    rope = _rope_ref(src[:, 512:], tab, pos)
    ref = torch.cat([lat, rope], -1)
    for t in range(T):
        page = int(pt[int(slot[t]), int(pos[t]) // 64])
        got = kv8[page, int(pos[t]) % 64].float() * ksc[page, int(pos[t]) % 64]
        assert _rel(got, ref[t]) < 4e-2
        assert abs(float(ksc[page, int(pos[t]) % 64]) - float(ref[t].abs().max() / 448)) < 5e-3 * float(ref[t].abs().max() / 448) + 1e-8


def test_absorb_and_fold_fused_kernels():
    from plow_b200.ops import mla, native
    from plow_b200.utils.rope import rope_table
    torch.manual_seed(0)
    H, T = 128, 70
    q = torch.randn(T, H * 192, device="cuda").bfloat16()
    wuk_t = (torch.randn(H * 512, 128, device="cuda") * 0.1).bfloat16()
    tab = torch.from_numpy(rope_table(4096, 64, 10000.0)).cuda()
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    q8, sq = mla.absorb(q, wuk_t, tab, pos, H, 1)
    native.check_status()
    q3 = q.view(T, H, 192).float()
    qabs = torch.einsum("thd,hcd->htc", q3[..., :128], wuk_t.view(H, 512, 128).float())
    qrope = _rope_ref(q3[..., 128:].permute(1, 0, 2), tab, pos)
    full = torch.cat([qabs, qrope], -1)
    assert _rel(sq, full.abs().amax(-1) / 448) < 5e-3
    assert _rel(q8.float() * sq[..., None], full) < 4e-2
    # fold: 3 requests with 1, 2 and 3 splits
    lens = [100, 40 * 64, 70 * 64 + 5]
    T2 = len(lens)
    ws = mla.DecodeWorkspace(T2, 8192, tiles_per_split=32)
    ws.opart.copy_(torch.randn_like(ws.opart.float()).bfloat16())
    ws.lse.copy_(torch.randn_like(ws.lse) * 3)
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    wuv = (torch.randn(H * 128, 512, device="cuda") * 0.1).bfloat16()
    ao = torch.empty(T2, H * 128, dtype=torch.bfloat16, device="cuda")
    aq, saq = mla.fold(ws, kvlen, wuv, T2, H, ao, want_fp8=True)
    native.check_status()
    for t, n in enumerate(lens):
        ns = min(ws.max_splits, -(-((n + 63) // 64) // 32))
        w = torch.softmax(ws.lse[t, :ns].float() * 0.6931471805599453, 0)          # 2^lse weights
        merged = (w[:, :, None] * ws.opart[t, :ns].float()).sum(0).bfloat16().float()   # [heads, 512]
        ref = torch.einsum("hc,hvc->hv", merged, wuv.view(H, 128, 512).float()).reshape(-1)
        assert _rel(ao[t], ref) < 1e-2
        assert _rel(aq[t].float().view(H, 128) * saq[:, t, None], ref.view(H, 128)) < 4e-2
