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
    # fold: requests with 1, 2, 3 and 13 splits (the kernel merges up to 16)
    lens = [100, 40 * 64, 70 * 64 + 5, 400 * 64 + 9]
    T2 = len(lens)
    ws = mla.DecodeWorkspace(T2, 32768, tiles_per_split=32)
    assert ws.max_splits == 16
    ws.opart.copy_(torch.randn_like(ws.opart.float()).bfloat16())
    ws.lse.copy_(torch.randn_like(ws.lse) * 3)
    kvlen = torch.tensor(lens, dtype=torch.int32, device="cuda")
    wuv = (torch.randn(H * 128, 512, device="cuda") * 0.1).bfloat16()
    ao = torch.empty(T2, H * 128, dtype=torch.bfloat16, device="cuda")
    aq, saq = mla.fold(ws, kvlen, wuv, T2, H, ao, want_fp8=True)
    native.check_status()
    for t, n in enumerate(lens):
        tiles = (n + 63) // 64
        ns = min(ws.max_splits, -(-tiles // 32))
        ns = -(-tiles // (-(-tiles // ns)))          # tiles are dealt evenly: the last split may vanish
        w = torch.softmax(ws.lse[t, :ns].float() * 0.6931471805599453, 0)          # 2^lse weights
        merged = (w[:, :, None] * ws.opart[t, :ns].float()).sum(0).bfloat16().float()   # [heads, 512]
        ref = torch.einsum("hc,hvc->hv", merged, wuv.view(H, 128, 512).float()).reshape(-1)
        assert _rel(ao[t], ref) < 1e-2
        assert _rel(aq[t].float().view(H, 128) * saq[:, t, None], ref.view(H, 128)) < 4e-2


@pytest.mark.parametrize("fp8_weight", [True, False])
def test_materialised_prefill_vs_reference(fp8_weight):
    """Gather the cached latent, rebuild K / V through kv_b_proj, rotate the queries, attend causally: against the
    same computation in fp32 PyTorch.  Two requests (one with a cached prefix, lengths off the 64-token grid) plus
    rows that are masked out (position -1) and must keep their previous output."""
    from plow_b200.ops import gemm as gemm_ops, mla, native, quant
    from plow_b200.utils.rope import rope_table
    H = 128
    lens = [300, 200]                   # cached tokens per request after this step's rows were written
    new = [130, 200]                    # the last `new` tokens of each are this step's rows
    n_slots, max_pages = 3, 8
    kv8, ksc, pt = _build_cache(lens, 12, max_pages, seed=3)
    pt_full = torch.zeros(n_slots, max_pages, dtype=torch.int32, device="cuda")
    pt_full[1], pt_full[2] = pt[0], pt[1]               # requests live in slots 1 and 2
    slots = [1, 2]
    g = torch.Generator(device="cuda").manual_seed(4)
    w = torch.randn(H * 256, 512, device="cuda", generator=g) * 0.05
    if fp8_weight:
        wq, sw = quant.quant_weight_128x128(w)
        w_ref = quant.dequant_weight_128x128(wq, sw).float()
    else:
        wq, sw = w.bfloat16(), None
        w_ref = wq.float()
    pad = 5                              # masked rows between and after the runs
    T = sum(new) + 2 * pad
    q = (torch.randn(T, H * 192, device="cuda", generator=g) * 0.5).bfloat16()
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    pos = torch.full((T,), -1, dtype=torch.int32, device="cuda")
    r = 0
    runs = []
    for s, L, n in zip(slots, lens, new):
        seq[r:r + n] = s
        pos[r:r + n] = torch.arange(L - n, L, dtype=torch.int32, device="cuda")
        runs.append((r, n, s, L))
        r += n + pad
    tab = torch.from_numpy(rope_table(4096, 64, 10000.0)).cuda()
    spans, base = [], 0
    for s, L in zip(slots, lens):
        spans.append([s, L, base, 0])
        base += -(-L // 64) * 64
    spans_d = torch.tensor(spans, dtype=torch.int32, device="cuda")
    ws = mla.PrefillWorkspace(1024, T, n_slots, max_pages, fp8_weight=fp8_weight)
    mla.latent_gather(ws, kv8, ksc, pt_full, spans_d, len(spans), max(-(-L // 64) for L in lens))
    if fp8_weight:
        gemm_ops.gemm(ws.lat8[:base, :512], wq, sx=ws.lat_scale, sw=sw, out=ws.kvb[:base], swap=False)
    else:
        gemm_ops.gemm(ws.lat16[:base], wq, out=ws.kvb[:base], swap=False)
    q_in = q.clone()
    mla.q_rope(q, tab, pos, H, 128, 64, 1)
    out = torch.full((T, H * 128), 7.0, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(192)
    mla.prefill_attention(q, ws, base, seq, pos, scale, out)
    torch.cuda.synchronize()
    native.check_status()
    kvd = kv8.float() * ksc[..., None]                        # [pages, 64, 576]
    worst = 0.0
    for (r0, n, s, L), sp in zip(runs, spans):
        pages = pt_full[s, :(L + 63) // 64].long()
        lat = kvd[pages].reshape(-1, 576)[:L]
        kvb = (lat[:, :512] @ w_ref.t()).view(L, H, 256)
        # what the kernel consumed: its own bf16 K / V
        got_kvb = ws.kvb[sp[2]:sp[2] + L].view(L, H, 256).float()
        assert _rel(got_kvb, kvb) < (3e-2 if fp8_weight else 1e-2)
        k = torch.cat([kvb[..., :128], lat[:, None, 512:].expand(L, H, 64)], -1)      # [L, H, 192]
        v = kvb[..., 128:]
        q3 = q_in[r0:r0 + n].view(n, H, 192).float()
        qr = _rope_ref(q3[..., 128:].permute(1, 0, 2), tab, pos[r0:r0 + n]).permute(1, 0, 2)
        qq = torch.cat([q3[..., :128], qr], -1)
        sc = torch.einsum("nhd,lhd->hnl", qq, k) * scale
        mask = torch.arange(L, device="cuda")[None, :] <= pos[r0:r0 + n, None].long()
        sc = sc.masked_fill(~mask[None], float("-inf"))
        ref = torch.einsum("hnl,lhd->nhd", sc.softmax(-1), v).reshape(n, H * 128)
        worst = max(worst, _rel(out[r0:r0 + n], ref))
    assert worst < 2e-2, worst
    masked = pos < 0
    assert torch.all(out[masked].float() == 7.0)
    assert torch.equal(q[masked], q_in[masked])
