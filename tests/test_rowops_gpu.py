"""Row-wise kernels vs plain fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _rms(x, g, eps, plus_one=False):
    y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)
    return y * ((1 + g.float()) if plus_one else g.float())


@pytest.mark.parametrize("R,W", [(5, 512), (64, 7168), (3, 1536), (17, 128)])
def test_rmsnorm_and_quant(R, W):
    from plow_b200.ops import quant, rowops
    x = torch.randn(R, W, device="cuda").bfloat16()
    g = (torch.randn(W, device="cuda") * 0.1 + 1).bfloat16()
    h, xq, sx = rowops.rmsnorm(x, g, 1e-6, want_fp8=True)
    ref = _rms(x, g, 1e-6)
    assert _rel(h, ref) < 5e-3
    assert _rel(quant.dequant_act_1x128(xq, sx), ref) < 4e-2
    sref = h.float().view(R, W // 128, 128).abs().amax(2).clamp_min(1e-10) / 448
    assert _rel(sx.t(), sref) < 1e-5


def test_rmsnorm_strided_plus_one():
    from plow_b200.ops import rowops
    x = torch.randn(9, 2112, device="cuda").bfloat16()
    g = (torch.randn(512, device="cuda") * 0.1).bfloat16()
    h, _, _ = rowops.rmsnorm(x, g, 1e-5, plus_one=True, width=512, col_ofs=1536)
    assert _rel(h, _rms(x[:, 1536:2048], g, 1e-5, True)) < 5e-3


def test_add_norm():
    from plow_b200.ops import quant, rowops
    x = torch.randn(33, 4096, device="cuda").bfloat16()
    d = torch.randn(33, 4096, device="cuda").bfloat16()
    g = torch.ones(4096, device="cuda").bfloat16()
    xo, h, xq, sx = rowops.add_norm(x, d, g, 1e-6, want_fp8=True)
    s = (x.float() + d.float()).bfloat16()
    assert torch.equal(xo, s)
    assert _rel(h, _rms(s, g, 1e-6)) < 5e-3
    assert _rel(quant.dequant_act_1x128(xq, sx), _rms(s, g, 1e-6)) < 4e-2


def test_quant_act_matches_torch():
    from plow_b200.ops import quant, rowops
    x = torch.randn(40, 2048, device="cuda").bfloat16()
    xq, sx = rowops.quant_act(x)
    rq, rs = quant.quant_act_1x128(x.float())
    assert _rel(sx, rs) < 1e-6
    assert _rel(quant.dequant_act_1x128(xq, sx), quant.dequant_act_1x128(rq, rs)) < 1e-2


def test_embed_argmax_gather():
    from plow_b200.ops import rowops
    tab = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (37,), device="cuda", dtype=torch.int32)
    assert torch.equal(rowops.embed(tab, ids), tab[ids.long()])
    lg = torch.randn(6, 129280, device="cuda")
    lg[2, 77] = lg[2, 5000] = 50.0     # tie: lowest index wins
    am = rowops.argmax(lg)
    assert am.tolist() == [int(v) for v in lg.argmax(-1).tolist()][:2] + [77] + lg[3:].argmax(-1).tolist()
    rows = torch.tensor([3, 0, 36], device="cuda", dtype=torch.int32)
    x = rowops.embed(tab, ids)
    assert torch.equal(rowops.row_gather(x, rows), x[rows.long()])


@pytest.mark.parametrize("E,k,ng,tg,sig", [(256, 8, 8, 4, True), (512, 10, 1, 1, False), (64, 6, 1, 1, True)])
def test_router_topk(E, k, ng, tg, sig):
    from plow_b200.models.config import FfnSpec
    from plow_b200.models.reference import ReferenceModel
    from plow_b200.ops import rowops
    T = 50
    logits = torch.randn(T, E, device="cuda")
    bias = torch.randn(E, device="cuda") * 0.1 if sig else None
    f = FfnSpec(kind="moe", n_experts=E, top_k=k, n_group=ng, topk_group=tg, score="sigmoid" if sig else "softmax",
                norm_topk=True, route_scale=2.5)
    idx, gate = ReferenceModel.route(None, logits, f, bias)
    table = rowops.router_topk(logits, bias, k, ng, tg, sig, True, 2.5)
    assert torch.equal(table[..., 0].long(), idx)
    assert _rel(rowops.table_gates(table), gate) < 1e-5


def test_moe_align_gather_combine():
    from plow_b200.ops import quant, rowops
    T, k, E, H = 64, 8, 32, 1024
    g = torch.Generator(device="cuda").manual_seed(0)
    eids = torch.stack([torch.randperm(48, device="cuda", generator=g)[:k] for _ in range(T)]).int()   # some experts are remote
    gates = torch.rand(T, k, device="cuda", generator=g)
    table = torch.stack([eids, gates.view(torch.int32)], -1).contiguous()
    grp_off, tile_prefix, row_of_pair, pair_of_row = rowops.moe_align(table, 8, E)
    local = (eids >= 8) & (eids < 8 + E)
    cnt = torch.bincount((eids[local] - 8).long(), minlength=E)
    assert grp_off.tolist() == [0] + cnt.cumsum(0).tolist()
    assert tile_prefix.tolist() == [0] + ((cnt + 127) // 128).cumsum(0).tolist()
    M = int(grp_off[-1])
    rop = row_of_pair.view(T, k)
    assert ((rop >= 0) == local).all()
    for e in range(E):
        rows = rop[eids == e + 8]
        assert ((rows >= grp_off[e]) & (rows < grp_off[e + 1])).all()
    assert sorted(pair_of_row[:M].tolist()) == sorted(torch.nonzero(local.view(-1)).view(-1).tolist())
    x = torch.randn(T, H, device="cuda").bfloat16()
    xq, sx = rowops.quant_act(x)
    xs, sxs = rowops.moe_gather(xq, sx, pair_of_row, grp_off[-1:], T * k, k)
    tok = (pair_of_row[:M] // k).long()
    assert torch.equal(xs[:M].view(torch.uint8), xq[tok].view(torch.uint8))
    assert torch.equal(sxs[:, :M], sx[:, tok])
    y = torch.randn(T * k, H, device="cuda").bfloat16()
    sh = torch.randn(T, H, device="cuda").bfloat16()
    out = rowops.moe_combine(y, sh, table, row_of_pair, T, H)
    ref = sh.float().clone()
    for j in range(k):
        m = rop[:, j] >= 0
        ref[m] += gates[m, j, None] * y[rop[m, j].long()].float()
    assert _rel(out, ref) < 5e-3


@pytest.mark.parametrize("E,k,ng,tg,sig,shared", [(32, 8, 1, 1, True, True), (64, 6, 8, 3, True, False), (16, 2, 1, 1, False, True)])
def test_moe_route_fused_matches_gemm_topk_align(E, k, ng, tg, sig, shared):
    """Router projection + top-k + align in one launch against the three separate steps (fp32 logits of the same bf16
    operands; the routing tables must agree wherever the top-k margins exceed the summation-order noise, and the
    layouts must describe the same grouping).  Run twice: the ticket counter re-arms itself."""
    from plow_b200.ops import native, rowops
    T, H = 64, 2048
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    w = (torch.randn(E, H, device="cuda", generator=g) * 0.05).bfloat16()
    bias = torch.randn(E, device="cuda", generator=g) * 0.1 if sig else None
    logits = x.float() @ w.float().t()
    ref_table = rowops.router_topk(logits, bias, k, ng, tg, sig, True, 2.5)
    ng_all = E + (1 if shared else 0)
    for _ in range(2):
        table = torch.zeros(T, k, 2, dtype=torch.int32, device="cuda")
        lg = torch.zeros(T, E, device="cuda")
        grp_off = torch.zeros(ng_all + 1, dtype=torch.int32, device="cuda")
        tile_prefix = torch.zeros(ng_all + 1, dtype=torch.int32, device="cuda")
        row_of_pair = torch.zeros(T * k, dtype=torch.int32, device="cuda")
        pair_of_row = torch.zeros(T * k + (T if shared else 0), dtype=torch.int32, device="cuda")
        ticket = getattr(test_moe_route_fused_matches_gemm_topk_align, "_ticket", None)
        if ticket is None:
            ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
            test_moe_route_fused_matches_gemm_topk_align._ticket = ticket
        native.call("plow_moe_route", table, lg, x, x.stride(0), w, bias, T, H, E, k, ng, tg, int(sig), 1, 2.5, 1, 0, E,
                    grp_off, tile_prefix, row_of_pair, pair_of_row, T if shared else 0, 0, ticket, None, None)
        torch.cuda.synchronize()
        native.check_status()
        assert int(ticket[0]) == 0
        assert _rel(lg, logits) < 1e-5
        same = (table[..., 0] == ref_table[..., 0]).all(1)
        assert same.float().mean() > 0.9                       # near-ties may flip with the summation order
        assert _rel(rowops.table_gates(table)[same], rowops.table_gates(ref_table)[same]) < 1e-4
        g2, t2, rop2, por2 = rowops.moe_align(table, 0, E, shared_rows=T if shared else 0)
        assert torch.equal(grp_off, g2) and torch.equal(tile_prefix, t2)
        M = int(grp_off[E])
        eid = table[..., 0].reshape(-1)
        rows = row_of_pair.long()
        assert (rows >= 0).all() and sorted(rows.tolist()) == list(range(M))
        assert torch.equal(pair_of_row[rows], torch.arange(T * k, dtype=torch.int32, device="cuda"))
        assert ((rows >= grp_off[eid.long()]) & (rows < grp_off[eid.long() + 1])).all()
        if shared:
            assert pair_of_row[M:].tolist() == [t * k for t in range(T)]
