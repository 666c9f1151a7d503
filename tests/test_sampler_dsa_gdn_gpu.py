"""Device sampler, sparse-attention indexer (scores + exact top-k) and gated-delta-rule kernels vs PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sampler_matches_reference_draws():
    from plow_b200.ops import sampler
    torch.manual_seed(0)
    rows, V = 12, 50000
    logits = (torch.randn(rows, V, device="cuda") * 3).float()
    temperature = torch.tensor([0.0, 1.0, 0.7, 1.3, 1.0, 1.0, 0.5, 1.0, 2.0, 1.0, 1.0, 0.9], device="cuda")
    top_k = torch.tensor([0, 0, 50, 0, 1, 0, 10, 1000, 0, 0, 5, 40], dtype=torch.int32, device="cuda")
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 1.0, 0.5, 0.8, 0.95, 1.0, 0.1, 1.0, 0.7], device="cuda")
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.05, 0.0, 0.2, 0.01], device="cuda")
    hits = total = 0
    for trial in range(4):
        u = torch.rand(rows, device="cuda")
        got = sampler.sample(logits, temperature, top_k, top_p, min_p, u=u).tolist()
        want = sampler.reference(logits, temperature, top_k, top_p, min_p, u)
        for r in range(rows):
            total += 1
            hits += got[r] == want[r]
            # whatever rounding does at a boundary, the drawn token must be inside the reference's support
            assert got[r] == want[r] or temperature[r] > 0
    assert hits >= total - 3, (hits, total)
    assert got[0] == int(logits[0].argmax()) and got[4] == int(logits[4].argmax())


def test_sampler_seeded_replay_and_distribution():
    from plow_b200.ops import sampler
    torch.manual_seed(1)
    V = 64
    logits = torch.randn(1, V, device="cuda").repeat(4096, 1).contiguous()
    seed = torch.arange(4096, dtype=torch.int64, device="cuda")
    a = sampler.sample(logits, seed=seed, step=3)
    b = sampler.sample(logits, seed=seed, step=3)
    c = sampler.sample(logits, seed=seed, step=4)
    assert torch.equal(a, b) and not torch.equal(a, c)
    freq = torch.bincount(a.long(), minlength=V).float() / 4096
    p = torch.softmax(logits[0], 0)
    assert (freq - p).abs().max().item() < 0.03


def _index_case(rows, lens, rot=64):
    from plow_b200.ops import dsa
    dev = "cuda"
    pages_per = (max(lens) + 63) // 64
    n_pages = rows * pages_per + 1
    cache = torch.zeros(n_pages, 64, 128, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    cs = torch.zeros(n_pages, 64, device=dev)
    pt = (torch.randperm(n_pages - 1, device=dev).int() + 1)[: rows * pages_per].view(rows, pages_per).contiguous()
    tab = torch.randn(max(lens) + 1, rot, device=dev)
    gamma, beta = torch.randn(128, device=dev), torch.randn(128, device=dev) * 0.1
    # fill the cache through the write kernel, one position per row per call
    for t in range(max(lens)):
        act = [r for r in range(rows) if t < lens[r]]
        k = torch.randn(len(act), 128, device=dev).bfloat16()
        pos = torch.full((len(act),), t, dtype=torch.int32, device=dev)
        seq = torch.tensor(act, dtype=torch.int32, device=dev)
        dsa.k_write(cache, cs, k, gamma, beta, tab, pos, seq, pt, rot)
    return cache, cs, pt, tab


def test_dsa_k_write_and_select():
    from plow_b200.ops import dsa, native
    torch.manual_seed(2)
    rows, lens, top_k, rot = 3, [40, 300, 129], 64, 64
    cache, cs, pt, tab = _index_case(rows, lens, rot)
    # spot-check one written row against LayerNorm + RoPE in fp32 (e4m3 tolerance)
    dev = "cuda"
    k = torch.randn(1, 128, device=dev).bfloat16()
    gamma, beta = torch.randn(128, device=dev), torch.randn(128, device=dev) * 0.1
    pos = torch.tensor([7], dtype=torch.int32, device=dev)
    seq = torch.tensor([0], dtype=torch.int32, device=dev)
    dsa.k_write(cache, cs, k, gamma, beta, tab, pos, seq, pt, rot)
    x = k[0].float()
    want = dsa._rope(((x - x.mean()) * torch.rsqrt(x.var(unbiased=False) + 1e-6) * gamma + beta)[None], tab[7][None], rot, 0)[0]
    got = cache[int(pt[0, 0]), 7].float() * cs[int(pt[0, 0]), 7]
    assert (got - want).abs().max().item() < 0.08 * want.abs().max().item()
    q = torch.randn(rows, 64 * 128, device=dev).bfloat16()
    w = torch.randn(rows, 64, device=dev)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev)
    seq = torch.arange(rows, dtype=torch.int32, device=dev)
    ws = dsa.SelectWorkspace(rows, max(lens), dev)
    sel = dsa.select(q, w, cache, cs, tab, pos, seq, pt, top_k, ws, rot)
    torch.cuda.synchronize()
    native.check_status()
    ref = dsa.reference_scores(q, w, cache, cs, tab, pos, seq, pt, rot)
    for r in range(rows):
        n = lens[r]
        got_sc = ws.scores[r, :n]
        assert (got_sc - ref[r]).abs().max().item() < 2e-2 * ref[r].abs().max().item() + 1e-3
        s = sel[r].tolist()
        if n <= top_k:
            assert s[:n] == list(range(n)) and all(v == -1 for v in s[n:])
        else:
            # exact with respect to the kernel's own scores: (score desc, lowest index on ties)
            order = torch.sort(got_sc, descending=True, stable=True).indices[:top_k]
            assert sorted(order.tolist()) == s


def test_gdn_prefill_then_decode_and_gated_norm():
    from plow_b200.ops import gdn
    torch.manual_seed(3)
    dev = "cuda"
    hk, hv, d, conv = 2, 4, 128, 4
    C = (2 * hk + hv) * d
    Z = hv * d
    slots = 3
    conv_w = torch.randn(C, conv, device=dev) * 0.5
    a_log = torch.randn(hv, device=dev) * 0.5
    dt_bias = torch.randn(hv, device=dev) * 0.5
    conv_state = torch.zeros(slots, C, conv - 1, device=dev)
    ssm_state = torch.zeros(slots, hv, d, d, device=dev)
    # step 1: sequence 2 prefills 37 tokens, sequence 0 prefills 5
    T1 = {2: 37, 0: 5}
    qkvz = (torch.randn(42, C + Z, device=dev)).bfloat16()
    ba = torch.randn(42, 2 * hv, device=dev).bfloat16()
    seq = torch.tensor([2] * 37 + [0] * 5, dtype=torch.int32, device=dev)
    pos = torch.tensor(list(range(37)) + list(range(5)), dtype=torch.int32, device=dev)
    out = gdn.gdn(qkvz, ba, conv_w, a_log, dt_bias, conv_state, ssm_state, pos, seq, hk, hv)
    torch.cuda.synchronize()
    o2, h2, S2 = gdn.reference(qkvz[:37], ba[:37], conv_w, a_log, dt_bias, hk, hv)
    o0, h0, S0 = gdn.reference(qkvz[37:], ba[37:], conv_w, a_log, dt_bias, hk, hv)
    assert (out[:37].float() - o2).abs().max().item() < 2e-2 * o2.abs().max().item() + 1e-3
    assert (out[37:].float() - o0).abs().max().item() < 2e-2 * o0.abs().max().item() + 1e-3
    assert (ssm_state[2] - S2).abs().max().item() < 1e-3 * S2.abs().max().item() + 1e-4
    assert (conv_state[2] - h2).abs().max().item() < 1e-5 and (conv_state[0] - h0).abs().max().item() < 1e-5
    # step 2: both decode one token (continuing from the stored states); an idle row is skipped
    qkvz2 = torch.randn(3, C + Z, device=dev).bfloat16()
    ba2 = torch.randn(3, 2 * hv, device=dev).bfloat16()
    seq2 = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    pos2 = torch.tensor([5, -1, 37], dtype=torch.int32, device=dev)
    out2 = gdn.gdn(qkvz2, ba2, conv_w, a_log, dt_bias, conv_state, ssm_state, pos2, seq2, hk, hv)
    torch.cuda.synchronize()
    r0, _, _ = gdn.reference(qkvz2[0:1], ba2[0:1], conv_w, a_log, dt_bias, hk, hv, conv_hist=h0, S=S0)
    r2, _, _ = gdn.reference(qkvz2[2:3], ba2[2:3], conv_w, a_log, dt_bias, hk, hv, conv_hist=h2, S=S2)
    assert (out2[0].float() - r0[0]).abs().max().item() < 2e-2 * r0.abs().max().item() + 1e-3
    assert (out2[2].float() - r2[0]).abs().max().item() < 2e-2 * r2.abs().max().item() + 1e-3
    # gated norm
    gamma = torch.randn(d, device=dev)
    on = gdn.gated_norm(out, qkvz, C, gamma, hv, d, 1e-6)
    o = out.float().view(42, hv, d)
    want = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma * torch.nn.functional.silu(qkvz[:, C:].float().view(42, hv, d))
    assert (on.float().view(42, hv, d) - want).abs().max().item() < 2e-2 * want.abs().max().item()
    g = torch.randn(42, hv * d, device=dev).bfloat16()
    sg = gdn.sigmoid_gate(out, g)
    assert (sg.float() - out.float() * torch.sigmoid(g.float())).abs().max().item() < 2e-2


def test_dsa_gather_feeds_dense_decode_kernel():
    """Sparse MLA: gathering each row's selected tokens into its compact cache and decoding over it equals decoding over
    a cache that holds exactly those tokens."""
    import math
    from plow_b200.ops import dsa, mla, native
    torch.manual_seed(6)
    dev = "cuda"
    T, ctx, top_k = 3, 700, 128
    pages_per = (ctx + 63) // 64
    n_pages = T * pages_per + 1
    kv8 = torch.randn(n_pages, 64, 576, device=dev).to(torch.float8_e4m3fn)
    ksc = torch.rand(n_pages, 64, device=dev) * 0.01 + 0.005
    pt = (torch.arange(T * pages_per, dtype=torch.int32, device=dev).view(T, pages_per) + 1).contiguous()
    seq = torch.arange(T, dtype=torch.int32, device=dev)
    pos = torch.tensor([ctx - 1, 99, 400], dtype=torch.int32, device=dev)
    sel = torch.full((T, top_k), -1, dtype=torch.int32, device=dev)
    for r in range(T):
        n = int(pos[r]) + 1
        pick = torch.arange(n) if n <= top_k else torch.randperm(n)[:top_k].sort().values
        sel[r, :len(pick)] = pick.int().to(dev)
    cc = dsa.CompactCache(T, top_k, 576, dev)
    dsa.gather(cc, sel, kv8, ksc, pos, seq, pt)
    torch.cuda.synchronize()
    assert cc.kvlen.tolist() == [128, 100, 128]
    # oracle cache: the selected rows copied with torch indexing
    okv = torch.zeros_like(cc.kv.view(torch.uint8))
    osc = torch.zeros_like(cc.scale)
    for r in range(T):
        n = int(cc.kvlen[r])
        t = sel[r, :n].long()
        pages = pt[r][(t // 64)].long()
        flat_kv = okv.view(T, top_k, 576)
        flat_kv[r, :n] = kv8.view(torch.uint8)[pages, t % 64]
        osc.view(T, top_k)[r, :n] = ksc[pages, t % 64]
    assert torch.equal(okv.view(T, top_k, 576)[0], cc.kv.view(torch.uint8).view(T, top_k, 576)[0])
    osmax = torch.zeros_like(cc.smax)
    osmax[:, 0] = osc.amax(1)
    assert torch.allclose(osmax[:, 0], cc.smax[:, 0])
    q8 = torch.randn(128, T, 576, device=dev).to(torch.float8_e4m3fn)
    sq = torch.rand(128, T, device=dev) * 0.01
    ws = mla.DecodeWorkspace(T, top_k + 64, tiles_per_split=64)
    a = torch.empty(128, T, 512, dtype=torch.bfloat16, device=dev)
    b = torch.empty_like(a)
    mla.decode(q8, sq, cc.kv, cc.scale, cc.smax, cc.page_table, cc.slot_of, cc.kvlen, ws, 1 / math.sqrt(192), out=a)
    mla.decode(q8, sq, okv.view(torch.float8_e4m3fn), osc, osmax, cc.page_table, cc.slot_of, cc.kvlen, ws, 1 / math.sqrt(192), out=b)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(a, b)


def test_gdn_chunked_prefill_matches_recurrence():
    """WY-form chunked prefill (64-token chunks, affine state scan) against the fp32 token-by-token recurrence: 1000
    tokens that do not fill the last chunk, continuing from a non-zero state, then a decode step of the kernel from the
    state the chunked path left."""
    from plow_b200.ops import gdn
    torch.manual_seed(7)
    dev = "cuda"
    hk, hv, d, conv = 2, 4, 128, 4
    C = (2 * hk + hv) * d
    conv_w = torch.randn(C, conv, device=dev) * 0.5
    a_log = torch.randn(hv, device=dev) * 0.5
    dt_bias = torch.randn(hv, device=dev) * 0.5
    T0, T1 = 100, 1000
    qkvz = torch.randn(T0 + T1, C + hv * d, device=dev).bfloat16()
    ba = torch.randn(T0 + T1, 2 * hv, device=dev).bfloat16()
    o_ref, h_ref, S_ref = gdn.reference(qkvz, ba, conv_w, a_log, dt_bias, hk, hv)
    _, h0, S0 = gdn.reference(qkvz[:T0], ba[:T0], conv_w, a_log, dt_bias, hk, hv)
    out, h1, S1 = gdn.chunked_prefill(qkvz[T0:], ba[T0:], conv_w, a_log, dt_bias, h0, S0, hk, hv)
    assert (out - o_ref[T0:]).abs().max().item() < 2e-3 * o_ref.abs().max().item() + 1e-4
    assert (S1 - S_ref).abs().max().item() < 2e-3 * S_ref.abs().max().item() + 1e-4
    assert (h1 - h_ref).abs().max().item() < 1e-5
    # the token-by-token kernel continues from that state
    conv_state = torch.zeros(1, C, conv - 1, device=dev)
    ssm_state = torch.zeros(1, hv, d, d, device=dev)
    conv_state[0], ssm_state[0] = h1, S1
    q2 = torch.randn(1, C + hv * d, device=dev).bfloat16()
    b2 = torch.randn(1, 2 * hv, device=dev).bfloat16()
    o2 = gdn.gdn(q2, b2, conv_w, a_log, dt_bias, conv_state, ssm_state, torch.tensor([T0 + T1], dtype=torch.int32, device=dev),
                 torch.zeros(1, dtype=torch.int32, device=dev), hk, hv)
    r2, _, _ = gdn.reference(q2, b2, conv_w, a_log, dt_bias, hk, hv, conv_hist=h_ref, S=S_ref)
    assert (o2[0].float() - r2[0]).abs().max().item() < 2e-2 * r2.abs().max().item() + 1e-3
