"""Each CUDA kernel alone against a plain fp32/fp64 torch statement of the same op, at
sizes other than the engine's tiny models: widths and vocabularies that are no power of
two, several head sizes, page sizes and group counts."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def K():
    from rustinfer_b200.ops import kernels
    return kernels


def tol(dtype):
    # one rounding to the storage type on the way out, measured against a float64 statement
    return 2e-6 if dtype == torch.float32 else 2 ** -8


def close_attention(got, case, ref):
    """bf16 attention: the output is rounded once (half an ulp of its size, 2^-9 relative) and
    the probabilities were rounded to bf16 before they met the values (2^-9 relative each,
    so at most 2^-9 of the largest |v| in the weighted mean): |err| <= 2^-9 (max|out| + max|v|)."""
    ref = ref.double().cpu()
    vmax = max(float(v.double().abs().max()) for v in case.v)
    bound = 2 ** -9 * (float(ref.abs().max()) + vmax)
    err = float((got.double().cpu() - ref).abs().max())
    assert err <= bound, f"max err {err:.3e} vs bound {bound:.3e}"


def close(got, ref, dtype, scale=None):
    ref = ref.double().cpu()
    scale = float(ref.abs().max()) if scale is None else scale
    err = float((got.double().cpu() - ref).abs().max())
    assert err <= tol(dtype) * max(scale, 1e-30), f"max err {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("tdt", DT)
@pytest.mark.parametrize("d,vocab", [(72, 131), (1000, 517), (4100, 33)])
def test_embed_gather(tdt, d, vocab):
    torch.manual_seed(0)
    table = torch.randn(vocab, d).to(tdt).to(dev())
    ids = torch.randint(0, vocab, (37,), dtype=torch.int32, device=dev())
    out = torch.empty(37, d, dtype=torch.float32, device=dev())
    K().embed_gather(ids, table, out)
    assert torch.equal(out.cpu(), P.embedding(table.cpu().double(), ids.tolist()).float())


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("wdt", DT)
@pytest.mark.parametrize("d", [80, 1000, 4100])
def test_add_rmsnorm(adt, wdt, d):
    torch.manual_seed(1)
    T, eps = 19, 3e-6
    h0 = (torch.randn(T, d) * 3).to(dev())
    delta = torch.randn(T, d).to(adt).to(dev())
    w = (1 + 0.3 * torch.randn(d)).to(wdt).to(dev())
    # with delta: h is updated, out is the norm of the sum
    h = h0.clone()
    out = torch.empty(T, d, dtype=adt, device=dev())
    K().add_rmsnorm(h, delta, w, eps, out)
    s = h0.double().cpu() + delta.double().cpu()
    assert torch.equal(h.cpu(), (h0 + delta.float()).cpu())           # the residual sum is fp32
    close(out, P.rmsnorm(s, w.double().cpu(), eps), adt)
    # without delta
    h = h0.clone()
    K().add_rmsnorm(h, None, w, eps, out)
    assert torch.equal(h, h0)
    close(out, P.rmsnorm(h0.double().cpu(), w.double().cpu(), eps), adt)
    # rows: only the chosen rows, h untouched
    rows = torch.tensor([18, 0, 7], dtype=torch.int32, device=dev())
    h = h0.clone()
    out3 = torch.empty(3, d, dtype=adt, device=dev())
    K().add_rmsnorm(h, delta, w, eps, out3, rows)
    assert torch.equal(h, h0)
    close(out3, P.rmsnorm(s[rows.cpu().long()], w.double().cpu(), eps), adt)
    K().residual_add(h, delta)
    assert torch.equal(h.cpu(), (h0 + delta.float()).cpu())


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("inter", [24, 1001, 8192])
def test_silu_mul(dt, inter):
    torch.manual_seed(2)
    gu = (torch.randn(11, 2 * inter) * 4).to(dt).to(dev())
    out = torch.empty(11, inter, dtype=dt, device=dev())
    K().silu_mul(gu, out)
    g, u = gu.double().cpu()[:, :inter], gu.double().cpu()[:, inter:]
    close(out, P.swiglu(g, u), dt)


@pytest.mark.parametrize("M,N,K_", [(1, 130, 96), (37, 53, 129), (64, 64, 16), (70, 391, 272), (5, 1000, 1000)])
def test_gemm_f32_is_exact_fp32(M, N, K_):
    torch.manual_seed(3)
    a = torch.randn(M, K_, device=dev())
    w = torch.randn(N, K_, device=dev())
    out = torch.empty(M, N, device=dev())
    K().gemm_f32(a, w, out)
    ref = a.double().cpu() @ w.double().cpu().T
    # fp32 products summed in fp32: error grows like sqrt(K) * 2^-24 of the row norms; TF32
    # inputs (10-bit mantissa) would miss this bound by three orders of magnitude
    bound = 4 * math.sqrt(K_) * 2 ** -24 * float(a.norm(dim=1).max() * w.norm(dim=1).max())
    assert float((out.double().cpu() - ref).abs().max()) <= bound
    # a row's result does not depend on the other rows of the batch: bit for bit
    one = torch.empty(1, N, device=dev())
    K().gemm_f32(a[M // 2: M // 2 + 1], w, one)
    assert torch.equal(one[0], out[M // 2])
    # strided views (a column block of a wider buffer)
    wide = torch.randn(M, K_ + 24, device=dev())
    K().gemm_f32(wide[:, 8: 8 + K_], w, out)
    assert torch.allclose(out.double().cpu(), wide[:, 8: 8 + K_].double().cpu() @ w.double().cpu().T, atol=bound)


# the last four have 512 tokens or more: tiles of 256 x 256 or 256 x 192 on CTA pairs (cta_group::2;
# the width that makes the waves of tiles shallower), with edges that are no multiple of the tile
# in any direction; the last one has several waves of the narrower tile
TC_SHAPES = [(1, 130, 96), (8, 3072, 2048), (17, 544, 96), (64, 391, 272), (65, 391, 272), (300, 130, 104),
             (200, 1000, 72), (128, 256, 64), (5, 16, 8), (512, 512, 256), (1000, 4000, 520), (777, 264, 72),
             (2040, 3080, 136),
             # many tokens: tiles of a CTA pair, 256 rows by 240, 192 and 224 columns (whatever evens out the waves)
             (2048, 2048, 72), (2048, 5120, 72), (1536, 2500, 72)]


@pytest.mark.parametrize("epi", ["bf16", "f32", "silu", "residual"])
@pytest.mark.parametrize("M,N,K_", TC_SHAPES)
def test_gemm_tc_against_float64(M, N, K_, epi):
    """The tcgen05 kernel in both orientations (few tokens: weight on the 128-row side),
    every epilogue, sizes that are no multiple of any tile."""
    torch.manual_seed(M + N)
    k = K()
    if epi == "silu":
        N -= N % 2                                      # gate/up pairs
    x = torch.randn(M, K_).bfloat16().to(dev())
    w = (torch.randn(N, K_) / math.sqrt(K_)).bfloat16().to(dev())
    ref = x.double().cpu() @ w.double().cpu().T
    if epi == "silu":
        ref = P.swiglu(ref[:, 0::2], ref[:, 1::2])
        out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=dev())
        k.gemm_tc(x, w, out, k.EPI_SILU)
        close(out, ref, torch.bfloat16)
    elif epi == "residual":
        base = torch.randn(M, N, device=dev())
        out = base.clone()
        k.gemm_tc(x, w, out, k.EPI_RESIDUAL)
        close(out, ref + base.double().cpu(), torch.float32)
    elif epi == "f32":
        out = torch.full((M, N), float("nan"), device=dev())
        k.gemm_tc(x, w, out, k.EPI_F32)
        close(out, ref, torch.float32)
    else:
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
        k.gemm_tc(x, w, out, k.EPI_BF16)
        close(out, ref, torch.bfloat16)
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0


@pytest.mark.parametrize("M,N,K_", [(2048, 2560, 4096), (2040, 2500, 4104), (2048, 3072, 8192)])
def test_gemm_tc_dealt_last_wave(M, N, K_):
    """Many tokens, a long K and a last wave of few tiles: the k-blocks of those tiles are dealt
    out over all CTA pairs and the parts meet in a buffer (or, added into the fp32 stream, where
    the whole would go).  Every epilogue; the same bits whichever pair finishes a tile."""
    torch.manual_seed(N)
    k = K()
    x = torch.randn(M, K_, device=dev()).bfloat16()
    w = (torch.randn(N, K_, device=dev()) / math.sqrt(K_)).bfloat16()
    ref = (x.double() @ w.double().T).cpu()                  # the oracle: a float64 product
    outs = []
    for _ in range(3):
        out = torch.full((M, N), float("nan"), device=dev())
        k.gemm_tc(x, w, out, k.EPI_F32)
        outs.append(out)
    # a sum of K products kept in fp32: |err| <= (K + 2) 2^-24 sum |x||w| (one rounding per
    # addition and per part); a k-block left out or added twice would be off by about 0.1
    bound = (K_ + 2) * 2.0 ** -24 * float((x.double().abs() @ w.double().abs().T).max())
    err = float((outs[0].double().cpu() - ref).abs().max())
    assert err <= bound, f"max err {err:.3e} vs bound {bound:.3e}"
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    k.gemm_tc(x, w, out, k.EPI_BF16)
    assert torch.equal(out, outs[0].bfloat16())              # the same sum, rounded once
    out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=dev())
    k.gemm_tc(x, w, out, k.EPI_SILU)
    f = outs[0].double().cpu()
    close(out, P.swiglu(f[:, 0::2], f[:, 1::2]), torch.bfloat16)
    base = torch.randn(M, N, device=dev())
    h = base.clone()
    k.gemm_tc(x, w, h, k.EPI_RESIDUAL)
    err = float((h.double().cpu() - (ref + base.double().cpu())).abs().max())
    assert err <= bound + 2.0 ** -23 * float(h.abs().max()), f"max err {err:.3e} vs bound {bound:.3e}"
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0
    # the counters are left zero: a second product of another shape right behind it
    x2 = torch.randn(70, 1032, device=dev()).bfloat16()
    w2 = (torch.randn(300, 1032, device=dev()) / 32).bfloat16()
    out2 = torch.full((70, 300), float("nan"), device=dev())
    k.gemm_tc(x2, w2, out2, k.EPI_F32, (1, 16, 7))
    close(out2, (x2.double() @ w2.double().T).cpu(), torch.float32)


@pytest.mark.parametrize("plan", [(1, 16, 1), (1, 16, 7), (1, 64, 3), (0, 16, 1), (0, 128, 2), (0, 256, 1), (0, 64, 5),
                                  (1, 16, 1, 64), (1, 32, 1, 104), (1, 16, 3, 72)])
def test_gemm_tc_plans_and_split_k(plan):
    """Every tile width and orientation on one problem, with and without K slices; the
    sliced result is the same bits whichever CTA finishes last (slices are added in order)."""
    torch.manual_seed(7)
    k = K()
    M, N, K_ = 70, 300, 1032
    x = torch.randn(M, K_).bfloat16().to(dev())
    w = (torch.randn(N, K_) / math.sqrt(K_)).bfloat16().to(dev())
    ref = x.double().cpu() @ w.double().cpu().T
    outs = []
    for _ in range(3):
        out = torch.full((M, N), float("nan"), device=dev())
        k.gemm_tc(x, w, out, k.EPI_F32, plan)
        outs.append(out)
    close(outs[0], ref, torch.float32)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0
    # K slices of a product that is added into the fp32 stream add their parts one by one
    base = torch.randn(M, N, device=dev())
    h = base.clone()
    k.gemm_tc(x, w, h, k.EPI_RESIDUAL, plan)
    close(h, ref + base.double().cpu(), torch.float32)
    # pairs of rows (gate, up) through SiLU, with tiles that cover fewer than 128 rows
    out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=dev())
    k.gemm_tc(x, w, out, k.EPI_SILU, plan)
    close(out, P.swiglu(ref[:, 0::2], ref[:, 1::2]), torch.bfloat16)
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0


def _rope_tables(positions, rot, theta=10000.0):
    f = P.rope_inv_freq(rot, theta, None)
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * f[None, :]
    return torch.cos(ang), torch.sin(ang)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("Hq,Hkv,hd,rot,page", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (6, 3, 48, 48, 16),
                                                (5, 5, 64, 32, 4), (8, 2, 128, 128, 32)])
def test_rope_scatter(dt, Hq, Hkv, hd, rot, page):
    torch.manual_seed(4)
    T, pages, maxpos = 23, 9, 200
    qkv0 = torch.randn(T, (Hq + 2 * Hkv) * hd).to(dt)
    pos = torch.randint(0, maxpos, (T,), dtype=torch.int32)
    c, s = _rope_tables(maxpos, rot)
    slots = torch.randperm(pages * page)[:T].to(torch.int32)
    slots[5] = -1                                                     # a token that is not stored
    cache = torch.full((pages, 2, Hkv, page, hd), 7.0, dtype=dt, device=dev())
    qkv = qkv0.clone().to(dev())
    K().rope_scatter(qkv, pos.to(dev()), c.float().to(dev()), s.float().to(dev()), slots.to(dev()), cache,
                     Hq, Hkv, hd, rot)
    x = qkv0.double().view(T, Hq + 2 * Hkv, hd)
    f = P.rope_inv_freq(rot, 10000.0, None)
    rotated = torch.cat([P.rope_rotate(x[..., :rot], pos, f), x[..., rot:]], dim=-1)
    got = qkv.double().cpu().view(T, Hq + 2 * Hkv, hd)
    close(got[:, :Hq], rotated[:, :Hq], dt)
    assert torch.equal(got[:, Hq:], x[:, Hq:])                        # k and v columns are left alone
    want = torch.full((pages, 2, Hkv, page, hd), 7.0, dtype=torch.float64)
    for t in range(T):
        if slots[t] < 0:
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        want[pg, 0, :, off] = rotated[t, Hq: Hq + Hkv]
        want[pg, 1, :, off] = x[t, Hq + Hkv:]
    close(cache, want, dt, scale=float(x.abs().max()))
    untouched = want == 7.0
    assert torch.equal(cache.double().cpu()[untouched], want[untouched])


@pytest.mark.parametrize("M,hidden,Hq,Hkv,hd,page", [
    (600, 136, 8, 2, 64, 16),                    # a ragged last row tile, three tiles of 256 columns
    (1030, 264, 6, 2, 128, 8),                   # heads of 128: a tile holds two heads
    (512, 72, 5, 0, 64, 16),                     # a layer that keeps no keys: q alone
    (700, 200, 24, 8, 128, 32),                  # the 3B grouping, many column tiles
])
def test_gemm_tc_with_rotary_epilogue(M, hidden, Hq, Hkv, hd, page):
    """q, k, v of many tokens with the rotary encoding and the cache write in the product's
    epilogue, against the float64 product rotated by the plain implementation; tokens without a
    slot are not stored and no other slot of the cache is touched."""
    torch.manual_seed(M + hd)
    k = K()
    N = (Hq + 2 * Hkv) * hd
    maxpos, pages = 300, (M + page - 1) // page + 3
    x = torch.randn(M, hidden).bfloat16()
    w = (torch.randn(N, hidden) / math.sqrt(hidden)).bfloat16()
    pos = torch.randint(0, maxpos, (M,), dtype=torch.int32)
    c, s_ = _rope_tables(maxpos, hd)
    slots = torch.randperm(pages * page)[:M].to(torch.int32)
    slots[7] = -1
    cache = torch.full((pages, 2, max(Hkv, 1), page, hd), 7.0, dtype=BF, device=dev()) if Hkv else None
    q = torch.full((M, Hq * hd), float("nan"), dtype=BF, device=dev())
    ran = k.gemm_tc_rope(x.to(dev()), w.to(dev()), q, pos.to(dev()), c.float().to(dev()), s_.float().to(dev()),
                         slots.to(dev()) if Hkv else None, cache, Hq, Hkv, hd)
    assert ran
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0
    y = (x.double() @ w.double().T).view(M, Hq + 2 * Hkv, hd)
    f = P.rope_inv_freq(hd, 10000.0, None)
    rotated = P.rope_rotate(y[:, : Hq + Hkv], pos, f)
    close(q.double().cpu().view(M, Hq, hd), rotated[:, :Hq], BF)
    if Hkv:
        want = torch.full((pages, 2, Hkv, page, hd), 7.0, dtype=torch.float64)
        for t in range(M):
            if slots[t] < 0:
                continue
            pg, off = int(slots[t]) // page, int(slots[t]) % page
            want[pg, 0, :, off] = rotated[t, Hq:]
            want[pg, 1, :, off] = y[t, Hq + Hkv:]
        close(cache, want, BF, scale=float(y.abs().max()))
        untouched = want == 7.0
        assert torch.equal(cache.double().cpu()[untouched], want[untouched])
    # fewer than 512 tokens: the caller is told to go the two-kernel way, and nothing is written
    q2 = torch.full((100, Hq * hd), float("nan"), dtype=BF, device=dev())
    assert not k.gemm_tc_rope(x[:100].contiguous().to(dev()), w.to(dev()), q2, pos[:100].to(dev()), c.float().to(dev()),
                              s_.float().to(dev()), slots[:100].to(dev()) if Hkv else None, cache, Hq, Hkv, hd)
    assert torch.isnan(q2.float()).all()


@pytest.mark.parametrize("M,hidden,inter,Hq,Hkv,hd,rot,page", [
    (8, 2048, 8192, 32, 8, 64, 64, 16),          # the shapes of a 1B decoder
    (4, 4096, 14336, 32, 8, 128, 128, 16),        # ... of an 8B one: rows of the stream staged four at a time
    (12, 3072, 8192, 24, 8, 128, 128, 32),        # ... of a 3B one, more than 8 tokens
    (5, 272, 552, 6, 2, 48, 32, 8),               # nothing a power of two, part of each head rotates
    (19, 520, 1040, 5, 5, 32, 32, 4),             # more than 16 tokens: the operand streams with the weights
    (40, 2048, 8192, 32, 8, 64, 64, 16),          # ... 33 or more: 64-token tiles
    (64, 272, 552, 6, 2, 48, 32, 8),
    (1, 136, 96, 3, 1, 16, 16, 16),
])
def test_decode_chain(M, hidden, inter, Hq, Hkv, hd, rot, page):
    """Five steps of a decoder layer's seam in one kernel: attention output times Wo into the
    stream, norm + gate/up + SiLU, down into the stream, norm + q,k,v, rotary + cache write;
    against the plain formulas in float64 from the same bf16 weights."""
    torch.manual_seed(M + hidden)
    k = K()
    d = dev()
    qdim, width = Hq * hd, (Hq + 2 * Hkv) * hd
    bf = lambda t: t.bfloat16().to(d)
    wo, wg, wu = torch.randn(hidden, qdim) / qdim ** 0.5, torch.randn(inter, hidden) / hidden ** 0.5, torch.randn(inter, hidden) / hidden ** 0.5
    wd, wqkv = torch.randn(hidden, inter) / inter ** 0.5, torch.randn(width, hidden) / hidden ** 0.5
    n1, n2 = 1 + 0.2 * torch.randn(hidden), 1 + 0.2 * torch.randn(hidden)
    wo_d, wd_d, wqkv_d = bf(wo), bf(wd), bf(wqkv)
    wgu_d = torch.stack([wg, wu], dim=1).reshape(2 * inter, hidden).bfloat16().to(d)     # rows alternate gate, up
    n1_d, n2_d = bf(n1), n2.to(d)                                                        # one norm weight in each dtype
    attn = torch.randn(M, qdim)
    h0 = torch.randn(M, hidden) * 2
    rows = 64                                                                            # buffers hold more rows than are used
    attn_d = torch.zeros(rows, qdim, dtype=torch.bfloat16, device=d); attn_d[:M] = bf(attn)
    h_d = torch.zeros(rows, hidden, dtype=torch.float32, device=d); h_d[:M] = h0.to(d)
    m_d = torch.full((rows, inter), 9.0, dtype=torch.bfloat16, device=d)
    qkv_d = torch.zeros(rows, width, dtype=torch.float32, device=d)
    q_d = torch.full((rows, qdim), 9.0, dtype=torch.bfloat16, device=d)
    xn_d = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=d)                      # wide steps only
    sq_a, sq_b = torch.zeros(rows, device=d), torch.zeros(rows, device=d)
    pages, maxpos = 12, 300
    pos = torch.randint(0, maxpos, (rows,), dtype=torch.int32)
    c, s_ = _rope_tables(maxpos, rot)
    slots = torch.randperm(pages * page)[:rows].to(torch.int32)
    if M > 2:
        slots[2] = -1                                                                    # a token that is not stored
    cache = torch.full((pages, 2, Hkv, page, hd), 7.0, dtype=torch.bfloat16, device=d)
    products = [k.ChainProduct(wo_d, attn_d, h_d, k.CHAIN_ADD_F32),
                k.ChainProduct(wgu_d, h_d, m_d, k.CHAIN_SILU_BF16, norm=(n1_d, 1e-5), xn=xn_d, rowsq=sq_a),
                k.ChainProduct(wd_d, m_d, h_d, k.CHAIN_ADD_F32),
                k.ChainProduct(wqkv_d, h_d, qkv_d, k.CHAIN_ADD_F32, norm=(n2_d, 3e-6), xn=xn_d, rowsq=sq_b)]
    rope = k.ChainRope(qkv_d, pos.to(d), c.float().to(d), s_.float().to(d), slots.to(d), q_d, cache, Hq, Hkv, hd, rot)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert k.decode_chain_fits(products, M, sms)
    for _ in range(2):                                       # twice: the barrier and the q,k,v buffer reset themselves
        h_d[:M] = h0.to(d)
        k.decode_chain(products, rope, M, sms)
    torch.cuda.synchronize()
    assert k.gemm_tc_error(d) == 0
    # ---- the same in float64 from the rounded weights
    D = lambda t: t.double().cpu()
    h1 = h0.double() + D(bf(attn)) @ D(wo_d).T
    x1 = P.rmsnorm(h1, D(n1_d), 1e-5)
    mid = P.swiglu(x1 @ D(bf(wg)).T, x1 @ D(bf(wu)).T)
    close(m_d[:M], mid, torch.bfloat16)
    assert torch.all(m_d[M:] == 9.0)
    h2 = h1 + D(m_d[:M]) @ D(wd_d).T                        # from the kernel's own rounded intermediate
    close(h_d[:M], h2, torch.bfloat16)
    x2 = P.rmsnorm(D(h_d[:M]), D(n2_d), 3e-6)
    qkv = (x2 @ D(wqkv_d).T).view(M, Hq + 2 * Hkv, hd)
    f = P.rope_inv_freq(rot, 10000.0, None)
    rotated = torch.cat([P.rope_rotate(qkv[..., :rot], pos[:M], f), qkv[..., rot:]], dim=-1)
    scale = float(qkv.abs().max())
    close(q_d[:M].view(M, Hq, hd), rotated[:, :Hq], torch.bfloat16, scale=scale)
    assert torch.all(q_d[M:] == 9.0)
    want = torch.full((pages, 2, Hkv, page, hd), 7.0, dtype=torch.float64)
    for t in range(M):
        if slots[t] < 0:
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        want[pg, 0, :, off] = rotated[t, Hq: Hq + Hkv]
        want[pg, 1, :, off] = qkv[t, Hq + Hkv:]
    close(cache, want, torch.bfloat16, scale=scale)
    untouched = want == 7.0
    assert torch.equal(cache.double().cpu()[untouched], want[untouched])
    assert torch.count_nonzero(qkv_d) == 0                   # left at zero for the next chain
    assert torch.count_nonzero(sq_a) == 0 and torch.count_nonzero(sq_b) == 0


class PagedCase:
    """A ragged batch laid out in a paged cache by hand, for the attention kernels."""

    def __init__(self, dt, Hq, Hkv, hd, page, kv_lens, q_lens, seed=0, poison=True):
        g = torch.Generator().manual_seed(seed)
        self.dt, self.Hq, self.Hkv, self.hd, self.page = dt, Hq, Hkv, hd, page
        self.kv_lens, self.q_lens = kv_lens, q_lens
        B = len(kv_lens)
        blocks = [(n + page - 1) // page for n in kv_lens]
        n_pages = sum(blocks) + 3
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.k = [torch.randn(n, Hkv, hd, generator=g).to(dt) for n in kv_lens]
        self.v = [torch.randn(n, Hkv, hd, generator=g).to(dt) for n in kv_lens]
        self.q = [torch.randn(n, Hq, hd, generator=g).to(dt) for n in q_lens]
        fill = float("nan") if poison else 0.0
        cache = torch.full((n_pages, 2, Hkv, page, hd), fill, dtype=dt)
        table = torch.zeros(B, max(blocks), dtype=torch.int32)
        at = 0
        for b in range(B):
            for j in range(blocks[b]):
                pg = perm[at]; at += 1
                table[b, j] = pg
                lo, hi = j * page, min((j + 1) * page, kv_lens[b])
                cache[pg, 0, :, : hi - lo] = self.k[b][lo:hi].transpose(0, 1)
                cache[pg, 1, :, : hi - lo] = self.v[b][lo:hi].transpose(0, 1)
        self.cache, self.table = cache.to(dev()), table.to(dev())
        cu = [0]
        for n in q_lens:
            cu.append(cu[-1] + n)
        self.cu_q = torch.tensor(cu, dtype=torch.int32, device=dev())
        self.kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=dev())
        self.q_all = torch.cat(self.q).reshape(cu[-1], Hq * hd).to(dev())

    def tiles(self, rows):
        te, tq = [], []
        for b, n in enumerate(self.q_lens):
            for j in range(0, n, rows):
                te.append(b); tq.append(j)
        return (torch.tensor(te, dtype=torch.int32, device=dev()),
                torch.tensor(tq, dtype=torch.int32, device=dev()))

    def reference(self, scale, window=None):
        outs = []
        for b, (n_kv, n_q) in enumerate(zip(self.kv_lens, self.q_lens)):
            # the entry's queries are the last n_q positions of its n_kv keys
            qfull = torch.zeros(n_kv, self.Hq, self.hd, dtype=torch.float64)
            qfull[n_kv - n_q:] = self.q[b].double()
            o = P.causal_gqa_attention(qfull, self.k[b].double(), self.v[b].double(), scale, window)
            outs.append(o[n_kv - n_q:])
        return torch.cat(outs).reshape(-1, self.Hq * self.hd)


ATT_SHAPES = [(4, 2, 16, 16), (3, 1, 32, 8), (6, 3, 48, 16), (8, 2, 64, 16), (4, 4, 128, 32),
              (2, 1, 256, 16), (10, 5, 80, 4)]


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("Hq,Hkv,hd,page", ATT_SHAPES)
def test_attention_plain_ragged(dt, Hq, Hkv, hd, page):
    # whole prompts, portions that start mid-page, single decode tokens, lengths at page edges
    kv_lens = [1, 17, 64, 65, 130, 33, 16]
    q_lens = [1, 17, 1, 2, 41, 33, 1]
    case = PagedCase(dt, Hq, Hkv, hd, page, kv_lens, q_lens, seed=hd)
    out = torch.empty_like(case.q_all)
    te, tq = case.tiles(16)
    scale = 1 / math.sqrt(hd)
    K().attention_plain(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                        Hq, Hkv, hd, scale, None)
    close(out, case.reference(scale), dt)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("window", [1, 5, 16, 40])
def test_attention_plain_window(dt, window):
    case = PagedCase(dt, 4, 2, 32, 8, [70, 9, 40], [30, 9, 1], seed=window)
    out = torch.empty_like(case.q_all)
    te, tq = case.tiles(16)
    K().attention_plain(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                        4, 2, 32, 0.2, window)
    close(out, case.reference(0.2, window), dt)


@pytest.mark.parametrize("dt", DT)
def test_attention_plain_finds_one_far_key(dt):
    """One key among hundreds carries the whole score: the output must be its value.
    A kernel that skips a page, a chunk or a page's last slot gets this visibly wrong."""
    Hq, Hkv, hd, page = 2, 1, 64, 16
    for far in (0, 15, 16, 63, 64, 255, 300, 310):
        case = PagedCase(dt, Hq, Hkv, hd, page, [311], [1], seed=far, poison=True)
        k = case.k[0].double()
        qv = (k[far, 0] / k[far, 0].norm() * 60.0)
        case.q_all = qv.repeat(Hq).to(dt).reshape(1, Hq * hd).to(dev())
        out = torch.empty_like(case.q_all)
        te, tq = case.tiles(16)
        K().attention_plain(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                            Hq, Hkv, hd, 1.0, None)
        want = case.v[0][far, 0].double().repeat(Hq)
        assert float((out.double().cpu()[0] - want).abs().max()) < 0.05, far


def test_attention_plain_is_bitwise_cut_invariant():
    """fp32: the same positions computed as one portion, as two, or token by token give the
    same bits, because keys are always visited in the same chunks from key 0."""
    Hq, Hkv, hd, page = 4, 2, 32, 8
    whole = PagedCase(torch.float32, Hq, Hkv, hd, page, [150], [150], seed=1, poison=False)
    out = torch.empty_like(whole.q_all)
    te, tq = whole.tiles(16)
    K().attention_plain(whole.q_all, out, whole.cache, whole.table, whole.cu_q, whole.kv_len, te, tq,
                        Hq, Hkv, hd, 0.3, None)
    for start, n in [(0, 7), (7, 50), (57, 1), (58, 92), (149, 1)]:
        cu = torch.tensor([0, n], dtype=torch.int32, device=dev())
        kvl = torch.tensor([start + n], dtype=torch.int32, device=dev())
        q = whole.q_all[start: start + n].contiguous()
        o = torch.empty_like(q)
        tiles_e = torch.zeros((n + 15) // 16, dtype=torch.int32, device=dev())
        tiles_q = torch.arange(0, n, 16, dtype=torch.int32, device=dev())
        K().attention_plain(q, o, whole.cache, whole.table, cu, kvl, tiles_e, tiles_q, Hq, Hkv, hd, 0.3, None)
        assert torch.equal(o, out[start: start + n])


# ------------------------------------------------------- tensor-core attention (bf16)
BF = torch.bfloat16
MMA_SHAPES = ATT_SHAPES + [(24, 8, 128, 16), (32, 1, 64, 16), (5, 1, 32, 8)]


def _mma_tiles(case, tpt, skip_decode):
    te, tq = [], []
    for b, n in enumerate(case.q_lens):
        if skip_decode and n == 1:
            continue
        for j in range(0, n, tpt):
            te.append(b); tq.append(j)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    return i32(te), i32(tq)


@pytest.mark.parametrize("Hq,Hkv,hd,page", MMA_SHAPES)
def test_attention_mma_prefill_ragged(Hq, Hkv, hd, page):
    kv_lens = [1, 17, 64, 65, 130, 33, 16, 300]
    q_lens = [1, 17, 1, 2, 41, 33, 1, 129]
    case = PagedCase(BF, Hq, Hkv, hd, page, kv_lens, q_lens, seed=hd + Hq)
    out = torch.full_like(case.q_all, float("nan"))
    tpt = K().mma_tokens_per_tile(Hq, Hkv)
    te, tq = _mma_tiles(case, tpt, skip_decode=False)
    scale = 1 / math.sqrt(hd)
    K().attention_prefill_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                               Hq, Hkv, hd, scale, None)
    close(out, case.reference(scale), BF)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("Hq,Hkv,hd,page", MMA_SHAPES)
def test_attention_mma_decode_and_prefill_side_by_side(Hq, Hkv, hd, page, splits):
    """Single-token entries go through the split-KV decode kernel, the others through the
    prefill kernel, into one output; lengths sit on and around page and tile edges."""
    kv_lens = [1, 64, 41, 65, 128, 500, 63, 129, 16]
    q_lens = [1, 1, 20, 1, 1, 1, 7, 1, 1]
    case = PagedCase(BF, Hq, Hkv, hd, page, kv_lens, q_lens, seed=hd + splits)
    out = torch.full_like(case.q_all, float("nan"))
    dec = [b for b, n in enumerate(q_lens) if n == 1]
    k = K()
    no, nl = k.decode_scratch_floats(len(dec), Hq, hd, splits)
    po = torch.full((no,), float("nan"), device=dev())
    pl = torch.full((nl,), float("nan"), device=dev())
    scale = 1 / math.sqrt(hd)
    k.attention_decode_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len,
                            torch.tensor(dec, dtype=torch.int32, device=dev()), len(dec), Hq, Hkv, hd, scale,
                            None, splits, po, pl)
    te, tq = _mma_tiles(case, k.mma_tokens_per_tile(Hq, Hkv), skip_decode=True)
    k.attention_prefill_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                             Hq, Hkv, hd, scale, None)
    close(out, case.reference(scale), BF)


@pytest.mark.parametrize("window", [1, 5, 16, 40, 100])
def test_attention_mma_window(window):
    Hq, Hkv, hd = 4, 2, 32
    case = PagedCase(BF, Hq, Hkv, hd, 8, [70, 9, 40, 200, 300], [30, 9, 1, 1, 150], seed=window)
    out = torch.full_like(case.q_all, float("nan"))
    k = K()
    te, tq = _mma_tiles(case, k.mma_tokens_per_tile(Hq, Hkv), skip_decode=True)
    k.attention_prefill_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                             Hq, Hkv, hd, 0.2, window)
    no, nl = k.decode_scratch_floats(2, Hq, hd, 3)
    k.attention_decode_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len,
                            torch.tensor([2, 3], dtype=torch.int32, device=dev()), 2, Hq, Hkv, hd, 0.2, window,
                            3, torch.empty(no, device=dev()), torch.empty(nl, device=dev()))
    close(out, case.reference(0.2, window), BF)


@pytest.mark.parametrize("kernel", ["decode", "prefill"])
def test_attention_mma_finds_one_far_key(kernel):
    Hq, Hkv, hd, page = 8, 2, 64, 16
    k = K()
    for far in (0, 15, 16, 63, 64, 255, 300, 310):
        case = PagedCase(BF, Hq, Hkv, hd, page, [311], [1], seed=far, poison=True)
        kk = case.k[0].double()
        rows = []
        for h in range(Hq):
            g = h // (Hq // Hkv)
            rows.append(kk[far, g] / kk[far, g].norm() * 60.0)
        case.q_all = torch.cat(rows).to(BF).reshape(1, Hq * hd).to(dev())
        out = torch.full_like(case.q_all, float("nan"))
        if kernel == "decode":
            no, nl = k.decode_scratch_floats(1, Hq, hd, 4)
            k.attention_decode_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, None, 1,
                                    Hq, Hkv, hd, 1.0, None, 4, torch.empty(no, device=dev()),
                                    torch.empty(nl, device=dev()))
        else:
            te, tq = _mma_tiles(case, k.mma_tokens_per_tile(Hq, Hkv), skip_decode=False)
            k.attention_prefill_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                                     Hq, Hkv, hd, 1.0, None)
        want = torch.cat([case.v[0][far, h // (Hq // Hkv)].double() for h in range(Hq)])
        assert float((out.double().cpu()[0] - want).abs().max()) < 0.05, far


# ------------------------------------------------ tcgen05 prompt attention (bf16, hd 64/128)
# groups of 3, 5, 7 and 12 heads do not divide the 128 rows of a tile: its last rows are padding
TC_ATT_SHAPES = [(8, 2, 64, 16), (32, 8, 64, 16), (4, 4, 64, 8), (16, 1, 64, 32), (8, 2, 128, 16), (24, 3, 128, 64),
                 (2, 2, 128, 8), (6, 2, 128, 16), (24, 8, 128, 16), (5, 1, 64, 16), (14, 2, 64, 32), (12, 1, 128, 8)]


@pytest.mark.parametrize("Hq,Hkv,hd,page", TC_ATT_SHAPES)
def test_attention_tc_prefill_ragged(Hq, Hkv, hd, page):
    """Whole prompts, portions that start mid-page and mid-tile, one-token entries; unused
    slots of the pages hold NaN, which must not leak through P V."""
    k = K()
    assert k.tc_attention_supports(Hq, Hkv, hd, page)
    kv_lens = [1, 17, 64, 65, 130, 33, 16, 300, 515]
    q_lens = [1, 17, 1, 2, 41, 33, 1, 129, 300]
    case = PagedCase(BF, Hq, Hkv, hd, page, kv_lens, q_lens, seed=hd + Hq, poison=True)
    out = torch.full_like(case.q_all, float("nan"))
    te, tq = _mma_tiles(case, k.tc_tokens_per_tile(Hq, Hkv), skip_decode=False)
    scale = 1 / math.sqrt(hd)
    k.attention_prefill_tc(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                           Hq, Hkv, hd, scale, None)
    close_attention(out, case, case.reference(scale))
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0


@pytest.mark.parametrize("window", [1, 5, 16, 40, 100])
def test_attention_tc_window(window):
    Hq, Hkv, hd = 8, 2, 64
    k = K()
    case = PagedCase(BF, Hq, Hkv, hd, 8, [70, 9, 40, 200, 300], [30, 9, 1, 1, 150], seed=window)
    out = torch.full_like(case.q_all, float("nan"))
    te, tq = _mma_tiles(case, k.tc_tokens_per_tile(Hq, Hkv), skip_decode=False)
    k.attention_prefill_tc(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                           Hq, Hkv, hd, 0.2, window)
    close_attention(out, case, case.reference(0.2, window))
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0


def test_attention_tc_finds_one_far_key():
    Hq, Hkv, hd, page = 8, 2, 64, 16
    k = K()
    for far in (0, 15, 16, 63, 64, 255, 300, 310):
        case = PagedCase(BF, Hq, Hkv, hd, page, [311], [1], seed=far, poison=True)
        kk = case.k[0].double()
        rows = [kk[far, h // (Hq // Hkv)] / kk[far, h // (Hq // Hkv)].norm() * 60.0 for h in range(Hq)]
        case.q_all = torch.cat(rows).to(BF).reshape(1, Hq * hd).to(dev())
        out = torch.full_like(case.q_all, float("nan"))
        te, tq = _mma_tiles(case, k.tc_tokens_per_tile(Hq, Hkv), skip_decode=False)
        k.attention_prefill_tc(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                               Hq, Hkv, hd, 1.0, None)
        want = torch.cat([case.v[0][far, h // (Hq // Hkv)].double() for h in range(Hq)])
        assert float((out.double().cpu()[0] - want).abs().max()) < 0.05, far


def _poison_before_window(case, window):
    """Keys no row of an entry may see (before the window of its first row) become NaN, keys and
    values alike, whole pages where the window has passed them: what a request finds where its
    given-back pages used to be."""
    cache = case.cache.cpu()
    table = case.table.cpu()
    for b, (n_kv, n_q) in enumerate(zip(case.kv_lens, case.q_lens)):
        lo = max(0, (n_kv - n_q) - window + 1)
        for key in range(lo):
            cache[int(table[b, key // case.page]), :, :, key % case.page] = float("nan")
    case.cache = cache.to(dev())


@pytest.mark.parametrize("window", [5, 40, 100, 130])
@pytest.mark.parametrize("Hq,Hkv,hd,page", [(8, 2, 64, 16), (4, 1, 128, 16), (6, 2, 128, 8), (8, 8, 64, 64)])
@pytest.mark.parametrize("path", ["decode_tma", "decode_cp_async", "prefill_tc", "prefill_mma"])
def test_attention_window_never_reads_what_lies_before_it(path, Hq, Hkv, hd, page, window):
    """Head sizes 64 and 128 (the kernels that fetch by TMA), a window, and NaN in every key
    and value before it: a probability of zero must not meet them."""
    k = K()
    kv_lens = [70, 9, 40, 200, 300, 515, 131]
    q_lens = [30, 9, 1, 1, 150, 1, 1]
    case = PagedCase(BF, Hq, Hkv, hd, page, kv_lens, q_lens, seed=window + hd, poison=True)
    _poison_before_window(case, window)
    out = torch.full_like(case.q_all, float("nan"))
    ref = case.reference(0.2, window)
    rows = []
    at = 0
    for n in q_lens:
        rows.append((at, n)); at += n
    if path.startswith("decode"):
        dec = [b for b, n in enumerate(q_lens) if n == 1]
        splits = 3
        no, nl = k.decode_scratch_floats(len(dec), Hq, hd, splits)
        k.attention_decode_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len,
                                torch.tensor(dec, dtype=torch.int32, device=dev()), len(dec), Hq, Hkv, hd, 0.2,
                                window, splits, torch.full((no,), float("nan"), device=dev()),
                                torch.full((nl,), float("nan"), device=dev()), by_tma=path == "decode_tma")
        keep = [rows[b][0] for b in dec]
    else:
        if path == "prefill_tc":
            if not k.tc_attention_supports(Hq, Hkv, hd, page):
                pytest.skip("geometry not taken by the tcgen05 kernel")
            te, tq = _mma_tiles(case, k.tc_tokens_per_tile(Hq, Hkv), skip_decode=False)
            k.attention_prefill_tc(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                                   Hq, Hkv, hd, 0.2, window)
        else:
            te, tq = _mma_tiles(case, k.mma_tokens_per_tile(Hq, Hkv), skip_decode=False)
            k.attention_prefill_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                                     Hq, Hkv, hd, 0.2, window)
        keep = list(range(out.shape[0]))
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0
    idx = torch.tensor(keep)
    assert not torch.isnan(out[idx.to(dev())]).any()
    close_attention(out[idx.to(dev())], case, ref[idx])


@pytest.mark.parametrize("V", [130, 391, 128256])
def test_argmax_lowest_index_wins(V):
    torch.manual_seed(5)
    logits = torch.randn(5, V, device=dev())
    logits[1, 7] = logits[1, V - 1] = 50.0
    logits[2, :] = 0.0
    logits[3, V - 1] = 60.0
    logits[4, 3] = float("nan")
    out = torch.empty(5, dtype=torch.int32, device=dev())
    K().argmax(logits, out)
    want = [P.argmax_lowest(torch.nan_to_num(r, nan=-1e30)) for r in logits.cpu()]
    assert out.tolist() == want and out[1] == 7 and out[2] == 0 and out[3] == V - 1


@pytest.mark.parametrize("by_sorting", [False, True])
@pytest.mark.parametrize("V", [130, 391, 5000, 128256])
def test_sample_matches_the_plain_sampler(V, by_sorting):
    """The kernel that finds the filters' boundaries and the drawn token bucket by bucket, and the
    one that sorts every row whole, against the plain sampler: same tokens.  (The bucketed kernel
    forms weights in 32-bit and sums them as integers; a row differs from the float64 statement only
    if a boundary falls within 1e-6 of a running sum, which these seeded rows do not.)"""
    g = torch.Generator().manual_seed(V)
    combos = [(0.8, 0, 1.0, 0.0), (1.0, 5, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05),
              (0.9, 40, 0.8, 0.01), (0.0, 0, 1.0, 0.0), (1.0, 1, 1.0, 0.0), (1.0, 0, 0.0, 0.0),
              (2.0, 3, 0.5, 0.2), (0.5, 1000, 0.95, 0.0), (1.0, 0, 0.3, 0.0)]
    rows = []
    for rep in range(4 if V < 100000 else 2):
        for c in combos:
            rows.append(c)
    R = len(rows)
    logits = (torch.randn(R, V, generator=g) * 3)
    logits[3, 10] = logits[3, 20] = logits[3].max() + 1          # equal logits: ascending id
    logits[4, :] = logits[4, :].round() + 0.0                    # many equal logits in every bucket (and no -0.0,
                                                                 # which the kernels order after +0.0, as a total order does)
    logits[5, 7] = float("-inf")
    logits[6, 9] = float("nan")                                  # counts as -inf
    logits[12, :] = (torch.randn(V, generator=g) * 0.05)         # a flat row: almost every token matters
    draws = torch.rand(R, generator=g, dtype=torch.float64)
    draws[1], draws[2] = 0.0, 1.0 - 1e-12
    k = K()
    scratch = torch.empty(k.sample_scratch_elems(R, V), dtype=torch.int64, device=dev())
    out = torch.full((R,), -7, dtype=torch.int32, device=dev())
    f = lambda i, dt: torch.tensor([r[i] for r in rows], dtype=dt, device=dev())
    k.sample(logits.to(dev()), scratch, f(0, torch.float32), f(1, torch.int32), f(2, torch.float32),
             f(3, torch.float32), draws.to(dev()), out, by_sorting=by_sorting)
    clean = torch.nan_to_num(logits, nan=float("-inf"))
    want = [P.sample_filtered(clean[i], *rows[i], float(draws[i])) for i in range(R)]
    assert out.tolist() == want


def test_sample_rows_the_buckets_cannot_take_fall_back_to_the_sort():
    """All logits equal (one bucket of 20,000 tokens, ordered by id alone), and a row whose maximum is
    +inf: the bucketed kernel hands them to the sorting kernel, and the tokens are the plain sampler's."""
    V = 20000
    g = torch.Generator().manual_seed(3)
    logits = torch.zeros(4, V)
    logits[1] = torch.randn(V, generator=g)
    logits[1, 5] = float("inf")
    logits[2] = torch.randn(V, generator=g).round() + 0.0        # a few values, thousands of tokens each
    logits[3] = torch.randn(V, generator=g)
    draws = torch.tensor([0.37, 0.5, 0.911, 0.2], dtype=torch.float64)
    k = K()
    scratch = torch.empty(k.sample_scratch_elems(4, V), dtype=torch.int64, device=dev())
    out = torch.full((4,), -7, dtype=torch.int32, device=dev())
    full = lambda v, dt: torch.full((4,), v, dtype=dt, device=dev())
    k.sample(logits.to(dev()), scratch, full(1.0, torch.float32), full(0, torch.int32), full(1.0, torch.float32),
             full(0.0, torch.float32), draws.to(dev()), out)
    assert out[0] == int(0.37 * V)                                # equal weights in id order
    assert out[1] == 5                                            # the one +inf takes all the weight
    want = [P.sample_filtered(logits[i], 1.0, 0, 1.0, 0.0, float(draws[i])) for i in (2, 3)]
    assert out[2:].tolist() == want


def test_sample_distribution_and_filters():
    """Many draws over a small row: frequencies follow softmax(logits/T) within the kept set."""
    V, R = 8, 4000
    base = torch.tensor([2.0, 1.0, 0.5, 0.0, -0.5, -1.0, -3.0, -8.0])
    logits = base.repeat(R, 1).to(dev())
    k = K()
    scratch = torch.empty(k.sample_scratch_elems(R, V), dtype=torch.int64, device=dev())
    out = torch.empty(R, dtype=torch.int32, device=dev())
    from rustinfer_b200.sampling.sampler import uniform_draw
    draws = torch.tensor([uniform_draw(11, p) for p in range(R)], dtype=torch.float64, device=dev())
    full = lambda v, dt: torch.full((R,), v, dtype=dt, device=dev())
    k.sample(logits, scratch, full(0.7, torch.float32), full(4, torch.int32), full(1.0, torch.float32),
             full(0.0, torch.float32), draws, out)
    counts = torch.bincount(out.cpu().long(), minlength=V).double()
    assert counts[4:].sum() == 0                                    # top-k 4
    p = torch.softmax(base[:4].double() / 0.7, dim=0)
    assert torch.allclose(counts[:4] / R, p, atol=0.03)


def test_kernels_refuse_what_they_cannot_do():
    from rustinfer_b200.ops.library import KernelError
    k = K()
    with pytest.raises(KernelError, match="CUDA tensors"):
        k.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))
    with pytest.raises(KernelError, match="multiples of 16"):
        from rustinfer_b200.ops import library
        library.attention_plain(24)
    with pytest.raises(KernelError):
        k.gemm_f32(torch.zeros(2, 3, device=dev()), torch.zeros(4, 5, device=dev()), torch.zeros(2, 4, device=dev()))
    with pytest.raises(KernelError):
        k.add_rmsnorm(torch.zeros(2, 8, device=dev()), None, torch.ones(9, device=dev()), 1e-5,
                      torch.zeros(2, 8, device=dev()))
