"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same op,
at sizes that the tiny models do not have: odd widths, head sizes in steps of 16,
groups of 1 to 8 query heads, pages of 1 to 64, row subsets and canary rows.
"""
import math

import pytest
import torch

import kernel_refs as R

pytestmark = pytest.mark.gpu

DEV = "cuda"
# 16-bit results carry one rounding of the result (2^-9 relative) on top of float arithmetic.
BF16_RTOL = 2.0 ** -7


def ops():
    from llm_infer_rust_b200.kernels import ops as o
    return o


def close(got, want, dtype, atol=1e-5, rtol=1e-5, bf16_atol=2e-3):
    if dtype == torch.bfloat16:
        atol, rtol = bf16_atol, BF16_RTOL
    torch.testing.assert_close(got.float(), want.float(), atol=atol, rtol=rtol)


def attention_atol(case):
    """Bound of the bfloat16 attention kernels' error: the tensor-core kernels round every probability
    to bfloat16 (2^-9 relative) as the operand of P.V, so an output is off by at most 2^-9 * sum p |v|
    <= 2^-9 * max |v|, and once more by its own rounding to bfloat16: 2^-8 * max |v| in all."""
    return 2.0 ** -8 * case["vmax"]


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,vocab", [(5, 7), (1000, 33), (4096, 11)])
def test_embedding(dtype, width, vocab):
    table = rnd(vocab, width, dtype=dtype)
    ids = torch.tensor([0, vocab - 1, 3, 3, 1], dtype=torch.int32, device=DEV)
    assert torch.equal(ops().embedding(ids, table, dtype), R.ref_embedding(ids, table, dtype))


def test_embedding_flags_a_token_outside_the_table():
    o = ops()
    table = rnd(10, 8)
    ids = torch.tensor([1, 10, -1], dtype=torch.int32, device=DEV)
    out = o.embedding(ids, table, torch.float32)
    assert torch.equal(out[0], table[1]) and out[1:].abs().sum() == 0
    with pytest.raises(o.KernelError, match="token id"):
        o.check_errors(torch.device(DEV))
    o.check_errors(torch.device(DEV))                         # the word is cleared


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,eps", [(1, 1, 1e-6), (7, 96, 1e-5), (33, 1000, 3e-6), (5, 5120, 1e-6)])
def test_rms_norm_and_residual_add(dtype, rows, width, eps):
    o = ops()
    x, res = rnd(rows, width, dtype=dtype), rnd(rows, width, dtype=dtype, seed=1)
    w = (1 + 0.1 * rnd(width, seed=2)).to(dtype)
    close(o.rms_norm(x, w, eps), R.ref_rms_norm(x, w, eps), dtype)
    want_y, want_r = R.ref_add_rms_norm(x, res, w, eps)
    r2 = res.clone()
    y = o.add_rms_norm(x.clone(), r2, w, eps)
    close(y, want_y, dtype)
    assert torch.equal(r2, want_r)
    # in place, a subset of rows, the residual left alone, float32 weight under a 16-bit engine
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    r3 = res.clone()
    y = o.add_rms_norm(x, r3, w.float(), eps, rows=idx, write_residual=False)
    close(y, want_y[idx.long()], dtype)
    assert torch.equal(r3, res)
    xin = x.clone()
    o.add_rms_norm(xin, res.clone(), w, eps, out=xin)
    close(xin, want_y, dtype)


def test_residual_rounding_fixture():
    # src/layers/ops.rs:455-479 of the reference: the UNROUNDED sum is normalised
    o = ops()
    x = torch.ones(1, 1024, dtype=torch.bfloat16, device=DEV)
    res = torch.tensor([0.00390625, 0.0078125], device=DEV).repeat(512)[None].to(torch.bfloat16)
    w = torch.ones(1024, dtype=torch.bfloat16, device=DEV)
    y = o.add_rms_norm(x, res, w, 1e-6)
    assert torch.equal(y, torch.ones_like(y))
    assert res[0, :2].tolist() == [1.0, 1.0078125]
    assert not torch.equal(o.rms_norm(res, w, 1e-6), torch.ones_like(y))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width", [(1, 1), (3, 224), (70, 1531)])
def test_silu_mul(dtype, tokens, width):
    gu = rnd(tokens, 2 * width, dtype=dtype, scale=3.0)
    close(ops().silu_mul(gu), R.ref_silu_mul(gu), dtype)


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 509, 96), (70, 130, 67), (64, 64, 16), (129, 3, 1000)])
def test_gemm_f32_is_true_32_bit_and_independent_of_the_batch(m, n, k):
    o = ops()
    a, w = rnd(m, k), rnd(n, k, seed=1)
    got = o.gemm_f32(a, w)
    want = (a.double() @ w.double().t())
    assert (got.double() - want).abs().max() <= 1e-6 * max(1.0, math.sqrt(k)) * want.abs().max().clamp_min(1.0)
    # a row's result is bit-identical whatever else is in the batch
    for r in {0, m // 2, m - 1}:
        assert torch.equal(o.gemm_f32(a[r:r + 1].contiguous(), w)[0], got[r])
    # and no reduced-precision mode: inputs that TF32 would round give the exact float product
    a2 = torch.full((1, 8), 1.0 + 2.0 ** -20, device=DEV)
    w2 = torch.full((1, 8), 1.0 + 2.0 ** -20, device=DEV)
    exact = 8 * (1.0 + 2.0 ** -20) ** 2
    assert abs(o.gemm_f32(a2, w2).item() - exact) < 1e-6 and abs(8.0 - exact) > 1e-5


@pytest.mark.parametrize("m,n,k", [(1, 509, 96), (7, 130, 64), (200, 96, 224)])
def test_linear_bf16_and_mixed(m, n, k):
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    close(o.linear(x, w), R.ref_linear(x, w), torch.bfloat16)
    got = o.linear(x, w, out_dtype=torch.float32)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, R.ref_linear(x, w, torch.float32), atol=1e-3, rtol=1e-3)
    # a weight kept in float32 under a 16-bit engine is multiplied in 32-bit
    close(o.linear(x, w.float()), R.ref_linear(x, w), torch.bfloat16)


def _bf(t):
    return t.to(torch.bfloat16).float()


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (5, 509, 96), (8, 1000, 1024), (13, 130, 3000), (16, 256, 2048),
                                   (3, 96, 12288), (16, 64, 12288), (2, 4000, 40),
                                   (8, 152001, 64),           # (a vocabulary: tiles of 256 weight rows)
                                   (5, 20000, 1088), (12, 19000, 2112)])   # (several waves of tiles: two CTAs an SM)
@pytest.mark.parametrize("with_norm", [False, True])
def test_few_row_product_plain(m, n, k, with_norm):
    """x . W^T for at most 16 rows, alone and with the residual add + norm as its prologue, in both output dtypes,
    with a gather of the rows; K long enough for a cluster to split it, N and K off every tile size."""
    o = ops()
    x, w = rnd(m + 3, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.05)
    rows = torch.tensor([(3 * i + 1) % (m + 3) for i in range(m)], dtype=torch.int32, device=DEV)
    res = rnd(m + 3, k, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(k, seed=3)).to(torch.bfloat16)
    for gather in (False, True):
        sel = rows.long() if gather else torch.arange(m, device=DEV)
        if with_norm:
            src = o.PendingNorm(x if gather else x[:m].contiguous(), res if gather else res[:m].contiguous(), nw, 1e-5,
                                rows=rows if gather else None, write_residual=not gather)
            s_sum = x[sel].float() + res[sel].float()
            # the kernel multiplies round(s * w) and applies the row's scale to the finished product
            xin, row_scale = _bf(s_sum * nw.float()), torch.rsqrt((s_sum * s_sum).mean(-1, keepdim=True) + 1e-5)
        else:
            src = x if gather else x[:m].contiguous()
            xin, row_scale = x[sel].float(), 1.0
        want = (xin @ w.float().t()) * row_scale
        for mode, dtype in ((o.EPI_PLAIN_F32, torch.float32), (o.EPI_PLAIN_BF16, torch.bfloat16)):
            got = o.skinny_linear(src, w, mode, x_rows=rows if (gather and not with_norm) else None)
            assert got.dtype == dtype and tuple(got.shape) == (m, n)
            scale = max(1.0, float(want.abs().max()))
            tol = 2e-3 * scale if dtype == torch.float32 else 2.0 ** -7 * scale
            assert (got.float() - want).abs().max() <= tol, (mode, gather)
        if with_norm and not gather:
            assert torch.equal(src.residual_out, s_sum.to(torch.bfloat16))         # the rounded sum is the new residual
            assert torch.equal(src.residual, res[:m])                              # the old one is left alone
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,inter,k", [(1, 64, 64), (7, 224, 96), (16, 3072, 1024), (4, 100, 4096),
                                       (6, 10100, 1088)])     # (several waves of tiles: two CTAs an SM)
def test_few_row_product_swiglu(m, inter, k):
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    got = o.skinny_linear(x, w, o.EPI_SWIGLU)
    gu = _bf(x.float() @ w.float().t())
    want = R.ref_silu_mul(gu.to(torch.bfloat16))
    assert tuple(got.shape) == (m, inter)
    assert (got.float() - want.float()).abs().max() <= 2.0 ** -6 * max(1.0, float(want.float().abs().max()))


@pytest.mark.parametrize("m,nh,nkv,d,k,with_norm", [(1, 4, 2, 64, 128, True), (9, 16, 8, 128, 1024, True),
                                                    (16, 3, 1, 64, 200, False), (5, 2, 2, 256, 512, True),
                                                    (3, 150, 2, 128, 1088, True)])       # (154 heads: several waves)
def test_few_row_product_qkv(m, nh, nkv, d, k, with_norm):
    """The fused QKV step against the separate kernels' references: projection, per-head norm, rotation, store."""
    o = ops()
    page, pages, max_pos, eps = 8, 6, 64, 1e-6
    n = (nh + 2 * nkv) * d
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    res = rnd(m, k, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(k, seed=3)).to(torch.bfloat16)
    qw, kw = (1 + 0.2 * rnd(d, seed=4)).to(torch.bfloat16), (1 + 0.2 * rnd(d, seed=5)).float()
    kw = kw.to(torch.bfloat16)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * \
        torch.exp(torch.arange(0, d, 2, dtype=torch.float64) * (-math.log(1e4) / d))[None]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    g = torch.Generator().manual_seed(6)
    positions = torch.randint(0, max_pos, (m,), generator=g).to(torch.int32).to(DEV)
    slots = (torch.randperm(page * pages, generator=g)[:m] + page).to(torch.int32)
    if m > 2:
        slots[2] = 0
    slots = slots.to(DEV)
    kc = torch.full((pages + 1, nkv, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
    vc = torch.full_like(kc, 7.0)
    q = torch.empty(m, nh * d, dtype=torch.bfloat16, device=DEV)
    if with_norm:
        src = o.PendingNorm(x, res, nw, 1e-5)
        s_sum = x.float() + res.float()
        xin, row_scale = _bf(s_sum * nw.float()), torch.rsqrt((s_sum * s_sum).mean(-1, keepdim=True) + 1e-5)
    else:
        src, xin, row_scale = x, x.float(), 1.0
    out = o.skinny_linear(src, w, o.EPI_QKV, qkv=dict(head_dim=d, num_heads=nh, num_kv_heads=nkv, q_out=q, k_cache=kc,
                                                      v_cache=vc, q_weight=qw, k_weight=kw, eps=eps, cos=cos, sin=sin,
                                                      rot_dim=d, positions=positions, slots=slots))
    assert out is q
    qkv = ((xin @ w.float().t()) * row_scale).to(torch.bfloat16)
    rq, rk, rv = R.ref_qkv_post(qkv, qw, kw, eps, cos, sin, d, positions, nh, nkv, d)
    want_k, want_v = torch.full_like(kc, 7.0), torch.full_like(vc, 7.0)
    R.ref_store_kv(want_k, want_v, rk, rv, slots)
    # the projection is rounded to bfloat16 on both sides, but from sums in another order: one more ulp
    for got, want in ((q.view(m, nh, d), rq), (kc, want_k), (vc, want_v)):
        torch.testing.assert_close(got.float(), want.float(), atol=2.0 ** -6 * max(1.0, float(want.float().abs().max())), rtol=2.0 ** -6)
    assert (kc[0] == 7.0).all() and (vc[0] == 7.0).all()
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,k0,hidden,n2,kind", [(1, 64, 128, 192, "plain"), (8, 2048, 1024, 6144, "swiglu"),
                                                 (5, 96, 200, 130, "plain"), (16, 3072, 1000, 256, "swiglu"),
                                                 (9, 512, 4096, 2 * 128 + 2 * 2 * 128, "qkv"), (3, 64, 72, 152001, "head")])
def test_few_row_products_hand_the_norm_between_them_from_one_to_the_next(m, k0, hidden, n2, kind):
    """A lazy product followed by a product behind the add + norm of its result: the first leaves the rounded sum
    and the rows' sums of squares (per tile of its columns), the second reads only its own columns.  Compared with
    the plain formula and with the same two products run one by one (where every CTA reads whole rows)."""
    o = ops()
    assert o.few_row_route == "single"
    a, w1 = rnd(m, k0, dtype=torch.bfloat16), rnd(hidden, k0, dtype=torch.bfloat16, seed=1, scale=0.05)
    res = rnd(m, hidden, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(hidden, seed=3)).to(torch.bfloat16)
    w2 = rnd(n2, hidden, dtype=torch.bfloat16, seed=4, scale=0.05)
    rows = torch.tensor([(2 * i + 1) % m for i in range(m)], dtype=torch.int32, device=DEV) if kind == "head" else None

    def second(src):
        if kind == "plain":
            return o.few_row_linear(src, w2, o.EPI_PLAIN_BF16)
        if kind == "head":
            return o.few_row_linear(src, w2, o.EPI_PLAIN_F32)
        if kind == "swiglu":
            return o.few_row_linear(src, w2, o.EPI_SWIGLU)
        q = torch.empty(m, 2 * 128, dtype=torch.bfloat16, device=DEV)
        return o.few_row_linear(src, w2, o.EPI_QKV, qkv=dict(head_dim=128, num_heads=2, num_kv_heads=2, q_out=q,
                                                             k_cache=None, v_cache=None, q_weight=None, k_weight=None,
                                                             eps=1e-6, cos=None, sin=None, rot_dim=0,
                                                             positions=torch.zeros(m, dtype=torch.int32, device=DEV),
                                                             slots=None)).clone()

    results = []
    for lazy in (True, False):
        y = o.few_row_linear(a, w1, o.EPI_PLAIN_BF16, lazy=lazy)
        assert (o._held is not None) == lazy
        src = o.PendingNorm(y, res, nw, 1e-5, rows=rows, write_residual=rows is None)
        out = second(src)
        assert o._held is None
        results.append((y.clone(), None if rows is not None else src.residual_out.clone(), out.clone()))
    (y1, sum1, out1), (y2, sum2, out2) = results
    assert torch.equal(y1, y2)
    y_want = a.float() @ w1.float().t()
    assert (y1.float() - y_want).abs().max() <= 2.0 ** -7 * max(1.0, float(y_want.abs().max()))
    s_sum = y1.float() + res.float()
    if rows is None:
        assert torch.equal(sum1, s_sum.to(torch.bfloat16)) and torch.equal(sum2, sum1)
    sel = rows.long() if rows is not None else torch.arange(m, device=DEV)
    xin = _bf(s_sum[sel] * nw.float())
    want = (xin @ w2.float().t()) * torch.rsqrt((s_sum[sel] * s_sum[sel]).mean(-1, keepdim=True) + 1e-5)
    if kind == "swiglu":
        want = R.ref_silu_mul(_bf(want).to(torch.bfloat16)).float()
    elif kind == "qkv":
        want = want[:, :2 * 128]
    scale = max(1.0, float(want.abs().max()))
    for got in (out1, out2):
        assert (got.float() - want).abs().max() <= 2.0 ** -6 * scale
    assert (out1.float() - out2.float()).abs().max() <= 2.0 ** -7 * scale
    o.check_errors(torch.device(DEV))


def test_a_held_product_is_launched_before_anything_else_runs():
    o = ops()
    a, w = rnd(4, 256, dtype=torch.bfloat16), rnd(384, 256, dtype=torch.bfloat16, seed=1, scale=0.05)
    y = o.few_row_linear(a, w, o.EPI_PLAIN_BF16, lazy=True)
    assert o._held is not None
    z = o.rms_norm(y, torch.ones(384, dtype=torch.bfloat16, device=DEV), 1e-6)       # any other wrapper launches it first
    assert o._held is None
    want = a.float() @ w.float().t()
    assert (y.float() - want).abs().max() <= 2.0 ** -7 * max(1.0, float(want.abs().max()))
    assert torch.isfinite(z.float()).all()
    y2 = o.few_row_linear(a, w, o.EPI_PLAIN_BF16, lazy=True)
    o.flush_chain()
    assert o._held is None and torch.equal(y, y2)


def test_few_row_product_refusals():
    o = ops()
    w = rnd(64, 64, dtype=torch.bfloat16)
    assert not o.skinny_ok(17, w, torch.bfloat16) and not o.skinny_ok(4, w.float(), torch.bfloat16)
    assert not o.skinny_ok(4, rnd(64, 60, dtype=torch.bfloat16), torch.bfloat16)          # K no multiple of 8
    assert not o.skinny_ok(4, w, torch.bfloat16, o.EPI_QKV, 48) and o.skinny_ok(4, w, torch.bfloat16, o.EPI_QKV, 64)
    assert not o.skinny_ok(16, rnd(8, 16384, dtype=torch.bfloat16), torch.bfloat16)       # too long for a cluster of 8
    with pytest.raises(o.KernelError, match="refuses"):
        o.skinny_linear(rnd(17, 64, dtype=torch.bfloat16), w)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 1024), (200, 304, 96), (1, 8, 8), (1000, 1000, 1000),
                                   (2048, 1024, 3072)])
def test_tcgen05_product(m, n, k):
    """The TMA-fed tcgen05 product (float sums in tensor memory) against a float reference: single and many
    tiles and k-blocks, more tiles than SMs (the persistent loop and both accumulators), tails in M, N and K."""
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16, scale=0.5), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    got = o.gemm_tc(x, w)
    want = x.float() @ w.float().t()
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (m, n)
    assert (got.float() - want).abs().max() <= 2.0 ** -8 * max(1.0, float(want.abs().max()))     # one bfloat16 rounding
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,inter,k", [(130, 256, 1024), (77, 100, 72), (2048, 3072, 1024), (300, 20000, 64)])
def test_tcgen05_product_with_swiglu_epilogue(m, inter, k):
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16, scale=0.5), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    got = o.gemm_tc(x, w, o.GEMM_SWIGLU)
    gu = (x.float() @ w.float().t()).to(torch.bfloat16)
    want = R.ref_silu_mul(gu).float()
    assert tuple(got.shape) == (m, inter)
    # gate and up are rounded to bfloat16 from sums in another order than the reference's: one ulp of each
    assert (got.float() - want).abs().max() <= 2.0 ** -6 * max(1.0, float(want.abs().max()))
    o.check_errors(torch.device(DEV))


def test_tcgen05_product_refusals():
    o = ops()
    assert not o.gemm_tc_ok(rnd(4, 60, dtype=torch.bfloat16), rnd(8, 60, dtype=torch.bfloat16))      # K no multiple of 8
    assert not o.gemm_tc_ok(rnd(4, 64), rnd(8, 64))                                                  # float32
    with pytest.raises(o.KernelError, match="tcgen05"):
        o.gemm_tc(rnd(4, 64), rnd(8, 64))


QKV_CASES = [  # nh, nkv, d, rot, eps, with_norm
    (4, 2, 16, 16, 1e-6, True), (6, 2, 32, 32, 1e-5, True), (5, 5, 48, 48, 3e-6, True),
    (8, 1, 128, 128, 1e-6, True), (3, 3, 80, 32, 1e-6, True), (2, 1, 64, 64, 1e-6, False),
    (1, 1, 256, 0, 1e-6, True),
    (3, 1, 40, 40, 1e-6, True), (2, 2, 72, 36, 1e-5, True), (4, 2, 42, 42, 1e-6, False),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,rot,eps,with_norm", QKV_CASES)
def test_qkv_post(dtype, nh, nkv, d, rot, eps, with_norm):
    o = ops()
    tokens, page, pages, max_pos = 19, 4, 9, 64
    qkv = rnd(tokens, (nh + 2 * nkv) * d, dtype=dtype)
    qw = (1 + 0.2 * rnd(d, seed=3)).to(dtype) if with_norm else None
    kw = (1 + 0.2 * rnd(d, seed=4)).to(dtype) if with_norm else None
    cos = sin = None
    if rot:
        ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * \
            torch.exp(torch.arange(0, rot, 2, dtype=torch.float64) * (-math.log(1e4) / rot))[None]
        cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    g = torch.Generator().manual_seed(5)
    positions = torch.randint(0, max_pos, (tokens,), generator=g).to(torch.int32).to(DEV)
    slots = (torch.randperm(page * pages, generator=g)[:tokens] + page).to(torch.int32)
    slots[3] = 0                                              # a padding row: writes nothing
    slots = slots.to(DEV)
    kc = torch.full((pages + 1, nkv, page, d), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((pages + 1, nkv, page, d), 7.0, dtype=dtype, device=DEV)
    q = torch.empty(tokens, nh * d, dtype=dtype, device=DEV)
    o.qkv_post(qkv, q, kc, vc, qw, kw, eps, cos, sin, rot, positions, slots, nh, nkv, d)
    rq, rk, rv = R.ref_qkv_post(qkv, qw, kw, eps, cos, sin, rot, positions, nh, nkv, d)
    close(q.view(tokens, nh, d), rq, dtype)
    want_k, want_v = torch.full_like(kc, 7.0), torch.full_like(vc, 7.0)
    R.ref_store_kv(want_k, want_v, rk, rv, slots)
    close(kc, want_k, dtype)
    assert torch.equal(vc, want_v)                            # values are copied as they are
    assert (kc[0] == 7.0).all() and (vc[0] == 7.0).all()      # the sink is never written
    # an execution that reads another entry's cache stores nothing
    kc2 = torch.zeros_like(kc)
    o.qkv_post(qkv, q, kc2, kc2.clone(), qw, kw, eps, cos, sin, rot, positions, None, nh, nkv, d)
    assert kc2.abs().sum() == 0
    o.check_errors(torch.device(DEV))


def test_qkv_post_flags_bad_positions_and_slots():
    o = ops()
    qkv = rnd(2, 3 * 16)
    cos = torch.ones(4, 8, device=DEV)
    kc = torch.zeros(3, 1, 2, 16, device=DEV)
    q = torch.empty(2, 16, device=DEV)
    pos = torch.tensor([0, 4], dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 3], dtype=torch.int32, device=DEV)
    o.qkv_post(qkv, q, kc, kc.clone(), None, None, 0.0, cos, torch.zeros_like(cos), 16, pos, slots, 1, 1, 16)
    with pytest.raises(o.KernelError, match="position"):
        o.check_errors(torch.device(DEV))
    slots = torch.tensor([2, 6], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    o.qkv_post(qkv, q, kc, kc.clone(), None, None, 0.0, cos, torch.zeros_like(cos), 16, pos, slots, 1, 1, 16)
    with pytest.raises(o.KernelError, match="slot"):
        o.check_errors(torch.device(DEV))


def paged_case(rows, nh, nkv, d, page, dtype, seed=0, poison=True):
    """rows: (prefix, q_len).  Returns everything the attention kernels take; pages are scattered and
    every slot that no live position owns holds a huge value (it must never be read into a result)."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-(p + n) // page) for p, n in rows]
    total_pages = sum(need) + 3
    perm = (torch.randperm(total_pages, generator=g) + 1).tolist()
    width = max(need) + 1
    table = torch.zeros(len(rows), width, dtype=torch.int32)
    kc = torch.full((total_pages + 1, nkv, page, d), 1e4 if poison else 0.0)
    vc = torch.full((total_pages + 1, nkv, page, d), -1e4 if poison else 0.0)
    at = 0
    for r, (p, n) in enumerate(rows):
        for lp in range(need[r]):
            table[r, lp] = perm[at]
            at += 1
        for pos in range(p + n):
            slot_page, off = table[r, pos // page], pos % page
            kc[slot_page, :, off] = torch.randn(nkv, d, generator=g)
            vc[slot_page, :, off] = torch.randn(nkv, d, generator=g)
    vmax = float(vc[vc > -1e3].abs().max()) if poison else float(vc.abs().max())
    tq = sum(n for _, n in rows)
    q = torch.randn(tq, nh * d, generator=g)
    cu = torch.tensor([0] + list(torch.tensor([n for _, n in rows]).cumsum(0)), dtype=torch.int32)
    kv_len = torch.tensor([p + n for p, n in rows], dtype=torch.int32)
    prefix = torch.tensor([p for p, _ in rows], dtype=torch.int32)
    dev = lambda t: t.to(DEV)
    return dict(q=dev(q.to(dtype)), kc=dev(kc.to(dtype)), vc=dev(vc.to(dtype)), table=dev(table), cu=dev(cu),
                kv_len=dev(kv_len), prefix=dev(prefix), vmax=vmax)


ATT_CASES = [  # nh, nkv, d, page, window
    (4, 2, 16, 4, None), (6, 2, 32, 16, None), (5, 5, 48, 8, 40), (8, 1, 128, 16, None),
    (16, 2, 64, 1, 7), (3, 1, 80, 64, None), (2, 2, 256, 16, 33), (32, 8, 128, 16, None),
    (8, 2, 128, 4, None), (16, 4, 128, 64, 100),
    # any even head size (rows of 80 and 144 bytes in bfloat16, and 84: no 16-byte alignment), and more than 32 query
    # heads per KV head (the all-sizes kernels serve them in chunks of 32)
    (4, 2, 40, 8, None), (6, 3, 72, 16, 20), (3, 1, 42, 4, None), (40, 1, 32, 16, None), (66, 2, 16, 8, 9),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,page,window", ATT_CASES)
def test_prefill_attention(dtype, nh, nkv, d, page, window):
    o = ops()
    rows = [(0, 1), (0, 37), (50, 2), (3, 64), (130, 5)]
    c = paged_case(rows, nh, nkv, d, page, dtype)
    scale = 0.7 / math.sqrt(d)
    out = torch.full_like(c["q"], 9.0)
    serve = torch.tensor([4, 1, 2, 3], dtype=torch.int32, device=DEV)       # row 0 is left out
    o.prefill_attention(c["q"], c["kc"], c["vc"], out, c["table"], c["cu"], c["kv_len"], c["prefix"], serve, 4,
                        64, nh, nkv, d, page, window, scale)
    want = R.ref_paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["kv_len"], c["prefix"], nh, nkv,
                                 d, page, window, scale, rows=[1, 2, 3, 4])
    close(out[1:], want[1:], dtype, atol=2e-5, rtol=1e-4, bf16_atol=attention_atol(c))
    assert (out[0] == 9.0).all()                              # a row that was not listed is not touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,page,window", ATT_CASES)
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_decode_attention(dtype, nh, nkv, d, page, window, splits):
    o = ops()
    rows = [(0, 1), (1, 1), (31, 1), (32, 1), (200, 1), (1023, 1), (0, 4)]
    c = paged_case(rows, nh, nkv, d, page, dtype, seed=1)
    scale = 1.0 / math.sqrt(d)
    out = torch.full_like(c["q"], 9.0)
    serve = torch.tensor([5, 0, 1, 2, 3, 4], dtype=torch.int32, device=DEV)
    need = o.decode_scratch_floats(6, nh, d, splits)
    scratch = torch.full((max(need, 1),), float("nan"), device=DEV)
    o.decode_attention(c["q"], c["kc"], c["vc"], out, scratch, c["table"], c["cu"], c["kv_len"], serve, 6, nh, nkv,
                       d, page, window, scale, splits)
    want = R.ref_paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["kv_len"], c["prefix"], nh, nkv,
                                 d, page, window, scale, rows=range(6))
    close(out[:6], want[:6], dtype, atol=2e-5, rtol=1e-4, bf16_atol=attention_atol(c))
    assert (out[6:] == 9.0).all()


@pytest.mark.parametrize("tiles_per_cta", [1, 2, 0])
@pytest.mark.parametrize("nh,nkv,window,page", [(16, 8, None, 16), (8, 1, None, 4), (4, 4, 200, 64), (32, 8, 77, 16),
                                                (6, 2, None, 128)])
def test_prefill_attention_over_many_key_blocks(nh, nkv, window, page, tiles_per_cta):
    """Head size 128, rows that span up to nine blocks of 128 keys, prefixes that are no multiple of a block, and
    one stretch of keys four times as large as the rest: the running maximum jumps there (the output accumulated
    so far is rescaled) and falls back behind it (the probabilities stay relative to the old maximum).  With one
    and with two tiles of 128 query vectors per CTA (rows whose second tile is short or empty among them)."""
    o = ops()
    d = 128
    rows = [(0, 700), (300, 333), (1000, 130), (5, 1), (0, 128)]
    c = paged_case(rows, nh, nkv, d, page, torch.bfloat16, seed=7)
    for r, (p, n) in enumerate(rows):
        for pos in range(512, min(640, p + n)):
            c["kc"][c["table"][r, pos // page], :, pos % page] *= 4.0
    scale = 1.5 / math.sqrt(d)
    out = torch.full_like(c["q"], 9.0)
    serve = torch.tensor([2, 0, 4, 1, 3], dtype=torch.int32, device=DEV)
    o.prefill_attention(c["q"], c["kc"], c["vc"], out, c["table"], c["cu"], c["kv_len"], c["prefix"], serve, 5,
                        700, nh, nkv, d, page, window, scale, tiles_per_cta=tiles_per_cta)
    o.check_errors(torch.device(DEV))
    want = R.ref_paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["kv_len"], c["prefix"], nh, nkv,
                                 d, page, window, scale)
    close(out, want, torch.bfloat16, bf16_atol=attention_atol(c))


def test_attention_finds_one_far_key_among_a_thousand():
    """One key far back scores high: whoever skips or misplaces it changes the result."""
    o = ops()
    nh, nkv, d, page = 4, 2, 64, 16
    for far in (0, 17, 511, 998):
        c = paged_case([(999, 1), (990, 10)], nh, nkv, d, page, torch.float32, seed=far, poison=False)
        for r in range(2):
            pg, off = c["table"][r, far // page], far % page
            c["kc"][pg, :, off] = 0.0
            c["kc"][pg, :, off, 0] = 50.0
            c["vc"][pg, :, off] = 3.0
        c["q"][:, 0::d] = 1.0                                  # dimension 0 of every head
        scale = 1.0
        out = torch.empty_like(c["q"])
        dec = torch.tensor([0], dtype=torch.int32, device=DEV)
        pf = torch.tensor([1], dtype=torch.int32, device=DEV)
        scratch = torch.empty(o.decode_scratch_floats(1, nh, d, 5), device=DEV)
        o.decode_attention(c["q"], c["kc"], c["vc"], out, scratch, c["table"], c["cu"], c["kv_len"], dec, 1, nh,
                           nkv, d, page, None, scale, 5)
        o.prefill_attention(c["q"], c["kc"], c["vc"], out, c["table"], c["cu"], c["kv_len"], c["prefix"], pf, 1, 10,
                            nh, nkv, d, page, None, scale)
        want = R.ref_paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["kv_len"], c["prefix"], nh,
                                     nkv, d, page, None, scale)
        torch.testing.assert_close(out, want, atol=2e-5, rtol=1e-4)
        # the far key takes all the weight, for the decoded token and for the portion's last query
        assert (out[0] - 3.0).abs().max() < 1e-3 and (out[-1] - 3.0).abs().max() < 1e-3


def test_window_edge_is_exact():
    """Keys at p - W (just outside) and p - W + 1 (just inside) carry the weight in turn."""
    o = ops()
    nh = nkv = 1
    d, page, W = 16, 4, 9
    for inside in (True, False):
        c = paged_case([(40, 1), (30, 11)], nh, nkv, d, page, torch.float32, seed=3, poison=False)
        c["q"][:] = 0.0
        c["q"][:, 0] = 1.0
        p = 40
        key = p - W + 1 if inside else p - W
        for r in range(2):
            c["kc"][c["table"][r, key // page], 0, key % page, 0] = 60.0
            c["vc"][c["table"][r, key // page], :, key % page] = 5.0
        out = torch.empty_like(c["q"])
        o.decode_attention(c["q"], c["kc"], c["vc"], out, None, c["table"], c["cu"], c["kv_len"],
                           torch.tensor([0], dtype=torch.int32, device=DEV), 1, nh, nkv, d, page, W, 1.0, 1)
        o.prefill_attention(c["q"], c["kc"], c["vc"], out, c["table"], c["cu"], c["kv_len"], c["prefix"],
                            torch.tensor([1], dtype=torch.int32, device=DEV), 1, 11, nh, nkv, d, page, W, 1.0)
        want = R.ref_paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["kv_len"], c["prefix"], nh,
                                     nkv, d, page, W, 1.0)
        torch.testing.assert_close(out, want, atol=2e-5, rtol=1e-4)
        hit = (out[0] - 5.0).abs().max() < 1e-3
        assert bool(hit) == inside
        assert (out[-1] - 5.0).abs().max() < 1e-3 if inside else True   # the portion's last query sits at p too


def test_refused_sizes_raise():
    o = ops()
    with pytest.raises(o.KernelError, match="head size"):
        o._attention(25)                                          # odd: the rotation pairs dimensions
    with pytest.raises(o.KernelError, match="head size"):
        o._attention(528)
    with pytest.raises(o.KernelError, match="CUDA tensors"):
        o.rms_norm(torch.ones(2, 4), torch.ones(4), 1e-6)
    with pytest.raises(o.KernelError, match="dtype"):
        o.rms_norm(torch.ones(2, 4, device=DEV, dtype=torch.float16), torch.ones(4, device=DEV), 1e-6)
    with pytest.raises(o.KernelError, match="non-contiguous"):
        o.silu_mul(torch.ones(4, 8, device=DEV).t())


def test_argmax_and_greedy_fixture():
    o = ops()
    logits = torch.tensor([[0.1, 2.0, 0.2], [3.0, 1.0, 0.5]], device=DEV)
    assert o.argmax(logits).tolist() == [1, 0]                # src/engine/sampling.rs:455-548
    big = rnd(5, 151936)
    big[2, 77] = big[2, 150000] = 50.0                        # ties: the lowest index
    assert o.argmax(big).tolist() == big.argmax(-1).tolist() and o.argmax(big)[2] == 77
    view = big[:, :1001]                                      # a strided view of a wider buffer
    assert o.argmax(view).tolist() == view.argmax(-1).tolist()


def _rows(temperature, top_k, top_p, seeds, counters):
    import numpy as np
    from llm_infer_rust_b200.sampling import SamplingParams, pack_rows
    p = SamplingParams(temperature, top_k, top_p)
    packed = pack_rows([(p, s, c) for s, c in zip(seeds, counters)])
    return torch.from_numpy(packed.view(np.uint8).reshape(len(seeds), 32)).to(DEV)


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, -1, 1.0), (0.8, -1, 1.0), (1.0, 2, 0.5), (1.3, 3, 1.0),
                                                     (0.7, -1, 0.6)])
def test_sampling_frequencies_follow_the_filtered_distribution(temperature, top_k, top_p):
    o = ops()
    probs = torch.tensor([0.4, 0.3, 0.2, 0.1, 0.0])
    logits = probs.clamp_min(1e-30).log()
    logits[4] = -float("inf")
    n = 20000
    batch = logits[None].repeat(n, 1).to(DEV)
    ids = o.sample(batch, _rows(temperature, top_k, top_p, [11] * n, range(n)))
    want = R.ref_filtered_probs(logits[None], temperature, top_k, top_p)[0]
    freq = torch.bincount(ids.long().cpu(), minlength=5).double() / n
    assert (freq - want).abs().max() < 0.015, (freq, want)
    assert freq[want == 0].sum() == 0
    if (top_k, top_p) == (2, 0.5):                            # src/engine/sampling.rs:736-757
        assert abs(freq[1] - 3 / 7) < 0.02 and freq[2:].sum() == 0


def test_sampling_depends_on_seed_and_counter_not_on_the_batch():
    o = ops()
    logits = rnd(6, 509, scale=2.0)
    seeds, counters = [5, 5, 6, 7, 8, 9], [0, 1, 0, 3, 3, 3]
    u = torch.empty(6, device=DEV)
    ids = o.sample(logits, _rows(0.8, -1, 1.0, seeds, counters), u)
    assert ((u >= 0) & (u < 1)).all() and len(set(u.tolist())) == 6
    for r in (0, 3, 5):
        alone = o.sample(logits[r:r + 1], _rows(0.8, -1, 1.0, seeds[r:r + 1], counters[r:r + 1]))
        assert alone.item() == ids[r].item()
    rev = o.sample(logits.flip(0).contiguous(), _rows(0.8, -1, 1.0, seeds[::-1], counters[::-1]))
    assert rev.flip(0).tolist() == ids.tolist()
    # the draw is the inverse CDF of the uniform number, in vocabulary order
    probs = torch.softmax(logits.double() / 0.8, -1).cumsum(-1).cpu()
    for r in range(6):
        want = int((probs[r] <= u[r].item() * probs[r, -1]).sum())
        assert abs(int(ids[r]) - want) <= 1
    # temperature 0 and top_p 0 are greedy
    assert o.sample(logits, _rows(0.0, -1, 1.0, seeds, counters)).tolist() == logits.argmax(-1).tolist()
    assert o.sample(logits, _rows(0.9, -1, 0.0, seeds, counters)).tolist() == logits.argmax(-1).tolist()
    assert o.sample(logits, _rows(0.9, 1, 1.0, seeds, counters)).tolist() == logits.argmax(-1).tolist()


def test_sampling_flags_rows_without_a_valid_token():
    o = ops()
    logits = torch.full((2, 16), float("nan"), device=DEV)
    logits[1, 3] = 1.0
    ids = o.sample(logits, _rows(1.0, -1, 1.0, [1, 1], [0, 0]))
    assert ids[0].item() == -1
    with pytest.raises(o.KernelError, match="sampling"):
        o.check_errors(torch.device(DEV))
