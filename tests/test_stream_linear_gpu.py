"""The few-row product for large weights in which every thread copies its own share of the weights
(csrc/stream_linear.cu) against the plain formulas: every shape of its launch (rows and warps of a CTA), sizes off
every tile, the norm before it and the norm after it, and its place in the routing of few-row products."""
import pytest
import torch

import kernel_refs as R

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from llm_infer_rust_b200.kernels import ops as o
    return o


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _bf(t):
    return t.to(torch.bfloat16).float()


# (groups of 16 weight rows a tile and warps that split K; 0, 0: the launcher's choice)
LAUNCHES = [(0, 0), (1, 24), (1, 3), (1, 8), (2, 8), (2, 1), (2, 12)]


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (5, 509, 96), (8, 1000, 1024), (13, 130, 1504), (16, 256, 2048),
                                   (3, 96, 6016), (7, 4099, 4096), (8, 20000, 1088)])
@pytest.mark.parametrize("norm", ["none", "add", "plain"])
def test_stream_product_plain(m, n, k, norm):
    """x . W^T alone, behind a residual add + norm and behind a norm without an add, in both output dtypes, with a
    gather of the rows, for every shape of the launch."""
    o = ops()
    x, w = rnd(m + 3, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.05)
    rows = torch.tensor([(3 * i + 1) % (m + 3) for i in range(m)], dtype=torch.int32, device=DEV)
    res = rnd(m + 3, k, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(k, seed=3)).to(torch.bfloat16)
    for gather in (False, True):
        sel = rows.long() if gather else torch.arange(m, device=DEV)
        xs, rs = (x, res) if gather else (x[:m].contiguous(), res[:m].contiguous())
        if norm == "none":
            xin, row_scale, s_sum = x[sel].float(), 1.0, None
        else:
            s_sum = x[sel].float() + (res[sel].float() if norm == "add" else 0.0)
            # the kernel multiplies round(s * w) and applies the row's scale to the finished product
            xin, row_scale = _bf(s_sum * nw.float()), torch.rsqrt((s_sum * s_sum).mean(-1, keepdim=True) + 1e-5)
        want = (xin @ w.float().t()) * row_scale
        scale = max(1.0, float(want.abs().max()))
        for rw, ks in LAUNCHES:
            for mode, dtype in ((o.EPI_PLAIN_F32, torch.float32), (o.EPI_PLAIN_BF16, torch.bfloat16)):
                if norm == "none":
                    src = xs
                else:
                    src = o.PendingNorm(xs, rs if norm == "add" else None, nw if rw != 2 else nw.float(), 1e-5,
                                        rows=rows if gather else None, write_residual=not gather)
                # without a norm also with the rows of x fetched beside the weights (as rows too long for shared memory are)
                for xd in ((0, 1) if norm == "none" else (-1,)):
                    # (every other shape also as clusters of two CTAs that stage half of the rows of x each)
                    got = o.stream_linear(src, w, mode, x_rows=rows if (gather and norm == "none") else None, rw=rw, ks=ks, xd=xd,
                                          pair=(rw + ks) % 2)
                    assert got.dtype == dtype and tuple(got.shape) == (m, n)
                    tol = 2e-3 * scale if dtype == torch.float32 else 2.0 ** -7 * scale
                    assert (got.float() - want).abs().max() <= tol, (mode, gather, rw, ks, xd)
                if norm == "add" and not gather:
                    assert torch.equal(src.residual_out, s_sum.to(torch.bfloat16))     # the rounded sum is the new residual
                    assert torch.equal(src.residual, res[:m])                          # the old one is left alone
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,n,k", [(3, 96, 12288), (16, 4100, 12288), (8, 40, 25600)])
def test_stream_product_with_rows_too_long_for_shared_memory(m, n, k):
    """Rows of x that do not fit shared memory (and have no norm before them) come with the weights' copies; the
    product that follows behind a norm gets its beginning all the same."""
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.05)
    assert not o.stream_ok(m, w, torch.bfloat16, norm=True) and o.stream_ok(m, w, torch.bfloat16, norm=False)
    want = x.float() @ w.float().t()
    scale = max(1.0, float(want.abs().max()))
    for rw, ks in [(0, 0), (1, 24), (1, 5), (2, 12)]:
        got = o.stream_linear(x, w, o.EPI_PLAIN_F32, rw=rw, ks=ks)
        assert (got - want).abs().max() <= 2e-3 * scale, (rw, ks)
    res = rnd(m, n, dtype=torch.bfloat16, seed=2)
    cols = o.stream_tile_cols(o.EPI_PLAIN_BF16, m, n, k, False)
    tiles = -(-n // cols)
    sum_out, stats = torch.empty_like(res), torch.zeros(tiles, 16, device=DEV)
    got = o.stream_linear(x, w, o.EPI_PLAIN_BF16, norm_after=(res, sum_out, stats))
    assert (got.float() - want).abs().max() <= 2.0 ** -7 * scale
    s_sum = got.float() + res.float()
    assert torch.equal(sum_out, s_sum.to(torch.bfloat16))
    torch.testing.assert_close(stats[:, :m].sum(0), (s_sum * s_sum).sum(-1), rtol=1e-4, atol=1e-3)
    with pytest.raises(o.KernelError):
        o.stream_linear(o.PendingNorm(x, None, torch.ones(k, dtype=torch.bfloat16, device=DEV), 1e-6), w)
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,inter,k", [(1, 16, 32), (7, 224, 96), (16, 3072, 1024), (4, 100, 4096), (6, 10100, 1088)])
@pytest.mark.parametrize("with_norm", [False, True])
def test_stream_product_swiglu(m, inter, k, with_norm):
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    res, nw = rnd(m, k, dtype=torch.bfloat16, seed=2), (1 + 0.1 * rnd(k, seed=3)).to(torch.bfloat16)
    if with_norm:
        s_sum = x.float() + res.float()
        gu = (_bf(s_sum * nw.float()) @ w.float().t()) * torch.rsqrt((s_sum * s_sum).mean(-1, keepdim=True) + 1e-6)
    else:
        gu = x.float() @ w.float().t()
    want = R.ref_silu_mul(_bf(gu).to(torch.bfloat16))
    for rw, ks in [(0, 0), (2, 8), (2, 3), (2, 24), (2, 1), (1, 8), (1, 5), (1, 24)]:
        src = o.PendingNorm(x, res, nw, 1e-6) if with_norm else x
        got = o.stream_linear(src, w, o.EPI_SWIGLU, rw=rw, ks=ks, xd=-1 if with_norm else ks % 2, pair=(ks // 2) % 2)
        assert tuple(got.shape) == (m, inter)
        assert (got.float() - want.float()).abs().max() <= 2.0 ** -6 * max(1.0, float(want.float().abs().max())), (rw, ks)
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,k0,hidden,n2,kind", [(1, 64, 128, 192, "plain"), (8, 2048, 1024, 6144, "swiglu"),
                                                 (5, 96, 200, 130, "plain"), (16, 3072, 1000, 256, "swiglu"),
                                                 (9, 512, 4096, 2 * 128 + 2 * 2 * 128, "qkv"), (3, 64, 72, 1000, "head")])
@pytest.mark.parametrize("first,second", [("stream", "ring"), ("ring", "stream"), ("stream", "stream")])
def test_routed_products_hand_the_norm_from_one_to_the_next(monkeypatch, m, k0, hidden, n2, kind, first, second):
    """A lazy product on one kernel followed by a product on the other behind the add + norm of its result, through
    the routing of few-row products: a streaming product begins the norm for a ring product that follows
    it (rounded sum and the rows' sums of squares per CTA), and gets nothing handed when it is the second (it adds up
    the rows itself).  Compared with the plain formula and with the same two products run one by one."""
    o = ops()
    if kind == "qkv" and second == "stream":
        pytest.skip("the QKV epilogue is the ring kernel's")
    a, w1 = rnd(m, k0, dtype=torch.bfloat16), rnd(hidden, k0, dtype=torch.bfloat16, seed=1, scale=0.05)
    res = rnd(m, hidden, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(hidden, seed=3)).to(torch.bfloat16)
    w2 = rnd(n2, hidden, dtype=torch.bfloat16, seed=4, scale=0.05)
    if (first == "stream" and k0 % 32) or (second == "stream" and hidden % 32):
        pytest.skip("the streaming kernel takes K in multiples of 32")
    # a rule of sizes routes: make it say what this case wants
    big = {id(w): name == "stream" for w, name in ((w1, first), (w2, second))}
    monkeypatch.setattr(o, "stream_takes",
                        lambda rows, weight, dtype, mode=o.EPI_PLAIN_BF16, norm=True: big.get(id(weight), False))

    def second_product(src):
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

    before = o.launch_count()
    results = []
    for lazy in (True, False):
        y = o.few_row_linear(a, w1, o.EPI_PLAIN_BF16, lazy=lazy)
        assert (o._held is not None) == lazy and (not lazy or o._held.stream == (first == "stream"))
        src = o.PendingNorm(y, res, nw, 1e-5)
        out = second_product(src)
        assert o._held is None
        results.append((y.clone(), src.residual_out.clone(), out.clone()))
    assert o.launch_count() - before == 4
    (y1, sum1, out1), (y2, sum2, out2) = results
    assert torch.equal(y1, y2)
    y_want = a.float() @ w1.float().t()
    assert (y1.float() - y_want).abs().max() <= 2.0 ** -7 * max(1.0, float(y_want.abs().max()))
    s_sum = y1.float() + res.float()
    assert torch.equal(sum1, s_sum.to(torch.bfloat16)) and torch.equal(sum2, sum1)
    want = (_bf(s_sum * nw.float()) @ w2.float().t()) * torch.rsqrt((s_sum * s_sum).mean(-1, keepdim=True) + 1e-5)
    if kind == "swiglu":
        want = R.ref_silu_mul(_bf(want).to(torch.bfloat16)).float()
    elif kind == "qkv":
        want = want[:, :2 * 128]
    scale = max(1.0, float(want.abs().max()))
    for got in (out1, out2):
        assert (got.float() - want).abs().max() <= 2.0 ** -6 * scale
    assert (out1.float() - out2.float()).abs().max() <= 2.0 ** -7 * scale
    o.check_errors(torch.device(DEV))


def test_stream_product_rule_and_refusals():
    o = ops()
    w = rnd(64, 64, dtype=torch.bfloat16)
    assert o.stream_ok(16, w, torch.bfloat16) and o.stream_ok(1, w, torch.bfloat16, o.EPI_SWIGLU)
    assert not o.stream_ok(17, w, torch.bfloat16) and not o.stream_ok(4, w.float(), torch.bfloat16)
    assert not o.stream_ok(4, w, torch.float32) and not o.stream_ok(4, w, torch.bfloat16, o.EPI_QKV)
    assert not o.stream_ok(4, rnd(64, 72, dtype=torch.bfloat16), torch.bfloat16)               # K no multiple of 32
    assert not o.stream_ok(4, rnd(63, 64, dtype=torch.bfloat16), torch.bfloat16, o.EPI_SWIGLU)
    assert not o.stream_takes(4, w, torch.bfloat16)                                            # far below the rule's size
    x = rnd(4, 64, dtype=torch.bfloat16)
    with pytest.raises(o.KernelError):
        o.stream_linear(rnd(17, 64, dtype=torch.bfloat16), w)
    with pytest.raises(o.KernelError):
        o.stream_linear(x, w, rw=3, ks=4)
    with pytest.raises(o.KernelError):
        o.stream_linear(x, w, rw=1, ks=25)
    assert o.stream_ok(8, rnd(16, 6016, dtype=torch.bfloat16), torch.bfloat16)
    assert not o.stream_ok(9, rnd(16, 6016, dtype=torch.bfloat16), torch.bfloat16)            # 16 rows of x do not fit
    assert not o.stream_ok(8, rnd(16, 12288, dtype=torch.bfloat16), torch.bfloat16)
    assert o.stream_ok(16, rnd(16, 12288, dtype=torch.bfloat16), torch.bfloat16, norm=False)  # (they come with the weights)
    o.check_errors(torch.device(DEV))
