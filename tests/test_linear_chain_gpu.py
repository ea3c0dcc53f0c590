"""The persistent kernel that runs a chain of few-row products (csrc/linear_chain.cu) against plain float32
PyTorch: single products at 1 to 64 rows (with the norm prologue, a gather of the rows, every epilogue), and
chains shaped like a decoder layer, where a product's epilogue does the add of the norm that follows it.
Sizes are off every tile size; each case runs twice, since tickets and barrier words are kept between launches."""
import math

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


@pytest.fixture(autouse=True, params=["narrow tiles where they apply", "wide tiles only"])
def chain_route(request):
    """Every case runs with the default rule (tiles of 16 weight rows for small weights and up to 32 rows of x) and
    with wide tiles forced."""
    o = ops()
    before, o.few_row_route = (o.few_row_route, o.chain_narrow_bytes), "chain"
    if request.param == "wide tiles only":
        o.chain_narrow_bytes = 0
    yield
    o.flush_chain()
    o.few_row_route, o.chain_narrow_bytes = before
    o.check_errors(torch.device(DEV))


def _normed(x, res, nw, eps):
    """What the prologue feeds the product (round(s * w)), the row's scale, and the rounded sum."""
    s = x.float() + (res.float() if res is not None else 0.0)
    return _bf(s * nw.float()), torch.rsqrt((s * s).mean(-1, keepdim=True) + eps), s.to(torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (5, 509, 96), (8, 1000, 1024), (13, 130, 3000), (16, 256, 2048),
                                   (3, 96, 12288), (17, 200, 520), (32, 1024, 1024), (48, 77, 4096), (64, 300, 2056),
                                   (8, 152001, 64), (64, 4096, 1024)])
@pytest.mark.parametrize("prologue", ["none", "add_norm", "norm"])
def test_single_product(m, n, k, prologue):
    o = ops()
    x, w = rnd(m + 3, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.05)
    rows = torch.tensor([(3 * i + 1) % (m + 3) for i in range(m)], dtype=torch.int32, device=DEV)
    res = rnd(m + 3, k, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(k, seed=3)).to(torch.bfloat16)
    for gather in (False, True):
        sel = rows.long() if gather else torch.arange(m, device=DEV)
        xs = x if gather else x[:m].contiguous()
        rs = res if gather else res[:m].contiguous()
        for mode, dtype in ((o.EPI_PLAIN_F32, torch.float32), (o.EPI_PLAIN_BF16, torch.bfloat16)):
            for _ in range(2):
                if prologue == "none":
                    src, xin, row_scale = xs, x[sel].float(), 1.0
                else:
                    with_res = prologue == "add_norm"
                    src = o.PendingNorm(xs, rs if with_res else None, nw, 1e-5, rows=rows if gather else None,
                                        write_residual=not gather)
                    xin, row_scale, rounded = _normed(x[sel], res[sel] if with_res else None, nw, 1e-5)
                got = o.few_row_linear(src, w, mode, x_rows=rows if (gather and prologue == "none") else None, lazy=True)
                assert o.chain_pending() == 1
                o.flush_chain()
                want = (xin @ w.float().t()) * row_scale
                assert got.dtype == dtype and tuple(got.shape) == (m, n)
                scale = max(1.0, float(want.abs().max()))
                tol = 2e-3 * scale if dtype == torch.float32 else 2.0 ** -7 * scale
                assert (got.float() - want).abs().max() <= tol, (mode, gather)
                if prologue == "add_norm" and not gather:
                    assert torch.equal(src.residual_out, rounded)
                    assert torch.equal(src.residual, res[:m])
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,inter,k", [(1, 64, 64), (7, 224, 96), (16, 3072, 1024), (4, 100, 4096), (33, 1000, 520),
                                       (64, 3072, 1024)])
def test_swiglu(m, inter, k):
    o = ops()
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    for _ in range(2):
        got = o.few_row_linear(x, w, o.EPI_SWIGLU, lazy=True)
        o.flush_chain()
        gu = _bf(x.float() @ w.float().t())
        want = R.ref_silu_mul(gu.to(torch.bfloat16))
        assert tuple(got.shape) == (m, inter)
        assert (got.float() - want.float()).abs().max() <= 2.0 ** -6 * max(1.0, float(want.float().abs().max()))


def _rope_tables(max_pos, d, theta=1e4):
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * \
        torch.exp(torch.arange(0, d, 2, dtype=torch.float64) * (-math.log(theta) / d))[None]
    return ang.cos().float().to(DEV), ang.sin().float().to(DEV)


@pytest.mark.parametrize("m,nh,nkv,d,k,with_norm", [(1, 4, 2, 64, 128, True), (9, 16, 8, 128, 1024, True),
                                                    (16, 3, 1, 64, 200, False), (5, 6, 2, 32, 96, True),
                                                    (40, 5, 5, 16, 64, True), (64, 32, 8, 128, 1024, True)])
def test_qkv(m, nh, nkv, d, k, with_norm):
    """Projection, per-head norm, rotation and cache store in the product's epilogue, against the separate
    references; a padding row (slot 0) writes nothing, the sink page stays as it was."""
    o = ops()
    page, pages, max_pos, eps = 8, 10, 64, 1e-6
    n = (nh + 2 * nkv) * d
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    res = rnd(m, k, dtype=torch.bfloat16, seed=2)
    nw = (1 + 0.1 * rnd(k, seed=3)).to(torch.bfloat16)
    qw, kw = (1 + 0.2 * rnd(d, seed=4)).to(torch.bfloat16), (1 + 0.2 * rnd(d, seed=5)).to(torch.bfloat16)
    cos, sin = _rope_tables(max_pos, d)
    g = torch.Generator().manual_seed(6)
    positions = torch.randint(0, max_pos, (m,), generator=g).to(torch.int32).to(DEV)
    slots = (torch.randperm(page * pages, generator=g)[:m] + page).to(torch.int32)
    if m > 2:
        slots[2] = 0
    slots = slots.to(DEV)
    for _ in range(2):
        kc = torch.full((pages + 1, nkv, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
        vc = torch.full_like(kc, 7.0)
        q = torch.empty(m, nh * d, dtype=torch.bfloat16, device=DEV)
        if with_norm:
            src = o.PendingNorm(x, res, nw, 1e-5)
            xin, row_scale, _ = _normed(x, res, nw, 1e-5)
        else:
            src, xin, row_scale = x, x.float(), 1.0
        out = o.few_row_linear(src, w, o.EPI_QKV, qkv=dict(head_dim=d, num_heads=nh, num_kv_heads=nkv, q_out=q, k_cache=kc,
                                                           v_cache=vc, q_weight=qw, k_weight=kw, eps=eps, cos=cos, sin=sin,
                                                           rot_dim=d, positions=positions, slots=slots), lazy=True)
        assert out is q
        o.flush_chain()
        qkv = ((xin @ w.float().t()) * row_scale).to(torch.bfloat16)
        rq, rk, rv = R.ref_qkv_post(qkv, qw, kw, eps, cos, sin, d, positions, nh, nkv, d)
        want_k, want_v = torch.full_like(kc, 7.0), torch.full_like(vc, 7.0)
        R.ref_store_kv(want_k, want_v, rk, rv, slots)
        for got, want in ((q.view(m, nh, d), rq), (kc, want_k), (vc, want_v)):
            torch.testing.assert_close(got.float(), want.float(), atol=2.0 ** -6 * max(1.0, float(want.float().abs().max())),
                                       rtol=2.0 ** -6)
        assert (kc[0] == 7.0).all() and (vc[0] == 7.0).all()
    o.check_errors(torch.device(DEV))


@pytest.mark.parametrize("m,hidden,nh,nkv,d,inter", [(1, 96, 6, 2, 32, 224), (8, 1024, 16, 8, 128, 3072),
                                                     (13, 520, 3, 1, 64, 1000), (64, 1024, 16, 8, 128, 3072),
                                                     (24, 4096, 32, 8, 128, 1024)])
@pytest.mark.parametrize("layers", [1, 3])
def test_chain_like_decoder_layers(m, hidden, nh, nkv, d, inter, layers):
    """attention output -> O -> (add, norm) gate/up, SiLU -> down -> (add, norm) next QKV, ``layers`` times in one
    chain (more than six products: several launches), the last one ending in a float32 head with a gather.
    The add of each norm is done by the epilogue of the product before it; the sums must equal the unfused ones."""
    o = ops()
    eps, qk_eps, page, max_pos = 1e-6, 1e-5, 16, 128
    pages = (m + page - 1) // page + 1
    cos, sin = _rope_tables(max_pos, d, 1e6)
    g = torch.Generator().manual_seed(7)
    positions = torch.randint(0, max_pos, (m,), generator=g).to(torch.int32).to(DEV)
    slots = (torch.randperm(page * pages, generator=g)[:m] + page).to(torch.int32).to(DEV)
    W = []
    for layer in range(layers):
        W.append(dict(
            o=rnd(hidden, nh * d, dtype=torch.bfloat16, seed=10 * layer + 1, scale=0.05),
            gu=rnd(2 * inter, hidden, dtype=torch.bfloat16, seed=10 * layer + 2, scale=0.05),
            down=rnd(hidden, inter, dtype=torch.bfloat16, seed=10 * layer + 3, scale=0.05),
            qkv=rnd((nh + 2 * nkv) * d, hidden, dtype=torch.bfloat16, seed=10 * layer + 4, scale=0.05),
            n1=(1 + 0.1 * rnd(hidden, seed=10 * layer + 5)).to(torch.bfloat16),
            n2=(1 + 0.1 * rnd(hidden, seed=10 * layer + 6)).float(),
            qw=(1 + 0.2 * rnd(d, seed=10 * layer + 7)).to(torch.bfloat16),
            kw=(1 + 0.2 * rnd(d, seed=10 * layer + 8)).to(torch.bfloat16)))
    head = rnd(777, hidden, dtype=torch.bfloat16, seed=99, scale=0.05)
    nf = (1 + 0.1 * rnd(hidden, seed=98)).to(torch.bfloat16)
    want_rows = torch.tensor([(5 * i + 2) % m for i in range(min(m, 7))], dtype=torch.int32, device=DEV)
    attn = [rnd(m, nh * d, dtype=torch.bfloat16, seed=50 + layer) for layer in range(layers)]
    res0 = rnd(m, hidden, dtype=torch.bfloat16, seed=60)

    flush_between = not (layers == 3 and m == 13)      # (one case leaves all twelve products in one chain)
    for _ in range(2):
        # ---- the chain (attention itself is not part of it: its outputs are given)
        caches, qs = [], []
        residual = res0
        launches = o.launch_count()
        for layer, w in enumerate(W):
            y = o.few_row_linear(attn[layer], w["o"], o.EPI_PLAIN_BF16, lazy=True)
            pn = o.PendingNorm(y, residual, w["n1"], eps)
            residual = pn.residual_out
            act = o.few_row_linear(pn, w["gu"], o.EPI_SWIGLU, lazy=True)
            y = o.few_row_linear(act, w["down"], o.EPI_PLAIN_BF16, lazy=True)
            if layer + 1 < layers:
                pn = o.PendingNorm(y, residual, w["n2"], eps)
                residual = pn.residual_out
                kc = torch.zeros((pages + 1, nkv, page, d), dtype=torch.bfloat16, device=DEV)
                vc = torch.zeros_like(kc)
                q = torch.empty(m, nh * d, dtype=torch.bfloat16, device=DEV)
                o.few_row_linear(pn, w["qkv"], o.EPI_QKV, qkv=dict(
                    head_dim=d, num_heads=nh, num_kv_heads=nkv, q_out=q, k_cache=kc, v_cache=vc, q_weight=w["qw"],
                    k_weight=w["kw"], eps=qk_eps, cos=cos, sin=sin, rot_dim=d, positions=positions, slots=slots), lazy=True)
                caches.append((kc, vc))
                qs.append(q)
                if flush_between:
                    o.flush_chain()      # (attention would run here)
        pn = o.PendingNorm(y, residual, nf, eps, rows=want_rows, write_residual=False)
        logits = o.few_row_linear(pn, head, o.EPI_PLAIN_F32, lazy=True)
        assert o.chain_pending() > 0
        o.flush_chain()
        assert o.chain_pending() == 0
        # one launch between two attentions; without them, six products a launch
        assert o.launch_count() - launches == (layers if flush_between else -(-4 * layers // 6))
        last_residual = residual

        # ---- the same with plain tensors, product by product
        r = res0
        for layer, w in enumerate(W):
            y_ref = _bf(attn[layer].float() @ w["o"].float().t())
            xin, sc, r = _normed(y_ref, r, w["n1"], eps)
            gu = _bf((xin @ w["gu"].float().t()) * sc)
            act_ref = R.ref_silu_mul(gu.to(torch.bfloat16))
            y_ref = _bf(act_ref.float() @ w["down"].float().t())
            if layer + 1 < layers:
                xin, sc, r = _normed(y_ref, r, w["n2"], eps)
                qkv = ((xin @ w["qkv"].float().t()) * sc).to(torch.bfloat16)
                rq, rk, rv = R.ref_qkv_post(qkv, w["qw"], w["kw"], qk_eps, cos, sin, d, positions, nh, nkv, d)
                want_k = torch.zeros((pages + 1, nkv, page, d), dtype=torch.bfloat16, device=DEV)
                want_v = torch.zeros_like(want_k)
                R.ref_store_kv(want_k, want_v, rk, rv, slots)
                kc, vc = caches[layer]
                for got, want in ((qs[layer].view(m, nh, d), rq), (kc, want_k), (vc, want_v)):
                    tol = 2.0 ** -5 * max(1.0, float(want.float().abs().max()))
                    assert (got.float() - want.float()).abs().max() <= tol, layer
        sel = want_rows.long()
        xin, sc, _ = _normed(y_ref[sel], r[sel], nf, eps)
        want_logits = (xin @ head.float().t()) * sc
        tol = 2.0 ** -5 * max(1.0, float(want_logits.abs().max()))
        assert (logits - want_logits).abs().max() <= tol
        assert (last_residual.float() - r.float()).abs().max() <= 2.0 ** -6 * max(1.0, float(r.float().abs().max()))
    o.check_errors(torch.device(DEV))


def test_refusals_and_routes():
    o = ops()
    w = rnd(64, 64, dtype=torch.bfloat16)
    assert o.chain_takes(64, w, torch.bfloat16) and not o.chain_takes(65, w, torch.bfloat16)
    assert not o.chain_takes(4, w.float(), torch.bfloat16) and not o.chain_takes(4, w, torch.float32)
    assert not o.chain_takes(4, rnd(64, 60, dtype=torch.bfloat16), torch.bfloat16)          # K no multiple of 8
    assert o.chain_takes(4, w, torch.bfloat16, o.EPI_QKV, 32) and not o.chain_takes(4, w, torch.bfloat16, o.EPI_QKV, 48)
    x = rnd(4, 64, dtype=torch.bfloat16)
    want = R.ref_linear(x, w)
    for route in ("chain", "single", "library"):
        o.few_row_route = route
        got = o.linear(x, w)
        o.flush_chain()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2.0 ** -7)
    o.few_row_route = "chain"
    with pytest.raises(o.KernelError):
        o.few_row_linear(rnd(65, 64, dtype=torch.bfloat16), w)          # neither kernel takes 65 rows
