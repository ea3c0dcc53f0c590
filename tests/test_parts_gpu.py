"""Each part alone, built from a ``PartSpec`` with sizes of its own, against the
plain implementation's function for the same part."""
import math

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def env(dtype=torch.float32, pes=None):
    from llm_infer_rust_b200.parts import BuildEnv
    return BuildEnv(dtype, DEV, pes or {})


def spec(kind, **params):
    from llm_infer_rust_b200 import PartSpec
    return PartSpec(kind, params)


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g, dtype=torch.float64) * scale


def bound(part, **tensors):
    for name, t in tensors.items():
        part.bind(name, t.to(part.env.dtype).to(DEV))
    assert not part.missing_params()
    return part


def test_norm_part():
    from llm_infer_rust_b200.parts import build_part
    w, x, r = 1 + 0.1 * rnd(200), rnd(9, 200), rnd(9, 200, seed=1)
    part = bound(build_part("norm", spec("rms_norm", width=200, eps=2e-5), env()), weight=w)
    got = part.forward(x.float().to(DEV)).double().cpu()
    assert (got - P.plain_rms_norm(x.float().double(), w.float().double(), 2e-5)).abs().max() < 1e-5
    res = r.float().to(DEV)
    got = part.forward_add(x.float().to(DEV), res).double().cpu()
    want, new_r = P.plain_add_rms_norm(x.float().double(), r.float().double(), w.float().double(), 2e-5)
    assert (got - want).abs().max() < 1e-5 and (res.double().cpu() - new_r).abs().max() < 1e-6
    with pytest.raises(ValueError, match="shape"):
        part.bind("weight", torch.ones(3))
    with pytest.raises(KeyError):
        part.bind("bias", torch.ones(200))


def test_rope_tables_follow_the_formula():
    from llm_infer_rust_b200.parts import build_part
    rope = build_part("position_encoding", spec("half_split_rope", rotary_dim=48, theta=5e4, max_positions=300), env())
    phi = P.plain_rope_angles(torch.arange(300), 48, 5e4, torch.float64)
    assert tuple(rope.cos.shape) == (300, 24) and rope.cos.dtype == torch.float32
    assert (rope.cos.double().cpu() - phi.cos()).abs().max() < 1e-7
    assert (rope.sin.double().cpu() - phi.sin()).abs().max() < 1e-7
    with pytest.raises(ValueError):
        build_part("position_encoding", spec("half_split_rope", rotary_dim=5, theta=1e4, max_positions=8), env())


def test_feed_forward_part():
    from llm_infer_rust_b200.parts import build_part
    h, i = 72, 100
    wg, wu, wd, x = rnd(i, h, scale=0.2), rnd(i, h, seed=1, scale=0.2), rnd(h, i, seed=2, scale=0.2), rnd(13, h)
    part = bound(build_part("feed_forward", spec("swiglu", hidden_size=h, intermediate_size=i), env()),
                 gate_up_proj=torch.cat([wg, wu]), down_proj=wd)
    got = part.forward(x.float().to(DEV)).double().cpu()
    want = P.plain_swiglu(x.float().double(), wg.float().double(), wu.float().double(), wd.float().double())
    assert (got - want).abs().max() < 1e-5 * max(1.0, want.abs().max())


def test_embedding_and_head_parts():
    from llm_infer_rust_b200.parts import build_part
    table = rnd(37, 24)
    emb = bound(build_part("embedding", spec("token_embedding", vocab_size=37, hidden_size=24), env()), weight=table)
    ids = torch.tensor([0, 36, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table.float()[ids.long().cpu()])
    head = bound(build_part("head", spec("linear_head", vocab_size=37, hidden_size=24, tied=False), env(torch.bfloat16)),
                 weight=table)
    x = rnd(3, 24).to(torch.bfloat16)
    got = head.forward(x.to(DEV))
    assert got.dtype == torch.float32                          # logits leave in float
    want = P.plain_lm_head(x.double(), table.to(torch.bfloat16).double())
    assert (got.double().cpu() - want).abs().max() < 1e-3 * max(1.0, want.abs().max())


def step_context(rt, mgr, rows, device=DEV):
    """rows: (request id, number of new tokens).  Pages are grown here; the caller advances."""
    from llm_infer_rust_b200.engine import context_from_layout
    req = rt.BatchRequest()
    req.ids = [r for r, _ in rows]
    req.counts = [n for _, n in rows]
    req.tokens = [0] * sum(n for _, n in rows)
    req.want_counts = [0] * len(rows)
    req.want_index = []
    for r, n in rows:
        assert mgr.grow(r, mgr.length(r) + n)
    plan = rt.plan_batch(mgr, req)
    host = torch.empty(plan.total_ints, dtype=torch.int32)
    layout = rt.build_batch(mgr, req, host.numpy())
    dev = host.to(device)
    scratch = {}

    def get_scratch(n):
        if "t" not in scratch or scratch["t"].numel() < n:
            scratch["t"] = torch.empty(n, dtype=torch.float32, device=device)
        return scratch["t"]

    pages = [mgr.group(g).page_size for g in range(mgr.num_groups())]
    return context_from_layout(layout, dev, host, pages, device, torch.float32, layout.max_kv_len, get_scratch)


@pytest.mark.parametrize("nh,nkv,d,window,qk_eps", [(6, 3, 32, None, 1e-5), (4, 1, 16, 11, 1e-6), (2, 2, 48, None, None)])
def test_attention_part_over_its_cache(nh, nkv, d, window, qk_eps):
    """The mixer alone: portions and decoded tokens of two requests against whole-sequence attention."""
    from llm_infer_rust_b200.cache import LayerCache
    from llm_infer_rust_b200.kernels.build import load_host_runtime
    from llm_infer_rust_b200.parts import build_part
    rt = load_host_runtime()
    hidden, page, theta, max_pos = 40, 4, 1e4, 128
    rope = build_part("position_encoding", spec("half_split_rope", rotary_dim=d, theta=theta, max_positions=max_pos), env())
    mixer = build_part("mixer", spec("gqa_attention", hidden_size=hidden, num_heads=nh, num_kv_heads=nkv, head_dim=d,
                                     qk_norm_eps=qk_eps, window=window, softmax_scale=1.0 / math.sqrt(d),
                                     position_encoding="rope"), env(pes={"rope": rope}))
    wq, wk, wv = rnd(nh * d, hidden, scale=0.3), rnd(nkv * d, hidden, seed=1, scale=0.3), rnd(nkv * d, hidden, seed=2, scale=0.3)
    wo = rnd(hidden, nh * d, seed=3, scale=0.3)
    params = dict(qkv_proj=torch.cat([wq, wk, wv]), o_proj=wo)
    qn = kn = None
    if qk_eps is not None:
        qn, kn = 1 + 0.2 * rnd(d, seed=4), 1 + 0.2 * rnd(d, seed=5)
        params.update(q_norm=qn, k_norm=kn)
    bound(mixer, **params)
    assert mixer.cache_spec().window == window and mixer.state_spec() is None

    xs = {1: rnd(50, hidden, seed=6), 2: rnd(23, hidden, seed=7)}

    def plain(x):
        f = lambda t: t.float().double()
        q, k, v = P.plain_qkv(f(x), f(wq), f(wk), f(wv), nh, nkv, d)
        if qk_eps is not None:
            q, k = P.plain_qk_norm(q, k, f(qn), f(kn), qk_eps)
        pos = torch.arange(x.shape[0])
        q, k = P.plain_rope(q, pos, theta), P.plain_rope(k, pos, theta)
        return P.plain_attention(q, k, v, window) @ f(wo).T

    want = {r: plain(x) for r, x in xs.items()}
    mgr = rt.CacheManager([rt.GroupSpec(page, 30, window or 0)], 4)
    cache = LayerCache(group=0, k=torch.zeros(31, nkv, page, d, device=DEV), v=torch.zeros(31, nkv, page, d, device=DEV))
    mgr.open(1)
    mgr.open(2)
    got = {1: [], 2: []}
    fed = {1: 0, 2: 0}
    for rows in ([(1, 30)], [(1, 1), (2, 2)], [(1, 7), (2, 1)], [(2, 19), (1, 1)], [(1, 11), (2, 1)]):
        ctx = step_context(rt, mgr, rows)
        x = torch.cat([xs[r][fed[r]: fed[r] + n] for r, n in rows]).float().to(DEV)
        y = mixer.forward(x, ctx, cache).double().cpu()
        at = 0
        for r, n in rows:
            got[r].append(y[at: at + n])
            at += n
            fed[r] += n
            mgr.advance(r, fed[r])
    for r in xs:
        err = (torch.cat(got[r]) - want[r]).abs().max()
        assert err < 1e-5 * max(1.0, want[r].abs().max()), (r, err)
    assert mgr.check() == ""


def test_block_arrangement_defers_the_second_add():
    from llm_infer_rust_b200 import LayerSpec
    from llm_infer_rust_b200.parts import Part, build_part, register_part

    class Doubler(Part):
        category = "mixer"

        def cache_spec(self):
            return None

        def state_spec(self):
            return None

        def forward(self, x, ctx, cache):
            return 2.0 * x

    class Negate(Part):
        category = "feed_forward"

        def forward(self, x):
            return -x

    register_part("mixer", "test_doubler", Doubler, replace=True)
    register_part("feed_forward", "test_negate", Negate, replace=True)
    layer = LayerSpec.pre_norm(spec("pre_norm_deferred_add"), spec("test_doubler"), spec("test_negate"),
                      spec("rms_norm", width=6, eps=1e-6))
    block = build_part("block", layer, env())
    w1, w2 = 1 + 0.1 * rnd(6), 1 + 0.1 * rnd(6, seed=1)
    bound(block.input_norm, weight=w1)
    bound(block.post_mixer_norm, weight=w2)
    assert sorted(block.children()) == ["feed_forward", "input_norm", "mixer", "post_mixer_norm"]
    h = rnd(4, 6).float()
    f = lambda t: t.float().double()
    # first block: residual = h
    out, res = block.forward(h.to(DEV).clone(), None, None, None)
    x = P.plain_rms_norm(f(h), f(w1), 1e-6)
    x2, r2 = P.plain_add_rms_norm(2 * x, f(h), f(w2), 1e-6)
    assert (out.double().cpu() + x2).abs().max() < 1e-5 and (res.double().cpu() - r2).abs().max() < 1e-5
    # a later block: the previous feed-forward's output is added by this block's input norm
    prev, prev_res = rnd(4, 6, seed=2).float(), rnd(4, 6, seed=3).float()
    out, res = block.forward(prev.to(DEV).clone(), prev_res.to(DEV).clone(), None, None)
    x, r1 = P.plain_add_rms_norm(f(prev), f(prev_res), f(w1), 1e-6)
    x2, r2 = P.plain_add_rms_norm(2 * x, r1, f(w2), 1e-6)
    assert (out.double().cpu() + x2).abs().max() < 1e-5 and (res.double().cpu() - r2).abs().max() < 1e-5


def test_model_is_put_together_from_the_spec(tiny):
    """Different mixers layer by layer, a layer named twice, an entry that reads another's cache."""
    import dataclasses
    from llm_infer_rust_b200 import Qwen3Config, RunEntry
    from llm_infer_rust_b200.cache import plan_cache
    from llm_infer_rust_b200.parts import DecoderModel
    base = Qwen3Config.parse(tiny["C"]["raw"]).model_spec()
    run = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(3, reads=1), RunEntry(2))
    model = DecoderModel(dataclasses.replace(base, run_list=run), torch.float32, DEV)
    assert len(model.blocks) == 4 and [b.mixer.window for b in model.blocks] == [40, None, 40, None]
    plan = plan_cache(model, 8, 4)
    # entries 0, 2, 4 keep a window of keys; 1 keeps all; 3 reads the pages of 1
    assert sorted(((g.window or 0), g.entries) for g in plan.groups) == [(0, [1]), (40, [0, 2, 4])]
    assert plan.group_of_entry[3] == plan.group_of_entry[1]
    shapes = model.parameter_shapes()
    assert shapes["layers.2.mixer.qkv_proj"] == (15 * 48, 80) and shapes["lm_head.weight"] == (301, 80)
    assert len(model.unbound_parameters()) == len(shapes)
    with pytest.raises(ValueError, match="another shape or window"):
        DecoderModel(dataclasses.replace(base, run_list=(RunEntry(0), RunEntry(1, reads=0))), torch.float32, DEV)
