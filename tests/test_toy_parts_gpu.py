"""Parts that the framework does not ship, defined here and plugged in through the
registries alone: a mixer with per-request state of its own (a linear recurrence),
an architecture that alternates it with attention, runs one layer twice and lets
the second run read the first run's keys and values; and a second architecture
with a feed-forward that routes every token to two of its experts (in one layer
only, beside a dense one) and a position encoding of its own (a partial rotation
over scaled positions).  Nothing under ``llm_infer_rust_b200/`` knows these parts;
the tests register, build, load and step them, cut in different ways, and compare
with plain whole-sequence implementations written here.
"""
import dataclasses
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- the toy parts
def register_toys():
    from llm_infer_rust_b200 import (Architecture, LayerSpec, ModelSpec, PartSpec, RunEntry,
                                     register_architecture)
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.parts import ParamDecl, Part, StateSpec, register_part
    from llm_infer_rust_b200.weights import SourceTensor, WeightBinding

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + W_in x_t;  y_t = W_out s_t.  The state s lives in the request's slot;
        a row that starts at position 0 starts from zeros."""
        category = "mixer"

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.hidden, self.n, self.decay = int(spec["hidden_size"]), int(spec["state_size"]), float(spec["decay"])

        def param_decls(self):
            return {"w_in": ParamDecl((self.n, self.hidden)), "w_out": ParamDecl((self.hidden, self.n))}

        def cache_spec(self):
            return None

        def state_spec(self):
            return StateSpec((self.n,), torch.float32)

        def forward(self, x, ctx, cache):
            """Works from the step's index arrays on the device alone (no number is read on the host), so the same
            code runs eagerly and inside a captured graph, whose context has no host copy."""
            u = ops.linear(x, self.params["w_in"]).float()                        # [T, n]
            row = ctx.row_of_token.long()                                         # [T]
            cu, slots = ctx.cu_q.long(), ctx.state_slots.long()
            t = torch.arange(u.shape[0], device=u.device)
            local = t - cu[row]                                                   # index of a token inside its row
            before = cache.state[slots] * (ctx.prefix_len != 0).to(torch.float32)[:, None]   # fresh rows start from zeros
            # s_t = decay^(i+1) s_before + sum over j <= t of the same row of decay^(t-j) u_j
            ages = (t[:, None] - t[None, :]).to(torch.float32)
            same = (row[:, None] == row[None, :]) & (t[None, :] <= t[:, None])
            weights = torch.where(same, torch.pow(torch.full_like(ages, self.decay), ages.clamp_min(0.0)),
                                  torch.zeros_like(ages))
            states = weights @ u + torch.pow(torch.full_like(local, self.decay, dtype=torch.float32),
                                             (local + 1).to(torch.float32))[:, None] * before[row]
            cache.state.index_copy_(0, slots, states[cu[1:] - 1])                 # (padding rows write the sink slot 0)
            return ops.linear(states.to(x.dtype), self.params["w_out"])

    register_part("mixer", "toy_decay", DecayMixer, replace=True)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        heads: int
        kv_heads: int
        head_dim: int
        inter: int
        vocab: int
        state: int
        decay: float
        eps: float
        theta: float
        max_pos: int

        @staticmethod
        def parse(raw):
            return ToyConfig(raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"],
                             raw["head_dim"], raw["intermediate_size"], raw["vocab_size"], raw["state_size"],
                             raw["decay"], raw["rms_norm_eps"], raw["rope_theta"], raw["max_position_embeddings"])

    def model_spec(c):
        norm = PartSpec("rms_norm", {"width": c.hidden, "eps": c.eps})
        ffn = PartSpec("swiglu", {"hidden_size": c.hidden, "intermediate_size": c.inter})
        attn = PartSpec("gqa_attention", {"hidden_size": c.hidden, "num_heads": c.heads, "num_kv_heads": c.kv_heads,
                                          "head_dim": c.head_dim, "qk_norm_eps": c.eps, "window": None,
                                          "softmax_scale": 1.0 / math.sqrt(c.head_dim), "position_encoding": "rope"})
        toy = PartSpec("toy_decay", {"hidden_size": c.hidden, "state_size": c.state, "decay": c.decay})
        block = PartSpec("pre_norm_deferred_add")
        return ModelSpec(
            architecture="ToyHybridForCausalLM", vocab_size=c.vocab, hidden_size=c.hidden, max_positions=c.max_pos,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.hidden}),
            layers=(LayerSpec.pre_norm(block, attn, ffn, norm), LayerSpec.pre_norm(block, toy, ffn, norm)),
            run_list=(RunEntry(0), RunEntry(1), RunEntry(0, reads=0), RunEntry(1)),
            final_norm=norm, lm_head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.hidden,
                                                              "tied": True}),
            position_encodings={"rope": PartSpec("half_split_rope", {"rotary_dim": c.head_dim, "theta": c.theta,
                                                                     "max_positions": c.max_pos})})

    def weight_plan(c):
        h, d = c.hidden, c.head_dim

        def common(i):
            return [WeightBinding(f"layers.{i}.input_norm.weight", (SourceTensor(f"l{i}.norm_in", (h,), "norm"),)),
                    WeightBinding(f"layers.{i}.post_mixer_norm.weight", (SourceTensor(f"l{i}.norm_post", (h,), "norm"),)),
                    WeightBinding(f"layers.{i}.feed_forward.gate_up_proj",
                                  (SourceTensor(f"l{i}.gate", (c.inter, h)), SourceTensor(f"l{i}.up", (c.inter, h)))),
                    WeightBinding(f"layers.{i}.feed_forward.down_proj", (SourceTensor(f"l{i}.down", (h, c.inter)),))]

        plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c.vocab, h)),))] + common(0) + common(1)
        plan += [WeightBinding("layers.0.mixer.qkv_proj", (SourceTensor("l0.q", (c.heads * d, h)),
                                                          SourceTensor("l0.k", (c.kv_heads * d, h)),
                                                          SourceTensor("l0.v", (c.kv_heads * d, h)))),
                 WeightBinding("layers.0.mixer.q_norm", (SourceTensor("l0.q_norm", (d,), "norm"),)),
                 WeightBinding("layers.0.mixer.k_norm", (SourceTensor("l0.k_norm", (d,), "norm"),)),
                 WeightBinding("layers.0.mixer.o_proj", (SourceTensor("l0.o", (h, c.heads * d)),)),
                 WeightBinding("layers.1.mixer.w_in", (SourceTensor("l1.w_in", (c.state, h)),)),
                 WeightBinding("layers.1.mixer.w_out", (SourceTensor("l1.w_out", (h, c.state)),)),
                 WeightBinding("final_norm.weight", (SourceTensor("norm", (h,), "norm"),)),
                 WeightBinding("lm_head.weight", (SourceTensor("head", (c.vocab, h)),), optional=True,
                               alias_of="embedding.weight")]
        return plan

    register_architecture(Architecture("ToyHybridForCausalLM", "toy_hybrid", ToyConfig.parse, model_spec, weight_plan),
                          replace=True)


RAW = {"model_type": "toy_hybrid", "architectures": ["ToyHybridForCausalLM"], "hidden_size": 72,
       "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 100,
       "vocab_size": 211, "state_size": 24, "decay": 0.9, "rms_norm_eps": 1e-5, "rope_theta": 1000.0,
       "max_position_embeddings": 96}


# ----------------------------------------------------------------------------- its plain twin
def plain_toy_forward(w, ids):
    w = {n: t.double() for n, t in w.items()}
    T = len(ids)
    pos = torch.arange(T)
    eps, theta = RAW["rms_norm_eps"], RAW["rope_theta"]
    h = P.plain_embedding(torch.tensor(ids), w["embed"])
    residual, kv_first = None, None
    for entry, (layer, reads) in enumerate([(0, None), (1, None), (0, 0), (1, None)]):
        pre = f"l{layer}."
        if residual is None:
            residual, x = h, P.plain_rms_norm(h, w[pre + "norm_in"], eps)
        else:
            x, residual = P.plain_add_rms_norm(h, residual, w[pre + "norm_in"], eps)
        if layer == 0:
            q, k, v = P.plain_qkv(x, w["l0.q"], w["l0.k"], w["l0.v"], 3, 1, 32)
            q, k = P.plain_qk_norm(q, k, w["l0.q_norm"], w["l0.k_norm"], eps)
            q, k = P.plain_rope(q, pos, theta), P.plain_rope(k, pos, theta)
            if reads is None:
                kv_first = (k, v)
            else:
                k, v = kv_first
            a = P.plain_attention(q, k, v) @ w["l0.o"].T
        else:
            u = x @ w["l1.w_in"].T
            s = torch.zeros(RAW["state_size"], dtype=torch.float64)
            states = []
            for t in range(T):
                s = RAW["decay"] * s + u[t]
                states.append(s)
            a = torch.stack(states) @ w["l1.w_out"].T
        x, residual = P.plain_add_rms_norm(a, residual, w[pre + "norm_post"], eps)
        h = P.plain_swiglu(x, w[pre + "gate"], w[pre + "up"], w[pre + "down"])
    x, _ = P.plain_add_rms_norm(h, residual, w["norm"], eps)
    return P.plain_lm_head(x, w["embed"])


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    register_toys()
    from llm_infer_rust_b200 import random_tensors, write_random_model
    from llm_infer_rust_b200.engine import Engine, StepEntry
    d = write_random_model(str(tmp_path), RAW, seed=4, norm_std=0.1)
    w = random_tensors(RAW, 4, norm_std=0.1)
    eng = Engine(d, dtype="float32", max_running_req=3, page_size=8, max_total_tokens=256, cuda_graph_bs=0)
    # what the framework derived from the parts: one paged group (two entries share one cache), state for entries 1 and 3
    assert len(eng.cache_plan.groups) == 1 and eng.cache_plan.groups[0].entries == [0]
    assert sorted(eng.cache_plan.state_entries) == [1, 3]
    assert eng.cache.layer_caches[2].k.data_ptr() == eng.cache.layer_caches[0].k.data_ptr()
    assert not eng.cache.layer_caches[2].writes and eng.cache.layer_caches[1].k is None
    assert tuple(eng.cache.layer_caches[1].state.shape) == (4, 24)

    g = torch.Generator().manual_seed(9)
    seqs = {r: torch.randint(0, 211, (n,), generator=g).tolist() for r, n in ((1, 80), (2, 37), (3, 64))}
    want = {r: plain_toy_forward(w, ids).numpy() for r, ids in seqs.items()}

    def feed(plan):
        """plan: list of steps, each a list of (request, count)."""
        fed = {r: 0 for r in seqs}
        got = {r: [] for r in seqs}
        for step in plan:
            entries = []
            for r, n in step:
                if fed[r] == 0:
                    eng.open_request(r)
                entries.append(StepEntry(r, seqs[r][fed[r]: fed[r] + n], list(range(n))))
                fed[r] += n
            logits = eng.step(entries).cpu().numpy()
            at = 0
            for r, n in step:
                got[r].append(logits[at: at + n])
                at += n
        eng.check_kernel_errors()
        for r in seqs:
            if fed[r]:
                eng.close_request(r)
        return {r: np.concatenate(v) for r, v in got.items() if v}

    whole = feed([[(1, 80)], [(2, 37)], [(3, 64)]])
    # the same slots are used again here: the state must start from zeros
    mixed = feed([[(1, 50), (2, 2)], [(1, 1), (2, 30), (3, 3)], [(1, 1), (2, 1), (3, 59)]] +
                 [[(1, 1), (2, 1), (3, 1)]] * 2 + [[(1, 1), (2, 1)]] * 2 + [[(1, 1)]] * 24)
    for name, got in (("whole", whole), ("mixed", mixed)):
        for r in seqs:
            scale = max(1.0, np.abs(want[r]).max())
            err = np.abs(got[r] - want[r]).max()
            assert err <= 1e-5 * scale, (name, r, err)


def test_the_stateful_toy_mixer_inside_decode_graphs(tmp_path):
    """bfloat16 with decode graphs on: a graph is captured on throw-away requests, so a live request's state
    advances once per step, also in the step that uses a graph for the first time; a padded batch (3 rows in the
    graph of 4) writes its padding row's state to the sink slot."""
    register_toys()
    from llm_infer_rust_b200 import random_tensors, write_random_model
    from llm_infer_rust_b200.engine import Engine, StepEntry
    d = write_random_model(str(tmp_path), RAW, seed=4, norm_std=0.1, dtype="bfloat16")
    w = {n: t.to(torch.bfloat16) for n, t in random_tensors(RAW, 4, norm_std=0.1).items()}
    eng = Engine(d, dtype="bfloat16", max_running_req=4, page_size=8, max_total_tokens=512, cuda_graph_bs=4)
    assert all(g.graph is not None for g in eng._graphs.values())
    g = torch.Generator().manual_seed(11)
    seqs = {r: torch.randint(0, 211, (n,), generator=g).tolist() for r, n in ((1, 60), (2, 41), (3, 52))}
    want = {r: plain_toy_forward(w, ids).numpy() for r, ids in seqs.items()}
    decoded = 20
    got = {r: [] for r in seqs}
    for r, ids in seqs.items():
        eng.open_request(r)
        n = len(ids) - decoded
        got[r].append(eng.step([StepEntry(r, ids[:n], list(range(n)))]).float().cpu().numpy())
    for k in range(decoded):
        live = [r for r in seqs if not (r == 2 and k >= 12)]        # 3 rows in the graph of 4, then 2 rows in the graph of 2
        logits = eng.step([StepEntry(r, [seqs[r][len(seqs[r]) - decoded + k]], [0]) for r in live]).float().cpu().numpy()
        for i, r in enumerate(live):
            got[r].append(logits[i:i + 1])
    eng.check_kernel_errors()
    for r, ids in seqs.items():
        rows = np.concatenate(got[r])
        ref = want[r][:rows.shape[0]]
        assert np.abs(rows - ref).max() <= 2.0 ** -5 * max(1.0, np.abs(ref).max()), r


# ----------------------------------------------------------------------------- routed experts, another position encoding
def register_routed_toys():
    from llm_infer_rust_b200 import (Architecture, LayerSpec, ModelSpec, PartSpec, RunEntry,
                                     register_architecture)
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.parts import ParamDecl, Part, register_part
    from llm_infer_rust_b200.weights import SourceTensor, WeightBinding

    class ScaledPartialRope(Part):
        """Rotates the first `rotary_dim` dims of a head (half-split pairs) by (p / position_scale) * theta^(-2i / rotary_dim).
        It offers what the attention mixer asks of a position encoding: cos, sin [max_positions, rotary_dim / 2], rot_dim."""
        category = "position_encoding"

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.rot_dim = int(spec["rotary_dim"])
            i = torch.arange(0, self.rot_dim, 2, dtype=torch.float64)
            inv_freq = float(spec["theta"]) ** (-i / self.rot_dim)
            pos = torch.arange(int(spec["max_positions"]), dtype=torch.float64) / float(spec["position_scale"])
            angle = pos[:, None] * inv_freq[None, :]
            self.cos = torch.cos(angle).float().to(env.device).contiguous()
            self.sin = torch.sin(angle).float().to(env.device).contiguous()

    register_part("position_encoding", "toy_scaled_partial_rope", ScaledPartialRope, replace=True)

    class TopTwoExperts(Part):
        """Router logits in float; every token goes to its `top_k` experts, weighted by the softmax over the
        chosen logits; each expert is a SwiGLU of its own.  The experts' matrices are stacked in two parameters."""
        category = "feed_forward"

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.h, self.inter = int(spec["hidden_size"]), int(spec["expert_size"])
            self.n, self.k = int(spec["num_experts"]), int(spec["top_k"])

        def param_decls(self):
            return {"router": ParamDecl((self.n, self.h)), "gate_up": ParamDecl((self.n * 2 * self.inter, self.h)),
                    "down": ParamDecl((self.n * self.h, self.inter))}

        def forward(self, x):
            logits = ops.linear(x, self.params["router"]).float()
            top, idx = logits.topk(self.k, dim=-1)
            weight = torch.softmax(top, dim=-1)
            out = torch.zeros(x.shape[0], self.h, dtype=torch.float32, device=x.device)
            for e in range(self.n):
                rows, slot = (idx == e).nonzero(as_tuple=True)
                if rows.numel() == 0:
                    continue
                gu = ops.linear(x[rows].contiguous(), self.params["gate_up"][e * 2 * self.inter: (e + 1) * 2 * self.inter])
                y = ops.linear(ops.silu_mul(gu), self.params["down"][e * self.h: (e + 1) * self.h])
                out.index_add_(0, rows, y.float() * weight[rows, slot][:, None])
            return out.to(x.dtype)

    register_part("feed_forward", "toy_top_two_experts", TopTwoExperts, replace=True)

    def parse(raw):
        return dict(raw)

    def model_spec(c):
        h, d = c["hidden_size"], c["head_dim"]
        norm = PartSpec("rms_norm", {"width": h, "eps": c["rms_norm_eps"]})
        attn = PartSpec("gqa_attention", {"hidden_size": h, "num_heads": c["num_attention_heads"],
                                          "num_kv_heads": c["num_key_value_heads"], "head_dim": d,
                                          "qk_norm_eps": None, "window": None, "softmax_scale": c["softmax_scale"],
                                          "position_encoding": "scaled"})
        dense = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": c["intermediate_size"]})
        routed = PartSpec("toy_top_two_experts", {"hidden_size": h, "expert_size": c["expert_size"],
                                                  "num_experts": c["num_experts"], "top_k": c["top_k"]})
        block = PartSpec("pre_norm_deferred_add")
        return ModelSpec(
            architecture="ToyRoutedForCausalLM", vocab_size=c["vocab_size"], hidden_size=h,
            max_positions=c["max_position_embeddings"],
            embedding=PartSpec("token_embedding", {"vocab_size": c["vocab_size"], "hidden_size": h}),
            layers=(LayerSpec.pre_norm(block, attn, dense, norm), LayerSpec.pre_norm(block, attn, routed, norm)),
            run_list=(RunEntry(0), RunEntry(1)), final_norm=norm,
            lm_head=PartSpec("linear_head", {"vocab_size": c["vocab_size"], "hidden_size": h, "tied": False}),
            position_encodings={"scaled": PartSpec("toy_scaled_partial_rope", {
                "rotary_dim": c["rotary_dim"], "theta": c["rope_theta"], "position_scale": c["position_scale"],
                "max_positions": c["max_position_embeddings"]})})

    def weight_plan(c):
        h, d, nh, nkv = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"]
        plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c["vocab_size"], h)),)),
                WeightBinding("final_norm.weight", (SourceTensor("norm", (h,), "norm"),)),
                WeightBinding("lm_head.weight", (SourceTensor("head", (c["vocab_size"], h)),))]
        for i in range(2):
            plan += [WeightBinding(f"layers.{i}.input_norm.weight", (SourceTensor(f"l{i}.norm_in", (h,), "norm"),)),
                     WeightBinding(f"layers.{i}.post_mixer_norm.weight", (SourceTensor(f"l{i}.norm_post", (h,), "norm"),)),
                     WeightBinding(f"layers.{i}.mixer.qkv_proj", (SourceTensor(f"l{i}.q", (nh * d, h)),
                                                                    SourceTensor(f"l{i}.k", (nkv * d, h)),
                                                                    SourceTensor(f"l{i}.v", (nkv * d, h)))),
                     WeightBinding(f"layers.{i}.mixer.o_proj", (SourceTensor(f"l{i}.o", (h, nh * d)),))]
        inter, ex = c["intermediate_size"], c["expert_size"]
        plan += [WeightBinding("layers.0.feed_forward.gate_up_proj", (SourceTensor("l0.gate", (inter, h)),
                                                                      SourceTensor("l0.up", (inter, h)))),
                 WeightBinding("layers.0.feed_forward.down_proj", (SourceTensor("l0.down", (h, inter)),)),
                 WeightBinding("layers.1.feed_forward.router", (SourceTensor("l1.router", (c["num_experts"], h), "norm"),)),
                 WeightBinding("layers.1.feed_forward.gate_up", tuple(
                     SourceTensor(f"l1.e{e}.{n}", (ex, h)) for e in range(c["num_experts"]) for n in ("gate", "up"))),
                 WeightBinding("layers.1.feed_forward.down", tuple(
                     SourceTensor(f"l1.e{e}.down", (h, ex)) for e in range(c["num_experts"])))]
        return plan

    register_architecture(Architecture("ToyRoutedForCausalLM", "toy_routed", parse, model_spec, weight_plan),
                          replace=True)


ROUTED = {"model_type": "toy_routed", "architectures": ["ToyRoutedForCausalLM"], "hidden_size": 88,
          "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 48, "rotary_dim": 32, "position_scale": 4.0,
          "softmax_scale": 0.2, "intermediate_size": 120, "expert_size": 56, "num_experts": 5, "top_k": 2,
          "vocab_size": 157, "rms_norm_eps": 1e-5, "rope_theta": 500.0, "max_position_embeddings": 128}


def plain_routed_forward(w, ids):
    c = ROUTED
    w = {n: t.double() for n, t in w.items()}
    T, d, rot = len(ids), c["head_dim"], c["rotary_dim"]
    inv_freq = c["rope_theta"] ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)
    angle = (torch.arange(T, dtype=torch.float64) / c["position_scale"])[:, None] * inv_freq[None]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]

    def rotate(x):                                             # [T, heads, d]: pairs (i, i + rot / 2) of the first rot dims
        a, b, rest = x[..., : rot // 2], x[..., rot // 2: rot], x[..., rot:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)

    h = P.plain_embedding(torch.tensor(ids), w["embed"])
    residual = None
    for i in range(2):
        pre = f"l{i}."
        if residual is None:
            residual, x = h, P.plain_rms_norm(h, w[pre + "norm_in"], c["rms_norm_eps"])
        else:
            x, residual = P.plain_add_rms_norm(h, residual, w[pre + "norm_in"], c["rms_norm_eps"])
        q, k, v = P.plain_qkv(x, w[pre + "q"], w[pre + "k"], w[pre + "v"], c["num_attention_heads"],
                              c["num_key_value_heads"], d)
        # (plain_attention divides by sqrt(d); this model's scale is a constant of its own)
        a = P.plain_attention(rotate(q) * (c["softmax_scale"] * math.sqrt(d)), rotate(k), v) @ w[pre + "o"].T
        x, residual = P.plain_add_rms_norm(a, residual, w[pre + "norm_post"], c["rms_norm_eps"])
        if i == 0:
            h = P.plain_swiglu(x, w["l0.gate"], w["l0.up"], w["l0.down"])
        else:
            logits = x @ w["l1.router"].T
            top, idx = logits.topk(c["top_k"], dim=-1)
            weight = torch.softmax(top, dim=-1)
            h = torch.zeros_like(x)
            for t in range(T):
                for j in range(c["top_k"]):
                    e = int(idx[t, j])
                    y = P.plain_swiglu(x[t: t + 1], w[f"l1.e{e}.gate"], w[f"l1.e{e}.up"], w[f"l1.e{e}.down"])
                    h[t] += weight[t, j] * y[0]
    x, _ = P.plain_add_rms_norm(h, residual, w["norm"], c["rms_norm_eps"])
    return P.plain_lm_head(x, w["head"])


def test_a_routed_feed_forward_and_another_position_encoding(tmp_path):
    register_routed_toys()
    from llm_infer_rust_b200 import random_tensors, write_random_model
    from llm_infer_rust_b200.engine import Engine, StepEntry
    d = write_random_model(str(tmp_path), ROUTED, seed=6, std=0.05, norm_std=0.3)
    w = random_tensors(ROUTED, 6, std=0.05, norm_std=0.3)
    eng = Engine(d, dtype="float32", max_running_req=3, page_size=4, max_total_tokens=192, cuda_graph_bs=0)
    assert type(eng.model.blocks[1].feed_forward).__name__ == "TopTwoExperts"
    assert type(eng.model.blocks[0].feed_forward).__name__ != "TopTwoExperts"
    g = torch.Generator().manual_seed(2)
    seqs = {r: torch.randint(0, ROUTED["vocab_size"], (n,), generator=g).tolist() for r, n in ((1, 90), (2, 41))}
    want = {r: plain_routed_forward(w, ids).numpy() for r, ids in seqs.items()}
    # every expert is used by some token, and no expert by all
    x = torch.randn(64, ROUTED["hidden_size"], generator=g)
    chosen = (x.double() @ w["l1.router"].double().T).topk(2, dim=-1).indices
    assert set(chosen.flatten().tolist()) == set(range(ROUTED["num_experts"]))

    def feed(plan):
        fed = {r: 0 for r in seqs}
        got = {r: [] for r in seqs}
        for step in plan:
            entries = []
            for r, n in step:
                if fed[r] == 0:
                    eng.open_request(r)
                entries.append(StepEntry(r, seqs[r][fed[r]: fed[r] + n], list(range(n))))
                fed[r] += n
            logits = eng.step(entries).cpu().numpy()
            at = 0
            for r, n in step:
                got[r].append(logits[at: at + n])
                at += n
        eng.check_kernel_errors()
        for r in seqs:
            eng.close_request(r)
        return {r: np.concatenate(v) for r, v in got.items()}

    whole = feed([[(1, 90)], [(2, 41)]])
    mixed = feed([[(1, 60), (2, 2)], [(1, 1), (2, 30)], [(1, 2), (2, 1)]] + [[(1, 1), (2, 1)]] * 8 + [[(1, 1)]] * 19)
    for name, got in (("whole", whole), ("mixed", mixed)):
        for r in seqs:
            scale = max(1.0, np.abs(want[r]).max())
            err = np.abs(got[r] - want[r]).max()
            assert err <= 1e-5 * scale, (name, r, err)


def test_an_unknown_part_is_refused_by_name():
    from llm_infer_rust_b200 import PartSpec
    from llm_infer_rust_b200.parts import BuildEnv, build_part
    with pytest.raises(KeyError, match="no mixer named 'nonesuch'"):
        build_part("mixer", PartSpec("nonesuch"), BuildEnv(torch.float32, torch.device("cuda"), {}))
