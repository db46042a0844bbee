"""A mixer with state of its own, an architecture that uses it, and a schedule that names a
layer twice and lets a layer read another layer's cache: all defined here, registered, built
from a model folder and stepped, without touching the library's files."""
import dataclasses
import json

import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
import replay
from citlali_b200.cache import StateRequirement
from citlali_b200.parts.linear import DenseLinear

pytestmark = pytest.mark.gpu


class RunningMeanMixer:
    """out_t = W . mean(h_0 .. h_t).  Per sequence it keeps the running sum and the count: a
    state of fixed size, in the cache's state region, carried from step to step."""

    def __init__(self, params, prefix):
        self.hidden = params["hidden_size"]
        self.proj = DenseLinear([f"{prefix}.proj.weight"], [self.hidden], self.hidden)

    def tensor_specs(self):
        return self.proj.tensor_specs()

    def cache_requirement(self):
        return StateRequirement((self.hidden + 1,), torch.float32)

    def bind(self, weights, ctx):
        self.proj.bind(weights, ctx)
        self.dtype = ctx.dtype

    # a step of single tokens finds its slots in the step's device tensors alone, so it can be captured in a graph
    graph_safe = True

    def forward(self, h, batch, cache_view, residual, write_cache=True):
        if batch.is_decode:
            slots = batch.row_slot.long()
            state = cache_view.storage.index_select(0, slots)
            state[:, :-1] += h.float()
            state[:, -1] += 1.0
            cache_view.storage.index_copy_(0, slots, state)
            self.proj.forward((state[:, :-1] / state[:, -1:]).to(self.dtype), accumulate_into=residual)
            return residual
        means = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        for b, slot in enumerate(batch.slots):
            state = cache_view.storage[slot]
            lo = sum(batch.n_new[:b])
            for r in range(lo, lo + batch.n_new[b]):          # rows of a sequence in order
                state[:-1] += h[r].float()
                state[-1] += 1.0
                means[r] = state[:-1] / state[-1]
        self.proj.forward(means.to(self.dtype), accumulate_into=residual)
        return residual


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["max_position_embeddings"])

    def to_dict(self):
        return {"architectures": ["ToyMeanForCausalLM"], **dataclasses.asdict(self)}

    def to_model_spec(self):
        H = self.hidden_size
        norm = lambda p: cb.PartSpec("rms_norm", {"size": H, "eps": 1e-5}, p)
        ff = lambda p: cb.PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": 2 * H}, p)
        attn = {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qk_norm_eps": 1e-5,
                "position": {"kind": "rotary_half_split", "theta": 1e4, "rotary_dim": 16}, "window": None}
        layer = lambda l, mixer: cb.LayerSpec("pre_norm_residual", {
            "mixer_norm": norm(f"l{l}.n1"), "mixer": mixer, "feed_forward_norm": norm(f"l{l}.n2"), "feed_forward": ff(f"l{l}.mlp")})
        layers = (
            layer(0, cb.PartSpec("running_mean", {"hidden_size": H}, "l0.mix")),
            layer(1, cb.PartSpec("gqa_attention", attn, "l1.attn")),
            layer(2, cb.PartSpec("gqa_attention", dict(attn, kv_projection=False), "l2.attn")),
        )
        # layer 0 runs twice (two states of its own); layer 2 has no keys and reads layer 1's
        schedule = (cb.ScheduleStep(0), cb.ScheduleStep(1), cb.ScheduleStep(0), cb.ScheduleStep(2, cache_of=1))
        return cb.ModelSpec("ToyMeanForCausalLM", self.vocab_size, H, self.max_position_embeddings, "emb.weight",
                            layers, schedule, norm("final"), "head.weight", False)


def plain_toy(w, tokens):
    T = len(tokens)
    x = plain.embedding(w["emb.weight"], tokens)
    pos = list(range(T))

    def mean_layer(x):
        h = plain.rms_norm(x, w["l0.n1.weight"], 1e-5)
        means = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
        x = x + plain.linear(means, w["l0.mix.proj.weight"])
        return x + plain.feed_forward(plain.rms_norm(x, w["l0.n2.weight"], 1e-5), w, "l0.mlp")

    x = mean_layer(x)
    h = plain.rms_norm(x, w["l1.n1.weight"], 1e-5)
    q = plain.linear(h, w["l1.attn.q_proj.weight"]).view(T, 4, 16)
    k = plain.linear(h, w["l1.attn.k_proj.weight"]).view(T, 2, 16)
    v = plain.linear(h, w["l1.attn.v_proj.weight"]).view(T, 2, 16)
    q = plain.rotary_half_split(plain.head_rms_norm(q, w["l1.attn.q_norm.weight"], 1e-5), pos, 1e4)
    k = plain.rotary_half_split(plain.head_rms_norm(k, w["l1.attn.k_norm.weight"], 1e-5), pos, 1e4)
    x = x + plain.linear(plain.causal_attention(q, k, v, 4, 2).reshape(T, 64), w["l1.attn.o_proj.weight"])
    x = x + plain.feed_forward(plain.rms_norm(x, w["l1.n2.weight"], 1e-5), w, "l1.mlp")
    x = mean_layer(x)
    h = plain.rms_norm(x, w["l2.n1.weight"], 1e-5)
    q2 = plain.linear(h, w["l2.attn.q_proj.weight"]).view(T, 4, 16)
    q2 = plain.rotary_half_split(plain.head_rms_norm(q2, w["l2.attn.q_norm.weight"], 1e-5), pos, 1e4)
    x = x + plain.linear(plain.causal_attention(q2, k, v, 4, 2).reshape(T, 64), w["l2.attn.o_proj.weight"])
    x = x + plain.feed_forward(plain.rms_norm(x, w["l2.n2.weight"], 1e-5), w, "l2.mlp")
    return plain.linear(plain.rms_norm(x, w["final.weight"], 1e-5), w["head.weight"])


class Top1RoutedFeedForward:
    """A feed-forward with routing: a router picks one of `experts` gated feed-forwards per token; the winner's
    output is scaled by its softmax probability.  Router logits, softmax and the choice are float32."""

    def __init__(self, params, prefix):
        self.hidden, self.inter, self.experts = params["hidden_size"], params["intermediate_size"], params["experts"]
        self.router = DenseLinear([f"{prefix}.router.weight"], [self.experts], self.hidden)
        self.gate_up = [DenseLinear([f"{prefix}.experts.{e}.gate.weight", f"{prefix}.experts.{e}.up.weight"],
                                    [self.inter, self.inter], self.hidden) for e in range(self.experts)]
        self.down = [DenseLinear([f"{prefix}.experts.{e}.down.weight"], [self.hidden], self.inter) for e in range(self.experts)]

    def tensor_specs(self):
        return self.router.tensor_specs() + [t for l in self.gate_up + self.down for t in l.tensor_specs()]

    def bind(self, weights, ctx):
        for l in [self.router] + self.gate_up + self.down:
            l.bind(weights, ctx)
        self.dtype = ctx.dtype

    def forward(self, h, batch, residual):
        logits = self.router.forward(h, out_dtype=torch.float32)
        prob = torch.softmax(logits, dim=-1)
        choice = torch.argmax(logits, dim=-1)
        for e in range(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel() == 0:
                continue
            x = h[rows].contiguous()
            gu = self.gate_up[e].forward(x, out_dtype=torch.float32)
            act = (torch.nn.functional.silu(gu[:, :self.inter]) * gu[:, self.inter:]).to(self.dtype)
            y = self.down[e].forward(act, out_dtype=torch.float32)
            residual[rows] += y * prob[rows, e][:, None]
        return residual


class SlowedRotary:
    """Another position encoding: the half-split rotation with every frequency divided by `factor`."""

    def __init__(self, params, head_dim):
        self.rotary_dim = head_dim
        i = torch.arange(head_dim // 2, dtype=torch.float64)
        self.inv_freq = (torch.pow(torch.tensor(float(params["theta"]), dtype=torch.float64), -2.0 * i / head_dim)
                         / float(params["factor"])).to(torch.float32)


@dataclasses.dataclass(frozen=True)
class RoutedConfig:
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["max_position_embeddings"])

    def to_dict(self):
        return {"architectures": ["ToyRoutedForCausalLM"], **dataclasses.asdict(self)}

    def to_model_spec(self):
        H = self.hidden_size
        norm = lambda p: cb.PartSpec("rms_norm", {"size": H, "eps": 1e-5}, p)
        attn = {"hidden_size": H, "num_heads": 4, "num_kv_heads": 4, "head_dim": 16, "qk_norm_eps": None,
                "position": {"kind": "slowed_rotary", "theta": 1e4, "factor": 4.0}, "window": 40}
        routed = cb.PartSpec("top1_routed", {"hidden_size": H, "intermediate_size": 48, "experts": 3}, "l0.moe")
        dense = cb.PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": 96}, "l1.mlp")
        layers = (
            cb.LayerSpec("pre_norm_residual", {"mixer_norm": norm("l0.n1"), "mixer": cb.PartSpec("gqa_attention", attn, "l0.attn"),
                                               "feed_forward_norm": norm("l0.n2"), "feed_forward": routed}),
            cb.LayerSpec("pre_norm_residual", {"mixer_norm": norm("l1.n1"),
                                               "mixer": cb.PartSpec("gqa_attention", dict(attn, window=None), "l1.attn"),
                                               "feed_forward_norm": norm("l1.n2"), "feed_forward": dense}),
        )
        return cb.ModelSpec("ToyRoutedForCausalLM", self.vocab_size, H, self.max_position_embeddings, "emb.weight",
                            layers, (cb.ScheduleStep(0), cb.ScheduleStep(1)), norm("final"), "head.weight", None)


def plain_routed(w, tokens):
    T = len(tokens)
    pos = list(range(T))
    x = plain.embedding(w["emb.weight"], tokens)

    def rotate(t):
        d = t.shape[-1]
        i = torch.arange(d // 2, dtype=torch.float64)
        inv = (torch.pow(torch.tensor(1e4, dtype=torch.float64), -2.0 * i / d) / 4.0).to(torch.float32)
        ang = (torch.tensor(pos, dtype=torch.float32)[:, None] * inv[None, :]).double()
        c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = t[..., :d // 2], t[..., d // 2:]
        return torch.cat([a * c - b * s_, a * s_ + b * c], dim=-1)

    def attention(x, pre, window):
        h = plain.rms_norm(x, w[f"{pre}.n1.weight"], 1e-5)
        q = rotate(plain.linear(h, w[f"{pre}.attn.q_proj.weight"]).view(T, 4, 16))
        k = rotate(plain.linear(h, w[f"{pre}.attn.k_proj.weight"]).view(T, 4, 16))
        v = plain.linear(h, w[f"{pre}.attn.v_proj.weight"]).view(T, 4, 16)
        return x + plain.linear(plain.causal_attention(q, k, v, 4, 4, window=window).reshape(T, 64), w[f"{pre}.attn.o_proj.weight"])

    x = attention(x, "l0", 40)
    h = plain.rms_norm(x, w["l0.n2.weight"], 1e-5)
    logits = plain.linear(h, w["l0.moe.router.weight"])
    prob = torch.softmax(logits, -1)
    choice = torch.argmax(logits, -1)
    margin = torch.topk(logits, 2, dim=-1).values
    y = torch.zeros_like(x)
    for t in range(T):
        e = int(choice[t])
        g = plain.linear(h[t:t + 1], w[f"l0.moe.experts.{e}.gate.weight"]); u = plain.linear(h[t:t + 1], w[f"l0.moe.experts.{e}.up.weight"])
        y[t] = plain.linear(plain.swiglu(g, u), w[f"l0.moe.experts.{e}.down.weight"])[0] * prob[t, e]
    x = x + y
    x = attention(x, "l1", None)
    x = x + plain.feed_forward(plain.rms_norm(x, w["l1.n2.weight"], 1e-5), w, "l1.mlp")
    return plain.linear(plain.rms_norm(x, w["final.weight"], 1e-5), w["emb.weight"]), (margin[:, 0] - margin[:, 1])


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """A feed-forward with routing, a position encoding of its own, a windowed and a full attention layer (two cache
    groups), a head that is tied because the folder holds none: registered from here, replayed in 32-bit against the oracle."""
    cb.register_part("feed_forward", "top1_routed", Top1RoutedFeedForward)
    cb.register_part("position", "slowed_rotary", SlowedRotary)
    cb.register_architecture("ToyRoutedForCausalLM", RoutedConfig)
    try:
        cfg = RoutedConfig(vocab_size=200, hidden_size=64, max_position_embeddings=256)
        folder = cb.write_random_model(str(tmp_path / "routed"), cfg, seed=8, dtype="float32")
        _, w = plain.load_folder(folder)
        session = cb.InferenceSession().load_model(folder, max_context=256, dtype="float32", max_batch=2)
        assert [g.requirement.window for g in session.cache.kv_groups] == [40, None] and session.runner is None
        assert session.model.tied
        import random
        rng = random.Random(5)
        reqs = [(f"m{i}", [rng.randrange(200) for _ in range(n)]) for i, n in enumerate([90, 12, 150])]
        want = {rid: plain_routed(w, toks) for rid, toks in reqs}
        for steps in (replay.whole(reqs), replay.tail(reqs), replay.batched(reqs, [60, 12, 1], 2)):
            got = replay.run_in_process(session, steps)
            for (rid, pos), row in got.items():
                ref, margins = want[rid]
                if float(margins[:pos + 1].min()) < 1e-4:
                    continue                   # a routing near-tie upstream: either expert is a right answer
                assert (row.double() - ref[pos]).abs().max() <= 2e-5 * ref[pos].abs().max() + 1e-6
        assert session.cache.pages_held() == 0
    finally:
        cb.unregister_part("feed_forward", "top1_routed")
        cb.unregister_part("position", "slowed_rotary")
        cb.unregister_architecture("ToyRoutedForCausalLM")


@pytest.fixture
def toy_registered():
    cb.register_part("mixer", "running_mean", RunningMeanMixer)
    cb.register_architecture("ToyMeanForCausalLM", ToyConfig)
    yield
    cb.unregister_part("mixer", "running_mean")
    cb.unregister_architecture("ToyMeanForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(toy_registered, tmp_path, dtype):
    cfg = ToyConfig(vocab_size=300, hidden_size=64, max_position_embeddings=256)
    folder = cb.write_random_model(str(tmp_path / "toy"), cfg, seed=3, dtype=dtype)
    assert json.load(open(f"{folder}/config.json"))["architectures"] == ["ToyMeanForCausalLM"]
    _, w = plain.load_folder(folder)
    session = cb.InferenceSession().load_model(folder, max_context=256, dtype=dtype, max_batch=2)
    assert len(session.cache.state_groups) == 1 and session.cache.state_groups[0].steps == [0, 2]
    assert len(session.cache.kv_groups) == 1 and session.cache.kv_groups[0].steps == [1]
    import random
    rng = random.Random(4)
    reqs = [(f"t{i}", [rng.randrange(300) for _ in range(n)]) for i, n in enumerate([70, 9, 41])]
    want = {rid: plain_toy(w, toks) for rid, toks in reqs}
    tolerance = 2e-5 if dtype == "float32" else 2.5e-2
    for steps in (replay.whole(reqs), replay.tail(reqs), replay.batched(reqs, [30, 9, 1], 2)):
        got = replay.run_in_process(session, steps)
        for (rid, pos), row in got.items():
            ref = want[rid][pos]
            assert (row.double() - ref).abs().max() <= tolerance * ref.abs().max() + 1e-6


def test_toy_mixer_with_state_decodes_inside_a_replayed_graph(toy_registered, tmp_path):
    """The toy mixer says it is graph-safe (its single-token path reads slots from the device), so the session
    captures the decode step with the mixer's state updates inside: five requests over two slots (states are
    zeroed when a slot is taken again) give the same tokens as plain launches, and the logits after a replayed
    run still match the oracle."""
    cfg = ToyConfig(vocab_size=300, hidden_size=64, max_position_embeddings=256)
    folder = cb.write_random_model(str(tmp_path / "toy"), cfg, seed=3, dtype="bfloat16")
    import random
    rng = random.Random(9)
    prompts = [[rng.randrange(300) for _ in range(n)] for n in (7, 40, 3, 19, 11)]
    opts = cb.GenerationOptions(max_new_tokens=25, max_context=256, stop_ids=[])
    session = cb.InferenceSession().load_model(folder, max_context=256, dtype="bfloat16", max_batch=2)
    assert session.runner is not None
    with_graph = [r.tokens for r in session.generate(prompts, opts)]
    assert len(session.runner.graphs) > 0 and all(len(t) == 25 for t in with_graph)
    plain_launches = cb.InferenceSession()
    plain_launches.use_graphs = False
    plain_launches.load_model(folder, max_context=256, dtype="bfloat16", max_batch=2)
    assert plain_launches.runner is None
    assert [r.tokens for r in plain_launches.generate(prompts, opts)] == with_graph
    # the engine's own continuation, fed whole to the oracle: the last logits it saw are the oracle's
    _, w = plain.load_folder(folder)
    slot = session.acquire()
    whole = prompts[1] + with_graph[1]
    logits = session.step([cb.StepEntry(slot, whole, [len(whole) - 1])])[0]
    session.release(slot)
    ref = plain_toy(w, whole)[-1]
    assert (logits.double().cpu() - ref).abs().max() <= 2.5e-2 * ref.abs().max()


def test_unknown_part_kind_in_a_spec_is_an_error(tmp_path):
    cfg = ToyConfig(vocab_size=300, hidden_size=64, max_position_embeddings=256)
    with pytest.raises(cb.CitlaliError, match="unknown mixer kind 'running_mean'"):
        cb.expected_tensors(cfg.to_model_spec())
