"""Arrangements of a layer that the library does not have, defined here and registered from outside: a layer with
four norms (one before and one after each of mixer and feed-forward), a layer whose mixer and feed-forward run side by
side on one norm, and a layer with a feed-forward only; an architecture made of them that scales its embedding rows
and its logits.  Built from a model folder, replayed whole, token by token and in batches against an oracle written
beside them.  None of this is a model of anyone's: it shows what a layer's description can say without a change to
the library's files."""
import dataclasses

import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
import replay

pytestmark = pytest.mark.gpu


class SandwichBlock:
    """x += post_a(mixer(pre_a(x))); x += post_f(feed_forward(pre_f(x))): the sub-layer's output goes through a norm
    of its own before it joins the residual stream, so the sub-layers write into a scratch stream first."""

    def __init__(self, layer_spec):
        p = layer_spec.part
        self.pre_a, self.post_a = cb.build_part("norm", p("pre_mixer_norm")), cb.build_part("norm", p("post_mixer_norm"))
        self.pre_f, self.post_f = cb.build_part("norm", p("pre_ff_norm")), cb.build_part("norm", p("post_ff_norm"))
        self.mixer = cb.build_part("mixer", p("mixer"))
        self.ff = cb.build_part("feed_forward", p("feed_forward"))

    def parts(self):
        return [self.pre_a, self.mixer, self.post_a, self.pre_f, self.ff, self.post_f]

    def tensor_specs(self):
        return [t for part in self.parts() for t in part.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def bind(self, weights, ctx):
        for part in self.parts():
            part.bind(weights, ctx)

    def forward(self, x, batch, cache_view, write_cache=True):
        y = torch.zeros_like(x)
        self.mixer.forward(self.pre_a.forward(x), batch, cache_view, y, write_cache)
        x += self.post_a.forward(y).float()
        y = torch.zeros_like(x)
        self.ff.forward(self.pre_f.forward(x), batch, y)
        x += self.post_f.forward(y).float()
        return x


class ParallelBlock:
    """x += mixer(h) + feed_forward(h) with one h = norm(x) for both."""

    def __init__(self, layer_spec):
        self.norm = cb.build_part("norm", layer_spec.part("norm"))
        self.mixer = cb.build_part("mixer", layer_spec.part("mixer"))
        self.ff = cb.build_part("feed_forward", layer_spec.part("feed_forward"))

    def parts(self):
        return [self.norm, self.mixer, self.ff]

    def tensor_specs(self):
        return [t for part in self.parts() for t in part.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def bind(self, weights, ctx):
        for part in self.parts():
            part.bind(weights, ctx)

    def forward(self, x, batch, cache_view, write_cache=True):
        h = self.norm.forward(x)
        self.mixer.forward(h, batch, cache_view, x, write_cache)       # both add into the stream; h was taken before
        self.ff.forward(h, batch, x)
        return x


@dataclasses.dataclass(frozen=True)
class BlocksConfig:
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["max_position_embeddings"])

    def to_dict(self):
        return {"architectures": ["ToyBlocksForCausalLM"], **dataclasses.asdict(self)}

    def to_model_spec(self):
        H = self.hidden_size
        norm = lambda p, eps=1e-5: cb.PartSpec("rms_norm", {"size": H, "eps": eps}, p)
        ff = lambda p, inter: cb.PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": inter}, p)
        attn = lambda p, rot: cb.PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 32, "qk_norm_eps": 1e-6,
            "position": {"kind": "rotary_half_split", "theta": 1e4, "rotary_dim": rot}, "window": None}, p)
        layers = (
            cb.LayerSpec("toy_sandwich", {"pre_mixer_norm": norm("l0.n1"), "mixer": attn("l0.attn", 8),
                                          "post_mixer_norm": norm("l0.n2", 3e-5), "pre_ff_norm": norm("l0.n3"),
                                          "feed_forward": ff("l0.mlp", 80), "post_ff_norm": norm("l0.n4", 2e-5)}),
            cb.LayerSpec("toy_parallel", {"norm": norm("l1.n"), "mixer": attn("l1.attn", 32), "feed_forward": ff("l1.mlp", 96)}),
            cb.LayerSpec("pre_norm_residual", {"feed_forward_norm": norm("l2.n"), "feed_forward": ff("l2.mlp", 48)}),
        )
        return cb.ModelSpec("ToyBlocksForCausalLM", self.vocab_size, H, self.max_position_embeddings, "emb.weight",
                            layers, tuple(cb.ScheduleStep(i) for i in range(3)), norm("final"), "head.weight", False,
                            embedding_scale=H ** 0.5, logit_scale=0.25)


def plain_blocks(w, tokens, H):
    T = len(tokens)
    pos = list(range(T))
    x = plain.embedding(w["emb.weight"], tokens) * (H ** 0.5)

    def attention(h, pre, rot):
        q = plain.head_rms_norm(plain.linear(h, w[f"{pre}.q_proj.weight"]).view(T, 4, 32), w[f"{pre}.q_norm.weight"], 1e-6)
        k = plain.head_rms_norm(plain.linear(h, w[f"{pre}.k_proj.weight"]).view(T, 2, 32), w[f"{pre}.k_norm.weight"], 1e-6)
        v = plain.linear(h, w[f"{pre}.v_proj.weight"]).view(T, 2, 32)
        part = lambda t: torch.cat([plain.rotary_half_split(t[..., :rot], pos, 1e4), t[..., rot:]], dim=-1)
        return plain.linear(plain.causal_attention(part(q), part(k), v, 4, 2).reshape(T, 128), w[f"{pre}.o_proj.weight"])

    a = attention(plain.rms_norm(x, w["l0.n1.weight"], 1e-5), "l0.attn", 8)
    x = x + plain.rms_norm(a, w["l0.n2.weight"], 3e-5)
    f = plain.feed_forward(plain.rms_norm(x, w["l0.n3.weight"], 1e-5), w, "l0.mlp")
    x = x + plain.rms_norm(f, w["l0.n4.weight"], 2e-5)
    h = plain.rms_norm(x, w["l1.n.weight"], 1e-5)
    x = x + attention(h, "l1.attn", 32) + plain.feed_forward(h, w, "l1.mlp")
    x = x + plain.feed_forward(plain.rms_norm(x, w["l2.n.weight"], 1e-5), w, "l2.mlp")
    return plain.linear(plain.rms_norm(x, w["final.weight"], 1e-5), w["head.weight"]) * 0.25


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_blocks_scales_and_a_partly_rotated_head(tmp_path, dtype):
    cb.register_part("block", "toy_sandwich", SandwichBlock)
    cb.register_part("block", "toy_parallel", ParallelBlock)
    cb.register_architecture("ToyBlocksForCausalLM", BlocksConfig)
    try:
        cfg = BlocksConfig(vocab_size=400, hidden_size=72, max_position_embeddings=256)
        folder = cb.write_random_model(str(tmp_path / "blocks"), cfg, seed=12, dtype=dtype)
        _, w = plain.load_folder(folder)
        session = cb.InferenceSession().load_model(folder, max_context=256, dtype=dtype, max_batch=2)
        assert [g.steps for g in session.cache.kv_groups] == [[0, 1]]        # the third layer keeps nothing
        # weights a step reads: what the layers declare as matrices, plus the output matrix
        size = 4 if dtype == "float32" else 2
        per_layer = [(128 + 64 + 64) * 72 + 72 * 128 + 3 * 72 * 80, (128 + 64 + 64) * 72 + 72 * 128 + 3 * 72 * 96, 3 * 72 * 48]
        assert session.model.weight_bytes_read_per_step() == size * (sum(per_layer) + 400 * 72)
        import random
        rng = random.Random(6)
        reqs = [(f"b{i}", [rng.randrange(400) for _ in range(n)]) for i, n in enumerate([80, 7, 130])]
        want = {rid: plain_blocks(w, toks, 72) for rid, toks in reqs}
        tolerance = 2e-5 if dtype == "float32" else 2.5e-2
        runs = []
        for steps in (replay.whole(reqs), replay.tail(reqs), replay.batched(reqs, [50, 7, 1], 2), replay.chunked(reqs, 2, 3)):
            got = replay.run_in_process(session, steps)
            runs.append(got)
            for (rid, pos), row in got.items():
                ref = want[rid][pos]
                assert (row.double() - ref).abs().max() <= tolerance * ref.abs().max() + 1e-6, (rid, pos)
        if dtype == "float32":
            for got in runs[1:]:
                for key, row in got.items():
                    assert torch.equal(row, runs[0][key])
        assert session.cache.pages_held() == 0
    finally:
        cb.unregister_part("block", "toy_sandwich")
        cb.unregister_part("block", "toy_parallel")
        cb.unregister_architecture("ToyBlocksForCausalLM")
