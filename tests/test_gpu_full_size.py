"""The benchmark's layer sizes (hidden 4096, 32 / 8 heads of 128, feed-forward 12288, vocabulary 151936), and those
of a second size of the family (hidden 5120, 40 / 8 heads, feed-forward 17408), with two
layers and random weights: the bfloat16 engine, whose kernels take their production shapes here (both forms of the
tensor-core product with K splits over clusters, the product on pairs of SMs, the tcgen05 prompt attention, the cluster decode attention, the wide
argmax), against the 32-bit engine on the same weight values; and the 32-bit engine against itself under another
way of cutting the tokens.  No plain-implementation run at this size: the 32-bit engine is checked against it on
the tiny configurations."""
import pytest
import torch

import citlali_b200 as cb
from citlali_b200 import ops
from helpers import random_tokens

pytestmark = pytest.mark.gpu

SHAPE = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=4096, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6,
             rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)


# another size of the family: 40 query heads on 8 key/value heads (groups of five), widths that are no power of two
OTHER = dict(hidden_size=5120, num_attention_heads=40, intermediate_size=17408)


@pytest.fixture(scope="module", params=["benchmark sizes", "hidden 5120, groups of five"])
def sessions(request):
    shape = dict(SHAPE)
    if request.param != "benchmark sizes":
        shape.update(OTHER)
    cfg = cb.config_from_dict(shape)
    s32 = cb.InferenceSession().load_random(cfg, seed=5, max_context=1024, dtype="float32", stored_dtype="bfloat16",
                                            max_batch=4, gain_spread=0.1)
    s16 = cb.InferenceSession().load_random(cfg, seed=5, max_context=1024, dtype="bfloat16", max_batch=4, gain_spread=0.1)
    return s32, s16, shape


def run(session, requests, cuts, want_tail):
    """Each request: its tokens cut at `cuts` (first step up to the cut, then one by one); logits of the last
    `want_tail` positions."""
    out = {}
    slots = {rid: session.acquire() for rid, _ in requests}
    first = [cb.StepEntry(slots[rid], toks[:cut], [p for p in range(max(0, len(toks) - want_tail), cut)])
             for (rid, toks), cut in zip(requests, cuts)]
    logits = session.step(first).float().cpu()
    r = 0
    for (rid, toks), cut in zip(requests, cuts):
        for p in range(max(0, len(toks) - want_tail), cut):
            out[(rid, p)] = logits[r]; r += 1
    pos = {rid: cut for (rid, _), cut in zip(requests, cuts)}
    live = [(rid, toks) for (rid, toks) in requests if pos[rid] < len(toks)]
    while live:
        entries = [cb.StepEntry(slots[rid], [toks[pos[rid]]], [0] if pos[rid] >= len(toks) - want_tail else [])
                   for rid, toks in live]
        logits = session.step(entries).float().cpu()
        r = 0
        for rid, toks in live:
            if pos[rid] >= len(toks) - want_tail:
                out[(rid, pos[rid])] = logits[r]; r += 1
            pos[rid] += 1
        live = [(rid, toks) for rid, toks in live if pos[rid] < len(toks)]
    for s in slots.values():
        session.release(s)
    session.check_device_errors()
    return out


def test_production_shapes_agree_with_the_32_bit_path(sessions):
    s32, s16, shape = sessions
    vocab = SHAPE["vocab_size"]
    requests = [("a", random_tokens(vocab, 300, 1)), ("b", random_tokens(vocab, 17, 2)), ("c", random_tokens(vocab, 130, 3)),
                ("d", random_tokens(vocab, 200, 4))]
    # 647 rows in the first step: the gate/up product of that many rows runs on pairs of SMs where the device has them
    if ops.gemm_tc_pair_plan(647, 2 * shape["intermediate_size"], shape["hidden_size"])["pairs"] >= 74:
        assert ops.gemm_tc_runs_on_pairs(647, 2 * shape["intermediate_size"], shape["hidden_size"], "cuda:0", swiglu=True)
    whole32 = run(s32, requests, [300, 17, 130, 200], 8)
    cut32 = run(s32, requests, [268, 1, 129, 180], 8)             # other cuts: the last tokens one by one
    assert set(whole32) == set(cut32) and len(whole32) == 32
    for key in whole32:
        assert torch.equal(whole32[key], cut32[key]), f"32-bit logits depend on the cut at {key}"
    whole16 = run(s16, requests, [300, 17, 130, 200], 8)
    cut16 = run(s16, requests, [268, 1, 129, 180], 8)
    worst = 0.0
    for key, ref in whole32.items():
        scale = float(ref.abs().max())
        for got in (whole16[key], cut16[key]):
            err = float((got - ref).abs().max())
            worst = max(worst, err / scale)
            assert err <= 2.5e-2 * scale, f"bfloat16 differs from 32-bit at {key}: {err:.3e} of {scale:.3e}"
    print(f"[hidden {shape['hidden_size']}] worst bfloat16 - float32 |diff| / max|logit| = {worst:.3e}")


def test_replayed_decode_steps_equal_plain_steps_at_production_shapes(sessions):
    """Greedy generation through the CUDA-graph decode runner against the same steps issued one by one."""
    _, s16, _ = sessions
    vocab = SHAPE["vocab_size"]
    prompts = [random_tokens(vocab, n, 10 + n) for n in (70, 3, 129)]
    res = s16.generate(prompts, cb.GenerationOptions(max_new_tokens=6, max_context=1024, stop_ids=[]))
    assert s16.runner is not None
    # the same by hand with the step function and the device argmax
    slots = [s16.acquire() for _ in prompts]
    logits = s16.step([cb.StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    toks = s16.sampler.sample(logits, 0.0, [])
    outs = [[t] for t in toks]
    for _ in range(5):
        logits = s16.step([cb.StepEntry(s, [o[-1]], [0]) for s, o in zip(slots, outs)])
        for o, t in zip(outs, s16.sampler.sample(logits, 0.0, [])):
            o.append(t)
    for s in slots:
        s16.release(s)
    assert [r.tokens for r in res] == outs


def test_generation_at_production_shapes_repeats_bit_for_bit(sessions):
    _, s16, _ = sessions
    vocab = SHAPE["vocab_size"]
    prompts = [random_tokens(vocab, n, 30 + n) for n in (200, 64, 1, 333)]
    opts = cb.GenerationOptions(max_new_tokens=96, max_context=1024, stop_ids=[], temperature=0.7, seed=3)
    a = [r.tokens for r in s16.generate(prompts, opts)]
    b = [r.tokens for r in s16.generate(prompts, opts)]
    assert a == b and all(len(t) == 96 for t in a)
