"""The benchmark's layer sizes (hidden 4096, 32 / 8 heads of 128, feed-forward 12288, vocabulary 151936), and those
of a second size of the family (hidden 5120, 40 / 8 heads, feed-forward 17408), with two
layers and random weights: the bfloat16 engine, whose kernels take their production shapes here (both forms of the
tensor-core product with K splits over clusters, the product on pairs of SMs, the tcgen05 prompt attention, the cluster decode attention, the wide
argmax), against the 32-bit engine on the same weight values; and the 32-bit engine against itself under another
way of cutting the tokens.  The plain implementation runs at these layer sizes too, with a vocabulary of 8,192
(its float64 copy of the real one would take 10 GB): both engines against it on a model folder."""
import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
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


@pytest.mark.parametrize("batch", [8, 64])
def test_replayed_decode_at_batch_8_and_64_equals_plain_steps(batch):
    """The captured decode step at the batch sizes the benchmark runs (at 64 the swapped product takes its widest
    tile and decode attention one block per sequence and head group) against ``session.step`` issued one by one:
    the same logits bit for bit and the same tokens, for unequal prompts, over several steps."""
    cfg = cb.config_from_dict(dict(SHAPE))
    s = cb.InferenceSession().load_random(cfg, seed=7, max_context=512, dtype="bfloat16", max_batch=batch, gain_spread=0.1)
    assert s.runner is not None
    vocab = SHAPE["vocab_size"]
    prompts = [random_tokens(vocab, 1 + (37 * i) % 150, 500 + i) for i in range(batch)]

    def run(with_graph):
        slots = [s.acquire() for _ in prompts]
        logits = s.step([cb.StepEntry(sl, p, [len(p) - 1]) for sl, p in zip(slots, prompts)])
        toks = s.sampler.sample(logits, 0.0, [])
        seen_tokens, seen_logits = [list(toks)], []
        for _ in range(5):
            if with_graph:
                s.runner.launch(slots, toks, 0.0, [])
                toks = s.runner.read_tokens(batch)
                seen_logits.append(s.runner.logits[(batch, True)].clone())
            else:
                logits = s.step([cb.StepEntry(sl, [t], [0]) for sl, t in zip(slots, toks)])
                toks = s.sampler.sample(logits, 0.0, [])
                seen_logits.append(logits.clone())
            seen_tokens.append(list(toks))
        for sl in slots:
            s.release(sl)
        s.check_device_errors()
        return seen_tokens, seen_logits

    graph_tokens, graph_logits = run(True)
    plain_tokens, plain_logits = run(False)
    assert graph_tokens == plain_tokens
    for a, b in zip(graph_logits, plain_logits):
        assert torch.equal(a, b)


def test_production_layer_sizes_against_the_plain_implementation(tmp_path):
    """Two layers of the benchmark's sizes (hidden 4096, 32 / 8 heads of 128, feed-forward 12288) written as a model
    folder with a vocabulary of 8,192, loaded by both engines and by the plain implementation (float64): prompts of
    unequal lengths in one step of 647 rows, then tokens one by one."""
    shape = dict(SHAPE, vocab_size=8192)
    cfg = cb.config_from_dict(shape)
    folder = str(tmp_path / "model")
    cb.write_random_model(folder, cfg, 77, dtype="bfloat16")
    pcfg, w = plain.load_folder(folder)
    lengths, decoded = [300, 17, 130, 200], 4
    toks = [random_tokens(8192, n + decoded, 900 + n) for n in lengths]
    want = [plain.model_logits(pcfg, w, t) for t in toks]
    del w
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 2.5e-2)):
        s = cb.InferenceSession().load_model(folder, max_context=512, dtype=dtype, max_batch=4)
        slots = [s.acquire() for _ in toks]
        tail = 8
        out = s.step([cb.StepEntry(sl, t[:n], list(range(max(0, n - tail), n))) for sl, t, n in zip(slots, toks, lengths)])
        out = out.double().cpu()
        got, r = [], 0
        for b, n in enumerate(lengths):
            for p in range(max(0, n - tail), n):
                got.append((b, p, out[r])); r += 1
        for j in range(decoded):
            out = s.step([cb.StepEntry(sl, [t[n + j]], [0]) for sl, t, n in zip(slots, toks, lengths)]).double().cpu()
            for b, n in enumerate(lengths):
                got.append((b, n + j, out[b]))
        s.check_device_errors()
        worst = 0.0
        for b, p, row in got:
            scale = float(want[b][p].abs().max())
            err = float((row - want[b][p]).abs().max())
            worst = max(worst, err / scale)
            assert err <= tol * scale + 1e-6, f"{dtype} sequence {b} position {p}: |diff| {err:.3e} of {scale:.3e}"
        print(f"[production layer sizes, {dtype}] worst |diff| / max|logit| = {worst:.3e} (limit {tol:.1e})")
        del s
        torch.cuda.empty_cache()
