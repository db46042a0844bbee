"""Replay on the GPU against the plain implementation: each request whole; with its last 32
tokens one by one; in batches of unequal lengths whose shorter requests end earlier, one
batch after another so that slots are used again.  In 32-bit and in bfloat16."""

import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
import replay
from helpers import TINY, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 40, 70, 128, 1, 33], "B": [1, 7, 23, 40, 150, 256, 64, 65],
           "C": [33, 64, 65, 300, 129, 2, 97], "D": [700, 129, 65, 260, 31]}

# float32: the engine and the exact (float64) evaluation of the same formulas differ by 32-bit
# rounding only.  bfloat16: activations are rounded to 8 significant bits at each store.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def requests_for(name):
    vocab = TINY[name]["vocab_size"]
    return [(f"r{i}", random_tokens(vocab, n, 100 * i + n)) for i, n in enumerate(LENGTHS[name])]


_plain_cache = {}


def plain_rows(model_dirs, name, stored):
    key = (name, stored)
    if key not in _plain_cache:
        cfg, w = plain.load_folder(model_dirs[key])
        _plain_cache[key] = {rid: plain.model_logits(cfg, w, toks) for rid, toks in requests_for(name)}
    return _plain_cache[key]


def session_for(model_dirs, name, dtype, max_batch=8, max_tokens=None):
    stored = "float32" if dtype == "float32" else "bfloat16"
    return cb.InferenceSession().load_model(model_dirs[(name, stored)], max_context=4096, dtype=dtype,
                                            max_batch=max_batch, max_tokens=max_tokens)


def check(got, want_rows, dtype, what):
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = want_rows[rid][pos]
        scale = float(ref.abs().max())
        err = float((row.double() - ref).abs().max())
        worst = max(worst, err / scale)
        assert err <= TOL[dtype] * scale + 1e-6, f"{what}: request {rid} position {pos}: |diff| {err:.3e} of {scale:.3e}"
    print(f"[{what}] worst |diff| / max|logit| = {worst:.3e} (limit {TOL[dtype]:.1e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_tail_and_batched_agree_with_plain(model_dirs, name, dtype):
    stored = "float32" if dtype == "float32" else "bfloat16"
    want = plain_rows(model_dirs, name, stored)
    reqs = requests_for(name)
    s = session_for(model_dirs, name, dtype, max_batch=3)
    whole = replay.run_in_process(s, replay.whole(reqs))
    assert len(whole) == sum(len(t) for _, t in reqs)
    check(whole, want, dtype, f"{name} {dtype} whole")
    tail = replay.run_in_process(s, replay.tail(reqs))
    assert set(tail) == set(whole)
    check(tail, want, dtype, f"{name} {dtype} tail-32")
    prompt_lens = [max(1, len(t) - (7 * i) % 40) for i, (_, t) in enumerate(reqs)]
    bat = replay.run_in_process(s, replay.batched(reqs, prompt_lens, 3))      # 3 slots, 7-8 requests
    check(bat, want, dtype, f"{name} {dtype} batched")
    assert s.cache.slots.free_count == 3 and s.cache.pages_held() == 0
    # how the tokens were cut into steps and what else was in the batch changes nothing beyond rounding
    for key, row in tail.items():
        if dtype == "float32":
            assert torch.equal(row, whole[key]), f"{name}: tail-32 differs from whole at {key}"
        else:
            assert (row - whole[key]).abs().max() <= TOL[dtype] * whole[key].abs().max()
    for key, row in bat.items():
        if dtype == "float32":
            assert torch.equal(row, whole[key]), f"{name}: batched differs from whole at {key}"
        else:
            assert (row - whole[key]).abs().max() <= TOL[dtype] * whole[key].abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_sequences_that_go_on_by_several_tokens_and_requests_that_join(model_dirs, name, dtype):
    """Steps whose sequences have unequal pasts AND bring unequal runs of 2 to 40 new tokens, three slots over
    two batches; and one running batch that requests join while the others decode.  Both against the plain
    implementation, and in 32-bit bitwise equal to each request run whole."""
    stored = "float32" if dtype == "float32" else "bfloat16"
    want = plain_rows(model_dirs, name, stored)
    reqs = requests_for(name)[:6]
    s = session_for(model_dirs, name, dtype, max_batch=3)
    whole = replay.run_in_process(s, replay.whole(reqs))
    steps = replay.chunked(reqs, 3, seed=5)
    assert any(len(st["entries"]) >= 2 and len({len(e["tokens"]) for e in st["entries"]}) >= 2 for st in steps[1:])
    cut = replay.run_in_process(s, steps)
    assert set(cut) == set(whole)
    check(cut, want, dtype, f"{name} {dtype} chunked")
    reqs3 = reqs[:3]
    lens = [max(1, len(t) - 20) for _, t in reqs3]
    joined = replay.run_in_process(s, replay.joining(reqs3, lens, every=4))
    check(joined, want, dtype, f"{name} {dtype} joining")
    assert s.cache.slots.free_count == 3 and s.cache.pages_held() == 0
    for got in (cut, joined):
        for key, row in got.items():
            if dtype == "float32":
                assert torch.equal(row, whole[key]), f"{name}: logits at {key} depend on the cut"
            else:
                assert (row - whole[key]).abs().max() <= TOL[dtype] * whole[key].abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model_dirs, dtype):
    """A 3-token prompt, then 250 tokens one by one (across four cache pages); and the first
    tokens of sequences: prompts of one token, logits at position 0."""
    stored = "float32" if dtype == "float32" else "bfloat16"
    cfg, w = plain.load_folder(model_dirs[("C", stored)])
    toks = random_tokens(cfg["vocab_size"], 253, 9)
    want = {"long": plain.model_logits(cfg, w, toks)}
    s = session_for(model_dirs, "C", dtype, max_batch=4)
    got = replay.run_in_process(s, replay.batched([("long", toks)], [3], 1))
    assert len(got) == 251
    check(got, want, dtype, f"C {dtype} long decoding")
    firsts = [(f"f{i}", [t]) for i, t in enumerate([0, 5, 776, 300])]
    want = {rid: plain.model_logits(cfg, w, t) for rid, t in firsts}
    got = replay.run_in_process(s, replay.batched(firsts, [1, 1, 1, 1], 4))
    check(got, want, dtype, f"C {dtype} first tokens")
    got1 = replay.run_in_process(s, replay.whole(firsts))
    for k in got:
        if dtype == "float32":
            assert torch.equal(got[k], got1[k])
        else:       # a step of single tokens and a step of prompts run different kernels: rounding only
            assert (got[k] - got1[k]).abs().max() <= TOL[dtype] * got1[k].abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reused_slot_does_not_see_what_it_held(model_dirs, dtype):
    """Fill every slot with long sequences, give them back, then run short ones in the same
    slots: keys and values past a slot's length belong to the earlier tenant."""
    stored = "float32" if dtype == "float32" else "bfloat16"
    cfg, w = plain.load_folder(model_dirs[("B", stored)])
    vocab = cfg["vocab_size"]
    s = session_for(model_dirs, "B", dtype, max_batch=2, max_tokens=2 * 256)
    long = [(f"l{i}", random_tokens(vocab, 200 + i, 50 + i)) for i in range(2)]
    replay.run_in_process(s, replay.batched(long, [190, 180], 2))
    short = [(f"s{i}", random_tokens(vocab, 20 + 30 * i, 70 + i)) for i in range(2)]
    got = replay.run_in_process(s, replay.batched(short, [10, 25], 2))
    want = {rid: plain.model_logits(cfg, w, t) for rid, t in short}
    check(got, want, dtype, f"B {dtype} reused slots")
    fresh = session_for(model_dirs, "B", dtype, max_batch=2, max_tokens=2 * 256)
    again = replay.run_in_process(fresh, replay.batched(short, [10, 25], 2))
    for k in got:
        assert torch.equal(got[k], again[k]), f"a reused slot changed the logits at {k}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, dtype):
    """The same through bin/trace_run as a separate process: its answers equal the in-process
    session's bit for bit, and steps that want nothing write no file."""
    stored = "float32" if dtype == "float32" else "bfloat16"
    name = "B"
    reqs = requests_for(name)[:5]
    steps = replay.batched(reqs, [1, 5, 20, 33, 100], 3)
    steps[1]["entries"][0]["want"] = []                       # a step entry that wants nothing
    vocab = TINY[name]["vocab_size"]
    got = replay.run_trace_run(model_dirs[(name, stored)], dtype, steps, vocab)
    want = plain_rows(model_dirs, name, stored)
    check(got, want, dtype, f"{name} {dtype} bin/trace_run")
    s = session_for(model_dirs, name, dtype, max_batch=3)
    same = replay.run_in_process(s, steps)
    assert set(same) == set(got)
    for k in got:
        assert torch.equal(got[k], same[k])


def test_step_refuses_what_it_cannot_run(model_dirs):
    s = session_for(model_dirs, "A", "float32", max_batch=2)
    a = s.acquire()
    with pytest.raises(cb.CitlaliError, match="out of vocab range"):
        s.step([cb.StepEntry(a, [512], [0])])
    with pytest.raises(cb.CitlaliError, match="was not acquired"):
        s.step([cb.StepEntry(1, [1], [0])])
    with pytest.raises(cb.CitlaliError, match="brings no tokens"):
        s.step([cb.StepEntry(a, [], [])])
    with pytest.raises(cb.CitlaliError, match="exceed max_context"):
        s.step([cb.StepEntry(a, [1] * 129, [])])
    with pytest.raises(cb.CitlaliError, match="place 3 of 2"):
        s.step([cb.StepEntry(a, [1, 2], [3])])
    s.step([cb.StepEntry(a, [1, 2], [])])
    b = s.acquire()
    with pytest.raises(cb.CitlaliError, match="twice in one step"):
        s.step([cb.StepEntry(a, [3], [0]), cb.StepEntry(a, [3], [0])])
    assert s.cache.length(a) == 2                              # refused steps changed nothing
    s.release(a); s.release(b)


def test_a_batch_of_forty_requests_of_very_unequal_lengths(tmp_path):
    """Forty requests decode together, three of them ten times longer than the rest: with one block a (row,
    key/value head) the decode attention deals the long rows' pages to several blocks by length and merges their
    results.  The batch, the long requests alone and the plain implementation agree."""
    cfg = cb.config_from_dict(dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=8,
                                   num_key_value_heads=4, head_dim=32, intermediate_size=208, vocab_size=600, rope_theta=1e4,
                                   rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2048))
    folder = cb.write_random_model(str(tmp_path / "forty"), cfg, 77, dtype="bfloat16")
    pcfg, w = plain.load_folder(folder)
    lengths = [20 + (37 * i) % 280 for i in range(37)] + [1500, 900, 1210]
    reqs = [(f"q{i}", random_tokens(600, n, 900 + i)) for i, n in enumerate(lengths)]
    want = {rid: plain.model_logits(pcfg, w, toks) for rid, toks in reqs}
    s = cb.InferenceSession().load_model(folder, max_context=2048, dtype="bfloat16", max_batch=40)
    prompt_lens = [len(t) - 6 for _, t in reqs]
    together = replay.run_in_process(s, replay.batched(reqs, prompt_lens, 40))
    check(together, want, "bfloat16", "forty together")
    assert len(together) == 40 * 7
    alone = replay.run_in_process(s, replay.batched(reqs[-3:], prompt_lens[-3:], 1))
    for key, row in alone.items():
        assert (row - together[key]).abs().max() <= TOL["bfloat16"] * together[key].abs().max()
    assert s.cache.pages_held() == 0
