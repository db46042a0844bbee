"""Generation through the entry points (Python and command line) against the plain loop."""
import json
import os
import subprocess
import sys

import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
from helpers import TINY, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# A logit of the engine differs from the plain one by at most TOL of the row's largest |logit| (the replay
# tests hold it to that), so where the plain top-2 margin exceeds twice that the argmax cannot differ.
NEED = {"float32": 2 * 2e-5, "bfloat16": 2 * 2.5e-2}
# The share of generated tokens that such a margin lets compare: nearly all in 32-bit; in bfloat16 about
# half (the top-2 gap of ~1000 near-Gaussian logits exceeds 5 % of the largest for about 55 % of rows).
FLOOR = {"float32": 0.8, "bfloat16": 0.35}


def compare_greedy(cfg, w, prompts, results, dtype):
    """Every generated token against the plain argmax on the very tokens the engine has produced so far.
    Returns (compared, total)."""
    compared = total = 0
    for r, (prompt, res) in enumerate(zip(prompts, results)):
        seq = list(prompt)
        for k, t in enumerate(res.tokens):
            logits = plain.model_logits(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            total += 1
            if float(top2[0] - top2[1]) > NEED[dtype] * float(logits.abs().max()):
                compared += 1
                assert t == plain.greedy(logits), f"request {r}: generated token {k} differs from the plain argmax"
            seq.append(t)
    return compared, total


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,steps", [("A", [5, 11, 17], 8), ("B", [1, 7, 23, 40], 12), ("C", [3, 30, 64], 12)])
def test_greedy_generation_matches_the_plain_loop(model_dirs, name, lengths, steps, dtype):
    stored = "float32" if dtype == "float32" else "bfloat16"
    cfg, w = plain.load_folder(model_dirs[(name, stored)])
    prompts = [random_tokens(cfg["vocab_size"], n, 7 + n) for n in lengths]
    session = cb.InferenceSession().load_model(model_dirs[(name, stored)], max_context=128, dtype=dtype, max_batch=4)
    streamed = []
    results = session.generate(prompts, cb.GenerationOptions(max_new_tokens=steps, max_context=128, stop_ids=[]),
                               on_token=lambda r, t: streamed.append((r, t)))
    for r, res in enumerate(results):
        assert res.generated_tokens == steps == len(res.tokens) and res.stop_reason == cb.StopReason.MAX_NEW_TOKENS
        assert [t for rr, t in streamed if rr == r] == res.tokens
    compared, total = compare_greedy(cfg, w, prompts, results, dtype)
    print(f"[{name} {dtype}] {compared} of {total} generated tokens had a margin that allows comparing")
    assert compared >= FLOOR[dtype] * total, f"only {compared} of {total} tokens could be compared"
    if not cfg.get("tie_word_embeddings"):
        # an untied random model does not simply repeat its last token (a tied one does: its output matrix is
        # its embedding), so agreeing with the plain loop says something about the layers
        assert any(t != p[-1] for p, res in zip(prompts, results) for t in res.tokens[:1])
    assert session.cache.slots.free_count == 4 and session.cache.pages_held() == 0
    # one request alone gives the same tokens as in the batch
    alone = session.generate([prompts[1]], cb.GenerationOptions(max_new_tokens=steps, max_context=128, stop_ids=[]))
    assert alone[0].tokens == results[1].tokens
    # the reference's names for one sequence
    seen = []
    once = session.generate_once_result(prompts[1], cb.GenerationOptions(max_new_tokens=steps, max_context=128, stop_ids=[]),
                                        on_token=seen.append)
    assert once.tokens == results[1].tokens == seen and once.generated_tokens == steps
    assert session.generate_once(prompts[0], cb.GenerationOptions(max_new_tokens=3, max_context=128, stop_ids=[])) == results[0].tokens[:3]


def test_head_sizes_the_single_token_kernel_refuses_step_without_graphs(tmp_path):
    """Head sizes 20 and 36 (even, no multiple of 8): in bfloat16 their attention runs the generic kernel, whose
    launch is sized from the host's lengths, so the session must not capture the decode step; generation goes
    through plain steps and agrees with the plain loop."""
    for case, (hidden, heads, kv, d) in enumerate([(72, 2, 1, 36), (80, 4, 2, 20)]):
        cfg = cb.config_from_dict(dict(
            architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=hidden, num_attention_heads=heads,
            num_key_value_heads=kv, head_dim=d, intermediate_size=176, vocab_size=600, rope_theta=1e4, rms_norm_eps=1e-6,
            tie_word_embeddings=False, max_position_embeddings=256))
        folder = str(tmp_path / f"m{case}")
        cb.write_random_model(folder, cfg, 70 + case, dtype="bfloat16")
        pcfg, w = plain.load_folder(folder)
        prompts = [random_tokens(600, n, 3 + n) for n in (70, 5, 33)]
        for dtype in ("bfloat16", "float32"):
            session = cb.InferenceSession().load_model(folder, max_context=256, dtype=dtype, max_batch=4)
            assert session.runner is None
            results = session.generate(prompts, cb.GenerationOptions(max_new_tokens=10, max_context=256, stop_ids=[]))
            compared, total = compare_greedy(pcfg, w, prompts, results, dtype)
            assert compared >= FLOOR[dtype] * total


def test_steps_issued_back_to_back_equal_steps_issued_one_by_one(model_dirs):
    """The graph runner's ``launch`` returns before the step has run.  Forty steps issued without waiting in
    between, each fed on the device with the token the step before sampled, give the tokens that the same steps
    give when the host waits for each: no step's inputs are overwritten before it has read them."""
    cfg = TINY["D"]
    prompts = [random_tokens(cfg["vocab_size"], n, 80 + n) for n in (60, 5, 100, 63)]
    session = cb.InferenceSession().load_model(model_dirs[("D", "bfloat16")], max_context=512, dtype="bfloat16", max_batch=4)
    runner = session.runner
    assert runner is not None

    def run(wait):
        slots = [session.acquire() for _ in prompts]
        first = session.prefill(slots, prompts, 0.0, [])
        runner.launch(slots, first, 0.0, [])
        seen = [runner.out_tokens[:4].clone()]
        for _ in range(40):
            if wait:
                torch.cuda.synchronize()
            runner.feed_back(4)
            runner.launch(slots, None, 0.0, [])
            seen.append(runner.out_tokens[:4].clone())
        torch.cuda.synchronize()
        for s in slots:
            session.release(s)
        return torch.stack(seen).tolist()

    assert run(wait=False) == run(wait=True)
    # the same 41 steps through the loop, which reads every token back
    res = session.generate(prompts, cb.GenerationOptions(max_new_tokens=42, max_context=512, stop_ids=[]))
    assert [list(col) for col in zip(*run(wait=False))] == [r.tokens[1:] for r in res]


def test_stop_tokens_early_finishers_and_many_batches(model_dirs):
    cfg, w = plain.load_folder(model_dirs[("C", "float32")])
    session = cb.InferenceSession().load_model(model_dirs[("C", "float32")], max_context=64, dtype="float32", max_batch=2)
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (3, 9, 4, 30, 6)]
    free = session.generate(prompts, cb.GenerationOptions(max_new_tokens=10, max_context=64, stop_ids=[]))
    assert all(r.generated_tokens == 10 for r in free)
    stop = free[1].tokens[4]
    res = session.generate(prompts, cb.GenerationOptions(max_new_tokens=10, max_context=64, stop_ids=[stop]))
    for f, r in zip(free, res):
        if stop in f.tokens:
            k = f.tokens.index(stop)
            assert r.tokens == f.tokens[:k] and r.stop_reason == cb.StopReason.EOS and r.generated_tokens == k
        else:
            assert r.tokens == f.tokens and r.stop_reason == cb.StopReason.MAX_NEW_TOKENS
    assert res[1].stop_reason == cb.StopReason.EOS
    # config C names eos ids 5 and 9: they are the default stop set
    assert session.model.spec.stop_token_ids == (5, 9)
    limited = session.generate([prompts[3]], cb.GenerationOptions(max_new_tokens=50, max_context=40, stop_ids=[]))
    assert limited[0].stop_reason == cb.StopReason.CONTEXT_LIMIT and limited[0].generated_tokens == 10
    assert limited[0].tokens == free[3].tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_follows_the_plain_cdf(model_dirs, dtype):
    stored = "float32" if dtype == "float32" else "bfloat16"
    cfg, w = plain.load_folder(model_dirs[("B", stored)])
    prompts = [random_tokens(cfg["vocab_size"], n, 90 + n) for n in (1, 7, 23, 40)]
    session = cb.InferenceSession().load_model(model_dirs[("B", stored)], max_context=128, dtype=dtype, max_batch=4)
    opts = cb.GenerationOptions(max_new_tokens=12, max_context=128, temperature=0.8, seed=1234, stop_ids=[])
    res = session.generate(prompts, opts)
    again = session.generate(prompts, opts)
    assert [r.tokens for r in res] == [r.tokens for r in again]                     # a fixed seed repeats
    other = session.generate(prompts, cb.GenerationOptions(max_new_tokens=12, max_context=128, temperature=0.8,
                                                           seed=99, stop_ids=[]))
    assert [r.tokens for r in res] != [r.tokens for r in other]
    alone = session.generate(prompts[2:3], opts)                                     # request index 0 now
    slack = 1e-5 if dtype == "float32" else 3e-2
    for r, (prompt, out) in enumerate(zip(prompts, res)):
        seq = list(prompt)
        for k, t in enumerate(out.tokens):
            cdf = plain.temperature_cdf(plain.model_logits(cfg, w, seq)[-1], 0.8)
            u = cb.uniform(1234, r, k)
            lo = float(cdf[t - 1]) if t > 0 else 0.0
            assert lo - slack <= u <= float(cdf[t]) + slack, f"request {r} token {k}: u={u} outside [{lo}, {float(cdf[t])}]"
            seq.append(t)
    assert len(alone[0].tokens) == 12


def test_command_line(model_dirs, tmp_path):
    cli = os.path.join(ROOT, "bin", "citlali_cli")
    model = model_dirs[("A", "float32")]
    prompts = [[1, 2, 3, 4, 5], [9, 8, 7]]
    out = subprocess.run([sys.executable, cli, "--model", model, "--prompt-ids", "1,2,3,4,5", "--prompt-ids", "9,8,7",
                          "--max-new-tokens", "6", "--ctx", "64", "--dtype", "float32", "--json"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    data = json.loads(out.stdout)
    session = cb.InferenceSession().load_model(model, max_context=64, dtype="float32", max_batch=8)
    want = session.generate(prompts, cb.GenerationOptions(max_new_tokens=6, max_context=64))
    assert [r["tokens"] for r in data["results"]] == [r.tokens for r in want]
    assert all(r["stop_reason"] == "max_new_tokens" for r in data["results"])
    assert "[stats] tokens=12" in out.stderr and "stop=max_new_tokens,max_new_tokens" in out.stderr
    info = subprocess.run([sys.executable, cli, "--model", model, "--info"], capture_output=True, text=True, timeout=120)
    assert info.returncode == 0 and "hidden_size: 64" in info.stdout and "vocab_size: 512" in info.stdout
    bad = subprocess.run([sys.executable, cli, "--model", model, "--frobnicate"], capture_output=True, text=True, timeout=120)
    assert bad.returncode == 1 and "unknown argument: --frobnicate" in bad.stderr


def test_long_generation_repeats_bit_for_bit_with_and_without_graphs(model_dirs):
    """300 decode steps at batch 4, twice through the replayed graph and once with plain launches: every kernel
    waits for its predecessor before touching shared buffers, so nothing may differ."""
    cfg = TINY["D"]
    prompts = [random_tokens(cfg["vocab_size"], n, 60 + n) for n in (5, 90, 31, 200)]
    opts = cb.GenerationOptions(max_new_tokens=300, max_context=1024, stop_ids=[])
    session = cb.InferenceSession().load_model(model_dirs[("D", "bfloat16")], max_context=1024, dtype="bfloat16", max_batch=4)
    assert session.runner is not None
    first = [r.tokens for r in session.generate(prompts, opts)]
    second = [r.tokens for r in session.generate(prompts, opts)]
    assert first == second and all(len(t) == 300 for t in first)
    plain_launches = cb.InferenceSession()
    plain_launches.use_graphs = False
    plain_launches.load_model(model_dirs[("D", "bfloat16")], max_context=1024, dtype="bfloat16", max_batch=4)
    assert plain_launches.runner is None
    assert [r.tokens for r in plain_launches.generate(prompts, opts)] == first
