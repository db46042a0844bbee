"""Sequences beyond 4,096 tokens against the plain implementation: a prompt of 4,160 tokens in one step (65 cache
pages; with head size 128 the tcgen05 prompt kernel walks up to 33 key tiles of 128), then 200 tokens one by one
past it (the split-context kernel over 66 to 69 pages), in 32-bit and in bfloat16.  The plain implementation takes
some ten seconds for the one sequence."""
import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
from helpers import TINY, SEEDS, random_tokens

pytestmark = pytest.mark.gpu

PROMPT, DECODED = 4160, 200
PLACES = [0, 1, 63, 64, 127, 128, 129, 1000, 2047, 2048, 3000, 4095, 4096, 4097, 4158, 4159]


@pytest.fixture(scope="module")
def long_case(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("long") / "model")
    cfg = cb.config_from_dict(dict(TINY["D"], max_position_embeddings=8192))
    cb.write_random_model(folder, cfg, SEEDS["D"], dtype="bfloat16")
    pcfg, w = plain.load_folder(folder)
    toks = random_tokens(pcfg["vocab_size"], PROMPT + DECODED, 4242)
    return folder, toks, plain.model_logits(pcfg, w, toks)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_prompt_of_4160_tokens_and_decoding_past_it(long_case, dtype, tol):
    folder, toks, want = long_case
    s = cb.InferenceSession().load_model(folder, max_context=PROMPT + DECODED, dtype=dtype, max_batch=2)
    slot = s.acquire()
    got = {}
    out = s.step([cb.StepEntry(slot, toks[:PROMPT], PLACES)]).double().cpu()
    for r, p in enumerate(PLACES):
        got[p] = out[r]
    for p in range(PROMPT, PROMPT + DECODED):
        got[p] = s.step([cb.StepEntry(slot, [toks[p]], [0])]).double().cpu()[0]
    s.release(slot)
    s.check_device_errors()
    worst = 0.0
    for p, row in got.items():
        scale = float(want[p].abs().max())
        err = float((row - want[p]).abs().max())
        worst = max(worst, err / scale)
        assert err <= tol * scale + 1e-6, f"{dtype} position {p}: |diff| {err:.3e} of {scale:.3e}"
    print(f"[4,160-token prompt + {DECODED} decoded, {dtype}] worst |diff| / max|logit| = {worst:.3e} (limit {tol:.1e})")
    # the same prompt in two steps (2,100 tokens, then 2,060 more on top of them): a run of many tokens over a long past
    slot = s.acquire()
    s.step([cb.StepEntry(slot, toks[:2100], [])])
    out = s.step([cb.StepEntry(slot, toks[2100:PROMPT], [p - 2100 for p in PLACES if p >= 2100])]).double().cpu()
    s.release(slot)
    for r, p in enumerate([p for p in PLACES if p >= 2100]):
        if dtype == "float32":
            assert torch.equal(out[r], got[p]), f"32-bit logits at {p} depend on the cut"
        else:
            assert float((out[r] - want[p]).abs().max()) <= tol * float(want[p].abs().max())
