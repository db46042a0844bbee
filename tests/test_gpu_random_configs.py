"""Configurations drawn at random (fixed seed): head sizes 16 to 256 in steps of 16 and two that are no
multiple of 8 (20, 36: bfloat16 then runs the generic attention kernels), one to four key/value
heads, groups of one to eight query heads, widths that are no multiple of 8 (68, 100: bfloat16 products then
run on the CUDA cores), intermediate sizes that are no multiple of 16 (100, 330: gate and up stacked whole,
the gate as a kernel of its own) and vocabularies that are no power of
two, one to three layers, tied or untied output matrix.  Two prompts of unequal lengths in one step, then
three tokens each one by one, in 32-bit and in bfloat16, against the plain implementation."""
import random

import pytest

import citlali_b200 as cb
import plain_qwen3 as plain
from citlali_b200.engine.step import StepEntry

pytestmark = pytest.mark.gpu


def draw(rng):
    nkv = rng.choice([1, 2, 3, 4])
    cfg = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=rng.choice([1, 2, 3]),
               hidden_size=rng.choice([64, 68, 72, 96, 100, 120, 128, 200, 256, 264]),
               num_attention_heads=nkv * rng.choice([1, 2, 3, 4, 5, 8]), num_key_value_heads=nkv,
               head_dim=rng.choice([16, 20, 32, 36, 48, 64, 80, 96, 112, 128, 256]),
               intermediate_size=rng.choice([80, 96, 100, 144, 208, 256, 330, 512, 1040]),
               vocab_size=rng.choice([300, 512, 777, 1000, 1536, 2049]), rope_theta=rng.choice([1e4, 1e6]),
               rms_norm_eps=rng.choice([1e-6, 1e-5]), tie_word_embeddings=rng.choice([True, False]),
               max_position_embeddings=1024, hidden_act="silu", attention_bias=False)
    lens = [rng.choice([1, 5, 47, 48, 63, 64, 65, 130, 200, 300]), rng.choice([2, 33, 100, 129, 257])]
    return cfg, lens


def test_the_draws_cover_the_odd_sizes():
    seen = [draw(random.Random(1000 + case))[0] for case in range(14)]
    assert any(c["head_dim"] % 8 for c in seen) and any(c["hidden_size"] % 8 for c in seen)
    assert any(c["intermediate_size"] % 16 for c in seen)


@pytest.mark.parametrize("case", range(14))
def test_random_configuration(case, tmp_path):
    rng = random.Random(1000 + case)
    cfgd, lens = draw(rng)
    cfg = cb.config_from_dict(dict(cfgd))
    cb.write_random_model(str(tmp_path), cfg, 100 + case, dtype="bfloat16")
    pcfg, w = plain.load_folder(str(tmp_path))
    decoded = 3
    toks = [[rng.randrange(cfg.vocab_size) for _ in range(n + decoded)] for n in lens]
    want = [plain.model_logits(pcfg, w, t) for t in toks]
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 2.5e-2)):
        s = cb.InferenceSession().load_model(str(tmp_path), max_context=512, dtype=dtype, max_batch=2)
        slots = [s.acquire(), s.acquire()]
        got = [[], []]
        out = s.step([StepEntry(slots[b], toks[b][:lens[b]], [lens[b] - 1]) for b in range(2)])
        for b in range(2):
            got[b].append((lens[b] - 1, out[b].double().cpu()))
        for j in range(decoded):
            out = s.step([StepEntry(slots[b], [toks[b][lens[b] + j]], [0]) for b in range(2)])
            for b in range(2):
                got[b].append((lens[b] + j, out[b].double().cpu()))
        s.check_device_errors()
        for b in range(2):
            for pos, g in got[b]:
                scale = float(want[b][pos].abs().max())
                err = float((g - want[b][pos]).abs().max())
                assert err <= tol * scale + 1e-6, f"{cfgd} lengths {lens} {dtype} sequence {b} position {pos}: |diff| {err:.3e} of {scale:.3e}"
