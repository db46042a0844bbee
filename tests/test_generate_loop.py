"""The generation loop's decisions, with a fake stepper: no device, no model."""
import pytest

import citlali_b200 as cb
from citlali_b200.engine.generate import GenerationOptions, StopReason, run_generation


class FakeStepper:
    """Sequence r's k-th generated token is script[r][k].  Keeps the books a real session keeps."""

    def __init__(self, scripts, slots=4):
        self.scripts = scripts
        self.free = list(range(slots))
        self.held = {}
        self.log = []
        self.prompt_of_slot = {}
        self.count = {}
        self.released = []

    def acquire(self):
        assert self.free, "no slot free"
        s = self.free.pop(0)
        self.held[s] = True
        return s

    def release(self, slot):
        assert slot in self.held, "released twice"
        del self.held[slot]
        self.free = sorted(self.free + [slot])
        self.released.append(slot)

    def _next(self, slot):
        r = self.prompt_of_slot[slot]
        k = self.count[slot]
        self.count[slot] += 1
        return self.scripts[r][k]

    def prefill(self, slots, prompts, temperature, uniforms):
        self.log.append(("prefill", list(slots), [len(p) for p in prompts], list(uniforms)))
        for s, p in zip(slots, prompts):
            assert s in self.held
            self.prompt_of_slot[s] = p[0]          # the prompt's first token names the request
            self.count[s] = 0
        return [self._next(s) for s in slots]

    def decode(self, slots, tokens, temperature, uniforms):
        self.log.append(("decode", list(slots), list(tokens), list(uniforms)))
        for s in slots:
            assert s in self.held
        return [self._next(s) for s in slots]


def test_stop_token_is_neither_emitted_nor_fed_and_shorter_sequences_leave():
    scripts = {0: [10, 11, 99, 0, 0], 1: [20, 99], 2: [30, 31, 32, 33, 34, 35]}
    st = FakeStepper(scripts)
    prompts = [[0, 1, 2], [1], [2, 5, 5, 5, 5]]
    res = run_generation(st, prompts, GenerationOptions(max_new_tokens=4, max_context=64), [99], 4)
    assert [r.tokens for r in res] == [[10, 11], [20], [30, 31, 32, 33]]
    assert [r.stop_reason for r in res] == [StopReason.EOS, StopReason.EOS, StopReason.MAX_NEW_TOKENS]
    assert [r.generated_tokens for r in res] == [2, 1, 4]
    kinds = [(k, s, t) for k, s, t, _ in st.log]
    assert kinds[0] == ("prefill", [0, 1, 2], [3, 1, 5])
    assert kinds[1] == ("decode", [0, 1, 2], [10, 20, 30])
    assert kinds[2] == ("decode", [0, 2], [11, 31])        # request 1 met its stop token and left
    assert kinds[3] == ("decode", [2], [32])               # request 0 too
    assert len(kinds) == 4                                  # no step is spent on a token nobody uses
    assert st.held == {} and sorted(st.released) == [0, 1, 2]


def test_batches_run_one_after_another_and_reuse_slots():
    scripts = {r: [100 + r] * 3 for r in range(5)}
    st = FakeStepper(scripts, slots=2)
    prompts = [[r, 7] for r in range(5)]
    got = []
    res = run_generation(st, prompts, GenerationOptions(max_new_tokens=2, max_context=64), [], 2,
                         on_token=lambda r, t: got.append((r, t)))
    assert all(r.tokens == [100 + i] * 2 for i, r in enumerate(res))
    prefills = [e for e in st.log if e[0] == "prefill"]
    assert [p[1] for p in prefills] == [[0, 1], [0, 1], [0]]
    assert got[:4] == [(0, 100), (1, 101), (0, 100), (1, 101)] and len(got) == 10
    assert st.held == {}


def test_context_limit_and_prompt_checks():
    st = FakeStepper({0: [1] * 10})
    res = run_generation(st, [[0, 1, 2, 3]], GenerationOptions(max_new_tokens=10, max_context=7), [], 1)
    assert res[0].stop_reason == StopReason.CONTEXT_LIMIT and res[0].generated_tokens == 3
    with pytest.raises(cb.CitlaliError, match="no room"):
        run_generation(st, [[0] * 7], GenerationOptions(max_context=7), [], 1)
    with pytest.raises(cb.CitlaliError, match="produced no tokens"):
        run_generation(st, [[]], GenerationOptions(), [], 1)
    with pytest.raises(cb.CitlaliError, match="no prompts"):
        run_generation(st, [], GenerationOptions(), [], 1)


def test_max_new_tokens_zero_takes_no_step():
    st = FakeStepper({0: [1]})
    res = run_generation(st, [[0]], GenerationOptions(max_new_tokens=0), [], 1)
    assert res[0].tokens == [] and st.log == []


def test_draws_depend_on_request_and_token_index_only():
    scripts = {r: [50 + r] * 4 for r in range(3)}
    a = FakeStepper(scripts); b = FakeStepper(scripts)
    prompts = [[0], [1], [2]]
    opts = GenerationOptions(max_new_tokens=3, temperature=0.8, seed=5, max_context=64)
    run_generation(a, prompts, opts, [], 3)
    run_generation(b, prompts, opts, [], 1)        # one request a batch
    def draws(st):
        out = {}
        for kind, slots, _, us in st.log:
            for s, u in zip(slots, us):
                out.setdefault(st.scripts and s, []).append(u)
        return out
    ua = [e[3] for e in a.log]
    # in the batch of three, step k draws (request, k) for each live request
    assert ua[0] == [cb.uniform(5, r, 0) for r in range(3)]
    assert ua[1] == [cb.uniform(5, r, 1) for r in range(3)]
    ub = [e[3] for e in b.log]
    assert ub[0] == [cb.uniform(5, 0, 0)] and ub[3] == [cb.uniform(5, 1, 0)]
    assert all(0.0 <= cb.uniform(1, r, k) < 1.0 for r in range(20) for k in range(20))
    assert len({cb.uniform(1, r, k) for r in range(20) for k in range(20)}) > 390
    greedy = FakeStepper(scripts)
    run_generation(greedy, prompts, GenerationOptions(max_new_tokens=2, max_context=64), [], 3)
    assert all(e[3] == [] for e in greedy.log)


def test_slots_are_given_back_when_a_step_fails():
    class Failing(FakeStepper):
        def decode(self, *a):
            raise RuntimeError("boom")
    st = Failing({0: [1, 2], 1: [3, 4]})
    with pytest.raises(RuntimeError):
        run_generation(st, [[0], [1]], GenerationOptions(max_new_tokens=3, max_context=64), [], 2)
    assert st.held == {}
