"""Building replay traces and running them, in-process or through bin/trace_run.

A request is (id, tokens).  A trace is a list of step records in the format bin/trace_run
reads.  Running a trace yields {(id, position): logits row}.
"""
import json
import os
import subprocess
import sys
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole(requests):
    """Each request alone, all its tokens in one step, logits everywhere."""
    steps = []
    for rid, toks in requests:
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail(requests, last=32):
    """Each request alone: all but the last `last` tokens in one step, then one by one."""
    steps = []
    for rid, toks in requests:
        head = max(len(toks) - last, 0)
        if head:
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head],
                                                           "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
    return steps


def batched(requests, prompt_lens, batch_size):
    """Batches of `batch_size` requests, one batch after another.  A batch starts with all its
    prompts (unequal lengths) in one step, logits at each prompt's end; then one token per live
    request per step; a request that runs out of tokens ends and the batch shrinks."""
    steps = []
    for first in range(0, len(requests), batch_size):
        group = list(zip(requests[first:first + batch_size], prompt_lens[first:first + batch_size]))
        entries, end = [], []
        for (rid, toks), n in group:
            entries.append({"id": rid, "tokens": toks[:n], "want": [n - 1]})
            if n == len(toks):
                end.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": end})
        pos = {rid: n for (rid, toks), n in group}
        live = [(rid, toks) for (rid, toks), n in group if n < len(toks)]
        while live:
            entries, end, nxt = [], [], []
            for rid, toks in live:
                entries.append({"id": rid, "tokens": [toks[pos[rid]]], "want": [0]})
                pos[rid] += 1
                if pos[rid] == len(toks):
                    end.append(rid)
                else:
                    nxt.append((rid, toks))
            steps.append({"step": len(steps), "entries": entries, "end": end})
            live = nxt
    return steps


def chunked(requests, batch_size, seed, low=2, high=40):
    """Batches of `batch_size` requests that start together and then go on together by several tokens a
    step: each live request brings its next `low`..`high` tokens (drawn per request and step), so that the
    sequences of a step have unequal pasts and unequal numbers of new tokens.  Logits everywhere."""
    import random
    rng = random.Random(seed)
    steps = []
    for first in range(0, len(requests), batch_size):
        pos = {rid: 0 for rid, _ in requests[first:first + batch_size]}
        live = list(requests[first:first + batch_size])
        while live:
            entries, end, nxt = [], [], []
            for rid, toks in live:
                n = min(rng.randint(low, high), len(toks) - pos[rid])
                entries.append({"id": rid, "tokens": toks[pos[rid]:pos[rid] + n], "want": list(range(n))})
                pos[rid] += n
                if pos[rid] == len(toks):
                    end.append(rid)
                else:
                    nxt.append((rid, toks))
            steps.append({"step": len(steps), "entries": entries, "end": end})
            live = nxt
    return steps


def joining(requests, prompt_lens, every):
    """One running batch that requests join while it runs: request i starts (its prompt in one step) at step
    `i * every`, in the same step in which earlier requests go on by one token.  Logits at each prompt's end
    and at every later token."""
    steps, pos, live, waiting, t = [], {}, [], list(zip(requests, prompt_lens)), 0
    while live or waiting:
        entries, end, nxt = [], [], []
        for rid, toks in live:
            entries.append({"id": rid, "tokens": [toks[pos[rid]]], "want": [0]})
            pos[rid] += 1
            (end if pos[rid] == len(toks) else nxt).append(rid if pos[rid] == len(toks) else (rid, toks))
        if waiting and t % every == 0:
            (rid, toks), n = waiting.pop(0)
            entries.append({"id": rid, "tokens": toks[:n], "want": [n - 1]})
            pos[rid] = n
            (end if n == len(toks) else nxt).append(rid if n == len(toks) else (rid, toks))
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
        live = nxt
        t += 1
    return steps


def max_live_tokens(steps):
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held, best = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        best = max(best, sum((n + 63) // 64 * 64 for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return best


def _collect(steps, rows_of_step):
    """{(id, position): row} from per-step logits."""
    out, pos = {}, {}
    for s in steps:
        rows = rows_of_step(s)
        r = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
        assert r == rows.shape[0]
    return out


def run_in_process(session, steps):
    import citlali_b200 as cb
    slots = {}

    def rows_of_step(s):
        entries = []
        for e in s["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = session.acquire()
            entries.append(cb.StepEntry(slots[e["id"]], e["tokens"], e["want"]))
        logits = session.step(entries).float().cpu()
        for rid in s["end"]:
            session.release(slots.pop(rid))
        return logits

    out = _collect(steps, rows_of_step)
    session.check_device_errors()
    assert slots == {}
    return out


def run_trace_run(model_dir, dtype, steps, vocab, max_tokens=None, env=None):
    """Drive bin/trace_run as a user would: steps on its standard input, one at a time, the next
    only after `done <step>` came back."""
    import numpy as np
    out_dir = tempfile.mkdtemp(prefix="trace_out_")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens or max_live_tokens(steps))]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()

    def rows_of_step(s):
        path = os.path.join(out_dir, f"{s['step']}.f32")
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted == 0:
            assert not os.path.exists(path)
            return torch.empty(0, vocab)
        return torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, vocab).copy())

    return _collect(steps, rows_of_step)
