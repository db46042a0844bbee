#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload 3|4 [--repetitions R]      the batch workloads of BASELINE.json's other shapes

Prints ONE JSON line.  For each batch size (8, and 1 and 64 unless --skip-points) the run is a real one: the
prompts (2,048 random tokens each) are prefilled in one step, then every sequence is decoded token by token up
to the context length (4,096) through the replayed decode step, each step fed on the device with the tokens
the step before sampled; CUDA events give the rate over the whole run and over windows of 64 steps at contexts
2,048, 3,072 and 4,096 (``points``).  ``value`` is decoded tokens a second at batch 8 over the last K steps
before the context length (the sequences are rewound and those W + K steps run again: the median of
``repetitions`` timings); ``e2e`` is the same steps through ``InferenceSession.decode`` with the step's tokens
coming from host memory and the sampled tokens read back every step.  ``prefill`` times one 2,048-token prompt
(``frac``: the matrix products' FLOPs over the time over the bf16 peak); ``roofline`` relates the decode step
to the bytes it must read; ``kernels`` times the kernels of a layer one kind at a time.  Several GPUs are not
supported.
"""
import argparse
import json
import os
import random
import re
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}     # an earlier measurement on this pool
QWEN3_8B = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                tie_word_embeddings=False, context=4096, prefill_tokens=2048)


def benchmark_shape():
    """The sizes of BASELINE.json's configs[2] (a sentence), read from it where it can be parsed."""
    shape = dict(QWEN3_8B)
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            text = json.load(f)["configs"][2]
        def num(pattern, cast=int):
            m = re.search(pattern, text)
            return cast(m.group(1).replace(",", "")) if m else None
        for key, pattern in (("num_hidden_layers", r"(\d+) layers"), ("hidden_size", r"hidden (\d+)"),
                             ("num_attention_heads", r"(\d+) q heads"), ("num_key_value_heads", r"(\d+) kv heads"),
                             ("head_dim", r"head_dim (\d+)"), ("intermediate_size", r"intermediate (\d+)"),
                             ("vocab_size", r"vocab (\d+)"), ("context", r"Context (\d+)"),
                             ("prefill_tokens", r"prefill ([\d,]+)-token")):
            v = num(pattern)
            if v:
                shape[key] = v
        shape["tie_word_embeddings"] = "untied" not in text
    except Exception:
        pass
    return shape


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            pk = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:          # a seconds-long loop under the power cap
                pk["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return pk
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


def workload_from_baseline(index):
    """A batch workload of BASELINE.json's configs (a sentence): the model's sizes, the number of
    prompts, the range of their lengths and the decode steps."""
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        text = json.load(f)["configs"][index]
    def num(pattern):
        m = re.search(pattern, text)
        if not m:
            raise SystemExit(f"bench.py: configs[{index}] of BASELINE.json does not say '{pattern}'")
        return int(m.group(1).replace(",", ""))
    span = re.search(r"lengths uniform in \[(\d+),\s*(\d+)\]", text)
    if not span:
        raise SystemExit(f"bench.py: configs[{index}] of BASELINE.json names no range of prompt lengths")
    return dict(name=text.split(":")[0].strip(), num_hidden_layers=num(r"(\d+) layers"), hidden_size=num(r"hidden (\d+)"),
                num_attention_heads=num(r"(\d+) q heads"), num_key_value_heads=num(r"(\d+) kv heads"),
                head_dim=num(r"head_dim (\d+)"), intermediate_size=num(r"intermediate (\d+)"),
                vocab_size=num(r"vocab (\d+)"), tie_word_embeddings="untied" not in text,
                prompts=num(r"Batch of (\d+) prompts"), shortest=int(span.group(1)), longest=int(span.group(2)),
                decode_steps=num(r"then (\d+) decode steps"))


def run_workload(index, repetitions, layers=None):
    """One of BASELINE.json's batch workloads through ``InferenceSession.generate``: unequal prompts in
    one step, then the decode steps, host tokens in and out.  Prints one JSON line: decoded tokens a
    second (the median run), the prompts' tokens a second, and both against their rooflines."""
    import torch
    import citlali_b200 as cb

    w = workload_from_baseline(index)
    layers_full = w["num_hidden_layers"]
    if layers:
        w["num_hidden_layers"] = min(int(layers), layers_full)       # fewer layers of the same sizes (a profiler capture)
    context = -(-(w["longest"] + w["decode_steps"]) // cb.PAGE_SIZE) * cb.PAGE_SIZE
    cfg = cb.config_from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=w["num_hidden_layers"], hidden_size=w["hidden_size"],
        num_attention_heads=w["num_attention_heads"], num_key_value_heads=w["num_key_value_heads"], head_dim=w["head_dim"],
        intermediate_size=w["intermediate_size"], vocab_size=w["vocab_size"], rope_theta=1e6, rms_norm_eps=1e-6,
        tie_word_embeddings=w["tie_word_embeddings"], max_position_embeddings=max(context, 40960)))
    pk = peaks()
    session = cb.InferenceSession().load_random(cfg, seed=1, max_context=context, dtype="bfloat16", device="cuda:0",
                                                max_batch=w["prompts"])
    rng = random.Random(0)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(w["shortest"], w["longest"]))]
               for _ in range(w["prompts"])]
    options = cb.GenerationOptions(max_new_tokens=w["decode_steps"], max_context=context, stop_ids=[])
    clocks = ClockSampler()
    runs = []
    for rep in range(1 + repetitions):
        if rep == 1:
            clocks.start()
        torch.cuda.synchronize()
        session.generate(prompts, options)
        torch.cuda.synchronize()
        if rep >= 1:
            runs.append(dict(session.stats))
        print(f"[bench] {w['name']} run {rep}: {session.stats}", file=sys.stderr, flush=True)
    clock_record = clocks.stop()
    # the median of each figure on its own (a run with the median decode time may hold a prompt step that a
    # page fault or an allocation disturbed)
    run = {k: statistics.median(r[k] for r in runs) for k in runs[0]}
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv, layers = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.num_hidden_layers
    layer_params = (nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I
    tokens = sum(len(p) for p in prompts)
    prefill_flops = (2.0 * tokens * layer_params * layers + 2.0 * H * cfg.vocab_size * len(prompts)
                     + layers * 4.0 * sum(n * (n + 1) / 2 for n in map(len, prompts)) * d * nq)
    kv_bytes_per_token = sum(2 * g.requirement.num_kv_heads * g.requirement.head_dim * 2 * len(g.steps)
                             for g in session.cache.kv_groups)
    steps = run["decode_tokens"] / len(prompts)
    step_bytes = session.model.weight_bytes_read_per_step() + (tokens + len(prompts) * steps / 2) * kv_bytes_per_token
    decode_ms = run["decode_s"] / steps * 1e3
    achieved = step_bytes / (decode_ms / 1e3) / 1e9
    print(json.dumps({
        "metric": f"decode tok/s, {len(prompts)} unequal prompts ({w['name']}, random bf16 weights)",
        "value": run["decode_tokens"] / run["decode_s"], "unit": "tok/s", "n_gpus": 1, "steps": int(steps), "warmup": 1,
        "ms_per_step": decode_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "ours",
        "timing": "host clock around InferenceSession.generate's prompt step and decode steps, tokens from and to the host",
        "config": {"model": w["name"], "layers": layers, "layers_full": layers_full, "hidden": H, "q_heads": nq, "kv_heads": nkv, "head_dim": d,
                   "intermediate": I, "vocab": cfg.vocab_size, "global_batch": len(prompts), "prompt_tokens": tokens,
                   "shortest": min(map(len, prompts)), "longest": max(map(len, prompts)), "decode_steps": int(steps),
                   "repetitions": repetitions, "parallelism": "single GPU", "peaks": pk["source"]},
        "prefill": {"value": tokens / run["prefill_s"], "tokens": tokens, "ms": run["prefill_s"] * 1e3,
                    "frac": prefill_flops / run["prefill_s"] / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes},
        "clocks": clock_record}))
    return 0


def run_reference(args):
    """The unmodified reference (built under baseline/_ref by ``baseline/reference_arm.py install``) at the
    benchmark's sizes: it serves ONE sequence, token by token, in FP16, so its line is decode at batch 1 near
    the context length; batches of 8 and 64 and a one-step prompt have no counterpart in it
    (src/runtime/session.cpp:69-74: the prompt is a loop over forward_token)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    try:
        import reference_arm
    except Exception as e:
        return unavailable(f"baseline/reference_arm.py cannot be imported: {e}")
    why = reference_arm.installed()
    source = os.environ.get("CITLALI_REFERENCE_SOURCE", os.path.join(os.sep, "root", "reference"))    # a checkout of the reference, if one is at hand
    if why and os.path.isdir(source):
        try:
            reference_arm.install(source)
            why = reference_arm.installed()
        except Exception as e:
            why = f"the reference could not be built here: {str(e)[-300:]}"
    if why:
        return unavailable(why)
    if args.gpus != 1:
        return unavailable("the reference runs one sequence on one GPU; several GPUs have no meaning for it")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device here; the reference has no CPU path")
    except Exception as e:
        return unavailable(f"torch is needed to make the random model file: {e}")
    shape = benchmark_shape()
    layers_full = shape["num_hidden_layers"]
    layers = args.layers or layers_full
    context = shape["context"]
    K, W = args.steps, max(args.warmup, 3)
    config = dict(num_hidden_layers=layers, hidden_size=shape["hidden_size"], num_attention_heads=shape["num_attention_heads"],
                  num_key_value_heads=shape["num_key_value_heads"], head_dim=shape["head_dim"],
                  intermediate_size=shape["intermediate_size"], vocab_size=shape["vocab_size"], rope_theta=shape["rope_theta"],
                  rms_norm_eps=shape["rms_norm_eps"], tie_word_embeddings=shape["tie_word_embeddings"],
                  max_position_embeddings=context)
    need = 2 * (layers * ((shape["num_attention_heads"] * 2 + shape["num_key_value_heads"] * 2) * shape["head_dim"]
                          * shape["hidden_size"] + 3 * shape["hidden_size"] * shape["intermediate_size"])
                + 2 * shape["vocab_size"] * shape["hidden_size"]) + (64 << 20)
    folder = None
    for base in (tempfile.gettempdir(), "/dev/shm"):
        try:
            if os.path.isdir(base) and shutil.disk_usage(base).free > need * 1.1:
                folder = tempfile.mkdtemp(prefix="citlali_reference_", dir=base)
                break
        except OSError:
            continue
    if folder is None:
        return unavailable(f"no temporary folder has the {need / 1e9:.0f} GB that the reference's model file needs")
    gguf = os.path.join(folder, "model.gguf")
    clocks = ClockSampler()
    try:
        t0 = time.time()
        size = reference_arm.gguf_random(config, gguf, seed=1, device="cuda:0",
                                         progress=lambda m: print(f"[bench] {m}", file=sys.stderr, flush=True))
        torch.cuda.empty_cache()
        print(f"[bench] reference arm: model file of {size / 1e9:.1f} GB written in {time.time() - t0:.0f} s",
              file=sys.stderr, flush=True)
        start = context - (1 + W + K)
        clocks.start()
        r = reference_arm.reference_decode(gguf, context, 1, W, K, start_position=start)
        clock_record = clocks.stop()
    except Exception as e:
        clocks.stop()
        return unavailable(f"the reference did not run: {str(e)[-300:]}")
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    print(f"[bench] reference arm: {r}", file=sys.stderr, flush=True)
    pk = peaks()
    kv_bytes_per_token = 2 * shape["num_key_value_heads"] * shape["head_dim"] * 2 * layers
    mean_len = (r["first_timed_position"] + r["last_timed_position"]) / 2.0 + 1
    step_bytes = need - (64 << 20) - 2 * shape["vocab_size"] * shape["hidden_size"] + mean_len * kv_bytes_per_token
    achieved = step_bytes / (r["ms_per_step"] / 1e3) / 1e9
    print(json.dumps({
        "metric": "decode tok/s @ batch 1 (Qwen3-8B shape, random fp16 weights): the reference serves one sequence",
        "value": r["tokens_per_second"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic: random weights N(0,0.02) in a GGUF file, token ids from its own greedy loop",
        "impl": "reference",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": layers_full, "hidden": shape["hidden_size"],
                   "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "global_batch": 1, "seq_len": context, "first_timed_position": r["first_timed_position"],
                   "parallelism": "single GPU", "compare_with": "points.decode_b1 of the other arm",
                   "no_counterpart": "batch 8 and 64, a one-step prompt (its prompt is a loop over single tokens)",
                   "timing": "host clock around QwenModel::forward_token, which synchronises the device every token",
                   "cache_below_start": "as allocated: its kernels' work depends on the position alone",
                   "peaks": pk["source"]},
        "e2e": {"value": r["tokens_per_second"], "unit": "tok/s", "h2d_bytes_per_step": 4,
                "d2h_bytes_per_step": 4 * shape["vocab_size"],
                "note": "forward_token is the reference's end-to-end step: token id in, all logits copied to the host, argmax there"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes},
        "load_seconds": r["load_seconds"], "clocks": clock_record}))
    return 0


class ClockSampler:
    """nvidia-smi in the background while something is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 6:
                    continue
                try:
                    sm.append(float(f[0])); mx.append(float(f[1]))
                except ValueError:
                    continue
                for name, v in zip(names, f[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="batch 8 only, no per-kernel timings")
    ap.add_argument("--workload", type=int, default=2,
                    help="which of BASELINE.json's configs to run: 2 (the benchmark configuration) or a batch workload (3, 4)")
    ap.add_argument("--repetitions", type=int, default=5, help="timed repetitions (the median is reported)")
    ap.add_argument("--run-from", type=int, default=None,
                    help="length of the prompts of the decode runs (default: the prefill length, 2,048); close to the context "
                         "length it makes a short run, as a profiler capture needs")
    args = ap.parse_args()

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: --gpus {args.gpus} is not supported (this library runs on a single device)")
        return 2

    if args.workload != 2:
        return run_workload(args.workload, max(1, args.repetitions), args.layers)

    import torch
    import citlali_b200 as cb
    from citlali_b200 import ops

    shape = benchmark_shape()
    layers_full = shape["num_hidden_layers"]
    layers = args.layers or layers_full
    context, prefill_tokens = shape["context"], shape["prefill_tokens"]
    K, W, R = args.steps, max(args.warmup, 3), max(1, args.repetitions)
    cfg = cb.config_from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=layers, hidden_size=shape["hidden_size"],
        num_attention_heads=shape["num_attention_heads"], num_key_value_heads=shape["num_key_value_heads"],
        head_dim=shape["head_dim"], intermediate_size=shape["intermediate_size"], vocab_size=shape["vocab_size"],
        rope_theta=shape["rope_theta"], rms_norm_eps=shape["rms_norm_eps"],
        tie_word_embeddings=shape["tie_word_embeddings"], max_position_embeddings=max(context, 40960)))
    pk = peaks()
    batches = [args.batch] if args.skip_points else sorted({args.batch, 1, 64})
    t_load = time.time()
    session = cb.InferenceSession().load_random(cfg, seed=1, max_context=context, dtype="bfloat16", device="cuda:0",
                                                max_batch=max(batches))
    torch.cuda.synchronize()
    print(f"[bench] model of {layers} layers ready in {time.time() - t_load:.0f} s", file=sys.stderr, flush=True)
    vocab = cfg.vocab_size
    rng = random.Random(0)
    clocks = ClockSampler()
    clocks.start()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    weight_bytes = session.model.weight_bytes_read_per_step()
    kv_bytes_per_token = sum(2 * g.requirement.num_kv_heads * g.requirement.head_dim * 2 * len(g.steps)
                             for g in session.cache.kv_groups)
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    layer_params = (nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I

    # ---- prefill: one prompt of 2,048 tokens ----------------------------------------------
    prompt = [rng.randrange(vocab) for _ in range(prefill_tokens)]
    times = []
    for i in range(3 + R):
        slot = session.acquire()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        logits = session.step([cb.StepEntry(slot, prompt, [prefill_tokens - 1])])
        session.sampler.sample_device(logits, 0.0, [])
        b.record()
        torch.cuda.synchronize()
        session.release(slot)
        if i >= 3:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)
    T = prefill_tokens
    gemm_flops = 2.0 * T * layer_params * layers + 2.0 * H * vocab
    attention_flops = layers * 4.0 * (T * (T + 1) / 2) * d * nq
    per_s = 1.0 / (prefill_ms / 1e3)
    prefill = {"value": T * per_s, "tokens": T, "ms": prefill_ms,
               "frac": gemm_flops * per_s / (pk["bf16_tflops"] * 1e12),
               "frac_counts": "matrix products only (the metric's definition), of the burst peak",
               "frac_with_attention": (gemm_flops + attention_flops) * per_s / (pk["bf16_tflops"] * 1e12),
               "tflops": gemm_flops * per_s / 1e12, "repetitions": R}
    if "bf16_tflops_sustained" in pk:
        prefill["frac_sustained"] = gemm_flops * per_s / (pk["bf16_tflops_sustained"] * 1e12)
    # The repetitions above follow one another at once and run under the power cap (about 1.5 GHz of 1.965 at 985 W);
    # the burst peak is a short product's.  The same step alone, after 200 ms of rest, is what a single prompt costs.
    rested = []
    for i in range(R):
        slot = session.acquire()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        time.sleep(0.2)
        a.record()
        logits = session.step([cb.StepEntry(slot, prompt, [prefill_tokens - 1])])
        session.sampler.sample_device(logits, 0.0, [])
        b.record()
        torch.cuda.synchronize()
        session.release(slot)
        rested.append(a.elapsed_time(b))
    prefill["ms_after_rest"] = statistics.median(rested)
    prefill["frac_after_rest"] = gemm_flops / (prefill["ms_after_rest"] / 1e3) / (pk["bf16_tflops"] * 1e12)
    print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)

    # ---- decode: a run from the prompts' end to the context length, then the last steps again ----------
    runner = session.runner

    def step_bytes(batch, mean_len):
        return weight_bytes + batch * mean_len * kv_bytes_per_token

    def decode_run(batch):
        slots = [session.acquire() for _ in range(batch)]
        run_from = min(args.run_from or prefill_tokens, context - (W + K) - 8)
        prompts = [[rng.randrange(vocab) for _ in range(run_from)] for _ in range(batch)]
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        first = session.prefill(slots, prompts, 0.0, [])
        b.record()
        torch.cuda.synchronize()
        out = {"prefill_ms": a.elapsed_time(b)}
        total = context - run_from                             # decode steps: positions run_from .. context-1
        window = max(1, min(64, total // 4))
        marks = {"ctx%d" % run_from: 0, "ctx%d" % ((run_from + context) // 2): total // 2 - window // 2,
                 "ctx%d" % context: total - window}
        starts = {max(at, 1): name for name, at in marks.items()}
        ends = {max(at, 1) + window - 1: name for name, at in marks.items()}
        events = {name: [ev(), ev()] for name in marks}
        runner.launch(slots, first, 0.0, [])                   # step 0 (captures the graph on first use)
        torch.cuda.synchronize()
        launches = 0
        start = ev(); start.record()
        for step in range(1, total):
            if step in starts:
                events[starts[step]][0].record()
            runner.feed_back(batch)
            launches = runner.launch(slots, None, 0.0, [])
            if step in ends:
                events[ends[step]][1].record()
        end = ev(); end.record()
        torch.cuda.synchronize()
        session.check_device_errors()
        out["run_tok_s"] = batch * (total - 1) / (start.elapsed_time(end) / 1e3)
        for name, (e0, e1) in events.items():
            out[name] = batch * window / (e0.elapsed_time(e1) / 1e3)
        # the last W + K steps again, R times on the device and R times end to end
        def rewind():
            for s in slots:
                session.cache.rewind(s, context - (W + K))
        dev_ms, e2e_ms = [], []
        for _ in range(R):
            rewind()
            runner.launch(slots, first, 0.0, [])
            for _ in range(W - 1):
                runner.feed_back(batch); runner.launch(slots, None, 0.0, [])
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            for _ in range(K):
                runner.feed_back(batch); runner.launch(slots, None, 0.0, [])
            b.record()
            torch.cuda.synchronize()
            dev_ms.append(a.elapsed_time(b) / K)
        for _ in range(R):
            rewind()
            tokens = list(first)
            for _ in range(W):
                tokens = session.decode(slots, tokens, 0.0, [])
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(K):
                tokens = session.decode(slots, tokens, 0.0, [])
            torch.cuda.synchronize()
            e2e_ms.append((time.perf_counter() - t0) / K * 1e3)
        session.check_device_errors()
        for s in slots:
            session.release(s)
        out.update(ms=statistics.median(dev_ms), e2e_ms=statistics.median(e2e_ms), launches=launches,
                   mean_len=context - (K - 1) / 2.0)
        out["tok_s"] = batch / (out["ms"] / 1e3)
        out["e2e_tok_s"] = batch / (out["e2e_ms"] / 1e3)
        out["frac"] = step_bytes(batch, out["mean_len"]) / (out["ms"] / 1e3) / 1e9 / pk["hbm_gbs"]
        return out

    runs = {}
    for bsz in batches:
        runs[bsz] = decode_run(bsz)
        print(f"[bench] decode b{bsz} {runs[bsz]}", file=sys.stderr, flush=True)
    main_run = runs[args.batch]
    points, point_fracs = {}, {}
    for bsz, r in runs.items():
        if bsz != args.batch:
            points[f"decode_b{bsz}"] = r["tok_s"]
            point_fracs[f"decode_b{bsz}"] = round(r["frac"], 4)
        for name, v in r.items():
            if name.startswith("ctx"):
                points[f"decode_b{bsz}_{name}"] = v
                ctx_len = int(name[3:]) + (32 if int(name[3:]) < context else -32)
                point_fracs[f"decode_b{bsz}_{name}"] = round(step_bytes(bsz, ctx_len) * v / bsz / 1e9 / pk["hbm_gbs"], 4)
        points[f"decode_b{bsz}_run"] = r["run_tok_s"]
        points[f"prefill_b{bsz}_tok_s"] = bsz * min(args.run_from or prefill_tokens, context - (W + K) - 8) / (r["prefill_ms"] / 1e3)

    kernels = {} if args.skip_points else time_kernels(session, cb, ops, torch, cfg, args.batch, context, prefill_tokens, pk)
    clock_record = clocks.stop()

    bytes_main = step_bytes(args.batch, main_run["mean_len"])
    achieved = bytes_main / (main_run["ms"] / 1e3) / 1e9
    h2d = int(runner._offsets[6] * 4)
    line = {
        "metric": f"decode tok/s @ batch {args.batch} (Qwen3-8B shape, random bf16 weights)",
        "value": main_run["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": main_run["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), prompts of uniform random token ids prefilled for real, "
                                 "decoded tokens fed back",
        "impl": "ours", "repetitions": R,
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": layers_full, "hidden": H,
                   "q_heads": nq, "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": context, "prefill_tokens": prefill_tokens,
                   "parallelism": "single GPU", "l2": "inputs larger than L2: every step reads all weights",
                   "peaks": pk["source"]},
        "e2e": {"value": main_run["e2e_tok_s"], "unit": "tok/s", "ms_per_step": main_run["e2e_ms"],
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": K * main_run["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": bytes_main},
        "points": points,
        "points_roofline_frac": point_fracs,
        "kernels": kernels,
        "clocks": clock_record,
    }
    print(json.dumps(line))
    return 0


def time_kernels(session, cb, ops, torch, cfg, batch, context, prefill_tokens, pk):
    """The kernels of a layer, one kind at a time: the same kernel on every layer's own weights and cache in
    turn (15 GB of weights between two uses of the same bytes, far more than L2 holds), the sweep captured in a
    CUDA graph and replayed, CUDA events around the replay, the mean per launch.  Decode at `batch` sequences of `context` - 1 cached tokens, and one prompt of
    `prefill_tokens` tokens.  Fractions: bytes the kernel must read over the time over the copy bandwidth
    (decode), FLOPs over the time over the bf16 burst peak (prompt)."""
    import math
    model, cache = session.model, session.cache
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nq, nkv, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    dev = model.ctx.device
    blocks = [model.layers[s.layer] for s in model.spec.schedule]
    out = {}
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def sweep(fn, count=len(blocks), rounds=3):
        # the sweep is captured once and replayed, so that no launch waits for the host
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn(0)                                      # outside capture first: kernel attributes, scratch buffers
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(count):
                fn(i)
        best = None
        for _ in range(rounds + 1):
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            t = a.elapsed_time(b) * 1e3 / count
            best = t if best is None else min(best, t)
        return best

    for what, rows, past in (("decode", batch, context - 1), ("prefill", prefill_tokens, 0)):
        nseq = batch if what == "decode" else 1
        slots = [session.acquire() for _ in range(nseq)]
        for s in slots:
            session.assume_cached(s, past + rows // nseq)
        entries = [cb.StepEntry(s, [0] * (rows // nseq), []) for s in slots]
        from citlali_b200.engine.step import pack_step
        step = pack_step(entries, [past] * nseq, V, dev)
        h = torch.randn(rows, H, device=dev).to(torch.bfloat16)
        x = torch.zeros(rows, H, dtype=torch.float32, device=dev)
        act = torch.randn(rows, I, device=dev).to(torch.bfloat16)
        o_in = torch.randn(rows, nq * d, device=dev).to(torch.bfloat16)
        qkv = torch.randn(rows, (nq + 2 * nkv) * d, device=dev).to(torch.bfloat16)
        attn_out = torch.empty(rows, nq * d, dtype=torch.bfloat16, device=dev)
        views = [cache.view(i) for i in range(len(blocks))]
        m = [b.mixer for b in blocks]
        f = [b.feed_forward for b in blocks]
        # decoding runs the layer norms inside the products around them (parts/block.py): the products are timed in
        # the form the step runs, the norm kernel remains for the first layer's rows and before the head
        fused = what == "decode" and getattr(blocks[0], "norms_in_products", False)
        sums = torch.ones(rows, H // 32, device=dev)
        emit = (torch.empty(rows, H, dtype=torch.bfloat16, device=dev), torch.empty(rows, H // 32, device=dev))
        scale = (sums, H, 1e-6)
        us = {
            "norm": sweep(lambda i: blocks[i].mixer_norm.forward(x)),
            "qkv": sweep(lambda i: m[i].qkv.forward(h, row_scale=scale if fused else None)),
            "norm_rope_cache": sweep(lambda i: ops.qk_norm_rope_cache(
                qkv, m[i].q_gain, m[i].k_gain, m[i].inv_freq, m[i].rotary_dim, step.row_slot, step.row_pos, views[i].page_table,
                views[i].keys, views[i].values, views[i].page_size, nq, nkv, d, float(m[i].eps))),
            # (the prompt kernel is called by name: inside a captured sweep the choice between kernels refuses the ones
            # whose launch depends on the step's lengths, which here are constants)
            "attention": sweep((lambda i: ops.attention(qkv, qkv.shape[1], views[i], step, attn_out, nq, nkv, d, 0,
                                                        1.0 / math.sqrt(d))) if what == "decode" else
                               (lambda i: ops.attention_prefill_tc(qkv, qkv.shape[1], views[i].keys, views[i].values,
                                                                   views[i].page_table, step.seq_start, step.seq_slot, step.seq_past,
                                                                   attn_out, 1, rows, nq, nkv, d, views[i].page_size, 0,
                                                                   1.0 / math.sqrt(d), model.ctx.error_flag))),
            "output": sweep(lambda i: m[i].o.forward(o_in, accumulate_into=x, emit=emit if fused else None)),
            "gate_up": sweep(lambda i: f[i].gate_up.forward_gated(h, f[i].run, row_scale=scale if fused else None)),
            "down": sweep(lambda i: f[i].down.forward(act, accumulate_into=x, emit=emit if fused else None)),
        }
        if what == "decode":
            hw = torch.randn(batch, H, device=dev).to(torch.bfloat16)
            us["head"] = sweep(lambda i: model.head.forward(hw, out_dtype=torch.float32), count=4)
        for s in slots:
            session.release(s)
        keys = rows // nseq + past
        if what == "decode":
            need = {"qkv": 2.0 * (nq + 2 * nkv) * d * H, "attention": 2.0 * 2 * nseq * keys * nkv * d, "output": 2.0 * H * nq * d,
                    "gate_up": 2.0 * 2 * I * H, "down": 2.0 * H * I, "head": 2.0 * V * H}
            for k, t in us.items():
                out[f"decode_{k}"] = {"us": round(t, 2)}
                if k in need:
                    out[f"decode_{k}"]["frac"] = round(need[k] / (t * 1e-6) / 1e9 / pk["hbm_gbs"], 3)
        else:
            need = {"qkv": 2.0 * rows * (nq + 2 * nkv) * d * H, "attention": 4.0 * (rows * (rows + 1) / 2) * d * nq,
                    "output": 2.0 * rows * H * nq * d, "gate_up": 2.0 * rows * 2 * I * H, "down": 2.0 * rows * H * I}
            for k, t in us.items():
                out[f"prefill_{k}"] = {"us": round(t, 1)}
                if k in need:
                    out[f"prefill_{k}"]["frac"] = round(need[k] / (t * 1e-6) / 1e12 / pk["bf16_tflops"], 3)
    out["note"] = ("us per launch in a replayed sweep over the layers, best of 4; decode products in the form the step runs "
                   "(the layer norms' work in their epilogues), the norm kernel itself runs twice a step; decode frac = bytes the kernel must read / time / "
                   "copy bandwidth, prefill frac = FLOPs / time / bf16 burst peak")
    return out


if __name__ == "__main__":
    sys.exit(main())
