"""citlali_cli: the command line, in the manner of the reference's (src/cli/main.cpp).

Kept from the reference with their names, defaults and meaning (main.cpp:203-247, :26-37):
``--model``, ``--max-new-tokens`` (256), ``--ctx`` / ``--context`` (2048), ``--info``,
``--help`` / ``-h``; an unknown argument and a missing value are errors worded as there
(main.cpp:196-201, :245-247); the closing ``[stats]`` line has the reference's fields
(main.cpp:149-157).  The reference's ``--prompt`` takes text; there is no tokenizer here, so
prompts are token ids: ``--prompt-ids 1,2,3`` (repeat it for a batch) or ``--prompt-file``
(a JSON list of lists).  Text modes, quantized residency and remote offload have no
counterpart: their options are refused with the reason.  Added: ``--temperature``, ``--seed``, ``--stop-ids``, ``--dtype``, ``--slots``,
``--json``, ``--random-weights SEED``.
"""
from __future__ import annotations

import json
import sys
import time
from dataclasses import dataclass, field
from typing import List, Optional

USAGE = """usage: citlali_cli --model <dir> (--prompt-ids 1,2,3 [--prompt-ids ...] | --prompt-file <json>) [options]
       citlali_cli --model <dir> --info

  --model <dir>            folder with config.json and model.safetensors
  --prompt-ids a,b,c       one prompt as token ids; repeat for a batch
  --prompt-file <json>     prompts as a JSON list of lists of token ids
  --max-new-tokens N       most tokens to generate per prompt (default 256)
  --ctx N, --context N     most tokens a sequence may hold, capped by the model's (default 2048)
  --temperature F          0 = greedy (default 0)
  --seed N                 seed of temperature sampling (default 0)
  --stop-ids a,b           stop tokens (default: eos_token_id of config.json)
  --dtype bfloat16|float32 compute precision (default bfloat16)
  --slots N                sequences run together (default 8)
  --random-weights SEED    ignore model.safetensors: random weights from this seed
  --info                   print the configuration and sizes; load no weights
  --json                   print results as one JSON object
  --help, -h               this text
"""


# options of the reference's command line (main.cpp:203-247) that have no counterpart here, and why
_NO_TOKENIZER = "this library has no tokenizer; give token ids with --prompt-ids 1,2,3 or --prompt-file <json>"
_NO_OFFLOAD = "quantized residency and remote offload are not part of this library"
REFERENCE_ONLY = {
    "--prompt": _NO_TOKENIZER, "--tokens": _NO_TOKENIZER, "--interactive": _NO_TOKENIZER,
    "--no-chat-template": _NO_TOKENIZER,
    "--quantized": _NO_OFFLOAD, "--offload": _NO_OFFLOAD, "--remote": _NO_OFFLOAD, "--remote-backend": _NO_OFFLOAD,
    "--remote-transport": _NO_OFFLOAD,
}


@dataclass
class CliArgs:
    model_path: str = ""
    prompts: List[List[int]] = field(default_factory=list)
    max_new_tokens: int = 256          # main.cpp:29
    max_context: int = 2048            # main.cpp:30
    temperature: float = 0.0
    seed: int = 0
    stop_ids: Optional[List[int]] = None
    dtype: str = "bfloat16"
    slots: int = 8
    random_weights: Optional[int] = None
    info: bool = False
    json: bool = False
    help: bool = False


def _ids(text: str, flag: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(" ", "").split(",") if t != ""]
    except ValueError:
        raise RuntimeError(f"{flag} takes comma-separated integers, got '{text}'") from None


def parse_args(argv: List[str]) -> CliArgs:
    args = CliArgs()
    i = 1
    while i < len(argv):
        arg = argv[i]

        def need_value(name):
            nonlocal i
            if i + 1 >= len(argv):
                raise RuntimeError("missing value for " + name)
            i += 1
            return argv[i]

        if arg == "--model":
            args.model_path = need_value(arg)
        elif arg == "--prompt-ids":
            args.prompts.append(_ids(need_value(arg), arg))
        elif arg == "--prompt-file":
            with open(need_value(arg), "r", encoding="utf-8") as f:
                data = json.load(f)
            if not (isinstance(data, list) and all(isinstance(p, list) for p in data)):
                raise RuntimeError("--prompt-file must hold a JSON list of lists of token ids")
            args.prompts.extend([[int(t) for t in p] for p in data])
        elif arg == "--max-new-tokens":
            args.max_new_tokens = int(need_value(arg))
        elif arg in ("--ctx", "--context"):
            args.max_context = int(need_value(arg))
        elif arg == "--temperature":
            args.temperature = float(need_value(arg))
        elif arg == "--seed":
            args.seed = int(need_value(arg))
        elif arg == "--stop-ids":
            args.stop_ids = _ids(need_value(arg), arg)
        elif arg == "--dtype":
            args.dtype = need_value(arg)
        elif arg == "--slots":
            args.slots = int(need_value(arg))
        elif arg == "--random-weights":
            args.random_weights = int(need_value(arg))
        elif arg == "--info":
            args.info = True
        elif arg == "--json":
            args.json = True
        elif arg in ("--help", "-h"):
            args.help = True
        elif arg in REFERENCE_ONLY:
            raise RuntimeError(f"{arg}: {REFERENCE_ONLY[arg]}")
        else:
            raise RuntimeError("unknown argument: " + arg)
        i += 1
    return args


def print_model_info(model_path: str, out=sys.stdout) -> None:
    """The parsed configuration and sizes, without loading weights (print_model_info,
    main.cpp:159-190)."""
    from .config.registry import config_from_model_dir
    from .engine.model import expected_tensors
    config = config_from_model_dir(model_path)
    spec = config.to_model_spec()
    tensors = expected_tensors(spec)
    params = 0
    for t in tensors:
        if t.optional and spec.tie_head_to_embedding is not False:
            continue
        n = 1
        for s in t.shape:
            n *= s
        params += n
    print(f"model: {model_path}", file=out)
    for key, value in config.describe().items():
        print(f"{key}: {value}", file=out)
    print(f"tensors: {len(tensors)}", file=out)
    print(f"parameters: {params}", file=out)
    print(f"bfloat16 weight bytes: {2 * params}", file=out)
    from .cache import KVRequirement, StateRequirement
    from .engine.model import cache_requirements_of
    kv = state = 0
    for req in cache_requirements_of(spec):
        if isinstance(req, KVRequirement):
            kv += 2 * req.num_kv_heads * req.head_dim
        elif isinstance(req, StateRequirement):
            n = torch_element_size(req.dtype)
            for s in req.shape:
                n *= s
            state += n
    print(f"cache bytes per token (bfloat16): {2 * kv}", file=out)
    if state:
        print(f"state bytes per sequence: {state}", file=out)


def torch_element_size(dtype) -> int:
    import torch
    return torch.tensor([], dtype=dtype).element_size()


def run_cli(argv: List[str]) -> int:
    args = parse_args(argv)
    if args.help:
        print(USAGE, end="")
        return 0
    if not args.model_path:
        raise RuntimeError("--model is required")
    if args.info:
        print_model_info(args.model_path)
        return 0
    if not args.prompts:
        raise RuntimeError("give at least one prompt: --prompt-ids or --prompt-file")
    from .config.registry import config_from_model_dir
    from .engine.generate import GenerationOptions
    from .engine.session import InferenceSession
    session = InferenceSession()
    print(f"loading {args.model_path} ({args.dtype}) ...", file=sys.stderr, flush=True)
    if args.random_weights is not None:
        session.load_random(config_from_model_dir(args.model_path), args.random_weights,
                            max_context=args.max_context, dtype=args.dtype, max_batch=args.slots,
                            gain_spread=0.1)
    else:
        session.load_model(args.model_path, max_context=args.max_context, dtype=args.dtype, max_batch=args.slots)
    options = GenerationOptions(max_new_tokens=args.max_new_tokens, max_context=args.max_context,
                                temperature=args.temperature, seed=args.seed, stop_ids=args.stop_ids)
    started = time.perf_counter()
    results = session.generate(args.prompts, options)
    seconds = time.perf_counter() - started
    generated = sum(r.generated_tokens for r in results)
    st = session.stats
    if args.json:
        print(json.dumps({
            "results": [{"tokens": r.tokens, "generated_tokens": r.generated_tokens,
                         "stop_reason": r.stop_reason.value} for r in results],
            "stats": {"tokens": generated, "time_s": seconds, **st}}))
    else:
        for i, r in enumerate(results):
            print(f"[{i}] " + ",".join(str(t) for t in r.tokens))
    speed = generated / seconds if seconds > 0 else 0.0
    stops = ",".join(r.stop_reason.value for r in results)
    pre_s, dec_s = st.get("prefill_s", 0.0), st.get("decode_s", 0.0)
    line = (f"[stats] tokens={generated} time={seconds:.3f}s speed={speed:.2f} tok/s stop={stops}"
            f" seqs={len(results)} prefill_tokens={int(st.get('prefill_tokens', 0))} prefill_s={pre_s:.3f}"
            f" decode_tokens={int(st.get('decode_tokens', 0))} decode_s={dec_s:.3f}")
    print(line, file=sys.stderr if args.json else sys.stdout)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = sys.argv if argv is None else argv
    try:
        return run_cli(argv)
    except Exception as e:                         # main.cpp:351-354: print the error, exit 1
        print(f"error: {e}", file=sys.stderr)
        return 1
