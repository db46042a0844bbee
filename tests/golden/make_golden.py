"""Makes the files in this folder: logits of the reference engine itself for tiny random models.

Needs a CUDA device (the reference has no CPU path) and the reference built by
``python baseline/reference_arm.py install <reference checkout>``.  For each case it writes a model
folder with this library's seeded random weights (float32), converts it to a float32 GGUF file with the
reference's tensor names and metadata, and feeds the token ids below, one token at a time from position 0,
through the reference's ``QwenModel::forward_token`` (src/model/qwen_model.cpp:239-419), reading its logits
after every token.  Stored per case: ``<case>.json`` (configuration name, weight seed, sequences, the
positions kept) and ``<case>.f32`` (little-endian float32 ``[kept rows, vocab]``, sequence after sequence).

    python tests/golden/make_golden.py --out tests/golden

``tests/test_golden_reference.py`` compares the plain implementation with these files on the CPU.
"""
import argparse
import json
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

# (configuration of tests/helpers.py, sequence lengths, how many last positions of each sequence are kept)
CASES = {
    "tiny_a": ("A", [25, 13], None),        # BASELINE's tiny A: prompts up to 17 tokens plus 8 decoded
    "tiny_b": ("B", [52, 13, 1], None),     # tiny B: prompts up to 40 tokens plus 12 decoded; a prompt of one token
    "tiny_c": ("C", [40], 8),               # head size 48, three key/value heads
    "tiny_d": ("D", [70], 8),               # the benchmark's head geometry; crosses a 64-token page
}


def main():
    import helpers
    import reference_arm
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    for case, (name, lengths, last) in CASES.items():
        vocab = helpers.TINY[name]["vocab_size"]
        sequences = [helpers.random_tokens(vocab, n, seed=1000 + 17 * i + len(case)) for i, n in enumerate(lengths)]
        with tempfile.TemporaryDirectory() as tmp:
            folder = helpers.make_model_dir(os.path.join(tmp, "model"), name, "float32")
            logits = reference_arm.reference_logits(folder, sequences, tmp,
                                                    context=helpers.TINY[name]["max_position_embeddings"])
        kept, rows = [], []
        for seq, l in zip(sequences, logits):
            places = list(range(len(seq))) if last is None else list(range(max(0, len(seq) - last), len(seq)))
            kept.append(places)
            rows.append(l[places])
        flat = np.concatenate(rows, axis=0).astype("<f4")
        flat.tofile(os.path.join(args.out, f"{case}.f32"))
        with open(os.path.join(args.out, f"{case}.json"), "w") as f:
            json.dump({"config": name, "weights_seed": helpers.SEEDS[name], "stored": "float32",
                       "sequences": sequences, "positions": kept, "vocab": vocab,
                       "reference": "xissleah/Citlali-LLM-Engine QwenModel::forward_token, float32 GGUF, FP16 engine"},
                      f)
        print(f"{case}: {flat.shape[0]} rows of {vocab}, max |logit| {np.abs(flat).max():.4f}", flush=True)


if __name__ == "__main__":
    main()
