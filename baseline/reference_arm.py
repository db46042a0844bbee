"""The reference engine as a measuring stick: build it, give it a model file, run it.

xissleah/Citlali-LLM-Engine is a CMake/C++/CUDA program that reads GGUF files and runs one
sequence through ``citlali::model::QwenModel`` (include/citlali/model/qwen_model.h:38-42).  This
module

* copies the reference's sources beside itself and builds them unmodified with CMake for sm_100a
  (``install``; needs the reference's checkout, nvcc and cmake, no GPU), together with
  ``reference_harness.cpp``, a small program of ours that calls the reference's public class;
* writes GGUF v3 files with the metadata ``QwenConfig::from_gguf`` reads
  (src/model/qwen_config.cpp:32-124) and the tensor names ``QwenModel::load`` asks for
  (src/model/qwen_model.cpp:69-71, :103-152), from a model folder of this library or from a
  configuration and a seed;
* runs the harness: logits for given token ids (the anchor of ``tests/plain_qwen3.py``), or the
  decode rate at batch 1 (``bench.py --impl reference``).

Nothing in the package imports this file; it is test and benchmark infrastructure.
"""
from __future__ import annotations

import json
import os
import shutil
import struct
import subprocess
import sys
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
SOURCE_DIR = os.path.join(REF_DIR, "source")
BUILD_DIR = os.path.join(REF_DIR, "build")
HARNESS = os.path.join(BUILD_DIR, "reference_harness")
HARNESS_SOURCE = os.path.join(HERE, "reference_harness.cpp")

GGUF_F32, GGUF_F16 = 0, 1
_META_U32, _META_F32, _META_STRING, _META_ARRAY = 4, 6, 8, 9
_ALIGN = 32


# ---- building -------------------------------------------------------------------------------

def installed() -> Optional[str]:
    """None if the harness is built, else why it cannot be used."""
    if not os.path.isfile(HARNESS):
        return (f"the reference is not built ({os.path.relpath(HARNESS, os.path.dirname(HERE))} is missing); "
                "run `python baseline/reference_arm.py install <path to the reference>` where its checkout is")
    if not os.access(HARNESS, os.X_OK):
        return "the reference harness is not executable"
    return None


def install(reference_root: str) -> str:
    """Copy the reference's sources (its Android/Vulkan tree left out), build them with its own
    CMakeLists.txt in Release mode for sm_100a, then build the harness against the library."""
    for need in ("CMakeLists.txt", "src", "include"):
        if not os.path.exists(os.path.join(reference_root, need)):
            raise RuntimeError(f"{reference_root} does not look like the reference: {need} is missing")
    if os.path.isdir(SOURCE_DIR):
        shutil.rmtree(SOURCE_DIR)
    os.makedirs(SOURCE_DIR)
    shutil.copy(os.path.join(reference_root, "CMakeLists.txt"), SOURCE_DIR)
    for sub in ("src", "include"):
        shutil.copytree(os.path.join(reference_root, sub), os.path.join(SOURCE_DIR, sub))
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    run = lambda cmd: subprocess.run(cmd, check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    run(["cmake", "-S", SOURCE_DIR, "-B", BUILD_DIR, "-DCMAKE_BUILD_TYPE=Release",
         "-DCMAKE_CUDA_ARCHITECTURES=100a", f"-DCMAKE_CUDA_COMPILER={nvcc}"])
    run(["cmake", "--build", BUILD_DIR, "-j", "8"])
    cuda_root = os.path.dirname(os.path.dirname(nvcc))
    run(["g++", "-O2", "-std=c++17", "-I", os.path.join(SOURCE_DIR, "include"), "-I", os.path.join(cuda_root, "include"),
         HARNESS_SOURCE, os.path.join(BUILD_DIR, "libcitlali_engine.a"),
         "-L", os.path.join(cuda_root, "lib64"), "-lcudart", "-lpthread", "-ldl",
         "-Wl,-rpath," + os.path.join(cuda_root, "lib64"), "-o", HARNESS])
    return HARNESS


# ---- GGUF -----------------------------------------------------------------------------------

def _gguf_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def gguf_name(hf_name: str) -> str:
    """The reference's tensor name for one of this library's (qwen_model.cpp:69-71, :103-152)."""
    fixed = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    if hf_name in fixed:
        return fixed[hf_name]
    parts = hf_name.split(".")
    assert parts[0] == "model" and parts[1] == "layers", hf_name
    layer, rest = parts[2], ".".join(parts[3:])
    table = {"input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
             "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
             "self_attn.o_proj.weight": "attn_output.weight", "self_attn.q_norm.weight": "attn_q_norm.weight",
             "self_attn.k_norm.weight": "attn_k_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
             "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
             "mlp.down_proj.weight": "ffn_down.weight"}
    return f"blk.{layer}.{table[rest]}"


def gguf_metadata(config: dict) -> List[Tuple[str, int, object]]:
    """The keys QwenConfig::from_gguf reads, from this library's config.json keys."""
    heads = int(config["num_attention_heads"])
    meta = [
        ("general.architecture", _META_STRING, "qwen3"),
        ("qwen3.context_length", _META_U32, int(config["max_position_embeddings"])),
        ("qwen3.embedding_length", _META_U32, int(config["hidden_size"])),
        ("qwen3.block_count", _META_U32, int(config["num_hidden_layers"])),
        ("qwen3.feed_forward_length", _META_U32, int(config["intermediate_size"])),
        ("qwen3.attention.head_count", _META_U32, heads),
        ("qwen3.attention.head_count_kv", _META_U32, int(config.get("num_key_value_heads", heads))),
        ("qwen3.attention.key_length", _META_U32, int(config.get("head_dim", int(config["hidden_size"]) // heads))),
        ("qwen3.attention.layer_norm_rms_epsilon", _META_F32, float(config["rms_norm_eps"])),
        ("qwen3.rope.freq_base", _META_F32, float(config["rope_theta"])),
        # the vocabulary size is the length of this array (qwen_config.cpp:44); the strings are never used here
        ("tokenizer.ggml.tokens", _META_ARRAY, [f"t{i}" for i in range(int(config["vocab_size"]))]),
    ]
    return meta


def write_gguf(path: str, config: dict, tensors: Sequence[Tuple[str, Tuple[int, ...], int]], fetch) -> int:
    """``tensors``: (GGUF name, shape as stored row-major [out, in] or [n], GGUF type); ``fetch(name)``
    returns the tensor's bytes (a buffer of exactly that many float32 or float16 values), called in
    order while the file is written, so that a large model never sits in memory whole.  Returns the
    file's size."""
    meta = gguf_metadata(config)
    head = bytearray()
    head += b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for key, kind, value in meta:
        head += _gguf_string(key) + struct.pack("<I", kind)
        if kind == _META_U32:
            head += struct.pack("<I", value)
        elif kind == _META_F32:
            head += struct.pack("<f", value)
        elif kind == _META_STRING:
            head += _gguf_string(value)
        else:
            head += struct.pack("<IQ", _META_STRING, len(value)) + b"".join(_gguf_string(s) for s in value)
    offset = 0
    sizes = []
    for name, shape, kind in tensors:
        count = int(np.prod(shape))
        nbytes = count * (4 if kind == GGUF_F32 else 2)
        dims = tuple(reversed(shape))                 # GGUF lists the fastest axis first: [in, out]
        head += _gguf_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", kind, offset)
        sizes.append(nbytes)
        offset += (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (-len(head) % _ALIGN))
        for (name, shape, kind), nbytes in zip(tensors, sizes):
            data = fetch(name)
            view = memoryview(data).cast("B")
            assert view.nbytes == nbytes, f"{name}: {view.nbytes} bytes given, {nbytes} expected"
            f.write(view)
            f.write(b"\0" * (-nbytes % _ALIGN))
        return f.tell()


def gguf_from_model_dir(model_dir: str, path: str, kind: int = GGUF_F32) -> dict:
    """The same weights as a model folder of this library (config.json, model.safetensors), as a
    GGUF file for the reference.  Values are widened to float32, or rounded to float16."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    handle = safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt")
    names = {gguf_name(n): n for n in handle.keys()}
    order = sorted(names)
    tensors = [(g, tuple(handle.get_slice(names[g]).get_shape()), kind) for g in order]

    def fetch(g):
        import torch
        t = handle.get_tensor(names[g]).to(torch.float32 if kind == GGUF_F32 else torch.float16)
        return t.contiguous().numpy()

    write_gguf(path, config, tensors, fetch)
    return config


def gguf_random(config: dict, path: str, seed: int, device: str = "cuda:0", layers: Optional[int] = None,
                progress=None) -> int:
    """A float16 GGUF of a configuration's shape with N(0, 0.02) matrices and norm gains of 1, made
    tensor by tensor on ``device``.  The values are not those of this library's random weights (its
    generator is keyed by tensor name); for a throughput measurement only the shapes matter."""
    import torch
    config = dict(config)
    if layers is not None:
        config["num_hidden_layers"] = layers
    H, I, V = int(config["hidden_size"]), int(config["intermediate_size"]), int(config["vocab_size"])
    nq = int(config["num_attention_heads"])
    nkv = int(config.get("num_key_value_heads", nq))
    d = int(config.get("head_dim", H // nq))
    tensors = [("token_embd.weight", (V, H), GGUF_F16), ("output_norm.weight", (H,), GGUF_F32)]
    if not config.get("tie_word_embeddings", False):
        tensors.append(("output.weight", (V, H), GGUF_F16))
    for l in range(int(config["num_hidden_layers"])):
        p = f"blk.{l}."
        tensors += [(p + "attn_norm.weight", (H,), GGUF_F32), (p + "attn_q.weight", (nq * d, H), GGUF_F16),
                    (p + "attn_k.weight", (nkv * d, H), GGUF_F16), (p + "attn_v.weight", (nkv * d, H), GGUF_F16),
                    (p + "attn_output.weight", (H, nq * d), GGUF_F16), (p + "attn_q_norm.weight", (d,), GGUF_F32),
                    (p + "attn_k_norm.weight", (d,), GGUF_F32), (p + "ffn_norm.weight", (H,), GGUF_F32),
                    (p + "ffn_gate.weight", (I, H), GGUF_F16), (p + "ffn_up.weight", (I, H), GGUF_F16),
                    (p + "ffn_down.weight", (H, I), GGUF_F16)]
    shapes = {n: (s, k) for n, s, k in tensors}
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    done = [0]

    def fetch(name):
        shape, kind = shapes[name]
        if kind == GGUF_F32:
            return np.ones(shape, dtype=np.float32)
        t = torch.empty(shape, dtype=torch.float16, device=device).normal_(0.0, 0.02, generator=gen)
        done[0] += 1
        if progress and done[0] % 40 == 0:
            progress(f"reference arm: wrote {done[0]} matrices")
        return t.cpu().numpy()

    return write_gguf(path, config, tensors, fetch)


# ---- running --------------------------------------------------------------------------------

def reference_logits(model_dir: str, sequences: Sequence[Sequence[int]], work_dir: str, context: int = 256,
                     kind: int = GGUF_F32) -> List[np.ndarray]:
    """Logits of the reference at every position of every sequence (each fed alone from position 0):
    a list of float32 arrays ``[len(sequence), vocab]``."""
    why = installed()
    if why:
        raise RuntimeError(why)
    gguf = os.path.join(work_dir, "model.gguf")
    config = gguf_from_model_dir(model_dir, gguf, kind)
    ids = os.path.join(work_dir, "tokens.txt")
    with open(ids, "w") as f:
        for s in sequences:
            f.write(" ".join(str(int(t)) for t in s) + "\n")
    out = os.path.join(work_dir, "logits.f32")
    r = subprocess.run([HARNESS, "logits", "--model", gguf, "--ctx", str(context), "--tokens", ids, "--out", out],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"the reference harness failed ({r.returncode}): {r.stderr[-2000:]}")
    flat = np.fromfile(out, dtype="<f4").reshape(-1, int(config["vocab_size"]))
    result, at = [], 0
    for s in sequences:
        result.append(flat[at:at + len(s)].copy())
        at += len(s)
    return result


def reference_decode(gguf: str, context: int, prompt_tokens: int, warmup: int, steps: int, start_position: int = 0,
                     timeout: float = 1500.0) -> dict:
    """Time ``steps`` greedy decode steps of the reference after ``prompt_tokens`` prompt tokens fed one by
    one from ``start_position`` and ``warmup`` untimed steps (the harness's ``decode`` mode)."""
    why = installed()
    if why:
        raise RuntimeError(why)
    r = subprocess.run([HARNESS, "decode", "--model", gguf, "--ctx", str(context), "--prompt-tokens", str(prompt_tokens),
                        "--start-position", str(start_position), "--warmup", str(warmup), "--steps", str(steps)], capture_output=True, text=True, timeout=timeout)
    if r.returncode != 0:
        raise RuntimeError(f"the reference harness failed ({r.returncode}): {r.stderr[-2000:]}")
    return json.loads(r.stdout.strip().splitlines()[-1])


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "install":
        print(install(sys.argv[2]))
    else:
        print("usage: python baseline/reference_arm.py install <path to the reference's checkout>", file=sys.stderr)
        sys.exit(2)
