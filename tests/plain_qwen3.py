"""A plain, slow implementation of the Qwen3 dense decoder: the tests' oracle.

Each function restates one formula of the reference and cites its lines.  The reference's model
code cannot run on a CPU (every op is a CUDA kernel and every weight goes through cudaMalloc,
src/compute/cuda/tensor.cu:56), but it builds unmodified for sm_100a and runs on a B200: its own
logits for four tiny random models are stored under ``tests/golden/`` (made by
``tests/golden/make_golden.py``), and ``tests/test_golden_reference.py`` holds this file to them on
the CPU, to 1.4e-3 of the largest logit as it stands (the reference's FP16 stores) and to 8e-4 when
this oracle rounds to FP16 where the reference does (``reference_model_logits``).

Whole sequences, no cache, one function per part, no code shared with the engine: it reads the
model folder with the ``safetensors`` package and ``json``, and computes with elementary torch
operations on the CPU.

All arithmetic runs in ``dtype`` (float64 by default, which makes the result the exact
value of the formulas up to ~1e-15; float32 is there to see what 32-bit evaluation in
another order gives).  The reference rounds to 16 bits at every store
(src/compute/cuda/kernels.cu:13-24); the exact oracle leaves that out, ``store_float16`` puts it in.
"""
import json
import math
import os

import torch


# ---- reading a model folder ----------------------------------------------------------

def load_folder(model_dir):
    """config.json as a dict and every tensor as float64 on the CPU."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    raw = load_file(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: v.to(torch.float64) for k, v in raw.items()}


# ---- the parts -----------------------------------------------------------------------

def embedding(table, tokens):
    """x = E[token]: a row copy with no scaling (kernels.cu:27-35, qwen_model.cpp:267)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x, gain, eps):
    """inv = rsqrt(sum(x^2)/n + eps); y = x * inv * gain; eps inside the root, gain multiplies
    (kernels.cu:73-92)."""
    inv = torch.rsqrt((x * x).sum(dim=-1, keepdim=True) / x.shape[-1] + eps)
    return x * inv * gain


def linear(x, weight):
    """y[r] = sum_i W[r, i] x[i], W row-major [out, in], no bias (kernels.cu:381-449)."""
    return x @ weight.t()


def head_rms_norm(x, gain, eps):
    """RMSNorm over each head's d elements, one gain [d] shared by all heads, same eps as the
    layer norms (kernels.cu:95-124, qwen_model.cpp:325-330).  x: [T, heads, d]."""
    return rms_norm(x, gain, eps)


def rotary_half_split(x, positions, theta):
    """NeoX pairing (i, i + d/2): f_i = theta^(-2i/d), a = p * f_i,
    (x_i, x_{i+d/2}) <- (x_i cos a - x_{i+d/2} sin a, x_i sin a + x_{i+d/2} cos a)
    (kernels.cu:485-521).  The reference evaluates f_i and a in 32-bit; so f_i is rounded to
    float32, the product p*f_i is a float32 product, and cos/sin are taken of that value.
    x: [T, heads, d]."""
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / d).to(torch.float32)
    pos = torch.as_tensor(positions, dtype=torch.float32)
    angle = (pos[:, None] * inv_freq[None, :]).to(torch.float64)       # float32 product, then exact
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def attention_scores(q, k, num_heads, num_kv_heads):
    """s[j, t] = (q_j . k_{t, g}) / sqrt(d), query head j reads KV head g = j // (nq/nkv)
    (kernels.cu:545-602; the map is :564-565, the scale :599).  q: [heads, d] of one token,
    k: [T, kv_heads, d].  Returns [heads, T]."""
    group = num_heads // num_kv_heads
    d = q.shape[-1]
    out = torch.empty(num_heads, k.shape[0], dtype=q.dtype)
    for j in range(num_heads):
        g = j // group
        out[j] = (k[:, g, :] @ q[j]) / math.sqrt(d)
    return out


def softmax_values(scores, v, num_heads, num_kv_heads):
    """m = max_t s_t; Z = sum_t exp(s_t - m); o[j] = sum_t (exp(s_t - m) / Z) v[t, g]
    (kernels.cu:605-649).  scores: [heads, T], v: [T, kv_heads, d]."""
    group = num_heads // num_kv_heads
    out = torch.empty(num_heads, v.shape[-1], dtype=v.dtype)
    for j in range(num_heads):
        g = j // group
        e = torch.exp(scores[j] - scores[j].max())
        p = e / e.sum()
        out[j] = p @ v[:, g, :]
    return out


def causal_attention(q, k, v, num_heads, num_kv_heads, window=None):
    """Token p attends to keys t <= p: the mask is the range of the loop, there is no window
    in the reference (kernels.cu:562, :625-645).  ``window`` (keys t > p - window) exists for
    the tests of the attention part alone.  q: [T, heads, d]; k, v: [T, kv_heads, d]."""
    T = q.shape[0]
    out = torch.empty(T, num_heads, v.shape[-1], dtype=q.dtype)
    for p in range(T):
        lo = 0 if window is None else max(0, p - window + 1)
        s = attention_scores(q[p], k[lo:p + 1], num_heads, num_kv_heads)
        out[p] = softmax_values(s, v[lo:p + 1], num_heads, num_kv_heads)
    return out


def swiglu(gate, up):
    """act = (g / (1 + exp(-g))) * u (kernels.cu:474-482)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def keep(t):
    """No rounding at a store: what the exact oracle does."""
    return t


def store_float16(t):
    """The reference's rounding at every store of an activation: its buffers hold FP16 bits and each
    kernel widens, computes in float and rounds once (kernels.cu:13-24).  With this as ``store`` (and
    weights rounded to FP16, src/model/weight_loader.cpp:457-459) the oracle follows the reference's
    own arithmetic; the scores and the logits stay unrounded as there (kernels.cu:599, :452-471)."""
    return t.to(torch.float16).to(t.dtype)


def attention_block(h, w, prefix, cfg, positions, store=keep):
    """q, k, v projections; q_norm and k_norm per head before the rotation; v untouched;
    attention; output projection (qwen_model.cpp:315-351).  ``store`` is applied wherever the
    reference writes a buffer: after each projection, each head norm, the rotation, the attention
    output and the output projection."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    T = h.shape[0]
    q = store(linear(h, w[f"{prefix}.q_proj.weight"])).view(T, nq, d)
    k = store(linear(h, w[f"{prefix}.k_proj.weight"])).view(T, nkv, d)
    v = store(linear(h, w[f"{prefix}.v_proj.weight"])).view(T, nkv, d)
    q = store(head_rms_norm(q, w[f"{prefix}.q_norm.weight"], eps))
    k = store(head_rms_norm(k, w[f"{prefix}.k_norm.weight"], eps))
    q = store(rotary_half_split(q, positions, cfg["rope_theta"]))
    k = store(rotary_half_split(k, positions, cfg["rope_theta"]))
    o = store(causal_attention(q, k, v, nq, nkv)).reshape(T, nq * d)
    return store(linear(o, w[f"{prefix}.o_proj.weight"]))


def feed_forward(h, w, prefix, store=keep):
    """gate and up projections, SiLU gate, down projection (qwen_model.cpp:360-370)."""
    g = store(linear(h, w[f"{prefix}.gate_proj.weight"]))
    u = store(linear(h, w[f"{prefix}.up_proj.weight"]))
    return store(linear(store(swiglu(g, u)), w[f"{prefix}.down_proj.weight"]))


def decoder_layer(x, w, i, cfg, positions, store=keep):
    """norm -> attention -> x += ; norm -> feed-forward -> x += (qwen_model.cpp:306-374).  The
    reference's residual stream is a 16-bit buffer too (kernels.cu:53-59): the sums are stored."""
    base = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    x = store(x + attention_block(store(rms_norm(x, w[f"{base}.input_layernorm.weight"], eps)), w,
                                  f"{base}.self_attn", cfg, positions, store))
    x = store(x + feed_forward(store(rms_norm(x, w[f"{base}.post_attention_layernorm.weight"], eps)), w,
                               f"{base}.mlp", store))
    return x


def head_weight(w):
    """The output matrix; absent means tied to the embedding (qwen_model.cpp:71-75)."""
    return w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]


def model_logits(cfg, w, tokens, dtype=torch.float64, store=keep):
    """Logits [T, vocab] at every position of one whole sequence (qwen_model.cpp:239-414):
    embedding, the layers, final norm, output matrix with no bias and no scaling."""
    w = {k: v.to(dtype) for k, v in w.items()}
    T = len(tokens)
    positions = list(range(T))
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions, store)
    h = store(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    return linear(h, head_weight(w))


def reference_model_logits(cfg, w, tokens):
    """The oracle run the reference's way: weights rounded to FP16 as its loader stores them, every
    activation rounded to FP16 where it writes a buffer."""
    w16 = {k: v.to(torch.float16).to(torch.float64) for k, v in w.items()}
    return model_logits(cfg, w16, tokens, torch.float64, store_float16)


# ---- sampling and the generation loop --------------------------------------------------

def greedy(logits):
    """Scan in index order, skip non-finite values, strict '>' so the lowest index wins ties,
    start at -inf with id 0 (qwen_model.cpp:448-465)."""
    best, best_id = -math.inf, 0
    for i, v in enumerate(logits.tolist()):
        if math.isfinite(v) and v > best:
            best, best_id = v, i
    return best_id


def temperature_cdf(logits, temperature):
    """Inclusive CDF of softmax(logits / temperature) in index order; non-finite logits get no
    mass.  (No counterpart in the reference, which samples greedily only, README.md:472.)"""
    l = logits.to(torch.float64)
    finite = torch.isfinite(l)
    l = torch.where(finite, l, torch.full_like(l, -math.inf))
    e = torch.where(finite, torch.exp((l - l[finite].max()) / temperature), torch.zeros_like(l))
    return torch.cumsum(e, 0) / e.sum()


def temperature_sample(logits, temperature, u):
    """The first index whose inclusive CDF exceeds u in [0, 1)."""
    cdf = temperature_cdf(logits, temperature)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float64), right=True))
    return min(idx, logits.numel() - 1)


def generate_greedy(cfg, w, prompt, max_new_tokens, stop_ids=(), max_context=None):
    """The reference's loop for one sequence (src/runtime/session.cpp:61-104): the stop test
    comes first and a stop token is neither emitted nor fed; every step re-runs the whole
    sequence here since there is no cache.  Returns (tokens, stop_reason)."""
    seq, out = list(prompt), []
    while True:
        nxt = greedy(model_logits(cfg, w, seq)[-1])
        if nxt in stop_ids:
            return out, "eos"
        out.append(nxt)
        seq.append(nxt)
        if len(out) >= max_new_tokens:
            return out, "max_new_tokens"
        if max_context is not None and len(seq) >= max_context:
            return out, "context_limit"
