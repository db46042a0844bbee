"""Each part alone, built through the registries with sizes the models do not use, against the
plain implementation's function for that part."""

import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
from citlali_b200.cache import SequenceCache
from citlali_b200.engine.step import StepEntry, pack_step
from citlali_b200.parts import BuildContext, part_class
from citlali_b200.parts.linear import DenseLinear
from citlali_b200.weights.loader import WeightHandle
from citlali_b200.weights.random_init import random_weights

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def ctx_for(dtype):
    return BuildContext(DEV, dtype, torch.zeros(4, dtype=torch.int32, device=DEV))


def handles(part, dtype, seed=1, gain_spread=0.3):
    w = random_weights(part.tensor_specs(), seed, dtype, matrix_std=0.2, gain_spread=gain_spread)
    return {n: WeightHandle(n, t.dtype, tuple(t.shape), t) for n, t in w.items()}, {n: t.double() for n, t in w.items()}


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype):
    scale = float(want.abs().max())
    err = float((got.double().cpu() - want).abs().max())
    assert err <= tol(dtype) * scale, f"|diff| {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    norm = part_class("norm", "rms_norm")({"size": 70, "eps": 1e-4}, "n")
    h, w = handles(norm, dtype)
    norm.bind(h, ctx_for(dtype))
    x = torch.randn(6, 70) * 2
    close(norm.forward(x.to(DEV)), plain.rms_norm(x.double(), w["n.weight"], 1e-4), dtype)
    idx = torch.tensor([5, 1], dtype=torch.int32, device=DEV)
    close(norm.forward(x.to(DEV), row_index=idx), plain.rms_norm(x.double()[[5, 1]], w["n.weight"], 1e-4), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_part_stacked_and_interleaved(dtype):
    ctx = ctx_for(dtype)
    lin = DenseLinear(["a", "b", "c"], [10, 6, 6], 24)
    h, w = handles(lin, dtype)
    lin.bind(h, ctx)
    x = torch.randn(5, 24).to(dtype)
    y = lin.forward(x.to(DEV))
    close(y, torch.cat([plain.linear(x.double(), w[n]) for n in "abc"], dim=1), dtype)
    res = torch.randn(5, 22)
    got = lin.forward(x.to(DEV), accumulate_into=res.to(DEV).clone())
    assert got.dtype == torch.float32
    close(got, res.double() + torch.cat([plain.linear(x.double(), w[n]) for n in "abc"], dim=1),
          torch.float32 if dtype == torch.float32 else dtype)
    inter = DenseLinear(["g", "u"], [32, 32], 24, interleave_run=16)
    h, w = handles(inter, dtype)
    inter.bind(h, ctx)
    y = inter.forward(x.to(DEV)).double().cpu().view(5, 2, 2, 16)
    close(y[:, :, 0].reshape(5, 32), plain.linear(x.double(), w["g"]), dtype)
    close(y[:, :, 1].reshape(5, 32), plain.linear(x.double(), w["u"]), dtype)
    with pytest.raises(cb.CitlaliError, match="unexpected tensor shape for a"):
        bad = dict(h); bad["a"] = WeightHandle("a", dtype, (3, 3), torch.zeros(3, 3, dtype=dtype))
        bad.update({"b": h["g"], "c": h["g"]}); lin.bind(bad, ctx)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [48, 50])
def test_feed_forward_part(dtype, inter):
    ff = part_class("feed_forward", "gated_silu")({"hidden_size": 40, "intermediate_size": inter}, "mlp")
    h, w = handles(ff, dtype)
    ff.bind(h, ctx_for(dtype))
    x = torch.randn(7, 40).to(dtype)
    res = torch.randn(7, 40)
    out = ff.forward(x.to(DEV), None, res.to(DEV).clone())
    close(out, res.double() + plain.feed_forward(x.double(), w, "mlp"), dtype)


ATTN = {"hidden_size": 40, "num_heads": 6, "num_kv_heads": 2, "head_dim": 48, "qk_norm_eps": 1e-5,
        "position": {"kind": "rotary_half_split", "theta": 3e4, "rotary_dim": 48}, "window": None}


class InterleavedRotary:
    """A position encoding defined here, with work of its own: pairs (2i, 2i + 1) of every q and k head are rotated
    by position * theta^(-2i/d).  It gives no frequency table, so the attention part calls ``apply``."""
    inv_freq = None

    def __init__(self, params, head_dim):
        self.theta, self.rotary_dim = float(params["theta"]), head_dim

    def apply(self, qkv, batch, num_q_heads, num_kv_heads, head_dim):
        rows = qkv.shape[0]
        heads = qkv[:, :(num_q_heads + num_kv_heads) * head_dim].view(rows, num_q_heads + num_kv_heads, head_dim // 2, 2)
        i = torch.arange(head_dim // 2, dtype=torch.float64, device=qkv.device)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64, device=qkv.device), -2.0 * i / head_dim).float()
        angle = batch.row_pos.float()[:, None] * inv[None, :]
        c, s_ = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        a, b = heads[..., 0].float(), heads[..., 1].float()
        heads[..., 0], heads[..., 1] = (a * c - b * s_).to(qkv.dtype), (a * s_ + b * c).to(qkv.dtype)


def plain_interleaved_rotary(t, positions, theta):
    d = t.shape[-1]
    i = torch.arange(d // 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / d).to(torch.float32)
    ang = (torch.tensor(positions, dtype=torch.float32)[:, None] * inv[None, :]).double()
    c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    pairs = t.reshape(*t.shape[:-1], d // 2, 2)
    a, b = pairs[..., 0], pairs[..., 1]
    return torch.stack([a * c - b * s_, a * s_ + b * c], dim=-1).reshape(t.shape)


def plain_attention_part(x, w, params, window=None, qk_norm=True, rotate=True):
    T = x.shape[0]
    nq, nkv, d = params["num_heads"], params["num_kv_heads"], params["head_dim"]
    q = plain.linear(x, w["a.q_proj.weight"]).view(T, nq, d)
    k = plain.linear(x, w["a.k_proj.weight"]).view(T, nkv, d)
    v = plain.linear(x, w["a.v_proj.weight"]).view(T, nkv, d)
    if qk_norm:
        q = plain.head_rms_norm(q, w["a.q_norm.weight"], params["qk_norm_eps"])
        k = plain.head_rms_norm(k, w["a.k_norm.weight"], params["qk_norm_eps"])
    if rotate == "interleaved":
        q = plain_interleaved_rotary(q, list(range(T)), params["position"]["theta"])
        k = plain_interleaved_rotary(k, list(range(T)), params["position"]["theta"])
    elif rotate:
        r = params["position"].get("rotary_dim", d)           # the first r elements of a head are rotated
        theta = params["position"]["theta"]
        q = torch.cat([plain.rotary_half_split(q[..., :r], list(range(T)), theta), q[..., r:]], dim=-1)
        k = torch.cat([plain.rotary_half_split(k[..., :r], list(range(T)), theta), k[..., r:]], dim=-1)
    o = plain.causal_attention(q, k, v, nq, nkv, window=window).reshape(T, nq * d)
    return plain.linear(o, w["a.o_proj.weight"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("variant", ["plain", "window", "no_norm_no_rotation", "partial_rotation", "position_with_apply"])
def test_attention_part_whole_and_token_by_token(dtype, variant):
    params = dict(ATTN)
    kwargs = {}
    if variant == "partial_rotation":
        params["position"] = {"kind": "rotary_half_split", "theta": 3e4, "rotary_dim": 16}
    if variant == "position_with_apply":
        cb.register_part("position", "interleaved_rotary", InterleavedRotary, replace=True)
        params["position"] = {"kind": "interleaved_rotary", "theta": 3e4}
        kwargs["rotate"] = "interleaved"
    if variant == "window":
        params["window"] = 9; kwargs["window"] = 9
    if variant == "no_norm_no_rotation":
        params["qk_norm_eps"] = None; params["position"] = {"kind": "none"}
        kwargs.update(qk_norm=False, rotate=False)
    attn = part_class("mixer", "gqa_attention")(params, "a")
    h, w = handles(attn, dtype, gain_spread=0.5)
    ctx = ctx_for(dtype)
    attn.bind(h, ctx)
    cache = SequenceCache([attn.cache_requirement()], 2, 64 * 6, 64 * 3, dtype, DEV)
    assert cache.kv_groups[0].requirement.window == params["window"]
    T = 75
    x = torch.randn(T, 40).to(dtype)
    want = plain_attention_part(x.double(), w, params, **kwargs)
    slot = cache.acquire(); other = cache.acquire()

    def run(sl, lo, hi):
        past = cache.length(sl)
        batch = pack_step([StepEntry(sl, [0] * (hi - lo), [])], [past], 10, DEV)
        cache.reserve(sl, hi)
        res = torch.zeros(hi - lo, 40, device=DEV)
        attn.forward(x[lo:hi].to(DEV).contiguous(), batch, cache.view(0), res)
        cache.commit(sl, hi)
        return res
    whole = run(slot, 0, T)
    close(whole, want, dtype)
    pieces = [run(other, 0, 40)] + [run(other, t, t + 1) for t in range(40, T)]
    close(torch.cat(pieces), want, dtype)
    if dtype == torch.float32:
        assert torch.equal(torch.cat(pieces), whole)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    spec = cb.LayerSpec(block="pre_norm_residual", parts={
        "mixer_norm": cb.PartSpec("rms_norm", {"size": 40, "eps": 1e-5}, "n1"),
        "mixer": cb.PartSpec("gqa_attention", dict(ATTN), "a"),
        "feed_forward_norm": cb.PartSpec("rms_norm", {"size": 40, "eps": 2e-5}, "n2"),
        "feed_forward": cb.PartSpec("gated_silu", {"hidden_size": 40, "intermediate_size": 48}, "mlp")})
    block = part_class("block", "pre_norm_residual")(spec)
    h, w = handles(block, dtype)
    block.bind(h, ctx_for(dtype))
    cache = SequenceCache([block.cache_requirement()], 1, 128, 128, dtype, DEV)
    slot = cache.acquire()
    T = 20
    x = torch.randn(T, 40)
    batch = pack_step([StepEntry(slot, [0] * T, [])], [0], 10, DEV)
    cache.reserve(slot, T)
    got = block.forward(x.to(DEV).clone(), batch, cache.view(0))
    xd = x.double()
    xd = xd + plain_attention_part(plain.rms_norm(xd, w["n1.weight"], 1e-5), w, ATTN)
    xd = xd + plain.feed_forward(plain.rms_norm(xd, w["n2.weight"], 2e-5), w, "mlp")
    close(got, xd, dtype)


@pytest.mark.parametrize("rows", [1, 20, 128, 129, 300])
def test_block_with_its_norms_inside_the_products(rows):
    """bfloat16, a width that is a multiple of 32: up to 128 rows the block's two norms run inside the products around
    them (the gain folded into the weights behind it, the rows emitted un-normalised with their sums of squares); from
    129 rows on the norm kernels run, without the gain.  Both against the plain block; and what one block leaves for
    the next block's first norm is taken up by it."""
    attn = {"hidden_size": 96, "num_heads": 6, "num_kv_heads": 2, "head_dim": 32, "qk_norm_eps": 1e-5,
            "position": {"kind": "rotary_half_split", "theta": 3e4, "rotary_dim": 32}, "window": None}
    spec = cb.LayerSpec(block="pre_norm_residual", parts={
        "mixer_norm": cb.PartSpec("rms_norm", {"size": 96, "eps": 1e-5}, "n1"),
        "mixer": cb.PartSpec("gqa_attention", dict(attn), "a"),
        "feed_forward_norm": cb.PartSpec("rms_norm", {"size": 96, "eps": 2e-5}, "n2"),
        "feed_forward": cb.PartSpec("gated_silu", {"hidden_size": 96, "intermediate_size": 160}, "mlp")})
    dtype = torch.bfloat16
    block = part_class("block", "pre_norm_residual")(spec)
    h, w = handles(block, dtype, gain_spread=0.5)
    block.bind(h, ctx_for(dtype))
    assert block.norms_in_products and torch.equal(block.mixer_norm.gain, torch.ones_like(block.mixer_norm.gain))
    cache = SequenceCache([block.cache_requirement()], 1, 512, 512, dtype, DEV)
    slot = cache.acquire()
    x = torch.randn(rows, 96) * 2
    batch = pack_step([StepEntry(slot, [0] * rows, [])], [0], 10, DEV)
    cache.reserve(slot, rows)
    got = block.forward(x.to(DEV).clone(), batch, cache.view(0))
    xd = x.double()
    xd = xd + plain_attention_part(plain.rms_norm(xd, w["n1.weight"], 1e-5), w, attn)
    xd = xd + plain.feed_forward(plain.rms_norm(xd, w["n2.weight"], 2e-5), w, "mlp")
    close(got, xd, dtype)
    carried = batch.norm_carry
    if rows <= 128:
        assert carried is not None and torch.equal(carried.rows, got.to(torch.bfloat16))
        want = (got.double().cpu() ** 2).view(rows, 3, 32).sum(-1)
        assert float((carried.sumsq.double().cpu() - want).abs().max()) <= 1e-5 * float(want.max())
        # the same block again on the updated rows: with what it left itself, and without (the rows re-read)
        cache.commit(slot, rows); cache.rewind(slot, 0)
        batch.norm_carry_in, batch.norm_carry = carried, None
        with_carry = block.forward(got.clone(), batch, cache.view(0))
        batch.norm_carry_in = batch.norm_carry = None
        without = block.forward(got.clone(), batch, cache.view(0))
        assert float((with_carry - without).abs().max()) <= 1e-6 * float(without.abs().max())
    else:
        assert carried is None
    # the 32-bit path keeps its norms as they are
    block32 = part_class("block", "pre_norm_residual")(spec)
    h32, _ = handles(block32, torch.float32, gain_spread=0.5)
    block32.bind(h32, ctx_for(torch.float32))
    assert not block32.norms_in_products


def test_unknown_kinds_are_named():
    with pytest.raises(cb.CitlaliError, match="unknown mixer kind 'conv'.*gqa_attention"):
        part_class("mixer", "conv")
    with pytest.raises(cb.CitlaliError, match="unknown part role"):
        part_class("pooling", "x")
