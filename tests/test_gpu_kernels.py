"""Each kernel alone against the plain implementation, at sizes the engine's models do not use,
with inputs made so that a fault shows (a far key among hundreds, a window's edge, shuffled
cache pages, ties and non-finite logits)."""
import math
import random

import pytest
import torch

import citlali_b200 as cb
import plain_qwen3 as plain
from citlali_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-6 if dtype == torch.float32 else 2 ** -8


def close(got, want, dtype, scale=None):
    want = want.double()
    scale = float(want.abs().max()) if scale is None else scale
    err = float((got.double().cpu() - want.cpu()).abs().max())
    assert err <= tol(dtype) * max(scale, 1e-30), f"|diff| {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 130, 17), (70, 65, 100), (129, 7, 333), (64, 64, 16)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_simt(M, N, K, dtype):
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).to(dtype); w = torch.randn(N, K, generator=g).to(dtype)
    want = x.double() @ w.double().t()
    y = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.gemm_simt(x.to(DEV), w.to(DEV), y)
    close(y, want, dtype)
    y32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_simt(x.to(DEV), w.to(DEV), y32)
    close(y32, want, torch.float32, scale=float(want.abs().max()) * (1 if dtype == torch.float32 else 1))
    base = torch.randn(M, N, generator=g)
    acc = base.clone().to(DEV)
    ops.gemm_simt(x.to(DEV), w.to(DEV), acc, accumulate=True)
    close(acc, base.double() + want, torch.float32)
    with pytest.raises(cb.CitlaliError, match="float32 output"):
        ops.gemm_simt(x.to(DEV), w.to(DEV), y.to(torch.bfloat16), accumulate=True)


def test_gemm_rows_do_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(77, 200, generator=g).to(DEV); w = torch.randn(90, 200, generator=g).to(DEV)
    full = torch.empty(77, 90, device=DEV); ops.gemm_simt(x, w, full)
    one = torch.empty(1, 90, device=DEV); ops.gemm_simt(x[40:41].contiguous(), w, one)
    assert torch.equal(full[40:41], one)


@pytest.mark.parametrize("hidden", [1, 100, 777, 4104])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gain_dtype", DTYPES)
def test_rms_norm(hidden, dtype, gain_dtype):
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(9, hidden, generator=g) * 3
    gain = (1 + 0.3 * torch.randn(hidden, generator=g)).to(gain_dtype)
    eps = 1e-3
    out = torch.empty(9, hidden, dtype=dtype, device=DEV)
    ops.rms_norm(x.to(DEV), gain.to(DEV), eps, out)
    close(out, plain.rms_norm(x.double(), gain.double(), eps), dtype)
    idx = torch.tensor([8, 0, 3], dtype=torch.int32)
    out = torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops.rms_norm(x.to(DEV), gain.to(DEV), eps, out, idx.to(DEV))
    close(out, plain.rms_norm(x.double()[idx.long()], gain.double(), eps), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_rows_and_the_fault_word(dtype):
    table = torch.randn(50, 24).to(dtype)
    toks = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    out = torch.empty(4, 24, device=DEV)
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.embed_rows(table.to(DEV), toks.to(DEV), out, flag)
    assert torch.equal(out.cpu(), plain.embedding(table, toks.tolist()).float()) and flag.tolist() == [0, 0, 0, 0]
    ops.embed_rows(table.to(DEV), torch.tensor([1, 50, -1, 2], dtype=torch.int32, device=DEV), out, flag)
    assert flag[0].item() == 1 and float(out[1].abs().sum()) == 0.0 and float(out[0].abs().sum()) > 0


def test_a_wait_that_runs_out_reports_and_leaves_the_device_usable():
    """The tensor-core kernels wait on their barriers through one function that gives up after a time limit.
    Here it waits two milliseconds on a barrier on which nothing arrives: it returns false, raises the block's
    abort word for the other threads, records its code and block in the fault word, and the kernel ends
    normally; a session that owns the fault word reports it and clears it, and the next product is right."""
    import tempfile
    from helpers import make_model_dir
    with tempfile.TemporaryDirectory() as tmp:
        make_model_dir(tmp, "A", "bfloat16")
        session = cb.InferenceSession().load_model(tmp, max_context=64, dtype="bfloat16", max_batch=2)
        flag = session.model.ctx.error_flag
        assert flag.tolist() == [0, 0, 0, 0]
        ok, abort = ops.wait_selftest(flag, limit_ms=2.0)
        assert (ok, abort) == (0, 1)
        assert flag.tolist()[1:3] == [900, 0]
        with pytest.raises(cb.CitlaliError, match="900"):
            session.check_device_errors()
        session.check_device_errors()               # reported once, then clear
        out = session.generate([[1, 2, 3]], cb.GenerationOptions(max_new_tokens=2, stop_ids=[]))
        assert len(out[0].tokens) == 2
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8, 256, generator=g).to(torch.bfloat16); w = torch.randn(128, 256, generator=g).to(torch.bfloat16)
    y = torch.empty(8, 128, device=DEV)
    ops.gemm_tc(x.to(DEV), w.to(DEV), y)
    close(y, x.double() @ w.double().t(), torch.float32)
    with pytest.raises(cb.CitlaliError, match="one second"):
        ops.wait_selftest(torch.zeros(4, dtype=torch.int32, device=DEV), limit_ms=5000.0)


@pytest.mark.parametrize("inter,run", [(48, 16), (50, 50), (160, 16), (7, 1)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(inter, run, dtype):
    g = torch.Generator().manual_seed(inter)
    gate = (torch.randn(5, inter, generator=g) * 3).to(dtype); up = torch.randn(5, inter, generator=g).to(dtype)
    packed = torch.stack([gate.view(5, -1, run), up.view(5, -1, run)], dim=2).reshape(5, 2 * inter)
    act = torch.empty(5, inter, dtype=dtype, device=DEV)
    ops.swiglu(packed.to(DEV).contiguous(), act, run)
    close(act, plain.swiglu(gate.double(), up.double()), dtype)
    with pytest.raises(cb.CitlaliError, match="does not divide"):
        ops.swiglu(packed.to(DEV).contiguous(), act, 3 if inter % 3 else 11)


def make_paged(k, v, lengths, page_size, dtype, slots_of=None, extra_pages=3, seed=0):
    """Lay per-sequence keys/values [T, nkv, d] out in shuffled pages.  Returns pools, table."""
    nkv, d = k[0].shape[1], k[0].shape[2]
    need = [(n + page_size - 1) // page_size for n in lengths]
    total = sum(need) + extra_pages
    order = list(range(total)); random.Random(seed).shuffle(order)
    slots_of = slots_of or list(range(len(lengths)))
    table = torch.zeros(max(slots_of) + 1, max(need) + 1, dtype=torch.int32)
    kp = torch.randn(total, nkv, page_size, d).mul(50).to(dtype)      # junk where nothing was written
    vp = torch.randn(total, nkv, page_size, d).mul(50).to(dtype)
    nxt = 0
    for s, n, ks, vs in zip(slots_of, lengths, k, v):
        for i in range((n + page_size - 1) // page_size):
            page = order[nxt]; nxt += 1
            table[s, i] = page
            lo, hi = i * page_size, min(n, (i + 1) * page_size)
            kp[page, :, :hi - lo] = ks[lo:hi].transpose(0, 1).to(dtype)
            vp[page, :, :hi - lo] = vs[lo:hi].transpose(0, 1).to(dtype)
    return kp, vp, table


@pytest.mark.parametrize("nq,nkv,d,page", [(4, 2, 16, 64), (6, 3, 48, 8), (5, 5, 80, 64), (8, 1, 128, 16), (2, 2, 256, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_qk_norm_rope_cache(nq, nkv, d, page, dtype):
    g = torch.Generator().manual_seed(d)
    lengths = [70, 3]                      # rows: sequence 0 brings positions 66..69, sequence 1 positions 0..2
    slots = [2, 0]
    rows_pos = [66, 67, 68, 69, 0, 1, 2]
    rows_slot = [2, 2, 2, 2, 0, 0, 0]
    M = len(rows_pos)
    qkv = torch.randn(M, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qg = (1 + 0.2 * torch.randn(d, generator=g)).to(dtype); kg = (1 + 0.2 * torch.randn(d, generator=g)).to(dtype)
    theta, eps = 1e4, 1e-5
    i = torch.arange(d // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2 * i / d).float()
    empty = [torch.zeros(n, nkv, d) for n in lengths]
    kp, vp, table = make_paged(empty, empty, lengths, page, dtype, slots_of=slots)
    kp, vp = kp.to(DEV), vp.to(DEV)
    before_k = kp.clone()
    dev = qkv.to(DEV).clone()
    ops.qk_norm_rope_cache(dev, qg.to(DEV), kg.to(DEV), inv_freq.to(DEV), d, torch.tensor(rows_slot, dtype=torch.int32, device=DEV),
                           torch.tensor(rows_pos, dtype=torch.int32, device=DEV), table.to(DEV), kp, vp, page, nq, nkv, d, eps)
    x = qkv.double()
    q = x[:, :nq * d].view(M, nq, d); k = x[:, nq * d:(nq + nkv) * d].view(M, nkv, d); v = x[:, (nq + nkv) * d:].view(M, nkv, d)
    q_want = plain.rotary_half_split(plain.head_rms_norm(q, qg.double(), eps), rows_pos, theta)
    k_want = plain.rotary_half_split(plain.head_rms_norm(k, kg.double(), eps), rows_pos, theta)
    close(dev[:, :nq * d].view(M, nq, d), q_want, dtype)
    touched = torch.zeros_like(kp, dtype=torch.bool)
    for r in range(M):
        pg = table[rows_slot[r], rows_pos[r] // page].item(); off = rows_pos[r] % page
        close(kp[pg, :, off], k_want[r], dtype, scale=float(k_want.abs().max()))
        assert torch.equal(vp[pg, :, off].cpu(), v[r].to(dtype))          # values are copied as they are
        touched[pg, :, off] = True
    assert torch.equal(kp[~touched], before_k[~touched])                  # nothing else was written
    # a layer that reads another layer's cache writes nothing
    kp2 = before_k.clone()
    ops.qk_norm_rope_cache(qkv.to(DEV).clone(), qg.to(DEV), kg.to(DEV), inv_freq.to(DEV), d,
                           torch.tensor(rows_slot, dtype=torch.int32, device=DEV), torch.tensor(rows_pos, dtype=torch.int32, device=DEV),
                           table.to(DEV), kp2, vp, page, nq, nkv, d, eps, write_cache=False)
    assert torch.equal(kp2, before_k)


@pytest.mark.parametrize("nq,nkv,d,rot,page", [(4, 2, 16, 8, 64), (6, 3, 48, 16, 8), (2, 1, 20, 10, 64), (2, 2, 256, 64, 64),
                                                (3, 1, 128, 2, 16)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_qk_norm_rope_cache_partial_rotation_and_keys_kept_in_the_row(nq, nkv, d, rot, page, dtype):
    """Only the first `rot` elements of a head are rotated, in pairs (i, i + rot/2); the rest are normed and pass
    through.  And the two-call form a position encoding with work of its own uses: the first call leaves the normed
    keys in the row and the cache alone, the second (no gains, zero frequencies) stores keys and values."""
    g = torch.Generator().manual_seed(d + rot)
    lengths, slots = [70, 3], [1, 0]
    rows_pos = [66, 67, 68, 69, 0, 1, 2]
    rows_slot = [1, 1, 1, 1, 0, 0, 0]
    M = len(rows_pos)
    qkv = torch.randn(M, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qg = (1 + 0.2 * torch.randn(d, generator=g)).to(dtype); kg = (1 + 0.2 * torch.randn(d, generator=g)).to(dtype)
    theta, eps = 1e4, 1e-5
    i = torch.arange(rot // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2 * i / rot).float()
    empty = [torch.zeros(n, nkv, d) for n in lengths]
    kp, vp, table = make_paged(empty, empty, lengths, page, dtype, slots_of=slots)
    kp, vp = kp.to(DEV), vp.to(DEV)
    before_k, before_v = kp.clone(), vp.clone()
    slot_t = torch.tensor(rows_slot, dtype=torch.int32, device=DEV)
    pos_t = torch.tensor(rows_pos, dtype=torch.int32, device=DEV)
    x = qkv.double()
    q = x[:, :nq * d].view(M, nq, d); k = x[:, nq * d:(nq + nkv) * d].view(M, nkv, d); v = x[:, (nq + nkv) * d:].view(M, nkv, d)

    def partly_rotated(t, gain):
        n = plain.head_rms_norm(t, gain.double(), eps)
        return torch.cat([plain.rotary_half_split(n[..., :rot], rows_pos, theta), n[..., rot:]], dim=-1)
    q_want, k_want = partly_rotated(q, qg), partly_rotated(k, kg)
    # one call: rotate part of the head, store
    dev = qkv.to(DEV).clone()
    ops.qk_norm_rope_cache(dev, qg.to(DEV), kg.to(DEV), inv_freq.to(DEV), rot, slot_t, pos_t, table.to(DEV), kp, vp, page,
                           nq, nkv, d, eps)
    close(dev[:, :nq * d].view(M, nq, d), q_want, dtype)
    for r in range(M):
        pg = table[rows_slot[r], rows_pos[r] // page].item(); off = rows_pos[r] % page
        close(kp[pg, :, off], k_want[r], dtype, scale=float(k_want.abs().max()))
        assert torch.equal(vp[pg, :, off].cpu(), v[r].to(dtype))
    # two calls: keys stay in the row first, the cache is written by the second
    kp2, vp2 = before_k.clone(), before_v.clone()
    dev2 = qkv.to(DEV).clone()
    ops.qk_norm_rope_cache(dev2, qg.to(DEV), kg.to(DEV), inv_freq.to(DEV), rot, slot_t, pos_t, table.to(DEV), kp2, vp2, page,
                           nq, nkv, d, eps, write_cache="keys_in_place")
    assert torch.equal(kp2, before_k) and torch.equal(vp2, before_v)
    assert torch.equal(dev2[:, :nq * d], dev[:, :nq * d])
    close(dev2[:, nq * d:(nq + nkv) * d].view(M, nkv, d), k_want, dtype)
    assert torch.equal(dev2[:, (nq + nkv) * d:].cpu(), qkv[:, (nq + nkv) * d:])
    ops.qk_norm_rope_cache(dev2, None, None, torch.zeros(d // 2, device=DEV), d, slot_t, pos_t, table.to(DEV), kp2, vp2, page,
                           nq, nkv, d, eps)
    assert torch.equal(kp2, kp) and torch.equal(vp2, vp)
    with pytest.raises(cb.CitlaliError, match="rotated part"):
        ops.qk_norm_rope_cache(dev2, None, None, torch.zeros((d + 2) // 2, device=DEV), d + 2, slot_t, pos_t, table.to(DEV),
                               kp2, vp2, page, nq, nkv, d, eps)


@pytest.mark.parametrize("M,N,K,splits", [(1, 64, 64, 0), (8, 4096, 1024, 0), (8, 4096, 1024, 1), (16, 96, 512, 2), (40, 160, 256, 4),
                                          (64, 2048, 2048, 0), (128, 256, 1024, 8), (5, 32, 8, 0)])
def test_products_that_do_a_norms_work(M, N, K, splits):
    """A product that adds into the residual rows also emits those rows as bfloat16 with the sums of their squares over
    groups of 32 features; the product behind it reads the rows un-normalised, with the norm's gain in its weights, and
    scales its result rows: together the numbers of norm -> product, without the norm's kernel.  Split and unsplit."""
    g = torch.Generator().manual_seed(M * N + K)
    act = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    x0 = torch.randn(M, N, generator=g) * 3
    x = x0.to(DEV).clone()
    rows = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    sums = torch.full((M, N // 32), float("nan"), dtype=torch.float32, device=DEV)
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.gemm_tc(act.to(DEV), w1.to(DEV), x, accumulate=True, error_flag=flag, force_splits=splits, emit=(rows, sums))
    want_x = x0.double() + act.double() @ w1.double().t()
    close(x, want_x, torch.float32, scale=float(want_x.abs().max()))
    assert torch.equal(rows, x.to(torch.bfloat16))                       # the very rows that were written, rounded once
    want_sums = (x.double().cpu() ** 2).view(M, N // 32, 32).sum(-1)
    assert float((sums.double().cpu() - want_sums).abs().max()) <= 1e-5 * float(want_sums.abs().max())
    # the same call without emitting gives the same rows bit for bit
    plain_x = x0.to(DEV).clone()
    ops.gemm_tc(act.to(DEV), w1.to(DEV), plain_x, accumulate=True, error_flag=flag, force_splits=splits)
    assert float((plain_x - x).abs().max()) <= 1e-6 * float(want_x.abs().max())
    # the product behind: rms_norm(x) * gain . w2^T, as (x . (gain * w2)^T) * inv_rms(x), stored and gated
    eps = 1e-5
    gain = 1 + 0.3 * torch.randn(N, generator=g)
    N2 = 96
    w2 = (torch.randn(N2, N, generator=g) * 0.05).to(torch.bfloat16)
    w2g = (w2.float() * gain[None, :]).to(torch.bfloat16)
    # the oracle takes the operands as the kernel gets them (rows and weights already rounded to bfloat16), in the
    # kernel's grouping: the plain norm's numbers up to that rounding of the operands
    inv = torch.rsqrt((x.double().cpu() ** 2).sum(-1, keepdim=True) / N + eps)
    want = (rows.double().cpu() @ w2g.double().t()) * inv
    h = plain.rms_norm(x.double().cpu(), gain.double(), eps)
    assert float((want - h @ w2.double().t()).abs().max()) <= 2e-2 * float(want.abs().max())
    if N % 8 == 0:
        y = torch.empty(M, N2, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(rows, w2g.to(DEV), y, error_flag=flag, force_splits=splits if N >= 64 * max(splits, 1) else 0,
                    row_scale=(sums, N, eps))
        close(y, want, torch.bfloat16)
        gated = torch.empty(M, N2 // 2, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(rows, w2g.to(DEV), gated, error_flag=flag, swiglu=True, row_scale=(sums, N, eps))
        gate = want.view(M, N2 // 32, 2, 16)
        close(gated, plain.swiglu(gate[:, :, 0], gate[:, :, 1]).reshape(M, N2 // 2), torch.bfloat16)
    assert flag.tolist() == [0, 0, 0, 0]


def test_norm_inputs_and_refusals_of_the_normed_product():
    x = torch.randn(7, 96) * 2
    rows = torch.empty(7, 96, dtype=torch.bfloat16, device=DEV); sums = torch.empty(7, 3, device=DEV)
    ops.norm_inputs(x.to(DEV), rows, sums)
    assert torch.equal(rows.cpu(), x.to(torch.bfloat16))
    assert float((sums.cpu().double() - (x.double() ** 2).view(7, 3, 32).sum(-1)).abs().max()) < 1e-4
    big = torch.zeros(600, 64, dtype=torch.bfloat16, device=DEV); w = torch.zeros(4096, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(cb.CitlaliError, match="prompt form"):
        ops.gemm_tc(big, w, torch.zeros(600, 4096, device=DEV), accumulate=True,
                    emit=(torch.zeros(600, 4096, dtype=torch.bfloat16, device=DEV), torch.zeros(600, 128, device=DEV)))
    with pytest.raises(cb.CitlaliError, match="multiple of 32"):
        ops.norm_inputs(torch.zeros(2, 40, device=DEV), torch.zeros(2, 40, dtype=torch.bfloat16, device=DEV), torch.zeros(2, 1, device=DEV))


def test_embedding_scale_and_logit_scale():
    table = torch.randn(50, 24)
    toks = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    plain_rows = torch.empty(3, 24, device=DEV); scaled = torch.empty(3, 24, device=DEV)
    ops.embed_rows(table.to(DEV), toks, plain_rows, flag)
    ops.embed_rows(table.to(DEV), toks, scaled, flag, scale=4.5)
    assert torch.equal(plain_rows.cpu(), table[[3, 49, 0]]) and torch.equal(scaled.cpu(), table[[3, 49, 0]] * 4.5)
    x = torch.randn(7, 1001, device=DEV)
    y = x.clone()
    ops.scale_(y, 0.125)
    assert torch.equal(y, x * 0.125)


def test_head_sizes_are_taken_or_refused():
    with pytest.raises(cb.CitlaliError, match="head size"):
        z = torch.zeros(1, 3 * 258, device=DEV)
        t = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.qk_norm_rope_cache(z, None, None, torch.zeros(129, device=DEV), 258, t, t, torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                               torch.zeros(1, 1, 64, 258, device=DEV), torch.zeros(1, 1, 64, 258, device=DEV), 64, 1, 1, 258, 1e-6)


def run_attention(q, k, v, past, n_new, nq, nkv, d, page, window, dtype, seed=0):
    """q: list of [n_new_b, nq, d]; k, v: list of [past_b + n_new_b, nkv, d] already final."""
    lengths = [p + n for p, n in zip(past, n_new)]
    kp, vp, table = make_paged(k, v, lengths, page, dtype, seed=seed)
    rows_slot, rows_pos = [], []
    for b, (p, n) in enumerate(zip(past, n_new)):
        rows_slot += [b] * n; rows_pos += list(range(p, p + n))
    qq = torch.cat([x.reshape(x.shape[0], nq * d) for x in q]).to(dtype)
    pad = torch.randn(qq.shape[0], 5).to(dtype)                      # queries lie inside a wider row
    qrow = torch.cat([qq, pad], dim=1).contiguous().to(DEV)
    out = torch.empty(qq.shape[0], nq * d, dtype=dtype, device=DEV)
    ops.attention_rows(qrow, qrow.shape[1], kp.to(DEV), vp.to(DEV), table.to(DEV),
                       torch.tensor(rows_slot, dtype=torch.int32, device=DEV), torch.tensor(rows_pos, dtype=torch.int32, device=DEV),
                       out, nq, nkv, d, page, window, max(lengths), 1.0 / math.sqrt(d))
    return out.view(-1, nq, d)


@pytest.mark.parametrize("nq,nkv,d,page", [(4, 2, 16, 64), (6, 3, 48, 8), (3, 1, 80, 64), (8, 2, 128, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_rows_prompts_and_single_tokens(nq, nkv, d, page, dtype):
    g = torch.Generator().manual_seed(nq * d)
    past, n_new = [0, 130, 5], [37, 1, 64]
    k = [torch.randn(p + n, nkv, d, generator=g).to(dtype).double() for p, n in zip(past, n_new)]
    v = [torch.randn(p + n, nkv, d, generator=g).to(dtype).double() for p, n in zip(past, n_new)]
    qfull = [(torch.randn(p + n, nq, d, generator=g) * 2).to(dtype).double() for p, n in zip(past, n_new)]
    got = run_attention([qf[p:] for qf, p in zip(qfull, past)], k, v, past, n_new, nq, nkv, d, page, 0, dtype)
    r = 0
    for b in range(3):
        want = plain.causal_attention(qfull[b], k[b], v[b], nq, nkv)[past[b]:]
        close(got[r:r + n_new[b]], want, dtype)
        r += n_new[b]


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_among_hundreds(dtype):
    """Random keys make attention nearly uniform and one missing key invisible.  Here key 3 of
    700 lines up with the query (score about 40 above the rest) and carries a value nothing else
    has: the output must be that value."""
    nq, nkv, d, page = 2, 1, 32, 64
    T = 700
    g = torch.Generator().manual_seed(1)
    k = torch.randn(T, nkv, d, generator=g) * 0.1
    v = torch.randn(T, nkv, d, generator=g)
    q = torch.zeros(1, nq, d); q[0, :, 0] = 16.0
    k[3, 0, 0] = 16.0                                    # q.k / sqrt(32) = 45
    v[3, 0] = torch.arange(d, dtype=torch.float32) - 7
    k, v, q = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
    got = run_attention([q], [k], [v], [T - 1], [1], nq, nkv, d, page, 0, dtype)
    want = plain.causal_attention(torch.cat([torch.zeros(T - 1, nq, d, dtype=torch.float64), q]), k, v, nq, nkv)[-1:]
    close(got, want, dtype)
    assert (got[0, 0].cpu().double() - v[3, 0]).abs().max() < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(dtype):
    """With a window of 5 the key at p-4 is the oldest one seen.  The key at p-5 would win every
    score if it were seen, so seeing it by mistake shows."""
    nq, nkv, d, page, W = 2, 2, 16, 8, 5
    T = 40
    g = torch.Generator().manual_seed(2)
    k = torch.randn(T, nkv, d, generator=g) * 0.1; v = torch.randn(T, nkv, d, generator=g)
    q = torch.randn(T, nq, d, generator=g) * 0.1
    p = T - 1
    q[p, :, 1] = 12.0
    k[p - W, :, 1] = 12.0; v[p - W] = 100.0              # just outside the window
    k[p - W + 1, :, 1] = 6.0                             # just inside
    k, v, q = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
    want = plain.causal_attention(q, k, v, nq, nkv, window=W)
    got = run_attention([q[10:]], [k], [v], [10], [T - 10], nq, nkv, d, page, W, dtype)
    close(got, want[10:], dtype)
    assert float(got[-1].abs().max()) < 10.0             # the value 100 stayed out
    wide = run_attention([q[10:]], [k], [v], [10], [T - 10], nq, nkv, d, page, 0, dtype)
    assert float(wide[-1].abs().max()) > 50.0            # without a window it is seen


def test_argmax_rows_rules():
    V = 1000
    logits = torch.randn(6, V)
    logits[0, 17] = 9.0; logits[0, 400] = 9.0                           # a tie: the lowest index
    logits[1, :] = float("nan")                                        # nothing finite: id 0
    logits[2, 5] = float("inf"); logits[2, 6] = float("nan"); logits[2, 999] = 50.0
    logits[3, 0] = 99.0
    logits[4, :] = -3.0                                                 # all equal
    tok = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.argmax_rows(logits.to(DEV), tok)
    assert tok.tolist() == [plain.greedy(r) for r in logits] and tok.tolist()[:5] == [17, 0, 999, 0, 0]
    big = torch.randn(5, 151936)                                        # wide rows are scanned by 64 blocks each
    big[1, :] = 3.0                                                      # all equal: index 0
    big[2, 100000] = 50.0; big[2, 5] = 50.0                              # a tie across segments: the lowest index
    big[3, :] = float("nan")                                             # nothing finite: id 0
    big[4, 151935] = 60.0; big[4, 77] = float("inf")
    tok = torch.zeros(5, dtype=torch.int32, device=DEV)
    ops.argmax_rows(big.to(DEV), tok)
    assert tok.tolist() == [int(big[0].argmax()), 0, 5, 0, 151935]


@pytest.mark.parametrize("V", [7, 1000, 4097, 151936])
def test_sample_rows_follows_the_cdf(V):
    g = torch.Generator().manual_seed(V)
    rows = 64
    logits = torch.randn(rows, V, generator=g) * 3
    logits[0, V // 2] = float("-inf"); logits[1, 0] = float("nan")
    temps = torch.full((rows,), 0.7); temps[5] = 0.0; temps[6] = 1.5
    us = torch.rand(rows, generator=g); us[2] = 0.0; us[3] = 0.99999994
    tok = torch.zeros(rows, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits.to(DEV), temps.to(DEV), us.to(DEV), tok)
    tok = tok.tolist()
    assert tok[5] == plain.greedy(logits[5])
    for r in range(rows):
        if r == 5:
            continue
        cdf = plain.temperature_cdf(logits[r], float(temps[r]))
        u = float(us[r])
        want = plain.temperature_sample(logits[r], float(temps[r]), u)
        if tok[r] != want:
            # 32-bit sums put the CDF's steps a few 1e-6 away from the exact ones: u must lie that close
            lo = float(cdf[tok[r] - 1]) if tok[r] > 0 else 0.0
            hi = float(cdf[tok[r]])
            assert lo - 2e-5 <= u <= hi + 2e-5 and hi > lo, f"row {r}: token {tok[r]}, exact {want}, u {u}"
        assert math.isfinite(float(logits[r, tok[r]]))


@pytest.fixture(params=["as planned", "one block"])
def one_block_or_pairs(request):
    """Runs a test of gemm_tc twice: with the dispatch as it stands, and with the pair kernel off, so that
    the one-block kernel is tested at many rows too."""
    if request.param == "one block":
        before = ops.gemm_tc_set_pair_rows(0)
        yield
        ops.gemm_tc_set_pair_rows(before)
    else:
        yield


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (5, 192, 64), (17, 1000, 96), (33, 130, 200), (64, 4096, 512),
                                   (100, 24, 4096), (128, 256, 512), (129, 256, 128), (300, 520, 200),
                                   (1000, 96, 72), (2048, 512, 1024), (1, 4096, 12288), (256, 4096, 4096), (200, 1000, 12288),
                                   (512, 4096, 2048)])
def test_gemm_tc(M, N, K, one_block_or_pairs):
    """The tensor-core product in both of its forms (weights on the wide side for few rows, rows
    on the wide side for many), with sizes that are no multiple of any tile, K that is split and
    K that is not, every output kind."""
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16); w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    scale = float(want.abs().max())
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    assert ops.gemm_tc_accepts(xd, wd, torch.empty(M, N, device=DEV))
    y32 = torch.full((M, N), 7.0, device=DEV)
    ops.gemm_tc(xd, wd, y32, error_flag=flag)
    err = float((y32.double().cpu() - want).abs().max())
    assert err <= 1e-5 * scale * max(1.0, math.sqrt(K / 64)), f"float32 out: |diff| {err:.3e} of {scale:.3e}"
    y16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(xd, wd, y16, error_flag=flag)
    close(y16, want, torch.bfloat16)
    base = torch.randn(M, N, generator=g)
    acc = base.to(DEV).clone()
    ops.gemm_tc(xd, wd, acc, accumulate=True, error_flag=flag)
    err = float((acc.double().cpu() - (base.double() + want)).abs().max())
    assert err <= 1e-5 * scale * max(1.0, math.sqrt(K / 64)) + 1e-6
    assert flag.tolist() == [0, 0, 0, 0]
    plan = ops.gemm_tc_plan(M, N, K, DEV)
    assert plan["swapped"] or M > 128          # few rows: the weights are the 128-row operand


def test_gemm_tc_rows_do_not_depend_on_the_batch():
    """Within one width of the narrow tile (up to 16, 32, 64, 128 rows) a row's result is the same
    bit for bit whatever else is in the batch; between widths the K split may differ, and with it
    the rounding."""
    g = torch.Generator().manual_seed(8)
    x = torch.randn(64, 4096, generator=g).to(torch.bfloat16).to(DEV); w = torch.randn(512, 4096, generator=g).to(torch.bfloat16).to(DEV)
    full = torch.empty(64, 512, device=DEV); ops.gemm_tc(x, w, full)
    sixteen = torch.empty(16, 512, device=DEV); ops.gemm_tc(x[20:36].contiguous(), w, sixteen)
    for rows in (1, 7, 16):
        part = torch.empty(rows, 512, device=DEV); ops.gemm_tc(x[20:20 + rows].contiguous(), w, part)
        assert torch.equal(part, sixteen[:rows]), f"{rows} rows alone differ from the same rows in a batch of 16"
    for rows in (33, 50):
        part = torch.empty(rows, 512, device=DEV); ops.gemm_tc(x[5:5 + rows].contiguous(), w, part)
        assert torch.equal(part, full[5:5 + rows]), f"{rows} rows alone differ from the same rows in a batch of 64"
    scale = float(full.abs().max())
    assert float((sixteen - full[20:36]).abs().max()) <= 2e-6 * scale


def test_gemm_tc_refusals():
    x = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV); w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    assert not ops.gemm_tc_accepts(x, w, torch.empty(4, 8, device=DEV))          # K = 20 is no multiple of 8
    with pytest.raises(cb.CitlaliError, match="multiple of 8"):
        ops.gemm_tc(x, w, torch.empty(4, 8, device=DEV))
    assert not ops.gemm_tc_accepts(x.float(), w, torch.empty(4, 8, device=DEV))


@pytest.mark.parametrize("nq,nkv,d,page,window", [(4, 2, 16, 64, 0), (6, 3, 48, 64, 0), (5, 5, 80, 8, 0), (32, 8, 128, 64, 0),
                                                  (12, 1, 64, 16, 0), (8, 2, 256, 64, 0), (6, 2, 112, 64, 300), (4, 2, 32, 8, 5)])
def test_attention_decode_split_over_the_context(nq, nkv, d, page, window):
    """Single new tokens at positions from 0 to 1100 (one to five chunks of four pages), several
    sequences at once, against the plain implementation; one sequence has a far key that wins."""
    g = torch.Generator().manual_seed(nq * d + page)
    dtype = torch.bfloat16
    lengths = [1, 2, 65, 256, 257, 700, 1101] if page == 64 else [1, 9, 33, 100]
    k = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lengths]
    v = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lengths]
    q = [(torch.randn(1, nq, d, generator=g) * 2).to(dtype).double() for n in lengths]
    if lengths[-1] > 600 and window == 0:
        q[-1][0, :, 3] = 20.0; k[-1][7, :, 3] = 20.0          # key 7 of 1101 takes nearly all the weight
    kp, vp, table = make_paged(k, v, lengths, page, dtype, seed=3)
    B = len(lengths)
    qrow = torch.cat([x.reshape(1, nq * d) for x in q]).to(dtype).to(DEV)
    out = torch.empty(B, nq * d, dtype=dtype, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    ops.attention_decode(qrow, nq * d, kp.to(DEV), vp.to(DEV), table.to(DEV), slots, pos, out, nq, nkv, d, page, window,
                         table.shape[1] * page, 1.0 / math.sqrt(d))
    for b, n in enumerate(lengths):
        qfull = torch.cat([torch.zeros(n - 1, nq, d, dtype=torch.float64), q[b]])
        want = plain.causal_attention(qfull, k[b], v[b], nq, nkv, window=window or None)[-1]
        got = out[b].view(nq, d)
        err = float((got.double().cpu() - want).abs().max())
        assert err <= 2 ** -8 * float(want.abs().max()), f"sequence of {n}: |diff| {err:.3e}"
    if lengths[-1] > 600 and window == 0:
        assert (out[-1].view(nq, d)[0].double().cpu() - v[-1][7, 0]).abs().max() < 0.1


@pytest.mark.parametrize("nq,nkv,d,window,scale_q8", [(8, 4, 128, 0, 256), (10, 2, 64, 0, 128), (4, 4, 32, 2000, 256), (40, 2, 16, 0, 64)])
def test_attention_decode_many_rows_of_unequal_lengths(nq, nkv, d, window, scale_q8):
    """Steps of so many rows that each (row, key/value head) gets one block: the pages of the rows that are much
    longer than the mean are dealt to several blocks on the device (their results merged by the block that finishes
    last), the others keep one.  Lengths from 1 to 3,000 in one step; a far key of the longest row takes all the
    weight of one head; the same step twice (the counters are back at zero) and with another run length."""
    import ctypes
    g = torch.Generator().manual_seed(nq + d)
    dtype, page = torch.bfloat16, 64
    rows = -(-152 // (nkv * -(-(nq // nkv) // 16)))
    rng = __import__("random").Random(d)
    lengths = [rng.choice((1, 3, 64, 65, 130, 200, 511, 513)) for _ in range(rows - 3)] + [3000, 1500, 2049]
    k = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lengths]
    v = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lengths]
    q = [(torch.randn(1, nq, d, generator=g) * 2).to(dtype).double() for n in lengths]
    far = rows - 3
    if window == 0:
        q[far][0, :, 3] = 20.0; k[far][7, :, 3] = 20.0
    kp, vp, table = make_paged(k, v, lengths, page, dtype, seed=3)
    qrow = torch.cat([x.reshape(1, nq * d) for x in q]).to(dtype).to(DEV)
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    kd, vd, td = kp.to(DEV), vp.to(DEV), table.to(DEV)
    lib = ops.lib()
    outs = []
    try:
        for on, q8 in ((1, scale_q8), (1, scale_q8), (0, 256)):
            lib.citlali_attention_decode_set_by_length(ctypes.c_int(on), ctypes.c_int(q8))
            out = torch.full((rows, nq * d), float("nan"), dtype=dtype, device=DEV)
            ops.attention_decode(qrow, nq * d, kd, vd, td, slots, pos, out, nq, nkv, d, page, window, table.shape[1] * page,
                                 1.0 / math.sqrt(d))
            outs.append(out)
    finally:
        lib.citlali_attention_decode_set_by_length(ctypes.c_int(1), ctypes.c_int(160))
    assert torch.equal(outs[0], outs[1])                       # the counters came back to zero
    assert not torch.equal(outs[0], outs[2])                   # and the long rows were in fact merged from several runs
    short = [b for b, n in enumerate(lengths) if n <= 1024]      # at most the sixteen pages of the shortest run
    assert torch.equal(outs[0][short], outs[2][short])         # rows that keep one block: the same arithmetic
    for b, n in enumerate(lengths):
        qfull = torch.cat([torch.zeros(n - 1, nq, d, dtype=torch.float64), q[b]])
        want = plain.causal_attention(qfull, k[b], v[b], nq, nkv, window=window or None)[-1]
        for out in (outs[0], outs[2]):
            err = float((out[b].view(nq, d).double().cpu() - want).abs().max())
            assert err <= 2 ** -8 * float(want.abs().max()), f"sequence of {n}: |diff| {err:.3e}"
    if window == 0:
        assert (outs[0][far].view(nq, d)[0].double().cpu() - v[far][7, 0]).abs().max() < 0.1


def test_attention_decode_one_long_sequence():
    """One sequence of 8,400 tokens in a cache laid out for more than 8,192: the blocks of a head group are a
    cluster of sixteen.  A far key takes nearly all the weight of one head; with a window only its keys count."""
    g = torch.Generator().manual_seed(11)
    dtype, page, nq, nkv, d, n = torch.bfloat16, 64, 8, 2, 128, 8400
    k = [torch.randn(n, nkv, d, generator=g).to(dtype).double()]
    v = [torch.randn(n, nkv, d, generator=g).to(dtype).double()]
    q = (torch.randn(1, nq, d, generator=g) * 2).to(dtype).double()
    q[0, 5, 9] = 20.0; k[0][4000, 1, 9] = 20.0
    kp, vp, table = make_paged(k, v, [n], page, dtype, seed=9)
    assert table.shape[1] > 128
    qrow = q.reshape(1, nq * d).to(dtype).to(DEV)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    for window in (0, 3000):
        out = torch.empty(1, nq * d, dtype=dtype, device=DEV)
        ops.attention_decode(qrow, nq * d, kp.to(DEV), vp.to(DEV), table.to(DEV), slots, pos, out, nq, nkv, d, page, window,
                             table.shape[1] * page, 1.0 / math.sqrt(d))
        lo = max(0, n - window) if window else 0
        want = plain.softmax_values(plain.attention_scores(q[0], k[0][lo:n], nq, nkv), v[0][lo:n], nq, nkv)
        got = out[0].view(nq, d)
        err = float((got.double().cpu() - want).abs().max())
        assert err <= 2 ** -8 * float(want.abs().max()), f"window {window}: |diff| {err:.3e}"
        if window == 0:
            assert (got[5].double().cpu() - v[0][4000, 1]).abs().max() < 0.1


@pytest.mark.parametrize("nq,nkv,d,window", [(4, 2, 16, 0), (6, 3, 48, 0), (3, 1, 80, 0), (8, 2, 128, 0), (2, 2, 256, 0),
                                             (4, 1, 64, 0), (5, 5, 112, 100), (4, 2, 32, 7), (2, 1, 96, 64)])
def test_attention_prefill_flash(nq, nkv, d, window):
    """Prompts and runs of tokens that continue a sequence, of lengths around the 64-token tiles,
    several sequences in one launch, against the plain implementation."""
    g = torch.Generator().manual_seed(nq * d + 1)
    dtype = torch.bfloat16
    past, n_new = [0, 130, 5, 0, 63, 200], [37, 1, 64, 129, 66, 300]
    k = [torch.randn(p + n, nkv, d, generator=g).to(dtype).double() for p, n in zip(past, n_new)]
    v = [torch.randn(p + n, nkv, d, generator=g).to(dtype).double() for p, n in zip(past, n_new)]
    qfull = [(torch.randn(p + n, nq, d, generator=g) * 1.5).to(dtype).double() for p, n in zip(past, n_new)]
    qfull[5][450, :, 2] = 18.0; k[5][11, :, 2] = 18.0           # row 450 finds key 11 among 451
    lengths = [p + n for p, n in zip(past, n_new)]
    kp, vp, table = make_paged(k, v, lengths, 64, dtype, seed=5)
    qq = torch.cat([qf[p:].reshape(-1, nq * d) for qf, p in zip(qfull, past)]).to(dtype)
    pad = torch.randn(qq.shape[0], 8).to(dtype)
    qrow = torch.cat([qq, pad], dim=1).contiguous().to(DEV)
    out = torch.empty(qq.shape[0], nq * d, dtype=dtype, device=DEV)
    starts = [0]
    for n in n_new:
        starts.append(starts[-1] + n)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    ops.attention_prefill(qrow, qrow.shape[1], kp.to(DEV), vp.to(DEV), table.to(DEV), i32(starts), i32(list(range(6))),
                          i32(past), out, 6, max(n_new), nq, nkv, d, 64, window, 1.0 / math.sqrt(d))
    for b in range(6):
        want = plain.causal_attention(qfull[b], k[b], v[b], nq, nkv, window=window or None)[past[b]:]
        got = out[starts[b]:starts[b + 1]].view(-1, nq, d)
        err = float((got.double().cpu() - want).abs().max())
        # P is rounded to bfloat16 before it multiplies V: 2^-9 relative per term on top of the output's rounding
        assert err <= 2 ** -7 * float(want.abs().max()), f"sequence {b}: |diff| {err:.3e} of {float(want.abs().max()):.3e}"
    if window == 0:
        assert (out[starts[5] + 250].view(nq, d)[0].double().cpu() - v[5][11, 0]).abs().max() < 0.1
    assert not ops.lib().citlali_attention_prefill_supports(40, 64) and not ops.lib().citlali_attention_prefill_supports(128, 16)


@pytest.mark.parametrize("nq,nkv,window", [(8, 2, 0), (3, 1, 0), (5, 5, 0), (4, 2, 100), (6, 2, 0), (3, 3, 150), (2, 1, 64)])
def test_attention_prefill_tcgen05(nq, nkv, window):
    """The tcgen05 prompt kernel alone (head size 128, pages of 64): groups with an even number of heads (two
    heads a block) and with an odd one (two row tiles a block), runs of 48 to 700 new tokens with and without
    cached tokens before them, several sequences in one launch, windows that end inside and across key tiles,
    a far key that takes nearly all the weight, against the plain implementation."""
    g = torch.Generator().manual_seed(nq * 7 + nkv + window)
    dtype, d = torch.bfloat16, 128
    assert ops.lib().citlali_attention_prefill_tc_supports(d, 64)
    past, n_new = [0, 130, 5, 0, 63, 200, 1], [48, 257, 64, 129, 300, 700, 128]
    k = [torch.randn(p + n, nkv, d, generator=g).to(dtype).double() for p, n in zip(past, n_new)]
    v = [torch.randn(p + n, nkv, d, generator=g).to(dtype).double() for p, n in zip(past, n_new)]
    qfull = [(torch.randn(p + n, nq, d, generator=g) * 1.5).to(dtype).double() for p, n in zip(past, n_new)]
    qfull[5][850, :, 2] = 18.0; k[5][11, :, 2] = 18.0           # row 850 finds key 11 among 851
    lengths = [p + n for p, n in zip(past, n_new)]
    kp, vp, table = make_paged(k, v, lengths, 64, dtype, seed=6)
    qq = torch.cat([qf[p:].reshape(-1, nq * d) for qf, p in zip(qfull, past)]).to(dtype)
    pad = torch.randn(qq.shape[0], 8).to(dtype)
    qrow = torch.cat([qq, pad], dim=1).contiguous().to(DEV)
    out = torch.full((qq.shape[0], nq * d), 7.0, dtype=dtype, device=DEV)
    starts = [0]
    for n in n_new:
        starts.append(starts[-1] + n)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    B = len(n_new)
    ops.attention_prefill_tc(qrow, qrow.shape[1], kp.to(DEV), vp.to(DEV), table.to(DEV), i32(starts), i32(list(range(B))),
                             i32(past), out, B, max(n_new), nq, nkv, d, 64, window, 1.0 / math.sqrt(d), error_flag=flag)
    torch.cuda.synchronize()
    assert flag.tolist() == [0, 0, 0, 0]
    for b in range(B):
        want = plain.causal_attention(qfull[b], k[b], v[b], nq, nkv, window=window or None)[past[b]:]
        got = out[starts[b]:starts[b + 1]].view(-1, nq, d)
        err = float((got.double().cpu() - want).abs().max())
        # P is rounded to bfloat16 before it multiplies V: 2^-9 relative per term on top of the output's rounding
        assert err <= 2 ** -7 * float(want.abs().max()), f"sequence {b}: |diff| {err:.3e} of {float(want.abs().max()):.3e}"
    if window == 0:
        assert (out[starts[5] + 650].view(nq, d)[0].double().cpu() - v[5][11, 0]).abs().max() < 0.1


@pytest.mark.parametrize("M,inter,K", [(1, 192, 64), (8, 12288, 512), (70, 160, 96), (128, 48, 64), (129, 64, 128),
                                       (400, 208, 120), (8, 2048, 4096), (33, 1024, 1024), (2048, 2048, 128),
                                       (1200, 1200, 64), (256, 1024, 2048), (300, 2048, 4096)])
def test_gemm_tc_gate_epilogue(M, inter, K, one_block_or_pairs):
    """silu(gate) * up straight from the product's epilogue, in both forms and with K split."""
    g = torch.Generator().manual_seed(M + inter)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wg = (torch.randn(inter, K, generator=g) * 0.2).to(torch.bfloat16); wu = (torch.randn(inter, K, generator=g) * 0.2).to(torch.bfloat16)
    want = plain.swiglu(x.double() @ wg.double().t(), x.double() @ wu.double().t())
    packed = torch.stack([wg.view(-1, 16, K), wu.view(-1, 16, K)], dim=1).reshape(2 * inter, K).contiguous()
    act = torch.empty(M, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x.to(DEV), packed.to(DEV), act, swiglu=True)
    close(act, want, torch.bfloat16)
    with pytest.raises(cb.CitlaliError, match="gate epilogue"):
        ops.gemm_tc(x.to(DEV), packed[:2 * inter - 16].contiguous().to(DEV), torch.empty(M, inter - 8, dtype=torch.bfloat16, device=DEV), swiglu=True)


def test_gemm_tc_on_pairs_of_sms_in_bands_of_row_tiles():
    """Many rows: the row tiles are taken in bands (their rows of x stay in L2 while the weight tiles pass by).  With
    bands of 4 row tiles (11 row tiles: bands of 4, 4 and 3) every tile is computed once and as without bands."""
    import ctypes
    M, N, K = 2700, 1100, 192
    if ops.gemm_tc_pair_plan(M, N, K)["pairs"] == 0:
        pytest.skip("this device runs no cluster of two blocks of that size")
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16); w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    xd, wd = x.to(DEV), w.to(DEV)
    lib = ops.lib()
    lib.citlali_gemm_tc_pair_set_band_bytes.restype = ctypes.c_long
    whole = torch.full((M, N), 7.0, device=DEV)
    ops.gemm_tc_pair(xd, wd, whole)                                     # default band: all 11 row tiles
    before = lib.citlali_gemm_tc_pair_set_band_bytes(ctypes.c_long(1))
    try:
        banded = torch.full((M, N), -7.0, device=DEV)
        ops.gemm_tc_pair(xd, wd, banded)
        acc = torch.ones(M, N, device=DEV)
        ops.gemm_tc_pair(xd, wd, acc, accumulate=True)                  # a tile done twice or never would show here
    finally:
        lib.citlali_gemm_tc_pair_set_band_bytes(ctypes.c_long(before))
    assert torch.equal(banded, whole)
    assert float((acc - 1.0 - whole).abs().max()) <= 1e-5 * float(want.abs().max())
    assert float((whole.double().cpu() - want).abs().max()) <= 1e-5 * float(want.abs().max()) * 2


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 264), (130, 144, 72), (1000, 1000, 512), (2048, 4096, 1024),
                                   (513, 96, 4096), (700, 1300, 2048), (2048, 4096, 4096)])
def test_gemm_tc_on_pairs_of_sms(M, N, K):
    """The product with cta_group::2 (two blocks of a cluster on one [256 x BN] tile), every output kind,
    sizes that are no multiple of any tile; and the same through gemm_tc's own dispatch."""
    if ops.gemm_tc_pair_plan(M, N, K)["pairs"] == 0:
        pytest.skip("this device runs no cluster of two blocks of that size")
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16); w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    scale = float(want.abs().max())
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    y32 = torch.full((M, N), 7.0, device=DEV)
    ops.gemm_tc_pair(xd, wd, y32, error_flag=flag)
    err = float((y32.double().cpu() - want).abs().max())
    assert err <= 1e-5 * scale * max(1.0, math.sqrt(K / 64)), f"float32 out: |diff| {err:.3e} of {scale:.3e}"
    again = torch.full((M, N), -3.0, device=DEV)
    ops.gemm_tc_pair(xd, wd, again, error_flag=flag)
    assert torch.equal(again, y32)
    y16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc_pair(xd, wd, y16, error_flag=flag)
    close(y16, want, torch.bfloat16)
    base = torch.randn(M, N, generator=g)
    acc = base.to(DEV).clone()
    ops.gemm_tc_pair(xd, wd, acc, accumulate=True, error_flag=flag)
    err = float((acc.double().cpu() - (base.double() + want)).abs().max())
    assert err <= 1e-5 * scale * max(1.0, math.sqrt(K / 64)) + 1e-6
    if N % 32 == 0:
        wg, wu = w[:N // 2] * 0.2, w[N // 2:] * 0.2
        wg, wu = wg.to(torch.bfloat16), wu.to(torch.bfloat16)
        packed = torch.stack([wg.view(-1, 16, K), wu.view(-1, 16, K)], dim=1).reshape(N, K).contiguous()
        act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc_pair(xd, packed.to(DEV), act, swiglu=True, error_flag=flag)
        close(act, plain.swiglu(x.double() @ wg.double().t(), x.double() @ wu.double().t()), torch.bfloat16)
    # the one-block kernel and the pair kernel add the K blocks in the same order; gemm_tc's own dispatch
    # gives the product to the one that its plan names
    one, two = torch.empty(M, N, device=DEV), torch.empty(M, N, device=DEV)
    before = ops.gemm_tc_set_pair_rows(0)
    try:
        assert not ops.gemm_tc_runs_on_pairs(M, N, K, DEV)
        ops.gemm_tc(xd, wd, one, error_flag=flag)
        ops.gemm_tc_set_pair_rows(128)
        ops.gemm_tc(xd, wd, two, error_flag=flag)
        assert torch.equal(two, y32 if ops.gemm_tc_runs_on_pairs(M, N, K, DEV) else one)
    finally:
        ops.gemm_tc_set_pair_rows(before)
    assert float((one - y32).abs().max()) <= 2e-6 * scale
    assert flag.tolist() == [0, 0, 0, 0]


def test_gemm_tc_pairs_where_their_waves_cost_less():
    """Prompts of Qwen3-8B's widths: the shapes that were measured faster on pairs go there, the others do not."""
    if ops.gemm_tc_pair_plan(2048, 4096, 4096)["pairs"] != 74 or ops.sm_count(DEV) != 148:
        pytest.skip("the expectations are those of 148 SMs")
    for (M, N, K, gate, want) in [(2048, 6144, 4096, False, True), (2048, 4096, 12288, False, True), (2048, 24576, 4096, True, True),
                                  (1536, 4096, 12288, False, False), (1024, 6144, 4096, False, False), (512, 24576, 4096, True, True),
                                  (384, 24576, 4096, True, False), (768, 4096, 4096, False, False), (8192, 4096, 4096, False, True)]:
        assert ops.gemm_tc_runs_on_pairs(M, N, K, DEV, swiglu=gate) == want, (M, N, K)


def test_gemm_tc_split_k_sums_in_one_order():
    """K split over a cluster of blocks: the same bits every time, and for every forced split the sum is right."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(8, 4096, generator=g).to(torch.bfloat16).to(DEV); w = torch.randn(4096, 4096, generator=g).to(torch.bfloat16).to(DEV)
    assert ops.gemm_tc_plan(8, 4096, 4096, DEV)["splits"] > 1
    y = torch.empty(8, 4096, device=DEV)
    outs = []
    for _ in range(3):
        ops.gemm_tc(x, w, y)
        outs.append(y.clone())
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    want = x.double() @ w.double().t()
    for splits in (1, 2, 3, 5, 8):
        ops.gemm_tc(x, w, y, force_splits=splits)
        assert ops.gemm_tc_plan(8, 4096, 4096, DEV, splits)["splits"] == splits
        assert float((y.double() - want).abs().max()) <= 1e-4 * float(want.abs().max())
