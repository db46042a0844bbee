"""Python face of the kernel library: one function per kernel, taking torch tensors.

Each function checks dtypes, shapes and contiguity, then calls the C entry point on the
current CUDA stream.  There is no CPU implementation and no library implementation behind
these functions: if the kernel library cannot be built or loaded, or a tensor is not on a
CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .errors import CitlaliError, require

_F32, _BF16 = 0, 1
_lib = None


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise CitlaliError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def lib():
    global _lib
    if _lib is None:
        from .csrc.build import load
        l = load()
        l.citlali_last_error.restype = ctypes.c_char_p
        _lib = l
    return _lib


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle.  Asked for at every launch, so by the quick route where torch has one
    (a step launches a few hundred kernels and the host must not be what a short prompt waits for)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0
_KERNELS_PER_CALL = {"attention_decode_merged": 2, "argmax_rows_wide": 2}


def launch_count() -> int:
    """Kernels of this library launched so far through this module (a split-K product counts
    its reduction, split-context attention its merge)."""
    return _launches


def _check(code: int, what: str):
    global _launches
    if code == 0:
        _launches += _KERNELS_PER_CALL.get(what, 1)
        return
    if code < 0:
        raise CitlaliError(f"{what} refused: {lib().citlali_last_error().decode()}")
    raise CitlaliError(f"{what}: CUDA error {code} at launch")


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            require(t.is_cuda, "kernels run on a CUDA device only; a tensor on the CPU was given")
            require(False, "kernels take contiguous tensors")


_i = ctypes.c_int
_f = ctypes.c_float


def embed_rows(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, error_flag: torch.Tensor,
               scale: float = 1.0):
    _need_cuda(table, tokens, out, error_flag)
    require(tokens.dtype == torch.int32 and out.dtype == torch.float32, "embed_rows: tokens int32, out float32")
    rows, hidden = out.shape
    require(table.shape[1] == hidden and tokens.numel() == rows, "embed_rows: shapes do not fit")
    _check(lib().citlali_embed_rows(_ptr(table), _i(_dtype_code(table)), _ptr(tokens), _ptr(out), _i(rows),
                                    _i(hidden), _i(table.shape[0]), _f(scale), _ptr(error_flag), _stream()), "embed_rows")


def scale_(x: torch.Tensor, scale: float):
    """x *= scale in place (float32)."""
    _need_cuda(x)
    require(x.dtype == torch.float32, "scale_: float32 only")
    _check(lib().citlali_scale(_ptr(x), ctypes.c_size_t(x.numel()), _f(scale), _stream()), "scale")


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
             row_index: Optional[torch.Tensor] = None):
    _need_cuda(x, gain, out, row_index)
    require(x.dtype == torch.float32, "rms_norm: the input rows are float32")
    rows, hidden = out.shape
    require(x.shape[1] == hidden and gain.numel() == hidden, "rms_norm: shapes do not fit")
    if row_index is not None:
        require(row_index.dtype == torch.int32 and row_index.numel() == rows, "rms_norm: bad row index")
    else:
        require(x.shape[0] == rows, "rms_norm: shapes do not fit")
    _check(lib().citlali_rms_norm(_ptr(x), _ptr(gain), _i(_dtype_code(gain)), _ptr(row_index), _ptr(out),
                                  _i(_dtype_code(out)), _i(rows), _i(hidden), _f(eps), _stream()), "rms_norm")


def swiglu(gate_up: torch.Tensor, act: torch.Tensor, run: int):
    _need_cuda(gate_up, act)
    rows, inter = act.shape
    require(gate_up.shape == (rows, 2 * inter) and gate_up.dtype == act.dtype, "swiglu: shapes or dtypes do not fit")
    _check(lib().citlali_swiglu(_ptr(gate_up), _ptr(act), _i(_dtype_code(act)), _i(rows), _i(inter), _i(run),
                                _stream()), "swiglu")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, accumulate: bool = False):
    _need_cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    require(w.shape[1] == K and y.shape == (M, N), "gemm_simt: shapes do not fit")
    _check(lib().citlali_gemm_simt(_ptr(x), _i(_dtype_code(x)), _ptr(w), _i(_dtype_code(w)), _ptr(y),
                                   _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(1 if accumulate else 0), _stream()),
           "gemm_simt")


def qk_norm_rope_cache(qkv, q_gain, k_gain, inv_freq, rotary_dim, row_slot, row_pos, page_table,
                       k_pool, v_pool, page_size, nq, nkv, head_dim, eps, write_cache=True):
    """Head RMSNorm of q and k (``q_gain``/``k_gain`` None: none), rotation of the first ``rotary_dim`` elements
    of each q and k head in pairs (i, i + rotary_dim/2), and the cache write, in one pass over the projection's
    rows.  ``write_cache``: True keys and values go to the cache; False nothing does; ``"keys_in_place"`` the
    normed, rotated keys go back into the row and the values stay, for a position encoding that works on the
    row before a second call stores it."""
    _need_cuda(qkv, q_gain, k_gain, inv_freq, row_slot, row_pos, page_table, k_pool, v_pool)
    rows = qkv.shape[0]
    require(qkv.shape[1] == (nq + 2 * nkv) * head_dim, "qk_norm_rope_cache: the projection's width does not fit")
    require(inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
            "qk_norm_rope_cache: bad frequency table")
    require(row_slot.dtype == torch.int32 and row_pos.dtype == torch.int32 and page_table.dtype == torch.int32,
            "qk_norm_rope_cache: index tensors are int32")
    gain_code = _dtype_code(q_gain) if q_gain is not None else _F32
    if q_gain is not None and k_gain is not None:
        require(q_gain.dtype == k_gain.dtype, "qk_norm_rope_cache: q and k gains differ in dtype")
    cache_code = _dtype_code(k_pool) if k_pool is not None else _dtype_code(qkv)
    _check(lib().citlali_qk_norm_rope_cache(
        _ptr(qkv), _i(_dtype_code(qkv)), _ptr(q_gain), _ptr(k_gain), _i(gain_code), _ptr(inv_freq), _i(rotary_dim),
        _ptr(row_slot), _ptr(row_pos), _ptr(page_table), _i(page_table.shape[1]), _ptr(k_pool), _ptr(v_pool),
        _i(cache_code), _i(page_size), _i(rows), _i(nq), _i(nkv), _i(head_dim), _f(eps),
        _i(2 if write_cache == "keys_in_place" else (1 if write_cache else 0)), _stream()), "qk_norm_rope_cache")


def attention_rows(q, q_stride, k_pool, v_pool, page_table, row_slot, row_pos, out, nq, nkv, head_dim,
                   page_size, window, max_keys, scale):
    _need_cuda(k_pool, v_pool, page_table, row_slot, row_pos, out)
    require(q.is_cuda, "kernels run on a CUDA device only")
    rows = out.shape[0]
    _check(lib().citlali_attention_rows(
        _ptr(q), _i(q_stride), _i(_dtype_code(q)), _ptr(k_pool), _ptr(v_pool), _i(_dtype_code(k_pool)),
        _ptr(page_table), _i(page_table.shape[1]), _ptr(row_slot), _ptr(row_pos), _ptr(out), _i(out.shape[1]),
        _i(rows), _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _i(max_keys), _f(scale),
        _stream()), "attention_rows")


def argmax_rows(logits: torch.Tensor, tokens: torch.Tensor):
    _need_cuda(logits, tokens)
    require(logits.dtype == torch.float32 and tokens.dtype == torch.int32, "argmax_rows: float32 in, int32 out")
    rows, vocab = logits.shape
    if vocab >= 8192:
        scratch = _scratch(logits.device, "argmax segments", rows * 128 * 4)
        _check(lib().citlali_argmax_rows_wide(_ptr(logits), _ptr(tokens), _ptr(scratch), _i(rows), _i(vocab), _stream()),
               "argmax_rows_wide")
        return
    _check(lib().citlali_argmax_rows(_ptr(logits), _ptr(tokens), _i(rows), _i(vocab), _stream()), "argmax_rows")


def sample_rows(logits, temperature, uniform, tokens):
    _need_cuda(logits, temperature, uniform, tokens)
    require(logits.dtype == torch.float32 and tokens.dtype == torch.int32 and temperature.dtype == torch.float32
            and uniform.dtype == torch.float32, "sample_rows: float32 in, int32 out")
    rows, vocab = logits.shape
    require(temperature.numel() >= rows and uniform.numel() >= rows and tokens.numel() >= rows,
            "sample_rows: per-row tensors are too short")
    _check(lib().citlali_sample_rows(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(tokens), _i(rows),
                                     _i(vocab), _stream()), "sample_rows")


# ---- choices between kernels ---------------------------------------------------------------

def attention_steps_from_device(dtype, head_dim: int) -> bool:
    """Whether a step of single tokens in this dtype and head size runs the split-context kernel, whose
    launch depends on no host-side length (the condition :func:`attention` tests first)."""
    return dtype == torch.bfloat16 and head_dim % 8 == 0 and head_dim <= 256


def attention(q, q_stride, cache_view, batch, out, nq, nkv, head_dim, window, scale):
    """Attention of every row of the step over its slot's cache.  ``q`` holds the rotated
    queries with ``q_stride`` elements between rows.  bfloat16 steps in which every sequence
    brings one token run the split-context kernel, whose launch does not depend on the
    sequences' lengths; everything else runs the generic kernel."""
    if batch.is_decode and attention_steps_from_device(q.dtype, head_dim):
        attention_decode(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table, batch.row_slot,
                         batch.row_pos, out, nq, nkv, head_dim, cache_view.page_size, window,
                         cache_view.page_table.shape[1] * cache_view.page_size, scale)
        return
    require(not torch.cuda.is_current_stream_capturing(),
            "attention: this dtype and head size run a kernel whose launch is sized from the host's lists of lengths, "
            "which a captured step would freeze; such a model steps without CUDA graphs")
    if (q.dtype == torch.bfloat16 and q_stride % 8 == 0 and out.shape[1] % 8 == 0 and batch.max_new >= 48
            and lib().citlali_attention_prefill_tc_supports(_i(head_dim), _i(cache_view.page_size))):
        attention_prefill_tc(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table, batch.seq_start,
                             batch.seq_slot, batch.seq_past, out, batch.sequences, batch.max_new, nq, nkv, head_dim,
                             cache_view.page_size, window, scale)
        return
    if (q.dtype == torch.bfloat16 and q_stride % 8 == 0
            and lib().citlali_attention_prefill_supports(_i(head_dim), _i(cache_view.page_size))):
        attention_prefill(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table, batch.seq_start,
                          batch.seq_slot, batch.seq_past, out, batch.sequences, batch.max_new, nq, nkv, head_dim,
                          cache_view.page_size, window, scale)
        return
    attention_rows(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table,
                   batch.row_slot, batch.row_pos, out, nq, nkv, head_dim, cache_view.page_size,
                   window, batch.max_keys, scale)


def attention_prefill(q, q_stride, k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out, sequences, max_new,
                      nq, nkv, head_dim, page_size, window, scale):
    _need_cuda(k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out)
    require(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
            "attention_prefill: bfloat16 only")
    _check(lib().citlali_attention_prefill(
        _ptr(q), _i(q_stride), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(seq_start), _ptr(seq_slot), _ptr(seq_past), _ptr(out), _i(out.shape[1]), _i(sequences), _i(max_new),
        _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _f(scale), _stream()), "attention_prefill")


def attention_prefill_tc(q, q_stride, k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out, sequences, max_new,
                         nq, nkv, head_dim, page_size, window, scale, error_flag=None):
    """Prompt attention on tcgen05 (head size 128, pages of 64)."""
    _need_cuda(k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out, error_flag)
    require(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
            "attention_prefill_tc: bfloat16 only")
    _check(lib().citlali_attention_prefill_tc(
        _ptr(q), _i(q_stride), _i(q.shape[0]), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[0]), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(seq_start), _ptr(seq_slot), _ptr(seq_past), _ptr(out), _i(out.shape[1]),
        _i(sequences), _i(max_new), _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _f(scale),
        _ptr(error_flag), _stream()), "attention_prefill_tc")


def attention_decode(q, q_stride, k_pool, v_pool, page_table, row_slot, row_pos, out, nq, nkv, head_dim,
                     page_size, window, max_positions, scale):
    _need_cuda(k_pool, v_pool, page_table, row_slot, row_pos, out)
    require(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
            "attention_decode: bfloat16 only")
    rows = out.shape[0]
    l = lib()
    l.citlali_attention_decode_scratch_floats.restype = ctypes.c_size_t
    need = l.citlali_attention_decode_scratch_floats(_i(rows), _i(nq), _i(head_dim), _i(page_size), _i(max_positions))
    ws = _scratch(q.device, "attention_decode", need * 4)
    counters = _scratch(q.device, "attention_decode counters", rows * nq * 4, zeroed=True)
    _check(l.citlali_attention_decode(
        _ptr(q), _i(q_stride), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(row_slot), _ptr(row_pos), _ptr(out), _i(out.shape[1]), _ptr(ws), ctypes.c_size_t(ws.numel() // 4),
        _ptr(counters), ctypes.c_size_t(counters.numel() // 4),
        _i(rows), _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _i(max_positions), _f(scale),
        _stream()),
        # one kernel whose blocks merge through distributed shared memory, or a partial and a merge kernel
        "attention_decode" if (page_size == 64 and q_stride % 8 == 0 and q.data_ptr() % 16 == 0
                               and head_dim in (16, 32, 48, 64, 80, 96, 112, 128, 256)) else "attention_decode_merged")


_sm_count = {}
_workspace = {}
_retired = []


def sm_count(device) -> int:
    idx = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def gemm_tc_plan(M: int, N: int, K: int, device, force_splits: int = 0) -> dict:
    """How the tensor-core product of this shape runs."""
    swapped, bn, splits = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib().citlali_gemm_tc_plan(_i(M), _i(N), _i(K), _i(sm_count(device)), _i(force_splits), ctypes.byref(swapped),
                               ctypes.byref(bn), ctypes.byref(splits))
    return {"swapped": bool(swapped.value), "bn": bn.value, "splits": splits.value}


def wait_selftest(error_flag: torch.Tensor, limit_ms: float = 2.0):
    """Run the tensor-core kernels' bounded wait on a barrier nothing arrives on; it gives up after
    ``limit_ms``.  Returns (the wait's return value, the block's abort word); ``error_flag[1..2]`` hold
    code 900 and the block."""
    _need_cuda(error_flag)
    result = torch.full((2,), -1, dtype=torch.int32, device=error_flag.device)
    _check(lib().citlali_wait_selftest(_ptr(error_flag), _ptr(result), ctypes.c_longlong(int(limit_ms * 1e6)), _stream()),
           "wait_selftest")
    ok, abort = result.tolist()
    return ok, abort


def gemm_tc_pair_plan(M: int, N: int, K: int) -> dict:
    """The pair kernel's tile width for this shape and how many clusters of two the device runs at once."""
    bn, pairs = ctypes.c_int(), ctypes.c_int()
    lib().citlali_gemm_tc_pair_plan(_i(M), _i(N), _i(K), ctypes.byref(bn), ctypes.byref(pairs))
    return {"bn": bn.value, "pairs": pairs.value}


def gemm_tc_set_pair_rows(rows: int) -> int:
    """From ``rows`` rows of ``x`` on, ``gemm_tc`` runs on pairs of SMs where their waves cost less
    (0: never). Returns the number that stood before."""
    return int(lib().citlali_gemm_tc_set_pair_rows(_i(rows)))


def gemm_tc_runs_on_pairs(M: int, N: int, K: int, device, swiglu: bool = False) -> bool:
    """Whether ``gemm_tc`` gives a product of this shape to the pair kernel."""
    return bool(lib().citlali_gemm_tc_runs_on_pairs(_i(M), _i(N), _i(K), _i(sm_count(device)), _i(1 if swiglu else 0)))


def gemm_tc_pair(x, w, y, accumulate=False, error_flag=None, swiglu=False):
    """``gemm_tc`` on pairs of SMs (tcgen05.mma with cta_group::2), whatever the number of rows."""
    _need_cuda(x, w, y, error_flag)
    M, K = x.shape
    N = w.shape[0]
    require(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and w.shape[1] == K
            and x.is_contiguous() and w.is_contiguous(),
            "gemm_tc_pair: operands must be contiguous bfloat16 with an inner size that is a multiple of 8")
    require(y.shape == (M, N // 2 if swiglu else N), "gemm_tc_pair: the output's shape does not fit")
    mode = (1 if accumulate else 0) | (2 if swiglu else 0)
    _check(lib().citlali_gemm_tc_pair(_ptr(x), _ptr(w), _ptr(y), _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(mode),
                                      _ptr(error_flag), _stream()), "gemm_tc_pair")


_zeroed_purposes = set()


def zero_counters() -> None:
    """Put the scratch buffers that hold counters back to zero, in place (captured graphs keep their addresses).  For
    after a kernel reported a fault: a step that gave up half-way may have left counters standing."""
    for (index, purpose), ws in _workspace.items():
        if purpose in _zeroed_purposes:
            ws.zero_()
    for purpose, ws in _retired:
        if purpose in _zeroed_purposes:
            ws.zero_()


def _scratch(device, purpose: str, nbytes: int, zeroed: bool = False) -> torch.Tensor:
    """One scratch buffer per device and purpose (split-context attention partials, argmax segments);
    it only grows.  Kernels on one stream use it one after another.  ``zeroed``: filled with zeros when it
    is made (for counters that every kernel leaves at zero)."""
    key = (torch.device(device).index or 0, purpose)
    ws = _workspace.get(key)
    if ws is None or ws.numel() < nbytes:
        require(not torch.cuda.is_current_stream_capturing(),
                f"the {purpose} scratch buffer would have to grow during graph capture; run the step once before capturing")
        if ws is not None:
            _retired.append((purpose, ws))          # a captured graph may still hold its address: it is kept, not freed
        ws = (torch.zeros if zeroed else torch.empty)(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspace[key] = ws
        if zeroed:
            _zeroed_purposes.add(purpose)
    return ws


def gemm_tc_accepts(x, w, y) -> bool:
    """The tensor-core product's shape rules: bfloat16 operands, an inner size that is a
    multiple of 8 (TMA needs rows of 16-byte multiples), 16-byte aligned starts."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.float32, torch.bfloat16)
            and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.is_contiguous() and w.is_contiguous() and y.is_contiguous())


def norm_inputs(x: torch.Tensor, rows_out: torch.Tensor, sumsq: torch.Tensor):
    """``rows_out = bfloat16(x)`` and ``sumsq[r, g]`` = the sum of squares of x[r]'s g-th group of 32 features."""
    _need_cuda(x, rows_out, sumsq)
    rows, hidden = x.shape
    require(x.dtype == torch.float32 and rows_out.dtype == torch.bfloat16 and sumsq.dtype == torch.float32
            and rows_out.shape == x.shape and sumsq.shape == (rows, hidden // 32), "norm_inputs: shapes or dtypes do not fit")
    _check(lib().citlali_norm_inputs(_ptr(x), _ptr(rows_out), _ptr(sumsq), _i(rows), _i(hidden), _stream()), "norm_inputs")


def gemm_tc_is_small_form(M: int, N: int, K: int, device) -> bool:
    """Whether the product of this shape runs the form for few rows of x, whose epilogue can do a norm's work."""
    return gemm_tc_plan(M, N, K, device)["swapped"]


def gemm_tc(x, w, y, accumulate=False, error_flag=None, swiglu=False, force_splits=0, emit=None, row_scale=None):
    """``y = x . w^T`` on the tensor cores.  ``accumulate``: ``y`` (float32) ``+=``.  ``swiglu``: ``w``'s
    rows alternate gate/up in runs of 16 and ``y`` is bfloat16 ``[M, N/2] = silu(gate) * up``.
    Few rows of x only: ``emit = (rows_bf16 [M, N], sumsq [M, N/32])`` (with ``accumulate``) also writes the updated
    rows as bfloat16 and the sums of their squares over groups of 32 features; ``row_scale = (sumsq [M, groups], dim,
    eps)`` multiplies result row m by ``rsqrt(sum(sumsq[m]) / dim + eps)``."""
    _need_cuda(x, w, y, error_flag)
    M, K = x.shape
    N = w.shape[0]
    require(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and w.shape[1] == K
            and x.is_contiguous() and w.is_contiguous(),
            "gemm_tc: operands must be contiguous bfloat16 with an inner size that is a multiple of 8")
    require(y.shape == (M, N // 2 if swiglu else N), "gemm_tc: the output's shape does not fit")
    mode = (1 if accumulate else 0) | (2 if swiglu else 0)
    if emit is None and row_scale is None:
        _check(lib().citlali_gemm_tc(_ptr(x), _ptr(w), _ptr(y), _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(mode),
                                     _i(force_splits), _ptr(error_flag), _i(sm_count(x.device)), _stream()), "gemm_tc")
        return
    emit_rows = emit_sumsq = scale_sumsq = None
    groups = dim = 0
    eps = 0.0
    if emit is not None:
        emit_rows, emit_sumsq = emit
        _need_cuda(emit_rows, emit_sumsq)
        require(emit_rows.dtype == torch.bfloat16 and emit_rows.shape == (M, N) and emit_sumsq.dtype == torch.float32
                and emit_sumsq.shape == (M, N // 32), "gemm_tc: the emitted rows or their sums have the wrong shape or dtype")
    if row_scale is not None:
        scale_sumsq, dim, eps = row_scale
        _need_cuda(scale_sumsq)
        require(scale_sumsq.dtype == torch.float32 and scale_sumsq.dim() == 2 and scale_sumsq.shape[0] == M,
                "gemm_tc: the sums of squares to scale by have the wrong shape or dtype")
        groups = scale_sumsq.shape[1]
    _check(lib().citlali_gemm_tc_normed(_ptr(x), _ptr(w), _ptr(y), _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(mode),
                                        _i(force_splits), _ptr(error_flag), _i(sm_count(x.device)), _ptr(emit_rows),
                                        _ptr(emit_sumsq), _ptr(scale_sumsq), _i(groups), _i(int(dim)), _f(float(eps)), _stream()),
           "gemm_tc")
