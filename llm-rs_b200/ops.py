"""Python face of the CUDA kernel library: each function checks its tensors and launches
one kernel (or one kernel and its combine step) on the current CUDA stream.

There is no CPU path: a tensor that is not on a CUDA device is refused, and a missing
library is an error (``csrc.build.KernelBuildError``), never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

launch_count = 0  # kernels launched through this module since import (read by the benchmark)


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _lib():
    return _build.library()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream's handle. (``torch.cuda.current_stream()`` builds a Python object every time: some
    7 us a call, 1.2 ms of the 6 ms the host needs to issue the 290 launches of a prefill step; the raw handle is
    asked for directly where this torch offers it.)"""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(rc: int, what: str, launches: int = 1) -> None:
    global launch_count
    if rc != 0:
        msg = _lib().llmrs_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what} failed (code {rc}): {msg}")
    launch_count += launches


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be on a CUDA device (this engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _row_stride(t: torch.Tensor, name: str) -> int:
    """Stride between rows of a 2-D view whose rows are dense."""
    if t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with dense rows, got sizes {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` widened to float32 (the residual stream's type)."""
    _need(table, "table")
    _need(ids, "ids", torch.int32)
    vocab, hidden = table.shape
    n = ids.numel()
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32)
    _check(_lib().llmrs_embedding(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), n, hidden, vocab,
                                  _stream()), "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += delta`` (when given), then ``out = h / sqrt(mean(h^2) + eps) * weight``.

    ``h`` is the float32 residual stream and is updated in place. With ``rows`` (int32
    indices) only those rows are normed, into ``out[i]``, and ``h`` is left as it is.
    """
    _need(h, "h", torch.float32)
    _need(weight, "weight", torch.float32)
    hidden = h.size(-1)
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements, rows have {hidden}")
    if delta is not None:
        _need(delta, "delta", act_dtype)
        if delta.shape != h.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
    n_rows = h.size(0) if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=act_dtype, device=h.device)
    _need(out, "out", act_dtype)
    _check(_lib().llmrs_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_rows, hidden,
                                    ctypes.c_float(eps), dtype_code(act_dtype), _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """``h += delta`` in float32, in place."""
    _need(h, "h", torch.float32)
    _need(delta, "delta")
    if delta.shape != h.shape:
        raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
    _check(_lib().llmrs_residual_add(_ptr(h), _ptr(delta), ctypes.c_longlong(h.numel()), dtype_code(delta.dtype),
                                     _stream()), "residual_add")
    return h


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, block: int = 0) -> torch.Tensor:
    """``out[t, c] = silu(gate(t, c)) * up(t, c)`` for ``gate_up`` of width 2I that holds gate and
    up in alternating runs of ``block`` columns (0: the plain layout, I gate columns then I up columns)."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    inter = two_i // 2
    block = block or inter
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype)
    _check(_lib().llmrs_silu_mul(_ptr(gate_up), _ptr(out), n, inter, block, dtype_code(gate_up.dtype), _stream()),
           "silu_mul")
    return out


GEMM_F32_SKINNY_MAX = 264       # products with at most this many output features take the kernel laid out for them
GEMM_F32_SKINNY_TOKENS = 8      # rows of x a block of that kernel holds in shared memory


def gemm_f32(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """True float32 ``x @ w.T (+ bias)`` with ``w`` of shape [N, K] (FFMA, no TF32). ``x`` may be bfloat16 rows: they
    are widened as they are read; weights, sums and the result stay float32."""
    _need(x, "x", contiguous=False)
    _need(w, "w", torch.float32)
    M, K = x.shape
    N = w.size(0)
    if w.size(1) != K:
        raise KernelError(f"x has {K} columns, w has {w.size(1)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, contiguous=False)
    code = dtype_code(x.dtype)     # refuses any other type
    smem = GEMM_F32_SKINNY_TOKENS * K * x.element_size()
    if N <= GEMM_F32_SKINNY_MAX and K % 4 == 0 and smem <= 200 * 1024 and w.data_ptr() % 16 == 0:
        # Few output features (a router, gates): the kernel that gives each feature a warp.
        _check(_lib().llmrs_gemm_f32_skinny(_ptr(x), code, ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(bias),
                                            _ptr(out), ctypes.c_longlong(_row_stride(out, "out")), M, N, K, _stream()),
               "gemm_f32")
        return out
    fn = _lib().llmrs_gemm_f32 if x.dtype == torch.float32 else _lib().llmrs_gemm_f32_bf16_rows
    _check(fn(_ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(bias), _ptr(out),
              ctypes.c_longlong(_row_stride(out, "out")), M, N, K, _stream()), "gemm_f32")
    return out


F32_ROWS_LIBRARY_MIN = 33     # steps of at least this many rows send ``product_f32`` of bfloat16 operands to the library


def product_f32(x: torch.Tensor, w_stored: torch.Tensor, w_f32: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """A product whose result must not be rounded below float32 (a router's logits, the gates of a recurrence):
    ``x @ w.T + bias`` as float32. ``w_stored`` is the weight as the folder stores it, ``w_f32`` the same widened.
    When the rows AND the stored weight are bfloat16, every product of two operands is exact in float32, so a
    tensor-core product with float32 accumulation and float32 output computes the same sum as the FFMA kernel up to
    the order of its terms: prompt portions take it (the library's, as the other products of large steps); steps of
    few rows and everything else take ``gemm_f32``."""
    if (x.dtype == torch.bfloat16 and w_stored.dtype == torch.bfloat16 and x.size(0) >= F32_ROWS_LIBRARY_MIN
            and x.is_contiguous()):
        return library_gemm(x, w_stored, bias, torch.float32)
    return gemm_f32(x, w_f32, bias)


def library_gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` in bfloat16 through the library (cuBLAS via ``torch``): the products of steps with
    many tokens that this package's own kernel does not take, as the reference's projections are calls into
    its tensor library (llm-core/src/backends/candle.rs:1276-1340). The only library kernel on the product path
    (not counted in ``launch_count``, which counts this package's own kernels)."""
    if out_dtype == torch.float32:
        y = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.to(torch.float32)
        return y
    return torch.nn.functional.linear(x, w, bias)


def qk_norm_rope_kvwrite(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                         q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                         cos_sin: Optional[torch.Tensor], positions: torch.Tensor, token_req: torch.Tensor,
                         block_table: torch.Tensor, cache: Optional[torch.Tensor], n_q_heads: int, n_kv_heads: int,
                         head_dim: int, rotary_dim: int, page_size: int, eps: float) -> None:
    """Per-head norm and rotation of ``q`` (in place) and ``k``; ``k`` and ``v`` go to their pages.

    ``q``, ``k``, ``v`` are 2-D views with dense rows (slices of one projection output
    are fine). ``k`` = ``v`` = None: this layer reads another layer's cache and writes none.
    ``cos_sin`` is [positions, rotary_dim/2, 2] float32, or None for no rotation.
    ``cache`` is one layer's [n_pages, n_kv_heads, 2, page_size, head_dim].
    """
    _need(q, "q", contiguous=False)
    dt = q.dtype
    n = q.size(0)
    for name, t in (("k", k), ("v", v)):
        if t is not None:
            _need(t, name, dt, contiguous=False)
    if (k is None) != (v is None):
        raise KernelError("k and v must both be given or both be None")
    if k is not None:
        _need(cache, "cache", dt)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("cos_sin", cos_sin)):
        if t is not None:
            _need(t, name, torch.float32)
    if cos_sin is not None and cos_sin.size(1) * 2 != rotary_dim:
        raise KernelError(f"cos_sin table is for rotary_dim {cos_sin.size(1) * 2}, asked {rotary_dim}")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    _check(_lib().llmrs_qk_norm_rope_kvwrite(
        _ptr(q), ctypes.c_longlong(_row_stride(q, "q")),
        _ptr(k), ctypes.c_longlong(_row_stride(k, "k") if k is not None else 0),
        _ptr(v), ctypes.c_longlong(_row_stride(v, "v") if v is not None else 0),
        _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_sin), _ptr(positions), _ptr(token_req), _ptr(block_table),
        block_table.size(1), _ptr(cache), n, n_q_heads, n_kv_heads, head_dim,
        rotary_dim if cos_sin is not None else 0, page_size, ctypes.c_float(eps), dtype_code(dt), _stream()),
        "qk_norm_rope_kvwrite")


def attn_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor, n_tiles: int,
                 q_start: torch.Tensor, n_new: torch.Tensor, cached_len: torch.Tensor, block_table: torch.Tensor,
                 n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                 prefer_tc: bool = False) -> None:
    """Causal attention of prompt portions over the paged cache (their own keys are already written).
    ``prefer_tc`` asks for the tcgen05 kernel (blocks of 128 queries) where it applies.

    ``tiles`` is int32 [n_tiles, 2]: (request row, offset of the tile's first query in
    the request's new tokens); a tile covers 64 queries.
    """
    _need(q, "q", contiguous=False)
    _need(out, "out", q.dtype, contiguous=False)
    _need(cache, "cache", q.dtype)
    for name, t in (("tiles", tiles), ("q_start", q_start), ("n_new", n_new), ("cached_len", cached_len),
                    ("block_table", block_table)):
        _need(t, name, torch.int32)
    _check(_lib().llmrs_attn_prefill(
        _ptr(q), ctypes.c_longlong(_row_stride(q, "q")), _ptr(out), ctypes.c_longlong(_row_stride(out, "out")),
        _ptr(cache), _ptr(tiles), n_tiles, _ptr(q_start), _ptr(n_new), _ptr(cached_len), _ptr(block_table),
        block_table.size(1), n_q_heads, n_kv_heads, head_dim, page_size, window, ctypes.c_float(scale),
        dtype_code(q.dtype), q.size(0), cache.size(0), 1 if prefer_tc else 0, _ptr(tc_error_flag(q.device)),
        _stream()), "attn_prefill")


def attn_decode_scratch_floats(n_dec: int, n_q_heads: int, head_dim: int, max_splits: int) -> int:
    return int(_lib_ll("llmrs_attn_decode_scratch_floats")(n_dec, n_q_heads, head_dim, max_splits))


_decode_capacity = {}


def attn_decode_capacity(head_dim: int, cluster: int, heads: int = 4, device=None, light: bool = False) -> int:
    """Blocks of the tensor-core decode attention kernel that the device holds at a time when they come in
    thread-block clusters of ``cluster`` (1 to 16) and serve ``heads`` query heads per key head (at most 16).
    ``light``: of the kernel with the ring of two tiles (``attn_decode(ring=2)``); 0 where it does not exist."""
    key = (head_dim, cluster, heads, device, light)
    if key not in _decode_capacity:
        blocks = ctypes.c_int()
        fn = _lib().llmrs_attn_decode_capacity_light if light else _lib().llmrs_attn_decode_capacity
        _check(fn(head_dim, cluster, heads, ctypes.byref(blocks)), "attn_decode_capacity", launches=0)
        _decode_capacity[key] = blocks.value
    return _decode_capacity[key]


def _lib_ll(name: str):
    fn = getattr(_lib(), name)
    fn.restype = ctypes.c_longlong
    return fn


def attn_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, dec_reqs: torch.Tensor, n_dec: int,
                q_start: torch.Tensor, cached_len: torch.Tensor, block_table: torch.Tensor, scratch: torch.Tensor,
                max_splits: int, split_keys: int, n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                window: int, scale: float, counters: Optional[torch.Tensor] = None,
                then: Optional[torch.Tensor] = None, ring: int = 0) -> None:
    """Attention of single new tokens (``dec_reqs``: int32 request rows) over the paged cache,
    the keys cut into splits of ``split_keys`` and merged; ``scratch`` is float32 workspace of
    ``attn_decode_scratch_floats`` elements. (bfloat16 with head_dim <= 128 and at most 16 splits: the splits
    of a request and key head run as one thread-block cluster and merge through distributed shared memory,
    one kernel; else a second kernel merges them.) With ``counters`` (int32, at least n_dec * n_q_heads,
    all zero; the call leaves them zero) the tensor-core kernel merges the splits itself instead
    of a second kernel doing it. ``ring`` = 2 asks for the tensor-core kernel with a ring of two tiles per warp, of
    which three blocks fit an SM instead of two (head_dim 128, at most 8 query heads per key head; elsewhere it
    changes nothing): for steps whose blocks then fit one wave and otherwise do not."""
    if then is not None:
        hint_next_weights(then, PREFETCH_BYTES_AFTER_ATTENTION)   # the weights of the product after attention
    _need(q, "q", contiguous=False)
    _need(out, "out", q.dtype, contiguous=False)
    _need(cache, "cache", q.dtype)
    _need(scratch, "scratch", torch.float32)
    for name, t in (("dec_reqs", dec_reqs), ("q_start", q_start), ("cached_len", cached_len),
                    ("block_table", block_table)):
        _need(t, name, torch.int32)
    need = attn_decode_scratch_floats(n_dec, n_q_heads, head_dim, max_splits)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode scratch holds {scratch.numel()} floats, {need} needed")
    if counters is not None:
        _need(counters, "counters", torch.int32)
        if counters.numel() < n_dec * n_q_heads:
            raise KernelError(f"attn_decode counters hold {counters.numel()} ints, {n_dec * n_q_heads} needed")
    if ring:
        fn = _lib().llmrs_attn_decode_next_ring
        fn.restype = None
        fn(int(ring))
    _check(_lib().llmrs_attn_decode(
        _ptr(q), ctypes.c_longlong(_row_stride(q, "q")), _ptr(out), ctypes.c_longlong(_row_stride(out, "out")),
        _ptr(cache), _ptr(dec_reqs), n_dec, _ptr(q_start), _ptr(cached_len), _ptr(block_table), block_table.size(1),
        _ptr(scratch), _ptr(counters), max_splits, split_keys, n_q_heads, n_kv_heads, head_dim, page_size, window,
        ctypes.c_float(scale), dtype_code(q.dtype), _stream()), "attn_decode",
        launches=1 if counters is not None or (q.dtype == torch.bfloat16 and head_dim <= 128 and max_splits <= 16
                                               and not _generic_only) else 2)


def scatter_tokens(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor, src_idx: torch.Tensor) -> None:
    """``dst[dst_idx[i]] = src[src_idx[i]]`` where ``dst_idx[i] >= 0`` (all int32, on the device)."""
    for name, t in (("dst", dst), ("dst_idx", dst_idx), ("src", src), ("src_idx", src_idx)):
        _need(t, name, torch.int32)
    _check(_lib().llmrs_scatter_tokens(_ptr(dst), _ptr(dst_idx), _ptr(src), _ptr(src_idx), dst_idx.numel(),
                                       _stream()), "scatter_tokens")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the first maximum of each row of float32 ``logits``."""
    _need(logits, "logits", torch.float32)
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32)
    _check(_lib().llmrs_argmax(_ptr(logits), n, vocab, _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], penalty: Optional[torch.Tensor], hist_tokens: Optional[torch.Tensor],
           hist_offsets: Optional[torch.Tensor], seeds: torch.Tensor, request_ids: torch.Tensor,
           gen_index: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Choose one token per row; ``logits`` (float32) are overwritten. See csrc/sampling.cu."""
    _need(logits, "logits", torch.float32)
    n, vocab = logits.shape
    _need(temperature, "temperature", torch.float32)
    for name, t, dt in (("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                        ("penalty", penalty, torch.float32), ("hist_tokens", hist_tokens, torch.int32),
                        ("hist_offsets", hist_offsets, torch.int32), ("seeds", seeds, torch.int64),
                        ("request_ids", request_ids, torch.int64), ("gen_index", gen_index, torch.int32)):
        if t is not None:
            _need(t, name, dt)
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(_lib().llmrs_sample(_ptr(logits), n, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(penalty),
                               _ptr(hist_tokens), _ptr(hist_offsets), _ptr(seeds), _ptr(request_ids),
                               _ptr(gen_index), _ptr(out), _stream()), "sample")
    return out


def philox_uniform(seed: int, request_id: int, index: int) -> float:
    """The uniform number in [0, 1) that the sampler draws for (seed, request, index); host code."""
    fn = _lib().llmrs_philox_uniform
    fn.restype = ctypes.c_float
    return float(fn(ctypes.c_ulonglong(seed & (2**64 - 1)), ctypes.c_ulonglong(request_id & (2**64 - 1)),
                    ctypes.c_uint(index)))


_generic_only = False


def attention_generic_only(on: bool) -> None:
    """Make bfloat16 attention take the generic kernels too (tests compare both implementations)."""
    global _generic_only
    _generic_only = bool(on)
    fn = _lib().llmrs_attention_generic_only
    fn.restype = None
    fn(1 if on else 0)


# -- bfloat16 products on tcgen05 ------------------------------------------------------------
EPILOGUE = {"store": 0, "residual": 1, "silu_mul": 2}
_tc_flags = {}


def tc_error_flag(device) -> torch.Tensor:
    """The int32 word the tcgen05 kernels write when one of their bounded waits ran out."""
    dev = torch.device(device)
    if dev not in _tc_flags:
        _tc_flags[dev] = torch.zeros((1,), dtype=torch.int32, device=dev)
    return _tc_flags[dev]


TC_ERROR_CODES = {1: "a tcgen05 product kernel gave up waiting on a barrier",
                  2: "the tcgen05 attention kernel gave up waiting on a barrier",
                  3: "the tcgen05 attention kernel found its shared memory misaligned"}


def tc_error_message(code: int) -> str:
    return f"{TC_ERROR_CODES.get(code, 'a tcgen05 kernel failed')} (code {code}); the step's output is invalid"


def check_tc_error(device) -> None:
    """Raise if a tcgen05 kernel (product or attention) gave up on a wait since the last check (synchronises)."""
    flag = tc_error_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        raise KernelError(tc_error_message(code))


def set_tc_wait_limit(polls: int = 0) -> None:
    """Polls of a barrier before a wait of the tcgen05 kernels gives up; 0 restores the default (2^22)."""
    lib = _lib()
    for name in ("llmrs_tc_set_wait_limit", "llmrs_attention_tc_set_wait_limit"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = None, [ctypes.c_uint]
        fn(int(polls))


def test_skip_copy(gemm_k_block: int = -1, attention_tile: int = -1) -> None:
    """For the test of the bounded waits only: the next launches of the tcgen05 product kernels leave out the
    copy of their k block ``gemm_k_block``, those of the attention kernel the keys of tile ``attention_tile``
    (-1: every copy is made, the default)."""
    lib = _lib()
    for name, v in (("llmrs_tc_test_skip_copy", gemm_k_block), ("llmrs_attention_tc_test_skip_copy", attention_tile)):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = None, [ctypes.c_int]
        fn(int(v))


test_skip_copy.__test__ = False     # not a test, whatever a collector makes of the name


# Bytes of the next kernel's weights that a decode kernel asks into the L2 when its own stream ends
# (LLMRS_PREFETCH_MB, 0 switches it off).
PREFETCH_BYTES = int(float(os.environ.get("LLMRS_PREFETCH_MB", "12")) * (1 << 20))
PREFETCH_BYTES_AFTER_ATTENTION = int(float(os.environ.get("LLMRS_PREFETCH_ATTN_MB", "12")) * (1 << 20))


def hint_next_weights(w: Optional[torch.Tensor], limit: Optional[int] = None) -> None:
    """Tell the next launch of a few-token product or of decode attention which weights the kernel AFTER it
    will stream: their first ``PREFETCH_BYTES`` are asked into the L2 when that launch's own loads are out.
    The hint is taken by the next such launch, whichever it is; ``None`` clears it."""
    fn = _lib().llmrs_set_next_prefetch
    limit = PREFETCH_BYTES if limit is None else limit
    if w is None or limit <= 0:
        fn(ctypes.c_void_p(0), ctypes.c_longlong(0))
        return
    n = min(w.numel() * w.element_size(), limit) // 16 * 16
    _check(fn(ctypes.c_void_p(w.data_ptr()), ctypes.c_longlong(n)), "set_next_prefetch", launches=0)


def debug_take():
    """The debug build's record (``LLMRS_DEBUG_KERNELS=1``): ``(code, value, where, count)`` of the index checks
    that failed since the last call, or None when nothing failed. Raises in a normal build, which checks nothing.
    Synchronises."""
    out = (ctypes.c_int * 4)()
    torch.cuda.synchronize()
    rc = _lib().llmrs_debug_take(out)
    if rc == 0:
        raise KernelError("this is not the debug build of the kernel library (set LLMRS_DEBUG_KERNELS=1 before import)")
    if rc < 0:
        raise KernelError("reading the debug record failed")
    return tuple(out) if out[3] else None


_SM_COUNT = {}


def sm_count(device) -> int:
    """SMs of the device (looked up once: the properties call costs microseconds, and products ask every time)."""
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def tc_splits(tokens: int, features: int, K: int, sms: int = 148) -> int:
    """Blocks of a cluster that share the k range of a skinny product: enough blocks to
    fill the GPU about twice, at least four 64-wide k blocks each."""
    if tokens > 64:
        return 1
    tiles = -(-features // 128)
    k_blocks = -(-K // 64)
    for s in (8, 4, 2):
        if tiles * s <= 2.2 * sms and k_blocks // s >= 4:
            return s
    return 1


def norm_parts(features: int, splits: int = 1, tokens: int = 1) -> int:
    """Rows of the sums of squares that a residual epilogue with ``emit`` writes: one per tile of features, 128
    wide for at most 64 tokens (the block of the cluster that owns a token writes the token's sum), 256 wide for
    more."""
    return -(-features // (128 if tokens <= 64 else 256))


def gemm_bf16_pairs(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, epilogue: str = "store",
                    out_dtype: torch.dtype = torch.bfloat16, acc_buffers: int = 2,
                    tmem_seen: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gemm_bf16`` for many tokens through the kernel that runs a tile of 256 x 256 on a pair of SMs
    (tcgen05.mma.cta_group::2; ``gemm_tc_pair_kernel`` in csrc/gemm_tcgen05.cu), called by itself. ``gemm_bf16``
    takes the same kernel from 129 tokens on (``use_tc_pairs``). ``acc_buffers``: accumulator tiles a block holds in
    tensor memory; ``tmem_seen`` (int32, one entry per block) receives the address each block was given."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    tokens, K = x.shape
    features = w.size(0)
    if w.size(1) != K:
        raise KernelError(f"x has {K} columns, w has {w.size(1)}")
    epi = EPILOGUE[epilogue]
    if epilogue == "residual":
        _need(out, "out", torch.float32)
        if out.shape != (tokens, features):
            raise KernelError(f"residual stream is {tuple(out.shape)}, product is {(tokens, features)}")
        odt = torch.float32
    else:
        width = features // 2 if epilogue == "silu_mul" else features
        odt = torch.bfloat16 if epilogue == "silu_mul" else out_dtype
        if out is None:
            out = torch.empty((tokens, width), dtype=odt, device=x.device)
        _need(out, "out", odt)
    if tmem_seen is not None:
        _need(tmem_seen, "tmem_seen", torch.int32)
        if tmem_seen.numel() < 2 * sm_count(x.device):
            raise KernelError("tmem_seen needs an entry per block (two per SM)")
    _check(_lib().llmrs_gemm_bf16_pairs(_ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(out),
                                        ctypes.c_longlong(out.stride(0)), tokens, features, K, epi, dtype_code(odt),
                                        acc_buffers, _ptr(tmem_seen), _ptr(tc_error_flag(x.device)), _stream()),
           "gemm_bf16_pairs")
    return out


def use_tc_pairs(on: bool) -> None:
    """Whether ``gemm_bf16`` sends steps of more than 128 tokens to the kernel on pairs of SMs (the default) or keeps
    them on the one-block persistent kernel."""
    fn = _lib().llmrs_tc_use_pairs
    fn.restype, fn.argtypes = None, [ctypes.c_int]
    fn(1 if on else 0)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, epilogue: str = "store",
              out_dtype: torch.dtype = torch.bfloat16, splits: Optional[int] = None, emit=None, scale=None,
              then: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T`` for bfloat16 ``x`` [tokens, K] and ``w`` [features, K] on tcgen05 (see csrc/gemm_tcgen05.cu).

    epilogue "store": returns [tokens, features] in ``out_dtype``. "residual": ``out`` is the
    float32 residual stream and gets the product added. "silu_mul": ``w`` alternates 64
    gate rows and 64 up rows; returns silu(gate) * up, [tokens, features / 2] bfloat16.

    A norm spread over two products: ``emit`` = (norm weight float32 [features], xw bfloat16 [tokens, features],
    parts float32 [norm_parts(features, splits, tokens), stride >= tokens]) makes a "residual" epilogue also write
    xw = (out + product) * weight and the sums of squares of each piece of the features;
    ``scale`` = (parts, n_parts, dim, eps) multiplies the product's rows by
    1 / sqrt(sum(parts[:n_parts, token]) / dim + eps).

    ``then`` (at most 64 tokens): the weights that the kernel after this one streams; their start is asked into
    the L2 when this product's own loads are out (``hint_next_weights``).
    """
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    tokens, K = x.shape
    if then is not None and tokens <= 64:
        hint_next_weights(then)
    features = w.size(0)
    if w.size(1) != K:
        raise KernelError(f"x has {K} columns, w has {w.size(1)}")
    epi = EPILOGUE[epilogue]
    if epilogue == "residual":
        _need(out, "out", torch.float32)
        if out.shape != (tokens, features):
            raise KernelError(f"residual stream is {tuple(out.shape)}, product is {(tokens, features)}")
        odt = torch.float32
    else:
        width = features // 2 if epilogue == "silu_mul" else features
        odt = torch.bfloat16 if epilogue == "silu_mul" else out_dtype
        if out is None:
            out = torch.empty((tokens, width), dtype=odt, device=x.device)
        _need(out, "out", odt)
    if splits is None:
        splits = tc_splits(tokens, features, K, sm_count(x.device))
    if emit is None and scale is None:
        _check(_lib().llmrs_gemm_bf16(_ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(out),
                                      ctypes.c_longlong(out.stride(0)), tokens, features, K, epi, dtype_code(odt),
                                      splits, _ptr(tc_error_flag(x.device)), _stream()), "gemm_bf16")
        return out
    e_w = e_xw = e_part = s_part = None
    stride = n_parts = dim = 0
    eps = 0.0
    if emit is not None:
        e_w, e_xw, e_part = emit
        _need(e_w, "emit weight", torch.float32)
        _need(e_xw, "emit xw", torch.bfloat16)
        _need(e_part, "emit parts", torch.float32)
        if e_w.numel() != features or e_xw.shape != (tokens, features) or e_part.size(0) < norm_parts(features, splits, tokens):
            raise KernelError("emit: weight, xw or parts do not fit the product")
        stride = e_part.size(1)
    if scale is not None:
        s_part, n_parts, dim, eps = scale
        _need(s_part, "scale parts", torch.float32)
        if emit is not None and s_part.size(1) != stride:
            raise KernelError("emit and scale parts must have rows of the same length")
        stride = s_part.size(1)
    _check(_lib().llmrs_gemm_bf16_norm(
        _ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(out), ctypes.c_longlong(out.stride(0)), tokens,
        features, K, epi, dtype_code(odt), splits, _ptr(e_w), _ptr(e_xw),
        ctypes.c_longlong(e_xw.stride(0) if e_xw is not None else 0), _ptr(e_part), _ptr(s_part), stride, n_parts, dim,
        ctypes.c_float(eps), _ptr(tc_error_flag(x.device)), _stream()), "gemm_bf16")
    return out


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor,
                  q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                  positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, n_q_heads: int,
                  n_kv_heads: int, page_size: int, eps: float, splits: Optional[int] = None, scale=None) -> torch.Tensor:
    """q | k | v = ``x @ w.T`` for at most 64 tokens and heads of 128 features, with the per-head norms,
    the rotation and the cache write in the product's epilogue: q lands in ``q_out`` (bfloat16
    [tokens, n_q_heads * 128]), k and v in the pages of ``cache`` that ``block_table`` names. The same
    arithmetic as ``gemm_bf16`` followed by ``qk_norm_rope_kvwrite``, one kernel and one rounding less.
    ``scale``: as in ``gemm_bf16`` (the rows of the product are scaled before the head norms)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(q_out, "q_out", torch.bfloat16)
    _need(cache, "cache", torch.bfloat16)
    tokens, K = x.shape
    features = (n_q_heads + 2 * n_kv_heads) * 128
    if w.shape != (features, K):
        raise KernelError(f"w is {tuple(w.shape)}, expected {(features, K)}")
    if q_out.shape != (tokens, n_q_heads * 128):
        raise KernelError(f"q_out is {tuple(q_out.shape)}, expected {(tokens, n_q_heads * 128)}")
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("cos_sin", cos_sin)):
        if t is not None:
            _need(t, name, torch.float32)
    if cos_sin is not None and cos_sin.size(1) != 64:
        raise KernelError(f"cos_sin table is for rotary_dim {cos_sin.size(1) * 2}, this kernel rotates 128")
    for name, t in (("positions", positions), ("token_req", token_req), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if splits is None:
        splits = tc_splits(tokens, features, K, sm_count(x.device))
    _check(_lib().llmrs_gemm_qkv_rope(
        _ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), tokens, K, splits, _ptr(q_out),
        ctypes.c_longlong(q_out.stride(0)), _ptr(cache), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_sin),
        _ptr(positions), _ptr(token_req), _ptr(block_table), block_table.size(1), n_q_heads, n_kv_heads, page_size,
        ctypes.c_float(eps), _ptr(scale[0] if scale else None), scale[0].size(1) if scale else 0,
        scale[1] if scale else 0, scale[2] if scale else 0, ctypes.c_float(scale[3] if scale else 0.0),
        _ptr(tc_error_flag(x.device)), _stream()), "gemm_qkv_rope")
    return q_out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K]: 64 rows of gate, the 64 matching rows of up, and so on (I a multiple of 64)."""
    I, K = gate.shape
    return torch.stack([gate.reshape(I // 64, 64, K), up.reshape(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()


def check_attention_error() -> None:
    """Raise if an attention kernel gave up on one of its bounded waits since the last check (synchronises).
    Launches through ``attn_prefill`` report into the word that ``check_tc_error`` reads; this also looks at
    the word inside the library, which launches without a word of the caller's use."""
    for dev in list(_tc_flags):
        check_tc_error(dev)
    lib = _lib()
    for name in ("llmrs_attention_tc_error",):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        if fn() > 0:
            raise KernelError(f"an attention kernel gave up waiting on a barrier ({name}); its output is invalid")


# -- blocks that norm a branch's output; token shift; soft cap ---------------------------------------
_LL = ctypes.c_longlong


def token_shift(x: torch.Tensor, mu: Optional[torch.Tensor], state: Optional[torch.Tensor], ctx,
                out_dtype: torch.dtype) -> torch.Tensor:
    """``y_t = x_t + (x_{t-1} - x_t) * mu`` over the float32 rows ``x`` of a step, rounded to ``out_dtype``. The row
    before a request's first token of the step comes from ``state[slot]`` (zeros after admission), which then takes
    the request's last row of the step. ``mu`` None: a plain conversion of ``x``."""
    _need(x, "x", torch.float32)
    n, width = x.shape
    out = torch.empty((n, width), dtype=out_dtype, device=x.device)
    if mu is not None:
        _need(mu, "mu", torch.float32)
        _need(state, "state", torch.float32)
        if mu.numel() != width or state.size(-1) != width:
            raise KernelError(f"token shift of width {width}: mu has {mu.numel()}, state rows {state.size(-1)}")
        args = (_ptr(ctx.token_req), _ptr(ctx.q_start), _ptr(ctx.n_new), _ptr(ctx.slot_ids))
    else:
        args = (None, None, None, None)
    _check(_lib().llmrs_token_shift(_ptr(x), _ptr(mu), _ptr(state), *args, _ptr(out), dtype_code(out_dtype), n, width,
                                    _stream()), "token_shift")
    return out


def outnorm_add(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``h += y / sqrt(mean(y^2) + eps) * weight`` row by row, in float32, in place."""
    _need(h, "h", torch.float32)
    _need(y, "y")
    _need(weight, "weight", torch.float32)
    if y.shape != h.shape or weight.numel() != h.size(-1):
        raise KernelError(f"outnorm_add: h {tuple(h.shape)}, y {tuple(y.shape)}, weight {weight.numel()}")
    _check(_lib().llmrs_outnorm_add(_ptr(h), _ptr(y), dtype_code(y.dtype), _ptr(weight), h.size(0), h.size(1),
                                    ctypes.c_float(eps), _stream()), "outnorm_add")
    return h


def softcap_(z: torch.Tensor, cap: float) -> torch.Tensor:
    """``z = cap * tanh(z / cap)`` in place (float32)."""
    _need(z, "z", torch.float32)
    _check(_lib().llmrs_softcap(_ptr(z), _LL(z.numel()), ctypes.c_float(cap), _stream()), "softcap")
    return z


def tanh_slice(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``tanh`` of a 2-D view with dense rows (a column slice of a wider product), as a contiguous tensor."""
    _need(x, "x", contiguous=False)
    out = torch.empty(tuple(x.shape), dtype=out_dtype, device=x.device)
    _check(_lib().llmrs_tanh_slice(_ptr(x), dtype_code(x.dtype), _LL(_row_stride(x, "x")), _ptr(out),
                                   dtype_code(out_dtype), x.size(0), x.size(1), _stream()), "tanh_slice")
    return out


# -- many small products in one launch ----------------------------------------------------------------
GROUPED_TILE_ROWS = 64      # rows of a tile of the grouped product; 128 where groups have many rows (``grouped_tile_rows``)


def grouped_tile_rows(n_rows: int, n_groups: int) -> int:
    """Rows per tile for ``moe_sort`` and ``gemm_grouped``: 128 when the groups hold some hundred rows each (prompts:
    a larger tile reads the weights half as often), else 64."""
    return 128 if n_rows >= 96 * n_groups else GROUPED_TILE_ROWS



def _strides3(t: torch.Tensor, name: str):
    """(row stride, batch stride) of a [rows, batches, cols] view with dense columns."""
    if t.dim() != 3 or (t.size(2) > 1 and t.stride(2) != 1):
        raise KernelError(f"{name} must be [rows, batches, cols] with dense columns, got {tuple(t.shape)} {t.stride()}")
    return t.stride(0), t.stride(1)


def grouped_use_tensor_cores(on: bool) -> None:
    """False: ``gemm_batched`` and ``gemm_grouped`` take the CUDA-core kernel for bfloat16 too (for tests that compare
    the two kernels). The default is True."""
    fn = _lib().llmrs_gemm_grouped_use_mma
    fn.restype, fn.argtypes = None, [ctypes.c_int]
    fn(1 if on else 0)


def gemm_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, round_x: bool = False) -> torch.Tensor:
    """``out[m, b, :] = w[b] @ x[m, b, :]`` for x [M, B, K] and out [M, B, N] (any row and batch strides) and
    w [B, N, K] contiguous: the heads of a tensor as batches, without a copy. float32 accumulation on the CUDA
    cores in a fixed order over k."""
    _need(x, "x", contiguous=False)
    _need(w, "w")
    _need(out, "out", contiguous=False)
    M, B, K = x.shape
    if w.dim() != 3 or w.size(0) != B or w.size(2) != K or out.shape != (M, B, w.size(1)):
        raise KernelError(f"gemm_batched: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    xs, xb = _strides3(x, "x")
    os_, ob = _strides3(out, "out")
    N = w.size(1)
    _check(_lib().llmrs_gemm_grouped(
        _ptr(x), dtype_code(x.dtype), _LL(xs), _LL(xb), _ptr(w), None, dtype_code(w.dtype), _LL(N * K), _ptr(out),
        dtype_code(out.dtype), _LL(os_), _LL(ob), M, N, K, B, None, None, 0, 0, None, int(round_x), ctypes.c_float(0),
        ctypes.c_float(0), ctypes.c_float(0), _stream()), "gemm_batched")
    return out


def gemm_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor,
                 src: Optional[torch.Tensor], w2: Optional[torch.Tensor] = None, round_x: bool = False,
                 limit: float = 0.0, alpha: float = 0.0, shift: float = 0.0,
                 tile_rows: int = GROUPED_TILE_ROWS) -> torch.Tensor:
    """Rows sorted by group against each group's own weights: ``out[r] = w[g(r)] @ x[src[r]]`` for the rows of every
    tile (``tiles`` [max, 3] = group, first row, at most ``tile_rows`` rows; ``n_tiles`` on the device; from ``moe_sort``). With ``w2`` the
    gated unit ``g * sigmoid(alpha * g) * (u + shift)``, g = min(w x, limit), u = clamp(w2 x, -limit, limit)."""
    _need(x, "x", contiguous=False)
    _need(w, "w")
    _need(out, "out")
    _need(tiles, "tiles", torch.int32)
    _need(n_tiles, "n_tiles", torch.int32)
    G, N, K = w.shape
    if x.size(1) != K or out.size(1) != N or (w2 is not None and w2.shape != w.shape):
        raise KernelError(f"gemm_grouped: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if src is not None:
        _need(src, "src", torch.int32)
    _check(_lib().llmrs_gemm_grouped(
        _ptr(x), dtype_code(x.dtype), _LL(_row_stride(x, "x")), _LL(0), _ptr(w), _ptr(w2), dtype_code(w.dtype),
        _LL(N * K), _ptr(out), dtype_code(out.dtype), _LL(out.stride(0)), _LL(0), out.size(0), N, K, 0, _ptr(tiles),
        _ptr(n_tiles), tiles.size(0), tile_rows, _ptr(src), int(round_x), ctypes.c_float(limit), ctypes.c_float(alpha),
        ctypes.c_float(shift), _stream()), "gemm_grouped")
    return out


# -- mixtures of experts --------------------------------------------------------------------------------
def moe_route_table(token_ids: torch.Tensor, table: torch.Tensor, n_experts: int):
    """Routing by token id: ``table`` [vocab, top] int32 names each id's experts, all weighted 1/top. Returns
    (expert_of int32 [tokens * top], weight_of float32 [tokens * top])."""
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table", torch.int32)
    vocab, top = table.shape
    n = token_ids.numel()
    expert_of = torch.empty((n * top,), dtype=torch.int32, device=table.device)
    weight_of = torch.empty((n * top,), dtype=torch.float32, device=table.device)
    _check(_lib().llmrs_moe_route_table(_ptr(token_ids), _ptr(table), _ptr(expert_of), _ptr(weight_of), n, top, vocab,
                                        n_experts, _stream()), "moe_route_table")
    return expert_of, weight_of


def moe_sort(expert_of: torch.Tensor, top: int, n_experts: int, tile_rows: int = GROUPED_TILE_ROWS,
             tiled_groups: int = -1):
    """Order the assignments by expert. Returns (row_of [assignments], src_token [assignments], tiles [max, 3],
    n_tiles [1]): see ``gemm_grouped``. With ``tiled_groups`` >= 0 only the first so many groups get tiles: the rows
    of the others are sorted but run no product."""
    _need(expert_of, "expert_of", torch.int32)
    n = expert_of.numel()
    dev = expert_of.device
    row_of = torch.empty((n,), dtype=torch.int32, device=dev)
    src_token = torch.empty((n,), dtype=torch.int32, device=dev)
    max_tiles = -(-n // tile_rows) + n_experts
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=dev)
    n_tiles = torch.empty((1,), dtype=torch.int32, device=dev)
    _check(_lib().llmrs_moe_sort(_ptr(expert_of), _ptr(row_of), _ptr(src_token), _ptr(tiles), _ptr(n_tiles), n, top,
                                 n_experts, tile_rows, tiled_groups, _stream()), "moe_sort")
    return row_of, src_token, tiles, n_tiles


def moe_combine(rows: torch.Tensor, row_of: torch.Tensor, weight_of: torch.Tensor, top: int,
                out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``out[t] = sum_k weight_of[t, k] * rows[row_of[t, k]]`` in float32, k in order."""
    _need(rows, "rows", torch.float32)
    n = row_of.numel() // top
    out = torch.empty((n, rows.size(1)), dtype=out_dtype, device=rows.device)
    _check(_lib().llmrs_moe_combine(_ptr(rows), _ptr(row_of), _ptr(weight_of), _ptr(out), dtype_code(out_dtype), n, top,
                                    rows.size(1), _stream()), "moe_combine")
    return out


# -- the generalized delta rule -------------------------------------------------------------------------
def delta_rule(r, k, v, gate, a_raw, decay_raw, decay_bias, a_bias, norm_w, state, ctx, n_heads: int, d: int,
               decay_scale: float, key_eps: float, norm_eps: float) -> torch.Tensor:
    """The recurrence of ``csrc/delta_rule.cu`` over a step's tokens. r, k, v, gate, a_raw: column slices
    [tokens, heads * d] of one product (equal row strides); decay_raw float32 [tokens, heads * d] contiguous;
    state float32 [slots, heads, d, d], updated in place. Returns [tokens, heads * d] in the activation type."""
    stride = _row_stride(r, "r")
    for name, t in (("k", k), ("v", v), ("gate", gate), ("a_raw", a_raw)):
        _need(t, name, r.dtype, contiguous=False)
        if _row_stride(t, name) != stride:
            raise KernelError("delta_rule: the slices must share their row stride")
    _need(decay_raw, "decay_raw", torch.float32)
    _need(state, "state", torch.float32)
    out = torch.empty((r.size(0), n_heads * d), dtype=r.dtype, device=r.device)
    work = torch.empty((7 * r.size(0) * n_heads * d,), dtype=torch.float32, device=r.device)     # six prepared rows and o
    _check(_lib().llmrs_delta_rule(
        _ptr(r), _ptr(k), _ptr(v), _ptr(gate), _ptr(a_raw), _LL(stride), dtype_code(r.dtype), _ptr(decay_raw),
        _ptr(decay_bias), _ptr(a_bias), _ptr(norm_w), _ptr(state), _ptr(ctx.q_start), _ptr(ctx.n_new),
        _ptr(ctx.slot_ids), _ptr(work), _ptr(out), r.size(0), ctx.n_requests, n_heads, d, ctypes.c_float(decay_scale),
        ctypes.c_float(key_eps), ctypes.c_float(norm_eps), _stream()), "delta_rule", 3)
    return out


# -- latent attention -----------------------------------------------------------------------------------
def latent_prepare(q: torch.Tensor, dkv: Optional[torch.Tensor], latent_norm_w, inv_freq: torch.Tensor, ctx, table,
                   cache: Optional[torch.Tensor], page_size: int, n_heads: int, dn: int, dr: int, rot_dims: int,
                   rank: int, eps: float, neighbours: bool = False, magnitude: float = 1.0) -> None:
    """Rotate the rot part of every query head of ``q`` ([tokens, heads * (dn + dr)] view) in place; with ``dkv``
    ([tokens, rank + dr] view) also norm the latent and rotate the shared key part into the pages ``cache``
    ([pages, 1, page_size * (rank + dr)]). Pair i of the rotation is the entries (i, i + rot_dims/2), with
    ``neighbours`` (2i, 2i + 1); cosines and sines are multiplied by ``magnitude``."""
    _need(q, "q", contiguous=False)
    _need(inv_freq, "inv_freq", torch.float64)
    if dkv is not None:
        _need(dkv, "dkv", q.dtype, contiguous=False)
        _need(cache, "cache", q.dtype)
    _check(_lib().llmrs_latent_prepare(
        _ptr(q), _LL(_row_stride(q, "q")), _ptr(dkv), _LL(0 if dkv is None else _row_stride(dkv, "dkv")),
        dtype_code(q.dtype), _ptr(latent_norm_w), _ptr(inv_freq), _ptr(ctx.positions), _ptr(ctx.token_req),
        _ptr(table), 0 if table is None else table.size(1), _ptr(cache), page_size, q.size(0), n_heads, dn, dr,
        rot_dims, rank, ctypes.c_float(eps), int(bool(neighbours)), ctypes.c_float(magnitude), _stream()),
        "latent_prepare")


LATENT_FEW_TOKENS = 64      # steps of at most this many tokens take the latent attention kernel laid out for latency


def latent_attention_splits(n_tokens: int, n_heads: int, span: int, sms: int, mma: bool = False):
    """(splits, keys per split) for a step of ``n_tokens`` whose tokens see at most ``span`` keys: few tokens (decoding)
    cut their keys over several blocks; many tokens are not cut. The CUDA-core kernel (a block per token and four
    heads) fills the device about four times, at 64 keys or more each (measured at 16 heads over a latent of 512 and
    4,096 keys: 8 tokens 165 us with 9 runs of keys, 133 us with 18; 64 tokens 1,194 us uncut, 812 us in 2 runs; more
    runs than that lose again). The tensor-core kernel (``mma``: a block per token and up to 32 heads) fills it about
    twice, at 128 keys or more each. Runs are multiples of 16 keys and cover ``span`` + 15 (a run starts at a multiple
    of 16 at or below the first visible key)."""
    span += 15
    if mma:
        blocks = n_tokens * -(-n_heads // latent_decode_mma_heads(n_heads))
        splits = min(max(1, (2 * sms) // max(blocks, 1)), max(1, span // 128))
    else:
        blocks = n_tokens * -(-n_heads // (4 if n_heads >= 4 else 1))
        splits = min(max(1, (4 * sms) // max(blocks, 1)), max(1, span // 64))
    if splits <= 1:
        return 1, 0
    keys = -(-(-(-span // splits)) // 16) * 16
    return -(-span // keys), keys


_latent_decode_mma = os.environ.get("LLMRS_LATENT_DECODE_MMA", "1") != "0"
_latent_decode_mma_sent = None


def latent_decode_mma(on: bool) -> None:
    """Steps of few tokens in bfloat16 take the tensor-core kernel of latent attention where the sizes fit (default,
    ``LLMRS_LATENT_DECODE_MMA=0`` at import switches it off), or always the CUDA-core kernel."""
    global _latent_decode_mma
    _latent_decode_mma = bool(on)


def latent_decode_mma_heads(n_heads: int) -> int:
    """Heads per block of the tensor-core kernel for steps of few tokens."""
    return 32 if n_heads > 16 else 16


def latent_decode_takes_mma(dtype: torch.dtype, rank: int, dr: int, page_size: int) -> bool:
    """Whether a step of few tokens with these sizes runs on the tensor cores (the kernel's own conditions)."""
    return (_latent_decode_mma and dtype == torch.bfloat16 and rank % 64 == 0 and rank <= 512 and dr % 16 == 0
            and page_size % 16 == 0)


def latent_attention(qa: torch.Tensor, q: torch.Tensor, gate: torch.Tensor, cache: torch.Tensor, table, ctx,
                     out: torch.Tensor, n_heads: int, dn: int, dr: int, rank: int, page_size: int, window: int,
                     scale: float, splits: int = 1, split_keys: int = 0) -> torch.Tensor:
    """Attention over cached latent rows with folded queries ``qa`` [tokens, heads, rank]; ``q`` the rotated
    projected queries, ``gate`` the raw per-head gates [tokens, heads]; ``out`` [tokens, heads, rank] (any strides).
    ``splits`` > 1 cuts every token's visible keys into that many runs of ``split_keys`` (which must cover the longest
    visible span) that separate blocks take; a second kernel merges them."""
    _need(qa, "qa", contiguous=False)
    _need(q, "q", qa.dtype, contiguous=False)
    _need(gate, "gate", qa.dtype, contiguous=False)
    _need(cache, "cache", qa.dtype)
    _need(out, "out", qa.dtype, contiguous=False)
    qs, qh = _strides3(qa, "qa")
    os_, oh = _strides3(out, "out")
    partial = None
    few = qa.size(0) <= LATENT_FEW_TOKENS       # the kernel laid out for latency always leaves partial results
    if few and splits <= 1:
        splits, split_keys = 1, 1 << 29
    if splits > 1 or few:
        n_floats = qa.size(0) * n_heads * splits * (rank + 2)
        partial = ctx.scratch("latent_attention", n_floats) if hasattr(ctx, "scratch") else torch.empty(
            (n_floats,), dtype=torch.float32, device=qa.device)
    global _latent_decode_mma_sent
    if _latent_decode_mma_sent != _latent_decode_mma:
        _lib().llmrs_latent_decode_mma(int(_latent_decode_mma))
        _latent_decode_mma_sent = _latent_decode_mma
    _check(_lib().llmrs_latent_attention(
        _ptr(qa), _LL(qs), _LL(qh), _ptr(q), _LL(_row_stride(q, "q")), dn, dn + dr, _ptr(gate),
        _LL(_row_stride(gate, "gate")), _ptr(cache), dtype_code(qa.dtype), _ptr(table), table.size(1),
        _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(out), _LL(os_), _LL(oh), qa.size(0), n_heads, rank, dr,
        page_size, window, ctypes.c_float(scale), splits, split_keys, _ptr(partial), int(few), _stream()),
        "latent_attention", 2 if partial is not None else 1)
    return out


def latent_prefill_tile_tokens(n_heads: int) -> int:
    """Tokens per tile of ``latent_attention_prefill`` for a number of heads."""
    return int(_lib().llmrs_latent_prefill_tile_tokens(n_heads))


def latent_attention_prefill(qa: torch.Tensor, q: torch.Tensor, gate: torch.Tensor, cache: torch.Tensor, table, ctx,
                             tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int, dn: int, dr: int,
                             rank: int, page_size: int, window: int, scale: float) -> bool:
    """``latent_attention`` for prompt portions in bfloat16 on the tensor cores. ``tiles`` int32 [n_tiles, 2]: first
    token of the step and number of tokens (at most ``latent_prefill_tile_tokens``) of consecutive tokens of one
    request. Returns False, having launched nothing, when the sizes do not fit the kernel (rank % 64, rot % 16,
    pages of a multiple of 16 keys): the caller then takes ``latent_attention``."""
    _need(qa, "qa", torch.bfloat16, contiguous=False)
    _need(q, "q", torch.bfloat16, contiguous=False)
    _need(gate, "gate", torch.bfloat16, contiguous=False)
    _need(cache, "cache", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    _need(tiles, "tiles", torch.int32)
    qs, qh = _strides3(qa, "qa")
    os_, oh = _strides3(out, "out")
    rc = _lib().llmrs_latent_attention_prefill(
        _ptr(qa), _LL(qs), _LL(qh), _ptr(q), _LL(_row_stride(q, "q")), dn, dn + dr, _ptr(gate),
        _LL(_row_stride(gate, "gate")), _ptr(cache), _ptr(table), table.size(1), _ptr(ctx.positions),
        _ptr(ctx.token_req), _ptr(tiles), n_tiles, _ptr(out), _LL(os_), _LL(oh), n_heads, rank, dr, page_size, window,
        ctypes.c_float(scale), _stream())
    if rc == -2:
        return False
    _check(rc, "latent_attention_prefill")
    return True


# -- blocks that norm after the residual sum; small element-wise kernels -----------------------------------
def post_norm(h: torch.Tensor, y: Optional[torch.Tensor], layer_scale: Optional[torch.Tensor], weight: torch.Tensor,
              alpha: float, eps: float, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``h = rms(alpha * h + y * layer_scale) * weight`` row by row, in place on the float32 stream ``h`` (``y`` and
    ``layer_scale`` may be None). With ``out_dtype`` the rows are also returned rounded to that type."""
    _need(h, "h", torch.float32)
    _need(weight, "weight", torch.float32)
    if y is not None:
        _need(y, "y")
        if y.shape != h.shape:
            raise KernelError(f"post_norm: h {tuple(h.shape)}, y {tuple(y.shape)}")
    if layer_scale is not None:
        _need(layer_scale, "layer_scale", torch.float32)
    if weight.numel() != h.size(1) or (layer_scale is not None and layer_scale.numel() != h.size(1)):
        raise KernelError(f"post_norm: rows of {h.size(1)}, weight {weight.numel()}")
    out = None if out_dtype is None else torch.empty(tuple(h.shape), dtype=out_dtype, device=h.device)
    _check(_lib().llmrs_post_norm(
        _ptr(h), _ptr(y), dtype_code(y.dtype) if y is not None else F32, _ptr(layer_scale), _ptr(weight), _ptr(out),
        dtype_code(out_dtype) if out_dtype is not None else F32, h.size(0), h.size(1), ctypes.c_float(alpha),
        ctypes.c_float(eps), _stream()), "post_norm")
    return out


def relu_sq(x: torch.Tensor) -> torch.Tensor:
    """``max(x, 0)^2`` element by element."""
    _need(x, "x")
    out = torch.empty_like(x)
    _check(_lib().llmrs_relu_sq(_ptr(x), _ptr(out), _LL(x.numel()), dtype_code(x.dtype), _stream()), "relu_sq")
    return out


def scale_(z: torch.Tensor, s: float) -> torch.Tensor:
    """``z *= s`` in place (float32)."""
    _need(z, "z", torch.float32)
    _check(_lib().llmrs_scale(_ptr(z), _LL(z.numel()), ctypes.c_float(s), _stream()), "scale")
    return z


# -- linear recurrences with a matrix state ---------------------------------------------------------------
def gate_scan(gates: torch.Tensor, cap: float, m_state: torch.Tensor, ctx, n_heads: int):
    """Exponential gates with a running maximum over a step's tokens (``csrc/linear_recurrence.cu``). ``gates``:
    float32 [tokens, 2 * heads], the input gate's pre-activations then the forget gate's; ``m_state`` float32
    [slots, heads], updated in place. Returns (decay, gain, floor), each float32 [tokens, heads]."""
    _need(gates, "gates", torch.float32, contiguous=False)
    _need(m_state, "m_state", torch.float32)
    n = gates.size(0)
    if gates.size(1) != 2 * n_heads or m_state.size(-1) != n_heads:
        raise KernelError(f"gate_scan: gates {tuple(gates.shape)}, state {tuple(m_state.shape)}, {n_heads} heads")
    decay, gain, floor = (torch.empty((n, n_heads), dtype=torch.float32, device=gates.device) for _ in range(3))
    _check(_lib().llmrs_gate_scan(_ptr(gates), _LL(_row_stride(gates, "gates")), ctypes.c_float(cap), _ptr(m_state),
                                  _ptr(ctx.q_start), _ptr(ctx.n_new), _ptr(ctx.slot_ids), _ptr(decay), _ptr(gain),
                                  _ptr(floor), ctx.n_requests, n_heads, _stream()), "gate_scan")
    return decay, gain, floor


def linear_recurrence(q, k, v, gate, norm_w, state, ctx, n_heads: int, dk: int, dv: int, norm_eps: float,
                      act_silu: bool = False, q_scale: float = 1.0, decay=None, head_decay=None, gain=None,
                      normaliser=None, floor=None, den_eps: float = 0.0, per_head_norm: bool = True) -> torch.Tensor:
    """``S_t = a_t S_(t-1) + (b_t k_t) v_t^T``, ``o_t = S_t^T q_t`` per head over a step's tokens, continued from and
    left in ``state`` [slots, heads, dk, dv]; then the output stage (division by the normaliser, RMS norm per head or
    over all heads, weight, sigmoid gate). q, k, v, gate: column slices of the activation type with dense rows;
    ``decay``/``gain`` float32 [tokens, heads] or None (``head_decay`` [heads]: one decay per head; nothing: 1);
    ``normaliser`` [slots, heads, dk] with ``floor`` [tokens, heads]: o is divided by
    ``max(|n . q|, floor) + den_eps``. Returns [tokens, heads * dv] in the activation type."""
    for name, t in (("q", q), ("k", k), ("v", v), ("gate", gate)):
        _need(t, name, q.dtype, contiguous=False)
    _need(state, "state", torch.float32)
    n = q.size(0)
    if q.size(1) != n_heads * dk or k.size(1) != n_heads * dk or v.size(1) != n_heads * dv or \
            gate.size(1) != n_heads * dv or tuple(state.shape[1:]) != (n_heads, dk, dv):
        raise KernelError(f"linear_recurrence: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, "
                          f"state {tuple(state.shape)} for {n_heads} heads of {dk} x {dv}")
    if (normaliser is None) != (floor is None):
        raise KernelError("linear_recurrence: normaliser and floor come together")
    dev = q.device
    work = torch.empty((int(_lib_ll("llmrs_linear_recurrence_work_floats")(n, n_heads, dk, dv)),), dtype=torch.float32,
                       device=dev)
    o_raw = torch.empty((n, n_heads * dv), dtype=torch.float32, device=dev)
    nq = torch.empty((n, n_heads), dtype=torch.float32, device=dev) if normaliser is not None else None
    _check(_lib().llmrs_linear_recurrence(
        _ptr(q), _ptr(k), _ptr(v), _LL(_row_stride(q, "q")), _LL(_row_stride(k, "k")), _LL(_row_stride(v, "v")),
        dtype_code(q.dtype), int(act_silu), ctypes.c_float(q_scale), _ptr(decay), _ptr(head_decay), _ptr(gain),
        _ptr(state), _ptr(normaliser), _ptr(ctx.q_start), _ptr(ctx.n_new), _ptr(ctx.slot_ids), _ptr(work),
        _ptr(o_raw), _ptr(nq), n, ctx.n_requests, n_heads, dk, dv, _stream()), "linear_recurrence", 2)
    out = torch.empty((n, n_heads * dv), dtype=q.dtype, device=dev)
    _check(_lib().llmrs_recurrence_output(
        _ptr(o_raw), _ptr(nq), _ptr(floor), ctypes.c_float(den_eps), _ptr(gate), _LL(_row_stride(gate, "gate")),
        dtype_code(q.dtype), _ptr(norm_w), _ptr(out), n, n_heads, dv, int(per_head_norm), ctypes.c_float(norm_eps),
        _stream()), "recurrence_output")
    return out


# -- attention with options on the score --------------------------------------------------------------------
MASK_CAUSAL, MASK_WINDOW, MASK_CHUNK = 0, 1, 2


def scored_prepare(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_norm_w, k_norm_w,
                   inv_freq: torch.Tensor, ctx, table, cache: Optional[torch.Tensor], n_q_heads: int,
                   n_kv_heads: int, dk: int, dv: int, rot_dims: int, page_size: int, eps: float,
                   unit_heads: bool = False, unit_values: bool = False, v_first: Optional[torch.Tensor] = None,
                   v_mix: Optional[torch.Tensor] = None) -> None:
    """Norm over the whole q and k rows, rotation, q rewritten in place, k and v into the pages ``cache``
    ([pages, kv heads, page_size * (dk + dv)]); with ``unit_heads`` every head of q and k is instead divided by its
    own root mean square after the rotation (no weights); with ``unit_values`` every head of v by its own before it is
    kept; with ``v_first`` (another layer's values of the same tokens) and ``v_mix`` (one float32 on the device) the
    kept value is ``(1 - v_mix) v + v_mix v_first``; see ``csrc/attention_scored.cu``."""
    _need(q, "q", contiguous=False)
    _need(inv_freq, "inv_freq", torch.float64)
    if k is not None:
        _need(k, "k", q.dtype, contiguous=False)
        _need(v, "v", q.dtype, contiguous=False)
        _need(cache, "cache", q.dtype)
    if v_first is not None:
        _need(v_first, "v_first", q.dtype, contiguous=False)
        _need(v_mix, "v_mix", torch.float32)
        if v is None or v_first.shape != v.shape:
            raise KernelError("scored_prepare: v_first must have the shape of v")
    _check(_lib().llmrs_scored_prepare(
        _ptr(q), _LL(_row_stride(q, "q")), _ptr(k), _LL(0 if k is None else _row_stride(k, "k")), _ptr(v),
        _LL(0 if v is None else _row_stride(v, "v")), dtype_code(q.dtype), _ptr(q_norm_w), _ptr(k_norm_w),
        _ptr(inv_freq), _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(table), 0 if table is None else table.size(1),
        _ptr(cache), q.size(0), n_q_heads, n_kv_heads, dk, dv, rot_dims, page_size, ctypes.c_float(eps),
        int(bool(unit_heads)), int(bool(unit_values)), _ptr(v_first),
        _LL(0 if v_first is None else _row_stride(v_first, "v_first")), _ptr(v_mix), _stream()), "scored_prepare")


def scored_generic_only(on: bool) -> None:
    """True: bfloat16 prompt portions take the kernel for any type too (tests compare it with the tensor-core one)."""
    fn = _lib().llmrs_scored_generic_only
    fn.restype, fn.argtypes = None, [ctypes.c_int]
    fn(1 if on else 0)


def scored_prefill(q, out, cache, tiles, n_tiles: int, ctx, table, n_q_heads: int, n_kv_heads: int, dk: int, dv: int,
                   page_size: int, scale: float, softcap: float, sink, mask: int, mask_size: int,
                   prefer_tc: bool = False, bias: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """Prompt portions (tiles of 64 queries: request, offset) through ``csrc/attention_scored.cu``. ``prefer_tc`` asks
    for the tcgen05 kernel where it applies (bfloat16, keys and values of 128 channels, pages of a multiple of 16
    keys; worth it when the portions are long). ``bias``: float32 [distances, query heads], added to the score of a
    key that many positions behind its query (the last row for every greater distance); ``out_scale`` multiplies
    the output."""
    _need(q, "q", contiguous=False)
    _need(out, "out", q.dtype, contiguous=False)
    _need(cache, "cache", q.dtype)
    _check_bias(bias, n_q_heads)
    _check(_lib().llmrs_scored_prefill(
        _ptr(q), _LL(_row_stride(q, "q")), _ptr(out), _LL(_row_stride(out, "out")), _ptr(cache), _ptr(tiles), n_tiles,
        _ptr(ctx.q_start), _ptr(ctx.n_new), _ptr(ctx.cached_len), _ptr(table), table.size(1), n_q_heads, n_kv_heads,
        dk, dv, page_size, ctypes.c_float(scale), ctypes.c_float(softcap), _ptr(sink), mask, mask_size, _ptr(bias),
        0 if bias is None else bias.size(0), ctypes.c_float(out_scale), dtype_code(q.dtype), q.size(0), cache.size(0),
        int(prefer_tc), _stream()), "scored_prefill")


def _check_bias(bias: Optional[torch.Tensor], n_q_heads: int) -> None:
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.dim() != 2 or bias.size(1) != n_q_heads or bias.size(0) < 1:
            raise KernelError(f"a distance bias of shape {tuple(bias.shape)} for {n_q_heads} query heads")


def scored_decode_group(n_q_heads: int, n_kv_heads: int, dk: int, dv: int, page_size: int, dtype: torch.dtype) -> int:
    """Query heads of one key head that a block of the decode kernel takes together (1, 2 or 4), or 0 where the rows
    cannot be read sixteen bytes a load and a block takes one query head with a warp per key."""
    return int(_lib().llmrs_scored_decode_group(n_q_heads, n_kv_heads, dk, dv, page_size, dtype_code(dtype)))


def scored_decode(q, out, cache, dec_reqs, n_dec: int, ctx, table, max_splits: int, split_keys: int, n_q_heads: int,
                  n_kv_heads: int, dk: int, dv: int, page_size: int, scale: float, softcap: float, sink, mask: int,
                  mask_size: int, bias: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """Requests that bring one token: runs of ``split_keys`` keys from each request's first visible key. ``bias`` and
    ``out_scale`` as in ``scored_prefill``."""
    _check_bias(bias, n_q_heads)
    _need(q, "q", contiguous=False)
    _need(out, "out", q.dtype, contiguous=False)
    _need(cache, "cache", q.dtype)
    n_floats = int(_lib_ll("llmrs_scored_decode_scratch_floats")(n_dec, n_q_heads, dv, max_splits))
    scratch = ctx.scratch("scored_decode", n_floats)
    _check(_lib().llmrs_scored_decode(
        _ptr(q), _LL(_row_stride(q, "q")), _ptr(out), _LL(_row_stride(out, "out")), _ptr(cache), _ptr(dec_reqs), n_dec,
        _ptr(ctx.q_start), _ptr(ctx.cached_len), _ptr(table), table.size(1), _ptr(scratch), max_splits, split_keys,
        n_q_heads, n_kv_heads, dk, dv, page_size, ctypes.c_float(scale), ctypes.c_float(softcap), _ptr(sink), mask,
        mask_size, _ptr(bias), 0 if bias is None else bias.size(0), ctypes.c_float(out_scale), dtype_code(q.dtype),
        _stream()), "scored_decode", 2)


# -- learned routers ----------------------------------------------------------------------------------------
def moe_route_top(logits: torch.Tensor, n_experts: int, top: int):
    """The ``top`` largest of each row's first ``n_experts`` logits (float32, rows may be wider), weighted by the
    softmax over the chosen logits only; among equal logits the lower expert wins. Returns (expert_of int32
    [tokens * top], weight_of float32 [tokens * top]) in order of falling logit."""
    _need(logits, "logits", torch.float32, contiguous=False)
    n = logits.size(0)
    if logits.size(1) < n_experts or not 1 <= top <= n_experts:
        raise KernelError(f"moe_route_top: logits {tuple(logits.shape)}, {n_experts} experts, top {top}")
    expert_of = torch.empty((n * top,), dtype=torch.int32, device=logits.device)
    weight_of = torch.empty((n * top,), dtype=torch.float32, device=logits.device)
    _check(_lib().llmrs_moe_route_top(_ptr(logits), _LL(_row_stride(logits, "logits")), _ptr(expert_of),
                                      _ptr(weight_of), n, n_experts, top, _stream()), "moe_route_top")
    return expert_of, weight_of


def moe_combine_shared(rows, row_of, weight_of, top: int, shared: Optional[torch.Tensor] = None,
                       shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``moe_combine`` plus an expert that every token uses: ``out[t] += sigmoid(shared_gate[t]) * shared[t]``
    (``shared_gate``: float32, one number per token, any stride; None: the shared rows are added as they are)."""
    _need(rows, "rows", torch.float32)
    n = row_of.numel() // top
    out = torch.empty((n, rows.size(1)), dtype=torch.float32, device=rows.device)
    if shared is not None:
        _need(shared, "shared")
        if shared.shape != out.shape:
            raise KernelError(f"moe_combine_shared: shared {tuple(shared.shape)}, out {tuple(out.shape)}")
    gate_stride = 0
    if shared_gate is not None:
        _need(shared_gate, "shared_gate", torch.float32, contiguous=False)
        gate_stride = shared_gate.stride(0)
    _check(_lib().llmrs_moe_combine_shared(
        _ptr(rows), _ptr(row_of), _ptr(weight_of), _ptr(shared), dtype_code(shared.dtype) if shared is not None else F32,
        _ptr(shared_gate), _LL(gate_stride), _ptr(out), n, top, rows.size(1), _stream()), "moe_combine_shared")
    return out


def head_gate(out: torch.Tensor, gate: torch.Tensor, n_heads: int, dv: int) -> torch.Tensor:
    """``out[t, h, :] *= sigmoid(gate[t, h])`` in place: ``out`` [tokens, heads * dv], ``gate`` [tokens, heads] (views
    with dense rows, the same type)."""
    _need(out, "out", contiguous=False)
    _need(gate, "gate", out.dtype, contiguous=False)
    if out.size(1) != n_heads * dv or gate.size(1) != n_heads or gate.size(0) != out.size(0):
        raise KernelError(f"head_gate: out {tuple(out.shape)}, gate {tuple(gate.shape)}, {n_heads} heads of {dv}")
    _check(_lib().llmrs_head_gate(_ptr(out), _LL(_row_stride(out, "out")), _ptr(gate), _LL(_row_stride(gate, "gate")),
                                  dtype_code(out.dtype), out.size(0), n_heads, dv, _stream()), "head_gate")
    return out


# -- a router that scores all experts, and experts that return their input ---------------------------------
def moe_route_biased(logits: torch.Tensor, bias: Optional[torch.Tensor], n_all: int, n_real: int, top: int):
    """Scores ``s = softmax(logits[:, :n_all])``; the ``top`` experts with the largest ``s + bias`` are chosen (the
    lower expert among equals) and weighted by ``s`` itself. Experts from ``n_real`` on are identity experts and are
    all reported as group ``n_real``. Returns (expert_of int32 [tokens * top], weight_of float32 [tokens * top]) in
    order of falling choice score."""
    _need(logits, "logits", torch.float32, contiguous=False)
    n = logits.size(0)
    if logits.size(1) < n_all or not 1 <= top <= n_all or not 0 <= n_real <= n_all:
        raise KernelError(f"moe_route_biased: logits {tuple(logits.shape)}, {n_all} experts ({n_real} real), top {top}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != n_all:
            raise KernelError(f"moe_route_biased: {bias.numel()} corrections for {n_all} experts")
    expert_of = torch.empty((n * top,), dtype=torch.int32, device=logits.device)
    weight_of = torch.empty((n * top,), dtype=torch.float32, device=logits.device)
    _check(_lib().llmrs_moe_route_biased(_ptr(logits), _LL(_row_stride(logits, "logits")), _ptr(bias), _ptr(expert_of),
                                         _ptr(weight_of), n, n_all, n_real, top, _stream()), "moe_route_biased")
    return expert_of, weight_of


def moe_combine_identity(rows: torch.Tensor, row_of: torch.Tensor, weight_of: torch.Tensor, expert_of: torch.Tensor,
                         x: torch.Tensor, top: int, n_real: int) -> torch.Tensor:
    """``moe_combine`` in which an assignment to group ``n_real`` stands for the token's own input row ``x[t]``."""
    _need(rows, "rows", torch.float32)
    _need(x, "x")
    n = row_of.numel() // top
    if x.size(0) != n or x.size(1) != rows.size(1):
        raise KernelError(f"moe_combine_identity: x {tuple(x.shape)}, rows of {rows.size(1)}, {n} tokens")
    out = torch.empty((n, rows.size(1)), dtype=torch.float32, device=rows.device)
    _check(_lib().llmrs_moe_combine_identity(_ptr(rows), _ptr(row_of), _ptr(weight_of), _ptr(expert_of), _ptr(x),
                                             dtype_code(x.dtype), _ptr(out), n, top, rows.size(1), n_real, _stream()),
           "moe_combine_identity")
    return out


# -- norms of a block that norms a branch before and after it ------------------------------------------------
def outnorm_add_norm(h: torch.Tensor, y: torch.Tensor, w_out: torch.Tensor, w_next: torch.Tensor, eps: float,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """``h += y / rms(y) * w_out`` in place (float32), and in the same pass ``h / rms(h) * w_next`` of the new rows,
    returned in ``out_dtype``: the norm on a branch's output, the residual sum and the norm ahead of the next branch."""
    _need(h, "h", torch.float32)
    _need(y, "y")
    _need(w_out, "w_out", torch.float32)
    _need(w_next, "w_next", torch.float32)
    if y.shape != h.shape or w_out.numel() != h.size(-1) or w_next.numel() != h.size(-1):
        raise KernelError(f"outnorm_add_norm: h {tuple(h.shape)}, y {tuple(y.shape)}, weights {w_out.numel()}, "
                          f"{w_next.numel()}")
    out = torch.empty(tuple(h.shape), dtype=out_dtype, device=h.device)
    _check(_lib().llmrs_outnorm_add_norm(_ptr(h), _ptr(y), dtype_code(y.dtype), _ptr(w_out), _ptr(w_next), _ptr(out),
                                         dtype_code(out_dtype), h.size(0), h.size(1), ctypes.c_float(eps), _stream()),
           "outnorm_add_norm")
    return out


OUTNORM_ADD_NORM_MAX_WIDTH = 12288


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight`` for rows of activations (a view with dense rows), float32 statistics;
    returns a contiguous tensor of the same type."""
    _need(x, "x", contiguous=False)
    _need(weight, "weight", torch.float32)
    if weight.numel() != x.size(1):
        raise KernelError(f"rmsnorm_rows: rows of {x.size(1)}, weight {weight.numel()}")
    out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    _check(_lib().llmrs_rmsnorm_rows(_ptr(x), _LL(_row_stride(x, "x")), dtype_code(x.dtype), _ptr(weight), _ptr(out),
                                     x.size(0), x.size(1), ctypes.c_float(eps), _stream()), "rmsnorm_rows")
    return out


# -- hyper-connections, the pair-table embedding, PolyNorm, the gated delta rule ----------------------------------------
HYPER_MAX_STREAMS = 16


def hyper_step(x: torch.Tensor, write=None, read=None, eps: float = 0.0, act_dtype: torch.dtype = torch.float32):
    """One pass over the streams ``x`` (float32 [tokens, streams * width], a token's streams side by side): with
    ``write`` = (y, mix, out) every stream becomes ``sum_s mix[s, t] x_s + out[t] y`` (in place; ``y`` [tokens, width]
    in float32 or the activation type, ``mix`` [streams, streams] and ``out`` [streams] float32 on the device); with
    ``read`` = (in_w, g) the normed ``u = sum_s in_w[s] x_s`` of the streams as they are AFTER the write is returned,
    ``u / sqrt(mean(u^2) + eps) * g`` with ``g`` one float32 on the device, rounded to ``act_dtype``."""
    _need(x, "x", torch.float32)
    y, mix, out = write if write is not None else (None, None, None)
    in_w, g = read if read is not None else (None, None)
    S = (mix.size(0) if mix is not None else in_w.numel())
    n, width = x.size(0), x.size(1) // S
    if x.size(1) != S * width or (y is not None and tuple(y.shape) != (n, width)):
        raise KernelError(f"hyper_step: x {tuple(x.shape)} for {S} streams, y {None if y is None else tuple(y.shape)}")
    for name, t, numel in (("mix", mix, S * S), ("out", out, S), ("in", in_w, S), ("g", g, 1)):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != numel:
                raise KernelError(f"hyper_step: {name} has {t.numel()} elements, expected {numel}")
    if y is not None:
        _need(y, "y")
    u = torch.empty((n, width), dtype=act_dtype, device=x.device) if read is not None else None
    _check(_lib().llmrs_hyper_step(_ptr(x), _ptr(y), 0 if y is None else dtype_code(y.dtype), _ptr(mix), _ptr(out),
                                   _ptr(in_w), _ptr(g), _ptr(u), dtype_code(act_dtype), n, S, width,
                                   ctypes.c_float(eps), _stream()), "hyper_step")
    return u


def hyper_leave(x: torch.Tensor, streams: int, write=None, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The sum of the streams of the given rows (int32 indices; None: all) as float32 [rows, width], taken after the
    pending ``write`` = (y, mix, out) when there is one; ``x`` is not changed."""
    _need(x, "x", torch.float32)
    y, mix, out = write if write is not None else (None, None, None)
    n, width = x.size(0), x.size(1) // streams
    n_rows = n if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if y is not None:
        _need(y, "y")
        _need(mix, "mix", torch.float32)
        _need(out, "out", torch.float32)
    total = torch.empty((n_rows, width), dtype=torch.float32, device=x.device)
    _check(_lib().llmrs_hyper_leave(_ptr(x), _ptr(y), 0 if y is None else dtype_code(y.dtype), _ptr(mix), _ptr(out),
                                    _ptr(rows), _ptr(total), n_rows, streams, width, _stream()), "hyper_leave")
    return total


def scaled_sum(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float) -> torch.Tensor:
    """``a * sa + b * sb`` in float32."""
    _need(a, "a", torch.float32)
    _need(b, "b", torch.float32)
    if a.shape != b.shape:
        raise KernelError(f"scaled_sum: {tuple(a.shape)} and {tuple(b.shape)}")
    out = torch.empty_like(a)
    _check(_lib().llmrs_scaled_sum(_ptr(a), _ptr(b), _ptr(out), _LL(a.numel()), ctypes.c_float(sa), ctypes.c_float(sb),
                                   _stream()), "scaled_sum")
    return out


def bigram_embedding(table: torch.Tensor, pairs: Optional[torch.Tensor], ctx, prev_state: Optional[torch.Tensor],
                     copies: int, scale: float, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """``table[id] * scale + pairs[(previous id * mul_prev + id * mul_cur) mod buckets]`` (row ``buckets`` for a
    sequence's first token) as float32 [tokens, copies * hidden], the same row ``copies`` times. ``prev_state``
    (float32 [slots, 1]) keeps every request's last token between steps. ``pairs`` None: the scaled table alone."""
    _need(table, "table")
    vocab, hidden = table.shape
    n = ctx.token_ids.numel()
    if pairs is not None:
        _need(pairs, "pairs", table.dtype)
        _need(prev_state, "prev_state", torch.float32)
        if tuple(pairs.shape) != (buckets + 1, hidden):
            raise KernelError(f"bigram_embedding: the pair table is {tuple(pairs.shape)}, expected {(buckets + 1, hidden)}")
    out = torch.empty((n, copies * hidden), dtype=torch.float32, device=table.device)
    _check(_lib().llmrs_bigram_embedding(
        _ptr(table), _ptr(pairs), dtype_code(table.dtype), _ptr(ctx.token_ids), _ptr(ctx.token_req), _ptr(ctx.q_start),
        _ptr(ctx.n_new), _ptr(ctx.cached_len), _ptr(ctx.slot_ids), _ptr(prev_state), _ptr(out), n, hidden, vocab,
        copies, ctypes.c_float(scale), buckets, _LL(mul_prev), _LL(mul_cur), _stream()), "bigram_embedding")
    return out


def poly_norm(z: torch.Tensor, coeff: torch.Tensor, eps: float) -> torch.Tensor:
    """``a N(z) + b N(z^2) + c N(z^3) + e`` row by row, N the division by the root mean square; ``coeff`` float32 [4]."""
    _need(z, "z")
    _need(coeff, "coeff", torch.float32)
    if z.dim() != 2 or coeff.numel() != 4:
        raise KernelError(f"poly_norm: z {tuple(z.shape)}, {coeff.numel()} coefficients")
    out = torch.empty_like(z)
    _check(_lib().llmrs_poly_norm(_ptr(z), _ptr(coeff), _ptr(out), z.size(0), z.size(1), ctypes.c_float(eps),
                                  dtype_code(z.dtype), _stream()), "poly_norm")
    return out


GD_CHUNKED = os.environ.get("LLMRS_GD_CHUNKED", "0") == "1"
_gd_chunked_set = None


def gated_delta_chunked(on: bool) -> None:
    """True: portions of 64 tokens and more take the gated delta rule in chunks of 32 tokens (five small float32 products
    per chunk) instead of token by token; the same numbers up to rounding. Off unless ``LLMRS_GD_CHUNKED=1``: the
    chunked kernel is bound by shared-memory reads and not ahead of the walk yet."""
    global _gd_chunked_set
    fn = _lib().llmrs_gated_delta_chunked
    fn.restype, fn.argtypes = None, [ctypes.c_int]
    fn(1 if on else 0)
    _gd_chunked_set = bool(on)


def gated_delta(x: torch.Tensor, gate: torch.Tensor, taps: torch.Tensor, ba: torch.Tensor, a_log: torch.Tensor,
                dt_bias: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, conv_state: torch.Tensor, ctx,
                n_kv_heads: int, n_heads: int, dk: int, dv: int, key_eps: float, q_scale: float, norm_eps: float,
                out: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
    """The gated delta rule of ``csrc/gated_delta.cu`` over a step's tokens. ``x``: the q | k | v channels that enter
    the short convolutions, a column slice with dense rows; ``gate``: [tokens, heads * dv] likewise; ``taps`` float32
    [channels, K]; ``ba`` float32 [tokens, 2 * heads] (write strength, then decay projection); ``state`` float32
    [slots, heads, dk, dv] and ``conv_state`` float32 [slots, K - 1, channels], both updated in place. Returns
    [tokens, heads * dv] in the activation type (``out``: a view to write into), multiplied by ``out_scale``."""
    C = 2 * n_kv_heads * dk + n_heads * dv
    K = taps.size(1)
    if _gd_chunked_set is None:
        gated_delta_chunked(GD_CHUNKED)
    _need(x, "x", contiguous=False)
    _need(gate, "gate", x.dtype, contiguous=False)
    for name, t in (("taps", taps), ("ba", ba), ("a_log", a_log), ("dt_bias", dt_bias), ("norm_w", norm_w),
                    ("state", state), ("conv_state", conv_state)):
        _need(t, name, torch.float32)
    n = x.size(0)
    if x.size(1) != C or tuple(taps.shape) != (C, K) or tuple(ba.shape) != (n, 2 * n_heads) or \
            tuple(state.shape[1:]) != (n_heads, dk, dv) or tuple(conv_state.shape[1:]) != (max(K - 1, 0), C) or \
            gate.size(1) != n_heads * dv or norm_w.numel() != dv:
        raise KernelError(f"gated_delta: x {tuple(x.shape)}, taps {tuple(taps.shape)}, ba {tuple(ba.shape)}, state "
                          f"{tuple(state.shape)}, conv_state {tuple(conv_state.shape)}, gate {tuple(gate.shape)}")
    if out is None:
        out = torch.empty((n, n_heads * dv), dtype=x.dtype, device=x.device)
    _need(out, "out", x.dtype, contiguous=False)
    work = torch.empty((int(_lib_ll("llmrs_gated_delta_work_floats")(n, ctx.n_requests, n_kv_heads, n_heads, dk, dv)),),
                       dtype=torch.float32, device=x.device)
    _check(_lib().llmrs_gated_delta(
        _ptr(x), _LL(_row_stride(x, "x")), _ptr(gate), _LL(_row_stride(gate, "gate")), dtype_code(x.dtype), _ptr(taps),
        _ptr(ba), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w), _ptr(state), _ptr(conv_state), _ptr(ctx.token_req),
        _ptr(ctx.q_start), _ptr(ctx.n_new), _ptr(ctx.slot_ids), _ptr(work), _ptr(out), _LL(_row_stride(out, "out")), n,
        ctx.n_requests, n_kv_heads, n_heads, dk, dv, K, ctypes.c_float(key_eps), ctypes.c_float(q_scale),
        ctypes.c_float(norm_eps), ctypes.c_float(out_scale), _stream()), "gated_delta", 4)
    return out
