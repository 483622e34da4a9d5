"""Python faces of the CUDA entry points: argument checks, pointers, the current stream.

Each function takes CUDA tensors, checks what the kernel assumes (device, dtype, contiguity of
the innermost dimension), passes raw pointers to the ``extern "C"`` symbol and raises
:class:`KernelError` when the entry point refuses or the launch fails. There is no fallback
to torch ops here: a missing extension is an error.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library

TS_F32, TS_BF16 = 0, 1
_ERRORS = {
    -1: "dtype not supported by this kernel",
    -2: "a size this kernel does not take",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "an argument was refused",
}

ACTIVATION_CODES = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "clamped_swish": 3}


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or its launch failed."""


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return TS_F32
    if dtype == torch.bfloat16:
        return TS_BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


_launches = 0


def launch_count() -> int:
    """How many kernels of this package have been launched so far in this process."""
    return _launches


def _check(code: int, name: str, launches: int = 1) -> None:
    """Raise for a refused call; else count the ``launches`` kernels the entry point started."""
    global _launches
    if code == 0:
        _launches += launches
        return
    if code in _ERRORS:
        raise KernelError(f"{name}: {_ERRORS[code]}")
    raise KernelError(f"{name}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream of the current device as a raw handle (asked of torch's C layer directly where
    it offers that: ``torch.cuda.current_stream()`` costs several microseconds of Python per launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() and t.stride(-1) != 1:
        raise KernelError(f"{name} must be contiguous in its last dimension")


_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(lib: str, symbol: str, argtypes: list, restype=c_int):
    fn = _functions.get(symbol)
    if fn is None:
        fn = getattr(load_library(lib), symbol)
        fn.argtypes = argtypes
        fn.restype = restype
        _functions[symbol] = fn
    return fn


# ---------------------------------------------------------------------------------------
# layer_ops.cu
# ---------------------------------------------------------------------------------------


def embedding(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """``residual[t] = float(table[ids[t]])``; ids int32 [T], residual fp32 [T, H]."""
    _need(ids, torch.int32, "ids"); _need(table, None, "table"); _need(residual, torch.float32, "residual")
    num_tokens, hidden = ids.numel(), table.shape[1]
    if residual.shape[-1] != hidden or residual.shape[0] < num_tokens or not residual.is_contiguous() or not table.is_contiguous():
        raise KernelError("embedding: residual must be contiguous [tokens, hidden]")
    fn = _fn("layer_ops", "ts_embedding", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(table.dtype), _ptr(ids), _ptr(table), _ptr(residual), num_tokens, hidden, table.shape[0], _ptr(status), _stream()), "embedding")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, num_rows: int | None = None) -> None:
    """Fused ``residual += delta`` and RMSNorm into ``out`` (see ``layer_ops.cu``)."""
    _need(residual, torch.float32, "residual"); _need(gain, torch.float32, "gain"); _need(out, None, "out")
    hidden = residual.shape[-1]
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if not delta.is_contiguous() or delta.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta must be contiguous [rows, hidden]")
    if not residual.is_contiguous() or not out.is_contiguous() or out.shape[-1] != hidden or gain.numel() != hidden:
        raise KernelError("add_rmsnorm: shapes do not agree")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        n = rows.numel() if num_rows is None else num_rows
    else:
        n = residual.shape[0] if num_rows is None else num_rows
    if out.shape[0] < n:
        raise KernelError("add_rmsnorm: out has too few rows")
    fn = _fn("layer_ops", "ts_add_rmsnorm", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(residual), _ptr(delta), _ptr(gain), _ptr(out), _ptr(rows), n, hidden, float(eps), _stream()), "add_rmsnorm")


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str, num_tokens: int | None = None,
            block: int = 0, limit: float = 0.0, alpha: float = 0.0) -> None:
    """``out[t, i] = act(gate[t, i]) * up[t, i]`` in fp32, rounded once; with ``clamped_swish``
    ``g sigmoid(alpha g) (u + 1)`` for ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``.

    ``block == 0``: a row of ``gate_up`` is ``[gate | up]``. ``block > 0``: gate and up alternate
    in runs of ``block`` features (``[g 0..b-1 | u 0..b-1 | g b..2b-1 | ...]``).
    """
    _need(gate_up, None, "gate_up"); _need(out, gate_up.dtype, "out")
    inter = out.shape[-1]
    if gate_up.shape[-1] != 2 * inter or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("act_mul: gate_up must be contiguous [tokens, 2 * intermediate]")
    if activation not in ACTIVATION_CODES:
        raise KernelError(f"act_mul: unknown activation {activation!r}")
    n = gate_up.shape[0] if num_tokens is None else num_tokens
    fn = _fn("layer_ops", "ts_act_mul", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(gate_up), _ptr(out), n, inter, ACTIVATION_CODES[activation], int(block),
              float(limit), float(alpha), _stream()), "act_mul")


def rope_cache_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                     block_table: torch.Tensor, k_pages: torch.Tensor | None, v_pages: torch.Tensor | None,
                     num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                     inv_freq: torch.Tensor | None, rotary_dim: int, factor: float, write_kv: bool,
                     status: torch.Tensor | None = None) -> None:
    """Bias, rotary encoding of q and k in fp32, and append of k, v to the paged cache."""
    _need(qkv, None, "qkv"); _need(positions, torch.int32, "positions"); _need(seq_of_token, torch.int32, "seq_of_token")
    _need(block_table, torch.int32, "block_table")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.dim() != 2 or qkv.shape[1] < width:
        raise KernelError("rope_cache_write: qkv is narrower than its heads")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != width:
            raise KernelError("rope_cache_write: bias length does not match the projected heads")
    page_size = 1
    if write_kv:
        if k_pages is None or v_pages is None:
            raise KernelError("rope_cache_write: pages are needed to write keys and values")
        _need(k_pages, qkv.dtype, "k_pages"); _need(v_pages, qkv.dtype, "v_pages")
        if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim):
            raise KernelError("rope_cache_write: pages must be contiguous [pages, page_size, kv_heads, head_dim]")
        page_size = k_pages.shape[1]
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_cache_write: inv_freq must hold rotary_dim / 2 values")
    fn = _fn("layer_ops", "ts_rope_cache_write",
             [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
              c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(positions), _ptr(seq_of_token),
              _ptr(block_table), block_table.stride(0), _ptr(k_pages), _ptr(v_pages), page_size, num_tokens,
              num_heads, num_kv_heads, head_dim, _ptr(inv_freq), rotary_dim, float(factor), int(write_kv),
              _ptr(status), _stream()), "rope_cache_write")


def head_norm_rope_write(qkv: torch.Tensor, q_gain: torch.Tensor | None, k_gain: torch.Tensor | None, eps: float,
                         positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                         k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, num_tokens: int, num_heads: int,
                         num_kv_heads: int, dim: int, vdim: int, inv_freq: torch.Tensor | None, rotary_dim: int,
                         interleaved: bool, write_kv: bool, status: torch.Tensor | None = None,
                         bias: torch.Tensor | None = None) -> None:
    """The projection's ``bias`` (float32, as wide as a row's heads, or ``None``), RMS norm per head of q and k (gains of
    ``dim`` floats shared by the heads, or ``None``), rotation of the first
    ``rotary_dim`` elements (pairs ``(2i, 2i + 1)`` when ``interleaved``, else ``(i, i + rotary_dim / 2)``), and the
    append of keys (``dim`` wide) and values (``vdim`` wide) to their pages; all in fp32, rounded once.

    ``qkv`` rows are ``[num_heads * dim | num_kv_heads * dim | num_kv_heads * vdim]``; queries are changed in place."""
    _need(qkv, None, "qkv"); _need(positions, torch.int32, "positions"); _need(seq_of_token, torch.int32, "seq_of_token")
    _need(block_table, torch.int32, "block_table")
    if qkv.dim() != 2 or qkv.shape[1] < (num_heads + num_kv_heads) * dim + num_kv_heads * vdim:
        raise KernelError("head_norm_rope_write: qkv is narrower than its heads")
    for name, gain in (("q_gain", q_gain), ("k_gain", k_gain)):
        if gain is not None:
            _need(gain, torch.float32, name)
            if gain.numel() != dim:
                raise KernelError(f"head_norm_rope_write: {name} must hold dim floats")
    page_size = 1
    if write_kv:
        if k_pages is None or v_pages is None:
            raise KernelError("head_norm_rope_write: pages are needed to write keys and values")
        _need(k_pages, qkv.dtype, "k_pages"); _need(v_pages, qkv.dtype, "v_pages")
        if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, dim)
                or tuple(v_pages.shape[2:]) != (num_kv_heads, vdim) or k_pages.shape[1] != v_pages.shape[1]):
            raise KernelError("head_norm_rope_write: pages must be contiguous [pages, page_size, kv_heads, dim | vdim]")
        page_size = k_pages.shape[1]
    if rotary_dim:
        if inv_freq is None:
            raise KernelError("head_norm_rope_write: a rotation needs its frequencies")
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("head_norm_rope_write: inv_freq must hold rotary_dim / 2 values")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != (num_heads + num_kv_heads) * dim + num_kv_heads * vdim or not bias.is_contiguous():
            raise KernelError("head_norm_rope_write: the bias must be as wide as a row's heads")
    fn = _fn("layer_ops", "ts_head_norm_rope_write",
             [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(q_gain), _ptr(k_gain), float(eps), _ptr(positions),
              _ptr(seq_of_token), _ptr(block_table), block_table.stride(0), _ptr(k_pages), _ptr(v_pages), page_size,
              num_tokens, num_heads, num_kv_heads, dim, vdim, _ptr(inv_freq), int(rotary_dim), 1 if interleaved else 0,
              1 if write_kv else 0, _ptr(status), _stream()), "head_norm_rope_write")


# ---------------------------------------------------------------------------------------
# attention_generic.cu
# ---------------------------------------------------------------------------------------


def paged_attention_generic(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                            num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                            window: int | None, scale: float, status: torch.Tensor | None = None) -> None:
    """Attention of every token over its sequence's pages; any dtype and head size <= 256.

    ``q`` is ``[tokens, >= num_heads * head_dim]`` (it may be the fused qkv buffer), ``out``
    ``[tokens, num_heads * head_dim]``.
    """
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(k_pages, q.dtype, "k_pages"); _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"); _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim):
        raise KernelError("paged_attention: pages must be contiguous [pages, page_size, kv_heads, head_dim]")
    if q.shape[1] < num_heads * head_dim or out.shape[1] < num_heads * head_dim:
        raise KernelError("paged_attention: q or out is narrower than its heads")
    fn = _fn("attention_generic", "ts_paged_attention_generic",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
              _ptr(block_table), block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens,
              k_pages.shape[1], num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), _ptr(status),
              _stream()), "paged_attention_generic")


def paged_attention_capped(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                           num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int,
                           window: int | None, scale: float, softcap: float = 0.0, sink: bool = False,
                           status: torch.Tensor | None = None, sink_values: torch.Tensor | None = None) -> None:
    """:func:`paged_attention_generic` with every option: value rows of ``v_dim`` elements, scores capped as
    ``softcap * tanh(score / softcap)`` (0: uncapped), and a ``sink`` (one more term in the softmax's denominator, as if
    one more key had no value; it scores 0, or ``sink_values[head]`` (float32, one a query head), taken as it is).
    ``out`` is ``[tokens, >= num_heads * v_dim]``."""
    _need_sink(sink, sink_values, num_heads)
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(k_pages, q.dtype, "k_pages"); _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"); _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim)
            or tuple(v_pages.shape[2:]) != (num_kv_heads, v_dim) or k_pages.shape[1] != v_pages.shape[1]):
        raise KernelError("paged_attention: pages must be contiguous [pages, page_size, kv_heads, head_dim | v_dim]")
    if q.shape[1] < num_heads * head_dim or out.shape[1] < num_heads * v_dim:
        raise KernelError("paged_attention: q or out is narrower than its heads")
    fn = _fn("attention_generic", "ts_paged_attention_capped",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
              _ptr(block_table), block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens,
              k_pages.shape[1], num_heads, num_kv_heads, head_dim, v_dim, int(window or 0), float(scale), float(softcap),
              1 if sink else 0, _ptr(sink_values), _ptr(status), _stream()), "paged_attention_capped")


def _need_sink(sink: bool, sink_values: torch.Tensor | None, num_heads: int) -> None:
    if sink_values is None:
        return
    _need(sink_values, torch.float32, "sink_values")
    if not sink or sink_values.numel() != num_heads or not sink_values.is_contiguous():
        raise KernelError("attention: sink_values must hold one float per query head, and go with a sink")


def paged_attention_capped_mma_takes(dtype: torch.dtype, dim: int, vdim: int, scale: float = 1.0) -> bool:
    """Whether the tensor-core kernel for portions of prompts takes these sizes (else the kernel for every size runs)."""
    return (dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 256 and 16 <= vdim <= 128
            and scale > 0.0)


def paged_attention_capped_mma(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                               block_table: torch.Tensor, query_start: torch.Tensor, context_lens: torch.Tensor,
                               num_tokens: int, num_seqs: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int,
                               window: int | None, scale: float, softcap: float = 0.0, sink: bool = False,
                               status: torch.Tensor | None = None, sink_values: torch.Tensor | None = None) -> None:
    """:func:`paged_attention_capped` for bfloat16 steps with portions of prompts, on tensor cores: tiles of 64
    positions of a request, found through ``query_start`` and ``context_lens`` (``[seqs + 1]`` and ``[seqs]``)."""
    for name, tensor in (("q", q), ("out", out), ("k_pages", k_pages), ("v_pages", v_pages)):
        _need(tensor, torch.bfloat16, name)
    _need(block_table, torch.int32, "block_table"); _need(query_start, torch.int32, "query_start"); _need(context_lens, torch.int32, "context_lens")
    if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim)
            or tuple(v_pages.shape[2:]) != (num_kv_heads, v_dim) or k_pages.shape[1] != v_pages.shape[1]):
        raise KernelError("paged_attention_capped_mma: pages must be contiguous [pages, page_size, kv_heads, head_dim | v_dim]")
    if q.shape[1] < num_heads * head_dim or out.shape[1] < num_heads * v_dim:
        raise KernelError("paged_attention_capped_mma: q or out is narrower than its heads")
    if query_start.numel() < num_seqs + 1 or context_lens.numel() < num_seqs:
        raise KernelError("paged_attention_capped_mma: fewer requests than asked for")
    fn = _fn("attention_capped_mma", "ts_paged_attention_capped_mma",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _need_sink(sink, sink_values, num_heads)
    _check(fn(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
              block_table.stride(0), _ptr(query_start), _ptr(context_lens), num_tokens, num_seqs, k_pages.shape[1],
              num_heads, num_kv_heads, head_dim, v_dim, int(window or 0), float(scale), float(softcap), 1 if sink else 0,
              _ptr(sink_values), _ptr(status), _stream()), "paged_attention_capped_mma")


# ---------------------------------------------------------------------------------------
# stream_ops.cu
# ---------------------------------------------------------------------------------------

PLAIN_ACTIVATION_CODES = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "tanh": 3}


def stream_norm(residual: torch.Tensor, deltas: tuple, shift: torch.Tensor | None, gain1: torch.Tensor | None,
                out1: torch.Tensor | None, gain2: torch.Tensor | None = None, out2: torch.Tensor | None = None,
                eps: float = 0.0, rows: torch.Tensor | None = None, num_rows: int | None = None,
                dtype: torch.dtype | None = None, mult: float = 1.0) -> None:
    """``x = residual + deltas[0] + deltas[1] + shift`` in fp32 (each optional), written back unless
    ``rows`` selects rows; then ``out1 = x / rms(x) * gain1`` and, if given, ``out2 = x / rms(x) * gain2``.
    With ``out1`` ``None`` only the sum is made (``dtype`` then names the deltas' type). With ``mult``
    other than 1 the sum is ``residual + mult * (deltas[0] + deltas[1]) + shift``."""
    _need(residual, torch.float32, "residual")
    hidden = residual.shape[-1]
    kind = out1.dtype if out1 is not None else (deltas[0].dtype if deltas else (dtype or torch.float32))
    if len(deltas) > 2:
        raise KernelError("stream_norm: at most two updates")
    for d in deltas:
        _need(d, kind, "delta")
        if not d.is_contiguous() or d.shape[-1] != hidden:
            raise KernelError("stream_norm: an update must be contiguous [rows, hidden]")
    if shift is not None:
        _need(shift, torch.float32, "shift")
        if shift.numel() != hidden or not shift.is_contiguous():
            raise KernelError("stream_norm: shift must hold hidden floats")
    for g, o, name in ((gain1, out1, "1"), (gain2, out2, "2")):
        if (g is None) != (o is None):
            raise KernelError("stream_norm: a gain goes with an output")
        if g is not None:
            _need(g, torch.float32, "gain" + name); _need(o, kind, "out" + name)
            if g.numel() != hidden or not o.is_contiguous() or o.shape[-1] != hidden:
                raise KernelError("stream_norm: shapes do not agree")
    if not residual.is_contiguous():
        raise KernelError("stream_norm: residual must be contiguous")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        n = rows.numel() if num_rows is None else num_rows
    else:
        n = residual.shape[0] if num_rows is None else num_rows
    for o in (out1, out2):
        if o is not None and o.shape[0] < n:
            raise KernelError("stream_norm: an output has too few rows")
    da = deltas[0] if len(deltas) > 0 else None
    db = deltas[1] if len(deltas) > 1 else None
    fn = _fn("stream_ops", "ts_stream_norm", [c_int] + [c_void_p] * 9 + [c_int, c_int, c_float, c_float, c_void_p])
    _check(fn(dtype_code(kind), _ptr(residual), _ptr(da), _ptr(db), _ptr(shift), _ptr(gain1), _ptr(out1), _ptr(gain2),
              _ptr(out2), _ptr(rows), n, hidden, float(eps), float(mult), _stream()), "stream_norm")


def norm_pair_mix(a: torch.Tensor, b: torch.Tensor, gain_a: torch.Tensor, gain_b: torch.Tensor, out: torch.Tensor,
                  num_rows: int, eps: float, weight_a: float = 0.5, weight_b: float = 0.5) -> None:
    """``out = weight_a * (a / rms(a) * gain_a) + weight_b * (b / rms(b) * gain_b)``: each input normed over its whole
    row on its own (``eps`` inside the root), in fp32, rounded once."""
    _need(a, None, "a"); _need(b, a.dtype, "b"); _need(out, a.dtype, "out")
    _need(gain_a, torch.float32, "gain_a"); _need(gain_b, torch.float32, "gain_b")
    hidden = a.shape[-1]
    if (not a.is_contiguous() or not b.is_contiguous() or not out.is_contiguous() or b.shape[-1] != hidden or out.shape[-1] != hidden
            or gain_a.numel() != hidden or gain_b.numel() != hidden or min(a.shape[0], b.shape[0], out.shape[0]) < num_rows):
        raise KernelError("norm_pair_mix: shapes do not agree")
    fn = _fn("stream_ops", "ts_norm_pair_mix",
             [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(fn(dtype_code(a.dtype), _ptr(a), _ptr(b), _ptr(gain_a), _ptr(gain_b), _ptr(out), num_rows, hidden, float(eps),
              float(weight_a), float(weight_b), _stream()), "norm_pair_mix")


def shift_mix(x: torch.Tensor, mu: torch.Tensor, last: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
              seq_of_token: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor, num_tokens: int, num_seqs: int) -> None:
    """``out[t, s] = x[t] + (x[t - 1] - x[t]) * mu[s]`` for every row ``s`` of ``mu`` (float32 ``[mixes, hidden]``), side by
    side in ``out`` ``[tokens, mixes * hidden]``. The row before a step's first token of a request is what ``last``
    (``[slots, hidden]``, the activation type) kept; before position 0 it is zeros. ``last`` then takes every
    request's last row of this step."""
    _need(x, None, "x"); _need(out, x.dtype, "out"); _need(last, x.dtype, "last"); _need(mu, torch.float32, "mu")
    for name, tensor in (("positions", positions), ("seq_of_token", seq_of_token), ("query_start", query_start), ("slots", slots)):
        _need(tensor, torch.int32, name)
    hidden = x.shape[-1]
    mixes = mu.shape[0]
    if (not x.is_contiguous() or not out.is_contiguous() or not last.is_contiguous() or not mu.is_contiguous() or mu.dim() != 2
            or mu.shape[1] != hidden or out.shape[-1] != mixes * hidden or last.shape[-1] != hidden
            or min(x.shape[0], out.shape[0], positions.numel(), seq_of_token.numel()) < num_tokens
            or query_start.numel() < num_seqs + 1 or slots.numel() < num_seqs):
        raise KernelError("shift_mix: shapes do not agree")
    fn = _fn("stream_ops", "ts_shift_mix", [c_int] + [c_void_p] * 8 + [c_int] * 4 + [c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), _ptr(mu), _ptr(last), _ptr(out), _ptr(positions), _ptr(seq_of_token),
              _ptr(query_start), _ptr(slots), num_tokens, num_seqs, hidden, mixes, _stream()), "shift_mix", launches=2)


def norm_add(residual: torch.Tensor, update: torch.Tensor | None, gain: torch.Tensor | None, copy: torch.Tensor | None,
             eps: float, mult: float, num_rows: int, dtype: torch.dtype | None = None) -> None:
    """``residual += mult * rms_norm(update) * gain`` in fp32 (the norm on a sublayer's output), and
    ``copy = residual`` in the activation type; without ``update`` only the copy is made."""
    _need(residual, torch.float32, "residual")
    hidden = residual.shape[-1]
    kind = update.dtype if update is not None else (copy.dtype if copy is not None else (dtype or torch.float32))
    for name, tensor in (("update", update), ("copy", copy)):
        if tensor is not None:
            _need(tensor, kind, name)
            if not tensor.is_contiguous() or tensor.shape[-1] != hidden or tensor.shape[0] < num_rows:
                raise KernelError(f"norm_add: {name} must be contiguous [rows, hidden]")
    if update is not None:
        if gain is None:
            raise KernelError("norm_add: an update goes with a gain")
        _need(gain, torch.float32, "gain")
        if gain.numel() != hidden:
            raise KernelError("norm_add: gain must hold hidden floats")
    if not residual.is_contiguous() or residual.shape[0] < num_rows:
        raise KernelError("norm_add: residual must be contiguous [rows, hidden]")
    fn = _fn("stream_ops", "ts_norm_add", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p])
    _check(fn(dtype_code(kind), _ptr(residual), _ptr(update), _ptr(gain), _ptr(copy), num_rows, hidden, float(eps),
              float(mult), _stream()), "norm_add")


def norm_add_norm(residual: torch.Tensor, update: torch.Tensor | None, gain_post: torch.Tensor | None, eps_post: float,
                  extra: torch.Tensor | None, gain_pre: torch.Tensor | None, eps_pre: float, out: torch.Tensor | None,
                  num_rows: int, dtype: torch.dtype | None = None, rows: torch.Tensor | None = None) -> None:
    """``residual += rms_norm(update) * gain_post`` (the norm taken over the update alone), ``residual += extra`` (float32
    rows), ``out = rms_norm(residual) * gain_pre``; every part optional, all in float32, ``out`` rounded once. With
    ``rows`` (int32) only the listed rows are worked and ``residual`` is not written. ``dtype`` names the activation
    type when neither ``update`` nor ``out`` is given."""
    _need(residual, torch.float32, "residual")
    hidden = residual.shape[-1]
    kind = update.dtype if update is not None else (out.dtype if out is not None else (dtype or torch.float32))
    if not residual.is_contiguous():
        raise KernelError("norm_add_norm: the residual must be contiguous")
    if update is not None:
        _need(update, kind, "update"); _need(gain_post, torch.float32, "gain_post")
        if not update.is_contiguous() or update.shape[-1] != hidden or gain_post.numel() != hidden:
            raise KernelError("norm_add_norm: the update and its gain must be as wide as the residual")
    if extra is not None:
        _need(extra, torch.float32, "extra")
        if not extra.is_contiguous() or extra.shape[-1] != hidden:
            raise KernelError("norm_add_norm: the added rows must be contiguous float32 rows as wide as the residual")
    if out is not None:
        _need(out, kind, "out"); _need(gain_pre, torch.float32, "gain_pre")
        if not out.is_contiguous() or out.shape[-1] != hidden or gain_pre.numel() != hidden or out.shape[0] < num_rows:
            raise KernelError("norm_add_norm: out and its gain must be as wide as the residual")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn("stream_ops", "ts_norm_add_norm", [c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_void_p,
                                                c_void_p, c_int, c_int, c_void_p])
    _check(fn(dtype_code(kind), _ptr(residual), _ptr(update), _ptr(gain_post), float(eps_post), _ptr(extra), _ptr(gain_pre),
              float(eps_pre), _ptr(out), _ptr(rows), int(num_rows), hidden, _stream()), "norm_add_norm")


def softcap_rows(data: torch.Tensor, cap: float, num_rows: int | None = None) -> None:
    """``data[:num_rows] = cap * tanh(data[:num_rows] / cap)`` in place; float32 rows."""
    _need(data, torch.float32, "data")
    if not data.is_contiguous():
        raise KernelError("softcap_rows: data must be contiguous")
    rows = data.shape[0] if num_rows is None else num_rows
    fn = _fn("stream_ops", "ts_softcap_rows", [c_void_p, c_longlong, c_float, c_void_p])
    _check(fn(_ptr(data), rows * (data.numel() // max(data.shape[0], 1)), float(cap), _stream()), "softcap_rows")


def activation(x: torch.Tensor, out: torch.Tensor, name: str, num_rows: int | None = None) -> None:
    """``out = act(x)`` for contiguous rows; ``relu2`` (the square of relu), ``gelu_tanh``, ``silu`` or ``tanh``."""
    _need(x, None, "x"); _need(out, x.dtype, "out")
    if name not in PLAIN_ACTIVATION_CODES:
        raise KernelError(f"activation: unknown activation {name!r}")
    if not x.is_contiguous() or not out.is_contiguous() or x.shape[-1] != out.shape[-1]:
        raise KernelError("activation: contiguous rows of one width are needed")
    n = x.shape[0] if num_rows is None else num_rows
    fn = _fn("stream_ops", "ts_activation", [c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), _ptr(out), n * x.shape[-1], PLAIN_ACTIVATION_CODES[name], _stream()), "activation")


def scale_rows(data: torch.Tensor, factor: float, num_rows: int | None = None) -> None:
    """``data[:rows] *= factor`` for contiguous float32 rows."""
    _need(data, torch.float32, "data")
    if not data.is_contiguous():
        raise KernelError("scale_rows: data must be contiguous")
    n = data.shape[0] if num_rows is None else num_rows
    fn = _fn("stream_ops", "ts_scale_rows", [c_void_p, c_longlong, c_float, c_void_p])
    _check(fn(_ptr(data), n * data.shape[-1], float(factor), _stream()), "scale_rows")


# ---------------------------------------------------------------------------------------
# conv_ops.cu
# ---------------------------------------------------------------------------------------


def causal_conv(x: torch.Tensor, first: int, weight: torch.Tensor, bias: torch.Tensor | None, tail: torch.Tensor,
                out: torch.Tensor, seq_of_token: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor,
                num_tokens: int, num_seqs: int, silu: bool = False, append: dict | None = None,
                status: torch.Tensor | None = None) -> None:
    """Short causal convolution per channel over columns ``[first, first + C)`` of ``x`` into ``out[:, :C]``.

    ``weight`` is float32 ``[C, taps]`` (the last tap multiplies the current position), ``tail``
    ``[slots, taps - 1, C]`` holds every request's last inputs and is brought up to date.
    ``append`` (``k_pages``, ``v_pages``, ``block_table``, ``positions``, ``k_first``, ``k_width``,
    ``v_first``, ``v_width``) also writes two ranges of the output channels to paged caches whose
    rows are ``[pages, page_size, k_width]`` and ``[pages, page_size, v_width]``.
    """
    _need(x, None, "x"); _need(out, x.dtype, "out"); _need(tail, x.dtype, "tail"); _need(weight, torch.float32, "weight")
    for name, tensor in (("seq_of_token", seq_of_token), ("query_start", query_start), ("slots", slots)):
        _need(tensor, torch.int32, name)
    channels, taps = weight.shape
    if not weight.is_contiguous() or x.dim() != 2 or out.dim() != 2 or x.shape[1] < first + channels or out.shape[1] < channels:
        raise KernelError("causal_conv: the matrices are narrower than the channels")
    if tail.dim() != 3 or not tail.is_contiguous() or tuple(tail.shape[1:]) != (taps - 1, channels):
        raise KernelError("causal_conv: tail must be contiguous [slots, taps - 1, channels]")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != channels:
            raise KernelError("causal_conv: bias length does not match the channels")
    if x.shape[0] < num_tokens or out.shape[0] < num_tokens or query_start.numel() < num_seqs + 1 or slots.numel() < num_seqs:
        raise KernelError("causal_conv: fewer rows than asked for")
    k_pages = v_pages = table = positions = None
    table_stride = page_size = k_first = k_width = v_first = v_width = 0
    if append is not None:
        k_pages, v_pages, table, positions = append["k_pages"], append["v_pages"], append["block_table"], append["positions"]
        _need(k_pages, x.dtype, "k_pages"); _need(v_pages, x.dtype, "v_pages")
        _need(table, torch.int32, "block_table"); _need(positions, torch.int32, "positions")
        k_first, k_width, v_first, v_width = (int(append[k]) for k in ("k_first", "k_width", "v_first", "v_width"))
        page_size, table_stride = k_pages.shape[1], table.stride(0)
        if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or k_pages[0, 0].numel() != k_width
                or v_pages[0, 0].numel() != v_width or v_pages.shape[1] != page_size):
            raise KernelError("causal_conv: the pages' rows do not match the widths to append")
    fn = _fn("conv_ops", "ts_causal_conv",
             [c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
              c_int, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), x.stride(0), int(first), _ptr(weight), _ptr(bias), _ptr(tail), _ptr(out),
              out.stride(0), _ptr(seq_of_token), _ptr(query_start), _ptr(slots), num_tokens, num_seqs, channels, taps,
              1 if silu else 0, _ptr(k_pages), _ptr(v_pages), _ptr(table), table_stride, _ptr(positions), page_size,
              k_first, k_width, v_first, v_width, _ptr(status), _stream()), "causal_conv", launches=2 if taps > 1 else 1)


# ---------------------------------------------------------------------------------------
# diff_attention.cu
# ---------------------------------------------------------------------------------------


def diff_attention(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                   block_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor, num_tokens: int,
                   num_heads: int, num_kv_heads: int, dim: int, vdim: int, window: int | None, scale: float,
                   lam: float, eps: float, out_scale: float, status: torch.Tensor | None = None) -> None:
    """Two softmax maps per head over one set of values, ``a1 - lam * a2``, unit RMS per head, times ``out_scale``.

    ``q`` is ``[tokens, >= heads * 2 * dim]``, ``out`` ``[tokens, >= heads * vdim]``, the pages
    ``[pages, page_size, kv_heads, 2 * dim]`` and ``[pages, page_size, kv_heads, vdim]``.
    """
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(k_pages, q.dtype, "k_pages"); _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"); _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, 2 * dim)
            or tuple(v_pages.shape[2:]) != (num_kv_heads, vdim) or k_pages.shape[1] != v_pages.shape[1]):
        raise KernelError("diff_attention: pages must be contiguous [pages, page_size, kv_heads, 2 * dim | vdim]")
    if q.shape[1] < num_heads * 2 * dim or out.shape[1] < num_heads * vdim:
        raise KernelError("diff_attention: q or out is narrower than its heads")
    fn = _fn("diff_attention", "ts_diff_attention",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_void_p, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
              _ptr(block_table), block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens,
              k_pages.shape[1], num_heads, num_kv_heads, dim, vdim, int(window or 0), float(scale), float(lam),
              float(eps), float(out_scale), _ptr(status), _stream()), "diff_attention")


def diff_attention_mma_takes(dtype: torch.dtype, dim: int, vdim: int, scale: float = 1.0) -> bool:
    """Whether the tensor-core kernel for portions of prompts takes these sizes (else the kernel for every size runs)."""
    return (dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128
            and scale > 0.0)


def diff_attention_mma(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                       block_table: torch.Tensor, query_start: torch.Tensor, context_lens: torch.Tensor, num_tokens: int,
                       num_seqs: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, window: int | None,
                       scale: float, lam: float, eps: float, out_scale: float, status: torch.Tensor | None = None) -> None:
    """:func:`diff_attention` for bfloat16 steps with portions of prompts, on tensor cores: tiles of 64 positions
    of a request, found through ``query_start`` and ``context_lens`` (``[seqs + 1]`` and ``[seqs]``)."""
    for name, tensor in (("q", q), ("out", out), ("k_pages", k_pages), ("v_pages", v_pages)):
        _need(tensor, torch.bfloat16, name)
    _need(block_table, torch.int32, "block_table"); _need(query_start, torch.int32, "query_start"); _need(context_lens, torch.int32, "context_lens")
    if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, 2 * dim)
            or tuple(v_pages.shape[2:]) != (num_kv_heads, vdim) or k_pages.shape[1] != v_pages.shape[1]):
        raise KernelError("diff_attention_mma: pages must be contiguous [pages, page_size, kv_heads, 2 * dim | vdim]")
    if q.shape[1] < num_heads * 2 * dim or out.shape[1] < num_heads * vdim:
        raise KernelError("diff_attention_mma: q or out is narrower than its heads")
    if query_start.numel() < num_seqs + 1 or context_lens.numel() < num_seqs:
        raise KernelError("diff_attention_mma: fewer requests than asked for")
    fn = _fn("diff_attention_mma", "ts_diff_attention_mma",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
              block_table.stride(0), _ptr(query_start), _ptr(context_lens), num_tokens, num_seqs, k_pages.shape[1],
              num_heads, num_kv_heads, dim, vdim, int(window or 0), float(scale), float(lam), float(eps),
              float(out_scale), _ptr(status), _stream()), "diff_attention_mma")


# ---------------------------------------------------------------------------------------
# ssd_ops.cu
# ---------------------------------------------------------------------------------------


def ssd_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, y: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor, num_seqs: int,
             heads: int, groups: int, vdim: int, state_size: int, num_tokens: int = 0) -> None:
    """The scalar-decay state-space recurrence over the step's positions of every request.

    ``xbc`` rows are ``[x: heads * vdim | B: groups * state | C: groups * state]`` (after the
    convolution and its activation), ``dt_raw`` ``[tokens, heads]`` (a view into the projection is
    fine), ``state`` float32 ``[slots, heads, vdim, state]``, ``y`` float32 ``[tokens, heads * vdim]``.
    ``num_tokens`` (the step's tokens, if known) only helps the launch choose its tiling.
    """
    _need(xbc, None, "xbc"); _need(dt_raw, xbc.dtype, "dt_raw"); _need(state, torch.float32, "state"); _need(y, torch.float32, "y")
    for name, tensor in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
        _need(tensor, torch.float32, name)
        if tensor.numel() != heads:
            raise KernelError(f"ssd_scan: {name} must hold one value per head")
    _need(query_start, torch.int32, "query_start"); _need(slots, torch.int32, "slots")
    inner = heads * vdim
    if xbc.shape[1] < inner + 2 * groups * state_size or dt_raw.shape[1] < heads:
        raise KernelError("ssd_scan: the inputs are narrower than their heads")
    if not y.is_contiguous() or y.shape[1] != inner or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, vdim, state_size):
        raise KernelError("ssd_scan: y must be [tokens, heads * vdim] and state [slots, heads, vdim, state]")
    fn = _fn("ssd_ops", "ts_ssd_scan", [c_int, c_void_p, c_longlong, c_void_p, c_longlong] + [c_void_p] * 7 + [c_int] * 6 + [c_void_p])
    _check(fn(dtype_code(xbc.dtype), _ptr(xbc), xbc.stride(0), _ptr(dt_raw), dt_raw.stride(0), _ptr(dt_bias), _ptr(a_log),
              _ptr(d_skip), _ptr(state), _ptr(y), _ptr(query_start), _ptr(slots), num_seqs, heads, groups, vdim, state_size,
              int(num_tokens), _stream()), "ssd_scan")


def selective_scan(x: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, bc: torch.Tensor, b_first: int, c_first: int,
                   a_log: torch.Tensor, d_skip: torch.Tensor, z: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                   query_start: torch.Tensor, slots: torch.Tensor, num_seqs: int, num_tokens: int) -> None:
    """The state-space recurrence with a state per channel and a decay per channel and state index, in float32:

    ``dt = softplus(dt_raw + dt_bias)``, ``S[c, n] = exp(dt[c] A[c, n]) S[c, n] + dt[c] x[c] B[n]`` with ``A = -exp(a_log)``,
    ``y[c] = sum_n S[c, n] C[n] + d_skip[c] x[c]``, ``out = y * silu(z)`` rounded once.

    ``x``, ``z`` and ``out`` are ``[tokens, inner]`` (columns of wider buffers are fine), ``dt_raw`` float32 contiguous
    ``[tokens, inner]``, ``bc`` holds ``B`` from column ``b_first`` and ``C`` from ``c_first`` (``N`` each), ``a_log`` float32
    ``[inner, N]``, ``state`` float32 ``[slots, inner, N]``."""
    _need(x, None, "x"); _need(bc, x.dtype, "bc"); _need(z, x.dtype, "z"); _need(out, x.dtype, "out")
    for name, tensor in (("dt_raw", dt_raw), ("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip), ("state", state)):
        _need(tensor, torch.float32, name)
    _need(query_start, torch.int32, "query_start"); _need(slots, torch.int32, "slots")
    inner, n_state = a_log.shape
    if (x.shape[1] != inner or z.shape[1] != inner or out.shape[1] != inner or not dt_raw.is_contiguous() or dt_raw.shape[1] != inner
            or dt_bias.numel() != inner or d_skip.numel() != inner or not a_log.is_contiguous() or not state.is_contiguous()
            or tuple(state.shape[1:]) != (inner, n_state) or bc.shape[1] < max(b_first, c_first) + n_state
            or any(t.stride(1) != 1 for t in (x, z, out, bc))):
        raise KernelError("selective_scan: shapes do not agree")
    if min(x.shape[0], z.shape[0], out.shape[0], bc.shape[0], dt_raw.shape[0]) < num_tokens or query_start.numel() < num_seqs + 1:
        raise KernelError("selective_scan: fewer rows than asked for")
    fn = _fn("ssd_ops", "ts_selective_scan",
             [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
              c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), x.stride(0), _ptr(dt_raw), _ptr(dt_bias), _ptr(bc), bc.stride(0), int(b_first),
              int(c_first), _ptr(a_log), _ptr(d_skip), _ptr(z), z.stride(0), _ptr(state), _ptr(out), out.stride(0),
              _ptr(query_start), _ptr(slots), num_seqs, inner, n_state, _stream()), "selective_scan")


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, num_tokens: int,
                     parts: int, eps: float) -> None:
    """``out = norm_parts(y * silu(z)) * weight``: ``y`` float32 ``[tokens, inner]``, ``z`` a view of ``inner`` columns."""
    _need(y, torch.float32, "y"); _need(z, None, "z"); _need(out, z.dtype, "out"); _need(weight, torch.float32, "weight")
    inner = y.shape[1]
    if not y.is_contiguous() or not out.is_contiguous() or out.shape[1] != inner or z.shape[1] < inner or weight.numel() != inner:
        raise KernelError("gated_group_norm: shapes do not agree")
    fn = _fn("ssd_ops", "ts_gated_group_norm", [c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(z.dtype), _ptr(y), _ptr(z), z.stride(0), _ptr(weight), _ptr(out), num_tokens, inner, parts,
              float(eps), _stream()), "gated_group_norm")


# ---------------------------------------------------------------------------------------
# latent_attention.cu
# ---------------------------------------------------------------------------------------


def latent_prepare(q: torch.Tensor, down: torch.Tensor | None, norm_weight: torch.Tensor | None, inv_freq: torch.Tensor,
                   amplitude: float, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                   pages: torch.Tensor, num_tokens: int, heads: int, dim: int, rot: int, rank: int, eps: float,
                   status: torch.Tensor | None = None, packed: torch.Tensor | None = None) -> None:
    """Rotate the last ``rot`` elements of every head of ``q`` (``[tokens, heads * (dim + rot)]``) in place and,
    when ``down`` (``[tokens, rank + rot]``) is given, append ``[rms_norm(latent) * norm_weight | rotated key part]``
    to ``pages`` (``[pages, page_size, 1, rank + rot]``). ``packed`` (``[tokens, heads * (rank + rot)]``) also receives
    every head's rotated elements behind the ``rank`` places of its carried query."""
    _need(q, None, "q"); _need(inv_freq, torch.float32, "inv_freq"); _need(pages, q.dtype, "pages")
    _need(positions, torch.int32, "positions"); _need(seq_of_token, torch.int32, "seq_of_token"); _need(block_table, torch.int32, "block_table")
    if q.shape[1] < heads * (dim + rot) or inv_freq.numel() * 2 != rot:
        raise KernelError("latent_prepare: q is narrower than its heads, or inv_freq does not hold rot / 2 values")
    if not pages.is_contiguous() or pages[0, 0].numel() != rank + rot:
        raise KernelError("latent_prepare: pages must be contiguous [pages, page_size, 1, rank + rot]")
    down_stride = 0
    if down is not None:
        _need(down, q.dtype, "down"); _need(norm_weight, torch.float32, "norm_weight")
        if down.shape[1] < rank + rot or norm_weight.numel() != rank:
            raise KernelError("latent_prepare: down must be [tokens, rank + rot] and norm_weight [rank]")
        down_stride = down.stride(0)
    packed_stride = 0
    if packed is not None:
        _need(packed, q.dtype, "packed")
        if packed.shape[1] < heads * (rank + rot) or packed.shape[0] < num_tokens:
            raise KernelError("latent_prepare: packed must be [tokens, heads * (rank + rot)]")
        packed_stride = packed.stride(0)
    fn = _fn("latent_attention", "ts_latent_prepare",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
              c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_longlong, c_void_p, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(down), down_stride, _ptr(norm_weight), _ptr(inv_freq),
              float(amplitude), _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.stride(0), _ptr(pages),
              pages.shape[1], num_tokens, heads, dim, rot, rank, float(eps), _ptr(packed), packed_stride, _ptr(status),
              _stream()), "latent_prepare")


def head_linear(x: torch.Tensor, in_head: int, weight: torch.Tensor, out: torch.Tensor, out_head: int, num_rows: int,
                gate: torch.Tensor | None = None) -> None:
    """``out[t, h * out_head + n] = sum_k x[t, h * in_head + k] * weight[h, n, k]`` for every head ``h`` in one launch;
    with ``gate`` (``[rows, >= heads]``, the same type) a head's outputs are multiplied by ``sigmoid(gate[t, h])``."""
    _need(x, None, "x"); _need(weight, x.dtype, "weight"); _need(out, x.dtype, "out")
    heads, n, k = weight.shape
    if gate is not None:
        _need(gate, x.dtype, "gate")
        if gate.dim() != 2 or gate.shape[0] < num_rows or gate.shape[1] < heads:
            raise KernelError("head_linear: the gate holds one number per row and head")
    if not weight.is_contiguous() or x.shape[1] < (heads - 1) * in_head + k or out.shape[1] < (heads - 1) * out_head + n:
        raise KernelError("head_linear: the rows are narrower than their heads")
    if x.shape[0] < num_rows or out.shape[0] < num_rows:
        raise KernelError("head_linear: fewer rows than asked for")
    fn = _fn("latent_attention", "ts_head_linear",
             [c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p,
              c_longlong, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), x.stride(0), int(in_head), _ptr(weight), _ptr(out), out.stride(0), int(out_head),
              num_rows, heads, n, k, _ptr(gate), 0 if gate is None else gate.stride(0), _stream()), "head_linear")


def latent_attention(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     seq_of_token: torch.Tensor, positions: torch.Tensor, num_tokens: int, heads: int, rank: int, rot: int,
                     window: int | None, scale: float, status: torch.Tensor | None = None) -> None:
    """Softmax attention of every (token, head) over its request's cached rows ``[latent | rotated part]``.

    ``q`` is ``[tokens, heads * (rank + rot)]`` (per head the query carried into the latent space, then its rotated
    part), ``out`` ``[tokens, heads * rank]`` (the weighted sum of the latents), ``pages`` ``[pages, page_size, 1, rank + rot]``."""
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(pages, q.dtype, "pages")
    _need(block_table, torch.int32, "block_table"); _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if not pages.is_contiguous() or pages[0, 0].numel() != rank + rot:
        raise KernelError("latent_attention: pages must be contiguous [pages, page_size, 1, rank + rot]")
    if q.shape[1] < heads * (rank + rot) or out.shape[1] < heads * rank:
        raise KernelError("latent_attention: q or out is narrower than its heads")
    if min(q.shape[0], out.shape[0], seq_of_token.numel(), positions.numel()) < num_tokens:
        raise KernelError("latent_attention: fewer rows than asked for")
    fn = _fn("latent_attention", "ts_latent_attention",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
              c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(pages), _ptr(block_table),
              block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens, pages.shape[1], heads, rank, rot,
              int(window or 0), float(scale), _ptr(status), _stream()), "latent_attention")


def latent_gather(pages: torch.Tensor, table_row: torch.Tensor, first: int, count: int, rows: torch.Tensor, padded: int,
                  status: torch.Tensor | None = None) -> None:
    """``rows[j] =`` the cached row of position ``first + j`` of the request whose block table is ``table_row``,
    ``j < count``; rows up to ``padded`` are zeroed."""
    _need(pages, None, "pages"); _need(rows, pages.dtype, "rows"); _need(table_row, torch.int32, "table_row")
    width = pages[0, 0].numel()
    if not pages.is_contiguous() or not rows.is_contiguous() or rows.shape[1] != width or rows.shape[0] < padded or count > padded:
        raise KernelError("latent_gather: rows must be contiguous [padded, row width]")
    if table_row.numel() * pages.shape[1] < first + count:
        raise KernelError("latent_gather: the block table is shorter than the range")
    fn = _fn("latent_attention", "ts_latent_gather", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(dtype_code(pages.dtype), _ptr(pages), _ptr(table_row), pages.shape[1], width, int(first), int(count), int(padded),
              _ptr(rows), _ptr(status), _stream()), "latent_gather")


def latent_softmax(scores: torch.Tensor, weights: torch.Tensor, heads: int, num_keys: int, first_query: int, first_key: int,
                   window: int | None, scale: float) -> None:
    """Softmax of ``scores`` (float32 ``[queries * heads, ld]``; row ``r`` is the query at position ``first_query + r // heads``,
    column ``j`` the key at ``first_key + j``) over the keys a query sees; ``weights`` (same shape) is zero elsewhere."""
    _need(scores, torch.float32, "scores"); _need(weights, None, "weights")
    if scores.dim() != 2 or tuple(weights.shape) != tuple(scores.shape) or not scores.is_contiguous() or not weights.is_contiguous():
        raise KernelError("latent_softmax: scores and weights must be contiguous and of one shape")
    if scores.shape[0] % heads or num_keys > scores.shape[1]:
        raise KernelError("latent_softmax: rows must be whole queries and the keys must fit a row")
    fn = _fn("latent_attention", "ts_latent_softmax", [c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p])
    _check(fn(dtype_code(weights.dtype), _ptr(scores), _ptr(weights), scores.shape[0], scores.shape[1], heads, num_keys,
              int(first_query), int(first_key), int(window or 0), float(scale), _stream()), "latent_softmax")


# ---------------------------------------------------------------------------------------
# retention_ops.cu
# ---------------------------------------------------------------------------------------


def retention_scratch_per_token(heads: int, dim: int, vdim: int) -> int:
    """Floats of scratch :func:`retention_scan` needs per token of a step (rotated q and k and the values, in fp32)."""
    fn = _fn("retention_ops", "ts_retention_scratch_per_token", [c_int, c_int, c_int])
    return int(fn(heads, dim, vdim))


def retention_scan(qkv: torch.Tensor, q_first: int, k_first: int, v_first: int, decay: torch.Tensor,
                   inv_freq: torch.Tensor, rot: int, amplitude: float, key_scale: float, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor, state: torch.Tensor,
                   y: torch.Tensor, scratch: torch.Tensor, num_tokens: int, num_seqs: int, heads: int, dim: int, vdim: int,
                   activation: str | None = None) -> None:
    """The decayed outer-product recurrence over the step's positions of every request.

    ``qkv`` rows hold q (``heads * dim`` from column ``q_first``), k (from ``k_first``) and v (``heads * vdim`` from
    ``v_first``) as projected; ``state`` is float32 ``[slots, heads, vdim, dim]``, ``y`` float32 ``[tokens, heads * vdim]``;
    ``scratch`` float32 with :func:`retention_scratch_per_token` floats per token. Two launches: the rotation of
    q and k (fp32), then the scan. With ``activation`` ``"silu"`` q, k and v pass it as they are read (then without a
    rotation)."""
    _need(qkv, None, "qkv"); _need(decay, torch.float32, "decay"); _need(inv_freq, torch.float32, "inv_freq")
    if activation not in (None, "silu") or (activation and rot):
        raise KernelError("retention_scan: the activation is silu or none, and goes with no rotation")
    _need(state, torch.float32, "state"); _need(y, torch.float32, "y"); _need(scratch, torch.float32, "scratch")
    for name, tensor in (("positions", positions), ("seq_of_token", seq_of_token), ("query_start", query_start), ("slots", slots)):
        _need(tensor, torch.int32, name)
    if decay.numel() != heads or inv_freq.numel() * 2 != rot:
        raise KernelError("retention_scan: decay must hold one value per head and inv_freq rot / 2 values")
    if max(q_first, k_first) + heads * dim > qkv.shape[1] or v_first + heads * vdim > qkv.shape[1]:
        raise KernelError("retention_scan: the rows are narrower than their heads")
    if not state.is_contiguous() or tuple(state.shape[1:]) != (heads, vdim, dim) or not y.is_contiguous() or y.shape[1] != heads * vdim:
        raise KernelError("retention_scan: state must be [slots, heads, vdim, dim] and y [tokens, heads * vdim]")
    if min(qkv.shape[0], y.shape[0], positions.numel(), seq_of_token.numel()) < num_tokens or query_start.numel() < num_seqs + 1:
        raise KernelError("retention_scan: fewer rows than asked for")
    if not scratch.is_contiguous() or scratch.numel() < num_tokens * retention_scratch_per_token(heads, dim, vdim):
        raise KernelError("retention_scan: the scratch is too small")
    if activation:
        fn = _fn("retention_ops", "ts_retention_scan_act",
                 [c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_float, c_int] + [c_void_p] * 7 + [c_int] * 5 + [c_void_p])
        _check(fn(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), int(q_first), int(k_first), int(v_first), _ptr(decay),
                  float(key_scale), 1, _ptr(positions), _ptr(seq_of_token), _ptr(query_start), _ptr(slots), _ptr(state), _ptr(y),
                  _ptr(scratch), num_tokens, num_seqs, heads, dim, vdim, _stream()), "retention_scan", launches=2)
        return
    fn = _fn("retention_ops", "ts_retention_scan",
             [c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_float] + [c_void_p] * 7 +
             [c_int] * 5 + [c_void_p])
    _check(fn(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), int(q_first), int(k_first), int(v_first), _ptr(decay),
              _ptr(inv_freq), int(rot), float(amplitude), float(key_scale), _ptr(positions), _ptr(seq_of_token), _ptr(query_start),
              _ptr(slots), _ptr(state), _ptr(y), _ptr(scratch), num_tokens, num_seqs, heads, dim, vdim, _stream()),
           "retention_scan", launches=2)


def head_norm_gate(y: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, num_tokens: int, heads: int, vdim: int, eps: float) -> None:
    """``out = y / rms_head(y) * silu(gate)``: ``y`` float32 ``[tokens, heads * vdim]``, ``gate`` a view of as many columns."""
    _need(y, torch.float32, "y"); _need(gate, None, "gate"); _need(out, gate.dtype, "out")
    if not y.is_contiguous() or not out.is_contiguous() or y.shape[1] != heads * vdim or out.shape[1] != heads * vdim or gate.shape[1] < heads * vdim:
        raise KernelError("head_norm_gate: shapes do not agree")
    fn = _fn("retention_ops", "ts_head_norm_gate", [c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(gate.dtype), _ptr(y), _ptr(gate), gate.stride(0), _ptr(out), num_tokens, heads, vdim, float(eps),
              _stream()), "head_norm_gate")


def part_norm_gate(y: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, num_tokens: int, parts: int, width: int, eps: float,
                   weight: torch.Tensor | None = None, gate_activation: str = "silu") -> None:
    """A row of ``y`` (float32 ``[tokens, parts * width]``) cut into ``parts`` equal parts, each divided by its own root
    mean square (``eps`` inside the root), times ``weight`` (float32, a row's worth, or ``None``), times
    ``silu(gate)`` or ``sigmoid(gate)``. ``parts`` = heads norms every head alone, ``parts`` = 1 the whole row."""
    _need(y, torch.float32, "y"); _need(gate, None, "gate"); _need(out, gate.dtype, "out")
    if gate_activation not in ("silu", "sigmoid"):
        raise KernelError("part_norm_gate: the gate's activation is silu or sigmoid")
    row = parts * width
    if not y.is_contiguous() or not out.is_contiguous() or y.shape[1] != row or out.shape[1] != row or gate.shape[1] < row:
        raise KernelError("part_norm_gate: shapes do not agree")
    if weight is not None:
        _need(weight, torch.float32, "weight")
        if weight.numel() != row or not weight.is_contiguous():
            raise KernelError("part_norm_gate: the weight must hold a row's worth of floats")
    fn = _fn("retention_ops", "ts_part_norm_gate",
             [c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p])
    _check(fn(dtype_code(gate.dtype), _ptr(y), _ptr(gate), gate.stride(0), _ptr(out), num_tokens, parts, width, float(eps),
              _ptr(weight), 1 if gate_activation == "sigmoid" else 0, _stream()), "part_norm_gate")


def chosen_decay_scratch_per_token(heads: int, dim: int, vdim: int) -> int:
    """Floats of scratch :func:`chosen_decay_scan` needs per token of a step (q, k, the decays and the values, in fp32)."""
    fn = _fn("retention_ops", "ts_chosen_decay_scratch_per_token", [c_int, c_int, c_int])
    return int(fn(heads, dim, vdim))


def chosen_decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bonus: torch.Tensor, decay_raw: torch.Tensor,
                      decay_bias: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, query_start: torch.Tensor,
                      slots: torch.Tensor, state: torch.Tensor, y: torch.Tensor, scratch: torch.Tensor, num_tokens: int,
                      num_seqs: int, heads: int, dim: int, vdim: int) -> None:
    """The recurrence with a decay the input chooses, per head, in float32:

    ``y_t = (S_{t-1} + diag(u) k_t v_t^T)^T q_t``, then ``S_t = diag(w_t) S_{t-1} + k_t v_t^T`` with
    ``w_t = exp(-exp(decay_raw_t + decay_bias))`` per key channel and ``u`` the ``bonus`` ``[heads, dim]``.

    ``q``, ``k`` (``[tokens, heads * dim]``) and ``v`` (``[tokens, heads * vdim]``) are views of columns of ONE buffer (the same
    row stride); ``decay_raw`` float32 ``[tokens, heads * dim]``; ``state`` float32 ``[slots, heads, vdim, dim]``; ``y`` float32
    ``[tokens, heads * vdim]``; ``scratch`` float32 with :func:`chosen_decay_scratch_per_token` floats per token."""
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        _need(tensor, q.dtype, name)
    for name, tensor in (("bonus", bonus), ("decay_raw", decay_raw), ("decay_bias", decay_bias), ("state", state), ("y", y), ("scratch", scratch)):
        _need(tensor, torch.float32, name)
    for name, tensor in (("positions", positions), ("seq_of_token", seq_of_token), ("query_start", query_start), ("slots", slots)):
        _need(tensor, torch.int32, name)
    size = q.element_size()
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim:
        raise KernelError("chosen_decay_scan: q, k and v must be columns of one buffer, heads * dim and heads * vdim wide")
    k_first, v_first = (k.data_ptr() - q.data_ptr()) // size, (v.data_ptr() - q.data_ptr()) // size
    if min(k_first, v_first) < 0 or (k.data_ptr() - q.data_ptr()) % size or (v.data_ptr() - q.data_ptr()) % size:
        raise KernelError("chosen_decay_scan: k and v must lie behind q in the buffer")
    if bonus.numel() != heads * dim or decay_bias.numel() != heads * dim or not decay_raw.is_contiguous() or decay_raw.shape[1] != heads * dim:
        raise KernelError("chosen_decay_scan: bonus, decay_bias and the rows of decay_raw hold heads * dim floats")
    if not state.is_contiguous() or tuple(state.shape[1:]) != (heads, vdim, dim) or not y.is_contiguous() or y.shape[1] != heads * vdim:
        raise KernelError("chosen_decay_scan: state must be [slots, heads, vdim, dim] and y [tokens, heads * vdim]")
    if min(q.shape[0], decay_raw.shape[0], y.shape[0], positions.numel(), seq_of_token.numel()) < num_tokens or query_start.numel() < num_seqs + 1:
        raise KernelError("chosen_decay_scan: fewer rows than asked for")
    if not scratch.is_contiguous() or scratch.numel() < num_tokens * chosen_decay_scratch_per_token(heads, dim, vdim):
        raise KernelError("chosen_decay_scan: the scratch is too small")
    fn = _fn("retention_ops", "ts_chosen_decay_scan",
             [c_int, c_void_p, c_longlong, c_int, c_int, c_int] + [c_void_p] * 10 + [c_int] * 5 + [c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), 0, int(k_first), int(v_first), _ptr(bonus), _ptr(decay_raw),
              _ptr(decay_bias), _ptr(positions), _ptr(seq_of_token), _ptr(query_start), _ptr(slots), _ptr(state), _ptr(y),
              _ptr(scratch), num_tokens, num_seqs, heads, dim, vdim, _stream()), "chosen_decay_scan", launches=2)


# ---------------------------------------------------------------------------------------
# moe_ops.cu
# ---------------------------------------------------------------------------------------


def moe_route(x: torch.Tensor, router: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor, num_tokens: int, top: int,
              groups: int = 1, keep: int = 1, score: str = "softmax", renormalize: bool = True) -> None:
    """Per token the ``top`` experts with the largest score among the ``keep`` best of ``groups`` groups (``chosen`` int32
    ``[tokens, top]``) and their weights (float32): the scores are a softmax over all experts or, with ``score="sigmoid"``,
    each expert's own sigmoid; the weights are the chosen scores over their sum, or as they are without ``renormalize``."""
    if score not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route: scores are a softmax or sigmoids, not {score!r}")
    mode = (1 if score == "sigmoid" else 0) | (0 if renormalize else 2)
    _need(x, None, "x"); _need(router, torch.float32, "router"); _need(chosen, torch.int32, "chosen"); _need(weights, torch.float32, "weights")
    experts, width = router.shape
    if not router.is_contiguous() or x.shape[1] != width or chosen.numel() < num_tokens * top or weights.numel() < num_tokens * top:
        raise KernelError("moe_route: shapes do not agree")
    fn = _fn("moe_ops", "ts_moe_route", [c_int, c_void_p, c_longlong, c_void_p] + [c_int] * 7 + [c_void_p] * 3)
    _check(fn(dtype_code(x.dtype), _ptr(x), x.stride(0), _ptr(router), num_tokens, width, experts, int(top), int(groups),
              int(keep), mode, _ptr(chosen), _ptr(weights), _stream()), "moe_route")


def _need_pair_weights(in_weights: torch.Tensor | None, pairs: int, name: str) -> None:
    if in_weights is not None:
        _need(in_weights, torch.float32, "in_weights")
        if in_weights.numel() < pairs or not in_weights.is_contiguous():
            raise KernelError(f"{name}: in_weights holds one float per (token, expert) pair")


def moe_pair_gate_up(x: torch.Tensor, gate_up: torch.Tensor, chosen: torch.Tensor, hidden: torch.Tensor, num_tokens: int,
                     top: int, activation: str, in_weights: torch.Tensor | None = None) -> None:
    """``hidden[t * top + k] = act(gate_e x_t) * (up_e x_t)`` for ``e = chosen[t, k]``; ``gate_up`` is ``[experts, 2 * ff, width]``.
    With ``in_weights`` (float32 ``[tokens, top]``) the expert reads ``in_weights[t, k] * x_t``."""
    _need_pair_weights(in_weights, num_tokens * top, "moe_pair_gate_up")
    _need(x, None, "x"); _need(gate_up, x.dtype, "gate_up"); _need(hidden, x.dtype, "hidden"); _need(chosen, torch.int32, "chosen")
    experts, twice, width = gate_up.shape
    ff = twice // 2
    if not gate_up.is_contiguous() or not hidden.is_contiguous() or x.shape[1] != width or hidden.shape[1] != ff or hidden.shape[0] < num_tokens * top:
        raise KernelError("moe_pair_gate_up: shapes do not agree")
    fn = _fn("moe_ops", "ts_moe_pair_gate_up", [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 5 + [c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), x.stride(0), _ptr(gate_up), _ptr(chosen), _ptr(in_weights), _ptr(hidden), num_tokens, width, ff,
              int(top), ACTIVATION_CODES[activation], _stream()), "moe_pair_gate_up")


def moe_pair_down(hidden: torch.Tensor, down: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor | None,
                  addend: torch.Tensor | None, out: torch.Tensor, num_tokens: int, top: int) -> None:
    """``out[t] = sum_k weights[t, k] * (down_e hidden[t * top + k]) (+ addend[t])``; ``down`` is ``[experts, width, ff]``;
    without ``weights`` every term counts once."""
    _need(hidden, None, "hidden"); _need(down, hidden.dtype, "down"); _need(out, hidden.dtype, "out")
    _need(chosen, torch.int32, "chosen")
    if weights is not None:
        _need(weights, torch.float32, "weights")
    experts, width, ff = down.shape
    if addend is not None:
        _need(addend, hidden.dtype, "addend")
        if not addend.is_contiguous() or addend.shape[1] != width:
            raise KernelError("moe_pair_down: addend must be contiguous [tokens, width]")
    if not down.is_contiguous() or not hidden.is_contiguous() or not out.is_contiguous() or hidden.shape[1] != ff or out.shape[1] != width:
        raise KernelError("moe_pair_down: shapes do not agree")
    fn = _fn("moe_ops", "ts_moe_pair_down", [c_int] + [c_void_p] * 6 + [c_int] * 4 + [c_void_p])
    _check(fn(dtype_code(hidden.dtype), _ptr(hidden), _ptr(down), _ptr(chosen), _ptr(weights), _ptr(addend), _ptr(out),
              num_tokens, width, ff, int(top), _stream()), "moe_pair_down")


def moe_expert_rows(gated: bool, rows_in: torch.Tensor, weights: torch.Tensor, counters: torch.Tensor, pair_of_row: torch.Tensor,
                    out: torch.Tensor, top: int, activation: str = "silu", in_weights: torch.Tensor | None = None) -> None:
    """Every expert's rows (in the order :func:`moe_sort` made) times that expert's matrix, the weights streamed once for up
    to eight rows at a time. ``gated``: ``rows_in`` is the step's inputs ``[tokens, width]`` (gathered through ``pair_of_row``),
    ``weights`` ``[experts, 2 * ff, width]`` and ``out[row] = act(gate x) * (up x)``; else ``rows_in`` is ``[pairs, ff]`` in
    expert order, ``weights`` ``[experts, width, ff]`` and ``out[row] = W rows_in[row]``. ``out`` has one row a pair.
    With ``in_weights`` (float32, one a pair; gated only) the expert reads its token's row times the pair's weight."""
    _need_pair_weights(in_weights if gated else None, out.shape[0], "moe_expert_rows")
    _need(rows_in, None, "rows_in"); _need(weights, rows_in.dtype, "weights"); _need(out, rows_in.dtype, "out")
    _need(counters, torch.int32, "counters"); _need(pair_of_row, torch.int32, "pair_of_row")
    experts, n_rows, k = weights.shape
    n_out = n_rows // 2 if gated else n_rows
    if not weights.is_contiguous() or not out.is_contiguous() or rows_in.shape[1] != k or out.shape[1] != n_out or counters.numel() < 2 * experts + 1:
        raise KernelError("moe_expert_rows: shapes do not agree")
    fn = _fn("moe_ops", "ts_moe_expert_rows", [c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p, c_void_p])
    _check(fn(dtype_code(rows_in.dtype), 1 if gated else 0, _ptr(rows_in), rows_in.stride(0), _ptr(weights), _ptr(counters),
              _ptr(pair_of_row), _ptr(out), k, n_out, int(top), experts, out.shape[0], ACTIVATION_CODES[activation],
              _ptr(in_weights if gated else None), _stream()), "moe_expert_rows")


MOE_EXPERT_ROWS_SMEM = 200 * 1024
"""Shared memory :func:`moe_expert_rows` may take: eight rows of the inner size."""


def moe_sort(chosen: torch.Tensor, num_pairs: int, experts: int, counters: torch.Tensor, place: torch.Tensor,
             pair_of_row: torch.Tensor) -> None:
    """Put the (token, expert) pairs in expert order: ``counters`` (int32 ``[3 * experts + 1]``) receives the counts and,
    from ``experts`` on, the first row of every expert (``experts + 1`` values); ``place[pair]`` is the pair's row and
    ``pair_of_row`` the inverse."""
    for name, tensor in (("chosen", chosen), ("counters", counters), ("place", place), ("pair_of_row", pair_of_row)):
        _need(tensor, torch.int32, name)
    if counters.numel() < 3 * experts + 1 or place.numel() < num_pairs or pair_of_row.numel() < num_pairs:
        raise KernelError("moe_sort: the index arrays are too small")
    fn = _fn("moe_ops", "ts_moe_sort", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(chosen), num_pairs, experts, _ptr(counters), _ptr(place), _ptr(pair_of_row), _stream()), "moe_sort",
           launches=1 if num_pairs <= 4096 and experts <= 2048 else 3)  # one block sorts a few pairs


def moe_gather(x: torch.Tensor, pair_of_row: torch.Tensor, rows: torch.Tensor, num_pairs: int, top: int,
               in_weights: torch.Tensor | None = None) -> None:
    """``rows[r] = x[pair_of_row[r] // top]``, times ``in_weights[pair_of_row[r]]`` if given (fp32 product, rounded once)."""
    _need_pair_weights(in_weights, num_pairs, "moe_gather")
    _need(x, None, "x"); _need(rows, x.dtype, "rows"); _need(pair_of_row, torch.int32, "pair_of_row")
    if not rows.is_contiguous() or rows.shape[1] != x.shape[1] or rows.shape[0] < num_pairs:
        raise KernelError("moe_gather: rows must be contiguous [pairs, width]")
    fn = _fn("moe_ops", "ts_moe_gather", [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), x.stride(0), _ptr(pair_of_row), _ptr(rows), num_pairs, x.shape[1], int(top),
              _ptr(in_weights), _stream()), "moe_gather")


def moe_combine(rows: torch.Tensor, place: torch.Tensor, weights: torch.Tensor | None, addend: torch.Tensor | None, out: torch.Tensor,
                num_tokens: int, top: int) -> None:
    """``out[t] = sum_k weights[t, k] * rows[place[t * top + k]] (+ addend[t])`` in fp32, rounded once; without ``weights``
    every row counts once."""
    _need(rows, None, "rows"); _need(out, rows.dtype, "out"); _need(place, torch.int32, "place")
    if weights is not None:
        _need(weights, torch.float32, "weights")
    width = out.shape[1]
    if addend is not None:
        _need(addend, rows.dtype, "addend")
        if not addend.is_contiguous() or addend.shape[1] != width:
            raise KernelError("moe_combine: addend must be contiguous [tokens, width]")
    if not rows.is_contiguous() or not out.is_contiguous() or rows.shape[1] != width:
        raise KernelError("moe_combine: shapes do not agree")
    fn = _fn("moe_ops", "ts_moe_combine", [c_int] + [c_void_p] * 5 + [c_int] * 3 + [c_void_p])
    _check(fn(dtype_code(rows.dtype), _ptr(rows), _ptr(place), _ptr(weights), _ptr(addend), _ptr(out), num_tokens, width,
              int(top), _stream()), "moe_combine")


# ---------------------------------------------------------------------------------------
# gemm_simt.cu
# ---------------------------------------------------------------------------------------


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None, m: int | None = None) -> None:
    """``out[:m] = a[:m] @ w.T (+ bias)`` with fp32 FFMA accumulation; any sizes."""
    _need(a, None, "a"); _need(w, a.dtype, "w"); _need(out, None, "out")
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2 or a.shape[1] != w.shape[1] or out.shape[1] != w.shape[0]:
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    rows = a.shape[0] if m is None else m
    if out.shape[0] < rows or a.shape[0] < rows:
        raise KernelError("gemm: fewer rows than asked for")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != w.shape[0]:
            raise KernelError("gemm: bias length does not match the output width")
    fn = _fn("gemm_simt", "ts_gemm_simt",
             [c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(a.dtype), dtype_code(out.dtype), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
              out.stride(0), rows, w.shape[0], a.shape[1], _stream()), "gemm_simt")


# ---------------------------------------------------------------------------------------
# sampling.cu
# ---------------------------------------------------------------------------------------


def argmax(logits: torch.Tensor, tokens: torch.Tensor, num_rows: int | None = None) -> None:
    _need(logits, torch.float32, "logits"); _need(tokens, torch.int32, "tokens")
    n = logits.shape[0] if num_rows is None else num_rows
    fn = _fn("sampling", "ts_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), n, logits.shape[1], _ptr(tokens), _stream()), "argmax")


def sample(logits: torch.Tensor, work: torch.Tensor, tokens: torch.Tensor, *, num_rows: int | None = None,
           temperature: torch.Tensor | None = None, top_k: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
           penalty: torch.Tensor | None = None, seed: torch.Tensor | None = None, counter: torch.Tensor | None = None,
           history: torch.Tensor | None = None, history_start: torch.Tensor | None = None,
           logprobs: torch.Tensor | None = None) -> None:
    """One token per row of fp32 ``logits``; per-row option arrays, ``None`` switches a stage off.

    ``work`` is fp32 scratch of at least ``[rows, vocab]``; ``seed`` is int64 (read as
    unsigned), ``counter`` int32 (the index of the token being generated).
    """
    _need(logits, torch.float32, "logits"); _need(work, torch.float32, "work"); _need(tokens, torch.int32, "tokens")
    n = logits.shape[0] if num_rows is None else num_rows
    vocab = logits.shape[1]
    if work.numel() < n * vocab or not work.is_contiguous():
        raise KernelError("sample: work must hold rows * vocab floats")
    for name, tensor, dtype in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                                ("top_p", top_p, torch.float32), ("penalty", penalty, torch.float32),
                                ("seed", seed, torch.int64), ("counter", counter, torch.int32),
                                ("history", history, torch.int32), ("history_start", history_start, torch.int32),
                                ("logprobs", logprobs, torch.float32)):
        if tensor is not None:
            _need(tensor, dtype, name)
    fn = _fn("sampling", "ts_sample", [c_void_p, c_longlong, c_void_p, c_int, c_int] + [c_void_p] * 11)
    _check(fn(_ptr(logits), logits.stride(0), _ptr(work), n, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
              _ptr(penalty), _ptr(seed), _ptr(counter), _ptr(history), _ptr(history_start), _ptr(tokens),
              _ptr(logprobs), _stream()), "sample")


def sample_slots(logits: torch.Tensor, work: torch.Tensor, tokens: torch.Tensor, num_rows: int, *, temperature: torch.Tensor,
                 top_k: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor, prompt_len: torch.Tensor,
                 seq_slot: torch.Tensor, seq_context: torch.Tensor, partial: torch.Tensor, chunks: int,
                 row_token: torch.Tensor | None = None, seq_of_token: torch.Tensor | None = None,
                 step_tokens: torch.Tensor | None = None, penalty: torch.Tensor | None = None,
                 seen: torch.Tensor | None = None, want_logprob: torch.Tensor | None = None,
                 logprobs: torch.Tensor | None = None) -> None:
    """One token per row with the options looked up by state slot (arrays over the slots).

    A row finds its request through a step's own index arrays: ``row_token`` (per row: the step's
    token whose logits the row holds; without it the row itself), ``seq_of_token`` (per token: its
    request in the step, negative for padding, whose row is skipped; without it the token itself),
    ``seq_slot`` and ``seq_context`` (per request: its state slot and its length after the step).
    The index of the token being generated is ``seq_context - prompt_len[slot]``. ``partial`` is
    zeroed int32 scratch of ``rows * (4 * chunks + 1)`` words; a row that needs one pass only
    (greedy, or a draw without top-k and top-p) is cut into ``chunks`` blocks.

    ``penalty`` (per slot) goes with ``seen`` (int32 ``[slots, ceil(vocab / 32)]``: the bitmap of the
    tokens each slot's request holds); ``step_tokens`` (per token of the step: its id) lets a row
    add the token its logits come from to that bitmap first. ``want_logprob`` (per slot, int32)
    goes with ``logprobs`` (float32 per row): the log-probability of the chosen token under the
    penalised row."""
    _need(logits, torch.float32, "logits"); _need(work, torch.float32, "work"); _need(tokens, torch.int32, "tokens")
    vocab = logits.shape[1]
    if work.numel() < num_rows * vocab or not work.is_contiguous():
        raise KernelError("sample_slots: work must hold rows * vocab floats")
    for name, tensor, dtype in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                                ("top_p", top_p, torch.float32), ("seed", seed, torch.int64), ("prompt_len", prompt_len, torch.int32),
                                ("seq_slot", seq_slot, torch.int32), ("seq_context", seq_context, torch.int32),
                                ("partial", partial, torch.int32)):
        _need(tensor, dtype, name)
    for name, tensor, dtype in (("row_token", row_token, torch.int32), ("seq_of_token", seq_of_token, torch.int32),
                                ("penalty", penalty, torch.float32), ("seen", seen, torch.int32),
                                ("step_tokens", step_tokens, torch.int32), ("want_logprob", want_logprob, torch.int32),
                                ("logprobs", logprobs, torch.float32)):
        if tensor is not None:
            _need(tensor, dtype, name)
    if partial.numel() < num_rows * (4 * chunks + 1):
        raise KernelError("sample_slots: partial is too small")
    if row_token is not None and row_token.numel() < num_rows:
        raise KernelError("sample_slots: row_token has fewer entries than rows")
    seen_words = 0
    if penalty is not None:
        if seen is None or seen.dim() != 2 or not seen.is_contiguous() or seen.shape[1] * 32 < vocab or seen.shape[0] < penalty.numel():
            raise KernelError("sample_slots: a penalty needs seen [slots, ceil(vocab / 32)]")
        seen_words = seen.shape[1]
    if (want_logprob is None) != (logprobs is None) or (logprobs is not None and logprobs.numel() < num_rows):
        raise KernelError("sample_slots: want_logprob and logprobs (one per row) go together")
    fn = _fn("sampling", "ts_sample_slots", [c_void_p, c_longlong, c_void_p, c_int, c_int] + [c_void_p] * 12 + [c_int] +
             [c_void_p] * 3 + [c_int] + [c_void_p] * 2)
    _check(fn(_ptr(logits), logits.stride(0), _ptr(work), num_rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
              _ptr(seed), _ptr(prompt_len), _ptr(row_token), _ptr(seq_of_token), _ptr(seq_slot), _ptr(seq_context),
              _ptr(step_tokens), _ptr(tokens), _ptr(partial), int(chunks), _ptr(penalty), _ptr(want_logprob),
              _ptr(seen if penalty is not None else None), seen_words, _ptr(logprobs), _stream()),
           "sample_slots", launches=2)  # the one-pass kernel, then the cluster kernel for rows with filters


def mark_seen(token_ids: torch.Tensor, seq_of_token: torch.Tensor, state_slots: torch.Tensor, penalty: torch.Tensor,
              seen: torch.Tensor, num_tokens: int, vocab: int) -> None:
    """Set, in ``seen`` (int32 ``[slots, ceil(vocab / 32)]``), the bit of every token of the step whose
    request's slot has a penalty other than 1 (``penalty`` per slot)."""
    for name, tensor, dtype in (("token_ids", token_ids, torch.int32), ("seq_of_token", seq_of_token, torch.int32),
                                ("state_slots", state_slots, torch.int32), ("penalty", penalty, torch.float32),
                                ("seen", seen, torch.int32)):
        _need(tensor, dtype, name)
    if token_ids.numel() < num_tokens or seq_of_token.numel() < num_tokens:
        raise KernelError("mark_seen: fewer tokens than asked for")
    if seen.dim() != 2 or not seen.is_contiguous() or seen.shape[1] * 32 < vocab or seen.shape[0] < penalty.numel():
        raise KernelError("mark_seen: seen must be [slots, ceil(vocab / 32)]")
    fn = _fn("sampling", "ts_mark_seen", [c_void_p] * 5 + [c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(token_ids), _ptr(seq_of_token), _ptr(state_slots), _ptr(penalty), _ptr(seen), seen.shape[1], num_tokens,
              vocab, _stream()), "mark_seen")


def sample_uniform_host(seed: int, counter: int, index: int) -> float:
    fn = _fn("sampling", "ts_sample_uniform_host", [ctypes.c_ulonglong, ctypes.c_uint, ctypes.c_uint], restype=c_float)
    return float(fn(seed & 0xFFFFFFFFFFFFFFFF, counter, index))
